"""Counterparts of ``vtpack/layers/sparse_ops.py``: ``batched_sparse_attention(q, k, v, q_lengths,
scale)`` (eval; ``sparse_ops.py:60-78``) and the differentiable ragged product
``batched_sparse_gemm(a, b, a_lengths, b_lengths, is_a_transposed, is_b_transposed)`` of the
training path (``sparse_ops.py:11-57``)."""
import torch
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from .. import _lib
from ..runtime import dtype_code, ptr, require_cuda, stream_ptr


def batched_sparse_attention(q, k, v, q_lengths, scale, flags: int = 0):
    """q [h,L,d], k/v [h,B,N,d], q_lengths int [B] (CPU, as in the reference) -> [h,L,d].

    The operands may be the permuted views the model makes of its Linear outputs; they
    are read through their strides, so the ``.contiguous()`` copies of the reference
    (``sparse_ops.py:64-66``) do not happen.  The result is a [h,L,d] view of an
    [L,h,d] buffer, so the model's ``transpose(0,1).reshape(-1,C)`` is free.
    """
    require_cuda(q, k, v)
    h, L, d = q.shape
    _, B, N, _ = k.shape
    if q.stride(2) != 1:
        q = q.contiguous()
    if k.stride(3) != 1 or v.stride(3) != 1 or k.stride() != v.stride():
        k, v = k.contiguous(), v.contiguous()
    lengths = q_lengths.to("cpu", torch.int64)
    offsets = torch.zeros(B + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(lengths, 0)
    assert int(offsets[-1]) == L, "q_lengths do not add up to the number of query rows"
    offsets = offsets.to(q.device, non_blocking=True)
    out = torch.empty(L, h, d, dtype=q.dtype, device=q.device)
    _lib.check(_lib.lib().vtp_sparse_attention(
        ptr(q), q.stride(1), q.stride(0), ptr(k), ptr(v), k.stride(1), k.stride(2), k.stride(0),
        ptr(out), h * d, d, dtype_code(q.dtype), B, N, h, d, ptr(offsets), L,
        int(lengths.max()) if B > 0 else 0, float(scale), int(flags), stream_ptr(q.device)))
    return out.permute(1, 0, 2)


def _offsets(lengths, device):
    lengths = lengths.to("cpu", torch.int64)
    off = torch.zeros(lengths.numel() + 1, dtype=torch.int32)
    off[1:] = torch.cumsum(lengths, 0)
    return off.to(device, non_blocking=True), int(off[-1]), int(lengths.max()) if lengths.numel() else 0


def _ragged_gemm(a, b, a_lengths, b_lengths, ta, tb):
    """One launch of ``vtp_batched_sparse_gemm``: a [H,La,ka], b [H,Lb,kb] -> the per-image products
    stacked along dim 1 (``batched_sparse_gemm.cu:150-196``)."""
    require_cuda(a, b)
    a, b = a.contiguous(), b.contiguous()
    H, B = a.shape[0], a_lengths.numel()
    a_off, a_total, a_max = _offsets(a_lengths, a.device)
    b_off, b_total, b_max = _offsets(b_lengths, a.device)
    assert a_total <= a.shape[1] and b_total <= b.shape[1], "lengths exceed the rows of the operands"
    if tb:
        assert b.shape[1] % B == 0 and int(b_lengths.min()) == b_max, \
            "a transposed b needs the same number of rows in every image"
    out_rows = B * a.shape[2] if ta else a_total
    out_cols = b_max if tb else b.shape[2]
    out = torch.empty(H, out_rows, out_cols, dtype=a.dtype, device=a.device)
    _lib.check(_lib.lib().vtp_batched_sparse_gemm(
        ptr(a), ptr(b), ptr(out), dtype_code(a.dtype), H, B, a.shape[1], a.shape[2], b.shape[1], b.shape[2],
        ptr(a_off), ptr(b_off), a_max, b_max, int(bool(ta)), int(bool(tb)), out_rows, out_cols,
        stream_ptr(a.device)))
    return out


class _BatchedSparseGEMM(Function):
    """Forward and backward are the same kernel with other transpose flags, wired as in
    ``sparse_ops.py:30-55``."""

    @staticmethod
    def forward(ctx, a, b, a_lengths, b_lengths, is_a_transposed, is_b_transposed):
        a, b = a.contiguous(), b.contiguous()
        ctx.ta, ctx.tb = bool(is_a_transposed), bool(is_b_transposed)
        ctx.lengths = (a_lengths, b_lengths)
        ctx.save_for_backward(a, b)
        return _ragged_gemm(a, b, a_lengths, b_lengths, ctx.ta, ctx.tb)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        a, b = ctx.saved_tensors
        la, lb = ctx.lengths
        g = grad_output.contiguous()
        if not ctx.ta:
            grad_a = _ragged_gemm(g, b, la, lb, False, not ctx.tb)
        else:
            grad_a = _ragged_gemm(b, g, lb, la, ctx.tb, True)
        if not ctx.tb:
            grad_b = _ragged_gemm(a, g, la, la, not ctx.ta, False)
        else:
            grad_b = _ragged_gemm(g, a, la, la, True, ctx.ta)
        return grad_a, grad_b, None, None, None, None


batched_sparse_gemm = _BatchedSparseGEMM.apply
