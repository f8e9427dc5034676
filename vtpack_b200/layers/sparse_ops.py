"""Forward-only counterpart of ``vtpack/layers/sparse_ops.py``:
``batched_sparse_attention(q, k, v, q_lengths, scale)`` (``sparse_ops.py:60-78``)."""
import torch

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
