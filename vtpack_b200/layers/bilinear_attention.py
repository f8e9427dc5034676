"""Counterpart of ``vtpack/layers/bilinear_attention.py``: ``bilinear_attention(input, grid, weight,
mode)`` with the reference's argument order, modes ("channel" default, "point") and gradients
(``bilinear_attention.py:9-45``), running the CUDA kernels of this library through the C ABI."""
import torch
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from .. import _lib
from ..runtime import dtype_code, ptr, require_cuda, stream_ptr

_MODES = {"point": 0, "channel": 1}


def _dims(input, grid):
    B, H, W, C = input.shape
    return B, H, W, C, grid.shape[1], grid.shape[2]


class _BilinearAttention(Function):
    """input [B,H,W,C], grid [B,G,P,2] (x, y in pixels), weight [B,G,P] ("point": -> [B,G,C]) or
    [B,G,C] ("channel": -> [B,G,P])."""

    @staticmethod
    def forward(ctx, input, grid, weight, mode="channel"):
        if mode not in _MODES:
            raise NotImplementedError(f"Mode {mode} is not supported")
        require_cuda(input, grid, weight)
        input = input.contiguous()
        grid = grid.to(input.dtype).contiguous()
        weight = weight.to(input.dtype).contiguous()
        B, H, W, C, G, P = _dims(input, grid)
        assert grid.shape == (B, G, P, 2) and weight.shape == (B, G, P if mode == "point" else C), \
            "grid must be [B,G,P,2] and weight [B,G,P] (point) or [B,G,C] (channel)"
        ctx.mode = mode
        ctx.save_for_backward(input, grid, weight)
        out = torch.empty(B, G, C if mode == "point" else P, dtype=input.dtype, device=input.device)
        _lib.check(_lib.lib().vtp_bilinear_attention_forward(
            ptr(input), ptr(grid), ptr(weight), ptr(out), dtype_code(input.dtype), _MODES[mode], B, H, W, C, G, P,
            stream_ptr(input.device)))
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        input, grid, weight = ctx.saved_tensors
        grad_output = grad_output.to(input.dtype).contiguous()
        B, H, W, C, G, P = _dims(input, grid)
        grad_input, grad_grid, grad_weight = torch.empty_like(input), torch.empty_like(grid), torch.empty_like(weight)
        _lib.check(_lib.lib().vtp_bilinear_attention_backward(
            ptr(grad_output), ptr(input), ptr(grid), ptr(weight), ptr(grad_input), ptr(grad_grid), ptr(grad_weight),
            dtype_code(input.dtype), _MODES[ctx.mode], B, H, W, C, G, P, stream_ptr(input.device)))
        return grad_input, grad_grid, grad_weight, None


bilinear_attention = _BilinearAttention.apply


def sparse_bilinear_attention_pointwise_forward(input, grid, weight, batches):
    """Point-mode bilinear attention over packed queries: input [B,H,W,C], grid [L,P,2], weight [L,P],
    batches int64 [L] (the image of each query) -> [L,C].  The counterpart of the reference's
    ``_C.sparse_bilinear_attention_pointwise_forward`` (``vision.cpp:28``); forward only, as there."""
    require_cuda(input, grid, weight, batches)
    input = input.contiguous()
    grid = grid.to(input.dtype).contiguous()
    weight = weight.to(input.dtype).contiguous()
    batches = batches.to(torch.int64).contiguous()
    B, H, W, C = input.shape
    L, P = grid.shape[0], grid.shape[1]
    assert grid.shape == (L, P, 2) and weight.shape == (L, P) and batches.shape == (L,)
    out = torch.empty(L, C, dtype=input.dtype, device=input.device)
    _lib.check(_lib.lib().vtp_sparse_bilinear_attention_forward(
        ptr(input), ptr(grid), ptr(weight), ptr(batches), ptr(out), dtype_code(input.dtype), B, H, W, C, L, P,
        stream_ptr(input.device)))
    return out
