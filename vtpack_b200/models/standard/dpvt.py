"""The deformable attention of the reference's DPVT (``vtpack/models/standard/dpvt.py:51-115``) over
this library's bilinear-sampling op: same class name, constructor arguments, parameter names and
initialisation, so a DPVT checkpoint's ``attn.*`` tensors load unchanged.  The dense layers stay in
PyTorch (as in the reference); the sampling and its three gradients run the CUDA kernels behind
``vtpack_b200.layers.bilinear_attention``.  The rest of the DPVT model (a standard, not a DGE,
pyramid) is plain PyTorch in the reference and is not repeated here.
"""
import math

import torch
import torch.nn as nn

from ...layers import bilinear_attention

__all__ = ["Attention", "grad_scale"]


class _GradScale(torch.autograd.Function):
    """Identity whose gradient is multiplied by ``scale`` (``dpvt.py:18-30``)."""

    @staticmethod
    def forward(ctx, input, scale=1.0):
        ctx.scale = scale
        return input

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output * ctx.scale, None


grad_scale = _GradScale.apply


class Attention(nn.Module):
    """Every token looks at ``num_points`` learned offsets around its own pixel, per head, and mixes
    the bilinearly sampled values with softmax weights predicted from the token itself."""

    def __init__(self, dim, num_heads=8, qkv_bias=False, qk_scale=None, attn_drop=0., proj_drop=0., num_points=1):
        super().__init__()
        assert dim % num_heads == 0, f"dim {dim} should be divided by num_heads {num_heads}."
        self.dim = dim
        self.num_heads = num_heads
        self.num_points = num_points
        self.v = nn.Linear(dim, dim, bias=qkv_bias)
        self.attn_weight = nn.Linear(dim, num_heads * num_points)
        self.attn_drop = nn.Dropout(attn_drop)
        self.proj = nn.Linear(dim, dim)
        self.proj_drop = nn.Dropout(proj_drop)
        self.offsets = nn.Linear(dim, num_heads * num_points * 2)
        self._reset_parameters()

    def _reset_parameters(self):
        """Zero offset weights; the bias spreads the heads' points along evenly spaced directions, the
        k-th point k pixels out (``dpvt.py:75-84``)."""
        nn.init.constant_(self.offsets.weight.data, 0.)
        theta = torch.arange(self.num_heads, dtype=torch.float32) * (2.0 * math.pi / self.num_heads)
        direction = torch.stack([theta.cos(), theta.sin()], -1)
        direction = direction / direction.abs().max(-1, keepdim=True)[0]
        steps = torch.arange(1, self.num_points + 1, dtype=torch.float32).view(1, -1, 1)
        self.offsets.bias = nn.Parameter((direction.view(self.num_heads, 1, 2) * steps).reshape(-1))

    @torch.no_grad()
    def get_reference_points(self, x, H, W):
        ys, xs = torch.meshgrid(torch.arange(H, device=x.device, dtype=x.dtype),
                                torch.arange(W, device=x.device, dtype=x.dtype), indexing="ij")
        return torch.stack([xs, ys], dim=-1).reshape(1, H * W, 1, 2)

    def forward(self, x, H, W):
        """x [B, H*W, C] -> [B, H*W, C] (``dpvt.py:92-115``)."""
        B, N, C = x.shape
        h, P, d = self.num_heads, self.num_points, C // self.num_heads
        v = self.v(x).reshape(B, N, h, d).permute(0, 2, 1, 3).reshape(B * h, H, W, d)
        offsets = self.offsets(x).reshape(B, N, h, P, 2).permute(0, 2, 1, 3, 4).reshape(B * h, N, P, 2)
        grid = grad_scale(self.get_reference_points(v, H, W) + offsets, 0.1)
        weight = self.attn_weight(x).reshape(B, N, h, P).permute(0, 2, 1, 3).reshape(B * h, N, P)
        weight = self.attn_drop(weight.softmax(dim=-1, dtype=v.dtype))
        out = bilinear_attention(v, grid, weight, "point")
        out = out.reshape(B, h, N, d).permute(0, 2, 1, 3).reshape(B, N, C)
        return self.proj_drop(self.proj(out))
