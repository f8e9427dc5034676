"""Eval-mode mirror of the reference's PVT+DGE block (``vtpack/models/dge/pvt_dge.py:19-146``): the
same class names, constructor arguments and state_dict keys, with ``Block.forward(x, H, W)`` as
one call into the CUDA library.  Keys and values come from the normed tokens reduced by the
stride-``sr_ratio`` convolution ``attn.sr`` and the LayerNorm ``attn.norm``; everything else is
the DeiT+DGE block.  Only the block is mirrored here; the pyramid wrapper around it (patch
embeddings between stages, position embeddings, head) is not.
"""
import ctypes

import torch
import torch.nn as nn

from ... import _lib
from ...layers import DynamicGrainedEncoder
from ...runtime import ptr, require_cuda, scratch, stream_ptr
from .deit_dge import Mlp, _WeightPack, _pack_block, _shape_struct

__all__ = ["Mlp", "Attention", "Block"]


class Attention(nn.Module):
    def __init__(self, dim, num_heads=8, qkv_bias=False, qk_scale=None, attn_drop=0., proj_drop=0., sr_ratio=1):
        super().__init__()
        assert dim % num_heads == 0, f"dim {dim} should be divided by num_heads {num_heads}."
        self.dim = dim
        self.num_heads = num_heads
        head_dim = dim // num_heads
        self.scale = qk_scale or head_dim ** -0.5
        self.q = nn.Linear(dim, dim, bias=qkv_bias)
        self.kv = nn.Linear(dim, dim * 2, bias=qkv_bias)
        self.attn_drop = nn.Dropout(attn_drop)
        self.proj = nn.Linear(dim, dim)
        self.proj_drop = nn.Dropout(proj_drop)
        self.sr_ratio = sr_ratio
        if sr_ratio > 1:
            self.sr = nn.Conv2d(dim, dim, kernel_size=sr_ratio, stride=sr_ratio)
            self.norm = nn.LayerNorm(dim)

    def complexity(self, num_inputs, num_queries):
        num_channels = self.dim
        comp = num_queries * (num_channels ** 2)  # q embed
        if self.sr_ratio > 1:
            comp += num_inputs * (num_channels ** 2)  # sr
            comp += num_inputs / (self.sr_ratio ** 2) * num_channels  # norm
        comp += (num_inputs / (self.sr_ratio ** 2) * (num_channels ** 2)) * 2  # kv embed
        comp += num_queries * num_inputs / (self.sr_ratio ** 2) * num_channels  # attention
        comp += num_queries * num_inputs / (self.sr_ratio ** 2) * self.num_heads * 3  # softmax
        comp += num_queries * num_channels ** 2  # proj
        return comp


class Block(nn.Module):

    def __init__(self, dim, num_heads, mlp_ratio=4., qkv_bias=False, qk_scale=None, drop=0., attn_drop=0.,
                 drop_path=0., act_layer=nn.GELU, norm_layer=nn.LayerNorm, sr_ratio=1, split_sizes=[2, 1]):
        super().__init__()
        self.dim = dim
        self.norm1 = norm_layer(dim)
        self.attn = Attention(dim, num_heads=num_heads, qkv_bias=qkv_bias, qk_scale=qk_scale,
                              attn_drop=attn_drop, proj_drop=drop, sr_ratio=sr_ratio)
        self.drop_path = nn.Identity()
        self.norm2 = norm_layer(dim)
        self.mlp = Mlp(in_features=dim, hidden_features=int(dim * mlp_ratio), act_layer=act_layer, drop=drop)
        self.dge = DynamicGrainedEncoder(in_channels=dim, split_sizes=split_sizes, complexity_handler=self.complexity)
        self.split_sizes = list(split_sizes)
        self.flags = 0
        self.fold_layernorm = sr_ratio <= 1      # the reduced keys need explicit LayerNorm rows
        self._pack = _WeightPack()

    def complexity(self, num_inputs, num_queries):
        comp = num_inputs * self.dim * 2  # norm1 and norm2
        comp += self.attn.complexity(num_inputs, num_queries)
        comp += self.mlp.complexity(num_inputs, num_queries)
        return comp

    def forward(self, x, H, W, forced_gate=None):
        """x [B, N, C] with N = H*W (+ extra tokens when sr_ratio == 1) -> [B, N, C]
        (``pvt_dge.py:140-146``), one C-ABI call.  ``forced_gate`` (fp32 [B,Hr,Wr,n_splits])
        replaces the router output."""
        if self.training:
            raise NotImplementedError("vtpack_b200 implements the eval-mode forward only")
        require_cuda(x)
        x = x.contiguous()
        B, N, C = x.shape
        s = _shape_struct(x.dtype, B, H, W, N - H * W, C, self.attn.num_heads, self.mlp.fc1.out_features,
                          self.split_sizes, self.norm1.eps, self.flags)
        if self.attn.sr_ratio > 1:
            s.sr_ratio = self.attn.sr_ratio
            s.sr_eps = float(self.attn.norm.eps)
        w = _pack_block(self, x.dtype)
        lib = _lib.lib()
        nbytes = lib.vtp_block_workspace_bytes(ctypes.byref(s))
        _lib.check(0 if nbytes >= 0 else int(nbytes))
        ws = scratch(x.device, nbytes)
        out = torch.empty_like(x)
        counts = torch.empty(B, dtype=torch.int32, device=x.device)
        if forced_gate is not None:
            forced_gate = forced_gate.to(device=x.device, dtype=torch.float32).contiguous()
        _lib.check(lib.vtp_dge_block_forward(ctypes.byref(s), ctypes.byref(w), ptr(x), ptr(out), ptr(forced_gate),
                                             ptr(counts), ptr(ws), nbytes, stream_ptr(x.device)))
        self.dge.states.update({"batches_device": counts, "input": x, "gate": None, "size": (H, W),
                                "num_extra_tokens": N - H * W})
        return out
