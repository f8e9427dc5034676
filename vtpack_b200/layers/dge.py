"""``DynamicGrainedEncoder`` / ``DynamicRouter`` with the reference's constructor,
parameters (``splits``, ``router.gate.*``), ``states`` dict and methods
(``vtpack/layers/dge.py:19-150``) on CUDA.  Eval mode runs the fused gate kernel; training mode
(Gumbel-softmax gate, ``dge.py:66-67``) keeps the router in autograd and moves tokens through the
differentiable ``grained_sample_compress`` / ``grained_sample_decompress``, or through the dense
all-grains form when ``sparse_train`` is off (``dge.py:69-73,92-96``)."""
import ctypes
import math
from typing import List

import torch
import torch.nn.functional as F
from torch import nn

from .. import _lib
from ..runtime import dtype_code, ptr, require_cuda, stream_ptr
from .grained_sample import (
    grained_sample_compress,
    grained_sample_compress_dense,
    grained_sample_decompress,
    grained_sample_decompress_dense,
    grained_sample_index_to_patch,
)


class DynamicRouter(nn.Module):
    """Region average pool + Linear(C -> n_splits) (``dge.py:115-150``)."""

    def __init__(self, num_channels, split_sizes, init_gate=0.95):
        super().__init__()
        self.num_channels = num_channels
        self.region_size = max(split_sizes)
        self.split_sizes = split_sizes
        self.init_gate = init_gate
        self.gate = nn.Linear(num_channels, len(split_sizes))
        self.init_parameters()

    def init_parameters(self):
        nn.init.trunc_normal_(self.gate.weight, std=.01)
        n = len(self.split_sizes)
        if n == 1:
            nn.init.constant_(self.gate.bias.data, 0)
        else:
            bias_value = math.log(math.sqrt(self.init_gate * (1 - n) / (self.init_gate - 1)))
            self.gate.bias.data[0] = bias_value
            self.gate.bias.data[1:] = -bias_value

    def complexity(self, num_inputs, num_queries):
        comp = num_inputs / (self.region_size ** 2) * self.num_channels
        comp += num_inputs / (self.region_size ** 2) * self.num_channels * len(self.split_sizes)
        return comp

    def forward(self, x):
        """x [B,H,W,C] -> gate logits [B,H/r,W/r,n_splits] (fp32 from the fused kernel in eval mode;
        in training mode the region mean and the Linear stay in autograd, ``dge.py:145-150``)."""
        if self.training:
            B, H, W, C = x.shape
            r = self.region_size
            pooled = x.reshape(B, H // r, r, W // r, r, C).mean(dim=(2, 4))
            return self.gate(pooled)
        require_cuda(x)
        x = x.contiguous()
        B, H, W, C = x.shape
        r = self.region_size
        logits = torch.empty(B, H // r, W // r, len(self.split_sizes), dtype=torch.float32, device=x.device)
        idx = torch.empty(B, H // r, W // r, dtype=torch.int32, device=x.device)
        gw, gb = self.gate.weight.detach().float().contiguous(), self.gate.bias.detach().float().contiguous()
        _lib.check(_lib.lib().vtp_router_gate(
            ptr(x), dtype_code(x.dtype), B, H, W, C, 0, r, ptr(gw), ptr(gb), len(self.split_sizes), ptr(logits),
            ptr(idx), stream_ptr(x.device)))
        self.last_indices = idx
        return logits


class DynamicGrainedEncoder(nn.Module):

    def __init__(self, in_channels: int, split_sizes: List[int], complexity_handler=None,
                 sparse_train: bool = False):
        super().__init__()
        self.region_size = max(split_sizes)
        self.in_channels = in_channels
        self.splits = nn.Parameter(torch.tensor(split_sizes), requires_grad=False)
        self.router = DynamicRouter(in_channels, split_sizes)
        self.complexity_handler = complexity_handler
        self.sparse_train = sparse_train
        self.states = {
            "comp": None, "input": None, "patches": None, "batches": None,
            "gate": None, "size": None, "num_extra_tokens": 0,
        }

    def get_complexity(self):
        """MAC accounting of the last forward (``dge.py:40-59``)."""
        if self.complexity_handler is None:
            return {"static": None, "dynamic": None}
        B, N, C = self.states["input"].shape
        gate = self.states["gate"]
        if gate is None:
            # fused forward: the kernels left the per-image query counts (extra tokens included) on
            # the device, which is the sum the reference recomputes from the gate; nothing is copied
            # to the host here
            num_queries = self.states["batches_device"].double()
        else:
            if not self.training:
                indices = gate.argmax(dim=-1, keepdim=True)
                gate = torch.zeros_like(gate).scatter_(-1, indices, 1.0)
            # in training mode the gate is the hard Gumbel-softmax sample: already one-hot, and it keeps
            # its straight-through gradient so a complexity loss can train the router
            num_queries = gate * (self.splits[None, None, None, :] ** 2)
            num_queries = num_queries.view(B, -1).double().sum(-1)
            num_queries = num_queries + self.states["num_extra_tokens"]
        num_inputs = num_queries.new_full([B], N, dtype=torch.double)
        dge_cp = self.router.complexity(num_inputs, num_queries)
        static_cp = self.complexity_handler(num_inputs, num_inputs) + dge_cp
        dynamic_cp = self.complexity_handler(num_inputs, num_queries) + dge_cp
        return {"static": static_cp, "dynamic": dynamic_cp}

    def compress(self, x, H, W):
        """x [B,N,C] -> packed queries [L,C] (``dge.py:61-85``)."""
        if self.training:
            return self._compress_train(x, H, W)
        require_cuda(x)
        x = x.contiguous()
        B, N, C = x.shape
        num_extra_tokens = N - H * W
        r = self.region_size
        S = self.splits.numel()
        gate = torch.empty(B, H // r, W // r, S, dtype=torch.float32, device=x.device)
        indices = torch.empty(B, H // r, W // r, dtype=torch.int32, device=x.device)
        gate_w = self.router.gate.weight.detach().float().contiguous()
        gate_b = self.router.gate.bias.detach().float().contiguous()
        _lib.check(_lib.lib().vtp_router_gate(
            ptr(x), dtype_code(x.dtype), B, H, W, C, num_extra_tokens, r, ptr(gate_w), ptr(gate_b), S, ptr(gate),
            ptr(indices), stream_ptr(x.device)))
        patches, batches = grained_sample_index_to_patch(indices, self.splits, r, num_extra_tokens)
        comp = grained_sample_compress(x, patches, H, W, num_extra_tokens)
        self.states.update({
            "comp": comp, "input": x, "patches": patches, "batches": batches,
            "gate": gate, "size": (H, W), "num_extra_tokens": num_extra_tokens,
        })
        return comp

    def decompress(self, x):
        """packed queries [L,C] -> tokens [B,N,C]: input + replicate(x - comp) (``dge.py:87-112``)."""
        if self.training:
            return self._decompress_train(x)
        st = self.states
        ref = st["input"]
        B, N, C = ref.shape
        H, W = st["size"]
        x = x.contiguous()
        p32 = st["patches"]._vtp_i32
        out = torch.empty_like(ref)
        _lib.check(_lib.lib().vtp_unpool_add(
            ptr(x), ptr(st["comp"]), dtype_code(x.dtype), B, N, C, W, st["num_extra_tokens"], ptr(p32), None,
            p32.shape[0], ptr(ref), ptr(out), stream_ptr(x.device)))
        return out

    # ------------------------------------------------------------------ training mode
    def _compress_train(self, x, H, W):
        """``dge.py:61-85`` with ``self.training``: hard Gumbel-softmax gate (straight-through), then
        either every grain of every region (dense) or the sampled grain only (``sparse_train``)."""
        B, N, C = x.shape
        num_extra_tokens = N - H * W
        gate = self.router(x[:, num_extra_tokens:, :].reshape(B, H, W, C))
        gate = F.gumbel_softmax(gate, dim=-1, hard=True)
        if not self.sparse_train:
            patches = None
            comp, batches = grained_sample_compress_dense(x, self.splits, self.region_size, H, W, num_extra_tokens)
        else:
            indices = gate.argmax(dim=-1)
            patches, batches = grained_sample_index_to_patch(indices, self.splits, self.region_size,
                                                             num_extra_tokens)
            comp = grained_sample_compress(x, patches, H, W, num_extra_tokens)
        self.states.update({
            "comp": comp, "input": x, "patches": patches, "batches": batches,
            "gate": gate, "size": (H, W), "num_extra_tokens": num_extra_tokens,
        })
        return comp

    def _decompress_train(self, x):
        """``dge.py:87-112`` with ``self.training``: the gate value (1 in the forward pass, carrying the
        straight-through gradient in the backward pass) multiplies the update of every query."""
        st = self.states
        x = x - st["comp"]
        H, W = st["size"]
        num_extra_tokens = st["num_extra_tokens"]
        if not self.sparse_train:
            return grained_sample_decompress_dense(x, st["gate"], st["input"], self.splits, self.region_size,
                                                   H, W, num_extra_tokens, True)
        B, N, C = st["input"].shape
        r = self.region_size
        gate = st["gate"].max(dim=-1, keepdim=True)[0]                       # [B,Hr,Wr,1]
        Hr, Wr = gate.shape[1:3]
        gate = gate.reshape(B, Hr, 1, Wr, 1, 1).expand(B, Hr, r, Wr, r, 1).reshape(B, H * W, 1)
        if num_extra_tokens > 0:
            gate = torch.cat([gate.new_ones([B, num_extra_tokens, 1]), gate], dim=1)
        gate = grained_sample_compress(gate, st["patches"], H, W, num_extra_tokens)
        return grained_sample_decompress(x * gate, st["patches"], st["input"], H, W, num_extra_tokens, True)
