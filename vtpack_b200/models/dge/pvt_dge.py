"""Mirror of the reference's PVT+DGE block (``vtpack/models/dge/pvt_dge.py:19-146``): the
same class names, constructor arguments and state_dict keys, with ``Block.forward(x, H, W)`` as
one call into the CUDA library.  Keys and values come from the normed tokens reduced by the
stride-``sr_ratio`` convolution ``attn.sr`` and the LayerNorm ``attn.norm``; everything else is
the DeiT+DGE block.  ``PyramidVisionTransformer`` (``pvt_dge.py:182-337``) sequences the stages
through the library's entry points: patch embedding = im2col + Linear + LayerNorm, position
embedding / cls rows = ``vtp_add_rows``, blocks, and between stages the token rows themselves
stand for the ``[B, C, H, W]`` map (``vtp_token_im2col`` gathers the 2 x 2 windows from them).
A block in training mode (``module.train()``) runs the reference's differentiable sequence
(``pvt_dge.py:77-146``) like the DeiT+DGE mirror does: dense layers through PyTorch autograd, token
movement and ragged attention products through this library's differentiable ops.
"""
import ctypes
from functools import partial

import torch
import torch.nn as nn

from ... import _lib
from ...layers import DynamicGrainedEncoder, batched_sparse_attention, batched_sparse_gemm
from ...runtime import dtype_code, ptr, require_cuda, scratch, scratch_generation, stream_ptr
from .deit_dge import DropPath, Mlp, _WeightPack, _pack_block, _shape_struct

__all__ = ["Mlp", "Attention", "Block", "PatchEmbed", "PyramidVisionTransformer",
           "pvt_dge_s124_tiny_256", "pvt_dge_s124_small_256", "pvt_dge_s124_medium_256", "pvt_dge_s124_large_256"]


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

    def forward(self, x, q, H, W, q_lengths):
        """x [B,N,C] normed tokens, q [L,C] normed queries -> [L,C] (``pvt_dge.py:77-114``), op by op
        through the parameters' own modules; differentiable in training mode.  The eval-mode fast
        path is ``Block.forward``, which never comes through here."""
        B, N, C = x.shape
        h, d = self.num_heads, C // self.num_heads
        q = self.q(q).reshape(-1, h, d).permute(1, 0, 2)
        if self.sr_ratio > 1:
            x_ = x.permute(0, 2, 1).reshape(B, C, H, W)
            x_ = self.norm(self.sr(x_).reshape(B, C, -1).permute(0, 2, 1))
            kv = self.kv(x_)
        else:
            kv = self.kv(x)
        kv = kv.reshape(B, -1, 2, h, d).permute(2, 3, 0, 1, 4)
        k, v = kv[0], kv[1]
        n_keys = kv.shape[3]
        if not self.training:
            o = batched_sparse_attention(q, k, v, q_lengths, self.scale).transpose(0, 1).reshape(-1, C)
        elif int(q_lengths.max() - q_lengths.min()) == 0:
            q = q.reshape(h, B, -1, d)
            attn = self.attn_drop(((q @ k.transpose(-1, -2)) * self.scale).softmax(dim=-1, dtype=v.dtype))
            o = (attn @ v).permute(1, 2, 0, 3).reshape(-1, C)
        else:
            kv_lengths = q_lengths.new_full([B], n_keys)
            k, v = k.reshape(h, -1, d), v.reshape(h, -1, d)
            attn = batched_sparse_gemm(q, k, q_lengths, kv_lengths, False, True) * self.scale
            attn = self.attn_drop(attn.softmax(dim=-1, dtype=v.dtype))
            o = batched_sparse_gemm(attn, v, q_lengths, kv_lengths, False, False).transpose(0, 1).reshape(-1, C)
        return self.proj_drop(self.proj(o))

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
        self.drop_path = DropPath(drop_path) if drop_path > 0. else nn.Identity()   # training mode only
        self.norm2 = norm_layer(dim)
        self.mlp = Mlp(in_features=dim, hidden_features=int(dim * mlp_ratio), act_layer=act_layer, drop=drop)
        self.dge = DynamicGrainedEncoder(in_channels=dim, split_sizes=split_sizes, complexity_handler=self.complexity)
        self.split_sizes = list(split_sizes)
        self.flags = 0
        self.fold_layernorm = sr_ratio <= 1      # bf16: norm1 into q and kv, norm2 into fc1 (GEMM epilogues)
        self.fold_q_fc1 = sr_ratio > 1           # with a spatial reduction: q and fc1 only, the keys are normalised
                                                 # on the way into the reducing convolution (the library runs norm2
                                                 # as its own pass where C <= 128: the fold does not pay there)
        self._pack = _WeightPack()

    def complexity(self, num_inputs, num_queries):
        comp = num_inputs * self.dim * 2  # norm1 and norm2
        comp += self.attn.complexity(num_inputs, num_queries)
        comp += self.mlp.complexity(num_inputs, num_queries)
        return comp

    def forward(self, x, H, W, forced_gate=None):
        """x [B, N, C] with N = H*W (+ extra tokens when sr_ratio == 1) -> [B, N, C]
        (``pvt_dge.py:140-146``), one C-ABI call.  ``forced_gate`` (fp32 [B,Hr,Wr,n_splits])
        replaces the router output.  In training mode: the reference's differentiable sequence."""
        if self.training:
            q = self.dge.compress(x, H, W)
            q = q + self.drop_path(self.attn(self.norm1(x), self.norm1(q), H, W, self.dge.states["batches"]))
            q = q + self.drop_path(self.mlp(self.norm2(q)))
            return self.dge.decompress(q)
        require_cuda(x)
        x = x.contiguous()
        B, N, C = x.shape
        s = _shape_struct(x.dtype, B, H, W, N - H * W, C, self.attn.num_heads, self.mlp.fc1.out_features,
                          self.split_sizes, self.norm1.eps, self.flags, self.attn.scale)
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


def stage_forward(blocks, x, H, W):
    """Eval forward of a stage's blocks (``pvt_dge.py:318-319``: ``for blk in block: x = blk(x, H, W)``) as ONE
    C-ABI call, ``vtp_dge_blocks_forward``: same results as calling the blocks one by one, but a block whose
    predecessor ran with folded LayerNorms finds its router decisions, per-image counts and token statistics
    already written by the predecessor's unpool.  Every block's ``dge.states`` is filled as by its own call."""
    blocks = list(blocks)
    require_cuda(x)
    x = x.contiguous()
    B, N, C = x.shape
    b0 = blocks[0]
    s = _shape_struct(x.dtype, B, H, W, N - H * W, C, b0.attn.num_heads, b0.mlp.fc1.out_features,
                      b0.split_sizes, b0.norm1.eps, b0.flags, b0.attn.scale)
    if b0.attn.sr_ratio > 1:
        s.sr_ratio = b0.attn.sr_ratio
        s.sr_eps = float(b0.attn.norm.eps)
    for blk in blocks[1:]:
        same = (blk.attn.num_heads == b0.attn.num_heads and blk.mlp.fc1.out_features == b0.mlp.fc1.out_features
                and blk.split_sizes == b0.split_sizes and blk.norm1.eps == b0.norm1.eps and blk.flags == b0.flags
                and blk.attn.scale == b0.attn.scale and blk.attn.sr_ratio == b0.attn.sr_ratio)
        if not same:
            raise ValueError("stage_forward: the blocks of a stage must share one shape")
    packs = (_lib.BlockWeights * len(blocks))(*[_pack_block(blk, x.dtype) for blk in blocks])
    lib = _lib.lib()
    nbytes = lib.vtp_block_workspace_bytes(ctypes.byref(s))
    _lib.check(0 if nbytes >= 0 else int(nbytes))
    ws = scratch(x.device, nbytes)
    out = torch.empty_like(x)
    counts = torch.empty(len(blocks), B, dtype=torch.int32, device=x.device)
    _lib.check(lib.vtp_dge_blocks_forward(ctypes.byref(s), packs, len(blocks), ptr(x), ptr(out), ptr(counts), ptr(ws),
                                          nbytes, stream_ptr(x.device)))
    for i, blk in enumerate(blocks):
        # (the input of a block after the first is overwritten in place; the complexity accounting only takes
        # its shape, which the stage's output buffer has too)
        blk.dge.states.update({"batches_device": counts[i], "input": x if i == 0 else out, "gate": None,
                               "size": (H, W), "num_extra_tokens": N - H * W})
    return out


class PatchEmbed(nn.Module):
    """Image (or previous stage's map) to patch embedding: convolution with kernel = stride =
    patch_size, then LayerNorm (``pvt_dge.py:149-179``)."""

    def __init__(self, img_size=224, patch_size=16, in_chans=3, embed_dim=768):
        super().__init__()
        self.img_size = (img_size, img_size)
        self.patch_size = (patch_size, patch_size)
        self.H, self.W = img_size // patch_size, img_size // patch_size
        self.num_patches = self.H * self.W
        self.proj = nn.Conv2d(in_chans, embed_dim, kernel_size=patch_size, stride=patch_size)
        self.norm = nn.LayerNorm(embed_dim)

    def forward(self, x):
        """[B, C_in, H, W] -> (tokens [B, H/p * W/p, C], (H/p, W/p)) (``pvt_dge.py:170-179``); used by the
        training-mode forward only, eval mode runs the embedding through the library."""
        H, W = x.shape[2] // self.patch_size[0], x.shape[3] // self.patch_size[1]
        return self.norm(self.proj(x).flatten(2).transpose(1, 2)), (H, W)

    def complexity(self, num_inputs, num_queries):
        comp = num_inputs * self.proj.in_channels * self.proj.out_channels
        comp += num_inputs / (self.patch_size[0] * self.patch_size[1]) * self.proj.out_channels  # norm
        return comp


def _matmul_rows(cols, weight, bias, flags=0, out_dtype=None):
    """cols [M, K] x weight [N, K]^T + bias through vtp_linear."""
    M, K = cols.shape
    N = weight.shape[0]
    y = torch.empty(M, N, dtype=out_dtype or cols.dtype, device=cols.device)
    b = None if bias is None else bias.detach().float().contiguous()
    _lib.check(_lib.lib().vtp_linear(ptr(cols), K, ptr(weight), ptr(b), None, 0, ptr(y), N, dtype_code(cols.dtype), M,
                                     None, N, K, flags, stream_ptr(cols.device)))
    return y


def _norm_rows(x, rows, C, row_stride, ln, eps=None, wb=None):
    y = torch.empty(rows, C, dtype=x.dtype, device=x.device)
    # both fp32 copies must be alive together: a temporary freed between the two would hand its memory to the other
    w, b = wb if wb is not None else (ln.weight.detach().float().contiguous(), ln.bias.detach().float().contiguous())
    _lib.check(_lib.lib().vtp_layernorm(ptr(x), dtype_code(x.dtype), rows, None, C, row_stride, ptr(w), ptr(b),
                                        float(ln.eps if eps is None else eps), ptr(y), stream_ptr(x.device)))
    return y


class PyramidVisionTransformer(nn.Module):

    def __init__(self, img_size=224, patch_size=16, in_chans=3, num_classes=1000, embed_dims=[64, 128, 256, 512],
                 num_heads=[1, 2, 4, 8], mlp_ratios=[4, 4, 4, 4], qkv_bias=False, qk_scale=None, drop_rate=0.,
                 attn_drop_rate=0., drop_path_rate=0., norm_layer=nn.LayerNorm,
                 depths=[3, 4, 6, 3], sr_ratios=[8, 4, 2, 1], num_stages=4,
                 split_sizes=[[2, 1], [2, 1], [2, 1], [2, 1]]):
        super().__init__()
        assert in_chans == 3, "the image im2col kernel is written for 3 channels"
        self.embed_dims = embed_dims
        self.num_classes = num_classes
        self.depths = depths
        self.num_stages = num_stages
        self.img_size = img_size
        dpr = [v.item() for v in torch.linspace(0, drop_path_rate, sum(depths))]   # drop rate grows with depth
        cur = 0
        for i in range(num_stages):
            patch_embed = PatchEmbed(img_size=img_size if i == 0 else img_size // (2 ** (i + 1)),
                                     patch_size=patch_size if i == 0 else 2,
                                     in_chans=in_chans if i == 0 else embed_dims[i - 1], embed_dim=embed_dims[i])
            num_patches = patch_embed.num_patches if i != num_stages - 1 else patch_embed.num_patches + 1
            pos_embed = nn.Parameter(torch.zeros(1, num_patches, embed_dims[i]))
            block = nn.ModuleList([Block(
                dim=embed_dims[i], num_heads=num_heads[i], mlp_ratio=mlp_ratios[i], qkv_bias=qkv_bias,
                qk_scale=qk_scale, drop=drop_rate, attn_drop=attn_drop_rate, drop_path=dpr[cur + j],
                norm_layer=norm_layer, sr_ratio=sr_ratios[i], split_sizes=split_sizes[i]) for j in range(depths[i])])
            cur += depths[i]
            setattr(self, f"patch_embed{i + 1}", patch_embed)
            setattr(self, f"pos_embed{i + 1}", pos_embed)
            setattr(self, f"pos_drop{i + 1}", nn.Dropout(p=drop_rate))
            setattr(self, f"block{i + 1}", block)
        self.norm = norm_layer(embed_dims[3]) if num_classes > 0 else nn.Identity()
        self.cls_token = nn.Parameter(torch.zeros(1, 1, embed_dims[3]))
        self.head = nn.Linear(embed_dims[3], num_classes) if num_classes > 0 else nn.Identity()
        for i in range(num_stages):
            nn.init.trunc_normal_(getattr(self, f"pos_embed{i + 1}"), std=.02)
        nn.init.trunc_normal_(self.cls_token, std=.02)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.trunc_normal_(m.weight, std=.02)
                if m.bias is not None:
                    nn.init.constant_(m.bias, 0)
            elif isinstance(m, nn.LayerNorm):
                nn.init.constant_(m.bias, 0)
                nn.init.constant_(m.weight, 1.0)
            elif isinstance(m, DynamicGrainedEncoder):
                m.router.init_parameters()
        self.last_counts = None

    def _const(self, name, sources, make, extra=()):
        """A tensor derived from parameters only (a weight matrix in GEMM layout and dtype, fp32 copies of bias and
        LayerNorm vectors, the resized position rows): made once and kept until one of ``sources`` changes, so an
        eval forward launches no conversion copies of its own."""
        cache = self.__dict__.setdefault("_consts", {})
        key = tuple((p.data_ptr(), p._version, p.dtype) for p in sources) + tuple(extra)
        hit = cache.get(name)
        if hit is None or hit[0] != key:
            with torch.no_grad():
                hit = (key, make())
            cache[name] = hit
        return hit[1]

    def forward_graph(self, x):
        """Eval forward through a CUDA graph captured for this input buffer (its contents may change between
        calls, its address and shape may not); returns the graph's own output tensor, overwritten by the next
        call.  The stages are sequenced from Python through some sixty small launches per forward; replaying
        them as one graph removes the host work between them.  The graph is captured again when a parameter
        has changed, when the per-device scratch buffer has been replaced, or for another input buffer."""
        if self.training:
            raise RuntimeError("forward_graph is an eval-mode path")
        key = (x.data_ptr(), tuple(x.shape), x.dtype,
               tuple((p.data_ptr(), p._version) for p in self.parameters()))
        g = getattr(self, "_graph", None)
        if g is None or g["key"] != key or g["scratch_gen"] != scratch_generation(x.device):
            cur = torch.cuda.current_stream(x.device)
            side = torch.cuda.Stream(x.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):          # warm-up outside capture: scratch, attributes, weight packs
                for _ in range(2):
                    self.forward(x)
            cur.wait_stream(side)
            torch.cuda.synchronize(x.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self.forward(x)
            g = {"key": key, "graph": graph, "out": out, "counts": self.last_counts, "x": x,
                 "scratch": scratch(x.device, 1), "scratch_gen": scratch_generation(x.device)}
            self._graph = g
        g["graph"].replay()
        self.last_counts = g["counts"]
        return g["out"]

    def _stage_pos_embed(self, pos_embed, patch_embed, H, W):
        """The stage's position embedding, bilinearly resized when the token grid is not the one it
        was made for (``pvt_dge.py:286-293``)."""
        if H * W == patch_embed.num_patches:
            return pos_embed
        grid = pos_embed.reshape(1, patch_embed.H, patch_embed.W, -1).permute(0, 3, 1, 2)
        grid = torch.nn.functional.interpolate(grid, size=(H, W), mode="bilinear", align_corners=False)
        return grid.reshape(1, -1, H * W).permute(0, 2, 1)

    def _forward_train(self, x):
        """Training mode (``pvt_dge.py:295-337``): the stages op by op in the parameters' dtype and in
        autograd, blocks in their training mode; with ``num_classes == 0`` the feature pyramid
        ``{"res2": .., "res5": ..}`` of ``[B, C_i, H_i, W_i]`` maps is returned."""
        B = x.shape[0]
        x = x.to(self.cls_token.dtype)
        outputs = {}
        for i in range(self.num_stages):
            patch_embed = getattr(self, f"patch_embed{i + 1}")
            pos_embed = getattr(self, f"pos_embed{i + 1}")
            x, (H, W) = patch_embed(x)
            if i == self.num_stages - 1:
                x = torch.cat((self.cls_token.expand(B, -1, -1), x), dim=1)
                pos_embed = torch.cat((pos_embed[:, 0:1], self._stage_pos_embed(pos_embed[:, 1:], patch_embed, H, W)),
                                      dim=1)
            else:
                pos_embed = self._stage_pos_embed(pos_embed, patch_embed, H, W)
            x = getattr(self, f"pos_drop{i + 1}")(x + pos_embed)
            for blk in getattr(self, f"block{i + 1}"):
                x = blk(x, H, W)
            if i != self.num_stages - 1:
                x = x.reshape(B, H, W, -1).permute(0, 3, 1, 2).contiguous()
                outputs[f"res{i + 2}"] = x
            elif self.num_classes == 0:
                outputs[f"res{i + 2}"] = x[:, 1:].reshape(B, H, W, -1).permute(0, 3, 1, 2).contiguous()
        if self.num_classes == 0:
            return outputs
        return self.head(self.norm(x)[:, 0])

    def forward(self, x):
        """images [B,3,S,S] on the device -> logits fp32 [B,num_classes], or with ``num_classes == 0``
        the feature pyramid ``{"res2": .., "res5": ..}`` of ``[B, C_i, H_i, W_i]`` maps
        (``pvt_dge.py:295-337``).  S may differ from the training resolution (the position embeddings
        are resized bilinearly, ``pvt_dge.py:286-293``) as long as every stage's grid divides into 4 x 4
        regions and reduction windows.  In training mode: the differentiable op-by-op sequence."""
        if self.training:
            return self._forward_train(x)
        require_cuda(x)
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.float()
        x = x.contiguous()
        B, _, S, _ = x.shape
        dtype = self.cls_token.dtype
        lib, st = _lib.lib(), stream_ptr(x.device)
        counts, outputs = [], {}
        tokens, H, W = None, 0, 0
        for i in range(self.num_stages):
            pe = getattr(self, f"patch_embed{i + 1}")
            pos_full = getattr(self, f"pos_embed{i + 1}").detach()
            C = self.embed_dims[i]
            P = pe.patch_size[0]
            if i == 0:
                if S % P:
                    raise ValueError(f"input size {S} is not a multiple of the patch size {P}")
                H = W = S // P
                KP = 3 * P * P
                padded = dtype == torch.bfloat16 and P % 8 != 0 and KP % 64 != 0
                ld = (KP + 63) // 64 * 64 if padded else KP
                wm = self._const(f"wm{i}", (pe.proj.weight,), lambda: torch.nn.functional.pad(
                    pe.proj.weight.detach().reshape(C, -1).to(dtype), (0, ld - KP)).contiguous(), (dtype, ld))
                if padded:
                    # 48 columns: pad the reduction to a whole 64-element block (zero columns in the rows and in
                    # the weight), which takes the GEMM from the CUDA-core kernel to the tensor-core one
                    cols = torch.empty(B * H * W, ld, dtype=dtype, device=x.device)
                    _lib.check(lib.vtp_patch_im2col_padded(ptr(x), dtype_code(x.dtype), B, S, P, dtype_code(dtype),
                                                           ptr(cols), ld, st))
                else:
                    cols = torch.empty(B * H * W, KP, dtype=dtype, device=x.device)
                    _lib.check(lib.vtp_patch_im2col(ptr(x), dtype_code(x.dtype), B, S, P, dtype_code(dtype), ptr(cols),
                                                    None, None, C, None, st))
            else:
                cols = torch.empty(B * (H // P) * (W // P), P * P * tokens.shape[-1], dtype=dtype, device=x.device)
                _lib.check(lib.vtp_token_im2col(ptr(tokens), dtype_code(dtype), B, H, W, tokens.shape[-1], P, ptr(cols), st))
                H, W = H // P, W // P
                wm = self._const(f"wm{i}", (pe.proj.weight,), lambda: pe.proj.weight.detach().permute(0, 2, 3, 1)
                                 .reshape(C, -1).to(dtype).contiguous(), (dtype,))
            bias = self._const(f"eb{i}", (pe.proj.bias,), lambda: pe.proj.bias.detach().float().contiguous())
            wb = self._const(f"en{i}", (pe.norm.weight, pe.norm.bias), lambda: (
                pe.norm.weight.detach().float().contiguous(), pe.norm.bias.detach().float().contiguous()))
            y = _matmul_rows(cols, wm, bias)
            HW = H * W
            last = i == self.num_stages - 1
            # the stage's position rows ([cls row;] grid rows), resized when the grid is not the trained one
            def make_pos(pos_full=pos_full, pe=pe, H=H, W=W, last=last):
                if last:
                    pos = torch.cat((pos_full[:, 0:1], self._stage_pos_embed(pos_full[:, 1:], pe, H, W)), dim=1)
                else:
                    pos = self._stage_pos_embed(pos_full, pe, H, W)
                return pos[0].to(dtype).contiguous()
            pos = self._const(f"pos{i}", (getattr(self, f"pos_embed{i + 1}"),), make_pos, (dtype, H, W))
            tokens = torch.empty(B, HW + (1 if last else 0), C, dtype=dtype, device=x.device)
            # tokens = norm(proj(x)) + pos_embed in one pass (written behind the cls slot in the last stage)
            _lib.check(lib.vtp_layernorm_add_rows(ptr(y), dtype_code(dtype), B * HW, C, C, ptr(wb[0]), ptr(wb[1]),
                                                  float(pe.norm.eps), ptr(pos), HW, 1 if last else 0, ptr(tokens), HW,
                                                  HW + (1 if last else 0), 1 if last else 0, st))
            if last:
                cls = self._const("cls", (self.cls_token,), lambda: self.cls_token.detach().reshape(1, C).contiguous())
                _lib.check(lib.vtp_add_rows(ptr(cls), 1, ptr(pos), 1, 0, ptr(tokens), 1, HW + 1, 0, dtype_code(dtype),
                                            B, C, st))
            stage = getattr(self, f"block{i + 1}")
            tokens = stage_forward(stage, tokens, H, W)
            counts.extend(blk.dge.states["batches_device"] for blk in stage)
            if self.num_classes == 0:
                grid_rows = tokens[:, 1:] if last else tokens
                outputs[f"res{i + 2}"] = grid_rows.reshape(B, H, W, C).permute(0, 3, 1, 2).contiguous()
        self.last_counts = counts
        if self.num_classes == 0:
            return outputs
        N = tokens.shape[1]
        C = tokens.shape[2]
        wb = self._const("norm", (self.norm.weight, self.norm.bias), lambda: (
            self.norm.weight.detach().float().contiguous(), self.norm.bias.detach().float().contiguous()))
        cls_n = _norm_rows(tokens, B, C, N * C, self.norm, wb=wb)
        head_w = self._const("head_w", (self.head.weight,), lambda: self.head.weight.detach().to(dtype).contiguous(), (dtype,))
        head_b = self._const("head_b", (self.head.bias,), lambda: self.head.bias.detach().float().contiguous())
        logits = _matmul_rows(cls_n, head_w, head_b, flags=_lib.FLAG_OUT_F32, out_dtype=torch.float32)
        self.last_counts = counts
        return logits


def _pvt(depths, **kwargs):
    return PyramidVisionTransformer(
        img_size=256, patch_size=4, embed_dims=[64, 128, 320, 512], num_heads=[1, 2, 5, 8], mlp_ratios=[8, 8, 4, 4],
        qkv_bias=True, norm_layer=partial(nn.LayerNorm, eps=1e-6), depths=depths, sr_ratios=[8, 4, 2, 1],
        split_sizes=[[4, 2, 1], [4, 2, 1], [4, 2, 1], [4, 2, 1]], **kwargs)


def pvt_dge_s124_tiny_256(pretrained=False, **kwargs):
    return _pvt([2, 2, 2, 2], **kwargs)


def pvt_dge_s124_small_256(pretrained=False, **kwargs):
    return _pvt([3, 4, 6, 3], **kwargs)


def pvt_dge_s124_medium_256(pretrained=False, **kwargs):
    return _pvt([3, 4, 18, 3], **kwargs)


def pvt_dge_s124_large_256(pretrained=False, **kwargs):
    return _pvt([3, 8, 27, 3], **kwargs)
