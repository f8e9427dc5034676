"""DeiT + Dynamic Grained Encoder on B200: fused eval-mode inference, op-by-op training mode.

Same classes, constructor arguments, parameter names (state_dict keys) and factory
names as ``vtpack/models/dge/deit_dge.py`` so checkpoints of the reference load
unchanged.  ``Block.forward`` and ``VisionTransformer.forward`` run as one C-ABI call
each (``vtp_dge_block_forward`` / ``vtp_deit_dge_forward``): every kernel is launched
from C++ on the current stream and the variable number of queries never leaves the
device.  ``Block.forward_unfused`` follows the reference's op-by-op sequence through
the ``vtpack_b200.layers`` functions (it synchronises once per block, as the reference
does).  In training mode (``module.train()``) the blocks run the reference's training sequence
(``deit_dge.py:79-98,123-130``): dense layers, LayerNorm, softmax and GELU through PyTorch's autograd
as in the reference, token movement and the ragged attention products through this library's
differentiable ``grained_sample_compress`` / ``grained_sample_decompress`` / ``batched_sparse_gemm``.
"""
import ctypes
import math
from functools import partial

import torch
import torch.nn as nn

from ... import _lib
from ...layers import DynamicGrainedEncoder, batched_sparse_attention, batched_sparse_gemm
from ...runtime import dtype_code, ptr, require_cuda, scratch, scratch_generation, stream_ptr

__all__ = [
    "deit_dge_s124_tiny_patch16_256", "deit_dge_s124_small_patch16_256",
    "deit_dge_s124_base_patch16_256",
]


def _linear(x, lin: nn.Linear, residual=None, gelu=False, flags=0):
    """y = act(x W^T + b) (+ residual) through vtp_linear; x is [M,K] contiguous."""
    x = x.contiguous()
    M, K = x.shape
    N = lin.out_features
    y = torch.empty(M, N, dtype=x.dtype, device=x.device)
    w = lin.weight.detach().to(x.dtype).contiguous()
    b = None if lin.bias is None else lin.bias.detach().float().contiguous()
    f = flags | (_lib.FLAG_GELU if gelu else 0)
    if residual is not None:
        residual = residual.contiguous()
    _lib.check(_lib.lib().vtp_linear(
        ptr(x), K, ptr(w), ptr(b), ptr(residual), N, ptr(y), N, dtype_code(x.dtype), M, None, N, K, f,
        stream_ptr(x.device)))
    return y


def _layernorm(x, ln: nn.LayerNorm):
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    y = torch.empty_like(x2)
    # both fp32 copies must be alive together: a temporary freed between the two would hand its memory to the other
    w, b = ln.weight.detach().float().contiguous(), ln.bias.detach().float().contiguous()
    _lib.check(_lib.lib().vtp_layernorm(
        ptr(x2), dtype_code(x2.dtype), x2.shape[0], None, x2.shape[1], x2.shape[1], ptr(w), ptr(b),
        float(ln.eps), ptr(y), stream_ptr(x.device)))
    return y.reshape(x.shape)


class Mlp(nn.Module):
    def __init__(self, in_features, hidden_features=None, out_features=None, act_layer=nn.GELU, drop=0.):
        super().__init__()
        out_features = out_features or in_features
        hidden_features = hidden_features or in_features
        self.fc1 = nn.Linear(in_features, hidden_features)
        self.act = act_layer()
        self.fc2 = nn.Linear(hidden_features, out_features)
        self.drop = nn.Dropout(drop)

    def complexity(self, num_inputs, num_queries):
        comp = num_queries * self.fc1.in_features * self.fc1.out_features
        comp += num_queries * self.fc1.out_features
        comp += num_queries * self.fc2.in_features * self.fc2.out_features
        return comp

    def forward(self, x, residual=None):
        if self.training:
            y = self.drop(self.fc2(self.drop(self.act(self.fc1(x)))))           # deit_dge.py:38-44
            return y if residual is None else residual + y
        return _linear(_linear(x, self.fc1, gelu=True), self.fc2, residual=residual)


class Attention(nn.Module):
    def __init__(self, dim, num_heads=8, qkv_bias=False, qk_scale=None, attn_drop=0., proj_drop=0.):
        super().__init__()
        self.dim = dim
        self.num_heads = num_heads
        head_dim = dim // num_heads
        self.scale = qk_scale or head_dim ** -0.5
        self.q = nn.Linear(dim, dim, bias=qkv_bias)
        self.kv = nn.Linear(dim, dim * 2, bias=qkv_bias)
        self.attn_drop = nn.Dropout(attn_drop)
        self.proj = nn.Linear(dim, dim)
        self.proj_drop = nn.Dropout(proj_drop)

    def complexity(self, num_inputs, num_queries):
        c = self.dim
        comp = num_queries * c ** 2
        comp += (num_inputs * c ** 2) * 2
        comp += (num_queries * num_inputs * c) * 2
        comp += num_queries * num_inputs * self.num_heads * 3
        comp += num_queries * c ** 2
        return comp

    def forward(self, x, q, q_lengths, residual=None):
        """x [B,N,C] (normed tokens), q [L,C] (normed queries) -> [L,C]
        (``deit_dge.py:70-98``)."""
        B, N, C = x.shape
        h = self.num_heads
        if self.training:
            y = self._forward_train(x, q, q_lengths)
            return y if residual is None else residual + y
        qh = _linear(q, self.q).reshape(-1, h, C // h).permute(1, 0, 2)
        kv = _linear(x.reshape(B * N, C), self.kv).reshape(B, N, 2, h, C // h).permute(2, 3, 0, 1, 4)
        o = batched_sparse_attention(qh, kv[0], kv[1], q_lengths, self.scale)
        o = o.transpose(0, 1).reshape(-1, C)
        return _linear(o, self.proj, residual=residual)

    def _forward_train(self, x, q, q_lengths):
        """Training branch of ``deit_dge.py:79-98``: a batched product when every image has the same
        number of queries, else the two ragged products with the softmax between them."""
        B, N, C = x.shape
        h, d = self.num_heads, C // self.num_heads
        q = self.q(q).reshape(-1, h, d).permute(1, 0, 2)
        kv = self.kv(x).reshape(B, N, 2, h, d).permute(2, 3, 0, 1, 4)
        k, v = kv[0], kv[1]
        if int(q_lengths.max() - q_lengths.min()) == 0:
            q = q.reshape(h, B, -1, d)
            attn = (q @ k.transpose(-1, -2)) * self.scale
            attn = self.attn_drop(attn.softmax(dim=-1, dtype=v.dtype))
            o = (attn @ v).permute(1, 2, 0, 3).reshape(-1, C)
        else:
            kv_lengths = q_lengths.new_full([B], N)
            k = k.reshape(h, -1, d)
            v = v.reshape(h, -1, d)
            attn = batched_sparse_gemm(q, k, q_lengths, kv_lengths, False, True) * self.scale
            attn = self.attn_drop(attn.softmax(dim=-1, dtype=v.dtype))
            o = batched_sparse_gemm(attn, v, q_lengths, kv_lengths, False, False)
            o = o.transpose(0, 1).reshape(-1, C)
        return self.proj_drop(self.proj(o))


class DropPath(nn.Module):
    """Stochastic depth: in training mode each row of the first axis keeps its residual branch with
    probability 1 - p, scaled by 1 / (1 - p); identity otherwise."""

    def __init__(self, p=0.):
        super().__init__()
        self.p = float(p)

    def forward(self, x):
        if not self.training or self.p == 0.:
            return x
        keep = 1.0 - self.p
        mask = x.new_empty((x.shape[0],) + (1,) * (x.dim() - 1)).bernoulli_(keep)
        return x * (mask / keep)


class _WeightPack:
    """Device pointers of one block's parameters in the layout the C ABI wants: matrices
    in the compute dtype, vectors fp32.  Rebuilt when a parameter changes."""

    def __init__(self):
        self.key = None
        self.tensors = None
        self.struct = None


def _param_key(mod: nn.Module, dtype):
    return (dtype, getattr(mod, "fold_layernorm", None), getattr(mod, "fold_q_fc1", None)) + tuple((p.data_ptr(), p._version, p.dtype) for p in mod.parameters())


def _pack_block(blk, dtype) -> _lib.BlockWeights:
    key = _param_key(blk, dtype)
    pk = blk._pack
    if pk.key != key:
        mat = lambda t: t.detach().to(dtype).contiguous()      # noqa: E731
        vec = lambda t: t.detach().float().contiguous()        # noqa: E731
        zeros = lambda n, ref: torch.zeros(n, dtype=torch.float32, device=ref.device)  # noqa: E731
        a, m = blk.attn, blk.mlp
        t = dict(
            norm1_w=vec(blk.norm1.weight), norm1_b=vec(blk.norm1.bias),
            q_w=mat(a.q.weight), q_b=vec(a.q.bias) if a.q.bias is not None else zeros(a.dim, a.q.weight),
            kv_w=mat(a.kv.weight),
            kv_b=vec(a.kv.bias) if a.kv.bias is not None else zeros(2 * a.dim, a.kv.weight),
            proj_w=mat(a.proj.weight), proj_b=vec(a.proj.bias),
            norm2_w=vec(blk.norm2.weight), norm2_b=vec(blk.norm2.bias),
            fc1_w=mat(m.fc1.weight), fc1_b=vec(m.fc1.bias),
            fc2_w=mat(m.fc2.weight), fc2_b=vec(m.fc2.bias),
            gate_w=vec(blk.dge.router.gate.weight), gate_b=vec(blk.dge.router.gate.bias),
        )
        sr = getattr(a, "sr", None)
        if sr is not None:
            # PVT spatial reduction: conv weight [C, C, sr, sr] -> matrix [C, sr*sr*C], columns (dy, dx, c_in)
            t["sr_w"] = mat(sr.weight.permute(0, 2, 3, 1).reshape(sr.weight.shape[0], -1))
            t["sr_b"] = vec(sr.bias) if sr.bias is not None else zeros(a.dim, sr.weight)
            t["sr_norm_w"], t["sr_norm_b"] = vec(a.norm.weight), vec(a.norm.bias)
        if dtype == torch.bfloat16 and (blk.fold_layernorm or (sr is not None and getattr(blk, "fold_q_fc1", False))):
            # LayerNorm folded into the Linear that follows it (weight preparation, once).  A block with a spatial
            # reduction folds q and fc1 only: its kv projection reads the reduced, separately normalised keys.
            folds = [("q", t["q_w"], t["q_b"], t["norm1_w"], t["norm1_b"]),
                     ("kv", t["kv_w"], t["kv_b"], t["norm1_w"], t["norm1_b"]),
                     ("fc1", t["fc1_w"], t["fc1_b"], t["norm2_w"], t["norm2_b"])]
            if sr is not None:
                del folds[1]
            for name, lin_w, lin_b, gw, gb in folds:
                wf = torch.empty_like(lin_w)
                sv = torch.empty(lin_w.shape[0], dtype=torch.float32, device=lin_w.device)
                cv = torch.empty_like(sv)
                _lib.check(_lib.lib().vtp_fold_layernorm(
                    ptr(lin_w), dtype_code(dtype), lin_w.shape[0], lin_w.shape[1], ptr(gw), ptr(gb), ptr(lin_b),
                    ptr(wf), ptr(sv), ptr(cv), stream_ptr(lin_w.device)))
                t[name + "_wf"], t[name + "_s"], t[name + "_c"] = wf, sv, cv
        s = _lib.BlockWeights()
        for k, v in t.items():
            setattr(s, k, v.data_ptr())
        pk.key, pk.tensors, pk.struct = key, t, s
    return pk.struct


def _shape_struct(x_dtype, B, H, W, num_extra, C, heads, hidden, splits, eps, flags, attn_scale=0.0):
    s = _lib.DgeShape()
    s.dtype = dtype_code(x_dtype)
    s.B, s.H, s.W, s.num_extra = B, H, W, num_extra
    s.C, s.heads, s.hidden = C, heads, hidden
    s.region = max(splits)
    s.n_splits = len(splits)
    for i, v in enumerate(splits):
        s.splits[i] = int(v)
    s.eps = float(eps)
    s.flags = int(flags)
    s.attn_scale = float(attn_scale)      # Attention.scale (qk_scale or head_dim ** -0.5)
    return s


class Block(nn.Module):

    def __init__(self, dim, num_heads, mlp_ratio=4., qkv_bias=False, qk_scale=None, drop=0., attn_drop=0.,
                 drop_path=0., act_layer=nn.GELU, norm_layer=nn.LayerNorm, split_sizes=[2, 1]):
        super().__init__()
        self.dim = dim
        self.norm1 = norm_layer(dim)
        self.attn = Attention(dim, num_heads=num_heads, qkv_bias=qkv_bias, qk_scale=qk_scale,
                              attn_drop=attn_drop, proj_drop=drop)
        self.drop_path = DropPath(drop_path) if drop_path > 0. else nn.Identity()   # training mode only
        self.norm2 = norm_layer(dim)
        mlp_hidden_dim = int(dim * mlp_ratio)
        self.mlp = Mlp(in_features=dim, hidden_features=mlp_hidden_dim, act_layer=act_layer, drop=drop)
        self.dge = DynamicGrainedEncoder(in_channels=dim, split_sizes=split_sizes,
                                         complexity_handler=self.complexity)
        self.split_sizes = list(split_sizes)
        self.flags = 0                          # _lib.FLAG_CUDA_CORES selects the CUDA-core kernels
        self.fold_layernorm = True              # bf16: LayerNorm applied inside the q / kv / fc1 GEMM epilogues
        self._pack = _WeightPack()

    def complexity(self, num_inputs, num_queries):
        comp = num_inputs * self.dim * 2
        comp += self.attn.complexity(num_inputs, num_queries)
        comp += self.mlp.complexity(num_inputs, num_queries)
        return comp

    def shape_struct(self, x):
        B, N, C = x.shape
        H = W = int(math.sqrt(N))
        return _shape_struct(x.dtype, B, H, W, N - H * W, C, self.attn.num_heads, self.mlp.fc1.out_features,
                             self.split_sizes, self.norm1.eps, self.flags, self.attn.scale)

    def forward(self, x, forced_gate=None, dense=False):
        """One C-ABI call for the whole block (``deit_dge.py:123-130``).  ``forced_gate``
        (fp32 [B,Hr,Wr,n_splits]) replaces the router output; ``dense`` runs the dense
        DeiT block built from the same weights instead.  In training mode: the reference's
        differentiable sequence."""
        if self.training:
            return self._forward_train(x)
        require_cuda(x)
        x = x.contiguous()
        s = self.shape_struct(x)
        w = _pack_block(self, x.dtype)
        lib = _lib.lib()
        nbytes = lib.vtp_block_workspace_bytes(ctypes.byref(s))
        ws = scratch(x.device, nbytes)
        out = torch.empty_like(x)
        if dense:
            _lib.check(lib.vtp_dense_block_forward(ctypes.byref(s), ctypes.byref(w), ptr(x), ptr(out), ptr(ws),
                                                   nbytes, stream_ptr(x.device)))
            return out
        counts = torch.empty(s.B, dtype=torch.int32, device=x.device)
        if forced_gate is not None:
            forced_gate = forced_gate.to(device=x.device, dtype=torch.float32).contiguous()
        _lib.check(lib.vtp_dge_block_forward(ctypes.byref(s), ctypes.byref(w), ptr(x), ptr(out), ptr(forced_gate),
                                             ptr(counts), ptr(ws), nbytes, stream_ptr(x.device)))
        self.dge.states.update({"batches_device": counts, "input": x, "gate": None, "size": (s.H, s.W),
                                "num_extra_tokens": s.num_extra})
        return out

    def _forward_train(self, x):
        """``deit_dge.py:123-130`` with ``self.training``."""
        B, N, C = x.shape
        H = W = int(math.sqrt(N))
        q = self.dge.compress(x, H, W)
        q = q + self.drop_path(self.attn(self.norm1(x), self.norm1(q), self.dge.states["batches"]))
        q = q + self.drop_path(self.mlp(self.norm2(q)))
        return self.dge.decompress(q)

    def forward_unfused(self, x):
        """The reference's sequence op by op through vtpack_b200.layers."""
        B, N, C = x.shape
        H = W = int(math.sqrt(N))
        q = self.dge.compress(x, H, W)
        q = self.attn(_layernorm(x, self.norm1), _layernorm(q, self.norm1), self.dge.states["batches"],
                      residual=q)
        q = self.mlp(_layernorm(q, self.norm2), residual=q)
        return self.dge.decompress(q)


class PatchEmbed(nn.Module):
    """Image to patch tokens: conv(kernel = stride = patch), flatten, transpose."""

    def __init__(self, img_size=224, patch_size=16, in_chans=3, embed_dim=768):
        super().__init__()
        self.img_size = img_size
        self.patch_size = patch_size
        self.num_patches = (img_size // patch_size) ** 2
        self.proj = nn.Conv2d(in_chans, embed_dim, kernel_size=patch_size, stride=patch_size)

    def forward(self, x):
        """Used by the training-mode forward only; eval mode runs the patch embedding inside the
        model's fused C-ABI call."""
        return self.proj(x).flatten(2).transpose(1, 2)


class VisionTransformer(nn.Module):
    """DeiT + DGE (``deit_dge.py:133-299``); cls token, no distillation token."""

    def __init__(self, img_size=224, patch_size=16, in_chans=3, num_classes=1000, embed_dim=768, depth=12,
                 num_heads=12, mlp_ratio=4., qkv_bias=True, qk_scale=None, representation_size=None,
                 distilled=False, drop_rate=0., attn_drop_rate=0., drop_path_rate=0., embed_layer=PatchEmbed,
                 norm_layer=None, act_layer=None, weight_init="", cls_token=True, split_sizes=[2, 1]):
        super().__init__()
        if distilled or representation_size or not cls_token or in_chans != 3:
            raise NotImplementedError("only the cls-token DeiT+DGE configuration is implemented")
        self.num_classes = num_classes
        self.num_features = self.embed_dim = embed_dim
        self.num_tokens = 1
        norm_layer = norm_layer or partial(nn.LayerNorm, eps=1e-6)
        act_layer = act_layer or nn.GELU
        self.patch_embed = embed_layer(img_size=img_size, patch_size=patch_size, in_chans=in_chans,
                                       embed_dim=embed_dim)
        num_patches = self.patch_embed.num_patches
        self.cls_token = nn.Parameter(torch.zeros(1, 1, embed_dim))
        self.dist_token = None
        self.pos_embed = nn.Parameter(torch.zeros(1, num_patches + self.num_tokens, embed_dim))
        self.pos_drop = nn.Dropout(p=drop_rate)
        dpr = [v.item() for v in torch.linspace(0, drop_path_rate, depth)]   # drop rate grows linearly with depth
        self.blocks = nn.Sequential(*[
            Block(dim=embed_dim, num_heads=num_heads, mlp_ratio=mlp_ratio, qkv_bias=qkv_bias, qk_scale=qk_scale,
                  drop=drop_rate, attn_drop=attn_drop_rate, drop_path=dpr[i], norm_layer=norm_layer,
                  act_layer=act_layer, split_sizes=split_sizes)
            for i in range(depth)])
        self.norm = norm_layer(embed_dim)
        self.pre_logits = nn.Identity()
        self.head = nn.Linear(self.num_features, num_classes)
        self.head_dist = None
        self.img_size, self.patch_size, self.depth = img_size, patch_size, depth
        self.split_sizes = list(split_sizes)
        self.flags = 0
        self.fold_layernorm = True
        self._pack = _WeightPack()
        self._graphs = {}
        self.last_counts = None
        # eval-mode options of the fused forward (vtp_forward_options):
        self.gate_image_bias = None     # fp32 [B, n_splits] added to every block's router logits of image b
        self.trace = False              # True: keep each block's input tokens and grain indices of the last
                                        # forward; "grains": the grain indices only
        self.last_tokens = None         # [depth, B, N, C] when trace
        self.last_grains = None         # int32 [depth, B, regions] when trace
        self._init_weights()

    def _init_weights(self):
        nn.init.trunc_normal_(self.pos_embed, std=.02)
        nn.init.trunc_normal_(self.cls_token, std=.02)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.trunc_normal_(m.weight, std=.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
            elif isinstance(m, nn.LayerNorm):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)
        for m in self.modules():
            if isinstance(m, DynamicGrainedEncoder):
                m.router.init_parameters()

    @torch.jit.ignore
    def no_weight_decay(self):
        return {"pos_embed", "cls_token"}

    def get_classifier(self):
        return self.head

    def compute_dtype(self):
        return self.head.weight.dtype

    def _pack_model(self, dtype):
        key = _param_key(self, dtype)
        pk = self._pack
        if pk.key != key:
            mat = lambda t: t.detach().to(dtype).contiguous()     # noqa: E731
            vec = lambda t: t.detach().float().contiguous()       # noqa: E731
            C = self.embed_dim
            t = dict(
                patch_w=mat(self.patch_embed.proj.weight.reshape(C, -1)), patch_b=vec(self.patch_embed.proj.bias),
                cls_token=mat(self.cls_token.reshape(C)), pos_embed=mat(self.pos_embed.reshape(-1, C)),
                norm_w=vec(self.norm.weight), norm_b=vec(self.norm.bias),
                head_w=mat(self.head.weight), head_b=vec(self.head.bias),
            )
            m = _lib.ModelWeights()
            for k, v in t.items():
                setattr(m, k, v.data_ptr())
            m.depth, m.patch, m.img_size, m.num_classes = self.depth, self.patch_size, self.img_size, self.num_classes
            blocks = (_lib.BlockWeights * self.depth)()
            for i, blk in enumerate(self.blocks):
                blk.flags = self.flags
                blk.fold_layernorm = self.fold_layernorm
                blocks[i] = _pack_block(blk, dtype)
            pk.key, pk.tensors, pk.struct = key, t, (m, blocks)
            self._graphs.clear()        # captured graphs hold the addresses of the previous pack
        return pk.struct

    def forward_graph(self, x, logits_out):
        """forward() through a CUDA graph captured for these input / output buffers (contents
        may change between calls, addresses and shapes may not)."""
        return _graph_forward(self, x, logits_out)

    def forward(self, x, logits_out=None):
        """images [B,3,S,S] on the device (fp32, or bf16 to halve the host-to-device copy of
        a bf16 model: the kernel rounds fp32 pixels to bf16 anyway) -> logits fp32
        [B,num_classes] (``deit_dge.py:267-299``) in one C-ABI call.  In training mode: the
        differentiable op-by-op sequence in the parameters' dtype."""
        if self.training:
            return self._forward_train(x)
        require_cuda(x)
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.float()
        x = x.contiguous()
        B = x.shape[0]
        dtype = self.compute_dtype()
        G = self.img_size // self.patch_size
        blk0 = self.blocks[0]
        s = _shape_struct(dtype, B, G, G, 1, self.embed_dim, blk0.attn.num_heads, blk0.mlp.fc1.out_features,
                          self.split_sizes, self.norm.eps, self.flags, blk0.attn.scale)
        m, blocks = self._pack_model(dtype)
        m.image_dtype = dtype_code(x.dtype)
        lib = _lib.lib()
        nbytes = lib.vtp_model_workspace_bytes(ctypes.byref(s), ctypes.byref(m))
        ws = scratch(x.device, nbytes)
        logits = logits_out if logits_out is not None else torch.empty(
            B, self.num_classes, dtype=torch.float32, device=x.device)
        counts = torch.empty(self.depth, B, dtype=torch.int32, device=x.device)
        opt = _lib.ForwardOptions()
        if self.gate_image_bias is not None:
            bias = self.gate_image_bias
            if (not bias.is_cuda or bias.dtype != torch.float32 or not bias.is_contiguous()
                    or tuple(bias.shape) != (B, len(self.split_sizes))):
                raise ValueError("gate_image_bias must be a contiguous fp32 CUDA tensor [B, n_splits]")
            opt.gate_image_bias = bias.data_ptr()
        if self.trace:
            if self.trace != "grains":
                self.last_tokens = torch.empty(self.depth, B, G * G + 1, self.embed_dim, dtype=dtype,
                                               device=x.device)
            self.last_grains = torch.empty(self.depth, B, (G // max(self.split_sizes)) ** 2, dtype=torch.int32,
                                           device=x.device)
            opt.grain_trace = self.last_grains.data_ptr()
            if self.trace != "grains":
                opt.tokens_trace = self.last_tokens.data_ptr()
        _lib.check(lib.vtp_deit_dge_forward_ex(ctypes.byref(s), ctypes.byref(m), blocks, ptr(x), ptr(logits),
                                               ptr(counts), ctypes.byref(opt), ptr(ws), nbytes,
                                               stream_ptr(x.device)))
        self.last_counts = counts
        # what get_complexity() of each block's encoder needs (dge.py:40-59): shapes only, and the
        # per-image query counts, which stay on the device
        tokens = torch.empty(0, device=x.device).expand(B, G * G + 1, 0)
        for i, blk in enumerate(self.blocks):
            blk.dge.states.update({"batches_device": counts[i], "input": tokens, "gate": None, "size": (G, G),
                                   "num_extra_tokens": 1})
        return logits

    def _forward_train(self, x):
        """``deit_dge.py:267-299`` with ``self.training`` (cls token, no distillation token)."""
        x = self.patch_embed(x.to(self.compute_dtype()))
        x = torch.cat((self.cls_token.expand(x.shape[0], -1, -1), x), dim=1)
        x = self.pos_drop(x + self.pos_embed)
        x = self.blocks(x)
        x = self.norm(x)
        return self.head(self.pre_logits(x[:, 0]))

    def complexity(self, x):
        """Static and dynamic MACs per image of the last forward, averaged over the batch
        (``deit_dge.py:233-249``, same formulae term by term); 0-d tensors on the device."""
        N = x.shape[1] * x.shape[2]
        comp = N * self.num_features * 3  # patch embed
        comp += self.num_features * self.num_classes  # classifier
        comp_static, comp_dynamic = [], []
        for blk in self.blocks:
            c = blk.dge.get_complexity()
            comp_static.append(c["static"])
            comp_dynamic.append(c["dynamic"])
        comp_static = (sum(comp_static) + comp).mean()
        comp_dynamic = (sum(comp_dynamic) + comp).mean()
        return {"static": comp_static, "dynamic": comp_dynamic}


class _CapturedForward:
    """A captured forward and everything whose address it holds."""

    def __init__(self, graph, keep, scratch_gen):
        self.graph, self.keep, self.scratch_gen = graph, keep, scratch_gen


def _graph_forward(model, x, logits_out):
    """Replay (capturing on first use) a CUDA graph of model.forward(x, logits_out) for these
    exact buffers: removes per-launch host work and shortens the gaps between kernels.

    A captured graph holds raw addresses: the input and output buffers, the packed (and folded)
    weights, the per-device scratch and the optional gate bias.  It is dropped, and captured
    again, when a parameter has changed since (load_state_dict, an optimizer step), when the
    scratch buffer has been replaced by a larger one, or when another gate bias tensor is set."""
    model._pack_model(model.compute_dtype())       # repacks after a parameter change and drops stale graphs
    bias = model.gate_image_bias
    key = (x.data_ptr(), tuple(x.shape), x.dtype, logits_out.data_ptr(), None if bias is None else bias.data_ptr(),
           model.trace, int(model.flags))
    g = model._graphs.get(key)
    if g is not None and g.scratch_gen != scratch_generation(x.device):
        g = None
    if g is None:
        cur = torch.cuda.current_stream(x.device)
        side = torch.cuda.Stream(x.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):          # warm-up outside capture: scratch, attributes, weight packs
            for _ in range(2):
                model.forward(x, logits_out)
        cur.wait_stream(side)
        torch.cuda.synchronize(x.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            model.forward(x, logits_out)
        keep = (x, logits_out, bias, model._pack.tensors, [blk._pack.tensors for blk in model.blocks],
                scratch(x.device, 1), model.last_counts, model.last_tokens, model.last_grains)
        g = _CapturedForward(graph, keep, scratch_generation(x.device))
        model._graphs[key] = g
    g.graph.replay()
    model.last_counts = g.keep[6]
    if model.trace:
        model.last_tokens, model.last_grains = g.keep[7], g.keep[8]
    return logits_out


def _make(embed_dim, num_heads, **kwargs):
    return VisionTransformer(img_size=256, patch_size=16, embed_dim=embed_dim, depth=12, num_heads=num_heads,
                             mlp_ratio=4, qkv_bias=True, norm_layer=partial(nn.LayerNorm, eps=1e-6),
                             split_sizes=[4, 2, 1], **kwargs)


def deit_dge_s124_tiny_patch16_256(pretrained=False, **kwargs):
    return _make(192, 3, **kwargs)


def deit_dge_s124_small_patch16_256(pretrained=False, **kwargs):
    return _make(384, 6, **kwargs)


def deit_dge_s124_base_patch16_256(pretrained=False, **kwargs):
    return _make(768, 12, **kwargs)
