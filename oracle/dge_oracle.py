"""CPU oracle for the Dynamic Grained Encoder (DGE) eval forward.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file;
only tests, the smoke check and the timed CPU baseline of the bench do.

A plain PyTorch (CPU, fp32 unless the caller passes another dtype) restatement
of the reference's eval path.  The reference's native half is CUDA-only and
has no tests of its own, so parity is pinned by:

  * running the reference's own, unmodified Python modules over these
    functions installed as ``vtpack._C`` (see ``oracle/ref_shim.py``) and
    committing the results as golden fixtures (``tests/golden``);
  * cross-checking the sparse ops against the reference's independent dense
    PyTorch implementations (``vtpack/layers/grained_sample.py:126-177``) and
    against the dense DeiT block (``vtpack/models/standard/deit.py:50-83``).

Each function cites the reference lines it follows.
"""
import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------
# vtpack._C restatements
# --------------------------------------------------------------------------

def grained_sample_index_to_patch(indices: torch.Tensor, split_sizes: torch.Tensor,
                                  region_size: int, num_extra_tokens: int
                                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Patch list from per-region grain indices.

    Follows ``vtpack/layers/csrc/grained_sample/grained_sample.cu:302-345``
    (host: sizes = split_sizes[indices]; lengths = [extra, size^2 ...];
    inclusive cumsum) and the kernel at ``:146-196``: every region writes
    ``size*size`` rows ``[b, y, x, step]``, ``step = region_size / size``,
    sub-patches row-major (dy outer, dx inner); each image's extra tokens
    come first as ``[b, -idx-1, <unwritten>, 1]``.  Column 2 of the
    extra-token rows is never written by the reference; 0 is stored here and
    comparisons must skip it.

    Returns ``patches`` int64 ``[L,4]`` and ``batch_lengths`` int64 ``[B]``.
    """
    indices = indices.to(torch.int64)
    split_sizes = split_sizes.to(torch.int64)
    B, Hr, Wr = indices.shape
    R = Hr * Wr
    sizes = split_sizes[indices].reshape(B, R)                # [B,R]
    n_rows = sizes * sizes                                    # rows per region
    batch_lengths = n_rows.sum(1) + num_extra_tokens          # [B]
    L = int(batch_lengths.sum())

    flat_sizes = sizes.reshape(-1)
    flat_rows = n_rows.reshape(-1)
    total_region_rows = int(flat_rows.sum())
    region_id = torch.repeat_interleave(torch.arange(B * R), flat_rows)
    region_start = torch.cumsum(flat_rows, 0) - flat_rows     # exclusive
    local = torch.arange(total_region_rows) - region_start[region_id]
    s = flat_sizes[region_id]
    step = region_size // s
    b = region_id // R
    ry = (region_id % R) // Wr
    rx = (region_id % R) % Wr
    dy = local // s
    dx = local % s
    rows = torch.stack([b, ry * region_size + dy * step, rx * region_size + dx * step, step], 1)

    patches = torch.zeros(L, 4, dtype=torch.int64)
    # destination of each region row: shifted by the extra tokens of images 0..b
    dst = torch.arange(total_region_rows) + (b + 1) * num_extra_tokens
    patches[dst] = rows
    if num_extra_tokens > 0:
        img_start = torch.cumsum(batch_lengths, 0) - batch_lengths
        for idx in range(num_extra_tokens):
            pos = img_start + idx
            patches[pos, 0] = torch.arange(B)
            patches[pos, 1] = -idx - 1
            patches[pos, 3] = 1
    return patches, batch_lengths


def _token_index(patches: torch.Tensor, width: int, num_extra_tokens: int):
    """Per patch row: (is_extra, batch, first-token index, size)."""
    b = patches[:, 0]
    y = patches[:, 1]
    x = patches[:, 2]
    size = patches[:, 3]
    is_extra = y < 0
    tok0 = torch.where(is_extra, -y - 1, y * width + x + num_extra_tokens)
    return is_extra, b, tok0, size


def grained_sample_compress(inp: torch.Tensor, patches: torch.Tensor, height: int,
                            width: int, num_extra_tokens: int) -> torch.Tensor:
    """Multi-grain average pooling ``[B,N,C] -> [L,C]``.

    Follows ``grained_sample.cu:31-69``: extra tokens are copied; otherwise
    the ``size*size`` tokens are summed (dy outer, dx inner, in the
    accumulate type) and the sum is divided by ``size*size``.
    """
    B, N, C = inp.shape
    L = patches.shape[0]
    is_extra, b, tok0, size = _token_index(patches, width, num_extra_tokens)
    acc_dtype = torch.float32 if inp.dtype in (torch.float16, torch.bfloat16) else inp.dtype
    out = torch.empty(L, C, dtype=inp.dtype)
    flat = inp.reshape(B * N, C)
    base = b * N + tok0
    sel = is_extra.nonzero().squeeze(1)
    out[sel] = flat[base[sel]]
    for s in torch.unique(size[~is_extra]).tolist():
        sel = ((size == s) & ~is_extra).nonzero().squeeze(1)
        acc = torch.zeros(sel.numel(), C, dtype=acc_dtype)
        for dy in range(s):
            for dx in range(s):
                acc = acc + flat[base[sel] + dy * width + dx].to(acc_dtype)
        out[sel] = (acc / (s * s)).to(inp.dtype)
    return out


def grained_sample_decompress(inp: torch.Tensor, patches: torch.Tensor, ref: torch.Tensor,
                              height: int, width: int, num_extra_tokens: int,
                              is_add_ref: bool) -> torch.Tensor:
    """Replicate-unpool ``[L,C] -> [B,N,C]`` with optional residual.

    Follows ``grained_sample.cu:107-144`` (add-ref) and ``:71-105`` (no ref):
    every token covered by a patch receives ``inp[patch] (+ ref[b,tok])``.
    """
    B, N, C = ref.shape
    is_extra, b, tok0, size = _token_index(patches, width, num_extra_tokens)
    out = torch.empty(B * N, C, dtype=inp.dtype)
    flat_ref = ref.reshape(B * N, C)
    base = b * N + tok0
    sel = is_extra.nonzero().squeeze(1)
    out[base[sel]] = inp[sel] + flat_ref[base[sel]] if is_add_ref else inp[sel]
    for s in torch.unique(size[~is_extra]).tolist():
        sel = ((size == s) & ~is_extra).nonzero().squeeze(1)
        for dy in range(s):
            for dx in range(s):
                t = base[sel] + dy * width + dx
                out[t] = inp[sel] + flat_ref[t] if is_add_ref else inp[sel]
    return out.reshape(B, N, C)


def batched_sparse_attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                     batch_lengths: torch.Tensor, scale: float) -> torch.Tensor:
    """Variable-length-query attention, ``q[h,L,d]``, ``k,v[h,B,N,d] -> [h,L,d]``.

    Follows ``vtpack/layers/csrc/batched_sparse_gemm/batched_sparse_gemm.cu:267-301``:
    per image ``S = scale * Q_i K_i^T`` (scale is the GEMM alpha), a
    max-subtracted softmax over all N keys, then ``O = S V_i``.
    """
    h, L, d = q.shape
    out = torch.empty(h, L, d, dtype=q.dtype)
    start = 0
    for i, m in enumerate(batch_lengths.tolist()):
        qi = q[:, start:start + m]                            # [h,m,d]
        attn = torch.matmul(qi, k[:, i].transpose(-1, -2)) * scale
        attn = torch.softmax(attn, dim=-1)
        out[:, start:start + m] = torch.matmul(attn, v[:, i])
        start += m
    return out


def batched_sparse_gemm_forward(a: torch.Tensor, b: torch.Tensor, a_lengths: torch.Tensor,
                                b_lengths: torch.Tensor, is_a_transposed: bool,
                                is_b_transposed: bool) -> torch.Tensor:
    """Ragged batched product of the training path, ``a[h,La,ka]``, ``b[h,Lb,kb]``.

    Follows ``vtpack/layers/csrc/batched_sparse_gemm/batched_sparse_gemm.cu:150-196``: image i owns
    the next ``a_lengths[i]`` rows of ``a`` and ``b_lengths[i]`` rows of ``b``; each slice is
    transposed when its flag is set, the per-image ``bmm`` results are concatenated along dim 1.
    """
    outs = []
    sa = sb = 0
    for la, lb in zip(a_lengths.tolist(), b_lengths.tolist()):
        ai, bi = a[:, sa:sa + la], b[:, sb:sb + lb]
        if is_a_transposed:
            ai = ai.transpose(-1, -2)
        if is_b_transposed:
            bi = bi.transpose(-1, -2)
        outs.append(torch.matmul(ai, bi))
        sa += la
        sb += lb
    return torch.cat(outs, dim=1)


def gumbel_softmax_fixed(noises):
    """Stand-in for ``torch.nn.functional.gumbel_softmax`` that draws its Gumbel noise from the given
    list (one tensor per call, in call order) instead of the random generator, so that a CPU run and
    a CUDA run of a training-mode forward sample the same gates.  Hard straight-through form: the
    forward value is the one-hot arg-max of softmax((logits + noise) / tau), the gradient that of the
    softmax."""
    it = iter(noises)

    def gumbel_softmax(logits, tau=1, hard=False, eps=1e-10, dim=-1):
        g = next(it).to(device=logits.device, dtype=logits.dtype)
        y_soft = ((logits + g) / tau).softmax(dim)
        if not hard:
            return y_soft
        index = y_soft.max(dim, keepdim=True)[1]
        y_hard = torch.zeros_like(logits).scatter_(dim, index, 1.0)
        return y_hard - y_soft.detach() + y_soft

    return gumbel_softmax


def make_gumbel_noise(shape, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(*shape, generator=g).clamp_(1e-6, 1.0 - 1e-6)
    return -torch.log(-torch.log(u))


# --------------------------------------------------------------------------
# Module-level restatements (weights passed as plain dicts of tensors)
# --------------------------------------------------------------------------

def router_forward(x_grid: torch.Tensor, gate_w: torch.Tensor, gate_b: torch.Tensor,
                   region_size: int) -> torch.Tensor:
    """``DynamicRouter.forward`` (``vtpack/layers/dge.py:145-150``):
    average pool over each region, then ``Linear(C -> n_splits)``."""
    x = x_grid.permute(0, 3, 1, 2)
    x = F.avg_pool2d(x, region_size, region_size)
    x = x.permute(0, 2, 3, 1)
    return F.linear(x, gate_w, gate_b)


def dge_block_forward(x: torch.Tensor, w: Dict[str, torch.Tensor], num_heads: int,
                      split_sizes: Sequence[int], eps: float = 1e-6,
                      forced_gate: Optional[torch.Tensor] = None,
                      trace: Optional[dict] = None, grid: Optional[Tuple[int, int]] = None,
                      sr_ratio: int = 1, sr_eps: float = 1e-5,
                      gate_image_bias: Optional[torch.Tensor] = None,
                      qk_scale: Optional[float] = None,
                      forced_indices: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Eval forward of one DeiT+DGE block, or of one PVT+DGE block when ``grid`` / ``sr_ratio``
    are given.

    PVT+DGE (``vtpack/models/dge/pvt_dge.py:140-146`` and ``Attention.forward`` ``:77-111``):
    the same block on an explicit H x W grid (stages 1-3 carry no extra token), whose keys
    and values come from the normed tokens reduced by a stride-``sr_ratio`` convolution
    (``attn.sr``) and a LayerNorm (``attn.norm``, PyTorch's default eps 1e-5, ``:62-63``).

    Follows ``Block.forward`` (``vtpack/models/dge/deit_dge.py:123-130``),
    ``DynamicGrainedEncoder.compress/decompress`` (``vtpack/layers/dge.py:61-112``),
    ``Attention.forward`` (``deit_dge.py:70-98``) and ``Mlp.forward`` (``:38-44``).
    ``w`` uses the reference's state_dict keys relative to the block
    (``norm1.weight``, ``attn.q.weight``, ``dge.router.gate.weight`` ...).
    ``forced_gate`` replaces the router output (teacher forcing).  ``gate_image_bias``
    (``[B, n_splits]``) is added to the router output of every region of image b: the reference
    has no such input, measurement configurations that force whole images to one grain do
    (large offsets).  ``qk_scale`` overrides ``head_dim ** -0.5`` (``deit_dge.py:52-53``).
    ``forced_indices`` (int ``[B, Hr, Wr]``) replaces the argmax of the gate: the block then follows
    grain decisions made elsewhere (e.g. by the device on its bf16 activations).
    """
    B, N, C = x.shape
    if grid is None:
        H = W = int(math.sqrt(N))
    else:
        H, W = grid
    num_extra = N - H * W
    region = max(split_sizes)
    splits = torch.tensor(list(split_sizes), dtype=torch.int64)

    # compress -----------------------------------------------------------
    if forced_gate is None:
        gate = router_forward(x[:, num_extra:, :].reshape(B, H, W, C),
                              w["dge.router.gate.weight"], w["dge.router.gate.bias"], region)
    else:
        gate = forced_gate
    if gate_image_bias is not None:
        gate = gate + gate_image_bias[:, None, None, :]
    indices = gate.argmax(dim=-1) if forced_indices is None else forced_indices.to(torch.int64)
    patches, batches = grained_sample_index_to_patch(indices, splits, region, num_extra)
    comp = grained_sample_compress(x, patches, H, W, num_extra)

    # attention ------------------------------------------------------------
    d = C // num_heads
    scale = qk_scale or d ** -0.5
    xn = F.layer_norm(x, (C,), w["norm1.weight"], w["norm1.bias"], eps)
    qn = F.layer_norm(comp, (C,), w["norm1.weight"], w["norm1.bias"], eps)
    q = F.linear(qn, w["attn.q.weight"], w.get("attn.q.bias")).reshape(-1, num_heads, d).permute(1, 0, 2)
    if sr_ratio > 1:
        # pvt_dge.py:81-85: the reshape needs N == H*W (no extra token in a reduced stage)
        xr = xn.permute(0, 2, 1).reshape(B, C, H, W)
        xr = F.conv2d(xr, w["attn.sr.weight"], w["attn.sr.bias"], stride=sr_ratio)
        xr = xr.reshape(B, C, -1).permute(0, 2, 1)
        keys_in = F.layer_norm(xr, (C,), w["attn.norm.weight"], w["attn.norm.bias"], sr_eps)
    else:
        keys_in = xn
    kv = F.linear(keys_in, w["attn.kv.weight"], w.get("attn.kv.bias"))
    kv = kv.reshape(B, keys_in.shape[1], 2, num_heads, d).permute(2, 3, 0, 1, 4)
    o = batched_sparse_attention_forward(q.contiguous(), kv[0].contiguous(), kv[1].contiguous(),
                                         batches, scale)
    o = o.transpose(0, 1).reshape(-1, C)
    a = F.linear(o, w["attn.proj.weight"], w["attn.proj.bias"])
    q1 = comp + a

    # mlp --------------------------------------------------------------------
    hdn = F.gelu(F.linear(F.layer_norm(q1, (C,), w["norm2.weight"], w["norm2.bias"], eps),
                          w["mlp.fc1.weight"], w["mlp.fc1.bias"]))
    q2 = q1 + F.linear(hdn, w["mlp.fc2.weight"], w["mlp.fc2.bias"])

    # decompress -------------------------------------------------------------
    out = grained_sample_decompress(q2 - comp, patches, x, H, W, num_extra, True)
    if trace is not None:
        trace.update(gate=gate, indices=indices, patches=patches, batches=batches, comp=comp,
                     q1=q1, q2=q2, attn_out=o)
    return out


def dense_block_forward(x: torch.Tensor, w: Dict[str, torch.Tensor], num_heads: int,
                        eps: float = 1e-6) -> torch.Tensor:
    """Dense DeiT block (``vtpack/models/standard/deit.py:50-62,79-83``) built from
    the DGE block's weights (q and kv concatenated into one qkv)."""
    B, N, C = x.shape
    d = C // num_heads
    xn = F.layer_norm(x, (C,), w["norm1.weight"], w["norm1.bias"], eps)
    qkv_w = torch.cat([w["attn.q.weight"], w["attn.kv.weight"]], 0)
    qkv_b = None
    if w.get("attn.q.bias") is not None:
        qkv_b = torch.cat([w["attn.q.bias"], w["attn.kv.bias"]], 0)
    qkv = F.linear(xn, qkv_w, qkv_b).reshape(B, N, 3, num_heads, d).permute(2, 0, 3, 1, 4)
    attn = (qkv[0] @ qkv[1].transpose(-2, -1)) * (d ** -0.5)
    attn = attn.softmax(dim=-1)
    y = (attn @ qkv[2]).transpose(1, 2).reshape(B, N, C)
    x = x + F.linear(y, w["attn.proj.weight"], w["attn.proj.bias"])
    hdn = F.gelu(F.linear(F.layer_norm(x, (C,), w["norm2.weight"], w["norm2.bias"], eps),
                          w["mlp.fc1.weight"], w["mlp.fc1.bias"]))
    return x + F.linear(hdn, w["mlp.fc2.weight"], w["mlp.fc2.bias"])


def block_weights(sd: Dict[str, torch.Tensor], i: int) -> Dict[str, torch.Tensor]:
    """Slice ``blocks.{i}.*`` out of a model state_dict."""
    p = f"blocks.{i}."
    return {k[len(p):]: v for k, v in sd.items() if k.startswith(p)}


def deit_dge_forward(images: torch.Tensor, sd: Dict[str, torch.Tensor], depth: int,
                     num_heads: int, split_sizes: Sequence[int], patch: int = 16,
                     eps: float = 1e-6, trace: Optional[List[dict]] = None,
                     gate_image_bias: Optional[torch.Tensor] = None,
                     features: Optional[list] = None,
                     forced_indices: Optional[Sequence[torch.Tensor]] = None) -> torch.Tensor:
    """Eval forward of DeiT+DGE, images ``[B,3,S,S] -> logits [B,classes]``.

    Follows ``VisionTransformer.forward_features/forward``
    (``vtpack/models/dge/deit_dge.py:267-299``): patch-embed conv (kernel =
    stride = patch) flattened to tokens, cls token prepended, position
    embedding added, ``depth`` DGE blocks, final LayerNorm, cls row, head.
    """
    x = F.conv2d(images, sd["patch_embed.proj.weight"], sd["patch_embed.proj.bias"], stride=patch)
    x = x.flatten(2).transpose(1, 2)
    cls = sd["cls_token"].expand(x.shape[0], -1, -1)
    x = torch.cat((cls, x), dim=1) + sd["pos_embed"]
    for i in range(depth):
        t = {} if trace is not None else None
        if t is not None:
            t["x_in"] = x
        x = dge_block_forward(x, block_weights(sd, i), num_heads, split_sizes, eps, trace=t,
                              gate_image_bias=gate_image_bias,
                              forced_indices=None if forced_indices is None else forced_indices[i])
        if trace is not None:
            trace.append(t)
    x = F.layer_norm(x, (x.shape[-1],), sd["norm.weight"], sd["norm.bias"], eps)
    if features is not None:
        features.append(x[:, 0])          # the normed cls rows the head reads
    return F.linear(x[:, 0], sd["head.weight"], sd["head.bias"])


PVT_CONFIGS = {
    # pvt_dge.py:375-392: the 256 px factories (tiny: depths 2,2,2,2; small: 3,4,6,3)
    "tiny": dict(embed_dims=(64, 128, 320, 512), num_heads=(1, 2, 5, 8), mlp_ratios=(8, 8, 4, 4),
                 depths=(2, 2, 2, 2), sr_ratios=(8, 4, 2, 1), patch_size=4),
    "small": dict(embed_dims=(64, 128, 320, 512), num_heads=(1, 2, 5, 8), mlp_ratios=(8, 8, 4, 4),
                  depths=(3, 4, 6, 3), sr_ratios=(8, 4, 2, 1), patch_size=4),
}


def pvt_dge_forward(images: torch.Tensor, sd: Dict[str, torch.Tensor], cfg: dict,
                    split_sizes: Sequence[int] = (4, 2, 1), eps: float = 1e-6,
                    trace: Optional[List[dict]] = None) -> torch.Tensor:
    """Eval forward of PVT+DGE, images ``[B,3,S,S] -> logits [B,classes]``.

    Follows ``PyramidVisionTransformer.forward_features/forward``
    (``vtpack/models/dge/pvt_dge.py:295-337``) at the training resolution (no position-embedding
    interpolation, ``:287-288``): per stage a patch-embedding convolution (kernel = stride = 4,
    then 2) followed by a LayerNorm with PyTorch's default eps 1e-5 (``PatchEmbed``, ``:149-179``),
    the position embedding, the stage's DGE blocks, and the token grid handed to the next stage
    as ``[B,C,H,W]``; the last stage gets the cls token in front; final LayerNorm, cls row, head.
    """
    B = images.shape[0]
    x = images
    n_stages = len(cfg["embed_dims"])
    for i in range(n_stages):
        p = cfg["patch_size"] if i == 0 else 2
        pre = f"patch_embed{i + 1}."
        x = F.conv2d(x, sd[pre + "proj.weight"], sd[pre + "proj.bias"], stride=p)
        H, W = x.shape[2], x.shape[3]
        x = x.flatten(2).transpose(1, 2)
        x = F.layer_norm(x, (x.shape[-1],), sd[pre + "norm.weight"], sd[pre + "norm.bias"], 1e-5)
        if i == n_stages - 1:
            x = torch.cat((sd["cls_token"].expand(B, -1, -1), x), dim=1)
        x = x + sd[f"pos_embed{i + 1}"]
        for j in range(cfg["depths"][i]):
            t = {} if trace is not None else None
            pfx = f"block{i + 1}.{j}."
            w = {k[len(pfx):]: v for k, v in sd.items() if k.startswith(pfx)}
            x = dge_block_forward(x, w, cfg["num_heads"][i], split_sizes, eps, trace=t, grid=(H, W),
                                  sr_ratio=cfg["sr_ratios"][i])
            if trace is not None:
                trace.append(t)
        if i != n_stages - 1:
            x = x.reshape(B, H, W, -1).permute(0, 3, 1, 2).contiguous()
    x = F.layer_norm(x, (x.shape[-1],), sd["norm.weight"], sd["norm.bias"], eps)
    return F.linear(x[:, 0], sd["head.weight"], sd["head.bias"])


def make_pvt_state_dict(cfg: dict, img_size: int = 256, num_classes: int = 1000,
                        split_sizes: Sequence[int] = (4, 2, 1), seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Random-init weights of PVT+DGE under the reference's state_dict keys (``pvt_dge.py:196-224``):
    matrices, convolutions, position embeddings and the cls token trunc-normal(std) in a fixed order
    from CPU generators, LayerNorm weights 1, every bias (the gates' included) 0."""
    g = torch.Generator().manual_seed(seed)

    def tn(*shape):
        t = torch.empty(*shape)
        torch.nn.init.trunc_normal_(t, std=std, a=-2 * std, b=2 * std, generator=g)
        return t

    sd = {}
    dims = cfg["embed_dims"]
    n_stages = len(dims)
    for i in range(n_stages):
        C = dims[i]
        p = cfg["patch_size"] if i == 0 else 2
        grid = img_size // (cfg["patch_size"] * 2 ** i)
        pre = f"patch_embed{i + 1}."
        sd[pre + "proj.weight"] = tn(C, 3 if i == 0 else dims[i - 1], p, p)
        sd[pre + "proj.bias"] = torch.zeros(C)
        sd[pre + "norm.weight"] = torch.ones(C)
        sd[pre + "norm.bias"] = torch.zeros(C)
        sd[f"pos_embed{i + 1}"] = tn(1, grid * grid + (1 if i == n_stages - 1 else 0), C)
        for j in range(cfg["depths"][i]):
            w = make_pvt_block_weights(C, cfg["mlp_ratios"][i], cfg["sr_ratios"][i], split_sizes,
                                       seed=seed * 1000 + 17 * i + j + 1, std=std)
            for k, v in w.items():
                sd[f"block{i + 1}.{j}.{k}"] = v
    sd["norm.weight"] = torch.ones(dims[-1])
    sd["norm.bias"] = torch.zeros(dims[-1])
    sd["cls_token"] = tn(1, 1, dims[-1])
    sd["head.weight"] = tn(num_classes, dims[-1])
    sd["head.bias"] = torch.zeros(num_classes)
    return sd


# --------------------------------------------------------------------------
# Seeded synthetic weights / inputs shared by tests, golden fixtures and bench
# --------------------------------------------------------------------------

MODEL_CONFIGS = {
    "tiny": dict(embed_dim=192, depth=12, num_heads=3),
    "small": dict(embed_dim=384, depth=12, num_heads=6),
    "base": dict(embed_dim=768, depth=12, num_heads=12),
}


def make_state_dict(embed_dim: int, depth: int, num_heads: int, img_size: int = 256,
                    patch: int = 16, num_classes: int = 1000, mlp_ratio: int = 4,
                    split_sizes: Sequence[int] = (4, 2, 1), seed: int = 0,
                    std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Random-init weights with the reference's state_dict keys
    (``deit_dge.py:155-216``): every weight matrix, the cls token and the
    position embedding are trunc-normal(std) drawn in a fixed order from one
    CPU generator; LayerNorm weights 1; every bias (the gate's included) 0."""
    g = torch.Generator().manual_seed(seed)

    def tn(*shape):
        t = torch.empty(*shape)
        torch.nn.init.trunc_normal_(t, std=std, a=-2 * std, b=2 * std, generator=g)
        return t

    C = embed_dim
    n_tok = (img_size // patch) ** 2 + 1
    sd = {
        "cls_token": tn(1, 1, C),
        "pos_embed": tn(1, n_tok, C),
        "patch_embed.proj.weight": tn(C, 3, patch, patch),
        "patch_embed.proj.bias": torch.zeros(C),
    }
    for i in range(depth):
        p = f"blocks.{i}."
        sd[p + "norm1.weight"] = torch.ones(C)
        sd[p + "norm1.bias"] = torch.zeros(C)
        sd[p + "attn.q.weight"] = tn(C, C)
        sd[p + "attn.q.bias"] = torch.zeros(C)
        sd[p + "attn.kv.weight"] = tn(2 * C, C)
        sd[p + "attn.kv.bias"] = torch.zeros(2 * C)
        sd[p + "attn.proj.weight"] = tn(C, C)
        sd[p + "attn.proj.bias"] = torch.zeros(C)
        sd[p + "norm2.weight"] = torch.ones(C)
        sd[p + "norm2.bias"] = torch.zeros(C)
        sd[p + "mlp.fc1.weight"] = tn(mlp_ratio * C, C)
        sd[p + "mlp.fc1.bias"] = torch.zeros(mlp_ratio * C)
        sd[p + "mlp.fc2.weight"] = tn(C, mlp_ratio * C)
        sd[p + "mlp.fc2.bias"] = torch.zeros(C)
        sd[p + "dge.splits"] = torch.tensor(list(split_sizes))
        sd[p + "dge.router.gate.weight"] = tn(len(split_sizes), C)
        sd[p + "dge.router.gate.bias"] = torch.zeros(len(split_sizes))
    sd["norm.weight"] = torch.ones(C)
    sd["norm.bias"] = torch.zeros(C)
    sd["head.weight"] = tn(num_classes, C)
    sd["head.bias"] = torch.zeros(num_classes)
    return sd


def make_pvt_block_weights(dim: int, mlp_ratio: int, sr_ratio: int, split_sizes: Sequence[int] = (4, 2, 1),
                           seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Random-init weights of one PVT+DGE block under the reference's state_dict keys
    (``pvt_dge.py:46-63,116-132``): matrices and the reduction convolution trunc-normal(std) in a
    fixed order from one CPU generator, LayerNorm weights 1, every bias 0."""
    g = torch.Generator().manual_seed(seed)

    def tn(*shape):
        t = torch.empty(*shape)
        torch.nn.init.trunc_normal_(t, std=std, a=-2 * std, b=2 * std, generator=g)
        return t

    C = dim
    w = {
        "norm1.weight": torch.ones(C), "norm1.bias": torch.zeros(C),
        "attn.q.weight": tn(C, C), "attn.q.bias": torch.zeros(C),
        "attn.kv.weight": tn(2 * C, C), "attn.kv.bias": torch.zeros(2 * C),
        "attn.proj.weight": tn(C, C), "attn.proj.bias": torch.zeros(C),
    }
    if sr_ratio > 1:
        w["attn.sr.weight"] = tn(C, C, sr_ratio, sr_ratio)
        w["attn.sr.bias"] = torch.zeros(C)
        w["attn.norm.weight"] = torch.ones(C)
        w["attn.norm.bias"] = torch.zeros(C)
    w.update({
        "norm2.weight": torch.ones(C), "norm2.bias": torch.zeros(C),
        "mlp.fc1.weight": tn(mlp_ratio * C, C), "mlp.fc1.bias": torch.zeros(mlp_ratio * C),
        "mlp.fc2.weight": tn(C, mlp_ratio * C), "mlp.fc2.bias": torch.zeros(C),
        "dge.splits": torch.tensor(list(split_sizes)),
        "dge.router.gate.weight": tn(len(split_sizes), C), "dge.router.gate.bias": torch.zeros(len(split_sizes)),
    })
    return w


def make_images(batch: int, img_size: int = 256, seed: int = 1) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(batch, 3, img_size, img_size, generator=g)


def make_tokens(batch: int, n_tokens: int, dim: int, seed: int = 1) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(batch, n_tokens, dim, generator=g)


def make_gate_logits(batch: int, hr: int, wr: int, n_splits: int = 3, seed: int = 2,
                     fine_bias: float = 0.0) -> torch.Tensor:
    """N(0,1) gate logits; ``fine_bias`` is added to grain index 0 (the finest
    split) to skew the fraction of fine regions."""
    g = torch.Generator().manual_seed(seed)
    t = torch.randn(batch, hr, wr, n_splits, generator=g)
    t[..., 0] += fine_bias
    return t


def round_bf16(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """fp32 copy of ``sd`` whose floating values are bf16-representable: the
    bf16 device path is compared with fp32 math on these."""
    return {k: (v.to(torch.bfloat16).to(torch.float32) if v.is_floating_point() else v)
            for k, v in sd.items()}


# --------------------------------------------------------------------------
# Seeded inputs of the training-path fixtures (shared by the fixture generator and the tests)
# --------------------------------------------------------------------------

def randn_seeded(shape, seed: int) -> torch.Tensor:
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def train_ops_inputs(C: int):
    """Tokens [2,257,C] (seed 1) and grain indices [2,4,4] (arg-max of the seed-2 gate logits)."""
    x = randn_seeded((2, 257, C), 1)
    gate = make_gate_logits(2, 4, 4, 3, seed=2)
    return x, gate.argmax(dim=-1)


TRAIN_BLOCK = dict(dim=64, heads=2, batch=2, noise_seed=21, grad_seed=22, weight_seed=5, token_seed=6)


def train_block_weights() -> Dict[str, torch.Tensor]:
    """Weights of the training-mode block fixture: trunc-normal matrices plus small random biases and
    LayerNorm offsets, so that every gradient path carries signal."""
    cfg = TRAIN_BLOCK
    sd = block_weights(make_state_dict(cfg["dim"], 1, cfg["heads"], seed=cfg["weight_seed"]), 0)
    g = torch.Generator().manual_seed(cfg["weight_seed"] + 100)
    for k, v in sd.items():
        if k.endswith("bias") and v.is_floating_point():
            sd[k] = v + 0.02 * torch.randn(v.shape, generator=g)
    return sd


TRAIN_PVT_BLOCK = dict(dim=32, heads=1, grid=16, sr=2, mlp_ratio=8, batch=2, noise_seed=23, grad_seed=24,
                       weight_seed=7, token_seed=8)


TRAIN_PVT_MODEL = dict(batch=2, weight_seed=0, image_seed=9, noise_seed=50, target=(3, 7),
                       grads=("patch_embed1.proj.weight", "block1.0.dge.router.gate.weight",
                              "block2.1.attn.sr.bias", "block2.1.attn.norm.weight", "block4.1.mlp.fc2.bias", "cls_token"))


def train_pvt_model_noises(cfg: dict, img_size: int = 256):
    """One Gumbel-noise tensor per block of a PVT+DGE model, in forward order (region grid of stage
    i: img_size / (4 * 2^i) / 4 per side)."""
    t = TRAIN_PVT_MODEL
    noises, k = [], 0
    for i, depth in enumerate(cfg["depths"]):
        r = img_size // (4 * 2 ** i) // 4
        for _ in range(depth):
            noises.append(make_gumbel_noise((t["batch"], r, r, 3), t["noise_seed"] + k))
            k += 1
    return noises


DPVT_ATTENTION = dict(dim=64, heads=4, points=3, H=8, W=6, batch=2, weight_seed=60, token_seed=61, grad_seed=62)


def dpvt_attention_weights() -> Dict[str, torch.Tensor]:
    """Seeded parameters of the deformable-attention fixture under the reference's state_dict keys
    (``dpvt.py:61-71``): random matrices, and offset weights large enough that points leave the map."""
    c = DPVT_ATTENTION
    C, h, P = c["dim"], c["heads"], c["points"]
    g = torch.Generator().manual_seed(c["weight_seed"])
    rn = lambda *shape, std: torch.randn(*shape, generator=g) * std      # noqa: E731
    return {
        "v.weight": rn(C, C, std=0.1), "v.bias": rn(C, std=0.1),
        "attn_weight.weight": rn(h * P, C, std=0.2), "attn_weight.bias": rn(h * P, std=0.2),
        "proj.weight": rn(C, C, std=0.1), "proj.bias": rn(C, std=0.1),
        "offsets.weight": rn(h * P * 2, C, std=0.3), "offsets.bias": rn(h * P * 2, std=2.0),
    }
