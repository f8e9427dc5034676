"""CPU tests that pin the oracle: golden fixtures produced by the reference's
own Python modules, and (when the reference checkout is present) cross-checks
against the reference's independent dense implementations."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import dge_oracle as O
from oracle import ref_shim

needs_ref = pytest.mark.skipif(not ref_shim.reference_available(),
                               reason="reference checkout not present")


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_layer_golden(golden_dir):
    g = _load(golden_dir, "layer_tiny_fp32.npz")
    sd = O.make_state_dict(192, 1, 3, seed=0)
    x = O.make_tokens(2, 257, 192, seed=1)
    gate = O.make_gate_logits(2, 4, 4, 3, seed=2)
    assert math.isclose(x.double().sum().item(), float(g["input_sum"]), rel_tol=0, abs_tol=1e-9)
    assert math.isclose(sum(v.double().sum().item() for v in sd.values()), float(g["weight_sum"]),
                        rel_tol=0, abs_tol=1e-9)
    assert math.isclose(gate.double().sum().item(), float(g["gate_sum"]), rel_tol=0, abs_tol=1e-9)
    tr = {}
    out = O.dge_block_forward(x, O.block_weights(sd, 0), 3, (4, 2, 1), forced_gate=gate, trace=tr)
    pg = torch.from_numpy(g["patches"].astype(np.int64))
    keep = pg[:, 1] >= 0
    assert torch.equal(tr["patches"][:, [0, 1, 3]], pg[:, [0, 1, 3]])
    assert torch.equal(tr["patches"][keep, 2], pg[keep, 2])
    assert tr["batches"].tolist() == g["batch_lengths"].tolist()
    assert torch.equal(tr["comp"][::7], torch.from_numpy(g["comp_rows"]))
    assert torch.equal(out, torch.from_numpy(g["out"]))


def test_model_golden(golden_dir):
    g = _load(golden_dir, "model_tiny_fp32.npz")
    sd = O.make_state_dict(192, 12, 3, seed=0)
    x = O.make_images(2, 256, seed=1)
    assert math.isclose(x.double().sum().item(), float(g["input_sum"]), rel_tol=0, abs_tol=1e-9)
    tr = []
    logits = O.deit_dge_forward(x, sd, 12, 3, (4, 2, 1), trace=tr)
    assert np.array_equal(np.stack([t["indices"].numpy() for t in tr]), g["grain_indices"])
    assert np.array_equal(np.stack([t["batches"].numpy() for t in tr]), g["batch_lengths"])
    assert torch.equal(logits, torch.from_numpy(g["logits"]))


def test_patch_order_and_counts():
    """Rows are ordered by (image, extra first, region row-major, dy, dx) and the
    per-image count is extra + sum(split^2)  (grained_sample.cu:146-196,302-345)."""
    g = torch.Generator().manual_seed(5)
    idx = torch.randint(0, 3, (3, 4, 4), generator=g)
    splits = torch.tensor([4, 2, 1])
    patches, lens = O.grained_sample_index_to_patch(idx, splits, 4, 1)
    assert lens.tolist() == (1 + (splits[idx] ** 2).reshape(3, -1).sum(1)).tolist()
    assert patches.shape[0] == int(lens.sum())
    row = 0
    for b in range(3):
        assert patches[row].tolist()[0:2] == [b, -1] and patches[row, 3] == 1
        row += 1
        for ry in range(4):
            for rx in range(4):
                s = int(splits[idx[b, ry, rx]])
                step = 4 // s
                for dy in range(s):
                    for dx in range(s):
                        assert patches[row].tolist() == [b, ry * 4 + dy * step, rx * 4 + dx * step, step]
                        row += 1
    assert row == patches.shape[0]


def test_empty_and_extreme_gates():
    splits = torch.tensor([4, 2, 1])
    # all coarse / all fine / no extra tokens
    for k, per_region in ((2, 1), (0, 16)):
        idx = torch.full((2, 4, 4), k)
        p, l = O.grained_sample_index_to_patch(idx, splits, 4, 1)
        assert l.tolist() == [1 + 16 * per_region] * 2
        p0, l0 = O.grained_sample_index_to_patch(idx, splits, 4, 0)
        assert l0.tolist() == [16 * per_region] * 2 and (p0[:, 1] >= 0).all()
    x = torch.randn(2, 257, 8)
    idx = torch.zeros(2, 4, 4, dtype=torch.int64)
    p, l = O.grained_sample_index_to_patch(idx, splits, 4, 1)
    comp = O.grained_sample_compress(x, p, 16, 16, 1)
    # all-fine: compress is a permutation of the tokens (region-major order)
    back = O.grained_sample_decompress(comp, p, torch.zeros_like(x), 16, 16, 1, True)
    assert torch.equal(back, x)


@needs_ref
def test_sparse_matches_reference_dense():
    """One-hot gate: the sparse ops equal the rows the reference's dense PyTorch
    functions select (vtpack/layers/grained_sample.py:126-177)."""
    _, gs, _, _ = ref_shim.reference_modules()
    g = torch.Generator().manual_seed(11)
    B, H, W, C = 3, 16, 16, 24
    x = torch.randn(B, H * W + 1, C, generator=g)
    splits = torch.tensor([4, 2, 1])
    idx = torch.randint(0, 3, (B, 4, 4), generator=g)
    patches, lens = O.grained_sample_index_to_patch(idx, splits, 4, 1)
    comp = O.grained_sample_compress(x, patches, H, W, 1)
    dense, dlen = gs.grained_sample_compress_dense(x, splits, 4, H, W, 1)
    dense = dense.reshape(B, -1, C)                      # [B, 1+256+64+16, C]
    starts = {1: 1, 2: 1 + 256, 4: 1 + 256 + 64}
    for r in range(patches.shape[0]):
        b, y, xx, step = patches[r].tolist()
        if y < 0:
            ref = dense[b, -y - 1]
        else:
            wi = W // step
            ref = dense[b, starts[step] + (y // step) * wi + xx // step]
        assert torch.allclose(comp[r], ref, rtol=1e-6, atol=1e-6)

    # decompress: scatter sparse rows into the dense layout, one-hot gate
    q = torch.randn(patches.shape[0], C, generator=g)
    gate = torch.zeros(B, 4, 4, 3).scatter_(-1, idx[..., None], 1.0)
    qd = torch.zeros(B, dense.shape[1], C)
    for r in range(patches.shape[0]):
        b, y, xx, step = patches[r].tolist()
        if y < 0:
            qd[b, -y - 1] = q[r]
        else:
            qd[b, starts[step] + (y // step) * (W // step) + xx // step] = q[r]
    ref_out = gs.grained_sample_decompress_dense(qd.reshape(-1, C), gate, x, splits, 4, H, W, 1, True)
    out = O.grained_sample_decompress(q, patches, x, H, W, 1, True)
    assert torch.allclose(out, ref_out, rtol=1e-6, atol=1e-6)


@needs_ref
def test_all_fine_equals_reference_dense_block():
    """Every region at split 4: the DGE block is the dense DeiT block
    (vtpack/models/standard/deit.py:50-83) with q|kv concatenated to qkv."""
    _, _, _, deit = ref_shim.reference_modules()
    C, h = 96, 3
    sd = O.make_state_dict(C, 1, h, seed=3)
    w = O.block_weights(sd, 0)
    x = O.make_tokens(2, 257, C, seed=4)
    gate = torch.zeros(2, 4, 4, 3)
    gate[..., 0] = 1.0
    out = O.dge_block_forward(x, w, h, (4, 2, 1), forced_gate=gate)
    blk = deit.Block(C, h, mlp_ratio=4, qkv_bias=True,
                     norm_layer=lambda d: torch.nn.LayerNorm(d, eps=1e-6))
    dsd = {k: v for k, v in w.items() if not k.startswith(("dge.", "attn.q.", "attn.kv."))}
    dsd["attn.qkv.weight"] = torch.cat([w["attn.q.weight"], w["attn.kv.weight"]], 0)
    dsd["attn.qkv.bias"] = torch.cat([w["attn.q.bias"], w["attn.kv.bias"]], 0)
    blk.load_state_dict(dsd, strict=True)
    blk.eval()
    with torch.no_grad():
        ref = blk(x)
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5)
    assert torch.allclose(O.dense_block_forward(x, w, h), ref, rtol=1e-5, atol=1e-5)


@needs_ref
def test_reference_modules_match_restatement():
    """The reference's Block/VisionTransformer over the _C stand-in equal the
    module-level restatement bit for bit."""
    _, _, deit_dge, _ = ref_shim.reference_modules()
    sd = O.make_state_dict(192, 2, 3, seed=7)
    m = deit_dge.VisionTransformer(img_size=256, patch_size=16, embed_dim=192, depth=2, num_heads=3,
                                   mlp_ratio=4, qkv_bias=True, split_sizes=[4, 2, 1])
    m.load_state_dict(sd, strict=True)
    m.eval()
    x = O.make_images(2, 256, seed=8)
    with torch.no_grad():
        ref = m(x)
    assert torch.equal(O.deit_dge_forward(x, sd, 2, 3, (4, 2, 1)), ref)


def test_pvt_block_golden(golden_dir):
    """The PVT+DGE block of the oracle against what the reference's pvt_dge.Block returned."""
    g = _load(golden_dir, "pvt_block_fp32.npz")
    w = O.make_pvt_block_weights(64, 8, 4, seed=3)
    x = O.make_tokens(2, 32 * 32, 64, seed=4)
    assert math.isclose(x.double().sum().item(), float(g["input_sum"]), rel_tol=0, abs_tol=1e-9)
    assert math.isclose(sum(v.double().sum().item() for v in w.values()), float(g["weight_sum"]),
                        rel_tol=0, abs_tol=1e-9)
    tr = {}
    out = O.dge_block_forward(x, w, 1, (4, 2, 1), trace=tr, grid=(32, 32), sr_ratio=4)
    assert np.array_equal(tr["indices"].numpy().astype(np.int8), g["grain_indices"])
    assert tr["batches"].tolist() == g["batch_lengths"].tolist()
    assert torch.equal(out, torch.from_numpy(g["out"]))


@needs_ref
@pytest.mark.parametrize("C,heads,H,sr,mr,extra", [(64, 1, 32, 8, 8, 0), (128, 2, 16, 4, 8, 0), (320, 5, 8, 2, 4, 0),
                                                   (512, 8, 8, 1, 4, 1)])
def test_pvt_block_matches_reference(C, heads, H, sr, mr, extra):
    """Every stage shape of the reference's PVT+DGE (last stage: no reduction, cls token in front)."""
    import importlib
    from functools import partial
    ref_shim.install()
    pvt = importlib.import_module("vtpack.models.dge.pvt_dge")
    w = O.make_pvt_block_weights(C, mr, sr, seed=5)
    blk = pvt.Block(C, heads, mlp_ratio=mr, qkv_bias=True, norm_layer=partial(torch.nn.LayerNorm, eps=1e-6),
                    sr_ratio=sr, split_sizes=[4, 2, 1]).eval()
    blk.load_state_dict(w, strict=True)
    x = O.make_tokens(2, H * H + extra, C, seed=6)
    with torch.no_grad():
        ref = blk(x, H, H)
    tr = {}
    out = O.dge_block_forward(x, w, heads, (4, 2, 1), trace=tr, grid=(H, H), sr_ratio=sr)
    assert tr["batches"].tolist() == blk.dge.states["batches"].tolist()
    assert torch.equal(out, ref)


def test_pvt_model_golden(golden_dir):
    """The PVT+DGE model of the oracle against what the reference's pvt_dge_s124_tiny_256 returned."""
    g = _load(golden_dir, "pvt_model_fp32.npz")
    cfg = O.PVT_CONFIGS["tiny"]
    sd = O.make_pvt_state_dict(cfg, seed=0)
    x = O.make_images(2, 256, seed=8)
    assert math.isclose(x.double().sum().item(), float(g["input_sum"]), rel_tol=0, abs_tol=1e-9)
    assert math.isclose(sum(v.double().sum().item() for v in sd.values()), float(g["weight_sum"]),
                        rel_tol=0, abs_tol=1e-9)
    tr = []
    logits = O.pvt_dge_forward(x, sd, cfg, trace=tr)
    assert [t["batches"].tolist() for t in tr] == g["batch_lengths"].tolist()
    assert torch.equal(logits, torch.from_numpy(g["logits"]))


# ------------------------------------------------------------------ training path

def test_train_ops_golden_known_answers(golden_dir):
    """The gradients the reference's autograd functions returned (fixture) against closed forms: a
    token receives 1/size^2 of its patch's gradient row; a packed row receives the sum over its
    tokens; the ragged products against per-image torch autograd."""
    z = _load(golden_dir, "train_ops_fp32.npz")
    splits = torch.tensor([4, 2, 1])
    for C in (32, 1):
        x, indices = O.train_ops_inputs(C)
        patches, lengths = O.grained_sample_index_to_patch(indices, splits, 4, 1)
        assert np.array_equal(lengths.numpy(), z[f"c{C}_lengths"])
        L = patches.shape[0]
        assert torch.equal(O.grained_sample_compress(x, patches, 16, 16, 1), torch.from_numpy(z[f"c{C}_comp"]))
        g1, g2 = O.randn_seeded((L, C), 11), O.randn_seeded((2, 257, C), 13)
        grad_x = torch.zeros(2, 257, C)
        grad_q = torch.zeros(L, C)
        for p, (b, y, xx, step) in enumerate(patches.tolist()):
            toks = [-y - 1] if y < 0 else [1 + (y + dy) * 16 + xx + dx for dy in range(step) for dx in range(step)]
            for t in toks:
                grad_x[b, t] = g1[p] / (step * step)
                grad_q[p] += g2[b, t]
        assert torch.allclose(grad_x, torch.from_numpy(z[f"c{C}_grad_x"]), rtol=0, atol=1e-7)
        assert torch.allclose(grad_q, torch.from_numpy(z[f"c{C}_grad_q"]), rtol=1e-6, atol=1e-6)

    h, d, N = 2, 8, 12
    la, lb = torch.tensor([5, 17, 9]), torch.full([3], N, dtype=torch.long)
    L = int(la.sum())
    q = O.randn_seeded((h, L, d), 31).requires_grad_(True)
    k = O.randn_seeded((h, 3 * N, d), 32).requires_grad_(True)
    v = O.randn_seeded((h, 3 * N, d), 33).requires_grad_(True)
    p = O.randn_seeded((h, L, N), 35).requires_grad_(True)
    s = O.batched_sparse_gemm_forward(q, k, la, lb, False, True)       # plain torch ops: autograd applies
    o = O.batched_sparse_gemm_forward(p, v, la, lb, False, False)
    gq, gk = torch.autograd.grad(s, (q, k), O.randn_seeded((h, L, N), 34))
    gp, gv = torch.autograd.grad(o, (p, v), O.randn_seeded((h, L, d), 36))
    for name, t in (("gemm_s", s), ("gemm_o", o), ("gemm_gq", gq), ("gemm_gk", gk), ("gemm_gp", gp), ("gemm_gv", gv)):
        assert torch.allclose(t.detach(), torch.from_numpy(z[name]), rtol=1e-5, atol=1e-6), name


def test_gumbel_stand_in_matches_torch_form():
    """The fixed-noise stand-in is F.gumbel_softmax with the noise made explicit: same forward value
    (one-hot) and same gradient as torch's straight-through form for that noise."""
    logits = O.randn_seeded((2, 4, 4, 3), 7).requires_grad_(True)
    noise = O.make_gumbel_noise((2, 4, 4, 3), 8)
    y = O.gumbel_softmax_fixed([noise])(logits, dim=-1, hard=True)
    assert torch.equal(y.detach().sum(-1), torch.ones(2, 4, 4)) and set(y.detach().unique().tolist()) <= {0.0, 1.0}
    assert torch.equal(y.detach().argmax(-1), (logits.detach() + noise).argmax(-1))
    w = O.randn_seeded((2, 4, 4, 3), 9)
    g, = torch.autograd.grad((y * w).sum(), logits)
    logits2 = logits.detach().clone().requires_grad_(True)
    g2, = torch.autograd.grad((((logits2 + noise).softmax(-1)) * w).sum(), logits2)
    assert torch.allclose(g, g2, atol=1e-7)


@needs_ref
def test_train_block_fixture_matches_reference(golden_dir):
    """The committed training-mode block fixture is what the reference's modules return here."""
    import torch.nn.functional as F
    _, _, deit_dge, _ = ref_shim.reference_modules()
    z = _load(golden_dir, "train_block_fp32.npz")
    cfg = O.TRAIN_BLOCK
    blk = deit_dge.Block(cfg["dim"], cfg["heads"], mlp_ratio=4, qkv_bias=True,
                         norm_layer=lambda d: torch.nn.LayerNorm(d, eps=1e-6), split_sizes=[4, 2, 1])
    blk.load_state_dict(O.train_block_weights(), strict=True)
    blk.train()
    blk.dge.sparse_train = True
    x = O.randn_seeded((cfg["batch"], 257, cfg["dim"]), cfg["token_seed"]).requires_grad_(True)
    real = F.gumbel_softmax
    F.gumbel_softmax = O.gumbel_softmax_fixed([O.make_gumbel_noise((cfg["batch"], 4, 4, 3), cfg["noise_seed"])])
    try:
        y = blk(x)
        (y * O.randn_seeded((cfg["batch"], 257, cfg["dim"]), cfg["grad_seed"])).sum().backward()
    finally:
        F.gumbel_softmax = real
    assert np.array_equal(np.asarray(blk.dge.states["batches"]), z["sparse_lengths"])
    assert torch.allclose(y.detach(), torch.from_numpy(z["sparse_out"]), rtol=1e-5, atol=1e-6)
    assert torch.allclose(x.grad, torch.from_numpy(z["sparse_grad_x"]), rtol=1e-4, atol=1e-6)


# ------------------------------------------------------------------ bilinear-sampling attention

@pytest.mark.parametrize("mode", ["point", "channel"])
def test_bilinear_attention_golden_and_autograd(golden_dir, mode):
    """The restated forward reproduces the fixture (made by the reference's autograd function over the
    stand-in), and the restated backward formulas equal torch autograd of the forward in float64 —
    two independent derivations of the three gradients."""
    from oracle import bilinear_oracle as BO
    z = _load(golden_dir, "bilinear_attention_fp32.npz")
    fwd = getattr(BO, f"bilinear_attention_{mode}wise_forward")
    bwd = getattr(BO, f"bilinear_attention_{mode}wise_backward")
    inp, grid, weight, grad_out = BO.make_bilinear_inputs(seed=BO.GOLDEN_SEEDS[mode], mode=mode, **BO.GOLDEN_CASE)
    assert torch.allclose(fwd(inp, grid, weight), torch.from_numpy(z[f"{mode}_out"]), rtol=1e-6, atol=1e-6)
    gi, gg, gw = bwd(grad_out, inp, grid, weight)
    for name, t in (("grad_input", gi), ("grad_grid", gg), ("grad_weight", gw)):
        assert torch.allclose(t, torch.from_numpy(z[f"{mode}_{name}"]), rtol=1e-5, atol=1e-5), name
    a, g, w = (t.double().requires_grad_(True) for t in (inp, grid, weight))
    auto = torch.autograd.grad(fwd(a, g, w), (a, g, w), grad_out.double())
    for t, ref in zip(bwd(grad_out.double(), a.detach(), g.detach(), w.detach()), auto):
        assert torch.allclose(t, ref, rtol=1e-10, atol=1e-10)
    # taps outside the map read zero: a point more than a pixel outside contributes nothing
    far = grid.clone()
    far[..., 0] = -1.5
    assert not fwd(inp, far, weight).any()


def test_forced_indices_and_image_bias_hooks():
    """The two hooks the parity tests and the bench use change nothing when they restate what the oracle
    does anyway, and force what they say when they do not."""
    sd = O.make_state_dict(192, 2, 3, seed=0)
    img = O.make_images(2, 256, seed=1)
    tr = []
    ref = O.deit_dge_forward(img, sd, 2, 3, (4, 2, 1), trace=tr)
    same = O.deit_dge_forward(img, sd, 2, 3, (4, 2, 1), forced_indices=[t["indices"] for t in tr])
    assert torch.equal(ref, same)
    bias = torch.zeros(2, 3)
    bias[0, 2] = 1e4            # image 0 all-coarse
    bias[1, 0] = 1e4            # image 1 all-fine
    tr2 = []
    O.deit_dge_forward(img, sd, 2, 3, (4, 2, 1), trace=tr2, gate_image_bias=bias)
    assert all(t["batches"].tolist() == [17, 257] for t in tr2)


@pytest.mark.parametrize("B,Hr,Wr,extra,seed", [(2, 4, 4, 1, 0), (3, 2, 3, 0, 1), (1, 8, 8, 2, 2)])
def test_two_restatements_agree_row_for_row(B, Hr, Wr, extra, seed):
    """The vectorised restatement against the scalar one (one kernel work item at a time, in the kernels'
    statement order): patch rows in the same ORDER, pooled rows and unpooled tokens bit for bit.  A permuted
    row order or a transposed sub-patch walk in either would show here, which look-ups by coordinate miss."""
    from oracle import scalar_check as S
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, 3, (B, Hr, Wr), generator=g)
    sp = torch.tensor([4, 2, 1])
    p_vec, l_vec = O.grained_sample_index_to_patch(idx, sp, 4, extra)
    p_sca, l_sca = S.index_to_patch(idx.numpy(), [4, 2, 1], 4, extra)
    assert l_vec.tolist() == l_sca.tolist()
    written = p_sca[:, 2] != -7                       # column 2 of extra-token rows is never written by the reference
    assert (written == (p_sca[:, 1] >= 0)).all()
    assert np.array_equal(p_vec.numpy()[:, [0, 1, 3]], p_sca[:, [0, 1, 3]])
    assert np.array_equal(p_vec.numpy()[written, 2], p_sca[written, 2])
    H, W, C = Hr * 4, Wr * 4, 5
    x = torch.randn(B, extra + H * W, C, generator=g)
    comp_vec = O.grained_sample_compress(x, p_vec, H, W, extra)
    comp_sca = S.compress(x.numpy(), p_vec.numpy(), W, extra)
    assert np.array_equal(comp_vec.numpy(), comp_sca)
    q = torch.randn(p_vec.shape[0], C, generator=g)
    out_vec = O.grained_sample_decompress(q, p_vec, x, H, W, extra, True)
    out_sca = S.decompress_add_ref(q.numpy(), p_vec.numpy(), x.numpy(), W, extra)
    assert not np.isnan(out_sca).any()                # every token belongs to exactly one patch
    assert np.array_equal(out_vec.numpy(), out_sca)
