"""GPU parity of the training path: gradients of the token movers, the ragged products, and a
training-mode DeiT+DGE block, against what the reference's own autograd functions returned on the
same seeded inputs (committed fixtures; tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from tests.gpu_util import O, rel_err

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = 1e-4          # fp32, relative to the largest reference value


@pytest.fixture(scope="module")
def layers():
    from vtpack_b200 import _lib, layers
    _lib.lib()
    return layers


def _golden(golden_dir, name):
    return {k: torch.from_numpy(v) for k, v in np.load(os.path.join(golden_dir, name)).items()}


@pytest.mark.parametrize("C", [32, 1])
def test_mover_gradients_match_reference(layers, golden_dir, C):
    z = _golden(golden_dir, "train_ops_fp32.npz")
    splits = torch.tensor([4, 2, 1])
    x, indices = O.train_ops_inputs(C)
    x = x.to(DEV).requires_grad_(True)
    patches, lengths = layers.grained_sample_index_to_patch(indices.to(DEV), splits, 4, 1)
    assert torch.equal(lengths, z[f"c{C}_lengths"])
    L = patches.shape[0]
    comp = layers.grained_sample_compress(x, patches, 16, 16, 1)
    assert torch.equal(comp.detach().cpu(), z[f"c{C}_comp"])
    grad_x, = torch.autograd.grad(comp, x, O.randn_seeded((L, C), 11).to(DEV))
    assert torch.equal(grad_x.cpu(), z[f"c{C}_grad_x"])            # a power-of-two scale: exact
    q = O.randn_seeded((L, C), 12).to(DEV).requires_grad_(True)
    ref = x.detach().clone().requires_grad_(True)
    tok = layers.grained_sample_decompress(q, patches, ref, 16, 16, 1, True)
    g2 = O.randn_seeded((2, 257, C), 13).to(DEV)
    grad_q, grad_ref = torch.autograd.grad(tok, (q, ref), g2)
    assert torch.equal(grad_ref, g2)
    assert rel_err(grad_q, z[f"c{C}_grad_q"]) < 1e-6
    # without the reference term the reference tensor receives a zero gradient (grained_sample.py:76-77)
    tok2 = layers.grained_sample_decompress(q, patches, ref, 16, 16, 1, False)
    _, grad_ref2 = torch.autograd.grad(tok2, (q, ref), g2)
    assert not grad_ref2.any()


@pytest.mark.parametrize("B,G,C", [(3, 16, 384), (2, 32, 64)])
def test_mover_gradients_bf16_and_adjoint(layers, B, G, C):
    """Size-independent property: <pool(x), g> == <x, pool_grad(g)> and the same for the unpool (the
    gradient kernels are the adjoints of the forward kernels); bf16 gradients round the fp32 ones."""
    splits = torch.tensor([4, 2, 1])
    gen = torch.Generator().manual_seed(B * G + C)
    indices = torch.randint(0, 3, (B, G // 4, G // 4), generator=gen).to(DEV)
    patches, _ = layers.grained_sample_index_to_patch(indices, splits, 4, 1)
    L, N = patches.shape[0], G * G + 1
    x = torch.randn(B, N, C, generator=gen).to(DEV).requires_grad_(True)
    g = torch.randn(L, C, generator=gen).to(DEV)
    comp = layers.grained_sample_compress(x, patches, G, G, 1)
    gx, = torch.autograd.grad(comp, x, g)
    lhs, rhs = (comp.detach().double() * g.double()).sum(), (x.detach().double() * gx.double()).sum()
    assert abs(float(lhs - rhs)) < 1e-6 * max(1.0, abs(float(lhs)))
    q = torch.randn(L, C, generator=gen).to(DEV).requires_grad_(True)
    gt = torch.randn(B, N, C, generator=gen).to(DEV)
    tok = layers.grained_sample_decompress(q, patches, x.detach(), G, G, 1, False)
    gq, = torch.autograd.grad(tok, q, gt)
    lhs, rhs = (tok.detach().double() * gt.double()).sum(), (q.detach().double() * gq.double()).sum()
    assert abs(float(lhs - rhs)) < 1e-6 * max(1.0, abs(float(lhs)))
    # bf16
    xb = x.detach().bfloat16().requires_grad_(True)
    gxb, = torch.autograd.grad(layers.grained_sample_compress(xb, patches, G, G, 1), xb, g.bfloat16())
    gx_ref, = torch.autograd.grad(layers.grained_sample_compress(x, patches, G, G, 1), x, g.bfloat16().float())
    assert torch.equal(gxb.float(), gx_ref)                             # exact: scale by 1, 1/4 or 1/16
    qb = q.detach().bfloat16().requires_grad_(True)
    tokb = layers.grained_sample_decompress(qb, patches, xb.detach(), G, G, 1, False)
    gqb, = torch.autograd.grad(tokb, qb, gt.bfloat16())
    tokf = layers.grained_sample_decompress(q, patches, x.detach(), G, G, 1, False)
    gqf, = torch.autograd.grad(tokf, q, gt.bfloat16().float())
    # fp32 sums, one rounding.  The fp32 and bf16 rows use different lane layouts of the region kernel, whose
    # partial sums are taken in a different order: the fp32 sums agree to rounding, so the bf16 results agree
    # except where a sum sits on a rounding boundary (one bf16 step, 2^-8 relative)
    assert rel_err(gqb.float(), gqf) < 4e-3
    step = gqf.abs().clamp_min(1e-3) * 2.0 ** -7
    assert bool(((gqb.float() - gqf.bfloat16().float()).abs() <= step).all())
    assert float((gqb != gqf.bfloat16()).float().mean()) < 1e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,G,C", [(3, 16, 384), (2, 32, 64), (5, 16, 192), (2, 16, 32)])
def test_unpool_grad_region_form_matches_the_list_walk(layers, dtype, B, G, C):
    """The gradient of the replicate-unpool for its packed rows in its two forms: a walk over the patch
    list (any list) and one thread block per region (a list made from grain indices).  fp32 sums in a
    different order: equal to fp32 rounding; the autograd function picks the region form when the list
    carries its regions.  Also checks the per-region first rows the Python side derives."""
    import ctypes
    from vtpack_b200 import _lib
    from vtpack_b200.runtime import dtype_code, ptr, stream_ptr
    lib = _lib.lib()
    splits = torch.tensor([4, 2, 1])
    gen = torch.Generator().manual_seed(B * 31 + G + C)
    indices = torch.randint(0, 3, (B, G // 4, G // 4), generator=gen).to(DEV)
    patches, _ = layers.grained_sample_index_to_patch(indices, splits, 4, 1)
    L, N = patches.shape[0], G * G + 1
    idx32, first, splits_l, region_size, Hr, Wr, extra = patches._vtp_regions
    # the first row of every region, read off the list itself: the row whose (y, x) is the region's corner
    pl = patches.cpu()
    corner = (pl[:, 1] >= 0) & (pl[:, 1] % 4 == 0) & (pl[:, 2] % 4 == 0)
    rows = torch.nonzero(corner).reshape(-1)
    rid = pl[rows, 0] * (Hr * Wr) + (pl[rows, 1] // 4) * Wr + pl[rows, 2] // 4
    want = torch.empty(B * Hr * Wr, dtype=torch.long)
    want[rid] = rows
    assert torch.equal(first.cpu().reshape(-1).long(), want)

    g = torch.randn(B, N, C, generator=gen).to(dtype).to(DEV)
    by_list = torch.empty(L, C, dtype=dtype, device=DEV)
    _lib.check(lib.vtp_unpool_grad(ptr(g), dtype_code(dtype), B, N, C, G, 1, ptr(patches._vtp_i32), None, L,
                                   ptr(by_list), stream_ptr(g.device)))
    supported = bool(lib.vtp_region_layout_supported(dtype_code(dtype), C))
    arr = (ctypes.c_int * 3)(4, 2, 1)
    by_region = torch.full((L, C), float("nan"), dtype=dtype, device=DEV)
    rc = lib.vtp_unpool_grad_regions(ptr(g), dtype_code(dtype), B, Hr, Wr, 4, C, 1, ptr(idx32), arr, 3, ptr(first),
                                     ptr(patches._vtp_offsets), L, ptr(by_region), stream_ptr(g.device))
    if not supported:
        assert rc == _lib.ERR_SHAPE          # rows of 4 chunks have no lane layout: the list walk is the general form
        return
    _lib.check(rc)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    # reference: the sum over each patch's tokens in fp64
    want_sum = torch.zeros(L, C, dtype=torch.float64)
    gd = g.double().cpu()
    for p in range(L):
        b, y, x, st = (int(v) for v in pl[p])
        if y < 0:
            want_sum[p] = gd[b, -y - 1]
        else:
            toks = [1 + (y + dy) * G + x + dx for dy in range(st) for dx in range(st)]
            want_sum[p] = gd[b, toks].sum(0)
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    assert rel_err(by_region.double().cpu(), want_sum) < tol
    assert rel_err(by_list.double().cpu(), want_sum) < tol
    if dtype == torch.float32:
        assert rel_err(by_region, by_list) < 1e-6
    # the autograd function takes the region form for this list
    q = torch.zeros(L, C, dtype=dtype, device=DEV, requires_grad=True)
    tok = layers.grained_sample_decompress(q, patches, torch.zeros(B, N, C, dtype=dtype, device=DEV), G, G, 1, False)
    gq, = torch.autograd.grad(tok, q, g)
    assert torch.equal(gq, by_region)
    # ... and the list walk for a list without them
    plain = patches.clone()
    tok = layers.grained_sample_decompress(q, plain, torch.zeros(B, N, C, dtype=dtype, device=DEV), G, G, 1, False)
    gq2, = torch.autograd.grad(tok, q, g)
    assert torch.equal(gq2, by_list)


def test_unpool_grad_region_form_skips_rows_beyond_the_declared_count(layers):
    """First rows supplied by the caller are checked against the declared row count: with grad_q declared 40
    rows shorter than the buffer the test owns, the regions whose patches end beyond that are skipped, the
    rows beyond stay untouched and the status word is set.  Nothing points outside an allocation."""
    import ctypes
    from vtpack_b200 import _lib
    from vtpack_b200.runtime import dtype_code, ptr, stream_ptr
    lib = _lib.lib()
    B, G, C = 2, 16, 384
    indices = torch.zeros(B, 4, 4, dtype=torch.int64, device=DEV)            # every region at the finest grain
    patches, _ = layers.grained_sample_index_to_patch(indices, torch.tensor([4, 2, 1]), 4, 1)
    L, N = patches.shape[0], G * G + 1
    idx32, first, _, _, Hr, Wr, _ = patches._vtp_regions
    g = torch.randn(B, N, C, device=DEV).bfloat16()
    out = torch.full((L, C), 7.0, dtype=torch.bfloat16, device=DEV)
    arr = (ctypes.c_int * 3)(4, 2, 1)
    declared = L - 40
    _lib.device_status()
    _lib.check(lib.vtp_unpool_grad_regions(ptr(g), dtype_code(g.dtype), B, Hr, Wr, 4, C, 1, ptr(idx32), arr, 3,
                                           ptr(first), ptr(patches._vtp_offsets), declared, ptr(out),
                                           stream_ptr(g.device)))
    torch.cuda.synchronize()
    assert _lib.device_status() == _lib.STATUS_BAD_INDEX
    assert bool((out[declared:] == 7.0).all())
    full = torch.empty(L, C, dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.vtp_unpool_grad_regions(ptr(g), dtype_code(g.dtype), B, Hr, Wr, 4, C, 1, ptr(idx32), arr, 3,
                                           ptr(first), ptr(patches._vtp_offsets), L, ptr(full), stream_ptr(g.device)))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    kept = int(first.reshape(-1)[first.reshape(-1) + 16 <= declared].max()) + 16     # rows of the regions that fit
    assert torch.equal(out[:kept], full[:kept])


def test_ragged_products_match_reference(layers, golden_dir):
    z = _golden(golden_dir, "train_ops_fp32.npz")
    h, d, N = 2, 8, 12
    la, lb = torch.tensor([5, 17, 9]), torch.full([3], N, dtype=torch.long)
    L = int(la.sum())
    q = O.randn_seeded((h, L, d), 31).to(DEV).requires_grad_(True)
    k = O.randn_seeded((h, 3 * N, d), 32).to(DEV).requires_grad_(True)
    v = O.randn_seeded((h, 3 * N, d), 33).to(DEV).requires_grad_(True)
    p = O.randn_seeded((h, L, N), 35).to(DEV).requires_grad_(True)
    s = layers.batched_sparse_gemm(q, k, la, lb, False, True)
    o = layers.batched_sparse_gemm(p, v, la, lb, False, False)
    gq, gk = torch.autograd.grad(s, (q, k), O.randn_seeded((h, L, N), 34).to(DEV))
    gp, gv = torch.autograd.grad(o, (p, v), O.randn_seeded((h, L, d), 36).to(DEV))
    for name, t in (("gemm_s", s), ("gemm_o", o), ("gemm_gq", gq), ("gemm_gk", gk), ("gemm_gp", gp), ("gemm_gv", gv)):
        assert t.shape == z[name].shape, name
        assert rel_err(t.detach(), z[name]) < 1e-5, name


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False)])
def test_ragged_products_all_flag_combinations(layers, dtype, ta, tb):
    """The transpose combinations the forward and backward passes use (both operands transposed
    would need the same row count in every image on both sides), ragged lengths (an empty image included) and sizes that are not
    multiples of the tile, against the CPU restatement in float64."""
    h, B, ka = 3, 4, 70
    la = torch.tensor([67, 0, 129, 5])
    gen = torch.Generator().manual_seed(17 + 2 * ta + tb)
    a = torch.randn(h, int(la.sum()), ka, generator=gen).to(dtype)
    if ta:          # op(a_i) is [ka, la]: b_i needs la rows (or la columns when transposed)
        lb = la if not tb else torch.full([B], 33, dtype=torch.long)
        kb = 41 if not tb else None
    else:           # op(a_i) is [la, ka]: b_i needs ka rows (or ka columns when transposed)
        lb = torch.full([B], ka, dtype=torch.long) if not tb else torch.full([B], 33, dtype=torch.long)
        kb = 41 if not tb else ka
    b = torch.randn(h, int(lb.sum()), kb, generator=gen).to(dtype)
    ref = O.batched_sparse_gemm_forward(a.double(), b.double(), la, lb, ta, tb)
    out = layers.batched_sparse_gemm(a.to(DEV), b.to(DEV), la, lb, ta, tb)
    assert out.shape == ref.shape and out.dtype == dtype
    assert rel_err(out.float(), ref) < (1e-5 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("keys,d,las", [(257, 64, [113, 41, 257, 0, 130]), (264, 64, [70, 129]), (65, 64, [33, 7]),
                                        (1025, 32, [300, 5])])
def test_ragged_products_model_shapes_bf16(layers, keys, d, las):
    """The six products of the training-mode attention (forward S = Q K^T and O = P V; backward dP = dO V^T,
    dQ = dS K, dK = dS^T Q, dV = P^T dO) at the model's shapes: 257 keys (rows of 514 bytes: unaligned rows, a
    one-column tail beside the 256-column tile, a reduction of 4 x 64 + 1), query counts below, at and above
    one 128-row tile, an image without queries; also 264 keys (an 8-column tail), 65 and 1025.  bf16 on tensor
    cores against float64 on the bf16-rounded operands."""
    h = 3
    B = len(las)
    la, lb = torch.tensor(las), torch.full([B], keys, dtype=torch.long)
    L = int(la.sum())
    gen = torch.Generator().manual_seed(keys + d + L)
    q = torch.randn(h, L, d, generator=gen).bfloat16()
    k = torch.randn(h, B * keys, d, generator=gen).bfloat16()
    p = torch.randn(h, L, keys, generator=gen).bfloat16()
    cases = [("S = Q K^T", q, k, la, lb, False, True), ("O = P V", p, k, la, lb, False, False),
             ("dK = dS^T Q", p, q, la, la, True, False)]
    for name, a, b, xa, xb, ta, tb in cases:
        ref = O.batched_sparse_gemm_forward(a.double(), b.double(), xa, xb, ta, tb)
        out = layers.batched_sparse_gemm(a.to(DEV), b.to(DEV), xa, xb, ta, tb)
        torch.cuda.synchronize()
        assert out.shape == ref.shape and out.dtype == torch.bfloat16, name
        assert rel_err(out.float(), ref) < 8e-3, name
    # operands that start 2 bytes into their storage (a view) cannot be fetched with aligned 16-byte loads: the
    # call takes the CUDA-core kernel and gives the same product to bf16 rounding
    def shifted(t):
        buf = torch.empty(t.numel() + 1, dtype=t.dtype, device=DEV)
        view = buf[1:].view(t.shape)
        view.copy_(t)
        assert view.data_ptr() % 16 != 0
        return view
    ref = O.batched_sparse_gemm_forward(q.double(), k.double(), la, lb, False, True)
    out = layers.batched_sparse_gemm(shifted(q), shifted(k), la, lb, False, True)
    assert rel_err(out.float(), ref) < 8e-3
    from vtpack_b200 import _lib
    assert _lib.device_status() == 0


def _train_block(mode):
    from vtpack_b200.models.dge import deit_dge
    cfg = O.TRAIN_BLOCK
    blk = deit_dge.Block(cfg["dim"], cfg["heads"], mlp_ratio=4, qkv_bias=True,
                         norm_layer=lambda d: torch.nn.LayerNorm(d, eps=1e-6), split_sizes=[4, 2, 1])
    blk.load_state_dict(O.train_block_weights(), strict=True)
    blk.to(DEV).train()
    blk.dge.sparse_train = mode == "sparse"
    return blk, cfg


@pytest.mark.parametrize("mode", ["sparse", "dense"])
def test_training_block_matches_reference(golden_dir, mode):
    """Forward value, input gradient, every parameter gradient and the complexity term of one
    training-mode block, with the reference's Gumbel noise injected."""
    z = _golden(golden_dir, "train_block_fp32.npz")
    blk, cfg = _train_block(mode)
    x = O.randn_seeded((cfg["batch"], 257, cfg["dim"]), cfg["token_seed"]).to(DEV).requires_grad_(True)
    g = O.randn_seeded((cfg["batch"], 257, cfg["dim"]), cfg["grad_seed"]).to(DEV)
    real = F.gumbel_softmax
    F.gumbel_softmax = O.gumbel_softmax_fixed([O.make_gumbel_noise((cfg["batch"], 4, 4, 3), cfg["noise_seed"])])
    try:
        y = blk(x)
        comp = blk.dge.get_complexity()
        ((y * g).sum() + 1e-9 * comp["dynamic"].sum()).backward()
    finally:
        F.gumbel_softmax = real
    assert torch.equal(torch.as_tensor(blk.dge.states["batches"]).cpu(), z[f"{mode}_lengths"])
    assert rel_err(comp["dynamic"].detach(), z[f"{mode}_comp_dynamic"]) < 1e-12
    assert rel_err(y.detach(), z[f"{mode}_out"]) < TOL
    assert rel_err(x.grad, z[f"{mode}_grad_x"]) < TOL
    checked = 0
    for name, prm in blk.named_parameters():
        key = f"{mode}_grad.{name}"
        if key in z:
            assert prm.grad is not None, name
            assert rel_err(prm.grad, z[key]) < 5 * TOL, name
            checked += 1
    assert checked == 16          # two LayerNorms, five Linears and the gate: weight and bias each


def test_training_model_step_and_eval_after():
    """A DeiT-Ti+DGE model takes an SGD step in training mode (sparse_train on): gradients reach the
    router and the patch embedding, and the fused eval forward afterwards runs on the updated
    weights (its packed copies are rebuilt)."""
    from vtpack_b200.models.dge import deit_dge
    torch.manual_seed(0)
    m = deit_dge.deit_dge_s124_tiny_patch16_256().to(DEV)
    for blk in m.blocks:
        blk.dge.sparse_train = True
    images = O.make_images(4, 256, seed=3).to(DEV)
    m.eval()
    with torch.no_grad():
        logits_before = m(images).clone()
    m.train()
    target = torch.tensor([1, 2, 3, 4], device=DEV)
    opt = torch.optim.SGD(m.parameters(), lr=1e-2)
    before = m.blocks[0].dge.router.gate.weight.detach().clone()
    logits = m(images)
    assert logits.shape == (4, 1000) and logits.requires_grad
    budget = torch.stack([blk.dge.get_complexity()["dynamic"].mean() for blk in m.blocks]).sum()
    loss = F.cross_entropy(logits, target) + 1e-10 * budget
    loss.backward()
    assert torch.isfinite(loss)
    params = dict(m.named_parameters())
    for name in ("patch_embed.proj.weight", "blocks.0.dge.router.gate.weight", "blocks.11.attn.kv.weight"):
        grad = params[name].grad
        assert grad is not None and torch.isfinite(grad).all() and grad.abs().max() > 0, name
    opt.step()
    assert not torch.equal(before, m.blocks[0].dge.router.gate.weight.detach())
    m.eval()
    with torch.no_grad():
        logits_after = m(images)
    assert torch.isfinite(logits_after).all() and not torch.equal(logits_after, logits_before)


def test_training_pvt_block_matches_reference(golden_dir):
    """A PVT+DGE block with spatial-reduction keys in training mode (sparse_train on): output,
    input gradient and all parameter gradients against the reference's."""
    from functools import partial
    from vtpack_b200.models.dge import pvt_dge
    z = _golden(golden_dir, "train_pvt_block_fp32.npz")
    cfg = O.TRAIN_PVT_BLOCK
    blk = pvt_dge.Block(cfg["dim"], cfg["heads"], mlp_ratio=cfg["mlp_ratio"], qkv_bias=True,
                        norm_layer=partial(torch.nn.LayerNorm, eps=1e-6), sr_ratio=cfg["sr"], split_sizes=[4, 2, 1])
    blk.load_state_dict(O.make_pvt_block_weights(cfg["dim"], cfg["mlp_ratio"], cfg["sr"], seed=cfg["weight_seed"]),
                        strict=True)
    blk.to(DEV).train()
    blk.dge.sparse_train = True
    G = cfg["grid"]
    x = O.randn_seeded((cfg["batch"], G * G, cfg["dim"]), cfg["token_seed"]).to(DEV).requires_grad_(True)
    g = O.randn_seeded((cfg["batch"], G * G, cfg["dim"]), cfg["grad_seed"]).to(DEV)
    real = F.gumbel_softmax
    F.gumbel_softmax = O.gumbel_softmax_fixed([O.make_gumbel_noise((cfg["batch"], G // 4, G // 4, 3), cfg["noise_seed"])])
    prev = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False          # the reduction convolution in full fp32
    try:
        y = blk(x, G, G)
        (y * g).sum().backward()
    finally:
        F.gumbel_softmax = real
        torch.backends.cudnn.allow_tf32 = prev
    assert torch.equal(blk.dge.states["batches"].cpu(), z["lengths"])
    assert rel_err(y, z["out"]) < TOL
    assert rel_err(x.grad, z["grad_x"]) < TOL
    checked = 0
    for name, prm in blk.named_parameters():
        if f"grad.{name}" in z:
            assert rel_err(prm.grad, z[f"grad.{name}"]) < 5 * TOL, name
            checked += 1
    assert checked == 20          # DeiT block's 16 plus the reduction convolution and its LayerNorm


def test_training_pvt_model_matches_reference(golden_dir):
    """PVT+DGE tiny in training mode (sparse_train on, one injected Gumbel-noise tensor per block):
    the same per-block query counts, logits, loss and parameter gradients as the reference."""
    from vtpack_b200.models.dge import pvt_dge
    z = _golden(golden_dir, "train_pvt_model_fp32.npz")
    cfg, t = O.PVT_CONFIGS["tiny"], O.TRAIN_PVT_MODEL
    m = pvt_dge.pvt_dge_s124_tiny_256()
    m.load_state_dict(O.make_pvt_state_dict(cfg, seed=t["weight_seed"]), strict=True)
    m.to(DEV).train()
    blocks = [b for i in range(4) for b in getattr(m, f"block{i + 1}")]
    for b in blocks:
        b.dge.sparse_train = True
    x = O.make_images(t["batch"], 256, seed=t["image_seed"]).to(DEV)
    real = F.gumbel_softmax
    F.gumbel_softmax = O.gumbel_softmax_fixed(O.train_pvt_model_noises(cfg))
    prev = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False          # the patch and reduction convolutions in full fp32
    try:
        logits = m(x)
        counts = torch.stack([b.dge.states["batches"].cpu() for b in blocks])
        loss = F.cross_entropy(logits, torch.tensor(t["target"], device=DEV))
        loss.backward()
    finally:
        F.gumbel_softmax = real
        torch.backends.cudnn.allow_tf32 = prev
    assert torch.equal(counts, z["counts"])
    assert rel_err(logits, z["logits"]) < TOL
    assert abs(float(loss.detach()) - float(z["loss"])) < 1e-4
    params = dict(m.named_parameters())
    for name in t["grads"]:
        assert rel_err(params[name].grad, z[f"grad.{name}"]) < 1e-3, name
    # the feature-pyramid variant returns the four stage maps
    m.num_classes = 0
    F.gumbel_softmax = O.gumbel_softmax_fixed(O.train_pvt_model_noises(cfg))
    try:
        with torch.no_grad():
            feats = m(x)
    finally:
        F.gumbel_softmax = real
    assert [tuple(feats[f"res{i}"].shape) for i in (2, 3, 4, 5)] == [(2, 64, 64, 64), (2, 128, 32, 32),
                                                                       (2, 320, 16, 16), (2, 512, 8, 8)]
