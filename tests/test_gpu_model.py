"""GPU parity of the block and model forwards (one C-ABI call each) against the golden
fixtures made by the reference's Python modules and against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from tests.gpu_util import O, rel_err

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _block(C, h, sd, dtype):
    from vtpack_b200.models.dge.deit_dge import Block
    blk = Block(C, h, mlp_ratio=4, qkv_bias=True, norm_layer=lambda d: torch.nn.LayerNorm(d, eps=1e-6),
                split_sizes=[4, 2, 1])
    blk.load_state_dict(O.block_weights(sd, 0), strict=True)
    return blk.eval().to(device=DEV, dtype=dtype)


def test_layer_fp32_golden(golden_dir):
    """Benchmark configuration 1: one DeiT-Ti DGE layer, fp32, B=2, injected gate logits; fp32
    tolerance 1e-4 relative."""
    g = np.load(os.path.join(golden_dir, "layer_tiny_fp32.npz"))
    sd = O.make_state_dict(192, 1, 3, seed=0)
    x = O.make_tokens(2, 257, 192, seed=1)
    gate = O.make_gate_logits(2, 4, 4, 3, seed=2)
    blk = _block(192, 3, sd, torch.float32)
    out = blk(x.to(DEV), forced_gate=gate)
    assert blk.dge.states["batches_device"].tolist() == g["batch_lengths"].tolist()
    assert rel_err(out, torch.from_numpy(g["out"])) < 1e-4
    # the op-by-op path through vtpack_b200.layers gives the same (router free-running there)
    blk.dge.router.gate.weight.data.zero_()
    out2 = blk.forward_unfused(x.to(DEV))       # zero gate weights -> all logits equal -> grain 0 everywhere
    ref2 = O.dge_block_forward(x, {**O.block_weights(sd, 0), "dge.router.gate.weight": torch.zeros(3, 192)},
                               3, (4, 2, 1))
    assert rel_err(out2, ref2) < 1e-4


@pytest.mark.parametrize("fine_bias", [-1e4, 0.0, 1e4])
def test_layer_fp32_vs_oracle(fine_bias):
    sd = O.make_state_dict(384, 1, 6, seed=3)
    x = O.make_tokens(3, 257, 384, seed=4)
    gate = O.make_gate_logits(3, 4, 4, 3, seed=5, fine_bias=fine_bias)
    ref = O.dge_block_forward(x, O.block_weights(sd, 0), 6, (4, 2, 1), forced_gate=gate)
    out = _block(384, 6, sd, torch.float32)(x.to(DEV), forced_gate=gate)
    assert rel_err(out, ref) < 1e-4


def test_layer_free_running_gate_fp32():
    sd = O.make_state_dict(192, 1, 3, seed=6)
    x = O.make_tokens(4, 257, 192, seed=7)
    tr = {}
    ref = O.dge_block_forward(x, O.block_weights(sd, 0), 3, (4, 2, 1), trace=tr)
    blk = _block(192, 3, sd, torch.float32)
    out = blk(x.to(DEV))
    assert blk.dge.states["batches_device"].tolist() == tr["batches"].tolist()
    assert rel_err(out, ref) < 1e-4
    assert rel_err(blk.forward_unfused(x.to(DEV)), ref) < 1e-4
    assert torch.equal(blk.dge.states["batches"], tr["batches"])


def test_all_fine_equals_dense_block_fp32():
    sd = O.make_state_dict(192, 1, 3, seed=8)
    x = O.make_tokens(2, 257, 192, seed=9)
    gate = torch.zeros(2, 4, 4, 3)
    gate[..., 0] = 1
    blk = _block(192, 3, sd, torch.float32)
    a = blk(x.to(DEV), forced_gate=gate)
    b = blk(x.to(DEV), dense=True)
    ref = O.dense_block_forward(x, O.block_weights(sd, 0), 3)
    assert rel_err(a, ref) < 1e-4 and rel_err(b, ref) < 1e-4


def test_layer_512px_skewed_fp32():
    """32x32 grid (N=1025, 64 regions); even images all-coarse, odd all-fine."""
    sd = O.make_state_dict(128, 1, 2, img_size=512, seed=10)
    x = O.make_tokens(4, 1025, 128, seed=11)
    gate = torch.zeros(4, 8, 8, 3)
    gate[0::2, ..., 2] = 1e4
    gate[1::2, ..., 0] = 1e4
    ref = O.dge_block_forward(x, O.block_weights(sd, 0), 2, (4, 2, 1), forced_gate=gate)
    blk = _block(128, 2, sd, torch.float32)
    out = blk(x.to(DEV), forced_gate=gate)
    assert blk.dge.states["batches_device"].tolist() == [65, 1025, 65, 1025]
    assert rel_err(out, ref) < 1e-4


@pytest.mark.parametrize("cuda_cores,fold", [(True, False), (False, False), (False, True)])
def test_layer_bf16_vs_fp32_oracle(cuda_cores, fold):
    """bf16 device path vs fp32 math on the bf16-rounded weights and input; with the
    tcgen05 kernels both with explicit LayerNorms and with LayerNorm folded into the GEMMs."""
    from vtpack_b200 import _lib
    sd = O.round_bf16(O.make_state_dict(384, 1, 6, seed=12))
    g = torch.Generator().manual_seed(15)
    for k in ("norm1", "norm2"):     # non-trivial LayerNorm affine so that folding is exercised
        sd[f"blocks.0.{k}.weight"] = (1 + 0.2 * torch.randn(384, generator=g)).bfloat16().float()
        sd[f"blocks.0.{k}.bias"] = (0.2 * torch.randn(384, generator=g)).bfloat16().float()
    x = (O.make_tokens(4, 257, 384, seed=13) + 0.5).bfloat16().float()
    gate = O.make_gate_logits(4, 4, 4, 3, seed=14)
    ref = O.dge_block_forward(x, O.block_weights(sd, 0), 6, (4, 2, 1), forced_gate=gate)
    blk = _block(384, 6, sd, torch.bfloat16)
    blk.fold_layernorm = fold
    blk.flags = _lib.FLAG_CUDA_CORES if cuda_cores else 0
    out = blk(x.bfloat16().to(DEV), forced_gate=gate)
    assert _lib.device_status() == 0
    assert float((out.float().cpu() - ref).abs().max()) < 6e-2      # |x| ~ 4: one bf16 ulp is 3e-2
    assert rel_err(out.float(), ref) < 1.5e-2


def _model(kind, sd, dtype, depth=12, flags=0, img_size=256):
    from vtpack_b200.models.dge import deit_dge
    cfg = O.MODEL_CONFIGS[kind]
    m = deit_dge.VisionTransformer(img_size=img_size, patch_size=16, embed_dim=cfg["embed_dim"], depth=depth,
                                   num_heads=cfg["num_heads"], mlp_ratio=4, qkv_bias=True, split_sizes=[4, 2, 1])
    m.load_state_dict(sd, strict=True)
    m.flags = flags
    return m.eval().to(device=DEV, dtype=dtype)


def test_model_fp32_golden(golden_dir):
    """Full DeiT-Ti+DGE, fp32, free-running router: logits, per-layer query counts."""
    g = np.load(os.path.join(golden_dir, "model_tiny_fp32.npz"))
    sd = O.make_state_dict(192, 12, 3, seed=0)
    m = _model("tiny", sd, torch.float32)
    logits = m(O.make_images(2, 256, seed=1).to(DEV))
    assert g["gate_margin"].min() > 1e-5        # no near-tie in the fixture: counts must match exactly
    assert np.array_equal(m.last_counts.cpu().numpy(), g["batch_lengths"])
    assert rel_err(logits, torch.from_numpy(g["logits"])) < 1e-4
    # MAC accounting of the same forward, from the counts the kernels left on the device
    comp = m.complexity(O.make_images(2, 256, seed=1))
    assert comp["static"].is_cuda and comp["dynamic"].is_cuda
    assert float(comp["static"]) == float(g["comp_static"])
    assert float(comp["dynamic"]) == float(g["comp_dynamic"])


@pytest.mark.parametrize("cuda_cores", [True, False])
def test_model_bf16_logits(cuda_cores):
    """Benchmark configuration 2 at reduced batch: DeiT-Ti+DGE bf16 vs the fp32 oracle on
    bf16-rounded weights; logits max-abs <= 2e-2, top-1 agreement reported."""
    from vtpack_b200 import _lib
    B = 16
    sd = O.round_bf16(O.make_state_dict(192, 12, 3, seed=0))
    img = O.make_images(B, 256, seed=1)
    tr = []
    ref = O.deit_dge_forward(img, sd, 12, 3, (4, 2, 1), trace=tr)
    m = _model("tiny", sd, torch.bfloat16, flags=_lib.FLAG_CUDA_CORES if cuda_cores else 0)
    logits = m(img.to(DEV)).cpu()
    assert _lib.device_status() == 0
    err = float((logits - ref).abs().max())
    agree = float((logits.argmax(-1) == ref.argmax(-1)).float().mean())
    counts_equal = float((m.last_counts.cpu().long() == torch.stack([t["batches"] for t in tr])).float().mean())
    print(f"bf16 logits max-abs err {err:.4f}, top-1 agreement {agree:.3f}, count agreement {counts_equal:.3f}")
    assert err < 2e-2


def test_model_bf16_top1_agreement_1024_images():
    """1024 images through DeiT-Ti+DGE in bf16 against the fp32 oracle on bf16-rounded weights:
    logits within 2e-2 max-abs, and the top-1 class agrees on every image whose oracle top-2 margin
    exceeds twice the largest logit error seen (with random-init weights the 1000 logits of an image
    lie within a few tenths of each other, so a closer call than that is a coin toss for any
    bf16 implementation); the raw agreement is printed."""
    from vtpack_b200 import _lib
    B, chunk = 1024, 256
    sd = O.round_bf16(O.make_state_dict(192, 12, 3, seed=0))
    m = _model("tiny", sd, torch.bfloat16)
    img = O.make_images(B, 256, seed=11)
    ref = torch.cat([O.deit_dge_forward(img[i:i + chunk], sd, 12, 3, (4, 2, 1)) for i in range(0, B, chunk)])
    logits = torch.cat([m(img[i:i + chunk].to(DEV)).cpu() for i in range(0, B, chunk)])
    assert _lib.device_status() == 0
    err = float((logits - ref).abs().max())
    top2 = ref.topk(2, dim=-1).values
    margin = top2[:, 0] - top2[:, 1]
    same = logits.argmax(-1) == ref.argmax(-1)
    clear = margin > 2 * err
    print(f"1024 images: logits max-abs err {err:.4f}, raw top-1 agreement {float(same.float().mean()):.4f}, "
          f"{int(clear.sum())} images with a clear margin, all agree: {bool(same[clear].all())}")
    assert err < 2e-2
    assert bool(same[clear].all())
    assert float(same.float().mean()) > 0.85


@pytest.mark.parametrize("dtype,depth,tol", [(torch.float32, 4, 1e-4), (torch.bfloat16, 12, 2e-2)])
def test_model_512px(dtype, depth, tol):
    """Benchmark configuration 5 shape through the whole-model entry point at reduced batch and width:
    512 x 512 images (32 x 32 grid + cls = 1025 tokens, 64 regions per image, 1025 keys = four
    256-key chunks + one tail key), free-running router.  fp32: logits within 1e-4 relative of
    the oracle wherever the per-layer query counts agree (they must, unless a gate is a near-tie);
    bf16: logits within 2e-2 max-abs of the fp32 oracle on bf16-rounded weights."""
    from vtpack_b200 import _lib
    sd = O.make_state_dict(192, depth, 3, img_size=512, seed=30)
    if dtype == torch.bfloat16:
        sd = O.round_bf16(sd)
    img = O.make_images(3, 512, seed=34)          # smallest top-2 gate margin of the fp32 run: 2.8e-4
    tr = []
    ref = O.deit_dge_forward(img, sd, depth, 3, (4, 2, 1), trace=tr)
    m = _model("tiny", sd, dtype, depth=depth, img_size=512)
    logits = m(img.to(DEV)).cpu()
    assert _lib.device_status() == 0
    counts_ref = torch.stack([t["batches"] for t in tr])
    assert int(counts_ref.min()) >= 65 and int(counts_ref.max()) <= 1025
    if dtype == torch.float32:
        assert torch.equal(m.last_counts.cpu().long(), counts_ref)
        assert rel_err(logits, ref) < tol
    else:
        assert float((logits - ref).abs().max()) < tol


def test_layer_512px_bf16_skewed():
    """Benchmark configuration 5 shape at reduced batch: 32x32 grid (1025 keys = 4 chunks of 256 + 1 tail
    key), even images all-coarse (65 queries), odd images all-fine (1025 queries), bf16."""
    from vtpack_b200 import _lib
    sd = O.round_bf16(O.make_state_dict(384, 1, 6, img_size=512, seed=20))
    x = O.make_tokens(4, 1025, 384, seed=21).bfloat16().float()
    gate = torch.zeros(4, 8, 8, 3)
    gate[0::2, ..., 2] = 1e4
    gate[1::2, ..., 0] = 1e4
    ref = O.dge_block_forward(x, O.block_weights(sd, 0), 6, (4, 2, 1), forced_gate=gate)
    blk = _block(384, 6, sd, torch.bfloat16)
    out = blk(x.bfloat16().to(DEV), forced_gate=gate)
    assert _lib.device_status() == 0
    assert blk.dge.states["batches_device"].tolist() == [65, 1025, 65, 1025]
    assert rel_err(out.float(), ref) < 1.5e-2


@pytest.mark.parametrize("fine_bias", [-1e4, -0.5, 0.7, 1e4])
def test_layer_gate_skew_bf16(fine_bias):
    """Benchmark configuration 4 at reduced batch: gate skew from all-coarse to all-fine."""
    sd = O.round_bf16(O.make_state_dict(384, 1, 6, seed=22))
    x = O.make_tokens(6, 257, 384, seed=23).bfloat16().float()
    gate = O.make_gate_logits(6, 4, 4, 3, seed=24, fine_bias=fine_bias)
    tr = {}
    ref = O.dge_block_forward(x, O.block_weights(sd, 0), 6, (4, 2, 1), forced_gate=gate, trace=tr)
    blk = _block(384, 6, sd, torch.bfloat16)
    out = blk(x.bfloat16().to(DEV), forced_gate=gate)
    assert blk.dge.states["batches_device"].tolist() == tr["batches"].tolist()
    assert rel_err(out.float(), ref) < 1.5e-2


def test_full_size_properties():
    """Benchmark configuration 3 size (DeiT-S, batch 256, bf16): properties that need no oracle run.
    Images are independent, so permuting the batch permutes the logits; every per-image query
    count is 1 + sum of 16 values from {1, 4, 16}, hence within [17, 257] and = 2 (mod 3); with
    every region forced to the finest grain the DGE block is the dense block."""
    from vtpack_b200 import _lib, synthetic
    B = 256
    model = synthetic.build_model("small", DEV, torch.bfloat16)
    img = synthetic.images(B, 256, seed=5).to(DEV)
    logits = model(img).clone()
    counts = model.last_counts.clone()
    assert torch.isfinite(logits).all()
    assert int(counts.min()) >= 17 and int(counts.max()) <= 257
    assert bool(((counts - 2) % 3 == 0).all())
    perm = torch.randperm(B, generator=torch.Generator().manual_seed(6)).to(DEV)
    logits_p = model(img[perm]).clone()
    counts_p = model.last_counts.clone()
    same = (counts_p == counts[:, perm]).float().mean().item()
    assert same > 0.999          # an image computes the same whatever its place in the batch
    keep = (counts_p == counts[:, perm]).all(0)
    assert float((logits_p[keep] - logits[perm][keep]).abs().max()) < 1e-2
    # graph replay gives what the kernel-by-kernel forward gives
    out = torch.empty_like(logits)
    model.forward_graph(img, out)
    model.forward_graph(img, out)
    keep2 = (model.last_counts == counts).all(0)
    assert keep2.float().mean().item() > 0.99
    assert float((out[keep2] - logits[keep2]).abs().max()) < 1e-2
    # all-fine DGE block == dense block
    blk = model.blocks[0]
    x = torch.randn(B, 257, 384, device=DEV, generator=torch.Generator(DEV).manual_seed(7)).bfloat16()
    gate = torch.zeros(B, 4, 4, 3)
    gate[..., 0] = 1.0
    a = blk(x, forced_gate=gate)
    assert blk.dge.states["batches_device"].tolist() == [257] * B
    b = blk(x, dense=True)
    assert rel_err(a.float(), b.float()) < 2e-2
    assert _lib.device_status() == 0


def _pvt_block(C, heads, mr, sr, w, dtype):
    from functools import partial
    from vtpack_b200.models.dge.pvt_dge import Block
    blk = Block(C, heads, mlp_ratio=mr, qkv_bias=True, norm_layer=partial(torch.nn.LayerNorm, eps=1e-6),
                sr_ratio=sr, split_sizes=[4, 2, 1])
    blk.load_state_dict(w, strict=True)
    return blk.eval().to(device=DEV, dtype=dtype)


def test_pvt_block_fp32_golden(golden_dir):
    """PVT+DGE block (spatial reduction 4, 64 keys per image) against the reference's own output."""
    from vtpack_b200 import _lib
    g = np.load(os.path.join(golden_dir, "pvt_block_fp32.npz"))
    w = O.make_pvt_block_weights(64, 8, 4, seed=3)
    blk = _pvt_block(64, 1, 8, 4, w, torch.float32)
    out = blk(O.make_tokens(2, 32 * 32, 64, seed=4).to(DEV), 32, 32)
    assert g["gate_margin"].min() > 1e-5
    assert blk.dge.states["batches_device"].tolist() == g["batch_lengths"].tolist()
    assert rel_err(out, torch.from_numpy(g["out"])) < 1e-4
    assert _lib.device_status() == 0


@pytest.mark.parametrize("C,heads,H,sr,mr,extra", [(64, 1, 64, 8, 8, 0), (128, 2, 32, 4, 8, 0), (320, 5, 16, 2, 4, 0),
                                                   (512, 8, 8, 1, 4, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pvt_block_stages(C, heads, H, sr, mr, extra, dtype):
    """The four stage shapes of PVT+DGE at 256 px (grids 64..8, reductions 8..1, the last with a cls
    token), gates teacher-forced: fp32 within 1e-4 of the oracle; bf16 against the fp32 oracle on
    bf16-rounded weights and inputs."""
    from vtpack_b200 import _lib
    B = 4
    w = O.make_pvt_block_weights(C, mr, sr, seed=7)
    x = O.make_tokens(B, H * H + extra, C, seed=8)
    if dtype == torch.bfloat16:
        w = O.round_bf16(w)
        x = x.bfloat16().float()
    gate = O.make_gate_logits(B, H // 4, H // 4, 3, seed=9)
    tr = {}
    ref = O.dge_block_forward(x, w, heads, (4, 2, 1), forced_gate=gate, trace=tr, grid=(H, H), sr_ratio=sr)
    blk = _pvt_block(C, heads, mr, sr, w, dtype)
    out = blk(x.to(DEV).to(dtype), H, H, forced_gate=gate)
    assert _lib.device_status() == 0
    assert blk.dge.states["batches_device"].tolist() == tr["batches"].tolist()
    err = rel_err(out.float(), ref)
    assert err < (1e-4 if dtype == torch.float32 else 2e-2), err


@pytest.mark.parametrize("C,heads,H,sr,mr,extra", [(64, 1, 64, 8, 8, 0), (128, 2, 32, 4, 8, 0), (320, 5, 16, 2, 4, 0),
                                                   (512, 8, 8, 1, 4, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pvt_stage_in_one_call_equals_block_by_block(C, heads, H, sr, mr, extra, dtype):
    """Three blocks of a stage through ``stage_forward`` (one C-ABI call; in bf16 a block's unpool leaves the
    next block's router decisions, counts and token statistics) against the same blocks called one by one
    (every block runs its own gate and patch-list kernels): identical per-image query counts for every
    block, outputs equal to within the last bit of a few sums whose order differs."""
    from vtpack_b200 import _lib
    from vtpack_b200.models.dge.pvt_dge import stage_forward
    B = 6
    blocks = [_pvt_block(C, heads, mr, sr, O.make_pvt_block_weights(C, mr, sr, seed=20 + i), dtype) for i in range(3)]
    x = O.make_tokens(B, H * H + extra, C, seed=8).to(DEV).to(dtype)
    one = x
    counts_one = []
    for blk in blocks:
        one = blk(one, H, H)
        counts_one.append(blk.dge.states["batches_device"].tolist())
    x_before = x.clone()
    got = stage_forward(blocks, x, H, H)
    assert _lib.device_status() == 0
    assert torch.equal(x, x_before)                       # the caller's tokens are not written
    assert [blk.dge.states["batches_device"].tolist() for blk in blocks] == counts_one
    assert len({tuple(c) for c in counts_one}) > 1        # the blocks did pick different grains
    assert rel_err(got.float(), one.float()) < (1e-6 if dtype == torch.float32 else 4e-3)
    assert blocks[1].dge.get_complexity()["dynamic"] is not None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pvt_model(golden_dir, dtype):
    """PVT+DGE tiny (4 stages, 8 blocks, patch 4: 4096 -> 64 tokens) through the mirror model: fp32
    against the reference's own logits and query counts; bf16 against the fp32 oracle on bf16-rounded
    weights (logits within 2e-2 max-abs)."""
    from vtpack_b200 import _lib
    from vtpack_b200.models.dge.pvt_dge import pvt_dge_s124_tiny_256
    g = np.load(os.path.join(golden_dir, "pvt_model_fp32.npz"))
    cfg = O.PVT_CONFIGS["tiny"]
    sd = O.make_pvt_state_dict(cfg, seed=0)
    img = O.make_images(2, 256, seed=8)
    if dtype == torch.bfloat16:
        sd = O.round_bf16(sd)
        ref = O.pvt_dge_forward(img, sd, cfg)
    else:
        ref = torch.from_numpy(g["logits"])
    m = pvt_dge_s124_tiny_256()
    m.load_state_dict(sd, strict=True)
    m = m.eval().to(device=DEV, dtype=dtype)
    logits = m(img.to(DEV)).cpu()
    assert _lib.device_status() == 0
    if dtype == torch.float32:
        assert g["gate_margin"].min() > 1e-5
        assert [c.tolist() for c in m.last_counts] == g["batch_lengths"].tolist()
        assert rel_err(logits, ref) < 1e-4
    else:
        assert float((logits - ref).abs().max()) < 2e-2


def test_pvt_model_follows_parameter_updates():
    """The eval forward keeps tensors derived from parameters (GEMM-layout weights, fp32 vectors, position rows);
    after parameters change in place — an optimizer step, load_state_dict — the next forward must use the new
    values: compared with a second model, loaded with the changed parameters, that has never run before."""
    from vtpack_b200.models.dge.pvt_dge import pvt_dge_s124_tiny_256
    sd = O.make_pvt_state_dict(O.PVT_CONFIGS["tiny"], seed=0)
    m = pvt_dge_s124_tiny_256()
    m.load_state_dict(sd, strict=True)
    m = m.eval().to(device=DEV, dtype=torch.bfloat16)
    img = O.make_images(2, 256, seed=8).to(DEV)
    first = m(img).clone()
    with torch.no_grad():
        m.patch_embed1.proj.weight.mul_(1.5)
        m.patch_embed2.norm.bias.add_(0.25)
        m.pos_embed3.add_(0.5)
        m.cls_token.add_(1.0)
        m.head.bias.add_(2.0)
    fresh = pvt_dge_s124_tiny_256()
    fresh.load_state_dict({k: v.float().cpu() for k, v in m.state_dict().items()}, strict=True)
    fresh = fresh.eval().to(device=DEV, dtype=torch.bfloat16)
    got, ref = m(img), fresh(img)
    assert torch.equal(got, ref)
    assert float((got - first).abs().max()) > 0.5


def test_pvt_model_other_input_size_and_pyramid(golden_dir):
    """PVT+DGE tiny in eval mode on 384 px images (position embeddings resized bilinearly) and its
    feature-pyramid variant (num_classes = 0), fp32, against the reference's own outputs."""
    from vtpack_b200 import _lib
    from vtpack_b200.models.dge.pvt_dge import pvt_dge_s124_tiny_256
    g = np.load(os.path.join(golden_dir, "pvt_model_384_fp32.npz"))
    sd = O.make_pvt_state_dict(O.PVT_CONFIGS["tiny"], seed=0)
    img = O.make_images(1, 384, seed=10).to(DEV)
    m = pvt_dge_s124_tiny_256()
    m.load_state_dict(sd, strict=True)
    m = m.eval().to(DEV)
    logits = m(img).cpu()
    assert _lib.device_status() == 0
    assert float(g["gate_margin"]) > 1e-5
    assert [c.tolist() for c in m.last_counts] == g["counts"].tolist()
    assert rel_err(logits, torch.from_numpy(g["logits"])) < 1e-4
    m0 = pvt_dge_s124_tiny_256(num_classes=0)
    m0.load_state_dict({k: v for k, v in sd.items() if not k.startswith(("head.", "norm."))}, strict=True)
    feats = m0.eval().to(DEV)(img)
    assert sorted(feats) == ["res2", "res3", "res4", "res5"]
    for k, v in feats.items():
        assert list(v.shape) == g[f"{k}_shape"].tolist(), k
        assert rel_err(v[:, :, ::8, ::8], torch.from_numpy(g[f"{k}_sub"])) < 1e-4, k
        assert abs(float(v.double().sum()) - float(g[f"{k}_sum"])) < 1e-4 * float(v.double().abs().sum()), k
