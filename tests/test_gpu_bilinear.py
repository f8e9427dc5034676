"""GPU parity of the bilinear-sampling attention ops (point and channel mode, forward and the three
gradients) against the reference's autograd function (committed fixture) and the CPU restatement."""
import os

import numpy as np
import pytest
import torch

from oracle import bilinear_oracle as BO
from tests.gpu_util import rel_err

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def op():
    from vtpack_b200 import _lib
    from vtpack_b200.layers import bilinear_attention
    _lib.lib()
    return bilinear_attention


def _run(op, inp, grid, weight, grad_out, mode, dtype=torch.float32):
    a, g, w = (t.to(DEV, dtype).requires_grad_(True) for t in (inp, grid, weight))
    y = op(a, g, w, mode)
    return (y.detach(),) + torch.autograd.grad(y, (a, g, w), grad_out.to(DEV, dtype))


@pytest.mark.parametrize("mode", ["point", "channel"])
def test_bilinear_attention_matches_reference(op, golden_dir, mode):
    z = np.load(os.path.join(golden_dir, "bilinear_attention_fp32.npz"))
    inp, grid, weight, grad_out = BO.make_bilinear_inputs(seed=BO.GOLDEN_SEEDS[mode], mode=mode, **BO.GOLDEN_CASE)
    y, gi, gg, gw = _run(op, inp, grid, weight, grad_out, mode)
    for name, t in (("out", y), ("grad_input", gi), ("grad_grid", gg), ("grad_weight", gw)):
        ref = torch.from_numpy(z[f"{mode}_{name}"])
        assert t.shape == ref.shape, name
        assert rel_err(t, ref) < 1e-5, name


@pytest.mark.parametrize("mode", ["point", "channel"])
@pytest.mark.parametrize("B,H,W,C,G,P", [(6, 16, 16, 64, 256, 9), (2, 32, 32, 64, 1024, 4), (3, 7, 5, 33, 35, 1),
                                         (1, 8, 8, 256, 64, 3)])
def test_bilinear_attention_shapes(op, mode, B, H, W, C, G, P):
    """Deformable-PVT shapes (heads folded into the batch, 64 channels per head, one query per pixel)
    and ragged ones (C not a multiple of the warp, a single point, the widest supported C)."""
    inp, grid, weight, grad_out = BO.make_bilinear_inputs(B, H, W, C, G, P, seed=B * 100 + C + P, mode=mode)
    fwd = getattr(BO, f"bilinear_attention_{mode}wise_forward")
    bwd = getattr(BO, f"bilinear_attention_{mode}wise_backward")
    refs = (fwd(inp.double(), grid.double(), weight.double()),) + bwd(grad_out.double(), inp.double(), grid.double(),
                                                                      weight.double())
    for name, t, ref in zip(("out", "grad_input", "grad_grid", "grad_weight"),
                            _run(op, inp, grid, weight, grad_out, mode), refs):
        assert rel_err(t, ref) < 2e-5, name
    # bf16: same inputs rounded once; outputs within bf16 resolution of the float64 result on them
    rb = lambda t: t.bfloat16().double()      # noqa: E731
    refs16 = (fwd(rb(inp), rb(grid), rb(weight)),) + bwd(rb(grad_out), rb(inp), rb(grid), rb(weight))
    got16 = _run(op, inp, grid, weight, grad_out, mode, torch.bfloat16)
    assert rel_err(got16[0].float(), refs16[0]) < 2e-2
    assert rel_err(got16[2].float(), refs16[2]) < 2e-2 and rel_err(got16[3].float(), refs16[3]) < 2e-2
    assert rel_err(got16[1].float(), refs16[1]) < 6e-2          # sums of bf16 atomics


def test_bilinear_attention_points_outside_and_non_finite(op):
    """Points far outside the map, at infinity or NaN read zero and leave zero gradients; nothing is
    dereferenced out of bounds."""
    inp, grid, weight, grad_out = BO.make_bilinear_inputs(2, 6, 6, 32, 10, 4, seed=5, mode="point")
    grid[0, :, 0, :] = 1e30
    grid[0, :, 1, :] = -1e30
    grid[1, :, 2, 0] = float("inf")
    grid[1, :, 3, 1] = float("nan")
    finite = grid.clone()
    finite[~torch.isfinite(finite) | (finite.abs() > 1e6)] = -3.0          # an equivalent all-outside point
    y, gi, _, gw = _run(op, inp, grid, weight, grad_out, "point")
    y2, gi2, _, gw2 = _run(op, inp, finite, weight, grad_out, "point")
    assert torch.isfinite(y).all() and torch.equal(y, y2) and torch.equal(gi, gi2) and torch.equal(gw, gw2)


def test_dpvt_attention_usage(op):
    """The call sequence of the deformable PVT's attention (dpvt.py:92-115): heads folded into the
    batch, reference points on the pixel grid plus learned offsets, softmax weights, "point" mode."""
    B, H, W, C, heads, P = 2, 8, 8, 128, 2, 4
    N, d = H * W, C // heads
    g = torch.Generator().manual_seed(9)
    v = torch.randn(B, N, heads, d, generator=g).permute(0, 2, 1, 3).reshape(-1, H, W, d)
    mh, mw = torch.meshgrid(torch.linspace(0, H - 1, H), torch.linspace(0, W - 1, W), indexing="ij")
    ref_points = torch.stack([mw, mh], dim=-1).reshape(1, N, 1, 2)
    offsets = torch.randn(B * heads, N, P, 2, generator=g) * 1.5
    weight = torch.randn(B * heads, N, P, generator=g).softmax(-1)
    grid = ref_points + offsets
    want = BO.bilinear_attention_pointwise_forward(v.double(), grid.double(), weight.double())
    got = op(v.to(DEV).contiguous(), grid.to(DEV), weight.to(DEV), "point")
    assert got.shape == (B * heads, N, d) and rel_err(got, want) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sparse_bilinear_attention_packed_queries(dtype):
    """Packed (variable number per image) queries: equal to the dense op on each image's slice, and to
    the CPU restatement; an image without queries and unsorted image indices included."""
    from vtpack_b200.layers import bilinear_attention, sparse_bilinear_attention_pointwise_forward
    B, H, W, C, P = 4, 9, 7, 48, 3
    g = torch.Generator().manual_seed(12)
    inp = torch.randn(B, H, W, C, generator=g)
    batches = torch.tensor([0] * 5 + [3] * 11 + [1] * 2 + [3] * 4)          # image 2 has no query
    L = batches.numel()
    grid = torch.rand(L, P, 2, generator=g) * torch.tensor([W + 3.0, H + 3.0]) - 2.0
    weight = torch.randn(L, P, generator=g)
    rb = (lambda t: t.to(dtype).double())
    want = BO.sparse_bilinear_attention_pointwise_forward(rb(inp), rb(grid), rb(weight), batches)
    got = sparse_bilinear_attention_pointwise_forward(inp.to(DEV, dtype), grid.to(DEV, dtype), weight.to(DEV, dtype),
                                                      batches.to(DEV))
    assert got.shape == (L, C) and got.dtype == dtype
    assert rel_err(got.float(), want) < (1e-5 if dtype == torch.float32 else 2e-2)
    sel = batches == 3
    dense = bilinear_attention(inp[3:4].to(DEV, dtype).contiguous(), grid[sel][None].to(DEV, dtype),
                               weight[sel][None].to(DEV, dtype), "point")[0]
    assert torch.equal(got[sel.to(DEV)], dense)


def test_dpvt_attention_module_matches_reference(golden_dir):
    """The deformable attention module (dpvt.py:51-115) over this library's op: output, input
    gradient and all eight parameter gradients against the reference's own module."""
    from oracle import dge_oracle as O
    from vtpack_b200.models.standard.dpvt import Attention
    z = np.load(os.path.join(golden_dir, "dpvt_attention_fp32.npz"))
    c = O.DPVT_ATTENTION
    att = Attention(c["dim"], num_heads=c["heads"], qkv_bias=True, num_points=c["points"])
    att.load_state_dict(O.dpvt_attention_weights(), strict=True)
    att.to(DEV)
    x = O.randn_seeded((c["batch"], c["H"] * c["W"], c["dim"]), c["token_seed"]).to(DEV).requires_grad_(True)
    y = att(x, c["H"], c["W"])
    (y * O.randn_seeded(tuple(y.shape), c["grad_seed"]).to(DEV)).sum().backward()
    assert rel_err(y, torch.from_numpy(z["out"])) < 1e-5
    assert rel_err(x.grad, torch.from_numpy(z["grad_x"])) < 1e-4
    n = 0
    for name, prm in att.named_parameters():
        assert rel_err(prm.grad, torch.from_numpy(z[f"grad.{name}"])) < 1e-4, name
        n += 1
    assert n == 8
