"""CPU restatement of the reference's bilinear-sampling attention ops.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the fixture generator and by oracle/ref_shim.py
(as the CPU stand-in behind the reference's own ``vtpack/layers/bilinear_attention.py``); never by
the shipped package.

Follows ``vtpack/layers/csrc/bilinear_attention/bilinear_attention.cu``: sampling ``:52-86``
(floor, four taps, zero outside the map), point-wise forward ``:88-132`` and backward ``:134-232``,
channel-wise forward ``:234-268`` and backward ``:270-362``.  The backward functions spell out the
reference's formulas term by term; tests/test_oracle.py checks them against torch autograd of the
forward restatement (an independent derivation).
"""
import torch


def _taps(inp: torch.Tensor, grid: torch.Tensor):
    """inp [B,H,W,C], grid [B,G,P,2] (x, y) -> tap values [4][B,G,P,C] (lt, rt, lb, rb; zero outside),
    their flat pixel indices and validity masks, and the fractions tx, ty [B,G,P]."""
    B, H, W, C = inp.shape
    _, G, P, _ = grid.shape
    x, y = grid[..., 0], grid[..., 1]
    x0, y0 = torch.floor(x).long(), torch.floor(y).long()
    tx, ty = x - x0, y - y0
    flat = inp.reshape(B, H * W, C)
    vals, idxs, oks = [], [], []
    for dy, dx in ((0, 0), (0, 1), (1, 0), (1, 1)):
        yy, xx = y0 + dy, x0 + dx
        ok = (yy >= 0) & (yy < H) & (xx >= 0) & (xx < W)
        idx = yy.clamp(0, H - 1) * W + xx.clamp(0, W - 1)
        v = flat.gather(1, idx.reshape(B, G * P, 1).expand(-1, -1, C)).reshape(B, G, P, C)
        vals.append(v * ok[..., None].to(inp.dtype))
        idxs.append(idx)
        oks.append(ok)
    return vals, idxs, oks, tx, ty


def _sample(inp, grid):
    (lt, rt, lb, rb), _, _, tx, ty = _taps(inp, grid)
    tx, ty = tx[..., None], ty[..., None]
    return (1 - tx) * (1 - ty) * lt + tx * (1 - ty) * rt + (1 - tx) * ty * lb + tx * ty * rb     # [B,G,P,C]


def bilinear_attention_pointwise_forward(inp, grid, weight):
    """weight [B,G,P] -> [B,G,C] (``bilinear_attention.cu:88-132``)."""
    return (_sample(inp, grid) * weight[..., None]).sum(dim=2)


def bilinear_attention_channelwise_forward(inp, grid, weight):
    """weight [B,G,C] -> [B,G,P] (``bilinear_attention.cu:234-268``)."""
    return (_sample(inp, grid) * weight[:, :, None, :]).sum(dim=-1)


def sparse_bilinear_attention_pointwise_forward(inp, grid, weight, batches):
    """Packed queries: grid [L,P,2], weight [L,P], batches int64 [L] -> [L,C]
    (``vtpack/layers/csrc/sparse_bilinear_attention/sparse_bilinear_attention.cu:88-171``): query i
    samples image batches[i]; otherwise the point-wise forward."""
    out = torch.empty(grid.shape[0], inp.shape[3], dtype=inp.dtype)
    for b in batches.unique().tolist():
        sel = batches == b
        out[sel] = bilinear_attention_pointwise_forward(inp[b:b + 1], grid[sel][None], weight[sel][None])[0]
    return out


def _backward(g_sample, inp, grid):
    """Common part of both backward kernels, given g_sample = d loss / d sample [B,G,P,C]: the
    scattered input gradient (``:183-194`` / ``:312-323``) and the point gradients (``:205-219`` /
    ``:334-348``)."""
    B, H, W, C = inp.shape
    (lt, rt, lb, rb), idxs, oks, tx, ty = _taps(inp, grid)
    txc, tyc = tx[..., None], ty[..., None]
    w4 = ((1 - txc) * (1 - tyc), txc * (1 - tyc), (1 - txc) * tyc, txc * tyc)
    grad_input = torch.zeros(B, H * W, C, dtype=inp.dtype)
    for wk, idx, ok in zip(w4, idxs, oks):
        contrib = g_sample * wk * ok[..., None].to(inp.dtype)
        grad_input.scatter_add_(1, idx.reshape(B, -1, 1).expand(-1, -1, C), contrib.reshape(B, -1, C))
    g_lt, g_rt, g_lb, g_rb = lt * g_sample, rt * g_sample, lb * g_sample, rb * g_sample
    gix = (-g_lt * (1 - tyc) + g_rt * (1 - tyc) - g_lb * tyc + g_rb * tyc).sum(-1)
    giy = (-g_lt * (1 - txc) - g_rt * txc + g_lb * (1 - txc) + g_rb * txc).sum(-1)
    sample = w4[0] * lt + w4[1] * rt + w4[2] * lb + w4[3] * rb
    return grad_input.reshape(B, H, W, C), torch.stack([gix, giy], dim=-1), sample


def bilinear_attention_pointwise_backward(grad_output, inp, grid, weight):
    """-> (grad_input [B,H,W,C], grad_grid [B,G,P,2], grad_weight [B,G,P]) (``:134-232``)."""
    g_sample = grad_output[:, :, None, :] * weight[..., None]
    grad_input, grad_grid, sample = _backward(g_sample, inp, grid)
    grad_weight = (sample * grad_output[:, :, None, :]).sum(-1)
    return grad_input, grad_grid, grad_weight


def bilinear_attention_channelwise_backward(grad_output, inp, grid, weight):
    """-> (grad_input [B,H,W,C], grad_grid [B,G,P,2], grad_weight [B,G,C]) (``:270-362``)."""
    g_sample = grad_output[..., None] * weight[:, :, None, :]
    grad_input, grad_grid, sample = _backward(g_sample, inp, grid)
    grad_weight = (sample * grad_output[..., None]).sum(2)
    return grad_input, grad_grid, grad_weight


GOLDEN_CASE = dict(B=2, H=9, W=11, C=40, G=23, P=5)      # tests/golden/bilinear_attention_fp32.npz
GOLDEN_SEEDS = {"point": 41, "channel": 42}


def make_bilinear_inputs(B, H, W, C, G, P, seed, mode):
    """Seeded inputs: a random map, sampling points spread over the map and a margin of two pixels
    around it (so that every in/out-of-bounds tap combination occurs), random weights."""
    g = torch.Generator().manual_seed(seed)
    inp = torch.randn(B, H, W, C, generator=g)
    grid = torch.rand(B, G, P, 2, generator=g) * torch.tensor([W + 3.0, H + 3.0]) - 2.0
    weight = torch.randn(B, G, P if mode == "point" else C, generator=g)
    grad_out = torch.randn(B, G, C if mode == "point" else P, generator=g)
    return inp, grid, weight, grad_out
