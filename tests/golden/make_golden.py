"""Generate the golden fixtures in this folder.

Runs the reference's own, unmodified Python modules (imported from its
checkout through ``oracle/ref_shim.py``) on seeded synthetic inputs and
stores what they return.  Needs the reference checkout; run from the repo
root:  ``python tests/golden/make_golden.py``.

Fixtures
  layer_tiny_fp32.npz   one DeiT-Ti DGE block, fp32, B=2, 16x16 grid + cls,
                        dim 192, 3 heads; weights seed 0, tokens seed 1,
                        gate logits seed 2 injected in place of the router.
  model_tiny_fp32.npz   full DeiT-Ti+DGE (12 blocks), fp32, B=2, images seed 1,
                        free-running router: logits, per-layer grain indices
                        and per-image query counts.
  pvt_block_fp32.npz    one PVT+DGE block (pvt_dge.py), fp32, B=2, 32x32 grid, no extra
                        token, dim 64, 1 head, mlp ratio 8, spatial reduction 4 (64 keys);
                        weights seed 3, tokens seed 4, free-running router.
  pvt_model_fp32.npz    full PVT+DGE tiny (pvt_dge_s124_tiny_256: 4 stages, 8 blocks), fp32, B=2,
                        weights seed 0, images seed 8, free-running router: logits and the
                        per-block per-image query counts.
  train_ops_fp32.npz    gradients of the training path's native ops from the reference's own autograd
                        functions: grained_sample_compress / _decompress (B=2, 16x16 grid + cls,
                        C=32 and the one-channel case) and batched_sparse_gemm in the two flag
                        combinations the model uses (forward values and both gradients).
  train_block_fp32.npz  one DeiT+DGE block (dim 64, 2 heads) in training mode, fp32, B=2, with
                        sparse_train on and off; Gumbel noise seed 21 injected through
                        oracle.dge_oracle.gumbel_softmax_fixed; output, input gradient and
                        parameter gradients for the loss sum(out * g), g seed 22.
  train_pvt_block_fp32.npz  one PVT+DGE block (dim 32, 1 head, 16x16 grid, spatial reduction 2) in
                        training mode with sparse_train on, fp32, B=2; Gumbel noise seed 23 injected;
                        output, input gradient, parameter gradients for sum(out * g), g seed 24.
  bilinear_attention_fp32.npz  the reference's bilinear_attention autograd function
                        (vtpack/layers/bilinear_attention.py) in both modes on B=2, 9x11 map, C=40,
                        G=23 queries, P=5 points reaching two pixels outside the map: output and the
                        three gradients.
  train_pvt_model_fp32.npz  PVT+DGE tiny (pvt_dge_s124_tiny_256) in training mode with sparse_train on,
                        fp32, B=2, one injected Gumbel-noise tensor per block: logits, cross-entropy
                        loss, per-block query counts and six (small) parameter gradients.
  pvt_model_384_fp32.npz  PVT+DGE tiny in eval mode on 384 px images (position embeddings resized), fp32,
                        B=1, weights seed 0, images seed 10: logits, per-block query counts, and the
                        feature pyramid of the same weights with num_classes = 0 (every 8th pixel of each
                        map and each map's float64 sum).
  dpvt_attention_fp32.npz  the reference's deformable attention module (dpvt.py Attention: dim 64, 4 heads,
                        3 points, 8x6 map, B=2) forward and backward: output, input gradient and all eight
                        parameter gradients for sum(out * g).
Inputs are regenerated from the seeds by the tests; each fixture carries a
float64 sum of its inputs so RNG drift is detected rather than misread as a
parity failure.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import bilinear_oracle as BO  # noqa: E402
from oracle import dge_oracle as O  # noqa: E402
from oracle import ref_shim  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def layer_fixture():
    _, _, deit_dge, _ = ref_shim.reference_modules()
    sd = O.make_state_dict(192, 1, 3, seed=0)
    x = O.make_tokens(2, 257, 192, seed=1)
    gate = O.make_gate_logits(2, 4, 4, 3, seed=2)
    blk = deit_dge.Block(192, 3, mlp_ratio=4, qkv_bias=True,
                         norm_layer=lambda d: torch.nn.LayerNorm(d, eps=1e-6),
                         split_sizes=[4, 2, 1])
    blk.load_state_dict(O.block_weights(sd, 0), strict=True)
    blk.eval()
    blk.dge.router.forward = lambda t: gate          # teacher-forced gate logits
    with torch.no_grad():
        out = blk(x)
    st = blk.dge.states
    np.savez_compressed(
        os.path.join(HERE, "layer_tiny_fp32.npz"),
        input_sum=np.float64(x.double().sum().item()),
        weight_sum=np.float64(sum(v.double().sum().item() for v in sd.values())),
        gate_sum=np.float64(gate.double().sum().item()),
        patches=st["patches"].numpy().astype(np.int16),
        batch_lengths=st["batches"].numpy(),
        comp_rows=st["comp"][::7].numpy(),
        out=out.numpy(),
    )
    print("layer:", out.shape, st["batches"].tolist())


def model_fixture():
    _, _, deit_dge, _ = ref_shim.reference_modules()
    sd = O.make_state_dict(192, 12, 3, seed=0)
    m = deit_dge.deit_dge_s124_tiny_patch16_256()
    m.load_state_dict(sd, strict=True)
    m.eval()
    x = O.make_images(2, 256, seed=1)
    with torch.no_grad():
        logits = m(x)
        idx, cnt, margin = [], [], []
        for blk in m.blocks:
            g = blk.dge.states["gate"]
            idx.append(g.argmax(-1).numpy())
            cnt.append(blk.dge.states["batches"].numpy())
            top2 = g.topk(2, dim=-1).values
            margin.append((top2[..., 0] - top2[..., 1]).numpy())
        comp = m.complexity(x)               # the reference's own MAC accounting of this forward
    np.savez_compressed(
        os.path.join(HERE, "model_tiny_fp32.npz"),
        input_sum=np.float64(x.double().sum().item()),
        weight_sum=np.float64(sum(v.double().sum().item() for v in sd.values())),
        logits=logits.numpy(),
        grain_indices=np.stack(idx).astype(np.int8),
        batch_lengths=np.stack(cnt),
        gate_margin=np.stack(margin),
        comp_static=np.float64(float(comp["static"])),
        comp_dynamic=np.float64(float(comp["dynamic"])),
    )
    print("model:", logits.shape, np.stack(cnt).tolist(), "min margin", float(np.stack(margin).min()),
          "MACs static/dynamic", float(comp["static"]), float(comp["dynamic"]))


def pvt_block_fixture():
    import importlib
    from functools import partial
    ref_shim.install()
    pvt = importlib.import_module("vtpack.models.dge.pvt_dge")
    C, heads, H, sr, mr = 64, 1, 32, 4, 8
    w = O.make_pvt_block_weights(C, mr, sr, seed=3)
    blk = pvt.Block(C, heads, mlp_ratio=mr, qkv_bias=True, norm_layer=partial(torch.nn.LayerNorm, eps=1e-6),
                    sr_ratio=sr, split_sizes=[4, 2, 1])
    blk.load_state_dict(w, strict=True)
    blk.eval()
    x = O.make_tokens(2, H * H, C, seed=4)
    with torch.no_grad():
        out = blk(x, H, H)
    st = blk.dge.states
    top2 = st["gate"].topk(2, dim=-1).values
    np.savez_compressed(
        os.path.join(HERE, "pvt_block_fp32.npz"),
        input_sum=np.float64(x.double().sum().item()),
        weight_sum=np.float64(sum(v.double().sum().item() for v in w.values())),
        grain_indices=st["gate"].argmax(-1).numpy().astype(np.int8),
        batch_lengths=st["batches"].numpy(),
        gate_margin=(top2[..., 0] - top2[..., 1]).numpy(),
        out=out.numpy(),
    )
    print("pvt block:", out.shape, st["batches"].tolist(), "min margin", float((top2[..., 0] - top2[..., 1]).min()))


def pvt_model_fixture():
    import importlib
    ref_shim.install()
    pvt = importlib.import_module("vtpack.models.dge.pvt_dge")
    cfg = O.PVT_CONFIGS["tiny"]
    sd = O.make_pvt_state_dict(cfg, seed=0)
    m = pvt.pvt_dge_s124_tiny_256()
    m.load_state_dict(sd, strict=True)
    m.eval()
    x = O.make_images(2, 256, seed=8)
    with torch.no_grad():
        logits = m(x)
    cnt, margin = [], []
    for i in range(4):
        for blk in getattr(m, f"block{i + 1}"):
            cnt.append(blk.dge.states["batches"].numpy())
            top2 = blk.dge.states["gate"].topk(2, dim=-1).values
            margin.append(float((top2[..., 0] - top2[..., 1]).min()))
    np.savez_compressed(
        os.path.join(HERE, "pvt_model_fp32.npz"),
        input_sum=np.float64(x.double().sum().item()),
        weight_sum=np.float64(sum(v.double().sum().item() for v in sd.values())),
        logits=logits.numpy(),
        batch_lengths=np.stack(cnt),
        gate_margin=np.array(margin),
    )
    print("pvt model:", logits.shape, np.stack(cnt).tolist(), "min margin", min(margin))


def train_ops_fixture():
    _, gs, _, _ = ref_shim.reference_modules()
    import importlib
    sparse_ops = importlib.import_module("vtpack.layers.sparse_ops")
    out = {}
    splits = torch.tensor([4, 2, 1])
    for C in (32, 1):
        x, indices = O.train_ops_inputs(C)
        x.requires_grad_(True)
        patches, lengths = gs.grained_sample_index_to_patch(indices, splits, 4, 1)
        L = patches.shape[0]
        comp = gs.grained_sample_compress(x, patches, 16, 16, 1)
        g1 = O.randn_seeded((L, C), 11)
        grad_x, = torch.autograd.grad(comp, x, g1.clone())
        q = O.randn_seeded((L, C), 12).requires_grad_(True)
        ref = x.detach().clone().requires_grad_(True)
        tok = gs.grained_sample_decompress(q, patches, ref, 16, 16, 1, True)
        g2 = O.randn_seeded((2, 257, C), 13)
        grad_q, grad_ref = torch.autograd.grad(tok, (q, ref), g2.clone())
        assert torch.equal(grad_ref, g2)
        out.update({f"c{C}_comp": comp.detach().numpy(), f"c{C}_grad_x": grad_x.numpy(),
                    f"c{C}_grad_q": grad_q.numpy(), f"c{C}_lengths": lengths.numpy()})
    # ragged products: queries [h, L, d] x keys [h, B*N, d]^T, then probabilities x values
    h, d, N = 2, 8, 12
    la = torch.tensor([5, 17, 9])
    lb = torch.full([3], N, dtype=torch.long)
    L = int(la.sum())
    qh = O.randn_seeded((h, L, d), 31).requires_grad_(True)
    kh = O.randn_seeded((h, 3 * N, d), 32).requires_grad_(True)
    vh = O.randn_seeded((h, 3 * N, d), 33).requires_grad_(True)
    s = sparse_ops.batched_sparse_gemm(qh, kh, la, lb, False, True)
    gs_ = O.randn_seeded((h, L, N), 34)
    gq, gk = torch.autograd.grad(s, (qh, kh), gs_.clone())
    p = O.randn_seeded((h, L, N), 35).requires_grad_(True)
    o = sparse_ops.batched_sparse_gemm(p, vh, la, lb, False, False)
    go = O.randn_seeded((h, L, d), 36)
    gp, gv = torch.autograd.grad(o, (p, vh), go.clone())
    out.update(gemm_s=s.detach().numpy(), gemm_gq=gq.numpy(), gemm_gk=gk.numpy(),
               gemm_o=o.detach().numpy(), gemm_gp=gp.numpy(), gemm_gv=gv.numpy())
    np.savez_compressed(os.path.join(HERE, "train_ops_fp32.npz"), **out)
    print("train_ops_fp32.npz", {k: v.shape for k, v in out.items()})


def train_block_fixture():
    _, _, deit_dge, _ = ref_shim.reference_modules()
    import torch.nn.functional as F
    cfg = O.TRAIN_BLOCK
    sd = O.train_block_weights()
    out = {}
    real = F.gumbel_softmax
    for mode in ("sparse", "dense"):
        blk = deit_dge.Block(cfg["dim"], cfg["heads"], mlp_ratio=4, qkv_bias=True,
                             norm_layer=lambda d: torch.nn.LayerNorm(d, eps=1e-6), split_sizes=[4, 2, 1])
        blk.load_state_dict(sd, strict=True)
        blk.train()
        blk.dge.sparse_train = mode == "sparse"
        x = O.randn_seeded((cfg["batch"], 257, cfg["dim"]), cfg["token_seed"]).requires_grad_(True)
        g = O.randn_seeded((cfg["batch"], 257, cfg["dim"]), cfg["grad_seed"])
        F.gumbel_softmax = O.gumbel_softmax_fixed([O.make_gumbel_noise((cfg["batch"], 4, 4, 3), cfg["noise_seed"])])
        try:
            y = blk(x)
            comp = blk.dge.get_complexity()
            loss = (y * g).sum() + 1e-9 * comp["dynamic"].sum()
            loss.backward()
        finally:
            F.gumbel_softmax = real
        out[f"{mode}_out"] = y.detach().numpy()
        out[f"{mode}_grad_x"] = x.grad.numpy()
        out[f"{mode}_lengths"] = np.asarray(blk.dge.states["batches"])
        out[f"{mode}_comp_dynamic"] = comp["dynamic"].detach().numpy()
        for name, prm in blk.named_parameters():
            if prm.grad is not None:
                out[f"{mode}_grad.{name}"] = prm.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "train_block_fp32.npz"), **out)
    print("train_block_fp32.npz", sorted(out)[:6], "...", len(out), "arrays")


def train_pvt_block_fixture():
    import importlib
    from functools import partial
    import torch.nn.functional as F
    ref_shim.install()
    pvt = importlib.import_module("vtpack.models.dge.pvt_dge")
    cfg = O.TRAIN_PVT_BLOCK
    w = O.make_pvt_block_weights(cfg["dim"], cfg["mlp_ratio"], cfg["sr"], seed=cfg["weight_seed"])
    blk = pvt.Block(cfg["dim"], cfg["heads"], mlp_ratio=cfg["mlp_ratio"], qkv_bias=True,
                    norm_layer=partial(torch.nn.LayerNorm, eps=1e-6), sr_ratio=cfg["sr"], split_sizes=[4, 2, 1])
    blk.load_state_dict(w, strict=True)
    blk.train()
    blk.dge.sparse_train = True
    G = cfg["grid"]
    x = O.randn_seeded((cfg["batch"], G * G, cfg["dim"]), cfg["token_seed"]).requires_grad_(True)
    g = O.randn_seeded((cfg["batch"], G * G, cfg["dim"]), cfg["grad_seed"])
    real = F.gumbel_softmax
    F.gumbel_softmax = O.gumbel_softmax_fixed([O.make_gumbel_noise((cfg["batch"], G // 4, G // 4, 3), cfg["noise_seed"])])
    try:
        y = blk(x, G, G)
        (y * g).sum().backward()
    finally:
        F.gumbel_softmax = real
    out = {"out": y.detach().numpy(), "grad_x": x.grad.numpy(), "lengths": np.asarray(blk.dge.states["batches"])}
    for name, prm in blk.named_parameters():
        if prm.grad is not None:
            out[f"grad.{name}"] = prm.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "train_pvt_block_fp32.npz"), **out)
    print("train_pvt_block_fp32.npz", out["lengths"], len(out), "arrays")


def bilinear_fixture():
    import importlib
    ref_shim.install()
    ba = importlib.import_module("vtpack.layers.bilinear_attention")
    out = {}
    for mode, seed in BO.GOLDEN_SEEDS.items():
        inp, grid, weight, grad_out = BO.make_bilinear_inputs(seed=seed, mode=mode, **BO.GOLDEN_CASE)
        inp.requires_grad_(True), grid.requires_grad_(True), weight.requires_grad_(True)
        y = ba.bilinear_attention(inp, grid, weight, mode)
        gi, gg, gw = torch.autograd.grad(y, (inp, grid, weight), grad_out)
        out.update({f"{mode}_out": y.detach().numpy(), f"{mode}_grad_input": gi.numpy(),
                    f"{mode}_grad_grid": gg.numpy(), f"{mode}_grad_weight": gw.numpy()})
    np.savez_compressed(os.path.join(HERE, "bilinear_attention_fp32.npz"), **out)
    print("bilinear_attention_fp32.npz", {k: v.shape for k, v in out.items()})


def train_pvt_model_fixture():
    import importlib
    import torch.nn.functional as F
    ref_shim.install()
    pvt = importlib.import_module("vtpack.models.dge.pvt_dge")
    cfg, t = O.PVT_CONFIGS["tiny"], O.TRAIN_PVT_MODEL
    m = pvt.pvt_dge_s124_tiny_256()
    m.load_state_dict(O.make_pvt_state_dict(cfg, seed=t["weight_seed"]), strict=True)
    m.train()
    blocks = [b for i in range(4) for b in getattr(m, f"block{i + 1}")]
    for b in blocks:
        b.dge.sparse_train = True
    x = O.make_images(t["batch"], 256, seed=t["image_seed"])
    real = F.gumbel_softmax
    F.gumbel_softmax = O.gumbel_softmax_fixed(O.train_pvt_model_noises(cfg))
    try:
        logits = m(x)
        counts = np.stack([np.asarray(b.dge.states["batches"]) for b in blocks])
        loss = F.cross_entropy(logits, torch.tensor(t["target"]))
        loss.backward()
    finally:
        F.gumbel_softmax = real
    params = dict(m.named_parameters())
    out = {"logits": logits.detach().numpy(), "loss": np.float64(loss.item()), "counts": counts}
    for name in t["grads"]:
        out[f"grad.{name}"] = params[name].grad.numpy()
    np.savez_compressed(os.path.join(HERE, "train_pvt_model_fp32.npz"), **out)
    print("train_pvt_model_fp32.npz loss", loss.item(), counts.tolist())


def pvt_384_fixture():
    import importlib
    ref_shim.install()
    pvt = importlib.import_module("vtpack.models.dge.pvt_dge")
    cfg = O.PVT_CONFIGS["tiny"]
    sd = O.make_pvt_state_dict(cfg, seed=0)
    x = O.make_images(1, 384, seed=10)
    out = {}
    m = pvt.pvt_dge_s124_tiny_256()
    m.load_state_dict(sd, strict=True)
    m.eval()
    with torch.no_grad():
        out["logits"] = m(x).numpy()
    blocks = [b for i in range(4) for b in getattr(m, f"block{i + 1}")]
    out["counts"] = np.stack([np.asarray(b.dge.states["batches"]) for b in blocks])
    out["gate_margin"] = np.float64(min(float((t.values[..., 0] - t.values[..., 1]).min()) for t in
                                        (b.dge.states["gate"].topk(2, dim=-1) for b in blocks)))
    m0 = pvt.pvt_dge_s124_tiny_256(num_classes=0)
    m0.load_state_dict({k: v for k, v in sd.items() if not k.startswith(("head.", "norm."))}, strict=True)
    m0.eval()
    with torch.no_grad():
        feats = m0(x)
    for k, v in feats.items():
        out[f"{k}_sub"] = v[:, :, ::8, ::8].numpy()
        out[f"{k}_sum"] = np.float64(v.double().sum().item())
        out[f"{k}_shape"] = np.asarray(v.shape)
    np.savez_compressed(os.path.join(HERE, "pvt_model_384_fp32.npz"), **out)
    print("pvt_model_384_fp32.npz", out["counts"].tolist(), "min gate margin", out["gate_margin"],
          {k: v.shape for k, v in feats.items()})


def dpvt_attention_fixture():
    import importlib
    ref_shim.install()
    dpvt = importlib.import_module("vtpack.models.standard.dpvt")
    c = O.DPVT_ATTENTION
    att = dpvt.Attention(c["dim"], num_heads=c["heads"], qkv_bias=True, num_points=c["points"])
    att.load_state_dict(O.dpvt_attention_weights(), strict=True)
    x = O.randn_seeded((c["batch"], c["H"] * c["W"], c["dim"]), c["token_seed"]).requires_grad_(True)
    y = att(x, c["H"], c["W"])
    (y * O.randn_seeded(tuple(y.shape), c["grad_seed"])).sum().backward()
    out = {"out": y.detach().numpy(), "grad_x": x.grad.numpy()}
    for name, prm in att.named_parameters():
        out[f"grad.{name}"] = prm.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "dpvt_attention_fp32.npz"), **out)
    print("dpvt_attention_fp32.npz", len(out), "arrays")


if __name__ == "__main__":
    layer_fixture()
    model_fixture()
    pvt_block_fixture()
    pvt_model_fixture()
    train_ops_fixture()
    train_block_fixture()
    train_pvt_block_fixture()
    bilinear_fixture()
    train_pvt_model_fixture()
    pvt_384_fixture()
    dpvt_attention_fixture()
