#!/usr/bin/env python
"""Throughput benchmark of the DeiT+DGE eval forward (BASELINE metric: images/sec).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = one forward of `--batch` synthetic 256x256 images per GPU through the whole
model (patch embed, 12 DGE blocks, head) with the logits all-gathered when N > 1.
Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the
reference's eval path on the host cores instead.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
STAGES = ["router_gate", "patch_list", "pool_ln1", "q_proj", "kv_proj", "attention", "out_proj", "ln2", "fc1_gelu",
          "fc2", "unpool_add"]
# DRAM bytes (read + written) of one launch of the dominant kernel on the roofline's workload (the kv
# projection at batch 256: M=65792, N=768, K=384), from the ncu capture summarised in
# profiles/linear_tc_kv_projection_m65792_n768_k384.md; scaled by the row count for other batch sizes
NCU_TRAFFIC_BYTES_PER_ROW = (51159296 + 43509504) / 65792


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {k: float(d.get(k, FALLBACK_PEAKS[k])) for k in FALLBACK_PEAKS}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while running."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_reference_rate(model_kind, batch, steps, warmup):
    """images/sec of the CPU restatement of the reference's eval forward (fp32, all host cores)."""
    from oracle import dge_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = O.MODEL_CONFIGS[model_kind]
    sd = O.make_state_dict(cfg["embed_dim"], cfg["depth"], cfg["num_heads"], seed=0)
    img = O.make_images(batch, 256, seed=1)
    with torch.no_grad():
        for _ in range(warmup):
            O.deit_dge_forward(img, sd, cfg["depth"], cfg["num_heads"], (4, 2, 1))
        t0 = time.perf_counter()
        for _ in range(steps):
            O.deit_dge_forward(img, sd, cfg["depth"], cfg["num_heads"], (4, 2, 1))
        dt = time.perf_counter() - t0
    return batch * steps / dt, dt / steps * 1e3, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    b = args.cpu_batch
    rate, ms, cores = cpu_reference_rate(args.model, b, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": "images/sec", "value": rate, "unit": "images/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"DeiT-{args.model}+DGE s124 256px eval forward, CPU, fp32", "batch_per_step": b},
        "cpu_baseline": {"value": rate, "unit": "images/s", "cores": cores, "kind": "port",
                         "sample": f"{args.steps} forwards of {b} images (same model/config), torch CPU fp32"},
        "e2e": {"value": rate, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def stage_profile(model, batch, device, iters, pk):
    """Per-kernel times of one DGE block (block 0 weights) on N(0,1) tokens, from events the
    library records between its launches; returns (rows, roofline of the dominant kernel)."""
    import ctypes
    from vtpack_b200 import _lib
    from vtpack_b200.models.dge.deit_dge import _pack_block
    from vtpack_b200.runtime import scratch
    blk = model.blocks[len(model.blocks) // 2]
    C, N = model.embed_dim, (model.img_size // model.patch_size) ** 2 + 1
    dtype = model.compute_dtype()
    e = 2 if dtype == torch.bfloat16 else 4
    x = torch.randn(batch, N, C, device=device, generator=torch.Generator(device).manual_seed(3)).to(dtype)
    out = torch.empty_like(x)
    s = blk.shape_struct(x)
    w = _pack_block(blk, dtype)
    lib = _lib.lib()
    nbytes = lib.vtp_block_workspace_bytes(ctypes.byref(s))
    ws = scratch(device, nbytes)
    counts = torch.empty(batch, dtype=torch.int32, device=device)
    n_ev = len(STAGES) + 1
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(n_ev)] for _ in range(iters)]
    stream = torch.cuda.current_stream(device)
    for it in range(iters + 2):
        row = evs[max(it - 2, 0)]
        for ev in row:
            ev.record(stream)            # creates the underlying cudaEvent_t
        arr = (ctypes.c_void_p * n_ev)(*[ev.cuda_event for ev in row])
        _lib.check(lib.vtp_dge_block_forward_timed(ctypes.byref(s), ctypes.byref(w), x.data_ptr(), out.data_ptr(),
                                                   None, counts.data_ptr(), ws.data_ptr(), nbytes, arr, n_ev,
                                                   stream.cuda_stream))
    torch.cuda.synchronize(device)
    L = int(counts.sum().item())
    ms = [sum(evs[i][j].elapsed_time(evs[i][j + 1]) for i in range(iters)) / iters for j in range(len(STAGES))]
    BN, H = batch * N, 4 * C
    work = {   # (kind, algorithmic bytes or flops)
        # LayerNorm is folded into the GEMM epilogues on the bf16 path: the pool writes comp rows
        # and 8 bytes of statistics per row; there is no LN2 kernel (its slot measures ~0)
        "router_gate": ("hbm", batch * (N - 1) * C * e), "patch_list": ("hbm", batch * 16 * 12),
        "pool_ln1": ("hbm", (BN + L) * C * e + (BN + 2 * L) * 8), "q_proj": ("tensor", 2 * L * C * C),
        "kv_proj": ("tensor", 4 * BN * C * C), "attention": ("tensor", 4 * L * N * C),
        "out_proj": ("tensor", 2 * L * C * C), "ln2": ("hbm", 0),
        "fc1_gelu": ("tensor", 2 * L * C * H), "fc2": ("tensor", 2 * L * C * H),
        "unpool_add": ("hbm", (2 * BN + 2 * L) * C * e),
    }
    rows = []
    for name, t in zip(STAGES, ms):
        kind, amount = work[name]
        if amount == 0:
            continue
        if kind == "hbm":
            ach, peak, unit = amount / (t * 1e-3) / 1e9, pk["hbm_gbs"], "GB/s"
        else:
            ach, peak, unit = amount / (t * 1e-3) / 1e12, pk["bf16_tflops_sustained"], "TFLOP/s"
        rows.append({"kernel": name, "ms": round(t, 4), "bound": kind, "achieved": round(ach, 1), "unit": unit,
                     "frac": round(ach / peak, 3)})
    gemm = [r for r in rows if r["kernel"] in ("q_proj", "kv_proj", "out_proj", "fc1_gelu", "fc2")]
    gemm_ms = sum(r["ms"] for r in gemm)
    gemm_flops = sum(work[r["kernel"]][1] for r in gemm)
    # the dominant kernel is the tcgen05 Linear; its roofline line is its largest launch (kv projection)
    kv = next(r for r in rows if r["kernel"] == "kv_proj")
    roof = {"kernel": "linear_tc_kernel, kv projection launch (M=B*N tokens, N=2C, K=C)", "bound": "tensor",
            "achieved": kv["achieved"], "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
            "frac": kv["frac"], "traffic": int(NCU_TRAFFIC_BYTES_PER_ROW * BN),
            "algorithmic_bytes": (BN * C + 2 * C * C + BN * 2 * C) * e,
            "all_linear_launches": {"achieved": round(gemm_flops / (gemm_ms * 1e-3) / 1e12, 1),
                                    "frac": round(gemm_flops / (gemm_ms * 1e-3) / 1e12 / pk["bf16_tflops_sustained"], 3),
                                    "share_of_block": round(gemm_ms / sum(ms), 3)}}
    t_roof = sum(work[r["kernel"]][1] / ((pk["hbm_gbs"] * 1e9) if r["bound"] == "hbm"
                                         else (pk["bf16_tflops_sustained"] * 1e12)) for r in rows
                 if r["kernel"] != "patch_list")
    return rows, roof, {"queries_per_image": L / batch, "block_ms": round(sum(ms), 4),
                        "kernel_weighted_roofline_frac": round(t_roof / (sum(ms) * 1e-3), 3)}


def kv_launch_roofline(model, batch, device, pk, iters=20):
    """The dominant kernel's largest launch on its own: the kv projection (M = batch*N token rows,
    N = 2C, K = C; operands + output exceed L2), `iters` launches back to back between two CUDA
    events on the launch stream.  The per-stage times of `stage_profile` bracket every launch with
    event records, which keeps the next launch from being queued behind the running one."""
    from vtpack_b200 import _lib
    lib = _lib.lib()
    C, N = model.embed_dim, (model.img_size // model.patch_size) ** 2 + 1
    M = batch * N
    gen = torch.Generator(device).manual_seed(9)
    x = torch.randn(M, C, device=device, generator=gen).bfloat16()
    w = (torch.randn(2 * C, C, device=device, generator=gen) * 0.05).bfloat16()
    b = torch.zeros(2 * C, device=device)
    y = torch.empty(M, 2 * C, device=device, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream(device)

    def launch():
        _lib.check(lib.vtp_linear(x.data_ptr(), C, w.data_ptr(), b.data_ptr(), None, 0, y.data_ptr(), 2 * C, 1, M, None,
                                  2 * C, C, 0, stream.cuda_stream))
    for _ in range(5):
        launch()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    e0.record(stream)
    for _ in range(iters):
        launch()
    e1.record(stream)
    torch.cuda.synchronize(device)
    us = e0.elapsed_time(e1) * 1e3 / iters
    flops = 2.0 * M * 2 * C * C
    ach = flops / (us * 1e-6) / 1e12
    return {"kernel": "linear_tc_kernel, kv projection launch (M=batch*N token rows, N=2C, K=C)", "bound": "tensor",
            "achieved": round(ach, 1), "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
            "frac": round(ach / pk["bf16_tflops_sustained"], 3), "traffic": int(NCU_TRAFFIC_BYTES_PER_ROW * M),
            "algorithmic_bytes": (M * C + 2 * C * C + M * 2 * C) * 2, "launch_us": round(us, 2),
            "timing": f"{iters} launches back to back between two CUDA events; 152 MB per launch at batch 256 (> L2)"}


def model_roofline(model, batch, counts, ms_per_step, pk, image_bytes):
    """Sum over the launches of one forward of the time the roofline allows each of them (the larger of
    flops / measured tensor peak and algorithmic bytes / measured copy bandwidth), against the measured step."""
    C, HW = model.embed_dim, (model.img_size // model.patch_size) ** 2
    N, H, e = HW + 1, 4 * model.embed_dim, 2
    BN = batch * N
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops_sustained"] * 1e12

    def gemm(M, Nn, K):
        return max(2.0 * M * Nn * K / tf, (M * K + Nn * K + M * Nn) * e / hbm)
    KP = 3 * model.patch_size ** 2
    t = batch * 3 * model.img_size ** 2 * (image_bytes + e) / hbm + gemm(batch * HW, C, KP) + gemm(batch, 1000, C)
    for i in range(len(model.blocks)):
        L = float(counts[i].sum())
        t += (BN + L) * C * e / hbm + gemm(L, C, C) + gemm(BN, 2 * C, C) + gemm(L, C, C) + gemm(L, H, C) + gemm(L, C, H)
        t += max(4.0 * L * N * C / tf, (2 * L * C + BN * 2 * C) * e / hbm) + (2 * BN + 2 * L) * C * e / hbm
    return {"roofline_ms": round(t * 1e3, 4), "measured_ms": round(ms_per_step, 4), "frac": round(t * 1e3 / ms_per_step, 3),
            "note": "kernel-weighted: sum of per-launch roofline times of one forward / measured ms_per_step"}


def launches_per_forward(model):
    """Kernels of this library in one forward: im2col, cls rows, patch-embed Linear, then per block
    pool, q, kv, attention, proj, fc1, fc2, unpool (LayerNorms are folded into the Linears and the
    unpool leaves the next block's gate decisions), the first block's gate + count + patch-list +
    counts reset, and the final LayerNorm + head.  The fp32 / CUDA-core path runs separate
    LayerNorm and gate kernels per block."""
    depth = len(model.blocks)
    if model.compute_dtype() == torch.bfloat16 and not model.flags:
        return 9 + 8 * depth
    return 5 + 12 * depth


def profile_case(which):
    """A small, self-contained case of one kernel family (three launches) for `ncu`: inputs
    larger than L2 but well under a GB, so a --set full capture ends within a minute or two."""
    import ctypes
    from vtpack_b200 import _lib, synthetic
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if which == "linear_kv":            # the kv projection of DeiT-S at batch 256: M=65792, N=768, K=384
        M, N, K = 65792, 768, 384
        x = torch.randn(M, K, device=dev).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
        b = torch.randn(N, device=dev)
        y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        for _ in range(3):
            _lib.check(lib.vtp_linear(x.data_ptr(), K, w.data_ptr(), b.data_ptr(), None, 0, y.data_ptr(), N, 1, M,
                                      None, N, K, 0, None))
    elif which == "attention":          # 256 images x 6 heads, 114 queries per image, 257 keys
        B, N, h, Li, d = 256, 257, 6, 114, 64
        C, L = h * d, B * Li
        q = torch.randn(L, C, device=dev).bfloat16()
        kv = torch.randn(B, N, 2 * C, device=dev).bfloat16()
        out = torch.empty(L, C, device=dev, dtype=torch.bfloat16)
        off = (torch.arange(B + 1, device=dev) * Li).int()
        for _ in range(3):
            _lib.check(lib.vtp_sparse_attention(q.data_ptr(), C, d, kv.data_ptr(), kv.data_ptr() + C * 2, N * 2 * C,
                                                2 * C, d, out.data_ptr(), C, d, 1, B, N, h, d, off.data_ptr(), L, 257,
                                                d ** -0.5, 0, None))
    elif which == "block":              # one DeiT-S DGE block at batch 256 (gate, pool, GEMMs, attention, unpool)
        model = synthetic.build_model("small", dev, torch.bfloat16, depth=2)
        x = torch.randn(256, 257, 384, device=dev).bfloat16()
        for _ in range(3):
            model.blocks[0](x)
    elif which == "train_ops":          # one launch of each training-path / bilinear kernel at model shapes
        from vtpack_b200 import layers
        B, G, C, heads = 256, 16, 384, 6
        N, d = G * G + 1, C // heads
        gen = torch.Generator(dev).manual_seed(1)
        indices = torch.randint(0, 3, (B, G // 4, G // 4), device=dev, generator=gen)
        patches, lengths = layers.grained_sample_index_to_patch(indices, torch.tensor([4, 2, 1]), 4, 1)
        L = patches.shape[0]
        x = torch.randn(B, N, C, device=dev, generator=gen).bfloat16().requires_grad_(True)
        comp = layers.grained_sample_compress(x, patches, G, G, 1)
        comp.backward(torch.randn(L, C, device=dev, generator=gen).bfloat16())               # pool_grad
        q = torch.randn(L, C, device=dev, generator=gen).bfloat16().requires_grad_(True)
        tok = layers.grained_sample_decompress(q, patches, x.detach(), G, G, 1, True)
        tok.backward(torch.randn(B, N, C, device=dev, generator=gen).bfloat16())             # unpool_grad
        qh = torch.randn(heads, L, d, device=dev, generator=gen).bfloat16()
        kh = torch.randn(heads, B * N, d, device=dev, generator=gen).bfloat16()
        kv_len = torch.full([B], N, dtype=torch.long)
        s_ = layers.batched_sparse_gemm(qh, kh, lengths, kv_len, False, True)                # ragged Q K^T
        layers.batched_sparse_gemm(s_, kh, lengths, kv_len, False, False)                    # ragged P V
        Bb, H, P = 32, 64, 9
        ys, xs = torch.meshgrid(torch.arange(H, device=dev), torch.arange(H, device=dev), indexing="ij")
        centre = torch.stack([xs, ys], dim=-1).reshape(1, H * H, 1, 2).float()
        for mode in ("point", "channel"):
            inp = torch.randn(Bb, H, H, 64, device=dev, generator=gen).bfloat16().requires_grad_(True)
            grid = (centre + 3.0 * torch.randn(Bb, H * H, P, 2, device=dev, generator=gen)).bfloat16().requires_grad_(True)
            wt = torch.randn(Bb, H * H, P if mode == "point" else 64, device=dev, generator=gen).bfloat16()
            wt.requires_grad_(True)
            y = layers.bilinear_attention(inp, grid, wt, mode)
            y.backward(torch.randn_like(y))
    else:
        raise SystemExit(f"unknown profile case {which}")
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def _torch_dense_block(x, blk):
    """The dense DeiT block as the reference runs it (vtpack/models/standard/deit.py:50-83):
    PyTorch ops on the GPU, explicit softmax(q k^T) v."""
    import torch.nn.functional as F
    B, N, C = x.shape
    h = blk.attn.num_heads
    xn = F.layer_norm(x, (C,), blk.norm1.weight, blk.norm1.bias, blk.norm1.eps)
    qkv_w = torch.cat([blk.attn.q.weight, blk.attn.kv.weight], 0)
    qkv_b = torch.cat([blk.attn.q.bias, blk.attn.kv.bias], 0)
    qkv = F.linear(xn, qkv_w, qkv_b).reshape(B, N, 3, h, C // h).permute(2, 0, 3, 1, 4)
    attn = (qkv[0] @ qkv[1].transpose(-2, -1)) * blk.attn.scale
    attn = attn.softmax(dim=-1)
    y = (attn @ qkv[2]).transpose(1, 2).reshape(B, N, C)
    x = x + F.linear(y, blk.attn.proj.weight, blk.attn.proj.bias)
    hdn = F.gelu(F.linear(F.layer_norm(x, (C,), blk.norm2.weight, blk.norm2.bias, blk.norm2.eps),
                          blk.mlp.fc1.weight, blk.mlp.fc1.bias))
    return x + F.linear(hdn, blk.mlp.fc2.weight, blk.mlp.fc2.bias)


def layer_sweep(args):
    """BASELINE config 4: one DeiT-S DGE layer at batch 256, gate logits N(0,1) plus a bias on
    the finest grain chosen by bisection so that the realised fraction of fine regions is
    0 / 0.25 / 0.5 / 1; against the dense block (this library's kernels, and PyTorch ops)."""
    from vtpack_b200 import _lib, synthetic
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    model = synthetic.build_model("small", dev, torch.bfloat16, depth=1)
    blk = model.blocks[0]
    B = args.batch
    x = torch.randn(B, 257, 384, device=dev, generator=torch.Generator(dev).manual_seed(3)).bfloat16()
    base = torch.randn(B, 4, 4, 3, generator=torch.Generator().manual_seed(2))

    def timeit(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3

    rows = []
    for frac in (0.0, 0.25, 0.5, 1.0):
        lo, hi = -50.0, 50.0
        for _ in range(60):                    # bisection on the bias of grain 0
            mid = 0.5 * (lo + hi)
            g = base.clone()
            g[..., 0] += mid
            f = float((g.argmax(-1) == 0).float().mean())
            lo, hi = (mid, hi) if f < frac else (lo, mid)
        g = base.clone()
        g[..., 0] += hi if frac > 0 else -1e4
        gate = g.to(dev)
        us = timeit(lambda: blk(x, forced_gate=gate))
        counts = blk.dge.states["batches_device"].float().mean().item()
        rows.append({"fine_fraction": round(float((g.argmax(-1) == 0).float().mean()), 3),
                     "queries_per_image": round(counts, 1), "dge_layer_us": round(us, 1)})
    dense_us = timeit(lambda: blk(x, dense=True))
    with torch.no_grad():
        torch_us = timeit(lambda: _torch_dense_block(x, blk))
    assert _lib.device_status() == 0
    print(json.dumps({"layer_sweep": rows, "dense_block_us_this_library": round(dense_us, 1),
                      "dense_block_us_pytorch_ops": round(torch_us, 1), "batch": B, "dtype": "bf16",
                      "model": "DeiT-S layer, 16x16 grid, 16 regions"}), flush=True)


def pvt_sweep(args):
    """The four stage shapes of PVT+DGE (small) at 256 px, one block each, bf16, free-running
    random-init gate: microseconds per block on the GPU, the FLOPs the block does and, beside it,
    the CPU oracle on a bounded sample (4 images)."""
    from functools import partial
    from oracle import dge_oracle as O
    from vtpack_b200 import _lib
    from vtpack_b200.models.dge.pvt_dge import Block
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B = args.batch
    torch.set_num_threads(os.cpu_count() or 1)
    rows = []
    for C, heads, H, sr, mr, extra in ((64, 1, 64, 8, 8, 0), (128, 2, 32, 4, 8, 0), (320, 5, 16, 2, 4, 0),
                                       (512, 8, 8, 1, 4, 1)):
        w = O.make_pvt_block_weights(C, mr, sr, seed=7)
        blk = Block(C, heads, mlp_ratio=mr, qkv_bias=True, norm_layer=partial(torch.nn.LayerNorm, eps=1e-6),
                    sr_ratio=sr, split_sizes=[4, 2, 1])
        blk.load_state_dict(w, strict=True)
        blk = blk.eval().to(device=dev, dtype=torch.bfloat16)
        N = H * H + extra
        x = torch.randn(B, N, C, device=dev, generator=torch.Generator(dev).manual_seed(3)).bfloat16()
        for _ in range(3):
            blk(x, H, H)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            blk(x, H, H)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / 20 * 1e3
        L = float(blk.dge.states["batches_device"].float().sum())
        nk = N if sr == 1 else (H // sr) ** 2
        flops = 2.0 * (L * C * C * 2 + B * nk * C * 2 * C + (B * N * C * C if sr > 1 else 0) + 2 * L * nk * C
                       + 2 * L * C * mr * C)
        xc = O.make_tokens(4, N, C, seed=8)
        t0 = time.perf_counter()
        O.dge_block_forward(xc, w, heads, (4, 2, 1), grid=(H, H), sr_ratio=sr)
        cpu_us = (time.perf_counter() - t0) * 1e6 / 4 * B
        rows.append({"stage": f"C={C} heads={heads} grid={H}x{H} sr={sr}", "queries_per_image": round(L / B, 1),
                     "keys": nk, "block_us": round(us, 1), "tflops": round(flops / us / 1e6, 1),
                     "cpu_oracle_us_scaled_to_batch": round(cpu_us)})
    # the whole PVT+DGE tiny model (4 stages, 8 blocks), kernel-by-kernel launches
    from vtpack_b200.models.dge.pvt_dge import pvt_dge_s124_tiny_256
    cfg = O.PVT_CONFIGS["tiny"]
    sd = O.make_pvt_state_dict(cfg, seed=0)
    m = pvt_dge_s124_tiny_256()
    m.load_state_dict(sd, strict=True)
    m = m.eval().to(device=dev, dtype=torch.bfloat16)
    img = torch.randn(B, 3, 256, 256, device=dev, generator=torch.Generator(dev).manual_seed(4))
    for _ in range(3):
        m(img)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        m(img)
    e1.record()
    torch.cuda.synchronize()
    model_ms = e0.elapsed_time(e1) / 10
    xc = O.make_images(4, 256, seed=5)
    t0 = time.perf_counter()
    O.pvt_dge_forward(xc, sd, cfg)
    cpu_rate = 4 / (time.perf_counter() - t0)
    assert _lib.device_status() == 0
    print(json.dumps({"pvt_sweep": rows, "batch": B, "dtype": "bf16",
                      "pvt_tiny_model": {"ms_per_forward": round(model_ms, 3), "images_per_s": round(B / model_ms * 1e3),
                                         "cpu_oracle_images_per_s": round(cpu_rate, 1)}}), flush=True)


def _time_us(fn, iters=20, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def train_ops_sweep(args):
    """The native ops of the training path and the bilinear-sampling ops at model shapes, bf16 unless
    noted: microseconds per call (CUDA events, 20 calls back to back, operands larger than L2 or
    rewritten every call), the algorithmic bytes or FLOPs of a call against the measured peaks, and
    beside the ragged products the reference's formulation (one library bmm per image and a
    concatenation, batched_sparse_gemm.cu:150-196) on the same GPU."""
    from vtpack_b200 import _lib, layers
    from vtpack_b200.runtime import dtype_code, ptr, stream_ptr
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    pk, pk_kind = peaks()
    gen = torch.Generator(dev).manual_seed(1)
    B, G, C, heads = args.batch, 16, 384, 6
    N, d = G * G + 1, C // heads
    rows = []
    # ---- token movers and their gradients (DeiT-S, batch 256, random grains)
    indices = torch.randint(0, 3, (B, G // 4, G // 4), device=dev, generator=gen)
    patches, lengths = layers.grained_sample_index_to_patch(indices, torch.tensor([4, 2, 1]), 4, 1)
    L = patches.shape[0]
    x = torch.randn(B, N, C, device=dev, generator=gen).bfloat16()
    q = torch.randn(L, C, device=dev, generator=gen).bfloat16()
    lib, st, p32 = _lib.lib(), stream_ptr(dev), patches._vtp_i32
    gx, gq = torch.empty_like(x), torch.empty_like(q)
    mover = lambda fn, src, dst: _lib.check(fn(ptr(src), dtype_code(src.dtype), B, N, C, G, 1, ptr(p32), None, L,   # noqa: E731
                                               ptr(dst), st))
    for name, fn, src, dst in (("pool_grad", lib.vtp_pool_grad, q, gx), ("unpool_grad", lib.vtp_unpool_grad, x, gq)):
        us = _time_us(lambda: mover(fn, src, dst))
        nbytes = (B * N + L) * C * 2
        rows.append({"op": name, "shape": f"B={B} N={N} C={C} L={L}", "us": round(us, 1),
                     "GB/s": round(nbytes / us / 1e3), "frac_of_hbm_peak": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)})
    # ---- ragged products of the training-mode attention: S = Q K^T and O = P V
    qh = torch.randn(heads, L, d, device=dev, generator=gen).bfloat16()
    kh = torch.randn(heads, B * N, d, device=dev, generator=gen).bfloat16()
    kv_len = torch.full([B], N, dtype=torch.long)
    prob = torch.randn(heads, L, N, device=dev, generator=gen).bfloat16()
    off = torch.zeros(B + 1, dtype=torch.long)
    off[1:] = torch.cumsum(lengths, 0)
    off = off.tolist()

    def per_image(a, b, tb):
        outs = []
        for i in range(B):
            bi = b[:, i * N:(i + 1) * N]
            outs.append(torch.bmm(a[:, off[i]:off[i + 1]], bi.transpose(-1, -2) if tb else bi))
        return torch.cat(outs, dim=1)

    for name, a, tb in (("ragged Q K^T", qh, True), ("ragged P V", prob, False)):
        us = _time_us(lambda: layers.batched_sparse_gemm(a, kh, lengths, kv_len, False, tb), iters=10)
        us_loop = _time_us(lambda: per_image(a, kh, tb), iters=3, warm=1)
        flops = 2.0 * heads * L * N * d
        rows.append({"op": name, "shape": f"heads={heads} L={L} keys={N} d={d}", "us": round(us, 1),
                     "tflops": round(flops / us / 1e6, 2), "per_image_bmm_loop_us": round(us_loop, 1)})
    # ---- bilinear-sampling attention at a deformable-PVT stage: 64 x 64 map, 64 channels per head
    Bb, H, P = max(1, B // 8), 64, 9
    for mode in ("point", "channel"):
        inp = torch.randn(Bb, H, H, 64, device=dev, generator=gen).bfloat16()
        # one query per pixel looking at P points within a few pixels of itself, as the model's offsets do
        ys, xs = torch.meshgrid(torch.arange(H, device=dev), torch.arange(H, device=dev), indexing="ij")
        centre = torch.stack([xs, ys], dim=-1).reshape(1, H * H, 1, 2).float()
        grid = (centre + 3.0 * torch.randn(Bb, H * H, P, 2, device=dev, generator=gen)).bfloat16()
        weight = torch.randn(Bb, H * H, P if mode == "point" else 64, device=dev, generator=gen).bfloat16()
        grad_out = torch.randn(Bb, H * H, 64 if mode == "point" else P, device=dev, generator=gen).bfloat16()
        a, g_, w = (t.requires_grad_(True) for t in (inp, grid, weight))
        us_f = _time_us(lambda: layers.bilinear_attention(inp, grid, weight, mode))
        y = layers.bilinear_attention(a, g_, w, mode)
        us_b = _time_us(lambda: torch.autograd.grad(y, (a, g_, w), grad_out, retain_graph=True), iters=10)
        taps = Bb * H * H * P * 4 * 64 * 2          # bytes the four corner rows of every point hold
        rows.append({"op": f"bilinear_attention {mode}", "shape": f"B*heads={Bb} map=64x64 C=64 P={P}",
                     "forward_us": round(us_f, 1), "backward_us": round(us_b, 1),
                     "forward_tap_GB/s": round(taps / us_f / 1e3)})
    assert _lib.device_status() == 0
    print(json.dumps({"train_ops_sweep": rows, "dtype": "bf16", "hbm_peak_gbs": pk["hbm_gbs"],
                      "peaks": pk_kind}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="small", choices=["tiny", "small", "base"])
    ap.add_argument("--batch", type=int, default=256, help="images per GPU per step")
    ap.add_argument("--cpu-batch", type=int, default=8, help="images per step of the CPU arm")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--cuda-cores", action="store_true", help="bf16: CUDA-core GEMM/attention instead of tcgen05")
    ap.add_argument("--no-graph", action="store_true", help="launch kernel by kernel instead of replaying a CUDA graph")
    ap.add_argument("--host-image-dtype", default="bf16", choices=["bf16", "f32"],
                    help="element type of the pinned host images of the end-to-end leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-stage-profile", action="store_true")
    ap.add_argument("--profile", default=None, choices=["linear_kv", "attention", "block", "train_ops"],
                    help="run a small case of one kernel family (for ncu) and exit")
    ap.add_argument("--layer-sweep", action="store_true",
                    help="time one DGE layer over gate skew against the dense block and exit")
    ap.add_argument("--pvt-sweep", action="store_true",
                    help="time one PVT+DGE block per stage shape (256 px) and exit")
    ap.add_argument("--train-ops-sweep", action="store_true",
                    help="time the training-path and bilinear-sampling ops at model shapes and exit")
    args = ap.parse_args()
    if args.train_ops_sweep:
        train_ops_sweep(args)
        return
    if args.profile:
        profile_case(args.profile)
        return
    if args.pvt_sweep:
        pvt_sweep(args)
        return
    if args.layer_sweep:
        layer_sweep(args)
        return
    if args.impl == "reference":
        run_reference(args)
        return

    import torch.distributed as dist
    from vtpack_b200 import _lib, parallel, synthetic
    from vtpack_b200.serve import HostPipeline

    rank, world, local = parallel.init_from_env("nccl")
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    _lib.lib()                                       # fails loudly if the CUDA library is missing
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    model = synthetic.build_model(args.model, device, dtype)
    if args.cuda_cores:
        model.flags = _lib.FLAG_CUDA_CORES
    B = args.batch
    img_dev = synthetic.images(B, 256, seed=1 + rank).to(device)          # 201 MB at B=256: larger than L2
    logits = torch.empty(B, 1000, device=device)
    gathered = torch.empty(world * B, 1000, device=device) if world > 1 else None

    use_graph = not args.no_graph

    def step():
        if use_graph:
            model.forward_graph(img_dev, logits)
        else:
            model(img_dev, logits_out=logits)
        if world > 1:
            dist.all_gather_into_tensor(gathered, logits)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms_total = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(ms_total, op=dist.ReduceOp.MAX)
    ms_total = float(ms_total.item())
    value = world * B * args.steps / (ms_total * 1e-3)

    # end to end: pinned host images -> device -> forward -> (gather) -> host logits, copies overlapped
    host_dt = torch.bfloat16 if (args.host_image_dtype == "bf16" and dtype == torch.bfloat16) else torch.float32
    pipe = HostPipeline(model, B, 256, device, world=world, image_dtype=host_dt, use_graph=use_graph)
    host = [synthetic.images(B, 256, seed=100 + rank + 7 * i).to(host_dt).pin_memory() for i in range(2)]
    batches = [host[i & 1] for i in range(args.steps)]
    pipe.run(batches[:max(args.warmup, 3)])
    barrier()
    t0 = time.perf_counter()
    e0.record()
    pipe.run(batches)
    e1.record()
    barrier()
    e2e_ms = torch.tensor([max(e0.elapsed_time(e1), 0.0)], device=device)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = world * B * args.steps / (float(e2e_ms.item()) * 1e-3)
    _ = t0
    clocks = sampler.stop() if sampler else None
    # the same leg with the host images in the other element type (1 GPU only, to keep multi-GPU runs short):
    # fp32 is what the reference's data loader hands over, bf16 is what this model rounds the pixels to anyway
    e2e_other = None
    if world == 1 and dtype == torch.bfloat16:
        other_dt = torch.float32 if host_dt == torch.bfloat16 else torch.bfloat16
        pipe2 = HostPipeline(model, B, 256, device, world=world, image_dtype=other_dt, use_graph=use_graph)
        host2 = [synthetic.images(B, 256, seed=200 + 7 * i).to(other_dt).pin_memory() for i in range(2)]
        batches2 = [host2[i & 1] for i in range(args.steps)]
        pipe2.run(batches2[:3])
        torch.cuda.synchronize(device)
        e0.record()
        pipe2.run(batches2)
        e1.record()
        torch.cuda.synchronize(device)
        e2e_other = {"host_images": str(other_dt).replace("torch.", ""),
                     "value": B * args.steps / (e0.elapsed_time(e1) * 1e-3), "unit": "images/s",
                     "h2d_bytes_per_step": pipe2.h2d_bytes}
    status = _lib.device_status()

    if rank == 0:
        pk, pk_src = peaks()
        line = {
            "metric": "images/sec", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": f"DeiT-{args.model}+DGE s124 (budget 0.5 stand-in: free-running random-init gate) "
                                   f"256px eval forward, batch {B}/GPU, logits all-gathered",
                       "batch_per_gpu": B, "global_batch": B * world, "parallelism": f"dp{world}",
                       "l2": "inputs larger than L2 (fp32 images 201 MB/step at B=256)",
                       "cuda_graph": use_graph, "e2e_host_images": str(host_dt).replace("torch.", "")},
            "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": pipe.h2d_bytes,
                    "d2h_bytes_per_step": pipe.d2h_bytes},
            # per forward: im2col, cls rows, patch-embed GEMM, final LayerNorm, head GEMM, first block's gate,
            # and per block: count, patch list, pool, 5 GEMMs, attention, unpool
            "gpu_launches": args.steps * launches_per_forward(model),
            "clocks": clocks, "device_status": status, "peaks": pk_src,
        }
        if e2e_other:
            line["e2e_other_host_dtype"] = e2e_other
        if dtype == torch.bfloat16 and not args.cuda_cores:
            line["roofline"] = kv_launch_roofline(model, B, device, pk)
            line["model_roofline"] = model_roofline(model, B, model.last_counts.cpu(), ms_total / args.steps, pk,
                                                    img_dev.element_size())
        if not args.no_stage_profile and dtype == torch.bfloat16:
            rows, roof, extra = stage_profile(model, B, device, 10, pk)
            line["roofline"]["all_linear_launches_of_a_block"] = roof["all_linear_launches"]
            line["kernels"] = rows
            line["block"] = extra
        if world == 1 and not args.no_cpu_baseline:
            rate, ms, cores = cpu_reference_rate(args.model, args.cpu_batch, 3, 1)
            line["cpu_baseline"] = {"value": rate, "unit": "images/s", "cores": cores, "kind": "port",
                                    "sample": f"3 forwards of {args.cpu_batch} images after 1 warm-up, fp32 torch CPU"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
