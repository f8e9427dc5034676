#!/usr/bin/env python
"""Throughput benchmark of the DeiT+DGE eval forward (metric: images/sec).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = one forward of `--batch` synthetic 256x256 images per GPU through the whole
model (patch embed, 12 DGE blocks, head) with the logits all-gathered when N > 1.
Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the
reference's eval path on the host cores instead.
"""
import argparse
import ctypes
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
NCU_TRAFFIC_BYTES_PER_ROW = (51173888 + 43880448) / 65792


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


def alternate_gate_bias(batch, n_splits=3, big=1e4):
    """The 512-pixel measurement configuration's gate skew: even images forced all-coarse (the last split, 1x1), odd images
    all-fine (the first split, 4x4), as a per-image offset of the router logits."""
    bias = torch.zeros(batch, n_splits)
    bias[0::2, n_splits - 1] = big
    bias[1::2, 0] = big
    return bias


def cpu_reference_rate(model_kind, batch, steps, warmup, img_size=256, gate_skew="none"):
    """images/sec of the CPU restatement of the reference's eval forward (fp32, all host cores)."""
    from oracle import dge_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = O.MODEL_CONFIGS[model_kind]
    sd = O.make_state_dict(cfg["embed_dim"], cfg["depth"], cfg["num_heads"], img_size=img_size, seed=0)
    img = O.make_images(batch, img_size, seed=1)
    bias = alternate_gate_bias(batch) if gate_skew == "alternate" else None
    with torch.no_grad():
        for _ in range(warmup):
            O.deit_dge_forward(img, sd, cfg["depth"], cfg["num_heads"], (4, 2, 1), gate_image_bias=bias)
        t0 = time.perf_counter()
        for _ in range(steps):
            O.deit_dge_forward(img, sd, cfg["depth"], cfg["num_heads"], (4, 2, 1), gate_image_bias=bias)
        dt = time.perf_counter() - t0
    return batch * steps / dt, dt / steps * 1e3, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    b = args.cpu_batch
    rate, ms, cores = cpu_reference_rate(args.model, b, args.steps, args.warmup, args.img_size, args.gate_skew)
    line = {
        "impl": "reference", "metric": "images/sec", "value": rate, "unit": "images/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"DeiT-{args.model}+DGE s124 {args.img_size}px eval forward, CPU, fp32"
                               + (", even images all-coarse / odd all-fine" if args.gate_skew == "alternate" else ""),
                   "batch_per_step": b},
        "cpu_baseline": {"value": rate, "unit": "images/s", "cores": cores, "kind": "port",
                         "sample": f"{args.steps} forwards of {b} images (same model/config), torch CPU fp32"},
        "e2e": {"value": rate, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def region_grains(x, gate_w, gate_b, G, device):
    """Grain index per region of tokens x [B, 1+G*G, C] under a router gate (the library's stand-alone gate kernel)."""
    from vtpack_b200 import _lib
    B, _, C = x.shape
    idx = torch.empty(B * (G // 4) ** 2, dtype=torch.int32, device=device)
    _lib.check(_lib.lib().vtp_router_gate(x.data_ptr(), 1 if x.dtype == torch.bfloat16 else 0, B, G, G, C, 1, 4,
                                          gate_w.data_ptr(), gate_b.data_ptr(), 3, None, idx.data_ptr(),
                                          torch.cuda.current_stream(device).cuda_stream))
    return idx


def unpool_rows(B, HW, L, fine):
    """Token-row transfers of the unpool + residual kernel: it writes every token row and reads every packed row
    of q; a region at the finest grain needs nothing else (its comp rows are copies of its tokens, so
    ref + (q - comp) = q), the other regions and the cls row also read their token rows and their comp rows."""
    N = HW + 1
    return B * N + L + (B * (1.0 - fine) * HW + B) + (L - fine * B * HW)


def front_back_ms(model, batch, device, image_bytes, iters=10):
    """The launches of a forward outside the blocks (im2col + cls rows, patch-embedding Linear, final LayerNorm
    of the cls rows, head), each timed as `iters` back-to-back launches through the C ABI."""
    from vtpack_b200 import _lib
    lib = _lib.lib()
    C, S, P = model.embed_dim, model.img_size, model.patch_size
    HW = (S // P) ** 2
    dtype = model.compute_dtype()
    t = model._pack.tensors
    img = torch.randn(batch, 3, S, S, device=device, dtype=torch.float32 if image_bytes == 4 else torch.bfloat16)
    cols = torch.empty(batch * HW, 3 * P * P, device=device, dtype=dtype)
    x = torch.empty(batch, HW + 1, C, device=device, dtype=dtype)
    cls_n = torch.empty(batch, C, device=device, dtype=dtype)
    logits = torch.empty(batch, 1000, device=device)
    st = torch.cuda.current_stream(device).cuda_stream
    code = 1 if dtype == torch.bfloat16 else 0
    calls = [
        lambda: lib.vtp_patch_im2col(img.data_ptr(), 0 if image_bytes == 4 else 1, batch, S, P, code, cols.data_ptr(),
                                     t["cls_token"].data_ptr(), t["pos_embed"].data_ptr(), C, x.data_ptr(), st),
        lambda: lib.vtp_linear(cols.data_ptr(), 3 * P * P, t["patch_w"].data_ptr(), t["patch_b"].data_ptr(),
                               x.data_ptr(), C, x.data_ptr(), C, code, batch * HW, None, C, 3 * P * P, 0, st),
        lambda: lib.vtp_layernorm(x.data_ptr(), code, batch, None, C, (HW + 1) * C, t["norm_w"].data_ptr(),
                                  t["norm_b"].data_ptr(), 1e-6, cls_n.data_ptr(), st),
        lambda: lib.vtp_linear(cls_n.data_ptr(), C, t["head_w"].data_ptr(), t["head_b"].data_ptr(), None, 0,
                               logits.data_ptr(), 1000, code, batch, None, 1000, C, _lib.FLAG_OUT_F32, st),
    ]
    total = 0.0
    for fn in calls:
        total += _time_us(lambda: _lib.check(fn()), iters=iters) * 1e-3
    return total


def stage_profile(model, batch, device, iters, pk, ms_per_step, tokens=None, forced=None):
    """Per-kernel times of one DGE block (the middle block's weights, on the tokens that block received in the
    model's own forward when `tokens` is given, else on N(0,1) tokens), from events the library records
    between its launches.  Every stage then sits between two event records, which keeps a launch from
    queueing behind the one in front of it: these are upper bounds of what a kernel costs inside the replayed
    graph.  `ms_in_step_est` scales them so that depth x block + the front/back launches equals the measured
    step.  Returns (rows, the five Linear launches together, block summary)."""
    import ctypes
    from vtpack_b200 import _lib
    from vtpack_b200.models.dge.deit_dge import _pack_block
    from vtpack_b200.runtime import scratch
    blk = model.blocks[len(model.blocks) // 2]
    G = model.img_size // model.patch_size
    C, N = model.embed_dim, G * G + 1
    dtype = model.compute_dtype()
    e = 2 if dtype == torch.bfloat16 else 4
    if tokens is not None:
        x = tokens.contiguous()
    else:
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
                                                   forced.data_ptr() if forced is not None else None,
                                                   counts.data_ptr(), ws.data_ptr(), nbytes, arr, n_ev,
                                                   stream.cuda_stream))
    torch.cuda.synchronize(device)
    L = int(counts.sum().item())
    if forced is not None:
        fine = float((forced.argmax(-1) == 0).float().mean().item())
    else:
        grains = region_grains(x, blk._pack.tensors["gate_w"], blk._pack.tensors["gate_b"], G, device)
        fine = float((grains == 0).float().mean().item())
    ms = [sum(evs[i][j].elapsed_time(evs[i][j + 1]) for i in range(iters)) / iters for j in range(len(STAGES))]
    BN, H, HW = batch * N, 4 * C, G * G
    work = {   # (kind, algorithmic bytes or flops)
        # LayerNorm is folded into the GEMM epilogues on the bf16 path: the pool writes comp rows
        # and 8 bytes of statistics per row; there is no LN2 kernel (its slot measures ~0)
        "router_gate": ("hbm", batch * (N - 1) * C * e), "patch_list": ("hbm", batch * 16 * 12),
        "pool_ln1": ("hbm", (BN + L) * C * e + (BN + 2 * L) * 8), "q_proj": ("tensor", 2 * L * C * C),
        "kv_proj": ("tensor", 4 * BN * C * C), "attention": ("tensor", 4 * L * N * C),
        "out_proj": ("tensor", 2 * L * C * C), "ln2": ("hbm", 0),
        "fc1_gelu": ("tensor", 2 * L * C * H), "fc2": ("tensor", 2 * L * C * H),
        "unpool_add": ("hbm", unpool_rows(batch, HW, L, fine) * C * e),
    }
    depth = len(model.blocks)
    fb_ms = front_back_ms(model, batch, device, 4)
    # inside a model forward the gate and the patch list of blocks 2.. come out of the previous block's unpool
    in_model = [t for name, t in zip(STAGES, ms) if name not in ("router_gate", "patch_list")]
    scale = max(ms_per_step - fb_ms, 0.0) / (depth * sum(in_model))
    rows = []
    for name, t in zip(STAGES, ms):
        kind, amount = work[name]
        if amount == 0:
            continue
        t_est = t * scale
        if kind == "hbm":
            ach, peak, unit = amount / (t_est * 1e-3) / 1e9, pk["hbm_gbs"], "GB/s"
        else:
            ach, peak, unit = amount / (t_est * 1e-3) / 1e12, pk["bf16_tflops_sustained"], "TFLOP/s"
        row = {"kernel": name, "ms_event_bracketed": round(t, 4), "ms_in_step_est": round(t_est, 4), "bound": kind,
               "achieved_in_step_est": round(ach, 1), "unit": unit, "frac_in_step_est": round(ach / peak, 3)}
        if name in ("router_gate", "patch_list"):
            row["note"] = "first block of a forward only"
        rows.append(row)
    gemm = [r for r in rows if r["kernel"] in ("q_proj", "kv_proj", "out_proj", "fc1_gelu", "fc2")]
    gemm_ms = sum(r["ms_event_bracketed"] for r in gemm)
    gemm_flops = sum(work[r["kernel"]][1] for r in gemm)
    tf_bracketed = gemm_flops / (gemm_ms * 1e-3) / 1e12
    tf_step = gemm_flops / (gemm_ms * scale * 1e-3) / 1e12
    all_linear = {"launches": "q, kv, out, fc1, fc2 projections of one block", "gflop": round(gemm_flops / 1e9, 1),
                  "achieved_event_bracketed": round(tf_bracketed, 1),
                  "frac_event_bracketed": round(tf_bracketed / pk["bf16_tflops_sustained"], 3),
                  "achieved_in_step_est": round(tf_step, 1),
                  "frac_in_step_est": round(tf_step / pk["bf16_tflops_sustained"], 3),
                  "peak": pk["bf16_tflops_sustained"], "peak_kind": "sustained cuBLAS bf16 (kernels timed inside a long step)",
                  "share_of_block": round(gemm_ms / sum(in_model), 3)}
    return rows, all_linear, {"queries_per_image": L / batch, "fine_region_fraction": round(fine, 3),
                              "block_ms_event_bracketed": round(sum(in_model), 4),
                              "block_ms_in_step_est": round(sum(in_model) * scale, 4),
                              "front_back_ms": round(fb_ms, 4), "depth": depth,
                              "check": "depth * block_ms_in_step_est + front_back_ms = ms_per_step"}


def kv_launch_roofline(model, batch, device, pk, iters=20):
    """The dominant kernel's largest launch on its own: the kv projection (M = batch*N token rows,
    N = 2C, K = C; operands + output exceed L2), `iters` launches back to back between two CUDA
    events on the launch stream.  A launch timed on its own is read against the burst cuBLAS figure."""
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
            "achieved": round(ach, 1), "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
            "frac": round(ach / pk["bf16_tflops"], 3), "peak_kind": "burst cuBLAS bf16 (launch timed on its own)",
            "frac_of_sustained_peak": round(ach / pk["bf16_tflops_sustained"], 3),
            "traffic": int(NCU_TRAFFIC_BYTES_PER_ROW * M),
            "traffic_note": "constant: dram read + write bytes of one launch from the committed ncu capture "
                            "(profiles/), scaled by the row count; not measured in this run",
            "algorithmic_bytes": (M * C + 2 * C * C + M * 2 * C) * 2, "launch_us": round(us, 2),
            "timing": f"{iters} launches back to back between two CUDA events; "
                      f"{(M * C + M * 2 * C) * 2 / 1e6:.0f} MB per launch (> L2)"}


def traced_forward(model, img_dev):
    """One launch-by-launch forward with the traces on: the fraction of regions at the finest grain in each
    block, and the tokens the middle block received (the input of the per-kernel profile)."""
    keep = model.trace
    model.trace = True
    model(img_dev)
    torch.cuda.synchronize(img_dev.device)
    f = (model.last_grains == 0).float().mean(dim=(1, 2)).cpu().tolist()
    mid = model.last_tokens[len(model.blocks) // 2].clone()
    model.trace = keep
    model.last_grains = model.last_tokens = None
    return f, mid


def model_roofline(model, batch, counts, ms_per_step, pk, image_bytes, fine):
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
        t += max(4.0 * L * N * C / tf, (2 * L * C + BN * 2 * C) * e / hbm) + unpool_rows(batch, HW, L, fine[i]) * C * e / hbm
    return {"roofline_ms": round(t * 1e3, 4), "measured_ms": round(ms_per_step, 4), "frac": round(t * 1e3 / ms_per_step, 3),
            "fine_region_fraction": round(sum(fine) / len(fine), 3),
            "note": "kernel-weighted: sum of per-launch roofline times of one forward / measured ms_per_step; "
                    "unpool bytes are what the kernel moves (fine regions read neither ref nor comp)"}


def launches_per_forward(model):
    """Kernels of this library in one forward: im2col, cls rows, patch-embed Linear, then per block
    pool, q, kv, attention, proj, fc1, fc2, unpool (LayerNorms are folded into the Linears and the
    unpool leaves the next block's gate decisions), the first block's gate + count + patch-list +
    counts reset, and the final LayerNorm + head.  The fp32 / CUDA-core path runs separate
    LayerNorm and gate kernels per block."""
    depth = len(model.blocks)
    if model.compute_dtype() == torch.bfloat16 and not model.flags:
        C = model.embed_dim
        # the q and kv projections share one launch when both widths are whole 64-column slabs
        paired = C >= 64 and C % 64 == 0
        return 9 + (7 if paired else 8) * depth
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
    elif which == "pvt_stage1":         # one stage-1 PVT+DGE block (C=64, 64x64 grid, reduction 8, hidden 512) at batch 32
        from functools import partial
        from vtpack_b200.models.dge.pvt_dge import Block
        torch.manual_seed(7)                # the modules' own random initialisation
        blk = Block(64, 1, mlp_ratio=8, qkv_bias=True, norm_layer=partial(torch.nn.LayerNorm, eps=1e-6), sr_ratio=8,
                    split_sizes=[4, 2, 1])
        blk = blk.eval().to(device=dev, dtype=torch.bfloat16)
        x = torch.randn(32, 64 * 64, 64, device=dev, generator=torch.Generator(dev).manual_seed(3)).bfloat16()
        for _ in range(2):
            blk(x, 64, 64)
        print("queries per image:", float(blk.dge.states["batches_device"].float().mean()))
    elif which == "pvt_model":          # three launch-by-launch eval forwards of PVT+DGE tiny at batch 256 (bf16)
        from vtpack_b200.models.dge.pvt_dge import pvt_dge_s124_tiny_256
        torch.manual_seed(0)                # the modules' own random initialisation
        m = pvt_dge_s124_tiny_256().eval().to(device=dev, dtype=torch.bfloat16)
        img = torch.randn(256, 3, 256, 256, device=dev, generator=torch.Generator(dev).manual_seed(4))
        for _ in range(3):
            m(img)
        print("queries per image and block:", [round(float(c.float().mean()), 1) for c in m.last_counts])
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
    """The layer-level configuration: one DeiT-S DGE layer at batch 256, gate logits N(0,1) plus a bias on
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


def pvt_model_roofline_ms(B, counts, pk):
    """Sum over the launches of one PVT+DGE tiny forward (256 px, bf16) of max(FLOPs / sustained tensor peak,
    algorithmic bytes / copy bandwidth), in ms.  `counts`: per block, the per-image query counts the forward
    left.  Bytes are each kernel's operands read or written once (the unpool as the reference defines it: token
    map in and out, packed rows and their pooled copies in); the stage embeddings count their im2col, GEMM,
    LayerNorm and position-embedding passes."""
    e = 2.0
    tf, bw = pk["bf16_tflops_sustained"] * 1e12, pk["hbm_gbs"] * 1e9
    t = lambda fl, by: max(fl / tf, by / bw)                  # noqa: E731
    total, blk = 0.0, 0
    cin, side = 3, 256
    for C, heads, H, sr, mr, extra, depth, P in ((64, 1, 64, 8, 8, 0, 2, 4), (128, 2, 32, 4, 8, 0, 2, 2),
                                                  (320, 5, 16, 2, 4, 0, 2, 2), (512, 8, 8, 1, 4, 1, 2, 2)):
        N = H * H + extra
        rows, krows = B * N, B * (N if sr == 1 else (H // sr) ** 2)
        in_bytes = B * cin * side * side * (4.0 if cin == 3 else e)
        K = cin * P * P
        total += t(0, in_bytes + B * H * H * K * e)                        # im2col
        total += t(2.0 * B * H * H * K * C, B * H * H * (K + C) * e)        # embedding GEMM
        total += 2 * t(0, 2 * rows * C * e)                                # its LayerNorm, position rows
        for j in range(depth):
            L = float(counts[blk].float().sum())
            blk += 1
            hid = mr * C
            if j == 0:
                total += t(0, rows * C * e)                                # gate + token statistics
            total += t(0, (rows + L) * C * e)                              # pool
            total += t(2 * L * C * C, 2 * L * C * e)                       # q
            if sr > 1:
                total += t(0, 2 * rows * C * e)                            # im2col of the reduction
                total += t(2.0 * krows * C * sr * sr * C, (rows + krows) * C * e)
                total += t(0, 2 * krows * C * e)                           # its LayerNorm
            total += t(2.0 * krows * 2 * C * C, krows * 3 * C * e)          # kv
            total += t(4.0 * L * (krows / B) * C, (2 * L * C + krows * 2 * C) * e)   # attention
            total += t(2 * L * C * C, 3 * L * C * e)                       # out projection + residual
            total += t(2 * L * C * hid, L * (C + hid) * e)                 # fc1
            total += t(2 * L * hid * C, L * (hid + 2 * C) * e)             # fc2 + residual
            total += t(0, (2 * rows + 2 * L) * C * e)                      # unpool
        cin, side = C, H
    total += t(2.0 * B * 512 * 1000, B * 1000 * 4.0)                       # head
    return total * 1e3


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
    # the same forward replayed as one CUDA graph (no host work between its ~60 launches)
    for _ in range(3):
        m.forward_graph(img)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(20):
        m.forward_graph(img)
    e1.record()
    torch.cuda.synchronize()
    graph_ms = e0.elapsed_time(e1) / 20
    diff = float((m.forward_graph(img) - m(img)).abs().max())
    xc = O.make_images(4, 256, seed=5)
    t0 = time.perf_counter()
    O.pvt_dge_forward(xc, sd, cfg)
    cpu_rate = 4 / (time.perf_counter() - t0)
    assert _lib.device_status() == 0
    pk, pk_kind = peaks()
    roof_ms = pvt_model_roofline_ms(B, m.last_counts, pk)
    print(json.dumps({"pvt_sweep": rows, "batch": B, "dtype": "bf16",
                      "pvt_tiny_model": {"ms_per_forward": round(model_ms, 3), "images_per_s": round(B / model_ms * 1e3),
                                         "ms_per_forward_graph": round(graph_ms, 3),
                                         "images_per_s_graph": round(B / graph_ms * 1e3),
                                         "graph_vs_launch_by_launch_max_abs_diff": diff,
                                         "cpu_oracle_images_per_s": round(cpu_rate, 1),
                                         "model_roofline": {"roofline_ms": round(roof_ms, 4), "measured_ms": round(graph_ms, 4),
                                                            "frac": round(roof_ms / graph_ms, 3), "peaks": pk_kind,
                                                            "note": "kernel-weighted: sum over the launches of one forward "
                                                                    "of max(FLOPs / sustained cuBLAS bf16 peak, algorithmic "
                                                                    "bytes / copy bandwidth) over the graph-replayed forward"}}}),
          flush=True)


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
    # the region-parallel form of unpool_grad (what the autograd function calls for a list made from grain indices)
    idx32, first, splits_l, region_size, Hr, Wr, _ = patches._vtp_regions
    arr = (ctypes.c_int * len(splits_l))(*splits_l)
    us = _time_us(lambda: _lib.check(lib.vtp_unpool_grad_regions(
        ptr(x), dtype_code(x.dtype), B, Hr, Wr, region_size, C, 1, ptr(idx32), arr, len(splits_l), ptr(first),
        ptr(patches._vtp_offsets), L, ptr(gq), st)))
    nbytes = (B * N + L) * C * 2
    rows.append({"op": "unpool_grad (regions)", "shape": f"B={B} N={N} C={C} L={L}", "us": round(us, 1),
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

    a_off = torch.tensor(off, dtype=torch.int32, device=dev)
    b_off = (torch.arange(B + 1, dtype=torch.int32) * N).to(dev)
    a_max = int(lengths.max())
    for name, a, tb in (("ragged Q K^T", qh, True), ("ragged P V", prob, False)):
        out_cols = N if tb else d
        out = torch.empty(heads, L, out_cols, dtype=torch.bfloat16, device=dev)
        # the launch itself (offsets already on the device), then the call a training step makes (the autograd
        # function: two host-side prefix sums and their copies, the output allocation, then the same launch)
        us = _time_us(lambda: _lib.check(lib.vtp_batched_sparse_gemm(
            ptr(a), ptr(kh), ptr(out), dtype_code(a.dtype), heads, B, a.shape[1], a.shape[2], kh.shape[1], d,
            ptr(a_off), ptr(b_off), a_max, N, 0, int(tb), L, out_cols, st)))
        us_call = _time_us(lambda: layers.batched_sparse_gemm(a, kh, lengths, kv_len, False, tb), iters=10)
        us_loop = _time_us(lambda: per_image(a, kh, tb), iters=3, warm=1)
        flops = 2.0 * heads * L * N * d
        nbytes = (a.numel() + kh.numel() + out.numel()) * 2
        rows.append({"op": name, "shape": f"heads={heads} L={L} keys={N} d={d}", "us": round(us, 1),
                     "tflops": round(flops / us / 1e6, 2), "GB/s": round(nbytes / us / 1e3),
                     "frac_of_hbm_peak": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3),
                     "us_through_autograd_function": round(us_call, 1), "per_image_bmm_loop_us": round(us_loop, 1)})
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


def h2d_rate_gbs(nbytes, device, world, iters=5):
    """GB/s of a pinned host-to-device copy of one step's images, every rank copying at the same time
    (max time over ranks): what the end-to-end leg's input traffic can reach on this host."""
    import torch.distributed as dist
    src = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    dst = torch.empty(nbytes, dtype=torch.uint8, device=device)
    dst.copy_(src, non_blocking=True)
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        dst.copy_(src, non_blocking=True)
    e1.record()
    torch.cuda.synchronize(device)
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return nbytes / (float(ms.item()) * 1e-3) / 1e9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="small", choices=["tiny", "small", "base", "pvt_tiny"],
                    help="DeiT+DGE size; pvt_tiny runs the PVT+DGE sweep and whole-model timing (same as --pvt-sweep)")
    ap.add_argument("--batch", type=int, default=256, help="images per GPU per step")
    ap.add_argument("--img-size", type=int, default=256, help="input side in pixels (512: 32x32 tokens, 64 regions)")
    ap.add_argument("--gate-skew", default="none", choices=["none", "alternate"],
                    help="alternate: even images forced all-coarse, odd all-fine (per-image gate bias of 1e4)")
    ap.add_argument("--cpu-batch", type=int, default=8, help="images per step of the CPU arm")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--cuda-cores", action="store_true", help="bf16: CUDA-core GEMM/attention instead of tcgen05")
    ap.add_argument("--no-graph", action="store_true", help="launch kernel by kernel instead of replaying a CUDA graph")
    ap.add_argument("--host-image-dtype", default="f32", choices=["bf16", "f32"],
                    help="element type of the pinned host images of the end-to-end leg (f32: what the reference's "
                         "data loader hands over)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-stage-profile", action="store_true")
    ap.add_argument("--profile", default=None, choices=["linear_kv", "attention", "block", "train_ops", "pvt_stage1", "pvt_model"],
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
    if args.pvt_sweep or args.model == "pvt_tiny":
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
    from vtpack_b200.serve import HostPipeline, LogitsGather

    rank, world, local = parallel.init_from_env("nccl")
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    _lib.lib()                                       # fails loudly if the CUDA library is missing
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    S = args.img_size
    model = synthetic.build_model(args.model, device, dtype, img_size=S)
    if args.cuda_cores:
        model.flags = _lib.FLAG_CUDA_CORES
    B = args.batch
    if args.gate_skew == "alternate":
        model.gate_image_bias = alternate_gate_bias(B).to(device)
    img_dev = synthetic.images(B, S, seed=1 + rank).to(device)          # 201 MB at B=256, 256 px: larger than L2
    # the logits leave on a side stream (all-gather when there are several ranks), double-buffered, so the
    # collective of step i runs under the forward of step i+1
    out = LogitsGather(B, 1000, device, world=world)

    use_graph = not args.no_graph
    step_no = [0]

    def step():
        slot = step_no[0] & 1
        step_no[0] += 1
        out.reusable(slot)
        if use_graph:
            model.forward_graph(img_dev, out.local[slot])
        else:
            model(img_dev, logits_out=out.local[slot])
        if world > 1:
            out.start(slot)

    def barrier():
        out.wait_all()
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
    out.wait_all()                                   # the last gathers are inside the timed region
    e1.record()
    barrier()
    ms_rank = e0.elapsed_time(e1)
    ms_all = torch.tensor([ms_rank], device=device)
    ms_min = ms_all.clone()
    if world > 1:
        dist.all_reduce(ms_all, op=dist.ReduceOp.MAX)
        dist.all_reduce(ms_min, op=dist.ReduceOp.MIN)
    ms_total = float(ms_all.item())
    value = world * B * args.steps / (ms_total * 1e-3)
    counts_cpu = model.last_counts.cpu()

    # end to end: pinned host images -> device -> forward -> (gather) -> host logits, copies overlapped
    host_dt = torch.bfloat16 if (args.host_image_dtype == "bf16" and dtype == torch.bfloat16) else torch.float32
    pipe = HostPipeline(model, B, S, device, world=world, image_dtype=host_dt, use_graph=use_graph)
    host = [synthetic.images(B, S, seed=100 + rank + 7 * i).to(host_dt).pin_memory() for i in range(2)]
    batches = [host[i & 1] for i in range(args.steps)]
    pipe.run(batches[:max(args.warmup, 3)])
    barrier()
    e0.record()
    pipe.run(batches)
    e1.record()
    barrier()
    e2e_ms = torch.tensor([max(e0.elapsed_time(e1), 0.0)], device=device)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = world * B * args.steps / (float(e2e_ms.item()) * 1e-3)
    clocks = sampler.stop() if sampler else None
    h2d_gbs = h2d_rate_gbs(pipe.h2d_bytes, device, world)
    # the same leg with the host images in the other element type (1 GPU only, to keep multi-GPU runs short):
    # fp32 is what the reference's data loader hands over, bf16 is what this model rounds the pixels to anyway
    e2e_other = None
    if world == 1 and dtype == torch.bfloat16:
        other_dt = torch.float32 if host_dt == torch.bfloat16 else torch.bfloat16
        del pipe
        pipe2 = HostPipeline(model, B, S, device, world=world, image_dtype=other_dt, use_graph=use_graph)
        host2 = [synthetic.images(B, S, seed=200 + 7 * i).to(other_dt).pin_memory() for i in range(2)]
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
        h2d_bytes, d2h_bytes = B * 3 * S * S * host[0].element_size(), B * 1000 * 4
    else:
        h2d_bytes, d2h_bytes = pipe.h2d_bytes, pipe.d2h_bytes
    status = _lib.device_status()

    if rank == 0:
        pk, pk_src = peaks()
        skew = ", even images all-coarse / odd all-fine" if args.gate_skew == "alternate" else \
            " (budget 0.5 stand-in: free-running random-init gate)"
        line = {
            "metric": "images/sec", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": f"DeiT-{args.model}+DGE s124{skew} {S}px eval forward, batch {B}/GPU, "
                                   f"logits all-gathered",
                       "batch_per_gpu": B, "global_batch": B * world, "parallelism": f"dp{world}",
                       "img_size": S, "gate_skew": args.gate_skew,
                       "queries_per_image": round(float(counts_cpu.float().mean()), 1),
                       "l2": f"inputs larger than L2 (fp32 images {B * 3 * S * S * 4 / 1e6:.0f} MB/step)",
                       "cuda_graph": use_graph, "e2e_host_images": str(host_dt).replace("torch.", ""),
                       "logits_gather": "side stream, double-buffered" if world > 1 else "single rank: none"},
            "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes,
                    "h2d_copy_alone_gbs_per_gpu": round(h2d_gbs, 1),
                    "h2d_note": "pinned-host-to-device copy of one step's images with nothing else running, all "
                                "ranks at once, max over ranks"},
            # per forward: im2col, cls rows, patch-embed GEMM, final LayerNorm, head GEMM, first block's gate,
            # and per block: count, patch list, pool, 5 GEMMs, attention, unpool
            "gpu_launches": args.steps * launches_per_forward(model),
            "clocks": clocks, "device_status": status, "peaks": pk_src,
            "rank_step_ms": {"max": ms_total / args.steps, "min": float(ms_min.item()) / args.steps},
        }
        if e2e_other:
            line["e2e_other_host_dtype"] = e2e_other
        mid_tokens = None
        if dtype == torch.bfloat16 and not args.cuda_cores:
            fine, mid_tokens = traced_forward(model, img_dev)
            line["roofline"] = kv_launch_roofline(model, B, device, pk)
            line["model_roofline"] = model_roofline(model, B, counts_cpu, ms_total / args.steps, pk,
                                                    img_dev.element_size(), fine)
        if not args.no_stage_profile and dtype == torch.bfloat16 and not args.cuda_cores:
            forced = None
            if model.gate_image_bias is not None:     # the block entry point takes forced logits, not a per-image bias
                R = (S // 16) // 4
                forced = model.gate_image_bias[:, None, None, :].expand(B, R, R, 3).contiguous()
            rows, all_linear, extra = stage_profile(model, B, device, 10, pk, ms_total / args.steps, mid_tokens, forced)
            line["roofline"]["all_linear_launches_of_a_block"] = all_linear
            line["roofline"]["frac_all_launches"] = all_linear["frac_in_step_est"]
            line["kernels"] = rows
            line["kernels_note"] = ("one block (the middle one's weights and the tokens it received in this forward), "
                                    "q and kv projections as separate launches (the forward pairs them in one); "
                                    "ms_event_bracketed: every stage sits between two event records, which keeps the "
                                    "next launch from queueing behind the running one: an upper bound. ms_in_step_est "
                                    "= that share scaled so that depth x block + front/back equals ms_per_step")
            line["block"] = extra
        if world == 1 and not args.no_cpu_baseline:
            rate, ms, cores = cpu_reference_rate(args.model, args.cpu_batch, 3, 1, S, args.gate_skew)
            line["cpu_baseline"] = {"value": rate, "unit": "images/s", "cores": cores, "kind": "port",
                                    "sample": f"3 forwards of {args.cpu_batch} images after 1 warm-up, fp32 torch CPU"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
