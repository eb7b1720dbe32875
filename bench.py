"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemv] [--impl reference]

Workload `gemv` (default): the Q8_0 decode mat-vec sweep over Llama-3-8B layer shapes
(4096->4096, 4096->14336, 14336->4096, 4096->128256) with M in {1, 2, 4, 8} bf16 activation rows.
One step = one pass over all 16 (shape, M) launches; a "token" is one activation row carried through
the four linears, so a step processes 15 tokens.  Weights are synthetic N(0, 0.02^2) quantized to Q8_0,
activations N(0, 1) in bf16.  Every launch reads a weight copy that was last touched at least one
full step (> 700 MB) earlier, so nothing is served from L2.

One JSON line is printed by rank 0.  `value` is timed with inputs resident in HBM (CUDA-graph replay
of the step, CUDA events); `e2e` times the same step through the public API with pinned host buffers
(host->device copy of every activation, device->host copy of every result inside the timed region);
`roofline` gives the mat-vec kernel's algorithmic bytes over its event-timed duration against the
measured HBM copy peak; `cpu_baseline` is the C oracle on the host cores.
`--impl reference` times the CPU restatement of the reference path alone (rank 0 only).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096), (4096, 128256)]   # (K, N)
MS = [1, 2, 4, 8]
METRIC = "quant_linear_decode_tokens_per_s"
UNIT = "tokens/s"


NCU_TRAFFIC_RATIO = 563.3 / 558.2   # measured DRAM traffic over algorithmic bytes, decode kernel


def algorithmic_bytes(k, n, m, x_size=2, y_size=4):
    return n * (k // 32) * 34 + m * k * x_size + m * n * y_size


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read-only query)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])), mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_q8_0_on_device(torch, n, k, gen, device):
    """N(0, 0.02^2) weights quantized to GGUF Q8_0 blocks on the device (benchmark data only; the byte format
    is the one tests/ checks against the oracle): d = absmax/127 (fp16), q = round(x/d)."""
    out = torch.empty((n, k // 32, 34), dtype=torch.uint8, device=device)
    rows_per = max(1, (1 << 26) // k)
    for r0 in range(0, n, rows_per):
        r1 = min(n, r0 + rows_per)
        w = torch.randn((r1 - r0, k // 32, 32), generator=gen, device=device, dtype=torch.float32) * 0.02
        d = w.abs().amax(dim=2, keepdim=True) / 127.0
        q = torch.round(w / torch.where(d > 0, d, torch.ones_like(d))).clamp(-127, 127).to(torch.int8)
        out[r0:r1, :, 0:2] = d.to(torch.float16).view(torch.uint8).reshape(r1 - r0, k // 32, 2)
        out[r0:r1, :, 2:] = q.view(torch.uint8)
    return out.reshape(n, -1)


def cpu_reference_step(threads, sample_shapes, weights_host, xs_host):
    """One pass of the sampled (shape, M) list through the C oracle; returns seconds."""
    from oracle import cbuild
    t0 = time.perf_counter()
    for (k, n) in sample_shapes:
        for m in MS:
            cbuild.linear("Q8_0", weights_host[(k, n)], None, None, xs_host[(k, m)], threads)
    return time.perf_counter() - t0


def host_weights_for_cpu(shapes):
    import numpy as np
    from oracle import formats as F
    rng = np.random.Generator(np.random.PCG64(2002))
    ws, xs = {}, {}
    for (k, n) in shapes:
        # block bytes for the CPU leg: random valid Q8_0 blocks (d = small positive fp16, random int8 codes)
        raw = rng.integers(0, 256, (n, k // 32, 34), dtype=np.uint8)
        raw[:, :, 0:2] = np.frombuffer(np.float16(0.0005).tobytes(), np.uint8)
        ws[(k, n)] = raw.reshape(n, -1)
        for m in MS:
            xs[(k, m)] = rng.standard_normal((m, k)).astype(np.float32)
    return ws, xs


def run_reference(args):
    """CPU restatement of the reference path (the reference itself is Rust and cannot be built without a Rust
    toolchain), all host threads, on the same workload: every step is the full 16-launch sweep."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cbuild
    cbuild.build()
    threads = os.cpu_count() or 1
    ws, xs = host_weights_for_cpu(SHAPES)
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_reference_step(threads, SHAPES, ws, xs)
    times = [cpu_reference_step(threads, SHAPES, ws, xs) for _ in range(args.steps)]
    total = sum(times)
    tokens = sum(MS) * args.steps
    value = tokens / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg2_q8_0_decode_gemv_sweep", "shapes_k_to_n": SHAPES, "m": MS,
                   "note": "CPU port of the reference's dequantize-then-dot path; reference Rust not buildable here"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "full 16-launch sweep per step"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_gemv(args):
    import torch
    import engine_b200 as hq
    from engine_b200 import _lib as L

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    gen = torch.Generator(device=dev)
    gen.manual_seed(2000 + rank)
    n_variants = 16                       # step variants, each reading a different weight copy
    layers = {}
    for (k, n) in SHAPES:
        nbytes = n * (k // 32) * 34
        copies = n_variants if nbytes < 128 * 2**20 else 2
        base = make_q8_0_on_device(torch, n, k, gen, dev)
        layers[(k, n)] = [hq.GgufMatMul(base if c == 0 else base.clone(), "Q8_0", k) for c in range(copies)]
    xs = {(k, m): torch.randn((m, k), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
          for (k, _) in SHAPES for m in MS}
    ys = {(n, m): torch.empty((m, n), dtype=torch.float32, device=dev) for (_, n) in SHAPES for m in MS}
    launches_per_step = len(SHAPES) * len(MS)

    # one scratch for every launch: they all run on one stream, and each call leaves the scratch zero-filled
    ws_bytes = max(int(L.lib().hq_linear_workspace_bytes(layers[(k, n)][0]._weight_struct(), m))
                   for (k, n) in SHAPES for m in MS)
    ws = torch.zeros(max(ws_bytes, 256), dtype=torch.uint8, device=dev)

    def launch(layer, k, n, m):
        rc = L.lib().hq_linear_forward_ws(layer._weight_struct(), xs[(k, m)].data_ptr(), L.DT_BF16, k,
                                          ys[(n, m)].data_ptr(), L.DT_F32, n, m, ws.data_ptr(), ws.numel(),
                                          layer._status_buf(dev).data_ptr(), torch.cuda.current_stream().cuda_stream)
        L.check(rc, "hq_linear_forward_ws")

    def step(variant: int):
        for (k, n) in SHAPES:
            ls = layers[(k, n)]
            layer = ls[variant % len(ls)]
            for m in MS:
                launch(layer, k, n, m)

    # ---- warm-up (eager; also sets kernel attributes before any capture) ------------------------------
    for w in range(max(args.warmup, 3)):
        step(w)
    torch.cuda.synchronize()

    # ---- parity spot check of what is being timed (one launch against torch's f32 matmul of the dequantized
    # weights: d * q) -------------------------------------------------------------------------------------
    k0, n0 = SHAPES[0]
    lay = layers[(k0, n0)][0]
    blk = lay.data.reshape(n0, k0 // 32, 34)
    deq = (blk[:, :, 0:2].contiguous().view(torch.float16).to(torch.float32) *
           blk[:, :, 2:].contiguous().view(torch.int8).to(torch.float32)).reshape(n0, k0)
    want = xs[(k0, 8)].to(torch.float32) @ deq.t()
    got = lay.forward_raw(xs[(k0, 8)], torch.float32)
    rel = float(torch.linalg.norm(got - want) / torch.linalg.norm(want))
    assert rel < 1e-3, f"bench self-check failed: rel-L2 {rel}"
    assert lay.device_status()[0] == 0
    del deq, want, got

    # ---- capture one CUDA graph per step variant ------------------------------------------------------------
    graphs = []
    side = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(side):
        for v in range(n_variants):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                step(v)
            graphs.append(g)
    torch.cuda.synchronize()
    for v in range(3):
        graphs[v].replay()
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- timed region: exactly K steps, device-resident inputs ----------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(args.steps):
        graphs[s % n_variants].replay()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)

    # ---- per-launch kernel durations: one CUDA graph of back-to-back launches per (shape, M), each launch on
    # a different weight copy, timed with CUDA events and divided by the launch count (a Python-driven launch
    # costs more host time than these kernels run for, so eager event pairs would time the host) -----------
    per = {}
    with torch.cuda.stream(side):
        for (k, n) in SHAPES:
            ls = layers[(k, n)]
            reps = len(ls) if len(ls) > 2 else 4
            for m in MS:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for r in range(reps):
                        launch(ls[r % len(ls)], k, n, m)
                per[(k, n, m)] = (g, reps)
    torch.cuda.synchronize()
    for key, (g, reps) in list(per.items()):
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) / reps)
        per[key] = statistics.median(ts)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the public API with pinned host buffers -------------------------------------------
    hx = {key: t.cpu().pin_memory() for key, t in xs.items()}
    hy = {key: torch.empty(t.shape, dtype=t.dtype).pin_memory() for key, t in ys.items()}
    h2d = sum(t.numel() * t.element_size() for t in hx.values())
    d2h = sum(t.numel() * t.element_size() for t in hy.values())

    def e2e_step(variant: int):
        for (k, n) in SHAPES:
            ls = layers[(k, n)]
            layer = ls[variant % len(ls)]
            for m in MS:
                xd = hx[(k, m)].to(dev, non_blocking=True)
                y = layer.forward_raw(xd, torch.float32)
                hy[(n, m)].copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    for v in range(3):
        e2e_step(v)
    barrier()
    t0 = time.perf_counter()
    for s in range(args.steps):
        e2e_step(s)
    barrier()
    e2e_s = time.perf_counter() - t0

    # ---- reduce over ranks -------------------------------------------------------------------------------------
    if dist is not None:
        tt = torch.tensor([ms_total, e2e_s * 1e3], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = float(tt[0]), float(tt[1])
    else:
        e2e_ms = e2e_s * 1e3
    tokens_per_step = sum(MS)
    value = world * tokens_per_step * args.steps / (ms_total / 1e3)
    e2e_value = world * tokens_per_step * args.steps / (e2e_ms / 1e3)

    if rank == 0:
        peak, peak_kind = load_peaks()
        step_bytes = sum(algorithmic_bytes(k, n, m) for (k, n) in SHAPES for m in MS)
        kern_ms = sum(per.values())
        achieved = step_bytes / (kern_ms / 1e3) / 1e9
        by_shape = {}
        for (k, n) in SHAPES:
            for m in MS:
                by_shape[f"{k}x{n}_m{m}"] = round(algorithmic_bytes(k, n, m) / (per[(k, n, m)] / 1e3) / 1e9, 1)
        # CPU baseline: the C oracle on the three Llama layer shapes without the vocabulary projection
        cpu = None
        try:
            from oracle import cbuild
            cbuild.build()
            sample = SHAPES[:3] if len(SHAPES) > 1 else SHAPES
            ws, hxs = host_weights_for_cpu(sample)
            threads = os.cpu_count() or 1
            cpu_reference_step(threads, sample, ws, hxs)
            dt = min(cpu_reference_step(threads, sample, ws, hxs) for _ in range(3))
            sample_bytes = sum(algorithmic_bytes(k, n, m) for (k, n) in sample for m in MS)
            # scaled to the full step by algorithmic bytes (the CPU path is bandwidth/dequant bound per weight)
            cpu = {"value": tokens_per_step / (dt * step_bytes / sample_bytes), "unit": UNIT, "cores": threads,
                   "kind": "port", "sample": "4096->4096, 4096->14336, 14336->4096 at M in {1,2,4,8}, scaled to the "
                                            "full sweep by algorithmic bytes"}
        except Exception as exc:  # the checker failing to build must not hide the GPU numbers
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"unavailable: {exc}"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
            "config": {"workload": "cfg2_q8_0_decode_gemv_sweep" if len(SHAPES) == 4 else "single_shape_profile_case",
                       "shapes_k_to_n": SHAPES, "m": MS, "x_dtype": "bf16", "y_dtype": "f32", "multi_gpu": "replicas only (dense GEMV is not sharded)",
                       "l2": "every launch reads a weight copy last touched >= 700 MB of traffic earlier",
                       "timing": "CUDA-graph replay per step, CUDA events"},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4),
                         # DRAM bytes per launch (average over the step's launches): the ncu capture of the
                         # 4096 -> 128256 launch read and wrote 563.3 MB for 558.2 MB of algorithmic bytes
                         # (profiles/gemv_int8_q8_0_4096x128256.md); the other launches are scaled by that ratio
                         "traffic": int(NCU_TRAFFIC_RATIO * step_bytes / launches_per_step),
                         "traffic_note": "algorithmic bytes x 1.009 (ncu dram bytes / algorithmic bytes of the "
                                         "4096x128256 launch)",
                         "peak_kind": peak_kind, "kernel": "hq::gemv_int8_kernel<Q8_0>", "launch_ms_sum": round(kern_ms, 4),
                         "bytes_per_step": step_bytes, "by_launch_gbs": by_shape,
                         "graph_step_gbs": round(step_bytes / (ms_total / args.steps / 1e3) / 1e9, 1)},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# ======================================================================================================
# MoE layer workloads (BASELINE configs 3-5): router -> dispatch tables -> gate/up projection with the gated
# activation fused -> down projection -> weighted reduce.  Router logits are an input of the step, as they
# are for the reference's moe_router_topk.
# ======================================================================================================
MOE_CFGS = {
    # name: (format, experts, top_k, hidden, intermediate, tokens, router mode, interleaved gate/up + biases)
    "moe_q4k": dict(fmt="Q4_K", e=128, k=8, h=2048, i=768, t=4096, router="softmax", inter=False,
                    label="cfg3_qwen3_30b_a3b_q4k_moe"),
    "moe_fp8": dict(fmt="FP8", e=256, k=8, h=7168, i=2048, t=4096, router="sigmoid_bias", inter=False,
                    shared=True, act_fp8=True, label="cfg4_deepseek_v3_block_fp8_moe"),
    "moe_mxfp4": dict(fmt="MXFP4", e=128, k=4, h=2880, i=2880, t=8192, router="topk_softmax", inter=True,
                      label="cfg5_gpt_oss_120b_mxfp4_moe"),
}


def _q4k_bank(torch, e, n, k, gen, dev):
    """N(0, 0.02^2) weights -> GGUF Q4_K super-blocks with a plain min/max quantizer, on the device, one expert at a
    time (benchmark data only): per 32-element sub-block scale = (max - min)/15 and min <= 0, both coded in 6 bits
    against the super-block's d / dmin."""
    out = torch.empty((e, n, k // 256, 144), dtype=torch.uint8, device=dev)
    for ex in range(e):
        w = torch.randn((n, k // 256, 8, 32), generator=gen, device=dev) * 0.02
        mn = torch.clamp(w.amin(dim=3), max=0.0)
        sc = (w.amax(dim=3) - mn) / 15.0
        d = (sc.amax(dim=2, keepdim=True) / 63.0).to(torch.float16)
        dmin = ((-mn).amax(dim=2, keepdim=True) / 63.0).to(torch.float16)
        df, dmf = d.float().clamp_min(1e-12), dmin.float().clamp_min(1e-12)
        ls = torch.clamp(torch.round(sc / df), 0, 63).to(torch.int32)
        lm = torch.clamp(torch.round(-mn / dmf), 0, 63).to(torch.int32)
        d1 = (d.float() * ls).unsqueeze(-1)
        m1 = (dmin.float() * lm).unsqueeze(-1)
        q = torch.clamp(torch.round((w + m1) / d1.clamp_min(1e-12)), 0, 15).to(torch.uint8)
        blk = out[ex]
        blk[:, :, 0:2] = d.view(torch.uint8).reshape(n, k // 256, 2)
        blk[:, :, 2:4] = dmin.view(torch.uint8).reshape(n, k // 256, 2)
        sb = torch.zeros((n, k // 256, 12), dtype=torch.int32, device=dev)
        sb[:, :, 0:4] = ls[:, :, 0:4] | ((ls[:, :, 4:8] >> 4) << 6)
        sb[:, :, 4:8] = lm[:, :, 0:4] | ((lm[:, :, 4:8] >> 4) << 6)
        sb[:, :, 8:12] = (ls[:, :, 4:8] & 0xF) | ((lm[:, :, 4:8] & 0xF) << 4)
        blk[:, :, 4:16] = sb.to(torch.uint8)
        blk[:, :, 16:] = (q[:, :, 0::2, :] | (q[:, :, 1::2, :] << 4)).reshape(n, k // 256, 128)
    return out.reshape(e, n, -1)


def _fp8_bank(torch, e, n, k, gen, dev):
    codes = torch.empty((e, n, k), dtype=torch.uint8, device=dev)
    scales = torch.empty((e, n // 128, k // 128), dtype=torch.float32, device=dev)
    for ex in range(e):
        w = (torch.randn((n // 128, 128, k // 128, 128), generator=gen, device=dev) * 0.02)
        s = w.abs().amax(dim=(1, 3)) / 448.0
        q = (w / s[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
        codes[ex] = q.view(torch.uint8).reshape(n, k)
        scales[ex] = s
    return codes, scales


def _mxfp4_bank(torch, e, n, k, gen, dev):
    blocks = torch.empty((e, n, k // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty((e, n, k // 32), dtype=torch.uint8, device=dev)
    for ex in range(e):
        w = torch.randn((n, k // 32, 32), generator=gen, device=dev) * 0.02
        amax = w.abs().amax(dim=2)
        ee = torch.clamp(torch.floor(torch.log2(amax / 6.0)) + 127, 0, 254)
        ee = torch.where(amax == 0, torch.full_like(ee, 127), ee)
        v = (w / torch.exp2(ee - 127).unsqueeze(-1)).abs()
        nib = ((v >= 0.25).int() + (v >= 0.75).int() + (v >= 1.25).int() + (v >= 1.75).int() + (v >= 2.5).int() +
               (v >= 3.5).int() + (v >= 5.0).int())
        nib = (nib | ((w < 0).int() << 3)).to(torch.uint8).reshape(n, k)
        blocks[ex] = nib[:, 0::2] | (nib[:, 1::2] << 4)
        scales[ex] = ee.to(torch.uint8)
    return blocks, scales


def build_moe_layer(torch, hq, cfg, gen, dev, e_local=None):
    """Banks for experts [0, e_local) of the layer (all experts when e_local is None)."""
    e = e_local or cfg["e"]
    h, i, fmt = cfg["h"], cfg["i"], cfg["fmt"]
    from engine_b200 import _lib as L

    def bank(n, k, bias):
        b = (torch.randn((e, n), generator=gen, device=dev) * 0.02).to(torch.bfloat16) if bias else None
        if fmt == "Q4_K":
            return hq.GgufMatMul(_q4k_bank(torch, e, n, k, gen, dev), "Q4_K", k, b)
        if fmt == "FP8":
            c, s = _fp8_bank(torch, e, n, k, gen, dev)
            return hq.BlockwiseFP8Linear(c, s, b)
        bl, sc = _mxfp4_bank(torch, e, n, k, gen, dev)
        return hq.MXFP4Layer(bl, sc, b)

    down = bank(h, i, cfg["inter"])
    if cfg["inter"]:
        return hq.MoEExperts(down, gate_up_proj=bank(2 * i, h, True), act=L.ACT_GPTOSS, limit=7.0, alpha=1.702)
    return hq.MoEExperts(down, bank(i, h, False), bank(i, h, False), act=L.ACT_SWIGLU)


def router_config(hq, cfg):
    from engine_b200 import _lib as L
    if cfg["router"] == "softmax":
        return hq.MoeRouterTopKConfig(cfg["k"], L.SCORE_SOFTMAX, L.WEIGHT_SCORE, True)
    if cfg["router"] == "sigmoid_bias":
        return hq.MoeRouterTopKConfig(cfg["k"], L.SCORE_SIGMOID, L.WEIGHT_SCORE, True, 1e-20, 2.5)
    return hq.MoeRouterTopKConfig(cfg["k"], L.SCORE_RAW, L.WEIGHT_SOFTMAX, False)


def gemm_kernel_name(cfg, tokens):
    """The expert GEMM kernel the library's dispatch takes for this layer (mirrors hq_moe_gather_forward's rule:
    MXFP4 always, Q4_K below 192 rows per expert, expand the weights into tensor memory)."""
    rows_per_expert = tokens * cfg["k"] / cfg["e"]
    ts = cfg["fmt"] == "MXFP4" or (cfg["fmt"] == "Q4_K" and rows_per_expert < 192)
    return ("hq::grouped_gemm_ts_kernel" if ts else "hq::grouped_gemm_kernel") + " (gate/up + down)"


def moe_flops(cfg, tokens, with_shared=False):
    per_expert = 2.0 * 3 * cfg["h"] * cfg["i"]
    return tokens * per_expert * (cfg["k"] + (1 if with_shared and cfg.get("shared") else 0))


def run_moe(args):
    import torch
    import engine_b200 as hq
    from engine_b200 import _lib as L
    from engine_b200.ep import ExpertParallelMoE

    cfg = dict(MOE_CFGS[args.workload])
    if args.tokens:
        cfg["t"] = args.tokens
    if args.experts:
        cfg["e"] = args.experts       # a smaller bank of the same expert shape (profiling cases that must stay small)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3000 + rank)
    e, k, h, t_global = cfg["e"], cfg["k"], cfg["h"], cfg["t"]
    # tokens are data-parallel, experts sharded E/world per rank.  Weak scaling (default): every rank brings the
    # configuration's token count; strong: the global count is split.
    weak = args.ep_scaling == "weak"
    t_local = t_global if weak else t_global // world
    t_global = t_local * world
    experts = build_moe_layer(torch, hq, cfg, gen, dev, e // world)
    ep = (ExpertParallelMoE(e, experts, wire_dtype=torch.float16, fp8_act=bool(cfg.get("act_fp8")),
                            chunks=args.ep_chunks) if world > 1 else None)
    shared = None
    if cfg.get("shared"):
        # the always-on shared expert: the same three projections as a one-expert bank over this rank's tokens
        shared = build_moe_layer(torch, hq, cfg, gen, dev, 1)
        shared_ids = torch.zeros((t_local, 1), dtype=torch.int32, device=dev)
        shared_w = torch.ones((t_local, 1), dtype=torch.float32, device=dev)
    rcfg = router_config(hq, cfg)
    sel_bias = (torch.randn(e, generator=gen, device=dev) * 0.01) if cfg["router"] == "sigmoid_bias" else None
    n_in = 4                                          # rotate inputs; the expert bank itself exceeds L2
    xs = [torch.randn((t_local, h), generator=gen, device=dev).to(torch.bfloat16) for _ in range(n_in)]
    logits = [torch.randn((t_local, e), generator=gen, device=dev) for _ in range(n_in)]
    launches = [0]

    def step(j, x=None, lg=None, force_16bit=False):
        x = xs[j % n_in] if x is None else x
        lg = logits[j % n_in] if lg is None else lg
        fused_call = ep is None and not cfg.get("act_fp8")      # router and experts in one library call
        top = None if fused_call else hq.moe_router_topk(lg, rcfg, sel_bias)
        if cfg.get("act_fp8") and not force_16bit:
            # block-scaled FP8 activations (per-token 1x128 dynamic quantization, the layer's own arithmetic): the
            # codes of weights and activations go into the FP8 MMA unconverted
            add = None
            if shared is not None:
                add = shared.forward_fp8_act(x, shared_w[:x.shape[0]], shared_ids[:x.shape[0]], out_dtype=torch.bfloat16)
            if ep is not None:
                return ep.forward(x, top.values, top.indices, shared_out=add, out_dtype=torch.bfloat16)
            return experts.forward_fp8_act(x, top.values, top.indices, shared_out=add, out_dtype=torch.bfloat16)
        if cfg.get("act_fp8"):
            # the same quantizer, but the experts see the dequantized codes as f16 (16-bit MMA): only used as the
            # cross-check of the FP8 path
            codes, scales = hq.fp8_vector_quantize(x)
            x = hq.fp8_vector_dequantize(codes, scales, torch.float16)
        add = None
        if shared is not None:
            add = shared.forward(x, shared_w[:x.shape[0]], shared_ids[:x.shape[0]], out_dtype=torch.bfloat16)
        if ep is not None:
            return ep.forward(x, top.values, top.indices, shared_out=add, out_dtype=torch.bfloat16)
        if fused_call:
            # one library call for the whole layer (router included): no host work between the launches
            return experts.forward_layer(x, lg, rcfg, sel_bias, shared_out=add, out_dtype=torch.bfloat16)
        return experts.forward(x, top.values, top.indices, shared_out=add, out_dtype=torch.bfloat16)

    for w in range(max(args.warmup, 3)):
        out = step(w)
    torch.cuda.synchronize()
    status = experts.down.device_status()
    assert status[0] == 0, f"device status {status}"
    assert bool(torch.isfinite(out.float()).all())
    # what is timed is checked against the decode kernel (itself pinned to the CPU oracle by the tests): same step,
    # tensor-core path switched off, first 64 tokens
    parity = None
    if world == 1:
        lib = L.lib()
        old = lib.hq_config_get(L.CFG_MOE_TENSOR_MIN_ROWS)
        n_chk = min(64, t_local)
        a = step(0)[:n_chk].float()
        lib.hq_config_set(L.CFG_MOE_TENSOR_MIN_ROWS, 1 << 40)
        try:
            b = step(0, xs[0][:n_chk].contiguous(), logits[0][:n_chk].contiguous(), force_16bit=True).float()
        finally:
            lib.hq_config_set(L.CFG_MOE_TENSOR_MIN_ROWS, old)
        parity = float(torch.linalg.norm(a - b) / torch.linalg.norm(b))
        # the FP8-activation path also quantizes the expert intermediate (about 3e-2), which the 16-bit check path
        # does not: it gets a looser gate here and its own parity tests against the oracle
        gate_tol = 6e-2 if cfg.get("act_fp8") else 1e-2
        assert parity < gate_tol, f"tensor-core path disagrees with the decode kernel: rel-L2 {parity}"

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s_ in range(args.steps):
        step(s_)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None

    # dominant kernel: the two expert projections, timed on their own at this rank's share of the work
    gemm_ms = None
    if world == 1:
        top = hq.moe_router_topk(logits[0], rcfg, sel_bias)
        tables = hq.moe_dispatch_build(top.indices, e)
        ts = []
        for r in range(6):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            x = xs[r % n_in]
            a.record()
            fwd = experts.forward_fp8_act if cfg.get("act_fp8") else experts.forward
            fwd(x, top.values, top.indices, out_dtype=torch.bfloat16, tables=tables, _skip_reduce=True)
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        gemm_ms = statistics.median(ts[1:])

    # end to end with pinned host buffers: activations + logits in, layer output back
    hx = [x.cpu().pin_memory() for x in xs]
    hl = [l_.cpu().pin_memory() for l_ in logits]
    hy = torch.empty((t_local, h), dtype=torch.bfloat16).pin_memory()

    def e2e_step(j):
        x = hx[j % n_in].to(dev, non_blocking=True)
        lg = hl[j % n_in].to(dev, non_blocking=True)
        hy.copy_(step(j, x, lg), non_blocking=True)
        torch.cuda.synchronize()

    for j in range(3):
        e2e_step(j)
    barrier()
    t0 = time.perf_counter()
    for j in range(args.steps):
        e2e_step(j)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    if dist is not None:
        tt = torch.tensor([ms_total, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = float(tt[0]), float(tt[1])
    value = t_global * args.steps / (ms_total / 1e3)
    e2e_value = t_global * args.steps / (e2e_ms / 1e3)
    if rank == 0:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
            os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
        peak_tf = float(peaks.get("bf16_tflops", 1590.0))
        roof = None
        if gemm_ms is not None:
            ach = moe_flops(cfg, t_global) / (gemm_ms / 1e3) / 1e12
            roof = {"bound": "tensor", "achieved": round(ach, 1), "peak": peak_tf, "unit": "TFLOP/s",
                    "frac": round(ach / peak_tf, 4), "traffic": None,
                    "peak_kind": "measured" if peaks else "fallback",
                    "kernel": gemm_kernel_name(cfg, t_global), "launch_ms_sum": round(gemm_ms, 4),
                    "note": "f16 operands: fraction of the measured dense 16-bit tensor peak"}
            if cfg.get("act_fp8"):
                # FP8 x FP8 MMA: still reported against the measured 16-bit peak (the only tensor peak the peaks
                # file holds); this repo's tcgen05 issue-rate probe gives 4289 TFLOP/s for the kernel's
                # 128 x 128 x 32 e4m3 instruction.  At 128 tokens per expert the layer reads every weight byte
                # once per ~1.5 token tiles, so the HBM figure is the one that binds.
                wbytes = 3 * (e // world) * cfg["i"] * h      # routed experts only: what the timed calls read
                roof.update({"kernel": "hq::fp8_grouped_kernel (gate, up, down) + row quantizers",
                             "note": "e4m3 x e4m3 MMA (kind::f8f6f4); fraction of the measured dense 16-bit peak",
                             "fp8_probe_peak_tflops": 4289.0,
                             "weight_stream_gbs": round(wbytes / (gemm_ms / 1e3) / 1e9, 1)})
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak" if weak else "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": cfg["label"], "format": cfg["fmt"], "experts": e, "top_k": k, "hidden": h,
                       "intermediate": cfg["i"], "tokens_global": t_global, "experts_per_gpu": e // world,
                       "parallelism": f"ep{world}" + (f" x{args.ep_chunks} chunks" if world > 1 and args.ep_chunks > 1 else ""), "l2": "expert banks exceed L2; activations rotate over 4 buffers"},
            "roofline": roof,
            "parity_vs_decode_kernel_rel_l2_bf16_out": parity,
            "cpu_baseline": None,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": t_local * (h * 2 + e * 4),
                    "d2h_bytes_per_step": t_local * h * 2, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": args.steps * 7,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="gemv", choices=["gemv"] + list(MOE_CFGS))
    ap.add_argument("--tokens", type=int, default=0, help="override the token count of a MoE workload")
    ap.add_argument("--ep-chunks", type=int, default=1,
                    help="MoE workloads on several GPUs: token chunks whose exchange overlaps the experts of other chunks")
    ap.add_argument("--experts", type=int, default=0, help="override the expert count of a MoE workload")
    ap.add_argument("--ep-scaling", default="weak", choices=["weak", "strong"],
                    help="MoE workloads on several GPUs: tokens per GPU fixed (weak) or global count split (strong)")
    ap.add_argument("--only", default=None, help="restrict the sweep to one KxN shape, e.g. 4096x128256 "
                    "(profiling aid; the reported line is then not the headline workload)")
    args = ap.parse_args()
    if args.only:
        k, n = (int(v) for v in args.only.lower().split("x"))
        global SHAPES
        SHAPES = [(k, n)]
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload in MOE_CFGS:
        run_moe(args)
        return
    run_gemv(args)


if __name__ == "__main__":
    main()
