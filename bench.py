"""Benchmark of the quantized-linear / sparse-MoE hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload moe_fp8] [--impl reference]

Default workload `moe_fp8`: one DeepSeek-V3-shaped block-FP8 MoE layer (256 routed experts, top-8, one shared expert,
hidden 7168, expert intermediate 2048, sigmoid router with bias) over 4096 tokens, block-scaled FP8 activations
(per-token 1x128).  One step = router -> dispatch tables -> gate/up projection with the gated activation ->
down projection -> weighted sum over the slots (+ the shared expert).  With N GPUs the experts are sharded E/N
per rank and the 4096 tokens are split N ways (fixed global token count: strong scaling); every step then
contains the two all-to-all exchanges of the expert-parallel layer.  Router logits are an input of the step, as
they are for the reference's moe_router_topk.  Data are synthetic: weights N(0, 0.02^2) quantized to the
layer's format, activations N(0, 1) in bf16.

`--workload moe_q4k | moe_mxfp4` run the Qwen3-30B-A3B-shaped Q4_K layer and the gpt-oss-120b-shaped MXFP4
layer the same way; `--workload gemv` runs the Q8_0 decode mat-vec sweep over Llama-3-8B shapes (replicas only),
which is also embedded in the default line as the `gemv` record on one GPU.

One JSON line is printed by rank 0.  `value` is timed with inputs resident in HBM (CUDA events); `e2e` times the
same step through the public API with pinned host buffers (host->device copy of activations and logits,
device->host copy of the result inside the timed region); `roofline` is the expert GEMM pair (gate/up + down)
timed by CUDA events inside the step; `cpu_baseline` is the CPU oracle on a token subset, which also checks the
GPU result for those tokens.  `--impl reference` times the CPU restatement of the reference path alone.
"""
from __future__ import annotations

import argparse
import ctypes as C
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
UNIT = "tokens/s"

# DRAM bytes over algorithmic bytes from the ncu captures under profiles/
NCU_TRAFFIC_RATIO_GEMV = 563.3 / 558.2      # hq::gemv_int8_kernel, 4096 -> 128256
NCU_TRAFFIC_RATIO_FP8 = 1573.4 / 1515.6     # hq::fp8_grouped_kernel, routed gate/up + down, 32 experts x 128 rows
NCU_TRAFFIC_RATIO_MX = 527.3 / 543.2        # hq::mx_grouped_kernel, gate/up + down, 32 experts x 256 rows
NCU_TRAFFIC_RATIO_Q4K = 118.8 / 181.3       # hq::grouped_gemm_kernel<Q4_K>, gate/up + down, 32 experts x 256 rows
                                            # (below 1: most of the f32 output rows are still in L2 at the end)


def algorithmic_bytes(k, n, m, x_size=2, y_size=4):
    return n * (k // 32) * 34 + m * k * x_size + m * n * y_size


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


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


def dist_env():
    return (int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")),
            int(os.environ.get("LOCAL_RANK", "0")))


# ======================================================================================================
# Q8_0 decode mat-vec sweep (benchmark configuration 2: Llama-3-8B shapes)
# ======================================================================================================
GEMV_METRIC = "quant_linear_decode_tokens_per_s"


def gemv_config():
    return {"workload": "cfg2_q8_0_decode_gemv_sweep" if len(SHAPES) == 4 else "single_shape_profile_case",
            "shapes_k_to_n": SHAPES, "m": MS, "x_dtype": "bf16", "y_dtype": "f32",
            "multi_gpu": "replicas only (dense GEMV is not sharded)",
            "l2": "every launch reads a weight copy last touched >= 700 MB of traffic earlier",
            "timing": "CUDA-graph replay per step, CUDA events"}


def gemv_host_data(shapes):
    import numpy as np
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


def gemv_cpu_step(threads, shapes, ws, xs):
    """One pass of the (shape, M) list through the C oracle; returns seconds."""
    from oracle import cbuild
    t0 = time.perf_counter()
    for (k, n) in shapes:
        for m in MS:
            cbuild.linear("Q8_0", ws[(k, n)], None, None, xs[(k, m)], threads)
    return time.perf_counter() - t0


def decode_other_formats(torch, dev, peak_gbs,
                         formats=("Q4_K", "Q6_K", "Q5_K", "Q4_0", "Q5_0", "Q4_1", "Q5_1", "Q2_K", "Q3_K", "MXFP4", "FP8"),
                         n=65536, reps=8, ms=(1, 4)):
    """Decode mat-vec of the other weight formats on one 4096 -> 65536 projection (88 - 268 MB of weights, streamed
    from HBM by every launch: see the fill below), M = 1 and 4: median launch duration by CUDA events, algorithmic
    GB/s and the fraction of the measured HBM peak.  A 256 MB fill is queued in front of every timed launch: it
    evicts L2 and keeps the GPU busy while the host enqueues the launch, so the events bracket the kernel alone."""
    import engine_b200 as hq
    from tests import hq_synth as S
    gen = torch.Generator(device=dev)
    gen.manual_seed(2100)
    k = 4096
    out = {}
    flush = torch.empty(256 * 2**20, dtype=torch.uint8, device=dev)

    def ggml_bytes(block_bytes, weights_per_block, f16_at):
        # any byte pattern is a valid block of these types; the f16 fields are set to 2^-11 (0x1000)
        raw = torch.randint(0, 256, (n, k // weights_per_block, block_bytes), generator=gen, device=dev,
                            dtype=torch.uint8)
        for o in f16_at:
            raw[:, :, o] = 0x00
            raw[:, :, o + 1] = 0x10
        return raw.reshape(n, -1)

    for fmt in formats:
        if fmt == "Q4_K":
            layer = hq.GgufMatMul(S.q4k_bank(torch, 1, n, k, gen, dev)[0], "Q4_K", k)
            wbytes = n * (k // 256) * 144
        elif fmt == "Q6_K":
            layer = hq.GgufMatMul(ggml_bytes(210, 256, (208,)), "Q6_K", k)
            wbytes = n * (k // 256) * 210
        elif fmt == "Q5_K":
            layer = hq.GgufMatMul(ggml_bytes(176, 256, (0, 2)), "Q5_K", k)
            wbytes = n * (k // 256) * 176
        elif fmt == "Q4_0":
            layer = hq.GgufMatMul(ggml_bytes(18, 32, (0,)), "Q4_0", k)
            wbytes = n * (k // 32) * 18
        elif fmt == "Q5_0":
            layer = hq.GgufMatMul(ggml_bytes(22, 32, (0,)), "Q5_0", k)
            wbytes = n * (k // 32) * 22
        elif fmt == "Q4_1":
            layer = hq.GgufMatMul(ggml_bytes(20, 32, (0, 2)), "Q4_1", k)
            wbytes = n * (k // 32) * 20
        elif fmt == "Q5_1":
            layer = hq.GgufMatMul(ggml_bytes(24, 32, (0, 2)), "Q5_1", k)
            wbytes = n * (k // 32) * 24
        elif fmt == "Q2_K":
            layer = hq.GgufMatMul(ggml_bytes(84, 256, (80, 82)), "Q2_K", k)
            wbytes = n * (k // 256) * 84
        elif fmt == "Q3_K":
            layer = hq.GgufMatMul(ggml_bytes(110, 256, (108,)), "Q3_K", k)
            wbytes = n * (k // 256) * 110
        elif fmt == "MXFP4":
            b, sc = S.mxfp4_bank(torch, 1, n, k, gen, dev)
            layer = hq.MXFP4Layer(b[0], sc[0])
            wbytes = n * k // 2 + n * k // 32
        else:
            c, sc = S.fp8_bank(torch, 1, n, k, gen, dev)
            layer = hq.BlockwiseFP8Linear(c[0], sc[0])
            wbytes = n * k + (n // 128) * (k // 128) * 4
        for m in ms:
            x = torch.randn((m, k), generator=gen, device=dev).to(torch.bfloat16)
            ts = []
            for r in range(reps):
                a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                flush.zero_()
                a.record()
                layer.forward_raw(x, torch.float32)
                b_.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b_))
            assert layer.device_status()[0] == 0
            t_ms = statistics.median(ts[2:] if len(ts) > 4 else ts)
            nbytes = wbytes + m * k * 2 + m * n * 4
            out[f"{fmt}_4096x{n}_m{m}"] = {"us": round(t_ms * 1e3, 1), "gbs": round(nbytes / t_ms / 1e6, 1),
                                           "frac": round(nbytes / t_ms / 1e6 / peak_gbs, 4)}
        del layer
        torch.cuda.empty_cache()
    return out


def gemv_measure(args, torch, dev, rank, world, dist, with_cpu=True):
    """Times the 16-launch sweep; returns the record (rank 0) or None."""
    import engine_b200 as hq
    from engine_b200 import _lib as L
    from tests import hq_synth as S

    gen = torch.Generator(device=dev)
    gen.manual_seed(2000 + rank)
    n_variants = 16                       # step variants, each reading a different weight copy
    layers = {}
    for (k, n) in SHAPES:
        nbytes = n * (k // 32) * 34
        copies = n_variants if nbytes < 128 * 2**20 else 2
        base = S.q8_0_matrix(torch, n, k, gen, dev)
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

    for w in range(max(args.warmup, 3)):
        step(w)
    torch.cuda.synchronize()
    # one launch against torch's f32 matmul of the dequantized weights (d * q); the oracle parity of this kernel at
    # every sweep shape is in tests/
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

    sampler = ClockSampler(dev.index)
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

    # per-launch kernel durations: one CUDA graph of back-to-back launches per (shape, M), each launch on a
    # different weight copy, timed with CUDA events and divided by the launch count: throughput under programmatic
    # dependent launch, not the isolated duration of one launch
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
    # isolated duration of single launches (event pair around one launch, stream otherwise idle)
    iso = {}
    for (k, n) in SHAPES:
        ls = layers[(k, n)]
        ts = []
        for r in range(6):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            launch(ls[r % len(ls)], k, n, 1)
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        iso[f"{k}x{n}_m1"] = round(statistics.median(ts[1:]) * 1e3, 1)
    clocks = sampler.stop() if rank == 0 else None

    # end to end through the public API with pinned host buffers
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
    e2e_ms = (time.perf_counter() - t0) * 1e3
    if dist is not None:
        tt = torch.tensor([ms_total, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = float(tt[0]), float(tt[1])
    del graphs
    if rank != 0:
        return None
    tokens_per_step = sum(MS)
    peaks = load_peaks()
    other = None
    if world == 1 and len(SHAPES) == 4:
        layers.clear()
        torch.cuda.empty_cache()
        other = decode_other_formats(torch, dev, peaks["hbm_gbs"])
    step_bytes = sum(algorithmic_bytes(k, n, m) for (k, n) in SHAPES for m in MS)
    kern_ms = sum(per.values())
    achieved = step_bytes / (kern_ms / 1e3) / 1e9
    by_shape = {f"{k}x{n}_m{m}": round(algorithmic_bytes(k, n, m) / (per[(k, n, m)] / 1e3) / 1e9, 1)
                for (k, n) in SHAPES for m in MS}
    cpu = None
    if with_cpu:
        try:
            from oracle import cbuild
            cbuild.build()
            sample = SHAPES[:3] if len(SHAPES) > 1 else SHAPES
            hws, hxs = gemv_host_data(sample)
            threads = os.cpu_count() or 1
            gemv_cpu_step(threads, sample, hws, hxs)
            dt = min(gemv_cpu_step(threads, sample, hws, hxs) for _ in range(3))
            sample_bytes = sum(algorithmic_bytes(k, n, m) for (k, n) in sample for m in MS)
            cpu = {"value": tokens_per_step / (dt * step_bytes / sample_bytes), "unit": UNIT, "cores": threads,
                   "kind": "port", "sample": "4096->4096, 4096->14336, 14336->4096 at M in {1,2,4,8}, scaled to the "
                                            "full sweep by algorithmic bytes"}
        except Exception as exc:  # the checker failing to build must not hide the GPU numbers
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"unavailable: {exc}"}
    return {
        "metric": GEMV_METRIC, "value": world * tokens_per_step * args.steps / (ms_total / 1e3), "unit": UNIT,
        "ms_per_step": ms_total / args.steps, "dtype": "s8", "config": gemv_config(),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4),
                     "frac_of_nominal_8tbs": round(achieved / 8000.0, 4),
                     "traffic": int(NCU_TRAFFIC_RATIO_GEMV * step_bytes / launches_per_step),
                     "traffic_note": "algorithmic bytes x 1.009 (ncu dram bytes / algorithmic bytes of the "
                                     "4096x128256 launch)",
                     "peak_kind": peaks["kind"], "kernel": "hq::gemv_int8_kernel<Q8_0>",
                     "launch_ms_sum": round(kern_ms, 4), "bytes_per_step": step_bytes,
                     "by_launch_gbs": by_shape,
                     "by_launch_note": "throughput of back-to-back launches under programmatic dependent launch",
                     "isolated_launch_us": iso,
                     "other_formats_decode": other,
                     "other_formats_note": "isolated launches through QuantMethod.forward (event pair around one "
                                           "call, weights larger than L2)",
                     "graph_step_gbs": round(step_bytes / (ms_total / args.steps / 1e3) / 1e9, 1)},
        "cpu_baseline": cpu,
        "e2e": {"value": world * tokens_per_step * args.steps / (e2e_ms / 1e3), "unit": UNIT,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }


def run_gemv(args):
    import torch
    world, rank, local_rank = dist_env()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    rec = gemv_measure(args, torch, dev, rank, world, dist)
    if rank == 0:
        line = {"metric": rec["metric"], "value": rec["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": rec["dtype"], "data": "synthetic",
                "config": rec["config"], "roofline": rec["roofline"], "cpu_baseline": rec["cpu_baseline"],
                "e2e": rec["e2e"], "gpu_launches": rec["gpu_launches"], "clocks": rec["clocks"]}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# ======================================================================================================
# MoE layer workloads (benchmark configurations 3-5)
# ======================================================================================================
MOE_METRIC = "moe_layer_tokens_per_s"


def moe_cfg(args):
    from tests import hq_synth as S
    cfg = dict(S.MOE_CFGS[args.workload])
    if args.tokens:
        cfg["t"] = args.tokens
    if args.experts:
        cfg["e"] = args.experts       # a smaller bank of the same expert shape (profiling cases that must stay small)
    if getattr(args, "act16", False):
        cfg["act_fp8"] = cfg["act_mx"] = False
    return cfg


def act_mode(cfg):
    """False (16-bit activations), True (1x128 FP8 activations) or "mx" (MXFP8 activations): the value the subset
    oracle takes for the same rounding points."""
    return True if cfg.get("act_fp8") else ("mx" if cfg.get("act_mx") else False)


def moe_config(cfg, world, scaling):
    """The `config` object of a MoE line; both arms print the same one."""
    return {"workload": cfg["label"], "format": cfg["fmt"], "experts": cfg["e"], "top_k": cfg["k"],
            "hidden": cfg["h"], "intermediate": cfg["i"], "shared_expert": bool(cfg.get("shared")),
            "tokens_global": cfg["t"], "experts_per_gpu": cfg["e"] // world, "parallelism": f"ep{world}",
            "scaling": scaling,
            "activation_mode": ("B: per-token 1x128 FP8 activations, e4m3 x e4m3 MMA" if cfg.get("act_fp8") else
                                "B: MXFP8 activations (e4m3 + e8m0 per 32), block-scaled e4m3 x e2m1 MMA"
                                if cfg.get("act_mx") else "A: 16-bit activations, weights expanded to f16"),
            "l2": "expert banks exceed L2; activations rotate over 4 buffers"}


def moe_flops(cfg, rows, shared_tokens=0):
    per_row = 2.0 * 3 * cfg["h"] * cfg["i"]
    return per_row * (rows + shared_tokens)


def probe_fp8_peak(torch, dev):
    """Dense issue rate of tcgen05.mma kind::f8f6f4 (e4m3, M = 128, N = 256) from every SM, in TFLOP/s."""
    from engine_b200 import _lib as L
    lib = L.lib()
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    flops = C.c_double(0.0)
    best = 0.0
    for it in range(4):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        rc = lib.hq_probe_tensor_peak(1, 256, 20000, status.data_ptr(), C.byref(flops),
                                      torch.cuda.current_stream().cuda_stream)
        b.record()
        torch.cuda.synchronize()
        if rc != 0 or int(status[0]) != 0:
            return None
        if it > 0:
            best = max(best, flops.value / (a.elapsed_time(b) / 1e3) / 1e12)
    return best


def run_moe(args):
    import numpy as np
    import torch
    import engine_b200 as hq
    from engine_b200 import _lib as L
    from engine_b200.ep import ExpertParallelMoE
    from tests import hq_synth as S

    cfg = moe_cfg(args)
    world, rank, local_rank = dist_env()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3000 + rank)
    e, k, h = cfg["e"], cfg["k"], cfg["h"]
    # tokens are data-parallel, experts sharded E/world per rank.  strong (default): the configuration's token count
    # is split over the ranks; weak: every rank brings the configuration's token count
    strong = args.ep_scaling == "strong"
    t_local = cfg["t"] // world if strong else cfg["t"]
    t_global = t_local * world
    fp8 = bool(cfg.get("act_fp8"))
    mx = bool(cfg.get("act_mx"))
    experts = S.build_moe_layer(torch, hq, cfg, gen, dev, e // world)
    ep = (ExpertParallelMoE(e, experts, top_k=k, hidden=h, capacity=t_local, wire_dtype=torch.bfloat16, fp8_act=fp8,
                            mx_act=mx, exchange=args.exchange) if (world > 1 or args.force_ep) else None)
    exchange_note = None
    if ep is not None and world > 1 and args.exchange == "p2p":
        # the symmetric buffers are set up collectively; if any rank cannot have them, every rank takes NCCL
        try:
            ep._symm_buffers(dev)
            ok = 1
        except Exception as exc:
            ok = 0
            exchange_note = f"symmetric memory unavailable ({type(exc).__name__}): all_to_all_single instead"
        agreed = torch.tensor([ok], device=dev, dtype=torch.int32)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed[0]) == 0:
            ep.exchange = "nccl"
            exchange_note = exchange_note or "symmetric memory unavailable on another rank: all_to_all_single instead"
    shared = S.build_moe_layer(torch, hq, cfg, gen, dev, 1) if cfg.get("shared") else None
    if shared is not None and not fp8:
        shared_ids = torch.zeros((t_local, 1), dtype=torch.int32, device=dev)
        shared_w = torch.ones((t_local, 1), dtype=torch.float32, device=dev)
    rcfg = S.router_config(hq, cfg)
    sel_bias = (torch.randn(e, generator=gen, device=dev) * 0.01) if cfg["router"] == "sigmoid_bias" else None
    n_in = 4                                          # rotate inputs; the expert bank itself exceeds L2
    xs = [torch.randn((t_local, h), generator=gen, device=dev).to(torch.bfloat16) for _ in range(n_in)]
    logits = [torch.randn((t_local, e), generator=gen, device=dev) for _ in range(n_in)]

    side_stream = torch.cuda.Stream(device=dev)

    def shared_fwd(x, out_dtype):
        if shared is None:
            return None
        if fp8:
            return shared.forward_fp8_dense(x, out_dtype)
        return shared.forward(x, shared_w[:x.shape[0]], shared_ids[:x.shape[0]], out_dtype=out_dtype)

    def step(j, x=None, lg=None, out_dtype=torch.bfloat16):
        x = xs[j % n_in] if x is None else x
        lg = logits[j % n_in] if lg is None else lg
        if ep is not None:
            sh, ev = None, None
            if shared is not None:
                # the shared expert depends on the activations only: it starts on its own stream before the router
                cur = torch.cuda.current_stream(dev)
                side_stream.wait_stream(cur)
                with torch.cuda.stream(side_stream):
                    sh = shared_fwd(x, out_dtype)
                    ev = side_stream.record_event()
            top = hq.moe_router_topk(lg, rcfg, sel_bias)
            return ep.forward(x, top.values, top.indices, out_dtype=out_dtype, shared_out=sh, shared_event=ev)
        if fp8:
            top = hq.moe_router_topk(lg, rcfg, sel_bias)
            return experts.forward_fp8_act(x, top.values, top.indices, shared_out=shared_fwd(x, out_dtype),
                                           out_dtype=out_dtype)
        if mx:
            top = hq.moe_router_topk(lg, rcfg, sel_bias)
            return experts.forward_mx_act(x, top.values, top.indices, shared_out=shared_fwd(x, out_dtype),
                                          out_dtype=out_dtype)
        # one library call for the whole layer (router included): no host work between the launches
        return experts.forward_layer(x, lg, rcfg, sel_bias, shared_out=shared_fwd(x, out_dtype), out_dtype=out_dtype)

    # launches of this library's kernels per step (the collectives' own kernels are not counted)
    if ep is not None:
        launches_per_step = 1 + 1 + 1 + 3 + (3 if (fp8 or mx) else 2) + 1 + 1 + \
            (4 if (shared is not None and fp8) else 0)
    elif fp8:
        launches_per_step = 1 + 3 + 3 + 1 + (4 if shared is not None else 0)
    elif mx:
        launches_per_step = 1 + 3 + 1 + 2 + 1          # router, dispatch build, row quantizer, two GEMMs, reduce
    else:
        launches_per_step = 1 + 3 + 1 + 2 + 1

    for w in range(max(args.warmup, 3)):
        out = step(w)
    torch.cuda.synchronize()
    status = experts.down.device_status()
    assert status[0] == 0, f"device status {status}"
    assert bool(torch.isfinite(out.float()).all())

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # The step as a CUDA graph per input set (launches, the two all-to-alls and the side-stream shared expert
    # included): with the experts sharded over several GPUs the step is short enough for the host-side launch
    # work to bound it otherwise.  Every rank captures the same sequence.
    graphs, graph_note = None, "off (--no-graph)"
    graph_events = []
    if not args.no_graph:
        try:
            experts.gemm_events = graph_events     # external event nodes around the two expert-GEMM launches
            cap = torch.cuda.Stream(device=dev)
            glist, gouts = [], []
            with torch.cuda.stream(cap):
                for j in range(n_in):
                    g = torch.cuda.CUDAGraph()
                    # thread-local error mode: the process group's watchdog thread polls its events meanwhile
                    with torch.cuda.graph(g, stream=cap, capture_error_mode="thread_local"):
                        gouts.append(step(j))
                    glist.append(g)
            torch.cuda.synchronize()
            for g in glist:
                g.replay()
            torch.cuda.synchronize()
            graphs, graph_note = glist, f"one CUDA graph per input set ({n_in}), replayed"
        except Exception as exc:
            if world > 1:
                raise       # a capture that broke off half-way has left collectives queued on this rank only
            # no graph: the eager loop below measures the same step
            graphs, graph_note = None, f"capture failed ({type(exc).__name__}), eager launches"
            torch.cuda.synchronize()
    assert experts.down.device_status()[0] == 0

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    experts.gemm_events = [] if graphs is None else None
    if graphs is None:
        graph_events = []
    barrier()
    if args.profiler_range:
        torch.cuda.profiler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s_ in range(args.steps):
        if graphs is not None:
            graphs[s_ % n_in].replay()
        else:
            step(s_)
    e1.record()
    barrier()
    if args.profiler_range:
        torch.cuda.profiler.stop()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    # dominant kernels: the expert GEMM pair of the routed experts, by CUDA events recorded around those two
    # launches on the stream they are launched on -- inside the timed steps when these are launched eagerly, in
    # separate eager steps after them when the timed steps are graph replays (events cannot be read back from a graph)
    gemm_ts = [a.elapsed_time(b) for a, b in (experts.gemm_events or [])]
    gemm_timing = "median over the timed steps of CUDA events around the two launches"
    if not gemm_ts and graph_events:
        try:       # one event pair per graph: what its last replay inside the timed steps recorded
            gemm_ts = [a.elapsed_time(b) for a, b in graph_events]
            gemm_timing = ("median over the graphs of the CUDA events (external event nodes) around the two "
                           "launches, as recorded by each graph's last replay inside the timed steps")
        except Exception:
            gemm_ts = []
    if not gemm_ts:
        experts.gemm_events = []
        for j in range(6):
            if ep is None and not (fp8 or mx):
                # the one-call layer path gives no place for events between its launches: the two-call route
                top = hq.moe_router_topk(logits[j % n_in], rcfg, sel_bias)
                experts.forward(xs[j % n_in], top.values, top.indices, out_dtype=torch.bfloat16)
            else:
                step(j)
        torch.cuda.synchronize()
        gemm_ts = [a.elapsed_time(b) for a, b in experts.gemm_events][2:]
        gemm_timing = "median of four separate eager runs of the same two launches after the timed steps"
    experts.gemm_events = None
    gemm_ms = statistics.median(gemm_ts) if gemm_ts else None
    # routed assignments this rank's experts received
    tables = getattr(experts, "_last_tables", None)
    rows_here = int(tables.expert_bounds[-1]) if tables is not None else t_local * k

    # end to end with pinned host buffers: activations + logits in, layer output back
    hx = [x.cpu().pin_memory() for x in xs]
    hl = [l_.cpu().pin_memory() for l_ in logits]
    hy = torch.empty((t_local, h), dtype=torch.bfloat16).pin_memory()

    # Every step copies its inputs in and its result out; the copies of neighbouring steps overlap the layer on
    # streams of their own (two device input sets and two output buffers in rotation), as a serving loop would
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    dx = [torch.empty_like(xs[0]) for _ in range(2)]
    dl = [torch.empty_like(logits[0]) for _ in range(2)]
    dout = [torch.empty((t_local, h), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    hys = [hy, torch.empty_like(hy).pin_memory()]
    main = torch.cuda.current_stream()

    e2e_graphs = None
    if graphs is not None:
        try:
            cap2 = torch.cuda.Stream(device=dev)
            eg = []
            with torch.cuda.stream(cap2):
                for b_ in range(2):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=cap2, capture_error_mode="thread_local"):
                        dout[b_].copy_(step(0, dx[b_], dl[b_]))
                    eg.append(g)
            torch.cuda.synchronize()
            e2e_graphs = eg
        except Exception:
            if world > 1:
                raise
            e2e_graphs = None
            torch.cuda.synchronize()

    def e2e_run(n_steps):
        ev_in = [None, None]          # inputs of slot b are on the device
        ev_done = [None, None]        # the layer has consumed slot b's inputs and produced slot b's output
        ev_out = [None, None]         # slot b's output has left the device
        for j in range(n_steps):
            b_ = j & 1
            with torch.cuda.stream(s_in):
                if ev_done[b_] is not None:
                    s_in.wait_event(ev_done[b_])
                dx[b_].copy_(hx[j % n_in], non_blocking=True)
                dl[b_].copy_(hl[j % n_in], non_blocking=True)
                ev_in[b_] = torch.cuda.Event()
                ev_in[b_].record(s_in)
            main.wait_event(ev_in[b_])
            if ev_out[b_] is not None:
                main.wait_event(ev_out[b_])
            if e2e_graphs is not None:
                e2e_graphs[b_].replay()
            else:
                dout[b_].copy_(step(j, dx[b_], dl[b_]))
            ev_done[b_] = torch.cuda.Event()
            ev_done[b_].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[b_])
                hys[b_].copy_(dout[b_], non_blocking=True)
                ev_out[b_] = torch.cuda.Event()
                ev_out[b_].record(s_out)
        torch.cuda.synchronize()

    e2e_run(3)
    barrier()
    t0 = time.perf_counter()
    e2e_run(args.steps)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    if dist is not None:
        tt = torch.tensor([ms_total, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = float(tt[0]), float(tt[1])
    value = t_global * args.steps / (ms_total / 1e3)
    e2e_value = t_global * args.steps / (e2e_ms / 1e3)

    # CPU baseline + parity of what was timed (one GPU only: the oracle needs every expert a token touches)
    cpu, parity = None, None
    if rank == 0 and world == 1:
        try:
            from oracle import cbuild
            cbuild.build()
            n_chk = args.cpu_tokens or (8 if cfg["fmt"] == "FP8" else 32)
            n_chk = min(n_chk, t_local)
            sel = np.linspace(0, t_local - 1, n_chk).astype(np.int64)
            x0 = xs[0][torch.as_tensor(sel, device=dev)].contiguous()
            l0 = logits[0][torch.as_tensor(sel, device=dev)].contiguous()
            got = step(0, xs[0], logits[0], out_dtype=torch.float32)[torch.as_tensor(sel, device=dev)].cpu().numpy()
            threads = os.cpu_count() or 1
            secs = []
            t_r = time.perf_counter()
            ids_o, w_o = S.oracle_router(cfg, l0.cpu().numpy(), None if sel_bias is None else sel_bias.cpu().numpy())
            t_r = time.perf_counter() - t_r
            x_np = x0.to(torch.float32).cpu().numpy()
            want = S.oracle_moe_subset(experts, x_np, ids_o, w_o, fp8_act=act_mode(cfg), threads=threads,
                                       timer=secs.append)
            if shared is not None:
                want = want + S.oracle_moe_subset(shared, x_np, np.zeros((n_chk, 1), np.int64),
                                                  np.ones((n_chk, 1), np.float32), fp8_act=fp8, threads=threads,
                                                  timer=secs.append)
            parity = float(np.linalg.norm(got - want) / np.linalg.norm(want))
            tol = 2e-3 if cfg["fmt"] in ("FP8", "MXFP4") else 1e-3
            if ep is not None:
                tol += 4.5e-3      # partial sums cross the exchange as bf16 rows (two roundings of 2^-9)
            assert parity <= tol, f"GPU layer output differs from the CPU oracle: rel-L2 {parity} > {tol}"
            cpu_s = sum(secs) + t_r
            cpu = {"value": n_chk / cpu_s, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"{n_chk} of the step's {t_local} tokens (evenly spaced) through the router, their "
                             f"{k} routed experts" + (" and the shared expert" if shared is not None else "") +
                             ": dequantize each expert row to f32, f32 dot (the reference's CPU arithmetic); "
                             "host copies of the experts' weights excluded from the time",
                   "seconds": round(cpu_s, 3)}
        except AssertionError:
            raise
        except Exception as exc:  # the checker failing to build must not hide the GPU numbers
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"unavailable: {exc}"}

    gemv = None
    if world == 1 and args.workload == "moe_fp8" and not args.no_gemv and not args.tokens and not args.experts:
        del xs, logits, hx, hl
        torch.cuda.empty_cache()
        g_args = argparse.Namespace(steps=max(20, args.steps), warmup=args.warmup)
        rec = gemv_measure(g_args, torch, dev, rank, world, None, with_cpu=True)
        gemv = {key: rec[key] for key in ("metric", "value", "unit", "ms_per_step", "dtype", "config", "roofline",
                                           "cpu_baseline", "e2e")}

    if rank == 0:
        peaks = load_peaks()
        roof = None
        if gemm_ms is not None:
            ach = moe_flops(cfg, rows_here) / (gemm_ms / 1e3) / 1e12
            e_l, i_ = e // world, cfg["i"]
            roof = {"bound": "tensor", "achieved": round(ach, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": round(ach / peaks["bf16_tflops"], 4), "traffic": None, "peak_kind": peaks["kind"],
                    "peak_note": "measured dense bf16 peak (cuBLAS burst)",
                    "launch_ms_sum": round(gemm_ms, 4), "rows": rows_here,
                    "timing": gemm_timing}
            if fp8:
                wbytes = 3 * e_l * i_ * h
                # algorithmic bytes of the pair: every weight once, activation codes in, intermediate codes out and
                # in again, 16-bit output rows
                abytes = wbytes + rows_here * (h + 2 * i_ + 2 * h) + rows_here * 4 * (h // 128 + 2 * (i_ // 128))
                p8 = probe_fp8_peak(torch, dev)
                roof.update({"kernel": "hq::fp8_grouped_kernel x2 (gate/up fused with SwiGLU + 1x128 quantizer; down)",
                             "fp8_peak_probe_tflops": None if p8 is None else round(p8, 1),
                             "frac_of_fp8_probe": None if not p8 else round(ach / p8, 4),
                             "frac_of_fp8_nominal_4500": round(ach / 4500.0, 4),
                             "algorithmic_bytes": abytes,
                             "hbm_gbs": round(abytes / (gemm_ms / 1e3) / 1e9, 1),
                             "hbm_frac_of_measured": round(abytes / (gemm_ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4),
                             "note": "at 128 rows per expert every weight byte feeds one token tile and every token "
                                     "tile is fetched once per weight tile: ncu shows DRAM at 30 % and the tensor "
                                     "pipe at 24 % while the SMs pull 6.2 TB/s from L2, the ceiling this kernel "
                                     "and a copy-only build of it settle at"})
                if NCU_TRAFFIC_RATIO_FP8 is not None:
                    roof["traffic"] = int(NCU_TRAFFIC_RATIO_FP8 * abytes / 2)
                    roof["traffic_note"] = "per launch: algorithmic bytes x the ncu dram/algorithmic ratio"
            elif mx:
                wbytes = 3 * e_l * i_ * h // 2 + 3 * e_l * i_ * h // 32
                abytes = wbytes + rows_here * (h + 2 * i_ + 2 * h) + rows_here * (h // 32 + 2 * (i_ // 32))
                roof.update({"kernel": "hq::mx_grouped_kernel x2 (gate/up fused with bias + clamped SwiGLU + MXFP8 "
                                       "quantizer; down)",
                             "frac_of_fp8_nominal_4500": round(ach / 4500.0, 4),
                             "algorithmic_bytes": abytes,
                             "hbm_gbs": round(abytes / (gemm_ms / 1e3) / 1e9, 1),
                             "hbm_frac_of_measured": round(abytes / (gemm_ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4),
                             "traffic": int(NCU_TRAFFIC_RATIO_MX * abytes / 2),
                             "traffic_note": "per launch: algorithmic bytes x the ncu dram/algorithmic ratio"})
            else:
                rows_per_expert = rows_here / max(1, e_l)
                ts_k = cfg["fmt"] == "MXFP4" or (cfg["fmt"] == "Q4_K" and rows_per_expert < 192)
                roof["kernel"] = ("hq::grouped_gemm_ts_kernel" if ts_k else "hq::grouped_gemm_kernel") + \
                                 " (gate/up + down)"
                bits = 4.5 if cfg["fmt"] == "Q4_K" else 4.25
                # every weight once, f16 token rows in, f16 intermediate out and in again, f32 rows out
                abytes = int(3 * e_l * i_ * h * bits / 8) + t_local * h * 2 + rows_here * (4 * i_ + 4 * h)
                roof["algorithmic_bytes"] = abytes
                roof["hbm_gbs"] = round(abytes / (gemm_ms / 1e3) / 1e9, 1)
                if cfg["fmt"] == "Q4_K":
                    roof["traffic"] = int(NCU_TRAFFIC_RATIO_Q4K * abytes / 2)
                    roof["traffic_note"] = "per launch: algorithmic bytes x the ncu dram/algorithmic ratio"
        line = {
            "metric": MOE_METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "e4m3" if fp8 else ("e4m3 x e2m1, e8m0 block scales" if mx else "f16"), "data": "synthetic",
            "config": moe_config(cfg, world, "strong" if strong else "weak"),
            "roofline": roof,
            "parity_vs_cpu_oracle_rel_l2": parity,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": t_local * (h * 2 + e * 4),
                    "d2h_bytes_per_step": t_local * h * 2, "ms_per_step": e2e_ms / args.steps,
                    "note": "host-to-device copies, layer and device-to-host copy of neighbouring steps overlap "
                            "(three streams, two buffer sets)"},
            "gpu_launches": args.steps * launches_per_step,
            "launch_mode": graph_note,
            "clocks": clocks,
        }
        if ep is not None:
            d_b, r_b = ep.wire_bytes_per_direction()
            line["exchange"] = {"transport": "all_to_all_single (NCCL)" if ep.exchange == "nccl" or world == 1 else
                                "hq_ep_push into symmetric memory + hq_ep_barrier",
                                "note": exchange_note,
                                "dispatch_bytes_per_rank": d_b, "return_bytes_per_rank": r_b,
                                "rows": "one per (token, destination rank); equal-sized slabs, no host read",
                                "wire": "e4m3 + f32 1x128 scales out, bf16 partial sums back" if fp8 else
                                        "bf16 rows out, bf16 partial sums back"}
        if gemv is not None:
            line["gemv"] = gemv
        print(json.dumps(line), flush=True)
    if dist is not None:
        if graphs is not None:
            # Graphs that hold captured collectives keep the communicator's teardown waiting (it did not return
            # within minutes): every rank finishes its work, meets the others once more and leaves the process
            # without destroying the group.
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)
        dist.destroy_process_group()


# ======================================================================================================
# --impl reference: the CPU restatement of the reference path, all host threads, bounded sample per step
# ======================================================================================================
def run_reference(args):
    world, rank, _ = dist_env()
    if rank != 0:
        return
    import numpy as np
    from oracle import cbuild
    cbuild.build()
    threads = os.cpu_count() or 1
    if args.workload == "gemv":
        ws, xs = gemv_host_data(SHAPES)
        for _ in range(max(1, min(args.warmup, 1))):
            gemv_cpu_step(threads, SHAPES, ws, xs)
        total = sum(gemv_cpu_step(threads, SHAPES, ws, xs) for _ in range(args.steps))
        value = sum(MS) * args.steps / total
        line = {"impl": "reference", "metric": GEMV_METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": gemv_config(),
                "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                                 "sample": "full 16-launch sweep per step"},
                "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return
    from tests import hq_synth as S
    from oracle import moe as M
    cfg = moe_cfg(args)
    fp8 = act_mode(cfg)
    e, k, h, i_ = cfg["e"], cfg["k"], cfg["h"], cfg["i"]
    n_tok = args.cpu_tokens or (2 if cfg["fmt"] == "FP8" else 16)     # tokens per step: a bounded sample of the step
    e_c = min(e, 16)                                                   # experts kept on the host
    rng = np.random.Generator(np.random.PCG64(4004))

    def host_bank(n, kk, count):
        """Random valid block bytes of the layer's format (the CPU arithmetic per weight does not depend on the
        values), with scales of the magnitude N(0, 0.02^2) weights give."""
        if cfg["fmt"] == "FP8":
            codes = rng.integers(0, 256, (count, n, kk), dtype=np.uint8)
            codes[(codes & 0x7F) == 0x7F] = 0x38                       # no NaN codes
            return ("FP8", codes, np.full((count, n // 128, kk // 128), 1.6e-4, np.float32), None)
        if cfg["fmt"] == "MXFP4":
            return ("MXFP4", rng.integers(0, 256, (count, n, kk // 2), dtype=np.uint8),
                    np.full((count, n, kk // 32), 120, np.uint8), np.zeros((count, n), np.float32))
        raw = rng.integers(0, 256, (count, n, kk // 256, 144), dtype=np.uint8)
        raw[..., 0:2] = np.frombuffer(np.float16(2e-4).tobytes(), np.uint8)
        raw[..., 2:4] = np.frombuffer(np.float16(2e-4).tobytes(), np.uint8)
        return ("Q4_K", raw.reshape(count, n, -1), None, None)

    def layer(count):
        if cfg["inter"]:
            return [host_bank(2 * i_, h, count)], host_bank(h, i_, count)
        return [host_bank(i_, h, count), host_bank(i_, h, count)], host_bank(h, i_, count)

    first, down = layer(e_c)
    sh = layer(1) if cfg.get("shared") else None
    act = (M.ACT_GPTOSS, 1, 7.0, 1.702) if cfg["inter"] else (M.ACT_SWIGLU, 0, 0.0, 1.702)
    sel_bias = (rng.standard_normal(e) * 0.01).astype(np.float32) if cfg["router"] == "sigmoid_bias" else None

    def one_step():
        x = rng.standard_normal((n_tok, h)).astype(np.float32)
        lg = rng.standard_normal((n_tok, e)).astype(np.float32)
        t0 = time.perf_counter()
        ids, w = S.oracle_router(cfg, lg, sel_bias)
        ids_c = (ids.astype(np.int64) % e_c)
        out = S.oracle_moe_host(first, down, e_c, act, x, ids_c, w, fp8_act=fp8, threads=threads)
        if sh is not None:
            out = out + S.oracle_moe_host(sh[0], sh[1], 1, act, x, np.zeros((n_tok, 1), np.int64),
                                          np.ones((n_tok, 1), np.float32), fp8_act=fp8, threads=threads)
        return time.perf_counter() - t0

    for _ in range(max(1, min(args.warmup, 2))):
        one_step()
    steps = args.steps
    total = sum(one_step() for _ in range(steps))
    value = n_tok * steps / total
    strong = args.ep_scaling == "strong"
    line = {"impl": "reference", "metric": MOE_METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / steps, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": moe_config(cfg, max(1, args.gpus), "strong" if strong else "weak"),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"{n_tok} tokens per step through the router, {k} routed experts" +
                                       (" and the shared expert" if sh is not None else "") +
                                       f" (expert ids folded onto {e_c} host-resident experts of the layer's shape): "
                                       "dequantize each expert row to f32, f32 dot; the Rust reference cannot be "
                                       "built here (no Rust toolchain)"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="moe_fp8",
                    choices=["gemv", "moe_q4k", "moe_fp8", "moe_mxfp4", "decode_formats"])
    ap.add_argument("--formats", default="", help="decode_formats: comma-separated weight formats (default: all)")
    ap.add_argument("--rows", type=int, default=65536, help="decode_formats: output rows of the 4096 -> rows matrix")
    ap.add_argument("--reps", type=int, default=8, help="decode_formats: timed launches per format and row count")
    ap.add_argument("--m", default="1,4", help="decode_formats: activation row counts")
    ap.add_argument("--tokens", type=int, default=0, help="override the global token count of a MoE workload")
    ap.add_argument("--profiler-range", action="store_true",
                    help="MoE workloads: bracket the timed steps with cudaProfilerStart/Stop, so that a profiler "
                         "started with --profile-from-start off sees the timed steps only")
    ap.add_argument("--exchange", default="p2p", choices=["nccl", "p2p"],
                    help="expert-parallel exchange: two NCCL all-to-alls, or stores into the peers' symmetric-memory "
                         "buffers by this library's own kernels followed by a flag barrier")
    ap.add_argument("--force-ep", action="store_true",
                    help="MoE workloads on one GPU: go through the expert-parallel pack / unpack / reduce kernels "
                         "anyway (the exchange degenerates to a local hand-over); profiling aid")
    ap.add_argument("--no-graph", action="store_true",
                    help="MoE workloads: launch every step eagerly instead of replaying a CUDA graph of it")
    ap.add_argument("--act16", action="store_true",
                    help="MoE workloads: 16-bit activations (mode A) instead of the quantized-activation path")
    ap.add_argument("--experts", type=int, default=0, help="override the expert count of a MoE workload")
    ap.add_argument("--ep-scaling", default="strong", choices=["weak", "strong"],
                    help="MoE workloads on several GPUs: global token count split (strong) or tokens per GPU fixed")
    ap.add_argument("--cpu-tokens", type=int, default=0, help="tokens of the CPU-oracle sample")
    ap.add_argument("--no-gemv", action="store_true", help="leave the decode mat-vec record out of the default line")
    ap.add_argument("--only", default=None, help="restrict the mat-vec sweep to one KxN shape, e.g. 4096x128256 "
                    "(profiling aid; the reported line is then not the headline workload)")
    args = ap.parse_args()
    if args.only:
        k, n = (int(v) for v in args.only.lower().split("x"))
        global SHAPES
        SHAPES = [(k, n)]
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload == "gemv":
        run_gemv(args)
        return
    if args.workload == "decode_formats":
        # profiling aid, one GPU: the decode mat-vec record of the default line alone
        import torch
        dev = torch.device("cuda:0")
        torch.cuda.set_device(dev)
        peak = load_peaks()["hbm_gbs"]
        kw = {"formats": tuple(args.formats.split(","))} if args.formats else {}
        print(json.dumps({"workload": "decode_formats", "peak_gbs": peak,
                          "decode": decode_other_formats(torch, dev, peak, n=args.rows, reps=args.reps,
                                                         ms=tuple(int(v) for v in args.m.split(",")), **kw)}))
        return
    run_moe(args)


if __name__ == "__main__":
    main()
