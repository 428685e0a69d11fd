#!/usr/bin/env python
"""Benchmark of the quantized-weight MatMul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-sweep]

Workload (config.workload): the I8 sweep configuration -- I8 per-channel weights, K=4096, N=11008,
f32 activations [M,4096], fused SiLU -- at M=1, the HBM-bound point the metric is quoted on.
A step is one pass of that layer over one activation batch.  Weights rotate over replicas
whose total size exceeds the 126 MB L2, so every step streams its weights from HBM.

  value     algorithmic GB/s with inputs resident in HBM (CUDA events around K steps)
  e2e       the same through the public API with host buffers: pinned H2D of the
            activations and D2H of the result inside every timed step
  roofline  algorithmic bytes per launch / average launch time vs the measured HBM peak
  sweep     the other (format, M) points of the metric, same method (not the headline); every point
            is first checked against the CPU oracle on slices of its output (parity_err)

With --gpus N > 1 (launched by torchrun, one rank per GPU) every rank holds an 11008-column
shard of an [4096, 11008*N] layer, activations are replicated and each step is one kernel per
rank: the shard's GEMV stores its outputs into every rank's gathered buffer over NVLink peer
memory and waits for the peers' shards.  Weak scaling, value = bytes all ranks streamed /
max-over-ranks time.  At every N the line also carries the two configurations that name several
GPUs: `strong_c3_f8_m1` (the FP8 K=8192 N=28672 layer at one batch row with its columns split over
the ranks) and `c5_chain` (32 layers of the decoder-shaped I4 projection set at 64 batch rows, every
projection column-sharded, outputs gathered by the GEMM's own peer stores).

--impl reference times the reference's CPU algorithm (the oracle port) on the host cores.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K_DIM, N_DIM, M_HEAD = 4096, 11008, 1
SIGMA = 0.02
L2_BYTES = 126 * 1000 * 1000
METRIC = "quant_matmul_i8_m1_hbm_gbs"
UNIT = "GB/s"
WORKLOAD = ("config2: I8 per-channel weights K=4096 N=11008 per GPU, f32 activations [1,4096], "
            "fused SiLU")


def algorithmic_bytes(fmt_bits: int, n: int, k: int, m: int, n_scales_bytes: int, bias: bool) -> int:
    """W + S + 4*M*K + 4*M*N (+ 4*N bias): packed weights, scale/zero arrays, f32
    activations in, f32 outputs out."""
    return n * k * fmt_bits // 8 + n_scales_bytes + 4 * m * k + 4 * m * n + (4 * n if bias else 0)


def philox_normal(seed, shape, sigma):
    rng = np.random.Generator(np.random.Philox(seed))
    return rng.standard_normal(shape, dtype=np.float32) * np.float32(sigma)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock/throttle samples while the GPU is under the benchmark's load."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.lines:
            if ts < t0 or ts > t1 + 0.15:
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(np.max(mx)) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm),
                "window": "warm-up + timed steps + untimed replay of the same kernel to >=1.5 s"}


# ------------------------------------------------------------------------------ ours


class Layer:
    """R device replicas of one quantized weight plus an arena with activation/output slots."""

    def __init__(self, backend, fnn, fmt, w_kn, m, bias=None, min_total_bytes=3 * L2_BYTES, quantized=None,
                 shard=None):
        """shard = (rank, world): keep this rank's contiguous range of output columns only (quantize
        the whole layer first, then slice the packed rows: the bytes of the unsharded weight)."""
        from fastnn_b200 import _lib as L
        self.fnn, self.L, self.backend, self.fmt, self.m = fnn, L, backend, fmt, m
        k, n = w_kn.shape
        self.quantized = quantized or fnn.quantize_weight_constant(w_kn, fmt)   # reused across batch sizes
        packed, scales, zeros, cb = self.quantized
        zp = zeros if fmt in (L.FMT_I8, L.FMT_I4, L.FMT_F4) else np.zeros(0, np.float32)
        meta = fnn.QuantizedWeightMeta(
            bit_width=8 if fmt in (L.FMT_I8, L.FMT_F8) else 4, scales=scales, zero_points=zp,
            shape=[n, k], quant_block_size=32 if fmt == L.FMT_I4CB else 0,
            codebooks=[cb] if fmt == L.FMT_I4CB else [], fmt=fmt)
        payload = packed.tobytes()
        if shard is not None:
            from fastnn_b200.parallel import shard_rows
            payload, meta = shard_rows(payload, meta, shard[0], shard[1])
            n = meta.shape[0]
            scales, zp = meta.scales, meta.zero_points
        self.k, self.n = k, n
        self.meta, self.payload = meta, payload
        self.words, self.scales, self.zp, self.cb = np.frombuffer(self.payload, np.uint32), scales, zp, cb
        self.bias = bias
        bits = 8 if fmt in (L.FMT_I8, L.FMT_F8) else 4
        wbytes = n * k * bits // 8
        self.replicas = max(2, -(-min_total_bytes // wbytes))
        self.weights = [backend.upload_qweight(self.payload, meta) for _ in range(self.replicas)]
        sbytes = scales.nbytes + (zp.nbytes if zp.size else 0) + (64 if fmt == L.FMT_I4CB else 0)
        self.alg_bytes = algorithmic_bytes(bits, n, k, m, sbytes, bias is not None)
        self.flops = 2 * m * k * n
        al = lambda x: -(-x // 256) * 256
        self.a_off, self.out_off = 0, al(m * k * 4)
        self.bias_off = self.out_off + al(m * n * 4)
        self.arena = backend.allocate_arena(self.bias_off + al(n * 4))
        self.has_bias = bias is not None
        if bias is not None:
            backend.write_arena(self.arena, self.bias_off, bias.tobytes())

    def set_activations(self, x):
        self.backend.write_arena(self.arena, self.a_off, np.ascontiguousarray(x, np.float32).tobytes())

    def launch(self, i, epi, path=0):
        b = self.backend
        rc = b.lib.fnn_cuda_qmatmul(b.ctx, self.weights[i % self.replicas].handle, self.arena.handle,
                                    self.a_off, self.out_off, self.bias_off if self.has_bias else -1,
                                    self.m, epi, path)
        if rc != 0:
            raise self.fnn.BackendError.from_status(rc)

    def output(self):
        raw = self.backend.read_arena(self.arena, self.out_off, self.m * self.n * 4)
        return np.frombuffer(raw, np.float32).reshape(self.m, self.n)

    def parity_err(self, epi, path=0, max_rows=64, width=64):
        """One launch on fresh activations, checked against the CPU oracle on three slices of output
        channels (first, middle, last `width`) and at most `max_rows` batch rows: max |err| / rms."""
        import oracle as orc   # the checker: never inside a timed region
        L, n, k, m = self.L, self.n, self.k, self.m
        x = philox_normal(4242 + m, (m, k), 1.0)
        self.set_activations(x)
        self.launch(0, epi, path)
        got = self.output()
        width = min(width, n)
        mid = (n // 2) // 16 * 16 + (8 if n >= 4 * width else 0)
        rows = np.unique(np.concatenate([np.arange(0, width), np.arange(mid, min(mid + width, n)),
                                         np.arange(n - width, n)]))
        ms = np.arange(m) if m <= max_rows else np.arange(0, m, m // max_rows)[:max_rows]
        wpr = -(-k // (4 if self.fmt in (L.FMT_I8, L.FMT_F8) else 8))
        sub_words = np.concatenate([self.words[: n * wpr].reshape(n, wpr)[rows].reshape(-1),
                                    np.zeros(16, np.uint32)])
        if self.fmt == L.FMT_I4CB:
            bpr = -(-k // 32)
            sub = orc.QWeight(self.fmt, len(rows), k, sub_words,
                              self.scales.reshape(n, bpr)[rows].reshape(-1).copy(), np.zeros(0, np.float32),
                              self.cb, 32)
        else:
            sub = orc.QWeight(self.fmt, len(rows), k, sub_words, self.scales[rows].copy(),
                              self.zp[rows].copy() if self.zp.size else np.zeros(0, np.float32))
        want = orc.qmatmul(sub, x[ms], self.bias[rows] if self.has_bias else None, epi).astype(np.float64)
        err = np.max(np.abs(got[np.ix_(ms, rows)] - want)) / max(np.sqrt(np.mean(want ** 2)), 1e-30)
        return float(err)

    def time_isolated(self, steps, epi, path=0):
        """Per-launch time with programmatic dependent launch off: the same graph replay over the
        rotating weight replicas, but every kernel starts only after the one before it has
        finished, so no launch overlaps its neighbour's tail.  Returns ms per launch."""
        lib, b = self.backend.lib, self.backend
        check(lib.fnn_cuda_ctx_set_overlap(b.ctx, 0), self.fnn)
        try:
            return self.time_steps(steps, 3, epi, path) / steps
        finally:
            check(lib.fnn_cuda_ctx_set_overlap(b.ctx, 1), self.fnn)

    def time_steps(self, steps, warmup, epi, path=0, min_seconds=0.0):
        """CUDA-event time of `steps` launches replayed from one captured graph."""
        b, lib = self.backend, self.backend.lib
        for i in range(max(warmup, 1)):
            self.launch(i, epi, path)
        b.synchronize()
        check(lib.fnn_cuda_graph_begin(b.ctx), self.fnn)
        for i in range(steps):
            self.launch(i, epi, path)
        g = ctypes.c_void_p()
        check(lib.fnn_cuda_graph_end(b.ctx, ctypes.byref(g)), self.fnn)
        check(lib.fnn_cuda_graph_launch(b.ctx, g), self.fnn)  # graph warm-up (upload)
        b.synchronize()
        ms = ctypes.c_float()
        check(lib.fnn_cuda_timer_start(b.ctx, 0), self.fnn)
        check(lib.fnn_cuda_graph_launch(b.ctx, g), self.fnn)
        check(lib.fnn_cuda_timer_stop(b.ctx, 0), self.fnn)
        check(lib.fnn_cuda_timer_elapsed_ms(b.ctx, 0, ctypes.byref(ms)), self.fnn)
        t_end = time.time() + min_seconds
        while time.time() < t_end:  # untimed: keeps the same load up for the clock sampler
            check(lib.fnn_cuda_graph_launch(b.ctx, g), self.fnn)
            b.synchronize()
        lib.fnn_cuda_graph_free(g)
        return float(ms.value)

    def close(self):
        for w in self.weights:
            w.close()
        self.arena.close()


def check(rc, fnn):
    if rc != 0:
        raise fnn.BackendError.from_status(rc)


def run_e2e(fnn, backend, w_kn, steps, warmup):
    """Public API, host buffers: AotExecutor.forward_pinned() = pinned H2D of x, the plan,
    D2H of y, synchronize -- every step.  Executors rotate so weights still exceed L2."""
    nodes = [{"op_type": "MatMul", "inputs": "[x, w]", "outputs": "[h]"},
             {"op_type": "Silu", "inputs": "[h]", "outputs": "[y]"}]
    n_exec = max(2, -(-3 * L2_BYTES // (K_DIM * N_DIM)))
    execs = [fnn.AotExecutor(nodes, {"w": w_kn}, ["x"], ["y"], {"x": [M_HEAD, K_DIM]}, quantize=8,
                             backend=backend) for _ in range(n_exec)]
    xs = [philox_normal(100 + i, (M_HEAD, K_DIM), 1.0) for i in range(8)]
    for e in execs:
        e.forward({"x": xs[0]})  # first call materialises constants and captures the replay
        e.bind_pinned()
    for i in range(max(warmup, 3)):
        e = execs[i % n_exec]
        e.pinned_inputs["x"][...] = xs[i % 8]
        e.forward_pinned()
    launches0 = backend.launch_count()
    t0 = time.perf_counter()
    acc = 0.0
    for i in range(steps):
        e = execs[i % n_exec]
        e.pinned_inputs["x"][...] = xs[i % 8]          # the step's input arrives in host memory
        y = e.forward_pinned()["y"]
        acc += float(y[0, 0])                           # the result is read on the host
    dt = time.perf_counter() - t0
    launches = backend.launch_count() - launches0
    return dt / steps, launches, M_HEAD * K_DIM * 4, M_HEAD * N_DIM * 4, acc


def cpu_baseline(w_kn, budget_s=12.0, max_iters=50):
    """The oracle's restatement of gemm_batch_packed_simd, timed on this host."""
    import oracle as orc
    q = orc.quantize_kn(orc.FMT_I8, w_kn)
    x = philox_normal(1, (M_HEAD, K_DIM), 1.0)
    orc.qmatmul(q, x, None, orc.EPI_SILU)
    times, t_all = [], time.perf_counter()
    while len(times) < max_iters and time.perf_counter() - t_all < budget_s:
        t = time.perf_counter()
        orc.qmatmul(q, x, None, orc.EPI_SILU)
        times.append(time.perf_counter() - t)
    info = orc.host_info()
    cores = info["physical_cores"] if M_HEAD >= info["physical_cores"] else 1
    return float(np.median(times)), len(times), cores, info


def sweep_points(L):
    return [  # label, fmt, K, N, Ms, sigma, epilogue, bias
        ("c2_i8", L.FMT_I8, 4096, 11008, (1, 4, 16, 128, 512), 0.02, L.EPI_SILU, False),
        ("c1_i4", L.FMT_I4, 4096, 4096, (1, 8), 0.02, L.EPI_NONE, True),
        ("c3_i4", L.FMT_I4, 8192, 28672, (1,), 0.015, L.EPI_NONE, False),
        ("c3_f8", L.FMT_F8, 8192, 28672, (1, 32, 512, 4096), 0.015, L.EPI_NONE, False),
        ("c3_f4", L.FMT_F4, 8192, 28672, (1, 32, 512, 4096), 0.015, L.EPI_NONE, False),
        ("c4_i4cb_up", L.FMT_I4CB, 2048, 8192, (1, 64), 0.02, L.EPI_GELU, True),
        ("c4_i4cb_down", L.FMT_I4CB, 8192, 2048, (64,), 0.02, L.EPI_NONE, True),
        ("i4cb_8192x8192", L.FMT_I4CB, 8192, 8192, (1,), 0.02, L.EPI_NONE, False),
        ("c5_i4_gateup", L.FMT_I4, 4096, 28672, (64,), 0.02, L.EPI_NONE, False),
        ("c5_i4_down", L.FMT_I4, 14336, 4096, (64,), 0.02, L.EPI_NONE, False),
        ("c5_i4_qkv", L.FMT_I4, 4096, 6144, (64,), 0.02, L.EPI_NONE, False),
    ]


def run_sweep(fnn, backend, peaks, budget_s=420.0, only=None, only_m=None, steps_override=None,
              path=0):
    from fastnn_b200 import _lib as L
    out, t_start = [], time.time()
    cache = {}
    for label, fmt, k, n, ms, sigma, epi, has_bias in sweep_points(L):
        if only is not None:
            if label != only:
                continue
            ms = tuple(m for m in ms if only_m is None or m == only_m) or (only_m,)
        if time.time() - t_start > budget_s:
            out.append({"point": label, "skipped": "sweep time budget"})
            continue
        key = (k, n, sigma)
        if key not in cache:
            cache.clear()
            cache[key] = philox_normal(7, (k, n), sigma)
        w = cache[key]
        bias = philox_normal(8, (n,), 0.01) if has_bias else None
        quantized = None
        for m in ms:
            layer = Layer(backend, fnn, fmt, w, m, bias, quantized=quantized)
            quantized = layer.quantized
            try:
                err = layer.parity_err(epi, path)       # checked before it is timed
                layer.set_activations(philox_normal(9, (m, k), 1.0))
                est = max(layer.alg_bytes / 3e12, layer.flops / 2e13)
                steps = steps_override or int(min(200, max(5, 0.05 / est)))
                ms_total = layer.time_steps(steps, 3, epi, path)
                t = ms_total / steps * 1e-3
                iso = layer.time_isolated(steps, epi, path)
                gbs, tfs = layer.alg_bytes / t / 1e9, layer.flops / t / 1e12
                out.append({"point": label, "m": m, "k": k, "n": n, "path": backend.last_path(),
                            "us": round(t * 1e6, 2), "isolated_us": round(iso * 1e3, 2),
                            "gbs": round(gbs, 1), "tflops": round(tfs, 2),
                            "hbm_frac": round(gbs / peaks["hbm_gbs"], 3),
                            "tensor_frac_bf16": round(tfs / peaks["bf16_tflops"], 3),
                            "parity_err": float(f"{err:.3g}")})
            finally:
                layer.close()
    return out


def run_ours(args):
    import torch
    import fastnn_b200 as fnn
    from fastnn_b200 import _lib as L

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    backend = fnn.CudaBackend(local)   # its own non-blocking stream: CUDA graphs are captured on it
    peaks = load_peaks()
    if args.only:  # one sweep point only (profiling aid): prints that point and exits
        pts = run_sweep(fnn, backend, peaks, only=args.only, only_m=args.only_m,
                        steps_override=args.steps, path=args.path)
        print(json.dumps({"sweep": pts}), flush=True)
        backend.close()
        return

    # every rank owns an 11008-column shard (seeded by rank) of the [4096, 11008*world] layer
    w_kn = philox_normal(1000 + rank, (K_DIM, N_DIM), SIGMA)
    layer = Layer(backend, fnn, L.FMT_I8, w_kn, M_HEAD)
    head_err = layer.parity_err(L.EPI_SILU)      # the timed kernel's output against the CPU oracle
    layer.set_activations(philox_normal(1, (M_HEAD, K_DIM), 1.0))

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t_load0 = time.time()
    launches0 = backend.launch_count()
    if world == 1:
        ms_total = layer.time_steps(args.steps, args.warmup, L.EPI_SILU, min_seconds=1.5)
        launches = args.steps
    else:
        ms_total, e2e_n = time_sharded(torch, dist, backend, layer, args, world, L)
        launches = args.steps + 1 + e2e_n["launches"]
    t_load1 = time.time()
    clocks = sampler.stop(t_load0, t_load1) if rank == 0 else None
    del launches0

    if world > 1:
        t = torch.tensor([ms_total, e2e_n["s_per_step"]], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, e2e_n["s_per_step"] = float(t[0].item()), float(t[1].item())
    per_step_s = ms_total / args.steps * 1e-3
    total_bytes = layer.alg_bytes * world
    value = total_bytes / per_step_s / 1e9
    path = backend.last_path()

    line = None
    if rank == 0:
        achieved = layer.alg_bytes / per_step_s / 1e9
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(per_step_s * 1e3, 6),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "m": M_HEAD, "k": K_DIM, "n_per_gpu": N_DIM, "format": "i8",
                       "kernel_path": path, "parity_err": float(f"{head_err:.3g}"),
                       "l2": f"weights rotate over {layer.replicas} replicas "
                             f"({layer.replicas * K_DIM * N_DIM // 1000000} MB > 126 MB L2)",
                       "parallelism": "single GPU" if world == 1 else
                                      f"column-sharded x{world}; outputs all-gathered by the GEMV's own "
                                      "peer stores over NVLink (no collective call)",
                       "algorithmic_bytes_per_step_per_gpu": layer.alg_bytes},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                         "traffic": NCU_TRAFFIC.get(("i8", K_DIM, N_DIM, M_HEAD), {}).get("bytes"),
                         "traffic_source": NCU_TRAFFIC.get(("i8", K_DIM, N_DIM, M_HEAD), {}).get("source"),
                         "peak_source": peaks["source"]},
            "clocks": clocks, "gpu_launches": launches,
        }
    if world == 1:
        iso_ms = layer.time_isolated(min(args.steps, 500), L.EPI_SILU)
        line["isolated_us"] = round(iso_ms * 1e3, 2)
        line["roofline"]["isolated_frac"] = round(layer.alg_bytes / (iso_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
        line["roofline"]["note"] = ("achieved/frac: back-to-back replay of one CUDA graph (the next launch's "
                                    "weight prefetch overlaps this one's tail); isolated_frac: one launch alone "
                                    "on the stream after an L2 flush")
        e2e_s, e2e_launches, h2d, d2h, _ = run_e2e(fnn, backend, w_kn, min(args.steps, 2000),
                                                   args.warmup)
        line["e2e"] = {"value": round(layer.alg_bytes / e2e_s / 1e9, 1), "unit": UNIT,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "us_per_step": round(e2e_s * 1e6, 2),
                       "api": "AotExecutor.forward_pinned (pinned H2D + plan + D2H + sync per step)"}
        line["gpu_launches"] = launches + e2e_launches
        t_med, iters, cores, info = cpu_baseline(w_kn)
        line["cpu_baseline"] = {
            "value": round(layer.alg_bytes / t_med / 1e9, 3), "unit": UNIT, "cores": cores,
            "kind": "port",
            "sample": f"the full M=1 layer, median of {iters} calls ({t_med * 1e3:.1f} ms each); "
                      f"single-threaded as the reference is for M < cores; simd_level="
                      f"{info['simd_level']}, k_tile={info['k_block_size']}"}
        if not args.no_sweep:
            line["sweep"] = run_sweep(fnn, backend, peaks)
    else:
        if rank == 0:
            line["e2e"] = {"value": round(total_bytes / e2e_n["s_per_step"] / 1e9, 1), "unit": UNIT,
                           "h2d_bytes_per_step": e2e_n["h2d"] * world, "d2h_bytes_per_step": e2e_n["d2h"] * world,
                           "us_per_step": round(e2e_n["s_per_step"] * 1e6, 2),
                           "api": "per rank and step one graph launch: pinned H2D of the activations, "
                                  "fnn_cuda_qmatmul_gather, fnn_cuda_gather_wait (unpack), pinned D2H of the "
                                  "gathered rows, synchronize"}
    layer.close()
    if not args.no_multi:
        # the multi-GPU configurations, at every N (N = 1 gives the base of each curve)
        strong = strong_scaling_c3(fnn, backend, rank, world, dist, peaks)
        chain = c5_chain(fnn, backend, rank, world, dist)
        if rank == 0:
            line["strong_c3_f8_m1"] = strong
            line["c5_chain"] = chain
            line["gpu_launches"] += 100 + 3 * 32 * chain["launches_per_layer"]
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    backend.close()


# dram__bytes_read.sum + dram__bytes_write.sum of one launch, keyed by (format, K, N, M), from ncu
# captures of `python bench.py --only <point> --only-m <M>`; `source` names the kernel and the date
# of the capture.  A point without an entry reports null.
NCU_TRAFFIC = {
    ("i8", 4096, 11008, 1): {"bytes": 45234432,
                             "source": "qmm_mma8_kernel (444 blocks of 256 threads), ncu --set full: 45.231872 MB read + 2.56 KB "
                                       "written per launch (profiles/qmm_mma8_i8_m1_config2.md)"},
}


def time_sharded(torch, dist, backend, layer, args, world, L):
    """N > 1: every step is ONE kernel per rank -- the shard's GEMV whose epilogue stores its columns
    into every rank's gathered buffer over NVLink peer memory as {value, step} words and which first
    checks that the previous step has arrived from every peer (fnn_cuda_qmatmul_gather), replayed from
    a CUDA graph that ends with fnn_cuda_gather_wait for the last step.  Barrier + synchronize on both
    sides; CUDA events on the launching stream; the caller takes the max over ranks.  Returns the
    device time in ms and the end-to-end (host buffers) measurement."""
    import ctypes
    rank = dist.get_rank()
    lib = backend.lib
    # one shared arena (gather buffers + flags); the layer's weight replicas rotate underneath it
    fused = FusedGatherLinearReplicas(backend, layer, rank, world, L.EPI_SILU)
    fused.set_activations(philox_normal(1, (layer.m, layer.k), 1.0))
    for i in range(max(args.warmup, 3)):
        fused.forward(i)
    backend.synchronize()
    dist.barrier()
    check(lib.fnn_cuda_graph_begin(backend.ctx), layer.fnn)
    for i in range(args.steps):
        fused.forward(i)
    fused.wait()   # the timed region ends only when the last step's shards have arrived from every peer
    g = ctypes.c_void_p()
    check(lib.fnn_cuda_graph_end(backend.ctx, ctypes.byref(g)), layer.fnn)
    check(lib.fnn_cuda_graph_launch(backend.ctx, g), layer.fnn)   # graph warm-up on every rank
    backend.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    ms = ctypes.c_float()
    check(lib.fnn_cuda_timer_start(backend.ctx, 0), layer.fnn)
    check(lib.fnn_cuda_graph_launch(backend.ctx, g), layer.fnn)
    check(lib.fnn_cuda_timer_stop(backend.ctx, 0), layer.fnn)
    check(lib.fnn_cuda_timer_elapsed_ms(backend.ctx, 0, ctypes.byref(ms)), layer.fnn)
    backend.synchronize()
    dist.barrier()
    t_end = time.time() + 1.5
    while time.time() < t_end:   # untimed: same load for the clock sampler, in lock step on all ranks
        check(lib.fnn_cuda_graph_launch(backend.ctx, g), layer.fnn)
        backend.synchronize()
        flag = torch.tensor([1 if time.time() < t_end else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            break
    lib.fnn_cuda_graph_free(g)
    # end to end at N ranks: every step goes host -> device -> all ranks -> host (wall clock, barrier
    # on both sides, max over ranks by the caller)
    fused.bind_pinned()
    xs = [philox_normal(100 + i, (layer.m, layer.k), 1.0) for i in range(8)]
    e2e_steps = min(args.steps, 2000)
    for i in range(max(args.warmup, 3)):
        fused.x_host[...] = xs[i % 8].ravel()
        fused.step_pinned(i)
    dist.barrier()
    t0 = time.perf_counter()
    acc = 0.0
    for i in range(e2e_steps):
        fused.x_host[...] = xs[i % 8].ravel()
        acc += float(fused.step_pinned(i)[0])
    dist.barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e = {"s_per_step": e2e_s, "steps": e2e_steps, "h2d": layer.m * layer.k * 4, "d2h": fused.plain_bytes,
           "launches": 2 * e2e_steps}
    fused.close()
    return float(ms.value), e2e


class FusedGatherLinearReplicas:
    """bench-side driver of fnn_cuda_qmatmul_gather over the Layer's rotating weight replicas."""

    def __init__(self, backend, layer, rank, world, epilogue):
        from fastnn_b200.parallel import PeerArena
        self.backend, self.layer, self.rank, self.world, self.epilogue = backend, layer, rank, world, epilogue
        self.n_stride = -(-layer.n // 4) * 4
        word_bytes = 2 * world * 4 * self.n_stride * 8      # {value, step} words, two slots of 4 rows
        self.counter_off = -(-word_bytes // 256) * 256
        self.plain_off = self.counter_off + 256           # f32 [world][m][n_stride] written by wait()
        self.plain_bytes = world * layer.m * self.n_stride * 4
        self.a_off = self.plain_off + -(-self.plain_bytes // 256) * 256
        self.pa = PeerArena(backend, self.a_off + layer.m * layer.k * 4, rank, world)
        self.arena, self.peers = self.pa.arena, self.pa.peers
        self.graphs, self.pinned = [], []

    def set_activations(self, x):
        self.backend.write_arena(self.arena, self.a_off, np.ascontiguousarray(x, np.float32).tobytes())

    def forward(self, i):
        layer, b = self.layer, self.backend
        rc = b.lib.fnn_cuda_qmatmul_gather(
            b.ctx, layer.weights[i % layer.replicas].handle, self.arena.device_ptr + self.a_off, None,
            layer.m, self.epilogue, self.rank, self.world, self.peers, 0, self.counter_off, self.n_stride)
        check(rc, layer.fnn)

    def wait(self, unpack=False):
        out = self.arena.device_ptr + self.plain_off if unpack else None
        check(self.backend.lib.fnn_cuda_gather_wait(self.backend.ctx, self.arena.device_ptr, 0, self.counter_off,
                                                    self.world, self.n_stride, out), self.layer.fnn)

    def bind_pinned(self):
        """Host-to-host step per weight replica as one captured graph: pinned H2D of the activations,
        the fused GEMV + gather, the consumer-side poll that unpacks the gathered rows, pinned D2H."""
        import ctypes
        lib, b, layer = self.backend.lib, self.backend, self.layer

        def pinned(nbytes):
            p = ctypes.c_void_p()
            check(lib.fnn_cuda_host_alloc(nbytes, ctypes.byref(p)), layer.fnn)
            self.pinned.append(p.value)
            return p.value, np.ctypeslib.as_array((ctypes.c_float * (nbytes // 4)).from_address(p.value))

        self.x_ptr, self.x_host = pinned(layer.m * layer.k * 4)
        self.y_ptr, self.y_host = pinned(self.plain_bytes)
        for i in range(layer.replicas):
            check(lib.fnn_cuda_graph_begin(b.ctx), layer.fnn)
            check(lib.fnn_cuda_arena_write_async(self.arena.handle, self.a_off, self.x_ptr, layer.m * layer.k * 4),
                  layer.fnn)
            self.forward(i)
            self.wait(unpack=True)
            check(lib.fnn_cuda_arena_read_async(self.arena.handle, self.plain_off, self.y_ptr, self.plain_bytes),
                  layer.fnn)
            g = ctypes.c_void_p()
            check(lib.fnn_cuda_graph_end(b.ctx, ctypes.byref(g)), layer.fnn)
            self.graphs.append(g)

    def step_pinned(self, i):
        check(self.backend.lib.fnn_cuda_graph_launch(self.backend.ctx, self.graphs[i % len(self.graphs)]),
              self.layer.fnn)
        self.backend.synchronize()
        return self.y_host

    def close(self):
        self.backend.synchronize()
        for g in self.graphs:
            self.backend.lib.fnn_cuda_graph_free(g)
        for ptr in self.pinned:
            self.backend.lib.fnn_cuda_host_free(ptr)
        self.pa.close()


def max_over_ranks(dist, value):
    if dist is None:
        return value
    import torch
    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sync_ranks(backend, dist):
    backend.synchronize()
    if dist is not None:
        import torch
        dist.barrier()
        torch.cuda.synchronize()


def time_graph(backend, fnn, enqueue, dist):
    """Capture `enqueue()` once, replay it once untimed, then time one replay between barriers with
    CUDA events on the launching stream; max over ranks.  Returns milliseconds."""
    lib = backend.lib
    sync_ranks(backend, dist)
    check(lib.fnn_cuda_graph_begin(backend.ctx), fnn)
    enqueue()
    g = ctypes.c_void_p()
    check(lib.fnn_cuda_graph_end(backend.ctx, ctypes.byref(g)), fnn)
    check(lib.fnn_cuda_graph_launch(backend.ctx, g), fnn)
    sync_ranks(backend, dist)
    ms = ctypes.c_float()
    check(lib.fnn_cuda_timer_start(backend.ctx, 2), fnn)
    check(lib.fnn_cuda_graph_launch(backend.ctx, g), fnn)
    check(lib.fnn_cuda_timer_stop(backend.ctx, 2), fnn)
    check(lib.fnn_cuda_timer_elapsed_ms(backend.ctx, 2, ctypes.byref(ms)), fnn)
    sync_ranks(backend, dist)
    lib.fnn_cuda_graph_free(g)
    return max_over_ranks(dist, float(ms.value))


def strong_scaling_c3(fnn, backend, rank, world, dist, peaks, steps=100):
    """The Llama-style FFN layer of the FP8 configuration, K=8192, N=28672, at one batch row, its
    output columns split over the ranks (strong scaling): every step is one fused GEMV + all-gather
    kernel per rank.  Rank 0 checks the gathered row against the CPU oracle on column slices of
    every rank's shard."""
    from fastnn_b200 import _lib as L
    k, n = 8192, 28672
    w = philox_normal(7, (k, n), 0.015)
    layer = Layer(backend, fnn, L.FMT_F8, w, 1, shard=(rank, world))
    fused = FusedGatherLinearReplicas(backend, layer, rank, world, L.EPI_NONE)
    x = philox_normal(11, (1, k), 1.0)
    fused.set_activations(x)
    fused.forward(0)
    fused.wait(unpack=True)
    backend.synchronize()
    raw = backend.read_arena(fused.arena, fused.plain_off, fused.plain_bytes)
    got = np.frombuffer(raw, np.float32).reshape(world, fused.n_stride)[:, :layer.n].reshape(-1)
    err = None
    if rank == 0:
        import oracle as orc
        packed, scales, zeros, _ = layer.quantized
        words = np.frombuffer(packed.tobytes(), np.uint32)
        wpr = k // 4
        rows = np.unique(np.concatenate([np.arange(r * (n // world), r * (n // world) + 32) for r in range(world)] +
                                        [np.arange(n - 32, n)]))
        sub = orc.QWeight(orc.FMT_F8, len(rows), k,
                          np.concatenate([words[: n * wpr].reshape(n, wpr)[rows].reshape(-1), np.zeros(16, np.uint32)]),
                          scales[rows].copy(), np.zeros(0, np.float32))
        want = orc.qmatmul(sub, x).astype(np.float64).ravel()
        err = float(np.max(np.abs(got[rows] - want)) / np.sqrt(np.mean(want ** 2)))
    for i in range(3):
        fused.forward(i)
    ms = time_graph(backend, fnn, lambda: ([fused.forward(i) for i in range(steps)], fused.wait()), dist)
    us = ms / steps * 1e3
    total_bytes = algorithmic_bytes(8, n, k, 1, 4 * n, False)
    out = {"workload": "FP8 e4m3 K=8192 N=28672 M=1, N split over the ranks, fused GEMV + all-gather",
           "scaling": "strong", "us_per_step": round(us, 2), "gbs": round(total_bytes / (us * 1e-6) / 1e9, 1),
           "hbm_frac_of_n_gpus": round(total_bytes / (us * 1e-6) / 1e9 / (peaks["hbm_gbs"] * world), 3),
           "parity_err": err if err is None else float(f"{err:.3g}"),
           "columns_per_rank": layer.n, "launches_per_step": 1}
    fused.close()
    layer.close()
    return out


def c5_chain(fnn, backend, rank, world, dist, layers=32, m=64, steps=3):
    """The decoder-shaped projection set: per layer QKV [4096, 6144], O [4096, 4096], gate/up
    [4096, 2 x 14336], down [14336, 4096], I4 per-channel weights, activations f32 [64, 4096], every
    projection column-sharded over the ranks with its outputs all-gathered (fused into the GEMM's
    epilogue as peer stores).  The glue between the projections, stated because the configuration
    gives none: a = qkv[:, :4096] (attention elided); r = a @ Wo + x; n = rms_norm(r);
    g = n @ Wgu; h = silu(g[:, :14336]) * g[:, 14336:]; x' = h @ Wd + r.  One layer's four weights are
    quantized on the host and uploaded once per layer (distinct device copies, so the chain streams
    layers x 54.5 MB / ranks from HBM per step and rank).  Rank 0 checks the first layer's output
    against the CPU oracle on eight of the 64 rows."""
    from fastnn_b200 import _lib as L
    from fastnn_b200.parallel import AllGatherLinear, PeerArena
    lib = backend.lib
    d, dq, dff = 4096, 6144, 14336
    al = lambda v: -(-v // 256) * 256
    off, cur = {}, 0
    for name, cols in (("x", d), ("qkv", dq), ("a", d), ("o", d), ("r", d), ("n", d), ("g", 2 * dff),
                       ("gate", dff), ("up", dff), ("dn", d)):
        off[name] = cur
        cur += al(m * cols * 4)
    off["ones"] = cur
    cur += al(d * 4)
    for name in ("c_qkv", "c_o", "c_g", "c_dn"):
        off[name] = cur
        cur += 256
    pa = PeerArena(backend, cur, rank, world)
    backend.write_arena(pa.arena, off["ones"], np.ones(d, np.float32).tobytes())
    shapes = {"qkv": (d, dq), "o": (d, d), "g": (d, 2 * dff), "dn": (dff, d)}
    quant, metas = {}, {}
    for i, (name, (k, n)) in enumerate(shapes.items()):
        w = philox_normal(500 + i, (k, n), 0.02)
        packed, scales, zeros, _ = fnn.quantize_weight_constant(w, L.FMT_I4)
        quant[name] = (packed.tobytes(), scales, zeros)
        metas[name] = fnn.QuantizedWeightMeta(bit_width=4, scales=scales, zero_points=zeros, shape=[n, k], fmt=L.FMT_I4)
    src = {"qkv": "x", "o": "a", "g": "n", "dn": "gate"}
    saved_path, backend.path = backend.path, L.PATH_TC       # the tcgen05 kernel needs no extra weight layout
    lin = [{name: AllGatherLinear(backend, quant[name][0], metas[name], rank, world, pa, off[name], off["c_" + name])
            for name in shapes} for _ in range(layers)]
    backend.path = saved_path
    A, base, f4 = pa.arena.handle, pa.device_ptr, 4
    eps = 1e-5

    def layer_ops(l):
        lin[l]["qkv"].forward(base + off["x"], m)
        check(lib.fnn_cuda_memcpy2d(backend.ctx, A, off["a"], d * f4, off["qkv"], dq * f4, d * f4, m), fnn)
        lin[l]["o"].forward(base + off["a"], m)
        check(lib.fnn_cuda_elementwise(backend.ctx, L.EW_ADD, A, off["o"], m * d, off["x"], m * d, off["r"], m * d), fnn)
        check(lib.fnn_cuda_rms_norm(backend.ctx, A, off["r"], m * d, off["ones"], d, d, eps, off["n"]), fnn)
        lin[l]["g"].forward(base + off["n"], m)
        check(lib.fnn_cuda_memcpy2d(backend.ctx, A, off["gate"], dff * f4, off["g"], 2 * dff * f4, dff * f4, m), fnn)
        check(lib.fnn_cuda_memcpy2d(backend.ctx, A, off["up"], dff * f4, off["g"] + dff * f4, 2 * dff * f4, dff * f4, m), fnn)
        check(lib.fnn_cuda_elementwise(backend.ctx, L.EW_SILU, A, off["gate"], m * dff, 0, 0, off["gate"], m * dff), fnn)
        check(lib.fnn_cuda_elementwise(backend.ctx, L.EW_MUL, A, off["gate"], m * dff, off["up"], m * dff,
                                       off["gate"], m * dff), fnn)
        lin[l]["dn"].forward(base + off["gate"], m)
        check(lib.fnn_cuda_elementwise(backend.ctx, L.EW_ADD, A, off["dn"], m * d, off["r"], m * d, off["x"], m * d), fnn)

    x0 = philox_normal(21, (m, d), 1.0)
    backend.write_arena(pa.arena, off["x"], x0.tobytes())
    launches0 = backend.launch_count()
    layer_ops(0)
    sync_ranks(backend, dist)
    launches_per_layer = backend.launch_count() - launches0
    got = np.frombuffer(backend.read_arena(pa.arena, off["x"], m * d * 4), np.float32).reshape(m, d)
    err = None
    if rank == 0:
        import oracle as orc
        rows = np.arange(0, m, m // 8)[:8]
        q = {name: orc.QWeight(orc.FMT_I4, shapes[name][1], shapes[name][0], np.frombuffer(quant[name][0], np.uint32),
                               quant[name][1], quant[name][2]) for name in shapes}
        xr = x0[rows]
        a = orc.qmatmul(q["qkv"], xr)[:, :d]
        r = orc.qmatmul(q["o"], np.ascontiguousarray(a)) + xr
        nrm = orc.rms_norm(r, np.ones(d, np.float32), eps)
        g = orc.qmatmul(q["g"], nrm)
        h = orc.epilogue(np.ascontiguousarray(g[:, :dff]), dff, None, orc.EPI_SILU) * g[:, dff:]
        want = (orc.qmatmul(q["dn"], np.ascontiguousarray(h)) + r).astype(np.float64)
        err = float(np.max(np.abs(got[rows] - want)) / np.sqrt(np.mean(want ** 2)))
    backend.write_arena(pa.arena, off["x"], x0.tobytes())
    for l in range(layers):      # warm-up pass over every layer (first use of each weight)
        layer_ops(l)
    sync_ranks(backend, dist)
    ms = time_graph(backend, fnn, lambda: [layer_ops(l) for _ in range(steps) for l in range(layers)], dist)
    us_layer = ms / (steps * layers) * 1e3
    wbytes = sum(k * n // 2 + 8 * n for k, n in shapes.values())
    flops = sum(2 * m * k * n for k, n in shapes.values())
    out = {"workload": f"{layers} layers x (QKV, O, gate/up, down), I4, activations [64, 4096], every projection "
                       f"column-sharded over {world} rank(s), outputs gathered by the GEMM's own peer stores",
           "us_per_layer": round(us_layer, 2), "ms_per_step": round(ms / steps, 3),
           "weight_gbs_all_ranks": round(wbytes / (us_layer * 1e-6) / 1e9, 1),
           "tflops_all_ranks": round(flops / (us_layer * 1e-6) / 1e12, 2),
           "launches_per_layer": launches_per_layer, "gathers_per_layer": 4 if world > 1 else 0,
           "parity_err_layer0": err if err is None else float(f"{err:.3g}")}
    for l in lin:
        for v in l.values():
            v.close()
    pa.close()
    return out


# ------------------------------------------------------------------------------ reference arm


def run_reference(args):
    """The reference's own CPU algorithm for the path (the oracle port of
    gemm_batch_packed_simd; the Rust crate cannot be built here), on the host cores, same
    workload/metric/unit.  Each step is one full M=1 layer call."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle as orc
    w_kn = philox_normal(1000, (K_DIM, N_DIM), SIGMA)
    q = orc.quantize_kn(orc.FMT_I8, w_kn)
    x = philox_normal(1, (M_HEAD, K_DIM), 1.0)
    sbytes = q.scales.nbytes + q.zeros.nbytes
    alg = algorithmic_bytes(8, N_DIM, K_DIM, M_HEAD, sbytes, False)
    warm = min(args.warmup, 50)
    for _ in range(warm):
        orc.qmatmul(q, x, None, orc.EPI_SILU)
    steps = args.steps
    t_budget, t0, done = 170.0, time.perf_counter(), 0
    while done < steps and time.perf_counter() - t0 < t_budget:
        orc.qmatmul(q, x, None, orc.EPI_SILU)
        done += 1
    dt = (time.perf_counter() - t0) / max(done, 1)
    info = orc.host_info()
    value = round(alg / dt / 1e9, 3)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
        "steps": done, "warmup": warm, "ms_per_step": round(dt * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "m": M_HEAD, "k": K_DIM, "n_per_gpu": N_DIM, "format": "i8"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "kind": "port",
                         "sample": f"{done} full M=1 layer calls; the reference threads only when "
                                   f"M >= physical cores ({info['physical_cores']}); simd_level="
                                   f"{info['simd_level']}"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-multi", action="store_true", help="skip the strong-scaling layer and the projection chain")
    ap.add_argument("--only", default=None, help="run one sweep point (e.g. c3_f4) and exit")
    ap.add_argument("--only-m", type=int, default=None, help="batch rows M for --only")
    ap.add_argument("--path", type=int, default=0, help="kernel family for --only (0 auto, 1 rows, 2 mma, 3 tc)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
