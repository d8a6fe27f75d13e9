#!/usr/bin/env python
"""Benchmark of the quantized matrix hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Default workload (the configuration the headline metric is quoted on): Q4_K x Q8_K mul_mat decode on
a Llama-3-8B-shaped layer, N = 14336, K = 4096, batch 1.  One step = one production_mul_mat_q4_k_decode
call: quantize the fp32 activation row to Q8_K, then the GEMV over every weight row.  Metric:
algorithmic bytes streamed per second (weights once + activation records + fp32 output).

Inputs are synthetic and seeded: weights ~N(0, 0.02) quantized to Q4_K with the CPU oracle's
quantize_row_q4_K restatement, activations ~N(0, 1).  Successive steps walk through several distinct
copies of the weight matrix whose total size exceeds twice the L2, so every step streams from HBM.

Prints ONE JSON line (rank 0).  With --impl reference the same workload runs on the host cores through
the reference's own GGML C (oracle/_ref, compiled from the reference sources) or, where that is
absent, this repository's C restatement of it.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (format, mode, N, K, M)
    "q4_k_decode_14336x4096": ("Q4_K", "decode", 14336, 4096, 1),
    "q4_k_decode_4096x4096": ("Q4_K", "decode", 4096, 4096, 1),
    "q4_k_decode_4096x14336": ("Q4_K", "decode", 4096, 14336, 1),
    "q4_0_decode_4096x4096": ("Q4_0", "decode", 4096, 4096, 1),
    "iq2_xxs_decode_28672x8192": ("IQ2_XXS", "decode", 28672, 8192, 1),
    "iq2_xs_decode_28672x8192": ("IQ2_XS", "decode", 28672, 8192, 1),
    "iq3_xxs_decode_28672x8192": ("IQ3_XXS", "decode", 28672, 8192, 1),
    "iq2_s_decode_28672x8192": ("IQ2_S", "decode", 28672, 8192, 1),
    "iq3_s_decode_28672x8192": ("IQ3_S", "decode", 28672, 8192, 1),
    "iq1_s_decode_28672x8192": ("IQ1_S", "decode", 28672, 8192, 1),
    "iq1_m_decode_28672x8192": ("IQ1_M", "decode", 28672, 8192, 1),
    "q2_k_decode_14336x4096": ("Q2_K", "decode", 14336, 4096, 1),
    "q3_k_decode_14336x4096": ("Q3_K", "decode", 14336, 4096, 1),
    "q5_k_decode_14336x4096": ("Q5_K", "decode", 14336, 4096, 1),
    "q6_k_decode_14336x4096": ("Q6_K", "decode", 14336, 4096, 1),
    "q4k_i16_decode_14336x4096": ("Q4K_I16", "decode", 14336, 4096, 1),   # persistent 16-row interleaved layout
    "q4_k_prefill_14336x4096": ("Q4_K", "prefill", 14336, 4096, 512),
    "q4_k_prefill_4096x4096": ("Q4_K", "prefill", 4096, 4096, 512),
    "q4_k_prefill_4096x14336": ("Q4_K", "prefill", 4096, 14336, 512),
    "tq1_0_prefill_28672x8192": ("TQ1_0", "prefill", 28672, 8192, 512),
    "q4_0_prefill_4096x4096": ("Q4_0", "prefill", 4096, 4096, 512),
    "q8_0_prefill_4096x4096": ("Q8_0", "prefill", 4096, 4096, 512),
    "iq2_xxs_prefill_4096x4096": ("IQ2_XXS", "prefill", 4096, 4096, 512),
    "q4_k_dequantize_14336x4096": ("Q4_K", "dequantize", 14336, 4096, 0),
    "q4_k_layer_decode_llama3_8b": ("Q4_K", "layer", 0, 4096, 1),     # the seven projections of one block, one call per step
}
DEFAULT_WORKLOAD = "q4_k_decode_14336x4096"

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the workload's dominant kernel, from the ncu
# captures summarised under profiles/ (a profiler cannot run inside a timed benchmark, so the figures are
# carried here; a sharded run scales them by the rank's share of the rows).  Writes that are still in L2
# when the kernel ends are not in these numbers.
NCU_DRAM_TRAFFIC = {
    "q4_k_decode_14336x4096": 33_078_272,
    "iq2_xxs_decode_28672x8192": 60_635_904,
    "q4_k_prefill_4096x4096": 11_885_568,
    "q8_0_prefill_4096x4096": 20_104_448,
    "iq2_xxs_prefill_4096x4096": 6_777_344,
    "tq1_0_prefill_28672x8192": 69_316_352,
    "q4_k_dequantize_14336x4096": 33_041_920 + 177_308_928,
}


def ncu_traffic(workload: str, share: float):
    full = NCU_DRAM_TRAFFIC.get(workload)
    return None if full is None else int(full * share)
L2_BYTES = 126 * 1024 * 1024
SEED = 20240611


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except ValueError:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def algorithmic_bytes(fmt: str, n: int, k: int, m: int) -> int:
    from weft_b200.formats import row_bytes

    act = "Q8_0" if fmt in ("Q4_0", "Q8_0") else "Q8_K"
    return n * row_bytes(fmt, k) + m * row_bytes(act, k) + 4 * m * n


def make_inputs(fmt: str, n: int, k: int, m: int, seed: int):
    """Seeded host inputs: packed weights (n, row_bytes) uint8, fp32 activations (m, k), codebook tables."""
    import oracle

    rng = np.random.default_rng(seed)
    fid = oracle.FORMAT_IDS[fmt]
    golden = np.load(ROOT / "tests" / "golden" / "golden.npz")
    grid, signs = golden[{"IQ2_XS": "iq2xs_grid", "IQ3_XXS": "iq3xxs_grid", "IQ2_S": "iq2s_grid", "IQ3_S": "iq3s_grid", "IQ1_S": "iq1s_grid", "IQ1_M": "iq1s_grid"}.get(fmt, "iq2xxs_grid")], golden["iq2xxs_signs"]
    base_rows = min(n, 1024)            # quantize 1024 distinct rows, rotate them to fill the matrix (timing is data-independent)
    if fmt == "TQ1_0":
        src = (rng.integers(-1, 2, size=(base_rows, k)) * np.float32(0.02)).astype(np.float32)
        base = oracle.quantize(fid, src)
    elif fmt in ("IQ2_XXS", "IQ2_XS", "IQ3_XXS", "IQ2_S", "IQ3_S", "IQ1_S", "IQ1_M"):
        if oracle.ref_available():
            base_rows = min(n, 128)
            base = oracle.ref_quantize_weights(fid, (rng.standard_normal((base_rows, k)) * 0.02).astype(np.float32))
        else:           # any index, sign index and scale is a valid record once the f16 scale is a small finite number
            base = rng.integers(0, 256, size=(base_rows, k // 256, oracle.RECORD_BYTES[fid]), dtype=np.uint8)
            if fmt == "IQ1_M":          # its f16 scale is spread over the top nibbles of the last eight bytes: keep it a small normal number
                base[:, :, 55] = (base[:, :, 55] & 0x0f) | 0x20
            base[:, :, 0:2] = (np.abs(rng.standard_normal((base_rows, k // 256))) * 0.01 + 1e-3).astype(np.float16).view(np.uint8).reshape(base_rows, -1, 2)
            base = base.reshape(base_rows, -1)
    elif fmt in ("Q2_K", "Q3_K", "Q5_K", "Q6_K"):
        if oracle.ref_available():
            base = oracle.ref_quantize_weights(fid, (rng.standard_normal((base_rows, k)) * 0.02).astype(np.float32))
        else:           # every bit pattern is a valid record once the f16 scales are small finite numbers
            nbytes, at, count = {"Q2_K": (84, 80, 2), "Q3_K": (110, 108, 1), "Q5_K": (176, 0, 2), "Q6_K": (210, 208, 1)}[fmt]
            base = rng.integers(0, 256, size=(base_rows, k // 256, nbytes), dtype=np.uint8)
            scales = (np.abs(rng.standard_normal((base_rows, k // 256, count))) * 1e-4 + 1e-5).astype(np.float16)
            base[:, :, at:at + 2 * count] = scales.view(np.uint8).reshape(base_rows, -1, 2 * count)
            base = base.reshape(base_rows, -1)
    else:
        base = oracle.quantize(fid, (rng.standard_normal((base_rows, k)) * 0.02).astype(np.float32))
    reps = -(-n // base_rows)
    w = np.concatenate([np.roll(base, s, axis=0) for s in range(reps)], axis=0)[:n]
    x = rng.standard_normal((m, k)).astype(np.float32)
    return np.ascontiguousarray(w), x, grid, signs


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int) -> None:
        self.device_index, self.proc, self.lines = device_index, None, []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxes, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1])); maxes.append(float(parts[2]))
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(maxes) if maxes else None,
                "samples": len(clocks), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ CPU side (reference arm and cpu_baseline)

def cpu_mul_mat_runner(fmt: str, n: int, k: int, m: int, w: np.ndarray, x: np.ndarray, grid, signs, threads: int):
    """Returns (callable running one full mul_mat on the host cores, kind)."""
    import oracle

    fid = oracle.FORMAT_IDS[fmt]
    act = oracle.ACTIVATION[fid]
    xq = np.zeros((m, oracle.row_bytes(act, k)), dtype=np.uint8)
    y = np.zeros((m, n), dtype=np.float32)
    if oracle.ref_available():
        lib = oracle.ref()
        quant = lib.weft_ref_quantize_q8_0 if act == oracle.Q8_0 else lib.weft_ref_quantize_q8_K
        pool = ThreadPoolExecutor(max_workers=threads)
        bounds = [(n * t // threads, n * (t + 1) // threads) for t in range(threads)]
        xp = x.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
        yp = y.ctypes.data_as(ctypes.POINTER(ctypes.c_float))

        def run_reference() -> None:
            for r in range(m):
                quant(x[r].ctypes.data_as(ctypes.POINTER(ctypes.c_float)), xq[r].ctypes.data, k)
            # ctypes drops the GIL during the call: the row ranges run on separate cores
            list(pool.map(lambda b: lib.weft_ref_mul_mat(fid, w.ctypes.data, xp, xq.ctypes.data, yp, n, k, m, b[0], b[1], 0), bounds))

        return run_reference, "reference"
    oracle.port().wo_set_threads(threads)

    def run_port() -> None:
        oracle.mul_mat(fid, w, x, n, k, m, rule=0, grid=grid, signs=signs)

    return run_port, "port"


def cpu_dequantize(fmt: str, n: int, k: int, w: np.ndarray, threads: int):
    """(callable dequantizing the whole matrix on the host cores, kind)."""
    import oracle

    fid = oracle.FORMAT_IDS[fmt]
    out = np.empty((n, k), dtype=np.float32)
    if oracle.ref_available() and fmt != "IQ2_XXS":
        lib = oracle.ref()
        pool = ThreadPoolExecutor(max_workers=threads)
        rb = oracle.row_bytes(fid, k)
        bounds = [(n * t // threads, n * (t + 1) // threads) for t in range(threads)]

        def run_rows(b):
            # one call per contiguous range: the reference dequantizer takes an element count, rows are contiguous
            lib.weft_ref_dequantize(fid, w.ctypes.data + b[0] * rb, out[b[0]:].ctypes.data_as(ctypes.POINTER(ctypes.c_float)), (b[1] - b[0]) * k)

        return (lambda: list(pool.map(run_rows, bounds))), "reference"
    oracle.port().wo_set_threads(threads)
    return (lambda: oracle.dequantize(fid, w, k)), "port"


def cpu_dequantize_line(args, fmt, n, k, w, grid, signs, threads) -> dict:
    import oracle
    from weft_b200.formats import row_bytes

    run, kind = cpu_dequantize(fmt, n, k, w, threads)
    run()
    times = []
    budget = time.perf_counter() + 60.0
    for _ in range(max(1, args.steps)):
        t0 = time.perf_counter(); run(); times.append(time.perf_counter() - t0)
        if time.perf_counter() > budget:
            break
    per = sum(times) / len(times)
    value = (n * row_bytes(fmt, k) + 4 * n * k) / per / 1e9
    return {"impl": "reference", "metric": "row_dequantize_algorithmic_gbps", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": len(times), "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "format": fmt, "mode": "dequantize", "N": n, "K": k, "cpu": oracle.cpu_model()},
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind, "sample": f"{len(times)} x full {n} x {k} dequantize"},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def reference_arm(args, fmt, mode, n, k, m) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle

    oracle.build(ref=True)
    threads = os.cpu_count() or 1
    if mode == "layer":         # the seven projections of one block (hidden = k), one after the other
        kv, ffn = k // 4, k * 7 // 2
        shapes = [(k, k), (kv, k), (kv, k), (k, k), (ffn, k), (ffn, k), (k, ffn)]
        runners, total, kind = [], 0, "port"
        for i, (rows, cols) in enumerate(shapes):
            w, x, grid, signs = make_inputs(fmt, rows, cols, 1, SEED + i)
            run, kind = cpu_mul_mat_runner(fmt, rows, cols, 1, w, x, grid, signs, threads)
            runners.append(run)
            total += algorithmic_bytes(fmt, rows, cols, 1)
        times, budget = [], time.perf_counter() + 120.0
        for _ in range(args.steps):
            t0 = time.perf_counter()
            for run in runners:
                run()
            times.append(time.perf_counter() - t0)
            if time.perf_counter() > budget:
                break
        per_step = sum(times) / len(times)
        value = total / per_step / 1e9
        print(json.dumps({
            "impl": "reference", "metric": "mul_mat_decode_algorithmic_gbps", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": len(times), "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8 dot, f32 accumulate", "data": "synthetic",
            "config": {"workload": args.workload, "format": fmt, "mode": "layer decode", "M": 1, "cpu": oracle.cpu_model(),
                       "code": "reference GGML C (oracle/_ref)" if kind == "reference" else "C restatement (oracle port)"},
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind, "sample": f"{len(times)} x the seven mul_mats of one block"},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    w, x, grid, signs = make_inputs(fmt, n, k, max(m, 1), SEED)
    if mode == "dequantize":
        print(json.dumps(cpu_dequantize_line(args, fmt, n, k, w, grid, signs, threads)))
        return
    sample_m = m if mode == "decode" else min(m, 4)       # prefill on CPU: a bounded slice of the token rows
    run, kind = cpu_mul_mat_runner(fmt, n, k, sample_m, w, x[:sample_m], grid, signs, threads)
    for _ in range(max(1, min(args.warmup, 3))):
        run()
    times = []
    budget = time.perf_counter() + 120.0
    for _ in range(args.steps):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() > budget:
            break
    per_step = sum(times) / len(times)
    if mode == "decode":
        metric, unit = "mul_mat_decode_algorithmic_gbps", "GB/s"
        value = algorithmic_bytes(fmt, n, k, m) / per_step / 1e9
    else:
        metric, unit = "mul_mat_prefill_int8_tops", "TOP/s"
        value = 2.0 * sample_m * n * k / per_step / 1e12
    sample = f"{len(times)} x full {fmt} mul_mat N={n} K={k} M={sample_m}" + ("" if sample_m == m else f" (of M={m})")
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": len(times),
        "warmup": args.warmup, "ms_per_step": per_step * 1e3 * (m / sample_m), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 dot, f32 accumulate", "data": "synthetic",
        "config": {"workload": args.workload, "format": fmt, "mode": mode, "N": n, "K": k, "M": m,
                   "cpu": oracle.cpu_model(), "code": "reference GGML C (oracle/_ref)" if kind == "reference" else "C restatement (oracle port)"},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ GPU side

def gpu_layer_decode(args, lib, check, stream, fmt, hidden, world, rank, local_rank) -> None:
    """The seven projections of a Llama-3-8B-shaped block at batch 1 (hidden 4096, 8 KV heads of 128, FFN 14336),
    issued as one weft_b200_mul_mat_chain call per step; a step is one block's worth of weights."""
    import torch

    import oracle
    from weft_b200.formats import row_bytes
    from weft_b200.layers import Projection, ProjectionChain

    if world > 1:
        raise SystemExit("the layer workload runs on one GPU")
    kv, ffn = hidden // 4, hidden * 7 // 2
    shapes = [("attn_q", hidden, hidden, "h", False), ("attn_k", kv, hidden, "h", True), ("attn_v", kv, hidden, "h", True),
              ("attn_output", hidden, hidden, "a", False), ("ffn_gate", ffn, hidden, "g", False), ("ffn_up", ffn, hidden, "g", True),
              ("ffn_down", hidden, ffn, "f", False)]
    rng = np.random.default_rng(SEED)
    inputs = {"h": hidden, "a": hidden, "g": hidden, "f": ffn}
    x_host = {key: rng.standard_normal((1, k)).astype(np.float32) for key, k in inputs.items()}
    x_dev = {key: torch.from_numpy(v).cuda() for key, v in x_host.items()}
    xq_dev = {key: torch.zeros((1, row_bytes("Q8_K", k)), dtype=torch.uint8, device="cuda") for key, k in inputs.items()}
    w_host = {name: make_inputs(fmt, n, k, 1, SEED + i)[0] for i, (name, n, k, _, _) in enumerate(shapes)}
    layer_bytes = sum(w.nbytes for w in w_host.values())
    copies = max(3, -(-2 * L2_BYTES // layer_bytes) + 1)
    w_dev = [{name: torch.from_numpy(w).cuda() for name, w in w_host.items()} for _ in range(copies)]
    y_dev = {name: torch.zeros((1, n), device="cuda") for name, n, _, _, _ in shapes}

    def chain_for(weights, x, xq, y) -> ProjectionChain:
        return ProjectionChain(lib, [Projection(fmt, weights[name].data_ptr(), x[key].data_ptr(), xq[key].data_ptr(), y[name].data_ptr(), n, k,
                                                reuse_xq=reuse) for name, n, k, key, reuse in shapes])

    chains = [chain_for(w_dev[c], x_dev, xq_dev, y_dev) for c in range(copies)]

    def step(i: int) -> None:
        chains[i % copies].run()

    step(0)
    torch.cuda.synchronize()
    check(lib.weft_b200_synchronize())
    worst = 0.0
    for name, n, k, key, _ in shapes:       # every projection against the oracle (first 128 rows)
        want, _ = oracle.mul_mat(oracle.FORMAT_IDS[fmt], w_host[name][:128], x_host[key], 128, k, 1, rule=1)
        got = y_dev[name][:, :128].cpu().numpy().astype(np.float64)
        worst = max(worst, float(np.linalg.norm(got - want) / max(np.linalg.norm(want.astype(np.float64)), 1e-30)))
    if not worst <= 1e-5:
        raise SystemExit(f"parity check failed before timing: relative L2 {worst}")

    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches_before = int(lib.weft_b200_launch_count())
    side, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    side.wait_stream(torch.cuda.current_stream())
    lib.weft_b200_set_stream(ctypes.c_void_p(side.cuda_stream))
    with torch.cuda.graph(graph, stream=side):
        for i in range(args.steps):
            step(args.warmup + i)
    lib.weft_b200_set_stream(ctypes.c_void_p(stream.cuda_stream))
    launches = int(lib.weft_b200_launch_count()) - launches_before
    graph.replay()
    torch.cuda.synchronize()
    begin.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    ms = begin.elapsed_time(end) / args.steps
    clocks = sampler.stop()

    # end to end: host (pinned) activations in, host outputs back, weights resident on the device
    pin = lambda t: t.pin_memory()
    x_pin = {key: pin(torch.from_numpy(v)) for key, v in x_host.items()}
    xq_pin = {key: pin(torch.zeros((1, row_bytes("Q8_K", k)), dtype=torch.uint8)) for key, k in inputs.items()}
    y_pin = {name: pin(torch.zeros((1, n))) for name, n, _, _, _ in shapes}
    host_chains = [chain_for(w_dev[c], x_pin, xq_pin, y_pin) for c in range(copies)]
    for i in range(3):
        host_chains[i % copies].run()
    torch.cuda.synchronize()
    e2e_steps = max(3, min(args.steps, 100))
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        host_chains[i % copies].run()
    check(lib.weft_b200_synchronize())
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if float((y_pin["ffn_down"] - y_dev["ffn_down"].cpu()).abs().max()) != 0.0:
        raise SystemExit("host-buffer path disagrees with the device-buffer path")

    peaks, peaks_kind = load_peaks()
    total = sum(algorithmic_bytes(fmt, n, k, 1) for _, n, k, _, _ in shapes)
    achieved = total / (ms * 1e-3) / 1e9
    line = {
        "metric": "mul_mat_decode_algorithmic_gbps", "value": achieved, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 dot (dp4a), f32 accumulate",
        "data": "synthetic",
        "config": {"workload": args.workload, "format": fmt, "mode": "layer decode", "M": 1,
                   "projections": {name: [n, k] for name, n, k, _, _ in shapes},
                   "l2": f"steps rotate over {copies} sets of layer weights ({copies * layer_bytes / 2**20:.0f} MiB > 2 x L2)",
                   "launch": "cuda graph replay of all steps, one weft_b200_mul_mat_chain call (7 kernels) per step",
                   "timed_scope": "7 x (activation quantize + mul_mat)", "seed": SEED, "parity_rel_l2_before_timing": worst},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "traffic": None, "peak_source": peaks_kind, "kernel": "gemv kernels of one block, back to back", "kernel_ms": ms,
                     "algorithmic_bytes_per_launch": total},
        "clocks": clocks, "gpu_launches": launches,
        "e2e": {"value": total / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(sum(4 * k for k in inputs.values())),
                "d2h_bytes_per_step": int(sum(4 * n for _, n, _, _, _ in shapes) + sum(row_bytes("Q8_K", k) for k in inputs.values())),
                "ms_per_step": e2e_s * 1e3, "what": "weft_b200_mul_mat_chain with host X/Xq/Y (pinned), weights resident in HBM"},
    }
    if not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        runners = [cpu_mul_mat_runner(fmt, n, k, 1, w_host[name], x_host[key], None, None, threads) for name, n, k, key, _ in shapes]
        kind = runners[0][1]
        times, t_end = [], time.perf_counter() + 12.0
        while time.perf_counter() < t_end and len(times) < 50:
            t0 = time.perf_counter()
            for run, _ in runners:
                run()
            times.append(time.perf_counter() - t0)
        per = sum(times) / len(times)
        line["cpu_baseline"] = {"value": total / per / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
                                "sample": f"{len(times)} x the seven mul_mats of one block", "cpu": oracle.cpu_model(), "ms_per_step": per * 1e3}
    print(json.dumps(line))


def gpu_dequantize(args, lib, check, stream, fmt, n, k, world, rank, local_rank, *, extras: bool = True):
    """row_dequantize over an (n, k) matrix, rows split across ranks (no collective: rows are independent).
    Returns the JSON record on rank 0, None on the others; extras = False leaves out the end-to-end and CPU legs."""
    import torch
    import torch.distributed as dist

    import oracle
    from weft_b200.formats import FORMAT_IDS, TQ1_POWERS, row_bytes

    w_host, _, grid, signs = make_inputs(fmt, n, k, 1, SEED)
    n0, n1 = n * rank // world, n * (rank + 1) // world
    rows = n1 - n0
    shard = w_host[n0:n1]
    copies = min(64, max(2, -(-2 * L2_BYTES // max(1, shard.nbytes)) + 1))
    w_dev = [torch.from_numpy(shard).cuda() for _ in range(copies)]
    y_dev = torch.empty((rows, k), device="cuda")
    grid_dev, signs_dev = torch.from_numpy(grid).cuda(), torch.from_numpy(signs).cuda()
    powers_dev = torch.tensor(TQ1_POWERS, dtype=torch.int32, device="cuda")
    name = {"Q4_0": "q4_0", "Q8_0": "q8_0", "Q4_K": "q4_k", "IQ2_XXS": "iq2_xxs", "TQ1_0": "tq1_0"}[fmt]
    fn = getattr(lib, f"row_dequantize_{name}_rows")
    extra = [grid_dev.data_ptr(), signs_dev.data_ptr()] if fmt == "IQ2_XXS" else [powers_dev.data_ptr()] if fmt == "TQ1_0" else []
    fn.argtypes = [ctypes.c_void_p] * (2 + len(extra)) + [ctypes.c_size_t] * 2

    def call(w_ptr, y_ptr):
        check(fn(w_ptr, *extra, y_ptr, rows, k))

    def step(i):
        call(w_dev[i % copies].data_ptr(), y_dev.data_ptr())

    step(0)
    torch.cuda.synchronize()
    want = oracle.dequantize(oracle.FORMAT_IDS[fmt], shard[:64], k, grid, signs)
    if not np.array_equal(y_dev[:64].cpu().numpy().view(np.uint32), want.view(np.uint32)):
        raise SystemExit("parity check failed before timing: dequantize is not bit-exact")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    before = lib.weft_b200_launch_count()
    times = []
    for r in range(max(1, args.replays)):       # each timing: `steps` direct launches between two events
        barrier()
        begin.record()
        for i in range(args.steps):
            step(args.warmup + r * args.steps + i)
        end.record()
        barrier()
        times.append(begin.elapsed_time(end) / args.steps)
    launches = int(lib.weft_b200_launch_count() - before) // max(1, args.replays)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor(times, device="cuda", dtype=torch.float64); dist.all_reduce(t, op=dist.ReduceOp.MAX); times = [float(v) for v in t.tolist()]
        lt = torch.tensor([launches], device="cuda"); dist.all_reduce(lt); launches = int(lt.item())
    ms = statistics.median(times)
    e2e_s = None
    if extras:
        # end to end: host record bytes in, host fp32 out (pinned), copies inside the timed region
        w_pin = torch.from_numpy(shard).pin_memory()
        y_pin = torch.empty((rows, k), dtype=torch.float32).pin_memory()
        e2e_steps = max(3, min(args.steps, 10))
        call(w_pin.data_ptr(), y_pin.data_ptr())
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            call(w_pin.data_ptr(), y_pin.data_ptr())
        torch.cuda.synchronize()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        if world > 1:
            t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64); dist.all_reduce(t, op=dist.ReduceOp.MAX); e2e_s = float(t.item())
        if not np.array_equal(y_pin[:64].numpy().view(np.uint32), want.view(np.uint32)):
            raise SystemExit("host-buffer dequantize is not bit-exact")
    del w_dev, y_dev
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    peaks, peaks_kind = load_peaks()
    total_bytes = n * row_bytes(fmt, k) + 4 * n * k
    shard_bytes = rows * row_bytes(fmt, k) + 4 * rows * k
    achieved = shard_bytes / (ms * 1e-3) / 1e9
    workload = next((name for name, spec in WORKLOADS.items() if spec[:4] == (fmt, "dequantize", n, k)), args.workload)
    line = {"metric": "row_dequantize_algorithmic_gbps", "value": total_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 (bit-exact)", "data": "synthetic",
            "config": {"workload": workload, "format": fmt, "mode": "dequantize", "N": n, "K": k,
                       "sharding": f"rows split {world} ways, no collective" if world > 1 else "none",
                       "l2": f"{copies} input copies rotate; the {4 * rows * k / 2**20:.0f} MiB output exceeds L2", "launch": "direct launches",
                       "timing": f"median of {len(times)} timings of {args.steps} launches, max over ranks",
                       "replay_spread": (max(times) - min(times)) / ms if len(times) > 1 else 0.0, "seed": SEED, "parity_rel_l2_before_timing": 0.0},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "traffic": ncu_traffic(workload, rows / n), "peak_source": peaks_kind, "kernel": "dequant kernel (per GPU)", "kernel_ms": ms,
                         "algorithmic_bytes_per_launch": shard_bytes},
            "clocks": clocks, "gpu_launches": launches}
    if e2e_s is not None:
        line["e2e"] = {"value": total_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(shard.nbytes), "d2h_bytes_per_step": int(4 * rows * k),
                       "ms_per_step": e2e_s * 1e3, "what": "row_dequantize_*_rows with host W and Y (pinned)"}
    if extras and not args.no_cpu_baseline and world == 1:
        threads = os.cpu_count() or 1
        run, kind = cpu_dequantize(fmt, n, k, w_host, threads)
        run()
        cpu_times, t_end = [], time.perf_counter() + 10.0
        while time.perf_counter() < t_end and len(cpu_times) < 100:
            t0 = time.perf_counter(); run(); cpu_times.append(time.perf_counter() - t0)
        per = sum(cpu_times) / len(cpu_times)
        line["cpu_baseline"] = {"value": total_bytes / per / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
                                "sample": f"{len(cpu_times)} x full {n} x {k} dequantize", "cpu": oracle.cpu_model(), "ms_per_step": per * 1e3}
    return line


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="weft_b200", choices=["weft_b200", "reference"])
    parser.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--collective", default="p2p", choices=["p2p", "nccl"],
                        help="N > 1: all-gather by the library's own peer-memory kernels (default) or by NCCL")
    parser.add_argument("--no-graph", action="store_true", help="time direct launches instead of a CUDA graph replay")
    parser.add_argument("--replays", type=int, default=5, help="timings taken of the K steps; the median is reported")
    parser.add_argument("--no-also", action="store_true", help="default workload only: leave out the compact records of the other configurations")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    fmt, mode, n, k, m = WORKLOADS[args.workload]
    layout = fmt                      # what the kernel is given
    if fmt == "Q4K_I16":              # Q4_K records, packed once by the kernel's _W_pack artifact function
        fmt = "Q4_K"
    if args.impl == "reference":
        reference_arm(args, fmt, mode, n, k, m)
        return

    import torch
    import torch.distributed as dist

    import oracle
    from weft_b200.formats import FORMAT_IDS, TQ1_POWERS, row_bytes
    from weft_b200.runtime.driver import Toolchain, last_error, load_library

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = load_library(Toolchain().resolve().compiler)
    if lib.weft_b200_init(local_rank):
        raise SystemExit("weft_b200_init failed: " + last_error(lib))
    # A real (non-default) stream: the library treats a NULL handle as "use your own stream", and the
    # events that time the run must sit on the stream the kernels are launched on.
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    assert stream.cuda_stream != 0
    lib.weft_b200_set_stream(ctypes.c_void_p(stream.cuda_stream))
    lib.weft_b200_set_async(1)

    def check(status: int) -> None:
        if status:
            raise SystemExit("weft_b200 call failed: " + last_error(lib))

    if mode == "dequantize":
        line = gpu_dequantize(args, lib, check, stream, fmt, n, k, world, rank, local_rank)
        if line is not None:
            print(json.dumps(line))
        if world > 1:
            dist.destroy_process_group()
        return
    if mode == "layer":
        gpu_layer_decode(args, lib, check, stream, fmt, k, world, rank, local_rank)
        return
    line = run_mul_mat(args, lib, check, stream, args.workload, world, rank, local_rank)
    if args.workload == DEFAULT_WORKLOAD and not args.no_also:
        records = also_records(args, lib, check, stream, world, rank, local_rank)
        if line is not None:
            line["also"] = records
    if line is not None:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_mul_mat(args, lib, check, stream, workload: str, world: int, rank: int, local_rank: int, *, extras: bool = True):
    """One mul_mat workload (decode or prefill), weight rows sharded over the ranks.  Returns the JSON record on rank 0,
    None on the others.  extras = False leaves out the end-to-end and CPU legs (the compact records of the default run)."""
    import torch
    import torch.distributed as dist

    import oracle
    from weft_b200.formats import FORMAT_IDS, TQ1_POWERS, row_bytes

    fmt, mode, n, k, m = WORKLOADS[workload]
    layout = fmt                      # what the kernel is given
    if fmt == "Q4K_I16":              # Q4_K records, packed once by the kernel's _W_pack artifact function
        fmt = "Q4_K"

    # ---- inputs, sharded by weight rows
    act = "Q8_0" if fmt in ("Q4_0", "Q8_0") else "Q8_K"
    w_host, x_host, grid, signs = make_inputs(fmt, n, k, m, SEED)
    n0, n1 = n * rank // world, n * (rank + 1) // world
    n_local = n1 - n0
    shard = w_host[n0:n1]
    copies = max(2, -(-2 * L2_BYTES // max(1, shard.nbytes)) + 1)
    copies = min(copies, 64)
    w_dev = [torch.from_numpy(shard).cuda() if c == 0 else None for c in range(copies)]
    if layout == "Q4K_I16":
        if n_local % 16:
            raise SystemExit(f"{n_local} rows per rank are not whole cohorts of 16")
        packed = torch.empty_like(w_dev[0])
        lib.q4_k_q8_k_gemv_W_pack.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t]
        check(lib.q4_k_q8_k_gemv_W_pack(w_dev[0].data_ptr(), packed.data_ptr(), n_local, k))
        torch.cuda.synchronize()
        w_dev[0] = packed
    for c in range(1, copies):
        w_dev[c] = w_dev[0].clone()
    x_dev = torch.from_numpy(x_host).cuda()
    xq_dev = torch.zeros((m, row_bytes(act, k)), dtype=torch.uint8, device="cuda")
    y_dev = torch.zeros((m, n), device="cuda")
    grid_dev = torch.from_numpy(grid).cuda()
    signs_dev = torch.from_numpy(signs).cuda()
    # the third table slot: the TQ1_0 powers, or for IQ1_M the float[65536] table of f16 bit patterns its reference kernel takes
    f16_table = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    powers_dev = torch.from_numpy(f16_table).cuda() if fmt == "IQ1_M" else torch.tensor(TQ1_POWERS, dtype=torch.int32, device="cuda")
    fid = 1008 if layout == "Q4K_I16" else FORMAT_IDS[fmt]
    mode_id = 0 if mode == "decode" else 1
    shard_fn = lib.weft_b200_mul_mat_shard
    shard_fn.argtypes = [ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 7 + [ctypes.c_size_t] * 4 + [ctypes.c_uint]
    gathered = torch.zeros((world * m, n_local), device="cuda") if world > 1 else None
    y_local = torch.zeros((m, n_local), device="cuda") if world > 1 else None
    # N > 1: the library's own all-gather over NVLink peer memory (peer stores from the GEMV itself and a flag
    # barrier in the same launch; a push kernel behind the tensor-core prefill), or NCCL with --collective nccl.
    peers = None
    collective = "none" if world == 1 else args.collective
    if world > 1 and collective == "p2p":
        from weft_b200.peers import STAGE_BYTES, SYNC_INTS, PeerBuffers

        try:
            peers = PeerBuffers(lib, world, rank, [4 * m * n, 4 * m * n, 4 * SYNC_INTS, STAGE_BYTES])
        except RuntimeError as error:
            sys.stderr.write(f"peer memory unavailable ({error}); using NCCL\n")
        usable = torch.tensor([1 if peers is not None else 0], device="cuda")
        dist.all_reduce(usable, op=dist.ReduceOp.MIN)
        if int(usable.item()) == 0:
            if peers is not None:
                peers.close(dist.barrier)
            peers, collective = None, "nccl"
    gather_fn = lib.weft_b200_mul_mat_shard_gather
    gather_fn.argtypes = ([ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 6 + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
                          + [ctypes.c_size_t] * 5 + [ctypes.c_uint])
    lib.weft_b200_peer_read.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    calls = [0]                       # gathers made so far: consecutive ones alternate between the two output buffers

    def step(i: int, flags: int = 0, x_ptr=None, xq_ptr=None) -> None:
        wbuf = w_dev[i % copies]
        x_ptr = x_dev.data_ptr() if x_ptr is None else x_ptr
        xq_ptr = xq_dev.data_ptr() if xq_ptr is None else xq_ptr
        if world == 1:
            check(shard_fn(fid, mode_id, wbuf.data_ptr(), x_ptr, xq_ptr, grid_dev.data_ptr(), signs_dev.data_ptr(),
                           powers_dev.data_ptr(), y_dev.data_ptr(), n_local, k, m, n, flags))
        elif peers is not None:
            out = calls[0] % 2
            calls[0] += 1
            check(gather_fn(fid, mode_id, wbuf.data_ptr(), x_ptr, xq_ptr, grid_dev.data_ptr(), signs_dev.data_ptr(),
                            powers_dev.data_ptr(), peers.tables[out], peers.tables[2], peers.tables[3], world, rank, n0, n_local, n, k, m, flags))
        else:
            check(shard_fn(fid, mode_id, wbuf.data_ptr(), x_ptr, xq_ptr, grid_dev.data_ptr(), signs_dev.data_ptr(),
                           powers_dev.data_ptr(), y_local.data_ptr(), n_local, k, m, n_local, flags))
            dist.all_gather_into_tensor(gathered, y_local)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if peers is not None:       # one trial step: if any rank's peer gather fails, every rank goes to NCCL together
        trial = 1
        try:
            step(0)
            torch.cuda.synchronize()
            check(lib.weft_b200_synchronize())
        except SystemExit as error:
            sys.stderr.write(f"rank {rank}: peer gather failed ({error}); using NCCL\n")
            trial = 0
        agreed = torch.tensor([trial], device="cuda")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            peers.close(dist.barrier)
            peers, collective = None, "nccl"

    # ---- parity spot check before timing (one step against the oracle, rank-local columns)
    step(0)
    torch.cuda.synchronize()
    check(lib.weft_b200_synchronize())
    if peers is not None:     # the gathered output of this rank: own columns, and a block computed by the next rank
        full = np.empty((m, n), dtype=np.float32)
        check(lib.weft_b200_peer_read(full.ctypes.data, peers.local[(calls[0] - 1) % 2], full.nbytes))
        got = full[:, n0:n1]
        other = (rank + 1) % world
        o0 = n * other // world
        span = min(64, n * (other + 1) // world - o0)
        want_other, _ = oracle.mul_mat(oracle.FORMAT_IDS[fmt], w_host[o0:o0 + span], x_host[:1], span, k, 1, rule=1, grid=grid, signs=signs)
        err_other = float(np.linalg.norm(full[:1, o0:o0 + span].astype(np.float64) - want_other) / max(np.linalg.norm(want_other.astype(np.float64)), 1e-30))
        if not err_other <= 1e-5:
            raise SystemExit(f"gathered columns of rank {other} differ from the oracle on rank {rank}: relative L2 {err_other}")
    else:
        got = (y_dev[:, n0:n1] if world == 1 else y_local).cpu().numpy()
    probe = min(n_local, 256)
    want, _ = oracle.mul_mat(oracle.FORMAT_IDS[fmt], shard[:probe], x_host[: min(m, 4)], probe, k, min(m, 4), rule=1, grid=grid, signs=signs)
    err = float(np.linalg.norm(got[: min(m, 4), :probe].astype(np.float64) - want) / max(np.linalg.norm(want.astype(np.float64)), 1e-30))
    if not err <= 1e-5:
        raise SystemExit(f"parity check failed before timing ({workload}): relative L2 {err}")

    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    replays = max(1, args.replays)

    def run_timed(fn, steps: int, first: int) -> tuple[list[float], str]:
        """Device times (ms) of `steps` consecutive calls of fn, taken `replays` times.  The calls are captured once
        into a CUDA graph and each timing is one replay of that graph between two events on the launching stream, so
        host launch cost (Python + ctypes, several microseconds per call, comparable to the kernel itself) stays out of
        the measurement.  An even number of steps keeps the two alternating gather buffers in step from replay to
        replay.  Falls back to direct launches when capture is refused."""
        if not args.no_graph:
            side = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            try:
                side.wait_stream(torch.cuda.current_stream())
                lib.weft_b200_set_stream(ctypes.c_void_p(side.cuda_stream))
                with torch.cuda.graph(graph, stream=side):
                    for i in range(steps):
                        fn(first + i)
                lib.weft_b200_set_stream(ctypes.c_void_p(stream.cuda_stream))
                graph.replay()          # untimed: first replay uploads the graph
                times = []
                for _ in range(replays):
                    barrier()
                    begin.record()
                    graph.replay()
                    end.record()
                    barrier()
                    times.append(begin.elapsed_time(end))
                return times, "cuda graph replay of all steps"
            except Exception as error:  # capture refused: measure direct launches instead
                lib.weft_b200_set_stream(ctypes.c_void_p(stream.cuda_stream))
                torch.cuda.synchronize()
                sys.stderr.write(f"graph capture unavailable ({error}); timing direct launches\n")
        times = []
        for _ in range(replays):
            barrier()
            begin.record()
            for i in range(steps):
                fn(first + i)
            end.record()
            barrier()
            times.append(begin.elapsed_time(end))
        return times, "direct launches"

    def over_ranks(values: list[float]) -> list[float]:
        if world == 1:
            return values
        t = torch.tensor(values, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    steps = args.steps + (args.steps % 2 if peers is not None else 0)

    # ---- timed region: K steps on the device, `replays` times
    for i in range(args.warmup + (args.warmup + calls[0]) % 2 if peers is not None else args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches_before = lib.weft_b200_launch_count()
    step_times, launch_mode = run_timed(step, steps, args.warmup)
    launches = int(lib.weft_b200_launch_count() - launches_before)     # kernels captured for one pass over the steps
    check(lib.weft_b200_synchronize())
    step_times = over_ranks(step_times)
    if world > 1:
        lt = torch.tensor([launches], device="cuda")
        dist.all_reduce(lt)
        launches = int(lt.item())
    ms_per_step = statistics.median(step_times) / steps

    # ---- the dominant kernel alone (activations already quantized, no collective): average launch duration
    def kernel_step(i: int) -> None:
        out = y_dev if world == 1 else y_local
        check(shard_fn(fid, mode_id, w_dev[i % copies].data_ptr(), x_dev.data_ptr(), xq_dev.data_ptr(), grid_dev.data_ptr(),
                       signs_dev.data_ptr(), powers_dev.data_ptr(), out.data_ptr(), n_local, k, m, n if world == 1 else n_local, 1))

    for i in range(args.warmup):
        kernel_step(i)
    barrier()
    kernel_times, _ = run_timed(kernel_step, steps, args.warmup)
    kernel_times = over_ranks(kernel_times)
    kernel_ms = statistics.median(kernel_times) / steps
    clocks = sampler.stop() if rank == 0 else None

    e2e = None
    if extras:
        # ---- end to end through the C ABI with host buffers (weights resident on the device): pinned X in, the FULL
        # (m, n) output back on the host.  One GPU: the plain entry point with host X / Xq / Y.  Several GPUs: the
        # gathering entry point with host X, then the gathered output read back from this rank's buffer.
        x_pin = torch.from_numpy(x_host).pin_memory()
        xq_pin = torch.zeros((m, row_bytes(act, k)), dtype=torch.uint8).pin_memory()
        y_pin = torch.zeros((m, n), dtype=torch.float32).pin_memory()
        grid_pin, signs_pin = torch.from_numpy(grid).pin_memory(), torch.from_numpy(signs).pin_memory()
        powers_pin = powers_dev if fmt == "IQ1_M" else torch.tensor(TQ1_POWERS, dtype=torch.int32).pin_memory()   # 256 KB: kept on the device
        y_page = np.zeros((m, n), dtype=np.float32)      # pageable memory, what a plain numpy caller of the reference passes
        x_page, xq_page = x_host.copy(), np.zeros((m, row_bytes(act, k)), dtype=np.uint8)

        # addresses taken once: a C caller of the entry point has them at hand, the interpreter would spend 2 us per step on them
        w_ptrs = [w.data_ptr() for w in w_dev]
        host_ptrs = {True: (x_pin.data_ptr(), xq_pin.data_ptr(), y_pin.data_ptr()),
                     False: (x_page.ctypes.data, xq_page.ctypes.data, y_page.ctypes.data)}
        table_ptrs = (grid_pin.data_ptr(), signs_pin.data_ptr(), powers_pin.data_ptr())

        def e2e_step(i: int, pinned: bool = True) -> None:
            if world == 1:
                xs = host_ptrs[pinned]
                check(shard_fn(fid, mode_id, w_ptrs[i % copies], xs[0], xs[1], table_ptrs[0], table_ptrs[1], table_ptrs[2],
                               xs[2], n_local, k, m, n, 0))
            elif peers is not None:
                step(i, 0, x_pin.data_ptr(), None)
                check(lib.weft_b200_peer_read(y_pin.data_ptr(), peers.local[(calls[0] - 1) % 2], 4 * m * n))
            else:
                step(i, 0, x_pin.data_ptr(), None)
                torch.cuda.synchronize()
                y_pin.view(m, world, n_local).copy_(gathered.view(world, m, n_local).permute(1, 0, 2))

        lib.weft_b200_set_async(0 if world == 1 else 1)
        e2e_steps = max(3, min(args.steps, 200))

        def e2e_time(pinned: bool) -> float:
            for i in range(3):
                e2e_step(i, pinned)
            barrier()
            t0 = time.perf_counter()
            for i in range(e2e_steps):
                e2e_step(3 + i, pinned)
            torch.cuda.synchronize()
            seconds = (time.perf_counter() - t0) / e2e_steps
            if world > 1:
                t = torch.tensor([seconds], device="cuda", dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                seconds = float(t.item())
            return seconds

        e2e_s = e2e_time(True)
        e2e_err = float(np.abs(y_pin.numpy()[: min(m, 4), n0:n0 + probe] - got[: min(m, 4), :probe]).max())
        if e2e_err != 0.0:
            raise SystemExit(f"host-buffer path disagrees with the device-buffer path by {e2e_err}")
        e2e_pageable_s = e2e_time(False) if world == 1 else None
        lib.weft_b200_set_async(1)
        e2e = {"seconds": e2e_s, "pageable_seconds": e2e_pageable_s, "h2d": int(x_pin.numel() * 4),
               "d2h": int(4 * m * n + (xq_pin.numel() if world == 1 else 0))}

    if peers is not None:
        torch.cuda.synchronize()
        peers.close(dist.barrier)
    del w_dev, x_dev, xq_dev, y_dev, gathered, y_local
    torch.cuda.empty_cache()
    if rank != 0:
        return None

    peaks, peaks_kind = load_peaks()
    total_bytes = algorithmic_bytes(fmt, n, k, m)
    spread = (max(step_times) - min(step_times)) / statistics.median(step_times) if len(step_times) > 1 else 0.0
    kernel_spread = (max(kernel_times) - min(kernel_times)) / statistics.median(kernel_times) if len(kernel_times) > 1 else 0.0
    if mode == "decode":
        metric, unit = "mul_mat_decode_algorithmic_gbps", "GB/s"
        value = total_bytes / (ms_per_step * 1e-3) / 1e9
        e2e_value = total_bytes / e2e["seconds"] / 1e9 if e2e else None
        e2e_pageable = total_bytes / e2e["pageable_seconds"] / 1e9 if e2e and e2e["pageable_seconds"] else None
        shard_bytes = algorithmic_bytes(fmt, n_local, k, m)
        achieved = shard_bytes / (kernel_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "traffic": ncu_traffic(workload, n_local / n), "peak_source": peaks_kind, "kernel": "gemv_kernel (per GPU)", "kernel_ms": kernel_ms,
                "kernel_ms_spread": kernel_spread, "algorithmic_bytes_per_launch": shard_bytes}
        dtype = "int8 dot (dp4a), f32 accumulate"
    else:
        metric, unit = "mul_mat_prefill_int8_tops", "TOP/s"
        ops = 2.0 * m * n * k
        value = ops / (ms_per_step * 1e-3) / 1e12
        e2e_value = ops / e2e["seconds"] / 1e12 if e2e else None
        e2e_pageable = ops / e2e["pageable_seconds"] / 1e12 if e2e and e2e["pageable_seconds"] else None
        achieved = 2.0 * m * n_local * k / (kernel_ms * 1e-3) / 1e12
        peak = 2.0 * peaks["bf16_tflops"]
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s", "frac": achieved / peak, "traffic": ncu_traffic(workload, n_local / n),
                "peak_source": peaks_kind + " bf16 dense x2 (no int8 entry in MEASURED_PEAKS.json)", "kernel": "prefill kernel (per GPU)",
                "kernel_ms": kernel_ms, "kernel_ms_spread": kernel_spread}
        int8_peak = measured_int8_peak(lib)
        if int8_peak:
            roof["int8_issue_peak"] = int8_peak
            roof["frac_of_int8_issue_peak"] = achieved / int8_peak
        dtype = "int8 tensor-core MMA, i32/f32 accumulate"

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype,
        "data": "synthetic",
        "config": {"workload": workload, "format": layout, "mode": mode, "N": n, "K": k, "M": m,
                   "sharding": (f"weight rows split {world} ways, fp32 outputs all-gathered " + ("by peer stores and a flag barrier inside the library's kernels (NVLink, CUDA IPC)" if collective == "p2p" else "(NCCL)")) if world > 1 else "none",
                   "l2": f"steps rotate over {copies} weight copies ({copies * shard.nbytes / 2**20:.0f} MiB per GPU > 2 x L2)",
                   "launch": launch_mode, "timing": f"median of {len(step_times)} replays of {steps} steps, max over ranks",
                   "replay_spread": spread, "timed_scope": "activation quantize + mul_mat" + (" + all-gather" if world > 1 else ""), "seed": SEED,
                   "parity_rel_l2_before_timing": err},
        "roofline": roof, "clocks": clocks, "gpu_launches": launches,
    }
    if e2e:
        line["e2e"] = {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                       "ms_per_step": e2e["seconds"] * 1e3,
                       "what": ("weft_b200_mul_mat_shard with host X/Xq/Y (pinned), weights resident in HBM" if world == 1 else
                                "weft_b200_mul_mat_shard_gather with host X (pinned) and the gathered (M, N) output read back to the host, weights resident in HBM")}
        if e2e_pageable:
            line["e2e"]["pageable"] = {"value": e2e_pageable, "ms_per_step": e2e["pageable_seconds"] * 1e3,
                                       "what": "the same call with pageable (plain numpy) X / Xq / Y, as the reference's FFI passes them"}
    if extras and not args.no_cpu_baseline and world == 1:
        threads = os.cpu_count() or 1
        sample_m = m if mode == "decode" else min(m, 2)
        run, kind = cpu_mul_mat_runner(fmt, n, k, sample_m, w_host, x_host[:sample_m], grid, signs, threads)
        run()
        times, t_end = [], time.perf_counter() + 12.0
        while time.perf_counter() < t_end and len(times) < 200:
            t0 = time.perf_counter(); run(); times.append(time.perf_counter() - t0)
        per = sum(times) / len(times)
        cpu_value = (algorithmic_bytes(fmt, n, k, m) / per / 1e9) if mode == "decode" else (2.0 * sample_m * n * k / per / 1e12)
        line["cpu_baseline"] = {"value": cpu_value, "unit": unit, "cores": threads, "kind": kind,
                                "sample": f"{len(times)} x full mul_mat N={n} K={k} M={sample_m}" + ("" if sample_m == m else f" of M={m}"),
                                "cpu": oracle.cpu_model(), "ms_per_step": per * 1e3 * (m / sample_m)}
        single = cpu_single_thread(fmt, n, k, sample_m, w_host, x_host[:sample_m], grid, signs)
        if single:
            single["value"] = (algorithmic_bytes(fmt, n, k, m) / single["seconds"] / 1e9) if mode == "decode" else (2.0 * sample_m * n * k / single["seconds"] / 1e12)
            single["unit"] = unit
            line["cpu_baseline"]["single_thread"] = single
    return line


_INT8_PEAK = []


def measured_int8_peak(lib):
    """TOP/s of a bare tcgen05.mma kind::i8 issue loop on every SM (weft_b200_mma_peak), measured once per process."""
    if not _INT8_PEAK:
        lib.weft_b200_mma_peak.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
        value = ctypes.c_double()
        _INT8_PEAK.append(float(value.value) if lib.weft_b200_mma_peak(0, ctypes.byref(value)) == 0 else None)
    return _INT8_PEAK[0]


def cpu_single_thread(fmt, n, k, m, w, x, grid, signs):
    """The reference's own protocol for its CPU numbers (doc/experiments/protocol.md:33-59): one pinned thread, a 64 MiB
    buffer rewritten between repetitions so that every repetition starts cold, median of the repetitions.  Bounded to a
    few seconds: at most 4096 weight rows per repetition."""
    import oracle

    rows = min(n, 4096)
    run, kind = cpu_mul_mat_runner(fmt, rows, k, m, np.ascontiguousarray(w[:rows]), x, grid, signs, 1)
    try:
        previous = os.sched_getaffinity(0)
        os.sched_setaffinity(0, {sorted(previous)[0]})
    except (AttributeError, OSError):
        previous = None
    evict = np.zeros(64 << 20, dtype=np.uint8)
    try:
        run()
        times, t_end = [], time.perf_counter() + 6.0
        while time.perf_counter() < t_end and len(times) < 10:
            evict += 1
            t0 = time.perf_counter(); run(); times.append(time.perf_counter() - t0)
    finally:
        if previous is not None:
            os.sched_setaffinity(0, previous)
    return {"seconds": statistics.median(times) * (n / rows), "kind": kind, "cores": 1,
            "sample": f"median of {len(times)} cold repetitions of {rows} of {n} rows, one pinned thread, 64 MiB rewritten between repetitions"}


#: the other configurations of the headline metric, reported as compact records beside the default line
ALSO_WORKLOADS = ["q4_0_decode_4096x4096", "q4_k_dequantize_14336x4096", "q4_k_decode_4096x4096", "q4_k_decode_4096x14336",
                  "q4_k_prefill_4096x4096", "q4_k_prefill_14336x4096", "q4_k_prefill_4096x14336", "iq2_xxs_decode_28672x8192",
                  "tq1_0_prefill_28672x8192"]
#: the ones the metric shards over several GPUs (prefill with N = 14336; the 28672 x 8192 layer)
ALSO_SHARDED = ["q4_k_prefill_14336x4096", "iq2_xxs_decode_28672x8192", "tq1_0_prefill_28672x8192"]


def also_records(args, lib, check, stream, world, rank, local_rank) -> list[dict]:
    """One compact record per further configuration of the metric, measured like the default line (median of the
    replays of `steps` graph-captured steps, weights rotating through more than twice the L2, parity checked first)."""
    import copy

    quick = copy.copy(args)
    quick.steps, quick.warmup = max(2, min(args.steps, 10)), 3
    records = []
    for workload in (ALSO_WORKLOADS if world == 1 else ALSO_SHARDED):
        fmt, mode, n, k, _ = WORKLOADS[workload]
        if mode == "dequantize":
            line = gpu_dequantize(quick, lib, check, stream, fmt, n, k, world, rank, local_rank, extras=False)
        else:
            line = run_mul_mat(quick, lib, check, stream, workload, world, rank, local_rank, extras=False)
        if line is not None:
            records.append({"workload": workload, "n_gpus": world, "ms_per_step": line["ms_per_step"], "value": line["value"], "unit": line["unit"],
                            "frac": line["roofline"]["frac"], "bound": line["roofline"]["bound"], "kernel_ms": line["roofline"]["kernel_ms"],
                            "parity_rel_l2": line["config"].get("parity_rel_l2_before_timing", 0.0), "replays": args.replays,
                            "replay_spread": line["config"].get("replay_spread"), "steps": line["steps"]})
    return records

if __name__ == "__main__":
    main()
