"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload gemv|decode|quantize] [--rows M] [--batch B]

Prints ONE JSON line.  Workloads:

* `gemv` (default) -- the W4A16 g128 decode product the headline metric is quoted on:
  K=4096, N=14336 (Llama-3-8B gate/up), x bf16 [M, K], M=1 for `value` (M=4 and 16 under
  `per_rows`, measured the same way).  One step is 64 launches cycling through 8 distinct
  weight sets (246 MB, larger than the 126 MB L2, so every launch streams its weights from
  HBM), recorded once into a CUDA graph and replayed.  Every number is the median of 5 trials
  of `--steps` replays each.  `value` calls the plain entry point; `chained_early` is the same
  chain with B200Q_EARLY_DEPENDENTS, the flag a caller sets when the next kernel is another
  product (which this chain is); `isolated` times one launch alone, from the host and, under
  `in_stream_order`, on the device (the chain with B200Q_NO_OVERLAP).  With N ranks every rank runs this on its own GPU and weight
  sets (`value` is the sum).  The line also carries `decode`: tokens/s of a Llama-3.1-8B-shaped
  int4 decoder step, tensor-parallel over the N ranks (linnet_b200/decoder.py), at batch 1, 8
  and 64, and `other_configs` (int8 GEMV, prefill GEMM against dequantize + library GEMM,
  quantize kernels).
* `--workload decode` -- only the decoder, tokens/s as `value`.
* `--workload quantize` -- bulk quantize / pack of Llama-3-70B-shaped bf16 weights to int4-g128
  and int8 per-channel, every tensor sharded by output rows over the N ranks (no exchange);
  one step is one decoder layer's seven tensors in both formats; GB/s of algorithmic bytes.

`--impl reference` times the reference's own CPU route for the same workload on the host
cores: the reference itself out of `oracle/_ref` where that has been built
(`cpu_baseline.kind` "reference"), else the oracle's restatement of it ("port").
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import tempfile
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

K_IN, N_OUT, GROUP = 4096, 14336, 128
WEIGHT_SETS = 8
LAUNCHES_PER_STEP = 64
TRIALS = 5
METRIC = "W4A16 g128 GEMV GB/s (% HBM peak); 8B-shape int4 decode tok/s at 1/2/4/8 GPU"


def gemv_bytes(rows: int, depth: int = K_IN, out: int = N_OUT) -> int:
    """Algorithmic bytes of one launch: packed nibbles + bf16 scales + u8 zero points,
    plus the activations read and the outputs written."""
    groups = depth // GROUP
    return out * depth // 2 + out * groups * 3 + rows * depth * 2 + rows * out * 2


def peaks() -> tuple[float, float, str]:
    """(HBM GB/s, dense bf16 TFLOP/s burst, "measured" | "fallback")."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        found = json.loads(path.read_text())
        return float(found["hbm_gbs"]), float(found["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def dram_traffic(key: str) -> dict | None:
    """DRAM bytes per launch of a kernel from its ncu capture, as recorded beside the ncu
    summaries (dram__bytes_read.sum + dram__bytes_write.sum); None when there is no capture."""
    path = ROOT / "profiles" / "dram_traffic.json"
    if not path.exists():
        return None
    return json.loads(path.read_text()).get(key)


def quantize_traffic(weights: int) -> dict:
    """DRAM bytes of one step of the quantize workload (both formats of `weights` weights): the
    per-weight traffic of the two kernels' ncu captures on 8192 x 8192 (it grows in proportion
    to the weights: every weight is read once and its level written once) times the weights."""
    found = [dram_traffic("quantize_int4_g128_8192x8192"), dram_traffic("quantize_int8_channel_8192x8192")]
    if not all(found):
        return {"traffic": None}
    per_weight = sum(f["bytes_per_launch"] for f in found) / (8192 * 8192)
    return {"traffic": per_weight * weights,
            "traffic_source": "per-weight DRAM bytes of the two kernels' ncu captures on 8192 x 8192 "
                              "(profiles/dram_traffic.json), times this step's weights"}


class Clocks:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.rows: list[list[str]] = []
        self.stop = threading.Event()
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _sample(self) -> None:
        try:
            out = subprocess.run(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
            for line in out.strip().splitlines():
                self.rows.append([c.strip() for c in line.split(",")])
        except Exception:
            pass

    def _run(self) -> None:
        while not self.stop.is_set():
            self._sample()
            self.stop.wait(0.1)

    def __enter__(self) -> "Clocks":
        self.thread.start()
        return self

    def __exit__(self, *exc: object) -> None:
        self.stop.set()
        self.thread.join(timeout=10)

    def summary(self) -> dict:
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        top = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) > 3 + i and r[3 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(top) if top else None, "reasons": reasons,
                "samples": len(sm)}


# ---- timing --------------------------------------------------------------------------


def time_replays(graph: torch.cuda.CUDAGraph, steps: int, warmup: int, barrier, reduce_max,
                 trials: int = TRIALS) -> dict:
    """Milliseconds per step: `trials` trials of `steps` replays, each device-timed with CUDA
    events on the current stream between barriers; the median trial (max over ranks)."""
    for _ in range(max(3, warmup)):
        graph.replay()
    torch.cuda.synchronize()
    per_step = []
    for _ in range(trials):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        barrier()
        per_step.append(reduce_max(start.elapsed_time(stop)) / steps)
    return {"ms_per_step": statistics.median(per_step), "trials_ms_per_step": per_step,
            "timed_seconds": sum(per_step) * steps / 1e3}


# ---- the reference's CPU route ---------------------------------------------------------


def reference_run(what: str, *extra: str, timeout: int = 900) -> dict | None:
    """Runs oracle/run_reference.py in a process that sees the reference built into
    oracle/_ref; None when that has not been built."""
    from oracle import build_ref

    if not build_ref.available():
        return None
    home = Path(tempfile.mkdtemp(prefix="linnet-home-"))
    env = build_ref.environment(home)
    done = subprocess.run([sys.executable, str(ROOT / "oracle" / "run_reference.py"), what, *extra], env=env,
                          capture_output=True, text=True, timeout=timeout)
    if done.returncode != 0:
        return None
    return json.loads(done.stdout.strip().splitlines()[-1])


def cpu_port_gemv(rows: int, sets: int, reps: int, warm: int) -> dict:
    """The oracle's restatement of the reference's CPU route (python/linnet/src/linnet/torch/
    native.py:417-424; src/backend/torch_source.cpp:1501-1504, :1568): W dequantized once to
    bf16 by `prepare`, then `F.linear(x, W)` per call, on every host core."""
    from oracle import linear_oracle as lo
    from oracle import quant_oracle as qo

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(0)
    weights = []
    for _ in range(sets):
        w = torch.randn(N_OUT, K_IN, generator=gen) * 0.02
        packed, scale, zero = qo.quantize_int4_groups(w.numpy(), GROUP)
        weights.append(lo.int4_weight(torch.from_numpy(packed), torch.from_numpy(scale).to(torch.bfloat16),
                                      torch.from_numpy(zero), torch.bfloat16))
    x = torch.randn(rows, K_IN, generator=gen).to(torch.bfloat16)
    times = []
    for i in range(warm + reps):
        t0 = time.perf_counter()
        for w in weights:
            torch.nn.functional.linear(x, w)
        if i >= warm:
            times.append((time.perf_counter() - t0) / len(weights))
    per_call = statistics.median(times)
    return {"seconds_per_call": per_call, "GB/s": gemv_bytes(rows) / per_call / 1e9, "cores": threads,
            "what": f"oracle restatement: F.linear(x[{rows},{K_IN}] bf16, W bf16 [{N_OUT},{K_IN}] dequantized once) "
                    f"over {sets} weight sets x {reps} passes after {warm}; bytes counted as the packed int4 layout's"}


def cpu_baseline_gemv(rows: int, sets: int, reps: int, warm: int) -> dict:
    """The reference's CPU route timed on this box's host cores: a bounded sample."""
    found = reference_run("gemv", "--rows", str(rows), "--sets", str(sets), "--reps", str(reps), "--warm", str(warm))
    kind = "reference"
    if found is None:
        found, kind = cpu_port_gemv(rows, sets, reps, warm), "port"
    return {"value": found["GB/s"], "unit": "GB/s", "cores": found["cores"], "kind": kind,
            "ms_per_call": found["seconds_per_call"] * 1e3, "sample": found["what"]}


# ---- synthetic weights -----------------------------------------------------------------


def make_weight_sets(device: torch.device, count: int):
    """`count` int4-g128 weight sets of W ~ N(0, 0.02) [N_OUT, K_IN], quantized by the
    GPU quantizer (bit-exact with the reference's), scales stored as bf16."""
    from linnet_b200 import quant

    sets = []
    gen = torch.Generator(device="cpu").manual_seed(0)
    for _ in range(count):
        w = (torch.randn(N_OUT, K_IN, generator=gen) * 0.02).to(device)
        packed, _scale, zero, stored = quant.quantize_int4_groups(w, GROUP, scale_dtype="bf16")
        sets.append((packed, stored, zero))
    return sets


# ---- the gemv workload -------------------------------------------------------------------


def run_gemv(args, rank: int, world: int, device: torch.device, barrier, reduce_max) -> dict:
    from linnet_b200 import kernels

    sets = make_weight_sets(device, WEIGHT_SETS)
    gen = torch.Generator().manual_seed(1)
    stream = torch.cuda.Stream(device)
    results: dict[str, dict] = {}
    clocks = None

    def chain(x: torch.Tensor, early: bool, overlap: bool = True) -> torch.cuda.CUDAGraph:
        for p, s, z in sets[:2]:
            kernels.int4_linear(x, p, s, z, early=early)  # warm: module load, attribute set-up
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(LAUNCHES_PER_STEP):
                p, s, z = sets[i % WEIGHT_SETS]
                kernels.int4_linear(x, p, s, z, early=early, overlap=overlap)
        return graph

    with torch.cuda.stream(stream):
        xs = {rows: torch.randn(rows, K_IN, generator=gen).to(torch.bfloat16).to(device)
              for rows in sorted({args.rows, 1, 4, 16})}
        graph = chain(xs[args.rows], False)
        with Clocks(device.index or 0) as clocks:
            results["main"] = time_replays(graph, args.steps, args.warmup, barrier, reduce_max)
        del graph
        for rows in (1, 4, 16):
            if rows == args.rows:
                results[str(rows)] = results["main"]
                continue
            graph = chain(xs[rows], False)
            results[str(rows)] = time_replays(graph, args.steps, 3, barrier, reduce_max)
            del graph
        graph = chain(xs[args.rows], True)
        results["early"] = time_replays(graph, args.steps, 3, barrier, reduce_max)
        del graph
        # the same chain in plain stream order: every launch starts when the one before it has
        # finished (no early start, no weight fetch under the predecessor)
        graph = chain(xs[args.rows], False, overlap=False)
        results["serial"] = time_replays(graph, args.steps, 3, barrier, reduce_max)
        del graph

        # One launch at a time with the stream drained in between: no overlap with a neighbour,
        # launch latency and the kernel's own ramp-up and drain all inside the number.
        alone = []
        for i in range(3 * WEIGHT_SETS + 3):
            p, s, z = sets[i % WEIGHT_SETS]
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            stream.synchronize()
            start.record(stream)
            kernels.int4_linear(xs[args.rows], p, s, z)
            stop.record(stream)
            stop.synchronize()
            if i >= 3:
                alone.append(start.elapsed_time(stop) * 1e3)
        isolated_us = reduce_max(statistics.median(alone))

        # End to end through the operator with HOST buffers: per step the activations come
        # from pinned host memory and the last result goes back to the host, all of it (copies
        # and the 64 products) one CUDA-graph replay followed by a wait for the result.
        rows = args.rows
        host_x = torch.randn(rows, K_IN, generator=gen).to(torch.bfloat16).pin_memory()
        host_y = torch.empty(rows, N_OUT, dtype=torch.bfloat16).pin_memory()
        dev_x = torch.empty(rows, K_IN, dtype=torch.bfloat16, device=device)
        for p, s, z in sets[:2]:
            kernels.int4_linear(dev_x, p, s, z)
        torch.cuda.synchronize()
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph, stream=stream):
            dev_x.copy_(host_x, non_blocking=True)
            y = None
            for i in range(LAUNCHES_PER_STEP):
                p, s, z = sets[i % WEIGHT_SETS]
                y = kernels.int4_linear(dev_x, p, s, z)
            host_y.copy_(y, non_blocking=True)
        for _ in range(3):
            e2e_graph.replay()
            stream.synchronize()
        e2e_trials = []
        for _ in range(TRIALS):
            barrier()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                e2e_graph.replay()
                stream.synchronize()
            e2e_trials.append(reduce_max((time.perf_counter() - t0) * 1e3) / args.steps)
        e2e_ms = statistics.median(e2e_trials)
        del e2e_graph
    hbm, _tf, peak_kind = peaks()
    ms_step = results["main"]["ms_per_step"]
    per_launch_s = ms_step / 1e3 / LAUNCHES_PER_STEP
    achieved = gemv_bytes(args.rows) / per_launch_s / 1e9
    traffic = dram_traffic(f"int4_gemv_k{K_IN}_n{N_OUT}_m{args.rows}")

    def rate(ms: float, m: int) -> dict:
        us = ms * 1e3 / LAUNCHES_PER_STEP
        return {"GB/s": gemv_bytes(m) / us / 1e3, "us_per_launch": us, "frac_hbm": gemv_bytes(m) / us / 1e3 / hbm}

    line = {
        "metric": METRIC,
        "value": achieved * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int4 weights, bf16 activations, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"W4A16 g128 GEMV K={K_IN} N={N_OUT} M={args.rows}",
                   "launches_per_step": LAUNCHES_PER_STEP, "weight_sets": WEIGHT_SETS,
                   "l2_policy": f"inputs larger than L2: {WEIGHT_SETS} weight sets, "
                                f"{WEIGHT_SETS * gemv_bytes(1) / 1e6:.0f} MB, visited round-robin",
                   "timing": f"median of {TRIALS} trials of --steps CUDA-graph replays, CUDA events on the "
                             f"launching stream, max over ranks",
                   "numerics": kernels.int4_numerics(), "replicas": world},
        "trials_ms_per_step": results["main"]["trials_ms_per_step"],
        "timed_seconds": results["main"]["timed_seconds"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s",
                     "frac": achieved / hbm, "peak_kind": peak_kind,
                     "frac_of_8tbs_nominal": achieved / 8000.0,
                     "algorithmic_bytes_per_launch": gemv_bytes(args.rows),
                     "us_per_launch": per_launch_s * 1e6,
                     "traffic": traffic["bytes_per_launch"] if traffic else None,
                     "traffic_source": traffic["source"] if traffic else None},
        "per_rows": {str(m): rate(results[str(m)]["ms_per_step"], m) for m in (1, 4, 16)},
        "chained_early": rate(results["early"]["ms_per_step"], args.rows),
        "isolated": {"us_per_launch": isolated_us, "GB/s": gemv_bytes(args.rows) / isolated_us / 1e3,
                     "how": "one launch between two events, the stream drained before each (the host's launch "
                            f"latency is inside); median over {3 * WEIGHT_SETS} launches visiting the weight sets in turn",
                     "in_stream_order": {**rate(results["serial"]["ms_per_step"], args.rows),
                                         "how": "the 64-launch graph with B200Q_NO_OVERLAP: every launch starts when "
                                                "the one before it has finished, on the device's own clock"}},
        "e2e": {"value": gemv_bytes(rows) * LAUNCHES_PER_STEP / (e2e_ms / 1e3) / 1e9 * world,
                "unit": "GB/s", "ms_per_step": e2e_ms, "trials_ms_per_step": e2e_trials,
                "h2d_bytes_per_step": rows * K_IN * 2, "d2h_bytes_per_step": rows * N_OUT * 2,
                "how": "one CUDA-graph replay per step: pinned host x -> device, 64 products, last y -> pinned "
                       "host, then a wait for it"},
        "gpu_launches": args.steps * LAUNCHES_PER_STEP * TRIALS,
        "clocks": clocks.summary() if clocks else None,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_gemv(args.rows, sets=4, reps=5, warm=2)
    if rank == 0 and not args.no_other_configs:
        del sets
        torch.cuda.empty_cache()
        line["other_configs"] = other_configs(device, with_cpu=world == 1 and not args.no_cpu_baseline)
    return line


def _time_us(fn, reps: int, warm: int = 3, trials: int = 3) -> float:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    found = []
    for _ in range(trials):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(reps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        found.append(start.elapsed_time(stop) * 1e3 / reps)
    return statistics.median(found)


def other_configs(device: torch.device, with_cpu: bool) -> dict:
    """Short measurements of the other workloads (not the headline): the int8 per-channel
    GEMV (BASELINE config 1 on the GPU, with the reference's CPU run beside it), the prefill
    dequant-GEMM at M=2048 beside a comparator that dequantizes the weight and calls the
    library GEMM (the reference's own many-row route, never the product path), and the bulk
    quantize / pack kernels on one 70B-shaped tensor.  Inputs are larger than L2 or rotated."""
    from linnet_b200 import kernels, quant

    hbm, bf16_peak, _ = peaks()
    out: dict = {}
    gen = torch.Generator(device=device).manual_seed(3)
    # int8 symmetric per-output-channel GEMV, M=1, K=N=4096 (16 weight sets = 268 MB)
    for width in (4096, 14336):
        count = 16 if width == 4096 else 6
        sets8 = []
        for _ in range(count):
            w = torch.empty(width, 4096, device=device).normal_(0, 0.02, generator=gen)
            q, s = quant.quantize_int8_groups(w, 4096, "f32")
            sets8.append((q, s.reshape(-1).contiguous()))
        x1 = torch.randn(1, 4096, device=device, generator=gen).to(torch.bfloat16)
        stream = torch.cuda.Stream(device)
        with torch.cuda.stream(stream):
            kernels.gemv8(x1, *sets8[0], False, 0, 1)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(64):
                    kernels.gemv8(x1, *sets8[i % count], False, 0, 1)
            us = _time_us(graph.replay, 20, trials=5) / 64
        nbytes = width * 4096 + width * 4 + 4096 * 2 + width * 2
        entry = {"us": us, "GB/s": nbytes / us / 1e3, "frac_hbm": nbytes / us / 1e3 / hbm,
                 "note": f"64 launches over {count} weight sets in one CUDA graph, median of 5 trials"}
        if width == 4096 and with_cpu:
            ref = reference_run("int8", "--rows", "1", "--reps", "5", "--warm", "2")
            if ref is not None:
                entry["cpu_baseline"] = {"value": ref["GB/s"], "unit": "GB/s", "cores": ref["cores"], "kind": "reference",
                                         "ms_per_call": ref["seconds_per_call"] * 1e3, "sample": ref["what"]}
        out[f"int8_gemv_M1_K4096_N{width}"] = entry
        del graph, sets8
    # prefill dequant-GEMM, M = 2048, beside dequantize + library GEMM
    x = torch.randn(2048, 14336, device=device, generator=gen).to(torch.bfloat16)
    for K, N in ((4096, 6144), (4096, 28672), (14336, 4096)):
        w = torch.empty(N, K, device=device, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
        packed, _s, zero, scale = quant.quantize_int4_groups(w, GROUP, scale_dtype="bf16")
        del w
        xk = x[:, :K].contiguous()
        us = _time_us(lambda: kernels.int4_linear(xk, packed, scale, zero), 10)
        us_cmp = _time_us(lambda: torch.matmul(xk, kernels.int4_dequantize(packed, scale, zero).T), 10)
        tf = 2.0 * 2048 * N * K / us / 1e6
        out[f"int4_gemm_M2048_K{K}_N{N}"] = {"us": us, "TFLOP/s": tf, "frac_bf16_peak": tf / bf16_peak,
                                             "comparator_dequantize_plus_library_gemm_us": us_cmp,
                                             "faster_than_comparator": us < us_cmp}
    # the 33..128-row range of the same kernel
    xk = x[:64, :4096].contiguous()
    w = torch.empty(28672, 4096, device=device, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
    packed, _s, zero, scale = quant.quantize_int4_groups(w, GROUP, scale_dtype="bf16")
    del w
    us = _time_us(lambda: kernels.int4_linear(xk, packed, scale, zero), 20)
    out["int4_gemm_M64_K4096_N28672"] = {"us": us, "GB/s": gemv_bytes(64, 4096, 28672) / us / 1e3,
                                         "frac_hbm": gemv_bytes(64, 4096, 28672) / us / 1e3 / hbm}
    del x, xk, packed, scale, zero
    torch.cuda.empty_cache()
    # W8A8 (the reference's many-row route of int8 layers under numerics="fast"): rows of x to int8,
    # then the int8 x int8 product on the tensor cores, M = 2048, K = 4096, N = 14336
    x8 = torch.randn(2048, 4096, device=device, generator=gen).to(torch.bfloat16)
    w8 = torch.empty(14336, 4096, device=device).normal_(0, 0.02, generator=gen)
    q8, s8 = quant.quantize_int8_groups(w8, 4096, "f32")
    s8 = s8.reshape(-1).contiguous()
    del w8
    if kernels.int8_mm_available(q8):
        xq, xs = kernels.int8_rows(x8)
        us_rows = _time_us(lambda: kernels.int8_rows(x8), 20)
        us_mm = _time_us(lambda: kernels.int8_mm(xq, q8, xs, s8, torch.bfloat16), 10)
        tops = 2.0 * 2048 * 14336 * 4096 / us_mm / 1e6
        us_w8a16 = _time_us(lambda: torch.matmul(x8, kernels.dequantize8(q8, s8, False, 0, 1, torch.bfloat16).T), 10)
        out["w8a8_M2048_K4096_N14336"] = {"int8_rows_us": us_rows, "int8_mm_us": us_mm, "TOP/s": tops,
                                          "frac_of_2x_bf16_peak": tops / (2 * bf16_peak),
                                          "comparator_dequantize_plus_library_gemm_us": us_w8a16}
    del x8, q8, s8
    torch.cuda.empty_cache()
    # bulk quantize/pack, one Llama-3-70B-shaped tensor (gate/up: 28672 x 8192, bf16 N(0, 0.015))
    w = torch.empty(28672, 8192, device=device, dtype=torch.bfloat16).normal_(0, 0.015, generator=gen)
    n = w.numel()
    us = _time_us(lambda: quant.quantize_int4_groups(w, GROUP, scale_dtype="bf16"), 10)
    b4 = n * 2 + n // 2 + (n // GROUP) * (4 + 2 + 1)
    out["quantize_int4_g128_28672x8192"] = {"us": us, "GB/s": b4 / us / 1e3, "frac_hbm": b4 / us / 1e3 / hbm}
    us = _time_us(lambda: quant.quantize_int8_groups(w, 8192, "f32"), 10)
    b8 = n * 2 + n + 28672 * 4
    out["quantize_int8_channel_28672x8192"] = {"us": us, "GB/s": b8 / us / 1e3, "frac_hbm": b8 / us / 1e3 / hbm}
    return out


# ---- the bulk quantize workload (Llama-3-70B shapes, sharded by output rows) -------------------

LAYER_70B = (("q", 8192, 8192), ("k", 1024, 8192), ("v", 1024, 8192), ("o", 8192, 8192),
             ("gate", 28672, 8192), ("up", 28672, 8192), ("down", 8192, 28672))
LAYERS_70B = 80


def quantize_bytes(out: int, depth: int) -> tuple[int, int]:
    """Algorithmic bytes of one tensor: bf16 in; int4-g128 packed + bf16 scale + u8 zero out
    (2.5234 B per weight); int8 + one f32 scale a row out (3 + 4/In B per weight)."""
    n = out * depth
    return n * 2 + n // 2 + (n // GROUP) * 3, n * 2 + n + out * 4


def run_quantize(args, rank: int, world: int, device: torch.device, barrier, reduce_max) -> dict:
    import numpy as np

    from linnet_b200 import quant
    from oracle import quant_oracle as qo

    hbm, _tf, peak_kind = peaks()
    shard = [(name, out // world, depth) for name, out, depth in LAYER_70B]
    for (name, out, _d) in LAYER_70B:
        if out % world:
            raise SystemExit(f"{world} ranks do not divide the {out} rows of {name}")
    # two differently seeded copies of one layer's shard (the timed steps alternate between them);
    # a shard of a layer is >= 214 MB of bf16, larger than L2
    layers = []
    for copy in range(2):
        gen = torch.Generator(device=device).manual_seed(1000 * (copy + 1) + rank)
        layers.append([torch.empty(out, depth, device=device, dtype=torch.bfloat16).normal_(0, 0.015, generator=gen)
                       for _n, out, depth in shard])

    def step(index: int) -> None:
        for w in layers[index % 2]:
            quant.quantize_int4_groups(w, GROUP, scale_dtype="bf16")
            quant.quantize_int8_groups(w, w.shape[1], "bf16")

    # bit-exactness, outside the timed region: sampled rows of every distinct shape against the oracle
    checked = []
    for (name, out, depth), w in zip(shard, layers[0]):
        rows = torch.linspace(0, out - 1, 5).long().unique().to(device)
        sample = w[rows].contiguous()
        packed, scale, zero, stored = quant.quantize_int4_groups(w, GROUP, scale_dtype="bf16")
        q8, s8 = quant.quantize_int8_groups(w, depth, "bf16")
        want_p, want_s, want_z = qo.quantize_int4_groups(sample.float().cpu().numpy(), GROUP)
        want_q8, want_s8 = qo.quantize_int8_groups(sample.float().cpu().numpy(), depth, "bf16")
        ok = (np.array_equal(packed[rows].cpu().numpy(), want_p) and np.array_equal(zero[rows].cpu().numpy(), want_z)
              and np.array_equal(scale[rows].cpu().numpy().view(np.uint32), want_s.view(np.uint32))
              and np.array_equal(q8[rows].cpu().numpy(), want_q8)
              and np.array_equal(s8[rows].cpu().numpy().view(np.uint32), want_s8.view(np.uint32)))
        checked.append({"tensor": name, "shard_shape": [out, depth], "rows_checked": int(rows.numel()), "bit_exact": bool(ok)})
        del packed, scale, zero, stored, q8, s8
    torch.cuda.empty_cache()
    if not all(c["bit_exact"] for c in checked):
        raise SystemExit(f"quantizer differs from the oracle: {checked}")

    for i in range(max(3, args.warmup)):
        step(i)
    torch.cuda.synchronize()
    per_step = []
    with Clocks(device.index or 0) as clocks:
        for _ in range(TRIALS):
            barrier()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for i in range(args.steps):
                step(i)
            stop.record()
            torch.cuda.synchronize()
            barrier()
            per_step.append(reduce_max(start.elapsed_time(stop)) / args.steps)
    ms_step = statistics.median(per_step)
    b4 = sum(quantize_bytes(out, depth)[0] for _n, out, depth in shard)
    b8 = sum(quantize_bytes(out, depth)[1] for _n, out, depth in shard)
    per_gpu = (b4 + b8) / (ms_step / 1e3) / 1e9
    # each format alone, one trial each, for the roofline of either kernel
    def alone(fn) -> float:
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(4):
            for w in layers[i % 2]:
                fn(w)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / 4
    ms4 = alone(lambda w: quant.quantize_int4_groups(w, GROUP, scale_dtype="bf16"))
    ms8 = alone(lambda w: quant.quantize_int8_groups(w, w.shape[1], "bf16"))

    # End to end with HOST buffers: per step one layer's bf16 shard comes from pinned host memory,
    # is quantized to both formats, and everything a checkpoint stores (packed int4, bf16 scales,
    # zero points; int8 levels, their scales) goes back to pinned host memory.
    host_in = [w.to("cpu").pin_memory() for w in layers[0]]
    host_out = None
    e2e_steps = max(1, min(args.steps, 3))

    def e2e_step() -> None:
        nonlocal host_out
        outs = []
        for src in host_in:
            w = src.to(device, non_blocking=True)
            packed, _scale, zero, stored = quant.quantize_int4_groups(w, GROUP, scale_dtype="bf16")
            q8, s8 = quant.quantize_int8_groups(w, w.shape[1], "bf16")
            outs.append((packed, stored, zero, q8, s8))
        if host_out is None:
            host_out = [[torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in group] for group in outs]
        for group, dst in zip(outs, host_out):
            for t, d in zip(group, dst):
                d.copy_(t, non_blocking=True)
        torch.cuda.synchronize()

    e2e_step()
    e2e_trials = []
    for _ in range(3):
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_trials.append(reduce_max((time.perf_counter() - t0) * 1e3) / e2e_steps)
    e2e_ms = statistics.median(e2e_trials)
    h2d = sum(t.numel() * 2 for t in host_in)
    d2h = sum(d.numel() * d.element_size() for group in host_out for d in group)
    del host_in, host_out
    elements_layer = sum(out * depth for _n, out, depth in LAYER_70B)
    line = {
        "metric": "bulk quantize/pack GB/s (Llama-3-70B shapes, int4-g128 + int8 per-channel)",
        "value": per_gpu * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16 in, f32 arithmetic (IEEE, bit-exact with the reference), u4 / i8 out", "data": "synthetic",
        "config": {"workload": f"bulk quantize/pack, Llama-3-70B layer shapes ({elements_layer / 1e6:.1f} M weights a layer, "
                               f"{LAYERS_70B} layers), every tensor sharded by output rows over {world} GPU(s); a step = one "
                               f"layer's seven tensors to int4-g128 and to int8 per-channel",
                   "l2_policy": "inputs larger than L2: two layer shards alternate",
                   "timing": f"median of {TRIALS} trials of --steps steps, CUDA events, max over ranks"},
        "trials_ms_per_step": per_step,
        "whole_model_seconds_at_this_rate": ms_step * LAYERS_70B / 1e3,
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": hbm, "unit": "GB/s", "frac": per_gpu / hbm,
                     "peak_kind": peak_kind, "algorithmic_bytes_per_step_per_gpu": b4 + b8,
                     "int4_g128": {"GB/s": b4 / (ms4 / 1e3) / 1e9, "frac": b4 / (ms4 / 1e3) / 1e9 / hbm},
                     "int8_channel": {"GB/s": b8 / (ms8 / 1e3) / 1e9, "frac": b8 / (ms8 / 1e3) / 1e9 / hbm},
                     **quantize_traffic(sum(out * depth for _n, out, depth in shard))},
        "parity": checked,
        "e2e": {"value": (b4 + b8) / (e2e_ms / 1e3) / 1e9 * world, "unit": "GB/s", "ms_per_step": e2e_ms,
                "trials_ms_per_step": e2e_trials, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "how": f"{e2e_steps} step(s) a trial: the layer's shard from pinned host memory to the device, both "
                       "quantizers, all results back to pinned host memory, then a wait; the same algorithmic "
                       "bytes as `value` over that time (the host link, not HBM, bounds it)"},
        "gpu_launches": args.steps * TRIALS * 2 * len(shard),
        "clocks": clocks.summary(),
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        # NumPy on one thread, 1024 rows of each distinct width, extrapolated to the layer
        total4 = total8 = 0.0
        sample = []
        for depth in sorted({d for _n, _o, d in LAYER_70B}):
            ref = reference_run("quantize", "--out", "1024", "--depth", str(depth), "--reps", "2")
            if ref is None:
                break
            rows = sum(out for _n, out, d in LAYER_70B if d == depth)
            total4 += ref["int4_g128"]["seconds"] * rows / 1024
            total8 += ref["int8_channel"]["seconds"] * rows / 1024
            sample.append(ref["what"])
        if sample:
            line["cpu_baseline"] = {"value": (b4 + b8) * world / (total4 + total8) / 1e9, "unit": "GB/s", "cores": 1,
                                    "kind": "reference", "extrapolated": True,
                                    "sample": "; ".join(sample) + "; scaled to one layer's rows"}
    return line


# ---- the reference arm ---------------------------------------------------------------------


def run_reference(args, rank: int, world: int) -> dict | None:
    if rank != 0:
        return None
    t0 = time.perf_counter()
    base = cpu_baseline_gemv(args.rows, sets=WEIGHT_SETS, reps=max(1, min(args.steps, 20)), warm=max(1, min(args.warmup, 3)))
    return {
        "impl": "reference",
        "metric": METRIC,
        "value": base["value"], "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": gemv_bytes(args.rows) * LAUNCHES_PER_STEP / base["value"] / 1e6,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 weights dequantized from int4, bf16 activations (CPU)", "data": "synthetic",
        "config": {"workload": f"W4A16 g128 GEMV K={K_IN} N={N_OUT} M={args.rows}",
                   "note": "the reference's CPU torch route on the host cores; one step of the GPU arm "
                           "(64 launches) is sampled as 8 calls over 8 weight sets",
                   "wall_s": time.perf_counter() - t0},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default=None, choices=["gemv", "decode", "quantize"])
    parser.add_argument("--rows", type=int, default=1)
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-other-configs", action="store_true")
    parser.add_argument("--no-decode", action="store_true")
    parser.add_argument("--fold-swiglu", action="store_true",
                        help="decode: the down projection forms silu(gate) * up itself where it can (one launch fewer a layer)")
    parser.add_argument("--no-fold-norm", action="store_true",
                        help="decode: residual add + RMS norm as kernels of their own even where the products can form them")
    parser.add_argument("--early", action="store_true",
                        help="decode: the products let their dependents start as soon as they have started")
    parser.add_argument("--single-batch", action="store_true",
                        help="decode: time only --batch, not 1 / 8 / 64 as well (for profiling)")
    parser.add_argument("--peer-protocol", default=None, choices=["words", "flags"],
                        help="exchange of the peer reduction (default: words on 2 ranks, flags on more)")
    parser.add_argument("--reduce", default="peer", choices=["peer", "nccl"],
                        help="tensor-parallel decode: one peer-memory kernel per reduction, or NCCL")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist

        # NCCL's log (when NCCL_DEBUG is set) goes to a file beside the output, not to stdout,
        # which carries the one JSON line.
        if os.environ.get("NCCL_DEBUG") and not os.environ.get("NCCL_DEBUG_FILE"):
            os.environ["NCCL_DEBUG_FILE"] = str(Path(tempfile.gettempdir()) / "nccl.%h.%p.log")
        # plain peer stores only: no NVLS multicast binding of the symmetric memory
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=device)

        def barrier() -> None:
            dist.barrier()

        def reduce_max(v: float) -> float:
            t = torch.tensor([v], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
    else:
        def barrier() -> None:
            return None

        def reduce_max(v: float) -> float:
            return v

    from linnet_b200 import decoder

    if args.workload == "quantize":
        line = run_quantize(args, rank, world, device, barrier, reduce_max)
    elif args.workload == "decode":
        line = decoder.bench(args, rank, world, device, barrier, reduce_max, Clocks)
    else:
        # The headline line is the same at every N: the GEMV of BASELINE's configs[1], each
        # rank streaming its own weight sets (the product shards by output rows with no
        # exchange, so more GPUs are more independent rows: weak scaling).  The second half
        # of the metric, decoder tokens/s tensor-parallel over the N ranks, rides along
        # under "decode".
        line = run_gemv(args, rank, world, device, barrier, reduce_max)
        if not args.no_decode:
            torch.cuda.empty_cache()
            dargs = argparse.Namespace(**vars(args))
            dargs.steps = max(10, args.steps // 4)
            dec = decoder.bench(dargs, rank, world, device, barrier, reduce_max, Clocks)
            line["decode"] = {"metric": "8B-shape int4 decode tok/s", "tensor_parallel": world,
                              "tok_s": dec["value"], "ms_per_step": dec["ms_per_step"],
                              "per_batch": dec["per_batch"], "e2e": dec["e2e"], "steps": dargs.steps,
                              "roofline": dec["roofline"], "config": dec["config"],
                              "reduce_route": dec["reduce_route"],
                              **{k: dec[k] for k in ("per_batch_nccl_route", "peer_vs_nccl", "peer_reduce_unavailable")
                                 if k in dec}}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
