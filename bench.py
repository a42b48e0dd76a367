"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload gemv|decode|kernels] [--rows M] [--batch B]

Prints ONE JSON line.  Workloads:

* `gemv` (default) -- the W4A16 g128 decode product the headline metric is
  quoted on: K=4096, N=14336 (Llama-3-8B gate/up), x bf16 [M, K], M=1 for `value`
  (M=4 and 16 are reported under `per_rows`).  One step is 64 launches cycling through
  8 distinct weight sets (246 MB, larger than the 126 MB L2, so every launch streams its
  weights from HBM), recorded once into a CUDA graph and replayed.
  With N ranks every rank runs this on its own GPU and weight sets (`value` is the sum).
  The line also carries `decode`: tokens/s of a Llama-3.1-8B-shaped int4 decoder step,
  tensor-parallel over the N ranks (linnet_b200/decoder.py), at batch 1, 8 and 64.
* `--workload decode` -- only the decoder, tokens/s as `value`.
* `--workload kernels [--case attention|glue|linear] [--rows M] [--batch B]` -- every kernel
  of a decode step timed alone (linnet_b200/kernel_times.py); not a bench line, a table.

`--impl reference` times the reference's own CPU route for the same workload (its
torch path: weight dequantized once, then bf16 `F.linear`) on the host cores.
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
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

K_IN, N_OUT, GROUP = 4096, 14336, 128
WEIGHT_SETS = 8
LAUNCHES_PER_STEP = 64


def gemv_bytes(rows: int) -> int:
    """Algorithmic bytes of one launch: packed nibbles + bf16 scales + u8 zero points,
    plus the activations read and the outputs written."""
    groups = K_IN // GROUP
    return N_OUT * K_IN // 2 + N_OUT * groups * 3 + rows * K_IN * 2 + rows * N_OUT * 2


def peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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
            self.stop.wait(0.2)

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


# ---- synthetic weights -----------------------------------------------------------


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


def cpu_reference_gemv(rows: int, sets: int, reps: int, warm: int) -> dict:
    """The reference's CPU route (python/linnet/src/linnet/torch/native.py:417-424;
    src/backend/torch_source.cpp:1501-1504, :1568): W dequantized once to bf16 by
    `prepare`, then `F.linear(x, W)` per call, on every host core."""
    from oracle import linear_oracle as lo
    from oracle import quant_oracle as qo

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(0)
    weights = []
    for _ in range(sets):
        w = torch.randn(N_OUT, K_IN, generator=gen) * 0.02
        packed, scale, zero = qo.quantize_int4_groups(w.numpy(), GROUP)
        weights.append(lo.int4_weight(torch.from_numpy(packed),
                                      torch.from_numpy(scale).to(torch.bfloat16),
                                      torch.from_numpy(zero), torch.bfloat16))
    x = torch.randn(rows, K_IN, generator=gen).to(torch.bfloat16)
    times = []
    for i in range(warm + reps):
        t0 = time.perf_counter()
        for w in weights:
            torch.nn.functional.linear(x, w)
        dt = time.perf_counter() - t0
        if i >= warm:
            times.append(dt / len(weights))
    per_call = statistics.median(times)
    return {"value": gemv_bytes(rows) / per_call / 1e9, "unit": "GB/s", "cores": threads,
            "kind": "port",
            "sample": f"{sets} weight sets x {reps} passes of F.linear(x[{rows},{K_IN}] bf16, W bf16 "
                      f"[{N_OUT},{K_IN}]) after {warm} warm-up passes; median per call "
                      f"{per_call * 1e3:.3f} ms; bytes counted as the packed int4 layout's"}


# ---- the gemv workload -------------------------------------------------------------


def time_graph(graph: torch.cuda.CUDAGraph, steps: int, warmup: int, barrier) -> float:
    """Milliseconds for `steps` replays, device-timed on the current stream."""
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    barrier()
    return start.elapsed_time(stop)


def run_gemv(args, rank: int, world: int, device: torch.device, barrier, reduce_max) -> dict:
    from linnet_b200 import kernels

    sets = make_weight_sets(device, WEIGHT_SETS)
    gen = torch.Generator().manual_seed(1)
    stream = torch.cuda.Stream(device)
    results: dict[int, float] = {}
    clocks = None
    with torch.cuda.stream(stream):
        for rows in (args.rows, *[m for m in (1, 4, 16) if m != args.rows]):
            x = torch.randn(rows, K_IN, generator=gen).to(torch.bfloat16).to(device)
            for p, s, z in sets[:2]:
                kernels.int4_linear(x, p, s, z)  # warm: module load, attribute set-up
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(LAUNCHES_PER_STEP):
                    p, s, z = sets[i % WEIGHT_SETS]
                    kernels.int4_linear(x, p, s, z)
            if rows == args.rows:
                with Clocks(device.index or 0) as clocks:
                    ms = time_graph(graph, args.steps, args.warmup, barrier)
            else:
                ms = time_graph(graph, max(3, args.steps // 4), 3, barrier)
                ms *= args.steps / max(3, args.steps // 4)
            results[rows] = reduce_max(ms) / args.steps  # ms per step
        # End to end through the operator with host buffers: per step the activations
        # come from pinned host memory and the last result goes back to the host.
        rows = args.rows
        host_x = torch.randn(rows, K_IN, generator=gen).to(torch.bfloat16).pin_memory()
        host_y = torch.empty(rows, N_OUT, dtype=torch.bfloat16).pin_memory()
        dev_x = torch.empty(rows, K_IN, dtype=torch.bfloat16, device=device)

        def e2e_step() -> None:
            dev_x.copy_(host_x, non_blocking=True)
            y = None
            for i in range(LAUNCHES_PER_STEP):
                p, s, z = sets[i % WEIGHT_SETS]
                y = kernels.int4_linear(dev_x, p, s, z)
            host_y.copy_(y, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        e2e_ms = reduce_max((time.perf_counter() - t0) * 1e3) / args.steps
    peak, peak_kind = peaks()
    per_launch_s = results[args.rows] / 1e3 / LAUNCHES_PER_STEP
    achieved = gemv_bytes(args.rows) / per_launch_s / 1e9
    line = {
        "metric": "W4A16 g128 GEMV GB/s (% HBM peak); 8B-shape int4 decode tok/s at 1/2/4/8 GPU",
        "value": achieved * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": results[args.rows], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int4 weights, bf16 activations, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"W4A16 g128 GEMV K={K_IN} N={N_OUT} M={args.rows}",
                   "launches_per_step": LAUNCHES_PER_STEP, "weight_sets": WEIGHT_SETS,
                   "l2_policy": f"inputs larger than L2: {WEIGHT_SETS} weight sets, "
                                f"{WEIGHT_SETS * gemv_bytes(1) / 1e6:.0f} MB, visited round-robin",
                   "timing": "CUDA events around graph replays on the launching stream",
                   "replicas": world},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": peak_kind,
                     "frac_of_8tbs_nominal": achieved / 8000.0,
                     "algorithmic_bytes_per_launch": gemv_bytes(args.rows),
                     "us_per_launch": per_launch_s * 1e6,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch at M=1, from the
                     # ncu capture summarised in profiles/int4_gemv_oct_k4096_n14336_m1.md
                     "traffic": 30774016 if args.rows == 1 else None},
        "per_rows": {str(m): {"GB/s": gemv_bytes(m) / (results[m] / 1e3 / LAUNCHES_PER_STEP) / 1e9,
                              "us_per_launch": results[m] * 1e3 / LAUNCHES_PER_STEP}
                     for m in sorted(results)},
        "e2e": {"value": gemv_bytes(rows) * LAUNCHES_PER_STEP / (e2e_ms / 1e3) / 1e9 * world,
                "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": rows * K_IN * 2, "d2h_bytes_per_step": rows * N_OUT * 2},
        "gpu_launches": args.steps * LAUNCHES_PER_STEP,
        "clocks": clocks.summary() if clocks else None,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_reference_gemv(args.rows, sets=4, reps=5, warm=2)
    if rank == 0 and not args.no_other_configs:
        del sets
        torch.cuda.empty_cache()
        line["other_configs"] = other_configs(device)
    return line


def _time_us(fn, reps: int, warm: int = 3) -> float:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / reps


def other_configs(device: torch.device) -> dict:
    """Short measurements of the other workloads (not the headline): the int8
    per-channel GEMV, the prefill dequant-GEMM at M=2048 and the bulk quantize/pack
    kernels on one 70B-shaped tensor.  Inputs are larger than L2 or rotated."""
    from linnet_b200 import kernels, quant

    bf16_peak = 1683.2
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        bf16_peak = float(json.loads(path.read_text())["bf16_tflops"])
    hbm, _ = peaks()
    out: dict = {}
    gen = torch.Generator(device=device).manual_seed(3)
    # int8 symmetric per-output-channel GEMV, M=1, K=N=4096 (16 weight sets = 268 MB)
    sets8 = []
    for _ in range(16):
        w = torch.empty(4096, 4096, device=device).normal_(0, 0.02, generator=gen)
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
                kernels.gemv8(x1, *sets8[i % 16], False, 0, 1)
        us = _time_us(graph.replay, 10) / 64
    nbytes = 4096 * 4096 + 4096 * 4 + 4096 * 2 + 4096 * 2
    out["int8_gemv_M1_K4096_N4096"] = {"us": us, "GB/s": nbytes / us / 1e3, "frac_hbm": nbytes / us / 1e3 / hbm,
                                       "note": "64 launches over 16 weight sets in one CUDA graph"}
    del graph
    del sets8
    # prefill dequant-GEMM, M = 2048
    x = torch.randn(2048, 14336, device=device, generator=gen).to(torch.bfloat16)
    for K, N in ((4096, 6144), (4096, 28672), (14336, 4096)):
        w = torch.empty(N, K, device=device, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
        packed, _s, zero, scale = quant.quantize_int4_groups(w, GROUP, scale_dtype="bf16")
        del w
        xk = x[:, :K].contiguous()
        us = _time_us(lambda: kernels.int4_linear(xk, packed, scale, zero), 10)
        tf = 2.0 * 2048 * N * K / us / 1e6
        out[f"int4_gemm_M2048_K{K}_N{N}"] = {"us": us, "TFLOP/s": tf, "frac_bf16_peak": tf / bf16_peak}
    del x, packed, scale, zero
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


def run_reference(args, rank: int, world: int) -> dict | None:
    if rank != 0:
        return None
    t0 = time.perf_counter()
    base = cpu_reference_gemv(args.rows, sets=WEIGHT_SETS, reps=max(1, args.steps), warm=max(1, args.warmup))
    return {
        "impl": "reference",
        "metric": "W4A16 g128 GEMV GB/s (% HBM peak); 8B-shape int4 decode tok/s at 1/2/4/8 GPU",
        "value": base["value"], "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": gemv_bytes(args.rows) * LAUNCHES_PER_STEP / base["value"] / 1e6,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 weights dequantized from int4, bf16 activations (CPU)", "data": "synthetic",
        "config": {"workload": f"W4A16 g128 GEMV K={K_IN} N={N_OUT} M={args.rows}",
                   "note": "reference CPU torch route on the host cores; one step of the GPU arm "
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
    parser.add_argument("--workload", default=None, choices=["gemv", "decode", "kernels"])
    parser.add_argument("--case", default="all", choices=["all", "attention", "glue", "linear"],
                        help="kernels: which kernel family to time")
    parser.add_argument("--tp", type=int, default=1, choices=[1, 2, 4, 8],
                        help="kernels: time the shapes of one rank of a tensor-parallel group of this size")
    parser.add_argument("--rows", type=int, default=None)
    parser.add_argument("--batch", type=int, default=None)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-other-configs", action="store_true")
    parser.add_argument("--no-decode", action="store_true")
    parser.add_argument("--single-batch", action="store_true",
                        help="decode: time only --batch, not 1 / 8 / 64 as well (for profiling)")
    parser.add_argument("--peer-protocol", default=None, choices=["words", "flags"],
                        help="exchange of the peer reduction (default: words on 2 ranks, flags on more)")
    parser.add_argument("--reduce", default="peer", choices=["peer", "nccl"],
                        help="tensor-parallel decode: one peer-memory kernel per reduction, or NCCL")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    one_size = (args.rows, args.batch)  # kernels: None sweeps the sizes
    args.rows = args.rows if args.rows is not None else 1
    args.batch = args.batch if args.batch is not None else 1

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

        os.environ.pop("NCCL_DEBUG", None)  # its banner would share stdout with the JSON line
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

    if args.workload == "kernels":
        from linnet_b200 import kernel_times

        if world > 1:
            raise SystemExit("--workload kernels runs on one GPU")
        line = {"workload": "kernels", "case": args.case, "unit": "us per launch, CUDA graph over rotating inputs",
                "tp_shard": args.tp, "results": kernel_times.run(device, args.case, *one_size, tp=args.tp)}
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
                              **({"per_batch_nccl_route": dec["per_batch_nccl_route"]}
                                 if "per_batch_nccl_route" in dec else {})}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
