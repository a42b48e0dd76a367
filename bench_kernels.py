"""Per-kernel timings of the decode step (`python bench_kernels.py --case ...`): each kernel alone,
recorded into a CUDA graph over rotating inputs larger than L2 (so every launch streams
from HBM, as inside a decode step where each layer has its own weights and cache) and
replayed back to back with programmatic dependent launch, as the decoder runs them.

Also the small, self-contained cases used for `ncu` captures: a few GB on the device at
most, one kernel family per case.
"""

from __future__ import annotations

import argparse
import json

import torch

from linnet_b200 import glue, kernels, quant

SHAPES = {"qkv": (4096, 6144), "o": (4096, 4096), "gate_up": (4096, 28672), "down": (14336, 4096),
          "up": (4096, 14336)}  # "up" is the headline shape of bench.py


def _timed(fn, sets: int, reps: int = 3) -> float:
    """Mean microseconds of one call of fn(i), i over `sets` rotating inputs."""
    for i in range(min(2, sets)):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for i in range(sets):
                fn(i)
        graph.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(reps):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / (reps * sets)


def attention(device: torch.device, batches=(1, 8, 64), max_seq: int = 2048, tp: int = 1) -> dict:
    nq, nkv, hd = 32 // tp, 8 // tp, 128
    out = {}
    for batch in batches:
        nbytes = batch * nkv * max_seq * hd * 4
        sets = max(2, min(32, int(400e6 / nbytes)))
        ck = [torch.randn(batch, nkv, max_seq, hd, device=device, dtype=torch.bfloat16) for _ in range(sets)]
        cv = [torch.randn(batch, nkv, max_seq, hd, device=device, dtype=torch.bfloat16) for _ in range(sets)]
        q = torch.randn(batch, nq, hd, device=device, dtype=torch.bfloat16)
        pos = torch.full((batch,), max_seq - 1, device=device, dtype=torch.long)
        us = _timed(lambda i: glue.decode_attention(q, ck[i], cv[i], pos), sets)
        out[f"attention_batch{batch}_seq{max_seq}"] = {
            "us": us, "GB/s": nbytes / us / 1e3, "splits": min(8, glue.attention_splits(batch, nkv, max_seq))}
        del ck, cv
    return out


def glue_kernels(device: torch.device, batches=(1, 8, 64)) -> dict:
    out = {}
    for batch in batches:
        x = torch.randn(batch, 4096, device=device, dtype=torch.bfloat16)
        delta = torch.randn_like(x)
        w = torch.ones(4096, device=device, dtype=torch.bfloat16)
        out[f"add_rmsnorm_batch{batch}"] = {"us": _timed(lambda i: glue.add_rmsnorm(x, delta, w, 1e-5), 64)}
        gate_up = torch.randn(batch, 28672, device=device, dtype=torch.bfloat16)
        out[f"silu_mul_batch{batch}"] = {"us": _timed(lambda i: glue.silu_mul(gate_up), 64)}
        qkv = torch.randn(batch, 6144, device=device, dtype=torch.bfloat16)
        ck = torch.zeros(batch, 8, 2048, 128, device=device, dtype=torch.bfloat16)
        cv = torch.zeros_like(ck)
        pos = torch.full((batch,), 2047, device=device, dtype=torch.long)
        out[f"rope_cache_batch{batch}"] = {
            "us": _timed(lambda i: glue.rope_cache(qkv, pos, ck, cv, 32, 8, 500000.0), 64)}
    return out


def linear(device: torch.device, rows=(1, 8, 16, 32, 64, 128), shapes=None, tp: int = 1) -> dict:
    gen = torch.Generator(device=device).manual_seed(0)
    out = {}
    for name in shapes or SHAPES:
        depth, width = SHAPES[name]
        if name in ("o", "down"):   # row split: a shard holds K / tp inputs
            depth //= tp
        else:                        # column split: a shard holds N / tp outputs
            width //= tp
        sets = max(2, min(64, int(300e6 / (depth * width * 0.53))))
        weights = []
        for _ in range(sets):
            packed = torch.randint(0, 256, (width, depth // 128, 64), device=device, dtype=torch.uint8, generator=gen)
            scale = (torch.rand(width, depth // 128, device=device, generator=gen) * 0.02 + 0.001).to(torch.bfloat16)
            zero = torch.randint(0, 16, (width, depth // 128), device=device, dtype=torch.uint8, generator=gen)
            weights.append((packed, scale, zero))
        nbytes = depth * width * (0.5 + 3 / 128)
        for m in rows:
            x = torch.randn(m, depth, device=device, dtype=torch.bfloat16)
            us = _timed(lambda i: kernels.int4_linear(x, *weights[i]), sets)
            out[f"int4_linear_{name}_K{depth}_N{width}_M{m}"] = {"us": us, "GB/s": nbytes / us / 1e3}
        del weights
    return out


def run(device: torch.device, case: str, rows: int | None, batch: int | None, tp: int = 1,
        shapes=None) -> dict:
    """`case`: attention | glue | linear | all.  `rows` / `batch` narrow the sweep to one size;
    `tp` times the shapes one rank of a tensor-parallel group of that size holds."""
    results: dict = {}
    if case in ("attention", "all"):
        results.update(attention(device, (batch,) if batch else (1, 8, 64), tp=tp))
    if case in ("glue", "all"):
        results.update(glue_kernels(device, (batch,) if batch else (1, 8, 64)))
    if case in ("linear", "all"):
        results.update(linear(device, (rows,) if rows else (1, 8, 16, 32, 64, 128), shapes=shapes, tp=tp))
    return results


def quantize(device: torch.device, out: int = 8192, depth: int = 8192) -> dict:
    """The group quantizers on one bf16 tensor larger than L2 (a few weight sets in turn)."""
    sets = 4
    ws = [torch.randn(out, depth, device=device, dtype=torch.bfloat16) * 0.015 for _ in range(sets)]
    results = {}
    us = _timed(lambda i: quant.quantize_int4_groups(ws[i], 128, scale_dtype="bf16"), sets)
    nbytes = out * depth * (2 + 0.5 + 3 / 128)
    results[f"quantize_int4_g128_{out}x{depth}"] = {"us": us, "GB/s": nbytes / us / 1e3}
    us = _timed(lambda i: quant.quantize_int8_groups(ws[i], depth, "bf16"), sets)
    nbytes = out * depth * 3 + out * 2
    results[f"quantize_int8_channel_{out}x{depth}"] = {"us": us, "GB/s": nbytes / us / 1e3}
    return results


def int8(device: torch.device, rows=(1, 4, 16), shapes=((4096, 4096), (4096, 14336))) -> dict:
    """`int8_linear` (per-channel scales) at decode row counts over weight sets larger than L2."""
    gen = torch.Generator(device=device).manual_seed(0)
    results = {}
    for depth, width in shapes:
        sets = max(2, min(64, int(300e6 / (depth * width))))
        ws = [(torch.randint(-127, 128, (width, depth), device=device, dtype=torch.int8, generator=gen),
               torch.rand(width, device=device, generator=gen) * 0.01 + 0.001) for _ in range(sets)]
        for m in rows:
            x = torch.randn(m, depth, device=device, dtype=torch.bfloat16)
            fn = kernels.gemv8 if m == 1 else kernels.w8a16
            us = _timed(lambda i: fn(x, ws[i][0], ws[i][1], False, 0, 1), sets)
            nbytes = depth * width + width * 4 + m * (depth + width) * 2
            results[f"int8_linear_K{depth}_N{width}_M{m}"] = {"us": us, "GB/s": nbytes / us / 1e3}
    return results


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--case", default="all", choices=["attention", "glue", "linear", "quantize", "int8", "all"])
    parser.add_argument("--rows", type=int, default=None)
    parser.add_argument("--batch", type=int, default=None)
    parser.add_argument("--tp", type=int, default=1)
    parser.add_argument("--shape", default=None, choices=sorted(SHAPES), help="one linear shape instead of all")
    parser.add_argument("--numerics", default="fast", choices=["fast", "exact"])
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_kernels.py needs a CUDA device")
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    kernels.set_int4_numerics(args.numerics)
    results = run(device, args.case, args.rows, args.batch, args.tp, [args.shape] if args.shape else None)
    if args.case in ("quantize", "all"):
        results.update(quantize(device))
    if args.case in ("int8", "all"):
        results.update(int8(device, (args.rows,) if args.rows else (1, 4, 16)))
    print(json.dumps(results, indent=1))


if __name__ == "__main__":
    main()
