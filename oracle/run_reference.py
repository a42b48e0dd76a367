"""Times the reference's own CPU implementation of the hot path (test and bench
infrastructure; never imported by the product).  Runs inside a process that sees `oracle/_ref`
(`oracle.build_ref.environment`) and prints one JSON object:

    python oracle/run_reference.py gemv --rows 1 --sets 4 --reps 5 --warm 2
        `Int4GroupLinear` K=4096 N=14336 g128 bf16 loaded by `linnet.torch.load(compile=True)`
        on the CPU (its `prepare` dequantizes the weight once, every call is a bf16 `F.linear`:
        src/backend/torch_source.cpp:1501-1504, :1568), `sets` different weights visited in turn.
    python oracle/run_reference.py int8 --rows 1 --reps 5
        `Int8Linear` 4096x4096 the same way (python/linnet/src/linnet/torch/quantized.py:193).
    python oracle/run_reference.py quantize --out 1024 --depth 8192 --reps 3
        `linnet.quant.quantize_int4_groups` and `quantize_int8_groups` (NumPy) on one tensor.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import tempfile
import time
from pathlib import Path

import numpy as np
import torch

LIN4 = """module bench.lin4
use std.quant::{Int4GroupLinear}
pub block Model<In: Dim, Out: Dim, Group: Dim, T: Float = bf16>
where Group > 0, Group % 2 == 0, In % Group == 0
{
    sub proj: Int4GroupLinear<In, Out, Group, T>
    pub entry forward<B: Dim>(x: Tensor[B, In; T]) -> Tensor[B, Out; T] {
        return proj.forward(x)
    }
}
"""

LIN8 = """module bench.lin8
use std.quant::{Int8Linear}
pub block Model<In: Dim, Out: Dim, T: Float = bf16>
{
    sub proj: Int8Linear<In, Out, T>
    pub entry forward<B: Dim>(x: Tensor[B, In; T]) -> Tensor[B, Out; T] {
        return proj.forward(x)
    }
}
"""


def _time_calls(models, x, reps: int, warm: int) -> float:
    times = []
    for i in range(warm + reps):
        t0 = time.perf_counter()
        for model in models:
            model.run_entry("forward", [x])
        dt = time.perf_counter() - t0
        if i >= warm:
            times.append(dt / len(models))
    return statistics.median(times)


def gemv(args) -> dict:
    import linnet.torch as lt
    from linnet import quant
    from safetensors.torch import save_file

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    work = Path(tempfile.mkdtemp(prefix="ref-gemv-"))
    (work / "lin4.linnet").write_text(LIN4, encoding="utf-8")
    gen = torch.Generator().manual_seed(0)
    models = []
    for index in range(args.sets):
        w = (torch.randn(args.out, args.depth, generator=gen) * 0.02).numpy()
        packed, scale, zero = quant.quantize_int4_groups(w, 128)
        save_file({"proj.weight": torch.from_numpy(packed), "proj.scale": torch.from_numpy(scale).to(torch.bfloat16),
                   "proj.zero": torch.from_numpy(zero)}, str(work / f"w{index}.safetensors"))
        models.append(lt.load(work / "lin4.linnet", generics={"In": args.depth, "Out": args.out, "Group": 128, "T": "bf16"},
                              std_root=os.environ["LINNET_STD"], weights=work / f"w{index}.safetensors", compile=True))
    x = torch.randn(args.rows, args.depth, generator=gen).to(torch.bfloat16)
    per_call = _time_calls(models, x, args.reps, args.warm)
    groups = args.depth // 128
    nbytes = args.out * args.depth // 2 + args.out * groups * 3 + args.rows * args.depth * 2 + args.rows * args.out * 2
    return {"seconds_per_call": per_call, "bytes_per_call": nbytes, "GB/s": nbytes / per_call / 1e9, "cores": threads,
            "what": f"linnet.torch.load(Int4GroupLinear {args.depth}->{args.out} g128 bf16, compile=True) on the CPU, "
                    f"run_entry over {args.sets} weight sets x {args.reps} passes after {args.warm} warm-up passes; "
                    f"bytes counted as the packed int4 layout's"}


def int8(args) -> dict:
    import linnet.torch as lt
    from linnet import quant
    from safetensors.torch import save_file

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    work = Path(tempfile.mkdtemp(prefix="ref-int8-"))
    (work / "lin8.linnet").write_text(LIN8, encoding="utf-8")
    torch.manual_seed(0)
    w = (torch.randn(args.out, args.depth) * 0.02).numpy()
    q, scale = quant.quantize_int8_groups(w, args.depth, "bf16")
    save_file({"proj.weight": torch.from_numpy(q), "proj.scale": torch.from_numpy(scale).to(torch.bfloat16)},
              str(work / "w.safetensors"))
    model = lt.load(work / "lin8.linnet", generics={"In": args.depth, "Out": args.out, "T": "bf16"},
                    std_root=os.environ["LINNET_STD"], weights=work / "w.safetensors", compile=True)
    x = torch.randn(args.rows, args.depth).to(torch.bfloat16)
    per_call = _time_calls([model], x, args.reps, args.warm)
    nbytes = args.out * args.depth + args.out * 4 + args.rows * args.depth * 2 + args.rows * args.out * 2
    return {"seconds_per_call": per_call, "bytes_per_call": nbytes, "GB/s": nbytes / per_call / 1e9, "cores": threads,
            "what": f"linnet.torch.load(Int8Linear {args.depth}->{args.out} bf16, compile=True) on the CPU, "
                    f"{args.reps} calls after {args.warm}"}


def quantize(args) -> dict:
    from linnet import quant

    rng = np.random.default_rng(0)
    w = (rng.standard_normal((args.out, args.depth)) * 0.015).astype(np.float32)
    w = torch.from_numpy(w).to(torch.bfloat16).float().numpy()  # bf16-valued, as the checkpoint holds them
    result = {"cores": 1, "elements": int(w.size)}
    for name, call in (("int4_g128", lambda: quant.quantize_int4_groups(w, 128)),
                       ("int8_channel", lambda: quant.quantize_int8_groups(w, args.depth, "bf16"))):
        times = []
        for _ in range(args.reps):
            t0 = time.perf_counter()
            call()
            times.append(time.perf_counter() - t0)
        result[name] = {"seconds": statistics.median(times)}
    result["what"] = f"linnet.quant.quantize_int4_groups / quantize_int8_groups (NumPy, one thread) on {args.out} x {args.depth}"
    return result


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("what", choices=["gemv", "int8", "quantize"])
    parser.add_argument("--rows", type=int, default=1)
    parser.add_argument("--out", type=int, default=None)
    parser.add_argument("--depth", type=int, default=None)
    parser.add_argument("--sets", type=int, default=4)
    parser.add_argument("--reps", type=int, default=5)
    parser.add_argument("--warm", type=int, default=2)
    args = parser.parse_args()
    defaults = {"gemv": (14336, 4096), "int8": (4096, 4096), "quantize": (1024, 8192)}[args.what]
    args.out = args.out or defaults[0]
    args.depth = args.depth or defaults[1]
    print(json.dumps({"gemv": gemv, "int8": int8, "quantize": quantize}[args.what](args)))


if __name__ == "__main__":
    main()
