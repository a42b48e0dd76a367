"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE.

Run where the reference has been built into `oracle/_ref` (`python -m oracle.build_ref`); the
outputs are committed so that the tests do not depend on it:

    python tests/golden/make_golden.py

Everything stored here comes out of the reference's own code:
`linnet.quant.quantize_int4_groups / quantize_int8_groups / pack_int4_groups`,
`linnet.weights.to_bf16_bits`, `linnet.torch.native.NATIVE[...]` (interpreter
implementations), `linnet.torch.quantized.int8_linear / int8_group_linear` (CPU
branch), `linnet.torch.load(...)` of small `Int4GroupLinear` / `Int8Linear`
cards, interpreted and as generated source, and `linnet.quant.quantize_checkpoint /
import_quantized` on small SafeTensors files.  Inputs are stored next to the
outputs so the tests never depend on a random generator's implementation.
"""

from __future__ import annotations

import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import build_ref  # noqa: E402

if not build_ref.available():
    raise SystemExit("oracle/_ref is missing: run `python -m oracle.build_ref` first")
REF_HOME = Path(tempfile.mkdtemp(prefix="linnet-home-"))
for key, value in build_ref.environment(REF_HOME).items():
    if key.startswith("LINNET_"):
        os.environ[key] = value
sys.path.insert(0, str(build_ref.OUT / "python"))
STD = str(build_ref.OUT / "stdlib")

from linnet import quant as refq  # noqa: E402
from linnet.weights import to_bf16_bits  # noqa: E402

HERE = Path(__file__).resolve().parent


def bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(a).to(torch.bfloat16).float().numpy()


def quantizer_cases() -> dict[str, np.ndarray]:
    """Inputs covering the reference's own quantizer tests plus edge cases."""
    rng = np.random.default_rng(0)
    cases: dict[str, tuple[np.ndarray, int]] = {}
    # tests/test_quant_groups.py:48-56 (OUT=64, IN=256, GROUP=128, default_rng(0)).
    cases["ref_test_64x256_g128"] = (rng.standard_normal((64, 256)).astype(np.float32), 128)
    cases["g32_72x512"] = ((rng.standard_normal((72, 512)) * 0.02).astype(np.float32), 32)
    cases["g16_16x128"] = ((rng.standard_normal((16, 128)) * 3.0).astype(np.float32), 16)
    cases["g64_24x256"] = ((rng.standard_normal((24, 256)) * 0.5).astype(np.float32), 64)
    cases["g256_8x1024"] = ((rng.standard_normal((8, 1024)) * 0.02).astype(np.float32), 256)
    # bf16-valued weights of the bulk-quantize workload, N(0, 0.015).
    cases["bf16_96x1024_g128"] = (
        bf16_round((rng.standard_normal((96, 1024)) * 0.015).astype(np.float32)), 128)
    # Edge cases: constant groups (scale falls back to 1), zeros, one-sided
    # ranges, huge and tiny magnitudes, exact ties.
    edge = np.zeros((8, 256), dtype=np.float32)
    edge[1, :] = 0.37
    edge[2, :128] = np.linspace(-1.0, 0.0, 128, dtype=np.float32)
    edge[2, 128:] = np.linspace(0.0, 2.0, 128, dtype=np.float32)
    edge[3, :] = (np.arange(256) % 16).astype(np.float32) * 0.5  # ties at .5 steps
    edge[4, :] = rng.standard_normal(256).astype(np.float32) * 1e-30
    edge[5, :] = rng.standard_normal(256).astype(np.float32) * 1e30
    edge[6, :] = -np.abs(rng.standard_normal(256).astype(np.float32))
    edge[7, :] = np.abs(rng.standard_normal(256).astype(np.float32)) + 5.0
    cases["edges_8x256_g128"] = (edge, 128)
    out: dict[str, np.ndarray] = {}
    for name, (w, group) in cases.items():
        packed, scale, zero = refq.quantize_int4_groups(w, group)
        out[f"q4/{name}/w"] = w
        out[f"q4/{name}/group"] = np.array(group)
        out[f"q4/{name}/packed"] = packed
        out[f"q4/{name}/scale"] = scale
        out[f"q4/{name}/scale_bf16_bits"] = to_bf16_bits(scale).reshape(scale.shape)
        out[f"q4/{name}/zero"] = zero
        # f16 storage of 1e30 / 1e-30 scales overflows or flushes to zero and the
        # reference then casts NaN to int8 (undefined), so the edge case skips it.
        for dtype in ("f32", "bf16") if name.startswith("edges") else ("f32", "bf16", "f16"):
            g8 = group if group >= 16 else 16
            q, s = refq.quantize_int8_groups(w, g8, dtype)
            out[f"q8/{name}/{dtype}/q"] = q
            out[f"q8/{name}/{dtype}/scale"] = s
            out[f"q8/{name}/{dtype}/group"] = np.array(g8)
        # per-output-channel: one group spanning the whole row
        q, s = refq.quantize_int8_groups(w, w.shape[1], "f32")
        out[f"q8/{name}/channel/q"] = q
        out[f"q8/{name}/channel/scale"] = s
        out[f"q8/{name}/channel/group"] = np.array(w.shape[1])
    return out


INT4_CARD = """\
module tests.q4

use std.quant::{Int4GroupLinear}

pub block Model<In: Dim, Out: Dim, Group: Dim, T: Float = f32>
where
    Group > 0,
    Group % 2 == 0,
    In % Group == 0
{
    sub proj: Int4GroupLinear<In, Out, Group, T>

    pub entry forward<B: Dim>(x: Tensor[B, In; T]) -> Tensor[B, Out; T] {
        return proj.forward(x)
    }
}
"""

INT8_CARD = """\
module tests.q8

use std.quant::{Int8Linear, Int8GroupLinear}

pub block Model<In: Dim, Out: Dim, T: Float = f32>
where In % 128 == 0 {
    sub rows: Int8Linear<In, Out, T>
    sub groups: Int8GroupLinear<In, Out, 128, T>

    pub entry by_rows<B: Dim>(x: Tensor[B, In; T]) -> Tensor[B, Out; T] {
        return rows.forward(x)
    }

    pub entry by_groups<B: Dim>(x: Tensor[B, In; T]) -> Tensor[B, Out; T] {
        return groups.forward(x)
    }
}
"""


def linear_cases() -> dict[str, np.ndarray]:
    """Layer outputs from the reference's torch path on the CPU."""
    from safetensors.torch import save_file

    from linnet.torch import load
    from linnet.torch import native, quantized

    std = STD
    out: dict[str, np.ndarray] = {}
    gen = torch.Generator().manual_seed(0)
    IN, OUT, GROUP = 256, 64, 128
    w = torch.randn(OUT, IN, generator=gen) * 0.02
    packed, scale, zero = refq.quantize_int4_groups(w.numpy(), GROUP)
    scale_bf16 = torch.from_numpy(scale).to(torch.bfloat16)
    tp, tz = torch.from_numpy(packed), torch.from_numpy(zero)
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        (tmp / "q4.linnet").write_text(INT4_CARD, encoding="utf-8")
        save_file({"proj.weight": tp, "proj.scale": scale_bf16, "proj.zero": tz},
                  str(tmp / "q4.safetensors"))
        for rows in (1, 3, 16, 40):
            x = torch.randn(rows, IN, generator=gen).to(torch.bfloat16)
            interp = native.NATIVE["torch.ops.aten._weight_int4pack_mm"](
                (x, tp, scale_bf16, tz, None))
            results = {}
            for mode in (False, True):
                model = load(tmp / "q4.linnet",
                             generics={"In": IN, "Out": OUT, "Group": GROUP, "T": "bf16"},
                             std_root=std, weights=tmp / "q4.safetensors", compile=mode)
                results[mode] = model.run_entry("forward", [x]).detach()
            assert torch.equal(results[False], results[True]), "interpreter != generated"
            assert torch.equal(results[False], interp), "card != NATIVE entry"
            out[f"lin4/rows{rows}/x_bits"] = x.view(torch.int16).numpy()
            out[f"lin4/rows{rows}/y_bits"] = interp.view(torch.int16).numpy()
        out["lin4/packed"] = packed
        out["lin4/scale_bits"] = scale_bf16.view(torch.int16).numpy()
        out["lin4/zero"] = zero

        # int8: per-row and per-group scales
        w8 = torch.randn(OUT, IN, generator=gen) * 0.02
        q_rows, s_rows = refq.quantize_int8_groups(w8.numpy(), IN, "bf16")
        q_grp, s_grp = refq.quantize_int8_groups(w8.numpy(), 128, "bf16")
        (tmp / "q8.linnet").write_text(INT8_CARD, encoding="utf-8")
        save_file({
            "rows.weight": torch.from_numpy(q_rows),
            "rows.scale": torch.from_numpy(s_rows).to(torch.bfloat16),
            "groups.weight": torch.from_numpy(q_grp),
            "groups.scale": torch.from_numpy(s_grp).to(torch.bfloat16),
        }, str(tmp / "q8.safetensors"))
        model = load(tmp / "q8.linnet", generics={"In": IN, "Out": OUT, "T": "bf16"},
                     std_root=std, weights=tmp / "q8.safetensors", compile=True)
        for rows in (1, 5, 16):
            x = torch.randn(rows, IN, generator=gen).to(torch.bfloat16)
            ops = quantized.int8_operands(torch.from_numpy(q_rows),
                                          torch.from_numpy(s_rows).reshape(-1), 0)
            y_rows = quantized.int8_linear(x, ops, None)
            gops = quantized.int8_group_operands(torch.from_numpy(q_grp),
                                                 torch.from_numpy(s_grp))
            y_grp = quantized.int8_group_linear(x, gops, None)
            assert torch.equal(model.run_entry("by_rows", [x]).detach(), y_rows)
            assert torch.equal(model.run_entry("by_groups", [x]).detach(), y_grp)
            out[f"lin8/rows{rows}/x_bits"] = x.view(torch.int16).numpy()
            out[f"lin8/rows{rows}/y_rows_bits"] = y_rows.view(torch.int16).numpy()
            out[f"lin8/rows{rows}/y_groups_bits"] = y_grp.view(torch.int16).numpy()
        out["lin8/q_rows"] = q_rows
        out["lin8/s_rows"] = s_rows
        out["lin8/q_groups"] = q_grp
        out["lin8/s_groups"] = s_grp
    return out


def checkpoint_cases() -> None:
    """`linnet.quant.quantize_checkpoint` / `import_quantized` on the small checkpoints of
    tests/checkpoint_cases.py: inputs and the reference's output files, verbatim."""
    import json
    import shutil

    sys.path.insert(0, str(ROOT / "tests"))
    import checkpoint_cases as cc

    target = HERE / "checkpoints"
    if target.exists():
        shutil.rmtree(target)
    target.mkdir()
    cases = cc.all_cases(target)
    for name, case in cases.items():
        paths = cc.convert(refq, case, target, target / f"{name}.expected.safetensors")
        case["quantized"] = paths
    (target / "cases.json").write_text(json.dumps(cases, indent=1) + "\n", encoding="utf-8")


def main() -> None:
    np.savez_compressed(HERE / "quantizer.npz", **quantizer_cases())
    np.savez_compressed(HERE / "linear.npz", **linear_cases())
    checkpoint_cases()
    for path in sorted(HERE.rglob("*")):
        if path.is_file() and path.suffix in (".npz", ".safetensors", ".json"):
            print(path.relative_to(HERE), path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
