"""Small SafeTensors checkpoints for the quantize / import tests: a float checkpoint, and
GPTQ and AWQ 4-bit checkpoints built from the public definitions of those formats (the same
construction the reference's tests use, python/linnet/tests/test_quant_groups.py:206-221).

GPTQ: `qweight` int32 [In/8, Out], eight consecutive INPUTS per word, lowest bits first;
`qzeros` int32 [Groups, Out/8], eight consecutive outputs per word, each zero point stored
less one (first checkpoint format); `scales` f16 [Groups, Out]; `g_idx` int32 [In], the group
of every input (any order under activation ordering).
AWQ (GEMM): `qweight` int32 [In, Out/8] and `qzeros` int32 [Groups, Out/8], eight outputs per
word with bits 4k holding output (0, 2, 4, 6, 1, 3, 5, 7)[k] of the eight; `scales` f16.
"""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch
from safetensors.torch import save_file

AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def float_checkpoint(path: Path, seed: int = 0, out: int = 64, depth: int = 256) -> None:
    gen = torch.Generator().manual_seed(seed)
    save_file({
        "model.proj.weight": (torch.randn(out, depth, generator=gen) * 0.02).to(torch.bfloat16),
        "model.other.weight": torch.randn(out // 2, depth, generator=gen) * 0.5,
        "model.half.weight": (torch.randn(16, depth, generator=gen) * 0.1).to(torch.float16),
        "model.norm.weight": torch.ones(depth, dtype=torch.bfloat16),
        "model.proj.bias": torch.randn(out, generator=gen).to(torch.bfloat16),
    }, str(path))


FLOAT_BINDINGS = {"proj.weight": "model.proj.weight", "tied.weight": "model.proj.weight",
                  "other.weight": "model.other.weight", "half.weight": "model.half.weight",
                  "norm.weight": "model.norm.weight", "proj.bias": "model.proj.bias"}


def _pack_words(values: np.ndarray, axis: int, order=tuple(range(8))) -> np.ndarray:
    """Eight 4-bit values along `axis` per int32: bits 4k hold element order[k] of each eight."""
    moved = np.moveaxis(values.astype(np.uint32), axis, -1)
    eights = moved.reshape(*moved.shape[:-1], -1, 8)
    word = np.zeros(eights.shape[:-1], dtype=np.uint32)
    for k in range(8):
        word |= eights[..., order[k]] << np.uint32(4 * k)
    return np.ascontiguousarray(np.moveaxis(word.view(np.int32), -1, axis))


def gptq_checkpoint(path: Path, seed: int, out: int, depth: int, group: int, act_order: bool) -> dict:
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 16, size=(depth, out))            # [In, Out] levels, rows in STORAGE order
    zero = rng.integers(1, 17, size=(depth // group, out))  # true zero points 1..16, stored less one
    scales = (rng.random((depth // group, out)) * 0.02 + 0.001).astype(np.float16)
    g_idx = np.arange(depth) // group
    if act_order:
        g_idx = g_idx[rng.permutation(depth)]
    tensors = {
        "layer.qweight": torch.from_numpy(_pack_words(q, 0)),
        "layer.qzeros": torch.from_numpy(_pack_words(zero - 1, 1)),
        "layer.scales": torch.from_numpy(scales),
        "layer.g_idx": torch.from_numpy(g_idx.astype(np.int32)),
        "layer.bias": torch.from_numpy(rng.standard_normal(out).astype(np.float32)),
        "embed.weight": torch.from_numpy(rng.standard_normal((8, depth)).astype(np.float32)),
    }
    save_file(tensors, str(path))
    return {"quant_method": "gptq", "bits": 4, "group_size": group}


def awq_checkpoint(path: Path, seed: int, out: int, depth: int, group: int) -> dict:
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 16, size=(depth, out))
    zero = rng.integers(0, 16, size=(depth // group, out))
    scales = (rng.random((depth // group, out)) * 0.02 + 0.001).astype(np.float16)
    tensors = {
        "layer.qweight": torch.from_numpy(_pack_words(q, 1, AWQ_ORDER)),
        "layer.qzeros": torch.from_numpy(_pack_words(zero, 1, AWQ_ORDER)),
        "layer.scales": torch.from_numpy(scales),
        "embed.weight": torch.from_numpy(rng.standard_normal((8, depth)).astype(np.float32)),
    }
    save_file(tensors, str(path))
    return {"quant_method": "awq", "w_bit": 4, "q_group_size": group, "version": "gemm"}


def all_cases(directory: Path) -> dict[str, dict]:
    """Writes every input checkpoint into `directory`; returns name -> how to convert it."""
    float_checkpoint(directory / "float.safetensors")
    cases = {
        "int4_bf16": {"kind": "quantize", "input": "float.safetensors", "bits": 4, "dtype": "bf16", "group": 128,
                      "patterns": ["proj.weight", "tied.weight", "half.*"]},
        "int4_f32_g64": {"kind": "quantize", "input": "float.safetensors", "bits": 4, "dtype": "f32", "group": 64,
                         "patterns": ["proj.*", "o*.weight", "half.weight"]},
        "int8_bf16": {"kind": "quantize", "input": "float.safetensors", "bits": 8, "dtype": "bf16", "group": 128,
                      "patterns": ["proj.weight", "other.weight"]},
        "int8_f16_channel": {"kind": "quantize", "input": "float.safetensors", "bits": 8, "dtype": "f16", "group": 256,
                             "patterns": ["other.weight"]},
    }
    cases["gptq"] = {"kind": "import", "input": "gptq.safetensors", "dtype": "bf16",
                     "config": gptq_checkpoint(directory / "gptq.safetensors", 1, 48, 256, 128, False)}
    cases["gptq_act_order"] = {"kind": "import", "input": "gptq_act.safetensors", "dtype": "f16",
                               "config": gptq_checkpoint(directory / "gptq_act.safetensors", 2, 40, 256, 64, True)}
    cases["awq"] = {"kind": "import", "input": "awq.safetensors", "dtype": "bf16",
                    "config": awq_checkpoint(directory / "awq.safetensors", 3, 64, 256, 128)}
    return cases


def convert(module, case: dict, directory: Path, output: Path, **extra) -> list[str]:
    """Runs `module.quantize_checkpoint` / `module.import_quantized` (the reference's
    `linnet.quant` or this package's `linnet_b200.checkpoint`) on a case."""
    source = directory / case["input"]
    if case["kind"] == "import":
        return module.import_quantized(source, output, dtype=case["dtype"], config=case["config"], **extra)
    return module.quantize_checkpoint(source, output, patterns=list(case["patterns"]), group=case["group"],
                                      dtype=case["dtype"], bindings=dict(FLOAT_BINDINGS), bits=case["bits"], **extra)
