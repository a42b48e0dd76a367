"""The CPU oracle reproduces what the reference itself produced (committed
fixtures made by `tests/golden/make_golden.py`), bit for bit."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import linear_oracle as lo
from oracle import quant_oracle as qo


def test_int4_quantizer_matches_reference_bytes(golden_quantizer):
    for name, case in golden_quantizer["q4"].items():
        packed, scale, zero = qo.quantize_int4_groups(case["w"], int(case["group"]))
        assert np.array_equal(packed, case["packed"]), name
        assert np.array_equal(scale.view(np.uint32), case["scale"].view(np.uint32)), name
        assert np.array_equal(zero, case["zero"]), name
        assert np.array_equal(qo.bf16_bits(scale), case["scale_bf16_bits"]), name


def test_int8_quantizer_matches_reference_bytes(golden_quantizer):
    for name, variants in golden_quantizer["q8"].items():
        w = golden_quantizer["q4"][name]["w"]
        for variant, case in variants.items():
            dtype = "f32" if variant == "channel" else variant
            q, scale = qo.quantize_int8_groups(w, int(case["group"]), dtype)
            assert np.array_equal(q, case["q"]), (name, variant)
            assert np.array_equal(scale.view(np.uint32), case["scale"].view(np.uint32)), (name, variant)


def test_reference_rounding_property(golden_quantizer):
    """tests/test_quant_groups.py:48-56 of the reference: error <= step/2."""
    case = golden_quantizer["q4"]["ref_test_64x256_g128"]
    packed, scale, zero = qo.quantize_int4_groups(case["w"], 128)
    assert packed.shape == (64, 2, 64) and packed.dtype == np.uint8
    err = np.abs(qo.dequantize_int4_groups(packed, scale, zero) - case["w"])
    assert np.all(err <= np.repeat(scale, 128, axis=1) / 2 + 1e-6)


def test_pack_roundtrip():
    rng = np.random.default_rng(3)
    levels = rng.integers(0, 16, size=(8, 256)).astype(np.uint8)
    packed = qo.pack_nibbles(levels, 64)
    assert packed.shape == (8, 4, 32)
    assert np.array_equal(qo.unpack_nibbles(packed).reshape(8, 256), levels)
    # low nibble is the even element (python/linnet/src/linnet/torch/packed.py:21-24)
    assert packed[0, 0, 0] == (levels[0, 0] | (levels[0, 1] << 4))


def _bf16(bits):
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


@pytest.mark.parametrize("rows", [1, 3, 16, 40])
def test_int4_linear_matches_reference(golden_linear, rows):
    g = golden_linear["lin4"]
    x = _bf16(g[f"rows{rows}"]["x_bits"])
    y = lo.int4_groups_linear(x, torch.from_numpy(g["packed"]), _bf16(g["scale_bits"]),
                              torch.from_numpy(g["zero"]))
    assert torch.equal(y.view(torch.int16), torch.from_numpy(g[f"rows{rows}"]["y_bits"]))


@pytest.mark.parametrize("rows", [1, 5, 16])
def test_int8_linear_matches_reference(golden_linear, rows):
    g = golden_linear["lin8"]
    x = _bf16(g[f"rows{rows}"]["x_bits"])
    y = lo.int8_linear(x, torch.from_numpy(g["q_rows"]), torch.from_numpy(g["s_rows"]))
    assert torch.equal(y.view(torch.int16), torch.from_numpy(g[f"rows{rows}"]["y_rows_bits"]))
    y = lo.int8_group_linear(x, torch.from_numpy(g["q_groups"]), torch.from_numpy(g["s_groups"]))
    assert torch.equal(y.view(torch.int16), torch.from_numpy(g[f"rows{rows}"]["y_groups_bits"]))
