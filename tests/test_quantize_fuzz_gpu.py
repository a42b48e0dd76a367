"""The GPU quantizers against the NumPy oracle, bit for bit, on tensors of the bench's row
lengths and on distributions that stress the rounding: many exact ties (multiples of 0.25),
tiny and huge magnitudes.  (The short, hand-picked cases are in test_quantize_gpu.py.)"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu

CASES = {
    "weights": (1024, 8192, 0.015),
    "long_rows": (256, 28672, 0.02),
    "ties": (1024, 4096, None),  # small integers / 4: quotients land on half-integers by the thousand
    "tiny": (256, 8192, 1e-4),
    "huge": (256, 8192, 300.0),
}


def _weight(name: str) -> torch.Tensor:
    rows, cols, sigma = CASES[name]
    gen = torch.Generator().manual_seed(len(name) + rows)
    if sigma is None:
        return (torch.randint(-40, 41, (rows, cols), generator=gen).float() * 0.25).to(torch.bfloat16)
    return (torch.randn(rows, cols, generator=gen) * sigma).to(torch.bfloat16)


def _same_bits(a: torch.Tensor, b: np.ndarray) -> bool:
    return np.array_equal(a.cpu().numpy().view(np.uint32).reshape(-1), b.astype(np.float32).view(np.uint32).reshape(-1))


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("group", [64, 128, 256])
def test_int4_groups_bit_exact(name, group):
    from linnet_b200 import quant

    w = _weight(name)
    packed, scale, zero = quant.quantize_int4_groups(w.cuda(), group)
    want_packed, want_scale, want_zero = qo.quantize_int4_groups(w.float().numpy(), group)
    assert np.array_equal(packed.cpu().numpy().reshape(want_packed.shape), want_packed)
    assert _same_bits(scale, want_scale)
    assert np.array_equal(zero.cpu().numpy().reshape(-1), want_zero.reshape(-1))


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize(("per_channel", "dtype"), [(True, "f32"), (True, "bf16"), (False, "bf16"), (False, "f32")])
def test_int8_groups_bit_exact(name, per_channel, dtype):
    from linnet_b200 import quant

    w = _weight(name)
    group = w.shape[1] if per_channel else 128
    q, scale = quant.quantize_int8_groups(w.cuda(), group, dtype)
    want_q, want_scale = qo.quantize_int8_groups(w.float().numpy(), group, dtype)
    assert np.array_equal(q.cpu().numpy().reshape(want_q.shape), want_q)
    assert _same_bits(scale, want_scale)
