"""GPU quantize / pack kernels against the reference's bytes (golden fixtures) and the
CPU oracle, bit for bit."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu


def _bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_int4_matches_reference_fixtures(golden_quantizer):
    from linnet_b200 import quant

    for name, case in golden_quantizer["q4"].items():
        packed, scale, zero, stored = quant.quantize_int4_groups(
            torch.from_numpy(case["w"]), int(case["group"]), scale_dtype="bf16")
        assert np.array_equal(packed.cpu().numpy(), case["packed"]), name
        assert np.array_equal(_bits(scale.cpu().numpy()), _bits(case["scale"])), name
        assert np.array_equal(zero.cpu().numpy(), case["zero"]), name
        got_bits = stored.view(torch.int16).cpu().numpy().view(np.uint16)
        assert np.array_equal(got_bits, case["scale_bf16_bits"]), name


def test_int8_matches_reference_fixtures(golden_quantizer):
    from linnet_b200 import quant

    for name, variants in golden_quantizer["q8"].items():
        w = golden_quantizer["q4"][name]["w"]
        for variant, case in variants.items():
            dtype = "f32" if variant == "channel" else variant
            q, scale = quant.quantize_int8_groups(torch.from_numpy(w), int(case["group"]), dtype)
            assert np.array_equal(q.cpu().numpy(), case["q"]), (name, variant)
            assert np.array_equal(_bits(scale.cpu().numpy()), _bits(case["scale"])), (name, variant)


def test_numpy_in_numpy_out(golden_quantizer):
    from linnet_b200 import quant

    case = golden_quantizer["q4"]["ref_test_64x256_g128"]
    packed, scale, zero = quant.quantize_int4_groups(case["w"], 128)
    assert isinstance(packed, np.ndarray) and packed.dtype == np.uint8
    assert np.array_equal(packed, case["packed"]) and np.array_equal(zero, case["zero"])
    assert np.array_equal(quant.pack_int4_groups(qo.unpack_nibbles(packed).reshape(64, 256), 128), packed)


@pytest.mark.parametrize("shape,group", [((512, 4096), 128), ((300, 1536), 64), ((64, 8192), 256),
                                         ((33, 96), 24), ((16, 40), 10), ((8, 6144), 2048),
                                         ((5, 28672), 4096)])
@pytest.mark.parametrize("source", ["bf16", "f32"])
def test_int4_matches_oracle(shape, group, source):
    from linnet_b200 import quant

    gen = torch.Generator().manual_seed(shape[0] * 7 + group)
    w = torch.randn(*shape, generator=gen) * 0.015
    if source == "bf16":
        w = w.to(torch.bfloat16)
    want = qo.quantize_int4_groups(w.float().numpy(), group)
    got = quant.quantize_int4_groups(w, group)
    for g, e in zip(got, want):
        assert np.array_equal(g.cpu().numpy().view(np.uint8), e.view(np.uint8))


@pytest.mark.parametrize("shape,group", [((256, 4096), 128), ((64, 8192), 8192), ((24, 28672), 28672),
                                         ((40, 1000), 1000), ((16, 96), 16), ((9, 20480), 20480 // 5)])
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_int8_matches_oracle(shape, group, dtype):
    from linnet_b200 import quant

    gen = torch.Generator().manual_seed(shape[0] + group)
    w = (torch.randn(*shape, generator=gen) * 0.015).to(torch.bfloat16)
    want_q, want_s = qo.quantize_int8_groups(w.float().numpy(), group, dtype)
    q, s = quant.quantize_int8_groups(w, group, dtype)
    assert np.array_equal(q.cpu().numpy(), want_q)
    assert np.array_equal(_bits(s.cpu().numpy()), _bits(want_s))


def _adversarial(rows: int, group: int, groups: int) -> np.ndarray:
    """Groups whose quotients land on exact half-integers (with even and odd zero points), sit
    one ulp either side of them, are clipped, are huge, or do not vary at all."""
    rng = np.random.default_rng(group)
    w = np.zeros((rows, groups, group), dtype=np.float32)
    for r in range(rows):
        for g in range(groups):
            kind = (r * groups + g) % 8
            halves = rng.integers(0, 31, size=group).astype(np.float32) * 0.5   # 0, 0.5, ... 15
            if kind == 0:      # step 1, zero 0: ties everywhere
                v = halves.copy(); v[0], v[1] = 0.0, 15.0
            elif kind == 1:    # step 1, zero 4 (from -3.5, itself a tie)
                v = halves - 3.5; v[0], v[1] = -3.5, 11.5
            elif kind == 2:    # step 1, zero 7: the zero's parity differs from kind 1's
                v = halves - 7.0; v[0], v[1] = -7.0, 8.0
            elif kind == 3:    # one ulp either side of the ties, odd step
                v = (halves * np.float32(0.3)).astype(np.float32)
                v = np.nextafter(v, np.where(rng.integers(0, 2, size=group) == 0, -np.inf, np.inf).astype(np.float32))
                v[0], v[1] = 0.0, np.float32(4.5)
            elif kind == 4:    # all positive and far from zero: the zero point clips, the levels clip
                v = (1000.0 + rng.random(group) * 0.01).astype(np.float32)
            elif kind == 5:    # huge magnitudes
                v = (rng.standard_normal(group) * 1e30).astype(np.float32)
            elif kind == 6:    # no variation: the step is replaced by 1
                v = np.full(group, -2.5 if r % 2 else 0.0, dtype=np.float32)
            else:              # ordinary weights
                v = (rng.standard_normal(group) * 0.015).astype(np.float32)
            w[r, g] = v
    return w.reshape(rows, groups * group)


@pytest.mark.parametrize("group,groups", [(128, 16), (64, 8), (32, 8), (16, 8), (256, 4), (24, 8), (4096, 2)])
def test_ties_clips_and_extremes(group, groups):
    from linnet_b200 import quant

    w = _adversarial(16, group, groups)
    want = qo.quantize_int4_groups(w, group)
    got = quant.quantize_int4_groups(torch.from_numpy(w), group)
    for g, e in zip(got, want):
        assert np.array_equal(g.cpu().numpy().view(np.uint8), e.view(np.uint8))
    # int8: make the largest magnitude of every group 127 * 2^k so that halves are ties there too
    w8 = w.copy().reshape(16, groups, group)
    w8[:, :, 2] = np.where(np.abs(w8).max(axis=2) < 127, 127.0, w8[:, :, 2])
    w8 = w8.reshape(16, groups * group)
    for dtype in ("f32", "bf16"):
        want_q, want_s = qo.quantize_int8_groups(w8, group, dtype)
        q, s = quant.quantize_int8_groups(torch.from_numpy(w8), group, dtype)
        assert np.array_equal(q.cpu().numpy(), want_q)
        assert np.array_equal(_bits(s.cpu().numpy()), _bits(want_s))


def test_empty_and_bad_arguments():
    from linnet_b200 import quant

    packed, scale, zero = quant.quantize_int4_groups(torch.zeros(0, 256), 128)
    assert packed.shape == (0, 2, 64) and scale.shape == (0, 2)
    with pytest.raises(quant.LinnetError, match="must be even and divide"):
        quant.quantize_int4_groups(torch.zeros(4, 100), 128)
    with pytest.raises(quant.LinnetError, match=r"\[Out, In\]"):
        quant.quantize_int8_groups(torch.zeros(4, 4, 4), 2)


def test_full_size_rounding_property():
    """At a bulk-quantize shape (28672 x 8192, bf16 N(0, 0.015)): every weight is
    within half a step of its level (the reference's own property test), and a
    checksum of the packed bytes of sampled rows equals the oracle's."""
    from linnet_b200 import kernels, quant

    gen = torch.Generator().manual_seed(70)
    rows, cols = 28672, 8192
    w = torch.empty(rows, cols, dtype=torch.bfloat16)
    for r0 in range(0, rows, 4096):
        w[r0:r0 + 4096] = (torch.randn(4096, cols, generator=gen) * 0.015).to(torch.bfloat16)
    wd = w.cuda()
    packed, scale, zero, stored = quant.quantize_int4_groups(wd, 128, scale_dtype="f32")
    levels = torch.stack([packed & 15, packed >> 4], dim=-1).reshape(rows, cols // 128, 128)
    deq = (levels.float() - zero.float()[..., None]) * scale[..., None]
    err = (deq.reshape(rows, cols) - wd.float()).abs()
    assert bool((err <= scale.repeat_interleave(128, dim=1) / 2 + 1e-6).all())
    sample = torch.arange(0, rows, 997)
    want = qo.quantize_int4_groups(w[sample].float().numpy(), 128)
    assert np.array_equal(packed[sample.cuda()].cpu().numpy(), want[0])
    assert np.array_equal(zero[sample.cuda()].cpu().numpy(), want[2])
    q8, s8 = quant.quantize_int8_groups(wd, cols, "f32")
    want8 = qo.quantize_int8_groups(w[sample].float().numpy(), cols, "f32")
    assert np.array_equal(q8[sample.cuda()].cpu().numpy(), want8[0])
    assert np.array_equal(_bits(s8[sample.cuda()].cpu().numpy()), _bits(want8[1]))
