"""NumPy restatement of the reference's offline quantizer (test infrastructure).

Each function names the reference routine it follows
(`python/linnet/src/linnet/quant.py`, `python/linnet/src/linnet/weights.py`).
All arithmetic is IEEE binary32 with NumPy's rounding (`np.round` is
round-half-to-even, `/` is a correctly rounded division); the CUDA quantizer
must reproduce these bytes exactly.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32


def bf16_bits(values: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns (uint16), round to nearest even.

    Follows `to_bf16_bits`, weights.py:74-79: add 0x7FFF plus the lowest kept
    bit to the f32 word and keep the top half.
    """
    words = np.ascontiguousarray(values, dtype=F32).view(np.uint32)
    bumped = words + np.uint32(0x7FFF) + ((words >> 16) & np.uint32(1))
    return (bumped >> 16).astype(np.uint16)


def bf16_value(bits: np.ndarray) -> np.ndarray:
    """bf16 bit patterns -> the f32 they denote (`from_bf16_bits`, weights.py:82-84)."""
    return (np.asarray(bits).view(np.uint16).astype(np.uint32) << 16).view(F32)


def round_to_stored(scale: np.ndarray, dtype: str) -> np.ndarray:
    """`scale` rounded through the dtype it will be stored in, back as f32.

    quant.py:117-118 (`decode_floats(stored, encode_floats(scale, stored))`).
    """
    if dtype == "f32":
        return scale.astype(F32)
    if dtype == "bf16":
        return bf16_value(bf16_bits(scale)).reshape(scale.shape)
    if dtype == "f16":
        return scale.astype(np.float16).astype(F32)
    raise ValueError(f"scales are stored as bf16, f16, or f32, not {dtype}")


def pack_nibbles(levels: np.ndarray, group: int) -> np.ndarray:
    """`[Out, In]` levels 0..15 -> `[Out, In/group, group/2]` bytes, even k in the
    low nibble (`pack_int4_groups`, quant.py:242-248)."""
    rows, cols = levels.shape
    g = levels.reshape(rows, cols // group, group).astype(np.uint8)
    return (g[..., 0::2] | (g[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    """Inverse of `pack_nibbles`: `[Out, G, group/2]` -> `[Out, G, group]` uint8."""
    rows, groups, half = packed.shape
    return np.stack([packed & 15, packed >> 4], axis=-1).reshape(rows, groups, 2 * half)


def quantize_int4_groups(weight: np.ndarray, group: int = 128):
    """Asymmetric 4-bit round-to-nearest per group of `group` inputs.

    Follows `quantize_int4_groups`, quant.py:83-99.  Returns
    `(packed u8 [Out, In/group, group/2], scale f32 [Out, In/group],
    zero u8 [Out, In/group])`.  The scale is NOT rounded to the storage dtype
    before the levels are chosen (it is rounded only when written,
    quant.py:205-209).
    """
    if weight.ndim != 2:
        raise ValueError(f"a linear weight is [Out, In]; this one is {list(weight.shape)}")
    rows, cols = weight.shape
    if group <= 0 or group % 2 != 0 or cols % group != 0:
        raise ValueError(f"groups of {group} must be even and divide the {cols} inputs")
    g = weight.astype(F32).reshape(rows, cols // group, group)
    lo = g.min(axis=-1)
    hi = g.max(axis=-1)
    step = (hi - lo) / F32(15.0)
    step = np.where(step > 0, step, F32(1.0)).astype(F32)
    zero = np.clip(np.round(-lo / step), 0, 15).astype(np.uint8)
    levels = np.clip(np.round(g / step[..., None]) + zero[..., None], 0, 15)
    return pack_nibbles(levels.reshape(rows, cols), group), step, zero


def quantize_int8_groups(weight: np.ndarray, group: int = 128, dtype: str = "f32"):
    """Symmetric int8 per group; per-output-channel is `group == In`.

    Follows `quantize_int8_groups`, quant.py:102-120: the scale is absmax/127,
    replaced by 1 where it is not positive, rounded through the storage dtype
    FIRST, and the levels are then rounded against that stored scale.
    Returns `(q i8 [Out, In], scale f32 [Out, In/group])`.
    """
    if weight.ndim != 2:
        raise ValueError(f"a linear weight is [Out, In]; this one is {list(weight.shape)}")
    rows, cols = weight.shape
    if group <= 0 or cols % group != 0:
        raise ValueError(f"groups of {group} must divide the {cols} inputs")
    g = weight.astype(F32).reshape(rows, cols // group, group)
    scale = np.abs(g).max(axis=-1) / F32(127.0)
    scale = np.where(scale > 0, scale, F32(1.0)).astype(F32)
    scale = round_to_stored(scale, dtype)
    q = np.clip(np.round(g / scale[..., None]), -127, 127).astype(np.int8)
    return q.reshape(rows, cols), scale


def dequantize_int4_groups(packed: np.ndarray, scale: np.ndarray, zero: np.ndarray) -> np.ndarray:
    """f32 `[Out, In]` weight of an int4 group layer (quant.py:131-136)."""
    q = unpack_nibbles(packed).astype(F32)
    w = (q - zero[..., None].astype(F32)) * scale[..., None].astype(F32)
    return w.reshape(packed.shape[0], -1)


def dequantize_int8_groups(q: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """f32 `[Out, In]` weight of an int8 group layer (quant.py:123-128)."""
    rows, cols = q.shape
    groups = scale.shape[1]
    g = q.astype(F32).reshape(rows, groups, cols // groups)
    return (g * scale[..., None].astype(F32)).reshape(rows, cols)
