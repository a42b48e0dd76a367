"""Group quantize / pack on the GPU, bit-exact with the reference's NumPy quantizer
(python/linnet/src/linnet/quant.py:83-120, :242-248).

Same functions and results: `quantize_int4_groups(weight, group)` returns
`(packed u8 [Out, In/group, group/2], scale f32 [Out, In/group], zero u8)`,
`quantize_int8_groups(weight, group, dtype)` returns `(q i8 [Out, In], scale f32)`.
A NumPy array in gives NumPy arrays out (computed on the current CUDA device); a torch
tensor in (f32 or bf16, CPU or CUDA) gives CUDA tensors out.
"""

from __future__ import annotations

import numpy as np
import torch

from . import _lib

_SCALE_CODES = {"f32": _lib.F32, "bf16": _lib.BF16, "f16": _lib.F16}
_TORCH_OF = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


class LinnetError(Exception):
    """Raised for the argument errors the reference reports with its `LinnetError`."""


def _device_weight(weight) -> tuple[torch.Tensor, bool]:
    as_numpy = isinstance(weight, np.ndarray)
    t = torch.from_numpy(np.ascontiguousarray(weight)) if as_numpy else weight
    if t.dim() != 2:
        raise LinnetError(f"a linear weight is [Out, In]; this one is {list(t.shape)}")
    if t.dtype not in (torch.float32, torch.bfloat16):
        t = t.float()  # the reference widens every float dtype to f32 first
    return t.cuda().contiguous(), as_numpy


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def quantize_int4_groups(weight, group: int = 128, *, scale_dtype: str | None = None):
    """`(packed, scale, zero)` for a `[Out, In]` weight; `scale` is f32.  With
    `scale_dtype` ("bf16", "f16", "f32") a fourth result is the scale as a checkpoint
    stores it (rounded to nearest even), computed in the same pass."""
    w, as_numpy = _device_weight(weight)
    out_features, in_features = w.shape
    if group <= 0 or group % 2 != 0 or in_features % group != 0:
        raise LinnetError(f"groups of {group} must be even and divide the {in_features} inputs")
    groups = in_features // group
    packed = torch.empty(out_features, groups, group // 2, dtype=torch.uint8, device=w.device)
    scale = torch.empty(out_features, groups, dtype=torch.float32, device=w.device)
    zero = torch.empty(out_features, groups, dtype=torch.uint8, device=w.device)
    stored = None
    if scale_dtype is not None:
        if scale_dtype not in _SCALE_CODES:
            raise LinnetError(f"scales are stored as bf16, f16, or f32, not {scale_dtype}")
        stored = torch.empty(out_features, groups, dtype=_TORCH_OF[scale_dtype], device=w.device)
    with torch.cuda.device(w.device):
        _lib.check(_lib.load().b200q_quantize_int4_groups(
            w.data_ptr(), _lib.BF16 if w.dtype == torch.bfloat16 else _lib.F32, out_features,
            in_features, group, packed.data_ptr(), scale.data_ptr(),
            stored.data_ptr() if stored is not None else None,
            _SCALE_CODES[scale_dtype or "f32"], zero.data_ptr(), _stream()))
    results = (packed, scale, zero) if stored is None else (packed, scale, zero, stored)
    if as_numpy:
        return tuple(r.float().cpu().numpy() if r.dtype in (torch.bfloat16, torch.float16)
                     else r.cpu().numpy() for r in results)
    return results


def quantize_int8_groups(weight, group: int = 128, dtype: str = "f32"):
    """`(q, scale)` for a `[Out, In]` weight: each group's largest magnitude over 127,
    rounded to `dtype` (the dtype it is stored in), and `q` the nearest levels against
    that stored scale; `scale` is f32."""
    w, as_numpy = _device_weight(weight)
    out_features, in_features = w.shape
    if group <= 0 or in_features % group != 0:
        raise LinnetError(f"groups of {group} must divide the {in_features} inputs")
    if dtype not in _SCALE_CODES:
        raise LinnetError(f"scales are stored as bf16, f16, or f32, not {dtype}")
    q = torch.empty(out_features, in_features, dtype=torch.int8, device=w.device)
    scale = torch.empty(out_features, in_features // group, dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        _lib.check(_lib.load().b200q_quantize_int8_groups(
            w.data_ptr(), _lib.BF16 if w.dtype == torch.bfloat16 else _lib.F32, out_features,
            in_features, group, _SCALE_CODES[dtype], q.data_ptr(), scale.data_ptr(), _stream()))
    if as_numpy:
        return q.cpu().numpy(), scale.cpu().numpy()
    return q, scale


def pack_int4_groups(q, group: int):
    """`[Out, In]` values in 0..15 as `[Out, In / group, group / 2]` bytes, low nibble
    first (quant.py:242-248).  Pure indexing; runs where `q` lives."""
    as_numpy = isinstance(q, np.ndarray)
    t = torch.from_numpy(np.ascontiguousarray(q)) if as_numpy else q
    out_features, in_features = t.shape
    grouped = t.reshape(out_features, in_features // group, group).to(torch.uint8)
    packed = grouped[..., 0::2] | (grouped[..., 1::2] << 4)
    return packed.numpy() if as_numpy else packed
