"""`std.quant`'s int8 linear layers as generated PyTorch calls them, on B200.

Mirror of python/linnet/src/linnet/torch/quantized.py for the int8 formats: each layer
is two calls, `*_operands` once per bound weights (run by `prepare`) and `*_linear`
per step.  The operand tuples have the reference's members
(`Int8Operands = (weight, scale_f32, rounded, fast)`, quantized.py:62-66).

Differences, all within this build's scope: the product always reads the weight as it
is (weight-only) -- `rounded` is carried but the 8-bit-activation route of
`numerics="fast"` past 32 rows (quantized.py:187-189) is not built; and there is no
dequantize-and-`F.linear` fallback for CPU tensors.
"""

from __future__ import annotations

import torch

from . import kernels

Int8Operands = tuple[torch.Tensor, torch.Tensor, int, int]
Int8GroupOperands = tuple[torch.Tensor, torch.Tensor, int, int]

_HALF = (torch.bfloat16, torch.float16)


def _finish(x: torch.Tensor, y: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    y = y.reshape(*x.shape[:-1], y.shape[-1])
    return y if bias is None else y + bias


def _require(x: torch.Tensor, who: str) -> None:
    if not x.is_cuda or x.dtype not in _HALF:
        raise RuntimeError(f"{who}: needs bf16 or f16 activations on a CUDA device "
                           f"(got {x.dtype} on {x.device}); this build has no other path")


def int8_operands(weight: torch.Tensor, scale: torch.Tensor, rounded: int) -> Int8Operands:
    """`weight` [Out, In] i8, `scale` [Out]: the weight and the scales as f32."""
    weight = weight.contiguous()
    return weight, scale.float().reshape(-1).contiguous(), rounded, int(weight.is_cuda)


def int8_linear(x: torch.Tensor, operands: Int8Operands, bias: torch.Tensor | None) -> torch.Tensor:
    weight, scale, _rounded, _fast = operands
    _require(x, "int8_linear")
    flat = x.reshape(-1, x.shape[-1])
    if flat.shape[0] == 1:
        y = kernels.gemv8(flat, weight, scale, False, 0, 1)
    else:
        y = kernels.w8a16(flat, weight, scale, False, 0, 1)
    return _finish(x, y, bias)


def int8_group_operands(weight: torch.Tensor, scale: torch.Tensor) -> Int8GroupOperands:
    """`weight` [Out, In] i8, `scale` [Out, In / group]: the weight, the scales as f32,
    and the group."""
    weight = weight.contiguous()
    group = weight.shape[1] // scale.shape[1]
    return weight, scale.float().contiguous(), group, int(weight.is_cuda)


def int8_group_linear(x: torch.Tensor, operands: Int8GroupOperands,
                      bias: torch.Tensor | None) -> torch.Tensor:
    weight, scale, group, _fast = operands
    _require(x, "int8_group_linear")
    flat = x.reshape(-1, x.shape[-1])
    if flat.shape[0] == 1:
        y = kernels.gemv8(flat, weight, scale, False, group, 1)
    else:
        y = kernels.w8a16(flat, weight, scale, False, group, 1)
    return _finish(x, y, bias)
