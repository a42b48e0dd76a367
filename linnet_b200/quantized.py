"""`std.quant`'s int8 linear layers as generated PyTorch calls them, on B200.

Mirror of python/linnet/src/linnet/torch/quantized.py for the int8 formats: each layer
is two calls, `*_operands` once per bound weights (run by `prepare`) and `*_linear`
per step.  The operand tuples have the reference's members
(`Int8Operands = (weight, scale_f32, rounded, fast)`, quantized.py:62-66).

Row-count dispatch as the reference's `_weight_only` (quantized.py:90-105): one row goes to
`gemv8`, up to `TILED_ROWS` rows to `w8a16` (both stream the int8 weight once through the
decode kernel), more rows dequantize the weight once with `dequantize8` and hand the dense
product to the library GEMM, which is the reference's own route for that range.  `rounded`
with more than `FEW_ROWS` rows takes the 8-bit-activation route (`int8_rows` + `int8_mm`,
quantized.py:187-189).  There is no fallback for CPU tensors.
"""

from __future__ import annotations

import torch

from . import kernels

Int8Operands = tuple[torch.Tensor, torch.Tensor, int, int]
Int8GroupOperands = tuple[torch.Tensor, torch.Tensor, int, int]

_HALF = (torch.bfloat16, torch.float16)

# Where the kernels switch (the reference's constants, python/linnet/src/linnet/quant.py:73-80).
FEW_ROWS = 32
TILED_ROWS = 64


def _weight_only(flat: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, group: int = 0) -> torch.Tensor:
    rows = flat.shape[0]
    if rows == 1:
        return kernels.gemv8(flat, weight, scale, False, group, 1)
    if rows <= TILED_ROWS:
        return kernels.w8a16(flat, weight, scale, False, group, 1)
    dequantized = kernels.dequantize8(weight, scale, False, group, 1, flat.dtype)
    # f32 accumulation all the way: the library may otherwise add split-K partial sums in the
    # 16-bit type, which alone costs more than the 1e-2 this layer is held to.
    matmul = torch.backends.cuda.matmul
    saved = (matmul.allow_bf16_reduced_precision_reduction, matmul.allow_fp16_reduced_precision_reduction)
    matmul.allow_bf16_reduced_precision_reduction = matmul.allow_fp16_reduced_precision_reduction = False
    try:
        return torch.nn.functional.linear(flat, dequantized)
    finally:
        matmul.allow_bf16_reduced_precision_reduction, matmul.allow_fp16_reduced_precision_reduction = saved


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
    weight, scale, rounded, _fast = operands
    _require(x, "int8_linear")
    flat = x.reshape(-1, x.shape[-1])
    if rounded and flat.shape[0] > FEW_ROWS and kernels.int8_mm_available(weight):
        q, row_scale = kernels.int8_rows(flat)
        y = kernels.int8_mm(q, weight, row_scale, scale, flat.dtype)
    else:
        y = _weight_only(flat, weight, scale)
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
    return _finish(x, _weight_only(flat, weight, scale, group), bias)
