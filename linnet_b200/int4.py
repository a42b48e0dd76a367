"""The int4 helpers the reference's generated PyTorch source defines for
`std.quant::linear_int4_groups` (text at src/backend/torch_source.cpp:1482-1570),
re-pointed at the sm_100a kernels.

`_int4_pack` runs once per bound weights (the generated `prepare`), `_int4_linear` per
call.  The packed value stays a 3-tuple, which is how the reference's own test tells
the fast path from the dequantized-weight fallback
(python/linnet/tests/test_quant_groups.py:138-141); here it holds the contiguous
`(packed, scale, zero)` themselves, because the kernels read the checkpoint layout
directly and no tinygemm repack is needed.
"""

from __future__ import annotations

import torch

from . import kernels


def _int4_pack(packed: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor):
    if not packed.is_cuda or scale.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError("_int4_pack: int4 layers need CUDA tensors with bf16 or f16 scales; "
                           "this build has no CPU or f32 path")
    return (packed.contiguous(), scale.contiguous(), zero.contiguous())


def _int4_weight(raw: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor) -> torch.Tensor:
    """The weight dequantized, in `scale`'s type: one kernel."""
    return kernels.int4_dequantize(raw, scale, zero)


def _int4_linear(x, packed, bias, raw, scale, zero):
    """Same signature as the generated helper; every row count goes to
    `linnet::int4_linear`, which picks the decode kernel or the tensor-memory GEMM."""
    flat = x.reshape(-1, x.shape[-1])
    if len(packed) == 3:
        y = kernels.int4_linear(flat, packed[0], packed[1], packed[2])
    else:
        y = kernels.int4_linear(flat, raw, scale, zero)
    y = y.reshape(*x.shape[:-1], y.shape[-1])
    return y if bias is None else y + bias
