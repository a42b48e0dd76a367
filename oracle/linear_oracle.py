"""PyTorch-on-CPU restatement of the reference's quantized linear layers
(test infrastructure; never imported by the product).

These are the results the reference itself produces when its generated source
or its interpreter runs the layers on a CPU: the weight is dequantized in f32,
rounded ONCE to the activation dtype, and multiplied by `F.linear`.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def unpack_levels(packed: torch.Tensor) -> torch.Tensor:
    """`[Out, G, group/2]` bytes -> `[Out, G, group]` levels, even k from the low
    nibble (`_codes`, python/linnet/src/linnet/torch/packed.py:21-24)."""
    rows, groups, half = packed.shape
    return torch.stack([packed & 15, packed >> 4], dim=-1).reshape(rows, groups, 2 * half)


def int4_weight(packed: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor,
                dtype: torch.dtype) -> torch.Tensor:
    """The `[Out, In]` weight an int4 group layer multiplies by, in `dtype`.

    `(q.float() - zero.float()) * scale.float()` then one cast
    (`_int4_pack` CPU branch, src/backend/torch_source.cpp:1501-1504;
    `_int4_groups_linear`, python/linnet/src/linnet/torch/native.py:417-424).
    """
    rows, groups, half = packed.shape
    q = unpack_levels(packed)
    w = (q.float() - zero.float()[..., None]) * scale.float()[..., None]
    return w.reshape(rows, groups * 2 * half).to(dtype)


def int4_groups_linear(x, packed, scale, zero, bias=None):
    """`std.quant::linear_int4_groups` as the reference's torch path computes it
    on a CPU (torch_source.cpp:1553-1570 last branch; native.py:417-424)."""
    flat = x.reshape(-1, x.shape[-1])
    y = F.linear(flat, int4_weight(packed, scale, zero, x.dtype))
    y = y.reshape(*x.shape[:-1], y.shape[-1])
    return y if bias is None else y + bias


def int4_groups_linear_f32(x, packed, scale, zero):
    """The op as `stdlib/quant.linnet:113-175` defines it, before any 16-bit rounding of the
    weight: `x . ((q - zero) * scale)^T` in f64 (returned as f32), and beside it the most the
    reference's torch path can differ from that through rounding every weight once to the
    activation type: `eps * |x| . |w|^T` with eps = 2^-9 (bf16) or 2^-12 (f16)."""
    rows, groups, half = packed.shape
    q = unpack_levels(packed)
    w = ((q.double() - zero.double()[..., None]) * scale.double()[..., None]).reshape(rows, groups * 2 * half)
    flat = x.reshape(-1, x.shape[-1]).double()
    eps = 2.0 ** -9 if x.dtype == torch.bfloat16 else 2.0 ** -12
    return (flat @ w.T).float(), (eps * (flat.abs() @ w.abs().T)).float()


def int8_weight(weight: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """`(weight.float() * scale[:, None]).to(dtype)` for a per-row scale `[Out]`, or
    the grouped form for `scale [Out, In/group]`
    (python/linnet/src/linnet/torch/quantized.py:193, :213-216)."""
    rows, cols = weight.shape
    scale = scale.float()
    if scale.dim() == 1 or scale.shape[-1] == 1 and scale.numel() == rows:
        return (weight.float() * scale.reshape(rows, 1)).to(dtype)
    groups = scale.shape[1]
    g = weight.float().reshape(rows, groups, cols // groups)
    return (g * scale[:, :, None]).reshape(rows, cols).to(dtype)


def int8_linear_f32(x, weight, scale):
    """`std.quant::linear_int8` as `stdlib/quant.linnet:13-97` defines it, before any 16-bit
    rounding of the weight: `x . (w * scale)^T` in f64 (returned as f32), and the most the
    reference's CPU route can differ from that through rounding every weight once to the
    activation type (as `int4_groups_linear_f32`)."""
    w = weight.double() * scale.double().reshape(-1, 1)
    flat = x.reshape(-1, x.shape[-1]).double()
    eps = 2.0 ** -9 if x.dtype == torch.bfloat16 else 2.0 ** -12
    return (flat @ w.T).float(), (eps * (flat.abs() @ w.abs().T)).float()


def int8_linear(x, weight, scale, bias=None):
    """`std.quant::linear_int8` on a CPU (`int8_linear`, quantized.py:183-194)."""
    flat = x.reshape(-1, x.shape[-1])
    y = F.linear(flat, int8_weight(weight, scale.reshape(-1), x.dtype))
    y = y.reshape(*x.shape[:-1], y.shape[-1])
    return y if bias is None else y + bias


def int8_group_linear(x, weight, scale, bias=None):
    """`std.quant::linear_int8_groups` on a CPU (`int8_group_linear`,
    quantized.py:205-218)."""
    flat = x.reshape(-1, x.shape[-1])
    y = F.linear(flat, int8_weight(weight, scale, x.dtype))
    y = y.reshape(*x.shape[:-1], y.shape[-1])
    return y if bias is None else y + bias


def int8_rows(x: torch.Tensor):
    """Every row of `x` rounded to int8 with its own scale, as the reference's `int8_rows`
    defines it (python/linnet/src/linnet/torch/kernels.py:669-693): scale = max(max|row|,
    1e-12) / 127; level = x / scale, half away from zero (`x + 0.5` or `x - 0.5`, then
    truncation), clamped to +-127.  IEEE f32 throughout.  Returns (q i8, scale f32 [rows, 1])."""
    v = x.float()
    top = v.abs().amax(dim=1, keepdim=True).clamp_min(1e-12)
    scale = top / torch.tensor(127.0)
    s = v / scale
    r = torch.where(s >= 0, s + 0.5, s - 0.5).clamp(-127.0, 127.0)
    return r.trunc().to(torch.int8), scale


def int8_mm(xq: torch.Tensor, weight: torch.Tensor, x_scale: torch.Tensor, scale: torch.Tensor,
            dtype: torch.dtype) -> torch.Tensor:
    """`(xq @ weight.T)` exactly in integers, then `* x_scale * scale` in f32 in that order,
    one rounding to `dtype` (kernels.py:805-836)."""
    acc = xq.to(torch.int64) @ weight.to(torch.int64).T
    y = acc.to(torch.float32) * x_scale.float().reshape(-1, 1)
    y = y * scale.float().reshape(1, -1)
    return y.to(dtype)


def shard_int4(packed, scale, zero, rank: int, shards: int, split: str):
    """One tensor-parallel rank's slice of an int4 layer.

    `split == "column"` cuts output rows (axis 0 of all three tensors);
    `split == "row"` cuts whole input groups (axis 1).  This is what the
    reference's loader does when a card's shapes are divided by `Shards`
    (`bind_weights`, python/linnet/src/linnet/torch/module.py:558-585).
    """
    axis = 0 if split == "column" else 1
    def cut(t):
        n = t.shape[axis] // shards
        return t.narrow(axis, rank * n, n).contiguous()
    return cut(packed), cut(scale), cut(zero)
