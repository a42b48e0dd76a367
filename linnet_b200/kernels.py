"""The torch operators of the quantized-linear path, backed by sm_100a CUDA kernels.

Same names, arguments and results as the reference's Triton operators
(python/linnet/src/linnet/torch/kernels.py): `int4_linear` (`linnet::int4_linear`,
:277-323), `gemv8` (`linnet::gemv8`, :375-434), `w8a16` (`linnet::w8a16`, :526-592),
`dequantize8` (:619-666), `int8_rows` (`linnet::rows8`, :705-753) and `int8_mm`
(`linnet::int8_mm`, :856-915).  Each is a `torch.library` custom op with a fake
implementation, so it is opaque to `torch.compile` and recordable into a CUDA graph;
outside `torch.compile` the kernel is launched directly (the reference does the same
to keep the host cost of a decoding step low, kernels.py:43-55).

All launches go to PyTorch's current stream, never synchronise and never mutate
their arguments.  There is no fallback: tensors must live on a B200.
"""

from __future__ import annotations

import torch

from . import _lib

_CODES = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}


def _code(dtype: torch.dtype, who: str) -> int:
    if dtype not in (torch.bfloat16, torch.float16):
        raise ValueError(f"{who}: activations are bf16 or f16, not {dtype}")
    return _CODES[dtype]


def _on_gpu(who: str, *tensors: torch.Tensor) -> torch.device:
    device = tensors[0].device
    for t in tensors:
        if not t.is_cuda or t.device != device:
            raise RuntimeError(
                f"{who}: every tensor must be on one CUDA device (there is no CPU path in "
                f"this build); got {[str(t.device) for t in tensors]}")
    return device


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class _Device:
    """Makes `device` current for the launch when it is not already."""

    def __init__(self, device: torch.device) -> None:
        self.guard = None if device.index == torch.cuda.current_device() else torch.cuda.device(device)

    def __enter__(self) -> None:
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc: object) -> None:
        if self.guard is not None:
            self.guard.__exit__(*exc)


# ---- int4 ----------------------------------------------------------------------

_exact_weights = False


def set_int4_numerics(mode: str) -> None:
    """How the decode kernels apply zero point and scale (int4, groups of 128) or the per-row
    scale (int8), for one and two rows.
    "fast" (the default; the reference picks these kernels under its `fast` numerics policy
    only, src/opt/candidates.cpp:28-33): in f32 on each group's sum of exact products.
    "exact": every weight rounded to the activation type first, bit for bit the weight the
    reference's torch path multiplies by (python/linnet/src/linnet/torch/native.py:417-424),
    at about twice the instructions.  Both stay within rtol/atol 1e-2 of that path on
    weights ~N(0, 0.02)."""
    global _exact_weights
    if mode not in ("fast", "exact"):
        raise ValueError(f"int4 numerics are 'fast' or 'exact', not {mode!r}")
    _exact_weights = mode == "exact"


def int4_numerics() -> str:
    return "exact" if _exact_weights else "fast"


def _int4_linear(x: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor,
                 zero: torch.Tensor, out: torch.Tensor | None = None, early: bool = False,
                 swiglu: bool = False, overlap: bool = True) -> torch.Tensor:
    rows, depth = x.shape
    if swiglu:
        depth //= 2
    width, groups, half = packed.shape
    group = 2 * half
    block_k = min(group, 128)
    if block_k < 16 or group % block_k or block_k & (block_k - 1):
        # The reference's own limit and message (kernels.py:292-294).
        raise ValueError(f"int4_linear: a group of {group} is not 16, 32, 64, or a multiple of 128")
    if depth != groups * group:
        raise ValueError(f"int4_linear: x has {depth} inputs, the weight {groups * group}")
    if scale.dtype != x.dtype:
        raise ValueError(f"int4_linear: scales are {scale.dtype}, activations {x.dtype}")
    if packed.dtype != torch.uint8 or zero.dtype != torch.uint8:
        raise ValueError("int4_linear: packed weights and zero points are uint8")
    device = _on_gpu("int4_linear", x, packed, scale, zero)
    x, packed, scale, zero = x.contiguous(), packed.contiguous(), scale.contiguous(), zero.contiguous()
    if out is None:
        y = torch.empty(rows, width, dtype=x.dtype, device=device)
    else:
        if out.shape != (rows, width) or out.dtype != x.dtype or out.device != device or not out.is_contiguous():
            raise ValueError(f"int4_linear: out must be a contiguous [{rows}, {width}] {x.dtype} tensor on {device}")
        y = out
    with _Device(device):
        flags = ((_lib.EXACT_WEIGHTS if _exact_weights else 0) | (_lib.EARLY_DEPENDENTS if early else 0)
                 | (0 if overlap else _lib.NO_OVERLAP))
        lib = _lib.load()
        if swiglu:
            # the kernel that forms silu(gate) * up while it stages its input, where it takes the
            # call; else the stand-alone kernel first
            status = lib.b200q_int4_linear_ex(
                x.data_ptr(), packed.data_ptr(), scale.data_ptr(), zero.data_ptr(), y.data_ptr(),
                rows, depth, width, group, _code(x.dtype, "int4_linear"), flags | _lib.SWIGLU_INPUT, _stream(device))
            if status == _lib.OK:
                return y
            if status != _lib.UNAVAILABLE:
                _lib.check(status)
            if x.dtype == torch.bfloat16:
                from . import glue

                x = glue.silu_mul(x)
            else:
                x = torch.nn.functional.silu(x[:, :depth]) * x[:, depth:]
        _lib.check(lib.b200q_int4_linear_ex(
            x.data_ptr(), packed.data_ptr(), scale.data_ptr(), zero.data_ptr(), y.data_ptr(),
            rows, depth, width, group, _code(x.dtype, "int4_linear"), flags, _stream(device)))
    return y


@torch.library.custom_op("linnet::int4_linear", mutates_args=(), device_types="cuda")
def _int4_linear_op(x: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor,
                    zero: torch.Tensor) -> torch.Tensor:
    return _int4_linear(x, packed, scale, zero)


@_int4_linear_op.register_fake
def _(x, packed, scale, zero):
    return x.new_empty(x.shape[0], packed.shape[0])


def int4_linear(x: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor,
                zero: torch.Tensor, out: torch.Tensor | None = None, early: bool = False,
                swiglu: bool = False, overlap: bool = True) -> torch.Tensor:
    """`F.linear(x, W)` for `x` [rows, In] (bf16 or f16) and the group-wise 4-bit weight
    of `std.quant::linear_int4_groups`: `packed` [Out, Groups, Group/2] u8 (even value
    low), `scale` and `zero` [Out, Groups].  Any row count: up to 16 rows stream the
    weight once at HBM speed, more go through the tensor-memory GEMM.  `out` (eager
    calls only) receives the result in place of a new tensor, e.g. a buffer in peer-mapped
    memory that a tensor-parallel reduction reads next.  `early` (eager calls only): the next
    kernel in the stream is another product of the same input, which may start prefetching its
    weights at once (`B200Q_EARLY_DEPENDENTS`).  `swiglu` (eager calls only): `x` is
    [rows, 2 In] and the product's input is `silu(x[:, :In]) * x[:, In:]`, formed inside the
    product for one and two rows (`B200Q_SWIGLU_INPUT`) and by `glue.silu_mul` otherwise.
    `overlap=False` (eager calls only): the one- and two-row kernel starts in plain stream order
    instead of early (`B200Q_NO_OVERLAP`)."""
    if out is None and not early and not swiglu and overlap and torch.compiler.is_compiling():
        return _int4_linear_op(x, packed, scale, zero)
    return _int4_linear(x, packed, scale, zero, out, early, swiglu, overlap)


def int4_linear_norm(x: torch.Tensor, delta: torch.Tensor | None, norm_weight: torch.Tensor, eps: float,
                     x_out: torch.Tensor | None, packed: torch.Tensor, scale: torch.Tensor,
                     zero: torch.Tensor) -> torch.Tensor | None:
    """A decoder layer's residual add, RMS norm and the product that follows as one launch
    (`b200q_int4_gemv_norm`): returns `F.linear(rms_norm(x + delta) * norm_weight, W)` and stores
    `x + delta` to `x_out` (a buffer other than `x`; unused when `delta` is None), or None where
    that kernel does not take the call (more than two rows, exact numerics, another dtype or
    group): the caller then runs `glue.add_rmsnorm` and `int4_linear`.  Eager calls only."""
    rows, depth = x.shape
    width, groups, half = packed.shape
    if _exact_weights or rows > 2 or 2 * half != 128 or x.dtype != torch.bfloat16 or depth != groups * 128:
        return None
    if scale.dtype != x.dtype or packed.dtype != torch.uint8 or zero.dtype != torch.uint8:
        raise ValueError("int4_linear_norm: bf16 scales, uint8 weights and zero points")
    device = _on_gpu("int4_linear_norm", x, norm_weight, packed, scale, zero)
    for t in (x, norm_weight, packed, scale, zero) + ((delta, x_out) if delta is not None else ()):
        if t is None or not t.is_contiguous():
            raise ValueError("int4_linear_norm: contiguous tensors (and x_out with delta)")
    y = torch.empty(rows, width, dtype=x.dtype, device=device)
    with _Device(device):
        status = _lib.load().b200q_int4_gemv_norm(
            x.data_ptr(), None if delta is None else delta.data_ptr(), norm_weight.data_ptr(), float(eps),
            None if delta is None else x_out.data_ptr(), packed.data_ptr(), scale.data_ptr(), zero.data_ptr(),
            y.data_ptr(), rows, depth, width, 128, _lib.BF16, 0, _stream(device))
    if status == _lib.UNAVAILABLE:
        return None
    _lib.check(status)
    return y


def int4_dequantize(packed: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor) -> torch.Tensor:
    """The [Out, In] weight in `scale`'s dtype, `(q - zero) * scale` rounded once: what
    the generated `_int4_weight` computes (src/backend/torch_source.cpp:1537-1551)."""
    width, groups, half = packed.shape
    device = _on_gpu("int4_dequantize", packed, scale, zero)
    packed, scale, zero = packed.contiguous(), scale.contiguous(), zero.contiguous()
    out = torch.empty(width, groups * 2 * half, dtype=scale.dtype, device=device)
    with _Device(device):
        _lib.check(_lib.load().b200q_int4_dequantize(
            packed.data_ptr(), scale.data_ptr(), zero.data_ptr(), out.data_ptr(), width,
            groups * 2 * half, 2 * half, _code(scale.dtype, "int4_dequantize"), _stream(device)))
    return out


# ---- int8 ----------------------------------------------------------------------


def _no_fp8(who: str, fp8: bool) -> None:
    if fp8:
        raise NotImplementedError(f"{who}: FP8 weights are outside this build (int8 only)")


def _eight_bit(who: str, x: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, fp8: bool,
               group: int, row_block: int) -> torch.Tensor:
    _no_fp8(who, fp8)
    if row_block != 1:
        raise NotImplementedError(f"{who}: block scales (row_block {row_block}) are an FP8 format")
    if weight.dtype != torch.int8:
        raise ValueError(f"{who}: int8 weights expected, got {weight.dtype}")
    rows, depth = x.shape
    width = weight.shape[0]
    if weight.shape[1] != depth:
        raise ValueError(f"{who}: x has {depth} inputs, the weight {weight.shape[1]}")
    device = _on_gpu(who, x, weight, scale)
    x, weight = x.contiguous(), weight.contiguous()
    scale = scale.float().contiguous()
    y = torch.empty(rows, width, dtype=x.dtype, device=device)
    with _Device(device):
        _lib.check(_lib.load().b200q_int8_linear_ex(
            x.data_ptr(), weight.data_ptr(), scale.data_ptr(), y.data_ptr(), rows, depth, width,
            group, _code(x.dtype, who), _lib.EXACT_WEIGHTS if _exact_weights else 0, _stream(device)))
    return y


@torch.library.custom_op("linnet::gemv8", mutates_args=(), device_types="cuda")
def _gemv8_op(x: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, fp8: bool, group: int,
              row_block: int) -> torch.Tensor:
    return _eight_bit("gemv8", x, weight, scale, fp8, group, row_block)


@_gemv8_op.register_fake
def _(x, weight, scale, fp8, group, row_block):
    return x.new_empty(x.shape[0], weight.shape[0])


@torch.library.custom_op("linnet::w8a16", mutates_args=(), device_types="cuda")
def _w8a16_op(x: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, fp8: bool, group: int,
              row_block: int) -> torch.Tensor:
    return _eight_bit("w8a16", x, weight, scale, fp8, group, row_block)


@_w8a16_op.register_fake
def _(x, weight, scale, fp8, group, row_block):
    return x.new_empty(x.shape[0], weight.shape[0])


def gemv8(x: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, fp8: bool, group: int,
          row_block: int) -> torch.Tensor:
    """`F.linear(x, W)` for one row `x` [1, In] and int8 weights [Out, In] times `scale`:
    one a row ([Out]) when `group` is 0, else [Out, In/group]."""
    if torch.compiler.is_compiling():
        return _gemv8_op(x, weight, scale, fp8, group, row_block)
    return _eight_bit("gemv8", x, weight, scale, fp8, group, row_block)


def w8a16(x: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, fp8: bool, group: int,
          row_block: int) -> torch.Tensor:
    """`F.linear(x, W)` for a few rows `x` [rows, In]; same weights as `gemv8`."""
    if torch.compiler.is_compiling():
        return _w8a16_op(x, weight, scale, fp8, group, row_block)
    return _eight_bit("w8a16", x, weight, scale, fp8, group, row_block)


def dequantize8(weight: torch.Tensor, scale: torch.Tensor, fp8: bool, group: int, row_block: int,
                dtype: torch.dtype) -> torch.Tensor:
    """The int8 weight of `gemv8` dequantized to `dtype` (f32 product, one rounding)."""
    _no_fp8("dequantize8", fp8)
    device = _on_gpu("dequantize8", weight, scale)
    width, depth = weight.shape
    weight, scale = weight.contiguous(), scale.float().contiguous()
    out = torch.empty(width, depth, dtype=dtype, device=device)
    with _Device(device):
        _lib.check(_lib.load().b200q_int8_dequantize(
            weight.data_ptr(), scale.data_ptr(), out.data_ptr(), width, depth, group,
            _code(dtype, "dequantize8"), _stream(device)))
    return out


# ---- int8 activations (W8A8) ------------------------------------------------------


def _int8_rows(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    rows, depth = x.shape
    device = _on_gpu("int8_rows", x)
    if depth % 8:
        raise ValueError(f"int8_rows: rows of {depth} inputs are not a multiple of 8")
    x = x.contiguous()
    q = torch.empty(rows, depth, dtype=torch.int8, device=device)
    scale = torch.empty(rows, 1, dtype=torch.float32, device=device)
    with _Device(device):
        _lib.check(_lib.load().b200q_int8_rows(x.data_ptr(), q.data_ptr(), scale.data_ptr(), rows, depth,
                                               _code(x.dtype, "int8_rows"), _stream(device)))
    return q, scale


@torch.library.custom_op("linnet::rows8", mutates_args=(), device_types="cuda")
def _rows8_op(x: torch.Tensor, fp8: bool) -> tuple[torch.Tensor, torch.Tensor]:
    _no_fp8("rows8", fp8)
    return _int8_rows(x)


@_rows8_op.register_fake
def _(x, fp8):
    return x.new_empty(x.shape, dtype=torch.int8), x.new_empty(x.shape[0], 1, dtype=torch.float32)


def int8_rows(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Each row of `x` [rows, In] rounded to int8 with a scale of its own (its largest magnitude
    over 127; levels rounded half away from zero): the rounded rows and the scales ([rows, 1],
    f32), as `int8_mm` takes them (the reference's `int8_rows`, kernels.py:705-753)."""
    if torch.compiler.is_compiling():
        return _rows8_op(x, False)
    return _int8_rows(x)


def int8_mm_available(weight: torch.Tensor) -> bool:
    """Whether `int8_mm` takes this weight: inputs a multiple of 128 (the reference asks the
    same, kernels.py:866-868, and outputs a multiple of 16, quantized.py:85-87)."""
    return weight.is_cuda and weight.shape[1] % 128 == 0 and weight.shape[0] % 16 == 0


def _int8_mm(x: torch.Tensor, weight: torch.Tensor, x_scale: torch.Tensor, scale: torch.Tensor,
             dtype: torch.dtype) -> torch.Tensor:
    rows, depth = x.shape
    width = weight.shape[0]
    if x.dtype != torch.int8 or weight.dtype != torch.int8:
        raise ValueError("int8_mm: int8 rows and int8 weights expected")
    if weight.shape[1] != depth or depth % 128:
        raise ValueError(f"int8_mm: {depth} inputs (a multiple of 128) against a weight of {weight.shape[1]}")
    device = _on_gpu("int8_mm", x, weight, x_scale, scale)
    x, weight = x.contiguous(), weight.contiguous()
    x_scale, scale = x_scale.float().reshape(-1).contiguous(), scale.float().reshape(-1).contiguous()
    if x_scale.numel() != rows or scale.numel() != width:
        raise ValueError("int8_mm: one scale a row of x and one a row of the weight")
    y = torch.empty(rows, width, dtype=dtype, device=device)
    with _Device(device):
        _lib.check(_lib.load().b200q_int8_mm(x.data_ptr(), weight.data_ptr(), x_scale.data_ptr(), scale.data_ptr(),
                                             y.data_ptr(), rows, depth, width, _code(dtype, "int8_mm"),
                                             _stream(device)))
    return y


@torch.library.custom_op("linnet::int8_mm", mutates_args=(), device_types="cuda")
def _int8_mm_op(x: torch.Tensor, weight: torch.Tensor, x_scale: torch.Tensor, scale: torch.Tensor,
                dtype: torch.dtype) -> torch.Tensor:
    return _int8_mm(x, weight, x_scale, scale, dtype)


@_int8_mm_op.register_fake
def _(x, weight, x_scale, scale, dtype):
    return x.new_empty(x.shape[0], weight.shape[0], dtype=dtype)


def int8_mm(x: torch.Tensor, weight: torch.Tensor, x_scale: torch.Tensor, scale: torch.Tensor,
            dtype: torch.dtype) -> torch.Tensor:
    """`(x @ weight.T) * x_scale * scale` in `dtype`, for int8 rows `x` [rows, In] with their
    scales ([rows, 1] f32, from `int8_rows`) and int8 weights [Out, In] with one scale a row
    ([Out]); the sum is exact in int32 on the tensor cores (kernels.py:856-915)."""
    if torch.compiler.is_compiling():
        return _int8_mm_op(x, weight, x_scale, scale, dtype)
    return _int8_mm(x, weight, x_scale, scale, dtype)


def _outside(name: str):
    def missing(*args: object, **kwargs: object):
        raise NotImplementedError(f"linnet.torch.kernels.{name} is outside this build "
                                  "(int4 / int8 layers)")
    missing.__name__ = name
    return missing


# Names the reference's `quantized.py` looks up on this module for the FP8 formats, which
# are not part of this build.
fp8_rows = _outside("fp8_rows")
fp8_groups = _outside("fp8_groups")
