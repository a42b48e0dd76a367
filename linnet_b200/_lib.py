"""ctypes binding of `libb200q.so`, the C-ABI library of sm_100a kernels
(`include/b200q.h`).  There is no CPU or PyTorch fallback: if the library is missing
or a call fails, this raises."""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int32, c_int64, c_void_p
from pathlib import Path

LIBRARY = Path(__file__).resolve().parent / "libb200q.so"

OK, ERROR, UNAVAILABLE = 0, 1, 2
F32, BF16, F16 = 0, 1, 2
EXACT_WEIGHTS, EARLY_DEPENDENTS, SWIGLU_INPUT, NO_OVERLAP = 1, 2, 4, 8

# name -> argument types, exactly the prototypes of include/b200q.h
PROTOTYPES: dict[str, list] = {
    "b200q_abi_version": [],
    "b200q_device_ok": [],
    "b200q_quantize_int4_groups": [c_void_p, c_int32, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                   c_void_p, c_int32, c_void_p, c_void_p],
    "b200q_quantize_int8_groups": [c_void_p, c_int32, c_int64, c_int64, c_int64, c_int32, c_void_p,
                                   c_void_p, c_void_p],
    "b200q_int4_linear": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                          c_int64, c_int32, c_void_p],
    "b200q_int4_gemv": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                        c_int64, c_int32, c_void_p],
    "b200q_int4_gemv_ex": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                           c_int64, c_int32, c_int32, c_void_p],
    "b200q_int4_linear_ex": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                             c_int64, c_int32, c_int32, c_void_p],
    "b200q_int4_gemm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                        c_int64, c_int32, c_void_p],
    "b200q_int4_gemm_status": [],
    "b200q_int4_dequantize": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                              c_int32, c_void_p],
    "b200q_int4_gemv_norm": [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int64, c_int64, c_int64, c_int64, c_int32, c_int32, c_void_p],
    "b200q_int8_linear": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                          c_int32, c_void_p],
    "b200q_int8_linear_ex": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                          c_int32, c_int32, c_void_p],
    "b200q_int8_rows": [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p],
    "b200q_int8_mm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32,
                      c_void_p],
    "b200q_int8_dequantize": [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32,
                              c_void_p],
    "b200q_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_void_p],
    "b200q_rope_cache": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                         c_int64, c_int64, c_float, c_void_p],
    "b200q_decode_attention_scratch_bytes": [c_int64, c_int64, c_int64, c_int64],
    "b200q_decode_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                               c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p],
    "b200q_decode_attention_cluster": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                       c_int64, c_int64, c_int64, c_int64, c_void_p],
    "b200q_rope_table": [c_void_p, c_int64, c_int64, c_float, c_void_p],
    "b200q_rope_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                             c_int64, c_int64, c_int64, c_int64, c_void_p],
    "b200q_decode_attention_static_scratch_limit": [],
    "b200q_decode_attention_static": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                      c_int64, c_int64, c_int64, c_int64, c_void_p],
    "b200q_decoder_status": [],
    "b200q_set_wait_limit_ns": [c_int64],
    "b200q_silu_mul": [c_void_p, c_void_p, c_int64, c_int64, c_void_p],
    "b200q_tp_allreduce_add_rmsnorm_flags": [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                             c_float, c_void_p],
    "b200q_tp_allreduce": [c_void_p, c_int64, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_int64, c_int32, c_void_p],
    "b200q_tp_allreduce_add_rmsnorm": [c_void_p, c_int64, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_void_p],
}


class B200QError(RuntimeError):
    """A b200q call returned B200Q_ERROR or B200Q_UNAVAILABLE."""


_lib: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built (`python -m linnet_b200._build`)."""
    global _lib
    if _lib is None:
        if not LIBRARY.exists():
            raise B200QError(
                f"{LIBRARY} is missing: build it with `python -m linnet_b200._build` "
                "(there is no fallback implementation)")
        lib = ctypes.CDLL(str(LIBRARY))
        for name, argtypes in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int64 if name.endswith(("_bytes", "_limit")) else c_int32
        lib.b200q_last_error.argtypes = []
        lib.b200q_last_error.restype = c_char_p
        if lib.b200q_abi_version() != 1:
            raise B200QError("libb200q.so has another ABI version; rebuild it")
        _lib = lib
    return _lib


def last_error() -> str:
    return load().b200q_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Raises for a non-zero status: ValueError for rejected arguments (as the
    reference's operators do), B200QError when the device cannot run the kernels."""
    if status == OK:
        return
    message = last_error()
    if status == UNAVAILABLE:
        raise B200QError(message)
    raise ValueError(message)
