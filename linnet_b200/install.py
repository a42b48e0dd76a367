"""Makes a process that uses the reference's `linnet.torch.load` dispatch its int4 / int8
quantized linear layers to the sm_100a kernels of this package, without editing the
reference.

    import linnet_b200.install; linnet_b200.install.install()
    import linnet.torch
    model = linnet.torch.load("model.linnet", weights=..., device="cuda", compile="cudagraphs")

What it replaces (all of it is looked up by name at run time in the reference):

1. `linnet.torch.kernels` -- the Triton module the generated source and
   `linnet.torch.quantized` import (`int4_linear`, `gemv8`, `w8a16`, `dequantize8`, ...;
   python/linnet/src/linnet/torch/kernels.py).  A stand-in module with the same names is
   put into `sys.modules` BEFORE the reference's is imported, so `linnet::int4_linear`,
   `linnet::gemv8` and `linnet::w8a16` are registered once, by this package.  (Two
   registrations of one op name raise, so call `install()` first in the process.)
2. `linnet.torch.quantized.int8_operands / int8_linear / int8_group_operands /
   int8_group_linear` (python/linnet/src/linnet/torch/quantized.py:176-218), which the
   generated source and the interpreter table `NATIVE` call.
3. `NATIVE["torch.ops.aten._weight_int4pack_mm"]`, the interpreter's int4 entry
   (python/linnet/src/linnet/torch/native.py:417-424, :557).
4. `linnet.torch.collectives.OneShot`, the small-message all-reduce behind
   `std.nn.parallel::all_reduce` (python/linnet/src/linnet/torch/collectives.py:56-167): the
   class `collectives.prepare` builds per group becomes `linnet_b200.tp.OneShot`, whose sums
   run `b200q_tp_allreduce` over peer memory with bounded waits.
5. The `_int4_pack`, `_int4_weight`, `_int4_linear` helpers that every generated module
   defines for itself (text at src/backend/torch_source.cpp:1482-1570): they are
   overwritten in each module right after `CompiledLinnetModule.import_source` imports it
   (python/linnet/src/linnet/torch/compiled.py:1035-1038).
"""

from __future__ import annotations

import sys
import types

_installed = False


def _stand_in() -> types.ModuleType:
    from . import kernels as ours

    module = types.ModuleType("linnet.torch.kernels")
    module.__doc__ = "Stand-in for linnet.torch.kernels backed by linnet_b200 (sm_100a CUDA kernels)."
    for name in ("int4_linear", "gemv8", "w8a16", "dequantize8", "int8_rows", "int8_mm", "fp8_rows",
                 "fp8_groups"):
        setattr(module, name, getattr(ours, name))
    # `mxfp4_experts`, the delta-rule kernels and the one-shot all-reduce kernel are absent
    # on purpose: their importers catch ImportError / AttributeError and take the
    # reference's PyTorch or NCCL route (generated source: try/except ImportError;
    # python/linnet/src/linnet/torch/collectives.py:128-131).
    return module


def _patch_generated(module: object) -> None:
    from . import int4

    for name in ("_int4_pack", "_int4_weight", "_int4_linear"):
        if hasattr(module, name):
            setattr(module, name, getattr(int4, name))
    if hasattr(module, "_int4_kernel"):
        from . import kernels

        setattr(module, "_int4_kernel", kernels.int4_linear)


def install() -> None:
    """Idempotent.  Must run before anything imports `linnet.torch.kernels`."""
    global _installed
    if _installed:
        return
    existing = sys.modules.get("linnet.torch.kernels")
    if existing is not None and not getattr(existing, "__doc__", "").startswith("Stand-in"):
        raise RuntimeError("linnet.torch.kernels is already imported: call linnet_b200.install.install() "
                           "before importing linnet.torch (its Triton ops and ours share op names)")
    from . import int4, quantized as ours_q

    sys.modules["linnet.torch.kernels"] = _stand_in()
    import linnet.torch as lt  # the reference; raises ImportError when it is not installed
    import linnet.torch.compiled as compiled
    import linnet.torch.native as native
    import linnet.torch.quantized as ref_q

    lt.kernels = sys.modules["linnet.torch.kernels"]
    ref_q.kernels = sys.modules["linnet.torch.kernels"]
    for name in ("int8_operands", "int8_linear", "int8_group_operands", "int8_group_linear"):
        setattr(ref_q, name, getattr(ours_q, name))

    def int4_native(args):
        x, packed, scale, zero, bias = args
        return int4._int4_linear(x, int4._int4_pack(packed, scale, zero), bias, packed, scale, zero)

    native.NATIVE["torch.ops.aten._weight_int4pack_mm"] = int4_native

    import linnet.torch.collectives as collectives

    from . import tp

    collectives.OneShot = tp.OneShot

    original = compiled.CompiledLinnetModule.import_source

    def import_source(self, source, name):
        module = original(self, source, name)
        _patch_generated(module)
        return module

    compiled.CompiledLinnetModule.import_source = import_source
    _installed = True
