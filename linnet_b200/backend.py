"""The B200 kernels as a Linnet backend, a plug-in under the reference's `linnet.backends`
contract (docs/backends.md; python/linnet/src/linnet/backends/contract.py:278-323; the template
this follows in use is examples/09-backends/marlin/linnet_marlin/__init__.py).

It takes the quantized `linear` calls of `stdlib/quant.linnet`:

    std.quant::linear_int4_groups(x, q, scale, zero, bias)     stdlib/quant.linnet:132-141
    std.quant::linear_int8(x, weight, scale, bias)             stdlib/quant.linnet:36-43
    std.quant::linear_int8_groups(x, weight, scale, bias)      stdlib/quant.linnet:72-79

and runs them with `linnet_b200.kernels` (`int4_linear`, `gemv8` / `w8a16`).  The kernels read
the checkpoint layout as the loader holds it, so nothing is repacked and nothing is kept
beside the model's weights except an f32 copy of an int8 layer's scales (the kernels take f32).

    import linnet.torch
    from linnet_b200.backend import B200Quant
    model = linnet.torch.load(card, weights=..., device="cuda", compile=True)
    plan = model.plan_for("decode", [token, pos], backends=[B200Quant()])

A package that ships this names it in its `linnet.backends` entry-point group:
`b200-quant = "linnet_b200.backend:B200Quant"`.

The `linnet.backends` types are imported when the class is used, not when this module is: the
product does not depend on the reference being installed.
"""

from __future__ import annotations

from collections.abc import Iterable, Sequence

import torch

INT4 = "std.quant::linear_int4_groups"
INT8 = "std.quant::linear_int8"
INT8_GROUPS = "std.quant::linear_int8_groups"
_DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16}
VERSION = "2"


def _contract():
    import linnet.backends as contract

    return contract


class B200Quant:
    """Takes the int4-group and int8 weight-only `linear` calls on a B200."""

    contract = 1  # the version of `linnet.backends` this was written for

    def __init__(self, any_device: bool = False) -> None:
        # `any_device`: for tests that stand an oracle in for the kernels on a CPU
        self._any_device = any_device

    @property
    def name(self) -> str:
        return "b200-quant"

    @property
    def version(self) -> str:
        return VERSION

    def probe(self, target):
        on_b200 = target.kind == "cuda" and tuple(target.capability)[:1] == (10,)
        if not (on_b200 or self._any_device):
            return None
        return _contract().Capabilities({"libb200q": VERSION}, frozenset(_DTYPES))

    def match(self, graph, target) -> Iterable:
        contract = _contract()
        persistent = set(graph.parameters.values())
        for callee, count in ((INT4, 5), (INT8, 4), (INT8_GROUPS, 4)):
            for call in graph.semantic_calls(callee):
                if len(call.arguments) != count:
                    continue
                x, weight = call.arguments[0], call.arguments[1]
                rest = call.arguments[2:-1]
                bias = call.arguments[-1]
                region = contract.Region.of(graph, call.start, call.stop, call.index)
                if x.dtype not in _DTYPES or weight.value not in persistent:
                    continue
                if bias.value is not None and bias.value not in persistent and bias.value not in region.inputs:
                    continue
                # every other operand is a weight of the model or something an earlier step made
                if any(v.value not in persistent and v.value not in region.inputs for v in rest):
                    continue
                if callee == INT4:
                    _out, groups, group = weight.shape
                    if rest[0].dtype != x.dtype or not (group in (16, 32, 64) or group % 128 == 0):
                        continue
                    if (groups * group) % 8 != 0:
                        continue
                if region.inputs[:1] != (x.value,):
                    continue
                yield region

    def compile(self, region, target, options):
        from linnet.compiler import PlanError

        if region.call is None:
            raise PlanError("b200-quant takes a quantized `linear` call")
        call = region.graph.calls[region.call]
        return _QuantLinear(region, call)

    def estimate_cost(self, region, target):
        return None


class _QuantLinear:
    """One quantized `linear` call.  Operands that are weights of the model are read from
    `context.parameters` by path at every call (a captured plan reads them where they are, and
    `copy_weights` rewrites them in place); operands an earlier step made (an `Int8Linear`'s
    scale, reshaped from `[Out, 1]`) arrive among the inputs."""

    def __init__(self, region, call) -> None:
        contract = _contract()
        graph = region.graph
        path_of = {value: path for path, value in graph.parameters.items()}
        self._callee = call.callee
        self._sources = []  # per operand after x: ("parameter", path) | ("input", position) | None
        for operand in call.arguments[1:]:
            if operand.value is None:
                self._sources.append(None)
            elif operand.value in path_of:
                self._sources.append(("parameter", path_of[operand.value]))
            else:
                self._sources.append(("input", region.inputs.index(operand.value)))
        weight = call.arguments[1]
        self._out = int(weight.shape[0])
        self._scale32: torch.Tensor | None = None  # an int8 layer's scales as the kernels take them
        values = graph.values
        held = 0 if call.callee == INT4 else 4 * int(torch.Size(call.arguments[2].shape).numel())
        self._meta = contract.ExecutableMeta(
            tuple(contract.TensorSpec(values[v].shape, values[v].dtype) for v in region.inputs),
            tuple(contract.TensorSpec(values[v].shape, values[v].dtype) for v in region.outputs),
            holds=held,
        )

    @property
    def meta(self):
        return self._meta

    def _operand(self, index: int, inputs: Sequence[torch.Tensor] | None, context) -> torch.Tensor | None:
        source = self._sources[index]
        if source is None:
            return None
        kind, where = source
        if kind == "parameter":
            return context.parameters[where]
        return None if inputs is None else inputs[where]

    def prepare(self, context) -> None:
        """Weights are used where they are; only an int8 layer's scales are converted (to f32,
        flat), into the same tensor when the weights have changed."""
        if self._callee == INT4:
            return
        scale = self._operand(1, None, context)
        if scale is None:  # made by an earlier step: converted at every call instead
            return
        wanted = scale.float().reshape(self._out, -1).contiguous()
        if self._scale32 is None or self._scale32.shape != wanted.shape:
            self._scale32 = wanted
        else:
            self._scale32.copy_(wanted)

    def execute(self, inputs: Sequence[torch.Tensor], outputs: Sequence[torch.Tensor], context) -> Sequence[torch.Tensor]:
        from . import kernels

        x = inputs[0]
        flat = x.reshape(-1, x.shape[-1])
        if self._callee == INT4:
            packed = self._operand(0, inputs, context)
            scale = self._operand(1, inputs, context)
            zero = self._operand(2, inputs, context)
            bias = self._operand(3, inputs, context)
            y = kernels.int4_linear(flat, packed, scale, zero)
        else:
            weight = self._operand(0, inputs, context)
            bias = self._operand(2, inputs, context)
            if self._sources[1][0] == "parameter":
                if self._scale32 is None:
                    self.prepare(context)
                scale = self._scale32
            else:
                scale = self._operand(1, inputs, context).float().reshape(self._out, -1)
            if self._callee == INT8:
                group, scale = 0, scale.reshape(-1)
            else:
                group = flat.shape[-1] // scale.shape[1]
            product = kernels.gemv8 if flat.shape[0] == 1 else kernels.w8a16
            y = product(flat, weight, scale, False, group, 1)
        if bias is not None:
            y = y + bias
        return [y.reshape(*x.shape[:-1], self._out)]


__all__ = ["B200Quant"]
