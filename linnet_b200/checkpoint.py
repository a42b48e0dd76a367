"""Quantizing a SafeTensors checkpoint on the GPU, file in, file out: the reference's
`linnet.quant.quantize_checkpoint` (python/linnet/src/linnet/quant.py:139-221) with the
rounding done by this package's CUDA quantizer instead of NumPy.

The output file is the reference's, byte for byte: the same tensor names (`<prefix>weight`,
`<prefix>scale`, `<prefix>zero`), SafeTensors dtypes (`U8` packed nibbles `[Out, In/G, G/2]` and
zero points, `I8` levels, scales `BF16` / `F16` / `F32`), tensor order, `{"format": "pt"}`
metadata and header padding (`write_safetensors`, python/linnet/src/linnet/weights.py:325-373),
because the quantizer is bit-exact and the writer lays the file out the same way.

SafeTensors here is read and written directly (an 8-byte length, a JSON header, raw tensor
bytes), one tensor at a time, so a checkpoint larger than host memory streams through.
"""

from __future__ import annotations

import fnmatch
import json
import struct
from collections.abc import Iterable, Iterator, Mapping
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from . import quant
from .quant import LinnetError

_FLOATS = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64}
_STORED = {"bf16": "BF16", "f16": "F16", "f32": "F32"}


@dataclass(frozen=True)
class RawTensor:
    """One tensor of a SafeTensors file as bytes (weights.py:232-238)."""

    name: str
    dtype: str
    shape: tuple[int, ...]
    data: bytes


def safetensors_files(weights: str | Path) -> list[Path]:
    """A file, or every `*.safetensors` of a directory in name order."""
    location = Path(weights)
    if location.is_dir():
        files = sorted(location.glob("*.safetensors"))
        if not files:
            raise LinnetError(f"no .safetensors file in {location}")
        return files
    return [location]


def iter_safetensors(weights: str | Path) -> Iterator[RawTensor]:
    """Every tensor of a checkpoint in header order, read one at a time."""
    for file in safetensors_files(weights):
        with file.open("rb") as handle:
            (size,) = struct.unpack("<Q", handle.read(8))
            header = json.loads(handle.read(size).decode("utf-8"))
            base = 8 + size
            for name, info in header.items():
                if name == "__metadata__":
                    continue
                start, end = (int(o) for o in info["data_offsets"])
                handle.seek(base + start)
                yield RawTensor(str(name), str(info["dtype"]), tuple(int(d) for d in info["shape"]),
                                handle.read(end - start))


def write_safetensors(path: str | Path, tensors: Iterable[tuple[str, str, tuple[int, ...], bytes]],
                      metadata: Mapping[str, str] | None = None) -> Path:
    """`(name, dtype, shape, bytes)` tensors as one SafeTensors file, laid out as the
    reference's writer lays it out (weights.py:337-373): compact JSON, metadata first, the
    header padded with spaces to a multiple of 8 bytes, tensors in the order given."""
    entries = list(tensors)
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    for name, dtype, shape, data in entries:
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [offset, offset + len(data)]}
        offset += len(data)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * (-len(encoded) % 8)
    target = Path(path)
    target.parent.mkdir(parents=True, exist_ok=True)
    with target.open("wb") as out:
        out.write(struct.pack("<Q", len(encoded)))
        out.write(encoded)
        for _, _, _, data in entries:
            out.write(data)
    return target


def read_bindings(bindings: str | Path) -> dict[str, str]:
    """A JSON object mapping Linnet parameter paths to checkpoint tensor names (weights.py:108-113)."""
    loaded = json.loads(Path(bindings).read_text(encoding="utf-8"))
    if not isinstance(loaded, dict):
        raise LinnetError("bindings must be a JSON object mapping parameter paths to tensor names")
    return {str(path): str(name) for path, name in loaded.items()}


def _paths_of(bindings: str | Path | Mapping[str, str] | None) -> dict[str, list[str]]:
    """Checkpoint name -> the Linnet paths bound to it (quant.py:184-194; weights.py:124-130)."""
    mapping = dict(bindings) if isinstance(bindings, Mapping) else read_bindings(bindings) if bindings is not None else {}
    paths: dict[str, list[str]] = {}
    for path, name in mapping.items():
        paths.setdefault(name, []).append(path)
    return paths


def _prefix(path: str) -> str:
    """What names a weight's siblings: `proj.` for `proj.weight` (quant.py:197-202)."""
    if path == "weight":
        return ""
    return path.removesuffix("weight") if path.endswith(".weight") else path + "."


def _device_floats(tensor: RawTensor, device: torch.device) -> torch.Tensor:
    """The tensor on the GPU as f32 or bf16 (bf16 widens exactly inside the kernel; f16 and
    f64 become f32 first, as the reference's `decode_floats` makes them, weights.py:87-95)."""
    if tensor.dtype not in _FLOATS:
        raise LinnetError(f"{tensor.dtype} is not a floating-point dtype")
    if len(tensor.shape) != 2:
        raise LinnetError(f"a linear weight is [Out, In]; `{tensor.name}` is {list(tensor.shape)}")
    host = torch.frombuffer(bytearray(tensor.data), dtype=_FLOATS[tensor.dtype]).reshape(tensor.shape)
    moved = host.to(device, non_blocking=False)
    return moved if moved.dtype in (torch.float32, torch.bfloat16) else moved.float()


def _bytes(t: torch.Tensor) -> bytes:
    return t.contiguous().cpu().view(torch.uint8).numpy().tobytes()


def quantize_tensor(values: torch.Tensor, group: int, dtype: str, bits: int,
                    prefix: str) -> list[tuple[str, str, tuple[int, ...], bytes]]:
    """One weight's output tensors, named and typed as the checkpoint holds them
    (`_int4_tensors`, `_scale_tensor`: quant.py:205-221; the int8 pair: quant.py:166-171)."""
    if bits == 8:
        q, scale = quant.quantize_int8_groups(values, group, dtype)
        stored = scale.to({"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype])
        return [(prefix + "weight", "I8", tuple(q.shape), _bytes(q)),
                (prefix + "scale", _STORED[dtype], tuple(scale.shape), _bytes(stored))]
    packed, _scale, zero, stored = quant.quantize_int4_groups(values, group, scale_dtype=dtype)
    return [(prefix + "weight", "U8", tuple(packed.shape), _bytes(packed)),
            (prefix + "scale", _STORED[dtype], tuple(stored.shape), _bytes(stored)),
            (prefix + "zero", "U8", tuple(zero.shape), _bytes(zero))]


def quantize_checkpoint(weights: str | Path, output: str | Path, *, patterns: Iterable[str], group: int = 128,
                        dtype: str = "bf16", bindings: str | Path | Mapping[str, str] | None = None,
                        bits: int = 4, device: torch.device | str | None = None) -> list[str]:
    """Writes `output` with every tensor of `weights` under its Linnet path (`bindings` maps
    paths to checkpoint names, as for loading), quantizing the `.weight` tensors whose path
    matches one of `patterns`: into `.weight`, `.scale` and `.zero` for `Int4GroupLinear`
    (`bits` 4), or `.weight` and `.scale` for `Int8GroupLinear` (`bits` 8).  Returns the
    quantized paths.  Same arguments, errors and output bytes as the reference's function
    (quant.py:139-181); `device` picks the GPU (default: the current one)."""
    if bits not in (4, 8):
        raise LinnetError(f"weights are quantized to 4 or 8 bits, not {bits}")
    if dtype not in _STORED:
        raise LinnetError(f"scales are stored as bf16, f16, or f32, not {dtype}")
    where = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    paths_of = _paths_of(bindings)
    chosen = list(patterns)
    out: list[tuple[str, str, tuple[int, ...], bytes]] = []
    quantized: list[str] = []
    with torch.cuda.device(where):
        for tensor in iter_safetensors(weights):
            for path in paths_of.get(tensor.name, [tensor.name]):
                if path.endswith(".weight") and any(fnmatch.fnmatchcase(path, p) for p in chosen):
                    out += quantize_tensor(_device_floats(tensor, where), group, dtype, bits, _prefix(path))
                    quantized.append(path)
                else:
                    out.append((path, tensor.dtype, tensor.shape, tensor.data))
    if not quantized:
        raise LinnetError("no weight matched " + ", ".join(chosen))
    write_safetensors(output, out, metadata={"format": "pt"})
    return quantized


# ---- GPTQ / AWQ checkpoints repacked for Int4GroupLinear --------------------------------------

# AWQ packs eight outputs to an int32 interleaved: bits 4k hold output _AWQ_ORDER[k] of the
# eight (quant.py:224-227).
_AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)
_AWQ_REVERSE = tuple(_AWQ_ORDER.index(k) for k in range(8))


def _nibbles(words: torch.Tensor, axis: int) -> torch.Tensor:
    """The eight 4-bit values of each int32, lowest bits first, laid along `axis`
    (quant.py:230-239), on the device `words` lives on."""
    shifts = torch.arange(0, 32, 4, device=words.device, dtype=torch.int32)
    values = (words.unsqueeze(-1) >> shifts) & 15  # arithmetic shift, then the mask: bits as stored
    values = torch.movedim(values, -1, axis + 1)
    shape = list(words.shape)
    shape[axis] *= 8
    return values.reshape(shape).to(torch.uint8)


def _setting(config: Mapping[str, object], key: str, alias: str, default: int) -> int:
    value = config.get(key, config.get(alias, default))
    try:
        return int(value)  # type: ignore[arg-type]
    except (TypeError, ValueError):
        raise LinnetError(f"the quantization_config's `{key}` is {value!r}, not a number") from None


def import_quantized(weights: str | Path, output: str | Path, *,
                     bindings: str | Path | Mapping[str, str] | None = None, dtype: str = "bf16",
                     config: Mapping[str, object] | None = None,
                     device: torch.device | str | None = None) -> list[str]:
    """Writes `output` with a 4-bit GPTQ or AWQ checkpoint's quantized linear layers repacked
    for `Int4GroupLinear` (`.weight`, `.scale` in `dtype`, `.zero`, and `.order` when a GPTQ
    layer's groups follow activation order) and every other tensor as it is: the reference's
    `import_quantized` for those two methods (quant.py:259-354), the unpacking and repacking
    done on the GPU.  Output bytes are the reference's."""
    if dtype not in _STORED:
        raise LinnetError(f"scales are stored as bf16, f16, or f32, not {dtype}")
    if config is None:
        location = Path(weights)
        directory = location if location.is_dir() else location.parent
        try:
            document = json.loads((directory / "config.json").read_text(encoding="utf-8"))
        except FileNotFoundError:
            raise LinnetError(f"no config.json beside {weights}; pass `config`") from None
        config = document.get("quantization_config")
        if not isinstance(config, Mapping):
            raise LinnetError(f"{directory / 'config.json'} has no quantization_config")
    method = str(config.get("quant_method", "")).lower()
    if method not in ("gptq", "awq"):
        raise LinnetError(f"a {method or 'unnamed'} checkpoint is not GPTQ or AWQ (the only ones this build repacks)")
    if _setting(config, "bits", "w_bit", 4) != 4:
        raise LinnetError("only 4-bit GPTQ and AWQ checkpoints repack into Int4GroupLinear")
    if method == "awq" and str(config.get("version", "gemm")).lower() != "gemm":
        raise LinnetError(f"AWQ's {config.get('version')} packing is not read; GEMM's is")
    group = _setting(config, "group_size", "q_group_size", 128)
    zero_offset = 1 if method == "gptq" and config.get("checkpoint_format", "gptq") == "gptq" else 0
    where = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    tensors = {tensor.name: tensor for tensor in iter_safetensors(weights)}
    paths_of = _paths_of(bindings)
    out: list[tuple[str, str, tuple[int, ...], bytes]] = []
    quantized: list[str] = []
    parts = (".qweight", ".qzeros", ".scales", ".g_idx")
    layers = sorted(name.removesuffix(".qweight") for name in tensors if name.endswith(".qweight"))
    taken = {layer + part for layer in layers for part in parts}

    def int32(tensor: RawTensor) -> torch.Tensor:
        return torch.frombuffer(bytearray(tensor.data), dtype=torch.int32).reshape(tensor.shape).to(where)

    for layer in layers:
        stored = tensors[layer + ".scales"]
        if stored.dtype not in _FLOATS:
            raise LinnetError(f"{stored.dtype} is not a floating-point dtype")
        scales = torch.frombuffer(bytearray(stored.data), dtype=_FLOATS[stored.dtype]).reshape(stored.shape).to(where).float()
        words, zero_words = int32(tensors[layer + ".qweight"]), int32(tensors[layer + ".qzeros"])
        order = None
        if method == "gptq":
            q = _nibbles(words, 0)  # [In, Out]
            zero = _nibbles(zero_words, 1).to(torch.int32) + zero_offset  # [Groups, Out]
            in_features = q.shape[0]
            group_of = torch.arange(in_features, device=where, dtype=torch.int32) // (in_features if group <= 0 else group)
            if layer + ".g_idx" in tensors:
                ids = int32(tensors[layer + ".g_idx"])
                if not torch.equal(ids, group_of):
                    # Activation order: taken in the order that sorts the group ids (stably),
                    # each group's inputs are contiguous.
                    order = torch.argsort(ids, stable=True).to(torch.int32)
                    if not torch.equal(ids[order.long()], group_of):
                        raise LinnetError(f"{layer}: its groups are not all the same size")
                    q = q[order.long()]
        else:
            columns = torch.arange(words.shape[1] * 8, device=where).reshape(-1, 8)[:, list(_AWQ_REVERSE)].reshape(-1)
            q = _nibbles(words, 1)[:, columns]  # [In, Out]
            zero = _nibbles(zero_words, 1)[:, columns].to(torch.int32)
        in_features, out_features = q.shape
        size = in_features if group <= 0 else group
        if in_features % size != 0 or tuple(zero.shape) != (in_features // size, out_features):
            raise LinnetError(f"{layer}: {in_features} inputs do not make groups of {size}")
        if zero.numel() and int(zero.max().item()) > 255:
            raise LinnetError(f"{layer}: a zero point past 255")
        packed = quant.pack_int4_groups(q.T.contiguous(), size)
        scale_t = scales.T.contiguous()
        stored_scale = scale_t.to({"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype])
        zero_t = zero.T.contiguous().to(torch.uint8)
        weight_name = layer + ".weight"
        for path in paths_of.get(weight_name, [weight_name]):
            prefix = _prefix(path)
            out += [(prefix + "weight", "U8", tuple(packed.shape), _bytes(packed)),
                    (prefix + "scale", _STORED[dtype], tuple(stored_scale.shape), _bytes(stored_scale)),
                    (prefix + "zero", "U8", tuple(zero_t.shape), _bytes(zero_t))]
            if order is not None:
                out.append((prefix + "order", "I32", (in_features,), _bytes(order)))
            quantized.append(path)
    if not quantized:
        raise LinnetError(f"no {method.upper()} layer (`.qweight`) in {weights}")
    # every other tensor as it is, under its Linnet paths (quant.py `_write_with_the_rest`)
    for name, tensor in tensors.items():
        if name in taken:
            continue
        for path in paths_of.get(name, [name]):
            out.append((path, tensor.dtype, tensor.shape, tensor.data))
    write_safetensors(output, out, metadata={"format": "pt"})
    return quantized


def numpy_bytes(array: np.ndarray) -> bytes:
    return np.ascontiguousarray(array).tobytes()
