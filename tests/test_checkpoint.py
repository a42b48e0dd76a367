"""`linnet_b200.checkpoint`: SafeTensors in, quantized SafeTensors out, byte for byte the file
the reference's `linnet.quant.quantize_checkpoint` / `import_quantized` writes
(python/linnet/src/linnet/quant.py:139-221, :259-354; tests mirrored:
python/linnet/tests/test_quant_groups.py:59-79 and :224-289, tests/test_quant_8bit.py:235-271).

`tests/golden/checkpoints/` holds small input checkpoints and the reference's own output files
(made by tests/golden/make_golden.py).  The GPTQ / AWQ repack is pure unpacking and indexing, so
it also runs on CPU tensors and is checked without a GPU; quantizing needs the CUDA quantizer.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import pytest
import torch

import checkpoint_cases as cc

GOLDEN = Path(__file__).resolve().parent / "golden" / "checkpoints"
CASES = json.loads((GOLDEN / "cases.json").read_text())


def test_writer_layout_round_trip(tmp_path):
    """Header: 8-byte length, compact JSON padded with spaces to 8 bytes, metadata first."""
    from linnet_b200 import checkpoint

    tensors = [("b.weight", "U8", (2, 3), bytes(range(6))), ("a", "F32", (1,), struct.pack("<f", 1.5))]
    path = checkpoint.write_safetensors(tmp_path / "t.safetensors", tensors, metadata={"format": "pt"})
    blob = path.read_bytes()
    (size,) = struct.unpack("<Q", blob[:8])
    assert size % 8 == 0
    header = json.loads(blob[8:8 + size])
    assert list(header) == ["__metadata__", "b.weight", "a"]
    assert header["a"]["data_offsets"] == [6, 10]
    back = list(checkpoint.iter_safetensors(path))
    assert [(t.name, t.dtype, t.shape, t.data) for t in back] == tensors


def test_argument_errors():
    from linnet_b200 import checkpoint

    with pytest.raises(checkpoint.LinnetError, match="4 or 8 bits"):
        checkpoint.quantize_checkpoint(GOLDEN / "float.safetensors", "/dev/null", patterns=["*"], bits=3)
    with pytest.raises(checkpoint.LinnetError, match="bf16, f16, or f32"):
        checkpoint.quantize_checkpoint(GOLDEN / "float.safetensors", "/dev/null", patterns=["*"], dtype="f64")
    with pytest.raises(checkpoint.LinnetError, match="not GPTQ or AWQ"):
        checkpoint.import_quantized(GOLDEN / "gptq.safetensors", "/dev/null", config={"quant_method": "hqq"},
                                    device="cpu")


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["kind"] == "import"])
def test_import_quantized_matches_the_reference_file(name, tmp_path):
    """GPTQ (with and without activation order) and AWQ repacked: the reference's bytes."""
    from linnet_b200 import checkpoint

    case = CASES[name]
    device = "cuda" if torch.cuda.is_available() else "cpu"
    paths = cc.convert(checkpoint, case, GOLDEN, tmp_path / "out.safetensors", device=device)
    assert paths == case["quantized"]
    assert (tmp_path / "out.safetensors").read_bytes() == (GOLDEN / f"{name}.expected.safetensors").read_bytes()
    names = [t.name for t in checkpoint.iter_safetensors(tmp_path / "out.safetensors")]
    assert ("layer.order" in names) == (name == "gptq_act_order")


@pytest.mark.gpu
@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["kind"] == "quantize"])
def test_quantize_checkpoint_matches_the_reference_file(name, tmp_path):
    """int4 (bf16 scales g128, f32 scales g64) and int8 (bf16 g128, f16 g256) with bindings,
    a tied tensor, bf16 / f16 / f32 inputs and tensors passed through untouched."""
    from linnet_b200 import checkpoint

    case = CASES[name]
    paths = cc.convert(checkpoint, case, GOLDEN, tmp_path / "out.safetensors")
    assert paths == case["quantized"]
    assert (tmp_path / "out.safetensors").read_bytes() == (GOLDEN / f"{name}.expected.safetensors").read_bytes()


@pytest.mark.gpu
def test_quantized_checkpoint_loads_into_the_linear(tmp_path):
    """What `quantize_checkpoint` wrote is what `int4_linear` takes."""
    from safetensors.torch import load_file

    from linnet_b200 import checkpoint, kernels
    from oracle import linear_oracle as lo

    cc.convert(checkpoint, CASES["int4_bf16"], GOLDEN, tmp_path / "q.safetensors")
    t = load_file(str(tmp_path / "q.safetensors"))
    x = torch.randn(3, 256, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    got = kernels.int4_linear(x.cuda(), t["proj.weight"].cuda(), t["proj.scale"].cuda(), t["proj.zero"].cuda())
    want = lo.int4_groups_linear(x, t["proj.weight"], t["proj.scale"], t["proj.zero"])
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=1e-2, atol=1e-2)
