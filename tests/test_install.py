"""`install()` re-points the reference's loader at this package.  Needs the reference
checkout and its compiler, which exist only in the build container: skipped elsewhere."""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import pytest

REF = Path(os.environ.get("LINNET_REF", "/root/reference"))
BIN = Path(os.environ.get("LINNET_BIN", "/tmp/linnet-build/linnet"))
ROOT = Path(__file__).resolve().parents[1]

SCRIPT = r'''
import sys, tempfile, pathlib
sys.path.insert(0, r"{root}")
sys.path.insert(0, r"{ref}/python/linnet/src")
import torch
from linnet_b200 import install
install.install()
import linnet.torch as lt
from linnet.torch import quantized, native
import linnet_b200.quantized as ours_q, linnet_b200.kernels as ours_k
assert sys.modules["linnet.torch.kernels"].int4_linear is ours_k.int4_linear
assert quantized.int8_linear is ours_q.int8_linear and quantized.kernels.gemv8 is ours_k.gemv8
assert torch.ops.linnet.int4_linear is not None
from safetensors.torch import save_file
SOURCE = """module tests.q4
use std.quant::{{Int4GroupLinear}}
pub block Model<In: Dim, Out: Dim, Group: Dim, T: Float = f32>
where Group > 0, Group % 2 == 0, In % Group == 0
{{
    sub proj: Int4GroupLinear<In, Out, Group, T>
    pub entry forward<B: Dim>(x: Tensor[B, In; T]) -> Tensor[B, Out; T] {{
        return proj.forward(x)
    }}
}}
"""
tmp = pathlib.Path(tempfile.mkdtemp())
(tmp / "q4.linnet").write_text(SOURCE)
save_file({{"proj.weight": torch.zeros(64, 2, 64, dtype=torch.uint8),
           "proj.scale": torch.ones(64, 2, dtype=torch.bfloat16),
           "proj.zero": torch.zeros(64, 2, dtype=torch.uint8)}}, str(tmp / "w.safetensors"))
for mode in (True, False):
    model = lt.load(tmp / "q4.linnet", generics={{"In": 256, "Out": 64, "Group": 128, "T": "bf16"}},
                    std_root=r"{ref}/stdlib", weights=tmp / "w.safetensors", compile=mode)
    try:
        model.run_entry("forward", [torch.zeros(3, 256, dtype=torch.bfloat16)])
    except RuntimeError as error:
        # CPU tensors reached this package's `_int4_pack`, which has no CPU path: the
        # generated source (compile=True) and the interpreter (compile=False) both dispatch here.
        assert "this build has no CPU" in str(error), error
    else:
        raise SystemExit("the reference's own CPU path ran: not dispatched")
print("dispatched")
'''


@pytest.mark.skipif(not (REF / "python/linnet/src/linnet").exists() or not BIN.exists(),
                    reason="needs the reference checkout and its compiler")
def test_load_dispatches_to_this_package(tmp_path):
    env = dict(os.environ, LINNET_BIN=str(BIN), LINNET_HOME=str(tmp_path / "home"))
    done = subprocess.run([sys.executable, "-c", SCRIPT.format(root=ROOT, ref=REF)], env=env,
                          capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-3000:]
    assert "dispatched" in done.stdout
