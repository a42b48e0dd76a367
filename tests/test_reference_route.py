"""The reference's own loader, `linnet.torch.load`, with this package installed into it,
against the reference alone: int4 / int8 cards, sibling projections, a weight refresh and a
two-layer Llama card, interpreted, as generated source and (on a GPU) replayed as CUDA graphs.

Both sides run as child processes of `tests/reference_route.py` (they register the same
`linnet::` operator names, so they cannot share a process) out of `oracle/_ref`, the copy of
the reference that `python -m oracle.build_ref` makes; without it the tests are skipped.

* `test_loader_hooks_on_cpu` (no GPU needed): install() + the reference's loader with the CUDA
  kernels replaced by the CPU oracle.  Everything between `linnet.torch.load` and this
  package's entry points is exercised -- generated `prepare` / `main`, the interpreter table,
  the 8-bit operand tuples, joined siblings, `copy_weights` -- and must reproduce the
  reference bit for bit, with every entry point actually called.
* `test_loader_route_on_gpu`: the same with the real kernels on `cuda`, compile modes False,
  True and "cudagraphs".  Tolerance: rtol 1e-2 / atol 1e-2 for the single layers; for the
  Llama card's logits `2e-2 * max|logits|`, because the reference's interpreter and its own
  generated source already differ by `1e-2 * max|logits|` on these inputs (bf16 rotary tables
  and attention).  The same bound pins `linnet_b200.decoder.Int4Decoder` on the same weights.
"""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
SCRIPT = ROOT / "tests" / "reference_route.py"


def _values(array: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(array.copy()).view(torch.bfloat16).float()


@pytest.fixture(scope="session")
def reference_run(tmp_path_factory):
    from oracle import build_ref

    if not build_ref.available():
        try:
            build_ref.build()
        except FileNotFoundError:
            pytest.skip("oracle/_ref is not built and there is no reference checkout to build it from")
    work = tmp_path_factory.mktemp("route")
    env = build_ref.environment(work / "home")
    done = subprocess.run([sys.executable, str(SCRIPT), "reference", str(work / "work")], env=env,
                          capture_output=True, text=True, timeout=1200)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    return work / "work", env, np.load(work / "work" / "reference.npz")


def _run_ours(work: Path, env: dict, *extra: str) -> None:
    done = subprocess.run([sys.executable, str(SCRIPT), "ours", str(work), *extra], env=env, capture_output=True,
                          text=True, timeout=1200)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-6000:]


ENTRY_POINTS = ("_int4_pack", "_int4_linear", "int8_operands", "int8_linear", "int8_group_operands",
                "int8_group_linear")


def test_reference_agrees_with_itself(reference_run):
    """The reference's interpreter and its generated source on the single layers: identical."""
    _, _, ref = reference_run
    for key in ref.files:
        if key.startswith("source/") and "llama4" not in key:
            assert np.array_equal(ref[key], ref["interp/" + key.split("/", 1)[1]]), key


def test_loader_hooks_on_cpu(reference_run):
    work, env, ref = reference_run
    _run_ours(work, env, "--device", "cpu", "--stub")
    ours = np.load(work / "ours_stub.npz")
    for name in ENTRY_POINTS:
        assert int(ours[f"calls/{name}"][0]) > 0, f"{name} was never reached through linnet.torch.load"
    for key in ref.files:
        assert key in ours.files, key
        assert np.array_equal(ours[key], ref[key]), key
    _plans_agree(ours, ref, exact=True)
    # weights replaced in place: the second call computes with the new ones
    assert not np.array_equal(ours["source/refresh/before"], ours["source/refresh/after"])
    assert np.array_equal(ours["source/refresh/after"], ours["source/refresh/other"])
    peak = max(_values(ref[f"source/llama4/logits{s}"]).abs().max().item() for s in range(3))
    for step in range(3):
        got, want = _values(ours[f"decoder/llama4/logits{step}"]), _values(ref[f"source/llama4/logits{step}"])
        assert (got - want).abs().max().item() <= 2e-2 * peak, step


def _plans_agree(ours, ref, exact: bool) -> None:
    """The B2 plug-in (`linnet_b200.backend.B200Quant`) under the reference's planner: every card's
    quantized linears were taken, ran, conform to the generated source, and the plan's outputs
    are the reference's."""
    assert int(ours["plan/executed"][0]) > 0
    peak = max(_values(ref[f"source/llama4/logits{s}"]).abs().max().item() for s in range(3))
    for name in ("lin4/y1", "lin4/y16", "lin8/rows1", "lin8/groups5"):
        assert int(ours[f"plan/{name}/regions"][0]) >= 1, name
        assert bool(ours[f"plan/{name}/conform"].all()), name
        got, want = _values(ours[f"plan/{name}"]), _values(ref[f"source/{name}"])
        if exact:
            assert torch.equal(got, want), name
        else:
            torch.testing.assert_close(got, want, rtol=1e-2, atol=1e-2, msg=lambda m: f"plan/{name}: {m}")
    for step in range(3):
        got, want = _values(ours[f"plan/llama4/logits{step}"]), _values(ref[f"source/llama4/logits{step}"])
        assert (got - want).abs().max().item() <= (0 if exact else 2e-2 * peak), step


@pytest.mark.gpu
def test_loader_route_on_gpu(reference_run):
    work, env, ref = reference_run
    _run_ours(work, env, "--device", "cuda")
    ours = np.load(work / "ours.npz")
    for name in ENTRY_POINTS + ("_eight_bit",):
        assert int(ours[f"calls/{name}"][0]) > 0, f"{name} was never reached through linnet.torch.load"
    assert int(ours["calls/_int4_linear"][0]) > 0
    _plans_agree(ours, ref, exact=False)
    peak = max(_values(ref[f"source/llama4/logits{s}"]).abs().max().item() for s in range(3))
    checked = 0
    for mode in ("interp", "source", "cudagraphs"):
        for key in ref.files:
            if not key.startswith("source/"):
                continue
            name = key.split("/", 1)[1]
            got, want = _values(ours[f"{mode}/{name}"]), _values(ref[key])
            assert got.shape == want.shape, (mode, name)
            if name.startswith("llama4"):
                assert (got - want).abs().max().item() <= 2e-2 * peak, (mode, name)
            elif name == "lin8/rows40":
                # More than 32 rows of a per-channel int8 layer under numerics="fast": on a GPU the
                # reference rounds the activations to 8 bits too (quantized.py:187-189), which its
                # CPU run, the one compared with here, never does.  The W8A8 product itself is
                # pinned bit for bit against the oracle in test_w8a8_gpu.py.
                assert (got - want).abs().max().item() <= 3e-2 * want.abs().max().item(), (mode, name)
            else:
                torch.testing.assert_close(got, want, rtol=1e-2, atol=1e-2, msg=lambda m: f"{mode}/{name}: {m}")
            checked += 1
    assert checked == 3 * sum(1 for key in ref.files if key.startswith("source/"))
    for mode in ("interp", "source", "cudagraphs"):
        assert not np.array_equal(ours[f"{mode}/refresh/before"], ours[f"{mode}/refresh/after"])
        torch.testing.assert_close(_values(ours[f"{mode}/refresh/after"]), _values(ours[f"{mode}/refresh/other"]),
                                   rtol=0, atol=0)
    for step in range(3):
        got, want = _values(ours[f"decoder/llama4/logits{step}"]), _values(ref[f"source/llama4/logits{step}"])
        assert (got - want).abs().max().item() <= 2e-2 * peak, step
