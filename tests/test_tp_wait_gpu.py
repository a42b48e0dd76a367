"""The bounded waits of the tensor-parallel kernels, exercised on ONE GPU without any fault: the
kernel is told it is rank 0 of 2, both receive areas are local buffers, and nobody ever plays
rank 1.  The wait for rank 1 runs out (2 ms here, `b200q_set_wait_limit_ns`), the kernel
returns, the error word says 100 + 1, the context stays usable, a second call does not wait
again, and after the host has cleared the word an ordinary launch succeeds.  (The reference's
one-shot all-reduce spins without a bound there, python/linnet/src/linnet/torch/kernels.py:1146-1148.)"""

from __future__ import annotations

import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

ROWS, HIDDEN = 4, 1024


@pytest.fixture
def short_wait():
    from linnet_b200 import _lib

    lib = _lib.load()
    _lib.check(lib.b200q_set_wait_limit_ns(2_000_000))
    yield lib
    _lib.check(lib.b200q_set_wait_limit_ns(1_000_000_000))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("protocol", ["words", "flags", "plain"])
def test_wait_for_a_missing_rank_runs_out(short_wait, protocol):
    from linnet_b200 import _lib, glue

    lib = short_wait
    dev = torch.device("cuda", 0)
    world = 2
    int64s = ctypes.c_int64 * world
    state = torch.zeros(3, dtype=torch.int32, device=dev)  # epoch, done, error
    counters = (state.data_ptr(), state.data_ptr() + 4, state.data_ptr() + 8)
    x = torch.randn(ROWS, HIDDEN, device=dev).to(torch.bfloat16)
    x_before = x.clone()
    weight = torch.ones(HIDDEN, device=dev, dtype=torch.bfloat16)
    y = torch.empty_like(x)
    partial = torch.randn(ROWS, HIDDEN, device=dev).to(torch.bfloat16)

    if protocol == "flags":
        areas = [torch.zeros(world, ROWS * HIDDEN, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        flags = [torch.zeros(world, ROWS, dtype=torch.int32, device=dev) for _ in range(world)]
        areas[0][0].copy_(partial.reshape(-1))
        area_ptrs, flag_ptrs = int64s(*[a.data_ptr() for a in areas]), int64s(*[f.data_ptr() for f in flags])

        def call() -> int:
            return lib.b200q_tp_allreduce_add_rmsnorm_flags(
                ctypes.addressof(area_ptrs), ctypes.addressof(flag_ptrs), ROWS * HIDDEN, ROWS, world, 0, *counters,
                x.data_ptr(), weight.data_ptr(), y.data_ptr(), ROWS, HIDDEN, 1e-5, _stream())
    else:
        slot_words = ROWS * HIDDEN // 2
        areas = [torch.zeros(world, slot_words, 2, dtype=torch.int32, device=dev) for _ in range(world)]
        area_ptrs = int64s(*[a.data_ptr() for a in areas])
        if protocol == "words":
            def call() -> int:
                return lib.b200q_tp_allreduce_add_rmsnorm(
                    ctypes.addressof(area_ptrs), slot_words, partial.data_ptr(), world, 0, *counters, x.data_ptr(),
                    weight.data_ptr(), y.data_ptr(), ROWS, HIDDEN, 1e-5, _stream())
        else:
            def call() -> int:
                return lib.b200q_tp_allreduce(ctypes.addressof(area_ptrs), slot_words, partial.data_ptr(), world, 0,
                                              *counters, y.data_ptr(), ROWS * HIDDEN, _lib.BF16, _stream())

    t0 = time.perf_counter()
    _lib.check(call())
    torch.cuda.synchronize()
    first = time.perf_counter() - t0
    assert int(state[2]) == 101, "the wait for rank 1 should have run out"
    assert first < 1.0, f"the 2 ms limit was not honoured ({first:.3f} s)"
    if protocol != "plain":
        assert torch.equal(x, x_before), "a reduction that gave up must leave the residual stream alone"
    # a later call does not wait again while the error stands
    t0 = time.perf_counter()
    _lib.check(call())
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5
    assert int(state[2]) == 101
    # the context is fine: clear the word, run an ordinary kernel
    state.zero_()
    got = glue.add_rmsnorm(x.clone(), None, weight, 1e-5)
    want = torch.nn.functional.rms_norm(x.float(), (HIDDEN,), weight.float(), 1e-5)
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2)


def test_wait_limit_argument_is_checked():
    from linnet_b200 import _lib

    lib = _lib.load()
    assert lib.b200q_set_wait_limit_ns(0) == _lib.ERROR
    assert "between 1 ns and 60 s" in _lib.last_error()
