"""`b200q_decode_attention_static`: the attention entry point for hosts that cannot
allocate device memory (fixed-arena runtimes, plug-ins without the allocator, callers
inside a stream capture).  Its split-KV partial results live in an array built into the
library instead of caller-owned scratch.  Called through the C ABI twice in a row (the
array keeps the first call's contents) and compared with `b200q_decode_attention`; also
checked: sizes beyond the built-in array are refused with a clear message.

This file sorts last so that a run stopping at the first failure has already run every
other test."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(batch, nq, nkv, hd, seq, seed):
    gen = torch.Generator().manual_seed(seed)
    dev = torch.device("cuda", 0)
    q = torch.randn(batch, nq, hd, generator=gen).to(torch.bfloat16).to(dev)
    k = torch.randn(batch, nkv, seq, hd, generator=gen).to(torch.bfloat16).to(dev)
    v = torch.randn(batch, nkv, seq, hd, generator=gen).to(torch.bfloat16).to(dev)
    pos = torch.randint(seq // 2, seq, (batch,), generator=gen).to(dev)
    return q, k, v, pos


def _with_scratch(lib, q, k, v, pos, splits):
    from linnet_b200 import _lib

    batch, nq, hd = q.shape
    nkv, seq = k.shape[1], k.shape[2]
    scratch = torch.empty(lib.b200q_decode_attention_scratch_bytes(batch, nq, hd, splits), dtype=torch.uint8,
                          device=q.device)
    out = torch.empty(batch, nq * hd, dtype=torch.bfloat16, device=q.device)
    _lib.check(lib.b200q_decode_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), pos.data_ptr(),
                                          out.data_ptr(), scratch.data_ptr(), batch, nq, nkv, hd, seq, splits,
                                          torch.cuda.current_stream().cuda_stream))
    return out


def _static(lib, q, k, v, pos, splits):
    from linnet_b200 import _lib

    batch, nq, hd = q.shape
    nkv, seq = k.shape[1], k.shape[2]
    out = torch.empty(batch, nq * hd, dtype=torch.bfloat16, device=q.device)
    _lib.check(lib.b200q_decode_attention_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), pos.data_ptr(),
                                                 out.data_ptr(), batch, nq, nkv, hd, seq, splits,
                                                 torch.cuda.current_stream().cuda_stream))
    return out


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    from linnet_b200 import _lib

    lib = _lib.load()
    torch.cuda.set_device(0)
    assert lib.b200q_decode_attention_static_scratch_limit() == 4 << 20
    # two different problems back to back: the second call finds the first one's partial
    # results in the shared array and must not be affected by them
    first = _inputs(2, 32, 8, 128, 512, seed=1)
    second = _inputs(3, 8, 2, 64, 200, seed=2)
    for args, splits in ((first, 16), (second, 3), (first, 16)):
        got = _static(lib, *args, splits)
        want = _with_scratch(lib, *args, splits)
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)


def test_static_scratch_refuses_what_does_not_fit():
    from linnet_b200 import _lib

    lib = _lib.load()
    q, k, v, pos = _inputs(1, 8, 2, 64, 64, seed=3)
    out = torch.empty(1, 8 * 64, dtype=torch.bfloat16, device=q.device)
    # 4096 rows x 64 heads x 8 splits x 130 floats is far beyond 4 MiB: refused on the host
    status = lib.b200q_decode_attention_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), pos.data_ptr(),
                                               out.data_ptr(), 4096, 64, 8, 128, 64, 8,
                                               torch.cuda.current_stream().cuda_stream)
    assert status == _lib.ERROR
    assert "built-in array holds" in _lib.last_error()
