"""Positions are device data: the decode-step kernels check them on the device.  A position
outside the cache stores nothing, forms no address outside the caches, and is reported by
`b200q_decoder_status`; positions of the wrong dtype are refused on the host."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

BATCH, NQ, NKV, HD, SEQ = 3, 4, 2, 64, 16


def _tensors():
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(0)
    qkv = torch.randn(BATCH, (NQ + 2 * NKV) * HD, device=dev, generator=gen).to(torch.bfloat16)
    # canaries around the caches: one extra batch row before and after, never to be touched
    cache_k = torch.full((BATCH + 2, NKV, SEQ, HD), 7.0, device=dev, dtype=torch.bfloat16)
    cache_v = torch.full((BATCH + 2, NKV, SEQ, HD), 7.0, device=dev, dtype=torch.bfloat16)
    return dev, qkv, cache_k, cache_v


def test_positions_of_the_wrong_type_are_refused():
    from linnet_b200 import glue

    dev, qkv, cache_k, cache_v = _tensors()
    with pytest.raises(ValueError, match="int64"):
        glue.rope_cache(qkv, torch.zeros(BATCH, dtype=torch.int32, device=dev), cache_k[1:-1], cache_v[1:-1], NQ, NKV, 1e4)
    with pytest.raises(ValueError, match="int64"):
        glue.rope_cache(qkv, torch.zeros(BATCH + 1, dtype=torch.int64, device=dev), cache_k[1:-1], cache_v[1:-1], NQ, NKV, 1e4)


@pytest.mark.parametrize("bad", [SEQ, -1, 1 << 40])
@pytest.mark.parametrize("fused", [False, True])
def test_a_position_outside_the_cache_is_reported_and_harmless(bad, fused):
    from linnet_b200 import glue

    dev, qkv, cache_k, cache_v = _tensors()
    inner_k, inner_v = cache_k[1:-1], cache_v[1:-1]
    glue.decoder_status()  # clear whatever an earlier test left
    positions = torch.tensor([2, bad, 5], dtype=torch.int64, device=dev)
    if fused:
        table = glue.rope_table(SEQ, HD, 1e4, dev)
        out = glue.rope_attention(qkv, positions, table, inner_k, inner_v, NQ, NKV, splits=2)
    else:
        q = glue.rope_cache(qkv, positions, inner_k, inner_v, NQ, NKV, 1e4)
        out = glue.decode_attention(q, inner_k, inner_v, positions, splits=2)
    torch.cuda.synchronize()
    with pytest.raises(ValueError, match="batch row 1"):
        glue.decoder_status()
    glue.decoder_status()  # reported once, then clear
    # nothing outside the caches was written, and nothing in the bad row's cache
    assert bool((cache_k[0] == 7).all()) and bool((cache_k[-1] == 7).all())
    assert bool((cache_v[0] == 7).all()) and bool((cache_v[-1] == 7).all())
    assert bool((inner_k[1] == 7).all()) and bool((inner_v[1] == 7).all())
    # the good rows were stored at their positions
    assert not bool((inner_k[0, :, 2] == 7).all()) and not bool((inner_k[2, :, 5] == 7).all())
    assert bool(torch.isfinite(out[0].float()).all()) and bool(torch.isfinite(out[2].float()).all())
    # and the context still works
    good = torch.tensor([1, 1, 1], dtype=torch.int64, device=dev)
    glue.rope_cache(qkv, good, inner_k, inner_v, NQ, NKV, 1e4)
    torch.cuda.synchronize()
    glue.decoder_status()
