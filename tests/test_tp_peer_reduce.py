"""The peer-memory all-reduce + residual add + RMSNorm kernel against NCCL + the
single-GPU kernel it replaces, and the reference-interface `OneShot` all-reduce, on 2, 4 and
8 GPUs of one box (each skipped with fewer)."""

from __future__ import annotations

import faulthandler
import gc
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from linnet_b200 import decoder as dec
from tests import decoder_util as du

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    faulthandler.dump_traceback_later(240, exit=True)  # a stuck rank ends itself, with a traceback
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        report = _checks(rank, world, dev)
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        torch.save(report, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        # every graph, model and symmetric-memory handle is gone by now (locals of _checks):
        # a captured NCCL collective that is still alive would keep this call waiting
        dist.destroy_process_group()
        faulthandler.cancel_dump_traceback_later()


def _config(world: int) -> dec.DecoderConfig:
    """Small, and every row-split shard still a whole number of 128-input groups."""
    if world <= 2:
        return dec.DecoderConfig.tiny()
    return dec.DecoderConfig(layers=2, hidden=256, heads=16, kv_heads=8, head_dim=64, mlp=1024, vocab=512, max_seq=32)


def _one_shot(rank: int, world: int, dev: torch.device) -> dict:
    """The cases of the reference's collective test (python/linnet/tests/torch/test_collectives.py: a
    4096-element bf16 message, one past the limit, 500 calls in a row, a captured chain replayed)."""
    from linnet_b200.tp import ONE_SHOT_BYTES, OneShot

    report = {}
    one = OneShot(dist.group.WORLD)

    def expected(x: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        total = torch.zeros(x.shape, device=dev)
        for part in parts:
            total += part.float()
        return total.to(x.dtype)

    gen = torch.Generator(device=dev).manual_seed(11 + rank)
    equal = True
    for dtype in (torch.bfloat16, torch.float16):
        for count in (4096, 8, ONE_SHOT_BYTES // 2):
            x = torch.randn(count, device=dev, generator=gen).to(dtype)
            equal &= bool(torch.equal(one(x), expected(x)))
    report["one_shot_exact"] = equal
    # past the limit and f32: the group's backend takes the message
    big = torch.randn(ONE_SHOT_BYTES // 2 + 8, device=dev, generator=gen).to(torch.bfloat16)
    wide = torch.randn(1000, device=dev, generator=gen)
    report["covers"] = (one.covers(big), one.covers(wide), one.covers(wide[:8].to(torch.bfloat16)))
    # (the library adds in bf16 in an order of its own: every one of its world - 1 roundings can be
    # off by 2^-9 of a running sum, the kernel's one rounding by 2^-9 of the total)
    close = bool(torch.allclose(one(big).float(), expected(big).float(), rtol=2e-2, atol=1e-2 * world))
    close &= bool(torch.allclose(one(wide), sum_f32(wide, world), rtol=1e-5, atol=1e-5))
    report["library_close"] = close
    # 500 calls in a row, each on the last one's result scaled back: nothing drifts or sticks
    x = torch.randn(4096, device=dev, generator=gen).to(torch.bfloat16)
    start, want = x.clone(), expected(x)
    for _ in range(500):
        got = one(start)
    report["many_calls_equal"] = bool(torch.equal(got, want))
    # a chain of 10 captured in a graph, replayed three times
    stream = torch.cuda.Stream(dev)
    with torch.cuda.stream(stream):
        one(start)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            v = start
            for _ in range(10):
                v = one(v) * (1.0 / world)
        outs = []
        for _ in range(3):
            graph.replay()
            torch.cuda.synchronize()
            outs.append(v.clone())
    chain = start
    for _ in range(10):
        chain = expected(chain) * (1.0 / world)
    report["graph_equal"] = all(bool(torch.equal(o, chain)) for o in outs)
    report["one_shot_error"] = one.error()
    del graph, v
    return report


def sum_f32(x: torch.Tensor, world: int) -> torch.Tensor:
    out = x.clone()
    dist.all_reduce(out)
    return out


def _checks(rank: int, world: int, dev: torch.device) -> dict:
    from linnet_b200 import glue, kernels
    from linnet_b200.tp import PeerReduce

    report: dict = {"kernel_exact": True, "kernel_error": 0, "decoder_max_diff": 0.0, "replay_equal": True,
                    "decoder_error": 0}
    for protocol in ("words", "flags"):  # both exchanges, whatever the default for this group size
        # 1. the kernel alone, three call sites visited round-robin, several epochs
        hidden, rows, sites = 1024, 5, 3
        reduce = PeerReduce(sites, 8, hidden, dev, protocol=protocol)
        gen = torch.Generator(device=dev).manual_seed(100 + rank)
        shared = torch.Generator(device=dev).manual_seed(7)
        weight = (1 + 0.1 * torch.randn(hidden, device=dev, generator=shared)).to(torch.bfloat16)
        exact = True
        for epoch in range(4):
            for site in range(sites):
                part = torch.randn(rows, hidden, device=dev, generator=gen).to(torch.bfloat16)
                x = torch.randn(rows, hidden, device=dev, generator=shared).to(torch.bfloat16)
                reduce.partial(site, rows).copy_(part)
                x_peer = x.clone()
                y_peer = reduce.add_rmsnorm(site, x_peer, weight, 1e-5)
                # what it replaces: all ranks' partials summed in rank order in f32, rounded once
                parts = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(parts, part)
                total = torch.zeros(rows, hidden, device=dev)
                for p in parts:
                    total += p.float()
                x_ref = x.clone()
                y_ref = glue.add_rmsnorm(x_ref, total.to(torch.bfloat16), weight, 1e-5)
                exact &= bool(torch.equal(x_peer, x_ref)) and bool(torch.equal(y_peer, y_ref))
        report["kernel_exact"] &= exact
        report["kernel_error"] |= reduce.error()

        # 2. the decoder: NCCL route and peer route produce the same logits, eagerly and replayed
        cfg = _config(world)
        whole = du.whole_model(cfg)
        logits = {}
        for route in ("nccl", "peer"):
            model = du.rank_model(cfg, whole, rank, world, kernels.int4_linear, device=dev)
            if route == "peer":
                model.enable_peer_reduce(4, protocol)
            logits[route] = du.run_steps(model, cfg, batch=4, steps=3, device=dev).float()
        report["decoder_max_diff"] = max(report["decoder_max_diff"],
                                         (logits["nccl"] - logits["peer"]).abs().max().item())
        report["decoder_scale"] = logits["nccl"].abs().max().item()

        tokens = torch.tensor([3, 5, 7, 9], device=dev)
        positions = torch.full((4,), 3, device=dev, dtype=torch.long)
        stream = torch.cuda.Stream(dev)
        with torch.cuda.stream(stream):
            eager = model.step(tokens, positions).clone()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                out = model.step(tokens, positions)
            for _ in range(5):
                graph.replay()
            torch.cuda.synchronize()
        report["replay_equal"] &= bool(torch.equal(out, eager))
        report["decoder_error"] |= model.peer_reduce.error()
        del graph, out, model, reduce
        gc.collect()
    report.update(_one_shot(rank, world, dev))
    return report


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_reduce_matches_nccl_route(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        report = torch.load(tmp_path / f"rank{rank}.pt")
        assert report["kernel_error"] == 0 and report["decoder_error"] == 0
        assert report["kernel_exact"], "peer reduction differs from the rank-ordered f32 sum"
        # two ranks: NCCL's bf16 sum and the f32 sum rounded once are the same number; more
        # ranks: NCCL rounds its running sums to bf16, the kernel rounds once
        assert report["decoder_max_diff"] <= (1e-3 if world == 2 else 3e-2) * report["decoder_scale"]
        assert report["replay_equal"]
        assert report["one_shot_error"] == 0
        assert report["one_shot_exact"], "OneShot differs from the rank-ordered f32 sum"
        assert report["covers"] == (False, False, True)
        assert report["library_close"], "a message past the one-shot limit differs from the library's sum"
        assert report["many_calls_equal"], "500 calls in a row drifted"
        assert report["graph_equal"], "a captured chain of calls differs from the eager chain"
