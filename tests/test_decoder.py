"""The tensor-parallel decoder: on the CPU the sharding and the collectives are checked
with the oracle as the linear operator (gloo, world size 2); on a GPU the same model
runs on the CUDA operators and must agree with the CPU oracle model."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from linnet_b200 import decoder as dec
from tests import decoder_util as du


def dense_reference(cfg, whole, batch, steps):
    """The same model with dequantized f32 weights and textbook attention."""
    from oracle import linear_oracle as lo

    def W(t):
        return lo.int4_weight(*t, torch.float32)

    gen = torch.Generator().manual_seed(3)
    hd = cfg.head_dim
    ks = [torch.zeros(batch, cfg.kv_heads, cfg.max_seq, hd) for _ in range(cfg.layers)]
    vs = [torch.zeros(batch, cfg.kv_heads, cfg.max_seq, hd) for _ in range(cfg.layers)]
    out = None
    for t in range(steps):
        tokens = torch.randint(0, cfg.vocab, (batch,), generator=gen)
        pos = torch.full((batch,), t, dtype=torch.long)
        x = whole["embed"][tokens].float()
        for i, L in enumerate(whole["layers"]):
            def norm(v, w):
                return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * w.float()
            h = norm(x, L["norm1"])
            q = (h @ W(L["q"]).T).reshape(batch, cfg.heads, hd)
            k = (h @ W(L["k"]).T).reshape(batch, cfg.kv_heads, hd)
            v = (h @ W(L["v"]).T).reshape(batch, cfg.kv_heads, hd)
            q, k = dec.rotary(q, pos, cfg.rope_theta), dec.rotary(k, pos, cfg.rope_theta)
            ks[i][:, :, t], vs[i][:, :, t] = k, v
            rep = cfg.heads // cfg.kv_heads
            kk = ks[i][:, :, :t + 1].repeat_interleave(rep, dim=1)
            vv = vs[i][:, :, :t + 1].repeat_interleave(rep, dim=1)
            att = torch.softmax(torch.einsum("bhd,bhsd->bhs", q, kk) / hd ** 0.5, dim=-1)
            o = torch.einsum("bhs,bhsd->bhd", att, vv).reshape(batch, -1)
            x = x + o @ W(L["o"]).T
            h = norm(x, L["norm2"])
            x = x + (torch.nn.functional.silu(h @ W(L["gate"]).T) * (h @ W(L["up"]).T)) @ W(L["down"]).T
        out = norm(x, whole["final_norm"]) @ W(whole["head"]).T
    return out


def test_single_rank_matches_dense_reference():
    cfg = dec.DecoderConfig.tiny()
    whole = du.whole_model(cfg)
    model = du.rank_model(cfg, whole, 0, 1, du.oracle_linear)
    got = du.run_steps(model, cfg, batch=3, steps=3).float()
    want = dense_reference(cfg, whole, 3, 3)
    assert got.shape == (3, cfg.vocab)
    torch.testing.assert_close(got, want, rtol=5e-2, atol=5e-2 * want.abs().max().item())


def test_shard_shapes_and_checks():
    cfg = dec.DecoderConfig.tiny()
    whole = du.whole_model(cfg)
    m = du.rank_model(cfg, whole, 1, 2, du.oracle_linear)
    w = m.layers[0]
    assert w.qkv[0].shape == ((cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim // 2, cfg.hidden // 128, 64)
    assert w.o[0].shape == (cfg.hidden, cfg.heads * cfg.head_dim // 2 // 128, 64)   # K groups halved
    assert w.down[1].shape == (cfg.hidden, cfg.mlp // 2 // 128)
    assert m.head[0].shape[0] == cfg.vocab // 2
    with pytest.raises(ValueError, match="do not divide"):
        dec.check_tp(cfg, 3)
    with pytest.raises(ValueError, match="whole groups"):
        dec.check_tp(dec.DecoderConfig(layers=1, hidden=256, heads=4, kv_heads=4, head_dim=64, mlp=512,
                                       vocab=512, max_seq=8), 4)
    full = dec.DecoderConfig.llama31_8b()
    for tp in (1, 2, 4, 8):
        dec.check_tp(full, tp)
    assert abs(full.int4_elements() - 7.5046e9) < 1e6


def test_attention_split_heuristic():
    """Pure host logic: a power of two, at least 64 positions a split, about two blocks per SM."""
    from linnet_b200 import glue

    assert glue.attention_splits(1, 8, 2048) == 32      # the cluster launch caps it at 8
    assert glue.attention_splits(8, 8, 2048) == 4
    assert glue.attention_splits(64, 8, 2048) == 1
    assert glue.attention_splits(1, 1, 2048) == 32
    assert glue.attention_splits(1, 8, 100) == 1        # fewer than 128 positions: no split
    for batch, nkv, seq in ((1, 8, 2048), (3, 2, 777), (200, 8, 4096)):
        splits = glue.attention_splits(batch, nkv, seq)
        assert splits & (splits - 1) == 0 and (splits == 1 or seq // splits >= 64)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        cfg = dec.DecoderConfig.tiny()
        whole = du.whole_model(cfg)
        model = du.rank_model(cfg, whole, rank, world, du.oracle_linear)
        logits = du.run_steps(model, cfg, batch=2, steps=3)
        torch.save(logits, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_whole_model(tmp_path):
    """Each rank holds half of every projection; one all-reduce per row-split layer and
    one all-gather of the logits reproduce the single-rank result on every rank."""
    world = 2
    mp.spawn(_tp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    cfg = dec.DecoderConfig.tiny()
    whole = du.whole_model(cfg)
    single = du.run_steps(du.rank_model(cfg, whole, 0, 1, du.oracle_linear), cfg, batch=2, steps=3).float()
    for rank in range(world):
        got = torch.load(tmp_path / f"rank{rank}.pt").float()
        assert got.shape == single.shape
        # partial sums are rounded to bf16 before they are added, so not bit-identical
        torch.testing.assert_close(got, single, rtol=3e-2, atol=3e-2 * single.abs().max().item())


@pytest.mark.gpu
def test_gpu_decoder_matches_cpu_oracle_decoder():
    from linnet_b200 import kernels

    cfg = dec.DecoderConfig.tiny()
    whole = du.whole_model(cfg)
    cpu = du.run_steps(du.rank_model(cfg, whole, 0, 1, du.oracle_linear), cfg, batch=4, steps=3).float()
    gpu_model = du.rank_model(cfg, whole, 0, 1, kernels.int4_linear, device="cuda")
    gpu = du.run_steps(gpu_model, cfg, batch=4, steps=3, device="cuda").float().cpu()
    torch.testing.assert_close(gpu, cpu, rtol=3e-2, atol=3e-2 * cpu.abs().max().item())


@pytest.mark.gpu
def test_fused_glue_equals_torch_glue():
    """The fused kernels between the linears against the PyTorch ops they replace."""
    from linnet_b200 import glue, kernels

    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(5)
    for hidden, rows in ((4096, 1), (256, 5), (1024, 64)):
        x = torch.randn(rows, hidden, generator=gen).to(torch.bfloat16).to(dev)
        d = torch.randn(rows, hidden, generator=gen).to(torch.bfloat16).to(dev)
        w = (1 + 0.1 * torch.randn(hidden, generator=gen)).to(torch.bfloat16).to(dev)
        want_x = x + d
        want = torch.nn.functional.rms_norm(want_x, (hidden,), w, 1e-5)
        got = glue.add_rmsnorm(x, d, w, 1e-5)
        assert torch.equal(x, want_x)
        torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-2)
        gu = torch.randn(rows, 2 * hidden, generator=gen).to(torch.bfloat16).to(dev)
        want = torch.nn.functional.silu(gu[:, :hidden]) * gu[:, hidden:]
        torch.testing.assert_close(glue.silu_mul(gu).float(), want.float(), rtol=1e-2, atol=1e-2)
    for nq, nkv, hd, S, batch in ((32, 8, 128, 2048, 1), (4, 2, 64, 32, 3), (8, 8, 128, 300, 2), (16, 2, 64, 128, 5)):
        qkv = torch.randn(batch, (nq + 2 * nkv) * hd, generator=gen).to(torch.bfloat16).to(dev)
        ck = torch.randn(batch, nkv, S, hd, generator=gen).to(torch.bfloat16).to(dev)
        cv = torch.randn(batch, nkv, S, hd, generator=gen).to(torch.bfloat16).to(dev)
        pos = torch.randint(0, S, (batch,), generator=gen).to(dev)
        pos[0] = S - 1
        ck2, cv2 = ck.clone(), cv.clone()
        ck_before, cv_before = ck.clone(), cv.clone()
        q, k, v = qkv.split([nq * hd, nkv * hd, nkv * hd], dim=-1)
        q_ref = dec.rotary(q.reshape(batch, nq, hd), pos, 500000.0)
        rows_i = torch.arange(batch, device=dev)
        ck2[rows_i, :, pos] = dec.rotary(k.reshape(batch, nkv, hd), pos, 500000.0)
        cv2[rows_i, :, pos] = v.reshape(batch, nkv, hd)
        q_got = glue.rope_cache(qkv, pos, ck, cv, nq, nkv, 500000.0)
        torch.testing.assert_close(q_got.float(), q_ref.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(ck.float(), ck2.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(cv, cv2)
        mask = (torch.arange(S, device=dev)[None, :] <= pos[:, None])[:, None, None, :]
        want = torch.nn.functional.scaled_dot_product_attention(
            q_ref[:, :, None, :], ck2, cv2, attn_mask=mask, enable_gqa=True).reshape(batch, nq * hd)
        for splits in (None, 1, 3, 8, 16):  # up to 8: one cluster launch; 16: partials + merge kernel
            got = glue.decode_attention(q_ref, ck2, cv2, pos, splits)
            torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        # rotary + cache write + attention in one launch, from the caches before the write
        table = glue.rope_table(S, hd, 500000.0, dev)
        for splits in (None, 1, 5):
            ck3, cv3 = ck_before.clone(), cv_before.clone()
            got = glue.rope_attention(qkv, pos, table, ck3, cv3, nq, nkv, splits)
            torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
            torch.testing.assert_close(ck3.float(), ck2.float(), rtol=2e-2, atol=2e-2)
            assert torch.equal(cv3, cv2)


@pytest.mark.gpu
def test_fused_and_torch_steps_agree():
    from linnet_b200 import kernels

    cfg = dec.DecoderConfig.tiny()
    whole = du.whole_model(cfg)
    outs = []
    for fused in (True, False):
        model = du.rank_model(cfg, whole, 0, 1, kernels.int4_linear, device="cuda")
        model.fused = fused
        outs.append(du.run_steps(model, cfg, batch=4, steps=3, device="cuda").float())
    torch.testing.assert_close(outs[0], outs[1], rtol=3e-2, atol=3e-2 * outs[1].abs().max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("batch", [1, 2, 3])
def test_folded_step_equals_unfolded_step(batch):
    """Residual add + RMS norm inside the products and silu(gate) * up inside the down projection
    (five launches a layer) give the logits and the caches of the step that runs them as kernels
    of their own, bit for bit, eagerly and replayed from a graph; three rows run unfolded either way."""
    from linnet_b200 import _lib, kernels, quant

    cfg = dec.DecoderConfig(layers=3, hidden=1024, heads=8, kv_heads=2, head_dim=128, mlp=2048, vocab=1024, max_seq=64)
    dev = torch.device("cuda", 0)
    model = dec.build_random(cfg, dev, rank=0, tp=1, seed=3, linear=kernels.int4_linear,
                             quantize=quant.quantize_int4_groups)
    tokens = torch.arange(5, 5 + batch, device=dev)
    results = {}
    for folded in (False, True):
        model.fold_norm = model.fold_swiglu = folded
        model.allocate_cache(batch, torch.Generator(device=dev).manual_seed(4))
        logits = []
        for step in range(3):
            positions = torch.full((batch,), 10 + step, device=dev, dtype=torch.long)
            logits.append(model.step(tokens + step, positions).clone())
        graph = torch.cuda.CUDAGraph()
        positions = torch.full((batch,), 13, device=dev, dtype=torch.long)
        eager = model.step(tokens, positions).clone()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            out = model.step(tokens, positions)
        for _ in range(5):
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, eager)
        results[folded] = (logits, [c.clone() for c in model.cache_k], [c.clone() for c in model.cache_v])
        del graph, out
    for a, b in zip(results[False][0], results[True][0]):
        assert torch.equal(a, b)
    for which in (1, 2):
        for a, b in zip(results[False][which], results[True][which]):
            assert torch.equal(a, b)
    _lib.check(_lib.load().b200q_int4_gemm_status())


@pytest.mark.gpu
@pytest.mark.parametrize("shape", ["tiny", "wide"])
def test_gpu_decoder_graph_replay(shape):
    """A captured step replays to the eager result, every time: inside a graph the kernels
    of a step overlap through programmatic dependent launch far more than in eager mode, so
    this is the test that catches a kernel reading its input too early or through a stale path."""
    from linnet_b200 import kernels, quant

    cfg = dec.DecoderConfig.tiny() if shape == "tiny" else dec.DecoderConfig(
        layers=3, hidden=1024, heads=8, kv_heads=2, head_dim=128, mlp=2048, vocab=1024, max_seq=256)
    dev = torch.device("cuda", 0)
    model = dec.build_random(cfg, dev, rank=0, tp=1, seed=1, linear=kernels.int4_linear,
                             quantize=quant.quantize_int4_groups)
    for batch in (2, 5):
        model.allocate_cache(batch, torch.Generator(device=dev).manual_seed(2))
        tokens = torch.arange(3, 3 + batch, device=dev)
        positions = torch.full((batch,), cfg.max_seq - 1, device=dev, dtype=torch.long)
        eager = model.step(tokens, positions).clone()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = model.step(tokens, positions)
        for _ in range(20):
            graph.replay()
            torch.cuda.synchronize()
            torch.testing.assert_close(out, eager, rtol=0, atol=0)
        del graph, out
