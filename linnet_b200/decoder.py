"""A Llama-3.1-8B-shaped int4 decoder for the decode benchmark: every linear layer is
an int4-g128 `linnet::int4_linear`, tensor-parallel the way the reference splits a card
by a `Shards` generic (docs/torch.md:210-220; python/linnet/tests/torch/test_shards.py:47-59):

* column split (output rows; packed / scale / zero cut along axis 0): fused q|k|v,
  fused gate|up, and the output head (followed by one all-gather of the logits);
* row split (whole input groups; cut along axis 1): o_proj and down_proj, each
  followed by ONE all-reduce of the `[batch, hidden]` partial sums
  (`std.nn.parallel::all_reduce`, stdlib/nn/parallel.linnet:9-11): NCCL, or after
  `enable_peer_reduce()` one peer-memory kernel that also does the residual add and the
  norm that follow (`linnet_b200.tp`);
* the KV cache and attention are split by KV heads.

Fusing q|k|v and gate|up is this build's own step at pack time (the reference joins
sibling projections only for dense and 8-bit layers, src/backend/torch_source.cpp:82-92);
the packed layout makes it a concatenation along the output axis.

The linear operator is injected (`linear=`): the product passes the CUDA operator, the
CPU tests pass the oracle, so the sharding and the collectives are exercised on `gloo`
ranks without a GPU.  Between the linears (RMSNorm, rotary embedding, cache write,
attention, SwiGLU) `step` has two routes with the same arithmetic: plain PyTorch ops (any
device; what the reference's generated source does, and what the CPU tests run) and, on a
GPU, the fused kernels of `linnet_b200.glue` (eight launches a layer instead of about fifty).
Either way a step is recorded into one CUDA graph per batch size, which is how the
reference's serving engine replays a decode step
(python/linnet/src/linnet/torch/compiled.py:430-503).
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist
import torch.nn.functional as F

Linear = Callable[[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor]


@dataclass(frozen=True)
class DecoderConfig:
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    mlp: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    eps: float = 1e-5
    max_seq: int = 2048
    group: int = 128

    @staticmethod
    def llama31_8b() -> "DecoderConfig":
        return DecoderConfig()

    @staticmethod
    def tiny() -> "DecoderConfig":
        return DecoderConfig(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=64, mlp=512,
                             vocab=512, max_seq=32)

    def int4_elements(self) -> int:
        per_layer = (self.hidden * (self.heads + 2 * self.kv_heads) * self.head_dim
                     + self.heads * self.head_dim * self.hidden + 3 * self.mlp * self.hidden)
        return per_layer * self.layers + self.vocab * self.hidden


Int4 = tuple[torch.Tensor, torch.Tensor, torch.Tensor]  # packed, scale, zero


def shard_rows(w: Int4, rank: int, shards: int) -> Int4:
    """Column split: this rank's block of output rows (axis 0 of all three tensors)."""
    n = w[0].shape[0] // shards
    return tuple(t[rank * n:(rank + 1) * n].contiguous() for t in w)  # type: ignore[return-value]


def shard_groups(w: Int4, rank: int, shards: int) -> Int4:
    """Row split: this rank's block of input groups (axis 1 of all three tensors)."""
    n = w[0].shape[1] // shards
    return tuple(t[:, rank * n:(rank + 1) * n].contiguous() for t in w)  # type: ignore[return-value]


def concat_rows(*ws: Int4) -> Int4:
    return tuple(torch.cat(parts, dim=0).contiguous() for parts in zip(*ws))  # type: ignore[return-value]


@dataclass
class LayerWeights:
    qkv: Int4
    o: Int4
    gate_up: Int4
    down: Int4
    norm1: torch.Tensor
    norm2: torch.Tensor


def shard_layer(cfg: DecoderConfig, q: Int4, k: Int4, v: Int4, o: Int4, gate: Int4, up: Int4,
                down: Int4, norm1: torch.Tensor, norm2: torch.Tensor, rank: int, tp: int) -> LayerWeights:
    """One rank's weights of a layer from the whole layer's quantized tensors."""
    return LayerWeights(
        qkv=concat_rows(shard_rows(q, rank, tp), shard_rows(k, rank, tp), shard_rows(v, rank, tp)),
        o=shard_groups(o, rank, tp),
        gate_up=concat_rows(shard_rows(gate, rank, tp), shard_rows(up, rank, tp)),
        down=shard_groups(down, rank, tp),
        norm1=norm1, norm2=norm2)


def check_tp(cfg: DecoderConfig, tp: int) -> None:
    if cfg.heads % tp or cfg.kv_heads % tp:
        raise ValueError(f"{tp} shards do not divide {cfg.heads} heads / {cfg.kv_heads} KV heads")
    for name, depth in (("o_proj", cfg.heads * cfg.head_dim), ("down_proj", cfg.mlp)):
        if (depth // tp) % cfg.group or depth % tp:
            raise ValueError(f"{name}: {depth} inputs over {tp} shards are not whole groups of {cfg.group}")
    if cfg.vocab % tp or cfg.mlp % tp:
        raise ValueError(f"{tp} shards do not divide the vocabulary or the MLP width")


def rotary(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotary embedding of `x` [B, heads, D] at `positions` [B] (halves rotated)."""
    half = x.shape[-1] // 2
    freqs = theta ** (-torch.arange(half, device=x.device, dtype=torch.float32) / half)
    angle = positions.to(torch.float32)[:, None] * freqs[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)


class Int4Decoder:
    """One tensor-parallel rank of the decoder.  `step` runs one decode step for
    `tokens` [B] at `positions` [B] and returns the full `[B, vocab]` logits."""

    def __init__(self, cfg: DecoderConfig, layers: list[LayerWeights], embed: torch.Tensor,
                 final_norm: torch.Tensor, head: Int4, *, linear: Linear, rank: int = 0, tp: int = 1,
                 group: "dist.ProcessGroup | None" = None, fused: bool | None = None) -> None:
        check_tp(cfg, tp)
        # Fused glue kernels by default wherever the model lives on a GPU.
        self.fused = embed.is_cuda if fused is None else fused
        self.early = False       # fused route: pass early=True to the products (programmatic dependent launch)
        # fused route: the down projection forms silu(gate) * up itself (swiglu=True).  Off by default:
        # every block of that product stages the whole input, so every block would evaluate all
        # 14336 silus of the 8B shape, which costs what the saved launch brings (measured on a B200,
        # batch 1: 1.911 ms a step folded against 1.849 ms with the kernel of its own).
        self.fold_swiglu = False
        self.fold_norm = False    # fused route, one rank, one or two rows: residual add and norm inside the products
        self.cfg, self.layers, self.embed, self.final_norm, self.head = cfg, layers, embed, final_norm, head
        self.linear, self.rank, self.tp, self.group = linear, rank, tp, group
        self.cache_k: list[torch.Tensor] = []
        self.cache_v: list[torch.Tensor] = []
        self.peer_reduce = None  # set by enable_peer_reduce()
        self.rope_table = None   # cos / sin of every position, made by allocate_cache()

    # -- state ---------------------------------------------------------------------
    def allocate_cache(self, batch: int, fill: "torch.Generator | None" = None) -> None:
        """A `[batch, kv_heads / tp, max_seq, head_dim]` cache per layer for K and V,
        filled ~N(0, 1) when a generator is given (the benchmark's synthetic history)."""
        cfg = self.cfg
        shape = (batch, cfg.kv_heads // self.tp, cfg.max_seq, cfg.head_dim)
        dev, dt = self.embed.device, self.embed.dtype
        self.cache_k, self.cache_v = [], []
        for _ in range(cfg.layers):
            for store in (self.cache_k, self.cache_v):
                t = torch.empty(shape, device=dev, dtype=dt)
                if fill is not None:
                    t.normal_(generator=fill)
                else:
                    t.zero_()
                store.append(t)
        if self.fused and dev.type == "cuda" and self.rope_table is None:
            from . import glue

            self.rope_table = glue.rope_table(cfg.max_seq, cfg.head_dim, cfg.rope_theta, dev)

    # -- collectives ---------------------------------------------------------------
    def _all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp > 1:
            dist.all_reduce(x, group=self.group)
        return x

    def _all_gather(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp == 1:
            return x
        rows, width = x.shape
        parts = torch.empty(self.tp * rows, width, device=x.device, dtype=x.dtype)
        dist.all_gather_into_tensor(parts, x.contiguous(), group=self.group)
        return parts.view(self.tp, rows, width).permute(1, 0, 2).reshape(rows, self.tp * width)

    # -- one decode step -----------------------------------------------------------
    def step(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        if self.fused:
            return self._step_fused(tokens, positions)
        return self._step_torch(tokens, positions)

    def enable_peer_reduce(self, max_rows: int, protocol: str | None = None) -> None:
        """Replaces each NCCL all-reduce + residual add + norm of the fused route by one
        peer-memory kernel (`linnet_b200.tp.PeerReduce`); collective: every rank calls it."""
        from .tp import PeerReduce

        if self.tp > 1:
            self.peer_reduce = PeerReduce(2 * self.cfg.layers, max_rows, self.cfg.hidden, self.embed.device,
                                          self.group, protocol)

    def _product(self, x: torch.Tensor, weight: Int4, **kwargs) -> torch.Tensor:
        if self.early:
            kwargs["early"] = True
        return self.linear(x, *weight, **kwargs)

    def _reduce_norm(self, site: int, x: torch.Tensor, inputs: torch.Tensor, weight: Int4,
                     norm: torch.Tensor, **kwargs) -> torch.Tensor:
        """x += all_reduce(linear(inputs, weight)); returns rms_norm(x) * norm."""
        from . import glue

        if self.peer_reduce is not None and x.shape[0] <= self.peer_reduce.max_rows:
            self._product(inputs, weight, out=self.peer_reduce.partial(site, x.shape[0]), **kwargs)
            return self.peer_reduce.add_rmsnorm(site, x, norm, self.cfg.eps)
        delta = self._all_reduce(self._product(inputs, weight, **kwargs))
        return glue.add_rmsnorm(x, delta, norm, self.cfg.eps)

    def _step_folded(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """One rank, one or two rows: every residual add + RMS norm runs inside the product that
        consumes it (`kernels.int4_linear_norm`): six launches a layer, five with `fold_swiglu`.  The residual stream alternates between two buffers (every block of a
        product reads the old one while one block writes the new one).  A product
        that does not take its shape runs as the two kernels it stands for."""
        from . import glue, kernels

        cfg = self.cfg
        x = self.embed[tokens]
        spare = torch.empty_like(x)

        def product(delta, norm, weight):
            """linear(rms_norm(x + delta) * norm, weight); the residual stream moves to the other buffer."""
            nonlocal x, spare
            y = kernels.int4_linear_norm(x, delta, norm, cfg.eps, spare, *weight)
            if y is None:  # not a shape of the folding kernel: the two kernels it stands for
                return self.linear(glue.add_rmsnorm(x, delta, norm, cfg.eps), *weight)
            if delta is not None:
                x, spare = spare, x
            return y

        delta = None
        for i, w in enumerate(self.layers):
            qkv = product(delta, w.norm1, w.qkv)
            attn = glue.rope_attention(qkv, positions, self.rope_table, self.cache_k[i], self.cache_v[i],
                                       cfg.heads, cfg.kv_heads)
            gate_up = product(self.linear(attn, *w.o), w.norm2, w.gate_up)
            if self.fold_swiglu:
                delta = self.linear(gate_up, *w.down, swiglu=True)
            else:
                delta = self.linear(glue.silu_mul(gate_up), *w.down)
        return product(delta, self.final_norm, self.head)

    def _step_fused(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        from . import glue

        cfg, tp = self.cfg, self.tp
        if self.fold_norm and tp == 1 and tokens.shape[0] <= 2:
            return self._step_folded(tokens, positions)
        nq, nkv = cfg.heads // tp, cfg.kv_heads // tp
        x = self.embed[tokens]           # the residual stream, updated in place
        h = glue.add_rmsnorm(x, None, self.layers[0].norm1, cfg.eps)
        for i, w in enumerate(self.layers):
            qkv = self._product(h, w.qkv)
            attn = glue.rope_attention(qkv, positions, self.rope_table, self.cache_k[i], self.cache_v[i], nq, nkv)
            h = self._reduce_norm(2 * i, x, attn, w.o, w.norm2)
            following = self.layers[i + 1].norm1 if i + 1 < len(self.layers) else self.final_norm
            if self.fold_swiglu:
                h = self._reduce_norm(2 * i + 1, x, self._product(h, w.gate_up), w.down, following, swiglu=True)
            else:
                act = glue.silu_mul(self._product(h, w.gate_up))
                h = self._reduce_norm(2 * i + 1, x, act, w.down, following)
        return self._all_gather(self._product(h, self.head))

    def _step_torch(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        cfg, tp = self.cfg, self.tp
        nq, nkv, hd = cfg.heads // tp, cfg.kv_heads // tp, cfg.head_dim
        batch = tokens.shape[0]
        rows = torch.arange(batch, device=tokens.device)
        mask = (torch.arange(cfg.max_seq, device=tokens.device)[None, :] <= positions[:, None])[:, None, None, :]
        x = self.embed[tokens]
        for i, w in enumerate(self.layers):
            h = F.rms_norm(x, (cfg.hidden,), w.norm1, cfg.eps)
            qkv = self.linear(h, *w.qkv)
            q, k, v = qkv.split([nq * hd, nkv * hd, nkv * hd], dim=-1)
            q = rotary(q.reshape(batch, nq, hd), positions, cfg.rope_theta)
            k = rotary(k.reshape(batch, nkv, hd), positions, cfg.rope_theta)
            self.cache_k[i][rows, :, positions] = k
            self.cache_v[i][rows, :, positions] = v.reshape(batch, nkv, hd)
            attn = F.scaled_dot_product_attention(q[:, :, None, :], self.cache_k[i], self.cache_v[i],
                                                  attn_mask=mask, enable_gqa=True)
            x = x + self._all_reduce(self.linear(attn.reshape(batch, nq * hd), *w.o))
            h = F.rms_norm(x, (cfg.hidden,), w.norm2, cfg.eps)
            gate_up = self.linear(h, *w.gate_up)
            gate, up = gate_up.split(cfg.mlp // tp, dim=-1)
            x = x + self._all_reduce(self.linear(F.silu(gate) * up, *w.down))
        x = F.rms_norm(x, (cfg.hidden,), self.final_norm, cfg.eps)
        return self._all_gather(self.linear(x, *self.head))


# ---- synthetic model ----------------------------------------------------------------


def random_int4(rows: int, depth: int, group: int, device: torch.device, gen: torch.Generator,
                quantize: Callable[..., tuple]) -> Int4:
    """W ~ N(0, 0.02) [rows, depth] in bf16, quantized int4-g`group`; scales kept as bf16."""
    parts = []
    step = max(1, (1 << 26) // depth)  # bound the temporary to 64 Mi elements
    for r0 in range(0, rows, step):
        w = torch.empty(min(step, rows - r0), depth, device=device, dtype=torch.float32)
        w.normal_(0.0, 0.02, generator=gen)
        packed, _scale, zero, stored = quantize(w.to(torch.bfloat16), group, scale_dtype="bf16")
        parts.append((packed, stored, zero))
    return concat_rows(*parts)


def build_random(cfg: DecoderConfig, device: torch.device, *, rank: int, tp: int, seed: int,
                 linear: Linear, quantize: Callable[..., tuple],
                 group: "dist.ProcessGroup | None" = None) -> Int4Decoder:
    """A rank's shard of a randomly initialised model, generated directly at shard size
    (the benchmark never needs the whole model in one place)."""
    check_tp(cfg, tp)
    gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    hd, H, G = cfg.head_dim, cfg.hidden, cfg.group
    layers = []
    for _ in range(cfg.layers):
        qkv = random_int4((cfg.heads + 2 * cfg.kv_heads) * hd // tp, H, G, device, gen, quantize)
        o = random_int4(H, cfg.heads * hd // tp, G, device, gen, quantize)
        gate_up = random_int4(2 * cfg.mlp // tp, H, G, device, gen, quantize)
        down = random_int4(H, cfg.mlp // tp, G, device, gen, quantize)
        ones = torch.ones(H, device=device, dtype=torch.bfloat16)
        layers.append(LayerWeights(qkv, o, gate_up, down, ones, ones.clone()))
    shared = torch.Generator(device=device).manual_seed(seed)  # replicated tensors: same on every rank
    embed = torch.empty(cfg.vocab, H, device=device, dtype=torch.bfloat16).normal_(0.0, 0.02, generator=shared)
    head = random_int4(cfg.vocab // tp, H, G, device, gen, quantize)
    return Int4Decoder(cfg, layers, embed, torch.ones(H, device=device, dtype=torch.bfloat16), head,
                       linear=linear, rank=rank, tp=tp, group=group)


def decode_bytes(cfg: DecoderConfig, batch: int, tp: int) -> int:
    """Algorithmic HBM bytes one rank reads per decode step: its int4 weights (0.5234 B
    per weight at g128) plus its share of the KV cache."""
    weights = cfg.int4_elements() * (0.5 + 3.0 / cfg.group) / tp
    kv = batch * cfg.layers * 2 * cfg.kv_heads * cfg.max_seq * cfg.head_dim * 2 / tp
    return int(weights + kv)


def bench(args, rank: int, world: int, device: torch.device, barrier, reduce_max, clocks_cls) -> dict:
    """The decode workload of bench.py: tokens/s of one CUDA-graph-replayed decode step
    at batch `args.batch` (and 1 / 8 / 64 under `per_batch`), tensor-parallel over all
    ranks."""
    import json
    from pathlib import Path

    from . import kernels, quant

    cfg = DecoderConfig.llama31_8b()
    model = build_random(cfg, device, rank=rank, tp=world, seed=0, linear=kernels.int4_linear,
                         quantize=quant.quantize_int4_groups)
    model.early = bool(getattr(args, "early", False))
    model.fold_swiglu = bool(getattr(args, "fold_swiglu", False))
    model.fold_norm = not getattr(args, "no_fold_norm", False)
    results: dict[int, dict] = {}
    nccl_results: dict[int, dict] = {}
    kept_logits: dict[tuple[str, int], torch.Tensor] = {}  # one step's logits per route and batch
    clocks = None
    stream = torch.cuda.Stream(device)
    batches = [args.batch]
    if not getattr(args, "single_batch", False):
        batches += [b for b in (1, 8, 64) if b != args.batch]
    e2e = {}
    route = getattr(args, "reduce", "peer") if world > 1 else "none"
    peer_reduce = None
    peer_unavailable = None
    if route == "peer":
        try:
            model.enable_peer_reduce(max(batches), getattr(args, "peer_protocol", None))
            peer_reduce = model.peer_reduce
        except Exception as exc:  # no symmetric memory on this box: the NCCL route is the product then
            peer_unavailable = f"{type(exc).__name__}: {exc}"[:200]
            route = "nccl"
    # With the peer route on, the NCCL route is timed beside it (it is the baseline the
    # fused kernel has to beat); the headline numbers are the selected route's.
    passes = [(route, batches)] + ([("nccl", sorted(set(batches)))] if route == "peer" else [])
    with torch.cuda.stream(stream):
        for which, batch in [(w, b) for w, bs in passes for b in bs]:
            headline = which == route
            model.peer_reduce = peer_reduce if which == "peer" else None
            fill = torch.Generator(device=device).manual_seed(7 + rank)
            model.allocate_cache(batch, fill)
            tok_gen = torch.Generator().manual_seed(11)
            host_tokens = torch.randint(0, cfg.vocab, (batch,), generator=tok_gen).pin_memory()
            tokens = host_tokens.to(device)
            positions = torch.full((batch,), cfg.max_seq - 1, device=device, dtype=torch.long)
            for _ in range(2):
                logits = model.step(tokens, positions)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                logits = model.step(tokens, positions)
                sampled = logits.argmax(dim=-1)  # greedy sampling stays on the device, inside the graph
            main = headline and batch == args.batch
            steps = args.steps if main else max(5, args.steps // 4)
            for _ in range(max(3, args.warmup if main else 3)):
                graph.replay()
            torch.cuda.synchronize()
            kept_logits[(which, batch)] = logits.float().clone()
            barrier()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

            def timed() -> float:
                torch.cuda.synchronize()
                start.record()
                for _ in range(steps):
                    graph.replay()
                stop.record()
                torch.cuda.synchronize()
                return start.elapsed_time(stop)

            if main:
                with clocks_cls(device.index or 0) as clocks:
                    ms = timed()
            else:
                ms = timed()
            barrier()
            ms_step = reduce_max(ms) / steps
            (results if headline else nccl_results)[batch] = {"tok_s": batch / (ms_step / 1e3), "ms_per_step": ms_step,
                              "GB_s_per_gpu": decode_bytes(cfg, batch, world) / (ms_step / 1e3) / 1e9}
            if main:
                # End to end, as the reference's serving loop runs a step (python/linnet/src/linnet/
                # serve/__init__.py:1606-1618, :1657-1681): token ids go in from pinned host memory,
                # the step and its sampling replay as one graph, the sampled ids are copied to
                # pinned host memory behind it, and the host reads them one step behind (it waits
                # for step i - 1's copy while step i runs).
                host_out = [torch.empty(batch, dtype=torch.long).pin_memory() for _ in range(2)]
                done = [torch.cuda.Event(), torch.cuda.Event()]
                checksum = 0
                barrier()
                t0 = time.perf_counter()
                for i in range(steps):
                    tokens.copy_(host_tokens, non_blocking=True)
                    graph.replay()
                    host_out[i % 2].copy_(sampled, non_blocking=True)
                    done[i % 2].record()
                    if i > 0:
                        done[(i - 1) % 2].synchronize()
                        checksum += int(host_out[(i - 1) % 2][0])
                done[(steps - 1) % 2].synchronize()
                checksum += int(host_out[(steps - 1) % 2][0])
                ms_e2e = reduce_max((time.perf_counter() - t0) * 1e3) / steps
                e2e = {"value": batch / (ms_e2e / 1e3), "unit": "tok/s", "ms_per_step": ms_e2e,
                       "h2d_bytes_per_step": batch * 8, "d2h_bytes_per_step": batch * 8,
                       "how": "ids from pinned host memory, one graph replay (step + argmax), sampled ids to "
                              "pinned host memory, read one step behind", "checksum": checksum}
            del graph, logits, sampled
            model.cache_k, model.cache_v = [], []
            torch.cuda.empty_cache()
    peaks_path = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text())["hbm_gbs"]) if peaks_path.exists() else 6650.0
    if peer_reduce is not None and peer_reduce.error():
        raise RuntimeError(f"peer reduction gave up waiting for a rank (code {peer_reduce.error()})")
    # The peer route against the NCCL route on the same step (same weights, cache and tokens):
    # parity of the multi-GPU reduction, carried by every multi-GPU bench line.
    peer_vs_nccl = None
    if nccl_results:
        worst, scale_of = 0.0, 0.0
        per_batch_diff = {}
        for batch in sorted(nccl_results):
            a, b = kept_logits[(route, batch)], kept_logits[("nccl", batch)]
            diff, top = float((a - b).abs().max()), float(b.abs().max())
            per_batch_diff[str(batch)] = {"max_abs": diff, "max_logit": top}
            worst, scale_of = max(worst, diff / max(top, 1e-6)), max(scale_of, top)
        worst = reduce_max(worst)
        # On 2 ranks both routes add the same two numbers (difference 0).  From 3 ranks on NCCL rounds
        # its partial sums to bf16 in an order of its own while the kernel sums in f32 in rank order
        # and rounds once; through 32 layers of a random network that grows to a few percent of the
        # largest logit (0.054 measured on 4 ranks).  The bound catches a broken reduction (missing
        # or doubled rank: O(1)), not rounding; bit-exactness of the kernel itself is a test
        # (tests/test_tp_peer_reduce.py).
        tolerance = 0.25
        peer_vs_nccl = {"peer_vs_nccl_max_abs_over_max_logit": worst, "tolerance": tolerance, "ok": worst <= tolerance,
                        "per_batch": per_batch_diff}
        if not peer_vs_nccl["ok"]:
            raise SystemExit(f"peer-memory reduction and NCCL disagree: {peer_vs_nccl}")
    main = results[args.batch]
    # per layer: 4 linears, 2 (reduce +) add + norm, rotary + cache write + attention, silu*mul;
    # then the first norm and the output head
    launches_per_step = cfg.layers * 8 + 2
    return {
        "metric": "W4A16 g128 GEMV GB/s (% HBM peak); 8B-shape int4 decode tok/s at 1/2/4/8 GPU",
        "value": main["tok_s"], "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": main["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "int4 weights, bf16 activations and KV cache, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"Llama-3.1-8B-shaped int4-g128 decoder, decode batch {args.batch}, "
                               f"2048-token bf16 KV cache, tensor parallel {world}",
                   "parallelism": f"tp{world}", "layers": cfg.layers, "hidden": cfg.hidden,
                   "l2_policy": "inputs larger than L2: 3.9 GB of weights / tp per step",
                   "timing": "CUDA events around CUDA-graph replays, max over ranks"},
        "roofline": {"bound": "hbm", "achieved": main["GB_s_per_gpu"], "peak": peak, "unit": "GB/s",
                     "frac": main["GB_s_per_gpu"] / peak,
                     "peak_kind": "measured" if peaks_path.exists() else "fallback",
                     "algorithmic_bytes_per_step_per_gpu": decode_bytes(cfg, args.batch, world),
                     "traffic": None},
        "per_batch": {str(b): results[b] for b in sorted(results)},
        "reduce_route": {"none": "single GPU: no reduction",
                         "peer": "one peer-memory kernel per row-split layer: all-reduce + residual add + RMSNorm"
                                 + (f" ({peer_reduce.protocol} exchange)" if peer_reduce is not None else ""),
                         "nccl": "NCCL all-reduce, then the add + RMSNorm kernel"}[route],
        **({"per_batch_nccl_route": {str(b): nccl_results[b] for b in sorted(nccl_results)}}
           if nccl_results else {}),
        **({"peer_reduce_unavailable": peer_unavailable} if peer_unavailable else {}),
        **({"peer_vs_nccl": peer_vs_nccl} if peer_vs_nccl else {}),
        "e2e": e2e,
        "gpu_launches": args.steps * launches_per_step,
        "clocks": clocks.summary() if clocks else None,
    }
