"""Builds a tiny whole model on the CPU with the oracle quantizer and shards it, for
the decoder tests."""

from __future__ import annotations

import torch

from linnet_b200 import decoder as dec
from oracle import linear_oracle as lo
from oracle import quant_oracle as qo


def quantized(rows: int, depth: int, group: int, gen: torch.Generator) -> dec.Int4:
    w = torch.randn(rows, depth, generator=gen) * 0.05
    packed, scale, zero = qo.quantize_int4_groups(w.numpy(), group)
    return (torch.from_numpy(packed), torch.from_numpy(scale).to(torch.bfloat16), torch.from_numpy(zero))


def whole_model(cfg: dec.DecoderConfig, seed: int = 0) -> dict:
    gen = torch.Generator().manual_seed(seed)
    hd, H, G = cfg.head_dim, cfg.hidden, cfg.group
    layers = []
    for _ in range(cfg.layers):
        layers.append(dict(
            q=quantized(cfg.heads * hd, H, G, gen), k=quantized(cfg.kv_heads * hd, H, G, gen),
            v=quantized(cfg.kv_heads * hd, H, G, gen), o=quantized(H, cfg.heads * hd, G, gen),
            gate=quantized(cfg.mlp, H, G, gen), up=quantized(cfg.mlp, H, G, gen),
            down=quantized(H, cfg.mlp, G, gen),
            norm1=(1 + 0.1 * torch.randn(H, generator=gen)).to(torch.bfloat16),
            norm2=(1 + 0.1 * torch.randn(H, generator=gen)).to(torch.bfloat16)))
    return dict(layers=layers, embed=(torch.randn(cfg.vocab, H, generator=gen) * 0.5).to(torch.bfloat16),
                final_norm=torch.ones(H, dtype=torch.bfloat16), head=quantized(cfg.vocab, H, G, gen))


def rank_model(cfg, whole, rank, tp, linear, device="cpu", group=None) -> dec.Int4Decoder:
    def to(t):
        return tuple(x.to(device) for x in t) if isinstance(t, tuple) else t.to(device)

    layers = []
    for L in whole["layers"]:
        w = dec.shard_layer(cfg, L["q"], L["k"], L["v"], L["o"], L["gate"], L["up"], L["down"],
                            L["norm1"], L["norm2"], rank, tp)
        layers.append(dec.LayerWeights(to(w.qkv), to(w.o), to(w.gate_up), to(w.down), to(w.norm1), to(w.norm2)))
    return dec.Int4Decoder(cfg, layers, to(whole["embed"]), to(whole["final_norm"]),
                           to(dec.shard_rows(whole["head"], rank, tp)), linear=linear, rank=rank, tp=tp,
                           group=group)


def oracle_linear(x, packed, scale, zero):
    return lo.int4_groups_linear(x, packed, scale, zero)


def run_steps(model: dec.Int4Decoder, cfg, batch: int, steps: int, device="cpu") -> torch.Tensor:
    """A few decode steps from an empty cache; returns the last logits."""
    model.allocate_cache(batch)
    gen = torch.Generator().manual_seed(3)
    logits = None
    for t in range(steps):
        tokens = torch.randint(0, cfg.vocab, (batch,), generator=gen).to(device)
        positions = torch.full((batch,), t, dtype=torch.long, device=device)
        logits = model.step(tokens, positions)
    return logits
