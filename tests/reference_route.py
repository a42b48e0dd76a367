"""Runs cards of quantized layers through the reference's own loader, `linnet.torch.load`,
once as the reference alone on a CPU and once with this package installed into it, and saves
what each computed.  `tests/test_reference_route.py` starts this file twice as a script (two
processes, because both sides register the same `linnet::` operator names) and compares:

    python tests/reference_route.py reference <dir>            # the reference itself, CPU
    python tests/reference_route.py ours <dir> --device cuda    # install() first, B200 kernels
    python tests/reference_route.py ours <dir> --device cpu --stub
        # install() first, CPU tensors, the kernels replaced by the CPU oracle: exercises the
        # loader hooks (generated source, interpreter, prepare, siblings, weight refresh)
        # where there is no GPU.  Test scaffolding only: the product has no CPU path.

The process must see the reference (`oracle/_ref`, made by `python -m oracle.build_ref`)
through `LINNET_BIN`, `LINNET_STD`, `LINNET_HOME` and `PYTHONPATH`
(`oracle.build_ref.environment`).

Cards and what they pin (reference tests they mirror in brackets):
  lin4      Int4GroupLinear, K=4096 N=14336 g128 bf16, rows 1/4/16/160: the headline shape
            through every row-count route [python/linnet/tests/test_quant_groups.py:81-162]
  lin8      Int8Linear 4096x4096 rows 1/40 (config 1) and Int8GroupLinear g128 rows 1/5
            [tests/test_quant_8bit.py:134-148]
  siblings  three Int8Linear projections of one input, which the generated source joins into
            one product [tests/test_quant_8bit.py:195-216; src/backend/torch_source.cpp:82-159]
  refresh   copy_weights() into a loaded int4 model, then the same call again: prepared
            values are rewritten in place [python/linnet/src/linnet/torch/compiled.py:539-564]
  llama4    the Llama example card (examples/01-llama) with its linears replaced by
            Int4GroupLinear, 2 layers, 3 decode steps of a batch of 2; the same weights also
            go to `linnet_b200.decoder.Int4Decoder` [tests/torch/test_shards.py:47-129 pattern]
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

LIN4 = """module route.lin4
use std.quant::{Int4GroupLinear}
pub block Model<In: Dim, Out: Dim, Group: Dim, T: Float = bf16>
where Group > 0, Group % 2 == 0, In % Group == 0
{
    sub proj: Int4GroupLinear<In, Out, Group, T>
    pub entry forward<B: Dim>(x: Tensor[B, In; T]) -> Tensor[B, Out; T] {
        return proj.forward(x)
    }
}
"""

LIN8 = """module route.lin8
use std.quant::{Int8Linear, Int8GroupLinear}
pub block Model<In: Dim, Out: Dim, Group: Dim, T: Float = bf16>
where Group > 0, In % Group == 0
{
    sub rows: Int8Linear<In, Out, T>
    sub groups: Int8GroupLinear<In, Out, Group, T>
    pub entry by_rows<B: Dim>(x: Tensor[B, In; T]) -> Tensor[B, Out; T] {
        return rows.forward(x)
    }
    pub entry by_groups<B: Dim>(x: Tensor[B, In; T]) -> Tensor[B, Out; T] {
        return groups.forward(x)
    }
}
"""

SIBLINGS = """module route.siblings
use std.quant::{Int8Linear}
pub block Model<In: Dim, Q: Dim, Kv: Dim, T: Float = bf16>
{
    sub q: Int8Linear<In, Q, T>
    sub k: Int8Linear<In, Kv, T>
    sub v: Int8Linear<In, Kv, T>
    pub entry forward<B: Dim>(x: Tensor[B, In; T]) -> (Tensor[B, Q; T], Tensor[B, Kv; T], Tensor[B, Kv; T]) {
        return (q.forward(x), k.forward(x), v.forward(x))
    }
}
"""

# The reference's Llama example (examples/01-llama/src/lib.linnet and attention.linnet) with
# every `Linear` replaced by `Int4GroupLinear<..., 128, T>`; rope tables and attention are the
# example's own modules, used unchanged from the copy under oracle/_ref.
LLAMA4 = """module llama4
use crate.rope::{THETA, tables}
use std.nn.attention::{grouped_attention}
use std.nn.cache::{write_at}
use std.nn.activations::{silu}
use std.nn.embedding::{Embedding}
use std.nn.norm::{RmsNorm}
use std.nn.rope::{rope}
use std.quant::{Int4GroupLinear}

block Attention<H: Dim, Heads: Dim, KvHeads: Dim, Batch: Dim, MaxSeq: Dim, T: Float>
where Heads > 0, KvHeads > 0, H % Heads == 0, Heads % KvHeads == 0, (H / Heads) % 2 == 0, MaxSeq > 0,
      H % 128 == 0
{
    sub q_proj: Int4GroupLinear<H, H, 128, T>
    sub k_proj: Int4GroupLinear<H, KvHeads * (H / Heads), 128, T>
    sub v_proj: Int4GroupLinear<H, KvHeads * (H / Heads), 128, T>
    sub o_proj: Int4GroupLinear<H, H, 128, T>
    state cache_k: Tensor[Batch, KvHeads, MaxSeq, H / Heads; T]
    state cache_v: Tensor[Batch, KvHeads, MaxSeq, H / Heads; T]

    pub fn decode(x: Tensor[Batch, 1, H; T], pos: i32) -> Tensor[Batch, 1, H; T] {
        let (cos_table, sin_table) = tables<MaxSeq, H / Heads, T>(THETA)
        let cos_at[d] = cos_table[cast<i64>(pos), d]
        let sin_at[d] = sin_table[cast<i64>(pos), d]
        let cos_row = reshape(cos_at, [1, H / Heads])
        let sin_row = reshape(sin_at, [1, H / Heads])
        let q = rope(heads<Batch, 1, Heads, H / Heads, T>(q_proj.forward(x)), cos_row, sin_row)
        let k = rope(heads<Batch, 1, KvHeads, H / Heads, T>(k_proj.forward(x)), cos_row, sin_row)
        let v = heads<Batch, 1, KvHeads, H / Heads, T>(v_proj.forward(x))
        cache_k = write_at(cache_k, k, pos)
        cache_v = write_at(cache_v, v, pos)
        let positions = iota<i32>(MaxSeq)
        let seen[s] = positions[s] <= pos
        let mixed = grouped_attention(q, cache_k, cache_v, rsqrt(cast<f32>(H / Heads)),
                                      some(reshape(seen, [1, MaxSeq])))
        return o_proj.forward(reshape(permute(mixed, [0, 2, 1, 3]), [Batch, 1, H]))
    }
}

fn heads<B: Dim, S: Dim, N: Dim, D: Dim, T: Float>(x: Tensor[B, S, N * D; T]) -> Tensor[B, N, S, D; T] {
    return permute(reshape(x, [B, S, N, D]), [0, 2, 1, 3])
}

block Mlp<H: Dim, Inner: Dim, T: Float>
where H % 128 == 0, Inner % 128 == 0
{
    sub gate: Int4GroupLinear<H, Inner, 128, T>
    sub up: Int4GroupLinear<H, Inner, 128, T>
    sub down: Int4GroupLinear<Inner, H, 128, T>
    pub fn forward<*S: Shape>(x: Tensor[*S, H; T]) -> Tensor[*S, H; T] {
        return down.forward(silu(gate.forward(x)) * up.forward(x))
    }
}

block Layer<H: Dim, Heads: Dim, KvHeads: Dim, Inner: Dim, Batch: Dim, MaxSeq: Dim, T: Float>
where Heads > 0, KvHeads > 0, H % Heads == 0, Heads % KvHeads == 0, (H / Heads) % 2 == 0, MaxSeq > 0,
      H % 128 == 0, Inner % 128 == 0
{
    sub attention_norm: RmsNorm<H, T>
    sub attention: Attention<H, Heads, KvHeads, Batch, MaxSeq, T>
    sub mlp_norm: RmsNorm<H, T>
    sub mlp: Mlp<H, Inner, T>
    pub fn decode(x: Tensor[Batch, 1, H; T], pos: i32) -> Tensor[Batch, 1, H; T] {
        let attended = x + attention.decode(attention_norm.forward(x), pos)
        return attended + mlp.forward(mlp_norm.forward(attended))
    }
}

pub block Model<Vocab: Dim, H: Dim, Heads: Dim, KvHeads: Dim, Inner: Dim, Layers: Dim, Batch: Dim,
                MaxSeq: Dim, T: Float = bf16>
where Heads > 0, KvHeads > 0, H % Heads == 0, Heads % KvHeads == 0, (H / Heads) % 2 == 0, MaxSeq > 0,
      H % 128 == 0, Inner % 128 == 0
{
    sub embedding: Embedding<Vocab, H, T>
    sub layers: [Layer<H, Heads, KvHeads, Inner, Batch, MaxSeq, T>; Layers]
    sub norm: RmsNorm<H, T>
    sub lm_head: Int4GroupLinear<H, Vocab, 128, T>

    pub entry decode(token: Tensor[Batch, 1; i32], pos: i32) -> Tensor[Batch, Vocab; T] {
        var x = embedding.forward(token)
        static for layer in layers {
            x = layer.decode(x, pos)
        }
        return lm_head.forward(norm.forward(x[:, 0, :]))
    }
}
"""

LLAMA_GENERICS = {"Vocab": 512, "H": 256, "Heads": 4, "KvHeads": 2, "Inner": 512, "Layers": 2, "Batch": 2,
                  "MaxSeq": 32, "T": "bf16"}
LIN4_GENERICS = {"In": 4096, "Out": 14336, "Group": 128, "T": "bf16"}
LIN8_GENERICS = {"In": 4096, "Out": 4096, "Group": 128, "T": "bf16"}
SIB_GENERICS = {"In": 512, "Q": 256, "Kv": 128, "T": "bf16"}
SMALL4_GENERICS = {"In": 256, "Out": 64, "Group": 128, "T": "bf16"}


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 results as their 16-bit patterns (NumPy has no bf16)."""
    return t.detach().to(torch.bfloat16).cpu().contiguous().view(torch.int16).numpy()


# ---- inputs and checkpoints: made once, by the reference process -------------------------------


def make_files(work: Path) -> None:
    """Cards, seeded checkpoints (quantized by the reference's own `linnet.quant`) and inputs."""
    from linnet import quant
    from safetensors.torch import save_file

    work.mkdir(parents=True, exist_ok=True)
    for name, text in (("lin4", LIN4), ("lin8", LIN8), ("siblings", SIBLINGS)):
        (work / f"{name}.linnet").write_text(text, encoding="utf-8")
    # the Llama card is a two-file package: `crate.rope` is the example's own rope.linnet
    package = work / "llama4"
    (package / "src").mkdir(parents=True, exist_ok=True)
    (package / "src" / "lib.linnet").write_text(LLAMA4, encoding="utf-8")
    import os
    example = Path(os.environ["LINNET_STD"]).parent / "examples" / "01-llama"
    (package / "src" / "rope.linnet").write_text((example / "src" / "rope.linnet").read_text(encoding="utf-8"),
                                                   encoding="utf-8")
    (package / "linnet.toml").write_text((example / "linnet.toml").read_text(encoding="utf-8").replace(
        'name = "llama"', 'name = "llama4"'), encoding="utf-8")

    gen = torch.Generator().manual_seed(0)

    def int4(prefix: str, out: int, depth: int, tensors: dict, std: float = 0.02) -> None:
        w = (torch.randn(out, depth, generator=gen) * std).numpy()
        packed, scale, zero = quant.quantize_int4_groups(w, 128)
        tensors[prefix + "weight"] = torch.from_numpy(packed)
        tensors[prefix + "scale"] = torch.from_numpy(scale).to(torch.bfloat16)
        tensors[prefix + "zero"] = torch.from_numpy(zero)

    def int8(prefix: str, out: int, depth: int, group: int, tensors: dict) -> None:
        w = (torch.randn(out, depth, generator=gen) * 0.02).numpy()
        q, scale = quant.quantize_int8_groups(w, group, "bf16")
        tensors[prefix + "weight"] = torch.from_numpy(q)
        tensors[prefix + "scale"] = torch.from_numpy(scale).to(torch.bfloat16)

    t: dict = {}
    int4("proj.", 14336, 4096, t)
    save_file(t, str(work / "lin4.safetensors"))
    t = {}
    int8("rows.", 4096, 4096, 4096, t)
    int8("groups.", 4096, 4096, 128, t)
    save_file(t, str(work / "lin8.safetensors"))
    t = {}
    int8("q.", 256, 512, 512, t)
    int8("k.", 128, 512, 512, t)
    int8("v.", 128, 512, 512, t)
    save_file(t, str(work / "siblings.safetensors"))
    for name in ("small_a", "small_b"):
        t = {}
        int4("proj.", 64, 256, t)
        save_file(t, str(work / f"{name}.safetensors"))
    g = LLAMA_GENERICS
    hd = g["H"] // g["Heads"]
    t = {"embedding.weight": (torch.randn(g["Vocab"], g["H"], generator=gen) * 0.5).to(torch.bfloat16),
         "norm.weight": (1 + 0.1 * torch.randn(g["H"], generator=gen)).to(torch.bfloat16)}
    for layer in range(g["Layers"]):
        p = f"layers.{layer}."
        t[p + "attention_norm.weight"] = (1 + 0.1 * torch.randn(g["H"], generator=gen)).to(torch.bfloat16)
        t[p + "mlp_norm.weight"] = (1 + 0.1 * torch.randn(g["H"], generator=gen)).to(torch.bfloat16)
        int4(p + "attention.q_proj.", g["H"], g["H"], t, 0.06)
        int4(p + "attention.k_proj.", g["KvHeads"] * hd, g["H"], t, 0.06)
        int4(p + "attention.v_proj.", g["KvHeads"] * hd, g["H"], t, 0.06)
        int4(p + "attention.o_proj.", g["H"], g["H"], t, 0.06)
        int4(p + "mlp.gate.", g["Inner"], g["H"], t, 0.06)
        int4(p + "mlp.up.", g["Inner"], g["H"], t, 0.06)
        int4(p + "mlp.down.", g["H"], g["Inner"], t, 0.06)
    int4("lm_head.", g["Vocab"], g["H"], t, 0.06)
    save_file(t, str(work / "llama4.safetensors"))

    inputs = {}
    for rows in (1, 4, 16, 160):
        inputs[f"lin4/x{rows}"] = bits(torch.randn(rows, 4096, generator=gen))
    for rows in (1, 5, 40):
        inputs[f"lin8/x{rows}"] = bits(torch.randn(rows, 4096, generator=gen))
    for rows in (1, 3):
        inputs[f"siblings/x{rows}"] = bits(torch.randn(rows, 512, generator=gen))
    inputs["refresh/x"] = bits(torch.randn(3, 256, generator=gen))
    inputs["llama4/tokens"] = torch.randint(0, g["Vocab"], (3, g["Batch"], 1), generator=gen).to(torch.int32).numpy()
    np.savez(work / "inputs.npz", **inputs)


def bf16(array: np.ndarray, device: str) -> torch.Tensor:
    return torch.from_numpy(array.copy()).view(torch.bfloat16).to(device)


# ---- the run, the same code on both sides ------------------------------------------------------


def run_cards(work: Path, device: str, modes: list, out: dict, std: str) -> None:
    import linnet.torch as lt

    inputs = np.load(work / "inputs.npz")

    def load(card: str, generics: dict, weights: str, mode, source: Path | None = None):
        return lt.load(source or work / f"{card}.linnet", generics=generics, std_root=std,
                       weights=work / f"{weights}.safetensors", device=device, compile=mode)

    for mode in modes:
        tag = {False: "interp", True: "source"}.get(mode, str(mode))
        model = load("lin4", LIN4_GENERICS, "lin4", mode)
        for rows in (1, 4, 16, 160):
            out[f"{tag}/lin4/y{rows}"] = bits(model.run_entry("forward", [bf16(inputs[f"lin4/x{rows}"], device)]))
        del model
        model = load("lin8", LIN8_GENERICS, "lin8", mode)
        for rows in (1, 40):
            out[f"{tag}/lin8/rows{rows}"] = bits(model.run_entry("by_rows", [bf16(inputs[f"lin8/x{rows}"], device)]))
        for rows in (1, 5):
            out[f"{tag}/lin8/groups{rows}"] = bits(model.run_entry("by_groups", [bf16(inputs[f"lin8/x{rows}"], device)]))
        del model
        model = load("siblings", SIB_GENERICS, "siblings", mode)
        for rows in (1, 3):
            q, k, v = model.run_entry("forward", [bf16(inputs[f"siblings/x{rows}"], device)])
            out[f"{tag}/siblings/q{rows}"], out[f"{tag}/siblings/k{rows}"] = bits(q), bits(k)
            out[f"{tag}/siblings/v{rows}"] = bits(v)
        del model
        # weights replaced in a model that has already run: the prepared values must follow
        model = load("lin4", SMALL4_GENERICS, "small_a", mode)
        other = load("lin4", SMALL4_GENERICS, "small_b", mode)
        x = bf16(inputs["refresh/x"], device)
        out[f"{tag}/refresh/before"] = bits(model.run_entry("forward", [x]))
        model.copy_weights(other)
        out[f"{tag}/refresh/after"] = bits(model.run_entry("forward", [x]))
        out[f"{tag}/refresh/other"] = bits(other.run_entry("forward", [x]))
        del model, other
        model = load("llama4", LLAMA_GENERICS, "llama4", mode, source=work / "llama4" / "src" / "lib.linnet")
        tokens = torch.from_numpy(inputs["llama4/tokens"]).to(device)
        for step in range(3):
            logits = model.run_entry("decode", [tokens[step], torch.tensor(step, dtype=torch.int32, device=device)])
            out[f"{tag}/llama4/logits{step}"] = bits(logits)
        del model


def run_plans(work: Path, device: str, out: dict, std: str, any_device: bool) -> None:
    """The same cards through the reference's planner with `linnet_b200.backend.B200Quant` as
    the only backend (docs/backends.md): `plan_for(..., measure=False)` gives it every region it
    matches, `plan.run` runs them, `conform` compares each region with the generated source."""
    import linnet.torch as lt

    from linnet_b200 import backend as plug

    inputs = np.load(work / "inputs.npz")
    executed = {"count": 0}
    inner = plug._QuantLinear.execute

    def counted(self, *args, **kwargs):
        executed["count"] += 1
        return inner(self, *args, **kwargs)

    plug._QuantLinear.execute = counted
    backend = plug.B200Quant(any_device=any_device)

    def load(card: str, generics: dict, weights: str, source: Path | None = None):
        return lt.load(source or work / f"{card}.linnet", generics=generics, std_root=std,
                       weights=work / f"{weights}.safetensors", device=device, compile=True)

    def through_plan(model, entry: str, args: list, name: str) -> None:
        plan = model.plan_for(entry, args, backends=[backend], measure=False)
        made = plan.run(args, model.context_for(plan))
        out[f"plan/{name}"] = bits(made[0])
        findings = list(model.conform(entry, args, backend))
        out[f"plan/{name}/regions"] = np.array([len(findings)])
        out[f"plan/{name}/conform"] = np.array([bool(f.passed) for f in findings])

    model = load("lin4", LIN4_GENERICS, "lin4")
    for rows in (1, 16):
        through_plan(model, "forward", [bf16(inputs[f"lin4/x{rows}"], device)], f"lin4/y{rows}")
    del model
    model = load("lin8", LIN8_GENERICS, "lin8")
    through_plan(model, "by_rows", [bf16(inputs["lin8/x1"], device)], "lin8/rows1")
    through_plan(model, "by_groups", [bf16(inputs["lin8/x5"], device)], "lin8/groups5")
    del model
    model = load("llama4", LLAMA_GENERICS, "llama4", source=work / "llama4" / "src" / "lib.linnet")
    tokens = torch.from_numpy(inputs["llama4/tokens"]).to(device)
    first = [tokens[0], torch.tensor(0, dtype=torch.int32, device=device)]
    plan = model.plan_for("decode", first, backends=[backend], measure=False)
    context = model.context_for(plan)
    for step in range(3):
        logits = plan.run([tokens[step], torch.tensor(step, dtype=torch.int32, device=device)], context)[0]
        out[f"plan/llama4/logits{step}"] = bits(logits)
    out["plan/executed"] = np.array([executed["count"]])
    plug._QuantLinear.execute = inner


def run_decoder(work: Path, device: str, out: dict, linear, fused: bool | None) -> None:
    """The same Llama checkpoint through `linnet_b200.decoder.Int4Decoder`."""
    from safetensors.torch import load_file

    from linnet_b200 import decoder as dec

    g = LLAMA_GENERICS
    cfg = dec.DecoderConfig(layers=g["Layers"], hidden=g["H"], heads=g["Heads"], kv_heads=g["KvHeads"],
                            head_dim=g["H"] // g["Heads"], mlp=g["Inner"], vocab=g["Vocab"], max_seq=g["MaxSeq"],
                            eps=1e-5)
    t = {k: v.to(device) for k, v in load_file(str(work / "llama4.safetensors")).items()}

    def int4(prefix: str):
        return (t[prefix + "weight"], t[prefix + "scale"], t[prefix + "zero"])

    layers = []
    for layer in range(g["Layers"]):
        p = f"layers.{layer}."
        layers.append(dec.shard_layer(cfg, int4(p + "attention.q_proj."), int4(p + "attention.k_proj."),
                                      int4(p + "attention.v_proj."), int4(p + "attention.o_proj."),
                                      int4(p + "mlp.gate."), int4(p + "mlp.up."), int4(p + "mlp.down."),
                                      t[p + "attention_norm.weight"], t[p + "mlp_norm.weight"], 0, 1))
    model = dec.Int4Decoder(cfg, layers, t["embedding.weight"], t["norm.weight"], int4("lm_head."), linear=linear,
                            fused=fused)
    model.allocate_cache(g["Batch"])
    tokens = torch.from_numpy(np.load(work / "inputs.npz")["llama4/tokens"]).to(device)
    for step in range(3):
        positions = torch.full((g["Batch"],), step, dtype=torch.long, device=device)
        out[f"decoder/llama4/logits{step}"] = bits(model.step(tokens[step, :, 0].long(), positions))


CALLS: dict[str, int] = {}


def count_calls() -> None:
    """Wraps the entry points the reference is supposed to reach in this package with
    counters, so that a run can show it went through them."""
    from linnet_b200 import int4, kernels, quantized

    def counted(module, name: str) -> None:
        inner = getattr(module, name)

        def wrapper(*args, **kwargs):
            CALLS[name] = CALLS.get(name, 0) + 1
            return inner(*args, **kwargs)

        wrapper.__name__ = name
        setattr(module, name, wrapper)

    counted(int4, "_int4_pack")
    counted(int4, "_int4_linear")
    counted(quantized, "int8_operands")
    counted(quantized, "int8_linear")
    counted(quantized, "int8_group_operands")
    counted(quantized, "int8_group_linear")
    counted(kernels, "_int4_linear")
    counted(kernels, "_eight_bit")


def stub_kernels() -> None:
    """CPU stand-ins for the CUDA kernels, from the oracle: lets a machine without a GPU drive
    install() and the reference's loader hooks end to end.  Never part of the product."""
    from linnet_b200 import int4, kernels, quantized
    from oracle import linear_oracle as lo

    def int4_linear(x, packed, scale, zero, out=None, early=False, swiglu=False, overlap=True):
        if swiglu:
            half = x.shape[-1] // 2
            x = torch.nn.functional.silu(x[..., :half]) * x[..., half:]
        y = lo.int4_groups_linear(x, packed, scale, zero)
        return y if out is None else out.copy_(y)

    def eight_bit(who, x, weight, scale, fp8, group, row_block):
        return lo.int8_linear(x, weight, scale) if group == 0 else lo.int8_group_linear(x, weight, scale)

    kernels._int4_linear = int4_linear
    kernels._eight_bit = eight_bit
    kernels.int4_dequantize = lambda p, s, z: lo.int4_weight(p, s, z, s.dtype)
    int4._int4_pack = lambda packed, scale, zero: (packed.contiguous(), scale.contiguous(), zero.contiguous())
    quantized._require = lambda x, who: None


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("role", choices=["reference", "ours"])
    parser.add_argument("work", type=Path)
    parser.add_argument("--device", default="cpu")
    parser.add_argument("--stub", action="store_true")
    args = parser.parse_args()
    import os

    std = os.environ["LINNET_STD"]
    out: dict = {}
    if args.role == "reference":
        make_files(args.work)
        run_cards(args.work, "cpu", [False, True], out, std)
        np.savez(args.work / "reference.npz", **out)
        return
    from linnet_b200 import install, kernels

    if args.stub:
        stub_kernels()
    count_calls()
    install.install()
    if args.stub:
        # the generated modules take `_int4_pack` / `_int4_linear` from linnet_b200.int4 at import
        # time, after stub_kernels() replaced them: nothing more to do
        modes = [False, True]
    else:
        modes = [False, True, "cudagraphs"]
    run_cards(args.work, args.device, modes, out, std)
    run_plans(args.work, args.device, out, std, any_device=args.stub)
    linear = kernels.int4_linear
    run_decoder(args.work, args.device, out, linear, fused=None if not args.stub else False)
    for name, count in CALLS.items():
        out[f"calls/{name}"] = np.array([count])
    np.savez(args.work / ("ours_stub.npz" if args.stub else "ours.npz"), **out)


if __name__ == "__main__":
    main()
