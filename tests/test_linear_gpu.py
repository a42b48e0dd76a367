"""int4 / int8 linear kernels (through the C ABI, via the torch operators) against the
CPU oracle of the reference's torch path.

Tolerance: rtol 1e-2 / atol 1e-2 on bf16 outputs with f32 accumulation (the bar this
build states), and additionally the reference's own kernel-test bound
`atol = 1e-2 * max|expected|` (python/linnet/tests/test_quant_groups.py:165-195).

Every int4 test runs in both numerics modes of the decode kernels.  "exact" reproduces the
reference's weights bit for bit and must meet the tolerance on any input.  "fast" (the
default) does not round the weights to 16 bits, so against the reference's torch path it
carries that path's own weight-rounding noise: on the nominal distributions (weights
~N(0, 0.02) through the quantizer) the plain tolerance must still hold; on the adversarial
random nibbles and scales of `random_int4` the allowance grows by the rigorous bound of that
noise (`2^-9 |x|.|w|^T`), and the result must ALSO be within the plain tolerance of the op's
definition computed without any weight rounding.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import linear_oracle as lo
from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-2, 1e-2


@pytest.fixture(params=["fast", "exact"], autouse=True)
def numerics(request):
    from linnet_b200 import kernels

    kernels.set_int4_numerics(request.param)
    yield request.param
    kernels.set_int4_numerics("fast")


def close(got: torch.Tensor, want: torch.Tensor, what: str = "", noise: torch.Tensor | None = None) -> None:
    """rtol/atol 1e-2 and the reference's `1e-2 max|expected|` bound; `noise` (fast numerics
    on adversarial inputs) widens the elementwise allowance by the reference's own
    weight-rounding bound."""
    got, want = got.float().cpu(), want.float().cpu()
    if noise is None:
        torch.testing.assert_close(got, want, rtol=RTOL, atol=ATOL, msg=lambda m: f"{what}: {m}")
    else:
        excess = (got - want).abs() - (ATOL + RTOL * want.abs() + noise.reshape(want.shape))
        assert excess.max().item() <= 0, f"{what}: {excess.max().item()} over the allowance"
    bound = 1e-2 * want.abs().max().item()
    assert (got - want).abs().max().item() <= bound + 1e-6, what


def close_int4(got, x, packed, scale, zero, what, bias=None, nominal=False):
    """Against the reference's torch path.  In fast mode on adversarial inputs the allowance
    grows by the bound of that path's own weight-rounding noise, and the same allowance must
    hold against the op's definition computed without rounding the weights (a kernel that
    reproduces the reference's rounding and one that skips it both meet both)."""
    from linnet_b200 import kernels

    want = lo.int4_groups_linear(x, packed, scale, zero, bias)
    if kernels.int4_numerics() == "exact" or nominal:
        close(got, want, what)
        return
    true, noise = lo.int4_groups_linear_f32(x, packed, scale, zero)
    true, noise = true.reshape(want.shape), noise.reshape(want.shape)
    if bias is not None:
        true = true + bias.float()
    close(got, want, what, noise=noise)
    close(got, true, what + " (definition)", noise=noise)


def random_int4(out, depth, group, dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    packed = torch.randint(0, 256, (out, depth // group, group // 2), generator=gen, dtype=torch.uint8)
    scale = (torch.rand(out, depth // group, generator=gen) * 0.02 + 0.001).to(dtype)
    zero = torch.randint(0, 16, (out, depth // group), generator=gen, dtype=torch.uint8)
    return packed, scale, zero, gen


def _bf16(bits):
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


@pytest.mark.parametrize("rows", [1, 3, 16, 40])
def test_int4_reference_fixture(golden_linear, rows):
    """Outputs the reference itself produced for an Int4GroupLinear card."""
    from linnet_b200 import kernels

    g = golden_linear["lin4"]
    x = _bf16(g[f"rows{rows}"]["x_bits"])
    want = _bf16(g[f"rows{rows}"]["y_bits"])
    got = kernels.int4_linear(x.cuda(), torch.from_numpy(g["packed"]).cuda(),
                              _bf16(g["scale_bits"]).cuda(), torch.from_numpy(g["zero"]).cuda())
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    close(got, want, f"fixture rows={rows}")


@pytest.mark.parametrize(("rows", "group", "out", "dtype"), [
    (8, 128, 72, torch.bfloat16),
    (37, 32, 72, torch.float16),
    (128, 64, 72, torch.bfloat16),
    (24, 128, 8448, torch.bfloat16),
])
def test_int4_reference_kernel_cases(rows, group, out, dtype):
    """The reference's kernel test, same seeds, shapes and bound
    (python/linnet/tests/test_quant_groups.py:165-195)."""
    from linnet_b200 import kernels

    width = 512
    generator = torch.Generator().manual_seed(rows)
    packed = torch.randint(0, 256, (out, width // group, group // 2), generator=generator, dtype=torch.uint8)
    scale = (torch.rand(out, width // group, generator=generator) * 0.02 + 0.001).to(dtype)
    zero = torch.randint(6, 10, (out, width // group), generator=generator, dtype=torch.uint8)
    x = torch.randn(rows, width, generator=generator).to(dtype)
    levels = torch.stack([packed & 15, packed >> 4], dim=-1).reshape(out, width // group, group)
    weight = (levels.float() - zero.float()[..., None]) * scale.float()[..., None]
    expected = x.float() @ weight.reshape(out, width).T
    got = kernels.int4_linear(x.cuda(), packed.cuda(), scale.cuda(), zero.cuda())
    assert got.shape == (rows, out) and got.dtype == dtype
    bound = 1e-2 * expected.abs().max().item()
    torch.testing.assert_close(got.float().cpu(), expected, rtol=0, atol=bound)


@pytest.mark.parametrize("rows", [1, 2, 4, 7, 8, 9, 15, 16, 17, 33])
@pytest.mark.parametrize(("depth", "out", "group"), [
    (512, 72, 128), (256, 17, 128), (1024, 16, 256), (384, 40, 64), (128, 8, 32), (256, 24, 16),
    (192, 20, 64), (96, 5, 32), (14336, 64, 128), (4096, 1000, 512),
])
def test_int4_shapes(rows, depth, out, group):
    from linnet_b200 import kernels

    packed, scale, zero, gen = random_int4(out, depth, group, torch.bfloat16, rows * 131 + depth)
    x = torch.randn(rows, depth, generator=gen).to(torch.bfloat16)
    got = kernels.int4_linear(x.cuda(), packed.cuda(), scale.cuda(), zero.cuda())
    close_int4(got, x, packed, scale, zero, f"rows={rows} depth={depth} out={out} group={group}")


@pytest.mark.parametrize("rows", [17, 20, 32, 33, 47, 64, 65, 100])
@pytest.mark.parametrize(("depth", "out", "dtype"), [
    (1024, 200, torch.bfloat16), (14336, 64, torch.bfloat16), (4096, 1000, torch.bfloat16),
    (2048, 72, torch.float16),
])
def test_int4_decode_kernel_many_rows(rows, depth, out, dtype):
    """b200q_int4_gemv_ex directly (the dispatcher would send 33 rows and more to the GEMM):
    17..32 and 33..64 rows per pass share the activations of a block in shared memory."""
    from linnet_b200 import _lib, kernels

    packed, scale, zero, gen = random_int4(out, depth, 128, dtype, rows * 7 + depth)
    x = torch.randn(rows, depth, generator=gen).to(dtype)
    xd, pd, sd, zd = x.cuda(), packed.cuda(), scale.cuda(), zero.cuda()
    y = torch.empty(rows, out, dtype=dtype, device="cuda")
    flags = _lib.EXACT_WEIGHTS if kernels.int4_numerics() == "exact" else 0
    _lib.check(_lib.load().b200q_int4_gemv_ex(xd.data_ptr(), pd.data_ptr(), sd.data_ptr(), zd.data_ptr(), y.data_ptr(),
                                              rows, depth, out, 128, _lib.BF16 if dtype == torch.bfloat16 else _lib.F16,
                                              flags, torch.cuda.current_stream().cuda_stream))
    close_int4(y, x, packed, scale, zero, f"rows={rows} depth={depth} out={out}")


@pytest.mark.parametrize("rows", [1, 5, 16])
def test_int4_f16(rows):
    from linnet_b200 import kernels

    packed, scale, zero, gen = random_int4(96, 1024, 128, torch.float16, 5 + rows)
    x = torch.randn(rows, 1024, generator=gen).to(torch.float16)
    got = kernels.int4_linear(x.cuda(), packed.cuda(), scale.cuda(), zero.cuda())
    close_int4(got, x, packed, scale, zero, f"f16 rows={rows}")


@pytest.fixture(scope="module")
def gate_up_weight():
    """Config: W ~ N(0, 0.02) [14336, 4096] quantized int4-g128 by the oracle quantizer,
    scales stored as bf16 (seed 0)."""
    gen = torch.Generator().manual_seed(0)
    w = torch.randn(14336, 4096, generator=gen) * 0.02
    packed, scale, zero = qo.quantize_int4_groups(w.numpy(), 128)
    return (torch.from_numpy(packed), torch.from_numpy(scale).to(torch.bfloat16),
            torch.from_numpy(zero), gen)


@pytest.mark.parametrize("rows", [1, 4, 16])
def test_int4_gate_up_shape(gate_up_weight, rows):
    """The headline decode shape: K=4096, N=14336, g128, M in {1, 4, 16}."""
    from linnet_b200 import kernels

    packed, scale, zero, gen = gate_up_weight
    x = torch.randn(rows, 4096, generator=gen).to(torch.bfloat16)
    got = kernels.int4_linear(x.cuda(), packed.cuda(), scale.cuda(), zero.cuda())
    close_int4(got, x, packed, scale, zero, f"gate/up rows={rows}", nominal=True)


def test_int4_down_shape_and_linearity():
    """K=14336, N=4096 (the row-split projection): oracle parity, and linearity in x,
    which holds at any size: f(x1 + x2) = f(x1) + f(x2) up to rounding."""
    from linnet_b200 import kernels

    packed, scale, zero, gen = random_int4(4096, 14336, 128, torch.bfloat16, 99)
    x1 = torch.randn(2, 14336, generator=gen).to(torch.bfloat16)
    dev = [t.cuda() for t in (packed, scale, zero)]
    got = kernels.int4_linear(x1.cuda(), *dev)
    close_int4(got, x1, packed, scale, zero, "down")
    x2 = (x1 * 0.5).to(torch.bfloat16)  # exact in bf16
    both = kernels.int4_linear((x1 + x2).cuda(), *dev).float()
    parts = got.float() + kernels.int4_linear(x2.cuda(), *dev).float()
    torch.testing.assert_close(both, parts, rtol=2e-2, atol=2e-2 * parts.abs().max().item())


@pytest.mark.parametrize("rows", [1, 2, 5])
@pytest.mark.parametrize(("depth", "out"), [(14336, 4096), (1024, 72)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_int4_swiglu_input(rows, depth, out, dtype):
    """`swiglu=True` (the product forms silu(gate) * up while it stages its input, for one and
    two rows) gives the bits of the stand-alone kernel followed by the product, and both follow
    the two PyTorch ops."""
    from linnet_b200 import glue, kernels

    packed, scale, zero, gen = random_int4(out, depth, 128, dtype, rows + depth)
    gate_up = (torch.randn(rows, 2 * depth, generator=gen) * 1.5).to(dtype).cuda()
    # what the two PyTorch ops make of it (silu rounded to the type, then the product)
    act = torch.nn.functional.silu(gate_up[:, :depth]) * gate_up[:, depth:]
    if dtype == torch.bfloat16:
        assert torch.equal(glue.silu_mul(gate_up), act)
    separate = kernels.int4_linear(act, packed.cuda(), scale.cuda(), zero.cuda())
    folded = kernels.int4_linear(gate_up, packed.cuda(), scale.cuda(), zero.cuda(), swiglu=True)
    assert torch.equal(folded, separate)
    close_int4(folded, act.cpu(), packed, scale, zero, f"swiglu rows={rows} depth={depth}")


def test_int4_plain_stream_order_is_the_same_product():
    """`overlap=False` (B200Q_NO_OVERLAP) only changes when the one-row kernel starts."""
    from linnet_b200 import kernels

    packed, scale, zero, gen = random_int4(1000, 4096, 128, torch.bfloat16, 21)
    x = torch.randn(1, 4096, generator=gen).to(torch.bfloat16).cuda()
    p, s, z = packed.cuda(), scale.cuda(), zero.cuda()
    want = kernels.int4_linear(x, p, s, z)
    for _ in range(3):
        assert torch.equal(kernels.int4_linear(x, p, s, z, overlap=False), want)


def test_int4_dequantize_is_exact():
    """`_int4_weight`: bit-for-bit the reference's arithmetic
    (python/linnet/tests/test_quant_groups.py:151-162)."""
    from linnet_b200 import int4

    for group, dtype in ((128, torch.bfloat16), (32, torch.float16), (6, torch.bfloat16)):
        packed, scale, zero, _ = random_int4(40, group * 6, group, dtype, group)
        want = lo.int4_weight(packed, scale, zero, dtype)
        got = int4._int4_weight(packed.cuda(), scale.cuda(), zero.cuda())
        assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16)), group


def test_generated_helpers_contract():
    """`_int4_pack` yields the 3-tuple the reference's test asserts, `_int4_linear`
    takes the generated call's arguments, bias and leading batch axes included."""
    from linnet_b200 import int4

    packed, scale, zero, gen = random_int4(64, 256, 128, torch.bfloat16, 3)
    bias = torch.randn(64, generator=gen).to(torch.bfloat16)
    x = torch.randn(2, 3, 256, generator=gen).to(torch.bfloat16)
    p, s, z = packed.cuda(), scale.cuda(), zero.cuda()
    prepared = int4._int4_pack(p, s, z)
    assert isinstance(prepared, tuple) and len(prepared) == 3
    got = int4._int4_linear(x.cuda(), prepared, bias.cuda(), p, s, z)
    assert got.shape == (2, 3, 64)
    close_int4(got, x, packed, scale, zero, "generated helpers", bias=bias)


# ---- int8 -------------------------------------------------------------------------


@pytest.mark.parametrize("rows", [1, 5, 16])
def test_int8_reference_fixture(golden_linear, rows):
    from linnet_b200 import quantized

    g = golden_linear["lin8"]
    x = _bf16(g[f"rows{rows}"]["x_bits"]).cuda()
    ops = quantized.int8_operands(torch.from_numpy(g["q_rows"]).cuda(),
                                  torch.from_numpy(g["s_rows"]).reshape(-1).cuda(), 0)
    close(quantized.int8_linear(x, ops, None), _bf16(g[f"rows{rows}"]["y_rows_bits"]), "rows")
    gops = quantized.int8_group_operands(torch.from_numpy(g["q_groups"]).cuda(),
                                         torch.from_numpy(g["s_groups"]).cuda())
    close(quantized.int8_group_linear(x, gops, None), _bf16(g[f"rows{rows}"]["y_groups_bits"]), "groups")


def close_int8(got, x, q, scale, what, bias=None):
    """One scale a row under fast numerics (the scale multiplies the f32 sum, as the
    reference's GPU kernel does): within the usual tolerance of the reference's CPU route once
    that route's own weight-rounding noise is allowed for, and as close to the definition."""
    want = lo.int8_linear(x, q, scale, bias)
    true, noise = lo.int8_linear_f32(x, q, scale)
    true, noise = true.reshape(want.shape), noise.reshape(want.shape)
    if bias is not None:
        true = true + bias.float()
    close(got, want, what, noise=noise)
    close(got, true, what + " (definition)", noise=noise)


@pytest.mark.parametrize("rows", [1, 2, 3, 8, 16, 17, 64])
@pytest.mark.parametrize(("depth", "out", "group"), [
    (4096, 4096, 0), (512, 72, 0), (256, 17, 128), (1024, 48, 64), (256, 24, 16), (96, 10, 32),
    (100, 7, 0), (14336, 32, 0),
])
def test_int8_shapes(rows, depth, out, group):
    from linnet_b200 import kernels, quantized

    gen = torch.Generator().manual_seed(rows + depth + out)
    w = torch.randn(out, depth, generator=gen) * 0.02
    q, scale = qo.quantize_int8_groups(w.numpy(), group or depth, "f32")
    q, scale = torch.from_numpy(q), torch.from_numpy(scale)
    x = torch.randn(rows, depth, generator=gen).to(torch.bfloat16)
    bias = torch.randn(out, generator=gen).to(torch.bfloat16)
    if group == 0:
        want = lo.int8_linear(x, q, scale.reshape(-1), bias)
        ops = quantized.int8_operands(q.cuda(), scale.reshape(-1).cuda(), 0)  # weight-only: inputs not rounded
        got = quantized.int8_linear(x.cuda(), ops, bias.cuda())
        if kernels.int4_numerics() == "fast":  # passes of one or two rows take the sum-scaled kernel
            close_int8(got, x, q, scale.reshape(-1), f"int8 rows={rows} depth={depth} out={out}", bias)
            return
    else:
        want = lo.int8_group_linear(x, q, scale, bias)
        ops = quantized.int8_group_operands(q.cuda(), scale.cuda())
        got = quantized.int8_group_linear(x.cuda(), ops, bias.cuda())
    close(got, want, f"int8 rows={rows} depth={depth} out={out} group={group}")


@pytest.mark.parametrize("rows", [1, 2])
@pytest.mark.parametrize(("depth", "out"), [(4096, 14344), (1024, 4096), (8192, 1000), (14336, 4096), (512, 16)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_int8_one_and_two_rows(rows, depth, out, dtype):
    """The shapes the two-plane TMA kernel takes under fast numerics (several rounds of tiles,
    a ragged last tile, more items than ring stages, K of one item) and, under exact numerics,
    the kernel that rounds every weight: both against the reference's CPU arithmetic."""
    from linnet_b200 import kernels

    gen = torch.Generator().manual_seed(rows + depth + out)
    w = torch.randn(out, depth, generator=gen) * 0.02
    q, scale = qo.quantize_int8_groups(w.numpy(), depth, "f32")
    q, scale = torch.from_numpy(q), torch.from_numpy(scale).reshape(-1)
    x = torch.randn(rows, depth, generator=gen).to(dtype)
    fn = kernels.gemv8 if rows == 1 else kernels.w8a16
    got = fn(x.cuda(), q.cuda(), scale.cuda(), False, 0, 1)
    if kernels.int4_numerics() == "fast":
        close_int8(got, x, q, scale, f"int8 rows={rows} depth={depth} out={out} {dtype}")
    else:
        close(got, lo.int8_linear(x, q, scale), f"int8 rows={rows} depth={depth} out={out} {dtype}")
    # linear in x: twice the input, twice the output, exactly (a power of two), except where an
    # f16 output is subnormal and doubling it cannot bring back the bits its rounding dropped
    twice = fn((x * 2).cuda(), q.cuda(), scale.cuda(), False, 0, 1)
    normal = got.abs() >= 1e-3
    assert torch.equal(twice[normal], (got * 2)[normal])
    from linnet_b200 import _lib
    _lib.check(_lib.load().b200q_int4_gemm_status())


def test_int8_config_one():
    """int8 symmetric per-output-channel, M=1, K=N=4096, W ~ N(0, 0.02), seed 0."""
    from linnet_b200 import kernels, quant

    torch.manual_seed(0)
    w = torch.randn(4096, 4096) * 0.02
    x = torch.randn(1, 4096).to(torch.bfloat16)
    q, scale = quant.quantize_int8_groups(w, 4096, "f32")
    want_q, want_s = qo.quantize_int8_groups(w.numpy(), 4096, "f32")
    assert np.array_equal(q.cpu().numpy(), want_q)
    want = lo.int8_linear(x, torch.from_numpy(want_q), torch.from_numpy(want_s).reshape(-1))
    got = kernels.gemv8(x.cuda(), q, scale.reshape(-1), False, 0, 1)
    assert got.shape == (1, 4096)
    close(got, want, "config 1")
    deq = kernels.dequantize8(q, scale.reshape(-1), False, 0, 1, torch.bfloat16)
    assert torch.equal(deq.cpu().view(torch.int16),
                       lo.int8_weight(torch.from_numpy(want_q), torch.from_numpy(want_s), torch.bfloat16).view(torch.int16))


def test_cuda_graph_capture():
    """The operators record into a CUDA graph and replay (no sync, no allocation in the
    C ABI; outputs come from PyTorch's graph pool)."""
    from linnet_b200 import kernels

    packed, scale, zero, gen = random_int4(256, 512, 128, torch.bfloat16, 11)
    p, s, z = packed.cuda(), scale.cuda(), zero.cuda()
    x = torch.randn(4, 512, generator=gen).to(torch.bfloat16)
    static = x.cuda()
    kernels.int4_linear(static, p, s, z)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = kernels.int4_linear(static, p, s, z)
    x2 = torch.randn(4, 512, generator=gen).to(torch.bfloat16)
    static.copy_(x2.cuda())
    graph.replay()
    torch.cuda.synchronize()
    close_int4(y, x2, packed, scale, zero, "graph replay")
