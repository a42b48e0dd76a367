"""W8A8: `int8_rows` (bit-exact with the definition) and `int8_mm` (exact int32 sums on the
tensor cores), and the layer route that uses them: `int8_linear` with `rounded` set and more
than 32 rows (python/linnet/src/linnet/torch/quantized.py:187-189).  Mirrors
python/linnet/tests/test_quant_8bit.py:315-341: rows {1, 3, 17, 64} weight-only within
`0.01 * max|want|`, and within `0.06 * max|want|` where the input is rounded to 8 bits."""

from __future__ import annotations

import pytest
import torch

from oracle import linear_oracle as lo
from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize(("rows", "depth"), [(1, 128), (5, 4096), (33, 512), (64, 14336), (3, 24576), (2, 8)])
def test_int8_rows_is_exact(rows, depth, dtype):
    from linnet_b200 import kernels

    gen = torch.Generator().manual_seed(rows * 7 + depth)
    x = torch.randn(rows, depth, generator=gen)
    x[0, : min(depth, 16)] = torch.tensor([0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 0.0, 127.0] * 2)[: min(depth, 16)] * 0.01
    if rows > 1:
        x[1] = 0.0  # a row of zeros: the scale floors at 1e-12 / 127
    x = x.to(dtype)
    want_q, want_s = lo.int8_rows(x)
    q, s = kernels.int8_rows(x.cuda())
    assert s.shape == (rows, 1) and q.dtype == torch.int8
    assert torch.equal(s.cpu().view(torch.int32), want_s.view(torch.int32))
    assert torch.equal(q.cpu(), want_q)


@pytest.mark.parametrize(("rows", "depth", "out"), [
    (33, 128, 16), (64, 512, 72), (128, 4096, 4096), (129, 1024, 272), (300, 4096, 1000), (2048, 4096, 6144),
    (2048, 14336, 4096), (1, 256, 48),
    # wide tiles whose width is chosen by how the tiles fill the multiprocessors (224, 240 rows of W
    # on 148 of them), ragged last tiles, an output width that is no multiple of 8
    (2048, 256, 14336), (1200, 128, 5001), (1500, 128, 9000),
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_int8_mm_is_exact(rows, depth, out, dtype):
    """Integer sums are exact, so the result is the oracle's bit for bit."""
    from linnet_b200 import kernels

    if dtype == torch.float16 and rows > 300:
        pytest.skip("one dtype is enough at the large shapes")
    gen = torch.Generator().manual_seed(rows + depth + out)
    xq = torch.randint(-127, 128, (rows, depth), generator=gen, dtype=torch.int8)
    w = torch.randint(-127, 128, (out, depth), generator=gen, dtype=torch.int8)
    xs = torch.rand(rows, 1, generator=gen) * 0.02 + 1e-3
    ws = torch.rand(out, generator=gen) * 0.01 + 1e-4
    want = lo.int8_mm(xq, w, xs, ws, dtype)
    got = kernels.int8_mm(xq.cuda(), w.cuda(), xs.cuda(), ws.cuda(), dtype)
    assert got.shape == (rows, out) and got.dtype == dtype
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("rows", [1, 3, 17, 64, 65, 128, 300, 2048])
@pytest.mark.parametrize("rounded", [0, 1])
def test_int8_linear_rows_and_routes(rows, rounded):
    """Every row-count route of `int8_linear`: the decode kernel (1, 2..64 rows), the
    dequantized weight and the library GEMM (more rows, weight-only), int8 activations (more
    than 32 rows with `rounded`)."""
    from linnet_b200 import quantized

    depth, out = 4096, 1024
    gen = torch.Generator().manual_seed(rows)
    w = torch.randn(out, depth, generator=gen) * 0.02
    q, scale = qo.quantize_int8_groups(w.numpy(), depth, "f32")
    q, scale = torch.from_numpy(q), torch.from_numpy(scale).reshape(-1)
    x = torch.randn(rows, depth, generator=gen).to(torch.bfloat16)
    # no bias here: it is added after the product has been rounded to bf16, so where the two
    # nearly cancel, one ulp of the product (a rounding any two correct GEMMs may take
    # differently) exceeds the elementwise bar; test_int8_shapes covers the bias
    want = lo.int8_linear(x, q, scale).float()
    got = quantized.int8_linear(x.cuda(), quantized.int8_operands(q.cuda(), scale.cuda(), rounded), None)
    bound = (0.06 if rounded and rows > quantized.FEW_ROWS else 0.01) * want.abs().max().item()
    assert (got.float().cpu() - want).abs().max().item() <= bound
    if not (rounded and rows > quantized.FEW_ROWS):
        # against the same product summed in f64 (what both the CPU oracle and the library GEMM
        # of the many-row route approximate)
        exact = (x.double() @ lo.int8_weight(q, scale, torch.bfloat16).double().T).float()
        torch.testing.assert_close(got.float().cpu(), exact, rtol=1e-2, atol=1e-2)
    else:
        # exactly the two kernels composed
        xq, xs = lo.int8_rows(x)
        composed = lo.int8_mm(xq, q, xs, scale, torch.bfloat16).float()
        torch.testing.assert_close(got.float().cpu(), composed, rtol=0, atol=0)


@pytest.mark.parametrize("rows", [65, 200])
def test_int8_group_linear_many_rows(rows):
    from linnet_b200 import quantized

    depth, out, group = 1024, 256, 128
    gen = torch.Generator().manual_seed(rows)
    w = torch.randn(out, depth, generator=gen) * 0.02
    q, scale = qo.quantize_int8_groups(w.numpy(), group, "f32")
    q, scale = torch.from_numpy(q), torch.from_numpy(scale)
    x = torch.randn(rows, depth, generator=gen).to(torch.bfloat16)
    want = lo.int8_group_linear(x, q, scale).float()
    got = quantized.int8_group_linear(x.cuda(), quantized.int8_group_operands(q.cuda(), scale.cuda()), None)
    torch.testing.assert_close(got.float().cpu(), want, rtol=1e-2, atol=1e-2)
