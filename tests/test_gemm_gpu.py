"""The tcgen05 dequant-GEMM (prompt-sized row counts) through the C ABI, against the
CPU oracle at sizes it finishes quickly, and at the prefill shapes against the exactly
dequantized weight multiplied by a library GEMM on the device (a cross-check of the
tiling, not an oracle) plus linearity."""

from __future__ import annotations

import pytest
import torch

from oracle import linear_oracle as lo

pytestmark = pytest.mark.gpu


def random_int4(out, depth, group, seed):
    gen = torch.Generator().manual_seed(seed)
    packed = torch.randint(0, 256, (out, depth // group, group // 2), generator=gen, dtype=torch.uint8)
    scale = (torch.rand(out, depth // group, generator=gen) * 0.02 + 0.001).to(torch.bfloat16)
    zero = torch.randint(0, 16, (out, depth // group), generator=gen, dtype=torch.uint8)
    return packed, scale, zero, gen


def gemm(x, packed, scale, zero):
    """Calls b200q_int4_gemm directly (not the row-count dispatcher)."""
    from linnet_b200 import _lib

    rows, depth = x.shape
    out = packed.shape[0]
    y = torch.empty(rows, out, dtype=torch.bfloat16, device=x.device)
    lib = _lib.load()
    _lib.check(lib.b200q_int4_gemm(x.data_ptr(), packed.data_ptr(), scale.data_ptr(), zero.data_ptr(),
                                   y.data_ptr(), rows, depth, out, 2 * packed.shape[2], _lib.BF16,
                                   torch.cuda.current_stream().cuda_stream))
    _lib.check(lib.b200q_int4_gemm_status())
    return y


def close(got, want, what):
    got, want = got.float().cpu(), want.float().cpu()
    torch.testing.assert_close(got, want, rtol=1e-2, atol=1e-2, msg=lambda m: f"{what}: {m}")


@pytest.mark.parametrize(("rows", "depth", "out", "group"), [
    (128, 64, 128, 64), (256, 128, 128, 128), (48, 512, 72, 128), (129, 256, 200, 64),
    (300, 1024, 384, 128), (257, 512, 130, 256), (1, 128, 16, 128), (640, 192, 136, 64),
    # up to 128 rows over a narrow weight: K split over a cluster of 2, 4 or 8 blocks
    (64, 4096, 4096, 128), (64, 14336, 512, 128), (100, 1024, 200, 64), (33, 640, 130, 64),
    (128, 1152, 256, 128), (17, 448, 130, 64),
    # weights wide enough for the tile width to be chosen by how the tiles fill the multiprocessors
    # (80, 96, 112, 144, 160, 192, 208, 240, 256 rows of W a tile on 148 of them), ragged last
    # tiles, one output width that is no multiple of 8 (element stores), one single-row-block case
    (130, 128, 9480, 64), (130, 192, 11848, 64), (300, 128, 7112, 128), (300, 192, 9480, 64),
    (300, 128, 10664, 64), (520, 128, 8632, 128), (520, 192, 9416, 64), (520, 128, 10984, 64),
    (520, 128, 11768, 128), (300, 128, 10666, 64), (40, 256, 11848, 64),
])
def test_gemm_matches_oracle(rows, depth, out, group):
    packed, scale, zero, gen = random_int4(out, depth, group, rows + depth + out)
    x = torch.randn(rows, depth, generator=gen).to(torch.bfloat16)
    want = lo.int4_groups_linear(x, packed, scale, zero)
    got = gemm(x.cuda(), packed.cuda(), scale.cuda(), zero.cuda())
    close(got, want, f"rows={rows} depth={depth} out={out} group={group}")


@pytest.mark.parametrize(("depth", "out"), [(4096, 6144), (4096, 28672), (14336, 4096)])
def test_gemm_prefill_shapes(depth, out):
    """M = 2048 at the three prefill shapes; W ~ N(0, 0.02) quantized on the GPU."""
    from linnet_b200 import kernels, quant

    gen = torch.Generator().manual_seed(depth + out)
    rows = 2048
    w = torch.empty(out, depth, dtype=torch.bfloat16)
    for r0 in range(0, out, 4096):
        r1 = min(out, r0 + 4096)
        w[r0:r1] = (torch.randn(r1 - r0, depth, generator=gen) * 0.02).to(torch.bfloat16)
    packed, _, zero, scale = quant.quantize_int4_groups(w.cuda(), 128, scale_dtype="bf16")
    x = torch.randn(rows, depth, generator=gen).to(torch.bfloat16).cuda()
    got = gemm(x, packed, scale, zero)
    dense = kernels.int4_dequantize(packed, scale, zero)  # bit-exact weight (tested elsewhere)
    ref = torch.nn.functional.linear(x, dense)
    torch.testing.assert_close(got.float(), ref.float(), rtol=1e-2, atol=1e-2)
    # a slice against the CPU oracle
    rows_s, cols_s = slice(0, 64), slice(0, 256)
    want = lo.int4_groups_linear(x[rows_s].cpu(), packed[cols_s].cpu(), scale[cols_s].cpu(), zero[cols_s].cpu())
    close(got[rows_s, cols_s], want, "oracle slice")
    # linearity: f(2x) == 2 f(x) exactly in bf16 (powers of two commute with rounding)
    twice = gemm((x * 2).to(torch.bfloat16), packed, scale, zero)
    assert torch.equal(twice, (got.float() * 2).to(torch.bfloat16))


def test_dispatcher_uses_gemm_for_many_rows():
    """`linnet::int4_linear` with a prompt's rows equals the direct GEMM call."""
    from linnet_b200 import kernels

    packed, scale, zero, gen = random_int4(256, 512, 128, 5)
    x = torch.randn(160, 512, generator=gen).to(torch.bfloat16).cuda()
    p, s, z = packed.cuda(), scale.cuda(), zero.cuda()
    assert torch.equal(kernels.int4_linear(x, p, s, z), gemm(x, p, s, z))
