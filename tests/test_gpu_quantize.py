"""Standalone quantisers on the GPU against the CPU oracle: byte-exact (identical fp inputs)."""

import numpy as np
import pytest
import torch

import oracle
from fim_testlib import DEV, same_bytes, to_dev

pytestmark = pytest.mark.gpu
E4M3, BF16 = torch.float8_e4m3fn, torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    import flashim_b200

    return flashim_b200.ops


@pytest.mark.parametrize("dtype", [BF16, torch.float32])
@pytest.mark.parametrize("shape", [(3, 5, 70), (7, 5, 32), (2, 9, 11, 128), (1, 1000), (33, 1024)])
def test_static_mxfp8_bytes(ops, dtype, shape):
    torch.manual_seed(0)
    x = (torch.randn(*shape) * 10).to(dtype)
    e = oracle.static_block_exponent(x)
    want = oracle.quantize_static_mx(x, e)
    got = ops.quantize_mxfp8.get("sm100")(to_dev(x), to_dev(e))
    assert got.values.shape == want.shape and got.logical_shape == tuple(shape)
    assert same_bytes(got.values.cpu(), want)
    # saturation beyond the calibrated range
    big = ops.quantize_mxfp8.get("sm100")(to_dev((x.float() * 1000).to(dtype)), to_dev(e))
    assert same_bytes(big.values.cpu(), oracle.quantize_static_mx((x.float() * 1000).to(dtype), e))


def test_static_mxfp8_golden(ops, golden):
    g = golden("formats")
    x, e = g("static_in", BF16), g("static_exponent")
    got = ops.quantize_mxfp8.get("sm100")(to_dev(x), to_dev(e))
    assert same_bytes(got.values.cpu(), g("static_out", E4M3))


def test_dynamic_mxfp8_exponent_boundaries(ops, golden):
    """Blocks whose amax sits within a few ulp of 448 * 2**k: the E8M0 byte must follow the fp32 log2 rule."""
    g = golden("formats")
    amax = g("amax")
    amax = amax[torch.isfinite(amax) & (amax < 3e38)]
    rows = amax.numel()
    x = torch.zeros(rows, 32)
    x[:, 5] = amax
    x[:, 9] = -amax * 0.5
    q, e = oracle.quantize_rows_dynamic(x)
    got_q, got_s = ops.quantize_mxfp8_dynamic.get("sm100")(to_dev(x))
    assert torch.equal(oracle.unswizzle_32_4_4(got_s.cpu(), rows, 1), e)
    assert same_bytes(got_q.cpu(), q)
    assert torch.equal(got_s.cpu(), oracle.swizzle_32_4_4(e))


@pytest.mark.parametrize("dtype", [BF16, torch.float32])
@pytest.mark.parametrize("rows,channels", [(50, 96), (1, 32), (300, 224), (4097, 128)])
def test_dynamic_mxfp8_bytes(ops, dtype, rows, channels):
    torch.manual_seed(1)
    x = (torch.randn(rows, channels) * torch.exp2(torch.randint(-8, 8, (rows, 1)).float())).to(dtype)
    x[rows // 2] = 0
    q, e = oracle.quantize_rows_dynamic(x)
    got_q, got_s = ops.quantize_mxfp8_dynamic.get("sm100")(to_dev(x))
    assert same_bytes(got_q.cpu(), q)
    assert torch.equal(got_s.cpu(), oracle.swizzle_32_4_4(e))


@pytest.mark.parametrize("dtype", [BF16, torch.float32])
@pytest.mark.parametrize("shape", [(40, 33), (2, 9, 11, 64), (5,), (100000,)])
def test_int8_bytes(ops, dtype, shape):
    torch.manual_seed(2)
    x = (torch.randn(*shape) * 3).to(dtype)
    scale = torch.tensor(0.037)
    got = ops.quantize_int8.get("sm100")(to_dev(x), to_dev(scale))
    assert torch.equal(got.values.cpu(), oracle.quantize_int8(x, scale))
    assert got.scale.dtype == torch.float32 and got.scale.numel() == 1


def test_int8_known_answers_and_ties(ops):
    # flashim tests/quant/test_int8.py:26-29 and the reciprocal-vs-division tie of tests/ops/test_depthwise_cuda.py
    x = torch.tensor([0.5, 1.5, 2.5, -0.5, 1000.0, -1000.0, 0.0, 0.0] * 2)
    got = ops.quantize_int8.get("sm100")(to_dev(x), to_dev(torch.tensor(1.0)))
    assert got.values.cpu().tolist()[:7] == [0, 2, 2, 0, 127, -127, 0]
    y = torch.full((16,), 3.375, dtype=BF16)
    scale = torch.tensor(0.03)
    assert torch.equal(ops.quantize_int8.get("sm100")(to_dev(y), to_dev(scale)).values.cpu(), oracle.quantize_int8(y, scale))


def test_empty_and_rejected_inputs(ops):
    from flashim_b200.ops import NoImplementation

    e = torch.zeros(1, dtype=torch.int8, device=DEV)
    out = ops.quantize_mxfp8.get("sm100")(torch.zeros(0, 32, device=DEV, dtype=BF16), e)
    assert out.values.shape == (0, 32)
    with pytest.raises(NoImplementation):  # CPU tensors never take a fallback
        ops.quantize_mxfp8(torch.zeros(4, 32, dtype=BF16), torch.zeros(1, dtype=torch.int8))


@pytest.mark.parametrize("dtype", [BF16, torch.float32])
@pytest.mark.parametrize("shape", [(2, 48, 9, 13), (1, 3, 5, 7), (3, 64, 16, 8), (1, 200, 11, 13), (2, 32, 1, 1),
                                   (1, 128, 40, 37)])
def test_static_mxfp8_reads_channels_first_in_place(ops, dtype, shape):
    """``x.permute(0, 2, 3, 1)`` of an NCHW tensor is quantised without a layout copy (flashim
    backends/triton/quantize.py:217-246): same bytes as the row-major path, ragged channels padded with zero codes."""
    torch.manual_seed(1)
    nchw = (torch.randn(*shape) * 6).to(dtype)
    view = nchw.permute(0, 2, 3, 1)
    assert not view.is_contiguous() or shape[1] == 1 or shape[2] * shape[3] == 1
    e = oracle.static_block_exponent(view)
    want = oracle.quantize_static_mx(view, e)
    got = ops.quantize_mxfp8.get("sm100")(to_dev(nchw).permute(0, 2, 3, 1), to_dev(e))
    assert got.values.shape == want.shape and got.logical_shape == tuple(view.shape)
    assert got.values.is_contiguous() and same_bytes(got.values.cpu(), want)


@pytest.mark.parametrize("dtype", [BF16, torch.float32])
@pytest.mark.parametrize("shape", [(2, 48, 9, 13), (1, 16, 5, 7), (3, 64, 16, 8), (1, 208, 11, 13), (1, 128, 40, 37)])
def test_static_int8_reads_channels_first_in_place(ops, dtype, shape):
    torch.manual_seed(2)
    nchw = (torch.randn(*shape) * 3).to(dtype)
    view = nchw.permute(0, 2, 3, 1)
    scale = torch.tensor(0.037)
    want = oracle.quantize_int8(view, scale)
    got = ops.quantize_int8.get("sm100")(to_dev(nchw).permute(0, 2, 3, 1), to_dev(scale))
    assert got.values.shape == want.shape and got.values.is_contiguous()
    assert torch.equal(got.values.cpu(), want)


def test_channels_first_quantisers_golden(ops, golden):
    g = golden("widening")
    for i in range(3):
        nchw = g(f"cf{i}_x", BF16 if i else torch.float32)
        got = ops.quantize_mxfp8.get("sm100")(to_dev(nchw).permute(0, 2, 3, 1), to_dev(g(f"cf{i}_e")))
        assert same_bytes(got.values.cpu(), g(f"cf{i}_q", E4M3)), f"case {i}"
        if nchw.shape[1] % 16 == 0:
            got8 = ops.quantize_int8.get("sm100")(to_dev(nchw).permute(0, 2, 3, 1), to_dev(torch.tensor(0.04)))
            assert torch.equal(got8.values.cpu(), g(f"cf{i}_i8")), f"int8 case {i}"


def test_int8_division_free_rounding_equals_true_division(ops):
    """The kernels reach round(value / scale) through a reciprocal and two fma refinement steps instead of a division:
    every bf16 value under 300 scales (random, short decimals where exact ties occur, powers of two, all-ones
    significands, tiny and huge) and random fp32 values must give the codes of the oracle's IEEE division."""
    g = torch.Generator().manual_seed(11)
    every_bf16 = torch.arange(-2**15, 2**15, dtype=torch.int32).to(torch.int16).view(BF16)
    every_bf16 = every_bf16[~torch.isnan(every_bf16.float())]
    scales = [0.03, 0.01, 0.1, 0.3, 0.05, 0.07, 1.0, 0.5, 0.25, 3.0, 1e-3, 7e-3, 1e-20, 1e-26, 1e-31, 1e20, 1e31,
              float(torch.tensor(0x3F7FFFFF, dtype=torch.int32).view(torch.float32)),   # all-ones significand
              float(torch.tensor(0x3CFFFFFF, dtype=torch.int32).view(torch.float32))]
    scales += (torch.rand(140, generator=g) * 0.2 + 1e-4).tolist()
    scales += torch.exp2(torch.rand(141, generator=g) * 40 - 30).tolist()
    quantise = ops.quantize_int8.get("sm100")
    x_dev = to_dev(every_bf16)
    for s in scales:
        scale = torch.tensor(s, dtype=torch.float32)
        got = quantise(x_dev, to_dev(scale)).values.cpu()
        want = oracle.quantize_int8(every_bf16, scale)
        assert torch.equal(got, want), f"scale {s!r}: {int((got != want).sum())} codes differ"
    wide = torch.randn(1 << 20, generator=g) * torch.exp2(torch.randint(-12, 10, (1 << 20,), generator=g).float())
    wide_dev = to_dev(wide)
    for s in scales[::15]:
        scale = torch.tensor(s, dtype=torch.float32)
        assert torch.equal(quantise(wide_dev, to_dev(scale)).values.cpu(), oracle.quantize_int8(wide, scale)), f"fp32, scale {s!r}"
