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
