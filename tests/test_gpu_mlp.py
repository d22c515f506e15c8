"""The residual MLP of a refiner block as one kernel (1x1 up conv + GELU + per-pixel requantisation, 1x1 down conv +
residual, the hidden tensor kept on chip) against the two conv launches it replaces: the same MMAs in the same order
and the same epilogue arithmetic, so the same bytes are required. The pair of launches is itself checked against the
CPU oracle (tests/test_gpu_conv_schedule.py, tests/test_gpu_refiner.py)."""
from __future__ import annotations

import pytest
import torch

import oracle
from fim_testlib import conv_schedule, same_bytes, to_dev

pytestmark = pytest.mark.gpu
E4M3, BF16 = torch.float8_e4m3fn, torch.bfloat16
POINT = (1, 1, 1, 1, 0, 0, 1, 1)


@pytest.fixture(scope="module")
def ops():
    import flashim_b200

    return flashim_b200.ops


def _block(shape, c, seed):
    g = torch.Generator().manual_seed(seed)
    rows = 1
    for n in shape:
        rows *= n
    x = (torch.randn(*shape, c, generator=g) * torch.exp2(torch.randint(-3, 4, (*shape, 1), generator=g).float())).to(BF16)
    w1 = (torch.randn(2 * c, c, generator=g) * 2).to(E4M3)
    e1 = torch.randint(-9, -4, (2 * c, c // 32), dtype=torch.int8, generator=g)
    w2 = (torch.randn(c, 2 * c, generator=g) * 2).to(E4M3)
    e2 = torch.randint(-9, -4, (c, 2 * c // 32), dtype=torch.int8, generator=g)
    b1 = torch.randn(2 * c, generator=g).to(BF16)
    b2 = torch.randn(c, generator=g).to(BF16)
    res = torch.randn(*shape, c, generator=g).to(BF16)
    return x, w1, oracle.swizzle_32_4_4(e1), b1, w2, oracle.swizzle_32_4_4(e2), b2, res


@pytest.mark.parametrize("max_ctas", [0, 1, 5])
@pytest.mark.parametrize("shape", [(1, 9, 13), (2, 37, 41), (3, 64, 64)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("channels", [128, 256])
def test_one_launch_equals_up_conv_then_down_conv(ops, channels, shape, max_ctas):
    """117, 3034 and 12288 pixels (a ragged last tile in the first two); with the CTAs capped one CTA walks every tile, so
    the weight ring, both accumulators and both hidden-operand buffers wrap many times."""
    x, w1, s1, b1, w2, s2, b2, res = _block(shape, channels, seed=channels + shape[1])
    xd, w1d, s1d, b1d, w2d, s2d, b2d, resd = to_dev(x, w1, s1, b1, w2, s2, b2, res)
    conv = ops.mxfp8_conv2d_fused.get("sm100")
    q, s = ops.quantize_mxfp8_dynamic.get("sm100")(xd)
    hq, hs = conv(q, s, w1d, s1d, b1d, *POINT, act="gelu", dynamic_out=True)
    want = conv(hq, hs, w2d, s2d, b2d, *POINT, residual=resd)
    with conv_schedule(0, max_ctas):
        got = ops.mxfp8_gelu_mlp_residual.get("sm100")(q, s, w1d, s1d, b1d, w2d, s2d, b2d, resd)
    assert got.shape == want.shape and got.dtype == BF16
    assert same_bytes(got, want)


def test_repeated_launches_give_the_same_bytes(ops):
    x, w1, s1, b1, w2, s2, b2, res = _block((2, 50, 50), 128, seed=7)
    xd, w1d, s1d, b1d, w2d, s2d, b2d, resd = to_dev(x, w1, s1, b1, w2, s2, b2, res)
    q, s = ops.quantize_mxfp8_dynamic.get("sm100")(xd)
    fused = ops.mxfp8_gelu_mlp_residual.get("sm100")
    first = fused(q, s, w1d, s1d, b1d, w2d, s2d, b2d, resd)
    for _ in range(10):
        assert same_bytes(fused(q, s, w1d, s1d, b1d, w2d, s2d, b2d, resd), first)


def test_other_widths_are_declined(ops):
    x, w1, s1, b1, w2, s2, b2, res = _block((1, 8, 8), 64, seed=3)
    xd, w1d, s1d, b1d, w2d, s2d, b2d, resd = to_dev(x, w1, s1, b1, w2, s2, b2, res)
    q, s = ops.quantize_mxfp8_dynamic.get("sm100")(xd)
    with pytest.raises(Exception):  # no implementation applies, and there is no fall-back
        ops.mxfp8_gelu_mlp_residual.get("sm100")(q, s, w1d, s1d, b1d, w2d, s2d, b2d, resd)
