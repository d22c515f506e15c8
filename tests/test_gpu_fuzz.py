"""Seeded random geometries through the C ABI against the CPU oracle: shapes the hand-picked cases do not name (odd
sizes, 1-pixel images, dilation with padding, channel counts on every supported tile width, batches that leave the last
CTA pair or the last tile half empty)."""

import random

import pytest
import torch
import torch.nn.functional as F

import oracle
from fim_testlib import bf16_ulp_distance, code_mismatch, rel_l2, same_bytes, to_dev

pytestmark = pytest.mark.gpu
E4M3, BF16 = torch.float8_e4m3fn, torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    import flashim_b200

    return flashim_b200.ops


def _geometries(seed: int, count: int):
    rng = random.Random(seed)
    for _ in range(count):
        k = rng.choice([1, 1, 3, 3, 5])
        dilation = rng.choice([1, 1, 2]) if k > 1 else 1
        pad = rng.choice([0, dilation * (k // 2)])
        cin = 32 * rng.choice([1, 2, 3, 4, 8, 16])
        cout = 32 * rng.choice([1, 2, 3, 4, 8, 16])
        batch = rng.choice([1, 2, 3, 5])
        extent = dilation * (k - 1) + 1
        height = rng.randint(max(1, extent - 2 * pad), 45)
        width = rng.randint(max(1, extent - 2 * pad), 45)
        yield cin, cout, k, pad, dilation, batch, height, width


@pytest.mark.parametrize("geometry", list(_geometries(11, 24)), ids=lambda g: "c%d-%d_k%d_p%d_d%d_b%d_%dx%d" % g)
def test_random_mxfp8_conv(ops, geometry):
    cin, cout, k, pad, dilation, batch, height, width = geometry
    g = torch.Generator().manual_seed(hash(geometry) & 0xFFFF)
    x = (torch.randn(batch, height, width, cin, generator=g) * 3).to(E4M3)
    ce = torch.randint(-6, 3, (cin // 32,), dtype=torch.int8, generator=g)
    w = (torch.randn(cout, k * k * cin, generator=g) * 2).to(E4M3)
    we = torch.randint(-9, -3, (cout, k * k * cin // 32), dtype=torch.int8, generator=g)
    bias = torch.randn(cout, generator=g).to(BF16)
    args = (k, k, 1, 1, pad, pad, dilation, dilation)
    want = oracle.mxfp8_conv2d(x, ce, w, we, bias, *args)
    got = ops.mxfp8_conv2d.get("sm100")(*to_dev(x, ce, w, we, bias), *args)
    assert got.shape == want.shape
    assert rel_l2(got, want) < 1e-3
    # fused static requantisation = the quantiser applied to the kernel's own bf16 output
    oe = oracle.static_block_exponent(got.cpu().float())
    chained = ops.mxfp8_conv2d.get("sm100")(*to_dev(x, ce, w, we, bias), *args, out_exponent=to_dev(oe))
    assert same_bytes(chained.cpu(), oracle.quantize_static_mx(got.cpu(), oe))


@pytest.mark.parametrize("geometry", list(_geometries(12, 16)), ids=lambda g: "c%d-%d_k%d_p%d_d%d_b%d_%dx%d" % g)
def test_random_int8_conv(ops, geometry):
    cin, cout, k, pad, dilation, batch, height, width = geometry
    g = torch.Generator().manual_seed(hash(geometry) & 0xFFFF)
    x = torch.randint(-127, 128, (batch, height, width, cin), dtype=torch.int8, generator=g)
    w = torch.randint(-127, 128, (cout, k * k * cin), dtype=torch.int8, generator=g)
    args = (k, k, 1, 1, pad, pad, dilation, dilation)
    acc = ops.int8_conv2d_accumulators.get("sm100")(*to_dev(x, w), *args)
    assert torch.equal(acc.cpu(), oracle.int8_conv2d_accumulators_ext(x, w, *args))
    a_scale, w_scale = torch.tensor(0.013), torch.rand(cout, generator=g) * 0.01 + 0.001
    bias = torch.randn(cout, generator=g).to(BF16)
    got = ops.int8_conv2d.get("sm100")(*to_dev(x, w, a_scale, w_scale, bias), *args)
    assert same_bytes(got.cpu(), oracle.int8_conv2d(x, w, a_scale, w_scale, bias, *args))


def _depthwise_shapes(seed: int, count: int):
    rng = random.Random(seed)
    for _ in range(count):
        yield rng.choice([1, 2, 3]), 32 * rng.choice([1, 2, 3, 4, 6, 8]), rng.randint(1, 70), rng.randint(1, 70)


@pytest.mark.parametrize("shape", list(_depthwise_shapes(13, 16)), ids=lambda s: "b%d_c%d_%dx%d" % s)
def test_random_depthwise(ops, shape):
    batch, channels, height, width = shape
    g = torch.Generator().manual_seed(hash(shape) & 0xFFFF)
    x = torch.randn(batch, channels, height, width, generator=g).to(BF16).contiguous(memory_format=torch.channels_last)
    w = (torch.randn(25, channels, generator=g) * 0.2).to(BF16)
    b = torch.randn(channels, generator=g)
    for act in ("relu", "gelu", "none"):
        want = oracle.depthwise5x5_act_ext(x, w, b, act)
        got = ops.depthwise5x5_act.get("sm100")(*to_dev(x, w, b), act).cpu()
        pre = oracle.depthwise5x5_fp32(x, w, b).permute(0, 2, 3, 1)
        close = (bf16_ulp_distance(got, want) <= 1) | ((got.float() - want.float()).abs() <= 3e-7 * pre.abs() + 1e-30)
        assert bool(close.all()), act
    q_ref, s_ref = oracle.depthwise5x5_relu_mxfp8(x, w, b)
    q, s = ops.depthwise5x5_relu_mxfp8.get("sm100")(*to_dev(x, w, b))
    assert float((s.cpu().view(torch.uint8) != s_ref.view(torch.uint8)).float().mean()) < 2e-3
    assert code_mismatch(q, q_ref) < 2e-3
    scale = torch.tensor(0.05)
    got8 = ops.depthwise5x5_relu_int8.get("sm100")(*to_dev(x, w, b, scale)).cpu()
    want8 = oracle.depthwise5x5_relu_int8(x, w, b, scale)
    delta = (got8.int() - want8.int()).abs()
    assert int(delta.max()) <= 1 and float((delta > 0).float().mean()) < 5e-3


def _widening_shapes(seed: int, count: int):
    rng = random.Random(seed)
    for _ in range(count):
        yield rng.choice([1, 2, 3]), 16 * rng.randint(1, 18), rng.randint(1, 40), rng.randint(1, 40)


@pytest.mark.parametrize("shape", list(_widening_shapes(31, 12)), ids=lambda s: "b%d_c%d_%dx%d" % s)
def test_random_channels_first_quantisers_and_pool(ops, shape):
    """Random NCHW shapes (pixel counts with and without the 4-pixel alignment of the vector loads, channel counts that end
    inside a 64-channel tile) through the in-place quantisers, and the same tensor through the max-pool quantiser."""
    b, c, h, w = shape
    g = torch.Generator().manual_seed(hash(shape) & 0xFFFF)
    nchw = (torch.randn(b, c, h, w, generator=g) * 4).to(BF16)
    view = nchw.permute(0, 2, 3, 1)
    e = oracle.static_block_exponent(view)
    scale = torch.tensor(0.031)
    device_view = to_dev(nchw).permute(0, 2, 3, 1)
    assert same_bytes(ops.quantize_mxfp8.get("sm100")(device_view, to_dev(e)).values.cpu(), oracle.quantize_static_mx(view, e))
    assert torch.equal(ops.quantize_int8.get("sm100")(device_view, to_dev(scale)).values.cpu(), oracle.quantize_int8(view, scale))
    from flashim_b200.backends.sm100 import kernels

    nhwc = view.contiguous()
    pooled = kernels.maxpool2_quantize_int8(to_dev(nhwc), to_dev(scale.reshape(1)))
    want = oracle.quantize_int8(F.max_pool2d(nchw.float(), 2).permute(0, 2, 3, 1).to(BF16), scale) if h > 1 and w > 1 else None
    assert pooled.shape == (b, h // 2, w // 2, c)
    if want is not None:
        assert torch.equal(pooled.cpu(), want)
