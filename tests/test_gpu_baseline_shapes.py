"""The kernels at the full shapes the benchmark runs (the conv shape sweep, the depthwise case and the refiner stack) against the CPU oracle, and one
launch per kernel family whose tensors hold more than 2**31 elements (64-bit offsets).

Config 3: batch 4, (H = W, C) in (100, 512), (200, 256), (400, 128), (800, 64), 3x3 pad 1 and 1x1, bf16 input -> static
MXFP8 -> conv + bias + GELU -> static and dynamic MXFP8 requantisation. The oracle's byte im2col of a whole batch would
need tens of GB for the large images, so the oracle runs one image (or a band of rows with its halo) at a time; a conv
output row depends on nothing else.
"""

import pytest
import torch

import oracle
from fim_testlib import DEV, bf16_ulp_distance, code_mismatch, rel_l2, same_bytes, to_dev

pytestmark = pytest.mark.gpu
E4M3, BF16 = torch.float8_e4m3fn, torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    import flashim_b200

    return flashim_b200.ops


def _bands(height: int, rows: int):
    for y0 in range(0, height, rows):
        yield y0, min(height, y0 + rows)


def _oracle_conv_band(q, ce, wq, we, bias, k, image, y0, y1, **kw):
    """Rows [y0, y1) of the oracle's conv output for one image: the band plus its halo rows, zero padding at the image
    border as the conv itself pads."""
    pad = k // 2
    h = q.shape[1]
    lo, hi = max(0, y0 - pad), min(h, y1 + pad)
    band = q[image: image + 1, lo:hi]
    top, bottom = pad - (y0 - lo), pad - (hi - y1)  # rows of conv padding this band still needs
    if top or bottom:
        band = torch.nn.functional.pad(band.view(torch.uint8), (0, 0, 0, 0, top, bottom)).view(E4M3)
    return oracle.mxfp8_conv2d_ext(band, ce, wq, we, bias, k, k, 1, 1, 0, pad, 1, 1, **kw)


CONFIG3 = [(100, 512), (200, 256), (400, 128), (800, 64)]


@pytest.mark.parametrize("k", [3, 1])
@pytest.mark.parametrize("size,channels", CONFIG3)
def test_config3_conv_with_fused_epilogue(ops, size, channels, k):
    from flashim_b200.quant import QuantizedWeight, calibrate_block32_exponent, swizzle_scales

    torch.manual_seed(2)
    n = 4
    x = torch.randn(n, size, size, channels).to(BF16)
    weight = torch.empty(channels, channels, k, k)
    torch.nn.init.kaiming_normal_(weight)
    bias = (torch.randn(channels) * 0.02).to(BF16)
    packed = QuantizedWeight.from_conv(weight)
    wq, we = packed.values, packed.scale_exponent
    ce = calibrate_block32_exponent(x)
    assert torch.equal(ce, oracle.static_block_exponent(x))

    xd = x.to(DEV)
    q = ops.quantize_mxfp8.get("sm100")(xd, ce.to(DEV)).values
    q_cpu = q.cpu()
    assert same_bytes(q_cpu, oracle.quantize_static_mx(x, ce))  # the quantiser at full size, byte for byte

    geometry = (k, k, 1, 1, k // 2, k // 2, 1, 1)
    fused = ops.mxfp8_conv2d_fused.get("sm100")
    args = (q, ce.to(DEV), wq.to(DEV), swizzle_scales(we).to(DEV), bias.to(DEV))
    dense = fused(*args, *geometry, act="gelu")  # bf16, before requantisation
    dense_cpu = dense.cpu()

    # against the oracle: every image, in bands of rows that keep the oracle's im2col below ~1 GB
    rows = max(1, min(size, (1 << 28) // (size * channels * k * k)))
    num = den = 0.0
    worst = 0
    for image in range(n):
        for y0, y1 in _bands(size, rows):
            want = _oracle_conv_band(q_cpu, ce, wq, we, bias, k, image, y0, y1, act="gelu")
            got = dense_cpu[image: image + 1, y0:y1]
            num += float((got.float() - want.float()).pow(2).sum())
            den += float(want.float().pow(2).sum())
            worst = max(worst, int(bf16_ulp_distance(got, want).max()))
    assert (num / den) ** 0.5 < 1e-3, (num / den) ** 0.5

    # the fused requantisations are the oracle quantisers applied to the kernel's own bf16 output
    oe = calibrate_block32_exponent(dense_cpu)
    static = fused(*args, *geometry, act="gelu", out_exponent=oe.to(DEV))
    assert same_bytes(static.cpu(), oracle.quantize_static_mx(dense_cpu, oe))
    dyn, scales = fused(*args, *geometry, act="gelu", dynamic_out=True)
    q_ref, e_ref = oracle.quantize_rows_dynamic(dense_cpu.reshape(-1, channels))
    assert same_bytes(dyn.cpu().reshape(-1, channels), q_ref)
    assert torch.equal(scales.cpu(), oracle.swizzle_32_4_4(e_ref))

    # GELU in the epilogue is torch's erf form on the bf16-rounded sum, exactly: compare with the kernel's own plain output
    plain = fused(*args, *geometry, act="none").cpu()
    assert same_bytes(dense_cpu, torch.nn.functional.gelu(plain.float()).to(BF16))


@pytest.mark.parametrize("shape", [(4, 200, 256), (4, 400, 128), (4, 100, 512)])
def test_config4_depthwise_gelu(ops, shape):
    n, size, channels = shape
    torch.manual_seed(3)
    x = torch.randn(n, size, size, channels).to(BF16)
    w = (torch.randn(25, channels) * 0.05).to(BF16)
    b = torch.randn(channels)
    value = x.permute(0, 3, 1, 2)
    got = ops.depthwise5x5_act.get("sm100")(value.to(DEV), w.to(DEV), b.to(DEV), "gelu").cpu()
    want = oracle.depthwise5x5_act_ext(value, w, b, "gelu")
    pre = oracle.depthwise5x5_fp32(value, w, b).permute(0, 2, 3, 1)
    d = bf16_ulp_distance(got, want)
    # 1 bf16 ulp, or the fp32 cancellation floor of x * 0.5 * (1 + erf(x / sqrt 2)) for strongly negative x
    bad = (d > 1) & ((got.float() - want.float()).abs() > 3e-7 * pre.abs() + 1e-30)
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} beyond tolerance"
    assert float((d > 0).float().mean()) < 0.02
    # the reference's own producer at this shape: ReLU -> MXFP8, E8M0 bytes and codes
    q, s = ops.depthwise5x5_relu_mxfp8.get("sm100")(value.to(DEV), w.to(DEV), b.to(DEV))
    q_ref, s_ref = oracle.depthwise5x5_relu_mxfp8(value, w, b)
    assert float((s.cpu().view(torch.uint8) != s_ref).float().mean()) < 1e-4
    assert code_mismatch(q, q_ref) < 1e-3


@pytest.mark.parametrize("size,channels", [(100, 512), (200, 256), (400, 128)])
def test_config5_refiner_block_chunk(ops, size, channels):
    """One 8-image chunk of each pyramid level through one refiner block (depthwise + GELU -> MXFP8 -> 1x1 up + GELU ->
    MXFP8 -> 1x1 down + residual), the launch shapes of the stack benchmark."""
    import flashim_b200

    model = flashim_b200.load("refiner-stack", "fp8", device=DEV, overrides={"arch.levels": [[size, channels]], "arch.blocks": 1})
    level = oracle.make_refiner_level_weights(channels, 1, torch.Generator().manual_seed(4))
    g = torch.Generator().manual_seed(40)
    x = torch.randn(8, size, size, channels, generator=g).to(BF16)
    got = model.levels[0].blocks[0](x.to(DEV)).cpu()
    num = den = 0.0
    for i in range(0, 8, 2):  # the oracle two images at a time
        want = oracle.refiner_block_ext(x[i: i + 2], level["blocks"][0])
        num += float((got[i: i + 2].float() - want.float()).pow(2).sum())
        den += float(want.float().pow(2).sum())
    assert (num / den) ** 0.5 < 2e-3, (num / den) ** 0.5


def test_more_than_2_to_31_elements(ops):
    """Tensors of 21 x 400 x 400 x 640 = 2.15e9 elements through the quantiser, the depthwise producer and a 1x1 conv:
    every offset beyond 2**31 must be formed in 64 bits. The last image (the one furthest out) is checked."""
    from flashim_b200.quant import QuantizedWeight, swizzle_scales

    n, size, channels = 21, 400, 640
    assert n * size * size * channels > 2**31
    g = torch.Generator(device=DEV).manual_seed(31)
    x = torch.randn(n, size, size, channels, generator=g, device=DEV, dtype=BF16)
    last = x[-1:].cpu()

    q, scales = ops.quantize_mxfp8_dynamic.get("sm100")(x)
    q_ref, e_ref = oracle.quantize_rows_dynamic(last.reshape(-1, channels).float())
    assert same_bytes(q[-1].cpu().reshape(-1, channels), q_ref)
    rows = n * size * size
    plain = oracle.unswizzle_32_4_4(scales.cpu(), rows, channels // 32)
    assert torch.equal(plain[-size * size:], e_ref)

    cpu_gen = torch.Generator().manual_seed(32)
    weight = torch.empty(64, channels, 1, 1)
    torch.nn.init.kaiming_normal_(weight, generator=cpu_gen)
    packed = QuantizedWeight.from_conv(weight)
    bias = (torch.randn(64, generator=cpu_gen) * 0.02).to(BF16)
    out = ops.mxfp8_conv2d_fused.get("sm100")(
        q, scales, packed.values.to(DEV), swizzle_scales(packed.scale_exponent).to(DEV), bias.to(DEV), 1, 1, 1, 1, 0, 0, 1, 1)
    want = oracle.mxfp8_conv2d_ext(q_ref.reshape(1, size, size, channels), e_ref, packed.values, packed.scale_exponent, bias,
                                   1, 1, 1, 1, 0, 0, 1, 1)
    assert rel_l2(out[-1:], want) < 1e-3
    del q, scales, out

    w = (torch.randn(25, channels, generator=cpu_gen) * 0.05).to(BF16)
    b = torch.randn(channels, generator=cpu_gen)
    dq, ds = ops.depthwise5x5_act_mxfp8.get("sm100")(x.permute(0, 3, 1, 2), w.to(DEV), b.to(DEV), "relu")
    q_ref, s_ref = oracle.depthwise5x5_act_mxfp8_ext(last.permute(0, 3, 1, 2), w, b, "relu")
    assert code_mismatch(dq[-size * size:], q_ref) < 1e-3
    plain = oracle.unswizzle_32_4_4(ds.cpu(), rows, channels // 32)
    assert float((plain[-size * size:] != s_ref).float().mean()) < 1e-4
