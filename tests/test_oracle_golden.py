"""The CPU oracle against (1) the known-answer vectors the reference's own tests hold and (2) outputs of the reference
implementation itself, stored in ``tests/golden`` by ``tests/golden/make_golden.py``. Everything is bit-exact."""

import hashlib

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle
from fim_testlib import same_bytes

E4M3 = torch.float8_e4m3fn
BF16 = torch.bfloat16


# -- known-answer vectors from the reference's tests -------------------------------------------------------------


def test_exponent_rule_known_answers():
    # flashim tests/quant/test_mx_format.py:13-17
    amax = torch.tensor([0.0, 448.0, 449.0, 1.0, 1e-30])
    e = oracle.e8m0_exponent(amax)
    assert e.dtype == torch.int8 and e.tolist() == [-127, 0, 1, -8, -108]


def test_int8_rounds_half_even_and_saturates():
    # flashim tests/quant/test_int8.py:26-29
    x = torch.tensor([[0.5, 1.5, 2.5, -0.5, 1000.0, -1000.0, 0.0]])
    assert oracle.quantize_int8(x, torch.tensor(1.0)).tolist() == [[0, 2, 2, 0, 127, -127, 0]]


@pytest.mark.parametrize("channels", [32, 1000, 1024])
def test_static_quantize_roundtrip_and_saturation(channels):
    # flashim tests/quant/test_mx_format.py:20-35
    torch.manual_seed(0)
    x = torch.randn(7, 5, channels) * 10
    e = oracle.static_block_exponent(x)
    q = oracle.quantize_static_mx(x, e)
    assert q.shape == (7, 5, oracle.round_up32(channels))
    back = oracle.dequantize_mx(q, e)[..., :channels]
    scale = torch.exp2(e.float()).repeat_interleave(32)[:channels]
    assert ((back - x).abs() <= x.abs() * 2**-4 + scale * 2**-10 + 1e-12).all()
    big = oracle.dequantize_mx(oracle.quantize_static_mx(x * 1000, e), e)[..., :channels]
    assert torch.isfinite(big).all() and (big.abs() <= 448 * scale + 1e-3).all()


def test_weight_packing_pads_both_dimensions():
    # flashim tests/quant/test_mx_format.py:37-42
    torch.manual_seed(0)
    w = torch.randn(100, 70)
    q, e = oracle.pack_mx_weight(w)
    assert q.shape == (128, 96) and e.shape == (128, 3)
    scale = torch.exp2(e.float()).repeat_interleave(32, dim=1)[:100, :70]
    assert ((oracle.dequantize_mx(q, e)[:100, :70] - w).abs() <= w.abs() * 2**-4 + scale * 2**-10 + 1e-12).all()


@pytest.mark.parametrize("rows,groups", [(1, 1), (300, 32), (128, 4), (5000, 24)])
def test_swizzle_is_invertible(rows, groups):
    # flashim tests/quant/test_mx_format.py:45-52
    torch.manual_seed(0)
    e = torch.randint(-20, 10, (rows, groups), dtype=torch.int8)
    assert torch.equal(oracle.unswizzle_32_4_4(oracle.swizzle_32_4_4(e), rows, groups), e)


def test_swizzle_offset_formula():
    e = torch.randint(-20, 10, (300, 7), dtype=torch.int8)
    flat = oracle.swizzle_32_4_4(e)
    tiles = 2
    for r, g in [(0, 0), (31, 3), (32, 0), (127, 6), (128, 4), (299, 5)]:
        offset = ((r // 128) * tiles + g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4
        assert int(flat[offset]) == int(e[r, g]) + 127


def test_int8_weight_quantization_is_per_channel_symmetric():
    # flashim tests/quant/test_int8.py:17-23
    torch.manual_seed(0)
    w = torch.randn(16, 64) * torch.rand(16, 1) * 5
    s = oracle.int8_weight_scales(w)
    q = oracle.quantize_int8(w, s[:, None])
    assert q.dtype == torch.int8 and q.abs().amax(dim=1).eq(127).all()
    assert ((q.float() * s[:, None] - w).abs() <= s[:, None] / 2 + 1e-6).all()


def test_tap_gather_matches_unfold():
    # flashim tests/quant/test_conv2d.py:23-28
    torch.manual_seed(0)
    x = torch.randint(-127, 127, (2, 13, 17, 5), dtype=torch.int8)
    cols = oracle.gather_taps(x, 3, 3, 2, 2, 1, 1, 1, 1)
    ho, wo = oracle.conv_out_size(13, 3, 2, 1, 1), oracle.conv_out_size(17, 3, 2, 1, 1)
    ref = F.unfold(x.permute(0, 3, 1, 2).float(), 3, padding=1, stride=2)
    ref = ref.reshape(2, 5, 9, -1).permute(0, 3, 2, 1).reshape(2 * ho * wo, -1)
    assert torch.equal(cols.float(), ref)


@pytest.mark.parametrize("case", [(64, 64, 3, 1, 1, 1), (48, 96, 3, 1, 1, 1), (32, 128, 7, 2, 3, 1),
                                  (128, 128, 1, 1, 0, 1), (64, 64, 3, 2, 1, 1), (32, 32, 3, 1, 2, 2)])
@pytest.mark.parametrize("fmt", ["int8", "fp8"])
def test_conv_matches_float(case, fmt):
    # flashim tests/quant/test_conv2d.py:31-51 (tolerances 0.02 / 0.06 relative L2 against the float conv)
    cin, cout, k, s, p, d = case
    torch.manual_seed(0)
    conv = torch.nn.Conv2d(cin, cout, k, s, p, d).eval()
    x = torch.randn(2, cin, 20, 28)
    with torch.no_grad():
        ref = conv(x)
    nhwc = x.permute(0, 2, 3, 1).to(BF16)
    geometry = (k, k, s, s, p, p, d, d)
    if fmt == "int8":
        w, ws = oracle.pack_int8_conv_weight(conv.weight.detach())
        a_scale = x.abs().max() / 127
        out = oracle.int8_conv2d(oracle.quantize_int8(nhwc, a_scale), w, a_scale, ws,
                                 conv.bias.detach().to(BF16), *geometry)
    else:
        w, we = oracle.pack_mx_conv_weight(conv.weight.detach())
        ce = oracle.static_block_exponent(nhwc)
        bias = F.pad(conv.bias.detach(), (0, w.shape[0] - cout)).to(BF16)
        out = oracle.mxfp8_conv2d(oracle.quantize_static_mx(nhwc, ce), ce, w, we, bias, *geometry)[..., :cout]
    out = out.permute(0, 3, 1, 2).float()
    assert out.shape == ref.shape
    assert (out - ref).norm() / ref.norm() < (0.02 if fmt == "int8" else 0.06)


# -- outputs of the reference implementation ------------------------------------------------------------------------


def test_formats_against_reference(golden):
    g = golden("formats")
    assert torch.equal(oracle.e8m0_exponent(g("amax")), g("amax_exponent"))
    x = g("static_in", BF16)
    e = oracle.static_block_exponent(x)
    assert torch.equal(e, g("static_exponent"))
    assert same_bytes(oracle.quantize_static_mx(x, e), g("static_out", E4M3))
    q, de = oracle.quantize_rows_dynamic(g("dynamic_in"))
    assert same_bytes(q, g("dynamic_out", E4M3)) and torch.equal(de, g("dynamic_exponent"))
    assert torch.equal(oracle.swizzle_32_4_4(g("swizzle_in")), g("swizzle_out"))
    wq, we = oracle.pack_mx_weight(g("weight_in"))
    assert same_bytes(wq, g("weight_out", E4M3)) and torch.equal(we, g("weight_exponent"))
    assert torch.equal(oracle.quantize_int8(g("int8_in"), g("int8_scale")), g("int8_out"))
    assert torch.equal(oracle.quantize_int8(g("int8_known_in"), torch.tensor(1.0)), g("int8_known_out"))
    ws = oracle.int8_weight_scales(g("int8_weight_in"))
    assert torch.equal(ws, g("int8_weight_scale"))
    assert torch.equal(oracle.quantize_int8(g("int8_weight_in"), ws[:, None]), g("int8_weight_out"))


def test_convs_against_reference(golden):
    g = golden("convs")
    for i, case in enumerate(g("cases").tolist()):
        cin, cout, *geometry, has_bias, relu, has_res, requant = case
        bias = g.get(f"mx{i}_bias", BF16)
        res = g.get(f"mx{i}_res", BF16)
        out = oracle.mxfp8_conv2d(
            g(f"mx{i}_x", E4M3), g(f"mx{i}_ce"), g(f"mx{i}_w", E4M3), g(f"mx{i}_we"), bias, *geometry,
            relu=bool(relu), residual=res, out_exponent=g.get(f"mx{i}_oe"),
        )
        want = g(f"mx{i}_out", E4M3 if requant else BF16)
        assert same_bytes(out, want), f"mxfp8 case {i}"
        out = oracle.int8_conv2d(
            g(f"i8{i}_x"), g(f"i8{i}_w"), torch.tensor(0.017), g(f"i8{i}_ws"), bias, *geometry,
            relu=bool(relu), residual=res, out_scale=torch.tensor(0.21) if requant else None,
        )
        want = g(f"i8{i}_out") if requant else g(f"i8{i}_out", BF16)
        assert same_bytes(out, want), f"int8 case {i}"


def test_depthwise_against_reference(golden):
    g = golden("depthwise")
    for i in range(3):
        x = g(f"dw{i}_x", BF16).permute(0, 3, 1, 2)
        w, b = g(f"dw{i}_w", BF16), g(f"dw{i}_b")
        q, s = oracle.depthwise5x5_relu_mxfp8(x, w, b)
        assert same_bytes(q, g(f"dw{i}_q", E4M3)) and torch.equal(s, g(f"dw{i}_s"))
        assert torch.equal(oracle.depthwise5x5_relu_int8(x, w, b, torch.tensor(0.03)), g(f"dw{i}_i8"))
        if i == 1:  # every block clipped by the ReLU: exponent byte 0 (2**-127), all-zero codes
            assert int(q.view(torch.uint8).max()) == 0
            assert int(oracle.unswizzle_32_4_4(s, q.shape[0], 1).max()) == -127


def test_module_packing_and_config1_against_reference(golden):
    g = golden("modules")
    wq, we = oracle.pack_mx_conv_weight(g("c1_weight"))
    assert same_bytes(wq, g("c1_packed", E4M3)) and torch.equal(we, g("c1_packed_exponent"))
    w8, s8 = oracle.pack_int8_conv_weight(g("c1_weight"))
    assert torch.equal(w8, g("c1_int8_packed")) and torch.equal(s8, g("c1_int8_scale"))
    sq, se = oracle.pack_mx_conv_weight(g("small_weight"))
    assert same_bytes(sq, g("small_packed", E4M3)) and torch.equal(se, g("small_packed_exponent"))
    # the benchmark's CPU-runnable case regenerated from its seed: [1, 64, 64, 128] fp32 -> 128 -> 128 3x3, static MXFP8
    torch.manual_seed(0)
    x = torch.randn(1, 64, 64, 128)
    assert torch.equal(x[0, :4, :4], g("c1_x_sample"))
    ce = oracle.static_block_exponent(x)
    assert torch.equal(ce, g("c1_exponent"))
    q = oracle.quantize_static_mx(x, ce)
    assert same_bytes(q[0, :4, :4], g("c1_q_sample", E4M3))
    out = oracle.mxfp8_conv2d(q, ce, wq, we, g("c1_bias").to(BF16), 3, 3, 1, 1, 1, 1, 1, 1)
    assert same_bytes(out[0, ::8, ::8], g("c1_out_sample", BF16))
    digest = hashlib.sha256(out.contiguous().view(torch.int16).numpy().tobytes()).digest()
    assert np.frombuffer(digest, dtype=np.uint8).tolist() == g("c1_out_sha256").tolist()


# -- internal consistency of the extensions --------------------------------------------------------------------------


def test_extension_reduces_to_reference_op():
    torch.manual_seed(1)
    x = (torch.randn(1, 6, 7, 64) * 3).to(E4M3)
    ce = torch.randint(-6, 3, (2,), dtype=torch.int8)
    w = (torch.randn(64, 9 * 64) * 2).to(E4M3)
    we = torch.randint(-9, -3, (64, 18), dtype=torch.int8)
    b = torch.randn(64).to(BF16)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    res = torch.randn(1, 6, 7, 64).to(BF16)
    for relu in (False, True):
        for r in (None, res):
            a = oracle.mxfp8_conv2d(x, ce, w, we, b, *geometry, relu=relu, residual=r)
            e = oracle.mxfp8_conv2d_ext(x, ce, w, we, b, *geometry, act="relu" if relu else "none", residual=r)
            assert same_bytes(a, e)
    # per-pixel exponents that happen to be constant reproduce the static result
    x1 = (torch.randn(1, 6, 7, 64) * 3).to(E4M3)
    w1 = (torch.randn(96, 64) * 2).to(E4M3)
    we1 = torch.randint(-9, -3, (96, 2), dtype=torch.int8)
    a = oracle.mxfp8_conv2d_ext(x1, ce, w1, we1, None, 1, 1, 1, 1, 0, 0, 1, 1)
    e = oracle.mxfp8_conv2d_ext(x1, ce.expand(42, 2).contiguous(), w1, we1, None, 1, 1, 1, 1, 0, 0, 1, 1)
    assert same_bytes(a, e)


def test_refiner_level_runs_and_is_deterministic():
    g = torch.Generator().manual_seed(4)
    level = oracle.make_refiner_level_weights(64, 2, g)
    x = torch.randn(1, 10, 12, 64, generator=g).to(BF16)
    a, b = oracle.refiner_level_ext(x, level), oracle.refiner_level_ext(x, level)
    assert a.shape == (1, 10, 12, 32) and a.dtype == BF16 and same_bytes(a, b)
    assert torch.isfinite(a.float()).all()


def test_gemm_ops_match_reference_outputs(golden):
    """mxfp8_scaled_mm and int8_linear of the reference (flashim/ops/gemm.py:40-98) on operands with row / group padding."""
    g = golden("gemms")
    for i in range(3):
        a, w = g(f"mm{i}_a", E4M3), g(f"mm{i}_w", E4M3)
        assert same_bytes(oracle.swizzle_32_4_4(g(f"mm{i}_ae")), g(f"mm{i}_sa"))
        out = oracle.mxfp8_scaled_mm(a, w.t(), g(f"mm{i}_sa"), g(f"mm{i}_sw"), g.get(f"mm{i}_bias", BF16))
        assert same_bytes(out, g(f"mm{i}_out", BF16)), f"scaled_mm case {i}"
        args = (g(f"li{i}_a"), g(f"li{i}_w"), torch.tensor(0.02), g(f"li{i}_ws"), g(f"li{i}_b", BF16))
        assert same_bytes(oracle.int8_linear(*args, relu=bool(i & 1)), g(f"li{i}_out", BF16)), f"int8_linear case {i}"
        assert same_bytes(oracle.int8_linear(*args, residual=g(f"li{i}_res", BF16)), g(f"li{i}_out_res", BF16))


def test_widening_ops_match_reference_outputs(golden):
    """int8_conv2d_maxpool (flashim/ops/conv.py:209-222) and the static quantisers on the channels-last view of NCHW
    tensors (flashim/ops/quantize.py:80-100) against outputs of the reference itself."""
    g = golden("widening")
    for i in range(3):
        k = int(g(f"pool{i}_k"))
        out, pooled = oracle.int8_conv2d_maxpool(
            g(f"pool{i}_x"), g(f"pool{i}_w"), torch.tensor(0.03), g(f"pool{i}_ws"), g(f"pool{i}_b", BF16), k, k, 1, 1,
            k // 2, k // 2, 1, 1, relu=bool(i != 1), out_scale=torch.tensor(0.02 + 0.01 * i))
        assert same_bytes(out, g(f"pool{i}_out", BF16)), f"conv output, case {i}"
        assert torch.equal(pooled, g(f"pool{i}_pooled")), f"pooled codes, case {i}"
        nchw = g(f"cf{i}_x", BF16 if i else torch.float32)
        view = nchw.permute(0, 2, 3, 1)
        exponent = g(f"cf{i}_e")
        assert torch.equal(oracle.static_block_exponent(view), exponent)
        assert same_bytes(oracle.quantize_static_mx(view, exponent), g(f"cf{i}_q", E4M3))
        if nchw.shape[1] % 16 == 0:
            assert torch.equal(oracle.quantize_int8(view, torch.tensor(0.04)), g(f"cf{i}_i8"))


def test_refiner_heads_match_reference_outputs(golden):
    """romav2_refiner_heads (flashim/ops/romav2.py:95-120): same torch operations, so the fp32 outputs are identical."""
    g = golden("widening")
    for i in range(3):
        z = g(f"heads{i}_z", BF16).permute(0, 3, 1, 2)
        warp, conf = oracle.romav2_refiner_heads(z, g(f"heads{i}_w"), g(f"heads{i}_b"), g(f"heads{i}_pw"), g(f"heads{i}_pc"), 4.0)
        assert torch.equal(warp, g(f"heads{i}_warp")) and torch.equal(conf, g(f"heads{i}_conf")), f"case {i}"


def test_refiner_input_matches_reference_outputs(golden):
    """romav2_refiner_input (flashim/ops/romav2.py:36-66) incl. local correlation, stacked directions and warps that leave
    the image: the oracle batches the window samples differently, the bf16 bytes are the same."""
    g = golden("widening")
    for i in range(3):
        radius, pair = (int(v) for v in g(f"rin{i}_cfg"))
        out = oracle.romav2_refiner_input(g(f"rin{i}_fa"), g(f"rin{i}_fb"), g(f"rin{i}_warp"), g(f"rin{i}_ew"), g(f"rin{i}_eb"),
                                          torch.tensor([3.0, 2.0]), radius, pair)
        assert out.is_contiguous(memory_format=torch.channels_last)
        assert same_bytes(out.permute(0, 2, 3, 1), g(f"rin{i}_out", BF16)), f"case {i}"


def test_linear_mlp_and_separable_blocks_match_reference_outputs(golden):
    """Static MXFP8 linear, gelu_quantize, the GELU MLP, INT8 linear with GELU / ReLU-before-residual, the bf16 depthwise +
    pointwise block and the two quantised composites, bit for bit against outputs of the reference itself."""
    g = golden("linears")
    for i in range(2):
        x, xe = g(f"lin{i}_x", E4M3), g(f"lin{i}_xe")
        w1, w1e, w2, w2e = g(f"lin{i}_w1", E4M3), g(f"lin{i}_w1e"), g(f"lin{i}_w2", E4M3), g(f"lin{i}_w2e")
        b1, he = g(f"lin{i}_b1", BF16), g(f"lin{i}_he")
        lin = oracle.mxfp8_linear(x, xe, b1, w1, w1e)
        assert same_bytes(lin, g(f"lin{i}_out", BF16))
        assert same_bytes(oracle.gelu_quantize(lin, he, input_bias=b1.float()), g(f"lin{i}_gq", E4M3))
        assert same_bytes(oracle.gelu_quantize(lin, he), g(f"lin{i}_gq_plain", E4M3))
        assert same_bytes(oracle.mxfp8_gelu_mlp(x, xe, w1, w1e, b1, he, w2, w2e), g(f"lin{i}_mlp", BF16))
        args = (g(f"li{i}_a"), g(f"li{i}_w"), torch.tensor(0.02), g(f"li{i}_ws"), g(f"li{i}_b", BF16))
        res = g(f"li{i}_res", BF16)
        assert same_bytes(oracle.int8_linear(*args, gelu=True), g(f"li{i}_gelu", BF16))
        assert same_bytes(oracle.int8_linear(*args, gelu=True, residual=res), g(f"li{i}_gelu_res", BF16))
        assert same_bytes(oracle.int8_linear(*args, relu=True, residual=res), g(f"li{i}_relu_res", BF16))
    for i in range(3):
        value = g(f"sep{i}_x", BF16).permute(0, 3, 1, 2)
        dw, db, pw, pb = g(f"sep{i}_dw", BF16), g(f"sep{i}_db"), g(f"sep{i}_pw", BF16), g(f"sep{i}_pb", BF16)
        assert same_bytes(oracle.depthwise5x5_relu_pointwise(value, dw, db, pw, pb), g(f"sep{i}_out", BF16))
        pq, pe = g(f"sep{i}_pq", E4M3), g(f"sep{i}_pe")
        assert same_bytes(oracle.depthwise5x5_relu_pointwise_mxfp8(value, dw, db, pq, oracle.swizzle_32_4_4(pe), pb), g(f"sep{i}_mx", BF16))
        assert same_bytes(oracle.depthwise5x5_relu_pointwise_int8(value, dw, db, g(f"sep{i}_w8"), g(f"sep{i}_ws"), pb, torch.tensor(0.03)),
                          g(f"sep{i}_i8", BF16))
