"""tcgen05 implicit-GEMM convs against the CPU oracle, called through the op registry (and so through the C ABI)."""

import pytest
import torch
import torch.nn.functional as F

import oracle
from fim_testlib import DEV, bf16_ulp_distance, code_mismatch, rel_l2, same_bytes, to_dev

pytestmark = pytest.mark.gpu
E4M3, BF16 = torch.float8_e4m3fn, torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    import flashim_b200

    return flashim_b200.ops


def _mx_operands(batch, height, width, cin, cout, kh, kw, seed=0, bias=True):
    # operands drawn as flashim tests/ops/test_ops_cuda.py:608-636 draws them
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(batch, height, width, cin, generator=g) * 3).to(E4M3)
    ce = torch.randint(-6, 3, (cin // 32,), dtype=torch.int8, generator=g)
    w = (torch.randn(cout, kh * kw * cin, generator=g) * 2).to(E4M3)
    we = torch.randint(-9, -3, (cout, kh * kw * cin // 32), dtype=torch.int8, generator=g)
    b = torch.randn(cout, generator=g).to(BF16) if bias else None
    return x, ce, w, we, b


MX_CASES = [  # cin, cout, kh, kw, ph, pw, dh, dw, (B, H, W)
    (128, 128, 1, 1, 0, 0, 1, 1, (2, 17, 19)),
    (64, 64, 3, 3, 1, 1, 1, 1, (2, 17, 19)),
    (224, 128, 3, 3, 1, 1, 1, 1, (2, 17, 19)),
    (512, 64, 3, 3, 1, 1, 1, 1, (2, 17, 19)),
    (96, 64, 5, 5, 2, 2, 1, 1, (2, 17, 19)),
    (32, 32, 3, 3, 2, 2, 2, 2, (2, 17, 19)),
    (128, 256, 3, 3, 1, 1, 1, 1, (1, 40, 33)),
    (256, 96, 3, 3, 0, 0, 1, 1, (1, 12, 12)),
    (128, 128, 3, 3, 1, 1, 1, 1, (1, 64, 64)),
]


@pytest.mark.parametrize("case", MX_CASES)
@pytest.mark.parametrize("has_bias", [True, False])
def test_mxfp8_conv2d(ops, case, has_bias):
    cin, cout, kh, kw, ph, pw, dh, dw, (b, h, w) = case
    x, ce, wq, we, bias = _mx_operands(b, h, w, cin, cout, kh, kw, bias=has_bias)
    geometry = (kh, kw, 1, 1, ph, pw, dh, dw)
    want = oracle.mxfp8_conv2d(x, ce, wq, we, bias, *geometry)
    fast = ops.mxfp8_conv2d.get("sm100")
    got = fast(*to_dev(x, ce, wq, we, bias), *geometry)
    assert got.shape == want.shape and got.dtype == BF16
    assert rel_l2(got, want) < 1e-3  # the bar of flashim tests/ops/test_ops_cuda.py:634 and of the north star
    relu = fast(*to_dev(x, ce, wq, we, bias), *geometry, relu=True)
    assert same_bytes(relu, F.relu(got))  # ReLU commutes with the bf16 rounding


def test_mxfp8_conv2d_golden(ops, golden):
    g = golden("convs")
    for i, case in enumerate(g("cases").tolist()):
        cin, cout, kh, kw, sh, sw, ph, pw, dh, dw, has_bias, relu, has_res, requant = case
        if (sh, sw) != (1, 1):
            continue
        args = (g(f"mx{i}_x", E4M3), g(f"mx{i}_ce"), g(f"mx{i}_w", E4M3), g(f"mx{i}_we"), g.get(f"mx{i}_bias", BF16))
        res, oe = g.get(f"mx{i}_res", BF16), g.get(f"mx{i}_oe")
        got = ops.mxfp8_conv2d.get("sm100")(*to_dev(*args), kh, kw, sh, sw, ph, pw, dh, dw, relu=bool(relu),
                                            residual=to_dev(res), out_exponent=to_dev(oe))
        if requant:
            assert code_mismatch(got, g(f"mx{i}_out", E4M3)) < 2e-2
        else:
            assert rel_l2(got, g(f"mx{i}_out", BF16)) < 1e-3


@pytest.mark.parametrize("layout", ["nhwc", "nchw", "narrow"])
def test_residual_relu_epilogue(ops, layout):
    # flashim tests/ops/test_ops_cuda.py:778-807
    x, ce, wq, we, bias = _mx_operands(2, 17, 19, 64, 96, 3, 3)
    g = torch.Generator().manual_seed(9)
    channels = 64 if layout == "narrow" else 96
    res = torch.randn(2, channels, 17, 19, generator=g).to(BF16)
    res_d = res.to(DEV)
    if layout != "nchw":
        res_d = res_d.contiguous(memory_format=torch.channels_last)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    want = oracle.mxfp8_conv2d(x, ce, wq, we, bias, *geometry, relu=True, residual=res.permute(0, 2, 3, 1))
    got = ops.mxfp8_conv2d.get("sm100")(*to_dev(x, ce, wq, we, bias), *geometry, relu=True, residual=res_d.permute(0, 2, 3, 1))
    assert (got >= 0).all()
    plain = oracle.mxfp8_conv2d(x, ce, wq, we, bias, *geometry).float()
    bound = plain.abs() * 2**-7 + 1e-6
    bound[..., :channels] += res.permute(0, 2, 3, 1).float().abs() * 2**-7
    assert ((got.cpu().float() - want.float()).abs() <= bound).all()


@pytest.mark.parametrize("cin,mid,k", [(64, 64, 3), (128, 256, 1), (256, 128, 3)])
@pytest.mark.parametrize("relu", [True, False])
def test_static_requant_equals_separate_quantize(ops, cin, mid, k, relu):
    # flashim tests/quant/test_conv2d.py:79-102: the epilogue's E4M3 bytes are those of quantising its own bf16 output
    x, ce, wq, we, bias = _mx_operands(2, 21, 26, cin, mid, k, k, seed=2)
    geometry = (k, k, 1, 1, k // 2, k // 2, 1, 1)
    xd = to_dev(x, ce, wq, we, bias)
    plain = ops.mxfp8_conv2d.get("sm100")(*xd, *geometry, relu=relu)
    oe = oracle.static_block_exponent(plain.cpu().float())
    chained = ops.mxfp8_conv2d.get("sm100")(*xd, *geometry, relu=relu, out_exponent=to_dev(oe))
    assert chained.dtype == E4M3
    assert same_bytes(chained.cpu(), oracle.quantize_static_mx(plain.cpu(), oe))
    separate = ops.quantize_mxfp8.get("sm100")(plain, to_dev(oe))
    assert same_bytes(chained, separate.values)


@pytest.mark.parametrize("act", ["none", "gelu", "relu"])
@pytest.mark.parametrize("k", [1, 3])
def test_fused_epilogues(ops, act, k):
    """Extensions: GELU, fp32 output, dynamic requantisation (bytes equal to quantising the kernel's own bf16 output)."""
    from flashim_b200.quant import swizzle_scales

    x, ce, wq, we, bias = _mx_operands(2, 13, 15, 128, 128, k, k, seed=4)
    geometry = (k, k, 1, 1, k // 2, k // 2, 1, 1)
    fast = ops.mxfp8_conv2d_fused.get("sm100")
    ws = swizzle_scales(we)
    xd = to_dev(x, ce, wq, ws, bias)
    want = oracle.mxfp8_conv2d_ext(x, ce, wq, we, bias, *geometry, act=act)
    got = fast(*xd, *geometry, act=act)
    assert rel_l2(got, want) < 1e-3
    if act == "none":
        f32 = fast(*xd, *geometry, out_fp32=True)
        assert f32.dtype == torch.float32
        assert rel_l2(f32, oracle.mxfp8_conv2d_ext(x, ce, wq, we, bias, *geometry, out_fp32=True)) < 1e-4
        assert same_bytes(f32.to(BF16), got)
    q, s = fast(*xd, *geometry, act=act, dynamic_out=True)
    q_ref, e_ref = oracle.quantize_rows_dynamic(got.cpu().reshape(-1, 128))
    assert same_bytes(q.cpu().reshape(-1, 128), q_ref)
    assert torch.equal(s.cpu(), oracle.swizzle_32_4_4(e_ref))


@pytest.mark.parametrize("rows_shape", [(1, 8, 16), (2, 25, 31), (1, 1, 1)])
@pytest.mark.parametrize("cin,cout", [(128, 256), (256, 128), (64, 32)])
def test_per_pixel_scales_pointwise(ops, rows_shape, cin, cout):
    """1x1 conv fed by a dynamic producer: E8M0 scale per (pixel, 32 channels) in the swizzled layout
    (ops.mxfp8_scaled_mm semantics, flashim/ops/gemm.py:40-52)."""
    from flashim_b200.quant import swizzle_scales

    b, h, w = rows_shape
    g = torch.Generator().manual_seed(6)
    dense = torch.randn(b * h * w, cin, generator=g) * torch.exp2(torch.randint(-4, 4, (b * h * w, 1), generator=g).float())
    q, e = oracle.quantize_rows_dynamic(dense)
    wq = (torch.randn(cout, cin, generator=g) * 2).to(E4M3)
    we = torch.randint(-9, -3, (cout, cin // 32), dtype=torch.int8, generator=g)
    bias = torch.randn(cout, generator=g).to(BF16)
    res = torch.randn(b, h, w, cout, generator=g).to(BF16)
    x = q.reshape(b, h, w, cin)
    want = oracle.mxfp8_conv2d_ext(x, e, wq, we, bias, 1, 1, 1, 1, 0, 0, 1, 1, residual=res)
    got = ops.mxfp8_conv2d_fused.get("sm100")(
        *to_dev(x, oracle.swizzle_32_4_4(e), wq, swizzle_scales(we), bias), 1, 1, 1, 1, 0, 0, 1, 1, residual=to_dev(res))
    assert rel_l2(got, want) < 1e-3


def test_baseline_config1(ops, golden):
    """The benchmark's CPU-runnable case: fp32 NHWC [1, 64, 64, 128] from seed 0, 128 -> 128 3x3 pad 1, static MXFP8, fp32 / bf16 out."""
    g = golden("modules")
    torch.manual_seed(0)
    x = torch.randn(1, 64, 64, 128)
    ce = g("c1_exponent")
    wq, we, bias = g("c1_packed", E4M3), g("c1_packed_exponent"), g("c1_bias").to(BF16)
    q = ops.quantize_mxfp8.get("sm100")(to_dev(x), to_dev(ce))
    assert same_bytes(q.values.cpu(), oracle.quantize_static_mx(x, ce))
    got = ops.mxfp8_conv2d.get("sm100")(q.values, *to_dev(ce, wq, we, bias), 3, 3, 1, 1, 1, 1, 1, 1)
    want = oracle.mxfp8_conv2d(q.values.cpu(), ce, wq, we, bias, 3, 3, 1, 1, 1, 1, 1, 1)
    assert rel_l2(got, want) < 1e-3
    assert rel_l2(got[0, ::8, ::8], g("c1_out_sample", BF16)) < 1e-3
    assert float((bf16_ulp_distance(got.cpu(), want) > 1).float().mean()) < 1e-3


# -- INT8 ---------------------------------------------------------------------------------------------------------


INT8_CASES = [  # cin, cout, kh, kw, ph, pw, dh, dw  (flashim tests/ops/test_ops_cuda.py:455-468, the stride-1 / Cin % 32 rows)
    (64, 64, 3, 3, 1, 1, 1, 1),
    (64, 64, 1, 1, 0, 0, 1, 1),
    (32, 32, 3, 3, 2, 2, 2, 2),
    (512, 64, 3, 3, 1, 1, 1, 1),
    (96, 64, 5, 5, 2, 2, 1, 1),
    (256, 256, 3, 3, 1, 1, 1, 1),
]


@pytest.mark.parametrize("case", INT8_CASES)
@pytest.mark.parametrize("has_bias", [True, False])
def test_int8_conv2d_bit_exact(ops, case, has_bias):
    cin, cout, kh, kw, ph, pw, dh, dw = case
    g = torch.Generator().manual_seed(0)
    x = torch.randint(-127, 128, (2, 17, 19, cin), dtype=torch.int8, generator=g)
    w = torch.randint(-127, 128, (cout, kh * kw * cin), dtype=torch.int8, generator=g)
    a_scale = torch.tensor(0.017)
    w_scale = torch.rand(cout, generator=g) * 0.01 + 0.001
    bias = torch.randn(cout, generator=g).to(BF16) if has_bias else None
    geometry = (kh, kw, 1, 1, ph, pw, dh, dw)
    acc = ops.int8_conv2d_accumulators.get("sm100")(*to_dev(x, w), *geometry)
    assert acc.dtype == torch.int32
    assert torch.equal(acc.cpu(), oracle.int8_conv2d_accumulators_ext(x, w, *geometry))
    fast = ops.int8_conv2d.get("sm100")
    got = fast(*to_dev(x, w, a_scale, w_scale, bias), *geometry)
    want = oracle.int8_conv2d(x, w, a_scale, w_scale, bias, *geometry)
    assert same_bytes(got.cpu(), want)  # exact sums and a separately rounded multiply / add epilogue
    assert same_bytes(fast(*to_dev(x, w, a_scale, w_scale, bias), *geometry, relu=True), F.relu(got))


def test_int8_conv2d_golden_and_chain(ops, golden):
    g = golden("convs")
    for i, case in enumerate(g("cases").tolist()):
        cin, cout, kh, kw, sh, sw, ph, pw, dh, dw, has_bias, relu, has_res, requant = case
        if (sh, sw) != (1, 1):
            continue
        bias, res = g.get(f"mx{i}_bias", BF16), g.get(f"mx{i}_res", BF16)
        got = ops.int8_conv2d.get("sm100")(
            *to_dev(g(f"i8{i}_x"), g(f"i8{i}_w"), torch.tensor(0.017), g(f"i8{i}_ws"), bias), kh, kw, sh, sw, ph, pw, dh, dw,
            relu=bool(relu), residual=to_dev(res), out_scale=to_dev(torch.tensor(0.21)) if requant else None)
        want = g(f"i8{i}_out") if requant else g(f"i8{i}_out", BF16)
        assert same_bytes(got.cpu(), want), f"int8 golden case {i}"


@pytest.mark.parametrize("shape", [(2, 16, 20), (1, 17, 19), (3, 9, 8), (1, 2, 2), (1, 64, 66)])
@pytest.mark.parametrize("cin,cout,k", [(64, 64, 3), (32, 96, 1), (128, 256, 3)])
def test_int8_conv2d_maxpool(ops, shape, cin, cout, k):
    """int8_conv2d_maxpool (flashim/ops/conv.py:209-222): the bf16 conv output and its 2x2 max pool as INT8 codes, both
    byte-equal to the oracle; odd heights / widths drop the trailing row / column."""
    b, h, w = shape
    g = torch.Generator().manual_seed(5)
    x = torch.randint(-127, 128, (b, h, w, cin), dtype=torch.int8, generator=g)
    wt = torch.randint(-127, 128, (cout, k * k * cin), dtype=torch.int8, generator=g)
    w_scale = torch.rand(cout, generator=g) * 2e-4 + 1e-5
    bias = torch.randn(cout, generator=g).to(BF16)
    a_scale, out_scale = torch.tensor(0.03), torch.tensor(0.025)
    geometry = (k, k, 1, 1, k // 2, k // 2, 1, 1)
    for relu in (True, False):
        out, pooled = ops.int8_conv2d_maxpool.get("sm100")(*to_dev(x, wt, a_scale, w_scale, bias), *geometry, relu=relu,
                                                           out_scale=to_dev(out_scale))
        want_out, want_pooled = oracle.int8_conv2d_maxpool(x, wt, a_scale, w_scale, bias, *geometry, relu=relu, out_scale=out_scale)
        assert same_bytes(out.cpu(), want_out)
        assert pooled.dtype == torch.int8 and pooled.shape == want_pooled.shape
        assert torch.equal(pooled.cpu(), want_pooled)


def test_int8_conv2d_maxpool_golden(ops, golden):
    g = golden("widening")
    for i in range(3):
        k = int(g(f"pool{i}_k"))
        out, pooled = ops.int8_conv2d_maxpool.get("sm100")(
            *to_dev(g(f"pool{i}_x"), g(f"pool{i}_w"), torch.tensor(0.03), g(f"pool{i}_ws"), g(f"pool{i}_b", BF16)), k, k, 1, 1,
            k // 2, k // 2, 1, 1, relu=bool(i != 1), out_scale=to_dev(torch.tensor(0.02 + 0.01 * i)))
        assert same_bytes(out.cpu(), g(f"pool{i}_out", BF16)) and torch.equal(pooled.cpu(), g(f"pool{i}_pooled")), f"case {i}"


def test_baseline_config2(ops):
    """The benchmark's INT8 case: bf16 NHWC [2, 100, 100, 256] from seed 1, 256 -> 256 3x3 pad 1, int32 sums bit-exact, bf16 out."""
    torch.manual_seed(1)
    x = torch.randn(2, 100, 100, 256).to(BF16)
    weight = torch.empty(256, 256, 3, 3)
    torch.nn.init.kaiming_normal_(weight)
    bias = (torch.randn(256) * 0.02).to(BF16)
    a_scale = (x.float().abs().max() / 127).reshape(())
    wq, ws = oracle.pack_int8_conv_weight(weight)
    q = ops.quantize_int8.get("sm100")(to_dev(x), to_dev(a_scale))
    assert torch.equal(q.values.cpu(), oracle.quantize_int8(x, a_scale))
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    acc = ops.int8_conv2d_accumulators.get("sm100")(q.values, to_dev(wq), *geometry)
    assert torch.equal(acc.cpu(), oracle.int8_conv2d_accumulators_ext(q.values.cpu(), wq, *geometry))
    got = ops.int8_conv2d.get("sm100")(q.values, *to_dev(wq, a_scale, ws, bias), *geometry)
    assert same_bytes(got.cpu(), oracle.int8_conv2d(q.values.cpu(), wq, a_scale, ws, bias, *geometry))


def test_unsupported_geometry_raises(ops):
    """A geometry outside what the kernels cover (stride 5 here) raises: there is no fallback to hide behind."""
    from flashim_b200.ops import NoImplementation

    x, ce, wq, we, bias = _mx_operands(1, 9, 9, 64, 64, 3, 3)
    with pytest.raises(NoImplementation):
        ops.mxfp8_conv2d(*to_dev(x, ce, wq, we, bias), 3, 3, 5, 5, 1, 1, 1, 1)
    report = ops.mxfp8_conv2d.explain(*to_dev(x, ce, wq, we, bias), 3, 3, 1, 1, 1, 1, 1, 1)
    assert report["sm100"] == "selected"


def test_repeated_launches_are_identical(ops):
    x, ce, wq, we, bias = _mx_operands(2, 40, 44, 256, 256, 3, 3, seed=8)
    xd = to_dev(x, ce, wq, we, bias)
    first = ops.mxfp8_conv2d.get("sm100")(*xd, 3, 3, 1, 1, 1, 1, 1, 1)
    for _ in range(10):
        assert same_bytes(ops.mxfp8_conv2d.get("sm100")(*xd, 3, 3, 1, 1, 1, 1, 1, 1), first)


# -- CTA pairs (clusters of two CTAs on one cta_group::2 instruction stream) -----------------------------------------


@pytest.mark.parametrize("shape", [(3, 8, 16), (1, 40, 33), (5, 17, 19)])
def test_int8_cta_pairs_cover_odd_row_tiles(ops, shape):
    """256-wide INT8 tiles run as CTA pairs that own two row tiles each; an odd number of row tiles leaves the last
    pair with a tile that does not exist (zero-filled loads, clipped stores). Sums stay exact."""
    b, h, w = shape
    g = torch.Generator().manual_seed(5)
    x = torch.randint(-127, 128, (b, h, w, 128), dtype=torch.int8, generator=g)
    weight = torch.randint(-127, 128, (256, 9 * 128), dtype=torch.int8, generator=g)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    acc = ops.int8_conv2d_accumulators.get("sm100")(*to_dev(x, weight), *geometry)
    assert torch.equal(acc.cpu(), oracle.int8_conv2d_accumulators_ext(x, weight, *geometry))
    a_scale, w_scale = torch.tensor(0.02), torch.rand(256, generator=g) * 0.01 + 0.001
    bias = torch.randn(256, generator=g).to(BF16)
    got = ops.int8_conv2d.get("sm100")(*to_dev(x, weight, a_scale, w_scale, bias), *geometry, relu=True)
    assert same_bytes(got.cpu(), oracle.int8_conv2d(x, weight, a_scale, w_scale, bias, *geometry, relu=True))


@pytest.mark.parametrize("flags", [128, 64, 256, 16])
def test_mxfp8_conv2d_scheduling_variants_agree(ops, flags):
    """The tuning switches that keep results valid — CTA pairs for MXFP8 (128), no pairs (64), no resident weight scales
    (256), no half-width tail tiles (16) — must give the bits of the default schedule (same MMAs, same epilogue)."""
    from flashim_b200 import _native

    x, ce, wq, we, bias = _mx_operands(3, 24, 40, 256, 512, 3, 3, seed=4)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    fast = ops.mxfp8_conv2d.get("sm100")
    want = fast(*to_dev(x, ce, wq, we, bias), *geometry)
    assert rel_l2(want, oracle.mxfp8_conv2d(x, ce, wq, we, bias, *geometry)) < 1e-3
    lib = _native.library()
    try:
        lib.fim_conv_tune(0, 0, flags)
        got = fast(*to_dev(x, ce, wq, we, bias), *geometry)
    finally:
        lib.fim_conv_tune(0, 0, 0)
    assert same_bytes(got, want)


# -- GEMMs (a 1x1 conv over M pixels): flashim/ops/gemm.py:40-98 -------------------------------------------------------


def test_mxfp8_scaled_mm_and_int8_linear_golden(ops, golden):
    g = golden("gemms")
    for i in range(3):
        a, w = g(f"mm{i}_a", E4M3), g(f"mm{i}_w", E4M3)
        got = ops.mxfp8_scaled_mm.get("sm100")(to_dev(a), to_dev(w).t(), to_dev(g(f"mm{i}_sa")), to_dev(g(f"mm{i}_sw")),
                                               to_dev(g.get(f"mm{i}_bias", BF16)))
        assert rel_l2(got, g(f"mm{i}_out", BF16)) < 1e-3, f"scaled_mm case {i}"
        assert float((bf16_ulp_distance(got.cpu(), g(f"mm{i}_out", BF16)) > 1).float().mean()) < 1e-2
        args = to_dev(g(f"li{i}_a"), g(f"li{i}_w"), torch.tensor(0.02), g(f"li{i}_ws"), g(f"li{i}_b", BF16))
        fast = ops.int8_linear.get("sm100")
        assert same_bytes(fast(*args, relu=bool(i & 1)).cpu(), g(f"li{i}_out", BF16)), f"int8_linear case {i}"
        assert same_bytes(fast(*args, residual=to_dev(g(f"li{i}_res", BF16))).cpu(), g(f"li{i}_out_res", BF16))
    # what the kernel does not cover is declined, not approximated
    a8, w8, s, ws, b = to_dev(g("li0_a"), g("li0_w"), torch.tensor(0.02), g("li0_ws"), g("li0_b", BF16))
    assert ops.int8_linear.explain(a8, w8, s, ws, b, relu=True, gelu=True)["sm100"] != "selected"


# -- GELU in the epilogue ------------------------------------------------------------------------------------------------


@pytest.mark.parametrize("scale", [0.02, 0.3, 2.0, 40.0])
def test_epilogue_gelu_is_torch_gelu_of_the_rounded_sum(ops, scale):
    """The epilogue looks GELU up in a table of torch's own erf-form results for every bf16 value. Against the kernel's
    plain bf16 output the GELU output must therefore be torch's, bit for bit, whatever the magnitude of the sums (tiny
    values halve, large positive ones pass, large negative ones vanish); against the oracle it stays within one bf16 ulp
    wherever the two pre-activation roundings agree."""
    from flashim_b200.quant import swizzle_scales

    x, ce, wq, we, bias = _mx_operands(2, 21, 23, 128, 256, 3, 3, seed=12)
    bias = (bias.float() * scale).to(BF16)
    we = (we.int() + int(torch.tensor(scale).log2().round())).clamp(-100, 100).to(torch.int8)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    fast = ops.mxfp8_conv2d_fused.get("sm100")
    xd = to_dev(x, ce, wq, swizzle_scales(we), bias)
    plain = fast(*xd, *geometry, act="none").cpu()
    got = fast(*xd, *geometry, act="gelu").cpu()
    assert same_bytes(got, F.gelu(plain.float()).to(BF16))
    want_plain = oracle.mxfp8_conv2d_ext(x, ce, wq, we, bias, *geometry)
    want = oracle.mxfp8_conv2d_ext(x, ce, wq, we, bias, *geometry, act="gelu")
    agree = bf16_ulp_distance(plain, want_plain) == 0
    assert float(agree.float().mean()) > 0.9
    assert same_bytes(got[agree], want[agree])
    assert rel_l2(got, want) < 1e-3


def test_int8_epilogue_gelu_and_early_relu(ops):
    """INT8 conv with the GELU epilogue (the order of flashim/ops/gemm.py:87-98: scales + bias -> bf16 -> GELU ->
    residual): bit-equal to torch's GELU of the kernel's exact plain output plus the residual."""
    g = torch.Generator().manual_seed(3)
    x = torch.randint(-127, 128, (2, 17, 19, 64), dtype=torch.int8, generator=g)
    w = torch.randint(-127, 128, (96, 9 * 64), dtype=torch.int8, generator=g)
    a_scale, w_scale = torch.tensor(0.004), torch.rand(96, generator=g) * 0.002 + 0.0002
    bias = torch.randn(96, generator=g).to(BF16)
    res = torch.randn(2, 17, 19, 96, generator=g).to(BF16)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    plain = oracle.int8_conv2d(x, w, a_scale, w_scale, bias, *geometry)
    from flashim_b200.backends.sm100.kernels import int8_conv2d_launch
    from flashim_b200 import _native

    xd, wd, sd, wsd, bd, rd = to_dev(x, w, a_scale.reshape(1), w_scale, bias, res)
    got = int8_conv2d_launch(xd, wd, sd, wsd, bd, rd, None, 3, 3, 1, 1, 1, 1, 1, 1, _native.ACT["gelu"], _native.OUT_BF16)
    assert same_bytes(got.cpu(), res + F.gelu(plain.float()).to(BF16))
    early = int8_conv2d_launch(xd, wd, sd, wsd, bd, rd, None, 3, 3, 1, 1, 1, 1, 1, 1, _native.ACT["relu_early"], _native.OUT_BF16)
    assert same_bytes(early.cpu(), res + F.relu(plain))
