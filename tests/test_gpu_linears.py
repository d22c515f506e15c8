"""The linears, the GELU MLP, the depthwise-separable blocks and strided / bf16 convs against reference-generated fixtures
(tests/golden/linears.npz, convs.npz) and the CPU oracle."""

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


def _close_bf16(got, want, worst=1e-2):
    """Products of the same operands summed in another order: rel-L2 below 1e-3 and all but a few values within one ulp."""
    assert rel_l2(got, want) < 1e-3
    assert float((bf16_ulp_distance(got.cpu(), want) > 1).float().mean()) < worst


def test_mxfp8_linear_gelu_quantize_and_mlp_golden(ops, golden):
    from flashim_b200.quant import QuantizedTensor, QuantizedWeight

    g = golden("linears")
    for i in range(2):
        x = QuantizedTensor(g(f"lin{i}_x", E4M3).to(DEV), g(f"lin{i}_xe").to(DEV), tuple(g(f"lin{i}_x", E4M3).shape))
        w1 = QuantizedWeight(g(f"lin{i}_w1", E4M3).to(DEV), g(f"lin{i}_w1e").to(DEV), tuple(g(f"lin{i}_w1", E4M3).shape))
        w2 = QuantizedWeight(g(f"lin{i}_w2", E4M3).to(DEV), g(f"lin{i}_w2e").to(DEV), tuple(g(f"lin{i}_w2", E4M3).shape))
        b1, he = g(f"lin{i}_b1", BF16).to(DEV), g(f"lin{i}_he").to(DEV)
        lin = ops.mxfp8_linear.get("sm100")(x, b1, w1)
        _close_bf16(lin, g(f"lin{i}_out", BF16))
        # GELU -> quantise on the reference's own bf16 input: the bytes of the reference (erf in fp32, one code in a thousand
        # may sit on the other side of a rounding boundary between two erf implementations)
        ref_lin = g(f"lin{i}_out", BF16).to(DEV)
        gq = ops.gelu_quantize.get("sm100")(ref_lin, he, input_bias=b1.float())
        assert gq.scale_exponent is he and code_mismatch(gq.values, g(f"lin{i}_gq", E4M3)) < 1e-3
        assert code_mismatch(ops.gelu_quantize.get("sm100")(ref_lin, he).values, g(f"lin{i}_gq_plain", E4M3)) < 1e-3
        mlp = ops.mxfp8_gelu_mlp.get("sm100")(x, w1, b1, he, w2)
        assert mlp.shape == g(f"lin{i}_mlp", BF16).shape
        assert rel_l2(mlp, g(f"lin{i}_mlp", BF16)) < 5e-3  # a hidden code that flips moves an output by its whole quantum
    assert ops.call_counts()["mxfp8_gelu_mlp"] == {"sm100": 2}


def test_int8_linear_gelu_and_relu_before_residual_golden(ops, golden):
    g = golden("linears")
    fast = ops.int8_linear.get("sm100")
    for i in range(2):
        args = to_dev(g(f"li{i}_a"), g(f"li{i}_w"), torch.tensor(0.02), g(f"li{i}_ws"), g(f"li{i}_b", BF16))
        res = to_dev(g(f"li{i}_res", BF16))
        assert same_bytes(fast(*args, gelu=True).cpu(), g(f"li{i}_gelu", BF16))
        assert same_bytes(fast(*args, gelu=True, residual=res).cpu(), g(f"li{i}_gelu_res", BF16))
        assert same_bytes(fast(*args, relu=True, residual=res).cpu(), g(f"li{i}_relu_res", BF16))
    assert ops.int8_linear.explain(*args, relu=True, gelu=True)["sm100"] != "selected"  # declined, not approximated


def test_separable_blocks_golden(ops, golden):
    g = golden("linears")
    for i in range(3):
        value = g(f"sep{i}_x", BF16).permute(0, 3, 1, 2).to(DEV)
        dw, db = to_dev(g(f"sep{i}_dw", BF16), g(f"sep{i}_db"))
        pw, pb = to_dev(g(f"sep{i}_pw", BF16), g(f"sep{i}_pb", BF16))
        out = ops.depthwise5x5_relu_pointwise.get("sm100")(value, dw, db, pw, pb)
        assert out.shape == value.shape and out.is_contiguous(memory_format=torch.channels_last)
        _close_bf16(out.permute(0, 2, 3, 1), g(f"sep{i}_out", BF16), worst=2e-2)
        pq, pe = g(f"sep{i}_pq", E4M3), g(f"sep{i}_pe")
        mx = ops.depthwise5x5_relu_pointwise_mxfp8.get("sm100")(
            value, dw, db, pq.to(DEV), oracle.swizzle_32_4_4(pe).to(DEV), (pe.to(torch.int16) + 127).to(torch.uint8).to(DEV), pb)
        assert rel_l2(mx.permute(0, 2, 3, 1), g(f"sep{i}_mx", BF16)) < 5e-3
        i8 = ops.depthwise5x5_relu_pointwise_int8.get("sm100")(
            value, dw, db, g(f"sep{i}_w8").to(DEV), g(f"sep{i}_ws").to(DEV), pb, torch.tensor(0.03, device=DEV))
        assert rel_l2(i8.permute(0, 2, 3, 1), g(f"sep{i}_i8", BF16)) < 5e-3


@pytest.mark.parametrize("shape", [(2, 17, 19, 64, 96, 3), (1, 40, 33, 128, 128, 1), (3, 9, 50, 32, 64, 5), (1, 64, 64, 256, 64, 1)])
def test_bf16_conv(shape):
    """The bf16 tensor-core conv (kind::f16) against torch's fp32 conv of the same bf16 operands."""
    from flashim_b200 import _native
    from flashim_b200.backends.sm100.kernels import bf16_conv2d_launch

    b, h, w, cin, cout, k = shape
    g = torch.Generator().manual_seed(21)
    x = torch.randn(b, h, w, cin, generator=g).to(BF16)
    weight = (torch.randn(cout, cin, k, k, generator=g) * 0.2).to(BF16)
    bias = torch.randn(cout, generator=g).to(BF16)
    packed = weight.permute(0, 2, 3, 1).reshape(cout, -1).contiguous()  # (ky, kx, c)
    got = bf16_conv2d_launch(x.to(DEV), packed.to(DEV), bias.to(DEV), None, k, k, 1, 1, k // 2, k // 2, 1, 1, _native.ACT["relu"])
    want = F.relu(F.conv2d(x.permute(0, 3, 1, 2).float(), weight.float(), bias.float(), padding=k // 2)).to(BF16).permute(0, 2, 3, 1)
    _close_bf16(got, want, worst=2e-2)


STRIDED = [  # cin, cout, k, stride, pad, (B, H, W)
    (64, 64, 3, 2, 1, (2, 17, 19)),
    (128, 96, 3, 2, 1, (1, 40, 33)),
    (32, 224, 3, 2, 1, (2, 21, 26)),
    (64, 128, 1, 2, 0, (2, 16, 16)),
    (96, 64, 5, 3, 2, (1, 30, 31)),
    (256, 256, 3, 2, 1, (2, 64, 48)),
]


@pytest.mark.parametrize("case", STRIDED, ids=lambda c: "c%d-%d_k%d_s%d_p%d" % c[:5])
def test_strided_convs(ops, case):
    """Stride 2 and 3 through the tensor map's element strides, MXFP8 and INT8, against the oracle (flashim
    tests/ops/test_ops_cuda.py:608-636 includes stride 2)."""
    cin, cout, k, stride, pad, (b, h, w) = case
    g = torch.Generator().manual_seed(13)
    x = (torch.randn(b, h, w, cin, generator=g) * 3).to(E4M3)
    ce = torch.randint(-6, 3, (cin // 32,), dtype=torch.int8, generator=g)
    wq = (torch.randn(cout, k * k * cin, generator=g) * 2).to(E4M3)
    we = torch.randint(-9, -3, (cout, k * k * cin // 32), dtype=torch.int8, generator=g)
    bias = torch.randn(cout, generator=g).to(BF16)
    geometry = (k, k, stride, stride, pad, pad, 1, 1)
    want = oracle.mxfp8_conv2d(x, ce, wq, we, bias, *geometry, relu=True)
    got = ops.mxfp8_conv2d.get("sm100")(*to_dev(x, ce, wq, we, bias), *geometry, relu=True)
    assert got.shape == want.shape and rel_l2(got, want) < 1e-3
    xi = torch.randint(-127, 128, (b, h, w, cin), dtype=torch.int8, generator=g)
    wi = torch.randint(-127, 128, (cout, k * k * cin), dtype=torch.int8, generator=g)
    acc = ops.int8_conv2d_accumulators.get("sm100")(*to_dev(xi, wi), *geometry)
    assert torch.equal(acc.cpu(), oracle.int8_conv2d_accumulators_ext(xi, wi, *geometry))


def test_strided_golden_cases(ops, golden):
    """The strided cases of the reference-generated conv fixtures (skipped while the kernel had no strided form)."""
    g = golden("convs")
    seen = 0
    for i, case in enumerate(g("cases").tolist()):
        cin, cout, kh, kw, sh, sw, ph, pw, dh, dw, has_bias, relu, has_res, requant = case
        if (sh, sw) == (1, 1):
            continue
        seen += 1
        args = (g(f"mx{i}_x", E4M3), g(f"mx{i}_ce"), g(f"mx{i}_w", E4M3), g(f"mx{i}_we"), g.get(f"mx{i}_bias", BF16))
        if args[2].shape[0] % 32:
            continue  # an unpadded Cout: the module pads to 32 before it calls the op
        res, oe = g.get(f"mx{i}_res", BF16), g.get(f"mx{i}_oe")
        got = ops.mxfp8_conv2d.get("sm100")(*to_dev(*args), kh, kw, sh, sw, ph, pw, dh, dw, relu=bool(relu),
                                            residual=to_dev(res), out_exponent=to_dev(oe))
        if requant:
            assert code_mismatch(got, g(f"mx{i}_out", E4M3)) < 2e-2
        else:
            assert rel_l2(got, g(f"mx{i}_out", BF16)) < 1e-3
        bias, res = g.get(f"mx{i}_bias", BF16), g.get(f"mx{i}_res", BF16)
        got8 = ops.int8_conv2d.get("sm100")(
            *to_dev(g(f"i8{i}_x"), g(f"i8{i}_w"), torch.tensor(0.017), g(f"i8{i}_ws"), bias), kh, kw, sh, sw, ph, pw, dh, dw,
            relu=bool(relu), residual=to_dev(res), out_scale=to_dev(torch.tensor(0.21)) if requant else None)
        want8 = g(f"i8{i}_out") if requant else g(f"i8{i}_out", BF16)
        assert same_bytes(got8.cpu(), want8), f"int8 golden case {i}"
    assert seen >= 1
