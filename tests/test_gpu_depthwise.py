"""Depthwise 5x5 kernels against the CPU oracle."""

import pytest
import torch

import oracle
from fim_testlib import DEV, bf16_ulp_distance, code_mismatch, same_bytes, to_dev

pytestmark = pytest.mark.gpu
E4M3, BF16 = torch.float8_e4m3fn, torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    import flashim_b200

    return flashim_b200.ops


def _inputs(batch, channels, height, width, seed=3, wscale=0.05):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(batch, channels, height, width, generator=g).to(BF16).contiguous(memory_format=torch.channels_last)
    w = (torch.randn(25, channels, generator=g) * wscale).to(BF16)
    b = torch.randn(channels, generator=g)
    return x, w, b


def _assert_bf16_close(got, want, x_fp32=None):
    """1 bf16 ulp, or the fp32 cancellation floor of ``x * 0.5 * (1 + erf(x / sqrt 2))`` for strongly negative GELU
    arguments, where the reference's own value is dominated by the rounding of ``1 + erf``."""
    d = bf16_ulp_distance(got.cpu(), want)
    bad = d > 1
    if x_fp32 is not None:
        bad &= (got.cpu().float() - want.float()).abs() > 3e-7 * x_fp32.abs() + 1e-30
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} beyond tolerance, max ulp {int(d.max())}"


SHAPES = [(2, 64, 9, 11), (1, 32, 5, 3), (2, 128, 7, 20), (1, 64, 1, 1), (3, 192, 4, 7), (1, 64, 33, 50),
          (1, 256, 40, 45), (2, 64, 3, 130)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("act", ["gelu", "relu", "none"])
def test_depthwise_bf16(ops, shape, act):
    x, w, b = _inputs(*shape)
    want = oracle.depthwise5x5_act_ext(x, w, b, act)
    got = ops.depthwise5x5_act.get("sm100")(*to_dev(x, w, b), act)
    assert got.shape == want.shape and got.dtype == BF16
    pre = oracle.depthwise5x5_fp32(x, w, b).permute(0, 2, 3, 1) if act == "gelu" else None
    _assert_bf16_close(got, want, pre)


@pytest.mark.parametrize("channels,hw", [(32, (7, 9)), (128, (50, 50)), (512, (7, 9)), (64, (20, 33))])
def test_depthwise_relu_mxfp8(ops, channels, hw):
    # flashim tests/ops/test_ops_cuda.py:57-69: E8M0 bytes equal, E4M3 code mismatch < 1e-3, all-zero rows -> 2**-127
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, channels, *hw, generator=g).contiguous(memory_format=torch.channels_last)
    w = (torch.randn(25, channels, generator=g) * 0.3).to(BF16)
    b = torch.randn(channels, generator=g)
    q_ref, s_ref = oracle.depthwise5x5_relu_mxfp8(x, w, b)
    q, s = ops.depthwise5x5_relu_mxfp8.get("sm100")(*to_dev(x, w, b))
    assert q.dtype == E4M3 and q.shape == q_ref.shape
    assert float((s.cpu().view(torch.uint8) != s_ref).float().mean()) < 1e-4  # an amax 1 fp32 ulp apart at a 448*2**k edge
    assert code_mismatch(q, q_ref) < 1e-3
    z, zs = ops.depthwise5x5_relu_mxfp8.get("sm100")(*to_dev(x, w, torch.full_like(b, -1e4)))
    assert int(z.cpu().view(torch.uint8).max()) == 0
    rows = 2 * hw[0] * hw[1]
    assert int(oracle.unswizzle_32_4_4(zs.cpu().view(torch.uint8), rows, channels // 32).max()) == -127


def test_depthwise_golden(ops, golden):
    g = golden("depthwise")
    for i in range(3):
        x = g(f"dw{i}_x", BF16).permute(0, 3, 1, 2)
        w, b = g(f"dw{i}_w", BF16), g(f"dw{i}_b")
        q, s = ops.depthwise5x5_relu_mxfp8.get("sm100")(*to_dev(x, w, b))
        assert float((s.cpu().view(torch.uint8) != g(f"dw{i}_s")).float().mean()) < 2e-3
        assert code_mismatch(q, g(f"dw{i}_q", E4M3)) < 2e-3
        q8 = ops.depthwise5x5_relu_int8.get("sm100")(*to_dev(x, w, b, torch.tensor(0.03)))
        ref8 = g(f"dw{i}_i8")
        assert (q8.cpu().int() - ref8.int()).abs().max() <= 1 and float((q8.cpu() != ref8).float().mean()) < 5e-3


@pytest.mark.parametrize("channels,height,width", [(32, 20, 33), (128, 48, 40), (512, 12, 17), (64, 7, 1)])
def test_depthwise_relu_int8(ops, channels, height, width):
    # flashim tests/quant/test_int8.py (depthwise producer): +-1 code, < 5e-3 mismatches (fp32 tap order)
    x, w, b = _inputs(2, channels, height, width, seed=0, wscale=0.2)
    scale = torch.tensor(0.03)
    want = oracle.depthwise5x5_relu_int8(x, w, b, scale)
    got = ops.depthwise5x5_relu_int8.get("sm100")(*to_dev(x, w, b, scale))
    assert got.dtype == torch.int8 and got.shape == want.shape
    assert (got.cpu().int() - want.int()).abs().max() <= 1
    assert float((got.cpu() != want).float().mean()) < 5e-3


def test_fused_quantiser_equals_standalone_on_own_output(ops):
    """The MXFP8 epilogue quantises the kernel's own fp32 values: with act='none' and exactly representable inputs the
    dense bf16 output is exact, so both paths must agree byte for byte."""
    g = torch.Generator().manual_seed(5)
    x = torch.randint(-4, 5, (1, 64, 12, 14), generator=g).to(BF16).contiguous(memory_format=torch.channels_last)
    w = torch.randint(-2, 3, (25, 64), generator=g).to(BF16)
    b = torch.randint(-3, 4, (64,), generator=g).float()
    dense = ops.depthwise5x5_act.get("sm100")(*to_dev(x, w, b), "none")  # integers: exact in bf16
    assert same_bytes(dense.cpu(), oracle.depthwise5x5_act_ext(x, w, b, "none"))
    q, s = ops.depthwise5x5_act_mxfp8.get("sm100")(*to_dev(x, w, b), "none")
    q_ref, e_ref = oracle.quantize_rows_dynamic(dense.cpu().reshape(-1, 64))
    assert same_bytes(q.cpu(), q_ref) and torch.equal(s.cpu(), oracle.swizzle_32_4_4(e_ref))


def test_repeated_launches_are_identical(ops):
    # stage-reuse race guard, after flashim tests/ops/test_ops_cuda.py:77-95
    x, w, b = _inputs(3, 128, 50, 70, seed=2, wscale=0.3)
    xd, wd, bd = to_dev(x, w, b)
    first = ops.depthwise5x5_relu_mxfp8.get("sm100")(xd, wd, bd)
    for _ in range(20):
        q, s = ops.depthwise5x5_relu_mxfp8.get("sm100")(xd, wd, bd)
        assert same_bytes(q, first[0]) and same_bytes(s, first[1])


def test_layout_handling(ops):
    x, w, b = _inputs(1, 64, 10, 12)
    want = oracle.depthwise5x5_act_ext(x, w, b, "relu")
    nchw = x.contiguous()  # not channels-last: the wrapper copies
    got = ops.depthwise5x5_act.get("sm100")(*to_dev(nchw, w, b), "relu")
    _assert_bf16_close(got, want)
    assert "sm100" in ops.depthwise5x5_act.explain(*to_dev(x, w, b), "relu")
    assert ops.depthwise5x5_act.explain(*to_dev(x, w, b), "relu")["sm100"] == "selected"


@pytest.mark.parametrize("variant", [1, 2, 3, 4])
def test_every_thread_layout_gives_the_same_results(ops, variant):
    """The kernel is compiled for several thread layouts (columns per lane x warps per CTA); the launcher picks one by
    image width. Each is forced in turn: dense outputs must be the bits of the automatic choice (the FMA order per
    element is the same), quantised outputs too."""
    from flashim_b200 import _native

    lib = _native.library()
    x, w, b = _inputs(2, 192, 37, 45, seed=7, wscale=0.2)
    xd, wd, bd = to_dev(x, w, b)
    scale = to_dev(torch.tensor(0.03))
    want = {
        "gelu": ops.depthwise5x5_act.get("sm100")(xd, wd, bd, "gelu"),
        "mx": ops.depthwise5x5_act_mxfp8.get("sm100")(xd, wd, bd, "gelu"),
        "relu_mx": ops.depthwise5x5_relu_mxfp8.get("sm100")(xd, wd, bd),
        "int8": ops.depthwise5x5_relu_int8.get("sm100")(xd, wd, bd, scale),
    }
    _assert_bf16_close(want["gelu"], oracle.depthwise5x5_act_ext(x, w, b, "gelu"), oracle.depthwise5x5_fp32(x, w, b).permute(0, 2, 3, 1))
    try:
        lib.fim_dw_tune(variant, 0)
        assert same_bytes(ops.depthwise5x5_act.get("sm100")(xd, wd, bd, "gelu"), want["gelu"])
        q, s = ops.depthwise5x5_act_mxfp8.get("sm100")(xd, wd, bd, "gelu")
        assert same_bytes(q, want["mx"][0]) and same_bytes(s, want["mx"][1])
        q, s = ops.depthwise5x5_relu_mxfp8.get("sm100")(xd, wd, bd)
        assert same_bytes(q, want["relu_mx"][0]) and same_bytes(s.view(torch.uint8), want["relu_mx"][1].view(torch.uint8))
        assert same_bytes(ops.depthwise5x5_relu_int8.get("sm100")(xd, wd, bd, scale), want["int8"])
    finally:
        lib.fim_dw_tune(0, 0)


def test_gelu_mxfp8_against_the_oracle(ops):
    """Depthwise + GELU quantised straight from fp32: E8M0 bytes equal the oracle's but for block maxima within rounding of
    a 448 * 2**k edge, and fewer than one code in a thousand differs."""
    x, w, b = _inputs(2, 128, 40, 52, seed=4, wscale=0.2)
    q, s = ops.depthwise5x5_act_mxfp8.get("sm100")(*to_dev(x, w, b), "gelu")
    q_ref, e_ref = oracle.depthwise5x5_act_mxfp8_ext(x, w, b, "gelu")
    assert float((s.cpu() != oracle.swizzle_32_4_4(e_ref)).float().mean()) < 1e-4
    assert code_mismatch(q, q_ref) < 1e-3
