"""The 1x1 conv that takes bf16 activations and quantises them inside the kernel (converter warps between the TMA landing
ring and the MMA stage) against (1) the standalone quantiser followed by the conv on quantised activations — the same
bits are required — and (2) the CPU oracle of that pair."""
from __future__ import annotations

import pytest
import torch

import oracle
from fim_testlib import conv_schedule, rel_l2, same_bytes, to_dev

pytestmark = pytest.mark.gpu
E4M3, BF16 = torch.float8_e4m3fn, torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    import flashim_b200

    return flashim_b200.ops


def _layer(cin, cout, seed):
    g = torch.Generator().manual_seed(seed)
    b, h, w = 2, 37, 41  # 3034 rows: 24 row tiles, the last one ragged
    x = (torch.randn(b, h, w, cin, generator=g) * torch.exp2(torch.randint(-4, 4, (b, h, w, 1), generator=g).float())).to(BF16)
    wq = (torch.randn(cout, cin, generator=g) * 2).to(E4M3)
    we = torch.randint(-9, -3, (cout, cin // 32), dtype=torch.int8, generator=g)
    bias = torch.randn(cout, generator=g).to(BF16)
    res = torch.randn(b, h, w, cout, generator=g).to(BF16)
    return x, wq, we, bias, res


@pytest.mark.parametrize("max_ctas", [0, 3])
@pytest.mark.parametrize("cin,cout", [(128, 128), (256, 256), (512, 256), (128, 32), (256, 512)])
def test_dynamic_quantiser_inside_the_conv(ops, cin, cout, max_ctas):
    x, wq, we, bias, res = _layer(cin, cout, seed=31)
    point = (1, 1, 1, 1, 0, 0, 1, 1)
    inside = ops.mxfp8_conv2d_bf16.get("sm100")
    outside = ops.mxfp8_conv2d_fused.get("sm100")
    xd, wd, sd, bd, rd = to_dev(x, wq, oracle.swizzle_32_4_4(we), bias, res)
    with conv_schedule(0, max_ctas):
        q, s = ops.quantize_mxfp8_dynamic.get("sm100")(xd)
        for epilogue in ({}, {"residual": rd}, {"act": "gelu"}):
            assert same_bytes(inside(xd, None, wd, sd, bd, **epilogue), outside(q, s, wd, sd, bd, *point, **epilogue)), epilogue
        a_q, a_s = inside(xd, None, wd, sd, bd, act="gelu", dynamic_out=True)
        b_q, b_s = outside(q, s, wd, sd, bd, *point, act="gelu", dynamic_out=True)
        assert same_bytes(a_q, b_q) and same_bytes(a_s, b_s)
        plain = inside(xd, None, wd, sd, bd)
    rows_q, rows_e = oracle.quantize_rows_dynamic(x.reshape(-1, cin))
    want = oracle.mxfp8_conv2d_ext(rows_q.reshape(x.shape), rows_e, wq, we, bias, *point)
    assert rel_l2(plain, want) < 1e-3


@pytest.mark.parametrize("cin,cout", [(128, 128), (384, 256)])
def test_static_quantiser_inside_the_conv(ops, cin, cout):
    x, wq, we, bias, res = _layer(cin, cout, seed=32)
    point = (1, 1, 1, 1, 0, 0, 1, 1)
    ce = oracle.static_block_exponent(x.float())
    xd, ced, wd, sd, bd, rd = to_dev(x, ce, wq, oracle.swizzle_32_4_4(we), bias, res)
    inside = ops.mxfp8_conv2d_bf16.get("sm100")
    outside = ops.mxfp8_conv2d_fused.get("sm100")
    with conv_schedule(0, 5):
        q = ops.quantize_mxfp8.get("sm100")(xd, ced).values
        assert same_bytes(inside(xd, ced, wd, sd, bd), outside(q, ced, wd, sd, bd, *point))
        assert same_bytes(inside(xd, ced, wd, sd, bd, residual=rd), outside(q, ced, wd, sd, bd, *point, residual=rd))
        got = inside(xd, ced, wd, sd, bd)
    want = oracle.mxfp8_conv2d_ext(oracle.quantize_static_mx(x, ce), ce, wq, we, bias, *point)
    assert rel_l2(got, want) < 1e-3


def test_declines_what_the_converter_does_not_take(ops):
    x, wq, we, bias, _ = _layer(64, 64, seed=33)
    with pytest.raises(Exception):
        ops.mxfp8_conv2d_bf16.get("sm100")(*to_dev(x, None, wq, oracle.swizzle_32_4_4(we), bias))
