"""The persistent tile loop of the tcgen05 conv against the CPU oracle.

A launch normally has one CTA per SM, so a test-sized problem gives every CTA at most one tile and never exercises what
the full-size layers rely on: the accumulator double buffer changing phase from tile to tile, the stage ring wrapping
between tiles, weight scales kept resident in tensor memory while consecutive tiles share their output channels (and
reloaded when they do not), the channel-tile-major tile order, and the half-width tiles of the last partial round. Here
the grid is capped at 1, 3 or 5 CTAs, so each CTA walks many tiles, and the results are compared with the oracle and,
bit for bit, with the uncapped launch (the same MMAs and the same epilogue arithmetic per tile, only on another CTA).
"""

import pytest
import torch

import oracle
from fim_testlib import DEV, conv_schedule, rel_l2, same_bytes, to_dev

pytestmark = pytest.mark.gpu
E4M3, BF16 = torch.float8_e4m3fn, torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    import flashim_b200

    return flashim_b200.ops


def _mx_operands(batch, height, width, cin, cout, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(batch, height, width, cin, generator=g) * 3).to(E4M3)
    ce = torch.randint(-6, 3, (cin // 32,), dtype=torch.int8, generator=g)
    w = (torch.randn(cout, k * k * cin, generator=g) * 2).to(E4M3)
    we = torch.randint(-9, -3, (cout, k * k * cin // 32), dtype=torch.int8, generator=g)
    bias = torch.randn(cout, generator=g).to(BF16)
    return x, ce, w, we, bias


# (batch, height, width, cin, cout, k), forced block_n: every tile width, block_k 128 / 64 / 32, one and several channel tiles
STATIC_CASES = [
    ((2, 24, 30, 128, 64, 3), 0),      # 64-wide tiles, two accumulators
    ((2, 24, 30, 128, 128, 3), 0),     # 128-wide
    ((3, 20, 28, 128, 384, 3), 128),   # 128-wide, three channel tiles: resident scales reloaded when the channels change
    ((2, 24, 30, 256, 256, 3), 0),     # 256-wide, one accumulator
    ((2, 33, 17, 128, 512, 3), 256),   # 256-wide, two channel tiles
    ((2, 24, 30, 64, 256, 3), 0),      # block_k 64: no resident scales
    ((2, 24, 30, 64, 256, 3), 256),    # the same with one 256-wide accumulator
    ((2, 19, 23, 96, 128, 5), 0),      # block_k 32, 5x5 taps
    ((3, 40, 40, 256, 256, 1), 0),     # 1x1 over flattened pixels
]


@pytest.mark.parametrize("max_ctas", [1, 3, 5])
@pytest.mark.parametrize("case", STATIC_CASES, ids=lambda c: "b%dx%dx%d_c%d-%d_k%d_bn%d" % (*c[0], c[1]))
def test_static_scales_many_tiles_per_cta(ops, case, max_ctas):
    (b, h, w, cin, cout, k), block_n = case
    x, ce, wq, we, bias = _mx_operands(b, h, w, cin, cout, k, seed=11)
    geometry = (k, k, 1, 1, k // 2, k // 2, 1, 1)
    fast = ops.mxfp8_conv2d.get("sm100")
    xd = to_dev(x, ce, wq, we, bias)
    want = oracle.mxfp8_conv2d(x, ce, wq, we, bias, *geometry)
    with conv_schedule(block_n):
        uncapped = fast(*xd, *geometry)
    with conv_schedule(block_n, max_ctas) as capped:
        plan = capped.schedule((b, h, w, cin, cout, k, k, k // 2, 1))
        assert plan["ctas"] == max_ctas and plan["split_tiles"] > max_ctas  # more than one round
        got = fast(*xd, *geometry)
        oe = oracle.static_block_exponent(got.cpu().float())
        chained = fast(*xd, *geometry, relu=True, out_exponent=to_dev(oe))
    assert rel_l2(got, want) < 1e-3
    assert same_bytes(got, uncapped)
    # fused requantisation in the same multi-tile schedule = the oracle quantiser on the kernel's own output
    assert same_bytes(chained.cpu(), oracle.quantize_static_mx(torch.relu(got.cpu()), oe))


def test_resident_scales_and_tile_order_are_exercised():
    """The cases above cover both tile orders and both kinds of weight-scale traffic (what the schedule says it does)."""
    seen = set()
    for (b, h, w, cin, cout, k), block_n in STATIC_CASES:
        with conv_schedule(block_n, 3) as capped:
            plan = capped.schedule((b, h, w, cin, cout, k, k, k // 2, 1))
        seen.add((plan["resident_k"] > 0, plan["n_major"], plan["accumulators"]))
    assert (True, 1, 2) in seen and (True, 1, 1) in seen and (False, 0, 1) in seen and (False, 0, 2) in seen


@pytest.mark.parametrize("max_ctas,shape", [(5, (3, 16, 32)), (7, (5, 16, 24)), (3, (7, 16, 8))])
def test_half_width_tail_round(ops, max_ctas, shape):
    """256-wide tiles whose last round would leave more than half of the CTAs idle: that round runs as half-width tiles.
    The schedule must say so, and the bits must equal those of the full-width schedule (flag 16) and match the oracle."""
    b, h, w = shape
    cin, cout, k = 128, 256, 3
    x, ce, wq, we, bias = _mx_operands(b, h, w, cin, cout, k, seed=5)
    geometry = (k, k, 1, 1, 1, 1, 1, 1)
    fast = ops.mxfp8_conv2d.get("sm100")
    xd = to_dev(x, ce, wq, we, bias)
    with conv_schedule(256, max_ctas) as capped:
        plan = capped.schedule((b, h, w, cin, cout, k, k, 1, 1))
        assert plan["split_tiles"] > plan["tiles"] > plan["full_tiles"] >= max_ctas, plan  # the split is active
        split = fast(*xd, *geometry)
        q_split, s_split = ops.mxfp8_conv2d_fused.get("sm100")(
            xd[0], xd[1], xd[2], to_dev(oracle.swizzle_32_4_4(we)), xd[4], *geometry, act="gelu", dynamic_out=True)
    with conv_schedule(256, max_ctas, 16) as whole:
        plan = whole.schedule((b, h, w, cin, cout, k, k, 1, 1))
        assert plan["split_tiles"] == plan["tiles"] == plan["full_tiles"], plan
        full = fast(*xd, *geometry)
        q_full, s_full = ops.mxfp8_conv2d_fused.get("sm100")(
            xd[0], xd[1], xd[2], to_dev(oracle.swizzle_32_4_4(we)), xd[4], *geometry, act="gelu", dynamic_out=True)
    assert rel_l2(split, oracle.mxfp8_conv2d(x, ce, wq, we, bias, *geometry)) < 1e-3
    assert same_bytes(split, full) and same_bytes(q_split, q_full) and same_bytes(s_split, s_full)


@pytest.mark.parametrize("max_ctas", [1, 3, 5])
@pytest.mark.parametrize("cin,cout,block_n", [(128, 256, 0), (256, 128, 0), (128, 64, 0), (512, 512, 256), (64, 128, 0)])
def test_per_pixel_scales_many_tiles_per_cta(ops, cin, cout, block_n, max_ctas):
    """1x1 conv fed by a dynamic producer (one E8M0 scale per pixel and 32 channels, loaded per stage) with the GELU +
    dynamic requantisation epilogue and with the residual epilogue, each CTA walking many row tiles."""
    b, h, w = 2, 37, 41
    g = torch.Generator().manual_seed(6)
    dense = torch.randn(b * h * w, cin, generator=g) * torch.exp2(torch.randint(-4, 4, (b * h * w, 1), generator=g).float())
    q, e = oracle.quantize_rows_dynamic(dense)
    wq = (torch.randn(cout, cin, generator=g) * 2).to(E4M3)
    we = torch.randint(-9, -3, (cout, cin // 32), dtype=torch.int8, generator=g)
    bias = torch.randn(cout, generator=g).to(BF16)
    res = torch.randn(b, h, w, cout, generator=g).to(BF16)
    x = q.reshape(b, h, w, cin)
    point = (1, 1, 1, 1, 0, 0, 1, 1)
    fast = ops.mxfp8_conv2d_fused.get("sm100")
    xd = to_dev(x, oracle.swizzle_32_4_4(e), wq, oracle.swizzle_32_4_4(we), bias)
    want = oracle.mxfp8_conv2d_ext(x, e, wq, we, bias, *point, residual=res)
    with conv_schedule(block_n, max_ctas) as capped:
        plan = capped.schedule((b, h, w, cin, cout, 1, 1, 0, 1), per_pixel=True)
        assert plan["ctas"] == max_ctas and plan["split_tiles"] > 4 * max_ctas
        got = fast(*xd, *point, residual=to_dev(res))
        plain = fast(*xd, *point, act="gelu")
        hq, hs = fast(*xd, *point, act="gelu", dynamic_out=True)
    assert rel_l2(got, want) < 1e-3
    assert rel_l2(plain, oracle.mxfp8_conv2d_ext(x, e, wq, we, bias, *point, act="gelu")) < 1e-3
    q_ref, e_ref = oracle.quantize_rows_dynamic(plain.cpu().reshape(-1, cout))
    assert same_bytes(hq.cpu().reshape(-1, cout), q_ref) and torch.equal(hs.cpu(), oracle.swizzle_32_4_4(e_ref))
    with conv_schedule(block_n):
        assert same_bytes(fast(*xd, *point, residual=to_dev(res)), got)


@pytest.mark.parametrize("max_ctas", [2, 6, 10])
@pytest.mark.parametrize("shape", [(3, 24, 20), (5, 17, 19)])
def test_int8_pairs_many_tiles_per_pair(ops, shape, max_ctas):
    """INT8 256-wide tiles run as CTA pairs; with the grid capped a pair walks several tiles (and an odd number of row
    tiles leaves the last pair half empty). Sums and outputs stay exact."""
    b, h, w = shape
    g = torch.Generator().manual_seed(5)
    x = torch.randint(-127, 128, (b, h, w, 128), dtype=torch.int8, generator=g)
    weight = torch.randint(-127, 128, (512, 9 * 128), dtype=torch.int8, generator=g)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    a_scale, w_scale = torch.tensor(0.02), torch.rand(512, generator=g) * 0.01 + 0.001
    bias = torch.randn(512, generator=g).to(BF16)
    with conv_schedule(0, max_ctas) as capped:
        plan = capped.schedule((b, h, w, 128, 512, 3, 3, 1, 1), int8=True)
        assert plan["pairs"] == 1 and plan["ctas"] == max_ctas and plan["tiles"] >= 2 * (max_ctas // 2)
        acc = ops.int8_conv2d_accumulators.get("sm100")(*to_dev(x, weight), *geometry)
        got = ops.int8_conv2d.get("sm100")(*to_dev(x, weight, a_scale, w_scale, bias), *geometry, relu=True)
    assert torch.equal(acc.cpu(), oracle.int8_conv2d_accumulators_ext(x, weight, *geometry))
    assert same_bytes(got.cpu(), oracle.int8_conv2d(x, weight, a_scale, w_scale, bias, *geometry, relu=True))


@pytest.mark.parametrize("max_ctas", [3])
def test_mxfp8_pairs_many_tiles_per_pair_agree_with_single_ctas(ops, max_ctas):
    x, ce, wq, we, bias = _mx_operands(3, 24, 40, 256, 512, 3, seed=4)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    fast = ops.mxfp8_conv2d.get("sm100")
    xd = to_dev(x, ce, wq, we, bias)
    with conv_schedule(0, 2 * max_ctas, 128) as paired:
        assert paired.schedule((3, 24, 40, 256, 512, 3, 3, 1, 1))["pairs"] == 1
        got = fast(*xd, *geometry)
    with conv_schedule(0, 0, 64):
        want = fast(*xd, *geometry)
    assert same_bytes(got, want)
    assert rel_l2(got, oracle.mxfp8_conv2d(x, ce, wq, we, bias, *geometry)) < 1e-3


def test_int8_pairs_half_width_tail_round(ops):
    """CTA pairs also finish a sparse last round as half-width tiles (the benchmark's INT8 case has 79 pair tiles for 74 pairs):
    the schedule says so and the sums stay exact."""
    b, h, w = 3, 24, 20
    g = torch.Generator().manual_seed(8)
    x = torch.randint(-127, 128, (b, h, w, 128), dtype=torch.int8, generator=g)
    weight = torch.randint(-127, 128, (512, 9 * 128), dtype=torch.int8, generator=g)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    with conv_schedule(0, 10) as capped:
        plan = capped.schedule((b, h, w, 128, 512, 3, 3, 1, 1), int8=True)
        assert plan["pairs"] == 1 and plan["split_tiles"] > plan["tiles"] > plan["full_tiles"], plan
        acc = ops.int8_conv2d_accumulators.get("sm100")(*to_dev(x, weight), *geometry)
    assert torch.equal(acc.cpu(), oracle.int8_conv2d_accumulators_ext(x, weight, *geometry))
    with conv_schedule(0, 10, 16) as whole:
        plan = whole.schedule((b, h, w, 128, 512, 3, 3, 1, 1), int8=True)
        assert plan["split_tiles"] == plan["tiles"]
    config2 = conv_schedule().__enter__()
    try:
        plan = config2.schedule((2, 100, 100, 256, 256, 3, 3, 1, 1), int8=True)
        assert plan["pairs"] == 1 and plan["tiles"] == 80 and plan["split_tiles"] == 86, plan  # 74 whole tiles + 6 split in two
    finally:
        config2.__exit__()


@pytest.mark.parametrize("max_ctas", [3, 11])
@pytest.mark.parametrize("cin,cout", [(128, 256), (256, 256), (512, 256), (256, 128)])
def test_fixed_epilogues_agree_with_the_general_one(ops, cin, cout, max_ctas):
    """The three 1x1 layers of a refiner block (projection, up conv with GELU + dynamic requantisation, down conv with a
    residual) run through epilogues fixed at compile time; tuning flag 1024 sends the same call through the general
    epilogue, which must give the same bytes. With 11 CTAs the 24 tiles of the 256-wide cases end in a split round."""
    b, h, w = 2, 37, 41
    g = torch.Generator().manual_seed(16)
    dense = torch.randn(b * h * w, cin, generator=g) * torch.exp2(torch.randint(-4, 4, (b * h * w, 1), generator=g).float())
    q, e = oracle.quantize_rows_dynamic(dense)
    wq = (torch.randn(cout, cin, generator=g) * 2).to(E4M3)
    we = torch.randint(-9, -3, (cout, cin // 32), dtype=torch.int8, generator=g)
    bias = torch.randn(cout, generator=g).to(BF16)
    res = to_dev(torch.randn(b, h, w, cout, generator=g).to(BF16))
    point = (1, 1, 1, 1, 0, 0, 1, 1)
    fast = ops.mxfp8_conv2d_fused.get("sm100")
    xd = to_dev(q.reshape(b, h, w, cin), oracle.swizzle_32_4_4(e), wq, oracle.swizzle_32_4_4(we), bias)

    def three():
        up_q, up_s = fast(*xd, *point, act="gelu", dynamic_out=True)
        return fast(*xd, *point), fast(*xd, *point, residual=res), up_q, up_s

    with conv_schedule(0, max_ctas) as capped:
        plan = capped.schedule((b, h, w, cin, cout, 1, 1, 0, 1), per_pixel=True)
        if max_ctas == 11 and cout == 256 and cout >= cin:  # 256-wide tiles: 24 of them, the last two split
            assert plan["split_tiles"] > plan["tiles"]
        fixed = three()
    with conv_schedule(0, max_ctas, flags=1024):
        general = three()
    for a, b_ in zip(fixed, general):
        assert same_bytes(a, b_)
    want = oracle.mxfp8_conv2d_ext(q.reshape(b, h, w, cin), e, wq, we, bias, *point)
    assert rel_l2(fixed[0], want) < 1e-3


@pytest.mark.parametrize("case", [(2, 24, 30, 64, 64, 3), (2, 24, 30, 128, 128, 3), (2, 24, 30, 256, 256, 3), (2, 24, 30, 64, 64, 1)],
                         ids=lambda c: "c%d-%d_k%d" % c[3:])
def test_gelu_static_epilogue_with_fixed_switches_agrees_with_the_general_one(ops, case):
    """Bias + GELU + static requantisation, the epilogue of the conv shape sweep, runs with its switches fixed at compile
    time for each tile width's usual K step (64-wide tiles with both sets of epilogue warps draining alternate tiles);
    flag 1024 reads the switches at run time instead. Same bytes, and the oracle quantiser on the kernel's own bf16."""
    b, h, w, cin, cout, k = case
    x, ce, wq, we, bias = _mx_operands(b, h, w, cin, cout, k, seed=21)
    geometry = (k, k, 1, 1, k // 2, k // 2, 1, 1)
    fused = ops.mxfp8_conv2d_fused.get("sm100")
    xd = to_dev(x, ce, wq, oracle.swizzle_32_4_4(we), bias)
    with conv_schedule(0, 5):
        dense = fused(*xd, *geometry, act="gelu")
        oe = to_dev(oracle.static_block_exponent(dense.cpu().float()))
        fixed = fused(*xd, *geometry, act="gelu", out_exponent=oe)
    with conv_schedule(0, 5, flags=1024):
        general = fused(*xd, *geometry, act="gelu", out_exponent=oe)
    assert same_bytes(fixed, general)
    assert same_bytes(fixed.cpu(), oracle.quantize_static_mx(dense.cpu(), oe.cpu()))
    assert rel_l2(dense, oracle.mxfp8_conv2d_ext(x, ce, wq, we, bias, *geometry, act="gelu")) < 1e-3


def test_int8_bias_epilogue_with_fixed_switches_agrees_with_the_general_one(ops):
    b, h, w = 3, 24, 20
    g = torch.Generator().manual_seed(8)
    x = torch.randint(-127, 128, (b, h, w, 128), dtype=torch.int8, generator=g)
    weight = torch.randint(-127, 128, (256, 9 * 128), dtype=torch.int8, generator=g)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    a_scale, w_scale = torch.tensor(0.02), torch.rand(256, generator=g) * 0.01 + 0.001
    bias = torch.randn(256, generator=g).to(BF16)
    args = to_dev(x, weight, a_scale, w_scale, bias)
    with conv_schedule(0, 6) as capped:
        assert capped.schedule((b, h, w, 128, 256, 3, 3, 1, 1), int8=True)["pairs"] == 1
        fixed = ops.int8_conv2d.get("sm100")(*args, *geometry)
    with conv_schedule(0, 6, flags=1024):
        general = ops.int8_conv2d.get("sm100")(*args, *geometry)
    assert same_bytes(fixed, general)
    assert same_bytes(fixed.cpu(), oracle.int8_conv2d(x, weight, a_scale, w_scale, bias, *geometry))


@pytest.mark.parametrize("max_ctas", [0, 4, 10])
@pytest.mark.parametrize("case", [(2, 44, 52, 64, 64, 3), (3, 37, 41, 128, 256, 3), (2, 50, 50, 64, 96, 1), (1, 31, 78, 256, 512, 3)],
                         ids=lambda c: "%dx%dx%d_c%d-%d_k%d" % c)
def test_pool_in_the_int8_epilogue_over_many_tiles_per_cta(ops, case, max_ctas):
    """int8_conv2d_maxpool takes the 2x2 max pool from each bf16 tile while it lies in shared memory for its own store. With
    the CTAs capped every CTA (or CTA pair, at 256 output channels) walks several tiles, so the pooled panels are reused
    many times; odd heights and widths leave tiles with a dropped row or column, and 96 channels a partial channel tile.
    Both outputs equal the oracle's bytes, and the pooled one equals the separate pooling pass over the bf16 output."""
    b, h, w, cin, cout, k = case
    g = torch.Generator().manual_seed(h * w + cout)
    x = torch.randint(-127, 128, (b, h, w, cin), dtype=torch.int8, generator=g)
    weight = torch.randint(-127, 128, (cout, k * k * cin), dtype=torch.int8, generator=g)
    w_scale = torch.rand(cout, generator=g) * 2e-4 + 1e-5
    bias = torch.randn(cout, generator=g).to(BF16)
    a_scale, out_scale = torch.tensor(0.03), torch.tensor(0.04)
    geometry = (k, k, 1, 1, k // 2, k // 2, 1, 1)
    from flashim_b200.backends.sm100 import kernels
    with conv_schedule(0, max_ctas) as capped:
        if max_ctas:
            sched = capped.schedule((b, h, w, cin, cout, k, k, k // 2, 1), int8=True)
            assert sched["tiles"] >= 2 * sched["ctas"] // (2 if sched["pairs"] else 1)
        out, pooled = ops.int8_conv2d_maxpool.get("sm100")(*to_dev(x, weight, a_scale, w_scale, bias), *geometry, relu=True,
                                                           out_scale=to_dev(out_scale))
    want_out, want_pooled = oracle.int8_conv2d_maxpool(x, weight, a_scale, w_scale, bias, *geometry, relu=True, out_scale=out_scale)
    assert same_bytes(out.cpu(), want_out)
    assert pooled.shape == want_pooled.shape and torch.equal(pooled.cpu(), want_pooled)
    assert torch.equal(pooled, kernels.maxpool2_quantize_int8(out, to_dev(out_scale.reshape(1))))


@pytest.mark.parametrize("max_ctas", [0, 3, 11])
@pytest.mark.parametrize("case", [(2, 24, 30, 64, 64, 3), (2, 24, 30, 128, 128, 3), (2, 37, 41, 128, 256, 1), (2, 37, 41, 256, 128, 1),
                                  (2, 24, 30, 96, 64, 5)], ids=lambda c: "c%d-%d_k%d" % c[3:])
def test_resident_weights_agree_with_streamed_weights(ops, case, max_ctas):
    """A layer with one output-channel tile whose weight matrix fits in shared memory loads it once per CTA; flag 2048 streams
    it through the stage ring per tile and K step instead. Same bytes for the dense output, for GELU + static requantisation
    and (1x1) for GELU + dynamic requantisation, also where the last round of 256-wide tiles is split."""
    b, h, w, cin, cout, k = case
    x, ce, wq, we, bias = _mx_operands(b, h, w, cin, cout, k, seed=41)
    geometry = (k, k, 1, 1, k // 2, k // 2, 1, 1)
    fused = ops.mxfp8_conv2d_fused.get("sm100")
    xd = to_dev(x, ce, wq, oracle.swizzle_32_4_4(we), bias)

    def run():
        dense = fused(*xd, *geometry)
        oe = to_dev(oracle.static_block_exponent(torch.nn.functional.gelu(dense.float()).cpu()))
        outs = [dense, fused(*xd, *geometry, act="gelu", out_exponent=oe)]
        if k == 1:
            outs += list(fused(*xd, *geometry, act="gelu", dynamic_out=True))
        return outs

    with conv_schedule(0, max_ctas, flags=4096):  # resident at every tile width (the default keeps it to 64-wide tiles)
        resident = run()
    with conv_schedule(0, max_ctas, flags=2048):
        streamed = run()
    for a, b_ in zip(resident, streamed):
        assert same_bytes(a, b_)
    assert rel_l2(resident[0], oracle.mxfp8_conv2d(x, ce, wq, we, bias, *geometry)) < 1e-3


def test_int8_resident_weights_agree_with_streamed_weights(ops):
    b, h, w = 3, 24, 20
    g = torch.Generator().manual_seed(9)
    x = torch.randint(-127, 128, (b, h, w, 64), dtype=torch.int8, generator=g)
    weight = torch.randint(-127, 128, (128, 9 * 64), dtype=torch.int8, generator=g)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    a_scale, w_scale = torch.tensor(0.02), torch.rand(128, generator=g) * 0.01 + 0.001
    bias = torch.randn(128, generator=g).to(BF16)
    args = to_dev(x, weight, a_scale, w_scale, bias)
    with conv_schedule(0, 4, flags=4096):
        resident = ops.int8_conv2d.get("sm100")(*args, *geometry)
    with conv_schedule(0, 4, flags=2048):
        streamed = ops.int8_conv2d.get("sm100")(*args, *geometry)
    assert same_bytes(resident, streamed)
    assert same_bytes(resident.cpu(), oracle.int8_conv2d(x, weight, a_scale, w_scale, bias, *geometry))


def test_gelu_epilogue_inside_cta_pairs(ops):
    """GELU looks its values up in a shared-memory table through 16-bit address halves; inside a cluster the second CTA's
    shared-memory addresses carry its rank in their upper bits, which the look-up has to put back. INT8 pairs are the
    default for 256-wide tiles (an int8_linear with GELU on 640 rows reaches them); the MXFP8 pair runs under flag 128."""
    g = torch.Generator().manual_seed(12)
    a = torch.randint(-127, 128, (640, 1024), dtype=torch.int8, generator=g)
    w = torch.randint(-127, 128, (256, 1024), dtype=torch.int8, generator=g)
    a_scale, w_scale = torch.tensor(0.01), torch.rand(256, generator=g) * 0.002 + 0.0002
    bias = torch.randn(256, generator=g).to(BF16)
    with conv_schedule(0, 4) as capped:
        assert capped.schedule((1, 1, 640, 1024, 256, 1, 1, 0, 1), int8=True)["pairs"] == 1
        got = ops.int8_linear.get("sm100")(*to_dev(a, w, a_scale, w_scale, bias), gelu=True)
    assert same_bytes(got.cpu(), oracle.int8_linear(a, w, a_scale, w_scale, bias, gelu=True))

    x, ce, wq, we, bias = _mx_operands(3, 24, 40, 256, 256, 3, seed=14)
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    fused = ops.mxfp8_conv2d_fused.get("sm100")
    xd = to_dev(x, ce, wq, oracle.swizzle_32_4_4(we), bias)
    with conv_schedule(0, 0, 64):
        dense = fused(*xd, *geometry, act="gelu")
        oe = to_dev(oracle.static_block_exponent(dense.cpu().float()))
        single = fused(*xd, *geometry, act="gelu", out_exponent=oe)
    with conv_schedule(0, 6, 128) as paired:
        assert paired.schedule((3, 24, 40, 256, 256, 3, 3, 1, 1))["pairs"] == 1
        assert same_bytes(fused(*xd, *geometry, act="gelu"), dense)
        assert same_bytes(fused(*xd, *geometry, act="gelu", out_exponent=oe), single)


@pytest.mark.parametrize("max_ctas", [2, 6])
@pytest.mark.parametrize("shape,cout", [((3, 24, 20), 128), ((2, 17, 19), 384)])
def test_mxfp8_pairs_of_128_wide_tiles_agree_with_single_ctas(ops, shape, cout, max_ctas):
    """Large spatial convs run their 128-wide block-scaled tiles as CTA pairs (64 weight rows per CTA); flag 16384 forces
    the pair on a small problem, flag 64 forbids it. Same bytes with bias, with GELU + static requantisation (the
    epilogue whose switches are fixed at compile time) and with ReLU + residual; an odd number of row tiles leaves the
    last pair half empty, three channel tiles reload the resident weight scales."""
    b, h, w = shape
    x, ce, wq, we, bias = _mx_operands(b, h, w, 128, cout, 3, seed=23)
    res = to_dev(torch.randn(b, h, w, cout, generator=torch.Generator().manual_seed(2)).to(BF16))
    geometry = (3, 3, 1, 1, 1, 1, 1, 1)
    fused = ops.mxfp8_conv2d_fused.get("sm100")
    xd = to_dev(x, ce, wq, oracle.swizzle_32_4_4(we), bias)

    def run(oe):
        return (fused(*xd, *geometry), fused(*xd, *geometry, act="gelu", out_exponent=oe),
                fused(*xd, *geometry, act="relu", residual=res))

    with conv_schedule(0, max_ctas, 64) as single:
        assert single.schedule((b, h, w, 128, cout, 3, 3, 1, 1))["pairs"] == 0
        oe = to_dev(oracle.static_block_exponent(torch.nn.functional.gelu(fused(*xd, *geometry).float()).cpu()))
        want = run(oe)
    with conv_schedule(0, max_ctas, 16384) as paired:
        assert paired.schedule((b, h, w, 128, cout, 3, 3, 1, 1))["pairs"] == 1
        got = run(oe)
    for a, b_ in zip(got, want):
        assert same_bytes(a, b_)
    assert rel_l2(got[0], oracle.mxfp8_conv2d(x, ce, wq, we, bias, *geometry)) < 1e-3
