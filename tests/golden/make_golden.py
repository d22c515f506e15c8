"""Generate ``tests/golden/*.npz`` by running the FlashIM reference implementation itself (CPU torch).

Usage (needs the reference checkout, which is not shipped with this repository)::

    FLASHIM_REFERENCE=/path/to/FlashIM python tests/golden/make_golden.py

Every array is stored as raw bytes (``uint8`` views for bf16 / E4M3 tensors) together with the inputs that produced
it, so the fixtures are independent of any random generator. ``tests/test_oracle_golden.py`` replays the inputs through
``oracle/`` and requires identical bytes.
"""

from __future__ import annotations

import hashlib
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REFERENCE = os.environ.get("FLASHIM_REFERENCE") or str(Path(__file__).resolve().parents[3] / "reference")  # a FlashIM checkout
sys.path.insert(0, REFERENCE)

from flashim import ops  # noqa: E402
from flashim.quant.formats import int8 as ref_int8  # noqa: E402
from flashim.quant.formats import mx as ref_mx  # noqa: E402
from flashim.quant.methods.conv2d import StaticInt8Conv2d, StaticMXFP8Conv2d  # noqa: E402
from flashim.quant.tensor import QuantizedWeight, quantize_int8_static, quantize_static  # noqa: E402


def raw(t: torch.Tensor) -> np.ndarray:
    """Bytes of a tensor with its shape kept (1-byte and 2-byte float dtypes become integer views)."""
    t = t.detach().contiguous()
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e8m0fnu):
        return t.view(torch.uint8).numpy()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def save(name: str, **arrays) -> None:
    np.savez_compressed(HERE / f"{name}.npz", **{k: raw(v) if isinstance(v, torch.Tensor) else np.asarray(v)
                                                   for k, v in arrays.items()})
    print(f"{name}.npz", {k: tuple(np.asarray(v).shape) if not isinstance(v, torch.Tensor) else tuple(v.shape)
                          for k, v in arrays.items()})


def boundary_amax() -> torch.Tensor:
    """amax values within +-64 ulp of ``448 * 2**k`` (where the fp32 log2 rule and the exact rule part ways: the flip
    point lies up to 39 ulp above the power of two, depending on the binade), plus zeros, tiny, huge and random values."""
    values = []
    for k in range(-60, 61):
        base = np.array([448.0 * 2.0**k], dtype=np.float32).view(np.int32)[0]
        values += [base + n for n in range(-64, 65)]
    edge = np.array(values, dtype=np.int32).view(np.float32)
    g = torch.Generator().manual_seed(10)
    rnd = torch.randn(4096, generator=g).abs() * torch.exp2(torch.randint(-30, 30, (4096,), generator=g).float())
    special = torch.tensor([0.0, 448.0, 449.0, 1.0, 1e-30, 1e30, 3.0e38, 1e-45])
    return torch.cat([torch.from_numpy(edge.copy()), rnd, special])


def formats() -> None:
    g = torch.Generator().manual_seed(11)
    amax = boundary_amax()
    x = (torch.randn(3, 5, 70, generator=g) * 4).to(torch.bfloat16)
    e_static = ref_mx.calibrate_block32_exponent(x)
    m = torch.randn(50, 96, generator=g) * torch.exp2(torch.randint(-8, 8, (50, 1), generator=g).float())
    m[7] = 0
    qd, ed = ref_mx.quantize_dynamic_2d(m)
    es = torch.randint(-20, 10, (300, 7), dtype=torch.int8, generator=g)
    w = torch.randn(100, 70, generator=g)
    qw = QuantizedWeight.from_float(w)
    xi = torch.randn(40, 33, generator=g) * 3
    si = torch.tensor(0.037)
    wi = torch.randn(16, 64, generator=g) * torch.rand(16, 1, generator=g) * 5
    wi[3] = 0
    save(
        "formats",
        amax=amax, amax_exponent=ref_mx.scale_exponent_from_amax(amax),
        static_in=x, static_exponent=e_static, static_out=quantize_static(x, e_static).values,
        dynamic_in=m, dynamic_out=qd, dynamic_exponent=ed,
        swizzle_in=es, swizzle_out=ref_mx.swizzle_scales(es),
        weight_in=w, weight_out=qw.values, weight_exponent=qw.scale_exponent,
        int8_in=xi, int8_scale=si, int8_out=quantize_int8_static(xi, si).values,
        int8_known_in=torch.tensor([[0.5, 1.5, 2.5, -0.5, 1000.0, -1000.0, 0.0]]),
        int8_known_out=quantize_int8_static(torch.tensor([[0.5, 1.5, 2.5, -0.5, 1000.0, -1000.0, 0.0]]),
                                            torch.tensor(1.0)).values,
        int8_weight_in=wi, int8_weight_scale=ref_int8.weight_scales(wi),
        int8_weight_out=ref_int8.quantize_symmetric(wi, ref_int8.weight_scales(wi)[:, None]),
    )


CONV_CASES = [  # cin, cout, kh, kw, sh, sw, ph, pw, dh, dw, bias, relu, residual, requant
    (64, 64, 3, 3, 1, 1, 1, 1, 1, 1, True, False, False, False),
    (64, 96, 3, 3, 1, 1, 1, 1, 1, 1, True, True, True, False),
    (128, 64, 1, 1, 1, 1, 0, 0, 1, 1, False, True, False, True),
    (32, 32, 3, 3, 2, 2, 1, 1, 1, 1, True, False, False, False),
    (32, 32, 3, 3, 1, 1, 2, 2, 2, 2, True, False, False, True),
    (96, 64, 5, 5, 1, 1, 2, 2, 1, 1, True, True, False, False),
]


def convs() -> None:
    g = torch.Generator().manual_seed(12)
    arrays = {"cases": np.array([[int(v) for v in case] for case in CONV_CASES], dtype=np.int32)}
    for i, (cin, cout, kh, kw, sh, sw, ph, pw, dh, dw, has_bias, relu, has_res, requant) in enumerate(CONV_CASES):
        k = kh * kw * cin
        # MXFP8: operands as the reference's block-scaled conv test draws them
        x = (torch.randn(2, 9, 11, cin, generator=g) * 3).to(torch.float8_e4m3fn)
        ce = torch.randint(-6, 3, (cin // 32,), dtype=torch.int8, generator=g)
        w = (torch.randn(cout, k, generator=g) * 2).to(torch.float8_e4m3fn)
        we = torch.randint(-9, -3, (cout, k // 32), dtype=torch.int8, generator=g)
        bias = torch.randn(cout, generator=g).to(torch.bfloat16) if has_bias else None
        geometry = (kh, kw, sh, sw, ph, pw, dh, dw)
        plain = ops.mxfp8_conv2d.get("reference")(x, ce, w, we, bias, *geometry)
        res = torch.randn(plain.shape, generator=g).to(torch.bfloat16) if has_res else None
        oe = ref_mx.calibrate_block32_exponent(plain.float().relu() if relu else plain.float()) if requant else None
        out = ops.mxfp8_conv2d.get("reference")(x, ce, w, we, bias, *geometry, relu=relu, residual=res, out_exponent=oe)
        arrays.update({f"mx{i}_x": raw(x), f"mx{i}_ce": raw(ce), f"mx{i}_w": raw(w), f"mx{i}_we": raw(we),
                       f"mx{i}_out": raw(out)})
        if bias is not None:
            arrays[f"mx{i}_bias"] = raw(bias)
        if res is not None:
            arrays[f"mx{i}_res"] = raw(res)
        if oe is not None:
            arrays[f"mx{i}_oe"] = raw(oe)
        # INT8
        xi = torch.randint(-127, 128, (2, 9, 11, cin), dtype=torch.int8, generator=g)
        wi = torch.randint(-127, 128, (cout, k), dtype=torch.int8, generator=g)
        a_scale = torch.tensor(0.017)
        w_scale = torch.rand(cout, generator=g) * 0.01 + 0.001
        o_scale = torch.tensor(0.21) if requant else None
        outi = ops.int8_conv2d.get("reference")(xi, wi, a_scale, w_scale, bias, *geometry, relu=relu, residual=res,
                                                out_scale=o_scale)
        arrays.update({f"i8{i}_x": raw(xi), f"i8{i}_w": raw(wi), f"i8{i}_ws": raw(w_scale), f"i8{i}_out": raw(outi)})
    save("convs", **arrays)


def depthwise() -> None:
    g = torch.Generator().manual_seed(13)
    arrays = {}
    for i, (c, h, w) in enumerate([(64, 9, 11), (32, 5, 3), (128, 7, 20)]):
        x = torch.randn(2, c, h, w, generator=g).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        weight = (torch.randn(25, c, generator=g) * 0.3).to(torch.bfloat16)
        bias = torch.randn(c, generator=g)
        if i == 1:
            bias[:] = -1e4  # every output is clipped by the ReLU: exponent -127 blocks
        q, s = ops.depthwise5x5_relu_mxfp8.get("reference")(x, weight, bias)
        qi = ops.depthwise5x5_relu_int8.get("reference")(x, weight, bias, torch.tensor(0.03))
        arrays.update({f"dw{i}_x": raw(x.permute(0, 2, 3, 1)), f"dw{i}_w": raw(weight), f"dw{i}_b": raw(bias),
                       f"dw{i}_q": raw(q), f"dw{i}_s": raw(s), f"dw{i}_i8": raw(qi)})
    save("depthwise", **arrays)


def modules() -> None:
    """Weight packing of the quantised conv modules, and the benchmark's CPU-runnable case ([1, 64, 64, 128], 128 -> 128 3x3) end to end through the module."""
    torch.manual_seed(0)
    x = torch.randn(1, 64, 64, 128)  # NHWC, config 1
    conv = torch.nn.Conv2d(128, 128, 3, 1, 1)
    torch.nn.init.kaiming_normal_(conv.weight)
    with torch.no_grad():
        conv.bias.copy_(torch.randn(128) * 0.02)
    ce = ref_mx.calibrate_block32_exponent(x)
    packed = StaticMXFP8Conv2d.from_conv(conv, ce)
    q = quantize_static(x, ce).values
    w = packed.weight_values.view(torch.float8_e4m3fn)
    out = ops.mxfp8_conv2d.get("reference")(q, ce, w, packed.weight_exponent, packed.bias_bf16, 3, 3, 1, 1, 1, 1, 1, 1)
    packed8 = StaticInt8Conv2d.from_conv(conv, torch.tensor(0.05))
    small = torch.nn.Conv2d(48, 40, 3, 1, 1)
    small_mx = StaticMXFP8Conv2d.from_conv(small, torch.zeros(2, dtype=torch.int8))
    save(
        "modules",
        c1_weight=conv.weight, c1_bias=conv.bias, c1_exponent=ce, c1_packed=w, c1_packed_exponent=packed.weight_exponent,
        c1_x_sample=x[0, :4, :4], c1_q_sample=q[0, :4, :4],
        c1_out_sample=out[0, ::8, ::8],
        c1_out_sha256=np.frombuffer(hashlib.sha256(raw(out).tobytes()).digest(), dtype=np.uint8),
        c1_int8_packed=packed8.weight_int8, c1_int8_scale=packed8.weight_scale,
        small_weight=small.weight, small_packed=small_mx.weight_values.view(torch.float8_e4m3fn),
        small_packed_exponent=small_mx.weight_exponent,
    )


def gemms() -> None:
    """Block-scaled MXFP8 GEMM and INT8 linear of the reference on small operands (rows and groups with padding)."""
    g = torch.Generator().manual_seed(17)
    arrays = {}
    for i, (m, k, n) in enumerate([(37, 64, 32), (130, 128, 96), (256, 256, 64)]):
        a = (torch.randn(m, k, generator=g) * 2).to(torch.float8_e4m3fn)
        w = (torch.randn(n, k, generator=g) * 2).to(torch.float8_e4m3fn)
        ae = torch.randint(-5, 4, (m, k // 32), dtype=torch.int8, generator=g)
        we = torch.randint(-8, -2, (n, k // 32), dtype=torch.int8, generator=g)
        bias = torch.randn(n, generator=g).to(torch.bfloat16) if i else None
        sa, sw = ref_mx.swizzle_scales(ae), ref_mx.swizzle_scales(we)
        out = ops.mxfp8_scaled_mm.get("reference")(a, w.t(), sa, sw, bias)
        arrays.update({f"mm{i}_a": raw(a), f"mm{i}_w": raw(w), f"mm{i}_ae": raw(ae), f"mm{i}_we": raw(we),
                       f"mm{i}_sa": raw(sa.view(torch.uint8)), f"mm{i}_sw": raw(sw.view(torch.uint8)), f"mm{i}_out": raw(out)})
        if bias is not None:
            arrays[f"mm{i}_bias"] = raw(bias)
        a8 = torch.randint(-127, 128, (m, k), dtype=torch.int8, generator=g)
        w8 = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g)
        ws = torch.rand(n, generator=g) * 0.01 + 0.001
        res = torch.randn(m, n, generator=g).to(torch.bfloat16)
        b8 = torch.randn(n, generator=g).to(torch.bfloat16)
        plain = ops.int8_linear.get("reference")(a8, w8, torch.tensor(0.02), ws, b8, relu=bool(i & 1))
        with_res = ops.int8_linear.get("reference")(a8, w8, torch.tensor(0.02), ws, b8, residual=res)
        arrays.update({f"li{i}_a": raw(a8), f"li{i}_w": raw(w8), f"li{i}_ws": raw(ws), f"li{i}_b": raw(b8), f"li{i}_res": raw(res),
                       f"li{i}_out": raw(plain), f"li{i}_out_res": raw(with_res)})
    save("gemms", **arrays)


def widening() -> None:
    """Ops either side of the conv: int8_conv2d_maxpool (flashim/ops/conv.py:209-222) with even and odd output sizes, and
    the static quantisers applied to the channels-last view of NCHW tensors (flashim/ops/quantize.py:80-100)."""
    g = torch.Generator().manual_seed(23)
    arrays = {}
    for i, (b, h, w, cin, cout, k) in enumerate([(2, 8, 10, 32, 32, 3), (1, 9, 7, 64, 64, 3), (1, 6, 6, 32, 64, 1)]):
        x = torch.randint(-127, 128, (b, h, w, cin), dtype=torch.int8, generator=g)
        wt = torch.randint(-127, 128, (cout, k * k * cin), dtype=torch.int8, generator=g)
        ws = torch.rand(cout, generator=g) * 2e-4 + 1e-5
        bias = torch.randn(cout, generator=g).to(torch.bfloat16)
        a_scale, out_scale = torch.tensor(0.03), torch.tensor(0.02 + 0.01 * i)
        out, pooled = ops.int8_conv2d_maxpool.get("reference")(x, wt, a_scale, ws, bias, k, k, 1, 1, k // 2, k // 2, 1, 1,
                                                               relu=bool(i != 1), out_scale=out_scale)
        arrays.update({f"pool{i}_x": raw(x), f"pool{i}_w": raw(wt), f"pool{i}_ws": raw(ws), f"pool{i}_b": raw(bias),
                       f"pool{i}_out": raw(out), f"pool{i}_pooled": raw(pooled), f"pool{i}_k": np.asarray(k)})
    for i, shape in enumerate([(2, 48, 5, 7), (1, 3, 4, 4), (1, 64, 6, 3)]):
        nchw = (torch.randn(*shape, generator=g) * 5).to(torch.bfloat16 if i else torch.float32)
        view = nchw.permute(0, 2, 3, 1)
        exponent = ref_mx.calibrate_block32_exponent(view)
        q = ops.quantize_mxfp8.get("reference")(view, exponent)
        arrays.update({f"cf{i}_x": raw(nchw), f"cf{i}_e": raw(exponent), f"cf{i}_q": raw(q.values)})
        if shape[1] % 16 == 0:
            arrays[f"cf{i}_i8"] = raw(ops.quantize_int8.get("reference")(view, torch.tensor(0.04)).values)
    for i, (b, c, h, w, prev_c) in enumerate([(2, 64, 7, 9, 1), (1, 128, 5, 6, 4), (1, 32, 3, 3, 4)]):
        z = torch.randn(b, c, h, w, generator=g).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        weight, bias = torch.randn(6, c, generator=g) * 0.3, torch.randn(6, generator=g)
        prev_warp = torch.rand(b, h, w, 2, generator=g) * 2 - 1
        prev_conf = torch.randn(b, h, w, prev_c, generator=g)
        warp, conf = ops.romav2_refiner_heads.get("reference")(z, weight, bias, prev_warp, prev_conf, 4.0)
        arrays.update({f"heads{i}_z": raw(z.permute(0, 2, 3, 1)), f"heads{i}_w": raw(weight), f"heads{i}_b": raw(bias),
                       f"heads{i}_pw": raw(prev_warp), f"heads{i}_pc": raw(prev_conf), f"heads{i}_warp": raw(warp),
                       f"heads{i}_conf": raw(conf)})
    for i, (b, h, w, p, e, radius, pair) in enumerate([(2, 6, 7, 32, 16, 3, 0), (2, 5, 4, 64, 8, 1, 1), (1, 4, 5, 16, 4, -1, 0)]):
        f_a, f_b = torch.randn(b, h, w, p, generator=g), torch.randn(b, h, w, p, generator=g)
        warp = torch.rand(b, h, w, 2, generator=g) * 2.6 - 1.3  # partly outside the image
        emb_w, emb_b = torch.randn(e, 2, 1, 1, generator=g), torch.randn(e, generator=g)
        out = ops.romav2_refiner_input.get("reference")(f_a, f_b, warp, emb_w, emb_b, torch.tensor([3.0, 2.0]), radius, pair)
        arrays.update({f"rin{i}_fa": raw(f_a), f"rin{i}_fb": raw(f_b), f"rin{i}_warp": raw(warp), f"rin{i}_ew": raw(emb_w),
                       f"rin{i}_eb": raw(emb_b), f"rin{i}_out": raw(out.permute(0, 2, 3, 1)),
                       f"rin{i}_cfg": np.asarray([radius, pair])})
    save("widening", **arrays)


def linears() -> None:
    """Static MXFP8 linear, the GELU MLP and its middle step, INT8 linear with the GELU and ReLU-before-residual epilogues,
    the bf16 depthwise + pointwise block and the two quantised composites (flashim/ops/gemm.py:58-157,
    flashim/ops/quantize.py:62-74, flashim/ops/conv.py:67-138)."""
    from flashim.quant.tensor import QuantizedTensor

    g = torch.Generator().manual_seed(29)
    arrays = {}
    for i, (rows, k, hidden, n) in enumerate([(77, 64, 128, 32), (300, 128, 256, 96)]):
        x = torch.randn(rows, k, generator=g).to(torch.bfloat16)
        xe = ref_mx.calibrate_block32_exponent(x)
        q = quantize_static(x, xe)
        w1 = QuantizedWeight.from_float(torch.randn(hidden, k, generator=g) * 0.2)
        w2 = QuantizedWeight.from_float(torch.randn(n, hidden, generator=g) * 0.2)
        b1 = (torch.randn(hidden, generator=g) * 0.3).to(torch.bfloat16)
        lin = ops.mxfp8_linear.get("reference")(q, b1, w1)
        he = ref_mx.calibrate_block32_exponent(torch.nn.functional.gelu(lin.float()))
        mlp = ops.mxfp8_gelu_mlp.get("reference")(q, w1, b1, he, w2)
        gq = ops.gelu_quantize.get("reference")(lin, he, input_bias=b1.float())
        gq_plain = ops.gelu_quantize.get("reference")(lin, he)
        arrays.update({f"lin{i}_x": raw(q.values), f"lin{i}_xe": raw(xe), f"lin{i}_w1": raw(w1.values), f"lin{i}_w1e": raw(w1.scale_exponent),
                       f"lin{i}_w2": raw(w2.values), f"lin{i}_w2e": raw(w2.scale_exponent), f"lin{i}_b1": raw(b1), f"lin{i}_he": raw(he),
                       f"lin{i}_out": raw(lin), f"lin{i}_mlp": raw(mlp), f"lin{i}_gq": raw(gq.values), f"lin{i}_gq_plain": raw(gq_plain.values)})
        a8 = torch.randint(-127, 128, (rows, k), dtype=torch.int8, generator=g)
        w8 = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g)
        ws = torch.rand(n, generator=g) * 0.002 + 0.0002
        b8 = torch.randn(n, generator=g).to(torch.bfloat16)
        res = torch.randn(rows, n, generator=g).to(torch.bfloat16)
        scale = torch.tensor(0.02)
        arrays.update({f"li{i}_a": raw(a8), f"li{i}_w": raw(w8), f"li{i}_ws": raw(ws), f"li{i}_b": raw(b8), f"li{i}_res": raw(res),
                       f"li{i}_gelu": raw(ops.int8_linear.get("reference")(a8, w8, scale, ws, b8, gelu=True)),
                       f"li{i}_gelu_res": raw(ops.int8_linear.get("reference")(a8, w8, scale, ws, b8, gelu=True, residual=res)),
                       f"li{i}_relu_res": raw(ops.int8_linear.get("reference")(a8, w8, scale, ws, b8, relu=True, residual=res))})
    for i, (b, c, h, w) in enumerate([(2, 32, 9, 11), (1, 64, 12, 7), (1, 128, 6, 10)]):
        value = torch.randn(b, c, h, w, generator=g).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        dw_w = (torch.randn(25, c, generator=g) * 0.2).to(torch.bfloat16)
        dw_b = torch.randn(c, generator=g)
        pw_w = (torch.randn(c, c, generator=g) * 0.2).to(torch.bfloat16)
        pw_b = torch.randn(c, generator=g).to(torch.bfloat16)
        out = ops.depthwise5x5_relu_pointwise.get("reference")(value, dw_w, dw_b, pw_w, pw_b)
        pq, pe = ref_mx.quantize_dynamic_2d(pw_w.float())
        fused = ops.depthwise5x5_relu_pointwise_mxfp8.get("reference")(
            value, dw_w, dw_b, pq, ref_mx.swizzle_scales(pe), ref_mx.exponent_to_e8m0(pe).view(torch.uint8), pw_b)
        w8 = torch.randint(-127, 128, (c, c), dtype=torch.int8, generator=g)
        ws = torch.rand(c, generator=g) * 0.002 + 0.0002
        fused8 = ops.depthwise5x5_relu_pointwise_int8.get("reference")(value, dw_w, dw_b, w8, ws, pw_b, torch.tensor(0.03))
        arrays.update({f"sep{i}_x": raw(value.permute(0, 2, 3, 1)), f"sep{i}_dw": raw(dw_w), f"sep{i}_db": raw(dw_b), f"sep{i}_pw": raw(pw_w),
                       f"sep{i}_pb": raw(pw_b), f"sep{i}_out": raw(out.permute(0, 2, 3, 1)), f"sep{i}_pq": raw(pq), f"sep{i}_pe": raw(pe),
                       f"sep{i}_mx": raw(fused.permute(0, 2, 3, 1)), f"sep{i}_w8": raw(w8), f"sep{i}_ws": raw(ws),
                       f"sep{i}_i8": raw(fused8.permute(0, 2, 3, 1))})
    save("linears", **arrays)


if __name__ == "__main__":
    torch.set_num_threads(8)
    which = sys.argv[1:] or ["formats", "convs", "depthwise", "modules", "gemms", "widening", "linears"]
    for name in which:
        globals()[name]()
