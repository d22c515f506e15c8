"""RoMaV2 refiner input kernel against the CPU oracle. Outputs are bf16 roundings of fp32 values computed in another
order (one bilinear blend of shared dot products instead of a blend per window sample): a value may land on the other
side of a bf16 rounding boundary, so the bar is 1 bf16 ulp, or 2e-5 absolute for values near zero."""

import pytest
import torch

import oracle
from fim_testlib import bf16_ulp_distance, to_dev

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    import flashim_b200

    return flashim_b200.ops


def _close(got, want, what, differing=0.02):
    assert got.dtype == BF16 and got.shape == want.shape, what
    got, want = got.cpu(), want.cpu()
    bad = (bf16_ulp_distance(got, want) > 1) & ((got.float() - want.float()).abs() > 2e-5)
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} beyond tolerance"
    if differing is not None:  # and almost all bytes are equal
        assert float((bf16_ulp_distance(got, want) > 0).float().mean()) < differing, what


CASES = [  # batch, h, w, P, E, radius, pair
    (2, 9, 11, 32, 16, 3, 0), (2, 8, 8, 64, 32, 2, 1), (1, 5, 7, 128, 8, 1, 0), (1, 6, 6, 16, 4, -1, 0), (4, 7, 5, 256, 64, 3, 2),
    (1, 1, 1, 8, 2, 0, 0), (1, 12, 10, 36, 5, 3, 0),
]


@pytest.mark.parametrize("case", CASES)
def test_refiner_input(ops, case):
    b, h, w, p, e, radius, pair = case
    g = torch.Generator().manual_seed(p + radius + 7)
    f_a, f_b = torch.randn(b, h, w, p, generator=g), torch.randn(b, h, w, p, generator=g)
    warp = torch.rand(b, h, w, 2, generator=g) * 2.6 - 1.3  # some positions outside the image: zeros padding
    emb_w, emb_b = torch.randn(e, 2, 1, 1, generator=g), torch.randn(e, generator=g)
    scale = torch.tensor([3.0, 2.0])
    want = oracle.romav2_refiner_input(f_a, f_b, warp, emb_w, emb_b, scale, radius, pair)
    got = ops.romav2_refiner_input.get("sm100")(*to_dev(f_a, f_b, warp, emb_w, emb_b, scale), radius, pair)
    assert got.is_contiguous(memory_format=torch.channels_last)
    k = (2 * radius + 1) ** 2 if radius >= 0 else 0
    assert got.shape == (b, 2 * p + e + k, h, w)
    assert torch.equal(got[:, :p].cpu(), want[:, :p])  # f_a: a plain rounding
    for name, lo, hi in (("warped f_b", p, 2 * p), ("embedding", 2 * p, 2 * p + e), ("correlation", 2 * p + e, 2 * p + e + k)):
        if hi > lo:
            _close(got[:, lo:hi], want[:, lo:hi], name)


def test_refiner_input_identity_warp_and_far_outside(ops):
    """The identity warp samples pixel centres exactly (f_b itself, correlation centre = <f_a, f_b> / sqrt(P)); a warp far
    outside the image gives zeros (and not-a-number coordinates do not fault)."""
    b, h, w, p = 1, 6, 8, 32
    g = torch.Generator().manual_seed(3)
    f_a, f_b = torch.randn(b, h, w, p, generator=g), torch.randn(b, h, w, p, generator=g)
    gy, gx = torch.meshgrid(torch.linspace(-1 + 1 / h, 1 - 1 / h, h), torch.linspace(-1 + 1 / w, 1 - 1 / w, w), indexing="ij")
    identity = torch.stack((gx, gy), dim=-1)[None].contiguous()
    emb_w, emb_b, scale = torch.zeros(4, 2), torch.zeros(4), torch.tensor([1.0, 1.0])
    got = ops.romav2_refiner_input.get("sm100")(*to_dev(f_a, f_b, identity, emb_w, emb_b, scale), 1, 0).cpu()
    want = oracle.romav2_refiner_input(f_a, f_b, identity, emb_w, emb_b, scale, 1, 0)
    # (samples that should vanish at the border are rounding noise of the order 1e-8 in both: no byte comparison here)
    _close(got[:, p:2 * p], want[:, p:2 * p], "warped f_b at the identity", differing=None)
    _close(got[:, 2 * p + 4:], want[:, 2 * p + 4:], "correlation at the identity", differing=None)
    centre = (f_a * f_b).sum(-1) / p**0.5
    assert torch.allclose(got[:, 2 * p + 4 + 4].float(), centre, rtol=1e-2, atol=1e-2)
    far = torch.full_like(identity, 40.0)
    far[0, 0, 0, 0] = float("nan")
    out = ops.romav2_refiner_input.get("sm100")(*to_dev(f_a, f_b, far, emb_w, emb_b, scale), 3, 0).cpu()
    sampled = torch.cat((out[:, p:2 * p], out[:, 2 * p + 4:]), dim=1).float()
    sampled[0, :, 0, 0] = 0.0  # the not-a-number coordinate: whatever comes out, the launch must survive it
    assert float(sampled.abs().max()) == 0.0


def test_refiner_input_golden(ops, golden):
    g = golden("widening")
    for i in range(3):
        radius, pair = (int(v) for v in g(f"rin{i}_cfg"))
        got = ops.romav2_refiner_input.get("sm100")(
            *to_dev(g(f"rin{i}_fa"), g(f"rin{i}_fb"), g(f"rin{i}_warp"), g(f"rin{i}_ew"), g(f"rin{i}_eb"), torch.tensor([3.0, 2.0])),
            radius, pair)
        _close(got.permute(0, 2, 3, 1), g(f"rin{i}_out", BF16), f"golden case {i}")
