"""RoMaV2 refiner heads kernel against the CPU oracle. The six dot products are fp32 sums of up to 512 terms in another
order than the oracle's: tolerance 2e-5 relative + 3e-5 absolute (a few ulp of the sum of the terms' magnitudes)."""

import pytest
import torch

import oracle
from fim_testlib import to_dev

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    import flashim_b200

    return flashim_b200.ops


def _close(got, want):
    assert got.dtype == torch.float32 and got.shape == want.shape
    assert torch.allclose(got.cpu(), want, rtol=2e-5, atol=3e-5), float((got.cpu() - want).abs().max())


@pytest.mark.parametrize("prev_channels", [1, 4])
@pytest.mark.parametrize("shape", [(2, 64, 17, 19), (1, 32, 1, 1), (1, 128, 40, 33), (3, 256, 5, 7), (1, 512, 9, 4), (1, 72, 6, 5)])
def test_refiner_heads(ops, shape, prev_channels):
    b, c, h, w = shape
    g = torch.Generator().manual_seed(c + prev_channels)
    z = torch.randn(b, c, h, w, generator=g).to(BF16).contiguous(memory_format=torch.channels_last)
    weight, bias = torch.randn(6, c, generator=g) * 0.3, torch.randn(6, generator=g) * 3  # softplus on both sides of 0 and of 20
    bias[3] += 25.0 if c == 64 else 0.0
    prev_warp = torch.rand(b, h, w, 2, generator=g) * 2 - 1
    prev_conf = torch.randn(b, h, w, prev_channels, generator=g)
    want_warp, want_conf = oracle.romav2_refiner_heads(z, weight, bias, prev_warp, prev_conf, 4.0)
    warp, conf = ops.romav2_refiner_heads.get("sm100")(*to_dev(z, weight, bias, prev_warp, prev_conf), 4.0)
    _close(warp, want_warp)
    _close(conf, want_conf)


def test_refiner_heads_golden_and_conv_weight_shape(ops, golden):
    g = golden("widening")
    for i in range(3):
        z = g(f"heads{i}_z", BF16).permute(0, 3, 1, 2)
        weight = g(f"heads{i}_w").reshape(6, -1, 1, 1)  # a 1x1 conv weight is accepted as it is
        warp, conf = ops.romav2_refiner_heads.get("sm100")(
            *to_dev(z, weight, g(f"heads{i}_b"), g(f"heads{i}_pw"), g(f"heads{i}_pc")), 4.0)
        _close(warp, g(f"heads{i}_warp"))
        _close(conf, g(f"heads{i}_conf"))


def test_refiner_heads_declines_what_it_cannot_read(ops):
    from flashim_b200.ops import NoImplementation

    z = torch.randn(1, 64, 4, 4, device="cuda", dtype=BF16)  # NCHW-contiguous, not channels-last
    args = (z, torch.zeros(6, 64, device="cuda"), torch.zeros(6, device="cuda"), torch.zeros(1, 4, 4, 2, device="cuda"),
            torch.zeros(1, 4, 4, 1, device="cuda"), 4.0)
    with pytest.raises(NoImplementation):
        ops.romav2_refiner_heads(*args)
