"""Comparison helpers shared by the test modules (imported by its own unique name: a `tests` package of another checkout
on sys.path must not be able to shadow it)."""

import os

import torch

def same_bytes(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Bitwise equality of two tensors of the same dtype family (fp8 / bf16 compared as integers)."""
    if a.shape != b.shape:
        return False
    size = a.element_size()
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[size]
    return torch.equal(a.contiguous().view(view), b.contiguous().view(view))


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in bf16 units in the last place between two bf16 tensors (monotone integer mapping of the bits)."""
    def key(t):
        bits = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(bits < 0, -(bits & 0x7FFF), bits)
    return (key(a) - key(b)).abs()


# Tests check the device status word after every launch (a kernel whose bounded wait ran out reports there).
os.environ.setdefault("FLASHIM_B200_CHECK", "1")

DEV = "cuda"


def to_dev(*tensors):
    out = tuple(None if t is None else t.to(DEV) for t in tensors)
    return out if len(out) > 1 else out[0]


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def code_mismatch(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.cpu().contiguous().view(torch.uint8) != b.cpu().contiguous().view(torch.uint8)).float().mean())


class conv_schedule:
    """Context manager around the schedule overrides of ``include/flashim_sm100_tune.h``: force the output-channel tile,
    cap the persistent grid (so a small problem makes every CTA walk many tiles) and pick between schedules that must
    all give the same bits."""

    def __init__(self, block_n: int = 0, max_ctas: int = 0, flags: int = 0) -> None:
        self.args = (block_n, max_ctas, flags)

    def __enter__(self):
        from flashim_b200 import _native

        self.lib = _native.library()
        self.lib.fim_conv_tune(*self.args)
        return self

    def __exit__(self, *exc):
        self.lib.fim_conv_tune(0, 0, 0)

    def schedule(self, geometry, int8: bool = False, per_pixel: bool = False) -> dict:
        """``fim_conv_schedule`` for (batch, height, width, cin, cout, kh, kw, pad, dilation) under the current overrides."""
        import ctypes

        from flashim_b200 import _native

        b, h, w, cin, cout, kh, kw, pad, dil = geometry
        g = _native.ConvGeometry(b, h, w, cin, cout, kh, kw, 1, 1, pad, pad, dil, dil)
        out = (ctypes.c_int * 8)()
        code = self.lib.fim_conv_schedule(ctypes.byref(g), int(int8), int(per_pixel), ctypes.byref(out))
        assert code == 0, code
        keys = ("tiles", "full_tiles", "split_tiles", "ctas", "pairs", "resident_k", "n_major", "accumulators")
        return dict(zip(keys, list(out)))
