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
