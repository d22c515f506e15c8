"""Build ``flashim_b200/_lib/libflashim_sm100.so`` from ``flashim_b200/csrc/*.cu`` with ``nvcc`` for sm_100a.

``python -m flashim_b200.build_native [--force]``. The arch flag must carry the ``a`` suffix: tcgen05 / tensor-memory
instructions do not exist in the forward-compatible ``sm_100`` target. The build is atomic (temporary file + rename),
so concurrent processes (one per GPU) can call it at the same time.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
SOURCES = ("quantize.cu", "depthwise.cu", "conv.cu", "refiner_heads.cu", "refiner_input.cu")
HEADERS = ("common.cuh",)
INCLUDE = PACKAGE.parent / "include"
OUTPUT = PACKAGE / "_lib" / "libflashim_sm100.so"
FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC")


def nvcc_path() -> str | None:
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if home and (Path(home) / "bin" / "nvcc").is_file():
            return str(Path(home) / "bin" / "nvcc")
    return shutil.which("nvcc")


def source_digest() -> str:
    h = hashlib.sha256(" ".join(FLAGS).encode())
    for name in (*SOURCES, *HEADERS):
        h.update((PACKAGE / "csrc" / name).read_bytes())
    for name in ("flashim_sm100.h", "flashim_sm100_tune.h"):
        h.update((INCLUDE / name).read_bytes())
    return h.hexdigest()[:16]


def build(force: bool = False, verbose: bool = False, output: Path = OUTPUT, defines: tuple[str, ...] = ()) -> Path:
    """Build the library (``output`` and ``defines`` serve measurement builds, e.g. ``-DFIM_PROBE_BUILD=1``)."""
    OUTPUT = output
    stamp = OUTPUT.with_suffix(".digest")
    digest = source_digest() + "".join(defines)
    if not force and OUTPUT.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
        return OUTPUT
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")
    OUTPUT.parent.mkdir(parents=True, exist_ok=True)
    temporary = OUTPUT.with_suffix(f".{os.getpid()}.tmp")
    command = [nvcc, *FLAGS, *defines, f"-I{INCLUDE}", *(["-Xptxas", "-v"] if verbose else []), "-o", str(temporary),
               *(str(PACKAGE / "csrc" / s) for s in SOURCES)]
    result = subprocess.run(command, capture_output=True, text=True, check=False)
    if result.returncode != 0:
        temporary.unlink(missing_ok=True)
        raise RuntimeError(f"nvcc failed:\n{result.stdout[-4000:]}\n{result.stderr[-4000:]}")
    if verbose:
        print(result.stderr)
    temporary.replace(OUTPUT)
    stamp.write_text(digest)
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
