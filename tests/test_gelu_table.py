"""The GELU table the conv epilogue looks up: the committed file is what the generator produces from torch's erf-form
GELU, and the kernel's integer arithmetic on it (restated by the generator) returns torch's result for every bf16 input."""

import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_committed_table_is_current_and_exact():
    script = ROOT / "flashim_b200" / "csrc" / "make_gelu_table.py"
    done = subprocess.run([sys.executable, str(script), "--check"], capture_output=True, text=True)
    assert done.returncode == 0, done.stdout + done.stderr
