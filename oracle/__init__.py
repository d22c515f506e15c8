"""CPU oracle for the sm_100a conv / depthwise path. TEST INFRASTRUCTURE ONLY.

This package restates, on the CPU with plain torch tensor arithmetic, the algorithms of FlashIM's torch reference
ops for the MXFP8 / INT8 implicit-GEMM conv2d and the depthwise 5x5 producers. It is the checker the CUDA kernels are
compared with; nothing in ``flashim_b200`` imports it. Only the test-suite, the smoke entry and the benchmark's
``cpu_baseline`` / ``--impl reference`` legs may use it.

Pinning: every function is checked against the reference's own known-answer vectors and against outputs of the
reference implementation itself, committed as fixtures under ``tests/golden`` (see ``tests/golden/make_golden.py``).
"""

from oracle.flashim_oracle import *  # noqa: F401,F403
