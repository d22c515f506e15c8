"""flashim_b200: hand-written sm_100a (B200) kernels for FlashIM's quantized convolution path — block-scaled MXFP8 and
INT8 implicit-GEMM ``conv2d`` on tcgen05 tensor cores, and the fused depthwise 5x5 producers — behind an op registry
with FlashIM's interface (``ops.<op>(...)``, ``op.get("sm100")``, ``op.explain``) and a ``load(name, preset)`` builder.

The compute path is CUDA only: without ``libflashim_sm100.so`` or without a compute-capability-10.0 device, ops raise.
"""

from flashim_b200 import ops, platforms, quant  # noqa: F401
from flashim_b200.backends.sm100.kernels import check_status  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name: str):
    # the builder imports torch.nn modules; keep `import flashim_b200` light
    if name in ("load", "resolve", "register_spec", "ModelSpec", "RunConfig", "build_config"):
        from flashim_b200 import build

        return getattr(build, name)
    raise AttributeError(name)
