"""tilefish_b200: an sm_100a (B200) backend for tilefish's quantized-inference hot path.

BlockScaled quantization (MXFP8 / MXFP4 / NVFP4 with swizzled scales), the block-scaled ``gemm`` library operator on
tcgen05 tensor cores, the fused ``residual_add_rmsnorm`` and SiLU-gate kernels and the ``mlp`` graph built from them,
behind tilefish's typed API. Hand-written CUDA reached through a C ABI; torch allocates tensors and nothing else.
"""

from .errors import (  # noqa: F401
    TilefishAttributeError,
    TilefishBuildError,
    TilefishDeclarationError,
    TilefishError,
    TilefishLoweringError,
    TilefishManifestError,
    TilefishPlanError,
    TilefishPreconditionError,
    TilefishRuntimeError,
    TilefishSpecError,
    TilefishTypeError,
)

__version__ = "0.1.0"
