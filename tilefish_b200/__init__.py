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

from .decorators import ExternOp, GraphOp, KernelOp, LibraryOp, Op, extern, graph, kernel, library  # noqa: F401,E402
from .dims import Dim, DimExpr, cdiv  # noqa: F401,E402
from .dtypes import BlockScaled, DType, bf16, bool_, e2m1, e4m3, e5m2, f16, f32, i32, i64, u8, ue8m0  # noqa: F401,E402
from .ir import BucketRequirement, Graph, Node, Requirement, Scalar, Value  # noqa: F401,E402
from .trace import contiguous, exp, gelu, max, mean, rsqrt, silu, sqrt, sum  # noqa: F401,E402,A004
from .types import ConstType, InOut, Marked, Out, Tensor, TensorType, const  # noqa: F401,E402

mxfp8 = BlockScaled(elem=e4m3, scale=ue8m0, block=32, axis=-1)
mxfp4 = BlockScaled(elem=e2m1, scale=ue8m0, block=32, axis=-1)
nvfp4 = BlockScaled(elem=e2m1, scale=e4m3, block=16, global_scale=f32)

__version__ = "0.2.0"

# `from tilefish_b200 import *` leaves the reductions out: `sum` and `max` would shadow the builtins (they stay reachable as attributes)
__all__ = [
    "BlockScaled", "BucketRequirement", "ConstType", "DType", "Dim", "DimExpr", "Graph", "GraphOp", "InOut", "KernelOp", "LibraryOp", "Marked", "Node", "Op", "Out",
    "Requirement", "Scalar", "Tensor", "TensorType", "TilefishAttributeError", "TilefishBuildError", "TilefishDeclarationError", "TilefishError",
    "TilefishLoweringError", "TilefishManifestError", "TilefishPlanError", "TilefishPreconditionError", "TilefishRuntimeError", "TilefishSpecError",
    "TilefishTypeError", "Value", "bf16", "bool_", "cdiv", "const", "contiguous", "e2m1", "e4m3", "e5m2", "exp", "extern", "f16", "gelu", "f32", "graph", "i32", "i64", "kernel",
    "library", "mean", "mxfp4", "mxfp8", "nvfp4", "rsqrt", "silu", "sqrt", "u8", "ue8m0",
]


def __getattr__(name):  # the run-time half imports torch lazily
    if name in ("run", "plan", "capture", "runtime", "quantize", "BlockScaledTensor", "bind_weights", "prepare", "run_step"):
        import importlib

        rt = importlib.import_module(".runtime", __name__)
        return rt if name == "runtime" else getattr(rt, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
