"""ctypes binding of the C ABI in include/tilefish_b200.h (the only way Python reaches the CUDA kernels).

There is no fallback: if the shared library is missing or fails to load, every operator raises
``TilefishRuntimeError`` naming the build command. Entry points return a status; a non-zero status becomes an exception
carrying ``tf_last_error()``, the way the reference's C ABI reports errors (crates/tilefish-capi/src/error.rs:86-102).
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int32, c_int64, c_void_p

from .errors import TilefishPreconditionError, TilefishRuntimeError

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "libtilefish_b200.so")

TF_OK = 0
TF_ERR_INVALID_ARGUMENT = 1
TF_ERR_ALIGNMENT = 2
TF_ERR_UNSUPPORTED = 3
TF_ERR_CUDA = 4
TF_ERR_WORKSPACE = 5
TF_ERR_DEVICE_TIMEOUT = 6

FMT_MXFP8, FMT_MXFP4, FMT_NVFP4 = 0, 1, 2
SCALES_PLAIN, SCALES_SWIZZLED = 0, 1
EPI_NONE, EPI_SILU_GATE, EPI_RESIDUAL = 0, 1, 2

_P = c_void_p
_FP = ctypes.POINTER(c_float)

# name -> (restype, argtypes); every symbol include/tilefish_b200.h declares
SIGNATURES = {
    "tf_version": (c_char_p, []),
    "tf_last_error": (c_char_p, []),
    "tf_device_status": (c_int32, [ctypes.POINTER(c_int32), ctypes.POINTER(c_int32)]),
    "tf_selftest_bounded_wait": (c_int32, [c_int32, _P]),
    "tf_set_sm_margin": (c_int32, [c_int32]),
    "tf_scale_bytes": (c_int64, [c_int32, c_int64, c_int64, c_int32]),
    "tf_quantize_mxfp8": (c_int32, [_P, c_int64, c_int64, c_int64, _P, _P, c_int32, _P]),
    "tf_quantize_mxfp4": (c_int32, [_P, c_int64, c_int64, c_int64, _P, _P, c_int32, _P]),
    "tf_quantize_nvfp4": (c_int32, [_P, c_int64, c_int64, c_int64, _P, _P, c_int32, _P, _P]),
    "tf_quantize_nvfp4_from_amax": (c_int32, [_P, c_int64, c_int64, c_int64, _P, _P, c_int32, _P, _P, _P]),
    "tf_nvfp4_global_scale": (c_int32, [_P, c_int64, c_int64, c_int64, _P, _P]),
    "tf_swizzle_scales": (c_int32, [_P, c_int64, c_int64, _P, _P]),
    "tf_unswizzle_scales": (c_int32, [_P, c_int64, c_int64, _P, _P]),
    "tf_residual_add_rmsnorm": (c_int32, [_P, _P, _P, _P, c_int64, c_int64, c_float, c_int32, _P, _P, c_int32, _P, _P, _P]),
    "tf_silu_gate": (c_int32, [_P, _P, c_int64, c_int64, c_int64, c_int64, _P, c_int64, _P]),
    "tf_gemm_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int32, c_int32]),
    "tf_gemm_splits": (c_int32, [c_int64, c_int64, c_int64, c_int32, c_int32]),
    "tf_gemm_blockscaled_partials": (c_int32, [_P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int32, _P, c_int64, _P, _P]),
    "tf_rmsnorm_quantize_rows": (c_int32, [_P, _P, c_int32, _P, _P, c_int64, _P, _P, _P, c_int64, c_int64, c_float, c_int32, _P, _P, _P, _P, _P]),
    "tf_gemm_blockscaled": (c_int32, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int32, c_int32, _P, _P, _P, _P, c_int64, _P, c_int64, _P]),
    "tf_gemm_static_scratch_bytes": (c_int64, []),
    "tf_gemm_blockscaled_static": (c_int32, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int32, c_int32, _P, _P, _P]),
    "tf_gemm_blockscaled_scatter": (c_int32, [_P, _P, _P, _P, _P, _P, _P, c_int32, c_int64, c_int64, c_int64, c_int64, c_int64, c_int32, c_int64, _P]),
    "tf_set_programmatic_launch": (c_int32, [c_int32]),
    "tf_tp_norm_exchange": (c_int32, [_P, _P, ctypes.c_uint64, c_int32, c_int32, c_int32, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int32, _P, _P,
                                      _P, _P, c_float, c_int32, c_int32, _P]),
    "tf_allreduce_bf16": (c_int32, [_P, _P, ctypes.c_uint64, c_int32, c_int32, c_int32, c_int64, c_int64, c_int32, _P]),
    "tf_plan_load": (c_int32, [c_char_p, c_char_p, ctypes.POINTER(_P)]),
    "tf_plan_free": (None, [_P]),
    "tf_plan_digest": (c_char_p, [_P]),
    "tf_plan_arena_bytes": (c_int64, [_P]),
    "tf_plan_step_count": (c_int32, [_P, c_int32]),
    "tf_plan_find_bucket": (c_int32, [_P, ctypes.POINTER(c_char_p), ctypes.POINTER(c_int64), c_int32]),
    "tf_plan_instantiate": (c_int32, [_P, _P, c_int64]),
    "tf_plan_bind": (c_int32, [_P, c_char_p, _P]),
    "tf_plan_launch": (c_int32, [_P, c_int32, _P]),
    "tf_plan_capture": (c_int32, [_P, c_int32, _P, ctypes.POINTER(c_int32)]),
    "tf_plan_replay": (c_int32, [_P, c_int32, _P]),
}

_lib = None


def load():
    """The loaded library (cached). Raises if it is not built: there is no other implementation to fall back to."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise TilefishRuntimeError(
            f"the sm_100a kernel library is missing ({LIB_PATH}); build it with `python tilefish_b200/csrc/build.py` "
            "(needs nvcc). There is no CPU or Triton fallback."
        )
    try:
        lib = ctypes.CDLL(LIB_PATH)
    except OSError as e:
        raise TilefishRuntimeError(f"cannot load {LIB_PATH}: {e}") from e
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise TilefishRuntimeError(f"{LIB_PATH} does not export {name}: rebuild it") from e
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    msg = load().tf_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(status: int, call: str) -> None:
    if status == TF_OK:
        return
    msg = last_error() or f"status {status}"
    if status in (TF_ERR_INVALID_ARGUMENT, TF_ERR_ALIGNMENT, TF_ERR_UNSUPPORTED, TF_ERR_WORKSPACE):
        kind = {TF_ERR_INVALID_ARGUMENT: "argument", TF_ERR_ALIGNMENT: "alignment", TF_ERR_UNSUPPORTED: "unsupported",
                TF_ERR_WORKSPACE: "workspace"}[status]
        raise TilefishPreconditionError(f"{call}: {msg}", kind=kind, arg=None)
    raise TilefishRuntimeError(f"{call}: {msg}")


def version() -> str:
    return load().tf_version().decode()


def device_status():
    """(status, detail) of the device-side status word; synchronizes the device and clears the word."""
    st, detail = c_int32(0), c_int32(0)
    check(load().tf_device_status(ctypes.byref(st), ctypes.byref(detail)), "tf_device_status")
    return st.value, detail.value


def scale_bytes(fmt: int, rows: int, k: int, layout: int) -> int:
    n = load().tf_scale_bytes(fmt, rows, k, layout)
    if n < 0:
        raise TilefishPreconditionError(f"tf_scale_bytes: bad arguments fmt={fmt} rows={rows} k={k} layout={layout}", kind="argument", arg=None)
    return n
