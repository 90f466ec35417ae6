"""The native replay loop behind ``tf_plan_*`` (csrc/plan_replay.cu), as a Python object.

``runtime.export`` writes a directory; ``NativePlan(directory, pin=...)`` hands it to the C++ loop, which verifies the digests itself,
owns the arena and runs or captures a bucket's steps with no interpreter between the launches: the role of the reference's Rust host
(crates/tilefish/src/plan_run.rs:678 ``PlanRun``, :1944 ``launch``, :2097 ``capture``) for this path. Python only binds the tensors'
addresses; it keeps the tensors alive for as long as they are bound.
"""

from __future__ import annotations

import ctypes
from typing import Any, Dict, Optional

from . import _native as N
from . import _plan as P
from .errors import TilefishPreconditionError, TilefishRuntimeError


class NativePlan:
    def __init__(self, directory: str, pin: Optional[str] = None, trust_directory: bool = False) -> None:
        P.check_anchor(pin, trust_directory)
        self._lib = N.load()
        handle = ctypes.c_void_p()
        N.check(self._lib.tf_plan_load(directory.encode(), pin.encode() if pin else None, ctypes.byref(handle)), "tf_plan_load")
        self._h = handle
        self._keep: Dict[str, Any] = {}
        self._instantiated = False

    @property
    def digest(self) -> str:
        return self._lib.tf_plan_digest(self._h).decode()

    @property
    def arena_bytes(self) -> int:
        return int(self._lib.tf_plan_arena_bytes(self._h))

    def step_count(self, bucket: int) -> int:
        return int(self._lib.tf_plan_step_count(self._h, bucket))

    def find_bucket(self, **values: int) -> int:
        names = (ctypes.c_char_p * len(values))(*[k.encode() for k in values])
        vals = (ctypes.c_int64 * len(values))(*[int(v) for v in values.values()])
        b = int(self._lib.tf_plan_find_bucket(self._h, names, vals, len(values)))
        if b < 0:
            raise TilefishPreconditionError(f"the plan has no bucket {values} (bucket semantics are exact: the host pads)", kind="bucket")
        return b

    def instantiate(self) -> None:
        """Allocates the arena (the only allocation of this object; call it before any stream capture)."""
        if not self._instantiated:
            N.check(self._lib.tf_plan_instantiate(self._h, None, 0), "tf_plan_instantiate")
            self._instantiated = True

    def bind(self, **tensors: Any) -> None:
        """Binds the caller's tensors to the plan's external buffers by name; a BlockScaledTensor binds its two or three parts."""
        from .kernels import BlockScaledTensor

        for name, t in tensors.items():
            if isinstance(t, BlockScaledTensor):
                parts = P.part_names(name, t.fmt)
                self._bind_one(parts["codes"], t.codes)
                self._bind_one(parts["scales"], t.scales)
                if "global" in parts:
                    self._bind_one(parts["global"], t.global_scale)
            else:
                self._bind_one(name, t)

    def _bind_one(self, name: str, t: Any) -> None:
        N.check(self._lib.tf_plan_bind(self._h, name.encode(), ctypes.c_void_p(t.data_ptr())), "tf_plan_bind")
        self._keep[name] = t

    @staticmethod
    def _stream(stream) -> int:
        import torch

        return torch.cuda.current_stream().cuda_stream if stream is None else getattr(stream, "cuda_stream", stream)

    def launch(self, bucket: int, stream=None) -> None:
        self.instantiate()
        N.check(self._lib.tf_plan_launch(self._h, bucket, ctypes.c_void_p(self._stream(stream))), "tf_plan_launch")

    def capture(self, bucket: int, stream=None) -> int:
        """Captures the bucket's steps into a CUDA graph the plan owns; returns its index for ``replay``. Needs a non-default stream."""
        import torch

        self.instantiate()
        if stream is None:
            stream = torch.cuda.Stream()
        g = ctypes.c_int32(-1)
        stream.wait_stream(torch.cuda.current_stream())
        N.check(self._lib.tf_plan_capture(self._h, bucket, ctypes.c_void_p(stream.cuda_stream), ctypes.byref(g)), "tf_plan_capture")
        return g.value

    def replay(self, graph: int, stream=None) -> None:
        N.check(self._lib.tf_plan_replay(self._h, graph, ctypes.c_void_p(self._stream(stream))), "tf_plan_replay")

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h:
            self._lib.tf_plan_free(self._h)
            self._h = None
            self._keep.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass
