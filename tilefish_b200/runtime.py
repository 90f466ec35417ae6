"""Running declarations: ``run`` (modes "jit" and "replay"), ``export``, ``plan``, ``capture``, ``bind_weights``, ``prepare``, ``run_step``.

Signatures and semantics follow the reference's run-time API (python/src/tilefish/runtime.py:1078-1147 ``export``, :1407-1449
``run``, :1343-1374 ``bind_weights`` / ``prepare`` / ``run_step``; docs/en/plan-schema-1.md:468-490): arguments are torch tensors
(a ``Tensor[..., BlockScaled]`` parameter takes a ``BlockScaledTensor``), ``InOut`` tensors are updated in place, results are
freshly allocated unless ``outputs=`` gives them, every precondition of every step is checked before the first launch, a replay
needs a trust anchor (``pin=`` or ``trust_directory=True``) and verifies the exported directory against it, ``taps=`` copies
buffers of the plan into the caller's tensors right after a step. Differences that the backend forces:

* ``mode="jit"`` launches the prebuilt sm_100a kernels directly: there is nothing to compile at run time;
* ``mode="reference"`` is refused: the torch interpreter of the reference is an oracle, not a product path, and this
  package has no CPU implementation of any operator.

The steps run through a ``Backend`` object with the reference's method names and signatures
(python/src/tilefish/_planrun.py:240-376): ``stream(index)``, ``alloc_arena(nbytes, index) -> (handle, address)``,
``load(built, index)``, ``launch(loaded, grid, args, stream, scratch=None)``, ``gemm(spec, algo, a, b, bias, out, workspace,
stream, index)``, ``copy``, ``memset``, ``capture_graph`` / ``replay_graph``: raw integer device addresses
(``address(buffer) + view.offset * itemsize``, docs/en/plan-schema-1.md:196) and scalars the host derives from the shapes.
``Sm100Backend`` passes them to the C ABI; a test substitutes a recording backend and needs no GPU.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

from . import _plan as P
from . import backend as B
from .decorators import GraphOp, KernelOp, LibraryOp, Op
from .dims import Dim, as_expr, evaluate
from .dtypes import TORCH_NAMES, BlockScaled
from .errors import TilefishManifestError, TilefishPreconditionError, TilefishRuntimeError
from .kernels import BlockScaledTensor, quantize  # noqa: F401  (re-exported: the run-time value of a BlockScaled tensor)
from ._plan import Plan, load_export, make_plan

MODES = ("jit", "replay", "reference")
FORMAT_IDS = {"mxfp8": 0, "mxfp4": 1, "nvfp4": 2}
EPILOGUE_IDS = {"none": 0, "silu_gate": 1, "residual": 2}
SCALES_SWIZZLED = 1


# ---- what a step launches ---------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class BuiltEntry:
    """A manifest entry as the runner hands it to ``Backend.load``: the C symbol, its pointer parameters and attributes."""

    stem: str
    kind: str
    symbol: str
    params: Tuple[str, ...]
    attrs: Tuple[Tuple[str, Any], ...]

    def attr(self, name: str, default: Any = None) -> Any:
        return dict(self.attrs).get(name, default)


@dataclass(frozen=True)
class GemmSpec:
    """The problem of one library step: what the reference's ``LibrarySpec`` is to its pinned GEMM (python/src/tilefish/_library.py:105-108)."""

    stem: str
    m: int
    n: int
    k: int
    format: str
    epilogue: str
    ldo: int
    workspace_bytes: int  # bytes the plan reserved
    a_global_scale_rows: int = 0


@dataclass(frozen=True)
class ScaledOperands:
    """Addresses a block-scaled GEMM takes beside the reference's (a, b, out): scale bytes, global scales and the fused outputs."""

    a_scales: int
    b_scales: int
    a_global: Optional[int] = None
    b_global: Optional[int] = None
    amax: Optional[int] = None
    q_codes: Optional[int] = None
    q_scales: Optional[int] = None


class Backend:
    """What a runner needs from torch and the kernel library; method names and signatures are the reference's
    (python/src/tilefish/_planrun.py:240-376), restricted to what this path uses."""

    def device_index(self, device: Any) -> int:
        raise NotImplementedError

    def current_device(self) -> int:
        raise NotImplementedError

    def capturing(self, index: int) -> bool:
        raise NotImplementedError

    def stream(self, index: int) -> int:
        raise NotImplementedError

    def alloc_arena(self, nbytes: int, index: int) -> Tuple[Any, int]:
        """``(handle, address)`` of ``nbytes`` bytes of device memory, 256-byte aligned."""
        raise NotImplementedError

    def empty(self, shape: Sequence[int], dtype: str, index: int) -> Any:
        raise NotImplementedError

    def load(self, built: BuiltEntry, index: int) -> Any:
        raise NotImplementedError

    def launch(self, loaded: Any, grid: Sequence[int], args: Sequence[Tuple[str, Any]], stream: int, scratch: Optional[int] = None) -> None:
        """Launch a kernel entry. ``args``: (type tag, value) pairs in the order of the entry point's parameters, the stream excluded
        (tags "ptr", "i32", "i64", "f32"); ``grid`` is empty: the entry points size their own grids."""
        raise NotImplementedError

    def copy(self, dst: int, src: int, nbytes: int, stream: int) -> None:
        raise NotImplementedError

    def memset(self, dst: int, nbytes: int, stream: int) -> None:
        raise NotImplementedError

    def gemm(self, spec: GemmSpec, algo: str, a: int, b: int, bias: Optional[int], out: Optional[int], workspace: int, stream: int, index: int,
             c: Optional[int] = None, *, scaled: Optional[ScaledOperands] = None) -> None:
        """Run a library step on device addresses, the workspace in the arena. ``a`` / ``b`` / ``out`` are the addresses of the element
        codes and of the bf16 result, ``c`` the f32 tensor the residual epilogue accumulates into, ``scaled`` the rest."""
        raise NotImplementedError

    def check_gemm(self, spec: GemmSpec, algo: str, index: int) -> None:
        """Refuse a step whose problem needs more workspace on this device than the plan reserved (once per bucket)."""

    def capture_graph(self, index: int, stream: Any, enqueue: Any) -> Any:
        raise NotImplementedError

    def replay_graph(self, graph: Any, stream: int) -> None:
        raise NotImplementedError

    def synchronize_stream(self, stream: int) -> None:
        raise NotImplementedError


_CTYPES = {"ptr": ctypes.c_void_p, "i32": ctypes.c_int32, "i64": ctypes.c_int64, "f32": ctypes.c_float}


class Sm100Backend(Backend):
    """torch for memory and streams, the C ABI (include/tilefish_b200.h) for every launch."""

    def __init__(self) -> None:
        import torch

        self.torch = torch

    def device_index(self, device: Any) -> int:
        if isinstance(device, int) and not isinstance(device, bool):
            return device
        d = self.torch.device(device)
        return d.index if d.index is not None else self.current_device()

    def current_device(self) -> int:
        return int(self.torch.cuda.current_device())

    def capturing(self, index: int) -> bool:
        with self.torch.cuda.device(index):
            return bool(self.torch.cuda.is_current_stream_capturing())

    def stream(self, index: int) -> int:
        return int(self.torch.cuda.current_stream(index).cuda_stream)

    def alloc_arena(self, nbytes: int, index: int) -> Tuple[Any, int]:
        t = self.torch.empty(max(nbytes, 1), dtype=self.torch.uint8, device=f"cuda:{index}")
        return t, int(t.data_ptr())

    def empty(self, shape: Sequence[int], dtype: str, index: int) -> Any:
        return self.torch.empty(tuple(shape), dtype=getattr(self.torch, TORCH_NAMES[dtype]), device=f"cuda:{index}")

    def load(self, built: BuiltEntry, index: int) -> Any:
        from . import _native as N

        lib = N.load()
        if built.symbol not in N.SIGNATURES:
            raise TilefishManifestError(f"entry '{built.stem}': the kernel library has no entry point {built.symbol}")
        return (built, lib)

    def launch(self, loaded: Any, grid: Sequence[int], args: Sequence[Tuple[str, Any]], stream: int, scratch: Optional[int] = None) -> None:
        from . import _native as N

        built, lib = loaded
        symbol = built.symbol if isinstance(built, BuiltEntry) else built
        values = [_CTYPES[tag](v) if v is not None else None for tag, v in args]
        N.check(getattr(lib, symbol)(*values, ctypes.c_void_p(stream)), symbol)

    def copy(self, dst: int, src: int, nbytes: int, stream: int) -> None:
        _cudart_check(_cudart().cudaMemcpyAsync(ctypes.c_void_p(dst), ctypes.c_void_p(src), ctypes.c_size_t(nbytes), 3, ctypes.c_void_p(stream)), "cudaMemcpyAsync")

    def memset(self, dst: int, nbytes: int, stream: int) -> None:
        _cudart_check(_cudart().cudaMemsetAsync(ctypes.c_void_p(dst), 0, ctypes.c_size_t(nbytes), ctypes.c_void_p(stream)), "cudaMemsetAsync")

    def gemm(self, spec: GemmSpec, algo: str, a: int, b: int, bias: Optional[int], out: Optional[int], workspace: int, stream: int, index: int,
             c: Optional[int] = None, *, scaled: Optional[ScaledOperands] = None) -> None:
        from . import _native as N

        if bias is not None:
            raise TilefishRuntimeError(f"step '{spec.stem}': the block-scaled GEMM has no bias operand")
        if scaled is None:
            raise TilefishRuntimeError(f"step '{spec.stem}': a block-scaled GEMM needs its scale addresses")
        P_ = ctypes.c_void_p
        N.check(N.load().tf_gemm_blockscaled(P_(a), P_(scaled.a_scales), P_(scaled.a_global), P_(b), P_(scaled.b_scales), P_(scaled.b_global), P_(out),
                                             spec.ldo, spec.m, spec.n, spec.k, FORMAT_IDS[spec.format], EPILOGUE_IDS[spec.epilogue], P_(c), P_(scaled.amax),
                                             P_(scaled.q_codes), P_(scaled.q_scales), spec.a_global_scale_rows, P_(workspace), spec.workspace_bytes, P_(stream)),
                "tf_gemm_blockscaled")

    def check_gemm(self, spec: GemmSpec, algo: str, index: int) -> None:
        from . import _native as N

        need = int(N.load().tf_gemm_workspace_bytes(spec.m, spec.n, spec.k, FORMAT_IDS[spec.format], EPILOGUE_IDS[spec.epilogue]))
        if need > spec.workspace_bytes:
            raise TilefishPreconditionError(f"step '{spec.stem}': on this device the GEMM needs {need} bytes of workspace, the plan reserved {spec.workspace_bytes} "
                                            f"(it was sized for {P.PLANNED_SM_COUNT} SMs); plan it again for this device", kind="workspace", arg="workspace")

    def capture_graph(self, index: int, stream: Any, enqueue: Any) -> Any:
        g = self.torch.cuda.CUDAGraph()
        with self.torch.cuda.graph(g, stream=stream):
            enqueue(self.stream(index))
        return g

    def replay_graph(self, graph: Any, stream: int) -> None:
        graph.replay()

    def synchronize_stream(self, stream: int) -> None:
        self.torch.cuda.synchronize()


_CUDART = None


def _cudart():
    """libcudart as torch loaded it: the plan's copy and memset steps are plain cudaMemcpyAsync / cudaMemsetAsync on the plan's stream."""
    global _CUDART
    if _CUDART is None:
        import glob

        import torch

        candidates = glob.glob(os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "cuda_runtime", "lib", "libcudart.so*")) + ["libcudart.so.12", "libcudart.so"]
        for c in candidates:
            try:
                _CUDART = ctypes.CDLL(c)
                break
            except OSError:
                continue
        if _CUDART is None:
            raise TilefishRuntimeError("cannot load libcudart for the plan's copy / memset steps")
    return _CUDART


def _cudart_check(code: int, call: str) -> None:
    if code != 0:
        raise TilefishRuntimeError(f"{call} failed with CUDA error {code}")


_DEFAULT_BACKEND: Optional[Backend] = None


def default_backend() -> Backend:
    global _DEFAULT_BACKEND
    if _DEFAULT_BACKEND is None:
        _DEFAULT_BACKEND = Sm100Backend()
    return _DEFAULT_BACKEND


# ---- binding arguments to a signature ------------------------------------------------------------------------------------
def _bind_dims(op: Op, tensors: Dict[str, Any]) -> Dict[Dim, int]:
    """Checks dtype, rank, format, device and contiguity of every argument and unifies the dimensions with the shapes."""
    import torch

    env: Dict[Dim, int] = {}
    device = None
    for p in op.signature.tensors:
        if p.name not in tensors:
            if p.access == "out":
                continue
            raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' is missing", kind="shape", arg=p.name)
        t = tensors[p.name]
        if isinstance(p.type.dtype, BlockScaled):
            if not isinstance(t, BlockScaledTensor):
                raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' must be a BlockScaledTensor ({p.type.dtype})", kind="dtype", arg=p.name)
            if t.fmt != p.type.dtype.format_name:
                raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' is {t.fmt}, the signature says {p.type.dtype}", kind="dtype", arg=p.name)
            if t.layout != "swizzled":
                raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' must carry swizzled scales", kind="contiguous", arg=p.name)
            shape, dev = t.shape, t.device
        else:
            if not isinstance(t, torch.Tensor):
                raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' must be a torch tensor", kind="dtype", arg=p.name)
            want = getattr(torch, TORCH_NAMES[p.type.dtype.name])
            if t.dtype != want:
                raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' is {t.dtype}, expected {want}", kind="dtype", arg=p.name)
            if p.type.contiguous and not t.is_contiguous():
                raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' is not contiguous", kind="contiguous", arg=p.name)
            if t.numel() and t.data_ptr() % 16:
                raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' is not 16-byte aligned", kind="pointer_alignment", arg=p.name)
            shape, dev = tuple(t.shape), t.device
        if not dev.type == "cuda":
            raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' is on {dev}; this backend runs on CUDA only", kind="device", arg=p.name)
        if device is None:
            device = dev
        elif dev != device:
            raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' is on {dev}, earlier arguments on {device}", kind="device", arg=p.name)
        if len(shape) != p.type.rank:
            raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' has rank {len(shape)}, expected {p.type.rank}", kind="rank", arg=p.name)
        for formal, actual in zip(p.type.shape, shape):
            e = as_expr(formal)
            if e.is_static:
                if e.offset != actual:
                    raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' has size {actual} where {formal} = {e.offset} is compiled in",
                                                    kind="static_size", arg=p.name)
                continue
            if len(e.terms) == 1 and e.offset == 0 and isinstance(e.terms[0][0], Dim):
                d, coef = e.terms[0]
                if actual % coef:
                    raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' has size {actual}, not a multiple of {coef}", kind="shape", arg=p.name)
                v = actual // coef
                if d in env and env[d] != v:
                    raise TilefishPreconditionError(f"{op.name}: dimension {d.name} is {env[d]} for an earlier argument but {v} for '{p.name}'",
                                                    kind="shape", arg=p.name)
                if d.divisible_by and v % d.divisible_by:
                    raise TilefishPreconditionError(f"{op.name}: {d.name} = {v} is not divisible by {d.divisible_by}", kind="divisible", arg=p.name)
                env[d] = v
            else:
                raise TilefishPreconditionError(f"{op.name}: size expression {formal} of '{p.name}' cannot be bound from a shape", kind="shape", arg=p.name)
    # what the calls inside the graph rely on beyond the declarations (recorded while the graph was traced)
    for req in getattr(getattr(op, "graph", None), "requirements", ()):
        v = evaluate(req.dim, env)
        if v is None:
            continue
        if hasattr(req, "buckets"):
            if v not in req.buckets:
                raise TilefishPreconditionError(f"{op.name}: {req.dim} = {v} is not one of {list(req.buckets)} (required by {req.origin})", kind="bucket", arg=None)
        elif v % req.divisor:
            raise TilefishPreconditionError(f"{op.name}: {req.dim} = {v} is not divisible by {req.divisor} (required by {req.origin})", kind="divisible", arg=None)
    written = [tensors[p.name] for p in op.signature.tensors if p.access != "in" and p.name in tensors]
    for w in written:
        for p in op.signature.tensors:
            o = tensors.get(p.name)
            if o is not None and o is not w and not isinstance(o, BlockScaledTensor) and not isinstance(w, BlockScaledTensor) and o.numel() and w.numel() \
                    and o.data_ptr() == w.data_ptr():
                raise TilefishPreconditionError(f"{op.name}: a written tensor aliases argument '{p.name}'", kind="alias", arg=p.name)
    return env


def _named_args(op: Op, args, kwargs) -> Dict[str, Any]:
    params = op.signature.tensors
    if len(args) > len(params):
        raise TilefishPreconditionError(f"{op.name}: takes {len(params)} tensors, {len(args)} were given", kind="shape")
    named = {p.name: a for p, a in zip(params, args)}
    for k, v in kwargs.items():
        if k in named:
            raise TilefishPreconditionError(f"{op.name}: argument '{k}' given twice", kind="shape", arg=k)
        const = next((c for c in op.signature.consts if c.name == k), None)
        if const is not None:
            if v != const.default:
                raise TilefishPreconditionError(f"{op.name}: const '{k}' is compiled in as {const.default!r}", kind="static_size", arg=k)
            continue
        named[k] = v
    return named


# ---- the runner ----------------------------------------------------------------------------------------------------------
def _row_major(shape: Sequence[int]) -> Tuple[int, ...]:
    strides, acc = [], 1
    for s in reversed(shape):
        strides.append(acc)
        acc *= int(s)
    return tuple(reversed(strides))


class _Bound:
    """One pointer argument of a step at a bucket: the buffer it names, its element shape and strides, and its byte offset."""

    __slots__ = ("name", "binding", "dtype", "shape", "strides", "byte_offset")

    def __init__(self, name: str, binding: str, dtype: str, shape: Tuple[int, ...], strides: Tuple[int, ...], byte_offset: int) -> None:
        self.name, self.binding, self.dtype, self.shape, self.strides, self.byte_offset = name, binding, dtype, shape, strides, byte_offset


class PlanRunner:
    """Executes a plan document: the arena is allocated once per device, every step's preconditions are checked before the first
    launch, then the steps of the selected bucket run in order on the device's current stream."""

    def __init__(self, doc: Dict[str, Any], manifest: Dict[str, Any], backend: Optional[Backend] = None) -> None:
        self.doc = doc
        self.manifest = manifest
        self.backend = backend or default_backend()
        self._arenas: Dict[int, Tuple[Any, int]] = {}
        self._loaded: Dict[Tuple[str, int], Any] = {}
        self._checked: set = set()
        self._buffers = {b["name"]: b for b in doc["buffers"]}
        self._algo = (manifest.get("library_file") or {}).get("sha256") or ""

    # -- buckets and addresses
    def bucket_index(self, values: Dict[str, int]) -> int:
        for i, b in enumerate(self.doc["buckets"]):
            if b["values"] == values:
                return i
        have = {n: v for n, v in self.doc["dims"].items()}
        raise TilefishPreconditionError(f"plan '{self.doc['graph']}': no bucket {values}; the plan has {have} (bucket semantics are exact: the host pads)",
                                        kind="bucket")

    def arena(self, index: int) -> Tuple[Any, int]:
        got = self._arenas.get(index)
        if got is None:
            if self.backend.capturing(index):
                raise TilefishRuntimeError(f"plan '{self.doc['graph']}': its arena would be allocated inside a stream capture; call prepare() or run it once first")
            handle, addr = self.backend.alloc_arena(self.doc["arena_bytes"], index)
            if addr % self.doc["arena_alignment"]:
                raise TilefishRuntimeError("the arena is not aligned to arena_alignment")
            got = self._arenas[index] = (handle, addr)
        return got

    def _entry(self, stem: str, kind: str, index: int):
        key = (stem, index)
        got = self._loaded.get(key)
        if got is None:
            e = self.manifest["library" if kind == "library" else "kernels"][stem]
            built = BuiltEntry(stem, kind, e["symbol"], tuple(e["params"]), tuple(sorted(e["attrs"].items())))
            got = self._loaded[key] = (built, e, self.backend.load(built, index))
        return got

    def _bind_args(self, step: Dict[str, Any], shapes: Dict[str, Tuple[str, Tuple[int, ...]]]) -> Dict[str, _Bound]:
        out: Dict[str, _Bound] = {}
        for a in step["args"]:
            dtype, shape = shapes[a["binding"]]
            v = a.get("view")
            if v is None:
                out[a["name"]] = _Bound(a["name"], a["binding"], dtype, tuple(shape), _row_major(shape), 0)
            else:
                out[a["name"]] = _Bound(a["name"], a["binding"], dtype, tuple(v["shape"]), tuple(v["strides"]), v["offset"] * P.ITEMSIZE[dtype])
        return out

    # -- one step as backend calls
    def _calls(self, step: Dict[str, Any], bound: Dict[str, _Bound], addr: Dict[str, int], index: int) -> List[Tuple[str, Any]]:
        """The backend calls of one step: ("memset", (dst, nbytes)), ("copy", (dst, src, nbytes)), ("launch", (loaded, args)) or
        ("gemm", (spec, a, b, out, workspace, c, scaled))."""
        kind = step["kind"]

        def ptr(name: str) -> Optional[int]:
            b = bound.get(name)
            return None if b is None else addr[b.binding] + b.byte_offset

        def nbytes(name: str) -> int:
            b = bound[name]
            return P._prod(b.shape) * P.ITEMSIZE[b.dtype]

        if kind == "memset":
            return [("memset", (ptr("dst"), nbytes("dst")))]
        if kind == "copy":
            return [("copy", (ptr("dst"), ptr("src"), nbytes("src")))]
        built, entry, loaded = self._entry(step["entry"], kind, index)
        attrs = entry["attrs"]
        sym = entry["symbol"]
        if kind == "library":
            a, bq = bound["a"], bound["b"]
            fmt, epi = attrs["format"], attrs.get("epilogue", "none")
            epb = P.ELEMS_PER_BYTE[fmt]
            m, k = a.shape[0], a.shape[1] * epb
            n_rows = bq.shape[0]
            n = n_rows // 2 if epi == "silu_gate" else n_rows
            out_b = bound.get("out")
            ws = self._buffers[step["workspace"]]
            spec = GemmSpec(step["entry"], m, n, k, fmt, epi, out_b.strides[0] if out_b is not None and len(out_b.shape) == 2 and m > 1 else n, ws["bytes"])
            scaled = ScaledOperands(ptr("a_scales"), ptr("b_scales"), ptr("a_global"), ptr("b_global"), ptr("amax"), ptr("q"), ptr("q_scales"))
            return [("gemm", (spec, ptr("a"), ptr("b"), ptr("out"), addr[step["workspace"]], ptr("residual"), scaled))]
        if sym == "tf_residual_add_rmsnorm":
            x = bound["x"]
            m, d = x.shape
            qf = attrs.get("q_format")
            args = [("ptr", ptr("x")), ("ptr", ptr("residual")), ("ptr", ptr("w")), ("ptr", ptr("out")), ("i64", m), ("i64", d), ("f32", P.f32_from_bits(attrs["eps_bits"])),
                    ("i32", FORMAT_IDS[qf] if qf else -1), ("ptr", ptr("q")), ("ptr", ptr("q_scales")), ("i32", SCALES_SWIZZLED), ("ptr", ptr("q_global")),
                    ("ptr", ptr("amax"))]
            return [("launch", (loaded, args))]
        if sym == "tf_silu_gate":
            g, u, o = bound["gate"], bound["up"], bound["out"]
            m, f = g.shape
            args = [("ptr", ptr("gate")), ("ptr", ptr("up")), ("i64", m), ("i64", f), ("i64", g.strides[0] if m > 1 else f), ("i64", u.strides[0] if m > 1 else f),
                    ("ptr", ptr("out")), ("i64", o.strides[0] if m > 1 else f)]
            return [("launch", (loaded, args))]
        if sym in ("tf_quantize_mxfp8", "tf_quantize_mxfp4"):
            x = bound["x"]
            m, k = x.shape
            args = [("ptr", ptr("x")), ("i64", m), ("i64", k), ("i64", x.strides[0] if m > 1 else k), ("ptr", ptr("q")), ("ptr", ptr("q_scales")), ("i32", SCALES_SWIZZLED)]
            return [("launch", (loaded, args))]
        if sym == "tf_quantize_nvfp4":
            x = bound["x"]
            m, k = x.shape
            ldx = x.strides[0] if m > 1 else k
            head = [("ptr", ptr("x")), ("i64", m), ("i64", k), ("i64", ldx)]
            if "amax" in bound:  # the producer reduced the amax: the quantizer derives the global scale from it
                l2 = self.backend.load(BuiltEntry(built.stem, "kernel", "tf_quantize_nvfp4_from_amax", built.params, built.attrs), index)
                return [("launch", (l2, head + [("ptr", ptr("q")), ("ptr", ptr("q_scales")), ("i32", SCALES_SWIZZLED), ("ptr", ptr("amax")), ("ptr", ptr("q_global"))]))]
            l1 = self.backend.load(BuiltEntry(built.stem, "kernel", "tf_nvfp4_global_scale", built.params, built.attrs), index)
            return [("launch", (l1, head + [("ptr", ptr("q_global"))])),
                    ("launch", (loaded, head + [("ptr", ptr("q")), ("ptr", ptr("q_scales")), ("i32", SCALES_SWIZZLED), ("ptr", ptr("q_global"))]))]
        raise TilefishRuntimeError(f"step '{step['entry']}': unknown kernel entry point {sym}")

    def _check_step(self, step: Dict[str, Any], bound: Dict[str, _Bound], addr: Dict[str, int]) -> None:
        for b in bound.values():
            if b.binding not in addr:
                raise TilefishPreconditionError(f"step '{step.get('entry', step['kind'])}': no tensor was given for buffer '{b.binding}'", kind="shape", arg=b.binding)
            p = addr[b.binding] + b.byte_offset
            align = 4 if b.shape in ((1,), ()) else 16
            if p % align:
                raise TilefishPreconditionError(f"step '{step.get('entry', step['kind'])}': the pointer of '{b.name}' is not {align}-byte aligned", kind="pointer_alignment",
                                                arg=b.name)

    def enqueue(self, bucket: int, addr: Dict[str, int], index: int, stream: int, taps: Optional[Dict[Any, Any]] = None, only_step: Optional[int] = None) -> None:
        """Checks every step of the bucket, then enqueues them (``only_step``: that one step) on ``stream``."""
        bdoc = self.doc["buckets"][bucket]
        shapes = P.buffer_shapes(self.doc, bdoc["values"])
        steps = bdoc["steps"]
        plan_calls: List[List[Tuple[str, Any]]] = []
        for i, st in enumerate(steps):
            if only_step is not None and i != only_step:
                plan_calls.append([])
                continue
            bound = self._bind_args(st, shapes)
            self._check_step(st, bound, addr)
            calls = self._calls(st, bound, addr, index)
            for what, payload in calls:
                if what == "gemm" and (bucket, i, index) not in self._checked:
                    self.backend.check_gemm(payload[0], self._algo, index)
                    self._checked.add((bucket, i, index))
            plan_calls.append(calls)
        tap_after = _tap_steps(taps, steps, shapes) if taps else {}
        # nothing was launched so far: every refusal above leaves the device untouched
        for i, calls in enumerate(plan_calls):
            for what, payload in calls:
                if what == "memset":
                    self.backend.memset(payload[0], payload[1], stream)
                elif what == "copy":
                    self.backend.copy(payload[0], payload[1], payload[2], stream)
                elif what == "launch":
                    self.backend.launch(payload[0], (), payload[1], stream)
                else:
                    spec, a, b, out, ws, c, scaled = payload
                    self.backend.gemm(spec, self._algo, a, b, None, out, ws, stream, index, c=c, scaled=scaled)
            for (name, dst) in tap_after.get(i, []):
                dtype, shape = shapes[name]
                self.backend.copy(int(dst.data_ptr()), addr[name], P._prod(shape) * P.ITEMSIZE[dtype], stream)

    # -- a whole call
    def addresses(self, tensors: Dict[str, Any], index: int) -> Dict[str, int]:
        """Device address of every buffer: the caller's tensors (a BlockScaledTensor gives two or three), the arena's regions."""
        _, base = self.arena(index)
        addr: Dict[str, int] = {}
        for b in self.doc["buffers"]:
            if b["offset"] is not None:
                addr[b["name"]] = base + b["offset"]
        for name, t in tensors.items():
            if isinstance(t, BlockScaledTensor):
                parts = P.part_names(name, t.fmt)
                addr[parts["codes"]] = int(t.codes.data_ptr())
                addr[parts["scales"]] = int(t.scales.data_ptr())
                if "global" in parts:
                    addr[parts["global"]] = int(t.global_scale.data_ptr())
            elif t is not None:
                addr[name] = int(t.data_ptr())
        return addr

    def run(self, values: Dict[str, int], tensors: Dict[str, Any], device, outputs: Any = None, taps: Optional[Dict[Any, Any]] = None):
        index = self.backend.device_index(device)
        bucket = self.bucket_index(values)
        shapes = P.buffer_shapes(self.doc, self.doc["buckets"][bucket]["values"])
        results = []
        if outputs is not None and not isinstance(outputs, (dict, list, tuple)):
            outputs = [outputs]  # one tensor for the one returned value
        given = outputs if isinstance(outputs, dict) else dict(zip(self.doc["outputs"], outputs)) if outputs is not None else {}
        bound = dict(tensors)
        for name in self.doc["outputs"]:
            dtype, shape = shapes[name]
            t = given.get(name)
            if t is None:
                t = self.backend.empty(shape, dtype, index)
            elif tuple(t.shape) != tuple(shape) or not t.is_contiguous() or str(t.dtype) != f"torch.{TORCH_NAMES[dtype]}":
                raise TilefishPreconditionError(f"output '{name}': expected a contiguous {dtype} tensor of shape {tuple(shape)}", kind="shape", arg=name)
            bound[name] = t
            results.append(t)
        addr = self.addresses(bound, index)
        self.enqueue(bucket, addr, index, self.backend.stream(index), taps=taps)
        if not results:
            return None
        return results[0] if len(results) == 1 else tuple(results)


def _tap_steps(taps: Dict[Any, Any], steps: List[Dict[str, Any]], shapes) -> Dict[int, List[Tuple[str, Any]]]:
    """{step index: [(buffer, destination tensor)]}: a tap is ``name`` (after the last step that writes the buffer) or ``(name, step)``."""
    out: Dict[int, List[Tuple[str, Any]]] = {}
    for key, dst in taps.items():
        name, at = (key, None) if isinstance(key, str) else key
        if name not in shapes:
            raise TilefishRuntimeError(f"taps: the plan has no buffer {name!r}")
        if at is None:
            writers = [i for i, st in enumerate(steps) for a in st["args"] if a["binding"] == name and (a["name"] in P.WRITTEN or a["name"] == "dst")]
            if not writers:
                raise TilefishRuntimeError(f"taps: no step writes buffer {name!r}")
            at = writers[-1]
        if not 0 <= int(at) < len(steps):
            raise TilefishRuntimeError(f"taps: the plan has {len(steps)} steps, not a step {at}")
        dtype, shape = shapes[name]
        if dst.numel() * dst.element_size() != P._prod(shape) * P.ITEMSIZE[dtype] or not dst.is_contiguous():
            raise TilefishPreconditionError(f"taps: the tensor for {name!r} must be contiguous and hold {dtype} {list(shape)}", kind="shape", arg=name)
        out.setdefault(int(at), []).append((name, dst))
    return out


def _library_identity() -> Dict[str, Any]:
    from . import _native

    with open(_native.LIB_PATH, "rb") as f:
        sha = hashlib.sha256(f.read()).hexdigest()
    return {"file": os.path.basename(_native.LIB_PATH), "sha256": sha, "version": _native.version()}


def plan(graph: GraphOp, buckets: Optional[Dict[str, Sequence[int]]] = None) -> Plan:
    """The launch plan of a graph (needs no GPU): ``.doc`` is the plan.json document, ``.digest`` its pin."""
    return make_plan(graph, buckets, exported=False)


class Export:
    def __init__(self, directory: str, plan_: Plan) -> None:
        self.directory, self.plan, self.manifest = directory, plan_, plan_.manifest

    @property
    def digest(self) -> str:
        return self.plan.digest

    @property
    def manifest_digest(self) -> str:
        return self.manifest["manifest_digest"]


def export(graph: GraphOp, directory: str, *, arch: str = "sm_100a", overwrite: bool = False, buckets: Optional[Dict[str, Sequence[int]]] = None) -> Export:
    """Writes ``manifest.json`` and ``plan.json`` for ``graph`` into ``directory`` and returns their digests. The manifest
    records the kernel library this process would run (file, sha256, version); a replay refuses another build."""
    if arch not in ("sm_100a", "sm_100"):
        raise TilefishRuntimeError(f"export: this backend builds for sm_100a only, not {arch}")
    pl = make_plan(graph, buckets, library=_library_identity())
    P.write_export(directory, pl, overwrite=overwrite)
    return Export(directory, pl)


_RUNNERS: Dict[Any, PlanRunner] = {}


def clear_caches() -> None:
    """Drops the runners (and with them the arenas) this module keeps; CUDA graphs captured from them must be dropped first."""
    _RUNNERS.clear()


def _jit_runner(graph: GraphOp, values: Dict[str, int], plan_: Optional[Plan] = None) -> PlanRunner:
    key = ("jit", id(graph), tuple(sorted(values.items())), id(plan_))
    r = _RUNNERS.get(key)
    if r is None:
        pl = plan_ if plan_ is not None else make_plan(graph, {n: [v] for n, v in values.items()}, exported=False)
        r = _RUNNERS[key] = PlanRunner(pl.doc, pl.manifest)
    return r


def _replay_runner(graph: GraphOp, directory: str, pin: Optional[str], trust_directory: bool) -> PlanRunner:
    P.check_anchor(pin, trust_directory)
    key = ("replay", os.path.abspath(directory), pin)
    r = _RUNNERS.get(key)
    if r is None:
        doc, manifest = load_export(directory, pin, trust_directory)
        lib = manifest["library_file"]
        mine = _library_identity()
        if lib.get("sha256") and lib["sha256"] != mine["sha256"]:
            raise TilefishManifestError(f"{directory}: exported against kernel library {lib['sha256'][:12]} ({lib.get('version')}), this process loads "
                                        f"{mine['sha256'][:12]} ({mine['version']}); re-export")
        if doc["graph"] != graph.name:
            raise TilefishRuntimeError(f"run: {directory} holds the plan of graph '{doc['graph']}', not '{graph.name}'")
        # a host that has the graph requires the document to be the plan it derives itself: a graph that changed since the export is stale
        fresh = make_plan(graph, doc["dims"], library=lib)
        if P.plan_digest(fresh.doc) != doc["plan_digest"]:
            raise TilefishManifestError(f"{directory}: the plan is stale: graph '{graph.name}' (or this package's planner) changed since the export; export again")
        r = _RUNNERS[key] = PlanRunner(doc, manifest)
    return r


def _check_run_options(mode: str, manifest: Any, pin: Optional[str], trust_directory: bool, is_graph: bool) -> None:
    if mode not in MODES:
        raise TilefishRuntimeError(f"unknown mode {mode!r}: use one of {', '.join(MODES)}")
    if mode == "reference":
        raise TilefishRuntimeError("run: mode='reference' is not part of this backend: it has no CPU implementation of any operator. The torch "
                                   "restatement used to check it lives outside the package, as test infrastructure")
    if trust_directory is not True and trust_directory is not False:
        raise TilefishRuntimeError(f"trust_directory= is True or False, got {trust_directory!r}")
    if pin is not None and not (isinstance(pin, str) and len(pin) == 64 and all(c in "0123456789abcdef" for c in pin)):
        raise TilefishRuntimeError(f"pin= is the 64 lowercase hex digits of a plan digest, got {pin!r}")
    if mode != "replay" and (pin is not None or trust_directory):
        raise TilefishRuntimeError(f"pin= and trust_directory= are for mode='replay' (they vouch for a plan directory); mode {mode!r} runs no plan directory")
    if is_graph and manifest is not None:
        raise TilefishRuntimeError("manifest= is for a kernel or an extern; a graph replays plan=<directory> (written by tilefish.runtime.export(graph, directory))")
    if not is_graph and mode == "replay":
        raise TilefishRuntimeError("run: mode='replay' replays a graph's exported plan; a single operator of this backend is a prebuilt kernel: run it with mode='jit'")


def _values_of(graph: GraphOp, env: Dict[Dim, int]) -> Dict[str, int]:
    return {d.name: env[d] for d in P.dynamic_dims(graph)}


def _graph_runner(op: GraphOp, mode: str, plan_: Any, pin: Optional[str], trust_directory: bool, values: Dict[str, int]) -> PlanRunner:
    if mode == "replay":
        if plan_ is None or isinstance(plan_, Plan):
            raise TilefishRuntimeError("run: mode='replay' needs plan=<exported directory>")
        return _replay_runner(op, str(plan_), pin, trust_directory)
    if plan_ is not None and not isinstance(plan_, Plan):
        raise TilefishRuntimeError("run: mode='jit' takes plan=tilefish.plan(graph, ...); a directory is replayed with mode='replay'")
    return _jit_runner(op, values, plan_)


def run(op: Op, /, *args, mode: str = "jit", manifest: Any = None, pin: Optional[str] = None, trust_directory: bool = False, **kwargs):
    """Runs a declaration on torch CUDA tensors. ``mode="jit"``: the prebuilt kernels, directly. ``mode="replay"``: the plan
    exported into directory ``plan=``, verified against ``pin=`` (or ``trust_directory=True``). ``outputs=`` gives the tensors the
    results are written into; ``taps={"t3": tensor, ("t5", 4): tensor}`` copies plan buffers into the caller's tensors right after
    a step (by default the last one that writes the buffer)."""
    from . import kernels as K

    is_graph = isinstance(op, GraphOp)
    _check_run_options(mode, manifest, pin, trust_directory, is_graph)
    plan_ = kwargs.pop("plan", None) if is_graph else None
    outputs = kwargs.pop("outputs", None)
    taps = kwargs.pop("taps", None) if is_graph else None
    K.require_cuda()
    named = _named_args(op, args, kwargs)
    env = _bind_dims(op, named)
    device = next(t.device for t in named.values())
    if is_graph:
        values = _values_of(op, env)
        runner = _graph_runner(op, mode, plan_, pin, trust_directory, values)
        return runner.run(values, named, device, outputs, taps)
    out = outputs if outputs is None or not isinstance(outputs, dict) else outputs.get("out")
    if isinstance(out, (list, tuple)):
        out = out[0]
    if isinstance(op, KernelOp):
        impl = B.match_kernel(op)
        p = [q.name for q in op.signature.tensors]
        if impl == "residual_add_rmsnorm":
            return K.residual_add_rmsnorm(named[p[0]], named[p[1]], named[p[2]], float(op.signature.consts[0].default), out=out)
        return K.silu_gate(named[p[0]], named[p[1]], out=out)
    if isinstance(op, LibraryOp):
        p = [q.name for q in op.signature.tensors]
        b = named[p[1]]
        if not isinstance(b, BlockScaledTensor):
            raise TilefishRuntimeError(f"run: {op.name}: this backend implements the gemm over BlockScaled weights only")
        return K.gemm(named[p[0]], b, out=out)
    raise TilefishRuntimeError(f"run: cannot run a {type(op).__name__}")


class CapturedPlan:
    """A graph's steps captured into a CUDA graph over fixed tensors; ``replay()`` relaunches it (one thread at a time). It keeps the
    externals, the outputs and the runner (hence the arena) alive."""

    def __init__(self, cuda_graph, result, runner: PlanRunner, externals, backend: Backend, index: int) -> None:
        self._graph, self.result, self._runner, self._externals, self._backend, self._index = cuda_graph, result, runner, externals, backend, index

    @property
    def outputs(self):
        return self.result

    def replay(self, stream: Any = None):
        self._backend.replay_graph(self._graph, self._backend.stream(self._index))
        return self.result


def capture(op: GraphOp, /, *externals, mode: str = "jit", plan: Any = None, pin: Optional[str] = None, trust_directory: bool = False, outputs: Any = None,
            stream: Any = None, taps: Any = None) -> CapturedPlan:
    """Runs the graph once eagerly (warm-up: the arena is allocated and kernel attributes are set outside the capture), then captures one
    run into a CUDA graph. The argument tensors and the returned tensors are fixed: write new inputs into them before ``replay()``."""
    import torch

    if not isinstance(op, GraphOp):
        raise TilefishRuntimeError(f"capture takes a @graph, got {op!r}")
    if plan is not None and mode == "jit" and not isinstance(plan, Plan):
        mode = "replay"
    _check_run_options(mode, None, pin, trust_directory, True)
    named = _named_args(op, externals, {})
    env = _bind_dims(op, named)
    values = _values_of(op, env)
    device = next(t.device for t in named.values())
    runner = _graph_runner(op, mode, plan, pin, trust_directory, values)
    backend = runner.backend
    index = backend.device_index(device)
    result = runner.run(values, named, device, outputs, taps)  # warm-up; also allocates the results the capture writes
    torch.cuda.synchronize()
    fixed = result if outputs is None else outputs
    fixed_map = fixed if isinstance(fixed, dict) else dict(zip(runner.doc["outputs"], fixed if isinstance(fixed, (list, tuple)) else [fixed]))
    graph = backend.capture_graph(index, stream, lambda _s: runner.run(values, named, device, fixed_map, taps))
    return CapturedPlan(graph, result, runner, named, backend, index)


class BoundWeights:
    """A graph with its weights bound once (``bind_weights``): ``run`` and ``capture`` take only the other arguments."""

    def __init__(self, op: GraphOp, weights: Dict[str, Any], options: Dict[str, Any]) -> None:
        self.op, self.weights, self.options = op, dict(weights), dict(options)

    def _all(self, args) -> List[Any]:
        it = iter(args)
        out = []
        for p in self.op.signature.tensors:
            if p.name in self.weights:
                out.append(self.weights[p.name])
            else:
                try:
                    out.append(next(it))
                except StopIteration:
                    raise TilefishPreconditionError(f"{self.op.name}: argument '{p.name}' is missing", kind="shape", arg=p.name) from None
        if next(it, None) is not None:
            raise TilefishPreconditionError(f"{self.op.name}: too many arguments beside the bound weights", kind="shape")
        return out

    def run(self, *args, **kwargs):
        return run(self.op, *self._all(args), **{**self.options, **kwargs})

    def capture(self, *args, **kwargs) -> CapturedPlan:
        return capture(self.op, *self._all(args), **{**self.options, **kwargs})


def bind_weights(op: GraphOp, weights: Dict[str, Any], **options: Any) -> BoundWeights:
    """Binds the weights of a graph that declares its roles (``@graph(inputs=..., weights=...)``) once: ``w = bind_weights(graph,
    {"w_gu": q_gu, ...}, mode="replay", plan="build/", pin=digest)``, then ``w.run(x, residual)`` and ``w.capture(x, residual)``."""
    if not isinstance(op, GraphOp) or not op.param_roles:
        raise TilefishRuntimeError("bind_weights takes a @graph that declares its roles (inputs=..., weights=...)")
    for name in weights:
        if op.param_roles.get(name) != "weight":
            raise TilefishRuntimeError(f"bind_weights: '{name}' is not a weight of graph '{op.name}' (weights: {[n for n, r in op.param_roles.items() if r == 'weight']})")
    missing = [n for n, r in op.param_roles.items() if r == "weight" and n not in weights]
    if missing:
        raise TilefishRuntimeError(f"bind_weights: no tensor for the weights {missing}")
    return BoundWeights(op, weights, options)


def prepare(op: GraphOp, *, mode: str = "jit", plan: Any = None, pin: Optional[str] = None, trust_directory: bool = False, device: Any = None,
            buckets: Optional[Dict[str, Sequence[int]]] = None) -> None:
    """Does ahead of time what a run does for itself the first time and what cannot happen inside a stream capture: loads the kernel
    library, verifies and loads the plan, allocates its arena on ``device`` and checks every library step's workspace there."""
    from . import kernels as K

    K.require_cuda()
    _check_run_options(mode, None, pin, trust_directory, True)
    backend = default_backend()
    index = backend.device_index(device) if device is not None else backend.current_device()
    if mode == "replay":
        runners = [_replay_runner(op, str(plan), pin, trust_directory)]
    else:
        dims = P.bucket_values(op, buckets)
        runners = [_jit_runner(op, c, plan if isinstance(plan, Plan) else None) for c in P.bucket_combinations(dims)] if not isinstance(plan, Plan) else [_jit_runner(op, {}, plan)]
    for r in runners:
        r.arena(index)


def run_step(op: GraphOp, step: int, buffers: Dict[str, Any], *, mode: str = "jit", plan: Any = None, pin: Optional[str] = None, trust_directory: bool = False,
             bucket: Optional[Dict[str, int]] = None) -> None:
    """Launches ONE step of a graph's (verified) plan on the caller's tensors: ``buffers`` gives a tensor for every buffer the step binds, by
    name (a BlockScaledTensor for a block-scaled one; not the workspace, which is the plan's arena)."""
    from . import kernels as K

    K.require_cuda()
    _check_run_options(mode, None, pin, trust_directory, True)
    if bucket is None:
        raise TilefishRuntimeError("run_step: give bucket={dimension: size}")
    runner = _graph_runner(op, mode, plan, pin, trust_directory, dict(bucket))
    bi = runner.bucket_index(dict(bucket))
    steps = runner.doc["buckets"][bi]["steps"]
    if not 0 <= step < len(steps):
        raise TilefishRuntimeError(f"run_step: the plan has {len(steps)} steps, not a step {step}")
    device = next(t.device for t in buffers.values())
    index = runner.backend.device_index(device)
    addr = runner.addresses(buffers, index)
    runner.enqueue(bi, addr, index, runner.backend.stream(index), only_step=step)
