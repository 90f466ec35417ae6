"""Running declarations: ``run`` (modes "jit" and "replay"), ``export``, ``plan``, ``capture``.

Signatures and semantics follow the reference's run-time API (python/src/tilefish/runtime.py:1078-1147 ``export``, :1407-1449
``run``; docs/en/plan-schema-1.md:468-490): arguments are torch tensors (a ``Tensor[..., BlockScaled]`` parameter takes a
``BlockScaledTensor``), ``InOut`` tensors are updated in place, results are freshly allocated, every precondition is checked
before the first launch, and a replay verifies the exported directory against its pin. Differences that the backend forces:

* ``mode="jit"`` launches the prebuilt sm_100a kernels directly: there is nothing to compile at run time;
* ``mode="reference"`` is refused: the torch interpreter of the reference is an oracle, not a product path, and this
  package has no CPU implementation of any operator;
* the steps run through a ``Backend`` object (``launch`` / ``gemm`` / ``alloc_arena``), the plug point the reference's
  runner has (python/src/tilefish/_planrun.py:240-376); tests substitute a recording backend.
"""

from __future__ import annotations

import hashlib
import os
from typing import Any, Dict, List, Optional, Tuple

from . import backend as B
from . import _plan as P
from .decorators import GraphOp, KernelOp, LibraryOp, Op
from .dims import Dim, as_expr
from .dtypes import TORCH_NAMES, BlockScaled
from .errors import TilefishPreconditionError, TilefishRuntimeError
from .kernels import BlockScaledTensor, quantize  # noqa: F401  (re-exported: the run-time value of a BlockScaled tensor)
from ._plan import Plan, load_export, make_plan

MODES = ("jit", "replay", "reference")


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
                if e.const != actual:
                    raise TilefishPreconditionError(f"{op.name}: argument '{p.name}' has size {actual} where {formal} = {e.const} is compiled in",
                                                    kind="static_size", arg=p.name)
                continue
            if len(e.terms) == 1 and e.const == 0 and isinstance(e.terms[0][0], Dim):
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


# ---- the backend: what actually launches -------------------------------------------------------------------------------------
class Backend:
    """The runner's plug: allocate the arena, launch a kernel step, run a library (gemm) step."""

    def alloc_arena(self, nbytes: int, device):
        raise NotImplementedError

    def launch(self, step: Dict[str, Any], tensors: Dict[str, Any]) -> None:
        raise NotImplementedError

    def gemm(self, step: Dict[str, Any], tensors: Dict[str, Any]) -> None:
        raise NotImplementedError


class Sm100Backend(Backend):
    """Calls the C ABI through tilefish_b200.kernels on the current CUDA stream."""

    def alloc_arena(self, nbytes: int, device):
        import torch

        return torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)

    @staticmethod
    def _resolve(name: str, tensors: Dict[str, Any]):
        """A buffer name, ``aux[i]`` (one float of the aux buffer) or ``t[:, i]`` (column half i of a [M, 2F] tensor)."""
        if name.endswith("]") and "[" in name:
            base, idx = name[:-1].split("[", 1)
            t = tensors[base]
            if idx.startswith(":,"):
                i = int(idx.split(",")[1])
                f = t.shape[1] // 2
                return t[:, i * f:(i + 1) * f]
            i = int(idx)
            return t[i:i + 1]
        return tensors[name]

    def launch(self, step, tensors) -> None:
        from . import kernels as K

        a, impl = step["args"], step["impl"]
        r = lambda k: self._resolve(a[k], tensors) if k in a else None  # noqa: E731
        if impl == "tf_residual_add_rmsnorm":
            K.residual_add_rmsnorm(r("x"), r("residual"), r("w"), step["attrs"]["eps"], out=r("out"), want_bf16="out" in a,
                                   quantize_to=step["attrs"].get("q_format"), q_out=r("q"), amax_out=r("amax"))
        elif impl == "tf_silu_gate":
            K.silu_gate(r("gate"), r("up"), out=r("out"))
        elif impl.startswith("tf_quantize_"):
            K.quantize(r("x"), step["attrs"]["format"], out=r("q"), amax=r("amax"))
        else:
            raise TilefishRuntimeError(f"step '{step['entry']}': unknown kernel entry point {impl}")

    def gemm(self, step, tensors) -> None:
        from . import kernels as K

        a = step["args"]
        K.gemm_blockscaled(self._resolve(a["a"], tensors), self._resolve(a["b"], tensors), epilogue=step["attrs"]["epilogue"],
                           out=self._resolve(a["out"], tensors) if "out" in a else None, want_bf16="out" in a,
                           q_out=self._resolve(a["q"], tensors) if "q" in a else None,
                           amax_out=self._resolve(a["amax"], tensors) if "amax" in a else None)


_DEFAULT_BACKEND: Optional[Backend] = None


def default_backend() -> Backend:
    global _DEFAULT_BACKEND
    if _DEFAULT_BACKEND is None:
        _DEFAULT_BACKEND = Sm100Backend()
    return _DEFAULT_BACKEND


# ---- the runner ----------------------------------------------------------------------------------------------------------
class PlanRunner:
    """Executes a plan document for one bucket: intermediates are views of one arena, steps run in order on the current stream."""

    def __init__(self, doc: Dict[str, Any], backend: Optional[Backend] = None) -> None:
        self.doc = doc
        self.backend = backend or default_backend()
        self._arenas: Dict[Tuple[str, Any], Dict[str, Any]] = {}

    def _intermediates(self, key: str, device) -> Dict[str, Any]:
        import torch

        cached = self._arenas.get((key, device))
        if cached is not None:
            return cached
        bucket = self.doc["buckets"][key]
        arena = self.backend.alloc_arena(bucket["arena_bytes"], device)
        if arena.data_ptr() % self.doc["arena_alignment"]:
            raise TilefishRuntimeError("the arena is not aligned to arena_alignment")
        out: Dict[str, Any] = {"__arena__": arena}
        formats = {b["name"]: b.get("format") for b in self.doc["buffers"]}
        types = {b["name"]: b["type"] for b in self.doc["buffers"]}
        for name, entry in bucket["buffers"].items():
            if "offset" not in entry:
                continue
            shape, offs, nbytes = tuple(entry["shape"]), entry["offset"], entry["bytes"]
            if formats[name]:
                fmt = formats[name]
                rows = 1
                for s in shape[:-1]:
                    rows *= s
                codes = arena[offs["codes"]:offs["codes"] + nbytes["codes"]].view(rows, -1)
                scales = arena[offs["scales"]:offs["scales"] + nbytes["scales"]]
                gs = arena[offs["global_scale"]:offs["global_scale"] + 4].view(torch.float32) if "global_scale" in offs else None
                out[name] = BlockScaledTensor(fmt, (rows, shape[-1]), codes, scales, gs, "swizzled")
            else:
                dt = torch.float32 if types[name].endswith("f32]") else torch.bfloat16
                out[name] = arena[offs["data"]:offs["data"] + nbytes["data"]].view(dt).view(shape)
        self._arenas[(key, device)] = out
        return out

    def run(self, key: str, tensors: Dict[str, Any], device, outputs: Optional[Dict[str, Any]] = None):
        import torch

        if key not in self.doc["buckets"]:
            raise TilefishPreconditionError(f"plan '{self.doc['graph']}': no bucket {key}; the plan has {sorted(self.doc['buckets'])} (bucket semantics are "
                                            "exact: the host pads)", kind="bucket")
        bound = dict(self._intermediates(key, device))
        bound.update(tensors)
        results = []
        for b in self.doc["buffers"]:
            if b["role"] == "output":
                shape = tuple(self.doc["buckets"][key]["buffers"][b["name"]]["shape"])
                t = (outputs or {}).get(b["name"])
                if t is None:
                    t = torch.empty(shape, dtype=torch.bfloat16, device=device)
                elif tuple(t.shape) != shape or t.dtype != torch.bfloat16 or not t.is_contiguous():
                    raise TilefishPreconditionError(f"output '{b['name']}': expected a contiguous bf16 tensor of shape {shape}", kind="shape", arg=b["name"])
                bound[b["name"]] = t
                results.append(t)
        if "aux" in bound:
            bound["aux"].zero_()
        for step in self.doc["steps"]:
            (self.backend.gemm if step["kind"] == "library" else self.backend.launch)(step, bound)
        if not results:
            return None
        return results[0] if len(results) == 1 else tuple(results)


def _library_identity() -> Dict[str, Any]:
    from . import _native

    with open(_native.LIB_PATH, "rb") as f:
        sha = hashlib.sha256(f.read()).hexdigest()
    return {"file": os.path.basename(_native.LIB_PATH), "sha256": sha, "version": _native.version()}


def plan(graph: GraphOp, buckets: Optional[Dict[str, List[int]]] = None) -> Plan:
    """The launch plan of a graph (needs no GPU): ``.doc`` is the plan.json document, ``.digest`` its pin."""
    return make_plan(graph, buckets)[0]


class Export:
    def __init__(self, directory: str, plan_: Plan, manifest: Dict[str, Any]) -> None:
        self.directory, self.plan, self.manifest = directory, plan_, manifest

    @property
    def digest(self) -> str:
        return self.plan.digest

    @property
    def manifest_digest(self) -> str:
        return self.manifest["manifest_digest"]


def export(graph: GraphOp, directory: str, *, arch: str = "sm_100a", overwrite: bool = False, buckets: Optional[Dict[str, List[int]]] = None) -> Export:
    """Writes ``manifest.json`` and ``plan.json`` for ``graph`` into ``directory`` and returns their digests. The manifest
    records the kernel library this process would run (file, sha256, version); a replay refuses another build."""
    if arch != "sm_100a":
        raise TilefishRuntimeError(f"export: this backend builds for sm_100a only, not {arch}")
    pl, manifest = make_plan(graph, buckets, library=_library_identity())
    P.write_export(directory, pl, manifest, overwrite=overwrite)
    return Export(directory, pl, manifest)


_RUNNERS: Dict[Any, PlanRunner] = {}


def _runner_for(graph: GraphOp, env: Dict[Dim, int]) -> Tuple[PlanRunner, str]:
    key = (id(graph), P.bucket_key(env))
    r = _RUNNERS.get(key)
    if r is None:
        pl, _ = make_plan(graph, {d.name: [v] for d, v in env.items()})
        r = _RUNNERS[key] = PlanRunner(pl.doc)
    return r, P.bucket_key(env)


def _replay_runner(directory: str, pin: Optional[str]) -> PlanRunner:
    key = ("replay", os.path.abspath(directory), pin)
    r = _RUNNERS.get(key)
    if r is None:
        doc, manifest = load_export(directory, pin)
        lib = manifest["library"]
        mine = _library_identity()
        if lib.get("sha256") and lib["sha256"] != mine["sha256"]:
            from .errors import TilefishManifestError

            raise TilefishManifestError(f"{directory}: exported against kernel library {lib['sha256'][:12]} ({lib.get('version')}), this process loads "
                                        f"{mine['sha256'][:12]} ({mine['version']}); re-export")
        r = _RUNNERS[key] = PlanRunner(doc)
    return r


def run(op: Op, *args, mode: str = "jit", plan: Optional[str] = None, pin: Optional[str] = None, outputs: Optional[Dict[str, Any]] = None, **kwargs):
    """Runs a declaration on torch CUDA tensors. ``mode="jit"``: the prebuilt kernels, directly. ``mode="replay"``: the plan
    exported into directory ``plan``, verified against ``pin``."""
    if mode not in MODES:
        raise TilefishRuntimeError(f"run: unknown mode {mode!r} (modes: {', '.join(MODES)})")
    if mode == "reference":
        raise TilefishRuntimeError("run: mode='reference' is not part of this backend: it has no CPU implementation of any operator. The torch "
                                   "restatement used to check it lives outside the package, as test infrastructure")
    from . import kernels as K

    K.require_cuda()
    named = _named_args(op, args, kwargs)
    env = _bind_dims(op, named)
    device = next(t.device for t in named.values())
    if isinstance(op, GraphOp):
        if mode == "replay":
            if plan is None:
                raise TilefishRuntimeError("run: mode='replay' needs plan=<exported directory>")
            runner = _replay_runner(plan, pin)
            if runner.doc["graph"] != op.name:
                raise TilefishRuntimeError(f"run: {plan} holds the plan of graph '{runner.doc['graph']}', not '{op.name}'")
            return runner.run(P.bucket_key(env), named, device, outputs)
        runner, key = _runner_for(op, env)
        return runner.run(key, named, device, outputs)
    if mode == "replay":
        raise TilefishRuntimeError("run: mode='replay' replays a graph's exported plan; run a single operator with mode='jit'")
    if isinstance(op, KernelOp):
        impl = B.match_kernel(op)
        if impl == "residual_add_rmsnorm":
            p = [q.name for q in op.signature.tensors]
            return K.residual_add_rmsnorm(named[p[0]], named[p[1]], named[p[2]], float(op.signature.consts[0].default), out=(outputs or {}).get("out"))
        p = [q.name for q in op.signature.tensors]
        return K.silu_gate(named[p[0]], named[p[1]], out=(outputs or {}).get("out"))
    if isinstance(op, LibraryOp):
        p = [q.name for q in op.signature.tensors]
        b = named[p[1]]
        if not isinstance(b, BlockScaledTensor):
            raise TilefishRuntimeError(f"run: {op.name}: this backend implements the gemm over BlockScaled weights only")
        return K.gemm(named[p[0]], b, out=(outputs or {}).get("out"))
    raise TilefishRuntimeError(f"run: cannot run a {type(op).__name__}")


class CapturedPlan:
    """A graph's steps captured into a CUDA graph over fixed tensors; ``replay()`` relaunches it (one thread at a time)."""

    def __init__(self, cuda_graph, result, stream) -> None:
        self._graph, self.result, self._stream = cuda_graph, result, stream

    def replay(self):
        self._graph.replay()
        return self.result


def capture(op: GraphOp, *args, plan: Optional[str] = None, pin: Optional[str] = None, **kwargs) -> CapturedPlan:
    """Runs the graph once eagerly (warm-up: module attributes are set outside the capture), then captures one run into a CUDA
    graph. The argument tensors and the returned tensors are fixed: write new inputs into them before ``replay()``."""
    import torch

    mode = "replay" if plan is not None else "jit"
    run(op, *args, mode=mode, plan=plan, pin=pin, **kwargs)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        result = run(op, *args, mode=mode, plan=plan, pin=pin, **kwargs)
    return CapturedPlan(g, result, torch.cuda.current_stream())
