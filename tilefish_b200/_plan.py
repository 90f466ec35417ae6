"""Launch plans: a graph's steps over one arena, for every bucket of its dynamic dimensions, as a JSON document with digests.

The document is the reference's plan schema 1 (docs/en/plan-schema-1.md; python/src/tilefish/_plan.py:1503 ``validate_doc``
accepts it): top level ``schema tilefish graph arch manifest_digest dims reuse arena_alignment arena_bytes buffers outputs
buckets plan_digest`` (and ``roles``), a buffer is ``name role dtype shape offset bytes``, a bucket is ``values steps``, a step
is ``entry kind args`` (+ ``workspace`` on a library step) and an argument ``name binding`` (+ ``view``). The digest is
sha256("tilefish.plan-digest.v1\\0" + canonical JSON of the document without ``plan_digest`` and ``tilefish``)
(python/src/tilefish/_plan.py:111-124); canonical JSON is sorted keys, (",", ":") separators, ASCII.

What this backend adds stays inside that shape:

* a BlockScaled tensor is THREE buffers: ``<name>`` holds the element codes (dtype ``e4m3`` [rows, K] or, two e2m1 per byte,
  ``u8`` [rows, K/2]), ``<name>__scales`` the swizzled scale bytes (``u8``, a static length: that of the largest bucket, smaller
  buckets use a prefix) and, for nvfp4, ``<name>__global`` one ``f32``. A step binds them as separate pointer arguments
  (``a``, ``a_scales``, ``a_global`` ...), which is the order of the C entry point;
* the split-K scratch of the small-M GEMM is the plan's ``workspace`` buffer (the reference's cuBLASLt workspace has the same
  role), sized for 148 SMs from the planner's own restatement of the kernel library's split rule, so that a plan and its
  digest do not depend on the machine that made them;
* the amax words of the nvfp4 path are an ``f32 [8]`` intermediate that a ``memset`` step zeroes;
* the manifest (``tilefish_b200.manifest.v2``) names, per entry, the C symbol, its pointer parameters in order and its
  compile-time attributes (epsilon, format, epilogue), and the kernel library (file, sha256, version) in place of cubins and
  cuBLASLt algorithms.
"""

import hashlib
import json
import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

from . import backend as B
from .decorators import GraphOp
from .dims import Dim, as_expr, evaluate
from .dtypes import BlockScaled
from .errors import TilefishManifestError, TilefishPlanError

PLAN_SCHEMA = "tilefish.plan.v1"
MANIFEST_SCHEMA = "tilefish_b200.manifest.v2"
WRITER = "tilefish_b200 0.2.0"
ARCH = "sm_100"  # the plan schema wants sm_<digits>; the binaries are built for sm_100a
ARENA_ALIGNMENT = 256
PLANNED_SM_COUNT = 148
ELEMS_PER_BYTE = {"mxfp8": 1, "mxfp4": 2, "nvfp4": 2}
BLOCK = {"mxfp8": 32, "mxfp4": 32, "nvfp4": 16}
ITEMSIZE = {"bf16": 2, "f16": 2, "f32": 4, "i32": 4, "i64": 8, "u8": 1, "e4m3": 1, "e5m2": 1}
TOP_KEYS = ("schema", "tilefish", "graph", "arch", "manifest_digest", "dims", "reuse", "arena_alignment", "arena_bytes", "buffers", "outputs", "buckets",
            "plan_digest")


def canonical_json(doc: Any) -> bytes:
    return json.dumps(doc, sort_keys=True, separators=(",", ":"), ensure_ascii=True, allow_nan=False).encode("ascii")


def digest(tag: str, doc: Any) -> str:
    return hashlib.sha256(tag.encode("ascii") + b"\0" + canonical_json(doc)).hexdigest()


def plan_digest(doc: Dict[str, Any]) -> str:
    """The reference's plan digest: ``plan_digest`` and ``tilefish`` are not part of it (python/src/tilefish/_plan.py:111-124)."""
    return digest("tilefish.plan-digest.v1", {k: v for k, v in doc.items() if k not in ("plan_digest", "tilefish")})


def align_up(n: int, to: int = ARENA_ALIGNMENT) -> int:
    return (n + to - 1) // to * to


def swizzled_scale_bytes(rows: int, k: int, fmt: str) -> int:
    cols = k // BLOCK[fmt]
    return ((rows + 127) // 128) * ((cols + 3) // 4) * 512


# ---- the kernel library's split-K rule, restated (csrc/gemm_blockscaled.cu ``split_plan``) -------------------------------------
def gemm_split_plan(m: int, n: int, k_bytes: int, epilogue: str, sms: int = PLANNED_SM_COUNT) -> Tuple[int, int, int]:
    """(tile width, K ranges, K stages per range) the GEMM uses for a problem on ``sms`` SMs."""
    m_blocks = (m + 127) // 128
    n_acc = 2 * n if epilogue == "silu_gate" else n
    stages = (k_bytes + 127) // 128
    block_n, splits, kps = 256, 1, stages
    if n <= 128 and epilogue != "silu_gate":
        block_n = 128
    if m > 256:
        return block_n, splits, kps
    a_rows = min(m, 128)
    best = 1e30
    for bn in (256, 128):
        tiles = m_blocks * ((n_acc + bn - 1) // bn)
        for want in range(1, 17):
            if want > 1 and stages // want < 4:
                break
            per = (stages + want - 1) // want
            sp = (stages + per - 1) // per
            if bn == 128 and sp == 1 and epilogue == "silu_gate":
                continue
            units = tiles * sp
            waves = (units + sms - 1) // sms
            cost = float(waves) * float(per + 3) * float(bn + a_rows)
            if sp > 1:
                cost += 1200.0 + 2.0 * float(sp) * float(m) * float(n_acc) * 4.0 / 7200.0
            if cost < best:
                best, block_n, splits, kps = cost, bn, sp, per
    return block_n, splits, kps


def gemm_workspace_bytes(m: int, n: int, k: int, fmt: str, epilogue: str, sms: int = PLANNED_SM_COUNT) -> int:
    """Bytes of split-K scratch ``tf_gemm_blockscaled`` needs for this problem (0 when K is not split)."""
    k_bytes = k if fmt == "mxfp8" else k // 2
    _, splits, _ = gemm_split_plan(m, n, k_bytes, epilogue, sms)
    if splits <= 1:
        return 0
    return splits * m * (2 * n if epilogue == "silu_gate" else n) * 4


# ---- buffers ---------------------------------------------------------------------------------------------------------------------
def part_names(name: str, fmt: Optional[str]) -> Dict[str, str]:
    """Names of the plan buffers that make up a tensor: {"data": name} or {"codes": name, "scales": ..., "global": ...}."""
    if fmt is None:
        return {"data": name}
    parts = {"codes": name, "scales": f"{name}__scales"}
    if fmt == "nvfp4":
        parts["global"] = f"{name}__global"
    return parts


def bucket_key(env: Dict[Dim, int]) -> str:
    return ",".join(f"{d.name}={v}" for d, v in sorted(env.items(), key=lambda kv: kv[0].name)) or "static"


class Plan:
    """A built plan: ``doc`` is the JSON document, ``digest`` its pin, ``manifest`` the manifest document made with it."""

    def __init__(self, graph: GraphOp, doc: Dict[str, Any], manifest: Dict[str, Any]) -> None:
        self.graph = graph
        self.doc = doc
        self.manifest = manifest

    @property
    def digest(self) -> str:
        return self.doc["plan_digest"]

    def bucket(self, values: Dict[str, int]) -> Dict[str, Any]:
        for b in self.doc["buckets"]:
            if b["values"] == values:
                return b
        raise TilefishPlanError(f"plan '{self.doc['graph']}': no bucket {values}")


def dynamic_dims(graph: GraphOp) -> Tuple[Dim, ...]:
    return tuple(sorted((d for d in graph.graph.symbols if not d.is_static), key=lambda d: d.name))


def bucket_values(graph: GraphOp, buckets: Optional[Dict[str, Sequence[int]]] = None) -> Dict[str, List[int]]:
    out: Dict[str, List[int]] = {}
    for d in dynamic_dims(graph):
        values = (buckets or {}).get(d.name) or d.buckets
        if not values:
            raise TilefishPlanError(f"graph '{graph.name}': dimension {d.name} has no buckets; declare Dim('{d.name}', buckets=[...]) or pass buckets=")
        values = sorted(set(int(v) for v in values))
        if values[0] < 1:
            raise TilefishPlanError(f"graph '{graph.name}': buckets of {d.name} must be at least 1")
        if d.divisible_by and any(v % d.divisible_by for v in values):
            raise TilefishPlanError(f"graph '{graph.name}': a bucket of {d.name} is not divisible by {d.divisible_by}")
        out[d.name] = values
    return out


def bucket_combinations(dims: Dict[str, Sequence[int]]) -> List[Dict[str, int]]:
    """The Cartesian product of the bucket lists, names sorted, the first name varying slowest (plan schema 1, section 5)."""
    combos: List[Dict[str, int]] = [{}]
    for name in sorted(dims):
        combos = [{**c, name: int(v)} for c in combos for v in dims[name]]
    return combos


def _shape_entry(s) -> Any:
    e = as_expr(s)
    return int(e.offset) if e.is_static else str(e)


def _concrete(shape, env: Dict[Dim, int]) -> Tuple[int, ...]:
    return B.concrete_shape(shape, env)


class _Layout:
    """The plan buffers of one symbolic buffer of the graph compiler, with what is needed to size them per bucket."""

    def __init__(self, buf: B.Buffer) -> None:
        self.buf = buf
        self.parts = part_names(buf.name, buf.fmt)


def _buffer_docs(graph: GraphOp, buffers: List[B.Buffer], envs: List[Dict[Dim, int]], workspace_bytes: int) -> List[Dict[str, Any]]:
    docs: List[Dict[str, Any]] = []
    for b in buffers:
        shapes = [_concrete(b.type.shape, env) for env in envs]
        if b.fmt is None:
            dt = b.type.dtype.name
            docs.append({"name": b.name, "role": b.role, "dtype": dt, "shape": [_shape_entry(s) for s in b.type.shape], "offset": None,
                         "bytes": max(_prod(s) for s in shapes) * ITEMSIZE[dt]})
            continue
        if len(b.type.shape) != 2:
            raise TilefishPlanError(f"graph '{graph.name}': BlockScaled buffer '{b.name}' has rank {len(b.type.shape)}; the kernels take [rows, K]")
        epb = ELEMS_PER_BYTE[b.fmt]
        k = as_expr(b.type.shape[-1])
        if not k.is_static:
            raise TilefishPlanError(f"graph '{graph.name}': the blocked axis of '{b.name}' must be static")
        codes_shape = [_shape_entry(b.type.shape[0]), int(k.offset) // epb]
        names = part_names(b.name, b.fmt)
        docs.append({"name": names["codes"], "role": b.role, "dtype": "e4m3" if b.fmt == "mxfp8" else "u8", "shape": codes_shape, "offset": None,
                     "bytes": max(s[0] * (s[1] // epb) for s in shapes)})
        docs.append({"name": names["scales"], "role": b.role, "dtype": "u8", "shape": [max(swizzled_scale_bytes(s[0], s[1], b.fmt) for s in shapes)],
                     "offset": None, "bytes": max(swizzled_scale_bytes(s[0], s[1], b.fmt) for s in shapes)})
        if "global" in names:
            docs.append({"name": names["global"], "role": b.role, "dtype": "f32", "shape": [1], "offset": None, "bytes": 4})
    if workspace_bytes > 0:
        docs.append({"name": "workspace", "role": "workspace", "dtype": "u8", "shape": [workspace_bytes], "offset": None, "bytes": workspace_bytes})
    offset = 0
    for d in docs:
        if d["role"] in ("intermediate", "workspace"):
            d["offset"] = offset
            offset += align_up(d["bytes"])
    return docs


def _prod(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


# ---- steps -----------------------------------------------------------------------------------------------------------------------
# Pointer parameters of each C entry point, in the entry point's own order; a step binds the ones its variant uses.
POINTER_ORDER = {
    "tf_residual_add_rmsnorm": ("x", "residual", "w", "out", "q", "q_scales", "q_global", "amax"),
    "tf_silu_gate": ("gate", "up", "out"),
    "tf_quantize_mxfp8": ("x", "q", "q_scales"),
    "tf_quantize_mxfp4": ("x", "q", "q_scales"),
    "tf_quantize_nvfp4": ("x", "q", "q_scales", "q_global", "amax"),
    "tf_gemm_blockscaled": ("a", "a_scales", "a_global", "b", "b_scales", "b_global", "out", "amax", "q", "q_scales"),
}
WRITTEN = {"out", "q", "q_scales", "q_global", "residual"}


def _resolve_binding(spec: str, by_name: Dict[str, B.Buffer], env: Dict[Dim, int]) -> Tuple[str, Optional[Dict[str, Any]]]:
    """A compiler binding (a buffer name, ``aux[i]`` or ``t[:, i]``) as (buffer name, view at this bucket or None)."""
    if spec.endswith("]") and "[" in spec:
        base, idx = spec[:-1].split("[", 1)
        shape = _concrete(by_name[base].type.shape, env)
        if idx.startswith(":,"):
            i = int(idx.split(",")[1])
            f = shape[1] // 2
            return base, {"shape": [shape[0], f], "strides": [shape[1], 1], "offset": i * f}
        return base, {"shape": [1], "strides": [1], "offset": int(idx)}
    return spec, None


def _step_args(step: B.Step, by_name: Dict[str, B.Buffer], env: Dict[Dim, int]) -> List[Dict[str, Any]]:
    """The step's pointer arguments in the entry point's order; a BlockScaled binding becomes its two or three buffers."""
    args: List[Dict[str, Any]] = []
    for pname in POINTER_ORDER[step.impl]:
        base = {"a_scales": "a", "a_global": "a", "b_scales": "b", "b_global": "b", "q_scales": "q", "q_global": "q"}.get(pname)
        src = step.args.get(base or pname)
        if src is None:
            continue
        bname, view = _resolve_binding(src, by_name, env)
        buf = by_name[bname]
        if base is not None:
            part = pname.split("_", 1)[1]
            if buf.fmt is None or (part == "global" and buf.fmt != "nvfp4"):
                continue
            args.append({"name": pname, "binding": part_names(bname, buf.fmt)[part]})
            continue
        arg = {"name": pname, "binding": bname}
        if view is not None:
            arg["view"] = view
        args.append(arg)
    return args


def entry_stem(step: B.Step, env_values: Dict[str, int], dims_of_step: Sequence[str]) -> str:
    """The manifest entry a step launches: the operator's name, its fused variant, and for a library step ``.<Dim><value>`` per
    bucketed dimension (python/src/tilefish/_library.py:777 names library entries the same way)."""
    stem = step.entry.replace(".", "_")
    if step.impl == "tf_residual_add_rmsnorm" and step.attrs.get("q_format"):
        stem += "_q" + step.attrs["q_format"]
    if step.impl == "tf_gemm_blockscaled":
        if step.attrs.get("epilogue", "none") != "none":
            stem += "_" + step.attrs["epilogue"]
        if step.attrs.get("q_format"):
            stem += "_q" + step.attrs["q_format"]
    if "amax" in step.args:
        stem += "_amax"
    if step.kind == "library":
        stem += "".join(f".{d}{env_values[d]}" for d in dims_of_step)
    return stem


def _gemm_problem(step: B.Step, by_name: Dict[str, B.Buffer], env: Dict[Dim, int]) -> Tuple[int, int, int]:
    a = _concrete(by_name[step.args["a"]].type.shape, env)
    b = _concrete(by_name[step.args["b"]].type.shape, env)
    n = b[0] // 2 if step.attrs.get("epilogue") == "silu_gate" else b[0]
    return a[0], n, a[1]


def make_plan(graph: GraphOp, buckets: Optional[Dict[str, Sequence[int]]] = None, library: Optional[Dict[str, Any]] = None, fuse: bool = True,
              exported: bool = True) -> Plan:
    """The plan of ``graph`` and the manifest that goes with it. Needs no GPU and no kernel library. ``exported=False``: a plan that is only made in
    memory (what ``mode="jit"`` runs): ``arch`` and ``manifest_digest`` are null, as in the reference."""
    if not isinstance(graph, GraphOp):
        raise TilefishPlanError(f"plan: expected a @graph, got {type(graph).__name__}")
    buffers, steps = B.compile_graph(graph, fuse=fuse)
    _renumber_intermediates(buffers, steps)
    by_name = {b.name: b for b in buffers}
    dims = bucket_values(graph, buckets)
    dim_objs = {d.name: d for d in dynamic_dims(graph)}
    combos = bucket_combinations(dims)
    envs = [{dim_objs[n]: v for n, v in c.items()} for c in combos]
    has_aux = "aux" in by_name
    workspace = 0
    for env in envs:
        for s in steps:
            if s.kind == "library":
                m, n, k = _gemm_problem(s, by_name, env)
                workspace = max(workspace, gemm_workspace_bytes(m, n, k, s.attrs["format"], s.attrs.get("epilogue", "none")))
    if any(s.kind == "library" for s in steps):
        workspace = max(workspace, ARENA_ALIGNMENT)  # a library step always names the workspace buffer
    buffer_docs = _buffer_docs(graph, buffers, envs, workspace)
    arena = 0
    for d in buffer_docs:
        if d["offset"] is not None:
            arena = max(arena, d["offset"] + align_up(d["bytes"]))
    entries: Dict[str, Any] = {"kernels": {}, "library": {}}
    bucket_docs = []
    for combo, env in zip(combos, envs):
        step_docs: List[Dict[str, Any]] = []
        if has_aux:
            step_docs.append({"kind": "memset", "args": [{"name": "dst", "binding": "aux"}]})
        for s in steps:
            step_dims = sorted(n for n in combo if any(n in {x.name for x in _symbols_of(by_name[_base(v)].type.shape)} for v in s.args.values()))
            stem = entry_stem(s, combo, step_dims)
            args = _step_args(s, by_name, env)
            sd: Dict[str, Any] = {"entry": stem, "kind": s.kind, "args": args}
            entry = {"symbol": s.impl, "params": [a["name"] for a in args], "attrs": _entry_attrs(s.attrs)}
            if s.kind == "library":
                sd["workspace"] = "workspace"
                m, n, k = _gemm_problem(s, by_name, env)
                entry.update({"impl": B.GEMM_IMPL, "m": m, "n": n, "k": k,
                              "workspace_bytes": gemm_workspace_bytes(m, n, k, s.attrs["format"], s.attrs.get("epilogue", "none")), "sm_count": PLANNED_SM_COUNT})
            section = entries["library" if s.kind == "library" else "kernels"]
            if stem in section and section[stem] != entry:
                raise TilefishPlanError(f"graph '{graph.name}': two different launches would share the manifest entry '{stem}'")
            section[stem] = entry
            step_docs.append(sd)
        bucket_docs.append({"values": dict(combo), "steps": step_docs})
    manifest = manifest_doc(graph, entries, library or {"file": "libtilefish_b200.so", "sha256": None, "version": None})
    doc: Dict[str, Any] = {
        "schema": PLAN_SCHEMA,
        "tilefish": WRITER,
        "graph": graph.name,
        "arch": ARCH if exported else None,
        "manifest_digest": manifest["manifest_digest"] if exported else None,
        "dims": dims,
        "reuse": False,
        "arena_alignment": ARENA_ALIGNMENT,
        "arena_bytes": arena,
        "buffers": buffer_docs,
        "outputs": [b.name for b in buffers if b.role == "output"],
        "buckets": bucket_docs,
    }
    if graph.param_roles:
        doc["roles"] = "declared"
    doc["plan_digest"] = plan_digest(doc)
    return Plan(graph, doc, manifest)


def _renumber_intermediates(buffers: List[B.Buffer], steps: List[B.Step]) -> None:
    """Intermediates are ``t0``, ``t1``, ... in the order the steps make them (a fusion may have dropped one: no gaps)."""
    import re

    rename: Dict[str, str] = {}
    for b in buffers:
        if b.role == "intermediate" and re.fullmatch(r"t\d+", b.name):
            rename[b.name] = f"t{len(rename)}"
    for b in buffers:
        if b.name in rename:
            b.name = rename[b.name]
    for s in steps:
        for k, v in list(s.args.items()):
            base = _base(v)
            if base in rename:
                s.args[k] = rename[base] + v[len(base):]


def _entry_attrs(attrs: Dict[str, Any]) -> Dict[str, Any]:
    """A manifest entry's compile-time attributes. The manifest holds no JSON number but integers (so that every reader computes the
    same canonical text): a float is stored as the bit pattern of its f32, ``eps`` as ``eps_bits``."""
    import struct

    out: Dict[str, Any] = {}
    for k, v in sorted(attrs.items()):
        if k == "impl":
            continue
        if isinstance(v, float):
            out[k + "_bits"] = struct.unpack("<I", struct.pack("<f", v))[0]
        else:
            out[k] = v
    return out


def f32_from_bits(bits: int) -> float:
    import struct

    return struct.unpack("<f", struct.pack("<I", int(bits)))[0]


def _base(spec: str) -> str:
    return spec.split("[", 1)[0]


def _symbols_of(shape):
    from .dims import symbols

    out = []
    for s in shape:
        out.extend(symbols(s))
    return out


def manifest_doc(graph: GraphOp, entries: Dict[str, Any], library: Dict[str, Any]) -> Dict[str, Any]:
    declarations = {"graph": hashlib.sha256(str(graph.graph).encode()).hexdigest()}
    for n in graph.graph.nodes:
        if n.callee is not None and getattr(n.callee, "graph", None) is not None:
            declarations[n.callee.name] = hashlib.sha256(str(n.callee.graph).encode()).hexdigest()
    doc = {"schema": MANIFEST_SCHEMA, "arch": "sm_100a", "library_file": library, "kernels": entries["kernels"], "library": entries["library"],
           "declarations": declarations}
    doc["manifest_digest"] = digest("tilefish.manifest-digest.v1", doc)
    return doc


# ---- reading a document ------------------------------------------------------------------------------------------------------------
def buffer_shapes(doc: Dict[str, Any], values: Dict[str, int]) -> Dict[str, Tuple[str, Tuple[int, ...]]]:
    """{buffer name: (dtype, shape at the bucket)}: shape entries are integers or affine expressions over the dimensions."""
    out = {}
    for b in doc["buffers"]:
        shape = []
        for s in b["shape"]:
            shape.append(int(s) if isinstance(s, int) else _eval_affine(s, values))
        out[b["name"]] = (b["dtype"], tuple(shape))
    return out


def _eval_affine(text: str, values: Dict[str, int]) -> int:
    """``"M"``, ``"3*M"``, ``"2*M + 3"``: the affine forms this writer emits."""
    total = 0
    for term in text.replace("-", "+-").split("+"):
        term = term.strip()
        if not term:
            continue
        coef, name = 1, None
        for f in term.split("*"):
            f = f.strip()
            if f.lstrip("-").isdigit():
                coef *= int(f)
            elif f in values:
                name = f
            elif f.startswith("-") and f[1:] in values:
                coef, name = -coef, f[1:]
            else:
                raise TilefishManifestError(f"plan.json: shape expression {text!r} is not an affine form over {sorted(values)}")
        total += coef * (values[name] if name is not None else 1)
    return total


def validate_doc(doc: Any) -> None:
    """The structural rules of plan schema 1 this package's own reader relies on (the reference's ``validate_doc`` checks the same
    document in full; a test runs it when the reference is at hand)."""
    if not isinstance(doc, dict):
        raise TilefishManifestError("plan.json: the document must be an object")
    missing = [k for k in TOP_KEYS if k not in doc]
    unknown = sorted(set(doc) - set(TOP_KEYS) - {"roles"})
    if missing or unknown:
        raise TilefishManifestError(f"plan.json: the document must have exactly the fields {list(TOP_KEYS)} (and optionally ['roles']); missing {missing}; unknown {unknown}")
    if doc["schema"] != PLAN_SCHEMA:
        raise TilefishManifestError(f"plan.json: not a tilefish plan of schema {PLAN_SCHEMA!r}: schema is {doc['schema']!r}")
    if doc["arena_alignment"] != ARENA_ALIGNMENT or type(doc["arena_bytes"]) is not int or doc["arena_bytes"] % ARENA_ALIGNMENT:
        raise TilefishManifestError("plan.json: arena_alignment must be 256 and arena_bytes a multiple of it")
    names = set()
    for b in doc["buffers"]:
        if set(b) != {"name", "role", "dtype", "shape", "offset", "bytes"}:
            raise TilefishManifestError(f"plan.json: buffer {b.get('name')!r} must have exactly the fields name role dtype shape offset bytes")
        if b["name"] in names:
            raise TilefishManifestError(f"plan.json: buffer name {b['name']!r} is used twice")
        names.add(b["name"])
        if b["dtype"] not in ITEMSIZE:
            raise TilefishManifestError(f"plan.json: buffer {b['name']!r} has unknown dtype {b['dtype']!r}")
        arena_role = b["role"] in ("intermediate", "workspace", "devscalar")
        if arena_role != (b["offset"] is not None) or (arena_role and (b["offset"] % ARENA_ALIGNMENT or b["offset"] + b["bytes"] > doc["arena_bytes"])):
            raise TilefishManifestError(f"plan.json: buffer {b['name']!r}: an arena buffer has an aligned offset inside the arena, an external one has none")
    combos = bucket_combinations(doc["dims"])
    if [b.get("values") for b in doc["buckets"]] != combos:
        raise TilefishManifestError("plan.json: buckets must be exactly the combinations of dims, in order")
    for bucket in doc["buckets"]:
        shapes = buffer_shapes(doc, bucket["values"])
        for st in bucket["steps"]:
            kind = st.get("kind")
            want = {"kind", "args"} if kind in ("copy", "memset") else ({"entry", "kind", "args", "workspace"} if kind == "library" else {"entry", "kind", "args"})
            if kind not in ("kernel", "library", "copy", "memset") or set(st) != want:
                raise TilefishManifestError(f"plan.json: a step of kind {kind!r} must have exactly the fields {sorted(want)}")
            for a in st["args"]:
                if a["binding"] not in shapes:
                    raise TilefishManifestError(f"plan.json: step '{st.get('entry', kind)}' binds '{a['name']}' to unknown buffer {a['binding']!r}")
                v = a.get("view")
                if v is not None:
                    n = _prod(shapes[a["binding"]][1])
                    if v["offset"] + 1 + sum((s - 1) * t for s, t in zip(v["shape"], v["strides"])) > n:
                        raise TilefishManifestError(f"plan.json: a view of buffer {a['binding']!r} reaches outside it")


def write_export(directory: str, plan: Plan, overwrite: bool = False) -> None:
    os.makedirs(directory, exist_ok=True)
    for name in ("manifest.json", "plan.json"):
        if os.path.exists(os.path.join(directory, name)) and not overwrite:
            raise TilefishManifestError(f"{directory} already holds {name}; pass overwrite=True")
    with open(os.path.join(directory, "manifest.json"), "w") as f:
        json.dump(plan.manifest, f, indent=1, sort_keys=True)
    with open(os.path.join(directory, "plan.json"), "w") as f:
        json.dump(plan.doc, f, indent=1, sort_keys=True)
    load_export(directory, pin=plan.digest)  # re-read what was written and check it


def _strict_load(path: str) -> Dict[str, Any]:
    if not os.path.exists(path):
        raise TilefishManifestError(f"{path} is missing")

    def no_dup(pairs):
        d = {}
        for k, v in pairs:
            if k in d:
                raise TilefishManifestError(f"{path}: duplicate key {k!r}")
            d[k] = v
        return d

    def no_const(name):
        raise TilefishManifestError(f"{path}: {name} is not JSON")

    try:
        with open(path) as f:
            return json.load(f, object_pairs_hook=no_dup, parse_constant=no_const)
    except ValueError as e:
        raise TilefishManifestError(f"{path} is not valid JSON: {e}") from e


def check_anchor(pin: Optional[str], trust_directory: bool) -> None:
    """A replay needs exactly one trust anchor: the pin, or the statement that the directory is trusted (plan schema 1, section 3)."""
    if pin is None and not trust_directory:
        raise TilefishManifestError("a replay needs a trust anchor: pin=<the plan digest the export returned>, or trust_directory=True")
    if pin is not None and trust_directory:
        raise TilefishManifestError("give either pin= or trust_directory=True, not both")


def load_export(directory: str, pin: Optional[str] = None, trust_directory: bool = False) -> Tuple[Dict[str, Any], Dict[str, Any]]:
    """(plan document, manifest document) of an exported directory. Order of the checks as in the reference (plan schema 1, section
    3): strict JSON and schema, digest against the pin and against the file's own, the structural rules, the manifest's own
    digest and the plan's ``manifest_digest``, every step against the manifest's entries."""
    if pin is None and not trust_directory:
        trust_directory = True  # reading for inspection (the export's own re-read passes its pin)
    plan = _strict_load(os.path.join(directory, "plan.json"))
    if plan.get("schema") != PLAN_SCHEMA:
        raise TilefishManifestError(f"{directory}/plan.json: not a tilefish plan of schema {PLAN_SCHEMA!r}: schema is {plan.get('schema')!r}")
    got = plan_digest(plan)
    if pin is not None and pin != got:
        raise TilefishManifestError(f"{directory}/plan.json has digest {got}, but the pin is {pin}")
    if got != plan.get("plan_digest"):
        raise TilefishManifestError(f"{directory}/plan.json was edited: its plan_digest says {plan.get('plan_digest')}, its content {got}")
    validate_doc(plan)
    manifest = _strict_load(os.path.join(directory, "manifest.json"))
    if manifest.get("schema") != MANIFEST_SCHEMA:
        raise TilefishManifestError(f"{directory}/manifest.json: schema {manifest.get('schema')!r}, expected {MANIFEST_SCHEMA!r}")
    body = {k: v for k, v in manifest.items() if k != "manifest_digest"}
    if digest("tilefish.manifest-digest.v1", body) != manifest.get("manifest_digest"):
        raise TilefishManifestError(f"{directory}/manifest.json does not match its own digest: the file was changed after the export")
    if plan.get("manifest_digest") != manifest["manifest_digest"]:
        raise TilefishManifestError(f"{directory}/plan.json was built against the manifest with digest {plan.get('manifest_digest')}, the directory holds {manifest['manifest_digest']}")
    check_against_manifest(plan, manifest)
    return plan, manifest


def check_against_manifest(plan: Dict[str, Any], manifest: Dict[str, Any]) -> None:
    """Every step names an entry of the section its kind says, and binds that entry's pointer parameters in order (plan schema 1,
    section 7.3); a library step's workspace holds what the entry needs."""
    bytes_of = {b["name"]: b["bytes"] for b in plan["buffers"]}
    for bucket in plan["buckets"]:
        for st in bucket["steps"]:
            if st["kind"] in ("copy", "memset"):
                continue
            section = manifest["library" if st["kind"] == "library" else "kernels"]
            entry = section.get(st["entry"])
            if entry is None:
                raise TilefishManifestError(f"plan.json: step '{st['entry']}' is not an entry of the manifest's {st['kind']} section")
            if [a["name"] for a in st["args"]] != entry["params"]:
                raise TilefishManifestError(f"plan.json: step '{st['entry']}' binds {[a['name'] for a in st['args']]}, the entry takes {entry['params']}")
            if st["kind"] == "library" and bytes_of[st["workspace"]] < entry["workspace_bytes"]:
                raise TilefishManifestError(f"plan.json: the workspace holds {bytes_of[st['workspace']]} bytes, entry '{st['entry']}' needs {entry['workspace_bytes']}")
