"""Launch plans: a graph's steps over one arena, per bucket of its dynamic dimensions, as a JSON document with digests.

Follows the reference's plan format in spirit (docs/en/plan-schema-1.md:41-66, :168-196; python/src/tilefish/_plan.py:111-124):
``schema`` "tilefish.plan.v1", a ``buffers`` table (inputs, weights, outputs, intermediates at 256-byte aligned arena
offsets), ordered ``steps`` of kind "kernel" or "library" per bucket, a ``manifest_digest`` and a ``plan_digest`` =
sha256("tilefish.plan-digest.v1\\0" + canonical JSON of the document without the digest). Canonical JSON is sorted keys,
(",", ":") separators, ASCII. Additions for this backend: a BlockScaled buffer is three bindings (codes, swizzled scale bytes,
optional f32 global scale), each with its own arena offset; the manifest names the CUDA library (file, sha256, version) and
the C entry point of every step instead of cubins and cuBLASLt algorithms.
"""

import hashlib
import json
import os
from typing import Any, Dict, List, Optional, Tuple

from . import backend as B
from .decorators import GraphOp
from .dims import Dim
from .dtypes import BlockScaled
from .errors import TilefishManifestError, TilefishPlanError

PLAN_SCHEMA = "tilefish.plan.v1"
MANIFEST_SCHEMA = "tilefish_b200.manifest.v1"
ARENA_ALIGNMENT = 256
ELEMS_PER_BYTE = {"mxfp8": 1, "mxfp4": 2, "nvfp4": 2}
BLOCK = {"mxfp8": 32, "mxfp4": 32, "nvfp4": 16}


def canonical_json(doc: Any) -> bytes:
    return json.dumps(doc, sort_keys=True, separators=(",", ":"), ensure_ascii=True).encode("ascii")


def digest(tag: str, doc: Any) -> str:
    return hashlib.sha256(tag.encode("ascii") + b"\0" + canonical_json(doc)).hexdigest()


def _align(n: int) -> int:
    return (n + ARENA_ALIGNMENT - 1) // ARENA_ALIGNMENT * ARENA_ALIGNMENT


def swizzled_scale_bytes(rows: int, k: int, fmt: str) -> int:
    cols = k // BLOCK[fmt]
    return ((rows + 127) // 128) * ((cols + 3) // 4) * 512


def buffer_parts(shape: Tuple[int, ...], dtype, fmt: Optional[str]) -> Dict[str, int]:
    """Bytes of each binding of a buffer: {"data": n} or {"codes": n, "scales": n, "global_scale": 4}."""
    if fmt is None:
        n = 1
        for s in shape:
            n *= s
        return {"data": n * dtype.itemsize}
    rows = 1
    for s in shape[:-1]:
        rows *= s
    k = shape[-1]
    parts = {"codes": rows * k // ELEMS_PER_BYTE[fmt], "scales": swizzled_scale_bytes(rows, k, fmt)}
    if fmt == "nvfp4":
        parts["global_scale"] = 4
    return parts


def bucket_key(env: Dict[Dim, int]) -> str:
    return ",".join(f"{d.name}={v}" for d, v in sorted(env.items(), key=lambda kv: kv[0].name)) or "static"


class Plan:
    """A built plan: ``doc`` is the JSON document, ``digest`` its pin."""

    def __init__(self, graph: GraphOp, doc: Dict[str, Any], buffers: List[B.Buffer], steps: List[B.Step]) -> None:
        self.graph = graph
        self.doc = doc
        self.buffers = buffers
        self.steps = steps

    @property
    def digest(self) -> str:
        return self.doc["plan_digest"]


def dynamic_dims(graph: GraphOp) -> Tuple[Dim, ...]:
    return tuple(d for d in graph.graph.symbols if not d.is_static)


def bucket_envs(graph: GraphOp, buckets: Optional[Dict[str, List[int]]] = None) -> List[Dict[Dim, int]]:
    dims = dynamic_dims(graph)
    envs: List[Dict[Dim, int]] = [{}]
    for d in dims:
        values = (buckets or {}).get(d.name) or d.buckets
        if not values:
            raise TilefishPlanError(f"graph '{graph.name}': dimension {d.name} has no buckets; declare Dim('{d.name}', buckets=[...]) or pass buckets=")
        if d.divisible_by and any(v % d.divisible_by for v in values):
            raise TilefishPlanError(f"graph '{graph.name}': a bucket of {d.name} is not divisible by {d.divisible_by}")
        envs = [{**e, d: int(v)} for e in envs for v in values]
    return envs


def layout_bucket(buffers: List[B.Buffer], env: Dict[Dim, int]) -> Tuple[Dict[str, Any], int]:
    """Arena offsets of the intermediates for one binding of the dynamic dimensions (no reuse: every intermediate has its own range)."""
    table: Dict[str, Any] = {}
    offset = 0
    for b in buffers:
        shape = B.concrete_shape(b.type.shape, env)
        dtype = b.type.dtype.elem if isinstance(b.type.dtype, BlockScaled) else b.type.dtype
        parts = buffer_parts(shape, dtype, b.fmt)
        entry: Dict[str, Any] = {"shape": list(shape), "bytes": parts}
        if b.role == "intermediate":
            offs = {}
            for k, n in parts.items():
                offs[k] = offset
                offset = _align(offset + n)
            entry["offset"] = offs
        table[b.name] = entry
    return table, offset


def manifest_doc(graph: GraphOp, steps: List[B.Step], library: Dict[str, Any]) -> Dict[str, Any]:
    entries = {}
    for s in steps:
        entries[s.entry] = {"kind": s.kind, "symbol": s.impl, "attrs": {k: v for k, v in s.attrs.items()}}
    declarations = {"graph": hashlib.sha256(str(graph.graph).encode()).hexdigest()}
    for n in graph.graph.nodes:
        if n.callee is not None and getattr(n.callee, "graph", None) is not None:
            declarations[n.callee.name] = hashlib.sha256(str(n.callee.graph).encode()).hexdigest()
    doc = {"schema": MANIFEST_SCHEMA, "arch": "sm_100a", "library": library, "entries": entries, "declarations": declarations}
    doc["manifest_digest"] = digest("tilefish.manifest-digest.v1", doc)
    return doc


def make_plan(graph: GraphOp, buckets: Optional[Dict[str, List[int]]] = None, library: Optional[Dict[str, Any]] = None, fuse: bool = True) -> Tuple[Plan, Dict[str, Any]]:
    """(plan, manifest document) of ``graph``. Needs no GPU."""
    if not isinstance(graph, GraphOp):
        raise TilefishPlanError(f"plan: expected a @graph, got {type(graph).__name__}")
    buffers, steps = B.compile_graph(graph, fuse=fuse)
    manifest = manifest_doc(graph, steps, library or {"file": "libtilefish_b200.so", "sha256": None, "version": None})
    doc: Dict[str, Any] = {
        "schema": PLAN_SCHEMA,
        "backend": "tilefish_b200/sm_100a",
        "graph": graph.name,
        "arena_alignment": ARENA_ALIGNMENT,
        "roles": "declared",
        "reuse": False,
        "buffers": [{"name": b.name, "role": b.role, "type": repr(b.type), **({"format": b.fmt} if b.fmt else {})} for b in buffers],
        "steps": [s.doc() for s in steps],
        "buckets": {},
        "manifest_digest": manifest["manifest_digest"],
    }
    for env in bucket_envs(graph, buckets):
        table, arena = layout_bucket(buffers, env)
        doc["buckets"][bucket_key(env)] = {"dims": {d.name: v for d, v in env.items()}, "arena_bytes": arena, "buffers": table}
    doc["plan_digest"] = digest("tilefish.plan-digest.v1", doc)
    return Plan(graph, doc, buffers, steps), manifest


# ---- files --------------------------------------------------------------------------------------------------------------
def write_export(directory: str, plan: Plan, manifest: Dict[str, Any], overwrite: bool = False) -> None:
    os.makedirs(directory, exist_ok=True)
    for name in ("manifest.json", "plan.json"):
        if os.path.exists(os.path.join(directory, name)) and not overwrite:
            raise TilefishManifestError(f"{directory} already holds {name}; pass overwrite=True")
    with open(os.path.join(directory, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
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

    try:
        with open(path) as f:
            return json.load(f, object_pairs_hook=no_dup)
    except ValueError as e:
        raise TilefishManifestError(f"{path} is not valid JSON: {e}") from e


def load_export(directory: str, pin: Optional[str] = None) -> Tuple[Dict[str, Any], Dict[str, Any]]:
    """(plan document, manifest document) of an exported directory, with every digest verified and ``pin`` compared."""
    manifest = _strict_load(os.path.join(directory, "manifest.json"))
    plan = _strict_load(os.path.join(directory, "plan.json"))
    if manifest.get("schema") != MANIFEST_SCHEMA:
        raise TilefishManifestError(f"{directory}/manifest.json: schema {manifest.get('schema')!r}, expected {MANIFEST_SCHEMA!r}")
    if plan.get("schema") != PLAN_SCHEMA:
        raise TilefishManifestError(f"{directory}/plan.json: schema {plan.get('schema')!r}, expected {PLAN_SCHEMA!r}")
    body = {k: v for k, v in manifest.items() if k != "manifest_digest"}
    if digest("tilefish.manifest-digest.v1", body) != manifest.get("manifest_digest"):
        raise TilefishManifestError(f"{directory}/manifest.json does not match its own digest: the file was changed after the export")
    body = {k: v for k, v in plan.items() if k != "plan_digest"}
    if digest("tilefish.plan-digest.v1", body) != plan.get("plan_digest"):
        raise TilefishManifestError(f"{directory}/plan.json does not match its own digest: the file was changed after the export")
    if plan.get("manifest_digest") != manifest["manifest_digest"]:
        raise TilefishManifestError(f"{directory}: plan.json was made for another manifest")
    if pin is not None and pin != plan["plan_digest"]:
        raise TilefishManifestError(f"{directory}: the plan's digest is {plan['plan_digest']}, the host pins {pin}")
    for key in ("buffers", "steps", "buckets", "arena_alignment"):
        if key not in plan:
            raise TilefishManifestError(f"{directory}/plan.json: key {key!r} is missing")
    return plan, manifest
