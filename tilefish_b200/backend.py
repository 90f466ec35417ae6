"""The sm_100a backend: which hand-written kernel runs a declaration, and how a graph becomes an ordered list of steps.

This replaces the reference's Triton lowering (python/src/tilefish/lower.py) and cuBLASLt pin (python/src/tilefish/_library.py)
for the operators of the quantized-inference path. Nothing is generated: a ``@kernel`` body is compared, structurally,
with the bodies the CUDA kernels implement (``TEMPLATES``); a body that matches none is refused with
``TilefishLoweringError`` (there is no fallback). A ``@graph`` is walked node by node into steps, the way the reference
plans a graph (python/src/tilefish/_plan.py:1209), with three fusions: the SiLU-gate arithmetic between two gemms becomes
the first gemm's epilogue (the reference folds arithmetic chains into library epilogues the same way,
python/src/tilefish/_fusion.py:1430-1530: every intermediate used once and not returned), the quantization of a gemm's bf16
activation is done by the kernel that produced it when that is the rmsnorm kernel (MX formats), and for nvfp4 the producer
also reduces the amax the quantizer needs.
"""

from typing import Any, Dict, List, Optional, Tuple

from .decorators import ExternOp, GraphOp, KernelOp, LibraryOp
from .dims import Dim, as_expr, evaluate
from .dtypes import BlockScaled, bf16, f32
from .errors import TilefishLoweringError, TilefishPlanError
from .ir import Graph, Node, Scalar, Value
from .types import InOut, Tensor, const

GEMM_IMPL = "sm100.gemm_blockscaled"


# ---- structural comparison of kernel bodies ---------------------------------------------------------------------------
def canonical(g: Graph) -> Tuple:
    """A name-free description of a kernel body: parameters (dtype, rank, access), nodes (op, operand references, attributes)."""
    pos = {v: i for i, v in enumerate(g.inputs)}
    where: Dict[Value, Tuple] = {}
    nodes = []
    for ni, n in enumerate(g.nodes):
        ins = []
        for x in n.inputs:
            if isinstance(x, Value):
                ins.append(("p", pos[x]) if x in pos else where[x])
            elif isinstance(x, Scalar):
                ins.append(("c", x.name is not None, str(x.dtype)) if x.name else ("s", float(x.value), str(x.dtype)))
        attrs = []
        for k, v in n.attrs.items():
            if k == "target":
                v = next(i for i, p in enumerate(g.inputs) if p.name == v)
            attrs.append((k, str(v)))
        nodes.append((n.op, tuple(ins), tuple(attrs)))
        for oi, o in enumerate(n.outputs):
            where[o] = ("n", ni, oi)
    params = tuple((str(v.type.dtype), v.type.rank, v.access) for v in g.inputs)
    outs = tuple(where[o] for o in g.outputs)
    return (params, tuple(nodes), outs, tuple(str(c[1]) for c in g.consts))


def _templates():
    from . import trace as tf
    from .decorators import kernel

    m, d = Dim("M"), Dim("D")

    @kernel
    def residual_add_rmsnorm(x: Tensor[m, d, bf16], residual: InOut[Tensor[m, d, f32]], w: Tensor[d, bf16], *, eps: const[f32] = 1e-6) -> Tensor[m, d, bf16]:
        r = residual + x.to(f32)
        residual[...] = r
        rstd = tf.rsqrt(tf.mean(r * r, axis=-1, keepdims=True) + eps)
        return (r * rstd * w.to(f32)).to(bf16)

    @kernel
    def silu_gate(g: Tensor[m, d, bf16], u: Tensor[m, d, bf16]) -> Tensor[m, d, bf16]:
        return (tf.silu(g.to(f32)) * u.to(f32)).to(bf16)

    return {"residual_add_rmsnorm": canonical(residual_add_rmsnorm.graph), "silu_gate": canonical(silu_gate.graph)}


TEMPLATES: Dict[str, Tuple] = {}


def match_kernel(op: KernelOp) -> str:
    """The name of the CUDA kernel that implements ``op``'s body ("residual_add_rmsnorm" or "silu_gate")."""
    if not TEMPLATES:
        TEMPLATES.update(_templates())
    want = canonical(op.graph)
    for name, tmpl in TEMPLATES.items():
        if tmpl == want:
            return name
    raise TilefishLoweringError(
        f"kernel '{op.name}': its body matches none of the hand-written sm_100a kernels ({', '.join(TEMPLATES)}); this backend generates no "
        "code and has no fallback", rule="no-template")


# ---- graph -> steps -------------------------------------------------------------------------------------------------------
class Step:
    """One launch. ``kind`` is "kernel" or "library"; ``impl`` names the C entry point; ``args`` maps the entry's parameters to
    buffer names; ``attrs`` carries compile-time values (eps, format, epilogue)."""

    __slots__ = ("entry", "kind", "impl", "args", "attrs")

    def __init__(self, entry: str, kind: str, impl: str, args: Dict[str, str], attrs: Dict[str, Any]) -> None:
        self.entry, self.kind, self.impl, self.args, self.attrs = entry, kind, impl, args, attrs

    def doc(self) -> Dict[str, Any]:
        return {"entry": self.entry, "kind": self.kind, "impl": self.impl, "args": dict(self.args), "attrs": dict(self.attrs)}


class Buffer:
    __slots__ = ("name", "role", "type", "fmt")

    def __init__(self, name: str, role: str, type_, fmt: Optional[str] = None) -> None:
        self.name, self.role, self.type, self.fmt = name, role, type_, fmt


def _users(g: Graph) -> Dict[Value, List[Node]]:
    users: Dict[Value, List[Node]] = {}
    for n in g.nodes:
        for x in n.inputs:
            if isinstance(x, Value):
                users.setdefault(x, []).append(n)
    return users


def _match_silu_region(g: Graph, split: Node, users):
    """split(t) -> (g, u); cast(g) -> silu; cast(u); mul; cast -> bf16, every intermediate used once.
    Returns (final cast, [the region's nodes]) or None."""
    if len(split.outputs) != 2:
        return None
    go, uo = split.outputs

    def only(v):
        u = users.get(v, [])
        return u[0] if len(u) == 1 and v not in g.outputs else None

    cg, cu = only(go), only(uo)
    if not (cg and cu and cg.op == "cast" and cu.op == "cast" and cg.attrs["to"] is f32 and cu.attrs["to"] is f32):
        return None
    si = only(cg.outputs[0])
    if not (si and si.op == "silu"):
        return None
    mu = only(si.outputs[0])
    if not (mu and mu.op == "mul" and mu is only(cu.outputs[0]) and mu.inputs == (si.outputs[0], cu.outputs[0])):
        return None
    fin = only(mu.outputs[0])
    if not (fin and fin.op == "cast" and fin.attrs["to"] is bf16):
        return None
    if go.type.dtype is not bf16:
        return None
    return fin, [split, cg, si, cu, mu, fin]


def compile_graph(op: GraphOp, fuse: bool = True) -> Tuple[List[Buffer], List[Step]]:
    """Buffers (parameters, outputs, intermediates) and ordered steps of a graph, in symbolic sizes."""
    g = op.graph
    users = _users(g)
    buffers: List[Buffer] = []
    name_of: Dict[Value, str] = {}
    for v in g.inputs:
        fmt = v.type.dtype.format_name if isinstance(v.type.dtype, BlockScaled) else None
        if isinstance(v.type.dtype, BlockScaled) and fmt is None:
            raise TilefishPlanError(f"graph '{g.name}': parameter '{v.name}' has format {v.type.dtype}, which this backend has no kernels for")
        buffers.append(Buffer(v.name, op.param_roles.get(v.name, "input"), v.type, fmt))
        name_of[v] = v.name
    out_names = {o: f"out{i}" for i, o in enumerate(g.outputs)}
    counter = [0]

    def new_buffer(v: Value, fmt: Optional[str] = None, type_=None) -> str:
        if v in out_names and fmt is None:
            nm, role = out_names[v], "output"
        else:
            nm, role = f"t{counter[0]}", "intermediate"
            counter[0] += 1
        buffers.append(Buffer(nm, role, type_ or v.type, fmt))
        return nm

    steps: List[Step] = []
    quantized: Dict[Tuple[Value, str], str] = {}  # (bf16 value, format) -> buffer holding its quantization
    producer_step: Dict[Value, Step] = {}
    skip: set = set()
    views: Dict[Value, Tuple[Value, int]] = {}  # a split output -> (source, part index)
    aux_needed = False
    amax_slots = [0]

    def quantized_operand(v: Value, fmt: str) -> str:
        nonlocal aux_needed
        key = (v, fmt)
        if key in quantized:
            return quantized[key]
        qtype = v.type
        nm = f"t{counter[0]}"
        counter[0] += 1
        buffers.append(Buffer(nm, "intermediate", qtype, fmt))
        src = producer_step.get(v)
        single_use = len(users.get(v, [])) == 1 and v not in g.outputs
        fusable = src is not None and "q" not in src.args and fmt != "nvfp4" and (
            src.impl == "tf_residual_add_rmsnorm" or (src.impl == "tf_gemm_blockscaled" and src.attrs["format"] == fmt and src.attrs["epilogue"] != "residual"))
        if fuse and fusable:
            src.args["q"] = nm
            src.attrs["q_format"] = fmt
            if single_use:  # nobody reads the bf16 copy: do not write it
                dropped = src.args.pop("out")
                buffers[:] = [b for b in buffers if b.name != dropped]
        else:
            attrs = {"format": fmt}
            args = {"x": name_of[v], "q": nm}
            if fmt == "nvfp4":
                aux_needed = True
                if fuse and src is not None and src.impl in ("tf_residual_add_rmsnorm", "tf_gemm_blockscaled") and "amax" not in src.args:
                    slot = amax_slots[0]
                    amax_slots[0] += 1
                    src.args["amax"] = f"aux[{slot}]"
                    args["amax"] = f"aux[{slot}]"
            steps.append(Step(f"quantize.{fmt}", "kernel", f"tf_quantize_{fmt}", args, attrs))
        quantized[key] = nm
        return nm

    for n in g.nodes:
        if n in skip:
            continue
        callee = n.callee
        if isinstance(callee, ExternOp):
            raise TilefishLoweringError(f"graph '{g.name}': '{callee.name}' is an extern kernel ({callee.triton}); this backend has no Triton and loads "
                                        "no foreign binaries: only the hand-written sm_100a kernels run", rule="no-extern")
        if isinstance(callee, KernelOp):
            impl = match_kernel(callee)
            params = callee.signature.tensors
            if impl == "residual_add_rmsnorm":
                args = {p.name if i > 2 else ("x", "residual", "w")[i]: name_of[v] for i, (p, v) in enumerate(zip(params, n.inputs))}
                args["out"] = new_buffer(n.outputs[0])
                st = Step(callee.name, "kernel", "tf_residual_add_rmsnorm", args, {"eps": float(n.attrs.get("consts", {}).get(callee.signature.consts[0].name, callee.signature.consts[0].default))})
            else:
                gv, uv = n.inputs
                args = {"gate": name_of[gv], "up": name_of[uv], "out": new_buffer(n.outputs[0])}
                st = Step(callee.name, "kernel", "tf_silu_gate", args, {})
            steps.append(st)
            name_of[n.outputs[0]] = args["out"]
            producer_step[n.outputs[0]] = st
            # the versions of the InOut tensors the call leaves behind live where the tensors do
            inout_names = n.attrs.get("inout", ())
            for new, pname in zip(n.outputs[len(n.outputs) - len(inout_names):], inout_names):
                src = next(v for p, v in zip(params, n.inputs) if p.name == pname)
                name_of[new] = name_of[src]
        elif isinstance(callee, LibraryOp):
            a, b = n.inputs
            if not isinstance(b.type.dtype, BlockScaled):
                raise TilefishPlanError(f"graph '{g.name}': {callee.name}({a.ref}, {b.ref}): this backend runs the gemm over BlockScaled weights only "
                                        f"(b is {b.type.dtype}); a bf16 gemm is the reference's cuBLASLt path, which is not part of it")
            fmt = b.type.dtype.format_name
            if callee.acc is not None and callee.acc is not f32:
                raise TilefishPlanError(f"graph '{g.name}': {callee.name} accumulates in {callee.acc}; the tensor-core kernel accumulates in f32")
            if isinstance(a.type.dtype, BlockScaled):
                a_name = name_of[a]
            else:
                a_name = quantized_operand(a, fmt)
            out_v = n.outputs[0]
            epilogue = "none"
            result_v = out_v
            u = users.get(out_v, [])
            if fuse and len(u) == 1 and u[0].op == "split" and out_v not in g.outputs and u[0].attrs["axis"] == out_v.type.rank - 1:
                region = _match_silu_region(g, u[0], users)
                half = as_expr(u[0].attrs["sizes"][0]).value
                if region is not None and half is not None and half % 128 == 0:
                    epilogue = "silu_gate"
                    result_v = region[0].outputs[0]
                    skip.update(region[1])
            args = {"a": a_name, "b": name_of[b], "out": new_buffer(result_v)}
            st = Step(callee.name, "library", "tf_gemm_blockscaled", args, {"format": fmt, "epilogue": epilogue, "impl": GEMM_IMPL})
            steps.append(st)
            name_of[result_v] = args["out"]
            producer_step[result_v] = st
        elif n.op == "split":
            for i, o in enumerate(n.outputs):
                views[o] = (n.inputs[0], i)
                name_of[o] = f"{name_of[n.inputs[0]]}[:, {i}]"
        elif n.op == "quantize":
            fmt = n.attrs["to"].format_name
            nm = quantized_operand(n.inputs[0], fmt)
            name_of[n.outputs[0]] = nm
        elif n.op == "cast" and isinstance(n.inputs[0], Value) and n.inputs[0] in views:
            # the unfused SiLU gate over the column halves of a tensor: cast(g), silu, cast(u), mul, cast as one kernel step
            src, idx = views[n.inputs[0]]
            split = n.inputs[0].producer
            region = _match_silu_region(g, split, users) if idx == 0 else None
            if region is None:
                raise TilefishPlanError(f"graph '{g.name}': the arithmetic on {n.inputs[0].ref} is not a launch of a declared operator and does not "
                                        "match the SiLU-gate pattern this backend has a kernel for")
            fin = region[0]
            go, uo = split.outputs
            args = {"gate": name_of[go], "up": name_of[uo], "out": new_buffer(fin.outputs[0])}
            st = Step("silu_gate", "kernel", "tf_silu_gate", args, {})
            steps.append(st)
            name_of[fin.outputs[0]] = args["out"]
            producer_step[fin.outputs[0]] = st
            skip.update(region[1])
        else:
            raise TilefishPlanError(f"graph '{g.name}': node `{n}` is not a launch of a declared operator, a view or a pattern this backend fuses")
    for o, nm in out_names.items():
        if name_of.get(o) != nm:
            raise TilefishPlanError(f"graph '{g.name}': returned value {o.ref} is a view or an input; a graph returns tensors its steps produce")
    if aux_needed:
        buffers.append(Buffer("aux", "intermediate", Tensor[8, f32]))
    return buffers, steps


def concrete_shape(shape, env: Dict[Dim, int]) -> Tuple[int, ...]:
    out = []
    for s in shape:
        v = evaluate(s, env)
        if v is None:
            raise TilefishPlanError(f"size {s} is not determined by the bound dimensions")
        out.append(int(v))
    return tuple(out)
