"""Declarations: ``@kernel`` (a traced body matched to a hand-written kernel), ``@library`` (an opaque typed operator: the
block-scaled gemm) and ``@graph`` (a model step over them).

Argument meaning, the objects returned (``KernelOp`` / ``LibraryOp`` / ``GraphOp`` with ``.name .signature .graph``) and the
call type-checking follow the reference (python/src/tilefish/decorators.py:184-193, :241-390, :396-741;
python/src/tilefish/signature.py:234, :797-1010): rank, dtype (BlockScaled formats must match exactly), contiguity and
dimensions are unified at every call, an ``InOut`` argument is consumed by the call. Annotations are evaluated at
declaration (no ``from __future__ import annotations`` in the declaring module).
"""

from __future__ import annotations

import inspect
from typing import Any, Dict, List, Optional, Tuple

from . import trace as T
from .dims import Dim, DimExpr, as_expr, divisible, simplify, symbols
from .dtypes import DType, same_format
from .errors import TilefishDeclarationError, TilefishTypeError
from .ir import Graph, Scalar, Value
from .types import ConstType, Marked, TensorType


class Param:
    __slots__ = ("name", "type", "access", "is_const", "const_dtype", "default", "dim")

    def __init__(self, name, type_=None, access="in", is_const=False, const_dtype=None, default=None):
        self.name, self.type, self.access = name, type_, access
        self.is_const, self.const_dtype, self.default = is_const, const_dtype, default
        self.dim = None  # an extern stub's runtime dimension parameter (`n_elem: n`): derived from the tensors at a call

    def __repr__(self) -> str:
        if self.is_const:
            return f"{self.name}: const[{self.const_dtype}] = {self.default!r}" if self.const_dtype is not None else f"{self.name}: const = {self.default!r}"
        if self.dim is not None:
            return f"{self.name}: {self.dim}"
        t = repr(self.type)
        if self.access == "inout":
            t = f"InOut[{t}]"
        elif self.access == "out":
            t = f"Out[{t}]"
        return f"{self.name}: {t}"


class Signature:
    def __init__(self, params: List[Param], returns: Tuple[TensorType, ...]) -> None:
        self.params = tuple(params)
        self.returns = tuple(returns)

    @property
    def tensors(self) -> Tuple[Param, ...]:
        return tuple(p for p in self.params if not p.is_const and p.dim is None)

    @property
    def consts(self) -> Tuple[Param, ...]:
        return tuple(p for p in self.params if p.is_const)

    def __repr__(self) -> str:
        rets = ", ".join(repr(r) for r in self.returns)
        if len(self.returns) != 1:
            rets = f"({rets})"
        return f"({', '.join(repr(p) for p in self.params)}) -> {rets}"


def parse_signature(fn, what: str) -> Signature:
    sig = inspect.signature(fn)
    params = []
    for name, p in sig.parameters.items():
        ann = p.annotation
        if isinstance(ann, str):
            raise TilefishDeclarationError(f"{what} '{fn.__name__}': annotations must be evaluated at declaration; remove "
                                           "`from __future__ import annotations` from the declaring module")
        if p.kind in (inspect.Parameter.VAR_POSITIONAL, inspect.Parameter.VAR_KEYWORD):
            raise TilefishDeclarationError(f"{what} '{fn.__name__}': *args/**kwargs are not allowed: every parameter is declared with its type")
        if what == "extern" and _extern_scalar(fn, name, p, params):
            continue
        if isinstance(ann, TensorType):
            params.append(Param(name, ann, "in"))
        elif isinstance(ann, Marked):
            params.append(Param(name, ann.type, ann.mode))
        elif isinstance(ann, ConstType):
            if p.kind is not inspect.Parameter.KEYWORD_ONLY or p.default is inspect.Parameter.empty:
                raise TilefishDeclarationError(f"{what} '{fn.__name__}': const parameter '{name}' must be keyword-only with a default")
            if ann.dtype is None:
                raise TilefishDeclarationError(f"{what} '{fn.__name__}': const parameter '{name}' needs a dtype (const[f32])")
            params.append(Param(name, None, "in", True, ann.dtype, p.default))
        elif ann is inspect.Parameter.empty:
            raise TilefishDeclarationError(f"{what} '{fn.__name__}': parameter '{name}' needs an annotation: Tensor[...], InOut[...], Out[...] or const[...]")
        else:
            raise TilefishDeclarationError(f"{what} '{fn.__name__}': parameter '{name}' has the unsupported annotation {ann!r}; a parameter is "
                                           "Tensor[...], InOut[...], Out[...] or const[...]")
    ret = sig.return_annotation
    if ret is inspect.Signature.empty or ret is None:
        returns: Tuple[TensorType, ...] = ()
    elif isinstance(ret, TensorType):
        returns = (ret,)
    elif isinstance(ret, tuple) and all(isinstance(r, TensorType) for r in ret):
        returns = tuple(ret)
    else:
        raise TilefishDeclarationError(f"{what} '{fn.__name__}': the return annotation must be a tensor type or a tuple of them")
    return Signature(params, returns)


def _extern_scalar(fn, name: str, p, params: List[Param]) -> bool:
    """The scalar parameters only an extern stub has: a runtime dimension (``n_elem: n``, derived from the tensors at a call) and a
    constexpr (``BLOCK: const = 1024``, typed or not, positional, fixed by the declaration). Appends it and returns True."""
    ann = p.annotation
    if isinstance(ann, (Dim, DimExpr)):
        e = as_expr(ann)
        if e.is_static:
            raise TilefishDeclarationError(f"extern '{fn.__name__}': parameter '{name}' is annotated with the static dimension {ann}; a size known at "
                                           f"declaration is a constexpr: write `{name}: const = {ann}`")
        q = Param(name, None, "in")
        q.dim = ann
        params.append(q)
        return True
    if isinstance(ann, ConstType):
        if p.default is inspect.Parameter.empty:
            raise TilefishDeclarationError(f"extern '{fn.__name__}': constexpr '{name}' needs a default: the value compiled into the binary")
        params.append(Param(name, None, "in", True, ann.dtype, p.default))
        return True
    return False


# ---- call type-checking: unify the callee's dimensions with the arguments' -------------------------------------------
def _require_divisible(callee: str, pname: str, d: Dim, axis: int, a) -> None:
    """The callee's ``d`` (declared ``divisible_by``) is bound to the caller's size ``a``: proven by the declarations, or a static
    violation (an error), or, for a symbolic size, a requirement recorded on the graph being traced (once per size and divisor)."""
    from .ir import Requirement
    from .trace import active as current_context

    n = d.divisible_by
    ctx = current_context()
    known = {r.dim: r.divisor for r in ctx.requirements if hasattr(r, "divisor")} if ctx is not None else {}
    if divisible(a, n, known):
        return
    if a.is_static:
        raise TilefishTypeError(f"{callee}: argument '{pname}': {d} requires divisible_by={n} but dimension {axis} is {a.offset}")
    if ctx is None:
        raise TilefishTypeError(f"{callee}: argument '{pname}' binds {d} to {simplify(a)}, which is not provably divisible by {n}")
    ctx.requirements.append(Requirement(a, n, f"{callee}: argument '{pname}'"))


def _require_bucket(callee: str, pname: str, d: Dim, axis: int, a, actual) -> None:
    """The callee's bucketed ``d`` is bound to the caller's size: one of the buckets (static), a bucketed dimension whose buckets all
    are the callee's, or a requirement recorded on the graph; a static miss and disjoint bucket sets are errors."""
    from .ir import BucketRequirement
    from .trace import active as current_context

    want = list(d.buckets)
    if a.is_static:
        if a.offset not in d.buckets:
            raise TilefishTypeError(f"{callee}: argument '{pname}': {d} is bucketed over {want} but dimension {axis} is {a.offset}")
        return
    have = actual.buckets if isinstance(actual, Dim) else None
    if have is not None:
        if set(have) <= set(want):
            return
        if not set(have) & set(want):
            raise TilefishTypeError(f"{callee}: argument '{pname}': {d} is bucketed over {want} but {actual} has buckets {list(have)} (no bucket in common)")
    ctx = current_context()
    if ctx is None:
        raise TilefishTypeError(f"{callee}: argument '{pname}' binds the bucketed {d} to {actual}, which is not known to be one of {want}")
    req = BucketRequirement(a, want, f"{callee}: argument '{pname}'")
    if req not in ctx.requirements:
        ctx.requirements.append(req)


def _unify(callee: str, pname: str, formal, actual, env: Dict[Dim, Any], axis: int = 0, arg_type=None, bound_by: Optional[Dict[Dim, str]] = None) -> None:
    """Binds the callee's dimensions in ``formal`` to the caller's size ``actual`` (axis ``axis`` of argument ``pname``)."""
    where = f"{callee}: argument '{pname}'" + (f" ({arg_type!r})" if arg_type is not None else "")
    f = as_expr(formal)
    if f.is_static:
        if as_expr(actual) != f:
            need = f"{formal} = {f.offset}" if isinstance(formal, Dim) else str(f.offset)
            raise TilefishTypeError(f"{where}: dimension {axis} is {actual}, but the signature requires {need}")
        return
    if f.offset == 0 and len(f.terms) == 1 and isinstance(f.terms[0][0], Dim):
        d, coef = f.terms[0]
        a = as_expr(actual)
        if coef != 1:
            if not (a.offset % coef == 0 and all(c % coef == 0 for _, c in a.terms)):
                raise TilefishTypeError(f"{where}: dimension {axis} is {actual}, which cannot match {formal}")
            from .dims import DimExpr

            a = DimExpr({k: c // coef for k, c in a.terms}, a.offset // coef)
        if d in env:
            if as_expr(env[d]) != a:
                by = f" ({d} was bound to {env[d]} by argument '{bound_by[d]}')" if bound_by and d in bound_by else ""
                raise TilefishTypeError(f"{where}: dimension {axis} is {actual}, but the signature requires {d} = {env[d]}{by}")
        else:
            if d.divisible_by:
                _require_divisible(callee, pname, d, axis, a)
            if d.buckets is not None and coef == 1:
                _require_bucket(callee, pname, d, axis, a, actual)
            env[d] = actual if coef == 1 else simplify(a)
            if bound_by is not None:
                bound_by[d] = pname
        return
    if as_expr(actual) != f:
        raise TilefishTypeError(f"{where}: dimension {axis} is {actual}, which cannot match {formal}")


def _substitute(x, env: Dict[Dim, Any]):
    if isinstance(x, Dim):
        return env.get(x, x) if not x.is_static else x
    e = as_expr(x)
    total = as_expr(e.offset)
    for a, c in e.terms:
        if isinstance(a, Dim) and a in env:
            total = total + as_expr(env[a]) * c
        else:
            from .dims import DimExpr

            total = total + DimExpr({a: c}, 0)
    return simplify(total)


def check_call(op: "Op", args: Tuple[Any, ...], kwargs: Dict[str, Any]) -> Tuple[List[Value], Dict[Dim, Any], Tuple[TensorType, ...], Dict[str, Any]]:
    sig = op.signature
    tensors = sig.tensors
    if len(args) > len(tensors):
        raise TilefishTypeError(f"{op.name}: takes {len(tensors)} tensor arguments, {len(args)} were given")
    bound: Dict[str, Any] = {p.name: a for p, a in zip(tensors, args)}
    known = {p.name for p in sig.params}
    for k, v in kwargs.items():
        if k in bound:
            raise TilefishTypeError(f"{op.name}: argument '{k}' given twice")
        if k not in known:
            raise TilefishTypeError(f"{op.name}: unexpected keyword argument '{k}'")
        bound[k] = v
    env: Dict[Dim, Any] = {}
    bound_by: Dict[Dim, str] = {}
    values = []
    for p in tensors:
        if p.access == "out" and p.name not in bound:
            continue
        if p.name not in bound:
            raise TilefishTypeError(f"{op.name}: missing a required argument: '{p.name}'")
        v = bound[p.name]
        if not isinstance(v, Value):
            raise TilefishTypeError(f"{op.name}: argument '{p.name}' must be a traced tensor of type {p.type!r}, got {type(v).__name__}")
        if v.consumed:
            raise TilefishTypeError(f"{op.name}: argument '{p.name}' ({v.ref}) was consumed by an earlier in-place call and cannot be read again")
        if v.type.rank != p.type.rank:
            raise TilefishTypeError(f"{op.name}: argument '{p.name}': expected rank {p.type.rank} ({p.type!r}), got rank {v.type.rank} ({v.type!r})")
        if not same_format(v.type.dtype, p.type.dtype, p.type.rank):
            raise TilefishTypeError(f"{op.name}: argument '{p.name}': expected dtype {p.type.dtype}, got {v.type.dtype}")
        if p.type.contiguous and not v.type.contiguous:
            raise TilefishTypeError(f"{op.name}: argument '{p.name}' is a strided view ({v.type!r}); the operator takes a contiguous tensor")
        for axis, (formal, actual) in enumerate(zip(p.type.shape, v.type.shape)):
            _unify(op.name, p.name, formal, actual, env, axis, v.type, bound_by)
        values.append(v)
    consts = {p.name: (op.check_const(p, bound[p.name]) if p.name in bound else p.default) for p in sig.consts}
    # writing in place to a read-only input of the graph being traced would change the caller's tensor behind its back
    for p, v in zip(tensors, values):
        if p.access == "inout" and getattr(v, "is_param", False) and v.access == "in":
            raise TilefishTypeError(f"{op.name}: argument '{p.name}' is written in place but '{v.name}' is a read-only input; declare it InOut[...] "
                                    "in the graph's signature")
    written = [v for p, v in zip(tensors, values) if p.access != "in"]
    if len({id(v) for v in written}) != len(written) or any(sum(1 for u in values if u is w) > 1 for w in written):
        raise TilefishTypeError(f"{op.name}: a written argument is passed more than once (aliasing)")
    rets = tuple(TensorType(tuple(_substitute(s, env) for s in r.shape), r.dtype, r.contiguous) for r in sig.returns)
    # an Out parameter the call does not pass is a result of the call: fresh storage, after the declared results, in declaration order
    rets += tuple(TensorType(tuple(_substitute(s, env) for s in p.type.shape), p.type.dtype, p.type.contiguous)
                  for p in tensors if p.access == "out" and p.name not in bound)
    return values, env, rets, consts


def _const_argument(op: "Op", p: Param, value):
    """A const argument given at a call: a python number, or a const parameter of the declaration being traced (passed through with the
    value it has there), as a value of the const's dtype."""
    if isinstance(value, (Scalar, T.Const)):
        value = value.value
    dt = p.const_dtype
    ok = isinstance(value, (int, float)) and not isinstance(value, bool)
    if dt is not None and dt.is_int:
        if not ok or isinstance(value, float):
            raise TilefishTypeError(f"{op.name}: argument '{p.name}' is const[{dt}] and needs an int, got {value!r}")
        return int(value)
    if not ok:
        raise TilefishTypeError(f"{op.name}: argument '{p.name}' is const[{dt}] and needs a number, got {value!r}")
    return float(value) if dt is None or dt.is_float else value


def _op_by_name(module: str, qualname: str):
    import importlib

    obj = importlib.import_module(module)
    for part in qualname.split("."):
        obj = getattr(obj, part)
    return obj


class Op:
    kind = "op"

    # a declared operator is a module-level object, like a function: copies are the object itself, pickles name it
    def __copy__(self):
        return self

    def __deepcopy__(self, memo):
        return self

    def __reduce__(self):
        return (_op_by_name, (self.fn.__module__, self.fn.__qualname__))

    def __init__(self, fn, name: Optional[str], signature: Signature) -> None:
        self.fn = fn
        self.name = name or fn.__name__
        self.signature = signature
        self.__doc__ = fn.__doc__
        self.__name__ = fn.__name__

    def __call__(self, *args, **kwargs):
        ctx = T.active()
        if ctx is None or not any(isinstance(a, Value) for a in list(args) + list(kwargs.values())):
            if ctx is None and not any(hasattr(a, "data_ptr") or hasattr(a, "codes") for a in list(args) + list(kwargs.values())):
                raise TilefishTypeError(f"{self.name}: an operator can only be called inside a graph or kernel body (tilefish.run executes one on tensors)")
            if ctx is not None:  # inside a trace every tensor argument is a traced value: let the call checker name the offender
                check_call(self, args, kwargs)
            from . import runtime

            return runtime.run(self, *args, **kwargs)
        # a kernel body may call a declared operator too (the call is traced as a node); such a kernel matches none of this backend's
        # hand-written kernels, so running it is refused by the lowering, not here
        values, _, rets, consts = check_call(self, args, kwargs)
        values = [ctx.latest(v) for v in values]  # a tensor an earlier in-place call updated is read at its current version
        attrs = self._call_attrs()
        # the call node as the reference prints it (python/src/tilefish/ir.py:133-206): after the declared results one output per InOut
        # parameter (the version of the tensor the call leaves behind), the consts with the values this call gives them, the names of the InOut parameters
        updated = [(p, v) for p, v in zip(self.signature.tensors, values) if p.access == "inout"]
        if consts:
            attrs["consts"] = consts
        if updated:
            attrs["inout"] = tuple(p.name for p, _ in updated)
        outs = ctx.emit(self.name, values, tuple(rets) + tuple(v.type for _, v in updated), attrs)
        ctx.nodes[-1].callee = self
        for (p, v), new in zip(updated, outs[len(rets):]):
            v.consumed = False  # the updated tensor is read back through the same name by later calls of the graph
            ctx.versions[v] = new
            root = v
            while root.producer is not None and root.producer.callee is not None and root in root.producer.outputs:
                k = root.producer.outputs.index(root) - (len(root.producer.outputs) - len(root.producer.attrs.get("inout", ())))
                if k < 0:
                    break
                names = root.producer.attrs["inout"]
                src = [x for q, x in zip(root.producer.callee.signature.tensors, root.producer.inputs) if q.name == names[k]]
                root = src[0]
            if root.is_param and root.access == "inout":
                ctx.finals[root.name] = new
        outs = outs[:len(rets)]
        if not outs:
            return None
        return outs[0] if len(outs) == 1 else outs

    def _call_attrs(self) -> Dict[str, Any]:
        return {"kind": self.kind}

    def check_const(self, p: Param, value):
        """A const argument given at a call, as a value of the const's dtype."""
        return _const_argument(self, p, value)

    def __repr__(self) -> str:
        return f"<{type(self).__name__} {self.name}{self.signature!r}>"


class LibraryOp(Op):
    """A typed operator with an opaque body. ``acc`` is the accumulator dtype; ``impl`` names the implementation, and is
    filled in with this backend's ("sm100.gemm_blockscaled") when the operands are block-scaled."""

    kind = "library"

    def __init__(self, fn, name, signature, acc: Optional[DType], impl: Optional[str]) -> None:
        super().__init__(fn, name, signature)
        self.acc = acc
        self.impl = impl

    def _call_attrs(self):
        return {"kind": "library", "acc": self.acc}


class KernelOp(Op):
    kind = "kernel"

    def __init__(self, fn, name, signature, graph: Graph, **options) -> None:
        super().__init__(fn, name, signature)
        self.graph = graph
        self.options = options


class GraphOp(Op):
    kind = "graph"

    def __init__(self, fn, name, signature, graph: Graph, param_roles: Dict[str, str]) -> None:
        super().__init__(fn, name, signature)
        self.graph = graph
        self.param_roles = param_roles

    @property
    def output_names(self) -> Tuple[str, ...]:
        return tuple(f"out{i}" for i in range(len(self.graph.outputs)))


def _trace(fn, kind: str, name: str, sig: Signature) -> Tuple[Graph, Tuple[TensorType, ...]]:
    with T.TraceContext(kind, name) as ctx:
        inputs = []
        call_args = []
        kw = {}
        for p in sig.params:
            if p.is_const:
                kw[p.name] = Scalar(p.default, p.const_dtype, p.name)
                continue
            v = Value(p.type, f"%{p.name}", ctx, is_param=True, access=p.access, name=p.name)
            inputs.append(v)
            call_args.append(v)
        result = fn(*call_args, **kw)
        if result is None:
            outs: List[Value] = []
        elif isinstance(result, Value):
            outs = [result]
        elif isinstance(result, (tuple, list)) and all(isinstance(r, Value) for r in result):
            outs = list(result)
        else:
            raise TilefishTypeError(f"{kind} '{name}': the body must return a traced tensor (or a tuple of them, or nothing), got {type(result).__name__}")
        for o in outs:
            if o.is_param and o.access == "out":
                raise TilefishTypeError(f"{kind} '{name}': cannot return Out parameter '{o.name}': an Out parameter is already a result of the operator")
        for p, v in zip(sig.tensors, inputs):
            if p.access == "out" and p.name not in ctx.finals:
                raise TilefishDeclarationError(f"{kind} '{name}': Out parameter '{p.name}' is never written")
            if p.access == "inout" and kind == "kernel" and p.name not in ctx.finals:
                raise TilefishDeclarationError(f"{kind} '{name}': InOut parameter '{p.name}' is never written")
        if sig.returns and len(sig.returns) != len(outs):
            raise TilefishTypeError(f"{kind} '{name}': the signature declares {len(sig.returns)} return value(s) but the body returns {len(outs)}")
        for i, o in enumerate(outs):
            if sig.returns and sig.returns[i] != o.type:
                raise TilefishTypeError(f"{kind} '{name}': return value {i} has type {o.type!r} but the declaration says {sig.returns[i]!r}")
            if o.is_param:
                raise TilefishDeclarationError(f"{kind} '{name}': a parameter cannot be returned as is")
        consts = [(p.name, p.const_dtype, p.default) for p in sig.consts]
        graph = Graph(kind, name, inputs, consts, ctx.nodes, outs, ctx.finals, tuple(ctx.requirements))
    return graph, tuple(o.type for o in outs)


def kernel(fn=None, *, name: Optional[str] = None, num_warps: Optional[int] = None, fp_fusion: bool = True, math: str = "fast", **ignored):
    """``@tilefish.kernel``: traces the body. The body must match one of the hand-written sm_100a kernels when it is run."""

    def wrap(f):
        sig = parse_signature(f, "kernel")
        graph, rets = _trace(f, "kernel", name or f.__name__, sig)
        sig = Signature(list(sig.params), rets)
        return KernelOp(f, name, sig, graph, num_warps=num_warps, fp_fusion=fp_fusion, math=math)

    return wrap(fn) if callable(fn) else wrap


def _results_are_determined(sig: Signature, what: str, name: str) -> None:
    """An opaque operator's results may only mention dimensions that a call can read off its input tensors."""
    known = set()
    for p in sig.tensors:
        if p.access != "out":
            for sz in p.type.shape:
                known.update(d.name for d in symbols(sz))
    results = [(f"return value {i}", r) for i, r in enumerate(sig.returns)] + [(f"Out parameter '{p.name}'", p.type) for p in sig.tensors if p.access == "out"]
    for label, t in results:
        free = sorted({d.name for sz in t.shape for d in symbols(sz) if d.is_dynamic} - known)
        if free:
            raise TilefishDeclarationError(f"{what} '{name}': {label} mentions dimension(s) {', '.join(free)} that no input tensor determines")


def library(name=None, *, acc: Optional[DType] = None, impl: Optional[str] = None, **ignored):
    """``@tilefish.library("gemm", acc=f32)``: a signature with an opaque body (``...``)."""
    if callable(name):
        raise TilefishDeclarationError("@library takes arguments: @library('gemm', acc=f32)")

    def wrap(f):
        sig = parse_signature(f, "library")
        if not sig.returns and not any(p.access != "in" for p in sig.tensors):
            raise TilefishDeclarationError(f"library '{f.__name__}': produces nothing: declare a return type (-> Tensor[...]) or an Out[...] / InOut[...] parameter")
        _results_are_determined(sig, "library", f.__name__)
        return LibraryOp(f, name, sig, acc, impl)

    return wrap


class ExternOp(Op):
    """A kernel that lives outside this package (``@tilefish.extern(triton="module:function", grid=...)``). It can be declared, called
    from graph bodies and type-checked like any operator; this backend has no Triton and generates no code, so a graph that contains
    one is refused when it is lowered."""

    kind = "extern"

    def __init__(self, fn, name, signature, triton: str, grid, options: Dict[str, Any]) -> None:
        super().__init__(fn, name, signature)
        self.triton, self.grid, self.options = triton, grid, options

    def _call_attrs(self):
        return {"kind": "extern", "triton": self.triton}

    def check_const(self, p: Param, value):
        if isinstance(value, (Scalar, T.Const)):
            value = value.value
        if value != p.default:
            raise TilefishTypeError(f"{self.name}: constexpr '{p.name}' is fixed to {p.default} by the extern declaration (it is compiled into the "
                                    f"binary) and cannot be changed to {value!r} at a call")
        return value


def extern(*, triton: Optional[str] = None, grid=None, num_warps: int = 4, name: Optional[str] = None, **options):
    """``@tilefish.extern(triton="module:function", grid=lambda n: (cdiv(n, 1024),))``: the declaration of a kernel written elsewhere.
    The stub lists the kernel's parameters: tensors (``Out[...]`` ones are the results of a call), runtime dimensions (``n_elem: n``)
    and constexprs (``BLOCK: const = 1024``); it returns nothing. Declaring and tracing work here; running does not (no Triton)."""
    if callable(triton) and getattr(triton, "__module__", None) and getattr(triton, "__name__", None):
        triton = f"{triton.__module__}:{triton.__name__}"  # the kernel itself: recorded by reference, never called here
    if not isinstance(triton, str) or triton.count(":") != 1 or not all(triton.split(":")):
        raise TilefishDeclarationError(f"extern: triton= names the kernel as 'module:function', got {triton!r}")
    if not isinstance(num_warps, int) or num_warps <= 0 or num_warps & (num_warps - 1):
        raise TilefishDeclarationError(f"extern: num_warps must be a power of two, got {num_warps!r}")

    def wrap(f):
        sig = parse_signature(f, "extern")
        if sig.returns:
            raise TilefishDeclarationError(f"extern '{f.__name__}': a kernel returns nothing: declare its results as Out[...] parameters")
        dims = set()
        for p in sig.params:
            for sz in (p.type.shape if p.type is not None else ([p.dim] if p.dim is not None else [])):
                dims.update(d.name for d in symbols(sz))
        if callable(grid):
            for q in inspect.signature(grid).parameters:
                if q not in dims:
                    raise TilefishDeclarationError(f"extern '{f.__name__}': grid parameter '{q}' is not a dimension of the signature ({', '.join(sorted(dims))})")
        _results_are_determined(sig, "extern", f.__name__)
        return ExternOp(f, name, sig, triton, grid, dict(options, num_warps=num_warps))

    return wrap


def graph(fn=None, *, name: Optional[str] = None, inputs: Tuple[str, ...] = (), weights: Tuple[str, ...] = (), **ignored):
    """``@tilefish.graph``: a model step; ``inputs=`` / ``weights=`` label read-only tensor parameters."""

    def wrap(f):
        sig = parse_signature(f, "graph")
        g, rets = _trace(f, "graph", name or f.__name__, sig)
        sig2 = Signature(list(sig.params), rets)
        roles = {}
        for p in sig2.tensors:
            if p.access != "in":
                roles[p.name] = p.access
            elif p.name in weights:
                roles[p.name] = "weight"
            elif p.name in inputs or not (inputs or weights):
                roles[p.name] = "input" if not p.type.is_blockscaled else "weight"
            else:
                roles[p.name] = "input"
        for n in tuple(inputs) + tuple(weights):
            if n not in {p.name for p in sig2.tensors}:
                raise TilefishDeclarationError(f"graph '{f.__name__}': '{n}' is not a tensor parameter")
        return GraphOp(f, name, sig2, g, roles)

    return wrap(fn) if callable(fn) else wrap
