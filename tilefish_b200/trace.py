"""Tracing: running a kernel or graph body over typed ``Value`` proxies; every operation type-checks and appends a node.

Typing rules follow the reference's built-in ops (python/src/tilefish/ops.py:1-30, :535-600, :916-970): no implicit dtype
promotion, python scalars and ``const`` parameters adopt the tensor's dtype, math ops are f32-only, a cast is a rounding
point exactly when the target cannot represent every value of the source, ``split`` along a non-leading axis gives strided
views. One addition: ``x.to(<BlockScaled>)`` of a bf16 tensor is allowed (the reference refuses it, ops.py:556-559) and
traces to a ``quantize`` node, which this backend runs with its quantization kernels.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

from .dims import as_expr, divisible, exact_ratio, simplify
from .dtypes import BlockScaled, DType, f32
from .errors import TilefishAttributeError, TilefishTypeError
from .ir import Node, Scalar, Value
from .types import TensorType, broadcast_shapes

_ACTIVE: List["TraceContext"] = []


def active() -> Optional["TraceContext"]:
    return _ACTIVE[-1] if _ACTIVE else None


class TraceContext:
    def __init__(self, kind: str, name: str) -> None:
        self.kind, self.name = kind, name
        self.nodes: List[Node] = []
        self.counter = 0
        self.finals: Dict[str, Value] = {}
        self.consts: Dict[str, Scalar] = {}
        self.versions: Dict[Value, Value] = {}  # a value an in-place call updated -> the version the call produced
        self.requirements: List = []  # divisibility of symbolic sizes that calls rely on and the declarations do not prove

    def new_value(self, type, name: Optional[str] = None, access: str = "in", is_param: bool = False) -> Value:
        """A value of this trace that no node produced: a parameter (what the decorators create for every tensor argument)."""
        ref = f"%{name}" if name else f"%{self.counter}"
        if not name:
            self.counter += 1
        return Value(type, ref, self, is_param=is_param, access=access, name=name)

    def latest(self, v: Value) -> Value:
        """The current version of ``v``: what a later read of a tensor that an in-place call updated refers to."""
        while v in self.versions:
            v = self.versions[v]
        return v

    def __enter__(self):
        _ACTIVE.append(self)
        return self

    def __exit__(self, *exc):
        _ACTIVE.pop()

    def emit(self, op: str, inputs: Sequence[Any], out_types: Sequence[TensorType], attrs: Optional[Dict[str, Any]] = None) -> Tuple[Value, ...]:
        node = Node(op, tuple(inputs), dict(attrs or {}))
        outs = []
        for i, t in enumerate(out_types):
            outs.append(Value(t, f"%{self.counter}", self, producer=node, index=i))
            self.counter += 1
        node.outputs = tuple(outs)
        self.nodes.append(node)
        return node.outputs


def _ctx_of(v: Value) -> TraceContext:
    ctx = active()
    if ctx is None:
        return v._ctx  # a context driven by hand (TraceContext.new_value): the value knows its trace
    if v._ctx is not ctx:
        raise TilefishTypeError(f"{v.ref} is used outside the declaration that traced it")
    return ctx


def _require_computable(v: Value, op: str) -> None:
    if not getattr(v.type.dtype, "computable", False):
        raise TilefishTypeError(f"{op}: {v.ref} has dtype {v.type.dtype}, which is storage only; cast it first (.to(f32))")


class Const:
    """A ``const`` parameter as a traced body sees it (reference: python/src/tilefish/trace.py:178-203): it combines with tensors; an
    untyped one (``dtype`` None) adopts the dtype of the tensor it meets, a typed one must match it."""

    __slots__ = ("name", "value", "dtype")

    def __init__(self, name: str, value, dtype) -> None:
        self.name, self.value, self.dtype = name, value, dtype

    def __repr__(self) -> str:
        return f"Const({self.name}={self.value!r})"

    def _refuse(self, other):
        if isinstance(other, Value):
            return NotImplemented  # the tensor's reflected operator handles it
        raise TilefishTypeError(f"const parameter '{self.name}' can only be combined with a tensor value, got {type(other).__name__}")

    __add__ = __radd__ = __sub__ = __rsub__ = __mul__ = __rmul__ = __truediv__ = __rtruediv__ = _refuse


def _operand(x, like: Value, op: str):
    """A tensor operand as is; a python scalar or const adopts ``like``'s dtype."""
    if isinstance(x, Value):
        return x
    if isinstance(x, Const):
        if x.value is None:
            raise TilefishTypeError(f"{op}: const parameter '{x.name}' has no default value to trace with")
        if x.dtype is not None and x.dtype is not like.type.dtype:
            raise TilefishTypeError(f"{op}: const {x.name} is {x.dtype} but the tensor is {like.type.dtype}")
        return Scalar(x.value, like.type.dtype, x.name)
    if isinstance(x, Scalar):
        if x.dtype is not like.type.dtype:
            raise TilefishTypeError(f"{op}: const {x.name} is {x.dtype} but the tensor is {like.type.dtype}")
        return x
    if isinstance(x, (int, float)) and not isinstance(x, bool):
        return Scalar(x, like.type.dtype)
    raise TilefishTypeError(f"{op}: unsupported operand {x!r}")


def binary(op: str, a, b) -> Value:
    like = a if isinstance(a, Value) else b
    ctx = _ctx_of(like)
    a, b = _operand(a, like, op), _operand(b, like, op)
    for v in (a, b):
        if isinstance(v, Value):
            _require_computable(v, op)
    if isinstance(a, Value) and isinstance(b, Value):
        if a.type.dtype is not b.type.dtype:
            raise TilefishTypeError(f"{op}: {a.ref} is {a.type.dtype} but {b.ref} is {b.type.dtype}; there is no implicit promotion, cast one side")
        shape = broadcast_shapes(a.type.shape, b.type.shape, op)
    else:
        shape = like.type.shape
    return ctx.emit(op, (a, b), (TensorType(shape, like.type.dtype),))[0]


def cast(x: Value, dtype) -> Value:
    ctx = _ctx_of(x)
    src = x.type.dtype
    if isinstance(dtype, BlockScaled):
        if isinstance(src, BlockScaled) or src.name != "bf16":
            raise TilefishTypeError(f"cast: only a bf16 tensor can be quantized to {dtype}, {x.ref} is {src}")
        if dtype.format_name is None:
            raise TilefishTypeError(f"cast: this backend has no quantizer for {dtype} (mxfp8, mxfp4 and nvfp4 are implemented)")
        if dtype.normalized(x.type.rank).axis != x.type.rank - 1:
            raise TilefishTypeError(f"cast: {dtype} must block the last axis")
        return ctx.emit("quantize", (x,), (TensorType(x.type.shape, dtype),), {"to": dtype, "rounding": True})[0]
    if isinstance(src, BlockScaled):
        raise TilefishTypeError(f"cast: dequantizing {x.ref} ({src}) is not an operation of this backend; the gemm consumes block-scaled operands directly")
    if not isinstance(dtype, DType):
        raise TilefishTypeError(f"cast: expected a dtype, got {dtype!r}")
    rounding = src.is_narrowing_to(dtype)
    return ctx.emit("cast", (x,), (TensorType(x.type.shape, dtype),), {"to": dtype, "rounding": rounding})[0]


def unary_f32(op: str, x: Value) -> Value:
    ctx = _ctx_of(x)
    if x.type.dtype is not f32:
        raise TilefishTypeError(f"{op}: needs an f32 tensor, {x.ref} is {x.type.dtype}; cast first")
    return ctx.emit(op, (x,), (TensorType(x.type.shape, f32),))[0]


def reduce(op: str, x: Value, axis, keepdims: bool) -> Value:
    ctx = _ctx_of(x)
    _require_computable(x, op)
    axes = (axis,) if isinstance(axis, int) else tuple(axis)
    rank = x.type.rank
    norm = []
    for ax in axes:
        a = ax + rank if ax < 0 else ax
        if not 0 <= a < rank:
            raise TilefishTypeError(f"{op}: axis {ax} is out of range for {x.type!r}")
        norm.append(a)
    if keepdims:
        shape = tuple(1 if i in norm else s for i, s in enumerate(x.type.shape))
    else:
        shape = tuple(s for i, s in enumerate(x.type.shape) if i not in norm)
    return ctx.emit(op, (x,), (TensorType(shape, x.type.dtype),), {"axes": tuple(norm), "keepdims": bool(keepdims)})[0]


def split(x: Value, size, axis: int = -1) -> Tuple[Value, ...]:
    ctx = _ctx_of(x)
    rank = x.type.rank
    ax = axis + rank if axis < 0 else axis
    if not 0 <= ax < rank:
        raise TilefishTypeError(f"split: axis {axis} is out of range for {x.type!r}")
    total, part = as_expr(x.type.shape[ax]), as_expr(size)
    if part.is_static and part.offset <= 0:
        raise TilefishTypeError(f"split: the part size must be positive, got {size}")
    # the number of parts must be one integer for every binding of the dimensions: a static quotient, or a constant ratio (2*F into F)
    count = exact_ratio(total, part)
    if count is None or count <= 0:
        raise TilefishTypeError(f"split: {x.type.shape[ax]} is not a whole number of parts of {size}")
    size = simplify(size)
    shape = tuple(size if i == ax else s for i, s in enumerate(x.type.shape))
    if isinstance(x.type.dtype, BlockScaled):
        fmt = x.type.dtype.normalized(rank)
        if fmt.axis == ax and not divisible(part, fmt.block):
            raise TilefishTypeError(f"split: parts of {size} along the blocked axis are not whole blocks of {fmt.block}")
    leading = all(as_expr(s) == as_expr(1) for s in x.type.shape[:ax])
    t = TensorType(shape, x.type.dtype, contiguous=leading and x.type.contiguous)
    return ctx.emit("split", (x,), (t,) * count, {"axis": ax, "sizes": (size,) * count})


def store(target: Value, value: Value) -> None:
    ctx = _ctx_of(target)
    if not target.is_param or target.access not in ("inout", "out"):
        raise TilefishTypeError(f"{target.ref} is not an InOut or Out parameter: it cannot be stored to")
    if not isinstance(value, Value) or value.type.dtype is not target.type.dtype:
        raise TilefishTypeError(f"store to {target.name}: the value must be a {target.type.dtype} tensor")
    if tuple(as_expr(s) for s in value.type.shape) != tuple(as_expr(s) for s in target.type.shape):
        raise TilefishTypeError(f"store to {target.name}: shape {value.type!r} does not match {target.type!r}")
    (out,) = ctx.emit("store", (target, value), (target.type,), {"target": target.name})
    ctx.finals[target.name] = out


# ---- the methods of a traced value ------------------------------------------------------------------------------------
def _install() -> None:
    Value.to = lambda self, dtype: cast(self, dtype)
    Value.split = lambda self, size, axis=-1: split(self, size, axis)
    Value.__add__ = lambda self, o: binary("add", self, o)
    Value.__radd__ = lambda self, o: binary("add", o, self)
    Value.__sub__ = lambda self, o: binary("sub", self, o)
    Value.__rsub__ = lambda self, o: binary("sub", o, self)
    Value.__mul__ = lambda self, o: binary("mul", self, o)
    Value.__rmul__ = lambda self, o: binary("mul", o, self)
    Value.__truediv__ = lambda self, o: binary("div", self, o)

    def setitem(self, key, value):
        if key is not Ellipsis:
            raise TilefishTypeError("only whole-tensor stores are supported: write `x[...] = value`")
        store(self, value)

    Value.__setitem__ = setitem

    def missing(self, name):
        raise TilefishAttributeError(f"traced values have no attribute {name!r}")

    Value.__getattr__ = missing


_install()


# ---- public math ops ----------------------------------------------------------------------------------------------------
def silu(x: Value) -> Value:
    return unary_f32("silu", x)


def sqrt(x: Value) -> Value:
    return unary_f32("sqrt", x)


def gelu(x: Value) -> Value:
    return unary_f32("gelu", x)


def contiguous(x: Value) -> Value:
    """A dense copy of a strided view (the type's ``contiguous`` flag set); a contiguous tensor is returned as is."""
    if x.type.contiguous:
        return x
    return _ctx_of(x).emit("contiguous", (x,), (TensorType(x.type.shape, x.type.dtype, contiguous=True),))[0]


def rsqrt(x: Value) -> Value:
    return unary_f32("rsqrt", x)


def exp(x: Value) -> Value:
    return unary_f32("exp", x)


def mean(x: Value, axis=-1, keepdims: bool = False) -> Value:
    return reduce("mean", x, axis, keepdims)


def reduce_sum(x: Value, axis=-1, keepdims: bool = False) -> Value:
    return reduce("sum", x, axis, keepdims)


def reduce_max(x: Value, axis=-1, keepdims: bool = False) -> Value:
    return reduce("max", x, axis, keepdims)


# the reference's spellings (tilefish.sum / tilefish.max); kept out of `import *` because they would shadow the builtins
sum = reduce_sum  # noqa: A001
max = reduce_max  # noqa: A001
