"""Tracing: running a kernel or graph body over typed ``Value`` proxies; every operation type-checks and appends a node.

Typing rules follow the reference's built-in ops (python/src/tilefish/ops.py:1-30, :535-600, :916-970): no implicit dtype
promotion, python scalars and ``const`` parameters adopt the tensor's dtype, the math functions take floating-point tensors, a
cast is a rounding point exactly when the target cannot represent every value of the source (a cast to the same dtype is the value
itself), an InOut parameter that was stored to is read at its stored copy (``.live``), an Out parameter is write-only, ``split`` along a non-leading axis gives strided
views. One addition: ``x.to(<BlockScaled>)`` of a bf16 tensor is allowed (the reference refuses it, ops.py:556-559) and
traces to a ``quantize`` node, which this backend runs with its quantization kernels.
"""

from __future__ import annotations

import builtins
from typing import Any, Dict, List, Optional, Sequence, Tuple

from .dims import as_expr, describe_pair, divisible, exact_ratio, simplify
from .dtypes import BlockScaled, DType, f32
from .errors import TilefishAttributeError, TilefishError, TilefishTypeError
from .ir import Node, Scalar, Value
from .types import TensorType

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


_SYMBOL = {"add": "+", "sub": "-", "mul": "*", "div": "/"}
_INT_RANGE = {"u8": (0, 255), "i32": (-(2**31), 2**31 - 1), "i64": (-(2**63), 2**63 - 1)}


def _read(v, ctx: Optional[TraceContext], what: str, where: str = "argument 'x'") -> Value:
    """``v`` as an operand that is read: a traced tensor of this trace, not a write-only Out parameter; for an InOut parameter that
    was stored to, the stored copy (its current version)."""
    if not isinstance(v, Value):
        raise TilefishTypeError(f"{what}: {where} must be a traced tensor value, got {type(v).__name__} ({v!r})")
    if ctx is not None and v._ctx is not ctx:
        raise TilefishTypeError(f"{what}: {where} ({v.ref}) belongs to a different trace: a value can only be used in the body that produced it")
    if v.is_param and v.access == "out":
        raise TilefishTypeError(f"{what}: {where} is the Out parameter '{v.name}', which is write-only: it has no value to read")
    return v._ctx.latest(v)


def _arith_dtype(v: Value, what: str, where: str) -> None:
    dt = v.type.dtype
    if isinstance(dt, BlockScaled):
        raise TilefishTypeError(f"{what}: {where} has the block-scaled dtype {dt}, which has no arithmetic (the gemm consumes it as it is)")
    if not getattr(dt, "computable", False):
        raise TilefishTypeError(f"{what}: {where} has storage dtype {dt}, which has no arithmetic; cast it first (.to(f32))")


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


def _scalar(x, like: Value, what: str, where: str):
    """A python number or a const as an operand of ``like``'s dtype."""
    dt = like.type.dtype
    name = None
    if isinstance(x, (Const, Scalar)):
        name, typed, value = x.name, x.dtype, x.value
        if value is None:
            raise TilefishTypeError(f"{what}: {where} const '{name}' has no value at trace time (give the parameter a default)")
        if typed is not None and typed is not dt:
            raise TilefishTypeError(f"{what}: {where} const '{name}' is const[{typed}] but the other operand has dtype {dt}; there is no implicit "
                                    f"promotion: cast the tensor first (.to({typed}))")
    elif isinstance(x, (int, float)) and not isinstance(x, bool):
        value = x
    else:
        raise TilefishTypeError(f"{what}: {where} must be a traced tensor, a python number or a const parameter, got {type(x).__name__} ({x!r})")
    if dt.is_float:
        value = float(value)
    else:
        if isinstance(value, float):
            raise TilefishTypeError(f"{what}: {where} {value!r} is a float scalar but the other operand has integer dtype {dt}; cast the tensor "
                                    "to a floating-point dtype first")
        lo, hi = _INT_RANGE.get(dt.name, (None, None))
        if lo is not None and not lo <= value <= hi:
            raise TilefishTypeError(f"{what}: {where} {value!r} does not fit the other operand's dtype {dt} ({lo}..{hi})")
    return Scalar(value, dt, name)


def _broadcast(a: Value, b: Value, what: str):
    sa, sb = a.type.shape, b.type.shape
    out = []
    for i in range(builtins.max(len(sa), len(sb))):  # this module's own `max` is the traced reduction
        x = sa[len(sa) - 1 - i] if i < len(sa) else 1
        y = sb[len(sb) - 1 - i] if i < len(sb) else 1
        if as_expr(x) == as_expr(y):
            out.append(x)
        elif as_expr(x) == as_expr(1):
            out.append(y)
        elif as_expr(y) == as_expr(1):
            out.append(x)
        else:
            dx, dy = describe_pair(x, y)
            raise TilefishTypeError(f"{what}: cannot broadcast {a.type!r} with {b.type!r}: dimension {dx} vs {dy} at axis {-(i + 1)}")
    return tuple(reversed(out))


def binary(op: str, a, b) -> Value:
    what = f"{op} ({_SYMBOL[op]})"
    like = a if isinstance(a, Value) else b
    ctx = _ctx_of(like)
    sides = []
    for x, where in ((a, "left operand"), (b, "right operand")):
        if isinstance(x, Value):
            x = _read(x, ctx, what, where)
            _arith_dtype(x, what, where)
            if op == "div" and not x.type.dtype.is_float:
                raise TilefishTypeError(f"{what}: {where} must be a floating-point tensor, got {x.type!r}; cast it first (.to(f32))")
        sides.append(x)
    a, b = sides
    like = a if isinstance(a, Value) else b
    if isinstance(a, Value) and isinstance(b, Value):
        if a.type.dtype is not b.type.dtype:
            raise TilefishTypeError(f"{what}: no implicit promotion between dtypes: left operand is {a.type!r}, right operand is {b.type!r}; "
                                    "cast one side (.to(dtype))")
        shape = _broadcast(a, b, what)
    else:
        a = a if isinstance(a, Value) else _scalar(a, like, what, "left operand")
        b = b if isinstance(b, Value) else _scalar(b, like, what, "right operand")
        shape = like.type.shape
    return ctx.emit(op, (a, b), (TensorType(shape, like.type.dtype),))[0]


def cast(x: Value, dtype) -> Value:
    ctx = _ctx_of(x) if isinstance(x, Value) else None
    x = _read(x, ctx, "to")
    src = x.type.dtype
    if isinstance(dtype, BlockScaled):
        if isinstance(src, BlockScaled) or src.name != "bf16":
            raise TilefishTypeError(f"cast: only a bf16 tensor can be quantized to the block-scaled dtype {dtype}, {x.ref} is {src}")
        if dtype.format_name is None:
            raise TilefishTypeError(f"cast: this backend has no quantizer for the block-scaled dtype {dtype} (mxfp8, mxfp4 and nvfp4 are implemented)")
        if dtype.normalized(x.type.rank).axis != x.type.rank - 1:
            raise TilefishTypeError(f"cast: {dtype} must block the last axis")
        return ctx.emit("quantize", (x,), (TensorType(x.type.shape, dtype),), {"to": dtype, "rounding": True})[0]
    if isinstance(src, BlockScaled):
        raise TilefishTypeError(f"cast: dequantizing {x.ref} (block-scaled dtype {src}) is not an operation of this backend; the gemm consumes block-scaled operands directly")
    if not isinstance(dtype, DType):
        raise TilefishTypeError(f"cast: expected a dtype, got {dtype!r}")
    if dtype is src:
        return x  # nothing to do: the same value (a view stays the view)
    rounding = src.is_narrowing_to(dtype)
    return ctx.emit("cast", (x,), (TensorType(x.type.shape, dtype),), {"to": dtype, "rounding": rounding})[0]


def unary(op: str, x) -> Value:
    ctx = _ctx_of(x) if isinstance(x, Value) else None
    x = _read(x, ctx, op)
    _arith_dtype(x, op, "argument 'x'")
    if not x.type.dtype.is_float:
        raise TilefishTypeError(f"{op}: argument 'x' must be a floating-point tensor, got {x.type!r}; cast it first (.to(f32))")
    return ctx.emit(op, (x,), (TensorType(x.type.shape, x.type.dtype),))[0]


def reduce(op: str, x, axis=None, keepdims: bool = False) -> Value:
    ctx = _ctx_of(x) if isinstance(x, Value) else None
    x = _read(x, ctx, op)
    _arith_dtype(x, op, "argument 'x'")
    if op == "mean" and not x.type.dtype.is_float:
        raise TilefishTypeError(f"{op}: argument 'x' must be a floating-point tensor, got {x.type!r}; cast it first (.to(f32))")
    rank = x.type.rank
    if axis is None:
        axes = tuple(range(rank))
    elif isinstance(axis, int) and not isinstance(axis, bool):
        axes = (axis,)
    elif isinstance(axis, (tuple, list)) and all(isinstance(a, int) and not isinstance(a, bool) for a in axis):
        axes = tuple(axis)
    else:
        raise TilefishTypeError(f"{op}: axis must be an int, a tuple of ints or None, got {axis!r}")
    norm = []
    for ax in axes:
        a = ax + rank if ax < 0 else ax
        if not 0 <= a < rank:
            raise TilefishTypeError(f"{op}: axis {ax} is out of range for {x.type!r}")
        if a in norm:
            raise TilefishTypeError(f"{op}: duplicate axes in {axis!r}")
        norm.append(a)
    if keepdims:
        shape = tuple(1 if i in norm else s for i, s in enumerate(x.type.shape))
    else:
        shape = tuple(s for i, s in enumerate(x.type.shape) if i not in norm)
    return ctx.emit(op, (x,), (TensorType(shape, x.type.dtype),), {"axes": tuple(sorted(norm)), "keepdims": bool(keepdims)})[0]


_MISSING = object()


def split(x: Value, size=_MISSING, axis=_MISSING) -> Tuple[Value, ...]:
    ctx = _ctx_of(x) if isinstance(x, Value) else None
    x = _read(x, ctx, "split")
    if size is _MISSING or axis is _MISSING:
        raise TilefishTypeError("split: needs a size and an axis: x.split(size, axis=...) (one size for equal chunks, or a list of sizes)")
    rank = x.type.rank
    if not isinstance(axis, int) or isinstance(axis, bool) or not -rank <= axis < rank:
        raise TilefishTypeError(f"split: axis {axis!r} is invalid for {x.type!r}")
    ax = axis + rank if axis < 0 else axis
    dim = x.type.shape[ax]
    total = as_expr(dim)
    explicit = isinstance(size, (list, tuple))
    sizes_in = list(size) if explicit else [size]
    parts = []
    for s in sizes_in:
        try:
            if isinstance(s, (bool, str, float)):
                raise TilefishTypeError("")
            parts.append(as_expr(s))
        except TilefishTypeError:
            raise TilefishTypeError(f"split: sizes must be ints or dimensions, got {s!r}") from None
    if explicit:
        acc = as_expr(0)
        for e in parts:
            acc = acc + e
        if simplify(acc) != simplify(total):
            raise TilefishTypeError(f"split: the sizes {list(sizes_in)} add up to {simplify(acc)} but axis {ax} of {x.type!r} is {dim}")
        sizes = [simplify(s) for s in sizes_in]
    else:
        # the number of chunks must be one integer for every binding of the dimensions: a static quotient, or a constant ratio (2*F into F)
        count = exact_ratio(total, parts[0])
        if count is None or count <= 0:
            raise TilefishTypeError(f"split: axis {ax} of {x.type!r} is not a whole number of chunks of size {size}")
        sizes = [simplify(size)] * count
    leading = all(as_expr(s) == as_expr(1) for s in x.type.shape[:ax])
    types = []
    for sz in sizes:
        e = as_expr(sz)
        try:
            if e.is_static and e.offset <= 0:
                raise TilefishTypeError(f"size {sz} is not positive")
            if isinstance(x.type.dtype, BlockScaled):
                fmt = x.type.dtype.normalized(rank)
                if fmt.axis == ax and not divisible(e, fmt.block):
                    raise TilefishTypeError(f"axis {ax} has size {sz}, which is not divisible by block={fmt.block}")
            types.append(TensorType(tuple(sz if i == ax else s for i, s in enumerate(x.type.shape)), x.type.dtype, contiguous=leading and x.type.contiguous))
        except TilefishError as err:
            raise TilefishTypeError(f"split: chunk type is invalid: {err}") from None
    return ctx.emit("split", (x,), tuple(types), {"axis": ax, "sizes": tuple(sizes)})


def permute(x: Value, *axes) -> Value:
    """A transposed view: the axes in another order (a strided view; nothing is copied)."""
    ctx = _ctx_of(x) if isinstance(x, Value) else None
    x = _read(x, ctx, "permute")
    if len(axes) == 1 and isinstance(axes[0], (tuple, list)):
        axes = tuple(axes[0])
    rank = x.type.rank
    if not all(isinstance(a, int) and not isinstance(a, bool) for a in axes):
        raise TilefishTypeError(f"permute: axes must be ints, got {axes!r}")
    norm = tuple(a + rank if a < 0 else a for a in axes)
    if sorted(norm) != list(range(rank)):
        raise TilefishTypeError(f"permute: {axes!r} is not a permutation of the {rank} axes of {x.type!r}")
    if norm == tuple(range(rank)):
        return x
    t = TensorType(tuple(x.type.shape[a] for a in norm), x.type.dtype, contiguous=False)
    return ctx.emit("permute", (x,), (t,), {"axes": norm})[0]


def store(target: Value, value) -> None:
    ctx = _ctx_of(target)
    what = f"store into '{target.name}'" if target.name else f"store into {target.ref}"
    if not target.is_param or target.access not in ("inout", "out"):
        raise TilefishTypeError(f"{what}: the parameter is read-only; declare it InOut[...] (or Out[...]) to write it")
    value = _read(value, ctx, what, "the stored value")
    want = target.type
    same = (value.type.rank == want.rank and value.type.dtype is want.dtype
            and all(as_expr(a) == as_expr(b) for a, b in zip(value.type.shape, want.shape)))
    view_in_kernel = same and not value.type.contiguous and ctx.kind == "kernel"
    if not same or view_in_kernel:
        hint = ("a strided view cannot be stored by a kernel body; compute from it (x * 1) or store it in a graph body" if view_in_kernel
                else "cast with .to(dtype) or fix the shape")
        raise TilefishTypeError(f"{what}: expected {want!r}, got {value.type!r}; {hint}")
    outs = (want,) if target.access == "inout" else ()
    made = ctx.emit("store", (target, value), outs, {"target": target.name})
    if made:
        ctx.versions[ctx.latest(target)] = made[0]
        ctx.finals[target.name] = made[0]
    else:
        ctx.finals[target.name] = value  # an Out parameter has no version to read back: what it holds is the stored value


# ---- the methods of a traced value ------------------------------------------------------------------------------------
def _install() -> None:
    def to(self, *args, **kwargs):
        if len(args) + len(kwargs) != 1 or (kwargs and "dtype" not in kwargs):
            raise TilefishTypeError("to: needs a dtype: x.to(f32)")
        return cast(self, args[0] if args else kwargs["dtype"])

    def split_method(self, *args, **kwargs):
        if len(args) > 2 or set(kwargs) - {"size", "axis"}:
            raise TilefishTypeError("split: needs a size and an axis: x.split(size, axis=...)")
        size = args[0] if args else kwargs.get("size", _MISSING)
        axis = args[1] if len(args) > 1 else kwargs.get("axis", _MISSING)
        return split(self, size, axis)

    Value.to = to
    Value.split = split_method
    Value.mean = lambda self, axis=None, keepdims=False: reduce("mean", self, axis, keepdims)
    Value.sum = lambda self, axis=None, keepdims=False: reduce("sum", self, axis, keepdims)
    Value.max = lambda self, axis=None, keepdims=False: reduce("max", self, axis, keepdims)
    Value.shape = property(lambda self: self.type.shape)
    Value.dtype = property(lambda self: self.type.dtype)
    Value.live = property(lambda self: self._ctx.latest(self))
    Value.ctx = property(lambda self: self._ctx)
    Value.__add__ = lambda self, o: binary("add", self, o)
    Value.__radd__ = lambda self, o: binary("add", o, self)
    Value.__sub__ = lambda self, o: binary("sub", self, o)
    Value.__rsub__ = lambda self, o: binary("sub", o, self)
    Value.__mul__ = lambda self, o: binary("mul", self, o)
    Value.__rmul__ = lambda self, o: binary("mul", o, self)
    Value.__truediv__ = lambda self, o: binary("div", self, o)
    Value.__rtruediv__ = lambda self, o: binary("div", o, self)

    def setitem(self, key, value):
        if key is not Ellipsis:
            raise TilefishTypeError("only whole-tensor assignment is supported: write `x[...] = value`")
        store(self, value)

    Value.__setitem__ = setitem

    def getitem(self, key):
        keys = key if isinstance(key, tuple) else (key,)
        for k in keys:
            if not (k is Ellipsis or isinstance(k, slice) or (isinstance(k, int) and not isinstance(k, bool))):
                raise TilefishTypeError(f"{self.ref}: an index must be a python int, ':' or '...', got {k!r}")
        raise TilefishTypeError(f"{self.ref}: indexing a traced tensor (a view of it) is not part of this backend's language; use split")

    Value.__getitem__ = getitem

    def refuse(message):
        def method(self, *args, **kwargs):
            raise TilefishTypeError(f"{self.ref}: {message}")

        return method

    Value.__iter__ = refuse("a traced tensor cannot be unpacked or iterated; split(...) returns its chunks")
    Value.__bool__ = refuse("a traced tensor has no truth value at trace time (its data does not exist yet)")
    unsupported = "this operator is not supported in M1 (the elementwise language is + - * / and the tilefish functions)"
    for name in ("__pos__", "__neg__", "__abs__", "__pow__", "__rpow__", "__matmul__", "__rmatmul__", "__len__", "__int__", "__float__", "__index__",
                 "__lshift__", "__rshift__", "__rlshift__", "__rrshift__", "__lt__", "__le__", "__gt__", "__ge__"):
        setattr(Value, name, refuse(unsupported))
    for name in ("__floordiv__", "__rfloordiv__", "__mod__", "__rmod__"):
        setattr(Value, name, refuse("integer division and remainder are not supported: use / on floating-point tensors"))
    for name in ("__invert__", "__and__", "__rand__", "__or__", "__ror__", "__xor__", "__rxor__"):
        setattr(Value, name, refuse("bitwise operators are not supported: a tensor of numbers is not a mask"))
    Value.reshape = refuse("reshape is not part of this backend's language")
    Value.permute = lambda self, *axes: permute(self, *axes)

    def missing(self, name):
        raise TilefishAttributeError(f"traced values have no attribute {name!r}")

    Value.__getattr__ = missing


_install()


# ---- public math ops ----------------------------------------------------------------------------------------------------
def silu(x: Value) -> Value:
    return unary("silu", x)


def sqrt(x: Value) -> Value:
    return unary("sqrt", x)


def gelu(x: Value) -> Value:
    return unary("gelu", x)


def contiguous(x: Value) -> Value:
    """A dense copy of a strided view (the type's ``contiguous`` flag set); a contiguous tensor is returned as is."""
    x = _read(x, _ctx_of(x) if isinstance(x, Value) else None, "contiguous")
    if x.type.contiguous:
        return x
    return _ctx_of(x).emit("contiguous", (x,), (TensorType(x.type.shape, x.type.dtype, contiguous=True),))[0]


def rsqrt(x: Value) -> Value:
    return unary("rsqrt", x)


def exp(x: Value) -> Value:
    return unary("exp", x)


def mean(x: Value, axis=None, keepdims: bool = False) -> Value:
    return reduce("mean", x, axis, keepdims)


def reduce_sum(x: Value, axis=None, keepdims: bool = False) -> Value:
    return reduce("sum", x, axis, keepdims)


def reduce_max(x: Value, axis=None, keepdims: bool = False) -> Value:
    return reduce("max", x, axis, keepdims)


# the reference's spellings (tilefish.sum / tilefish.max); kept out of `import *` because they would shadow the builtins
sum = reduce_sum  # noqa: A001
max = reduce_max  # noqa: A001
