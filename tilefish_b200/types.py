"""Tensor types: ``Tensor[M, D, bf16]``, ``InOut[...]``, ``Out[...]``, ``const[f32]``.

Spellings and equality follow the reference (python/src/tilefish/types.py:65-258, :520-641): a tensor type is immutable, is
written ``Tensor[M, D, bf16]`` when dense and ``View[...]`` when it is a strided view (what ``split`` along a non-leading
axis gives), and two types are equal when shape, dtype and contiguity are equal.
"""

from __future__ import annotations

from typing import Optional, Tuple, Union

from .dims import Dim, DimExpr, DimLike, as_expr, simplify
from .dtypes import BlockScaled, DType, same_format
from .errors import TilefishDeclarationError, TilefishTypeError


class TensorType:
    __slots__ = ("shape", "dtype", "contiguous")

    def __init__(self, shape: Tuple[DimLike, ...], dtype: Union[DType, BlockScaled], contiguous: bool = True) -> None:
        if not isinstance(dtype, (DType, BlockScaled)):
            raise TilefishDeclarationError(f"Tensor[...]: the last entry must be a dtype, got {dtype!r}")
        norm = []
        for s in shape:
            if isinstance(s, bool) or not isinstance(s, (Dim, DimExpr, int)):
                raise TilefishDeclarationError(f"Tensor[...]: a size must be a Dim, a size expression or an int, got {s!r}")
            s = simplify(s)
            if isinstance(s, int) and not isinstance(s, Dim) and s <= 0:
                raise TilefishDeclarationError(f"Tensor[...]: a size must be positive, got {s}")
            norm.append(s)
        if isinstance(dtype, BlockScaled):
            if not norm:
                raise TilefishDeclarationError("a block-scaled tensor needs at least one axis")
            dtype.check_shape(tuple(norm))
        object.__setattr__(self, "shape", tuple(norm))
        object.__setattr__(self, "dtype", dtype)
        object.__setattr__(self, "contiguous", bool(contiguous))

    def __setattr__(self, key, value):
        raise AttributeError("TensorType is immutable")

    def __reduce__(self):  # copies and pickles are rebuilt through the constructor (the slots cannot be set from outside)
        return (TensorType, (self.shape, self.dtype, self.contiguous))

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def is_blockscaled(self) -> bool:
        return isinstance(self.dtype, BlockScaled)

    @property
    def scale_shape(self) -> Optional[Tuple[DimLike, ...]]:
        return self.dtype.scale_shape(self.shape) if self.is_blockscaled else None

    @property
    def scale_type(self) -> Optional["TensorType"]:
        return TensorType(self.scale_shape, self.dtype.scale) if self.is_blockscaled else None

    def as_view(self) -> "TensorType":
        return TensorType(self.shape, self.dtype, contiguous=False)

    def materialized(self) -> "TensorType":
        """The type of a dense copy: a view's contiguous twin, a contiguous type itself."""
        return self if self.contiguous else TensorType(self.shape, self.dtype, contiguous=True)

    def with_dtype(self, dtype) -> "TensorType":
        return TensorType(self.shape, dtype, self.contiguous)

    def with_shape(self, shape) -> "TensorType":
        return TensorType(tuple(shape), self.dtype, True)

    def __eq__(self, other) -> bool:
        if not isinstance(other, TensorType):
            return NotImplemented
        return (self.rank == other.rank and self.contiguous == other.contiguous and same_format(self.dtype, other.dtype, self.rank)
                and all(as_expr(a) == as_expr(b) for a, b in zip(self.shape, other.shape)))

    def __hash__(self) -> int:
        return hash((tuple(hash(as_expr(s)) for s in self.shape), str(self.dtype), self.contiguous))

    def __repr__(self) -> str:
        head = "Tensor" if self.contiguous else "View"
        return f"{head}[{', '.join([str(s) for s in self.shape] + [str(self.dtype)])}]"

    __str__ = __repr__


class _TensorFactory:
    """``Tensor[d0, ..., dtype]``."""

    def __getitem__(self, items) -> TensorType:
        if not isinstance(items, tuple):
            items = (items,)
        if not items:
            raise TilefishDeclarationError("Tensor[...] needs a dtype")
        return TensorType(tuple(items[:-1]), items[-1])

    def __repr__(self) -> str:
        return "Tensor"


Tensor = _TensorFactory()


class Marked:
    """``InOut[T]`` / ``Out[T]``: a parameter the operator writes."""

    __slots__ = ("mode", "type")

    def __init__(self, mode: str, type_: TensorType) -> None:
        self.mode, self.type = mode, type_

    def __eq__(self, o) -> bool:
        return isinstance(o, Marked) and (self.mode, self.type) == (o.mode, o.type)

    def __hash__(self) -> int:
        return hash((self.mode, self.type))

    def __repr__(self) -> str:
        return f"{'InOut' if self.mode == 'inout' else 'Out'}[{self.type!r}]"


class _MarkFactory:
    def __init__(self, mode: str) -> None:
        self.mode = mode

    def __getitem__(self, t) -> Marked:
        if not isinstance(t, TensorType):
            raise TilefishDeclarationError(f"{'InOut' if self.mode == 'inout' else 'Out'}[...] takes a tensor type, got {t!r}")
        return Marked(self.mode, t)


InOut = _MarkFactory("inout")
Out = _MarkFactory("out")


class ConstType:
    """``const[f32]``: a keyword-only scalar of a declaration; a call inside a graph may give it another value than its default (the call
    node records it), ``tilefish.run`` of a built plan may only restate the value the plan was built with."""

    __slots__ = ("dtype",)

    def __init__(self, dtype: Optional[DType] = None) -> None:
        self.dtype = dtype

    def __getitem__(self, dtype: DType) -> "ConstType":
        if not isinstance(dtype, DType):
            raise TilefishDeclarationError(f"const[...] takes a dtype, got {dtype!r}")
        return ConstType(dtype)

    def __eq__(self, o) -> bool:
        return isinstance(o, ConstType) and self.dtype is o.dtype

    def __hash__(self) -> int:
        return hash(("const", self.dtype))

    def __repr__(self) -> str:
        return "const" if self.dtype is None else f"const[{self.dtype}]"


const = ConstType()


def broadcast_shapes(a: Tuple[DimLike, ...], b: Tuple[DimLike, ...], what: str) -> Tuple[DimLike, ...]:
    """numpy-style broadcasting over sizes (a size of 1 stretches); anything else must be equal."""
    out = []
    ra, rb = len(a), len(b)
    for i in range(max(ra, rb)):
        x = a[ra - 1 - i] if i < ra else 1
        y = b[rb - 1 - i] if i < rb else 1
        if as_expr(x) == as_expr(y):
            out.append(x)
        elif as_expr(x) == as_expr(1):
            out.append(y)
        elif as_expr(y) == as_expr(1):
            out.append(x)
        else:
            raise TilefishTypeError(f"{what}: shapes {_fmt(a)} and {_fmt(b)} do not broadcast ({x} vs {y})")
    return tuple(reversed(out))


def _fmt(shape) -> str:
    return "[" + ", ".join(str(s) for s in shape) + "]"
