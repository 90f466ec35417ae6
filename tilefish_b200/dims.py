"""Dimensions: named sizes that live in tensor types.

Mirrors the public behaviour of the reference's ``Dim`` (python/src/tilefish/dims.py:541-647): a dimension is static
(``Dim("D", 2560)``: compares equal to its int), dynamic (``Dim("M")``), dynamic with a divisibility promise
(``Dim("K", divisible_by=32)``) or bucketed (``Dim("M", buckets=[1, 32])``). Arithmetic on dimensions gives a ``DimExpr``:
an integer-affine combination of atoms (dynamic dimensions and ``cdiv`` terms), with static dimensions folded into
constants, so that ``2 * F == F + F`` and ``2 * Dim("F", 3072) == 6144``.
"""

from __future__ import annotations

from typing import Dict, Iterable, Optional, Tuple, Union

from .errors import TilefishDeclarationError, TilefishTypeError

DimLike = Union["Dim", "DimExpr", int]


class Dim:
    __slots__ = ("name", "value", "divisible_by", "buckets")

    def __init__(self, name: str, value: Optional[int] = None, *, divisible_by: Optional[int] = None, buckets: Optional[Iterable[int]] = None) -> None:
        if not isinstance(name, str) or not name.isidentifier():
            raise TilefishDeclarationError(f"Dim: the name must be an identifier, got {name!r}")
        if value is not None and (isinstance(value, bool) or not isinstance(value, int) or value <= 0):
            raise TilefishDeclarationError(f"Dim('{name}'): a static size must be a positive int, got {value!r}")
        if divisible_by is not None and (not isinstance(divisible_by, int) or divisible_by <= 0):
            raise TilefishDeclarationError(f"Dim('{name}'): divisible_by must be a positive int, got {divisible_by!r}")
        if value is not None and divisible_by is not None and value % divisible_by:
            raise TilefishDeclarationError(f"Dim('{name}', {value}) is not divisible by {divisible_by}")
        b = None
        if buckets is not None:
            if value is not None:
                raise TilefishDeclarationError(f"Dim('{name}'): a static dimension cannot have buckets")
            b = tuple(buckets)
            if not b or any(isinstance(x, bool) or not isinstance(x, int) or x <= 0 for x in b) or list(b) != sorted(set(b)):
                raise TilefishDeclarationError(f"Dim('{name}'): buckets must be sorted, unique, positive ints, got {list(b)!r}")
            if divisible_by is not None and any(x % divisible_by for x in b):
                raise TilefishDeclarationError(f"Dim('{name}'): every bucket must be divisible by {divisible_by}")
        object.__setattr__(self, "name", name)
        object.__setattr__(self, "value", value)
        object.__setattr__(self, "divisible_by", divisible_by)
        object.__setattr__(self, "buckets", b)

    def __setattr__(self, key, value):  # immutable
        raise AttributeError("Dim is immutable")

    @property
    def is_static(self) -> bool:
        return self.value is not None

    def _key(self):
        return (self.name, self.divisible_by, self.buckets)

    def __eq__(self, other) -> bool:
        if isinstance(other, Dim):
            if self.is_static or other.is_static:
                return self.value == other.value and self.value is not None
            return self._key() == other._key()
        if isinstance(other, int) and not isinstance(other, bool):
            return self.value == other
        if isinstance(other, DimExpr):
            return as_expr(self) == other
        return NotImplemented

    def __hash__(self) -> int:
        return hash(self.value) if self.is_static else hash(self._key())

    def __repr__(self) -> str:
        parts = [repr(self.name)]
        if self.value is not None:
            parts.append(str(self.value))
        if self.divisible_by is not None:
            parts.append(f"divisible_by={self.divisible_by}")
        if self.buckets is not None:
            parts.append(f"buckets={list(self.buckets)}")
        return f"Dim({', '.join(parts)})"

    def __str__(self) -> str:
        return self.name

    # arithmetic -> DimExpr
    def __add__(self, o):
        return as_expr(self) + o

    __radd__ = __add__

    def __sub__(self, o):
        return as_expr(self) - o

    def __mul__(self, o):
        return as_expr(self) * o

    __rmul__ = __mul__

    def __floordiv__(self, o):
        return as_expr(self) // o


class _Cdiv:
    """The atom ``cdiv(expr, n)`` of an expression that does not divide exactly."""

    __slots__ = ("expr", "n")

    def __init__(self, expr: "DimExpr", n: int) -> None:
        self.expr, self.n = expr, n

    def __eq__(self, o) -> bool:
        return isinstance(o, _Cdiv) and self.n == o.n and self.expr == o.expr

    def __hash__(self) -> int:
        return hash(("cdiv", self.n, self.expr))

    def __str__(self) -> str:
        return f"cdiv({self.expr}, {self.n})"

    name = property(lambda self: str(self))


Atom = Union[Dim, _Cdiv]


class DimExpr:
    """const + sum(coef * atom), atoms being dynamic ``Dim``s or ``cdiv`` terms; immutable and hashable."""

    __slots__ = ("terms", "const")

    def __init__(self, terms: Dict[Atom, int], const: int = 0) -> None:
        clean = {a: c for a, c in terms.items() if c != 0}
        object.__setattr__(self, "terms", tuple(sorted(clean.items(), key=lambda kv: str(kv[0]))))
        object.__setattr__(self, "const", int(const))

    def __setattr__(self, key, value):
        raise AttributeError("DimExpr is immutable")

    @property
    def is_static(self) -> bool:
        return not self.terms

    @property
    def value(self) -> Optional[int]:
        return self.const if self.is_static else None

    def _dict(self) -> Dict[Atom, int]:
        return dict(self.terms)

    def __add__(self, o):
        o = as_expr(o)
        d = self._dict()
        for a, c in o.terms:
            d[a] = d.get(a, 0) + c
        return DimExpr(d, self.const + o.const)

    __radd__ = __add__

    def __neg__(self):
        return DimExpr({a: -c for a, c in self.terms}, -self.const)

    def __sub__(self, o):
        return self + (-as_expr(o))

    def __rsub__(self, o):
        return as_expr(o) - self

    def __mul__(self, o):
        o = as_expr(o)
        if o.is_static:
            return DimExpr({a: c * o.const for a, c in self.terms}, self.const * o.const)
        if self.is_static:
            return o * self
        raise TilefishTypeError(f"the product of two dynamic sizes ({self}) * ({o}) is not an affine size")

    __rmul__ = __mul__

    def __floordiv__(self, n):
        if not isinstance(n, int) or n <= 0:
            raise TilefishTypeError(f"a size can only be divided by a positive int, got {n!r}")
        if not divisible(self, n):
            raise TilefishTypeError(f"({self}) // {n}: {self} is not provably divisible by {n}; use cdiv")
        return cdiv(self, n)

    def __eq__(self, o) -> bool:
        if isinstance(o, (Dim, int, DimExpr)) and not isinstance(o, bool):
            o = as_expr(o)
            return self.terms == o.terms and self.const == o.const
        return NotImplemented

    def __hash__(self) -> int:
        if self.is_static:
            return hash(self.const)
        if self.const == 0 and len(self.terms) == 1 and self.terms[0][1] == 1 and isinstance(self.terms[0][0], Dim):
            return hash(self.terms[0][0])
        return hash((self.terms, self.const))

    def __str__(self) -> str:
        if self.is_static:
            return str(self.const)
        parts = []
        for a, c in self.terms:
            parts.append(str(a) if c == 1 else f"{c}*{a}")
        s = " + ".join(parts)
        if self.const:
            s += f" + {self.const}" if self.const > 0 else f" - {-self.const}"
        return s

    def __repr__(self) -> str:
        return f"DimExpr({self})"


def as_expr(x: DimLike) -> DimExpr:
    if isinstance(x, DimExpr):
        return x
    if isinstance(x, Dim):
        return DimExpr({}, x.value) if x.is_static else DimExpr({x: 1}, 0)
    if isinstance(x, int) and not isinstance(x, bool):
        return DimExpr({}, x)
    raise TilefishTypeError(f"expected a Dim, a size expression or an int, got {x!r}")


def simplify(x: DimLike) -> DimLike:
    """The canonical spelling of a size inside a type: the ``Dim`` itself when it is one (a static one keeps its name and
    compares equal to its int), an int for any other static size, else the expression."""
    if isinstance(x, Dim):
        return x
    e = as_expr(x)
    if e.is_static:
        return e.const
    if e.const == 0 and len(e.terms) == 1 and e.terms[0][1] == 1 and isinstance(e.terms[0][0], Dim):
        return e.terms[0][0]
    return e


def divisible(x: DimLike, n: int) -> bool:
    """Whether ``x`` is provably a multiple of ``n`` from the declarations alone."""
    e = as_expr(x)
    if e.const % n:
        return False
    for a, c in e.terms:
        unit = a.divisible_by or 1 if isinstance(a, Dim) else 1
        if isinstance(a, Dim) and a.buckets is not None and all(b % n == 0 for b in a.buckets):
            continue
        if (c * unit) % n:
            return False
    return True


def cdiv(x: DimLike, n: int) -> DimLike:
    """ceil(x / n) as a size: exact when ``x`` is static or provably divisible term by term, else an opaque ``cdiv`` atom."""
    if isinstance(x, int) and not isinstance(x, bool):
        return -(-x // n)
    e = as_expr(x)
    if e.is_static:
        return -(-e.const // n)
    if e.const % n == 0 and all(c % n == 0 for _, c in e.terms):
        return simplify(DimExpr({a: c // n for a, c in e.terms}, e.const // n))
    return DimExpr({_Cdiv(e, n): 1}, 0)


def symbols(x: DimLike) -> Tuple[Dim, ...]:
    out = []
    for a, _ in as_expr(x).terms:
        if isinstance(a, Dim):
            out.append(a)
        else:
            out.extend(symbols(a.expr))
    return tuple(out)


def evaluate(x: DimLike, env: Dict[Dim, int]) -> Optional[int]:
    """The value of ``x`` with the dynamic dimensions bound by ``env``; None when one is unbound."""
    e = as_expr(x)
    total = e.const
    for a, c in e.terms:
        if isinstance(a, Dim):
            v = env.get(a)
        else:
            inner = evaluate(a.expr, env)
            v = None if inner is None else -(-inner // a.n)
        if v is None:
            return None
        total += c * v
    return total
