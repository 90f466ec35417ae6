"""Dimensions: named sizes that live in tensor types.

Mirrors the public behaviour of the reference's ``Dim`` / ``DimExpr`` / ``cdiv`` (python/src/tilefish/dims.py:541-647 and its
tests, python/tests/test_dims.py): a dimension is static (``Dim("D", 2560)``: compares equal to its int and can be used as
one), dynamic (``Dim("M")``), dynamic with a divisibility promise (``Dim("K", divisible_by=32)``) or bucketed
(``Dim("M", buckets=[1, 32])``). Arithmetic on dimensions gives a ``DimExpr``: an integer-affine combination
``offset + sum(coef * atom)`` of atoms (dynamic dimensions and ``cdiv`` nodes), with static dimensions folded into the
offset, so that ``2 * F == F + F`` and ``2 * Dim("F", 3072) == 6144``. Everything outside that language (products of two
dynamic sizes, true division, ``%``, ``**``, ordering, use as an integer) raises ``TilefishTypeError`` for a symbolic size
and works as on ints for a static one.
"""

from __future__ import annotations

from math import gcd
from typing import Dict, Iterable, Mapping, Optional, Tuple, Union

from .errors import TilefishDeclarationError, TilefishTypeError

DimLike = Union["Dim", "DimExpr", int]


def _is_int(x) -> bool:
    return isinstance(x, int) and not isinstance(x, bool)


def _lcm(a: int, b: int) -> int:
    return a * b // gcd(a, b)


class _SizeOps:
    """Operators shared by ``Dim`` and ``DimExpr``: the affine ones build expressions, the others work on static sizes only."""

    __slots__ = ()

    # ---- the affine language ----
    def __add__(self, o):
        return as_expr(self)._add(_operand(self, "+", o))

    def __radd__(self, o):
        return _operand(self, "+", o)._add(as_expr(self))

    def __sub__(self, o):
        return as_expr(self)._add(_operand(self, "-", o)._scale(-1))

    def __rsub__(self, o):
        return _operand(self, "-", o)._add(as_expr(self)._scale(-1))

    def __neg__(self):
        return as_expr(self)._scale(-1)

    def __pos__(self):
        return as_expr(self)

    def __mul__(self, o):
        a, b = as_expr(self), _operand(self, "*", o)
        if b.is_static:
            return a._scale(b.offset)
        if a.is_static:
            return b._scale(a.offset)
        raise TilefishTypeError(f"({a}) * ({b}): sizes are affine (an int times a dimension, sums of those); the product of two symbolic sizes is not")

    __rmul__ = __mul__

    def __floordiv__(self, o):
        a = as_expr(self)
        n = _static_value(o)
        if n is None or n <= 0:
            raise TilefishTypeError(f"({a}) // {o}: the divisor must be a positive static int")
        if a.is_static:
            return DimExpr.const(a.offset // n)
        if a.offset % n or any(c % n for _, c in a.terms):
            raise TilefishTypeError(f"({a}) // {n} is not provably exact (every coefficient and the offset must be multiples of {n}); use tilefish.cdiv")
        return DimExpr({t: c // n for t, c in a.terms}, a.offset // n)

    def __rfloordiv__(self, o):
        n = _static_value(self)
        if n is None or n <= 0 or not _is_int(o):
            raise TilefishTypeError(f"{o!r} // ({self}): the divisor must be a positive static int")
        return o // n

    # ---- outside the affine language: static sizes behave as their ints, symbolic ones refuse ----
    def _int(self, what: str) -> int:
        v = _static_value(self)
        if v is None:
            raise TilefishTypeError(f"{self} is symbolic and cannot be used as an integer ({what})")
        return v

    def __index__(self) -> int:
        return self._int("an index, a range bound or a count")

    def __int__(self) -> int:
        return self._int("int()")

    def __float__(self) -> float:
        return float(self._int("float()"))

    def __abs__(self):
        return abs(self._int("abs()"))

    def __truediv__(self, o):
        raise TilefishTypeError(f"({self}) / {o!r}: true division is not a size; use // for an exact division or tilefish.cdiv for a rounded-up one")

    def __rtruediv__(self, o):
        raise TilefishTypeError(f"{o!r} / ({self}): true division is not a size; use // for an exact division or tilefish.cdiv for a rounded-up one")

    def _other_int(self, op: str, o) -> int:
        v = _static_value(o) if isinstance(o, (Dim, DimExpr)) or _is_int(o) else None
        if v is None:
            raise TilefishTypeError(f"({self}) {op} {o!r}: not defined for sizes")
        return v

    def __mod__(self, o):
        return self._int("%") % self._other_int("%", o)

    def __rmod__(self, o):
        return self._other_int("%", o) % self._int("%")

    def __pow__(self, o):
        return self._int("**") ** self._other_int("**", o)

    def __rpow__(self, o):
        return self._other_int("**", o) ** self._int("**")

    def __lt__(self, o):
        return self._int("<") < self._other_int("<", o)

    def __le__(self, o):
        return self._int("<=") <= self._other_int("<=", o)

    def __gt__(self, o):
        return self._int(">") > self._other_int(">", o)

    def __ge__(self, o):
        return self._int(">=") >= self._other_int(">=", o)

    # ---- reasoning ----
    def is_divisible_by(self, n: int, known: Optional[Mapping] = None) -> bool:
        """Whether the size is provably a multiple of ``n``: from the declarations (``divisible_by``, buckets, static values)
        and from ``known``, a mapping from dimensions, ``cdiv`` nodes or whole expressions to a divisor the caller vouches for."""
        return divisible(self, n, known)

    def exact_div(self, other) -> Optional[int]:
        """The integer ``q`` with ``self == q * other`` for every binding of the dimensions, or None."""
        return exact_ratio(self, other)

    def subst(self, mapping: Mapping) -> "DimLike":
        """The size with dimensions replaced (simultaneously) by other sizes."""
        return substitute(self, mapping)

    def free_dims(self):
        return set(symbols(self))


class Dim(_SizeOps):
    __slots__ = ("name", "_value", "divisible_by", "buckets")

    def __init__(self, name: str, value: Optional[int] = None, *, divisible_by: Optional[int] = None, buckets: Optional[Iterable[int]] = None) -> None:
        if not isinstance(name, str) or not name.isidentifier():
            raise TilefishDeclarationError(f"Dim: the name must be an identifier, got {name!r}")
        if value is not None and (not _is_int(value) or value <= 0):
            raise TilefishDeclarationError(f"Dim('{name}'): a static size must be a positive int, got {value!r}")
        if divisible_by is not None and (not _is_int(divisible_by) or divisible_by <= 0):
            raise TilefishDeclarationError(f"Dim('{name}'): divisible_by must be a positive int, got {divisible_by!r}")
        if value is not None and divisible_by is not None and value % divisible_by:
            raise TilefishDeclarationError(f"Dim('{name}', {value}) is not divisible by {divisible_by}")
        b = None
        if buckets is not None:
            try:
                b = tuple(buckets) if not isinstance(buckets, (str, bytes)) else None
            except TypeError:
                b = None
            if b is None or any(not _is_int(x) for x in b):
                raise TilefishDeclarationError(f"Dim('{name}'): buckets must be a list of ints, got {buckets!r}")
            if value is not None:
                raise TilefishDeclarationError(f"Dim('{name}'): a static dimension cannot have buckets")
            if not b or any(x <= 0 for x in b) or len(set(b)) != len(b):
                raise TilefishDeclarationError(f"Dim('{name}'): buckets must be a non-empty list of distinct positive ints, got {list(b)!r}")
            b = tuple(sorted(b))
            if divisible_by is not None and any(x % divisible_by for x in b):
                raise TilefishDeclarationError(f"Dim('{name}'): every bucket must be divisible by {divisible_by}")
        object.__setattr__(self, "name", name)
        object.__setattr__(self, "_value", value)
        object.__setattr__(self, "divisible_by", divisible_by)
        object.__setattr__(self, "buckets", b)

    def __setattr__(self, key, value):  # immutable
        raise AttributeError("Dim is immutable")

    def __delattr__(self, key):
        raise AttributeError("Dim is immutable")

    def __reduce__(self):
        return (_rebuild_dim, (self.name, self._value, self.divisible_by, self.buckets))

    @property
    def is_static(self) -> bool:
        return self._value is not None

    @property
    def is_dynamic(self) -> bool:
        return self._value is None

    @property
    def value(self) -> int:
        if self._value is None:
            raise TilefishTypeError(f"{self!r} is symbolic: it has no value until a call binds it")
        return self._value

    def folded(self):
        """A static dimension as the constant expression of its value (what a host sees); a dynamic one unchanged."""
        return DimExpr.const(self._value) if self.is_static else self

    def _key(self):
        return (self.name, self.divisible_by, self.buckets)

    def __eq__(self, other) -> bool:
        if isinstance(other, Dim):
            if self.is_static or other.is_static:
                return self._value == other._value and self._value is not None
            return self._key() == other._key()
        if _is_int(other):
            return self._value == other
        if isinstance(other, DimExpr):
            return as_expr(self) == other
        return NotImplemented

    def __ne__(self, other) -> bool:
        r = self.__eq__(other)
        return r if r is NotImplemented else not r

    def __hash__(self) -> int:
        return hash(self._value) if self.is_static else hash(self._key())

    def __repr__(self) -> str:
        parts = [repr(self.name)]
        if self._value is not None:
            parts.append(str(self._value))
        if self.divisible_by is not None:
            parts.append(f"divisible_by={self.divisible_by}")
        if self.buckets is not None:
            parts.append(f"buckets={list(self.buckets)}")
        return f"Dim({', '.join(parts)})"

    def __str__(self) -> str:
        return self.name


def _rebuild_dim(name, value, divisible_by, buckets):
    return Dim(name, value, divisible_by=divisible_by, buckets=buckets)


class _Cdiv:
    """The atom ``cdiv(num, den)`` of a quotient that does not fold: ``den`` is a positive int or a symbolic size."""

    __slots__ = ("num", "den")

    def __init__(self, num: "DimExpr", den) -> None:
        self.num, self.den = num, den

    def __eq__(self, o) -> bool:
        return isinstance(o, _Cdiv) and self.den == o.den and self.num == o.num

    def __hash__(self) -> int:
        return hash(("cdiv", self.den if _is_int(self.den) else hash(self.den), self.num))

    def __str__(self) -> str:
        return f"cdiv({self.num}, {self.den})"

    __repr__ = __str__
    name = property(lambda self: str(self))
    divisible_by = None
    buckets = None

    # the old spelling of the two parts
    expr = property(lambda self: self.num)
    n = property(lambda self: self.den)


Atom = Union[Dim, _Cdiv]


class DimExpr(_SizeOps):
    """offset + sum(coef * atom), atoms being dynamic ``Dim``s or ``cdiv`` nodes; immutable and hashable."""

    __slots__ = ("terms", "offset")

    def __init__(self, terms: Union[Dict[Atom, int], Iterable[Tuple[Atom, int]]], offset: int = 0) -> None:
        items = terms.items() if isinstance(terms, dict) else terms
        merged: Dict[Atom, int] = {}
        for a, c in items:
            merged[a] = merged.get(a, 0) + c
        clean = [(a, c) for a, c in merged.items() if c != 0]
        clean.sort(key=lambda kv: (str(kv[0]), repr(kv[0])))
        object.__setattr__(self, "terms", tuple(clean))
        object.__setattr__(self, "offset", int(offset))

    @classmethod
    def const(cls, value: int) -> "DimExpr":
        return cls({}, value)

    def __setattr__(self, key, value):
        raise AttributeError("DimExpr is immutable")

    def __reduce__(self):
        return (DimExpr, (list(self.terms), self.offset))

    @property
    def is_static(self) -> bool:
        return not self.terms

    @property
    def is_dynamic(self) -> bool:
        return bool(self.terms)

    @property
    def value(self) -> int:
        if self.terms:
            raise TilefishTypeError(f"{self} is symbolic: it has no value until a call binds its dimensions")
        return self.offset

    def folded(self):
        return self

    def _add(self, o: "DimExpr") -> "DimExpr":
        return DimExpr(list(self.terms) + list(o.terms), self.offset + o.offset)

    def _scale(self, k: int) -> "DimExpr":
        return DimExpr([(a, c * k) for a, c in self.terms], self.offset * k)

    def __eq__(self, o) -> bool:
        if isinstance(o, (Dim, DimExpr)) or _is_int(o):
            o = as_expr(o)
            return self.terms == o.terms and self.offset == o.offset
        return NotImplemented

    def __ne__(self, o) -> bool:
        r = self.__eq__(o)
        return r if r is NotImplemented else not r

    def __hash__(self) -> int:
        if self.is_static:
            return hash(self.offset)
        if self.offset == 0 and len(self.terms) == 1 and self.terms[0][1] == 1 and isinstance(self.terms[0][0], Dim):
            return hash(self.terms[0][0])
        return hash((self.terms, self.offset))

    def __str__(self) -> str:
        if self.is_static:
            return str(self.offset)
        out = ""
        for a, c in self.terms:
            body = str(a) if abs(c) == 1 else f"{abs(c)}*{a}"
            if not out:
                out = body if c > 0 else f"-{body}"
            else:
                out += f" + {body}" if c > 0 else f" - {body}"
        if self.offset:
            out += f" + {self.offset}" if self.offset > 0 else f" - {-self.offset}"
        return out

    def __repr__(self) -> str:
        return f"DimExpr({self})"


def _static_value(x) -> Optional[int]:
    if _is_int(x):
        return x
    if isinstance(x, Dim):
        return x._value
    if isinstance(x, DimExpr):
        return x.offset if x.is_static else None
    return None


def _operand(left, op: str, x) -> DimExpr:
    if isinstance(x, (Dim, DimExpr)) or _is_int(x):
        return as_expr(x)
    raise TilefishTypeError(f"({left}) {op} {x!r}: sizes combine with ints and other sizes only")


def as_expr(x: DimLike) -> DimExpr:
    if isinstance(x, DimExpr):
        return x
    if isinstance(x, Dim):
        return DimExpr({}, x._value) if x.is_static else DimExpr({x: 1}, 0)
    if _is_int(x):
        return DimExpr({}, x)
    raise TilefishTypeError(f"expected a Dim, a size expression or an int, got {x!r}")


def simplify(x: DimLike) -> DimLike:
    """The canonical spelling of a size inside a type: the ``Dim`` itself when it is one (a static one keeps its name and
    compares equal to its int), an int for any other static size, else the expression."""
    if isinstance(x, Dim):
        return x
    e = as_expr(x)
    if e.is_static:
        return e.offset
    if e.offset == 0 and len(e.terms) == 1 and e.terms[0][1] == 1 and isinstance(e.terms[0][0], Dim):
        return e.terms[0][0]
    return e


def _known_divisor(known: Optional[Mapping], key) -> int:
    if not known:
        return 1
    for k, d in known.items():
        if isinstance(k, _Cdiv):
            same = isinstance(key, _Cdiv) and k == key
        elif isinstance(key, _Cdiv):
            ke = as_expr(k)
            same = ke.offset == 0 and len(ke.terms) == 1 and ke.terms[0] == (key, 1)
        else:
            same = isinstance(k, (Dim, DimExpr)) and as_expr(k) == as_expr(key) and (not isinstance(k, Dim) or not isinstance(key, Dim) or k == key)
        if same and _is_int(d) and d > 0:
            return d
    return 1


def divisible(x: DimLike, n: int, known: Optional[Mapping] = None) -> bool:
    """Whether ``x`` is provably a multiple of ``n``: every term and the offset must be, each on its own."""
    if not _is_int(n) or n <= 0:
        raise TilefishTypeError(f"is_divisible_by: the divisor must be a positive int, got {n!r}")
    e = as_expr(x)
    if known and not e.is_static and _known_divisor(known, e) % n == 0:
        return True  # a fact about the whole expression
    if e.offset % n:
        return False
    for a, c in e.terms:
        unit = 1
        if isinstance(a, Dim):
            unit = a.divisible_by or 1
            if a.buckets is not None:
                g = 0
                for b in a.buckets:
                    g = gcd(g, b)
                unit = _lcm(unit, g)
        unit = _lcm(unit, _known_divisor(known, a))
        if (c * unit) % n:
            return False
    return True


def exact_ratio(x: DimLike, y: DimLike) -> Optional[int]:
    """The integer q with x == q * y identically, or None (different shapes, a non-integer ratio, a zero divisor)."""
    a, b = as_expr(x), as_expr(y)
    if b.is_static and b.offset == 0:
        return None
    if a.is_static and a.offset == 0:
        return 0
    if tuple(t for t, _ in a.terms) != tuple(t for t, _ in b.terms):
        return None
    q = None
    pairs = [(ca, cb) for (_, ca), (_, cb) in zip(a.terms, b.terms)]
    if a.offset or b.offset:
        pairs.append((a.offset, b.offset))
    for ca, cb in pairs:
        if cb == 0 or ca % cb:
            return None
        if q is None:
            q = ca // cb
        elif q != ca // cb:
            return None
    return q


def cdiv(x: DimLike, n: DimLike) -> DimLike:
    """ceil(x / n) as a size: an int for ints, exact when it folds (a static quotient, coefficients that divide, a constant ratio
    of two expressions), else a ``cdiv`` node."""
    dv = _static_value(n)
    if dv is not None and dv <= 0:
        raise TilefishTypeError(f"cdiv: the divisor must be positive, got {n!r}")
    if not (isinstance(n, (Dim, DimExpr)) or _is_int(n)):
        raise TilefishTypeError(f"cdiv: the divisor must be a size or a positive int, got {n!r}")
    if _is_int(x) and _is_int(n):
        return -(-x // n)
    e = as_expr(x)
    if dv is not None:
        if e.is_static:
            return -(-e.offset // dv)
        if e.offset % dv == 0 and all(c % dv == 0 for _, c in e.terms):
            return simplify(DimExpr([(a, c // dv) for a, c in e.terms], e.offset // dv))
        return DimExpr({_Cdiv(e, dv): 1}, 0)
    q = exact_ratio(e, n)
    if q is not None:
        return q
    return DimExpr({_Cdiv(e, as_expr(n)): 1}, 0)


def substitute(x: DimLike, mapping: Mapping) -> DimLike:
    e = as_expr(x)
    total = DimExpr.const(e.offset)
    for a, c in e.terms:
        if isinstance(a, Dim):
            repl = a
            for k, v in mapping.items():
                if isinstance(k, Dim) and k == a:
                    repl = v
                    break
            total = total._add(as_expr(repl)._scale(c))
        else:
            inner = cdiv(substitute(a.num, mapping), a.den if _is_int(a.den) else substitute(a.den, mapping))
            total = total._add(as_expr(inner)._scale(c))
    return simplify(total) if not total.is_static else total.offset


def symbols(x: DimLike) -> Tuple[Dim, ...]:
    out = []
    for a, _ in as_expr(x).terms:
        if isinstance(a, Dim):
            out.append(a)
        else:
            out.extend(symbols(a.num))
            if not _is_int(a.den):
                out.extend(symbols(a.den))
    return tuple(out)


def evaluate(x: DimLike, env: Dict[Dim, int]) -> Optional[int]:
    """The value of ``x`` with the dynamic dimensions bound by ``env``; None when one is unbound."""
    e = as_expr(x)
    total = e.offset
    for a, c in e.terms:
        if isinstance(a, Dim):
            v = env.get(a)
        else:
            num = evaluate(a.num, env)
            den = a.den if _is_int(a.den) else evaluate(a.den, env)
            v = None if num is None or den is None or den <= 0 else -(-num // den)
        if v is None:
            return None
        total += c * v
    return total


def describe_pair(a: DimLike, b: DimLike) -> Tuple[str, str]:
    """How to name two sizes in one message: by name when that tells them apart, else with their declarations spelled out."""
    sa, sb = str(a), str(b)
    if sa != sb:
        return sa, sb
    if isinstance(a, Dim) and isinstance(b, Dim):
        return repr(a), repr(b)

    def spelled(x, s):
        dims = sorted({repr(d) for d in symbols(x)})
        return f"{s} with {', '.join(dims)}" if dims else s

    return spelled(a, sa), spelled(b, sb)
