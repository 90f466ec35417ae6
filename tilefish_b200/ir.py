"""The traced form of a kernel or graph body: typed SSA values, nodes and the graph with its text form.

The text form, the node attributes and the ``ops()`` / ``rounding_points()`` helpers follow the reference
(python/src/tilefish/ir.py:133-206, python/src/tilefish/trace.py:224-572), which its tests pin
(python/tests/test_graphs.py:51-119).
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

from .dtypes import DType
from .types import TensorType


class Scalar:
    """A python scalar or ``const`` that adopted the dtype of the tensor it was combined with."""

    __slots__ = ("value", "dtype", "name")

    def __init__(self, value, dtype: DType, name: Optional[str] = None) -> None:
        self.value, self.dtype, self.name = value, dtype, name

    def __repr__(self) -> str:
        return f"{self.name}:{self.dtype}" if self.name else f"{self.value!r}:{self.dtype}"

    def __eq__(self, o) -> bool:
        if not isinstance(o, Scalar):
            return NotImplemented
        return (self.value, self.dtype, self.name) == (o.value, o.dtype, o.name) and type(self.value) is type(o.value)

    def __hash__(self) -> int:
        return hash((self.value, str(self.dtype), self.name))


class Value:
    """An SSA value of a trace. Arithmetic and methods on it append nodes to the active trace (see trace.py)."""

    __slots__ = ("type", "ref", "producer", "index", "is_param", "access", "name", "consumed", "_ctx")

    def __init__(self, type_: TensorType, ref: str, ctx, *, producer=None, index: int = 0, is_param: bool = False, access: str = "in",
                 name: Optional[str] = None) -> None:
        self.type = type_
        self.ref = ref
        self.producer = producer
        self.index = index
        self.is_param = is_param
        self.access = access
        self.name = name
        self.consumed = False
        self._ctx = ctx

    def __repr__(self) -> str:
        return f"Value({self.ref}: {self.type!r})"

    __hash__ = object.__hash__


def _fmt_attr(v: Any) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (tuple, list)):
        return "(" + ", ".join(_fmt_attr(x) for x in v) + ("," if len(v) == 1 else "") + ")"
    if isinstance(v, dict):
        return "{" + ", ".join(f"{k}: {_fmt_attr(x)}" for k, x in v.items()) + "}"
    return str(v)


class Node:
    __slots__ = ("op", "inputs", "outputs", "attrs", "callee")

    def __init__(self, op: str, inputs: Tuple[Any, ...], attrs: Dict[str, Any]) -> None:
        self.callee = None  # the declared operator a call node calls
        self.op = op
        self.inputs = tuple(inputs)
        self.outputs: Tuple[Value, ...] = ()
        self.attrs = attrs

    @property
    def output_types(self) -> Tuple[TensorType, ...]:
        return tuple(o.type for o in self.outputs)

    @property
    def is_rounding_point(self) -> bool:
        return self.op == "cast" and bool(self.attrs.get("rounding"))

    def __str__(self) -> str:
        outs = ", ".join(f"{o.ref}: {o.type!r}" for o in self.outputs)
        args = ", ".join(i.ref if isinstance(i, Value) else repr(i) for i in self.inputs)
        s = f"{outs} = {self.op}({args})"
        if self.attrs:
            s += " {" + ", ".join(f"{k}={_fmt_attr(v)}" for k, v in self.attrs.items()) + "}"
        if self.is_rounding_point:
            s += "  # rounding point"
        return s

    __repr__ = __str__


class Requirement:
    """A precondition on a symbolic size found while type-checking a call: ``dim`` must be a multiple of ``divisor`` because
    ``origin`` (an operator's argument) declares so. The host that launches the graph checks it against the actual sizes
    (reference: python/src/tilefish/ir.py:34-50)."""

    __slots__ = ("dim", "divisor", "origin")

    def __init__(self, dim, divisor: int, origin: str) -> None:
        from .dims import as_expr

        object.__setattr__(self, "dim", as_expr(dim))
        object.__setattr__(self, "divisor", int(divisor))
        object.__setattr__(self, "origin", origin)

    def __setattr__(self, key, value):
        raise AttributeError("Requirement is immutable")

    def __reduce__(self):
        return (Requirement, (self.dim, self.divisor, self.origin))

    def __eq__(self, o) -> bool:
        return isinstance(o, Requirement) and (self.dim, self.divisor, self.origin) == (o.dim, o.divisor, o.origin)

    def __hash__(self) -> int:
        return hash((self.dim, self.divisor, self.origin))

    def __str__(self) -> str:
        e = self.dim
        atom = e.offset == 0 and len(e.terms) == 1 and e.terms[0][1] == 1
        dim = str(e) if atom else f"({e})"  # % binds tighter than +
        return f"{dim} % {self.divisor} == 0  (required by {self.origin})"

    def __repr__(self) -> str:
        return f"Requirement({self.dim}, {self.divisor}, {self.origin!r})"


class BucketRequirement:
    """A symbolic size must take one of ``buckets`` because ``origin`` (an operator's argument) is declared over those buckets and the
    caller's declaration does not prove it; checked against the actual sizes by the host (reference: python/src/tilefish/ir.py)."""

    __slots__ = ("dim", "buckets", "origin")

    def __init__(self, dim, buckets, origin: str) -> None:
        from .dims import as_expr

        object.__setattr__(self, "dim", as_expr(dim))
        object.__setattr__(self, "buckets", tuple(buckets))
        object.__setattr__(self, "origin", origin)

    def __setattr__(self, key, value):
        raise AttributeError("BucketRequirement is immutable")

    def __reduce__(self):
        return (BucketRequirement, (self.dim, self.buckets, self.origin))

    def __eq__(self, o) -> bool:
        return isinstance(o, BucketRequirement) and (self.dim, self.buckets, self.origin) == (o.dim, o.buckets, o.origin)

    def __hash__(self) -> int:
        return hash((self.dim, self.buckets, self.origin))

    def __str__(self) -> str:
        return f"{self.dim} in {list(self.buckets)}  (required by {self.origin})"

    def __repr__(self) -> str:
        return f"BucketRequirement({self.dim}, {list(self.buckets)}, {self.origin!r})"


class Graph:
    def __init__(self, kind: str, name: str, inputs: List[Value], consts: List[Tuple[str, DType, Any]], nodes: List[Node], outputs: List[Value],
                 finals: Dict[str, Value], requirements: Tuple[Any, ...] = ()) -> None:
        self.kind = kind
        self.name = name
        self.inputs = tuple(inputs)
        self.consts = tuple(consts)
        self.nodes = tuple(nodes)
        self.outputs = tuple(outputs)
        self.finals = dict(finals)
        self.requirements = tuple(requirements)

    def ops(self) -> List[str]:
        return [n.op for n in self.nodes]

    def rounding_points(self) -> List[Node]:
        return [n for n in self.nodes if n.is_rounding_point]

    @property
    def symbols(self):
        from .dims import symbols

        seen = []
        for v in self.inputs:
            for s in v.type.shape:
                for d in symbols(s):
                    if d not in seen:
                        seen.append(d)
        return tuple(seen)

    def __str__(self) -> str:
        params = []
        for v in self.inputs:
            p = f"{v.ref}: {v.type!r}"
            if v.access != "in":
                p += f" [{v.access}]"
            params.append(p)
        for name, dtype, default in self.consts:
            params.append(f"{name}: const[{dtype}] = {default!r}")
        rets = ", ".join(repr(o.type) for o in self.outputs)
        lines = [f"{self.kind} {self.name}({', '.join(params)}) -> ({rets}):"]
        lines += [f"  {n}" for n in self.nodes]
        lines.append("  return" + (" " + ", ".join(o.ref for o in self.outputs) if self.outputs else ""))
        for target, v in self.finals.items():
            lines.append(f"  final {target} = {v.ref}")
        for r in self.requirements:
            lines.append(f"  requires {r}")
        return "\n".join(lines)
