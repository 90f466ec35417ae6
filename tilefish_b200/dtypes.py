"""Element types and the BlockScaled quantization formats.

Names, fields and spellings follow the reference (python/src/tilefish/dtypes.py:14-232): ``bf16 f16 f32 i32 i64 u8 e4m3
e5m2 e2m1 ue8m0`` and ``BlockScaled(elem, scale, block, axis=-1, global_scale=None)``. The narrow float types are storage
only (``computable`` is False: cast first). Unlike the reference, a BlockScaled tensor can be produced and consumed at run
time here: ``format_name`` maps a BlockScaled type to the kernel format ("mxfp8", "mxfp4", "nvfp4") this backend implements.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .dims import DimLike, as_expr, cdiv, divisible, simplify
from .errors import TilefishDeclarationError, TilefishTypeError


@dataclass(frozen=True)
class DType:
    name: str
    bits: int
    kind: str  # "float", "int", "uint", "bool"
    exp_bits: int = 0
    man_bits: int = 0
    computable: bool = True

    @property
    def is_float(self) -> bool:
        return self.kind == "float"

    @property
    def is_int(self) -> bool:
        return self.kind in ("int", "uint")

    @property
    def signed(self) -> bool:
        return self.kind in ("float", "int") and self.name != "ue8m0"

    @property
    def elems_per_byte(self) -> int:
        return 8 // self.bits if self.bits < 8 else 1

    @property
    def itemsize(self) -> int:
        return max(1, self.bits // 8)

    @property
    def storage_bits(self) -> int:
        """Bits of the unit the type is stored in: a byte for the sub-byte types (two e2m1 per byte), else its own width."""
        return max(8, self.bits)

    # the dtypes are singletons: copies and pickles give the same object back, so `is` comparisons survive them
    def __copy__(self) -> "DType":
        return self

    def __deepcopy__(self, memo) -> "DType":
        return self

    def __reduce__(self):
        return (_dtype_by_name, (self.name,))

    def can_represent(self, other: "DType") -> bool:
        """Whether every value of ``other`` is a value of this type (a cast from ``other`` is then not a rounding point)."""
        if self is other:
            return True
        if self.is_float and other.is_float:
            return self.exp_bits >= other.exp_bits and self.man_bits >= other.man_bits and self.name != "ue8m0"
        if self.is_float and other.is_int:
            return self.man_bits + 1 >= other.bits
        if self.is_int and other.is_int:
            return self.bits > other.bits or (self.bits == other.bits and self.kind == other.kind)
        return False

    def is_narrowing_to(self, dst: "DType") -> bool:
        return not dst.can_represent(self)

    def __repr__(self) -> str:
        return self.name

    __str__ = __repr__


def _dtype_by_name(name: str) -> "DType":
    return ALL[name]


bf16 = DType("bf16", 16, "float", 8, 7)
f16 = DType("f16", 16, "float", 5, 10)
f32 = DType("f32", 32, "float", 8, 23)
i32 = DType("i32", 32, "int")
i64 = DType("i64", 64, "int")
u8 = DType("u8", 8, "uint")
e4m3 = DType("e4m3", 8, "float", 4, 3, computable=False)
e5m2 = DType("e5m2", 8, "float", 5, 2, computable=False)
e2m1 = DType("e2m1", 4, "float", 2, 1, computable=False)
ue8m0 = DType("ue8m0", 8, "float", 8, 0, computable=False)
bool_ = DType("bool", 8, "bool")

ALL = {d.name: d for d in (bf16, f16, f32, i32, i64, u8, e4m3, e5m2, e2m1, ue8m0, bool_)}
TORCH_NAMES = {"bf16": "bfloat16", "f16": "float16", "f32": "float32", "i32": "int32", "i64": "int64", "u8": "uint8", "bool": "bool"}


@dataclass(frozen=True)
class BlockScaled:
    """``block`` consecutive elements along ``axis`` share one ``scale``; an optional per-tensor ``global_scale``."""

    elem: DType
    scale: DType
    block: int
    axis: int = -1
    global_scale: Optional[DType] = None

    def __post_init__(self) -> None:
        if not isinstance(self.elem, DType) or not isinstance(self.scale, DType):
            raise TilefishDeclarationError("BlockScaled: elem and scale must be dtypes")
        if not isinstance(self.block, int) or self.block <= 0:
            raise TilefishDeclarationError(f"BlockScaled: block must be a positive int, got {self.block!r}")
        if self.block % self.elem.elems_per_byte:
            raise TilefishDeclarationError(f"BlockScaled: {self.elem} packs {self.elem.elems_per_byte} elements per byte, so block must be a multiple of "
                                           f"{self.elem.elems_per_byte}, got {self.block}")
        if self.global_scale is not None and not isinstance(self.global_scale, DType):
            raise TilefishDeclarationError("BlockScaled: global_scale must be a dtype or None")

    # the fields a tensor type shares with a plain dtype
    @property
    def name(self) -> str:
        return str(self)

    @property
    def bits(self) -> int:
        return self.elem.bits

    computable = False
    is_float = True
    is_int = False

    def normalized(self, rank: int) -> "BlockScaled":
        """The same format with ``axis`` counted from the front."""
        ax = self.axis + rank if self.axis < 0 else self.axis
        if not 0 <= ax < rank:
            raise TilefishTypeError(f"{self}: axis {self.axis} is out of range for a rank-{rank} tensor")
        return BlockScaled(self.elem, self.scale, self.block, ax, self.global_scale)

    def check_shape(self, shape: Tuple[DimLike, ...]) -> None:
        ax = self.normalized(len(shape)).axis
        if not divisible(shape[ax], self.block):
            size = shape[ax]
            hint = "" if as_expr(size).is_static else f"; declare the dimension with divisible_by={self.block} (or a multiple of it)"
            raise TilefishTypeError(f"{self}: axis {ax} has size {size}, which is not divisible by block={self.block}{hint}")

    def scale_shape(self, shape: Tuple[DimLike, ...]) -> Tuple[DimLike, ...]:
        self.check_shape(shape)
        ax = self.normalized(len(shape)).axis
        return tuple(simplify(cdiv(s, self.block)) if i == ax else s for i, s in enumerate(shape))

    @property
    def format_name(self) -> Optional[str]:
        """The kernel format this type maps to, or None when this backend has no kernels for it."""
        key = (self.elem.name, self.scale.name, self.block, self.global_scale.name if self.global_scale else None)
        return {("e4m3", "ue8m0", 32, None): "mxfp8", ("e2m1", "ue8m0", 32, None): "mxfp4", ("e2m1", "e4m3", 16, "f32"): "nvfp4"}.get(key)

    def __repr__(self) -> str:
        s = f"BlockScaled(elem={self.elem}, scale={self.scale}, block={self.block}, axis={self.axis}"
        if self.global_scale is not None:
            s += f", global_scale={self.global_scale}"
        return s + ")"

    def __str__(self) -> str:
        s = f"blockscaled({self.elem}, {self.scale}, {self.block}"
        if self.global_scale is not None:
            s += f", global_scale={self.global_scale}"
        return s + ")"


def same_format(a, b, rank: int) -> bool:
    """dtype equality as the call checker needs it: BlockScaled formats must match exactly, up to how ``axis`` is spelled."""
    if isinstance(a, BlockScaled) and isinstance(b, BlockScaled):
        return a.normalized(rank) == b.normalized(rank)
    return a is b or a == b
