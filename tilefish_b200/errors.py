"""Exception types. Names, bases and the ``kind``/``arg`` attributes follow the reference's python/src/tilefish/errors.py:8-95
so that code catching tilefish's errors keeps working against this backend."""

from __future__ import annotations


class TilefishError(Exception):
    """Base class of every error raised by this package."""


class TilefishTypeError(TilefishError, TypeError):
    """A type, shape, dtype or divisibility rule was violated."""


class TilefishDeclarationError(TilefishError, ValueError):
    """A dimension, dtype, signature or decorator was declared incorrectly."""


class TilefishSpecError(TilefishError, ValueError):
    """A declaration cannot be given a kernel of this backend."""


class TilefishPlanError(TilefishError, ValueError):
    """A graph cannot be turned into a launch plan."""


class TilefishLoweringError(TilefishError, ValueError):
    """A kernel body matches none of the hand-written sm_100a kernels (this backend generates no code)."""

    def __init__(self, message: str, *, rule: "str | None" = None, causes=()) -> None:
        super().__init__(message)
        self.rule = rule
        self.causes = tuple(causes)


class TilefishAttributeError(TilefishError, AttributeError):
    """An attribute or method that traced values do not have."""


class TilefishBuildError(TilefishError, RuntimeError):
    """The kernel library could not be built."""


class TilefishRuntimeError(TilefishError, RuntimeError):
    """An operator cannot be run: no CUDA device, the kernel library is missing, a CUDA call failed, unknown mode."""


class TilefishManifestError(TilefishRuntimeError):
    """An exported directory cannot be replayed: a file is missing or malformed, or a digest does not match its pin."""


class TilefishPreconditionError(TilefishRuntimeError):
    """An argument violates a precondition of the kernel it would run on.

    ``kind`` names the rule ("dtype", "rank", "shape", "static_size", "divisible", "bucket", "pointer_alignment",
    "contiguous", "device", "alias", ...); ``arg`` is the argument it is about, when there is one.
    """

    def __init__(self, message: str, *, kind: str, arg: "str | None" = None) -> None:
        super().__init__(message)
        self.kind = kind
        self.arg = arg
