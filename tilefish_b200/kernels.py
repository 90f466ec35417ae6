"""Tensor-level entry to the sm_100a kernels: torch tensors in, C ABI calls out.

torch is used for allocation, the current stream and nothing else. Every precondition the kernels rely on is checked
here before anything is enqueued (dtype, rank, contiguity, device, 16-byte alignment, divisibility), the way the
reference checks a launch (python/src/tilefish/_launch.py:263-315, :433-500); failures raise
``TilefishPreconditionError(kind=..., arg=...)``. The shared library re-validates cheaply and returns a status.
"""

from __future__ import annotations

import ctypes
from typing import Optional

from . import _native as N
from .errors import TilefishPreconditionError, TilefishRuntimeError

FORMATS = {"mxfp8": N.FMT_MXFP8, "mxfp4": N.FMT_MXFP4, "nvfp4": N.FMT_NVFP4}
BLOCK = {"mxfp8": 32, "mxfp4": 32, "nvfp4": 16}
ELEMS_PER_BYTE = {"mxfp8": 1, "mxfp4": 2, "nvfp4": 2}
EPILOGUES = {"none": N.EPI_NONE, "silu_gate": N.EPI_SILU_GATE, "residual": N.EPI_RESIDUAL}


def _torch():
    import torch

    return torch


def _pre(cond: bool, msg: str, kind: str, arg: Optional[str] = None) -> None:
    if not cond:
        raise TilefishPreconditionError(msg, kind=kind, arg=arg)


def _check(t, name: str, dtype, rank: Optional[int] = None, device=None, align: int = 16) -> None:
    torch = _torch()
    _pre(isinstance(t, torch.Tensor), f"{name}: expected a torch tensor, got {type(t).__name__}", "dtype", name)
    _pre(t.is_cuda, f"{name}: the tensor is on {t.device}; this backend runs on CUDA only (no CPU fallback)", "device", name)
    _pre(t.dtype == dtype, f"{name}: expected {dtype}, got {t.dtype}", "dtype", name)
    if rank is not None:
        _pre(t.dim() == rank, f"{name}: expected rank {rank}, got {t.dim()}", "rank", name)
    if device is not None:
        _pre(t.device == device, f"{name}: on {t.device}, the other arguments are on {device}", "device", name)
    _pre(t.numel() == 0 or t.data_ptr() % align == 0, f"{name}: the data pointer is not {align}-byte aligned", "pointer_alignment", name)


def _dense(t, name: str) -> None:
    _pre(t.is_contiguous(), f"{name}: must be contiguous (strides {tuple(t.stride())})", "contiguous", name)


def _stream(stream) -> int:
    """The raw handle of ``stream`` (None: torch's current stream). Results and scratch tensors these wrappers allocate come from torch's
    caching allocator, which orders reuse by torch's CURRENT stream: a launch on another stream must not outlive them unnoticed, so a
    ``stream=`` that is not the current one is refused unless it is a ``torch.cuda.Stream`` the caller made current
    (``with torch.cuda.stream(s): ...``) or the caller passes every output and workspace itself."""
    torch = _torch()
    current = torch.cuda.current_stream().cuda_stream
    if stream is None:
        return current
    handle = getattr(stream, "cuda_stream", stream)
    if handle != current:
        raise TilefishPreconditionError("stream= is not torch's current stream: tensors allocated here would be recycled in the current stream's order while the "
                                        "launch runs on another. Make the stream current (with torch.cuda.stream(s)) and call without stream=", kind="argument", arg="stream")
    return handle


class BlockScaledTensor:
    """Run-time value of a ``Tensor[rows, K, BlockScaled(...)]``: element codes, scale bytes and (nvfp4) the f32 global scale.

    ``codes``   uint8 [rows, K] (mxfp8) or [rows, K/2] (fp4: element 2i in bits 0-3 of byte i)
    ``scales``  uint8, flat; ``layout`` is "swizzled" (the sm_100 MMA operand layout, what the GEMM consumes) or "plain" ([rows, K/block])
    ``global_scale``  float32 [1] on the device for nvfp4, else None
    """

    __slots__ = ("fmt", "shape", "codes", "scales", "global_scale", "layout", "gs_rows")

    def __init__(self, fmt: str, shape, codes, scales, global_scale=None, layout: str = "swizzled", gs_rows: int = 0) -> None:
        if fmt not in FORMATS:
            raise TilefishPreconditionError(f"unknown block-scaled format {fmt!r}", kind="dtype")
        self.fmt = fmt
        self.shape = tuple(int(s) for s in shape)
        self.codes = codes
        self.scales = scales
        self.global_scale = global_scale
        self.layout = layout
        self.gs_rows = gs_rows  # nvfp4: 0 = one global scale; else global_scale[i] belongs to rows [i * gs_rows, (i + 1) * gs_rows)

    @property
    def device(self):
        return self.codes.device

    @property
    def block(self) -> int:
        return BLOCK[self.fmt]

    def plain_scales(self):
        """The scale bytes as a [rows, K/block] uint8 tensor (un-swizzled on the device when needed)."""
        rows, k = self.shape
        cols = k // self.block
        if self.layout == "plain":
            return self.scales.view(rows, cols)
        return unswizzle_scales(self.scales, rows, cols)

    def nbytes(self) -> int:
        n = self.codes.numel() + self.scales.numel()
        return n + (4 if self.global_scale is not None else 0)

    def __repr__(self) -> str:
        return f"BlockScaledTensor({self.fmt}, shape={self.shape}, scales={self.layout})"


def scale_bytes(fmt: str, rows: int, k: int, layout: str = "swizzled") -> int:
    return N.scale_bytes(FORMATS[fmt], rows, k, N.SCALES_SWIZZLED if layout == "swizzled" else N.SCALES_PLAIN)


def nvfp4_global_scale(x, *, out=None, stream=None):
    """float32 [1] on the device: max|x| / 2688, computed in stream order."""
    torch = _torch()
    _check(x, "x", torch.bfloat16, 2)
    _pre(x.stride(1) == 1 and x.stride(0) % 16 == 0 and x.shape[1] % 16 == 0, "x: rows must be dense, K and the row stride multiples of 16", "contiguous", "x")
    _pre(x.numel() == 0 or x.data_ptr() % 32 == 0, "x: the data pointer is not 32-byte aligned", "pointer_alignment", "x")
    if out is None:
        out = torch.empty(1, dtype=torch.float32, device=x.device)
    m, k = x.shape
    N.check(N.load().tf_nvfp4_global_scale(x.data_ptr(), m, k, x.stride(0), out.data_ptr(), _stream(stream)), "tf_nvfp4_global_scale")
    return out


def quantize(x, fmt: str, *, layout: str = "swizzled", global_scale=None, amax=None, out: Optional[BlockScaledTensor] = None,
             stream=None) -> BlockScaledTensor:
    """BlockScaled quantization of a bf16 [M, K] tensor along K.

    nvfp4 needs the tensor's global scale: given as ``global_scale`` (float32 [1] on the device), derived inside the kernel
    from ``amax`` (float32 [1] holding max|x|, e.g. the ``amax_out`` of the producing kernel), or computed by an extra pass.
    """
    torch = _torch()
    _pre(fmt in FORMATS, f"unknown block-scaled format {fmt!r}", "dtype", "fmt")
    _pre(layout in ("swizzled", "plain"), f"unknown scale layout {layout!r}", "argument", "layout")
    _check(x, "x", torch.bfloat16, 2)
    m, k = x.shape
    _pre(x.stride(1) == 1 and (m <= 1 or (x.stride(0) >= k and x.stride(0) % 16 == 0)), "x: rows must be dense with a row stride that is a multiple of 16", "contiguous", "x")
    _pre(k % 32 == 0 and k > 0, f"x: K={k} is not a multiple of 32", "divisible", "x")
    _pre(m == 0 or x.data_ptr() % 32 == 0, "x: the data pointer is not 32-byte aligned (the quantizer uses 256-bit loads)", "pointer_alignment", "x")
    ldx = x.stride(0) if m > 1 else k
    lay = N.SCALES_SWIZZLED if layout == "swizzled" else N.SCALES_PLAIN
    if out is not None:  # preallocated result (a plan's arena): same format, shape and layout
        _pre(out.fmt == fmt and out.shape == (m, k) and out.layout == layout, f"out: expected a {fmt} {layout} tensor of shape {(m, k)}", "shape", "out")
        codes, scales = out.codes, out.scales
    else:
        codes = torch.empty((m, k // ELEMS_PER_BYTE[fmt]), dtype=torch.uint8, device=x.device)
        scales = torch.empty(N.scale_bytes(FORMATS[fmt], m, k, lay), dtype=torch.uint8, device=x.device)
    s = _stream(stream)
    lib = N.load()
    gs = None
    if m == 0:  # nothing to launch (an empty tensor has no data pointer)
        if fmt == "nvfp4":
            gs = global_scale if global_scale is not None else torch.zeros(1, dtype=torch.float32, device=x.device)
        return BlockScaledTensor(fmt, (m, k), codes, scales, gs, layout)
    if fmt == "nvfp4" and amax is not None:
        _check(amax, "amax", torch.float32, None, x.device, align=4)
        _pre(amax.numel() == 1 and global_scale is None, "amax: expected one element and no global_scale", "shape", "amax")
        gs = out.global_scale if out is not None and out.global_scale is not None else torch.empty(1, dtype=torch.float32, device=x.device)
        N.check(lib.tf_quantize_nvfp4_from_amax(x.data_ptr(), m, k, ldx, codes.data_ptr(), scales.data_ptr(), lay, amax.data_ptr(), gs.data_ptr(), s),
                "tf_quantize_nvfp4_from_amax")
    elif fmt == "nvfp4":
        if global_scale is None:
            gs = nvfp4_global_scale(x, out=out.global_scale if out is not None else None, stream=stream)
        else:
            _check(global_scale, "global_scale", torch.float32, None, x.device, align=4)
            _pre(global_scale.numel() == 1, "global_scale: expected one element", "shape", "global_scale")
            gs = global_scale
        N.check(lib.tf_quantize_nvfp4(x.data_ptr(), m, k, ldx, codes.data_ptr(), scales.data_ptr(), lay, gs.data_ptr(), s), "tf_quantize_nvfp4")
    elif fmt == "mxfp8":
        N.check(lib.tf_quantize_mxfp8(x.data_ptr(), m, k, ldx, codes.data_ptr(), scales.data_ptr(), lay, s), "tf_quantize_mxfp8")
    else:
        N.check(lib.tf_quantize_mxfp4(x.data_ptr(), m, k, ldx, codes.data_ptr(), scales.data_ptr(), lay, s), "tf_quantize_mxfp4")
    return BlockScaledTensor(fmt, (m, k), codes, scales, gs, layout)


def swizzle_scales(plain, *, stream=None):
    torch = _torch()
    _check(plain, "plain", torch.uint8, 2)
    _dense(plain, "plain")
    rows, cols = plain.shape
    out = torch.empty(((rows + 127) // 128) * ((cols + 3) // 4) * 512, dtype=torch.uint8, device=plain.device)
    N.check(N.load().tf_swizzle_scales(plain.data_ptr(), rows, cols, out.data_ptr(), _stream(stream)), "tf_swizzle_scales")
    return out


def unswizzle_scales(swizzled, rows: int, cols: int, *, stream=None):
    torch = _torch()
    _check(swizzled, "swizzled", torch.uint8, 1)
    need = ((rows + 127) // 128) * ((cols + 3) // 4) * 512
    _pre(swizzled.numel() >= need, f"swizzled: {swizzled.numel()} bytes, {need} needed for [{rows}, {cols}]", "shape", "swizzled")
    out = torch.empty((rows, cols), dtype=torch.uint8, device=swizzled.device)
    N.check(N.load().tf_unswizzle_scales(swizzled.data_ptr(), rows, cols, out.data_ptr(), _stream(stream)), "tf_unswizzle_scales")
    return out


def residual_add_rmsnorm(x, residual, w, eps: float = 1e-6, *, out=None, quantize_to: Optional[str] = None, want_bf16: bool = True,
                         q_global_scale=None, amax_out=None, q_out: Optional[BlockScaledTensor] = None, stream=None):
    """``residual += f32(x)`` in place; returns bf16 ``rmsnorm(residual) * w`` and/or its BlockScaled quantization.

    Returns ``out`` (bf16), or ``(out, q)`` when ``quantize_to`` is given (``out`` is None with ``want_bf16=False``).
    ``amax_out`` (float32 [1], zeroed by the caller) receives max|out| through an atomic max.
    """
    torch = _torch()
    _check(x, "x", torch.bfloat16, 2)
    _check(residual, "residual", torch.float32, 2, x.device)
    _check(w, "w", torch.bfloat16, 1, x.device)
    for t, n in ((x, "x"), (residual, "residual"), (w, "w")):
        _dense(t, n)
    m, d = x.shape
    _pre(tuple(residual.shape) == (m, d), f"residual: shape {tuple(residual.shape)}, expected {(m, d)}", "shape", "residual")
    _pre(tuple(w.shape) == (d,), f"w: shape {tuple(w.shape)}, expected {(d,)}", "shape", "w")
    _pre(d % 8 == 0, f"x: D={d} is not a multiple of 8", "divisible", "x")
    if want_bf16:
        if out is None:
            out = torch.empty((m, d), dtype=torch.bfloat16, device=x.device)
        else:
            _check(out, "out", torch.bfloat16, 2, x.device)
            _dense(out, "out")
            _pre(tuple(out.shape) == (m, d), "out: wrong shape", "shape", "out")
            _pre(out.data_ptr() != x.data_ptr(), "out aliases x", "alias", "out")
    else:
        _pre(quantize_to is not None, "nothing to compute: want_bf16=False without quantize_to", "argument")
        out = None
    q = None
    qfmt, qc, qs, qg = -1, None, None, None
    if quantize_to is not None:
        _pre(quantize_to in FORMATS, f"unknown block-scaled format {quantize_to!r}", "dtype", "quantize_to")
        _pre(d % 32 == 0, f"x: D={d} is not a multiple of 32 (needed to quantize)", "divisible", "x")
        qfmt = FORMATS[quantize_to]
        if q_out is not None:
            _pre(q_out.fmt == quantize_to and q_out.shape == (m, d) and q_out.layout == "swizzled", "q_out: wrong format or shape", "shape", "q_out")
            codes, scales = q_out.codes, q_out.scales
        else:
            codes = torch.empty((m, d // ELEMS_PER_BYTE[quantize_to]), dtype=torch.uint8, device=x.device)
            scales = torch.empty(N.scale_bytes(qfmt, m, d, N.SCALES_SWIZZLED), dtype=torch.uint8, device=x.device)
        if quantize_to == "nvfp4":
            _pre(q_global_scale is not None, "nvfp4 output needs q_global_scale (a float32 [1] device tensor)", "argument", "q_global_scale")
            _check(q_global_scale, "q_global_scale", torch.float32, None, x.device, align=4)
            qg = q_global_scale
        q = BlockScaledTensor(quantize_to, (m, d), codes, scales, qg, "swizzled")
        qc, qs = codes.data_ptr(), scales.data_ptr()
    N.check(
        N.load().tf_residual_add_rmsnorm(x.data_ptr(), residual.data_ptr(), w.data_ptr(), out.data_ptr() if out is not None else None, m, d,
                                         float(eps), qfmt, qc, qs, N.SCALES_SWIZZLED, qg.data_ptr() if qg is not None else None,
                                         _amax_ptr(amax_out, x.device), _stream(stream)),
        "tf_residual_add_rmsnorm",
    )
    return out if q is None else (out, q)


def _amax_ptr(amax_out, device):
    if amax_out is None:
        return None
    _check(amax_out, "amax_out", _torch().float32, None, device, align=4)
    _pre(amax_out.numel() == 1, "amax_out: expected one element", "shape", "amax_out")
    return amax_out.data_ptr()


def silu_gate(t, up=None, *, out=None, stream=None):
    """bf16 [M, F] = silu(gate) * up. ``silu_gate(t)`` takes the column halves of a bf16 [M, 2F] tensor; ``silu_gate(gate, up)``
    two bf16 [M, F] tensors (rows dense, row strides multiples of 8: strided views of a wider tensor are fine)."""
    torch = _torch()
    _check(t, "t", torch.bfloat16, 2)
    if up is None:
        m, two_f = t.shape
        _pre(two_f % 16 == 0, f"t: {two_f} columns; the halves must be multiples of 8", "divisible", "t")
        f = two_f // 2
        gate, up = t[:, :f], t[:, f:]
    else:
        gate = t
        _check(up, "up", torch.bfloat16, 2, gate.device)
        m, f = gate.shape
        _pre(tuple(up.shape) == (m, f), f"up: shape {tuple(up.shape)}, expected {(m, f)}", "shape", "up")
        _pre(f % 8 == 0, f"gate: F={f} is not a multiple of 8", "divisible", "gate")
    for v, nm in ((gate, "gate"), (up, "up")):
        _pre(v.stride(1) == 1 and (m <= 1 or v.stride(0) % 8 == 0), f"{nm}: rows must be dense with a row stride that is a multiple of 8", "contiguous", nm)
    if out is None:
        out = torch.empty((m, f), dtype=torch.bfloat16, device=t.device)
    else:
        _check(out, "out", torch.bfloat16, 2, t.device)
        _dense(out, "out")
        _pre(tuple(out.shape) == (m, f), "out: wrong shape", "shape", "out")
    if m == 0:
        return out
    ldg = gate.stride(0) if m > 1 else f
    ldu = up.stride(0) if m > 1 else f
    N.check(N.load().tf_silu_gate(gate.data_ptr(), up.data_ptr(), m, f, ldg, ldu, out.data_ptr(), f, _stream(stream)), "tf_silu_gate")
    return out


def set_programmatic_launch(enabled: bool) -> None:
    """Process-wide: launch this library's kernels as programmatic dependents (each may be scheduled while its predecessor on
    the stream drains, and waits for it before touching memory). Same results; hides launch latency in chains of short kernels."""
    N.check(N.load().tf_set_programmatic_launch(1 if enabled else 0), "tf_set_programmatic_launch")


def gemm_workspace_bytes(m: int, n: int, k: int, fmt: str, epilogue: str = "none") -> int:
    return int(N.load().tf_gemm_workspace_bytes(m, n, k, FORMATS[fmt], EPILOGUES[epilogue]))


def gemm_blockscaled(a: BlockScaledTensor, b: BlockScaledTensor, *, epilogue: str = "none", out=None, residual=None, amax_out=None,
                     quantize_out: bool = False, q_out: Optional[BlockScaledTensor] = None, want_bf16: bool = True, workspace=None, stream=None):
    """bf16 [M, N] = deq(a)[M, K] @ deq(b)[N, K]^T on tcgen05 block-scaled MMA, f32 accumulate.

    ``epilogue="silu_gate"``: b has 2N rows (gate rows then up rows); the result is silu(gate) * up, [M, N].
    ``epilogue="residual"``: also ``residual[M, N] += f32(out)`` (f32, in place).
    ``quantize_out=True`` (MX formats): the epilogue also quantizes the result in the operands' format, byte for byte what
    ``quantize(out, fmt)`` gives, and the call returns ``(out, q)``; with ``want_bf16=False`` the bf16 copy is not written
    (``out`` is None). ``q_out`` supplies preallocated storage for it.
    """
    torch = _torch()
    _pre(isinstance(a, BlockScaledTensor) and isinstance(b, BlockScaledTensor), "a and b must be BlockScaledTensor", "dtype")
    _pre(a.fmt == b.fmt, f"a is {a.fmt} but b is {b.fmt}: block-scaled formats must match exactly", "dtype", "b")
    _pre(a.layout == "swizzled" and b.layout == "swizzled", "the GEMM consumes swizzled scales", "contiguous")
    _pre(epilogue in EPILOGUES, f"unknown epilogue {epilogue!r}", "argument", "epilogue")
    m, k = a.shape
    nb, kb = b.shape
    _pre(k == kb, f"K differs: a is {a.shape}, b is {b.shape}", "shape", "b")
    n = nb // 2 if epilogue == "silu_gate" else nb
    if epilogue == "silu_gate":
        _pre(nb % 256 == 0, f"silu_gate: b has {nb} rows; each half must be a multiple of 128", "divisible", "b")
    _pre(a.device == b.device, "a and b are on different devices", "device", "b")
    for t, nm in ((a.codes, "a.codes"), (b.codes, "b.codes"), (a.scales, "a.scales"), (b.scales, "b.scales")):
        _check(t, nm, torch.uint8, None, a.device)
        _dense(t, nm)
    if a.fmt == "nvfp4":
        _pre(a.global_scale is not None and b.global_scale is not None, "nvfp4 operands need their global scales", "argument")
    quantize_out = quantize_out or q_out is not None
    q = None
    if quantize_out:
        _pre(a.fmt != "nvfp4", "a quantized gemm output needs the tensor's global scale first: not available for nvfp4", "dtype", "quantize_out")
        _pre(epilogue != "residual" and n % 32 == 0, "quantize_out needs n % 32 == 0 and is not available with the residual epilogue", "divisible", "quantize_out")
        if q_out is not None:
            _pre(q_out.fmt == a.fmt and q_out.shape == (m, n) and q_out.layout == "swizzled", "q_out: wrong format or shape", "shape", "q_out")
            q = q_out
        else:
            q = BlockScaledTensor(a.fmt, (m, n), torch.empty((m, n // ELEMS_PER_BYTE[a.fmt]), dtype=torch.uint8, device=a.device),
                                  torch.empty(N.scale_bytes(FORMATS[a.fmt], m, n, N.SCALES_SWIZZLED), dtype=torch.uint8, device=a.device), None, "swizzled")
    else:
        _pre(want_bf16, "nothing to compute: want_bf16=False without quantize_out", "argument")
    if not want_bf16:
        out = None
    elif out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    else:
        _check(out, "out", torch.bfloat16, 2, a.device)
        _pre(tuple(out.shape) == (m, n) and out.stride(1) == 1 and (m <= 1 or out.stride(0) % 8 == 0), "out: wrong shape or strides", "shape", "out")
    ldo = out.stride(0) if (out is not None and m > 1) else n
    res_ptr = None
    if epilogue == "residual":
        _pre(residual is not None, "epilogue='residual' needs the f32 residual", "argument", "residual")
        _check(residual, "residual", torch.float32, 2, a.device)
        _dense(residual, "residual")
        _pre(tuple(residual.shape) == (m, n), "residual: wrong shape", "shape", "residual")
        res_ptr = residual.data_ptr()
    need = gemm_workspace_bytes(m, n, k, a.fmt, epilogue)
    ws_ptr, ws_bytes = None, 0
    if need > 0:
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
        _pre(workspace.numel() * workspace.element_size() >= need, f"workspace: {need} bytes needed", "workspace", "workspace")
        ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    N.check(
        N.load().tf_gemm_blockscaled(
            a.codes.data_ptr(), a.scales.data_ptr(), a.global_scale.data_ptr() if a.global_scale is not None else None,
            b.codes.data_ptr(), b.scales.data_ptr(), b.global_scale.data_ptr() if b.global_scale is not None else None,
            out.data_ptr() if out is not None else None, ldo, m, n, k, FORMATS[a.fmt], EPILOGUES[epilogue], res_ptr, _amax_ptr(amax_out, a.device),
            q.codes.data_ptr() if q is not None and m > 0 else None, q.scales.data_ptr() if q is not None and m > 0 else None, a.gs_rows, ws_ptr, ws_bytes,
            _stream(stream)),
        "tf_gemm_blockscaled",
    )
    return (out, q) if quantize_out else out


def gemm_blockscaled_scatter(a: BlockScaledTensor, b: BlockScaledTensor, out_ptrs, rows_per_owner: int, ldo: int, *, stream=None) -> None:
    """``deq(a) @ deq(b)^T`` whose row block i (``rows_per_owner`` rows) is written, as bf16 with row stride ``ldo``, to the device
    address ``out_ptrs[i]``: this GPU's memory or a peer's (plain stores from the epilogue). The tensor-parallel second GEMM uses
    it to deliver each rank's rows of its partial result to that rank. Shapes the GEMM would split along K are refused
    (``gemm_workspace_bytes(...) > 0``)."""
    torch = _torch()
    _pre(isinstance(a, BlockScaledTensor) and isinstance(b, BlockScaledTensor), "a and b must be BlockScaledTensor", "dtype")
    _pre(a.fmt == b.fmt, f"a is {a.fmt} but b is {b.fmt}: block-scaled formats must match exactly", "dtype", "b")
    _pre(a.layout == "swizzled" and b.layout == "swizzled", "the GEMM consumes swizzled scales", "contiguous")
    m, k = a.shape
    n, kb = b.shape
    _pre(k == kb, f"K differs: a is {a.shape}, b is {b.shape}", "shape", "b")
    owners = len(out_ptrs)
    _pre(1 <= owners <= 8 and rows_per_owner > 0 and rows_per_owner % 128 == 0 and m == owners * rows_per_owner,
         f"M={m} must be {owners} destinations x rows_per_owner={rows_per_owner} (a multiple of 128)", "divisible", "out_ptrs")
    _pre(ldo >= n and ldo % 8 == 0 and n % 8 == 0, "n and ldo must be multiples of 8 with ldo >= n", "alignment", "ldo")
    _pre(all(int(p) and int(p) % 16 == 0 for p in out_ptrs), "every destination must be a 16-byte aligned device address", "alignment", "out_ptrs")
    _pre(gemm_workspace_bytes(m, n, k, a.fmt, "none") == 0, "this shape is split along K: it has no scattered output", "shape", "a")
    for t, nm in ((a.codes, "a.codes"), (b.codes, "b.codes"), (a.scales, "a.scales"), (b.scales, "b.scales")):
        _check(t, nm, torch.uint8, None, a.device)
        _dense(t, nm)
    if a.fmt == "nvfp4":
        _pre(a.global_scale is not None and b.global_scale is not None, "nvfp4 operands need their global scales", "argument")
    ptrs = (ctypes.c_uint64 * owners)(*[int(p) for p in out_ptrs])
    N.check(
        N.load().tf_gemm_blockscaled_scatter(
            a.codes.data_ptr(), a.scales.data_ptr(), a.global_scale.data_ptr() if a.global_scale is not None else None,
            b.codes.data_ptr(), b.scales.data_ptr(), b.global_scale.data_ptr() if b.global_scale is not None else None,
            ptrs, owners, rows_per_owner, ldo, m, n, k, FORMATS[a.fmt], a.gs_rows, _stream(stream)),
        "tf_gemm_blockscaled_scatter",
    )


def gemm_splits(m: int, n: int, k: int, fmt: str, epilogue: str = "none") -> int:
    """How many K ranges the GEMM cuts this problem into (1: not split; more than 1 only for few rows)."""
    return int(N.load().tf_gemm_splits(m, n, k, FORMATS[fmt], EPILOGUES[epilogue]))


class SplitKPartials:
    """The f32 partial sums a split-K GEMM left in its workspace: ``splits`` planes [M, N], to be summed in split order, scaled by
    the product of the operands' nvfp4 global scales and rounded to bf16 by the consumer (``rmsnorm_quantize_rows``)."""

    __slots__ = ("workspace", "splits", "shape", "a_global_scale", "b_global_scale")

    def __init__(self, workspace, splits, shape, a_global_scale, b_global_scale) -> None:
        self.workspace, self.splits, self.shape = workspace, splits, shape
        self.a_global_scale, self.b_global_scale = a_global_scale, b_global_scale


def gemm_blockscaled_partials(a: BlockScaledTensor, b: BlockScaledTensor, *, workspace=None, stream=None) -> SplitKPartials:
    """The first pass of a split-K GEMM only: ``deq(a) @ deq(b)^T`` stays in ``workspace`` as f32 partial sums for a consumer that
    sums them itself. Only for shapes the GEMM splits along K (``gemm_splits(...) > 1``: few rows, long K)."""
    torch = _torch()
    _pre(isinstance(a, BlockScaledTensor) and isinstance(b, BlockScaledTensor), "a and b must be BlockScaledTensor", "dtype")
    _pre(a.fmt == b.fmt, f"a is {a.fmt} but b is {b.fmt}: block-scaled formats must match exactly", "dtype", "b")
    _pre(a.layout == "swizzled" and b.layout == "swizzled", "the GEMM consumes swizzled scales", "contiguous")
    m, k = a.shape
    n, kb = b.shape
    _pre(k == kb, f"K differs: a is {a.shape}, b is {b.shape}", "shape", "b")
    _pre(a.gs_rows == 0, "partial sums carry one global scale for the whole of a", "argument", "a")
    _pre(gemm_splits(m, n, k, a.fmt) > 1, "this shape is not split along K: there are no partial sums to leave", "shape", "a")
    for t, nm in ((a.codes, "a.codes"), (b.codes, "b.codes"), (a.scales, "a.scales"), (b.scales, "b.scales")):
        _check(t, nm, torch.uint8, None, a.device)
        _dense(t, nm)
    if a.fmt == "nvfp4":
        _pre(a.global_scale is not None and b.global_scale is not None, "nvfp4 operands need their global scales", "argument")
    need = gemm_workspace_bytes(m, n, k, a.fmt, "none")
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
    _pre(workspace.numel() * workspace.element_size() >= need, f"workspace: {need} bytes needed", "workspace", "workspace")
    splits = ctypes.c_int32(0)
    N.check(
        N.load().tf_gemm_blockscaled_partials(
            a.codes.data_ptr(), a.scales.data_ptr(), a.global_scale.data_ptr() if a.global_scale is not None else None,
            b.codes.data_ptr(), b.scales.data_ptr(), b.global_scale.data_ptr() if b.global_scale is not None else None,
            m, n, k, FORMATS[a.fmt], workspace.data_ptr(), workspace.numel() * workspace.element_size(), ctypes.byref(splits), _stream(stream)),
        "tf_gemm_blockscaled_partials",
    )
    return SplitKPartials(workspace, int(splits.value), (m, n), a.global_scale, b.global_scale)


def rmsnorm_quantize_rows(x, residual, w, eps: float, fmt: str, q_out: BlockScaledTensor, *, sync=None, out=None, stream=None) -> BlockScaledTensor:
    """Few rows (at most one per SM): ``residual += x``, rmsnorm and the BlockScaled quantization of the result in ONE launch; the
    same bytes as ``residual_add_rmsnorm`` followed by ``quantize``. ``x`` is a bf16 [M, D] tensor or the ``SplitKPartials`` of the
    GEMM that produced it (then that GEMM's reduction pass is part of this launch too). ``q_out`` is preallocated storage whose
    scale bytes were zeroed when it was allocated (padding is never written); for nvfp4 it carries the float32 [1] that receives
    the tensor-wide scale, and ``sync`` is an int32 [2] device tensor the caller zeroes before every call."""
    torch = _torch()
    _pre(fmt in FORMATS, f"unknown block-scaled format {fmt!r}", "dtype", "fmt")
    _check(residual, "residual", torch.float32, 2)
    dev = residual.device
    m, d = residual.shape
    _check(w, "w", torch.bfloat16, 1, dev)
    _dense(residual, "residual")
    _dense(w, "w")
    _pre(tuple(w.shape) == (d,), f"w: shape {tuple(w.shape)}, expected {(d,)}", "shape", "w")
    _pre(d % 32 == 0, f"D={d} is not a multiple of 32", "divisible", "residual")
    _pre(q_out.fmt == fmt and q_out.shape == (m, d) and q_out.layout == "swizzled", "q_out: wrong format or shape", "shape", "q_out")
    xp, pp, splits, ags, bgs = None, None, 0, None, None
    if isinstance(x, SplitKPartials):
        _pre(x.shape == (m, d), f"partial sums of shape {x.shape}, expected {(m, d)}", "shape", "x")
        pp, splits = x.workspace.data_ptr(), x.splits
        if x.a_global_scale is not None:
            ags, bgs = x.a_global_scale.data_ptr(), x.b_global_scale.data_ptr()
    else:
        _check(x, "x", torch.bfloat16, 2, dev)
        _dense(x, "x")
        _pre(tuple(x.shape) == (m, d), f"x: shape {tuple(x.shape)}, expected {(m, d)}", "shape", "x")
        xp = x.data_ptr()
    if out is not None:
        _check(out, "out", torch.bfloat16, 2, dev)
        _dense(out, "out")
        _pre(tuple(out.shape) == (m, d), "out: wrong shape", "shape", "out")
    if m == 0:
        return q_out
    gs_ptr, sync_ptr = None, None
    if fmt == "nvfp4":
        _pre(q_out.global_scale is not None and sync is not None, "nvfp4 needs q_out.global_scale and the zeroed sync words", "argument", "sync")
        _check(sync, "sync", torch.int32, None, dev, align=8)
        _pre(sync.numel() >= 2, "sync: two 32-bit words", "shape", "sync")
        gs_ptr, sync_ptr = q_out.global_scale.data_ptr(), sync.data_ptr()
    N.check(
        N.load().tf_rmsnorm_quantize_rows(xp, pp, splits, ags, bgs, 0, residual.data_ptr(), w.data_ptr(), out.data_ptr() if out is not None else None,
                                          m, d, float(eps), FORMATS[fmt], q_out.codes.data_ptr(), q_out.scales.data_ptr(),
                                          gs_ptr, sync_ptr, _stream(stream)),
        "tf_rmsnorm_quantize_rows",
    )
    return q_out


def gemm(a, b: BlockScaledTensor, *, epilogue: str = "none", out=None, residual=None, a_global_scale=None, a_amax=None, amax_out=None,
         stream=None):
    """The library ``gemm``: ``a`` is bf16 [M, K] (quantized on the fly in b's format) or already a BlockScaledTensor."""
    if not isinstance(a, BlockScaledTensor):
        a = quantize(a, b.fmt, global_scale=a_global_scale, amax=a_amax, stream=stream)
    return gemm_blockscaled(a, b, epilogue=epilogue, out=out, residual=residual, amax_out=amax_out, stream=stream)


def require_cuda() -> None:
    torch = _torch()
    if not torch.cuda.is_available():
        raise TilefishRuntimeError("no CUDA device: this backend has no CPU path")
    N.load()
