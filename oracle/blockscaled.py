"""CPU oracle for the quantized-inference hot path (TEST INFRASTRUCTURE, not product code).

Only tests, the smoke check and the CPU-baseline legs of the benchmark may import this module; the product path
(`tilefish_b200`) never does, and fails loudly when its CUDA library is missing.

What is restated here, in torch on the CPU, and what it follows in the reference project (paths are relative to the
reference repository):

* ``f32_to_bf16``            python/src/tilefish/_reference.py:76-88   (RNE on the bit pattern, canonical NaN 0x7FFF)
* ``cast_e4m3``              python/src/tilefish/_reference.py:121-141 (clamp to +-448, then torch's RNE cast: satfinite)
* ``residual_add_rmsnorm``   README.md:53-63 as interpreted by python/src/tilefish/_reference.py:309-324,369-386
                             (one f32 add, ``mean = sum * f32(1/D)``, ``torch.rsqrt``, one rounding to bf16)
* ``silu_gate``              README.md:83-84; ``silu = x * (1 / (1 + exp(-x)))`` python/src/tilefish/_reference.py:365-366
* ``reference_gemm``         python/src/tilefish/_library.py:1346-1356 (operands widened to f32, multiplied, one rounding)

Parity for those is pinned by fixtures generated from the reference itself (tests/golden/make_golden.py).

PARITY UNPINNED for everything block-scaled: the reference only *types* ``BlockScaled`` (python/src/tilefish/dtypes.py:145-232);
it refuses to quantize (python/src/tilefish/ops.py:556-559), to run a block-scaled tensor (python/src/tilefish/_launch.py:166-171)
and has no scale layout code. The functions ``quantize_*``, ``swizzle_scales``, ``dequantize`` and ``gemm_blockscaled``
below are therefore this project's own frozen definition; the only inherited rules are the element cast above, the
type facts (block 32/32/16, ue8m0/ue8m0/e4m3 scales, two e2m1 codes per byte, f32 global scale) and
``global = amax / (448 * 6)``.

Frozen quantization rules (every step is one exactly-specified f32 or integer operation):

MX (ue8m0 scale, block 32; e4m3 or e2m1 elements)
    amax      = max |x| over the block, compared on the 15 magnitude bits of the bf16 words
    E         = biased exponent field of amax (0 for zero/subnormal)
    scale     = 127 if amax == 0 else clamp(E - emax_elem, 0, 254), emax_elem = 8 (e4m3) or 2 (e2m1)
    code      = cast_elem(f32(x) * 2**(127 - scale))            (the product is exact; values above the element
                maximum saturate: the OCP "floor" convention)
NVFP4 (e4m3 scale, block 16, f32 global scale)
    gs        = amax_tensor / 2688.0f                           (one division; or given by the caller)
    s8        = cast_e4m3(amax_block * (1.0f / (6.0f * gs)))    (ONE reciprocal per tensor, one multiply per block;
                0 when gs == 0 or the block is all zero)
    d         = f32(s8) * gs                                    (decode scale, one multiply)
    code      = cast_e2m1(f32(x) * (1.0f / d))                  (ONE reciprocal per block, one multiply per element;
                all codes 0 when d == 0)
e2m1 cast: magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}; round to nearest, ties to the even code; saturate at 6
    (infinities included); the sign bit is kept (-0 is 0x8); NaN becomes 0x7 (+6), what the sm_100 conversion gives.
Packing: element 2i in bits 0-3, element 2i+1 in bits 4-7.
Swizzled scale layout: 128-row x 4-column tiles of 512 bytes, row-tile major; inside a tile byte(r, c) =
    (r % 32) * 16 + (r // 32) * 4 + c; padding bytes are zero.
"""

from __future__ import annotations

import torch

E4M3_MAX = 448.0
E2M1_MAX = 6.0
NVFP4_GLOBAL_DIVISOR = 2688.0  # 448 * 6

FORMATS = {
    # name: (element, scale dtype, block, emax of the element)
    "mxfp8": ("e4m3", "ue8m0", 32, 8),
    "mxfp4": ("e2m1", "ue8m0", 32, 2),
    "nvfp4": ("e2m1", "e4m3", 16, None),
}


# ----------------------------------------------------------------------------------------------------------------------
# element casts
# ----------------------------------------------------------------------------------------------------------------------
def f32_to_bf16(x: torch.Tensor) -> torch.Tensor:
    """f32 -> bf16, round to nearest even on the bits, NaN -> 0x7FFF (python/src/tilefish/_reference.py:76-88)."""
    b = x.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    rounded = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    word = torch.where(torch.isnan(x), torch.full_like(b, 0x7FFF), rounded) & 0xFFFF
    return torch.where(word >= 0x8000, word - 0x10000, word).to(torch.int16).view(torch.bfloat16)


def cast_e4m3(x: torch.Tensor) -> torch.Tensor:
    """f32 -> e4m3fn code bytes (uint8): RNE, saturating at +-448, NaN stays NaN (python/src/tilefish/_reference.py:137-138)."""
    return x.to(torch.float32).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_to_f32(codes: torch.Tensor) -> torch.Tensor:
    return codes.view(torch.float8_e4m3fn).to(torch.float32)


def cast_e2m1(x: torch.Tensor) -> torch.Tensor:
    """f32 -> e2m1 code (uint8 in 0..15): RNE with ties to the even code, saturating at +-6, sign kept, NaN -> 0x7."""
    x = x.to(torch.float32)
    a = x.abs()
    code = (
        (a > 0.25).to(torch.uint8)
        + (a >= 0.75).to(torch.uint8)
        + (a > 1.25).to(torch.uint8)
        + (a >= 1.75).to(torch.uint8)
        + (a > 2.5).to(torch.uint8)
        + (a >= 3.5).to(torch.uint8)
        + (a > 5.0).to(torch.uint8)
    )
    sign = (x.view(torch.int32) < 0).to(torch.uint8) << 3
    out = code | sign
    return torch.where(torch.isnan(x), torch.full_like(out, 0x7), out)


_E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def e2m1_to_f32(codes: torch.Tensor) -> torch.Tensor:
    return _E2M1_VALUES[codes.to(torch.int64)]


def pack_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] nibbles -> [..., K/2] bytes, element 2i in the low nibble."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()


def unpack_e2m1(packed: torch.Tensor) -> torch.Tensor:
    lo = packed & 0xF
    hi = packed >> 4
    return torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


# ----------------------------------------------------------------------------------------------------------------------
# block-scaled quantization (this project's frozen definition; unpinned in the reference)
# ----------------------------------------------------------------------------------------------------------------------
def _bf16_magnitude_bits(x: torch.Tensor) -> torch.Tensor:
    assert x.dtype == torch.bfloat16
    return x.contiguous().view(torch.int16).to(torch.int32) & 0x7FFF


def _pow2(exp_field: torch.Tensor) -> torch.Tensor:
    """The f32 whose biased exponent field is ``exp_field`` (1..254) and mantissa 0."""
    return (exp_field.to(torch.int32) << 23).view(torch.float32)


def quantize_mx(x: torch.Tensor, fmt: str):
    """bf16 [M, K] -> (codes, scales[M, K/32] uint8). codes: [M, K] e4m3 bytes (mxfp8) or [M, K/2] packed e2m1 (mxfp4)."""
    elem, _, block, emax = FORMATS[fmt]
    assert block == 32 and emax is not None
    m, k = x.shape
    assert k % block == 0
    mag = _bf16_magnitude_bits(x).view(m, k // block, block)
    amax = mag.amax(dim=-1)
    e = amax >> 7
    scale = torch.where(amax == 0, torch.full_like(e, 127), (e - emax).clamp(0, 254))
    inv = _pow2(254 - scale)  # 2**(127 - scale): exponent field 254 - scale, always a normal f32
    q = x.to(torch.float32).view(m, k // block, block) * inv.unsqueeze(-1)
    q = q.view(m, k)
    if elem == "e4m3":
        codes = cast_e4m3(q)
    else:
        codes = pack_e2m1(cast_e2m1(q))
    return codes, scale.to(torch.uint8)


def nvfp4_global_scale(x: torch.Tensor) -> torch.Tensor:
    """0-d f32: amax|x| / 2688 (one IEEE division)."""
    amax = _bf16_magnitude_bits(x).amax()
    amax_f = (amax.to(torch.int32) << 16).view(torch.float32)
    return amax_f / torch.tensor(NVFP4_GLOBAL_DIVISOR, dtype=torch.float32)


def quantize_nvfp4(x: torch.Tensor, global_scale: "torch.Tensor | None" = None):
    """bf16 [M, K] -> (codes [M, K/2] packed e2m1, scales [M, K/16] e4m3 bytes, global_scale 0-d f32)."""
    m, k = x.shape
    block = 16
    assert k % block == 0
    gs = nvfp4_global_scale(x) if global_scale is None else global_scale.to(torch.float32).reshape(())
    xf = x.to(torch.float32).view(m, k // block, block)
    amax = xf.abs().amax(dim=-1)  # NaN-free inputs; exact in f32
    t = torch.tensor(E2M1_MAX, dtype=torch.float32) * gs
    inv_t = torch.ones((), dtype=torch.float32) / t
    dead = (gs == 0) | (amax == 0)
    s = torch.where(dead, torch.zeros_like(amax), amax * inv_t)
    s8 = torch.where(dead, torch.zeros_like(s).to(torch.uint8), cast_e4m3(s))
    d = e4m3_to_f32(s8) * gs
    inv = torch.where(d == 0, torch.zeros_like(d), 1.0 / d)
    q = xf * inv.unsqueeze(-1)
    codes = cast_e2m1(q)
    codes = torch.where((d == 0).unsqueeze(-1), torch.zeros_like(codes), codes)
    return pack_e2m1(codes.view(m, k)), s8, gs


def quantize(x: torch.Tensor, fmt: str, global_scale: "torch.Tensor | None" = None):
    """(codes, scales, global_scale or None) with scales in the plain [M, K/block] layout."""
    if fmt == "nvfp4":
        return quantize_nvfp4(x, global_scale)
    codes, scales = quantize_mx(x, fmt)
    return codes, scales, None


def dequantize(codes: torch.Tensor, scales: torch.Tensor, fmt: str, global_scale: "torch.Tensor | None" = None) -> torch.Tensor:
    """f32 [M, K]: element * block scale (* global scale), with the association ``f32(code) * (f32(s8) * gs)``."""
    elem, scale_dtype, block, _ = FORMATS[fmt]
    vals = e4m3_to_f32(codes) if elem == "e4m3" else e2m1_to_f32(unpack_e2m1(codes))
    m, k = vals.shape
    if scale_dtype == "ue8m0":
        sc = scales.to(torch.int32)
        # 2**(s-127); s == 0 is 2**-127 (a subnormal f32), s == 255 is NaN by the format
        d = torch.where(sc == 0, torch.full_like(sc, 0x00400000), sc << 23).view(torch.float32)
        d = torch.where(sc == 255, torch.full_like(d, float("nan")), d)
    else:
        d = e4m3_to_f32(scales) * global_scale.to(torch.float32).reshape(())
    return (vals.view(m, k // block, block) * d.unsqueeze(-1)).view(m, k)


# ----------------------------------------------------------------------------------------------------------------------
# swizzled scale layout (pure integer map)
# ----------------------------------------------------------------------------------------------------------------------
def swizzled_scale_bytes(rows: int, cols: int) -> int:
    return ((rows + 127) // 128) * ((cols + 3) // 4) * 512


def swizzle_offsets(rows: int, cols: int) -> torch.Tensor:
    """int64 [rows, cols]: byte offset of scale (r, c) in the swizzled buffer."""
    r = torch.arange(rows, dtype=torch.int64).unsqueeze(1)
    c = torch.arange(cols, dtype=torch.int64).unsqueeze(0)
    n_ct = (cols + 3) // 4
    tile = (r // 128) * n_ct + (c // 4)
    rr = r % 128
    return tile * 512 + (rr % 32) * 16 + (rr // 32) * 4 + (c % 4)


def swizzle_scales(scales: torch.Tensor) -> torch.Tensor:
    """uint8 [rows, cols] -> flat uint8 [swizzled_scale_bytes(rows, cols)], padding zero."""
    rows, cols = scales.shape
    out = torch.zeros(swizzled_scale_bytes(rows, cols), dtype=torch.uint8)
    out[swizzle_offsets(rows, cols).reshape(-1)] = scales.reshape(-1)
    return out


def unswizzle_scales(buf: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    return buf[swizzle_offsets(rows, cols).reshape(-1)].reshape(rows, cols)


# ----------------------------------------------------------------------------------------------------------------------
# the operators of the path
# ----------------------------------------------------------------------------------------------------------------------
def residual_add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float = 1e-6):
    """Returns (new_residual f32, out bf16). README.md:53-63 in the reference's ``reference`` mode."""
    r = residual + x.to(torch.float32)
    d = r.shape[-1]
    inv_d = torch.ones((), dtype=torch.float32) / torch.tensor(float(d), dtype=torch.float32)
    mean = torch.sum(r * r, dim=-1, keepdim=True) * inv_d
    rstd = torch.rsqrt(mean + torch.tensor(eps, dtype=torch.float32))
    out = f32_to_bf16(r * rstd * w.to(torch.float32))
    return r, out


def silu_gate(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """bf16( silu(f32(g)) * f32(u) ), silu(x) = x * (1 / (1 + exp(-x)))."""
    gf = g.to(torch.float32)
    s = gf * (1.0 / (1.0 + torch.exp(-gf)))
    return f32_to_bf16(s * u.to(torch.float32))


def reference_gemm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """bf16( f32(a)[M,K] @ f32(b)[N,K]^T ): python/src/tilefish/_library.py:1346-1356 ("TN", f32 accumulate, one rounding)."""
    return f32_to_bf16(a.to(torch.float32) @ b.to(torch.float32).t())


def gemm_blockscaled(qa, qb, fmt: str) -> torch.Tensor:
    """qa, qb = (codes, plain scales, global scale|None). bf16( deq(qa) @ deq(qb)^T ), f32 accumulate."""
    a = dequantize(qa[0], qa[1], fmt, qa[2])
    b = dequantize(qb[0], qb[1], fmt, qb[2])
    return f32_to_bf16(a @ b.t())


def gemm_bf16_a(a_bf16: torch.Tensor, qb, fmt: str, a_global_scale: "torch.Tensor | None" = None) -> torch.Tensor:
    """The library ``gemm`` given a bf16 ``a``: quantize ``a`` along K in ``b``'s format, then the block-scaled product."""
    qa = quantize(a_bf16, fmt, a_global_scale)
    return gemm_blockscaled(qa, qb, fmt)


def mlp(x: torch.Tensor, q_gu, q_d, fmt: str) -> torch.Tensor:
    """README ``mlp`` graph: gemm(x, w_gu) -> split(F) -> silu(g)*u -> gemm(a, w_d); activations quantized at both gemms."""
    t = gemm_bf16_a(x, q_gu, fmt)
    f = t.shape[-1] // 2
    a = silu_gate(t[:, :f], t[:, f:])
    return gemm_bf16_a(a, q_d, fmt)


def decoder_block(x, residual, w_n, q_gu, q_d, fmt: str, eps: float = 1e-6):
    """residual_add_rmsnorm then ``mlp``. Returns (new_residual, out)."""
    r, h = residual_add_rmsnorm(x, residual, w_n, eps)
    return r, mlp(h, q_gu, q_d, fmt)


# ----------------------------------------------------------------------------------------------------------------------
# the tensor-parallel MLP stack, restated rank by rank (no counterpart in the reference, which has no cross-device exchange:
# this is the definition the multi-GPU kernels are checked against)
# ----------------------------------------------------------------------------------------------------------------------
def tp_shard_gu(q_gu, fmt: str, rank: int, world: int):
    """Rank ``rank``'s rows of the quantized ``w_gu`` [2F, H]: gate rows [rF/n, (r+1)F/n) and the matching up rows."""
    f = q_gu[0].shape[0] // 2
    fl = f // world
    rows = torch.cat([torch.arange(rank * fl, (rank + 1) * fl), torch.arange(f + rank * fl, f + (rank + 1) * fl)])
    return (q_gu[0][rows], q_gu[1][rows], q_gu[2])


def tp_shard_d(q_d, fmt: str, rank: int, world: int):
    """Rank ``rank``'s K-slice of the quantized ``w_d`` [H, F]: columns [rF/n, (r+1)F/n) of codes and of block scales."""
    elem, _, block, _ = FORMATS[fmt]
    epb = 1 if elem == "e4m3" else 2
    f = q_d[1].shape[1] * block
    fl = f // world
    return (q_d[0][:, rank * fl // epb:(rank + 1) * fl // epb].contiguous(), q_d[1][:, rank * fl // block:(rank + 1) * fl // block].contiguous(), q_d[2])


def rank_order_sum_bf16(parts) -> torch.Tensor:
    """bf16( ((0 + p0) + p1) + ... ): the ranks' bf16 partial results summed in f32 in rank order and rounded once, which is
    what the peer-load paths of the exchange kernels compute (tilefish_b200/csrc/allreduce.cu)."""
    acc = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:
        acc = acc + p.to(torch.float32)
    return f32_to_bf16(acc)


def _gemm_rowblocks(qa_blocks, qb, fmt: str) -> torch.Tensor:
    """bf16( deq(A) @ deq(B)^T ) where A is a stack of row blocks that were quantized separately (each with its own nvfp4
    global scale): the GEMM's ``a_global_scale_rows`` form."""
    a = torch.cat([dequantize(c, s, fmt, g) for (c, s, g) in qa_blocks])
    b = dequantize(qb[0], qb[1], fmt, qb[2])
    return f32_to_bf16(a @ b.t())


def tp_mlp_stack(x, residual, layers, fmt: str, world: int, *, norm: str = "replicated", spans=None, eps: float = 1e-6):
    """The tensor-parallel MLP stack as the kernels compute it, on one CPU. Returns (residual_out f32, y bf16).

    ``layers``: [(w_n bf16 [H], quantize(w_gu), quantize(w_d))] with the FULL quantized weights (plain scales); every rank's
    shard is cut from them. ``spans``: the row chunks [(begin, end)] (each chunk is its own tensor for the nvfp4 global
    scales); default one chunk.

    ``norm="replicated"`` (exchange = all-reduce of the partial results): per block and chunk
        h = rmsnorm(residual += x);  hq = quantize(h)           (nvfp4: global scale of the chunk's amax)
        rank r:  a_r = silu_gate(bf16 gemm(hq, w_gu shard r));  aq_r = quantize(a_r)   (nvfp4: amax of ITS [rows, F/n])
                 y_r = bf16 gemm(aq_r, w_d shard r)
        x_next = rank_order_sum_bf16(y_0 .. y_{n-1})
    ``norm="row_sharded"`` (the fused exchange and the scatter/gather mode): rank r normalises and quantizes rows
        [r R, (r+1) R) of every chunk (R = rows / n), nvfp4 with the global scale of ITS row block; the first GEMM multiplies the
        gathered row blocks, each with its own global scale; everything else as above.
    """
    assert norm in ("replicated", "row_sharded")
    m = x.shape[0]
    spans = spans or [(0, m)]
    res = residual.clone()
    xs = x
    for (w_n, q_gu, q_d) in layers:
        nxt = torch.empty_like(xs)
        for (lo, hi) in spans:
            r, h = residual_add_rmsnorm(xs[lo:hi], res[lo:hi], w_n, eps)
            res[lo:hi] = r
            if norm == "replicated":
                blocks = [quantize(h, fmt)]
            else:
                rr = (hi - lo) // world
                assert rr * world == hi - lo
                blocks = [quantize(h[k * rr:(k + 1) * rr], fmt) for k in range(world)]
            parts = []
            for rank in range(world):
                sh_gu = tp_shard_gu(q_gu, fmt, rank, world)
                t = _gemm_rowblocks(blocks, sh_gu, fmt)
                fl = t.shape[1] // 2
                a = silu_gate(t[:, :fl], t[:, fl:])
                parts.append(gemm_bf16_a(a, tp_shard_d(q_d, fmt, rank, world), fmt))
            nxt[lo:hi] = rank_order_sum_bf16(parts)
        xs = nxt
    return res, xs


def mlp_stack_unquantized(x, residual, layers, fmt: str, eps: float = 1e-6):
    """The stack with NO activation quantization and no bf16 rounding between the operators: f32 throughout, against the dequantized
    weights. Not what the kernels compute; the yardstick for how far ANY quantized run is from the arithmetic it approximates."""
    res = residual.clone()
    xs = x.to(torch.float32)
    for (w_n, q_gu, q_d) in layers:
        res = res + xs
        d = res.shape[-1]
        rstd = torch.rsqrt((res * res).sum(dim=-1, keepdim=True) * (1.0 / d) + eps)
        h = res * rstd * w_n.to(torch.float32)
        t = h @ dequantize(q_gu[0], q_gu[1], fmt, q_gu[2]).t()
        f = t.shape[1] // 2
        g = t[:, :f]
        a = g * (1.0 / (1.0 + torch.exp(-g))) * t[:, f:]
        xs = a @ dequantize(q_d[0], q_d[1], fmt, q_d[2]).t()
    return res, xs


def compare(got: torch.Tensor, ref: torch.Tensor) -> dict:
    """The figures every parity statement of a bf16 result uses: max|d| / max|ref|, relative Frobenius error, fraction of
    elements that differ."""
    g, r = got.to(torch.float32), ref.to(torch.float32)
    top = float(r.abs().max())
    return {
        "max_rel": float((g - r).abs().max()) / (top if top > 0 else 1.0),
        "rel_fro": float((g - r).norm() / r.norm()) if float(r.norm()) > 0 else float((g - r).norm()),
        "frac_diff": float((g != r).float().mean()),
    }


# ----------------------------------------------------------------------------------------------------------------------
# seeded synthetic inputs of the benchmark configurations
# ----------------------------------------------------------------------------------------------------------------------
def randn(shape, seed: int, dtype=torch.float32, scale: float = 1.0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * scale).to(dtype)


def outlier_input(m: int, k: int, seed: int = 0) -> torch.Tensor:
    """bf16 [m, k] ~ N(0, 1) with about 1 % of the entries (uniform positions) scaled by 100."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((m, k), generator=g, dtype=torch.float32)
    mask = torch.rand((m, k), generator=g) < 0.01
    return torch.where(mask, x * 100.0, x).to(torch.bfloat16)
