// Per-thread core of the BlockScaled quantizers: one thread owns 8 consecutive bf16 values (one 128-bit load); the
// 4 (block 32) or 2 (block 16) adjacent lanes that share a scale block combine their maxima with warp shuffles.
//
// Every arithmetic step is a single correctly rounded f32 operation or an integer operation, in a fixed order, so the
// bytes are the same as the torch restatement's:
//   MX     amax on the 15 magnitude bits; E = amax >> 7; scale = amax == 0 ? 127 : max(E - emax, 0);
//          code = cast(f32(x) * 2^(127 - scale))                      (exact product)
//   NVFP4  s8 = e4m3(amax * (1 / (6 * gs))); d = f32(s8) * gs; code = e2m1(f32(x) * (1 / d)); zero when gs == 0 or d == 0
#pragma once

#include "common.cuh"

namespace tf {

// Maximum of the 15 magnitude bits of the 8 bf16 words of v (packed 16-bit unsigned maxima, then the two halves).
__device__ __forceinline__ uint32_t amax_bits8(const uint4& v) {
  const uint32_t k = 0x7FFF7FFFu;
  uint32_t t = __vimax3_u16x2(v.x & k, v.y & k, v.z & k);
  t = __vimax3_u16x2(t, v.w & k, 0u);
  return max(t & 0xFFFFu, t >> 16);
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Quantizes the 8 bf16 values of `v`. All 32 lanes of the warp must call it together (lanes without data pass zeros).
// Returns the packed codes in c0 (and c1 for 8-bit elements) and the scale byte of the lane's block.
// nvfp4: gs is the tensor's global scale and inv_t = 1 / (6 * gs), both uniform over the kernel.
template <int FMT>
__device__ __forceinline__ void quantize_vec8(const uint4& v, float gs, float inv_t, uint32_t& c0, uint32_t& c1, uint32_t& scale) {
  uint32_t m = amax_bits8(v);
  m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
  if (FMT != TF_FMT_NVFP4) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));

  if (FMT == TF_FMT_NVFP4) {
    const float amax = __uint_as_float(m << 16);
    uint32_t s8 = 0;
    if (gs != 0.0f && m != 0) s8 = cvt_e4m3x2(__fmul_rn(amax, inv_t), 0.0f) & 0xFFu;
    const float d = __fmul_rn(e4m3_to_f32(s8), gs);
    const bool zero = (d == 0.0f);
    const float inv = zero ? 0.0f : __frcp_rn(d);
    scale = s8;
    c0 = cvt_e2m1x2(__fmul_rn(bf16lo_to_f32(v.x), inv), __fmul_rn(bf16hi_to_f32(v.x), inv)) |
         (cvt_e2m1x2(__fmul_rn(bf16lo_to_f32(v.y), inv), __fmul_rn(bf16hi_to_f32(v.y), inv)) << 8) |
         (cvt_e2m1x2(__fmul_rn(bf16lo_to_f32(v.z), inv), __fmul_rn(bf16hi_to_f32(v.z), inv)) << 16) |
         (cvt_e2m1x2(__fmul_rn(bf16lo_to_f32(v.w), inv), __fmul_rn(bf16hi_to_f32(v.w), inv)) << 24);
    if (zero) c0 = 0;
    c1 = 0;
    return;
  }

  const int emax = (FMT == TF_FMT_MXFP8) ? 8 : 2;
  const int e = (int)(m >> 7) - emax;
  scale = (m == 0) ? 127u : (uint32_t)max(e, 0);
  // 2^(127 - scale) as two packed bf16: a power of two times a bf16 is exact in bf16 (a result below the normal range loses
  // bits, but it is then far below half of the smallest code and becomes a signed zero either way)
  const uint32_t inv1 = (254u - scale) << 7;
  const uint32_t inv2 = inv1 | (inv1 << 16);
  const uint32_t q0 = mul_bf16x2(v.x, inv2), q1 = mul_bf16x2(v.y, inv2), q2 = mul_bf16x2(v.z, inv2), q3 = mul_bf16x2(v.w, inv2);
  if (FMT == TF_FMT_MXFP8) {
    c0 = cvt_e4m3x2(bf16lo_to_f32(q0), bf16hi_to_f32(q0)) | (cvt_e4m3x2(bf16lo_to_f32(q1), bf16hi_to_f32(q1)) << 16);
    c1 = cvt_e4m3x2(bf16lo_to_f32(q2), bf16hi_to_f32(q2)) | (cvt_e4m3x2(bf16lo_to_f32(q3), bf16hi_to_f32(q3)) << 16);
  } else {
    c0 = cvt_e2m1x2(bf16lo_to_f32(q0), bf16hi_to_f32(q0)) | (cvt_e2m1x2(bf16lo_to_f32(q1), bf16hi_to_f32(q1)) << 8) |
         (cvt_e2m1x2(bf16lo_to_f32(q2), bf16hi_to_f32(q2)) << 16) | (cvt_e2m1x2(bf16lo_to_f32(q3), bf16hi_to_f32(q3)) << 24);
    c1 = 0;
  }
}

// 16 consecutive bf16 values per thread (one 256-bit load): half the shuffles, scale arithmetic and address arithmetic per element
// of the 8-value form. A block of 32 is two adjacent lanes; an nvfp4 block of 16 is the thread's own. Same arithmetic, same bytes.
// codes: 4 words (e4m3) or 2 words (e2m1).
template <int FMT>
__device__ __forceinline__ void quantize_vec16(const uint32_t (&w)[8], float gs, float inv_t, uint32_t (&codes)[4], uint32_t& scale) {
  const uint32_t k = 0x7FFF7FFFu;
  uint32_t t0 = __vimax3_u16x2(w[0] & k, w[1] & k, w[2] & k);
  uint32_t t1 = __vimax3_u16x2(w[3] & k, w[4] & k, w[5] & k);
  t0 = __vimax3_u16x2(t0, w[6] & k, w[7] & k);
  t0 = __vimax3_u16x2(t0, t1, 0u);
  uint32_t m = max(t0 & 0xFFFFu, t0 >> 16);
  if (FMT != TF_FMT_NVFP4) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));

  if (FMT == TF_FMT_NVFP4) {
    const float amax = __uint_as_float(m << 16);
    uint32_t s8 = 0;
    if (gs != 0.0f && m != 0) s8 = cvt_e4m3x2(__fmul_rn(amax, inv_t), 0.0f) & 0xFFu;
    const float d = __fmul_rn(e4m3_to_f32(s8), gs);
    const bool zero = (d == 0.0f);
    const float inv = zero ? 0.0f : __frcp_rn(d);
    scale = s8;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t c = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        c |= cvt_e2m1x2(__fmul_rn(bf16lo_to_f32(w[4 * h + j]), inv), __fmul_rn(bf16hi_to_f32(w[4 * h + j]), inv)) << (8 * j);
      codes[h] = zero ? 0u : c;
    }
    codes[2] = codes[3] = 0;
    return;
  }
  const int emax = (FMT == TF_FMT_MXFP8) ? 8 : 2;
  const int e = (int)(m >> 7) - emax;
  scale = (m == 0) ? 127u : (uint32_t)max(e, 0);
  const uint32_t inv1 = (254u - scale) << 7;
  const uint32_t inv2 = inv1 | (inv1 << 16);
  uint32_t q[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) q[j] = mul_bf16x2(w[j], inv2);
  if (FMT == TF_FMT_MXFP8) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      codes[j] = cvt_e4m3x2(bf16lo_to_f32(q[2 * j]), bf16hi_to_f32(q[2 * j])) | (cvt_e4m3x2(bf16lo_to_f32(q[2 * j + 1]), bf16hi_to_f32(q[2 * j + 1])) << 16);
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t c = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) c |= cvt_e2m1x2(bf16lo_to_f32(q[4 * h + j]), bf16hi_to_f32(q[4 * h + j])) << (8 * j);
      codes[h] = c;
    }
    codes[2] = codes[3] = 0;
  }
}

// Stores the codes of 16 elements (vector index `vec` of 16-element vectors in row `row`) and the block's scale byte.
template <int FMT>
__device__ __forceinline__ void store_quantized16(uint8_t* __restrict__ codes_out, uint8_t* __restrict__ scales, int swizzled, int64_t row, int vec,
                                                  int64_t k, const uint32_t (&codes)[4], uint32_t scale) {
  if (FMT == TF_FMT_MXFP8) {
    *reinterpret_cast<uint4*>(codes_out + row * k + (int64_t)vec * 16) = make_uint4(codes[0], codes[1], codes[2], codes[3]);
  } else {
    *reinterpret_cast<uint2*>(codes_out + row * (k >> 1) + (int64_t)vec * 8) = make_uint2(codes[0], codes[1]);
  }
  if (FMT == TF_FMT_NVFP4 || (vec & 1) == 0) {
    const int64_t cols = k / (FMT == TF_FMT_NVFP4 ? 16 : 32);
    const int64_t c = (FMT == TF_FMT_NVFP4) ? vec : (vec >> 1);
    const int64_t off = swizzled ? swizzled_scale_offset(row, c, (cols + 3) >> 2) : row * cols + c;
    scales[off] = (uint8_t)scale;
  }
}

// Stores one thread's codes (8 elements starting at element column `col` of row `row`) and, from the first lane of each
// block, the scale byte. `vec` is the index of the 8-element vector inside the row.
template <int FMT>
__device__ __forceinline__ void store_quantized(uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, int swizzled,
                                                int64_t row, int vec, int64_t k, uint32_t c0, uint32_t c1, uint32_t scale) {
  if (FMT == TF_FMT_MXFP8) {
    *reinterpret_cast<uint2*>(codes + row * k + (int64_t)vec * 8) = make_uint2(c0, c1);
  } else {
    *reinterpret_cast<uint32_t*>(codes + row * (k >> 1) + (int64_t)vec * 4) = c0;
  }
  const int lanes_per_block = (FMT == TF_FMT_NVFP4) ? 2 : 4;
  if ((vec & (lanes_per_block - 1)) == 0) {
    const int blk = (FMT == TF_FMT_NVFP4) ? 16 : 32;
    const int64_t cols = k / blk;
    const int64_t c = vec / lanes_per_block;
    const int64_t off = swizzled ? swizzled_scale_offset(row, c, (cols + 3) >> 2) : row * cols + c;
    scales[off] = (uint8_t)scale;
  }
}

}  // namespace tf
