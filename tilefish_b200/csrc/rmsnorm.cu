// residual_add_rmsnorm row kernel, optionally fused with the BlockScaled quantization of its bf16 result.
//
//   r = residual + f32(x)           one exact f32 add; written back to residual
//   out = bf16(r * rstd * f32(w))   rstd = rsqrt(sum(r*r) * f32(1/D) + eps); the only rounding point is the bf16 cast
//
// HBM-bound: 12 bytes per element (2 read x, 4 read + 4 write residual, 2 write out), plus the quantized copy when asked
// for. One block per row (grid-stride), 128-bit loads, the row's r values stay in registers between the reduction and the
// normalisation, warp-shuffle + shared-memory block reduction.
#include "async_copy.cuh"
#include "quant_core.cuh"

namespace tf {

template <int VPT, int QFMT>  // VPT: 8-element vectors per thread; QFMT: -1 none, else TF_FMT_*
__global__ void __launch_bounds__(512) residual_add_rmsnorm_kernel(const uint4* __restrict__ x, float4* __restrict__ residual,
                                                                   const uint4* __restrict__ w, uint4* __restrict__ out, int64_t m, int d,
                                                                   float eps, float inv_d, uint8_t* __restrict__ q_codes,
                                                                   uint8_t* __restrict__ q_scales, int q_swizzled,
                                                                   const float* __restrict__ q_gs_ptr, unsigned int* __restrict__ out_amax) {
  __shared__ float warp_sums[16];
  __shared__ unsigned int warp_amax[16];
  uint32_t amax_bits = 0;  // over every row this thread touches; combined once at the end
  __shared__ float row_rstd;
  const int nvec = d >> 3;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  griddep_launch_dependents();
  griddep_wait();
  const float gs = (QFMT == TF_FMT_NVFP4) ? __ldg(q_gs_ptr) : 0.0f;
  const float inv_t = (QFMT == TF_FMT_NVFP4 && gs != 0.0f) ? __frcp_rn(__fmul_rn(6.0f, gs)) : 0.0f;

  for (int64_t row = blockIdx.x; row < m; row += gridDim.x) {
    const uint4* xr = x + row * nvec;
    float4* rr = residual + row * (nvec * 2);
    float r[VPT][8];
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * nthreads;
      if (v < nvec) {
        const uint4 xv = __ldcs(xr + v);
        const float4 a = __ldcs(rr + 2 * v), b = __ldcs(rr + 2 * v + 1);
        r[i][0] = __fadd_rn(a.x, bf16lo_to_f32(xv.x));
        r[i][1] = __fadd_rn(a.y, bf16hi_to_f32(xv.x));
        r[i][2] = __fadd_rn(a.z, bf16lo_to_f32(xv.y));
        r[i][3] = __fadd_rn(a.w, bf16hi_to_f32(xv.y));
        r[i][4] = __fadd_rn(b.x, bf16lo_to_f32(xv.z));
        r[i][5] = __fadd_rn(b.y, bf16hi_to_f32(xv.z));
        r[i][6] = __fadd_rn(b.z, bf16lo_to_f32(xv.w));
        r[i][7] = __fadd_rn(b.w, bf16hi_to_f32(xv.w));
        __stcs(rr + 2 * v, make_float4(r[i][0], r[i][1], r[i][2], r[i][3]));
        __stcs(rr + 2 * v + 1, make_float4(r[i][4], r[i][5], r[i][6], r[i][7]));
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(r[i][j], r[i][j], acc);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) r[i][j] = 0.0f;
      }
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if ((tid & 31) == 0) warp_sums[tid >> 5] = acc;
    __syncthreads();
    if (tid < 32) {
      float s = (tid < (nthreads >> 5)) ? warp_sums[tid] : 0.0f;
      for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
      if (tid == 0) row_rstd = __frsqrt_rn(__fadd_rn(__fmul_rn(s, inv_d), eps));
    }
    __syncthreads();
    const float rstd = row_rstd;

#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * nthreads;
      const bool has = v < nvec;
      uint4 o = make_uint4(0, 0, 0, 0);
      if (has) {
        const uint4 wv = __ldg(w + v);
        o.x = pack_bf16x2(__fmul_rn(__fmul_rn(r[i][0], rstd), bf16lo_to_f32(wv.x)), __fmul_rn(__fmul_rn(r[i][1], rstd), bf16hi_to_f32(wv.x)));
        o.y = pack_bf16x2(__fmul_rn(__fmul_rn(r[i][2], rstd), bf16lo_to_f32(wv.y)), __fmul_rn(__fmul_rn(r[i][3], rstd), bf16hi_to_f32(wv.y)));
        o.z = pack_bf16x2(__fmul_rn(__fmul_rn(r[i][4], rstd), bf16lo_to_f32(wv.z)), __fmul_rn(__fmul_rn(r[i][5], rstd), bf16hi_to_f32(wv.z)));
        o.w = pack_bf16x2(__fmul_rn(__fmul_rn(r[i][6], rstd), bf16lo_to_f32(wv.w)), __fmul_rn(__fmul_rn(r[i][7], rstd), bf16hi_to_f32(wv.w)));
        if (out) __stcs(out + row * nvec + v, o);
        if (out_amax) amax_bits = max(amax_bits, amax_bits8(o));
      }
      if (QFMT >= 0) {
        // uniform over the block: i * nthreads < nvec decides whether any thread has a vector in this round
        if (i * nthreads < nvec) {
          uint32_t c0, c1, sc;
          quantize_vec8<(QFMT < 0 ? 0 : QFMT)>(o, gs, inv_t, c0, c1, sc);
          if (has) store_quantized<(QFMT < 0 ? 0 : QFMT)>(q_codes, q_scales, q_swizzled, row, v, d, c0, c1, sc);
        }
      }
    }
    __syncthreads();  // warp_sums / row_rstd are reused by the next row
  }
  if (out_amax) {  // one atomic per block
    for (int o = 16; o > 0; o >>= 1) amax_bits = max(amax_bits, __shfl_xor_sync(0xFFFFFFFFu, amax_bits, o));
    if ((tid & 31) == 0) warp_amax[tid >> 5] = amax_bits;
    __syncthreads();
    if (tid == 0) {
      for (int wi = 1; wi < (nthreads >> 5); ++wi) amax_bits = max(amax_bits, warp_amax[wi]);
      if (amax_bits) atomicMax(out_amax, amax_bits << 16);
    }
  }
}

template <int VPT>
static void launch_vpt(int qfmt, dim3 grid, dim3 block, cudaStream_t s, const uint4* x, float4* res, const uint4* w, uint4* out, int64_t m, int d,
                       float eps, float inv_d, uint8_t* qc, uint8_t* qs, int qsw, const float* qgs, unsigned int* amax) {
  switch (qfmt) {
    case TF_FMT_MXFP8: launch_dependent(residual_add_rmsnorm_kernel<VPT, TF_FMT_MXFP8>, grid, block, 0, s, x, res, w, out, m, d, eps, inv_d, qc, qs, qsw, qgs, amax); break;
    case TF_FMT_MXFP4: launch_dependent(residual_add_rmsnorm_kernel<VPT, TF_FMT_MXFP4>, grid, block, 0, s, x, res, w, out, m, d, eps, inv_d, qc, qs, qsw, qgs, amax); break;
    case TF_FMT_NVFP4: launch_dependent(residual_add_rmsnorm_kernel<VPT, TF_FMT_NVFP4>, grid, block, 0, s, x, res, w, out, m, d, eps, inv_d, qc, qs, qsw, qgs, amax); break;
    default: launch_dependent(residual_add_rmsnorm_kernel<VPT, -1>, grid, block, 0, s, x, res, w, out, m, d, eps, inv_d, qc, qs, qsw, qgs, amax); break;
  }
}


// ---- few rows: the split-K sum, the residual add, the normalisation and the quantization in one launch ----------------------------
// One CTA per row (the caller guarantees rows <= SMs, so every CTA is resident). The row's x comes either from a bf16 tensor or from
// the f32 planes a split-K GEMM left in its workspace: summed in split order, scaled by the product of the GEMM's nvfp4 global scales
// and rounded to bf16, which is exactly what that GEMM's own reduction pass stores. The thread mapping, the order of the sums and
// every rounding are those of residual_add_rmsnorm_kernel, so the bytes are the same as from the separate launches.
// nvfp4: the tensor-wide scale needs every row's amax, so the CTAs meet once (an arrival counter in `sync`, zeroed by the caller; the
// wait is bounded: on a timeout the device status words get TF_ERR_DEVICE_TIMEOUT and the CTA skips its stores). The normalised row
// stays in registers across the barrier.
constexpr unsigned long long kRowsBarrierLimitNs = 1000000000ull;

template <int VPT, int QFMT>
__global__ void __launch_bounds__(512) rmsnorm_quantize_rows_kernel(const uint4* __restrict__ x, const float* __restrict__ partials, int splits,
                                                                    const float* __restrict__ a_gs, const float* __restrict__ b_gs, int a_gs_rows,
                                                                    float4* __restrict__ residual, const uint4* __restrict__ w, uint4* __restrict__ out,
                                                                    int m, int d, float eps, float inv_d, uint8_t* __restrict__ q_codes,
                                                                    uint8_t* __restrict__ q_scales, float* __restrict__ q_gs_out,
                                                                    unsigned int* __restrict__ sync, int* __restrict__ status) {
  __shared__ float warp_sums[16];
  __shared__ unsigned int warp_amax[16];
  __shared__ float row_rstd;
  __shared__ float gs_s;
  __shared__ int ok_s;
  const int nvec = d >> 3;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int row = blockIdx.x;
  griddep_launch_dependents();
  griddep_wait();
  float alpha = 1.0f;
  if (splits > 0 && a_gs && b_gs) alpha = __fmul_rn(__ldg(a_gs + (a_gs_rows > 0 ? row / a_gs_rows : 0)), __ldg(b_gs));
  const int64_t plane = (int64_t)m * d;
  float4* rr = residual + (int64_t)row * (nvec * 2);
  float r[VPT][8];
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * nthreads;
    if (v < nvec) {
      uint4 xv;
      if (splits > 0) {
        float s8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) s8[j] = 0.0f;
        const float* base = partials + (int64_t)row * d + v * 8;
        for (int sp = 0; sp < splits; ++sp) {
          const float4 x0 = __ldcs(reinterpret_cast<const float4*>(base + sp * plane)), x1 = __ldcs(reinterpret_cast<const float4*>(base + sp * plane) + 1);
          s8[0] += x0.x; s8[1] += x0.y; s8[2] += x0.z; s8[3] += x0.w; s8[4] += x1.x; s8[5] += x1.y; s8[6] += x1.z; s8[7] += x1.w;
        }
        xv = make_uint4(pack_bf16x2(__fmul_rn(s8[0], alpha), __fmul_rn(s8[1], alpha)), pack_bf16x2(__fmul_rn(s8[2], alpha), __fmul_rn(s8[3], alpha)),
                        pack_bf16x2(__fmul_rn(s8[4], alpha), __fmul_rn(s8[5], alpha)), pack_bf16x2(__fmul_rn(s8[6], alpha), __fmul_rn(s8[7], alpha)));
      } else {
        xv = __ldcs(x + (int64_t)row * nvec + v);
      }
      const float4 a = __ldcs(rr + 2 * v), b = __ldcs(rr + 2 * v + 1);
      r[i][0] = __fadd_rn(a.x, bf16lo_to_f32(xv.x));
      r[i][1] = __fadd_rn(a.y, bf16hi_to_f32(xv.x));
      r[i][2] = __fadd_rn(a.z, bf16lo_to_f32(xv.y));
      r[i][3] = __fadd_rn(a.w, bf16hi_to_f32(xv.y));
      r[i][4] = __fadd_rn(b.x, bf16lo_to_f32(xv.z));
      r[i][5] = __fadd_rn(b.y, bf16hi_to_f32(xv.z));
      r[i][6] = __fadd_rn(b.z, bf16lo_to_f32(xv.w));
      r[i][7] = __fadd_rn(b.w, bf16hi_to_f32(xv.w));
      __stcs(rr + 2 * v, make_float4(r[i][0], r[i][1], r[i][2], r[i][3]));
      __stcs(rr + 2 * v + 1, make_float4(r[i][4], r[i][5], r[i][6], r[i][7]));
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(r[i][j], r[i][j], acc);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) r[i][j] = 0.0f;
    }
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
  if ((tid & 31) == 0) warp_sums[tid >> 5] = acc;
  __syncthreads();
  if (tid < 32) {
    float s = (tid < (nthreads >> 5)) ? warp_sums[tid] : 0.0f;
    for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    if (tid == 0) row_rstd = __frsqrt_rn(__fadd_rn(__fmul_rn(s, inv_d), eps));
  }
  __syncthreads();
  const float rstd = row_rstd;

  uint4 o4[VPT];
  uint32_t amax_bits = 0;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * nthreads;
    o4[i] = make_uint4(0, 0, 0, 0);
    if (v < nvec) {
      const uint4 wv = __ldg(w + v);
      o4[i].x = pack_bf16x2(__fmul_rn(__fmul_rn(r[i][0], rstd), bf16lo_to_f32(wv.x)), __fmul_rn(__fmul_rn(r[i][1], rstd), bf16hi_to_f32(wv.x)));
      o4[i].y = pack_bf16x2(__fmul_rn(__fmul_rn(r[i][2], rstd), bf16lo_to_f32(wv.y)), __fmul_rn(__fmul_rn(r[i][3], rstd), bf16hi_to_f32(wv.y)));
      o4[i].z = pack_bf16x2(__fmul_rn(__fmul_rn(r[i][4], rstd), bf16lo_to_f32(wv.z)), __fmul_rn(__fmul_rn(r[i][5], rstd), bf16hi_to_f32(wv.z)));
      o4[i].w = pack_bf16x2(__fmul_rn(__fmul_rn(r[i][6], rstd), bf16lo_to_f32(wv.w)), __fmul_rn(__fmul_rn(r[i][7], rstd), bf16hi_to_f32(wv.w)));
      if (out) __stcs(out + (int64_t)row * nvec + v, o4[i]);
      amax_bits = max(amax_bits, amax_bits8(o4[i]));
    }
  }

  float gs = 0.0f, inv_t = 0.0f;
  if (QFMT == TF_FMT_NVFP4) {
    for (int o = 16; o > 0; o >>= 1) amax_bits = max(amax_bits, __shfl_xor_sync(0xFFFFFFFFu, amax_bits, o));
    if ((tid & 31) == 0) warp_amax[tid >> 5] = amax_bits;
    __syncthreads();
    if (tid == 0) {
      for (int wi = 1; wi < (nthreads >> 5); ++wi) amax_bits = max(amax_bits, warp_amax[wi]);
      if (amax_bits) atomicMax(sync, amax_bits << 16);
      __threadfence();
      atomicAdd(sync + 1, 1u);
      // every row's CTA arrives (all are resident: rows <= SMs); bounded, the timer is read only every 64 polls
      int ok = 1;
      const unsigned long long t0 = globaltimer_ns();
      unsigned int seen;
      for (uint32_t spins = 1;; ++spins) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(sync + 1) : "memory");
        if (seen >= gridDim.x) break;
        if ((spins & 0x3F) == 0 && globaltimer_ns() - t0 > kRowsBarrierLimitNs) {
          if (atomicCAS(&status[0], 0, TF_ERR_DEVICE_TIMEOUT) == 0) status[1] = 12 * 65536 + (int)blockIdx.x;
          ok = 0;
          break;
        }
      }
      unsigned int amax_all;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(amax_all) : "l"(sync) : "memory");
      const float g = __fdiv_rn(__uint_as_float(amax_all), 2688.0f);
      gs_s = g;
      ok_s = ok;
      if (ok && blockIdx.x == 0) q_gs_out[0] = g;
    }
    __syncthreads();
    if (!ok_s) return;
    gs = gs_s;
    inv_t = gs != 0.0f ? __frcp_rn(__fmul_rn(6.0f, gs)) : 0.0f;
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * nthreads;
    if (i * nthreads < nvec) {  // uniform over the block: whole warps quantize together (lanes without data pass zeros)
      uint32_t c0, c1, sc;
      quantize_vec8<QFMT>(o4[i], gs, inv_t, c0, c1, sc);
      if (v < nvec) store_quantized<QFMT>(q_codes, q_scales, 1, row, v, d, c0, c1, sc);
    }
  }
}

template <int VPT>
static void launch_rows_vpt(int qfmt, dim3 grid, dim3 block, cudaStream_t s, const uint4* x, const float* partials, int splits, const float* a_gs,
                            const float* b_gs, int a_gs_rows, float4* res, const uint4* w, uint4* out, int m, int d, float eps, float inv_d, uint8_t* qc,
                            uint8_t* qs, float* qgs, unsigned int* sync, int* status) {
  switch (qfmt) {
    case TF_FMT_MXFP8: launch_dependent(rmsnorm_quantize_rows_kernel<VPT, TF_FMT_MXFP8>, grid, block, 0, s, x, partials, splits, a_gs, b_gs, a_gs_rows, res, w, out, m, d, eps, inv_d, qc, qs, qgs, sync, status); break;
    case TF_FMT_MXFP4: launch_dependent(rmsnorm_quantize_rows_kernel<VPT, TF_FMT_MXFP4>, grid, block, 0, s, x, partials, splits, a_gs, b_gs, a_gs_rows, res, w, out, m, d, eps, inv_d, qc, qs, qgs, sync, status); break;
    default: launch_dependent(rmsnorm_quantize_rows_kernel<VPT, TF_FMT_NVFP4>, grid, block, 0, s, x, partials, splits, a_gs, b_gs, a_gs_rows, res, w, out, m, d, eps, inv_d, qc, qs, qgs, sync, status); break;
  }
}

}  // namespace tf

using namespace tf;

extern "C" tf_status tf_residual_add_rmsnorm(const void* x, void* residual, const void* w, void* out, int64_t m, int64_t d, float eps,
                                             int32_t q_format, void* q_codes, void* q_scales, int32_t q_layout, const float* q_global_scale,
                                             float* out_amax, void* stream_) {
  clear_error();
  cudaStream_t stream = (cudaStream_t)stream_;
  TF_CHECK_ARG(x && residual && w, "%s: null pointer", __func__);
  TF_CHECK_ARG(m >= 0 && d > 0, "%s: bad shape m=%lld d=%lld", __func__, (long long)m, (long long)d);
  TF_CHECK_ARG(q_format >= -1 && q_format <= TF_FMT_NVFP4, "%s: unknown q_format %d", __func__, q_format);
  TF_CHECK_ARG(out || q_format >= 0, "%s: neither out nor a quantized output was given", __func__);
  if (d % 8 != 0) return fail(TF_ERR_UNSUPPORTED, "%s: d=%lld is not a multiple of 8", __func__, (long long)d);
  if (d > 32768) return fail(TF_ERR_UNSUPPORTED, "%s: d=%lld exceeds 32768", __func__, (long long)d);
  TF_CHECK_ALIGNED(x, 16, "x");
  TF_CHECK_ALIGNED(residual, 16, "residual");
  TF_CHECK_ALIGNED(w, 16, "w");
  if (out) TF_CHECK_ALIGNED(out, 16, "out");
  if (q_format >= 0) {
    TF_CHECK_ARG(q_codes && q_scales, "%s: q_codes/q_scales missing", __func__);
    TF_CHECK_ARG(q_layout == TF_SCALES_PLAIN || q_layout == TF_SCALES_SWIZZLED, "%s: unknown scale layout %d", __func__, q_layout);
    TF_CHECK_ARG(q_format != TF_FMT_NVFP4 || q_global_scale, "%s: nvfp4 needs a global scale", __func__);
    if (d % 32 != 0) return fail(TF_ERR_UNSUPPORTED, "%s: quantized output needs d %% 32 == 0", __func__);
    TF_CHECK_ALIGNED(q_codes, 16, "q_codes");
    const int64_t cols = d / (q_format == TF_FMT_NVFP4 ? 16 : 32);
    if (q_layout == TF_SCALES_SWIZZLED && m > 0 && ((m & 127) || (cols & 3)))
      TF_CUDA(cudaMemsetAsync(q_scales, 0, (size_t)tf_scale_bytes(q_format, m, d, q_layout), stream));
  }
  if (m == 0) return TF_OK;

  const int nvec = (int)(d >> 3);
  int vpt = (nvec + 511) / 512;
  vpt = vpt <= 1 ? 1 : vpt <= 2 ? 2 : vpt <= 4 ? 4 : 8;
  int threads = (nvec + vpt - 1) / vpt;
  threads = (threads + 31) / 32 * 32;
  const int64_t cap = (int64_t)sm_count() * (2048 / threads);
  dim3 grid((unsigned)(m < cap ? m : cap)), block(threads);
  const float inv_d = 1.0f / (float)d;  // correctly rounded f32 reciprocal of D (IEEE division on the host)
  const uint4* xp = static_cast<const uint4*>(x);
  float4* rp = static_cast<float4*>(residual);
  const uint4* wp = static_cast<const uint4*>(w);
  uint4* op = static_cast<uint4*>(out);
  uint8_t* qc = static_cast<uint8_t*>(q_codes);
  uint8_t* qs = static_cast<uint8_t*>(q_scales);
  const int qsw = q_layout == TF_SCALES_SWIZZLED;
  switch (vpt) {
    case 1: launch_vpt<1>(q_format, grid, block, stream, xp, rp, wp, op, m, (int)d, eps, inv_d, qc, qs, qsw, q_global_scale, reinterpret_cast<unsigned int*>(out_amax)); break;
    case 2: launch_vpt<2>(q_format, grid, block, stream, xp, rp, wp, op, m, (int)d, eps, inv_d, qc, qs, qsw, q_global_scale, reinterpret_cast<unsigned int*>(out_amax)); break;
    case 4: launch_vpt<4>(q_format, grid, block, stream, xp, rp, wp, op, m, (int)d, eps, inv_d, qc, qs, qsw, q_global_scale, reinterpret_cast<unsigned int*>(out_amax)); break;
    default: launch_vpt<8>(q_format, grid, block, stream, xp, rp, wp, op, m, (int)d, eps, inv_d, qc, qs, qsw, q_global_scale, reinterpret_cast<unsigned int*>(out_amax)); break;
  }
  TF_LAUNCH_CHECK();
  return TF_OK;
}

extern "C" tf_status tf_rmsnorm_quantize_rows(const void* x, const float* partials, int32_t splits, const float* a_global_scale,
                                              const float* b_global_scale, int64_t a_global_scale_rows, void* residual, const void* w, void* out,
                                              int64_t m, int64_t d, float eps, int32_t q_format, void* q_codes, void* q_scales, float* q_global_scale,
                                              uint32_t* sync, void* stream_) {
  clear_error();
  cudaStream_t stream = (cudaStream_t)stream_;
  TF_CHECK_ARG(residual && w && q_codes && q_scales, "%s: null pointer", __func__);
  TF_CHECK_ARG((x != nullptr) != (partials != nullptr && splits > 0), "%s: give either x or split-K partial sums (splits > 0)", __func__);
  TF_CHECK_ARG(splits >= 0 && splits <= 64, "%s: splits must be in 0..64", __func__);
  TF_CHECK_ARG(q_format >= TF_FMT_MXFP8 && q_format <= TF_FMT_NVFP4, "%s: unknown q_format %d", __func__, q_format);
  TF_CHECK_ARG(d > 0 && m >= 0, "%s: bad shape m=%lld d=%lld", __func__, (long long)m, (long long)d);
  TF_CHECK_ARG(a_global_scale_rows >= 0, "%s: a_global_scale_rows must not be negative", __func__);
  TF_CHECK_ARG((a_global_scale == nullptr) == (b_global_scale == nullptr), "%s: the two GEMM global scales go together", __func__);
  TF_CHECK_ARG(q_format != TF_FMT_NVFP4 || (q_global_scale && sync), "%s: nvfp4 needs q_global_scale and the two zeroed sync words", __func__);
  if (d % 32 != 0 || d > 32768) return fail(TF_ERR_UNSUPPORTED, "%s: d=%lld must be a multiple of 32 and at most 32768", __func__, (long long)d);
  if (m > sm_count())
    return fail(TF_ERR_UNSUPPORTED, "%s: m=%lld exceeds the %d SMs (one resident CTA per row); use tf_residual_add_rmsnorm and tf_quantize_*", __func__,
                (long long)m, sm_count());
  if (x) TF_CHECK_ALIGNED(x, 16, "x");
  if (partials) TF_CHECK_ALIGNED(partials, 16, "partials");
  TF_CHECK_ALIGNED(residual, 16, "residual");
  TF_CHECK_ALIGNED(w, 16, "w");
  if (out) TF_CHECK_ALIGNED(out, 16, "out");
  TF_CHECK_ALIGNED(q_codes, 16, "q_codes");
  if (sync) TF_CHECK_ALIGNED(sync, 8, "sync");
  if (m == 0) return TF_OK;
  int* status = device_status_words();
  if (!status) return fail(TF_ERR_CUDA, "%s: cannot locate the device status words", __func__);
  const int nvec = (int)(d >> 3);
  int vpt = (nvec + 511) / 512;
  vpt = vpt <= 1 ? 1 : vpt <= 2 ? 2 : vpt <= 4 ? 4 : 8;
  int threads = (nvec + vpt - 1) / vpt;
  threads = (threads + 31) / 32 * 32;
  dim3 grid((unsigned)m), block(threads);
  const float inv_d = 1.0f / (float)d;
  const uint4* xp = static_cast<const uint4*>(x);
  float4* rp = static_cast<float4*>(residual);
  const uint4* wp = static_cast<const uint4*>(w);
  uint4* op = static_cast<uint4*>(out);
  uint8_t* qc = static_cast<uint8_t*>(q_codes);
  uint8_t* qs = static_cast<uint8_t*>(q_scales);
  switch (vpt) {
    case 1: launch_rows_vpt<1>(q_format, grid, block, stream, xp, partials, splits, a_global_scale, b_global_scale, (int)a_global_scale_rows, rp, wp, op, (int)m, (int)d, eps, inv_d, qc, qs, q_global_scale, sync, status); break;
    case 2: launch_rows_vpt<2>(q_format, grid, block, stream, xp, partials, splits, a_global_scale, b_global_scale, (int)a_global_scale_rows, rp, wp, op, (int)m, (int)d, eps, inv_d, qc, qs, q_global_scale, sync, status); break;
    case 4: launch_rows_vpt<4>(q_format, grid, block, stream, xp, partials, splits, a_global_scale, b_global_scale, (int)a_global_scale_rows, rp, wp, op, (int)m, (int)d, eps, inv_d, qc, qs, q_global_scale, sync, status); break;
    default: launch_rows_vpt<8>(q_format, grid, block, stream, xp, partials, splits, a_global_scale, b_global_scale, (int)a_global_scale_rows, rp, wp, op, (int)m, (int)d, eps, inv_d, qc, qs, q_global_scale, sync, status); break;
  }
  TF_LAUNCH_CHECK();
  return TF_OK;
}
