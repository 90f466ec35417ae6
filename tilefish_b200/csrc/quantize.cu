// BlockScaled quantization row kernels (bf16 -> MXFP8 / MXFP4 / NVFP4) and the scale-layout helpers.
//
// HBM-bound: every thread moves one 256-bit vector of 16 bf16 per step (coalesced: consecutive lanes, consecutive
// vectors), block maxima are combined with at most one warp shuffle, codes leave as 16-byte (e4m3) or 8-byte (e2m1)
// coalesced stores. Algorithmic bytes per element: 2 + 1 + 1/32 (mxfp8), 2 + 0.5 + 1/32 (mxfp4), 2 + 0.5 + 1/16 (nvfp4).
#include "quant_core.cuh"

namespace tf {

constexpr int kQuantThreads = 256;
constexpr int kQuantUnroll = 2;

// Block = (TPR threads along the row) x (256 / TPR rows); rows are taken grid-stride.
__device__ __forceinline__ void load_256(const void* p, uint32_t (&w)[8]) {
  asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
               : "l"(p));
}

// gs_ptr holds the nvfp4 global scale, or (gs_out != nullptr) the tensor's amax from which it is derived here.
// One thread = 16 consecutive bf16 (one 256-bit load); block = (TPR threads along the row) x (256 / TPR rows).
template <int FMT>
__global__ void __launch_bounds__(kQuantThreads) quantize_rows_kernel(const uint8_t* __restrict__ x, int64_t m, int64_t k, int64_t ldx,
                                                                      uint8_t* __restrict__ codes, uint8_t* __restrict__ scales,
                                                                      int swizzled, const float* __restrict__ gs_ptr, float* __restrict__ gs_out) {
  const int tpr = blockDim.x;
  const int nvec = (int)(k >> 4);
  griddep_launch_dependents();
  griddep_wait();
  float gs = (FMT == TF_FMT_NVFP4) ? __ldg(gs_ptr) : 0.0f;
  if (FMT == TF_FMT_NVFP4 && gs_out != nullptr) {
    gs = __fdiv_rn(gs, 2688.0f);
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && threadIdx.y == 0) gs_out[0] = gs;
  }
  const float inv_t = (FMT == TF_FMT_NVFP4 && gs != 0.0f) ? __frcp_rn(__fmul_rn(6.0f, gs)) : 0.0f;
  const int64_t row_stride = (int64_t)gridDim.x * blockDim.y;
  // Both loops run the same number of times for every thread of the block, so the warp shuffle inside quantize_vec16 always
  // sees whole warps; threads without data (row >= m or vector >= nvec) quantize zeros and store nothing. nvec is even and
  // tpr a power of two >= 2, so the two lanes of one 32-element block have data together.
  for (int64_t row_base = (int64_t)blockIdx.x * blockDim.y; row_base < m; row_base += row_stride) {
    const int64_t row = row_base + threadIdx.y;
    const bool row_ok = row < m;
    const uint8_t* xr = x + (row_ok ? row : 0) * ldx * 2;
    // gridDim.y cuts the row into segments of whole rounds (few, long rows: more CTAs than row blocks)
    const int rounds = (nvec + kQuantUnroll * tpr - 1) / (kQuantUnroll * tpr);
    const int rounds_per_seg = (rounds + (int)gridDim.y - 1) / (int)gridDim.y;
    const int base_begin = (int)blockIdx.y * rounds_per_seg * kQuantUnroll * tpr;
    const int base_end = min(nvec, base_begin + rounds_per_seg * kQuantUnroll * tpr);
    for (int base = base_begin; base < base_end; base += kQuantUnroll * tpr) {  // kQuantUnroll 256-bit loads in flight per thread
      uint32_t v[kQuantUnroll][8];
      bool has[kQuantUnroll];
#pragma unroll
      for (int j = 0; j < kQuantUnroll; ++j) {
        const int vj = base + threadIdx.x + j * tpr;
        has[j] = row_ok && vj < nvec;
        if (has[j]) {
          load_256(xr + (int64_t)vj * 32, v[j]);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[j][e] = 0;
        }
      }
#pragma unroll
      for (int j = 0; j < kQuantUnroll; ++j) {
        if (base + j * tpr < nvec) {  // uniform over the block
          uint32_t c[4], sc;
          quantize_vec16<FMT>(v[j], gs, inv_t, c, sc);
          if (has[j]) store_quantized16<FMT>(codes, scales, swizzled, row, base + threadIdx.x + j * tpr, k, c, sc);
        }
      }
    }
  }
}

// max |x| over the tensor as the f32 bit pattern of a bf16 magnitude: 256-bit loads, four in flight per thread.
__global__ void __launch_bounds__(256) amax_bits_kernel(const uint8_t* __restrict__ x, int64_t m, int nvec, int64_t ldx,
                                                        unsigned int* __restrict__ out_bits) {
  const uint32_t k = 0x7FFF7FFFu;
  uint32_t acc = 0;  // two packed 16-bit maxima
  const int64_t total = m * nvec;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const bool dense = ldx == (int64_t)nvec * 16;
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
    uint32_t v[4][8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t i = i0 + j * stride;
      if (i < total) {
        int64_t off = i * 32;
        if (!dense) {
          const int64_t row = i / nvec;
          off = (row * ldx + (i - row * nvec) * 16) * 2;
        }
        load_256(x + off, v[j]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] = 0;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t t0 = __vimax3_u16x2(v[j][0] & k, v[j][1] & k, v[j][2] & k);
      uint32_t t1 = __vimax3_u16x2(v[j][3] & k, v[j][4] & k, v[j][5] & k);
      t0 = __vimax3_u16x2(t0, v[j][6] & k, v[j][7] & k);
      acc = __vimax3_u16x2(acc, t0, t1);
    }
  }
  uint32_t mx = max(acc & 0xFFFFu, acc >> 16);
  for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
  __shared__ uint32_t warp_max[8];
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) mx = max(mx, warp_max[w]);
    if (mx) atomicMax(out_bits, mx << 16);  // the f32 bit pattern of a non-negative bf16 orders like the integer
  }
}

__global__ void finalize_global_scale_kernel(float* gs) { gs[0] = __fdiv_rn(gs[0], 2688.0f); }

__global__ void __launch_bounds__(256) swizzle_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows, int64_t cols,
                                                      int to_swizzled) {
  const int64_t n_ct = (cols + 3) >> 2;
  const int64_t total = rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    const int64_t off = swizzled_scale_offset(r, c, n_ct);
    if (to_swizzled) dst[off] = src[i];
    else dst[i] = src[off];
  }
}

static int block_of(int format) { return format == TF_FMT_NVFP4 ? 16 : 32; }

static tf_status check_quant_args(const char* fn, const void* x, int64_t m, int64_t k, int64_t ldx, const void* codes, const void* scales,
                                  int layout) {
  if (!x || !codes || !scales) return fail(TF_ERR_INVALID_ARGUMENT, "%s: null pointer", fn);
  if (m < 0 || k <= 0) return fail(TF_ERR_INVALID_ARGUMENT, "%s: bad shape m=%lld k=%lld", fn, (long long)m, (long long)k);
  if (layout != TF_SCALES_PLAIN && layout != TF_SCALES_SWIZZLED) return fail(TF_ERR_INVALID_ARGUMENT, "%s: unknown scale layout %d", fn, layout);
  if (k % 32 != 0) return fail(TF_ERR_UNSUPPORTED, "%s: k=%lld is not a multiple of 32", fn, (long long)k);
  if (ldx < k || ldx % 8 != 0) return fail(TF_ERR_ALIGNMENT, "%s: ldx=%lld must be >= k and a multiple of 8", fn, (long long)ldx);
  if (k > (int64_t)1 << 30) return fail(TF_ERR_UNSUPPORTED, "%s: k too large", fn);
  if ((uintptr_t)x % 16 || (uintptr_t)codes % 16) return fail(TF_ERR_ALIGNMENT, "%s: x and codes must be 16-byte aligned", fn);
  if ((uintptr_t)x % 32 || ldx % 16) return fail(TF_ERR_ALIGNMENT, "%s: x must be 32-byte aligned with ldx a multiple of 16 (256-bit loads)", fn);
  return TF_OK;
}

template <int FMT>
static tf_status launch_quantize(const char* fn, const void* x, int64_t m, int64_t k, int64_t ldx, void* codes, void* scales, int layout,
                                 const float* gs, cudaStream_t stream, float* gs_out = nullptr) {
  tf_status st = check_quant_args(fn, x, m, k, ldx, codes, scales, layout);
  if (st != TF_OK) return st;
  if (FMT == TF_FMT_NVFP4 && !gs) return fail(TF_ERR_INVALID_ARGUMENT, "%s: nvfp4 needs a global scale", fn);
  if (m == 0) return TF_OK;
  const int64_t cols = k / block_of(FMT);
  if (layout == TF_SCALES_SWIZZLED && ((m & 127) || (cols & 3)))
    TF_CUDA(cudaMemsetAsync(scales, 0, (size_t)tf_scale_bytes(FMT, m, k, layout), stream));
  int tpr = 2;
  while (tpr < kQuantThreads && tpr * kQuantUnroll < (k >> 4)) tpr <<= 1;
  const int rpb = kQuantThreads / tpr;
  const int64_t blocks_needed = (m + rpb - 1) / rpb;
  const int64_t cap = (int64_t)sm_count() * 8;
  dim3 block(tpr, rpb);
  dim3 grid((unsigned)(blocks_needed < cap ? blocks_needed : cap));
  const int64_t rounds = ((k >> 4) + kQuantUnroll * tpr - 1) / (kQuantUnroll * tpr);
  if (blocks_needed < 2 * sm_count() && rounds > 1) {  // few long rows: cut them into segments so that every SM gets work
    const int64_t want = (2 * sm_count() + blocks_needed - 1) / blocks_needed;
    grid.y = (unsigned)(want < rounds ? want : rounds);
  }
  TF_CUDA(launch_dependent(quantize_rows_kernel<FMT>, grid, block, 0, stream, static_cast<const uint8_t*>(x), m, k, ldx, static_cast<uint8_t*>(codes),
                           static_cast<uint8_t*>(scales), (int)(layout == TF_SCALES_SWIZZLED), gs, gs_out));
  return TF_OK;
}

}  // namespace tf

using namespace tf;

extern "C" {

int64_t tf_scale_bytes(int32_t format, int64_t rows, int64_t k, int32_t layout) {
  if (format < TF_FMT_MXFP8 || format > TF_FMT_NVFP4 || rows < 0 || k < 0) return -1;
  const int64_t blk = block_of(format);
  if (k % blk) return -1;
  const int64_t cols = k / blk;
  if (layout == TF_SCALES_PLAIN) return rows * cols;
  if (layout == TF_SCALES_SWIZZLED) return ((rows + 127) / 128) * ((cols + 3) / 4) * 512;
  return -1;
}

tf_status tf_quantize_mxfp8(const void* x, int64_t m, int64_t k, int64_t ldx, void* codes, void* scales, int32_t layout, void* stream) {
  clear_error();
  return launch_quantize<TF_FMT_MXFP8>(__func__, x, m, k, ldx, codes, scales, layout, nullptr, (cudaStream_t)stream);
}
tf_status tf_quantize_mxfp4(const void* x, int64_t m, int64_t k, int64_t ldx, void* codes, void* scales, int32_t layout, void* stream) {
  clear_error();
  return launch_quantize<TF_FMT_MXFP4>(__func__, x, m, k, ldx, codes, scales, layout, nullptr, (cudaStream_t)stream);
}
tf_status tf_quantize_nvfp4(const void* x, int64_t m, int64_t k, int64_t ldx, void* codes, void* scales, int32_t layout,
                            const float* global_scale, void* stream) {
  clear_error();
  return launch_quantize<TF_FMT_NVFP4>(__func__, x, m, k, ldx, codes, scales, layout, global_scale, (cudaStream_t)stream);
}

tf_status tf_quantize_nvfp4_from_amax(const void* x, int64_t m, int64_t k, int64_t ldx, void* codes, void* scales, int32_t layout,
                                      const float* amax, float* global_scale_out, void* stream) {
  clear_error();
  TF_CHECK_ARG(amax && global_scale_out, "%s: null pointer", __func__);
  if (m == 0) {  // no kernel runs for an empty tensor: derive the scale with the one-thread kernel
    TF_CUDA(cudaMemcpyAsync(global_scale_out, amax, sizeof(float), cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    finalize_global_scale_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(global_scale_out);
    TF_LAUNCH_CHECK();
    return TF_OK;
  }
  return launch_quantize<TF_FMT_NVFP4>(__func__, x, m, k, ldx, codes, scales, layout, amax, (cudaStream_t)stream, global_scale_out);
}

tf_status tf_nvfp4_global_scale(const void* x, int64_t m, int64_t k, int64_t ldx, float* out, void* stream_) {
  clear_error();
  cudaStream_t stream = (cudaStream_t)stream_;
  TF_CHECK_ARG(x && out, "%s: null pointer", __func__);
  TF_CHECK_ARG(m >= 0 && k > 0 && k % 16 == 0 && ldx >= k && ldx % 16 == 0, "%s: bad shape (k and ldx must be multiples of 16)", __func__);
  TF_CHECK_ALIGNED(x, 32, "x");
  TF_CUDA(cudaMemsetAsync(out, 0, sizeof(float), stream));
  if (m > 0) {
    const int64_t total = m * (k >> 4);
    const int64_t need = (total + 1023) / 1024, cap = (int64_t)sm_count() * 8;
    amax_bits_kernel<<<(unsigned)(need < cap ? need : cap), 256, 0, stream>>>(static_cast<const uint8_t*>(x), m, (int)(k >> 4), ldx,
                                                                              reinterpret_cast<unsigned int*>(out));
    TF_LAUNCH_CHECK();
  }
  finalize_global_scale_kernel<<<1, 1, 0, stream>>>(out);
  TF_LAUNCH_CHECK();
  return TF_OK;
}

static tf_status swizzle_impl(const char* fn, const void* src, void* dst, int64_t rows, int64_t cols, int to_swizzled, cudaStream_t stream) {
  if (!src || !dst) return fail(TF_ERR_INVALID_ARGUMENT, "%s: null pointer", fn);
  if (rows < 0 || cols < 0) return fail(TF_ERR_INVALID_ARGUMENT, "%s: bad shape", fn);
  if (to_swizzled) {
    const size_t bytes = (size_t)(((rows + 127) / 128) * ((cols + 3) / 4) * 512);
    if (bytes) TF_CUDA(cudaMemsetAsync(dst, 0, bytes, stream));
  }
  const int64_t total = rows * cols;
  if (total == 0) return TF_OK;
  const int64_t need = (total + 255) / 256, cap = (int64_t)sm_count() * 8;
  swizzle_kernel<<<(unsigned)(need < cap ? need : cap), 256, 0, stream>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows,
                                                                          cols, to_swizzled);
  TF_LAUNCH_CHECK();
  return TF_OK;
}

tf_status tf_swizzle_scales(const void* plain, int64_t rows, int64_t cols, void* swizzled, void* stream) {
  clear_error();
  return swizzle_impl(__func__, plain, swizzled, rows, cols, 1, (cudaStream_t)stream);
}
tf_status tf_unswizzle_scales(const void* swizzled, int64_t rows, int64_t cols, void* plain, void* stream) {
  clear_error();
  return swizzle_impl(__func__, swizzled, plain, rows, cols, 0, (cudaStream_t)stream);
}

}  // extern "C"
