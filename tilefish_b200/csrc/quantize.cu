// BlockScaled quantization row kernels (bf16 -> MXFP8 / MXFP4 / NVFP4) and the scale-layout helpers.
//
// HBM-bound: every thread moves one 256-bit vector of 16 bf16 per step (coalesced: consecutive lanes, consecutive
// vectors), block maxima are combined with at most one warp shuffle, codes leave as 16-byte (e4m3) or 8-byte (e2m1)
// coalesced stores. Algorithmic bytes per element: 2 + 1 + 1/32 (mxfp8), 2 + 0.5 + 1/32 (mxfp4), 2 + 0.5 + 1/16 (nvfp4).
#include "async_copy.cuh"
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

// ---- the streaming form: rows staged through a shared-memory ring by bulk copies -------------------------------------------
// Used by the mxfp8 quantizer and the amax pass (see use_ring). For long rows (k >= 2048) the input is cut into chunks of up to 2048 consecutive bf16 of one row (4 KB). Every CTA owns a ring
// of kRingStages chunk buffers; thread 0 keeps the ring full with cp.async.bulk (one 4 KB request per chunk, completion counted
// on an mbarrier), so each CTA has (kRingStages - 1) x 4 KB in flight whatever its threads are doing, and eight CTAs fit on an
// SM: the loads no longer wait for registers. The 128 threads then take 32 bytes each from the stage (16 consecutive bf16,
// the same thread <-> element mapping and the same arithmetic as quantize_rows_kernel, hence the same bytes), hand the stage
// back, and quantize and store while the next copies are in flight. Waits are bounded (async_copy.cuh).
constexpr int kRingThreads = 128;
constexpr int kRingChunkVecs = kRingThreads;        // 16-element vectors per chunk
constexpr int kRingChunkBytes = kRingChunkVecs * 32;
constexpr int kRingMaxStages = 8;
constexpr unsigned long long kRingWaitLimitNs = 1000000000ull;
constexpr int kModeAmax = 3;  // MODE of ring_rows_kernel beyond the three formats: only the tensor's amax

__device__ __forceinline__ void lds_256(uint32_t addr, uint32_t (&w)[8]) {
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "r"(addr + 16));
}

// Dynamic shared memory: `stages` chunk buffers of 4 KB, then one mbarrier per stage.
template <int MODE>
__global__ void __launch_bounds__(kRingThreads) ring_rows_kernel(const uint8_t* __restrict__ x, int64_t m, int64_t k, int64_t ldx,
                                                                 uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, int swizzled,
                                                                 const float* __restrict__ gs_ptr, float* __restrict__ gs_out,
                                                                 unsigned int* __restrict__ amax_bits_out, int* __restrict__ status, int stages) {
  extern __shared__ __align__(128) uint8_t ring_smem[];
  __shared__ int abort_flag;
  constexpr int FMT = MODE == kModeAmax ? TF_FMT_MXFP8 : MODE;
  const uint32_t ring = smem_u32(ring_smem);
  const uint32_t bars = ring + (uint32_t)stages * kRingChunkBytes;
  const int t = threadIdx.x;
  const int nvec = (int)(k >> 4);
  const int cpr = (nvec + kRingChunkVecs - 1) / kRingChunkVecs;  // chunks per row
  const int64_t total = m * cpr;
  const int64_t stride = gridDim.x;
  if (t == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(bars + 8 * s, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  griddep_launch_dependents();
  griddep_wait();

  float gs = 0.0f, inv_t = 0.0f;
  if (MODE == TF_FMT_NVFP4) {
    gs = __ldg(gs_ptr);
    if (gs_out != nullptr) {
      gs = __fdiv_rn(gs, 2688.0f);
      if (blockIdx.x == 0 && t == 0) gs_out[0] = gs;
    }
    inv_t = gs != 0.0f ? __frcp_rn(__fmul_rn(6.0f, gs)) : 0.0f;
  }

  // thread 0: one bulk copy per chunk; a chunk is vectors [c * 128, min(nvec, c * 128 + 128)) of its row
  auto issue = [&](int64_t chunk, int stage) {
    const int64_t row = chunk / cpr;
    const int v0 = (int)(chunk - row * cpr) * kRingChunkVecs;
    const int nv = min(kRingChunkVecs, nvec - v0);
    const uint32_t bar = bars + 8 * stage;
    mbar_expect_tx(bar, (uint32_t)nv * 32u);
    bulk_load(ring + (uint32_t)stage * kRingChunkBytes, x + (row * ldx + (int64_t)v0 * 16) * 2, (uint32_t)nv * 32u, bar);
  };
  int64_t chunk = blockIdx.x;
  if (t == 0) {
    for (int s = 0; s < stages; ++s)
      if (chunk + s * stride < total) issue(chunk + s * stride, s);
  }
  uint32_t acc = 0;  // MODE == kModeAmax: two packed 16-bit maxima
  int stage = 0;
  uint32_t phase = 0;
  for (; chunk < total; chunk += stride) {
    const int64_t row = chunk / cpr;
    const int v0 = (int)(chunk - row * cpr) * kRingChunkVecs;
    const bool has = v0 + t < nvec;
    bool ok = mbar_wait_bounded(bars + 8 * stage, phase, &abort_flag, status, 10, kRingWaitLimitNs);
    uint32_t w[8];
    if (ok && has) {
      lds_256(ring + (uint32_t)stage * kRingChunkBytes + t * 32, w);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) w[e] = 0;
    }
    // every thread has taken its bytes (or the wait ran out somewhere: then all leave together)
    if (!__syncthreads_and(ok)) break;
    if (t == 0 && chunk + stages * stride < total) issue(chunk + stages * stride, stage);
    if (MODE == kModeAmax) {
      const uint32_t km = 0x7FFF7FFFu;
      uint32_t t0 = __vimax3_u16x2(w[0] & km, w[1] & km, w[2] & km);
      uint32_t t1 = __vimax3_u16x2(w[3] & km, w[4] & km, w[5] & km);
      t0 = __vimax3_u16x2(t0, w[6] & km, w[7] & km);
      acc = __vimax3_u16x2(acc, t0, t1);
    } else {
      uint32_t c[4], sc;
      quantize_vec16<FMT>(w, gs, inv_t, c, sc);  // whole warps: lanes without data quantize zeros
      if (has) store_quantized16<FMT>(codes, scales, swizzled, row, v0 + t, k, c, sc);
    }
    if (++stage == stages) {
      stage = 0;
      phase ^= 1;
    }
  }
  if (MODE == kModeAmax) {
    uint32_t mx = max(acc & 0xFFFFu, acc >> 16);
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    __shared__ uint32_t warp_max[kRingThreads / 32];
    if ((t & 31) == 0) warp_max[t >> 5] = mx;
    __syncthreads();
    if (t == 0) {
      for (int wi = 1; wi < kRingThreads / 32; ++wi) mx = max(mx, warp_max[wi]);
      if (mx) atomicMax(amax_bits_out, mx << 16);
    }
  }
  if (t == 0 && abort_flag) {  // a wait ran out: give copies still in flight time to land before shared memory is released
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

// Whether the streaming form serves this shape: rows of at least one full chunk, enough chunks to fill the GPU once. Measured on
// B200 (65536 x 4096, back-to-back launches): the amax pass gains 10 % (96 % of the copy rate) and mxfp8 9 % (90 %); the
// e2m1 formats are issue-bound rather than load-bound and lose, so they keep the register form.
static bool use_ring(int mode, int64_t m, int64_t k) {
  if (mode != TF_FMT_MXFP8 && mode != kModeAmax) return false;
  const int64_t cpr = ((k >> 4) + kRingChunkVecs - 1) / kRingChunkVecs;
  return k >= 2048 && m * cpr >= 2 * (int64_t)sm_count();
}

struct RingLaunch {
  unsigned grid;
  int stages;
  size_t smem;
};

// Ring depth and CTAs per SM: stages x 4 KB per CTA, CTAs x that per SM in flight.
static RingLaunch ring_launch(int mode, int64_t m, int64_t k) {
  RingLaunch r;
  r.stages = 4;
  const int ctas_per_sm = mode == kModeAmax ? 8 : 6;
  r.smem = (size_t)r.stages * kRingChunkBytes + 8 * (size_t)r.stages;
  const int64_t cpr = ((k >> 4) + kRingChunkVecs - 1) / kRingChunkVecs;
  const int64_t total = m * cpr, cap = (int64_t)sm_count() * ctas_per_sm;
  r.grid = (unsigned)(total < cap ? total : cap);
  return r;
}

template <int MODE>
static cudaError_t ring_configure() {
  static thread_local int configured_dev = -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (configured_dev == dev) return cudaSuccess;
  e = cudaFuncSetAttribute(ring_rows_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingMaxStages * (kRingChunkBytes + 8));
  if (e != cudaSuccess) return e;
  // the ring is all these kernels use of the SM's memory: let the carve-out hold as many CTAs' rings as possible
  e = cudaFuncSetAttribute(ring_rows_kernel<MODE>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return e;
  configured_dev = dev;
  return cudaSuccess;
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
  if (use_ring(FMT, m, k)) {
    int* status = device_status_words();
    if (!status) return fail(TF_ERR_CUDA, "%s: cannot locate the device status words", fn);
    TF_CUDA(ring_configure<FMT>());
    const RingLaunch rl = ring_launch(FMT, m, k);
    TF_CUDA(launch_dependent(ring_rows_kernel<FMT>, dim3(rl.grid), dim3(kRingThreads), rl.smem, stream, static_cast<const uint8_t*>(x), m, k, ldx,
                             static_cast<uint8_t*>(codes), static_cast<uint8_t*>(scales), (int)(layout == TF_SCALES_SWIZZLED), gs, gs_out,
                             (unsigned int*)nullptr, status, rl.stages));
    return TF_OK;
  }
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
    if (use_ring(kModeAmax, m, k)) {
      int* status = device_status_words();
      if (!status) return fail(TF_ERR_CUDA, "%s: cannot locate the device status words", __func__);
      TF_CUDA(ring_configure<kModeAmax>());
      const RingLaunch rl = ring_launch(kModeAmax, m, k);
      ring_rows_kernel<kModeAmax><<<rl.grid, kRingThreads, rl.smem, stream>>>(static_cast<const uint8_t*>(x), m, k, ldx, nullptr, nullptr, 0, nullptr, nullptr,
                                                                              reinterpret_cast<unsigned int*>(out), status, rl.stages);
      TF_LAUNCH_CHECK();
      finalize_global_scale_kernel<<<1, 1, 0, stream>>>(out);
      TF_LAUNCH_CHECK();
      return TF_OK;
    }
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
