// Block-scaled GEMM for sm_100a: out[M,N] = bf16( sum_k deq(a)[m,k] * deq(b)[n,k] ), f32 accumulation in tensor memory.
//
// One persistent CTA per SM walks output tiles of 128 x BLOCK_N. Three warp roles:
//   warp 0   operand loads: TMA tiled loads of the A and B code tiles (128-byte swizzle) into a ring of shared-memory stages,
//            signalled through mbarriers (complete_tx). ONE instruction per stage: lane 0 loads the A tile, lanes 1-2 the
//            128-row halves of the B tile (issuing a TMA copy costs the issuing thread 40-90 clocks; six copies issued one
//            after another by one thread made that thread, not the memory system, the limit of the whole kernel)
//   warp 6   scale loads: bulk copies of the pre-swizzled scale tiles of the same stage, again one instruction (lane 0 the A
//            scales, lanes 1-2 the B scales); both load warps arrive on the stage's "full" barrier with their own byte counts
//   warp 1   MMA issuer: copies the scale tiles shared -> tensor memory (tcgen05.cp) and issues
//            tcgen05.mma.kind::{mxf8f6f4, mxf4, mxf4nvf4}.block_scale, 4 per stage (32 bytes of K each); tcgen05.commit frees
//            the stage and, after the last one, hands the accumulator to the epilogue
//   warps 2-5 and 7-10   epilogue, two groups of four warps: a warp reads its 32 lanes of the accumulator (tcgen05.ld), the groups
//            share the columns (even / odd 32-column chunks); scale, fused epilogue (none / SiLU gate / residual add), bf16
//            stores. With short K (10-20 stages per tile) one group of four could not drain a tile as fast as the MMAs fill one
// The accumulator is double-buffered in tensor memory (overlapped for 256-column tiles, see TileCfg), so a tile's epilogue
// runs while the next tile's MMAs are issued.
// No TMA multicast, no clusters. Every mbarrier wait is bounded (about one second): on a timeout the kernel records
// TF_ERR_DEVICE_TIMEOUT in a device status word, every role leaves its loop, tensor memory is freed and the kernel returns.
//
// Scale layout consumed: the 512-byte 128x4 tiles described in the header; one tile feeds 4 tensor-memory columns through
// tcgen05.cp.32x128b.warpx4, byte k of a column being the scale of K-block k (selected by the SF-id field of the instruction
// descriptor for the MX formats; NVFP4 uses all four bytes per MMA).
#include <cuda.h>

#include <atomic>
#include <cstdlib>

#include "async_copy.cuh"
#include "quant_core.cuh"

namespace tf {

__device__ int g_device_status[2];  // [0] status, [1] detail

constexpr int kBlockM = 128;
constexpr int kStageKBytes = 128;  // bytes of K per row per stage: one 128-byte swizzle atom
constexpr int kAStageBytes = kBlockM * kStageKBytes;
constexpr int kGemmThreads = 352;  // 11 warps: operand loads, MMA issue, epilogue group 0 (4), scale loads, epilogue group 1 (4)
constexpr int kPairThreads = 192;  // the CTA-pair kernel keeps one load warp
constexpr int kSmemLimit = 227 * 1024;
constexpr unsigned long long kWaitLimitNs = 1000000000ull;

template <int FMT>
struct FmtTraits;
template <>
struct FmtTraits<TF_FMT_MXFP8> {
  static constexpr int kSfTiles = 1;  // 512-byte scale tiles per operand row-tile per stage
  static constexpr uint32_t kElemFormat = 0, kScaleIsE8 = 1;
};
template <>
struct FmtTraits<TF_FMT_MXFP4> {
  static constexpr int kSfTiles = 2;
  static constexpr uint32_t kElemFormat = 1, kScaleIsE8 = 1;
};
template <>
struct FmtTraits<TF_FMT_NVFP4> {
  static constexpr int kSfTiles = 4;
  static constexpr uint32_t kElemFormat = 1, kScaleIsE8 = 0;
};

template <int FMT, int BLOCK_N>
struct TileCfg {
  static constexpr int kNB = BLOCK_N / 128;  // 128-row halves of the B tile
  static constexpr int kST = FmtTraits<FMT>::kSfTiles;
  static constexpr int kBStageBytes = BLOCK_N * kStageKBytes;
  static constexpr int kSfaStageBytes = kST * 512;
  static constexpr int kSfbStageBytes = kST * 512 * kNB;
  static constexpr int kStageBytes = kAStageBytes + kBStageBytes + kSfaStageBytes + kSfbStageBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kStagesRaw = (kSmemLimit - 1024 - kBarrierBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;
  // Tensor memory (512 columns): two accumulators used by alternate tiles, so that the epilogue of one tile runs under the
  // MMAs of the next, then two scale buffers used by alternate stages. Two 256-column accumulators plus 96 scale columns do
  // not fit, so with BLOCK_N = 256 the accumulators OVERLAP: accumulator 1 starts at column 160 and shares columns
  // [160, 256) with accumulator 0. The epilogue first moves the shared columns of its tile into registers, then releases
  // the next tile's MMAs, then drains the rest. With BLOCK_N = 128 the accumulators are disjoint.
  static constexpr int kAccStride = BLOCK_N == 256 ? 160 : BLOCK_N;  // first column of accumulator 1
  static constexpr int kOverlapChunks = BLOCK_N == 256 ? 3 : 0;      // 32-column chunks both accumulators cover
  static constexpr int kTmemSfSet = kST * 4 * (1 + kNB);             // columns of one scale buffer: A scales then B scales
  static constexpr int kTmemSfBase = kAccStride + BLOCK_N;           // 416 or 256
  static constexpr int kTmemSfa = kTmemSfBase;                       // first column of the A scales of buffer 0
  static constexpr int kTmemSfb = kTmemSfBase + kST * 4;             // first column of the B scales of buffer 0
  static constexpr int kTmemUsed = kTmemSfBase + 2 * kTmemSfSet;
  static constexpr int kTmemCols = 512;
  static_assert(kTmemUsed <= 512, "tensor memory budget");
};

struct GemmParams {
  int m, n, n_rows_b, k_bytes;
  int num_k_stages, sf_col_tiles;  // K stages per tile; 512-byte tiles per scale row-tile
  int m_blocks, n_blocks, num_tiles;
  int sfb_row_tiles;
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* a_gs;
  const float* b_gs;
  uint16_t* out;
  int64_t ldo;
  float* residual;
  unsigned int* out_amax;
  int splits, k_stages_per_split;  // split-K: every (tile, split) accumulates a K range into the f32 workspace
  float* ws;
  uint8_t* q_codes;   // optional MX-quantized copy of the output (same format as the operands), swizzled scales
  uint8_t* q_scales;
  int a_gs_rows;  // 0: a has one global scale; else a_gs[row / a_gs_rows] (row blocks quantized separately, e.g. gathered from ranks)
  int a_box_bytes;  // bytes one A load brings per stage: 128 bytes x the rows of its box (fewer than 128 rows when M is small)
  // Scattered output (tf_gemm_blockscaled_scatter): rows [i * scatter_rows, (i + 1) * scatter_rows) go to scatter_out[i], a
  // [scatter_rows, n] matrix with leading dimension ldo that may live in another GPU's memory (plain stores over NVLink).
  // scatter_rows is a multiple of 128, so a tile has one destination. 0: everything goes to `out`.
  int scatter_rows;
  uint16_t* scatter_out[8];
};

// The address of output row `row`: in `out`, or in the row block's own destination.
__device__ __forceinline__ uint16_t* out_row_ptr(const GemmParams& p, int row) {
  if (p.scatter_rows == 0) return p.out + (int64_t)row * p.ldo;
  const int owner = row / p.scatter_rows;
  uint16_t* base = p.scatter_out[0];
#pragma unroll
  for (int i = 1; i < 8; ++i)
    if (i == owner) base = p.scatter_out[i];
  return base + (int64_t)(row - owner * p.scatter_rows) * p.ldo;
}

// ---- PTX wrappers ----------------------------------------------------------------------------------------------------------
// ---- thread-block-cluster helpers (the 2-CTA kernel) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// tcgen05.commit of a CTA pair: arrives on the barrier at the same offset in both CTAs (a barrier signal, not a data multicast).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask) : "memory");
}
// TMA load issued by either CTA of a pair: the destination is this CTA's shared memory, the mbarrier may be the peer's
// (cta_group::2 lifts the same-CTA rule). No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
               : "memory");
}
__device__ __forceinline__ void tc_cp_sf_pair(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
template <int FMT>
__device__ __forceinline__ void tc_mma_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  if (FMT == TF_FMT_MXFP8) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n}" ::"r"(d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else if (FMT == TF_FMT_MXFP4) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n}" ::"r"(d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}" ::"r"(d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  }
}

// Bounded wait. Returns false when the limit ran out here or another role already gave up (abort flag).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where,
                                          unsigned long long limit_ns = kWaitLimitNs) {
  return mbar_wait_bounded(bar, parity, abort_flag, g_device_status, where, limit_ns);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(map),
               "r"(x), "r"(y), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
template <int FMT>
__device__ __forceinline__ void tc_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  if (FMT == TF_FMT_MXFP8) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n}" ::"r"(d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else if (FMT == TF_FMT_MXFP4) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n}" ::"r"(d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}" ::"r"(d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  }
}
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets row (lane base + t), v[j] = column (base + j).
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
      "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
        "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
        "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile stored by TMA with the 128-byte swizzle: rows 128 bytes apart, 8-row
// groups 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Descriptor of one 512-byte scale tile for tcgen05.cp.32x128b: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}

__device__ __forceinline__ uint64_t make_desc(uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; }
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xFFFFFFFF;\n selp.b32 %0, 1, 0, p;\n}" : "=r"(pred));
  return pred != 0;
}


// Self-test of the bounded wait: one thread waits on an mbarrier that nothing arrives at; the wait must give up after limit_ns,
// record TF_ERR_DEVICE_TIMEOUT (detail: wait 9) and return, leaving the context usable.
__global__ void bounded_wait_selftest_kernel(unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    (void)mbar_wait(smem_u32(&bar), 0, &abort_flag, 9, limit_ns);
  }
}

// ---- epilogue helpers ------------------------------------------------------------------------------------------------------
// Stores 32 consecutive bf16 outputs of one row (packed two per word) and applies the residual / amax side effects.
// The 32 outputs a thread holds are exactly one MX block of its row: amax, scale byte and codes by the quantizer's rules
// (quant_core.cuh), written as the A operand of the next GEMM. FMT is the operands' (and the output's) format.
template <int FMT>
__device__ __forceinline__ void store_chunk_quantized(const GemmParams& p, const uint32_t (&packed)[16], int row, int col) {
  if (FMT == TF_FMT_NVFP4) return;
  const uint32_t k = 0x7FFF7FFFu;
  uint32_t t = 0;
#pragma unroll
  for (int j = 0; j < 16; j += 2) t = __vimax3_u16x2(t, packed[j] & k, packed[j + 1] & k);
  const uint32_t mx = max(t & 0xFFFFu, t >> 16);
  const int emax = (FMT == TF_FMT_MXFP8) ? 8 : 2;
  const int e = (int)(mx >> 7) - emax;
  const uint32_t scale = (mx == 0) ? 127u : (uint32_t)max(e, 0);
  const uint32_t inv1 = (254u - scale) << 7;
  const uint32_t inv2 = inv1 | (inv1 << 16);
  uint32_t q[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) q[j] = mul_bf16x2(packed[j], inv2);
  if (FMT == TF_FMT_MXFP8) {
    uint32_t c[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      c[j] = cvt_e4m3x2(bf16lo_to_f32(q[2 * j]), bf16hi_to_f32(q[2 * j])) | (cvt_e4m3x2(bf16lo_to_f32(q[2 * j + 1]), bf16hi_to_f32(q[2 * j + 1])) << 16);
    uint4* dst = reinterpret_cast<uint4*>(p.q_codes + (int64_t)row * p.n + col);
    dst[0] = make_uint4(c[0], c[1], c[2], c[3]);
    dst[1] = make_uint4(c[4], c[5], c[6], c[7]);
  } else {
    uint32_t c[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) w |= cvt_e2m1x2(bf16lo_to_f32(q[4 * h + j]), bf16hi_to_f32(q[4 * h + j])) << (8 * j);
      c[h] = w;
    }
    *reinterpret_cast<uint4*>(p.q_codes + (int64_t)row * (p.n >> 1) + (col >> 1)) = make_uint4(c[0], c[1], c[2], c[3]);
  }
  p.q_scales[swizzled_scale_offset(row, col >> 5, ((p.n >> 5) + 3) >> 2)] = (uint8_t)scale;
}

__device__ __forceinline__ void store_256(void* dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t e, uint32_t f, uint32_t g, uint32_t h) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(a), "r"(b), "r"(c), "r"(d), "r"(e), "r"(f), "r"(g), "r"(h) : "memory");
}

template <int EPI, int FMT>
__device__ __forceinline__ void store_chunk(const GemmParams& p, const uint32_t (&packed)[16], int row, int col, uint32_t& amax2) {
  if (row >= p.m) return;
  if (p.q_codes && col + 32 <= p.n) store_chunk_quantized<FMT>(p, packed, row, col);
  if (!p.out) return;
  uint16_t* orow = out_row_ptr(p, row) + col;
  // 32-byte stores (whole L2 sectors, half as many store transactions per row) where the row's chunk is whole and 32-byte aligned
  const bool wide = col + 32 <= p.n && (reinterpret_cast<uintptr_t>(orow) & 31u) == 0;
  if (wide) {
    store_256(orow, packed[0], packed[1], packed[2], packed[3], packed[4], packed[5], packed[6], packed[7]);
    store_256(orow + 16, packed[8], packed[9], packed[10], packed[11], packed[12], packed[13], packed[14], packed[15]);
  }
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if (col + g * 8 + 8 <= p.n) {
      if (!wide) *reinterpret_cast<uint4*>(orow + g * 8) = make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
      if (p.out_amax) {
#pragma unroll
        for (int e = 0; e < 4; ++e) amax2 = __vmaxu2(amax2, packed[4 * g + e] & 0x7FFF7FFFu);
      }
      if (EPI == TF_EPI_RESIDUAL) {
        float4* rp = reinterpret_cast<float4*>(p.residual + (int64_t)row * p.n + col + g * 8);
        float4 r0 = rp[0], r1 = rp[1];
        r0.x = __fadd_rn(r0.x, bf16lo_to_f32(packed[4 * g]));
        r0.y = __fadd_rn(r0.y, bf16hi_to_f32(packed[4 * g]));
        r0.z = __fadd_rn(r0.z, bf16lo_to_f32(packed[4 * g + 1]));
        r0.w = __fadd_rn(r0.w, bf16hi_to_f32(packed[4 * g + 1]));
        r1.x = __fadd_rn(r1.x, bf16lo_to_f32(packed[4 * g + 2]));
        r1.y = __fadd_rn(r1.y, bf16hi_to_f32(packed[4 * g + 2]));
        r1.z = __fadd_rn(r1.z, bf16lo_to_f32(packed[4 * g + 3]));
        r1.w = __fadd_rn(r1.w, bf16hi_to_f32(packed[4 * g + 3]));
        rp[0] = r0;
        rp[1] = r1;
      }
    }
  }
}

// Which epilogue warps read chunk `c` (32 accumulator columns): GRP < 0: this warp reads all of them (the CTA-pair kernel has four
// epilogue warps); GRP 0 / 1: the one-CTA kernel's two groups of four warps share the columns, alternating between the groups (with the
// SiLU gate: by the gate chunk; its up chunk goes with it).
template <int GRP, int EPI, int BLOCK_N>
__device__ __forceinline__ constexpr bool chunk_is_mine(int c) {
  // the unit a group owns is a PAIR of adjacent chunks where there are at least four (a thread then writes 128 contiguous bytes of its
  // output row, a whole line), else single chunks
  constexpr int kUnits = (EPI == TF_EPI_SILU_GATE) ? BLOCK_N / 64 : BLOCK_N / 32;
  const int u = (EPI == TF_EPI_SILU_GATE) ? (c % (BLOCK_N / 64)) : c;
  return GRP < 0 || ((kUnits >= 4 ? (u >> 1) : u) & 1) == GRP;
}

// One tile's epilogue for accumulator BUF (compile time, so that the chunks held in registers are indexed statically).
// t_acc: tensor-memory address of the accumulator for this warp's 32 lanes. Returns after the last store.
template <int FMT, int BLOCK_N, int EPI, int BUF, int GRP, bool CLUSTER_BAR = false>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t t_acc, uint32_t bar_release, int lane, int row, int col0, float alpha,
                                              uint32_t& amax2) {
  using Cfg = TileCfg<FMT, BLOCK_N>;
  constexpr int kOutCols = (EPI == TF_EPI_SILU_GATE) ? BLOCK_N / 2 : BLOCK_N;
  constexpr int kOv = Cfg::kOverlapChunks;
  constexpr int kOvFirst = (BUF == 0) ? (BLOCK_N / 32 - kOv) : 0;  // first chunk (of this accumulator) the other accumulator also covers
  uint32_t ov[kOv > 0 ? kOv : 1][32];  // rows of chunks this warp does not read are never touched and cost no registers
  bool any_ov = false;
#pragma unroll
  for (int i = 0; i < kOv; ++i) {
    if (chunk_is_mine<GRP, EPI, BLOCK_N>(kOvFirst + i)) {
      tc_ld32(t_acc + (kOvFirst + i) * 32, ov[i]);
      any_ov = true;
    }
  }
  if (any_ov) tc_wait_ld();
  // the columns shared with the other accumulator are in registers (or there are none): the next tile's MMAs may start
  tc_fence_before();
  __syncwarp();
  if (lane == 0) {
    if (CLUSTER_BAR) mbar_arrive_cluster(bar_release);
    else mbar_arrive(bar_release);
  }

#pragma unroll
  for (int c = 0; c < kOutCols / 32; ++c) {
    if (!chunk_is_mine<GRP, EPI, BLOCK_N>(c)) continue;
    uint32_t v[32], packed[16];
    const bool v_in_regs = kOv > 0 && c >= kOvFirst && c < kOvFirst + kOv;
    if (v_in_regs) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = ov[(c - kOvFirst) < 0 ? 0 : ((c - kOvFirst) >= kOv ? 0 : (c - kOvFirst))][j];
    } else {
      tc_ld32(t_acc + c * 32, v);
    }
    if (EPI == TF_EPI_SILU_GATE) {
      uint32_t u[32];
      const int cu = BLOCK_N / 64 + c;  // the up chunk that pairs with gate chunk c
      const bool u_in_regs = kOv > 0 && cu >= kOvFirst && cu < kOvFirst + kOv;
      if (u_in_regs) {
#pragma unroll
        for (int j = 0; j < 32; ++j) u[j] = ov[(cu - kOvFirst) < 0 ? 0 : ((cu - kOvFirst) >= kOv ? 0 : (cu - kOvFirst))][j];
      } else {
        tc_ld32(t_acc + cu * 32, u);
      }
      if (!v_in_regs || !u_in_regs) tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        // the GEMM result is bf16 (one rounding); the gate then reads it back as f32, as the unfused graph does
        const uint32_t g2 = pack_bf16x2(__fmul_rn(__uint_as_float(v[2 * j]), alpha), __fmul_rn(__uint_as_float(v[2 * j + 1]), alpha));
        const uint32_t u2 = pack_bf16x2(__fmul_rn(__uint_as_float(u[2 * j]), alpha), __fmul_rn(__uint_as_float(u[2 * j + 1]), alpha));
        const float lo = __fmul_rn(silu_f32(bf16lo_to_f32(g2)), bf16lo_to_f32(u2));
        const float hi = __fmul_rn(silu_f32(bf16hi_to_f32(g2)), bf16hi_to_f32(u2));
        packed[j] = pack_bf16x2(lo, hi);
      }
    } else {
      if (!v_in_regs) tc_wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j)
        packed[j] = pack_bf16x2(__fmul_rn(__uint_as_float(v[2 * j]), alpha), __fmul_rn(__uint_as_float(v[2 * j + 1]), alpha));
    }
    store_chunk<EPI, FMT>(p, packed, row, col0 + c * 32, amax2);
  }
}

// Split-K: dumps this (tile, split)'s raw f32 accumulator rows into the workspace [splits][M][acc columns].
template <int FMT, int BLOCK_N, int BUF, int GRP>
__device__ __forceinline__ void epilogue_partial(const GemmParams& p, uint32_t t_acc, uint32_t bar_release, int lane, int row, int col0,
                                                 float* __restrict__ ws_row) {
  using Cfg = TileCfg<FMT, BLOCK_N>;
  constexpr int kOv = Cfg::kOverlapChunks;
  constexpr int kOvFirst = (BUF == 0) ? (BLOCK_N / 32 - kOv) : 0;
  uint32_t ov[kOv > 0 ? kOv : 1][32];
  bool any_ov = false;
#pragma unroll
  for (int i = 0; i < kOv; ++i) {
    if (chunk_is_mine<GRP, TF_EPI_NONE, BLOCK_N>(kOvFirst + i)) {
      tc_ld32(t_acc + (kOvFirst + i) * 32, ov[i]);
      any_ov = true;
    }
  }
  if (any_ov) tc_wait_ld();
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar_release);
#pragma unroll
  for (int c = 0; c < BLOCK_N / 32; ++c) {
    if (!chunk_is_mine<GRP, TF_EPI_NONE, BLOCK_N>(c)) continue;
    uint32_t v[32];
    const bool in_regs = kOv > 0 && c >= kOvFirst && c < kOvFirst + kOv;
    if (in_regs) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = ov[(c - kOvFirst) < 0 ? 0 : ((c - kOvFirst) >= kOv ? 0 : (c - kOvFirst))][j];
    } else {
      tc_ld32(t_acc + c * 32, v);
      tc_wait_ld();
    }
    if (row < p.m) {
      const int col = col0 + c * 32;
#pragma unroll
      for (int g = 0; g < 8; ++g)
        if (col + g * 4 + 4 <= p.n)
          *reinterpret_cast<uint4*>(ws_row + col + g * 4) = make_uint4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
    }
  }
}

// Split-K second pass: sums the partials in split order (deterministic), then the same epilogue arithmetic as the one-pass
// kernel. n_acc = accumulator columns (2 * n with the SiLU gate), one thread per 8 output columns.
template <int EPI, int QFMT>  // QFMT: -1, or the MX format of a quantized copy of the output
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ ws, int splits, int m, int n, int n_acc, const float* a_gs,
                                                            const float* b_gs, uint16_t* __restrict__ out, int64_t ldo, float* __restrict__ residual,
                                                            unsigned int* __restrict__ out_amax, uint8_t* __restrict__ q_codes,
                                                            uint8_t* __restrict__ q_scales, int a_gs_rows) {
  griddep_launch_dependents();
  griddep_wait();
  const float alpha0 = (a_gs && b_gs) ? __fmul_rn(__ldg(a_gs), __ldg(b_gs)) : 1.0f;
  const int nvec = n >> 3;
  const int64_t total = (int64_t)m * nvec;
  const int64_t plane = (int64_t)m * n_acc;
  uint32_t amax2 = 0;
  // every thread runs the same number of rounds (the quantizer's shuffles need whole warps); n is a multiple of 32 when a
  // quantized copy is asked for, so the 4 lanes of one block have data together
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x; i0 < total; i0 += stride) {
    const int64_t i = i0 + threadIdx.x;
    const bool live = i < total;
    if (!live && QFMT < 0) continue;
    const int row = live ? (int)(i / nvec) : 0, col = live ? (int)(i - (int64_t)row * nvec) * 8 : 0;
    float acc[8], up[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = up[j] = 0.0f;
    const float alpha = (a_gs && b_gs && a_gs_rows > 0) ? __fmul_rn(__ldg(a_gs + row / a_gs_rows), __ldg(b_gs)) : alpha0;
    const float* base = ws + (int64_t)row * n_acc + col;
    for (int sp = 0; sp < (live ? splits : 0); ++sp) {
      const float4 x0 = __ldcs(reinterpret_cast<const float4*>(base + sp * plane)), x1 = __ldcs(reinterpret_cast<const float4*>(base + sp * plane) + 1);
      acc[0] += x0.x; acc[1] += x0.y; acc[2] += x0.z; acc[3] += x0.w; acc[4] += x1.x; acc[5] += x1.y; acc[6] += x1.z; acc[7] += x1.w;
      if (EPI == TF_EPI_SILU_GATE) {
        const float4 u0 = __ldcs(reinterpret_cast<const float4*>(base + n + sp * plane)), u1 = __ldcs(reinterpret_cast<const float4*>(base + n + sp * plane) + 1);
        up[0] += u0.x; up[1] += u0.y; up[2] += u0.z; up[3] += u0.w; up[4] += u1.x; up[5] += u1.y; up[6] += u1.z; up[7] += u1.w;
      }
    }
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t g2 = pack_bf16x2(__fmul_rn(acc[2 * j], alpha), __fmul_rn(acc[2 * j + 1], alpha));
      if (EPI == TF_EPI_SILU_GATE) {
        const uint32_t u2 = pack_bf16x2(__fmul_rn(up[2 * j], alpha), __fmul_rn(up[2 * j + 1], alpha));
        packed[j] = pack_bf16x2(__fmul_rn(silu_f32(bf16lo_to_f32(g2)), bf16lo_to_f32(u2)), __fmul_rn(silu_f32(bf16hi_to_f32(g2)), bf16hi_to_f32(u2)));
      } else {
        packed[j] = g2;
      }
      amax2 = __vmaxu2(amax2, packed[j] & 0x7FFF7FFFu);
    }
    if (QFMT >= 0) {
      uint32_t c0, c1, sc;
      quantize_vec8<(QFMT < 0 ? 0 : QFMT)>(make_uint4(packed[0], packed[1], packed[2], packed[3]), 0.0f, 0.0f, c0, c1, sc);
      if (live) store_quantized<(QFMT < 0 ? 0 : QFMT)>(q_codes, q_scales, 1, row, col >> 3, n, c0, c1, sc);
    }
    if (!live) continue;
    if (out) *reinterpret_cast<uint4*>(out + (int64_t)row * ldo + col) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    if (EPI == TF_EPI_RESIDUAL) {
      float4* rp = reinterpret_cast<float4*>(residual + (int64_t)row * n + col);
      float4 r0 = rp[0], r1 = rp[1];
      r0.x = __fadd_rn(r0.x, bf16lo_to_f32(packed[0])); r0.y = __fadd_rn(r0.y, bf16hi_to_f32(packed[0]));
      r0.z = __fadd_rn(r0.z, bf16lo_to_f32(packed[1])); r0.w = __fadd_rn(r0.w, bf16hi_to_f32(packed[1]));
      r1.x = __fadd_rn(r1.x, bf16lo_to_f32(packed[2])); r1.y = __fadd_rn(r1.y, bf16hi_to_f32(packed[2]));
      r1.z = __fadd_rn(r1.z, bf16lo_to_f32(packed[3])); r1.w = __fadd_rn(r1.w, bf16hi_to_f32(packed[3]));
      rp[0] = r0;
      rp[1] = r1;
    }
  }
  if (out_amax) {
    uint32_t mx = max(amax2 & 0xFFFFu, amax2 >> 16);
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if ((threadIdx.x & 31) == 0 && mx) atomicMax(out_amax, mx << 16);
  }
}

// ---- the kernel ------------------------------------------------------------------------------------------------------------
template <int FMT, int BLOCK_N, int EPI, bool SPLITK>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                                            const __grid_constant__ CUtensorMap tma_b, const GemmParams p) {
  using Cfg = TileCfg<FMT, BLOCK_N>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kNB = Cfg::kNB;
  constexpr int kST = Cfg::kST;
  constexpr int kOutCols = (EPI == TF_EPI_SILU_GATE) ? BLOCK_N / 2 : BLOCK_N;  // output columns per tile
  static_assert(EPI != TF_EPI_SILU_GATE || BLOCK_N == 256, "the SiLU-gate epilogue pairs a 128-column gate tile with its up tile");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a = smem_base;
  const uint32_t smem_b = smem_a + kStages * kAStageBytes;
  const uint32_t smem_sfa = smem_b + kStages * Cfg::kBStageBytes;
  const uint32_t smem_sfb = smem_sfa + kStages * Cfg::kSfaStageBytes;
  const uint32_t bars = smem_sfb + kStages * Cfg::kSfbStageBytes;  // 8-byte aligned
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kStages, bar_tmem_full = bars + 16 * kStages, bar_tmem_empty = bar_tmem_full + 8;
  const uint32_t tmem_slot = bar_tmem_empty + 8;
  const uint32_t abort_slot = tmem_slot + 4;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + (abort_slot - smem_base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  griddep_launch_dependents();  // the next kernel on the stream may be scheduled; it waits for this one before touching memory

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 2);  // the operand-load warp and the scale-load warp
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_tmem_full, 1);
    mbar_init(bar_tmem_empty, 8);  // every epilogue warp, once it holds its share of the columns both accumulators cover
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // whole warp: allocate tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  griddep_wait();  // barriers and tensor memory are set up; nothing of global memory was touched before the previous kernel is done

  if (warp == 0 || warp == 6) {
    // ---------------- load warps: warp 0 the operand tiles (TMA), warp 6 the scale tiles (bulk copies) ----------------
    // The whole warp runs the loops; lane 0 serves the A side, lane 1 + nb the 128-row half nb of the B tile, so that one
    // instruction per stage issues all of the warp's copies.
    const bool scales = warp == 6;
    const int nb = lane - 1;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
      const int split = SPLITK ? tile / (p.m_blocks * p.n_blocks) : 0;
      const int rest = SPLITK ? tile % (p.m_blocks * p.n_blocks) : tile;
      const int m_blk = rest % p.m_blocks, n_blk = rest / p.m_blocks;
      const int ks_begin = split * p.k_stages_per_split;
      const int ks_end = min(ks_begin + p.k_stages_per_split, p.num_k_stages);
      int n_b_ok = 0;  // B halves that lie inside the matrix (uniform)
#pragma unroll
      for (int i = 0; i < kNB; ++i)
        n_b_ok += (((EPI == TF_EPI_SILU_GATE) ? i * p.n + n_blk * 128 : n_blk * BLOCK_N + i * 128) < p.n_rows_b) ? 1 : 0;
      // this lane's copy: source row (operands) or scale row-tile, destination inside a stage
      const int my_row = lane == 0 ? m_blk * kBlockM : ((EPI == TF_EPI_SILU_GATE) ? nb * p.n + n_blk * 128 : n_blk * BLOCK_N + nb * 128);
      const bool mine = lane == 0 || (lane <= kNB && my_row < p.n_rows_b);
      const CUtensorMap* my_map = lane == 0 ? &tma_a : &tma_b;
      const uint32_t my_dst = scales ? (lane == 0 ? smem_sfa : smem_sfb + (uint32_t)(nb < 0 ? 0 : nb) * kST * 512)
                                     : (lane == 0 ? smem_a : smem_b + (uint32_t)(nb < 0 ? 0 : nb) * 128 * kStageKBytes);
      const uint32_t my_stage_bytes = scales ? (lane == 0 ? Cfg::kSfaStageBytes : Cfg::kSfbStageBytes) : (lane == 0 ? kAStageBytes : Cfg::kBStageBytes);
      const uint8_t* my_sf = (lane == 0 ? p.sfa : p.sfb) + (int64_t)((lane == 0 ? my_row : (my_row < 0 ? 0 : my_row)) >> 7) * p.sf_col_tiles * 512;
      for (int ks = ks_begin; ks < ks_end; ++ks) {
        ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, 1);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        const uint32_t full = bar_full + 8 * stage;
        if (scales) {
          int sf_tiles = p.sf_col_tiles - ks * kST;
          sf_tiles = sf_tiles > kST ? kST : sf_tiles;
          const uint32_t sf_bytes = (uint32_t)sf_tiles * 512u;
          if (lane == 0) mbar_expect_tx(full, sf_bytes * (uint32_t)(1 + n_b_ok));
          __syncwarp();
          if (mine) bulk_load(my_dst + stage * my_stage_bytes, my_sf + (int64_t)ks * kST * 512, sf_bytes, full);
        } else {
          if (lane == 0) mbar_expect_tx(full, (uint32_t)p.a_box_bytes + (uint32_t)n_b_ok * (128u * kStageKBytes));
          __syncwarp();
          if (mine) tma_load_2d(my_dst + stage * my_stage_bytes, my_map, ks * kStageKBytes, my_row, full);
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (!ok && lane == 0) {
      // give copies already in flight time to land before shared memory is released
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp runs the loops (so every value below is warp-uniform and lives in the uniform datapath); one elected lane
    // issues the tcgen05 instructions. A full stage is straight-line code: its descriptors differ from the stage's base by
    // compile-time constants added to the low word (the 14-bit address field cannot carry out for addresses below 256 KB).
    constexpr uint32_t idesc_base = (FmtTraits<FMT>::kElemFormat << 7) | (FmtTraits<FMT>::kElemFormat << 10) | ((uint32_t)(BLOCK_N >> 3) << 17) |
                                    (FmtTraits<FMT>::kScaleIsE8 << 23) | ((uint32_t)(kBlockM >> 4) << 24);
    constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024 B, version 1, SWIZZLE_128B
    constexpr uint32_t kDescHiSf = (128u >> 4) | (1u << 14);                   // SBO 128 B, version 1, no swizzle
    const bool elected = elect_one();
    int stage = 0;
    uint32_t phase = 0, tile_phase = 0, sf_buf = 0, acc_buf = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
      ok = mbar_wait(bar_tmem_empty, tile_phase ^ 1, abort_flag, 2);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tmem_acc = tmem_base + acc_buf * Cfg::kAccStride;
      acc_buf ^= 1;
      const int split = SPLITK ? tile / (p.m_blocks * p.n_blocks) : 0;
      const int n_blk = (SPLITK ? tile % (p.m_blocks * p.n_blocks) : tile) / p.m_blocks;
      const int ks_begin = split * p.k_stages_per_split;
      const int ks_end = min(ks_begin + p.k_stages_per_split, p.num_k_stages);
      bool all_b = true;
      bool b_ok[kNB];
#pragma unroll
      for (int nb = 0; nb < kNB; ++nb) {
        b_ok[nb] = ((EPI == TF_EPI_SILU_GATE) ? nb * p.n + n_blk * 128 : n_blk * BLOCK_N + nb * 128) < p.n_rows_b;
        all_b = all_b && b_ok[nb];
      }
      for (int ks = ks_begin; ks < ks_end; ++ks) {
        ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, 3);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_sfa = tmem_base + Cfg::kTmemSfa + sf_buf * Cfg::kTmemSfSet;
        const uint32_t tmem_sfb = tmem_base + Cfg::kTmemSfb + sf_buf * Cfg::kTmemSfSet;
        sf_buf ^= 1;
        const uint32_t sfa_lo = ((smem_sfa + stage * Cfg::kSfaStageBytes) & 0x3FFFFu) >> 4;
        const uint32_t sfb_lo = ((smem_sfb + stage * Cfg::kSfbStageBytes) & 0x3FFFFu) >> 4;
        const uint32_t a_lo = (((smem_a + stage * kAStageBytes) & 0x3FFFFu) >> 4) | (1u << 16);
        const uint32_t b_lo = (((smem_b + stage * Cfg::kBStageBytes) & 0x3FFFFu) >> 4) | (1u << 16);
        const int sf_left = p.sf_col_tiles - ks * kST;
        const int k_left = p.k_bytes - ks * kStageKBytes;
        const uint32_t first = (ks > ks_begin) ? 1u : 0u;
        if (elected) {
          if (sf_left >= kST && k_left >= kStageKBytes && all_b) {
#pragma unroll
            for (int t = 0; t < kST; ++t) {
              tc_cp_sf(tmem_sfa + t * 4, make_desc(sfa_lo + t * 32, kDescHiSf));
#pragma unroll
              for (int nb = 0; nb < kNB; ++nb) tc_cp_sf(tmem_sfb + (t * kNB + nb) * 4, make_desc(sfb_lo + (nb * kST + t) * 32, kDescHiSf));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              constexpr int kDummy = 0;
              (void)kDummy;
              const int t = (FMT == TF_FMT_MXFP8) ? 0 : (FMT == TF_FMT_MXFP4) ? (j >> 1) : j;
              const uint32_t sf_id = (FMT == TF_FMT_MXFP8) ? (uint32_t)j : (FMT == TF_FMT_MXFP4) ? (uint32_t)((j & 1) * 2) : 0u;
              tc_mma<FMT>(tmem_acc, make_desc(a_lo + j * 2, kDescHiSw128), make_desc(b_lo + j * 2, kDescHiSw128),
                          idesc_base | (sf_id << 4) | (sf_id << 29), tmem_sfa + t * 4, tmem_sfb + t * kNB * 4, j > 0 ? 1u : first);
            }
          } else {  // ragged stage: fewer scale tiles, fewer MMAs or a B half that lies outside the matrix
            const int sf_tiles = sf_left > kST ? kST : sf_left;
            for (int t = 0; t < sf_tiles; ++t) {
              tc_cp_sf(tmem_sfa + t * 4, make_desc(sfa_lo + t * 32, kDescHiSf));
#pragma unroll
              for (int nb = 0; nb < kNB; ++nb)
                if (b_ok[nb]) tc_cp_sf(tmem_sfb + (t * kNB + nb) * 4, make_desc(sfb_lo + (nb * kST + t) * 32, kDescHiSf));
            }
            const int n_mma = k_left >= kStageKBytes ? 4 : (k_left + 31) >> 5;
            for (int j = 0; j < n_mma; ++j) {
              const int t = (FMT == TF_FMT_MXFP8) ? 0 : (FMT == TF_FMT_MXFP4) ? (j >> 1) : j;
              const uint32_t sf_id = (FMT == TF_FMT_MXFP8) ? (uint32_t)j : (FMT == TF_FMT_MXFP4) ? (uint32_t)((j & 1) * 2) : 0u;
              tc_mma<FMT>(tmem_acc, make_desc(a_lo + j * 2, kDescHiSw128), make_desc(b_lo + j * 2, kDescHiSw128),
                          idesc_base | (sf_id << 4) | (sf_id << 29), tmem_sfa + t * 4, tmem_sfb + t * kNB * 4, j > 0 ? 1u : first);
            }
          }
          tc_commit(bar_empty + 8 * stage);  // the stage is free once these MMAs have read it
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) break;
      if (elected) tc_commit(bar_tmem_full);  // accumulator complete
      __syncwarp();
      tile_phase ^= 1;
    }
  } else {
    // ---------------- epilogue (warps 2..5 = group 0, warps 7..10 = group 1; warp w reads lanes 32*(w%4) .. +31) ----------------
    const int q = warp & 3;
    const int grp = warp >= 7 ? 1 : 0;
    const float alpha = (FMT == TF_FMT_NVFP4) ? __fmul_rn(__ldg(p.a_gs), __ldg(p.b_gs)) : 1.0f;
    uint32_t tile_phase = 0, acc_buf = 0;
    uint32_t amax2 = 0;  // running max of |out| as two packed bf16 magnitudes
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
      const int split = SPLITK ? tile / (p.m_blocks * p.n_blocks) : 0;
      const int rest = SPLITK ? tile % (p.m_blocks * p.n_blocks) : tile;
      const int m_blk = rest % p.m_blocks, n_blk = rest / p.m_blocks;
      bool ok = mbar_wait(bar_tmem_full, tile_phase, abort_flag, 4);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m_blk * kBlockM + q * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
      const int col0 = n_blk * kOutCols;
      const float alpha_t = (FMT == TF_FMT_NVFP4 && p.a_gs_rows > 0) ? __fmul_rn(__ldg(p.a_gs + min(row, p.m - 1) / p.a_gs_rows), __ldg(p.b_gs)) : alpha;
      if (SPLITK) {
        float* ws_row = p.ws + ((int64_t)split * p.m + row) * p.n;
        if (acc_buf == 0) {
          if (grp == 0) epilogue_partial<FMT, BLOCK_N, 0, 0>(p, t_row, bar_tmem_empty, lane, row, col0, ws_row);
          else epilogue_partial<FMT, BLOCK_N, 0, 1>(p, t_row, bar_tmem_empty, lane, row, col0, ws_row);
        } else {
          if (grp == 0) epilogue_partial<FMT, BLOCK_N, 1, 0>(p, t_row + Cfg::kAccStride, bar_tmem_empty, lane, row, col0, ws_row);
          else epilogue_partial<FMT, BLOCK_N, 1, 1>(p, t_row + Cfg::kAccStride, bar_tmem_empty, lane, row, col0, ws_row);
        }
      } else if (acc_buf == 0) {
        if (grp == 0) epilogue_tile<FMT, BLOCK_N, EPI, 0, 0>(p, t_row, bar_tmem_empty, lane, row, col0, alpha_t, amax2);
        else epilogue_tile<FMT, BLOCK_N, EPI, 0, 1>(p, t_row, bar_tmem_empty, lane, row, col0, alpha_t, amax2);
      } else {
        if (grp == 0) epilogue_tile<FMT, BLOCK_N, EPI, 1, 0>(p, t_row + Cfg::kAccStride, bar_tmem_empty, lane, row, col0, alpha_t, amax2);
        else epilogue_tile<FMT, BLOCK_N, EPI, 1, 1>(p, t_row + Cfg::kAccStride, bar_tmem_empty, lane, row, col0, alpha_t, amax2);
      }
      acc_buf ^= 1;
      tile_phase ^= 1;
    }
    if (!SPLITK && p.out_amax) {  // one atomic per warp
      uint32_t mx = max(amax2 & 0xFFFFu, amax2 >> 16);
      for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
      if (lane == 0 && mx) atomicMax(p.out_amax, mx << 16);
    }
  }

  // ---------------- teardown: every thread arrives, then the allocating warp frees tensor memory ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
  }
}

// ---- the 2-CTA kernel ------------------------------------------------------------------------------------------------------
// Two CTAs of a cluster (a pair of SMs) compute one 256 x 256 tile with tcgen05.mma.cta_group::2: CTA r of the pair holds rows
// [128 r, 128 r + 128) of the A tile and of the B tile in its own shared memory and the accumulator of its 128 rows in its own
// tensor memory. Per 32 K MACs per K-byte each SM now fills 256 operand rows instead of 384, which is what the one-CTA kernel
// is bound by. Each CTA loads its own halves with plain (non-multicast) TMA; the scale tiles of all 256 B rows are loaded by
// both CTAs (4 KB per stage). The leader (rank 0) issues the scale copies and MMAs for both; barriers that both CTAs wait on
// are signalled with tcgen05.commit's multicast arrive; the peer's producer and epilogue signal the leader through
// cluster-mapped mbarrier addresses. Same bounded waits and teardown as the one-CTA kernel, plus a cluster barrier at both ends.
template <int FMT, int EPI>
struct PairCfg {
  static constexpr int kST = FmtTraits<FMT>::kSfTiles;
  static constexpr int kBHalfBytes = 128 * kStageKBytes;
  static constexpr int kSfaStageBytes = kST * 512;
  static constexpr int kSfbStageBytes = kST * 512 * 2;
  static constexpr int kStageBytes = kAStageBytes + kBHalfBytes + kSfaStageBytes + kSfbStageBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kStagesRaw = (kSmemLimit - 1024 - kBarrierBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;
};

template <int FMT, int EPI>
__global__ void __launch_bounds__(kPairThreads, 1) gemm_blockscaled_pair_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                                                 const __grid_constant__ CUtensorMap tma_b,
                                                                                 const __grid_constant__ CUtensorMap tma_sfa,
                                                                                 const __grid_constant__ CUtensorMap tma_sfb, const GemmParams p) {
  constexpr int BLOCK_N = 256;
  using Cfg = TileCfg<FMT, BLOCK_N>;  // tensor-memory layout (per CTA: 128 lanes x 256 columns) is the one-CTA kernel's
  using PC = PairCfg<FMT, EPI>;
  constexpr int kStages = PC::kStages;
  constexpr int kST = PC::kST;
  constexpr int kNB = 2;
  constexpr int kOutCols = (EPI == TF_EPI_SILU_GATE) ? BLOCK_N / 2 : BLOCK_N;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a = smem_base;
  const uint32_t smem_b = smem_a + kStages * kAStageBytes;
  const uint32_t smem_sfa = smem_b + kStages * PC::kBHalfBytes;
  const uint32_t smem_sfb = smem_sfa + kStages * PC::kSfaStageBytes;
  const uint32_t bars = smem_sfb + kStages * PC::kSfbStageBytes;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kStages, bar_tmem_full = bars + 16 * kStages, bar_tmem_empty = bar_tmem_full + 8;
  const uint32_t tmem_slot = bar_tmem_empty + 8;
  const uint32_t abort_slot = tmem_slot + 4;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + (abort_slot - smem_base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 2);   // one arrive.expect_tx from each CTA's producer (used in the leader only)
      mbar_init(bar_empty + 8 * s, 1);  // the leader's commit arrives in both CTAs
    }
    mbar_init(bar_tmem_full, 1);
    mbar_init(bar_tmem_empty, 8);  // 4 epilogue warps of each CTA (used in the leader only)
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the same warp of both CTAs allocates the pair's tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anything crosses
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ---------------- producer (each CTA loads its own halves; completion is counted on the leader's barrier) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
        const int m_blk = tile % p.m_blocks, n_blk = tile / p.m_blocks;
        int b_row[kNB], b_rt[kNB];
        bool b_ok[kNB];
#pragma unroll
        for (int nb = 0; nb < kNB; ++nb) {
          b_row[nb] = (EPI == TF_EPI_SILU_GATE) ? nb * p.n + n_blk * 128 : n_blk * BLOCK_N + nb * 128;
          b_rt[nb] = b_row[nb] >> 7;
          b_ok[nb] = b_row[nb] < p.n_rows_b;
        }
        const int a_row = m_blk * 256 + (int)rank * 128;
        const bool a_ok = a_row < p.m;
        for (int ks = 0; ks < p.num_k_stages; ++ks) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, 1)) {
            ok = false;
            break;
          }
          // scale tiles come through tensor maps too ([tiles, 512 bytes] as 128 x u32 rows; a box is always kST tiles, rows
          // past the end read as zero), because only the tensor form of the copy may signal the peer's barrier
          constexpr uint32_t sf_bytes = (uint32_t)kST * 512u;
          uint32_t tx = 0;
          if (a_ok) tx += kAStageBytes + sf_bytes;
          if (b_ok[rank]) tx += PC::kBHalfBytes;
#pragma unroll
          for (int nb = 0; nb < kNB; ++nb)
            if (b_ok[nb]) tx += sf_bytes;
          const uint32_t full = mapa_shared(bar_full + 8 * stage, 0);  // the leader's barrier
          mbar_expect_tx_cluster(full, tx);
          if (a_ok) {
            tma_load_2d_pair(smem_a + stage * kAStageBytes, &tma_a, ks * kStageKBytes, a_row, full);
            tma_load_2d_pair(smem_sfa + stage * PC::kSfaStageBytes, &tma_sfa, 0, (a_row >> 7) * p.sf_col_tiles + ks * kST, full);
          }
          if (b_ok[rank]) tma_load_2d_pair(smem_b + stage * PC::kBHalfBytes, &tma_b, ks * kStageKBytes, b_row[rank], full);
#pragma unroll
          for (int nb = 0; nb < kNB; ++nb)
            if (b_ok[nb]) tma_load_2d_pair(smem_sfb + stage * PC::kSfbStageBytes + nb * kST * 512, &tma_sfb, 0, b_rt[nb] * p.sf_col_tiles + ks * kST, full);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (rank == 0) {
      constexpr uint32_t idesc_base = (FmtTraits<FMT>::kElemFormat << 7) | (FmtTraits<FMT>::kElemFormat << 10) | ((uint32_t)(BLOCK_N >> 3) << 17) |
                                      (FmtTraits<FMT>::kScaleIsE8 << 23) | ((uint32_t)(256 >> 4) << 24);
      constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kDescHiSf = (128u >> 4) | (1u << 14);
      const bool elected = elect_one();
      int stage = 0;
      uint32_t phase = 0, tile_phase = 0, sf_buf = 0, acc_buf = 0;
      bool ok = true;
      for (int tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
        ok = mbar_wait(bar_tmem_empty, tile_phase ^ 1, abort_flag, 2);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + acc_buf * Cfg::kAccStride;
        acc_buf ^= 1;
        for (int ks = 0; ks < p.num_k_stages; ++ks) {
          ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, 3);
          ok = __all_sync(0xFFFFFFFFu, ok);
          if (!ok) break;
          tc_fence_after();
          const uint32_t tmem_sfa = tmem_base + Cfg::kTmemSfa + sf_buf * Cfg::kTmemSfSet;
          const uint32_t tmem_sfb = tmem_base + Cfg::kTmemSfb + sf_buf * Cfg::kTmemSfSet;
          sf_buf ^= 1;
          const uint32_t sfa_lo = ((smem_sfa + stage * PC::kSfaStageBytes) & 0x3FFFFu) >> 4;
          const uint32_t sfb_lo = ((smem_sfb + stage * PC::kSfbStageBytes) & 0x3FFFFu) >> 4;
          const uint32_t a_lo = (((smem_a + stage * kAStageBytes) & 0x3FFFFu) >> 4) | (1u << 16);
          const uint32_t b_lo = (((smem_b + stage * PC::kBHalfBytes) & 0x3FFFFu) >> 4) | (1u << 16);
          const int sf_left = p.sf_col_tiles - ks * kST;
          const int k_left = p.k_bytes - ks * kStageKBytes;
          const int sf_tiles = sf_left > kST ? kST : sf_left;
          const int n_mma = k_left >= kStageKBytes ? 4 : (k_left + 31) >> 5;
          if (elected) {
#pragma unroll
            for (int t = 0; t < kST; ++t) {
              if (t < sf_tiles) {
                tc_cp_sf_pair(tmem_sfa + t * 4, make_desc(sfa_lo + t * 32, kDescHiSf));
#pragma unroll
                for (int nb = 0; nb < kNB; ++nb) tc_cp_sf_pair(tmem_sfb + (t * kNB + nb) * 4, make_desc(sfb_lo + (nb * kST + t) * 32, kDescHiSf));
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (j < n_mma) {
                const int t = (FMT == TF_FMT_MXFP8) ? 0 : (FMT == TF_FMT_MXFP4) ? (j >> 1) : j;
                const uint32_t sf_id = (FMT == TF_FMT_MXFP8) ? (uint32_t)j : (FMT == TF_FMT_MXFP4) ? (uint32_t)((j & 1) * 2) : 0u;
                tc_mma_pair<FMT>(tmem_acc, make_desc(a_lo + j * 2, kDescHiSw128), make_desc(b_lo + j * 2, kDescHiSw128),
                                 idesc_base | (sf_id << 4) | (sf_id << 29), tmem_sfa + t * 4, tmem_sfb + t * kNB * 4, (j > 0 || ks > 0) ? 1u : 0u);
              }
            }
            tc_commit_pair(bar_empty + 8 * stage);  // frees the stage in both CTAs
          }
          __syncwarp();
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (elected) tc_commit_pair(bar_tmem_full);  // both CTAs' epilogues may read their accumulator halves
        __syncwarp();
        tile_phase ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue: each CTA drains its own 128 rows; the release goes to the leader's barrier ----------------
    const int q = warp & 3;
    const float alpha = (FMT == TF_FMT_NVFP4) ? __fmul_rn(__ldg(p.a_gs), __ldg(p.b_gs)) : 1.0f;
    const uint32_t release = mapa_shared(bar_tmem_empty, 0);
    uint32_t tile_phase = 0, acc_buf = 0;
    uint32_t amax2 = 0;
    for (int tile = pair; tile < p.num_tiles; tile += num_pairs) {
      const int m_blk = tile % p.m_blocks, n_blk = tile / p.m_blocks;
      bool ok = mbar_wait(bar_tmem_full, tile_phase, abort_flag, 4);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m_blk * 256 + (int)rank * 128 + q * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
      const int col0 = n_blk * kOutCols;
      const float alpha_t = (FMT == TF_FMT_NVFP4 && p.a_gs_rows > 0) ? __fmul_rn(__ldg(p.a_gs + min(row, p.m - 1) / p.a_gs_rows), __ldg(p.b_gs)) : alpha;
      if (acc_buf == 0)
        epilogue_tile<FMT, BLOCK_N, EPI, 0, -1, true>(p, t_row, release, lane, row, col0, alpha_t, amax2);
      else
        epilogue_tile<FMT, BLOCK_N, EPI, 1, -1, true>(p, t_row + Cfg::kAccStride, release, lane, row, col0, alpha_t, amax2);
      acc_buf ^= 1;
      tile_phase ^= 1;
    }
    if (p.out_amax) {
      uint32_t mx = max(amax2 & 0xFFFFu, amax2 >> 16);
      for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
      if (lane == 0 && mx) atomicMax(p.out_amax, mx << 16);
    }
  }

  // ---------------- teardown: nobody leaves while the peer may still touch this CTA's shared or tensor memory ----------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// A [rows, k_bytes] byte matrix, boxes of 128 rows x 128 bytes, 128-byte swizzle, out-of-range bytes read as zero.
static tf_status make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k_bytes, int box_rows = 128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(TF_ERR_CUDA, "tf_gemm_blockscaled: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {(cuuint64_t)k_bytes, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)k_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)kStageKBytes, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TF_ERR_CUDA, "tf_gemm_blockscaled: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TF_OK;
}

// SMs the persistent GEMM leaves free (for a collective running beside it in another stream).
static std::atomic<int> g_sm_margin{0};  // process-wide (tf_set_sm_margin); atomic so that a concurrent reader sees the old or the new value
static int gemm_sms() {
  const int n = sm_count() - g_sm_margin.load(std::memory_order_relaxed);
  return n < 2 ? 2 : n;
}

// Split-K plan of a problem: how many K ranges each output tile is cut into, so that small-M problems (few tiles, long K: the
// weight-streaming regime) still occupy every SM. Depends only on the sizes and the SM count: the workspace query and the launch
// agree by construction.
struct SplitPlan {
  int block_n, splits, k_stages_per_split;
};

// Small M (at most two row blocks): the GEMM streams the weights once and is bound by how evenly that stream is spread over
// the SMs. Measured on B200: one CTA's TMA pipeline draws about one 128-byte row segment per 4 clocks from HBM (about
// 60 GB/s), so the time of a launch is the largest number of row segments any CTA fetches. The plan minimises
//   waves * (K stages per unit + 3 stages of fill and drain) * (rows of B + rows of A per stage)  +  cost of the reduction pass
// over tile width {256, 128} and 1..16 K ranges, in units of one row segment (about 2.4 ns).
static SplitPlan split_plan(int64_t m, int64_t n, int64_t k_bytes, int epilogue) {
  SplitPlan sp;
  const int sms = sm_count();
  const int64_t m_blocks = (m + kBlockM - 1) / kBlockM;
  const int64_t n_acc = epilogue == TF_EPI_SILU_GATE ? 2 * n : n;
  const int64_t stages = (k_bytes + kStageKBytes - 1) / kStageKBytes;
  sp.block_n = 256;
  sp.splits = 1;
  sp.k_stages_per_split = (int)stages;
  if (n <= 128 && epilogue != TF_EPI_SILU_GATE) sp.block_n = 128;
  if (m > 256) return sp;
  const int64_t a_rows = m < kBlockM ? m : kBlockM;
  double best = 1e30;
  for (int bn = 256; bn >= 128; bn -= 128) {
    const int64_t tiles = m_blocks * ((n_acc + bn - 1) / bn);
    for (int64_t want = 1; want <= 16; ++want) {
      if (want > 1 && stages / want < 4) break;  // a K range shorter than the pipeline is all fill and drain
      const int64_t kps = (stages + want - 1) / want;
      const int64_t splits = (stages + kps - 1) / kps;
      if (bn == 128 && splits == 1 && epilogue == TF_EPI_SILU_GATE) continue;  // the fused SiLU gate pairs two 128-column halves
      const int64_t units = tiles * splits;
      const int64_t waves = (units + sms - 1) / sms;
      double cost = (double)waves * (double)(kps + 3) * (double)(bn + a_rows);
      if (splits > 1) cost += 1200.0 + 2.0 * (double)splits * (double)m * (double)n_acc * 4.0 / 7200.0;
      if (cost < best) {
        best = cost;
        sp.block_n = bn;
        sp.splits = (int)splits;
        sp.k_stages_per_split = (int)kps;
      }
    }
  }
  return sp;
}

template <int FMT, int BLOCK_N, int EPI, bool SPLITK>
static tf_status launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, cudaStream_t stream) {
  using Cfg = TileCfg<FMT, BLOCK_N>;
  auto kernel = gemm_blockscaled_kernel<FMT, BLOCK_N, EPI, SPLITK>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  TF_CUDA(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    TF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured_dev = dev;
  }
  constexpr int out_cols = (EPI == TF_EPI_SILU_GATE) ? BLOCK_N / 2 : BLOCK_N;
  p.n_blocks = (p.n + out_cols - 1) / out_cols;
  p.num_tiles = p.m_blocks * p.n_blocks * p.splits;
  const int grid = p.num_tiles < gemm_sms() ? p.num_tiles : gemm_sms();
  TF_CUDA(launch_dependent(kernel, dim3(grid), dim3(kGemmThreads), (size_t)Cfg::kSmemBytes, stream, ta, tb, p));
  return TF_OK;
}

// The swizzled scale buffer as a [tiles, 128 x u32] matrix: a box is kST consecutive 512-byte tiles, no swizzle.
static tf_status make_scale_map(CUtensorMap* map, const void* base, int64_t tiles, int box_tiles) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(TF_ERR_CUDA, "tf_gemm_blockscaled: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {128u, (cuuint64_t)tiles};
  const cuuint64_t strides[1] = {512u};
  const cuuint32_t box[2] = {128u, (cuuint32_t)box_tiles};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TF_ERR_CUDA, "tf_gemm_blockscaled: cuTensorMapEncodeTiled (scales) failed with CUresult %d", (int)r);
  return TF_OK;
}

template <int FMT, int EPI>
static tf_status launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, cudaStream_t stream) {
  using PC = PairCfg<FMT, EPI>;
  CUtensorMap tsa, tsb;
  tf_status st = make_scale_map(&tsa, p.sfa, (int64_t)((p.m + 127) / 128) * p.sf_col_tiles, PC::kST);
  if (st != TF_OK) return st;
  st = make_scale_map(&tsb, p.sfb, (int64_t)p.sfb_row_tiles * p.sf_col_tiles, PC::kST);
  if (st != TF_OK) return st;
  auto kernel = gemm_blockscaled_pair_kernel<FMT, EPI>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  TF_CUDA(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    TF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PC::kSmemBytes));
    configured_dev = dev;
  }
  constexpr int out_cols = (EPI == TF_EPI_SILU_GATE) ? 128 : 256;
  p.m_blocks = (p.m + 255) / 256;
  p.n_blocks = (p.n + out_cols - 1) / out_cols;
  p.num_tiles = p.m_blocks * p.n_blocks;
  int pairs = gemm_sms() / 2;
  if (p.num_tiles < pairs) pairs = p.num_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = PC::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TF_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, tsa, tsb, p));
  return TF_OK;
}

// Whether the 2-CTA kernel serves this problem: asked for (TF_GEMM_TWO_CTA=1 in the environment; the one-CTA kernel measured
// faster on B200 under its power cap and is the default), more than one 128-row block, a full pair tile wide, no split-K.
static bool use_pair_kernel(const GemmParams& p, const SplitPlan& sp) {
  static const int enabled = getenv("TF_GEMM_TWO_CTA") ? atoi(getenv("TF_GEMM_TWO_CTA")) : 0;
  return enabled && sp.splits == 1 && p.m > 128 && p.n_rows_b >= 256;
}

template <int FMT>
static tf_status dispatch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, int epilogue, const SplitPlan& sp, cudaStream_t stream,
                               bool partials_only = false) {
  if (sp.splits > 1) {
    // first pass: plain accumulation over all accumulator columns into the workspace; second pass: reduce + epilogue
    const int n_out = p.n;
    float* residual = p.residual;
    unsigned int* amax = p.out_amax;
    p.n = p.n_rows_b;
    p.out_amax = nullptr;
    uint8_t* qc = p.q_codes;
    p.q_codes = nullptr;  // the quantized copy is produced by the second pass
    tf_status st = sp.block_n == 128 ? launch_gemm<FMT, 128, TF_EPI_NONE, true>(ta, tb, p, stream) : launch_gemm<FMT, 256, TF_EPI_NONE, true>(ta, tb, p, stream);
    if (st != TF_OK) return st;
    if (partials_only) return TF_OK;  // the caller's next kernel sums the planes (tf_gemm_blockscaled_partials)
    p.q_codes = qc;
    const int64_t total = (int64_t)p.m * (n_out >> 3);
    const int64_t need = (total + 255) / 256, cap = (int64_t)sm_count() * 8;
    const unsigned grid = (unsigned)(need < cap ? need : cap);
    const float* ags = FMT == TF_FMT_NVFP4 ? p.a_gs : nullptr;
    const float* bgs = FMT == TF_FMT_NVFP4 ? p.b_gs : nullptr;
#define TF_REDUCE(EPI_, Q_) \
  launch_dependent(splitk_reduce_kernel<EPI_, Q_>, dim3(grid), dim3(256), 0, stream, (const float*)p.ws, (int)sp.splits, (int)p.m, (int)n_out, (int)p.n_rows_b, ags, bgs, \
                   p.out, p.ldo, residual, amax, p.q_codes, p.q_scales, (int)p.a_gs_rows)
    const int qf = p.q_codes ? FMT : -1;
    if (epilogue == TF_EPI_SILU_GATE) {
      if (qf == TF_FMT_MXFP8) TF_REDUCE(TF_EPI_SILU_GATE, TF_FMT_MXFP8);
      else if (qf == TF_FMT_MXFP4) TF_REDUCE(TF_EPI_SILU_GATE, TF_FMT_MXFP4);
      else TF_REDUCE(TF_EPI_SILU_GATE, -1);
    } else if (epilogue == TF_EPI_RESIDUAL) {
      TF_REDUCE(TF_EPI_RESIDUAL, -1);
    } else {
      if (qf == TF_FMT_MXFP8) TF_REDUCE(TF_EPI_NONE, TF_FMT_MXFP8);
      else if (qf == TF_FMT_MXFP4) TF_REDUCE(TF_EPI_NONE, TF_FMT_MXFP4);
      else TF_REDUCE(TF_EPI_NONE, -1);
    }
#undef TF_REDUCE
    TF_LAUNCH_CHECK();
    return TF_OK;
  }
  if (use_pair_kernel(p, sp)) {
    if (epilogue == TF_EPI_SILU_GATE) return launch_gemm_pair<FMT, TF_EPI_SILU_GATE>(ta, tb, p, stream);
    if (epilogue == TF_EPI_RESIDUAL) return launch_gemm_pair<FMT, TF_EPI_RESIDUAL>(ta, tb, p, stream);
    return launch_gemm_pair<FMT, TF_EPI_NONE>(ta, tb, p, stream);
  }
  if (epilogue == TF_EPI_SILU_GATE) return launch_gemm<FMT, 256, TF_EPI_SILU_GATE, false>(ta, tb, p, stream);
  if (epilogue == TF_EPI_RESIDUAL)
    return sp.block_n == 256 ? launch_gemm<FMT, 256, TF_EPI_RESIDUAL, false>(ta, tb, p, stream) : launch_gemm<FMT, 128, TF_EPI_RESIDUAL, false>(ta, tb, p, stream);
  return sp.block_n == 256 ? launch_gemm<FMT, 256, TF_EPI_NONE, false>(ta, tb, p, stream) : launch_gemm<FMT, 128, TF_EPI_NONE, false>(ta, tb, p, stream);
}

// Scratch of tf_gemm_blockscaled_static: lives in the library's device image, one copy per GPU that loads the library,
// from load to process exit. Host code may not use this name as a pointer: it is a host-side stand-in for the symbol.
constexpr int64_t kStaticScratchBytes = 8ll << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int* device_status_words() {
  constexpr int kMaxDevices = 64;
  static int* cached[kMaxDevices] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (!cached[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_device_status) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<int*>(ptr);
  }
  return cached[dev];
}

}  // namespace tf

using namespace tf;

extern "C" {

tf_status tf_device_status(int32_t* status, int32_t* detail) {
  clear_error();
  TF_CHECK_ARG(status != nullptr, "%s: null pointer", __func__);
  int host[2] = {0, 0};
  TF_CUDA(cudaDeviceSynchronize());
  TF_CUDA(cudaMemcpyFromSymbol(host, g_device_status, sizeof(host)));
  if (host[0] != 0) {
    const int zero[2] = {0, 0};
    TF_CUDA(cudaMemcpyToSymbol(g_device_status, zero, sizeof(zero)));
  }
  *status = host[0];
  if (detail) *detail = host[1];
  return TF_OK;
}

tf_status tf_set_sm_margin(int32_t sms) {
  clear_error();
  TF_CHECK_ARG(sms >= 0 && sms <= 64, "%s: the margin must be in 0..64", __func__);
  g_sm_margin.store(sms, std::memory_order_relaxed);
  return TF_OK;
}

tf_status tf_selftest_bounded_wait(int32_t limit_ms, void* stream) {
  clear_error();
  TF_CHECK_ARG(limit_ms > 0 && limit_ms <= 2000, "%s: limit_ms must be in 1..2000", __func__);
  bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned long long)limit_ms * 1000000ull);
  TF_LAUNCH_CHECK();
  return TF_OK;
}

int64_t tf_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int32_t format, int32_t epilogue) {
  if (m <= 0 || n <= 0 || k <= 0 || format < TF_FMT_MXFP8 || format > TF_FMT_NVFP4 || epilogue < TF_EPI_NONE || epilogue > TF_EPI_RESIDUAL) return 0;
  const int64_t k_bytes = format == TF_FMT_MXFP8 ? k : k / 2;
  const SplitPlan sp = split_plan(m, n, k_bytes, epilogue);
  if (sp.splits <= 1) return 0;
  const int64_t n_acc = epilogue == TF_EPI_SILU_GATE ? 2 * n : n;
  return (int64_t)sp.splits * m * n_acc * 4;
}

static tf_status static_scratch_address(void** out) {
  // The device address of g_static_scratch, looked up once per device (with that device current) and cached.
  constexpr int kMaxDevices = 64;
  static void* cached[kMaxDevices] = {nullptr};
  int dev = 0;
  TF_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(TF_ERR_UNSUPPORTED, "tf_gemm_blockscaled_static: device ordinal %d is beyond %d", dev, kMaxDevices);
  if (!cached[dev]) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(TF_ERR_CUDA, "tf_gemm_blockscaled_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return TF_OK;
}

int32_t tf_gemm_splits(int64_t m, int64_t n, int64_t k, int32_t format, int32_t epilogue) {
  if (m <= 0 || n <= 0 || k <= 0 || format < TF_FMT_MXFP8 || format > TF_FMT_NVFP4 || epilogue < TF_EPI_NONE || epilogue > TF_EPI_RESIDUAL) return 0;
  return split_plan(m, n, format == TF_FMT_MXFP8 ? k : k / 2, epilogue).splits;
}

int64_t tf_gemm_static_scratch_bytes(void) { return kStaticScratchBytes; }

tf_status tf_gemm_blockscaled_static(const void* a_codes, const void* a_scales, const float* a_global_scale, const void* b_codes,
                                     const void* b_scales, const float* b_global_scale, void* out, int64_t ldo, int64_t m, int64_t n, int64_t k,
                                     int32_t format, int32_t epilogue, void* epilogue_arg, float* out_amax, void* stream) {
  clear_error();
  const int64_t need = tf_gemm_workspace_bytes(m, n, k, format, epilogue);
  if (need > kStaticScratchBytes)
    return fail(TF_ERR_WORKSPACE,
                "tf_gemm_blockscaled_static: this problem needs %lld bytes of scratch, the built-in scratch holds %lld; use tf_gemm_blockscaled "
                "with a caller-provided workspace",
                (long long)need, (long long)kStaticScratchBytes);
  void* scratch = nullptr;
  if (need > 0) {
    const tf_status st = static_scratch_address(&scratch);
    if (st != TF_OK) return st;
  }
  return tf_gemm_blockscaled(a_codes, a_scales, a_global_scale, b_codes, b_scales, b_global_scale, out, ldo, m, n, k, format, epilogue, epilogue_arg,
                             out_amax, nullptr, nullptr, 0, scratch, need > 0 ? kStaticScratchBytes : 0, stream);
}

}  // extern "C"

// The GEMM entry points. `scatter_ptrs` (null for tf_gemm_blockscaled): the destinations of the row blocks, see GemmParams.
// `partial_splits` (non-null for tf_gemm_blockscaled_partials): only the first pass of a split-K problem runs; receives the number of planes.
static tf_status gemm_entry(const char* fn, const void* a_codes, const void* a_scales, const float* a_global_scale, const void* b_codes,
                            const void* b_scales, const float* b_global_scale, void* out, int64_t ldo, int64_t m, int64_t n, int64_t k, int32_t format,
                            int32_t epilogue, void* epilogue_arg, float* out_amax, void* q_codes, void* q_scales, int64_t a_global_scale_rows,
                            void* workspace, int64_t workspace_bytes, const uint64_t* scatter_ptrs, int32_t owners, int64_t rows_per_owner,
                            void* stream_, int32_t* partial_splits = nullptr) {
  cudaStream_t stream = (cudaStream_t)stream_;
  TF_CHECK_ARG(format >= TF_FMT_MXFP8 && format <= TF_FMT_NVFP4, "%s: unknown format %d", fn, format);
  TF_CHECK_ARG(epilogue >= TF_EPI_NONE && epilogue <= TF_EPI_RESIDUAL, "%s: unknown epilogue %d", fn, epilogue);
  TF_CHECK_ARG(m >= 0 && n > 0 && k > 0, "%s: bad shape m=%lld n=%lld k=%lld", fn, (long long)m, (long long)n, (long long)k);
  if (m == 0) return TF_OK;
  TF_CHECK_ARG(a_codes && a_scales && b_codes && b_scales && (out || q_codes || partial_splits), "%s: null pointer", fn);
  TF_CHECK_ARG((q_codes == nullptr) == (q_scales == nullptr), "%s: q_codes and q_scales go together", fn);
  if (q_codes) {
    if (format == TF_FMT_NVFP4)
      return fail(TF_ERR_UNSUPPORTED, "%s: a quantized output needs the tensor's global scale first; nvfp4 outputs are quantized by tf_quantize_nvfp4_from_amax", fn);
    if (epilogue == TF_EPI_RESIDUAL) return fail(TF_ERR_UNSUPPORTED, "%s: the residual epilogue has no quantized output", fn);
    if (n % 32 != 0) return fail(TF_ERR_UNSUPPORTED, "%s: a quantized output needs n %% 32 == 0", fn);
    TF_CHECK_ALIGNED(q_codes, 16, "q_codes");
    const int64_t cols = n / 32;
    if ((m & 127) || (cols & 3)) TF_CUDA(cudaMemsetAsync(q_scales, 0, (size_t)tf_scale_bytes(format, m, n, TF_SCALES_SWIZZLED), stream));
  }
  TF_CHECK_ARG(epilogue != TF_EPI_RESIDUAL || out, "%s: the residual epilogue needs out", fn);
  TF_CHECK_ARG(a_global_scale_rows >= 0 && a_global_scale_rows % 128 == 0, "%s: a_global_scale_rows must be 0 or a multiple of 128", fn);
  TF_CHECK_ARG(format != TF_FMT_NVFP4 || (a_global_scale && b_global_scale), "%s: nvfp4 needs both global scales", fn);
  TF_CHECK_ARG(epilogue != TF_EPI_RESIDUAL || epilogue_arg, "%s: the residual epilogue needs its f32 residual", fn);
  if (k % 32 != 0) return fail(TF_ERR_UNSUPPORTED, "%s: k=%lld is not a multiple of 32", fn, (long long)k);
  if (n % 8 != 0 || ldo % 8 != 0 || ldo < n) return fail(TF_ERR_ALIGNMENT, "%s: n and ldo must be multiples of 8 with ldo >= n", fn);
  if (epilogue == TF_EPI_SILU_GATE && n % 128 != 0) return fail(TF_ERR_UNSUPPORTED, "%s: the SiLU-gate epilogue needs n %% 128 == 0", fn);
  if (m > (1 << 30) || n > (1 << 30) || k > (1 << 30)) return fail(TF_ERR_UNSUPPORTED, "%s: a dimension exceeds 2^30", fn);
  TF_CHECK_ALIGNED(a_codes, 16, "a_codes");
  TF_CHECK_ALIGNED(b_codes, 16, "b_codes");
  TF_CHECK_ALIGNED(a_scales, 16, "a_scales");
  TF_CHECK_ALIGNED(b_scales, 16, "b_scales");
  if (out) TF_CHECK_ALIGNED(out, 16, "out");
  if (epilogue == TF_EPI_RESIDUAL) TF_CHECK_ALIGNED(epilogue_arg, 16, "residual");

  const int64_t k_bytes = (format == TF_FMT_MXFP8) ? k : k / 2;
  const int64_t n_rows_b = (epilogue == TF_EPI_SILU_GATE) ? 2 * n : n;
  const int64_t block = (format == TF_FMT_NVFP4) ? 16 : 32;
  CUtensorMap ta, tb;
  // M < 128: the A box covers only the rows that exist (in steps of 16), so every stage asks TMA for fewer row segments (measured:
  // 10 % on the M = 1 decode step). The rows of the shared-memory tile beyond the box are never written; they feed accumulator
  // rows that are never stored.
  const int a_box_rows = m >= kBlockM ? kBlockM : (int)((m + 15) / 16 * 16);
  tf_status st = make_operand_map(&ta, a_codes, m, k_bytes, a_box_rows);
  if (st != TF_OK) return st;
  st = make_operand_map(&tb, b_codes, n_rows_b, k_bytes);
  if (st != TF_OK) return st;

  GemmParams p;
  p.m = (int)m;
  p.n = (int)n;
  p.n_rows_b = (int)n_rows_b;
  p.k_bytes = (int)k_bytes;
  p.num_k_stages = (int)((k_bytes + kStageKBytes - 1) / kStageKBytes);
  p.sf_col_tiles = (int)((k / block + 3) / 4);
  p.m_blocks = (int)((m + kBlockM - 1) / kBlockM);
  p.n_blocks = 0;
  p.num_tiles = 0;
  p.sfb_row_tiles = (int)((n_rows_b + 127) / 128);
  p.sfa = static_cast<const uint8_t*>(a_scales);
  p.sfb = static_cast<const uint8_t*>(b_scales);
  p.a_gs = a_global_scale;
  p.b_gs = b_global_scale;
  p.out = static_cast<uint16_t*>(out);
  p.ldo = ldo;
  p.residual = static_cast<float*>(epilogue_arg);
  p.out_amax = reinterpret_cast<unsigned int*>(out_amax);
  p.q_codes = static_cast<uint8_t*>(q_codes);
  p.q_scales = static_cast<uint8_t*>(q_scales);
  p.a_gs_rows = (int)a_global_scale_rows;
  p.a_box_bytes = a_box_rows * kStageKBytes;
  p.scatter_rows = 0;
  for (int i = 0; i < 8; ++i) p.scatter_out[i] = nullptr;
  const SplitPlan sp = split_plan(m, n, k_bytes, epilogue);
  if (scatter_ptrs) {
    if (sp.splits > 1)
      return fail(TF_ERR_UNSUPPORTED, "%s: this shape is split along K (tf_gemm_workspace_bytes > 0), which has no scattered output", fn);
    p.scatter_rows = (int)rows_per_owner;
    for (int i = 0; i < owners; ++i) p.scatter_out[i] = reinterpret_cast<uint16_t*>(scatter_ptrs[i]);
  }
  if (partial_splits) {
    if (sp.splits <= 1) return fail(TF_ERR_UNSUPPORTED, "%s: this shape is not split along K (tf_gemm_splits == 1): there are no partial sums to leave", fn);
    *partial_splits = sp.splits;
  }
  p.splits = sp.splits;
  p.k_stages_per_split = sp.k_stages_per_split;
  p.ws = static_cast<float*>(workspace);
  if (sp.splits > 1) {
    const int64_t need = (int64_t)sp.splits * m * n_rows_b * 4;
    if (!workspace || workspace_bytes < need)
      return fail(TF_ERR_WORKSPACE, "%s: this problem is split %d ways along K and needs a %lld-byte workspace (tf_gemm_workspace_bytes)", fn,
                  sp.splits, (long long)need);
    TF_CHECK_ALIGNED(workspace, 256, "workspace");
  }
  switch (format) {
    case TF_FMT_MXFP8: return dispatch_gemm<TF_FMT_MXFP8>(ta, tb, p, epilogue, sp, stream, partial_splits != nullptr);
    case TF_FMT_MXFP4: return dispatch_gemm<TF_FMT_MXFP4>(ta, tb, p, epilogue, sp, stream, partial_splits != nullptr);
    default: return dispatch_gemm<TF_FMT_NVFP4>(ta, tb, p, epilogue, sp, stream, partial_splits != nullptr);
  }
}

extern "C" {

tf_status tf_gemm_blockscaled(const void* a_codes, const void* a_scales, const float* a_global_scale, const void* b_codes, const void* b_scales,
                              const float* b_global_scale, void* out, int64_t ldo, int64_t m, int64_t n, int64_t k, int32_t format,
                              int32_t epilogue, void* epilogue_arg, float* out_amax, void* q_codes, void* q_scales,
                              int64_t a_global_scale_rows, void* workspace, int64_t workspace_bytes, void* stream) {
  clear_error();
  return gemm_entry(__func__, a_codes, a_scales, a_global_scale, b_codes, b_scales, b_global_scale, out, ldo, m, n, k, format, epilogue, epilogue_arg,
                    out_amax, q_codes, q_scales, a_global_scale_rows, workspace, workspace_bytes, nullptr, 0, 0, stream);
}

tf_status tf_gemm_blockscaled_partials(const void* a_codes, const void* a_scales, const float* a_global_scale, const void* b_codes, const void* b_scales,
                                       const float* b_global_scale, int64_t m, int64_t n, int64_t k, int32_t format, void* workspace,
                                       int64_t workspace_bytes, int32_t* splits, void* stream) {
  clear_error();
  TF_CHECK_ARG(splits != nullptr, "%s: null pointer", __func__);
  return gemm_entry(__func__, a_codes, a_scales, a_global_scale, b_codes, b_scales, b_global_scale, nullptr, n, m, n, k, format, TF_EPI_NONE, nullptr,
                    nullptr, nullptr, nullptr, 0, workspace, workspace_bytes, nullptr, 0, 0, stream, splits);
}

tf_status tf_gemm_blockscaled_scatter(const void* a_codes, const void* a_scales, const float* a_global_scale, const void* b_codes, const void* b_scales,
                                      const float* b_global_scale, const uint64_t* out_ptrs, int32_t owners, int64_t rows_per_owner, int64_t ldo,
                                      int64_t m, int64_t n, int64_t k, int32_t format, int64_t a_global_scale_rows, void* stream) {
  clear_error();
  TF_CHECK_ARG(out_ptrs != nullptr, "%s: null pointer", __func__);
  TF_CHECK_ARG(owners >= 1 && owners <= 8, "%s: owners must be in 1..8", __func__);
  TF_CHECK_ARG(rows_per_owner > 0 && rows_per_owner % 128 == 0 && rows_per_owner <= (1 << 24), "%s: rows_per_owner must be a positive multiple of 128",
               __func__);
  TF_CHECK_ARG(m == (int64_t)owners * rows_per_owner, "%s: m=%lld is not owners x rows_per_owner", __func__, (long long)m);
  for (int i = 0; i < owners; ++i)
    if (!out_ptrs[i] || out_ptrs[i] % 16) return fail(TF_ERR_ALIGNMENT, "%s: destination %d is null or not 16-byte aligned", __func__, i);
  return gemm_entry(__func__, a_codes, a_scales, a_global_scale, b_codes, b_scales, b_global_scale, reinterpret_cast<void*>(out_ptrs[0]), ldo, m, n, k,
                    format, TF_EPI_NONE, nullptr, nullptr, nullptr, nullptr, a_global_scale_rows, nullptr, 0, out_ptrs, owners, rows_per_owner, stream);
}

}  // extern "C"
