// In-place bf16 sum all-reduce over NVLink / NVSwitch for the tensor-parallel MLP: one kernel per rank, peers' buffers mapped
// into this GPU's address space (symmetric memory allocated and exchanged by the host side).
//
// Three data paths; rank r owns slice r of the range in all of them:
//   switch reduce   (multicast mapping, reduce_in_switch): for every 16-byte vector of its slice a rank issues
//               multimem.ld_reduce (NVSwitch returns the sum of all ranks' copies) and multimem.st (NVSwitch writes it into all
//               ranks' buffers). One pass, each GPU receives about `size` bytes. The switch's bf16 result is within one bf16
//               step of the exact sum but not always the nearest value (measured: about a fifth of the elements of a two-rank
//               sum differ from round-to-nearest).
//   peer reduce + multicast store   (multicast mapping): the rank sums its slice over plain peer loads (f32, rank order, rounded
//               to nearest even once) and multimem.st writes the result to all ranks. Each GPU receives about 2 x size bytes.
//   peer loads  (no multicast mapping): the same sum, stored into the rank's own buffer; after a barrier every rank copies
//               the other slices from their owners.
// No TMA anywhere in this file. The second kernel of the file, tp_norm_exchange_kernel, fuses the same sum with the next block's
// residual add, rmsnorm and quantization and gathers the quantized rows instead (its own comment is further down).
//
// Cross-GPU barriers are flags in peer memory: every rank stores a monotonically increasing value into its slot of every
// peer's flag array (st.release.sys) and spins on its own array (ld.acquire.sys). The value is derived from a call counter kept
// in this rank's device memory and advanced by the kernel itself, so a CUDA-graph replay (which repeats the same launch
// arguments) still produces fresh values. Every spin is bounded by %globaltimer (two seconds): on a timeout the kernel writes an
// error word into the state block and returns; nothing traps and nothing spins forever. The kernels of all ranks must be
// running at the same time for the barriers to complete: that holds because every rank is its own GPU.
#include "async_copy.cuh"
#include "quant_core.cuh"

namespace tf {

constexpr int kArMaxWorld = 8;
constexpr int kArThreads = 512;
constexpr unsigned long long kArWaitLimitNs = 2000000000ull;

// Layout of the per-rank state block (symmetric memory, zero-initialised by the host): 32-bit flag slots [0, 8), then
// 64-bit words at byte 64: call counter, local grid-barrier counter, its value at the start of the call, error word (0 = healthy,
// 1 = a local grid barrier gave up, 2 = a peer never arrived), wait limit in nanoseconds (0 = the two-second default; the host
// writes it, the kernels only read it). 128 bytes in all.
struct ArParams {
  unsigned long long bufs[kArMaxWorld];
  unsigned long long states[kArMaxWorld];
  unsigned long long mc_ptr;
  int rank, world, reduce_in_switch;
  long long offset_bytes;
  long long count;  // bf16 elements
};

__device__ __forceinline__ unsigned long long ar_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_acquire_gpu64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// All CTAs of this launch meet; `target` is the value the monotonic counter reaches when every CTA has arrived. Returns false
// (to every thread of the CTA) once any wait of this launch has given up; later waits then return at once.
__device__ __forceinline__ bool ar_grid_sync(unsigned long long* counter, unsigned long long target, volatile unsigned long long* error_word,
                                             unsigned long long limit_ns) {
  __shared__ int ok_s;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    atomicAdd(counter, 1ull);
    const unsigned long long t0 = ar_timer();
    // block 0 may itself be inside a cross-rank wait of up to limit_ns before it arrives here: allow twice that, so that a
    // missing peer is reported as such (2) and not as a local barrier that gave up (1)
    while (*error_word == 0 && ld_acquire_gpu64(counter) < target) {
      if (ar_timer() - t0 > 2 * limit_ns) *error_word = 1;
    }
    ok_s = *error_word == 0;
  }
  __syncthreads();
  return ok_s != 0;
}

// Block 0 tells every peer "this rank reached `value`" and waits until every peer told it the same.
__device__ __forceinline__ void ar_cross_barrier(const ArParams& p, unsigned int value, volatile unsigned long long* error_word,
                                                 unsigned long long limit_ns) {
  if (blockIdx.x == 0 && threadIdx.x < p.world) {
    __threadfence_system();
    unsigned int* peer_flags = reinterpret_cast<unsigned int*>(p.states[threadIdx.x]);
    st_release_sys(peer_flags + p.rank, value);
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(p.states[p.rank]) + threadIdx.x;
    const unsigned long long t0 = ar_timer();
    while (*error_word == 0 && (int)(ld_acquire_sys(mine) - value) < 0) {
      if (ar_timer() - t0 > limit_ns) *error_word = 2;
    }
  }
}

__device__ __forceinline__ void multimem_ld_reduce_bf16x8(unsigned long long addr, uint4& v) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(addr)
               : "memory");
}
__device__ __forceinline__ void multimem_st_16(unsigned long long addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ uint4 ld_peer_16(unsigned long long addr) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(addr) : "memory");
  return v;
}

__global__ void __launch_bounds__(kArThreads, 1) allreduce_bf16_kernel(const ArParams p) {
  unsigned long long* state64 = reinterpret_cast<unsigned long long*>(p.states[p.rank] + 64);
  unsigned long long* call_counter = state64;      // calls completed on this rank (the same on every rank of a healthy group)
  unsigned long long* grid_counter = state64 + 1;  // arrivals at local grid barriers, all calls
  unsigned long long* grid_base = state64 + 2;     // value of grid_counter when this call started
  volatile unsigned long long* error_word = state64 + 3;
  const unsigned long long limit_ns = state64[4] ? state64[4] : kArWaitLimitNs;
  // Both words are rewritten by block 0 only after the last grid barrier of a call, which every CTA reaches after these reads.
  const unsigned long long call = ld_acquire_gpu64(call_counter);
  const unsigned long long gbase = ld_acquire_gpu64(grid_base);
  const unsigned long long g = gridDim.x;
  const unsigned int flag = (unsigned int)(call * 4ull);
  const long long per_rank = (p.count >> 3) / p.world;  // 16-byte vectors in each rank's slice
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (long long)gridDim.x * blockDim.x;
  const unsigned long long my_buf = p.bufs[p.rank] + p.offset_bytes;
  const bool multicast = p.mc_ptr != 0;
  unsigned long long syncs = 0;

  // every rank's input is complete: its producer kernel finished before this kernel started on its stream
  ar_cross_barrier(p, flag + 1, error_word, limit_ns);
  bool ok = ar_grid_sync(grid_counter, gbase + (++syncs) * g, error_word, limit_ns);

  if (ok && multicast && p.reduce_in_switch) {
    const unsigned long long mc = p.mc_ptr + p.offset_bytes + (unsigned long long)(p.rank * per_rank) * 16ull;
    // four independent reductions in flight per thread
    long long i = tid;
    for (; i + 3 * nthreads < per_rank; i += 4 * nthreads) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) multimem_ld_reduce_bf16x8(mc + (unsigned long long)(i + u * nthreads) * 16ull, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u) multimem_st_16(mc + (unsigned long long)(i + u * nthreads) * 16ull, v[u]);
    }
    for (; i < per_rank; i += nthreads) {
      uint4 v;
      multimem_ld_reduce_bf16x8(mc + (unsigned long long)i * 16ull, v);
      multimem_st_16(mc + (unsigned long long)i * 16ull, v);
    }
  } else if (ok) {
    // this rank's slice, summed in f32 over every rank's copy in rank order (plain peer loads, all of a vector's copies and
    // two vectors in flight per thread), rounded once; written to every rank through the switch, or to this rank's buffer
    const unsigned long long slice = (unsigned long long)(p.rank * per_rank) * 16ull + p.offset_bytes;
    const unsigned long long dst = multicast ? p.mc_ptr + slice : p.bufs[p.rank] + slice;
    constexpr int kVec = 2;
    for (long long i0 = tid; i0 < per_rank; i0 += kVec * nthreads) {
      uint4 v[kVec][kArMaxWorld];
#pragma unroll
      for (int u = 0; u < kVec; ++u) {
        const long long i = i0 + u * nthreads;
#pragma unroll
        for (int r = 0; r < kArMaxWorld; ++r)
          if (r < p.world && i < per_rank) v[u][r] = ld_peer_16(p.bufs[r] + slice + (unsigned long long)i * 16ull);
      }
#pragma unroll
      for (int u = 0; u < kVec; ++u) {
        const long long i = i0 + u * nthreads;
        if (i >= per_rank) break;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll
        for (int r = 0; r < kArMaxWorld; ++r) {
          if (r < p.world) {
            const uint4 w = v[u][r];
            acc[0] += bf16lo_to_f32(w.x); acc[1] += bf16hi_to_f32(w.x); acc[2] += bf16lo_to_f32(w.y); acc[3] += bf16hi_to_f32(w.y);
            acc[4] += bf16lo_to_f32(w.z); acc[5] += bf16hi_to_f32(w.z); acc[6] += bf16lo_to_f32(w.w); acc[7] += bf16hi_to_f32(w.w);
          }
        }
        const uint4 o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
        if (multicast) multimem_st_16(dst + (unsigned long long)i * 16ull, o);
        else *reinterpret_cast<uint4*>(dst + (unsigned long long)i * 16ull) = o;
      }
    }
  }
  // all local CTAs wrote their part; then all ranks did: every slice is final everywhere (multicast) or at its owner
  ok = ar_grid_sync(grid_counter, gbase + (++syncs) * g, error_word, limit_ns);
  ar_cross_barrier(p, flag + 2, error_word, limit_ns);
  ok = ar_grid_sync(grid_counter, gbase + (++syncs) * g, error_word, limit_ns);

  if (!multicast) {
    if (ok) {
      // shot 2: fetch the other ranks' slices from their owners
      for (int d = 1; d < p.world; ++d) {
        const int r = (p.rank + d) % p.world;
        const unsigned long long src = p.bufs[r] + p.offset_bytes + (unsigned long long)(r * per_rank) * 16ull;
        const unsigned long long dst = my_buf + (unsigned long long)(r * per_rank) * 16ull;
        long long i = tid;
        for (; i + 3 * nthreads < per_rank; i += 4 * nthreads) {
          uint4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u] = ld_peer_16(src + (unsigned long long)(i + u * nthreads) * 16ull);
#pragma unroll
          for (int u = 0; u < 4; ++u) *reinterpret_cast<uint4*>(dst + (unsigned long long)(i + u * nthreads) * 16ull) = v[u];
        }
        for (; i < per_rank; i += nthreads) *reinterpret_cast<uint4*>(dst + (unsigned long long)i * 16ull) = ld_peer_16(src + (unsigned long long)i * 16ull);
      }
    }
    // no rank may overwrite its buffer (its next producer kernel) while a peer still reads it: once all local CTAs are done
    // reading, tell the peers and wait for theirs. The multicast path reads nothing after the second barrier.
    ar_grid_sync(grid_counter, gbase + (++syncs) * g, error_word, limit_ns);
    ar_cross_barrier(p, flag + 3, error_word, limit_ns);
  }
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *grid_base = gbase + syncs * g;
    __threadfence();
    *call_counter = call + 1ull;
  }
}

// ---- the tensor-parallel exchange fused with the next block's normalisation -------------------------------------------------
// One kernel per rank replaces, between two blocks of the MLP stack, the all-reduce of the second GEMM's partial results, the
// residual_add_rmsnorm of the next block and the quantization of its output: with the normalisation sharded by rows, rank r
//   1. sums ITS rows of the partial results over the ranks (peer loads in rank order, f32, rounded to bf16 once: the value a
//      bf16 all-reduce would have delivered; or the switch's multimem.ld_reduce), adds them into its rows of the f32 residual
//      stream and normalises them (the arithmetic and thread mapping of residual_add_rmsnorm_kernel: the same bytes),
//   2. derives the nvfp4 global scale of its row block from the block's amax (a grid-wide barrier inside the kernel),
//   3. quantizes its rows and writes codes, swizzled scales and the global scale into EVERY rank's buffers (multimem.st through
//      the switch, or one store per peer), so that every rank holds the quantized activation of all rows for its first GEMM.
// Per GPU and block the bytes received drop from 2 x (all-reduce of bf16 [M, H]) to (1/n of it, or (n-1)/n with peer loads)
// + 0.28 x: the activation crosses the links in 4.5 bits per element instead of 16, and the normalisation work is divided by n.
struct NxParams {
  ArParams ar;  // bufs = every rank's symmetric buffer; offset_bytes / count unused
  long long partial_off, codes_off, scales_off, gs_off;  // byte offsets inside the symmetric buffer (this row chunk's regions)
  int rows_total, d;  // rows of the chunk over all ranks (a multiple of 128 x world), row length
  int sum_peers;      // 0: the partial region already holds complete values on every rank (the stack's input); 1: pull this rank's rows
                      // from every rank's buffer; 2: every rank's partials for this rank's rows lie in this rank's buffer, one slot each
  float* residual;    // this rank's rows of the residual stream, f32 [rows_total / world, d], updated in place
  const uint4* w;     // bf16 [d]
  uint4* h_scratch;   // bf16 [rows_total / world, d]: the normalised rows between the two passes
  unsigned int* amax; // one word, zeroed by the caller
  float eps, inv_d;
};

template <int BYTES>
__device__ __forceinline__ void store_all_ranks(const ArParams& p, long long off, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  if (p.mc_ptr) {
    const unsigned long long addr = p.mc_ptr + off;
    if (BYTES == 16) asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
    else if (BYTES == 8) asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(addr), "r"(a), "r"(b) : "memory");
    else asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(addr), "r"(a) : "memory");
  } else {
    for (int r = 0; r < p.world; ++r) {
      const unsigned long long addr = p.bufs[r] + off;
      if (BYTES == 16) *reinterpret_cast<uint4*>(addr) = make_uint4(a, b, c, d);
      else if (BYTES == 8) *reinterpret_cast<uint2*>(addr) = make_uint2(a, b);
      else *reinterpret_cast<uint32_t*>(addr) = a;
    }
  }
}

// One 16-element piece of a normalised row (all 32 lanes of a warp together: the quantizer and the scale packing shuffle): quantizes it and
// writes codes and, from the first lane of each group, the four scale bytes of four consecutive blocks into every rank's buffers.
template <int QFMT>
__device__ __forceinline__ void quantize_store_piece(const ArParams& p, const NxParams& q, const uint32_t (&w8)[8], bool has, long long grow, int v, float gs,
                                                     float inv_t) {
  constexpr int kBlk = (QFMT == TF_FMT_NVFP4) ? 16 : 32;
  constexpr int kLanesPerWord = (QFMT == TF_FMT_NVFP4) ? 4 : 8;  // lanes (16 elements each) whose blocks share one 4-byte scale word
  const int lane = threadIdx.x & 31;
  const int n_ct = ((q.d / kBlk) + 3) >> 2;
  uint32_t codes[4], sc;
  quantize_vec16<QFMT>(w8, gs, inv_t, codes, sc);
  // four consecutive blocks' scale bytes are four consecutive bytes of the swizzled layout: gather them into the first lane
  uint32_t word = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int src = (lane & ~(kLanesPerWord - 1)) + k * (kLanesPerWord / 4);
    word |= (__shfl_sync(0xFFFFFFFFu, sc, src) & 0xFFu) << (8 * k);
  }
  if (!has) return;
  if (QFMT == TF_FMT_MXFP8) store_all_ranks<16>(p, q.codes_off + grow * q.d + (long long)v * 16, codes[0], codes[1], codes[2], codes[3]);
  else store_all_ranks<8>(p, q.codes_off + grow * (q.d >> 1) + (long long)v * 8, codes[0], codes[1], 0, 0);
  if ((lane & (kLanesPerWord - 1)) == 0) {
    const long long c = (QFMT == TF_FMT_NVFP4) ? v : (v >> 1);  // first of the word's four scale columns
    store_all_ranks<4>(p, q.scales_off + swizzled_scale_offset(grow, c, n_ct), word, 0, 0, 0);
  }
}

// Shared-memory ring of tp_norm_exchange_kernel. One extra warp feeds it with bulk copies (cp.async.bulk, no multicast; the source may
// be a peer's memory), the other warps consume it, so the loads of the next rows are in flight while the current row is reduced,
// normalised and stored. A segment is 256 vectors of a row: in pass 1 that is 4 KB of every bf16 source plus 8 KB of the f32
// residual, in pass 2 8 KB of normalised bf16 (256 pieces of 16 elements). Every consumer warp passes every segment in order (waits
// for it, reads its own part if it has one, arrives on the stage's "empty" barrier), so both roles count segments alike.
constexpr int kNxSegVecs = 256;
constexpr int kNxSrcBytes = kNxSegVecs * 16;
constexpr int kNxMaxStages = 8;
constexpr int kNxSmemBudget = 220 * 1024;

__device__ __forceinline__ uint4 lds_128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 lds_128f(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
// Orders this thread's earlier generic-proxy accesses before later accesses of the async proxy (bulk copies) to the same memory.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void consumer_barrier(int nthreads) { asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory"); }

struct NxRing {
  uint32_t base, full, empty;  // shared-memory addresses: stage buffers, then one "full" and one "empty" mbarrier per stage
  int stages, stage_bytes;  // stages is a power of two (log2 in stage_shift)
  int stage_shift;
  volatile int* abort_flag;
  int* status;  // the state block's error word as two 32-bit words: a wait that runs out stores TF_ERR_DEVICE_TIMEOUT and where
  unsigned long long limit_ns;
  __device__ __forceinline__ uint32_t buf(uint32_t g) const { return base + (g & (uint32_t)(stages - 1)) * (uint32_t)stage_bytes; }
  __device__ __forceinline__ uint32_t full_bar(uint32_t g) const { return full + 8u * (g & (uint32_t)(stages - 1)); }
  __device__ __forceinline__ uint32_t empty_bar(uint32_t g) const { return empty + 8u * (g & (uint32_t)(stages - 1)); }
  __device__ __forceinline__ uint32_t parity(uint32_t g) const { return (g >> stage_shift) & 1u; }
  // consumer: segment g has landed
  __device__ __forceinline__ bool wait_full(uint32_t g) const { return mbar_wait_bounded(full_bar(g), parity(g), abort_flag, status, 21, limit_ns); }
  // consumer warp: done with segment g (all lanes have taken their bytes)
  __device__ __forceinline__ void release(uint32_t g) const {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(empty_bar(g));
  }
  // producer warp: the stage of segment g is free again (the whole warp learns the outcome)
  __device__ __forceinline__ bool wait_empty(uint32_t g) const {
    int alive = 1;
    if ((threadIdx.x & 31) == 0 && g >= (uint32_t)stages) alive = mbar_wait_bounded(empty_bar(g), parity(g) ^ 1u, abort_flag, status, 22, limit_ns);
    return __shfl_sync(0xFFFFFFFFu, alive, 0) != 0;
  }
};

template <int VPT, int QFMT, bool SW>  // SW: the partial results are summed by the switch (multimem.ld_reduce), not from the ring
__global__ void __launch_bounds__(544, 1) tp_norm_exchange_kernel(const NxParams q, int stages, int stage_bytes) {
  extern __shared__ __align__(128) uint8_t nx_smem[];
  __shared__ int abort_flag;
  const ArParams& p = q.ar;
  unsigned long long* state64 = reinterpret_cast<unsigned long long*>(p.states[p.rank] + 64);
  unsigned long long* call_counter = state64;
  unsigned long long* grid_counter = state64 + 1;
  unsigned long long* grid_base = state64 + 2;
  volatile unsigned long long* error_word = state64 + 3;
  const unsigned long long limit_ns = state64[4] ? state64[4] : kArWaitLimitNs;
  const unsigned long long call = ld_acquire_gpu64(call_counter);
  const unsigned long long gbase = ld_acquire_gpu64(grid_base);
  const unsigned long long g = gridDim.x;
  const unsigned int flag = (unsigned int)(call * 4ull);
  unsigned long long syncs = 0;
  constexpr int kRows = VPT <= 2 ? 2 : 1;  // rows per round of pass 1 (registers: 8 f32 per vector per row)
  __shared__ float warp_sums[kRows][16];
  __shared__ unsigned int warp_amax[16];
  __shared__ float row_rstd[kRows];
  const int tid = threadIdx.x, lane = tid & 31;
  const int nthreads = blockDim.x - 32;  // consumer threads (the thread mapping of residual_add_rmsnorm_kernel); the last warp feeds the ring
  const bool producer = tid >= nthreads;
  const int nvec = q.d >> 3;
  const int rows_local = q.rows_total / p.world;
  const int row0 = p.rank * rows_local;
  // bf16 sources of a row's sum that come through the ring (the switch reduction reads global memory itself)
  const int n_src = !q.sum_peers ? 1 : (p.reduce_in_switch ? 0 : p.world);

  NxRing ring;
  ring.base = smem_u32(nx_smem);
  ring.full = ring.base + (uint32_t)stages * (uint32_t)stage_bytes;
  ring.empty = ring.full + 8u * (uint32_t)stages;
  ring.stages = stages;
  ring.stage_bytes = stage_bytes;
  ring.stage_shift = 31 - __clz(stages);
  ring.abort_flag = &abort_flag;
  ring.status = reinterpret_cast<int*>(state64 + 3);
  ring.limit_ns = limit_ns;
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(ring.full + 8 * s, 1);
      mbar_init(ring.empty + 8 * s, nthreads >> 5);
    }
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  // every rank's partial results are complete (and, when the producers delivered them, have landed in this rank's buffer)
  ar_cross_barrier(p, flag + 1, error_word, limit_ns);
  bool ok = ar_grid_sync(grid_counter, gbase + (++syncs) * g, error_word, limit_ns);

  uint32_t seg = 0;  // segments this CTA has been through; the producer warp and the consumer warps count alike
  // ---- pass 1: sum over the ranks, residual add, normalise (this rank's rows) ----
  uint32_t amax_bits = 0;
  const int nseg1 = (nvec + kNxSegVecs - 1) / kNxSegVecs;
  if (ok && producer) {
    fence_proxy_async();
    bool alive = true;
    for (int row = blockIdx.x; alive && row < rows_local; row += gridDim.x) {
      for (int s = 0; s < nseg1; ++s, ++seg) {
        alive = ring.wait_empty(seg);
        if (!alive) break;
        const int v0 = s * kNxSegVecs;
        const uint32_t nv = (uint32_t)min(kNxSegVecs, nvec - v0);
        if (lane == 0) mbar_expect_tx(ring.full_bar(seg), nv * (16u * (uint32_t)n_src + 32u));
        __syncwarp();
        if (lane < n_src) {
          unsigned long long src;
          if (q.sum_peers == 2) src = p.bufs[p.rank] + q.partial_off + (((long long)lane * rows_local + row) * nvec + v0) * 16;
          else src = p.bufs[q.sum_peers ? lane : p.rank] + q.partial_off + (((long long)row0 + row) * nvec + v0) * 16;
          bulk_load(ring.buf(seg) + (uint32_t)lane * kNxSrcBytes, reinterpret_cast<const void*>(src), nv * 16u, ring.full_bar(seg));
        } else if (lane == n_src) {
          bulk_load(ring.buf(seg) + (uint32_t)n_src * kNxSrcBytes, q.residual + ((long long)row * nvec + v0) * 8, nv * 32u, ring.full_bar(seg));
        }
      }
    }
  } else if (ok) {
    // kRows rows per round (in the producer's order: this CTA's rows, one after the other): their arithmetic interleaves and they
    // share the two block barriers; the sums of a row are still formed by the same threads in the same order
    for (int base = blockIdx.x; base < rows_local; base += gridDim.x * kRows) {
      float r[kRows][VPT][8];
      float acc[kRows];
      // the switch's sums of this round's vectors: all requested before the first is used (each takes a round trip through the switch)
      uint4 xs[SW ? kRows : 1][SW ? VPT : 1];
      if (SW && q.sum_peers) {
#pragma unroll
        for (int rw = 0; rw < kRows; ++rw) {
          const int row = base + rw * (int)gridDim.x;
#pragma unroll
          for (int i = 0; i < VPT; ++i) {
            const int v = tid + i * nthreads;
            xs[SW ? rw : 0][SW ? i : 0] = make_uint4(0, 0, 0, 0);
            if (row < rows_local && v < nvec)
              multimem_ld_reduce_bf16x8(p.mc_ptr + q.partial_off + (((long long)row0 + row) * nvec + v) * 16, xs[SW ? rw : 0][SW ? i : 0]);
          }
        }
      }
#pragma unroll
      for (int rw = 0; rw < kRows; ++rw) {
        const int row = base + rw * (int)gridDim.x;
        acc[rw] = 0.0f;
        if (row >= rows_local) {  // no such row: nothing was loaded for it
#pragma unroll
          for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) r[rw][i][j] = 0.0f;
          continue;
        }
        const long long grow = row0 + row;
        float4* rr = reinterpret_cast<float4*>(q.residual) + (long long)row * (nvec * 2);
        int s_next = 0;  // the next segment of this row this warp has not passed
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = tid + i * nthreads;
          const int v_warp = v - lane;
          bool has = false;
          uint4 xv = make_uint4(0, 0, 0, 0);
          float4 a4 = make_float4(0.f, 0.f, 0.f, 0.f), b4 = a4;
          if (v_warp < nvec) {
            const int s_mine = v_warp >> 8;
            for (; s_next < s_mine; ++s_next) {  // segments other warps read
              ring.wait_full(seg + s_next);
              ring.release(seg + s_next);
            }
            const uint32_t gseg = seg + s_mine;
            has = ring.wait_full(gseg) && v < nvec;
            if (has) {
              const uint32_t sb = ring.buf(gseg);
              const uint32_t slot = (uint32_t)(v & (kNxSegVecs - 1));
              if (!q.sum_peers) {
                xv = lds_128(sb + slot * 16);
              } else if (SW) {
                xv = xs[SW ? rw : 0][SW ? i : 0];
              } else {
                float s8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) s8[j] = 0.0f;
#pragma unroll
                for (int k = 0; k < kArMaxWorld; ++k) {
                  if (k < p.world) {
                    const uint4 pv = lds_128(sb + (uint32_t)k * kNxSrcBytes + slot * 16);
                    s8[0] += bf16lo_to_f32(pv.x); s8[1] += bf16hi_to_f32(pv.x); s8[2] += bf16lo_to_f32(pv.y); s8[3] += bf16hi_to_f32(pv.y);
                    s8[4] += bf16lo_to_f32(pv.z); s8[5] += bf16hi_to_f32(pv.z); s8[6] += bf16lo_to_f32(pv.w); s8[7] += bf16hi_to_f32(pv.w);
                  }
                }
                xv = make_uint4(pack_bf16x2(s8[0], s8[1]), pack_bf16x2(s8[2], s8[3]), pack_bf16x2(s8[4], s8[5]), pack_bf16x2(s8[6], s8[7]));
              }
              a4 = lds_128f(sb + (uint32_t)n_src * kNxSrcBytes + slot * 32);
              b4 = lds_128f(sb + (uint32_t)n_src * kNxSrcBytes + slot * 32 + 16);
            }
            ring.release(gseg);
            s_next = s_mine + 1;
          }
          if (has) {
            r[rw][i][0] = __fadd_rn(a4.x, bf16lo_to_f32(xv.x));
            r[rw][i][1] = __fadd_rn(a4.y, bf16hi_to_f32(xv.x));
            r[rw][i][2] = __fadd_rn(a4.z, bf16lo_to_f32(xv.y));
            r[rw][i][3] = __fadd_rn(a4.w, bf16hi_to_f32(xv.y));
            r[rw][i][4] = __fadd_rn(b4.x, bf16lo_to_f32(xv.z));
            r[rw][i][5] = __fadd_rn(b4.y, bf16hi_to_f32(xv.z));
            r[rw][i][6] = __fadd_rn(b4.z, bf16lo_to_f32(xv.w));
            r[rw][i][7] = __fadd_rn(b4.w, bf16hi_to_f32(xv.w));
            __stcs(rr + 2 * v, make_float4(r[rw][i][0], r[rw][i][1], r[rw][i][2], r[rw][i][3]));
            __stcs(rr + 2 * v + 1, make_float4(r[rw][i][4], r[rw][i][5], r[rw][i][6], r[rw][i][7]));
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[rw] = fmaf(r[rw][i][j], r[rw][i][j], acc[rw]);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) r[rw][i][j] = 0.0f;
          }
        }
        for (; s_next < nseg1; ++s_next) {
          ring.wait_full(seg + s_next);
          ring.release(seg + s_next);
        }
        seg += (uint32_t)nseg1;
      }
#pragma unroll
      for (int rw = 0; rw < kRows; ++rw) {
        for (int o = 16; o > 0; o >>= 1) acc[rw] += __shfl_xor_sync(0xFFFFFFFFu, acc[rw], o);
        if (lane == 0) warp_sums[rw][tid >> 5] = acc[rw];
      }
      consumer_barrier(nthreads);
      if (abort_flag) break;  // a copy never landed: every consumer sees the flag here and leaves with the others
      if (tid < 32) {
#pragma unroll
        for (int rw = 0; rw < kRows; ++rw) {
          float sm = (tid < (nthreads >> 5)) ? warp_sums[rw][tid] : 0.0f;
          for (int o = 8; o > 0; o >>= 1) sm += __shfl_xor_sync(0xFFFFFFFFu, sm, o);
          if (tid == 0) row_rstd[rw] = __frsqrt_rn(__fadd_rn(__fmul_rn(sm, q.inv_d), q.eps));
        }
      }
      consumer_barrier(nthreads);
#pragma unroll
      for (int rw = 0; rw < kRows; ++rw) {
        const int row = base + rw * (int)gridDim.x;
        const float rstd = row_rstd[rw];
        if (row < rows_local) {
#pragma unroll
          for (int i = 0; i < VPT; ++i) {
            const int v = tid + i * nthreads;
            if (v < nvec) {
              const uint4 wv = __ldg(q.w + v);
              uint4 o;
              o.x = pack_bf16x2(__fmul_rn(__fmul_rn(r[rw][i][0], rstd), bf16lo_to_f32(wv.x)), __fmul_rn(__fmul_rn(r[rw][i][1], rstd), bf16hi_to_f32(wv.x)));
              o.y = pack_bf16x2(__fmul_rn(__fmul_rn(r[rw][i][2], rstd), bf16lo_to_f32(wv.y)), __fmul_rn(__fmul_rn(r[rw][i][3], rstd), bf16hi_to_f32(wv.y)));
              o.z = pack_bf16x2(__fmul_rn(__fmul_rn(r[rw][i][4], rstd), bf16lo_to_f32(wv.z)), __fmul_rn(__fmul_rn(r[rw][i][5], rstd), bf16hi_to_f32(wv.z)));
              o.w = pack_bf16x2(__fmul_rn(__fmul_rn(r[rw][i][6], rstd), bf16lo_to_f32(wv.w)), __fmul_rn(__fmul_rn(r[rw][i][7], rstd), bf16hi_to_f32(wv.w)));
              q.h_scratch[(long long)row * nvec + v] = o;
              amax_bits = max(amax_bits, amax_bits8(o));
            }
          }
        }
      }
      // warp_sums / row_rstd are rewritten only after the next round's first consumer barrier, which every thread reaches after these reads
    }
    if (QFMT == TF_FMT_NVFP4) {  // the row block's amax: one atomic per CTA
      for (int o = 16; o > 0; o >>= 1) amax_bits = max(amax_bits, __shfl_xor_sync(0xFFFFFFFFu, amax_bits, o));
      if (lane == 0) warp_amax[tid >> 5] = amax_bits;
      consumer_barrier(nthreads);
      if (tid == 0) {
        for (int wi = 1; wi < (nthreads >> 5); ++wi) amax_bits = max(amax_bits, warp_amax[wi]);
        if (amax_bits) atomicMax(q.amax, amax_bits << 16);
      }
    }
    fence_proxy_async();  // pass 2 reads the normalised rows back with bulk copies
  }
  ok = ar_grid_sync(grid_counter, gbase + (++syncs) * g, error_word, limit_ns);
  // both roles restart the segment count together (a pass that was cut short leaves them apart; then ok is false and pass 2 is skipped)
  const int my_rows = blockIdx.x < rows_local ? (rows_local - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  seg = (uint32_t)my_rows * (uint32_t)nseg1;

  // ---- pass 2: quantize this rank's rows into every rank's buffers ----
  const int nvec16 = q.d >> 4;
  const int nseg2 = (nvec16 + kNxSegVecs - 1) / kNxSegVecs;
  if (ok && producer) {
    fence_proxy_async();
    bool alive = true;
    for (int row = blockIdx.x; alive && row < rows_local; row += gridDim.x) {
      for (int s = 0; s < nseg2; ++s, ++seg) {
        alive = ring.wait_empty(seg);
        if (!alive) break;
        const int v0 = s * kNxSegVecs;
        const uint32_t nv = (uint32_t)min(kNxSegVecs, nvec16 - v0);
        if (lane == 0) {
          mbar_expect_tx(ring.full_bar(seg), nv * 32u);
          bulk_load(ring.buf(seg), q.h_scratch + ((long long)row * nvec16 + v0) * 2, nv * 32u, ring.full_bar(seg));
        }
      }
    }
  } else if (ok) {
    float gs = 0.0f, inv_t = 0.0f;
    if (QFMT == TF_FMT_NVFP4) {
      gs = __fdiv_rn(__uint_as_float(*reinterpret_cast<volatile unsigned int*>(q.amax)), 2688.0f);
      inv_t = gs != 0.0f ? __frcp_rn(__fmul_rn(6.0f, gs)) : 0.0f;
      if (blockIdx.x == 0 && tid == 0) store_all_ranks<4>(p, q.gs_off + 4ll * p.rank, __float_as_uint(gs), 0, 0, 0);
    }
    const int rounds = (nvec16 + nthreads - 1) / nthreads;
    // this warp's piece of one row: passes the row's segments before it, waits for its own, takes its 32 bytes
    auto fetch = [&](uint32_t seg_row, int& s_next, int v, uint32_t (&w8)[8]) -> bool {
      const int s_mine = (v - lane) >> 8;
      for (; s_next < s_mine; ++s_next) {
        ring.wait_full(seg_row + s_next);
        ring.release(seg_row + s_next);
      }
      const uint32_t gseg = seg_row + s_mine;
      const bool has = ring.wait_full(gseg) && v < nvec16;
      if (has) {
        const uint32_t a = ring.buf(gseg) + (uint32_t)(v & (kNxSegVecs - 1)) * 32;
        const uint4 lo = lds_128(a), hi = lds_128(a + 16);
        w8[0] = lo.x; w8[1] = lo.y; w8[2] = lo.z; w8[3] = lo.w; w8[4] = hi.x; w8[5] = hi.y; w8[6] = hi.z; w8[7] = hi.w;
      }
      ring.release(gseg);
      s_next = s_mine + 1;
      return has;
    };
    auto pass_rest = [&](uint32_t seg_row, int& s_next) {
      for (; s_next < nseg2; ++s_next) {
        ring.wait_full(seg_row + s_next);
        ring.release(seg_row + s_next);
      }
    };
    if (rounds == 1) {
      // rows of up to one piece per thread: kRows2 rows per round (in the producer's order), so that a warp's quantizations interleave
      constexpr int kRows2 = 4;
      const bool active = tid - lane < nvec16;  // whole warps only: the quantizer and the scale packing shuffle
      for (int base = blockIdx.x; base < rows_local; base += gridDim.x * kRows2) {
        uint32_t wq[kRows2][8];
        bool has[kRows2];
#pragma unroll
        for (int rw = 0; rw < kRows2; ++rw) {
#pragma unroll
          for (int e = 0; e < 8; ++e) wq[rw][e] = 0;
          has[rw] = false;
          if (base + rw * (int)gridDim.x < rows_local) {
            int s_next = 0;
            if (active) has[rw] = fetch(seg, s_next, tid, wq[rw]);
            pass_rest(seg, s_next);
            seg += (uint32_t)nseg2;
          }
        }
        if (active) {
#pragma unroll
          for (int rw = 0; rw < kRows2; ++rw)
            if (base + rw * (int)gridDim.x < rows_local) quantize_store_piece<QFMT>(p, q, wq[rw], has[rw], row0 + base + rw * (int)gridDim.x, tid, gs, inv_t);
        }
        if (abort_flag) break;  // a warp's own waits return at once after the flag is up; nothing here meets the other warps
      }
    } else {
      for (int row = blockIdx.x; row < rows_local; row += gridDim.x) {
        int s_next = 0;
        for (int rd = 0; rd < rounds; ++rd) {
          const int v = rd * nthreads + tid;
          if (v - lane >= nvec16) break;
          uint32_t w8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          const bool has = fetch(seg, s_next, v, w8);
          quantize_store_piece<QFMT>(p, q, w8, has, row0 + row, v, gs, inv_t);
        }
        pass_rest(seg, s_next);
        seg += (uint32_t)nseg2;
        if (abort_flag) break;
      }
    }
  }
  // every rank's rows have landed everywhere
  ar_grid_sync(grid_counter, gbase + (++syncs) * g, error_word, limit_ns);
  ar_cross_barrier(p, flag + 2, error_word, limit_ns);
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *grid_base = gbase + syncs * g;
    __threadfence();
    *call_counter = call + 1ull;
  }
  if (tid == 0 && abort_flag) {  // a wait ran out: give copies still in flight time to land before shared memory is released
    const unsigned long long t0 = ar_timer();
    while (ar_timer() - t0 < 200000ull) __nanosleep(1000);
  }
}

}  // namespace tf

using namespace tf;

extern "C" tf_status tf_allreduce_bf16(const uint64_t* buffer_ptrs, const uint64_t* state_ptrs, uint64_t multicast_ptr, int32_t reduce_in_switch, int32_t rank,
                                       int32_t world, int64_t offset_bytes, int64_t count, int32_t num_ctas, void* stream) {
  clear_error();
  TF_CHECK_ARG(buffer_ptrs && state_ptrs, "%s: null pointer", __func__);
  TF_CHECK_ARG(world >= 2 && world <= kArMaxWorld && rank >= 0 && rank < world, "%s: bad rank %d / world %d (2..8 ranks)", __func__, rank, world);
  TF_CHECK_ARG(count > 0 && count % (8 * world) == 0, "%s: count must be a positive multiple of 8 x world", __func__);
  TF_CHECK_ARG(offset_bytes >= 0 && offset_bytes % 16 == 0, "%s: offset_bytes must be a multiple of 16", __func__);
  TF_CHECK_ARG(num_ctas >= 1 && num_ctas <= 148, "%s: num_ctas must be in 1..148", __func__);
  ArParams p;
  for (int i = 0; i < kArMaxWorld; ++i) {
    p.bufs[i] = i < world ? buffer_ptrs[i] : 0;
    p.states[i] = i < world ? state_ptrs[i] : 0;
    if (i < world && (!p.bufs[i] || !p.states[i] || p.bufs[i] % 16 || p.states[i] % 16)) return fail(TF_ERR_ALIGNMENT, "%s: peer pointer %d is null or unaligned", __func__, i);
  }
  p.mc_ptr = multicast_ptr;
  p.reduce_in_switch = reduce_in_switch != 0 && multicast_ptr != 0;
  p.rank = rank;
  p.world = world;
  p.offset_bytes = offset_bytes;
  p.count = count;
  int grid = num_ctas;
  const int sms = sm_count();
  if (grid > sms) grid = sms;
  allreduce_bf16_kernel<<<grid, kArThreads, 0, (cudaStream_t)stream>>>(p);
  TF_LAUNCH_CHECK();
  return TF_OK;
}

template <int VPT, int QFMT, bool SW>
static cudaError_t launch_norm_exchange_sw(int grid, int threads, cudaStream_t stream, const NxParams& q, int stages, int stage_bytes) {
  const size_t smem = (size_t)stages * stage_bytes + 16 * (size_t)stages;
  static thread_local int configured_dev = -1;  // per instantiation: the kernel may use all of the SM's shared memory
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (configured_dev != dev) {
    e = cudaFuncSetAttribute(tp_norm_exchange_kernel<VPT, QFMT, SW>, cudaFuncAttributeMaxDynamicSharedMemorySize, kNxSmemBudget + 16 * kNxMaxStages);
    if (e != cudaSuccess) return e;
    configured_dev = dev;
  }
  tp_norm_exchange_kernel<VPT, QFMT, SW><<<grid, threads + 32, smem, stream>>>(q, stages, stage_bytes);
  return cudaGetLastError();
}

template <int VPT, int QFMT>
static cudaError_t launch_norm_exchange_fmt(int grid, int threads, cudaStream_t stream, const NxParams& q, int stages, int stage_bytes) {
  if (q.sum_peers && q.ar.reduce_in_switch) return launch_norm_exchange_sw<VPT, QFMT, true>(grid, threads, stream, q, stages, stage_bytes);
  return launch_norm_exchange_sw<VPT, QFMT, false>(grid, threads, stream, q, stages, stage_bytes);
}

template <int VPT>
static cudaError_t launch_norm_exchange(int q_format, int grid, int threads, cudaStream_t stream, const NxParams& q, int stages, int stage_bytes) {
  switch (q_format) {
    case TF_FMT_MXFP8: return launch_norm_exchange_fmt<VPT, TF_FMT_MXFP8>(grid, threads, stream, q, stages, stage_bytes);
    case TF_FMT_MXFP4: return launch_norm_exchange_fmt<VPT, TF_FMT_MXFP4>(grid, threads, stream, q, stages, stage_bytes);
    default: return launch_norm_exchange_fmt<VPT, TF_FMT_NVFP4>(grid, threads, stream, q, stages, stage_bytes);
  }
}

extern "C" tf_status tf_tp_norm_exchange(const uint64_t* buffer_ptrs, const uint64_t* state_ptrs, uint64_t multicast_ptr, int32_t reduce_in_switch,
                                         int32_t rank, int32_t world, int64_t partial_offset, int64_t codes_offset, int64_t scales_offset,
                                         int64_t gs_offset, int64_t rows_total, int64_t d, int32_t sum_peers, void* residual_rows, const void* w,
                                         void* h_scratch, float* amax, float eps, int32_t q_format, int32_t num_ctas, void* stream) {
  clear_error();
  TF_CHECK_ARG(buffer_ptrs && state_ptrs && residual_rows && w && h_scratch, "%s: null pointer", __func__);
  TF_CHECK_ARG(world >= 1 && world <= kArMaxWorld && rank >= 0 && rank < world, "%s: bad rank %d / world %d (1..8 ranks)", __func__, rank, world);
  TF_CHECK_ARG(q_format >= TF_FMT_MXFP8 && q_format <= TF_FMT_NVFP4, "%s: unknown format %d", __func__, q_format);
  TF_CHECK_ARG(q_format != TF_FMT_NVFP4 || amax, "%s: nvfp4 needs the amax word", __func__);
  TF_CHECK_ARG(rows_total > 0 && rows_total % (128 * world) == 0, "%s: rows must be a positive multiple of 128 x world", __func__);
  TF_CHECK_ARG(rows_total <= (1 << 24), "%s: too many rows", __func__);
  if (d <= 0 || d % 128 != 0 || d > 32768) return fail(TF_ERR_UNSUPPORTED, "%s: d=%lld must be a multiple of 128, at most 32768", __func__, (long long)d);
  TF_CHECK_ARG(partial_offset >= 0 && partial_offset % 16 == 0 && codes_offset >= 0 && codes_offset % 16 == 0 && scales_offset >= 0 &&
                   scales_offset % 16 == 0 && gs_offset >= 0 && gs_offset % 16 == 0,
               "%s: offsets must be multiples of 16", __func__);
  TF_CHECK_ARG(num_ctas >= 1 && num_ctas <= 148, "%s: num_ctas must be in 1..148", __func__);
  TF_CHECK_ALIGNED(residual_rows, 16, "residual_rows");
  TF_CHECK_ALIGNED(w, 16, "w");
  TF_CHECK_ALIGNED(h_scratch, 16, "h_scratch");
  NxParams q;
  for (int i = 0; i < kArMaxWorld; ++i) {
    q.ar.bufs[i] = i < world ? buffer_ptrs[i] : 0;
    q.ar.states[i] = i < world ? state_ptrs[i] : 0;
    if (i < world && (!q.ar.bufs[i] || !q.ar.states[i] || q.ar.bufs[i] % 16 || q.ar.states[i] % 16))
      return fail(TF_ERR_ALIGNMENT, "%s: peer pointer %d is null or unaligned", __func__, i);
  }
  q.ar.mc_ptr = multicast_ptr;
  q.ar.reduce_in_switch = reduce_in_switch != 0 && multicast_ptr != 0;
  q.ar.rank = rank;
  q.ar.world = world;
  q.ar.offset_bytes = 0;
  q.ar.count = 0;
  q.partial_off = partial_offset;
  q.codes_off = codes_offset;
  q.scales_off = scales_offset;
  q.gs_off = gs_offset;
  q.rows_total = (int)rows_total;
  q.d = (int)d;
  TF_CHECK_ARG(sum_peers >= 0 && sum_peers <= 2, "%s: sum_peers must be 0, 1 or 2", __func__);
  TF_CHECK_ARG(sum_peers != 2 || !(reduce_in_switch && multicast_ptr), "%s: the switch reduction cannot sum delivered (sum_peers = 2) partials", __func__);
  q.sum_peers = world > 1 ? sum_peers : 0;
  q.residual = static_cast<float*>(residual_rows);
  q.w = static_cast<const uint4*>(w);
  q.h_scratch = static_cast<uint4*>(h_scratch);
  q.amax = reinterpret_cast<unsigned int*>(amax);
  q.eps = eps;
  q.inv_d = 1.0f / (float)d;
  // the thread mapping of residual_add_rmsnorm_kernel, so that the row sums are formed in the same order
  const int nvec = (int)(d >> 3);
  int vpt = (nvec + 511) / 512;
  vpt = vpt <= 1 ? 1 : vpt <= 2 ? 2 : vpt <= 4 ? 4 : 8;
  int threads = (nvec + vpt - 1) / vpt;
  threads = (threads + 31) / 32 * 32;
  int grid = num_ctas;
  const int sms = sm_count();
  if (grid > sms) grid = sms;
  const int64_t rows_local = rows_total / world;
  if (grid > rows_local) grid = (int)rows_local;
  // the ring: a stage holds one segment of every bf16 source of the sum plus the f32 residual (pass 1), or 8 KB of normalised rows (pass 2)
  const int n_src = !q.sum_peers ? 1 : (q.ar.reduce_in_switch ? 0 : world);
  const int stage_bytes = n_src * kNxSrcBytes + kNxSegVecs * 32;
  int stages = kNxMaxStages;  // a power of two
  while (stages > 1 && stages * stage_bytes > kNxSmemBudget) stages >>= 1;
  cudaError_t e;
  switch (vpt) {
    case 1: e = launch_norm_exchange<1>(q_format, grid, threads, (cudaStream_t)stream, q, stages, stage_bytes); break;
    case 2: e = launch_norm_exchange<2>(q_format, grid, threads, (cudaStream_t)stream, q, stages, stage_bytes); break;
    case 4: e = launch_norm_exchange<4>(q_format, grid, threads, (cudaStream_t)stream, q, stages, stage_bytes); break;
    default: e = launch_norm_exchange<8>(q_format, grid, threads, (cudaStream_t)stream, q, stages, stage_bytes); break;
  }
  if (e != cudaSuccess) return fail(TF_ERR_CUDA, "%s: launch failed: %s", __func__, cudaGetErrorString(e));
  return TF_OK;
}
