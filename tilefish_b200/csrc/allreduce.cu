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
// No TMA anywhere in this file.
//
// Cross-GPU barriers are flags in peer memory: every rank stores a monotonically increasing value into its slot of every
// peer's flag array (st.release.sys) and spins on its own array (ld.acquire.sys). The value is derived from a call counter kept
// in this rank's device memory and advanced by the kernel itself, so a CUDA-graph replay (which repeats the same launch
// arguments) still produces fresh values. Every spin is bounded by %globaltimer (two seconds): on a timeout the kernel writes an
// error word into the state block and returns; nothing traps and nothing spins forever. The kernels of all ranks must be
// running at the same time for the barriers to complete: that holds because every rank is its own GPU.
#include "common.cuh"

namespace tf {

constexpr int kArMaxWorld = 8;
constexpr int kArThreads = 512;
constexpr unsigned long long kArWaitLimitNs = 2000000000ull;

// Layout of the per-rank state block (symmetric memory, zero-initialised by the host): 32-bit flag slots [0, 8), then
// 64-bit words at byte 64: call counter, local grid-barrier counter, its value at the start of the call, error word (0 = healthy,
// 1 = a local grid barrier gave up, 2 = a peer never arrived). 128 bytes in all.
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
__device__ __forceinline__ bool ar_grid_sync(unsigned long long* counter, unsigned long long target, volatile unsigned long long* error_word) {
  __shared__ int ok_s;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    atomicAdd(counter, 1ull);
    const unsigned long long t0 = ar_timer();
    while (*error_word == 0 && ld_acquire_gpu64(counter) < target) {
      if (ar_timer() - t0 > kArWaitLimitNs) *error_word = 1;
    }
    ok_s = *error_word == 0;
  }
  __syncthreads();
  return ok_s != 0;
}

// Block 0 tells every peer "this rank reached `value`" and waits until every peer told it the same.
__device__ __forceinline__ void ar_cross_barrier(const ArParams& p, unsigned int value, volatile unsigned long long* error_word) {
  if (blockIdx.x == 0 && threadIdx.x < p.world) {
    __threadfence_system();
    unsigned int* peer_flags = reinterpret_cast<unsigned int*>(p.states[threadIdx.x]);
    st_release_sys(peer_flags + p.rank, value);
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(p.states[p.rank]) + threadIdx.x;
    const unsigned long long t0 = ar_timer();
    while (*error_word == 0 && (int)(ld_acquire_sys(mine) - value) < 0) {
      if (ar_timer() - t0 > kArWaitLimitNs) *error_word = 2;
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
  ar_cross_barrier(p, flag + 1, error_word);
  bool ok = ar_grid_sync(grid_counter, gbase + (++syncs) * g, error_word);

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
  ok = ar_grid_sync(grid_counter, gbase + (++syncs) * g, error_word);
  ar_cross_barrier(p, flag + 2, error_word);
  ok = ar_grid_sync(grid_counter, gbase + (++syncs) * g, error_word);

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
    ar_grid_sync(grid_counter, gbase + (++syncs) * g, error_word);
    ar_cross_barrier(p, flag + 3, error_word);
  }
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *grid_base = gbase + syncs * g;
    __threadfence();
    *call_counter = call + 1ull;
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
