// Shared host/device helpers of the sm_100a backend.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/tilefish_b200.h"

namespace tf {

// ---- host: status + thread-local last error ------------------------------------------------------------------------
tf_status fail(tf_status code, const char* fmt, ...);
void clear_error();
int sm_count();

#define TF_CHECK_ARG(cond, ...)                                   \
  do {                                                            \
    if (!(cond)) return tf::fail(TF_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)
#define TF_CHECK_ALIGNED(ptr, bytes, name)                                                                  \
  do {                                                                                                      \
    if ((reinterpret_cast<uintptr_t>(ptr) % (bytes)) != 0)                                                  \
      return tf::fail(TF_ERR_ALIGNMENT, "%s: %s must be %d-byte aligned", __func__, name, (int)(bytes));    \
  } while (0)
#define TF_CUDA(call)                                                                                       \
  do {                                                                                                      \
    cudaError_t e__ = (call);                                                                               \
    if (e__ != cudaSuccess) return tf::fail(TF_ERR_CUDA, "%s: %s failed: %s", __func__, #call, cudaGetErrorString(e__)); \
  } while (0)
#define TF_LAUNCH_CHECK() TF_CUDA(cudaGetLastError())

// Programmatic dependent launch (tf_set_programmatic_launch): a kernel launched through launch_dependent() may be scheduled
// while the kernel before it on the stream is still draining, so that its launch latency and set-up overlap that tail. Every
// kernel launched this way executes griddep_wait() before its first access to global memory, which blocks until the previous
// kernel has completed and its writes are visible. Off: a plain stream-ordered launch.
bool programmatic_launch_enabled();
void set_programmatic_launch(bool on);

#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = programmatic_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// ---- device: bit-level conversions -----------------------------------------------------------------------------------
#ifdef __CUDACC__

// Wait for the previous kernel on the stream (returns at once in a plain launch); let the next one be scheduled early.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float bf16lo_to_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// f32 -> bf16 word, round to nearest even, NaN -> 0x7FFF (what cvt.rn.bf16.f32 gives).
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  uint16_t r;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// two f32 -> two e4m3 bytes (lo in bits 0-7), RNE, saturating to +-448, NaN -> 0x7F.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
// two f32 -> two e2m1 nibbles in one byte (lo in bits 0-3), RNE ties-to-even, saturating to +-6.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint16_t r;
  asm("{ .reg .b8 t;\n cvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n mov.b16 %0, {t, 0}; }" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
// one e4m3 byte -> f32 (exact).
__device__ __forceinline__ float e4m3_to_f32(uint32_t code) {
  uint32_t h2;
  uint16_t c = (uint16_t)code;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(c));
  float f;
  asm("{ .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %1;\n cvt.f32.f16 %0, lo; }" : "=f"(f) : "r"(h2));
  return f;
}

// silu(x) = x * (1 / (1 + exp(-x))) with the hardware's approximate exp2 and reciprocal (what the reference's own binaries use:
// ex2.approx and div.full). One definition for the stand-alone kernel and the GEMM epilogue, so both give the same bytes.
__device__ __forceinline__ float silu_f32(float g) { return __fmul_rn(g, __fdividef(1.0f, __fadd_rn(1.0f, __expf(-g)))); }

// Byte offset of scale entry (r, c) of a [rows, cols] scale tensor in the swizzled layout; n_ct = ceil(cols / 4).
__host__ __device__ __forceinline__ int64_t swizzled_scale_offset(int64_t r, int64_t c, int64_t n_ct) {
  int64_t tile = (r >> 7) * n_ct + (c >> 2);
  int rr = (int)(r & 127);
  return tile * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (int)(c & 3);
}

#endif  // __CUDACC__

}  // namespace tf
