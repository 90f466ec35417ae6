// SiLU gate of two bf16 [M, F] operands, e.g. the column halves of a [M, 2F] matrix (the stand-alone form; the GEMM also has
// it as an epilogue).
//   out[m, j] = bf16( silu(f32(t[m, j])) * f32(t[m, F + j]) ),  silu(x) = x * (1 / (1 + exp(-x)))
// HBM-bound elementwise kernel: 6 bytes per output element, 128-bit loads and stores.
#include "common.cuh"

namespace tf {

__device__ __forceinline__ float silu_gate1(float g, float u) {
  return __fmul_rn(silu_f32(g), u);
}

__global__ void __launch_bounds__(256) silu_gate_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, int64_t m, int fvec,
                                                        int64_t ldg_vec, int64_t ldu_vec, uint4* __restrict__ out, int64_t ldo_vec) {
  const int64_t total = m * fvec;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += 2 * stride) {  // two vector pairs in flight
    uint4 g[2], u[2];
    int64_t oidx[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int64_t i = i0 + j * stride;
      oidx[j] = -1;
      if (i < total) {
        const int64_t row = i / fvec;
        const int v = (int)(i - row * fvec);
        g[j] = __ldcs(gate + row * ldg_vec + v);
        u[j] = __ldcs(up + row * ldu_vec + v);
        oidx[j] = row * ldo_vec + v;
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (oidx[j] < 0) continue;
      uint4 o;
      o.x = pack_bf16x2(silu_gate1(bf16lo_to_f32(g[j].x), bf16lo_to_f32(u[j].x)), silu_gate1(bf16hi_to_f32(g[j].x), bf16hi_to_f32(u[j].x)));
      o.y = pack_bf16x2(silu_gate1(bf16lo_to_f32(g[j].y), bf16lo_to_f32(u[j].y)), silu_gate1(bf16hi_to_f32(g[j].y), bf16hi_to_f32(u[j].y)));
      o.z = pack_bf16x2(silu_gate1(bf16lo_to_f32(g[j].z), bf16lo_to_f32(u[j].z)), silu_gate1(bf16hi_to_f32(g[j].z), bf16hi_to_f32(u[j].z)));
      o.w = pack_bf16x2(silu_gate1(bf16lo_to_f32(g[j].w), bf16lo_to_f32(u[j].w)), silu_gate1(bf16hi_to_f32(g[j].w), bf16hi_to_f32(u[j].w)));
      __stcs(out + oidx[j], o);
    }
  }
}

}  // namespace tf

using namespace tf;

extern "C" tf_status tf_silu_gate(const void* gate, const void* up, int64_t m, int64_t f, int64_t ldg, int64_t ldu, void* out, int64_t ldo,
                                  void* stream) {
  clear_error();
  TF_CHECK_ARG(gate && up && out, "%s: null pointer", __func__);
  TF_CHECK_ARG(m >= 0 && f > 0, "%s: bad shape m=%lld f=%lld", __func__, (long long)m, (long long)f);
  if (f % 8 || ldg % 8 || ldu % 8 || ldo % 8 || ldg < f || ldu < f || ldo < f)
    return fail(TF_ERR_ALIGNMENT, "%s: f and the row strides must be multiples of 8, strides >= f", __func__);
  TF_CHECK_ALIGNED(gate, 16, "gate");
  TF_CHECK_ALIGNED(up, 16, "up");
  TF_CHECK_ALIGNED(out, 16, "out");
  if (m == 0) return TF_OK;
  const int64_t total = m * (f >> 3);
  const int64_t need = (total + 511) / 512, cap = (int64_t)sm_count() * 8;
  silu_gate_kernel<<<(unsigned)(need < cap ? need : cap), 256, 0, (cudaStream_t)stream>>>(
      static_cast<const uint4*>(gate), static_cast<const uint4*>(up), m, (int)(f >> 3), ldg >> 3, ldu >> 3, static_cast<uint4*>(out), ldo >> 3);
  TF_LAUNCH_CHECK();
  return TF_OK;
}
