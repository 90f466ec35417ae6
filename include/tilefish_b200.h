/*
 * tilefish_b200 -- C ABI of the sm_100a backend for tilefish's quantized-inference hot path.
 *
 * Conventions (modelled on the reference's C ABI, crates/tilefish-capi/include/tilefish.h:388-430 and
 * crates/tilefish-capi/src/error.rs:14-102):
 *   - every entry point returns a tf_status (0 = OK); tf_last_error() gives the message of the last failure on the
 *     calling thread;
 *   - tensors are regions the caller vouches for: plain device pointers plus sizes, caller-owned, caller-ordered;
 *   - the stream is a borrowed CUDA stream handle (NULL = the legacy default stream); calls only enqueue work and
 *     never synchronize or allocate, unless their comment says otherwise; the CUDA context is left as found;
 *   - nothing is allocated inside a launch: scratch memory is passed in as a workspace;
 *   - no C++ exception crosses the boundary.
 *
 * The reference binds this path through three leaves, which these entry points replace:
 *   - a Triton cubin launched with cuLaunchKernel  (python/src/tilefish/_cuda.py:356-458)  -> the row kernels below;
 *   - a pinned cublasLtMatmul                      (python/src/tilefish/_cublaslt.py:1372-1455) -> tf_gemm_blockscaled;
 *   - the runner back-end interface                (python/src/tilefish/_planrun.py:240-376: launch / gemm).
 */
#ifndef TILEFISH_B200_H
#define TILEFISH_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define TF_API __attribute__((visibility("default")))
#else
#define TF_API
#endif

typedef int32_t tf_status;

enum {
  TF_OK = 0,
  TF_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, unknown enum value */
  TF_ERR_ALIGNMENT = 2,        /* a pointer or leading dimension is not aligned as the entry point requires */
  TF_ERR_UNSUPPORTED = 3,      /* a shape this build has no kernel for (K not a multiple of the block, D too large ...) */
  TF_ERR_CUDA = 4,             /* a CUDA runtime/driver call failed; the message carries its error string */
  TF_ERR_WORKSPACE = 5,        /* the workspace is too small (see the *_workspace_bytes query) */
  TF_ERR_DEVICE_TIMEOUT = 6    /* a bounded wait inside a kernel ran out (read by tf_device_status) */
};

/* BlockScaled formats (python/src/tilefish/dtypes.py:145-232; README.md:47-49 of the reference). */
enum {
  TF_FMT_MXFP8 = 0, /* e4m3 elements, ue8m0 scale, block 32 */
  TF_FMT_MXFP4 = 1, /* e2m1 elements (two per byte, element 2i in bits 0-3), ue8m0 scale, block 32 */
  TF_FMT_NVFP4 = 2  /* e2m1 elements, e4m3 scale, block 16, f32 global scale */
};

/* Scale-byte layouts. PLAIN is row-major [rows, K/block]. SWIZZLED is the sm_100 block-scaled MMA operand layout:
 * 128-row x 4-column tiles of 512 bytes, row-tile major; inside a tile byte(r, c) = (r%32)*16 + (r/32)*4 + c; rows are
 * padded to 128 and columns to 4 with zero bytes. */
enum { TF_SCALES_PLAIN = 0, TF_SCALES_SWIZZLED = 1 };

/* GEMM epilogues. */
enum {
  TF_EPI_NONE = 0,      /* out[M,N] = bf16(acc) */
  TF_EPI_SILU_GATE = 1, /* b holds gate rows [0,N) then up rows [N,2N): out[M,N] = bf16(silu(bf16(acc_g)) * bf16(acc_u)) */
  TF_EPI_RESIDUAL = 2   /* out[M,N] = bf16(acc); residual_f32[M,N] += f32(out) */
};

/* Library identity and errors. Replaces tilefish_version / tilefish_last_error (crates/tilefish-capi/src/error.rs:86-102). */
TF_API const char* tf_version(void);
TF_API const char* tf_last_error(void);

/* Reads and clears the device-side status word that kernels with bounded waits set when a wait runs out.
 * SYNCHRONIZES the device. *status is TF_OK or TF_ERR_DEVICE_TIMEOUT; *detail identifies the wait that gave up. */
TF_API tf_status tf_device_status(int32_t* status, int32_t* detail);

/* PROCESS-WIDE and not synchronized with calls in flight on other threads (set it while no other thread launches): the persistent GEMM
 * launches on (SM count - sms) SMs from now on, for every caller in the process, tf_gemm_blockscaled_static included; a CUDA graph keeps
 * the grid that was in force when it was captured. Purpose: so that a collective running beside it in
 * another stream (the tensor-parallel MLP overlaps one row chunk's all-reduce with the other chunk's GEMMs) finds free SMs.
 * 0 restores the default. No counterpart in the reference (its GEMM is cuBLASLt's `sm_count_target`, python/src/tilefish/_cublaslt.py). */
TF_API tf_status tf_set_sm_margin(int32_t sms);

/* Programmatic dependent launch for this library's kernels (off by default; PROCESS-WIDE, as tf_set_sm_margin). On: the quantize, rmsnorm, GEMM and
 * split-K reduction kernels are launched so that each may be scheduled while the kernel before it on the stream is still
 * draining; each waits (griddepcontrol.wait) for that kernel to complete before its first access to global memory, so results
 * are unchanged. It hides launch latency and kernel set-up in chains of short kernels (small M, decode, many GPUs). No
 * counterpart in the reference. */
TF_API tf_status tf_set_programmatic_launch(int32_t enabled);

/* Failure-detection self-test (no counterpart in the reference): launches one thread that waits on a barrier nothing will ever
 * signal, with the given limit. The wait gives up, records TF_ERR_DEVICE_TIMEOUT (detail 9 * 65536) in the device status word
 * and the kernel returns normally; the context stays usable. Exercises the mechanism every wait of the GEMM relies on. */
TF_API tf_status tf_selftest_bounded_wait(int32_t limit_ms, void* stream);

/* Bytes of the scale tensor of a [rows, k] operand in `format`, in `layout`. Returns -1 on a bad argument. */
TF_API int64_t tf_scale_bytes(int32_t format, int64_t rows, int64_t k, int32_t layout);

/* BlockScaled quantization of a bf16 matrix along its last axis. The reference types this operation but refuses to run
 * it (python/src/tilefish/ops.py:556-559); these entry points are what `x.to(mxfp8)` lowers to here.
 *   x        bf16 [m, k], row stride ldx elements (ldx >= k, ldx % 16 == 0), 32-byte aligned (256-bit loads)
 *   codes    [m, k] bytes (mxfp8) or [m, k/2] bytes (fp4), dense, 16-byte aligned
 *   scales   tf_scale_bytes(format, m, k, layout) bytes; with TF_SCALES_SWIZZLED the padding is zeroed by the call
 *   k        a multiple of 32
 * nvfp4: global_scale points to ONE f32 on the device holding amax(|x|)/2688 (tf_nvfp4_global_scale computes it). */
TF_API tf_status tf_quantize_mxfp8(const void* x, int64_t m, int64_t k, int64_t ldx, void* codes, void* scales, int32_t layout, void* stream);
TF_API tf_status tf_quantize_mxfp4(const void* x, int64_t m, int64_t k, int64_t ldx, void* codes, void* scales, int32_t layout, void* stream);
TF_API tf_status tf_quantize_nvfp4(const void* x, int64_t m, int64_t k, int64_t ldx, void* codes, void* scales, int32_t layout,
                            const float* global_scale, void* stream);
/* Same, but the global scale is derived inside the kernel from a device f32 holding amax(|x|) (as produced by the out_amax
 * argument of tf_residual_add_rmsnorm / tf_gemm_blockscaled): global_scale_out[0] = amax[0] / 2688.0f is also written for
 * the GEMM that consumes the result. Saves the separate amax pass over x. */
TF_API tf_status tf_quantize_nvfp4_from_amax(const void* x, int64_t m, int64_t k, int64_t ldx, void* codes, void* scales, int32_t layout,
                                      const float* amax, float* global_scale_out, void* stream);
/* global_scale_out[0] = max|x| / 2688.0f (one IEEE division), computed on the device in stream order. */
TF_API tf_status tf_nvfp4_global_scale(const void* x, int64_t m, int64_t k, int64_t ldx, float* global_scale_out, void* stream);

/* Plain <-> swizzled scale bytes ([rows, cols] scale entries). The swizzled buffer's padding is zeroed. */
TF_API tf_status tf_swizzle_scales(const void* plain, int64_t rows, int64_t cols, void* swizzled, void* stream);
TF_API tf_status tf_unswizzle_scales(const void* swizzled, int64_t rows, int64_t cols, void* plain, void* stream);

/* residual_add_rmsnorm (README.md:53-63 of the reference; its Triton lowering python/tests/golden/residual_add_rmsnorm.py):
 *   r = residual + f32(x); residual <- r; out = bf16(r * rsqrt(mean(r*r) + eps) * f32(w)), mean = sum * f32(1/D).
 *   x bf16 [m, d]; residual f32 [m, d] (updated in place); w bf16 [d]; all dense and 16-byte aligned; d % 8 == 0.
 *   out      bf16 [m, d] or NULL when only the quantized output is wanted
 *   q_format -1 for none, else a TF_FMT_*: the bf16 result is also quantized along d (d % 32 == 0) into q_codes/q_scales
 *            exactly as tf_quantize_* would quantize `out`; nvfp4 needs q_global_scale (given, on the device).
 *   out_amax NULL, or a device f32 the caller zeroed: max(|out|) is combined into it with an atomic max (the f32 bit
 *            pattern of a non-negative value orders like an unsigned integer). */
TF_API tf_status tf_residual_add_rmsnorm(const void* x, void* residual, const void* w, void* out, int64_t m, int64_t d, float eps,
                                  int32_t q_format, void* q_codes, void* q_scales, int32_t q_layout, const float* q_global_scale,
                                  float* out_amax, void* stream);

/* Few rows (m <= the number of SMs, e.g. a decode step): residual_add_rmsnorm AND the BlockScaled quantization of its result in one
 * launch, one CTA per row; what the reference's graph does with a kernel launch (python/src/tilefish/_cuda.py:356-458) plus a cast
 * it types but does not run (python/src/tilefish/ops.py:556-559). Same arithmetic, order and roundings as tf_residual_add_rmsnorm
 * followed by tf_quantize_*: the bytes are identical.
 *   x         bf16 [m, d], or NULL when the input is given as split-K partial sums:
 *   partials / splits   the f32 planes [splits][m][d] tf_gemm_blockscaled_partials left in its workspace: summed in split order,
 *             multiplied by a_global_scale[a_global_scale_rows ? row / a_global_scale_rows : 0] * b_global_scale[0] (both NULL: 1)
 *             and rounded to bf16, exactly as that GEMM's own reduction pass would have stored them
 *   residual f32 [m, d] (updated in place), w bf16 [d], out bf16 [m, d] or NULL; d a multiple of 32
 *   q_format  TF_FMT_*; q_codes, q_scales (swizzled) as tf_quantize_* writes them, EXCEPT that padding bytes of q_scales are not
 *             touched: zero the buffer once when it is allocated
 *   nvfp4: the tensor-wide scale amax / 2688 is formed inside the launch (the CTAs meet once at a bounded barrier; a timeout is
 *             reported by tf_device_status) and stored to q_global_scale[0]; sync points at two 32-bit words (8-byte aligned) that
 *             the caller zeroes before EVERY call (amax bits, arrivals). Other formats: q_global_scale and sync may be NULL. */
TF_API tf_status tf_rmsnorm_quantize_rows(const void* x, const float* partials, int32_t splits, const float* a_global_scale,
                                          const float* b_global_scale, int64_t a_global_scale_rows, void* residual, const void* w, void* out,
                                          int64_t m, int64_t d, float eps, int32_t q_format, void* q_codes, void* q_scales,
                                          float* q_global_scale, uint32_t* sync, void* stream);

/* SiLU gate (README.md:83-84; the fused region of python/src/tilefish/_fusion.py):
 *   out[m, j] = bf16( silu(f32(gate[m, j])) * f32(up[m, j]) ), silu(x) = x * (1 / (1 + exp(-x))).
 *   gate, up bf16 [m, f] with row strides ldg, ldu (the column halves of a [m, 2f] tensor t are gate = t, up = t + f,
 *   ldg = ldu = 2f); out bf16 [m, f] with row stride ldo; f and the strides are multiples of 8. */
TF_API tf_status tf_silu_gate(const void* gate, const void* up, int64_t m, int64_t f, int64_t ldg, int64_t ldu, void* out, int64_t ldo,
                       void* stream);

/* Block-scaled GEMM on tcgen05 tensor cores: out[M,N] = bf16( sum_k deq(a)[m,k] * deq(b)[n,k] ), f32 accumulate.
 * Replaces the pinned cublasLtMatmul of `@tilefish.library("gemm", acc=f32)` (python/src/tilefish/_library.py:9-16) for
 * BlockScaled operands, which the reference cannot run.
 *   a_codes [m, k] (or k/2) bytes, b_codes [n_rows, k] bytes, dense, 16-byte aligned, k % 32 == 0
 *   a_scales, b_scales   SWIZZLED scale bytes of the two operands
 *   a_global_scale, b_global_scale   device f32 (nvfp4) or NULL
 *   out      bf16 [m, n] row stride ldo (ldo % 8 == 0)
 *   epilogue TF_EPI_*: with TF_EPI_SILU_GATE b has 2n rows (n % 128 == 0); with TF_EPI_RESIDUAL epilogue_arg is the f32
 *            residual [m, n] (dense)
 *   out_amax NULL, or a device f32 the caller zeroed: max(|out|) is combined into it with an atomic max
 *   q_codes, q_scales   NULL, or (MX formats, n % 32 == 0, not with TF_EPI_RESIDUAL) the output is ALSO quantized, in the operands'
 *            format, exactly as tf_quantize_* would quantize `out` (every epilogue thread holds whole 32-element blocks):
 *            codes [m, n] or [m, n/2], swizzled scales. `out` may then be NULL (the bf16 copy is not written)
 *   a_global_scale_rows   0: a has one global scale. Else (a multiple of 128) a_global_scale is an array and rows
 *            [i * a_global_scale_rows, (i+1) * a_global_scale_rows) of a use entry i: row blocks that were quantized separately
 *            (each with the global scale of its own amax), e.g. activation rows gathered from the ranks of a tensor-parallel group
 *   workspace / workspace_bytes   at least tf_gemm_workspace_bytes(...) bytes, 256-byte aligned (may be NULL when 0) */
TF_API int64_t tf_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int32_t format, int32_t epilogue);
TF_API tf_status tf_gemm_blockscaled(const void* a_codes, const void* a_scales, const float* a_global_scale, const void* b_codes,
                              const void* b_scales, const float* b_global_scale, void* out, int64_t ldo, int64_t m, int64_t n,
                              int64_t k, int32_t format, int32_t epilogue, void* epilogue_arg, float* out_amax, void* q_codes, void* q_scales,
                              int64_t a_global_scale_rows, void* workspace, int64_t workspace_bytes, void* stream);

/* The same GEMM for callers that cannot hand over a workspace. (No counterpart in the reference.)
 *
 * Some hosts of this library run where device memory cannot be allocated at call time: a serving process whose memory pool
 * was sized and frozen at start-up, a plugin that is only given the tensors of its operator, a real-time loop that may not
 * enter the allocator. tf_gemm_blockscaled needs a workspace for small-M problems (it cuts K into ranges and sums the
 * partial products in a second pass); this variant takes that workspace from a fixed 8 MiB array inside the library's
 * device image instead (tf_gemm_static_scratch_bytes() returns the size). Every GPU that loads the library carries the
 * array until the process exits.
 *   - A problem whose workspace (tf_gemm_workspace_bytes) exceeds the array is refused with TF_ERR_WORKSPACE before anything
 *     is launched; problems that need no workspace run exactly as tf_gemm_blockscaled does.
 *   - The first call on a device looks the array's address up (once per device, with that device current). Make that first
 *     call before starting any stream capture.
 *   - The call allocates nothing: no cudaMalloc / cudaFree, no allocating library routine.
 *   - All calls on a device share the one array and it keeps the previous call's contents. Nothing in it has to start at
 *     zero (every partial sum that is read was written by the same call first), but two calls that run at the same time on
 *     one GPU (two streams, two threads) overwrite each other's partial sums: order them on one stream.
 *   - The looked-up address is cached per device ordinal for the life of the process: it does not survive a cudaDeviceReset.
 * Arguments as tf_gemm_blockscaled without workspace / workspace_bytes, and without q_codes, q_scales and a_global_scale_rows (passed
 * on as NULL / NULL / 0): no fused quantized copy of the output, one global scale for the whole of `a`. */
TF_API int64_t tf_gemm_static_scratch_bytes(void);
TF_API tf_status tf_gemm_blockscaled_static(const void* a_codes, const void* a_scales, const float* a_global_scale, const void* b_codes,
                                     const void* b_scales, const float* b_global_scale, void* out, int64_t ldo, int64_t m, int64_t n,
                                     int64_t k, int32_t format, int32_t epilogue, void* epilogue_arg, float* out_amax, void* stream);

/* The first pass of a split-K problem only (epilogue TF_EPI_NONE): the f32 partial sums stay in the workspace as `*splits` planes
 * [splits][m][n] for a consumer that sums them itself (tf_rmsnorm_quantize_rows: the few-rows step between two blocks, where a separate
 * reduction launch costs as much as the arithmetic). No counterpart in the reference. Shapes that are not split along K
 * (tf_gemm_splits == 1) are refused with TF_ERR_UNSUPPORTED. Other arguments as tf_gemm_blockscaled (one global scale for `a`). */
TF_API int32_t tf_gemm_splits(int64_t m, int64_t n, int64_t k, int32_t format, int32_t epilogue);
TF_API tf_status tf_gemm_blockscaled_partials(const void* a_codes, const void* a_scales, const float* a_global_scale, const void* b_codes,
                                              const void* b_scales, const float* b_global_scale, int64_t m, int64_t n, int64_t k, int32_t format,
                                              void* workspace, int64_t workspace_bytes, int32_t* splits, void* stream);

/* The GEMM with a scattered output: the tensor-parallel second GEMM (w_d split along K) whose epilogue delivers each row block of
 * its partial result straight to the rank that will sum it, so that no separate kernel has to pull the partial results across
 * NVLink afterwards. No counterpart in the reference (it has no cross-device exchange).
 *   out_ptrs[owners]   device addresses valid ON THIS GPU (peer-mapped, or local for this rank's own block): rows
 *            [i * rows_per_owner, (i + 1) * rows_per_owner) of the result are written to out_ptrs[i] as a bf16 [rows_per_owner, n]
 *            matrix with row stride ldo, by plain 16-byte stores from the epilogue (no TMA, nothing waits on a peer). The caller
 *            orders the reads behind the kernel (tf_tp_norm_exchange's first barrier does).
 *   owners 1..8; rows_per_owner a multiple of 128; m == owners * rows_per_owner
 * No epilogue operator, no amax, no quantized copy. Shapes that tf_gemm_blockscaled would split along K
 * (tf_gemm_workspace_bytes > 0: few rows) are refused with TF_ERR_UNSUPPORTED: use tf_gemm_blockscaled and let the consumer pull.
 * Other arguments as tf_gemm_blockscaled. */
TF_API tf_status tf_gemm_blockscaled_scatter(const void* a_codes, const void* a_scales, const float* a_global_scale, const void* b_codes,
                                      const void* b_scales, const float* b_global_scale, const uint64_t* out_ptrs, int32_t owners,
                                      int64_t rows_per_owner, int64_t ldo, int64_t m, int64_t n, int64_t k, int32_t format,
                                      int64_t a_global_scale_rows, void* stream);

/* In-place bf16 sum all-reduce over the ranks of a tensor-parallel group, one call (one kernel) per rank, each on its own GPU.
 * Replaces the cross-rank sum the reference leaves to the caller's framework; the MLP path's only exchange: partial results of
 * the second GEMM (w_d split along K) summed over the ranks.
 *   buffer_ptrs[world]  device addresses, valid ON THIS GPU, of every rank's data buffer (peer-mapped; entry `rank` is this
 *            rank's own). All ranks use the same offset and count: symmetric memory.
 *   state_ptrs[world]   the same for every rank's 128-byte state block, zeroed once by the host before the first call and
 *            never touched by it again. Calls that may run at the same time on one GPU need separate state blocks.
 *   multicast_ptr   0, or the address of a multicast (NVSwitch) mapping of the data buffers. With 0: plain peer loads,
 *            reduce-scatter then all-gather. Else each rank sums its slice over peer loads and multimem.st writes the result to all
 *            ranks, or, with
 *   reduce_in_switch   nonzero, the switch itself sums (multimem.ld_reduce): half the bytes received per GPU, but the switch's
 *            bf16 result is only within one bf16 step of the exact sum, not always the nearest value. The other two paths sum
 *            in f32 in rank order and round to nearest even once.
 *   offset_bytes (multiple of 16), count (bf16 elements, multiple of 8 * world)   the range of the buffers that is summed
 *   num_ctas   CTAs of the kernel (1..148); they must all be resident at once, so leave that many SMs to it when other
 *            kernels run beside it (tf_set_sm_margin)
 * Every rank must make the same sequence of calls on a state block. The
 * waits on the peers are bounded (two seconds, or the number of nanoseconds the host stored in the 64-bit word at byte 96 of this
 * rank's state block): a rank that never arrives makes the kernel return with a nonzero error word (the 64-bit word at byte 88 of
 * the state block: 1 = this rank's own CTAs never all met, 2 = a peer never arrived; the state blocks must then be zeroed again on
 * all ranks). */
TF_API tf_status tf_allreduce_bf16(const uint64_t* buffer_ptrs, const uint64_t* state_ptrs, uint64_t multicast_ptr, int32_t reduce_in_switch,
                                   int32_t rank, int32_t world, int64_t offset_bytes, int64_t count, int32_t num_ctas, void* stream);

/* The tensor-parallel exchange between two blocks of the MLP stack fused with the next block's residual_add_rmsnorm and the
 * quantization of its output; one call (one kernel) per rank. With the normalisation sharded by rows, rank r sums ITS rows
 * of the second GEMM's partial results over the ranks (f32 over peer loads in rank order, rounded to bf16 once; or in the
 * switch with reduce_in_switch), adds them into its rows of the f32 residual stream, normalises them exactly as
 * tf_residual_add_rmsnorm does, quantizes them exactly as tf_quantize_* does (nvfp4: with the global scale of the row
 * block's own amax) and writes codes, swizzled scales and the global scale into EVERY rank's buffers, so that each rank
 * holds the quantized activation of all rows for its first GEMM (tf_gemm_blockscaled with a_global_scale_rows = rows / world).
 * No counterpart in the reference.
 *   buffer_ptrs / state_ptrs / multicast_ptr / reduce_in_switch / rank / world / num_ctas   as tf_allreduce_bf16 (world may be 1)
 *   partial_offset   byte offset, inside every rank's buffer, of the bf16 [rows_total, d] partial results
 *   codes_offset, scales_offset, gs_offset   byte offsets of the outputs: codes [rows_total, d] (e4m3) or [rows_total, d/2]
 *            (e2m1), swizzled scales of a [rows_total, d] tensor, f32 [world] global scales (nvfp4; 16-byte aligned)
 *   rows_total (a multiple of 128 * world), d (a multiple of 128)
 *   sum_peers   0: the partial region already holds complete values on this rank (the input of the first block).
 *            1: every rank's buffer holds that rank's partial results for all rows; this rank pulls its rows from all of them.
 *            2: this rank's OWN buffer holds every rank's partial results for this rank's rows, delivered there by
 *            tf_gemm_blockscaled_scatter: source rank s at rows [s * rows_total / world, ...) of the partial region. The sum
 *            reads local memory only (same order, same bytes as 1); not with reduce_in_switch.
 *   residual_rows   this rank's rows [rank * rows_total / world, ...) of the residual stream, f32, updated in place
 *   w bf16 [d]; h_scratch bf16 [rows_total / world, d] (scratch); amax one zeroed f32 (nvfp4) */
TF_API tf_status tf_tp_norm_exchange(const uint64_t* buffer_ptrs, const uint64_t* state_ptrs, uint64_t multicast_ptr, int32_t reduce_in_switch,
                                     int32_t rank, int32_t world, int64_t partial_offset, int64_t codes_offset, int64_t scales_offset,
                                     int64_t gs_offset, int64_t rows_total, int64_t d, int32_t sum_peers, void* residual_rows, const void* w,
                                     void* h_scratch, float* amax, float eps, int32_t q_format, int32_t num_ctas, void* stream);

/* ---- a native replay loop for exported plans ------------------------------------------------------------------------------------
 * The C counterpart of the reference's Rust host for this path (crates/tilefish/src/plan_run.rs:678 PlanRun, :1944 launch, :2097
 * capture; C ABI crates/tilefish-capi/include/tilefish.h): it reads the directory runtime.export() wrote (plan.json in the
 * reference's plan schema 1, docs/en/plan-schema-1.md, and this backend's manifest.json), then runs a bucket's steps with no
 * interpreter between the launches, or captures them into a CUDA graph.
 *   tf_plan_load         strict JSON; the plan's digest is recomputed and compared with `pin` (64 hex digits; NULL = the caller trusts
 *                        the directory) and with the file's own; the manifest's digest likewise; every step must name a manifest entry.
 *                        Needs no GPU.
 *   tf_plan_instantiate  the arena: `arena` (256-byte aligned, at least tf_plan_arena_bytes) or, with NULL, one cudaMalloc made here
 *                        (the only allocation of this API; freed by tf_plan_free). Nothing is allocated afterwards.
 *   tf_plan_bind         the caller's tensor for an external buffer, by the buffer's name in the plan ("x", "residual", "w_gu",
 *                        "w_gu__scales", "w_gu__global", "out0" ...). Pointers stay bound until rebound.
 *   tf_plan_find_bucket  the index of the bucket whose dimensions have exactly these values, or -1 (bucket semantics are exact).
 *   tf_plan_launch       resolves and checks every step of the bucket with the real addresses (bindings present, 16-byte alignment,
 *                        workspace large enough on this device) BEFORE the first launch, then enqueues the steps in order on `stream`.
 *   tf_plan_capture      the same checks, then the steps captured on `stream` (not the legacy default stream) into a CUDA graph that
 *                        the plan object owns; *graph_out is its index. The graph holds the addresses bound at capture time.
 *   tf_plan_replay       launches a captured graph on `stream`.
 * A plan object is used by one thread at a time. */
typedef struct tf_plan tf_plan;
TF_API tf_status tf_plan_load(const char* directory, const char* pin, tf_plan** out);
TF_API void tf_plan_free(tf_plan* plan);
TF_API const char* tf_plan_digest(const tf_plan* plan);
TF_API int64_t tf_plan_arena_bytes(const tf_plan* plan);
TF_API int32_t tf_plan_step_count(const tf_plan* plan, int32_t bucket);
TF_API int32_t tf_plan_find_bucket(const tf_plan* plan, const char* const* dim_names, const int64_t* values, int32_t n);
TF_API tf_status tf_plan_instantiate(tf_plan* plan, void* arena, int64_t arena_bytes);
TF_API tf_status tf_plan_bind(tf_plan* plan, const char* buffer, void* device_ptr);
TF_API tf_status tf_plan_launch(tf_plan* plan, int32_t bucket, void* stream);
TF_API tf_status tf_plan_capture(tf_plan* plan, int32_t bucket, void* stream, int32_t* graph_out);
TF_API tf_status tf_plan_replay(tf_plan* plan, int32_t graph, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TILEFISH_B200_H */
