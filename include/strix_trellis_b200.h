/* strix_trellis_b200.h -- additions of the B200 runtime that the reference ABI has no
 * name for.  None of them changes the behaviour of an entry point declared in
 * strix_trellis.h.  Most are the stage probes that the reference keeps inside its GPU
 * harness (tests/gpu_runtime.hip: isolated Q decode, input checkpoints,
 * output_transform on a known core, docs/GPU_TESTS.md:97-109); here they are callable
 * through the C ABI so that parity tests in any language can use them.
 */
#ifndef STRIX_TRELLIS_B200_H
#define STRIX_TRELLIS_B200_H

#include "strix_trellis.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Decode prepared weights to Q [I][N] binary16 (row-major, I rows) with the
 * production decoder device function.  Stands in for the reference harness's
 * isolated Q probe (tests/gpu_runtime.hip, docs/GPU_TESTS.md:97-100) and computes
 * what python/strix_trellis/codec.py:165-173 (dequantize_rotated) computes.
 * out_bytes >= I*N*2; device memory of the context's device. */
strix_status strix_b200_dequantize(strix_context context, strix_weights weights, void *out_f16,
                                   uint64_t out_bytes, const strix_stream *stream);

/* Input checkpoints of the staged contract for x [rows][I] F32 (contiguous):
 * scaled_f16 = RN16(RN32(x*suh)), hadamard_f32 = H128(scaled), core_f16 = RN16(hadamard)
 * (python/strix_trellis/linear.py:111-124; reference kernel src/transforms.hpp:8-26).
 * Any output pointer may be NULL.  Each non-NULL output holds rows*I elements. */
strix_status strix_b200_input_stages(strix_context context, strix_weights weights, const float *x,
                                     uint32_t rows, void *scaled_f16, float *hadamard_f32,
                                     void *core_f16, const strix_stream *stream);

/* Output stages on a caller-supplied core [splits][rows][N] F32: planes summed in
 * ascending order from +0, H128, svh, bias, alpha, beta (linear.py:146-163; reference
 * kernel src/transforms.hpp:28-52).  y is [rows][N] contiguous. */
strix_status strix_b200_output_stages(strix_context context, strix_weights weights,
                                      const float *core, uint32_t splits, uint32_t rows, float alpha,
                                      float beta, float *y, const strix_stream *stream);

/* Core product in the CPU contract's accumulation order (ascending input index, one
 * fused multiply-add per term; bit-identical to linear.py:127-143 because products of
 * two binary16 values are exact in binary32).  core_f16 [rows][I], core_out [rows][N],
 * rows <= 64.  A parity instrument: slow, not a production path. */
strix_status strix_b200_core_exact(strix_context context, strix_weights weights, const void *core_f16,
                                   uint32_t rows, float *core_out, const strix_stream *stream);

/* K partitions the fused GEMV uses for `rows` rows of these weights (fixes the
 * association of the partial sums; counterpart of linear_split_count,
 * src/backend.hip:22-45). */
strix_status strix_b200_gemv_splits(strix_context context, strix_weights weights, uint32_t rows,
                                    uint32_t *out_splits);

/* Work split of the fused GEMV for a layer of `inputs` x `outputs` on `grid` persistent CTAs
 * (the kernel uses grid = min(SM count, units)): out[0], out[1] = the unit range CTA `cta`
 * streams (a unit = one 128-column block x 128 inputs, column block major); out[2], out[3] =
 * the first and last CTA that contribute to `column_block`.  A block with out[2] < out[3] is
 * folded by CTA out[2], which waits for the partial planes of the CTAs above it.  Pure host
 * arithmetic (no context, no device): lets the split and the direction of those waits be
 * checked on a machine without a GPU.  No counterpart in the reference. */
strix_status strix_b200_gemv_partition(uint64_t inputs, uint64_t outputs, uint32_t grid, uint32_t cta,
                                       uint64_t column_block, uint64_t out[4]);

/* Reads and clears the context's device status word.  Non-zero means that a bounded
 * wait inside a kernel gave up (bit 0 weight ring full-wait, bit 1 empty-wait, bit 2
 * drain at exit, bit 3 tensor pipeline, bit 4 split-K fold); results of that launch are invalid,
 * and after bit 4 the plan whose launch it was should be recreated (its fold scratch may hold
 * words of the abandoned launch; direct strix_gemv calls reset their scratch on every call).
 * Synchronises the device.  No counterpart in the reference (its kernels never wait). */
strix_status strix_b200_device_status(strix_context context, uint32_t *out_bits);

/* Turns programmatic dependent launch of this library's kernels on (default) or off.
 * With it, a kernel starts streaming its (immutable) weights while the previous
 * kernel of the stream drains, and waits for that kernel before it reads activations
 * or writes anything.  No counterpart in the reference. */
strix_status strix_b200_set_programmatic_launch(strix_context context, uint32_t enabled);

/* Routed-expert combine at a token's home rank, for callers that run the expert projections
 * elsewhere (expert parallelism): y[t] = alpha * sum over slots s ascending, from +0, of
 * RN32(scores[t,s] * rows[t,s,:]) + beta * y[t]; a score of exactly zero skips its slot
 * (the combine of strix_tp_moe_plan_submit, reference src/tp_moe.hip:112-164, on its own).
 * rows: F32 [tokens, top_k, width] contiguous, scores: F32 [tokens, top_k], y: F32 rows
 * y_stride elements apart; all device memory of the context's device.  beta == 0 never
 * reads y.  While `stream` is being captured into a graph the pointers are not inspected
 * (the driver queries that do it would invalidate the capture).  No counterpart as a
 * separate entry point in the reference. */
strix_status strix_b200_moe_combine(strix_context context, const float *rows, const float *scores,
                                    uint32_t tokens, uint32_t top_k, uint32_t width, float *y,
                                    uint64_t y_stride, float alpha, float beta,
                                    const strix_stream *stream);

/* strix_gemv for callers that may not allocate.  It has no counterpart in the reference.
 *
 * Some engines hand every byte of device memory to their own arena when they start and
 * never call the CUDA allocator again: a cudaMalloc in the middle of a decode loop
 * serialises the whole device, and with the arena holding everything it would simply
 * fail.  Such a caller has nowhere to take the GEMV's split-K scratch from.  This entry
 * point needs none: its partial planes sit in a fixed array of
 * STRIX_B200_NOALLOC_SCRATCH_BYTES inside the library image (every GPU that loads the
 * library holds that array until the process exits).  It calls no allocating routine.
 *
 * Same operator and same results as strix_gemv (rows 0..8); desc->workspace must be
 * NULL/0; tensors are still the caller's.  Limits: outputs <= STRIX_B200_NOALLOC_MAX_OUTPUTS
 * and at most 192 SMs; anything larger returns STRIX_ERROR_INSUFFICIENT_BUFFER.
 * The first call on a device looks up the array's device address (one runtime query);
 * make that first call before starting any stream capture.  All calls on a device share
 * the one array, so two calls that can overlap on the GPU (different streams without an
 * ordering between them) race; keep them in one stream or order them with events. */
#define STRIX_B200_NOALLOC_MAX_OUTPUTS UINT64_C(524288)
#define STRIX_B200_NOALLOC_SCRATCH_BYTES UINT64_C(1589248)
strix_status strix_b200_gemv_noalloc(strix_context context, const strix_matmul_desc *desc,
                                     const strix_stream *stream);

#ifdef __cplusplus
}
#endif
#endif /* STRIX_TRELLIS_B200_H */
