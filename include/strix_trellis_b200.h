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

/* Decode-rate probe: the fused GEMV's inner loop (production decoder + the same mma) on tiles
 * of these weights held in shared memory, `warps_per_sm` warps per SM (4..32, a multiple of
 * four; the fused GEMV runs 16), `iterations` passes, on every SM; no global traffic, barriers
 * or fold.  *clocks_per_tile = SM clocks per 16x16 tile per SM
 * sub-partition: the instruction-issue cost of the decoder and therefore the ceiling of every
 * kernel built on it (bytes/s <= 4 * SMs * clock / clocks_per_tile * bytes per tile).
 * Synchronous; allocates two small buffers.  Counterpart of the reference's decode
 * microbenchmark (src/microbench.hip modes 0-4, bench/README.md:24-31). */
strix_status strix_b200_decode_rate(strix_context context, strix_weights weights, uint32_t iterations,
                                    uint32_t warps_per_sm, double *clocks_per_tile,
                                    const strix_stream *stream);

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
 * drain at exit, bit 3 tensor pipeline, bit 4 split-K fold, bit 5 a peer exchange that never
 * completed); results of that launch are invalid,
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

/* The combine above with a per-token validity mask: a token whose row_valid entry is zero gets
 * a NaN row (the reference's answer to an invalid device route, src/tp_moe.hip:131-138).
 * row_valid may be NULL (all rows valid). */
strix_status strix_b200_moe_combine_rows(strix_context context, const float *rows, const float *scores,
                                         const int32_t *row_valid, uint32_t tokens, uint32_t top_k,
                                         uint32_t width, float *y, uint64_t y_stride, float alpha,
                                         float beta, const strix_stream *stream);

/* ---- expert parallelism ------------------------------------------------------------------
 * A device-routed plan's bank as a window of the router's id space: route id g is bank entry
 * g - first_expert when that is inside the bank, lives on another rank when g < experts_total
 * (its slot runs nothing here and does not invalidate the row), and invalidates the row
 * otherwise.  After this call strix_tp_moe_plan_submit yields this rank's contribution (the
 * sum over its own experts' slots, the reference's per-rank semantics,
 * include/strix_trellis.h:215-216); the default window is the whole bank.  Every rank applies
 * the same row rules (ids in range and distinct, scores finite and non-negative), so all ranks
 * agree on which rows are valid.  The call also re-plans how finely the grouped launches cut K,
 * for the routes this rank expects to own (all routes x bank / experts_total), within the
 * scratch the plan was created with.  No counterpart as an entry point in the reference. */
strix_status strix_b200_moe_plan_set_window(strix_tp_moe_plan plan, uint32_t first_expert,
                                            uint32_t experts_total);
/* Routing, gate/up, SwiGLU and down projections of the routes this rank owns, without the
 * combine: the per-route output rows stay in plan memory for an exchange to carry home. */
strix_status strix_b200_moe_plan_projections(strix_tp_moe_plan plan);
/* Where those rows are: each = F32 [tokens * top_k][model] (rows of routes owned elsewhere are
 * not written), row_valid = int32 [tokens] (device-routed plans; NULL otherwise). */
strix_status strix_b200_moe_plan_rows(strix_tp_moe_plan plan, const float **each,
                                      const int32_t **row_valid);

/* Diagnostics: the gate and up projection rows that strix_tp_moe_plan_gate_up left in plan
 * memory, F32 [tokens * top_k][intermediate] each, before SwiGLU combined them into the
 * hidden rows at the start of the caller's workspace. */
strix_status strix_b200_moe_plan_gate_up_rows(strix_tp_moe_plan plan, const float **gate,
                                              const float **up);

/* ---- exchange between the ranks of one node through peer memory over NVLink -----------------
 * The shard-boundary steps of the tensor- and expert-parallel layers as single kernels that
 * store straight into the other ranks' memory: no library collective, no host
 * synchronisation, capturable into a CUDA graph.  The reference has no inter-rank
 * communication (README.md:773); it only fixes the arithmetic of these steps
 * (docs/TP_RANK.md:150-156).
 *
 * Every rank creates an ARENA and publishes its 64-byte handle to the other ranks (any host
 * channel); a GROUP maps all arenas of the node.  The first STRIX_B200_PEER_CONTROL_BYTES of
 * an arena belong to the library; the caller assigns the rest as REGIONS (byte offsets,
 * multiples of 256) to the exchanges it runs.  A region holds two copies of an exchange's
 * payload, used alternately, so a layer may run back to back.  All ranks must issue the same
 * sequence of exchanges on a group.  A rank that never shows up makes the others give up after
 * several seconds: bit 5 of the status word (strix_b200_device_status) is set and the result of
 * that exchange is invalid.  `local_count` consecutive ranks starting at `first_rank` may live
 * in this process on this device: per-rank arguments are then arrays of `local_count` entries
 * (one entry in production). */
#define STRIX_B200_PEER_MAX_RANKS 8
#define STRIX_B200_PEER_HANDLE_BYTES 64
#define STRIX_B200_PEER_CONTROL_BYTES UINT64_C(2304)
typedef struct strix_b200_peer_group_impl *strix_b200_peer_group;

strix_status strix_b200_peer_arena_create(strix_context context, uint64_t bytes, void **arena,
                                          unsigned char *handle /* [64] */);
strix_status strix_b200_peer_arena_destroy(strix_context context, void *arena);
/* handles: world x 64 bytes in rank order (entries of local ranks are ignored; may be NULL
 * when every rank is local). */
strix_status strix_b200_peer_group_create(strix_context context, void *const *local_arenas,
                                          uint32_t local_count, uint32_t first_rank,
                                          uint64_t arena_bytes, const unsigned char *handles,
                                          uint32_t world, strix_b200_peer_group *out);
strix_status strix_b200_peer_group_destroy(strix_b200_peer_group group);
/* How many times a wait for a peer polls before it gives up, sets bit 5 of the device status
 * word and lets its kernel return (default 2^23, several seconds).  After a wait has run out the
 * group's exchange numbering no longer matches its peers': destroy it and make a new one. */
strix_status strix_b200_peer_group_set_wait_polls(strix_b200_peer_group group, uint32_t polls);

/* rows[i] (count floats, count even, 8-byte aligned) of every rank is replaced by the sum over
 * ranks, added in ascending rank order from +0: identical bits on every rank.  Meant for the
 * few rows a decode step produces: every value travels with its own arrival mark, which
 * doubles the bytes and removes a round trip.  Region size: 2 * world * count * 8 bytes. */
strix_status strix_b200_peer_sum(strix_b200_peer_group group, float *const *rows, uint64_t count,
                                 uint64_t region, const strix_stream *stream);

/* Every rank's block into one matrix on every rank; up to three matrices of 32-bit words
 * travel in one exchange.  Rank r contributes rows[r] x width[r] words (contiguous) placed at
 * (row_at[r], col_at[r]) of the total_rows x total_cols result (total_rows = max row_at+rows).
 * result[i] != NULL receives a private contiguous copy; with NULL the result is read in the
 * arena at region + parity * total_rows * total_cols * 4.  Region size per matrix:
 * 2 * total_rows * total_cols * 4 bytes. */
/* flags: with STRIX_B200_PEER_GATHER_TAGGED every word travels with the exchange number beside
 * it (8 bytes per word, no fence and no flag step: the lowest latency).  Then every matrix needs
 * a result pointer, even widths, column offsets and total_cols, and a region of
 * 2 * total_rows * total_cols * 8 bytes. */
#define STRIX_B200_PEER_GATHER_TAGGED 1u
typedef struct strix_b200_peer_matrix {
    const void *block[STRIX_B200_PEER_MAX_RANKS];  /* per local rank */
    void *result[STRIX_B200_PEER_MAX_RANKS];       /* per local rank, or NULL */
    uint32_t width[STRIX_B200_PEER_MAX_RANKS];     /* per rank, 32-bit words */
    uint32_t col_at[STRIX_B200_PEER_MAX_RANKS];    /* per rank */
    uint64_t total_cols;
    uint64_t region;
} strix_b200_peer_matrix;
typedef struct strix_b200_peer_gather_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t matrices; /* 1..3 */
    uint32_t flags;    /* zero or STRIX_B200_PEER_GATHER_TAGGED */
    uint32_t rows[STRIX_B200_PEER_MAX_RANKS];   /* per rank */
    uint32_t row_at[STRIX_B200_PEER_MAX_RANKS]; /* per rank */
    strix_b200_peer_matrix matrix[3];
    uint64_t reserved[2];
} strix_b200_peer_gather_desc;
strix_status strix_b200_peer_gather(strix_b200_peer_group group, const strix_b200_peer_gather_desc *desc,
                                    const strix_stream *stream);

/* Routed rows back to the home rank of their token.  Tokens are laid out rank-major (token t
 * lives on rank t / tokens_per_rank).  A rank stores the row of route (t, s) when row_valid[t]
 * is non-zero and ids[t, s] lies in its window; it lands at row (t % tokens_per_rank) * top_k + s
 * of the home rank's region (2 * tokens_per_rank * top_k * width * 4 bytes, parity as above). */
typedef struct strix_b200_peer_return_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    const float *each[STRIX_B200_PEER_MAX_RANKS];       /* per local rank: [tokens * top_k][width] */
    const uint32_t *ids[STRIX_B200_PEER_MAX_RANKS];     /* per local rank: [tokens][top_k] */
    const int32_t *row_valid[STRIX_B200_PEER_MAX_RANKS];/* per local rank: [tokens] */
    uint32_t first_expert[STRIX_B200_PEER_MAX_RANKS];   /* per local rank */
    uint32_t experts[STRIX_B200_PEER_MAX_RANKS];        /* per local rank */
    uint32_t tokens;
    uint32_t tokens_per_rank;
    uint32_t top_k;
    uint32_t flags; /* zero */
    uint64_t width; /* floats per row, multiple of 4 */
    uint64_t region;
    uint64_t reserved[2];
} strix_b200_peer_return_desc;
strix_status strix_b200_peer_return_routes(strix_b200_peer_group group,
                                           const strix_b200_peer_return_desc *desc,
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
 * NULL/0; tensors are still the caller's.  Limit: the array holds one partial plane per
 * persistent CTA and activation row, enough for eight rows on a device of up to 256 SMs; a
 * launch that would need more returns STRIX_ERROR_INSUFFICIENT_BUFFER.
 * The first call on a device looks up the array's device address (one runtime query);
 * make that first call before starting any stream capture.  All calls on a device share
 * the one array, so two calls that can overlap on the GPU (different streams without an
 * ordering between them) race; keep them in one stream or order them with events. */
#define STRIX_B200_NOALLOC_SCRATCH_BYTES UINT64_C(1048576)
strix_status strix_b200_gemv_noalloc(strix_context context, const strix_matmul_desc *desc,
                                     const strix_stream *stream);

#ifdef __cplusplus
}
#endif
#endif /* STRIX_TRELLIS_B200_H */
