/* strix_trellis.h -- C ABI of the B200 (sm_100a) EXL3 trellis linear-layer runtime.
 *
 * This header declares, symbol for symbol and field for field, the operator surface
 * of the reference project's include/strix_trellis.h (ABI version 1), so that an
 * engine written against that header links against this library unchanged.  Each
 * declaration names the reference line range it stands in for.  Behavioural
 * differences of the B200 implementation are listed once, here:
 *
 *   - strix_stream::hip_stream carries a cudaStream_t (the field keeps its name).
 *   - strix_context_create admits devices of compute capability 10.x.
 *   - Geometry is not whitelisted: every entry point accepts any input/output size
 *     that is a positive multiple of 128 and integer rates 1..8.  The routed-expert
 *     plans take the top-k from route_ids_count / rows (1..16), rows up to
 *     STRIX_B200_MOE_MAX_ROWS and banks up to STRIX_B200_MOE_MAX_BANK experts.
 *   - The prepared weight layout is private (the reference says so too, :111-112):
 *     preparation regroups tiles per 128 output columns once, on the device.
 *   - Entry points that only exist to select between gfx1151 schedules of the SAME
 *     arithmetic (_tiled, _splitk, _r1, split3 MoE) accept their arguments, validate
 *     them and run this library's one schedule; A8R (different arithmetic, off by
 *     default in the reference) returns STRIX_ERROR_NOT_IMPLEMENTED.
 *
 * Conventions (reference :11-14): descriptors are zero-initialised, then struct_size
 * and abi_version are set; reserved fields stay zero; dimensions and strides count
 * elements, buffer sizes and transport offsets count bytes; no ownership moves.
 */
#ifndef STRIX_TRELLIS_H
#define STRIX_TRELLIS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- versions and constants (reference :15-23) ------------------------------- */
#define STRIX_TRELLIS_ABI_VERSION UINT32_C(1)
#define STRIX_TRELLIS_VERSION_MAJOR 0
#define STRIX_TRELLIS_VERSION_MINOR 3
#define STRIX_TRELLIS_VERSION_PATCH 0
#define STRIX_TRELLIS_TRANSPORT_VERSION UINT32_C(1)
#define STRIX_TRELLIS_WORKSPACE_ALIGNMENT UINT32_C(256)
#define STRIX_EXL3_MARKER_3INST UINT32_C(0)
#define STRIX_EXL3_MARKER_MCG UINT32_C(0xCBAC1FED)
#define STRIX_EXL3_MARKER_MUL1 UINT32_C(0x83DCD12D)

/* ---- enumerations (reference :25-57) ----------------------------------------- */
typedef enum strix_status {
    STRIX_SUCCESS = 0,
    STRIX_ERROR_INVALID_ARGUMENT = 1,
    STRIX_ERROR_ABI_MISMATCH = 2,
    STRIX_ERROR_UNSUPPORTED_FORMAT = 3,
    STRIX_ERROR_UNSUPPORTED_DEVICE = 4,
    STRIX_ERROR_INSUFFICIENT_BUFFER = 5,
    STRIX_ERROR_OUT_OF_MEMORY = 6,
    STRIX_ERROR_BACKEND = 7,
    STRIX_ERROR_NOT_IMPLEMENTED = 8
} strix_status;

typedef enum strix_dtype {
    STRIX_DTYPE_INVALID = 0,
    STRIX_DTYPE_F16 = 1,  /* reserved and rejected by the reference (include/strix_trellis.h:62); honoured here */
    STRIX_DTYPE_BF16 = 2, /* for the tensors of gemv / gemm / linear plans / TP dense plans: widened exactly on load, */
                          /* rounded to nearest even on store; the arithmetic in between is the float32 contract */
    STRIX_DTYPE_F32 = 3
} strix_dtype;

typedef enum strix_transport_format {
    STRIX_TRANSPORT_INVALID = 0,
    STRIX_TRANSPORT_EXL3_CANONICAL = 1
} strix_transport_format;

typedef enum strix_codebook {
    STRIX_CODEBOOK_3INST = 0,
    STRIX_CODEBOOK_MCG = 1,
    STRIX_CODEBOOK_MUL1 = 2
} strix_codebook;

/* ---- host transport of one quantised linear (reference :59-109) ---------------- */
/* Blob metadata.  rows = N (outputs), columns = I (inputs), both multiples of 128.
 * bits_x2 is even, 2..16.  marker must equal the STRIX_EXL3_MARKER_* of codebook.
 * Payloads are little endian: trellis int16 [I/16][N/16][16*bits], suh f16 [I],
 * svh f16 [N], optional bias f32 [N] (offset and size both zero when absent). */
typedef struct strix_exl3_metadata_v1 {
    uint32_t struct_size;
    uint32_t transport_version;
    uint64_t rows;
    uint64_t columns;
    uint32_t bits_x2;
    strix_codebook codebook;
    uint32_t marker;
    uint32_t flags;
    uint64_t trellis_offset;
    uint64_t trellis_bytes;
    uint64_t suh_offset;
    uint64_t suh_bytes;
    uint64_t svh_offset;
    uint64_t svh_bytes;
    uint64_t bias_offset;
    uint64_t bias_bytes;
    uint64_t reserved[4];
} strix_exl3_metadata_v1;

/* One contiguous host blob plus its metadata. */
typedef struct strix_exl3_transport_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    strix_transport_format format;
    uint32_t transport_version;
    const void *data;
    uint64_t data_bytes;
    const void *metadata;
    uint64_t metadata_bytes;
    uint64_t rows;
    uint64_t columns;
    uint64_t reserved[4];
} strix_exl3_transport_desc;

/* A borrowed host byte range; any alignment; readable until prepare returns. */
typedef struct strix_host_region {
    const void *data;
    uint64_t bytes;
} strix_host_region;

/* The same transport as four independent host regions (no staging blob). */
typedef struct strix_exl3_parts_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t transport_version;
    uint32_t bits_x2;
    uint64_t rows;
    uint64_t columns;
    strix_codebook codebook;
    uint32_t marker;
    strix_host_region trellis;
    strix_host_region suh;
    strix_host_region svh;
    strix_host_region bias;
    uint64_t reserved[4];
} strix_exl3_parts_desc;

/* ---- opaque handles (reference :113-117) -------------------------------------- */
typedef struct strix_context_impl *strix_context;
typedef struct strix_weights_impl *strix_weights;
typedef struct strix_linear_plan_impl *strix_linear_plan;
typedef struct strix_tp_dense_plan_impl *strix_tp_dense_plan;
typedef struct strix_tp_moe_plan_impl *strix_tp_moe_plan;

#define STRIX_OPERATION_GEMV UINT32_C(0)
#define STRIX_OPERATION_GEMM UINT32_C(1)

/* ---- call descriptors (reference :120-181) ------------------------------------- */
/* A borrowed stream.  NULL selects the device's default stream. */
typedef struct strix_stream {
    uint32_t struct_size;
    uint32_t abi_version;
    void *hip_stream;
    uint64_t reserved[2];
} strix_stream;

typedef struct strix_context_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    int32_t device_ordinal;
    uint32_t flags;
    uint64_t reserved[4];
} strix_context_desc;

/* Row-major device tensor, F32, rank 1 or 2.  The buffer lives on the context's
 * device and outlives the stream work that uses it. */
typedef struct strix_tensor_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    void *data;
    uint64_t buffer_bytes;
    strix_dtype dtype;
    uint32_t rank;
    uint64_t shape[2];
    uint64_t strides[2];
    uint64_t reserved[4];
} strix_tensor_desc;

/* output = alpha * Linear(input) + beta * output, bias inside Linear.
 * GEMV: [I]->[N] or [B,I]->[B,N], B = 0..8.  GEMM: rank 2, any B.  B = 0 validates
 * and submits nothing.  beta == 0 never reads the old output.  A zero-initialised
 * alpha means zero.  Workspace: caller-owned, 256-byte aligned, size from
 * strix_matmul_workspace_bytes. */
typedef struct strix_matmul_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    strix_weights weights;
    strix_tensor_desc input;
    strix_tensor_desc output;
    float alpha;
    float beta;
    void *workspace;
    uint64_t workspace_bytes;
    uint64_t reserved[4];
} strix_matmul_desc;

/* Pre-routed experts: one ordinary matmul per group on disjoint slices, one shared
 * workspace (group workspaces must be NULL/0).  Routing is the caller's. */
typedef struct strix_grouped_moe_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    const strix_matmul_desc *groups;
    uint64_t group_count;
    void *workspace;
    uint64_t workspace_bytes;
    uint64_t reserved[4];
} strix_grouped_moe_desc;

/* ---- per-rank tensor-parallel surface (reference :183-262) --------------------- */
/* The reference's fixed limits, kept for source compatibility.  This library's
 * own limits are the STRIX_B200_* values below. */
#define STRIX_TP_TOP_K UINT32_C(6)
#define STRIX_TP_MAX_ROWS UINT32_C(8)
#define STRIX_TP_MAX_EXPERTS UINT32_C(48)
#define STRIX_TP_MAX_BANK_EXPERTS UINT32_C(256)
#define STRIX_B200_MOE_MAX_TOP_K UINT32_C(16)
#define STRIX_B200_MOE_MAX_ROWS UINT32_C(4096)
#define STRIX_B200_MOE_MAX_BANK UINT32_C(1024)

/* One routed expert: gate/up [N=inter, I=hidden], down [N=hidden, I=inter]. */
typedef struct strix_tp_expert_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t expert_id;
    uint32_t flags;
    strix_weights gate;
    strix_weights up;
    strix_weights down;
    uint64_t reserved[2];
} strix_tp_expert_desc;

/* Routed-expert block with HOST routes, copied at plan creation:
 *   hidden[r,s] = SiLU(gate_e(X[r])) * up_e(X[r])
 *   Y[r] = alpha * sum over slots s ascending from +0 of score[r,s]*down_e(hidden[r,s])
 *          + beta * Y[r]
 * route_ids / route_scores are row-major [R, top_k]; ids distinct within a row;
 * scores finite and non-negative, never renormalised; an exactly zero score skips
 * its slot.  Workspace: F32 [R, top_k, inter], 256-byte aligned.  The result is the
 * LOCAL contribution of this rank; reduction across ranks belongs to the caller. */
typedef struct strix_tp_moe_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    strix_tensor_desc input;
    strix_tensor_desc output;
    const strix_tp_expert_desc *experts;
    uint64_t expert_count;
    const uint32_t *route_ids;
    uint64_t route_ids_count;
    const float *route_scores;
    uint64_t route_scores_count;
    void *workspace;
    uint64_t workspace_bytes;
    float alpha;
    float beta;
    uint64_t reserved[4];
} strix_tp_moe_desc;

/* The same block with a persistent bank and DEVICE routes read at every submit.
 * experts[i].expert_id == i.  An id outside the bank, a duplicate within a row or a
 * negative / non-finite score makes that row's output NaN; nothing outside the bank
 * is ever read. */
typedef struct strix_tp_moe_device_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    strix_tensor_desc input;
    strix_tensor_desc output;
    const strix_tp_expert_desc *experts;
    uint64_t expert_count;
    const uint32_t *route_ids;
    uint64_t route_ids_bytes;
    const float *route_scores;
    uint64_t route_scores_bytes;
    void *workspace;
    uint64_t workspace_bytes;
    float alpha;
    float beta;
    uint64_t reserved[4];
} strix_tp_moe_device_desc;

/* ---- core entry points (reference :264-309) ------------------------------------ */
uint32_t strix_get_abi_version(void);
const char *strix_status_string(strix_status status);
/* Sets headers, nested F32 tensor headers, alpha = 1, beta = 0. */
void strix_matmul_desc_init(strix_matmul_desc *desc);
strix_status strix_context_create(const strix_context_desc *desc, strix_context *out);
strix_status strix_context_destroy(strix_context context);
/* Upload and regroup; the stream is synchronised before return, so host bytes may
 * be released immediately. */
strix_status strix_weights_prepare(strix_context context,
                                   const strix_exl3_transport_desc *transport,
                                   const strix_stream *stream, strix_weights *out);
strix_status strix_weights_prepare_parts(strix_context context,
                                         const strix_exl3_parts_desc *parts,
                                         const strix_stream *stream, strix_weights *out);
strix_status strix_weights_destroy(strix_weights weights);
#define STRIX_TRELLIS_HAS_WEIGHTS_SPAN 1
/* Read-only view of the single device allocation behind prepared weights. */
strix_status strix_weights_device_span(strix_weights weights, const void **data,
                                       uint64_t *bytes);
strix_status strix_matmul_workspace_bytes(strix_context context,
                                          const strix_matmul_desc *desc, uint64_t *out_bytes);
strix_status strix_gemv(strix_context context, const strix_matmul_desc *desc,
                        const strix_stream *stream);
strix_status strix_gemm(strix_context context, const strix_matmul_desc *desc,
                        const strix_stream *stream);
/* Frozen call: validate once, then submit with no allocation, copy, synchronisation
 * or pointer/stream query; submit may be captured into a CUDA graph. */
strix_status strix_linear_plan_create(strix_context context, const strix_matmul_desc *desc,
                                      const strix_stream *stream, uint32_t operation,
                                      strix_linear_plan *out);
strix_status strix_linear_plan_submit(strix_linear_plan plan);
strix_status strix_linear_plan_destroy(strix_linear_plan plan);
strix_status strix_grouped_moe_workspace_bytes(strix_context context,
                                               const strix_grouped_moe_desc *desc,
                                               uint64_t *out_bytes);
strix_status strix_grouped_moe(strix_context context, const strix_grouped_moe_desc *desc,
                               const strix_stream *stream);

/* ---- TP dense plans (reference :311-334, :395-404) ------------------------------ */
/* F32 row views: unit channel stride, row stride >= width; rows 1..8; workspace as
 * returned by strix_tp_dense_workspace_bytes (zero when one K partition suffices). */
strix_status strix_tp_dense_plan_create(strix_context context, const strix_matmul_desc *desc,
                                        const strix_stream *stream, strix_tp_dense_plan *out);
strix_status strix_tp_dense_plan_create_tiled(strix_context context,
                                              const strix_matmul_desc *desc,
                                              const strix_stream *stream,
                                              uint32_t rows_per_block, strix_tp_dense_plan *out);
#define STRIX_TP_SPLITK_SINGLE UINT32_C(0)
#define STRIX_TP_SPLITK_TWO UINT32_C(1)
strix_status strix_tp_dense_workspace_bytes(strix_context context,
                                            const strix_matmul_desc *desc,
                                            uint32_t rows_per_block, uint64_t *out_bytes);
strix_status strix_tp_dense_plan_create_splitk(strix_context context,
                                               const strix_matmul_desc *desc,
                                               const strix_stream *stream,
                                               uint32_t rows_per_block, uint32_t strategy,
                                               strix_tp_dense_plan *out);

/* ---- paired projections and SwiGLU (reference :335-383) -------------------------- */
typedef struct strix_tp_dense_pair_member {
    strix_weights weights;
    strix_tensor_desc output;
    float alpha;
    float beta;
} strix_tp_dense_pair_member;

/* Two projections of one shared input in one submission. */
typedef struct strix_tp_dense_pair_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    strix_tensor_desc input;
    strix_tp_dense_pair_member member[2];
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t rows_per_block;
    uint32_t strategy;
    uint64_t reserved[4];
} strix_tp_dense_pair_desc;

/* hidden_output = SiLU(gate(X)) * up(X); optional contiguous diagnostics. */
typedef struct strix_tp_swiglu_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    strix_tensor_desc input;
    strix_weights gate;
    strix_weights up;
    strix_tensor_desc hidden_output;
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t rows_per_block;
    uint32_t strategy;
    float *diagnostic_gate;
    float *diagnostic_up;
    uint64_t diagnostic_bytes;
    uint64_t reserved[4];
} strix_tp_swiglu_desc;

typedef struct strix_tp_dense_pair_plan_impl *strix_tp_dense_pair_plan;
typedef struct strix_tp_dense_pair_plan_impl *strix_tp_swiglu_plan;
void strix_tp_dense_pair_desc_init(strix_tp_dense_pair_desc *desc);
void strix_tp_swiglu_desc_init(strix_tp_swiglu_desc *desc);
strix_status strix_tp_dense_pair_workspace_bytes(strix_context context,
                                                 const strix_tp_dense_pair_desc *desc,
                                                 uint64_t *out_bytes);
strix_status strix_tp_dense_pair_plan_create(strix_context context,
                                             const strix_tp_dense_pair_desc *desc,
                                             const strix_stream *stream,
                                             strix_tp_dense_pair_plan *out);
strix_status strix_tp_dense_pair_plan_submit(strix_tp_dense_pair_plan plan);
strix_status strix_tp_dense_pair_plan_destroy(strix_tp_dense_pair_plan plan);
strix_status strix_tp_swiglu_workspace_bytes(strix_context context,
                                             const strix_tp_swiglu_desc *desc,
                                             uint64_t *out_bytes);
strix_status strix_tp_swiglu_plan_create(strix_context context,
                                         const strix_tp_swiglu_desc *desc,
                                         const strix_stream *stream, strix_tp_swiglu_plan *out);
strix_status strix_tp_swiglu_plan_submit(strix_tp_swiglu_plan plan);
strix_status strix_tp_swiglu_plan_destroy(strix_tp_swiglu_plan plan);

/* ---- dense "r1" identities (reference :384-416) ----------------------------------- */
#define STRIX_DENSE_R1_S4 UINT32_C(0)
#define STRIX_DENSE_R1_LEGACY UINT32_C(1)
strix_status strix_tp_dense_r1_workspace_bytes(strix_context context,
                                               const strix_matmul_desc *desc,
                                               uint32_t rows_per_block, uint32_t identity,
                                               uint64_t *out_bytes);
strix_status strix_tp_dense_plan_create_r1(strix_context context, const strix_matmul_desc *desc,
                                           const strix_stream *stream, uint32_t rows_per_block,
                                           uint32_t identity, strix_tp_dense_plan *out);
strix_status strix_tp_dense_plan_submit(strix_tp_dense_plan plan);
strix_status strix_tp_dense_plan_destroy(strix_tp_dense_plan plan);
strix_status strix_tp_dense_pair_r1_workspace_bytes(strix_context context,
                                                    const strix_tp_dense_pair_desc *desc,
                                                    uint32_t identity, uint64_t *out_bytes);
strix_status strix_tp_dense_pair_plan_create_r1(strix_context context,
                                                const strix_tp_dense_pair_desc *desc,
                                                const strix_stream *stream, uint32_t identity,
                                                strix_tp_dense_plan *out);

/* ---- grouped strided GEMV (reference :417-466) ------------------------------------- */
#define STRIX_TRELLIS_HAS_GROUPED_GEMV 1
#define STRIX_GEMV_ROW_INVARIANT_R1 UINT32_C(1)
/* G <= 8 independent linears of one geometry and rate in one dispatch:
 *   output[r][g*output_group_stride + n] = Linear_g(input[r][g*input_group_stride + i])
 * alpha 1, beta 0, rows 1..8, strides in F32 elements. */
typedef struct strix_grouped_gemv_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    const strix_weights *weights;
    uint64_t group_count;
    uint32_t rows;
    uint32_t flags;
    const float *input;
    uint64_t input_row_stride;
    uint64_t input_group_stride;
    uint64_t input_buffer_bytes;
    float *output;
    uint64_t output_row_stride;
    uint64_t output_group_stride;
    uint64_t output_buffer_bytes;
    void *workspace;
    uint64_t workspace_bytes;
    uint64_t reserved[4];
} strix_grouped_gemv_desc;
typedef struct strix_grouped_gemv_plan_impl *strix_grouped_gemv_plan;
strix_status strix_grouped_gemv_workspace_bytes(strix_context context,
                                                const strix_grouped_gemv_desc *desc,
                                                uint64_t *out_bytes);
strix_status strix_grouped_gemv_plan_create(strix_context context,
                                            const strix_grouped_gemv_desc *desc,
                                            const strix_stream *stream,
                                            strix_grouped_gemv_plan *out);
strix_status strix_grouped_gemv_plan_submit(strix_grouped_gemv_plan plan);
strix_status strix_grouped_gemv_plan_destroy(strix_grouped_gemv_plan plan);

/* ---- routed-expert plans (reference :467-523) --------------------------------------- */
void strix_tp_moe_desc_init(strix_tp_moe_desc *desc);
void strix_tp_moe_device_desc_init(strix_tp_moe_device_desc *desc);
strix_status strix_tp_moe_workspace_bytes(strix_context context, const strix_tp_moe_desc *desc,
                                          uint64_t *out_bytes);
strix_status strix_tp_moe_plan_create(strix_context context, const strix_tp_moe_desc *desc,
                                      const strix_stream *stream, strix_tp_moe_plan *out);
strix_status strix_tp_moe_plan_create_device(strix_context context,
                                             const strix_tp_moe_device_desc *desc,
                                             const strix_stream *stream, strix_tp_moe_plan *out);
strix_status strix_tp_moe_split_workspace_bytes(strix_context context,
                                                const strix_tp_moe_desc *desc,
                                                uint64_t *out_bytes);
strix_status strix_tp_moe_plan_create_split(strix_context context, const strix_tp_moe_desc *desc,
                                            const strix_stream *stream, strix_tp_moe_plan *out);
strix_status strix_tp_moe_plan_create_device_split(strix_context context,
                                                   const strix_tp_moe_device_desc *desc,
                                                   const strix_stream *stream,
                                                   strix_tp_moe_plan *out);
strix_status strix_tp_moe_plan_create_a8r(strix_context context, const strix_tp_moe_desc *desc,
                                          const strix_stream *stream, strix_tp_moe_plan *out);
strix_status strix_tp_moe_plan_create_device_a8r(strix_context context,
                                                 const strix_tp_moe_device_desc *desc,
                                                 const strix_stream *stream,
                                                 strix_tp_moe_plan *out);
strix_status strix_tp_moe_plan_down_core(strix_tp_moe_plan plan);
strix_status strix_tp_moe_plan_down_finish(strix_tp_moe_plan plan);
strix_status strix_tp_moe_plan_down_reference_core(strix_tp_moe_plan plan);
strix_status strix_tp_moe_plan_submit(strix_tp_moe_plan plan);
strix_status strix_tp_moe_plan_gate_up(strix_tp_moe_plan plan);
strix_status strix_tp_moe_plan_down(strix_tp_moe_plan plan);
strix_status strix_tp_moe_plan_destroy(strix_tp_moe_plan plan);

/* Every submission status covers validation and enqueue only (reference :525-527);
 * asynchronous device errors surface through the CUDA runtime. */
#ifdef __cplusplus
}
#endif
#endif /* STRIX_TRELLIS_H */
