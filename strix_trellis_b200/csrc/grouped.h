// Grouped linears: many independent complete linears of ONE geometry (inputs, outputs)
// in one launch, each with its own weights (any rate 1..8), its own gathered input rows and
// scattered output rows.  Building block of the routed-expert, SwiGLU and grouped-GEMV plans.
#pragma once
#include "backend.h"

namespace st {

constexpr int kGroupRows = 8;

// One problem.  rows == 0 marks an unused slot (its CTAs exit at once).
// Input row r is x + x_row[r]*x_stride, output row r is y + y_row[r]*y_stride.
struct GroupedProblem {
    DeviceWeights w;
    const float* x;
    float* y;
    long long x_stride, y_stride;
    int rows;
    int x_row[kGroupRows];
    int y_row[kGroupRows];
    unsigned int* counters;  // [outputs/128], zero between launches
    float* partials;         // [outputs/128][splits][rows][128]
};

struct GroupedPlan {
    int splits;          // K partitions per column block of a launch
    int scratch_splits;  // partitions the per-problem scratch is sized for (>= splits)
    int stages;
    int ctas_per_problem;
    int stage_stride;
    size_t smem_bytes;
    size_t counter_bytes_per_problem;
    size_t partial_bytes_per_problem;  // for kGroupRows rows
};
// `problems` = the number of problems a launch is EXPECTED to have live (it sets the partition
// count).  `headroom` sizes the scratch for that many times the planned partitions, so that
// replan_grouped may choose more of them later, when the expectation changes.
GroupedPlan plan_grouped(int inputs, int outputs, int max_bits, int problems, int sm_count, int headroom = 1);
GroupedPlan replan_grouped(const GroupedPlan& sized, int inputs, int outputs, int max_bits, int problems, int sm_count);
// `problems` lives in device memory; slots with rows == 0 are skipped on the device.
cudaError_t launch_grouped(const GroupedProblem* problems, int problem_count, int inputs, int outputs,
                           int codebook, const GroupedPlan& plan, unsigned int* status, bool programmatic,
                           cudaStream_t stream);

// hidden[r][c] = SwiGLU(gate[r][c], up[r][c]); gate/up contiguous [rows][width], hidden rows
// `out_stride` apart (src/tp_moe_activation.hpp:52-59).
cudaError_t launch_swiglu(const float* gate, const float* up, float* hidden, int rows, int width,
                          long long out_stride, bool programmatic, cudaStream_t stream);

// Device-side routing for a persistent expert bank: validates each token's route row and
// groups the valid routes by expert into problem slots of up to kGroupRows rows each
// (slot tables hold tokens*top_k slots; unused ones get rows = 0).
struct MoeBankEntry { DeviceWeights gate, up, down; };
// The bank is a window of the router's id space: id g is bank entry g - first_expert when that
// lies in [0, bank_count), belongs to another rank when g < experts_total (its slot runs nothing
// here and does not invalidate the row), and is invalid otherwise.  first_expert = 0 and
// experts_total = bank_count is the single-rank case.
struct MoeWindow { int first_expert, experts_total; };
cudaError_t launch_moe_route(const unsigned int* route_ids, const float* route_scores, int tokens, int top_k,
                             const MoeBankEntry* bank, int bank_count, MoeWindow window, GroupedProblem* gate_up,
                             GroupedProblem* down, int* row_valid, bool programmatic, cudaStream_t stream);

// Routed-expert combine: y[t] = alpha * sum_{s ascending, from +0} RN32(score[t,s]*each[t,s]) + beta*y[t];
// a zero score skips its slot; a row flagged invalid becomes NaN (src/tp_moe.hip:112-164).
// With `route_ids` and a window, slots whose expert lives on another rank are skipped: the
// result is this rank's contribution (the reference's per-rank semantics, include/strix_trellis.h:215-216).
cudaError_t launch_moe_combine(const float* each, const float* scores, const int* row_valid, int tokens,
                               int top_k, int outputs, float* y, long long y_stride, float alpha, float beta,
                               bool programmatic, cudaStream_t stream, const unsigned int* route_ids = nullptr,
                               int first_expert = 0, int bank_count = 0);

}  // namespace st
