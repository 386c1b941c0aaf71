// Row counts above 8 that do not reach the tensor-core prefill kernel's minimum tile
// run as 8-row chunks of the fused GEMV, the same decomposition the reference uses for
// its vector route
// (src/backend.hip:141-146).  Same arithmetic per row as strix_gemv.
#include "backend.h"

namespace st {

GemmPlan plan_gemm_chunked(const DeviceWeights& w, int rows, int sm_count) {
    (void)rows;
    GemmPlan plan{};
    const GemvPlan g = plan_gemv(w, 8, sm_count);
    plan.act_bytes = 0;
    plan.workspace_bytes = g.counter_bytes + g.partial_bytes;
    plan.tile_m = 8;
    plan.tile_n = 128;
    plan.sm_count = sm_count;
    plan.tensor_core = false;
    return plan;
}

cudaError_t launch_gemm_chunked(const LinearCall& call, int sm_count, void* workspace, bool programmatic_launch,
                                cudaStream_t stream) {
    // Chunks of 8 rows use the 8-row plan; a shorter tail uses its own plan, whose
    // scratch requirement is never larger.
    bool zeroed = false;
    for (int begin = 0; begin < call.rows; begin += 8) {
        LinearCall part = call;
        part.rows = call.rows - begin < 8 ? call.rows - begin : 8;
        part.x = reinterpret_cast<const float*>(reinterpret_cast<const unsigned char*>(call.x) +
                                                (size_t)begin * call.x_stride * dtype_bytes(call.x_dtype));
        part.y = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(call.y) +
                                          (size_t)begin * call.y_stride * dtype_bytes(call.y_dtype));
        const GemvPlan g = plan_gemv(call.w, part.rows, sm_count);
        if (!zeroed) {  // the first chunk is the largest: its scratch covers the others'
            const cudaError_t e = reset_gemv_scratch(workspace, g, stream);
            if (e != cudaSuccess) return e;
            zeroed = true;
        }
        const cudaError_t e = launch_gemv(part, g, workspace, programmatic_launch, stream);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace st
