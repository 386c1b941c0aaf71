// Routed-expert and SwiGLU plans.  Reference counterpart: src/tp_api.inc:1-192, 265-721.
#include "api_internal.h"

using namespace sapi;

namespace {
template <class D> void init_moe_desc(D* d) {
    if (!d) return;
    *d = {};
    d->struct_size = sizeof(*d);
    d->abi_version = STRIX_TRELLIS_ABI_VERSION;
    d->alpha = 1.0f;
    d->input.struct_size = d->output.struct_size = sizeof(strix_tensor_desc);
    d->input.abi_version = d->output.abi_version = STRIX_TRELLIS_ABI_VERSION;
    d->input.dtype = d->output.dtype = STRIX_DTYPE_F32;
    d->input.rank = d->output.rank = 2;
}
}  // namespace

extern "C" {

void strix_tp_moe_desc_init(strix_tp_moe_desc* d) { init_moe_desc(d); }
void strix_tp_moe_device_desc_init(strix_tp_moe_device_desc* d) { init_moe_desc(d); }
void strix_tp_swiglu_desc_init(strix_tp_swiglu_desc* d) {
    if (!d) return;
    *d = {};
    d->struct_size = sizeof(*d);
    d->abi_version = STRIX_TRELLIS_ABI_VERSION;
    d->input.struct_size = d->hidden_output.struct_size = sizeof(strix_tensor_desc);
    d->input.abi_version = d->hidden_output.abi_version = STRIX_TRELLIS_ABI_VERSION;
    d->input.dtype = d->hidden_output.dtype = STRIX_DTYPE_F32;
    d->input.rank = d->hidden_output.rank = 2;
}

#define ST_UNBUILT_QUERY(name, desc_t)                                                  \
    strix_status name(strix_context, const desc_t*, uint64_t* out) {                    \
        if (out) *out = 0;                                                               \
        return STRIX_ERROR_NOT_IMPLEMENTED;                                              \
    }
#define ST_UNBUILT_CREATE(name, desc_t, plan_t)                                          \
    strix_status name(strix_context, const desc_t*, const strix_stream*, plan_t* out) {  \
        if (out) *out = nullptr;                                                         \
        return STRIX_ERROR_NOT_IMPLEMENTED;                                              \
    }
#define ST_UNBUILT_PLAN(name, plan_t) \
    strix_status name(plan_t) { return STRIX_ERROR_NOT_IMPLEMENTED; }

ST_UNBUILT_QUERY(strix_tp_swiglu_workspace_bytes, strix_tp_swiglu_desc)
ST_UNBUILT_CREATE(strix_tp_swiglu_plan_create, strix_tp_swiglu_desc, strix_tp_swiglu_plan)
ST_UNBUILT_PLAN(strix_tp_swiglu_plan_submit, strix_tp_swiglu_plan)
ST_UNBUILT_PLAN(strix_tp_swiglu_plan_destroy, strix_tp_swiglu_plan)
ST_UNBUILT_QUERY(strix_tp_moe_workspace_bytes, strix_tp_moe_desc)
ST_UNBUILT_CREATE(strix_tp_moe_plan_create, strix_tp_moe_desc, strix_tp_moe_plan)
ST_UNBUILT_CREATE(strix_tp_moe_plan_create_device, strix_tp_moe_device_desc, strix_tp_moe_plan)
ST_UNBUILT_QUERY(strix_tp_moe_split_workspace_bytes, strix_tp_moe_desc)
ST_UNBUILT_CREATE(strix_tp_moe_plan_create_split, strix_tp_moe_desc, strix_tp_moe_plan)
ST_UNBUILT_CREATE(strix_tp_moe_plan_create_device_split, strix_tp_moe_device_desc, strix_tp_moe_plan)
ST_UNBUILT_CREATE(strix_tp_moe_plan_create_a8r, strix_tp_moe_desc, strix_tp_moe_plan)
ST_UNBUILT_CREATE(strix_tp_moe_plan_create_device_a8r, strix_tp_moe_device_desc, strix_tp_moe_plan)
ST_UNBUILT_PLAN(strix_tp_moe_plan_down_core, strix_tp_moe_plan)
ST_UNBUILT_PLAN(strix_tp_moe_plan_down_finish, strix_tp_moe_plan)
ST_UNBUILT_PLAN(strix_tp_moe_plan_down_reference_core, strix_tp_moe_plan)
ST_UNBUILT_PLAN(strix_tp_moe_plan_submit, strix_tp_moe_plan)
ST_UNBUILT_PLAN(strix_tp_moe_plan_gate_up, strix_tp_moe_plan)
ST_UNBUILT_PLAN(strix_tp_moe_plan_down, strix_tp_moe_plan)
ST_UNBUILT_PLAN(strix_tp_moe_plan_destroy, strix_tp_moe_plan)

}  // extern "C"
