// Per-rank dense tensor-parallel plans: strided row views, rows 1..8, one fused launch
// per projection.  Reference counterpart: src/tp_api.inc:196-264 (dense), src/
// tp_split_api.inc (split-K, pair), src/dense_r1_api.inc, src/dense_r1_group_api.inc
// (grouped GEMV).  The reference's creators differ only in the gfx1151 schedule they
// pick; here they all run the fused GEMV kernel and differ only in who owns scratch.
#include "api_internal.h"
#include "grouped.h"

using namespace sapi;

struct strix_tp_dense_plan_impl {
    strix_context owner;
    std::vector<strix_weights> retained;
    std::vector<st::LinearCall> calls;
    std::vector<void*> scratch;  // per call; owned by the caller or by the weights
    cudaStream_t stream;
    // grouped strided GEMV: every group is one problem of ONE grouped launch
    st::GroupedProblem* problems = nullptr;  // device table inside the caller's workspace
    int problem_count = 0;
    st::GroupedPlan grouped{};
    int inputs = 0, outputs = 0, codebook = 0;
};

namespace {

strix_status submit_plan(strix_tp_dense_plan_impl* p) {
    if (!p) return STRIX_ERROR_INVALID_ARGUMENT;
    const strix_status s = context_check(p->owner);
    if (s != STRIX_SUCCESS) return s;
    if (p->problem_count)
        return cuda_status(st::launch_grouped(p->problems, p->problem_count, p->inputs, p->outputs, p->codebook,
                                              p->grouped, p->owner->status, p->owner->programmatic_launch, p->stream));
    for (size_t i = 0; i < p->calls.size(); ++i) {
        const cudaError_t e = enqueue_linear(p->owner, p->calls[i], p->scratch[i], false, p->stream);
        if (e != cudaSuccess) return cuda_status(e);
    }
    return STRIX_SUCCESS;
}

void release_plan(strix_tp_dense_plan_impl* p) {
    for (strix_weights w : p->retained) --w->plan_refs;
}

// Scratch for one call.  Library-owned scratch hangs off the weights handle so that a
// captured graph stays valid after the plan is gone; it is marked empty here once.
strix_status provide_scratch(strix_context c, strix_weights w, int rows, void* caller, uint64_t caller_bytes,
                             uint64_t caller_offset, cudaStream_t cs, void*& out) {
    const st::GemvPlan gp = st::plan_gemv(w->device, rows, c->sm_count);
    const uint64_t need = gp.counter_bytes + gp.partial_bytes;
    out = nullptr;
    if (!need) return STRIX_SUCCESS;
    cudaError_t e;
    if (caller) {
        if (caller_offset > caller_bytes || need > caller_bytes - caller_offset)
            return STRIX_ERROR_INSUFFICIENT_BUFFER;
        out = static_cast<unsigned char*>(caller) + caller_offset;
    } else {
        e = cudaMalloc(&out, need);
        if (e != cudaSuccess) { (void)cudaGetLastError(); return cuda_status(e); }
        try { w->plan_scratch.push_back(out); } catch (...) { (void)cudaFree(out); return STRIX_ERROR_OUT_OF_MEMORY; }
    }
    e = st::reset_gemv_scratch(out, gp, cs);
    return cuda_status(e);
}

// mode 0: workspace must be NULL/0, scratch is library-owned; mode 1: the caller
// supplies the queried workspace.
strix_status create_dense(strix_context c, const strix_matmul_desc* d, const strix_stream* stream,
                          uint32_t rows_per_block, int mode, strix_tp_dense_plan* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    View v{};
    s = view_check(c, d, false, v);
    if (s != STRIX_SUCCESS) return s;
    if (v.rows < 1 || v.rows > 8 || rows_per_block > (uint32_t)v.rows) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const uint64_t need = linear_workspace(c, d->weights->device, v.rows);
    if (mode == 0) {
        if (d->workspace || d->workspace_bytes) return STRIX_ERROR_INVALID_ARGUMENT;
        s = storage_check(c, *d, v, 0, nullptr, 0);
    } else {
        s = storage_check(c, *d, v, need, d->workspace, d->workspace_bytes);
    }
    if (s != STRIX_SUCCESS) return s;
    strix_tp_dense_plan_impl* p = new (std::nothrow) strix_tp_dense_plan_impl{};
    if (!p) return STRIX_ERROR_OUT_OF_MEMORY;
    p->owner = c;
    p->stream = cs;
    void* scratch = nullptr;
    s = provide_scratch(c, d->weights, v.rows, mode ? d->workspace : nullptr, d->workspace_bytes, 0, cs, scratch);
    if (s == STRIX_SUCCESS) s = cuda_status(cudaStreamSynchronize(cs));
    if (s != STRIX_SUCCESS) { delete p; return s; }
    p->calls.push_back(make_call(c, *d, v));
    p->scratch.push_back(scratch);
    p->retained.push_back(d->weights);
    ++d->weights->plan_refs;
    *out = p;
    return STRIX_SUCCESS;
}

strix_status dense_workspace(strix_context c, const strix_matmul_desc* d, uint32_t rows_per_block,
                             uint64_t* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = 0;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    View v{};
    s = view_check(c, d, false, v);
    if (s != STRIX_SUCCESS) return s;
    if (v.rows < 1 || v.rows > 8 || rows_per_block > (uint32_t)v.rows) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    *out = linear_workspace(c, d->weights->device, v.rows);
    return STRIX_SUCCESS;
}

// The pair descriptor as two ordinary matmul descriptors over one input.
strix_status pair_members(const strix_tp_dense_pair_desc* d, strix_matmul_desc (&m)[2]) {
    strix_status s = header(d);
    if (s != STRIX_SUCCESS) return s;
    for (int i = 0; i < 2; ++i) {
        strix_matmul_desc_init(&m[i]);
        m[i].weights = d->member[i].weights;
        m[i].input = d->input;
        m[i].output = d->member[i].output;
        m[i].alpha = d->member[i].alpha;
        m[i].beta = d->member[i].beta;
    }
    return STRIX_SUCCESS;
}

strix_status pair_workspace(strix_context c, const strix_tp_dense_pair_desc* d, uint64_t* out,
                            uint64_t (&offsets)[2]) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = 0;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    strix_matmul_desc m[2];
    s = pair_members(d, m);
    if (s != STRIX_SUCCESS) return s;
    uint64_t total = 0;
    for (int i = 0; i < 2; ++i) {
        View v{};
        s = view_check(c, &m[i], false, v);
        if (s != STRIX_SUCCESS) return s;
        if (v.rows < 1 || v.rows > 8) return STRIX_ERROR_UNSUPPORTED_FORMAT;
        offsets[i] = total;
        total += st::align_up(linear_workspace(c, m[i].weights->device, v.rows));
    }
    *out = total;
    return STRIX_SUCCESS;
}

strix_status create_pair(strix_context c, const strix_tp_dense_pair_desc* d, const strix_stream* stream,
                         strix_tp_dense_plan_impl** out) {
    *out = nullptr;
    uint64_t need = 0, offsets[2] = {0, 0};
    strix_status s = pair_workspace(c, d, &need, offsets);
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    strix_matmul_desc m[2];
    pair_members(d, m);
    View v[2];
    for (int i = 0; i < 2; ++i) {
        s = view_check(c, &m[i], false, v[i]);
        if (s == STRIX_SUCCESS) s = storage_check(c, m[i], v[i], (i || !d->workspace) ? 0 : need, d->workspace, d->workspace_bytes);
        if (s != STRIX_SUCCESS) return s;
    }
    if (overlap(m[0].output.data, v[0].y_bytes, m[1].output.data, v[1].y_bytes))
        return STRIX_ERROR_INVALID_ARGUMENT;
    strix_tp_dense_plan_impl* p = new (std::nothrow) strix_tp_dense_plan_impl{};
    if (!p) return STRIX_ERROR_OUT_OF_MEMORY;
    p->owner = c;
    p->stream = cs;
    for (int i = 0; i < 2 && s == STRIX_SUCCESS; ++i) {
        void* scratch = nullptr;
        s = provide_scratch(c, m[i].weights, v[i].rows, d->workspace ? d->workspace : nullptr,
                            d->workspace_bytes, offsets[i], cs, scratch);
        p->calls.push_back(make_call(c, m[i], v[i]));
        p->scratch.push_back(scratch);
    }
    if (s == STRIX_SUCCESS) s = cuda_status(cudaStreamSynchronize(cs));
    if (s != STRIX_SUCCESS) { delete p; return s; }
    for (int i = 0; i < 2; ++i) { p->retained.push_back(m[i].weights); ++m[i].weights->plan_refs; }
    *out = p;
    return STRIX_SUCCESS;
}

}  // namespace

extern "C" {

strix_status strix_tp_dense_plan_create(strix_context c, const strix_matmul_desc* d,
                                        const strix_stream* s, strix_tp_dense_plan* out) {
    return create_dense(c, d, s, 0, 0, out);
}
strix_status strix_tp_dense_plan_create_tiled(strix_context c, const strix_matmul_desc* d,
                                              const strix_stream* s, uint32_t rows_per_block,
                                              strix_tp_dense_plan* out) {
    return create_dense(c, d, s, rows_per_block, 0, out);
}
strix_status strix_tp_dense_workspace_bytes(strix_context c, const strix_matmul_desc* d,
                                            uint32_t rows_per_block, uint64_t* out) {
    return dense_workspace(c, d, rows_per_block, out);
}
strix_status strix_tp_dense_plan_create_splitk(strix_context c, const strix_matmul_desc* d,
                                               const strix_stream* s, uint32_t rows_per_block,
                                               uint32_t strategy, strix_tp_dense_plan* out) {
    if (out) *out = nullptr;
    if (strategy != STRIX_TP_SPLITK_SINGLE && strategy != STRIX_TP_SPLITK_TWO)
        return STRIX_ERROR_INVALID_ARGUMENT;
    return create_dense(c, d, s, rows_per_block, 1, out);
}
strix_status strix_tp_dense_r1_workspace_bytes(strix_context c, const strix_matmul_desc* d,
                                               uint32_t rows_per_block, uint32_t identity, uint64_t* out) {
    if (out) *out = 0;
    if (identity != STRIX_DENSE_R1_S4 && identity != STRIX_DENSE_R1_LEGACY) return STRIX_ERROR_INVALID_ARGUMENT;
    return dense_workspace(c, d, rows_per_block, out);
}
strix_status strix_tp_dense_plan_create_r1(strix_context c, const strix_matmul_desc* d,
                                           const strix_stream* s, uint32_t rows_per_block,
                                           uint32_t identity, strix_tp_dense_plan* out) {
    if (out) *out = nullptr;
    if (identity != STRIX_DENSE_R1_S4 && identity != STRIX_DENSE_R1_LEGACY) return STRIX_ERROR_INVALID_ARGUMENT;
    return create_dense(c, d, s, rows_per_block, 1, out);
}
strix_status strix_tp_dense_plan_submit(strix_tp_dense_plan p) { return submit_plan(p); }
strix_status strix_tp_dense_plan_destroy(strix_tp_dense_plan p) {
    if (!p) return STRIX_ERROR_INVALID_ARGUMENT;
    release_plan(p);
    delete p;
    return STRIX_SUCCESS;
}

void strix_tp_dense_pair_desc_init(strix_tp_dense_pair_desc* d) {
    if (!d) return;
    *d = {};
    d->struct_size = sizeof(*d);
    d->abi_version = STRIX_TRELLIS_ABI_VERSION;
    d->input.struct_size = sizeof(strix_tensor_desc);
    d->input.abi_version = STRIX_TRELLIS_ABI_VERSION;
    d->input.dtype = STRIX_DTYPE_F32;
    d->input.rank = 2;
    for (auto& m : d->member) {
        m.output.struct_size = sizeof(strix_tensor_desc);
        m.output.abi_version = STRIX_TRELLIS_ABI_VERSION;
        m.output.dtype = STRIX_DTYPE_F32;
        m.output.rank = 2;
        m.alpha = 1.0f;
    }
}
strix_status strix_tp_dense_pair_workspace_bytes(strix_context c, const strix_tp_dense_pair_desc* d,
                                                 uint64_t* out) {
    uint64_t offsets[2];
    return pair_workspace(c, d, out, offsets);
}
strix_status strix_tp_dense_pair_plan_create(strix_context c, const strix_tp_dense_pair_desc* d,
                                             const strix_stream* s, strix_tp_dense_pair_plan* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    strix_tp_dense_plan_impl* p = nullptr;
    const strix_status st = create_pair(c, d, s, &p);
    if (st != STRIX_SUCCESS) return st;
    *out = reinterpret_cast<strix_tp_dense_pair_plan>(p);
    return STRIX_SUCCESS;
}
strix_status strix_tp_dense_pair_plan_submit(strix_tp_dense_pair_plan p) {
    return submit_plan(reinterpret_cast<strix_tp_dense_plan_impl*>(p));
}
strix_status strix_tp_dense_pair_plan_destroy(strix_tp_dense_pair_plan p) {
    return strix_tp_dense_plan_destroy(reinterpret_cast<strix_tp_dense_plan_impl*>(p));
}
strix_status strix_tp_dense_pair_r1_workspace_bytes(strix_context c, const strix_tp_dense_pair_desc* d,
                                                    uint32_t identity, uint64_t* out) {
    if (out) *out = 0;
    if (identity != STRIX_DENSE_R1_LEGACY) return STRIX_ERROR_INVALID_ARGUMENT;
    return strix_tp_dense_pair_workspace_bytes(c, d, out);
}
strix_status strix_tp_dense_pair_plan_create_r1(strix_context c, const strix_tp_dense_pair_desc* d,
                                                const strix_stream* s, uint32_t identity,
                                                strix_tp_dense_plan* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    if (identity != STRIX_DENSE_R1_LEGACY) return STRIX_ERROR_INVALID_ARGUMENT;
    return create_pair(c, d, s, out);
}

// ---- grouped strided GEMV ------------------------------------------------------------
static strix_status grouped_views(strix_context c, const strix_grouped_gemv_desc* d,
                                  std::vector<strix_matmul_desc>& m, std::vector<View>& v,
                                  std::vector<uint64_t>& offsets, uint64_t& total) {
    strix_status s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (!d->weights || d->group_count < 1 || d->group_count > 8 || d->rows < 1 || d->rows > 8 ||
        d->flags != STRIX_GEMV_ROW_INVARIANT_R1)
        return STRIX_ERROR_INVALID_ARGUMENT;
    total = 0;
    for (uint64_t g = 0; g < d->group_count; ++g) {
        strix_weights w = d->weights[g];
        if (!w || w->owner != c) return STRIX_ERROR_INVALID_ARGUMENT;
        const st::DeviceWeights& w0 = d->weights[0]->device;
        if (w->device.inputs != w0.inputs || w->device.outputs != w0.outputs || w->device.bits != w0.bits ||
            w->device.codebook != w0.codebook)
            return STRIX_ERROR_UNSUPPORTED_FORMAT;
        strix_matmul_desc one;
        strix_matmul_desc_init(&one);
        one.weights = w;
        const uint64_t in_off = g * d->input_group_stride, out_off = g * d->output_group_stride;
        if (d->output_group_stride < (uint64_t)w0.outputs && d->group_count > 1) return STRIX_ERROR_INVALID_ARGUMENT;
        if (in_off * 4 > d->input_buffer_bytes || out_off * 4 > d->output_buffer_bytes)
            return STRIX_ERROR_INSUFFICIENT_BUFFER;
        one.input.data = const_cast<float*>(d->input) + in_off;
        one.input.buffer_bytes = d->input_buffer_bytes - in_off * 4;
        one.output.data = d->output + out_off;
        one.output.buffer_bytes = d->output_buffer_bytes - out_off * 4;
        one.input.rank = one.output.rank = 2;
        one.input.shape[0] = one.output.shape[0] = d->rows;
        one.input.shape[1] = w0.inputs;
        one.output.shape[1] = w0.outputs;
        one.input.strides[0] = d->rows > 1 ? d->input_row_stride : (uint64_t)w0.inputs;
        one.output.strides[0] = d->rows > 1 ? d->output_row_stride : (uint64_t)w0.outputs;
        one.input.strides[1] = one.output.strides[1] = 1;
        View view{};
        s = view_check(c, &one, false, view);
        if (s != STRIX_SUCCESS) return s;
        for (size_t h = 0; h < m.size(); ++h)
            if (d->rows == 1 ? overlap(one.output.data, view.y_bytes, m[h].output.data, v[h].y_bytes)
                             : d->output_row_stride < (d->group_count - 1) * d->output_group_stride + w0.outputs)
                return STRIX_ERROR_INVALID_ARGUMENT;
        m.push_back(one);
        v.push_back(view);
        offsets.push_back(total);
    }
    // one grouped launch: [problem table][per group: arrival counters, partial planes]
    const st::DeviceWeights& w0 = d->weights[0]->device;
    const st::GroupedPlan gp = st::plan_grouped(w0.inputs, w0.outputs, w0.bits, (int)d->group_count, c->sm_count);
    total = st::align_up(d->group_count * sizeof(st::GroupedProblem)) +
            d->group_count * (gp.counter_bytes_per_problem + gp.partial_bytes_per_problem);
    return STRIX_SUCCESS;
}

strix_status strix_grouped_gemv_workspace_bytes(strix_context c, const strix_grouped_gemv_desc* d,
                                                uint64_t* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = 0;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    std::vector<strix_matmul_desc> m; std::vector<View> v; std::vector<uint64_t> off; uint64_t total = 0;
    s = grouped_views(c, d, m, v, off, total);
    if (s == STRIX_SUCCESS) *out = total;
    return s;
}

strix_status strix_grouped_gemv_plan_create(strix_context c, const strix_grouped_gemv_desc* d,
                                            const strix_stream* stream, strix_grouped_gemv_plan* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    std::vector<strix_matmul_desc> m; std::vector<View> v; std::vector<uint64_t> off; uint64_t total = 0;
    s = grouped_views(c, d, m, v, off, total);
    if (s != STRIX_SUCCESS) return s;
    for (size_t g = 0; g < m.size(); ++g) {
        s = storage_check(c, m[g], v[g], g ? 0 : total, d->workspace, d->workspace_bytes);
        if (s != STRIX_SUCCESS) return s;
    }
    strix_tp_dense_plan_impl* p = new (std::nothrow) strix_tp_dense_plan_impl{};
    if (!p) return STRIX_ERROR_OUT_OF_MEMORY;
    p->owner = c;
    p->stream = cs;
    {
        const st::DeviceWeights& w0 = m[0].weights->device;
        p->grouped = st::plan_grouped(w0.inputs, w0.outputs, w0.bits, (int)m.size(), c->sm_count);
        p->inputs = w0.inputs; p->outputs = w0.outputs; p->codebook = w0.codebook;
        p->problem_count = (int)m.size();
        unsigned char* base = static_cast<unsigned char*>(d->workspace);
        p->problems = reinterpret_cast<st::GroupedProblem*>(base);
        const size_t table = st::align_up(m.size() * sizeof(st::GroupedProblem));
        const size_t each = p->grouped.counter_bytes_per_problem + p->grouped.partial_bytes_per_problem;
        std::vector<st::GroupedProblem> host(m.size());
        for (size_t g = 0; g < m.size(); ++g) {
            st::GroupedProblem& pr = host[g];
            pr = st::GroupedProblem{};
            pr.w = m[g].weights->device;
            pr.x = static_cast<const float*>(m[g].input.data);
            pr.y = static_cast<float*>(m[g].output.data);
            pr.x_stride = (long long)v[g].x_stride;
            pr.y_stride = (long long)v[g].y_stride;
            pr.rows = v[g].rows;
            for (int k = 0; k < pr.rows; ++k) pr.x_row[k] = pr.y_row[k] = k;
            pr.counters = reinterpret_cast<unsigned int*>(base + table + g * each);
            pr.partials = reinterpret_cast<float*>(base + table + g * each + p->grouped.counter_bytes_per_problem);
        }
        cudaError_t e = cudaMemsetAsync(base + table, 0, m.size() * each, cs);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(p->problems, host.data(), host.size() * sizeof(st::GroupedProblem),
                                cudaMemcpyHostToDevice, cs);
        const cudaError_t done = cudaStreamSynchronize(cs);  // `host` leaves scope; counters are zero for every replay
        s = cuda_status(e != cudaSuccess ? e : done);
    }
    if (s != STRIX_SUCCESS) { delete p; return s; }
    for (auto& one : m) { p->retained.push_back(one.weights); ++one.weights->plan_refs; }
    *out = reinterpret_cast<strix_grouped_gemv_plan>(p);
    return STRIX_SUCCESS;
}
strix_status strix_grouped_gemv_plan_submit(strix_grouped_gemv_plan p) {
    return submit_plan(reinterpret_cast<strix_tp_dense_plan_impl*>(p));
}
strix_status strix_grouped_gemv_plan_destroy(strix_grouped_gemv_plan p) {
    return strix_tp_dense_plan_destroy(reinterpret_cast<strix_tp_dense_plan_impl*>(p));
}

}  // extern "C"
