// Routed-expert and SwiGLU plans.  Reference counterpart: src/tp_api.inc:1-192, 265-721,
// src/tp_moe.hip, src/tp_moe_policy.hpp:20-52 (host routing rules), src/tp_moe_routes.hpp
// (device routing rules).  Arithmetic contract (docs/TP_RANK.md:64-76):
//   hidden[r,s] = SiLU(gate_e(X[r])) * up_e(X[r]);  Y[r] = alpha*sum_s score*down_e(hidden) + beta*Y[r]
// with every projection a complete linear, slots summed ascending from +0, zero scores skipped.
// Launch structure here: grouped gate+up linears -> SwiGLU -> grouped down linears -> combine.
// The caller's workspace holds `hidden` [R, top_k, inter] exactly as in the reference; all
// other scratch (gate/up planes, per-route down outputs, problem tables) is owned by the plan.
#include <algorithm>

#include "api_internal.h"
#include "grouped.h"

using namespace sapi;

struct strix_tp_moe_plan_impl {
    strix_context owner = nullptr;
    cudaStream_t stream{};
    std::vector<strix_weights> retained;
    int tokens = 0, top_k = 0, model = 0, inter = 0, codebook = 2, max_bits = 0;
    bool device_routed = false;
    void* block = nullptr;  // one plan-owned device allocation
    st::GroupedProblem *gu = nullptr, *down = nullptr;
    int gu_count = 0, down_count = 0;
    st::MoeBankEntry* bank = nullptr;
    int bank_count = 0;
    const unsigned int* route_ids = nullptr;  // device (device-routed plans)
    const float* scores = nullptr;            // device
    int* row_valid = nullptr;                 // device (device-routed plans)
    float *hidden = nullptr, *g = nullptr, *u = nullptr, *each = nullptr;
    st::GroupedPlan gu_plan{}, down_plan{};
    float* y = nullptr;
    long long y_stride = 0;
    float alpha = 1.f, beta = 0.f;
    st::MoeWindow window{0, 0};  // device-routed plans: where the bank sits in the router's id space
};

// A dense pair-style plan with SwiGLU: two grouped problems + the activation.
struct strix_tp_dense_pair_plan_impl {
    strix_context owner = nullptr;
    cudaStream_t stream{};
    strix_weights gate = nullptr, up = nullptr;
    void* block = nullptr;
    st::GroupedProblem* problems = nullptr;
    st::GroupedPlan plan{};
    float *g = nullptr, *u = nullptr, *hidden = nullptr;
    long long hidden_stride = 0;
    int rows = 0, inter = 0, inputs = 0, codebook = 2;
    bool is_swiglu = false;
};

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

// F32 rank-2 row view [rows, width]: unit channel stride, row stride >= width.
strix_status row_view(const strix_tensor_desc& t, uint64_t rows, uint64_t width, uint64_t& stride, uint64_t& bytes) {
    strix_status s = header(&t);
    if (s != STRIX_SUCCESS) return s;
    if (enum_bits(t.dtype) != STRIX_DTYPE_F32 || t.rank != 2 || t.shape[0] != rows || t.shape[1] != width ||
        t.strides[1] != 1 || t.strides[0] < width)
        return STRIX_ERROR_UNSUPPORTED_FORMAT;
    stride = t.strides[0];
    uint64_t elements = 0;
    if (!mul_ok(rows - 1, stride, elements) || elements > UINT64_MAX - width) return STRIX_ERROR_INVALID_ARGUMENT;
    elements += width;
    if (!mul_ok(elements, 4, bytes) || !range_ok(t.data, bytes)) return STRIX_ERROR_INVALID_ARGUMENT;
    if (bytes > t.buffer_bytes) return STRIX_ERROR_INSUFFICIENT_BUFFER;
    if (!t.data || reinterpret_cast<uintptr_t>(t.data) % 4) return STRIX_ERROR_INVALID_ARGUMENT;
    return STRIX_SUCCESS;
}

struct Geometry { int model, inter, codebook, max_bits; };

strix_status expert_geometry(strix_context c, const strix_tp_expert_desc* experts, uint64_t count, Geometry& g) {
    if (!experts || !count) return STRIX_ERROR_INVALID_ARGUMENT;
    g = Geometry{0, 0, 0, 0};
    for (uint64_t i = 0; i < count; ++i) {
        const strix_tp_expert_desc& e = experts[i];
        if (e.struct_size != sizeof(e) || e.abi_version != STRIX_TRELLIS_ABI_VERSION) return STRIX_ERROR_ABI_MISMATCH;
        if (e.flags || e.reserved[0] || e.reserved[1]) return STRIX_ERROR_INVALID_ARGUMENT;
        const strix_weights ws[3] = {e.gate, e.up, e.down};
        for (strix_weights w : ws)
            if (!w || w->owner != c) return STRIX_ERROR_INVALID_ARGUMENT;
        const st::DeviceWeights &ga = e.gate->device, &up = e.up->device, &dn = e.down->device;
        if (i == 0) g = Geometry{ga.inputs, ga.outputs, ga.codebook, 0};
        if (ga.inputs != g.model || up.inputs != g.model || ga.outputs != g.inter || up.outputs != g.inter ||
            dn.inputs != g.inter || dn.outputs != g.model || ga.codebook != g.codebook || up.codebook != g.codebook ||
            dn.codebook != g.codebook)
            return STRIX_ERROR_UNSUPPORTED_FORMAT;
        g.max_bits = st::heavier_rate(g.max_bits ? g.max_bits : ga.bits, st::heavier_rate(ga.bits, st::heavier_rate(up.bits, dn.bits)));
    }
    return STRIX_SUCCESS;
}

struct Carver {  // bump allocator over one device block (sizes only when base == nullptr)
    unsigned char* base = nullptr;
    size_t used = 0;
    template <class T> T* take(size_t count) {
        used = st::align_up(used);
        T* p = base ? reinterpret_cast<T*>(base + used) : nullptr;
        used += count * sizeof(T);
        return p;
    }
};

// Problems a step is expected to have when `routes` routes spread evenly over `bank` experts,
// eight rows per problem.
int expected_problems(int routes, int bank) {
    if (routes < 1) routes = 1;
    const int chunks = (routes + bank * st::kGroupRows - 1) / (bank * st::kGroupRows);
    return std::min(routes, bank * chunks);
}

void fill_problem(st::GroupedProblem& p, const st::DeviceWeights& w, const float* x, long long xs, float* y,
                  long long ys, unsigned int* counters, float* partials) {
    p = st::GroupedProblem{};
    p.w = w;
    p.x = x;
    p.y = y;
    p.x_stride = xs;
    p.y_stride = ys;
    p.counters = counters;
    p.partials = partials;
}

// Lays out the plan-owned block and (when `p->block` is set) fills pointers.
size_t layout_block(strix_tp_moe_plan_impl* p, int gu_slots, int down_slots, bool with_scores) {
    Carver c{static_cast<unsigned char*>(p->block)};
    const size_t routes = (size_t)p->tokens * p->top_k;
    p->gu = c.take<st::GroupedProblem>(gu_slots);
    p->down = c.take<st::GroupedProblem>(down_slots);
    p->bank = c.take<st::MoeBankEntry>(p->bank_count);
    p->row_valid = c.take<int>(p->device_routed ? p->tokens : 0);
    float* scores = c.take<float>(with_scores ? routes : 0);
    if (with_scores) p->scores = scores;
    p->g = c.take<float>(routes * p->inter);
    p->u = c.take<float>(routes * p->inter);
    p->each = c.take<float>(routes * p->model);
    // per-problem scratch: counters then partial planes
    unsigned char* gu_scratch = c.take<unsigned char>(
        (size_t)gu_slots * (p->gu_plan.counter_bytes_per_problem + p->gu_plan.partial_bytes_per_problem));
    unsigned char* dn_scratch = c.take<unsigned char>(
        (size_t)down_slots * (p->down_plan.counter_bytes_per_problem + p->down_plan.partial_bytes_per_problem));
    (void)gu_scratch;
    (void)dn_scratch;
    return st::align_up(c.used);
}

unsigned char* scratch_of(strix_tp_moe_plan_impl* p, bool down, int slot) {
    // recompute the scratch base the same way layout_block did
    Carver c{static_cast<unsigned char*>(p->block)};
    const size_t routes = (size_t)p->tokens * p->top_k;
    const int gu_slots = p->gu_count, down_slots = p->down_count;
    c.take<st::GroupedProblem>(gu_slots);
    c.take<st::GroupedProblem>(down_slots);
    c.take<st::MoeBankEntry>(p->bank_count);
    c.take<int>(p->device_routed ? p->tokens : 0);
    c.take<float>(p->device_routed ? 0 : routes);
    c.take<float>(routes * p->inter);
    c.take<float>(routes * p->inter);
    c.take<float>(routes * p->model);
    const size_t gu_each = p->gu_plan.counter_bytes_per_problem + p->gu_plan.partial_bytes_per_problem;
    const size_t dn_each = p->down_plan.counter_bytes_per_problem + p->down_plan.partial_bytes_per_problem;
    unsigned char* gu_scratch = c.take<unsigned char>((size_t)gu_slots * gu_each);
    unsigned char* dn_scratch = c.take<unsigned char>((size_t)down_slots * dn_each);
    return down ? dn_scratch + (size_t)slot * dn_each : gu_scratch + (size_t)slot * gu_each;
}

void destroy_plan(strix_tp_moe_plan_impl* p) {
    if (p->block) (void)cudaFree(p->block);
    delete p;
}

// Common validation of X, Y, workspace, scalars.  Fills tokens/model/inter and pointers.
template <class D>
strix_status common_check(strix_context c, const D* d, const Geometry& g, int tokens, int top_k,
                          uint64_t& xs, uint64_t& ys, uint64_t& xb, uint64_t& yb, uint64_t& hidden_bytes) {
    if (!std::isfinite(d->alpha) || !std::isfinite(d->beta)) return STRIX_ERROR_INVALID_ARGUMENT;
    strix_status s = row_view(d->input, (uint64_t)tokens, (uint64_t)g.model, xs, xb);
    if (s != STRIX_SUCCESS) return s;
    s = row_view(d->output, (uint64_t)tokens, (uint64_t)g.model, ys, yb);
    if (s != STRIX_SUCCESS) return s;
    hidden_bytes = (uint64_t)tokens * top_k * g.inter * sizeof(float);
    if (d->workspace_bytes < hidden_bytes) return STRIX_ERROR_INSUFFICIENT_BUFFER;
    if (!d->workspace || reinterpret_cast<uintptr_t>(d->workspace) % kAlign || !range_ok(d->workspace, d->workspace_bytes))
        return STRIX_ERROR_INVALID_ARGUMENT;
    if (overlap(d->input.data, xb, d->output.data, yb) || overlap(d->workspace, d->workspace_bytes, d->input.data, xb) ||
        overlap(d->workspace, d->workspace_bytes, d->output.data, yb))
        return STRIX_ERROR_INVALID_ARGUMENT;
    s = device_buffer(c, d->input.data, xb, 4);
    if (s == STRIX_SUCCESS) s = device_buffer(c, d->output.data, yb, 4);
    if (s == STRIX_SUCCESS) s = device_buffer(c, d->workspace, d->workspace_bytes, kAlign);
    return s;
}

strix_status host_shape(const strix_tp_moe_desc* d, int& tokens, int& top_k) {
    strix_status s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (d->input.rank != 2) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const uint64_t r = d->input.shape[0];
    if (r < 1 || r > STRIX_B200_MOE_MAX_ROWS) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    if (!d->route_ids || !d->route_scores || d->route_ids_count != d->route_scores_count ||
        d->route_ids_count % r || d->route_ids_count / r < 1 || d->route_ids_count / r > STRIX_B200_MOE_MAX_TOP_K)
        return STRIX_ERROR_INVALID_ARGUMENT;
    if (d->expert_count < 1 || d->expert_count > STRIX_B200_MOE_MAX_BANK) return STRIX_ERROR_INVALID_ARGUMENT;
    tokens = (int)r;
    top_k = (int)(d->route_ids_count / r);
    return STRIX_SUCCESS;
}

// Host routing rules (reference src/tp_moe_policy.hpp:20-52): expert ids unique, every
// route id present, ids distinct within a row, scores finite and non-negative, no expert
// left unused.  Returns per-route expert indices.
strix_status host_routing(const strix_tp_moe_desc* d, int tokens, int top_k, std::vector<int>& route_expert) {
    const int count = (int)d->expert_count;
    for (int e = 0; e < count; ++e)
        for (int q = 0; q < e; ++q)
            if (d->experts[e].expert_id == d->experts[q].expert_id) return STRIX_ERROR_INVALID_ARGUMENT;
    std::vector<int> used(count, 0);
    route_expert.assign((size_t)tokens * top_k, -1);
    for (int r = 0; r < tokens; ++r)
        for (int s = 0; s < top_k; ++s) {
            const int route = r * top_k + s;
            const uint32_t id = d->route_ids[route];
            const float score = d->route_scores[route];
            if (!std::isfinite(score) || score < 0.0f) return STRIX_ERROR_INVALID_ARGUMENT;
            for (int q = 0; q < s; ++q)
                if (d->route_ids[r * top_k + q] == id) return STRIX_ERROR_INVALID_ARGUMENT;
            int e = 0;
            while (e < count && d->experts[e].expert_id != id) ++e;
            if (e == count) return STRIX_ERROR_INVALID_ARGUMENT;
            used[e] = 1;
            route_expert[route] = e;
        }
    for (int e = 0; e < count; ++e)
        if (!used[e]) return STRIX_ERROR_INVALID_ARGUMENT;
    return STRIX_SUCCESS;
}

strix_status enqueue_gate_up(strix_tp_moe_plan_impl* p) {
    cudaError_t e = cudaSuccess;
    if (p->device_routed)
        e = st::launch_moe_route(p->route_ids, p->scores, p->tokens, p->top_k, p->bank, p->bank_count, p->window, p->gu,
                                 p->down, p->row_valid, p->owner->programmatic_launch, p->stream);
    if (e == cudaSuccess)
        e = st::launch_grouped(p->gu, p->gu_count, p->model, p->inter, p->codebook, p->gu_plan, p->owner->status,
                               p->owner->programmatic_launch, p->stream);
    if (e == cudaSuccess)
        e = st::launch_swiglu(p->g, p->u, p->hidden, p->tokens * p->top_k, p->inter, p->inter,
                              p->owner->programmatic_launch, p->stream);
    return cuda_status(e);
}

strix_status enqueue_down(strix_tp_moe_plan_impl* p, bool combine = true) {
    cudaError_t e = st::launch_grouped(p->down, p->down_count, p->inter, p->model, p->codebook, p->down_plan,
                                       p->owner->status, p->owner->programmatic_launch, p->stream);
    if (e == cudaSuccess && combine) {
        const bool partial = p->device_routed && p->window.experts_total != p->bank_count;  // other ranks own some slots
        e = st::launch_moe_combine(p->each, p->scores, p->device_routed ? p->row_valid : nullptr, p->tokens, p->top_k,
                                   p->model, p->y, p->y_stride, p->alpha, p->beta, p->owner->programmatic_launch,
                                   p->stream, partial ? p->route_ids : nullptr, p->window.first_expert, p->bank_count);
    }
    return cuda_status(e);
}

strix_status create_host(strix_context c, const strix_tp_moe_desc* d, const strix_stream* stream,
                         strix_tp_moe_plan* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    int tokens = 0, top_k = 0;
    s = host_shape(d, tokens, top_k);
    if (s != STRIX_SUCCESS) return s;
    Geometry g{};
    s = expert_geometry(c, d->experts, d->expert_count, g);
    if (s != STRIX_SUCCESS) return s;
    uint64_t xs, ys, xb, yb, hidden_bytes;
    s = common_check(c, d, g, tokens, top_k, xs, ys, xb, yb, hidden_bytes);
    if (s != STRIX_SUCCESS) return s;
    std::vector<int> route_expert;
    s = host_routing(d, tokens, top_k, route_expert);
    if (s != STRIX_SUCCESS) return s;

    // group routes by expert, eight rows per problem (all routes for gate/up, scored ones for down)
    const int experts = (int)d->expert_count, routes = tokens * top_k;
    std::vector<std::vector<int>> by_expert(experts);
    for (int r = 0; r < routes; ++r) by_expert[route_expert[r]].push_back(r);
    struct Chunk { int expert; std::vector<int> routes; };
    std::vector<Chunk> gu_chunks, down_chunks;
    for (int e = 0; e < experts; ++e) {
        std::vector<int> scored;
        for (int r : by_expert[e])
            if (d->route_scores[r] != 0.0f) scored.push_back(r);
        for (size_t i = 0; i < by_expert[e].size(); i += st::kGroupRows)
            gu_chunks.push_back({e, {by_expert[e].begin() + i, by_expert[e].begin() + std::min(by_expert[e].size(), i + st::kGroupRows)}});
        for (size_t i = 0; i < scored.size(); i += st::kGroupRows)
            down_chunks.push_back({e, {scored.begin() + i, scored.begin() + std::min(scored.size(), i + st::kGroupRows)}});
    }
    strix_tp_moe_plan_impl* p = new (std::nothrow) strix_tp_moe_plan_impl;
    if (!p) return STRIX_ERROR_OUT_OF_MEMORY;
    p->owner = c;
    p->stream = cs;
    p->tokens = tokens; p->top_k = top_k; p->model = g.model; p->inter = g.inter; p->codebook = g.codebook;
    p->gu_count = 2 * (int)gu_chunks.size();
    p->down_count = (int)down_chunks.size();
    p->gu_plan = st::plan_grouped(g.model, g.inter, g.max_bits, p->gu_count, c->sm_count);
    p->down_plan = st::plan_grouped(g.inter, g.model, g.max_bits, std::max(p->down_count, 1), c->sm_count);
    const size_t bytes = layout_block(p, p->gu_count, p->down_count, true);
    cudaError_t e = cudaMalloc(&p->block, bytes);
    if (e != cudaSuccess) { (void)cudaGetLastError(); delete p; return cuda_status(e); }
    layout_block(p, p->gu_count, p->down_count, true);
    p->hidden = static_cast<float*>(d->workspace);
    p->y = static_cast<float*>(d->output.data);
    p->y_stride = (long long)ys;
    p->alpha = d->alpha; p->beta = d->beta;

    std::vector<st::GroupedProblem> host_gu(p->gu_count), host_dn(p->down_count);
    const float* x = static_cast<const float*>(d->input.data);
    for (size_t i = 0; i < gu_chunks.size(); ++i) {
        const strix_tp_expert_desc& ex = d->experts[gu_chunks[i].expert];
        for (int half = 0; half < 2; ++half) {
            st::GroupedProblem& pr = host_gu[2 * i + half];
            unsigned char* sc = scratch_of(p, false, (int)(2 * i + half));
            fill_problem(pr, half ? ex.up->device : ex.gate->device, x, (long long)xs, half ? p->u : p->g, g.inter,
                         reinterpret_cast<unsigned int*>(sc),
                         reinterpret_cast<float*>(sc + p->gu_plan.counter_bytes_per_problem));
            pr.rows = (int)gu_chunks[i].routes.size();
            for (int k = 0; k < pr.rows; ++k) {
                pr.x_row[k] = gu_chunks[i].routes[k] / top_k;  // token
                pr.y_row[k] = gu_chunks[i].routes[k];          // route
            }
        }
    }
    for (size_t i = 0; i < down_chunks.size(); ++i) {
        const strix_tp_expert_desc& ex = d->experts[down_chunks[i].expert];
        st::GroupedProblem& pr = host_dn[i];
        unsigned char* sc = scratch_of(p, true, (int)i);
        fill_problem(pr, ex.down->device, p->hidden, g.inter, p->each, g.model, reinterpret_cast<unsigned int*>(sc),
                     reinterpret_cast<float*>(sc + p->down_plan.counter_bytes_per_problem));
        pr.rows = (int)down_chunks[i].routes.size();
        for (int k = 0; k < pr.rows; ++k) pr.x_row[k] = pr.y_row[k] = down_chunks[i].routes[k];
    }
    // zero the whole block (counters must start at zero), then upload tables and scores
    e = cudaMemsetAsync(p->block, 0, bytes, cs);
    if (e == cudaSuccess && p->gu_count)
        e = cudaMemcpyAsync(p->gu, host_gu.data(), host_gu.size() * sizeof(st::GroupedProblem), cudaMemcpyHostToDevice, cs);
    if (e == cudaSuccess && p->down_count)
        e = cudaMemcpyAsync(p->down, host_dn.data(), host_dn.size() * sizeof(st::GroupedProblem), cudaMemcpyHostToDevice, cs);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(const_cast<float*>(p->scores), d->route_scores, (size_t)routes * sizeof(float),
                            cudaMemcpyHostToDevice, cs);
    const cudaError_t done = cudaStreamSynchronize(cs);  // host tables may go away after return
    if (e != cudaSuccess || done != cudaSuccess) { destroy_plan(p); return cuda_status(e != cudaSuccess ? e : done); }
    for (int i = 0; i < experts; ++i)
        for (strix_weights w : {d->experts[i].gate, d->experts[i].up, d->experts[i].down}) {
            if (std::find(p->retained.begin(), p->retained.end(), w) == p->retained.end()) {
                p->retained.push_back(w);  // each handle retained once, even when shared
                ++w->plan_refs;
            }
        }
    *out = p;
    return STRIX_SUCCESS;
}

strix_status create_device(strix_context c, const strix_tp_moe_device_desc* d, const strix_stream* stream,
                           strix_tp_moe_plan* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (d->input.rank != 2) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const uint64_t r = d->input.shape[0];
    if (r < 1 || r > STRIX_B200_MOE_MAX_ROWS) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    if (!d->route_ids || !d->route_scores || d->route_ids_bytes != d->route_scores_bytes ||
        d->route_ids_bytes % (4 * r) || d->route_ids_bytes / (4 * r) < 1 ||
        d->route_ids_bytes / (4 * r) > STRIX_B200_MOE_MAX_TOP_K)
        return STRIX_ERROR_INVALID_ARGUMENT;
    const int tokens = (int)r, top_k = (int)(d->route_ids_bytes / (4 * r));
    if (d->expert_count < (uint64_t)top_k || d->expert_count > STRIX_B200_MOE_MAX_BANK) return STRIX_ERROR_INVALID_ARGUMENT;
    Geometry g{};
    s = expert_geometry(c, d->experts, d->expert_count, g);
    if (s != STRIX_SUCCESS) return s;
    for (uint64_t i = 0; i < d->expert_count; ++i)
        if (d->experts[i].expert_id != i) return STRIX_ERROR_INVALID_ARGUMENT;  // bank position = router id
    uint64_t xs, ys, xb, yb, hidden_bytes;
    s = common_check(c, d, g, tokens, top_k, xs, ys, xb, yb, hidden_bytes);
    if (s != STRIX_SUCCESS) return s;
    s = device_buffer(c, d->route_ids, d->route_ids_bytes, 4);
    if (s == STRIX_SUCCESS) s = device_buffer(c, d->route_scores, d->route_scores_bytes, 4);
    if (s != STRIX_SUCCESS) return s;

    strix_tp_moe_plan_impl* p = new (std::nothrow) strix_tp_moe_plan_impl;
    if (!p) return STRIX_ERROR_OUT_OF_MEMORY;
    const int routes = tokens * top_k;
    p->owner = c; p->stream = cs; p->device_routed = true;
    p->tokens = tokens; p->top_k = top_k; p->model = g.model; p->inter = g.inter; p->codebook = g.codebook;
    p->gu_count = 2 * routes;
    p->down_count = routes;
    p->bank_count = (int)d->expert_count;
    p->window = st::MoeWindow{0, p->bank_count};
    // the K partition is planned for the problems a step is EXPECTED to have (routes spread evenly
    // over the bank, eight rows per problem), not for the slots it may have at most
    const int spread = expected_problems(routes, p->bank_count);
    p->max_bits = g.max_bits;
    // Scratch for up to four times the planned partitions (while it stays under 128 MB): a
    // window set later means fewer local routes, and fewer problems want more partitions.
    int headroom = 4;
    for (;; headroom /= 2) {
        p->gu_plan = st::plan_grouped(g.model, g.inter, g.max_bits, 2 * spread, c->sm_count, headroom);
        p->down_plan = st::plan_grouped(g.inter, g.model, g.max_bits, spread, c->sm_count, headroom);
        const size_t scratch = (size_t)p->gu_count * p->gu_plan.partial_bytes_per_problem +
                               (size_t)p->down_count * p->down_plan.partial_bytes_per_problem;
        if (headroom == 1 || scratch <= ((size_t)128 << 20)) break;
    }
    const size_t bytes = layout_block(p, p->gu_count, p->down_count, false);
    cudaError_t e = cudaMalloc(&p->block, bytes);
    if (e != cudaSuccess) { (void)cudaGetLastError(); delete p; return cuda_status(e); }
    layout_block(p, p->gu_count, p->down_count, false);
    p->hidden = static_cast<float*>(d->workspace);
    p->route_ids = d->route_ids;
    p->scores = d->route_scores;
    p->y = static_cast<float*>(d->output.data);
    p->y_stride = (long long)ys;
    p->alpha = d->alpha; p->beta = d->beta;
    // static part of every per-route slot; the device routing kernel fills weights and rows
    std::vector<st::GroupedProblem> host_gu(p->gu_count), host_dn(p->down_count);
    std::vector<st::MoeBankEntry> bank(p->bank_count);
    const float* x = static_cast<const float*>(d->input.data);
    for (int route = 0; route < routes; ++route) {
        for (int half = 0; half < 2; ++half) {
            st::GroupedProblem& pr = host_gu[2 * route + half];
            unsigned char* sc = scratch_of(p, false, 2 * route + half);
            fill_problem(pr, st::DeviceWeights{}, x, (long long)xs, half ? p->u : p->g, g.inter,
                         reinterpret_cast<unsigned int*>(sc),
                         reinterpret_cast<float*>(sc + p->gu_plan.counter_bytes_per_problem));
            pr.x_row[0] = route / top_k;
            pr.y_row[0] = route;
        }
        st::GroupedProblem& pr = host_dn[route];
        unsigned char* sc = scratch_of(p, true, route);
        fill_problem(pr, st::DeviceWeights{}, p->hidden, g.inter, p->each, g.model, reinterpret_cast<unsigned int*>(sc),
                     reinterpret_cast<float*>(sc + p->down_plan.counter_bytes_per_problem));
        pr.x_row[0] = pr.y_row[0] = route;
    }
    for (int i = 0; i < p->bank_count; ++i)
        bank[i] = st::MoeBankEntry{d->experts[i].gate->device, d->experts[i].up->device, d->experts[i].down->device};
    e = cudaMemsetAsync(p->block, 0, bytes, cs);
    if (e == cudaSuccess) e = cudaMemcpyAsync(p->gu, host_gu.data(), host_gu.size() * sizeof(st::GroupedProblem), cudaMemcpyHostToDevice, cs);
    if (e == cudaSuccess) e = cudaMemcpyAsync(p->down, host_dn.data(), host_dn.size() * sizeof(st::GroupedProblem), cudaMemcpyHostToDevice, cs);
    if (e == cudaSuccess) e = cudaMemcpyAsync(p->bank, bank.data(), bank.size() * sizeof(st::MoeBankEntry), cudaMemcpyHostToDevice, cs);
    const cudaError_t done = cudaStreamSynchronize(cs);
    if (e != cudaSuccess || done != cudaSuccess) { destroy_plan(p); return cuda_status(e != cudaSuccess ? e : done); }
    for (int i = 0; i < p->bank_count; ++i)
        for (strix_weights w : {d->experts[i].gate, d->experts[i].up, d->experts[i].down})
            if (std::find(p->retained.begin(), p->retained.end(), w) == p->retained.end()) {
                p->retained.push_back(w);
                ++w->plan_refs;
            }
    *out = p;
    return STRIX_SUCCESS;
}

}  // namespace

extern "C" {

void strix_tp_moe_desc_init(strix_tp_moe_desc* d) { init_moe_desc(d); }
void strix_tp_moe_device_desc_init(strix_tp_moe_device_desc* d) { init_moe_desc(d); }

strix_status strix_tp_moe_workspace_bytes(strix_context c, const strix_tp_moe_desc* d, uint64_t* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = 0;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    int tokens = 0, top_k = 0;
    s = host_shape(d, tokens, top_k);
    if (s != STRIX_SUCCESS) return s;
    Geometry g{};
    s = expert_geometry(c, d->experts, d->expert_count, g);
    if (s != STRIX_SUCCESS) return s;
    *out = (uint64_t)tokens * top_k * g.inter * sizeof(float);  // hidden [R, top_k, inter]
    return STRIX_SUCCESS;
}
strix_status strix_tp_moe_split_workspace_bytes(strix_context c, const strix_tp_moe_desc* d, uint64_t* out) {
    return strix_tp_moe_workspace_bytes(c, d, out);
}
strix_status strix_tp_moe_plan_create(strix_context c, const strix_tp_moe_desc* d, const strix_stream* s,
                                      strix_tp_moe_plan* out) {
    return create_host(c, d, s, out);
}
// The reference's split3 creators select another schedule of the same arithmetic.
strix_status strix_tp_moe_plan_create_split(strix_context c, const strix_tp_moe_desc* d, const strix_stream* s,
                                            strix_tp_moe_plan* out) {
    return create_host(c, d, s, out);
}
strix_status strix_tp_moe_plan_create_device(strix_context c, const strix_tp_moe_device_desc* d,
                                             const strix_stream* s, strix_tp_moe_plan* out) {
    return create_device(c, d, s, out);
}
strix_status strix_tp_moe_plan_create_device_split(strix_context c, const strix_tp_moe_device_desc* d,
                                                   const strix_stream* s, strix_tp_moe_plan* out) {
    return create_device(c, d, s, out);
}
// A8R is a different arithmetic (int8 activations) and is off by default in the reference.
strix_status strix_tp_moe_plan_create_a8r(strix_context, const strix_tp_moe_desc*, const strix_stream*,
                                          strix_tp_moe_plan* out) {
    if (out) *out = nullptr;
    return STRIX_ERROR_NOT_IMPLEMENTED;
}
strix_status strix_tp_moe_plan_create_device_a8r(strix_context, const strix_tp_moe_device_desc*,
                                                 const strix_stream*, strix_tp_moe_plan* out) {
    if (out) *out = nullptr;
    return STRIX_ERROR_NOT_IMPLEMENTED;
}
strix_status strix_tp_moe_plan_gate_up(strix_tp_moe_plan p) {
    if (!p) return STRIX_ERROR_INVALID_ARGUMENT;
    const strix_status s = context_check(p->owner);
    return s != STRIX_SUCCESS ? s : enqueue_gate_up(p);
}
strix_status strix_tp_moe_plan_down(strix_tp_moe_plan p) {
    if (!p) return STRIX_ERROR_INVALID_ARGUMENT;
    const strix_status s = context_check(p->owner);
    return s != STRIX_SUCCESS ? s : enqueue_down(p);
}
strix_status strix_tp_moe_plan_submit(strix_tp_moe_plan p) {
    if (!p) return STRIX_ERROR_INVALID_ARGUMENT;
    strix_status s = context_check(p->owner);
    if (s == STRIX_SUCCESS) s = enqueue_gate_up(p);
    if (s == STRIX_SUCCESS) s = enqueue_down(p);
    return s;
}
// ---- expert parallelism: the bank as a window of the router's id space ------------------------
strix_status strix_b200_moe_plan_set_window(strix_tp_moe_plan p, uint32_t first_expert, uint32_t experts_total) {
    if (!p || !p->device_routed) return STRIX_ERROR_INVALID_ARGUMENT;
    if (experts_total > INT_MAX || (uint64_t)first_expert + (uint64_t)p->bank_count > experts_total)
        return STRIX_ERROR_INVALID_ARGUMENT;
    p->window = st::MoeWindow{(int)first_expert, (int)experts_total};
    // of all routes, about bank / experts_total are this rank's: plan the partitions for those
    const long long routes = (long long)p->tokens * p->top_k;
    const int local = (int)std::max<long long>(1, (routes * p->bank_count + experts_total - 1) / experts_total);
    const int spread = expected_problems(local, p->bank_count);
    const int sms = p->owner->sm_count;
    p->gu_plan = st::replan_grouped(p->gu_plan, p->model, p->inter, p->max_bits, 2 * spread, sms);
    p->down_plan = st::replan_grouped(p->down_plan, p->inter, p->model, p->max_bits, spread, sms);
    return STRIX_SUCCESS;
}
// Routing, gate/up, SwiGLU and down of the routes this rank owns; no combine.
strix_status strix_b200_moe_plan_projections(strix_tp_moe_plan p) {
    if (!p) return STRIX_ERROR_INVALID_ARGUMENT;
    strix_status s = context_check(p->owner);
    if (s == STRIX_SUCCESS) s = enqueue_gate_up(p);
    if (s == STRIX_SUCCESS) s = enqueue_down(p, false);
    return s;
}
strix_status strix_b200_moe_plan_rows(strix_tp_moe_plan p, const float** each, const int32_t** row_valid) {
    if (each) *each = nullptr;
    if (row_valid) *row_valid = nullptr;
    if (!p || !each || !row_valid) return STRIX_ERROR_INVALID_ARGUMENT;
    *each = p->each;
    *row_valid = p->device_routed ? p->row_valid : nullptr;
    return STRIX_SUCCESS;
}
strix_status strix_b200_moe_plan_gate_up_rows(strix_tp_moe_plan p, const float** gate, const float** up) {
    if (gate) *gate = nullptr;
    if (up) *up = nullptr;
    if (!p || !gate || !up) return STRIX_ERROR_INVALID_ARGUMENT;
    *gate = p->g;
    *up = p->u;
    return STRIX_SUCCESS;
}

// Staged diagnostics of the reference's split3 schedule have no counterpart in this one.
strix_status strix_tp_moe_plan_down_core(strix_tp_moe_plan) { return STRIX_ERROR_NOT_IMPLEMENTED; }
strix_status strix_tp_moe_plan_down_finish(strix_tp_moe_plan) { return STRIX_ERROR_NOT_IMPLEMENTED; }
strix_status strix_tp_moe_plan_down_reference_core(strix_tp_moe_plan) { return STRIX_ERROR_NOT_IMPLEMENTED; }
strix_status strix_tp_moe_plan_destroy(strix_tp_moe_plan p) {
    if (!p) return STRIX_ERROR_INVALID_ARGUMENT;
    for (strix_weights w : p->retained) --w->plan_refs;
    destroy_plan(p);
    return STRIX_SUCCESS;
}

// ---- SwiGLU plan: hidden_output = SiLU(gate(X)) * up(X), rows 1..8 -----------------------------
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

static strix_status swiglu_shape(strix_context c, const strix_tp_swiglu_desc* d, int& rows, uint64_t& xs,
                                 uint64_t& hs, uint64_t& xb, uint64_t& hb, uint64_t& need) {
    strix_status s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (!d->gate || !d->up || d->gate->owner != c || d->up->owner != c) return STRIX_ERROR_INVALID_ARGUMENT;
    const st::DeviceWeights &g = d->gate->device, &u = d->up->device;
    if (g.inputs != u.inputs || g.outputs != u.outputs || g.codebook != u.codebook) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    if (d->input.rank != 2 || d->input.shape[0] < 1 || d->input.shape[0] > 8) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    rows = (int)d->input.shape[0];
    s = row_view(d->input, rows, g.inputs, xs, xb);
    if (s == STRIX_SUCCESS) s = row_view(d->hidden_output, rows, g.outputs, hs, hb);
    if (s != STRIX_SUCCESS) return s;
    const st::GroupedPlan plan = st::plan_grouped(g.inputs, g.outputs, st::heavier_rate(g.bits, u.bits), 2, c->sm_count);
    need = st::align_up((uint64_t)2 * rows * g.outputs * 4) +
           2 * (plan.counter_bytes_per_problem + plan.partial_bytes_per_problem) + st::align_up(2 * sizeof(st::GroupedProblem));
    return STRIX_SUCCESS;
}

strix_status strix_tp_swiglu_workspace_bytes(strix_context c, const strix_tp_swiglu_desc* d, uint64_t* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = 0;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    int rows; uint64_t xs, hs, xb, hb, need;
    s = swiglu_shape(c, d, rows, xs, hs, xb, hb, need);
    if (s == STRIX_SUCCESS) *out = need;
    return s;
}

strix_status strix_tp_swiglu_plan_create(strix_context c, const strix_tp_swiglu_desc* d, const strix_stream* stream,
                                         strix_tp_swiglu_plan* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    int rows; uint64_t xs, hs, xb, hb, need;
    s = swiglu_shape(c, d, rows, xs, hs, xb, hb, need);
    if (s != STRIX_SUCCESS) return s;
    if (d->workspace_bytes < need) return STRIX_ERROR_INSUFFICIENT_BUFFER;
    if (!d->workspace || reinterpret_cast<uintptr_t>(d->workspace) % kAlign) return STRIX_ERROR_INVALID_ARGUMENT;
    // Optional diagnostics: the gate / up projections land in the caller's contiguous
    // [rows, inter] buffers instead of the workspace.
    const uint64_t diag_need = (uint64_t)rows * d->gate->device.outputs * 4;
    for (float* diag : {d->diagnostic_gate, d->diagnostic_up}) {
        if (!diag) continue;
        if (d->diagnostic_bytes < diag_need) return STRIX_ERROR_INSUFFICIENT_BUFFER;
        if (overlap(diag, diag_need, d->input.data, xb) || overlap(diag, diag_need, d->hidden_output.data, hb) ||
            overlap(diag, diag_need, d->workspace, d->workspace_bytes))
            return STRIX_ERROR_INVALID_ARGUMENT;
        s = device_buffer(c, diag, diag_need, 4);
        if (s != STRIX_SUCCESS) return s;
    }
    if (d->diagnostic_gate && d->diagnostic_up && overlap(d->diagnostic_gate, diag_need, d->diagnostic_up, diag_need))
        return STRIX_ERROR_INVALID_ARGUMENT;
    if (overlap(d->input.data, xb, d->hidden_output.data, hb) || overlap(d->workspace, d->workspace_bytes, d->input.data, xb) ||
        overlap(d->workspace, d->workspace_bytes, d->hidden_output.data, hb))
        return STRIX_ERROR_INVALID_ARGUMENT;
    s = device_buffer(c, d->input.data, xb, 4);
    if (s == STRIX_SUCCESS) s = device_buffer(c, d->hidden_output.data, hb, 4);
    if (s == STRIX_SUCCESS) s = device_buffer(c, d->workspace, d->workspace_bytes, kAlign);
    if (s != STRIX_SUCCESS) return s;
    strix_tp_dense_pair_plan_impl* p = new (std::nothrow) strix_tp_dense_pair_plan_impl;
    if (!p) return STRIX_ERROR_OUT_OF_MEMORY;
    const st::DeviceWeights &g = d->gate->device, &u = d->up->device;
    p->owner = c; p->stream = cs; p->gate = d->gate; p->up = d->up; p->is_swiglu = true;
    p->rows = rows; p->inter = g.outputs; p->inputs = g.inputs; p->codebook = g.codebook;
    p->plan = st::plan_grouped(g.inputs, g.outputs, st::heavier_rate(g.bits, u.bits), 2, c->sm_count);
    Carver carve{static_cast<unsigned char*>(d->workspace)};
    p->g = carve.take<float>((size_t)rows * g.outputs);
    p->u = p->g + (size_t)rows * g.outputs;
    carve.used = st::align_up((size_t)2 * rows * g.outputs * 4);
    if (d->diagnostic_gate) p->g = d->diagnostic_gate;
    if (d->diagnostic_up) p->u = d->diagnostic_up;
    const size_t each = p->plan.counter_bytes_per_problem + p->plan.partial_bytes_per_problem;
    unsigned char* scratch = carve.take<unsigned char>(2 * each);
    p->problems = carve.take<st::GroupedProblem>(2);
    p->hidden = static_cast<float*>(d->hidden_output.data);
    p->hidden_stride = (long long)hs;
    st::GroupedProblem host[2];
    for (int half = 0; half < 2; ++half) {
        fill_problem(host[half], half ? u : g, static_cast<const float*>(d->input.data), (long long)xs, half ? p->u : p->g,
                     g.outputs, reinterpret_cast<unsigned int*>(scratch + half * each),
                     reinterpret_cast<float*>(scratch + half * each + p->plan.counter_bytes_per_problem));
        host[half].rows = rows;
        for (int k = 0; k < rows; ++k) host[half].x_row[k] = host[half].y_row[k] = k;
    }
    cudaError_t e = cudaMemsetAsync(scratch, 0, 2 * each, cs);
    if (e == cudaSuccess) e = cudaMemcpyAsync(p->problems, host, sizeof(host), cudaMemcpyHostToDevice, cs);
    const cudaError_t done = cudaStreamSynchronize(cs);
    if (e != cudaSuccess || done != cudaSuccess) { delete p; return cuda_status(e != cudaSuccess ? e : done); }
    ++d->gate->plan_refs;
    ++d->up->plan_refs;
    *out = p;
    return STRIX_SUCCESS;
}

strix_status strix_tp_swiglu_plan_submit(strix_tp_swiglu_plan p) {
    if (!p || !p->is_swiglu) return STRIX_ERROR_INVALID_ARGUMENT;
    const strix_status s = context_check(p->owner);
    if (s != STRIX_SUCCESS) return s;
    cudaError_t e = st::launch_grouped(p->problems, 2, p->inputs, p->inter, p->codebook, p->plan, p->owner->status,
                                       p->owner->programmatic_launch, p->stream);
    if (e == cudaSuccess)
        e = st::launch_swiglu(p->g, p->u, p->hidden, p->rows, p->inter, p->hidden_stride, p->owner->programmatic_launch,
                              p->stream);
    return cuda_status(e);
}

strix_status strix_tp_swiglu_plan_destroy(strix_tp_swiglu_plan p) {
    if (!p || !p->is_swiglu) return STRIX_ERROR_INVALID_ARGUMENT;
    --p->gate->plan_refs;
    --p->up->plan_refs;
    delete p;
    return STRIX_SUCCESS;
}

}  // extern "C"
