// The prefill driver: the op sequence of the reference's Forward (crates/decide-engine/src/
// forward.rs:1129-1142 encode_chunk, 1191-1254 encode_layer, 1266-1276 encode_mlp, 1312-1328 head)
// over the dc_* kernels, for a batch of packed requests on one stream.
//
// The model object owns the activation buffers (forward.rs:124-180 does the same) and borrows the
// weights. Requests are concatenated row-wise into one M for every GEMM and row kernel; conv, delta
// rule and attention take the per-request row offsets. Nothing is allocated, JIT-compiled or
// tensor-map-encoded by a forward after the first one of a given shape.
#include <algorithm>
#include <array>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "common.cuh"

struct dc_model {
    dc_ctx* ctx = nullptr;
    dc_dims d{};
    std::vector<dc_layer_weights> layers;
    const void* embed = nullptr;
    const float* final_norm = nullptr;
    uint32_t max_rows = 0, max_seqs = 0, max_answers = 0, max_cand = 0;
    uint32_t act_dtype = DC_ACT_F16;   // the context's 16-bit type when the model was created: the type its weights are stored in
    // derived
    uint32_t key_dim = 0, value_dim = 0, conv_dim = 0, lin_in_n = 0, q_dim = 0, kv_dim = 0, att_in_n = 0, p_ld = 0;
    uint32_t gate_cols = 0;   // columns of each of the b and a blocks of the fused Gated DeltaNet projection: gdn_nv rounded up to 16
    // device buffers
    char* arena = nullptr;
    size_t arena_bytes = 0;
    float *x = nullptr, *p = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr, *xs = nullptr, *logits = nullptr,
          *inv_freq = nullptr;
    float* xr = nullptr;      // tensor-parallel shard only: this rank's partial output of a row-split projection, all-reduced in place
    void *h = nullptr, *g = nullptr, *mlp = nullptr, *qo = nullptr, *kc = nullptr, *vc = nullptr;
    uint32_t *ids = nullptr, *pos = nullptr, *seq_start = nullptr, *ans_rows = nullptr, *cand = nullptr, *ncand = nullptr;
    // answer-row buffers of the pruned last layer (forward.rs:1150-1186): normed rows, q|gate projection, q, attention
    // output, MLP intermediate, and per answer row its position in its request and its request's first cache row
    void *hs = nullptr, *qa = nullptr, *ga = nullptr, *mlpa = nullptr;
    float* ps = nullptr;
    uint32_t *ans_pos = nullptr, *ans_kv = nullptr;
    // work skipping (the reference's defaults: both on)
    bool prune = true;      // last layer: everything after K/V for the answer rows only (set_pruning, forward.rs:517-522)
    bool truncate = true;   // each request stops after its last answer row (forward.rs:830-831)
    // Chunked prefill of ONE request and the prefix snapshot (forward.rs:919-942, 645-673): state that outlives a chunk.
    // Per Gated DeltaNet layer the 3 raw conv rows and the recurrent state, per attention layer its own K/V cache.
    struct Carry {
        char* mem = nullptr;
        uint32_t kv_rows = 0;               // rows each K/V cache holds
        std::vector<void*> kc, vc;          // [layer] -> [max_rows, kv_dim] in the 16-bit type (null for linear layers)
        std::vector<float*> conv, state;    // [layer] -> [3, conv_dim], [nv, dv, dk] (null for attention layers)
    } carry, snap;
    // CUDA graphs of the batched forward: one per (rows, requests, longest request, answer rows, switches), captured the first
    // time that shape runs and replayed afterwards on the model's own stream (the caller's stream is joined by events;
    // the legacy default stream cannot be captured). A 603-token forward is ~350 short kernels: replayed as a graph it is
    // no longer bound by the host's enqueue rate.
    bool use_graphs = true;
    cudaStream_t graph_stream = nullptr;
    cudaEvent_t graph_in = nullptr, graph_out = nullptr;
    struct GraphEntry {
        cudaGraphExec_t exec = nullptr;
        uint64_t launches = 0;              // kernels in the graph, for the context's launch count
    };
    std::map<std::array<uint32_t, 6>, GraphEntry> graphs;
    uint32_t chunk_rows = 0;                // 0 = one request runs whole (no carry needed)
    std::vector<uint32_t> snap_ids;         // token ids of the captured prefix; empty = no snapshot
    uint32_t last_route = 0;                // 0 full, 1 from the prefix snapshot, 2 from a cached state
    uint32_t last_start = 0;                // first row the last prefill computed
    // The state cache (forward.rs:704-731, 845-905): on the snapshot route a request whose ids contain the marker leaves
    // the state after the marker here; a later request that starts with exactly those ids runs from the end of them.
    struct StateEntry {
        Carry c;
        std::vector<uint32_t> ids;          // the ids the state was captured from (prefix, state, marker)
        uint64_t id = 0;                    // never reused: tells a replay whether its entry is still here
    };
    std::vector<StateEntry> states;         // most recently used first
    std::vector<Carry> free_states;         // buffers of forgotten entries, kept for the next captures
    uint32_t state_capacity = 2;            // DEFAULT_STATE_ENTRIES (forward.rs:75)
    std::vector<uint32_t> state_marker{550, 39087, 10485, 198};   // STATE_MARKER (forward.rs:70)
    uint64_t next_state_id = 1;
    struct Chunk {
        uint32_t c0, c1, a0, na;            // rows [c0, c1) of the request; its answers are sorted slots [a0, a0 + na)
        bool capture = false;               // the request's state ends with this chunk: keep the carried state after it
    };
    // the batch the last dc_model_prefill left on the device, as it was laid out after truncation
    struct Resident {
        std::vector<uint32_t> given_seq_start;   // what the caller passed
        uint32_t rows = 0, n_seq = 0, max_len = 0, n_ans = 0, given_rows = 0;
        bool single = false;                     // ran through forward_single (chunks / snapshot)
        uint32_t row0 = 0;                       // first row computed (the snapshot's or the cached state's length, or 0)
        uint64_t state_id = 0;                   // the cached state it started from (0: the snapshot, when row0 > 0)
        std::vector<Chunk> chunks;
    } cur;
    // pinned host staging for the host-buffer entry point
    char* host = nullptr;
    size_t host_bytes = 0;
    // per-op profiler (the reference's DECIDE_PROFILE_PERKERNEL table, crates/decide-metal/src/profile.rs:29-101)
    uint32_t layer_limit = 0;  // 0 = all layers
    bool profiling = false;
    struct Span {
        const char* name;
        cudaEvent_t a, b;
    };
    std::vector<Span> spans;
    std::vector<cudaEvent_t> event_pool;
    std::vector<std::pair<std::string, std::pair<double, uint64_t>>> totals;
};

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

bool is_attention_layer(const dc_dims& d, uint32_t l) { return (l + 1) % d.full_attn_interval == 0; }

struct Prof {
    dc_model* m;
    cudaStream_t s;
    const char* name;
    size_t idx = 0;
    Prof(dc_model* m_, cudaStream_t s_, const char* n) : m(m_), s(s_), name(n) {
        if (!m->profiling) return;
        auto get = [&]() {
            if (m->event_pool.empty()) {
                cudaEvent_t e;
                cudaEventCreate(&e);
                return e;
            }
            cudaEvent_t e = m->event_pool.back();
            m->event_pool.pop_back();
            return e;
        };
        dc_model::Span sp{name, get(), get()};
        cudaEventRecord(sp.a, s);
        idx = m->spans.size();
        m->spans.push_back(sp);
    }
    ~Prof() {
        if (m->profiling) cudaEventRecord(m->spans[idx].b, s);
    }
};

#define RUN(name, call)                  \
    do {                                 \
        Prof _p(m, s, name);             \
        int _rc = (call);                \
        if (_rc != DC_OK) return _rc;    \
    } while (0)

// While a forward is being enqueued the context's workspace may not grow: everything was reserved at
// dc_model_create, and an op that asks for more is a refused call, not a hidden free + malloc.
struct FreezeWorkspace {
    dc_ctx* c;
    bool was;
    explicit FreezeWorkspace(dc_ctx* ctx) : c(ctx), was(ctx->workspace_frozen) { c->workspace_frozen = true; }
    ~FreezeWorkspace() { c->workspace_frozen = was; }
};

int forward_device(dc_model* m, cudaStream_t s, uint32_t rows, uint32_t n_seq, uint32_t max_len, uint32_t n_ans) {
    dc_ctx* c = m->ctx;
    const dc_dims& d = m->d;
    DC_REQUIRE(c, c->act_dtype == m->act_dtype, "forward: the context's 16-bit type was changed after dc_model_create (the weights are stored in the type it had then)");
    FreezeWorkspace frozen(c);
    const uint32_t H = d.hidden;
    void* st = s;
    RUN("embed", dc_embed(c, st, m->ids, m->embed, m->x, rows, H));
    const uint32_t n_run = m->layer_limit ? std::min(m->layer_limit, d.n_layers) : d.n_layers;
    // Last-layer pruning applies to a full run that ends in a head over answer rows, when the last layer is full attention.
    // A layer limit (the per-layer residual dump) turns it off: that caller wants every row of the residual.
    // Tensor-parallel shard: the out / down projections see only this rank's input columns, so their outputs are partial
    // sums. They go to `xr`, are all-reduced over the group, and join the residual inside the next norm (`pending`).
    const bool tp = c->tp_world > 1;
    bool pending = false;
    const bool x16 = c->tp_exchange16;   // the partial sums are stored, exchanged and added in the 16-bit type
    auto norm = [&](const float* wn) -> int {
        if (pending) {
            pending = false;
            return x16 ? dc_add16_rmsnorm(c, st, m->x, m->xr, wn, m->h, rows, H, d.eps, 1) : dc_add_rmsnorm(c, st, m->x, m->xr, wn, m->h, rows, H, d.eps, 1);
        }
        return dc_rmsnorm(c, st, m->x, wn, m->h, nullptr, rows, H, H, H, d.eps, 1);
    };
    auto project_back = [&](const char* name, const void* a, const void* wt, uint32_t kk) -> int {
        if (!tp) {
            Prof _p(m, s, name);
            return dc_gemm(c, st, a, wt, m->x, rows, H, kk, kk, kk, H, DC_EPI_ADD_F32, d.swiglu_block);
        }
        {
            Prof _p(m, s, name);
            const int rc = dc_gemm(c, st, a, wt, m->xr, rows, H, kk, kk, kk, H, x16 ? DC_EPI_STORE_BF16 : DC_EPI_STORE_F32, d.swiglu_block);
            if (rc != DC_OK) return rc;
        }
        Prof _p(m, s, "all_reduce");
        pending = true;
        return x16 ? dc_tp_all_reduce_16(c, st, m->xr, static_cast<size_t>(rows) * H) : dc_tp_all_reduce_f32(c, st, m->xr, static_cast<size_t>(rows) * H);
    };
    const bool pruned = m->prune && !tp && m->layer_limit == 0 && n_ans > 0 && is_attention_layer(d, d.n_layers - 1);
    for (uint32_t l = 0; l < n_run; ++l) {
        const dc_layer_weights& w = m->layers[l];
        if (pruned && l + 1 == d.n_layers) {
            // Every row still needs its K and V (the answer rows attend to them); nothing else of a non-answer row is
            // read again. So: norm and the k|v rows of the in-projection for all rows, then q|gate, attention, the output
            // projection and the MLP for the answer rows only (forward.rs:1150-1186).
            const uint32_t qn = (d.attn_gate ? 2 : 1) * m->q_dim;   // q|gate (or q) rows of w_in, then k|v
            const uint32_t kvn = 2 * m->kv_dim;
            const void* w_kv = static_cast<const char*>(w.w_in) + static_cast<size_t>(qn) * H * 2;
            RUN("rmsnorm", dc_rmsnorm(c, st, m->x, w.in_norm, m->h, nullptr, rows, H, H, H, d.eps, 1));
            RUN("gemm_attn_kv", dc_gemm(c, st, m->h, w_kv, m->p, rows, kvn, H, H, H, kvn, DC_EPI_STORE_F32, d.swiglu_block));
            RUN("kv_norm_rope", dc_kv_norm_rope(c, st, m->p, w.k_norm, m->inv_freq, m->kc, m->vc, rows, kvn, 0, m->kv_dim, 0, m->pos, m->max_rows,
                                                d.nkv, d.head_dim, d.rot_dim, d.eps));
            RUN("gather_rows", dc_gather_rows_bf16(c, st, m->h, m->ans_rows, m->hs, n_ans, H));
            RUN("gemm_ans_q", dc_gemm(c, st, m->hs, w.w_in, m->ps, n_ans, qn, H, H, H, qn, DC_EPI_STORE_F32, d.swiglu_block));
            RUN("q_norm_rope", dc_q_norm_rope(c, st, m->ps, w.q_norm, m->inv_freq, m->ans_pos, m->qa, n_ans, qn, d.nq, d.head_dim, d.rot_dim, d.eps));
            RUN("attention_rows", dc_attention_rows(c, st, m->qa, m->kc, m->vc, d.attn_gate ? m->ps + m->q_dim : nullptr, m->ans_pos, m->ans_kv, m->ga,
                                                    n_ans, qn, d.nq, d.nkv, d.head_dim));
            RUN("gather_rows", dc_gather_rows_f32(c, st, m->x, m->ans_rows, m->xs, n_ans, H));
            RUN("gemm_ans_out", dc_gemm(c, st, m->ga, w.w_out, m->xs, n_ans, H, m->q_dim, m->q_dim, m->q_dim, H, DC_EPI_ADD_F32, d.swiglu_block));
            RUN("rmsnorm", dc_rmsnorm(c, st, m->xs, w.post_norm, m->hs, nullptr, n_ans, H, H, H, d.eps, 1));
            RUN("gemm_ans_gate_up", dc_gemm(c, st, m->hs, w.w_gu, m->mlpa, n_ans, 2 * d.inter, H, H, H, d.inter, DC_EPI_SWIGLU_BF16, d.swiglu_block));
            RUN("gemm_ans_down", dc_gemm(c, st, m->mlpa, w.w_down, m->xs, n_ans, H, d.inter, d.inter, d.inter, H, DC_EPI_ADD_F32, d.swiglu_block));
            RUN("final_head", dc_final_head(c, st, m->xs, m->final_norm, m->embed, m->cand, m->ncand, m->logits, n_ans, H, m->max_cand, d.eps));
            return DC_OK;
        }
        RUN("rmsnorm", norm(w.in_norm));
        uint32_t out_k;
        if (!is_attention_layer(d, l)) {
            const uint32_t ld = m->lin_in_n;
            RUN("gemm_gdn_in", dc_gemm(c, st, m->h, w.w_in, m->p, rows, ld, H, H, H, ld, DC_EPI_STORE_F32, d.swiglu_block));
            const float* b = m->p + m->conv_dim + m->value_dim;  // fused order qkv|z|b|a (config.rs:14-17)
            const float* a = b + m->gate_cols;
            if (dc_conv_gated_delta_supported(c)) {
                // conv + SiLU + L2 norm inside the delta rule's first kernel: q, k, v never reach memory
                RUN("gated_delta", dc_conv_gated_delta(c, st, m->p, nullptr, w.conv_w, a, b, w.a_log, w.dt_bias, nullptr, nullptr, m->o, rows, ld, 0,
                                                       d.gdn_nk, d.gdn_nv, d.gdn_dk, d.gdn_dv, m->seq_start, n_seq, max_len));
            } else {
                RUN("conv_silu_l2", dc_conv_silu_l2(c, st, m->p, nullptr, w.conv_w, m->q, m->k, m->v, rows, ld, d.gdn_nk, d.gdn_nv,
                                                    d.gdn_dk, d.gdn_dv, m->seq_start, n_seq, max_len));
                RUN("gated_delta", dc_gated_delta(c, st, m->q, m->k, m->v, a, b, w.a_log, w.dt_bias, nullptr, nullptr, m->o, rows, ld, 0,
                                                  d.gdn_nk, d.gdn_nv, d.gdn_dk, d.gdn_dv, m->seq_start, n_seq, max_len));
            }
            RUN("gated_rmsnorm_silu", dc_gated_rmsnorm_silu(c, st, m->o, m->p + m->conv_dim, w.gnorm, m->g, rows, d.gdn_nv, d.gdn_dv, ld, d.eps));
            out_k = m->value_dim;
        } else {
            const uint32_t ld = m->att_in_n;
            const uint32_t kcol = d.attn_gate ? 2 * m->q_dim : m->q_dim;  // q|gate|k|v or q|k|v (config.rs:25-29)
            const uint32_t vcol = kcol + m->kv_dim;
            RUN("gemm_attn_in", dc_gemm(c, st, m->h, w.w_in, m->p, rows, ld, H, H, H, ld, DC_EPI_STORE_F32, d.swiglu_block));
            RUN("q_norm_rope", dc_q_norm_rope(c, st, m->p, w.q_norm, m->inv_freq, m->pos, m->qo, rows, ld, d.nq, d.head_dim, d.rot_dim, d.eps));
            RUN("kv_norm_rope", dc_kv_norm_rope(c, st, m->p, w.k_norm, m->inv_freq, m->kc, m->vc, rows, ld, kcol, vcol, 0, m->pos,
                                                m->max_rows, d.nkv, d.head_dim, d.rot_dim, d.eps));
            RUN("attention", dc_attention(c, st, m->qo, m->kc, m->vc, d.attn_gate ? m->p + m->q_dim : nullptr, m->pos, m->g, rows, ld, d.nq,
                                          d.nkv, d.head_dim, m->seq_start, n_seq, max_len));
            out_k = m->q_dim;
        }
        if (int rc = project_back("gemm_out", m->g, w.w_out, out_k); rc != DC_OK) return rc;
        RUN("rmsnorm", norm(w.post_norm));
        RUN("gemm_gate_up", dc_gemm(c, st, m->h, w.w_gu, m->mlp, rows, 2 * d.inter, H, H, H, d.inter, DC_EPI_SWIGLU_BF16, d.swiglu_block));
        if (int rc = project_back("gemm_down", m->mlp, w.w_down, d.inter); rc != DC_OK) return rc;
    }
    if (pending)
        RUN("add_partial", x16 ? dc_add16_rmsnorm(c, st, m->x, m->xr, nullptr, nullptr, rows, H, d.eps, 1) : dc_add_rmsnorm(c, st, m->x, m->xr, nullptr, nullptr, rows, H, d.eps, 1));
    if (n_ans && n_run == d.n_layers) {
        RUN("gather_rows", dc_gather_rows_f32(c, st, m->x, m->ans_rows, m->xs, n_ans, H));
        RUN("final_head", dc_final_head(c, st, m->xs, m->final_norm, m->embed, m->cand, m->ncand, m->logits, n_ans, H, m->max_cand, d.eps));
    }
    return DC_OK;
}

// The batched forward, replayed from a CUDA graph when it can be: not while per-op profiling is on (events per op), not
// on a tensor-parallel shard (the collective library's calls are left out of capture), not with a layer limit.
int run_forward(dc_model* m, cudaStream_t s, uint32_t rows, uint32_t n_seq, uint32_t max_len, uint32_t n_ans) {
    dc_ctx* c = m->ctx;
    if (!m->use_graphs || m->profiling || c->tp_world > 1 || m->layer_limit != 0 || !m->graph_stream)
        return forward_device(m, s, rows, n_seq, max_len, n_ans);
    const std::array<uint32_t, 6> key = {rows, n_seq, max_len, n_ans, static_cast<uint32_t>(m->prune) | (c->act_dtype << 1) | (c->gemm_impl << 2) | (c->attn_impl << 3) |
                                                                          (c->delta_impl << 4) | (c->attn_engine << 5) | (c->delta_engine << 6) | (c->delta_split << 7),
                                         0u};
    auto it = m->graphs.find(key);
    if (it == m->graphs.end()) {
        // First time this shape runs: one eager pass (it fills the tensor-map cache and is the result of this call), and a
        // capture of the same enqueue sequence for the calls that follow.
        int rc = forward_device(m, s, rows, n_seq, max_len, n_ans);
        if (rc != DC_OK) return rc;
        if (m->graphs.size() >= 64) return DC_OK;   // a bounded cache; further shapes simply run eagerly
        const uint64_t before = c->launches;
        if (cudaStreamBeginCapture(m->graph_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
            cudaGetLastError();
            return DC_OK;
        }
        rc = forward_device(m, m->graph_stream, rows, n_seq, max_len, n_ans);
        cudaGraph_t graph = nullptr;
        const cudaError_t e = cudaStreamEndCapture(m->graph_stream, &graph);
        dc_model::GraphEntry entry;
        entry.launches = c->launches - before;
        c->launches = before;                        // nothing ran during capture
        if (rc == DC_OK && e == cudaSuccess && graph && cudaGraphInstantiate(&entry.exec, graph, 0) == cudaSuccess) {
            cudaGraphUpload(entry.exec, m->graph_stream);   // device-side resources now, not at the first replay
            cudaStreamSynchronize(m->graph_stream);
            m->graphs.emplace(key, entry);
        } else {
            cudaGetLastError();
        }
        if (graph) cudaGraphDestroy(graph);
        c->last_error.clear();
        return DC_OK;
    }
    cudaError_t e = cudaEventRecord(m->graph_in, s);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(m->graph_stream, m->graph_in, 0);
    if (e == cudaSuccess) e = cudaGraphLaunch(it->second.exec, m->graph_stream);
    if (e == cudaSuccess) e = cudaEventRecord(m->graph_out, m->graph_stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s, m->graph_out, 0);
    if (e != cudaSuccess) return dc_fail(c, DC_CUDA_ERROR, "forward: graph launch failed: %s", cudaGetErrorString(e));
    c->launches += it->second.launches;
    return DC_OK;
}

// Device memory of one carried state; `kv_rows` = rows each K/V cache can hold (0: the model's row capacity). A Carry
// that is too small is released and made again.
bool ensure_carry(dc_model* m, dc_model::Carry& c, uint32_t kv_rows = 0) {
    if (kv_rows == 0) kv_rows = m->max_rows;
    if (c.mem && c.kv_rows >= kv_rows) return true;
    cudaSetDevice(m->ctx->device);
    if (c.mem) {
        cudaFree(c.mem);   // waits for the work that uses it
        c.mem = nullptr;
    }
    const dc_dims& d = m->d;
    const size_t kv = align_up(static_cast<size_t>(kv_rows) * m->kv_dim * 2, 1024), cv = align_up(static_cast<size_t>(3) * m->conv_dim * 4, 1024),
                 st = align_up(static_cast<size_t>(d.gdn_nv) * d.gdn_dv * d.gdn_dk * 4, 1024);
    size_t total = 0;
    for (uint32_t l = 0; l < d.n_layers; ++l) total += is_attention_layer(d, l) ? 2 * kv : cv + st;
    if (cudaMalloc(&c.mem, total) != cudaSuccess) {
        cudaGetLastError();
        c.mem = nullptr;
        c.kv_rows = 0;
        return false;
    }
    c.kv_rows = kv_rows;
    m->ctx->allocs++;
    c.kc.assign(d.n_layers, nullptr);
    c.vc.assign(d.n_layers, nullptr);
    c.conv.assign(d.n_layers, nullptr);
    c.state.assign(d.n_layers, nullptr);
    size_t off = 0;
    for (uint32_t l = 0; l < d.n_layers; ++l) {
        if (is_attention_layer(d, l)) {
            c.kc[l] = c.mem + off;
            c.vc[l] = c.mem + off + kv;
            off += 2 * kv;
        } else {
            c.conv[l] = reinterpret_cast<float*>(c.mem + off);
            c.state[l] = reinterpret_cast<float*>(c.mem + off + cv);
            off += cv + st;
        }
    }
    return true;
}

// Copies the carried state of rows [0, rows) from one Carry to another on the stream (snapshot capture and restore).
int copy_carry(dc_model* m, cudaStream_t s, const dc_model::Carry& from, dc_model::Carry& to, uint32_t rows) {
    const dc_dims& d = m->d;
    cudaError_t e = cudaSuccess;
    for (uint32_t l = 0; l < d.n_layers && e == cudaSuccess; ++l) {
        if (is_attention_layer(d, l)) {
            const size_t bytes = static_cast<size_t>(rows) * m->kv_dim * 2;
            e = cudaMemcpyAsync(to.kc[l], from.kc[l], bytes, cudaMemcpyDeviceToDevice, s);
            if (e == cudaSuccess) e = cudaMemcpyAsync(to.vc[l], from.vc[l], bytes, cudaMemcpyDeviceToDevice, s);
        } else {
            e = cudaMemcpyAsync(to.conv[l], from.conv[l], static_cast<size_t>(3) * m->conv_dim * 4, cudaMemcpyDeviceToDevice, s);
            if (e == cudaSuccess)
                e = cudaMemcpyAsync(to.state[l], from.state[l], static_cast<size_t>(d.gdn_nv) * d.gdn_dv * d.gdn_dk * 4, cudaMemcpyDeviceToDevice, s);
        }
    }
    if (e != cudaSuccess) return dc_fail(m->ctx, DC_CUDA_ERROR, "copying the carried state failed: %s", cudaGetErrorString(e));
    return DC_OK;
}

// Where a request's state ends (state_boundary, forward.rs:1503-1512): one past the first occurrence of `marker` in
// ids[prefix, limit), `limit` being the first answer row; 0 when there is none. Correctness never rests on it: an entry
// serves only ids that start with exactly the ids it was captured from.
uint32_t state_boundary(const uint32_t* ids, uint32_t prefix, const std::vector<uint32_t>& marker, uint32_t limit) {
    const uint32_t n = static_cast<uint32_t>(marker.size());
    if (n == 0 || limit < prefix + n) return 0;
    for (uint32_t i = prefix; i + n <= limit; ++i)
        if (std::equal(marker.begin(), marker.end(), ids + i)) return i + n;
    return 0;
}

// ONE request, chunk by chunk (encode_chunk over chunks(start, end), forward.rs:919-942, 1129-1142): all layers of a chunk,
// then the next chunk. Linear layers carry their conv rows and recurrent state from chunk to chunk; attention layers append
// the chunk's K/V rows to their own cache and attend over rows 0..=position. `row0 > 0` continues from state already in
// `carry` (the restored prefix snapshot or cached state). After a chunk marked `capture` the carried state is copied to
// `capture` (the reference snapshots inside the chunk, forward.rs:869-873; here the chunk ends at the state's boundary). The ids and absolute positions of the whole request are on the device.
int forward_single(dc_model* m, cudaStream_t s, const std::vector<dc_model::Chunk>& chunks, uint32_t n_ans, dc_model::Carry* capture = nullptr) {
    dc_ctx* c = m->ctx;
    const dc_dims& d = m->d;
    const uint32_t H = d.hidden;
    void* st = s;
    DC_REQUIRE(c, c->act_dtype == m->act_dtype, "forward: the context's 16-bit type was changed after dc_model_create");
    DC_REQUIRE(c, c->tp_world <= 1, "forward: chunked prefill and the prefix snapshot are not available on a tensor-parallel shard");
    FreezeWorkspace frozen(c);
    const uint32_t n_run = m->layer_limit ? std::min(m->layer_limit, d.n_layers) : d.n_layers;
    const bool fused = dc_conv_gated_delta_supported(c) != 0;
    for (const dc_model::Chunk& ch : chunks) {
        const uint32_t n = ch.c1 - ch.c0;
        const bool first = ch.c0 == 0;
        RUN("embed", dc_embed(c, st, m->ids + ch.c0, m->embed, m->x, n, H));
        for (uint32_t l = 0; l < n_run; ++l) {
            const dc_layer_weights& w = m->layers[l];
            RUN("rmsnorm", dc_rmsnorm(c, st, m->x, w.in_norm, m->h, nullptr, n, H, H, H, d.eps, 1));
            uint32_t out_k;
            if (!is_attention_layer(d, l)) {
                const uint32_t ld = m->lin_in_n;
                RUN("gemm_gdn_in", dc_gemm(c, st, m->h, w.w_in, m->p, n, ld, H, H, H, ld, DC_EPI_STORE_F32, d.swiglu_block));
                const float* b = m->p + m->conv_dim + m->value_dim;
                const float* a = b + m->gate_cols;
                const float* prev = first ? nullptr : m->carry.conv[l];
                const float* s_in = first ? nullptr : m->carry.state[l];
                if (fused) {
                    RUN("gated_delta", dc_conv_gated_delta(c, st, m->p, prev, w.conv_w, a, b, w.a_log, w.dt_bias, s_in, m->carry.state[l], m->o, n, ld, 1,
                                                           d.gdn_nk, d.gdn_nv, d.gdn_dk, d.gdn_dv, nullptr, 1, n));
                } else {
                    RUN("conv_silu_l2", dc_conv_silu_l2(c, st, m->p, prev, w.conv_w, m->q, m->k, m->v, n, ld, d.gdn_nk, d.gdn_nv, d.gdn_dk, d.gdn_dv, nullptr, 1, n));
                    RUN("gated_delta", dc_gated_delta(c, st, m->q, m->k, m->v, a, b, w.a_log, w.dt_bias, s_in, m->carry.state[l], m->o, n, ld, 1,
                                                      d.gdn_nk, d.gdn_nv, d.gdn_dk, d.gdn_dv, nullptr, 1, n));
                }
                // the 3 raw rows that end this chunk, after the conv has read the old ones (conv.rs:38-46)
                RUN("conv_state_update", dc_conv_state_update(c, st, m->p, prev, m->carry.conv[l], n, ld, m->conv_dim));
                RUN("gated_rmsnorm_silu", dc_gated_rmsnorm_silu(c, st, m->o, m->p + m->conv_dim, w.gnorm, m->g, n, d.gdn_nv, d.gdn_dv, ld, d.eps));
                out_k = m->value_dim;
            } else {
                const uint32_t ld = m->att_in_n;
                const uint32_t kcol = d.attn_gate ? 2 * m->q_dim : m->q_dim;
                RUN("gemm_attn_in", dc_gemm(c, st, m->h, w.w_in, m->p, n, ld, H, H, H, ld, DC_EPI_STORE_F32, d.swiglu_block));
                RUN("q_norm_rope", dc_q_norm_rope(c, st, m->p, w.q_norm, m->inv_freq, m->pos + ch.c0, m->qo, n, ld, d.nq, d.head_dim, d.rot_dim, d.eps));
                RUN("kv_norm_rope", dc_kv_norm_rope(c, st, m->p, w.k_norm, m->inv_freq, m->carry.kc[l], m->carry.vc[l], n, ld, kcol, kcol + m->kv_dim, ch.c0, nullptr,
                                                    m->max_rows, d.nkv, d.head_dim, d.rot_dim, d.eps));
                RUN("attention", dc_attention(c, st, m->qo, m->carry.kc[l], m->carry.vc[l], d.attn_gate ? m->p + m->q_dim : nullptr, m->pos + ch.c0, m->g, n, ld,
                                              d.nq, d.nkv, d.head_dim, nullptr, 1, ch.c1));   // cache rows 0 .. c1 are in use
                out_k = m->q_dim;
            }
            RUN("gemm_out", dc_gemm(c, st, m->g, w.w_out, m->x, n, H, out_k, out_k, out_k, H, DC_EPI_ADD_F32, d.swiglu_block));
            RUN("rmsnorm", dc_rmsnorm(c, st, m->x, w.post_norm, m->h, nullptr, n, H, H, H, d.eps, 1));
            RUN("gemm_gate_up", dc_gemm(c, st, m->h, w.w_gu, m->mlp, n, 2 * d.inter, H, H, H, d.inter, DC_EPI_SWIGLU_BF16, d.swiglu_block));
            RUN("gemm_down", dc_gemm(c, st, m->mlp, w.w_down, m->x, n, H, d.inter, d.inter, d.inter, H, DC_EPI_ADD_F32, d.swiglu_block));
        }
        if (ch.na && n_run == d.n_layers)   // this chunk's answer rows (chunk-relative, sorted) into their slots
            RUN("gather_rows", dc_gather_rows_f32(c, st, m->x, m->ans_rows + ch.a0, m->xs + static_cast<size_t>(ch.a0) * H, ch.na, H));
        if (ch.capture && capture)          // rows 0 .. c1 of every K/V cache and every linear layer's state are final now
            RUN("state_capture", copy_carry(m, s, m->carry, *capture, ch.c1));
    }
    if (n_ans && n_run == d.n_layers)
        RUN("final_head", dc_final_head(c, st, m->xs, m->final_norm, m->embed, m->cand, m->ncand, m->logits, n_ans, H, m->max_cand, d.eps));
    return DC_OK;
}

void collect_profile(dc_model* m) {
    for (auto& sp : m->spans) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, sp.a, sp.b);
        auto it = std::find_if(m->totals.begin(), m->totals.end(), [&](auto& e) { return e.first == sp.name; });
        if (it == m->totals.end()) m->totals.push_back({sp.name, {ms, 1}});
        else {
            it->second.first += ms;
            it->second.second += 1;
        }
        m->event_pool.push_back(sp.a);
        m->event_pool.push_back(sp.b);
    }
    m->spans.clear();
}

}  // namespace

extern "C" {

dc_model* dc_model_create(dc_ctx* ctx, const dc_dims* dims, const dc_layer_weights* layers, const void* embed,
                          const float* final_norm, uint32_t max_rows, uint32_t max_seqs, uint32_t max_answers,
                          uint32_t max_cand) {
    if (!ctx) return nullptr;
    auto fail = [&](const char* msg) -> dc_model* {
        dc_fail(ctx, DC_INVALID_ARG, "dc_model_create: %s", msg);
        return nullptr;
    };
    if (!dims || !layers || !embed || !final_norm) return fail("null argument");
    const dc_dims& d = *dims;
    if (d.hidden % 32 || d.inter % 32 || d.hidden == 0 || d.n_layers == 0) return fail("hidden and intermediate sizes must be multiples of 32");
    if (d.head_dim != 128) return fail("attention head_dim must be 128");
    if (d.gdn_dk != 128 || d.gdn_dv != 128) return fail("Gated DeltaNet head dims must be 128");
    if (d.nkv == 0 || d.nq % d.nkv || d.gdn_nk == 0 || d.gdn_nv % d.gdn_nk) return fail("head counts do not divide");
    if (d.full_attn_interval == 0 || d.swiglu_block != 16) return fail("full_attn_interval must be positive and swiglu_block 16");
    if (d.rot_dim % 8 || d.rot_dim > d.head_dim || d.rot_dim == 0) return fail("rotary dims must be a multiple of 8 within head_dim");
    if (max_rows == 0 || max_seqs == 0 || max_cand == 0) return fail("capacities must be positive");

    dc_model* m = new dc_model();
    m->ctx = ctx;
    m->d = d;
    m->layers.assign(layers, layers + d.n_layers);
    m->embed = embed;
    m->final_norm = final_norm;
    m->max_rows = max_rows;
    m->max_seqs = max_seqs;
    m->max_answers = max_answers ? max_answers : 1;
    m->max_cand = max_cand;
    m->act_dtype = ctx->act_dtype;
    m->key_dim = d.gdn_nk * d.gdn_dk;
    m->value_dim = d.gdn_nv * d.gdn_dv;
    m->conv_dim = 2 * m->key_dim + m->value_dim;
    m->gate_cols = (d.gdn_nv + 15u) / 16u * 16u;
    m->lin_in_n = m->conv_dim + m->value_dim + 2 * m->gate_cols;
    m->q_dim = d.nq * d.head_dim;
    m->kv_dim = d.nkv * d.head_dim;
    m->att_in_n = (d.attn_gate ? 2 : 1) * m->q_dim + 2 * m->kv_dim;
    m->p_ld = std::max(m->lin_in_n, m->att_in_n);
    if (m->lin_in_n % 32) {
        delete m;
        return fail("the fused Gated DeltaNet projection width must be a multiple of 32");
    }

    const size_t R = max_rows, A = m->max_answers;
    struct Want {
        void** ptr;
        size_t bytes;
    };
    std::vector<Want> wants = {
        {reinterpret_cast<void**>(&m->x), R * d.hidden * 4},
        {&m->h, R * d.hidden * 2},
        {reinterpret_cast<void**>(&m->p), R * m->p_ld * 4},
        {reinterpret_cast<void**>(&m->q), R * m->key_dim * 4},
        {reinterpret_cast<void**>(&m->k), R * m->key_dim * 4},
        {reinterpret_cast<void**>(&m->v), R * m->value_dim * 4},
        {reinterpret_cast<void**>(&m->o), R * m->value_dim * 4},
        {&m->g, R * std::max(m->value_dim, m->q_dim) * 2},
        {&m->mlp, R * d.inter * 2},
        {&m->qo, R * m->q_dim * 2},
        {&m->kc, R * m->kv_dim * 2},
        {&m->vc, R * m->kv_dim * 2},
        {reinterpret_cast<void**>(&m->xs), A * d.hidden * 4},
        {reinterpret_cast<void**>(&m->logits), A * max_cand * 4},
        {reinterpret_cast<void**>(&m->inv_freq), (d.rot_dim / 2) * 4},
        {reinterpret_cast<void**>(&m->ids), R * 4},
        {reinterpret_cast<void**>(&m->pos), R * 4},
        {reinterpret_cast<void**>(&m->seq_start), (static_cast<size_t>(max_seqs) + 1) * 4},
        {reinterpret_cast<void**>(&m->ans_rows), A * 4},
        {reinterpret_cast<void**>(&m->cand), A * max_cand * 4},
        {reinterpret_cast<void**>(&m->ncand), A * 4},
        {&m->hs, A * d.hidden * 2},
        {reinterpret_cast<void**>(&m->ps), A * 2 * m->q_dim * 4},
        {&m->qa, A * m->q_dim * 2},
        {&m->ga, A * m->q_dim * 2},
        {&m->mlpa, A * d.inter * 2},
        {reinterpret_cast<void**>(&m->ans_pos), A * 4},
        {reinterpret_cast<void**>(&m->ans_kv), A * 4},
        {reinterpret_cast<void**>(&m->xr), ctx->tp_world > 1 ? R * d.hidden * 4 : 0},
    };
    size_t total = 0;
    for (auto& wnt : wants) total += align_up(wnt.bytes, 1024);
    cudaSetDevice(ctx->device);
    if (cudaMalloc(&m->arena, total) != cudaSuccess) {
        cudaGetLastError();
        delete m;
        dc_fail(ctx, DC_CUDA_ERROR, "dc_model_create: cannot allocate %zu bytes of activations", total);
        return nullptr;
    }
    m->arena_bytes = total;
    size_t off = 0;
    for (auto& wnt : wants) {
        *wnt.ptr = m->arena + off;
        off += align_up(wnt.bytes, 1024);
    }
    ctx->allocs++;
    // scratch of the chunked delta rule and of the attention's transposed V for the largest batch, so that no forward
    // allocates; every kernel variant opted in to its shared memory now (Gemm::warm_up's role, gemm.rs:89-107)
    void* ws = nullptr;
    size_t ws_bytes = std::max(dc_gated_delta_scratch_bytes(max_rows, max_seqs, d.gdn_nv), dc_attention_tc_scratch_bytes(max_rows, max_seqs, d.nkv));
    for (uint32_t r = 1; r <= m->max_answers; ++r)   // the answer rows' attention slices the keys more finely the fewer rows there are
        ws_bytes = std::max(ws_bytes, dc_attention_rows_scratch_bytes(ctx, r, d.nq, d.nkv));
    if (dc_get_workspace(ctx, ws_bytes, "dc_model_create", &ws) != DC_OK ||
        dc_warm_up(ctx) != DC_OK) {
        cudaFree(m->arena);
        delete m;
        return nullptr;
    }
    // RoPE inverse frequencies in fp32, as the reference and HF compute them (config.rs:44-46)
    std::vector<float> f(d.rot_dim / 2);
    for (uint32_t i = 0; i < d.rot_dim / 2; ++i)
        f[i] = 1.0f / powf(d.rope_theta, static_cast<float>(2 * i) / static_cast<float>(d.rot_dim));
    cudaMemcpy(m->inv_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice);
    m->host_bytes = align_up(R * 4, 64) * 2 + align_up((max_seqs + 1) * 4, 64) + align_up(A * 4, 64) * 4 + align_up(A * max_cand * 4, 64) * 2;
    if (cudaMallocHost(&m->host, m->host_bytes) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(m->arena);
        delete m;
        dc_fail(ctx, DC_CUDA_ERROR, "dc_model_create: cannot allocate pinned staging");
        return nullptr;
    }
    ctx->allocs++;
    if (cudaStreamCreateWithFlags(&m->graph_stream, cudaStreamNonBlocking) != cudaSuccess || cudaEventCreateWithFlags(&m->graph_in, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&m->graph_out, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        m->graph_stream = nullptr;      // graphs are an optimisation: without the stream the forward runs eagerly
    }
    if (const char* g = getenv("DECIDE_GRAPHS")) m->use_graphs = !(g[0] == '0' && g[1] == 0);
    return m;
}

void dc_model_destroy(dc_model* m) {
    if (!m) return;
    cudaSetDevice(m->ctx->device);
    collect_profile(m);
    for (auto e : m->event_pool) cudaEventDestroy(e);
    for (auto& g : m->graphs) cudaGraphExecDestroy(g.second.exec);
    if (m->graph_in) cudaEventDestroy(m->graph_in);
    if (m->graph_out) cudaEventDestroy(m->graph_out);
    if (m->graph_stream) cudaStreamDestroy(m->graph_stream);
    if (m->arena) cudaFree(m->arena);
    if (m->carry.mem) cudaFree(m->carry.mem);
    if (m->snap.mem) cudaFree(m->snap.mem);
    for (auto& e : m->states) cudaFree(e.c.mem);
    for (auto& c : m->free_states) cudaFree(c.mem);
    if (m->host) cudaFreeHost(m->host);
    delete m;
}

size_t dc_model_activation_bytes(dc_model* m) { return m ? m->arena_bytes : 0; }

int dc_model_set_layer_limit(dc_model* m, uint32_t n) {
    if (!m) return DC_INVALID_ARG;
    m->layer_limit = n;
    return DC_OK;
}

int dc_model_set_profiling(dc_model* m, uint32_t on) {
    if (!m) return DC_INVALID_ARG;
    m->profiling = on != 0;
    return DC_OK;
}

// Writes "name total_ms calls" lines, largest first; returns the length needed.
size_t dc_model_profile(dc_model* m, char* buf, size_t len) {
    if (!m) return 0;
    cudaDeviceSynchronize();
    collect_profile(m);
    auto rows = m->totals;
    std::sort(rows.begin(), rows.end(), [](auto& a, auto& b) { return a.second.first > b.second.first; });
    std::string out;
    char line[160];
    for (auto& r : rows) {
        snprintf(line, sizeof line, "%s %.4f %llu\n", r.first.c_str(), r.second.first, static_cast<unsigned long long>(r.second.second));
        out += line;
    }
    if (buf && len) snprintf(buf, len, "%s", out.c_str());
    m->totals.clear();
    return out.size();
}

static int check_batch(dc_model* m, uint32_t n_seq, const uint32_t* seq_start, uint32_t n_ans, uint32_t* rows, uint32_t* max_len) {
    dc_ctx* ctx = m->ctx;
    DC_REQUIRE(ctx, n_seq >= 1 && n_seq <= m->max_seqs, "forward: %u requests (capacity %u)", n_seq, m->max_seqs);
    DC_REQUIRE(ctx, seq_start[0] == 0, "forward: seq_start[0] must be 0");
    uint32_t ml = 0;
    for (uint32_t i = 0; i < n_seq; ++i) {
        DC_REQUIRE(ctx, seq_start[i + 1] > seq_start[i], "forward: request %u is empty", i);
        ml = std::max(ml, seq_start[i + 1] - seq_start[i]);
    }
    *rows = seq_start[n_seq];
    *max_len = ml;
    DC_REQUIRE(ctx, *rows <= m->max_rows, "forward: %u rows (capacity %u)", *rows, m->max_rows);
    DC_REQUIRE(ctx, n_ans <= m->max_answers, "forward: %u answer rows (capacity %u)", n_ans, m->max_answers);
    return DC_OK;
}

// Whole prefill with HOST buffers: copies ids / offsets / answers in, runs every layer, copies the
// candidate logits out and waits. The analogue of Forward::logits (forward.rs:704-731) for a batch.
//
// Tail truncation (forward.rs:830-831): nothing after a request's last answer row can reach a logit (the model is
// causal and no state is kept), so each request is packed only up to that row; answer rows are renumbered to
// match. A request without answer rows is kept whole.
int dc_model_prefill(dc_model* m, void* stream, const uint32_t* ids, const uint32_t* seq_start, uint32_t n_seq,
                     const uint32_t* ans_rows, const uint32_t* cand, const uint32_t* ncand, uint32_t n_ans, float* logits) {
    if (!m) return DC_INVALID_ARG;
    dc_ctx* ctx = m->ctx;
    DC_REQUIRE(ctx, ids && seq_start && (n_ans == 0 || (ans_rows && cand && ncand && logits)), "prefill: null argument");
    uint32_t given_rows = 0, max_len = 0;
    int rc = check_batch(m, n_seq, seq_start, n_ans, &given_rows, &max_len);
    if (rc != DC_OK) return rc;
    for (uint32_t i = 0; i < n_ans; ++i) {
        DC_REQUIRE(ctx, ans_rows[i] < given_rows, "prefill: answer row %u is past the %u rows", ans_rows[i], given_rows);
        DC_REQUIRE(ctx, ncand[i] >= 1 && ncand[i] <= m->max_cand, "prefill: answer %u has %u candidates (1..%u)", i, ncand[i], m->max_cand);
        for (uint32_t j = 0; j < ncand[i]; ++j)
            DC_REQUIRE(ctx, cand[static_cast<size_t>(i) * m->max_cand + j] < m->d.vocab, "prefill: candidate id out of the vocabulary");
    }
    for (uint32_t i = 0; i < given_rows; ++i) DC_REQUIRE(ctx, ids[i] < m->d.vocab, "prefill: token id %u out of the vocabulary", ids[i]);

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // stage through pinned memory: ids, positions, offsets, answers
    char* hp = m->host;
    auto take = [&](size_t bytes) {
        char* r = hp;
        hp += align_up(bytes, 64);
        return r;
    };
    uint32_t* h_ids = reinterpret_cast<uint32_t*>(take(static_cast<size_t>(m->max_rows) * 4));
    uint32_t* h_pos = reinterpret_cast<uint32_t*>(take(static_cast<size_t>(m->max_rows) * 4));
    uint32_t* h_seq = reinterpret_cast<uint32_t*>(take((static_cast<size_t>(m->max_seqs) + 1) * 4));
    uint32_t* h_ans = reinterpret_cast<uint32_t*>(take(static_cast<size_t>(m->max_answers) * 4));
    uint32_t* h_ncand = reinterpret_cast<uint32_t*>(take(static_cast<size_t>(m->max_answers) * 4));
    uint32_t* h_apos = reinterpret_cast<uint32_t*>(take(static_cast<size_t>(m->max_answers) * 4));
    uint32_t* h_akv = reinterpret_cast<uint32_t*>(take(static_cast<size_t>(m->max_answers) * 4));
    uint32_t* h_cand = reinterpret_cast<uint32_t*>(take(static_cast<size_t>(m->max_answers) * m->max_cand * 4));
    float* h_logits = reinterpret_cast<float*>(take(static_cast<size_t>(m->max_answers) * m->max_cand * 4));

    // request of each answer row, and each request's length after truncation
    std::vector<uint32_t> ans_seq(n_ans), keep(n_seq);
    for (uint32_t i = 0; i < n_seq; ++i) keep[i] = m->truncate && m->layer_limit == 0 && n_ans ? 0u : seq_start[i + 1] - seq_start[i];
    for (uint32_t i = 0; i < n_ans; ++i) {
        const uint32_t sq = static_cast<uint32_t>(std::upper_bound(seq_start, seq_start + n_seq + 1, ans_rows[i]) - seq_start) - 1u;
        ans_seq[i] = sq;
        keep[sq] = std::max(keep[sq], ans_rows[i] - seq_start[sq] + 1u);
    }
    uint32_t rows = 0;
    max_len = 0;
    for (uint32_t i = 0; i < n_seq; ++i) {
        if (keep[i] == 0) keep[i] = seq_start[i + 1] - seq_start[i];   // no answer row in this request: kept whole
        h_seq[i] = rows;
        memcpy(h_ids + rows, ids + seq_start[i], static_cast<size_t>(keep[i]) * 4);
        for (uint32_t r = 0; r < keep[i]; ++r) h_pos[rows + r] = r;
        rows += keep[i];
        max_len = std::max(max_len, keep[i]);
    }
    h_seq[n_seq] = rows;
    for (uint32_t i = 0; i < n_ans; ++i) {
        h_apos[i] = ans_rows[i] - seq_start[ans_seq[i]];
        h_akv[i] = h_seq[ans_seq[i]];
        h_ans[i] = h_akv[i] + h_apos[i];
    }
    if (n_ans) {
        memcpy(h_ncand, ncand, static_cast<size_t>(n_ans) * 4);
        memcpy(h_cand, cand, static_cast<size_t>(n_ans) * m->max_cand * 4);
    }
    // One request may run chunk by chunk and / or start from the prefix snapshot (Forward's plan: Full | Snapshot,
    // forward.rs:708-729). The snapshot serves a request that begins with the captured ids, is longer than them, and has
    // every answer row past them.
    const uint32_t P = static_cast<uint32_t>(m->snap_ids.size());
    bool from_snapshot = n_seq == 1 && P > 0 && rows > P && m->layer_limit == 0 && std::equal(m->snap_ids.begin(), m->snap_ids.end(), h_ids);
    uint32_t first_row = rows;
    for (uint32_t i = 0; i < n_ans; ++i) first_row = std::min(first_row, h_ans[i]);
    from_snapshot = from_snapshot && first_row >= P;
    // On the snapshot route: a follow-up runs from the longest cached state its ids start with (Plan::Hit); a request with
    // a new state captures it at the boundary the marker gives (Plan::Capture), forward.rs:708-729.
    int hit = -1;
    uint32_t boundary = 0;
    if (from_snapshot && n_ans > 0) {
        for (size_t i = 0; i < m->states.size(); ++i) {
            const auto& e = m->states[i];
            if (e.ids.size() <= first_row && std::equal(e.ids.begin(), e.ids.end(), h_ids) &&
                (hit < 0 || e.ids.size() > m->states[hit].ids.size()))
                hit = static_cast<int>(i);
        }
        if (hit < 0 && m->state_capacity > 0) boundary = state_boundary(h_ids, P, m->state_marker, first_row);
    }
    const uint32_t row0 = hit >= 0 ? static_cast<uint32_t>(m->states[hit].ids.size()) : from_snapshot ? P : 0u;
    const bool single = n_seq == 1 && (m->chunk_rows > 0 || from_snapshot);
    std::vector<uint32_t> order(n_ans);          // sorted slot -> the caller's answer index
    std::vector<dc_model::Chunk> chunks;
    if (single) {
        for (uint32_t i = 0; i < n_ans; ++i) order[i] = i;
        std::stable_sort(order.begin(), order.end(), [&](uint32_t x, uint32_t y) { return h_ans[x] < h_ans[y]; });
        const uint32_t step = m->chunk_rows ? m->chunk_rows : rows - row0;
        uint32_t slot = 0;
        for (uint32_t c0 = row0; c0 < rows;) {
            dc_model::Chunk ch{c0, std::min(rows, c0 + step), slot, 0};
            if (boundary > c0 && boundary <= ch.c1) {   // the state ends inside this chunk: end the chunk there
                ch.c1 = boundary;
                ch.capture = true;
            }
            c0 = ch.c1;
            while (slot < n_ans && h_ans[order[slot]] < ch.c1) ++slot;
            ch.na = slot - ch.a0;
            chunks.push_back(ch);
        }
        // answers in sorted order: chunk-relative rows, candidates permuted alike
        std::vector<uint32_t> rel(n_ans);
        for (const auto& ch : chunks)
            for (uint32_t a = ch.a0; a < ch.a0 + ch.na; ++a) rel[a] = h_ans[order[a]] - ch.c0;
        for (uint32_t a = 0; a < n_ans; ++a) {
            h_ncand[a] = ncand[order[a]];
            memcpy(h_cand + static_cast<size_t>(a) * m->max_cand, cand + static_cast<size_t>(order[a]) * m->max_cand, static_cast<size_t>(m->max_cand) * 4);
        }
        memcpy(h_ans, rel.data(), static_cast<size_t>(n_ans) * 4);
    }
    m->last_route = hit >= 0 ? 2u : from_snapshot ? 1u : 0u;
    m->last_start = row0;
    m->cur.single = single;
    m->cur.row0 = row0;
    m->cur.state_id = hit >= 0 ? m->states[hit].id : 0;
    m->cur.chunks = chunks;
    m->cur.given_seq_start.assign(seq_start, seq_start + n_seq + 1);
    m->cur.rows = rows;
    m->cur.n_seq = n_seq;
    m->cur.max_len = max_len;
    m->cur.n_ans = n_ans;
    m->cur.given_rows = given_rows;

    cudaError_t e = cudaMemcpyAsync(m->ids, h_ids, static_cast<size_t>(rows) * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->pos, h_pos, static_cast<size_t>(rows) * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->seq_start, h_seq, (static_cast<size_t>(n_seq) + 1) * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess && n_ans) e = cudaMemcpyAsync(m->ans_rows, h_ans, static_cast<size_t>(n_ans) * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess && n_ans) e = cudaMemcpyAsync(m->ans_pos, h_apos, static_cast<size_t>(n_ans) * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess && n_ans) e = cudaMemcpyAsync(m->ans_kv, h_akv, static_cast<size_t>(n_ans) * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess && n_ans) e = cudaMemcpyAsync(m->ncand, h_ncand, static_cast<size_t>(n_ans) * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess && n_ans) e = cudaMemcpyAsync(m->cand, h_cand, static_cast<size_t>(n_ans) * m->max_cand * 4, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "prefill: host-to-device copy failed: %s", cudaGetErrorString(e));

    dc_model::StateEntry fresh;   // Plan::Capture: new buffers, a forgotten entry's, or the least recently used entry's
    if (boundary) {
        if (!m->free_states.empty()) {
            fresh.c = m->free_states.back();
            m->free_states.pop_back();
        } else if (m->states.size() >= m->state_capacity) {
            fresh.c = m->states.back().c;
            m->states.pop_back();
        }
        if (!ensure_carry(m, fresh.c, boundary)) return dc_fail(ctx, DC_CUDA_ERROR, "prefill: cannot allocate a state-cache entry of %u rows", boundary);
        fresh.ids.assign(h_ids, h_ids + boundary);
        fresh.id = m->next_state_id++;
    }
    if (single) {
        if (hit >= 0) rc = copy_carry(m, s, m->states[hit].c, m->carry, row0);
        else if (from_snapshot) rc = copy_carry(m, s, m->snap, m->carry, P);
        if (rc == DC_OK) rc = forward_single(m, s, chunks, n_ans, boundary ? &fresh.c : nullptr);
    } else {
        rc = run_forward(m, s, rows, n_seq, max_len, n_ans);
    }
    if (rc == DC_OK && n_ans) {
        e = cudaMemcpyAsync(h_logits, m->logits, static_cast<size_t>(n_ans) * m->max_cand * 4, cudaMemcpyDeviceToHost, s);
        if (e != cudaSuccess) rc = dc_fail(ctx, DC_CUDA_ERROR, "prefill: device-to-host copy failed: %s", cudaGetErrorString(e));
    }
    if (rc == DC_OK) rc = dc_check_status(ctx, s);  // synchronises
    if (rc != DC_OK) {
        if (fresh.c.mem) m->free_states.push_back(fresh.c);   // its contents are unknown; its buffers serve the next capture
        return rc;
    }
    if (boundary) {                       // the new state is the most recently used
        m->cur.state_id = 0;              // a replay of this request starts from the snapshot again
        m->states.insert(m->states.begin(), std::move(fresh));
    } else if (hit > 0) {
        std::rotate(m->states.begin(), m->states.begin() + hit, m->states.begin() + hit + 1);
    }
    if (n_ans) {
        if (single) {   // back from sorted slots to the caller's order
            for (uint32_t a = 0; a < n_ans; ++a)
                memcpy(logits + static_cast<size_t>(order[a]) * m->max_cand, h_logits + static_cast<size_t>(a) * m->max_cand, static_cast<size_t>(m->max_cand) * 4);
        } else {
            memcpy(logits, h_logits, static_cast<size_t>(n_ans) * m->max_cand * 4);
        }
        // non-finite logits are an error, as forward.rs:906-913
        for (uint32_t i = 0; i < n_ans; ++i)
            for (uint32_t j = 0; j < ncand[i]; ++j)
                if (!std::isfinite(logits[static_cast<size_t>(i) * m->max_cand + j]))
                    return dc_fail(ctx, DC_CUDA_ERROR, "prefill: non-finite logit for answer %u candidate %u", i, j);
    }
    return DC_OK;
}

// The same pass with inputs already resident in the model's device buffers (set by a previous
// dc_model_prefill of the same batch): enqueues only, no copies, no synchronisation. The batch runs as that
// prefill laid it out (truncated to each request's last answer row when truncation was on).
int dc_model_forward_resident(dc_model* m, void* stream, const uint32_t* seq_start, uint32_t n_seq, uint32_t n_ans) {
    if (!m) return DC_INVALID_ARG;
    dc_ctx* ctx = m->ctx;
    DC_REQUIRE(ctx, seq_start, "forward_resident: null argument");
    DC_REQUIRE(ctx, m->cur.n_seq == n_seq && m->cur.n_ans == n_ans && m->cur.given_seq_start.size() == static_cast<size_t>(n_seq) + 1 &&
                        std::equal(seq_start, seq_start + n_seq + 1, m->cur.given_seq_start.begin()),
               "forward_resident: this is not the batch the last dc_model_prefill left on the device");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (m->cur.single) {
        if (m->cur.row0) {
            const dc_model::Carry* from = &m->snap;
            if (m->cur.state_id) {
                from = nullptr;
                for (const auto& e : m->states)
                    if (e.id == m->cur.state_id) from = &e.c;
                DC_REQUIRE(ctx, from, "forward_resident: the cached state the last dc_model_prefill started from is no longer held");
            }
            const int rc = copy_carry(m, s, *from, m->carry, m->cur.row0);
            if (rc != DC_OK) return rc;
        }
        return forward_single(m, s, m->cur.chunks, n_ans);
    }
    return run_forward(m, s, m->cur.rows, n_seq, m->cur.max_len, n_ans);
}

// Forward::set_chunk (forward.rs:504-510): a single request runs in chunks of at most `rows` rows, all layers of a chunk
// before the next, with the linear layers' state and the attention layers' K/V carried across (0 = whole requests).
int dc_model_set_chunk(dc_model* m, uint32_t rows) {
    if (!m) return DC_INVALID_ARG;
    if (rows && !ensure_carry(m, m->carry)) return dc_fail(m->ctx, DC_CUDA_ERROR, "dc_model_set_chunk: cannot allocate the carried state");
    m->chunk_rows = rows;
    return DC_OK;
}

// Forward::build_snapshot (forward.rs:645-673): runs the constant prefix once and keeps every layer's state after it.
// n = 0 drops the snapshot.
int dc_model_build_snapshot(dc_model* m, void* stream, const uint32_t* prefix_ids, uint32_t n) {
    if (!m) return DC_INVALID_ARG;
    dc_ctx* ctx = m->ctx;
    m->snap_ids.clear();
    dc_model_forget_states(m);
    if (n == 0) return DC_OK;
    DC_REQUIRE(ctx, prefix_ids && n < m->max_rows, "build_snapshot: %u prefix rows (capacity %u)", n, m->max_rows);
    for (uint32_t i = 0; i < n; ++i) DC_REQUIRE(ctx, prefix_ids[i] < m->d.vocab, "build_snapshot: token id %u out of the vocabulary", prefix_ids[i]);
    if (!ensure_carry(m, m->carry) || !ensure_carry(m, m->snap)) return dc_fail(ctx, DC_CUDA_ERROR, "build_snapshot: cannot allocate the carried state");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    std::vector<uint32_t> pos(n);
    for (uint32_t i = 0; i < n; ++i) pos[i] = i;
    cudaError_t e = cudaMemcpyAsync(m->ids, prefix_ids, static_cast<size_t>(n) * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m->pos, pos.data(), static_cast<size_t>(n) * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);   // the staging vectors are pageable
    if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "build_snapshot: copy failed: %s", cudaGetErrorString(e));
    std::vector<dc_model::Chunk> chunks;
    const uint32_t step = m->chunk_rows ? m->chunk_rows : n;
    for (uint32_t c0 = 0; c0 < n; c0 += step) chunks.push_back({c0, std::min(n, c0 + step), 0, 0});
    const uint32_t limit = m->layer_limit;
    m->layer_limit = 0;
    int rc = forward_single(m, s, chunks, 0);
    m->layer_limit = limit;
    if (rc == DC_OK) rc = copy_carry(m, s, m->carry, m->snap, n);
    if (rc == DC_OK) rc = dc_check_status(ctx, s);
    if (rc != DC_OK) return rc;
    m->snap_ids.assign(prefix_ids, prefix_ids + n);
    m->cur = dc_model::Resident();   // the device no longer holds a batch
    return DC_OK;
}

// 0: the last dc_model_prefill ran every row; 1: it started from the prefix snapshot; 2: from a cached state (Route,
// forward.rs:196-206). dc_model_last_start: the first row it computed (last_start, forward.rs:686-692).
uint32_t dc_model_last_route(dc_model* m) { return m ? m->last_route : 0; }
uint32_t dc_model_last_start(dc_model* m) { return m ? m->last_start : 0; }

// Forward::set_state_cache (forward.rs:735-744): hold up to `entries` states (at most DC_MAX_STATE_ENTRIES; 0 = off).
// Shrinking evicts the least recently used entries and releases their memory.
int dc_model_set_state_cache(dc_model* m, uint32_t entries) {
    if (!m) return DC_INVALID_ARG;
    DC_REQUIRE(m->ctx, entries <= DC_MAX_STATE_ENTRIES, "a state cache of %u entries; at most %u", entries, DC_MAX_STATE_ENTRIES);
    cudaSetDevice(m->ctx->device);
    m->state_capacity = entries;
    while (m->states.size() > entries) {
        cudaFree(m->states.back().c.mem);
        m->states.pop_back();
    }
    while (m->states.size() + m->free_states.size() > entries) {
        cudaFree(m->free_states.back().mem);
        m->free_states.pop_back();
    }
    return DC_OK;
}

// Forward::forget_states (forward.rs:746-752): every cached state is forgotten; the buffers serve the next captures.
void dc_model_forget_states(dc_model* m) {
    if (!m) return;
    for (auto& e : m->states) m->free_states.push_back(e.c);
    m->states.clear();
}

uint32_t dc_model_state_cache_capacity(dc_model* m) { return m ? m->state_capacity : 0; }

// Forward::cached_states (forward.rs:759-763): the length in tokens of each cached state, most recently used first. Writes
// at most `cap` lengths and returns how many states are held.
uint32_t dc_model_cached_states(dc_model* m, uint32_t* lens, uint32_t cap) {
    if (!m) return 0;
    for (size_t i = 0; i < m->states.size() && i < cap && lens; ++i) lens[i] = static_cast<uint32_t>(m->states[i].ids.size());
    return static_cast<uint32_t>(m->states.size());
}

// Forward::set_state_marker (forward.rs:765-772): the token ids that end a request's state. Empties the cache.
int dc_model_set_state_marker(dc_model* m, const uint32_t* ids, uint32_t n) {
    if (!m) return DC_INVALID_ARG;
    DC_REQUIRE(m->ctx, ids && n > 0, "an empty state marker");
    m->state_marker.assign(ids, ids + n);
    dc_model_forget_states(m);
    return DC_OK;
}

// on = 0: every forward is enqueued kernel by kernel; on = 1 (default; DECIDE_GRAPHS=0 turns it off at creation): a batched
// forward of a shape seen before is replayed from its CUDA graph.
int dc_model_set_graphs(dc_model* m, uint32_t on) {
    if (!m) return DC_INVALID_ARG;
    m->use_graphs = on != 0;
    return DC_OK;
}
size_t dc_model_graph_count(dc_model* m) { return m ? m->graphs.size() : 0; }

int dc_model_set_pruning(dc_model* m, uint32_t on) {
    if (!m) return DC_INVALID_ARG;
    m->prune = on != 0;
    return DC_OK;
}

int dc_model_set_truncation(dc_model* m, uint32_t on) {
    if (!m) return DC_INVALID_ARG;
    m->truncate = on != 0;
    return DC_OK;
}

// Rows the last dc_model_prefill actually ran (after truncation), for throughput accounting.
uint32_t dc_model_resident_rows(dc_model* m) { return m ? m->cur.rows : 0; }

// Device address of a named activation buffer, for per-layer parity checks
// (the reference's debug_layers, forward.rs:778-797).
void* dc_model_buffer(dc_model* m, const char* name) {
    if (!m || !name) return nullptr;
    const std::string n(name);
    if (n == "x") return m->x;
    if (n == "h") return m->h;
    if (n == "p") return m->p;
    if (n == "g") return m->g;
    if (n == "mlp") return m->mlp;
    if (n == "logits") return m->logits;
    if (n == "xs") return m->xs;
    return nullptr;
}

// Synchronous copy of the first `bytes` bytes of a named activation buffer to host memory.
int dc_model_read_buffer(dc_model* m, const char* name, void* dst, size_t bytes) {
    if (!m) return DC_INVALID_ARG;
    void* src = dc_model_buffer(m, name);
    if (!src || !dst) return dc_fail(m->ctx, DC_INVALID_ARG, "dc_model_read_buffer: unknown buffer or null destination");
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return dc_fail(m->ctx, DC_CUDA_ERROR, "dc_model_read_buffer: %s", cudaGetErrorString(e));
    return DC_OK;
}

}  // extern "C"
