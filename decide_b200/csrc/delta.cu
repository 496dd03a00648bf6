// Gated delta rule (the Gated-DeltaNet recurrence), fp32 throughout.
// Replaces kernels/delta.metal and delta_fast.metal; spec cpu_ref.rs:101-129:
//   g = exp(-exp(A_log) * softplus(a + dt_bias)),  beta = sigmoid(b)
//   S <- g S;  kv = S k;  delta = (v - kv) beta;  S <- S + k (x) delta;  o = S q
// with the state S[h] stored [dv][dk].
//
// This file holds the SEQUENTIAL kernel, the reference's own algorithm (delta.metal, delta_fast.metal),
// kept as the baseline (DECIDE_DELTA=baseline) that bisects the chunked kernel of delta_chunk.cu.
// A group of DKS lanes owns one value column of one head and keeps that state
// row in registers (128/DKS values per lane), so the two dot products per token are in-register
// FMA chains plus log2(DKS) shuffles. Tokens are staged through shared memory 16 at a time. The
// value columns of all heads and sequences run in parallel; DKS trades per-thread work for more
// threads when there are few sequences.
#include "common.cuh"

size_t dc_delta_chunk_scratch_bytes(uint32_t t, uint32_t n_seq, uint32_t nv);
int dc_gated_delta_chunked(dc_ctx* ctx, cudaStream_t s, const float* q, const float* k, const float* v, const float* a, const float* b,
                           const float* a_log, const float* dt_bias, const float* state_in, float* state_out, float* o, uint32_t t,
                           uint32_t ldab, uint32_t write_state, uint32_t nk, uint32_t nv, const uint32_t* seq_start, uint32_t n_seq,
                           uint32_t max_len, uint32_t split, const float* praw, uint32_t ldp, const float* conv_w, const float* conv_prev);

namespace {

using namespace dc;

constexpr int kThreads = 128;
constexpr int kGroup = 16;  // tokens staged per shared-memory refill

template <int DKS>
__global__ void __launch_bounds__(kThreads)
gated_delta_seq_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                       const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ a_log,
                       const float* __restrict__ dt_bias, const float* state_in, float* state_out,
                       float* __restrict__ o, uint32_t t, uint32_t ldab, uint32_t nk, uint32_t nv, uint32_t write_state,
                       const uint32_t* __restrict__ seq_start) {
    constexpr int COLS = kThreads / DKS;   // value columns per block
    constexpr int NV4 = 32 / DKS;          // float4 of the state row per lane
    __shared__ float4 ks[kGroup][32];
    __shared__ float4 qs[kGroup][32];
    __shared__ float vs[kGroup][COLS];
    __shared__ float gs[kGroup], bs[kGroup];

    const uint32_t seq = blockIdx.z, h = blockIdx.y;
    const uint32_t hk = h / (nv / nk);
    const uint32_t row_lo = seq_start ? seq_start[seq] : 0u;
    const uint32_t len = seq_start ? seq_start[seq + 1] - row_lo : t;
    const int part = threadIdx.x % DKS;
    const uint32_t col = blockIdx.x * COLS + threadIdx.x / DKS;

    // lane `part` holds float4 number part + DKS*j (j < NV4) of the state row: consecutive lanes read
    // consecutive float4 of k and q from shared memory (no bank conflicts)
    float4 S[NV4];
    const size_t srow = ((static_cast<size_t>(seq) * nv + h) * 128 + col) * 128;
#pragma unroll
    for (int j = 0; j < NV4; ++j)
        S[j] = state_in ? reinterpret_cast<const float4*>(state_in + srow)[part + DKS * j] : make_float4(0.f, 0.f, 0.f, 0.f);

    const float neg_a = -expf(a_log[h]);
    const float dtb = dt_bias[h];

    for (uint32_t s0 = 0; s0 < len; s0 += kGroup) {
        const uint32_t n = min(static_cast<uint32_t>(kGroup), len - s0);
        __syncthreads();  // the previous group has been consumed
        for (uint32_t e = threadIdx.x; e < n * 32; e += kThreads) {
            const uint32_t i = e >> 5, c = e & 31;
            const size_t row = row_lo + s0 + i;
            ks[i][c] = reinterpret_cast<const float4*>(k + (row * nk + hk) * 128)[c];
            qs[i][c] = reinterpret_cast<const float4*>(q + (row * nk + hk) * 128)[c];
        }
        for (uint32_t e = threadIdx.x; e < n * COLS; e += kThreads) {
            const uint32_t i = e / COLS, c = e % COLS;
            vs[i][c] = v[((row_lo + s0 + i) * static_cast<size_t>(nv) + h) * 128 + blockIdx.x * COLS + c];
        }
        if (threadIdx.x < n) {
            const size_t row = row_lo + s0 + threadIdx.x;
            gs[threadIdx.x] = expf(neg_a * softplus_precise(a[row * ldab + h] + dtb));
            bs[threadIdx.x] = 1.0f / (1.0f + expf(-b[row * ldab + h]));
        }
        __syncthreads();
        for (uint32_t i = 0; i < n; ++i) {
            const float g = gs[i], beta = bs[i];
            float kv0 = 0.f, kv1 = 0.f, kv2 = 0.f, kv3 = 0.f;
#pragma unroll
            for (int j = 0; j < NV4; ++j) {
                const float4 kk = ks[i][part + DKS * j];
                kv0 = fmaf(S[j].x, kk.x, kv0);
                kv1 = fmaf(S[j].y, kk.y, kv1);
                kv2 = fmaf(S[j].z, kk.z, kv2);
                kv3 = fmaf(S[j].w, kk.w, kv3);
            }
            float kv = (kv0 + kv1) + (kv2 + kv3);
#pragma unroll
            for (int off = DKS / 2; off > 0; off >>= 1) kv += __shfl_xor_sync(0xffffffffu, kv, off);
            const float delta = (vs[i][threadIdx.x / DKS] - g * kv) * beta;
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int j = 0; j < NV4; ++j) {
                const float4 kk = ks[i][part + DKS * j];
                const float4 qq = qs[i][part + DKS * j];
                S[j].x = fmaf(kk.x, delta, g * S[j].x);
                S[j].y = fmaf(kk.y, delta, g * S[j].y);
                S[j].z = fmaf(kk.z, delta, g * S[j].z);
                S[j].w = fmaf(kk.w, delta, g * S[j].w);
                o0 = fmaf(S[j].x, qq.x, o0);
                o1 = fmaf(S[j].y, qq.y, o1);
                o2 = fmaf(S[j].z, qq.z, o2);
                o3 = fmaf(S[j].w, qq.w, o3);
            }
            float ov = (o0 + o1) + (o2 + o3);
#pragma unroll
            for (int off = DKS / 2; off > 0; off >>= 1) ov += __shfl_xor_sync(0xffffffffu, ov, off);
            if (part == 0) o[((row_lo + s0 + i) * static_cast<size_t>(nv) + h) * 128 + col] = ov;
        }
    }
    if (write_state) {
#pragma unroll
        for (int j = 0; j < NV4; ++j) reinterpret_cast<float4*>(state_out + srow)[part + DKS * j] = S[j];
    }
}

template <int DKS>
void launch_seq(cudaStream_t s, const float* q, const float* k, const float* v, const float* a, const float* b,
                const float* a_log, const float* dt_bias, const float* state_in, float* state_out, float* o, uint32_t t,
                uint32_t ldab, uint32_t nk, uint32_t nv, uint32_t write_state, const uint32_t* seq_start, uint32_t n_seq) {
    dim3 grid(DKS, nv, n_seq);
    gated_delta_seq_kernel<DKS><<<grid, kThreads, 0, s>>>(q, k, v, a, b, a_log, dt_bias, state_in, state_out, o, t, ldab, nk, nv,
                                                          write_state, seq_start);
}

inline bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace

extern "C" int dc_gated_delta(dc_ctx* ctx, void* stream, const float* q, const float* k, const float* v, const float* a,
                              const float* b, const float* a_log, const float* dt_bias, const float* state_in,
                              float* state_out, float* o, uint32_t t, uint32_t ldab, uint32_t write_state, uint32_t nk,
                              uint32_t nv, uint32_t dk, uint32_t dv, const uint32_t* seq_start, uint32_t n_seq, uint32_t max_len) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, q && k && v && a && b && a_log && dt_bias && o, "gated_delta: null operand");
    DC_REQUIRE(ctx, !write_state || state_out, "gated_delta: write_state without a state_out buffer");
    if (dk != 128 || dv != 128) return dc_fail(ctx, DC_UNSUPPORTED, "gated_delta: head dims %u/%u (built for 128/128)", dk, dv);
    DC_REQUIRE(ctx, nk >= 1 && nv % nk == 0, "gated_delta: %u value heads over %u key heads", nv, nk);
    DC_REQUIRE(ctx, ldab >= nv, "delta: ldab = %u must cover the %u value heads", ldab, nv);
    DC_REQUIRE(ctx, aligned16(q) && aligned16(k) && (!state_in || aligned16(state_in)) && (!state_out || aligned16(state_out)),
               "gated_delta: q, k and the state must be 16-byte aligned");
    if (!seq_start) {
        DC_REQUIRE(ctx, t >= 1, "delta: T must be at least 1");
        n_seq = 1;
        max_len = t;
    }
    if (max_len == 0 || max_len > t) max_len = t;
    DC_REQUIRE(ctx, n_seq >= 1 && n_seq <= 65535, "gated_delta: %u sequences", n_seq);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (ctx->delta_impl == DC_IMPL_FAST) {
        DC_REQUIRE(ctx, aligned16(v) && aligned16(o) && ldab >= nv, "gated_delta (chunked): v and o must be 16-byte aligned");
        return dc_gated_delta_chunked(ctx, s, q, k, v, a, b, a_log, dt_bias, state_in, state_out, o, t, ldab, write_state, nk, nv, seq_start, n_seq,
                                      max_len, ctx->delta_split, nullptr, 0, nullptr, nullptr);
    }
    // Baseline: the sequential recurrence. Enough threads to fill the GPU: one lane per value column when there are many sequences,
    // up to 8 lanes per column for a single sequence.
    const uint64_t cols = static_cast<uint64_t>(n_seq) * nv * 128;
    const uint64_t want = static_cast<uint64_t>(ctx->sm_count) * 512;
    if (cols >= want)
        launch_seq<1>(s, q, k, v, a, b, a_log, dt_bias, state_in, state_out, o, t, ldab, nk, nv, write_state, seq_start, n_seq);
    else if (cols * 4 >= want)
        launch_seq<4>(s, q, k, v, a, b, a_log, dt_bias, state_in, state_out, o, t, ldab, nk, nv, write_state, seq_start, n_seq);
    else
        launch_seq<8>(s, q, k, v, a, b, a_log, dt_bias, state_in, state_out, o, t, ldab, nk, nv, write_state, seq_start, n_seq);
    return dc_check_launch(ctx, "gated_delta");
}

extern "C" int dc_conv_gated_delta_supported(dc_ctx* ctx) {
    return ctx && ctx->delta_impl == DC_IMPL_FAST && ctx->delta_engine == DC_ENGINE_TCGEN05 && ctx->delta_split == 3;
}

extern "C" int dc_conv_gated_delta(dc_ctx* ctx, void* stream, const float* p, const float* prev, const float* w, const float* a, const float* b,
                                   const float* a_log, const float* dt_bias, const float* state_in, float* state_out, float* o, uint32_t t,
                                   uint32_t ldp, uint32_t write_state, uint32_t nk, uint32_t nv, uint32_t dk, uint32_t dv,
                                   const uint32_t* seq_start, uint32_t n_seq, uint32_t max_len) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, p && w && a && b && a_log && dt_bias && o, "conv_gated_delta: null operand");
    DC_REQUIRE(ctx, !write_state || state_out, "conv_gated_delta: write_state without a state_out buffer");
    if (dk != 128 || dv != 128) return dc_fail(ctx, DC_UNSUPPORTED, "conv_gated_delta: head dims %u/%u (built for 128/128)", dk, dv);
    DC_REQUIRE(ctx, nk >= 1 && nv % nk == 0, "conv_gated_delta: %u value heads over %u key heads", nv, nk);
    DC_REQUIRE(ctx, ldp >= (2 * nk + nv) * 128 && ldp % 4 == 0, "conv_gated_delta: ldp = %u must cover the qkv columns and be a multiple of 4", ldp);
    DC_REQUIRE(ctx, aligned16(p) && aligned16(w) && aligned16(o) && (!prev || aligned16(prev)) && (!state_in || aligned16(state_in)) &&
                        (!state_out || aligned16(state_out)),
               "conv_gated_delta: p, w, prev, o and the state must be 16-byte aligned");
    if (!dc_conv_gated_delta_supported(ctx))
        return dc_fail(ctx, DC_UNSUPPORTED, "conv_gated_delta: needs the fast delta rule on the tcgen05 engine with split 3");
    if (!seq_start) {
        DC_REQUIRE(ctx, t >= 1, "conv_gated_delta: T must be at least 1");
        n_seq = 1;
        max_len = t;
    }
    if (max_len == 0 || max_len > t) max_len = t;
    DC_REQUIRE(ctx, n_seq >= 1 && n_seq <= 65535, "conv_gated_delta: %u sequences", n_seq);
    // a, b are columns of the same rows as p: their row stride is ldp
    return dc_gated_delta_chunked(ctx, static_cast<cudaStream_t>(stream), nullptr, nullptr, nullptr, a, b, a_log, dt_bias, state_in, state_out, o, t, ldp,
                                  write_state, nk, nv, seq_start, n_seq, max_len, 3, p, ldp, w, prev);
}

extern "C" size_t dc_gated_delta_scratch_bytes(uint32_t t, uint32_t n_seq, uint32_t nv) { return dc_delta_chunk_scratch_bytes(t, n_seq ? n_seq : 1, nv); }
