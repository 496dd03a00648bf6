// Causal GQA attention for a FEW query rows scattered over packed K/V caches: the answer rows of the
// pruned last layer (crates/decide-engine/src/forward.rs:1176-1178 hands Attn::attention the answer
// rows and their positions; kernels/attn.rs:93). Row r attends cache rows kv_start[r] .. kv_start[r]
// + qpos[r] of its own request.
//
// With a handful of query rows there is nothing to tile on the tensor cores: the work is reading each
// request's K and V once. One CTA per (query row, kv head, slice of the keys), one warp per query head
// of the group, so the group's heads share the K/V rows through L1. Per tile of 256 cache rows a warp
// (1) scores them with lanes over KEYS (a lane reads whole 256-byte K rows, q comes from shared memory
// as a broadcast), (2) turns the scores into weights 2^(s - m) with the running maximum, (3)
// accumulates P V with lanes over the 128 DIMS (a V row is one coalesced 256-byte read per warp).
// Everything is fp32; scale and log2(e) are folded into one multiply as in the other attention kernels.
//
// A batch of many answer rows fills the GPU with one slice per row. A single request has 1..16 answer
// rows: its keys are then cut into slices (at most kMaxSlices, each a multiple of 32 keys) so that
// about two CTAs per SM run; every slice leaves its unnormalised sum, maximum and weight total in the
// workspace and a second kernel adds the slices in slice order (the result does not depend on which
// CTA finished first).
#include "common.cuh"

namespace {

using namespace dc;

constexpr int HD = 128;
constexpr int TK = 256;          // cache rows per tile
constexpr int kMaxGroup = 16;    // query heads per kv head
constexpr int kPvUnroll = 16;    // V rows requested together in the P V loop
constexpr int kMaxSlices = 32;
constexpr int kPart = HD + 2;    // floats of one slice's partial: 128 sums, maximum, weight total
constexpr float kMasked = -1e30f;

// Keys of slice z of a row with n keys cut into `slices`: [lo, hi), lo a multiple of 32.
__device__ __forceinline__ void slice_bounds(uint32_t n, uint32_t slices, uint32_t z, uint32_t& lo, uint32_t& hi) {
    const uint32_t len = ((n + slices - 1) / slices + 31u) & ~31u;
    lo = min(n, z * len);
    hi = min(n, lo + len);
}

template <typename Act>
__global__ void __launch_bounds__(kMaxGroup * 32)
attn_rows_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ kc, const uint16_t* __restrict__ vc, const float* __restrict__ gate,
                 const uint32_t* __restrict__ qpos, const uint32_t* __restrict__ kv_start, uint16_t* __restrict__ y, float* __restrict__ part,
                 uint32_t ldg, uint32_t nq, uint32_t nkv, float scale_log2) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t r = blockIdx.x, kvh = blockIdx.y, group = nq / nkv, slices = gridDim.z;
    const uint32_t h = kvh * group + warp;
    float* qs = smem + warp * HD;                       // this head's query, fp32
    float* sc = smem + group * HD + warp * TK;          // this head's scores / weights of the current tile
    {
        const uint2 qv = reinterpret_cast<const uint2*>(q + (static_cast<size_t>(r) * nq + h) * HD)[lane];
        *reinterpret_cast<float4*>(qs + 4 * lane) = make_float4(Act::lo(qv.x), Act::hi(qv.x), Act::lo(qv.y), Act::hi(qv.y));
    }
    __syncwarp();
    uint32_t j_lo, j_hi;
    slice_bounds(qpos[r] + 1u, slices, blockIdx.z, j_lo, j_hi);
    const size_t base = kv_start ? kv_start[r] : 0u;
    float m = kMasked, l = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
    for (uint32_t j0 = j_lo; j0 < j_hi; j0 += TK) {
        const uint32_t cnt = min(static_cast<uint32_t>(TK), j_hi - j0);
        // (1) scores, lanes over keys
        float mx = kMasked;
        for (uint32_t j = lane; j < cnt; j += 32) {
            const uint4* kr = reinterpret_cast<const uint4*>(kc + ((base + j0 + j) * nkv + kvh) * HD);
            float s = 0.f;
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                const uint4 kv = kr[c];
                const float4 qa = *reinterpret_cast<const float4*>(qs + 8 * c), qb = *reinterpret_cast<const float4*>(qs + 8 * c + 4);
                s += qa.x * Act::lo(kv.x) + qa.y * Act::hi(kv.x) + qa.z * Act::lo(kv.y) + qa.w * Act::hi(kv.y) +
                     qb.x * Act::lo(kv.z) + qb.y * Act::hi(kv.z) + qb.z * Act::lo(kv.w) + qb.w * Act::hi(kv.w);
            }
            s *= scale_log2;
            sc[j] = s;
            mx = fmaxf(mx, s);
        }
        mx = warp_max(mx);
        const float m_new = fmaxf(m, mx);
        const float corr = exp2f(m - m_new);
        // (2) weights, still lanes over keys
        float psum = 0.f;
        for (uint32_t j = lane; j < cnt; j += 32) {
            const float p = exp2f(sc[j] - m_new);
            sc[j] = p;
            psum += p;
        }
        l = l * corr + warp_sum(psum);
        o0 *= corr; o1 *= corr; o2 *= corr; o3 *= corr;
        m = m_new;
        __syncwarp();
        // (3) P V, lanes over dims
        const uint16_t* vbase = vc + ((base + j0) * nkv + kvh) * HD + 4 * lane;
        const size_t vstride = static_cast<size_t>(nkv) * HD;
        uint32_t j = 0;
        for (; j + kPvUnroll <= cnt; j += kPvUnroll) {   // many V rows in flight per lane: the loop is bound by load latency
            uint2 v[kPvUnroll];
#pragma unroll
            for (int u = 0; u < kPvUnroll; ++u) v[u] = *reinterpret_cast<const uint2*>(vbase + (j + u) * vstride);
#pragma unroll
            for (int u = 0; u < kPvUnroll; ++u) {
                const float p = sc[j + u];
                o0 += p * Act::lo(v[u].x); o1 += p * Act::hi(v[u].x); o2 += p * Act::lo(v[u].y); o3 += p * Act::hi(v[u].y);
            }
        }
        for (; j < cnt; ++j) {
            const uint2 v = *reinterpret_cast<const uint2*>(vbase + j * vstride);
            const float p = sc[j];
            o0 += p * Act::lo(v.x); o1 += p * Act::hi(v.x); o2 += p * Act::lo(v.y); o3 += p * Act::hi(v.y);
        }
        __syncwarp();
    }
    if (slices > 1) {   // this slice's unnormalised sums, maximum and weight total (an empty slice: zeros, kMasked, 0)
        float* pp = part + ((static_cast<size_t>(r) * nq + h) * slices + blockIdx.z) * kPart;
        *reinterpret_cast<float2*>(pp + 4 * lane) = make_float2(o0, o1);
        *reinterpret_cast<float2*>(pp + 4 * lane + 2) = make_float2(o2, o3);
        if (lane == 0) *reinterpret_cast<float2*>(pp + HD) = make_float2(m, l);
        return;
    }
    const float inv = 1.0f / l;
    o0 *= inv; o1 *= inv; o2 *= inv; o3 *= inv;
    if (gate) {
        const float4 g = *reinterpret_cast<const float4*>(gate + static_cast<size_t>(r) * ldg + h * HD + 4 * lane);
        o0 *= 1.0f / (1.0f + expf(-g.x));
        o1 *= 1.0f / (1.0f + expf(-g.y));
        o2 *= 1.0f / (1.0f + expf(-g.z));
        o3 *= 1.0f / (1.0f + expf(-g.w));
    }
    uint2 out;
    out.x = Act::pack(o0, o1);
    out.y = Act::pack(o2, o3);
    reinterpret_cast<uint2*>(y + (static_cast<size_t>(r) * nq + h) * HD)[lane] = out;
}

// Adds the slices of one (row, head) in slice order: one warp per head, lanes over dims as above.
template <typename Act>
__global__ void __launch_bounds__(128)
attn_rows_join_kernel(const float* __restrict__ part, const float* __restrict__ gate, uint16_t* __restrict__ y, uint32_t ldg, uint32_t nq,
                      uint32_t heads_total, uint32_t slices) {
    const int lane = threadIdx.x & 31;
    const uint32_t rh = blockIdx.x * 4 + (threadIdx.x >> 5);   // row * nq + head
    if (rh >= heads_total) return;
    const float* pp = part + static_cast<size_t>(rh) * slices * kPart;
    float m = kMasked;
    for (uint32_t s = 0; s < slices; ++s) m = fmaxf(m, pp[s * kPart + HD]);
    float l = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
    for (uint32_t s = 0; s < slices; ++s) {
        const float2 ml = *reinterpret_cast<const float2*>(pp + s * kPart + HD);
        if (ml.y == 0.f) continue;   // an empty slice
        const float w = exp2f(ml.x - m);
        const float2 a = *reinterpret_cast<const float2*>(pp + s * kPart + 4 * lane), b = *reinterpret_cast<const float2*>(pp + s * kPart + 4 * lane + 2);
        l += w * ml.y;
        o0 += w * a.x; o1 += w * a.y; o2 += w * b.x; o3 += w * b.y;
    }
    const float inv = 1.0f / l;
    o0 *= inv; o1 *= inv; o2 *= inv; o3 *= inv;
    const uint32_t r = rh / nq, h = rh % nq;
    if (gate) {
        const float4 g = *reinterpret_cast<const float4*>(gate + static_cast<size_t>(r) * ldg + h * HD + 4 * lane);
        o0 *= 1.0f / (1.0f + expf(-g.x));
        o1 *= 1.0f / (1.0f + expf(-g.y));
        o2 *= 1.0f / (1.0f + expf(-g.z));
        o3 *= 1.0f / (1.0f + expf(-g.w));
    }
    uint2 out;
    out.x = Act::pack(o0, o1);
    out.y = Act::pack(o2, o3);
    reinterpret_cast<uint2*>(y + static_cast<size_t>(rh) * HD)[lane] = out;
}

inline bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

// Slices per row: enough CTAs for two per SM, none when the rows alone give that many.
uint32_t slices_for(const dc_ctx* ctx, uint32_t rows, uint32_t nkv) {
    const uint32_t want = 2u * static_cast<uint32_t>(ctx->sm_count), have = rows * nkv;
    if (have >= want) return 1;
    return std::min<uint32_t>(kMaxSlices, (want + have - 1) / have);
}

}  // namespace

extern "C" size_t dc_attention_rows_scratch_bytes(dc_ctx* ctx, uint32_t rows, uint32_t nq, uint32_t nkv) {
    if (!ctx || !nkv) return 0;
    const uint32_t s = slices_for(ctx, rows, nkv);
    return s > 1 ? static_cast<size_t>(rows) * nq * s * kPart * sizeof(float) : 0;
}

extern "C" int dc_attention_rows(dc_ctx* ctx, void* stream, const void* q, const void* kc, const void* vc, const float* gate,
                                 const uint32_t* qpos, const uint32_t* kv_start, void* y, uint32_t rows, uint32_t ldg, uint32_t nq,
                                 uint32_t nkv, uint32_t hd) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, q && kc && vc && qpos && y, "attention_rows: null operand");
    DC_REQUIRE(ctx, rows >= 1, "attention_rows: rows must be at least 1");
    if (hd != HD) return dc_fail(ctx, DC_UNSUPPORTED, "attention_rows: head_dim %u (built for 128)", hd);
    DC_REQUIRE(ctx, nkv >= 1 && nq % nkv == 0, "attention_rows: %u query heads over %u kv heads", nq, nkv);
    if (nq / nkv > kMaxGroup) return dc_fail(ctx, DC_UNSUPPORTED, "attention_rows: %u query heads per kv head (at most %d)", nq / nkv, kMaxGroup);
    DC_REQUIRE(ctx, !gate || (ldg >= nq * hd && ldg % 4 == 0 && aligned16(gate)), "attention_rows: ldg = %u must cover the gate columns, be a multiple of 4, gate 16-byte aligned", ldg);
    DC_REQUIRE(ctx, aligned16(q) && aligned16(kc) && aligned16(vc) && reinterpret_cast<uintptr_t>(y) % 8 == 0, "attention_rows: q, kc, vc must be 16-byte aligned");
    DC_REQUIRE(ctx, nkv <= 65535, "attention_rows: %u kv heads", nkv);
    const uint32_t group = nq / nkv;
    const size_t smem = static_cast<size_t>(group) * (HD + TK) * sizeof(float);   // at most 24 KB
    const float scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(hd));
    const uint32_t slices = slices_for(ctx, rows, nkv);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* part = nullptr;
    if (slices > 1) {
        void* ws = nullptr;
        if (int rc = dc_get_workspace(ctx, dc_attention_rows_scratch_bytes(ctx, rows, nq, nkv), "attention_rows", &ws); rc != DC_OK) return rc;
        part = static_cast<float*>(ws);
    }
    const bool f16 = ctx->act_dtype == DC_ACT_F16;
    auto kern = f16 ? attn_rows_kernel<ActF16> : attn_rows_kernel<ActBF16>;
    kern<<<dim3(rows, nkv, slices), group * 32, smem, s>>>(static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(kc),
                                                           static_cast<const uint16_t*>(vc), gate, qpos, kv_start, static_cast<uint16_t*>(y), part,
                                                           ldg, nq, nkv, scale_log2);
    if (int rc = dc_check_launch(ctx, "attention (answer rows)"); rc != DC_OK) return rc;
    if (slices > 1) {
        auto join = f16 ? attn_rows_join_kernel<ActF16> : attn_rows_join_kernel<ActBF16>;
        join<<<(rows * nq + 3) / 4, 128, 0, s>>>(part, gate, static_cast<uint16_t*>(y), ldg, nq, rows * nq, slices);
        return dc_check_launch(ctx, "attention (answer rows, joining the slices)");
    }
    return DC_OK;
}
