// Attention prep: zero-centred per-head RMSNorm + rotary embedding of q and k, and the K/V cache
// write. Replaces kernels/rope.metal:24-63; spec cpu_ref.rs:149-162 (head_norm_rope).
// One warp per (row, group of up to 4 heads); a lane holds 4 consecutive dims per 128-dim slab as a float4.
// RoPE pairs dims (i, i + rot/2) with angle = pos * inv_freq[i] in fp32 and precise sin/cos, worked out once
// per row and warp; the partner value comes from another lane by shuffle.
#include "common.cuh"

namespace {

using namespace dc;

constexpr int kWarps = 8;

// Rotation of the 4 dims a lane holds in slab 0 (the rotary part, rot <= 128): cos, and sin with the sign
// of the pair's half folded in; computed once per row and reused for every head of the row. Lane l holds
// dims 4l..4l+3; the partner dims are +-rot/2 away, i.e. in lane l +- rot/8.
struct Rot {
    float4 cs, sn;
    int src;       // lane that holds the partner dims (this lane itself outside the rotary part)
    bool in_rot;
};
__device__ __forceinline__ Rot rope_angles(const float* __restrict__ inv_freq, uint32_t rot, float pos, int lane) {
    Rot r;
    const int half = static_cast<int>(rot >> 1);
    const int d0 = 4 * lane;
    r.in_rot = d0 < static_cast<int>(rot);
    const bool lower = d0 < half;
    const int partner = lower ? lane + (half >> 2) : lane - (half >> 2);
    r.src = r.in_rot ? partner : lane;
    r.cs = make_float4(1.f, 1.f, 1.f, 1.f);
    r.sn = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r.in_rot) {
        const int f0 = lower ? d0 : d0 - half;
        const float4 fr = *reinterpret_cast<const float4*>(inv_freq + f0);
        const float sgn = lower ? -1.0f : 1.0f;
        sincosf(pos * fr.x, &r.sn.x, &r.cs.x);
        sincosf(pos * fr.y, &r.sn.y, &r.cs.y);
        sincosf(pos * fr.z, &r.sn.z, &r.cs.z);
        sincosf(pos * fr.w, &r.sn.w, &r.cs.w);
        r.sn.x *= sgn; r.sn.y *= sgn; r.sn.z *= sgn; r.sn.w *= sgn;
    }
    return r;
}

// Normalises and rotates one head held as HD/128 float4 per lane. `v[c]` are dims c*128 + 4*lane + {0..3};
// RoPE pairs dims (i, i + rot/2) with angle = pos * inv_freq[i] in fp32 and precise sin/cos.
template <int HD>
__device__ __forceinline__ void norm_rope(float4 (&v)[HD / 128], const float* __restrict__ w, const Rot& r, float eps, int lane) {
    constexpr int NC = HD / 128;
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < NC; ++c) ss += v[c].x * v[c].x + v[c].y * v[c].y + v[c].z * v[c].z + v[c].w * v[c].w;
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / static_cast<float>(HD) + eps);
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        const float4 g = reinterpret_cast<const float4*>(w)[c * 32 + lane];
        v[c].x = v[c].x * inv * (1.0f + g.x);
        v[c].y = v[c].y * inv * (1.0f + g.y);
        v[c].z = v[c].z * inv * (1.0f + g.z);
        v[c].w = v[c].w * inv * (1.0f + g.w);
    }
    const float px = __shfl_sync(0xffffffffu, v[0].x, r.src);
    const float py = __shfl_sync(0xffffffffu, v[0].y, r.src);
    const float pz = __shfl_sync(0xffffffffu, v[0].z, r.src);
    const float pw = __shfl_sync(0xffffffffu, v[0].w, r.src);
    if (r.in_rot) {
        v[0].x = v[0].x * r.cs.x + px * r.sn.x;
        v[0].y = v[0].y * r.cs.y + py * r.sn.y;
        v[0].z = v[0].z * r.cs.z + pz * r.sn.z;
        v[0].w = v[0].w * r.cs.w + pw * r.sn.w;
    }
}

template <typename Act>
__device__ __forceinline__ void store_16x4(uint16_t* dst, const float4& v) {
    uint2 o;
    o.x = Act::pack(v.x, v.y);
    o.y = Act::pack(v.z, v.w);
    *reinterpret_cast<uint2*>(dst) = o;
}

// One warp per (row, group of G consecutive heads): the row's sin/cos are worked out once per warp.
template <int HD, typename Act, int G>
__global__ void __launch_bounds__(kWarps * 32)
q_norm_rope_kernel(const float* __restrict__ pq, const float* __restrict__ qw, const float* __restrict__ inv_freq,
                   const uint32_t* __restrict__ qpos, uint16_t* __restrict__ qo, uint32_t rows, uint32_t ldq,
                   uint32_t nq, uint32_t rot, float eps) {
    const uint32_t groups = nq / G;
    const uint32_t idx = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (idx >= rows * groups) return;
    const uint32_t r = idx / groups, h0 = (idx - r * groups) * G;
    const int lane = threadIdx.x & 31;
    constexpr int NC = HD / 128;
    float4 v[G][NC];
    const float* src = pq + static_cast<size_t>(r) * ldq + h0 * HD;
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < NC; ++c) v[g][c] = reinterpret_cast<const float4*>(src + g * HD)[c * 32 + lane];
    const Rot rt = rope_angles(inv_freq, rot, static_cast<float>(qpos[r]), lane);
    uint16_t* dst = qo + (static_cast<size_t>(r) * nq + h0) * HD;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        norm_rope<HD>(v[g], qw, rt, eps, lane);
#pragma unroll
        for (int c = 0; c < NC; ++c) store_16x4<Act>(dst + g * HD + c * 128 + 4 * lane, v[g][c]);
    }
}

// Head slots 0..nkv-1 are the k heads (norm + rope into the K cache), nkv..2nkv-1 the v heads (copied
// to the V cache). Without `pos`, row r is at position pos0 + r and is written to cache row pos0 + r
// (the reference's single-sequence form). With `pos` (packed sequences), row r is rotated for
// position pos[r] and written to cache row r.
template <int HD, typename Act, int G>
__global__ void __launch_bounds__(kWarps * 32)
kv_norm_rope_kernel(const float* __restrict__ pkv, const float* __restrict__ kw, const float* __restrict__ inv_freq,
                    const uint32_t* __restrict__ pos, uint16_t* __restrict__ kc, uint16_t* __restrict__ vc,
                    uint32_t rows, uint32_t ldkv, uint32_t kcol, uint32_t vcol, uint32_t pos0, uint32_t nkv, uint32_t rot,
                    float eps) {
    const uint32_t groups = 2 * nkv / G;   // nkv is a multiple of G: a group holds k heads only or v heads only
    const uint32_t idx = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (idx >= rows * groups) return;
    const uint32_t r = idx / groups, slot0 = (idx - r * groups) * G;
    const int lane = threadIdx.x & 31;
    constexpr int NC = HD / 128;
    const bool is_k = slot0 < nkv;
    const uint32_t h0 = is_k ? slot0 : slot0 - nkv;
    const float* src = pkv + static_cast<size_t>(r) * ldkv + (is_k ? kcol : vcol) + h0 * HD;
    float4 v[G][NC];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < NC; ++c) v[g][c] = reinterpret_cast<const float4*>(src + g * HD)[c * 32 + lane];
    const uint32_t p = pos ? pos[r] : pos0 + r;
    const size_t crow = pos ? r : pos0 + r;
    uint16_t* dst = (is_k ? kc : vc) + (crow * nkv + h0) * HD;
    Rot rt;
    if (is_k) rt = rope_angles(inv_freq, rot, static_cast<float>(p), lane);
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (is_k) norm_rope<HD>(v[g], kw, rt, eps, lane);
#pragma unroll
        for (int c = 0; c < NC; ++c) store_16x4<Act>(dst + g * HD + c * 128 + 4 * lane, v[g][c]);
    }
}

inline bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace

extern "C" {

int dc_q_norm_rope(dc_ctx* ctx, void* stream, const float* pq, const float* qw, const float* inv_freq,
                   const uint32_t* qpos, void* qo, uint32_t rows, uint32_t ldq, uint32_t nq, uint32_t hd, uint32_t rot,
                   float eps) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, pq && qw && inv_freq && qpos && qo, "q_norm_rope: null operand");
    if (hd != 128 && hd != 256) return dc_fail(ctx, DC_UNSUPPORTED, "q_norm_rope: head_dim %u (built for 128 and 256)", hd);
    DC_REQUIRE(ctx, rot % 8 == 0 && rot <= 128 && rot <= hd, "q_norm_rope: rotary dims %u must be a multiple of 8, at most 128", rot);
    DC_REQUIRE(ctx, ldq >= nq * hd && ldq % 4 == 0, "q_norm_rope: ldq = %u must cover the %u q columns and be a multiple of 4", ldq, nq * hd);
    DC_REQUIRE(ctx, aligned16(pq) && aligned16(qw) && aligned16(inv_freq) && reinterpret_cast<uintptr_t>(qo) % 8 == 0, "q_norm_rope: misaligned operand");
    if (rows == 0) return DC_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool f16 = ctx->act_dtype == DC_ACT_F16;
    uint16_t* out = static_cast<uint16_t*>(qo);
    // four heads per warp when the head count allows it (head_dim 128), else one
    auto go = [&](auto kern, uint32_t g) {
        const uint32_t blocks = (rows * (nq / g) + kWarps - 1) / kWarps;
        kern<<<blocks, kWarps * 32, 0, s>>>(pq, qw, inv_freq, qpos, out, rows, ldq, nq, rot, eps);
    };
    if (hd == 128 && nq % 4 == 0) {
        if (f16) go(q_norm_rope_kernel<128, ActF16, 4>, 4);
        else go(q_norm_rope_kernel<128, ActBF16, 4>, 4);
    } else if (hd == 128) {
        if (f16) go(q_norm_rope_kernel<128, ActF16, 1>, 1);
        else go(q_norm_rope_kernel<128, ActBF16, 1>, 1);
    } else {
        if (f16) go(q_norm_rope_kernel<256, ActF16, 1>, 1);
        else go(q_norm_rope_kernel<256, ActBF16, 1>, 1);
    }
    return dc_check_launch(ctx, "q_norm_rope");
}

int dc_kv_norm_rope(dc_ctx* ctx, void* stream, const float* pkv, const float* kw, const float* inv_freq, void* kc, void* vc,
                    uint32_t rows, uint32_t ldkv, uint32_t kcol, uint32_t vcol, uint32_t pos0, const uint32_t* pos,
                    uint32_t cache_rows, uint32_t nkv, uint32_t hd, uint32_t rot, float eps) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, pkv && kw && inv_freq && kc && vc, "kv_norm_rope: null operand");
    if (hd != 128 && hd != 256) return dc_fail(ctx, DC_UNSUPPORTED, "kv_norm_rope: head_dim %u (built for 128 and 256)", hd);
    DC_REQUIRE(ctx, rot % 8 == 0 && rot <= 128 && rot <= hd, "kv_norm_rope: rotary dims %u must be a multiple of 8, at most 128", rot);
    DC_REQUIRE(ctx, ldkv % 4 == 0 && kcol % 4 == 0 && vcol % 4 == 0 && kcol + nkv * hd <= ldkv && vcol + nkv * hd <= ldkv,
               "kv_norm_rope: the k (col %u) and v (col %u) heads must lie inside rows of stride %u at multiples of 4", kcol, vcol, ldkv);
    DC_REQUIRE(ctx, (pos ? rows : pos0 + rows) <= cache_rows, "kv_norm_rope: rows %u..%u overrun the %u-row cache",
               pos ? 0 : pos0, (pos ? rows : pos0 + rows), cache_rows);
    DC_REQUIRE(ctx, aligned16(pkv) && aligned16(kw) && aligned16(inv_freq) && reinterpret_cast<uintptr_t>(kc) % 8 == 0 && reinterpret_cast<uintptr_t>(vc) % 8 == 0,
               "kv_norm_rope: misaligned operand");
    if (rows == 0) return DC_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool f16 = ctx->act_dtype == DC_ACT_F16;
    uint16_t* ko = static_cast<uint16_t*>(kc);
    uint16_t* vo = static_cast<uint16_t*>(vc);
    auto go = [&](auto kern, uint32_t g) {
        const uint32_t blocks = (rows * (2 * nkv / g) + kWarps - 1) / kWarps;
        kern<<<blocks, kWarps * 32, 0, s>>>(pkv, kw, inv_freq, pos, ko, vo, rows, ldkv, kcol, vcol, pos0, nkv, rot, eps);
    };
    if (hd == 128 && nkv % 4 == 0) {
        if (f16) go(kv_norm_rope_kernel<128, ActF16, 4>, 4);
        else go(kv_norm_rope_kernel<128, ActBF16, 4>, 4);
    } else if (hd == 128) {
        if (f16) go(kv_norm_rope_kernel<128, ActF16, 1>, 1);
        else go(kv_norm_rope_kernel<128, ActBF16, 1>, 1);
    } else {
        if (f16) go(kv_norm_rope_kernel<256, ActF16, 1>, 1);
        else go(kv_norm_rope_kernel<256, ActBF16, 1>, 1);
    }
    return dc_check_launch(ctx, "kv_norm_rope");
}

}  // extern "C"
