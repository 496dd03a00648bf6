// Small-M GEMM: Y = X * W^T for M <= 16 rows (the answer rows of the pruned last layer), a weight-
// streaming kernel bound by HBM, not by the tensor cores.
//
// Replaces the reference's `gemm_nt_small` (kernels/gemm_fast.metal:470-517, chosen for M <= 16 by
// gemm_configs.rs:252-267): no shared-memory staging of W, optional split over K. Here:
//   * a warp owns 16 output columns (two n8 tiles) and one of KS contiguous K ranges; it streams its
//     16 W rows with 128-bit loads that bypass L1, 4 steps (128 k) in flight per lane;
//   * the products run on mma.sync m16n8k16 (all 16 A rows of the instruction = the M rows, zero rows
//     beyond M). The k index inside an instruction is permuted so that a lane's 128-bit load of 8
//     consecutive k feeds two MMAs directly: X is loaded with the same permutation (from L1, where
//     the few X rows stay resident), so no shuffle or shared memory sits between load and MMA;
//   * the KS partial tiles meet in shared memory and are summed in K-range order (fixed order: results
//     do not depend on scheduling), then the epilogue (the four of kernels/gemm.rs:16-26) stores rows.
#include "common.cuh"

namespace {

using namespace dc;

constexpr int kWarps = 8;
constexpr int kUnroll = 4;   // 32-k steps in flight per lane

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <typename Act>
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if constexpr (Act::kUmmaFormat == 0) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// ks_log2: log2 of the K split (1, 2, 4 or 8 ranges). A CTA of 8 warps covers 8 / KS column pairs of 16.
template <int EPI, typename Act>
__global__ void __launch_bounds__(kWarps * 32)
gemm_small_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, void* __restrict__ y, uint32_t m, uint32_t n, uint32_t k,
                  uint32_t ldx, uint32_t ldw, uint32_t ldy, uint32_t ks_log2) {
    __shared__ float red[kWarps][2][32 * 4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t ks_n = 1u << ks_log2;
    const uint32_t ks = static_cast<uint32_t>(warp) & (ks_n - 1u);
    const uint32_t pair = static_cast<uint32_t>(warp) >> ks_log2;
    const uint32_t pairs_per_cta = kWarps >> ks_log2;
    const uint32_t span = 16u * pairs_per_cta;                 // output columns of this CTA
    const uint32_t cta_col0 = blockIdx.x * span;
    const uint32_t col0 = cta_col0 + 16u * pair;

    float acc[2][4] = {};
    if (col0 < n) {
        const uint32_t steps = k >> 5;
        const uint32_t per = (steps + ks_n - 1u) >> ks_log2;
        const uint32_t s0 = ks * per, s1 = min(steps, s0 + per);
        const uint4* wp0 = reinterpret_cast<const uint4*>(w + static_cast<size_t>(col0 + g) * ldw) + t;
        const uint4* wp1 = reinterpret_cast<const uint4*>(w + static_cast<size_t>(col0 + 8 + g) * ldw) + t;
        const bool r0 = static_cast<uint32_t>(g) < m, r1 = static_cast<uint32_t>(g) + 8u < m;
        const uint4* xp0 = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r0 ? g : 0) * ldx) + t;
        const uint4* xp1 = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r1 ? g + 8 : 0) * ldx) + t;
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        for (uint32_t s = s0; s < s1; s += kUnroll) {
            uint4 wa[kUnroll], wb[kUnroll], xa[kUnroll], xb[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const bool on = s + u < s1;
                const uint32_t o = (s + u) * 4u;   // a step is 32 elements = four 16-byte pieces, one per t
                wa[u] = on ? ld_stream(wp0 + o) : zero;
                wb[u] = on ? ld_stream(wp1 + o) : zero;
                xa[u] = (on && r0) ? __ldg(xp0 + o) : zero;
                xb[u] = (on && r1) ? __ldg(xp1 + o) : zero;
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                // A registers: {row g, k-slots 2t..}, {row g+8, 2t..}, {row g, 2t+8..}, {row g+8, 2t+8..}
                mma_16816<Act>(acc[0], xa[u].x, xb[u].x, xa[u].y, xb[u].y, wa[u].x, wa[u].y);
                mma_16816<Act>(acc[0], xa[u].z, xb[u].z, xa[u].w, xb[u].w, wa[u].z, wa[u].w);
                mma_16816<Act>(acc[1], xa[u].x, xb[u].x, xa[u].y, xb[u].y, wb[u].x, wb[u].y);
                mma_16816<Act>(acc[1], xa[u].z, xb[u].z, xa[u].w, xb[u].w, wb[u].z, wb[u].w);
            }
        }
    }
    *reinterpret_cast<float4*>(&red[warp][0][lane * 4]) = make_float4(acc[0][0], acc[0][1], acc[0][2], acc[0][3]);
    *reinterpret_cast<float4*>(&red[warp][1][lane * 4]) = make_float4(acc[1][0], acc[1][1], acc[1][2], acc[1][3]);
    __syncthreads();

    // element (row, local column) of the CTA's 16 x span block: fragment slot of the accumulator that holds it
    auto value = [&](uint32_t row, uint32_t cl) {
        const uint32_t p = cl >> 4, tile = (cl >> 3) & 1u, c = cl & 7u;
        const uint32_t slot = ((row & 7u) * 4u + (c >> 1)) * 4u + (row >> 3) * 2u + (c & 1u);
        float v = 0.0f;
        for (uint32_t q = 0; q < ks_n; ++q) v += red[(p << ks_log2) + q][tile][slot];   // K ranges in order
        return v;
    };
    const uint32_t out_span = EPI == DC_EPI_SWIGLU_BF16 ? span >> 1 : span;
    for (uint32_t e = threadIdx.x; e < m * out_span; e += kWarps * 32) {
        const uint32_t row = e / out_span, oc = e - row * out_span;
        if constexpr (EPI == DC_EPI_SWIGLU_BF16) {
            // gate|up blocks of 16 columns alternate: output column oc of this CTA <- columns 32 (oc / 16) + oc % 16 (+ 16)
            const uint32_t cl = ((oc >> 4) << 5) + (oc & 15u);
            if (cta_col0 + cl >= n) continue;
            const float gate = value(row, cl), up = value(row, cl + 16u);
            static_cast<uint16_t*>(y)[static_cast<size_t>(row) * ldy + (cta_col0 >> 1) + oc] = Act::to16(silu_f(gate) * up);
        } else {
            if (cta_col0 + oc >= n) continue;
            const float v = value(row, oc);
            const size_t o = static_cast<size_t>(row) * ldy + cta_col0 + oc;
            if constexpr (EPI == DC_EPI_STORE_F32) static_cast<float*>(y)[o] = v;
            else if constexpr (EPI == DC_EPI_ADD_F32) static_cast<float*>(y)[o] += v;
            else static_cast<uint16_t*>(y)[o] = Act::to16(v);
        }
    }
}

template <int EPI>
int launch_small(dc_ctx* ctx, cudaStream_t s, const void* x, const void* w, void* y, uint32_t m, uint32_t n, uint32_t k, uint32_t ldx,
                 uint32_t ldw, uint32_t ldy, uint32_t ks_log2) {
    const uint32_t span = 16u * (kWarps >> ks_log2);
    const uint32_t grid = (n + span - 1) / span;
    const auto* xp = static_cast<const uint16_t*>(x);
    const auto* wp = static_cast<const uint16_t*>(w);
    if (ctx->act_dtype == DC_ACT_F16) gemm_small_kernel<EPI, ActF16><<<grid, kWarps * 32, 0, s>>>(xp, wp, y, m, n, k, ldx, ldw, ldy, ks_log2);
    else gemm_small_kernel<EPI, ActBF16><<<grid, kWarps * 32, 0, s>>>(xp, wp, y, m, n, k, ldx, ldw, ldy, ks_log2);
    return dc_check_launch(ctx, "gemm (small M)");
}

}  // namespace

// K split of the small-M kernel for a shape: the smallest of 1, 2, 4, 8 ranges that gives the chip about two
// thousand warps to stream with, each range at least 4 steps of 32 long; the SwiGLU epilogue needs a gate block and
// its up block (32 columns) inside one CTA, so it stops at 4.
uint32_t dc_gemm_small_ks_log2(uint32_t n, uint32_t k, uint32_t epi) {
    const uint32_t pairs = n / 16u, steps = k / 32u;
    const uint32_t max_log2 = epi == DC_EPI_SWIGLU_BF16 ? 2u : 3u;
    uint32_t l = 0;
    while (l < max_log2 && (pairs << l) < 2048u && (steps >> (l + 1)) >= 4u) ++l;
    return l;
}

int dc_gemm_small(dc_ctx* ctx, cudaStream_t s, const void* x, const void* w, void* y, uint32_t m, uint32_t n, uint32_t k, uint32_t ldx,
                  uint32_t ldw, uint32_t ldy, uint32_t epi) {
    const uint32_t l = dc_gemm_small_ks_log2(n, k, epi);
    switch (epi) {
        case DC_EPI_STORE_F32: return launch_small<DC_EPI_STORE_F32>(ctx, s, x, w, y, m, n, k, ldx, ldw, ldy, l);
        case DC_EPI_ADD_F32: return launch_small<DC_EPI_ADD_F32>(ctx, s, x, w, y, m, n, k, ldx, ldw, ldy, l);
        case DC_EPI_STORE_BF16: return launch_small<DC_EPI_STORE_BF16>(ctx, s, x, w, y, m, n, k, ldx, ldw, ldy, l);
        default: return launch_small<DC_EPI_SWIGLU_BF16>(ctx, s, x, w, y, m, n, k, ldx, ldw, ldy, l);
    }
}
