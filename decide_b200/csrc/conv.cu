// Depthwise causal conv (kernel 4) + SiLU over the qkv columns of the Gated-DeltaNet input
// projection, the per-head L2 norm of q and k, and the conv state update.
// Replaces kernels/conv.metal:5-51; spec cpu_ref.rs:55-95.
//
// One warp owns one head slot (128 channels, a float4 per lane) over a block of consecutive rows and
// slides a 3-row register window down the rows, so every raw row is read once per warp (plus a
// 3-row halo per block). Slots 0..nk-1 are q heads, nk..2nk-1 k heads, the rest v heads.
#include "common.cuh"

namespace {

using namespace dc;

constexpr int kWarps = 4;
constexpr int kRowsPerWarp = 32;

// seq_start: [n_seq + 1] row offsets of packed sequences, or null for one sequence of `t` rows.
// prev: [n_seq, 3, conv_dim] raw rows before each sequence (oldest first), or null for zeros.
__global__ void __launch_bounds__(kWarps * 32)
conv_silu_l2_kernel(const float* __restrict__ p, const float* __restrict__ prev, const float* __restrict__ w,
                    float* __restrict__ q, float* __restrict__ k, float* __restrict__ v, uint32_t t, uint32_t ldp,
                    uint32_t nk, uint32_t nv, const uint32_t* __restrict__ seq_start) {
    const uint32_t slots = 2 * nk + nv;
    const uint32_t conv_dim = slots * 128;
    const uint32_t seq = blockIdx.z;
    const uint32_t row_lo = seq_start ? seq_start[seq] : 0u;
    const uint32_t len = seq_start ? seq_start[seq + 1] - row_lo : t;
    const uint32_t slot = blockIdx.y * kWarps + (threadIdx.x >> 5);
    const uint32_t s0 = blockIdx.x * kRowsPerWarp;
    if (slot >= slots || s0 >= len) return;
    const int lane = threadIdx.x & 31;
    const uint32_t c0 = slot * 128 + 4 * lane;

    // taps of this lane's 4 channels: w is [conv_dim, 4]
    const float4 w0 = reinterpret_cast<const float4*>(w)[c0 + 0];
    const float4 w1 = reinterpret_cast<const float4*>(w)[c0 + 1];
    const float4 w2 = reinterpret_cast<const float4*>(w)[c0 + 2];
    const float4 w3 = reinterpret_cast<const float4*>(w)[c0 + 3];

    auto raw = [&](int s) -> float4 {  // raw row s of this sequence; s may be -3..-1
        if (s >= 0) return *reinterpret_cast<const float4*>(p + static_cast<size_t>(row_lo + s) * ldp + c0);
        if (prev) return *reinterpret_cast<const float4*>(prev + (static_cast<size_t>(seq) * 3 + (3 + s)) * conv_dim + c0);
        return make_float4(0.f, 0.f, 0.f, 0.f);
    };
    float4 x0 = raw(static_cast<int>(s0) - 3), x1 = raw(static_cast<int>(s0) - 2), x2 = raw(static_cast<int>(s0) - 1);
    const uint32_t s_end = min(s0 + kRowsPerWarp, len);
    const bool is_q = slot < nk, is_k = !is_q && slot < 2 * nk;
    const float qscale = 0.08838834764831845f;  // 128^-1/2
    auto emit = [&](uint32_t s, const float4& x3) {
        float4 y;
        // channel c0+0 uses taps w0.{x,y,z,w} on rows s-3..s, and so on
        y.x = silu_f(fmaf(w0.w, x3.x, fmaf(w0.z, x2.x, fmaf(w0.y, x1.x, w0.x * x0.x))));
        y.y = silu_f(fmaf(w1.w, x3.y, fmaf(w1.z, x2.y, fmaf(w1.y, x1.y, w1.x * x0.y))));
        y.z = silu_f(fmaf(w2.w, x3.z, fmaf(w2.z, x2.z, fmaf(w2.y, x1.z, w2.x * x0.z))));
        y.w = silu_f(fmaf(w3.w, x3.w, fmaf(w3.z, x2.w, fmaf(w3.y, x1.w, w3.x * x0.w))));
        x0 = x1;
        x1 = x2;
        x2 = x3;
        const size_t row = row_lo + s;
        if (is_q || is_k) {
            const float ss = warp_sum(y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w);
            const float inv = rsqrtf(ss + 1e-6f) * (is_q ? qscale : 1.0f);
            y.x *= inv;
            y.y *= inv;
            y.z *= inv;
            y.w *= inv;
            float* dst = (is_q ? q : k) + (row * nk + (is_q ? slot : slot - nk)) * 128 + 4 * lane;
            *reinterpret_cast<float4*>(dst) = y;
        } else {
            float* dst = v + (row * nv + (slot - 2 * nk)) * 128 + 4 * lane;
            *reinterpret_cast<float4*>(dst) = y;
        }
    };
    // four rows' loads in flight at a time
    uint32_t s = s0;
    for (; s + 4 <= s_end; s += 4) {
        const float4 a0 = raw(static_cast<int>(s)), a1 = raw(static_cast<int>(s) + 1), a2 = raw(static_cast<int>(s) + 2), a3 = raw(static_cast<int>(s) + 3);
        emit(s, a0);
        emit(s + 1, a1);
        emit(s + 2, a2);
        emit(s + 3, a3);
    }
    for (; s < s_end; ++s) emit(s, raw(static_cast<int>(s)));
}

// prev_out[i] = raw row (t - 3 + i) of the chunk, drawn from prev_in when t < 3; in-place safe
// because every thread reads its 3 values before writing them (conv.metal:37-51).
__global__ void conv_state_update_kernel(const float* __restrict__ p, const float* __restrict__ prev_in,
                                         float* __restrict__ prev_out, uint32_t t, uint32_t ldp, uint32_t conv_dim) {
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= conv_dim) return;
    float r[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const int s = static_cast<int>(t) - 3 + i;
        r[i] = s >= 0 ? p[static_cast<size_t>(s) * ldp + c] : (prev_in ? prev_in[(3 + s) * conv_dim + c] : 0.0f);
    }
#pragma unroll
    for (int i = 0; i < 3; ++i) prev_out[i * conv_dim + c] = r[i];
}

inline bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace

extern "C" {

int dc_conv_silu_l2(dc_ctx* ctx, void* stream, const float* p, const float* prev, const float* w, float* q, float* k,
                    float* v, uint32_t t, uint32_t ldp, uint32_t nk, uint32_t nv, uint32_t dk, uint32_t dv,
                    const uint32_t* seq_start, uint32_t n_seq, uint32_t max_len) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, p && w && q && k && v, "conv_silu_l2: null operand");
    if (dk != 128 || dv != 128) return dc_fail(ctx, DC_UNSUPPORTED, "conv_silu_l2: head dims %u/%u (built for 128/128)", dk, dv);
    const uint32_t conv_dim = (2 * nk + nv) * 128;
    DC_REQUIRE(ctx, ldp >= conv_dim && ldp % 4 == 0, "conv_silu_l2: ldp = %u must cover the %u qkv columns and be a multiple of 4", ldp, conv_dim);
    DC_REQUIRE(ctx, aligned16(p) && aligned16(w) && aligned16(q) && aligned16(k) && aligned16(v) && (!prev || aligned16(prev)), "conv_silu_l2: misaligned operand");
    if (!seq_start) {
        n_seq = 1;
        max_len = t;
    }
    DC_REQUIRE(ctx, n_seq >= 1 && n_seq <= 65535, "conv_silu_l2: %u sequences", n_seq);
    if (max_len == 0) return DC_OK;
    dim3 grid((max_len + kRowsPerWarp - 1) / kRowsPerWarp, (2 * nk + nv + kWarps - 1) / kWarps, n_seq);
    conv_silu_l2_kernel<<<grid, kWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(p, prev, w, q, k, v, t, ldp, nk, nv, seq_start);
    return dc_check_launch(ctx, "conv_silu_l2");
}

int dc_conv_state_update(dc_ctx* ctx, void* stream, const float* p, const float* prev_in, float* prev_out, uint32_t t,
                         uint32_t ldp, uint32_t conv_dim) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, p && prev_out, "conv_state_update: null operand");
    DC_REQUIRE(ctx, ldp >= conv_dim, "conv_state_update: ldp = %u must cover the %u qkv columns", ldp, conv_dim);
    conv_state_update_kernel<<<(conv_dim + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(p, prev_in, prev_out, t, ldp, conv_dim);
    return dc_check_launch(ctx, "conv_state_update");
}

}  // extern "C"
