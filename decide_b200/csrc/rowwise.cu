// HBM-bound row kernels: RMSNorm, embedding gather, row gathers, the candidate-row logit head and
// the gated RMSNorm. One warp per row (or per (row, head)), 128-bit loads and stores, shuffle
// reductions. They replace kernels/rmsnorm.metal, embed.metal, head.metal and gnorm.metal.
#include <atomic>

#include "common.cuh"

namespace {

using namespace dc;

constexpr int kWarpsPerBlock = 8;

// y[r] = x[rowmap[r]] * rsqrt(mean(x^2) + eps) * (w or 1 + w); spec cpu_ref.rs:11-22.
template <typename Act>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, uint16_t* __restrict__ y,
               const uint32_t* __restrict__ rowmap, uint32_t rows, uint32_t h, uint32_t ld_in, uint32_t ld_out, float eps,
               uint32_t add_one) {
    const uint32_t r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint32_t src = rowmap ? rowmap[r] : r;
    const float4* xr = reinterpret_cast<const float4*>(x + static_cast<size_t>(src) * ld_in);
    const float4* wr = reinterpret_cast<const float4*>(w);
    const uint32_t nv = h >> 2;
    float ss = 0.0f;
    for (uint32_t i = lane; i < nv; i += 32) {
        const float4 v = xr[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / static_cast<float>(h) + eps);
    const float one = add_one ? 1.0f : 0.0f;
    uint2* yr = reinterpret_cast<uint2*>(y + static_cast<size_t>(r) * ld_out);
    for (uint32_t i = lane; i < nv; i += 32) {
        const float4 v = xr[i];
        const float4 g = wr[i];
        uint2 o;
        o.x = Act::pack(v.x * inv * (one + g.x), v.y * inv * (one + g.y));
        o.y = Act::pack(v.z * inv * (one + g.z), v.w * inv * (one + g.w));
        yr[i] = o;
    }
}

// The same for rows of exactly NV4 * 128 values: the row stays in registers between the two passes and all of its
// loads are in flight at once.
template <typename Act, int NV4>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rmsnorm_reg_kernel(const float* __restrict__ x, const float* __restrict__ w, uint16_t* __restrict__ y,
                   const uint32_t* __restrict__ rowmap, uint32_t rows, uint32_t ld_in, uint32_t ld_out, float eps, uint32_t add_one) {
    const uint32_t r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint32_t src = rowmap ? rowmap[r] : r;
    const float4* xr = reinterpret_cast<const float4*>(x + static_cast<size_t>(src) * ld_in);
    const float4* wr = reinterpret_cast<const float4*>(w);
    float4 v[NV4];
#pragma unroll
    for (int i = 0; i < NV4; ++i) v[i] = xr[lane + 32 * i];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV4; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / static_cast<float>(NV4 * 128) + eps);
    const float one = add_one ? 1.0f : 0.0f;
    uint2* yr = reinterpret_cast<uint2*>(y + static_cast<size_t>(r) * ld_out);
#pragma unroll
    for (int i = 0; i < NV4; ++i) {
        const float4 g = wr[lane + 32 * i];
        uint2 o;
        o.x = Act::pack(v[i].x * inv * (one + g.x), v[i].y * inv * (one + g.y));
        o.y = Act::pack(v[i].z * inv * (one + g.z), v[i].w * inv * (one + g.w));
        yr[lane + 32 * i] = o;
    }
}

// x[r] += add[r]; then (y != null) y[r] = x[r] * rsqrt(mean(x^2) + eps) * (w or 1 + w). The partial-sum add of a tensor-parallel
// group (the all-reduced output of a row-split projection joins the residual; the reference's ane_add_partial,
// kernels/ane.metal:10-18) fused with the RMSNorm that follows it. `add` is fp32, or (ADD16) in the context's 16-bit type when
// the group exchanges 16-bit partial sums. NV4 > 0: rows of exactly NV4 * 128 values stay in registers between the passes.
template <typename Act, bool ADD16>
__device__ __forceinline__ float4 load_add4(const void* add, size_t row, uint32_t h, uint32_t i) {
    if constexpr (ADD16) {
        const uint2 v = reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(add) + row * h)[i];
        return make_float4(Act::lo(v.x), Act::hi(v.x), Act::lo(v.y), Act::hi(v.y));
    } else {
        return reinterpret_cast<const float4*>(static_cast<const float*>(add) + row * h)[i];
    }
}

template <typename Act, bool ADD16, int NV4>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
add_rmsnorm_kernel(float* __restrict__ x, const void* __restrict__ add, const float* __restrict__ w, uint16_t* __restrict__ y, uint32_t rows,
                   uint32_t h, float eps, uint32_t add_one) {
    const uint32_t r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    float4* xr = reinterpret_cast<float4*>(x + static_cast<size_t>(r) * h);
    const float4* wr = reinterpret_cast<const float4*>(w);
    uint2* yr = reinterpret_cast<uint2*>(y + static_cast<size_t>(r) * h);
    const float one = add_one ? 1.0f : 0.0f;
    float ss = 0.0f;
    if constexpr (NV4 > 0) {
        float4 v[NV4];
#pragma unroll
        for (int i = 0; i < NV4; ++i) v[i] = xr[lane + 32 * i];
#pragma unroll
        for (int i = 0; i < NV4; ++i) {
            const float4 a = load_add4<Act, ADD16>(add, r, h, lane + 32 * i);
            v[i].x += a.x; v[i].y += a.y; v[i].z += a.z; v[i].w += a.w;
            xr[lane + 32 * i] = v[i];
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
        if (!y) return;
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / static_cast<float>(NV4 * 128) + eps);
#pragma unroll
        for (int i = 0; i < NV4; ++i) {
            const float4 g = wr[lane + 32 * i];
            uint2 o;
            o.x = Act::pack(v[i].x * inv * (one + g.x), v[i].y * inv * (one + g.y));
            o.y = Act::pack(v[i].z * inv * (one + g.z), v[i].w * inv * (one + g.w));
            yr[lane + 32 * i] = o;
        }
    } else {
        const uint32_t nv = h >> 2;
        for (uint32_t i = lane; i < nv; i += 32) {
            float4 v = xr[i];
            const float4 a = load_add4<Act, ADD16>(add, r, h, i);
            v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            xr[i] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        if (!y) return;
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / static_cast<float>(h) + eps);
        for (uint32_t i = lane; i < nv; i += 32) {
            const float4 v = xr[i];   // this lane's own stores of the first pass
            const float4 g = wr[i];
            uint2 o;
            o.x = Act::pack(v.x * inv * (one + g.x), v.y * inv * (one + g.y));
            o.y = Act::pack(v.z * inv * (one + g.z), v.w * inv * (one + g.w));
            yr[i] = o;
        }
    }
}

// out[t] = float(table[ids[t]]); embed.metal:4-13.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
embed_kernel(const uint32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table, float* __restrict__ out, uint32_t t,
             uint32_t h) {
    const uint32_t r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= t) return;
    const int lane = threadIdx.x & 31;
    const uint2* src = reinterpret_cast<const uint2*>(table + static_cast<size_t>(ids[r]) * h);
    float4* dst = reinterpret_cast<float4*>(out + static_cast<size_t>(r) * h);
    for (uint32_t i = lane; i < (h >> 2); i += 32) {
        const uint2 v = src[i];
        dst[i] = make_float4(bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y));
    }
}

// out[i] = x[rowmap[i]], rows of `row_bytes` bytes (a multiple of 16); head.metal:9-28.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
gather_rows_kernel(const uint4* __restrict__ x, const uint32_t* __restrict__ rowmap, uint4* __restrict__ out, uint32_t rows,
                   uint32_t vec_per_row) {
    const uint32_t r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint4* src = x + static_cast<size_t>(rowmap[r]) * vec_per_row;
    uint4* dst = out + static_cast<size_t>(r) * vec_per_row;
    for (uint32_t i = lane; i < vec_per_row; i += 32) dst[i] = src[i];
}

// One warp per (row, candidate): final zero-centred RMSNorm of the row, then the dot product with the
// candidate's bf16 embedding row, all in fp32 (head.metal:32-59; spec cpu_ref.rs:192-198). The table
// rows are read from the device-resident table by id.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
final_head_kernel(const float* __restrict__ x, const float* __restrict__ w, const __nv_bfloat16* __restrict__ table,
                  const uint32_t* __restrict__ cand, const uint32_t* __restrict__ ncand, float* __restrict__ logits,
                  uint32_t h, uint32_t max_cand, float eps) {
    const uint32_t r = blockIdx.x;
    const uint32_t c = blockIdx.y * kWarpsPerBlock + (threadIdx.x >> 5);
    const uint32_t nc = min(ncand[r], max_cand);
    if (c >= nc) return;
    const int lane = threadIdx.x & 31;
    const float4* xr = reinterpret_cast<const float4*>(x + static_cast<size_t>(r) * h);
    const float4* wr = reinterpret_cast<const float4*>(w);
    const uint32_t nv = h >> 2;
    float ss = 0.0f;
    for (uint32_t i = lane; i < nv; i += 32) {
        const float4 v = xr[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / static_cast<float>(h) + eps);
    const uint2* er = reinterpret_cast<const uint2*>(table + static_cast<size_t>(cand[static_cast<size_t>(r) * max_cand + c]) * h);
    float dot = 0.0f;
    for (uint32_t i = lane; i < nv; i += 32) {
        const float4 v = xr[i];
        const float4 g = wr[i];
        const uint2 e = er[i];
        dot = fmaf(v.x * inv * (1.0f + g.x), bf16_lo(e.x), dot);
        dot = fmaf(v.y * inv * (1.0f + g.y), bf16_hi(e.x), dot);
        dot = fmaf(v.z * inv * (1.0f + g.z), bf16_lo(e.y), dot);
        dot = fmaf(v.w * inv * (1.0f + g.w), bf16_hi(e.y), dot);
    }
    dot = warp_sum(dot);
    if (lane == 0) logits[static_cast<size_t>(r) * max_cand + c] = dot;
}

// Per (row, value head): RMSNorm over dv = 128 with fp32 weight (no +1), times silu(z);
// gnorm.metal:6-25, spec cpu_ref.rs:132-145. One warp per (row, head), one float4 per lane.
// One warp per (row, group of G consecutive heads): all of the group's loads are in flight together.
template <typename Act, int G>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
gated_rmsnorm_silu_kernel(const float* __restrict__ o, const float* __restrict__ z, const float* __restrict__ w,
                          uint16_t* __restrict__ y, uint32_t t, uint32_t nv_heads, uint32_t ldz, float eps) {
    const uint32_t groups = nv_heads / G;
    const uint32_t idx = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (idx >= t * groups) return;
    const uint32_t s = idx / groups, h0 = (idx - s * groups) * G;
    const int lane = threadIdx.x & 31;
    const size_t head0 = static_cast<size_t>(s) * nv_heads + h0;
    float4 v[G], zz[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        v[g] = reinterpret_cast<const float4*>(o + (head0 + g) * 128)[lane];
        zz[g] = reinterpret_cast<const float4*>(z + static_cast<size_t>(s) * ldz + (h0 + g) * 128)[lane];
    }
    const float4 gw = reinterpret_cast<const float4*>(w)[lane];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float ss = warp_sum(v[g].x * v[g].x + v[g].y * v[g].y + v[g].z * v[g].z + v[g].w * v[g].w);
        const float inv = rsqrtf(ss * (1.0f / 128.0f) + eps);
        uint2 out;
        out.x = Act::pack(v[g].x * inv * gw.x * silu_f(zz[g].x), v[g].y * inv * gw.y * silu_f(zz[g].y));
        out.y = Act::pack(v[g].z * inv * gw.z * silu_f(zz[g].z), v[g].w * inv * gw.w * silu_f(zz[g].w));
        reinterpret_cast<uint2*>(y + (head0 + g) * 128)[lane] = out;
    }
}

// bf16 -> fp16 with the converter's precision-loss counters (convert.rs:73-90): [1] subnormal results,
// [2] non-zero values flushed to zero, [3] finite values that overflow to infinity.
__global__ void __launch_bounds__(256)
convert_bf16_to_f16_kernel(const uint16_t* src, uint16_t* dst, size_t n, unsigned long long* counters) {
    unsigned long long sub = 0, flushed = 0, over = 0;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float x = __uint_as_float(static_cast<uint32_t>(src[i]) << 16);
        const __half h = __float2half_rn(x);
        const uint16_t bits = __half_as_ushort(h);
        const uint16_t mag = bits & 0x7fffu;
        if (mag == 0x7c00u && isfinite(x)) ++over;
        else if (mag == 0 && x != 0.0f) ++flushed;
        else if (mag != 0 && mag < 0x0400u) ++sub;
        dst[i] = bits;
    }
    sub = __reduce_add_sync(0xffffffffu, static_cast<unsigned>(sub));
    flushed = __reduce_add_sync(0xffffffffu, static_cast<unsigned>(flushed));
    over = __reduce_add_sync(0xffffffffu, static_cast<unsigned>(over));
    if ((threadIdx.x & 31) == 0) {
        if (sub) atomicAdd(&counters[1], sub);
        if (flushed) atomicAdd(&counters[2], flushed);
        if (over) atomicAdd(&counters[3], over);
    }
}

// Scratch of dc_convert_bf16_to_f16_noalloc: the four precision-loss counters, resident in every
// GPU that loads the library. In host code this name is only a stand-in for the device symbol; the
// device address comes from cudaGetSymbolAddress (see noalloc_counters()).
static __device__ __align__(256) unsigned long long g_noalloc_counters[4];

inline uint32_t blocks_for(uint32_t warps) { return (warps + kWarpsPerBlock - 1) / kWarpsPerBlock; }
inline bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace

extern "C" {

int dc_convert_bf16_to_f16(dc_ctx* ctx, void* stream, const void* src, void* dst, size_t n, dc_convert_report* report) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, src && dst, "convert: null operand");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    void* ws = nullptr;
    if (int rc = dc_get_workspace(ctx, 64, "convert", &ws); rc != DC_OK) return rc;
    unsigned long long* counters = static_cast<unsigned long long*>(ws);
    cudaError_t e = cudaMemsetAsync(counters, 0, 32, s);
    if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "convert: %s", cudaGetErrorString(e));
    if (n) {
        const size_t want = (n + 255) / 256;
        const uint32_t blocks = static_cast<uint32_t>(want < static_cast<size_t>(ctx->sm_count) * 16 ? want : static_cast<size_t>(ctx->sm_count) * 16);
        convert_bf16_to_f16_kernel<<<blocks, 256, 0, s>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), n, counters);
        int rc = dc_check_launch(ctx, "convert_bf16_to_f16");
        if (rc != DC_OK) return rc;
    }
    unsigned long long host[4] = {0, 0, 0, 0};
    e = cudaMemcpyAsync(host, counters, 32, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "convert: %s", cudaGetErrorString(e));
    if (report) {
        report->values += n;
        report->f16_subnormal += host[1];
        report->f16_flushed_to_zero += host[2];
        report->f16_overflow += host[3];
    }
    return DC_OK;
}

// Device address of g_noalloc_counters on the current device, looked up once per device.
static cudaError_t noalloc_counters(int device, unsigned long long** out) {
    constexpr int kMaxDevices = 64;
    static std::atomic<unsigned long long*> cached[kMaxDevices];   // threads may race on a device's first call: same value, stored atomically
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    unsigned long long* p = cached[device].load(std::memory_order_acquire);
    if (!p) {
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_counters);
        if (e != cudaSuccess) return e;
        cached[device].store(p, std::memory_order_release);
    }
    *out = p;
    return cudaSuccess;
}

int dc_convert_bf16_to_f16_noalloc(void* stream, const void* src, void* dst, size_t n, dc_convert_report* report, char* err,
                                   size_t err_len) {
    auto fail = [&](int code, const char* msg, const char* detail) {
        if (err && err_len) snprintf(err, err_len, "dc_convert_bf16_to_f16_noalloc: %s%s%s", msg, detail ? ": " : "", detail ? detail : "");
        return code;
    };
    if (err && err_len) err[0] = 0;
    if (!src || !dst) return fail(DC_INVALID_ARG, "null operand", nullptr);
    if (n > DC_NOALLOC_MAX_VALUES) return fail(DC_INVALID_ARG, "more than DC_NOALLOC_MAX_VALUES (2^32) values in one call; split the tensor", nullptr);
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(DC_CUDA_ERROR, "no current device", cudaGetErrorString(e));
    unsigned long long* counters = nullptr;
    e = noalloc_counters(device, &counters);
    if (e != cudaSuccess) return fail(DC_CUDA_ERROR, "cannot resolve the scratch symbol", cudaGetErrorString(e));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    e = cudaMemsetAsync(counters, 0, 4 * sizeof(unsigned long long), s);  // the array keeps the last call's counts
    if (e != cudaSuccess) return fail(DC_CUDA_ERROR, "clearing the scratch failed", cudaGetErrorString(e));
    if (n) {
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess || sms <= 0) return fail(DC_CUDA_ERROR, "cannot read the SM count", e != cudaSuccess ? cudaGetErrorString(e) : nullptr);
        const size_t want = (n + 255) / 256;
        const uint32_t blocks = static_cast<uint32_t>(want < static_cast<size_t>(sms) * 16 ? want : static_cast<size_t>(sms) * 16);
        convert_bf16_to_f16_kernel<<<blocks, 256, 0, s>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), n, counters);
        e = cudaGetLastError();
        if (e != cudaSuccess) return fail(DC_CUDA_ERROR, "launch failed", cudaGetErrorString(e));
    }
    unsigned long long host[4] = {0, 0, 0, 0};
    e = cudaMemcpyAsync(host, counters, sizeof host, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(DC_CUDA_ERROR, "reading the counters back failed", cudaGetErrorString(e));
    if (report) {
        report->values += n;
        report->f16_subnormal += host[1];
        report->f16_flushed_to_zero += host[2];
        report->f16_overflow += host[3];
    }
    return DC_OK;
}

int dc_rmsnorm(dc_ctx* ctx, void* stream, const float* x, const float* w, void* y, const uint32_t* rowmap, uint32_t rows,
               uint32_t h, uint32_t ld_in, uint32_t ld_out, float eps, uint32_t add_one) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, x && w && y, "rmsnorm: null operand");
    DC_REQUIRE(ctx, h <= ld_in && h <= ld_out, "rmsnorm: H = %u exceeds a row stride (ld_in = %u, ld_out = %u)", h, ld_in, ld_out);
    DC_REQUIRE(ctx, h % 4 == 0 && ld_in % 4 == 0 && ld_out % 4 == 0 && h > 0, "rmsnorm: H and the row strides must be multiples of 4");
    DC_REQUIRE(ctx, aligned16(x) && aligned16(w) && reinterpret_cast<uintptr_t>(y) % 8 == 0, "rmsnorm: misaligned operand");
    if (rows == 0) return DC_OK;
    if (h == 2560) {   // the benchmark model's hidden size: the register-resident form
        if (ctx->act_dtype == DC_ACT_F16)
            rmsnorm_reg_kernel<ActF16, 20><<<blocks_for(rows), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(
                x, w, static_cast<uint16_t*>(y), rowmap, rows, ld_in, ld_out, eps, add_one);
        else
            rmsnorm_reg_kernel<ActBF16, 20><<<blocks_for(rows), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(
                x, w, static_cast<uint16_t*>(y), rowmap, rows, ld_in, ld_out, eps, add_one);
    } else if (ctx->act_dtype == DC_ACT_F16)
        rmsnorm_kernel<ActF16><<<blocks_for(rows), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(
            x, w, static_cast<uint16_t*>(y), rowmap, rows, h, ld_in, ld_out, eps, add_one);
    else
        rmsnorm_kernel<ActBF16><<<blocks_for(rows), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(
            x, w, static_cast<uint16_t*>(y), rowmap, rows, h, ld_in, ld_out, eps, add_one);
    return dc_check_launch(ctx, "rmsnorm");
}

static int add_rmsnorm_any(dc_ctx* ctx, void* stream, float* x, const void* add, bool add16, const float* w, void* y, uint32_t rows, uint32_t h, float eps,
                           uint32_t add_one) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, x && add && (!y || w), "add_rmsnorm: null operand");
    DC_REQUIRE(ctx, h % 4 == 0 && h > 0, "add_rmsnorm: H = %u must be a multiple of 4", h);
    DC_REQUIRE(ctx, aligned16(x) && aligned16(add) && (!y || (aligned16(w) && reinterpret_cast<uintptr_t>(y) % 8 == 0)), "add_rmsnorm: misaligned operand");
    if (rows == 0) return DC_OK;
    const bool f16 = ctx->act_dtype == DC_ACT_F16;
    auto go = [&](auto kern) { kern<<<blocks_for(rows), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(x, add, w, static_cast<uint16_t*>(y), rows, h, eps, add_one); };
    if (h == 2560) {
        if (add16) f16 ? go(add_rmsnorm_kernel<ActF16, true, 20>) : go(add_rmsnorm_kernel<ActBF16, true, 20>);
        else f16 ? go(add_rmsnorm_kernel<ActF16, false, 20>) : go(add_rmsnorm_kernel<ActBF16, false, 20>);
    } else {
        if (add16) f16 ? go(add_rmsnorm_kernel<ActF16, true, 0>) : go(add_rmsnorm_kernel<ActBF16, true, 0>);
        else f16 ? go(add_rmsnorm_kernel<ActF16, false, 0>) : go(add_rmsnorm_kernel<ActBF16, false, 0>);
    }
    return dc_check_launch(ctx, "add_rmsnorm");
}

int dc_add_rmsnorm(dc_ctx* ctx, void* stream, float* x, const float* add, const float* w, void* y, uint32_t rows, uint32_t h, float eps,
                   uint32_t add_one) {
    return add_rmsnorm_any(ctx, stream, x, add, false, w, y, rows, h, eps, add_one);
}

int dc_add16_rmsnorm(dc_ctx* ctx, void* stream, float* x, const void* add16, const float* w, void* y, uint32_t rows, uint32_t h, float eps,
                     uint32_t add_one) {
    return add_rmsnorm_any(ctx, stream, x, add16, true, w, y, rows, h, eps, add_one);
}

int dc_embed(dc_ctx* ctx, void* stream, const uint32_t* ids, const void* table, float* out, uint32_t t, uint32_t h) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, ids && table && out, "embed: null operand");
    DC_REQUIRE(ctx, h % 4 == 0 && h > 0, "embed: H = %u must be a multiple of 4", h);
    DC_REQUIRE(ctx, reinterpret_cast<uintptr_t>(table) % 8 == 0 && aligned16(out), "embed: misaligned operand");
    if (t == 0) return DC_OK;
    embed_kernel<<<blocks_for(t), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        ids, static_cast<const __nv_bfloat16*>(table), out, t, h);
    return dc_check_launch(ctx, "embed");
}

static int gather_rows(dc_ctx* ctx, void* stream, const void* x, const uint32_t* rowmap, void* out, uint32_t rows,
                       size_t row_bytes, const char* what) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, x && rowmap && out, "%s: null operand", what);
    DC_REQUIRE(ctx, row_bytes % 16 == 0 && row_bytes > 0 && aligned16(x) && aligned16(out), "%s: rows must be whole 16-byte vectors", what);
    if (rows == 0) return DC_OK;
    gather_rows_kernel<<<blocks_for(rows), kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(x), rowmap, static_cast<uint4*>(out), rows, static_cast<uint32_t>(row_bytes / 16));
    return dc_check_launch(ctx, what);
}

int dc_gather_rows_f32(dc_ctx* ctx, void* stream, const float* x, const uint32_t* rowmap, float* out, uint32_t rows, uint32_t h) {
    return gather_rows(ctx, stream, x, rowmap, out, rows, static_cast<size_t>(h) * 4, "gather_rows_f32");
}

int dc_gather_rows_bf16(dc_ctx* ctx, void* stream, const void* x, const uint32_t* rowmap, void* out, uint32_t rows, uint32_t h) {
    return gather_rows(ctx, stream, x, rowmap, out, rows, static_cast<size_t>(h) * 2, "gather_rows_bf16");
}

int dc_final_head(dc_ctx* ctx, void* stream, const float* x, const float* w, const void* table, const uint32_t* cand,
                  const uint32_t* ncand, float* logits, uint32_t rows, uint32_t h, uint32_t max_cand, float eps) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, x && w && table && cand && ncand && logits, "final_head: null operand");
    DC_REQUIRE(ctx, h % 4 == 0 && h > 0 && max_cand >= 1, "final_head: H = %u must be a multiple of 4 and max_cand >= 1", h);
    DC_REQUIRE(ctx, aligned16(x) && aligned16(w) && reinterpret_cast<uintptr_t>(table) % 8 == 0, "final_head: misaligned operand");
    if (rows == 0) return DC_OK;
    dim3 grid(rows, (max_cand + kWarpsPerBlock - 1) / kWarpsPerBlock);
    final_head_kernel<<<grid, kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        x, w, static_cast<const __nv_bfloat16*>(table), cand, ncand, logits, h, max_cand, eps);
    return dc_check_launch(ctx, "final_head");
}

int dc_gated_rmsnorm_silu(dc_ctx* ctx, void* stream, const float* o, const float* z, const float* w, void* y, uint32_t t,
                          uint32_t nv, uint32_t dv, uint32_t ldz, float eps) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, o && z && w && y, "gated_rmsnorm_silu: null operand");
    if (dv != 128) return dc_fail(ctx, DC_UNSUPPORTED, "gated_rmsnorm_silu: value head dim %u (built for 128)", dv);
    DC_REQUIRE(ctx, ldz >= nv * dv && ldz % 4 == 0, "gated_rmsnorm_silu: ldz = %u must cover %u columns and be a multiple of 4", ldz, nv * dv);
    DC_REQUIRE(ctx, aligned16(o) && aligned16(z) && aligned16(w) && reinterpret_cast<uintptr_t>(y) % 8 == 0, "gated_rmsnorm_silu: misaligned operand");
    if (t == 0) return DC_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool f16 = ctx->act_dtype == DC_ACT_F16;
    uint16_t* out = static_cast<uint16_t*>(y);
    if (nv % 4 == 0) {   // four heads per warp
        if (f16) gated_rmsnorm_silu_kernel<ActF16, 4><<<blocks_for(t * (nv / 4)), kWarpsPerBlock * 32, 0, st>>>(o, z, w, out, t, nv, ldz, eps);
        else gated_rmsnorm_silu_kernel<ActBF16, 4><<<blocks_for(t * (nv / 4)), kWarpsPerBlock * 32, 0, st>>>(o, z, w, out, t, nv, ldz, eps);
    } else {
        if (f16) gated_rmsnorm_silu_kernel<ActF16, 1><<<blocks_for(t * nv), kWarpsPerBlock * 32, 0, st>>>(o, z, w, out, t, nv, ldz, eps);
        else gated_rmsnorm_silu_kernel<ActBF16, 1><<<blocks_for(t * nv), kWarpsPerBlock * 32, 0, st>>>(o, z, w, out, t, nv, ldz, eps);
    }
    return dc_check_launch(ctx, "gated_rmsnorm_silu");
}

}  // extern "C"
