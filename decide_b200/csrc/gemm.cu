// dc_gemm: argument contract, kernel choice, and the baseline kernel.
//
// The contract is the reference's Gemm::gemm (crates/decide-engine/src/kernels/gemm.rs:138-175):
// Y = X * W^T, fp32 accumulation, four epilogues. `fast` = the tcgen05 kernels of gemm_tc.cu;
// `baseline` = a plain shared-memory-tiled CUDA-core kernel kept, like the reference's
// kernels/gemm.metal, so that parity problems can be bisected (DECIDE_GEMM=baseline).
#include "common.cuh"

int dc_gemm_tc(dc_ctx* ctx, cudaStream_t stream, const void* x, const void* w, void* y, uint32_t m, uint32_t n,
               uint32_t k, uint32_t ldx, uint32_t ldw, uint32_t ldy, uint32_t epi, uint32_t bn_override);
uint32_t dc_gemm_plan_bn(uint32_t m, uint32_t n, uint32_t k, int sm_count);
int dc_gemm_small(dc_ctx* ctx, cudaStream_t s, const void* x, const void* w, void* y, uint32_t m, uint32_t n, uint32_t k, uint32_t ldx,
                  uint32_t ldw, uint32_t ldy, uint32_t epi);

namespace {

using namespace dc;

constexpr int RT = 64;   // output tile edge of the baseline kernel
constexpr int RK = 16;   // its k step

// One thread computes a 4 x 4 patch of the 64 x 64 output tile. For the SwiGLU epilogue the tile is
// 64 OUTPUT columns: column j pairs W row gate(j) = (j / sb) * 2 sb + j % sb with row gate(j) + sb.
template <int EPI, typename Act>
__global__ void __launch_bounds__(256)
gemm_baseline_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, void* __restrict__ y,
                     uint32_t m, uint32_t n, uint32_t k, uint32_t ldx, uint32_t ldw, uint32_t ldy, uint32_t sb) {
    constexpr bool kSwiglu = (EPI == DC_EPI_SWIGLU_BF16);
    __shared__ float xs[RK][RT + 1];
    __shared__ float ws[kSwiglu ? 2 : 1][RK][RT + 1];
    const uint32_t n_out = kSwiglu ? n / 2 : n;
    const uint32_t row0 = blockIdx.y * RT, col0 = blockIdx.x * RT;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[kSwiglu ? 2 : 1][4][4] = {};

    for (uint32_t k0 = 0; k0 < k; k0 += RK) {
        // 64 rows x 16 k-values per operand tile: 1024 elements, 4 per thread
        for (int e = threadIdx.x; e < RT * RK; e += 256) {
            const int r = e / RK, kk = e % RK;
            const uint32_t gr = row0 + r;
            xs[kk][r] = (gr < m && k0 + kk < k) ? Act::one(x[static_cast<size_t>(gr) * ldx + k0 + kk]) : 0.0f;
            const uint32_t j = col0 + r;
            if (j < n_out && k0 + kk < k) {
                if constexpr (kSwiglu) {
                    const uint32_t g = (j / sb) * 2 * sb + (j % sb);
                    ws[0][kk][r] = Act::one(w[static_cast<size_t>(g) * ldw + k0 + kk]);
                    ws[1][kk][r] = Act::one(w[static_cast<size_t>(g + sb) * ldw + k0 + kk]);
                } else {
                    ws[0][kk][r] = Act::one(w[static_cast<size_t>(j) * ldw + k0 + kk]);
                }
            } else {
                ws[0][kk][r] = 0.0f;
                if constexpr (kSwiglu) ws[1][kk][r] = 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < RK; ++kk) {
            float xv[4], wv[kSwiglu ? 2 : 1][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int p = 0; p < (kSwiglu ? 2 : 1); ++p)
#pragma unroll
                for (int j = 0; j < 4; ++j) wv[p][j] = ws[p][kk][tx * 4 + j];
#pragma unroll
            for (int p = 0; p < (kSwiglu ? 2 : 1); ++p)
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[p][i][j] = fmaf(xv[i], wv[p][j], acc[p][i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t r = row0 + ty * 4 + i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t c = col0 + tx * 4 + j;
            if (c >= n_out) continue;
            const size_t o = static_cast<size_t>(r) * ldy + c;
            if constexpr (EPI == DC_EPI_STORE_F32) static_cast<float*>(y)[o] = acc[0][i][j];
            else if constexpr (EPI == DC_EPI_ADD_F32) static_cast<float*>(y)[o] += acc[0][i][j];
            else if constexpr (EPI == DC_EPI_STORE_BF16) static_cast<uint16_t*>(y)[o] = Act::to16(acc[0][i][j]);
            else {
                const float g = acc[0][i][j];
                static_cast<uint16_t*>(y)[o] = Act::to16(g / (1.0f + expf(-g)) * acc[1][i][j]);
            }
        }
    }
}

template <int EPI>
int launch_baseline(dc_ctx* ctx, cudaStream_t s, const void* x, const void* w, void* y, uint32_t m, uint32_t n, uint32_t k,
                    uint32_t ldx, uint32_t ldw, uint32_t ldy, uint32_t sb) {
    const uint32_t n_out = EPI == DC_EPI_SWIGLU_BF16 ? n / 2 : n;
    dim3 grid((n_out + RT - 1) / RT, (m + RT - 1) / RT);
    if (ctx->act_dtype == DC_ACT_F16)
        gemm_baseline_kernel<EPI, ActF16><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(w), y, m, n, k, ldx, ldw, ldy, sb);
    else
        gemm_baseline_kernel<EPI, ActBF16><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(w), y, m, n, k, ldx, ldw, ldy, sb);
    return dc_check_launch(ctx, "gemm (baseline)");
}

}  // namespace

extern "C" int dc_gemm(dc_ctx* ctx, void* stream, const void* x, const void* w, void* y, uint32_t m, uint32_t n,
                       uint32_t k, uint32_t ldx, uint32_t ldw, uint32_t ldy, uint32_t epilogue, uint32_t swiglu_block) {
    if (!ctx) return DC_INVALID_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DC_REQUIRE(ctx, x && w && y, "gemm: null operand");
    DC_REQUIRE(ctx, epilogue <= DC_EPI_SWIGLU_BF16, "gemm: unknown epilogue %u", epilogue);
    DC_REQUIRE(ctx, n % 32 == 0 && k % 32 == 0 && n > 0 && k > 0, "gemm: N = %u and K = %u must be multiples of 32", n, k);
    DC_REQUIRE(ctx, m >= 1, "gemm: M must be at least 1");
    DC_REQUIRE(ctx, ldx >= k && ldw >= k, "gemm: row strides ldx = %u, ldw = %u must cover K = %u", ldx, ldw, k);
    const uint32_t y_cols = epilogue == DC_EPI_SWIGLU_BF16 ? n / 2 : n;
    DC_REQUIRE(ctx, ldy >= y_cols, "gemm: row stride ldy = %u must cover the %u output columns", ldy, y_cols);
    if (epilogue == DC_EPI_SWIGLU_BF16)
        DC_REQUIRE(ctx, swiglu_block >= 1 && n % (2 * swiglu_block) == 0, "gemm: N = %u is not a whole number of gate|up block pairs of %u", n, swiglu_block);

    if (ctx->gemm_impl == DC_IMPL_BASELINE) {
        switch (epilogue) {
            case DC_EPI_STORE_F32: return launch_baseline<DC_EPI_STORE_F32>(ctx, s, x, w, y, m, n, k, ldx, ldw, ldy, swiglu_block);
            case DC_EPI_STORE_BF16: return launch_baseline<DC_EPI_STORE_BF16>(ctx, s, x, w, y, m, n, k, ldx, ldw, ldy, swiglu_block);
            case DC_EPI_ADD_F32: return launch_baseline<DC_EPI_ADD_F32>(ctx, s, x, w, y, m, n, k, ldx, ldw, ldy, swiglu_block);
            default: return launch_baseline<DC_EPI_SWIGLU_BF16>(ctx, s, x, w, y, m, n, k, ldx, ldw, ldy, swiglu_block);
        }
    }

    // Fast path: what TMA (16-byte rows and bases) and the vector stores of the epilogue need.
    DC_REQUIRE(ctx, ldx % 8 == 0 && ldw % 8 == 0, "gemm (fast): ldx = %u and ldw = %u must be multiples of 8", ldx, ldw);
    DC_REQUIRE(ctx, reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0,
               "gemm (fast): x and w must be 16-byte aligned");
    const bool out_f32 = epilogue == DC_EPI_STORE_F32 || epilogue == DC_EPI_ADD_F32;
    DC_REQUIRE(ctx, ldy % (out_f32 ? 4 : 8) == 0, "gemm (fast): ldy = %u must be a multiple of %d", ldy, out_f32 ? 4 : 8);
    DC_REQUIRE(ctx, reinterpret_cast<uintptr_t>(y) % 16 == 0, "gemm (fast): y must be 16-byte aligned");
    if (epilogue == DC_EPI_SWIGLU_BF16 && swiglu_block != 16)
        return dc_fail(ctx, DC_UNSUPPORTED, "gemm (fast): the SwiGLU epilogue pairs columns 16 apart; swiglu_block = %u", swiglu_block);
    // M <= 16 (answer rows): the weight-streaming kernel, as the reference's table picks gemm_nt_small (gemm_configs.rs:252-267)
    if (m <= DC_GEMM_SMALL_MAX_M) return dc_gemm_small(ctx, s, x, w, y, m, n, k, ldx, ldw, ldy, epilogue);
    return dc_gemm_tc(ctx, s, x, w, y, m, n, k, ldx, ldw, ldy, epilogue, 0);
}

// Test hook: the fast kernel with a forced tile width (128 or 256), so both instantiations are
// exercised whatever the plan would pick.
extern "C" int dc_gemm_tile(dc_ctx* ctx, void* stream, const void* x, const void* w, void* y, uint32_t m, uint32_t n,
                            uint32_t k, uint32_t ldx, uint32_t ldw, uint32_t ldy, uint32_t epilogue, uint32_t bn) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, bn == 128 || bn == 192 || bn == 224 || bn == 256, "gemm: tile width %u is not 128, 192, 224 or 256", bn);
    DC_REQUIRE(ctx, x && w && y && m >= 1 && n % 32 == 0 && k % 32 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldy % 8 == 0 &&
                        epilogue <= DC_EPI_SWIGLU_BF16,
               "gemm: bad arguments");
    return dc_gemm_tc(ctx, static_cast<cudaStream_t>(stream), x, w, y, m, n, k, ldx, ldw, ldy, epilogue, bn);
}

extern "C" uint32_t dc_gemm_plan(dc_ctx* ctx, uint32_t m, uint32_t n) {
    return dc_gemm_plan_bn(m, n, 0, ctx ? ctx->sm_count : 148);
}
