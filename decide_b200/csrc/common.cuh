// Shared host-side declarations of the library: the context object behind the
// opaque dc_ctx handle, error latching, and small device helpers.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <tuple>

#include "../../include/decide_cuda.h"

typedef CUresult (*dc_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                       CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                       CUtensorMapFloatOOBfill);

// (base pointer, rows, cols, row stride in elements, box rows)
typedef std::tuple<const void*, uint32_t, uint32_t, uint32_t, uint32_t> dc_tmap_key;

struct dc_ctx {
    int device = 0;
    int sm_count = 0;
    int smem_optin = 0;
    int* status_dev = nullptr;       // device status word, 0 = healthy; set by a kernel whose bounded wait ran out
    int* status_host = nullptr;      // pinned staging for dc_check_status
    std::string last_error;          // latched message, cleared when read
    dc_encode_tiled_fn encode_tiled = nullptr;
    std::map<dc_tmap_key, CUtensorMap> tmaps;   // tensor-map cache, filled on first use of an operand
    uint64_t launches = 0;           // kernels enqueued through this context
    uint32_t gemm_impl = DC_IMPL_FAST;
    uint32_t attn_impl = DC_IMPL_FAST;
    uint32_t delta_impl = DC_IMPL_FAST;
    uint32_t delta_engine = DC_ENGINE_TCGEN05;  // serial kernel of the chunked delta rule (split 3)
    uint32_t attn_engine = DC_ENGINE_TCGEN05;   // fast attention for packed batches
    uint32_t delta_split = 3;         // chunked delta rule: 3 = hi/lo split operands (near fp32), 1 = single bf16 pass
    uint32_t act_dtype = DC_ACT_F16;  // type of every 16-bit GEMM operand: activations and weight matrices
    float* gemm_part_ws = nullptr;   // partial accumulators of K-split tail tiles: sm_count x 128 x 256 fp32
    int* gemm_part_cnt = nullptr;    // arrival counters of split tiles: sm_count x 4 row quadrants, zero between launches
    void* workspace = nullptr;       // scratch for the chunked delta rule and other multi-pass ops
    size_t workspace_bytes = 0;
    bool workspace_frozen = false;   // an op that needs more scratch than is reserved fails instead of allocating
    uint64_t allocs = 0;             // device/pinned allocations this context made (dc_open, workspace growth)
    uint64_t tmap_encodes = 0;       // tensor maps encoded (cache misses)
    void* tp_comm = nullptr;         // NCCL communicator of the tensor-parallel group (dc_tp_init), or null
    uint32_t tp_world = 1, tp_rank = 0;
    bool tp_exchange16 = false;      // partial sums cross the links in the 16-bit type (half the bytes) instead of fp32
};

int dc_fail(dc_ctx* ctx, int code, const char* fmt, ...);
int dc_check_launch(dc_ctx* ctx, const char* what);
// Hands out the context's scratch workspace, at least `bytes` long, in *out. Growing it frees and
// allocates device memory (a device-wide synchronisation): callers that must not allocate inside a
// request reserve up front (dc_reserve_workspace) and freeze it (dc_set_workspace_frozen), after
// which a larger demand is DC_INVALID_ARG naming `who`.
int dc_get_workspace(dc_ctx* ctx, size_t bytes, const char* who, void** out);
// One-time per-device kernel set-up of each family (opt-in shared-memory sizes): what dc_warm_up runs.
int dc_gemm_warm(dc_ctx* ctx);
int dc_attention_warm(dc_ctx* ctx);
int dc_attention_tc_warm(dc_ctx* ctx);
int dc_delta_chunk_warm(dc_ctx* ctx);
// Cached 2-D tensor map over a 16-bit row-major matrix [rows][cols] (row stride ld elements): boxes of
// box_rows x 64 elements, 128-byte swizzle, zero fill outside the matrix.
int dc_make_tmap(dc_ctx* ctx, const void* base, uint32_t rows, uint32_t cols, uint32_t ld, uint32_t box_rows, bool f16, CUtensorMap* out);
// Status-word value that is not a wait id: a query position at or past the cache length the caller gave (dc_attention).
#define DC_STATUS_POSITION_PAST_CACHE 70
// tcgen05 attention for packed prefill batches, or (seq_start null) `rows` query rows of one sequence over cache rows
// 0 .. kv_len (attn_tc.cu), and the scratch it takes from the workspace.
int dc_attention_tc(dc_ctx* ctx, cudaStream_t s, const void* q, const void* kc, const void* vc, const float* gate, const uint32_t* qpos, void* y,
                    uint32_t rows, uint32_t ldg, uint32_t nq, uint32_t nkv, const uint32_t* seq_start, uint32_t n_seq, uint32_t max_len, uint32_t kv_len);
size_t dc_attention_tc_scratch_bytes(uint32_t rows, uint32_t n_seq, uint32_t nkv);

#define DC_REQUIRE(ctx, cond, ...)                                            \
    do {                                                                      \
        if (!(cond)) return dc_fail((ctx), DC_INVALID_ARG, __VA_ARGS__);      \
    } while (0)

namespace dc {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + __expf(-x)); }
// Precise: feeds the recurrence's decay gate, whose error compounds over tokens.
__device__ __forceinline__ float softplus_precise(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// The two 16-bit formats. Every 16-bit GEMM operand of a context, activations (normed rows, gated
// outputs, the MLP intermediate, attention q/k/v) and weight matrices alike, is stored in that
// context's type; the embedding table is always bf16.
struct ActBF16 {
    static constexpr uint32_t kUmmaFormat = 1;  // tcgen05 instruction-descriptor code for bf16
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    static __device__ __forceinline__ float lo(uint32_t v) { return __uint_as_float(v << 16); }
    static __device__ __forceinline__ float hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
    static __device__ __forceinline__ float one(uint16_t v) { return __uint_as_float(static_cast<uint32_t>(v) << 16); }
    static __device__ __forceinline__ uint16_t to16(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
};
struct ActF16 {
    static constexpr uint32_t kUmmaFormat = 0;  // fp16
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    static __device__ __forceinline__ float lo(uint32_t v) { return __half2float(__ushort_as_half(static_cast<unsigned short>(v & 0xffffu))); }
    static __device__ __forceinline__ float hi(uint32_t v) { return __half2float(__ushort_as_half(static_cast<unsigned short>(v >> 16))); }
    static __device__ __forceinline__ float one(uint16_t v) { return __half2float(__ushort_as_half(v)); }
    static __device__ __forceinline__ uint16_t to16(float f) { return __half_as_ushort(__float2half_rn(f)); }
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

}  // namespace dc
