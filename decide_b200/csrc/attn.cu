// Causal grouped-query attention with the optional sigmoid output gate, head_dim 128.
// Replaces kernels/attn_fast.metal (fast) and kernels/attn.metal (baseline); spec cpu_ref.rs:167-188.
//
// Fast kernel: one CTA per (64 query rows, query head, sequence); 4 warps x 16 rows. K and V tiles of
// 64 cache rows are staged in XOR-swizzled shared memory; QK^T and PV run on mma.sync m16n8k16 bf16
// with fp32 accumulators; softmax is online in fp32 with exp2 (log2 e folded into the scale). As in
// the reference's fast kernel (attn_fast.metal:270-282) the weights are rounded to the MMA operand
// type once and the row sum is taken over the ROUNDED weights, so outputs are exactly normalised;
// masked scores use a finite -1e30 sentinel (attn.metal:20-21). The gate is applied in the store.
//
// Baseline kernel: one warp per (row, head) walking the cache one position at a time in fp32.
#include "common.cuh"

namespace {

using namespace dc;

constexpr int HD = 128;
constexpr int BQ = 64;   // query rows per CTA
constexpr int BKV = 64;  // cache rows per tile
constexpr int kThreads = 128;
constexpr float kMasked = -1e30f;
constexpr uint32_t kTcMinChunkRows = 64;   // a chunk of at least this many rows over a longer cache runs on the tcgen05 kernel

// element (row, col) of a [rows][128] bf16 tile: 16-byte chunks XOR-swizzled by the row
__device__ __forceinline__ uint32_t tile_off(int row, int col) {
    return static_cast<uint32_t>(row * HD + ((((col >> 3) ^ (row & 7)) << 3) | (col & 7)));
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const uint16_t* p) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const uint16_t* p) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
template <typename Act>
__device__ __forceinline__ void mma_16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (Act::kUmmaFormat == 1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Copies `nrows` x 128 bf16 (rows beyond `valid` zero-filled) from global (row stride `ld`) into a swizzled tile.
__device__ __forceinline__ void load_tile(uint16_t* tile, const uint16_t* src, size_t ld, int valid) {
    for (int e = threadIdx.x; e < BKV * (HD / 8); e += kThreads) {
        const int r = e >> 4, c = e & 15;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (r < valid) val = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * ld + c * 8);
        *reinterpret_cast<uint4*>(tile + tile_off(r, c * 8)) = val;
    }
}

// The same copy with cp.async (16 bytes per request, zero fill past `valid`): completes with the
// thread's next cp.async.wait_group, so the next K/V tiles stream in under the current tile's MMAs.
// Thread t copies chunk (t & 15) of rows (t >> 4) + 8 i: the swizzled chunk position is the same for
// all its rows, so source and destination advance by constants.
__device__ __forceinline__ void load_tile_async(uint16_t* tile, const uint16_t* src, size_t ld, int valid) {
    const int r0 = threadIdx.x >> 4, c = threadIdx.x & 15;
    uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(tile + tile_off(r0, c * 8)));
    const uint16_t* g = src + static_cast<size_t>(r0) * ld + c * 8;
#pragma unroll
    for (int i = 0; i < BKV / 8; ++i) {
        const int bytes = r0 + 8 * i < valid ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(bytes ? g : src), "r"(bytes) : "memory");
        dst += 8 * HD * 2;
        g += 8 * ld;
    }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename Act>
__global__ void __launch_bounds__(kThreads, 3)
attn_fast_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ kc, const uint16_t* __restrict__ vc,
                 const float* __restrict__ gate, const uint32_t* __restrict__ qpos, uint16_t* __restrict__ y, uint32_t rows,
                 uint32_t ldg, uint32_t nq, uint32_t nkv, float scale_log2, const uint32_t* __restrict__ seq_start) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint16_t* kv_tiles = reinterpret_cast<uint16_t*>(smem_raw);   // two stages of (K tile, V tile)
    uint16_t* qs = kv_tiles + 2 * BKV * HD;                       // the Q tile borrows stage 1 until its fragments are in registers
    int* qp = reinterpret_cast<int*>(kv_tiles + 4 * BKV * HD);  // [BQ] position of each query row, -1 = no row

    const uint32_t seq = blockIdx.z, h = blockIdx.y, kvh = h / (nq / nkv);
    const uint32_t row_lo = seq_start ? seq_start[seq] : 0u;
    const uint32_t len = seq_start ? seq_start[seq + 1] - row_lo : rows;
    const uint32_t qb = gridDim.x - 1 - blockIdx.x;  // longest rows first
    const uint32_t r0 = qb * BQ;
    if (r0 >= len) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int valid_q = min(static_cast<int>(len - r0), BQ);

    load_tile(qs, q + (static_cast<size_t>(row_lo + r0) * nq + h) * HD, static_cast<size_t>(nq) * HD, valid_q);
    if (threadIdx.x < BQ) qp[threadIdx.x] = static_cast<int>(threadIdx.x) < valid_q ? static_cast<int>(qpos[row_lo + r0 + threadIdx.x]) : -1;
    __syncthreads();
    int kv_end = 0;
    for (int i = 0; i < BQ; ++i) kv_end = max(kv_end, qp[i] + 1);

    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk)
        ldsm_x4(qf[kk], qs + tile_off(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kk * 16 + (lane >> 4) * 8));

    const int qp0 = qp[warp * 16 + (lane >> 2)], qp1 = qp[warp * 16 + (lane >> 2) + 8];
    int qp_warp_max = max(qp0, qp1), qp_warp_min = min(qp0, qp1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        qp_warp_max = max(qp_warp_max, __shfl_xor_sync(0xffffffffu, qp_warp_max, o));
        qp_warp_min = min(qp_warp_min, __shfl_xor_sync(0xffffffffu, qp_warp_min, o));
    }
    float m0 = kMasked, m1 = kMasked, l0 = 0.f, l1 = 0.f;
    float oacc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;

    const uint16_t* kbase = kc + (static_cast<size_t>(row_lo) * nkv + kvh) * HD;
    const uint16_t* vbase = vc + (static_cast<size_t>(row_lo) * nkv + kvh) * HD;
    const size_t ldkv = static_cast<size_t>(nkv) * HD;

    __syncthreads();  // every warp has its Q fragments: stage 1 may be overwritten
    // two-stage pipeline: tile it+1 is in flight while tile it is multiplied
    load_tile_async(kv_tiles, kbase, ldkv, min(kv_end, BKV));
    load_tile_async(kv_tiles + BKV * HD, vbase, ldkv, min(kv_end, BKV));
    cp_async_commit();
    int stage = 0;
    for (int j0 = 0; j0 < kv_end; j0 += BKV, stage ^= 1) {
        const int j1 = j0 + BKV;
        if (j1 < kv_end) {
            uint16_t* nxt = kv_tiles + (stage ^ 1) * 2 * BKV * HD;
            load_tile_async(nxt, kbase + static_cast<size_t>(j1) * ldkv, ldkv, min(kv_end - j1, BKV));
            load_tile_async(nxt + BKV * HD, vbase + static_cast<size_t>(j1) * ldkv, ldkv, min(kv_end - j1, BKV));
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint16_t* ks = kv_tiles + stage * 2 * BKV * HD;
        const uint16_t* vs = ks + BKV * HD;

        // 16-column groups of this tile that at least one row of this warp may see, and whether the whole
        // tile is visible to every row of the warp (then no mask is needed); both warp-uniform
        const int np_lim = qp_warp_max < j0 ? 0 : min(BKV / 16, (qp_warp_max - j0) / 16 + 1);
        const bool no_mask = j0 + BKV - 1 <= qp_warp_min;

        float sacc[BKV / 8][4];
#pragma unroll
        for (int i = 0; i < BKV / 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
        if (np_lim > 0) {
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
                for (int np = 0; np < BKV / 16; ++np) {
                    if (np < np_lim) {
                        uint32_t bfr[4];
                        ldsm_x4(bfr, ks + tile_off(np * 16 + (lane & 7) + (lane >> 4) * 8, kk * 16 + ((lane >> 3) & 1) * 8));
                        mma_16<Act>(sacc[2 * np], qf[kk], bfr[0], bfr[1]);
                        mma_16<Act>(sacc[2 * np + 1], qf[kk], bfr[2], bfr[3]);
                    }
                }
            }
        }
        // scale, causal mask, running max
        float mx0 = kMasked, mx1 = kMasked;
        if (no_mask) {
#pragma unroll
            for (int i = 0; i < BKV / 8; ++i) {
                sacc[i][0] *= scale_log2;
                sacc[i][1] *= scale_log2;
                sacc[i][2] *= scale_log2;
                sacc[i][3] *= scale_log2;
                mx0 = fmaxf(mx0, fmaxf(sacc[i][0], sacc[i][1]));
                mx1 = fmaxf(mx1, fmaxf(sacc[i][2], sacc[i][3]));
            }
        } else {
#pragma unroll
            for (int i = 0; i < BKV / 8; ++i) {
                const int c = j0 + i * 8 + 2 * (lane & 3);
                sacc[i][0] = c <= qp0 ? sacc[i][0] * scale_log2 : kMasked;
                sacc[i][1] = c + 1 <= qp0 ? sacc[i][1] * scale_log2 : kMasked;
                sacc[i][2] = c <= qp1 ? sacc[i][2] * scale_log2 : kMasked;
                sacc[i][3] = c + 1 <= qp1 ? sacc[i][3] * scale_log2 : kMasked;
                mx0 = fmaxf(mx0, fmaxf(sacc[i][0], sacc[i][1]));
                mx1 = fmaxf(mx1, fmaxf(sacc[i][2], sacc[i][3]));
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float corr0 = ex2(m0 - mn0), corr1 = ex2(m1 - mn1);
        m0 = mn0;
        m1 = mn1;
        float rs0 = 0.f, rs1 = 0.f;
        uint32_t pf[BKV / 16][4];
#pragma unroll
        for (int i = 0; i < BKV / 8; ++i) {
            // a masked score stays masked even when the whole row is masked so far (m = sentinel)
            const float p0 = sacc[i][0] > 0.5f * kMasked ? ex2(sacc[i][0] - mn0) : 0.f;
            const float p1 = sacc[i][1] > 0.5f * kMasked ? ex2(sacc[i][1] - mn0) : 0.f;
            const float p2 = sacc[i][2] > 0.5f * kMasked ? ex2(sacc[i][2] - mn1) : 0.f;
            const float p3 = sacc[i][3] > 0.5f * kMasked ? ex2(sacc[i][3] - mn1) : 0.f;
            const uint32_t lo = Act::pack(p0, p1), hi = Act::pack(p2, p3);
            rs0 += Act::lo(lo) + Act::hi(lo);
            rs1 += Act::lo(hi) + Act::hi(hi);
            pf[i >> 1][(i & 1) * 2] = lo;
            pf[i >> 1][(i & 1) * 2 + 1] = hi;
        }
        l0 = l0 * corr0 + rs0;
        l1 = l1 * corr1 + rs1;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            oacc[i][0] *= corr0;
            oacc[i][1] *= corr0;
            oacc[i][2] *= corr1;
            oacc[i][3] *= corr1;
        }
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
            if (kk >= np_lim) break;   // the weights of those cache rows are all zero for this warp
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                uint32_t bfr[4];
                ldsm_x4_trans(bfr, vs + tile_off(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 16 + (lane >> 4) * 8));
                mma_16<Act>(oacc[2 * dp], pf[kk], bfr[0], bfr[1]);
                mma_16<Act>(oacc[2 * dp + 1], pf[kk], bfr[2], bfr[3]);
            }
        }
        __syncthreads();  // this stage is free for the prefetch of the iteration after next
    }
    // row sums live split over the 4 lanes of a quad
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.0f / l0 : 0.f, inv1 = l1 > 0.f ? 1.0f / l1 : 0.f;
    const int lr0 = warp * 16 + (lane >> 2), lr1 = lr0 + 8;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int d = i * 8 + 2 * (lane & 3);
        if (lr0 < valid_q) {
            const size_t row = row_lo + r0 + lr0;
            float a = oacc[i][0] * inv0, b = oacc[i][1] * inv0;
            if (gate) {
                const float2 g = *reinterpret_cast<const float2*>(gate + row * ldg + h * HD + d);
                a *= sigmoid_f(g.x);
                b *= sigmoid_f(g.y);
            }
            *reinterpret_cast<uint32_t*>(y + (row * nq + h) * HD + d) = Act::pack(a, b);
        }
        if (lr1 < valid_q) {
            const size_t row = row_lo + r0 + lr1;
            float a = oacc[i][2] * inv1, b = oacc[i][3] * inv1;
            if (gate) {
                const float2 g = *reinterpret_cast<const float2*>(gate + row * ldg + h * HD + d);
                a *= sigmoid_f(g.x);
                b *= sigmoid_f(g.y);
            }
            *reinterpret_cast<uint32_t*>(y + (row * nq + h) * HD + d) = Act::pack(a, b);
        }
    }
}

// One warp per (row, head): online softmax over cache rows 0..=qpos, fp32 (attn.metal:6-39).
template <typename Act>
__global__ void __launch_bounds__(256)
attn_baseline_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ kc, const uint16_t* __restrict__ vc,
                     const float* __restrict__ gate, const uint32_t* __restrict__ qpos, uint16_t* __restrict__ y, uint32_t rows,
                     uint32_t ldg, uint32_t nq, uint32_t nkv, float scale, const uint32_t* __restrict__ seq_start, uint32_t n_seq) {
    const uint32_t idx = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (idx >= rows * nq) return;
    const uint32_t r = idx / nq, h = idx - r * nq, kvh = h / (nq / nkv);
    const int lane = threadIdx.x & 31;
    uint32_t row_lo = 0;
    if (seq_start) {
        for (uint32_t s = 0; s < n_seq; ++s)
            if (r >= seq_start[s]) row_lo = seq_start[s];
    }
    const uint2 qv = reinterpret_cast<const uint2*>(q + static_cast<size_t>(idx) * HD)[lane];
    const float q0 = Act::lo(qv.x), q1 = Act::hi(qv.x), q2 = Act::lo(qv.y), q3 = Act::hi(qv.y);
    float m = kMasked, l = 0.f, a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    const uint32_t n = qpos[r] + 1;
    for (uint32_t j = 0; j < n; ++j) {
        const size_t off = (static_cast<size_t>(row_lo + j) * nkv + kvh) * HD;
        const uint2 kvv = reinterpret_cast<const uint2*>(kc + off)[lane];
        float s = q0 * Act::lo(kvv.x) + q1 * Act::hi(kvv.x) + q2 * Act::lo(kvv.y) + q3 * Act::hi(kvv.y);
        s = warp_sum(s) * scale;
        const float mn = fmaxf(m, s);
        const float corr = expf(m - mn), p = expf(s - mn);
        const uint2 vv = reinterpret_cast<const uint2*>(vc + off)[lane];
        l = l * corr + p;
        a0 = a0 * corr + p * Act::lo(vv.x);
        a1 = a1 * corr + p * Act::hi(vv.x);
        a2 = a2 * corr + p * Act::lo(vv.y);
        a3 = a3 * corr + p * Act::hi(vv.y);
        m = mn;
    }
    const float inv = 1.0f / l;
    float o0 = a0 * inv, o1 = a1 * inv, o2 = a2 * inv, o3 = a3 * inv;
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
    reinterpret_cast<uint2*>(y + static_cast<size_t>(idx) * HD)[lane] = out;
}

inline bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace

namespace {
constexpr size_t kFastSmem = 4 * BKV * HD * 2 + BQ * sizeof(int);
}
int dc_attention_warm(dc_ctx* ctx) {
    static bool attr_set[16] = {};
    if (!attr_set[ctx->device & 15]) {
        cudaError_t e = cudaFuncSetAttribute(attn_fast_kernel<ActF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kFastSmem));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_fast_kernel<ActBF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kFastSmem));
        if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "attention: cannot opt in to %zu bytes of shared memory: %s", kFastSmem, cudaGetErrorString(e));
        attr_set[ctx->device & 15] = true;
    }
    return DC_OK;
}

extern "C" int dc_attention(dc_ctx* ctx, void* stream, const void* q, const void* kc, const void* vc, const float* gate,
                            const uint32_t* qpos, void* y, uint32_t rows, uint32_t ldg, uint32_t nq, uint32_t nkv, uint32_t hd,
                            const uint32_t* seq_start, uint32_t n_seq, uint32_t max_len) {
    if (!ctx) return DC_INVALID_ARG;
    DC_REQUIRE(ctx, q && kc && vc && qpos && y, "attention: null operand");
    DC_REQUIRE(ctx, rows >= 1, "attention: rows must be at least 1");
    if (hd != HD) return dc_fail(ctx, DC_UNSUPPORTED, "attention: head_dim %u (built for 128)", hd);
    DC_REQUIRE(ctx, nkv >= 1 && nq % nkv == 0, "attention: %u query heads over %u kv heads", nq, nkv);
    DC_REQUIRE(ctx, !gate || (ldg >= nq * hd && ldg % 4 == 0 && aligned16(gate)), "attention: ldg = %u must cover the gate columns, be a multiple of 4, gate 16-byte aligned", ldg);
    DC_REQUIRE(ctx, aligned16(q) && aligned16(kc) && aligned16(vc) && reinterpret_cast<uintptr_t>(y) % 8 == 0, "attention: q, kc, vc must be 16-byte aligned");
    uint32_t kv_len = 0;   // without seq_start: max_len, if given, is the number of cache rows in use (every position is below it)
    if (!seq_start) {
        n_seq = 1;
        kv_len = max_len;
        max_len = rows;
    }
    DC_REQUIRE(ctx, n_seq >= 1 && n_seq <= 65535 && nq <= 65535, "attention: %u sequences", n_seq);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float scale = 1.0f / sqrtf(static_cast<float>(hd));
    if (ctx->attn_impl == DC_IMPL_BASELINE) {
        auto kern = ctx->act_dtype == DC_ACT_F16 ? attn_baseline_kernel<ActF16> : attn_baseline_kernel<ActBF16>;
        kern<<<(rows * nq + 7) / 8, 256, 0, s>>>(static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(kc), static_cast<const uint16_t*>(vc),
                                                 gate, qpos, static_cast<uint16_t*>(y), rows, ldg, nq, nkv, scale, seq_start, n_seq);
        return dc_check_launch(ctx, "attention (baseline)");
    }
    // The tcgen05 kernel takes packed batches, and a chunk of one sequence that continues a longer cache when the caller says
    // how long the cache is (a short chunk stays on the mma.sync kernel: transposing V for it would cost more than it saves).
    if (ctx->attn_engine == DC_ENGINE_TCGEN05 && (seq_start || (kv_len >= rows && rows >= kTcMinChunkRows)))
        return dc_attention_tc(ctx, s, q, kc, vc, gate, qpos, y, rows, ldg, nq, nkv, seq_start, n_seq, max_len, kv_len);
    constexpr size_t smem = kFastSmem;
    auto fast = ctx->act_dtype == DC_ACT_F16 ? attn_fast_kernel<ActF16> : attn_fast_kernel<ActBF16>;
    {
        const int rc = dc_attention_warm(ctx);
        if (rc != DC_OK) return rc;
    }
    dim3 grid((max_len + BQ - 1) / BQ, nq, n_seq);
    fast<<<grid, kThreads, smem, s>>>(static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(kc),
                                                  static_cast<const uint16_t*>(vc), gate, qpos, static_cast<uint16_t*>(y), rows, ldg,
                                                  nq, nkv, scale * 1.4426950408889634f, seq_start);
    return dc_check_launch(ctx, "attention");
}
