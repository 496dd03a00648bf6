// Y = X * W^T with fused epilogues on the 5th-generation tensor cores (tcgen05), 16-bit operands
// (bf16 or fp16, the context's 16-bit type), fp32 accumulation in tensor memory (TMEM).
//
// Replaces the reference's tiled GEMM `gemm_nt_fast*` (kernels/gemm_fast.metal:289-351) and its
// four epilogues (kernels/gemm.rs:16-26). Structure of one CTA (192 threads, one CTA per SM,
// persistent over output tiles of 128 x BN):
//   warp 0      TMA producer: X tile [128 x 64] and W tile [BN x 64] per k-block into a ring of
//               128-byte-swizzled shared-memory stages (plain loads issued by this CTA for itself only);
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x BN x 16) over each stage and
//               commits the stage back to the producer; owns the TMEM allocation;
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (one row per thread, 32 columns at
//               a time), apply the epilogue, store to global.
// Two accumulators (2 x BN TMEM columns) let the epilogue of tile i overlap the main loop of
// tile i+1. M, N and K tails come from TMA's out-of-bounds zero fill plus masked stores.
// Every mbarrier wait is bounded; on expiry the CTA sets the status word, drains its own
// copies in flight, frees its TMEM and returns.
#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

namespace {

using namespace dc;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;

constexpr uint32_t kGroupM = 16;                             // row tiles walked together (see tile_coords)
constexpr int kEpiLd = 36;                                   // padded row of the per-warp epilogue staging tile
constexpr uint32_t kEpiBytes = 4 * 32 * kEpiLd * 4;          // 4 epilogue warps x [32][36] fp32

struct GemmArgs {
    uint32_t m, n, k, ldy;
    uint32_t m_tiles, n_tiles, k_blocks, group_m;
    uint32_t idesc;  // tcgen05 instruction descriptor: A and B in the context's 16-bit type, D = fp32
    // Work units: the first `full_tiles` tiles are whole tiles; each of the remaining (tail-wave) tiles
    // is cut into `split` parts along K of `kb_per_part` k-blocks, so the last wave fills the SMs too.
    uint32_t full_tiles, split, kb_per_part;
    float* part_ws;   // [tail tile][part][128][BN] fp32 partial accumulators
    int* part_cnt;    // [tail tile][4 row quadrants] arrival counters, zero between launches
};

struct Unit {
    uint32_t tile, part, kb0, kb1;
    bool split;
};
__device__ __forceinline__ Unit unit_of(uint32_t u, const GemmArgs& a) {
    Unit w;
    if (u < a.full_tiles || a.split == 1u) {
        w.tile = u;
        w.part = 0;
        w.kb0 = 0;
        w.kb1 = a.k_blocks;
        w.split = false;
    } else {
        const uint32_t v = u - a.full_tiles;
        w.tile = a.full_tiles + v / a.split;
        w.part = v - (v / a.split) * a.split;
        w.kb0 = w.part * a.kb_per_part;
        w.kb1 = min(a.k_blocks, w.kb0 + a.kb_per_part);
        w.split = true;
    }
    return w;
}

template <int BN>
struct Cfg {
    static constexpr int kStages = BN >= 224 ? 4 : (BN == 192 ? 5 : 6);   // what fits in 227 KB beside the epilogue staging
    static constexpr uint32_t kABytes = BM * BK * 2;
    static constexpr uint32_t kBBytes = BN * BK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr uint32_t kBarBytes = 256;
    static constexpr uint32_t kSmemBytes = 1024 + kStages * kStageBytes + kBarBytes + kEpiBytes;
};

// Output tiles are walked in groups of `group_m` row tiles: inside a group the row tile moves
// fastest, so the CTAs running at one time share a few W stripes and one X group in L2, and W is
// streamed from HBM once per group.
__device__ __forceinline__ void tile_coords(uint32_t t, const GemmArgs& a, uint32_t& tm, uint32_t& tn) {
    const uint32_t per_group = a.group_m * a.n_tiles;
    const uint32_t g = t / per_group;
    const uint32_t local = t - g * per_group;
    const uint32_t m0 = g * a.group_m;
    const uint32_t gsz = min(a.group_m, a.m_tiles - m0);
    tn = local / gsz;
    tm = m0 + (local - tn * gsz);
}

__device__ __forceinline__ bool wait_quiet(uint64_t* bar, uint32_t parity) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > kWaitLimitNs) return false;
    }
    return true;
}


// Bounded wait until an arrival counter in global memory reaches `want` (all parts of a K-split tile have parked their sums).
__device__ __forceinline__ bool wait_at_least(const volatile int* cnt, int want, volatile uint32_t* abort_flag, int* status, int code) {
    if (*cnt >= want) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (*cnt < want) {
        if ((++spins & 63u) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
                *abort_flag = 1u;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
    return true;
}

// One 32-row x 32-column chunk of the accumulator. tcgen05.ld hands each thread one ROW (32 columns);
// stored like that, a warp instruction would touch 32 different 128-byte lines. The chunk goes through
// a per-warp shared-memory tile instead and is re-read with 8 lanes per row, so every global
// load/store instruction covers 4 whole rows segments (fully used sectors).
template <int EPI, typename Act>
__device__ __forceinline__ void epilogue_chunk(void* __restrict__ y, float* __restrict__ st, size_t row0, uint32_t m, uint32_t col0,
                                               uint32_t ldy, const uint32_t (&r)[32], int lane) {
    if constexpr (EPI == DC_EPI_STORE_BF16 || EPI == DC_EPI_SWIGLU_BF16) {
        // 16-bit outputs: a thread's 32 columns are 64 (or, after SwiGLU, 32) contiguous bytes, stored directly
        const size_t row = row0 + lane;
        if (row >= m) return;
        if constexpr (EPI == DC_EPI_STORE_BF16) {
            uint4* p = reinterpret_cast<uint4*>(static_cast<uint16_t*>(y) + row * ldy + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = Act::pack(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
                v.y = Act::pack(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                v.z = Act::pack(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                v.w = Act::pack(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                p[j] = v;
            }
        } else {
            // SwiGLU over interleaved blocks of 16: columns [0,16) of this chunk are the gate, [16,32) the
            // up projection of the same 16 output columns (cpu_ref.rs:39-50)
            uint4* p = reinterpret_cast<uint4*>(static_cast<uint16_t*>(y) + row * ldy + (col0 >> 1));
            float o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = silu_f(__uint_as_float(r[j])) * __uint_as_float(r[16 + j]);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint4 v;
                v.x = Act::pack(o[8 * j], o[8 * j + 1]);
                v.y = Act::pack(o[8 * j + 2], o[8 * j + 3]);
                v.z = Act::pack(o[8 * j + 4], o[8 * j + 5]);
                v.w = Act::pack(o[8 * j + 6], o[8 * j + 7]);
                p[j] = v;
            }
        }
    } else {
        // fp32 outputs: tcgen05.ld hands each thread one ROW (32 columns = 128 bytes); stored like that, a
        // warp instruction would touch 32 different lines. The chunk goes through a per-warp
        // shared-memory tile and is re-read with 8 lanes per row, so each global instruction covers 4
        // whole 128-byte row segments.
        float4* mine = reinterpret_cast<float4*>(st + lane * kEpiLd);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            mine[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        __syncwarp();
        const int sub = lane >> 3, l8 = lane & 7;
        float* yf = static_cast<float*>(y) + col0 + 4 * l8;
        float4 old[8];
        if constexpr (EPI == DC_EPI_ADD_F32) {
#pragma unroll
            for (int it = 0; it < 8; ++it) {   // all eight reads of the residual in flight before the first add
                const size_t row = row0 + it * 4 + sub;
                old[it] = row < m ? __ldcg(reinterpret_cast<const float4*>(yf + row * ldy)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + sub;
            const size_t row = row0 + rr;
            float4 v = *reinterpret_cast<const float4*>(st + rr * kEpiLd + 4 * l8);
            if constexpr (EPI == DC_EPI_ADD_F32) {
                v.x += old[it].x; v.y += old[it].y; v.z += old[it].z; v.w += old[it].w;
            }
            if (row < m) *reinterpret_cast<float4*>(yf + row * ldy) = v;
        }
        __syncwarp();
    }
}

template <int BN, int EPI, typename Act>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
               void* __restrict__ y, const GemmArgs a, int* __restrict__ status) {
    using C = Cfg<BN>;
    constexpr int S = C::kStages;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + S * C::kABytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * C::kStageBytes);
    uint64_t* full = bars;                 // [S]   producer -> MMA: stage filled
    uint64_t* empty = bars + S;            // [S]   MMA -> producer: stage consumed
    uint64_t* acc_full = bars + 2 * S;     // [2]   MMA -> epilogue: accumulator complete
    uint64_t* acc_empty = bars + 2 * S + 2;  // [2] epilogue -> MMA: accumulator drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* epi_stage = reinterpret_cast<float*>(smem + S * C::kStageBytes + C::kBarBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t num_tiles = a.m_tiles * a.n_tiles;
    const uint32_t num_units = a.full_tiles + (num_tiles - a.full_tiles) * a.split;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        *abort_flag = 0u;
        fence_mbar_init();
        tma_prefetch_desc(&tm_x);
        tma_prefetch_desc(&tm_w);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t s = 0, ph = 0, issued = 0;
            bool ok = true;
            for (uint32_t u = blockIdx.x; ok && u < num_units; u += gridDim.x) {
                const Unit w = unit_of(u, a);
                uint32_t tm, tn;
                tile_coords(w.tile, a, tm, tn);
                for (uint32_t kb = w.kb0; kb < w.kb1; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, status, 1)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&full[s], C::kStageBytes);
                    tma_load_2d(smem_a + s * C::kABytes, &tm_x, &full[s], static_cast<int32_t>(kb * BK),
                                static_cast<int32_t>(tm * BM));
                    tma_load_2d(smem_b + s * C::kBBytes, &tm_w, &full[s], static_cast<int32_t>(kb * BK),
                                static_cast<int32_t>(tn * BN));
                    ++issued;
                    if (++s == S) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
            if (!ok) {
                // Leave only after this CTA's copies in flight have landed (or their own limit ran out):
                // the last min(issued, S) stages, newest first.
                uint32_t n_back = issued < static_cast<uint32_t>(S) ? issued : static_cast<uint32_t>(S);
                uint32_t bs = s, bph = ph;
                for (uint32_t j = 0; j < n_back; ++j) {
                    if (bs == 0) {
                        bs = S - 1;
                        bph ^= 1u;
                    } else {
                        --bs;
                    }
                    if (!wait_quiet(&full[bs], bph)) break;
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = a.idesc;
            uint32_t s = 0, ph = 0, lt = 0;
            bool ok = true;
            for (uint32_t u = blockIdx.x; ok && u < num_units; u += gridDim.x, ++lt) {
                const Unit w = unit_of(u, a);
                const uint32_t acc = lt & 1u, acc_ph = (lt >> 1) & 1u;
                if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1u, abort_flag, status, 2)) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (uint32_t kb = w.kb0; kb < w.kb1; ++kb) {
                    if (!mbar_wait(&full[s], ph, abort_flag, status, 3)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint64_t ad = umma_desc_k128(smem_u32(smem_a + s * C::kABytes));
                    const uint64_t bd = umma_desc_k128(smem_u32(smem_b + s * C::kBBytes));
#pragma unroll
                    for (uint32_t kk = 0; kk < BK / 16; ++kk) {
                        // 16 elements along K = 32 bytes = 2 units of the descriptor's 16-byte address field
                        umma_bf16_ss(d_tmem, ad + 2 * kk, bd + 2 * kk, idesc, (kb != w.kb0 || kk != 0u) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);
                    if (++s == S) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (ok) umma_commit(&acc_full[acc]);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const uint32_t q = static_cast<uint32_t>(warp) & 3u;  // TMEM lane quadrant this warp may read
        uint32_t lt = 0;
        for (uint32_t u = blockIdx.x; u < num_units; u += gridDim.x, ++lt) {
            const Unit w = unit_of(u, a);
            uint32_t tm, tn;
            tile_coords(w.tile, a, tm, tn);
            const uint32_t acc = lt & 1u, acc_ph = (lt >> 1) & 1u;
            if constexpr (EPI == DC_EPI_ADD_F32) {
                // The residual block this warp will read-modify-write is pulled into L2 while the tile's main loop still
                // runs (for a K-split tile: by every part, long before the last one to arrive needs it): a lane asks for
                // the 128-byte lines of its own row.
                const size_t prow = static_cast<size_t>(tm) * BM + q * 32u + lane;
                if (prow < a.m) {
                    const float* yrow = static_cast<const float*>(y) + prow * a.ldy + tn * BN;
#pragma unroll
                    for (uint32_t c = 0; c < BN / 32; ++c)
                        if (tn * BN + c * 32u < a.n) asm volatile("prefetch.global.L2 [%0];" ::"l"(yrow + c * 32u));
                }
            }
            bool ok = mbar_wait(&acc_full[acc], acc_ph, abort_flag, status, 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            const size_t row0 = static_cast<size_t>(tm) * BM + q * 32u;
            float* st = epi_stage + (warp - 2) * 32 * kEpiLd;
            const uint32_t taddr = tmem_base + ((q * 32u) << 16) + acc * BN;
            if (!w.split) {
#pragma unroll 1
                for (uint32_t c = 0; c < BN / 32; ++c) {
                    const uint32_t col0 = tn * BN + c * 32u;
                    if (col0 >= a.n) break;
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + c * 32u, r);
                    tmem_ld_wait();
                    epilogue_chunk<EPI, Act>(y, st, row0, a.m, col0, a.ldy, r, lane);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[acc]);
            } else {
                // One part of a K-split tile. The P parts of a tile run at the same time on P SMs (one unit per CTA in the
                // tail wave). Each parks its raw accumulator in the workspace, laid out [part][32-column chunk][128 rows][32] so
                // that every warp instruction moves 4 whole rows of a chunk (512 contiguous bytes), and counts itself in. When
                // all P have arrived, the parts SHARE the fix-up: part p sums chunks p, p + P, ... over all parts IN PART ORDER
                // (so the result does not depend on timing) and runs the normal epilogue on them. The wait is for parts that are
                // resident by construction (grid <= SMs), and bounded all the same. The counter goes P up on arrival, P up on
                // leaving; whoever leaves last puts it back to zero.
                const uint32_t rt = w.tile - a.full_tiles;
                const uint32_t P = a.split;
                const int sub = lane >> 3, l8 = lane & 7;
                constexpr uint32_t kChunkFloats = BM * 32;                 // one chunk of all 128 rows
                constexpr uint32_t kPartFloats = BM * BN;
                const uint32_t n_chunks = min(static_cast<uint32_t>(BN / 32), (a.n - tn * BN + 31u) / 32u);
                float* tile_ws = a.part_ws + static_cast<size_t>(rt * P) * kPartFloats + q * 32u * 32u;
                float* mine = tile_ws + static_cast<size_t>(w.part) * kPartFloats;
#pragma unroll 1
                for (uint32_t c = 0; c < n_chunks; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + c * 32u, r);
                    tmem_ld_wait();
                    float4* row = reinterpret_cast<float4*>(st + lane * kEpiLd);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        row[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                    __syncwarp();
                    float* dst = mine + c * kChunkFloats;
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = it * 4 + sub;
                        __stcg(reinterpret_cast<float4*>(dst + rr * 32 + 4 * l8), *reinterpret_cast<const float4*>(st + rr * kEpiLd + 4 * l8));
                    }
                    __syncwarp();
                }
                tc_fence_before_sync();
                __threadfence();
                __syncwarp();
                int* cnt = a.part_cnt + rt * 4u + q;
                bool go = true;
                if (lane == 0) {
                    mbar_arrive(&acc_empty[acc]);        // the accumulator is free: everything else works from the workspace
                    atomicAdd(cnt, 1);
                    go = wait_at_least(cnt, static_cast<int>(P), abort_flag, status, 5);
                }
                go = __shfl_sync(0xffffffffu, go ? 1 : 0, 0) != 0;
                if (!go) break;
                __threadfence();
                __syncwarp();
#pragma unroll 1
                for (uint32_t c = w.part; c < n_chunks; c += P) {
                    const uint32_t col0 = tn * BN + c * 32u;
                    float4 sum[8];
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        sum[it] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if constexpr (EPI == DC_EPI_ADD_F32) {   // the residual is requested together with the first parts
                            const size_t row = row0 + it * 4 + sub;
                            if (row < a.m) sum[it] = __ldcg(reinterpret_cast<const float4*>(static_cast<const float*>(y) + row * a.ldy + col0 + 4 * l8));
                        }
                    }
                    const float* src = tile_ws + c * kChunkFloats;
#pragma unroll
                    for (uint32_t pt = 0; pt < 4; pt += 2) {     // two parts' loads in flight together
                        if (pt < P) {
                            float4 v0[8], v1[8];
#pragma unroll
                            for (int it = 0; it < 8; ++it) {
                                v0[it] = __ldcg(reinterpret_cast<const float4*>(src + pt * kPartFloats + (it * 4 + sub) * 32 + 4 * l8));
                                v1[it] = pt + 1 < P ? __ldcg(reinterpret_cast<const float4*>(src + (pt + 1) * kPartFloats + (it * 4 + sub) * 32 + 4 * l8))
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
#pragma unroll
                            for (int it = 0; it < 8; ++it) {
                                sum[it].x = (sum[it].x + v0[it].x) + v1[it].x;
                                sum[it].y = (sum[it].y + v0[it].y) + v1[it].y;
                                sum[it].z = (sum[it].z + v0[it].z) + v1[it].z;
                                sum[it].w = (sum[it].w + v0[it].w) + v1[it].w;
                            }
                        }
                    }
                    if constexpr (EPI == DC_EPI_ADD_F32 || EPI == DC_EPI_STORE_F32) {
                        // fp32 outputs: the sums already sit in the layout the stores want (a warp instruction covers 4 whole rows)
                        float* yf = static_cast<float*>(y);
#pragma unroll
                        for (int it = 0; it < 8; ++it) {
                            const size_t row = row0 + it * 4 + sub;
                            if (row < a.m) *reinterpret_cast<float4*>(yf + row * a.ldy + col0 + 4 * l8) = sum[it];
                        }
                    } else {
                        // 16-bit outputs: back to one row per thread for the common epilogue
#pragma unroll
                        for (int it = 0; it < 8; ++it) *reinterpret_cast<float4*>(st + (it * 4 + sub) * kEpiLd + 4 * l8) = sum[it];
                        __syncwarp();
                        uint32_t r[32];
                        const uint4* row = reinterpret_cast<const uint4*>(st + lane * kEpiLd);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint4 v = row[j];
                            r[4 * j] = v.x;
                            r[4 * j + 1] = v.y;
                            r[4 * j + 2] = v.z;
                            r[4 * j + 3] = v.w;
                        }
                        __syncwarp();
                        epilogue_chunk<EPI, Act>(y, st, row0, a.m, col0, a.ldy, r, lane);
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    const int before = atomicAdd(cnt, 1);
                    if (before == 2 * static_cast<int>(P) - 1) atomicExch(cnt, 0);
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        __syncwarp();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

int make_tmap(dc_ctx* ctx, const void* base, uint32_t rows, uint32_t cols, uint32_t ld, uint32_t box_rows, bool f16,
              CUtensorMap* out) {
    const dc_tmap_key key(base, rows, cols, ld, box_rows | (f16 ? 0x10000u : 0u));
    auto it = ctx->tmaps.find(key);
    if (it != ctx->tmaps.end()) {
        *out = it->second;
        return DC_OK;
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    CUresult r = ctx->encode_tiled(&m, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return dc_fail(ctx, DC_CUDA_ERROR, "gemm: cuTensorMapEncodeTiled failed (%d) for [%u x %u] ld %u", static_cast<int>(r),
                       rows, cols, ld);
    if (ctx->tmaps.size() >= 8192) ctx->tmaps.clear();
    ctx->tmaps.emplace(key, m);
    ctx->tmap_encodes++;
    *out = m;
    return DC_OK;
}

template <int BN, int EPI, typename Act>
int opt_in(dc_ctx* ctx) {
    using C = Cfg<BN>;
    static bool attr_set[16] = {};
    if (!attr_set[ctx->device & 15]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, Act>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "gemm: cannot opt in to %u bytes of shared memory: %s", C::kSmemBytes, cudaGetErrorString(e));
        attr_set[ctx->device & 15] = true;
    }
    return DC_OK;
}

template <int BN, int EPI, typename Act>
int launch(dc_ctx* ctx, cudaStream_t stream, const CUtensorMap& tx, const CUtensorMap& tw, void* y, const GemmArgs& a) {
    using C = Cfg<BN>;
    auto kern = gemm_tc_kernel<BN, EPI, Act>;
    if (int rc = opt_in<BN, EPI, Act>(ctx); rc != DC_OK) return rc;
    const uint32_t units = a.full_tiles + (a.m_tiles * a.n_tiles - a.full_tiles) * a.split;
    const uint32_t grid = units < static_cast<uint32_t>(ctx->sm_count) ? units : static_cast<uint32_t>(ctx->sm_count);
    kern<<<grid, kThreads, C::kSmemBytes, stream>>>(tx, tw, y, a, ctx->status_dev);
    return dc_check_launch(ctx, "gemm (tcgen05)");
}

template <int BN>
int launch_epi(dc_ctx* ctx, cudaStream_t stream, const CUtensorMap& tx, const CUtensorMap& tw, void* y, const GemmArgs& a,
               uint32_t epi) {
    const bool f16 = ctx->act_dtype == DC_ACT_F16;
    switch (epi) {
        case DC_EPI_STORE_F32: return launch<BN, DC_EPI_STORE_F32, ActBF16>(ctx, stream, tx, tw, y, a);
        case DC_EPI_ADD_F32: return launch<BN, DC_EPI_ADD_F32, ActBF16>(ctx, stream, tx, tw, y, a);
        case DC_EPI_STORE_BF16:
            return f16 ? launch<BN, DC_EPI_STORE_BF16, ActF16>(ctx, stream, tx, tw, y, a) : launch<BN, DC_EPI_STORE_BF16, ActBF16>(ctx, stream, tx, tw, y, a);
        default:
            return f16 ? launch<BN, DC_EPI_SWIGLU_BF16, ActF16>(ctx, stream, tx, tw, y, a) : launch<BN, DC_EPI_SWIGLU_BF16, ActBF16>(ctx, stream, tx, tw, y, a);
    }
}

template <int BN>
int warm_bn(dc_ctx* ctx) {
    int rc = opt_in<BN, DC_EPI_STORE_F32, ActBF16>(ctx);
    if (rc == DC_OK) rc = opt_in<BN, DC_EPI_ADD_F32, ActBF16>(ctx);
    if (rc == DC_OK) rc = opt_in<BN, DC_EPI_STORE_BF16, ActF16>(ctx);
    if (rc == DC_OK) rc = opt_in<BN, DC_EPI_STORE_BF16, ActBF16>(ctx);
    if (rc == DC_OK) rc = opt_in<BN, DC_EPI_SWIGLU_BF16, ActF16>(ctx);
    if (rc == DC_OK) rc = opt_in<BN, DC_EPI_SWIGLU_BF16, ActBF16>(ctx);
    return rc;
}

}  // namespace

// Every (tile width x epilogue x 16-bit type) variant made launchable now: the role of Gemm::warm_up
// (crates/decide-engine/src/kernels/gemm.rs:89-107), which builds each pipeline before the first request.
int dc_gemm_warm(dc_ctx* ctx) {
    int rc = warm_bn<256>(ctx);
    if (rc == DC_OK) rc = warm_bn<224>(ctx);
    if (rc == DC_OK) rc = warm_bn<192>(ctx);
    if (rc == DC_OK) rc = warm_bn<128>(ctx);
    return rc;
}

namespace {
// One warp; lane 0 waits on a barrier that never completes, with the same bounded wait every kernel here uses.
__global__ void wait_timeout_selftest_kernel(int* __restrict__ status) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        dc::mbar_init(&bar, 1);
        abort_flag = 0u;
        dc::fence_mbar_init();
    }
    __syncwarp();
    if (threadIdx.x == 0) dc::mbar_wait(&bar, 0u, &abort_flag, status, 99);
    __syncwarp();
}
}  // namespace

extern "C" int dc_selftest_wait_timeout(dc_ctx* ctx, void* stream) {
    if (!ctx) return DC_INVALID_ARG;
    wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctx->status_dev);
    return dc_check_launch(ctx, "selftest (wait timeout)");
}

int dc_make_tmap(dc_ctx* ctx, const void* base, uint32_t rows, uint32_t cols, uint32_t ld, uint32_t box_rows, bool f16, CUtensorMap* out) {
    return make_tmap(ctx, base, rows, cols, ld, box_rows, f16, out);
}

// Tile plan: the analogue of gemm_configs::plan (crates/decide-metal/src/gemm_configs.rs:312).
// Whole waves of 128 x BN tiles run as whole tiles; the tiles of the last, partial wave are cut along
// K into up to 4 parts so that wave fills the SMs as well. The tile width is the cheapest of 256, 224,
// 192 and 128 under this model, calibrated on the B200: time = waves x (time of one tile); a narrower
// tile takes tile_time() of a 256-wide one (less than proportionally less: its operand feed, not only
// its MMAs, sets its pace). A split tile costs its share of the main loop plus the fix-up: every part
// parks its sums in the workspace and the parts share the summing, worth ~kFixup k-blocks of main loop.
namespace {
struct Plan {
    uint32_t bn, full_tiles, split, kb_per_part;
    double cost;
};
constexpr double kFixup = 14.0;   // k-blocks of main loop a split tile's park + shared fix-up is worth (~7 us)
constexpr uint32_t kMinPartBlocks = 24;   // shorter parts did not pay on the B200: K = 2560 cut in four ran slower than whole tiles
// measured on whole waves of the gate_up projection at 2,307 rows: one wave of 128 x BN tiles against one of 128 x 256
double tile_time(uint32_t bn) { return bn == 256 ? 1.0 : bn == 224 ? 0.87 : bn == 192 ? 0.78 : 0.65; }

Plan plan_for(uint32_t bn, uint32_t m, uint32_t n, uint32_t k, uint32_t sms, uint32_t epi, uint32_t max_split = 4) {
    (void)epi;
    const uint32_t tiles = ((m + BM - 1) / BM) * ((n + bn - 1) / bn);
    const uint32_t k_blocks = (k + BK - 1) / BK;
    const uint32_t rest = tiles % sms;
    Plan p{bn, tiles - rest, 1, k_blocks, 0.0};
    auto tail_of = [&](uint32_t split) {
        const uint32_t per = (k_blocks + split - 1) / split;
        if (split == 1) return 1.0;
        return static_cast<double>(per) / k_blocks + kFixup / k_blocks;
    };
    if (rest > 0) {
        const uint32_t cap = sms / rest < max_split ? sms / rest : max_split;
        for (uint32_t split = 2; split <= cap; ++split)
            if (k_blocks / split >= kMinPartBlocks && tail_of(split) < tail_of(p.split)) p.split = split;
    }
    p.kb_per_part = (k_blocks + p.split - 1) / p.split;
    const double tail = rest == 0 ? 0.0 : tail_of(p.split);
    p.cost = (tiles / sms + tail) * tile_time(bn);
    return p;
}
Plan best_plan(uint32_t m, uint32_t n, uint32_t k, uint32_t sms, uint32_t bn_override, uint32_t epi, uint32_t max_split = 4) {
    if (bn_override) return plan_for(bn_override, m, n, k, sms, epi, max_split);
    Plan best = plan_for(256, m, n, k, sms, epi, max_split);
    for (uint32_t bn : {224u, 192u, 128u}) {
        const Plan c = plan_for(bn, m, n, k, sms, epi, max_split);
        if (c.cost < best.cost * 0.95) best = c;   // a narrower tile has to win by a margin (the model is good to a few percent)
    }
    return best;
}
// DECIDE_GEMM_SPLIT caps the K split of tail-wave tiles (1 = never split); the fix-up sums at most 4 parts.
uint32_t max_split_from_env() {
    static const uint32_t v = [] {
        const char* e = getenv("DECIDE_GEMM_SPLIT");
        const int n = e ? atoi(e) : 4;
        return static_cast<uint32_t>(n < 1 ? 1 : (n > 4 ? 4 : n));
    }();
    return v;
}
// DECIDE_GEMM_BN forces a tile width for every shape (a measuring aid, like the reference's DECIDE_GEMM switches).
uint32_t bn_from_env() {
    static const uint32_t v = [] {
        const char* e = getenv("DECIDE_GEMM_BN");
        const int n = e ? atoi(e) : 0;
        return static_cast<uint32_t>((n == 128 || n == 192 || n == 224 || n == 256) ? n : 0);
    }();
    return v;
}
}  // namespace

uint32_t dc_gemm_plan_bn(uint32_t m, uint32_t n, uint32_t k, int sm_count) {
    return best_plan(m, n, k ? k : 2560, sm_count, bn_from_env(), DC_EPI_STORE_F32, max_split_from_env()).bn;
}

extern "C" uint32_t dc_gemm_plan_for(dc_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, uint32_t epilogue, uint32_t bn, uint32_t* tail_split) {
    if (bn != 0 && bn != 128 && bn != 192 && bn != 224 && bn != 256) return 0;
    const Plan pl = best_plan(m, n, k ? k : 2560, ctx ? static_cast<uint32_t>(ctx->sm_count) : 148u, bn ? bn : bn_from_env(), epilogue, max_split_from_env());
    if (tail_split) *tail_split = pl.split;
    return pl.bn;
}

extern "C" uint32_t dc_gemm_plan_k(dc_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, uint32_t* tail_split) {
    return dc_gemm_plan_for(ctx, m, n, k, DC_EPI_ADD_F32, 0, tail_split);
}

int dc_gemm_tc(dc_ctx* ctx, cudaStream_t stream, const void* x, const void* w, void* y, uint32_t m, uint32_t n,
               uint32_t k, uint32_t ldx, uint32_t ldw, uint32_t ldy, uint32_t epi, uint32_t bn_override) {
    const Plan pl = best_plan(m, n, k, static_cast<uint32_t>(ctx->sm_count), bn_override ? bn_override : bn_from_env(), epi, max_split_from_env());
    const uint32_t bn = pl.bn;
    GemmArgs a;
    a.m = m;
    a.n = n;
    a.k = k;
    a.ldy = ldy;
    a.m_tiles = (m + BM - 1) / BM;
    a.n_tiles = (n + bn - 1) / bn;
    a.k_blocks = (k + BK - 1) / BK;
    // Row tiles per group: W is streamed from HBM once per group, and the group's X rows (group_m x 128 x K 16-bit values)
    // have to stay in L2 beside the W stripes in flight. DECIDE_GEMM_GROUP_M overrides (a measuring aid).
    static const uint32_t group_env = getenv("DECIDE_GEMM_GROUP_M") ? static_cast<uint32_t>(atoi(getenv("DECIDE_GEMM_GROUP_M"))) : 0u;
    const uint32_t group_want = group_env ? group_env : kGroupM;
    a.group_m = a.m_tiles < group_want ? a.m_tiles : group_want;
    a.full_tiles = pl.full_tiles;
    a.split = pl.split;
    a.kb_per_part = pl.kb_per_part;
    a.part_ws = ctx->gemm_part_ws;
    a.part_cnt = ctx->gemm_part_cnt;
    const bool f16 = ctx->act_dtype == DC_ACT_F16;
    // Both operands carry the same format code: kind::f16 with an fp16 A and a bf16 B raises an
    // illegal-instruction fault on sm_100a.
    const uint32_t fmt = f16 ? ActF16::kUmmaFormat : ActBF16::kUmmaFormat;
    a.idesc = umma_idesc(fmt, fmt, BM, static_cast<int>(bn));
    CUtensorMap tx, tw;
    int rc = make_tmap(ctx, x, m, k, ldx, BM, f16, &tx);
    if (rc != DC_OK) return rc;
    rc = make_tmap(ctx, w, n, k, ldw, bn, f16, &tw);
    if (rc != DC_OK) return rc;
    switch (bn) {
        case 256: return launch_epi<256>(ctx, stream, tx, tw, y, a, epi);
        case 224: return launch_epi<224>(ctx, stream, tx, tw, y, a, epi);
        case 192: return launch_epi<192>(ctx, stream, tx, tw, y, a, epi);
        default: return launch_epi<128>(ctx, stream, tx, tw, y, a, epi);
    }
}
