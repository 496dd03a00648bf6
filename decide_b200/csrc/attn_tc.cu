// Causal grouped-query attention on tcgen05 (head_dim 128, packed sequences): the fast path of
// dc_attention for prefill batches. Same arithmetic contract as the mma.sync kernel of attn.cu
// (spec cpu_ref.rs:167-188; reference kernels attn_fast.metal:289-411): fp32 scores and online softmax,
// weights rounded once to the 16-bit operand type, optional sigmoid output gate in the store. The row
// sum is taken in fp32 BEFORE that rounding (the mma.sync kernel sums the rounded weights; the two
// differ by about 2^-12 of the sum, far inside the operand type's own rounding).
//
// One CTA per (128 query rows of a sequence, query head), two CTAs per SM. Per tile of 128 cache rows:
//   S = Q K^T    tcgen05.mma, Q and K as K-major swizzled tiles loaded by TMA, S in tensor memory
//   softmax      8 warps, one thread per (row, half of the 128 columns): scores out of tensor memory,
//                mask, running maximum (the two halves of a row meet through shared memory), exp2,
//                and the 16-bit weights written back INTO the columns the scores came from
//   O += P V     tcgen05.mma with P as the tensor-memory A operand and V^T (value dim x cache row,
//                cache rows contiguous) as the K-major B tile
// V arrives as [cache row][head][128]; a small kernel first transposes it into scratch as
// [head][128][column], each sequence starting on a column that is a multiple of 8 so that every TMA
// tile starts on a 16-byte boundary; the gaps between sequences are zero-filled because a zero weight
// times a stale NaN would still poison the sum.
// The running maximum is lazy: O and the row sum are rescaled only when the maximum grows by more than
// 2^8, so most tiles skip the read-modify-write of O in tensor memory; weights stay below 2^8.
// Warp 8 issues the TMA copies and the MMAs. Every wait is a bounded mbarrier wait; when one gives up
// the CTA raises the status word, waits for its copies and MMAs in flight, frees its tensor memory and
// returns.
#include "common.cuh"
#include "ptx.cuh"

namespace {

using namespace dc;

constexpr int HD = 128;
constexpr int TQ = 128;    // query rows per CTA
constexpr int TKV = 128;   // cache rows per tile
constexpr int kThreads = 288;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColO = 128;
constexpr float kMasked = -1e30f;
constexpr float kRescaleStep = 8.0f;   // log2 units
constexpr int kStatusPositionPastCache = DC_STATUS_POSITION_PAST_CACHE;

struct Smem {
    static constexpr size_t kAtom = 128 * 128;          // [128 rows][64 x 16 bit]
    static constexpr size_t kQ = 0;
    static constexpr size_t kK = kQ + 2 * kAtom;
    static constexpr size_t kV = kK + 2 * kAtom;
    static constexpr size_t kBars = kV + 2 * kAtom;
    static constexpr size_t kMx = kBars + 128;           // float [2 tiles][2 halves][128 rows]
    static constexpr size_t kQp = kMx + 2 * 2 * 128 * 4;  // int [128] + the tile's maximum
    static constexpr size_t kBytes = kQp + 129 * 4 + 12 + 1024;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Barrier between the two warps that share a row quadrant: an mbarrier with one arrival per warp, bounded like every wait here.
__device__ __forceinline__ bool pair_sync(uint64_t* bar, uint32_t& phase, int lane, volatile uint32_t* abort_flag, int* status) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
    const bool ok = mbar_wait(bar, phase, abort_flag, status, 53);
    phase ^= 1u;
    return ok;
}

// Column of the transposed V scratch where sequence `seq` (first row `row_lo`) starts.
__host__ __device__ __forceinline__ uint32_t vt_col(uint32_t row_lo, uint32_t seq) { return ((row_lo + 7u) & ~7u) + 8u * seq; }

// vt[(head * 128 + d) * ldt + vt_col(seq) + t] = vc[(row_lo + t) * nkv * 128 + head * 128 + d]; columns from the end of a
// sequence to the start of the next one are zero-filled.
__global__ void __launch_bounds__(256) v_transpose_kernel(const uint16_t* __restrict__ vc, uint16_t* __restrict__ vt, uint32_t rows, uint32_t nkv,
                                                          uint32_t ldt, const uint32_t* __restrict__ seq_start, uint32_t n_seq, uint32_t kv_len) {
    __shared__ uint16_t tile[64][HD + 8];
    const uint32_t seq = blockIdx.z, head = blockIdx.y, t0 = blockIdx.x * 64;
    // without seq_start: one sequence whose cache is rows 0 .. kv_len
    const uint32_t row_lo = seq_start ? seq_start[seq] : 0u, len = seq_start ? seq_start[seq + 1] - row_lo : kv_len;
    const uint32_t col0 = vt_col(row_lo, seq);
    const uint32_t col_end = seq_start && seq + 1 < n_seq ? vt_col(seq_start[seq + 1], seq + 1) : ldt;   // first column of the next sequence
    if (col0 + t0 >= col_end) return;
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
        const int r = e >> 4, c8 = (e & 15) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t0 + r < len) v = *reinterpret_cast<const uint4*>(vc + (static_cast<size_t>(row_lo) + t0 + r) * nkv * HD + head * HD + c8);
        *reinterpret_cast<uint4*>(&tile[r][c8]) = v;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < HD * 8; e += 256) {
        const int d = e >> 3, c = e & 7;   // 8 columns t0 + 8c .. of output row d
        if (col0 + t0 + 8 * c >= col_end) continue;
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = static_cast<uint32_t>(tile[8 * c + 2 * i][d]) | (static_cast<uint32_t>(tile[8 * c + 2 * i + 1][d]) << 16);
        *reinterpret_cast<uint4*>(vt + (static_cast<size_t>(head) * HD + d) * ldt + col0 + t0 + 8 * c) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}


template <typename Act>
__global__ void __launch_bounds__(kThreads, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
               const float* __restrict__ gate, const uint32_t* __restrict__ qpos, uint16_t* __restrict__ y, uint32_t ldg, uint32_t nq, uint32_t nkv,
               float scale_log2, const uint32_t* __restrict__ seq_start, uint32_t q_len, uint32_t kv_len, int* __restrict__ status) {
    const uint32_t seq = blockIdx.z, head = blockIdx.y;
    // without seq_start: q_len query rows of one sequence (a chunk that continues a longer cache; the cache starts at row 0
    // and each query row's position says how far it attends)
    const uint32_t row_lo = seq_start ? seq_start[seq] : 0u, len = seq_start ? seq_start[seq + 1] - row_lo : q_len;
    // query tiles are handed out last-first: the tiles with the most cache rows to visit start first
    const uint32_t r0 = (gridDim.x - 1 - blockIdx.x) * TQ;
    if (r0 >= len) return;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sQ = smem + Smem::kQ;
    uint8_t* sK = smem + Smem::kK;
    uint8_t* sV = smem + Smem::kV;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;
    uint64_t* v_full = bars + 2;
    uint64_t* s_done = bars + 3;     // S = Q K^T of a tile finished (and every product before it)
    uint64_t* pv_done = bars + 4;    // O += P V of a tile finished
    uint64_t* p_ready = bars + 5;    // the 8 softmax warps have written P (and rescaled O)
    uint64_t* drain_bar = bars + 6;
    uint64_t* pair_bar = bars + 8;   // [4] the two softmax warps of a row quadrant
    uint64_t* gate_bar = bars + 12;  // the 8 softmax warps have staged the gate tile
    uint64_t* out_bar = bars + 13;   // the 8 softmax warps have staged the output tile
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* never_flag = tmem_slot + 2;
    float* mx = reinterpret_cast<float*>(smem + Smem::kMx);
    int* qp = reinterpret_cast<int*>(smem + Smem::kQp);
    int* qp_max = qp + 128;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(q_full, 1);
        mbar_init(k_full, 1);
        mbar_init(v_full, 1);
        mbar_init(s_done, 1);
        mbar_init(pv_done, 1);
        mbar_init(p_ready, 8);
        mbar_init(drain_bar, 1);
        for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 2);
        mbar_init(gate_bar, 8);
        mbar_init(out_bar, 8);
        *abort_flag = 0u;
        *never_flag = 0u;
        *qp_max = -1;
        fence_mbar_init();
    }
    if (warp == 8) {
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
        }
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (tid < TQ) {
        const int p = r0 + tid < len ? static_cast<int>(qpos[row_lo + r0 + tid]) : -1;
        qp[tid] = p;
        int m = p;
#pragma unroll
        for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) atomicMax(qp_max, m);
    }
    __syncthreads();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t n_tiles = static_cast<uint32_t>(*qp_max + TKV) / TKV;   // cache rows 0..=max qpos; 0 only if no row is valid
    // One sequence with the cache length given: a position at or past it breaks the caller's promise (the maps end there,
    // so nothing out of bounds is read, but the result would miss keys): reported through the status word.
    if (!seq_start && tid == 0 && *qp_max >= static_cast<int>(kv_len)) atomicCAS(status, 0, kStatusPositionPastCache);

    if (warp == 8) {
        // ------------------------------------------------------------------ issuer (one thread)
        if (lane == 0 && n_tiles) {
            const uint32_t hk = head / (nq / nkv);
            const int32_t vcol0 = static_cast<int32_t>(vt_col(row_lo, seq));
            uint32_t k_issued = 0, k_waited = 0, v_issued = 0, v_waited = 0;
            bool q_pending = true;
            auto load_k = [&](uint32_t j) {
                mbar_arrive_expect_tx(k_full, 2 * Smem::kAtom);
                tma_load_2d(sK, &tm_k, k_full, static_cast<int32_t>(hk * HD), static_cast<int32_t>(row_lo + j * TKV));
                tma_load_2d(sK + Smem::kAtom, &tm_k, k_full, static_cast<int32_t>(hk * HD + 64), static_cast<int32_t>(row_lo + j * TKV));
                k_issued = j + 1;
            };
            auto load_v = [&](uint32_t j) {
                mbar_arrive_expect_tx(v_full, 2 * Smem::kAtom);
                tma_load_2d(sV, &tm_v, v_full, vcol0 + static_cast<int32_t>(j * TKV), static_cast<int32_t>(hk * HD));
                tma_load_2d(sV + Smem::kAtom, &tm_v, v_full, vcol0 + static_cast<int32_t>(j * TKV + 64), static_cast<int32_t>(hk * HD));
                v_issued = j + 1;
            };
            mbar_arrive_expect_tx(q_full, 2 * Smem::kAtom);
            tma_load_2d(sQ, &tm_q, q_full, static_cast<int32_t>(head * HD), static_cast<int32_t>(row_lo + r0));
            tma_load_2d(sQ + Smem::kAtom, &tm_q, q_full, static_cast<int32_t>(head * HD + 64), static_cast<int32_t>(row_lo + r0));
            load_k(0);
            load_v(0);
            constexpr uint32_t idesc = umma_idesc(Act::kUmmaFormat, Act::kUmmaFormat, TQ, TKV);
            const uint64_t dq = umma_desc_k128(smem_u32(sQ)), dk = umma_desc_k128(smem_u32(sK)), dvt = umma_desc_k128(smem_u32(sV));
            constexpr uint64_t kAtomStep = Smem::kAtom >> 4;
            bool ok = mbar_wait(q_full, 0u, abort_flag, status, 41);
            q_pending = !ok;
            // S = Q K^T of tile j: queued as soon as K has landed. For j > 0 that is right behind O += P V of tile j - 1:
            // the products execute in issue order, so the scores overwrite the weights only after they have been consumed.
            auto issue_s = [&](uint32_t j) {
                if (!mbar_wait(k_full, j & 1u, abort_flag, status, 42)) return false;
                k_waited = j + 1;
                tc_fence_after_sync();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint64_t off = (ks >> 2) * kAtomStep + 2 * (ks & 3);
                    if (ks == 0) umma_bf16_ss<false>(tmem_base + kColS, dq + off, dk + off, idesc);
                    else umma_bf16_ss<true>(tmem_base + kColS, dq + off, dk + off, idesc);
                }
                umma_commit(s_done);
                return true;
            };
            if (ok) ok = issue_s(0);
            for (uint32_t j = 0; ok && j < n_tiles; ++j) {
                const uint32_t ph = j & 1u;
                if (!(ok = mbar_wait(s_done, ph, abort_flag, status, 43))) break;   // the K tile is free again
                if (j + 1 < n_tiles) load_k(j + 1);
                if (!(ok = mbar_wait(p_ready, ph, abort_flag, status, 44))) break;
                if (!(ok = mbar_wait(v_full, ph, abort_flag, status, 45))) break;
                v_waited = j + 1;
                tc_fence_after_sync();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    // P of cache rows 16 ks .. sits in 8 columns of the half of S it was computed from
                    const uint32_t pcol = tmem_base + kColS + (ks >> 2) * 64 + 8 * (ks & 3);
                    const uint64_t off = (ks >> 2) * kAtomStep + 2 * (ks & 3);
                    if (j == 0 && ks == 0) umma_bf16_ts<false>(tmem_base + kColO, pcol, dvt + off, idesc);
                    else umma_bf16_ts<true>(tmem_base + kColO, pcol, dvt + off, idesc);
                }
                umma_commit(pv_done);
                if (j + 1 < n_tiles && !(ok = issue_s(j + 1))) break;
                if (!(ok = mbar_wait(pv_done, ph, abort_flag, status, 46))) break;   // the V tile is free again
                if (j + 1 < n_tiles) load_v(j + 1);
            }
            if (*abort_flag) {
                // nothing may still be writing this CTA's shared or tensor memory when it exits
                if (q_pending) mbar_wait(q_full, 0u, never_flag, status, 47);
                for (uint32_t i = k_waited; i < k_issued; ++i) mbar_wait(k_full, i & 1u, never_flag, status, 47);
                for (uint32_t i = v_waited; i < v_issued; ++i) mbar_wait(v_full, i & 1u, never_flag, status, 47);
                umma_commit(drain_bar);
                mbar_wait(drain_bar, 0u, never_flag, status, 48);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax warps
        const int q = warp & 3, hh = warp >> 2;
        const int row = 32 * q + lane;
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(32 * q) << 16);
        const int qp_r = qp[row];
        float m_used = kMasked, l = 0.f;
        uint32_t pair_ph = 0;
        uint32_t j = 0;
        for (; j < n_tiles; ++j) {
            const uint32_t ph = j & 1u;
            if (!mbar_wait(s_done, ph, abort_flag, status, 51)) break;
            __syncwarp();
            tc_fence_after_sync();
            if (gate && j + 1 == n_tiles) {
                // The last S = Q K^T is done, so the Q and K tiles (64 KB, contiguous) are free: stage the 128 x 128 fp32 gate
                // tile there with row-wise (coalesced) asynchronous copies; it lands while this tile is being processed.
                // Row r holds its 32 16-byte chunks at positions c ^ (r & 31), so that the per-row reads of the epilogue
                // spread over the banks. Warp w stages rows 16 w .. 16 w + 15.
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int gr = 16 * warp + i;
                    if (r0 + gr < len) {
                        const float* src = gate + (static_cast<size_t>(row_lo) + r0 + gr) * ldg + head * HD + 4 * lane;
                        const uint32_t dst = smem_u32(sQ + gr * 512 + ((lane ^ (gr & 31)) << 4));
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
                    }
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            // raw scores of this thread's half row; the scale (with log2 e folded in) is applied inside the exp2
            float t[64];
            {
                uint32_t r[32];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    tmem_ld_32x32(tlane + kColS + 64 * hh + 32 * half, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) t[32 * half + e] = __uint_as_float(r[e]);
                }
            }
            const int kv0 = static_cast<int>(j * TKV) + 64 * hh;
            const int visible = qp_r - kv0 + 1;    // columns e < visible may be attended
            if (visible < 64) {
#pragma unroll
                for (int e = 0; e < 64; ++e) t[e] = e < visible ? t[e] : kMasked;
            }
            float lm0 = kMasked, lm1 = kMasked;
#pragma unroll
            for (int e = 0; e < 64; e += 4) {
                lm0 = fmaxf(lm0, fmaxf(t[e], t[e + 1]));
                lm1 = fmaxf(lm1, fmaxf(t[e + 2], t[e + 3]));
            }
            float* mxj = mx + ph * 256;
            mxj[hh * 128 + row] = fmaxf(lm0, lm1);
            if (!pair_sync(&pair_bar[q], pair_ph, lane, abort_flag, status)) break;
            // maximum of the tile in exp2 units; a fully masked row keeps the sentinel
            const float m_raw = fmaxf(mxj[row], mxj[128 + row]);
            const float m_tile = m_raw > 0.5f * kMasked ? m_raw * scale_log2 : kMasked;
            const bool grow = m_tile - m_used > kRescaleStep;
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                // O and the row sum follow the new maximum (lanes whose maximum stays put scale by 1)
                const float alpha = grow ? ex2(m_used - m_tile) : 1.0f;
                l *= alpha;
#pragma unroll
                for (int part = 0; part < 4; ++part) {   // 16 columns at a time: load, scale, store
                    uint32_t r[16];
                    tmem_ld_32x32_x16(tlane + kColO + 64 * hh + 16 * part, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
                    tmem_st_32x32_x16(tlane + kColO + 64 * hh + 16 * part, r);
                }
                tmem_st_wait();
            }
            if (grow) m_used = m_tile;
            // weights 2^(s * scale - m): a masked score (-1e30) gives exactly 0 as long as the row has a maximum; a row without
            // one (nothing visible yet) gets zeros explicitly. The row sum adds the weights before they are rounded to 16 bits.
            uint32_t pk[32];
            if (m_used > 0.5f * kMasked) {
                float l0 = 0.f, l1 = 0.f;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float p0 = ex2(fmaf(t[2 * i], scale_log2, -m_used));
                    const float p1 = ex2(fmaf(t[2 * i + 1], scale_log2, -m_used));
                    pk[i] = Act::pack(p0, p1);
                    l0 += p0;
                    l1 += p1;
                }
                l += l0 + l1;
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) pk[i] = 0u;
            }
            {
                uint32_t a[16], b[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    a[i] = pk[i];
                    b[i] = pk[16 + i];
                }
                tmem_st_32x32_x16(tlane + kColS + 64 * hh, a);
                tmem_st_32x32_x16(tlane + kColS + 64 * hh + 16, b);
            }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);
        }
        if (j == n_tiles && n_tiles) {
            const bool row_ok = qp_r >= 0;
            asm volatile("cp.async.wait_all;" ::: "memory");   // this thread's share of the gate tile has landed
            float* ls = mx + ((n_tiles & 1u) ? 256 : 0);   // the half of the exchange buffer the last tile did not use
            ls[hh * 128 + row] = l;
            bool pair_ok = pair_sync(&pair_bar[q], pair_ph, lane, abort_flag, status);   // the two halves of a row add their sums
            if (pair_ok && gate) {   // all 8 warps have staged their rows of the gate tile
                __syncwarp();
                if (lane == 0) mbar_arrive(gate_bar);
                pair_ok = mbar_wait(gate_bar, 0u, abort_flag, status, 54);
            }
            if (pair_ok && mbar_wait(pv_done, (n_tiles - 1) & 1u, abort_flag, status, 52)) {
                __syncwarp();
                tc_fence_after_sync();
                const float l_tot = ls[row] + ls[128 + row];
                const float inv = row_ok && l_tot > 0.f ? 1.0f / l_tot : 0.f;
                // The output tile goes through the V tile's shared memory (free after the last product) so that it leaves in
                // whole 256-byte rows: thread-per-row stores would touch 32 different lines per instruction. Row r keeps its 16
                // chunks of 16 bytes at positions c ^ (r & 15).
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t r[32];
                    tmem_ld_32x32(tlane + kColO + 64 * hh + 32 * half, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float o[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(r[8 * c + e]) * inv;
                        if (gate) {
                            const int ch = 16 * hh + 8 * half + 2 * c;   // 16-byte chunk of this row's 128 gate values
                            const float4 g0 = *reinterpret_cast<const float4*>(sQ + row * 512 + ((ch ^ (row & 31)) << 4));
                            const float4 g1 = *reinterpret_cast<const float4*>(sQ + row * 512 + (((ch + 1) ^ (row & 31)) << 4));
                            const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                            for (int e = 0; e < 8; ++e) o[e] = __fdividef(o[e], 1.0f + __expf(-gv[e]));
                        }
                        const int oc = 8 * hh + 4 * half + c;   // 16-byte chunk of this row's 128 outputs
                        *reinterpret_cast<uint4*>(sV + row * 256 + ((oc ^ (row & 15)) << 4)) =
                            make_uint4(Act::pack(o[0], o[1]), Act::pack(o[2], o[3]), Act::pack(o[4], o[5]), Act::pack(o[6], o[7]));
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(out_bar);
                if (mbar_wait(out_bar, 0u, abort_flag, status, 55)) {
                    // warp w sends rows 16 w .. 16 w + 15, two rows per instruction
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int orow = 16 * warp + 2 * i + (lane >> 4), oc = lane & 15;
                        if (r0 + orow < len && qp[orow] >= 0) {
                            const uint4 v = *reinterpret_cast<const uint4*>(sV + orow * 256 + ((oc ^ (orow & 15)) << 4));
                            *reinterpret_cast<uint4*>(y + (static_cast<size_t>(row_lo) + r0 + orow) * nq * HD + head * HD + 8 * oc) = v;
                        }
                    }
                }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");   // (only matters when the loop was left early)
        __syncwarp();
        tmem_ld_wait();
    }

    // ------------------------------------------------------------------------------ teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after_sync();
        __syncwarp();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace


// Scratch the tcgen05 attention path needs for the transposed V of `rows` packed cache rows.
size_t dc_attention_tc_scratch_bytes(uint32_t rows, uint32_t n_seq, uint32_t nkv) {
    const size_t ldt = ((static_cast<size_t>(rows) + 7) & ~static_cast<size_t>(7)) + 8 * static_cast<size_t>(n_seq);
    return static_cast<size_t>(nkv) * HD * ldt * 2;
}

extern "C" size_t dc_attention_scratch_bytes(uint32_t rows, uint32_t n_seq, uint32_t nkv) { return dc_attention_tc_scratch_bytes(rows, n_seq, nkv); }

int dc_attention_tc_warm(dc_ctx* ctx) {
    static bool attr_set[16] = {};
    if (!attr_set[ctx->device & 15]) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel<ActF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Smem::kBytes));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_tc_kernel<ActBF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Smem::kBytes));
        if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "attention: cannot opt in to %zu bytes of shared memory: %s", Smem::kBytes, cudaGetErrorString(e));
        attr_set[ctx->device & 15] = true;
    }
    return DC_OK;
}

int dc_attention_tc(dc_ctx* ctx, cudaStream_t s, const void* q, const void* kc, const void* vc, const float* gate, const uint32_t* qpos, void* y,
                    uint32_t rows, uint32_t ldg, uint32_t nq, uint32_t nkv, const uint32_t* seq_start, uint32_t n_seq, uint32_t max_len, uint32_t kv_len) {
    // Packed batch (seq_start): query rows and cache rows are packed alike, `rows` of each. One sequence without seq_start:
    // `rows` query rows (a chunk) over cache rows 0 .. kv_len.
    const bool f16 = ctx->act_dtype == DC_ACT_F16;
    const uint32_t kv_rows = seq_start ? rows : kv_len, kv_max = seq_start ? max_len : kv_len;
    const uint32_t ldt = ((kv_rows + 7u) & ~7u) + 8u * n_seq;
    void* ws = nullptr;
    int rc = dc_get_workspace(ctx, dc_attention_tc_scratch_bytes(kv_rows, n_seq, nkv), "attention", &ws);
    if (rc != DC_OK) return rc;
    uint16_t* vt = static_cast<uint16_t*>(ws);
    CUtensorMap tq, tk, tv;
    rc = dc_make_tmap(ctx, q, rows, nq * HD, nq * HD, TQ, f16, &tq);
    if (rc == DC_OK) rc = dc_make_tmap(ctx, kc, kv_rows, nkv * HD, nkv * HD, TKV, f16, &tk);   // rows past the end read as zeros
    if (rc == DC_OK) rc = dc_make_tmap(ctx, vt, nkv * HD, ldt, ldt, HD, f16, &tv);
    if (rc != DC_OK) return rc;
    v_transpose_kernel<<<dim3((kv_max + 16 + 63) / 64, nkv, n_seq), 256, 0, s>>>(static_cast<const uint16_t*>(vc), vt, kv_rows, nkv, ldt, seq_start, n_seq, kv_len);
    rc = dc_check_launch(ctx, "attention (V transpose)");
    if (rc != DC_OK) return rc;
    rc = dc_attention_tc_warm(ctx);
    if (rc != DC_OK) return rc;
    const float scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(HD));
    const dim3 grid((max_len + TQ - 1) / TQ, nq, n_seq);
    auto kern = f16 ? attn_tc_kernel<ActF16> : attn_tc_kernel<ActBF16>;
    kern<<<grid, kThreads, Smem::kBytes, s>>>(tq, tk, tv, gate, qpos, static_cast<uint16_t*>(y), ldg, nq, nkv, scale_log2, seq_start, rows, kv_len, ctx->status_dev);
    return dc_check_launch(ctx, "attention (tcgen05)");
}
