// Chunk-64 gated delta rule (the WY / UT-transform form) on tensor cores.
//
// Same recurrence as the sequential kernel of delta.cu (spec cpu_ref.rs:101-129), regrouped per
// chunk of C = 64 tokens as the reference's gold model does (the torch_chunk_gated_delta_rule of the
// transformers Qwen3.5 model). With G_i the cumulative log decay inside the chunk, beta_i the write
// strength and S the state before the chunk (here S is [dk][dv]):
//   L   = strictly-lower( beta_i (k_i . k_j) e^{G_i - G_j} )            T = (I + L)^-1
//   W   = T (beta k e^{G})                 U = T (beta v)
//   v'  = U - W S                          o = (q e^{G}) S + lower((q_i . k_j) e^{G_i - G_j}) v'
//   S  <- e^{G_last} S + (k e^{G_last - G})^T v'
// Kernel 1 (all chunks of all heads and sequences in parallel) builds T, W, U and the masked q.k
// matrix into scratch. Kernel 2 walks the chunks of one (sequence, head, value-column block) in
// order with the state in registers. All products run on mma.sync bf16 with fp32 accumulation; by
// default every fp32 operand is split into hi + lo bf16 parts (3 MMAs per product, relative error
// ~1e-5 against fp32), because a single bf16/fp16 pass puts ~5e-4 relative error into o.
#include "common.cuh"
#include "mma.cuh"
#include "ptx.cuh"

namespace {

using namespace dc;

constexpr int C = 64;            // chunk length
constexpr int D = 128;           // dk = dv
constexpr int LD = 65;           // padded row stride of the fp32 64x64 work matrices

// Scratch of one (chunk, head), written by kernel 1 in exactly the shared-memory form kernel 2 wants
// (bf16 hi [+ lo] tiles, already swizzled), so kernel 2 fills its operands with flat cp.async copies:
//   W  [64][128]   T (beta k e^G)                       A operand of W S
//   Qg [64][128]   q e^G                                A operand of (q e^G) S
//   Kd [64][128]   k e^{G_last - G}                     A^T operand of the state update
//   A  [64][64]    lower((q_i . k_j) e^{G_i - G_j})     A operand of A v'
//   U  [64][128]   fp32, T (beta v)
//   e^{G_last}
template <int SPLIT>
struct Slot {
    static constexpr int NL = SPLIT == 3 ? 2 : 1;            // tiles per operand: hi (+ lo)
    static constexpr size_t kW = 0;                           // byte offsets
    static constexpr size_t kQg = kW + NL * C * D * 2;
    static constexpr size_t kKd = kQg + NL * C * D * 2;
    static constexpr size_t kA = kKd + NL * C * D * 2;
    static constexpr size_t kU = kA + NL * C * C * 2;
    static constexpr size_t kDecay = kU + C * D * 4;
    static constexpr size_t kBytes = kDecay + 16;
};

// The same scratch for the tcgen05 form of kernel 2 (split 3 only). Every bf16 tile is K-major with
// 128-byte rows of 64 elements and the 128-byte swizzle a tensor-map copy would produce (the 16-byte
// chunk c of row r sits at chunk position c ^ (r & 7)), so tcgen05.mma reads it through a shared-
// memory descriptor after one flat bulk copy:
//   WQ  [hi|lo][k-atom 2][128 rows][64]   B operand of S W^T | S Qg^T: W in rows 0..63 and Qg in rows
//       64..127 for even chunks of a sequence, the other way round for odd chunks
//   AK  [hi|lo]{ A [64 i][64 j] ; Kd^T [128 dk][64 j] }                   B operands of v'^T A^T and v'^T Kd
//   U, e^{G_last} as above
struct SlotTC {
    static constexpr size_t kAtom128 = 128 * 128;             // bytes of one k-atom of a 128-row tile
    static constexpr size_t kWQ = 0;
    static constexpr size_t kWQPart = 2 * kAtom128;           // hi or lo
    static constexpr size_t kAK = kWQ + 2 * kWQPart;
    static constexpr size_t kAKPart = 64 * 128 + kAtom128;    // hi or lo: A then Kd^T
    static constexpr size_t kU = kAK + 2 * kAKPart;
    static constexpr size_t kDecay = kU + C * D * 4;
    static constexpr size_t kBytes = kDecay + 16;
};
static_assert(SlotTC::kBytes == Slot<3>::kBytes && SlotTC::kU == Slot<3>::kU, "both scratch layouts share slot size and the U offset");

// Element offset of (row, k) in a K-major tile of ROWS rows made of 64-element k-atoms, 128-byte swizzle.
template <int ROWS>
__device__ __forceinline__ int umma_off(int row, int k) {
    return (k >> 6) * ROWS * 64 + row * 64 + ((((k & 63) >> 3) ^ (row & 7)) << 3) + (k & 7);
}
// hi/lo bf16 stores (four values, 8 bytes per part) at an element offset of a tile pair; the lo tile lies `lo_bytes` after the hi tile
__device__ __forceinline__ void tc_put4(uint8_t* hi_base, size_t lo_bytes, int off, const float4& v) {
    const __nv_bfloat162 h0 = __floats2bfloat162_rn(v.x, v.y), h1 = __floats2bfloat162_rn(v.z, v.w);
    const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);
    const __nv_bfloat162 l0 = __floats2bfloat162_rn(v.x - f0.x, v.y - f0.y), l1 = __floats2bfloat162_rn(v.z - f1.x, v.w - f1.y);
    uint2 w;
    w.x = *reinterpret_cast<const uint32_t*>(&h0);
    w.y = *reinterpret_cast<const uint32_t*>(&h1);
    *reinterpret_cast<uint2*>(hi_base + 2 * off) = w;
    w.x = *reinterpret_cast<const uint32_t*>(&l0);
    w.y = *reinterpret_cast<const uint32_t*>(&l1);
    *reinterpret_cast<uint2*>(hi_base + lo_bytes + 2 * off) = w;
}

struct ChunkArgs {
    const float *q, *k, *v, *a, *b, *a_log, *dt_bias;
    const float* state_in;
    float* state_out;
    float* o;
    uint8_t* scratch;
    const uint32_t* seq_start;
    uint32_t t, ldab, nk, nv, write_state;
    // fused conv (tcgen05 kernel 1 only): raw projection rows (stride ldp: q | k | v channels), taps [channels][4],
    // the 3 raw rows before each sequence (or null); q, k, v above are then unused
    const float* praw;
    const float* conv_w;
    const float* conv_prev;
    uint32_t ldp;
};

__device__ __forceinline__ void seq_bounds(const ChunkArgs& p, uint32_t seq, uint32_t& row_lo, uint32_t& len) {
    row_lo = p.seq_start ? p.seq_start[seq] : 0u;
    len = p.seq_start ? p.seq_start[seq + 1] - row_lo : p.t;
}
// Scratch slot of chunk c of a sequence: row_lo / 64 + seq + c never collides between sequences.
template <int SPLIT>
__device__ __forceinline__ uint8_t* slot_ptr(const ChunkArgs& p, uint32_t row_lo, uint32_t seq, uint32_t c, uint32_t h) {
    const size_t slot = static_cast<size_t>(row_lo / C + seq + c);
    return p.scratch + (slot * p.nv + h) * Slot<SPLIT>::kBytes;
}

// ---------------------------------------------------------------------------------------------
// Inverse of I + L for a strictly lower triangular 64x64 L (fp32, row stride LD) into N, by 16x16
// blocks: the four diagonal blocks by in-warp forward substitution, then the off-diagonal blocks
// one block-diagonal at a time, N_ij = -N_ii * sum_{k=j}^{i-1} L_ik N_kj. Called by warps 0..3 only,
// which synchronise among themselves on named barrier 1.
__device__ __forceinline__ void bar4() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ void invert_unit_lower(const float* __restrict__ L, float* __restrict__ N, float* __restrict__ P, int warp, int lane) {
    {   // diagonal block `warp`: lane l < 16 holds column l; row i of the result needs rows < i
        const int b0 = 16 * warp;
        const int l = lane & 15;
        float a[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) a[i] = L[(b0 + i) * LD + b0 + l];
#pragma unroll
        for (int i = 1; i < 16; ++i) {
            float acc = a[i];
#pragma unroll
            for (int j = 0; j < i; ++j) {
                const float cij = __shfl_sync(0xffffffffu, a[i], j);  // L[i][j], not yet overwritten
                acc = fmaf(-cij, a[j], acc);                           // a[j] is already row j of the result
            }
            // (I + L)^-1 = I + X with X_i = -L_i - sum_j L_ij X_j; a[] holds Y = -X: Y_i = L_i - sum_j L_ij Y_j
            a[i] = acc;
        }
        if (lane < 16) {
#pragma unroll
            for (int i = 0; i < 16; ++i) N[(b0 + i) * LD + b0 + l] = (i == l) ? 1.0f : (l < i ? -a[i] : 0.0f);
        }
        // blocks above the diagonal are zero
        for (int e = lane; e < 16 * 16 * 3; e += 32) {
            const int jb = e / 256, r = (e / 16) % 16, cc = e % 16;
            const int bj = (warp + 1 + jb);
            if (bj < 4) N[(b0 + r) * LD + 16 * bj + cc] = 0.0f;
        }
    }
    float* Pw = P + warp * 16 * 17;
    const int r = lane >> 1, c0 = (lane & 1) * 8;
    for (int d = 1; d < 4; ++d) {
        bar4();
        const int i = d + warp, j = warp;  // block (i, j) with i - j = d
        if (i < 4) {
            float acc[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[c] = 0.f;
            for (int kb = j; kb < i; ++kb) {
#pragma unroll 4
                for (int t = 0; t < 16; ++t) {
                    const float lv = L[(16 * i + r) * LD + 16 * kb + t];
                    const float* nrow = N + (16 * kb + t) * LD + 16 * j + c0;
#pragma unroll
                    for (int c = 0; c < 8; ++c) acc[c] = fmaf(lv, nrow[c], acc[c]);
                }
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) Pw[r * 17 + c0 + c] = acc[c];
            __syncwarp();
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[c] = 0.f;
#pragma unroll 4
            for (int t = 0; t < 16; ++t) {
                const float nv = N[(16 * i + r) * LD + 16 * i + t];
#pragma unroll
                for (int c = 0; c < 8; ++c) acc[c] = fmaf(nv, Pw[t * 17 + c0 + c], acc[c]);
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) N[(16 * i + r) * LD + 16 * j + c0 + c] = -acc[c];
        }
    }
    bar4();
}


// (x0, x1) at (row, col) of a swizzled bf16 tile pair [rows][CW] in GLOBAL memory: hi at `base`, lo right after it.
template <int CW, int ROWS, int SPLIT>
__device__ __forceinline__ void gput2(uint8_t* base, int row, int col, float x0, float x1) {
    __nv_bfloat16* hi = reinterpret_cast<__nv_bfloat16*>(base);
    put2<CW, SPLIT>(hi, hi + ROWS * CW, row, col, x0, x1);
}

template <int CW, int ROWS, int SPLIT>
__device__ __forceinline__ void gput4(uint8_t* base, int row, int col, const float4& v) {
    __nv_bfloat16* hi = reinterpret_cast<__nv_bfloat16*>(base);
    put4<CW, SPLIT>(hi, hi + ROWS * CW, row, col, v);
}

// ---------------------------------------------------------------------------------------------
// Kernel 1 on mma.sync (DC_ENGINE_MMA_SYNC, and split 1): one CTA (8 warps) per (chunk, head, sequence), two CTAs per SM. Shared memory: K and Q
// tiles (hi, lo), reused later for beta*k*e^G and beta*v; the fp32 L and N matrices; T tiles aliased
// onto L.
constexpr size_t kPrepSmem = 4 * C * D * 2 + 2 * C * LD * 4 + 4 * 16 * 17 * 4 + 5 * C * 4;

template <int SPLIT>
__global__ void __launch_bounds__(256, 2) delta_chunk_prepare_kernel(const ChunkArgs p) {
    using SL = Slot<SPLIT>;
    extern __shared__ __align__(16) uint8_t smem[];
    __nv_bfloat16* kh = reinterpret_cast<__nv_bfloat16*>(smem);
    __nv_bfloat16* kl = kh + C * D;
    __nv_bfloat16* qh = kl + C * D;
    __nv_bfloat16* ql = qh + C * D;
    float* Lf = reinterpret_cast<float*>(ql + C * D);
    float* Nf = Lf + C * LD;
    float* Pf = Nf + C * LD;
    float* Gs = Pf + 4 * 16 * 17;
    float* Bs = Gs + C;
    __nv_bfloat16* th = reinterpret_cast<__nv_bfloat16*>(Lf);  // T tiles reuse L once the inverse is in N
    __nv_bfloat16* tl = th + C * C;

    const uint32_t seq = blockIdx.z, h = blockIdx.y, c = blockIdx.x;
    uint32_t row_lo, len;
    seq_bounds(p, seq, row_lo, len);
    const uint32_t r0 = c * C;
    if (r0 >= len) return;
    const int n = static_cast<int>(min(static_cast<uint32_t>(C), len - r0));
    const uint32_t hk = h / (p.nv / p.nk);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wr = warp & 3, wc = warp >> 2;
    const size_t row_base = static_cast<size_t>(row_lo) + r0;
    uint8_t* slot = slot_ptr<SPLIT>(p, row_lo, seq, c, h);
    // gates; rows past the sequence end are padding: no decay, no write (g = 0, beta = 0, k = v = q = 0)
    if (tid < C) {
        float g = 0.f, be = 0.f;
        if (tid < n) {
            const size_t row = row_base + tid;
            g = -expf(p.a_log[h]) * softplus_precise(p.a[row * p.ldab + h] + p.dt_bias[h]);
            be = 1.0f / (1.0f + expf(-p.b[row * p.ldab + h]));
        }
        Nf[tid] = g;  // staging for the prefix sum
        Bs[tid] = be;
    }
    __syncthreads();
    if (tid < C) {
        float acc = 0.f;
        for (int i = 0; i <= tid; ++i) acc += Nf[i];
        Gs[tid] = acc;
    }
    __syncthreads();
    const float glast = Gs[C - 1];
    if (tid == 0) *reinterpret_cast<float*>(slot + SL::kDecay) = expf(glast);
    // per-row scale factors: e^G (for q), e^{G_last - G} (for k), beta e^G (for W's operand)
    float* Eq = Bs + C;
    float* Ek = Eq + C;
    float* Es = Ek + C;
    if (tid < C) {
        const float g = Gs[tid];
        Eq[tid] = expf(g);
        Ek[tid] = expf(glast - g);
        Es[tid] = Bs[tid] * expf(g);
    }
    __syncthreads();

    {   // K and Q tiles into shared memory; q e^G and k e^{G_last - G} tiles straight to scratch
        float4 kv[8], qv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = tid + 256 * i, r = e >> 5, c4 = (e & 31) * 4;
            kv[i] = qv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < n) {
                kv[i] = *reinterpret_cast<const float4*>(p.k + ((row_base + r) * p.nk + hk) * D + c4);
                qv[i] = *reinterpret_cast<const float4*>(p.q + ((row_base + r) * p.nk + hk) * D + c4);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = tid + 256 * i, r = e >> 5, c4 = (e & 31) * 4;
            put4<D, SPLIT>(kh, kl, r, c4, kv[i]);
            put4<D, SPLIT>(qh, ql, r, c4, qv[i]);
            const float eq = Eq[r], ek = Ek[r];
            gput4<D, C, SPLIT>(slot + SL::kQg, r, c4, make_float4(qv[i].x * eq, qv[i].y * eq, qv[i].z * eq, qv[i].w * eq));
            gput4<D, C, SPLIT>(slot + SL::kKd, r, c4, make_float4(kv[i].x * ek, kv[i].y * ek, kv[i].z * ek, kv[i].w * ek));
        }
    }
    __syncthreads();
    const int m0 = 16 * wr;
    {   // k.k^T and q.k^T: 16 rows x 32 columns per warp
        float akk[4][4], aqk[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) akk[i][j] = aqk[i][j] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t kah[4], kal[4], qah[4], qal[4];
            lda<D>(kah, kh, m0, 16 * ks, lane);
            lda<D>(qah, qh, m0, 16 * ks, lane);
            if constexpr (SPLIT == 3) {
                lda<D>(kal, kl, m0, 16 * ks, lane);
                lda<D>(qal, ql, m0, 16 * ks, lane);
            }
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t bh[4], bl[4];
                ldb_nt<D>(bh, kh, 32 * wc + 16 * np, 16 * ks, lane);
                if constexpr (SPLIT == 3) ldb_nt<D>(bl, kl, 32 * wc + 16 * np, 16 * ks, lane);
                mma_split<SPLIT>(akk[2 * np], akk[2 * np + 1], kah, kal, bh, bl);
                mma_split<SPLIT>(aqk[2 * np], aqk[2 * np + 1], qah, qal, bh, bl);
            }
        }
        const int i0 = m0 + (lane >> 2), i1 = i0 + 8;
        const float g0 = Gs[i0], g1 = Gs[i1], b0 = Bs[i0], b1 = Bs[i1];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int jb = 32 * wc + nt * 8 + 2 * (lane & 3);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = jb + e;
                const float gj = Gs[j];
                const float d0 = j <= i0 ? expf(g0 - gj) : 0.f;
                const float d1 = j <= i1 ? expf(g1 - gj) : 0.f;
                Lf[i0 * LD + j] = j < i0 ? b0 * akk[nt][e] * d0 : 0.f;
                Lf[i1 * LD + j] = j < i1 ? b1 * akk[nt][2 + e] * d1 : 0.f;
                aqk[nt][e] *= d0;
                aqk[nt][2 + e] *= d1;
            }
            gput2<C, C, SPLIT>(slot + SL::kA, i0, jb, aqk[nt][0], aqk[nt][1]);
            gput2<C, C, SPLIT>(slot + SL::kA, i1, jb, aqk[nt][2], aqk[nt][3]);
        }
    }
    __syncthreads();
    if (warp < 4) {
        // warps 0..3: T = (I + L)^-1, then its bf16 tiles (which reuse L's storage)
        invert_unit_lower(Lf, Nf, Pf, warp, lane);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int e = tid + 128 * i, r = e >> 5, c2 = (e & 31) * 2;
            put2<C, SPLIT>(th, tl, r, c2, Nf[r * LD + c2], Nf[r * LD + c2 + 1]);
        }
    } else {
        // warps 4..7 meanwhile: beta*k*e^G into the Q tiles, beta*v into the K tiles (both [token][feature])
        const int t2 = tid - 128;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
            float4 kv[8], vv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int e = t2 + 128 * (8 * half + i), r = e >> 5, c4 = (e & 31) * 4;
                kv[i] = vv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r < n) {
                    kv[i] = *reinterpret_cast<const float4*>(p.k + ((row_base + r) * p.nk + hk) * D + c4);
                    vv[i] = *reinterpret_cast<const float4*>(p.v + ((row_base + r) * p.nv + h) * D + c4);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int e = t2 + 128 * (8 * half + i), r = e >> 5, c4 = (e & 31) * 4;
                const float be = Bs[r], sk = Es[r];
                kv[i].x *= sk; kv[i].y *= sk; kv[i].z *= sk; kv[i].w *= sk;
                vv[i].x *= be; vv[i].y *= be; vv[i].z *= be; vv[i].w *= be;
                put4<D, SPLIT>(qh, ql, r, c4, kv[i]);
                put4<D, SPLIT>(kh, kl, r, c4, vv[i]);
            }
        }
    }
    __syncthreads();

    // W = T (beta k e^G), U = T (beta v): 16 rows x 64 columns per warp
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
        const __nv_bfloat16* bh_t = which == 0 ? qh : kh;
        const __nv_bfloat16* bl_t = which == 0 ? ql : kl;
        float acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll
        for (int ks = 0; ks < C / 16; ++ks) {
            uint32_t ah[4], al[4];
            lda<C>(ah, th, m0, 16 * ks, lane);
            if constexpr (SPLIT == 3) lda<C>(al, tl, m0, 16 * ks, lane);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t bh[4], bl[4];
                ldb_nn<D>(bh, bh_t, 16 * ks, 64 * wc + 16 * np, lane);
                if constexpr (SPLIT == 3) ldb_nn<D>(bl, bl_t, 16 * ks, 64 * wc + 16 * np, lane);
                mma_split<SPLIT>(acc[2 * np], acc[2 * np + 1], ah, al, bh, bl);
            }
        }
        const int i0 = m0 + (lane >> 2), i1 = i0 + 8;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int j = 64 * wc + nt * 8 + 2 * (lane & 3);
            if (which == 0) {
                gput2<D, C, SPLIT>(slot + SL::kW, i0, j, acc[nt][0], acc[nt][1]);
                gput2<D, C, SPLIT>(slot + SL::kW, i1, j, acc[nt][2], acc[nt][3]);
            } else {
                float* sU = reinterpret_cast<float*>(slot + SL::kU);
                *reinterpret_cast<float2*>(sU + i0 * D + j) = make_float2(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<float2*>(sU + i1 * D + j) = make_float2(acc[nt][2], acc[nt][3]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Kernel 2: one CTA (8 warps) per (value-column block of DVB, head, sequence) walks the chunks in
// order. The state block S[dk][DVB] lives in registers (warp w owns dk rows 16w..16w+15) and, split
// into bf16 tiles, in shared memory as the B operand of W S and (q e^G) S. The chunk operands arrive
// by cp.async in two groups that overlap with the MMAs: {W, Qg} of chunk c+1 stream in while chunk c
// does its second half, {Kd, A} of chunk c while it does its first half.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void copy_async(uint8_t* dst, const uint8_t* src, int bytes, int tid) {
    for (int o = tid * 16; o < bytes; o += 256 * 16) cp_async16(dst + o, src + o);
}

template <int DVB, int SPLIT>
constexpr size_t apply_smem() {
    return Slot<SPLIT>::kU + static_cast<size_t>(Slot<SPLIT>::NL) * 2 * (D * DVB + C * DVB);
}

template <int DVB, int SPLIT>
__global__ void __launch_bounds__(256, 1) delta_chunk_apply_kernel(const ChunkArgs p) {
    using SL = Slot<SPLIT>;
    constexpr int NL = SL::NL;
    constexpr int NTW = DVB / 16;                     // n-tiles per warp for the 64-row products
    constexpr int NTS = DVB / 8;                      // n-tiles of the state block
    extern __shared__ __align__(16) uint8_t smem[];
    // the first kU bytes mirror a scratch slot: W, Qg | Kd, A
    __nv_bfloat16* Wh = reinterpret_cast<__nv_bfloat16*>(smem + SL::kW);   __nv_bfloat16* Wl = Wh + (NL - 1) * C * D;
    __nv_bfloat16* Qh = reinterpret_cast<__nv_bfloat16*>(smem + SL::kQg);  __nv_bfloat16* Ql = Qh + (NL - 1) * C * D;
    __nv_bfloat16* Kh = reinterpret_cast<__nv_bfloat16*>(smem + SL::kKd);  __nv_bfloat16* Kl = Kh + (NL - 1) * C * D;
    __nv_bfloat16* Ah = reinterpret_cast<__nv_bfloat16*>(smem + SL::kA);   __nv_bfloat16* Al = Ah + (NL - 1) * C * C;
    __nv_bfloat16* Sh = reinterpret_cast<__nv_bfloat16*>(smem + SL::kU);   __nv_bfloat16* Sl = Sh + (NL - 1) * D * DVB;
    __nv_bfloat16* Vh = Sh + NL * D * DVB;                                 __nv_bfloat16* Vl = Vh + (NL - 1) * C * DVB;

    const uint32_t seq = blockIdx.z, h = blockIdx.y;
    const int dv0 = blockIdx.x * DVB;
    uint32_t row_lo, len;
    seq_bounds(p, seq, row_lo, len);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wr = warp & 3, wc = warp >> 2;
    const int m0 = 16 * wr;                 // row strip of the 64-row products
    const int nw0 = wc * (DVB / 2);         // column half of this warp in those products
    const int ms = 16 * warp;               // dk rows of the state owned by this warp
    const int i0 = lane >> 2, cq = 2 * (lane & 3);

    // state block into registers: Sreg[nt][{0,1}] = S[ms+i0][8nt+cq+{0,1}], [{2,3}] = row ms+i0+8
    float Sreg[NTS][4];
    const size_t sbase = (static_cast<size_t>(seq) * p.nv + h) * D * D;   // [dv][dk]
#pragma unroll
    for (int nt = 0; nt < NTS; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int dk = ms + i0 + (e >> 1) * 8, dv = dv0 + nt * 8 + cq + (e & 1);
            Sreg[nt][e] = p.state_in ? p.state_in[sbase + static_cast<size_t>(dv) * D + dk] : 0.f;
        }

    const uint32_t n_chunks = (len + C - 1) / C;
    if (n_chunks) copy_async(smem + SL::kW, slot_ptr<SPLIT>(p, row_lo, seq, 0, h) + SL::kW, static_cast<int>(SL::kKd - SL::kW), tid);
    cp_async_commit();
    for (uint32_t c = 0; c < n_chunks; ++c) {
        const uint32_t r0 = c * C;
        const int n = static_cast<int>(min(static_cast<uint32_t>(C), len - r0));
        const size_t row_base = static_cast<size_t>(row_lo) + r0;
        const uint8_t* slot = slot_ptr<SPLIT>(p, row_lo, seq, c, h);
        const float* sU = reinterpret_cast<const float*>(slot + SL::kU);

        copy_async(smem + SL::kKd, slot + SL::kKd, static_cast<int>(SL::kU - SL::kKd), tid);
        cp_async_commit();
        // U values this thread will need after the first products, and the chunk's total decay
        float2 u0[NTW], u1[NTW];
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
            const int col = dv0 + nw0 + nt * 8 + cq;
            u0[nt] = *reinterpret_cast<const float2*>(sU + (m0 + i0) * D + col);
            u1[nt] = *reinterpret_cast<const float2*>(sU + (m0 + i0 + 8) * D + col);
        }
        const float dl = *reinterpret_cast<const float*>(slot + SL::kDecay);
#pragma unroll
        for (int nt = 0; nt < NTS; ++nt) {
            put2<DVB, SPLIT>(Sh, Sl, ms + i0, nt * 8 + cq, Sreg[nt][0], Sreg[nt][1]);
            put2<DVB, SPLIT>(Sh, Sl, ms + i0 + 8, nt * 8 + cq, Sreg[nt][2], Sreg[nt][3]);
        }
        cp_async_wait<1>();   // {W, Qg} of this chunk have landed (issued one iteration ago)
        __syncthreads();

        // v' = U - W S   and   o = (q e^G) S   for rows m0.., columns nw0..
        float vp[NTW][4], oi[NTW][4];
#pragma unroll
        for (int i = 0; i < NTW; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) vp[i][j] = oi[i][j] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t wah[4], wal[4], qah[4], qal[4];
            lda<D>(wah, Wh, m0, 16 * ks, lane);
            lda<D>(qah, Qh, m0, 16 * ks, lane);
            if constexpr (SPLIT == 3) {
                lda<D>(wal, Wl, m0, 16 * ks, lane);
                lda<D>(qal, Ql, m0, 16 * ks, lane);
            }
#pragma unroll
            for (int np = 0; np < NTW / 2; ++np) {
                uint32_t bh[4], bl[4];
                ldb_nn<DVB>(bh, Sh, 16 * ks, nw0 + 16 * np, lane);
                if constexpr (SPLIT == 3) ldb_nn<DVB>(bl, Sl, 16 * ks, nw0 + 16 * np, lane);
                mma_split<SPLIT>(vp[2 * np], vp[2 * np + 1], wah, wal, bh, bl);
                mma_split<SPLIT>(oi[2 * np], oi[2 * np + 1], qah, qal, bh, bl);
            }
        }
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
            const int col = nw0 + nt * 8 + cq;
            put2<DVB, SPLIT>(Vh, Vl, m0 + i0, col, u0[nt].x - vp[nt][0], u0[nt].y - vp[nt][1]);
            put2<DVB, SPLIT>(Vh, Vl, m0 + i0 + 8, col, u1[nt].x - vp[nt][2], u1[nt].y - vp[nt][3]);
        }
        cp_async_wait<0>();   // {Kd, A} of this chunk
        __syncthreads();      // v' tiles and {Kd, A} visible; everyone is done with W, Qg and the S tiles
        if (c + 1 < n_chunks) copy_async(smem + SL::kW, slot_ptr<SPLIT>(p, row_lo, seq, c + 1, h) + SL::kW, static_cast<int>(SL::kKd - SL::kW), tid);
        cp_async_commit();

        // o += lower(q.k e^{..}) v'
#pragma unroll
        for (int ks = 0; ks < C / 16; ++ks) {
            uint32_t ah[4], al[4];
            lda<C>(ah, Ah, m0, 16 * ks, lane);
            if constexpr (SPLIT == 3) lda<C>(al, Al, m0, 16 * ks, lane);
#pragma unroll
            for (int np = 0; np < NTW / 2; ++np) {
                uint32_t bh[4], bl[4];
                ldb_nn<DVB>(bh, Vh, 16 * ks, nw0 + 16 * np, lane);
                if constexpr (SPLIT == 3) ldb_nn<DVB>(bl, Vl, 16 * ks, nw0 + 16 * np, lane);
                mma_split<SPLIT>(oi[2 * np], oi[2 * np + 1], ah, al, bh, bl);
            }
        }
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
            const int col = dv0 + nw0 + nt * 8 + cq;
            if (m0 + i0 < n) *reinterpret_cast<float2*>(p.o + ((row_base + m0 + i0) * p.nv + h) * D + col) = make_float2(oi[nt][0], oi[nt][1]);
            if (m0 + i0 + 8 < n) *reinterpret_cast<float2*>(p.o + ((row_base + m0 + i0 + 8) * p.nv + h) * D + col) = make_float2(oi[nt][2], oi[nt][3]);
        }

        // S <- e^{G_last} S + (k e^{G_last - G})^T v'   for dk rows ms..ms+15, all DVB columns
#pragma unroll
        for (int nt = 0; nt < NTS; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) Sreg[nt][e] *= dl;
#pragma unroll
        for (int ks = 0; ks < C / 16; ++ks) {
            uint32_t ah[4], al[4];
            lda_t<D>(ah, Kh, 16 * ks, ms, lane);
            if constexpr (SPLIT == 3) lda_t<D>(al, Kl, 16 * ks, ms, lane);
#pragma unroll
            for (int np = 0; np < NTS / 2; ++np) {
                uint32_t bh[4], bl[4];
                ldb_nn<DVB>(bh, Vh, 16 * ks, 16 * np, lane);
                if constexpr (SPLIT == 3) ldb_nn<DVB>(bl, Vl, 16 * ks, 16 * np, lane);
                mma_split<SPLIT>(Sreg[2 * np], Sreg[2 * np + 1], ah, al, bh, bl);
            }
        }
        __syncthreads();  // every warp is done with {Kd, A}, v' and the S tiles before they are overwritten
    }
    cp_async_wait<0>();
    if (p.write_state) {
#pragma unroll
        for (int nt = 0; nt < NTS; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int dk = ms + i0 + (e >> 1) * 8, dv = dv0 + nt * 8 + cq + (e & 1);
                p.state_out[sbase + static_cast<size_t>(dv) * D + dk] = Sreg[nt][e];
            }
    }
}

// ---------------------------------------------------------------------------------------------
// Kernel 2 on tcgen05: one CTA (8 warps) per (sequence, head) walks the chunks in order. Everything is
// transposed so that the 128 value columns are the M dimension (= TMEM lanes) of every product:
//   acc_v [dv][64]      = S W^T                  (then v'^T = U^T - acc_v)
//   acc_o [dv][64] x 2  = S Qg^T + v'^T A^T      (= o^T; two buffers, alternating by chunk)
//   acc_ds[dv][128]     = v'^T Kd                (the state increment)
// The A operands, S [dv][dk] and v'^T [dv][j], are written by the threads (thread = one dv row = one
// TMEM lane) as packed bf16 hi and lo parts straight into tensor memory, so the MMAs fetch only their B
// operands (W|Qg, A, Kd^T: K-major swizzled tiles, one flat 112 KB bulk copy per chunk, double-
// buffered) from shared memory; with both operands in shared memory these small products are bound by
// shared-memory bandwidth. Each product runs as lo*hi + hi*lo + hi*hi into one fp32 accumulator. The
// fp32 state stays in registers: warp w owns TMEM lanes 32(w%4).. (value columns) and the dk half w/4.
// All 512 TMEM columns are used: 320 of accumulators, 128 of S, 64 of v'.
// The serial chain of a chunk is: S -> S W^T -> v' -> v'^T Kd -> state. The two products that only feed
// o (S Qg^T, v'^T A^T) are issued behind the chain's products; o of chunk c is read out and stored
// while S W^T of chunk c+1 runs.
// Thread 0 issues the bulk copies and the MMAs. Every wait, the block-wide ones included, is a bounded
// mbarrier wait; when one gives up the CTA raises the status word, waits for its copies and MMAs in
// flight, frees its tensor memory and returns.
struct TcSmem {
    static constexpr size_t kOps = SlotTC::kU;                // W|Qg then A|Kd^T, hi and lo: the head of a scratch slot
    static constexpr size_t kBars = 2 * kOps;
    static constexpr size_t kBytes = kBars + 128 + 1024;      // barriers and flags; slack to align the base to 1 KB
};
static_assert(SlotTC::kWQ == 0 && SlotTC::kAK == 2 * SlotTC::kWQPart && SlotTC::kU == SlotTC::kAK + 2 * SlotTC::kAKPart, "operands are contiguous");
constexpr uint32_t kTcTmemCols = 512;
// accumulator columns (o: + 64 per buffer) and the packed-bf16 A operands (two K elements per column)
// S W^T and S Qg^T come out of ONE N=128 product: its 128 output columns are [acc_v | o buffer 0] for even chunks and
// [o buffer 1 | acc_v] for odd ones (kernel 1 swaps the row halves of the W|Qg tile accordingly), so acc_v sits between the two.
constexpr uint32_t kTcColO1 = 0, kTcColV = 64, kTcColO0 = 128, kTcColDs = 192, kTcColSHi = 320, kTcColSLo = 384, kTcColVHi = 448, kTcColVLo = 480;
constexpr uint32_t kABytes = 64 * 128;   // one (hi or lo) A tile; the Kd^T tile follows it

// Block-wide barrier on an mbarrier with one arrival per warp.
__device__ __forceinline__ bool tc_block_sync(uint64_t* bar, uint32_t& phase, int lane, volatile uint32_t* abort_flag, int* status, int code) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
    const bool ok = mbar_wait(bar, phase, abort_flag, status, code);
    phase ^= 1u;
    return ok;
}
// 2n fp32 values -> n columns of packed bf16 hi parts and n of lo parts
template <int N>
__device__ __forceinline__ void tc_split_pack(const float* x, uint32_t (&hi)[N], uint32_t (&lo)[N]) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
        const float2 hf = __bfloat1622float2(h2);
        const __nv_bfloat162 l2 = __floats2bfloat162_rn(x[2 * i] - hf.x, x[2 * i + 1] - hf.y);
        hi[i] = *reinterpret_cast<const uint32_t*>(&h2);
        lo[i] = *reinterpret_cast<const uint32_t*>(&l2);
    }
}
// D[tmem] (+)= A B^T with split operands over KSTEPS steps of 16 along K: A parts in tensor memory (8 columns
// per step), B parts K-major in shared memory with 128-byte rows (2 descriptor units of 16 bytes per step).
template <int KSTEPS>
__device__ __forceinline__ void tc_mma_split(uint32_t d_tmem, uint32_t a_hi, uint32_t a_lo, uint64_t b_hi, uint64_t b_lo, uint32_t idesc, bool accumulate) {
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        if (accumulate || ks > 0) umma_bf16_ts<true>(d_tmem, a_lo + 8 * ks, b_hi + 2 * ks, idesc);
        else umma_bf16_ts<false>(d_tmem, a_lo + 8 * ks, b_hi + 2 * ks, idesc);
        umma_bf16_ts<true>(d_tmem, a_hi + 8 * ks, b_lo + 2 * ks, idesc);
        umma_bf16_ts<true>(d_tmem, a_hi + 8 * ks, b_hi + 2 * ks, idesc);
    }
}


constexpr int kTcThreads = 288;   // warps 0..7 work on the rows, warp 8 issues the copies and the MMAs

__global__ void __launch_bounds__(kTcThreads, 1) delta_chunk_apply_tc_kernel(const ChunkArgs p, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TcSmem::kBars);
    uint64_t* full = bars + 0;       // [2] bulk copy of a chunk's operands landed in buffer b
    uint64_t* m1_done = bars + 2;    // S W^T finished
    uint64_t* ds_done = bars + 3;    // v'^T Kd finished (and S Qg^T before it)
    uint64_t* o_done = bars + 4;     // v'^T A^T finished: o^T complete, the chunk's operand buffer is free
    uint64_t* all_bar = bars + 5;    // block-wide barrier (9 arrivals, one per warp)
    uint64_t* drain_bar = bars + 6;  // teardown: MMAs still in flight
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* never_flag = tmem_slot + 2;   // stays 0: the teardown waits do not give up early

    const uint32_t seq = blockIdx.y, h = blockIdx.x;
    uint32_t row_lo, len;
    seq_bounds(p, seq, row_lo, len);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t n_chunks = (len + C - 1) / C;

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        mbar_init(m1_done, 1);
        mbar_init(ds_done, 1);
        mbar_init(o_done, 1);
        mbar_init(all_bar, 9);
        mbar_init(drain_bar, 1);
        *abort_flag = 0u;
        *never_flag = 0u;
        fence_mbar_init();
    }
    if (warp == 8) {
        tmem_alloc(tmem_slot, kTcTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 8) {
        // ------------------------------------------------------------------ issuer (one thread)
        if (lane == 0 && n_chunks) {
            uint32_t loads_issued = 0, loads_waited = 0, sync_ph = 0;
            auto load_ops = [&](uint32_t c) {   // the bulk copy of chunk c's operands into buffer c & 1
                mbar_arrive_expect_tx(&full[c & 1u], static_cast<uint32_t>(TcSmem::kOps));
                bulk_load(smem + (c & 1u) * TcSmem::kOps, slot_ptr<3>(p, row_lo, seq, c, h), static_cast<uint32_t>(TcSmem::kOps), &full[c & 1u]);
                loads_issued = c + 1;
            };
            auto sync_all = [&](int code) {
                mbar_arrive(all_bar);
                const bool ok = mbar_wait(all_bar, sync_ph, abort_flag, status, code);
                sync_ph ^= 1u;
                return ok;
            };
            load_ops(0);
            if (n_chunks > 1) load_ops(1);
            constexpr uint32_t idesc128 = umma_idesc(1, 1, 128, 128), idesc64 = umma_idesc(1, 1, 128, 64);
            const uint32_t t_shi = tmem_base + kTcColSHi, t_slo = tmem_base + kTcColSLo, t_vhi = tmem_base + kTcColVHi, t_vlo = tmem_base + kTcColVLo;
            // descriptors of the B tiles of operand buffer 0; buffer 1 lies kOps bytes (in 16-byte units) further
            const uint64_t d_wq_hi = umma_desc_k128(smem_u32(smem + SlotTC::kWQ)), d_wq_lo = umma_desc_k128(smem_u32(smem + SlotTC::kWQ + SlotTC::kWQPart));
            const uint64_t d_ak_hi = umma_desc_k128(smem_u32(smem + SlotTC::kAK)), d_ak_lo = umma_desc_k128(smem_u32(smem + SlotTC::kAK + SlotTC::kAKPart));
            constexpr uint64_t kBufStep = TcSmem::kOps >> 4, kAtomStep = SlotTC::kAtom128 >> 4, kKdStep = kABytes >> 4;
            for (uint32_t c = 0; c < n_chunks; ++c) {
                const uint32_t ph = c & 1u;
                const uint64_t boff = ph * kBufStep;
                if (!sync_all(21)) break;                                 // S is in tensor memory
                if (!mbar_wait(&full[ph], (c >> 1) & 1u, abort_flag, status, 22)) break;
                loads_waited = c + 1;
                tc_fence_after_sync();
#pragma unroll
                for (int ka = 0; ka < 2; ++ka)                            // [S W^T | S Qg^T] or [S Qg^T | S W^T]: acc_v and o buffer ph
                    tc_mma_split<4>(tmem_base + (ph ? kTcColO1 : kTcColV), t_shi + 32 * ka, t_slo + 32 * ka, d_wq_hi + boff + ka * kAtomStep,
                                    d_wq_lo + boff + ka * kAtomStep, idesc128, ka != 0);
                umma_commit(m1_done);
                if (c > 0 && c + 1 < n_chunks) {
                    // every product of the previous chunk is finished: its operand buffer takes the next chunk's
                    if (!mbar_wait(o_done, ph ^ 1u, abort_flag, status, 26)) break;
                    load_ops(c + 1);
                }
                if (!sync_all(24)) break;                                 // v' is in tensor memory
                tc_fence_after_sync();
                tc_mma_split<4>(tmem_base + kTcColDs, t_vhi, t_vlo, d_ak_hi + boff + kKdStep, d_ak_lo + boff + kKdStep, idesc128, false);
                umma_commit(ds_done);
                tc_mma_split<4>(tmem_base + (ph ? kTcColO1 : kTcColO0), t_vhi, t_vlo, d_ak_hi + boff, d_ak_lo + boff, idesc64, true);
                umma_commit(o_done);
            }
            if (*abort_flag) {
                // nothing may still be writing this CTA's shared or tensor memory when it exits
                for (uint32_t i = loads_waited; i < loads_issued; ++i) mbar_wait(&full[i & 1u], (i >> 1) & 1u, never_flag, status, 31);
                umma_commit(drain_bar);
                mbar_wait(drain_bar, 0u, never_flag, status, 32);
            }
        }
    } else {
        // ------------------------------------------------------------------ row workers
        const int q = warp & 3, hh = warp >> 2;
        const int dv = 32 * q + lane;
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(32 * q) << 16);
        // state row dv, dk half hh
        float Sreg[64];
        const size_t sbase = (static_cast<size_t>(seq) * p.nv + h) * D * D + static_cast<size_t>(dv) * D + 64 * hh;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.state_in) v4 = *reinterpret_cast<const float4*>(p.state_in + sbase + 4 * i);
            Sreg[4 * i] = v4.x; Sreg[4 * i + 1] = v4.y; Sreg[4 * i + 2] = v4.z; Sreg[4 * i + 3] = v4.w;
        }
        // the thread's 64 state values as 32 hi and 32 lo columns of TMEM lane dv
        auto write_s = [&]() {
#pragma unroll
            for (int part = 0; part < 2; ++part) {
                uint32_t hi[16], lo[16];
                tc_split_pack<16>(Sreg + 32 * part, hi, lo);
                tmem_st_32x32_x16(tlane + kTcColSHi + 32 * hh + 16 * part, hi);
                tmem_st_32x32_x16(tlane + kTcColSLo + 32 * hh + 16 * part, lo);
            }
            tmem_st_wait();
        };
        // o rows j = 32 hh .. + 31 (of `n` valid), column dv, from o buffer `buf`
        auto store_o = [&](uint32_t buf, size_t row_base, int n) {
            uint32_t r[32];
            tmem_ld_32x32(tlane + (buf ? kTcColO1 : kTcColO0) + 32 * hh, r);
            tmem_ld_wait();
            float* op = p.o + ((row_base + 32 * hh) * p.nv + h) * D + dv;
#pragma unroll
            for (int e = 0; e < 32; ++e)
                if (32 * hh + e < n) op[static_cast<size_t>(e) * p.nv * D] = __uint_as_float(r[e]);
        };
        uint32_t sync_ph = 0;
        // U^T values of this thread for one chunk: rows j = 32 hh + e, column dv. Fetched one chunk ahead.
        float u[32];
        auto load_u = [&](uint32_t c) {
            const float* sU = reinterpret_cast<const float*>(slot_ptr<3>(p, row_lo, seq, c, h) + SlotTC::kU) + (32 * hh) * D + dv;
#pragma unroll
            for (int e = 0; e < 32; ++e) u[e] = sU[e * D];
        };
        if (n_chunks) {
            load_u(0);
            write_s();
        }
        uint32_t c = 0;
        for (; c < n_chunks; ++c) {
            const uint32_t ph = c & 1u;
            const uint8_t* slot = slot_ptr<3>(p, row_lo, seq, c, h);
            const bool more = c + 1 < n_chunks;

            // S is in tensor memory; acc_v, acc_ds and o buffer `ph` have been read
            tc_fence_before_sync();
            if (!tc_block_sync(all_bar, sync_ph, lane, abort_flag, status, 21)) break;
            // while the first product runs: o of the previous chunk
            const float dl = *reinterpret_cast<const float*>(slot + SlotTC::kDecay);
            if (c > 0) {
                if (!mbar_wait(o_done, ph ^ 1u, abort_flag, status, 26)) break;
                __syncwarp();
                tc_fence_after_sync();
                store_o(ph ^ 1u, static_cast<size_t>(row_lo) + (c - 1) * C, C);
            }
            if (!mbar_wait(m1_done, ph, abort_flag, status, 23)) break;
            __syncwarp();
            tc_fence_after_sync();
            {   // v'^T = U^T - S W^T for rows j = 32 hh .. + 31 -> 16 hi and 16 lo columns of lane dv
                uint32_t r[32];
                tmem_ld_32x32(tlane + kTcColV + 32 * hh, r);
                tmem_ld_wait();
                float x[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) x[e] = u[e] - __uint_as_float(r[e]);
                uint32_t hi[16], lo[16];
                tc_split_pack<16>(x, hi, lo);
                tmem_st_32x32_x16(tlane + kTcColVHi + 16 * hh, hi);
                tmem_st_32x32_x16(tlane + kTcColVLo + 16 * hh, lo);
                tmem_st_wait();
            }
            tc_fence_before_sync();
            if (!tc_block_sync(all_bar, sync_ph, lane, abort_flag, status, 24)) break;
            if (more) load_u(c + 1);   // lands while the state increment is computed
            if (!mbar_wait(ds_done, ph, abort_flag, status, 29)) break;
            __syncwarp();
            tc_fence_after_sync();
#pragma unroll
            for (int half = 0; half < 2; ++half) {   // S <- e^{G_last} S + increment, dk = 64 hh + 32 half ..
                uint32_t r[32];
                tmem_ld_32x32(tlane + kTcColDs + 64 * hh + 32 * half, r);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) Sreg[32 * half + e] = fmaf(dl, Sreg[32 * half + e], __uint_as_float(r[e]));
            }
            if (more) write_s();
        }
        if (c == n_chunks && n_chunks) {   // o of the last chunk
            const uint32_t last = n_chunks - 1;
            if (mbar_wait(o_done, last & 1u, abort_flag, status, 30)) {
                __syncwarp();
                tc_fence_after_sync();
                store_o(last & 1u, static_cast<size_t>(row_lo) + last * C, static_cast<int>(len - last * C));
            }
        }
        __syncwarp();
        tmem_ld_wait();
        if (c == n_chunks && p.write_state) {
            float* so = p.state_out + sbase;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                *reinterpret_cast<float4*>(so + 4 * i) = make_float4(Sreg[4 * i], Sreg[4 * i + 1], Sreg[4 * i + 2], Sreg[4 * i + 3]);
        }
    }

    // ------------------------------------------------------------------------------ teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after_sync();
        __syncwarp();
        tmem_dealloc(tmem_base, kTcTmemCols);
    }
}

template <int DVB, int SPLIT>
int launch_apply(dc_ctx* ctx, cudaStream_t s, const ChunkArgs& a, uint32_t n_seq) {
    constexpr size_t smem = apply_smem<DVB, SPLIT>();
    static bool attr_set[16] = {};
    auto kern = delta_chunk_apply_kernel<DVB, SPLIT>;
    if (!attr_set[ctx->device & 15]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "gated_delta: cannot opt in to %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        attr_set[ctx->device & 15] = true;
    }
    kern<<<dim3(D / DVB, a.nv, n_seq), 256, smem, s>>>(a);
    return dc_check_launch(ctx, "gated_delta (chunk apply)");
}

// ---------------------------------------------------------------------------------------------
// Kernel 1 on tcgen05 (split 3, the scratch layout of the tcgen05 kernel 2): one CTA (8 warps) per
// (chunk, head, sequence), two CTAs per SM, 256 TMEM columns.
//   X = [k rows ; q rows] (128 x 128, bf16 hi/lo K-major tiles in shared memory, written row-wise by the
//       threads that loaded the rows)            acc1 = X k^T  ->  k.k^T (lanes 0..63) and q.k^T (lanes 64..127)
//   L, A out of acc1 (thread = row); the 64 x 64 inverse T on warps 0..3 in fp32 as in the mma.sync kernel,
//   while warps 4..7 (thread = feature column d) read k and v column-wise from global memory (coalesced
//   across the warp) and write (beta k e^G)^T and (beta v)^T as packed hi/lo A operands into tensor memory,
//   and Kd^T to scratch.
//   acc1 = (beta k e^G)^T T^T = W^T,  acc2 = (beta v)^T T^T = U^T    (T as the K-major B tile)
//   W^T goes back through shared memory into the row-major tile kernel 2 wants; U^T is stored as it is.
// Thread 0 issues the MMAs; the two waits on their completion are bounded, and a wait that gives up
// makes the whole CTA skip to the teardown (the decision is taken block-wide).
struct PrepTcSmem {
    static constexpr size_t kX = 0;                           // X tiles [hi|lo][2 k-atoms][128][64]; later the W staging tiles
    static constexpr size_t kL = kX + 4 * SlotTC::kAtom128;   // fp32 L [64][65]; later the T tiles [hi|lo][64][64]
    static constexpr size_t kN = kL + C * LD * 4;             // fp32 inverse
    static constexpr size_t kP = kN + C * LD * 4;             // scratch of the block inverse
    static constexpr size_t kG = kP + 4 * 16 * 17 * 4;        // G, beta, e^G, e^{G_last - G}, beta e^G, 1/|k|
    static constexpr size_t kBars = kG + 6 * C * 4;
    static constexpr size_t kBytes = kBars + 64 + 1024;
};
static_assert(2 * 64 * 128 <= C * LD * 4, "the T tiles fit where L was");
constexpr uint32_t kPrepTmemCols = 256;
constexpr uint32_t kPColAcc1 = 0, kPColAcc2 = 64, kPColKHi = 128, kPColKLo = 160, kPColVHi = 192, kPColVLo = 224;

__device__ __forceinline__ void split8_store(uint8_t* hi_dst, uint8_t* lo_dst, const float (&x)[8]) {
    uint32_t h[4], l[4];
    tc_split_pack<4>(x, h, l);
    *reinterpret_cast<uint4*>(hi_dst) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4*>(lo_dst) = make_uint4(l[0], l[1], l[2], l[3]);
}

// SiLU with the fast reciprocal (2 ulp): inside the fused conv, where an IEEE division per element would cost more than the conv.
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <bool CONV>
__global__ void __launch_bounds__(256, 2) delta_chunk_prepare_tc_kernel(const ChunkArgs p, int* __restrict__ status) {
    // heads fastest: CTAs that run at the same time read neighbouring 512-byte pieces of the same rows
    const uint32_t seq = blockIdx.z, h = blockIdx.x, c = blockIdx.y;
    uint32_t row_lo, len;
    seq_bounds(p, seq, row_lo, len);
    const uint32_t r0 = c * C;
    if (r0 >= len) return;
    const int n = static_cast<int>(min(static_cast<uint32_t>(C), len - r0));
    const uint32_t hk = h / (p.nv / p.nk);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const size_t row_base = static_cast<size_t>(row_lo) + r0;
    uint8_t* slot = slot_ptr<3>(p, row_lo, seq, c, h);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sX = smem + PrepTcSmem::kX;
    float* Lf = reinterpret_cast<float*>(smem + PrepTcSmem::kL);
    uint8_t* sT = smem + PrepTcSmem::kL;
    float* Nf = reinterpret_cast<float*>(smem + PrepTcSmem::kN);
    float* Pf = reinterpret_cast<float*>(smem + PrepTcSmem::kP);
    float* Gs = reinterpret_cast<float*>(smem + PrepTcSmem::kG);
    float* Bs = Gs + C;
    float* Eq = Bs + C;
    float* Ek = Eq + C;
    float* Es = Ek + C;
    float* Kinv = Es + C;   // fused conv: 1 / |k row| so that the column-wise pass can normalise what it recomputes
    uint64_t* mma_bar = reinterpret_cast<uint64_t*>(smem + PrepTcSmem::kBars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_bar + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    if (tid == 0) {
        mbar_init(mma_bar, 1);
        *abort_flag = 0u;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, kPrepTmemCols);
        tmem_relinquish();
    }
    // Fused conv: channels of this head's q, k, v in the raw projection rows; raw row s of the sequence (s may be -3..-1:
    // the rows before it, from conv_prev or zero)
    const uint32_t conv_dim = (2 * p.nk + p.nv) * D;
    const uint32_t ch_q = hk * D, ch_k = (p.nk + hk) * D, ch_v = (2 * p.nk + h) * D;
    auto raw4 = [&](int s, uint32_t ch) -> float4 {
        if (s >= static_cast<int>(len)) return make_float4(0.f, 0.f, 0.f, 0.f);
        if (s >= 0) return *reinterpret_cast<const float4*>(p.praw + (static_cast<size_t>(row_lo) + s) * p.ldp + ch);
        if (p.conv_prev) return *reinterpret_cast<const float4*>(p.conv_prev + (static_cast<size_t>(seq) * 3 + (3 + s)) * conv_dim + ch);
        return make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto raw1 = [&](int s, uint32_t ch) -> float {   // callers keep s below the sequence length
        if (s >= 0) return p.praw[(static_cast<size_t>(row_lo) + s) * p.ldp + ch];
        return p.conv_prev ? p.conv_prev[(static_cast<size_t>(seq) * 3 + (3 + s)) * conv_dim + ch] : 0.f;
    };
    // Pull the chunk's rows into L2 before anything else: each thread one 128-byte line of a k, a q and a v row (v is
    // wanted much later and column-wise; k and q a little later row-wise, after the gates).
    {
        const int r = tid >> 2;
        if (r < n) {
            const float* krow = CONV ? p.praw + (row_base + r) * p.ldp + ch_k : p.k + ((row_base + r) * p.nk + hk) * D;
            const float* qrow = CONV ? p.praw + (row_base + r) * p.ldp + ch_q : p.q + ((row_base + r) * p.nk + hk) * D;
            const float* vrow = CONV ? p.praw + (row_base + r) * p.ldp + ch_v : p.v + ((row_base + r) * p.nv + h) * D;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(krow + 32 * (tid & 3)));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(qrow + 32 * (tid & 3)));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(vrow + 32 * (tid & 3)));
        }
    }
    // gates of the 64 rows on threads 0..63, cumulative log decay by warp scans; rows past the sequence end are
    // padding: no decay, no write (g = 0, beta = 0, k = v = q = 0). Warps 0..1 do this before they request their
    // share of the rows below, so that nothing has to stay in registers across the transcendental code.
    float g_row = 0.f, be_row = 0.f;
    if (tid < C) {
        if (tid < n) {
            const size_t row = row_base + tid;
            g_row = -expf(p.a_log[h]) * softplus_precise(p.a[row * p.ldab + h] + p.dt_bias[h]);
            be_row = 1.0f / (1.0f + expf(-p.b[row * p.ldab + h]));
        }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, g_row, o);
            if (lane >= o) g_row += up;
        }
        if (lane == 31) Es[warp] = g_row;   // the warp's total, parked where beta e^G will go
    }
    // K and Q rows, a warp per row and instruction (coalesced; a float4 per lane). Plain: element e = tid + 256 i is row
    // e >> 5. Fused conv: warp w owns rows 8 w .. 8 w + 7 (slot i = row 8 w + i) and slides the 4-tap window down them.
    float4 kv[8], qv[8];
    if constexpr (!CONV) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = tid + 256 * i, r = e >> 5, c4 = (e & 31) * 4;
            kv[i] = qv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < n) {
                kv[i] = *reinterpret_cast<const float4*>(p.k + ((row_base + r) * p.nk + hk) * D + c4);
                qv[i] = *reinterpret_cast<const float4*>(p.q + ((row_base + r) * p.nk + hk) * D + c4);
            }
        }
    } else {
        // depthwise causal conv (4 taps) + SiLU, then the L2 norm over the head's 128 channels (eps inside the square
        // root; q also times 128^-1/2): conv.metal:5-35, cpu_ref.rs:55-81
        const int s0 = static_cast<int>(r0) + 8 * warp;
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {   // 0: k rows, 1: q rows (one copy of the code: the kernel must stay inside the instruction cache)
            const uint32_t ch = (which == 0 ? ch_k : ch_q) + 4 * lane;
            const float4 w0 = reinterpret_cast<const float4*>(p.conv_w)[ch + 0], w1 = reinterpret_cast<const float4*>(p.conv_w)[ch + 1];
            const float4 w2 = reinterpret_cast<const float4*>(p.conv_w)[ch + 2], w3 = reinterpret_cast<const float4*>(p.conv_w)[ch + 3];
            float4 x[11];
#pragma unroll
            for (int i = 0; i < 11; ++i) x[i] = raw4(s0 - 3 + i, ch);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float4 y;
                y.x = silu_fast(fmaf(w0.w, x[i + 3].x, fmaf(w0.z, x[i + 2].x, fmaf(w0.y, x[i + 1].x, w0.x * x[i].x))));
                y.y = silu_fast(fmaf(w1.w, x[i + 3].y, fmaf(w1.z, x[i + 2].y, fmaf(w1.y, x[i + 1].y, w1.x * x[i].y))));
                y.z = silu_fast(fmaf(w2.w, x[i + 3].z, fmaf(w2.z, x[i + 2].z, fmaf(w2.y, x[i + 1].z, w2.x * x[i].z))));
                y.w = silu_fast(fmaf(w3.w, x[i + 3].w, fmaf(w3.z, x[i + 2].w, fmaf(w3.y, x[i + 1].w, w3.x * x[i].w))));
                const float ss = warp_sum(y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w);
                const bool live = 8 * warp + i < n;
                const float rn = live ? rsqrtf(ss + 1e-6f) : 0.f;
                const float inv = which == 0 ? rn : rn * 0.08838834764831845f;
                y.x *= inv; y.y *= inv; y.z *= inv; y.w *= inv;
                qv[i] = y;
                if (which == 0 && lane == 0) Kinv[8 * warp + i] = rn;
            }
            if (which == 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) kv[i] = qv[i];
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    {
        const float tot0 = Es[0], glast = tot0 + Es[1];
        __syncthreads();   // both totals are read before Es is overwritten
        if (tid < C) {
            const float g = g_row + (warp == 1 ? tot0 : 0.f);
            Gs[tid] = g;
            Bs[tid] = be_row;
            Eq[tid] = expf(g);
            Ek[tid] = tid < n ? expf(glast - g) : 0.f;   // a padded row contributes nothing to the state
            Es[tid] = be_row * expf(g);
            if (tid == 0) *reinterpret_cast<float*>(slot + SlotTC::kDecay) = expf(glast);
        }
        __syncthreads();
    }

    {   // X tiles: k rows 0..63, q rows 64..127 (K-major, 8 bytes of hi and of lo per thread and row); q e^G to scratch
        const size_t lo_bytes = 2 * SlotTC::kAtom128;
        const int wq0 = c & 1u ? 0 : 64;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = CONV ? 8 * warp + i : (tid + 256 * i) >> 5, c4 = 4 * lane;
            tc_put4(sX, lo_bytes, umma_off<128>(r, c4), kv[i]);
            tc_put4(sX, lo_bytes, umma_off<128>(64 + r, c4), qv[i]);
            const float eq = Eq[r];
            tc_put4(slot + SlotTC::kWQ, SlotTC::kWQPart, umma_off<128>(wq0 + r, c4), make_float4(qv[i].x * eq, qv[i].y * eq, qv[i].z * eq, qv[i].w * eq));
        }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    constexpr uint32_t idesc64 = umma_idesc(1, 1, 128, 64);
    if (tid == 0) {   // acc1 = X k^T: 2 k-atoms x 4 steps, hi/lo terms
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint64_t off = (ks >> 2) * (SlotTC::kAtom128 >> 4) + 2 * (ks & 3);
            const uint64_t dh = umma_desc_k128(smem_u32(sX)) + off, dl = umma_desc_k128(smem_u32(sX + 2 * SlotTC::kAtom128)) + off;
            if (ks == 0) umma_bf16_ss<false>(tmem_base + kPColAcc1, dl, dh, idesc64);
            else umma_bf16_ss<true>(tmem_base + kPColAcc1, dl, dh, idesc64);
            umma_bf16_ss<true>(tmem_base + kPColAcc1, dh, dl, idesc64);
            umma_bf16_ss<true>(tmem_base + kPColAcc1, dh, dh, idesc64);
        }
        umma_commit(mma_bar);
    }
    bool ok = mbar_wait(mma_bar, 0u, abort_flag, status, 61);
    ok = __syncthreads_and(ok);
    if (ok) {
        tc_fence_after_sync();
        const int q4 = warp & 3, hh = warp >> 2;
        const int lrow = 32 * q4 + lane;                    // TMEM lane = X row
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(32 * q4) << 16);
        {   // L (lanes 0..63) into shared memory, A (lanes 64..127) to scratch; columns j = 32 hh ..
            uint32_t r[32];
            tmem_ld_32x32(tlane + kPColAcc1 + 32 * hh, r);
            tmem_ld_wait();
            const int i = lrow & 63;
            const float gi = Gs[i], bi = Bs[i];
            if (lrow < 64) {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int j = 32 * hh + e;
                    const float w = bi * __uint_as_float(r[e]) * __expf(gi - Gs[j]);
                    Lf[i * LD + j] = j < i ? w : 0.f;
                }
            } else {
                uint8_t* ah = sX + i * 128;   // staging mirrors the scratch layout of A | Kd^T, hi then lo
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    float x[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int j = 32 * hh + 8 * cc + e;
                        const float w = __uint_as_float(r[8 * cc + e]) * __expf(gi - Gs[j]);
                        x[e] = j <= i ? w : 0.f;
                    }
                    const int pos = ((4 * hh + cc) ^ (i & 7)) << 4;
                    split8_store(ah + pos, ah + SlotTC::kAKPart + pos, x);
                }
            }
        }
        tc_fence_before_sync();
        __syncthreads();
        if (warp < 4) {
            // warps 0..3: T = (I + L)^-1, then its K-major hi/lo tiles (which reuse L's storage)
            invert_unit_lower(Lf, Nf, Pf, warp, lane);
            const int trw = tid & 63, th = tid >> 6;   // row, 32-column half
            float tv[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) tv[e] = Nf[trw * LD + 32 * th + e];
            bar4();                                    // every row of L has been consumed before the tiles overwrite it
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                float x[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = tv[8 * cc + e];
                const int pos = ((4 * th + cc) ^ (trw & 7)) << 4;
                split8_store(sT + trw * 128 + pos, sT + 64 * 128 + trw * 128 + pos, x);
            }
            // ... then (beta v)^T into tensor memory, thread = value column d (the other four warps are busy with k)
            const int d = tid;
            const uint32_t tl4 = tmem_base + (static_cast<uint32_t>(32 * warp) << 16);
            const float* vp = CONV ? nullptr : p.v + (row_base * p.nv + h) * D + d;
            float4 tw = make_float4(0.f, 0.f, 0.f, 0.f);
            float x0 = 0.f, x1 = 0.f, x2 = 0.f;
            if constexpr (CONV) {
                tw = reinterpret_cast<const float4*>(p.conv_w)[ch_v + d];
                x0 = raw1(static_cast<int>(r0) - 3, ch_v + d);
                x1 = raw1(static_cast<int>(r0) - 2, ch_v + d);
                x2 = raw1(static_cast<int>(r0) - 1, ch_v + d);
            }
#pragma unroll 1
            for (int b = 0; b < 2; ++b) {
                float x[32];
                if constexpr (!CONV) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) x[e] = vp[static_cast<size_t>(min(32 * b + e, n - 1)) * p.nv * D];
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) x[e] = p.praw[(row_base + min(32 * b + e, n - 1)) * p.ldp + ch_v + d];
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const float x3 = x[e];
                        x[e] = silu_fast(fmaf(tw.w, x3, fmaf(tw.z, x2, fmaf(tw.y, x1, tw.x * x0))));
                        x0 = x1; x1 = x2; x2 = x3;
                    }
                }
#pragma unroll
                for (int e = 0; e < 32; ++e) x[e] *= Bs[32 * b + e];
                uint32_t hi[16], lo[16];
                tc_split_pack<16>(x, hi, lo);
                tmem_st_32x32_x16(tl4 + kPColVHi + 16 * b, hi);
                tmem_st_32x32_x16(tl4 + kPColVLo + 16 * b, lo);
            }
            tmem_st_wait();
        } else {
            // warps 4..7: thread = key column d. (beta k e^G)^T into tensor memory, Kd^T to the staging tiles
            const int d = tid - 128;
            const uint32_t tl4 = tmem_base + (static_cast<uint32_t>(32 * (warp - 4)) << 16);
            const float* kp = CONV ? nullptr : p.k + (row_base * p.nk + hk) * D + d;
            uint8_t* kdh = sX + kABytes + d * 128;   // staged like A
            // rows past the end are read from the last valid row and scaled by zero (beta, and e^{G_last - G}, are 0 there)
            // Fused conv: the column's raw values slide through the 4 taps; k is divided by its row norms from above.
            float4 tw = make_float4(0.f, 0.f, 0.f, 0.f);
            float x0 = 0.f, x1 = 0.f, x2 = 0.f;
            if constexpr (CONV) {
                tw = reinterpret_cast<const float4*>(p.conv_w)[ch_k + d];
                x0 = raw1(static_cast<int>(r0) - 3, ch_k + d);
                x1 = raw1(static_cast<int>(r0) - 2, ch_k + d);
                x2 = raw1(static_cast<int>(r0) - 1, ch_k + d);
            }
#pragma unroll 1
            for (int b = 0; b < 2; ++b) {   // 32 chunk rows at a time
                float kc[32];
                if constexpr (!CONV) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) kc[e] = kp[static_cast<size_t>(min(32 * b + e, n - 1)) * p.nk * D];
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) kc[e] = p.praw[(row_base + min(32 * b + e, n - 1)) * p.ldp + ch_k + d];
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const float x3 = kc[e];
                        kc[e] = silu_fast(fmaf(tw.w, x3, fmaf(tw.z, x2, fmaf(tw.y, x1, tw.x * x0)))) * Kinv[32 * b + e];
                        x0 = x1; x1 = x2; x2 = x3;
                    }
                }
                float x[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) x[e] = kc[e] * Es[32 * b + e];
                uint32_t hi[16], lo[16];
                tc_split_pack<16>(x, hi, lo);
                tmem_st_32x32_x16(tl4 + kPColKHi + 16 * b, hi);
                tmem_st_32x32_x16(tl4 + kPColKLo + 16 * b, lo);
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    float y[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) y[e] = kc[8 * cc + e] * Ek[32 * b + 8 * cc + e];
                    const int pos = ((4 * b + cc) ^ (d & 7)) << 4;
                    split8_store(kdh + pos, kdh + SlotTC::kAKPart + pos, y);
                }
            }
            tmem_st_wait();
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        if (tid == 0) {   // W^T = (beta k e^G)^T T^T, U^T = (beta v)^T T^T
            tc_fence_after_sync();
            const uint64_t th_d = umma_desc_k128(smem_u32(sT)), tl_d = umma_desc_k128(smem_u32(sT + 64 * 128));
            tc_mma_split<4>(tmem_base + kPColAcc1, tmem_base + kPColKHi, tmem_base + kPColKLo, th_d, tl_d, idesc64, false);
            tc_mma_split<4>(tmem_base + kPColAcc2, tmem_base + kPColVHi, tmem_base + kPColVLo, th_d, tl_d, idesc64, false);
            umma_commit(mma_bar);
        }
        {   // while those run: the staged A | Kd^T tiles (48 KB, laid out as in scratch) leave in whole lines
            const uint4* src = reinterpret_cast<const uint4*>(sX);
            uint4* dst = reinterpret_cast<uint4*>(slot + SlotTC::kAK);
#pragma unroll
            for (int i = 0; i < 12; ++i) dst[tid + 256 * i] = src[tid + 256 * i];
        }
        ok = mbar_wait(mma_bar, 1u, abort_flag, status, 62);
        ok = __syncthreads_and(ok);
        if (ok) {
            tc_fence_after_sync();
            const int d = lrow;   // TMEM lane = feature column; columns i = 32 hh ..
            {   // W^T -> the row-major staging tiles [hi|lo][2 k-atoms][64 rows][64] where X was
                uint32_t r[32];
                tmem_ld_32x32(tlane + kPColAcc1 + 32 * hh, r);
                tmem_ld_wait();
                uint8_t* wh = sX + (d >> 6) * (64 * 128) + (d & 7) * 2;
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int i = 32 * hh + e;
                    const float w = __uint_as_float(r[e]);
                    const __nv_bfloat16 whi = __float2bfloat16_rn(w);
                    const __nv_bfloat16 wlo = __float2bfloat16_rn(w - __bfloat162float(whi));
                    const int off = i * 128 + ((((d & 63) >> 3) ^ (i & 7)) << 4);
                    *reinterpret_cast<__nv_bfloat16*>(wh + off) = whi;
                    *reinterpret_cast<__nv_bfloat16*>(wh + 2 * (64 * 128) + off) = wlo;
                }
            }
            {   // U [64 rows][128 dv] fp32: a warp writes 128 contiguous bytes of a row per instruction
                uint32_t r[32];
                tmem_ld_32x32(tlane + kPColAcc2 + 32 * hh, r);
                tmem_ld_wait();
                float* up = reinterpret_cast<float*>(slot + SlotTC::kU) + (32 * hh) * D + d;
#pragma unroll
                for (int e = 0; e < 32; ++e) up[e * D] = __uint_as_float(r[e]);
            }
            __syncthreads();
            // staging -> scratch: W occupies rows 0..63 (even chunks) or 64..127 (odd chunks) of each k-atom of the W|Qg tiles
            const int wrow0 = c & 1u ? 64 : 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int e = tid + 256 * i;             // 16-byte chunk of the 32 KB
                const int seg = e >> 9, o = (e & 511) * 16;   // segment = part * 2 + k-atom, 8 KB each
                const uint4 v = *reinterpret_cast<const uint4*>(sX + seg * (64 * 128) + o);
                *reinterpret_cast<uint4*>(slot + SlotTC::kWQ + (seg >> 1) * SlotTC::kWQPart + (seg & 1) * SlotTC::kAtom128 + wrow0 * 128 + o) = v;
            }
        }
    }
    // ------------------------------------------------------------------------------ teardown
    tmem_ld_wait();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        __syncwarp();
        tmem_dealloc(tmem_base, kPrepTmemCols);
    }
}

int launch_chunked_tc(dc_ctx* ctx, cudaStream_t s, const ChunkArgs& a, uint32_t n_seq, uint32_t max_chunks) {
    static bool attr_set[16] = {};
    auto prep = a.praw ? delta_chunk_prepare_tc_kernel<true> : delta_chunk_prepare_tc_kernel<false>;
    auto apply = delta_chunk_apply_tc_kernel;
    if (!attr_set[ctx->device & 15]) {
        cudaError_t e = cudaFuncSetAttribute(delta_chunk_prepare_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(PrepTcSmem::kBytes));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(delta_chunk_prepare_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(PrepTcSmem::kBytes));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(apply, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(TcSmem::kBytes));
        if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "gated_delta: cannot opt in to %zu bytes of shared memory: %s", TcSmem::kBytes, cudaGetErrorString(e));
        attr_set[ctx->device & 15] = true;
    }
    prep<<<dim3(a.nv, max_chunks, n_seq), 256, PrepTcSmem::kBytes, s>>>(a, ctx->status_dev);
    int rc = dc_check_launch(ctx, "gated_delta (chunk prepare, tcgen05)");
    if (rc != DC_OK) return rc;
    apply<<<dim3(a.nv, n_seq), kTcThreads, TcSmem::kBytes, s>>>(a, ctx->status_dev);
    return dc_check_launch(ctx, "gated_delta (chunk apply, tcgen05)");
}

template <int SPLIT>
int launch_chunked(dc_ctx* ctx, cudaStream_t s, const ChunkArgs& a, uint32_t n_seq, uint32_t max_chunks) {
    static bool attr_set[16] = {};
    auto prep = delta_chunk_prepare_kernel<SPLIT>;
    if (!attr_set[ctx->device & 15]) {
        cudaError_t e = cudaFuncSetAttribute(prep, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kPrepSmem));
        if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "gated_delta: cannot opt in to %zu bytes of shared memory: %s", kPrepSmem, cudaGetErrorString(e));
        attr_set[ctx->device & 15] = true;
    }
    prep<<<dim3(max_chunks, a.nv, n_seq), 256, kPrepSmem, s>>>(a);
    int rc = dc_check_launch(ctx, "gated_delta (chunk prepare)");
    if (rc != DC_OK) return rc;
    // few (sequence, head) pairs: split the value columns over more CTAs
    if (static_cast<uint64_t>(n_seq) * a.nv >= static_cast<uint64_t>(ctx->sm_count)) return launch_apply<128, SPLIT>(ctx, s, a, n_seq);
    return launch_apply<32, SPLIT>(ctx, s, a, n_seq);
}

}  // namespace

// Opts every chunked delta-rule kernel in to its dynamic shared-memory size on the context's device, so that no
// forward has to (the first launch of each variant would do it otherwise).
int dc_delta_chunk_warm(dc_ctx* ctx) {
    static bool done[16] = {};
    if (done[ctx->device & 15]) return DC_OK;
    auto opt_in = [](auto kern, size_t bytes) { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)); };
    cudaError_t e = opt_in(delta_chunk_prepare_tc_kernel<true>, PrepTcSmem::kBytes);
    if (e == cudaSuccess) e = opt_in(delta_chunk_prepare_tc_kernel<false>, PrepTcSmem::kBytes);
    if (e == cudaSuccess) e = opt_in(delta_chunk_apply_tc_kernel, TcSmem::kBytes);
    if (e == cudaSuccess) e = opt_in(delta_chunk_prepare_kernel<1>, kPrepSmem);
    if (e == cudaSuccess) e = opt_in(delta_chunk_prepare_kernel<3>, kPrepSmem);
    if (e == cudaSuccess) e = opt_in(delta_chunk_apply_kernel<128, 1>, apply_smem<128, 1>());
    if (e == cudaSuccess) e = opt_in(delta_chunk_apply_kernel<32, 1>, apply_smem<32, 1>());
    if (e == cudaSuccess) e = opt_in(delta_chunk_apply_kernel<128, 3>, apply_smem<128, 3>());
    if (e == cudaSuccess) e = opt_in(delta_chunk_apply_kernel<32, 3>, apply_smem<32, 3>());
    if (e != cudaSuccess) return dc_fail(ctx, DC_CUDA_ERROR, "gated_delta: cannot opt in to the kernels' shared memory: %s", cudaGetErrorString(e));
    done[ctx->device & 15] = true;
    return DC_OK;
}

size_t dc_delta_chunk_scratch_bytes(uint32_t t, uint32_t n_seq, uint32_t nv) {
    return (static_cast<size_t>(t) / C + n_seq + 1) * nv * Slot<3>::kBytes;
}

int dc_gated_delta_chunked(dc_ctx* ctx, cudaStream_t s, const float* q, const float* k, const float* v, const float* a, const float* b,
                           const float* a_log, const float* dt_bias, const float* state_in, float* state_out, float* o, uint32_t t,
                           uint32_t ldab, uint32_t write_state, uint32_t nk, uint32_t nv, const uint32_t* seq_start, uint32_t n_seq,
                           uint32_t max_len, uint32_t split, const float* praw, uint32_t ldp, const float* conv_w, const float* conv_prev) {
    ChunkArgs args{q, k, v, a, b, a_log, dt_bias, state_in, state_out, o, nullptr, seq_start, t, ldab, nk, nv, write_state, praw, conv_w, conv_prev, ldp};
    if (praw && !(split == 3 && ctx->delta_engine == DC_ENGINE_TCGEN05))
        return dc_fail(ctx, DC_UNSUPPORTED, "conv_gated_delta: the fused form exists for the tcgen05 engine with split 3 only");
    const size_t bytes = dc_delta_chunk_scratch_bytes(t, n_seq, nv);
    void* ws = nullptr;
    if (int rc = dc_get_workspace(ctx, bytes, "gated_delta", &ws); rc != DC_OK) return rc;
    args.scratch = static_cast<uint8_t*>(ws);
    const uint32_t max_chunks = (max_len + C - 1) / C;
    if (split == 1) return launch_chunked<1>(ctx, s, args, n_seq, max_chunks);
    if (ctx->delta_engine == DC_ENGINE_TCGEN05) return launch_chunked_tc(ctx, s, args, n_seq, max_chunks);
    return launch_chunked<3>(ctx, s, args, n_seq, max_chunks);
}
