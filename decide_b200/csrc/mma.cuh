// Warp-level building blocks for small matrix products on mma.sync m16n8k16 (bf16 in, fp32 out)
// over XOR-swizzled bf16 tiles in shared memory, with optional error-compensated operands.
//
// A product in "split 3" mode takes every fp32 operand as hi + lo, two bf16 values (16 mantissa bits
// together), and accumulates hi*hi + hi*lo + lo*hi in fp32: relative error ~2^-16 per element instead
// of bf16's 2^-9, at three MMAs per product. "split 1" uses hi*hi only.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>

namespace dc {

// Offset (in bf16 elements) of (row, col) in a [rows][C] tile whose 16-byte chunks are XOR-swizzled
// by the row so that ldmatrix reads of 8 consecutive rows hit 8 different bank groups.
template <int C>
__device__ __forceinline__ int tile_off(int row, int col) {
    static_assert(C == 32 || C == 64 || C == 128, "tile width");
    const int chunk = col >> 3;
    const int phys = (C == 32) ? (chunk ^ ((row >> 1) & 3)) : (chunk ^ (row & 7));
    return row * C + (phys << 3) + (col & 7);
}

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const __nv_bfloat16* p) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const __nv_bfloat16* p) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A fragment (16 rows x 16 k) of a row-major [m][k] tile.
template <int C>
__device__ __forceinline__ void lda(uint32_t (&a)[4], const __nv_bfloat16* t, int m0, int k0, int lane) {
    ldsm4(a, t + tile_off<C>(m0 + (lane & 7) + ((lane >> 3) & 1) * 8, k0 + (lane >> 4) * 8));
}
// A fragment of a tile stored transposed, [k][m] (m contiguous).
template <int C>
__device__ __forceinline__ void lda_t(uint32_t (&a)[4], const __nv_bfloat16* t, int k0, int m0, int lane) {
    const int j = lane >> 3;
    ldsm4t(a, t + tile_off<C>(k0 + (lane & 7) + (j >> 1) * 8, m0 + (j & 1) * 8));
}
// B fragments for two n-tiles (n0, n0+8) x 16 k of an operand stored [n][k] (k contiguous): b[0..1], b[2..3].
template <int C>
__device__ __forceinline__ void ldb_nt(uint32_t (&b)[4], const __nv_bfloat16* t, int n0, int k0, int lane) {
    ldsm4(b, t + tile_off<C>(n0 + (lane & 7) + (lane >> 4) * 8, k0 + ((lane >> 3) & 1) * 8));
}
// B fragments for two n-tiles of an operand stored [k][n] (n contiguous).
template <int C>
__device__ __forceinline__ void ldb_nn(uint32_t (&b)[4], const __nv_bfloat16* t, int k0, int n0, int lane) {
    ldsm4t(b, t + tile_off<C>(k0 + (lane & 7) + ((lane >> 3) & 1) * 8, n0 + (lane >> 4) * 8));
}

// acc += A * B for one 16x16 A fragment and two n-tiles, with operand splitting.
template <int SPLIT>
__device__ __forceinline__ void mma_split(float (&c0)[4], float (&c1)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4],
                                          const uint32_t (&bh)[4], const uint32_t (&bl)[4]) {
    if constexpr (SPLIT == 3) {
        mma16816(c0, al, bh[0], bh[1]);
        mma16816(c1, al, bh[2], bh[3]);
        mma16816(c0, ah, bl[0], bl[1]);
        mma16816(c1, ah, bl[2], bl[3]);
    }
    mma16816(c0, ah, bh[0], bh[1]);
    mma16816(c1, ah, bh[2], bh[3]);
}

// Writes the pair (x0, x1) at (row, col), col even, as hi (and lo) bf16x2 into swizzled tiles.
template <int C, int SPLIT>
__device__ __forceinline__ void put2(__nv_bfloat16* hi, __nv_bfloat16* lo, int row, int col, float x0, float x1) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
    const int off = tile_off<C>(row, col);
    *reinterpret_cast<__nv_bfloat162*>(hi + off) = h;
    if constexpr (SPLIT == 3) {
        const float2 hf = __bfloat1622float2(h);
        *reinterpret_cast<__nv_bfloat162*>(lo + off) = __floats2bfloat162_rn(x0 - hf.x, x1 - hf.y);
    }
}
// Four values at (row, col), col a multiple of 4: one 8-byte store per tile.
template <int C, int SPLIT>
__device__ __forceinline__ void put4(__nv_bfloat16* hi, __nv_bfloat16* lo, int row, int col, const float4& v) {
    const __nv_bfloat162 h0 = __floats2bfloat162_rn(v.x, v.y), h1 = __floats2bfloat162_rn(v.z, v.w);
    const int off = tile_off<C>(row, col);
    uint2 w;
    w.x = *reinterpret_cast<const uint32_t*>(&h0);
    w.y = *reinterpret_cast<const uint32_t*>(&h1);
    *reinterpret_cast<uint2*>(hi + off) = w;
    if constexpr (SPLIT == 3) {
        const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);
        const __nv_bfloat162 l0 = __floats2bfloat162_rn(v.x - f0.x, v.y - f0.y), l1 = __floats2bfloat162_rn(v.z - f1.x, v.w - f1.y);
        w.x = *reinterpret_cast<const uint32_t*>(&l0);
        w.y = *reinterpret_cast<const uint32_t*>(&l1);
        *reinterpret_cast<uint2*>(lo + off) = w;
    }
}

}  // namespace dc
