// Device helpers shared by the bitplane kernels: the operand layout and the register
// bit-matrix transpose that turns plane words into byte-packed codes.
//
// Operand layout (reference project paths): qweight int32 [P][N][K/32], plane 0 is the
// MSB of the parent code (any_precision/quantization/pack.py:90-96).  Inside a row,
// word t of a group of E words (E = 32 for every full 1024-weight group, E = (K%1024)/32
// for the last partial group) holds, in byte j counted from the most significant byte and
// bit e counted from that byte's most significant bit, the plane bit of weight
//     k = group_base + 8*E*j + 8*t + e                      (pack.py:12-76).
// The reference kernels read the same map back in matmul.cuh:86,95-125 and
// dequant.cuh:217,226-240.  This file restates that map; it shares no code with them.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace ap {

// One stage of the 8x8 bit-matrix transpose, applied to the four byte lanes of a word at
// once.  Rows a (index i, with i & D == 0) and b (index i + D) exchange their off-diagonal
// DxD blocks: columns with (c & D) != 0 of a swap with columns with (c & D) == 0 of b.
// Bitwise select: mask ? a : b.  Written as one LOP3 (truth table 0xE4 = (a & c) | (b & ~c)):
// left to itself the compiler spends two LOP3 on "(x & M) | (y & ~M)" with immediate masks.
template <uint32_t MASK>
__device__ __forceinline__ uint32_t bitsel(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xE4;" : "=r"(d) : "r"(a), "r"(b), "n"(MASK));
    return d;
}

template <int D>
__device__ __forceinline__ void swap_blocks(uint32_t& a, uint32_t& b) {
    constexpr uint32_t M = (D == 4) ? 0xF0F0F0F0u : (D == 2) ? 0xCCCCCCCCu : 0xAAAAAAAAu;
    const uint32_t na = bitsel<M>(b << D, a);       // (a & ~M) | ((b << D) & M)
    const uint32_t nb = bitsel<M>(b, a >> D);       // ((a >> D) & ~M) | (b & M)
    a = na;
    b = nb;
}

// planes[p], p = 0..W-1 (plane 0 = code MSB): one int32 word of each plane, same word
// position.  On return cw[e], e = 0..7, is a word whose byte (3 - j) is the W-bit code of
// the weight at (byte group j, bit e), shifted left by SHIFT: four codes per word.
// SHIFT > 0 (W + SHIFT <= 8) lets a code byte serve directly as a byte offset into a table
// of 2^SHIFT-byte entries.
template <int W, int SHIFT = 0>
__device__ __forceinline__ void transpose_codes(const uint32_t (&planes)[W], uint32_t (&cw)[8]) {
    static_assert(W + SHIFT <= 8, "code does not fit a byte");
    // Row i of the bit matrix carries bit i of the output byte, i.e. plane W-1-(i-SHIFT).
    uint32_t r[8];
#pragma unroll
    for (int i = 0; i < 8; i++) r[i] = (i >= SHIFT && i - SHIFT < W) ? planes[W - 1 - (i - SHIFT)] : 0u;
#pragma unroll
    for (int i = 0; i < 4; i++) swap_blocks<4>(r[i], r[i + 4]);
#pragma unroll
    for (int i = 0; i < 8; i++)
        if ((i & 2) == 0) swap_blocks<2>(r[i], r[i + 2]);
#pragma unroll
    for (int i = 0; i < 8; i++)
        if ((i & 1) == 0) swap_blocks<1>(r[i], r[i + 1]);
    // Row c now holds, in each byte, the code of the weight whose plane bit sat at bit c of
    // that byte, i.e. e = 7 - c.
#pragma unroll
    for (int e = 0; e < 8; e++) cw[e] = r[7 - e];
}

// For W <= 4: a 4x4 transpose inside every nibble instead of 8x8 inside every byte.  On
// return nb[c], c = 0..3, holds in byte (3 - j) two codes: the high nibble is the code of
// the weight at bit e = 3 - c of byte group j, the low nibble that of e = 7 - c.  The byte
// is therefore the index of the weight pair (e, e + 4) into a table of pairs.
template <int W>
__device__ __forceinline__ void transpose_nibbles(const uint32_t (&planes)[W], uint32_t (&nb)[4]) {
    static_assert(W <= 4, "nibble codes need W <= 4");
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; i++) r[i] = (i < W) ? planes[W - 1 - i] : 0u;
    swap_blocks<2>(r[0], r[2]);
    swap_blocks<2>(r[1], r[3]);
    swap_blocks<1>(r[0], r[1]);
    swap_blocks<1>(r[2], r[3]);
#pragma unroll
    for (int c = 0; c < 4; c++) nb[c] = r[c];
}

// For W <= 4, pairs of NEIGHBOURING weights: the plane index is exchanged with bits 2 and 1 of the bit position
// instead of bits 1 and 0.  On return pr[c], c = 0..3, holds in byte (3 - j) the codes of the weights e = 6 - 2c
// and e = 7 - 2c of byte group j, interleaved bit by bit: bit 2i + 1 of the byte is bit i of the code of the even
// weight (e = 6 - 2c), bit 2i that of the odd weight (e = 7 - 2c).  The byte is the index of that pair into a
// table of pairs, and the pair's activations are one 32-bit word of the activation row as it lies in memory.
template <int W>
__device__ __forceinline__ void transpose_pairs(const uint32_t (&planes)[W], uint32_t (&pr)[4]) {
    static_assert(W <= 4, "pair codes need W <= 4");
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; i++) r[i] = (i < W) ? planes[W - 1 - i] : 0u;
    swap_blocks<4>(r[0], r[2]);
    swap_blocks<4>(r[1], r[3]);
    swap_blocks<2>(r[0], r[1]);
    swap_blocks<2>(r[2], r[3]);
#pragma unroll
    for (int c = 0; c < 4; c++) pr[c] = r[c];
}

// Bit i of v moved to bit 2i (v below 16): the place of one code's bits inside the index byte of transpose_pairs.
__host__ __device__ constexpr uint32_t spread_bits(uint32_t v) {
    return (v & 1u) | ((v & 2u) << 1) | ((v & 4u) << 2) | ((v & 8u) << 3);
}

// Geometry of a row for kernels that read 16-byte vectors (4 consecutive words) of a
// row-plane.  Requires K % 128 == 0 so that rows and the partial group are whole vectors.
struct RowGeom {
    int vecs;        // K / 128: 16-byte vectors per row-plane
    int full_vecs;   // vectors inside full 1024-weight groups
    int tail_stride; // 8 * E of the partial group, in weights (0 if none)
};

__host__ __device__ inline RowGeom make_geom(int K) {
    RowGeom g;
    g.vecs = K / 128;
    g.full_vecs = (K / 1024) * 8;
    g.tail_stride = (K % 1024) / 4;
    return g;
}

// For vector u of a row: weights base + stride*j + 8*word + e, j = 0..3, word = 0..3, e = 0..7.
__device__ __forceinline__ void vec_span(const RowGeom& g, int u, int& base, int& stride) {
    if (u < g.full_vecs) {
        base = (u >> 3) * 1024 + (u & 7) * 32;
        stride = 256;
    } else {
        base = (g.full_vecs >> 3) * 1024 + (u - g.full_vecs) * 32;
        stride = g.tail_stride;
    }
}

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ldg_stream(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

}  // namespace ap
