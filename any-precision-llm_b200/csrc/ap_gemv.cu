// matmul_kbit (decode GEMV) for sm_100a:
//     y[m][n] = sum_k x[m][k] * lut[n][code_w(n,k)]
// with fp32 accumulation.  Replaces the reference's matmul_kbit host function and its
// matmul_kbit_32<maxm,bits,use_ksplit> kernels (any_precision/modules/kernels/main.cu:93-143,
// matmul.cuh:16-167), which accumulate in fp16 with one multiply-add per weight per batch row.
//
// This file holds
//   * the pieces every decode kernel shares: the lookup helpers (PRMT-built table addresses), the
//     mma.sync wrapper and process_word, which turns one plane word of two rows into eight MMAs;
//   * launch_gemv, which picks a kernel for a call;
//   * two fallback kernels: gemv_kbit_mma_kernel (per-lane cp.async ring; taken when the planes
//     cannot be described to the TMA unit, or with AP_GEMV_LOADER=cpasync) and
//     gemv_kbit_plain_kernel (one warp per row, fp32 multiply-adds; for K % 128 != 0, N % 16 != 0
//     or unaligned pointers).
// The kernel that runs by default, gemv_kbit_tma_kernel, is in ap_gemv_tma.cuh (included below).
//
// Common design.  A thread block owns 16 output rows and its eight warps split K.  Plane words
// are transposed into byte-packed codes in registers (ap_bitplane.cuh); a code byte and the
// lane's byte offset form a shared-memory address with one PRMT; for w <= 4 a byte holds the
// codes of TWO weights and indexes a table of fp16 pairs, halving the lookups.  The dot products
// run on the tensor pipe (mma.sync m16n8k16, fp32 accumulators) with the 16 rows on the M side
// and the batch (up to 8) on the N side, so batch 1..8 cost the same and no multiply-add is
// issued per weight.  What bounds the arithmetic on a B200 is instruction issue and the integer
// ALU pipe (bit transposes and address permutes), not shared-memory bandwidth and not HBM.
// The kernels are programmatic-dependent-launch secondaries: they request weights and build
// their tables before waiting for the previous kernel in the stream and read activations after.
#include "ap_bitplane.cuh"
#include "ap_kernels.h"

#include <stdlib.h>

namespace ap {

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    // Not volatile: the accumulator operands carry the only ordering that matters, and the
    // compiler is free to interleave table lookups of later tiles with earlier MMAs.
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Table reads.  Not volatile so that they can be scheduled freely; every address is derived
// from a base that is redefined after the barrier that publishes the table (see below).
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint32_t v;                                             // zero-extended by the load itself
    asm("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Address of table entry number (byte `b` of `word`) for entries of ENTRY bytes: one PRMT to
// isolate the byte (ALU pipe) and one integer multiply-add (FMA pipe), so that the two
// address instructions of a lookup do not queue on the same pipe.
template <int ENTRY>
__device__ __forceinline__ uint32_t entry_addr(uint32_t word, int b, uint32_t base) {
    uint32_t idx, addr;
    asm("prmt.b32 %0, %1, 0, %2;" : "=r"(idx) : "r"(word), "r"(0x4440u | (uint32_t)b));
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(addr) : "r"(idx), "n"(ENTRY), "r"(base));
    return addr;
}

// The same lookup address with no arithmetic: for a table whose entries of one code are 256 bytes
// apart, (code << 8) | lane_byte is one PRMT of the code word and a register holding the lane's byte
// offset (below 128, so its upper bytes are zero).  The table's own address is a link-time constant
// that the load takes as its immediate offset.
__device__ __forceinline__ uint32_t entry_offset_direct(uint32_t word, int b, uint32_t lane_byte) {
    uint32_t off;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(off) : "r"(word), "r"(lane_byte), "r"(0x7704u | ((uint32_t)b << 4)));
    return off;
}

template <int BYTES>
__device__ __forceinline__ void cp_async(uint32_t dst, const void* src) {
    if constexpr (BYTES == 16)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    else
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kGemvMaxWarps = 8;

#ifdef AP_GEMV_PROFILE
// Lab builds only: per-block stamps of the kernel's phases (never compiled into the library).
// A launch is told apart by its output pointer: launch l writes out_base + l * out_stride bytes.
constexpr int kProfLaunches = 16, kProfBlocks = 1024, kProfSlots = 16;
__device__ unsigned long long ap_gemv_prof[kProfLaunches * kProfBlocks * kProfSlots];
__device__ const char* ap_prof_out_base;
__device__ long long ap_prof_out_stride;
__device__ __forceinline__ unsigned long long* prof_init(const void* out) {
    if (threadIdx.x == 0 && blockIdx.x < kProfBlocks && blockIdx.y == 0 && ap_prof_out_stride > 0) {
        const long long l = (static_cast<const char*>(out) - ap_prof_out_base) / ap_prof_out_stride;
        if (l >= 0 && l < kProfLaunches) return ap_gemv_prof + (l * kProfBlocks + blockIdx.x) * kProfSlots;
    }
    return nullptr;
}
__device__ __forceinline__ void prof_mark(unsigned long long* p, int slot) {
    if (p) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); p[slot] = t; }
}
__device__ __forceinline__ void prof_clk(unsigned long long* p, int slot) {
    if (p) p[slot] = (unsigned long long)clock64();
}
#define AP_PROF_INIT unsigned long long* ap_prof_p = prof_init(out)
#define AP_PROF(slot) prof_mark(ap_prof_p, slot)
#define AP_CLK(slot) prof_clk(ap_prof_p, slot)
#else
#define AP_PROF_INIT
#define AP_PROF(slot)
#define AP_CLK(slot)
#endif

template <int W>
struct GemvCfg {
    static constexpr int C = 1 << W;
    static constexpr bool kRegLut = (W == 3);                // 8-entry tables live in registers (PRMT lookups)
    static constexpr int kVec = (W >= 6) ? 2 : 4;            // int32 words per lane, plane and step
    // Shared-memory table, w >= 4: [code][lane] of 32-bit entries (T[row g][code], T[row g+8][code]).
    // A lane only ever touches its own bank, so random codes cost one wavefront per lookup.
    static constexpr int kTableBytes = kRegLut ? 0 : C * 128;
    static constexpr int kRawStride = C + 8;                 // halfs; staged source rows, padded by 16 bytes
    static constexpr int kPlaneBytes = 32 * 2 * W * kVec * 4;  // one warp, one stage: the plane words
    // ... followed by the activations of the step as B fragments: 4*kVec items of 16 bytes for
    // each of 4 * mpad lanes (mpad = batch rounded up to 1, 2, 4 or 8)
    __host__ __device__ static constexpr int stage_bytes(int mpad) { return kPlaneBytes + 4 * kVec * 16 * 4 * mpad; }
    static constexpr int kRedBytes = kGemvMaxWarps * 128 * 4;
    __host__ __device__ static constexpr int total(int stages, int mpad) {
        return 128 + kTableBytes + kRedBytes + kGemvMaxWarps * stages * stage_bytes(mpad);
    }
    static_assert(kRegLut || 16 * kRawStride * 2 <= kTableBytes, "staged rows must fit inside the table region");
};

// One plane word of both rows (wa, wb: the word of every needed plane) against its 32 activations
// per row (xv[j]: the eight consecutive halfs of byte group j): decode, look up, 8 MMAs.
// MODE 0: w = 3 looks its register tables up with PRMT; w >= 4 reads a table of 128-byte code
//         stripes at address tab_a / tab_b (one multiply-add per lookup).
// MODE 1: the table has 256-byte code stripes at the constant shared address tab_const, and
//         tab_a / tab_b are the lane's byte offsets inside a stripe instead of addresses.
// MODE 2: w <= 4; the table is indexed by the codes of TWO weights and an entry is the fp16 pair itself: one
//         32-bit load per two weights and no packing.  Stripes and tab_const / tab_a / tab_b as in MODE 1.
//         Which two weights: see kNeighbourPairs.
// MODE 3: the pair table without a copy per lane (32-byte stripes; tab_const + pair_half is the rows g + 8's table).
// Pairs of neighbouring weights (transpose_pairs: the index byte interleaves the two codes, the activations are
// used as loaded, and at w = 3 the table has 64 stripes) or the two nibbles of a byte of transpose_nibbles (weights
// e and e + 4; the activations are re-paired with four permutes per byte group).  Measured per shape on a B200:
// neighbours win at w = 3 (2 % for one row, 20 % for eight rows on launches of many blocks, whose table halves)
// and with the compact table of mode 3 (up to 3 %); at w = 4 with the full table they win 3-4 % on 4096 x 4096
// and 4096 x 11008 but lose 3 % on 11008 x 4096 (11.9 -> 12.3 us), so that case has both (NB chosen per launch:
// nibbles for launches of many blocks).
template <int W, int MODE>
constexpr bool kNeighbourPairs = (MODE == 3) || (MODE == 2 && W == 3);

template <int W, int MODE = 0, bool NB = kNeighbourPairs<W, MODE>>
__device__ __forceinline__ void process_word(const uint32_t (&wa)[W], const uint32_t (&wb)[W], const uint4 (&xv)[4],
                                             float (&acc)[2][4], const uint32_t (&lut_lo)[2][2],
                                             const uint32_t (&lut_hi)[2][2], uint32_t tab_a, uint32_t tab_b,
                                             uint32_t tab_const = 0u, bool valid = true, uint32_t pair_half = 0u) {
    // `valid` false (a word past the end of a short last group): the weights are taken as zero
    // without looking anything up, so that no table entry, finite or not, meets the (zeroed) activations.
    using Cfg = GemvCfg<W>;
    if constexpr (MODE == 3) {
        // Compact pair tables: as mode 2, but an entry lives at index * 32 + g * 4 of its row set's table, i.e. the
        // permuted (index << 8 | g * 32) shifted right by three.
        uint32_t na[4], nb[4];
        transpose_pairs<W>(wa, na);
        transpose_pairs<W>(wb, nb);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t qa[4], qb[4];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                qa[c] = valid ? lds_u32(tab_const + (entry_offset_direct(na[c], 3 - j, tab_a) >> 3)) : 0u;
                qb[c] = valid ? lds_u32(tab_const + pair_half + (entry_offset_direct(nb[c], 3 - j, tab_b) >> 3)) : 0u;
            }
            mma16816(acc[0], qa[1], qb[1], qa[0], qb[0], xv[j].z, xv[j].w);
            mma16816(acc[1], qa[3], qb[3], qa[2], qb[2], xv[j].x, xv[j].y);
        }
    } else if constexpr (MODE == 2) {
        // Pair tables: byte (3 - j) of na[c] / nb[c] is the index of a weight pair of byte group j: the neighbours
        // (e = 6 - 2c, e = 7 - 2c), or (e = 3 - c, e = 7 - c) with the nibble transpose.  One byte group at a time:
        // eight lookups and two MMAs, so that only eight looked-up words are alive at once.
        uint32_t na[4], nb[4];
        if constexpr (NB) {
            transpose_pairs<W>(wa, na);
            transpose_pairs<W>(wb, nb);
        } else {
            transpose_nibbles<W>(wa, na);
            transpose_nibbles<W>(wb, nb);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t qa[4], qb[4];                           // fp16x2 weight pairs of rows g and g + 8
#pragma unroll
            for (int c = 0; c < 4; c++) {
                qa[c] = valid ? lds_u32(tab_const + entry_offset_direct(na[c], 3 - j, tab_a)) : 0u;
                qb[c] = valid ? lds_u32(tab_const + entry_offset_direct(nb[c], 3 - j, tab_b)) : 0u;
            }
            if constexpr (NB) {
                // the pair's activations (x[6-2c], x[7-2c]) are a word of the row as it was loaded; the two words of
                // an MMA in the order they were loaded in, which is the register pair the instruction wants
                mma16816(acc[0], qa[1], qb[1], qa[0], qb[0], xv[j].z, xv[j].w);
                mma16816(acc[1], qa[3], qb[3], qa[2], qb[2], xv[j].x, xv[j].y);
            } else {
                // activations paired like the weights: xq[c] = (x[7-c], x[3-c])
                uint32_t xq[4];
                xq[0] = __byte_perm(xv[j].w, xv[j].y, 0x7632);
                xq[1] = __byte_perm(xv[j].w, xv[j].y, 0x5410);
                xq[2] = __byte_perm(xv[j].z, xv[j].x, 0x7632);
                xq[3] = __byte_perm(xv[j].z, xv[j].x, 0x5410);
#pragma unroll
                for (int h = 0; h < 2; h++)
                    mma16816(acc[h], qa[2 * h], qb[2 * h], qa[2 * h + 1], qb[2 * h + 1], xq[2 * h], xq[2 * h + 1]);
            }
        }
    } else if constexpr (Cfg::kRegLut) {
        // w = 3 without pair tables: the row's eight table entries live in four registers and a byte permute with
        // the nibble codes as selectors is the lookup.
        uint32_t na[4], nb[4];
        transpose_nibbles<W>(wa, na);
        transpose_nibbles<W>(wb, nb);
        // wq[row][c][j]: fp16x2 (W[e = 7-c], W[e = 3-c]) of byte group j
        uint32_t wq[2][4][4];
#pragma unroll
        for (int c = 0; c < 4; c++) {
#pragma unroll
            for (int hs = 0; hs < 2; hs++) {     // selector half: nibbles of byte groups (3,2) then (1,0)
                const uint32_t sa = hs ? (na[c] >> 16) : na[c], sb = hs ? (nb[c] >> 16) : nb[c];
                const uint32_t alo = __byte_perm(lut_lo[0][0], lut_lo[0][1], sa);
                const uint32_t ahi = __byte_perm(lut_hi[0][0], lut_hi[0][1], sa);
                const uint32_t blo = __byte_perm(lut_lo[1][0], lut_lo[1][1], sb);
                const uint32_t bhi = __byte_perm(lut_hi[1][0], lut_hi[1][1], sb);
                wq[0][c][3 - 2 * hs] = __byte_perm(alo, ahi, 0x5140);
                wq[0][c][2 - 2 * hs] = __byte_perm(alo, ahi, 0x7362);
                wq[1][c][3 - 2 * hs] = __byte_perm(blo, bhi, 0x5140);
                wq[1][c][2 - 2 * hs] = __byte_perm(blo, bhi, 0x7362);
            }
            if (!valid) {
#pragma unroll
                for (int j = 0; j < 4; j++) wq[0][c][j] = wq[1][c][j] = 0u;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // activations paired the same way: xq[c] = (x[7-c], x[3-c])
            uint32_t xq[4];
            xq[0] = __byte_perm(xv[j].w, xv[j].y, 0x7632);
            xq[1] = __byte_perm(xv[j].w, xv[j].y, 0x5410);
            xq[2] = __byte_perm(xv[j].z, xv[j].x, 0x7632);
            xq[3] = __byte_perm(xv[j].z, xv[j].x, 0x5410);
#pragma unroll
            for (int h = 0; h < 2; h++)
                mma16816(acc[h], wq[0][2 * h][j], wq[1][2 * h][j], wq[0][2 * h + 1][j], wq[1][2 * h + 1][j],
                         xq[2 * h], xq[2 * h + 1]);
        }
    } else {
        uint32_t ca[8], cb[8];
        transpose_codes<W>(wa, ca);
        transpose_codes<W>(wb, cb);
#pragma unroll
        for (int j = 0; j < 4; j++) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint32_t va[4] = {0u, 0u, 0u, 0u}, vb[4] = {0u, 0u, 0u, 0u};
                if (valid) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        if constexpr (MODE == 1) {
                            va[e] = lds_u16(tab_const + entry_offset_direct(ca[4 * h + e], 3 - j, tab_a));
                            vb[e] = lds_u16(tab_const + entry_offset_direct(cb[4 * h + e], 3 - j, tab_b));
                        } else {
                            va[e] = lds_u16(entry_addr<128>(ca[4 * h + e], 3 - j, tab_a));
                            vb[e] = lds_u16(entry_addr<128>(cb[4 * h + e], 3 - j, tab_b));
                        }
                    }
                }
                const uint32_t a0 = __byte_perm(va[0], va[1], 0x5410), a2 = __byte_perm(va[2], va[3], 0x5410);
                const uint32_t a1 = __byte_perm(vb[0], vb[1], 0x5410), a3 = __byte_perm(vb[2], vb[3], 0x5410);
                const uint32_t b0 = h ? xv[j].z : xv[j].x;
                const uint32_t b1 = h ? xv[j].w : xv[j].y;
                mma16816(acc[h], a0, a1, a2, a3, b0, b1);
            }
        }
    }
}

template <int W>
__global__ void __launch_bounds__(kGemvMaxWarps * 32, 2)
gemv_kbit_mma_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ q, long long plane_stride,
                     const uint16_t* __restrict__ lut, __half* __restrict__ out, int M, int N, int K, int mpad,
                     int nstages, int split_words, float* __restrict__ partials, int* __restrict__ tickets) {
    using Cfg = GemvCfg<W>;
    constexpr int C = Cfg::C, VEC = Cfg::kVec;
    constexpr int kThreads = kGemvMaxWarps * 32;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((128u - (static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw)) & 127u)) & 127u);
    unsigned char* table = smem;
    float* red = reinterpret_cast<float*>(smem + Cfg::kTableBytes);
    unsigned char* ring = smem + Cfg::kTableBytes + Cfg::kRedBytes;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int nwarps = kGemvMaxWarps;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * 16;
    const int words = K >> 5;
    const int full_words = (K >> 10) << 5;                   // words inside full 1024-weight groups
    const int tail_stride = (K & 1023) >> 2;                 // 8 * E of the partial group
    // Split-K: blockIdx.y takes the words [w_begin, w_end) of every row (split_words is a multiple of 32,
    // so a split is whole 1024-weight groups); with one split this is the whole row.
    const int w_begin = blockIdx.y * split_words;
    const int w_end = (w_begin + split_words < words) ? (w_begin + split_words) : words;
    const int steps = (w_end - w_begin + 4 * VEC - 1) / (4 * VEC);     // a step: 4 lanes x VEC words of a row
    const uint32_t* qa = q + (size_t)(row0 + g) * words;
    const uint32_t* qb = q + (size_t)(row0 + g + 8) * words;

    // Batch column g of the MMA is row g of x.  Columns >= M are never stored, so their lanes
    // read the fragments of column g % mpad instead of being masked.
    const __half* xrow = x + (size_t)(g < M ? g : 0) * K;
    const bool copies_x = g < M;

    // This warp's ring: per stage [row a/b][plane][lane] x VEC words, then [item][x lane] x 16 bytes.
    const int stage_bytes = Cfg::stage_bytes(mpad);
    const uint32_t ring_sh = static_cast<uint32_t>(__cvta_generic_to_shared(ring)) + warp * nstages * stage_bytes;
    const uint32_t plane_lane = ring_sh + lane * (VEC * 4);
    const uint32_t x_lane = ring_sh + Cfg::kPlaneBytes + (((g & (mpad - 1)) << 2) + t) * 16;
    const int x_item_bytes = 64 * mpad;
    auto slot = [&](int stage, int ab, int p) -> uint32_t {
        return plane_lane + stage * stage_bytes + (ab * W + p) * (32 * VEC * 4);
    };
    // weights of word `word0 + wd`, byte group j, bit e:  k = kbase + 8*wd + kstride*j + e
    auto span = [&](int word0, int& kbase, int& kstride) {
        if (word0 >= w_end) { kbase = 0; kstride = 0; }          // out of range: never used, any address will do
        else if (word0 < full_words) { kbase = (word0 >> 5) * 1024 + (word0 & 31) * 8; kstride = 256; }
        else { kbase = full_words * 32 + (word0 - full_words) * 8; kstride = tail_stride; }
    };
    auto issue_planes = [&](int s, int stage) {
        const int word0 = w_begin + VEC * (4 * s + t);
        if (s < steps && word0 < w_end) {
#pragma unroll
            for (int p = 0; p < W; p++) {
                cp_async<VEC * 4>(slot(stage, 0, p), qa + (size_t)p * plane_stride + word0);
                cp_async<VEC * 4>(slot(stage, 1, p), qb + (size_t)p * plane_stride + word0);
            }
        }
    };
    auto issue_x = [&](int s, int stage) {
        if (s < steps && copies_x) {
            int kbase, kstride;
            span(w_begin + VEC * (4 * s + t), kbase, kstride);
#pragma unroll
            for (int wd = 0; wd < VEC; wd++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    cp_async<16>(x_lane + stage * stage_bytes + (wd * 4 + j) * x_item_bytes,
                                 xrow + kbase + 8 * wd + kstride * j);
        }
    };
    AP_PROF_INIT;
    AP_PROF(0);
    // Tables first: their source rows are requested before the (much larger) plane stream, so
    // that they do not queue behind it in the memory system.
    // w = 3: this lane's two rows' tables as byte planes in registers, (T0..T3, T4..T7) x (low, high byte)
    uint32_t lut_lo[2][2] = {{0u, 0u}, {0u, 0u}}, lut_hi[2][2] = {{0u, 0u}, {0u, 0u}};
    uint16_t* raw = reinterpret_cast<uint16_t*>(table);      // w >= 4: the 16 source rows, staged inside the table region
    if constexpr (Cfg::kRegLut) {
#pragma unroll
        for (int ab = 0; ab < 2; ab++) {
            const uint4 tv = __ldg(reinterpret_cast<const uint4*>(lut + (size_t)(row0 + g + 8 * ab) * C));
            lut_lo[ab][0] = __byte_perm(tv.x, tv.y, 0x6420);
            lut_lo[ab][1] = __byte_perm(tv.z, tv.w, 0x6420);
            lut_hi[ab][0] = __byte_perm(tv.x, tv.y, 0x7531);
            lut_hi[ab][1] = __byte_perm(tv.z, tv.w, 0x7531);
        }
    } else {
        const uint32_t raw_sh = static_cast<uint32_t>(__cvta_generic_to_shared(raw));
        const uint4* src = reinterpret_cast<const uint4*>(lut + (size_t)row0 * C);   // 16 rows, contiguous
        for (int i = tid; i < 16 * C / 8; i += kThreads) {
            const int r = (i * 8) / C, c0 = (i * 8) % C;
            cp_async<16>(raw_sh + (r * Cfg::kRawStride + c0) * 2, src + i);
        }
    }
    cp_async_commit();                                       // group: tables (empty for w = 3)
    AP_PROF(5);
    // Then the weights: they never depend on the previous kernel in the stream.  With a large
    // table (w >= 6) they are requested only after the table is built: a layer's worth of
    // per-lane copies backs up in the SM's load/store pipeline, and the shared-memory traffic of
    // the table build would sit behind it for microseconds.
    constexpr bool kTableFirst = (W >= 6);
    if constexpr (!kTableFirst) {
        issue_planes(warp, 0);
        cp_async_commit();                                   // group: planes of step 0
        if (nstages > 1) issue_planes(warp + nwarps, 1);
        cp_async_commit();                                   // group: planes of step 1 (possibly empty)
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    AP_PROF(6);

    if constexpr (!Cfg::kRegLut) {
        // Spread the staged rows into the [code][lane] table.  The staging area lies inside the
        // table region, so every thread first pulls its share into registers.
        constexpr int kItems = C * 8;                        // (4 consecutive codes) x (32 lanes)
        constexpr int kPerThread = (kItems + kThreads - 1) / kThreads;
        uint2 lo[kPerThread], hi[kPerThread];
        if constexpr (kTableFirst) cp_async_wait<0>(); else cp_async_wait<2>();   // this thread's pieces of the rows have landed
        __syncthreads();                                     // ... and everybody else's
        AP_PROF(7);
#pragma unroll
        for (int n = 0; n < kPerThread; n++) {
            const int i = tid + n * kThreads;
            if (i < kItems) {
                const int L = i & 31, cb = i >> 5, gg = L >> 2;
                lo[n] = *reinterpret_cast<const uint2*>(raw + gg * Cfg::kRawStride + 4 * cb);
                hi[n] = *reinterpret_cast<const uint2*>(raw + (gg + 8) * Cfg::kRawStride + 4 * cb);
            }
        }
        __syncthreads();
        uint32_t* tab = reinterpret_cast<uint32_t*>(table);
#pragma unroll
        for (int n = 0; n < kPerThread; n++) {
            const int i = tid + n * kThreads;
            if (i < kItems) {
                const int L = i & 31, cb = i >> 5;
                uint32_t* dst = tab + (4 * cb) * 32 + L;
                dst[0] = __byte_perm(lo[n].x, hi[n].x, 0x5410);
                dst[32] = __byte_perm(lo[n].x, hi[n].x, 0x7632);
                dst[64] = __byte_perm(lo[n].y, hi[n].y, 0x5410);
                dst[96] = __byte_perm(lo[n].y, hi[n].y, 0x7632);
            }
        }
        __syncthreads();
    }
    if constexpr (kTableFirst) {
        issue_planes(warp, 0);
        cp_async_commit();                                   // group: planes of step 0
        if (nstages > 1) issue_planes(warp + nwarps, 1);
        cp_async_commit();                                   // group: planes of step 1 (possibly empty)
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    AP_PROF(1);
    uint32_t table_sh = static_cast<uint32_t>(__cvta_generic_to_shared(table));
    asm volatile("" : "+r"(table_sh)::"memory");             // lookups may not move above the barrier
    const uint32_t tab_a = table_sh + lane * 4, tab_b = tab_a + 2;   // this lane's bank: row g, row g+8

    // Activations (and the output) may come from the previous kernel in the stream.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    issue_x(warp, 0);
    cp_async_commit();                                       // group: x of step 0
    if (nstages > 1) issue_x(warp + nwarps, 1);
    cp_async_commit();                                       // group: x of step 1 (possibly empty)
    // Everything a warp needs for its first two steps is requested up front (measured: requesting
    // one step ahead instead loses 10-25 %).  From here on at most one younger group (the next
    // step's) may be pending when a step starts.

    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};

    int stage = 0;
    for (int s = warp; s < steps; s += nwarps, stage = (nstages > 1) ? (stage ^ 1) : 0) {
        const int word0 = w_begin + VEC * (4 * s + t);
        const bool valid = word0 < w_end;                    // false only in the last, partial step of a row
        cp_async_wait<1>();                                  // this step's planes and x have landed
        if (s == warp) AP_PROF(2);
        const uint32_t xs = x_lane + stage * stage_bytes;

#pragma unroll
        for (int half = 0; half < VEC / 2; half++) {
            // two words of every plane, both rows
            uint32_t pa[W][2], pb[W][2];
#pragma unroll
            for (int p = 0; p < W; p++) {
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(pa[p][0]), "=r"(pa[p][1])
                             : "r"(slot(stage, 0, p) + half * 8));
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(pb[p][0]), "=r"(pb[p][1])
                             : "r"(slot(stage, 1, p) + half * 8));
            }
#pragma unroll
            for (int w2 = 0; w2 < 2; w2++) {
                const int wd = half * 2 + w2;
                uint32_t wa[W], wb[W];
#pragma unroll
                for (int p = 0; p < W; p++) { wa[p] = pa[p][w2]; wb[p] = pb[p][w2]; }
                // activations of this word: 4 runs (j) of 8 consecutive halfs, as staged by issue_x
                uint4 xv[4];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(xv[j].x), "=r"(xv[j].y), "=r"(xv[j].z), "=r"(xv[j].w)
                                 : "r"(xs + (wd * 4 + j) * x_item_bytes));
                if (!valid) {
                    // Lanes past the end of the row hold stale ring contents: zero activations
                    // against weights that process_word takes as zero without a lookup.
#pragma unroll
                    for (int p = 0; p < W; p++) wa[p] = wb[p] = 0u;
#pragma unroll
                    for (int j = 0; j < 4; j++) xv[j] = make_uint4(0u, 0u, 0u, 0u);
                }
                process_word<W>(wa, wb, xv, acc, lut_lo, lut_hi, tab_a, tab_b, 0u, valid);
            }
        }
        // the stage just consumed is free: refill it with the step after next
        if (nstages > 1) {
            issue_planes(s + 2 * nwarps, stage);
            issue_x(s + 2 * nwarps, stage);
        }
        cp_async_commit();
    }
    cp_async_wait<0>();
    AP_PROF(3);

    // Combine the warps' partial tiles: acc = {(g, 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)}.
    float* mine = red + warp * 128;
    mine[g * 8 + 2 * t] = acc[0][0] + acc[1][0];
    mine[g * 8 + 2 * t + 1] = acc[0][1] + acc[1][1];
    mine[(g + 8) * 8 + 2 * t] = acc[0][2] + acc[1][2];
    mine[(g + 8) * 8 + 2 * t + 1] = acc[0][3] + acc[1][3];
    __syncthreads();
    if (gridDim.y == 1) {
        for (int i = tid; i < 16 * M; i += kThreads) {
            const int m = i >> 4, r = i & 15;            // 16 consecutive rows per m: 32-byte stores
            float sum = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < nwarps; w2++) sum += red[w2 * 128 + r * 8 + m];
            out[(size_t)m * N + row0 + r] = __float2half_rn(sum);
        }
    } else {
        // Split-K: park this split's fp32 tile in the workspace; the CTA that draws the last ticket
        // for the tile adds the splits up in a fixed order (so the result does not depend on which
        // CTA that is), stores fp16 and hands the ticket counter back at zero.
        const int S = gridDim.y;
        for (int i = tid; i < 16 * M; i += kThreads) {
            const int m = i >> 4, r = i & 15;
            float sum = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < nwarps; w2++) sum += red[w2 * 128 + r * 8 + m];
            __stcg(partials + ((size_t)blockIdx.y * M + m) * N + row0 + r, sum);
        }
        __threadfence();
        __syncthreads();
        int* flag = reinterpret_cast<int*>(red);         // the reduction buffer is free again
        if (tid == 0) *flag = (atomicAdd(tickets + blockIdx.x, 1) == S - 1);
        __syncthreads();
        if (*flag) {
            __threadfence();
            for (int i = tid; i < 16 * M; i += kThreads) {
                const int m = i >> 4, r = i & 15;
                float sum = 0.f;
                for (int sp = 0; sp < S; sp++) sum += __ldcg(partials + ((size_t)sp * M + m) * N + row0 + r);
                out[(size_t)m * N + row0 + r] = __float2half_rn(sum);
            }
            if (tid == 0) tickets[blockIdx.x] = 0;
        }
    }
    AP_PROF(4);
}

}  // namespace ap

#include "ap_gemv_tma.cuh"

namespace ap {

// Plain kernel for shapes the fast kernel does not take: one warp per output row, one
// plane word per lane per group, fp32 multiply-adds.
template <int W>
__global__ void __launch_bounds__(128)
gemv_kbit_plain_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ q, long long plane_stride,
                       const uint16_t* __restrict__ lut, __half* __restrict__ out, int M, int N, int K) {
    constexpr int C = 1 << W;
    __shared__ uint16_t tab[4][C];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;
    if (row >= N) return;
    for (int c = lane; c < C; c += 32) tab[warp][c] = lut[(size_t)row * C + c];
    __syncwarp();
    const int words = K >> 5, full_groups = K >> 10, tail_e = (K & 1023) >> 5;
    const int groups = full_groups + (tail_e ? 1 : 0);
    float acc[8];
#pragma unroll
    for (int m = 0; m < 8; m++) acc[m] = 0.f;
    const uint32_t* qrow = q + (size_t)row * words;
    for (int gi = 0; gi < groups; gi++) {
        const int E = (gi < full_groups) ? 32 : tail_e;
        if (lane >= E) continue;
        uint32_t planes[W], cw[8];
#pragma unroll
        for (int p = 0; p < W; p++) planes[p] = qrow[(size_t)p * plane_stride + gi * 32 + lane];
        transpose_codes<W>(planes, cw);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k0 = gi * 1024 + 8 * E * j + 8 * lane;
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const __half_raw hr = {tab[warp][(cw[e] >> (8 * (3 - j))) & 0xffu]};
                const float wv = __half2float(__half(hr));
                for (int m = 0; m < M; m++) acc[m] += wv * __half2float(x[(size_t)m * K + k0 + e]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < 8; m++) {
        float s = acc[m];
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0 && m < M) out[(size_t)m * N + row] = __float2half_rn(s);
    }
}

template <int W>
static cudaError_t launch_w(const void* x, const void* q, long long plane_stride, const void* lut, void* out, int M,
                            int N, int K, bool fast, int splits, float* partials, int* tickets, cudaStream_t stream,
                            const GemvEpilogue* epi = nullptr) {
    auto xp = static_cast<const __half*>(x);
    auto qp = static_cast<const uint32_t*>(q);
    auto lp = static_cast<const uint16_t*>(lut);
    auto op = static_cast<__half*>(out);
    // Planes by tiled TMA unless AP_GEMV_LOADER=cpasync asks for the per-lane cp.async loader (or the
    // driver cannot encode the tensor map).
    static const bool want_tma = [] {
        const char* e = getenv("AP_GEMV_LOADER");
        return !(e && e[0] == 'c');
    }();
    if (epi) {
        // the decoder's epilogues: only the TMA kernel has them (decode batches, aligned operands)
        if (!fast || !want_tma || M > 8) return cudaErrorNotSupported;
        bool used = false;
        cudaError_t te = launch_tma<W>(xp, qp, plane_stride, lp, op, M, N, K, splits, partials, tickets, stream, &used, epi);
        return (used || te != cudaSuccess) ? te : cudaErrorNotSupported;
    }
    if (M > 8) {
        // Eight batch rows per pass.  The TMA kernel takes all passes in one launch (grid z) when K is not
        // split; everything else runs them one after the other.
        if (fast && want_tma && splits <= 1) {
            bool used = false;
            cudaError_t te = launch_tma<W>(xp, qp, plane_stride, lp, op, M, N, K, 1, nullptr, nullptr, stream, &used);
            if (used || te != cudaSuccess) return te;
        }
        for (int m0 = 0; m0 < M; m0 += 8) {
            const int mc = (M - m0 < 8) ? (M - m0) : 8;
            cudaError_t e = launch_w<W>(xp + (size_t)m0 * K, q, plane_stride, lut, op + (size_t)m0 * N, mc, N, K, fast, splits,
                                        partials, tickets, stream);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    if (!fast) {
        gemv_kbit_plain_kernel<W><<<(N + 3) / 4, 128, 0, stream>>>(xp, qp, plane_stride, lp, op, M, N, K);
        return cudaGetLastError();
    }
    if (want_tma) {
        bool used = false;
        cudaError_t te = launch_tma<W>(xp, qp, plane_stride, lp, op, M, N, K, splits, partials, tickets, stream, &used);
        if (used || te != cudaSuccess) return te;
    }
    const int warps = kGemvMaxWarps;
    // words per split: whole 1024-weight groups
    const int groups = (K + 1023) / 1024;
    if (splits > groups) splits = groups;
    if (splits < 1 || partials == nullptr || tickets == nullptr) splits = 1;
    const int split_words = ((groups + splits - 1) / splits) * 32;
    splits = (K / 32 + split_words - 1) / split_words;
    const int steps = (split_words + 4 * GemvCfg<W>::kVec - 1) / (4 * GemvCfg<W>::kVec);
    const int stages = (steps > warps) ? 2 : 1;
    const int mpad = (M <= 1) ? 1 : (M <= 2) ? 2 : (M <= 4) ? 4 : 8;
    const int smem = GemvCfg<W>::total(stages, mpad);
    // The dynamic shared memory limit is a per-device function attribute: raise it once per device.
    static bool attr_done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        e = cudaFuncSetAttribute(gemv_kbit_mma_kernel<W>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 GemvCfg<W>::total(2, 8));
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(N / 16, splits);
    cfg.blockDim = dim3(warps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemv_kbit_mma_kernel<W>, xp, qp, plane_stride, lp, op, M, N, K, mpad, stages,
                              split_words, partials, tickets);
}

cudaError_t take_gemv_wait_flag(int* flag) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    e = cudaMemcpyFromSymbol(flag, ap_gemv_wait_expired, sizeof(int));
    if (e != cudaSuccess || *flag == 0) return e;
    const int zero = 0;
    return cudaMemcpyToSymbol(ap_gemv_wait_expired, &zero, sizeof(int));
}

bool gemv_fast_path(const void* x, const void* qweight, long long plane_stride, const void* lut, int N, int K) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(qweight) |
                           reinterpret_cast<uintptr_t>(lut)) & 15) == 0;
    return aligned && (K % 128 == 0) && (N % 16 == 0) && (plane_stride % 4 == 0);
}

cudaError_t launch_gemv(const void* x, const void* qweight, long long plane_stride, const void* lut, void* out,
                        int M, int N, int K, int w_bits, int splits, float* partials, int* tickets,
                        cudaStream_t stream, const GemvEpilogue* epi) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(qweight) |
                           reinterpret_cast<uintptr_t>(lut)) & 15) == 0;
    const bool fast = aligned && (K % 128 == 0) && (N % 16 == 0) && (plane_stride % 4 == 0);
    switch (w_bits) {
        case 3: return launch_w<3>(x, qweight, plane_stride, lut, out, M, N, K, fast, splits, partials, tickets, stream, epi);
        case 4: return launch_w<4>(x, qweight, plane_stride, lut, out, M, N, K, fast, splits, partials, tickets, stream, epi);
        case 5: return launch_w<5>(x, qweight, plane_stride, lut, out, M, N, K, fast, splits, partials, tickets, stream, epi);
        case 6: return launch_w<6>(x, qweight, plane_stride, lut, out, M, N, K, fast, splits, partials, tickets, stream, epi);
        case 7: return launch_w<7>(x, qweight, plane_stride, lut, out, M, N, K, fast, splits, partials, tickets, stream, epi);
        case 8: return launch_w<8>(x, qweight, plane_stride, lut, out, M, N, K, fast, splits, partials, tickets, stream, epi);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ap
