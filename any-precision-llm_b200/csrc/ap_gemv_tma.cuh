// Decode GEMV with the planes brought in by tiled TMA (cp.async.bulk.tensor) instead of per-lane
// cp.async.  Included by ap_gemv.cu, which provides GemvCfg, process_word, cp_async and AP_PROF.
//
// Why: per-lane copies go through the SM's load/store pipeline.  A layer's worth of them takes
// about 2 us to pass through it whether the data comes from HBM or from L2, nothing else that uses
// that pipeline (table build, table lookups) moves meanwhile, and a warp cannot start on its first
// step before it has issued the copies of all its steps.  The TMA engine takes one instruction per
// box and writes shared memory on its own.
//
// Geometry.  qweight is described to the TMA engine as a 3-D int32 tensor [planes][N][K/32].  A
// CTA owns 16 rows; a row is cut into chunks of 32 words (one 1024-weight group; the last group may
// be shorter, the box then reads zeros past the row end).  One box = [w planes][16 rows][32 words],
// 2 KB per plane, with the 128-byte swizzle (16-byte piece j of row r lands at piece j ^ (r & 7)),
// so that the eight rows a half-warp reads do not all sit in the same banks.  The chunk's
// activations follow in natural order (plain bulk copies, one per batch row).  Each buffer has a
// `full` mbarrier that counts the bytes in.  A chunk is four steps of 8 words; step s goes to warp
// s % 8; the warp that took a chunk's first step waits for the other three (an `empty` mbarrier per
// buffer, one arrival per warp) and re-arms the buffer with a later chunk.
// Waits are bounded: on expiry the warp records it in ap_gemv_wait_expired and stops working.
#pragma once

#include <cuda.h>

#include "ap_tensormap.h"

#include <new>

namespace ap {

constexpr int kTmaChunkWords = 32;
constexpr int kTmaRingCap = 4;                             // chunk buffers per block at most (deeper rings measured no faster)
constexpr int kTmaXPitch = 1024 * 2 + 16;                  // bytes per batch row of a chunk's activations
constexpr uint32_t kTmaSpinLimit = 1u << 17;

__device__ int ap_gemv_wait_expired = 0;

struct TrueType { static constexpr bool value = true; };
struct FalseType { static constexpr bool value = false; };

// OCC: thread blocks per SM the kernel variant is built for (2 or 3).  Three blocks need a
// register cap of 80, which costs instruction-level parallelism, and a smaller shared-memory
// footprint; that pays only when a launch has more blocks than two per SM can hold at once.
// MODE: 0 .. 3 and 5 as below; 2, 3 and 5 are possible for w <= 4 only, and at w = 4 the 64 KB table of modes 2 and 5
// leaves room for the activations of at most two batch rows per chunk, so larger batches use mode 3 there.
template <int W, int OCC, int MODE>
struct GemvTmaCfg {
    // Table modes (see process_word):
    //  2 (w = 3, 4): indexed by the codes of two weights (see kNeighbourPairs: one byte of transpose_nibbles at
    //    w = 4, of transpose_pairs at w = 3); a 256-byte stripe per index holds the fp16 pair of the lane's row g
    //    (bytes 0..127, lane * 4) and of its row g + 8 (bytes 128..255).  256 stripes at w = 4 (64 KB), 64 at
    //    w = 3 (16 KB).
    //  1 (w = 5..7): one code's entries are spread over a 256-byte stripe (the lanes use the first
    //    128 bytes), so that a lookup address is a byte permute of the code word and nothing else.
    //  0 (w = 8): that table would be 64 KB; it keeps 128-byte stripes and a multiply-add per lookup.
    //  3 (w = 3, 4): the pair table of mode 2 without a copy per lane: one 32-byte stripe per index holds the eight
    //    rows g (a second table 8 KB further the rows g + 8): 16 KB at w = 4 instead of 64.  The four lanes of a row
    //    now share four banks instead of owning one each (about two wavefronts per lookup) and an address costs a
    //    shift more; it is for batches whose activations do not fit beside the 64 KB table.
    //  5 (w = 4): mode 2 with pairs of neighbouring weights (kNb) instead of the nibble pairs.
    static constexpr int kMode = MODE == 5 ? 2 : MODE;
    static constexpr bool kNb = MODE == 5 || kNeighbourPairs<W, MODE>;
    static_assert(MODE == 0 || (MODE == 1 && W >= 4 && W <= 7) || ((MODE == 2 || MODE == 3) && W <= 4) || (MODE == 5 && W == 4),
                  "table mode does not fit w_bits");
    static constexpr int kPairHalf = (W == 4 ? 256 : 64) * 32;        // mode 3: bytes of the rows-g table
    static constexpr bool kDirect = kMode != 0;
    static constexpr int kEntryWords = kDirect ? 64 : 32;
    static constexpr int kTableBytes = kMode == 2 ? (W == 4 ? 65536 : 64 * 256)
                                       : kMode == 3 ? 2 * kPairHalf
                                                  : (kMode == 1 ? GemvCfg<W>::C * 256 : GemvCfg<W>::kTableBytes);
    static constexpr int kPlaneBytes = W * 16 * 128;         // one box
    __host__ __device__ static constexpr int buffer_bytes(int mpad) {
        return (kPlaneBytes + mpad * kTmaXPitch + 1023) & ~1023;
    }
    // Chunk buffers, 2..4: what fits beside the table when OCC blocks share an SM (about 74 KB
    // each for three, 110 KB each for two).
    __host__ __device__ static constexpr int buffers(int mpad) {
        const int fixed = 1024 + kTableBytes + GemvCfg<W>::kRedBytes + 256;
        const int n = ((OCC == 3 ? 74 : 110) * 1024 - fixed) / buffer_bytes(mpad);
        return n > kTmaRingCap ? kTmaRingCap : (n < 2 ? 2 : n);
    }
    __host__ __device__ static constexpr int total(int mpad) {
        return 1024 + buffers(mpad) * buffer_bytes(mpad) + kTableBytes + GemvCfg<W>::kRedBytes + 256;
    }
};

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kTmaSpinLimit; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void tensor_g2s_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}

// ---------------------------------------------------------------------------------------------- the decoder's epilogues
// Batch row `m`'s rsqrt(mean square + eps) from the per-tile sums of squares that the launch which wrote the
// residual stream left behind, added in a fixed order (lane-strided, then a shuffle tree).  Called by warp m.
__device__ __forceinline__ void dec_row_scale(const GemvEpilogue& epi, int m, int lane, float* rn_s) {
    float ss = 0.f;
    for (int i = lane; i < epi.ssq_blocks; i += 32) ss += __ldcg(epi.ssq_in + (size_t)m * epi.ssq_blocks + i);
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o2);
    if (lane == 0) rn_s[m] = rsqrtf(ss * epi.inv_width + epi.eps);
}

// What becomes of a finished 16-row tile in the decoder's variants.  The fp32 product of tile row r with batch
// row m is the sum of the eight warps' partial tiles in shared memory (`red`, S == 0) or of the S split-K
// partials in the workspace.  Modes:
//   1, 3  the 16 rows are eight gate rows followed by the eight up rows of the same features (a gated MLP's two
//         projections stacked tile by tile); the tile's output is the eight values silu(gate) * up, rounded like
//         the separate operations would be (both projections to fp16, the activation to fp16, then the product);
//   2, 3  the activations were a residual stream times the norm weights, NOT yet divided by its root mean
//         square: the products are scaled by rn_s[m] = rsqrt(mean square + eps) first (a matrix product commutes
//         with a scale per batch row);
//   4     residual update: resid[m][row] += fp16(product), and the output is the new residual times the next
//         norm's weight, with this tile's sum of squares of the new residual in ssq_out[m][tile];
//   5     the tile goes to the all-reduce inboxes of all ranks (tensor parallelism: a row-parallel layer's
//         partial result), nothing is stored locally.
// The mode is the kernel's template argument DEC (0 = the plain kernel): one instantiation per mode, because the
// main loop's machine code turned out to depend on what follows it (a common variant with the mode read at run
// time ran the same loop 0.3-1.4 us per launch slower).
template <int DEC>
__device__ __forceinline__ void dec_epilogue(const GemvEpilogue& epi, const float* red, const float* partials, int S, int M, int N,
                                          int row0, __half* out, int tid, const float* rn_s, float pre_h, float pre_w,
                                          uint32_t pre_seq) {
    constexpr int kThreads = kGemvMaxWarps * 32;
    auto total = [&](int m, int r) {
        float sum = 0.f;
        if (S == 0) {
#pragma unroll
            for (int w2 = 0; w2 < kGemvMaxWarps; w2++) sum += red[w2 * 128 + r * 8 + m];
        } else {
            for (int sp = 0; sp < S; sp++) sum += __ldcg(partials + ((size_t)sp * M + m) * N + row0 + r);
        }
        return sum;
    };
    if constexpr (DEC == 5) {
        // Two neighbouring rows' fp16 sums and the call's number make one 8-byte store, which arrives whole; element
        // e of the [M][N] result lives at byte (e / 2) * 8 of the sender's slot in the call's generation.
        const uint32_t seq = pre_seq + 1u;
        const unsigned long long slot = kCommHeaderBytes + ((unsigned long long)(seq & 1u) * kCommMaxWorld + epi.rank) * 2ull * epi.cap;
        for (int i = tid; i < 8 * M; i += kThreads) {
            const int m = i >> 3, r = 2 * (i & 7);
            const __half2 v = __floats2half2_rn(total(m, r), total(m, r + 1));
            const uint32_t word = *reinterpret_cast<const uint32_t*>(&v);
            const unsigned long long at = slot + (((unsigned long long)m * N + row0 + r) >> 1) * 8ull;
            for (int p = 0; p < epi.world; p++)
                asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(epi.peer[p] + at), "r"(word), "r"(seq) : "memory");
        }
        return;
    }
    constexpr int mode = DEC;
    if constexpr (mode == 1 || mode == 3) {
        for (int i = tid; i < 8 * M; i += kThreads) {
            const int m = i >> 3, r = i & 7;
            float gs = total(m, r), us = total(m, r + 8);
            if (mode == 3) { gs *= rn_s[m]; us *= rn_s[m]; }
            const float gf = __half2float(__float2half_rn(gs)), uf = __half2float(__float2half_rn(us));
            const float a = __half2float(__float2half_rn(gf / (1.f + __expf(-gf))));
            out[(size_t)m * (N >> 1) + (row0 >> 1) + r] = __float2half_rn(a * uf);
        }
    } else if constexpr (mode == 2) {
        for (int i = tid; i < 16 * M; i += kThreads) {
            const int m = i >> 4, r = i & 15;
            out[(size_t)m * N + row0 + r] = __float2half_rn(total(m, r) * rn_s[m]);
        }
    } else if (tid < 128) {                                  // mode 4; four whole warps: 16 lanes per batch row
        const int m = tid >> 4, r = tid & 15;
        float sq = 0.f;
        if (m < M) {
            const size_t at = (size_t)m * N + row0 + r;
            const float o = __half2float(__float2half_rn(total(m, r)));
            const __half hn = __float2half_rn(pre_h + o);    // the old residual and the norm weight were fetched early
            epi.resid[at] = hn;
            const float hf = __half2float(hn);
            out[at] = __float2half_rn(hf * pre_w);
            sq = hf * hf;
        }
#pragma unroll
        for (int o2 = 8; o2 > 0; o2 >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o2);
        if (m < M && r == 0) epi.ssq_out[(size_t)m * gridDim.x + blockIdx.x] = sq;
    }
}

template <int W, int OCC, int MODE, int DEC = 0, bool SPLIT = true, bool ONE = false>
__global__ void __launch_bounds__(kGemvMaxWarps * 32, OCC)
gemv_kbit_tma_kernel(const __grid_constant__ CUtensorMap qmap, const __half* __restrict__ x,
                     const uint16_t* __restrict__ lut, __half* __restrict__ out, int M_, int N, int K, int mpad_,
                     int split_chunks, float* __restrict__ partials, int* __restrict__ tickets,
                     const __grid_constant__ GemvEpilogue epi) {
    using Cfg = GemvCfg<W>;
    using T = GemvTmaCfg<W, OCC, MODE>;
    constexpr int C = Cfg::C;
    constexpr int kThreads = kGemvMaxWarps * 32;
    // ONE: the instantiation for a single activation row (the ring's depth and strides are then constants).  It
    // exists for the precisions where it measured faster (w = 4, 7, 8: +3 to +4 %; w = 5, 6 lost 4 to 5 %).
    int M = ONE ? 1 : M_;
    const int mpad = ONE ? 1 : mpad_;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // The table sits at the start of the dynamic area, so that its shared address is a constant.
    unsigned char* table = smem_raw;
    const uint32_t after_table = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw)) + (uint32_t)T::kTableBytes;
    unsigned char* smem = smem_raw + T::kTableBytes + ((1024u - (after_table & 1023u)) & 1023u);
    const int nbuf = T::buffers(mpad);
    const int buf_bytes = T::buffer_bytes(mpad);
    unsigned char* bufs = smem;                                           // 1024-byte aligned boxes
    float* red = reinterpret_cast<float*>(smem + nbuf * buf_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(red) + Cfg::kRedBytes);   // full[nbuf][2]
    // then empty[nbuf]: one arrival per warp that has finished its step of the buffer's chunk; the barriers take 96 of
    // the 256 bytes kept for them, and the decoder variants keep eight floats at byte 128 (rsqrt(mean square + eps)
    // per batch row)
    float* rn_s = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + 128);

    // More than eight batch rows (no split-K then): blockIdx.z takes rows [8 z, 8 z + 8) of x and out, so
    // that the passes over the planes run side by side in one launch and the later ones read them from L2.
    {
        const int mz = blockIdx.z * 8;
        x += (size_t)mz * K;
        out += (size_t)mz * N;
        M = (M - mz < 8) ? (M - mz) : 8;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * 16;
    const int words = K >> 5;
    const int all_chunks = (words + kTmaChunkWords - 1) / kTmaChunkWords;
    // Split-K: blockIdx.y takes chunks [c_begin, c_end) of every row.
    const int c_begin = blockIdx.y * split_chunks;
    const int c_end = (c_begin + split_chunks < all_chunks) ? (c_begin + split_chunks) : all_chunks;
    const int nchunks = c_end - c_begin;
    const uint32_t bufs_sh = static_cast<uint32_t>(__cvta_generic_to_shared(bufs));
    const uint32_t bar_sh = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
    // words of chunk number c of the row (32, less for a short last group)
    auto chunk_words = [&](int c) { return (c == all_chunks - 1) ? (words - c * kTmaChunkWords) : kTmaChunkWords; };

    // Barrier of local chunk i.  A parity wait only tells "the phase of that parity is over", so a
    // warp may wait for a phase only if it has seen the one before it end.  Chunks alternate between
    // two sets of four warps, and with an odd number of buffers so do the uses of one buffer; blocks
    // of planes may also land out of order.  Hence two barriers per buffer, taken in turn by its
    // uses: a barrier's phases are then all waited for by the same four warps, in order.
    // (buffer b = i % nbuf in its use number rnd = i / nbuf; the main loop carries b and rnd along instead of
    // dividing)
    auto bar_at = [&](int b, int rnd) { return bar_sh + 8u * (uint32_t)(2 * b + (rnd & 1)); };
    // Request local chunk i (row chunk c_begin + i) into its buffer b in its use rnd.  Called by a whole warp.
    auto request_planes = [&](int i, int b, int rnd) {
        if (lane == 0) {
            const uint32_t bar = bar_at(b, rnd);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)T::kPlaneBytes) : "memory");
            tensor_g2s_3d(bufs_sh + b * buf_bytes, &qmap, (c_begin + i) * kTmaChunkWords, row0, 0, bar);
        }
        __syncwarp();
    };
    auto request_x = [&](int i, int b, int rnd) {
        const int c = c_begin + i;
        const uint32_t bytes = (uint32_t)chunk_words(c) * 64u;            // 32 weights per word, 2 bytes each
        const uint32_t bar = bar_at(b, rnd);
        if (lane == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes * (uint32_t)M) : "memory");
        __syncwarp();
        if (lane < M)
            bulk_g2s(bufs_sh + b * buf_bytes + T::kPlaneBytes + lane * kTmaXPitch, x + (size_t)lane * K + (size_t)c * 1024, bytes, bar);
        __syncwarp();
    };

    AP_PROF_INIT;
    AP_PROF(0);
    if (tid == 0) {
        for (int b = 0; b < nbuf; b++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_sh + 16u * b), "r"(2u) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_sh + 16u * b + 8u), "r"(2u) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_sh + 16u * kTmaRingCap + 8u * b), "r"(4u) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&qmap)) : "memory");
    }
    // Tables: w = 3 straight into registers, otherwise staged with ordinary cp.async (small).
    uint32_t lut_lo[2][2] = {{0u, 0u}, {0u, 0u}}, lut_hi[2][2] = {{0u, 0u}, {0u, 0u}};
    uint16_t* raw = reinterpret_cast<uint16_t*>(table);
    if constexpr (Cfg::kRegLut && T::kMode != 2 && T::kMode != 3) {
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
        const uint4* src = reinterpret_cast<const uint4*>(lut + (size_t)row0 * C);
        for (int i = tid; i < 16 * C / 8; i += kThreads) {
            const int r = (i * 8) / C, c0 = (i * 8) % C;
            cp_async<16>(raw_sh + (r * Cfg::kRawStride + c0) * 2, src + i);
        }
        cp_async_commit();
    }
    __syncthreads();                                         // barriers initialised
    const int first = nchunks < nbuf ? nchunks : nbuf;
    if (warp == 0) {
        for (int i = 0; i < first; i++) request_planes(i, i, 0);   // weights never depend on the previous kernel
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    AP_PROF(6);

    if constexpr (T::kMode == 2) {
        // Pair table.  The four lanes t = 0..3 of a row pair (g, g + 8) hold the same entries, side by
        // side: one 16-byte store writes all four.  A thread serves row (g or g + 8, by `half`) and a
        // few (low code, high code) pairs; the entry is fp16 T[lo] in the low half, T[hi] in the high.
        cp_async_wait<0>();
        __syncthreads();
        const int bg = lane & 7, half = (lane >> 3) & 1, sub = lane >> 4;
        const uint16_t* row = raw + (bg + 8 * half) * Cfg::kRawStride;
        constexpr int kHi = (C == 16) ? 16 : 4;              // high codes per thread
        const int lo = (C == 16) ? (warp + 8 * sub) : warp;
        const int hi0 = (C == 16) ? 0 : 4 * sub;
        const uint32_t tlo = row[lo];
        uint32_t thi[kHi / 2];
#pragma unroll
        for (int i = 0; i < kHi / 2; i++) thi[i] = *reinterpret_cast<const uint32_t*>(row + hi0 + 2 * i);
        __syncthreads();                                     // the staged rows lie inside the table region
        // index byte: hi << 4 | lo for the nibble pairs; for neighbouring pairs the bits of the low half's code at
        // the odd places and those of the high half's at the even ones
        constexpr bool kNb = T::kNb;
        const uint32_t first = kNb ? ((spread_bits((uint32_t)lo) << 1) | spread_bits((uint32_t)hi0)) : (uint32_t)(lo + 16 * hi0);
        const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(table)) + first * 256 + half * 128 + bg * 16;
#pragma unroll
        for (int i = 0; i < kHi; i++) {
            const uint32_t v = __byte_perm(tlo, thi[i >> 1], (i & 1) ? 0x7610u : 0x5410u);
            const uint32_t step = (kNb ? spread_bits((uint32_t)i) : 16u * (uint32_t)i) * 256u;
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst + step), "r"(v) : "memory");
        }
        __syncthreads();
    } else if constexpr (T::kMode == 3) {
        // Compact pair table: entry (lo, hi, row r) = fp16 T[r][lo] in the low half, T[r][hi] in the high half, at
        // index * 32 + (r & 7) * 4 of the table of its row set (rows 0..7, rows 8..15); the index has the bits of lo
        // at its odd places and those of hi at its even places (transpose_pairs).  Thread tid serves row tid & 15
        // and the pairs number (tid >> 4) + 16 n: with 16 codes lo is fixed per thread and hi = n.
        static_assert(kThreads == 256, "the pair numbering below assumes 256 threads");
        constexpr int kEntries = C * C * 16;
        constexpr int kPerThread = (kEntries + kThreads - 1) / kThreads;
        uint32_t val[kPerThread];
        cp_async_wait<0>();
        __syncthreads();
        const int r = tid & 15, t4 = tid >> 4;
#pragma unroll
        for (int n = 0; n < kPerThread; n++) {
            const int lo = (C == 16) ? t4 : (t4 + 16 * n) % C, hi = (C == 16) ? n : (t4 + 16 * n) / C;
            if (C == 16 || hi < C)
                val[n] = (uint32_t)raw[r * Cfg::kRawStride + lo] | ((uint32_t)raw[r * Cfg::kRawStride + hi] << 16);
        }
        __syncthreads();                                     // the staged rows lie inside the table region
        const uint32_t tab_sh = static_cast<uint32_t>(__cvta_generic_to_shared(table)) + (r >> 3) * T::kPairHalf + (r & 7) * 4;
#pragma unroll
        for (int n = 0; n < kPerThread; n++) {
            const int lo = (C == 16) ? t4 : (t4 + 16 * n) % C, hi = (C == 16) ? n : (t4 + 16 * n) / C;
            if (C == 16 || hi < C) {
                const uint32_t dst = tab_sh + ((spread_bits((uint32_t)lo) << 1) | spread_bits((uint32_t)hi)) * 32;
                asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst), "r"(val[n]) : "memory");
            }
        }
        __syncthreads();
    } else if constexpr (!Cfg::kRegLut) {
        // Spread the staged rows into the [code][lane] table (the staging area lies inside the table
        // region).  An entry is (T[row g][code], T[row g + 8][code]); the four lanes t = 0..3 of a row
        // pair hold the same entries side by side, so one 16-byte store writes all four.
        constexpr int kItems = C * 2;                        // (block of four codes, g)
        constexpr int kPerThread = (kItems + kThreads - 1) / kThreads;
        uint2 lo[kPerThread], hi[kPerThread];
        cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for (int n = 0; n < kPerThread; n++) {
            const int i = tid + n * kThreads;
            if (i < kItems) {
                const int gg = i & 7, cb = i >> 3;
                lo[n] = *reinterpret_cast<const uint2*>(raw + gg * Cfg::kRawStride + 4 * cb);
                hi[n] = *reinterpret_cast<const uint2*>(raw + (gg + 8) * Cfg::kRawStride + 4 * cb);
            }
        }
        __syncthreads();
        const uint32_t tab_sh = static_cast<uint32_t>(__cvta_generic_to_shared(table));
#pragma unroll
        for (int n = 0; n < kPerThread; n++) {
            const int i = tid + n * kThreads;
            if (i < kItems) {
                const int gg = i & 7, cb = i >> 3;
                constexpr int EB = T::kEntryWords * 4;           // bytes between consecutive codes
                const uint32_t dst = tab_sh + (4 * cb) * EB + gg * 16;
                const uint32_t v0 = __byte_perm(lo[n].x, hi[n].x, 0x5410), v1 = __byte_perm(lo[n].x, hi[n].x, 0x7632);
                const uint32_t v2 = __byte_perm(lo[n].y, hi[n].y, 0x5410), v3 = __byte_perm(lo[n].y, hi[n].y, 0x7632);
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(v0) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst + EB), "r"(v1) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst + 2 * EB), "r"(v2) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst + 3 * EB), "r"(v3) : "memory");
            }
        }
        __syncthreads();
    }
    AP_PROF(1);
    // Lookups may not move above the barrier that published the table: every lookup address is
    // derived from a register that is redefined here.
    const uint32_t table_const = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
    uint32_t tab_a, tab_b;
    if constexpr (T::kDirect) {
        tab_a = T::kMode == 3 ? (lane >> 2) * 32 : lane * 4;
        asm volatile("" : "+r"(tab_a)::"memory");
        tab_b = T::kMode == 3 ? tab_a : tab_a + (T::kMode == 2 ? 128 : 2);
    } else {
        uint32_t table_sh = table_const;
        asm volatile("" : "+r"(table_sh)::"memory");
        tab_a = table_sh + lane * 4;
        tab_b = tab_a + 2;
    }

    // Activations (and the output) may come from the previous kernel in the stream.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    AP_PROF(7);
    if (warp == 0) {
        for (int i = 0; i < first; i++) request_x(i, i, 0);
    }
    if constexpr (DEC == 2 || DEC == 3) {
        // by the warps that do not issue the copies, while the first chunks travel
        if (kGemvMaxWarps - 1 - warp < M) dec_row_scale(epi, kGemvMaxWarps - 1 - warp, lane, rn_s);
    }

    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const int total_steps = nchunks * 4;
    const uint32_t x_lane = T::kPlaneBytes + (g & (mpad - 1)) * kTmaXPitch;
    // this lane's 8 bytes inside a 128-byte box row: piece 2*sl + (t >> 1), swizzled with the row
    const uint32_t row_a = (uint32_t)g * 128u, row_b = (uint32_t)(g + 8) * 128u;
    bool ok = true;

    // this warp's steps are two chunks apart: its buffer index and the buffer's use number move along with it
    int b = warp >> 2, rnd = 0;                              // nbuf >= 2, so chunk 0 or 1 is buffer 0 or 1, first use
    for (int s = warp; s < total_steps && ok; s += kGemvMaxWarps) {
        const int i = s >> 2, sl = s & 3;
        const int cw_words = chunk_words(c_begin + i);
        const int wic = 8 * sl + 2 * t;                      // this lane's first word inside the chunk
        const bool valid = wic < cw_words;
        const uint32_t buf = bufs_sh + b * buf_bytes;
        // Every step waits for its chunk, even an empty one of a short last chunk: its "done" below
        // must not be counted while the buffer still holds an earlier chunk.
        ok = mbar_wait_bounded(bar_at(b, rnd), (uint32_t)(rnd >> 1) & 1u);
        if (s == warp) AP_PROF(2);
        if (ok && 8 * sl < cw_words) {                       // the step has at least one word (warp-uniform)
            const uint32_t piece = ((uint32_t)(2 * sl + (t >> 1)) ^ (uint32_t)(g & 7)) << 4;
            const uint32_t off = piece + (uint32_t)(t & 1) * 8u;
            uint32_t pa[W][2], pb[W][2];
#pragma unroll
            for (int p = 0; p < W; p++) {
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(pa[p][0]), "=r"(pa[p][1])
                             : "r"(buf + p * 2048 + row_a + off));
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(pb[p][0]), "=r"(pb[p][1])
                             : "r"(buf + p * 2048 + row_b + off));
            }
            // run j of word wd inside the chunk's activations: element 8*(wic + wd) + 8*cw_words*j
            const uint32_t xw = buf + x_lane + (uint32_t)wic * 16u;
            const uint32_t xj = (uint32_t)cw_words * 16u;
            // A step is either whole (all of its eight words lie inside the row: every step of every
            // full 1024-weight group, and most steps of a short last group) or cut (K / 32 % 8 == 4: the
            // lanes t >= 2 of the last step have no words).  The whole case is compiled with the mask
            // as a constant, so that the common path carries no selects or branches for it.
            auto two_words = [&](auto whole) {
                constexpr bool kWhole = decltype(whole)::value;
                const bool valid_w = kWhole || valid;
#pragma unroll
                for (int wd = 0; wd < 2; wd++) {
                    uint32_t wa[W], wb[W];
#pragma unroll
                    for (int p = 0; p < W; p++) { wa[p] = pa[p][wd]; wb[p] = pb[p][wd]; }
                    // Only the lanes of batch columns that exist (g < mpad) load activations.  The other lanes feed the
                    // MMA whatever their registers hold: a column of the product depends on its own column of
                    // activations only, and the columns past the batch are never stored.  (Zeroing the sixteen
                    // registers per word instead cost 1.6 % of the bench.)
                    uint4 xv[4];
#pragma unroll
                    for (int j = 0; j < 4; j++)               // no instruction: whatever the registers hold (columns never stored)
                        asm("" : "=r"(xv[j].x), "=r"(xv[j].y), "=r"(xv[j].z), "=r"(xv[j].w));
                    if (g < mpad) {
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(xv[j].x), "=r"(xv[j].y), "=r"(xv[j].z), "=r"(xv[j].w)
                                         : "r"(xw + wd * 16 + j * xj));
                    }
                    if (!valid_w) {
                        // Words past the end of the row: the box holds zeros there, the activation
                        // area holds leftovers.  Zero activations against weights that process_word
                        // takes as zero without a lookup.
#pragma unroll
                        for (int p = 0; p < W; p++) wa[p] = wb[p] = 0u;
#pragma unroll
                        for (int j = 0; j < 4; j++) xv[j] = make_uint4(0u, 0u, 0u, 0u);
                    }
#ifdef AP_GEMV_LAB_NO_WORD_MATH
                    // lab builds only: everything but the per-word arithmetic (loads, waits, hand-back, reduction)
                    acc[0][0] += __uint_as_float((wa[0] ^ wb[W - 1] ^ xv[0].x ^ xv[3].w) & 0x3fffffffu);
#else
                    process_word<W, T::kMode, T::kNb>(wa, wb, xv, acc, lut_lo, lut_hi, tab_a, tab_b, table_const, valid_w, T::kPairHalf);
#endif
                }
            };
            if (8 * sl + 8 <= cw_words) two_words(TrueType{});
            else two_words(FalseType{});
        }
        // This warp is done with the buffer (its plane words and activations are in registers or
        // consumed): it says so on the buffer's `empty` barrier and moves on.  The warp that took the
        // chunk's first step waits for all four and re-arms the buffer with a later chunk; the other
        // three never wait for one another.
        __syncwarp();
        const uint32_t empty = bar_sh + 16u * kTmaRingCap + 8u * (uint32_t)b;
        if (lane == 0) asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(empty) : "memory");
        const int inext = i + nbuf;
        if (sl == 0 && ok && inext < nchunks) {
            ok = mbar_wait_bounded(empty, (uint32_t)rnd & 1u);
            if (ok) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                request_planes(inext, b, rnd + 1);
                request_x(inext, b, rnd + 1);
            }
        }
        b += 2;                                              // kGemvMaxWarps / 4 chunks further
        if (b >= nbuf) { b -= nbuf; rnd++; }
    }
    if (!ok && lane == 0) atomicExch(&ap_gemv_wait_expired, 1);
    AP_PROF(3);

    // Mode 4 of the decoder variants: this thread's old residual and norm weight, requested before the reduction
    // below so that their round trip hides behind it.
    float pre_h = 0.f, pre_w = 0.f;
    uint32_t pre_seq = 0u;
    if constexpr (DEC == 4) {
        if (tid < 16 * M) {
            pre_h = __half2float(epi.resid[(size_t)(tid >> 4) * N + row0 + (tid & 15)]);
            pre_w = __half2float(epi.norm_w[row0 + (tid & 15)]);
        }
    }
    // push variant: the number of all-reduce calls completed so far, from this rank's communication buffer (written
    // by the previous call's last block, which this launch's dependency wait has seen end)
    if constexpr (DEC == 5) pre_seq = __ldcg(reinterpret_cast<const uint32_t*>(epi.peer[epi.rank]));
    // Combine the warps' partial tiles: acc = {(g, 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)}.
    float* mine = red + warp * 128;
    mine[g * 8 + 2 * t] = acc[0][0] + acc[1][0];
    mine[g * 8 + 2 * t + 1] = acc[0][1] + acc[1][1];
    mine[(g + 8) * 8 + 2 * t] = acc[0][2] + acc[1][2];
    mine[(g + 8) * 8 + 2 * t + 1] = acc[0][3] + acc[1][3];
    __syncthreads();
    // What becomes of a finished 16-row tile: plain kernels round the fp32 products to fp16 and store them; the
    // decoder's variants (DEC) hand them to dec_epilogue.
    if (!SPLIT || gridDim.y == 1) {
        if constexpr (DEC) {
            dec_epilogue<DEC>(epi, red, nullptr, 0, M, N, row0, out, tid, rn_s, pre_h, pre_w, pre_seq);
        } else {
            for (int i = tid; i < 16 * M; i += kThreads) {
                const int m = i >> 4, r = i & 15;            // 16 consecutive rows per m: 32-byte stores
                float sum = 0.f;
#pragma unroll
                for (int w2 = 0; w2 < kGemvMaxWarps; w2++) sum += red[w2 * 128 + r * 8 + m];
                out[(size_t)m * N + row0 + r] = __float2half_rn(sum);
            }
        }
    } else {
        // Split-K: park this split's fp32 tile in the workspace; the CTA that draws the last ticket
        // for the tile adds the splits up in a fixed order, stores fp16 and zeroes the ticket counter.
        const int S = gridDim.y;
        for (int i = tid; i < 16 * M; i += kThreads) {
            const int m = i >> 4, r = i & 15;
            float sum = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < kGemvMaxWarps; w2++) sum += red[w2 * 128 + r * 8 + m];
            __stcg(partials + ((size_t)blockIdx.y * M + m) * N + row0 + r, sum);
        }
        __threadfence();
        __syncthreads();
        int* flag = reinterpret_cast<int*>(red);
        if (tid == 0) *flag = (atomicAdd(tickets + blockIdx.x, 1) == S - 1);
        __syncthreads();
        if (*flag) {
            __threadfence();
            if constexpr (DEC) {
                dec_epilogue<DEC>(epi, nullptr, partials, S, M, N, row0, out, tid, rn_s, pre_h, pre_w, pre_seq);
            } else {
                for (int i = tid; i < 16 * M; i += kThreads) {
                    const int m = i >> 4, r = i & 15;
                    float sum = 0.f;
                    for (int sp = 0; sp < S; sp++) sum += __ldcg(partials + ((size_t)sp * M + m) * N + row0 + r);
                    out[(size_t)m * N + row0 + r] = __float2half_rn(sum);
                }
            }
            if (tid == 0) tickets[blockIdx.x] = 0;
        }
    }
    AP_PROF(4);
}

// ---------------------------------------------------------------------------------------------- host
// Describe planes 0..w-1 of qweight as [w][N][K/32] int32 with a [w][16][32] box, 128-byte swizzle.
static bool encode_plane_map(CUtensorMap* map, const void* qweight, long long plane_stride, int N, int K, int w_bits);

// A map depends only on (address, plane stride, N, K, w_bits), and a serving loop calls the same
// layers over and over: the encoded maps are kept in a small per-thread, direct-mapped cache so that
// the driver's encoder runs once per layer and precision, not once per call.
static bool make_plane_map(CUtensorMap* map, const void* qweight, long long plane_stride, int N, int K, int w_bits) {
    struct Entry {
        const void* q;
        long long stride;
        int N, K, w;
        bool valid;
        CUtensorMap map;
    };
    constexpr unsigned kSlots = 1024;
    thread_local static Entry* cache = nullptr;
    if (cache == nullptr) cache = new (std::nothrow) Entry[kSlots]();
    if (cache == nullptr) return encode_plane_map(map, qweight, plane_stride, N, K, w_bits);
    const unsigned long long h = (reinterpret_cast<unsigned long long>(qweight) >> 8) * 0x9E3779B97F4A7C15ull + (unsigned)w_bits * 0x85EBCA6Bu;
    Entry& e = cache[(h >> 40) % kSlots];
    if (e.valid && e.q == qweight && e.stride == plane_stride && e.N == N && e.K == K && e.w == w_bits) {
        *map = e.map;
        return true;
    }
    if (!encode_plane_map(map, qweight, plane_stride, N, K, w_bits)) return false;
    e.q = qweight; e.stride = plane_stride; e.N = N; e.K = K; e.w = w_bits; e.map = *map; e.valid = true;
    return true;
}

static bool encode_plane_map(CUtensorMap* map, const void* qweight, long long plane_stride, int N, int K, int w_bits) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)(K / 32), (cuuint64_t)N, (cuuint64_t)w_bits};
    const cuuint64_t strides[2] = {(cuuint64_t)(K / 32) * 4u, (cuuint64_t)plane_stride * 4u};
    const cuuint32_t box[3] = {(cuuint32_t)kTmaChunkWords, 16u, (cuuint32_t)w_bits};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<void*>(qweight), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int W, int OCC, int MODE, int DEC = 0>
static cudaError_t launch_tma_occ(const CUtensorMap& map, const __half* x, const uint16_t* lut, __half* out, int M, int N,
                                  int K, int splits, int split_chunks, float* partials, int* tickets, cudaStream_t stream,
                                  const GemvEpilogue& epi) {
    using T = GemvTmaCfg<W, OCC, MODE>;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    static bool attr_done[64] = {};
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        int most = 0;
        for (int mp = 1; mp <= 8; mp *= 2) most = T::total(mp) > most ? T::total(mp) : most;
        e = cudaFuncSetAttribute(gemv_kbit_tma_kernel<W, OCC, MODE, DEC, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(gemv_kbit_tma_kernel<W, OCC, MODE, DEC, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) return e;
        if constexpr (W == 4 || W == 7 || W == 8) {
            e = cudaFuncSetAttribute(gemv_kbit_tma_kernel<W, OCC, MODE, DEC, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
            if (e != cudaSuccess) return e;
            e = cudaFuncSetAttribute(gemv_kbit_tma_kernel<W, OCC, MODE, DEC, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
            if (e != cudaSuccess) return e;
        }
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    const int mpad = (M <= 1) ? 1 : (M <= 2) ? 2 : (M <= 4) ? 4 : 8;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(N / 16, splits, (M + 7) / 8);           // more than eight batch rows: only with splits == 1
    cfg.blockDim = dim3(kGemvMaxWarps * 32);
    cfg.dynamicSmemBytes = T::total(mpad);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    constexpr bool kOne = (W == 4 || W == 7 || W == 8);      // single-row instantiations: where they measured faster
    if constexpr (kOne) {
        if (M == 1 && splits <= 1)
            return cudaLaunchKernelEx(&cfg, gemv_kbit_tma_kernel<W, OCC, MODE, DEC, false, true>, map, x, lut, out, M, N, K, mpad,
                                      split_chunks, partials, tickets, epi);
        if (M == 1)
            return cudaLaunchKernelEx(&cfg, gemv_kbit_tma_kernel<W, OCC, MODE, DEC, true, true>, map, x, lut, out, M, N, K, mpad,
                                      split_chunks, partials, tickets, epi);
    }
    if (splits <= 1)                                         // no K split: the instantiation without that epilogue
        return cudaLaunchKernelEx(&cfg, gemv_kbit_tma_kernel<W, OCC, MODE, DEC, false, false>, map, x, lut, out, M, N, K, mpad,
                                  split_chunks, partials, tickets, epi);
    return cudaLaunchKernelEx(&cfg, gemv_kbit_tma_kernel<W, OCC, MODE, DEC, true, false>, map, x, lut, out, M, N, K, mpad, split_chunks,
                              partials, tickets, epi);
}

template <int W>
static cudaError_t launch_tma(const __half* x, const uint32_t* q, long long plane_stride, const uint16_t* lut, __half* out,
                              int M, int N, int K, int splits, float* partials, int* tickets, cudaStream_t stream,
                              bool* used, const GemvEpilogue* epi = nullptr) {
    *used = false;
    if (epi && M > 8) return cudaSuccess;                    // the decoder's epilogues are for decode batches
    const GemvEpilogue plain = {};
    CUtensorMap map;
    if (!make_plane_map(&map, q, plane_stride, N, K, W)) return cudaSuccess;      // caller falls back to cp.async
    const int chunks = (K + 1023) / 1024;
    if (splits > chunks) splits = chunks;
    if (splits < 1 || partials == nullptr || tickets == nullptr) splits = 1;
    const int split_chunks = (chunks + splits - 1) / splits;
    splits = (chunks + split_chunks - 1) / split_chunks;
    *used = true;
    // Three blocks per SM (80 registers) only where two per SM could not hold the launch at once and
    // the table leaves room for enough chunk buffers: measured, that is w = 3 from about 450 blocks on;
    // everywhere else (w = 5, and w = 4 with the compact pair table) it loses.
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            sms = 148;
    }
    if (M > 8 && splits > 1) { *used = false; return cudaSuccess; }              // the caller runs the passes one by one
    const bool many_blocks = (long long)(N / 16) * splits * ((M + 7) / 8) >= 3LL * sms;
#define AP_TMA_GO(OCC_, MODE_) \
    do {                                                                                                                         \
        if (!epi) return launch_tma_occ<W, OCC_, MODE_, 0>(map, x, lut, out, M, N, K, splits, split_chunks, partials, tickets, stream, plain); \
        switch (epi->mode) {                                                                                                     \
            case 1: return launch_tma_occ<W, OCC_, MODE_, 1>(map, x, lut, out, M, N, K, splits, split_chunks, partials, tickets, stream, *epi); \
            case 2: return launch_tma_occ<W, OCC_, MODE_, 2>(map, x, lut, out, M, N, K, splits, split_chunks, partials, tickets, stream, *epi); \
            case 3: return launch_tma_occ<W, OCC_, MODE_, 3>(map, x, lut, out, M, N, K, splits, split_chunks, partials, tickets, stream, *epi); \
            case 4: return launch_tma_occ<W, OCC_, MODE_, 4>(map, x, lut, out, M, N, K, splits, split_chunks, partials, tickets, stream, *epi); \
            case 5: return launch_tma_occ<W, OCC_, MODE_, 5>(map, x, lut, out, M, N, K, splits, split_chunks, partials, tickets, stream, *epi); \
            default: return cudaErrorInvalidValue;                                                                               \
        }                                                                                                                        \
    } while (0)
    if constexpr (W == 3) {
        if (many_blocks) AP_TMA_GO(3, 2);
        AP_TMA_GO(2, 2);
    } else if constexpr (W == 4) {
        if (M <= 2 && many_blocks) AP_TMA_GO(2, 2);          // nibble pairs (3 % faster than neighbours on 11008 x 4096)
        if (M <= 2) AP_TMA_GO(2, 5);                         // neighbouring pairs (3-4 % faster on 4096 x 4096, 4096 x 11008)
        AP_TMA_GO(2, 3);                                     // more rows: the compact pair table (8 % faster than mode 1)
    } else if constexpr (W <= 7) {
        AP_TMA_GO(2, 1);
    } else {
        AP_TMA_GO(2, 0);
    }
#undef AP_TMA_GO
}

}  // namespace ap
