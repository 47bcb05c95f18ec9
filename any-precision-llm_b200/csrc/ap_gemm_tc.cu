// Prefill path for sm_100a: out[M][N] = x[M][K] * W_w[N][K]^T with the weight dequantised on the
// fly into shared-memory tiles and multiplied on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory).
//
// Replaces, for M above the GEMV range, the reference's two-step prefill in
// any_precision/modules/AnyPrecisionLinear.py:60-62: dequant_kbit (kernels/dequant.cuh:177-242)
// writes the whole fp16 weight to HBM, torch.matmul reads it back.  Here the fp16 weight never
// leaves the SM.
//
// Orientation.  The MMA's M side (128 TMEM lanes) is a block of 128 weight rows, its N side is a
// block of BM tokens (64, 128 or 256): D[n][m] += A[n][k] * B[m][k].  The reduction order over k is
// free, so k-tiles follow the packed format: eight consecutive plane words of a row hold 256
// weights whose byte group j (j = 0..3) is a run of 64 CONSECUTIVE weights, so k-tile (words
// 8u..8u+7, byte group j) needs a plain [BM tokens][64 halfs] box of x: one tiled TMA copy,
// swizzled by the TMA unit.  Four such k-tiles make a super-tile, the unit a producer thread
// dequantises from one bit transpose of its words.
//
// The template parameter TM selects how the operands travel (the default, for K % 256 == 0, is 3):
//   TM = 3  planes by tiled TMA ([w][128 rows][8 or 16 words] boxes into a double buffer), sixteen
//           producer warps (four threads per weight row); the dequantised weights go straight into
//           TENSOR MEMORY (tcgen05.st into a ring of 128-column super-stages beside the accumulator,
//           the producer's row being its TMEM lane) and the MMA takes A from tensor memory; the
//           shared memory goes to the activation ring.  w = 3 looks its table up from registers.
//   TM = 2  the same loaders, but A is stored as 16-byte swizzled chunks in shared-memory stages
//           (fence.proxy.async) and read from there by the MMA.
//   TM = 1  as TM = 2 with the planes read from global memory by the producers (one 16-byte load
//           per plane, thread and eight words): where two plane buffers would not leave three stages.
//   TM = 0  K % 256 != 0: k-tiles of two words; eight producer warps gather the eight scattered
//           runs of x with 16-byte cp.async, signalling a stage when their copies have landed.
//
// Roles in a CTA (TM >= 2; TM <= 1 has eight producer warps):
//   warps 0-15 producers: dequantise, then, after the main loop, drain TMEM (tcgen05.ld), convert
//              to fp16 and store the transposed tile (or park fp32 partials for split-K).
//   warp 16    allocates TMEM; one lane issues four tcgen05.mma.cta_group::1.kind::f16 per k-tile
//              and one tcgen05.commit per super-tile.  For token blocks up to 128 a further warp is a
//              second issuer: each takes every other super-tile into an accumulator of its own and
//              the read-out adds the two (rings have an even number of hand-over units, so that a
//              barrier is always waited on by the same issuer).
//   warp 17    one lane issues the TMA copies (planes two groups ahead, activations as stages free).
// The kernel is a programmatic-dependent-launch secondary: TMEM allocation, barriers, tables and
// the first plane boxes come before the dependency wait, activations and the output after it.
// Every wait is bounded: on expiry the kernel raises a status flag, skips the remaining work,
// still frees its tensor memory and returns.
#include <cstdlib>

#include "ap_bitplane.cuh"
#include "ap_kernels.h"
#include "ap_tensormap.h"

namespace ap {

namespace tc {

constexpr int kBN = 128;            // weight rows per CTA = MMA M
constexpr int kBK = 64;             // weights per k-tile = one 128-byte swizzle row
// Producer threads per weight row: two (eight warps); four (sixteen warps) in the variant that reads the
// planes from shared memory, where more warps only add lookups in flight and no global requests.
__host__ __device__ constexpr int producers_for(int tm) { return tm >= 2 ? 512 : 256; }
// MMA-issuing warps: two, each with an accumulator of its own and every other super-tile, where the weights
// are in tensor memory and two accumulators fit beside them (a tcgen05.mma costs its issuing thread about
// 70 cycles whatever its size, which bounds a small token block)
__host__ __device__ constexpr int issuers_for(int bm, int tm) { return (tm == 3 && bm <= 128) ? 2 : 1; }
__host__ __device__ constexpr int threads_for(int bm, int tm) {
    return producers_for(tm) + (tm >= 1 ? 64 : 32) + 32 * (issuers_for(bm, tm) - 1);
}
constexpr uint32_t kSpinLimit = 1u << 18;   // mbarrier.try_wait attempts before giving up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait for the phase with the given parity.  Returns false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; i++) {
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

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart (SBO), LBO unused (1), descriptor
    // version 1 (sm_100), layout type 2 (SWIZZLE_128B); the tile base is 1024-byte aligned.
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t hi = 64u | (1u << 14) | (2u << 29);
    return (static_cast<uint64_t>(hi) << 32) | lo;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same with the A operand in tensor memory: lane = row, 32-bit column = two consecutive k.
__device__ __forceinline__ void umma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <int W>
struct Smem {
    static constexpr int C = 1 << W;
    // Table for the 128 rows, free of bank conflicts: [code][row / 64][lane] of 32-bit entries
    // holding (T[row 32*(2h) + lane][code], T[row 32*(2h+1) + lane][code]): a lane of warp q reads
    // half q & 1 of entry [code][q >> 1][lane], always in its own bank.
    static constexpr int kTableBytes = C * 256;
    __host__ __device__ static constexpr int a_stage_bytes() { return kBN * 128; }
    __host__ __device__ static constexpr int b_stage_bytes(int bm) { return bm * 128; }
    // plane buffers of the variant that brings the planes in by TMA: two, each [W][128 rows][8 words]
    __host__ __device__ static constexpr int plane_buf_bytes() { return W * kBN * 32; }
    __host__ __device__ static constexpr int plane_bytes(bool ptma) { return ptma ? 2 * plane_buf_bytes() : 0; }
    // Stages of the weight (A) ring.  Without TMA the activation (B) ring has as many and moves in step.
    __host__ __device__ static constexpr int stages(int bm, bool ptma) {
        const int per = a_stage_bytes() + b_stage_bytes(bm);
        const int room = 220 * 1024 - kTableBytes - 1024 - plane_bytes(ptma);
        const int s = room / per;
        return s > 6 ? 6 : s;
    }
    // TMA variants: the activation ring is decoupled from the weight ring and deeper.  A tile of activations
    // is asked for as soon as its buffer is free, long before the producers reach that k-tile: the round
    // trip of a TMA box of 64..256 rows (2-3 us) then hides behind several k-tiles instead of one ring cycle.
    __host__ __device__ static constexpr int a_stages_tma(int bm, bool ptma) {
        const int s = stages(bm, ptma);
        return s > 4 ? 4 : (s > 3 ? 3 : s);
    }
    __host__ __device__ static constexpr int b_stages_tma(int bm, bool ptma) {
        const int room = 220 * 1024 - kTableBytes - 1024 - plane_bytes(ptma) - a_stages_tma(bm, ptma) * a_stage_bytes();
        const int s = room / b_stage_bytes(bm);
        return s > 12 ? 12 : s;
    }
    // Variant 3 keeps the dequantised weights in tensor memory (a ring of eight 32-column stages beside the
    // accumulator), not in shared memory: no weight stages here, more room for the activation ring.
    __host__ __device__ static constexpr int a_ring_stages(int bm, int tm) {
        return tm == 0 ? stages(bm, false) : (tm == 3 ? 8 : a_stages_tma(bm, tm == 2));
    }
    __host__ __device__ static constexpr int a_ring_bytes(int bm, int tm) {
        return tm == 3 ? 0 : a_ring_stages(bm, tm) * a_stage_bytes();
    }
    // Words per row of a plane box.  The TMA unit moves a box row by row, and rows of 32 bytes (eight
    // words) are what bounds the kernel (measured: the time per k-tile did not depend on anything the
    // producers do); variant 3 takes the longest rows (32 or 16 words = 4 or 2 super-tiles per box) that
    // still leave three activation stages, eight for token blocks up to 128 (two groups of four stages are
    // what the second MMA issuer needs, and it is worth more than long rows).
    __host__ __device__ static constexpr int plane_words(int bm, int tm) {
        if (tm != 3) return 8;
        for (int pw = 32; pw >= 16; pw /= 2) {
            const int room = 220 * 1024 - kTableBytes - 1024 - 2 * W * kBN * pw * 4;
            if (room >= (bm <= 128 ? 8 : 3) * b_stage_bytes(bm)) return pw;
        }
        return 8;
    }
    __host__ __device__ static constexpr int plane_buf_bytes(int bm, int tm) { return W * kBN * plane_words(bm, tm) * 4; }
    __host__ __device__ static constexpr int plane_bytes(int bm, int tm) { return tm >= 2 ? 2 * plane_buf_bytes(bm, tm) : 0; }
    __host__ __device__ static constexpr int b_ring_stages(int bm, int tm) {
        if (tm == 0) return stages(bm, false);
        const int room = 220 * 1024 - kTableBytes - 1024 - plane_bytes(bm, tm) - a_ring_bytes(bm, tm);
        const int s = room / b_stage_bytes(bm);
        return s > 12 ? 12 : s;
    }
    __host__ __device__ static constexpr int total(int bm, int tm) {
        return 1024 + kTableBytes + a_ring_bytes(bm, tm) + b_ring_stages(bm, tm) * b_stage_bytes(bm) + plane_bytes(bm, tm) + 512;
    }
};

// TM: 0 = activations gathered by the producers (any K % 128 == 0); 1 = activations by TMA, planes read
// from global memory by the producers; 2 = activations and planes by TMA (K % 256 == 0 for both).
template <int W, int BM, int TM>
__global__ void __launch_bounds__(threads_for(BM, TM), 1)
gemm_kbit_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap qmap,
                    const __half* __restrict__ x, const uint32_t* __restrict__ q, long long plane_stride,
                    const uint16_t* __restrict__ lut, __half* __restrict__ out, int M, int N, int K, int* status,
                    float* __restrict__ partials, int* __restrict__ tickets) {
    using S = Smem<W>;
    constexpr bool BTMA = TM >= 1, PTMA = TM >= 2, ATMEM = TM == 3, ATMEM_ = ATMEM;
    constexpr int kProducers = producers_for(TM);
    constexpr int kMmaWarp = kProducers / 32, kLoadWarp = kMmaWarp + 1;
    constexpr int kWpt = 1024 / kProducers;                  // plane words per thread and super-tile: 4 or 2
    constexpr int C = 1 << W;
    constexpr int kStages = S::a_ring_stages(BM, TM);                                      // weight ring
    // activation ring; with the weights in tensor memory its stages are released in groups of kGB
    constexpr int kStagesBRaw = S::b_ring_stages(BM, TM);
    constexpr int kGB = !ATMEM_ ? 1 : (kStagesBRaw >= 8 ? 4 : (kStagesBRaw >= 4 ? 2 : 1));
    // Two issuers (where the block has the extra warp and the activation ring holds two groups of four): both
    // rings then have an even number of hand-over units (super-stages, activation groups), so that a unit and
    // its barriers always belong to the same issuer.
    constexpr int kIssuers = (issuers_for(BM, TM) > 1 && kGB == 4) ? 2 : 1;
    constexpr int kStagesB = kIssuers > 1 ? kStagesBRaw / 8 * 8 : kStagesBRaw / kGB * kGB;
    // with groups of four the activation tiles of a super-tile also ARRIVE on one barrier: the MMA thread
    // then waits twice per four k-tiles (weights, activations) instead of five times
    constexpr bool kBGroupFull = kGB == 4;
    constexpr uint32_t kTmemCols = ATMEM ? 512u : (uint32_t)BM;      // accumulator (+ weight ring at column 256)
    // weight ring in tensor memory: super-stages of four k-tiles (128 columns); three of them beside an
    // accumulator of up to 128 columns, two beside a wider one
    constexpr uint32_t kTmemA = 256u;                         // after the accumulator(s): kIssuers x BM columns
    constexpr int kSuper = 2;
    static_assert(kIssuers * BM <= (int)kTmemA, "accumulators overlap the weight ring");
    constexpr int kPW = S::plane_words(BM, TM);               // words per row of a plane box
    constexpr int kGroup = kPW / 8;                          // super-tiles per plane box
    constexpr bool kPSwz = TM == 3;                          // plane boxes swizzled (32/64/128-byte mode by row length)
    constexpr int kPlaneBuf = S::plane_buf_bytes(BM, TM);
    constexpr int kAStage = S::a_stage_bytes(), kBStage = S::b_stage_bytes(BM);
    static_assert(kStages >= 2 && kStagesB >= 2, "not enough shared memory for two stages");
    static_assert(BM % 32 == 0 && BM >= 32 && BM <= 256, "MMA N: a multiple of 32 up to 256");

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // The table sits at the start of the dynamic area: its shared address is then a link-time constant
    // that the lookups take as their immediate offset.
    uint32_t* table = reinterpret_cast<uint32_t*>(smem_raw);
    const uint32_t after_table = smem_u32(smem_raw) + (uint32_t)S::kTableBytes;
    unsigned char* smem = smem_raw + S::kTableBytes + ((1024u - (after_table & 1023u)) & 1023u);
    unsigned char* a_tiles = smem;                                   // kStages x [128 rows][128 bytes], swizzled
    unsigned char* b_tiles = smem + S::a_ring_bytes(BM, TM);         // kStagesB x [BM rows][128 bytes], swizzled
    unsigned char* p_tiles = b_tiles + kStagesB * kBStage;           // PTMA: 2 x [W][128 rows][8 words]
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_tiles + S::plane_bytes(BM, TM));
    // bars[0..kStages) = full, bars[kStages..2*kStages) = empty, bars[2*kStages] = accumulator ready,
    // then planes full[2], planes empty[2], then activation ring full[kStagesB], empty[kStagesB]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 5 + 2 * kStagesB);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * kBN, m0 = blockIdx.y * BM;
    // Dependent launch: the next kernel of the stream may start its prologue now.  This kernel reads weights
    // (planes, tables: never written on the stream) before its own dependency wait and everything else (x, the
    // workspace, out, status) after it: the loader waits before its first activation tile, the producers before
    // the read-out, and every data path to them runs through those two.  Without the loader warp the
    // producers read x themselves, so everybody waits here.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if constexpr (!BTMA) asm volatile("griddepcontrol.wait;" ::: "memory");
    const int words = K >> 5;
    // Split-K (gridDim.z > 1, TMA variants only): this block takes the super-tiles (groups of eight plane
    // words = four k-tiles) [st_base, st_base + supers_l) of every row; stage and barrier bookkeeping
    // below counts k-tiles from the block's own first one.
    int st_base = 0, supers_l = words >> 3, ktiles = K >> 6;
    if (gridDim.z > 1) {
        const int per = ((words >> 3) + gridDim.z - 1) / gridDim.z;
        st_base = blockIdx.z * per;
        supers_l = (words >> 3) - st_base < per ? (words >> 3) - st_base : per;
        ktiles = 4 * supers_l;
    }
    const int full_words = (K >> 10) << 5, tail_stride = (K & 1023) >> 2;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    const uint32_t accum_bar = bar0 + 8u * (2 * kStages);
    auto pfull_bar = [&](int b) { return bar0 + 8u * (2 * kStages + 1 + b); };
    auto pempty_bar = [&](int b) { return bar0 + 8u * (2 * kStages + 3 + b); };
    auto bfull_bar = [&](int s) { return bar0 + 8u * (2 * kStages + 5 + s); };
    auto bempty_bar = [&](int s) { return bar0 + 8u * (2 * kStages + 5 + kStagesB + s); };

    if (tid == 0) {
        // full: in the TMA variants one arrival per producer warp (its lane 0, after the warp has synchronised)
        // plus the loader's; otherwise one per producer thread, each after its own activation copies landed
        for (int s = 0; s < kStages; s++) { mbar_init(full_bar(s), BTMA ? kProducers / 32 : kProducers); mbar_init(empty_bar(s), 1); }
        for (int s = 0; s < kStagesB; s++) { mbar_init(bfull_bar(s), 1); mbar_init(bempty_bar(s), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(pfull_bar(b), 1); mbar_init(pempty_bar(b), kProducers / 32); }
        if constexpr (BTMA) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&xmap)) : "memory");
        if constexpr (PTMA) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&qmap)) : "memory");
        mbar_init(accum_bar, kIssuers);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Table: thread i < 128 spreads row n0 + i over its own bank.
    if (tid < kBN) {
        const int hq = tid >> 6, hb = (tid >> 5) & 1;       // which 64-row half, which 16-bit half of the entry
        uint16_t* tab16 = reinterpret_cast<uint16_t*>(table);
        const uint16_t* src = lut + (size_t)(n0 + tid) * C;
        for (int c8 = 0; c8 < C; c8 += 8) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + c8));
            const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t h = (vv[i >> 1] >> (16 * (i & 1))) & 0xffffu;
                tab16[(((c8 + i) * 2 + hq) * 32 + lane) * 2 + hb] = (uint16_t)h;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    bool ok = true;

    if (warp < kMmaWarp) {
        // ---------------------------------------------------------------- producers
        // Thread (r, wd): weight row n0 + r, plane word `wd` of every k-tile (32 of its 64 weights).
        const int r = tid & (kBN - 1), wd = tid >> 7;
        const uint32_t* qrow = q + (size_t)(n0 + r) * words;
        // byte offset of this row's entry inside a code's 256-byte stripe (below 256: it is byte 0 of
        // every lookup address, the code is byte 1)
        uint32_t tab_lane = ((r >> 6) * 32 + lane) * 4 + ((r >> 5) & 1) * 2;
        asm volatile("" : "+r"(tab_lane)::"memory");        // table reads stay below the barrier that published it
        const uint32_t table_const = smem_u32(smem_raw);
        const uint32_t a_row = smem_u32(a_tiles) + r * 128;
        const int sw = r & 7;
        // w = 3 with the weights in tensor memory: the row's eight table entries live in four registers
        // (low bytes, high bytes) and a byte permute with the nibble codes as selectors IS the lookup: no
        // shared-memory reads at all for the dequantisation (the shared-memory pipe is what bounds a token
        // block of 256: table reads + the MMAs' reads of the activation tile + its TMA writes).
        constexpr bool kRegLut = (W == 3) && ATMEM;
        uint32_t lut_lo[2] = {0u, 0u}, lut_hi[2] = {0u, 0u};
        if constexpr (kRegLut) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(lut + (size_t)(n0 + r) * C));
            lut_lo[0] = __byte_perm(v.x, v.y, 0x6420); lut_lo[1] = __byte_perm(v.z, v.w, 0x6420);
            lut_hi[0] = __byte_perm(v.x, v.y, 0x7531); lut_hi[1] = __byte_perm(v.z, v.w, 0x7531);
        }
        // Planes arrive 4 words (two k-tiles) at a time, two such groups ahead; the L2 is warmed
        // further ahead with prefetches.
        if constexpr (BTMA) {
            // Thread (r, hf): words 8*st + kWpt*hf .. of super-tile st (eight words = four k-tiles).
            const int hf = wd;                               // tid >> 7
            const int supers = supers_l;
            uint32_t cur[W][kWpt], nxt[W][kWpt];
            auto load_super = [&](uint32_t (&dst)[W][kWpt], int st) {
#pragma unroll
                for (int p = 0; p < W; p++) {
                    const uint4 v = *reinterpret_cast<const uint4*>(qrow + (size_t)p * plane_stride + 8 * (st_base + st) + 4 * hf);
                    dst[p][0] = v.x; dst[p][1] = v.y;
                    if constexpr (kWpt == 4) { dst[p][2] = v.z; dst[p][3] = v.w; }
                }
            };
            if constexpr (!PTMA) load_super(cur, 0);
            for (int st = 0; st < supers && ok; st++) {
                if constexpr (PTMA) {
                    // this super-tile's planes were brought into a buffer by the loader warp
                    const int pg = st / kGroup, u = st % kGroup, pb = pg & 1;      // box, super-tile inside it, buffer
                    if (u == 0) ok = mbar_wait(pfull_bar(pb), (pg >> 1) & 1);
                    if (!ok) break;
                    // this thread's words inside its row of the box; swizzled boxes: 16-byte chunk ^ f(row)
                    const uint32_t o = (uint32_t)u * 32u + (uint32_t)hf * (kWpt * 4);
                    const uint32_t swz = !kPSwz ? 0u : (kPW == 32 ? (uint32_t)(r & 7) : kPW == 16 ? (uint32_t)((r >> 1) & 3) : (uint32_t)((r >> 2) & 1));
                    const uint32_t src = smem_u32(p_tiles) + pb * kPlaneBuf + r * (kPW * 4) + ((((o >> 4) ^ swz) << 4) | (o & 15u));
#pragma unroll
                    for (int p = 0; p < W; p++) {
                        if constexpr (kWpt == 4)
                            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(cur[p][0]), "=r"(cur[p][1]), "=r"(cur[p][2]), "=r"(cur[p][3]) : "r"(src + p * (kBN * kPW * 4)));
                        else
                            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(cur[p][0]), "=r"(cur[p][1]) : "r"(src + p * (kBN * kPW * 4)));
                    }
                    if (u == kGroup - 1 || st == supers - 1) {           // last read of this box
                        __syncwarp();
                        if (lane == 0) mbar_arrive(pempty_bar(pb));
                    }
                } else {
                    if (st + 1 < supers) load_super(nxt, st + 1);
                    if (hf == 0 && 8 * (st_base + st) + 64 < words) {
#pragma unroll
                        for (int p = 0; p < W; p++)
                            asm volatile("prefetch.global.L2 [%0];" ::"l"(qrow + (size_t)p * plane_stride + 8 * (st_base + st) + 64));
                    }
                }
                uint32_t cw[kWpt][8];
                uint32_t pk[kWpt][4][4];                     // kRegLut: [word][byte group j][pair of weights]
#pragma unroll
                for (int i = 0; i < kWpt; i++) {
                    uint32_t planes[W];
#pragma unroll
                    for (int p = 0; p < W; p++) planes[p] = cur[p][i];
                    if constexpr (kRegLut) {
                        // nb[c], byte 3 - j: high nibble = code of weight e = 3 - c, low nibble = e = 7 - c
                        uint32_t nb[4], wq[4][4];            // wq[c][j] = fp16x2 (W[7 - c], W[3 - c]) of byte group j
                        transpose_nibbles<(W <= 4 ? W : 4)>(reinterpret_cast<const uint32_t (&)[(W <= 4 ? W : 4)]>(planes), nb);
#pragma unroll
                        for (int c = 0; c < 4; c++)
#pragma unroll
                            for (int hs = 0; hs < 2; hs++) {
                                const uint32_t sel = hs ? (nb[c] >> 16) : nb[c];
                                const uint32_t lo = __byte_perm(lut_lo[0], lut_lo[1], sel);
                                const uint32_t hi = __byte_perm(lut_hi[0], lut_hi[1], sel);
                                wq[c][3 - 2 * hs] = __byte_perm(lo, hi, 0x5140);
                                wq[c][2 - 2 * hs] = __byte_perm(lo, hi, 0x7362);
                            }
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            pk[i][j][0] = __byte_perm(wq[3][j], wq[2][j], 0x7632);   // weights e = 0, 1
                            pk[i][j][1] = __byte_perm(wq[1][j], wq[0][j], 0x7632);   // 2, 3
                            pk[i][j][2] = __byte_perm(wq[3][j], wq[2][j], 0x5410);   // 4, 5
                            pk[i][j][3] = __byte_perm(wq[1][j], wq[0][j], 0x5410);   // 6, 7
                        }
                    } else {
                        transpose_codes<W>(planes, cw[i]);
                    }
                }
                if constexpr (ATMEM) {
                    // The tensor-memory ring is handed over in super-stages of four stages = the four k-tiles of a
                    // super-tile: one barrier pair per super-stage, so that the producers and, above all,
                    // the MMA thread pay one wait and one commit per four k-tiles (a tcgen05.commit costs the
                    // issuing thread about as much as two MMAs).
                    ok = mbar_wait(empty_bar(st % kSuper), ((st / kSuper) & 1) ^ 1);
                    if (!ok) break;
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int kt = 4 * st + j;
                    const int s = kt % kStages;
                    if constexpr (!ATMEM) {
                        ok = ok && mbar_wait(empty_bar(s), ((kt / kStages) & 1) ^ 1);
                        if (!ok) break;
                    }
                    const uint32_t a_dst = a_row + s * kAStage;
#pragma unroll
                    for (int i = 0; i < kWpt; i++) {
                        uint32_t p0, p1, p2, p3;
                        if constexpr (kRegLut) {
                            p0 = pk[i][j][0]; p1 = pk[i][j][1]; p2 = pk[i][j][2]; p3 = pk[i][j][3];
                        } else {
                            uint32_t h[8];
#pragma unroll
                            for (int e = 0; e < 8; e++) {
                                uint32_t off;                // (code << 8) | entry byte: one byte permute
                                asm("prmt.b32 %0, %1, %2, %3;" : "=r"(off) : "r"(cw[i][e]), "r"(tab_lane), "r"(0x7704u | ((uint32_t)(3 - j) << 4)));
                                asm("ld.shared.u16 %0, [%1];" : "=r"(h[e]) : "r"(table_const + off));
                            }
                            p0 = __byte_perm(h[0], h[1], 0x5410); p1 = __byte_perm(h[2], h[3], 0x5410);
                            p2 = __byte_perm(h[4], h[5], 0x5410); p3 = __byte_perm(h[6], h[7], 0x5410);
                        }
                        const int c = kWpt * hf + i;         // chunk = word inside the super-tile
                        if constexpr (ATMEM) {
                            // row = this thread's TMEM lane, eight weights = four 32-bit columns of the stage
                            const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + kTmemA + 128u * (st % kSuper) + 32u * j + 4u * c;
                            asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};"
                                         ::"r"(taddr), "r"(p0), "r"(p1), "r"(p2), "r"(p3) : "memory");
                        } else {
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a_dst + ((c ^ sw) << 4)),
                                         "r"(p0), "r"(p1), "r"(p2), "r"(p3) : "memory");
                        }
                    }
                    if constexpr (!ATMEM) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA
                        __syncwarp();
                        if (lane == 0) mbar_arrive(full_bar(s));
                    }
                }
                if constexpr (ATMEM) {
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_bar(st % kSuper));
                }
                if constexpr (!PTMA) {
#pragma unroll
                    for (int p = 0; p < W; p++)
#pragma unroll
                        for (int i = 0; i < kWpt; i++) cur[p][i] = nxt[p][i];
                }
            }
        } else {
        const int groups = (words + 3) >> 2;
        // A stage is signalled kLag k-tiles after it was written, so that up to kLag activation copies
        // stay in flight; the producers hold kLag + 1 stages, the MMA needs at least one more.
        constexpr int kLag = (kStages >= 5) ? 3 : (kStages == 4) ? 2 : 1;
        uint4 cur[W], nxt[W], nx2[W];
        auto load_group = [&](uint4 (&dst)[W], int gidx) {
#pragma unroll
            for (int p = 0; p < W; p++) {
                const uint32_t* src = qrow + (size_t)p * plane_stride + 4 * gidx;
                if (4 * gidx + 4 <= words) dst[p] = *reinterpret_cast<const uint4*>(src);
                else { const uint2 t2 = *reinterpret_cast<const uint2*>(src); dst[p] = make_uint4(t2.x, t2.y, 0u, 0u); }
            }
        };
        load_group(cur, 0);
        if (groups > 1) load_group(nxt, 1);
        for (int kt = 0; kt < ktiles && ok; kt++) {
            const int s = kt % kStages;
            if ((kt & 1) == 0) {
                if ((kt >> 1) + 2 < groups) load_group(nx2, (kt >> 1) + 2);
                if (wd == 0 && 2 * kt + 64 < words) {
#pragma unroll
                    for (int p = 0; p < W; p++)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(qrow + (size_t)p * plane_stride + 2 * kt + 64));
                }
            }
            ok = mbar_wait(empty_bar(s), ((kt / kStages) & 1) ^ 1);
            if (!ok) break;
            if constexpr (!BTMA) {
                // where this k-tile's eight runs live in a row of x
                const int word0 = 2 * kt;
                int kbase, kstride;
                if (word0 < full_words) { kbase = (word0 >> 5) * 1024 + (word0 & 31) * 8; kstride = 256; }
                else { kbase = full_words * 32 + (word0 - full_words) * 8; kstride = tail_stride; }
                // B stage: chunk c = 2*j + wd of token row m  <-  x[m][kbase + 8*wd + kstride*j .. +8)
                const uint32_t b_stage = smem_u32(b_tiles) + s * kBStage;
#pragma unroll
                for (int i = 0; i < BM * 8 / kProducers; i++) {
                    const int idx = tid + i * kProducers;
                    const int m = idx >> 3, c = idx & 7;
                    const int mg = (m0 + m < M) ? (m0 + m) : (M - 1);
                    const __half* src = x + (size_t)mg * K + kbase + 8 * (c & 1) + kstride * (c >> 1);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(b_stage + m * 128 + ((c ^ (m & 7)) << 4)), "l"(src) : "memory");
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            // A stage: this thread's word -> chunks 2*j + wd, j = 0..3, of its row
            {
                uint32_t planes[W], cw[8];
                const int widx = 2 * (kt & 1) + wd;          // word of the current group of four
#pragma unroll
                for (int p = 0; p < W; p++)
                    planes[p] = (widx == 0) ? cur[p].x : (widx == 1) ? cur[p].y : (widx == 2) ? cur[p].z : cur[p].w;
                transpose_codes<W>(planes, cw);
                const uint32_t a_dst = a_row + s * kAStage;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint32_t h[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        uint32_t off;                        // (code << 8) | entry byte: one byte permute
                        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(off) : "r"(cw[e]), "r"(tab_lane), "r"(0x7704u | ((uint32_t)(3 - j) << 4)));
                        asm("ld.shared.u16 %0, [%1];" : "=r"(h[e]) : "r"(table_const + off));
                    }
                    const int c = 2 * j + wd;
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a_dst + ((c ^ sw) << 4)),
                                 "r"(__byte_perm(h[0], h[1], 0x5410)), "r"(__byte_perm(h[2], h[3], 0x5410)),
                                 "r"(__byte_perm(h[4], h[5], 0x5410)), "r"(__byte_perm(h[6], h[7], 0x5410))
                                 : "memory");
                }
            }
            if constexpr (BTMA) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA
                mbar_arrive(full_bar(s));
            } else if (kt >= kLag) {
                // k-tile kt - kLag is complete once its activations have landed; younger copies fly on.
                asm volatile("cp.async.wait_group %0;" ::"n"(kLag) : "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(full_bar((kt - kLag) % kStages));
            }
            if (kt & 1) {
#pragma unroll
                for (int p = 0; p < W; p++) { cur[p] = nxt[p]; nxt[p] = nx2[p]; }
            }
        }
        if constexpr (!BTMA) {
            if (ok) {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                for (int kt = (ktiles > kLag ? ktiles - kLag : 0); kt < ktiles; kt++) mbar_arrive(full_bar(kt % kStages));
            }
        }
        }
        // ---------------------------------------------------------------- epilogue
        if constexpr (BTMA) asm volatile("griddepcontrol.wait;" ::: "memory");
        if (ok) ok = mbar_wait(accum_bar, 0);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // warp w may touch TMEM lanes 32*(w%4)..+31; the warps that share a lane group split the columns
            constexpr int kColParts = kProducers / 128;
            const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
            __half* orow = out + n0 + (warp & 3) * 32 + lane;               // column n of the output
            const int cbeg = (warp >> 2) * (BM / kColParts), cend = cbeg + BM / kColParts;
#pragma unroll 1
            for (int c0 = cbeg; c0 < cend; c0 += 16) {
                uint32_t v[16];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(taddr + c0));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (kIssuers > 1 && supers_l > 1) {
                    // the second issuer's accumulator (it exists once the block has two super-tiles)
                    uint32_t u[16];
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
                          "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
                        : "r"(taddr + BM + c0));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(u[i]));
                }
                if (gridDim.z == 1) {
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const int m = m0 + c0 + i;
                        if (m < M) orow[(size_t)m * N] = __float2half_rn(__uint_as_float(v[i]));
                    }
                } else {
                    // split-K: park the fp32 tile; the block that draws the tile's last ticket adds them up
                    float* prow = partials + (size_t)blockIdx.z * M * N + n0 + (warp & 3) * 32 + lane;
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const int m = m0 + c0 + i;
                        if (m < M) __stcg(prow + (size_t)m * N, __uint_as_float(v[i]));
                    }
                }
            }
        }
        if (gridDim.z > 1) {
            // Every producer thread comes here, whatever happened above: the barrier below counts them all.
            int* s_last = reinterpret_cast<int*>(tmem_slot + 1);
            const int tile = blockIdx.y * gridDim.x + blockIdx.x;
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(kProducers) : "memory");
            if (tid == 0) *s_last = (atomicAdd(tickets + tile, 1) == (int)gridDim.z - 1);
            asm volatile("bar.sync 1, %0;" ::"n"(kProducers) : "memory");
            if (*s_last) {
                __threadfence();
                constexpr int kColParts2 = kProducers / 128;
                const int n = n0 + (warp & 3) * 32 + lane;
                const int cb = (warp >> 2) * (BM / kColParts2);
                // four token rows at a time, all ranges' loads issued before the first is used (at most 8 ranges)
                const int Z = gridDim.z;
                for (int c = cb; c < cb + BM / kColParts2; c += 4) {
                    float v[4][8];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int m = m0 + c + u;
#pragma unroll
                        for (int z = 0; z < 8; z++)
                            v[u][z] = (m < M && z < Z) ? __ldcg(partials + ((size_t)z * M + m) * N + n) : 0.f;
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int m = m0 + c + u;
                        float sum = 0.f;
#pragma unroll
                        for (int z = 0; z < 8; z++) sum += v[u][z];          // range order, fixed
                        if (m < M) out[(size_t)m * N + n] = __float2half_rn(sum);
                    }
                }
                if (tid == 0) tickets[tile] = 0;                 // handed back at zero for the next call
            }
        }
    } else if (BTMA && warp == kLoadWarp) {
        // ---------------------------------------------------------------- activation loader
        if (lane == 0) {
            const int supers = supers_l;
            // planes of super-tile st -> buffer st & 1 (waits until the producers have read that buffer's last use)
            const int boxes = (supers + kGroup - 1) / kGroup;
            // planes of box pg (kGroup super-tiles) -> buffer pg & 1 (waits until the producers have read that buffer's last use)
            auto request_planes = [&](int pg) {
                const int pb = pg & 1;
                if (!mbar_wait(pempty_bar(pb), ((pg >> 1) & 1) ^ 1)) return false;
                const uint32_t bar = pfull_bar(pb);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)kPlaneBuf) : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                    ::"r"(smem_u32(p_tiles) + pb * kPlaneBuf), "l"(reinterpret_cast<uint64_t>(&qmap)), "r"(8 * st_base + kPW * pg), "r"(n0), "r"(0), "r"(bar)
                    : "memory");
                return true;
            };
            if constexpr (PTMA) {
                ok = request_planes(0);
                if (ok && boxes > 1) ok = request_planes(1);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");      // x may be the previous kernel's output
            for (int kt = 0; kt < ktiles && ok; kt++) {
                if constexpr (PTMA) {
                    // when the activations of a box's first k-tile are asked for: the planes of the next box
                    if (kt % (4 * kGroup) == 0 && kt > 0 && kt / (4 * kGroup) + 1 < boxes) {
                        ok = request_planes(kt / (4 * kGroup) + 1);
                        if (!ok) break;
                    }
                }
                const int s = kt % kStagesB;
                if (kt % kGB == 0) ok = mbar_wait(bempty_bar(s / kGB), ((kt / kStagesB) & 1) ^ 1);   // the group's buffers are free
                if (!ok) break;
                const uint32_t bar = kBGroupFull ? bfull_bar(s / 4) : bfull_bar(s);
                if (!kBGroupFull || (kt & 3) == 0)
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)(kBGroupFull ? 4 * kBStage : kBStage)) : "memory");
                // k-tile kt = (super-tile st, byte group j): 64 consecutive weights of every row of x
                const int st = st_base + (kt >> 2), j = kt & 3;
                const int w0 = 8 * st;                                       // first plane word of the super-tile
                int k0;
                if (w0 < full_words) k0 = (w0 >> 5) * 1024 + 256 * j + (w0 & 31) * 8;
                else k0 = full_words * 32 + tail_stride * j + (w0 - full_words) * 8;
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(smem_u32(b_tiles) + s * kBStage), "l"(reinterpret_cast<uint64_t>(&xmap)), "r"(k0), "r"(m0), "r"(bar)
                    : "memory");
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- MMA issuer(s)
        // Issuer `which` takes the super-tiles st with st % kIssuers == which and accumulates them in columns
        // [which * BM, +BM); the read-out adds the accumulators.  A commit tracks the MMAs of the committing
        // thread only, so each stage is still released by exactly one commit.
        constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(BM >> 3) << 17) | ((uint32_t)(kBN >> 4) << 24);
        static_assert(kIssuers == 1 || (kGB == 4 && kStagesB % 8 == 0 && kSuper % 2 == 0), "rings must not alternate between issuers");
        const int which = (warp != kMmaWarp) ? 1 : 0;
        if (kIssuers == 1 && which) ok = true, ktiles = 0;                          // a spare warp without a role
        const uint32_t tmem_d = tmem_base + (uint32_t)(which * BM);
        const int supers_mine = (supers_l - which + kIssuers - 1) / kIssuers;       // may be 0 for the second issuer
        if (kIssuers > 1 && supers_mine <= 0 && lane == 0) mbar_arrive(accum_bar);
        for (int kt = 0; kt < ktiles && ok; kt++) {
            if (kIssuers > 1 && ((kt >> 2) % kIssuers) != which) continue;
            const int s = kt % kStages, sb = kt % kStagesB;
            if constexpr (ATMEM) {
                if ((kt & 3) == 0) ok = mbar_wait(full_bar((kt >> 2) % kSuper), ((kt >> 2) / kSuper) & 1);   // a whole super-tile of weights
            } else {
                ok = mbar_wait(full_bar(s), (kt / kStages) & 1);
            }
            if constexpr (kBGroupFull) {
                if (ok && (kt & 3) == 0) ok = mbar_wait(bfull_bar(sb / 4), (kt / kStagesB) & 1);
            } else {
                if (ok && BTMA) ok = mbar_wait(bfull_bar(sb), (kt / kStagesB) & 1);
            }
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint64_t adesc = make_desc(smem_u32(a_tiles) + s * kAStage);
                const uint64_t bdesc = make_desc(smem_u32(b_tiles) + sb * kBStage);
                const bool first = kt == 4 * which;                   // this issuer's first k-tile starts its accumulator
#pragma unroll
                for (int kk = 0; kk < kBK / 16; kk++) {
                    if constexpr (ATMEM)
                        umma_f16_ta(tmem_d, tmem_base + kTmemA + 128u * ((kt >> 2) % kSuper) + 32u * (kt & 3) + 8u * kk, bdesc + 2 * kk, idesc,
                                    (!first || kk > 0) ? 1u : 0u);
                    else
                        umma_f16(tmem_d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (!first || kk > 0) ? 1u : 0u);
                }
                // commits free the stages when these MMAs retire
                if constexpr (ATMEM) {
                    if ((kt & 3) == 3) umma_commit(empty_bar((kt >> 2) % kSuper));        // the super-stage of the weight ring
                    if (kt % kGB == kGB - 1) umma_commit(bempty_bar(sb / kGB));            // the group of activation stages
                } else {
                    umma_commit(empty_bar(s));
                    if constexpr (BTMA) umma_commit(bempty_bar(sb));
                }
                if (kt == (kIssuers > 1 ? 4 * (which + kIssuers * (supers_mine - 1)) + 3 : ktiles - 1)) umma_commit(accum_bar);   // this issuer's last k-tile
            }
            __syncwarp();
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");              // (returns at once by now) status may be shared
    if (!ok && status != nullptr) atomicExch(status, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// x as a plain [M][K] fp16 matrix, box = [BM tokens][64 consecutive halfs] (128 bytes per token row).
static bool make_x_map(CUtensorMap* map, const void* x, int M, int K, int bm) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2u};
    const cuuint32_t box[2] = {64u, (cuuint32_t)bm};
    const cuuint32_t estr[2] = {1u, 1u};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// planes 0..w-1 as [w][N][K/32] int32, box = [w][128 rows][8 words] (one super-tile of a block of rows)
static bool make_q_map(CUtensorMap* map, const void* q, long long plane_stride, int N, int K, int w_bits, int box_words = 8,
                       bool swizzled = false) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)(K / 32), (cuuint64_t)N, (cuuint64_t)w_bits};
    const cuuint64_t strides[2] = {(cuuint64_t)(K / 32) * 4u, (cuuint64_t)plane_stride * 4u};
    const cuuint32_t box[3] = {(cuuint32_t)box_words, (cuuint32_t)kBN, (cuuint32_t)w_bits};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUtensorMapSwizzle swz = !swizzled ? CU_TENSOR_MAP_SWIZZLE_NONE
                                  : (box_words == 32 ? CU_TENSOR_MAP_SWIZZLE_128B
                                                     : (box_words == 16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B));
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<void*>(q), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int W, int BM, int TM>
static cudaError_t launch_variant(const CUtensorMap& xmap, const CUtensorMap& qmap, const void* x, const void* q,
                                  long long plane_stride, const void* lut, void* out, int M, int N, int K, int* status,
                                  int splits, float* partials, int* tickets, cudaStream_t stream) {
    const int smem = Smem<W>::total(BM, TM);
    static bool attr_done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        e = cudaFuncSetAttribute(gemm_kbit_tc_kernel<W, BM, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    if (TM == 0 || partials == nullptr || tickets == nullptr || splits < 1) splits = 1;
    const int supers = K / 256;
    if (splits > 1) {                                        // at most 8 ranges, none empty
        if (splits > 8) splits = 8;
        if (splits > supers) splits = supers;
        const int per = (supers + splits - 1) / splits;
        splits = (supers + per - 1) / per;
    }
    dim3 grid(N / kBN, (M + BM - 1) / BM, splits);
    // Programmatic dependent launch: the kernel may start while the previous kernel of the stream drains; it
    // touches nothing that kernel may have written (x, out, the workspace, status) before its dependency wait.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads_for(BM, TM));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_kbit_tc_kernel<W, BM, TM>, xmap, qmap, static_cast<const __half*>(x),
                              static_cast<const uint32_t*>(q), plane_stride, static_cast<const uint16_t*>(lut),
                              static_cast<__half*>(out), M, N, K, status, partials, tickets);
}

template <int W, int BM>
static cudaError_t launch_bm(const void* x, const void* q, long long plane_stride, const void* lut, void* out, int M,
                             int N, int K, int* status, int splits, float* partials, int* tickets, cudaStream_t stream) {
    CUtensorMap xmap = {}, qmap = {};
    if (K % 256 == 0 && make_x_map(&xmap, x, M, K, BM)) {
        // planes by TMA too where the two plane buffers still leave room for three stages
        // weights in tensor memory unless AP_GEMM_A_TMEM=0 asks for the shared-memory variants
        static const bool a_tmem = [] { const char* v = getenv("AP_GEMM_A_TMEM"); return v == nullptr || v[0] != '0'; }();
        if (a_tmem && make_q_map(&qmap, q, plane_stride, N, K, W, Smem<W>::plane_words(BM, 3), true))
            return launch_variant<W, BM, 3>(xmap, qmap, x, q, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
        if constexpr (Smem<W>::stages(BM, true) >= 3) {
            if (make_q_map(&qmap, q, plane_stride, N, K, W))
                return launch_variant<W, BM, 2>(xmap, qmap, x, q, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
        }
        return launch_variant<W, BM, 1>(xmap, qmap, x, q, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
    }
    return launch_variant<W, BM, 0>(xmap, qmap, x, q, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
}

template <int W>
static cudaError_t launch_w(const void* x, const void* q, long long plane_stride, const void* lut, void* out, int M,
                            int N, int K, int* status, int splits, float* partials, int* tickets, cudaStream_t stream) {
    // Every CTA dequantises its 128 weight rows once per k-tile whatever the token block, and that, not
    // the MMA, is what a k-tile costs: the best token block is the largest that the rows need (one
    // block of tokens if 256 hold them), so that no weight is dequantised twice without need; with
    // several blocks of tokens, the largest block that still leaves no more rounds of CTAs.
    int sms = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const int nblk = N / kBN;
    auto rounds = [&](int bm) { return (nblk * ((M + bm - 1) / bm) + sms - 1) / sms; };
    if (M <= 64) return launch_bm<W, 64>(x, q, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
    if (M <= 128) return launch_bm<W, 128>(x, q, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
    if (rounds(256) <= rounds(128)) return launch_bm<W, 256>(x, q, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
    return launch_bm<W, 128>(x, q, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
}

}  // namespace tc

bool gemm_tc_supported(const void* x, const void* qweight, long long plane_stride, const void* lut, const void* out,
                       int M, int N, int K) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(lut) |
                           reinterpret_cast<uintptr_t>(qweight)) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 1) == 0;
    return aligned && M >= 1 && N % tc::kBN == 0 && K % 128 == 0 && plane_stride % 4 == 0;
}

int gemm_tc_suggested_splits(int M, int N, int K) {
    // K ranges per block of rows so that the grid has about one thread block per SM; only the TMA variants split
    if (K % 256 != 0 || N % tc::kBN != 0 || M > 256) return 1;
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int bm = M <= 64 ? 64 : (M <= 128 ? 128 : 256);
    const int ctas = (N / tc::kBN) * ((M + bm - 1) / bm);
    int splits = sms / (ctas > 0 ? ctas : 1);
    if (splits > 8) splits = 8;
    if (splits > K / 256) splits = K / 256;
    return splits < 2 ? 1 : splits;
}

cudaError_t launch_gemm_tc(const void* x, const void* qweight, long long plane_stride, const void* lut, void* out, int M,
                           int N, int K, int w_bits, int* status, int splits, float* partials, int* tickets,
                           cudaStream_t stream) {
    switch (w_bits) {
        case 3: return tc::launch_w<3>(x, qweight, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
        case 4: return tc::launch_w<4>(x, qweight, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
        case 5: return tc::launch_w<5>(x, qweight, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
        case 6: return tc::launch_w<6>(x, qweight, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
        case 7: return tc::launch_w<7>(x, qweight, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
        case 8: return tc::launch_w<8>(x, qweight, plane_stride, lut, out, M, N, K, status, splits, partials, tickets, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ap
