// Seed + incremental-upscale quantisation of a weight matrix on the GPU: one thread block per row.
//
// Replaces the reference's CPU path any_precision/quantization/quantize.py:85-187
// (_seed_and_upscale_layer: numba, one row per CPU thread) together with :13-76 (_upscale_group,
// _increment_group) and the two 1-D k-means routines it takes from the flash1dkmeans package:
//   1. sample weight = sensitivity, zero where the weight is zero (:118-120);
//   2. sort the row by value, keeping equal values in their original order (:124-128);
//   3. fp64 inclusive prefix sums of w and w * x over the sorted row; a row whose sample weights sum
//      to zero is treated as unweighted (:130-143);
//   4. 2^seed_bit clusters by 1-D k-means on the prefix sums: a start of equal weight mass, then Lloyd
//      iterations (a value goes left of a midpoint if it is <= it) until the borders repeat or max_iter
//      assignments were made (:145-157; the package starts from a random k-means++ draw instead, so
//      its result is not reproducible and not reproduced);
//   5. for every further bit every cluster is split in two: the split is the first position whose value
//      lies above the midpoint of the two sides' weighted means, found by binary search; an empty
//      cluster hands its centroid to both children (:43-74).  Tables are fp32 at every level and fp16
//      when stored (:157,:205-207);
//   6. the parent-precision cluster index of every weight, in its original position, is its code
//      (:171-180).
// The arithmetic is written with explicit round-to-nearest fp64 intrinsics so that no multiply-add is
// fused, and the prefix sums add in a fixed blocked order (1024 runs of consecutive positions, each left
// to right, then the runs' totals left to right, then offset + local sum):
// the CPU checker restates exactly this order and the results agree bit for bit.
//
// Shared memory: the sort keys (4 bytes) and original positions (2 bytes) of the row padded to a
// power of two, at most 32768 values (192 KB); the prefix sums (16 bytes per value) live in a
// per-block slice of a caller-provided workspace and are read back through L2 by the binary searches.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/anyprec_b200.h"

namespace {

constexpr int kRuns = 1024;                                // runs of the blocked prefix sums (fixed: it defines the rounding)
constexpr int kMaxClusters = 256;

__device__ __forceinline__ uint32_t key_of(float x) {
    const uint32_t u = __float_as_uint(__fadd_rn(x, 0.0f));          // -0.0 sorts (and counts) as 0.0
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float val_of(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// (the prefix sums were written by this block a few steps earlier: plain cached-in-L2 loads, never the
// read-only path)
__device__ __forceinline__ double range_sum(const double* prefix, int a, int b) {
    if (b <= a) return 0.0;
    const double hi = __ldcg(prefix + b - 1);
    return a > 0 ? __dsub_rn(hi, __ldcg(prefix + a - 1)) : hi;
}

// start + number of sorted values in [start, stop) that are <= v
__device__ __forceinline__ int count_le(const uint32_t* keys, int start, int stop, double v) {
    int lo = start, hi = stop;
    while (lo < hi) {
        const int m = (lo + hi) >> 1;
        if ((double)val_of(keys[m]) <= v) lo = m + 1;
        else hi = m;
    }
    return lo;
}

// Split of the non-empty cluster [start, stop): centroids of the two sides and the split position.  The sums over
// [start, d) and [d, stop) are prefix[d - 1] - prefix[start - 1] and prefix[stop - 1] - prefix[d - 1]: the two ends
// are read once, and every step of the search has its two loads (weights, weights * values at d - 1) in flight
// together, one trip to L2 per step.
__device__ void two_cluster(const uint32_t* keys, const double* wp, const double* wxp, int start, int stop, double& c0,
                            double& c1, int& division) {
    if (stop - start == 1) {
        c0 = c1 = (double)val_of(keys[start]);
        division = stop;
        return;
    }
    const double w_lo = start > 0 ? __ldcg(wp + start - 1) : 0.0, x_lo = start > 0 ? __ldcg(wxp + start - 1) : 0.0;
    const double w_hi = __ldcg(wp + stop - 1), x_hi = __ldcg(wxp + stop - 1);
    // sums of [start, d) and [d, stop) from the prefix values at d - 1 (d > start, so d - 1 >= 0)
    auto left = [&](double at, double lo) { return start > 0 ? __dsub_rn(at, lo) : at; };
    int lo = start + 1, hi = stop - 1;
    while (lo < hi) {
        const int d = (lo + hi) >> 1;
        const double w_at = __ldcg(wp + d - 1), x_at = __ldcg(wxp + d - 1);
        const double wl = left(w_at, w_lo), wr = __dsub_rn(w_hi, w_at);
        bool move_right;
        if (wl <= 0.0) move_right = true;
        else if (wr <= 0.0) move_right = false;
        else {
            const double mid = __dmul_rn(__dadd_rn(__ddiv_rn(left(x_at, x_lo), wl), __ddiv_rn(__dsub_rn(x_hi, x_at), wr)), 0.5);
            move_right = (double)val_of(keys[d]) <= mid;
        }
        if (move_right) lo = d + 1;
        else hi = d;
    }
    const int d = lo;
    const double w_at = __ldcg(wp + d - 1), x_at = __ldcg(wxp + d - 1);
    const double wl = left(w_at, w_lo), wr = __dsub_rn(w_hi, w_at);
    c0 = wl > 0.0 ? __ddiv_rn(left(x_at, x_lo), wl) : (double)val_of(keys[d - 1]);
    c1 = wr > 0.0 ? __ddiv_rn(__dsub_rn(x_hi, x_at), wr) : (double)val_of(keys[d]);
    division = d;
}

// THREADS: 1024, one block per SM, or 512, two per SM, for rows short enough that two fit the shared memory: most
// of a row's time is spent in steps that keep one thread per cluster busy and wait on L2, which a second block
// overlaps.
template <int THREADS>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS)
seed_upscale_kernel(const float* __restrict__ weight, const float* __restrict__ sens, int N, int K, int Kpad, int seed_bit,
                    int parent_bit, int max_iter, uint8_t* __restrict__ codes, __half* __restrict__ luts, double* __restrict__ work) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint32_t* keys = reinterpret_cast<uint32_t*>(smem);
    uint16_t* idx = reinterpret_cast<uint16_t*>(smem + (size_t)Kpad * 4);
    constexpr int kThreads = THREADS;
    static_assert(THREADS > kMaxClusters && kRuns % THREADS == 0, "one thread per cluster border; whole runs per thread");
    double* tot = reinterpret_cast<double*>(smem + (size_t)Kpad * 6);           // [3][kRuns]: w, w * x, x
    double* cent = tot + 3 * kRuns;                                              // [kMaxClusters]
    float* level = reinterpret_cast<float*>(cent + kMaxClusters);                // [2][kMaxClusters] fp32 tables
    int* bord = reinterpret_cast<int*>(level + 2 * kMaxClusters);                // [2][kMaxClusters + 4]
    constexpr int kBordStride = kMaxClusters + 4;
    const int tid = threadIdx.x;
    double* wp = work + (size_t)blockIdx.x * 2 * K;
    double* wxp = wp + K;
    const int run = (K + kRuns - 1) / kRuns;                 // positions per run; run r is [r * run, (r + 1) * run) cut at K

    for (int row = blockIdx.x; row < N; row += gridDim.x) {
        const float* xr = weight + (size_t)row * K;
        const float* sr = sens + (size_t)row * K;
        // ---- 2. sort (value, original position) ascending: bitonic network over the padded row
        for (int i = tid; i < Kpad; i += kThreads) {
            keys[i] = i < K ? key_of(xr[i]) : 0xFFFFFFFFu;
            idx[i] = (uint16_t)i;
        }
        __syncthreads();
        for (int k = 2; k <= Kpad; k <<= 1) {
            for (int j = k >> 1; j > 0; j >>= 1) {
                for (int t = tid; t < (Kpad >> 1); t += kThreads) {
                    const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1)), l = i + j;
                    const uint32_t ka = keys[i], kb = keys[l];
                    const uint16_t ia = idx[i], ib = idx[l];
                    const bool gt = ka > kb || (ka == kb && ia > ib);
                    if (gt == ((i & k) == 0)) {
                        keys[i] = kb; keys[l] = ka;
                        idx[i] = ib; idx[l] = ia;
                    }
                }
                __syncthreads();
            }
        }
        // ---- 3. prefix sums: totals of every thread's run, their exclusive scan, then offset + local sum
        for (int r = tid; r < kRuns; r += kThreads) {
            const int r0 = r * run < K ? r * run : K, r1 = (r + 1) * run < K ? (r + 1) * run : K;
            double tw = 0.0, twx = 0.0, tx = 0.0;
            for (int e = r0; e < r1; e++) {
                const float x = val_of(keys[e]);
                const float w = __fmul_rn(sr[idx[e]], x != 0.0f ? 1.0f : 0.0f);
                tw = __dadd_rn(tw, (double)w);
                twx = __dadd_rn(twx, __dmul_rn((double)x, (double)w));
                tx = __dadd_rn(tx, (double)x);
            }
            tot[r] = tw;
            tot[kRuns + r] = twx;
            tot[2 * kRuns + r] = tx;
        }
        __syncthreads();
        if (tid < 3) {
            double acc = 0.0;
            double* t = tot + tid * kRuns;
            for (int i = 0; i < kRuns; i++) {
                const double v = t[i];
                t[i] = acc;
                acc = __dadd_rn(acc, v);
            }
            if (tid == 0) cent[0] = acc;                     // the row's total sample weight
        }
        __syncthreads();
        const bool unweighted = cent[0] == 0.0;
        __syncthreads();
        for (int r = tid; r < kRuns; r += kThreads) {
            const int r0 = r * run < K ? r * run : K, r1 = (r + 1) * run < K ? (r + 1) * run : K;
            double lw = 0.0, lwx = 0.0;
            const double ow = tot[r], owx = unweighted ? tot[2 * kRuns + r] : tot[kRuns + r];
            for (int e = r0; e < r1; e++) {
                const float x = val_of(keys[e]);
                if (unweighted) {
                    lwx = __dadd_rn(lwx, (double)x);
                    wp[e] = (double)(e + 1);
                } else {
                    const float w = __fmul_rn(sr[idx[e]], x != 0.0f ? 1.0f : 0.0f);
                    lw = __dadd_rn(lw, (double)w);
                    lwx = __dadd_rn(lwx, __dmul_rn((double)x, (double)w));
                    wp[e] = __dadd_rn(ow, lw);
                }
                wxp[e] = __dadd_rn(owx, lwx);
            }
        }
        __syncthreads();
        // ---- 4. seed clusters
        const int k0 = 1 << seed_bit;
        int* b_cur = bord;
        int* b_new = bord + kBordStride;
        const double total = __ldcg(wp + K - 1);
        if (tid <= k0) {
            int b = tid == 0 ? 0 : K;
            if (tid > 0 && tid < k0) {
                const double target = __ddiv_rn(__dmul_rn(total, (double)tid), (double)k0);
                int lo = 0, hi = K;
                while (lo < hi) {
                    const int m = (lo + hi) >> 1;
                    if (__ldcg(wp + m) <= target) lo = m + 1;
                    else hi = m;
                }
                b = lo;
            }
            b_new[tid] = b;
        }
        __syncthreads();
        if (tid <= k0) {                                     // borders never step back
            int b = b_new[0];
            for (int j = 1; j <= tid; j++) b = b_new[j] > b ? b_new[j] : b;
            b_cur[tid] = tid == k0 ? K : b;
        }
        __syncthreads();
        if (tid < k0) {
            const int a = b_cur[tid], b = b_cur[tid + 1];
            const double ws = range_sum(wp, a, b), xs = range_sum(wxp, a, b);       // both requested together
            cent[tid] = ws > 0.0 ? __ddiv_rn(xs, ws) : (double)val_of(keys[a < K - 1 ? a : K - 1]);
        }
        __syncthreads();
        for (int it = 0; it < max_iter; it++) {
            if (tid <= k0) {
                int b = tid == 0 ? 0 : K;
                if (tid > 0 && tid < k0) b = count_le(keys, 0, K, __dmul_rn(__dadd_rn(cent[tid - 1], cent[tid]), 0.5));
                b_new[tid] = b;
            }
            __syncthreads();
            int mine = 0;
            bool same = true;
            if (tid <= k0) {
                mine = b_new[0];
                for (int j = 1; j <= tid; j++) mine = b_new[j] > mine ? b_new[j] : mine;
                if (tid == k0) mine = K;
                same = mine == b_cur[tid];
            }
            if (__syncthreads_and(same)) break;
            if (tid <= k0) b_cur[tid] = mine;
            __syncthreads();
            if (tid < k0) {
                const int a = b_cur[tid], b = b_cur[tid + 1];
                const double ws = range_sum(wp, a, b), xs = range_sum(wxp, a, b);
                if (ws > 0.0) cent[tid] = __ddiv_rn(xs, ws);
            }
            __syncthreads();
        }
        // ---- 5. tables: the seed level, then one split of every cluster per further bit
        float* l_cur = level;
        float* l_new = level + kMaxClusters;
        size_t lut_off = 0;                                  // halfs before this level's [N][2^bit] table
        if (tid < k0) {
            const float c = __double2float_rn(cent[tid]);
            l_cur[tid] = c;
            luts[lut_off + (size_t)row * k0 + tid] = __float2half_rn(c);
        }
        __syncthreads();
        for (int bit = seed_bit; bit < parent_bit; bit++) {
            const int kc = 1 << bit;
            lut_off += (size_t)N * kc;
            if (tid < kc) {
                const int a = b_cur[tid], b = b_cur[tid + 1];
                float c0, c1;
                int d;
                if (a == b) {
                    c0 = c1 = l_cur[tid];
                    d = a;
                } else {
                    double d0, d1;
                    two_cluster(keys, wp, wxp, a, b, d0, d1, d);
                    c0 = __double2float_rn(d0);
                    c1 = __double2float_rn(d1);
                }
                l_new[2 * tid] = c0;
                l_new[2 * tid + 1] = c1;
                b_new[2 * tid] = a;
                b_new[2 * tid + 1] = d;
                if (tid == kc - 1) b_new[2 * kc] = K;
                __half2 h = __floats2half2_rn(c0, c1);
                *reinterpret_cast<__half2*>(luts + lut_off + (size_t)row * 2 * kc + 2 * tid) = h;
            }
            __syncthreads();
            float* lt = l_cur; l_cur = l_new; l_new = lt;
            int* bt = b_cur; b_cur = b_new; b_new = bt;
        }
        // ---- 6. codes: sorted position i lies in the cluster c with b[c] <= i < b[c + 1]
        const int kp = 1 << parent_bit;
        uint8_t* cr = codes + (size_t)row * K;
        for (int i = tid; i < K; i += kThreads) {
            int lo = 0, hi = kp;                             // last c in [0, kp) with b[c] <= i
            while (lo < hi) {
                const int m = (lo + hi + 1) >> 1;
                if (m < kp && b_cur[m] <= i) lo = m;
                else hi = m - 1;
            }
            cr[idx[i]] = (uint8_t)lo;
        }
        __syncthreads();
    }
}

size_t smem_bytes(int Kpad) {
    return (size_t)Kpad * 6 + 3 * kRuns * sizeof(double) + kMaxClusters * sizeof(double) + 2 * kMaxClusters * sizeof(float) +
           2 * (kMaxClusters + 4) * sizeof(int);
}

int padded(int K) {
    int p = 8;                                               // keeps the arrays behind the keys 8-byte aligned
    while (p < K) p <<= 1;
    return p;
}

}  // namespace

extern "C" size_t ap_seed_upscale_workspace_bytes(int K, int blocks) {
    if (K < 1 || blocks < 1) return 0;
    return (size_t)blocks * 2 * K * sizeof(double);
}

extern "C" int ap_seed_upscale(const void* weight, const void* sensitivity, int N, int K, int seed_bits, int parent_bits,
                               int max_iter, void* codes, void* luts, void* workspace, size_t workspace_bytes, void* stream) {
    if (!weight || !sensitivity || !codes || !luts || !workspace) return AP_ERR_NULL_POINTER;
    if (seed_bits < 1 || parent_bits > 8 || seed_bits > parent_bits) return AP_ERR_BAD_BITS;
    if (N < 1 || K < 1 || max_iter < 0) return AP_ERR_BAD_SHAPE;
    if (K > 32768) return AP_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(sensitivity) | reinterpret_cast<uintptr_t>(luts)) & 3)
        return AP_ERR_BAD_ALIGNMENT;
    if (reinterpret_cast<uintptr_t>(workspace) & 7) return AP_ERR_BAD_ALIGNMENT;
    const size_t per_block = (size_t)2 * K * sizeof(double);
    size_t blocks = workspace_bytes / per_block;
    if (blocks < 1) return AP_ERR_BAD_SHAPE;
    if (blocks > (size_t)N) blocks = N;
    const int Kpad = padded(K);
    const size_t smem = smem_bytes(Kpad);
    // two blocks of 512 threads per SM where two rows fit the shared memory (with all of it carved out for shared
    // memory: the driver's default carve-out left room for one)
    const bool two = 2 * (smem + 1024) <= 227 * 1024;
    auto kernel = two ? seed_upscale_kernel<512> : seed_upscale_kernel<1024>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return AP_ERR_LAUNCH;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return AP_ERR_LAUNCH;
    kernel<<<(unsigned)blocks, two ? 512 : 1024, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(weight), static_cast<const float*>(sensitivity), N, K, Kpad, seed_bits, parent_bits, max_iter,
        static_cast<uint8_t*>(codes), static_cast<__half*>(luts), static_cast<double*>(workspace));
    return cudaGetLastError() == cudaSuccess ? AP_OK : AP_ERR_LAUNCH;
}
