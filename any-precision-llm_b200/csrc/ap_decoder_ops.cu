// Small element-wise kernels around the linear layers of a decoder step, so that a decode step is
// a handful of launches per layer instead of dozens of framework kernels: the any-precision GEMVs
// of a 7B model take a few microseconds each, and everything between them is launch-bound.
//
// The reference leaves these operations to Hugging Face's LlamaDecoderLayer (its model wrapper,
// any_precision/modules/AnyPrecisionForCausalLM.py:54-60, builds the stock model and swaps only the
// linears); its own fuse_layers is an unimplemented stub (:186-190).  Nothing here has a counterpart
// in the reference's kernels.
//
//   ap_add_rmsnorm   h += delta (optional), y = h * rsqrt(mean(h^2) + eps) * weight      one block per row
//   ap_rope_cache    rotary embedding of q and k at each row's position, k and v written into the
//                    KV cache at that position                                           one block per row
//   ap_silu_mul      y = silu(gate) * up for gate|up side by side or tile by tile         grid-stride
//   ap_decode_attention  (and ap_decode_attention_rope, which rotates q and k and writes the cache itself)
//                    one query per sequence against its KV cache up to the query's position
//                    (grouped-query heads), softmax in fp32                              one block per (head, sequence)
// All fp16 in and out with fp32 arithmetic.  Positions come from device memory, so that a captured
// CUDA graph can be replayed for every step of a generation.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/anyprec_b200.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(1024)
add_rmsnorm_kernel(__half* __restrict__ h, const __half* __restrict__ delta, const __half* __restrict__ weight,
                   __half* __restrict__ y, int hidden, float eps) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int kKeep = 8;                                 // half2 values a thread keeps in registers (hidden <= 16384)
    const int row = blockIdx.x, nthr = blockDim.x;
    __half* hr = h + (size_t)row * hidden;
    const __half* dr = delta ? delta + (size_t)row * hidden : nullptr;
    __shared__ float part[32];
    __half2 keep[kKeep];
    float ss = 0.f;
    // Every load of the row is issued before anything is reduced: the kernel is one memory round trip,
    // a block reduction and one store, which is what a microsecond-scale launch can afford.
#pragma unroll
    for (int k = 0; k < kKeep; k++) {
        const int i = (threadIdx.x + k * nthr) * 2;
        if (i < hidden) {
            __half2 v = *reinterpret_cast<const __half2*>(hr + i);
            if (dr) {
                const float2 a = __half22float2(v), d = __half22float2(*reinterpret_cast<const __half2*>(dr + i));
                v = __floats2half2_rn(a.x + d.x, a.y + d.y);
                *reinterpret_cast<__half2*>(hr + i) = v;    // the updated residual stream
            }
            keep[k] = v;
            const float2 f = __half22float2(v);
            ss += f.x * f.x + f.y * f.y;
        }
    }
    for (int i = (threadIdx.x + kKeep * nthr) * 2; i < hidden; i += nthr * 2) {      // rows longer than the registers hold
        __half2 v = *reinterpret_cast<const __half2*>(hr + i);
        if (dr) {
            const float2 a = __half22float2(v), d = __half22float2(*reinterpret_cast<const __half2*>(dr + i));
            v = __floats2half2_rn(a.x + d.x, a.y + d.y);
            *reinterpret_cast<__half2*>(hr + i) = v;
        }
        const float2 f = __half22float2(v);
        ss += f.x * f.x + f.y * f.y;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < (nthr >> 5); w++) tot += part[w];
    const float scale = rsqrtf(tot / (float)hidden + eps);
    auto emit = [&](int i, __half2 v) {
        const float2 f = __half22float2(v);
        const float2 g = __half22float2(*reinterpret_cast<const __half2*>(weight + i));
        // the same rounding order as the usual formulation: normalise, round to fp16, scale
        const float2 nf = __half22float2(__floats2half2_rn(f.x * scale, f.y * scale));
        *reinterpret_cast<__half2*>(y + (size_t)row * hidden + i) = __floats2half2_rn(nf.x * g.x, nf.y * g.y);
    };
#pragma unroll
    for (int k = 0; k < kKeep; k++) {
        const int i = (threadIdx.x + k * nthr) * 2;
        if (i < hidden) emit(i, keep[k]);
    }
    for (int i = (threadIdx.x + kKeep * nthr) * 2; i < hidden; i += nthr * 2) emit(i, *reinterpret_cast<const __half2*>(hr + i));
}

// One rotated pair (x[i], x[i + head_dim / 2]) -> (a c - b s, b c + a s), every product and sum rounded on its
// own so that the stand-alone kernel and the attention kernel that rotates on the fly give the same bits.
__device__ __forceinline__ float rot_lo(float a, float b, float c, float s) { return __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)); }
__device__ __forceinline__ float rot_hi(float a, float b, float c, float s) { return __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s)); }

// qkv: [rows][(heads + 2 kv_heads) * head_dim] = q | k | v of one token per row.  Rotates q in place
// (pairs (i, i + head_dim/2), the "rotate half" convention) and writes rotated k and plain v into the
// caches [sequences][kv_heads][max_seq][head_dim] at position pos[row] of sequence row / rows_per_seq.
__global__ void __launch_bounds__(128)
rope_cache_kernel(__half* __restrict__ qkv, const float* __restrict__ cos_sin, const int* __restrict__ pos,
                  __half* __restrict__ k_cache, __half* __restrict__ v_cache, int heads, int kv_heads, int head_dim,
                  int max_seq, int rows_per_seq) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // one block per (head slot, row): q heads, then k heads, then v heads; a thread per rotated pair
    const int slot = blockIdx.x, row = blockIdx.y;
    const int seq = row / rows_per_seq;
    const int p = pos[row];
    if (p < 0 || p >= max_seq) return;                       // out of range: leave everything untouched
    const int half_dim = head_dim >> 1;
    __half* base = qkv + (size_t)row * (heads + 2 * kv_heads) * head_dim + (size_t)slot * head_dim;
    if (slot < heads + kv_heads) {
        const float* cs = cos_sin + (size_t)p * head_dim;    // [cos(half_dim) | sin(half_dim)] of position p
        for (int i = threadIdx.x; i < half_dim; i += blockDim.x) {
            const float a = __half2float(base[i]), b = __half2float(base[i + half_dim]);
            const float c = cs[i], s = cs[half_dim + i];
            const __half ra = __float2half_rn(rot_lo(a, b, c, s)), rb = __float2half_rn(rot_hi(a, b, c, s));
            if (slot < heads) {
                base[i] = ra;
                base[i + half_dim] = rb;
            } else {
                __half* dst = k_cache + (((size_t)seq * kv_heads + (slot - heads)) * max_seq + p) * head_dim;
                dst[i] = ra;
                dst[i + half_dim] = rb;
            }
        }
    } else {
        __half* dst = v_cache + (((size_t)seq * kv_heads + (slot - heads - kv_heads)) * max_seq + p) * head_dim;
        for (int i = threadIdx.x; i < head_dim; i += blockDim.x) dst[i] = base[i];
    }
}

__global__ void __launch_bounds__(256)
silu_mul_kernel(const __half* __restrict__ gate_up, __half* __restrict__ y, int rows, int ffn, int tiled) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t total = (size_t)rows * ffn / 2;
    for (size_t it = blockIdx.x * (size_t)blockDim.x + threadIdx.x; it < total; it += (size_t)gridDim.x * blockDim.x) {
        const size_t row = (it * 2) / ffn, i = (it * 2) % ffn;
        // gate | up side by side, or (tiled) eight gate then eight up values of the same features in every 16
        const size_t gi = tiled ? (i >> 3) * 16 + (i & 7) : i, ui = tiled ? gi + 8 : ffn + i;
        const float2 g = __half22float2(*reinterpret_cast<const __half2*>(gate_up + row * 2 * ffn + gi));
        const float2 u = __half22float2(*reinterpret_cast<const __half2*>(gate_up + row * 2 * ffn + ui));
        // silu in fp32, rounded to fp16 before the product, as a framework would evaluate act(gate) * up
        const __half2 a = __floats2half2_rn(g.x / (1.f + __expf(-g.x)), g.y / (1.f + __expf(-g.y)));
        const float2 af = __half22float2(a);
        *reinterpret_cast<__half2*>(y + row * ffn + i) = __floats2half2_rn(af.x * u.x, af.y * u.y);
    }
}

// One query token per sequence: out[b][h] = softmax(q[b][h] . K[b][kv(h)][0..pos[b]] * scale) V[b][kv(h)][0..pos[b]].
// The cached positions of a (head, sequence) are cut into gridDim.z ranges, one block of 256 threads each: a
// decode step has few heads (32 for a 7B model at batch 1) and a single SM pulls a head's K and V far too
// slowly, so the ranges give every SM a share.  Scores: one position per thread (its whole K row with 16-byte
// loads, all in flight at once), so no shuffles per position; block maximum and sum; then the weighted V sum
// with eight head elements per thread and the range's positions dealt over 256 / (D / 8) groups of threads.
// Each block parks (maximum, sum, unnormalised vector) in `scratch`; the block that draws the last ticket of a
// (head, sequence) merges the ranges in index order, writes fp16 and hands the ticket back at zero.  fp32
// throughout.
//
// ROPE: the rows of `qkv` are the raw q | k | v of the new token (position pos[b]), the caches hold the earlier
// positions only.  The block rotates its q on the fly; the one thread that owns position pos[b] takes k from
// `qkv`, rotates it and (in the first query head of a KV group) stores it in the cache; v of that position is
// read from `qkv` and stored likewise.  No block reads position pos[b] from the caches, so the writes race with
// nothing in this launch.  Rounding as in rope_cache_kernel followed by the plain kernel.
template <int D, bool ROPE>
__global__ void __launch_bounds__(256)
decode_attention_kernel(const __half* __restrict__ qkv, int q_row_stride, const __half* k_cache, const __half* v_cache,
                        const int* __restrict__ pos, __half* __restrict__ out, int heads, int kv_heads, int max_seq, float scale,
                        float* __restrict__ scratch, int* __restrict__ tickets, const float* __restrict__ cos_sin,
                        __half* k_cache_w, __half* v_cache_w) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int kThreads = 256, kTile = kThreads;
    constexpr int kDT = D / 8;                               // threads across the head dimension (eight elements each)
    constexpr int kGroups = kThreads / kDT;                  // position groups in the V phase
    static_assert(D % 8 == 0 && kThreads % kDT == 0 && D <= kThreads, "head dimension");
    const int h = blockIdx.x, b = blockIdx.y, z = blockIdx.z, S = gridDim.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int n = pos[b] + 1;
    n = n < 0 ? 0 : (n > max_seq ? max_seq : n);
    const int per = (n + S - 1) / S;
    const int p_begin = z * per, p_end = (p_begin + per < n) ? (p_begin + per) : n;
    const int kvh = h / (heads / kv_heads);
    const __half* kb = k_cache + ((size_t)b * kv_heads + kvh) * max_seq * D;
    const __half* vb = v_cache + ((size_t)b * kv_heads + kvh) * max_seq * D;
    __shared__ float sq[D];
    __shared__ __align__(16) __half sk[D];                   // ROPE: the new token's rotated k
    __shared__ float sw[kTile];
    __shared__ float red[8];
    __shared__ float sacc[kGroups][D];
    __shared__ int s_last;
    // the new token's position, if this launch brings it along and it lies inside the cache
    const int pn = (ROPE && pos[b] >= 0 && pos[b] < max_seq) ? pos[b] : -1;
    const bool writer = ROPE && (h % (heads / kv_heads)) == 0;
    const __half* vraw = qkv + (size_t)b * q_row_stride + (size_t)(heads + kv_heads + kvh) * D;
    if (ROPE && pn >= 0) {
        const float* cs = cos_sin + (size_t)pn * D;
        const __half* qr = qkv + (size_t)b * q_row_stride + (size_t)h * D;
        for (int i = tid; i < D; i += kThreads) {
            const int j = i < D / 2 ? i : i - D / 2;
            const float a = __half2float(qr[j]), bq = __half2float(qr[j + D / 2]);
            const float r = i < D / 2 ? rot_lo(a, bq, cs[j], cs[D / 2 + j]) : rot_hi(a, bq, cs[j], cs[D / 2 + j]);
            sq[i] = __half2float(__float2half_rn(r)) * scale;
        }
        if (pn >= p_begin && pn < p_end) {                   // this block's range holds the new position
            const __half* kraw = qkv + (size_t)b * q_row_stride + (size_t)(heads + kvh) * D;
            for (int i = tid; i < D / 2; i += kThreads) {
                const float a = __half2float(kraw[i]), bk = __half2float(kraw[i + D / 2]);
                sk[i] = __float2half_rn(rot_lo(a, bk, cs[i], cs[D / 2 + i]));
                sk[i + D / 2] = __float2half_rn(rot_hi(a, bk, cs[i], cs[D / 2 + i]));
            }
        }
    } else {
        for (int i = tid; i < D; i += kThreads) sq[i] = __half2float(qkv[(size_t)b * q_row_stride + (size_t)h * D + i]) * scale;
    }
    __syncthreads();
    if (ROPE && writer && pn >= p_begin && pn < p_end && tid < D / 8) {
        const size_t at = (((size_t)b * kv_heads + kvh) * max_seq + pn) * D;
        reinterpret_cast<uint4*>(k_cache_w + at)[tid] = reinterpret_cast<const uint4*>(sk)[tid];
        reinterpret_cast<uint4*>(v_cache_w + at)[tid] = reinterpret_cast<const uint4*>(vraw)[tid];
    }
    const int dt = tid % kDT, grp = tid / kDT;
    float m = -INFINITY, l = 0.f;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int t0 = p_begin; t0 < p_end; t0 += kTile) {
        const int p = t0 + tid;
        const int cnt = (p_end - t0 < kTile) ? (p_end - t0) : kTile;
        // This thread's V rows are requested together with its K row when they are few enough to wait in
        // registers (the usual case: a range of at most kPre * kGroups positions), so that the kernel is one
        // round trip to memory rather than two.
        constexpr int kPre = 6;
        const bool pre = cnt <= kPre * kGroups;
        uint4 vpre[kPre];
        float s = -INFINITY;
        uint4 kv[D / 8];
        if (ROPE && p == pn && p < p_end) {                  // the new token's rotated k waits in shared memory
#pragma unroll
            for (int i = 0; i < D / 8; i++) kv[i] = reinterpret_cast<const uint4*>(sk)[i];
        } else if (p < p_end) {
            const uint4* row = reinterpret_cast<const uint4*>(kb + (size_t)p * D);
#pragma unroll
            for (int i = 0; i < D / 8; i++) kv[i] = row[i];
        }
        // row of v at cached position q2: the new token's comes from `qkv`
        auto v_row = [&](int q2) {
            return reinterpret_cast<const uint4*>((ROPE && q2 == pn) ? vraw + 8 * dt : vb + (size_t)q2 * D + 8 * dt);
        };
        if (pre) {
#pragma unroll
            for (int i = 0; i < kPre; i++) {
                const int j = grp + i * kGroups;
                vpre[i] = (j < cnt) ? *v_row(t0 + j) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
        if (p < p_end) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < D / 8; i++) {
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&kv[i].x));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&kv[i].y));
                const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&kv[i].z));
                const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&kv[i].w));
                a += sq[8 * i] * f0.x + sq[8 * i + 1] * f0.y + sq[8 * i + 2] * f1.x + sq[8 * i + 3] * f1.y +
                     sq[8 * i + 4] * f2.x + sq[8 * i + 5] * f2.y + sq[8 * i + 6] * f3.x + sq[8 * i + 7] * f3.y;
            }
            s = a;
        }
        float tm = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
        if (lane == 0) red[warp] = tm;
        __syncthreads();
        tm = red[0];
#pragma unroll
        for (int w2 = 1; w2 < 8; w2++) tm = fmaxf(tm, red[w2]);
        const float m_new = fmaxf(m, tm);
        const float corr = (m == -INFINITY) ? 0.f : __expf(m - m_new);
        const float w = (p < p_end) ? __expf(s - m_new) : 0.f;
        sw[tid] = w;
        float ts = warp_sum(w);
        __syncthreads();                                     // red[] has been read by everybody
        if (lane == 0) red[warp] = ts;
        __syncthreads();                                     // sw[] and the warp sums are complete
        ts = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < 8; w2++) ts += red[w2];
        l = l * corr + ts;
        m = m_new;
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] *= corr;
        auto add_row = [&](const uint4& v, float wj) {
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
            const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
            const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
            acc[0] += wj * f0.x; acc[1] += wj * f0.y; acc[2] += wj * f1.x; acc[3] += wj * f1.y;
            acc[4] += wj * f2.x; acc[5] += wj * f2.y; acc[6] += wj * f3.x; acc[7] += wj * f3.y;
        };
        if (pre) {
#pragma unroll
            for (int i = 0; i < kPre; i++) {
                const int j = grp + i * kGroups;
                if (j < cnt) add_row(vpre[i], sw[j]);
            }
        } else {
#pragma unroll 4
            for (int j = grp; j < cnt; j += kGroups) add_row(*v_row(t0 + j), sw[j]);
        }
        __syncthreads();                                     // sw[] and red[] are rewritten by the next tile
    }
#pragma unroll
    for (int i = 0; i < 8; i++) sacc[grp][8 * dt + i] = acc[i];
    __syncthreads();
    float o = 0.f;
    if (tid < D)
        for (int g2 = 0; g2 < kGroups; g2++) o += sacc[g2][tid];
    __half* dst = out + ((size_t)b * heads + h) * D;
    if (S == 1) {
        if (tid < D) dst[tid] = __float2half_rn(l > 0.f ? o / l : 0.f);
        return;
    }
    // park this range's (m, l, vector); the last block of the (head, sequence) merges all ranges in index order
    float* mine = scratch + (((size_t)b * heads + h) * S + z) * (D + 2);
    if (tid < D) __stcg(mine + 2 + tid, o);
    if (tid == 0) { __stcg(mine, m); __stcg(mine + 1, l); }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(tickets + b * heads + h, 1) == S - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* all = scratch + ((size_t)b * heads + h) * S * (D + 2);
    // running merge in range order: every load is independent of the others, so they overlap
    float mm = -INFINITY, tot = 0.f, val = 0.f;
    for (int r = 0; r < S; r++) {
        const float mr = __ldcg(all + (size_t)r * (D + 2)), lr = __ldcg(all + (size_t)r * (D + 2) + 1);
        const float vr = (tid < D) ? __ldcg(all + (size_t)r * (D + 2) + 2 + tid) : 0.f;
        const float m2 = fmaxf(mm, mr);
        const float fa = (mm == -INFINITY) ? 0.f : __expf(mm - m2), fb = (mr == -INFINITY) ? 0.f : __expf(mr - m2);
        tot = tot * fa + lr * fb;
        val = val * fa + vr * fb;
        mm = m2;
    }
    if (tid < D) dst[tid] = __float2half_rn(tot > 0.f ? val / tot : 0.f);
    if (tid == 0) tickets[b * heads + h] = 0;
}

template <typename... Args>
cudaError_t launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace

extern "C" int ap_add_rmsnorm(void* h, const void* delta, const void* weight, void* y, int rows, int hidden, float eps,
                              void* stream) {
    if (!h || !weight || !y) return AP_ERR_NULL_POINTER;
    if (rows < 1 || hidden < 2 || hidden % 2) return AP_ERR_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(y) |
         reinterpret_cast<uintptr_t>(delta)) & 3)
        return AP_ERR_BAD_ALIGNMENT;
    const int threads = hidden >= 2048 ? 1024 : (hidden >= 512 ? 256 : 64);
    cudaError_t e = launch_pdl(add_rmsnorm_kernel, dim3(rows), dim3(threads), static_cast<cudaStream_t>(stream),
                               static_cast<__half*>(h), static_cast<const __half*>(delta),
                               static_cast<const __half*>(weight), static_cast<__half*>(y), hidden, eps);
    return e == cudaSuccess ? AP_OK : AP_ERR_LAUNCH;
}

extern "C" int ap_rope_cache(void* qkv, const void* cos_sin, const void* pos, void* k_cache, void* v_cache, int rows,
                             int rows_per_seq, int heads, int kv_heads, int head_dim, int max_seq, void* stream) {
    if (!qkv || !cos_sin || !pos || !k_cache || !v_cache) return AP_ERR_NULL_POINTER;
    if (rows < 1 || rows_per_seq < 1 || heads < 1 || kv_heads < 1 || head_dim < 2 || head_dim % 2 || max_seq < 1)
        return AP_ERR_BAD_SHAPE;
    const int threads = head_dim / 2 >= 128 ? 128 : (head_dim / 2 >= 64 ? 64 : 32);
    cudaError_t e = launch_pdl(rope_cache_kernel, dim3(heads + 2 * kv_heads, rows), dim3(threads), static_cast<cudaStream_t>(stream),
                               static_cast<__half*>(qkv), static_cast<const float*>(cos_sin), static_cast<const int*>(pos),
                               static_cast<__half*>(k_cache), static_cast<__half*>(v_cache), heads, kv_heads, head_dim,
                               max_seq, rows_per_seq);
    return e == cudaSuccess ? AP_OK : AP_ERR_LAUNCH;
}

extern "C" int ap_silu_mul(const void* gate_up, void* y, int rows, int ffn, int tiled, void* stream) {
    if (!gate_up || !y) return AP_ERR_NULL_POINTER;
    if (rows < 1 || ffn < 2 || ffn % 2 || (tiled && ffn % 8)) return AP_ERR_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(y)) & 3) return AP_ERR_BAD_ALIGNMENT;
    const size_t total = (size_t)rows * ffn / 2;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 1184) blocks = 1184;
    cudaError_t e = launch_pdl(silu_mul_kernel, dim3(blocks), dim3(256), static_cast<cudaStream_t>(stream),
                               static_cast<const __half*>(gate_up), static_cast<__half*>(y), rows, ffn, tiled);
    return e == cudaSuccess ? AP_OK : AP_ERR_LAUNCH;
}

extern "C" size_t ap_decode_attention_scratch_bytes(int sequences, int heads, int head_dim, int splits) {
    if (sequences < 1 || heads < 1 || head_dim < 1 || splits < 2) return 0;
    // tickets (one int per head and sequence, rounded up to 256 bytes) followed by the partial results
    const size_t tickets = ((size_t)sequences * heads * sizeof(int) + 255) & ~static_cast<size_t>(255);
    return tickets + (size_t)sequences * heads * splits * (head_dim + 2) * sizeof(float);
}

namespace {

int decode_attention_impl(const void* qkv, int q_row_stride, const void* cos_sin, void* k_cache, void* v_cache, const void* pos,
                          void* out, int sequences, int heads, int kv_heads, int head_dim, int max_seq, float scale, int splits,
                          void* scratch, void* stream) {
    if (!qkv || !k_cache || !v_cache || !pos || !out) return AP_ERR_NULL_POINTER;
    const int need_stride = cos_sin ? (heads + 2 * kv_heads) * head_dim : heads * head_dim;
    if (sequences < 1 || heads < 1 || kv_heads < 1 || heads % kv_heads || max_seq < 1 || q_row_stride < need_stride ||
        splits < 1 || splits > 64)
        return AP_ERR_BAD_SHAPE;
    if (splits > 1 && !scratch) return AP_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
         reinterpret_cast<uintptr_t>(scratch) | reinterpret_cast<uintptr_t>(cos_sin)) & 15)
        return AP_ERR_BAD_ALIGNMENT;
    if (cos_sin && (q_row_stride % 8 || head_dim % 16)) return AP_ERR_BAD_ALIGNMENT;     // 16-byte rows of raw k and v
    const dim3 grid(heads, sequences, splits), block(256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto q = static_cast<const __half*>(qkv);
    auto k = static_cast<const __half*>(k_cache);
    auto v = static_cast<const __half*>(v_cache);
    auto kw = static_cast<__half*>(k_cache);
    auto vw = static_cast<__half*>(v_cache);
    auto p = static_cast<const int*>(pos);
    auto o = static_cast<__half*>(out);
    auto cs = static_cast<const float*>(cos_sin);
    int* tickets = static_cast<int*>(scratch);
    const size_t ticket_bytes = ((size_t)sequences * heads * sizeof(int) + 255) & ~static_cast<size_t>(255);
    float* partials = scratch ? reinterpret_cast<float*>(static_cast<char*>(scratch) + ticket_bytes) : nullptr;
    cudaError_t e;
#define AP_ATTN(D_)                                                                                                              \
    e = cos_sin ? launch_pdl(decode_attention_kernel<D_, true>, grid, block, st, q, q_row_stride, k, v, p, o, heads, kv_heads,   \
                             max_seq, scale, partials, tickets, cs, kw, vw)                                                      \
                : launch_pdl(decode_attention_kernel<D_, false>, grid, block, st, q, q_row_stride, k, v, p, o, heads, kv_heads,  \
                             max_seq, scale, partials, tickets, cs, kw, vw)
    switch (head_dim) {
        case 32: AP_ATTN(32); break;
        case 64: AP_ATTN(64); break;
        case 128: AP_ATTN(128); break;
        case 256: AP_ATTN(256); break;
        default: return AP_ERR_UNSUPPORTED;
    }
#undef AP_ATTN
    return e == cudaSuccess ? AP_OK : AP_ERR_LAUNCH;
}

}  // namespace

extern "C" int ap_decode_attention(const void* qkv, int q_row_stride, const void* k_cache, const void* v_cache,
                                   const void* pos, void* out, int sequences, int heads, int kv_heads, int head_dim,
                                   int max_seq, float scale, int splits, void* scratch, void* stream) {
    return decode_attention_impl(qkv, q_row_stride, nullptr, const_cast<void*>(k_cache), const_cast<void*>(v_cache), pos, out,
                                 sequences, heads, kv_heads, head_dim, max_seq, scale, splits, scratch, stream);
}

extern "C" int ap_decode_attention_rope(const void* qkv, int q_row_stride, const void* cos_sin, void* k_cache, void* v_cache,
                                        const void* pos, void* out, int sequences, int heads, int kv_heads, int head_dim,
                                        int max_seq, float scale, int splits, void* scratch, void* stream) {
    if (!cos_sin) return AP_ERR_NULL_POINTER;
    return decode_attention_impl(qkv, q_row_stride, cos_sin, k_cache, v_cache, pos, out, sequences, heads, kv_heads, head_dim,
                                 max_seq, scale, splits, scratch, stream);
}
