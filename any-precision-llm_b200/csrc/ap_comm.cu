// One-shot all-reduce over peer memory for the outputs of row-parallel layers (tensor parallelism).
//
// No counterpart in the reference, which runs on one device.  After a row-parallel matmul_kbit every
// rank holds a partial [M][N] fp16 result; the sum over ranks is needed on every rank.  At decode
// sizes (M*N*2 bytes = 16..128 KB) a ring or tree collective is all latency, so here every rank
//   1. stores its partial into slot `rank` of an inbox on EVERY rank (plain 16-byte stores through
//      NVLink / NVSwitch peer mappings, nothing else).  Every 16-byte store carries 8 bytes of payload and
//      the call's sequence number twice: {word, seq, word, seq}.  An aligned 8-byte half of a store
//      arrives whole, so a reader that finds the number beside a word knows the word is this call's:
//      no fence, no separate flag, one trip over the link;
//   2. polls the `world` slots of its own inbox (volatile loads, bounded) until every line of its
//      share carries the call's number, adds them in rank order with fp32 accumulation and writes fp16.
// The rank order is the same everywhere, so all ranks end with bit-identical results.
//
// Memory: one communication buffer per rank, allocated here with cudaMalloc and exchanged between
// the processes of one node as CUDA IPC handles (ap_comm_* below).  Layout of a buffer:
//   [0, 4 KB)           header (private): word 0 = calls completed, word 1 = blocks of the running
//                       call that are done, word 2 = error word
//   [4 KB, 20 KB)       unused (kept so that the inbox stays where it was)
//   then                inbox[2][kMaxWorld][2 * cap]    two generations, used in turn; 2 * cap because half
//                       of every line is sequence numbers
// The call counter lives on the device, so a captured CUDA graph can be replayed: every block of a
// launch reads it (after the previous kernel in the stream is over), the call's number is that
// plus one, and the block that finishes last writes it back.  All ranks advance in step because
// they issue the same sequence of calls.  The inbox generation is the call number's low bit, the
// same for every block of a call whatever its size, so consecutive calls always alternate
// generations even when their element counts (and with them the number of blocks and each
// block's range) differ.  Two generations are enough: a rank finishes call c only after it has
// read call c's lines from every rank, a rank stores its first line of call c only after all of its
// call c-1 is over (stream order), so when a fast rank stores call c+1 into the generation that
// call c-1 used, every rank is done reading call c-1.  Sequence numbers start at 1 and the buffer
// starts zeroed, so a line never carries a call's number before that call wrote it.
//
// Every wait is bounded.  When one runs out the block records it in `status` (if given) and in the
// buffer's own error word and returns without a result; nothing can spin forever.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstring>

#include "anyprec_b200.h"
#include "ap_kernels.h"

namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxBlocks = 64;
constexpr int kThreads = 256;
constexpr size_t kSeqBytes = 4096;
constexpr size_t kFlagBytes = (size_t)kMaxWorld * kMaxBlocks * sizeof(uint32_t) * 8;   // padded: 32 B per flag
constexpr size_t kHeaderBytes = kSeqBytes + kFlagBytes;
static_assert(kHeaderBytes == ap::kCommHeaderBytes && kMaxWorld == ap::kCommMaxWorld, "the decode kernel's push epilogue uses this layout");
constexpr uint32_t kSpinLimit = 1u << 21;                  // polls of a thread's lines before it gives up (seconds)
constexpr int kVecPerBlock = kThreads;                     // payload vectors (16 bytes) per block: one per thread

struct PeerTable {
    unsigned char* buf[kMaxWorld];
};

// lines of (generation, sender): payload vector v is lines 2v and 2v + 1
__device__ __forceinline__ uint4* inbox_slot(unsigned char* base, int gen, int from_rank, size_t cap) {
    return reinterpret_cast<uint4*>(base + kHeaderBytes + ((size_t)gen * kMaxWorld + from_rank) * 2 * cap);
}
__device__ __forceinline__ void st_line(uint4* p, uint32_t a, uint32_t b, uint32_t seq) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(p), "r"(a), "r"(seq), "r"(b) : "memory");
}
__device__ __forceinline__ uint4 ld_line(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float2 h2f(uint32_t u) {
    __half2 h = *reinterpret_cast<__half2*>(&u);
    return __half22float2(h);
}
__device__ __forceinline__ uint32_t f2h(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// RES: the sum is a row-parallel layer's output that a pre-norm decoder adds to its residual stream and
// normalises next.  The grid is (rows x blocks per row), a block's range lies inside one row of `row_vec`
// vectors, and step 4 becomes resid += fp16(sum) in place, out = new resid * norm_w (not yet divided by the root
// mean square), ssq_out[row][block of the row] = sum of squares of the new resid in the block's range: what
// ap_matmul_kbit_prenorm takes.  All ranks compute the same bits, so the replicated residual streams stay equal.
// PUSH false: the partial results are in the inboxes already (the decode kernel's epilogue stored them there,
// ap_matmul_kbit_push); this launch only collects.
template <bool RES, bool PUSH>
__global__ void __launch_bounds__(kThreads)
allreduce_oneshot_kernel(PeerTable peers, const uint4* __restrict__ src, uint4* __restrict__ out, int n_vec, int rank,
                         int world, size_t cap, int* __restrict__ status, int row_vec, int blocks_per_row,
                         uint4* __restrict__ resid, const uint4* __restrict__ norm_w, float* __restrict__ ssq_out) {
    unsigned char* mine = peers.buf[rank];
    uint32_t* header = reinterpret_cast<uint32_t*>(mine);      // [0] calls, [1] blocks done, [2] error
    __shared__ uint32_t s_seq;
    // Launched as a programmatic dependent of the kernel that produces `src` (the row-parallel
    // matmul_kbit), so that this kernel's launch overlaps that kernel's tail; the next kernel in the
    // stream may start its own prologue now and finds `out` complete when its dependency wait
    // returns.  Nothing of this kernel's state is read before the wait: the call counter was
    // written by the previous call of this kernel, which is only known to be over after it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) s_seq = __ldcg(header) + 1u;
    __syncthreads();
    const uint32_t seq = s_seq;
    const int gen = seq & 1u;

    // this block's contiguous share of the vector
    int v0, v1, row_base = 0;
    if constexpr (RES) {
        const int m = blockIdx.x / blocks_per_row, j = blockIdx.x % blocks_per_row;
        const int per = (row_vec + blocks_per_row - 1) / blocks_per_row;
        row_base = m * row_vec;
        v0 = row_base + (j * per < row_vec ? j * per : row_vec);
        v1 = row_base + ((j + 1) * per < row_vec ? (j + 1) * per : row_vec);
    } else {
        const int per_block = (n_vec + gridDim.x - 1) / gridDim.x;
        v0 = blockIdx.x * per_block;
        v1 = (v0 + per_block < n_vec) ? (v0 + per_block) : n_vec;
    }

    // Every block reads the call counter before it gets here, so the block that counts itself
    // last may advance it: the next call (after this kernel in stream order) then sees seq.
    auto finish = [&]() {
        __syncthreads();
        if (threadIdx.x == 0) {
            if (atomicAdd(header + 1, 1u) == gridDim.x - 1) {
                header[1] = 0u;
                __stcg(header, seq);
            }
        }
    };
    // 1. push: this thread's vectors, to every rank
    if constexpr (PUSH) {
        for (int v = v0 + threadIdx.x; v < v1; v += kThreads) {
            const uint4 val = src[v];
            for (int p = 0; p < world; p++) {
                uint4* line = inbox_slot(peers.buf[p], gen, rank, cap) + 2 * (size_t)v;
                st_line(line, val.x, val.y, seq);
                st_line(line + 1, val.z, val.w, seq);
            }
        }
    }
    // 2. poll the same vectors' lines from every rank, add in rank order
    float sq = 0.f;
    bool ok = true;
    for (int v = v0 + threadIdx.x; v < v1 && ok; v += kThreads) {
        uint4 la[kMaxWorld], lb[kMaxWorld];
        bool ready = false;
        for (uint32_t spin = 0; spin < kSpinLimit && !ready; spin++) {
            ready = true;
#pragma unroll
            for (int p = 0; p < kMaxWorld; p++) {
                if (p < world) {
                    const uint4* line = inbox_slot(mine, gen, p, cap) + 2 * (size_t)v;
                    la[p] = ld_line(line);
                    lb[p] = ld_line(line + 1);
                }
            }
#pragma unroll
            for (int p = 0; p < kMaxWorld; p++)
                if (p < world) ready = ready && la[p].y == seq && la[p].w == seq && lb[p].y == seq && lb[p].w == seq;
        }
        if (!ready) { ok = false; break; }
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int p = 0; p < kMaxWorld; p++) {
            if (p < world) {
                const float2 a = h2f(la[p].x), b = h2f(la[p].z), c = h2f(lb[p].x), d = h2f(lb[p].z);
                acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
                acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
            }
        }
        uint4 r;
        r.x = f2h(acc[0], acc[1]);
        r.y = f2h(acc[2], acc[3]);
        r.z = f2h(acc[4], acc[5]);
        r.w = f2h(acc[6], acc[7]);
        if constexpr (RES) {
            const uint4 hv = resid[v], wv = norm_w[v - row_base];
            uint4 hn, y;
            auto one = [&](uint32_t sum2, uint32_t h2, uint32_t w2, uint32_t& hn2, uint32_t& y2) {
                const float2 o = h2f(sum2), hf = h2f(h2), wf = h2f(w2);
                hn2 = f2h(hf.x + o.x, hf.y + o.y);
                const float2 n = h2f(hn2);
                y2 = f2h(n.x * wf.x, n.y * wf.y);
                sq += n.x * n.x + n.y * n.y;
            };
            one(r.x, hv.x, wv.x, hn.x, y.x);
            one(r.y, hv.y, wv.y, hn.y, y.y);
            one(r.z, hv.z, wv.z, hn.z, y.z);
            one(r.w, hv.w, wv.w, hn.w, y.w);
            resid[v] = hn;
            out[v] = y;
        } else {
            out[v] = r;
        }
    }
    if (!ok) {                                               // a peer's lines never came: say so, stay in step
        if (status) atomicExch(status, 1);
        header[2] = 1u;                                      // the buffer's own error word
    }
    if constexpr (RES) {
        // the block's sum of squares in a fixed order: shuffle tree, then the warps' sums left to right
        __shared__ float s_sq[kThreads / 32];
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o2);
        if ((threadIdx.x & 31) == 0) s_sq[threadIdx.x >> 5] = sq;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.f;
            for (int w2 = 0; w2 < kThreads / 32; w2++) t += s_sq[w2];
            ssq_out[blockIdx.x] = t;
        }
    }
    finish();
}

thread_local char g_comm_err[256] = "";

int comm_fail(cudaError_t e) {
    snprintf(g_comm_err, sizeof(g_comm_err), "%s", cudaGetErrorString(e));
    return AP_ERR_LAUNCH;
}

}  // namespace

extern "C" size_t ap_comm_buffer_bytes(size_t max_payload_bytes) {
    const size_t cap = (max_payload_bytes + 255) & ~static_cast<size_t>(255);
    return kHeaderBytes + 2 * static_cast<size_t>(kMaxWorld) * 2 * cap;
}

extern "C" int ap_comm_alloc(size_t bytes, void** ptr) {
    if (!ptr || bytes < kHeaderBytes) return AP_ERR_BAD_SHAPE;
    cudaError_t e = cudaMalloc(ptr, bytes);
    if (e != cudaSuccess) return comm_fail(e);
    e = cudaMemset(*ptr, 0, bytes);
    if (e != cudaSuccess) return comm_fail(e);
    e = cudaDeviceSynchronize();
    return e == cudaSuccess ? AP_OK : comm_fail(e);
}

extern "C" int ap_comm_free(void* ptr) {
    cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? AP_OK : comm_fail(e);
}

extern "C" int ap_comm_export(void* ptr, unsigned char* handle64) {
    if (!ptr || !handle64) return AP_ERR_NULL_POINTER;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) return comm_fail(e);
    memcpy(handle64, &h, 64);
    return AP_OK;
}

extern "C" int ap_comm_open(const unsigned char* handle64, void** ptr) {
    if (!ptr || !handle64) return AP_ERR_NULL_POINTER;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    return e == cudaSuccess ? AP_OK : comm_fail(e);
}

extern "C" int ap_comm_close(void* ptr) {
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? AP_OK : comm_fail(e);
}

extern "C" const char* ap_comm_last_error(void) { return g_comm_err; }

namespace {

int allreduce_impl(const void* src, void* out, int count, void* const* peer_buffers, int rank, int world,
                   size_t max_payload_bytes, int* status, void* stream, int rows, void* resid, const void* norm_weight,
                   void* ssq_out, bool pushed = false) {
    if (pushed) src = out;                                   // not read
    if (!src || !out || !peer_buffers) return AP_ERR_NULL_POINTER;
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || count < 8 || count % 8) return AP_ERR_BAD_SHAPE;
    const size_t cap = (max_payload_bytes + 255) & ~static_cast<size_t>(255);
    if (static_cast<size_t>(count) * 2 > cap) return AP_ERR_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out)) & 15) return AP_ERR_BAD_ALIGNMENT;
    PeerTable t;
    for (int p = 0; p < kMaxWorld; p++) {
        t.buf[p] = p < world ? static_cast<unsigned char*>(peer_buffers[p]) : nullptr;
        if (p < world && (!t.buf[p] || (reinterpret_cast<uintptr_t>(t.buf[p]) & 255))) return AP_ERR_BAD_ALIGNMENT;
    }
    const int n_vec = count / 8;
    // the same grid on every rank for a given count: blocks of different ranks pair up by index
    int blocks = (n_vec + kVecPerBlock - 1) / kVecPerBlock;
    blocks = blocks < 1 ? 1 : (blocks > kMaxBlocks ? kMaxBlocks : blocks);
    int row_vec = 0, bpr = 0;
    if (resid) {
        if (!norm_weight || !ssq_out) return AP_ERR_NULL_POINTER;
        if (rows < 1 || count % rows || (count / rows) % 8) return AP_ERR_BAD_SHAPE;
        if ((reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(norm_weight)) & 15 ||
            reinterpret_cast<uintptr_t>(ssq_out) & 3)
            return AP_ERR_BAD_ALIGNMENT;
        row_vec = count / rows / 8;
        bpr = ap_allreduce_residual_blocks(rows, count / rows);
        if (bpr < 1) return AP_ERR_UNSUPPORTED;
        blocks = rows * bpr;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const uint4* sp = static_cast<const uint4*>(src);
    uint4* op = static_cast<uint4*>(out);
    uint4* rp = static_cast<uint4*>(resid);
    const uint4* wp = static_cast<const uint4*>(norm_weight);
    float* qp = static_cast<float*>(ssq_out);
    cudaError_t e;
    if (resid && !pushed) e = cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<true, true>, t, sp, op, n_vec, rank, world, cap, status, row_vec, bpr, rp, wp, qp);
    else if (resid) e = cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<true, false>, t, sp, op, n_vec, rank, world, cap, status, row_vec, bpr, rp, wp, qp);
    else if (!pushed) e = cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<false, true>, t, sp, op, n_vec, rank, world, cap, status, 0, 0, rp, wp, qp);
    else e = cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<false, false>, t, sp, op, n_vec, rank, world, cap, status, 0, 0, rp, wp, qp);
    return e == cudaSuccess ? AP_OK : comm_fail(e);
}

}  // namespace

extern "C" int ap_allreduce_residual_blocks(int rows, int row_len) {
    if (rows < 1 || row_len < 8 || row_len % 8) return 0;
    const int bpr = (row_len / 8 + kVecPerBlock - 1) / kVecPerBlock;
    return rows * bpr <= kMaxBlocks ? bpr : 0;
}

extern "C" int ap_allreduce_oneshot(const void* src, void* out, int count, void* const* peer_buffers, int rank, int world,
                                    size_t max_payload_bytes, int* status, void* stream) {
    return allreduce_impl(src, out, count, peer_buffers, rank, world, max_payload_bytes, status, stream, 0, nullptr, nullptr,
                          nullptr);
}

extern "C" int ap_allreduce_oneshot_collect(void* out, int rows, int row_len, void* resid, const void* norm_weight,
                                            void* ssq_out, void* const* peer_buffers, int rank, int world,
                                            size_t max_payload_bytes, int* status, void* stream) {
    if (rows < 1 || row_len < 8) return AP_ERR_BAD_SHAPE;
    return allreduce_impl(nullptr, out, rows * row_len, peer_buffers, rank, world, max_payload_bytes, status, stream, rows, resid,
                          norm_weight, ssq_out, true);
}

extern "C" int ap_allreduce_oneshot_residual(const void* src, void* out, int rows, int row_len, void* resid,
                                             const void* norm_weight, void* ssq_out, void* const* peer_buffers, int rank,
                                             int world, size_t max_payload_bytes, int* status, void* stream) {
    if (!resid) return AP_ERR_NULL_POINTER;
    if (rows < 1 || row_len < 8) return AP_ERR_BAD_SHAPE;
    return allreduce_impl(src, out, rows * row_len, peer_buffers, rank, world, max_payload_bytes, status, stream, rows, resid,
                          norm_weight, ssq_out);
}
