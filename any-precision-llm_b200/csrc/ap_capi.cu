// extern "C" entry points of libanyprec_sm100.so: argument checks, then launch.
#include "../../include/anyprec_b200.h"
#include "ap_kernels.h"

#include <stdio.h>

#include <mutex>

namespace {

thread_local char g_cuda_err[256] = "";

int cuda_fail(cudaError_t e) {
    snprintf(g_cuda_err, sizeof g_cuda_err, "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
    return AP_ERR_LAUNCH;
}

int check_common(const void* qweight, int64_t plane_stride, const void* lut, const void* out, int N, int K,
                 int w_bits) {
    if (!qweight || !lut || !out) return AP_ERR_NULL_POINTER;
    if (w_bits < 3 || w_bits > 8) return AP_ERR_BAD_BITS;
    if (N < 1 || K < 32 || K % 32 != 0) return AP_ERR_BAD_SHAPE;
    if (plane_stride < (int64_t)N * (K / 32)) return AP_ERR_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(qweight) & 3) || (reinterpret_cast<uintptr_t>(lut) & 1))
        return AP_ERR_BAD_ALIGNMENT;
    return AP_OK;
}

}  // namespace

extern "C" int ap_version(void) { return 1; }

extern "C" const char* ap_strerror(int code) {
    switch (code) {
        case AP_OK: return "ok";
        case AP_ERR_NULL_POINTER: return "null pointer argument";
        case AP_ERR_BAD_BITS: return "w_bits must be in [3, 8]";
        case AP_ERR_BAD_SHAPE: return "bad shape: need N >= 1, M >= 1, K a positive multiple of 32, plane_stride >= N*K/32";
        case AP_ERR_BAD_ALIGNMENT: return "pointer not aligned as required";
        case AP_ERR_LAUNCH: return "CUDA launch failed (see ap_last_cuda_error)";
        case AP_ERR_BAD_DEVICE: return "no usable CUDA device";
        case AP_ERR_UNSUPPORTED: return "shape or alignment not supported by this entry point";
        case AP_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the library's built-in scratch area holds";
        default: return "unknown error code";
    }
}

extern "C" const char* ap_last_cuda_error(void) { return g_cuda_err; }

extern "C" int ap_take_wait_expired(void) {
    int flag = 0;
    cudaError_t e = ap::take_gemv_wait_flag(&flag);
    if (e != cudaSuccess) return cuda_fail(e);
    return flag ? 1 : 0;
}

extern "C" int ap_dequant_kbit(const void* qweight, int64_t plane_stride, const void* lut, void* out, int N, int K,
                               int w_bits, void* stream) {
    int rc = check_common(qweight, plane_stride, lut, out, N, K, w_bits);
    if (rc != AP_OK) return rc;
    if (reinterpret_cast<uintptr_t>(out) & 15) return AP_ERR_BAD_ALIGNMENT;
    cudaError_t e = ap::launch_dequant(qweight, plane_stride, lut, out, N, K, w_bits,
                                       static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? AP_OK : cuda_fail(e);
}

namespace {

// The ticket counters take a fixed area at the start of every workspace, whatever the shape, so that a
// workspace which served one shape can serve another: a counter never lies where partial sums were.
constexpr size_t kTicketAreaBytes = AP_TICKET_AREA_BYTES;
size_t ticket_bytes(int) { return kTicketAreaBytes; }
bool tickets_fit(int N) { return static_cast<size_t>((N + 15) / 16) * sizeof(int) <= kTicketAreaBytes; }

int matmul_impl(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out, int M, int N,
                int K, int w_bits, int splits, void* workspace, size_t workspace_bytes, void* stream,
                const ap::GemvEpilogue* epi = nullptr) {
    int rc = check_common(qweight, plane_stride, lut, out, N, K, w_bits);
    if (rc != AP_OK) return rc;
    if (!x) return AP_ERR_NULL_POINTER;
    if (M < 1) return AP_ERR_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 1) || (reinterpret_cast<uintptr_t>(out) & 1)) return AP_ERR_BAD_ALIGNMENT;
    int* tickets = nullptr;
    float* partials = nullptr;
    if (splits > 1) {
        if (!workspace) return AP_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(workspace) & 255) return AP_ERR_BAD_ALIGNMENT;
        if (!tickets_fit(N)) return AP_ERR_UNSUPPORTED;
        const int mc = M < 8 ? M : 8;
        if (workspace_bytes < ticket_bytes(N) + static_cast<size_t>(splits) * mc * N * sizeof(float)) return AP_ERR_BAD_SHAPE;
        tickets = static_cast<int*>(workspace);
        partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + ticket_bytes(N));
    }
    const char* xp = static_cast<const char*>(x);
    char* op = static_cast<char*>(out);
    // eight batch rows per pass over the planes; the launcher runs the passes (side by side where it can)
    cudaError_t e = ap::launch_gemv(xp, qweight, plane_stride, lut, op, M, N, K, w_bits, splits, partials, tickets,
                                    static_cast<cudaStream_t>(stream), epi);
    if (e == cudaErrorNotSupported) return AP_ERR_UNSUPPORTED;
    return e == cudaSuccess ? AP_OK : cuda_fail(e);
}

}  // namespace

extern "C" int ap_matmul_kbit(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                              int M, int N, int K, int w_bits, void* stream) {
    return matmul_impl(x, qweight, plane_stride, lut, out, M, N, K, w_bits, 1, nullptr, 0, stream);
}

extern "C" size_t ap_matmul_kbit_workspace_bytes(int M, int N, int splits) {
    if (M < 1 || N < 1 || splits < 2) return 0;
    return ticket_bytes(N) + static_cast<size_t>(splits) * (M < 8 ? M : 8) * N * sizeof(float);
}

extern "C" int ap_matmul_kbit_splitk(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                                     int M, int N, int K, int w_bits, int splits, void* workspace,
                                     size_t workspace_bytes, void* stream) {
    if (splits < 1) return AP_ERR_BAD_SHAPE;
    return matmul_impl(x, qweight, plane_stride, lut, out, M, N, K, w_bits, splits, workspace, workspace_bytes, stream);
}

extern "C" int ap_matmul_kbit_gated(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                                    int M, int N, int K, int w_bits, int splits, void* workspace, size_t workspace_bytes,
                                    void* stream) {
    if (splits < 1 || N % 16 != 0 || M > 8) return M > 8 || N % 16 ? AP_ERR_UNSUPPORTED : AP_ERR_BAD_SHAPE;
    ap::GemvEpilogue epi = {};
    epi.mode = 1;
    return matmul_impl(x, qweight, plane_stride, lut, out, M, N, K, w_bits, splits, workspace, workspace_bytes, stream, &epi);
}

extern "C" int ap_matmul_kbit_prenorm(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                                      int M, int N, int K, int w_bits, int splits, void* workspace, size_t workspace_bytes,
                                      int gated, const void* ssq, int ssq_blocks, int width, float eps, void* stream) {
    if (!ssq) return AP_ERR_NULL_POINTER;
    if (splits < 1 || ssq_blocks < 1 || width < 1) return AP_ERR_BAD_SHAPE;
    if (N % 16 != 0 || M > 8) return AP_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(ssq) & 3) return AP_ERR_BAD_ALIGNMENT;
    ap::GemvEpilogue epi = {};
    epi.mode = gated ? 3 : 2;
    epi.ssq_in = static_cast<const float*>(ssq);
    epi.ssq_blocks = ssq_blocks;
    epi.inv_width = 1.0f / static_cast<float>(width);
    epi.eps = eps;
    return matmul_impl(x, qweight, plane_stride, lut, out, M, N, K, w_bits, splits, workspace, workspace_bytes, stream, &epi);
}

extern "C" int ap_matmul_kbit_push(const void* x, const void* qweight, int64_t plane_stride, const void* lut, int M, int N,
                                   int K, int w_bits, int splits, void* workspace, size_t workspace_bytes,
                                   void* const* peer_buffers, int rank, int world, size_t max_payload_bytes, void* stream) {
    if (!peer_buffers) return AP_ERR_NULL_POINTER;
    if (splits < 1 || world < 1 || world > ap::kCommMaxWorld || rank < 0 || rank >= world) return AP_ERR_BAD_SHAPE;
    if (N % 16 != 0 || M > 8) return AP_ERR_UNSUPPORTED;
    const size_t cap = (max_payload_bytes + 255) & ~static_cast<size_t>(255);
    if (static_cast<size_t>(M) * N * 2 > cap) return AP_ERR_BAD_SHAPE;
    ap::GemvEpilogue epi = {};
    epi.mode = 5;
    for (int p = 0; p < world; p++) {
        if (!peer_buffers[p] || (reinterpret_cast<uintptr_t>(peer_buffers[p]) & 255)) return AP_ERR_BAD_ALIGNMENT;
        epi.peer[p] = static_cast<unsigned char*>(peer_buffers[p]);
    }
    epi.rank = rank;
    epi.world = world;
    epi.cap = cap;
    // `out` is not written in this mode; the checks want a non-null, even address
    return matmul_impl(x, qweight, plane_stride, lut, peer_buffers[rank], M, N, K, w_bits, splits, workspace, workspace_bytes, stream,
                       &epi);
}

extern "C" int ap_matmul_kbit_residual(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                                       int M, int N, int K, int w_bits, int splits, void* workspace, size_t workspace_bytes,
                                       void* resid, const void* norm_weight, void* ssq_out, void* stream) {
    if (!resid || !norm_weight || !ssq_out) return AP_ERR_NULL_POINTER;
    if (splits < 1) return AP_ERR_BAD_SHAPE;
    if (N % 16 != 0 || M > 8) return AP_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(norm_weight)) & 1 || reinterpret_cast<uintptr_t>(ssq_out) & 3)
        return AP_ERR_BAD_ALIGNMENT;
    ap::GemvEpilogue epi = {};
    epi.mode = 4;
    epi.resid = static_cast<__half*>(resid);
    epi.norm_w = static_cast<const __half*>(norm_weight);
    epi.ssq_out = static_cast<float*>(ssq_out);
    return matmul_impl(x, qweight, plane_stride, lut, out, M, N, K, w_bits, splits, workspace, workspace_bytes, stream, &epi);
}

// ---------------------------------------------------------------------------------------------
// Split-K GEMV for callers that cannot hand the library any scratch memory of their own.
//
// The scratch lives in this file-scope device array.  Every GPU that loads the library carries
// it until the process exits.  In host code the name below is only a handle for the runtime: the
// device address has to be asked for with cudaGetSymbolAddress, on the device in question.
constexpr size_t kBuiltinScratchBytes = AP_BUILTIN_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char ap_builtin_scratch[kBuiltinScratchBytes];

namespace {

// Device address of ap_builtin_scratch on the current device (resolved once per device; host threads
// that race for the first call on a device are serialised, and only one of them issues the clear).
int builtin_scratch(void** ptr, cudaStream_t stream) {
    static void* addr[64] = {};
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev < 0 || dev >= 64) return AP_ERR_BAD_DEVICE;
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, ap_builtin_scratch);
        if (e != cudaSuccess) return cuda_fail(e);
        // The ticket counters at the front must read zero before the first use.  A freshly loaded
        // module has them zero already; clearing once more costs nothing and covers a device whose
        // earlier work was cut short.
        e = cudaMemsetAsync(p, 0, kBuiltinScratchBytes, stream);
        if (e != cudaSuccess) return cuda_fail(e);
        addr[dev] = p;
    }
    *ptr = addr[dev];
    return AP_OK;
}

}  // namespace

extern "C" size_t ap_builtin_scratch_bytes(void) { return kBuiltinScratchBytes; }

extern "C" int ap_matmul_kbit_splitk_noalloc(const void* x, const void* qweight, int64_t plane_stride, const void* lut,
                                             void* out, int M, int N, int K, int w_bits, int splits, void* stream) {
    if (splits < 1 || M < 1 || N < 1 || K < 32) return AP_ERR_BAD_SHAPE;
    // The split count the kernel will really use: never more ranges than 1024-weight groups, and none
    // at all on the shapes that take the plain kernel.  The scratch limit applies to that count.
    const int groups = (K + 1023) / 1024;
    if (splits > groups) splits = groups;
    if (!ap::gemv_fast_path(x, qweight, plane_stride, lut, N, K)) splits = 1;
    if (splits > 1 && ap_matmul_kbit_workspace_bytes(M, N, splits) > kBuiltinScratchBytes) return AP_ERR_SCRATCH_LIMIT;
    void* scratch = nullptr;
    if (splits > 1) {
        int rc = builtin_scratch(&scratch, static_cast<cudaStream_t>(stream));
        if (rc != AP_OK) return rc;
    }
    return matmul_impl(x, qweight, plane_stride, lut, out, M, N, K, w_bits, splits, scratch, kBuiltinScratchBytes, stream);
}

namespace {

int gemm_impl(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out, int M, int N, int K,
              int w_bits, int* status, int splits, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_common(qweight, plane_stride, lut, out, N, K, w_bits);
    if (rc != AP_OK) return rc;
    if (!x) return AP_ERR_NULL_POINTER;
    if (M < 1) return AP_ERR_BAD_SHAPE;
    if (!ap::gemm_tc_supported(x, qweight, plane_stride, lut, out, M, N, K)) return AP_ERR_UNSUPPORTED;
    float* partials = nullptr;
    int* tickets = nullptr;
    if (splits > 1) {
        if (!workspace) return AP_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(workspace) & 255) return AP_ERR_BAD_ALIGNMENT;
        if (K % 256 != 0) return AP_ERR_UNSUPPORTED;
        const size_t tiles = static_cast<size_t>(N / 128) * ((M + 63) / 64);
        if (tiles * sizeof(int) > kTicketAreaBytes) return AP_ERR_UNSUPPORTED;
        if (workspace_bytes < kTicketAreaBytes + static_cast<size_t>(splits) * M * N * sizeof(float)) return AP_ERR_BAD_SHAPE;
        tickets = static_cast<int*>(workspace);
        partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + kTicketAreaBytes);
    }
    cudaError_t e = ap::launch_gemm_tc(x, qweight, plane_stride, lut, out, M, N, K, w_bits, status, splits, partials,
                                       tickets, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? AP_OK : cuda_fail(e);
}

}  // namespace

extern "C" int ap_gemm_kbit(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out, int M,
                            int N, int K, int w_bits, int* status, void* stream) {
    return gemm_impl(x, qweight, plane_stride, lut, out, M, N, K, w_bits, status, 1, nullptr, 0, stream);
}

extern "C" int ap_gemm_kbit_splits(int M, int N, int K) {
    if (M < 1 || N < 1 || K < 1) return 1;
    return ap::gemm_tc_suggested_splits(M, N, K);
}

extern "C" size_t ap_gemm_kbit_workspace_bytes(int M, int N, int splits) {
    if (M < 1 || N < 1 || splits < 2) return 0;
    return kTicketAreaBytes + static_cast<size_t>(splits) * M * N * sizeof(float);
}

extern "C" int ap_gemm_kbit_splitk(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                                   int M, int N, int K, int w_bits, int* status, int splits, void* workspace,
                                   size_t workspace_bytes, void* stream) {
    if (splits < 1) return AP_ERR_BAD_SHAPE;
    return gemm_impl(x, qweight, plane_stride, lut, out, M, N, K, w_bits, status, splits, workspace, workspace_bytes, stream);
}
