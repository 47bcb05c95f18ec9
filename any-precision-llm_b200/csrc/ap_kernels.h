// Internal launch interface between the C-ABI translation unit and the kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace ap {

// What the decode kernel's decoder variants do with a finished tile (see the epilogue of
// gemv_kbit_tma_kernel): mode 1 gated (silu(gate) * up of stacked rows), 2 scaled by the per-row
// rsqrt(mean square + eps) taken from `ssq_in` ([M][ssq_blocks] partial sums of squares, mean over
// 1 / inv_width values), 3 both, 4 residual update (`resid` [M][N] += product; out = new residual *
// `norm_w`; `ssq_out` [M][N / 16] partial sums of squares of the new residual), 5 push to the peers' inboxes.
// Layout of a rank's communication buffer (ap_comm.cu): header, then inbox[2 generations][kCommMaxWorld senders]
// [2 * cap bytes]; sixteen-byte lines {word, seq, word, seq}.
constexpr int kCommMaxWorld = 8;
constexpr unsigned long long kCommHeaderBytes = 20480;

struct GemvEpilogue {
    int mode;
    const float* ssq_in;
    int ssq_blocks;
    float inv_width;
    float eps;
    __half* resid;
    const __half* norm_w;
    float* ssq_out;
    // mode 5: the product is a row-parallel layer's partial result; instead of storing it, the tile is pushed
    // into slot `rank` of the all-reduce inbox of every rank (the first step of ap_allreduce_oneshot, done
    // from here; ap_allreduce_oneshot_collect does the rest)
    unsigned char* peer[kCommMaxWorld];
    int rank, world;
    unsigned long long cap;
};

// All launchers enqueue on `stream`, never synchronise, never allocate, and return the
// launch status from cudaGetLastError().
cudaError_t launch_dequant(const void* qweight, long long plane_stride, const void* lut, void* out, int N,
                           int K, int w_bits, cudaStream_t stream);

// `splits` > 1 cuts K into that many ranges handled by different CTAs (fast kernel only); it needs
// `partials` (splits*M*N floats, any contents) and `tickets` (N/16 ints, zero on entry, zero again
// on completion).  With splits <= 1 or null scratch pointers every CTA takes a whole row range.
// `epi` non-null: one of the decoder's epilogues (modes 1 and 3: `out` is [M][N/2]); only the fast kernel has
// them (cudaErrorNotSupported otherwise; M <= 8).
cudaError_t launch_gemv(const void* x, const void* qweight, long long plane_stride, const void* lut, void* out,
                        int M, int N, int K, int w_bits, int splits, float* partials, int* tickets,
                        cudaStream_t stream, const GemvEpilogue* epi = nullptr);
bool gemv_fast_path(const void* x, const void* qweight, long long plane_stride, const void* lut, int N, int K);
// Reads (after synchronising the device) and clears the flag that a decode kernel sets when one of its
// bounded waits ran out.
cudaError_t take_gemv_wait_flag(int* flag);

// Fused dequantise + tensor-core GEMM for prefill.  gemm_tc_supported() says whether the shape and
// alignment qualify (N % 128 == 0, K % 128 == 0, 16-byte aligned x, qweight and lut).  `status` may be null;
// otherwise the kernel stores 1 there if one of its bounded waits ran out.
bool gemm_tc_supported(const void* x, const void* qweight, long long plane_stride, const void* lut, const void* out,
                       int M, int N, int K);
// `splits` > 1 cuts K into ranges taken by different thread blocks (for layers with few blocks of rows):
// fp32 partial tiles go to `partials` ([splits][M][N]), the block that draws a tile's last ticket adds them in
// range order; `tickets` (one int per tile, zero before the first call) are handed back at zero.
cudaError_t launch_gemm_tc(const void* x, const void* qweight, long long plane_stride, const void* lut, void* out, int M,
                           int N, int K, int w_bits, int* status, int splits, float* partials, int* tickets,
                           cudaStream_t stream);
// The split count that gives the fused kernel about one thread block per SM (1 = do not split).
int gemm_tc_suggested_splits(int M, int N, int K);

}  // namespace ap
