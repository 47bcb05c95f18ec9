// Internal launch interface between the C-ABI translation unit and the kernels.
#pragma once

#include <cuda_runtime.h>

namespace ap {

// All launchers enqueue on `stream`, never synchronise, never allocate, and return the
// launch status from cudaGetLastError().
cudaError_t launch_dequant(const void* qweight, long long plane_stride, const void* lut, void* out, int N,
                           int K, int w_bits, cudaStream_t stream);

// `splits` > 1 cuts K into that many ranges handled by different CTAs (fast kernel only); it needs
// `partials` (splits*M*N floats, any contents) and `tickets` (N/16 ints, zero on entry, zero again
// on completion).  With splits <= 1 or null scratch pointers every CTA takes a whole row range.
// `gated` != 0: the rows are a gated MLP's gate and up projections stacked tile by tile (eight gate rows, then
// the eight up rows of the same features, per 16 rows) and `out` is [M][N/2] = silu(gate) * up; only the fast
// kernel has that epilogue (cudaErrorNotSupported otherwise; M <= 8).
cudaError_t launch_gemv(const void* x, const void* qweight, long long plane_stride, const void* lut, void* out,
                        int M, int N, int K, int w_bits, int splits, float* partials, int* tickets,
                        cudaStream_t stream, int gated = 0);
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
