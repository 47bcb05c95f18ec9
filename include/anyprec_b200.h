/*
 * C ABI of libanyprec_sm100.so: the any-precision bitplane serving kernels for NVIDIA
 * B200 (sm_100a).
 *
 * The reference project (SNU-ARC/any-precision-llm) exposes this path as a pybind11/libtorch
 * module, any_precision_ext, with two functions (any_precision/modules/kernels/main.cu:145-148).
 * The entry points below are what a binding for that module calls; the Python module
 * any_precision_ext shipped beside this header binds them with ctypes.
 *
 * Conventions common to every entry point
 *   - All pointers are device pointers on the current CUDA device; the caller owns every
 *     buffer.  Nothing is allocated, freed or synchronised inside the library.
 *   - Work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = default stream).
 *   - Return value: 0 on success, a negative AP_ERR_* code otherwise (never exit(), in
 *     contrast to HANDLE_ERROR in main.cu:5-12).  ap_strerror() names the code.
 *   - qweight: int32 [planes][N][K/32]; plane p starts `plane_stride` int32 words after plane
 *     p-1 (N*K/32 for a contiguous tensor; larger for a row slice of a wider tensor).
 *     Plane 0 is the MSB of the parent code; only planes 0..w_bits-1 are read.
 *   - lut: fp16 [N][2^w_bits], contiguous, the table of precision w_bits.
 *   - 3 <= w_bits <= 8, K % 32 == 0.
 */
#ifndef ANYPREC_B200_H
#define ANYPREC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AP_OK 0
#define AP_ERR_NULL_POINTER (-1)
#define AP_ERR_BAD_BITS (-2)
#define AP_ERR_BAD_SHAPE (-3)
#define AP_ERR_BAD_ALIGNMENT (-4)
#define AP_ERR_LAUNCH (-5)
#define AP_ERR_BAD_DEVICE (-6)
#define AP_ERR_UNSUPPORTED (-7)
#define AP_ERR_SCRATCH_LIMIT (-8)

/* Ticket counters at the start of every split-K workspace (one per 16 output rows: N <= 262144). */
#define AP_TICKET_AREA_BYTES (64u * 1024u)

/* Size of the scratch area built into the library for ap_matmul_kbit_splitk_noalloc. */
#define AP_BUILTIN_SCRATCH_BYTES (2u * 1024u * 1024u)

/* Library ABI version (integer, bumped on incompatible change). */
int ap_version(void);

/* Static, NUL-terminated description of an AP_* code. */
const char* ap_strerror(int code);

/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* ap_last_cuda_error(void);

/*
 * Diagnostic with no counterpart in the reference.  Every wait inside the decode kernels (on the
 * arrival of a block of planes) is bounded; a kernel whose wait ran out stops working on its tile,
 * sets a flag on its device and returns, so its output is not valid.  This call synchronises the
 * current device, returns 1 if the flag was set since the last call (and clears it), 0 if not, or a
 * negative AP_ERR_* code.  Not for the serving loop: it synchronises.
 */
int ap_take_wait_expired(void);

/*
 * out[N][K] (fp16, natural k order) = lut[n][code_w(n, k)].
 * Replaces dequant_kbit(qweight, lut, w_bits) -> Tensor  (kernels/main.cu:60-91, kernel
 * dequant_kbit_store<bits> in kernels/dequant.cuh:177-242).  Bit-exact with it.
 * `out` must be 16-byte aligned.
 */
int ap_dequant_kbit(const void* qweight, int64_t plane_stride, const void* lut, void* out,
                    int N, int K, int w_bits, void* stream);

/*
 * out[M][N] (fp16) = x[M][K] (fp16) times the dequantised weight, transposed, accumulated in fp32.
 * Replaces matmul_kbit(in, qweight, lut, w_bits) -> Tensor  (kernels/main.cu:93-143, kernels
 * matmul_kbit_32<maxm,bits,use_ksplit> in kernels/matmul.cuh:16-167).  The reference accepts
 * 1 <= M <= 8; here any M >= 1 is taken (rows are processed eight at a time).
 */
int ap_matmul_kbit(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                   int M, int N, int K, int w_bits, void* stream);

/*
 * matmul_kbit with K cut into `splits` ranges that different thread blocks take (for layers with
 * few rows, e.g. tensor-parallel shards, which would otherwise leave most of the GPU idle).  The
 * splits are added up in a fixed order, so results do not depend on scheduling.  No counterpart in
 * the reference (its use_ksplit variant, kernels/matmul.cuh:139-155, splits inside one block).
 *   workspace        device memory, 256-byte aligned, at least ap_matmul_kbit_workspace_bytes(M, N,
 *                    splits) bytes.  Its first AP_TICKET_AREA_BYTES are ticket counters: they
 *                    must be ZERO before the first call and are left zero by every call; the rest
 *                    needs no initialisation.  One workspace can serve calls of different shapes.
 *                    N above 262144 with splits > 1 is refused (AP_ERR_UNSUPPORTED).
 *   Calls that may overlap on the GPU (different streams) must not share a workspace.
 * Shapes the fast kernel does not take (N % 16, K % 128, 16-byte alignment) ignore `splits`.
 */
size_t ap_matmul_kbit_workspace_bytes(int M, int N, int splits);
int ap_matmul_kbit_splitk(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                          int M, int N, int K, int w_bits, int splits, void* workspace, size_t workspace_bytes,
                          void* stream);

/*
 * matmul_kbit of a gated MLP's two projections at once, with the activation in the epilogue.  No counterpart
 * in the reference (it calls gate_proj and up_proj separately and leaves act(gate) * up to the framework).
 * qweight / lut hold BOTH projections stacked tile by tile: of every 16 rows the first eight are gate rows
 * f .. f+7 and the last eight the up rows of the same features (N = 2 * features, a multiple of 16;
 * packing.interleave_gate_up builds that operand).  out[M][N/2] (fp16) = silu(gate) * up, rounded as the
 * separate operations would round (both products to fp16, the activation to fp16, then their product).
 * M <= 8 and operands that the fast kernel takes (K % 128 == 0, 16-byte aligned x, qweight, lut) only:
 * AP_ERR_UNSUPPORTED otherwise.  `splits`, `workspace` as for ap_matmul_kbit_splitk (splits = 1: no workspace).
 */
int ap_matmul_kbit_gated(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                         int M, int N, int K, int w_bits, int splits, void* workspace, size_t workspace_bytes,
                         void* stream);

/*
 * The decode product with a pre-norm decoder's residual add and RMSNorm folded into it (no counterpart in the
 * reference, which runs the stock Hugging Face decoder layer around its linears).  A pair of calls replaces
 * "h += linear_1(...); y = rmsnorm(h) * g; z = linear_2(y)":
 *   ap_matmul_kbit_residual  p = x W^T as ap_matmul_kbit_splitk computes it; resid[M][N] (fp16) += fp16(p) in place;
 *                            out[M][N] = fp16(new resid * norm_weight[N]) (NOT yet divided by the root mean square);
 *                            ssq_out[M][N / 16] (fp32) = per 16-row tile the sum of squares of the new resid.
 *   ap_matmul_kbit_prenorm   out = fp16(r_m * (x W^T)) with r_m = rsqrt(sum(ssq[m][0 .. ssq_blocks)) / width + eps):
 *                            x is the `out` of ap_matmul_kbit_residual, ssq its ssq_out, width its N; a product
 *                            commutes with a scale per batch row, so this is linear_2(rmsnorm(h) * g) up to fp16
 *                            rounding of x.  gated != 0: additionally the epilogue of ap_matmul_kbit_gated
 *                            (operand stacked tile by tile, out[M][N / 2]), the scale applied before the activation.
 * Same limits as ap_matmul_kbit_gated (M <= 8, N % 16 == 0, fast-kernel operands), AP_ERR_UNSUPPORTED otherwise.
 */
int ap_matmul_kbit_prenorm(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                           int M, int N, int K, int w_bits, int splits, void* workspace, size_t workspace_bytes,
                           int gated, const void* ssq, int ssq_blocks, int width, float eps, void* stream);
int ap_matmul_kbit_residual(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                            int M, int N, int K, int w_bits, int splits, void* workspace, size_t workspace_bytes,
                            void* resid, const void* norm_weight, void* ssq_out, void* stream);

/*
 * ap_matmul_kbit_splitk for callers that have no way to provide a workspace: code that runs where
 * device allocation is off limits (inside a serving loop with a frozen memory pool, under a
 * framework that owns every byte of device memory, in a plugin that is handed only its inputs and
 * outputs).  It has no counterpart in the reference.  The scratch is a 2 MiB area compiled into
 * the library (AP_BUILTIN_SCRATCH_BYTES; each GPU that loads the library holds it until the
 * process ends); nothing is allocated or freed, by this call or by anything it calls.
 *   - Problems with ap_matmul_kbit_workspace_bytes(M, N, splits) above that size are refused with
 *     AP_ERR_SCRATCH_LIMIT (splits = 8 at M = 1 fits up to N = 63488); use fewer splits
 *     or the workspace variant.
 *   - The first call on a device looks the area's device address up and clears it on `stream`;
 *     make that first call before capturing `stream` into anything, like any other set-up work,
 *     and let it COMPLETE (synchronise its stream once) before any call on another stream or from
 *     another host thread: the clear is ordered only on the first caller's stream.
 *   - All calls on a device share the one area and leave their partial sums in it; only the
 *     ticket counters are kept at zero.  Two such calls that can run at the same time on the GPU
 *     (different streams) would corrupt each other: serialise them.
 */
size_t ap_builtin_scratch_bytes(void);
int ap_matmul_kbit_splitk_noalloc(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                                  int M, int N, int K, int w_bits, int splits, void* stream);

/*
 * Prefill: out[M][N] (fp16) = x[M][K] times the dequantised weight, transposed, with the weight
 * dequantised tile by tile inside the kernel and multiplied on the tensor cores (fp32 accumulate).
 * Replaces the two-step path of any_precision/modules/AnyPrecisionLinear.py:60-62, i.e.
 * dequant_kbit (kernels/main.cu:60-91) followed by torch.matmul on the materialised fp16 weight.
 * Requires N % 128 == 0, K % 128 == 0, x, qweight and lut 16-byte aligned, plane_stride a
 * multiple of 4; returns AP_ERR_UNSUPPORTED otherwise (use ap_dequant_kbit + a GEMM then).
 * `status` is an optional device int (may be NULL): the kernel writes 1 there if one of its
 * internal bounded waits expired, in which case `out` is incomplete.
 */
int ap_gemm_kbit(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                 int M, int N, int K, int w_bits, int* status, void* stream);

/*
 * ap_gemm_kbit with K cut into `splits` ranges that different thread blocks take, for layers with few
 * blocks of 128 rows (a 4096-row layer has 32 of them for 148 SMs).  fp32 partial tiles go through the
 * workspace and are added in range order by the block that finishes a tile last, so results do not
 * depend on scheduling.  No counterpart in the reference.
 *   ap_gemm_kbit_splits(M, N, K)               the split count that gives about one block per SM (1 = none)
 *   ap_gemm_kbit_workspace_bytes(M, N, splits)  AP_TICKET_AREA_BYTES + splits * M * N * 4
 *   workspace  256-byte aligned device memory; its first AP_TICKET_AREA_BYTES are ticket counters, ZERO
 *              before the first call and left zero by every call (the same workspace can serve
 *              ap_matmul_kbit_splitk); the rest needs no initialisation.  Needs K % 256 == 0.
 */
int ap_gemm_kbit_splits(int M, int N, int K);
size_t ap_gemm_kbit_workspace_bytes(int M, int N, int splits);
int ap_gemm_kbit_splitk(const void* x, const void* qweight, int64_t plane_stride, const void* lut, void* out,
                        int M, int N, int K, int w_bits, int* status, int splits, void* workspace,
                        size_t workspace_bytes, void* stream);

/*
 * Tensor parallelism: one-shot all-reduce (sum) of the fp16 outputs of row-parallel layers over
 * peer memory.  No counterpart in the reference (single device).  Every rank stores its partial
 * result into an inbox on every rank, every 16-byte store carrying the call's sequence number beside
 * its 8 bytes of payload, polls (bounded) its own inbox until all ranks' lines carry that number and adds
 * them in rank order with fp32 accumulation, so that all ranks end with identical bits.  For the ranks of ONE node, one process per GPU.
 *
 * Set-up (these calls allocate, synchronise and are not for the serving loop):
 *   ap_comm_buffer_bytes(max_payload)  size of a rank's communication buffer for payloads of up to
 *                                      max_payload bytes (count * 2) and up to 8 ranks
 *   ap_comm_alloc / ap_comm_free       cudaMalloc'ed, zero-filled buffer on the current device
 *   ap_comm_export                     64-byte CUDA IPC handle of a buffer, to be sent to the peers
 *   ap_comm_open / ap_comm_close       map / unmap a peer's buffer from its handle
 *   ap_comm_last_error                 text of the last CUDA error seen by these calls
 * The call:
 *   ap_allreduce_oneshot(src, out, count, peer_buffers, rank, world, max_payload, status, stream)
 *     src, out      device fp16[count], 16-byte aligned, count a multiple of 8; may be the same
 *     peer_buffers  host array of `world` device pointers, entry `rank` being the caller's own
 *                   buffer, the others the mapped peer buffers; same max_payload on all ranks
 *     status        optional device int, set to 1 if a wait ran out (the output is then invalid;
 *                   nothing spins forever)
 *   All ranks must issue the same sequence of calls, call by call with the same count on every
 *   rank; the counts of consecutive calls may differ freely (the inbox generation is taken from a
 *   per-call counter, not from the call's size).  Calls of one communication buffer must be
 *   stream-ordered on each rank.  Nothing is allocated or synchronised; the call can be captured
 *   in a CUDA graph and replayed.
 *   ap_allreduce_oneshot_residual(src, out, rows, row_len, resid, norm_weight, ssq_out, ...)
 *     the same sum for a row-parallel layer's output [rows][row_len] that a pre-norm decoder adds to its
 *     residual stream: resid[rows][row_len] (fp16, 16-byte aligned, replicated on the ranks) += fp16(sum) in
 *     place, out = new resid * norm_weight[row_len] (NOT yet divided by the root mean square), and
 *     ssq_out[rows][b] (fp32), b < ap_allreduce_residual_blocks(rows, row_len), the sums of squares of the new
 *     resid over the blocks' ranges: the x, ssq and ssq_blocks of ap_matmul_kbit_prenorm (width = row_len).
 *     Counts as one call of the sequence above.  ap_allreduce_residual_blocks returns 0 where the shape is not
 *     supported (rows * blocks above 64).
 *   ap_matmul_kbit_push + ap_allreduce_oneshot_collect
 *     the all-reduce of a row-parallel product with its first step done by the product itself: the decode kernel's
 *     epilogue stores every finished tile straight into the inboxes of all ranks (no local result), and the collect
 *     call polls, sums in rank order and, with `resid` given, does what ap_allreduce_oneshot_residual does after its
 *     sum (resid NULL: out = the sum).  The pair counts as one call of the sequence; every rank must use the pair (or
 *     the one-kernel form) for the same call.  ap_matmul_kbit_push: operands and limits as ap_matmul_kbit_gated
 *     (M <= 8, N % 16 == 0, fast-kernel operands), M * N * 2 <= max_payload_bytes.
 */
int ap_matmul_kbit_push(const void* x, const void* qweight, int64_t plane_stride, const void* lut, int M, int N, int K,
                        int w_bits, int splits, void* workspace, size_t workspace_bytes, void* const* peer_buffers,
                        int rank, int world, size_t max_payload_bytes, void* stream);
int ap_allreduce_oneshot_collect(void* out, int rows, int row_len, void* resid, const void* norm_weight, void* ssq_out,
                                 void* const* peer_buffers, int rank, int world, size_t max_payload_bytes, int* status,
                                 void* stream);
int ap_allreduce_residual_blocks(int rows, int row_len);
int ap_allreduce_oneshot_residual(const void* src, void* out, int rows, int row_len, void* resid, const void* norm_weight,
                                  void* ssq_out, void* const* peer_buffers, int rank, int world, size_t max_payload_bytes,
                                  int* status, void* stream);
size_t ap_comm_buffer_bytes(size_t max_payload_bytes);
int ap_comm_alloc(size_t bytes, void** ptr);
int ap_comm_free(void* ptr);
int ap_comm_export(void* ptr, unsigned char* handle64);
int ap_comm_open(const unsigned char* handle64, void** ptr);
int ap_comm_close(void* ptr);
const char* ap_comm_last_error(void);
int ap_allreduce_oneshot(const void* src, void* out, int count, void* const* peer_buffers, int rank, int world,
                         size_t max_payload_bytes, int* status, void* stream);

/*
 * The packed format on the device.  ap_pack_codes replaces the bitplane loop and byte permutation of the
 * reference's CPU packer (any_precision/quantization/pack.py:12-76,86-99): codes uint8 [N][K] (values below
 * 2^parent_bits, rows 8-byte aligned: K % 32 == 0 and an 8-byte aligned base) -> qweight int32
 * [parent_bits][N][K/32], plane 0 = MSB.  ap_unpack_codes is the inverse for the top w_bits planes
 * (codes of precision w_bits); the reference has it only implicitly, in its kernels.  Used to build
 * operands and to re-pack K-shards whose last group is partial.
 */
int ap_pack_codes(const void* codes, void* qweight, int64_t plane_stride, int N, int K, int parent_bits, void* stream);
int ap_unpack_codes(const void* qweight, int64_t plane_stride, void* codes, int N, int K, int w_bits, void* stream);

/*
 * Element-wise operations between the linear layers of a Llama-style decoder step, so that a decode
 * step is a few launches per layer.  No counterpart in the reference's kernels: the reference runs the
 * stock Hugging Face decoder layer around its linears (any_precision/modules/AnyPrecisionForCausalLM.py:
 * 54-60; its fuse_layers, :186-190, is a stub).  fp16 in and out, fp32 arithmetic, launched as
 * programmatic dependents like the other kernels.
 *   ap_add_rmsnorm  h[rows][hidden] += delta (delta may be NULL), then y = h * rsqrt(mean(h^2) + eps) * weight
 *   ap_rope_cache   qkv[rows][(heads + 2 kv_heads) * head_dim] holds q | k | v of one token per row;
 *                   q is rotated in place (pairs (i, i + head_dim/2)), rotated k and plain v are stored
 *                   at position pos[row] of sequence row / rows_per_seq in k_cache / v_cache
 *                   [sequences][kv_heads][max_seq][head_dim] (rows_per_seq = 1 for a decode step).
 *                   cos_sin: fp32 [max_seq][head_dim] = cos(head_dim/2) | sin(head_dim/2) per position;
 *                   pos: device int32[rows] (a row whose position is outside [0, max_seq) is skipped)
 *   ap_silu_mul     y[rows][ffn] = silu(gate) * up for gate_up[rows][2 * ffn] = gate | up, or (tiled != 0,
 *                   ffn % 8 == 0) of every 16 values eight gate then eight up values of the same features:
 *                   the output of a plain product with the operand of ap_matmul_kbit_gated
 *   ap_decode_attention  one query token per sequence: out[b][h][:] = softmax(q . K[0..pos[b]] * scale) V[0..pos[b]]
 *                   with q = qkv[b * q_row_stride + h * head_dim ...] (the rotated q part of the q|k|v row),
 *                   caches as in ap_rope_cache, grouped-query heads (heads % kv_heads == 0), head_dim 32, 64,
 *                   128 or 256, out fp16 [sequences][heads * head_dim].  `splits` > 1 cuts every head's cached
 *                   positions into that many ranges taken by different thread blocks (a decode step has few
 *                   heads); it needs `scratch`: 16-byte aligned device memory of
 *                   ap_decode_attention_scratch_bytes(...) bytes whose first sequences * heads ints are ticket
 *                   counters, ZERO before the first call and left zero by every call
 *   ap_decode_attention_rope  ap_rope_cache (rows_per_seq = 1) and ap_decode_attention in one launch: the rows of
 *                   qkv are the RAW q | k | v of the new token (q_row_stride >= (heads + 2 kv_heads) * head_dim, a
 *                   multiple of 8; head_dim a multiple of 16), the caches hold the earlier positions; q and k are
 *                   rotated on the fly, the rotated k and v of position pos[b] are stored in the caches (qkv itself
 *                   is left as it was), and the result equals the two separate calls bit for bit.  A position
 *                   outside [0, max_seq) rotates and stores nothing, as in ap_rope_cache.
 */
int ap_add_rmsnorm(void* h, const void* delta, const void* weight, void* y, int rows, int hidden, float eps,
                   void* stream);
int ap_rope_cache(void* qkv, const void* cos_sin, const void* pos, void* k_cache, void* v_cache, int rows,
                  int rows_per_seq, int heads, int kv_heads, int head_dim, int max_seq, void* stream);
int ap_silu_mul(const void* gate_up, void* y, int rows, int ffn, int tiled, void* stream);
size_t ap_decode_attention_scratch_bytes(int sequences, int heads, int head_dim, int splits);
int ap_decode_attention(const void* qkv, int q_row_stride, const void* k_cache, const void* v_cache, const void* pos,
                        void* out, int sequences, int heads, int kv_heads, int head_dim, int max_seq, float scale,
                        int splits, void* scratch, void* stream);
int ap_decode_attention_rope(const void* qkv, int q_row_stride, const void* cos_sin, void* k_cache, void* v_cache,
                             const void* pos, void* out, int sequences, int heads, int kv_heads, int head_dim, int max_seq,
                             float scale, int splits, void* scratch, void* stream);

/*
 * Seed + incremental-upscale quantisation of a weight matrix, one thread block per row.  Replaces the
 * reference's CPU routine any_precision/quantization/quantize.py:85-187 (_seed_and_upscale_layer, numba) with
 * its helpers :13-76 and the two 1-D k-means routines it takes from the flash1dkmeans package (restated with
 * a deterministic start; see the kernel's file header).  group_count = 1 only (one table per row), as the
 * reference's packer requires (pack.py:126-127).
 *   weight, sensitivity  fp32 [N][K] (sensitivity = the sample weights, e.g. squared gradients; >= 0)
 *   codes                uint8 [N][K]: parent_bits-bit cluster index of every weight; its top b bits index
 *                        the b-bit table
 *   luts                 fp16: for b = seed_bits .. parent_bits in turn a table [N][2^b], one after the other
 *                        (N * (2^(parent_bits + 1) - 2^seed_bits) halfs in all), ascending along a row
 *   max_iter             Lloyd assignments of the seed k-means (the reference passes 50, quantize.py:148)
 *   workspace            8-byte aligned device memory, ap_seed_upscale_workspace_bytes(K, blocks) bytes for
 *                        `blocks` rows in flight; the call runs min(N, workspace_bytes / (16 K)) blocks
 * 1 <= seed_bits <= parent_bits <= 8; K <= 32768 (a row is sorted in shared memory), else AP_ERR_UNSUPPORTED.
 * Weights must be finite.  Equal values keep their original order in the sort.
 */
size_t ap_seed_upscale_workspace_bytes(int K, int blocks);
int ap_seed_upscale(const void* weight, const void* sensitivity, int N, int K, int seed_bits, int parent_bits,
                    int max_iter, void* codes, void* luts, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* ANYPREC_B200_H */
