// The packed bitplane format on the GPU: codes -> planes (the reference's packer) and back.
//
// The reference packs on the CPU with numpy/numba, one process per decoder layer
// (any_precision/quantization/pack.py:79-114: MSB-first bitplanes with np.packbits, then the per-row
// byte permutation of :12-76).  Here a thread produces one int32 word of every plane directly from
// the 32 codes that the format assigns to it: word t of a group of E words (E = 32 in a full
// 1024-weight group, (K % 1024) / 32 in the last, partial one), byte j from the most significant
// byte, bit e from that byte's most significant bit, is the plane bit of weight
//     k = group_base + 8 E j + 8 t + e,
// so the thread reads four runs of eight consecutive codes (8-byte loads).  Used to synthesise
// operands on the device and to re-pack K-shards for tensor parallelism; the inverse serves the
// same re-packing and the tests.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/anyprec_b200.h"

namespace {

__device__ __forceinline__ void word_geometry(int wd, int K, int& base, int& stride) {
    const int full_words = (K >> 10) << 5;
    if (wd < full_words) {
        base = (wd >> 5) * 1024 + (wd & 31) * 8;
        stride = 256;
    } else {
        base = full_words * 32 + (wd - full_words) * 8;
        stride = (K & 1023) >> 2;                            // 8 E of the partial group
    }
}

template <int P>
__global__ void __launch_bounds__(256)
pack_codes_kernel(const uint8_t* __restrict__ codes, uint32_t* __restrict__ q, long long plane_stride, int N, int K) {
    const int words = K >> 5;
    const long long total = (long long)N * words;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(idx / words), wd = (int)(idx % words);
        int base, stride;
        word_geometry(wd, K, base, stride);
        uint32_t out[P];
#pragma unroll
        for (int p = 0; p < P; p++) out[p] = 0u;
        const uint8_t* row = codes + (size_t)n * K + base;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint2 v = *reinterpret_cast<const uint2*>(row + (size_t)j * stride);   // eight codes, code e in byte e
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const uint32_t c = ((e < 4 ? v.x : v.y) >> (8 * (e & 3))) & 0xffu;
#pragma unroll
                for (int p = 0; p < P; p++) out[p] |= ((c >> (P - 1 - p)) & 1u) << (31 - (8 * j + e));
            }
        }
#pragma unroll
        for (int p = 0; p < P; p++) q[(size_t)p * plane_stride + idx] = out[p];
    }
}

__global__ void __launch_bounds__(256)
unpack_codes_kernel(const uint32_t* __restrict__ q, long long plane_stride, uint8_t* __restrict__ codes, int N, int K,
                    int w_bits) {
    const int words = K >> 5;
    const long long total = (long long)N * words;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(idx / words), wd = (int)(idx % words);
        int base, stride;
        word_geometry(wd, K, base, stride);
        uint32_t plane[8];
        for (int p = 0; p < w_bits; p++) plane[p] = q[(size_t)p * plane_stride + idx];
        uint8_t* row = codes + (size_t)n * K + base;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t lo = 0u, hi = 0u;
#pragma unroll
            for (int e = 0; e < 8; e++) {
                uint32_t c = 0u;
                for (int p = 0; p < w_bits; p++) c |= ((plane[p] >> (31 - (8 * j + e))) & 1u) << (w_bits - 1 - p);
                if (e < 4) lo |= c << (8 * e); else hi |= c << (8 * (e - 4));
            }
            *reinterpret_cast<uint2*>(row + (size_t)j * stride) = make_uint2(lo, hi);
        }
    }
}

int grid_for(long long total) {
    long long b = (total + 255) / 256;
    return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

}  // namespace

extern "C" int ap_pack_codes(const void* codes, void* qweight, int64_t plane_stride, int N, int K, int parent_bits,
                             void* stream) {
    if (!codes || !qweight) return AP_ERR_NULL_POINTER;
    if (N < 1 || K < 32 || K % 32 || plane_stride < (int64_t)N * (K / 32)) return AP_ERR_BAD_SHAPE;
    if (parent_bits < 1 || parent_bits > 8) return AP_ERR_BAD_BITS;
    if ((reinterpret_cast<uintptr_t>(codes) & 7) || (reinterpret_cast<uintptr_t>(qweight) & 3)) return AP_ERR_BAD_ALIGNMENT;
    const uint8_t* c = static_cast<const uint8_t*>(codes);
    uint32_t* q = static_cast<uint32_t*>(qweight);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = grid_for((long long)N * (K / 32));
    switch (parent_bits) {
        case 1: pack_codes_kernel<1><<<grid, 256, 0, st>>>(c, q, plane_stride, N, K); break;
        case 2: pack_codes_kernel<2><<<grid, 256, 0, st>>>(c, q, plane_stride, N, K); break;
        case 3: pack_codes_kernel<3><<<grid, 256, 0, st>>>(c, q, plane_stride, N, K); break;
        case 4: pack_codes_kernel<4><<<grid, 256, 0, st>>>(c, q, plane_stride, N, K); break;
        case 5: pack_codes_kernel<5><<<grid, 256, 0, st>>>(c, q, plane_stride, N, K); break;
        case 6: pack_codes_kernel<6><<<grid, 256, 0, st>>>(c, q, plane_stride, N, K); break;
        case 7: pack_codes_kernel<7><<<grid, 256, 0, st>>>(c, q, plane_stride, N, K); break;
        default: pack_codes_kernel<8><<<grid, 256, 0, st>>>(c, q, plane_stride, N, K); break;
    }
    return cudaGetLastError() == cudaSuccess ? AP_OK : AP_ERR_LAUNCH;
}

extern "C" int ap_unpack_codes(const void* qweight, int64_t plane_stride, void* codes, int N, int K, int w_bits,
                               void* stream) {
    if (!codes || !qweight) return AP_ERR_NULL_POINTER;
    if (N < 1 || K < 32 || K % 32 || plane_stride < (int64_t)N * (K / 32)) return AP_ERR_BAD_SHAPE;
    if (w_bits < 1 || w_bits > 8) return AP_ERR_BAD_BITS;
    if ((reinterpret_cast<uintptr_t>(codes) & 7) || (reinterpret_cast<uintptr_t>(qweight) & 3)) return AP_ERR_BAD_ALIGNMENT;
    unpack_codes_kernel<<<grid_for((long long)N * (K / 32)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint32_t*>(qweight), plane_stride, static_cast<uint8_t*>(codes), N, K, w_bits);
    return cudaGetLastError() == cudaSuccess ? AP_OK : AP_ERR_LAUNCH;
}
