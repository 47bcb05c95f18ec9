// Lab harness for the decode kernel: times back-to-back launches of distinct layers and, in a build with
// -DAP_GEMV_PROFILE, prints per-launch phase stamps (%globaltimer, per thread block: start, dependents
// released, tables built, dependency wait returned, first chunk landed, arithmetic done, end).
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I include [-DAP_GEMV_PROFILE] \
//        [-DAP_GEMV_LAB_NO_WORD_MATH] -o gemv_phase_stamps any-precision-llm_b200/examples/gemv_phase_stamps.cu
//   ./gemv_phase_stamps N K M w_bits_digits         e.g.  ./gemv_phase_stamps 4096 11008 1 348
//
// -DAP_GEMV_LAB_NO_WORD_MATH removes the per-word arithmetic (bit transposes, lookups, MMAs) and keeps
// everything else of the kernel: what remains is the cost of the launch, the loader and the epilogue.
// The stamps of a launch are told apart by its output pointer (launch l writes out + l * stride).
#include "../csrc/ap_gemv.cu"

#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <vector>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); exit(1); } } while (0)

__global__ void fill_words(uint32_t* p, size_t n, uint32_t seed) {
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    const size_t st = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += st) {
        uint32_t x = (uint32_t)i * 2654435761u + seed;
        x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
        p[i] = x;
    }
}
__global__ void fill_halfs(__half* p, size_t n, uint32_t seed, float scale) {
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    const size_t st = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += st) {
        uint32_t x = (uint32_t)i * 2654435761u + seed;
        x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15;
        p[i] = __float2half(((x & 0xffff) / 65536.f - 0.5f) * scale);
    }
}

int main(int argc, char** argv) {
    if (argc < 5) { printf("usage: %s N K M w_bits_digits\n", argv[0]); return 2; }
    const int N = atoi(argv[1]), K = atoi(argv[2]), M = atoi(argv[3]);
    const char* wlist = argv[4];
    const int L = 12;                                        // distinct layers per sequence (operands larger than L2)
    std::vector<uint32_t*> q(L);
    std::vector<__half*> lut(L);
    __half *x, *out;
    const size_t qn = (size_t)8 * N * K / 32;
    for (int i = 0; i < L; i++) {
        CK(cudaMalloc(&q[i], qn * 4));
        fill_words<<<1024, 256>>>(q[i], qn, i);
        CK(cudaMalloc(&lut[i], (size_t)N * 256 * 2));
        fill_halfs<<<256, 256>>>(lut[i], (size_t)N * 256, i, 0.04f);
    }
    const long long stride = ((long long)M * N * 2 + 255) / 256 * 256;
    CK(cudaMalloc(&x, (size_t)M * K * 2));
    fill_halfs<<<64, 256>>>(x, (size_t)M * K, 99, 2.f);
    CK(cudaMalloc(&out, (size_t)stride * L));
    CK(cudaDeviceSynchronize());
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    for (const char* wp = wlist; *wp; wp++) {
        const int w = *wp - '0';
        if (w < 3 || w > 8) continue;
        auto seq = [&]() {
            for (int i = 0; i < L; i++)
                CK(ap::launch_gemv(x, q[i], (long long)N * K / 32, lut[i], (char*)out + stride * i, M, N, K, w, 1, nullptr, nullptr, 0));
        };
#ifdef AP_GEMV_PROFILE
        const long long zero = 0;
        const char* base = (const char*)out;
        CK(cudaMemcpyToSymbol(ap::ap_prof_out_stride, &zero, sizeof zero));
#endif
        for (int it = 0; it < 3; it++) seq();
        CK(cudaDeviceSynchronize());
        cudaEventRecord(e0);
        for (int it = 0; it < 5; it++) seq();
        cudaEventRecord(e1);
        CK(cudaDeviceSynchronize());
        float ms;
        cudaEventElapsedTime(&ms, e0, e1);
        const double us = ms * 1e3 / (5 * L);
        const double bytes = (double)N * K * w / 8 + (double)N * (1 << w) * 2 + M * K * 2 + M * N * 2;
        printf("== N=%d K=%d w=%d M=%d: %.2f us/launch  %.0f GB/s\n", N, K, w, M, us, bytes / us / 1e3);
#ifdef AP_GEMV_PROFILE
        CK(cudaMemcpyToSymbol(ap::ap_prof_out_base, &base, sizeof base));
        CK(cudaMemcpyToSymbol(ap::ap_prof_out_stride, &stride, sizeof stride));
        CK(cudaDeviceSynchronize());
        seq();
        CK(cudaDeviceSynchronize());
        std::vector<unsigned long long> h((size_t)ap::kProfLaunches * ap::kProfBlocks * ap::kProfSlots);
        CK(cudaMemcpyFromSymbol(h.data(), ap::ap_gemv_prof, h.size() * 8));
        const int ctas = std::min(N / 16, ap::kProfBlocks);
        unsigned long long tref = ~0ull;
        for (int c = 0; c < ctas; c++) tref = std::min(tref, h[((size_t)4 * ap::kProfBlocks + c) * ap::kProfSlots + 0]);
        printf("   launch: start(min avg max) | dependents released | tables built | wait returned(min avg max) | first chunk | "
               "arithmetic done(avg max) | end(avg max)     [ns after the first block of launch 4]\n");
        for (int l = 4; l <= 8; l++) {
            double mn[16], av[16], mx[16];
            for (int s = 0; s < 16; s++) { mn[s] = 1e18; av[s] = 0; mx[s] = -1e18; }
            for (int c = 0; c < ctas; c++)
                for (int s = 0; s < 16; s++) {
                    const double t = (double)h[((size_t)l * ap::kProfBlocks + c) * ap::kProfSlots + s] - (double)tref;
                    mn[s] = std::min(mn[s], t); mx[s] = std::max(mx[s], t); av[s] += t / ctas;
                }
            printf("   %d: %6.0f %6.0f %6.0f | %6.0f | %6.0f | %6.0f %6.0f %6.0f | %6.0f | %6.0f %6.0f | %6.0f %6.0f\n", l, mn[0], av[0],
                   mx[0], av[6], av[1], mn[7], av[7], mx[7], av[2], av[3], mx[3], av[4], mx[4]);
        }
#endif
    }
    return 0;
}
