// Install-time conversion of a weight tensor from one of the boundary formats to the
// internal layout described in kernels.h.  Runs once per tensor; not on the hot path.
//
// Boundary 2-bit code (cuda/ter_cuda_forward_packed.cu:371-372): 0 -> 0, 1 -> +1,
// 2 -> -1, 3 -> 0.  Internal code: u = trit + 1.
#include "kernels.h"

namespace terb {

namespace {

// boundary code -> internal code, per 2-bit field: 0->1, 1->2, 2->0, 3->1
__device__ __forceinline__ uint32_t recode_byte(uint32_t b) {
    uint32_t out = 0;
#pragma unroll
    for (int f = 0; f < 4; ++f) {
        uint32_t c = (b >> (2 * f)) & 3u;
        uint32_t u = (c == 1u) ? 2u : ((c == 2u) ? 0u : 1u);
        out |= u << (2 * f);
    }
    return out;
}

__global__ void recode_v11_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int K, int nbc,
                                  int Kpad, int nbc_pad) {
    const size_t total = (size_t)nbc_pad * (size_t)Kpad;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int jb = (int)(i / (size_t)Kpad), k = (int)(i % (size_t)Kpad);
        uint32_t v = 0x55u;
        if (jb < nbc && k < K) v = recode_byte(src[(size_t)jb * K + k]);
        dst[weight_offset(jb, k, Kpad)] = (uint8_t)v;
    }
}

__global__ void recode_rowmajor_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int K, int nbc,
                                       int Kpad, int nbc_pad) {
    const size_t total = (size_t)nbc_pad * (size_t)Kpad;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int jb = (int)(i / (size_t)Kpad), k = (int)(i % (size_t)Kpad);
        uint32_t v = 0x55u;
        if (jb < nbc && k < K) v = recode_byte(src[(size_t)k * nbc + jb]);
        dst[weight_offset(jb, k, Kpad)] = (uint8_t)v;
    }
}

__global__ void pack_i32_kernel(const int32_t* __restrict__ src, uint8_t* __restrict__ dst, int K, int N, int Kpad,
                                int nbc_pad, int* __restrict__ bad_count) {
    const size_t total = (size_t)nbc_pad * (size_t)Kpad;
    int bad = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int jb = (int)(i / (size_t)Kpad), k = (int)(i % (size_t)Kpad);
        uint32_t v = 0x55u;
        if (k < K) {
            v = 0;
#pragma unroll
            for (int f = 0; f < 4; ++f) {
                const int j = 4 * jb + f;
                int t = 0;
                if (j < N) {
                    t = src[(size_t)k * N + j];
                    if (t < -1 || t > 1) { ++bad; t = 0; }
                }
                v |= (uint32_t)(t + 1) << (2 * f);
            }
        }
        dst[weight_offset(jb, k, Kpad)] = (uint8_t)v;
    }
    if (bad) atomicAdd(bad_count, bad);
}

inline int grid_for(size_t total) {
    size_t g = (total + 255) / 256;
    return (int)(g > 148 * 16 ? 148 * 16 : (g < 1 ? 1 : g));
}

}  // namespace

cudaError_t launch_recode_v11(const uint8_t* src, uint8_t* dst, int K, int N, int Kpad, int Npad, cudaStream_t st) {
    recode_v11_kernel<<<grid_for((size_t)(Npad / 4) * Kpad), 256, 0, st>>>(src, dst, K, N / 4, Kpad, Npad / 4);
    return cudaGetLastError();
}
cudaError_t launch_recode_rowmajor(const uint8_t* src, uint8_t* dst, int K, int N, int Kpad, int Npad,
                                   cudaStream_t st) {
    recode_rowmajor_kernel<<<grid_for((size_t)(Npad / 4) * Kpad), 256, 0, st>>>(src, dst, K, N / 4, Kpad, Npad / 4);
    return cudaGetLastError();
}
cudaError_t launch_pack_i32(const int32_t* src, uint8_t* dst, int K, int N, int Kpad, int Npad, int* bad_count,
                            cudaStream_t st) {
    pack_i32_kernel<<<grid_for((size_t)(Npad / 4) * Kpad), 256, 0, st>>>(src, dst, K, N, Kpad, Npad / 4, bad_count);
    return cudaGetLastError();
}

}  // namespace terb
