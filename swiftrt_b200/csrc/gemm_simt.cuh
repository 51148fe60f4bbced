// Strided SIMT GEMM: the path for views that TMA cannot address (unaligned bases, strides
// that are not multiples of 16 bytes, no unit stride, overlapping or repeated elements),
// for outputs with arbitrary strides, and for fp32 when exact fp32 products are wanted.
//
// Every output element is accumulated by one thread in k = 0 .. K-1 order with a rounded
// fp32 product followed by a rounded fp32 add (no fused multiply-add), which is the
// accumulation order and rounding of the reference CPU loop
// (Sources/SwiftRTCore/platform/cpu/functions/CpuMath.swift:1141-1161); the tiling only
// changes which thread owns which element.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_tcgen05.cuh"   // conversions and apply_activation

namespace srt {

struct SimtParams {
    uint32_t M, N, K, batch;
    const void* a; const void* b; void* out; const void* bias;
    long long a_b, a_m, a_k;     // element strides of the logical operands
    long long b_b, b_k, b_n;
    long long o_b, o_m, o_n;
    long long bias_stride;
    uint32_t has_bias, act;
    uint32_t a_k_fast, b_n_fast; // which index the loader walks fastest (coalescing only)
};

constexpr int kSimtTile = 64;
constexpr int kSimtK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const SimtParams p)
{
    __shared__ float As[kSimtK][kSimtTile + 1];
    __shared__ float Bs[kSimtK][kSimtTile + 1];

    const uint32_t tid = threadIdx.x;
    const uint32_t tx = tid & 15, ty = tid >> 4;
    const uint32_t batch = blockIdx.z;
    const uint32_t m0 = blockIdx.y * kSimtTile, n0 = blockIdx.x * kSimtTile;
    const T* A = static_cast<const T*>(p.a) + static_cast<long long>(batch) * p.a_b;
    const T* B = static_cast<const T*>(p.b) + static_cast<long long>(batch) * p.b_b;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (uint32_t k0 = 0; k0 < p.K; k0 += kSimtK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t e = tid + i * 256;          // 1024 elements per tile
            uint32_t mm, kk;
            if (p.a_k_fast) { kk = e & 15; mm = e >> 4; } else { mm = e & 63; kk = e >> 6; }
            const uint32_t gm = m0 + mm, gk = k0 + kk;
            As[kk][mm] = (gm < p.M && gk < p.K)
                             ? to_float<T>(A[static_cast<long long>(gm) * p.a_m + static_cast<long long>(gk) * p.a_k])
                             : 0.0f;
            uint32_t nn, kb;
            if (p.b_n_fast) { nn = e & 63; kb = e >> 6; } else { kb = e & 15; nn = e >> 4; }
            const uint32_t gn = n0 + nn, gk2 = k0 + kb;
            Bs[kb][nn] = (gn < p.N && gk2 < p.K)
                             ? to_float<T>(B[static_cast<long long>(gk2) * p.b_k + static_cast<long long>(gn) * p.b_n])
                             : 0.0f;
        }
        __syncthreads();
        const uint32_t kmax = min(static_cast<uint32_t>(kSimtK), p.K - k0);
        for (uint32_t kk = 0; kk < kmax; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
        }
        __syncthreads();
    }

    T* O = static_cast<T*>(p.out) + static_cast<long long>(batch) * p.o_b;
    const T* bias = static_cast<const T*>(p.bias);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t gm = m0 + ty + 16 * i;
        if (gm >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t gn = n0 + tx + 16 * j;
            if (gn >= p.N) continue;
            float v = acc[i][j];
            if (p.has_bias) v = __fadd_rn(v, to_float<T>(bias[static_cast<long long>(gn) * p.bias_stride]));
            v = apply_activation(p.act, v);
            O[static_cast<long long>(gm) * p.o_m + static_cast<long long>(gn) * p.o_n] = from_float<T>(v);
        }
    }
}

}  // namespace srt
