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

constexpr int kSimtTile = 64;       // default tile edge; 32 when a 64-tile grid would leave most SMs idle
constexpr int kSimtK = 16;          // k-tile of the 64 x 64 kernel; the 32 x 32 kernel takes 32 (half as many block-wide syncs)

// TILE x TILE outputs per 256-thread block, (TILE/16)^2 per thread.  The global loads of k-tile
// t + 1 are issued into registers before k-tile t is multiplied, so their latency overlaps the math.
// Small tiles are bound by the latency of one k-tile round trip (load, sync, multiply, sync), so
// they take a k-tile twice as deep.
template <typename T, int TILE>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const SimtParams p)
{
    constexpr int KT = TILE == 32 ? 32 : kSimtK;   // k-tile depth
    constexpr int R = TILE / 16;                   // outputs per thread along each axis
    constexpr int LD = TILE * KT / 256;            // elements of each operand tile a thread loads
    __shared__ float As[KT][TILE + 1];
    __shared__ float Bs[KT][TILE + 1];

    const uint32_t tid = threadIdx.x;
    const uint32_t tx = tid & 15, ty = tid >> 4;
    const uint32_t batch = blockIdx.z;
    const uint32_t m0 = blockIdx.y * TILE, n0 = blockIdx.x * TILE;
    const T* A = static_cast<const T*>(p.a) + static_cast<long long>(batch) * p.a_b;
    const T* B = static_cast<const T*>(p.b) + static_cast<long long>(batch) * p.b_b;

    float acc[R][R];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) acc[i][j] = 0.0f;

    // element e of a tile -> (row/column, k) so that consecutive threads walk the contiguous index
    uint32_t a_mm[LD], a_kk[LD], b_nn[LD], b_kk[LD];
#pragma unroll
    for (int i = 0; i < LD; ++i) {
        const uint32_t e = tid + i * 256;
        if (p.a_k_fast) { a_kk[i] = e % KT; a_mm[i] = e / KT; } else { a_mm[i] = e % TILE; a_kk[i] = e / TILE; }
        if (p.b_n_fast) { b_nn[i] = e % TILE; b_kk[i] = e / TILE; } else { b_kk[i] = e % KT; b_nn[i] = e / KT; }
    }
    auto fetch = [&](uint32_t k0, float (&ra)[LD], float (&rb)[LD]) {
#pragma unroll
        for (int i = 0; i < LD; ++i) {
            const uint32_t gm = m0 + a_mm[i], gk = k0 + a_kk[i];
            ra[i] = (gm < p.M && gk < p.K)
                        ? to_float<T>(A[static_cast<long long>(gm) * p.a_m + static_cast<long long>(gk) * p.a_k]) : 0.0f;
            const uint32_t gn = n0 + b_nn[i], gk2 = k0 + b_kk[i];
            rb[i] = (gn < p.N && gk2 < p.K)
                        ? to_float<T>(B[static_cast<long long>(gk2) * p.b_k + static_cast<long long>(gn) * p.b_n]) : 0.0f;
        }
    };

    float ra[LD], rb[LD];
    fetch(0, ra, rb);
    for (uint32_t k0 = 0; k0 < p.K; k0 += KT) {
#pragma unroll
        for (int i = 0; i < LD; ++i) {
            As[a_kk[i]][a_mm[i]] = ra[i];
            Bs[b_kk[i]][b_nn[i]] = rb[i];
        }
        __syncthreads();
        if (k0 + KT < p.K) fetch(k0 + KT, ra, rb);
        const uint32_t kmax = min(static_cast<uint32_t>(KT), p.K - k0);
        for (uint32_t kk = 0; kk < kmax; ++kk) {
            float av[R], bv[R];
#pragma unroll
            for (int i = 0; i < R; ++i) av[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < R; ++j) bv[j] = Bs[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < R; ++i)
#pragma unroll
                for (int j = 0; j < R; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
        }
        __syncthreads();
    }

    T* O = static_cast<T*>(p.out) + static_cast<long long>(batch) * p.o_b;
    const T* bias = static_cast<const T*>(p.bias);
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const uint32_t gm = m0 + ty + 16 * i;
        if (gm >= p.M) continue;
#pragma unroll
        for (int j = 0; j < R; ++j) {
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
