// Second pass of a split-K product: sums the fp32 partial results that the tensor-core kernels
// wrote to a workspace laid out [split][batch][M][N] (dense, N contiguous), in split order with
// rounded fp32 adds, then applies bias and activation, rounds once to the output type and stores
// through the output view's strides.
#pragma once
#include "gemm_tcgen05.cuh"

namespace srt {

struct ReduceParams {
    const float* ws;
    uint32_t splits;
    unsigned long long slice;        // elements per split: batch * M * N
    uint32_t M, N, batch;
    void* out;
    long long o_b, o_m, o_n;         // element strides of the output view
    const void* bias;
    long long bias_stride;
    uint32_t bias_mode;              // 0 none, 1 one value per column, 2 one value per row
    uint32_t act;
};

// VEC consecutive columns per thread (4 when N is a multiple of 4, else 1).
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const ReduceParams p)
{
    // launched as a programmatic dependent of the partial-sum kernel: scheduled early, held here until
    // that kernel has completed and its partial sums are visible
    grid_dependency_wait();
    const unsigned long long groups = p.slice / VEC;
    const T* const bias = static_cast<const T*>(p.bias);
    T* const out = static_cast<T*>(p.out);
    for (unsigned long long g = blockIdx.x * 256ull + threadIdx.x; g < groups; g += gridDim.x * 256ull) {
        const unsigned long long idx = g * VEC;
        float acc[VEC];
        if constexpr (VEC == 4) {
            const float4 v = *reinterpret_cast<const float4*>(p.ws + idx);
            acc[0] = v.x; acc[1] = v.y; acc[2] = v.z; acc[3] = v.w;
            for (uint32_t s = 1; s < p.splits; ++s) {
                const float4 w = *reinterpret_cast<const float4*>(p.ws + s * p.slice + idx);
                acc[0] = __fadd_rn(acc[0], w.x); acc[1] = __fadd_rn(acc[1], w.y);
                acc[2] = __fadd_rn(acc[2], w.z); acc[3] = __fadd_rn(acc[3], w.w);
            }
        } else {
            acc[0] = p.ws[idx];
            for (uint32_t s = 1; s < p.splits; ++s) acc[0] = __fadd_rn(acc[0], p.ws[s * p.slice + idx]);
        }
        const uint32_t n = static_cast<uint32_t>(idx % p.N);
        const unsigned long long row_index = idx / p.N;
        const uint32_t m = static_cast<uint32_t>(row_index % p.M);
        const uint32_t b = static_cast<uint32_t>(row_index / p.M);
        T* dst = out + static_cast<long long>(b) * p.o_b + static_cast<long long>(m) * p.o_m + static_cast<long long>(n) * p.o_n;
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            float v = acc[j];
            if (p.bias_mode == 1) v = __fadd_rn(v, to_float<T>(bias[static_cast<long long>(n + j) * p.bias_stride]));
            else if (p.bias_mode == 2) v = __fadd_rn(v, to_float<T>(bias[static_cast<long long>(m) * p.bias_stride]));
            v = apply_activation(p.act, v);
            dst[static_cast<long long>(j) * p.o_n] = from_float<T>(v);
        }
    }
}

}  // namespace srt
