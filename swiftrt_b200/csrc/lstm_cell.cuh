// The elementwise halves of one LSTM cell step around its fused product
// (Sources/SwiftRTLayers/Recurrent.swift:255-266):
//     gateInput = concatenate(input, hidden, axis: 1)              concat_kernel
//     fused     = matmul(gateInput, fusedWeight, bias: fusedBias)  the tensor-core / strided matmul
//     i, u, f, o = sigmoid, tanh, sigmoid, sigmoid of the four column blocks of fused
//     cell'   = cell * f + i * u                                    lstm_gates_kernel
//     hidden' = tanh(cell') * o
// Both kernels are HBM-bound streaming passes; the gate pass reads 4 + 1 and writes 2 elements per
// hidden unit.  Arithmetic is fp32 with one rounding per stored tensor: cell' is rounded to the
// element type first and hidden' is computed from the rounded value, as the reference does when it
// materialises newCellState before tanh.
#pragma once
#include "gemm_tcgen05.cuh"

namespace srt {

struct ConcatParams {
    const void* x; const void* h; void* out;     // out: dense [rows x (nx + nh)]
    long long x_m, x_n, h_m, h_n;                // element strides of the two inputs
    uint32_t rows, nx, nh;
};

template <typename T>
__global__ void __launch_bounds__(256)
concat_kernel(const ConcatParams p)
{
    const uint32_t width = p.nx + p.nh;
    const unsigned long long total = static_cast<unsigned long long>(p.rows) * width;
    for (unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < total; i += gridDim.x * 256ull) {
        const uint32_t r = static_cast<uint32_t>(i / width), c = static_cast<uint32_t>(i % width);
        const T* src = c < p.nx ? static_cast<const T*>(p.x) + static_cast<long long>(r) * p.x_m + static_cast<long long>(c) * p.x_n
                                : static_cast<const T*>(p.h) + static_cast<long long>(r) * p.h_m +
                                      static_cast<long long>(c - p.nx) * p.h_n;
        static_cast<T*>(p.out)[i] = *src;
    }
}

struct LstmGateParams {
    const void* fused;                           // dense [rows x 4 hidden]: input | update | forget | output
    const void* cell; void* new_cell; void* new_hidden;
    long long c_m, c_n, nc_m, nc_n, nh_m, nh_n;  // element strides
    uint32_t rows, hidden;
};

template <typename T>
__global__ void __launch_bounds__(256)
lstm_gates_kernel(const LstmGateParams p)
{
    const unsigned long long total = static_cast<unsigned long long>(p.rows) * p.hidden;
    const T* fused = static_cast<const T*>(p.fused);
    for (unsigned long long idx = blockIdx.x * 256ull + threadIdx.x; idx < total; idx += gridDim.x * 256ull) {
        const uint32_t r = static_cast<uint32_t>(idx / p.hidden), j = static_cast<uint32_t>(idx % p.hidden);
        const T* row = fused + static_cast<unsigned long long>(r) * 4 * p.hidden;
        const float gi = apply_activation(kActSigmoid, to_float<T>(row[j]));
        const float gu = apply_activation(kActTanh, to_float<T>(row[p.hidden + j]));
        const float gf = apply_activation(kActSigmoid, to_float<T>(row[2 * p.hidden + j]));
        const float go = apply_activation(kActSigmoid, to_float<T>(row[3 * p.hidden + j]));
        const float c = to_float<T>(static_cast<const T*>(p.cell)[static_cast<long long>(r) * p.c_m + static_cast<long long>(j) * p.c_n]);
        const T nc = from_float<T>(__fadd_rn(__fmul_rn(c, gf), __fmul_rn(gi, gu)));
        static_cast<T*>(p.new_cell)[static_cast<long long>(r) * p.nc_m + static_cast<long long>(j) * p.nc_n] = nc;
        const float nh = __fmul_rn(apply_activation(kActTanh, to_float<T>(nc)), go);
        static_cast<T*>(p.new_hidden)[static_cast<long long>(r) * p.nh_m + static_cast<long long>(j) * p.nh_n] = from_float<T>(nh);
    }
}

}  // namespace srt
