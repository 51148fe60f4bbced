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

// VEC elements (16 bytes) per thread when both inputs are row-contiguous and 16-byte aligned and
// nx, nh are multiples of VEC; otherwise VEC = 1 with arbitrary strides.
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
concat_kernel(const ConcatParams p)
{
    const uint32_t wx = p.nx / VEC, wh = p.nh / VEC, width = wx + wh;      // chunks per output row
    const T* x = static_cast<const T*>(p.x);
    const T* h = static_cast<const T*>(p.h);
    T* out = static_cast<T*>(p.out);
    for (uint32_t r = blockIdx.x; r < p.rows; r += gridDim.x) {
        T* orow = out + static_cast<unsigned long long>(r) * (p.nx + p.nh);
        for (uint32_t c = threadIdx.x; c < width; c += 256) {
            if constexpr (VEC > 1) {
                const T* src = c < wx ? x + static_cast<long long>(r) * p.x_m + static_cast<long long>(c) * VEC
                                      : h + static_cast<long long>(r) * p.h_m + static_cast<long long>(c - wx) * VEC;
                *reinterpret_cast<uint4*>(orow + static_cast<unsigned long long>(c) * VEC) = *reinterpret_cast<const uint4*>(src);
            } else {
                orow[c] = c < wx ? x[static_cast<long long>(r) * p.x_m + static_cast<long long>(c) * p.x_n]
                                 : h[static_cast<long long>(r) * p.h_m + static_cast<long long>(c - wx) * p.h_n];
            }
        }
    }
}

// Gate nonlinearities.  Float32 uses the library functions (the reference's golden LSTM states are
// pinned to 1e-6); for 16-bit elements, whose rounding step is 2^-9 or 2^-12 of the value, the
// hardware exponential (relative error ~1e-6) is exact enough and several times cheaper.
template <typename T> __device__ __forceinline__ float gate_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
template <> __device__ __forceinline__ float gate_sigmoid<float>(float x) { return apply_activation(kActSigmoid, x); }
template <typename T> __device__ __forceinline__ float gate_tanh(float x) { return 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * x)); }
template <> __device__ __forceinline__ float gate_tanh<float>(float x) { return apply_activation(kActTanh, x); }

struct LstmGateParams {
    const void* fused;                           // dense [rows x 4 hidden]: input | update | forget | output
    const void* cell; void* new_cell; void* new_hidden;
    long long c_m, c_n, nc_m, nc_n, nh_m, nh_n;  // element strides
    uint32_t rows, hidden;
};

// One thread per VEC consecutive hidden units of one row (VEC = 16 bytes' worth when the state
// tensors are row-contiguous and aligned, else 1).
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
lstm_gates_kernel(const LstmGateParams p)
{
    const uint32_t hchunks = p.hidden / VEC;
    const uint32_t rows_per_pass = 256 / (hchunks < 256 ? hchunks : 256);       // >= 1
    const T* fused = static_cast<const T*>(p.fused);
    const T* cell = static_cast<const T*>(p.cell);
    T* new_cell = static_cast<T*>(p.new_cell);
    T* new_hidden = static_cast<T*>(p.new_hidden);
    // a block walks row groups; inside a group thread t owns (row t / hchunks, chunk t % hchunks) when a
    // row is narrower than the block, else chunks t, t + 256, ... of one row
    for (uint32_t r0 = blockIdx.x * rows_per_pass; r0 < p.rows; r0 += gridDim.x * rows_per_pass) {
        const uint32_t sub = hchunks < 256 ? threadIdx.x / hchunks : 0;
        const uint32_t r = r0 + sub;
        if (sub >= rows_per_pass || r >= p.rows) continue;
        const T* frow = fused + static_cast<unsigned long long>(r) * 4 * p.hidden;
        for (uint32_t ch = hchunks < 256 ? threadIdx.x % hchunks : threadIdx.x; ch < hchunks; ch += 256) {
            const uint32_t j0 = ch * VEC;
            __align__(16) T gi[VEC], gu[VEC], gf[VEC], go[VEC], c[VEC], nc[VEC], nh[VEC];
            if constexpr (VEC > 1) {
                *reinterpret_cast<uint4*>(gi) = *reinterpret_cast<const uint4*>(frow + j0);
                *reinterpret_cast<uint4*>(gu) = *reinterpret_cast<const uint4*>(frow + p.hidden + j0);
                *reinterpret_cast<uint4*>(gf) = *reinterpret_cast<const uint4*>(frow + 2 * p.hidden + j0);
                *reinterpret_cast<uint4*>(go) = *reinterpret_cast<const uint4*>(frow + 3 * p.hidden + j0);
                *reinterpret_cast<uint4*>(c) = *reinterpret_cast<const uint4*>(cell + static_cast<long long>(r) * p.c_m + j0);
            } else {
                gi[0] = frow[j0]; gu[0] = frow[p.hidden + j0]; gf[0] = frow[2 * p.hidden + j0]; go[0] = frow[3 * p.hidden + j0];
                c[0] = cell[static_cast<long long>(r) * p.c_m + static_cast<long long>(j0) * p.c_n];
            }
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                const float i = gate_sigmoid<T>(to_float<T>(gi[v]));
                const float u = gate_tanh<T>(to_float<T>(gu[v]));
                const float f = gate_sigmoid<T>(to_float<T>(gf[v]));
                const float o = gate_sigmoid<T>(to_float<T>(go[v]));
                nc[v] = from_float<T>(__fadd_rn(__fmul_rn(to_float<T>(c[v]), f), __fmul_rn(i, u)));
                nh[v] = from_float<T>(__fmul_rn(gate_tanh<T>(to_float<T>(nc[v])), o));
            }
            if constexpr (VEC > 1) {
                *reinterpret_cast<uint4*>(new_cell + static_cast<long long>(r) * p.nc_m + j0) = *reinterpret_cast<const uint4*>(nc);
                *reinterpret_cast<uint4*>(new_hidden + static_cast<long long>(r) * p.nh_m + j0) = *reinterpret_cast<const uint4*>(nh);
            } else {
                new_cell[static_cast<long long>(r) * p.nc_m + static_cast<long long>(j0) * p.nc_n] = nc[0];
                new_hidden[static_cast<long long>(r) * p.nh_m + static_cast<long long>(j0) * p.nh_n] = nh[0];
            }
        }
    }
}

// Column order for the fused LSTM epilogue: out[r][4 j + g] = in[r][g hidden + j], i.e. the four gate columns of
// hidden unit j side by side (the reference keeps the gates as four column blocks, Recurrent.swift:173, 203-213).
// Run once per weight (and bias, rows = 1) when a cell is built.
struct InterleaveParams {
    const void* in; void* out;
    long long in_m, in_n, out_m;         // element strides (out columns are contiguous)
    uint32_t rows, hidden;
};

template <typename T>
__global__ void __launch_bounds__(256)
lstm_interleave_kernel(const InterleaveParams p)
{
    const unsigned long long cols = 4ull * p.hidden, total = cols * p.rows;
    const T* in = static_cast<const T*>(p.in);
    T* out = static_cast<T*>(p.out);
    for (unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < total; i += gridDim.x * 256ull) {
        const uint32_t r = static_cast<uint32_t>(i / cols), c = static_cast<uint32_t>(i % cols);
        const uint32_t j = c >> 2, g = c & 3;
        out[static_cast<long long>(r) * p.out_m + c] = in[static_cast<long long>(r) * p.in_m + static_cast<long long>(g * p.hidden + j) * p.in_n];
    }
}

// ---------------------------------------------------------------------------------------------
// GRU cell (Sources/SwiftRTLayers/Recurrent.swift:328-337), around two fused products:
//     [reset | update] = sigmoid([x | h] . [[resetW1 | updateW1], [resetW2 | updateW2]] + [resetB | updateB])
//     gateInput2       = [x | reset * h]                                   gru_reset_kernel (in place)
//     output           = tanh(gateInput2 . [[outputW1], [outputW2]] + outputB)
//     newState         = (1 - update) * h + (1 - update) * output          gru_state_kernel
// (the last line is the reference's formula as written: both terms carry 1 - update).
struct GruParams {
    void* gate_in;                   // dense [rows x (nx + nh)]: x | h, the h half is overwritten with reset * h
    const void* gates;               // dense [rows x 2 nh]: reset | update (after the sigmoid)
    const void* output;              // dense [rows x nh]: after the tanh
    const void* hidden; void* new_hidden;
    long long h_m, h_n, nh_m, nh_n;  // element strides
    uint32_t rows, nx, nh;
};

template <typename T>
__global__ void __launch_bounds__(256)
gru_reset_kernel(const GruParams p)
{
    T* cat = static_cast<T*>(p.gate_in);
    const T* gates = static_cast<const T*>(p.gates);
    const unsigned long long total = static_cast<unsigned long long>(p.rows) * p.nh;
    for (unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < total; i += gridDim.x * 256ull) {
        const uint32_t r = static_cast<uint32_t>(i / p.nh), j = static_cast<uint32_t>(i % p.nh);
        T* h = cat + static_cast<unsigned long long>(r) * (p.nx + p.nh) + p.nx + j;
        const float reset = to_float<T>(gates[static_cast<unsigned long long>(r) * 2 * p.nh + j]);
        *h = from_float<T>(__fmul_rn(reset, to_float<T>(*h)));
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
gru_state_kernel(const GruParams p)
{
    const T* gates = static_cast<const T*>(p.gates);
    const T* output = static_cast<const T*>(p.output);
    const T* hidden = static_cast<const T*>(p.hidden);
    T* new_hidden = static_cast<T*>(p.new_hidden);
    const unsigned long long total = static_cast<unsigned long long>(p.rows) * p.nh;
    for (unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < total; i += gridDim.x * 256ull) {
        const uint32_t r = static_cast<uint32_t>(i / p.nh), j = static_cast<uint32_t>(i % p.nh);
        const float update = to_float<T>(gates[static_cast<unsigned long long>(r) * 2 * p.nh + p.nh + j]);
        const float h = to_float<T>(hidden[static_cast<long long>(r) * p.h_m + static_cast<long long>(j) * p.h_n]);
        const float o = to_float<T>(output[i]);
        const float keep = __fsub_rn(1.0f, update);
        new_hidden[static_cast<long long>(r) * p.nh_m + static_cast<long long>(j) * p.nh_n] =
            from_float<T>(__fadd_rn(__fmul_rn(keep, h), __fmul_rn(keep, o)));
    }
}

}  // namespace srt
