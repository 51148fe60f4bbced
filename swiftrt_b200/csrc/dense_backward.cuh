// Backward of the Dense epilogue: dz = dy * act'(y) and dbias = column sums of dz, in one pass
// over dy and y (HBM-bound: reads 2 and writes 1 element per output element).
//
//   pass 1  grid (column blocks, row chunks): each block walks its rows with 8 warps, a thread
//           owning VEC consecutive columns; dz is rounded to the element type and stored, the
//           ROUNDED values are summed per column in fp32; the block's column sums go to
//           partial[chunk][N] (fp32 scratch).
//   pass 2  dbias[n] = partial[0][n] + partial[1][n] + ... in chunk order (deterministic), one
//           rounding to the element type.
// The derivative uses the forward OUTPUT y (relu: y > 0, sigmoid: y (1 - y), tanh: 1 - y^2),
// as cuDNN's activation backward does in the reference
// (Sources/SwiftRTCore/platform/cuda/layers/CudaActivation.swift:101-127).  GELU is not a function
// of its own output, so for gelu / geluTanh the second tensor is the PRE-activation value z and the
// derivative is evaluated there:
//     gelu'(z)     = Phi(z) + z phi(z)                      (Phi, phi: standard normal cdf / pdf)
//     geluTanh'(z) = (1 + t) / 2 + z (1 - t^2) u'(z) / 2,   t = tanh(u), u = sqrt(2/pi) (z + 0.044715 z^3)
// activation_forward_kernel is the matching forward pass y = act(z) for layers that keep z.
#pragma once
#include "gemm_tcgen05.cuh"

namespace srt {

struct DenseBackwardParams {
    const void* dy; const void* y; void* dz;
    long long dy_b, dy_m, dy_n;      // element strides (batch, row, column)
    long long y_b, y_m, y_n;
    long long dz_b, dz_m, dz_n;
    uint32_t M, N, batch;            // rows per batch item, columns, batch items
    uint32_t rows_per_chunk;         // over the flattened batch * M rows
    uint32_t act;
    float* partial;                  // [chunks][N]
};

__device__ __forceinline__ float activation_grad(uint32_t act, float g, float o)
{
    switch (act) {
    case kActRelu: return o > 0.0f ? g : 0.0f;
    case kActSigmoid: return __fmul_rn(g, __fmul_rn(o, __fsub_rn(1.0f, o)));
    case kActTanh: return __fmul_rn(g, __fsub_rn(1.0f, __fmul_rn(o, o)));
    case kActGelu: {
        const float cdf = 0.5f * (1.0f + erff(o * 0.70710678118654752440f));
        const float pdf = 0.39894228040143267794f * expf(-0.5f * o * o);
        return g * (cdf + o * pdf);
    }
    case kActGeluTanh: {
        const float u = 0.7978845608028654f * (o + 0.044715f * o * o * o);
        const float t = tanhf(u);
        const float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * o * o);
        return g * (0.5f * (1.0f + t) + 0.5f * o * (1.0f - t * t) * du);
    }
    default: return g;
    }
}

// VEC consecutive columns per thread: 8 (16-bit) or 4 (fp32) with 16-byte accesses when every
// tensor is column-contiguous and aligned, else 1.
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
dense_backward_kernel(const DenseBackwardParams p)
{
    __shared__ float red[8][32 * VEC + 1];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t col0 = (blockIdx.x * 32 + lane) * VEC;
    const unsigned long long total_rows = static_cast<unsigned long long>(p.batch) * p.M;
    const unsigned long long r_begin = static_cast<unsigned long long>(blockIdx.y) * p.rows_per_chunk;
    unsigned long long r_end = r_begin + p.rows_per_chunk;
    if (r_end > total_rows) r_end = total_rows;
    const T* dy = static_cast<const T*>(p.dy);
    const T* y = static_cast<const T*>(p.y);
    T* dz = static_cast<T*>(p.dz);

    float sum[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) sum[j] = 0.0f;

    if (col0 < p.N) {
        // two rows per iteration: both rows' loads are issued before either row is used
        for (unsigned long long r = r_begin + warp; r < r_end; r += 16) {
            __align__(16) T g[2][VEC];
            __align__(16) T o[2][VEC];
            long long o_dz[2];
            bool live[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const unsigned long long ru = r + 8ull * u;
                live[u] = ru < r_end;
                if (!live[u]) continue;
                const uint32_t b = static_cast<uint32_t>(ru / p.M), m = static_cast<uint32_t>(ru % p.M);
                const long long o_dy = b * p.dy_b + m * p.dy_m + static_cast<long long>(col0) * p.dy_n;
                const long long o_y = b * p.y_b + m * p.y_m + static_cast<long long>(col0) * p.y_n;
                o_dz[u] = b * p.dz_b + m * p.dz_m + static_cast<long long>(col0) * p.dz_n;
                if constexpr (VEC > 1) {
                    *reinterpret_cast<uint4*>(g[u]) = *reinterpret_cast<const uint4*>(dy + o_dy);
                    if (y) *reinterpret_cast<uint4*>(o[u]) = *reinterpret_cast<const uint4*>(y + o_y);
                } else {
                    g[u][0] = dy[o_dy];
                    if (y) o[u][0] = y[o_y];
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (!live[u]) continue;
                __align__(16) T d[VEC];
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    const float gf = to_float<T>(g[u][j]);
                    const float df = y ? activation_grad(p.act, gf, to_float<T>(o[u][j])) : gf;
                    d[j] = from_float<T>(df);
                    sum[j] = __fadd_rn(sum[j], to_float<T>(d[j]));
                }
                if (dz) {
                    if constexpr (VEC > 1) *reinterpret_cast<uint4*>(dz + o_dz[u]) = *reinterpret_cast<const uint4*>(d);
                    else dz[o_dz[u]] = d[0];
                }
            }
        }
    }
    if (p.partial == nullptr) return;
#pragma unroll
    for (int j = 0; j < VEC; ++j) red[warp][lane * VEC + j] = sum[j];
    __syncthreads();
    // 8 warps x (32 * VEC) columns -> one sum per column, warps added in order
    for (uint32_t c = threadIdx.x; c < 32 * VEC; c += 256) {
        const uint32_t col = blockIdx.x * 32 * VEC + c;
        if (col >= p.N) continue;
        float s = red[0][c];
#pragma unroll
        for (int w = 1; w < 8; ++w) s = __fadd_rn(s, red[w][c]);
        p.partial[static_cast<unsigned long long>(blockIdx.y) * p.N + col] = s;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
dense_backward_finish_kernel(const float* partial, uint32_t chunks, uint32_t N, T* dbias, long long dbias_stride)
{
    const uint32_t n = blockIdx.x * 256 + threadIdx.x;
    if (n >= N) return;
    float s = partial[n];
    for (uint32_t c = 1; c < chunks; ++c) s = __fadd_rn(s, partial[static_cast<unsigned long long>(c) * N + n]);
    dbias[static_cast<long long>(n) * dbias_stride] = from_float<T>(s);
}

// y = act(z), elementwise over a rank-2/3 view (any strides; VEC as above).  Reuses
// DenseBackwardParams: dy = z (input), dz = y (output).
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
activation_forward_kernel(const DenseBackwardParams p)
{
    const unsigned long long cols = (p.N + VEC - 1) / VEC;
    const unsigned long long total = static_cast<unsigned long long>(p.batch) * p.M * cols;
    const T* z = static_cast<const T*>(p.dy);
    T* y = static_cast<T*>(p.dz);
    for (unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < total; i += gridDim.x * 256ull) {
        const uint32_t c = static_cast<uint32_t>(i % cols) * VEC;
        const unsigned long long r = i / cols;
        const uint32_t b = static_cast<uint32_t>(r / p.M), m = static_cast<uint32_t>(r % p.M);
        const long long o_in = b * p.dy_b + m * p.dy_m + static_cast<long long>(c) * p.dy_n;
        const long long o_out = b * p.dz_b + m * p.dz_m + static_cast<long long>(c) * p.dz_n;
        if constexpr (VEC > 1) {
            __align__(16) T v[VEC];
            *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(z + o_in);
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[j] = from_float<T>(apply_activation(p.act, to_float<T>(v[j])));
            *reinterpret_cast<uint4*>(y + o_out) = *reinterpret_cast<const uint4*>(v);
        } else {
            y[o_out] = from_float<T>(apply_activation(p.act, to_float<T>(z[o_in])));
        }
    }
}

}  // namespace srt
