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

constexpr uint32_t kInFlight = 4;     // slices whose loads are issued together

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
        // the slices are added in split order, but their loads are issued kInFlight at a time: a chain of
        // dependent L2 round trips would otherwise set the duration of this pass
        float acc[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[j] = 0.0f;
        for (uint32_t s0 = 0; s0 < p.splits; s0 += kInFlight) {
            if constexpr (VEC == 4) {
                float4 w[kInFlight];
#pragma unroll
                for (uint32_t j = 0; j < kInFlight; ++j)
                    if (s0 + j < p.splits) w[j] = *reinterpret_cast<const float4*>(p.ws + (s0 + j) * p.slice + idx);
#pragma unroll
                for (uint32_t j = 0; j < kInFlight; ++j)
                    if (s0 + j < p.splits) {
                        if (s0 + j == 0) { acc[0] = w[j].x; acc[1] = w[j].y; acc[2] = w[j].z; acc[3] = w[j].w; }
                        else {
                            acc[0] = __fadd_rn(acc[0], w[j].x); acc[1] = __fadd_rn(acc[1], w[j].y);
                            acc[2] = __fadd_rn(acc[2], w[j].z); acc[3] = __fadd_rn(acc[3], w[j].w);
                        }
                    }
            } else {
                float w[kInFlight];
#pragma unroll
                for (uint32_t j = 0; j < kInFlight; ++j)
                    if (s0 + j < p.splits) w[j] = p.ws[(s0 + j) * p.slice + idx];
#pragma unroll
                for (uint32_t j = 0; j < kInFlight; ++j)
                    if (s0 + j < p.splits) acc[0] = (s0 + j == 0) ? w[j] : __fadd_rn(acc[0], w[j]);
            }
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

// The same pass for an output whose contiguous dimension is M (a transposed plan: column-order
// results, and the small-batch plans whose row-major result is the transpose of what was computed).
// A block sums a 32 x 32 tile reading along N (contiguous in the workspace), turns it in shared
// memory and writes along M (contiguous in the output), so both sides are coalesced.
template <typename T>
__global__ void __launch_bounds__(256)
splitk_reduce_transposed_kernel(const ReduceParams p)
{
    grid_dependency_wait();
    __shared__ float tile[32][33];
    const uint32_t n0 = blockIdx.x * 32, m0 = blockIdx.y * 32, b = blockIdx.z;
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const T* const bias = static_cast<const T*>(p.bias);
    // the four rows of a thread: all loads of up to kInFlight slices first, then the ordered sums
    float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (uint32_t s0 = 0; s0 < p.splits; s0 += kInFlight) {
        float w[4][kInFlight];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t m = m0 + ty + 8 * i, n = n0 + tx;
            const unsigned long long idx = (static_cast<unsigned long long>(b) * p.M + m) * p.N + n;
#pragma unroll
            for (uint32_t j = 0; j < kInFlight; ++j)
                w[i][j] = (m < p.M && n < p.N && s0 + j < p.splits) ? p.ws[(s0 + j) * p.slice + idx] : 0.0f;
        }
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i)
#pragma unroll
            for (uint32_t j = 0; j < kInFlight; ++j)
                if (s0 + j < p.splits) sum[i] = (s0 + j == 0) ? w[i][j] : __fadd_rn(sum[i], w[i][j]);
    }
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t m = m0 + ty + 8 * i, n = n0 + tx;
        float acc = 0.0f;
        if (m < p.M && n < p.N) {
            acc = sum[i];
            if (p.bias_mode == 1) acc = __fadd_rn(acc, to_float<T>(bias[static_cast<long long>(n) * p.bias_stride]));
            else if (p.bias_mode == 2) acc = __fadd_rn(acc, to_float<T>(bias[static_cast<long long>(m) * p.bias_stride]));
            acc = apply_activation(p.act, acc);
        }
        tile[ty + 8 * i][tx] = acc;
    }
    __syncthreads();
    T* const out = static_cast<T*>(p.out) + static_cast<long long>(b) * p.o_b;
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t m = m0 + tx, n = n0 + ty + 8 * i;
        if (m < p.M && n < p.N)
            out[static_cast<long long>(m) * p.o_m + static_cast<long long>(n) * p.o_n] = from_float<T>(tile[tx][ty + 8 * i]);
    }
}

// ---------------------------------------------------------------------------------------------
// Ordering the ranks of one machine without a collective.  Every rank owns an array of 64-bit flags in
// peer-mapped memory, one slot per rank.  After its product a rank writes the step's number into ITS slot
// of every peer's array (peer_signal_kernel: system-scope fence, then the stores); before it reads what
// the others wrote it waits until every other slot of its own array has reached that number
// (peer_wait_kernel).  Each GPU runs only its own two kernels, so nothing here waits for another launch
// on the same GPU.  The wait is bounded: when the limit runs out it sets kStatusPeerTimeout in the status
// word and returns, and the stream goes on.
constexpr uint32_t kStatusPeerTimeout = 16u;
constexpr int kMaxFlagSlots = 8;

struct PeerSignalParams {
    unsigned long long* peer_flags[kMaxFlagSlots];     // the other ranks' flag arrays, mapped into this process
    int count;
    int slot;                                          // this rank's slot
    unsigned long long epoch;
};

__global__ void peer_signal_kernel(const PeerSignalParams p)
{
    if (threadIdx.x < static_cast<unsigned>(p.count)) {
        __threadfence_system();                        // everything this GPU stored before is visible before the flag
        *reinterpret_cast<volatile unsigned long long*>(p.peer_flags[threadIdx.x] + p.slot) = p.epoch;
    }
}

__global__ void peer_wait_kernel(const volatile unsigned long long* flags, int slots, int skip, unsigned long long epoch,
                                 unsigned long long limit_cycles)
{
    if (threadIdx.x != 0) return;
    const long long t0 = clock64();
    for (int s = 0; s < slots; ++s) {
        if (s == skip) continue;
        while (flags[s] < epoch) {
            if (static_cast<unsigned long long>(clock64() - t0) > limit_cycles) {
                atomicOr(&g_gemm_status, kStatusPeerTimeout);
                return;
            }
            __nanosleep(200);
        }
    }
    __threadfence_system();                            // what follows on this stream sees the peers' stores
}

}  // namespace srt
