// Re-layout of matrices between the storage orders of the reference's tensors
// (Order, Sources/SwiftRTCore/tensor/Tensor.swift:172-236):
//     C = alpha . op(A) + beta . op(B)
// with every operand in its own order and element type -- what cublasLtMatrixTransform does for the
// descriptors that Sources/SwiftRTCore/platform/cuda/cublaslt/MatrixTransform.swift:21-129 and
// MatrixLayout.swift:21-204 wrap (the reference creates them and never runs the transform).
//
// Element (r, c) of a stored matrix with leading dimension ld lives at
//     row              r ld + c
//     col              c ld + r
//     colTiled32       (c / 32) ld + r 32 + c % 32                       ld >= 32 rows
//     colTiledTC32x32  (c / 32) ld + (r / 32) 1024 + t(r % 32) 32 + c % 32,
//                      t(q) = ((q % 8) / 2 * 4 + q / 8) * 2 + q % 2      ld >= 32 roundUp(rows, 32)
// (Tensor.swift:188-192 and :219-231 state the two tiled formulas).  colTiledTC32x8 is not computed: the
// reference gives no element formula for it and names it a Turing-only operand layout (Tensor.swift:204-217).
//
// Two kernels, both bound by HBM (every element is read once per operand and written once); V consecutive
// elements along the contiguous axis travel as one access of up to 16 bytes (V = 16 / the widest element type,
// when base addresses, leading dimensions and batch strides allow it; else V = 1):
//   matrix_transform_stream_kernel   every operand is contiguous along the same LOGICAL axis (row <-> tiled
//       orders, col <-> col, or the other way round with a transpose): a thread reads a vector of each
//       operand, forms fma(beta, b, alpha a) in fp32 and writes the vector where C's order puts it (a pure
//       re-layout -- alpha = 1, beta = 0, one element type -- moves the bits untouched).
//   matrix_transform_tile_kernel     the contiguous axes differ (a transposition): a CTA takes 64 x 64
//       logical elements of C, reads the operands along their own contiguous axis into a padded fp32 tile in
//       shared memory, and writes C along its contiguous axis.
//   matrix_transform_transpose_kernel  the same case for a pure re-layout of 1- or 2-byte elements (see below).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace srt {

enum : int32_t { kOrderCol = 0, kOrderRow = 1, kOrderColTiled32 = 2, kOrderColTiledTC32x8 = 3, kOrderColTiledTC32x32 = 4 };
enum : int32_t { kTypeF32 = 0, kTypeF16 = 2, kTypeI8 = 3, kTypeBF16 = 14 };

struct StoredMatrix {
    void* ptr;
    long long ld, batch_stride;          // elements
    int32_t order, type;
    uint32_t transposed;                 // the logical operand is the transpose of what is stored
};

struct TransformParams {
    StoredMatrix a, b, c;
    float alpha, beta;
    uint32_t use_b;
    uint32_t rows, cols, batch;          // of C (and of op(A), op(B))
    uint32_t tiles_r, tiles_c;
};

__host__ __device__ __forceinline__ long long stored_offset(int32_t order, long long ld, uint32_t r, uint32_t c)
{
    switch (order) {
    case kOrderRow: return static_cast<long long>(r) * ld + c;
    case kOrderCol: return static_cast<long long>(c) * ld + r;
    case kOrderColTiled32: return static_cast<long long>(c >> 5) * ld + static_cast<long long>(r) * 32 + (c & 31);
    default: {                            // kOrderColTiledTC32x32
        const uint32_t q = r & 31;
        const uint32_t t = (((q & 7) >> 1) * 4 + (q >> 3)) * 2 + (q & 1);
        return static_cast<long long>(c >> 5) * ld + static_cast<long long>(r >> 5) * 1024 + t * 32 + (c & 31);
    }
    }
}

// which LOGICAL axis of the operand is contiguous in memory: true = along a row (consecutive c)
__host__ __device__ __forceinline__ bool runs_along_columns(const StoredMatrix& m)
{
    const bool stored = m.order != kOrderCol;          // row and both tiled orders keep 32 or more consecutive c together
    return stored != (m.transposed != 0);
}

template <typename T> __device__ __forceinline__ float element_to_float(T x);
template <> __device__ __forceinline__ float element_to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float element_to_float<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float element_to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float element_to_float<int8_t>(int8_t x) { return static_cast<float>(x); }

// one rounding to the element type; Int8 rounds to nearest even and saturates (NaN becomes 0)
template <typename T> __device__ __forceinline__ T element_from_float(float v);
template <> __device__ __forceinline__ float element_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half element_from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 element_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ int8_t element_from_float<int8_t>(float v)
{
    const float r = rintf(v);
    return static_cast<int8_t>(r != r ? 0.0f : fminf(fmaxf(r, -128.0f), 127.0f));
}

template <typename T, int V> struct alignas(sizeof(T) * V) ElementPack { T x[V]; };

template <typename T, int V>
__device__ __forceinline__ void load_pack(const void* base, long long off, float (&v)[V])
{
    const ElementPack<T, V> pk = *reinterpret_cast<const ElementPack<T, V>*>(static_cast<const T*>(base) + off);
#pragma unroll
    for (int i = 0; i < V; ++i) v[i] = element_to_float<T>(pk.x[i]);
}

template <typename T, int V>
__device__ __forceinline__ void store_pack(void* base, long long off, const float (&v)[V])
{
    ElementPack<T, V> pk;
#pragma unroll
    for (int i = 0; i < V; ++i) pk.x[i] = element_from_float<T>(v[i]);
    *reinterpret_cast<ElementPack<T, V>*>(static_cast<T*>(base) + off) = pk;
}

// V elements that are consecutive in memory from element offset `off`; `count` < V at a ragged edge
template <int V>
__device__ __forceinline__ void load_run(const StoredMatrix& m, long long off, uint32_t count, float (&v)[V])
{
    if (count >= V) {
        switch (m.type) {
        case kTypeF32: load_pack<float, V>(m.ptr, off, v); break;
        case kTypeF16: load_pack<__half, V>(m.ptr, off, v); break;
        case kTypeBF16: load_pack<__nv_bfloat16, V>(m.ptr, off, v); break;
        default: load_pack<int8_t, V>(m.ptr, off, v); break;
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
        float one[1] = {0.0f};
        if (i < count) {
            switch (m.type) {
            case kTypeF32: load_pack<float, 1>(m.ptr, off + i, one); break;
            case kTypeF16: load_pack<__half, 1>(m.ptr, off + i, one); break;
            case kTypeBF16: load_pack<__nv_bfloat16, 1>(m.ptr, off + i, one); break;
            default: load_pack<int8_t, 1>(m.ptr, off + i, one); break;
            }
        }
        v[i] = one[0];
    }
}

template <int V>
__device__ __forceinline__ void store_run(const StoredMatrix& m, long long off, uint32_t count, const float (&v)[V])
{
    if (count >= V) {
        switch (m.type) {
        case kTypeF32: store_pack<float, V>(m.ptr, off, v); break;
        case kTypeF16: store_pack<__half, V>(m.ptr, off, v); break;
        case kTypeBF16: store_pack<__nv_bfloat16, V>(m.ptr, off, v); break;
        default: store_pack<int8_t, V>(m.ptr, off, v); break;
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
        if (i < count) {
            const float one[1] = {v[i]};
            switch (m.type) {
            case kTypeF32: store_pack<float, 1>(m.ptr, off + i, one); break;
            case kTypeF16: store_pack<__half, 1>(m.ptr, off + i, one); break;
            case kTypeBF16: store_pack<__nv_bfloat16, 1>(m.ptr, off + i, one); break;
            default: store_pack<int8_t, 1>(m.ptr, off + i, one); break;
            }
        }
    }
}

// offset of LOGICAL element (r, c) of an operand
__device__ __forceinline__ long long logical_offset(const StoredMatrix& m, uint32_t batch, uint32_t r, uint32_t c)
{
    return batch * m.batch_stride + (m.transposed ? stored_offset(m.order, m.ld, c, r) : stored_offset(m.order, m.ld, r, c));
}

constexpr uint32_t kTransformTile = 64;
constexpr uint32_t kTransformThreads = 256;

// moves V elements of `size` bytes each without looking at them
template <typename U, int V>
__device__ __forceinline__ void copy_run(const StoredMatrix& src, long long src_off, const StoredMatrix& dst, long long dst_off, uint32_t count)
{
    if (count >= V) {
        *reinterpret_cast<ElementPack<U, V>*>(static_cast<U*>(dst.ptr) + dst_off) =
            *reinterpret_cast<const ElementPack<U, V>*>(static_cast<const U*>(src.ptr) + src_off);
        return;
    }
    for (uint32_t i = 0; i < count; ++i) static_cast<U*>(dst.ptr)[dst_off + i] = static_cast<const U*>(src.ptr)[src_off + i];
}

// every operand contiguous along the same logical axis: `along_columns` says which.
// RAW: alpha = 1, beta = 0 and equal element types -- a pure re-layout, the bits are moved as they are.
template <int V, bool RAW>
__global__ void __launch_bounds__(kTransformThreads)
matrix_transform_stream_kernel(const TransformParams p)
{
    const bool along_columns = runs_along_columns(p.c);
    const uint32_t fast = along_columns ? p.cols : p.rows, slow = along_columns ? p.rows : p.cols;
    const uint32_t nvec = (fast + V - 1) / V;
    const unsigned long long total = static_cast<unsigned long long>(p.batch) * slow * nvec;
    for (unsigned long long i = blockIdx.x * static_cast<unsigned long long>(kTransformThreads) + threadIdx.x; i < total;
         i += static_cast<unsigned long long>(gridDim.x) * kTransformThreads) {
        const uint32_t f = static_cast<uint32_t>(i % nvec) * V;
        const unsigned long long rest = i / nvec;
        const uint32_t s = static_cast<uint32_t>(rest % slow), bt = static_cast<uint32_t>(rest / slow);
        const uint32_t r = along_columns ? s : f, c = along_columns ? f : s;
        const uint32_t count = fast - f;                  // >= V except in the last vector of a run
        if constexpr (RAW) {
            const long long src = logical_offset(p.a, bt, r, c), dst = logical_offset(p.c, bt, r, c);
            switch (p.a.type) {
            case kTypeF32: copy_run<uint32_t, V>(p.a, src, p.c, dst, count); break;
            case kTypeI8: copy_run<uint8_t, V>(p.a, src, p.c, dst, count); break;
            default: copy_run<uint16_t, V>(p.a, src, p.c, dst, count); break;
            }
            continue;
        }
        float v[V];
        load_run<V>(p.a, logical_offset(p.a, bt, r, c), count, v);
#pragma unroll
        for (int k = 0; k < V; ++k) v[k] *= p.alpha;
        if (p.use_b) {
            float w[V];
            load_run<V>(p.b, logical_offset(p.b, bt, r, c), count, w);
#pragma unroll
            for (int k = 0; k < V; ++k) v[k] = __fmaf_rn(p.beta, w[k], v[k]);
        }
        store_run<V>(p.c, logical_offset(p.c, bt, r, c), count, v);
    }
}

template <int V>
__global__ void __launch_bounds__(kTransformThreads)
matrix_transform_tile_kernel(const TransformParams p)
{
    __shared__ float tile[kTransformTile][kTransformTile + 1];
    constexpr uint32_t kVecPerRun = kTransformTile / V, kVecPerTile = kTransformTile * kVecPerRun;
    const uint32_t per_batch = p.tiles_r * p.tiles_c;
    const unsigned long long total = static_cast<unsigned long long>(per_batch) * p.batch;
    const bool a_cols = runs_along_columns(p.a), b_cols = runs_along_columns(p.b), c_cols = runs_along_columns(p.c);
    for (unsigned long long t = blockIdx.x; t < total; t += gridDim.x) {
        const uint32_t bt = static_cast<uint32_t>(t / per_batch);
        const uint32_t in_batch = static_cast<uint32_t>(t - static_cast<unsigned long long>(bt) * per_batch);
        // consecutive CTAs walk along the axis on which C is contiguous
        const uint32_t tr = c_cols ? in_batch / p.tiles_c : in_batch % p.tiles_r;
        const uint32_t tc = c_cols ? in_batch % p.tiles_c : in_batch / p.tiles_r;
        const uint32_t r0 = tr * kTransformTile, c0 = tc * kTransformTile;
        // operand X, phase: 0 = A (tile = alpha a), 1 = B (tile = fma(beta, b, tile))
        auto read_operand = [&](const StoredMatrix& m, bool cols_fast, uint32_t phase) {
            for (uint32_t e = threadIdx.x; e < kVecPerTile; e += kTransformThreads) {
                const uint32_t lf = (e % kVecPerRun) * V, ls = e / kVecPerRun;
                const uint32_t lr = cols_fast ? ls : lf, lc = cols_fast ? lf : ls;
                const uint32_t r = r0 + lr, c = c0 + lc;
                if (r >= p.rows || c >= p.cols) continue;
                const uint32_t left = cols_fast ? p.cols - c : p.rows - r;
                float v[V];
                load_run<V>(m, logical_offset(m, bt, r, c), left, v);
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    float& cell = cols_fast ? tile[lr][lc + k] : tile[lr + k][lc];
                    cell = phase == 0 ? p.alpha * v[k] : __fmaf_rn(p.beta, v[k], cell);
                }
            }
            __syncthreads();
        };
        read_operand(p.a, a_cols, 0);
        if (p.use_b) read_operand(p.b, b_cols, 1);
        for (uint32_t e = threadIdx.x; e < kVecPerTile; e += kTransformThreads) {
            const uint32_t lf = (e % kVecPerRun) * V, ls = e / kVecPerRun;
            const uint32_t lr = c_cols ? ls : lf, lc = c_cols ? lf : ls;
            const uint32_t r = r0 + lr, c = c0 + lc;
            if (r >= p.rows || c >= p.cols) continue;
            float v[V];
#pragma unroll
            for (int k = 0; k < V; ++k) v[k] = c_cols ? tile[lr][lc + k] : tile[lr + k][lc];
            store_run<V>(p.c, logical_offset(p.c, bt, r, c), c_cols ? p.cols - c : p.rows - r, v);
        }
        __syncthreads();
    }
}

// Pure transposing re-layout of 1- or 2-byte elements (alpha = 1, beta = 0, one element type, contiguous axes of
// source and destination differ, extents multiples of the tile): the fp32 tile above would spend its time on one
// shared-memory access per element, so here elements stay packed in 32-bit words.  X is the axis along which the
// source is contiguous, Y the destination's.  A thread reads E = 4 / S source runs of 16 bytes (consecutive in Y),
// transposes their E x E blocks in registers (byte permutes) into words of E consecutive Y elements, and writes
// them to T[x][y / E]; then 16 bytes along Y are read back per thread and stored.  The word index is XOR-ed with
// the run index of x so that the eight runs a warp writes at once fall into different banks.
template <int S>
__global__ void __launch_bounds__(kTransformThreads)
matrix_transform_transpose_kernel(const TransformParams p)
{
    constexpr uint32_t E = 4 / S;                  // elements per word
    constexpr uint32_t XE = 16 / S;                // elements per 16-byte run
    constexpr uint32_t TX = 8 * XE, TY = 32 * E;   // tile: 128 x 128 (S = 1) or 64 x 64 (S = 2) elements
    __shared__ __align__(16) uint32_t T[TX][32];
    const bool x_is_col = runs_along_columns(p.a);
    const uint32_t tiles_x = (x_is_col ? p.cols : p.rows) / TX, tiles_y = (x_is_col ? p.rows : p.cols) / TY;
    const unsigned long long per_batch = static_cast<unsigned long long>(tiles_x) * tiles_y, total = per_batch * p.batch;
    const uint32_t tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
    const char* const src = static_cast<const char*>(p.a.ptr);
    char* const dst = static_cast<char*>(p.c.ptr);
    for (unsigned long long t = blockIdx.x; t < total; t += gridDim.x) {
        const uint32_t bt = static_cast<uint32_t>(t / per_batch);
        const uint32_t in_batch = static_cast<uint32_t>(t - bt * per_batch);
        const uint32_t x0 = (in_batch / tiles_y) * TX, y0 = (in_batch % tiles_y) * TY;     // consecutive CTAs walk along Y
        uint4 run[E];
#pragma unroll
        for (uint32_t i = 0; i < E; ++i) {
            const uint32_t x = x0 + tx * XE, y = y0 + ty * E + i;
            const long long off = x_is_col ? logical_offset(p.a, bt, y, x) : logical_offset(p.a, bt, x, y);
            run[i] = *reinterpret_cast<const uint4*>(src + off * S);
        }
#pragma unroll
        for (uint32_t b = 0; b < 4; ++b) {          // word b of every run: an E x E block
            uint32_t in[E], out[E];
#pragma unroll
            for (uint32_t i = 0; i < E; ++i) in[i] = b == 0 ? run[i].x : b == 1 ? run[i].y : b == 2 ? run[i].z : run[i].w;
            if constexpr (S == 1) {
                const uint32_t t0 = __byte_perm(in[0], in[1], 0x5140), t1 = __byte_perm(in[2], in[3], 0x5140);
                const uint32_t t2 = __byte_perm(in[0], in[1], 0x7362), t3 = __byte_perm(in[2], in[3], 0x7362);
                out[0] = __byte_perm(t0, t1, 0x5410); out[1] = __byte_perm(t0, t1, 0x7632);
                out[2] = __byte_perm(t2, t3, 0x5410); out[3] = __byte_perm(t2, t3, 0x7632);
            } else {
                out[0] = __byte_perm(in[0], in[1], 0x5410); out[1] = __byte_perm(in[0], in[1], 0x7632);
            }
#pragma unroll
            for (uint32_t k = 0; k < E; ++k) T[tx * XE + b * E + k][ty ^ (tx << 2)] = out[k];
        }
        __syncthreads();
#pragma unroll
        for (uint32_t e = threadIdx.x; e < TX * 8; e += kTransformThreads) {
            const uint32_t q = e & 7, xi = e >> 3;
            const uint4 v = *reinterpret_cast<const uint4*>(&T[xi][(4 * q) ^ (((xi / XE) & 7) << 2)]);
            const uint32_t x = x0 + xi, y = y0 + q * 4 * E;
            const long long off = x_is_col ? logical_offset(p.c, bt, y, x) : logical_offset(p.c, bt, x, y);
            *reinterpret_cast<uint4*>(dst + off * S) = v;
        }
        __syncthreads();
    }
}

}  // namespace srt
