/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the SwiftRT matmul hot path.
 *
 * This file restates, in plain C, the arithmetic of the reference's CPU matmul so that
 * the CUDA kernels can be checked against it.  Nothing in the shipped library links,
 * loads or calls this code; only the tests, the smoke check and the benchmark's
 * cpu_baseline / reference arm do.
 *
 * The reference implementation is Swift and needs the Swift-for-TensorFlow toolchain,
 * which is not available, so it cannot be compiled; the restatement is pinned by the
 * known-answer literals of the reference's own tests
 * (Tests/SwiftRTCoreTests/test_AlgebraicField.swift:551-645), which are the only
 * vectors the reference holds for this path.  Dense (bias + activation), bf16/fp16
 * numerics, strided views and col-order are NOT pinned by any reference test
 * ("parity unpinned" for those): the reference never executes them.
 *
 * What is followed, by reference file:line
 *   - loop nest and accumulation order, rank 2:
 *       Sources/SwiftRTCore/platform/cpu/functions/CpuMath.swift:1141-1161
 *     for r { for c { out[r,c] = sum over k = 0..K-1, in order, of lhs[r,k]*rhs[k,c] } }
 *     accumulated in the element's Value type, one rounding for the product and one
 *     for the add (no fused multiply-add), one conversion to the Stored type at the end.
 *   - rank 3 (batched): same with an outer batch loop, CpuMath.swift:1164-1186.
 *   - transposes are stride swaps of the last two dims (views, no copy):
 *       Sources/SwiftRTCore/tensor/TensorInit.swift:844-886
 *   - BFloat16: Stored = upper 16 bits, Value = Float; decode bits<<16, encode
 *     round-to-nearest-even with NaN -> 0x7fff:
 *       Sources/SwiftRTCore/platform/common/BFloat16.swift:53-85
 *   - Float16: round-to-nearest-even encode / exact decode:
 *       Sources/SwiftRTCore/platform/common/Float16.swift:54-134
 *     Two Value types exist in the reference: Float (emulated, fp32 accumulate,
 *     Float16.swift:173-211) and native Float16 (Linux, every product and partial sum
 *     rounded to fp16, Float16.swift:12-16).  `f16_native` selects between them.
 *   - ReLU in the style of cpu_max (x >= 0 ? x : 0), CpuMath.swift:1189-1198.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -fopenmp).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* dtype ids equal the reference's srtDataType values (Modules/SwiftRTCuda/tensor_api.h:34-38,
 * which alias cudaDataType: CUDA_R_32F = 0, CUDA_R_16F = 2, CUDA_R_16BF = 14). */
enum { ORACLE_F32 = 0, ORACLE_F16 = 2, ORACLE_BF16 = 14 };

/* activation ids equal ActivationType's raw values
 * (Sources/SwiftRTCore/platform/common/FunctionProperties.swift:44-51); gelu is an
 * addition that the reference does not have. */
enum {
    ORACLE_ACT_SIGMOID = 0,
    ORACLE_ACT_RELU = 1,
    ORACLE_ACT_TANH = 2,
    ORACLE_ACT_CLIPPED_RELU = 3,
    ORACLE_ACT_ELU = 4,
    ORACLE_ACT_IDENTITY = 5,
    ORACLE_ACT_GELU = 6,
    ORACLE_ACT_GELU_TANH = 7
};

/* ---------------------------------------------------------------- element codecs */

static inline float bits2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f2bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* BFloat16.swift:79-81 */
float oracle_bf16_to_f32(uint16_t v) { return bits2f((uint32_t)v << 16); }

/* BFloat16.swift:53-77: truncate, keep the discarded half in `rem`, round to nearest even */
uint16_t oracle_f32_to_bf16(float f)
{
    uint32_t x = f2bits(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
    uint32_t rem = x << 16;
    uint16_t raw = (uint16_t)(x >> 16);
    if (rem > 0x80000000u || (rem == 0x80000000u && (raw & 1u))) raw += 1;
    return raw;
}

/* Float16.swift:104-134 */
float oracle_f16_to_f32(uint16_t h)
{
    uint32_t sign = (h >> 15) & 1u;
    uint32_t exponent = (h >> 10) & 0x1fu;
    uint32_t mantissa = (uint32_t)(h & 0x3ffu) << 13;
    if (exponent == 0x1f) {
        if (mantissa != 0) { sign = 0; mantissa = 0x7fffffu; }
        exponent = 0xff;
    } else if (exponent == 0) {
        if (mantissa != 0) {
            uint32_t msb;
            exponent = 0x71;
            do { msb = mantissa & 0x400000u; mantissa <<= 1; exponent -= 1; } while (msb == 0);
            mantissa &= 0x7fffffu;
        }
    } else {
        exponent += 0x70;
    }
    return bits2f((sign << 31) | (exponent << 23) | mantissa);
}

/* Float16.swift:54-102 */
uint16_t oracle_f32_to_f16(float f)
{
    uint32_t x = f2bits(f);
    uint32_t u = x & 0x7fffffffu;
    if (u > 0x7f800000u) return 0x7fff;
    uint32_t sign = (x >> 16) & 0x8000u;
    if (u > 0x477fefffu) return (uint16_t)(sign | 0x7c00u);
    if (u < 0x33000001u) return (uint16_t)sign;
    uint32_t exponent = (u >> 23) & 0xffu;
    uint32_t mantissa = u & 0x7fffffu;
    uint32_t shift;
    if (exponent > 0x70) {
        shift = 13;
        exponent -= 0x70;
    } else {
        shift = 0x7e - exponent;
        exponent = 0;
        mantissa |= 0x800000u;
    }
    uint32_t lsb = 1u << shift, lsb_s1 = lsb >> 1, lsb_m1 = lsb - 1;
    uint32_t remainder = mantissa & lsb_m1;
    mantissa >>= shift;
    if (remainder > lsb_s1 || (remainder == lsb_s1 && (mantissa & 1u))) {
        mantissa += 1;
        if ((mantissa & 0x3ffu) == 0) { exponent += 1; mantissa = 0; }
    }
    return (uint16_t)(sign | (exponent << 10) | mantissa);
}

/* round a double that is the exact sum or product of two fp16 values to fp16 (one rounding).
 * float is wide enough for a product (22 significant bits) but not always for a sum, so the
 * native-fp16 variant computes in double and rounds once through this helper. */
static inline uint16_t f64_to_f16_once(double d)
{
    /* a double -> float conversion could round twice; go through float only when exact */
    float f = (float)d;
    if ((double)f == d) return oracle_f32_to_f16(f);
    /* inexact in float: nudge to round-to-odd so that the second rounding is innocuous */
    uint32_t b = f2bits(f);
    double back = (double)f;
    if ((b & 1u) == 0) {
        if ((back < d) == (f >= 0.0f)) b += 1; else b -= 1;
    }
    return oracle_f32_to_f16(bits2f(b));
}

void oracle_convert_f32_to(int dtype, const float* src, void* dst, size_t n)
{
    if (dtype == ORACLE_F32) { memcpy(dst, src, n * 4); return; }
    uint16_t* d = (uint16_t*)dst;
    if (dtype == ORACLE_BF16) for (size_t i = 0; i < n; ++i) d[i] = oracle_f32_to_bf16(src[i]);
    else                      for (size_t i = 0; i < n; ++i) d[i] = oracle_f32_to_f16(src[i]);
}

void oracle_convert_to_f32(int dtype, const void* src, float* dst, size_t n)
{
    if (dtype == ORACLE_F32) { memcpy(dst, src, n * 4); return; }
    const uint16_t* s = (const uint16_t*)src;
    if (dtype == ORACLE_BF16) for (size_t i = 0; i < n; ++i) dst[i] = oracle_bf16_to_f32(s[i]);
    else                      for (size_t i = 0; i < n; ++i) dst[i] = oracle_f16_to_f32(s[i]);
}

static inline float load_value(int dtype, const void* p, size_t idx)
{
    switch (dtype) {
    case ORACLE_F32: return ((const float*)p)[idx];
    case ORACLE_BF16: return oracle_bf16_to_f32(((const uint16_t*)p)[idx]);
    default: return oracle_f16_to_f32(((const uint16_t*)p)[idx]);
    }
}

static inline void store_value(int dtype, void* p, size_t idx, float v)
{
    switch (dtype) {
    case ORACLE_F32: ((float*)p)[idx] = v; break;
    case ORACLE_BF16: ((uint16_t*)p)[idx] = oracle_f32_to_bf16(v); break;
    default: ((uint16_t*)p)[idx] = oracle_f32_to_f16(v); break;
    }
}

static inline float activate(int act, float x)
{
    switch (act) {
    case ORACLE_ACT_RELU: return x >= 0.0f ? x : 0.0f;          /* NaN -> 0, as cpu_max */
    case ORACLE_ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
    case ORACLE_ACT_TANH: return tanhf(x);
    case ORACLE_ACT_GELU: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
    case ORACLE_ACT_GELU_TANH: {
        float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
        return 0.5f * x * (1.0f + tanhf(u));
    }
    default: return x;
    }
}

/* ---------------------------------------------------------------- the matmul itself */

typedef struct {
    int dtype;
    size_t batch, M, N, K;
    /* element strides of the logical (already transposed) operands */
    ptrdiff_t a_b, a_m, a_k;
    ptrdiff_t b_b, b_k, b_n;
    ptrdiff_t o_b, o_m, o_n;
    const void* a; const void* b; void* out;
    const void* bias; ptrdiff_t bias_s; int act; int has_epilogue;
    int f16_native;
} mm_args;

/* one output row, loop order c then k: exactly the reference's nest */
static void row_faithful(const mm_args* g, size_t n, size_t r)
{
    for (size_t c = 0; c < g->N; ++c) {
        float acc = 0.0f;
        if (g->dtype == ORACLE_F16 && g->f16_native) {
            uint16_t h = 0;
            for (size_t k = 0; k < g->K; ++k) {
                double x = oracle_f16_to_f32(((const uint16_t*)g->a)[n * g->a_b + r * g->a_m + k * g->a_k]);
                double y = oracle_f16_to_f32(((const uint16_t*)g->b)[n * g->b_b + k * g->b_k + c * g->b_n]);
                uint16_t p = f64_to_f16_once(x * y);
                h = f64_to_f16_once((double)oracle_f16_to_f32(h) + (double)oracle_f16_to_f32(p));
            }
            acc = oracle_f16_to_f32(h);
        } else {
            for (size_t k = 0; k < g->K; ++k) {
                float x = load_value(g->dtype, g->a, n * g->a_b + r * g->a_m + k * g->a_k);
                float y = load_value(g->dtype, g->b, n * g->b_b + k * g->b_k + c * g->b_n);
                float p = x * y;        /* -ffp-contract=off: product rounded, then added */
                acc += p;
            }
        }
        if (g->has_epilogue) {
            if (g->bias) acc = acc + load_value(g->dtype, g->bias, c * g->bias_s);
            acc = activate(g->act, acc);
        }
        store_value(g->dtype, g->out, n * g->o_b + r * g->o_m + c * g->o_n, acc);
    }
}

/* A block of up to ORACLE_ROW_BLOCK output rows, loop order k, row, c with one row of
 * accumulators per output row.  Every element still receives its products in k = 0..K-1 order
 * with the same two roundings, so the result is bit-identical to row_faithful; only the memory
 * access pattern differs (each row of B is read once per block of rows instead of once per row). */
#define ORACLE_ROW_BLOCK 8
#define ORACLE_COL_BLOCK 1024
static void rows_fast(const mm_args* g, size_t n, size_t r0, size_t nrows, float* acc)
{
    /* column blocks keep the accumulators (8 x 1024 floats) in the L1 cache */
    for (size_t c0 = 0; c0 < g->N; c0 += ORACLE_COL_BLOCK) {
        const size_t nc = g->N - c0 < ORACLE_COL_BLOCK ? g->N - c0 : ORACLE_COL_BLOCK;
        for (size_t i = 0; i < nrows * ORACLE_COL_BLOCK; ++i) acc[i] = 0.0f;
        for (size_t k = 0; k < g->K; ++k) {
            float x[ORACLE_ROW_BLOCK];
            for (size_t i = 0; i < nrows; ++i)
                x[i] = load_value(g->dtype, g->a, n * g->a_b + (r0 + i) * g->a_m + k * g->a_k);
            if (g->dtype == ORACLE_F32 && g->b_n == 1) {
                const float* brow = (const float*)g->b + n * g->b_b + k * g->b_k + c0;
                for (size_t i = 0; i < nrows; ++i) {
                    float* ar = acc + i * ORACLE_COL_BLOCK;
                    const float xi = x[i];
                    for (size_t c = 0; c < nc; ++c) { float p = xi * brow[c]; ar[c] += p; }
                }
            } else if (g->dtype == ORACLE_BF16 && g->b_n == 1) {
                const uint16_t* brow = (const uint16_t*)g->b + n * g->b_b + k * g->b_k + c0;
                for (size_t i = 0; i < nrows; ++i) {
                    float* ar = acc + i * ORACLE_COL_BLOCK;
                    const float xi = x[i];
                    for (size_t c = 0; c < nc; ++c) { float p = xi * bits2f((uint32_t)brow[c] << 16); ar[c] += p; }
                }
            } else {
                for (size_t c = 0; c < nc; ++c) {
                    float y = load_value(g->dtype, g->b, n * g->b_b + k * g->b_k + (c0 + c) * g->b_n);
                    for (size_t i = 0; i < nrows; ++i) { float p = x[i] * y; acc[i * ORACLE_COL_BLOCK + c] += p; }
                }
            }
        }
        for (size_t i = 0; i < nrows; ++i)
            for (size_t c = 0; c < nc; ++c) {
                float v = acc[i * ORACLE_COL_BLOCK + c];
                if (g->has_epilogue) {
                    if (g->bias) v = v + load_value(g->dtype, g->bias, (c0 + c) * g->bias_s);
                    v = activate(g->act, v);
                }
                store_value(g->dtype, g->out, n * g->o_b + (r0 + i) * g->o_m + (c0 + c) * g->o_n, v);
            }
    }
}

/*
 * rank is 2 or 3.  shape/stride arrays have `rank` entries and describe the tensors as
 * stored (before the transpose flags are applied), in elements, exactly like the
 * reference's srtTensorDescriptor.  A batch stride of 0 broadcasts that operand.
 * bias may be NULL; act is an ActivationType raw value; has_epilogue = 0 gives the plain
 * matmul (the reference's matmul(bias:) ignores the bias, Matmul.swift:57-72).
 * mode 0 = faithful loop order on one thread; mode 1 = k-outer loop order over blocks of rows,
 * `threads` OpenMP threads over the blocks (bit-identical results).
 * row_begin/row_end restrict the computed output rows (for bounded samples); pass 0, M.
 * Returns 0, or a negative code on a shape error.
 */
int oracle_matmul(int dtype, int rank,
                  const void* a, const size_t* a_shape, const size_t* a_strides, int transA,
                  const void* b, const size_t* b_shape, const size_t* b_strides, int transB,
                  void* out, const size_t* o_shape, const size_t* o_strides,
                  const void* bias, size_t bias_stride, int act, int has_epilogue,
                  int f16_native, int mode, int threads,
                  size_t row_begin, size_t row_end)
{
    if (rank != 2 && rank != 3) return -1;
    if (dtype != ORACLE_F32 && dtype != ORACLE_F16 && dtype != ORACLE_BF16) return -2;
    int q = rank - 2;
    mm_args g;
    memset(&g, 0, sizeof g);
    g.dtype = dtype;
    g.batch = rank == 3 ? o_shape[0] : 1;
    g.M = o_shape[q]; g.N = o_shape[q + 1];
    size_t a_rows = a_shape[q], a_cols = a_shape[q + 1];
    size_t b_rows = b_shape[q], b_cols = b_shape[q + 1];
    size_t aM = transA ? a_cols : a_rows, aK = transA ? a_rows : a_cols;
    size_t bK = transB ? b_cols : b_rows, bN = transB ? b_rows : b_cols;
    if (aM != g.M || bN != g.N || aK != bK) return -3;
    if (rank == 3 && (a_shape[0] != g.batch || b_shape[0] != g.batch)) return -4;
    g.K = aK;
    g.a_m = (ptrdiff_t)(transA ? a_strides[q + 1] : a_strides[q]);
    g.a_k = (ptrdiff_t)(transA ? a_strides[q] : a_strides[q + 1]);
    g.b_k = (ptrdiff_t)(transB ? b_strides[q + 1] : b_strides[q]);
    g.b_n = (ptrdiff_t)(transB ? b_strides[q] : b_strides[q + 1]);
    g.o_m = (ptrdiff_t)o_strides[q]; g.o_n = (ptrdiff_t)o_strides[q + 1];
    if (rank == 3) { g.a_b = (ptrdiff_t)a_strides[0]; g.b_b = (ptrdiff_t)b_strides[0]; g.o_b = (ptrdiff_t)o_strides[0]; }
    g.a = a; g.b = b; g.out = out;
    g.bias = bias; g.bias_s = (ptrdiff_t)bias_stride; g.act = act; g.has_epilogue = has_epilogue;
    g.f16_native = f16_native;
    if (row_end > g.M) row_end = g.M;

    if (mode == 0 || (dtype == ORACLE_F16 && f16_native)) {
        for (size_t n = 0; n < g.batch; ++n)
            for (size_t r = row_begin; r < row_end; ++r) row_faithful(&g, n, r);
        return 0;
    }
    if (threads < 1) threads = 1;
    const size_t rows = row_end - row_begin;
    const size_t blocks_per_item = (rows + ORACLE_ROW_BLOCK - 1) / ORACLE_ROW_BLOCK;
    const long total = (long)(g.batch * blocks_per_item);
#pragma omp parallel num_threads(threads)
    {
        float* acc = (float*)malloc(sizeof(float) * ORACLE_ROW_BLOCK * ORACLE_COL_BLOCK);
#pragma omp for schedule(dynamic, 1)
        for (long i = 0; i < total; ++i) {
            size_t n = (size_t)i / blocks_per_item;
            size_t r0 = row_begin + ((size_t)i % blocks_per_item) * ORACLE_ROW_BLOCK;
            size_t nr = row_end - r0 < ORACLE_ROW_BLOCK ? row_end - r0 : ORACLE_ROW_BLOCK;
            rows_fast(&g, n, r0, nr, acc);
        }
        free(acc);
    }
    return 0;
}

/* The un-fused composition that chaining the reference's own ops would give for a
 * 16-bit element type: matmul (rounded to the stored type), then add bias (rounded),
 * then activation (rounded).  Used once by the tests to show the fused single-rounding
 * epilogue stays within tolerance of it. */
int oracle_bias_activation_unfused(int dtype, void* y, size_t rows, size_t cols,
                                   const void* bias, int act)
{
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < cols; ++c) {
            float v = load_value(dtype, y, r * cols + c);
            if (bias) {
                v = v + load_value(dtype, bias, c);
                store_value(dtype, y, r * cols + c, v);
                v = load_value(dtype, y, r * cols + c);
            }
            store_value(dtype, y, r * cols + c, activate(act, v));
        }
    return 0;
}

/* ---------------------------------------------------------------- Dense backward helpers
 * The reference leaves the bias / activation derivatives of matmul unimplemented
 * (Sources/SwiftRTCore/differentiable/MathDerivatives.swift:520-554 are fatalError()), so
 * there is nothing executable to follow; this restates what composing the reference's own
 * pieces would compute:
 *   dz = dy * act'(y)   elementwise in the Value type, stored in the element type, with the
 *        derivative written in terms of the forward OUTPUT y, as cuDNN's activation backward
 *        does (platform/cuda/layers/CudaActivation.swift:101-127): relu: y > 0 ? dy : 0,
 *        sigmoid: dy*y*(1-y), tanh: dy*(1-y*y), identity: dy; GELU is not a function of its own
 *        output, so for gelu / geluTanh `y` holds the PRE-activation values z and
 *        dz = dy * (Phi(z) + z phi(z)), resp. the derivative of 0.5 z (1 + tanh(u(z)));
 *   dbias[n] = sum over rows m = 0..M-1, in order, of dz[m][n]   -- cpu_sum along axis 0
 *        (platform/cpu/functions/CpuReduce.swift:69-96).  The reference's loop keeps the running
 *        sum in the OUTPUT tensor, i.e. rounds it to the element type after every row
 *        (`stepwise` = 1); with `stepwise` = 0 the sum is kept in fp32 and rounded once, which is
 *        the graded variant (same choice as fp32 accumulation for the 16-bit matmul).
 * dy, y, dz are dense row-major [M x N]; dbias has N elements.  Returns 0.
 */
int oracle_bias_activation_backward(int dtype, const void* dy, const void* y, size_t M, size_t N, int act,
                                    void* dz, void* dbias, int stepwise)
{
    if (dtype != ORACLE_F32 && dtype != ORACLE_F16 && dtype != ORACLE_BF16) return -2;
    float* acc = (float*)malloc(sizeof(float) * (N ? N : 1));
    for (size_t n = 0; n < N; ++n) acc[n] = 0.0f;
    for (size_t m = 0; m < M; ++m)
        for (size_t n = 0; n < N; ++n) {
            const float g = load_value(dtype, dy, m * N + n);
            const float o = load_value(dtype, y, m * N + n);
            float d;
            switch (act) {
            case ORACLE_ACT_RELU: d = o > 0.0f ? g : 0.0f; break;
            case ORACLE_ACT_SIGMOID: { float t = o * (1.0f - o); d = g * t; break; }
            case ORACLE_ACT_TANH: { float t = o * o; t = 1.0f - t; d = g * t; break; }
            case ORACLE_ACT_GELU: {
                const float cdf = 0.5f * (1.0f + erff(o * 0.70710678118654752440f));
                const float pdf = 0.39894228040143267794f * expf(-0.5f * o * o);
                d = g * (cdf + o * pdf);
                break;
            }
            case ORACLE_ACT_GELU_TANH: {
                const float u = 0.7978845608028654f * (o + 0.044715f * o * o * o);
                const float t = tanhf(u);
                const float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * o * o);
                d = g * (0.5f * (1.0f + t) + 0.5f * o * (1.0f - t * t) * du);
                break;
            }
            default: d = g; break;
            }
            store_value(dtype, dz, m * N + n, d);
            const float stored = load_value(dtype, dz, m * N + n);
            if (stepwise) {
                store_value(dtype, dbias, n, m == 0 ? stored : load_value(dtype, dbias, n) + stored);
            } else {
                acc[n] = acc[n] + stored;
            }
        }
    if (!stepwise)
        for (size_t n = 0; n < N; ++n) store_value(dtype, dbias, n, acc[n]);
    free(acc);
    return 0;
}

/* y = act(z) elementwise over `count` dense elements, one rounding to the element type. */
int oracle_activation_forward(int dtype, const void* z, void* y, size_t count, int act)
{
    if (dtype != ORACLE_F32 && dtype != ORACLE_F16 && dtype != ORACLE_BF16) return -2;
    for (size_t i = 0; i < count; ++i) store_value(dtype, y, i, activate(act, load_value(dtype, z, i)));
    return 0;
}

int oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
