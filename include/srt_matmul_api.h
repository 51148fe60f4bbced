/*
 * srt_matmul_api.h -- C ABI of the B200 (sm_100a) matmul / batched matmul / Dense path.
 *
 * A sibling of the reference's Modules/SwiftRTCuda/*_api.h headers: every operator is
 *     cudaError_t srtOp(const void* a, const srtTensorDescriptor* aDesc, ...,
 *                       void* out, const srtTensorDescriptor* oDesc, cudaStream_t stream);
 * (Modules/SwiftRTCuda/math_api.h:75-87).  Pointers are device addresses of the first
 * element of the view; descriptors and their arrays only need to live for the call;
 * work is enqueued on `stream` and the call returns without synchronising (a split-K
 * workspace that has to grow is replaced without waiting: the old buffer is freed in stream
 * order).  Every call works on the device that `stream` belongs to, whatever device is
 * current on the calling thread (it is made current for the duration of the call and the
 * caller's device restored): the reference's queues launch on their stream without selecting
 * a device (platform/cuda/functions/CudaMath.swift:117-125), and so may callers of this
 * library.  The legacy and per-thread default streams mean the current device.
 * cudaErrorNotSupported means "this dtype / layout is outside this library" (the Swift
 * caller then takes its own CPU route, cuda/device/CudaPlatform.swift:135-144); any
 * other non-zero code is an error.  The library has no CPU fallback and calls no
 * cuBLAS / cublasLt.
 */
#ifndef SRT_MATMUL_API_H
#define SRT_MATMUL_API_H

#include <stddef.h>
#include <stdint.h>
#include <stdbool.h>

#ifdef SRT_MATMUL_NO_CUDA_HEADERS
/* for FFI generators that cannot see the CUDA toolkit: same ABI */
typedef int cudaError_t;
typedef struct CUstream_st* cudaStream_t;
#else
#include <cuda_runtime_api.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------------------------------
 * Data types.  Values equal the reference's srtDataType, which aliases cudaDataType
 * (Modules/SwiftRTCuda/tensor_api.h:31-38): CUDA_R_32F = 0, CUDA_R_16F = 2, CUDA_R_16BF = 14.
 * Only these three are computed; every other value returns cudaErrorNotSupported.
 */
#ifndef SRT_TENSOR_API_TYPES
#define SRT_TENSOR_API_TYPES
typedef enum {
    srtUnknownType = -1,
    real32F  = 0,
    real64F  = 1,
    real16F  = 2,
    real8I   = 3,
    real16BF = 14
} srtDataType;

/* Storage order.  Values equal cublasLtOrder_t, which the reference's descriptor uses
 * (tensor_api.h:76; Order.cublas, cublaslt/MatrixLayout.swift:221-231).  The matmul entry points
 * compute row and col only and return cudaErrorNotSupported for the tiled orders; srtMatrixTransform
 * moves matrices into and out of them. */
typedef enum {
    srtOrderCol = 0,
    srtOrderRow = 1,
    srtOrderColTiled32 = 2,         /* CUBLASLT_ORDER_COL32 */
    srtOrderColTiledTC32x8 = 3,     /* CUBLASLT_ORDER_COL4_4R2_8C */
    srtOrderColTiledTC32x32 = 4     /* CUBLASLT_ORDER_COL32_2R_4R4 */
} srtOrder;

/* Replaces srtTensorDescriptor of Modules/SwiftRTCuda/tensor_api.h:70-87 field for field
 * (`order` keeps the width and values of cublasLtOrder_t, so the struct layout is equal).
 * `shape`, `strides` and `logicalStrides` have `rank` entries; strides are in elements.
 * The matmul entry points read type, rank, shape and strides only: majorness and leading
 * dimensions are derived from strides[], never from `order` (for col order the reference's
 * Tensor.leadingDimension, cuda/device/CudaPlatform.swift:298-311, would be 1). */
typedef struct {
    srtDataType type;
    uint32_t rank;
    srtOrder order;
    size_t count;
    size_t spanCount;
    const size_t* shape;
    const size_t* strides;
    const size_t* logicalStrides;
} srtTensorDescriptor;
#endif

/* Raw values equal ActivationType (Sources/SwiftRTCore/platform/common/
 * FunctionProperties.swift:44-51).  srtActivationGelu / GeluTanh are additions (the
 * reference enum has no GELU).  clippedRelu and elu take coefficients the Dense layer
 * never supplies and return cudaErrorNotSupported. */
typedef enum {
    srtActivationSigmoid     = 0,
    srtActivationRelu        = 1,
    srtActivationTanh        = 2,
    srtActivationClippedRelu = 3,
    srtActivationElu         = 4,
    srtActivationIdentity    = 5,
    srtActivationGelu        = 6,
    srtActivationGeluTanh    = 7
} srtActivationType;

/* ---------------------------------------------------------------------------------------
 * srtMatmul: out = op(a) . op(b), fp32 accumulation, one rounding to the element type.
 *
 * Replaces the bodies of CudaQueue.matmul for TensorR2 and TensorR3
 * (Sources/SwiftRTCore/platform/cuda/functions/CudaMatmul.swift:25-42 and :44-61, which
 * today always run the CPU loop CpuMath.swift:1141-1186) and with them the cublasLt
 * descriptor plumbing under platform/cuda/cublaslt/.
 *
 * rank 2: a [M x K] (or [K x M] when transA), b [K x N] (or [N x K] when transB), out [M x N].
 * rank 3: dimension 0 is the batch (shape[0] of `out`); an input whose shape[0] is 1 or
 *         whose strides[0] is 0 is broadcast over the batch.  An input may also be rank 2
 *         while `out` is rank 3 (the reference's left/right batch forms).
 * All three tensors have the same `type`.  Any non-negative element strides are accepted:
 * views that meet the TMA rules (16-byte aligned base, one unit stride in the last two
 * dims, the other strides multiples of 16 bytes) run on the tensor-core kernel, the rest
 * on a strided SIMT kernel.  `out` is write-only, may be a strided view, and must not
 * alias an input.  Inputs may alias each other.  An `out` without elements (M, N or the batch
 * is 0) succeeds and launches nothing; K = 0 writes activation(0 + bias) to every element.
 */
cudaError_t srtMatmul(
    const void* a, const srtTensorDescriptor* aDesc, bool transA,
    const void* b, const srtTensorDescriptor* bDesc, bool transB,
    void* out, const srtTensorDescriptor* oDesc,
    cudaStream_t stream);

/* srtMatmulBiasActivation: out = activation(op(a) . op(b) + bias), bias broadcast along
 * rows (bias[n] is added to column n), everything after the dot product in fp32 with one
 * final rounding.  `bias` may be NULL (then biasDesc is ignored); it is rank 1 with N
 * elements and the same `type` as the other tensors.
 *
 * Supplies what matmul(_:transposed:_:transposed:bias:) declares but does not compute
 * (Sources/SwiftRTCore/operators/Matmul.swift:57-72 drops the bias at :70) and what
 * Dense.callAsFunction declares (Sources/SwiftRTLayers/Dense.swift:21-40 returns its
 * input); the fused epilogue stands in for MatmulEpilogue {none, relu, bias, biasRelu}
 * (platform/cuda/cublaslt/MatmulOperation.swift:384-411) and for the separate cuDNN
 * activation call (platform/cuda/layers/CudaActivation.swift:61-83).
 */
cudaError_t srtMatmulBiasActivation(
    const void* a, const srtTensorDescriptor* aDesc, bool transA,
    const void* b, const srtTensorDescriptor* bDesc, bool transB,
    const void* bias, const srtTensorDescriptor* biasDesc,
    srtActivationType activation,
    void* out, const srtTensorDescriptor* oDesc,
    cudaStream_t stream);

/* srtBiasActivationBackward: the backward of the fused epilogue of srtMatmulBiasActivation.
 *     dz[.., m, n] = dy[.., m, n] * activation'(y[.., m, n])          (one rounding)
 *     dbias[n]     = sum over batch and rows of dz[.., m, n]          (fp32 sum, one rounding)
 * Supplies the derivatives that the reference leaves as fatalError() -- _vjpMatmul with bias
 * (Sources/SwiftRTCore/differentiable/MathDerivatives.swift:520-554) -- in the form the reference's
 * cuDNN activation backward uses (derivative from the forward OUTPUT y,
 * platform/cuda/layers/CudaActivation.swift:101-127).  With dz the remaining gradients are two
 * srtMatmul calls with transpose flags, exactly as matmulGradients composes them
 * (MathDerivatives.swift:460-482): dX = dz . W^T, dW = X^T . dz.
 * dy, y, dz: rank 2 [M x N] or rank 3 [batch x M x N], same type and shape, any strides.  y may
 * be NULL for srtActivationIdentity; dz or dbias may be NULL when not wanted; dz may alias dy.
 * identity, relu, sigmoid and tanh take the forward output in `y`.  GELU is not a function of its
 * own output: for srtActivationGelu and srtActivationGeluTanh `y` must hold the PRE-activation
 * values z = op(a).op(b) + bias (the result of srtMatmulBiasActivation with
 * srtActivationIdentity; srtActivationForward then gives the layer's output), and
 * dz = dy * gelu'(z).  The coefficient activations return cudaErrorNotSupported.  The column sums
 * use the library's per-(device, stream) workspace.
 */
cudaError_t srtBiasActivationBackward(
    const void* dy, const srtTensorDescriptor* dyDesc,
    const void* y, const srtTensorDescriptor* yDesc,
    srtActivationType activation,
    void* dz, const srtTensorDescriptor* dzDesc,
    void* dbias, const srtTensorDescriptor* dbiasDesc,
    cudaStream_t stream);

/* srtActivationForward: y = activation(z), elementwise, one rounding.  z, y: rank 2 or 3, same
 * type and shape, any strides; y may alias z.  For layers that keep their pre-activation values for
 * the backward pass (GELU): the product runs with srtActivationIdentity into z, this call produces
 * the layer's output, and srtBiasActivationBackward receives z.  Stands in for the reference's
 * separate activation call (platform/cuda/layers/CudaActivation.swift:61-83). */
cudaError_t srtActivationForward(
    const void* z, const srtTensorDescriptor* zDesc,
    srtActivationType activation,
    void* y, const srtTensorDescriptor* yDesc,
    cudaStream_t stream);

/* ---------------------------------------------------------------------------------------
 * srtMatrixTransform: C = alpha . op(A) + beta . op(B), every matrix in its own storage order and
 * element type -- the re-layout operation between row / col and the tiled tensor-core orders.
 *
 * Replaces cublasLtMatrixTransform for the descriptors the reference wraps but never runs:
 * MatrixTransform (Sources/SwiftRTCore/platform/cuda/cublaslt/MatrixTransform.swift:21-129: scale type,
 * pointer mode, transA, transB) and MatrixLayout (cublaslt/MatrixLayout.swift:21-204: type, order, rows,
 * cols, leadingDimension, batchCount, batchStride -- srtMatrixLayout has the same fields).
 *
 * rows / cols / ld describe the matrix as STORED; op(X) is the stored matrix or its transpose, and op(A),
 * op(B) and C must agree in rows, cols and batchCount.  Element (r, c) of a stored matrix lives at
 *   srtOrderRow              r ld + c
 *   srtOrderCol              c ld + r
 *   srtOrderColTiled32       (c / 32) ld + r 32 + c % 32                                   ld >= 32 rows
 *   srtOrderColTiledTC32x32  (c / 32) ld + (r / 32) 1024 + t(r % 32) 32 + c % 32,
 *                            t(q) = ((q % 8) / 2 * 4 + q / 8) * 2 + q % 2                  ld >= 32 roundUp(rows, 32)
 * (the formulas of Order, tensor/Tensor.swift:188-192 and :219-231).  srtOrderColTiledTC32x8 returns
 * cudaErrorNotSupported: the reference states no element formula for it and names it an operand layout of
 * SM 7.2 / 7.5 only (Tensor.swift:204-217).  srtMatrixLayoutLeadingDimension gives the smallest valid ld.
 *
 * Types: real32F, real16F, real16BF, real8I in any combination; alpha and beta are host floats (the
 * default pointer mode and the fp32 scale type of the wrapper), the sum is formed in fp32 and rounded once
 * (Int8: to nearest even, saturated to [-128, 127]).  B may be NULL when *beta is 0.  C must not overlap
 * A or B.  One launch on `stream`, no workspace; a C without elements succeeds without a launch.
 */
typedef struct {
    srtDataType type;
    srtOrder order;
    uint64_t rows;
    uint64_t cols;
    int64_t leadingDimension;       /* elements */
    int32_t batchCount;             /* >= 1 */
    int64_t batchStride;            /* elements between consecutive matrices */
} srtMatrixLayout;

cudaError_t srtMatrixTransform(
    const float* alpha, const void* A, const srtMatrixLayout* aLayout, bool transA,
    const float* beta, const void* B, const srtMatrixLayout* bLayout, bool transB,
    void* C, const srtMatrixLayout* cLayout, cudaStream_t stream);

/* Smallest leading dimension of a rows x cols matrix in `order` (the rule of Tensor.leadingDimension,
 * cuda/device/CudaPlatform.swift:298-311, written in terms of the stored rows as cublasLt defines it),
 * and the number of elements a buffer for it must hold.  0 for an order that is not computed. */
uint64_t srtMatrixLayoutLeadingDimension(srtOrder order, uint64_t rows, uint64_t cols);
uint64_t srtMatrixLayoutElementCount(srtOrder order, uint64_t rows, uint64_t cols, uint64_t leadingDimension);

/* ---------------------------------------------------------------------------------------
 * Plan query and tuning knobs.  Stand in for MatmulAlgorithm.query / .search
 * (platform/cuda/cublaslt/MatmulAlgorithmSearch.swift:51-100, 128-216), MatmulTile /
 * MatmulStages (MatmulAlgorithm.swift:593-800) and MatmulPreferences.maxWorkspaceSize
 * (MatmulPreferences.swift:85-254).
 */
typedef enum {
    srtMatmulKernelNone    = 0,
    srtMatmulKernelSimt    = 1,   /* strided SIMT kernel, fp32 multiply and add in the reference's order */
    srtMatmulKernelTcgen05 = 2,   /* TMA + tcgen05 tensor-core kernel, one CTA per tile */
    srtMatmulKernelTcgen05Pair = 3, /* TMA + tcgen05 cta_group::2 kernel, CTA pair per tile */
    srtMatmulKernelTcgen05Split = 4, /* Float32 as 3 x TF32 on the tensor cores (hi/lo split in shared memory) */
    srtMatmulKernelTf32x3Pair = 5   /* Float32, CTA pair per tile: one TF32 pass + BFloat16 correction terms; op(a) is
                                       streamed once, op(b) is pre-split by a pack pass into the workspace */
} srtMatmulKernel;

typedef struct {
    int32_t kernel;        /* srtMatmulKernel that a call with these arguments launches */
    int32_t tileM, tileN, tileK;
    int32_t stages;        /* shared-memory pipeline depth */
    int32_t ctas;          /* grid size (persistent CTAs) */
    int32_t tiles;         /* output tiles over all batch items */
    int32_t swapped;       /* 1 when computed as out^T = op(b)^T . op(a)^T (col-order out; a few rows against a wide operand) */
    int32_t aMajor, bMajor;/* 0 = K-major, 1 = MN-major operand as the kernel sees it */
    int32_t fp32Split;     /* 1 when fp32 runs as 3 x TF32 on the tensor cores */
    int32_t splitK;        /* > 1: the reduction is cut into this many parts, summed by a second kernel */
    size_t  workspaceBytes;/* device scratch of the call: fp32 partial sums (split-K) or the pre-split operand (kernel 5), else 0 */
    size_t  dynamicSmemBytes;
} srtMatmulPlan;

/* Fills `plan` with what srtMatmulBiasActivation would launch for these descriptors and
 * pointers (alignment matters, so the pointers are part of the key).  Launches nothing. */
cudaError_t srtMatmulQueryPlan(
    const void* a, const srtTensorDescriptor* aDesc, bool transA,
    const void* b, const srtTensorDescriptor* bDesc, bool transB,
    const void* out, const srtTensorDescriptor* oDesc,
    srtMatmulPlan* plan);

/* Process-wide overrides, 0 = automatic.  forceKernel: an srtMatmulKernel value (a forced
 * tensor-core kernel still falls back to SIMT for views that TMA cannot address; Float32
 * always takes the 3 x TF32 kernel when a tensor-core kernel is forced);
 * tileN: 64, 128 or 256; stages: 2..8; maxCtas: cap on the persistent grid. */
cudaError_t srtMatmulSetTuning(int32_t forceKernel, int32_t tileN, int32_t stages, int32_t maxCtas);

/* srtMatmulTune: measures, for this exact call, every kernel and tile width the element type allows
 * (the cost model's own choice first), keeps the fastest in the process's plan table and leaves
 * `out` holding the product.  Later calls with the same signature -- sizes, element type, which
 * strides are 1, bias or not -- use the tuned choice whenever no process-wide tuning is set.
 * Stands in for MatmulAlgorithm.search and its timing loop
 * (Sources/SwiftRTCore/platform/cuda/cublaslt/MatmulAlgorithmSearch.swift:128-216).
 * Synchronises `stream` (it times with events on it).  `best` and `bestMicroseconds` may be NULL. */
cudaError_t srtMatmulTune(
    const void* a, const srtTensorDescriptor* aDesc, bool transA,
    const void* b, const srtTensorDescriptor* bDesc, bool transB,
    const void* bias, const srtTensorDescriptor* biasDesc,
    srtActivationType activation,
    void* out, const srtTensorDescriptor* oDesc,
    cudaStream_t stream, srtMatmulPlan* best, float* bestMicroseconds);

/* The plan table as a text file (one line per tuned signature), so that tuning survives the
 * process: Save writes all entries, Load merges a file into the table (`entries`, if not NULL,
 * receives the number read), Clear empties the table.  A file named by the environment variable
 * SRT_MATMUL_PLAN_CACHE is loaded before the first plan is made.  Entries are specific to the GPU
 * model they were measured on. */
cudaError_t srtMatmulPlanCacheSave(const char* path);
cudaError_t srtMatmulPlanCacheLoad(const char* path, int32_t* entries);
cudaError_t srtMatmulPlanCacheClear(void);

/* Split-K override, process-wide: 0 = automatic (Float32 with K > 2048; few tiles with a long
 * reduction), 1 = never, n > 1 = cut the reduction into (up to) n parts whenever the tensor-core
 * kernel for one CTA per tile runs.  The fp32 partial sums live in a workspace that the library
 * keeps per (device, stream) and grows on demand with cudaMalloc. */
cudaError_t srtMatmulSetSplitK(int32_t splits);

/* Frees the per-(device, stream) workspaces (split-K partial sums, column-sum partials, the
 * recurrent cells' intermediates) after synchronising their devices; later calls allocate again.
 * A workspace that was handed out while its stream was being captured is part of a CUDA graph that
 * may still be replayed: it is kept unless `includeCaptured` is true (pass true only when those
 * graphs will not run again).  Stands in for MatmulPreferences.maxWorkspaceSize = 0
 * (platform/cuda/cublaslt/MatmulPreferences.swift:85-254) as the way to give scratch back. */
cudaError_t srtMatmulReleaseWorkspaces(bool includeCaptured);

/* srtMatmulNoAlloc: srtMatmul for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference.  It exists for hosts that cannot call
 * cudaMalloc at the point where the product is needed: code that runs inside a region where the
 * allocator is locked or forbidden (a real-time loop, a callback from another runtime that owns
 * all device memory, a process whose memory pool was handed out in full at start-up).  srtMatmul
 * itself allocates only for split-K products, whose fp32 partial sums need scratch; here that
 * scratch is a 16 MiB array compiled into the library instead of a cudaMalloc'ed workspace, and
 * the call performs no cudaMalloc, cudaFree or other allocating call.
 *
 * Same arguments, result and kernels as srtMatmul.  Differences:
 *  - a split-K product whose partial sums (splitK x batch x M x N x 4 bytes, see
 *    srtMatmulQueryPlan) exceed 16 MiB is refused with cudaErrorInvalidValue and an explanatory
 *    srtMatmulGetLastErrorString(); nothing is launched.  Products that are not split need no
 *    scratch and are never refused for their size;
 *  - the first call on a device looks up the scratch array's device address
 *    (cudaGetSymbolAddress, with that device current); make that first call outside any stream
 *    capture;
 *  - "allocates nothing" holds once the kernels a call launches are resident: under CUDA's lazy
 *    module loading the first launch of each kernel variant (per element type, tile width and
 *    reduce pass) loads its code, which takes device memory inside the driver.  Make the first
 *    call for each shape class where that is allowed (at start-up), as with the capture note;
 *  - repeated calls with the same arguments reuse the prepared launch (no planning, no tensor-map
 *    encoding), like srtMatmul;
 *  - all calls on a device share the one array: two split-K calls that overlap on the GPU (on
 *    different streams) corrupt each other's partial sums.  Calls on one stream are safe.  The
 *    array keeps what the last call wrote; no call depends on its previous contents.
 */
cudaError_t srtMatmulNoAlloc(
    const void* a, const srtTensorDescriptor* aDesc, bool transA,
    const void* b, const srtTensorDescriptor* bDesc, bool transB,
    void* out, const srtTensorDescriptor* oDesc,
    cudaStream_t stream);

/* srtLstmCell: one time step of an LSTM cell, a caller of the fused product.
 *
 * Computes what LSTMCell.callAsFunction composes from separate operators
 * (Sources/SwiftRTLayers/Recurrent.swift:255-266):
 *     fused   = matmul(concatenate(input, hidden, axis: 1), fusedWeight, bias: fusedBias)
 *     i, u, f, o = sigmoid, tanh, sigmoid, sigmoid of the column blocks 0..3 of fused (Part: input,
 *               update, forget, output; Recurrent.swift:173)
 *     newCell   = cell * f + i * u
 *     newHidden = tanh(newCell) * o
 * input [batch x inputSize], hidden / cell / newCell / newHidden [batch x hiddenSize], fusedWeight
 * [(inputSize + hiddenSize) x 4 hiddenSize], fusedBias [4 hiddenSize] (may be NULL); all of one element
 * type, rank 2 (bias rank 1), any strides.  newCell may alias cell and newHidden may alias hidden.
 * hidden may be NULL when `input` is the concatenation already, [batch x (inputSize + hiddenSize)] (a caller
 * that keeps the hidden state inside its gate-input buffer saves the concatenation; newHidden may then be a
 * view into the next step's gate input).
 * Three launches on `stream`: a concatenation, the product (srtMatmulBiasActivation) and the gate
 * pass; the two intermediates live in the library's per-(device, stream) workspace. */
cudaError_t srtLstmCell(
    const void* input, const srtTensorDescriptor* inputDesc,
    const void* hidden, const srtTensorDescriptor* hiddenDesc,
    const void* cell, const srtTensorDescriptor* cellDesc,
    const void* fusedWeight, const srtTensorDescriptor* weightDesc,
    const void* fusedBias, const srtTensorDescriptor* biasDesc,
    void* newCell, const srtTensorDescriptor* newCellDesc,
    void* newHidden, const srtTensorDescriptor* newHiddenDesc,
    cudaStream_t stream);

/* srtLstmCellFused: srtLstmCell with the gate pass inside the product's epilogue -- the fused product
 * [batch x 4 hiddenSize] never reaches memory and the step is one launch (two with the concatenation).
 * For that the four gate columns of a hidden unit must sit side by side: `interleavedWeight` and
 * `interleavedBias` are fusedWeight / fusedBias with column 4 j + g = original column g hiddenSize + j,
 * produced once per cell by srtLstmInterleaveGates.  Same tensors and aliasing rules as srtLstmCell otherwise
 * (hidden may be NULL for a pre-concatenated gate input).  The gates see the fp32 pre-activations (srtLstmCell
 * rounds the fused product to the element type first, as matmul(bias:) returns it), so results agree with
 * srtLstmCell within the element type's rounding, not bit for bit.
 * Float16 / BFloat16, hiddenSize a multiple of 8, row-contiguous 16-byte aligned state tensors, and a product
 * that runs on a 16-bit tensor-core kernel in one pass; anything else returns cudaErrorNotSupported and the
 * caller uses srtLstmCell (Recurrent.swift:255-266 is the definition of both). */
cudaError_t srtLstmCellFused(
    const void* input, const srtTensorDescriptor* inputDesc,
    const void* hidden, const srtTensorDescriptor* hiddenDesc,
    const void* cell, const srtTensorDescriptor* cellDesc,
    const void* interleavedWeight, const srtTensorDescriptor* weightDesc,
    const void* interleavedBias, const srtTensorDescriptor* biasDesc,
    void* newCell, const srtTensorDescriptor* newCellDesc,
    void* newHidden, const srtTensorDescriptor* newHiddenDesc,
    cudaStream_t stream);

/* out[.., 4 j + g] = in[.., g hiddenSize + j]: the column order srtLstmCellFused expects, for a rank-2 weight
 * [rows x 4 hiddenSize] or a rank-1 bias [4 hiddenSize]; `out` has the shape of `in` and contiguous columns. */
cudaError_t srtLstmInterleaveGates(
    const void* in, const srtTensorDescriptor* inDesc,
    void* out, const srtTensorDescriptor* outDesc,
    cudaStream_t stream);

/* srtRnnCell: one time step of BasicRNNCell (Sources/SwiftRTLayers/Recurrent.swift:110-161):
 *     newHidden = tanh(matmul(concatenate(input, hidden, axis: 1), weight) + bias)
 * weight [(inputSize + hiddenSize) x hiddenSize]; bias [hiddenSize] or, as the reference stores it,
 * [1 x hiddenSize]; NULL for none.  Two launches: the concatenation and the product with its fused
 * bias + tanh epilogue. */
cudaError_t srtRnnCell(
    const void* input, const srtTensorDescriptor* inputDesc,
    const void* hidden, const srtTensorDescriptor* hiddenDesc,
    const void* weight, const srtTensorDescriptor* weightDesc,
    const void* bias, const srtTensorDescriptor* biasDesc,
    void* newHidden, const srtTensorDescriptor* newHiddenDesc,
    cudaStream_t stream);

/* srtGruCell: one time step of a GRU cell (Sources/SwiftRTLayers/Recurrent.swift:328-337), with the
 * reference's six products fused into two:
 *     [reset | update] = sigmoid(concatenate(input, hidden) . gateWeight + gateBias)
 *     output           = tanh(concatenate(input, reset * hidden) . outputWeight + outputBias)
 *     newHidden        = (1 - update) * hidden + (1 - update) * output      (as the reference writes it)
 * gateWeight [(inputSize + hiddenSize) x 2 hiddenSize] holds [[resetWeight1 | updateWeight1],
 * [resetWeight2 | updateWeight2]], gateBias [2 hiddenSize] = [resetBias | updateBias]; outputWeight
 * [(inputSize + hiddenSize) x hiddenSize] = [[outputWeight1], [outputWeight2]], outputBias [hiddenSize].
 * Biases may be NULL.  Five launches on `stream`: the concatenation, two products with fused bias +
 * sigmoid / tanh epilogues and two elementwise passes; intermediates live in the library's workspace.
 * newHidden may alias hidden. */
cudaError_t srtGruCell(
    const void* input, const srtTensorDescriptor* inputDesc,
    const void* hidden, const srtTensorDescriptor* hiddenDesc,
    const void* gateWeight, const srtTensorDescriptor* gateWeightDesc,
    const void* gateBias, const srtTensorDescriptor* gateBiasDesc,
    const void* outputWeight, const srtTensorDescriptor* outputWeightDesc,
    const void* outputBias, const srtTensorDescriptor* outputBiasDesc,
    void* newHidden, const srtTensorDescriptor* newHiddenDesc,
    cudaStream_t stream);

/* ---- several GPUs of one machine, one process per GPU -----------------------------------------
 *
 * The reference has no multi-GPU path: its only data-parallel construct partitions axis 0 of a
 * CPU tensor over threads that write disjoint views of one shared output
 * (Sources/SwiftRTCore/operators/pmap.swift:26-72).  The entry points below are that idea for
 * GPUs: every rank computes one block of C (its columns, rows or batch items) and writes it into
 * ITS view of a full-size C -- in its own buffer and in every peer's buffer. */

/* A buffer that other processes can map (cudaIpcMemHandle_t, 64 bytes). */
typedef struct { unsigned char bytes[64]; } srtPeerMemHandle;

/* cudaMalloc + cudaIpcGetMemHandle on the current device.  Send `handle` to the other ranks. */
cudaError_t srtPeerMemAlloc(size_t bytes, void** ptr, srtPeerMemHandle* handle);
/* Maps another rank's buffer into this process (peer access is enabled on demand).  A process
 * cannot open its own handle. */
cudaError_t srtPeerMemOpen(const srtPeerMemHandle* handle, void** ptr);
/* Ordering the ranks without a collective.  Each rank keeps an array of (at most 8) 64-bit flags in a buffer
 * from srtPeerMemAlloc, zeroed once, slot r belonging to rank r.
 * srtPeerSignal enqueues on `stream`: after everything enqueued before it, store `epoch` into slot `slot` (this
 * rank's) of every array in peerFlags (the other ranks' arrays, mapped with srtPeerMemOpen).
 * srtPeerWait enqueues on `stream`: wait until every slot of this rank's own array except `skipSlot` holds a
 * value >= epoch; what follows on the stream then sees what those ranks stored before their signal.  The wait
 * is bounded (timeoutNs, 0 = 2 s): when it runs out, bit 4 of the status word (srtMatmulCheckStatus) is set and
 * the stream continues.  Use increasing epochs (1, 2, ...).  Every GPU runs only its own two small kernels. */
cudaError_t srtPeerSignal(void* const* peerFlags, int32_t peerCount, int32_t slot, uint64_t epoch, cudaStream_t stream);
cudaError_t srtPeerWait(const void* localFlags, int32_t slots, int32_t skipSlot, uint64_t epoch, uint64_t timeoutNs, cudaStream_t stream);
/* Unmaps a pointer obtained from srtPeerMemOpen. */
cudaError_t srtPeerMemClose(void* ptr);
/* Frees a buffer obtained from srtPeerMemAlloc (after every peer has closed its mapping). */
cudaError_t srtPeerMemFree(void* ptr);

/* srtMatmulAllGather: srtMatmulBiasActivation whose result block is also delivered to peers.
 *
 * `out`/`oDesc` is this rank's block of C as a view into its own full-size buffer.  peerOut[i]
 * (0 <= i < peerCount <= 7) is the first element of the same view -- same shape, strides and
 * offset -- in the buffer of another GPU, mapped with srtPeerMemOpen (an address in a buffer of
 * the same GPU is accepted too).  For products that run on the CTA-pair tensor-core kernel with
 * a 16-byte aligned, row-contiguous output view, the kernel's epilogue stores each finished tile
 * to the local and to all peer buffers, so the transfer overlaps the product; every other product
 * runs as srtMatmulBiasActivation followed by one strided copy per peer on `stream`.
 *
 * Completion: the peers' copies are complete when `stream` has drained on THIS rank.  No rank
 * waits for another on the device; before reading blocks written by others, synchronise the
 * ranks on the host (each rank: cudaStreamSynchronize, then a barrier). */
cudaError_t srtMatmulAllGather(
    const void* a, const srtTensorDescriptor* aDesc, bool transA,
    const void* b, const srtTensorDescriptor* bDesc, bool transB,
    const void* bias, const srtTensorDescriptor* biasDesc,
    srtActivationType activation,
    void* out, const srtTensorDescriptor* oDesc,
    int32_t peerCount, void* const* peerOut,
    cudaStream_t stream);

/* srtMatmulAllGatherMulticast: the same delivery through an NVLink multicast (NVLS) mapping.
 *
 * `multicastOut` is the first element of the output view in a multicast mapping of the full-size
 * buffers of all ranks (every rank's buffer bound to one multicast object, e.g. the multicast_ptr of
 * torch.distributed._symmetric_memory); `out` is the same view in this rank's own buffer.  The
 * epilogue stores each tile once with multimem.st and the NVSwitch replicates it into every rank's
 * buffer, this rank's included, so each byte leaves the GPU once instead of once per peer.
 * Only for products that run on the CTA-pair kernel with a 16-byte aligned, row-contiguous output
 * whose rows are a multiple of 16 bytes long; anything else returns cudaErrorNotSupported and the
 * caller uses srtMatmulAllGather.  Completion as for srtMatmulAllGather. */
cudaError_t srtMatmulAllGatherMulticast(
    const void* a, const srtTensorDescriptor* aDesc, bool transA,
    const void* b, const srtTensorDescriptor* bDesc, bool transB,
    const void* bias, const srtTensorDescriptor* biasDesc,
    srtActivationType activation,
    void* out, const srtTensorDescriptor* oDesc,
    void* multicastOut,
    cudaStream_t stream);

/* Which dimension of the result the GPUs divide among themselves. */
typedef enum {
    srtShardBatch = 0,   /* batch items (dimension 0 of rank-3 tensors) */
    srtShardM     = 1,   /* rows of op(a) and of the result */
    srtShardN     = 2    /* columns of op(b) and of the result (bias entries with them) */
} srtShardAxis;

/* Balanced contiguous [start, stop) of `total` items for `rank` of `world`; block boundaries are
 * multiples of `align` (0 or 1: none), the last block takes the remainder.  The arithmetic of the
 * reference's pmap partitions (Sources/SwiftRTCore/platform/common/pmap.swift:26-72). */
cudaError_t srtShardRange(size_t total, int32_t world, int32_t rank, size_t align, size_t* start, size_t* stop);

/* srtMatmulSharded: one rank's share of a product divided over `world` GPUs, one process (or one
 * stream) per GPU.  The descriptors describe the FULL logical tensors; a, b, bias and out point at
 * this GPU's copies of them (only the owned slices of the sharded operand are read).  The call
 * narrows the operands and the result to block `rank` along `axis` (srtShardRange; column blocks of
 * the N axis are aligned to 16 bytes) and runs srtMatmulBiasActivation on the views, writing this
 * rank's block into its place in `out`.  peerOut[i] (peerCount <= 7, may be 0) is the first element
 * of the FULL result buffer of another GPU mapped into this process, multicastOut (may be NULL) the
 * first element of the full result in an NVLink multicast mapping: with either, the block is also
 * delivered there (srtMatmulAllGather / srtMatmulAllGatherMulticast; a product the multicast form
 * does not take goes peer by peer when peers are given).  A rank without a block (more ranks than
 * items) launches nothing.  No collective and no wait for another GPU; completion as for
 * srtMatmulAllGather.  The GPU form of the reference's pmap (pmap.swift:26-72). */
cudaError_t srtMatmulSharded(
    srtShardAxis axis, int32_t world, int32_t rank,
    const void* a, const srtTensorDescriptor* aDesc, bool transA,
    const void* b, const srtTensorDescriptor* bDesc, bool transB,
    const void* bias, const srtTensorDescriptor* biasDesc,
    srtActivationType activation,
    void* out, const srtTensorDescriptor* oDesc,
    int32_t peerCount, void* const* peerOut, void* multicastOut,
    cudaStream_t stream);

/* srtMatmulShardedDevices: the same from ONE process that drives several GPUs (one SwiftRT queue
 * per device): streams[i] belongs to device i of the call, a[i], b[i], bias[i] (bias may be NULL)
 * and out[i] are that device's copies of the full tensors.  Block i is enqueued on streams[i]; with
 * `gather` every block is also stored into the other devices' result buffers (peer access is
 * enabled on demand), so that after all streams have drained every out[i] holds the whole result.
 * `multicastOut` (may be NULL; used with `gather`): the multicast mapping of the out[] buffers when they come from
 * srtMulticastAlloc -- eligible products then store every tile once and the NVSwitch replicates it.
 * At most 8 devices.  Returns after enqueuing; synchronise every stream before reading. */
cudaError_t srtMatmulShardedDevices(
    srtShardAxis axis, int32_t nDevices, const cudaStream_t* streams,
    const void* const* a, const srtTensorDescriptor* aDesc, bool transA,
    const void* const* b, const srtTensorDescriptor* bDesc, bool transB,
    const void* const* bias, const srtTensorDescriptor* biasDesc,
    srtActivationType activation,
    void* const* out, const srtTensorDescriptor* oDesc,
    bool gather, void* multicastOut);

/* NVLink multicast buffers for ONE process that drives several GPUs: one physical allocation of `bytes`
 * (rounded up to the multicast granularity) on each device, all bound to one multicast object.
 * localPtrs[i] is device i's buffer (addressable from every listed device), *multicastPtr the multicast
 * mapping: a multimem store to it lands in every device's buffer at the same offset -- what
 * srtMatmulAllGatherMulticast / srtMatmulShardedDevices(…, multicastOut) write through.  Built on the driver's
 * virtual-memory and multicast entry points (cuMulticastCreate / cuMulticastBindMem / cuMemMap), obtained at
 * run time; cudaErrorNotSupported when a device or the driver has no multicast.  The reference has no counterpart
 * (its device memory is one cub-cached cudaMalloc per tensor, Modules/SwiftRTCuda/memory.cu:31-41).
 * Processes that each own one GPU exchange such allocations through file descriptors instead; that plumbing
 * is not part of this library (torch.distributed._symmetric_memory provides it for the Python mirror). */
typedef void* srtMulticastBuffer;
cudaError_t srtMulticastAlloc(int32_t nDevices, const int32_t* devices, size_t bytes, void** localPtrs, void** multicastPtr,
                              srtMulticastBuffer* handle);
/* Synchronises the devices, unmaps and frees everything srtMulticastAlloc made. */
cudaError_t srtMulticastFree(srtMulticastBuffer handle);

/* Wall-clock limit of every pipeline wait inside the tensor-core kernels of the current device, in
 * nanoseconds (0 restores the default of 2 s).  A wait that runs out ends its kernel in an orderly
 * way and sets the status word below; the result of that launch is invalid.  For tests of that
 * path: production code has no reason to change the limit. */
cudaError_t srtMatmulSetWaitLimit(uint64_t nanoseconds);

/* Device-side status of the last tensor-core launches on the device of `stream`: 0 = all
 * pipeline waits completed; non-zero = a bounded wait gave up (the code says which) and
 * the result of that launch is invalid.  Synchronises `stream` and resets the status. */
cudaError_t srtMatmulCheckStatus(cudaStream_t stream, uint32_t* status);

/* Number of kernels this library has launched since it was loaded (all streams). */
uint64_t srtMatmulLaunchCount(void);

/* Text of the last argument error on the calling thread ("" when none). */
const char* srtMatmulGetLastErrorString(void);

#ifdef __cplusplus
}
#endif
#endif /* SRT_MATMUL_API_H */
