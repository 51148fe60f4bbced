// C++ host-side mirror of the reference's operator interface for the matmul path, above the C ABI
// of include/srt_matmul_api.h.  Same names, argument meaning and error behaviour as the Swift
// originals (the reference's host code is Swift, which is compiled code; no Swift toolchain is
// available, so this mirror stands where CudaQueue.matmul / matmul() / Dense would call the ABI):
//   Tensor<E>, .t view, Order            Sources/SwiftRTCore/tensor/Tensor.swift:26-54, 177-236,
//                                        tensor/TensorInit.swift:844-886
//   array(range, shape)                  Sources/SwiftRTCore/numpy/arrayInit.swift (range-filled tensors of the tests)
//   matmul(lhs, transposed:, rhs, transposed:)            operators/Matmul.swift:29-45
//   matmul(..., bias:)                                    operators/Matmul.swift:57-72
//   matmulGradients                                       differentiable/MathDerivatives.swift:460-482
//   Dense                                                 Sources/SwiftRTLayers/Dense.swift:21-71
//   LSTMCell, its State and the time-step loop            Sources/SwiftRTLayers/Recurrent.swift:165-266, 346-370
// Header-only; link against libsrt_b200.so and the CUDA runtime.  Every product runs on the GPU
// through srtMatmul*; there is no host fallback.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cassert>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "srt_matmul_api.h"

namespace srt_host {

enum class Order { col = 0, row = 1, colTiled32 = 2, colTiledTC32x8 = 3, colTiledTC32x32 = 4 };   // Tensor.swift:177-231
enum class ActivationType { sigmoid = 0, relu, tanh, clippedRelu, elu, identity, gelu, geluTanh };

template <typename E> struct ElementTraits;
template <> struct ElementTraits<float> {
    static constexpr srtDataType type = real32F;
    static float from(float v) { return v; }
    static float to(float v) { return v; }
};
template <> struct ElementTraits<__half> {
    static constexpr srtDataType type = real16F;
    static __half from(float v) { return __float2half_rn(v); }
    static float to(__half v) { return __half2float(v); }
};
template <> struct ElementTraits<__nv_bfloat16> {
    static constexpr srtDataType type = real16BF;
    static __nv_bfloat16 from(float v) { return __float2bfloat16_rn(v); }
    static float to(__nv_bfloat16 v) { return __bfloat162float(v); }
};

struct Error : std::runtime_error {
    cudaError_t code;
    Error(cudaError_t c, const std::string& what) : std::runtime_error(what), code(c) {}
};
inline void check(cudaError_t e, const char* what)
{
    if (e == cudaSuccess) return;
    std::string text = std::string(what) + ": " + cudaGetErrorString(e);
    const char* detail = srtMatmulGetLastErrorString();
    if (detail && *detail) text += std::string(" (") + detail + ")";
    throw Error(e, text);
}

// A tensor of rank 1..3 in device memory: shape, element strides, order and a shared buffer.
// Views (.t, slices) share the buffer, as the reference's tensors share their storage.
template <typename E>
class Tensor {
public:
    std::vector<size_t> shape, strides;
    Order order = Order::row;

    Tensor() = default;
    Tensor(std::vector<size_t> shape_, Order order_ = Order::row) : shape(std::move(shape_)), order(order_)
    {
        strides = stridesFor(shape, order);
        void* p = nullptr;
        check(cudaMalloc(&p, count() * sizeof(E) + 16), "cudaMalloc");
        buffer_ = std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
    }
    // strides(for:) of tensor/Shape.swift:274-300: col order swaps the strides of the last two dims
    static std::vector<size_t> stridesFor(const std::vector<size_t>& shape, Order order)
    {
        const size_t r = shape.size();
        std::vector<size_t> s(r, 1);
        for (size_t i = r; i-- > 1;) s[i - 1] = s[i] * shape[i];
        if (order == Order::col && r >= 2) {
            s[r - 2] = 1;
            s[r - 1] = shape[r - 2];
        }
        return s;
    }
    size_t rank() const { return shape.size(); }
    size_t count() const { size_t n = 1; for (size_t d : shape) n *= d; return n; }
    E* data() const { return reinterpret_cast<E*>(static_cast<char*>(buffer_.get()) + offset_ * sizeof(E)); }

    // transposed view of the last two dims: swaps shape and strides, no copy (TensorInit.swift:844-886)
    Tensor t() const
    {
        assert(rank() >= 2);
        Tensor v = *this;
        const size_t r = rank();
        std::swap(v.shape[r - 1], v.shape[r - 2]);
        std::swap(v.strides[r - 1], v.strides[r - 2]);
        return v;
    }

    // logical (row-major order of indices) element values <-> host floats
    void assign(const std::vector<float>& values)
    {
        assert(values.size() == count());
        std::vector<E> phys(span());
        forEachIndex([&](size_t logical, size_t offset) { phys[offset] = ElementTraits<E>::from(values[logical]); });
        check(cudaMemcpy(data(), phys.data(), phys.size() * sizeof(E), cudaMemcpyHostToDevice), "cudaMemcpy H2D");
    }
    std::vector<float> values(cudaStream_t stream = nullptr) const
    {
        check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
        std::vector<E> phys(span());
        check(cudaMemcpy(phys.data(), data(), phys.size() * sizeof(E), cudaMemcpyDeviceToHost), "cudaMemcpy D2H");
        std::vector<float> out(count());
        forEachIndex([&](size_t logical, size_t offset) { out[logical] = ElementTraits<E>::to(phys[offset]); });
        return out;
    }

    // srtTensorDescriptor on the caller's stack, as withTensor builds it (CudaExtensions.swift:24-84)
    srtTensorDescriptor descriptor() const
    {
        srtTensorDescriptor d;
        d.type = ElementTraits<E>::type;
        d.rank = static_cast<uint32_t>(rank());
        d.order = order == Order::row ? srtOrderRow : srtOrderCol;
        d.count = count();
        d.spanCount = span();
        d.shape = shape.data();
        d.strides = strides.data();
        d.logicalStrides = strides.data();
        return d;
    }

private:
    std::shared_ptr<void> buffer_;
    size_t offset_ = 0;

    size_t span() const
    {
        size_t s = 1;
        for (size_t i = 0; i < rank(); ++i) s += (shape[i] - 1) * strides[i];
        return s;
    }
    template <typename F>
    void forEachIndex(F f) const
    {
        const size_t n = count(), r = rank();
        std::vector<size_t> idx(r, 0);
        for (size_t logical = 0; logical < n; ++logical) {
            size_t offset = 0;
            for (size_t i = 0; i < r; ++i) offset += idx[i] * strides[i];
            f(logical, offset);
            for (size_t i = r; i-- > 0;) {
                if (++idx[i] < shape[i]) break;
                idx[i] = 0;
            }
        }
    }
};

// array(0..<n, shape): range-filled tensor, the fixture of the reference's matmul tests
template <typename E = float>
Tensor<E> array(size_t begin, size_t end, std::vector<size_t> shape, Order order = Order::row)
{
    Tensor<E> t(std::move(shape), order);
    std::vector<float> v;
    for (size_t i = begin; i < end; ++i) v.push_back(static_cast<float>(i));
    t.assign(v);
    return t;
}
template <typename E = float>
Tensor<E> array(const std::vector<float>& values, std::vector<size_t> shape, Order order = Order::row)
{
    Tensor<E> t(std::move(shape), order);
    t.assign(values);
    return t;
}
template <typename E>
Tensor<E> ones(std::vector<size_t> shape)
{
    Tensor<E> t(std::move(shape));
    t.assign(std::vector<float>(t.count(), 1.0f));
    return t;
}

namespace detail {
template <typename E>
std::vector<size_t> resultShape(const Tensor<E>& lhs, bool tl, const Tensor<E>& rhs, bool tr)
{
    const size_t lr = lhs.rank(), rr = rhs.rank();
    const size_t lM = tl ? lhs.shape[lr - 1] : lhs.shape[lr - 2], lK = tl ? lhs.shape[lr - 2] : lhs.shape[lr - 1];
    const size_t rK = tr ? rhs.shape[rr - 1] : rhs.shape[rr - 2], rN = tr ? rhs.shape[rr - 2] : rhs.shape[rr - 1];
    // the reference asserts here (Matmul.swift:35)
    if (lK != rK) throw Error(cudaErrorInvalidValue, "matmul inner dimensions must be equal");
    std::vector<size_t> shape;
    if (lr == 3 || rr == 3) shape.push_back(lr == 3 ? lhs.shape[0] : rhs.shape[0]);
    shape.push_back(lM);
    shape.push_back(rN);
    return shape;
}
}  // namespace detail

// queue-level form: result passed in (CpuMath.swift:355-369), may be a view
template <typename E>
void matmul(const Tensor<E>& lhs, bool transposeLhs, const Tensor<E>& rhs, bool transposeRhs, Tensor<E>& out,
            cudaStream_t stream = nullptr)
{
    const srtTensorDescriptor a = lhs.descriptor(), b = rhs.descriptor(), o = out.descriptor();
    check(srtMatmul(lhs.data(), &a, transposeLhs, rhs.data(), &b, transposeRhs, out.data(), &o, stream), "srtMatmul");
}

// matmul(_:transposed:_:transposed:): result allocated dense in lhs's order (Matmul.swift:36-38)
template <typename E>
Tensor<E> matmul(const Tensor<E>& lhs, bool transposeLhs, const Tensor<E>& rhs, bool transposeRhs,
                 cudaStream_t stream = nullptr)
{
    Tensor<E> out(detail::resultShape(lhs, transposeLhs, rhs, transposeRhs), lhs.order);
    matmul(lhs, transposeLhs, rhs, transposeRhs, out, stream);
    return out;
}
template <typename E>
Tensor<E> matmul(const Tensor<E>& lhs, const Tensor<E>& rhs, cudaStream_t stream = nullptr)
{
    return matmul(lhs, false, rhs, false, stream);
}

// matmul(..., bias:) and the Dense epilogue: activation(op(lhs) . op(rhs) + bias)
template <typename E>
Tensor<E> matmul(const Tensor<E>& lhs, bool transposeLhs, const Tensor<E>& rhs, bool transposeRhs, const Tensor<E>& bias,
                 ActivationType activation = ActivationType::identity, cudaStream_t stream = nullptr)
{
    Tensor<E> out(detail::resultShape(lhs, transposeLhs, rhs, transposeRhs), lhs.order);
    const srtTensorDescriptor a = lhs.descriptor(), b = rhs.descriptor(), o = out.descriptor(), bd = bias.descriptor();
    check(srtMatmulBiasActivation(lhs.data(), &a, transposeLhs, rhs.data(), &b, transposeRhs, bias.data(), &bd,
                                  static_cast<srtActivationType>(activation), out.data(), &o, stream),
          "srtMatmulBiasActivation");
    return out;
}

// matmulGradients (MathDerivatives.swift:460-482): two more matmul calls with transpose flags
template <typename E>
std::pair<Tensor<E>, Tensor<E>> matmulGradients(const Tensor<E>& out, const Tensor<E>& lhs, bool transposeLhs,
                                                const Tensor<E>& rhs, bool transposeRhs, cudaStream_t stream = nullptr)
{
    if (!transposeLhs && !transposeRhs) return {matmul(out, false, rhs, true, stream), matmul(lhs, true, out, false, stream)};
    if (!transposeLhs && transposeRhs) return {matmul(out, false, rhs, false, stream), matmul(lhs, true, out, false, stream)};
    if (transposeLhs && !transposeRhs) return {matmul(out, false, rhs, true, stream), matmul(lhs, false, out, false, stream)};
    return {matmul(out, true, rhs, true, stream), matmul(lhs, true, out, true, stream)};
}

// Dense<Shape2, E>: y = activation(x . weight + bias) (Dense.swift:21-55)
template <typename E>
struct Dense {
    Tensor<E> weight, bias;
    ActivationType activation;
    Dense(Tensor<E> weight_, Tensor<E> bias_, ActivationType activation_)
        : weight(std::move(weight_)), bias(std::move(bias_)), activation(activation_)
    {
        // Dense.swift:48-49
        if (bias.rank() != 1 || bias.shape[0] != weight.shape[1])
            throw Error(cudaErrorInvalidValue, "bias.shape[0] must equal weight.shape[1]");
    }
    Tensor<E> operator()(const Tensor<E>& input, cudaStream_t stream = nullptr) const
    {
        return matmul(input, false, weight, false, bias, activation, stream);
    }
};

// LSTMCell (Recurrent.swift:165-266): fusedWeight [(inputSize + hiddenSize) x 4 hiddenSize], fusedBias
// [4 hiddenSize]; one call is one time step through srtLstmCell.
template <typename E>
struct LSTMCell {
    struct State { Tensor<E> cell, hidden; };
    Tensor<E> fusedWeight, fusedBias;
    size_t hiddenSize;
    LSTMCell(Tensor<E> fusedWeight_, Tensor<E> fusedBias_)
        : fusedWeight(std::move(fusedWeight_)), fusedBias(std::move(fusedBias_)), hiddenSize(fusedWeight.shape[1] / 4)
    {
        if (fusedWeight.rank() != 2 || fusedWeight.shape[1] % 4 != 0 || fusedBias.rank() != 1 ||
            fusedBias.shape[0] != fusedWeight.shape[1])
            throw Error(cudaErrorInvalidValue, "fusedWeight is [(inputSize + hiddenSize) x 4 hiddenSize], fusedBias [4 hiddenSize]");
    }
    // zeroState(for:) (Recurrent.swift:245-248)
    State zeroState(const Tensor<E>& input) const
    {
        State s{Tensor<E>({input.shape[0], hiddenSize}), Tensor<E>({input.shape[0], hiddenSize})};
        s.cell.assign(std::vector<float>(s.cell.count(), 0.0f));
        s.hidden.assign(std::vector<float>(s.hidden.count(), 0.0f));
        return s;
    }
    State operator()(const Tensor<E>& input, const State& state, cudaStream_t stream = nullptr) const
    {
        State next{Tensor<E>({input.shape[0], hiddenSize}), Tensor<E>({input.shape[0], hiddenSize})};
        const srtTensorDescriptor x = input.descriptor(), h = state.hidden.descriptor(), c = state.cell.descriptor(),
                                  w = fusedWeight.descriptor(), b = fusedBias.descriptor(), nc = next.cell.descriptor(),
                                  nh = next.hidden.descriptor();
        check(srtLstmCell(input.data(), &x, state.hidden.data(), &h, state.cell.data(), &c, fusedWeight.data(), &w,
                          fusedBias.data(), &b, next.cell.data(), &nc, next.hidden.data(), &nh, stream),
              "srtLstmCell");
        return next;
    }
};

// RecurrentLayer.callAsFunction(_:initialState:) (Recurrent.swift:356-370)
template <typename E>
std::vector<typename LSTMCell<E>::State> runSequence(const LSTMCell<E>& cell, const std::vector<Tensor<E>>& inputs,
                                                     const typename LSTMCell<E>::State& initialState,
                                                     cudaStream_t stream = nullptr)
{
    std::vector<typename LSTMCell<E>::State> outputs;
    typename LSTMCell<E>::State state = initialState;
    for (const Tensor<E>& x : inputs) {
        state = cell(x, state, stream);
        outputs.push_back(state);
    }
    return outputs;
}

// MatrixLayout (cublaslt/MatrixLayout.swift:21-204): the same properties, a plain value instead of a cublasLt handle.
struct MatrixLayout {
    srtDataType type = real32F;
    Order order = Order::row;
    size_t rows = 0, cols = 0;
    long long leadingDimension = 0;
    int batchCount = 1;
    long long batchStride = 0;

    MatrixLayout() = default;
    MatrixLayout(srtDataType type_, Order order_, size_t rows_, size_t cols_, int batchCount_ = 1)
        : type(type_), order(order_), rows(rows_), cols(cols_), batchCount(batchCount_)
    {
        leadingDimension = static_cast<long long>(srtMatrixLayoutLeadingDimension(static_cast<srtOrder>(order), rows, cols));
        batchStride = static_cast<long long>(elementCount());
    }
    // MatrixLayout.init(_ tensor:) (MatrixLayout.swift:27-47) for a row- or col-ordered rank-2 tensor
    template <typename E>
    explicit MatrixLayout(const Tensor<E>& t)
        : type(ElementTraits<E>::type), order(t.strides[t.rank() - 1] == 1 ? Order::row : Order::col), rows(t.shape[t.rank() - 2]),
          cols(t.shape[t.rank() - 1])
    {
        leadingDimension = static_cast<long long>(order == Order::row ? t.strides[t.rank() - 2] : t.strides[t.rank() - 1]);
        batchStride = static_cast<long long>(elementCount());
    }
    size_t elementCount() const
    {
        return srtMatrixLayoutElementCount(static_cast<srtOrder>(order), rows, cols, static_cast<uint64_t>(leadingDimension));
    }
    size_t bufferElements() const { return rows && cols ? (batchCount - 1) * static_cast<size_t>(batchStride) + elementCount() : 0; }
    srtMatrixLayout raw() const
    {
        return srtMatrixLayout{type, static_cast<srtOrder>(order), rows, cols, leadingDimension, batchCount, batchStride};
    }
};

// MatrixTransform (cublaslt/MatrixTransform.swift:21-129): transA / transB and host scalars; callAsFunction runs
// C = alpha . op(A) + beta . op(B), which the reference's wrapper only describes.
struct MatrixTransform {
    bool transA = false, transB = false;
    void operator()(float alpha, const void* a, const MatrixLayout& aLayout, float beta, const void* b, const MatrixLayout* bLayout,
                    void* c, const MatrixLayout& cLayout, cudaStream_t stream = nullptr) const
    {
        const srtMatrixLayout la = aLayout.raw(), lc = cLayout.raw();
        srtMatrixLayout lb{};
        if (bLayout) lb = bLayout->raw();
        check(srtMatrixTransform(&alpha, a, &la, transA, &beta, b, bLayout ? &lb : nullptr, transB, c, &lc, stream),
              "srtMatrixTransform");
    }
};

}  // namespace srt_host
