// The reference's matmul tests, restated over the C++ host mirror (swiftrt_b200/host/srt_host.hpp),
// which calls the CUDA library through its C ABI.  Literals: Tests/SwiftRTCoreTests/
// test_AlgebraicField.swift:551-645 (test_matmul is live there, the batched ones are commented out
// but numerically valid), and the LSTM golden sequence of Tests/SwiftRTLayerTests/test_Recurrent.swift.
// Argument: path of tests/golden/lstm_kat.json.  Exit code 0 = all checks passed; needs a GPU.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "srt_host.hpp"

using namespace srt_host;

static int failures = 0;
#define EXPECT(cond) do { if (!(cond)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); ++failures; } } while (0)

static bool equal(const std::vector<float>& a, std::initializer_list<float> b) { return a == std::vector<float>(b); }

static void test_matmul()
{
    auto a = array(0, 6, {3, 2});
    auto b = array(0, 8, {2, 4});
    auto c = matmul(a, b);
    EXPECT(equal(c.values(), {4, 5, 6, 7, 12, 17, 22, 27, 20, 29, 38, 47}));
    // pullback(at: a, b) { matmul($0, $1) }(ones(like: c))
    auto g = matmulGradients(ones<float>({3, 4}), a, false, b, false);
    EXPECT(equal(g.first.values(), {6, 22, 6, 22, 6, 22}));
    EXPECT(equal(g.second.values(), {6, 6, 6, 6, 9, 9, 9, 9}));
}

static void test_batchMatmul()
{
    auto a = array(0, 12, {2, 3, 2});
    auto b = array(0, 16, {2, 2, 4});
    auto c = matmul(a, b);
    EXPECT(equal(c.values(), {4, 5, 6, 7, 12, 17, 22, 27, 20, 29, 38, 47,
                              132, 145, 158, 171, 172, 189, 206, 223, 212, 233, 254, 275}));
    auto g = matmulGradients(ones<float>({2, 3, 4}), a, false, b, false);
    EXPECT(equal(g.first.values(), {6, 22, 6, 22, 6, 22, 38, 54, 38, 54, 38, 54}));
    EXPECT(equal(g.second.values(), {6, 6, 6, 6, 9, 9, 9, 9, 24, 24, 24, 24, 27, 27, 27, 27}));
}

static void test_leftAndRightBatchMatmul()
{
    auto a3 = array(0, 12, {2, 3, 2});
    auto b2 = array(0, 8, {2, 4});
    auto c = matmul(a3, b2);                       // rank-2 rhs used for every batch item
    std::vector<float> v = c.values();
    EXPECT(equal(std::vector<float>(v.begin(), v.begin() + 12), {4, 5, 6, 7, 12, 17, 22, 27, 20, 29, 38, 47}));
    auto a2 = array(0, 6, {3, 2});
    auto b3 = array(0, 16, {2, 2, 4});
    auto d = matmul(a2, b3);
    EXPECT(equal(d.values(), {4, 5, 6, 7, 12, 17, 22, 27, 20, 29, 38, 47,
                              12, 13, 14, 15, 52, 57, 62, 67, 92, 101, 110, 119}));
}

static void test_transposes_orders_and_types()
{
    // .t views and col order describe the same logical matrices: same products
    auto a = array(0, 6, {3, 2});
    auto b = array(0, 8, {2, 4});
    auto at = array({0, 2, 4, 1, 3, 5}, {2, 3});   // a transposed, stored
    auto bt = array({0, 4, 1, 5, 2, 6, 3, 7}, {4, 2});
    const std::initializer_list<float> want = {4, 5, 6, 7, 12, 17, 22, 27, 20, 29, 38, 47};
    EXPECT(equal(matmul(at, true, b, false).values(), want));
    EXPECT(equal(matmul(a, false, bt, true).values(), want));
    EXPECT(equal(matmul(at, true, bt, true).values(), want));
    EXPECT(equal(matmul(at.t(), false, bt.t(), false).values(), want));
    auto a_col = array(0, 6, {3, 2}, Order::col);  // logical values equal, storage [0,2,4,1,3,5]
    auto c_col = matmul(a_col, b);
    EXPECT(c_col.order == Order::col && c_col.strides[0] == 1 && c_col.strides[1] == 3);
    EXPECT(equal(c_col.values(), want));
    EXPECT(equal(matmul(array<__nv_bfloat16>(0, 6, {3, 2}), array<__nv_bfloat16>(0, 8, {2, 4})).values(), want));
    EXPECT(equal(matmul(array<__half>(0, 6, {3, 2}), array<__half>(0, 8, {2, 4})).values(), want));
}

static void test_dense_and_errors()
{
    auto x = array({1, -2, 3, -4, 5, -6}, {3, 2});
    auto w = array({1, 0, -1, 2, 0.5f, 1, -1, 0}, {2, 4});
    auto bias = array({0.5f, -0.5f, 0, 100}, {4});
    Dense<float> layer(w, bias, ActivationType::relu);
    // x.w + b = [[0.5,-2.5,1,102],[1.5,-4.5,1,106],[2.5,-6.5,1,110]] -> relu
    EXPECT(equal(layer(x).values(), {0.5f, 0, 1, 102, 1.5f, 0, 1, 106, 2.5f, 0, 1, 110}));
    bool threw = false;
    try { matmul(array(0, 6, {3, 2}), array(0, 12, {3, 4})); } catch (const Error& e) { threw = e.code == cudaErrorInvalidValue; }
    EXPECT(threw);
    threw = false;
    try { Dense<float>(w, array({1, 2, 3}, {3}), ActivationType::relu); } catch (const Error&) { threw = true; }
    EXPECT(threw);
}

// Row order -> colTiledTC32x32 -> row order: the round trip returns the values, and an element sits where the
// order's formula (Tensor.swift:222) puts it.
static void test_matrix_transform()
{
    const size_t rows = 70, cols = 45;
    std::vector<float> v(rows * cols);
    for (size_t i = 0; i < v.size(); ++i) v[i] = static_cast<float>(i % 251) - 125.0f;
    auto x = array(v, {rows, cols});
    MatrixLayout rowLayout(x), tiled(real32F, Order::colTiledTC32x32, rows, cols);
    EXPECT(tiled.leadingDimension == 32 * 96 && rowLayout.leadingDimension == (long long)cols);
    float* buf = nullptr;
    EXPECT(cudaMalloc(&buf, tiled.bufferElements() * sizeof(float)) == cudaSuccess);
    Tensor<float> y({rows, cols});
    MatrixTransform transform;
    transform(1.0f, x.data(), rowLayout, 0.0f, nullptr, nullptr, buf, tiled);
    transform(2.0f, buf, tiled, 0.0f, nullptr, nullptr, y.data(), MatrixLayout(y));
    std::vector<float> twice(v);
    for (float& f : twice) f *= 2.0f;
    EXPECT(y.values() == twice);
    const size_t r = 37, c = 40, q = r % 32;
    const size_t off = (c / 32) * tiled.leadingDimension + (r / 32) * 1024 + (((q % 8) / 2 * 4 + q / 8) * 2 + q % 2) * 32 + c % 32;
    float one = 0;
    EXPECT(cudaMemcpy(&one, buf + off, sizeof one, cudaMemcpyDeviceToHost) == cudaSuccess && one == v[r * cols + c]);
    bool threw = false;
    try { transform(1.0f, x.data(), rowLayout, 0.0f, nullptr, nullptr, buf, MatrixLayout(real32F, Order::colTiledTC32x32, rows, cols + 1)); }
    catch (const Error& e) { threw = e.code == cudaErrorInvalidValue; }
    EXPECT(threw);
    cudaFree(buf);
}

// All numbers of the (possibly nested) array stored under `key` in a JSON text, flattened.
static std::vector<float> json_numbers(const std::string& text, const std::string& key)
{
    std::vector<float> out;
    size_t pos = text.find("\"" + key + "\"");
    if (pos == std::string::npos) return out;
    pos = text.find('[', pos);
    int depth = 0;
    for (size_t i = pos; i < text.size(); ++i) {
        const char ch = text[i];
        if (ch == '[') ++depth;
        else if (ch == ']') { if (--depth == 0) break; }
        else if (ch == '-' || (ch >= '0' && ch <= '9')) {
            char* end = nullptr;
            out.push_back(std::strtof(text.c_str() + i, &end));
            i = static_cast<size_t>(end - text.c_str()) - 1;
        }
    }
    return out;
}

// The reference's LSTM golden data (Tests/SwiftRTLayerTests/test_Recurrent.swift:97-167), read from the
// fixture next to the Python tests: four time steps, hidden state after each, final cell state, to 1e-6.
static void test_lstm_golden_sequence(const char* fixture)
{
    std::ifstream in(fixture);
    EXPECT(in.good());
    if (!in.good()) return;
    std::stringstream buf;
    buf << in.rdbuf();
    const std::string text = buf.str();
    const auto inputs = json_numbers(text, "inputs"), w = json_numbers(text, "fused_weight"), b = json_numbers(text, "fused_bias"),
               c0 = json_numbers(text, "initial_cell"), h0 = json_numbers(text, "initial_hidden"),
               want_h = json_numbers(text, "expected_hidden_per_step"), want_c = json_numbers(text, "expected_final_cell");
    EXPECT(inputs.size() == 16 && w.size() == 128 && b.size() == 16 && want_h.size() == 16 && want_c.size() == 4);
    if (failures) return;
    LSTMCell<float> cell(array(w, {8, 16}), array(b, {16}));
    EXPECT(cell.hiddenSize == 4);
    std::vector<Tensor<float>> steps;
    for (int t = 0; t < 4; ++t) steps.push_back(array(std::vector<float>(inputs.begin() + 4 * t, inputs.begin() + 4 * t + 4), {1, 4}));
    LSTMCell<float>::State init{array(c0, {1, 4}), array(h0, {1, 4})};
    const auto outputs = runSequence(cell, steps, init);
    EXPECT(outputs.size() == 4);
    float worst = 0.0f;
    for (int t = 0; t < 4; ++t) {
        const auto h = outputs[t].hidden.values();
        for (int j = 0; j < 4; ++j) worst = std::fmax(worst, std::fabs(h[j] - want_h[4 * t + j]));
    }
    const auto c = outputs.back().cell.values();
    for (int j = 0; j < 4; ++j) worst = std::fmax(worst, std::fabs(c[j] - want_c[j]));
    EXPECT(worst <= 1e-6f);
    const auto zero = cell.zeroState(steps[0]);
    EXPECT(zero.cell.shape == std::vector<size_t>({1, 4}) && zero.hidden.values() == std::vector<float>(4, 0.0f));
}

int main(int argc, char** argv)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { std::printf("no CUDA device\n"); return 2; }
    test_matmul();
    test_batchMatmul();
    test_leftAndRightBatchMatmul();
    test_transposes_orders_and_types();
    test_dense_and_errors();
    test_matrix_transform();
    test_lstm_golden_sequence(argc > 1 ? argv[1] : "tests/golden/lstm_kat.json");
    uint32_t status = 1;
    EXPECT(srtMatmulCheckStatus(nullptr, &status) == cudaSuccess && status == 0);
    std::printf(failures ? "%d check(s) FAILED\n" : "all host-mirror checks passed (%d failures)\n", failures);
    return failures ? 1 : 0;
}
