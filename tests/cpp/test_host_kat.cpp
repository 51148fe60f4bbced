// The reference's matmul tests, restated over the C++ host mirror (swiftrt_b200/host/srt_host.hpp),
// which calls the CUDA library through its C ABI.  Literals: Tests/SwiftRTCoreTests/
// test_AlgebraicField.swift:551-645 (test_matmul is live there, the batched ones are commented out
// but numerically valid).  Exit code 0 = all checks passed; needs a GPU.
#include <cstdio>
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

int main()
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { std::printf("no CUDA device\n"); return 2; }
    test_matmul();
    test_batchMatmul();
    test_leftAndRightBatchMatmul();
    test_transposes_orders_and_types();
    test_dense_and_errors();
    uint32_t status = 1;
    EXPECT(srtMatmulCheckStatus(nullptr, &status) == cudaSuccess && status == 0);
    std::printf(failures ? "%d check(s) FAILED\n" : "all host-mirror checks passed (%d failures)\n", failures);
    return failures ? 1 : 0;
}
