// Tests of the C++ host layer (nz:: API) written the way NeuZephyr's own GoogleTest cases are
// (test/Test.cpp): build small tensors / nodes, compute the expectation on the host, compare with
// Tensor::operator== (abs 1e-6 or rel 1e-5). Test names match the reference's. Needs a GPU.
#include <NeuZephyr/Model.cuh>
#include <NeuZephyr/TensorOperations.cuh>

#include <cmath>
#include <cstdio>
#include <functional>
#include <random>
#include <string>
#include <vector>

using namespace nz;
using namespace nz::data;
using namespace nz::nodes;
using namespace nz::nodes::io;
using namespace nz::nodes::calc;

static int g_failed = 0, g_checks = 0;
static std::string g_current;
#define EXPECT_TRUE(cond)                                                                  \
    do {                                                                                   \
        g_checks++;                                                                        \
        if (!(cond)) {                                                                     \
            g_failed++;                                                                    \
            printf("  FAILED %s: %s (line %d)\n", g_current.c_str(), #cond, __LINE__);     \
        }                                                                                  \
    } while (0)
#define EXPECT_EQ(a, b) EXPECT_TRUE((a) == (b))
#define EXPECT_NEAR(a, b, tol) EXPECT_TRUE(std::fabs((double)(a) - (double)(b)) <= (tol))

struct TestCase {
    const char* name;
    std::function<void()> fn;
};
static std::vector<TestCase>& registry() {
    static std::vector<TestCase> r;
    return r;
}
struct Registrar {
    Registrar(const char* n, std::function<void()> f) { registry().push_back({n, std::move(f)}); }
};
#define TEST(suite, name)                                                \
    static void test_##suite##_##name();                                 \
    static Registrar reg_##suite##_##name(#suite "." #name, test_##suite##_##name); \
    static void test_##suite##_##name()

static std::vector<float> uniform(size_t n, float lo, float hi, unsigned seed) {
    std::mt19937 gen(seed);
    std::uniform_real_distribution<float> d(lo, hi);
    std::vector<float> v(n);
    for (auto& x : v) x = d(gen);
    return v;
}
static bool close_vec(const std::vector<float>& a, const std::vector<float>& b, double abs_tol = 1e-6, double rel = 1e-5) {
    if (a.size() != b.size()) return false;
    for (size_t i = 0; i < a.size(); i++) {
        const double d = std::fabs((double)a[i] - (double)b[i]);
        const double m = std::max(std::fabs((double)a[i]), std::fabs((double)b[i]));
        if (!(d <= abs_tol || d <= rel * m)) {
            printf("    mismatch at %zu: %g vs %g\n", i, a[i], b[i]);
            return false;
        }
    }
    return true;
}

// ---- test/Test.cpp:119-180: Tensor::operator* with N / C broadcast (fp32-accurate product) ----
TEST(TensorBasic, TensorMultiplicationTest) {
    const size_t n = 2, c = 3, m = 2, k = 3, p = 2;
    Tensor tensor1({n, 1, m, k});
    Tensor tensor2({1, c, k, p});
    std::vector<float> data1(n * m * k), data2(c * k * p);
    for (size_t i = 0; i < data1.size(); i++) data1[i] = (float)(i + 1);
    for (size_t i = 0; i < data2.size(); i++) data2[i] = (float)(i + 1);
    tensor1.dataInject(data1.begin(), data1.end());
    tensor2.dataInject(data2.begin(), data2.end());
    Tensor result = tensor1 * tensor2;
    EXPECT_TRUE(result.shape() == Dimension(n, c, m, p));
    std::vector<float> expected(n * c * m * p);
    for (size_t i = 0; i < n; i++)
        for (size_t j = 0; j < c; j++)
            for (size_t r = 0; r < m; r++)
                for (size_t q = 0; q < p; q++) {
                    float s = 0.f;
                    for (size_t t = 0; t < k; t++) s += data1[(i * m + r) * k + t] * data2[(j * k + t) * p + q];
                    expected[((i * c + j) * m + r) * p + q] = s;
                }
    Tensor want({n, c, m, p});
    want.dataInject(expected.begin(), expected.end());
    EXPECT_TRUE(result == want);
    // shapes that do not broadcast are refused (src/TensorOperations.cuh:1001-1003)
    bool threw = false;
    try {
        Tensor bad({1, 1, 4, 2});
        Tensor r2 = tensor1 * bad;
    } catch (const std::invalid_argument&) {
        threw = true;
    }
    EXPECT_TRUE(threw);
}

// operator* against a host product in double on random data: within abs 4e-6 or rel 1e-5 everywhere (the
// reference's rule is abs 1e-6 or rel 1e-5; results near zero miss its absolute part by the tensor core's
// truncating accumulator), which the fp16-operand tensor-core product misses by two orders of magnitude
TEST(TensorBasic, TensorMultiplicationRandomMatchesHostProduct) {
    const size_t m = 70, k = 200, p = 90;
    auto a = uniform(2 * m * k, -1, 1, 3), b = uniform(k * p, -1, 1, 4);
    Tensor A({2, 1, m, k}), B({1, 1, k, p});
    A.dataInject(a.begin(), a.end());
    B.dataInject(b.begin(), b.end());
    Tensor C = A * B;
    std::vector<float> expected(2 * m * p);
    for (size_t i = 0; i < 2; i++)
        for (size_t r = 0; r < m; r++)
            for (size_t q = 0; q < p; q++) {
                double s = 0;
                for (size_t t = 0; t < k; t++) s += (double)a[(i * m + r) * k + t] * (double)b[t * p + q];
                expected[(i * m + r) * p + q] = (float)s;
            }
    Tensor want({2, 1, m, p});
    want.dataInject(expected.begin(), expected.end());
    EXPECT_TRUE(close_vec(C.hostData(), expected, 4e-6, 1e-5));
    Tensor viaTensorCore({2, 1, m, p});
    GEMMTensorCore(viaTensorCore, A, B);
    EXPECT_TRUE(viaTensorCore != want);  // fp16 operand rounding is visible under the reference's rule
}

// ---- test/Test.cpp:708-751 ----
TEST(TensorCore, TensorCoreGEMMTest) {
    const size_t n = 2, c = 3, m = 2, k = 3, p = 2;
    Tensor tensor1({n, 1, m, k});
    Tensor tensor2({1, c, k, p});
    tensor1.dataInject({1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12});
    tensor2.dataInject({1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18});
    Tensor result({n, c, m, p});
    GEMMTensorCore(result, tensor1, tensor2);
    Tensor expected({n, c, m, p});
    expected.dataInject({22, 28, 49, 64, 58, 64, 139, 154, 94, 100, 229, 244,
                         76, 100, 103, 136, 220, 244, 301, 334, 364, 388, 499, 532});
    EXPECT_EQ(result, expected);
}

// ---- test/Test.cpp:753-818 ----
TEST(NodeBasic, MatMulForward) {
    InputNode input1({2, 1, 2, 3});
    InputNode input2({1, 3, 3, 2});
    input1.dataInject({1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12});
    input2.dataInject({1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18});
    MatMulNode mul(&input1, &input2);
    mul.forward();
    Tensor expected({2, 3, 2, 2});
    expected.dataInject({22, 28, 49, 64, 58, 64, 139, 154, 94, 100, 229, 244,
                         76, 100, 103, 136, 220, 244, 301, 334, 364, 388, 499, 532});
    Tensor got(mul.output->shape());
    got.dataInject(mul.output->hostData().begin(), mul.output->hostData().end());
    EXPECT_TRUE(close_vec(mul.output->hostData(), expected.hostData()));
}

// ---- test/Test.cpp:820-842 ----
TEST(NodeBasic, MatMulBackwardSpecial) {
    const size_t n = 2, c = 3, m = 2, k = 3, p = 2;
    InputNode input1({n, 1, m, k}, true);
    InputNode input2({1, c, k, p}, true);
    input1.output->fill(1);
    input2.output->fill(1);
    input1.output->zeroGrad();
    input2.output->zeroGrad();
    MatMulNode mul(&input1, &input2);
    mul.output->fill(1, true);
    mul.backward();
    Tensor expected1({n, 1, m, k}, true);
    Tensor expected2({1, c, k, p}, true);
    expected1.fill(1);
    expected1.fill(2 * c, true);
    expected2.fill(1);
    expected2.fill(2 * n, true);
    EXPECT_EQ(expected1, *input1.output);
    EXPECT_EQ(expected2, *input2.output);
}

// ---- test/Test.cpp:844-903 ----
TEST(NodeBasic, MatMulBackwardNormal) {
    const size_t n = 2, c = 3, m = 2, k = 3, p = 2;
    std::vector<float> Adata = {1, 2, 3, 4, 5, 6, 2, 3, 4, 5, 6, 7, 3, 4, 5, 6, 7, 8,
                                1, 2, 3, 4, 5, 6, 2, 3, 4, 5, 6, 7, 3, 4, 5, 6, 7, 8};
    std::vector<float> Bdata = {1, 4, 2, 5, 3, 6, 2, 5, 3, 6, 4, 7, 3, 6, 4, 7, 5, 8};
    std::vector<float> Cgrad(24, 1.f);
    std::vector<float> Agrad = {5, 7, 9, 5, 7, 9, 7, 9, 11, 7, 9, 11, 9, 11, 13, 9, 11, 13,
                                5, 7, 9, 5, 7, 9, 7, 9, 11, 7, 9, 11, 9, 11, 13, 9, 11, 13};
    std::vector<float> Bgrad = {10, 10, 14, 14, 18, 18, 14, 14, 18, 18, 22, 22, 18, 18, 22, 22, 26, 26};
    InputNode input1({n, c, m, k}, true);
    InputNode input2({1, c, k, p}, true);
    input1.dataInject(Adata.begin(), Adata.end());
    input2.dataInject(Bdata.begin(), Bdata.end());
    input1.output->zeroGrad();
    input2.output->zeroGrad();
    MatMulNode mul(&input1, &input2);
    mul.output->dataInject(Cgrad.begin(), Cgrad.end(), true);
    mul.backward();
    EXPECT_TRUE(close_vec(input1.output->hostGrad(), Agrad));
    EXPECT_TRUE(close_vec(input2.output->hostGrad(), Bgrad));
}

// ---- test/Test.cpp:615-706 ----
TEST(NodesBasic, AddForwardAndBackward) {
    const size_t n = 2, c = 3, h = 4, w = 5;
    auto d1 = uniform(n * h * w, -10, 10, 1), d2 = uniform(c * h * w, -10, 10, 2);
    InputNode input1({n, 1, h, w}, true);
    InputNode input2({1, c, h, w}, true);
    input1.dataInject(d1.begin(), d1.end());
    input2.dataInject(d2.begin(), d2.end());
    input1.output->zeroGrad();
    input2.output->zeroGrad();
    AddNode add(&input1, &input2);
    add.forward();
    std::vector<float> expected(n * c * h * w);
    for (size_t i = 0; i < n; i++)
        for (size_t j = 0; j < c; j++)
            for (size_t t = 0; t < h * w; t++) expected[(i * c + j) * h * w + t] = d1[i * h * w + t] + d2[j * h * w + t];
    EXPECT_TRUE(close_vec(add.output->hostData(), expected));
    // AddBackwardSpecial: all-ones upstream gradient
    std::vector<float> ones(n * c * h * w, 1.f);
    add.output->dataInject(ones.begin(), ones.end(), true);
    add.backward();
    EXPECT_TRUE(close_vec(input1.output->hostGrad(), std::vector<float>(n * h * w, (float)c)));
    EXPECT_TRUE(close_vec(input2.output->hostGrad(), std::vector<float>(c * h * w, (float)n)));
}

TEST(NodesBasic, AddBackwardNormal) {
    const size_t n = 2, c = 3, h = 4, w = 5;
    InputNode inputData({n, c, h, w}, true);
    InputNode Weights({1, c, h, w}, true);
    inputData.output->zeroGrad();
    Weights.output->zeroGrad();
    AddNode add(&inputData, &Weights);
    auto g = uniform(n * c * h * w, -10, 10, 3);
    std::vector<float> wg(c * h * w, 0.f);
    for (size_t l = 0; l < n; l++)
        for (size_t i = 0; i < c * h * w; i++) wg[i] += g[l * c * h * w + i];
    add.output->dataInject(g.begin(), g.end(), true);
    add.backward();
    EXPECT_TRUE(close_vec(inputData.output->hostGrad(), g));
    EXPECT_TRUE(close_vec(Weights.output->hostGrad(), wg, 1e-5));
}

// ---- test/Test.cpp:2880-3072 (index rule restated with correctly sized buffers) ----
TEST(TensorBasic, img2colTest) {
    const size_t n = 2, c = 3, h = 4, w = 5, kh = 3, kw = 3, stride = 1, pad = 1;
    const size_t Ho = (h + 2 * pad - kh) / stride + 1, Wo = (w + 2 * pad - kw) / stride + 1;
    auto in = uniform(n * c * h * w, 0.1f, 0.9f, 4);
    std::vector<float> expected(n * Ho * Wo * kh * kw * c, 0.f);
    for (size_t b = 0; b < n; ++b)
        for (size_t i = 0; i < Ho; ++i)
            for (size_t j = 0; j < Wo; ++j)
                for (size_t r = 0; r < kh; ++r)
                    for (size_t s = 0; s < kw; ++s)
                        for (size_t ci = 0; ci < c; ++ci) {
                            const int hi = (int)(i * stride) - (int)pad + (int)r, wi = (int)(j * stride) - (int)pad + (int)s;
                            float v = 0.f;
                            if (hi >= 0 && hi < (int)h && wi >= 0 && wi < (int)w) v = in[b * c * h * w + ci * h * w + hi * w + wi];
                            expected[b * Ho * Wo * kh * kw * c + (i * Wo + j) * kh * kw * c + ci * kh * kw + r * kw + s] = v;
                        }
    Tensor input({n, c, h, w});
    input.dataInject(in.begin(), in.end());
    auto result = tensorImg2col(input, kh, kw, stride, pad);
    EXPECT_TRUE(result.shape() == Dimension(n, 1, Ho * Wo, kh * kw * c));
    EXPECT_TRUE(close_vec(result.hostData(), expected));
    // node forward / backward
    InputNode node({n, c, h, w}, true);
    node.dataInject(in.begin(), in.end());
    node.output->zeroGrad();
    Img2ColNode col(&node, kh, kw, stride, pad);
    col.forward();
    EXPECT_TRUE(close_vec(col.output->hostData(), expected));
    auto g = uniform(expected.size(), 0.1f, 0.9f, 5);
    col.output->dataInject(g.begin(), g.end(), true);
    col.backward();
    std::vector<float> dx(n * c * h * w, 0.f);
    for (size_t b = 0; b < n; ++b)
        for (size_t pos = 0; pos < Ho * Wo; ++pos)
            for (size_t m = 0; m < c * kh * kw; ++m) {
                const size_t ci = m / (kh * kw), r = (m % (kh * kw)) / kw, s = m % kw;
                const int hi = (int)((pos / Wo) * stride) - (int)pad + (int)r, wi = (int)((pos % Wo) * stride) - (int)pad + (int)s;
                if (hi >= 0 && hi < (int)h && wi >= 0 && wi < (int)w)
                    dx[b * c * h * w + ci * h * w + hi * w + wi] += g[(b * Ho * Wo + pos) * c * kh * kw + m];
            }
    EXPECT_TRUE(close_vec(node.output->hostGrad(), dx, 1e-5));
}

// ---- test/Test.cpp:3074-3177 ----
TEST(TenorBasic, col2imgTest) {
    const size_t n = 2, c = 3, h = 4, w = 5;
    auto in = uniform(n * c * h * w, 0.1f, 0.9f, 6);
    std::vector<float> expected(n * c * h * w);
    for (size_t i = 0; i < n; i++)
        for (size_t j = 0; j < c; j++)
            for (size_t k = 0; k < h; k++)
                for (size_t l = 0; l < w; l++)
                    expected[i * c * h * w + j * h * w + k * w + l] = in[i * c * h * w + (k * w + l) * c + j];
    Tensor input({n, 1, h * w, c});
    input.dataInject(in.begin(), in.end());
    auto result = tensorCol2img(input, h, w);
    EXPECT_TRUE(close_vec(result.hostData(), expected));
    InputNode node({n, 1, h * w, c}, true);
    node.dataInject(in.begin(), in.end());
    Col2ImgNode c2i(&node, h, w);
    c2i.forward();
    EXPECT_TRUE(close_vec(c2i.output->hostData(), expected));
    c2i.output->dataInject(expected.begin(), expected.end(), true);
    c2i.backward();
    EXPECT_TRUE(close_vec(node.output->hostGrad(), in));
}

// ---- test/Test.cpp:1054-1108 ----
TEST(NodeBasic, ReLUForwardBackward) {
    auto in = uniform(2 * 3 * 4 * 5, -1, 1, 7), g = uniform(2 * 3 * 4 * 5, -1, 1, 8);
    InputNode node({2, 3, 4, 5}, true);
    node.dataInject(in.begin(), in.end());
    ReLUNode relu(&node);
    relu.forward();
    std::vector<float> e(in.size()), ge(in.size());
    for (size_t i = 0; i < in.size(); i++) {
        e[i] = in[i] > 0 ? in[i] : 0;
        ge[i] = in[i] > 0 ? g[i] : 0;
    }
    EXPECT_TRUE(close_vec(relu.output->hostData(), e));
    relu.output->dataInject(g.begin(), g.end(), true);
    relu.backward();
    EXPECT_TRUE(close_vec(node.output->hostGrad(), ge));
}

// ---- test/Test.cpp:3179-3385 ----
TEST(NodeBasic, AveragePoolingForwardBackward) {
    const size_t n = 2, c = 3, h = 4, w = 5, pool = 2, stride = 2, pad = 0;
    const size_t Ho = (h + 2 * pad - pool) / stride + 1, Wo = (w + 2 * pad - pool) / stride + 1;
    auto in = uniform(n * c * h * w, 0.1f, 0.9f, 9);
    std::vector<float> e(n * c * Ho * Wo, 0.f);
    for (size_t bc = 0; bc < n * c; bc++)
        for (size_t k = 0; k < Ho; k++)
            for (size_t l = 0; l < Wo; l++) {
                float s = 0;
                int cnt = 0;
                for (size_t r = 0; r < pool; r++)
                    for (size_t t = 0; t < pool; t++) {
                        const size_t hi = k * stride + r, wi = l * stride + t;
                        if (hi < h && wi < w) { s += in[bc * h * w + hi * w + wi]; cnt++; }
                    }
                e[bc * Ho * Wo + k * Wo + l] = s / cnt;
            }
    InputNode node({n, c, h, w}, true);
    node.dataInject(in.begin(), in.end());
    node.output->zeroGrad();
    AveragePoolingNode ap(&node, pool, stride, pad);
    ap.forward();
    EXPECT_TRUE(close_vec(ap.output->hostData(), e));
    auto g = uniform(e.size(), 0.1f, 0.9f, 10);
    ap.output->dataInject(g.begin(), g.end(), true);
    ap.backward();
    std::vector<float> dx(in.size(), 0.f);
    for (size_t bc = 0; bc < n * c; bc++)
        for (size_t k = 0; k < Ho; k++)
            for (size_t l = 0; l < Wo; l++)
                for (size_t r = 0; r < pool; r++)
                    for (size_t t = 0; t < pool; t++) {
                        const size_t hi = k * stride + r, wi = l * stride + t;
                        if (hi < h && wi < w) dx[bc * h * w + hi * w + wi] += g[bc * Ho * Wo + k * Wo + l] / (pool * pool);
                    }
    EXPECT_TRUE(close_vec(node.output->hostGrad(), dx));
}

// ---- test/Test.cpp:1735-1870 ----
TEST(NodeBasic, SoftmaxForwardBackward) {
    const size_t n = 3, m = 8;
    auto in = uniform(n * m, -1, 1, 11), g = uniform(n * m, -1, 1, 12);
    InputNode node({n, 1, m, 1}, true);
    node.dataInject(in.begin(), in.end());
    SoftmaxNode sm(&node);
    sm.roundLikeReference = false;
    sm.forward();
    std::vector<float> y(n * m), dx(n * m);
    for (size_t b = 0; b < n; b++) {
        double s = 0;
        for (size_t i = 0; i < m; i++) s += std::exp((double)in[b * m + i]);
        for (size_t i = 0; i < m; i++) y[b * m + i] = (float)(std::exp((double)in[b * m + i]) / s);
        double dot = 0;
        for (size_t i = 0; i < m; i++) dot += (double)y[b * m + i] * g[b * m + i];
        for (size_t i = 0; i < m; i++) dx[b * m + i] = (float)(y[b * m + i] * (g[b * m + i] - dot));
    }
    EXPECT_TRUE(close_vec(sm.output->hostData(), y, 1e-6, 1e-5));
    sm.output->dataInject(g.begin(), g.end(), true);
    sm.backward();
    EXPECT_TRUE(close_vec(node.output->hostGrad(), dx, 1e-6, 1e-4));
}

// ---- test/Test.cpp:1937-2000, 2774-2825 ----
TEST(NodeLoss, BCEForwardBackward) {
    const size_t n = 4 * 16;
    auto p = uniform(n, 0.1f, 0.9f, 13), tr = uniform(n, 0.f, 1.f, 14);
    for (auto& v : tr) v = v > 0.5f ? 1.f : 0.f;
    InputNode pred({4, 1, 16, 1}, true);
    InputNode target({4, 1, 16, 1});
    pred.dataInject(p.begin(), p.end());
    target.dataInject(tr.begin(), tr.end());
    loss::BinaryCrossEntropyNode bce(&pred, &target);
    bce.forward();
    double e = 0;
    std::vector<float> ge(n);
    for (size_t i = 0; i < n; i++) {
        e += (-tr[i] * std::log((double)p[i]) - (1 - tr[i]) * std::log(1.0 - p[i])) / n;
        ge[i] = (float)(((double)p[i] - tr[i]) / ((double)p[i] * (1.0 - p[i])) / n);
    }
    EXPECT_NEAR(bce.getLoss(), e, 1e-2);  // the reference compares losses to 1e-2
    EXPECT_NEAR(bce.getLoss(), e, 1e-5);
    bce.backward();
    EXPECT_TRUE(close_vec(pred.output->hostGrad(), ge, 1e-7, 1e-5));
}

// ---- test/Test.cpp:2398-2451 ----
TEST(OptimizerBasic, AdamTest) {
    const size_t sz = 2 * 3 * 3 * 4;
    const float lr = 0.01f, b1 = 0.9f, b2 = 0.999f, eps = 1e-6f;
    auto data = uniform(sz, -10, 10, 15), grad = uniform(sz, -10, 10, 16);
    std::vector<float> m(sz, 0.f), v(sz, 0.f), e = data;
    for (int it = 1; it <= 2; it++)
        for (size_t i = 0; i < sz; i++) {
            m[i] = b1 * m[i] + (1 - b1) * grad[i];
            v[i] = b2 * v[i] + (1 - b2) * grad[i] * grad[i];
            const float mm = m[i] / (1 - std::pow(b1, (float)it)), vv = v[i] / (1 - std::pow(b2, (float)it));
            e[i] = e[i] - (lr / (std::sqrt(vv) + eps)) * mm;
        }
    InputNode input({2, 3, 3, 4}, true);
    input.dataInject(data.begin(), data.end());
    input.dataInject(grad.begin(), grad.end(), true);
    opt::Adam optimizer(lr, b1, b2);
    optimizer.step(&input);
    optimizer.step(&input);
    EXPECT_TRUE(close_vec(input.output->hostData(), e, 1e-6, 2e-5));
}

// ---- a model in the style of README.md:62-90 and Model.* tests (test/Test.cpp:2721-2878):
// the fused graph must agree with the reference's node-by-node composition on the same weights.
class SegModel : public Model {
public:
    InputNode input, target;
    Node* out = nullptr;
    SegModel(size_t batch, size_t hw, bool fused) : input({batch, 3, hw, hw}), target({batch, 1, 16, 1}) {
        setFused(fused);
        computeGraph.addInput(&input);
        computeGraph.addInput(&target);
        auto x = Conv2d(&input, 16, 3, 3, 1, 1, true, false, fused);
        if (!fused) x = ReLU(x);
        x = Conv2d(x, 16, 3, 3, 1, 1);
        x = AvgPool2d(x, 5, 2);
        x = Linear(x, 16);
        out = Softmax(x);
        BCELoss(out, &target);
    }
};

TEST(Model, FusedEqualsNodeByNodeOneAdamStep) {
    const size_t batch = 3, hw = 12;
    SegModel a(batch, hw, true), b(batch, hw, false);
    auto x = uniform(batch * 3 * hw * hw, -1, 1, 20);
    std::vector<float> tg(batch * 16);
    std::mt19937 gen(21);
    for (auto& v : tg) v = (gen() & 1) ? 1.f : 0.f;
    a.input.dataInject(x.begin(), x.end());
    b.input.dataInject(x.begin(), x.end());
    a.target.dataInject(tg.begin(), tg.end());
    b.target.dataInject(tg.begin(), tg.end());
    // identical small weights in both; parameter order differs only by where biases are created
    auto pa = a.parameters(), pb = b.parameters();
    EXPECT_EQ(pa.size(), pb.size());
    // fused order: w1,b1,w2,b2,wl,bl ; node-by-node order: w1,b1,w2,b2,wl,bl (Bias creates its node after Mul)
    for (size_t i = 0; i < pa.size(); i++) {
        EXPECT_EQ(pa[i]->output->size(), pb[i]->output->size());
        auto w = uniform(pa[i]->output->size(), -0.2f, 0.2f, 30 + (unsigned)i);
        pa[i]->dataInject(w.begin(), w.end());
        pb[i]->dataInject(w.begin(), w.end());
    }
    a.graph().zeroGrad();
    b.graph().zeroGrad();
    a.forward();
    b.forward();
    EXPECT_TRUE(close_vec(a.out->output->hostData(), b.out->output->hostData(), 1e-5, 1e-3));
    EXPECT_NEAR(a.getLoss(), b.getLoss(), 1e-4);
    a.backward();
    b.backward();
    for (size_t i = 0; i < pa.size(); i++)
        EXPECT_TRUE(close_vec(pa[i]->output->hostGrad(), pb[i]->output->hostGrad(), 2e-5, 2e-2));
    opt::Adam oa(0.01f, 0.9f, 0.999f), ob(0.01f, 0.9f, 0.999f);
    oa.perCallTimeStep = ob.perCallTimeStep = false;  // same t for every parameter in both graphs
    oa.nextIteration();
    ob.nextIteration();
    a.update(&oa);
    b.update(&ob);
    for (size_t i = 0; i < pa.size(); i++)
        EXPECT_TRUE(close_vec(pa[i]->output->hostData(), pb[i]->output->hostData(), 2e-3, 1e-2));
    // gradients are zeroed by update (src/Model.cu:20-23)
    for (size_t i = 0; i < pa.size(); i++) {
        auto g = pa[i]->output->hostGrad();
        bool allzero = true;
        for (float v : g) allzero &= (v == 0.f);
        EXPECT_TRUE(allzero);
    }
}

// The fused Conv2dNode takes its composed fallback (img2col + GEMM + col2img through the library's node-level
// entry points) for strides other than 1 and non-square kernels. With more output columns than output channels
// a shape mix-up in that fallback's backward would read past dY; the fused graph must agree with the
// node-by-node composition on the output, the loss and every gradient, the input's included.
class StridedModel : public Model {
public:
    InputNode input, target;
    Node* out = nullptr;
    StridedModel(size_t batch, size_t hw, bool fused) : input({batch, 3, hw, hw}, true), target({batch, 1, 4, 1}) {
        setFused(fused);
        computeGraph.addInput(&input);
        computeGraph.addInput(&target);
        auto x = Conv2d(&input, 8, 3, 2, 2, 1);  // 3x2 kernel, stride 2, pad 1: 8 channels, 12 x 13 outputs
        x = Linear(x, 4);
        out = Softmax(x);
        BCELoss(out, &target);
    }
};

TEST(Model, FusedFallbackStride2NonSquareEqualsNodeByNode) {
    const size_t batch = 2, hw = 24;
    StridedModel a(batch, hw, true), b(batch, hw, false);
    auto x = uniform(batch * 3 * hw * hw, -1, 1, 50);
    std::vector<float> tg(batch * 4);
    std::mt19937 gen(51);
    for (auto& v : tg) v = (gen() & 1) ? 1.f : 0.f;
    a.input.dataInject(x.begin(), x.end());
    b.input.dataInject(x.begin(), x.end());
    a.target.dataInject(tg.begin(), tg.end());
    b.target.dataInject(tg.begin(), tg.end());
    auto pa = a.parameters(), pb = b.parameters();
    EXPECT_EQ(pa.size(), pb.size());
    for (size_t i = 0; i < pa.size() && i < pb.size(); i++) {
        EXPECT_EQ(pa[i]->output->size(), pb[i]->output->size());
        auto w = uniform(pa[i]->output->size(), -0.2f, 0.2f, 60 + (unsigned)i);
        pa[i]->dataInject(w.begin(), w.end());
        pb[i]->dataInject(w.begin(), w.end());
    }
    a.graph().zeroGrad();
    b.graph().zeroGrad();
    a.forward();
    b.forward();
    EXPECT_TRUE(close_vec(a.out->output->hostData(), b.out->output->hostData(), 1e-5, 1e-3));
    EXPECT_NEAR(a.getLoss(), b.getLoss(), 1e-4);
    a.backward();
    b.backward();
    for (size_t i = 0; i < pa.size() && i < pb.size(); i++)
        EXPECT_TRUE(close_vec(pa[i]->output->hostGrad(), pb[i]->output->hostGrad(), 2e-5, 2e-2));
    EXPECT_TRUE(close_vec(a.input.output->hostGrad(), b.input.output->hostGrad(), 2e-5, 2e-2));
}

TEST(Model, LossDecreasesOverSteps) {
    SegModel m(4, 16, true);
    auto x = uniform(4 * 3 * 16 * 16, -1, 1, 40);
    std::vector<float> tg(4 * 16);
    std::mt19937 gen(41);
    for (auto& v : tg) v = (gen() & 1) ? 1.f : 0.f;
    m.input.dataInject(x.begin(), x.end());
    m.target.dataInject(tg.begin(), tg.end());
    for (auto* p : m.parameters()) {
        auto w = uniform(p->output->size(), -0.1f, 0.1f, 50);
        p->dataInject(w.begin(), w.end());
    }
    m.graph().zeroGrad();
    opt::Adam adam(0.01f, 0.9f, 0.999f);
    float first = 0, last = 0, prev_total = 0;
    for (int it = 0; it < 8; it++) {
        m.forward();
        const float total = m.getLoss();  // accumulates like the reference's loss node
        const float step_loss = total - prev_total;
        prev_total = total;
        if (it == 0) first = step_loss;
        last = step_loss;
        m.backward();
        m.update(&adam);
    }
    EXPECT_TRUE(std::isfinite(last));
    EXPECT_TRUE(last < first);
}

TEST(Model, UpdateStepsParametersOnlyUnlessAsked) {
    // The reference steps every node that requires a gradient (src/ComputeGraph.cu:541-547),
    // activations included; here that is opt-in because forward() overwrites them anyway.
    for (int all = 0; all < 2; all++) {
        SegModel m(2, 12, true);
        auto x = uniform(2 * 3 * 12 * 12, -1, 1, 60);
        std::vector<float> tg(2 * 16, 1.f);
        m.input.dataInject(x.begin(), x.end());
        m.target.dataInject(tg.begin(), tg.end());
        for (auto* p : m.parameters()) {
            auto w = uniform(p->output->size(), -0.1f, 0.1f, 61);
            p->dataInject(w.begin(), w.end());
        }
        m.graph().zeroGrad();
        m.graph().stepIntermediateNodes(all != 0);
        m.forward();
        m.backward();
        const auto hidden_before = m.out->inputs[0]->output->hostData();  // the Linear node's output
        const auto w_before = m.parameters()[0]->output->hostData();
        opt::Adam adam(0.01f, 0.9f, 0.999f);
        m.update(&adam);
        const auto hidden_after = m.out->inputs[0]->output->hostData();
        const auto w_after = m.parameters()[0]->output->hostData();
        bool hidden_same = true, w_same = true;
        for (size_t i = 0; i < hidden_before.size(); i++) hidden_same &= (hidden_before[i] == hidden_after[i]);
        for (size_t i = 0; i < w_before.size(); i++) w_same &= (w_before[i] == w_after[i]);
        EXPECT_TRUE(!w_same);
        EXPECT_EQ(hidden_same, all == 0);
    }
    // ComputeGraph::update leaves gradients alone; Model::update zeroes them (src/Model.cu:20-23)
    SegModel m(2, 12, true);
    auto x = uniform(2 * 3 * 12 * 12, -1, 1, 62);
    std::vector<float> tg(2 * 16, 0.f);
    m.input.dataInject(x.begin(), x.end());
    m.target.dataInject(tg.begin(), tg.end());
    for (auto* p : m.parameters()) {
        auto w = uniform(p->output->size(), -0.1f, 0.1f, 63);
        p->dataInject(w.begin(), w.end());
    }
    m.graph().zeroGrad();
    m.forward();
    m.backward();
    opt::Adam adam(0.01f, 0.9f, 0.999f);
    m.graph().update(&adam);
    bool any = false;
    for (float v : m.parameters()[0]->output->hostGrad()) any |= (v != 0.f);
    EXPECT_TRUE(any);
}

// ---- ComputeGraph::save / load (src/ComputeGraph.cu:553-811) with four-extent shapes and Adam state ----
TEST(ComputeGraph, SaveLoadRoundTripResumesTraining) {
    const char* path = "/tmp/nz_host_tests_graph.json";
    SegModel m(2, 12, true);
    auto x = uniform(2 * 3 * 12 * 12, -1, 1, 70);
    std::vector<float> tg(2 * 16);
    std::mt19937 gen(71);
    for (auto& v : tg) v = (gen() & 1) ? 1.f : 0.f;
    m.input.dataInject(x.begin(), x.end());
    m.target.dataInject(tg.begin(), tg.end());
    for (size_t i = 0; i < m.parameters().size(); i++) {
        auto w = uniform(m.parameters()[i]->output->size(), -0.2f, 0.2f, 72 + (unsigned)i);
        m.parameters()[i]->dataInject(w.begin(), w.end());
    }
    m.graph().zeroGrad();
    opt::Adam adam(0.001f, 0.9f, 0.999f);
    m.forward();
    m.backward();
    m.update(&adam);
    m.forward();
    m.backward();  // saved with live gradients and one step of Adam history
    m.graph().save(path, &adam);

    graph::ComputeGraph g2;
    opt::Adam adam2(0.001f, 0.9f, 0.999f);
    g2.load(path, &adam2);
    EXPECT_EQ(g2.getNodes().size(), m.graph().getNodes().size());
    EXPECT_EQ(adam2.counter(), adam.counter());
    // every tensor (all four extents) and every gradient came back bit for bit
    const auto& a = m.graph().getNodes();
    const auto& b = g2.getNodes();
    for (size_t i = 0; i < a.size() && i < b.size(); i++) {
        EXPECT_TRUE(a[i]->type == b[i]->type);
        EXPECT_TRUE(a[i]->output->shape() == b[i]->output->shape());
        EXPECT_TRUE(a[i]->output->hostData() == b[i]->output->hostData());
        if (a[i]->output->requiresGrad()) EXPECT_TRUE(a[i]->output->hostGrad() == b[i]->output->hostGrad());
    }
    // and training resumes identically: same Adam moments, same per-call time steps
    m.update(&adam);
    g2.update(&adam2);
    g2.zeroGrad();
    EXPECT_EQ(adam2.counter(), adam.counter());
    size_t pi = 0;
    for (size_t i = 0; i < a.size(); i++)
        if (a[i]->inputs.empty() && a[i]->output->requiresGrad()) {
            EXPECT_TRUE(a[i]->output->hostData() == b[i]->output->hostData());
            pi++;
        }
    EXPECT_EQ(pi, m.parameters().size());
    m.forward();
    g2.forward();
    EXPECT_TRUE(close_vec(m.out->output->hostData(), g2.getOutputs().at(0)->inputs[0]->output->hostData(), 1e-6, 1e-5));
    // an unknown node type and a second load are refused
    bool threw = false;
    try {
        g2.load(path);
    } catch (const std::runtime_error&) {
        threw = true;
    }
    EXPECT_TRUE(threw);
    remove(path);
}

TEST(ComputeGraph, LoadsFileInTheReferenceLayout) {
    // what the reference's save() writes: two extents in "shape", default stream precision
    const char* path = "/tmp/nz_host_tests_ref_layout.json";
    FILE* f = fopen(path, "w");
    fputs("[\n  {\n    \"type\": \"Input\",\n    \"name\": \"Input_0\",\n    \"pre\": [],\n    \"post\": [2],\n"
          "    \"shape\": [1, 1],\n    \"data\": [1, 2, 3, 4.5],\n    \"requires_grad\": true,\n    \"grad\": [0, 0, 0, 0]\n  },\n"
          "  {\n    \"type\": \"Input\",\n    \"name\": \"Input_1\",\n    \"pre\": [],\n    \"post\": [2],\n"
          "    \"shape\": [1, 1],\n    \"data\": [10, 20, 30, 40],\n    \"requires_grad\": false,\n    \"grad\": []\n  },\n"
          "  {\n    \"type\": \"Add\",\n    \"name\": \"Add_2\",\n    \"pre\": [0, 1],\n    \"post\": [],\n"
          "    \"shape\": [1, 1],\n    \"data\": [0, 0, 0, 0],\n    \"requires_grad\": true,\n    \"grad\": [0, 0, 0, 0]\n  }\n]\n", f);
    fclose(f);
    graph::ComputeGraph g;
    g.load(path);
    EXPECT_EQ(g.getNodes().size(), (size_t)3);
    EXPECT_TRUE(g["Add_2"] != nullptr && g["Input_1"] != nullptr && g["nope"] == nullptr);
    EXPECT_TRUE(g["Input_0"]->output->shape() == Dimension(1, 1, 4, 1));
    g.forward();
    const auto sum = g["Add_2"]->output->hostData();
    EXPECT_TRUE(sum == std::vector<float>({11.f, 22.f, 33.f, 44.5f}));
    remove(path);
}

TEST(StreamManager, OrderingAndSync) {
    auto& sm = cuStrm::StreamManager<float>::Instance();
    EXPECT_EQ(sm.streamCount(), (size_t)16);
    // a chain of dependent operations issued on rotating streams must be ordered by the events
    Tensor t({1, 1, 256, 256});
    t.fill(1.f);
    for (int i = 0; i < 40; i++) {
        Tensor u = ReLU(t);  // reads t on a fresh stream
        t.fill((float)(i + 2));  // writes t on yet another stream: must wait for the reader
        auto h = u.hostData();
        bool ok = true;
        for (float v : h) ok &= (v == (float)(i + 1));
        EXPECT_TRUE(ok);
    }
    sm.sync();
}

int main(int argc, char** argv) {
    const std::string filter = argc > 1 ? argv[1] : "";
    int ran = 0;
    for (auto& t : registry()) {
        if (!filter.empty() && std::string(t.name).find(filter) == std::string::npos) continue;
        g_current = t.name;
        const int before = g_failed;
        try {
            t.fn();
        } catch (const std::exception& e) {
            g_failed++;
            printf("  EXCEPTION in %s: %s\n", t.name, e.what());
        }
        printf("[%s] %s\n", g_failed == before ? "  OK  " : "FAILED", t.name);
        ran++;
    }
    cuStrm::StreamManager<float>::Instance().sync();
    int status = 0;
    nzb_device_status(&status);
    printf("%d tests, %d checks, %d failures, device status %d\n", ran, g_checks, g_failed, status);
    return (g_failed || status) ? 1 : 0;
}
