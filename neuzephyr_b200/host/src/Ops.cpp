// Tensor-level operations and raw-pointer wrappers: StreamManager ordering around libnzb calls.
#include <NeuZephyr/TensorOperations.cuh>

#include <nzb.h>

#include <algorithm>

namespace nz::data {

using SM = cuStrm::StreamManager<float>;

static void shape4(const Dimension& d, int64_t* out) {
    for (int i = 0; i < 4; i++) out[i] = (int64_t)d[i];
}

static void gemm4(bool backward, float* A, float* B, float* C, const Dimension& sa, const Dimension& sb,
                  const Dimension& sc) {
    int64_t a[4], b[4], c[4];
    shape4(sa, a); shape4(sb, b); shape4(sc, c);
    size_t bytes = 0;
    NZB_CHECK(nzb_tensorcore_gemm_workspace_bytes(a, b, c, &bytes));
    SM::Instance().run({C}, {A, B}, [&](cudaStream_t s) {
        void* ws = SM::Instance().scratch(bytes, s);
        const int rc = backward ? nzb_gemm_backward(A, B, C, a, b, c, ws, bytes, s)
                                : nzb_tensorcore_gemm(A, B, C, a, b, c, ws, bytes, s);
        SM::Instance().releaseScratch(ws, s);
        NZB_CHECK(rc);
    });
}

void iTensorCoreGEMM(float* A, float* B, float* C, const Dimension& sa, const Dimension& sb, const Dimension& sc) {
    gemm4(false, A, B, C, sa, sb, sc);
}
void iGEMMBackward(float* A, float* B, float* C, const Dimension& sa, const Dimension& sb, const Dimension& sc) {
    gemm4(true, A, B, C, sa, sb, sc);
}

void iGeneralMatrixMul(float* A, float* B, float* C, const Dimension& sa, const Dimension& sb, const Dimension& sc) {
    int64_t a[4], b[4], c[4];
    shape4(sa, a); shape4(sb, b); shape4(sc, c);
    size_t bytes = 0;
    NZB_CHECK(nzb_matmul_f32_workspace_bytes(a, b, c, &bytes));
    SM::Instance().run({C}, {A, B}, [&](cudaStream_t s) {
        void* ws = SM::Instance().scratch(bytes, s);
        const int rc = nzb_matmul_f32(A, B, C, a, b, c, ws, bytes, s);
        SM::Instance().releaseScratch(ws, s);
        NZB_CHECK(rc);
    });
}
void tensorGeneralMatrixMul(Tensor& out, const Tensor& lhs, const Tensor& rhs) {
    if (!lhs.shape().isBroadcastCompatible(rhs.shape()) || lhs.shape().W() != rhs.shape().H())
        throw std::invalid_argument("Shapes are not broadcast compatible.");
    iGeneralMatrixMul(lhs.data(), rhs.data(), out.data(), lhs.shape(), rhs.shape(), out.shape());
}

Tensor Tensor::operator*(const Tensor& other) const {
    Tensor result(Dimension(std::max(shape_.N(), other.shape_.N()), std::max(shape_.C(), other.shape_.C()), shape_.H(),
                            other.shape_.W()),
                  requires_grad_ || other.requires_grad_);
    tensorGeneralMatrixMul(result, *this, other);
    return result;
}

void iGemm(const float* A, const float* B, float* C, size_t M, size_t N, size_t K, bool transA, bool transB,
           bool accumulate, const float* bias, int bias_mode, bool relu) {
    nzb_gemm_desc d{};
    d.M = (int64_t)M; d.N = (int64_t)N; d.K = (int64_t)K;
    d.lda = transA ? (int64_t)M : (int64_t)K;
    d.ldb = transB ? (int64_t)K : (int64_t)N;
    d.ldc = (int64_t)N;
    d.transA = transA; d.transB = transB;
    d.batch[0] = d.batch[1] = 1;
    d.accumulate = accumulate; d.relu = relu;
    d.bias_mode = bias ? bias_mode : NZB_BIAS_NONE;
    d.bias_ld = (int64_t)N;
    size_t bytes = 0;
    NZB_CHECK(nzb_gemm_workspace_bytes(&d, &bytes));
    SM::Instance().run({C}, {A, B, bias}, [&](cudaStream_t s) {
        void* ws = SM::Instance().scratch(bytes, s);
        const int rc = nzb_gemm(&d, A, B, C, bias, ws, bytes, s);
        SM::Instance().releaseScratch(ws, s);
        NZB_CHECK(rc);
    });
}

void iImg2col(float* out, float* in, size_t Ho, size_t Wo, size_t C, size_t Kh, size_t Kw, size_t stride, size_t pad,
              size_t H, size_t W, size_t batch) {
    SM::Instance().run({out}, {in}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_img2col(out, in, Ho, Wo, C, Kh, Kw, stride, pad, H, W, batch, s));
    });
}
void iImg2colBackward(float* out, float* in, size_t Ho, size_t Wo, size_t C, size_t Kh, size_t Kw, size_t stride,
                      size_t pad, size_t H, size_t W, size_t batch) {
    SM::Instance().run({out}, {in}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_img2col_backward(out, in, Ho, Wo, C, Kh, Kw, stride, pad, H, W, batch, s));
    });
}
void iCol2img(float* out, float* in, size_t Ho, size_t Wo, size_t Cout, size_t batches) {
    SM::Instance().run({out}, {in}, [&](cudaStream_t s) { NZB_CHECK(nzb_col2img(out, in, Ho, Wo, Cout, batches, s)); });
}
void iCol2imgBackward(float* out, float* in, size_t Ho, size_t Wo, size_t Cout, size_t batches) {
    SM::Instance().run({out}, {in},
                       [&](cudaStream_t s) { NZB_CHECK(nzb_col2img_backward(out, in, Ho, Wo, Cout, batches, s)); });
}
void iMatrixAdd(float* out, float* a, float* b, const Dimension& sa, const Dimension& sb) {
    int64_t x[4], y[4];
    shape4(sa, x); shape4(sb, y);
    SM::Instance().run({out}, {a, b}, [&](cudaStream_t s) { NZB_CHECK(nzb_add_broadcast(out, a, b, x, y, s)); });
}
void iAddBackward(float* gin, float* gout, const Dimension& sin, const Dimension& sout) {
    int64_t x[4], y[4];
    shape4(sin, x); shape4(sout, y);
    SM::Instance().run({gin}, {gout}, [&](cudaStream_t s) { NZB_CHECK(nzb_add_backward(gin, gout, x, y, s)); });
}
void iRELU(float* out, float* in, size_t n) {
    SM::Instance().run({out}, {in}, [&](cudaStream_t s) { NZB_CHECK(nzb_relu(out, in, n, s)); });
}
void iReLUBackward(float* gin, float* x, float* gout, size_t n) {
    SM::Instance().run({gin}, {x, gout}, [&](cudaStream_t s) { NZB_CHECK(nzb_relu_backward(gin, x, gout, n, s)); });
}
void iAveragePooling(float* out, float* in, size_t pool, size_t stride, size_t pad, size_t batches, size_t channels,
                     size_t H, size_t W, size_t Ho, size_t Wo) {
    SM::Instance().run({out}, {in}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_avgpool(out, in, pool, stride, pad, batches, channels, H, W, Ho, Wo, s));
    });
}
void iMaxPooling(float* out, float* position, float* in, size_t pool, size_t stride, size_t pad, size_t batches,
                 size_t channels, size_t H, size_t W, size_t Ho, size_t Wo) {
    SM::Instance().run({out, position}, {in}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_maxpool(out, position, in, pool, stride, pad, batches, channels, H, W, Ho, Wo, s));
    });
}
void iMaxPoolingBackward(float* gin, float* position, float* gout, size_t pool, size_t stride, size_t pad,
                         size_t batches, size_t channels, size_t H, size_t W, size_t Ho, size_t Wo) {
    SM::Instance().run({gin}, {position, gout}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_maxpool_backward(gin, position, gout, pool, stride, pad, batches, channels, H, W, Ho, Wo, s));
    });
}
void iSoftmaxBCE(float* probs, float* loss, float* logits, float* target, size_t batches, size_t n) {
    SM::Instance().run({probs, loss}, {logits, target}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_softmax_bce_forward(probs, loss, logits, target, batches, n, s));
    });
}
void iSoftmaxBCEBackward(float* dlogits, float* probs, float* target, size_t batches, size_t n, bool round_f16) {
    SM::Instance().run({dlogits}, {probs, target}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_softmax_bce_backward(dlogits, probs, target, batches, n, round_f16 ? 1 : 0, s));
    });
}
void iAveragePoolingBackwardOverwrite(float* gin, float* gout, size_t pool, size_t stride, size_t pad, size_t batches,
                                      size_t channels, size_t H, size_t W, size_t Ho, size_t Wo) {
    SM::Instance().run({gin}, {gout}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_avgpool_backward_ex(gin, gout, pool, stride, pad, batches, channels, H, W, Ho, Wo, 1, s));
    });
}
void iAveragePoolingBackward(float* gin, float* gout, size_t pool, size_t stride, size_t pad, size_t batches,
                             size_t channels, size_t H, size_t W, size_t Ho, size_t Wo) {
    SM::Instance().run({gin}, {gout}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_avgpool_backward(gin, gout, pool, stride, pad, batches, channels, H, W, Ho, Wo, s));
    });
}
void iSoftmax(float* out, float* in, size_t batches, size_t n) {
    SM::Instance().run({out}, {in}, [&](cudaStream_t s) { NZB_CHECK(nzb_softmax(out, in, batches, n, s)); });
}
void iSoftmaxBackward(float* gin, float* y, float* gout, size_t batches, size_t n, bool round_f16) {
    SM::Instance().run({gin}, {y, gout}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_softmax_backward(gin, y, gout, batches, n, round_f16 ? 1 : 0, s));
    });
}
void iBCE(float* loss, float* predict, float* target, size_t n) {
    SM::Instance().run({loss}, {predict, target}, [&](cudaStream_t s) { NZB_CHECK(nzb_bce(loss, predict, target, n, s)); });
}
void iBCEBackward(float* out, float* predict, float* target, size_t n) {
    SM::Instance().run({out}, {predict, target},
                       [&](cudaStream_t s) { NZB_CHECK(nzb_bce_backward(out, predict, target, n, s)); });
}
void iExpand(float* out, float* in, size_t per_batch, size_t batches) {
    SM::Instance().run({out}, {in}, [&](cudaStream_t s) { NZB_CHECK(nzb_expand(out, in, per_batch, batches, s)); });
}
void iFill(float* data, float value, size_t n) {
    SM::Instance().run({data}, {}, [&](cudaStream_t s) { NZB_CHECK(nzb_fill(data, value, n, s)); });
}

void GEMMTensorCore(Tensor& out, const Tensor& lhs, const Tensor& rhs) {
    if (!lhs.shape().isBroadcastCompatible(rhs.shape()) || lhs.shape().W() != rhs.shape().H())
        throw std::invalid_argument("Shapes are not broadcast compatible.");
    iTensorCoreGEMM(lhs.data(), rhs.data(), out.data(), lhs.shape(), rhs.shape(), out.shape());
}

Tensor transpose(const Tensor& in) {
    const auto s = in.shape();
    Tensor out(Dimension(s.N(), s.C(), s.W(), s.H()), in.requiresGrad());
    // [H][W] -> [W][H] per matrix: the {P, C} <-> {C, P} permutation kernel with P = H, C = W
    iCol2img(out.data(), in.data(), s.H(), 1, s.W(), s.N() * s.C());
    if (in.requiresGrad()) iCol2img(out.grad(), in.grad(), s.H(), 1, s.W(), s.N() * s.C());
    return out;
}
Tensor tensorImg2col(const Tensor& in, size_t Kh, size_t Kw, size_t stride, size_t pad) {
    const auto s = in.shape();
    const size_t Ho = (s.H() + 2 * pad - Kh) / stride + 1, Wo = (s.W() + 2 * pad - Kw) / stride + 1;
    Tensor out(Dimension(s.N(), 1, Ho * Wo, s.C() * Kh * Kw));
    iImg2col(out.data(), in.data(), Ho, Wo, s.C(), Kh, Kw, stride, pad, s.H(), s.W(), s.N());
    return out;
}
Tensor tensorCol2img(const Tensor& in, size_t Ho, size_t Wo) {
    const auto s = in.shape();
    Tensor out(Dimension(s.N(), s.W(), Ho, Wo));
    iCol2img(out.data(), in.data(), Ho, Wo, s.W(), s.N());
    return out;
}
Tensor tensorAveragePooling(const Tensor& in, size_t pool, size_t stride, size_t pad) {
    const auto s = in.shape();
    const size_t Ho = (s.H() + 2 * pad - pool) / stride + 1, Wo = (s.W() + 2 * pad - pool) / stride + 1;
    Tensor out(Dimension(s.N(), s.C(), Ho, Wo));
    iAveragePooling(out.data(), in.data(), pool, stride, pad, s.N(), s.C(), s.H(), s.W(), Ho, Wo);
    return out;
}
void tensorMatrixAdd(Tensor& out, const Tensor& lhs, const Tensor& rhs) {
    if (!lhs.shape().isBroadcastCompatible(rhs.shape()) || lhs.shape().H() != rhs.shape().H() ||
        lhs.shape().W() != rhs.shape().W())
        throw std::invalid_argument("Shapes are not broadcast compatible.");
    iMatrixAdd(out.data(), lhs.data(), rhs.data(), lhs.shape(), rhs.shape());
}
Tensor ReLU(const Tensor& in) {
    Tensor out(in.shape());
    iRELU(out.data(), in.data(), in.size());
    return out;
}
Tensor Softmax(const Tensor& in) {
    Tensor out(in.shape());
    const auto s = in.shape();
    iSoftmax(out.data(), in.data(), s.N() * s.C(), s.H() * s.W());
    return out;
}

}  // namespace nz::data
