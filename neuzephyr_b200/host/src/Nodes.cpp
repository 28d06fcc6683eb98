// Node implementations. Gradient write semantics follow the reference node by node:
// overwrite - ReLU, Reshape, Col2Img, Softmax, loss nodes, same-shape Add;
// accumulate - MatMul, Img2Col, AveragePooling, broadcast Add, Expand, and the fused nodes.
#include <NeuZephyr/Nodes.cuh>
#include <NeuZephyr/TensorOperations.cuh>

#include <nzb.h>

namespace nz::nodes {

using data::Dimension;
using SM = cuStrm::StreamManager<float>;

namespace io {
InputNode::InputNode(const Tensor::shape_type& shape, bool requires_grad) {
    output = std::make_shared<Tensor>(shape, requires_grad);
    type = "Input";
}
InputNode::InputNode(const Tensor& tensor) {
    output = std::make_shared<Tensor>(tensor);
    type = "Input";
}

OutputNode::OutputNode(Node* input) {
    inputs.push_back(input);
    output = input->output;
    type = "Output";
    SM::Instance().malloc(&loss_dev_, sizeof(float));
    SM::Instance().memset(loss_dev_, 0, sizeof(float));
}
OutputNode::~OutputNode() {
    try {
        SM::Instance().free(loss_dev_);
    } catch (...) {
    }
}
void OutputNode::forward() {}
void OutputNode::backward() {}
Tensor::value_type OutputNode::getLoss() const {
    float h = 0.f;
    SM::Instance().memcpy(&h, loss_dev_, sizeof(float), cudaMemcpyDeviceToHost);
    return h;
}
void OutputNode::resetLoss() { SM::Instance().memset(loss_dev_, 0, sizeof(float)); }
}  // namespace io

namespace calc {

// ---- Add (src/Nodes.cu:79-146) ----
AddNode::AddNode(Node* l, Node* r) {
    const auto a = l->output->shape(), b = r->output->shape();
    if (!a.isBroadcastCompatible(b) || a.H() != b.H() || a.W() != b.W())
        throw std::invalid_argument("Shapes are not broadcast compatible.");
    inputs = {l, r};
    output = std::make_shared<Tensor>(a.Broadcast(b), l->output->requiresGrad() || r->output->requiresGrad());
    type = "Add";
}
void AddNode::forward() { data::tensorMatrixAdd(*output, *inputs[0]->output, *inputs[1]->output); }
void AddNode::backward() {
    for (Node* in : inputs)
        if (in->output->requiresGrad())
            data::iAddBackward(in->output->grad(), output->grad(), in->output->shape(), output->shape());
}

// ---- MatMul (src/Nodes.cu:148-182) ----
MatMulNode::MatMulNode(Node* l, Node* r) {
    const auto a = l->output->shape(), b = r->output->shape();
    if (!a.isBroadcastCompatible(b) || a.W() != b.H()) throw std::invalid_argument("Shapes are not broadcast compatible.");
    inputs = {l, r};
    output = std::make_shared<Tensor>(Dimension(std::max(a.N(), b.N()), std::max(a.C(), b.C()), a.H(), b.W()),
                                      l->output->requiresGrad() || r->output->requiresGrad());
    type = "MatMul";
}
void MatMulNode::forward() { data::GEMMTensorCore(*output, *inputs[0]->output, *inputs[1]->output); }
void MatMulNode::backward() {
    // The reference materialises transposes and calls iGEMMBackward; here the transposition is
    // folded into the operand staging of the batched kernel (transA / transB).
    const Tensor& A = *inputs[0]->output;
    const Tensor& B = *inputs[1]->output;
    const auto sa = A.shape(), sb = B.shape(), sc = output->shape();
    auto run = [&](bool for_a) {
        nzb_gemm_desc d{};
        // dA[M x K] += dC[M x N] * B^T ;  dB[K x N] += A^T * dC
        d.M = for_a ? sa.H() : sa.W();
        d.N = for_a ? sa.W() : sb.W();
        d.K = for_a ? sb.W() : sa.H();
        d.batch[0] = (int32_t)sc.N();
        d.batch[1] = (int32_t)sc.C();
        const Dimension& sl = for_a ? sc : sa;  // left operand tensor
        const Dimension& sr = for_a ? sb : sc;  // right operand tensor
        const Dimension& so = for_a ? sa : sb;  // gradient receiver
        d.transA = for_a ? 0 : 1;
        d.transB = for_a ? 1 : 0;
        d.lda = sl.W(); d.ldb = sr.W(); d.ldc = so.W();
        for (int k = 0; k < 2; k++) {
            d.strideA[k] = sl[k] > 1 ? (int64_t)sl.getStride(k) : 0;
            d.strideB[k] = sr[k] > 1 ? (int64_t)sr.getStride(k) : 0;
            d.strideC[k] = so[k] > 1 ? (int64_t)so.getStride(k) : 0;
        }
        d.accumulate = 1;
        const float* L = for_a ? output->grad() : A.data();
        const float* R = for_a ? B.data() : output->grad();
        float* O = for_a ? A.grad() : B.grad();
        size_t bytes = 0;
        NZB_CHECK(nzb_gemm_workspace_bytes(&d, &bytes));
        SM::Instance().run({O}, {L, R}, [&](cudaStream_t s) {
            void* ws = SM::Instance().scratch(bytes, s);
            const int rc = nzb_gemm(&d, L, R, O, nullptr, ws, bytes, s);
            SM::Instance().releaseScratch(ws, s);
            NZB_CHECK(rc);
        });
    };
    if (A.requiresGrad()) run(true);
    if (B.requiresGrad()) run(false);
}

// ---- ReLU (src/Nodes.cu:344-364) ----
ReLUNode::ReLUNode(Node* input) {
    inputs = {input};
    output = std::make_shared<Tensor>(input->output->shape(), input->output->requiresGrad());
    type = "ReLU";
}
void ReLUNode::forward() { data::iRELU(output->data(), inputs[0]->output->data(), output->size()); }
void ReLUNode::backward() {
    if (inputs[0]->output->requiresGrad())
        data::iReLUBackward(inputs[0]->output->grad(), inputs[0]->output->data(), output->grad(), output->size());
}

// ---- Reshape (src/Nodes.cu:550-571) ----
ReshapeNode::ReshapeNode(Node* input, const Tensor::shape_type& shape) {
    if (input->output->shape().size() != shape.size())
        throw std::invalid_argument("ReshapeNode: input and new shape must have the same number of elements");
    inputs = {input};
    output = std::make_shared<Tensor>(shape, input->output->requiresGrad());
    type = "Reshape";
}
void ReshapeNode::forward() {
    SM::Instance().memcpy(output->data(), inputs[0]->output->data(), output->size() * sizeof(float),
                          cudaMemcpyDeviceToDevice);
}
void ReshapeNode::backward() {
    if (inputs[0]->output->requiresGrad())
        SM::Instance().memcpy(inputs[0]->output->grad(), output->grad(), output->size() * sizeof(float),
                              cudaMemcpyDeviceToDevice);
}

// ---- Expand (src/Nodes.cu:573-603) ----
ExpandNode::ExpandNode(Node* input, Tensor::size_type newBatch) {
    const auto s = input->output->shape();
    if (s[0] != 1) throw std::invalid_argument("ExpandNode: input must have batch size 1");
    inputs = {input};
    output = std::make_shared<Tensor>(Dimension(newBatch, s[1], s[2], s[3]), input->output->requiresGrad());
    type = "Expand";
}
void ExpandNode::forward() {
    const auto s = inputs[0]->output->shape();
    data::iExpand(output->data(), inputs[0]->output->data(), s[1] * s[2] * s[3], output->shape()[0]);
}
void ExpandNode::backward() {
    if (inputs[0]->output->requiresGrad()) {
        // Compress: the batch copies' gradients are summed into the single input (accumulate)
        const auto so = output->shape();
        data::iAddBackward(inputs[0]->output->grad(), output->grad(), inputs[0]->output->shape(), so);
    }
}

// ---- Img2Col (src/Nodes.cu:605-640) ----
Img2ColNode::Img2ColNode(Node* input, Tensor::size_type kh, Tensor::size_type kw, Tensor::size_type stride,
                         Tensor::size_type pad)
    : kh_(kh), kw_(kw), stride_(stride), pad_(pad) {
    const auto s = input->output->shape();
    ho_ = (s.H() + 2 * pad - kh) / stride + 1;
    wo_ = (s.W() + 2 * pad - kw) / stride + 1;
    inputs = {input};
    output = std::make_shared<Tensor>(Dimension(s.N(), 1, ho_ * wo_, s.C() * kh * kw), input->output->requiresGrad());
    type = "Img2Col";
}
void Img2ColNode::forward() {
    const auto s = inputs[0]->output->shape();
    data::iImg2col(output->data(), inputs[0]->output->data(), ho_, wo_, s.C(), kh_, kw_, stride_, pad_, s.H(), s.W(),
                   s.N());
}
void Img2ColNode::backward() {
    if (inputs[0]->output->requiresGrad()) {
        const auto s = inputs[0]->output->shape();
        data::iImg2colBackward(inputs[0]->output->grad(), output->grad(), ho_, wo_, s.C(), kh_, kw_, stride_, pad_,
                               s.H(), s.W(), s.N());
    }
}

// ---- Col2Img (src/Nodes.cu:642-665) ----
Col2ImgNode::Col2ImgNode(Node* input, Tensor::size_type ho, Tensor::size_type wo) : ho_(ho), wo_(wo) {
    const auto s = input->output->shape();
    if (s.H() != ho * wo) throw std::invalid_argument("Col2ImgNode: rows do not match the output size");
    cout_ = s.W();
    inputs = {input};
    output = std::make_shared<Tensor>(Dimension(s.N(), cout_, ho, wo), input->output->requiresGrad());
    type = "Col2Img";
}
void Col2ImgNode::forward() {
    data::iCol2img(output->data(), inputs[0]->output->data(), ho_, wo_, cout_, output->shape().N());
}
void Col2ImgNode::backward() {
    if (inputs[0]->output->requiresGrad())
        data::iCol2imgBackward(inputs[0]->output->grad(), output->grad(), ho_, wo_, cout_, output->shape().N());
}

// ---- AveragePooling (src/Nodes.cu; kernels src/OperationKernels.cu:1404-1490) ----
AveragePoolingNode::AveragePoolingNode(Node* input, Tensor::size_type pool, Tensor::size_type stride,
                                       Tensor::size_type pad)
    : pool_(pool), stride_(stride), pad_(pad) {
    const auto s = input->output->shape();
    inputs = {input};
    output = std::make_shared<Tensor>(
        Dimension(s.N(), s.C(), (s.H() + 2 * pad - pool) / stride + 1, (s.W() + 2 * pad - pool) / stride + 1),
        input->output->requiresGrad());
    type = "AveragePooling";
}
void AveragePoolingNode::forward() {
    const auto s = inputs[0]->output->shape(), o = output->shape();
    data::iAveragePooling(output->data(), inputs[0]->output->data(), pool_, stride_, pad_, s.N(), s.C(), s.H(),
                          s.W(), o.H(), o.W());
}
void AveragePoolingNode::backward() {
    if (inputs[0]->output->requiresGrad()) {
        const auto s = inputs[0]->output->shape(), o = output->shape();
        if (inputs[0]->output->gradOverwritten())
            data::iAveragePoolingBackwardOverwrite(inputs[0]->output->grad(), output->grad(), pool_, stride_, pad_, s.N(),
                                                   s.C(), s.H(), s.W(), o.H(), o.W());
        else
            data::iAveragePoolingBackward(inputs[0]->output->grad(), output->grad(), pool_, stride_, pad_, s.N(), s.C(),
                                          s.H(), s.W(), o.H(), o.W());
    }
}

// ---- MaxPooling (src/Nodes.cu:716-743) ----
MaxPoolingNode::MaxPoolingNode(Node* input, Tensor::size_type pool, Tensor::size_type stride, Tensor::size_type pad)
    : pool_(pool), stride_(stride), pad_(pad) {
    const auto s = input->output->shape();
    const Dimension o(s.N(), s.C(), (s.H() + 2 * pad - pool) / stride + 1, (s.W() + 2 * pad - pool) / stride + 1);
    inputs = {input};
    output = std::make_shared<Tensor>(o, input->output->requiresGrad());
    position_ = std::make_shared<Tensor>(o, false);
    type = "MaxPooling";
}
void MaxPoolingNode::forward() {
    const auto s = inputs[0]->output->shape(), o = output->shape();
    data::iMaxPooling(output->data(), position_->data(), inputs[0]->output->data(), pool_, stride_, pad_, s.N(), s.C(),
                      s.H(), s.W(), o.H(), o.W());
}
void MaxPoolingNode::backward() {
    if (inputs[0]->output->requiresGrad()) {
        const auto s = inputs[0]->output->shape(), o = output->shape();
        data::iMaxPoolingBackward(inputs[0]->output->grad(), position_->data(), output->grad(), pool_, stride_, pad_,
                                  s.N(), s.C(), s.H(), s.W(), o.H(), o.W());
    }
}

// ---- Softmax over each {H,W} matrix (src/Nodes.cu:524-548) ----
SoftmaxNode::SoftmaxNode(Node* input) {
    inputs = {input};
    output = std::make_shared<Tensor>(input->output->shape(), input->output->requiresGrad());
    type = "Softmax";
}
void SoftmaxNode::forward() {
    if (handledByLoss) return;
    const auto s = output->shape();
    data::iSoftmax(output->data(), inputs[0]->output->data(), s.N() * s.C(), s.H() * s.W());
}
void SoftmaxNode::backward() {
    if (handledByLoss) return;
    if (inputs[0]->output->requiresGrad()) {
        const auto s = output->shape();
        data::iSoftmaxBackward(inputs[0]->output->grad(), output->data(), output->grad(), s.N() * s.C(),
                               s.H() * s.W(), roundLikeReference);
    }
}

// ---- fused Conv2d ----
Conv2dNode::Conv2dNode(Node* x, Node* weight, Node* bias, Tensor::size_type kh, Tensor::size_type kw,
                       Tensor::size_type stride, Tensor::size_type pad, bool relu)
    : kh_(kh), kw_(kw), stride_(stride), pad_(pad), relu_(relu) {
    const auto sx = x->output->shape(), sw = weight->output->shape();
    if (sw.H() != sx.C() * kh * kw || (sw.N() != 1 && sw.N() != sx.N()) || sw.C() != 1)
        throw std::invalid_argument("Conv2dNode: weight must be {1|N, 1, C*Kh*Kw, Cout}");
    const size_t ho = (sx.H() + 2 * pad - kh) / stride + 1, wo = (sx.W() + 2 * pad - kw) / stride + 1;
    if (bias) {
        const auto sb = bias->output->shape();
        if (sb.N() != 1 || sb.C() != 1 || sb.H() != ho * wo || sb.W() != sw.W())
            throw std::invalid_argument("Conv2dNode: bias must be {1, 1, Ho*Wo, Cout}");
    }
    inputs = {x, weight};
    if (bias) inputs.push_back(bias);
    output = std::make_shared<Tensor>(Dimension(sx.N(), sw.W(), ho, wo), true);
    type = "Conv2d";
}
static nzb_conv_desc conv_desc(const Tensor& x, const Tensor& w, size_t kh, size_t kw, size_t stride, size_t pad) {
    nzb_conv_desc d{};
    const auto sx = x.shape(), sw = w.shape();
    d.N = sx.N(); d.C = sx.C(); d.H = sx.H(); d.W = sx.W();
    d.Cout = sw.W(); d.Kh = kh; d.Kw = kw; d.stride = stride; d.pad = pad;
    d.weights_per_sample = sw.N() > 1;
    return d;
}
void Conv2dNode::forward() {
    const Tensor& x = *inputs[0]->output;
    const Tensor& w = *inputs[1]->output;
    const float* b = inputs.size() > 2 ? inputs[2]->output->data() : nullptr;
    nzb_conv_desc d = conv_desc(x, w, kh_, kw_, stride_, pad_);
    d.bias_mode = b ? NZB_BIAS_MATRIX : NZB_BIAS_NONE;
    d.relu = relu_;
    size_t bytes = 0;
    NZB_CHECK(nzb_conv2d_workspace_bytes(&d, &bytes));
    SM::Instance().run({output->data()}, {x.data(), w.data(), b}, [&](cudaStream_t s) {
        void* ws = SM::Instance().scratch(bytes, s);
        const int rc = nzb_conv2d_forward(&d, x.data(), w.data(), b, output->data(), ws, bytes, s);
        SM::Instance().releaseScratch(ws, s);
        NZB_CHECK(rc);
    });
}
void Conv2dNode::backward() {
    const Tensor& x = *inputs[0]->output;
    const Tensor& w = *inputs[1]->output;
    nzb_conv_desc d = conv_desc(x, w, kh_, kw_, stride_, pad_);
    {
        // one library call for the whole layer when the shape allows: dY is read once (ReLU mask,
        // fp16 copies for both tensor-core kernels, bias gradient), nothing is materialised
        nzb_conv_desc f = d;
        const bool want_db = inputs.size() > 2 && inputs[2]->output->requiresGrad();
        f.relu = relu_;
        f.bias_mode = want_db ? NZB_BIAS_MATRIX : NZB_BIAS_NONE;
        f.overwrite_dx = x.gradOverwritten() ? 1 : 0;
        size_t fused_bytes = 0;
        if (nzb_conv2d_backward_workspace_bytes(&f, &fused_bytes) == NZB_OK) {
            float* db = want_db ? inputs[2]->output->grad() : nullptr;
            float* dw = w.requiresGrad() ? w.grad() : nullptr;
            float* dx = x.requiresGrad() ? x.grad() : nullptr;
            const float* y = relu_ ? output->data() : nullptr;
            const float* g = output->grad();
            SM::Instance().run({db, dw, dx}, {x.data(), w.data(), y, g}, [&](cudaStream_t s) {
                void* ws = SM::Instance().scratch(fused_bytes, s);
                const int rc = nzb_conv2d_backward(&f, x.data(), w.data(), y, g, dx, dw, db, ws, fused_bytes, s);
                SM::Instance().releaseScratch(ws, s);
                NZB_CHECK(rc);
            });
            return;
        }
    }
    float* dy = output->grad();
    if (relu_) {
        // dY' = dY * (Y > 0), kept in a private buffer so that output->grad() is left as received
        if (!masked_) masked_ = std::make_unique<Tensor>(output->shape());
        data::iReLUBackward(masked_->data(), output->data(), output->grad(), output->size());
        dy = masked_->data();
    }
    size_t bytes = 0;
    NZB_CHECK(nzb_conv2d_workspace_bytes(&d, &bytes));
    if (inputs.size() > 2 && inputs[2]->output->requiresGrad()) {
        float* db = inputs[2]->output->grad();
        SM::Instance().run({db}, {dy}, [&](cudaStream_t s) { NZB_CHECK(nzb_conv2d_backward_bias(&d, dy, db, s)); });
    }
    if (w.requiresGrad()) {
        float* dw = w.grad();
        SM::Instance().run({dw}, {x.data(), dy}, [&](cudaStream_t s) {
            void* ws = SM::Instance().scratch(bytes, s);
            const int rc = nzb_conv2d_backward_weight(&d, x.data(), dy, dw, ws, bytes, s);
            SM::Instance().releaseScratch(ws, s);
            NZB_CHECK(rc);
        });
    }
    if (x.requiresGrad()) {
        float* dx = x.grad();
        if (stride_ == 1 && kh_ == kw_ && pad_ <= kh_ - 1) {
            d.overwrite_dx = x.gradOverwritten() ? 1 : 0;
            SM::Instance().run({dx}, {dy, w.data()}, [&](cudaStream_t s) {
                void* ws = SM::Instance().scratch(bytes, s);
                const int rc = nzb_conv2d_backward_data(&d, dy, w.data(), dx, ws, bytes, s);
                SM::Instance().releaseScratch(ws, s);
                NZB_CHECK(rc);
            });
        } else {
            // general stride: the reference's composition on library kernels (accumulates: clear first
            // if nothing else did)
            if (x.gradOverwritten()) SM::Instance().memset(dx, 0, x.size() * sizeof(float));
            const auto so = output->shape();
            const size_t K = x.shape().C() * kh_ * kw_, P = so.H() * so.W();
            // dY {N, Cout, Ho, Wo} -> {N, 1, Ho*Wo, Cout}: the channel extent is C(), not the row width
            Tensor dmm(Dimension(so.N(), 1, P, so.C()));
            data::iCol2imgBackward(dmm.data(), dy, so.H(), so.W(), so.C(), so.N());
            Tensor dcol(Dimension(so.N(), 1, P, K));
            dcol.clear();
            Tensor wT = data::transpose(w);
            data::iGEMMBackward(dmm.data(), wT.data(), dcol.data(), dmm.shape(), wT.shape(), dcol.shape());
            data::iImg2colBackward(dx, dcol.data(), so.H(), so.W(), x.shape().C(), kh_, kw_, stride_, pad_,
                                   x.shape().H(), x.shape().W(), so.N());
        }
    }
}

// ---- fused Linear ----
LinearNode::LinearNode(Node* x, Node* weight, Node* bias, bool relu) : relu_(relu) {
    const auto sx = x->output->shape(), sw = weight->output->shape();
    const size_t in = sx.C() * sx.H() * sx.W();
    if (sw.N() != 1 || sw.C() != 1 || sw.W() != in) throw std::invalid_argument("LinearNode: weight must be {1,1,out,in}");
    if (bias) {
        const auto sb = bias->output->shape();
        if (sb.size() != sw.H()) throw std::invalid_argument("LinearNode: bias must hold one value per output");
    }
    inputs = {x, weight};
    if (bias) inputs.push_back(bias);
    output = std::make_shared<Tensor>(Dimension(sx.N(), 1, sw.H(), 1), true);
    type = "Linear";
}
void LinearNode::forward() {
    const Tensor& x = *inputs[0]->output;
    const Tensor& w = *inputs[1]->output;
    const float* b = inputs.size() > 2 ? inputs[2]->output->data() : nullptr;
    nzb_linear_desc d{};
    d.batch = x.shape().N(); d.in_features = w.shape().W(); d.out_features = w.shape().H(); d.relu = relu_;
    size_t bytes = 0;
    NZB_CHECK(nzb_linear_workspace_bytes(&d, &bytes));
    SM::Instance().run({output->data()}, {x.data(), w.data(), b}, [&](cudaStream_t s) {
        void* ws = SM::Instance().scratch(bytes, s);
        const int rc = nzb_linear_forward(&d, x.data(), w.data(), b, output->data(), ws, bytes, s);
        SM::Instance().releaseScratch(ws, s);
        NZB_CHECK(rc);
    });
}
void LinearNode::backward() {
    const Tensor& x = *inputs[0]->output;
    const Tensor& w = *inputs[1]->output;
    nzb_linear_desc d{};
    d.batch = x.shape().N(); d.in_features = w.shape().W(); d.out_features = w.shape().H(); d.relu = relu_;
    d.overwrite_dx = x.gradOverwritten() ? 1 : 0;
    float* dx = x.requiresGrad() ? x.grad() : nullptr;
    float* dw = w.requiresGrad() ? w.grad() : nullptr;
    float* db = (inputs.size() > 2 && inputs[2]->output->requiresGrad()) ? inputs[2]->output->grad() : nullptr;
    size_t bytes = 0;
    NZB_CHECK(nzb_linear_workspace_bytes(&d, &bytes));
    SM::Instance().run({dx, dw, db}, {x.data(), w.data(), output->data(), output->grad()}, [&](cudaStream_t s) {
        void* ws = SM::Instance().scratch(bytes, s);
        const int rc = nzb_linear_backward(&d, x.data(), w.data(), output->data(), output->grad(), dx, dw, db, ws,
                                           bytes, s);
        SM::Instance().releaseScratch(ws, s);
        NZB_CHECK(rc);
    });
}

}  // namespace calc

namespace loss {
// mean binary cross-entropy over all elements (src/Nodes.cu:813-849)
BinaryCrossEntropyNode::BinaryCrossEntropyNode(Node* input1, Node* input2) : io::OutputNode(input1) {
    if (input1->output->shape() != input2->output->shape()) throw std::invalid_argument("input1 and input2 should have the same shape");
    inputs.push_back(input2);
    type = "BinaryCrossEntropy";
}
void BinaryCrossEntropyNode::fuseWithSoftmax(bool on) {
    auto* sm = dynamic_cast<calc::SoftmaxNode*>(inputs[0]);
    if (softmax_) softmax_->handledByLoss = false;
    softmax_ = nullptr;
    // the one-kernel head handles vectors of up to 1024 elements
    if (on && sm && sm->output->shape().H() * sm->output->shape().W() <= 1024) {
        softmax_ = sm;
        sm->handledByLoss = true;
    }
}
void BinaryCrossEntropyNode::forward() {
    if (softmax_) {
        const auto s = softmax_->output->shape();
        data::iSoftmaxBCE(softmax_->output->data(), loss_dev_, softmax_->inputs[0]->output->data(),
                          inputs[1]->output->data(), s.N() * s.C(), s.H() * s.W());
        return;
    }
    data::iBCE(loss_dev_, inputs[0]->output->data(), inputs[1]->output->data(), output->size());
}
void BinaryCrossEntropyNode::backward() {
    if (softmax_) {
        Node* logits = softmax_->inputs[0];
        if (logits->output->requiresGrad()) {
            const auto s = softmax_->output->shape();
            data::iSoftmaxBCEBackward(logits->output->grad(), softmax_->output->data(), inputs[1]->output->data(),
                                      s.N() * s.C(), s.H() * s.W(), softmax_->roundLikeReference);
        }
        return;
    }
    if (output->requiresGrad())
        data::iBCEBackward(output->grad(), inputs[0]->output->data(), inputs[1]->output->data(), output->size());
}
}  // namespace loss

}  // namespace nz::nodes
