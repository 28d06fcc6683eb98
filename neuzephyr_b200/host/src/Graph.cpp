// ComputeGraph, optimizers and Model of the host layer.
#include <NeuZephyr/ComputeGraph.cuh>
#include <NeuZephyr/Model.cuh>
#include <NeuZephyr/Optimizer.cuh>
#include <NeuZephyr/TensorOperations.cuh>

#include <algorithm>
#include <cmath>
#include <queue>
#include <unordered_map>

#include <nzb.h>

namespace nz::graph {

using nodes::Node;

bool ComputeGraph::inGraph(Node* node) const { return std::find(nodes_.begin(), nodes_.end(), node) != nodes_.end(); }
void ComputeGraph::addNode(Node* node) {
    if (inGraph(node)) return;
    nodes_.push_back(node);
    ticks_before_.push_back(pending_ticks_);
    pending_ticks_ = 0;
    sorted_ = false;
}
void ComputeGraph::addInput(nodes::io::InputNode* node) {
    inputs_.push_back(node);
    addNode(node);
}
void ComputeGraph::addOutput(nodes::io::OutputNode* node) {
    outputs_.push_back(node);
    addNode(node);
}
// Kahn's algorithm over the inputs relation (src/ComputeGraph.cu:258-296)
void ComputeGraph::topologicalSort() {
    std::unordered_map<Node*, int> indeg;
    std::unordered_map<Node*, std::vector<Node*>> users;
    for (Node* n : nodes_) indeg[n] = 0;
    for (Node* n : nodes_)
        for (Node* in : n->inputs) {
            if (!indeg.count(in)) throw std::runtime_error("a node's input is not part of the graph");
            indeg[n]++;
            users[in].push_back(n);
        }
    std::queue<Node*> q;
    for (Node* n : nodes_)
        if (indeg[n] == 0) q.push(n);
    sorted_nodes_.clear();
    while (!q.empty()) {
        Node* n = q.front();
        q.pop();
        sorted_nodes_.push_back(n);
        for (Node* u : users[n])
            if (--indeg[u] == 0) q.push(u);
    }
    if (sorted_nodes_.size() != nodes_.size()) throw std::runtime_error("Graph has cycle");
    sorted_ = true;
}
void ComputeGraph::forward() {
    if (!sorted_) topologicalSort();
    for (Node* n : sorted_nodes_) n->forward();
}
void ComputeGraph::backward(const std::function<void(Node*)>& after_node) {
    if (!sorted_) topologicalSort();
    for (auto it = sorted_nodes_.rbegin(); it != sorted_nodes_.rend(); ++it) {
        (*it)->backward();
        if (after_node) after_node(*it);
    }
}
void ComputeGraph::zeroGrad() const {
    for (Node* n : nodes_) n->output->zeroGrad();
}
void ComputeGraph::update(opt::Optimizer* optimizer, const std::function<void()>& before_step) const {
    if (before_step) before_step();
    for (size_t i = 0; i < nodes_.size(); i++) {
        Node* n = nodes_[i];
        if (ticks_before_[i]) optimizer->skip(ticks_before_[i]);
        if (!n->output->requiresGrad()) continue;
        if (step_intermediates_ || n->inputs.empty()) optimizer->step(n);
        else optimizer->skip(1);  // the reference steps this activation (src/ComputeGraph.cu:541-547)
    }
    if (pending_ticks_) optimizer->skip(pending_ticks_);
}
float ComputeGraph::getLoss() const {
    if (outputs_.empty()) throw std::runtime_error("No output node");
    return outputs_[0]->getLoss();
}

}  // namespace nz::graph

namespace nz::opt {

using SM = cuStrm::StreamManager<float>;

SGD::SGD(float lr) { learning_rate = lr; }
void SGD::step(nodes::Node* input) {
    // data -= lr * grad: scale a copy of the gradient by -lr and add it in place
    data::Tensor& t = *input->output;
    const float lr = learning_rate;
    data::Tensor tmp(t.shape());
    SM::Instance().memcpy(tmp.data(), t.grad(), t.size() * sizeof(float), cudaMemcpyDeviceToDevice);
    SM::Instance().run({tmp.data()}, {}, [&](cudaStream_t s) { NZB_CHECK(nzb_scale(tmp.data(), -lr, t.size(), s)); });
    data::iMatrixAdd(t.data(), t.data(), tmp.data(), t.shape(), t.shape());
}

Adam::Adam(float lr, float beta1, float beta2) : beta1_(beta1), beta2_(beta2) { learning_rate = lr; }
void Adam::step(nodes::Node* input) {
    data::Tensor& t = *input->output;
    auto& m = m_[input];
    auto& v = v_[input];
    if (!m) {
        m = std::make_unique<data::Tensor>(t.shape());
        v = std::make_unique<data::Tensor>(t.shape());
        m->clear();
        v->clear();
    }
    it_++;  // one time step per call, shared by all parameters (src/Optimizer.cu:86-102)
    const int tstep = perCallTimeStep ? it_ : (it_shared_ > 0 ? it_shared_ : 1);
    SM::Instance().run({t.data(), m->data(), v->data()}, {t.grad()}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_adam(t.data(), m->data(), v->data(), t.grad(), learning_rate, beta1_, beta2_, epsilon_, tstep,
                           (int64_t)t.size(), s));
    });
}

}  // namespace nz::opt

namespace nz {

using data::Dimension;
using data::Tensor;
namespace calc = nodes::calc;
namespace io = nodes::io;

Model::~Model() {
    cuStrm::StreamManager<float>::Instance().sync();
    for (Node* n : hiddenNodes) delete n;
}
Model::Node* Model::own(Node* n, bool parameter) {
    hiddenNodes.push_back(n);
    computeGraph.addNode(n);
    if (parameter) params_.push_back(n);
    return n;
}
Tensor& Model::forward() {
    computeGraph.forward();
    return *computeGraph.getOutputs().at(0)->output;
}
void Model::backward() {
    grads_synced_ = false;
    param_synced_.assign(params_.size(), false);
    if (!(comm_ && comm_->world() > 1 && overlap_sync_)) {
        computeGraph.backward();
        return;
    }
    // Data parallel: a parameter's gradient is complete once every node that reads the
    // parameter has run its backward. Its all-reduce is queued on the communication stream at
    // that point (ordered after the gradient's writers by the stream manager), so it runs
    // under the rest of the backward pass. Every rank walks the same graph in the same order,
    // so the collectives are issued in the same order everywhere.
    std::vector<int> remaining(params_.size(), 0);
    for (Node* n : computeGraph.getNodes())
        for (Node* in : n->inputs)
            for (size_t i = 0; i < params_.size(); i++)
                if (params_[i] == in) remaining[i]++;
    computeGraph.backward([&](Node* n) {
        for (Node* in : n->inputs)
            for (size_t i = 0; i < params_.size(); i++)
                if (params_[i] == in && --remaining[i] == 0) {
                    comm_->allReduceAverage(in->output->grad(), in->output->size());
                    param_synced_[i] = true;
                }
    });
}
void Model::syncGradients() {
    if (comm_ && comm_->world() > 1 && !grads_synced_)
        for (size_t i = 0; i < params_.size(); i++)
            if (i >= param_synced_.size() || !param_synced_[i])
                comm_->allReduceAverage(params_[i]->output->grad(), params_[i]->output->size());
    grads_synced_ = true;
    param_synced_.assign(params_.size(), true);
}
void Model::update(opt::Optimizer* optimizer) {
    computeGraph.update(optimizer, [this]() { syncGradients(); });
    computeGraph.zeroGrad();
    grads_synced_ = false;
}
Tensor::value_type Model::getLoss() const { return computeGraph.getLoss(); }

Model::Node* Model::Add(Node* lhs, Node* rhs) {
    computeGraph.addNode(lhs);
    computeGraph.addNode(rhs);
    return own(new calc::AddNode(lhs, rhs));
}
Model::Node* Model::Mul(Node* lhs, Node* rhs) {
    computeGraph.addNode(lhs);
    computeGraph.addNode(rhs);
    return own(new calc::MatMulNode(lhs, rhs));
}
Model::Node* Model::Bias(Node* input) {
    const auto s = input->output->shape();
    auto* param = new io::InputNode(Dimension(1, s[1], s[2], s[3]), true);
    param->output->randomize();
    own(param, true);
    return Add(input, param);
}
Model::Node* Model::Reshape(Node* input, const Tensor::shape_type& shape) {
    computeGraph.addNode(input);
    return own(new calc::ReshapeNode(input, shape));
}
Model::Node* Model::Linear(Node* input, size_t outSize) {
    computeGraph.addNode(input);
    const auto s = input->output->shape();
    const size_t inSize = s[1] * s[2] * s[3];
    // node order of the reference (src/Model.cu:87-103): [Reshape], weight, MatMul, bias, Add
    if (fused_) {
        if (s[2] != inSize && input->output->requiresGrad()) computeGraph.addPhantomSteps(1);  // Reshape
        auto* w = new io::InputNode(Dimension(1, 1, outSize, inSize), true);
        w->output->randomize();
        own(w, true);
        computeGraph.addPhantomSteps(1);  // MatMul
        auto* b = new io::InputNode(Dimension(1, 1, outSize, 1), true);
        b->output->randomize();
        own(b, true);
        return own(new calc::LinearNode(input, w, b, false));  // stands for Add
    }
    Node* shaped = s[2] != inSize ? Reshape(input, Dimension(s[0], 1, inSize, 1)) : input;
    auto* w = new io::InputNode(Dimension(1, 1, outSize, inSize), true);
    w->output->randomize();
    own(w, true);
    return Bias(Mul(w, shaped));
}
Model::Node* Model::ReLU(Node* input) {
    computeGraph.addNode(input);
    return own(new calc::ReLUNode(input));
}
Model::Node* Model::Softmax(Node* input) {
    computeGraph.addNode(input);
    const auto s = input->output->shape();
    const size_t size = s[1] * s[2] * s[3];
    Node* shaped = s[2] != size ? Reshape(input, Dimension(s[0], 1, size, 1)) : input;
    return own(new calc::SoftmaxNode(shaped));
}
Model::Node* Model::TargetExpand(Node* input, const Tensor::shape_type& shape) {
    computeGraph.addNode(input);
    const auto s = input->output->shape();
    if (s == shape) return input;
    if (s[0] != 1 || s[1] != shape[1] || s[2] != shape[2] || s[3] != shape[3])
        throw std::runtime_error("The input data cannot be expanded.");
    return own(new calc::ExpandNode(input, shape.N()));
}
Model::Node* Model::Img2Col(Node* input, size_t kh, size_t kw, size_t stride, size_t pad) {
    computeGraph.addNode(input);
    return own(new calc::Img2ColNode(input, kh, kw, stride, pad));
}
Model::Node* Model::Col2Img(Node* input, size_t ho, size_t wo) {
    computeGraph.addNode(input);
    return own(new calc::Col2ImgNode(input, ho, wo));
}
Model::Node* Model::Conv2d(Node* input, size_t outChannels, size_t kh, size_t kw, size_t stride, size_t pad, bool bias,
                           bool perSampleWeights, bool fuseRelu) {
    computeGraph.addNode(input);
    const auto s = input->output->shape();
    const size_t ho = (s.H() + 2 * pad - kh) / stride + 1, wo = (s.W() + 2 * pad - kw) / stride + 1;
    auto* w = new io::InputNode(Dimension(perSampleWeights ? s.N() : 1, 1, s.C() * kh * kw, outChannels), true);
    w->output->randomize();
    own(w, true);
    if (fused_) {
        // The fused node stands for Img2Col, MatMul, [Add], Col2Img, [ReLU] (src/Model.cu:244-263):
        // every one of them that requires a gradient is one optimizer tick in the reference, placed
        // where that node sits relative to the parameters. The fused node itself is the last of them.
        int before_bias = (input->output->requiresGrad() ? 1 : 0) + 1;  // Img2Col (if x needs a gradient), MatMul
        int after_bias = (bias ? 1 : 0) + 1 + (fuseRelu ? 1 : 0);       // Add, Col2Img, ReLU
        Node* b = nullptr;
        if (bias) {
            computeGraph.addPhantomSteps(before_bias);
            auto* bn = new io::InputNode(Dimension(1, 1, ho * wo, outChannels), true);
            bn->output->randomize();
            b = own(bn, true);
            computeGraph.addPhantomSteps(after_bias - 1);
        } else {
            computeGraph.addPhantomSteps(before_bias + after_bias - 1);
        }
        return own(new calc::Conv2dNode(input, w, b, kh, kw, stride, pad, fuseRelu));
    }
    Node* col = Img2Col(input, kh, kw, stride, pad);
    Node* res = Mul(col, w);
    if (bias) res = Bias(res);
    res = Col2Img(res, ho, wo);
    return fuseRelu ? ReLU(res) : res;
}
Model::Node* Model::AvgPool2d(Node* input, size_t pool, size_t stride, size_t pad) {
    computeGraph.addNode(input);
    return own(new calc::AveragePoolingNode(input, pool, stride, pad));
}
void Model::BCELoss(Node* input, Node* target) {
    computeGraph.addNode(input);
    Node* expanded = TargetExpand(target, input->output->shape());
    auto* bce = new nodes::loss::BinaryCrossEntropyNode(input, expanded);
    hiddenNodes.push_back(bce);
    computeGraph.addOutput(bce);
}

}  // namespace nz
