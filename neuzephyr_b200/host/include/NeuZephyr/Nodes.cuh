// Autograd nodes on the contraction path (mirrors include/NeuZephyr/Nodes.cuh, src/Nodes.cu):
// io::InputNode; calc::{Add, MatMul, ReLU, Reshape, Expand, Img2Col, Col2Img, AveragePooling,
// Softmax}Node; loss::BinaryCrossEntropyNode; plus two fused nodes without a counterpart in the
// reference, calc::Conv2dNode and calc::LinearNode, that collapse the compositions Model::Conv2d
// and Model::Linear build. Gradient write semantics (overwrite vs accumulate) follow the
// reference node by node.
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "Tensor.cuh"

namespace nz::nodes {

using data::Tensor;

class Node {
public:
    std::vector<Node*> inputs;
    std::shared_ptr<Tensor> output;
    std::string type;
    virtual ~Node() = default;
    virtual void forward() = 0;
    virtual void backward() = 0;
    // constructor arguments beyond the input nodes (kernel sizes, strides, flags ...), in constructor
    // order: what ComputeGraph::save writes so that ComputeGraph::load can rebuild the node
    virtual std::vector<size_t> attributes() const { return {}; }
    void dataInject(Tensor::value_type* data, bool grad = false) const { output->dataInject(data, grad); }
    template <typename It>
    void dataInject(It begin, It end, bool grad = false) const { output->dataInject(begin, end, grad); }
    void dataInject(const std::initializer_list<Tensor::value_type>& data, bool grad = false) const {
        output->dataInject(data, grad);
    }
};

namespace io {
class InputNode : public Node {
public:
    explicit InputNode(const Tensor::shape_type& shape, bool requires_grad = false);
    explicit InputNode(const Tensor& tensor);
    void forward() override {}
    void backward() override {}
};

// Base of loss nodes: accumulates a scalar loss on the device (the reference's loss nodes do
// "loss +=" and never reset, src/Nodes.cu:785-802; resetLoss() is provided here).
class OutputNode : public Node {
public:
    explicit OutputNode(Node* input);
    ~OutputNode() override;
    void forward() override;
    void backward() override;
    Tensor::value_type getLoss() const;  // synchronises the loss value to the host
    void resetLoss();

protected:
    float* loss_dev_ = nullptr;
};
}  // namespace io

namespace calc {
class AddNode : public Node {
public:
    AddNode(Node* input_left, Node* input_right);
    void forward() override;
    void backward() override;
};

class MatMulNode : public Node {
public:
    MatMulNode(Node* input_left, Node* input_right);
    void forward() override;
    void backward() override;
};

class ReLUNode : public Node {
public:
    explicit ReLUNode(Node* input);
    void forward() override;
    void backward() override;
};

class ReshapeNode : public Node {
public:
    ReshapeNode(Node* input, const Tensor::shape_type& shape);
    void forward() override;
    void backward() override;
    std::vector<size_t> attributes() const override {
        const auto s = output->shape();
        return {s[0], s[1], s[2], s[3]};
    }
};

class ExpandNode : public Node {
public:
    ExpandNode(Node* input, Tensor::size_type newBatch);
    void forward() override;
    void backward() override;
    std::vector<size_t> attributes() const override { return {output->shape().N()}; }
};

class Img2ColNode : public Node {
public:
    Img2ColNode(Node* input, Tensor::size_type kernelHeight, Tensor::size_type kernelWidth,
                Tensor::size_type stride, Tensor::size_type padding);
    void forward() override;
    void backward() override;
    std::vector<size_t> attributes() const override { return {kh_, kw_, stride_, pad_}; }

private:
    Tensor::size_type kh_, kw_, stride_, pad_, ho_, wo_;
};

class Col2ImgNode : public Node {
public:
    Col2ImgNode(Node* input, Tensor::size_type outputHeight, Tensor::size_type outputWidth);
    void forward() override;
    void backward() override;
    std::vector<size_t> attributes() const override { return {ho_, wo_}; }

private:
    Tensor::size_type ho_, wo_, cout_;
};

class AveragePoolingNode : public Node {
public:
    AveragePoolingNode(Node* input, Tensor::size_type poolSize, Tensor::size_type stride,
                       Tensor::size_type padding);
    void forward() override;
    void backward() override;
    std::vector<size_t> attributes() const override { return {pool_, stride_, pad_}; }

private:
    Tensor::size_type pool_, stride_, pad_;
};

// MaxPoolingNode (src/Nodes.cu:716-743; kernels src/OperationKernels.cu:1507-1573)
class MaxPoolingNode : public Node {
public:
    MaxPoolingNode(Node* input, Tensor::size_type poolSize, Tensor::size_type stride, Tensor::size_type padding);
    void forward() override;
    void backward() override;
    std::vector<size_t> attributes() const override { return {pool_, stride_, pad_}; }

private:
    Tensor::size_type pool_, stride_, pad_;
    std::shared_ptr<Tensor> position_;  // arg-max index of every window, as a float
};

class SoftmaxNode : public Node {
public:
    explicit SoftmaxNode(Node* input);
    void forward() override;
    void backward() override;
    // set by a loss node that computes softmax + loss (and their backward) in one kernel: this node's own
    // forward / backward then do nothing (its output is still the probabilities, written by the loss node)
    bool handledByLoss = false;
    // true (default): round the Jacobian and the upstream gradient to fp16 like the reference's
    // tensor-core product in SoftmaxNode::backward (src/Nodes.cu:538-548)
    bool roundLikeReference = true;
};

// Fused Img2Col -> MatMul -> Bias -> [ReLU] -> Col2Img (Model::Conv2d, src/Model.cu:244-263).
// inputs: {x, weight {wN,1,C*Kh*Kw,Cout}, [bias {1,1,Ho*Wo,Cout}]}
class Conv2dNode : public Node {
public:
    Conv2dNode(Node* x, Node* weight, Node* bias, Tensor::size_type kernelHeight, Tensor::size_type kernelWidth,
               Tensor::size_type stride, Tensor::size_type padding, bool relu);
    void forward() override;
    void backward() override;
    std::vector<size_t> attributes() const override { return {kh_, kw_, stride_, pad_, relu_ ? 1u : 0u}; }

private:
    Tensor::size_type kh_, kw_, stride_, pad_;
    bool relu_;
    std::unique_ptr<Tensor> masked_;  // dY * (Y > 0) when ReLU is fused
};

// Fused Reshape -> MatMul(W, x) -> Bias -> [ReLU] (Model::Linear, src/Model.cu:87-103).
// inputs: {x {N,*,*,*} with C*H*W = in, weight {1,1,out,in}, [bias {1,1,out,1}]}; output {N,1,out,1}
class LinearNode : public Node {
public:
    LinearNode(Node* x, Node* weight, Node* bias, bool relu);
    void forward() override;
    void backward() override;
    std::vector<size_t> attributes() const override { return {relu_ ? 1u : 0u}; }

private:
    bool relu_;
};
}  // namespace calc

namespace loss {
class BinaryCrossEntropyNode : public io::OutputNode {
public:
    BinaryCrossEntropyNode(Node* input1, Node* input2);  // prediction, target
    void forward() override;
    void backward() override;
    // When the prediction comes from a SoftmaxNode, compute softmax + loss in one kernel and their two
    // backward steps in another (Model::BCELoss turns this on for fused models). Results are those of the
    // two nodes run one after the other.
    void fuseWithSoftmax(bool on);

private:
    calc::SoftmaxNode* softmax_ = nullptr;
};
}  // namespace loss

}  // namespace nz::nodes
