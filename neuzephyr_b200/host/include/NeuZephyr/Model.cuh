// nz::Model: base class users derive from; builds the compute graph through protected layer
// builders and exposes forward / backward / update / getLoss (mirrors
// include/NeuZephyr/Model.cuh:265-1146, src/Model.cu). With fused == true (default) Linear and
// Conv2d create one fused node each; with fused == false they create exactly the node chains the
// reference creates (Reshape -> MatMul -> Bias, Img2Col -> MatMul -> Bias -> Col2Img).
#pragma once
#include <memory>
#include <vector>

#include "ComputeGraph.cuh"
#include "DataParallel.cuh"

namespace nz {

class Model {
public:
    Model() = default;
    virtual ~Model();
    data::Tensor& forward();
    void backward();
    // optimizer step on every node that requires a gradient, then zeroGrad. With a
    // data-parallel communicator attached, parameter gradients are averaged over ranks first.
    void update(opt::Optimizer* optimizer);
    // averages the parameter gradients over the ranks of the attached communicator (no-op without
    // one); update() calls it, it is public so that gradients can be inspected after the exchange
    void syncGradients();
    data::Tensor::value_type getLoss() const;

    void setFused(bool fused) { fused_ = fused; }
    void setCommunicator(dist::Communicator* comm) { comm_ = comm; }
    // all-reduce each parameter gradient as soon as its last consumer's backward has been queued
    // (default), or all of them in update() / syncGradients()
    void setOverlapGradientSync(bool on) { overlap_sync_ = on; }
    // Sharded optimizer step for data-parallel runs: each rank receives only its slice of every
    // averaged gradient (reduce-scatter instead of all-reduce), updates that slice of the weights and
    // of the optimizer's state, and the updated slices are gathered on all ranks (all-gather) under the
    // next forward pass. Same bytes on the wire as the all-reduce, but the optimizer's pass over the
    // parameters shrinks with the number of ranks instead of being repeated on every one. Parameters
    // whose size is not a multiple of the world size keep the all-reduce. Results are those of the
    // unsharded step.
    void setShardedOptimizer(bool on) { shard_optimizer_ = on; }
    // after syncGradients(): makes every rank hold the complete averaged gradients also when the
    // optimizer is sharded (for inspection; update() does not need it)
    void gatherGradients();
    // parameter nodes (weights / biases created by the builders), in creation order
    const std::vector<nodes::Node*>& parameters() const { return params_; }
    graph::ComputeGraph& graph() { return computeGraph; }

protected:
    using Node = nodes::Node;
    graph::ComputeGraph computeGraph;
    std::vector<Node*> hiddenNodes;

    Node* Add(Node* lhs, Node* rhs);
    Node* Mul(Node* lhs, Node* rhs);
    Node* Bias(Node* input);
    Node* Reshape(Node* input, const data::Tensor::shape_type& shape);
    Node* Linear(Node* input, size_t outSize);
    Node* ReLU(Node* input);
    Node* Softmax(Node* input);
    Node* TargetExpand(Node* input, const data::Tensor::shape_type& shape);
    Node* Img2Col(Node* input, size_t kernelHeight, size_t kernelWidth, size_t stride, size_t padding);
    Node* Col2Img(Node* input, size_t outputHeight, size_t outputWidth);
    // perSampleWeights == true reproduces the reference's allocation of one weight matrix per
    // batch sample (src/Model.cu:249-253); false shares one {1,1,C*Kh*Kw,Cout} matrix.
    Node* Conv2d(Node* input, size_t outChannels, size_t kernelHeight, size_t kernelWidth, size_t stride,
                 size_t padding, bool bias = true, bool perSampleWeights = false, bool fuseRelu = false);
    Node* AvgPool2d(Node* input, size_t poolSize, size_t stride, size_t padding = 0);
    Node* MaxPool2d(Node* input, size_t poolSize, size_t stride, size_t padding = 0);
    void BCELoss(Node* input, Node* target);

private:
    Node* own(Node* n, bool parameter = false);
    bool sharded(size_t param_index) const;
    void exchangeGradient(size_t param_index);
    bool shard_optimizer_ = false;
    bool fused_ = true;
    bool gradients_marked_ = false;
    bool grads_synced_ = false;
    bool overlap_sync_ = true;
    std::vector<bool> param_synced_;
    dist::Communicator* comm_ = nullptr;
    std::vector<Node*> params_;
};

}  // namespace nz
