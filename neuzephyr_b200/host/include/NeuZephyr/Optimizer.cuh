// Optimizers used by the training step (mirrors include/NeuZephyr/Optimizer.cuh,
// src/Optimizer.cu:79-102): SGD and Adam. Adam keeps the reference's quirk of one time step per
// step(Node*) call (the counter is shared by all parameters), eps 1e-6.
#pragma once
#include <memory>
#include <unordered_map>
#include <utility>
#include <vector>

#include "Nodes.cuh"

namespace nz::opt {

class Optimizer {
public:
    virtual ~Optimizer() = default;
    virtual void step(nodes::Node* input) = 0;
    // `n` step() calls the reference would have made on nodes this graph does not step
    // (activations, nodes folded into a fused node): only per-call state advances.
    virtual void skip(int n) { (void)n; }
    // ComputeGraph::update brackets its loop with these: an optimizer may collect the step() calls in
    // between and run them as one launch in endBatch() (Adam does). The default runs each step at once.
    virtual void beginBatch() {}
    virtual void endBatch() {}
    // Restricts the steps of `node` to elements [offset, offset + count) of its tensor (count == 0: the
    // whole tensor again). A data-parallel run with a sharded optimizer gives every rank its own slice.
    void setSlice(nodes::Node* node, size_t offset, size_t count) {
        if (count) slices_[node] = {offset, count};
        else slices_.erase(node);
    }

protected:
    std::pair<size_t, size_t> sliceOf(nodes::Node* node) const {
        auto it = slices_.find(node);
        return it == slices_.end() ? std::pair<size_t, size_t>{0, node->output->size()} : it->second;
    }
    std::unordered_map<nodes::Node*, std::pair<size_t, size_t>> slices_;

public:
    // Checkpointing (ComputeGraph::save / load): a name, the per-call counter, and per node the state
    // vectors the optimizer keeps (empty when it keeps none for that node).
    virtual const char* name() const { return "Optimizer"; }
    virtual long counter() const { return 0; }
    virtual void setCounter(long) {}
    virtual std::vector<std::vector<float>> exportState(nodes::Node*) const { return {}; }
    virtual void importState(nodes::Node*, const std::vector<std::vector<float>>&) {}

protected:
    float learning_rate = 0.f;
};

class SGD : public Optimizer {
public:
    explicit SGD(float learning_rate);
    void step(nodes::Node* input) override;
    const char* name() const override { return "SGD"; }
};

class Adam : public Optimizer {
public:
    Adam(float learning_rate, float beta1, float beta2);
    void step(nodes::Node* input) override;
    void skip(int n) override { it_ += n; }
    void beginBatch() override;
    void endBatch() override;  // one nzb_adam_multi launch over every tensor stepped since beginBatch()
    const char* name() const override { return "Adam"; }
    long counter() const override { return it_; }
    void setCounter(long it) override { it_ = (int)it; }
    // {first moments, second moments} of a node, in host memory
    std::vector<std::vector<float>> exportState(nodes::Node* node) const override;
    void importState(nodes::Node* node, const std::vector<std::vector<float>>& state) override;
    // false restores "one time step per optimisation step" semantics: call nextIteration() once
    // per Model::update and every parameter uses the same t
    bool perCallTimeStep = true;
    void nextIteration() { it_shared_++; }

private:
    float beta1_, beta2_, epsilon_ = 1e-6f;
    int it_ = 0, it_shared_ = 0;
    bool batching_ = false;
    std::vector<std::pair<nodes::Node*, int>> batch_;  // (node, time step) collected between begin / endBatch
    std::unordered_map<nodes::Node*, std::unique_ptr<data::Tensor>> m_, v_;
};

}  // namespace nz::opt
