// Optimizers used by the training step (mirrors include/NeuZephyr/Optimizer.cuh,
// src/Optimizer.cu:79-102): SGD and Adam. Adam keeps the reference's quirk of one time step per
// step(Node*) call (the counter is shared by all parameters), eps 1e-6.
#pragma once
#include <memory>
#include <unordered_map>

#include "Nodes.cuh"

namespace nz::opt {

class Optimizer {
public:
    virtual ~Optimizer() = default;
    virtual void step(nodes::Node* input) = 0;
    // `n` step() calls the reference would have made on nodes this graph does not step
    // (activations, nodes folded into a fused node): only per-call state advances.
    virtual void skip(int n) { (void)n; }

protected:
    float learning_rate = 0.f;
};

class SGD : public Optimizer {
public:
    explicit SGD(float learning_rate);
    void step(nodes::Node* input) override;
};

class Adam : public Optimizer {
public:
    Adam(float learning_rate, float beta1, float beta2);
    void step(nodes::Node* input) override;
    void skip(int n) override { it_ += n; }
    // false restores "one time step per optimisation step" semantics: call nextIteration() once
    // per Model::update and every parameter uses the same t
    bool perCallTimeStep = true;
    void nextIteration() { it_shared_++; }

private:
    float beta1_, beta2_, epsilon_ = 1e-6f;
    int it_ = 0, it_shared_ = 0;
    std::unordered_map<nodes::Node*, std::unique_ptr<data::Tensor>> m_, v_;
};

}  // namespace nz::opt
