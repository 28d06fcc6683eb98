// nz::graph::ComputeGraph: node container, Kahn topological sort, forward / backward /
// update / zeroGrad loops (mirrors include/NeuZephyr/ComputeGraph.cuh,
// src/ComputeGraph.cu:258-296, 405-438, 541-547). Serialisation is not part of this path.
#pragma once
#include <functional>
#include <vector>

#include "Nodes.cuh"
#include "Optimizer.cuh"

namespace nz::graph {

class ComputeGraph {
public:
    ComputeGraph() = default;
    bool inGraph(nodes::Node* node) const;
    void addNode(nodes::Node* node);
    void addInput(nodes::io::InputNode* node);
    void addOutput(nodes::io::OutputNode* node);
    void topologicalSort();
    bool isSorted() const { return sorted_; }
    void forward();
    // `after_node`, when given, runs after each node's backward (in reverse topological order)
    void backward(const std::function<void(nodes::Node*)>& after_node = nullptr);
    void zeroGrad() const;
    // Optimizer step, in insertion order, on the nodes whose output requires a gradient
    // (src/ComputeGraph.cu:541-547); gradients are left as they are (Model::update zeroes them,
    // src/Model.cu:20-23). `before_step` runs once after backward and before the first optimizer
    // step (the data-parallel all-reduce hooks in here).
    // The reference also steps every intermediate node (activations), whose values the next
    // forward() overwrites: that is several full passes over the largest tensors of the model
    // for no effect on training, so it is off by default. stepIntermediateNodes(true) restores
    // it for code that reads a hidden node's output between update() and the next forward().
    // Either way every gradient-requiring node the reference would step advances the optimizer's
    // per-call counter (Optimizer::skip), so Adam's bias-correction exponent t of each parameter
    // is the reference's: nodes that are skipped here count one tick each, and a fused node
    // declares the reference nodes it stands for with addPhantomSteps().
    void update(opt::Optimizer* optimizer, const std::function<void()>& before_step = nullptr) const;
    void stepIntermediateNodes(bool on) { step_intermediates_ = on; }
    // `n` optimizer ticks that belong to gradient-requiring reference nodes which have no node of
    // their own in this graph (a fused node collapses several); they are placed before the next
    // node that is added, or at the end of the list.
    void addPhantomSteps(int n) { pending_ticks_ += n; }
    float getLoss() const;
    const std::vector<nodes::Node*>& getNodes() const { return nodes_; }
    const std::vector<nodes::io::OutputNode*>& getOutputs() const { return outputs_; }

private:
    std::vector<nodes::Node*> nodes_, sorted_nodes_;
    std::vector<nodes::io::InputNode*> inputs_;
    std::vector<nodes::io::OutputNode*> outputs_;
    std::vector<int> ticks_before_;  // per entry of nodes_: phantom optimizer ticks that precede it
    int pending_ticks_ = 0;
    bool sorted_ = false;
    bool step_intermediates_ = false;
};

}  // namespace nz::graph
