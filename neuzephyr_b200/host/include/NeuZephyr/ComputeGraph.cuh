// nz::graph::ComputeGraph: node container, Kahn topological sort, forward / backward /
// update / zeroGrad loops, save / load (mirrors include/NeuZephyr/ComputeGraph.cuh,
// src/ComputeGraph.cu:258-296, 405-438, 541-547, 553-811).
#pragma once
#include <functional>
#include <memory>
#include <string>
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
    // Marks the gradient buffers that one node alone writes in full -- the output of a non-parameter node
    // that feeds exactly one consumer of type Conv2d / Linear (as their first input) or AveragePooling --
    // as overwritten (Tensor::setGradOverwritten): zeroGrad() then skips them and the consumer's backward
    // stores instead of adding. Same results, one clearing pass and one read of the largest tensors of a
    // model less per step. Model turns it on for fused models; off by default for hand-built graphs.
    void overwriteSingleConsumerGradients(bool on);
    // `n` optimizer ticks that belong to gradient-requiring reference nodes which have no node of
    // their own in this graph (a fused node collapses several); they are placed before the next
    // node that is added, or at the end of the list.
    void addPhantomSteps(int n) { pending_ticks_ += n; }
    float getLoss() const;
    // Checkpoint of the whole graph in the reference's text layout (src/ComputeGraph.cu:553-639): a JSON
    // array with one object per node in topological order -- "type", "name", "pre", "post", "shape",
    // "data", "requires_grad", "grad", one key per line. Three things differ from the reference's files:
    // "shape" holds all four extents (the reference writes the first two and reloads every tensor as
    // {N, C, 1, 1}-sized, :598-600, :752-753), numbers are printed with nine significant digits so that
    // fp32 values survive the round trip, and nodes whose constructors take more than their inputs carry
    // them in "attr". With an optimizer, its per-node state ("opt_state") and a trailing
    // {"type": "Optimizer", ...} object with its per-call counter are written too, so that training
    // resumes with the same Adam moments and time steps.
    void save(const std::string& path, const opt::Optimizer* optimizer = nullptr);
    // Rebuilds a graph from such a file into this (empty) graph: nodes are created by type from their
    // saved inputs and attributes, data and gradients injected, optimizer state restored when both the
    // file and the call provide an optimizer. Files written by the reference itself load as far as they
    // go: their two-extent "shape" is read as {N, C, count / (N*C), 1}. The graph owns the nodes it loads.
    void load(const std::string& path, opt::Optimizer* optimizer = nullptr);
    // node by its saved / generated name ("<type>_<index in topological order>")
    nodes::Node* operator[](const std::string& name) const;
    const std::vector<nodes::Node*>& getNodes() const { return nodes_; }
    const std::vector<nodes::io::OutputNode*>& getOutputs() const { return outputs_; }

private:
    std::vector<nodes::Node*> nodes_, sorted_nodes_;
    std::vector<nodes::io::InputNode*> inputs_;
    std::vector<nodes::io::OutputNode*> outputs_;
    std::vector<std::unique_ptr<nodes::Node>> owned_;  // nodes created by load()
    std::vector<std::string> names_;                  // per entry of sorted_nodes_ after save / load
    std::vector<int> ticks_before_;  // per entry of nodes_: phantom optimizer ticks that precede it
    int pending_ticks_ = 0;
    bool sorted_ = false;
    bool step_intermediates_ = false;
};

}  // namespace nz::graph
