// ComputeGraph, optimizers and Model of the host layer.
#include <NeuZephyr/ComputeGraph.cuh>
#include <NeuZephyr/Model.cuh>
#include <NeuZephyr/Optimizer.cuh>
#include <NeuZephyr/TensorOperations.cuh>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <queue>
#include <string>
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
void ComputeGraph::overwriteSingleConsumerGradients(bool on) {
    std::unordered_map<Node*, std::vector<Node*>> users;
    for (Node* n : nodes_)
        for (Node* in : n->inputs) users[in].push_back(n);
    for (Node* n : nodes_) {
        bool mark = false;
        if (on && !n->inputs.empty() && n->output->requiresGrad() && users[n].size() == 1) {
            Node* u = users[n][0];
            const bool first = !u->inputs.empty() && u->inputs[0] == n &&
                               std::count(u->inputs.begin(), u->inputs.end(), n) == 1;
            mark = first && (u->type == "Conv2d" || u->type == "Linear" || u->type == "AveragePooling");
        }
        // an output node shares its input's tensor: never mark that one
        for (Node* o : outputs_)
            if (!o->inputs.empty() && o->inputs[0] == n) mark = false;
        n->output->setGradOverwritten(mark);
    }
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
    optimizer->beginBatch();
    for (size_t i = 0; i < nodes_.size(); i++) {
        Node* n = nodes_[i];
        if (ticks_before_[i]) optimizer->skip(ticks_before_[i]);
        if (!n->output->requiresGrad()) continue;
        if (step_intermediates_ || n->inputs.empty()) optimizer->step(n);
        else optimizer->skip(1);  // the reference steps this activation (src/ComputeGraph.cu:541-547)
    }
    if (pending_ticks_) optimizer->skip(pending_ticks_);
    optimizer->endBatch();
}
// ---- save / load (src/ComputeGraph.cu:553-811) -------------------------------------------------
namespace {
void write_floats(FILE* f, const std::vector<float>& v) {
    fputc('[', f);
    for (size_t i = 0; i < v.size(); i++) fprintf(f, i ? ", %.9g" : "%.9g", (double)v[i]);
    fputc(']', f);
}
// text between the first '[' and the matching last ']' after `key` on this line
bool bracket_body(const std::string& line, const char* key, std::string* body) {
    const size_t k = line.find(key);
    if (k == std::string::npos) return false;
    const size_t a = line.find('[', k), b = line.rfind(']');
    if (a == std::string::npos || b == std::string::npos || b < a) return false;
    *body = line.substr(a + 1, b - a - 1);
    return true;
}
template <class T>
std::vector<T> parse_numbers(const std::string& body) {
    std::vector<T> out;
    const char* p = body.c_str();
    while (*p) {
        while (*p == ' ' || *p == ',' || *p == '\t') p++;
        if (!*p) break;
        char* end = nullptr;
        const double v = strtod(p, &end);
        if (end == p) break;
        out.push_back((T)v);
        p = end;
    }
    return out;
}
std::string quoted_value(const std::string& line, const char* key) {
    const size_t k = line.find(key);
    if (k == std::string::npos) return "";
    const size_t a = line.find('"', k + strlen(key)), b = a == std::string::npos ? a : line.find('"', a + 1);
    return b == std::string::npos ? "" : line.substr(a + 1, b - a - 1);
}
}  // namespace

void ComputeGraph::save(const std::string& path, const opt::Optimizer* optimizer) {
    if (path.empty()) throw std::runtime_error("Path cannot be empty");
    if (!sorted_) topologicalSort();
    if (sorted_nodes_.empty()) throw std::runtime_error("Graph not sorted");
    FILE* f = fopen(path.c_str(), "w");
    if (!f) throw std::runtime_error("Failed to open file for writing");
    auto index_of = [&](Node* n) {
        return (long)(std::find(sorted_nodes_.begin(), sorted_nodes_.end(), n) - sorted_nodes_.begin());
    };
    names_.resize(sorted_nodes_.size());
    fprintf(f, "[\n");
    for (size_t i = 0; i < sorted_nodes_.size(); i++) {
        Node* n = sorted_nodes_[i];
        if (names_[i].empty()) names_[i] = n->type + "_" + std::to_string(i);
        fprintf(f, "  {\n    \"type\": \"%s\",\n    \"name\": \"%s\",\n    \"pre\": [", n->type.c_str(), names_[i].c_str());
        for (size_t j = 0; j < n->inputs.size(); j++) fprintf(f, j ? ", %ld" : "%ld", index_of(n->inputs[j]));
        fprintf(f, "],\n    \"post\": [");
        bool first = true;
        for (Node* u : sorted_nodes_)
            if (std::find(u->inputs.begin(), u->inputs.end(), n) != u->inputs.end()) {
                fprintf(f, first ? "%ld" : ", %ld", index_of(u));
                first = false;
            }
        const auto shape = n->output->shape();
        fprintf(f, "],\n    \"shape\": [%zu, %zu, %zu, %zu],\n", shape[0], shape[1], shape[2], shape[3]);
        const size_t pos = (size_t)(std::find(nodes_.begin(), nodes_.end(), n) - nodes_.begin());
        fprintf(f, "    \"order\": %zu,\n    \"ticks\": %d,\n    \"attr\": [", pos, pos < ticks_before_.size() ? ticks_before_[pos] : 0);
        const auto attr = n->attributes();
        for (size_t j = 0; j < attr.size(); j++) fprintf(f, j ? ", %zu" : "%zu", attr[j]);
        fprintf(f, "],\n    \"data\": ");
        write_floats(f, n->output->hostData());
        fprintf(f, ",\n    \"requires_grad\": %s,\n    \"grad\": ", n->output->requiresGrad() ? "true" : "false");
        write_floats(f, n->output->requiresGrad() ? n->output->hostGrad() : std::vector<float>());
        if (optimizer) {
            const auto state = optimizer->exportState(n);
            for (size_t k = 0; k < state.size(); k++) {
                fprintf(f, ",\n    \"opt_state_%zu\": ", k);
                write_floats(f, state[k]);
            }
        }
        fprintf(f, "\n  },\n");
    }
    // trailer: what belongs to the graph as a whole
    fprintf(f, "  {\n    \"type\": \"Optimizer\",\n    \"name\": \"%s\",\n    \"counter\": %ld,\n    \"pending_ticks\": %d\n  }\n]\n",
            optimizer ? optimizer->name() : "none", optimizer ? optimizer->counter() : 0L, pending_ticks_);
    if (fclose(f) != 0) throw std::runtime_error("Failed to write " + path);
}

void ComputeGraph::load(const std::string& path, opt::Optimizer* optimizer) {
    if (path.empty()) throw std::runtime_error("Path cannot be empty");
    if (!nodes_.empty()) throw std::runtime_error("Graph already loaded");
    std::ifstream in(path);
    if (!in.is_open()) throw std::runtime_error("Failed to open file for reading");
    struct Rec {
        std::string type, name;
        std::vector<long> pre, shape, attr;
        std::vector<float> data, grad;
        std::vector<std::vector<float>> opt;
        bool requires_grad = false;
        long order = -1, ticks = 0, counter = 0, pending = 0;
    };
    std::vector<Rec> recs;
    Rec cur;
    bool open = false;
    std::string line, body;
    while (std::getline(in, line)) {
        if (!open) {
            if (line.find('{') != std::string::npos) {
                open = true;
                cur = Rec();
            }
            continue;
        }
        if (line.find("\"type\":") != std::string::npos) cur.type = quoted_value(line, "\"type\":");
        else if (line.find("\"name\":") != std::string::npos) cur.name = quoted_value(line, "\"name\":");
        else if (bracket_body(line, "\"pre\":", &body)) cur.pre = parse_numbers<long>(body);
        else if (line.find("\"post\":") != std::string::npos) {}
        else if (bracket_body(line, "\"shape\":", &body)) cur.shape = parse_numbers<long>(body);
        else if (bracket_body(line, "\"attr\":", &body)) cur.attr = parse_numbers<long>(body);
        else if (bracket_body(line, "\"data\":", &body)) cur.data = parse_numbers<float>(body);
        else if (line.find("\"requires_grad\":") != std::string::npos) cur.requires_grad = line.find("true") != std::string::npos;
        else if (bracket_body(line, "\"grad\":", &body)) cur.grad = parse_numbers<float>(body);
        else if (line.find("\"opt_state_") != std::string::npos && bracket_body(line, "\"opt_state_", &body)) cur.opt.push_back(parse_numbers<float>(body));
        else if (line.find("\"order\":") != std::string::npos) cur.order = atol(line.c_str() + line.find(':') + 1);
        else if (line.find("\"ticks\":") != std::string::npos) cur.ticks = atol(line.c_str() + line.find(':') + 1);
        else if (line.find("\"counter\":") != std::string::npos) cur.counter = atol(line.c_str() + line.find(':') + 1);
        else if (line.find("\"pending_ticks\":") != std::string::npos) cur.pending = atol(line.c_str() + line.find(':') + 1);
        else if (line.find('}') != std::string::npos) {
            open = false;
            recs.push_back(cur);
        }
    }
    using data::Dimension;
    namespace calc = nodes::calc;
    namespace io = nodes::io;
    std::vector<Node*> created;
    std::vector<std::pair<long, Node*>> order;
    std::vector<int> ticks;
    for (const Rec& r : recs) {
        if (r.type == "Optimizer") {
            if (optimizer && r.name == optimizer->name()) optimizer->setCounter(r.counter);
            pending_ticks_ = (int)r.pending;
            continue;
        }
        auto in_node = [&](size_t k) -> Node* {
            if (k >= r.pre.size() || r.pre[k] < 0 || (size_t)r.pre[k] >= created.size())
                throw std::runtime_error("node " + r.name + " refers to an input that is not defined before it");
            return created[(size_t)r.pre[k]];
        };
        auto attr = [&](size_t k) -> size_t {
            if (k >= r.attr.size()) throw std::runtime_error("node " + r.name + " (" + r.type + ") lacks a constructor attribute");
            return (size_t)r.attr[k];
        };
        Dimension shape(1, 1, 1, 1);
        if (r.shape.size() == 4) shape = Dimension(r.shape[0], r.shape[1], r.shape[2], r.shape[3]);
        else if (r.shape.size() == 2) {
            // a file written by the reference: only N and C were kept; the rest is the element count
            const size_t nc = (size_t)std::max(1L, r.shape[0] * r.shape[1]);
            shape = Dimension(r.shape[0], r.shape[1], std::max<size_t>(1, r.data.size() / nc), 1);
        } else throw std::runtime_error("node " + r.name + " has no usable shape");
        Node* n = nullptr;
        io::OutputNode* out = nullptr;
        if (r.type == "Input") n = new io::InputNode(shape, r.requires_grad);
        else if (r.type == "Output") n = out = new io::OutputNode(in_node(0));
        else if (r.type == "Add") n = new calc::AddNode(in_node(0), in_node(1));
        else if (r.type == "MatMul") n = new calc::MatMulNode(in_node(0), in_node(1));
        else if (r.type == "ReLU") n = new calc::ReLUNode(in_node(0));
        else if (r.type == "Reshape") n = new calc::ReshapeNode(in_node(0), shape);
        else if (r.type == "Expand") n = new calc::ExpandNode(in_node(0), shape[0]);
        else if (r.type == "Img2Col") n = new calc::Img2ColNode(in_node(0), attr(0), attr(1), attr(2), attr(3));
        else if (r.type == "Col2Img") n = new calc::Col2ImgNode(in_node(0), attr(0), attr(1));
        else if (r.type == "AveragePooling") n = new calc::AveragePoolingNode(in_node(0), attr(0), attr(1), attr(2));
        else if (r.type == "MaxPooling") n = new calc::MaxPoolingNode(in_node(0), attr(0), attr(1), attr(2));
        else if (r.type == "Softmax") n = new calc::SoftmaxNode(in_node(0));
        else if (r.type == "Conv2d")
            n = new calc::Conv2dNode(in_node(0), in_node(1), r.pre.size() > 2 ? in_node(2) : nullptr, attr(0), attr(1),
                                     attr(2), attr(3), attr(4) != 0);
        else if (r.type == "Linear")
            n = new calc::LinearNode(in_node(0), in_node(1), r.pre.size() > 2 ? in_node(2) : nullptr, attr(0) != 0);
        else if (r.type == "BinaryCrossEntropy") n = out = new nodes::loss::BinaryCrossEntropyNode(in_node(0), in_node(1));
        else throw std::runtime_error("node type '" + r.type + "' is not part of this library");
        owned_.emplace_back(n);
        created.push_back(n);
        names_.push_back(r.name);
        // a loss node's output IS its input's tensor: nothing of its own to restore
        if (!out) {
            if (r.data.size() != n->output->size())
                throw std::runtime_error("node " + r.name + " holds " + std::to_string(r.data.size()) + " values, its shape needs " +
                                         std::to_string(n->output->size()));
            n->output->dataInject(const_cast<float*>(r.data.data()));
            if (n->output->requiresGrad() && r.grad.size() == n->output->size())
                n->output->dataInject(const_cast<float*>(r.grad.data()), true);
        }
        if (optimizer && !r.opt.empty()) optimizer->importState(n, r.opt);
        order.emplace_back(r.order >= 0 ? r.order : (long)order.size(), n);
        ticks.push_back((int)r.ticks);
        if (out) outputs_.push_back(out);
        else if (r.type == "Input") inputs_.push_back(static_cast<io::InputNode*>(n));
    }
    // insertion order of the saved graph: it decides which per-call time step Adam gives each parameter
    std::vector<size_t> perm(order.size());
    for (size_t i = 0; i < perm.size(); i++) perm[i] = i;
    std::stable_sort(perm.begin(), perm.end(), [&](size_t a, size_t b) { return order[a].first < order[b].first; });
    for (size_t i : perm) {
        nodes_.push_back(order[i].second);
        ticks_before_.push_back(ticks[i]);
    }
    sorted_nodes_ = created;
    sorted_ = true;
}

nodes::Node* ComputeGraph::operator[](const std::string& name) const {
    for (size_t i = 0; i < names_.size() && i < sorted_nodes_.size(); i++)
        if (names_[i] == name) return sorted_nodes_[i];
    return nullptr;
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
    if (batching_) {
        batch_.emplace_back(input, tstep);
        return;
    }
    const auto sl = sliceOf(input);
    SM::Instance().run({t.data(), m->data(), v->data()}, {t.grad()}, [&](cudaStream_t s) {
        NZB_CHECK(nzb_adam(t.data() + sl.first, m->data() + sl.first, v->data() + sl.first, t.grad() + sl.first,
                           learning_rate, beta1_, beta2_, epsilon_, tstep, (int64_t)sl.second, s));
    });
}

void Adam::beginBatch() {
    batching_ = true;
    batch_.clear();
}
void Adam::endBatch() {
    batching_ = false;
    if (batch_.empty()) return;
    // one launch for all tensors: ordered after every pending use of the tensors it writes (weights and
    // moments) and after the writers of the gradients it reads (the all-reduce of a data-parallel step)
    std::vector<nzb_adam_tensor> list(batch_.size());
    auto& sm = SM::Instance();
    cudaStream_t s = sm.getStream();
    for (size_t i = 0; i < batch_.size(); i++) {
        data::Tensor& t = *batch_[i].first->output;
        data::Tensor& m = *m_[batch_[i].first];
        data::Tensor& v = *v_[batch_[i].first];
        sm.streamWait(t.data(), s, true);
        sm.streamWait(m.data(), s, true);
        sm.streamWait(v.data(), s, true);
        sm.streamWait(t.grad(), s, false);
        const auto sl = sliceOf(batch_[i].first);
        list[i] = nzb_adam_tensor{t.data() + sl.first, m.data() + sl.first, v.data() + sl.first, t.grad() + sl.first,
                                  nullptr, (int64_t)sl.second, batch_[i].second, 0};
    }
    NZB_CHECK(nzb_adam_multi(list.data(), (int)list.size(), learning_rate, beta1_, beta2_, epsilon_, s));
    for (size_t i = 0; i < batch_.size(); i++) {
        data::Tensor& t = *batch_[i].first->output;
        sm.recordData(t.data(), s);
        sm.recordData(m_[batch_[i].first]->data(), s);
        sm.recordData(v_[batch_[i].first]->data(), s);
        sm.recordRead(t.grad(), s);
    }
    batch_.clear();
}

std::vector<std::vector<float>> Adam::exportState(nodes::Node* node) const {
    auto m = m_.find(node);
    auto v = v_.find(node);
    if (m == m_.end() || v == v_.end() || !m->second || !v->second) return {};
    return {m->second->hostData(), v->second->hostData()};
}
void Adam::importState(nodes::Node* node, const std::vector<std::vector<float>>& state) {
    if (state.size() != 2 || state[0].size() != node->output->size() || state[1].size() != node->output->size())
        throw std::runtime_error("Adam state of a node does not match its size");
    auto& m = m_[node];
    auto& v = v_[node];
    m = std::make_unique<data::Tensor>(node->output->shape());
    v = std::make_unique<data::Tensor>(node->output->shape());
    m->dataInject(const_cast<float*>(state[0].data()));
    v->dataInject(const_cast<float*>(state[1].data()));
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
    if (fused_ && !gradients_marked_) {
        computeGraph.overwriteSingleConsumerGradients(true);
        gradients_marked_ = true;
    }
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
                    exchangeGradient(i);
                    param_synced_[i] = true;
                }
    });
}
bool Model::sharded(size_t i) const {
    return shard_optimizer_ && comm_ && comm_->world() > 1 && params_[i]->output->size() % (size_t)comm_->world() == 0;
}
void Model::exchangeGradient(size_t i) {
    Tensor& t = *params_[i]->output;
    // sharded optimizer: this rank only needs the average of the slice it will update
    if (sharded(i)) comm_->reduceScatterAverage(t.grad(), t.size());
    else comm_->allReduceAverage(t.grad(), t.size());
}
void Model::syncGradients() {
    if (comm_ && comm_->world() > 1 && !grads_synced_)
        for (size_t i = 0; i < params_.size(); i++)
            if (i >= param_synced_.size() || !param_synced_[i]) exchangeGradient(i);
    grads_synced_ = true;
    param_synced_.assign(params_.size(), true);
}
void Model::gatherGradients() {
    syncGradients();
    if (!(comm_ && comm_->world() > 1)) return;
    for (size_t i = 0; i < params_.size(); i++)
        if (sharded(i)) comm_->allGather(params_[i]->output->grad(), params_[i]->output->size());
}
void Model::update(opt::Optimizer* optimizer) {
    const bool dp = comm_ && comm_->world() > 1;
    for (size_t i = 0; i < params_.size(); i++) {
        const size_t n = params_[i]->output->size();
        if (dp && sharded(i)) optimizer->setSlice(params_[i], (size_t)comm_->rank() * (n / comm_->world()), n / comm_->world());
        else optimizer->setSlice(params_[i], 0, 0);
    }
    computeGraph.update(optimizer, [this]() { syncGradients(); });
    // every rank stepped its own slice of a sharded parameter: collect the updated slices. Queued in
    // creation order, which is the order the next forward pass needs the parameters in, so the large
    // ones that come last travel under the first layers' kernels.
    if (dp)
        for (size_t i = 0; i < params_.size(); i++)
            if (sharded(i)) comm_->allGather(params_[i]->output->data(), params_[i]->output->size());
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
Model::Node* Model::MaxPool2d(Node* input, size_t pool, size_t stride, size_t pad) {
    computeGraph.addNode(input);
    return own(new calc::MaxPoolingNode(input, pool, stride, pad));
}
void Model::BCELoss(Node* input, Node* target) {
    computeGraph.addNode(input);
    Node* expanded = TargetExpand(target, input->output->shape());
    auto* bce = new nodes::loss::BinaryCrossEntropyNode(input, expanded);
    if (fused_) bce->fuseWithSoftmax(true);
    hiddenNodes.push_back(bce);
    computeGraph.addOutput(bce);
}

}  // namespace nz
