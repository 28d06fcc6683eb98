// Drives the UNMODIFIED NeuZephyr library (built by build_ref.sh) through its public API
// so that its results and timings can be set beside the sm_100a kernels on identical
// inputs. Test/benchmark infrastructure only.
//
//   ref_harness gemm_file  A.bin B.bin C.bin aN aC M K bN bC N      forward, GEMMTensorCore
//   ref_harness gemm_bwd   A.bin B.bin C.bin aN aC M K bN bC N cN cC  iGEMMBackward into C (C.bin read, then overwritten)
//   ref_harness gemm_bench M N K steps warmup e2e                   prints one JSON line
//   ref_harness linear_bench B In Out steps warmup                  Model::Linear -> ReLU -> MSELoss, forward + backward
//   ref_harness conv_bench N C H W Cout k pad steps warmup          Model::Conv2d -> ReLU -> MSELoss, forward + backward
//   ref_harness model_bench B S steps warmup                        the README-style segmentation model, one Adam step
//   ref_harness conv_file  dir N C H W Cout k stride pad shared relu  Img2Col -> MatMul -> Add -> Col2Img [-> ReLU] with injected
//                                                                     weights: reads x,w,b,dy .bin from dir, writes y,dx,dw,db .bin
//   ref_harness linear_file dir B In Out relu                       Reshape-free Model::Linear chain, same files
//   ref_harness model_file dir B S steps shared                     the segmentation model as Model's builders compose it, built
//                                                                   node by node so that parameters can be injected: reads x,t,p0..p5,
//                                                                   writes loss.txt, g0..g5 (first backward), q<step>_<i> (after each update)
#include <NeuZephyr/Model.cuh>
#include <NeuZephyr/Optimizer.cuh>
#include <NeuZephyr/Tensor.cuh>
#include <NeuZephyr/TensorOperations.cuh>

#include <NeuZephyr/ComputeGraph.cuh>
#include <NeuZephyr/Nodes.cuh>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

using nz::data::Tensor;

static std::vector<float> read_bin(const char* path, size_t n) {
    std::vector<float> v(n);
    FILE* f = fopen(path, "rb");
    if (!f || fread(v.data(), sizeof(float), n, f) != n) {
        fprintf(stderr, "cannot read %zu floats from %s\n", n, path);
        exit(2);
    }
    fclose(f);
    return v;
}
static void write_bin(const char* path, const std::vector<float>& v) {
    FILE* f = fopen(path, "wb");
    if (!f || fwrite(v.data(), sizeof(float), v.size(), f) != v.size()) {
        fprintf(stderr, "cannot write %s\n", path);
        exit(2);
    }
    fclose(f);
}
static double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

static std::string in_dir(const std::string& dir, const std::string& name) { return dir + "/" + name; }

using nz::nodes::Node;
using nz::nodes::io::InputNode;
namespace calc = nz::nodes::calc;

// A chain of reference nodes driven by hand, the way test/Test.cpp drives single nodes: forward in
// creation order, the upstream gradient injected into the last node, backward in reverse order.
struct Chain {
    std::vector<Node*> nodes;
    template <class T>
    T* add(T* n) {
        nodes.push_back(n);
        return n;
    }
    void forward() {
        for (Node* n : nodes) n->forward();
    }
    void backward(float* dy) {
        // full synchronisation between the phases: the library orders its launches per data pointer,
        // and nothing here should depend on how it orders a clear against a later accumulation
        cudaDeviceSynchronize();
        for (Node* n : nodes)
            if (n->output->requiresGrad()) n->output->zeroGrad();
        cudaDeviceSynchronize();
        nodes.back()->output->dataInject(dy, true);
        cudaDeviceSynchronize();
        for (auto it = nodes.rbegin(); it != nodes.rend(); ++it) (*it)->backward();
        cudaDeviceSynchronize();
    }
    ~Chain() {
        for (Node* n : nodes) delete n;
    }
};

// The segmentation model in the node order Model::Conv2d / ReLU / AvgPool2d / Linear / Softmax /
// BCELoss create (src/Model.cu:87-103, 185-202, 244-263, 317-325), on a ComputeGraph of its own.
struct SegGraph {
    nz::graph::ComputeGraph g;
    std::vector<Node*> owned, params;
    InputNode *input, *target;
    template <class T>
    T* add(T* n, bool param = false) {
        owned.push_back(n);
        g.addNode(n);
        if (param) params.push_back(n);
        return n;
    }
    Node* conv(Node* in, size_t cout, size_t k, size_t pad, bool shared) {
        const auto s = in->output->shape();
        auto* w = add(new InputNode({shared ? 1 : s.N(), 1, s.C() * k * k, cout}, true), true);
        auto* col = add(new calc::Img2ColNode(in, k, k, 1, pad));
        auto* mm = add(new calc::MatMulNode(col, w));
        auto* b = add(new InputNode({1, mm->output->shape()[1], mm->output->shape()[2], mm->output->shape()[3]}, true), true);
        auto* sum = add(new calc::AddNode(mm, b));
        return add(new calc::Col2ImgNode(sum, s.H() + 2 * pad - k + 1, s.W() + 2 * pad - k + 1));
    }
    SegGraph(size_t B, size_t S, bool shared) {
        input = new InputNode({B, 3, S, S});
        target = new InputNode({B, 1, 16, 1});
        owned.push_back(input);
        owned.push_back(target);
        g.addNode(input);
        Node* x = conv(input, 16, 3, 1, shared);
        x = add(new calc::ReLUNode(x));
        x = conv(x, 16, 3, 1, shared);
        x = add(new calc::AveragePoolingNode(x, 5, 2, 0));
        const auto s = x->output->shape();
        const size_t in = s[1] * s[2] * s[3];
        x = add(new calc::ReshapeNode(x, {s[0], 1, in, 1}));
        auto* w = add(new InputNode({1, 1, 16, in}, true), true);
        x = add(new calc::MatMulNode(w, x));
        auto* b = add(new InputNode({1, 1, 16, 1}, true), true);
        x = add(new calc::AddNode(x, b));
        x = add(new calc::SoftmaxNode(x));
        g.addNode(target);
        auto* bce = new nz::nodes::loss::BinaryCrossEntropyNode(x, target);
        owned.push_back(bce);
        g.addOutput(bce);
    }
    ~SegGraph() {
        for (Node* n : owned) delete n;
    }
};

// Reference models built with the reference's own Model builders (src/Model.cu).
class RefLinear : public nz::Model {
public:
    nz::nodes::io::InputNode input, target;
    RefLinear(size_t B, size_t In, size_t Out) : input({B, 1, In, 1}), target({B, 1, Out, 1}) {
        auto x = Linear(&input, Out);
        x = ReLU(x);
        MSELoss(x, &target);
    }
};
class RefConv : public nz::Model {
public:
    nz::nodes::io::InputNode input, target;
    RefConv(size_t N, size_t C, size_t H, size_t W, size_t Co, size_t k, size_t pad)
        : input({N, C, H, W}), target({N, Co, H + 2 * pad - k + 1, W + 2 * pad - k + 1}) {
        auto x = Conv2d(&input, Co, k, k, 1, pad);
        x = ReLU(x);
        MSELoss(x, &target);
    }
};
class RefSeg : public nz::Model {
public:
    nz::nodes::io::InputNode input, target;
    RefSeg(size_t B, size_t S) : input({B, 3, S, S}), target({B, 1, 16, 1}) {
        auto x = Conv2d(&input, 16, 3, 3, 1, 1);
        x = ReLU(x);
        x = Conv2d(x, 16, 3, 3, 1, 1);
        x = AvgPool2d(x, 5, 2);
        x = Linear(x, 16);
        x = Softmax(x);
        BCELoss(x, &target);
    }
};

template <class M>
static void time_model(M& model, const char* name, int steps, int warmup, bool update, double images) {
    model.input.output->randomize(7);
    model.target.output->fill(0.5f);
    nz::opt::Adam adam(0.01f, 0.9f, 0.999f);
    auto step = [&]() {
        model.forward();
        model.backward();
        if (update) model.update(&adam);
    };
    for (int i = 0; i < warmup; i++) step();
    cudaDeviceSynchronize();
    const double t0 = now_ms();
    for (int i = 0; i < steps; i++) step();
    cudaDeviceSynchronize();
    const double ms = (now_ms() - t0) / steps;
    printf("{\"mode\": \"%s\", \"ms_per_step\": %.4f, \"img_per_s\": %.3f, \"steps\": %d}\n", name, ms,
           images / ms * 1e3, steps);
}

int main(int argc, char** argv) {
    if (argc < 2) return 1;
    const std::string mode = argv[1];
    if (mode == "linear_bench" && argc == 7) {
        RefLinear m(atoll(argv[2]), atoll(argv[3]), atoll(argv[4]));
        time_model(m, "linear_bench", atoi(argv[5]), atoi(argv[6]), false, (double)atoll(argv[2]));
        return 0;
    }
    if (mode == "conv_bench" && argc == 11) {
        RefConv m(atoll(argv[2]), atoll(argv[3]), atoll(argv[4]), atoll(argv[5]), atoll(argv[6]), atoll(argv[7]),
                  atoll(argv[8]));
        time_model(m, "conv_bench", atoi(argv[9]), atoi(argv[10]), false, (double)atoll(argv[2]));
        return 0;
    }
    if (mode == "model_bench" && argc == 6) {
        RefSeg m(atoll(argv[2]), atoll(argv[3]));
        time_model(m, "model_bench", atoi(argv[4]), atoi(argv[5]), true, (double)atoll(argv[2]));
        return 0;
    }
    if (mode == "conv_file" && argc == 14) {
        const std::string dir = argv[2];
        const size_t N = atoll(argv[3]), C = atoll(argv[4]), H = atoll(argv[5]), W = atoll(argv[6]), Co = atoll(argv[7]);
        const size_t k = atoll(argv[8]), stride = atoll(argv[9]), pad = atoll(argv[10]);
        const bool shared = atoi(argv[11]) != 0, relu = atoi(argv[12]) != 0, with_bias = atoi(argv[13]) != 0;
        const size_t Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1, K = C * k * k;
        Chain c;
        auto* x = c.add(new InputNode({N, C, H, W}, true));
        auto* w = c.add(new InputNode({shared ? 1 : N, 1, K, Co}, true));
        auto* col = c.add(new calc::Img2ColNode(x, k, k, stride, pad));
        Node* y = c.add(new calc::MatMulNode(col, w));
        InputNode* b = nullptr;
        if (with_bias) {
            b = c.add(new InputNode({1, 1, Ho * Wo, Co}, true));
            y = c.add(new calc::AddNode(y, b));
        }
        y = c.add(new calc::Col2ImgNode(y, Ho, Wo));
        if (relu) y = c.add(new calc::ReLUNode(y));
        auto hx = read_bin(in_dir(dir, "x.bin").c_str(), N * C * H * W);
        auto hw = read_bin(in_dir(dir, "w.bin").c_str(), (shared ? 1 : N) * K * Co);
        auto hdy = read_bin(in_dir(dir, "dy.bin").c_str(), N * Co * Ho * Wo);
        x->output->dataInject(hx.data());
        w->output->dataInject(hw.data());
        if (b) {
            auto hb = read_bin(in_dir(dir, "b.bin").c_str(), Ho * Wo * Co);
            b->output->dataInject(hb.data());
        }
        c.forward();
        write_bin(in_dir(dir, "ref_y.bin").c_str(), y->output->hostData());
        c.backward(hdy.data());
        write_bin(in_dir(dir, "ref_dx.bin").c_str(), x->output->hostGrad());
        write_bin(in_dir(dir, "ref_dw.bin").c_str(), w->output->hostGrad());
        if (b) write_bin(in_dir(dir, "ref_db.bin").c_str(), b->output->hostGrad());
        return 0;
    }
    if (mode == "linear_file" && argc == 7) {
        const std::string dir = argv[2];
        const size_t B = atoll(argv[3]), In = atoll(argv[4]), Out = atoll(argv[5]);
        const bool relu = atoi(argv[6]) != 0;
        Chain c;
        auto* x = c.add(new InputNode({B, 1, In, 1}, true));
        auto* w = c.add(new InputNode({1, 1, Out, In}, true));
        Node* y = c.add(new calc::MatMulNode(w, x));
        auto* b = c.add(new InputNode({1, 1, Out, 1}, true));
        y = c.add(new calc::AddNode(y, b));
        if (relu) y = c.add(new calc::ReLUNode(y));
        auto hx = read_bin(in_dir(dir, "x.bin").c_str(), B * In);
        auto hw = read_bin(in_dir(dir, "w.bin").c_str(), Out * In);
        auto hb = read_bin(in_dir(dir, "b.bin").c_str(), Out);
        auto hdy = read_bin(in_dir(dir, "dy.bin").c_str(), B * Out);
        x->output->dataInject(hx.data());
        w->output->dataInject(hw.data());
        b->output->dataInject(hb.data());
        c.forward();
        write_bin(in_dir(dir, "ref_y.bin").c_str(), y->output->hostData());
        c.backward(hdy.data());
        write_bin(in_dir(dir, "ref_dx.bin").c_str(), x->output->hostGrad());
        write_bin(in_dir(dir, "ref_dw.bin").c_str(), w->output->hostGrad());
        write_bin(in_dir(dir, "ref_db.bin").c_str(), b->output->hostGrad());
        return 0;
    }
    if (mode == "model_file" && argc == 7) {
        const std::string dir = argv[2];
        const size_t B = atoll(argv[3]), S = atoll(argv[4]);
        const int steps = atoi(argv[5]);
        const bool shared = atoi(argv[6]) != 0;
        SegGraph m(B, S, shared);
        auto hx = read_bin(in_dir(dir, "x.bin").c_str(), B * 3 * S * S);
        auto ht = read_bin(in_dir(dir, "t.bin").c_str(), B * 16);
        m.input->output->dataInject(hx.data());
        m.target->output->dataInject(ht.data());
        for (size_t i = 0; i < m.params.size(); i++) {
            auto hp = read_bin(in_dir(dir, "p" + std::to_string(i) + ".bin").c_str(), m.params[i]->output->size());
            m.params[i]->output->dataInject(hp.data());
        }
        // ComputeGraph::zeroGrad() would dereference the loss node's output, which the reference only
        // sets in OutputNode::forward(): clear the gradients node by node instead
        for (Node* n : m.owned)
            if (n->output && n->output->requiresGrad()) n->output->zeroGrad();
        cudaDeviceSynchronize();
        nz::opt::Adam adam(0.01f, 0.9f, 0.999f);
        FILE* lf = fopen(in_dir(dir, "ref_loss.txt").c_str(), "w");
        for (int s = 0; s < steps; s++) {
            m.g.forward();
            cudaDeviceSynchronize();
            fprintf(lf, "%.9g\n", m.g.getLoss());  // accumulates over steps, as the reference's loss node does
            m.g.backward();
            cudaDeviceSynchronize();
            if (s == 0)
                for (size_t i = 0; i < m.params.size(); i++)
                    write_bin(in_dir(dir, "ref_g" + std::to_string(i) + ".bin").c_str(), m.params[i]->output->hostGrad());
            m.g.update(&adam);  // Model::update (src/Model.cu:20-23)
            m.g.zeroGrad();
            cudaDeviceSynchronize();
            for (size_t i = 0; i < m.params.size(); i++)
                write_bin(in_dir(dir, "ref_q" + std::to_string(s) + "_" + std::to_string(i) + ".bin").c_str(),
                          m.params[i]->output->hostData());
        }
        fclose(lf);
        return 0;
    }
    if (mode == "gemm_file" && argc == 12) {
        const size_t aN = atoll(argv[5]), aC = atoll(argv[6]), M = atoll(argv[7]), K = atoll(argv[8]);
        const size_t bN = atoll(argv[9]), bC = atoll(argv[10]), N = atoll(argv[11]);
        Tensor A({aN, aC, M, K}), B({bN, bC, K, N});
        Tensor C({std::max(aN, bN), std::max(aC, bC), M, N});
        auto a = read_bin(argv[2], aN * aC * M * K), b = read_bin(argv[3], bN * bC * K * N);
        A.dataInject(a.data());
        B.dataInject(b.data());
        nz::data::GEMMTensorCore(C, A, B);
        write_bin(argv[4], C.hostData());
        return 0;
    }
    if (mode == "gemm_bwd" && argc == 14) {
        const size_t aN = atoll(argv[5]), aC = atoll(argv[6]), M = atoll(argv[7]), K = atoll(argv[8]);
        const size_t bN = atoll(argv[9]), bC = atoll(argv[10]), N = atoll(argv[11]);
        const size_t cN = atoll(argv[12]), cC = atoll(argv[13]);
        Tensor A({aN, aC, M, K}), B({bN, bC, K, N}), C({cN, cC, M, N});
        auto a = read_bin(argv[2], aN * aC * M * K), b = read_bin(argv[3], bN * bC * K * N);
        auto c = read_bin(argv[4], cN * cC * M * N);
        A.dataInject(a.data());
        B.dataInject(b.data());
        C.dataInject(c.data());
        nz::data::iGEMMBackward(A.data(), B.data(), C.data(), A.shape(), B.shape(), C.shape());
        write_bin(argv[4], C.hostData());
        return 0;
    }
    if (mode == "gemm_bench" && argc == 8) {
        const size_t M = atoll(argv[2]), N = atoll(argv[3]), K = atoll(argv[4]);
        const int steps = atoi(argv[5]), warmup = atoi(argv[6]), e2e = atoi(argv[7]);
        std::vector<float> a(M * K), b(K * N);
        unsigned long long s = 88172645463325252ull;  // xorshift64, uniform[-1,1]
        auto next = [&]() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return (float)((s >> 40) / 8388608.0 - 1.0); };
        for (auto& x : a) x = next();
        for (auto& x : b) x = next();
        Tensor A({1, 1, M, K}), B({1, 1, K, N}), C({1, 1, M, N});
        A.dataInject(a.data());
        B.dataInject(b.data());
        double checksum = 0;
        auto step = [&]() {
            if (e2e) {
                A.dataInject(a.data());
                B.dataInject(b.data());
            }
            nz::data::GEMMTensorCore(C, A, B);
            if (e2e) {
                auto h = C.hostData();
                checksum += h[0];
            } else {
                C.sync();
            }
        };
        for (int i = 0; i < warmup; i++) step();
        cudaDeviceSynchronize();
        // every step timed on its own, closed by the library's own completion wait (Tensor::sync inside
        // step(), or the blocking hostData copy): no device-wide synchronisation inside the loop, which
        // would make the stream-ordered pool give its memory back and re-map about 1 GB on the next call.
        // The median is the steady-state figure, the list shows the outliers.
        std::vector<double> each(steps);
        for (int i = 0; i < steps; i++) {
            const double t0 = now_ms();
            step();
            each[i] = now_ms() - t0;
        }
        cudaDeviceSynchronize();
        std::vector<double> sorted = each;
        std::sort(sorted.begin(), sorted.end());
        const double ms = sorted[sorted.size() / 2];
        double mean = 0;
        for (double v : each) mean += v / steps;
        printf("{\"ms_per_step\": %.6f, \"mean_ms_per_step\": %.6f, \"tflops\": %.6f, \"M\": %zu, \"N\": %zu, \"K\": %zu, "
               "\"e2e\": %d, \"checksum\": %.6g, \"steps\": %d, \"warmup\": %d, \"each_ms\": [",
               ms, mean, 2.0 * M * N * K / ms / 1e9, M, N, K, e2e, checksum, steps, warmup);
        for (int i = 0; i < steps; i++) printf("%s%.3f", i ? ", " : "", each[i]);
        printf("]}\n");
        return 0;
    }
    fprintf(stderr, "bad arguments\n");
    return 1;
}
