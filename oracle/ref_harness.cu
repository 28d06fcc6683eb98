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
#include <NeuZephyr/Model.cuh>
#include <NeuZephyr/Optimizer.cuh>
#include <NeuZephyr/Tensor.cuh>
#include <NeuZephyr/TensorOperations.cuh>

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
        const double t0 = now_ms();
        for (int i = 0; i < steps; i++) step();
        cudaDeviceSynchronize();
        const double ms = (now_ms() - t0) / steps;
        printf("{\"ms_per_step\": %.6f, \"tflops\": %.6f, \"M\": %zu, \"N\": %zu, \"K\": %zu, \"e2e\": %d, \"checksum\": %.6g}\n",
               ms, 2.0 * M * N * K / ms / 1e9, M, N, K, e2e, checksum);
        return 0;
    }
    fprintf(stderr, "bad arguments\n");
    return 1;
}
