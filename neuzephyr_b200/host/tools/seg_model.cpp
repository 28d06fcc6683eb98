// The README-style segmentation model of the benchmark configuration, on the nz:: host layer:
//   input {B,3,S,S} -> Conv2d(3->16,3x3,s1,p1) -> ReLU -> Conv2d(16->16,3x3,s1,p1) -> AvgPool2d(5,2)
//   -> Linear(->16) -> Softmax -> BCE against {B,1,16,1} targets; Adam(0.01, 0.9, 0.999).
// One process per GPU; with WORLD_SIZE > 1 the batch is sharded over ranks and parameter
// gradients are averaged with NCCL before the Adam step.
//
//   seg_model bench  <global_batch> <size> <steps> <warmup>   one JSON line on rank 0
//   seg_model check  <global_batch> <size>                    sharded step == full-batch step (rank 0 verifies)
//   seg_model phases <global_batch> <size> <steps> <warmup>   as bench, preceded by a line with forward / backward / update times
//   seg_model check  <global_batch> <size> emulate <W> [dir]  the same comparison on ONE GPU: the W shards run one after the
//                                                             other and their gradients are averaged on the host; with dir,
//                                                             writes sharded_g<i>.bin / full_g<i>.bin (the gradients compared)
//   seg_model step_file <dir> <batch> <size> <steps> <shared> [lr]  (Adam learning rate, default 0.01)
//                                                             reads x.bin, t.bin, p0..p5.bin (float32) from dir, runs `steps`
//                                                             training steps, writes loss.txt, g0..g5.bin (gradients of the first
//                                                             backward) and q<step>_<i>.bin (parameters after each update);
//                                                             shared = 0 gives every sample its own convolution weights, as
//                                                             the reference's Model::Conv2d allocates them
#include <NeuZephyr/Model.cuh>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

using namespace nz;
using nz::data::Tensor;
using nz::nodes::io::InputNode;

class SegModel : public Model {
public:
    InputNode input, target;
    SegModel(size_t batch, size_t size, bool perSample = false)
        : input({batch, 3, size, size}), target({batch, 1, 16, 1}) {
        computeGraph.addInput(&input);
        computeGraph.addInput(&target);
        auto x = Conv2d(&input, 16, 3, 3, 1, 1, true, perSample, /*fuseRelu=*/true);
        x = Conv2d(x, 16, 3, 3, 1, 1, true, perSample);
        x = AvgPool2d(x, 5, 2);
        x = Linear(x, 16);
        x = Softmax(x);
        BCELoss(x, &target);
    }
};

// Seeded values: uniform(-1,1)-like inputs and Kaiming-uniform weights (bound sqrt(6/fan_in)).
static void fill_uniform(std::vector<float>& v, float bound, unsigned seed) {
    std::mt19937 gen(seed);
    std::uniform_real_distribution<float> d(-bound, bound);
    for (auto& x : v) x = d(gen);
}
static void init_params(SegModel& m, size_t size) {
    const auto& p = m.parameters();  // w1, b1, w2, b2, wl, bl
    const size_t pooled = (size - 5) / 2 + 1;
    const float bounds[6] = {std::sqrt(6.f / 27.f), 0.f, std::sqrt(6.f / 144.f), 0.f,
                             std::sqrt(6.f / (16.f * pooled * pooled)), 0.f};
    for (size_t i = 0; i < p.size(); i++) {
        std::vector<float> w(p[i]->output->size(), 0.f);
        if (bounds[i] > 0.f) fill_uniform(w, bounds[i], 31 + (unsigned)i);
        p[i]->dataInject(w.data());
    }
    m.graph().zeroGrad();
}
static void make_batch(std::vector<float>& x, std::vector<float>& t, size_t batch, size_t size) {
    x.resize(batch * 3 * size * size);
    t.resize(batch * 16);
    fill_uniform(x, 1.f, 30);
    std::mt19937 gen(34);
    for (auto& v : t) v = (gen() & 1) ? 1.f : 0.f;
}
static std::vector<float> read_bin(const std::string& path, size_t n) {
    std::vector<float> v(n);
    FILE* f = fopen(path.c_str(), "rb");
    if (!f || fread(v.data(), sizeof(float), n, f) != n) {
        fprintf(stderr, "cannot read %zu floats from %s\n", n, path.c_str());
        exit(2);
    }
    fclose(f);
    return v;
}
static void write_bin(const std::string& path, const std::vector<float>& v) {
    FILE* f = fopen(path.c_str(), "wb");
    if (!f || fwrite(v.data(), sizeof(float), v.size(), f) != v.size()) {
        fprintf(stderr, "cannot write %s\n", path.c_str());
        exit(2);
    }
    fclose(f);
}
// step_file: a training run on injected data and parameters, results written as raw float32 files
static int step_file(const std::string& dir, size_t B, size_t S, int steps, bool shared, float lr) {
    SegModel model(B, S, !shared);
    auto x = read_bin(dir + "/x.bin", B * 3 * S * S), t = read_bin(dir + "/t.bin", B * 16);
    model.input.dataInject(x.data());
    model.target.dataInject(t.data());
    const auto& params = model.parameters();
    for (size_t i = 0; i < params.size(); i++) {
        auto p = read_bin(dir + "/p" + std::to_string(i) + ".bin", params[i]->output->size());
        params[i]->dataInject(p.data());
    }
    model.graph().zeroGrad();
    opt::Adam adam(lr, 0.9f, 0.999f);
    FILE* lf = fopen((dir + "/loss.txt").c_str(), "w");
    for (int s = 0; s < steps; s++) {
        model.forward();
        fprintf(lf, "%.9g\n", model.getLoss());  // accumulated over the steps, like the reference's loss node
        model.backward();
        if (s == 0)
            for (size_t i = 0; i < params.size(); i++)
                write_bin(dir + "/g" + std::to_string(i) + ".bin", params[i]->output->hostGrad());
        model.update(&adam);
        for (size_t i = 0; i < params.size(); i++)
            write_bin(dir + "/q" + std::to_string(s) + "_" + std::to_string(i) + ".bin", params[i]->output->hostData());
    }
    fclose(lf);
    cuStrm::StreamManager<float>::Instance().sync();
    int status = 0;
    nzb_device_status(&status);
    return status ? 1 : 0;
}
// Sharded-versus-full comparison shared by both forms of `check`: gradients relative to the largest
// full-batch gradient of the tensor, parameters after one Adam step where the gradient's sign is stable.
struct CheckResult {
    double worst_g = 0, worst_p = 0;
};
static void compare_param(CheckResult& r, const std::vector<float>& g, const std::vector<float>& fg,
                          const std::vector<float>* a, const std::vector<float>* c) {
    double gmax = 0, gnum = 0;
    for (size_t k = 0; k < fg.size(); k++) gmax = std::max(gmax, std::fabs((double)fg[k]));
    for (size_t k = 0; k < fg.size(); k++) {
        gnum = std::max(gnum, std::fabs((double)g[k] - fg[k]));
        // Adam's first step moves a weight by about lr * sign(g): compare weights only where the
        // gradient is well away from zero, so that its sign cannot flip with summation order
        if (a && std::fabs(fg[k]) > 1e-3 * gmax && std::fabs(fg[k]) > 1e-4)
            r.worst_p = std::max(r.worst_p, std::fabs((double)(*a)[k] - (*c)[k]));
    }
    r.worst_g = std::max(r.worst_g, gnum / (gmax > 0 ? gmax : 1));
}
// Gradients are GEMM operands rounded to fp16. A shard's loss is a mean over fewer elements, so its
// upstream gradients are larger by the world size than the full batch's, and values move in and out
// of fp16's subnormal range: the sharded average differs from the full-batch gradient by fp16
// rounding noise (measured against an fp64 host gradient in tests/test_model_gpu.py), not only by
// fp32 summation order.
static const double kGradTol = 2e-3, kParamTol = 1e-4;

static double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
    if (argc < 4) {
        fprintf(stderr, "usage: seg_model bench|check <global_batch> <size> [steps warmup]\n");
        return 2;
    }
    const std::string mode = argv[1];
    if (mode == "step_file") {
        if (argc != 7 && argc != 8) {
            fprintf(stderr, "usage: seg_model step_file <dir> <batch> <size> <steps> <shared> [learning rate]\n");
            return 2;
        }
        CHECK(cudaSetDevice(getenv("LOCAL_RANK") ? atoi(getenv("LOCAL_RANK")) : 0));
        return step_file(argv[2], atoll(argv[3]), atoll(argv[4]), atoi(argv[5]), atoi(argv[6]) != 0,
                         argc == 8 ? (float)atof(argv[7]) : 0.01f);
    }
    const size_t B = atoll(argv[2]), S = atoll(argv[3]);
    if (mode == "check" && argc >= 6 && std::string(argv[4]) == "emulate") {
        // the data-parallel arithmetic on one GPU: each of the W shards runs alone on its slice of
        // the batch, the host averages their gradients, and the average is compared with the
        // gradient of the whole batch
        const size_t W = atoll(argv[5]);
        const std::string dir = argc > 6 ? argv[6] : "";
        CHECK(cudaSetDevice(getenv("LOCAL_RANK") ? atoi(getenv("LOCAL_RANK")) : 0));
        if (W == 0 || B % W) {
            fprintf(stderr, "global batch must divide by the number of shards\n");
            return 2;
        }
        const size_t b = B / W, xs = 3 * S * S;
        std::vector<float> x, t;
        make_batch(x, t, B, S);
        auto& sm = cuStrm::StreamManager<float>::Instance();
        std::vector<std::vector<double>> avg;
        double loss = 0;
        for (size_t r = 0; r < W; r++) {
            SegModel shard(b, S);
            init_params(shard, S);
            shard.input.dataInject(x.data() + r * b * xs);
            shard.target.dataInject(t.data() + r * b * 16);
            shard.forward();
            loss += shard.getLoss() / W;
            shard.backward();
            sm.sync();
            for (size_t i = 0; i < shard.parameters().size(); i++) {
                const auto g = shard.parameters()[i]->output->hostGrad();
                if (avg.size() <= i) avg.emplace_back(g.size(), 0.0);
                for (size_t k = 0; k < g.size(); k++) avg[i][k] += (double)g[k] / W;
            }
        }
        SegModel full(B, S);
        init_params(full, S);
        full.input.dataInject(x.data());
        full.target.dataInject(t.data());
        full.forward();
        const float full_loss = full.getLoss();
        full.backward();
        sm.sync();
        CheckResult res;
        for (size_t i = 0; i < full.parameters().size(); i++) {
            const auto fg = full.parameters()[i]->output->hostGrad();
            std::vector<float> g(avg[i].begin(), avg[i].end());
            compare_param(res, g, fg, nullptr, nullptr);
            if (!dir.empty()) {
                write_bin(dir + "/sharded_g" + std::to_string(i) + ".bin", g);
                write_bin(dir + "/full_g" + std::to_string(i) + ".bin", fg);
                write_bin(dir + "/p" + std::to_string(i) + ".bin", full.parameters()[i]->output->hostData());
            }
        }
        if (!dir.empty()) {
            write_bin(dir + "/x.bin", x);
            write_bin(dir + "/t.bin", t);
        }
        const bool ok = res.worst_g <= kGradTol && std::fabs(loss - full_loss) <= 1e-4 * std::fabs(full_loss) + 1e-6;
        printf("{\"mode\": \"check\", \"world\": %zu, \"emulated\": true, \"loss_sharded\": %.7f, \"loss_full\": %.7f, "
               "\"max_rel_grad_diff\": %.3e, \"ok\": %s}\n", W, loss, full_loss, res.worst_g, ok ? "true" : "false");
        return ok ? 0 : 1;
    }
    const int rank = getenv("RANK") ? atoi(getenv("RANK")) : 0;
    const int world = getenv("WORLD_SIZE") ? atoi(getenv("WORLD_SIZE")) : 1;
    const int local = getenv("LOCAL_RANK") ? atoi(getenv("LOCAL_RANK")) : rank;
    CHECK(cudaSetDevice(local));
    dist::Communicator* comm = dist::Communicator::fromEnvironment();
    if (B % world) {
        fprintf(stderr, "global batch must divide by the world size\n");
        return 2;
    }
    const size_t b = B / world;
    std::vector<float> x, t;
    make_batch(x, t, B, S);
    const size_t xs = 3 * S * S;
    int rc = 0;
    {
        SegModel model(b, S);
        model.setCommunicator(comm);
        // NZ_DP_SHARD_OPTIMIZER=0 keeps the replicated optimizer step (all-reduce, every rank updates
        // every parameter); the default shards it (reduce-scatter, update of 1/world, all-gather)
        model.setShardedOptimizer(!(getenv("NZ_DP_SHARD_OPTIMIZER") && getenv("NZ_DP_SHARD_OPTIMIZER")[0] == '0'));
        init_params(model, S);
        model.input.dataInject(x.data() + rank * b * xs);
        model.target.dataInject(t.data() + rank * b * 16);
        opt::Adam adam(0.01f, 0.9f, 0.999f);
        auto& sm = cuStrm::StreamManager<float>::Instance();
        if (mode == "check") {
            model.forward();
            const float local_loss = model.getLoss();
            model.backward();
            model.gatherGradients();  // complete averaged gradients on every rank, for the comparison
            std::vector<std::vector<float>> grads;
            for (auto* p : model.parameters()) grads.push_back(p->output->hostGrad());
            model.update(&adam);
            sm.sync();
            const float loss = comm ? comm->allReduceSumHost(local_loss) / world : local_loss;
            if (rank == 0) {
                // the same step on the full batch, alone
                SegModel full(B, S);
                init_params(full, S);
                full.input.dataInject(x.data());
                full.target.dataInject(t.data());
                opt::Adam adam2(0.01f, 0.9f, 0.999f);
                full.forward();
                const float full_loss = full.getLoss();
                full.backward();
                std::vector<std::vector<float>> fgrads;
                for (auto* p : full.parameters()) fgrads.push_back(p->output->hostGrad());
                full.update(&adam2);
                sm.sync();
                CheckResult res;
                for (size_t i = 0; i < model.parameters().size(); i++) {
                    const auto a = model.parameters()[i]->output->hostData();
                    const auto c = full.parameters()[i]->output->hostData();
                    compare_param(res, grads[i], fgrads[i], &a, &c);
                }
                const double worst_g = res.worst_g, worst_p = res.worst_p;
                const bool ok = worst_g <= kGradTol && worst_p <= kParamTol &&
                                std::fabs(loss - full_loss) <= 1e-4 * std::fabs(full_loss) + 1e-6;
                printf("{\"mode\": \"check\", \"world\": %d, \"loss_sharded\": %.7f, \"loss_full\": %.7f, "
                       "\"max_rel_grad_diff\": %.3e, \"max_abs_param_diff\": %.3e, \"ok\": %s}\n",
                       world, loss, full_loss, worst_g, worst_p, ok ? "true" : "false");
                rc = ok ? 0 : 1;
            }
            if (comm) comm->barrier();
        } else {
            const int steps = argc > 4 ? atoi(argv[4]) : 5, warmup = argc > 5 ? atoi(argv[5]) : 2;
            auto step = [&]() {
                model.forward();
                model.backward();
                model.update(&adam);
            };
            for (int i = 0; i < warmup; i++) step();
            sm.sync();
            if (mode == "phases") {
                // forward / backward / update timed apart, each closed by a full synchronisation
                double tf = 0, tb = 0, tu = 0;
                for (int i = 0; i < steps; i++) {
                    CHECK(cudaDeviceSynchronize());
                    const double a = now_ms();
                    model.forward();
                    sm.sync();
                    CHECK(cudaDeviceSynchronize());
                    const double b2 = now_ms();
                    model.backward();
                    sm.sync();
                    CHECK(cudaDeviceSynchronize());
                    const double c = now_ms();
                    model.update(&adam);
                    sm.sync();
                    CHECK(cudaDeviceSynchronize());
                    const double d = now_ms();
                    tf += b2 - a; tb += c - b2; tu += d - c;
                }
                if (rank == 0)
                    printf("{\"mode\": \"phases\", \"world\": %d, \"global_batch\": %zu, \"size\": %zu, \"forward_ms\": %.3f, "
                           "\"backward_ms\": %.3f, \"update_ms\": %.3f}\n", world, B, S, tf / steps, tb / steps, tu / steps);
            }
            if (comm) comm->barrier();
            const double t0 = now_ms();
            for (int i = 0; i < steps; i++) step();
            sm.sync();
            CHECK(cudaDeviceSynchronize());
            double ms = (now_ms() - t0) / steps;
            if (comm) {
                // max over ranks: every rank contributes its own time, slowest wins
                float mine = (float)ms, worst = 0.f;
                for (int r = 0; r < world; r++) worst = std::max(worst, comm->allReduceSumHost(r == rank ? mine : 0.f));
                ms = worst;
            }
            int status = 0;
            nzb_device_status(&status);
            if (rank == 0) {
                // the accumulated loss can be NaN at full size: with Adam(lr 0.01) and a 4.16 M fan-in the
                // logits saturate after the first step and BCE evaluates 0 * log 0, as the reference does
                const float loss = model.getLoss();
                char lbuf[32];
                if (std::isfinite(loss)) snprintf(lbuf, sizeof(lbuf), "%.6f", loss);
                else snprintf(lbuf, sizeof(lbuf), "null");
                printf("{\"mode\": \"bench\", \"world\": %d, \"global_batch\": %zu, \"size\": %zu, \"steps\": %d, "
                       "\"ms_per_step\": %.4f, \"img_per_s\": %.2f, \"loss_total\": %s, \"status\": %d}\n",
                       world, B, S, steps, ms, B / ms * 1e3, lbuf, status);
            }
            if (comm) comm->barrier();
        }
    }
    delete comm;
    return rc;
}
