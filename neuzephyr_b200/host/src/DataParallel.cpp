// NCCL data-parallel communicator of the host layer (one process per GPU).
#include <NeuZephyr/DataParallel.cuh>
#include <NeuZephyr/StreamManager.cuh>

#include <nccl.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace nz::dist {

using SM = cuStrm::StreamManager<float>;

#define NCCL_TRY(call)                                                                        \
    do {                                                                                      \
        ncclResult_t r_ = (call);                                                             \
        if (r_ != ncclSuccess)                                                                \
            throw std::runtime_error(std::string("NCCL: ") + ncclGetErrorString(r_) + " in " #call); \
    } while (0)

Communicator::Communicator(int rank, int world, const std::string& id_file, int device, double timeout_s)
    : rank_(rank), world_(world) {
    CHECK(cudaSetDevice(device));
    ncclUniqueId id;
    if (rank == 0) {
        NCCL_TRY(ncclGetUniqueId(&id));
        const std::string tmp = id_file + ".tmp";
        FILE* f = fopen(tmp.c_str(), "wb");
        if (!f || fwrite(&id, sizeof(id), 1, f) != 1) throw std::runtime_error("cannot write " + tmp);
        fclose(f);
        if (rename(tmp.c_str(), id_file.c_str()) != 0) throw std::runtime_error("cannot publish " + id_file);
    } else {
        const auto t0 = std::chrono::steady_clock::now();
        for (;;) {
            FILE* f = fopen(id_file.c_str(), "rb");
            if (f) {
                const size_t n = fread(&id, sizeof(id), 1, f);
                fclose(f);
                if (n == 1) break;
            }
            if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s)
                throw std::runtime_error("timed out waiting for the NCCL id file " + id_file);
            std::this_thread::sleep_for(std::chrono::milliseconds(20));
        }
    }
    ncclComm_t c;
    NCCL_TRY(ncclCommInitRank(&c, world, id, rank));
    comm_ = c;
    cudaStream_t s;
    CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    stream_ = s;
    CHECK(cudaMalloc(&scalar_, sizeof(float)));
}

Communicator* Communicator::fromEnvironment() {
    const char* r = getenv("RANK");
    const char* w = getenv("WORLD_SIZE");
    if (!r || !w || atoi(w) <= 1) return nullptr;
    const char* lr = getenv("LOCAL_RANK");
    const char* port = getenv("MASTER_PORT");
    const char* idf = getenv("NZ_DP_ID_FILE");
    std::string file = idf ? idf : std::string("/tmp/nz_dp_") + (port ? port : "0") + ".id";
    return new Communicator(atoi(r), atoi(w), file, lr ? atoi(lr) : atoi(r));
}

Communicator::~Communicator() {
    if (comm_) ncclCommDestroy(static_cast<ncclComm_t>(comm_));
    if (stream_) cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
    if (scalar_) cudaFree(scalar_);
}

void Communicator::allReduceAverage(float* grad, size_t n) {
    if (world_ <= 1 || n == 0) return;
    cudaStream_t s = static_cast<cudaStream_t>(stream_);
    // like any other operation: wait for the gradient's pending writers and readers, run on the
    // communication stream, publish a writer event so that the optimizer step orders after it
    SM::Instance().streamWait(grad, s, true);
    NCCL_TRY(ncclAllReduce(grad, grad, n, ncclFloat32, ncclAvg, static_cast<ncclComm_t>(comm_), s));
    SM::Instance().recordData(grad, s);
}

void Communicator::allReduceAverageOn(float* grad, size_t n, void* cuda_stream) {
    if (world_ <= 1 || n == 0) return;
    NCCL_TRY(ncclAllReduce(grad, grad, n, ncclFloat32, ncclAvg, static_cast<ncclComm_t>(comm_),
                           static_cast<cudaStream_t>(cuda_stream)));
}

float Communicator::allReduceSumHost(float v) {
    if (world_ <= 1) return v;
    cudaStream_t s = static_cast<cudaStream_t>(stream_);
    CHECK(cudaMemcpyAsync(scalar_, &v, sizeof(float), cudaMemcpyHostToDevice, s));
    NCCL_TRY(ncclAllReduce(scalar_, scalar_, 1, ncclFloat32, ncclSum, static_cast<ncclComm_t>(comm_), s));
    float out = 0.f;
    CHECK(cudaMemcpyAsync(&out, scalar_, sizeof(float), cudaMemcpyDeviceToHost, s));
    CHECK(cudaStreamSynchronize(s));
    return out;
}

void Communicator::barrier() { (void)allReduceSumHost(0.f); }

}  // namespace nz::dist

// ---- C ABI over the communicator (include/nzb_dp.h) ----------------------------------------------
#include <nzb_dp.h>

namespace {
thread_local std::string g_dp_error;
int dp_fail(int code, const std::string& what) {
    g_dp_error = what;
    return code;
}
}  // namespace

extern "C" {

const char* nzb_dp_last_error_string(void) { return g_dp_error.c_str(); }

int nzb_dp_init(int rank, int world, const char* id_file, int device, double timeout_s, void** comm_out) {
    if (!comm_out || !id_file) return dp_fail(NZB_ERR_BAD_ARG, "comm_out and id_file must be non-null");
    if (world < 1 || rank < 0 || rank >= world) return dp_fail(NZB_ERR_BAD_ARG, "rank outside [0, world)");
    try {
        *comm_out = new nz::dist::Communicator(rank, world, id_file, device, timeout_s > 0 ? timeout_s : 60.0);
    } catch (const std::exception& e) {
        *comm_out = nullptr;
        return dp_fail(NZB_ERR_CUDA, e.what());
    }
    return NZB_OK;
}

int nzb_dp_allreduce_avg(void* comm, float* grad, size_t n, void* stream) {
    if (!comm || (!grad && n)) return dp_fail(NZB_ERR_BAD_ARG, "null communicator or buffer");
    try {
        static_cast<nz::dist::Communicator*>(comm)->allReduceAverageOn(grad, n, stream);
    } catch (const std::exception& e) {
        return dp_fail(NZB_ERR_CUDA, e.what());
    }
    return NZB_OK;
}

int nzb_dp_world(void* comm, int* rank_out, int* world_out) {
    if (!comm) return dp_fail(NZB_ERR_BAD_ARG, "null communicator");
    auto* c = static_cast<nz::dist::Communicator*>(comm);
    if (rank_out) *rank_out = c->rank();
    if (world_out) *world_out = c->world();
    return NZB_OK;
}

int nzb_dp_finalize(void* comm) {
    delete static_cast<nz::dist::Communicator*>(comm);
    return NZB_OK;
}

}  // extern "C"
