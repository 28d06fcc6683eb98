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

namespace {
struct RendezvousHeader {
    uint64_t magic, nonce;
    int64_t created_ns;  // wall clock (system_clock) of the writer
    uint64_t bytes;
};
constexpr uint64_t kRendezvousMagic = 0x4e5a44503152657aull;  // "NZDP1Rez"
int64_t wall_ns() {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::system_clock::now().time_since_epoch())
        .count();
}
uint64_t fnv1a(uint64_t h, const char* s) {
    for (; s && *s; s++) h = (h ^ (unsigned char)*s) * 1099511628211ull;
    return h;
}
}  // namespace

void rendezvousPublish(const std::string& file, const void* payload, size_t bytes, uint64_t nonce) {
    std::remove(file.c_str());  // whatever an earlier run left behind
    const std::string tmp = file + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    const RendezvousHeader h{kRendezvousMagic, nonce, wall_ns(), (uint64_t)bytes};
    if (!f || fwrite(&h, sizeof(h), 1, f) != 1 || fwrite(payload, bytes, 1, f) != 1) {
        if (f) fclose(f);
        throw std::runtime_error("cannot write " + tmp);
    }
    fclose(f);
    if (rename(tmp.c_str(), file.c_str()) != 0) throw std::runtime_error("cannot publish " + file);
}

void rendezvousWait(const std::string& file, void* payload, size_t bytes, uint64_t nonce, double timeout_s,
                    double max_age_s) {
    const auto t0 = std::chrono::steady_clock::now();
    const int64_t started = wall_ns();
    std::string why = "no file";
    for (;;) {
        FILE* f = fopen(file.c_str(), "rb");
        if (f) {
            RendezvousHeader h{};
            const bool got = fread(&h, sizeof(h), 1, f) == 1 && h.magic == kRendezvousMagic && h.bytes == bytes &&
                             fread(payload, bytes, 1, f) == 1;
            fclose(f);
            if (!got) why = "unreadable or foreign record";
            else if (h.nonce != nonce) why = "record of another launch (nonce differs)";
            else if ((double)(started - h.created_ns) * 1e-9 > max_age_s) why = "stale record (older than this launch)";
            else return;
        }
        if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s)
            throw std::runtime_error("timed out waiting for the rendezvous file " + file + " (" + why + ")");
        std::this_thread::sleep_for(std::chrono::milliseconds(10));
    }
}

uint64_t launchNonce() {
    if (const char* n = getenv("NZ_DP_NONCE")) return strtoull(n, nullptr, 0);
    uint64_t h = 1469598103934665603ull;
    h = fnv1a(h, getenv("MASTER_ADDR"));
    h = fnv1a(h, getenv("MASTER_PORT"));
    h = fnv1a(h, getenv("TORCHELASTIC_RUN_ID"));
    return h;
}

CollectiveWatchdog::Outcome CollectiveWatchdog::wait() {
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        last_code = poll();
        polls++;
        if (last_code == 0) return Done;
        const bool failed = last_code != 1;
        const bool late = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > deadline_s;
        if (failed || late) {
            if (abort && !aborted) abort();
            aborted = true;
            return failed ? Failed : TimedOut;
        }
        std::this_thread::sleep_for(std::chrono::duration<double>(poll_interval_s));
    }
}

Communicator::Communicator(int rank, int world, const std::string& id_file, int device, double timeout_s)
    : rank_(rank), world_(world) {
    CHECK(cudaSetDevice(device));
    ncclUniqueId id;
    const uint64_t nonce = launchNonce();
    if (rank == 0) {
        NCCL_TRY(ncclGetUniqueId(&id));
        rendezvousPublish(id_file, &id, sizeof(id), nonce);
    } else {
        // a record must not predate this rank's start by more than the time ranks may take to come up
        rendezvousWait(id_file, &id, sizeof(id), nonce, timeout_s, timeout_s);
    }
    ncclComm_t c;
    NCCL_TRY(ncclCommInitRank(&c, world, id, rank));
    comm_ = c;
    // ncclCommInitRank returns once every rank has joined, i.e. has read the record
    if (rank == 0) std::remove(id_file.c_str());
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
    if (comm_ && !aborted_) ncclCommDestroy(static_cast<ncclComm_t>(comm_));
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

void Communicator::reduceScatterAverage(float* grad, size_t n) {
    if (world_ <= 1 || n == 0) return;
    if (n % (size_t)world_) throw std::invalid_argument("reduceScatterAverage: size is not a multiple of the world size");
    cudaStream_t s = static_cast<cudaStream_t>(stream_);
    const size_t chunk = n / (size_t)world_;
    SM::Instance().streamWait(grad, s, true);
    NCCL_TRY(ncclReduceScatter(grad, grad + (size_t)rank_ * chunk, chunk, ncclFloat32, ncclAvg,
                               static_cast<ncclComm_t>(comm_), s));
    SM::Instance().recordData(grad, s);
}

void Communicator::allGather(float* data, size_t n) {
    if (world_ <= 1 || n == 0) return;
    if (n % (size_t)world_) throw std::invalid_argument("allGather: size is not a multiple of the world size");
    cudaStream_t s = static_cast<cudaStream_t>(stream_);
    const size_t chunk = n / (size_t)world_;
    SM::Instance().streamWait(data, s, true);
    NCCL_TRY(ncclAllGather(data + (size_t)rank_ * chunk, data, chunk, ncclFloat32, static_cast<ncclComm_t>(comm_), s));
    SM::Instance().recordData(data, s);
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

void Communicator::waitHealthy(double deadline_s) {
    if (world_ <= 1 || aborted_) return;
    cudaStream_t s = static_cast<cudaStream_t>(stream_);
    ncclComm_t c = static_cast<ncclComm_t>(comm_);
    CollectiveWatchdog w;
    w.deadline_s = deadline_s;
    w.poll = [&]() -> int {
        ncclResult_t state = ncclSuccess;
        const ncclResult_t q = ncclCommGetAsyncError(c, &state);
        if (q != ncclSuccess) return 100 + (int)q;
        if (state != ncclSuccess && state != ncclInProgress) return 100 + (int)state;
        const cudaError_t e = cudaStreamQuery(s);
        if (e == cudaSuccess) return 0;
        if (e == cudaErrorNotReady) return 1;
        return 1000 + (int)e;
    };
    w.abort = [&]() {
        ncclCommAbort(c);
        aborted_ = true;
    };
    const auto out = w.wait();
    if (out == CollectiveWatchdog::Failed)
        throw std::runtime_error("NCCL reported an asynchronous error (code " + std::to_string(w.last_code) +
                                 "); the communicator was aborted");
    if (out == CollectiveWatchdog::TimedOut)
        throw std::runtime_error("collectives did not finish within the host deadline; the communicator was aborted");
}

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

int nzb_dp_wait_healthy(void* comm, double deadline_s) {
    if (!comm) return dp_fail(NZB_ERR_BAD_ARG, "null communicator");
    try {
        static_cast<nz::dist::Communicator*>(comm)->waitHealthy(deadline_s > 0 ? deadline_s : 30.0);
    } catch (const std::exception& e) {
        return dp_fail(NZB_ERR_CUDA, e.what());
    }
    return NZB_OK;
}

int nzb_dp_rendezvous_publish(const char* file, const void* payload, size_t bytes, uint64_t nonce) {
    if (!file || !payload) return dp_fail(NZB_ERR_BAD_ARG, "null argument");
    try {
        nz::dist::rendezvousPublish(file, payload, bytes, nonce);
    } catch (const std::exception& e) {
        return dp_fail(NZB_ERR_CUDA, e.what());
    }
    return NZB_OK;
}

int nzb_dp_rendezvous_wait(const char* file, void* payload, size_t bytes, uint64_t nonce, double timeout_s,
                           double max_age_s) {
    if (!file || !payload) return dp_fail(NZB_ERR_BAD_ARG, "null argument");
    try {
        nz::dist::rendezvousWait(file, payload, bytes, nonce, timeout_s, max_age_s);
    } catch (const std::exception& e) {
        return dp_fail(NZB_ERR_CUDA, e.what());
    }
    return NZB_OK;
}

int nzb_dp_watchdog_run(const int* poll_script, int n, double deadline_s, int* polls_out, int* aborted_out) {
    if (!poll_script || n < 1) return dp_fail(NZB_ERR_BAD_ARG, "empty poll script");
    nz::dist::CollectiveWatchdog w;
    int i = 0, aborts = 0;
    w.deadline_s = deadline_s;
    w.poll = [&]() { return poll_script[i < n - 1 ? i++ : n - 1]; };  // the last entry repeats
    w.abort = [&]() { aborts++; };
    const int out = (int)w.wait();
    if (polls_out) *polls_out = w.polls;
    if (aborted_out) *aborted_out = aborts;
    return out;
}

int nzb_dp_finalize(void* comm) {
    delete static_cast<nz::dist::Communicator*>(comm);
    return NZB_OK;
}

}  // extern "C"
