// nz::dist::Communicator: batch-sharded data parallelism over NCCL, one process per GPU.
// NeuZephyr itself is single-GPU; this is the layer that lets Model::update average the
// parameter gradients of all ranks (ncclAllReduce, ncclAvg) right before the optimizer step,
// submitted through StreamManager like any other operation: the all-reduce waits for the
// gradient's pending writers and publishes a writer event on it.
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <string>

namespace nz::dist {

// File rendezvous used to hand the NCCL unique id from rank 0 to the other ranks. A record carries
// a magic word, the launcher's nonce and its creation time, so that a file left behind by an earlier
// or crashed run is never taken for this run's: readers ignore records whose nonce differs or that
// were written more than `max_age_s` before the reader started waiting. The writer removes any old
// file first and publishes with a rename, so a reader never sees a partial record. Host-only code.
void rendezvousPublish(const std::string& file, const void* payload, size_t bytes, uint64_t nonce);
// Blocks until a valid record appears; throws std::runtime_error("timed out ...") after timeout_s.
void rendezvousWait(const std::string& file, void* payload, size_t bytes, uint64_t nonce, double timeout_s,
                    double max_age_s);
// Nonce of this launch: NZ_DP_NONCE if set, else a hash of MASTER_ADDR, MASTER_PORT and
// TORCHELASTIC_RUN_ID (equal on all ranks of one launch).
uint64_t launchNonce();

// Watches a collective that has been queued: polls its state until it is done, reports an error, or
// a host deadline passes; on error or deadline it calls `abort` once so that no rank stays blocked in
// a collective a peer never joined. poll() returns 0 = finished, 1 = in progress, anything else = the
// failing code (NCCL: ncclCommGetAsyncError + stream query; tests: a scripted sequence).
struct CollectiveWatchdog {
    enum Outcome { Done = 0, Failed = 1, TimedOut = 2 };
    std::function<int()> poll;
    std::function<void()> abort;
    double deadline_s = 30.0;
    double poll_interval_s = 0.001;
    int last_code = 0;
    int polls = 0;
    bool aborted = false;
    Outcome wait();
};

class Communicator {
public:
    // rank / world size / rendezvous file: rank 0 writes the NCCL unique id to `id_file`, the
    // others wait for it (bounded by timeout_s). device = CUDA device of this process.
    Communicator(int rank, int world, const std::string& id_file, int device, double timeout_s = 60.0);
    // reads RANK, WORLD_SIZE, LOCAL_RANK and NZ_DP_ID_FILE (default /tmp/nz_dp_<MASTER_PORT>.id)
    static Communicator* fromEnvironment();
    ~Communicator();
    int rank() const { return rank_; }
    int world() const { return world_; }
    // in-place average over all ranks of n floats at `grad` (device memory)
    void allReduceAverage(float* grad, size_t n);
    // Sharded form of the same exchange: rank r receives the average of elements [r*n/world, (r+1)*n/world)
    // in place (ncclReduceScatter; the rest of the buffer keeps this rank's own values), and the inverse,
    // which fills every rank's buffer from the slices the ranks own (ncclAllGather). n must be a
    // multiple of the world size. Ordered through the stream manager like allReduceAverage.
    void reduceScatterAverage(float* grad, size_t n);
    void allGather(float* data, size_t n);
    // the same collective on a stream the caller orders itself (no StreamManager bookkeeping)
    void allReduceAverageOn(float* grad, size_t n, void* cuda_stream);
    // in-place sum of a small host-visible value (used for reporting the loss)
    float allReduceSumHost(float v);
    void barrier();
    // Host-side health check of the communicator: waits (at most deadline_s) for everything queued on
    // the communication stream while polling ncclCommGetAsyncError; on an asynchronous error or when
    // the deadline passes it aborts the communicator (ncclCommAbort) and throws, instead of leaving
    // this rank blocked in a collective that a failed peer never joins.
    void waitHealthy(double deadline_s = 30.0);
    bool aborted() const { return aborted_; }

private:
    int rank_, world_;
    void* comm_ = nullptr;    // ncclComm_t
    void* stream_ = nullptr;  // dedicated communication stream
    float* scalar_ = nullptr;
    bool aborted_ = false;
};

}  // namespace nz::dist
