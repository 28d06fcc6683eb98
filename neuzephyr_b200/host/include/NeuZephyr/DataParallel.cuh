// nz::dist::Communicator: batch-sharded data parallelism over NCCL, one process per GPU.
// NeuZephyr itself is single-GPU; this is the layer that lets Model::update average the
// parameter gradients of all ranks (ncclAllReduce, ncclAvg) right before the optimizer step,
// submitted through StreamManager like any other operation: the all-reduce waits for the
// gradient's pending writers and publishes a writer event on it.
#pragma once
#include <cstddef>
#include <string>

namespace nz::dist {

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
    // the same collective on a stream the caller orders itself (no StreamManager bookkeeping)
    void allReduceAverageOn(float* grad, size_t n, void* cuda_stream);
    // in-place sum of a small host-visible value (used for reporting the loss)
    float allReduceSumHost(float v);
    void barrier();

private:
    int rank_, world_;
    void* comm_ = nullptr;    // ncclComm_t
    void* stream_ = nullptr;  // dedicated communication stream
    float* scalar_ = nullptr;
};

}  // namespace nz::dist
