// Error policy of the host layer. NeuZephyr's CHECK macro resets the device and throws
// (include/NeuZephyr/NeuZephyrCudaErrorHandling.cuh:62-118); on a shared GPU that is not
// acceptable, so here a failing CUDA or libnzb call throws nz::CudaException and leaves the
// device alone.
#pragma once
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include <nzb.h>

namespace nz {

class CudaException : public std::runtime_error {
public:
    CudaException(const std::string& what, const char* file, int line)
        : std::runtime_error(what + " (" + file + ":" + std::to_string(line) + ")") {}
};

}  // namespace nz

#define CHECK(call)                                                                      \
    do {                                                                                 \
        const cudaError_t nz_err_ = (call);                                              \
        if (nz_err_ != cudaSuccess)                                                      \
            throw ::nz::CudaException(cudaGetErrorString(nz_err_), __FILE__, __LINE__);  \
    } while (0)

#define NZB_CHECK(call)                                                               \
    do {                                                                              \
        const int nz_rc_ = (call);                                                    \
        if (nz_rc_ == NZB_ERR_BAD_ARG) throw std::invalid_argument(nzb_last_error_string()); \
        if (nz_rc_ != NZB_OK) throw ::nz::CudaException(nzb_last_error_string(), __FILE__, __LINE__); \
    } while (0)
