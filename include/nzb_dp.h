/*
 * nzb_dp.h -- data-parallel gradient exchange, C ABI. Exported by libneuzephyr_host.so (the
 * library that links NCCL); status codes are those of nzb.h.
 *
 * NeuZephyr has no multi-GPU path; these three calls are what a one-process-per-GPU launcher adds
 * around Model::update (src/Model.cu:20-23): every rank averages each parameter gradient with all
 * other ranks before the optimizer step, which makes a batch-sharded step equal to the full-batch
 * step. The C++ form of the same thing is nz::dist::Communicator / Model::setCommunicator.
 */
#ifndef NZB_DP_H_
#define NZB_DP_H_

#include "nzb.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Joins rank `rank` of `world` on CUDA device `device`. Rank 0 publishes the NCCL unique id through
 * the file `id_file` (a path every rank can read); the others wait for it, at most timeout_s seconds
 * (<= 0: 60 s). Collective: every rank must call it. */
NZB_API int nzb_dp_init(int rank, int world, const char* id_file, int device, double timeout_s, void** comm_out);

/* In-place average over all ranks of n floats at grad (device memory), queued on `stream`
 * (ncclAllReduce, ncclAvg). Order it after the kernels that write grad and before the optimizer
 * kernel, with stream order or events. Every rank must issue its calls in the same order. */
NZB_API int nzb_dp_allreduce_avg(void* comm, float* grad, size_t n, void* stream);

NZB_API int nzb_dp_world(void* comm, int* rank_out, int* world_out);
NZB_API int nzb_dp_finalize(void* comm);
NZB_API const char* nzb_dp_last_error_string(void);

#ifdef __cplusplus
}
#endif
#endif /* NZB_DP_H_ */
