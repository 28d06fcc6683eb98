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
#include <stdint.h>

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

/* Host-side health check: waits, at most deadline_s seconds (<= 0: 30 s), for the collectives queued
 * on the communicator's own stream while polling ncclCommGetAsyncError. On an asynchronous NCCL error,
 * or when the deadline passes (a peer died or never joined), it calls ncclCommAbort and returns
 * NZB_ERR_CUDA with the reason in nzb_dp_last_error_string(); the communicator must then be finalized. */
NZB_API int nzb_dp_wait_healthy(void* comm, double deadline_s);

/* The file rendezvous behind nzb_dp_init, host-only (no GPU, no NCCL). A record is {magic, nonce,
 * creation time, payload}; publish removes any older file and renames the new one into place; wait
 * accepts only a record with the same nonce that is not older than max_age_s relative to the moment
 * the wait began, and gives up after timeout_s with "timed out" in nzb_dp_last_error_string(). */
NZB_API int nzb_dp_rendezvous_publish(const char* file, const void* payload, size_t bytes, uint64_t nonce);
NZB_API int nzb_dp_rendezvous_wait(const char* file, void* payload, size_t bytes, uint64_t nonce, double timeout_s,
                                   double max_age_s);

/* Runs the watchdog logic of nzb_dp_wait_healthy on a scripted sequence of poll results instead of
 * NCCL (0 = finished, 1 = in progress, other = error code; the last entry repeats): returns 0 done,
 * 1 failed, 2 deadline passed; *aborted_out counts calls of the abort hook. For tests on hosts
 * without GPUs. */
NZB_API int nzb_dp_watchdog_run(const int* poll_script, int n, double deadline_s, int* polls_out, int* aborted_out);

NZB_API int nzb_dp_world(void* comm, int* rank_out, int* world_out);
NZB_API int nzb_dp_finalize(void* comm);
NZB_API const char* nzb_dp_last_error_string(void);

#ifdef __cplusplus
}
#endif
#endif /* NZB_DP_H_ */
