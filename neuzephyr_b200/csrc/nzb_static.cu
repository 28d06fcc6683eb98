// nzb_gemm_static: the GEMM of nzb_gemm for callers that must not allocate.
//
// Who needs this: a host program whose device memory is entirely owned by another
// allocator (an inference server or training framework that reserved the whole GPU at
// start-up, so a cudaMalloc from a plug-in fails or fragments its pool), or a steady-state
// loop in which allocation calls are forbidden because they may synchronise the device.
// Such a caller can hand over inputs and outputs but has nowhere to get the fp16 staging
// scratch that nzb_gemm asks for. Here that scratch is a fixed array inside the library
// image, so this entry point calls no cudaMalloc, cudaFree, cudaHostAlloc or any other
// allocating routine -- not even the mapped status word the other entry points create.
//
// Cost and limits: every GPU on which this library is loaded holds
// NZB_STATIC_SCRATCH_BYTES (32 MiB) for the life of the process. Problems whose staged
// operands exceed it are rejected with NZB_ERR_WORKSPACE. All calls share the one array and it keeps the
// previous call's contents; the staging kernels rewrite every byte the GEMM reads
// (including the zero fill of the K padding), so nothing has to be cleared, but two calls
// that overlap on the GPU (different streams, no ordering between them) race on it.
// A bounded device-side wait that expires on this path is recorded in a device-resident
// word of the library image (not in the mapped word nzb_device_status reads);
// nzb_gemm_static_status / nzb_gemm_static_status_reset read and clear it with plain
// stream-ordered copies, so the no-allocation property holds for them too.
#include <cuda_fp16.h>

#include <mutex>

#include "nzb_internal.h"

namespace nzb {

constexpr size_t kStaticScratchBytes = NZB_STATIC_SCRATCH_BYTES;

// File-scope device arrays. In host code these names are host-side stand-ins, not device
// addresses: the device addresses are looked up once per device by static_setup().
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ int g_static_status[4];

struct StaticState {
    bool ready = false;
    void* scratch = nullptr;  // device address of g_static_scratch on this device
    int* status = nullptr;    // device address of g_static_status on this device
    int sm_count = 0;
};
static StaticState g_static[64];
static std::mutex g_static_mu;

// Once per device, with that device current.
static int static_setup(StaticState** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return fail(NZB_ERR_NO_DEVICE, "no CUDA device is current");
    }
    std::lock_guard<std::mutex> lk(g_static_mu);
    StaticState& s = g_static[dev];
    if (!s.ready) {
        int major = 0, sms = 0;
        NZB_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        NZB_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (major != 10) return fail(NZB_ERR_NO_DEVICE, "device %d is not sm_100; this library holds sm_100a code only", dev);
        void* p = nullptr;
        NZB_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        void* st = nullptr;
        NZB_CUDA_TRY(cudaGetSymbolAddress(&st, g_static_status));
        if (!p || !st || (reinterpret_cast<uintptr_t>(p) & 255)) return fail(NZB_ERR_CUDA, "static scratch address lookup returned an unusable pointer");
        s.scratch = p;
        s.status = static_cast<int*>(st);
        s.sm_count = sms;
        s.ready = true;
    }
    *out = &s;
    return NZB_OK;
}

}  // namespace nzb

using namespace nzb;

extern "C" {

int nzb_gemm_static(const nzb_gemm_desc* desc, const float* A, const float* B, float* C, const float* bias,
                    void* stream) {
    Plan pl;
    int rc = make_plan(desc, &pl);
    if (rc != NZB_OK) return rc;
    if (desc->M == 0 || desc->N == 0) return NZB_OK;
    if (!A || !B || !C) return fail(NZB_ERR_BAD_ARG, "A, B and C must be non-null");
    if (desc->bias_mode != NZB_BIAS_NONE && !bias) return fail(NZB_ERR_BAD_ARG, "bias_mode set but bias is null");
    if (desc->K == 0) return fail(NZB_ERR_UNSUPPORTED, "K = 0 is not supported");
    const size_t need = pl.a_bytes + pl.b_bytes;
    if (need > kStaticScratchBytes)
        return fail(NZB_ERR_WORKSPACE,
                    "nzb_gemm_static: staged operands need %zu bytes, the built-in scratch holds %zu; "
                    "use nzb_gemm with a caller-provided workspace", need, kStaticScratchBytes);
    StaticState* st;
    rc = static_setup(&st);  // first call on a device looks up the array's device address
    if (rc != NZB_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    __half* A16 = reinterpret_cast<__half*>(st->scratch);
    __half* B16 = reinterpret_cast<__half*>(static_cast<unsigned char*>(st->scratch) + pl.a_bytes);
    rc = stage_operands(&pl, desc, A, B, A16, B16, st->sm_count, s);
    if (rc != NZB_OK) return rc;
    DeviceState ds;
    ds.sm_count = st->sm_count;
    ds.status_dev = st->status;
    pl.g.C = C;
    pl.g.bias = bias;
    return launch_gemm_on(pl.g, ds, s);
}

int nzb_gemm_static_status(int* status_out, void* stream) {
    if (!status_out) return fail(NZB_ERR_BAD_ARG, "status_out is null");
    StaticState* st;
    int rc = static_setup(&st);
    if (rc != NZB_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // ordered after the work already queued on `stream`; the host waits for the copy only
    NZB_CUDA_TRY(cudaMemcpyAsync(status_out, st->status, sizeof(int), cudaMemcpyDeviceToHost, s));
    NZB_CUDA_TRY(cudaStreamSynchronize(s));
    return NZB_OK;
}

int nzb_gemm_static_status_reset(void* stream) {
    StaticState* st;
    int rc = static_setup(&st);
    if (rc != NZB_OK) return rc;
    NZB_CUDA_TRY(cudaMemsetAsync(st->status, 0, sizeof(int), static_cast<cudaStream_t>(stream)));
    return NZB_OK;
}

}  // extern "C"
