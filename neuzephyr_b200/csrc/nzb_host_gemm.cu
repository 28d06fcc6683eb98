// nzb_gemm_host: C = op(A) * op(B) with all three matrices in HOST memory, as one pipelined call.
//
// Stands in for the sequence a NeuZephyr user writes around GEMMTensorCore
// (include/NeuZephyr/TensorOperations.cuh:1024-1028): Tensor::dataInject for both operands
// (src/Tensor.cu, a blocking cudaMemcpy each), the GEMM, Tensor::hostData for the result
// (another blocking copy). Those four steps run back to back there; here the left operand is
// cut into row blocks and three streams overlap them:
//   copy-in stream : B, then A block 0, A block 1, ...
//   caller's stream: stage B once; per block: stage A block, GEMM block
//   copy-out stream: C block i as soon as its GEMM is done
// PCIe is full duplex, so copy-out of block i runs under copy-in of block i+1 and the call is
// bound by the larger direction instead of their sum. Host buffers should be pinned; pageable
// memory still gives correct results, without the overlap.
#include <cuda_fp16.h>

#include <mutex>

#include "nzb_internal.h"

namespace nzb {

constexpr int kHostMaxBlocks = 16;

struct HostPipe {
    bool ready = false;
    cudaStream_t in = nullptr, out = nullptr;
    cudaEvent_t start = nullptr, b_in = nullptr, tail = nullptr;
    cudaEvent_t a_in[kHostMaxBlocks], c_done[kHostMaxBlocks];
};
static std::mutex g_pipe_mu;       // guards creation
static std::mutex g_enqueue_mu;    // one call at a time enqueues on a device's pipe (its events are reused)
static HostPipe g_pipes[64];

static int get_pipe(HostPipe** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return fail(NZB_ERR_NO_DEVICE, "no CUDA device is current");
    }
    std::lock_guard<std::mutex> lk(g_pipe_mu);
    HostPipe& p = g_pipes[dev];
    if (!p.ready) {
        NZB_CUDA_TRY(cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking));
        NZB_CUDA_TRY(cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking));
        NZB_CUDA_TRY(cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming));
        NZB_CUDA_TRY(cudaEventCreateWithFlags(&p.b_in, cudaEventDisableTiming));
        NZB_CUDA_TRY(cudaEventCreateWithFlags(&p.tail, cudaEventDisableTiming));
        for (int i = 0; i < kHostMaxBlocks; i++) {
            NZB_CUDA_TRY(cudaEventCreateWithFlags(&p.a_in[i], cudaEventDisableTiming));
            NZB_CUDA_TRY(cudaEventCreateWithFlags(&p.c_done[i], cudaEventDisableTiming));
        }
        p.ready = true;
    }
    *out = &p;
    return NZB_OK;
}

struct HostLayout {
    size_t a32, b32, c32, bias, stage, total;
};
static int host_layout(const nzb_gemm_desc* d, HostLayout* L) {
    if (!d) return fail(NZB_ERR_BAD_ARG, "descriptor is null");
    if (d->batch[0] != 1 || d->batch[1] != 1) return fail(NZB_ERR_UNSUPPORTED, "nzb_gemm_host takes one matrix product (batch extents 1)");
    if (d->transA) return fail(NZB_ERR_UNSUPPORTED, "nzb_gemm_host cuts A into row blocks: A must be stored M x K");
    if (d->accumulate) return fail(NZB_ERR_UNSUPPORTED, "nzb_gemm_host overwrites C");
    if (d->bias_mode == NZB_BIAS_MATRIX) return fail(NZB_ERR_UNSUPPORTED, "nzb_gemm_host takes a row or column bias");
    Plan pl;
    int rc = make_plan(d, &pl);
    if (rc != NZB_OK) return rc;
    const int64_t b_rows = d->transB ? d->N : d->K;
    L->a32 = (size_t)round_up(d->M * d->lda * 4, 256);
    L->b32 = (size_t)round_up(b_rows * d->ldb * 4, 256);
    L->c32 = (size_t)round_up(d->M * d->ldc * 4, 256);
    L->bias = (size_t)round_up((d->bias_mode == NZB_BIAS_ROW ? d->N : d->bias_mode == NZB_BIAS_COL ? d->M : 0) * 4, 256);
    L->stage = pl.a_bytes + pl.b_bytes;
    L->total = L->a32 + L->b32 + L->c32 + L->bias + L->stage;
    return NZB_OK;
}

}  // namespace nzb

using namespace nzb;

extern "C" {

int nzb_gemm_host_workspace_bytes(const nzb_gemm_desc* desc, size_t* bytes_out) {
    if (!bytes_out) return fail(NZB_ERR_BAD_ARG, "bytes_out is null");
    HostLayout L;
    int rc = host_layout(desc, &L);
    if (rc != NZB_OK) return rc;
    *bytes_out = L.total;
    return NZB_OK;
}

int nzb_gemm_host(const nzb_gemm_desc* desc, const float* hostA, const float* hostB, float* hostC, const float* host_bias,
                  void* workspace, size_t workspace_bytes, void* stream) {
    HostLayout L;
    int rc = host_layout(desc, &L);
    if (rc != NZB_OK) return rc;
    const nzb_gemm_desc& d = *desc;
    if (d.M == 0 || d.N == 0) return NZB_OK;
    if (d.K == 0) return fail(NZB_ERR_UNSUPPORTED, "K = 0 is not supported");
    if (!hostA || !hostB || !hostC) return fail(NZB_ERR_BAD_ARG, "A, B and C must be non-null");
    if (d.bias_mode != NZB_BIAS_NONE && !host_bias) return fail(NZB_ERR_BAD_ARG, "bias_mode set but bias is null");
    if (!workspace || workspace_bytes < L.total) return fail(NZB_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", L.total, workspace ? workspace_bytes : (size_t)0);
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(NZB_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    DeviceState* ds;
    rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    HostPipe* pp;
    rc = get_pipe(&pp);
    if (rc != NZB_OK) return rc;
    std::lock_guard<std::mutex> enqueue_lock(g_enqueue_mu);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint8_t* w = reinterpret_cast<uint8_t*>(workspace);
    float* A32 = reinterpret_cast<float*>(w);
    float* B32 = reinterpret_cast<float*>(w + L.a32);
    float* C32 = reinterpret_cast<float*>(w + L.a32 + L.b32);
    float* bias32 = reinterpret_cast<float*>(w + L.a32 + L.b32 + L.c32);
    uint8_t* stage = w + L.a32 + L.b32 + L.c32 + L.bias;

    // row blocks: multiples of 256 rows (one CTA-pair tile), at most kHostMaxBlocks of them
    int64_t rows = round_up((d.M + 7) / 8, 256);
    if (rows < 512) rows = 512;
    while ((d.M + rows - 1) / rows > kHostMaxBlocks) rows += 256;
    const int64_t nblk = (d.M + rows - 1) / rows;

    Plan pl;  // staging layout of the whole problem: B16 is shared, A16 is written block by block
    rc = make_plan(desc, &pl);
    if (rc != NZB_OK) return rc;
    __half* A16 = reinterpret_cast<__half*>(stage);
    __half* B16 = reinterpret_cast<__half*>(stage + pl.a_bytes);

    // everything queued on the caller's stream so far precedes the first copy
    NZB_CUDA_TRY(cudaEventRecord(pp->start, s));
    NZB_CUDA_TRY(cudaStreamWaitEvent(pp->in, pp->start, 0));
    NZB_CUDA_TRY(cudaStreamWaitEvent(pp->out, pp->start, 0));
    const int64_t b_rows = d.transB ? d.N : d.K, b_cols = d.transB ? d.K : d.N;
    NZB_CUDA_TRY(cudaMemcpy2DAsync(B32, (size_t)d.ldb * 4, hostB, (size_t)d.ldb * 4, (size_t)b_cols * 4, (size_t)b_rows,
                                   cudaMemcpyHostToDevice, pp->in));
    if (d.bias_mode != NZB_BIAS_NONE)
        NZB_CUDA_TRY(cudaMemcpyAsync(bias32, host_bias, (size_t)(d.bias_mode == NZB_BIAS_ROW ? d.N : d.M) * 4,
                                     cudaMemcpyHostToDevice, pp->in));
    NZB_CUDA_TRY(cudaEventRecord(pp->b_in, pp->in));
    for (int64_t b = 0; b < nblk; b++) {
        const int64_t r0 = b * rows, nr = d.M - r0 < rows ? d.M - r0 : rows;
        NZB_CUDA_TRY(cudaMemcpy2DAsync(A32 + r0 * d.lda, (size_t)d.lda * 4, hostA + r0 * d.lda, (size_t)d.lda * 4,
                                       (size_t)d.K * 4, (size_t)nr, cudaMemcpyHostToDevice, pp->in));
        NZB_CUDA_TRY(cudaEventRecord(pp->a_in[b], pp->in));
    }
    // B is staged once
    NZB_CUDA_TRY(cudaStreamWaitEvent(s, pp->b_in, 0));
    if (pl.g.b_mn)
        rc = launch_cast_on(ds->sm_count, B32, B16, d.K, d.N, d.ldb, pl.Np, 0, 1, 1, 0, 0, s);
    else
        rc = launch_cast_on(ds->sm_count, B32, B16, d.N, d.K, d.ldb, pl.Kp, d.transB ? 0 : 1, 1, 1, 0, 0, s);
    if (rc != NZB_OK) return rc;
    for (int64_t b = 0; b < nblk; b++) {
        const int64_t r0 = b * rows, nr = d.M - r0 < rows ? d.M - r0 : rows;
        NZB_CUDA_TRY(cudaStreamWaitEvent(s, pp->a_in[b], 0));
        __half* A16b = A16 + r0 * pl.Kp;
        rc = launch_cast_on(ds->sm_count, A32 + r0 * d.lda, A16b, nr, d.K, d.lda, pl.Kp, 0, 1, 1, 0, 0, s);
        if (rc != NZB_OK) return rc;
        GemmLaunch g = pl.g;
        g.A16 = A16b;
        g.B16 = B16;
        g.M = nr;
        g.C = C32 + r0 * d.ldc;
        g.bias = d.bias_mode == NZB_BIAS_NONE ? nullptr : (d.bias_mode == NZB_BIAS_COL ? bias32 + r0 : bias32);
        rc = launch_gemm_on(g, *ds, s);
        if (rc != NZB_OK) return rc;
        NZB_CUDA_TRY(cudaEventRecord(pp->c_done[b], s));
        NZB_CUDA_TRY(cudaStreamWaitEvent(pp->out, pp->c_done[b], 0));
        NZB_CUDA_TRY(cudaMemcpy2DAsync(hostC + r0 * d.ldc, (size_t)d.ldc * 4, C32 + r0 * d.ldc, (size_t)d.ldc * 4,
                                       (size_t)d.N * 4, (size_t)nr, cudaMemcpyDeviceToHost, pp->out));
    }
    // the caller's stream completes only when the last block of C has reached the host
    NZB_CUDA_TRY(cudaEventRecord(pp->tail, pp->out));
    NZB_CUDA_TRY(cudaStreamWaitEvent(s, pp->tail, 0));
    return NZB_OK;
}

}  // extern "C"
