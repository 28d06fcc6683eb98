// extern "C" entry points of libnzb: argument validation, workspace carving and the
// mapping from NeuZephyr's 4-D shapes to the kernel launch description.
#include <cuda_fp16.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "nzb_internal.h"

namespace nzb {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

static std::mutex g_mu;
static DeviceState g_states[64];

int get_device_state(DeviceState** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return fail(NZB_ERR_NO_DEVICE, "no CUDA device is current");
    }
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = g_states[dev];
    if (s.device != dev) {
        cudaDeviceProp prop;
        NZB_CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
        if (prop.major != 10) return fail(NZB_ERR_NO_DEVICE, "device %d is sm_%d%d; this library holds sm_100a code only", dev, prop.major, prop.minor);
        int* h = nullptr;
        NZB_CUDA_TRY(cudaHostAlloc(&h, sizeof(int) * 16, cudaHostAllocMapped));
        for (int i = 0; i < 16; i++) h[i] = 0;
        int* d = nullptr;
        NZB_CUDA_TRY(cudaHostGetDevicePointer(&d, h, 0));
        s.sm_count = prop.multiProcessorCount;
        s.cc_major = prop.major;
        s.status_host = h;
        s.status_dev = d;
        s.device = dev;
    }
    *out = &s;
    return NZB_OK;
}

int ensure_dynamic_smem(std::atomic<uint64_t>& done, const void* kernel, int bytes) {
    int dev = -1;
    NZB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(NZB_ERR_NO_DEVICE, "device ordinal %d is outside 0..63", dev);
    const uint64_t bit = 1ull << dev;
    if (done.load(std::memory_order_acquire) & bit) return NZB_OK;
    NZB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done.fetch_or(bit, std::memory_order_release);
    return NZB_OK;
}

int get_encode_tiled(EncodeTiledFn* out) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        NZB_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !p) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    *out = fn;
    return NZB_OK;
}

int make_plan(const nzb_gemm_desc* d, Plan* pl) {
    if (!d) return fail(NZB_ERR_BAD_ARG, "descriptor is null");
    if (d->M < 0 || d->N < 0 || d->K < 0) return fail(NZB_ERR_BAD_ARG, "negative extent");
    if (d->batch[0] < 1 || d->batch[1] < 1) return fail(NZB_ERR_BAD_ARG, "batch extents must be >= 1");
    const int64_t a_rows = d->transA ? d->K : d->M, a_cols = d->transA ? d->M : d->K;
    const int64_t b_rows = d->transB ? d->N : d->K, b_cols = d->transB ? d->K : d->N;
    (void)a_rows; (void)b_rows;
    if (d->lda < a_cols || d->ldb < b_cols || d->ldc < d->N) return fail(NZB_ERR_BAD_ARG, "leading dimension smaller than the row length");
    if (d->bias_mode < NZB_BIAS_NONE || d->bias_mode > NZB_BIAS_MATRIX) return fail(NZB_ERR_BAD_ARG, "unknown bias mode");
    if (d->bias_mode == NZB_BIAS_MATRIX && d->bias_ld < d->N) return fail(NZB_ERR_BAD_ARG, "bias_ld smaller than N");
    pl->M = d->M; pl->N = d->N; pl->K = d->K;
    pl->Kp = round_up(d->K > 0 ? d->K : 1, kOperandKAlign);
    const int64_t e0 = d->batch[0], e1 = d->batch[1];
    pl->nA0 = (e0 > 1 && d->strideA[0] != 0) ? e0 : 1;
    pl->nA1 = (e1 > 1 && d->strideA[1] != 0) ? e1 : 1;
    pl->nB0 = (e0 > 1 && d->strideB[0] != 0) ? e0 : 1;
    pl->nB1 = (e1 > 1 && d->strideB[1] != 0) ? e1 : 1;
    pl->Mp = round_up(d->M > 0 ? d->M : 1, kOperandKAlign);
    pl->Np = round_up(d->N > 0 ? d->N : 1, kOperandKAlign);
    GemmLaunch& g = pl->g;
    g = GemmLaunch{};
    // A stored K x M and B stored K x N keep their layout (MN-major copies); a narrow right
    // operand is transposed instead, because an MN-major tile is at least 64 columns wide.
    g.a_mn = d->transA ? 1 : 0;
    g.b_mn = (!d->transB && d->N > 32) ? 1 : 0;
    g.lda16 = pl->Mp;
    g.ldb16 = pl->Np;
    pl->a_bytes = (size_t)round_up(pl->nA0 * pl->nA1 * (g.a_mn ? d->K * pl->Mp : pl->M * pl->Kp) * 2, 256);
    pl->b_bytes = (size_t)round_up(pl->nB0 * pl->nB1 * (g.b_mn ? d->K * pl->Np : pl->N * pl->Kp) * 2, 256);
    g.nA = pl->nA0 * pl->nA1;
    g.nB = pl->nB0 * pl->nB1;
    g.M = d->M; g.N = d->N; g.K = d->K; g.Kp = pl->Kp;
    g.ldc = d->ldc;
    const int64_t ext[2] = {e0, e1};
    for (int k = 0; k < 2; k++) {
        const bool reduce = ext[k] > 1 && d->strideC[k] == 0;
        g.out_e[k] = reduce ? 1 : (int32_t)ext[k];
        g.red_e[k] = reduce ? (int32_t)ext[k] : 1;
        g.c_stride[k] = reduce ? 0 : d->strideC[k];
    }
    g.a_mul[0] = pl->nA0 > 1 ? pl->nA1 : 0;
    g.a_mul[1] = pl->nA1 > 1 ? 1 : 0;
    g.b_mul[0] = pl->nB0 > 1 ? pl->nB1 : 0;
    g.b_mul[1] = pl->nB1 > 1 ? 1 : 0;
    g.bias_mode = d->bias_mode;
    g.bias_ld = d->bias_ld;
    g.accumulate = d->accumulate ? 1 : 0;
    g.relu = d->relu ? 1 : 0;
    // One matrix product with float4-aligned rows: the CTA-pair kernel's converter warps can stage the
    // operands themselves (pointer alignment and the kernel choice are checked at launch).
    pl->fusable = e0 == 1 && e1 == 1 && d->M % 4 == 0 && d->N % 4 == 0 && d->K % 4 == 0 && d->lda % 4 == 0 &&
                  d->ldb % 4 == 0 && (g.b_mn || d->transB) &&
                  (pl->M + 255) / 256 + (pl->N + 255) / 256 <= kFuseMaxPanels &&
                  // enough tiles for two rounds of the persistent grid: below that the wait for the first
                  // panels is a visible share of the run and three small kernels are as fast
                  ((pl->M + 255) / 256) * ((pl->N + 255) / 256) >= 148;
    return NZB_OK;
}

int stage_operands(Plan* pl, const nzb_gemm_desc* d, const float* A, const float* B, __half* A16, __half* B16,
                   int sm_count, cudaStream_t stream) {
    GemmLaunch& g = pl->g;
    int rc;
    if (g.a_mn)  // stored K x M: keep rows = k
        rc = launch_cast_on(sm_count, A, A16, d->K, d->M, d->lda, pl->Mp, 0, pl->nA0, pl->nA1, d->strideA[0],
                            d->strideA[1], stream);
    else  // stored M x K
        rc = launch_cast_on(sm_count, A, A16, d->M, d->K, d->lda, pl->Kp, 0, pl->nA0, pl->nA1, d->strideA[0],
                            d->strideA[1], stream);
    if (rc != NZB_OK) return rc;
    if (g.b_mn)  // stored K x N: keep rows = k
        rc = launch_cast_on(sm_count, B, B16, d->K, d->N, d->ldb, pl->Np, 0, pl->nB0, pl->nB1, d->strideB[0],
                            d->strideB[1], stream);
    else  // stored N x K: plain; stored K x N with few columns: transpose into N rows of K
        rc = launch_cast_on(sm_count, B, B16, d->N, d->K, d->ldb, pl->Kp, d->transB ? 0 : 1, pl->nB0, pl->nB1,
                            d->strideB[0], d->strideB[1], stream);
    if (rc != NZB_OK) return rc;
    g.A16 = A16;
    g.B16 = B16;
    return NZB_OK;
}

// NZB_FUSED_STAGING=0 in the environment keeps the separate staging kernels (read once per process).
static bool fused_staging_enabled() {
    static const bool on = [] {
        const char* e = getenv("NZB_FUSED_STAGING");
        return !(e && e[0] == '0');
    }();
    return on;
}

static int run_gemm(const nzb_gemm_desc* d, const float* A, const float* B, float* C, const float* bias, void* ws,
                    size_t ws_bytes, cudaStream_t stream) {
    Plan pl;
    int rc = make_plan(d, &pl);
    if (rc != NZB_OK) return rc;
    if (d->M == 0 || d->N == 0) return NZB_OK;
    if (!A || !B || !C) return fail(NZB_ERR_BAD_ARG, "A, B and C must be non-null");
    if (d->bias_mode != NZB_BIAS_NONE && !bias) return fail(NZB_ERR_BAD_ARG, "bias_mode set but bias is null");
    if (d->K == 0) return fail(NZB_ERR_UNSUPPORTED, "K = 0 is not supported");
    const size_t need = pl.a_bytes + pl.b_bytes + kFuseSyncBytes;
    if (!ws || ws_bytes < need) return fail(NZB_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, ws ? ws_bytes : (size_t)0);
    if (reinterpret_cast<uintptr_t>(ws) & 255) return fail(NZB_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    __half* A16 = reinterpret_cast<__half*>(ws);
    __half* B16 = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(ws) + pl.a_bytes);
    DeviceState* ds;
    rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    pl.g.C = C;
    pl.g.bias = bias;
    const bool aligned = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0;
    if (pl.fusable && aligned && fused_staging_enabled() && gemm_uses_pair_kernel(pl.g, ds->sm_count)) {
        // one kernel: its converter warps write the fp16 copies while its tensor-core warps consume them
        unsigned* sync = reinterpret_cast<unsigned*>(reinterpret_cast<uint8_t*>(ws) + pl.a_bytes + pl.b_bytes);
        const size_t used = 4 * (size_t)(8 + (pl.M + 255) / 256 + (pl.N + 255) / 256);
        NZB_CUDA_TRY(cudaMemsetAsync(sync, 0, used, stream));
        pl.g.A16 = A16;
        pl.g.B16 = B16;
        pl.g.A32 = A;
        pl.g.B32 = B;
        pl.g.lda32 = d->lda;
        pl.g.ldb32 = d->ldb;
        pl.g.fuse_sync = sync;
        return launch_gemm(pl.g, stream);
    }
    rc = stage_operands(&pl, d, A, B, A16, B16, ds->sm_count, stream);
    if (rc != NZB_OK) return rc;
    return launch_gemm(pl.g, stream);
}

// NeuZephyr 4-D shapes -> descriptor (TensorCoreGEMMParallel / GEMMBackwardParallel rules).
static int desc_from_shapes(const int64_t* sa, const int64_t* sb, const int64_t* sc, int backward, nzb_gemm_desc* d) {
    if (!sa || !sb || !sc) return fail(NZB_ERR_BAD_ARG, "shape pointer is null");
    for (int i = 0; i < 4; i++)
        if (sa[i] < 0 || sb[i] < 0 || sc[i] < 0) return fail(NZB_ERR_BAD_ARG, "negative extent");
    *d = nzb_gemm_desc{};
    d->M = sa[2]; d->K = sa[3]; d->N = sb[3];
    if (sb[2] != d->K) return fail(NZB_ERR_BAD_ARG, "A.W (%lld) != B.H (%lld)", (long long)sa[3], (long long)sb[2]);
    if (sc[2] != d->M || sc[3] != d->N) return fail(NZB_ERR_BAD_ARG, "C matrix extent does not match A.H x B.W");
    d->lda = d->K; d->ldb = d->N; d->ldc = d->N;
    for (int k = 0; k < 2; k++) {
        const int64_t a = sa[k], b = sb[k], c = sc[k];
        const int64_t e = a > b ? a : b;
        if (a < 1 || b < 1 || c < 1) return fail(NZB_ERR_BAD_ARG, "batch extents must be >= 1");
        if ((a != e && a != 1) || (b != e && b != 1)) return fail(NZB_ERR_BAD_ARG, "batch extents are not broadcast compatible");
        if (backward ? (c != e && c != 1) : (c != e)) return fail(NZB_ERR_BAD_ARG, "C batch extent does not match the operands");
        if (e > INT32_MAX) return fail(NZB_ERR_UNSUPPORTED, "batch extent exceeds 2^31");
        d->batch[k] = (int32_t)e;
    }
    // contiguous strides {C*H*W, H*W}; extent-1 dimensions broadcast (src/OperationKernels.cu:978-986)
    d->strideA[0] = sa[0] > 1 ? sa[1] * d->M * d->K : 0;
    d->strideA[1] = sa[1] > 1 ? d->M * d->K : 0;
    d->strideB[0] = sb[0] > 1 ? sb[1] * d->K * d->N : 0;
    d->strideB[1] = sb[1] > 1 ? d->K * d->N : 0;
    d->strideC[0] = sc[0] > 1 ? sc[1] * d->M * d->N : 0;
    d->strideC[1] = sc[1] > 1 ? d->M * d->N : 0;
    d->accumulate = backward ? 1 : 0;
    return NZB_OK;
}

}  // namespace nzb

using namespace nzb;

extern "C" {

int nzb_version(void) { return 100; }

const char* nzb_last_error_string(void) { return g_err; }

int nzb_device_status(int* status_out) {
    if (!status_out) return fail(NZB_ERR_BAD_ARG, "status_out is null");
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    *status_out = *reinterpret_cast<volatile int*>(ds->status_host);
    return NZB_OK;
}

int nzb_device_status_reset(void) {
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    *reinterpret_cast<volatile int*>(ds->status_host) = 0;
    return NZB_OK;
}

int nzb_gemm_workspace_bytes(const nzb_gemm_desc* desc, size_t* bytes_out) {
    if (!bytes_out) return fail(NZB_ERR_BAD_ARG, "bytes_out is null");
    Plan pl;
    int rc = make_plan(desc, &pl);
    if (rc != NZB_OK) return rc;
    *bytes_out = pl.a_bytes + pl.b_bytes + kFuseSyncBytes;
    return NZB_OK;
}

int nzb_gemm_kernel_launches(const nzb_gemm_desc* desc, const float* A, const float* B, int* launches_out) {
    if (!launches_out) return fail(NZB_ERR_BAD_ARG, "launches_out is null");
    Plan pl;
    int rc = make_plan(desc, &pl);
    if (rc != NZB_OK) return rc;
    DeviceState* ds;
    rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    const bool aligned = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0;
    const bool fused = pl.fusable && aligned && fused_staging_enabled() && gemm_uses_pair_kernel(pl.g, ds->sm_count);
    *launches_out = (desc->M == 0 || desc->N == 0) ? 0 : (fused ? 1 : 3);
    return NZB_OK;
}

int nzb_gemm(const nzb_gemm_desc* desc, const float* A, const float* B, float* C, const float* bias, void* workspace,
             size_t workspace_bytes, void* stream) {
    return run_gemm(desc, A, B, C, bias, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int nzb_gemm_f16(const nzb_gemm_desc* desc, const void* A16, const void* B16, int64_t ldk, float* C,
                 const float* bias, void* stream) {
    if (!desc) return fail(NZB_ERR_BAD_ARG, "descriptor is null");
    nzb_gemm_desc d = *desc;
    d.transA = 0; d.transB = 1; d.lda = d.K; d.ldb = d.K;  // layout fields are not used on this path
    Plan pl;
    int rc = make_plan(&d, &pl);
    if (rc != NZB_OK) return rc;
    if (d.M == 0 || d.N == 0) return NZB_OK;
    if (!A16 || !B16 || !C) return fail(NZB_ERR_BAD_ARG, "A16, B16 and C must be non-null");
    if (d.bias_mode != NZB_BIAS_NONE && !bias) return fail(NZB_ERR_BAD_ARG, "bias_mode set but bias is null");
    if (ldk < d.K || ldk % 8 != 0) return fail(NZB_ERR_BAD_ARG, "ldk must be >= K and a multiple of 8");
    if ((reinterpret_cast<uintptr_t>(A16) | reinterpret_cast<uintptr_t>(B16)) & 15) return fail(NZB_ERR_BAD_ARG, "fp16 operands must be 16-byte aligned");
    pl.g.Kp = ldk;
    pl.g.a_mn = pl.g.b_mn = 0;  // this entry point takes K-major copies
    pl.g.A16 = reinterpret_cast<const __half*>(A16);
    pl.g.B16 = reinterpret_cast<const __half*>(B16);
    pl.g.C = C;
    pl.g.bias = bias;
    return launch_gemm(pl.g, static_cast<cudaStream_t>(stream));
}

int nzb_tensorcore_gemm_workspace_bytes(const int64_t shapeA[4], const int64_t shapeB[4], const int64_t shapeC[4],
                                        size_t* bytes_out) {
    nzb_gemm_desc d;
    // the backward form accepts a superset of C shapes and needs the same scratch
    int rc = desc_from_shapes(shapeA, shapeB, shapeC, 1, &d);
    if (rc != NZB_OK) return rc;
    return nzb_gemm_workspace_bytes(&d, bytes_out);
}

int nzb_tensorcore_gemm(const float* A, const float* B, float* C, const int64_t shapeA[4], const int64_t shapeB[4],
                        const int64_t shapeC[4], void* workspace, size_t workspace_bytes, void* stream) {
    nzb_gemm_desc d;
    int rc = desc_from_shapes(shapeA, shapeB, shapeC, 0, &d);
    if (rc != NZB_OK) return rc;
    return run_gemm(&d, A, B, C, nullptr, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int nzb_gemm_backward(const float* A, const float* B, float* C, const int64_t shapeA[4], const int64_t shapeB[4],
                      const int64_t shapeC[4], void* workspace, size_t workspace_bytes, void* stream) {
    nzb_gemm_desc d;
    int rc = desc_from_shapes(shapeA, shapeB, shapeC, 1, &d);
    if (rc != NZB_OK) return rc;
    return run_gemm(&d, A, B, C, nullptr, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int nzb_cast_f32_f16(const float* in, void* out_f16, int64_t rows, int64_t cols, int64_t ld_in, int64_t ld_out,
                     int transpose, void* stream) {
    if (!in || !out_f16) return fail(NZB_ERR_BAD_ARG, "null pointer");
    if (rows < 0 || cols < 0) return fail(NZB_ERR_BAD_ARG, "negative extent");
    if (reinterpret_cast<uintptr_t>(out_f16) & 15) return fail(NZB_ERR_BAD_ARG, "fp16 destination must be 16-byte aligned");
    return launch_cast(in, reinterpret_cast<__half*>(out_f16), rows, cols, ld_in, ld_out, transpose, 1, 1, 0, 0,
                       static_cast<cudaStream_t>(stream));
}

}  // extern "C"
