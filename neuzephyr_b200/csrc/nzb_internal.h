// Host-side internals shared by the translation units of libnzb.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>
#include <cuda_fp16.h>

#include <atomic>

#include "../../include/nzb.h"

namespace nzb {

// Records the message returned by nzb_last_error_string() and passes the code through.
int fail(int code, const char* fmt, ...);

#define NZB_CUDA_TRY(expr)                                                                         \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return ::nzb::fail(NZB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                               __FILE__, __LINE__);                                                \
    } while (0)

// Per-device state created on first use: SM count, the mapped status word kernels write
// when a bounded wait expires, and the driver entry point for tensor-map encoding.
struct DeviceState {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0;
    int* status_host = nullptr;  // mapped, pinned
    int* status_dev = nullptr;   // device alias of status_host
};
int get_device_state(DeviceState** out);

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
int get_encode_tiled(EncodeTiledFn* out);

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device property of a kernel: `done` holds one
// bit per device ordinal (< 64) on which this kernel has been given `bytes` already. Callers racing on
// the first use both set the attribute, which is harmless.
int ensure_dynamic_smem(std::atomic<uint64_t>& done, const void* kernel, int bytes);

// Channels-last convolution (nzb_conv_nhwc.cu): stride 1, shared weights, 16 / 32 / 64k input channels.
struct NhwcPlan {
    bool ok;
    int Cb;             // channels per operand row block: 16, 32 or 64
    int BN;             // output channels per tile
    int stages;         // input rows the shared-memory ring holds
    int64_t w_bytes;    // staged weights
    int64_t per_image;  // channels-last fp16 copy of one image
    int64_t nchunk;     // images staged and convolved per pass
    int64_t bias_bytes; // transposed copy of a {Ho*Wo, R} bias matrix
};
// Cin, Hin, Win: the tensor the taps slide over; R: output channels; wN: weight sets (1 = shared).
NhwcPlan nhwc_plan(int64_t N, int64_t Cin, int64_t Hin, int64_t Win, int64_t R, int64_t Kh, int64_t Kw, int64_t stride,
                   int64_t Ho, int64_t Wo, int64_t wN);
// Y {N, R, Ho, Wo} (op)= conv(X {N, Cin, Hin, Win}, w); flip selects the backward-data form of the weights
// (w is always the layer's {1, 1, C*Kh*Kw, Cout} tensor). ws holds w_bytes + nchunk * per_image + bias_bytes.
struct ConvNhwcRun {
    const float* X;
    float* Y;
    const float* bias;
    const float* w;
    int64_t N, Cin, Hin, Win, R, Kh, Kw, pad, Ho, Wo;
    int64_t layerC, layerCout;  // the layer's own channel counts (weight tensor extents)
    int32_t bias_mode, accumulate, relu, flip;
};
int run_conv_nhwc(const ConvNhwcRun& r, const NhwcPlan& pl, void* ws, cudaStream_t stream);

// fp16 operand copy layout: rows x Kp halves, Kp = K rounded up to one 128-byte line.
constexpr int64_t kOperandKAlign = 64;

// Launchers (defined in the .cu files). All return NZB_* codes.
// Batched fp32 -> fp16 cast of `nmat` matrices; matrix b starts at in + b*in_batch_stride
// and out + b*rows*ld_out.
int launch_cast(const float* in, __half* out, int64_t rows, int64_t cols, int64_t ld_in, int64_t ld_out,
                int transpose, int64_t nmat0, int64_t nmat1, int64_t in_stride0, int64_t in_stride1,
                cudaStream_t stream);

struct GemmLaunch {
    // fp16 operands: A' [nA][M][Kp], B' [nB][N][Kp]
    const __half* A16;
    const __half* B16;
    int64_t nA, nB;  // number of matrices in each operand copy
    int64_t M, N, K, Kp;
    float* C;
    int64_t ldc;
    // batch grid; for each dimension d exactly one of out_e[d] / red_e[d] is > 1
    int32_t out_e[2], red_e[2];
    int64_t a_mul[2], b_mul[2];  // matrix-index multipliers of A' / B' along each batch dimension
    int64_t c_stride[2];         // element stride of C along each (output) batch dimension
    const float* bias;
    int32_t bias_mode;
    int64_t bias_ld;
    int32_t accumulate, relu;
    int32_t force_single_cta;  // keep the 128 x BN single-CTA kernel even where the CTA-pair kernel applies
    // MN-major copies: A' [nA][K][lda16] (contiguous along m) / B' [nB][K][ldb16] (contiguous along n)
    // instead of the K-major layout above; the leading dimension is a multiple of 8 halves.
    int32_t a_mn, b_mn;
    int64_t lda16, ldb16;
    // In-kernel staging (CTA-pair kernel only): when fuse_sync is non-null the copies A16 / B16 have
    // NOT been written yet; the kernel's converter warps round the fp32 sources into them, panel by
    // panel in the order the tiles need them, while the tensor cores work on finished panels.
    // fuse_sync points to kFuseSyncBytes of device memory zeroed on the launch stream.
    const float* A32;
    const float* B32;
    int64_t lda32, ldb32;
    unsigned* fuse_sync;
    // device scalar multiplied into every product before accumulate / bias (null: none)
    const float* alpha;
};
// Counters of the in-kernel staging: next chunk, then one finished-chunk count per 256-wide panel.
constexpr size_t kFuseSyncBytes = 16384;
constexpr int64_t kFuseMaxPanels = (int64_t)(kFuseSyncBytes / 4) - 8;
int launch_gemm(const GemmLaunch& g, cudaStream_t stream);
// True when launch_gemm_on() takes the CTA-pair kernel for this launch.
bool gemm_uses_pair_kernel(const GemmLaunch& g, int sm_count);
// Same launches with the device facts supplied by the caller instead of looked up
// (ds needs sm_count and status_dev only).
int launch_gemm_on(const GemmLaunch& g, const DeviceState& ds, cudaStream_t stream);
int launch_cast_on(int sm_count, const float* in, __half* out, int64_t rows, int64_t cols, int64_t ld_in,
                   int64_t ld_out, int transpose, int64_t nmat0, int64_t nmat1, int64_t in_stride0,
                   int64_t in_stride1, cudaStream_t stream);

// The same staging pass with an optional mask (same layout as `in`): elements whose mask value is
// not > 0 are staged as zero, which folds ReLU's backward into the operand copy.
int launch_cast_masked(int sm_count, const float* in, const float* mask, __half* out, int64_t rows, int64_t cols,
                       int64_t ld_in, int64_t ld_out, int transpose, int64_t nmat0, int64_t nmat1, int64_t in_stride0,
                       int64_t in_stride1, cudaStream_t stream);

// Resolved view of a descriptor (nzb_api.cu).
struct Plan {
    int64_t M, N, K, Kp;
    int64_t Mp, Np;  // leading dimensions of MN-major copies
    int64_t nA0, nA1, nB0, nB1;  // matrices in the fp16 copies along each batch dimension
    size_t a_bytes, b_bytes;
    bool fusable;  // one matrix product whose staging the CTA-pair kernel can do itself
    GemmLaunch g;
};
int make_plan(const nzb_gemm_desc* d, Plan* pl);
// Stages both fp32 operands of a planned GEMM as fp16 copies (two row-preserving casts; a
// transposing pass only for a K x N right operand with N <= 32) and fills pl->g.A16 / B16.
int stage_operands(Plan* pl, const nzb_gemm_desc* d, const float* A, const float* B, __half* A16, __half* B16,
                   int sm_count, cudaStream_t stream);

#ifdef __CUDACC__
// One Adam update (AdamKernel, src/OperationKernels.cu:753-766) with every rounding step spelled out, so
// that the per-tensor kernel and the multi-tensor kernel give bit-identical results whatever the compiler
// would otherwise contract. c1 = 1 - beta1^t, c2 = 1 - beta2^t. Returns the new weight, updates m and v.
__device__ __forceinline__ float adam_update(float p, float& m, float& v, float g, float lr, float beta1, float beta2,
                                             float eps, float c1, float c2) {
    m = __fmaf_rn(m, beta1, __fmul_rn(g, __fsub_rn(1.f, beta1)));
    v = __fmaf_rn(v, beta2, __fmul_rn(__fmul_rn(g, g), __fsub_rn(1.f, beta2)));
    const float step = __fdiv_rn(__fmul_rn(lr, __fdiv_rn(m, c1)), __fadd_rn(__fsqrt_rn(__fdiv_rn(v, c2)), eps));
    return __fsub_rn(p, step);
}
#endif

}  // namespace nzb
