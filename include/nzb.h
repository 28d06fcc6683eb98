/*
 * nzb.h - C ABI of the B200 (sm_100a) kernel library behind NeuZephyr's dense-contraction path.
 *
 * Every entry point is asynchronous on the stream it is given, never synchronises the
 * host, never resets the device and reports failure through its return code.
 * Pointers are device pointers to contiguous fp32 storage unless stated otherwise.
 * File:line citations name the NeuZephyr interface an entry point stands in for.
 */
#ifndef NZB_H
#define NZB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define NZB_API __declspec(dllexport)
#else
#define NZB_API __attribute__((visibility("default")))
#endif

/* ---- status codes ------------------------------------------------------ */
enum {
    NZB_OK = 0,
    NZB_ERR_BAD_ARG = 1,        /* null pointer, negative extent, inconsistent shapes */
    NZB_ERR_UNSUPPORTED = 2,    /* shape outside what the kernels handle */
    NZB_ERR_WORKSPACE = 3,      /* workspace missing or smaller than nzb_*_workspace_bytes() */
    NZB_ERR_CUDA = 4,           /* a CUDA runtime/driver call failed; see nzb_last_error_string() */
    NZB_ERR_DEVICE_TIMEOUT = 5, /* a bounded device-side wait expired (reported by nzb_device_status) */
    NZB_ERR_NO_DEVICE = 6       /* no sm_100 device is current */
};

enum { NZB_BIAS_NONE = 0, NZB_BIAS_ROW = 1, NZB_BIAS_COL = 2, NZB_BIAS_MATRIX = 3 };

/*
 * General descriptor: C[b] (op)= op(A[b]) * op(B[b]) over a two-dimensional batch grid
 * (the N and C extents of NeuZephyr's 4-D tensors). fp32 in memory, operands rounded to
 * fp16 (round-to-nearest-even) for the tensor cores, fp32 accumulation.
 *
 *   op(A) is M x K, op(B) is K x N, C is M x N, all row-major.
 *   transA = 0: A is stored M x K with leading dimension lda; 1: stored K x M.
 *   transB = 0: B is stored K x N with leading dimension ldb; 1: stored N x K.
 *   batch[d]   extent of batch dimension d (>= 1).
 *   strideX[d] element stride of operand X along batch dimension d. 0 on A or B
 *              broadcasts that operand; 0 on C with batch[d] > 1 SUMS the products of
 *              that dimension into one C (the reference's batch-reducing backward).
 *   accumulate 0: C is overwritten (Cutting, src/OperationKernels.cu:862-871);
 *              1: the result is added to C (CuttingAndCompress, :873-883).
 *   bias_mode  NZB_BIAS_ROW: bias[N] added to every row; NZB_BIAS_COL: bias[M] added to
 *              every column; NZB_BIAS_MATRIX: bias[M x N] with leading dimension bias_ld
 *              (NeuZephyr's untied conv bias {1,1,Ho*Wo,Cout}). Bias is shared by all batches.
 *   relu       apply max(x, 0) after bias (and after accumulate).
 */
typedef struct nzb_gemm_desc {
    int64_t M, N, K;
    int64_t lda, ldb, ldc;
    int32_t transA, transB;
    int32_t batch[2];
    int64_t strideA[2], strideB[2], strideC[2];
    int32_t accumulate;
    int32_t bias_mode;
    int64_t bias_ld;
    int32_t relu;
    int32_t reserved;
} nzb_gemm_desc;

/* Library / device ------------------------------------------------------- */

/* Version of this ABI (major * 100 + minor). */
NZB_API int nzb_version(void);

/* Human-readable text for the most recent non-OK return on the calling thread. */
NZB_API const char* nzb_last_error_string(void);

/*
 * Reads the device-side status word of the current device: 0 when no kernel of this
 * library gave up on a bounded wait since the last nzb_device_status_reset(). The word
 * lives in mapped host memory; call after synchronising the stream(s) of interest.
 * Replaces the reference's CHECK macro policy (cudaDeviceReset + throw,
 * include/NeuZephyr/NeuZephyrCudaErrorHandling.cuh:101-118) with a queryable status.
 */
NZB_API int nzb_device_status(int* status_out);
NZB_API int nzb_device_status_reset(void);

/*
 * Lets one bounded device-side wait run out, on purpose and harmlessly: launches a two-warp kernel
 * whose warps wait on an mbarrier nothing arrives at, one of them with a budget of limit_cycles SM
 * cycles (1 .. 2^28). That warp gives up, raises the CTA's abort flag, the other warp sees the flag
 * and leaves too, and the kernel writes NZB_ERR_DEVICE_TIMEOUT to the status word -- the same helpers
 * and the same sequence as in the GEMM and convolution kernels, without any copy in flight or tensor
 * memory held. *roles_left_dev (device int) receives the number of warps that left through the abort
 * path (2). Afterwards nzb_device_status() reads NZB_ERR_DEVICE_TIMEOUT until it is reset, and the
 * context is as usable as before. No counterpart in NeuZephyr, whose error policy is cudaDeviceReset
 * (include/NeuZephyr/NeuZephyrCudaErrorHandling.cuh:101-118).
 */
NZB_API int nzb_selftest_wait_timeout(long long limit_cycles, int* roles_left_dev, void* stream);

/* GEMM -------------------------------------------------------------------- */

/* Scratch bytes nzb_gemm needs for this descriptor (fp16 operand copies + 16 KiB of staging counters). */
NZB_API int nzb_gemm_workspace_bytes(const nzb_gemm_desc* desc, size_t* bytes_out);

/*
 * The tensor-core GEMM: replaces nz::krnl::TensorCoreGEMM / TensorCoreGEMMParallel /
 * GEMMBackwardParallel (src/OperationKernels.cu:885-912, :914-1026, :1028-1144; declared
 * include/NeuZephyr/OperationKernels.cuh:911-921) including their Padding / Cutting /
 * CuttingAndCompress passes, and optionally the bias add (MatrixAddKernel, :12-37) and
 * ReLU (:230-240) that follow it in Model::Linear / Model::Conv2d graphs.
 * workspace must be 256-byte aligned device memory of at least
 * nzb_gemm_workspace_bytes() bytes, private to this call until the stream reaches its end.
 */
NZB_API int nzb_gemm(const nzb_gemm_desc* desc, const float* A, const float* B, float* C, const float* bias,
                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * Number of kernels nzb_gemm launches for this descriptor and these operand addresses on the current
 * device: 1 when the GEMM kernel stages its own operands (one matrix product of at least 148 output
 * tiles of 256 x 256, rows that are multiples of four floats, 16-byte aligned operands; converter warps
 * inside the CTA-pair kernel round the fp32 operands to fp16 panel by panel while its tensor-core warps
 * consume finished panels), 3 otherwise (two staging kernels and the GEMM). The environment variable
 * NZB_FUSED_STAGING=0, read once per process, forces the three-kernel form.
 */
NZB_API int nzb_gemm_kernel_launches(const nzb_gemm_desc* desc, const float* A, const float* B, int* launches_out);

/*
 * Same seam as nz::data::iTensorCoreGEMM(float* A, float* B, float* C, const Dimension&
 * shapeA, shapeB, shapeC) (include/NeuZephyr/TensorOperations.cuh:1021-1024,
 * src/TensorOperations.cu:112-115): shapes are {N, C, H, W}; M = A.H, K = A.W, N = B.W;
 * an operand whose N (or C) extent is 1 is broadcast along that dimension; C is overwritten.
 */
NZB_API int nzb_tensorcore_gemm_workspace_bytes(const int64_t shapeA[4], const int64_t shapeB[4],
                                                const int64_t shapeC[4], size_t* bytes_out);
NZB_API int nzb_tensorcore_gemm(const float* A, const float* B, float* C, const int64_t shapeA[4],
                                const int64_t shapeB[4], const int64_t shapeC[4], void* workspace,
                                size_t workspace_bytes, void* stream);

/*
 * Same seam as nz::data::iGEMMBackward (include/NeuZephyr/TensorOperations.cuh:1026-1031,
 * src/TensorOperations.cu:117-120): the products of all max(A.N,B.N) x max(A.C,B.C)
 * batches are ADDED to C; along a dimension where C's extent is 1 they are summed into
 * the single C matrix (src/OperationKernels.cu:1121-1137).
 */
NZB_API int nzb_gemm_backward(const float* A, const float* B, float* C, const int64_t shapeA[4],
                              const int64_t shapeB[4], const int64_t shapeC[4], void* workspace,
                              size_t workspace_bytes, void* stream);

/*
 * fp32-accurate matrix product on the tensor cores: the seam of Tensor::operator* /
 * tensorGeneralMatrixMul / iGeneralMatrixMul (src/Tensor.cu:343-350,
 * include/NeuZephyr/TensorOperations.cuh:998-1019, src/TensorOperations.cu:104-110), whose SIMT kernel
 * (GeneralMatrixMulKernel, src/OperationKernels.cu:65-123) multiplies in fp32. Shapes are {N, C, H, W}
 * as for nzb_tensorcore_gemm, N and C of extent 1 broadcast, C is overwritten. Every operand is scaled
 * by a power of two and split into two fp16 numbers (hi + lo, 23-24 significant bits); the product keeps
 * hi*hi + hi*lo + lo*hi, computed as one fp16 GEMM of three times the contraction length with fp32
 * accumulation, and the epilogue undoes the scaling. Results agree with an fp64 product to about 1e-6
 * of the largest result (the fp16-operand product: 3e-4): the reference's own vectors are reproduced
 * exactly, and on random data 99 % or more of the elements satisfy Tensor::operator=='s rule (abs 1e-6
 * or rel 1e-5) -- what is left is the tensor core's truncating fp32 accumulator on results near zero,
 * not the split, which alone is good to 1e-7. Cost is about three times nzb_tensorcore_gemm. Elements
 * more than 17 binades below an operand's largest magnitude lose relative (not absolute) precision, and
 * results below about 1e-30 lose accuracy when the contraction is shared among CTAs (fp32 atomics flush
 * subnormal addends).
 */
NZB_API int nzb_matmul_f32_workspace_bytes(const int64_t shapeA[4], const int64_t shapeB[4], const int64_t shapeC[4],
                                           size_t* bytes_out);
NZB_API int nzb_matmul_f32(const float* A, const float* B, float* C, const int64_t shapeA[4], const int64_t shapeB[4],
                           const int64_t shapeC[4], void* workspace, size_t workspace_bytes, void* stream);

/*
 * nzb_gemm for callers that cannot allocate device memory: a plug-in inside a server or
 * framework that reserved the whole GPU for its own pool, or a steady-state loop where an
 * allocation call (and the device synchronisation it may imply) is not allowed. Same
 * descriptor, operands, results and status codes as nzb_gemm, but the fp16 staging scratch
 * is a fixed array of NZB_STATIC_SCRATCH_BYTES inside the library image, so the call makes
 * no cudaMalloc / cudaFree / host-allocation call at all. It has no counterpart in
 * NeuZephyr (whose drivers allocate three temporaries per call,
 * src/OperationKernels.cu:930-932); it exists for embedding.
 *   - Every GPU on which the library is loaded holds the array until the process exits.
 *   - Descriptors whose staged operands (nzb_gemm_workspace_bytes) exceed it return
 *     NZB_ERR_WORKSPACE with an explanatory nzb_last_error_string().
 *   - The first call on each device looks up the array's device address (with that
 *     device current); make that first call before starting any stream capture.
 *   - All calls share the array, which keeps the last call's contents. Nothing needs
 *     clearing (the staging kernels rewrite all bytes the GEMM reads), but calls that
 *     overlap on the GPU race on it: keep them ordered on one stream or with events.
 */
#define NZB_STATIC_SCRATCH_BYTES ((size_t)32 << 20)
NZB_API int nzb_gemm_static(const nzb_gemm_desc* desc, const float* A, const float* B, float* C, const float* bias,
                            void* stream);
/*
 * The status word of the nzb_gemm_static path (no counterpart in NeuZephyr either). That path cannot
 * use the mapped host word nzb_device_status reads, because creating it allocates; a bounded
 * device-side wait that gives up during nzb_gemm_static writes NZB_ERR_DEVICE_TIMEOUT into a word
 * inside the library image instead. nzb_gemm_static_status copies that word to *status_out after
 * the work already queued on `stream` (it waits for that stream, and allocates nothing);
 * nzb_gemm_static_status_reset queues its clearing on `stream`.
 */
NZB_API int nzb_gemm_static_status(int* status_out, void* stream);
NZB_API int nzb_gemm_static_status_reset(void* stream);

/*
 * nzb_gemm for operands and result in HOST memory, as one pipelined call. Replaces the sequence a
 * NeuZephyr user writes around the GEMM: Tensor::dataInject for A and B (src/Tensor.cu, one
 * blocking cudaMemcpy each), GEMMTensorCore (include/NeuZephyr/TensorOperations.cuh:1024-1028),
 * Tensor::hostData for C (another blocking copy). A is cut into row blocks; host-to-device
 * copies, staging + GEMM per block, and device-to-host copies of finished blocks run on three
 * streams, so the two PCIe directions overlap each other and the compute.
 *   - desc: one matrix product (batch extents 1), transA = 0, accumulate = 0, bias NONE / ROW / COL;
 *     bias, if any, is a host pointer too.
 *   - host buffers should be pinned (cudaHostAlloc / cudaHostRegister); pageable memory gives the
 *     same results without the overlap.
 *   - workspace: device memory, nzb_gemm_host_workspace_bytes (fp32 images of A, B, C + staging).
 *   - stream: work queued on it before the call precedes the first copy; when the stream reaches
 *     the end of the call all of C is in host memory.
 */
NZB_API int nzb_gemm_host_workspace_bytes(const nzb_gemm_desc* desc, size_t* bytes_out);
NZB_API int nzb_gemm_host(const nzb_gemm_desc* desc, const float* hostA, const float* hostB, float* hostC,
                          const float* host_bias, void* workspace, size_t workspace_bytes, void* stream);

/*
 * The GEMM alone on operands that are already staged as fp16: A16 holds op(A) as
 * [nA][M][ldk] and B16 holds op(B)^T as [nB][N][ldk] (both K-major, ldk >= K, ldk % 8 == 0,
 * 16-byte aligned), e.g. written by nzb_cast_f32_f16 or kept as fp16 shadow copies of
 * weights. This is the seam of GeneralMatrixMulTensorKernel itself (half operands in,
 * fp32 out; src/OperationKernels.cu:821-844) with the crop/accumulate and bias/ReLU
 * epilogue fused. lda/ldb/transA/transB of the descriptor are ignored; a zero batch stride
 * of A or B still means "broadcast", any non-zero value means "densely packed matrices".
 */
NZB_API int nzb_gemm_f16(const nzb_gemm_desc* desc, const void* A16, const void* B16, int64_t ldk, float* C,
                         const float* bias, void* stream);

/*
 * fp32 -> fp16 (round to nearest even) copy of `rows` x `cols` with source leading
 * dimension ld_in into a dense fp16 matrix with leading dimension ld_out (columns
 * cols..ld_out-1 are zero filled): the Padding kernel (src/OperationKernels.cu:846-860)
 * as a stand-alone pass. transpose != 0 reads the source as cols x rows.
 */
NZB_API int nzb_cast_f32_f16(const float* in, void* out_f16, int64_t rows, int64_t cols, int64_t ld_in,
                             int64_t ld_out, int transpose, void* stream);

/* Linear ----------------------------------------------------------------------------------- */

/*
 * Linear layer as Model::Linear composes it (src/Model.cu:87-103): x {batch, in}, w {out, in}
 * (the reference's {1,1,out,in}), bias {out} ({1,1,out,1}), y {batch, out} (the reference's
 * {batch,1,out,1}); relu applies max(.,0) (a following ReLUNode, src/Nodes.cu:344-364).
 * One GEMM instead of one padded matrix-vector product per sample
 * (src/OperationKernels.cu:977-999).
 */
typedef struct nzb_linear_desc {
    int64_t batch, in_features, out_features;
    int32_t relu;
    int32_t overwrite_dx;  /* backward: dx = ... instead of dx += ... (a gradient buffer with one consumer) */
} nzb_linear_desc;

NZB_API int nzb_linear_workspace_bytes(const nzb_linear_desc* desc, size_t* bytes_out);
NZB_API int nzb_linear_forward(const nzb_linear_desc* desc, const float* x, const float* w, const float* bias,
                               float* y, void* workspace, size_t workspace_bytes, void* stream);
/*
 * Backward of the same composition (ReLUNode::backward -> AddNode::backward ->
 * MatMulNode::backward, src/Nodes.cu:356-364, 99-146, 169-182) without the two transposes and
 * the per-sample launches: dx += dy' w, dw += dy'^T x, dbias += column sums of dy', with
 * dy' = dy * (y > 0) when relu is set (y is the forward output). Null outputs are skipped.
 */
NZB_API int nzb_linear_backward(const nzb_linear_desc* desc, const float* x, const float* w, const float* y,
                                const float* dy, float* dx, float* dw, float* dbias, void* workspace,
                                size_t workspace_bytes, void* stream);

/* Convolution ------------------------------------------------------------------------------ */

/*
 * Conv2d as NeuZephyr composes it (Model::Conv2d, src/Model.cu:244-263):
 *   x {N, C, H, W} NCHW; w {wN, 1, C*Kh*Kw, Cout} row-major with k = c*Kh*Kw + kh*Kw + kw and
 *   wN = 1 (shared) or N (weights_per_sample: one matrix per sample, as the reference
 *   allocates them); y {N, Cout, Ho, Wo}; Ho = (H + 2 pad - Kh)/stride + 1.
 *   bias_mode NZB_BIAS_MATRIX: bias {1, 1, Ho*Wo, Cout} (the reference's untied bias);
 *   NZB_BIAS_ROW: one value per output channel.
 *   accumulate: y += result; relu: max(., 0) last.
 */
typedef struct nzb_conv_desc {
    int64_t N, C, H, W, Cout, Kh, Kw, stride, pad;
    int32_t weights_per_sample;
    int32_t bias_mode;
    int32_t relu;
    int32_t accumulate;
    int32_t overwrite_dx;  /* backward calls: dx = ... instead of dx += ... (a gradient buffer with one consumer
                              needs neither clearing before nor reading during the backward pass) */
    int32_t reserved;
} nzb_conv_desc;

/* Scratch bytes for any of the nzb_conv2d_* calls with this descriptor (fp16 weight staging). */
NZB_API int nzb_conv2d_workspace_bytes(const nzb_conv_desc* desc, size_t* bytes_out);

/*
 * Forward: one implicit-GEMM kernel in place of Img2Col -> MatMul -> Bias -> [ReLU] -> Col2Img
 * (src/Nodes.cu:624-630, 165-167, 95-97, 344-354, 655-658; kernels src/OperationKernels.cu:1308-1335,
 * 821-1026, 12-37, 230-240, 1364-1382). fp32 in/out, operands rounded to fp16, fp32 accumulation.
 */
NZB_API int nzb_conv2d_forward(const nzb_conv_desc* desc, const float* x, const float* w, const float* bias,
                               float* y, void* workspace, size_t workspace_bytes, void* stream);

/*
 * dx += gradient of the forward with respect to x: replaces col2imgBackward ->
 * MatMulNode::backward's dA = dC * B^T (transpose + GEMMBackwardParallel) -> img2colBackward's
 * atomicAdd scatter (src/Nodes.cu:660-665, 169-176, 632-640; src/OperationKernels.cu:1384-1402,
 * 125-160, 1028-1144, 1337-1362) with one gather-form implicit GEMM over dy. stride 1, square kernels.
 */
NZB_API int nzb_conv2d_backward_data(const nzb_conv_desc* desc, const float* dy, const float* w, float* dx,
                                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * dw {wN,1,C*Kh*Kw,Cout} += gradient with respect to the weights, summed over the batch when
 * the weights are shared: replaces transpose(col) + GEMMBackwardParallel (src/Nodes.cu:177-181,
 * src/OperationKernels.cu:125-160, 1028-1144) over the materialised im2col buffer with two fp16
 * staging passes and one split-k GEMM.
 */
NZB_API int nzb_conv2d_backward_weight(const nzb_conv_desc* desc, const float* x, const float* dy, float* dw,
                                       void* workspace, size_t workspace_bytes, void* stream);

/*
 * dbias {1,1,Ho*Wo,Cout} += sum over the batch of dy (AddNode::backward's gradCopy on the
 * bias after col2imgBackward, src/Nodes.cu:106-121, 660-665).
 */
NZB_API int nzb_conv2d_backward_bias(const nzb_conv_desc* desc, const float* dy, float* dbias, void* stream);

/*
 * The whole backward of one convolution layer on shared staging: dbias += sum over images of dY',
 * dW += ..., dX += ..., with dY' = dY * (Y > 0) when desc->relu is set (y is the layer's forward
 * output). Stands in for the same reference code as the three calls above plus ReLUNode::backward
 * (src/Nodes.cu), but reads dY once: one pass masks it, writes the fp16 copies both tensor-core
 * kernels consume and accumulates the bias gradient. Any of dx, dw, dbias may be null.
 *   - handled shapes: stride 1, square kernel up to 4x4, pad <= K-1, input and output rows of at
 *     least 32 pixels, bias gradient as the {Ho*Wo, Cout} matrix (desc->bias_mode NZB_BIAS_MATRIX);
 *     nzb_conv2d_backward_workspace_bytes returns NZB_ERR_UNSUPPORTED otherwise and the caller
 *     uses the separate entry points.
 */
NZB_API int nzb_conv2d_backward_workspace_bytes(const nzb_conv_desc* desc, size_t* bytes_out);
NZB_API int nzb_conv2d_backward(const nzb_conv_desc* desc, const float* x, const float* w, const float* y,
                                const float* dy, float* dx, float* dw, float* dbias, void* workspace,
                                size_t workspace_bytes, void* stream);

/* Node operations around the contraction ---------------------------------------------- */

/*
 * nz::data::iImg2col / iImg2colBackward (include/NeuZephyr/TensorOperations.cuh:1108-1114,
 * src/TensorOperations.cu:135-149; img2colKernel / img2colBackwardKernel,
 * src/OperationKernels.cu:1308-1362). out is {batch, 1, H_out*W_out, C*K_h*K_w}; the backward
 * ADDS the scattered column gradient to dx (gather form, no atomics).
 */
NZB_API int nzb_img2col(float* out, const float* in, int64_t H_out, int64_t W_out, int64_t C, int64_t K_h,
                        int64_t K_w, int64_t stride, int64_t pad, int64_t H_in, int64_t W_in, int64_t batch,
                        void* stream);
NZB_API int nzb_img2col_backward(float* dx, const float* dcol, int64_t H_out, int64_t W_out, int64_t C, int64_t K_h,
                                 int64_t K_w, int64_t stride, int64_t pad, int64_t H_in, int64_t W_in, int64_t batch,
                                 void* stream);

/*
 * nz::data::iCol2img / iCol2imgBackward (include/NeuZephyr/TensorOperations.cuh:1132-1146;
 * col2imgKernel / col2imgBackwardKernel, src/OperationKernels.cu:1364-1402):
 * {b, 1, H*W, C} -> {b, C, H, W} and back; both overwrite.
 */
NZB_API int nzb_col2img(float* out, const float* in, int64_t H_out, int64_t W_out, int64_t C_out, int64_t batches,
                        void* stream);
NZB_API int nzb_col2img_backward(float* out, const float* in, int64_t H_out, int64_t W_out, int64_t C_out,
                                 int64_t batches, void* stream);

/*
 * AddNode forward / backward (src/Nodes.cu:95-146; MatrixAddKernel src/OperationKernels.cu:12-37,
 * gradCopyKernel :1230-1236). Shapes are {N,C,H,W}; N and C broadcast. Backward: an input of
 * the output's shape receives a copy (overwrite); a broadcast input receives += the sum over
 * the batches it was broadcast to (the reference's racy per-slice launches, made deterministic).
 */
NZB_API int nzb_add_broadcast(float* out, const float* a, const float* b, const int64_t shapeA[4],
                              const int64_t shapeB[4], void* stream);
NZB_API int nzb_add_backward(float* gin, const float* gout, const int64_t shapeIn[4], const int64_t shapeOut[4],
                             void* stream);

/* ReLU and its backward (overwrite), src/OperationKernels.cu:230-253. */
NZB_API int nzb_relu(float* out, const float* in, int64_t n, void* stream);
NZB_API int nzb_relu_backward(float* gin, const float* x, const float* gout, int64_t n, void* stream);

/*
 * Average pooling, divisor = in-bounds taps (src/OperationKernels.cu:1404-1490). The backward
 * ADDS to gin (gather form of the reference's atomicAdd scatter).
 */
NZB_API int nzb_avgpool(float* out, const float* in, int64_t pool, int64_t stride, int64_t pad, int64_t batches,
                        int64_t channels, int64_t H_in, int64_t W_in, int64_t H_out, int64_t W_out, void* stream);
NZB_API int nzb_avgpool_backward(float* gin, const float* gout, int64_t pool, int64_t stride, int64_t pad,
                                 int64_t batches, int64_t channels, int64_t H_in, int64_t W_in, int64_t H_out,
                                 int64_t W_out, void* stream);
/* The same with overwrite != 0: gin is WRITTEN (as if it had been zero), so a gradient buffer with a single
 * consumer needs neither clearing before nor reading during the backward pass. */
NZB_API int nzb_avgpool_backward_ex(float* gin, const float* gout, int64_t pool, int64_t stride, int64_t pad,
                                    int64_t batches, int64_t channels, int64_t H_in, int64_t W_in, int64_t H_out,
                                    int64_t W_out, int overwrite, void* stream);

/*
 * Softmax over each of `batches` vectors of n elements, fully on the device (the reference
 * syncs the host once per vector for the exp-sum: Tensor::expSum, src/Tensor.cu:713-735;
 * SummationExpKernel / SoftmaxKernel, src/OperationKernels.cu:477-523), and
 * SoftmaxNode::backward (src/Nodes.cu:538-548): gin = J(y) * gout (overwrite).
 * round_f16 != 0 rounds J and gout to fp16 as the reference's GEMM does.
 */
NZB_API int nzb_softmax(float* out, const float* in, int64_t batches, int64_t n, void* stream);
NZB_API int nzb_softmax_backward(float* gin, const float* y, const float* gout, int64_t batches, int64_t n,
                                 int round_f16, void* stream);

/*
 * Binary cross-entropy, mean over n elements (BinaryCrossEntropyKernel / BCEBackwardKernel,
 * src/OperationKernels.cu:648-704). nzb_bce ADDS the loss to the device scalar loss_out
 * (the reference's loss node accumulates too, src/Nodes.cu:822-840).
 */
NZB_API int nzb_bce(float* loss_out, const float* predict, const float* target, int64_t n, void* stream);
NZB_API int nzb_bce_backward(float* out, const float* predict, const float* target, int64_t n, void* stream);

/* Adam step with explicit t (AdamKernel, src/OperationKernels.cu:753-773; opt::Adam::step, src/Optimizer.cu:86-102). */
NZB_API int nzb_adam(float* data, float* m, float* v, const float* grad, float lr, float beta1, float beta2,
                     float eps, int t, int64_t n, void* stream);

/*
 * Adam over all tensors of a model in ONE launch: opt::Adam::step (src/Optimizer.cu:86-102) is called once
 * per tensor by ComputeGraph::update (src/ComputeGraph.cu:541-547), one AdamKernel launch each. Every
 * tensor carries its own time step t (the reference's counter advances per step() call). shadow_f16,
 * when non-null, receives the updated weights rounded to fp16 (n halves): the operand copy the tensor
 * cores read, written by the pass that already holds the new value. Same arithmetic as nzb_adam.
 */
typedef struct nzb_adam_tensor {
    float* data;
    float* m;
    float* v;
    const float* grad;
    void* shadow_f16;
    int64_t n;
    int32_t t;
    int32_t reserved;
} nzb_adam_tensor;
NZB_API int nzb_adam_multi(const nzb_adam_tensor* tensors, int count, float lr, float beta1, float beta2, float eps,
                           void* stream);

/*
 * The softmax + binary-cross-entropy head as one kernel each way: SoftmaxNode::forward followed by
 * BinaryCrossEntropyNode::forward (src/Nodes.cu:534-536, 822-840; the reference syncs the host once per
 * vector for the exp-sum and once for the loss), and BinaryCrossEntropyNode::backward followed by
 * SoftmaxNode::backward (src/Nodes.cu:842-848, 538-548). probs {batches, n} receives the softmax, *loss
 * (device scalar) is incremented by the mean BCE over all batches*n elements; the backward OVERWRITES
 * dlogits with J(probs) * dBCE, with J and dBCE rounded to fp16 first when round_f16 != 0 (what the
 * reference's tensor-core product does). n <= 1024.
 */
NZB_API int nzb_softmax_bce_forward(float* probs, float* loss, const float* logits, const float* target,
                                    int64_t batches, int64_t n, void* stream);
NZB_API int nzb_softmax_bce_backward(float* dlogits, const float* probs, const float* target, int64_t batches,
                                     int64_t n, int round_f16, void* stream);

/*
 * Max pooling (MaxPoolingKernel / MaxPoolingBackwardKernel, src/OperationKernels.cu:1507-1573; iMaxPooling
 * / iMaxPoolingBackward): the first maximum in row-major window order wins, its index within the window is
 * stored as a float in `position` {batches, channels, H_out, W_out}, an empty window yields 0. The backward
 * ADDS each upstream gradient to the input element recorded as its window's maximum (gather form of the
 * reference's atomicAdd scatter).
 */
NZB_API int nzb_maxpool(float* out, float* position, const float* in, int64_t pool, int64_t stride, int64_t pad,
                        int64_t batches, int64_t channels, int64_t H_in, int64_t W_in, int64_t H_out, int64_t W_out,
                        void* stream);
NZB_API int nzb_maxpool_backward(float* gin, const float* position, const float* gout, int64_t pool, int64_t stride,
                                 int64_t pad, int64_t batches, int64_t channels, int64_t H_in, int64_t W_in,
                                 int64_t H_out, int64_t W_out, void* stream);

/* FillKernel (src/OperationKernels.cu:1146-1156), ExpandKernel (:1282-1296; batch broadcast copy), in-place scale. */
NZB_API int nzb_fill(float* data, float value, int64_t n, void* stream);
NZB_API int nzb_expand(float* out, const float* in, int64_t per_batch, int64_t batches, void* stream);
NZB_API int nzb_scale(float* data, float factor, int64_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NZB_H */
