// Tensor-level operations of the contraction path and the raw-pointer `i*` wrappers under
// them (mirrors include/NeuZephyr/TensorOperations.cuh / src/TensorOperations.cu). Every
// function picks a stream from StreamManager, orders itself after the operands' pending work,
// calls the sm_100a kernel library (libnzb) and publishes an event on what it wrote.
#pragma once
#include "Tensor.cuh"

namespace nz::data {

// C = A x B on the tensor cores (fp16 operands, fp32 accumulate); overwrite. Raw-pointer seam
// of the reference: include/NeuZephyr/TensorOperations.cuh:1021-1024.
void iTensorCoreGEMM(float* A, float* B, float* C, const Dimension& shapeA, const Dimension& shapeB,
                     const Dimension& shapeC);
// C += A x B, summed over broadcast batch dimensions of C (:1026-1031).
void iGEMMBackward(float* A, float* B, float* C, const Dimension& shapeA, const Dimension& shapeB,
                   const Dimension& shapeC);
// C = A x B at fp32 accuracy: the seam of iGeneralMatrixMul (src/TensorOperations.cu:104-110), taking the
// operands' shapes instead of precomputed offset lists; overwrite, N / C of extent 1 broadcast.
void iGeneralMatrixMul(float* A, float* B, float* C, const Dimension& shapeA, const Dimension& shapeB,
                       const Dimension& shapeC);
// out = lhs x rhs (include/NeuZephyr/TensorOperations.cuh:998-1019); throws std::invalid_argument for
// shapes that are not broadcast compatible, as the reference does.
void tensorGeneralMatrixMul(Tensor& out, const Tensor& lhs, const Tensor& rhs);
// General form with transposed operands and fused epilogue (no reference counterpart; used by the
// fused nodes): C (op)= op(A) op(B) for single matrices.
void iGemm(const float* A, const float* B, float* C, size_t M, size_t N, size_t K, bool transA, bool transB,
           bool accumulate, const float* bias = nullptr, int bias_mode = 0, bool relu = false);

void iImg2col(float* out, float* in, size_t H_out, size_t W_out, size_t C, size_t K_h, size_t K_w, size_t stride,
              size_t pad, size_t H_in, size_t W_in, size_t batch);
void iImg2colBackward(float* out, float* in, size_t H_out, size_t W_out, size_t C, size_t K_h, size_t K_w,
                      size_t stride, size_t pad, size_t H_in, size_t W_in, size_t batch);
void iCol2img(float* out, float* in, size_t H_out, size_t W_out, size_t C_out, size_t batches);
void iCol2imgBackward(float* out, float* in, size_t H_out, size_t W_out, size_t C_out, size_t batches);
void iMatrixAdd(float* out, float* a, float* b, const Dimension& shapeA, const Dimension& shapeB);
void iAddBackward(float* gin, float* gout, const Dimension& shapeIn, const Dimension& shapeOut);
void iRELU(float* out, float* in, size_t n);
void iReLUBackward(float* gin, float* x, float* gout, size_t n);
void iAveragePooling(float* out, float* in, size_t pool, size_t stride, size_t pad, size_t batches, size_t channels,
                     size_t H_in, size_t W_in, size_t H_out, size_t W_out);
void iAveragePoolingBackward(float* gin, float* gout, size_t pool, size_t stride, size_t pad, size_t batches,
                             size_t channels, size_t H_in, size_t W_in, size_t H_out, size_t W_out);
// iMaxPooling / iMaxPoolingBackward (include/NeuZephyr/TensorOperations.cuh; kernels
// src/OperationKernels.cu:1507-1573): position holds each window's arg-max index as a float
void iMaxPooling(float* out, float* position, float* in, size_t pool, size_t stride, size_t pad, size_t batches,
                 size_t channels, size_t H_in, size_t W_in, size_t H_out, size_t W_out);
void iMaxPoolingBackward(float* gin, float* position, float* gout, size_t pool, size_t stride, size_t pad,
                         size_t batches, size_t channels, size_t H_in, size_t W_in, size_t H_out, size_t W_out);
// the softmax + BCE head in one kernel each way (no counterpart in the reference)
void iSoftmaxBCE(float* probs, float* loss, float* logits, float* target, size_t batches, size_t n);
void iSoftmaxBCEBackward(float* dlogits, float* probs, float* target, size_t batches, size_t n, bool round_f16);
// gin = ... instead of gin += ... (for a gradient buffer marked Tensor::gradOverwritten())
void iAveragePoolingBackwardOverwrite(float* gin, float* gout, size_t pool, size_t stride, size_t pad, size_t batches,
                                      size_t channels, size_t H_in, size_t W_in, size_t H_out, size_t W_out);
void iSoftmax(float* out, float* in, size_t batches, size_t n);
void iSoftmaxBackward(float* gin, float* y, float* gout, size_t batches, size_t n, bool round_f16);
void iBCE(float* loss, float* predict, float* target, size_t n);
void iBCEBackward(float* out, float* predict, float* target, size_t n);
void iExpand(float* out, float* in, size_t per_batch, size_t batches);
void iFill(float* data, float value, size_t n);

// GEMMTensorCore(out, A, B): the user-facing tensor-core product
// (include/NeuZephyr/TensorOperations.cuh:1024-1028). Unlike the reference it validates shapes.
void GEMMTensorCore(Tensor& out, const Tensor& lhs, const Tensor& rhs);
// out-of-place per-matrix transpose of data (and grad), :1071-1086
Tensor transpose(const Tensor& in);
Tensor tensorImg2col(const Tensor& in, size_t K_h, size_t K_w, size_t stride, size_t pad);
Tensor tensorCol2img(const Tensor& in, size_t H_out, size_t W_out);
Tensor tensorAveragePooling(const Tensor& in, size_t pool, size_t stride, size_t pad);
void tensorMatrixAdd(Tensor& out, const Tensor& lhs, const Tensor& rhs);
Tensor ReLU(const Tensor& in);
Tensor Softmax(const Tensor& in);

}  // namespace nz::data
