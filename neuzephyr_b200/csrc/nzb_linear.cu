// Linear layer as NeuZephyr builds it (Model::Linear, src/Model.cu:87-103):
//   Reshape{N,1,in,1} -> MatMul(W{1,1,out,in}, x) -> Bias{1,1,out,1} [-> ReLU]
// The reference runs it as N separate matrix-vector products padded to 16 columns, one
// kernel launch per sample (src/OperationKernels.cu:977-999). Here the batch is a GEMM
// dimension: Y[N x out] = X[N x in] * W^T (+ bias, ReLU) in one launch, and the backward
//   dX += dY' * W,  dW += dY'^T * X,  db += column sums of dY',  dY' = dY * (Y > 0)
// runs on the same kernel family with the ReLU mask folded into the operand staging. The
// three fp16 copies (dY', W, X) keep their row-major layout: each GEMM reads them K-major or
// MN-major as its contraction requires, so no operand is transposed in memory.
#include <cuda_fp16.h>

#include "nzb_internal.h"

namespace nzb {

// db[o] += sum_b dy[b][o] * (mask ? y[b][o] > 0 : 1). Blocks own a 32-column strip and a
// slice of rows; partial sums are added atomically (fp32), like the reference's gradCopy.
__global__ void __launch_bounds__(256) bias_grad_rows_kernel(float* __restrict__ db, const float* __restrict__ dy,
                                                             const float* __restrict__ mask, int64_t rows,
                                                             int64_t cols, int64_t rows_per_block) {
    __shared__ float part[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t strips = (cols + 31) >> 5;
    const int64_t strip = blockIdx.x % strips, slice = blockIdx.x / strips;
    const int64_t c = strip * 32 + tx;
    const int64_t r0 = slice * rows_per_block;
    const int64_t r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
    float s = 0.f;
    if (c < cols)
        for (int64_t r = r0 + ty; r < r1; r += 8) {
            const float g = __ldg(dy + r * cols + c);
            s += (!mask || __ldg(mask + r * cols + c) > 0.f) ? g : 0.f;
        }
    part[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && c < cols) {
#pragma unroll
        for (int i = 1; i < 8; i++) s += part[i][tx];
        atomicAdd(db + c, s);
    }
}

struct LinearSizes {
    int64_t B, In, Out, Inp, Outp, Bp;
    size_t x16, w16, total_fwd;           // forward: X [B][Inp], W [Out][Inp]
    size_t dy16, total_bwd;               // backward: dY' [B][Outp] plus the two above
};
static void linear_sizes(const nzb_linear_desc* d, LinearSizes* z) {
    z->B = d->batch; z->In = d->in_features; z->Out = d->out_features;
    z->Inp = round_up(z->In, 64); z->Outp = round_up(z->Out, 64); z->Bp = round_up(z->B, 64);
    z->x16 = (size_t)round_up(z->B * z->Inp * 2, 256);
    z->w16 = (size_t)round_up(z->Out * z->Inp * 2, 256);
    z->total_fwd = z->x16 + z->w16 + kFuseSyncBytes;  // the forward is one nzb_gemm call
    z->dy16 = (size_t)round_up(z->B * z->Outp * 2, 256);
    z->total_bwd = z->dy16 + z->w16 + z->x16;
}

static int check_linear(const nzb_linear_desc* d) {
    if (!d) return fail(NZB_ERR_BAD_ARG, "descriptor is null");
    if (d->batch < 0 || d->in_features < 1 || d->out_features < 1) return fail(NZB_ERR_BAD_ARG, "bad extent");
    return NZB_OK;
}

}  // namespace nzb

using namespace nzb;

extern "C" {

int nzb_linear_workspace_bytes(const nzb_linear_desc* d, size_t* bytes_out) {
    if (!bytes_out) return fail(NZB_ERR_BAD_ARG, "bytes_out is null");
    int rc = check_linear(d);
    if (rc != NZB_OK) return rc;
    LinearSizes z;
    linear_sizes(d, &z);
    *bytes_out = z.total_fwd > z.total_bwd ? z.total_fwd : z.total_bwd;
    return NZB_OK;
}

int nzb_linear_forward(const nzb_linear_desc* d, const float* x, const float* w, const float* bias, float* y,
                       void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_linear(d);
    if (rc != NZB_OK) return rc;
    if (d->batch == 0) return NZB_OK;
    if (!x || !w || !y) return fail(NZB_ERR_BAD_ARG, "x, w and y must be non-null");
    nzb_gemm_desc g{};
    g.M = d->batch; g.N = d->out_features; g.K = d->in_features;
    g.lda = g.K; g.ldb = g.K; g.ldc = g.N;
    g.transA = 0; g.transB = 1;  // W is stored [out][in] = N x K
    g.batch[0] = g.batch[1] = 1;
    g.bias_mode = bias ? NZB_BIAS_ROW : NZB_BIAS_NONE;
    g.bias_ld = g.N;
    g.relu = d->relu ? 1 : 0;
    return nzb_gemm(&g, x, w, y, bias, workspace, workspace_bytes, stream);
}

int nzb_linear_backward(const nzb_linear_desc* d, const float* x, const float* w, const float* y, const float* dy,
                        float* dx, float* dw, float* dbias, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_linear(d);
    if (rc != NZB_OK) return rc;
    if (d->batch == 0) return NZB_OK;
    if (!dy) return fail(NZB_ERR_BAD_ARG, "dy must be non-null");
    if (d->relu && !y) return fail(NZB_ERR_BAD_ARG, "the ReLU mask needs the forward output y");
    if ((dx && !w) || (dw && !x)) return fail(NZB_ERR_BAD_ARG, "dx needs w and dw needs x");
    LinearSizes z;
    linear_sizes(d, &z);
    if (!workspace || workspace_bytes < z.total_bwd) return fail(NZB_ERR_WORKSPACE, "workspace of %zu bytes needed", z.total_bwd);
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(NZB_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    DeviceState* ds;
    rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float* mask = d->relu ? y : nullptr;
    uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
    __half* dy16 = reinterpret_cast<__half*>(base);
    __half* w16 = reinterpret_cast<__half*>(base + z.dy16);
    __half* x16 = reinterpret_cast<__half*>(base + z.dy16 + z.w16);
    if (dbias) {
        const int64_t strips = (z.Out + 31) / 32;
        int64_t slices = ((int64_t)ds->sm_count * 8 + strips - 1) / strips;
        if (slices > (z.B + 63) / 64) slices = (z.B + 63) / 64;
        if (slices < 1) slices = 1;
        const int64_t rpb = (z.B + slices - 1) / slices;
        bias_grad_rows_kernel<<<(unsigned)(strips * slices), 256, 0, s>>>(dbias, dy, mask, z.B, z.Out, rpb);
        NZB_CUDA_TRY(cudaGetLastError());
    }
    // dY' [B][Outp]: K-major left operand of dX (k = Out) and MN-major left operand of dW (k = B)
    rc = launch_cast_masked(ds->sm_count, dy, mask, dy16, z.B, z.Out, z.Out, z.Outp, 0, 1, 1, 0, 0, s);
    if (rc != NZB_OK) return rc;
    if (dx) {
        // dX[B x In] += dY'[B x Out] * W[Out x In]: W as stored is the MN-major right operand
        rc = launch_cast_masked(ds->sm_count, w, nullptr, w16, z.Out, z.In, z.In, z.Inp, 0, 1, 1, 0, 0, s);
        if (rc != NZB_OK) return rc;
        GemmLaunch g{};
        g.A16 = dy16; g.B16 = w16; g.nA = g.nB = 1;
        g.M = z.B; g.N = z.In; g.K = z.Out; g.Kp = z.Outp;
        g.b_mn = 1; g.ldb16 = z.Inp;
        g.C = dx; g.ldc = z.In;
        g.out_e[0] = g.out_e[1] = g.red_e[0] = g.red_e[1] = 1;
        g.accumulate = d->overwrite_dx ? 0 : 1;
        rc = launch_gemm(g, s);
        if (rc != NZB_OK) return rc;
    }
    if (dw) {
        // dW[Out x In] += dY'^T[Out x B] * X[B x In]: both operands as stored, contraction along rows
        rc = launch_cast_masked(ds->sm_count, x, nullptr, x16, z.B, z.In, z.In, z.Inp, 0, 1, 1, 0, 0, s);
        if (rc != NZB_OK) return rc;
        GemmLaunch g{};
        g.A16 = dy16; g.B16 = x16; g.nA = g.nB = 1;
        g.M = z.Out; g.N = z.In; g.K = z.B; g.Kp = z.Bp;
        g.a_mn = 1; g.lda16 = z.Outp;
        g.b_mn = 1; g.ldb16 = z.Inp;
        g.C = dw; g.ldc = z.In;
        g.out_e[0] = g.out_e[1] = g.red_e[0] = g.red_e[1] = 1;
        g.accumulate = 1;
        rc = launch_gemm(g, s);
        if (rc != NZB_OK) return rc;
    }
    return NZB_OK;
}

}  // extern "C"
