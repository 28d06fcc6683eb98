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

// dW[o][j] += sum_b dY'[b][o] * X[b][j] for a layer with few outputs and a short batch (the contraction): a
// 16 x In weight gradient with a contraction of 8 .. 256 is a poor fit for 128-row tensor-core tiles (the GEMM
// kernel ran it at 15 % of the DRAM rate, one k block per tile), and it is bound by reading X once. A thread owns
// four consecutive input features and 16 outputs; dY' (masked, rounded to fp16 like every operand) sits in shared
// memory and is read as broadcasts; X is read as fp32 float4, rounded to fp16 in registers (no staged copy),
// products of two fp16 values are exact in fp32 and are accumulated with fp32 FMAs.
template <int BMAX>
__global__ void __launch_bounds__(256) linear_wgrad_small_kernel(float* __restrict__ dw, const float* __restrict__ dy,
                                                                 const float* __restrict__ mask,
                                                                 const float* __restrict__ x, int B, int64_t In, int Out) {
    __shared__ __align__(16) float sdy[BMAX][16];
    const int o0 = blockIdx.y * 16;
    for (int i = threadIdx.x; i < B * 16; i += 256) {
        const int b = i >> 4, o = o0 + (i & 15);
        float g = 0.f;
        if (o < Out) {
            g = __ldg(dy + (int64_t)b * Out + o);
            if (mask && !(__ldg(mask + (int64_t)b * Out + o) > 0.f)) g = 0.f;
        }
        sdy[b][i & 15] = __half2float(__float2half_rn(g));
    }
    __syncthreads();
    const int64_t groups = In >> 2;
    for (int64_t gidx = blockIdx.x * 256ll + threadIdx.x; gidx < groups; gidx += gridDim.x * 256ll) {
        const float* xp = x + gidx * 4;
        float acc[16][4];
#pragma unroll
        for (int o = 0; o < 16; o++) acc[o][0] = acc[o][1] = acc[o][2] = acc[o][3] = 0.f;
#pragma unroll 4
        for (int b = 0; b < B; b++) {
            const float4 xv = __ldg(reinterpret_cast<const float4*>(xp + (int64_t)b * In));
            const float x0 = __half2float(__float2half_rn(xv.x)), x1 = __half2float(__float2half_rn(xv.y)),
                        x2 = __half2float(__float2half_rn(xv.z)), x3 = __half2float(__float2half_rn(xv.w));
            const float4* d4 = reinterpret_cast<const float4*>(&sdy[b][0]);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float4 dv = d4[q];
                const float dd[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    acc[q * 4 + i][0] = fmaf(dd[i], x0, acc[q * 4 + i][0]);
                    acc[q * 4 + i][1] = fmaf(dd[i], x1, acc[q * 4 + i][1]);
                    acc[q * 4 + i][2] = fmaf(dd[i], x2, acc[q * 4 + i][2]);
                    acc[q * 4 + i][3] = fmaf(dd[i], x3, acc[q * 4 + i][3]);
                }
            }
        }
#pragma unroll
        for (int o = 0; o < 16; o++) {
            if (o0 + o < Out) {
                float4* dst = reinterpret_cast<float4*>(dw + (int64_t)(o0 + o) * In + gidx * 4);
                float4 w4 = *dst;
                w4.x += acc[o][0]; w4.y += acc[o][1]; w4.z += acc[o][2]; w4.w += acc[o][3];
                *dst = w4;
            }
        }
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
    if (dw && z.Out <= 32 && z.B <= 256 && z.In % 4 == 0 && z.In >= 4096 &&
        ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dw)) & 15) == 0) {
        // few outputs, short contraction, long rows: bound by reading X once (see linear_wgrad_small_kernel)
        int64_t blocks = (z.In / 4 + 255) / 256;
        const int64_t cap = (int64_t)ds->sm_count * 8;
        if (blocks > cap) blocks = cap;
        const dim3 grid((unsigned)blocks, (unsigned)((z.Out + 15) / 16));
        if (z.B <= 64)
            linear_wgrad_small_kernel<64><<<grid, 256, 0, s>>>(dw, dy, mask, x, (int)z.B, z.In, (int)z.Out);
        else
            linear_wgrad_small_kernel<256><<<grid, 256, 0, s>>>(dw, dy, mask, x, (int)z.B, z.In, (int)z.Out);
        NZB_CUDA_TRY(cudaGetLastError());
    } else if (dw) {
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
