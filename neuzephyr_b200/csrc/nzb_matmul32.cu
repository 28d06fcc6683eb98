// fp32-accurate matrix product on the fp16 tensor cores: stands in for NeuZephyr's SIMT
// GeneralMatrixMulKernel (src/OperationKernels.cu:65-123) behind Tensor::operator* and
// tensorGeneralMatrixMul (src/Tensor.cu:343-350, include/NeuZephyr/TensorOperations.cuh:998-1019).
//
// Each fp32 operand is scaled by a power of two (so that its largest magnitude sits at 2^13..2^14) and
// split into two fp16 numbers, x*s = hi + lo with hi = fp16(x*s) and lo = fp16(x*s - hi): together they
// carry 23-24 significant bits. The product keeps the three leading terms,
//     A*B = (Ahi*Bhi + Ahi*Blo + Alo*Bhi) / (sA*sB)           (the dropped Alo*Blo is below 2^-24 of a term)
// and all three run as ONE ordinary fp16 GEMM with fp32 accumulation by concatenating along the
// contraction: A' = [Ahi | Alo | Ahi] (M x 3K) and B' = [Blo ; Bhi ; Bhi] (3K x N). The two small cross
// terms come FIRST: the tensor core adds into its fp32 accumulator with truncation, so small addends that
// arrive while the accumulator is still small keep their bits, and their finished sum is rounded once when
// the large hi*hi terms follow (the other order loses a few bits of every cross term). The kernels are
// those of nzb_gemm; the epilogue multiplies by 1/(sA*sB), read from device memory (nothing syncs the host).
// Cost: three times the fp16 GEMM plus one pass over each operand for its largest magnitude and one for
// the split.
#include <cuda_fp16.h>

#include "nzb_internal.h"

namespace nzb {

// ---- largest magnitude of an operand (bit pattern of |x| is monotone for finite floats) -------------
__global__ void __launch_bounds__(256) absmax_kernel(const float* __restrict__ x, int64_t n, unsigned* __restrict__ out) {
    unsigned m = 0;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    const int64_t n4 = (reinterpret_cast<uintptr_t>(x) & 15) == 0 ? n / 4 : 0;
    for (int64_t j = i; j < n4; j += stride) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(x) + j);
        m = max(max(m, __float_as_uint(fabsf(v.x))), max(__float_as_uint(fabsf(v.y)),
                max(__float_as_uint(fabsf(v.z)), __float_as_uint(fabsf(v.w)))));
    }
    for (int64_t j = n4 * 4 + i; j < n; j += stride) m = max(m, __float_as_uint(fabsf(__ldg(x + j))));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m) atomicMax(out, m);
}

// scales[0] = sA, scales[1] = sB (powers of two), scales[2] = 1 / (sA * sB)
__global__ void split_scales_kernel(const unsigned* __restrict__ amax_bits, float* __restrict__ scales) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    float s[2];
    for (int i = 0; i < 2; i++) {
        const float m = __uint_as_float(amax_bits[i]);
        int e = 0;
        if (m > 0.f && isfinite(m)) frexpf(m, &e);  // m = f * 2^e, f in [0.5, 1)
        else e = 14;                                 // all zero (or not finite): any scale will do
        const int shift = max(-120, min(120, 14 - e));  // the scale and its reciprocal stay normal floats
        s[i] = ldexpf(1.0f, shift);                  // largest magnitude lands in [2^13, 2^14)
        scales[i] = s[i];
    }
    scales[2] = (1.0f / s[0]) * (1.0f / s[1]);       // exact: powers of two
}

__device__ __forceinline__ void split2(float x, float s, __half& hi, __half& lo) {
    const float v = x * s;  // exact (power of two) unless it leaves fp32's range
    hi = __float2half_rn(v);
    lo = __float2half_rn(v - __half2float(hi));
}

// Operand stored rows x K (contraction along the row): copy [rows][3*Kseg], segment j of a row holds
// the high part except segment lo_seg, which holds the low part. Four k per thread.
__global__ void __launch_bounds__(256) split_kmajor_kernel(const float* __restrict__ src, __half* __restrict__ dst,
                                                           int64_t rows, int K, int64_t ld_src, int Kseg, int lo_seg,
                                                           int64_t nmat, int64_t mat_stride_src,
                                                           const float* __restrict__ scale) {
    const float s = __ldg(scale);
    const int k4 = Kseg >> 2;
    const int64_t total = nmat * rows * k4;
    for (int64_t u = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; u < total;
         u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = u / k4;  // row over all matrices
        const int k = static_cast<int>(u - r * k4) * 4;
        const int64_t mat = r / rows, rr = r - mat * rows;
        const float* sp = src + mat * mat_stride_src + rr * ld_src + k;
        __half h[4], l[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float x = k + j < K ? __ldg(sp + j) : 0.f;
            split2(x, s, h[j], l[j]);
        }
        __half* dp = dst + r * (3 * static_cast<int64_t>(Kseg)) + k;
        uint2 hv, lv;
        __half2 t0 = __halves2half2(h[0], h[1]), t1 = __halves2half2(h[2], h[3]);
        __half2 u0 = __halves2half2(l[0], l[1]), u1 = __halves2half2(l[2], l[3]);
        hv.x = *reinterpret_cast<uint32_t*>(&t0); hv.y = *reinterpret_cast<uint32_t*>(&t1);
        lv.x = *reinterpret_cast<uint32_t*>(&u0); lv.y = *reinterpret_cast<uint32_t*>(&u1);
#pragma unroll
        for (int seg = 0; seg < 3; seg++)
            *reinterpret_cast<uint2*>(dp + static_cast<int64_t>(seg) * Kseg) = seg == lo_seg ? lv : hv;
    }
}

// Operand stored K x cols (contraction along the rows, as the right operand of a row-major product):
// copy [3*Kseg][ld_dst], row block j holds the high part except block lo_seg, which holds the low part.
// Four columns per thread; columns cols..ld_dst-1 and rows K..Kseg-1 of every block are written as zero.
__global__ void __launch_bounds__(256) split_mnmajor_kernel(const float* __restrict__ src, __half* __restrict__ dst,
                                                            int K, int64_t cols, int64_t ld_src, int Kseg,
                                                            int64_t ld_dst, int lo_seg, int64_t nmat,
                                                            int64_t mat_stride_src, const float* __restrict__ scale) {
    const float s = __ldg(scale);
    const int64_t c4 = ld_dst >> 2;
    const int64_t total = nmat * Kseg * c4;
    const bool vec = (ld_src & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (mat_stride_src & 3) == 0;
    for (int64_t u = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; u < total;
         u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t row = u / c4;  // k row over all matrices
        const int64_t c = (u - row * c4) * 4;
        const int64_t mat = row / Kseg;
        const int k = static_cast<int>(row - mat * Kseg);
        float x[4] = {0.f, 0.f, 0.f, 0.f};
        if (k < K) {
            const float* sp = src + mat * mat_stride_src + static_cast<int64_t>(k) * ld_src + c;
            if (vec && c + 3 < cols) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(sp));
                x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (c + j < cols) x[j] = __ldg(sp + j);
            }
        }
        __half h[4], l[4];
#pragma unroll
        for (int j = 0; j < 4; j++) split2(x[j], s, h[j], l[j]);
        __half2 t0 = __halves2half2(h[0], h[1]), t1 = __halves2half2(h[2], h[3]);
        __half2 u0 = __halves2half2(l[0], l[1]), u1 = __halves2half2(l[2], l[3]);
        uint2 hv, lv;
        hv.x = *reinterpret_cast<uint32_t*>(&t0); hv.y = *reinterpret_cast<uint32_t*>(&t1);
        lv.x = *reinterpret_cast<uint32_t*>(&u0); lv.y = *reinterpret_cast<uint32_t*>(&u1);
        __half* dp = dst + (mat * 3 * Kseg + k) * ld_dst + c;
#pragma unroll
        for (int seg = 0; seg < 3; seg++)
            *reinterpret_cast<uint2*>(dp + static_cast<int64_t>(seg) * Kseg * ld_dst) = seg == lo_seg ? lv : hv;
    }
}

// Narrow right operand (N <= 32), stored K x N: K-major copy [N][3*Kseg] through a transposing read.
__global__ void __launch_bounds__(256) split_transpose_kernel(const float* __restrict__ src, __half* __restrict__ dst,
                                                              int K, int64_t N, int64_t ld_src, int Kseg, int lo_seg,
                                                              int64_t nmat, int64_t mat_stride_src,
                                                              const float* __restrict__ scale) {
    const float s = __ldg(scale);
    const int64_t total = nmat * N * Kseg;
    for (int64_t u = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; u < total;
         u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = u / Kseg;  // output row (n over all matrices)
        const int k = static_cast<int>(u - r * Kseg);
        const int64_t mat = r / N, n = r - mat * N;
        const float x = k < K ? __ldg(src + mat * mat_stride_src + static_cast<int64_t>(k) * ld_src + n) : 0.f;
        __half h, l;
        split2(x, s, h, l);
        __half* dp = dst + r * (3 * static_cast<int64_t>(Kseg)) + k;
        for (int seg = 0; seg < 3; seg++) dp[static_cast<int64_t>(seg) * Kseg] = seg == lo_seg ? l : h;
    }
}

struct Matmul32Plan {
    Plan pl;          // batch / broadcast resolution of the plain descriptor
    int64_t Kseg;     // contraction extent of one term, rounded up to 64
    int b_mn;         // right operand keeps its K x N layout (N > 32)
    size_t a_bytes, b_bytes, misc_bytes, total;
};

static int plan_matmul32(const nzb_gemm_desc* d, Matmul32Plan* m) {
    int rc = make_plan(d, &m->pl);
    if (rc != NZB_OK) return rc;
    const Plan& pl = m->pl;
    m->Kseg = round_up(pl.K > 0 ? pl.K : 1, 64);
    m->b_mn = pl.N > 32 ? 1 : 0;
    const int64_t nA = pl.nA0 * pl.nA1, nB = pl.nB0 * pl.nB1;
    m->a_bytes = (size_t)round_up(nA * pl.M * 3 * m->Kseg * 2, 256);
    m->b_bytes = (size_t)round_up(nB * (m->b_mn ? 3 * m->Kseg * pl.Np : pl.N * 3 * m->Kseg) * 2, 256);
    m->misc_bytes = 256;  // two magnitude words, three scales
    m->total = m->a_bytes + m->b_bytes + m->misc_bytes;
    return NZB_OK;
}

static int desc_for_shapes(const int64_t* sa, const int64_t* sb, const int64_t* sc, nzb_gemm_desc* d) {
    if (!sa || !sb || !sc) return fail(NZB_ERR_BAD_ARG, "shape pointer is null");
    for (int i = 0; i < 4; i++)
        if (sa[i] < 0 || sb[i] < 0 || sc[i] < 0) return fail(NZB_ERR_BAD_ARG, "negative extent");
    *d = nzb_gemm_desc{};
    d->M = sa[2]; d->K = sa[3]; d->N = sb[3];
    if (sb[2] != d->K) return fail(NZB_ERR_BAD_ARG, "A.W (%lld) != B.H (%lld)", (long long)sa[3], (long long)sb[2]);
    if (sc[2] != d->M || sc[3] != d->N) return fail(NZB_ERR_BAD_ARG, "C matrix extent does not match A.H x B.W");
    d->lda = d->K; d->ldb = d->N; d->ldc = d->N;
    for (int k = 0; k < 2; k++) {
        const int64_t a = sa[k], b = sb[k], c = sc[k], e = a > b ? a : b;
        if (a < 1 || b < 1 || c != e || (a != e && a != 1) || (b != e && b != 1))
            return fail(NZB_ERR_BAD_ARG, "batch extents are not broadcast compatible");
        if (e > INT32_MAX) return fail(NZB_ERR_UNSUPPORTED, "batch extent exceeds 2^31");
        d->batch[k] = (int32_t)e;
    }
    d->strideA[0] = sa[0] > 1 ? sa[1] * d->M * d->K : 0;
    d->strideA[1] = sa[1] > 1 ? d->M * d->K : 0;
    d->strideB[0] = sb[0] > 1 ? sb[1] * d->K * d->N : 0;
    d->strideB[1] = sb[1] > 1 ? d->K * d->N : 0;
    d->strideC[0] = sc[0] > 1 ? sc[1] * d->M * d->N : 0;
    d->strideC[1] = sc[1] > 1 ? d->M * d->N : 0;
    return NZB_OK;
}

}  // namespace nzb

using namespace nzb;

extern "C" {

int nzb_matmul_f32_workspace_bytes(const int64_t shapeA[4], const int64_t shapeB[4], const int64_t shapeC[4],
                                   size_t* bytes_out) {
    if (!bytes_out) return fail(NZB_ERR_BAD_ARG, "bytes_out is null");
    nzb_gemm_desc d;
    int rc = desc_for_shapes(shapeA, shapeB, shapeC, &d);
    if (rc != NZB_OK) return rc;
    Matmul32Plan m;
    rc = plan_matmul32(&d, &m);
    if (rc != NZB_OK) return rc;
    *bytes_out = m.total;
    return NZB_OK;
}

int nzb_matmul_f32(const float* A, const float* B, float* C, const int64_t shapeA[4], const int64_t shapeB[4],
                   const int64_t shapeC[4], void* workspace, size_t workspace_bytes, void* stream) {
    nzb_gemm_desc d;
    int rc = desc_for_shapes(shapeA, shapeB, shapeC, &d);
    if (rc != NZB_OK) return rc;
    Matmul32Plan m;
    rc = plan_matmul32(&d, &m);
    if (rc != NZB_OK) return rc;
    if (d.M == 0 || d.N == 0) return NZB_OK;
    if (!A || !B || !C) return fail(NZB_ERR_BAD_ARG, "A, B and C must be non-null");
    if (d.K == 0) return fail(NZB_ERR_UNSUPPORTED, "K = 0 is not supported");
    if (3 * m.Kseg > INT32_MAX - 256) return fail(NZB_ERR_UNSUPPORTED, "contraction extent too large");
    if (!workspace || workspace_bytes < m.total)
        return fail(NZB_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", m.total, workspace ? workspace_bytes : (size_t)0);
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(NZB_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    DeviceState* ds;
    rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const Plan& pl = m.pl;
    uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
    __half* A16 = reinterpret_cast<__half*>(base);
    __half* B16 = reinterpret_cast<__half*>(base + m.a_bytes);
    unsigned* amax = reinterpret_cast<unsigned*>(base + m.a_bytes + m.b_bytes);
    float* scales = reinterpret_cast<float*>(amax + 8);
    const int64_t nA = pl.nA0 * pl.nA1, nB = pl.nB0 * pl.nB1;
    const int64_t a_elems = nA * pl.M * pl.K, b_elems = nB * pl.K * pl.N;  // contiguous NeuZephyr tensors
    const int blocks = ds->sm_count * 8;
    NZB_CUDA_TRY(cudaMemsetAsync(amax, 0, 32, s));
    absmax_kernel<<<blocks, 256, 0, s>>>(A, a_elems, amax);
    absmax_kernel<<<blocks, 256, 0, s>>>(B, b_elems, amax + 1);
    split_scales_kernel<<<1, 32, 0, s>>>(amax, scales);
    // A: rows x K, terms hi | lo | hi; B: lo ; hi ; hi. The source matrices of an operand are contiguous.
    split_kmajor_kernel<<<blocks, 256, 0, s>>>(A, A16, pl.M, (int)pl.K, d.lda, (int)m.Kseg, 1, nA, pl.M * pl.K, scales);
    if (m.b_mn)
        split_mnmajor_kernel<<<blocks, 256, 0, s>>>(B, B16, (int)pl.K, pl.N, d.ldb, (int)m.Kseg, pl.Np, 0, nB,
                                                    pl.K * pl.N, scales + 1);
    else
        split_transpose_kernel<<<blocks, 256, 0, s>>>(B, B16, (int)pl.K, pl.N, d.ldb, (int)m.Kseg, 0, nB, pl.K * pl.N,
                                                      scales + 1);
    NZB_CUDA_TRY(cudaGetLastError());
    GemmLaunch g = pl.g;
    g.A16 = A16;
    g.B16 = B16;
    g.K = 3 * m.Kseg;
    g.Kp = 3 * m.Kseg;
    g.a_mn = 0;
    g.b_mn = m.b_mn;
    g.ldb16 = pl.Np;
    g.C = C;
    g.alpha = scales + 2;
    return launch_gemm_on(g, *ds, s);
}

}  // extern "C"
