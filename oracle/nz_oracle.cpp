// Host restatement of NeuZephyr's dense-contraction path (TEST INFRASTRUCTURE ONLY).
//
// This file is the correctness oracle and the timed CPU baseline. It is never
// linked into, loaded by, or called from the product library: only the test
// suite, the smoke check and the benchmark's cpu_baseline / reference legs may
// load it. Every function cites the reference source it restates
// (paths relative to the NeuZephyr source tree).
//
// Parity status: pinned. The literal vectors of the reference's own GoogleTest
// cases (test/Test.cpp) are replayed against these functions by
// tests/test_oracle_kat.py.
//
// Build: g++ -O3 -fopenmp -shared -fPIC nz_oracle.cpp -o libnz_oracle.so
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

#define NZO_API extern "C" __attribute__((visibility("default")))
#if defined(__x86_64__)
#define NZO_CLONES __attribute__((target_clones("avx512f", "avx2", "default")))
#else
#define NZO_CLONES
#endif

typedef int64_t i64;

// ---------------------------------------------------------------------------
// fp16 rounding: what Padding does with __float2half (round-to-nearest-even),
// src/OperationKernels.cu:846-860. Bit-level so that it does not depend on the
// host having F16C.
// ---------------------------------------------------------------------------
static inline uint16_t f32_to_f16_bits(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7c00u | ((x > 0x7f800000u) ? 0x0200u : 0u));
    }
    if (x >= 0x477ff000u) {  // rounds to >= 65520 -> inf
        return (uint16_t)(sign | 0x7c00u);
    }
    if (x < 0x38800000u) {  // subnormal half or zero
        if (x < 0x33000000u) return (uint16_t)sign;  // < 2^-25 -> 0 (ties at 2^-25 go to even = 0)
        const int e = (int)(x >> 23);                // biased exponent, 102..112
        uint32_t m = (x & 0x7fffffu) | 0x800000u;    // 24-bit significand
        const int shift = 126 - e;                   // bits to drop so that 1 ulp = 2^-24
        const uint32_t half_ulp = 1u << (shift - 1);
        const uint32_t rem = m & ((1u << shift) - 1);
        uint32_t r = m >> shift;
        if (rem > half_ulp || (rem == half_ulp && (r & 1u))) r++;
        return (uint16_t)(sign | r);
    }
    // normal half
    uint32_t r = x - 0x38000000u;  // rebias exponent 127 -> 15
    const uint32_t rem = r & 0x1fffu;
    r >>= 13;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) r++;
    return (uint16_t)(sign | r);
}

static inline float f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu;
    uint32_t x;
    if (e == 0) {
        if (m == 0) {
            x = sign;
        } else {
            int s = 0;
            while (!(m & 0x400u)) { m <<= 1; s++; }
            m &= 0x3ffu;
            x = sign | ((uint32_t)(113 - s) << 23) | (m << 13);
        }
    } else if (e == 31) {
        x = sign | 0x7f800000u | (m << 13);
    } else {
        x = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}

static inline float round_f16(float f) { return f16_bits_to_f32(f32_to_f16_bits(f)); }

NZO_API void nzo_round_f16(const float* in, float* out, i64 n) {
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; i++) out[i] = round_f16(in[i]);
}

NZO_API void nzo_f32_to_f16_bits(const float* in, uint16_t* out, i64 n) {
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; i++) out[i] = f32_to_f16_bits(in[i]);
}

NZO_API int nzo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// ---------------------------------------------------------------------------
// Single-matrix kernels. op(A) is M x K, op(B) is K x N, C is M x N, all
// row-major with leading dimensions. acc64 != 0 accumulates in double (the
// ground truth); otherwise in float (the timed CPU baseline, same arithmetic
// class as the fp32 accumulators of the WMMA fragments,
// src/OperationKernels.cu:834-841).
// ---------------------------------------------------------------------------
NZO_CLONES
static void gemm_f32_rowmajor(const float* A, i64 lda, const float* B, i64 ldb, float* C, i64 ldc,
                              i64 M, i64 N, i64 K, int add) {
    // i-k-j ordering with row blocking: the inner loop is a contiguous axpy
    // that the compiler vectorises. Threads split rows.
    const i64 KB = 256, NB = 1024;
#pragma omp parallel
    {
        std::vector<float> acc((size_t)NB);
#pragma omp for schedule(dynamic, 4)
        for (i64 i = 0; i < M; i++) {
            for (i64 j0 = 0; j0 < N; j0 += NB) {
                const i64 jn = std::min(NB, N - j0);
                float* __restrict__ a = acc.data();
                for (i64 j = 0; j < jn; j++) a[j] = 0.f;
                for (i64 k0 = 0; k0 < K; k0 += KB) {
                    const i64 kn = std::min(KB, K - k0);
                    for (i64 k = 0; k < kn; k++) {
                        const float av = A[i * lda + k0 + k];
                        const float* __restrict__ b = B + (k0 + k) * ldb + j0;
                        for (i64 j = 0; j < jn; j++) a[j] += av * b[j];
                    }
                }
                float* c = C + i * ldc + j0;
                if (add) for (i64 j = 0; j < jn; j++) c[j] += a[j];
                else     for (i64 j = 0; j < jn; j++) c[j] = a[j];
            }
        }
    }
}

NZO_CLONES
static void gemm_f64_rowmajor(const float* A, i64 lda, const float* B, i64 ldb, double* C, i64 ldc,
                              i64 M, i64 N, i64 K) {
    const i64 NB = 512;
#pragma omp parallel
    {
        std::vector<double> acc((size_t)NB);
#pragma omp for schedule(dynamic, 4)
        for (i64 i = 0; i < M; i++) {
            for (i64 j0 = 0; j0 < N; j0 += NB) {
                const i64 jn = std::min(NB, N - j0);
                double* __restrict__ a = acc.data();
                for (i64 j = 0; j < jn; j++) a[j] = 0.0;
                for (i64 k = 0; k < K; k++) {
                    const double av = (double)A[i * lda + k];
                    const float* __restrict__ b = B + k * ldb + j0;
                    for (i64 j = 0; j < jn; j++) a[j] += av * (double)b[j];
                }
                double* c = C + i * ldc + j0;
                for (i64 j = 0; j < jn; j++) c[j] = a[j];
            }
        }
    }
}

// C(double, M x N) = A(M x K) * B(K x N), optional fp16 rounding of operands.
NZO_API void nzo_gemm_f64(const float* A, const float* B, double* C, i64 M, i64 N, i64 K, int round_operands) {
    std::vector<float> Ar, Br;
    if (round_operands) {
        Ar.resize((size_t)(M * K));
        Br.resize((size_t)(K * N));
        nzo_round_f16(A, Ar.data(), M * K);
        nzo_round_f16(B, Br.data(), K * N);
        A = Ar.data();
        B = Br.data();
    }
    gemm_f64_rowmajor(A, K, B, N, C, N, M, N, K);
}

// Selected rows of C only (for the sampled check of large problems):
// Crows[r, :] = A[rows[r], :] * B.
NZO_API void nzo_gemm_f64_rows(const float* A, const float* B, double* Crows, const i64* rows, i64 nrows,
                               i64 M, i64 N, i64 K, int round_operands) {
    (void)M;
    std::vector<float> Ar((size_t)(nrows * K));
    for (i64 r = 0; r < nrows; r++)
        for (i64 k = 0; k < K; k++) {
            const float v = A[rows[r] * K + k];
            Ar[(size_t)(r * K + k)] = round_operands ? round_f16(v) : v;
        }
    std::vector<float> Br;
    if (round_operands) {
        Br.resize((size_t)(K * N));
        nzo_round_f16(B, Br.data(), K * N);
        B = Br.data();
    }
    gemm_f64_rowmajor(Ar.data(), K, B, N, Crows, N, nrows, N, K);
}

// ---------------------------------------------------------------------------
// Batched forward GEMM over the (N, C) batch grid with per-dimension broadcast:
// restates krnl::TensorCoreGEMMParallel (src/OperationKernels.cu:914-1026):
//  * M = A.H, K = A.W, N = B.W                               (:918-920)
//  * operands rounded to fp16, zero padded to multiples of 16 (:943-973; the
//    zero padding contributes nothing to the sums and is not materialised)
//  * C has max(A.N,B.N) x max(A.C,B.C) matrices; an operand whose N (or C)
//    extent is 1 is reused for every index of that dimension  (:978-986)
//  * the result OVERWRITES C (Cutting, :862-871, :1012-1019)
// shapeX = {N, C, H, W}. acc64: 0 = float accumulation into C (float*),
// 1 = double accumulation, result stored to Cd (double*).
// ---------------------------------------------------------------------------
static void batched_gemm(const float* A, const float* B, float* C, double* Cd,
                         const i64* shapeA, const i64* shapeB, const i64* shapeC,
                         int round_operands, int backward) {
    const i64 M = shapeA[2], K = shapeA[3], N = shapeB[3];
    const i64 aN = shapeA[0], aC = shapeA[1], bN = shapeB[0], bC = shapeB[1];
    const i64 cN = shapeC[0], cC = shapeC[1];
    const i64 pN = std::max(aN, bN), pC = std::max(aC, bC);  // padded_C_shape of the backward driver (:1040-1041)
    std::vector<float> Ar, Br;
    if (round_operands) {
        Ar.resize((size_t)(aN * aC * M * K));
        Br.resize((size_t)(bN * bC * K * N));
        nzo_round_f16(A, Ar.data(), aN * aC * M * K);
        nzo_round_f16(B, Br.data(), bN * bC * K * N);
        A = Ar.data();
        B = Br.data();
    }
    const i64 nI = backward ? pN : cN, nJ = backward ? pC : cC;
    std::vector<double> tmp;
    std::vector<float> tmpf;
    if (Cd) tmp.resize((size_t)(M * N)); else if (backward) tmpf.resize((size_t)(M * N));
    for (i64 i = 0; i < nI; i++) {
        for (i64 j = 0; j < nJ; j++) {
            const i64 offA = (aN > 1 ? i * aC * M * K : 0) + (aC > 1 ? j * M * K : 0);
            const i64 offB = (bN > 1 ? i * bC * K * N : 0) + (bC > 1 ? j * K * N : 0);
            // forward: every C matrix is written once (:1006-1019);
            // backward: C offset is 0 along a dimension of extent 1, which sums
            // the products of all broadcast batches (:1121-1137, CuttingAndCompress :873-883)
            const i64 offC = backward ? ((cN > 1 ? i * cC * M * N : 0) + (cC > 1 ? j * M * N : 0))
                                      : (i * cC * M * N + j * M * N);
            if (Cd) {
                gemm_f64_rowmajor(A + offA, K, B + offB, N, tmp.data(), N, M, N, K);
                double* c = Cd + offC;
                if (backward) for (i64 t = 0; t < M * N; t++) c[t] += tmp[(size_t)t];
                else          for (i64 t = 0; t < M * N; t++) c[t] = tmp[(size_t)t];
            } else if (backward) {
                // the reference forms the full product first and then atomically adds it
                gemm_f32_rowmajor(A + offA, K, B + offB, N, tmpf.data(), N, M, N, K, 0);
                float* c = C + offC;
                for (i64 t = 0; t < M * N; t++) c[t] += tmpf[(size_t)t];
            } else {
                gemm_f32_rowmajor(A + offA, K, B + offB, N, C + offC, N, M, N, K, 0);
            }
        }
    }
}

NZO_API void nzo_gemm_forward(const float* A, const float* B, float* C, const i64* shapeA, const i64* shapeB,
                              const i64* shapeC, int round_operands) {
    batched_gemm(A, B, C, nullptr, shapeA, shapeB, shapeC, round_operands, 0);
}
NZO_API void nzo_gemm_forward_f64(const float* A, const float* B, double* C, const i64* shapeA, const i64* shapeB,
                                  const i64* shapeC, int round_operands) {
    batched_gemm(A, B, nullptr, C, shapeA, shapeB, shapeC, round_operands, 0);
}
// Restates krnl::GEMMBackwardParallel (src/OperationKernels.cu:1028-1144): same
// products, ACCUMULATED into C (which the caller must have initialised).
NZO_API void nzo_gemm_backward(const float* A, const float* B, float* C, const i64* shapeA, const i64* shapeB,
                               const i64* shapeC, int round_operands) {
    batched_gemm(A, B, C, nullptr, shapeA, shapeB, shapeC, round_operands, 1);
}
NZO_API void nzo_gemm_backward_f64(const float* A, const float* B, double* C, const i64* shapeA, const i64* shapeB,
                                   const i64* shapeC, int round_operands) {
    batched_gemm(A, B, nullptr, C, shapeA, shapeB, shapeC, round_operands, 1);
}

// Per-matrix transpose of an {N,C,H,W} tensor -> {N,C,W,H}
// (TransposeKernel, src/OperationKernels.cu:125-160; transpose<T>,
// include/NeuZephyr/TensorOperations.cuh:1071-1086).
NZO_API void nzo_transpose(const float* in, float* out, i64 batches, i64 H, i64 W) {
#pragma omp parallel for schedule(static)
    for (i64 b = 0; b < batches; b++)
        for (i64 h = 0; h < H; h++)
            for (i64 w = 0; w < W; w++) out[b * H * W + w * H + h] = in[b * H * W + h * W + w];
}

// ---------------------------------------------------------------------------
// im2col / col2img (src/OperationKernels.cu:1308-1402)
// ---------------------------------------------------------------------------
// out[b][ho*Wo+wo][c*Kh*Kw + kh*Kw + kw] = in[b][c][ho*s-p+kh][wo*s-p+kw] or 0 (:1308-1328)
NZO_API void nzo_img2col(float* out, const float* in, i64 H_out, i64 W_out, i64 C, i64 K_h, i64 K_w,
                         i64 stride, i64 pad, i64 H_in, i64 W_in, i64 batch) {
    const i64 KK = C * K_h * K_w;
#pragma omp parallel for collapse(2) schedule(static)
    for (i64 b = 0; b < batch; b++)
        for (i64 k = 0; k < H_out * W_out; k++) {
            float* o = out + (b * H_out * W_out + k) * KK;
            for (i64 m = 0; m < KK; m++) {
                const i64 c = m / (K_h * K_w);
                const i64 h = (k / W_out) * stride - pad + (m % (K_h * K_w)) / K_w;
                const i64 w = (k % W_out) * stride - pad + m % K_w;
                o[m] = (h >= 0 && h < H_in && w >= 0 && w < W_in)
                           ? in[b * C * H_in * W_in + c * H_in * W_in + h * W_in + w] : 0.f;
            }
        }
}

// dX += scatter(dcol) (:1337-1355). Accumulates into out (the reference uses atomicAdd on
// a gradient buffer that the caller zeroed). Summation here is in double per target
// element to give an order-independent ground truth, then added once.
NZO_API void nzo_img2col_backward(float* out, const float* in, i64 H_out, i64 W_out, i64 C, i64 K_h, i64 K_w,
                                  i64 stride, i64 pad, i64 H_in, i64 W_in, i64 batch) {
    const i64 KK = C * K_h * K_w;
#pragma omp parallel for collapse(2) schedule(static)
    for (i64 b = 0; b < batch; b++)
        for (i64 c = 0; c < C; c++) {
            std::vector<double> acc((size_t)(H_in * W_in), 0.0);
            for (i64 k = 0; k < H_out * W_out; k++)
                for (i64 r = 0; r < K_h * K_w; r++) {
                    const i64 h = (k / W_out) * stride - pad + r / K_w;
                    const i64 w = (k % W_out) * stride - pad + r % K_w;
                    if (h >= 0 && h < H_in && w >= 0 && w < W_in)
                        acc[(size_t)(h * W_in + w)] += (double)in[(b * H_out * W_out + k) * KK + c * K_h * K_w + r];
                }
            float* o = out + b * C * H_in * W_in + c * H_in * W_in;
            for (i64 t = 0; t < H_in * W_in; t++) o[t] += (float)acc[(size_t)t];
        }
}

// NHWC-like [b][h*Wo+w][c] -> NCHW [b][c][h][w] (:1364-1376)
NZO_API void nzo_col2img(float* out, const float* in, i64 H_out, i64 W_out, i64 C_out, i64 batches) {
    const i64 HW = H_out * W_out;
#pragma omp parallel for collapse(2) schedule(static)
    for (i64 b = 0; b < batches; b++)
        for (i64 c = 0; c < C_out; c++)
            for (i64 p = 0; p < HW; p++) out[b * C_out * HW + c * HW + p] = in[b * C_out * HW + p * C_out + c];
}

// inverse permutation, OVERWRITES out (:1384-1396)
NZO_API void nzo_col2img_backward(float* out, const float* in, i64 H_out, i64 W_out, i64 C_out, i64 batches) {
    const i64 HW = H_out * W_out;
#pragma omp parallel for collapse(2) schedule(static)
    for (i64 b = 0; b < batches; b++)
        for (i64 p = 0; p < HW; p++)
            for (i64 c = 0; c < C_out; c++) out[b * C_out * HW + p * C_out + c] = in[b * C_out * HW + c * HW + p];
}

// ---------------------------------------------------------------------------
// Broadcast add and its backward (AddNode, src/Nodes.cu:95-146; MatrixAddKernel
// src/OperationKernels.cu:12-37; gradCopyKernel :1230-1236).
// ---------------------------------------------------------------------------
// out{max N, max C, H, W} = a + b with N/C broadcast.
NZO_API void nzo_add_broadcast(float* out, const float* a, const float* b, const i64* shapeA, const i64* shapeB) {
    const i64 oN = std::max(shapeA[0], shapeB[0]), oC = std::max(shapeA[1], shapeB[1]);
    const i64 HW = shapeA[2] * shapeA[3];
    for (i64 i = 0; i < oN; i++)
        for (i64 j = 0; j < oC; j++) {
            const float* pa = a + ((shapeA[0] > 1 ? i * shapeA[1] : 0) + (shapeA[1] > 1 ? j : 0)) * HW;
            const float* pb = b + ((shapeB[0] > 1 ? i * shapeB[1] : 0) + (shapeB[1] > 1 ? j : 0)) * HW;
            float* po = out + (i * oC + j) * HW;
#pragma omp parallel for schedule(static)
            for (i64 t = 0; t < HW; t++) po[t] = pa[t] + pb[t];
        }
}

// Gradient of one input of the add. Same shape: copy (overwrite, Nodes.cu:101-105).
// Broadcast input: gin += sum over the broadcast batch slices of gout (Nodes.cu:106-121).
// The reference issues one unsynchronised "+=" launch per slice; the defined result
// is the sum, taken here in double.
NZO_API void nzo_add_backward(float* gin, const float* gout, const i64* shapeIn, const i64* shapeOut) {
    const i64 HW = shapeOut[2] * shapeOut[3];
    const i64 oN = shapeOut[0], oC = shapeOut[1];
    if (shapeIn[0] == oN && shapeIn[1] == oC) {
        std::memcpy(gin, gout, sizeof(float) * (size_t)(oN * oC * HW));
        return;
    }
    const i64 nIn = shapeIn[0] * shapeIn[1];
    std::vector<double> acc((size_t)(nIn * HW), 0.0);
    for (i64 i = 0; i < oN; i++)
        for (i64 j = 0; j < oC; j++) {
            const i64 oi = (shapeIn[0] > 1 ? i * shapeIn[1] : 0) + (shapeIn[1] > 1 ? j : 0);
            const float* g = gout + (i * oC + j) * HW;
            double* a = acc.data() + oi * HW;
            for (i64 t = 0; t < HW; t++) a[t] += (double)g[t];
        }
    for (i64 t = 0; t < nIn * HW; t++) gin[t] += (float)acc[(size_t)t];
}

// ReLU (src/OperationKernels.cu:230-248). Backward OVERWRITES.
NZO_API void nzo_relu(float* out, const float* in, i64 n) {
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; i++) out[i] = in[i] > 0.f ? in[i] : 0.f;
}
NZO_API void nzo_relu_backward(float* gin, const float* x, const float* gout, i64 n) {
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; i++) gin[i] = x[i] > 0.f ? gout[i] : 0.f;
}

// ---------------------------------------------------------------------------
// Average pooling (src/OperationKernels.cu:1404-1482): the divisor counts only
// in-bounds taps. Backward ACCUMULATES into gin.
// ---------------------------------------------------------------------------
NZO_API void nzo_avgpool(float* out, const float* in, i64 pool, i64 stride, i64 pad, i64 batches, i64 channels,
                         i64 H_in, i64 W_in, i64 H_out, i64 W_out) {
#pragma omp parallel for schedule(static)
    for (i64 bc = 0; bc < batches * channels; bc++)
        for (i64 h = 0; h < H_out; h++)
            for (i64 w = 0; w < W_out; w++) {
                float s = 0.f;
                i64 cnt = 0;
                for (i64 i = 0; i < pool; i++)
                    for (i64 j = 0; j < pool; j++) {
                        const i64 hi = h * stride - pad + i, wi = w * stride - pad + j;
                        if (hi >= 0 && hi < H_in && wi >= 0 && wi < W_in) {
                            s += in[bc * H_in * W_in + hi * W_in + wi];
                            cnt++;
                        }
                    }
                out[bc * H_out * W_out + h * W_out + w] = cnt > 0 ? s / (float)cnt : 0.f;
            }
}

NZO_API void nzo_avgpool_backward(float* gin, const float* gout, i64 pool, i64 stride, i64 pad, i64 batches,
                                  i64 channels, i64 H_in, i64 W_in, i64 H_out, i64 W_out) {
#pragma omp parallel for schedule(static)
    for (i64 bc = 0; bc < batches * channels; bc++) {
        std::vector<double> acc((size_t)(H_in * W_in), 0.0);
        for (i64 h = 0; h < H_out; h++)
            for (i64 w = 0; w < W_out; w++) {
                i64 cnt = 0;
                for (i64 i = 0; i < pool; i++)
                    for (i64 j = 0; j < pool; j++) {
                        const i64 hi = h * stride - pad + i, wi = w * stride - pad + j;
                        if (hi >= 0 && hi < H_in && wi >= 0 && wi < W_in) cnt++;
                    }
                // without padding the reference divides by pool*pool (:1457); with padding by the count (:1477)
                const float div = pad ? (float)cnt : (float)(pool * pool);
                const float g = gout[bc * H_out * W_out + h * W_out + w] / div;
                for (i64 i = 0; i < pool; i++)
                    for (i64 j = 0; j < pool; j++) {
                        const i64 hi = h * stride - pad + i, wi = w * stride - pad + j;
                        if (hi >= 0 && hi < H_in && wi >= 0 && wi < W_in) acc[(size_t)(hi * W_in + wi)] += (double)g;
                    }
            }
        float* o = gin + bc * H_in * W_in;
        for (i64 t = 0; t < H_in * W_in; t++) o[t] += (float)acc[(size_t)t];
    }
}

// Max pooling (MaxPoolingKernel / MaxPoolingBackwardKernel, src/OperationKernels.cu:1507-1573): first
// maximum in row-major window order (strict >), its window index stored as a float; empty window -> 0.
NZO_API void nzo_maxpool(float* out, float* position, const float* in, i64 pool, i64 stride, i64 pad, i64 batches,
                         i64 channels, i64 H_in, i64 W_in, i64 H_out, i64 W_out) {
#pragma omp parallel for schedule(static)
    for (i64 bc = 0; bc < batches * channels; bc++)
        for (i64 h = 0; h < H_out; h++)
            for (i64 w = 0; w < W_out; w++) {
                float best = -1e20f;
                i64 best_i = 0;
                for (i64 i = 0; i < pool; i++)
                    for (i64 j = 0; j < pool; j++) {
                        const i64 hi = h * stride - pad + i, wi = w * stride - pad + j;
                        if (hi >= 0 && hi < H_in && wi >= 0 && wi < W_in) {
                            const float v = in[bc * H_in * W_in + hi * W_in + wi];
                            if (v > best) {
                                best = v;
                                best_i = i * pool + j;
                            }
                        }
                    }
                out[bc * H_out * W_out + h * W_out + w] = best == -1e20f ? 0.f : best;
                position[bc * H_out * W_out + h * W_out + w] = (float)best_i;
            }
}
// gin += scatter of gout to the recorded maxima (the reference's atomicAdd), summed in double per element
NZO_API void nzo_maxpool_backward(float* gin, const float* position, const float* gout, i64 pool, i64 stride, i64 pad,
                                  i64 batches, i64 channels, i64 H_in, i64 W_in, i64 H_out, i64 W_out) {
#pragma omp parallel for schedule(static)
    for (i64 bc = 0; bc < batches * channels; bc++) {
        std::vector<double> acc((size_t)(H_in * W_in), 0.0);
        for (i64 h = 0; h < H_out; h++)
            for (i64 w = 0; w < W_out; w++) {
                const i64 o = bc * H_out * W_out + h * W_out + w;
                const i64 idx = (i64)position[o];
                const i64 hi = h * stride - pad + idx / pool, wi = w * stride - pad + idx % pool;
                if (hi >= 0 && hi < H_in && wi >= 0 && wi < W_in) acc[(size_t)(hi * W_in + wi)] += (double)gout[o];
            }
        float* g = gin + bc * H_in * W_in;
        for (i64 t = 0; t < H_in * W_in; t++) g[t] += (float)acc[(size_t)t];
    }
}

// ---------------------------------------------------------------------------
// Softmax over each {H,W} matrix flattened (n = H*W), no max subtraction
// (src/OperationKernels.cu:477-523, include/NeuZephyr/TensorOperations.cuh:379-392),
// its Jacobian (:536-553) and the node backward dX = J * dY, which the reference
// evaluates with the fp16 tensor-core GEMM (src/Nodes.cu:538-548).
// ---------------------------------------------------------------------------
NZO_API void nzo_softmax(float* out, const float* in, i64 batches, i64 n) {
    for (i64 b = 0; b < batches; b++) {
        double s = 0.0;
        for (i64 i = 0; i < n; i++) s += std::exp((double)in[b * n + i]);
        for (i64 i = 0; i < n; i++) out[b * n + i] = (float)(std::exp((double)in[b * n + i]) / s);
    }
}
NZO_API void nzo_softmax_jacobian(float* out, const float* y, i64 batches, i64 n) {
    for (i64 b = 0; b < batches; b++)
        for (i64 i = 0; i < n; i++)
            for (i64 j = 0; j < n; j++) {
                const float yi = y[b * n + i], yj = y[b * n + j];
                out[b * n * n + i * n + j] = (i == j) ? yi * (1.f - yi) : -yi * yj;
            }
}
// dX = J(y) * dY per batch, in double; round_operands rounds J and dY to fp16 first as the
// reference's GEMM does. OVERWRITES gin.
NZO_API void nzo_softmax_backward(float* gin, const float* y, const float* gout, i64 batches, i64 n,
                                  int round_operands) {
    for (i64 b = 0; b < batches; b++)
        for (i64 i = 0; i < n; i++) {
            double s = 0.0;
            for (i64 j = 0; j < n; j++) {
                const float yi = y[b * n + i], yj = y[b * n + j];
                float Jij = (i == j) ? yi * (1.f - yi) : -yi * yj;
                float g = gout[b * n + j];
                if (round_operands) { Jij = round_f16(Jij); g = round_f16(g); }
                s += (double)Jij * (double)g;
            }
            gin[b * n + i] = (float)s;
        }
}

// ---------------------------------------------------------------------------
// Binary cross-entropy, mean over all n elements (src/OperationKernels.cu:648-699).
// ---------------------------------------------------------------------------
NZO_API double nzo_bce(const float* predict, const float* real, i64 n) {
    double s = 0.0;
    for (i64 i = 0; i < n; i++)
        s += (-(double)real[i] * std::log((double)predict[i]) -
              (1.0 - (double)real[i]) * std::log(1.0 - (double)predict[i])) / (double)n;
    return s;
}
NZO_API void nzo_bce_backward(float* out, const float* predict, const float* real, i64 n) {
    for (i64 i = 0; i < n; i++) {
        const double p = predict[i], t = real[i];
        out[i] = (float)(((p - t) / (p * (1.0 - p))) / (double)n);
    }
}

// ---------------------------------------------------------------------------
// Adam (src/OperationKernels.cu:753-766; opt::Adam::step src/Optimizer.cu:86-102,
// default eps 1e-6). t is the value the optimizer's counter holds for this call.
// ---------------------------------------------------------------------------
NZO_API void nzo_adam(float* data, float* m, float* v, const float* grad, float lr, float beta1, float beta2,
                      float eps, int t, i64 n) {
    const double c1 = 1.0 - std::pow((double)beta1, (double)t);
    const double c2 = 1.0 - std::pow((double)beta2, (double)t);
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; i++) {
        const float g = grad[i];
        const float mt = m[i] * beta1 + g * (1.f - beta1);
        const float vt = v[i] * beta2 + g * g * (1.f - beta2);
        const double mh = (double)mt / c1, vh = (double)vt / c2;
        data[i] -= (float)((double)lr * mh / (std::sqrt(vh) + (double)eps));
        m[i] = mt;
        v[i] = vt;
    }
}

// ---------------------------------------------------------------------------
// Conv2d forward / backward as the reference composes it
// (Model::Conv2d, src/Model.cu:244-263): Img2Col -> MatMul(col, W) -> [+bias] -> Col2Img.
//   x   {N, C, H, W}            NCHW
//   w   {wN, 1, C*Kh*Kw, Cout}  row-major [K][Cout]; wN = 1 (shared) or N (one per sample)
//   bias {1, 1, Ho*Wo, Cout} or null
//   y   {N, Cout, Ho, Wo}
// Double accumulation with optional fp16 rounding of both GEMM operands.
// relu applies max(.,0) to y.
// ---------------------------------------------------------------------------
NZO_API void nzo_conv2d_forward(float* y, const float* x, const float* w, const float* bias, i64 N, i64 C, i64 H,
                                i64 W, i64 Cout, i64 Kh, i64 Kw, i64 stride, i64 pad, i64 wN, int round_operands,
                                int relu) {
    const i64 Ho = (H + 2 * pad - Kh) / stride + 1, Wo = (W + 2 * pad - Kw) / stride + 1;
    const i64 KK = C * Kh * Kw;
    std::vector<float> wr((size_t)(wN * KK * Cout));
    for (i64 t = 0; t < wN * KK * Cout; t++) wr[(size_t)t] = round_operands ? round_f16(w[t]) : w[t];
#pragma omp parallel for collapse(2) schedule(static)
    for (i64 b = 0; b < N; b++)
        for (i64 p = 0; p < Ho * Wo; p++) {
            std::vector<double> acc((size_t)Cout, 0.0);
            const float* wb = wr.data() + (wN > 1 ? b * KK * Cout : 0);
            const i64 ho = p / Wo, wo = p % Wo;
            for (i64 c = 0; c < C; c++)
                for (i64 kh = 0; kh < Kh; kh++)
                    for (i64 kw = 0; kw < Kw; kw++) {
                        const i64 h = ho * stride - pad + kh, ww = wo * stride - pad + kw;
                        if (h < 0 || h >= H || ww < 0 || ww >= W) continue;
                        float xv = x[b * C * H * W + c * H * W + h * W + ww];
                        if (round_operands) xv = round_f16(xv);
                        const float* wrow = wb + (c * Kh * Kw + kh * Kw + kw) * Cout;
                        for (i64 o = 0; o < Cout; o++) acc[(size_t)o] += (double)xv * (double)wrow[o];
                    }
            for (i64 o = 0; o < Cout; o++) {
                double v = acc[(size_t)o] + (bias ? (double)bias[p * Cout + o] : 0.0);
                if (relu && v < 0.0) v = 0.0;
                y[b * Cout * Ho * Wo + o * Ho * Wo + p] = (float)v;
            }
        }
}

// Backward of the same composition (col2imgBackward -> AddNode::backward ->
// MatMulNode::backward -> img2colBackward; src/Nodes.cu:660-665, 99-146, 169-182, 632-640).
//   dy {N, Cout, Ho, Wo}
//   dx {N, C, H, W}            += (may be null)
//   dw {wN, 1, K, Cout}        += ; summed over the batch when wN == 1 (may be null)
//   dbias {1,1,Ho*Wo,Cout}     += sum over batch (may be null)
// The GEMM operands (dy, w^T, col^T) are rounded to fp16 when round_operands.
NZO_API void nzo_conv2d_backward(float* dx, float* dw, float* dbias, const float* dy, const float* x, const float* w,
                                 i64 N, i64 C, i64 H, i64 W, i64 Cout, i64 Kh, i64 Kw, i64 stride, i64 pad, i64 wN,
                                 int round_operands) {
    const i64 Ho = (H + 2 * pad - Kh) / stride + 1, Wo = (W + 2 * pad - Kw) / stride + 1;
    const i64 KK = C * Kh * Kw, HW = Ho * Wo;
    if (dbias) {
#pragma omp parallel for schedule(static)
        for (i64 p = 0; p < HW; p++)
            for (i64 o = 0; o < Cout; o++) {
                double s = 0.0;
                for (i64 b = 0; b < N; b++) s += (double)dy[b * Cout * HW + o * HW + p];
                dbias[p * Cout + o] += (float)s;
            }
    }
    if (dw) {
        // dW[k][o] = sum_{b,p} col[b][p][k] * dy[b][o][p]
        std::vector<double> acc((size_t)(wN * KK * Cout), 0.0);
#pragma omp parallel for schedule(static)
        for (i64 k = 0; k < KK; k++) {
            const i64 c = k / (Kh * Kw), kh = (k % (Kh * Kw)) / Kw, kw = k % Kw;
            for (i64 b = 0; b < N; b++) {
                double* a = acc.data() + (wN > 1 ? b * KK * Cout : 0) + k * Cout;
                for (i64 p = 0; p < HW; p++) {
                    const i64 h = (p / Wo) * stride - pad + kh, ww = (p % Wo) * stride - pad + kw;
                    if (h < 0 || h >= H || ww < 0 || ww >= W) continue;
                    float xv = x[b * C * H * W + c * H * W + h * W + ww];
                    if (round_operands) xv = round_f16(xv);
                    for (i64 o = 0; o < Cout; o++) {
                        float g = dy[b * Cout * HW + o * HW + p];
                        if (round_operands) g = round_f16(g);
                        a[o] += (double)xv * (double)g;
                    }
                }
            }
        }
        for (i64 t = 0; t < wN * KK * Cout; t++) dw[t] += (float)acc[(size_t)t];
    }
    if (dx) {
        // dcol[b][p][k] = sum_o dy[b][o][p] * w[k][o]; dx = scatter-add of dcol
#pragma omp parallel for collapse(2) schedule(static)
        for (i64 b = 0; b < N; b++)
            for (i64 c = 0; c < C; c++) {
                std::vector<double> acc((size_t)(H * W), 0.0);
                const float* wb = w + (wN > 1 ? b * KK * Cout : 0);
                for (i64 p = 0; p < HW; p++)
                    for (i64 kh = 0; kh < Kh; kh++)
                        for (i64 kw = 0; kw < Kw; kw++) {
                            const i64 h = (p / Wo) * stride - pad + kh, ww = (p % Wo) * stride - pad + kw;
                            if (h < 0 || h >= H || ww < 0 || ww >= W) continue;
                            const float* wrow = wb + (c * Kh * Kw + kh * Kw + kw) * Cout;
                            double s = 0.0;
                            for (i64 o = 0; o < Cout; o++) {
                                float g = dy[b * Cout * HW + o * HW + p], wv = wrow[o];
                                if (round_operands) { g = round_f16(g); wv = round_f16(wv); }
                                s += (double)g * (double)wv;
                            }
                            acc[(size_t)(h * W + ww)] += s;
                        }
                float* o = dx + b * C * H * W + c * H * W;
                for (i64 t = 0; t < H * W; t++) o[t] += (float)acc[(size_t)t];
            }
    }
}

// ---------------------------------------------------------------------------
// Timed CPU baseline entry: plain C = A*B, fp16-rounded operands, fp32
// accumulation, all OpenMP threads. Rounding is done outside the timed part by
// the caller if desired (pre_rounded != 0).
// ---------------------------------------------------------------------------
NZO_API void nzo_gemm_f32(const float* A, const float* B, float* C, i64 M, i64 N, i64 K, int round_operands) {
    std::vector<float> Ar, Br;
    if (round_operands) {
        Ar.resize((size_t)(M * K));
        Br.resize((size_t)(K * N));
        nzo_round_f16(A, Ar.data(), M * K);
        nzo_round_f16(B, Br.data(), K * N);
        A = Ar.data();
        B = Br.data();
    }
    gemm_f32_rowmajor(A, K, B, N, C, N, M, N, K, 0);
}
