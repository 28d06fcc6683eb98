// Training-step operations beside the contraction kernels: one-launch Adam over all parameters of a
// model, the softmax + binary-cross-entropy head as one forward and one backward kernel, and max
// pooling in gather form. Each names the NeuZephyr code it stands in for (paths relative to the
// NeuZephyr tree). All HBM-bound; 64-bit indexing.
#include <cuda_fp16.h>

#include "nzb_internal.h"

namespace nzb {

// ---- Adam over a list of tensors in ONE launch ---------------------------------------------------
// opt::Adam::step (src/Optimizer.cu:86-102) launches AdamKernel (src/OperationKernels.cu:753-766)
// once per tensor; here a block walks 4096-element chunks of whichever tensor its chunk index falls
// into, with float4 accesses where the tensor allows. Every tensor carries its own time step (the
// reference's counter advances per step() call). Optionally writes the updated weights' fp16 copy
// (round to nearest even), which is what the tensor cores read in the next forward.
constexpr int kAdamMaxTensors = 24;
constexpr int kAdamChunk = 4096;
struct AdamEntry {
    float* data;
    float* m;
    float* v;
    const float* grad;
    __half* shadow;   // optional fp16 copy of the updated data
    int64_t n;
    int64_t first_chunk;  // running sum of ceil(n / kAdamChunk)
    float c1, c2;         // 1 - beta1^t, 1 - beta2^t
};
struct AdamList {
    AdamEntry e[kAdamMaxTensors];
    int count;
    int64_t total_chunks;
    float lr, beta1, beta2, eps;
};

__device__ __forceinline__ float adam_one(float& m, float& v, float p, float g, const AdamList& L, float c1, float c2) {
    return adam_update(p, m, v, g, L.lr, L.beta1, L.beta2, L.eps, c1, c2);
}

__global__ void __launch_bounds__(256) adam_multi_kernel(const __grid_constant__ AdamList L) {
    for (int64_t chunk = blockIdx.x; chunk < L.total_chunks; chunk += gridDim.x) {
        int t = 0;
        while (t + 1 < L.count && L.e[t + 1].first_chunk <= chunk) t++;
        const AdamEntry& e = L.e[t];
        const int64_t i0 = (chunk - e.first_chunk) * kAdamChunk;
        const int64_t n = min(static_cast<int64_t>(kAdamChunk), e.n - i0);
        const bool vec = ((reinterpret_cast<uintptr_t>(e.data) | reinterpret_cast<uintptr_t>(e.m) |
                           reinterpret_cast<uintptr_t>(e.v) | reinterpret_cast<uintptr_t>(e.grad)) & 15) == 0 &&
                         (e.shadow == nullptr || (reinterpret_cast<uintptr_t>(e.shadow) & 7) == 0);
        if (vec) {
            for (int64_t i = i0 + threadIdx.x * 4; i + 3 < i0 + n; i += 256 * 4) {
                float4 p = *reinterpret_cast<float4*>(e.data + i);
                float4 m = *reinterpret_cast<float4*>(e.m + i);
                float4 v = *reinterpret_cast<float4*>(e.v + i);
                const float4 g = __ldcs(reinterpret_cast<const float4*>(e.grad + i));
                p.x = adam_one(m.x, v.x, p.x, g.x, L, e.c1, e.c2);
                p.y = adam_one(m.y, v.y, p.y, g.y, L, e.c1, e.c2);
                p.z = adam_one(m.z, v.z, p.z, g.z, L, e.c1, e.c2);
                p.w = adam_one(m.w, v.w, p.w, g.w, L, e.c1, e.c2);
                *reinterpret_cast<float4*>(e.data + i) = p;
                *reinterpret_cast<float4*>(e.m + i) = m;
                *reinterpret_cast<float4*>(e.v + i) = v;
                if (e.shadow) {
                    const __half2 lo = __floats2half2_rn(p.x, p.y), hi = __floats2half2_rn(p.z, p.w);
                    uint2 u;
                    u.x = *reinterpret_cast<const uint32_t*>(&lo);
                    u.y = *reinterpret_cast<const uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(e.shadow + i) = u;
                }
            }
        }
        // the tail of a chunk that is not a multiple of four, or everything of an unaligned tensor
        const int64_t done = vec ? (n / 4) * 4 : 0;
        for (int64_t i = i0 + done + threadIdx.x; i < i0 + n; i += 256) {
            float m = e.m[i], v = e.v[i];
            const float p = adam_one(m, v, e.data[i], e.grad[i], L, e.c1, e.c2);
            e.data[i] = p;
            e.m[i] = m;
            e.v[i] = v;
            if (e.shadow) e.shadow[i] = __float2half_rn(p);
        }
    }
}

// ---- softmax + binary cross-entropy as one head ----------------------------------------------------
// Forward: SoftmaxKernel after SummationExpKernel (src/OperationKernels.cu:477-523; the row maximum is
// subtracted first, which changes nothing mathematically and keeps large logits finite) and
// BinaryCrossEntropyKernel (:648-699, mean over ALL batches*n elements, added to *loss). One warp per
// vector; n <= 1024.
__global__ void __launch_bounds__(128) softmax_bce_forward_kernel(float* __restrict__ probs, float* __restrict__ loss,
                                                                  const float* __restrict__ logits,
                                                                  const float* __restrict__ target, int64_t batches,
                                                                  int n, float total) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    float part = 0.f;
    for (int64_t b = warp; b < batches; b += nwarps) {
        const float* x = logits + b * n;
        float mx = -INFINITY;
        for (int i = lane; i < n; i += 32) mx = fmaxf(mx, x[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float s = 0.f;
        for (int i = lane; i < n; i += 32) s += expf(x[i] - mx);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        for (int i = lane; i < n; i += 32) {
            const float p = expf(x[i] - mx) / s;
            probs[b * n + i] = p;
            const float t = target[b * n + i];
            part += (-t * logf(p) - (1.f - t) * logf(1.f - p)) / total;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0 && part != 0.f) atomicAdd(loss, part);
}

// Backward of the head: BCEBackwardKernel (src/OperationKernels.cu:701-704), then SoftmaxNode::backward
// (src/Nodes.cu:538-548): dX = J(y) dY with J = diag(y) - y y^T. The reference forms J and runs the
// product through its tensor-core GEMM, so J and dY are rounded to fp16 there; round_f16 reproduces
// that, otherwise the product is the exact fp32 formula y_i (dY_i - sum_j y_j dY_j). OVERWRITES dx.
__global__ void __launch_bounds__(128) softmax_bce_backward_kernel(float* __restrict__ dx, const float* __restrict__ probs,
                                                                   const float* __restrict__ target, int64_t batches,
                                                                   int n, float total, int round_f16) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t b = warp; b < batches; b += nwarps) {
        const float* y = probs + b * n;
        const float* t = target + b * n;
        for (int i = lane; i < n; i += 32) {
            const float yi = y[i];
            float acc = 0.f;
            for (int j = 0; j < n; j++) {
                const float yj = y[j];
                float g = ((yj - t[j]) / (yj * (1.f - yj))) / total;
                float J = i == j ? yi * (1.f - yi) : -yi * yj;
                if (round_f16) {
                    g = __half2float(__float2half_rn(g));
                    J = __half2float(__float2half_rn(J));
                }
                acc += J * g;
            }
            dx[b * n + i] = acc;
        }
    }
}

// ---- max pooling (MaxPoolingKernel / MaxPoolingBackwardKernel, src/OperationKernels.cu:1507-1573) ---
// Forward keeps the reference's conventions: the first maximum in row-major window order wins (strict
// >), its index i*pool+j within the window is stored as a float in `position`, an empty window gives 0.
__global__ void __launch_bounds__(256) maxpool_kernel(float* __restrict__ out, float* __restrict__ position,
                                                      const float* __restrict__ in, int pool, int stride, int pad,
                                                      int64_t bc, int H, int W, int Ho, int Wo) {
    const int64_t total = bc * Ho * Wo;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t plane = idx / (static_cast<int64_t>(Ho) * Wo);
        const int rem = static_cast<int>(idx - plane * Ho * Wo);
        const int h = rem / Wo, w = rem - h * Wo;
        const float* p = in + plane * H * W;
        float best = -1e20f;
        int best_i = 0;
        for (int i = 0; i < pool; i++) {
            const int hi = h * stride - pad + i;
            if (hi < 0 || hi >= H) continue;
            for (int j = 0; j < pool; j++) {
                const int wi = w * stride - pad + j;
                if (wi < 0 || wi >= W) continue;
                const float v = __ldg(p + static_cast<int64_t>(hi) * W + wi);
                if (v > best) {
                    best = v;
                    best_i = i * pool + j;
                }
            }
        }
        out[idx] = best == -1e20f ? 0.f : best;
        position[idx] = static_cast<float>(best_i);
    }
}
// Backward in gather form: every input element adds the upstream gradients of the windows whose
// recorded maximum it is (the reference scatters with atomicAdd; same sums, fixed order). ADDS to gin.
__global__ void __launch_bounds__(256) maxpool_backward_kernel(float* __restrict__ gin, const float* __restrict__ position,
                                                               const float* __restrict__ gout, int pool, int stride,
                                                               int pad, int64_t bc, int H, int W, int Ho, int Wo) {
    const int64_t total = bc * H * W;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t plane = idx / (static_cast<int64_t>(H) * W);
        const int rem = static_cast<int>(idx - plane * H * W);
        const int hi = rem / W, wi = rem - hi * W;
        // windows (h, w) that contain (hi, wi): h*stride - pad <= hi < h*stride - pad + pool
        const int h_lo = max(0, (hi + pad - pool + stride) / stride), h_hi = min(Ho - 1, (hi + pad) / stride);
        const int w_lo = max(0, (wi + pad - pool + stride) / stride), w_hi = min(Wo - 1, (wi + pad) / stride);
        float acc = 0.f;
        for (int h = h_lo; h <= h_hi; h++)
            for (int w = w_lo; w <= w_hi; w++) {
                const int i = hi - (h * stride - pad), j = wi - (w * stride - pad);
                if (i < 0 || i >= pool || j < 0 || j >= pool) continue;
                const int64_t o = plane * Ho * Wo + static_cast<int64_t>(h) * Wo + w;
                if (static_cast<int>(__ldg(position + o)) == i * pool + j) acc += __ldg(gout + o);
            }
        if (acc != 0.f) gin[idx] += acc;
    }
}

}  // namespace nzb

using namespace nzb;

extern "C" {

int nzb_adam_multi(const nzb_adam_tensor* tensors, int count, float lr, float beta1, float beta2, float eps,
                   void* stream) {
    if (count < 0 || (count > 0 && !tensors)) return fail(NZB_ERR_BAD_ARG, "null tensor list");
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    for (int base = 0; base < count; base += kAdamMaxTensors) {
        AdamList L{};
        L.lr = lr; L.beta1 = beta1; L.beta2 = beta2; L.eps = eps;
        int64_t chunks = 0;
        for (int i = base; i < count && L.count < kAdamMaxTensors; i++) {
            const nzb_adam_tensor& t = tensors[i];
            if (t.n < 0 || (t.n > 0 && (!t.data || !t.m || !t.v || !t.grad))) return fail(NZB_ERR_BAD_ARG, "tensor %d: null pointer or negative size", i);
            if (t.t < 1) return fail(NZB_ERR_BAD_ARG, "tensor %d: t must be >= 1", i);
            if (t.n == 0) continue;
            AdamEntry& e = L.e[L.count++];
            e.data = t.data; e.m = t.m; e.v = t.v; e.grad = t.grad;
            e.shadow = reinterpret_cast<__half*>(t.shadow_f16);
            e.n = t.n;
            e.first_chunk = chunks;
            e.c1 = 1.f - powf(beta1, (float)t.t);
            e.c2 = 1.f - powf(beta2, (float)t.t);
            chunks += (t.n + kAdamChunk - 1) / kAdamChunk;
        }
        if (L.count == 0) continue;
        L.total_chunks = chunks;
        const int64_t cap = (int64_t)ds->sm_count * 8;
        adam_multi_kernel<<<(unsigned)(chunks < cap ? chunks : cap), 256, 0, s>>>(L);
        NZB_CUDA_TRY(cudaGetLastError());
    }
    return NZB_OK;
}

int nzb_softmax_bce_forward(float* probs, float* loss, const float* logits, const float* target, int64_t batches,
                            int64_t n, void* stream) {
    if (!probs || !loss || !logits || !target) return fail(NZB_ERR_BAD_ARG, "null pointer");
    if (batches < 0 || n < 1 || n > 1024) return fail(NZB_ERR_UNSUPPORTED, "n must be in [1, 1024]");
    if (batches == 0) return NZB_OK;
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    int64_t blocks = (batches + 3) / 4;
    if (blocks > (int64_t)ds->sm_count * 8) blocks = (int64_t)ds->sm_count * 8;
    softmax_bce_forward_kernel<<<(unsigned)blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        probs, loss, logits, target, batches, (int)n, (float)(batches * n));
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}

int nzb_softmax_bce_backward(float* dlogits, const float* probs, const float* target, int64_t batches, int64_t n,
                             int round_f16, void* stream) {
    if (!dlogits || !probs || !target) return fail(NZB_ERR_BAD_ARG, "null pointer");
    if (batches < 0 || n < 1 || n > 1024) return fail(NZB_ERR_UNSUPPORTED, "n must be in [1, 1024]");
    if (batches == 0) return NZB_OK;
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    int64_t blocks = (batches + 3) / 4;
    if (blocks > (int64_t)ds->sm_count * 8) blocks = (int64_t)ds->sm_count * 8;
    softmax_bce_backward_kernel<<<(unsigned)blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        dlogits, probs, target, batches, (int)n, (float)(batches * n), round_f16);
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}

static int pool_args_ok(int64_t pool, int64_t stride, int64_t pad, int64_t batches, int64_t channels, int64_t H,
                        int64_t W, int64_t Ho, int64_t Wo) {
    if (pool < 1 || stride < 1 || pad < 0 || batches < 0 || channels < 0 || H < 1 || W < 1 || Ho < 1 || Wo < 1)
        return fail(NZB_ERR_BAD_ARG, "bad pooling extent");
    if (H > INT32_MAX / 2 || W > INT32_MAX / 2 || pool > 4096) return fail(NZB_ERR_UNSUPPORTED, "pooling extent too large");
    return NZB_OK;
}

int nzb_maxpool(float* out, float* position, const float* in, int64_t pool, int64_t stride, int64_t pad, int64_t batches,
                int64_t channels, int64_t H_in, int64_t W_in, int64_t H_out, int64_t W_out, void* stream) {
    if (!out || !position || !in) return fail(NZB_ERR_BAD_ARG, "null pointer");
    int rc = pool_args_ok(pool, stride, pad, batches, channels, H_in, W_in, H_out, W_out);
    if (rc != NZB_OK) return rc;
    DeviceState* ds;
    rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    const int64_t total = batches * channels * H_out * W_out;
    if (total == 0) return NZB_OK;
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)ds->sm_count * 16) blocks = (int64_t)ds->sm_count * 16;
    maxpool_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        out, position, in, (int)pool, (int)stride, (int)pad, batches * channels, (int)H_in, (int)W_in, (int)H_out, (int)W_out);
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}

int nzb_maxpool_backward(float* gin, const float* position, const float* gout, int64_t pool, int64_t stride, int64_t pad,
                         int64_t batches, int64_t channels, int64_t H_in, int64_t W_in, int64_t H_out, int64_t W_out,
                         void* stream) {
    if (!gin || !position || !gout) return fail(NZB_ERR_BAD_ARG, "null pointer");
    int rc = pool_args_ok(pool, stride, pad, batches, channels, H_in, W_in, H_out, W_out);
    if (rc != NZB_OK) return rc;
    DeviceState* ds;
    rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    const int64_t total = batches * channels * H_in * W_in;
    if (total == 0) return NZB_OK;
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)ds->sm_count * 16) blocks = (int64_t)ds->sm_count * 16;
    maxpool_backward_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        gin, position, gout, (int)pool, (int)stride, (int)pad, batches * channels, (int)H_in, (int)W_in, (int)H_out,
        (int)W_out);
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}

}  // extern "C"
