// HBM-bound node operations around the contraction path: im2col / col2img and their
// backwards, broadcast add and its gradient, ReLU, average pooling, softmax, binary
// cross-entropy, Adam, fill / expand. Each replaces the NeuZephyr kernel named beside it
// (paths relative to the NeuZephyr tree). Gradient kernels keep the reference's
// overwrite / accumulate contract; scatter-with-atomicAdd kernels are rewritten in gather
// form, so results do not depend on thread scheduling. 64-bit indexing throughout.
#include <cuda_fp16.h>

#include "nzb_internal.h"

namespace nzb {

static inline unsigned grid_for(int64_t n, int block, int sm_count, int per_sm = 16) {
    int64_t b = (n + block - 1) / block;
    const int64_t cap = (int64_t)sm_count * per_sm;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (unsigned)b;
}

#define NZB_GRID_STRIDE(i, n) \
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < (n); i += (int64_t)gridDim.x * blockDim.x)

// ---- im2col (img2colKernel, src/OperationKernels.cu:1308-1328) ----------------------------
// out[b][p][c*Kh*Kw + kh*Kw + kw] = in[b][c][ho*s - pad + kh][wo*s - pad + kw] or 0, p = ho*Wo + wo
__global__ void __launch_bounds__(256) img2col_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                      int64_t Ho, int64_t Wo, int64_t C, int64_t Kh, int64_t Kw,
                                                      int64_t stride, int64_t pad, int64_t H, int64_t W,
                                                      int64_t total) {
    const int64_t KK = C * Kh * Kw, KHW = Kh * Kw;
    NZB_GRID_STRIDE(idx, total) {
        const int64_t m = idx % KK;
        const int64_t bp = idx / KK;
        const int64_t p = bp % (Ho * Wo);
        const int64_t b = bp / (Ho * Wo);
        const int64_t c = m / KHW, r = m % KHW;
        const int64_t h = (p / Wo) * stride - pad + r / Kw;
        const int64_t w = (p % Wo) * stride - pad + r % Kw;
        out[idx] = (h >= 0 && h < H && w >= 0 && w < W) ? __ldg(in + ((b * C + c) * H + h) * W + w) : 0.f;
    }
}

// img2colBackwardKernel (:1337-1355) in gather form: every dX element sums the column
// entries that were copied from it, then ADDS the sum to dX (the reference atomically
// accumulates into a gradient buffer).
__global__ void __launch_bounds__(256) img2col_backward_kernel(float* __restrict__ dx, const float* __restrict__ dcol,
                                                               int64_t Ho, int64_t Wo, int64_t C, int64_t Kh,
                                                               int64_t Kw, int64_t stride, int64_t pad, int64_t H,
                                                               int64_t W, int64_t total) {
    const int64_t KK = C * Kh * Kw;
    NZB_GRID_STRIDE(idx, total) {
        const int64_t w = idx % W;
        const int64_t h = (idx / W) % H;
        const int64_t c = (idx / (W * H)) % C;
        const int64_t b = idx / (W * H * C);
        float s = 0.f;
        for (int64_t kh = 0; kh < Kh; kh++) {
            const int64_t hn = h + pad - kh;
            if (hn < 0 || hn % stride) continue;
            const int64_t ho = hn / stride;
            if (ho >= Ho) continue;
            for (int64_t kw = 0; kw < Kw; kw++) {
                const int64_t wn = w + pad - kw;
                if (wn < 0 || wn % stride) continue;
                const int64_t wo = wn / stride;
                if (wo >= Wo) continue;
                s += __ldg(dcol + ((b * Ho * Wo) + ho * Wo + wo) * KK + c * Kh * Kw + kh * Kw + kw);
            }
        }
        dx[idx] += s;
    }
}

// ---- col2img / col2imgBackward (:1364-1396): batched [P][C] <-> [C][P] transposes ----------
// dir 0: out[b][c][p] = in[b][p][c]; dir 1: out[b][p][c] = in[b][c][p]. Both OVERWRITE.
__global__ void __launch_bounds__(256) batched_transpose_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                                int64_t R, int64_t Cc, int64_t batches) {
    // in: [batches][R][Cc] -> out: [batches][Cc][R]
    __shared__ float tile[32][33];
    const int64_t tr = (R + 31) >> 5, tc = (Cc + 31) >> 5;
    const int64_t total = batches * tr * tc;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
        const int64_t b = t / (tr * tc);
        const int64_t rem = t % (tr * tc);
        const int64_t r0 = (rem / tc) << 5, c0 = (rem % tc) << 5;
        const float* src = in + b * R * Cc;
        float* dst = out + b * R * Cc;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int64_t r = r0 + ty + i * 8, c = c0 + tx;
            tile[ty + i * 8][tx] = (r < R && c < Cc) ? __ldg(src + r * Cc + c) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int64_t c = c0 + ty + i * 8, r = r0 + tx;
            if (c < Cc && r < R) dst[c * R + r] = tile[tx][ty + i * 8];
        }
        __syncthreads();
    }
}

// ---- broadcast add (MatrixAddKernel :12-37 via tensorMatrixAdd) and its gradient ----------
__global__ void __launch_bounds__(256) add_broadcast_kernel(float* __restrict__ out, const float* __restrict__ a,
                                                            const float* __restrict__ b, int64_t HW, int64_t oC,
                                                            int64_t aN, int64_t aC, int64_t bN, int64_t bC,
                                                            int64_t total) {
    NZB_GRID_STRIDE(idx, total) {
        const int64_t t = idx % HW;
        const int64_t ij = idx / HW;
        const int64_t i = ij / oC, j = ij % oC;
        const int64_t ia = (aN > 1 ? i * aC : 0) + (aC > 1 ? j : 0);
        const int64_t ib = (bN > 1 ? i * bC : 0) + (bC > 1 ? j : 0);
        out[idx] = __ldg(a + ia * HW + t) + __ldg(b + ib * HW + t);
    }
}

// gin[(i',j')][t] += sum over the output batches that map onto (i',j') of gout (gradCopy,
// :1230-1254, whose per-slice "+=" launches race in the reference; this is the defined sum).
__global__ void __launch_bounds__(256) add_backward_reduce_kernel(float* __restrict__ gin,
                                                                  const float* __restrict__ gout, int64_t HW,
                                                                  int64_t oN, int64_t oC, int64_t iN, int64_t iC,
                                                                  int64_t total) {
    NZB_GRID_STRIDE(idx, total) {
        const int64_t t = idx % HW;
        const int64_t ij = idx / HW;
        const int64_t i = ij / iC, j = ij % iC;
        float s = 0.f;
        const int64_t n0 = iN > 1 ? i : 0, n1 = iN > 1 ? i + 1 : oN;
        const int64_t c0 = iC > 1 ? j : 0, c1 = iC > 1 ? j + 1 : oC;
        for (int64_t n = n0; n < n1; n++)
            for (int64_t c = c0; c < c1; c++) s += __ldg(gout + (n * oC + c) * HW + t);
        gin[idx] += s;
    }
}

// ---- ReLU (:230-248) ---------------------------------------------------------------------
__global__ void __launch_bounds__(256) relu_kernel(float* __restrict__ out, const float* __restrict__ in, int64_t n) {
    NZB_GRID_STRIDE(i, n) out[i] = fmaxf(in[i], 0.f);
}
__global__ void __launch_bounds__(256) relu_backward_kernel(float* __restrict__ gin, const float* __restrict__ x,
                                                            const float* __restrict__ gout, int64_t n) {
    NZB_GRID_STRIDE(i, n) gin[i] = x[i] > 0.f ? gout[i] : 0.f;
}

// ---- average pooling (:1404-1482) -------------------------------------------------------------
__global__ void __launch_bounds__(256) avgpool_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                      int64_t pool, int64_t stride, int64_t pad, int64_t H, int64_t W,
                                                      int64_t Ho, int64_t Wo, int64_t total) {
    NZB_GRID_STRIDE(idx, total) {
        const int64_t w = idx % Wo, h = (idx / Wo) % Ho, bc = idx / (Wo * Ho);
        const float* src = in + bc * H * W;
        float s = 0.f;
        int cnt = 0;
        for (int64_t i = 0; i < pool; i++) {
            const int64_t hi = h * stride - pad + i;
            if (hi < 0 || hi >= H) continue;
            for (int64_t j = 0; j < pool; j++) {
                const int64_t wi = w * stride - pad + j;
                if (wi < 0 || wi >= W) continue;
                s += __ldg(src + hi * W + wi);
                cnt++;
            }
        }
        out[idx] = cnt > 0 ? s / (float)cnt : 0.f;
    }
}

// Gather form of AveragePoolingBackwardKernel: gin[bc][hi][wi] += sum over windows that
// contain (hi,wi) of gout / divisor; the divisor is pool*pool without padding and the
// in-bounds tap count with padding, as in the reference (:1457, :1477).
__global__ void __launch_bounds__(256) avgpool_backward_kernel(float* __restrict__ gin, const float* __restrict__ gout,
                                                               int64_t pool, int64_t stride, int64_t pad, int64_t H,
                                                               int64_t W, int64_t Ho, int64_t Wo, int64_t total) {
    NZB_GRID_STRIDE(idx, total) {
        const int64_t wi = idx % W, hi = (idx / W) % H, bc = idx / (W * H);
        const float* g = gout + bc * Ho * Wo;
        // windows h with h*stride - pad <= hi <= h*stride - pad + pool - 1
        int64_t h_lo = (hi + pad - pool + 1 + stride - 1);
        h_lo = h_lo <= 0 ? 0 : h_lo / stride;
        int64_t h_hi = (hi + pad) / stride;
        if (h_hi > Ho - 1) h_hi = Ho - 1;
        int64_t w_lo = (wi + pad - pool + 1 + stride - 1);
        w_lo = w_lo <= 0 ? 0 : w_lo / stride;
        int64_t w_hi = (wi + pad) / stride;
        if (w_hi > Wo - 1) w_hi = Wo - 1;
        float s = 0.f;
        for (int64_t h = h_lo; h <= h_hi; h++) {
            const int64_t hs = h * stride - pad;
            const int64_t ch = min(hs + pool, H) - max(hs, (int64_t)0);
            for (int64_t w = w_lo; w <= w_hi; w++) {
                const int64_t ws = w * stride - pad;
                const int64_t cw = min(ws + pool, W) - max(ws, (int64_t)0);
                const float div = pad ? (float)(ch * cw) : (float)(pool * pool);
                s += __ldg(g + h * Wo + w) / div;
            }
        }
        gin[idx] += s;
    }
}


// Stride 2, no padding, every window inside the image, rows 16-byte aligned (W % 4 == 0): a thread
// produces FOUR consecutive outputs of one row. Their windows span 2*4 + POOL - 2 input columns, read
// as float4 (three per input row for POOL = 5), summed down the rows first and then across each
// window: 15 vector loads for four outputs instead of 100 scalar ones.
template <int POOL>
__global__ void __launch_bounds__(256) avgpool_s2_quad_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                              int H, int W, int Ho, int Wo, int planes) {
    constexpr int NV = (8 + POOL - 2 + 3) / 4;  // float4 per input row
    const int groups = (Wo + 3) >> 2, per = Ho * groups;
    constexpr float inv = 1.f / (float)(POOL * POOL);
    for (int bc = blockIdx.y; bc < planes; bc += gridDim.y) {
        const float* src = in + (int64_t)bc * H * W;
        float* dst = out + (int64_t)bc * Ho * Wo;
        for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < per; idx += gridDim.x * blockDim.x) {
            const int h = idx / groups, w0 = (idx - h * groups) * 4;
            const float* base = src + (int64_t)(2 * h) * W + 2 * w0;
            float col[NV * 4];
#pragma unroll
            for (int c = 0; c < NV * 4; c++) col[c] = 0.f;
#pragma unroll
            for (int i = 0; i < POOL; i++) {
#pragma unroll
                for (int v = 0; v < NV; v++) {
                    if (2 * w0 + 4 * v < W) {  // the last group of a row may not need (or have) the last vector
                        const float4 x = __ldg(reinterpret_cast<const float4*>(base + (int64_t)i * W) + v);
                        col[4 * v] += x.x; col[4 * v + 1] += x.y; col[4 * v + 2] += x.z; col[4 * v + 3] += x.w;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (w0 + j < Wo) {
                    float s = 0.f;
#pragma unroll
                    for (int c = 0; c < POOL; c++) s += col[2 * j + c];
                    dst[(int64_t)h * Wo + w0 + j] = s * inv;
                }
            }
        }
    }
}

// 32-bit-index forms of the two pooling kernels for planes below 2^31 elements: blockIdx.y
// walks the (batch, channel) planes, so a thread only splits a plane offset into (h, w).
__global__ void __launch_bounds__(256) avgpool_plane_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                            int pool, int stride, int pad, int H, int W, int Ho,
                                                            int Wo, int planes) {
    const int per = Ho * Wo;
    for (int bc = blockIdx.y; bc < planes; bc += gridDim.y) {
        const float* src = in + (int64_t)bc * H * W;
        float* dst = out + (int64_t)bc * per;
        for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < per; idx += gridDim.x * blockDim.x) {
            const int h = idx / Wo, w = idx - h * Wo;
            const int h0 = h * stride - pad, w0 = w * stride - pad;
            const int i0 = max(h0, 0), i1 = min(h0 + pool, H), j0 = max(w0, 0), j1 = min(w0 + pool, W);
            float s = 0.f;
            for (int i = i0; i < i1; i++) {
                const float* row = src + (int64_t)i * W;
                for (int j = j0; j < j1; j++) s += __ldg(row + j);
            }
            const int cnt = (i1 - i0) * (j1 - j0);
            dst[idx] = cnt > 0 ? s / (float)cnt : 0.f;
        }
    }
}

// Compile-time window forms of both pooling kernels (no padding): all loops have fixed trip
// counts and unroll, and a window that lies inside the image needs no bounds test. The generic
// kernels below take any other (pool, stride, pad).
template <int POOL, int STRIDE>
__global__ void __launch_bounds__(256) avgpool_fixed_kernel(float* __restrict__ out, const float* __restrict__ in, int H,
                                                            int W, int Ho, int Wo, int planes) {
    const int per = Ho * Wo;
    for (int bc = blockIdx.y; bc < planes; bc += gridDim.y) {
        const float* src = in + (int64_t)bc * H * W;
        float* dst = out + (int64_t)bc * per;
        for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < per; idx += gridDim.x * blockDim.x) {
            const int h = idx / Wo, w = idx - h * Wo;
            const int h0 = h * STRIDE, w0 = w * STRIDE;
            const float* base = src + (int64_t)h0 * W + w0;
            float s = 0.f;
            if (h0 + POOL <= H && w0 + POOL <= W) {
#pragma unroll
                for (int i = 0; i < POOL; i++)
#pragma unroll
                    for (int j = 0; j < POOL; j++) s += __ldg(base + i * W + j);
                dst[idx] = s / (float)(POOL * POOL);
            } else {
                int cnt = 0;
#pragma unroll
                for (int i = 0; i < POOL; i++)
#pragma unroll
                    for (int j = 0; j < POOL; j++)
                        if (h0 + i < H && w0 + j < W) {
                            s += __ldg(base + i * W + j);
                            cnt++;
                        }
                dst[idx] = cnt > 0 ? s / (float)cnt : 0.f;
            }
        }
    }
}

// Stride 2, no padding, W % 4 == 0: a thread owns two input rows x four columns. The windows that
// cover that tile form a small rectangle of the output gradient (3 x 4 values for pool 5), loaded
// once with one bounds predicate per row and per column; the eight sums are separable (first down
// the rows each input row belongs to, then along the columns each input column belongs to), and the
// division by pool^2 is a multiplication by its reciprocal. The kernel is bound by instruction issue,
// not by memory (77 % issue slots busy before these three changes, 37 instructions per output), so the
// instruction count is what matters. (The reference adds gout / pool^2 term by term with atomics in no
// fixed order; both are within an ulp or two of the exact sum.)
template <int POOL>
__global__ void __launch_bounds__(256) avgpool_backward_s2_kernel(float* __restrict__ gin,
                                                                  const float* __restrict__ gout, int H, int W, int Ho,
                                                                  int Wo, int planes, int overwrite) {
    constexpr int NH = (POOL - 1) / 2 + 1;      // windows covering rows 2a, 2a+1
    constexpr int NW = (POOL - 1 + 3) / 2 + 1;  // windows covering columns 4b .. 4b+3
    constexpr int base = (2 - POOL) >> 1;       // floor((2 - POOL) / 2)
    const int W4 = W >> 2, H2 = (H + 1) >> 1, per = H2 * W4;
    constexpr float inv = 1.0f / (float)(POOL * POOL);
    for (int bc = blockIdx.y; bc < planes; bc += gridDim.y) {
        const float* g = gout + (int64_t)bc * Ho * Wo;
        float* dst = gin + (int64_t)bc * H * W;
        for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < per; idx += gridDim.x * blockDim.x) {
            const int a = idx / W4, wi0 = (idx - a * W4) * 4, hi0 = 2 * a;
            // candidate windows: rows hb .. hb+NH-1, columns wb .. wb+NW-1 (may reach outside: masked)
            const int hb = (hi0 - POOL + 2) >> 1;  // ceil((hi0 - POOL + 1) / 2), also right when negative
            const int wb = (wi0 - POOL + 2) >> 1;
            bool wok[NW];
#pragma unroll
            for (int dw = 0; dw < NW; dw++) wok[dw] = (unsigned)(wb + dw) < (unsigned)Wo;
            float v[NH][NW];
#pragma unroll
            for (int dh = 0; dh < NH; dh++) {
                const bool hok = (unsigned)(hb + dh) < (unsigned)Ho;
                const float* grow = g + (hb + dh) * Wo + wb;  // 32-bit offset inside one plane
#pragma unroll
                for (int dw = 0; dw < NW; dw++) v[dh][dw] = (hok && wok[dw]) ? __ldg(grow + dw) : 0.f;
            }
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int hi = hi0 + r;
                if (hi >= H) break;
                // Windows of row hi0 + r and of column wi0 + j, as offsets from hb / wb: with hi0 even and
                // wi0 a multiple of 4 they depend on r and j only, so after unrolling they are constants
                // (windows outside the gradient were loaded as zeros above).
                const int h_lo = ((r - POOL + 2) >> 1) - base, h_hi = (r >> 1) - base;
                float col[NW];
#pragma unroll
                for (int dw = 0; dw < NW; dw++) {
                    col[dw] = 0.f;
#pragma unroll
                    for (int dh = 0; dh < NH; dh++)
                        if (dh >= h_lo && dh <= h_hi) col[dw] += v[dh][dw];
                }
                float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int w_lo = ((j - POOL + 2) >> 1) - base, w_hi = (j >> 1) - base;
#pragma unroll
                    for (int dw = 0; dw < NW; dw++)
                        if (dw >= w_lo && dw <= w_hi) s[j] += col[dw];
                }
                float4* d4 = reinterpret_cast<float4*>(dst + hi * W + wi0);
                // every input element is visited exactly once: overwriting needs no cleared buffer
                float4 o = overwrite ? make_float4(0.f, 0.f, 0.f, 0.f) : *d4;
                o.x += s[0] * inv; o.y += s[1] * inv; o.z += s[2] * inv; o.w += s[3] * inv;
                *d4 = o;
            }
        }
    }
}

// Four consecutive input columns per thread (W % 4 == 0): the windows that cover them overlap, so
// each gradient value is loaded once for the four, and the update of the input gradient is one
// 16-byte read-modify-write. The terms are summed before the single division by pool^2 (the
// reference adds gout / pool^2 term by term with atomics, in no fixed order; both are within an
// ulp or two of the exact sum).
template <int POOL, int STRIDE>
__global__ void __launch_bounds__(256) avgpool_backward_fixed_kernel(float* __restrict__ gin,
                                                                     const float* __restrict__ gout, int H, int W,
                                                                     int Ho, int Wo, int planes) {
    constexpr int NH = (POOL + STRIDE - 1) / STRIDE;          // windows that can cover one row
    constexpr int NW = (POOL + 3 + STRIDE - 1) / STRIDE + 1;  // windows that can cover four columns
    const int W4 = W >> 2, per = H * W4;
    for (int bc = blockIdx.y; bc < planes; bc += gridDim.y) {
        const float* g = gout + (int64_t)bc * Ho * Wo;
        float* dst = gin + (int64_t)bc * H * W;
        for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < per; idx += gridDim.x * blockDim.x) {
            const int hi = idx / W4, wi0 = (idx - hi * W4) * 4;
            const int hn = hi - POOL + STRIDE;
            const int h_lo = hn <= 0 ? 0 : hn / STRIDE, h_hi = min(hi / STRIDE, Ho - 1);
            const int wn0 = wi0 - POOL + STRIDE;
            const int wbase = wn0 <= 0 ? 0 : wn0 / STRIDE;  // first window of column wi0
            // which of the NW candidate windows covers which of the four columns
            uint32_t mask = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int wn = wi0 + j - POOL + STRIDE;
                const int lo = wn <= 0 ? 0 : wn / STRIDE, hi_w = min((wi0 + j) / STRIDE, Wo - 1);
#pragma unroll
                for (int d = 0; d < NW; d++)
                    if (wbase + d >= lo && wbase + d <= hi_w) mask |= 1u << (d * 4 + j);
            }
            float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int dh = 0; dh < NH; dh++) {
                const int h = h_lo + dh;
                if (h > h_hi) break;
                const float* grow = g + (int64_t)h * Wo + wbase;
#pragma unroll
                for (int d = 0; d < NW; d++) {
                    const float v = (wbase + d < Wo && ((mask >> (d * 4)) & 15u)) ? __ldg(grow + d) : 0.f;
#pragma unroll
                    for (int j = 0; j < 4; j++) s[j] += ((mask >> (d * 4 + j)) & 1u) ? v : 0.f;
                }
            }
            float4* d4 = reinterpret_cast<float4*>(dst + (int64_t)hi * W + wi0);
            float4 o = *d4;
            constexpr float full = (float)(POOL * POOL);
            o.x += s[0] / full; o.y += s[1] / full; o.z += s[2] / full; o.w += s[3] / full;
            *d4 = o;
        }
    }
}

// Unpadded pooling, four consecutive input columns per thread (W % 4 == 0): the windows that cover
// them overlap, so each gradient value is loaded once for the four, and the update of the input
// gradient is one 16-byte read-modify-write. The terms are summed before the single division by
// pool^2 (the reference adds gout / pool^2 term by term with atomics, in no fixed order; both are
// within an ulp or two of the exact sum).
template <int STRIDE>
__global__ void __launch_bounds__(256) avgpool_backward_quad_kernel(float* __restrict__ gin,
                                                                    const float* __restrict__ gout, int pool,
                                                                    int stride_rt, int H, int W, int Ho, int Wo,
                                                                    int planes) {
    const int stride = STRIDE > 0 ? STRIDE : stride_rt;
    const int W4 = W >> 2, per = H * W4;
    const float full = (float)(pool * pool);
    for (int bc = blockIdx.y; bc < planes; bc += gridDim.y) {
        const float* g = gout + (int64_t)bc * Ho * Wo;
        float* dst = gin + (int64_t)bc * H * W;
        for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < per; idx += gridDim.x * blockDim.x) {
            const int hi = idx / W4, wi0 = (idx - hi * W4) * 4;
            const int hn = hi - pool + stride;
            const int h_lo = hn <= 0 ? 0 : hn / stride, h_hi = min(hi / stride, Ho - 1);
            int w_lo[4], w_hi[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int wn = wi0 + j - pool + stride;
                w_lo[j] = wn <= 0 ? 0 : wn / stride;
                w_hi[j] = min((wi0 + j) / stride, Wo - 1);
            }
            float s[4] = {0.f, 0.f, 0.f, 0.f};
            for (int h = h_lo; h <= h_hi; h++) {
                const float* grow = g + (int64_t)h * Wo;
                for (int w = w_lo[0]; w <= w_hi[3]; w++) {
                    const float v = __ldg(grow + w);
#pragma unroll
                    for (int j = 0; j < 4; j++) s[j] += (w >= w_lo[j] && w <= w_hi[j]) ? v : 0.f;
                }
            }
            float4* d4 = reinterpret_cast<float4*>(dst + (int64_t)hi * W + wi0);
            float4 o = *d4;
            o.x += s[0] / full; o.y += s[1] / full; o.z += s[2] / full; o.w += s[3] / full;
            *d4 = o;
        }
    }
}

// STRIDE > 0 fixes the stride at compile time (shifts instead of divisions); 0 = any stride.
template <int STRIDE>
__global__ void __launch_bounds__(256) avgpool_backward_plane_kernel(float* __restrict__ gin,
                                                                     const float* __restrict__ gout, int pool,
                                                                     int stride_rt, int pad, int H, int W, int Ho,
                                                                     int Wo, int planes) {
    const int stride = STRIDE > 0 ? STRIDE : stride_rt;
    const int per = H * W;
    const float full = (float)(pool * pool);
    for (int bc = blockIdx.y; bc < planes; bc += gridDim.y) {
        const float* g = gout + (int64_t)bc * Ho * Wo;
        float* dst = gin + (int64_t)bc * per;
        for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < per; idx += gridDim.x * blockDim.x) {
            const int hi = idx / W, wi = idx - hi * W;
            // windows h with h*stride - pad <= hi <= h*stride - pad + pool - 1
            const int hn = hi + pad - pool + stride, wn = wi + pad - pool + stride;
            const int h_lo = hn <= 0 ? 0 : hn / stride, w_lo = wn <= 0 ? 0 : wn / stride;
            const int h_hi = min((hi + pad) / stride, Ho - 1), w_hi = min((wi + pad) / stride, Wo - 1);
            float s = 0.f;
            if (pad == 0) {
                // every window is complete: one divisor. The terms are summed before the division
                // (the reference adds gout / pool^2 term by term, atomically and in no fixed order;
                // both are within an ulp or two of the exact sum).
                for (int h = h_lo; h <= h_hi; h++) {
                    const float* grow = g + (int64_t)h * Wo;
                    for (int w = w_lo; w <= w_hi; w++) s += __ldg(grow + w);
                }
                s = s / full;
            } else {
                for (int h = h_lo; h <= h_hi; h++) {
                    const int hs = h * stride - pad;
                    const int ch = min(hs + pool, H) - max(hs, 0);
                    const float* grow = g + (int64_t)h * Wo;
                    for (int w = w_lo; w <= w_hi; w++) {
                        const int ws = w * stride - pad;
                        const int cw = min(ws + pool, W) - max(ws, 0);
                        s += __ldg(grow + w) / (float)(ch * cw);
                    }
                }
            }
            dst[idx] += s;
        }
    }
}

// ---- softmax over each matrix of n elements (:477-523; Tensor::expSum) -----------------------
// One warp per matrix for n <= 1024 * 32; larger n loops. exp(x - max) / sum: the same value
// as the reference's exp(x) / sum(exp(x)) whenever the latter does not overflow.
__global__ void __launch_bounds__(256) softmax_kernel(float* __restrict__ out, const float* __restrict__ in, int64_t n,
                                                      int64_t batches) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t b = warp; b < batches; b += nwarps) {
        const float* x = in + b * n;
        float mx = -INFINITY;
        for (int64_t i = lane; i < n; i += 32) mx = fmaxf(mx, x[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float s = 0.f;
        for (int64_t i = lane; i < n; i += 32) s += expf(x[i] - mx);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        for (int64_t i = lane; i < n; i += 32) out[b * n + i] = expf(x[i] - mx) / s;
    }
}

// SoftmaxNode::backward (src/Nodes.cu:538-548): dX = J(y) dY with J = diag(y) - y y^T.
// The reference forms J (SoftmaxJacobianKernel :536-553) and multiplies with its fp16
// tensor-core GEMM; round_f16 != 0 reproduces that operand rounding (J and dY to fp16)
// with fp32 accumulation. round_f16 == 0 is the exact fp32 form y*(dY - <dY,y>).
// OVERWRITES gin. One warp per matrix.
__global__ void __launch_bounds__(256) softmax_backward_kernel(float* __restrict__ gin, const float* __restrict__ y,
                                                               const float* __restrict__ gout, int64_t n,
                                                               int64_t batches, int round_f16) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t b = warp; b < batches; b += nwarps) {
        const float* yy = y + b * n;
        const float* g = gout + b * n;
        if (!round_f16) {
            float dot = 0.f;
            for (int64_t i = lane; i < n; i += 32) dot += yy[i] * g[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            for (int64_t i = lane; i < n; i += 32) gin[b * n + i] = yy[i] * (g[i] - dot);
        } else {
            for (int64_t i = lane; i < n; i += 32) {
                const float yi = yy[i];
                float s = 0.f;
                for (int64_t j = 0; j < n; j++) {
                    const float yj = yy[j];
                    const float Jij = (i == j) ? yi * (1.f - yi) : -yi * yj;
                    s += __half2float(__float2half_rn(Jij)) * __half2float(__float2half_rn(g[j]));
                }
                gin[b * n + i] = s;
            }
        }
    }
}

// ---- binary cross-entropy (:648-699): mean over all n elements ----------------------------------
// loss_out[0] += sum_i (-t log p - (1-t) log(1-p)) / n  (the caller zeroes loss_out when it wants
// the value of this call alone; the reference's loss node also accumulates, src/Nodes.cu:822-840).
__global__ void __launch_bounds__(256) bce_kernel(float* __restrict__ loss_out, const float* __restrict__ p,
                                                  const float* __restrict__ t, int64_t n) {
    __shared__ float part[8];
    float s = 0.f;
    NZB_GRID_STRIDE(i, n) s += (-t[i] * logf(p[i]) - (1.f - t[i]) * logf(1.f - p[i])) / (float)n;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        s = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (threadIdx.x == 0) atomicAdd(loss_out, s);
    }
}
__global__ void __launch_bounds__(256) bce_backward_kernel(float* __restrict__ out, const float* __restrict__ p,
                                                           const float* __restrict__ t, int64_t n) {
    NZB_GRID_STRIDE(i, n) out[i] = ((p[i] - t[i]) / (p[i] * (1.f - p[i]))) / (float)n;
}

// ---- Adam (AdamKernel :753-766) ---------------------------------------------------------------
__global__ void __launch_bounds__(256) adam_kernel(float* __restrict__ data, float* __restrict__ m,
                                                   float* __restrict__ v, const float* __restrict__ grad, float lr,
                                                   float beta1, float beta2, float eps, float c1, float c2, int64_t n) {
    NZB_GRID_STRIDE(i, n) {
        float mt = m[i], vt = v[i];
        data[i] = adam_update(data[i], mt, vt, grad[i], lr, beta1, beta2, eps, c1, c2);
        m[i] = mt;
        v[i] = vt;
    }
}

// ---- fill / expand / scale (FillKernel :1146-1151, ExpandKernel :1282-1290) --------------------
__global__ void __launch_bounds__(256) fill_kernel(float* __restrict__ data, float value, int64_t n) {
    NZB_GRID_STRIDE(i, n) data[i] = value;
}
__global__ void __launch_bounds__(256) expand_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                     int64_t per_batch, int64_t total) {
    NZB_GRID_STRIDE(i, total) out[i] = __ldg(in + i % per_batch);
}
__global__ void __launch_bounds__(256) scale_kernel(float* __restrict__ data, float s, int64_t n) {
    NZB_GRID_STRIDE(i, n) data[i] *= s;
}

}  // namespace nzb

using namespace nzb;

#define NZB_OPS_PROLOGUE()                    \
    DeviceState* ds;                          \
    {                                         \
        int rc_ = get_device_state(&ds);      \
        if (rc_ != NZB_OK) return rc_;        \
    }                                         \
    cudaStream_t s = static_cast<cudaStream_t>(stream)

#define NZB_OPS_EPILOGUE()                \
    NZB_CUDA_TRY(cudaGetLastError());     \
    return NZB_OK

extern "C" {

int nzb_img2col(float* out, const float* in, int64_t H_out, int64_t W_out, int64_t C, int64_t K_h, int64_t K_w,
                int64_t stride, int64_t pad, int64_t H_in, int64_t W_in, int64_t batch, void* stream) {
    if (!out || !in) return fail(NZB_ERR_BAD_ARG, "null pointer");
    if (stride < 1 || H_out < 0 || W_out < 0 || C < 0 || batch < 0) return fail(NZB_ERR_BAD_ARG, "bad extent");
    NZB_OPS_PROLOGUE();
    const int64_t total = batch * H_out * W_out * C * K_h * K_w;
    if (total == 0) return NZB_OK;
    img2col_kernel<<<grid_for(total, 256, ds->sm_count), 256, 0, s>>>(out, in, H_out, W_out, C, K_h, K_w, stride, pad,
                                                                      H_in, W_in, total);
    NZB_OPS_EPILOGUE();
}

int nzb_img2col_backward(float* dx, const float* dcol, int64_t H_out, int64_t W_out, int64_t C, int64_t K_h,
                         int64_t K_w, int64_t stride, int64_t pad, int64_t H_in, int64_t W_in, int64_t batch,
                         void* stream) {
    if (!dx || !dcol) return fail(NZB_ERR_BAD_ARG, "null pointer");
    if (stride < 1) return fail(NZB_ERR_BAD_ARG, "bad stride");
    NZB_OPS_PROLOGUE();
    const int64_t total = batch * C * H_in * W_in;
    if (total == 0) return NZB_OK;
    img2col_backward_kernel<<<grid_for(total, 256, ds->sm_count), 256, 0, s>>>(dx, dcol, H_out, W_out, C, K_h, K_w,
                                                                               stride, pad, H_in, W_in, total);
    NZB_OPS_EPILOGUE();
}

int nzb_col2img(float* out, const float* in, int64_t H_out, int64_t W_out, int64_t C_out, int64_t batches,
                void* stream) {
    if (!out || !in) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    const int64_t R = H_out * W_out;
    if (R * C_out * batches == 0) return NZB_OK;
    const int64_t tiles = batches * ((R + 31) / 32) * ((C_out + 31) / 32);
    batched_transpose_kernel<<<grid_for(tiles, 1, ds->sm_count, 32), 256, 0, s>>>(out, in, R, C_out, batches);
    NZB_OPS_EPILOGUE();
}

int nzb_col2img_backward(float* out, const float* in, int64_t H_out, int64_t W_out, int64_t C_out, int64_t batches,
                         void* stream) {
    if (!out || !in) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    const int64_t R = H_out * W_out;
    if (R * C_out * batches == 0) return NZB_OK;
    const int64_t tiles = batches * ((R + 31) / 32) * ((C_out + 31) / 32);
    batched_transpose_kernel<<<grid_for(tiles, 1, ds->sm_count, 32), 256, 0, s>>>(out, in, C_out, R, batches);
    NZB_OPS_EPILOGUE();
}

int nzb_add_broadcast(float* out, const float* a, const float* b, const int64_t shapeA[4], const int64_t shapeB[4],
                      void* stream) {
    if (!out || !a || !b || !shapeA || !shapeB) return fail(NZB_ERR_BAD_ARG, "null pointer");
    if (shapeA[2] != shapeB[2] || shapeA[3] != shapeB[3]) return fail(NZB_ERR_BAD_ARG, "matrix extents differ");
    for (int k = 0; k < 2; k++)
        if (shapeA[k] != shapeB[k] && shapeA[k] != 1 && shapeB[k] != 1)
            return fail(NZB_ERR_BAD_ARG, "batch extents are not broadcast compatible");
    NZB_OPS_PROLOGUE();
    const int64_t oN = shapeA[0] > shapeB[0] ? shapeA[0] : shapeB[0];
    const int64_t oC = shapeA[1] > shapeB[1] ? shapeA[1] : shapeB[1];
    const int64_t HW = shapeA[2] * shapeA[3], total = oN * oC * HW;
    if (total == 0) return NZB_OK;
    add_broadcast_kernel<<<grid_for(total, 256, ds->sm_count), 256, 0, s>>>(out, a, b, HW, oC, shapeA[0], shapeA[1],
                                                                            shapeB[0], shapeB[1], total);
    NZB_OPS_EPILOGUE();
}

int nzb_add_backward(float* gin, const float* gout, const int64_t shapeIn[4], const int64_t shapeOut[4],
                     void* stream) {
    if (!gin || !gout || !shapeIn || !shapeOut) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    const int64_t HW = shapeOut[2] * shapeOut[3];
    if (shapeIn[0] == shapeOut[0] && shapeIn[1] == shapeOut[1]) {
        // same shape: the gradient is copied (overwrite), src/Nodes.cu:101-105
        NZB_CUDA_TRY(cudaMemcpyAsync(gin, gout, sizeof(float) * (size_t)(shapeOut[0] * shapeOut[1] * HW),
                                     cudaMemcpyDeviceToDevice, s));
        return NZB_OK;
    }
    const int64_t total = shapeIn[0] * shapeIn[1] * HW;
    if (total == 0) return NZB_OK;
    add_backward_reduce_kernel<<<grid_for(total, 256, ds->sm_count), 256, 0, s>>>(gin, gout, HW, shapeOut[0],
                                                                                  shapeOut[1], shapeIn[0], shapeIn[1],
                                                                                  total);
    NZB_OPS_EPILOGUE();
}

int nzb_relu(float* out, const float* in, int64_t n, void* stream) {
    if (!out || !in) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    if (n <= 0) return NZB_OK;
    relu_kernel<<<grid_for(n, 256, ds->sm_count), 256, 0, s>>>(out, in, n);
    NZB_OPS_EPILOGUE();
}

int nzb_relu_backward(float* gin, const float* x, const float* gout, int64_t n, void* stream) {
    if (!gin || !x || !gout) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    if (n <= 0) return NZB_OK;
    relu_backward_kernel<<<grid_for(n, 256, ds->sm_count), 256, 0, s>>>(gin, x, gout, n);
    NZB_OPS_EPILOGUE();
}

int nzb_avgpool(float* out, const float* in, int64_t pool, int64_t stride, int64_t pad, int64_t batches,
                int64_t channels, int64_t H_in, int64_t W_in, int64_t H_out, int64_t W_out, void* stream) {
    if (!out || !in) return fail(NZB_ERR_BAD_ARG, "null pointer");
    if (pool < 1 || stride < 1) return fail(NZB_ERR_BAD_ARG, "bad window");
    NZB_OPS_PROLOGUE();
    const int64_t total = batches * channels * H_out * W_out;
    if (total == 0) return NZB_OK;
    if (H_in * W_in < INT32_MAX && batches * channels < INT32_MAX && pool < 65536 && stride < 65536 && pad < 65536) {
        const int64_t per = H_out * W_out, planes = batches * channels;
        int64_t gx = (per + 255) / 256;
        const int64_t capx = ((int64_t)ds->sm_count * 16 + planes - 1) / planes;
        if (gx > capx) gx = capx;
        const int64_t gy = planes < 65535 ? planes : 65535;
        const bool s2 = pad == 0 && stride == 2 && (pool == 5 || pool == 3 || pool == 2);
        if (s2 && W_in % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (H_out - 1) * 2 + pool <= H_in &&
            (W_out - 1) * 2 + pool <= W_in) {
            int64_t gq = (H_out * ((W_out + 3) / 4) + 255) / 256;
            if (gq > capx) gq = capx;
            const dim3 gridq((unsigned)gq, (unsigned)gy);
            if (pool == 5)
                avgpool_s2_quad_kernel<5><<<gridq, 256, 0, s>>>(out, in, (int)H_in, (int)W_in, (int)H_out, (int)W_out, (int)planes);
            else if (pool == 3)
                avgpool_s2_quad_kernel<3><<<gridq, 256, 0, s>>>(out, in, (int)H_in, (int)W_in, (int)H_out, (int)W_out, (int)planes);
            else
                avgpool_s2_quad_kernel<2><<<gridq, 256, 0, s>>>(out, in, (int)H_in, (int)W_in, (int)H_out, (int)W_out, (int)planes);
            NZB_OPS_EPILOGUE();
        }
        if (pad == 0 && ((pool == 5 && stride == 2) || (pool == 2 && stride == 2) || (pool == 3 && stride == 2))) {
            const dim3 grid((unsigned)gx, (unsigned)gy);
            if (pool == 5)
                avgpool_fixed_kernel<5, 2><<<grid, 256, 0, s>>>(out, in, (int)H_in, (int)W_in, (int)H_out, (int)W_out, (int)planes);
            else if (pool == 3)
                avgpool_fixed_kernel<3, 2><<<grid, 256, 0, s>>>(out, in, (int)H_in, (int)W_in, (int)H_out, (int)W_out, (int)planes);
            else
                avgpool_fixed_kernel<2, 2><<<grid, 256, 0, s>>>(out, in, (int)H_in, (int)W_in, (int)H_out, (int)W_out, (int)planes);
            NZB_OPS_EPILOGUE();
        }
        avgpool_plane_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, s>>>(out, in, (int)pool, (int)stride, (int)pad,
                                                                             (int)H_in, (int)W_in, (int)H_out,
                                                                             (int)W_out, (int)planes);
        NZB_OPS_EPILOGUE();
    }
    avgpool_kernel<<<grid_for(total, 256, ds->sm_count), 256, 0, s>>>(out, in, pool, stride, pad, H_in, W_in, H_out,
                                                                      W_out, total);
    NZB_OPS_EPILOGUE();
}

int nzb_avgpool_backward(float* gin, const float* gout, int64_t pool, int64_t stride, int64_t pad, int64_t batches,
                         int64_t channels, int64_t H_in, int64_t W_in, int64_t H_out, int64_t W_out, void* stream) {
    return nzb_avgpool_backward_ex(gin, gout, pool, stride, pad, batches, channels, H_in, W_in, H_out, W_out, 0, stream);
}

int nzb_avgpool_backward_ex(float* gin, const float* gout, int64_t pool, int64_t stride, int64_t pad, int64_t batches,
                            int64_t channels, int64_t H_in, int64_t W_in, int64_t H_out, int64_t W_out, int overwrite,
                            void* stream) {
    if (!gin || !gout) return fail(NZB_ERR_BAD_ARG, "null pointer");
    if (pool < 1 || stride < 1) return fail(NZB_ERR_BAD_ARG, "bad window");
    NZB_OPS_PROLOGUE();
    const int64_t total = batches * channels * H_in * W_in;
    if (total == 0) return NZB_OK;
    // overwrite: the stride-2 kernels below write every element themselves; every other form clears gin
    // first and then accumulates as usual
    const bool direct = overwrite && pad == 0 && W_in % 4 == 0 && (reinterpret_cast<uintptr_t>(gin) & 15) == 0 &&
                        stride == 2 && (pool == 5 || pool == 3 || pool == 2) && H_in * W_in < INT32_MAX &&
                        batches * channels < INT32_MAX;
    if (overwrite && !direct) NZB_CUDA_TRY(cudaMemsetAsync(gin, 0, (size_t)total * sizeof(float), s));
    const int ovw = direct ? 1 : 0;
    if (H_in * W_in < INT32_MAX && batches * channels < INT32_MAX && pool < 65536 && stride < 65536 && pad < 65536) {
        const int64_t per = H_in * W_in, planes = batches * channels;
        int64_t gx = (per + 255) / 256;
        const int64_t capx = ((int64_t)ds->sm_count * 16 + planes - 1) / planes;
        if (gx > capx) gx = capx;
        const int64_t gy = planes < 65535 ? planes : 65535;
        const dim3 grid((unsigned)gx, (unsigned)gy);
        if (pad == 0 && W_in % 4 == 0 && (reinterpret_cast<uintptr_t>(gin) & 15) == 0) {
            int64_t gq = (per / 4 + 255) / 256;
            if (gq > capx) gq = capx;
            const dim3 gridq((unsigned)gq, (unsigned)gy);
            if (stride == 2 && (pool == 5 || pool == 3 || pool == 2)) {
                int64_t g2 = (((H_in + 1) / 2) * (W_in / 4) + 255) / 256;
                if (g2 > capx) g2 = capx;
                const dim3 grid2((unsigned)g2, (unsigned)gy);
                if (pool == 5)
                    avgpool_backward_s2_kernel<5><<<grid2, 256, 0, s>>>(gin, gout, (int)H_in, (int)W_in, (int)H_out, (int)W_out, (int)planes, ovw);
                else if (pool == 3)
                    avgpool_backward_s2_kernel<3><<<grid2, 256, 0, s>>>(gin, gout, (int)H_in, (int)W_in, (int)H_out, (int)W_out, (int)planes, ovw);
                else
                    avgpool_backward_s2_kernel<2><<<grid2, 256, 0, s>>>(gin, gout, (int)H_in, (int)W_in, (int)H_out, (int)W_out, (int)planes, ovw);
                NZB_OPS_EPILOGUE();
            }
            if (stride == 1)
                avgpool_backward_quad_kernel<1><<<gridq, 256, 0, s>>>(gin, gout, (int)pool, 1, (int)H_in, (int)W_in,
                                                                      (int)H_out, (int)W_out, (int)planes);
            else if (stride == 2)
                avgpool_backward_quad_kernel<2><<<gridq, 256, 0, s>>>(gin, gout, (int)pool, 2, (int)H_in, (int)W_in,
                                                                      (int)H_out, (int)W_out, (int)planes);
            else
                avgpool_backward_quad_kernel<0><<<gridq, 256, 0, s>>>(gin, gout, (int)pool, (int)stride, (int)H_in,
                                                                      (int)W_in, (int)H_out, (int)W_out, (int)planes);
            NZB_OPS_EPILOGUE();
        }
        if (stride == 1)
            avgpool_backward_plane_kernel<1><<<grid, 256, 0, s>>>(gin, gout, (int)pool, 1, (int)pad, (int)H_in, (int)W_in,
                                                                  (int)H_out, (int)W_out, (int)planes);
        else if (stride == 2)
            avgpool_backward_plane_kernel<2><<<grid, 256, 0, s>>>(gin, gout, (int)pool, 2, (int)pad, (int)H_in, (int)W_in,
                                                                  (int)H_out, (int)W_out, (int)planes);
        else
            avgpool_backward_plane_kernel<0><<<grid, 256, 0, s>>>(gin, gout, (int)pool, (int)stride, (int)pad, (int)H_in,
                                                                  (int)W_in, (int)H_out, (int)W_out, (int)planes);
        NZB_OPS_EPILOGUE();
    }
    avgpool_backward_kernel<<<grid_for(total, 256, ds->sm_count), 256, 0, s>>>(gin, gout, pool, stride, pad, H_in,
                                                                               W_in, H_out, W_out, total);
    NZB_OPS_EPILOGUE();
}

int nzb_softmax(float* out, const float* in, int64_t batches, int64_t n, void* stream) {
    if (!out || !in) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    if (batches <= 0 || n <= 0) return NZB_OK;
    softmax_kernel<<<grid_for(batches * 32, 256, ds->sm_count), 256, 0, s>>>(out, in, n, batches);
    NZB_OPS_EPILOGUE();
}

int nzb_softmax_backward(float* gin, const float* y, const float* gout, int64_t batches, int64_t n, int round_f16,
                         void* stream) {
    if (!gin || !y || !gout) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    if (batches <= 0 || n <= 0) return NZB_OK;
    softmax_backward_kernel<<<grid_for(batches * 32, 256, ds->sm_count), 256, 0, s>>>(gin, y, gout, n, batches,
                                                                                      round_f16);
    NZB_OPS_EPILOGUE();
}

int nzb_bce(float* loss_out, const float* predict, const float* target, int64_t n, void* stream) {
    if (!loss_out || !predict || !target) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    if (n <= 0) return NZB_OK;
    bce_kernel<<<grid_for(n, 256, ds->sm_count, 4), 256, 0, s>>>(loss_out, predict, target, n);
    NZB_OPS_EPILOGUE();
}

int nzb_bce_backward(float* out, const float* predict, const float* target, int64_t n, void* stream) {
    if (!out || !predict || !target) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    if (n <= 0) return NZB_OK;
    bce_backward_kernel<<<grid_for(n, 256, ds->sm_count), 256, 0, s>>>(out, predict, target, n);
    NZB_OPS_EPILOGUE();
}

int nzb_adam(float* data, float* m, float* v, const float* grad, float lr, float beta1, float beta2, float eps, int t,
             int64_t n, void* stream) {
    if (!data || !m || !v || !grad) return fail(NZB_ERR_BAD_ARG, "null pointer");
    if (t < 1) return fail(NZB_ERR_BAD_ARG, "t must be >= 1");
    NZB_OPS_PROLOGUE();
    if (n <= 0) return NZB_OK;
    const float c1 = 1.f - powf(beta1, (float)t), c2 = 1.f - powf(beta2, (float)t);
    adam_kernel<<<grid_for(n, 256, ds->sm_count), 256, 0, s>>>(data, m, v, grad, lr, beta1, beta2, eps, c1, c2, n);
    NZB_OPS_EPILOGUE();
}

int nzb_fill(float* data, float value, int64_t n, void* stream) {
    if (!data) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    if (n <= 0) return NZB_OK;
    fill_kernel<<<grid_for(n, 256, ds->sm_count), 256, 0, s>>>(data, value, n);
    NZB_OPS_EPILOGUE();
}

int nzb_expand(float* out, const float* in, int64_t per_batch, int64_t batches, void* stream) {
    if (!out || !in) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    const int64_t total = per_batch * batches;
    if (total <= 0) return NZB_OK;
    expand_kernel<<<grid_for(total, 256, ds->sm_count), 256, 0, s>>>(out, in, per_batch, total);
    NZB_OPS_EPILOGUE();
}

int nzb_scale(float* data, float factor, int64_t n, void* stream) {
    if (!data) return fail(NZB_ERR_BAD_ARG, "null pointer");
    NZB_OPS_PROLOGUE();
    if (n <= 0) return NZB_OK;
    scale_kernel<<<grid_for(n, 256, ds->sm_count), 256, 0, s>>>(data, factor, n);
    NZB_OPS_EPILOGUE();
}

}  // extern "C"
