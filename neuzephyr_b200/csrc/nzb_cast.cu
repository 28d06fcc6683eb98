// fp32 -> fp16 operand staging (HBM-bound). Replaces the Padding kernel
// (NeuZephyr src/OperationKernels.cu:846-860) and, in its transposing form, the
// TransposeKernel pass (:125-160) that MatMulNode::backward runs before its GEMMs:
// the destination is always a dense K-major fp16 matrix [rows][ld_out] whose columns
// cols..ld_out-1 are zero.
#include <cuda_fp16.h>

#include "nzb_internal.h"

namespace nzb {

struct CastParams {
    const float* in;
    __half* out;
    int64_t rows, cols, ld_in, ld_out;
    int64_t nmat1;  // extent of the inner batch dimension
    int64_t in_stride0, in_stride1;
    int64_t nmat;  // total matrices
    const float* mask;  // optional, same layout as `in`: elements whose mask value is <= 0 are staged as 0
};

// Row-preserving cast. One thread produces 8 consecutive halves (one 16-byte store).
template <bool VEC>
__global__ void __launch_bounds__(256) cast_rows_kernel(const CastParams p) {
    const int64_t units_per_row = p.ld_out >> 3;
    const int64_t total = p.nmat * p.rows * units_per_row;
    for (int64_t u = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; u < total;
         u += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c8 = u % units_per_row;
        const int64_t rm = u / units_per_row;
        const int64_t row = rm % p.rows;
        const int64_t mat = rm / p.rows;
        const float* src = p.in + (mat / p.nmat1) * p.in_stride0 + (mat % p.nmat1) * p.in_stride1 + row * p.ld_in;
        const int64_t c = c8 * 8;
        float v[8];
        if (VEC && c + 8 <= p.cols) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(src + c));
            const float4 b = __ldg(reinterpret_cast<const float4*>(src + c + 4));
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            if (p.mask) {
                const float* mk = p.mask + (src - p.in);
                const float4 ma = __ldg(reinterpret_cast<const float4*>(mk + c));
                const float4 mb = __ldg(reinterpret_cast<const float4*>(mk + c + 4));
                v[0] = ma.x > 0.f ? v[0] : 0.f; v[1] = ma.y > 0.f ? v[1] : 0.f;
                v[2] = ma.z > 0.f ? v[2] : 0.f; v[3] = ma.w > 0.f ? v[3] : 0.f;
                v[4] = mb.x > 0.f ? v[4] : 0.f; v[5] = mb.y > 0.f ? v[5] : 0.f;
                v[6] = mb.z > 0.f ? v[6] : 0.f; v[7] = mb.w > 0.f ? v[7] : 0.f;
            }
        } else {
            const float* mk = p.mask ? p.mask + (src - p.in) : nullptr;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                v[j] = (c + j < p.cols) ? __ldg(src + c + j) : 0.f;
                if (mk && c + j < p.cols && !(__ldg(mk + c + j) > 0.f)) v[j] = 0.f;
            }
        }
        uint4 o;
        __half2 h;
        h = __floats2half2_rn(v[0], v[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2half2_rn(v[2], v[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2half2_rn(v[4], v[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2half2_rn(v[6], v[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
        *reinterpret_cast<uint4*>(p.out + (mat * p.rows + row) * p.ld_out + c) = o;
    }
}

// Transposing cast: source is stored [cols][rows] (leading dimension ld_in), destination
// [rows][ld_out]. 64 x 64 tiles through shared memory; both sides coalesced.
__global__ void __launch_bounds__(256) cast_transpose_kernel(const CastParams p) {
    __shared__ float tile[64][65];
    const int64_t tiles_r = (p.rows + 63) >> 6;
    const int64_t tiles_c = p.ld_out >> 6;  // ld_out is a multiple of 64
    const int64_t total = p.nmat * tiles_r * tiles_c;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // load mapping: 64 x 4
    const int wl = threadIdx.x & 31, wr = threadIdx.x >> 5;  // store mapping: 32 pairs x 8 rows
    for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
        const int64_t tc = t % tiles_c;
        const int64_t tm = t / tiles_c;
        const int64_t tr = tm % tiles_r;
        const int64_t mat = tm / tiles_r;
        const float* src = p.in + (mat / p.nmat1) * p.in_stride0 + (mat % p.nmat1) * p.in_stride1;
        const float* mk = p.mask ? p.mask + (src - p.in) : nullptr;
        const int64_t r0 = tr << 6, c0 = tc << 6;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int cl = i * 4 + ty;
            const int64_t c = c0 + cl, r = r0 + tx;
            float v = (c < p.cols && r < p.rows) ? __ldg(src + c * p.ld_in + r) : 0.f;
            if (mk && c < p.cols && r < p.rows && !(__ldg(mk + c * p.ld_in + r) > 0.f)) v = 0.f;
            tile[cl][tx] = v;
        }
        __syncthreads();
        __half* dst = p.out + mat * p.rows * p.ld_out;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int rl = i * 8 + wr;
            const int64_t r = r0 + rl;
            if (r < p.rows) {
                const __half2 h = __floats2half2_rn(tile[2 * wl][rl], tile[2 * wl + 1][rl]);
                *reinterpret_cast<__half2*>(dst + r * p.ld_out + c0 + 2 * wl) = h;
            }
        }
        __syncthreads();
    }
}

int launch_cast(const float* in, __half* out, int64_t rows, int64_t cols, int64_t ld_in, int64_t ld_out,
                int transpose, int64_t nmat0, int64_t nmat1, int64_t in_stride0, int64_t in_stride1,
                cudaStream_t stream) {
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    return launch_cast_on(ds->sm_count, in, out, rows, cols, ld_in, ld_out, transpose, nmat0, nmat1, in_stride0,
                          in_stride1, stream);
}

int launch_cast_on(int sm_count, const float* in, __half* out, int64_t rows, int64_t cols, int64_t ld_in,
                   int64_t ld_out, int transpose, int64_t nmat0, int64_t nmat1, int64_t in_stride0,
                   int64_t in_stride1, cudaStream_t stream) {
    if (rows <= 0 || nmat0 <= 0 || nmat1 <= 0) return NZB_OK;
    if (ld_out % 64 != 0 || ld_out < cols) return fail(NZB_ERR_BAD_ARG, "fp16 leading dimension must be a multiple of 64 and >= cols");
    return launch_cast_masked(sm_count, in, nullptr, out, rows, cols, ld_in, ld_out, transpose, nmat0, nmat1, in_stride0,
                              in_stride1, stream);
}

int launch_cast_masked(int sm_count, const float* in, const float* mask, __half* out, int64_t rows, int64_t cols,
                       int64_t ld_in, int64_t ld_out, int transpose, int64_t nmat0, int64_t nmat1, int64_t in_stride0,
                       int64_t in_stride1, cudaStream_t stream) {
    if (rows <= 0 || nmat0 <= 0 || nmat1 <= 0) return NZB_OK;
    if (ld_out % 64 != 0 || ld_out < cols) return fail(NZB_ERR_BAD_ARG, "fp16 leading dimension must be a multiple of 64 and >= cols");
    CastParams p{in, out, rows, cols, ld_in, ld_out, nmat1, in_stride0, in_stride1, nmat0 * nmat1, mask};
    if (!transpose) {
        const int64_t total = p.nmat * rows * (ld_out >> 3);
        int64_t blocks = (total + 255) / 256;
        const int64_t cap = (int64_t)sm_count * 16;
        if (blocks > cap) blocks = cap;
        const bool vec = (ld_in % 4 == 0) && (in_stride0 % 4 == 0) && (in_stride1 % 4 == 0) &&
                         ((reinterpret_cast<uintptr_t>(in) & 15) == 0) &&
                         (!mask || (reinterpret_cast<uintptr_t>(mask) & 15) == 0);
        if (vec) cast_rows_kernel<true><<<(unsigned)blocks, 256, 0, stream>>>(p);
        else cast_rows_kernel<false><<<(unsigned)blocks, 256, 0, stream>>>(p);
    } else {
        const int64_t total = p.nmat * ((rows + 63) >> 6) * (ld_out >> 6);
        int64_t blocks = total;
        const int64_t cap = (int64_t)sm_count * 16;
        if (blocks > cap) blocks = cap;
        cast_transpose_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
    }
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}

}  // namespace nzb
