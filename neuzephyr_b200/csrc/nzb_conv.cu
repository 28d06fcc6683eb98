// Convolution as an implicit GEMM on sm_100a: no im2col buffer is ever materialised.
//
// Replaces the composition Model::Conv2d builds (NeuZephyr src/Model.cu:244-263):
//   Img2Col (img2colKernel, src/OperationKernels.cu:1308-1328) -> MatMul (the WMMA GEMM,
//   :821-1026) -> Bias (MatrixAddKernel :12-37) -> [ReLU :230-240] -> Col2Img (:1364-1376)
// by ONE kernel, and its backward-data half (col2imgBackward -> GEMMBackward(dC, W^T) ->
// img2colBackward atomics, src/Nodes.cu:660-665, 169-176, 632-640) by the same kernel run
// on dY with flipped taps (gather form, no atomics).
//
// GEMM view: M = output pixels of one image (tiles of 128 consecutive pixels), N = output
// channels, K = C*Kh*Kw in the reference's order k = c*Kh*Kw + kh*Kw + kw.
//   A tile (128 pixels x 64 k): gathered straight from the NCHW fp32 input by the producer
//     warps, rounded to fp16 (RN) in registers and written to shared memory in the
//     tensor core's M-major 128-byte-swizzled layout (pixels are the contiguous direction
//     of both the input image rows and the tile).
//   B tile (BN channels x 64 k): fp16 K-major weights staged once per call, loaded by TMA.
//   D: fp32 accumulators in tensor memory (double buffered).
//   Epilogue: lanes are consecutive pixels, so each channel is written to NCHW with
//     coalesced stores straight from registers, after bias (per pixel x channel matrix as in
//     NeuZephyr, or per channel) / accumulate / ReLU.
// (Generic kernel) CTA = 704 threads: warp 0 weight TMA, warp 1 MMA issue + tensor-memory owner, warps 2-5
// epilogue, warps 6-21 A-tile producers in two groups of eight that fill alternate ring
// stages (every lane keeps 32 gathers in flight, so global-load latency overlaps between
// the groups). Persistent over (image, pixel tile, channel tile).
// Every wait is bounded as in the GEMM kernel.
#include <cuda_fp16.h>

#include <cstdlib>

#include "nzb_internal.h"
#include "nzb_ptx.cuh"

namespace nzb {

struct ConvParams {
    const float* X;  // gathered tensor {N, C, H, W}
    float* Y;        // result {N, Cout, Ho, Wo}
    const float* bias;
    int32_t C, H, W, Cout, Kh, Kw, stride, pad;
    int32_t Ho, Wo, HoWo, K;
    int32_t k_blocks, last_ksteps;
    int32_t tiles_per_image, tiles_n;
    int32_t w_per_sample;  // weight matrix index = image index
    int32_t bias_mode;     // NZB_BIAS_NONE, NZB_BIAS_ROW ([Cout]) or NZB_BIAS_MATRIX ([Ho*Wo][Cout])
    int32_t accumulate, relu;
    // row mode: a tile is a segment of one output row
    int32_t tiles_per_row, tile_px, win_pitch;  // win_pitch: fp32 elements per window row (TMA box width)
    uint32_t win_bytes;                         // bytes one window copy delivers
    int64_t total_tiles;
    int* status;
};

template <int BN_, int STAGES_>
struct ConvCfg {
    static constexpr int BN = BN_, STAGES = STAGES_;
    static constexpr int A_BYTES = 128 * 64 * 2;
    static constexpr int B_BYTES = BN * 64 * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_BYTES = 256;
    static constexpr int EPI_BYTES = 4 * 32 * 33 * 4;  // per epilogue warp: 32 x 33 floats for the bias transpose
    static constexpr int KTAB_BYTES = 16 * 32 * 8;     // per producer warp: 32 (offset, kh, kw) entries
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + KTAB_BYTES + BAR_BYTES;
    static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
    static constexpr int CHUNK = (BN < 32) ? BN : 32;
    static constexpr int THREADS = 22 * 32;
    static_assert(STAGE_BYTES % 1024 == 0, "operand tiles must stay 1024-byte aligned");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared memory of an sm_100 CTA");
};

// A operand descriptor: M-major, SWIZZLE_128B. The tile is stored as 2 pixel blocks of 64
// (8192 bytes apart = leading byte offset) x 8 k-groups of 8 (1024 bytes apart = stride
// byte offset); inside a 1024-byte atom row r = k % 8 holds 64 pixels (128 bytes) with its
// 16-byte chunks XOR-swizzled by r.
__device__ __forceinline__ uint64_t make_sw128_mmajor_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>(8192 >> 4) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// kind::f16, fp16 operands, fp32 accumulate, A M-major (bit 15), B K-major.
__host__ __device__ constexpr uint32_t make_idesc_conv(uint32_t M, uint32_t N) {
    return (1u << 4) | (1u << 15) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

struct ConvTile {
    int32_t img, mt, nt;
};
__device__ __forceinline__ ConvTile decode_conv_tile(const ConvParams& p, int64_t tile) {
    // channel tiles innermost so that the CTAs sharing an input window run together
    ConvTile t;
    t.nt = static_cast<int32_t>(tile % p.tiles_n);
    const int64_t r = tile / p.tiles_n;
    t.mt = static_cast<int32_t>(r % p.tiles_per_image);
    t.img = static_cast<int32_t>(r / p.tiles_per_image);
    return t;
}

template <class Cfg, bool ACC>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
conv2d_igemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmW, const ConvParams p) {
    using namespace ptx;
    constexpr int BN = Cfg::BN, STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* epi = reinterpret_cast<float*>(smem + STAGES * Cfg::STAGE_BYTES);
    int2* ktab_all = reinterpret_cast<int2*>(smem + STAGES * Cfg::STAGE_BYTES + Cfg::EPI_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES + Cfg::EPI_BYTES + Cfg::KTAB_BYTES);
    uint64_t* full = bars;                     // [STAGES] weights landed (tx) + the producer group's arrival
    uint64_t* empty = bars + STAGES;           // [STAGES]
    uint64_t* tfull = bars + 2 * STAGES;       // [2]
    uint64_t* tempty = bars + 2 * STAGES + 2;  // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);  // warp-uniform by construction
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmW);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 2);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], 4);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- weight TMA ----------------
        uint32_t it = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
            const ConvTile t = decode_conv_tile(p, tile);
            const int32_t zw = p.w_per_sample ? t.img : 0;
            for (int32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_relaxed_warp(&empty[s], ph ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    mbar_arrive_expect_tx(&full[s], Cfg::B_BYTES);
                    tma_load_3d(smem + s * Cfg::STAGE_BYTES + Cfg::A_BYTES, &tmW, kb * 64, t.nt * BN, zw, &full[s]);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) {
            // Wait (one bounded budget in total) for weight copies still in flight.
            const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0;
            const long long t0 = clock64();
            for (uint32_t j = first; j < it; j++) {
                while (!mbar_try_wait(&full[j % STAGES], (j / STAGES) & 1)) {
                    if (clock64() - t0 > kWaitCycleLimit) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        constexpr uint32_t idesc = make_idesc_conv(128, BN);
        uint32_t it = 0, tcount = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, tcount++) {
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            if (!mbar_wait_relaxed_warp(&tempty[acc], aph ^ 1, abort_flag)) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BN;
            for (int32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_relaxed_warp(&full[s], ph, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
                const uint64_t da = make_sw128_mmajor_desc(sa);
                const uint64_t db = make_sw128_kmajor_desc(sa + Cfg::A_BYTES);
                const int32_t ksteps = (kb == p.k_blocks - 1) ? p.last_ksteps : 4;
                if (elect_one()) {
                    // A: one k step = two 8-k groups = 2048 bytes = 128 address units;
                    // B: one k step = 32 bytes = 2 address units
                    mma_f16_ss(d_tmem, da, db, idesc, kb > 0 ? 1u : 0u);
                    if (ksteps > 1) mma_f16_ss(d_tmem, da + 128, db + 2, idesc, 1u);
                    if (ksteps > 2) mma_f16_ss(d_tmem, da + 256, db + 4, idesc, 1u);
                    if (ksteps > 3) mma_f16_ss(d_tmem, da + 384, db + 6, idesc, 1u);
                    mma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (ok && elect_one()) mma_commit(&tfull[acc]);
            __syncwarp();
        }
    } else if (warp < 6) {
        // ---------------- epilogue: lanes = consecutive pixels, coalesced per channel ----------------
        const int q = warp & 3;
        uint32_t tcount = 0;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, tcount++) {
            const ConvTile t = decode_conv_tile(p, tile);
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            if (!mbar_wait_relaxed(&tfull[acc], aph, abort_flag)) break;
            tc_fence_after();
            const int32_t pix0 = t.mt * 128 + q * 32;
            const int32_t pix = pix0 + lane;
            const bool pix_ok = pix < p.HoWo;
            float* yb = p.Y + (static_cast<int64_t>(t.img) * p.Cout) * p.HoWo + pix;
            float* bt = epi + (warp - 2) * 32 * 33;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += Cfg::CHUNK) {
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c0;
                uint32_t v[Cfg::CHUNK];
                if constexpr (Cfg::CHUNK == 32) tmem_ld_32x32(taddr, v);
                else tmem_ld_32x16(taddr, v);
                const int32_t co0 = t.nt * BN + c0;
                if (p.bias_mode == NZB_BIAS_MATRIX) {
                    // bias is [pixel][channel]: read with lanes along channels (coalesced), transpose in
                    // shared memory so that each lane ends up with its own pixel's row
                    constexpr int RPI = 32 / Cfg::CHUNK;
                    const int32_t co = co0 + (lane % Cfg::CHUNK);
                    float bv[32 / RPI];
#pragma unroll
                    for (int i = 0; i < 32 / RPI; i++) {
                        const int32_t pp = pix0 + i * RPI + lane / Cfg::CHUNK;
                        bv[i] = (pp < p.HoWo && co < p.Cout) ? __ldg(p.bias + static_cast<int64_t>(pp) * p.Cout + co) : 0.f;
                    }
#pragma unroll
                    for (int i = 0; i < 32 / RPI; i++) bt[(i * RPI + lane / Cfg::CHUNK) * 33 + (lane % Cfg::CHUNK)] = bv[i];
                    __syncwarp();
                }
                tmem_ld_wait();
                // values to accumulate onto are fetched 16 at a time (one memory round trip per group,
                // and few enough registers that the producer warps' budget is not squeezed)
                constexpr int G = Cfg::CHUNK < 16 ? Cfg::CHUNK : 16;
#pragma unroll
                for (int g0 = 0; g0 < Cfg::CHUNK; g0 += G) {
                    float old[ACC ? G : 1];
                    if constexpr (ACC) {
#pragma unroll
                        for (int j = 0; j < G; j++)
                            old[j] = (pix_ok && co0 + g0 + j < p.Cout)
                                         ? yb[static_cast<int64_t>(co0 + g0 + j) * p.HoWo] : 0.f;
                    }
                    if (pix_ok) {
#pragma unroll
                        for (int j = 0; j < G; j++) {
                            const int32_t co = co0 + g0 + j;
                            if (co < p.Cout) {
                                float x = __uint_as_float(v[g0 + j]);
                                if constexpr (ACC) x += old[j];
                                if (p.bias_mode == NZB_BIAS_MATRIX) x += bt[lane * 33 + g0 + j];
                                else if (p.bias_mode == NZB_BIAS_ROW) x += __ldg(p.bias + co);
                                if (p.relu) x = fmaxf(x, 0.f);
                                yb[static_cast<int64_t>(co) * p.HoWo] = x;
                            }
                        }
                    }
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[acc]);
        }
    } else {
        // ---------------- A-tile producers: gather + round + swizzled store ----------------
        // Two groups of eight warps; group g fills the stages of k blocks with (it & 1) == g.
        // Inside a group, warp wi owns pixels [32*(wi&3), +32) of the tile (one per lane) and
        // k columns [32*(wi>>2), +32) of the k block. k-dependent quantities are warp-uniform.
        const int pw = warp - 6;
        const int grp = pw >> 3, wi = pw & 7;
        const int pq = wi & 3, khalf = wi >> 2;
        const int KHW = p.Kh * p.Kw;
        const int plane = p.H * p.W;
        int2* ktab = ktab_all + pw * 32;
        // byte offset of this lane's pixel inside a 128-byte atom row is fixed:
        // pixel m = 32*pq + lane -> 64-pixel block mb = pq >> 1, element e = 32*(pq&1) + lane,
        // 16-byte chunk e >> 3, byte (e & 7) * 2
        const int e = 32 * (pq & 1) + lane;
        const uint32_t chunk = e >> 3, inchunk = (e & 7) * 2;
        uint32_t it = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
            const ConvTile t = decode_conv_tile(p, tile);
            const int32_t pix = t.mt * 128 + pq * 32 + lane;
            const bool pv = pix < p.HoWo;
            const int32_t ho = pix / p.Wo;
            const int32_t h0 = ho * p.stride - p.pad, w0 = (pix - ho * p.Wo) * p.stride - p.pad;
            // validity of every kernel row / column for this pixel, one bit each (Kh, Kw <= 31)
            uint32_t vh = 0, vw = 0;
            if (pv) {
                for (int i = 0; i < p.Kh; i++) vh |= ((unsigned)(h0 + i) < (unsigned)p.H ? 1u : 0u) << i;
                for (int i = 0; i < p.Kw; i++) vw |= ((unsigned)(w0 + i) < (unsigned)p.W ? 1u : 0u) << i;
            }
            const float* xb = p.X + static_cast<int64_t>(t.img) * p.C * plane + static_cast<int64_t>(h0) * p.W + w0;
            for (int32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                if ((it & 1) != (uint32_t)grp) continue;
                // lane j describes k column j of this warp's 32: element offset c*H*W + kh*W + kw and
                // the (kh, kw) bit positions; columns past K point at bit 31, which is never set
                {
                    const int32_t k = kb * 64 + khalf * 32 + lane;
                    const int32_t c = k / KHW;
                    const int32_t r = k - c * KHW;
                    const int32_t kh = r / p.Kw, kw = r - kh * p.Kw;
                    const bool kin = k < p.K;
                    ktab[lane] = make_int2(kin ? c * plane + kh * p.W + kw : 0, kin ? (kh | (kw << 8)) : (31 | (31 << 8)));
                }
                __syncwarp();
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&empty[s], ph ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                uint8_t* sA = smem + s * Cfg::STAGE_BYTES + (pq >> 1) * 8192 + khalf * 4096;
                float a[32];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const int4 e2 = *reinterpret_cast<const int4*>(ktab + j);  // two entries, broadcast read
                    const bool in0 = ((vh >> (e2.y & 0xff)) & (vw >> (e2.y >> 8)) & 1u) != 0;
                    const bool in1 = ((vh >> (e2.w & 0xff)) & (vw >> (e2.w >> 8)) & 1u) != 0;
                    a[j] = in0 ? __ldg(xb + e2.x) : 0.f;
                    a[j + 1] = in1 ? __ldg(xb + e2.z) : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    // k column j of this half: 8-k group j >> 3 (1024-byte atom), row j & 7
                    const uint32_t off = (j >> 3) * 1024 + (j & 7) * 128 + (((chunk ^ (j & 7)) & 7) << 4) + inchunk;
                    *reinterpret_cast<__half*>(sA + off) = __float2half_rn(a[j]);
                }
                // All eight warps of the group have written their part of the stage: one thread then
                // orders those generic-proxy writes before the tensor core's async-proxy reads and
                // publishes the stage. (One proxy fence per stage instead of one per thread: the
                // fence sits on the causality path between every write and the MMA that reads it.)
                asm volatile("bar.sync %0, 256;" ::"r"(1 + grp) : "memory");
                if (wi == 0 && lane == 0) {
                    fence_proxy_async_smem();
                    mbar_arrive(&full[s]);
                }
            }
        }
    }

    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) {
        *p.status = NZB_ERR_DEVICE_TIMEOUT;
        __threadfence_system();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}


// ---------------------------------------------------------------------------
// Row mode: the kernel used whenever an output row is at least 32 pixels wide and the input
// row pitch is a multiple of 16 bytes. A tile is a segment of ONE output row (at most 128
// pixels), so the input it touches is a small window: Kh input rows x ((pixels-1)*stride + Kw)
// columns per channel. For every k block, TMA copies that window for the block's channels
// (a 4-D box of the NCHW fp32 tensor; padding and tails arrive as zeros) into a ring of
// shared-memory window buffers, several k blocks ahead; the producer warps then expand the
// taps from shared memory into the tensor core's A tile, rounding to fp16 on the way. Each
// input element is fetched from global memory once per tile and k block instead of once per
// tap, no per-element bounds test is left, and global-load latency is off the critical path.
// ---------------------------------------------------------------------------
template <int BN_, int STAGES_, int NWIN_>
struct ConvRowCfg {
    static constexpr int BN = BN_, STAGES = STAGES_;
    static constexpr int A_BYTES = 128 * 64 * 2;
    static constexpr int B_BYTES = BN * 64 * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_BYTES = 256;
    static constexpr int EPI_BYTES = 4 * 32 * 33 * 4;
    static constexpr int KTAB_ENTRIES = 4096;  // window offset of every k (whole contraction), built once
    static constexpr int KTAB_BYTES = KTAB_ENTRIES * 4;
    static constexpr int NWIN = NWIN_;        // window ring depth (windows are fetched this far ahead)
    static constexpr int WIN_BYTES = 16384;   // one window buffer (fp32)
    static constexpr int SMEM_BYTES =
        1024 + STAGES * STAGE_BYTES + NWIN * WIN_BYTES + EPI_BYTES + KTAB_BYTES + BAR_BYTES;
    static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
    static constexpr int CHUNK = (BN < 32) ? BN : 32;
    static constexpr int THREADS = 23 * 32;
    static_assert(STAGE_BYTES % 1024 == 0, "operand tiles must stay 1024-byte aligned");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared memory of an sm_100 CTA");
};

struct ConvRowTile {
    int32_t img, ho, wo0, npx, nt;
};
__device__ __forceinline__ ConvRowTile decode_row_tile(const ConvParams& p, int64_t tile) {
    ConvRowTile t;
    t.nt = static_cast<int32_t>(tile % p.tiles_n);
    int64_t r = tile / p.tiles_n;
    const int32_t seg = static_cast<int32_t>(r % p.tiles_per_row);
    r /= p.tiles_per_row;
    t.ho = static_cast<int32_t>(r % p.Ho);
    t.img = static_cast<int32_t>(r / p.Ho);
    t.wo0 = seg * p.tile_px;
    t.npx = min(p.tile_px, p.Wo - t.wo0);
    return t;
}

template <class Cfg, bool ACC>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
conv2d_rows_tcgen05_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                           const ConvParams p) {
    using namespace ptx;
    constexpr int BN = Cfg::BN, STAGES = Cfg::STAGES, NWIN = Cfg::NWIN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* win_all = smem + STAGES * Cfg::STAGE_BYTES;
    float* epi = reinterpret_cast<float*>(win_all + NWIN * Cfg::WIN_BYTES);
    int* ktab_all = reinterpret_cast<int*>(win_all + NWIN * Cfg::WIN_BYTES + Cfg::EPI_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(win_all + NWIN * Cfg::WIN_BYTES + Cfg::EPI_BYTES + Cfg::KTAB_BYTES);
    uint64_t* full = bars;                             // [STAGES] weights landed + tap group arrived
    uint64_t* empty = bars + STAGES;                   // [STAGES]
    uint64_t* tfull = bars + 2 * STAGES;               // [2]
    uint64_t* tempty = bars + 2 * STAGES + 2;          // [2]
    uint64_t* wfull = bars + 2 * STAGES + 4;           // [NWIN] window landed
    uint64_t* wempty = bars + 2 * STAGES + 4 + NWIN;   // [NWIN] window consumed by the 8 warps of a group
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4 + 2 * NWIN);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int KHW = p.Kh * p.Kw;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmW);
        prefetch_tensormap(&tmX);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 9);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], 4);
        }
        for (int w = 0; w < NWIN; w++) {
            mbar_init(&wfull[w], 1);
            mbar_init(&wempty[w], 8);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    // window offset of every k of the (64-padded) contraction: ((c - first channel of k's block) * Kh + kh)
    // * pitch + kw; columns past K get -1. Built once; the tap loop only reads it.
    for (int k = threadIdx.x; k < p.k_blocks * 64; k += Cfg::THREADS) {
        const int c = k / KHW;
        const int r = k - c * KHW;
        const int kh = r / p.Kw, kw = r - kh * p.Kw;
        ktab_all[k] = k < p.K ? ((c - ((k >> 6) << 6) / KHW) * p.Kh + kh) * p.win_pitch + kw : -1;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA: weight tiles ----------------
        uint32_t it = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
            const ConvRowTile t = decode_row_tile(p, tile);
            const int32_t zw = p.w_per_sample ? t.img : 0;
            for (int32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&empty[s], ph ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    mbar_arrive_expect_tx(&full[s], Cfg::B_BYTES);
                    tma_load_3d(smem + s * Cfg::STAGE_BYTES + Cfg::A_BYTES, &tmW, kb * 64, t.nt * BN, zw, &full[s]);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) {
            const long long t0 = clock64();
            const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0;
            for (uint32_t j = first; j < it; j++)
                while (!mbar_try_wait(&full[j % STAGES], (j / STAGES) & 1))
                    if (clock64() - t0 > kWaitCycleLimit) break;
        }
    } else if (warp == 22) {
        // ---------------- TMA: image windows, up to NWIN k blocks ahead of their use ----------------
        uint32_t it = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
            const ConvRowTile t = decode_row_tile(p, tile);
            const int32_t h_base = t.ho * p.stride - p.pad;
            const int32_t w_base = t.wo0 * p.stride - p.pad;
            const int32_t x0 = (w_base >= 0 ? w_base : w_base - 3) / 4 * 4;  // floor to a multiple of 4 elements
            for (int32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                const uint32_t ws = it % NWIN, wph = (it / NWIN) & 1;
                if (!mbar_wait_warp(&wempty[ws], wph ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    mbar_arrive_expect_tx(&wfull[ws], p.win_bytes);
                    tma_load_4d(win_all + ws * Cfg::WIN_BYTES, &tmX, x0, h_base, (kb * 64) / KHW, t.img, &wfull[ws]);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) {
            // one bounded budget for copies still in flight
            const long long t0 = clock64();
            const uint32_t first = it > (uint32_t)NWIN ? it - NWIN : 0;
            for (uint32_t j = first; j < it; j++)
                while (!mbar_try_wait(&wfull[j % NWIN], (j / NWIN) & 1))
                    if (clock64() - t0 > kWaitCycleLimit) break;
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        constexpr uint32_t idesc = make_idesc_conv(128, BN);
        uint32_t it = 0, tcount = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, tcount++) {
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            if (!mbar_wait_warp(&tempty[acc], aph ^ 1, abort_flag)) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BN;
            for (int32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&full[s], ph, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
                const uint64_t da = make_sw128_mmajor_desc(sa);
                const uint64_t db = make_sw128_kmajor_desc(sa + Cfg::A_BYTES);
                const int32_t ksteps = (kb == p.k_blocks - 1) ? p.last_ksteps : 4;
                if (elect_one()) {
                    mma_f16_ss(d_tmem, da, db, idesc, kb > 0 ? 1u : 0u);
                    if (ksteps > 1) mma_f16_ss(d_tmem, da + 128, db + 2, idesc, 1u);
                    if (ksteps > 2) mma_f16_ss(d_tmem, da + 256, db + 4, idesc, 1u);
                    if (ksteps > 3) mma_f16_ss(d_tmem, da + 384, db + 6, idesc, 1u);
                    mma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (ok && elect_one()) mma_commit(&tfull[acc]);
            __syncwarp();
        }
    } else if (warp < 6) {
        // ---------------- epilogue ----------------
        const int q = warp & 3;
        float* bt = epi + (warp - 2) * 32 * 33;
        uint32_t tcount = 0;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, tcount++) {
            const ConvRowTile t = decode_row_tile(p, tile);
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            if (!mbar_wait_relaxed(&tfull[acc], aph, abort_flag)) break;
            tc_fence_after();
            const int32_t m0 = q * 32;
            const int32_t pix0 = t.ho * p.Wo + t.wo0 + m0;
            const int32_t pix = pix0 + lane;
            const bool pix_ok = m0 + lane < t.npx;
            float* yb = p.Y + (static_cast<int64_t>(t.img) * p.Cout) * p.HoWo + pix;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += Cfg::CHUNK) {
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c0;
                uint32_t v[Cfg::CHUNK];
                if constexpr (Cfg::CHUNK == 32) tmem_ld_32x32(taddr, v);
                else tmem_ld_32x16(taddr, v);
                const int32_t co0 = t.nt * BN + c0;
                if (p.bias_mode == NZB_BIAS_MATRIX) {
                    // bias is [pixel][channel]: read with lanes along channels (coalesced, all loads in
                    // flight together), transpose through shared memory so each lane gets its pixel's row
                    constexpr int RPI = 32 / Cfg::CHUNK;  // pixel rows covered per load instruction
                    const int32_t co = co0 + (lane % Cfg::CHUNK);
                    float bv[32 / RPI];
#pragma unroll
                    for (int i = 0; i < 32 / RPI; i++) {
                        const int r = i * RPI + lane / Cfg::CHUNK;
                        bv[i] = (m0 + r < t.npx && co < p.Cout)
                                    ? __ldg(p.bias + static_cast<int64_t>(pix0 + r) * p.Cout + co) : 0.f;
                    }
#pragma unroll
                    for (int i = 0; i < 32 / RPI; i++) bt[(i * RPI + lane / Cfg::CHUNK) * 33 + (lane % Cfg::CHUNK)] = bv[i];
                    __syncwarp();
                }
                tmem_ld_wait();
                // values to accumulate onto are fetched 16 at a time (one memory round trip per group,
                // and few enough registers that the producer warps' budget is not squeezed)
                constexpr int G = Cfg::CHUNK < 16 ? Cfg::CHUNK : 16;
#pragma unroll
                for (int g0 = 0; g0 < Cfg::CHUNK; g0 += G) {
                    float old[ACC ? G : 1];
                    if constexpr (ACC) {
#pragma unroll
                        for (int j = 0; j < G; j++)
                            old[j] = (pix_ok && co0 + g0 + j < p.Cout)
                                         ? yb[static_cast<int64_t>(co0 + g0 + j) * p.HoWo] : 0.f;
                    }
                    if (pix_ok) {
#pragma unroll
                        for (int j = 0; j < G; j++) {
                            const int32_t co = co0 + g0 + j;
                            if (co < p.Cout) {
                                float x = __uint_as_float(v[g0 + j]);
                                if constexpr (ACC) x += old[j];
                                if (p.bias_mode == NZB_BIAS_MATRIX) x += bt[lane * 33 + g0 + j];
                                else if (p.bias_mode == NZB_BIAS_ROW) x += __ldg(p.bias + co);
                                if (p.relu) x = fmaxf(x, 0.f);
                                yb[static_cast<int64_t>(co) * p.HoWo] = x;
                            }
                        }
                    }
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[acc]);
        }
    } else {
        // ---------------- tap expansion: window (fp32, shared) -> A tile (fp16, swizzled) ----------------
        // Two groups of eight warps; group g serves the k blocks with (it & 1) == g. Inside a group
        // warp wi owns pixels [32*(wi&3), +32) (one per lane) and k columns [32*(wi>>2), +32).
        const int pw = warp - 6;
        const int grp = pw >> 3, wi = pw & 7;
        const int pq = wi & 3, khalf = wi >> 2;
        const int e = 32 * (pq & 1) + lane;
        const uint32_t chunk = e >> 3, inchunk = (e & 7) * 2;
        // byte offset of this lane's element inside each of the 8 rows of a 1024-byte atom (swizzled)
        uint32_t rowoff[8];
#pragma unroll
        for (int r = 0; r < 8; r++) rowoff[r] = r * 128 + (((chunk ^ r) & 7) << 4) + inchunk;
        const int mcol = (pq * 32 + lane) * p.stride;  // this lane's pixel as a column offset
        const bool k_tail = (p.K & 63) != 0;
        uint32_t it = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
            const ConvRowTile t = decode_row_tile(p, tile);
            const int32_t w_base = t.wo0 * p.stride - p.pad;
            const int32_t x0 = (w_base >= 0 ? w_base : w_base - 3) / 4 * 4;
            const int lane_off = mcol + (w_base - x0);
            for (int32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                if ((it & 1) != (uint32_t)grp) continue;
                const uint32_t ws = it % NWIN, wph = (it / NWIN) & 1;
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&wfull[ws], wph, abort_flag) || !mbar_wait_warp(&empty[s], ph ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                const float* wl = reinterpret_cast<const float*>(win_all + ws * Cfg::WIN_BYTES) + lane_off;
                const int* kt = ktab_all + kb * 64 + khalf * 32;
                uint8_t* sA = smem + s * Cfg::STAGE_BYTES + (pq >> 1) * 8192 + khalf * 4096;
                float a[32];
                if (k_tail && kb == p.k_blocks - 1) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const int4 o = *reinterpret_cast<const int4*>(kt + j);  // broadcast read
                        a[j] = o.x >= 0 ? wl[o.x] : 0.f;
                        a[j + 1] = o.y >= 0 ? wl[o.y] : 0.f;
                        a[j + 2] = o.z >= 0 ? wl[o.z] : 0.f;
                        a[j + 3] = o.w >= 0 ? wl[o.w] : 0.f;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const int4 o = *reinterpret_cast<const int4*>(kt + j);
                        a[j] = wl[o.x];
                        a[j + 1] = wl[o.y];
                        a[j + 2] = wl[o.z];
                        a[j + 3] = wl[o.w];
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&wempty[ws]);  // window may be refilled
#pragma unroll
                for (int j = 0; j < 32; j++)
                    *reinterpret_cast<__half*>(sA + (j >> 3) * 1024 + rowoff[j & 7]) = __float2half_rn(a[j]);
                // order this warp's generic-proxy writes before the tensor core's async-proxy reads,
                // then publish its part of the stage (8 warps + the weight copy complete the barrier)
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[s]);
            }
        }
    }

    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) {
        *p.status = NZB_ERR_DEVICE_TIMEOUT;
        __threadfence_system();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// TMA im2col mode (stride 1, Kh and Kw <= 4, output rows of at least 32 pixels): the
// tensor core's A tile is delivered by TMA alone, no thread touches it.
//
// The input is staged once per call as Kw fp16 copies, copy kw holding the image shifted
// left by kw - pad columns with the horizontal padding written as zeros:
//   XS[kw][img][c][h][w'] = half(X[img][c][h][w' + kw - pad])        (row pitch Wp, 16-byte multiple)
// With that, the im2col slice for tap column kw, channels [16*cb, +16), all Kh tap rows and
// 64 consecutive output pixels of output row ho is the dense box
//   XS[kw][img][16*cb .. +16][ho - pad .. + Kh][wo0 .. + 64]
// of a 5-D tensor map: 16*Kh rows (k = ci*Kh + kh) of 64 pixels, which with SWIZZLE_128B is
// exactly the M-major operand layout of tcgen05.mma (vertical padding = TMA zero fill). A
// k block is one (kw, cb) pair; the contraction order is k' = ((kw*CB + cb)*16 + ci)*Kh + kh
// and the weights are staged in that order (channels padded to a multiple of 16 with zeros,
// every block padded to 64 columns).
//
// CTA = 192 threads: warp 0 TMA (two image boxes + one weight box per stage), warp 1 MMA,
// warps 2-5 epilogue straight into NCHW. Narrow channel tiles leave room for two CTAs per SM.
// ---------------------------------------------------------------------------
// internal bias mode of the TMA kernel: the {Ho*Wo, Cout} bias matrix transposed to {Cout, Ho*Wo}
constexpr int kBiasMatrixT = 4;

// out[c][r] = in[r][c] for an R x C fp32 matrix (the bias matrix, once per forward call)
__global__ void __launch_bounds__(256) transpose_f32_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                            int64_t R, int64_t C) {
    __shared__ float tile[32][33];
    const int64_t tiles_c = (C + 31) / 32, tiles = ((R + 31) / 32) * tiles_c;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t r0 = (t / tiles_c) * 32, c0 = (t % tiles_c) * 32;
#pragma unroll
        for (int i = ty; i < 32; i += 8)
            if (r0 + i < R && c0 + tx < C) tile[i][tx] = __ldg(in + (r0 + i) * C + c0 + tx);
        __syncthreads();
#pragma unroll
        for (int i = ty; i < 32; i += 8)
            if (c0 + i < C && r0 + tx < R) out[(c0 + i) * R + r0 + tx] = tile[tx][i];
        __syncthreads();
    }
}

struct ConvTmaParams {
    float* Y;
    const float* bias;
    int32_t Cout, Kh, Kw, pad;
    int32_t Ho, Wo, HoWo;
    int32_t cblks;     // ceil(C / 16)
    int32_t k_blocks;  // Kw * cblks
    int32_t tiles_per_row, tiles_n;
    int32_t w_per_sample, img0;  // img0: first image of this chunk (index into Y / weights; XS is chunk-local)
    int32_t bias_mode, relu;
    uint32_t stage_tx;  // bytes one stage's three copies deliver
    int64_t total_tiles;
    int* status;
};

template <int BN_, int STAGES_, int MINB_>
struct ConvTmaCfg {
    static constexpr int BN = BN_, STAGES = STAGES_, MIN_BLOCKS = MINB_;
    static constexpr int A_BYTES = 2 * 8192;  // two 64-pixel blocks of up to 64 k rows
    static constexpr int B_BYTES = BN * 64 * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + BAR_BYTES;
    static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
    static constexpr int CHUNK = (BN < 32) ? BN : 32;
    static constexpr int THREADS = 6 * 32;
    static_assert(STAGE_BYTES % 1024 == 0, "operand tiles must stay 1024-byte aligned");
    static_assert((SMEM_BYTES + 1024) * MINB_ <= 233472, "exceeds the 228 KB shared memory of an sm_100 SM");
    static_assert(TMEM_COLS * MINB_ <= 512, "exceeds the tensor memory of an SM");
};

struct ConvTmaTile {
    int32_t img, ho, wo0, npx, nt;
};
__device__ __forceinline__ ConvTmaTile decode_tma_tile(const ConvTmaParams& p, int64_t tile64) {
    // the host keeps total_tiles below 2^31: 32-bit divisions (a 64-bit one costs hundreds of cycles)
    ConvTmaTile t;
    const uint32_t tile = static_cast<uint32_t>(tile64);
    uint32_t r = tile / (uint32_t)p.tiles_n;
    t.nt = static_cast<int32_t>(tile - r * (uint32_t)p.tiles_n);
    const uint32_t r2 = r / (uint32_t)p.tiles_per_row;
    const int32_t seg = static_cast<int32_t>(r - r2 * (uint32_t)p.tiles_per_row);
    const uint32_t r3 = r2 / (uint32_t)p.Ho;
    t.ho = static_cast<int32_t>(r2 - r3 * (uint32_t)p.Ho);
    t.img = static_cast<int32_t>(r3);
    t.wo0 = seg * 128;
    t.npx = min(128, p.Wo - t.wo0);
    return t;
}

template <class Cfg, bool ACC>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::MIN_BLOCKS)
conv2d_tma_tcgen05_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                          const ConvTmaParams p) {
    using namespace ptx;
    constexpr int BN = Cfg::BN, STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tfull = bars + 2 * STAGES;
    uint64_t* tempty = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmW);
        prefetch_tensormap(&tmX);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], 4);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA: image boxes and weight tiles ----------------
        uint32_t it = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
            const ConvTmaTile t = decode_tma_tile(p, tile);
            const int32_t zw = p.w_per_sample ? p.img0 + t.img : 0;
            int32_t kw = 0, cb = 0;
            for (int32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&empty[s], ph ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
                    mbar_arrive_expect_tx(&full[s], p.stage_tx);
                    tma_load_5d(sa, &tmX, t.wo0, t.ho - p.pad, cb * 16, t.img, kw, &full[s]);
                    tma_load_5d(sa + 8192, &tmX, t.wo0 + 64, t.ho - p.pad, cb * 16, t.img, kw, &full[s]);
                    tma_load_3d(sa + Cfg::A_BYTES, &tmW, kb * 64, t.nt * BN, zw, &full[s]);
                }
                __syncwarp();
                if (++cb == p.cblks) {
                    cb = 0;
                    kw++;
                }
            }
        }
        if (!ok && lane == 0) {
            const long long t0 = clock64();
            const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0;
            for (uint32_t j = first; j < it; j++)
                while (!mbar_try_wait(&full[j % STAGES], (j / STAGES) & 1))
                    if (clock64() - t0 > kWaitCycleLimit) break;
        }
    } else if (warp == 1) {
        // ---------------- MMA issue: Kh steps of 16 k rows per block ----------------
        constexpr uint32_t idesc = make_idesc_conv(128, BN);
        uint32_t it = 0, tcount = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, tcount++) {
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            if (!mbar_wait_warp(&tempty[acc], aph ^ 1, abort_flag)) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BN;
            for (int32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&full[s], ph, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
                const uint64_t da = make_sw128_mmajor_desc(sa);
                const uint64_t db = make_sw128_kmajor_desc(sa + Cfg::A_BYTES);
                if (elect_one()) {
                    mma_f16_ss(d_tmem, da, db, idesc, kb > 0 ? 1u : 0u);
                    if (p.Kh > 1) mma_f16_ss(d_tmem, da + 128, db + 2, idesc, 1u);
                    if (p.Kh > 2) mma_f16_ss(d_tmem, da + 256, db + 4, idesc, 1u);
                    if (p.Kh > 3) mma_f16_ss(d_tmem, da + 384, db + 6, idesc, 1u);
                    mma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (ok && elect_one()) mma_commit(&tfull[acc]);
            __syncwarp();
        }
    } else {
        // ---------------- epilogue: lanes are pixels, one coalesced store per channel ----------------
        const int q = warp & 3;
        uint32_t tcount = 0;
        for (int64_t tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, tcount++) {
            const ConvTmaTile t = decode_tma_tile(p, tile);
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            if (!mbar_wait_relaxed(&tfull[acc], aph, abort_flag)) break;
            tc_fence_after();
            const int32_t m0 = q * 32;
            const int32_t pix0 = t.ho * p.Wo + t.wo0 + m0;
            const int32_t pix = pix0 + lane;
            const bool pix_ok = m0 + lane < t.npx;
            float* yb = p.Y + (static_cast<int64_t>(p.img0 + t.img) * p.Cout) * p.HoWo + pix;
            if (m0 < t.npx) {  // warp-uniform: this quarter of the tile holds pixels
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += Cfg::CHUNK) {
                    const int32_t co0 = t.nt * BN + c0;
                    if (co0 >= p.Cout) break;
                    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c0;
                    // Addends first (bias and, when accumulating, the values already in Y): they do not
                    // depend on the accumulator, so their memory latency overlaps the tensor-memory load.
                    // Every mode decision is taken once per chunk, not per element (a branch per element
                    // costs more than the store it guards).
                    float add[Cfg::CHUNK];
                    const bool whole = co0 + Cfg::CHUNK <= p.Cout;
                    float* yg = yb + static_cast<int64_t>(co0) * p.HoWo;
                    if (p.bias_mode == NZB_BIAS_MATRIX) {
                        // bias is [pixel][channel]: this lane's pixel owns CHUNK consecutive floats
                        const float* bp = p.bias + static_cast<int64_t>(pix_ok ? pix : pix0) * p.Cout + co0;
                        if (whole && (p.Cout & 3) == 0) {
#pragma unroll
                            for (int j = 0; j < Cfg::CHUNK; j += 4) {
                                const float4 b4 = __ldg(reinterpret_cast<const float4*>(bp + j));
                                add[j] = b4.x; add[j + 1] = b4.y; add[j + 2] = b4.z; add[j + 3] = b4.w;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < Cfg::CHUNK; j++) add[j] = co0 + j < p.Cout ? __ldg(bp + j) : 0.f;
                        }
                    } else if (p.bias_mode == kBiasMatrixT) {
                        // the bias matrix transposed to [channel][pixel] by the launcher: lanes are
                        // consecutive pixels, so every load is one contiguous 128-byte request
                        const float* bp = p.bias + static_cast<int64_t>(co0) * p.HoWo + (pix_ok ? pix : pix0);
#pragma unroll
                        for (int j = 0; j < Cfg::CHUNK; j++)
                            add[j] = (whole || co0 + j < p.Cout) ? __ldg(bp + static_cast<int64_t>(j) * p.HoWo) : 0.f;
                    } else if (p.bias_mode == NZB_BIAS_ROW) {
#pragma unroll
                        for (int j = 0; j < Cfg::CHUNK; j++) add[j] = __ldg(p.bias + min(co0 + j, p.Cout - 1));
                    } else {
#pragma unroll
                        for (int j = 0; j < Cfg::CHUNK; j++) add[j] = 0.f;
                    }
                    if constexpr (ACC) {
                        if (pix_ok) {
                            if (whole) {
#pragma unroll
                                for (int j = 0; j < Cfg::CHUNK; j++) add[j] += yg[static_cast<int64_t>(j) * p.HoWo];
                            } else {
#pragma unroll
                                for (int j = 0; j < Cfg::CHUNK; j++)
                                    if (co0 + j < p.Cout) add[j] += yg[static_cast<int64_t>(j) * p.HoWo];
                            }
                        }
                    }
                    uint32_t v[Cfg::CHUNK];
                    if constexpr (Cfg::CHUNK == 32) tmem_ld_32x32(taddr, v);
                    else tmem_ld_32x16(taddr, v);
                    tmem_ld_wait();
                    const float floor_v = p.relu ? 0.f : -INFINITY;
                    if (pix_ok) {
                        if (whole) {
#pragma unroll
                            for (int j = 0; j < Cfg::CHUNK; j++)
                                yg[static_cast<int64_t>(j) * p.HoWo] = fmaxf(__uint_as_float(v[j]) + add[j], floor_v);
                        } else {
#pragma unroll
                            for (int j = 0; j < Cfg::CHUNK; j++)
                                if (co0 + j < p.Cout)
                                    yg[static_cast<int64_t>(j) * p.HoWo] = fmaxf(__uint_as_float(v[j]) + add[j], floor_v);
                        }
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[acc]);
        }
    }

    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) {
        *p.status = NZB_ERR_DEVICE_TIMEOUT;
        __threadfence_system();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// The 8 + KW - 1 values x[w0 - pad .. w0 - pad + 8 + KW - 2] of one image row (zero outside [0, W)).
// When the row is 16-byte aligned and the eight central values lie inside it, they come as two float4
// loads and only the KW - 1 halo values as scalars: 4 load instructions instead of 10 for KW = 3, and the
// vector loads of a warp are contiguous. PAD is a template argument so that every register index is
// static (the caller switches on the run-time pad).
template <int KW, int PAD>
__device__ __forceinline__ void load_shift_window_p(float (&v)[8 + KW - 1], const float* __restrict__ src, int w0,
                                                    int W, bool row_aligned) {
    if (row_aligned && w0 + 8 <= W) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(src + w0));
        const float4 b = __ldg(reinterpret_cast<const float4*>(src + w0 + 4));
        const float c[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 8 + KW - 1; j++) {
            if (j >= PAD && j < PAD + 8) {
                v[j] = c[j - PAD];
            } else {
                const int w = w0 + j - PAD;
                v[j] = (unsigned)w < (unsigned)W ? __ldg(src + w) : 0.f;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8 + KW - 1; j++) {
            const int w = w0 + j - PAD;
            v[j] = (unsigned)w < (unsigned)W ? __ldg(src + w) : 0.f;
        }
    }
}
template <int KW>
__device__ __forceinline__ void load_shift_window(float (&v)[8 + KW - 1], const float* __restrict__ src, int w0, int pad,
                                                  int W, bool row_aligned) {
    if (pad == 0) load_shift_window_p<KW, 0>(v, src, w0, W, row_aligned);
    else if (pad == 1 && KW > 1) load_shift_window_p<KW, (KW > 1 ? 1 : 0)>(v, src, w0, W, row_aligned);
    else if (pad == 2 && KW > 2) load_shift_window_p<KW, (KW > 2 ? 2 : 0)>(v, src, w0, W, row_aligned);
    else load_shift_window_p<KW, KW - 1>(v, src, w0, W, row_aligned);
}

// Input staging for the TMA im2col mode: Kw shifted fp16 copies, 8 output columns per thread
// (one 16-byte store per copy). rows = images * C * H of this chunk.
template <int KW>
__global__ void __launch_bounds__(256) shift_copies_kernel(__half* __restrict__ xs, const float* __restrict__ x,
                                                           int64_t rows, int W, int Wp, int pad) {
    const int W8 = Wp >> 3;
    const int64_t total = rows * W8;
    const int64_t copy_stride = rows * Wp;
    const bool aligned = (W & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;  // every row starts on 16 bytes
    for (int64_t u = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; u < total; u += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = u / W8;
        const int w0 = (int)(u - row * W8) * 8;
        const float* src = x + row * W;
        float v[8 + KW - 1];
        load_shift_window<KW>(v, src, w0, pad, W, aligned);
#pragma unroll
        for (int kw = 0; kw < KW; kw++) {
            uint4 o;
            __half2 t;
            t = __floats2half2_rn(v[kw], v[kw + 1]); o.x = *reinterpret_cast<uint32_t*>(&t);
            t = __floats2half2_rn(v[kw + 2], v[kw + 3]); o.y = *reinterpret_cast<uint32_t*>(&t);
            t = __floats2half2_rn(v[kw + 4], v[kw + 5]); o.z = *reinterpret_cast<uint32_t*>(&t);
            t = __floats2half2_rn(v[kw + 6], v[kw + 7]); o.w = *reinterpret_cast<uint32_t*>(&t);
            *reinterpret_cast<uint4*>(xs + kw * copy_stride + row * Wp + w0) = o;
        }
    }
}

// One pass over dY for the whole backward of a convolution layer: applies ReLU's mask (Y > 0),
// writes the KW shifted fp16 copies the data-gradient kernel reads (copy `pad` is the unshifted one,
// which the weight-gradient kernel reads) and adds the batch sum into the {Ho*Wo, Cout} bias-gradient
// matrix. A block owns 32 channels x 64 pixels of one output row and walks the images of the chunk,
// so every bias element has one owner (no atomics) and is written once, through a shared-memory
// transpose that makes the [pixel][channel] writes contiguous.
template <int KW, int CT>
__global__ void __launch_bounds__(256) dy_prepare_kernel(__half* __restrict__ xs, const float* __restrict__ dy,
                                                         const float* __restrict__ ymask, float* __restrict__ dbias,
                                                         int n, int Cout, int Ho, int Wo, int Wp, int pad, int only_kw) {
    // a block owns CT channels x PX pixels of one output row (CT = 16 or 32, PX = 128 or 64)
    constexpr int UNITS = 256 / CT, PX = UNITS * 8;
    __shared__ float tile[PX][CT + 1];
    const int segs = (Wp + PX - 1) / PX, cblks = (Cout + CT - 1) / CT;
    const int co_l = threadIdx.x / UNITS, w8 = threadIdx.x % UNITS;
    const int64_t copy_stride = (int64_t)n * Cout * Ho * Wp;
    const bool aligned = (Wo & 3) == 0 && (reinterpret_cast<uintptr_t>(dy) & 15) == 0;
    const bool aligned_mask = (Wo & 3) == 0 && (reinterpret_cast<uintptr_t>(ymask) & 15) == 0;
    for (int64_t blk = blockIdx.x; blk < (int64_t)cblks * Ho * segs; blk += gridDim.x) {
        const int seg = (int)(blk % segs);
        const int ho = (int)((blk / segs) % Ho);
        const int cb = (int)(blk / ((int64_t)segs * Ho));
        const int co = cb * CT + co_l, w0 = seg * PX + w8 * 8;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] = 0.f;
        if (co < Cout && w0 < Wp) {
            for (int img = 0; img < n; img++) {
                const int64_t row = ((int64_t)img * Cout + co) * Ho + ho;
                const float* src = dy + row * Wo;
                const float* msk = ymask ? ymask + row * Wo : nullptr;
                float v[8 + KW - 1];
                load_shift_window<KW>(v, src, w0, pad, Wo, aligned);
                if (msk) {
                    float mv[8 + KW - 1];
                    load_shift_window<KW>(mv, msk, w0, pad, Wo, aligned_mask);
#pragma unroll
                    for (int j = 0; j < 8 + KW - 1; j++)
                        if (!(mv[j] > 0.f)) v[j] = 0.f;  // outside the row both are zero already
                }
#pragma unroll
                for (int kw = 0; kw < KW; kw++) {
                    if (only_kw >= 0 && kw != only_kw) continue;
                    uint4 o;
                    __half2 t;
                    t = __floats2half2_rn(v[kw], v[kw + 1]); o.x = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2half2_rn(v[kw + 2], v[kw + 3]); o.y = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2half2_rn(v[kw + 4], v[kw + 5]); o.z = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2half2_rn(v[kw + 6], v[kw + 7]); o.w = *reinterpret_cast<uint32_t*>(&t);
                    *reinterpret_cast<uint4*>(xs + kw * copy_stride + row * Wp + w0) = o;
                }
                if (dbias) {
                    // the unshifted values v[pad .. pad + 7] (pad <= KW - 1), with static register indices
#pragma unroll
                    for (int pp = 0; pp < KW; pp++)
                        if (pp == pad) {
#pragma unroll
                            for (int j = 0; j < 8; j++) acc[j] += v[j + pp];
                        }
                }
            }
        }
        if (dbias) {
#pragma unroll
            for (int j = 0; j < 8; j++) tile[w8 * 8 + j][co_l] = acc[j];
            __syncthreads();
            const int c2 = threadIdx.x % CT;
#pragma unroll
            for (int i = 0; i < PX * CT / 256; i++) {
                const int px = threadIdx.x / CT + i * (256 / CT);
                const int w = seg * PX + px, c = cb * CT + c2;
                if (w < Wo && c < Cout) dbias[((int64_t)ho * Wo + w) * Cout + c] += tile[px][c2];
            }
            __syncthreads();
        }
    }
}

// Weight staging for the TMA im2col mode, forward (flip = 0) and backward-data (flip = 1) forms.
//   out[wb][r][k'],  k' = (kw*CB + cb)*64 + ci*Kh + kh,  cin = cb*16 + ci  (zero for cin >= Cin and
//   for the columns 16*Kh..63 of every block: a block is one aligned 128-byte row segment, so a
//   weight tile costs the TMA unit one request per row)
//   forward:  r = co,  cin = c:   w[wb][(c*Kh + kh)*Kw + kw][co]
//   backward: r = c,   cin = co:  w[wb][(c*Kh + (Kh-1-kh))*Kw + (Kw-1-kw)][co]
// with w = {wN, 1, C*Kh*Kw, Cout} as the reference stores it.
__global__ void __launch_bounds__(256) tma_weights_kernel(__half* __restrict__ out, const float* __restrict__ w,
                                                          int64_t C, int64_t Cout, int64_t Kh, int64_t Kw, int64_t wN,
                                                          int flip) {
    const int64_t Cin = flip ? Cout : C, R = flip ? C : Cout;
    const int64_t CB = (Cin + 15) / 16, Kt = Kw * CB * 64;
    const int64_t total = wN * R * Kt;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t k = i % Kt, r = (i / Kt) % R, wb = i / (Kt * R);
        const int64_t j = k % 64, blk = k / 64;
        const int64_t kh = j % Kh, ci = j / Kh, cb = blk % CB, kw = blk / CB;
        const int64_t cin = cb * 16 + ci;
        float v = 0.f;
        if (ci < 16 && cin < Cin) {
            const int64_t c = flip ? r : cin, co = flip ? cin : r;
            const int64_t kh2 = flip ? Kh - 1 - kh : kh, kw2 = flip ? Kw - 1 - kw : kw;
            v = __ldg(w + wb * C * Kh * Kw * Cout + ((c * Kh + kh2) * Kw + kw2) * Cout + co);
        }
        out[i] = __float2half_rn(v);
    }
}

// ---------------------------------------------------------------------------
// Weight gradient in the TMA im2col mode: dW[k][co] += sum over pixels of col[pixel][k] * dY[pixel][co].
// The contraction runs over pixels, so both operands are K-major with pixels contiguous:
//   A (128 rows of k x 128 pixels): the same boxes of the shifted copies the forward kernel
//     loads -- rows (ci, kh) of tap column kw, here up to 128/Kh channels per box -- read as a
//     K-major operand;
//   B (BN channels x 128 pixels): boxes of an fp16 copy of dY with the same row pitch, whose
//     columns past Wo are zero, so that the extra columns of a copy never contribute.
// A k block is 128 pixels of one output row (two 64-pixel boxes per operand). An output tile
// (one tap column x one channel block x BN output channels) is shared among several CTAs
// along the pixel space; partial sums are added to dW with fp32 atomics.
// ---------------------------------------------------------------------------
struct WgradParams {
    float* dW;  // {wN, 1, C*Kh*Kw, Cout}
    int32_t C, Cout, Kh, Kw, pad;
    int32_t Ho, segs;        // segs = ceil(Wo / 128)
    int32_t cbw;             // channels per A box (cbw * Kh <= 128)
    int32_t cblks;           // ceil(C / cbw)
    int32_t tiles_n;         // ceil(Cout / BN)
    int32_t tiles;           // Kw * cblks * tiles_n
    int32_t groups;          // separate outputs: images when weights are per sample, else 1
    int32_t imgs_per_group;  // images contracted into one output
    int32_t splits;          // CTAs sharing one (tile, group)
    int32_t img0;            // first image of this chunk (selects the per-sample dW)
    int32_t w_per_sample;
    uint32_t stage_tx;
    int64_t kb_per_group;  // imgs_per_group * Ho * segs
    int64_t total_items;   // tiles * groups * splits
    int* status;
};

template <int BN_, int STAGES_, int MINB_ = 1>
struct WgradCfg {
    static constexpr int BN = BN_, STAGES = STAGES_, MIN_BLOCKS = MINB_;
    static constexpr int A_BYTES = 2 * 16384;       // two 64-pixel halves of 128 k rows
    static constexpr int B_BYTES = 2 * BN * 128;    // two 64-pixel halves of BN channels
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + BAR_BYTES;
    static constexpr int TMEM_COLS = (BN < 32) ? 32 : BN;
    static constexpr int THREADS = 6 * 32;
    static_assert(STAGE_BYTES % 1024 == 0, "operand tiles must stay 1024-byte aligned");
    static_assert((SMEM_BYTES + 1024) * MINB_ <= 233472, "exceeds the 228 KB shared memory of an sm_100 SM");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::MIN_BLOCKS)
conv2d_wgrad_tma_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDY,
                        const WgradParams p) {
    using namespace ptx;
    constexpr int BN = Cfg::BN, STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tfull = bars + 2 * STAGES;   // [1]
    uint64_t* tempty = bars + 2 * STAGES + 1;  // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmX);
        prefetch_tensormap(&tmDY);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(tfull, 1);
        mbar_init(tempty, 4);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // item -> (tile, group, split); tile -> (kw, cb, nt)
    auto item_range = [&](uint32_t item, int32_t& kw, int32_t& cb, int32_t& nt, int32_t& group, uint32_t& kk0,
                          uint32_t& kk1) {
        const uint32_t split = item % (uint32_t)p.splits;
        uint32_t r = item / (uint32_t)p.splits;
        group = (int32_t)(r % (uint32_t)p.groups);
        r /= (uint32_t)p.groups;
        nt = (int32_t)(r % (uint32_t)p.tiles_n);
        r /= (uint32_t)p.tiles_n;
        cb = (int32_t)(r % (uint32_t)p.cblks);
        kw = (int32_t)(r / (uint32_t)p.cblks);
        kk0 = (uint32_t)(p.kb_per_group * split / p.splits);
        kk1 = (uint32_t)(p.kb_per_group * (split + 1) / p.splits);
    };

    if (warp == 0) {
        // ---------------- TMA ----------------
        uint32_t it = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < p.total_items && ok; item += gridDim.x) {
            int32_t kw, cb, nt, group;
            uint32_t kk0, kk1;
            item_range((uint32_t)item, kw, cb, nt, group, kk0, kk1);
            // k block -> (image, output row, segment), advanced incrementally
            const uint32_t per_img = (uint32_t)(p.Ho * p.segs);
            int32_t img = (int32_t)(kk0 / per_img);
            uint32_t rem = kk0 - (uint32_t)img * per_img;
            int32_t ho = (int32_t)(rem / (uint32_t)p.segs), seg = (int32_t)(rem % (uint32_t)p.segs);
            img += p.w_per_sample ? group : 0;
            for (uint32_t kk = kk0; kk < kk1; kk++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&empty[s], ph ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
                    uint8_t* sb = sa + Cfg::A_BYTES;
                    const int32_t w0 = seg * 128;
                    mbar_arrive_expect_tx(&full[s], p.stage_tx);
                    tma_load_5d(sa, &tmX, w0, ho - p.pad, cb * p.cbw, img, kw, &full[s]);
                    tma_load_5d(sa + 16384, &tmX, w0 + 64, ho - p.pad, cb * p.cbw, img, kw, &full[s]);
                    tma_load_4d(sb, &tmDY, w0, ho, nt * BN, img, &full[s]);
                    tma_load_4d(sb + BN * 128, &tmDY, w0 + 64, ho, nt * BN, img, &full[s]);
                }
                __syncwarp();
                if (++seg == p.segs) {
                    seg = 0;
                    if (++ho == p.Ho) {
                        ho = 0;
                        img++;
                    }
                }
            }
        }
        if (!ok && lane == 0) {
            const long long t0 = clock64();
            const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0;
            for (uint32_t j = first; j < it; j++)
                while (!mbar_try_wait(&full[j % STAGES], (j / STAGES) & 1))
                    if (clock64() - t0 > kWaitCycleLimit) break;
        }
    } else if (warp == 1) {
        // ---------------- MMA: 8 steps of 16 pixels per k block ----------------
        constexpr uint32_t idesc = make_idesc_f16_f32(128, BN);
        uint32_t it = 0, icount = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < p.total_items && ok; item += gridDim.x, icount++) {
            int32_t kw, cb, nt, group;
            uint32_t kk0, kk1;
            item_range((uint32_t)item, kw, cb, nt, group, kk0, kk1);
            if (!mbar_wait_warp(tempty, (icount & 1) ^ 1, abort_flag)) break;
            tc_fence_after();
            for (uint32_t kk = kk0; kk < kk1; kk++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&full[s], ph, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
                const uint64_t da0 = make_sw128_kmajor_desc(sa), da1 = make_sw128_kmajor_desc(sa + 16384);
                const uint64_t db0 = make_sw128_kmajor_desc(sa + Cfg::A_BYTES);
                const uint64_t db1 = make_sw128_kmajor_desc(sa + Cfg::A_BYTES + BN * 128);
                if (elect_one()) {
                    mma_f16_ss(tmem_base, da0, db0, idesc, kk > kk0 ? 1u : 0u);
                    mma_f16_ss(tmem_base, da0 + 2, db0 + 2, idesc, 1u);
                    mma_f16_ss(tmem_base, da0 + 4, db0 + 4, idesc, 1u);
                    mma_f16_ss(tmem_base, da0 + 6, db0 + 6, idesc, 1u);
                    mma_f16_ss(tmem_base, da1, db1, idesc, 1u);
                    mma_f16_ss(tmem_base, da1 + 2, db1 + 2, idesc, 1u);
                    mma_f16_ss(tmem_base, da1 + 4, db1 + 4, idesc, 1u);
                    mma_f16_ss(tmem_base, da1 + 6, db1 + 6, idesc, 1u);
                    mma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (ok && elect_one()) mma_commit(tfull);
            __syncwarp();
        }
    } else {
        // ---------------- epilogue: lane = k row, atomic adds into dW[k][co .. co+BN) ----------------
        const int q = warp & 3;
        uint32_t icount = 0;
        for (int64_t item = blockIdx.x; item < p.total_items; item += gridDim.x, icount++) {
            int32_t kw, cb, nt, group;
            uint32_t kk0, kk1;
            item_range((uint32_t)item, kw, cb, nt, group, kk0, kk1);
            if (!mbar_wait_relaxed(tfull, icount & 1, abort_flag)) break;
            tc_fence_after();
            const int32_t m = q * 32 + lane;  // row of the tile: (channel in box, kh)
            const int32_t ci = m / p.Kh, kh = m - ci * p.Kh;
            const int32_t c = cb * p.cbw + ci;
            const bool row_ok = kk1 > kk0 && ci < p.cbw && c < p.C;
            const int64_t K = (int64_t)p.C * p.Kh * p.Kw;
            float* dst = p.dW + (p.w_per_sample ? (int64_t)(p.img0 + group) * K * p.Cout : 0) +
                         ((int64_t)(c * p.Kh + kh) * p.Kw + kw) * p.Cout + nt * BN;
            constexpr int CH = BN < 16 ? BN : 16;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CH) {
                if (nt * BN + c0 >= p.Cout) break;
                uint32_t v[16];
                tmem_ld_32x16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c0, v);
                tmem_ld_wait();
                if (row_ok) {
                    if (nt * BN + c0 + 16 <= p.Cout) {
#pragma unroll
                        for (int j = 0; j < 16; j++) atomicAdd(dst + c0 + j, __uint_as_float(v[j]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (nt * BN + c0 + j < p.Cout) atomicAdd(dst + c0 + j, __uint_as_float(v[j]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty);
        }
    }

    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) {
        *p.status = NZB_ERR_DEVICE_TIMEOUT;
        __threadfence_system();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// Weight gradient with the tap columns stacked along N (3x3 .. 3-wide kernels, up to 64 output channels).
//
// A tcgen05.mma costs about the same whatever its N, and the kernel above issues 8 instructions of N = BN per
// 128 pixels FOR EACH tap column, each time against another shifted copy of x. Substituting u = wo + kw - pad,
//   dW[(ci,kh),kw][co] = sum_{ho,u} x[ci][ho+kh-pad][u] * dY[co][ho][u - kw + pad],
// the shift moves to dY, and the Kw shifted copies of dY already exist (the data gradient reads them: copy kw'
// holds dY shifted by kw' - (K-1-pad), so tap column kw reads copy K-1-kw). One instruction then multiplies
// the UNSHIFTED x rows (16 channels x Kh rows) by all Kw copies at once: B has Kw*BN rows (copy, channel),
// the accumulator Kw*BN columns. A third of the instructions, and x is staged once instead of Kw times.
// ---------------------------------------------------------------------------
template <int BN_, int STAGES_, int MINB_>
struct WgradStackCfg {
    static constexpr int BN = BN_, STAGES = STAGES_, MIN_BLOCKS = MINB_, NS = 3;
    static constexpr int BNN = NS * BN;             // accumulator columns: (copy, channel)
    static constexpr int A_BYTES = 2 * 8192;        // two 64-pixel halves of up to 64 k rows (16 channels x Kh)
    static constexpr int B_HALF = BNN * 128;        // one 64-pixel half of NS * BN rows
    static constexpr int STAGE_BYTES = A_BYTES + 2 * B_HALF;
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + BAR_BYTES;
    static constexpr int TMEM_COLS = BNN <= 64 ? 64 : BNN <= 128 ? 128 : 256;
    static constexpr int THREADS = 6 * 32;
    static_assert(STAGE_BYTES % 1024 == 0 && B_HALF % 1024 == 0, "operand tiles must stay 1024-byte aligned");
    static_assert(BNN % 16 == 0 && BNN <= 256, "instruction N");
    static_assert((SMEM_BYTES + 1024) * MINB_ <= 233472, "exceeds the 228 KB shared memory of an sm_100 SM");
    static_assert(TMEM_COLS * MINB_ <= 512, "exceeds the tensor memory of an SM");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::MIN_BLOCKS)
conv2d_wgrad_stacked_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDY,
                            const WgradParams p) {
    using namespace ptx;
    constexpr int BN = Cfg::BN, STAGES = Cfg::STAGES, BNN = Cfg::BNN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tfull = bars + 2 * STAGES;
    uint64_t* tempty = bars + 2 * STAGES + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmX);
        prefetch_tensormap(&tmDY);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(tfull, 1);
        mbar_init(tempty, 4);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // item -> (tile, group, split); tile -> (cb, nt). p.segs counts 128-column blocks of the INPUT width.
    auto item_range = [&](uint32_t item, int32_t& cb, int32_t& nt, int32_t& group, uint32_t& kk0, uint32_t& kk1) {
        const uint32_t split = item % (uint32_t)p.splits;
        uint32_t r = item / (uint32_t)p.splits;
        group = (int32_t)(r % (uint32_t)p.groups);
        r /= (uint32_t)p.groups;
        nt = (int32_t)(r % (uint32_t)p.tiles_n);
        cb = (int32_t)(r / (uint32_t)p.tiles_n);
        kk0 = (uint32_t)(p.kb_per_group * split / p.splits);
        kk1 = (uint32_t)(p.kb_per_group * (split + 1) / p.splits);
    };

    if (warp == 0) {
        // ---------------- TMA ----------------
        uint32_t it = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < p.total_items && ok; item += gridDim.x) {
            int32_t cb, nt, group;
            uint32_t kk0, kk1;
            item_range((uint32_t)item, cb, nt, group, kk0, kk1);
            const uint32_t per_img = (uint32_t)(p.Ho * p.segs);
            int32_t img = (int32_t)(kk0 / per_img);
            uint32_t rem = kk0 - (uint32_t)img * per_img;
            int32_t ho = (int32_t)(rem / (uint32_t)p.segs), seg = (int32_t)(rem % (uint32_t)p.segs);
            img += p.w_per_sample ? group : 0;
            for (uint32_t kk = kk0; kk < kk1; kk++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&empty[s], ph ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
                    uint8_t* sb = sa + Cfg::A_BYTES;
                    const int32_t w0 = seg * 128;
                    mbar_arrive_expect_tx(&full[s], p.stage_tx);
                    tma_load_4d(sa, &tmX, w0, ho - p.pad, cb * 16, img, &full[s]);
                    tma_load_4d(sa + 8192, &tmX, w0 + 64, ho - p.pad, cb * 16, img, &full[s]);
                    tma_load_5d(sb, &tmDY, w0, ho, nt * BN, img, 0, &full[s]);
                    tma_load_5d(sb + Cfg::B_HALF, &tmDY, w0 + 64, ho, nt * BN, img, 0, &full[s]);
                }
                __syncwarp();
                if (++seg == p.segs) {
                    seg = 0;
                    if (++ho == p.Ho) {
                        ho = 0;
                        img++;
                    }
                }
            }
        }
        if (!ok && lane == 0) {
            const long long t0 = clock64();
            const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0;
            for (uint32_t j = first; j < it; j++)
                while (!mbar_try_wait(&full[j % STAGES], (j / STAGES) & 1))
                    if (clock64() - t0 > kWaitCycleLimit) break;
        }
    } else if (warp == 1) {
        // ---------------- MMA: 8 steps of 16 pixels per k block, N = NS * BN ----------------
        constexpr uint32_t idesc = make_idesc_f16_f32(128, BNN);
        uint32_t it = 0, icount = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < p.total_items && ok; item += gridDim.x, icount++) {
            int32_t cb, nt, group;
            uint32_t kk0, kk1;
            item_range((uint32_t)item, cb, nt, group, kk0, kk1);
            if (!mbar_wait_warp(tempty, (icount & 1) ^ 1, abort_flag)) break;
            tc_fence_after();
            for (uint32_t kk = kk0; kk < kk1; kk++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&full[s], ph, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
                const uint64_t da0 = make_sw128_kmajor_desc(sa), da1 = make_sw128_kmajor_desc(sa + 8192);
                const uint64_t db0 = make_sw128_kmajor_desc(sa + Cfg::A_BYTES);
                const uint64_t db1 = make_sw128_kmajor_desc(sa + Cfg::A_BYTES + Cfg::B_HALF);
                if (elect_one()) {
                    mma_f16_ss(tmem_base, da0, db0, idesc, kk > kk0 ? 1u : 0u);
                    mma_f16_ss(tmem_base, da0 + 2, db0 + 2, idesc, 1u);
                    mma_f16_ss(tmem_base, da0 + 4, db0 + 4, idesc, 1u);
                    mma_f16_ss(tmem_base, da0 + 6, db0 + 6, idesc, 1u);
                    mma_f16_ss(tmem_base, da1, db1, idesc, 1u);
                    mma_f16_ss(tmem_base, da1 + 2, db1 + 2, idesc, 1u);
                    mma_f16_ss(tmem_base, da1 + 4, db1 + 4, idesc, 1u);
                    mma_f16_ss(tmem_base, da1 + 6, db1 + 6, idesc, 1u);
                    mma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (ok && elect_one()) mma_commit(tfull);
            __syncwarp();
        }
    } else {
        // ---------------- epilogue: lane = k row (channel, kh); columns = (copy, channel out) ----------------
        const int q = warp & 3;
        uint32_t icount = 0;
        for (int64_t item = blockIdx.x; item < p.total_items; item += gridDim.x, icount++) {
            int32_t cb, nt, group;
            uint32_t kk0, kk1;
            item_range((uint32_t)item, cb, nt, group, kk0, kk1);
            if (!mbar_wait_relaxed(tfull, icount & 1, abort_flag)) break;
            tc_fence_after();
            const int32_t m = q * 32 + lane;
            const int32_t ci = m / p.Kh, kh = m - ci * p.Kh;
            const int32_t c = cb * 16 + ci;
            const bool row_ok = kk1 > kk0 && ci < 16 && c < p.C;
            const int64_t K = (int64_t)p.C * p.Kh * p.Kw;
            float* row = p.dW + (p.w_per_sample ? (int64_t)(p.img0 + group) * K * p.Cout : 0) +
                         (int64_t)(c * p.Kh + kh) * p.Kw * p.Cout + nt * BN;
            if (q * 32 < 16 * p.Kh) {  // warp-uniform: quarters past the last k row hold nothing
#pragma unroll 1
                for (int c0 = 0; c0 < BNN; c0 += 16) {
                    const int32_t copy = c0 / BN, co0 = c0 - copy * BN;
                    if (nt * BN + co0 >= p.Cout) continue;
                    uint32_t v[16];
                    tmem_ld_32x16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c0, v);
                    tmem_ld_wait();
                    if (row_ok) {
                        float* dst = row + (int64_t)(p.Kw - 1 - copy) * p.Cout + co0;  // copy kw' serves tap column K-1-kw'
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (nt * BN + co0 + j < p.Cout) atomicAdd(dst + j, __uint_as_float(v[j]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty);
        }
    }

    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) {
        *p.status = NZB_ERR_DEVICE_TIMEOUT;
        __threadfence_system();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// Weight staging for backward-data: W2[c][co*Kh*Kw + kh'*Kw + kw'] =
//   half(W[wb][(c*Kh + (Kh-1-kh'))*Kw + (Kw-1-kw')][co])  -- the flipped-tap kernel whose
// forward convolution over dY is the gradient with respect to the input.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) flip_weights_kernel(__half* __restrict__ out, const float* __restrict__ w,
                                                           int64_t C, int64_t Cout, int64_t Kh, int64_t Kw, int64_t Kp2,
                                                           int64_t wN) {
    const int64_t K2 = Cout * Kh * Kw;
    const int64_t total = wN * C * Kp2;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t k2 = i % Kp2;
        const int64_t c = (i / Kp2) % C;
        const int64_t b = i / (Kp2 * C);
        float v = 0.f;
        if (k2 < K2) {
            const int64_t co = k2 / (Kh * Kw), r = k2 % (Kh * Kw);
            const int64_t kh = Kh - 1 - r / Kw, kw = Kw - 1 - r % Kw;
            v = __ldg(w + (b * C * Kh * Kw + (c * Kh + kh) * Kw + kw) * Cout + co);
        }
        out[i] = __float2half_rn(v);
    }
}

// ---------------------------------------------------------------------------
// Weight gradient staging. dW[k][co] += sum over (b, p) of col[b][p][k] * dy[b][co][p] is a GEMM
// with a very long contraction (b, p); both operands are staged K-major in fp16:
//   colT[k][bl*HoWo + p] = half(x[b0+bl][c][ho*s-pad+kh][wo*s-pad+kw])   (k = c*Kh*Kw + kh*Kw + kw)
//   dyT [co][bl*HoWo + p] = half(dy[b0+bl][co][p])
// and the split-k GEMM kernel does the rest. (The reference materialises the fp32 im2col
// buffer, transposes it and runs GEMMBackwardParallel: src/Nodes.cu:177-181.)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) im2col_f16_kmajor_kernel(__half* __restrict__ out, const float* __restrict__ x,
                                                                int C, int H, int W, int Kh, int Kw, int stride,
                                                                int pad, int Ho, int Wo, int64_t b0, int nb, int K,
                                                                int64_t Qp) {
    // blockIdx.y = k row (one (c, kh, kw) per block row); a thread produces 8 consecutive q
    // (one 16-byte store), walking (image, ho, wo) incrementally.
    const int k = blockIdx.y;
    const int c = k / (Kh * Kw), r = k % (Kh * Kw);
    const int kh = r / Kw, kw = r % Kw;
    const int HoWo = Ho * Wo;
    const int64_t Q = (int64_t)nb * HoWo;
    __half* orow = out + (int64_t)k * Qp;
    for (int64_t q0 = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * 8; q0 < Q;
         q0 += (int64_t)gridDim.x * blockDim.x * 8) {
        int bl = (int)(q0 / HoWo);
        const int pp = (int)(q0 - (int64_t)bl * HoWo);
        int ho = pp / Wo, wo = pp - ho * Wo;
        float v[8];
        if (wo + 8 <= Wo && q0 + 8 <= Q) {
            // all eight pixels lie in one output row: one row pointer, column checks only at the edges
            const int h = ho * stride - pad + kh, w0 = wo * stride - pad + kw;
            if ((unsigned)h >= (unsigned)H) {
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = 0.f;
            } else {
                const float* row = x + (((b0 + bl) * C + c) * (int64_t)H + h) * W;
                if (w0 >= 0 && w0 + 7 * stride < W) {
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] = __ldg(row + w0 + j * stride);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int w = w0 + j * stride;
                        v[j] = (unsigned)w < (unsigned)W ? __ldg(row + w) : 0.f;
                    }
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                v[j] = 0.f;
                if (q0 + j < Q) {
                    const int h = ho * stride - pad + kh, w = wo * stride - pad + kw;
                    if ((unsigned)h < (unsigned)H && (unsigned)w < (unsigned)W)
                        v[j] = __ldg(x + (((b0 + bl) * C + c) * (int64_t)H + h) * W + w);
                }
                if (++wo == Wo) {
                    wo = 0;
                    if (++ho == Ho) {
                        ho = 0;
                        bl++;
                    }
                }
            }
        }
        uint4 o;
        __half2 t;
        t = __floats2half2_rn(v[0], v[1]); o.x = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2half2_rn(v[2], v[3]); o.y = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2half2_rn(v[4], v[5]); o.z = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2half2_rn(v[6], v[7]); o.w = *reinterpret_cast<uint32_t*>(&t);
        *reinterpret_cast<uint4*>(orow + q0) = o;  // q0 % 8 == 0 and Qp % 64 == 0: aligned, inside the row
    }
}

__global__ void __launch_bounds__(256) dy_f16_kmajor_kernel(__half* __restrict__ out, const float* __restrict__ dy,
                                                            int Cout, int HoWo, int64_t b0, int nb, int64_t Qp) {
    const int co = blockIdx.y;
    const int64_t Q = (int64_t)nb * HoWo;
    __half* orow = out + (int64_t)co * Qp;
    const bool vec = (HoWo % 8 == 0) && ((reinterpret_cast<uintptr_t>(dy) & 15) == 0);
    for (int64_t q0 = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * 8; q0 < Q;
         q0 += (int64_t)gridDim.x * blockDim.x * 8) {
        float v[8];
        if (vec) {
            const int bl = (int)(q0 / HoWo);
            const int pp = (int)(q0 - (int64_t)bl * HoWo);
            const float* src = dy + ((b0 + bl) * Cout + co) * (int64_t)HoWo + pp;
            const float4 a = __ldg(reinterpret_cast<const float4*>(src));
            const float4 b = __ldg(reinterpret_cast<const float4*>(src + 4));
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int64_t q = q0 + j;
                v[j] = 0.f;
                if (q < Q) {
                    const int64_t bl = q / HoWo, pp = q - bl * HoWo;
                    v[j] = __ldg(dy + ((b0 + bl) * Cout + co) * (int64_t)HoWo + pp);
                }
            }
        }
        uint4 o;
        __half2 t;
        t = __floats2half2_rn(v[0], v[1]); o.x = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2half2_rn(v[2], v[3]); o.y = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2half2_rn(v[4], v[5]); o.z = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2half2_rn(v[6], v[7]); o.w = *reinterpret_cast<uint32_t*>(&t);
        *reinterpret_cast<uint4*>(orow + q0) = o;
    }
}

// dbias[p][co] += sum_b dy[b][co][p]   (AddNode::backward on the untied conv bias after
// col2imgBackward; src/Nodes.cu:106-121, 660-665). Tiled transpose-reduce, coalesced both ways.
__global__ void __launch_bounds__(256) conv_bias_grad_kernel(float* __restrict__ dbias, const float* __restrict__ dy,
                                                             int64_t N, int64_t Cout, int64_t HoWo) {
    __shared__ float tile[32][33];
    const int64_t tp = (HoWo + 31) >> 5, tc = (Cout + 31) >> 5;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int64_t t = blockIdx.x; t < tp * tc; t += gridDim.x) {
        const int64_t p0 = (t / tc) << 5, c0 = (t % tc) << 5;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int64_t co = c0 + ty + i * 8, pp = p0 + tx;
            float s = 0.f;
            if (co < Cout && pp < HoWo)
                for (int64_t b = 0; b < N; b++) s += __ldg(dy + (b * Cout + co) * HoWo + pp);
            tile[ty + i * 8][tx] = s;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int64_t pp = p0 + ty + i * 8, co = c0 + tx;
            if (pp < HoWo && co < Cout) dbias[pp * Cout + co] += tile[tx][ty + i * 8];
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
static int make_weight_map(CUtensorMap* map, const __half* base, int64_t K, int64_t Kp, int64_t rows, int64_t nmat,
                           int box_rows) {
    EncodeTiledFn enc;
    int rc = get_encode_tiled(&enc);
    if (rc != NZB_OK) return rc;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)nmat};
    cuuint64_t strides[2] = {(cuuint64_t)Kp * 2, (cuuint64_t)rows * (cuuint64_t)Kp * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return NZB_OK;
}

// Runs the implicit-GEMM kernel: Y (op)= conv(X, W16) with W16 staged as [wN][Cout][Kp].
struct ConvRun {
    const float* X;
    float* Y;
    const float* bias;
    int64_t N, C, H, W, Cout, Kh, Kw, stride, pad, Ho, Wo;
    int32_t w_per_sample, bias_mode, accumulate, relu;
};

template <class Cfg>
static int run_conv_cfg(const ConvRun& r, const __half* W16, int64_t Kp, int64_t wN, const DeviceState& ds,
                        cudaStream_t stream) {
    ConvParams p{};
    p.X = r.X; p.Y = r.Y; p.bias = r.bias;
    p.C = (int32_t)r.C; p.H = (int32_t)r.H; p.W = (int32_t)r.W; p.Cout = (int32_t)r.Cout;
    p.Kh = (int32_t)r.Kh; p.Kw = (int32_t)r.Kw; p.stride = (int32_t)r.stride; p.pad = (int32_t)r.pad;
    p.Ho = (int32_t)r.Ho; p.Wo = (int32_t)r.Wo; p.HoWo = (int32_t)(r.Ho * r.Wo);
    p.K = (int32_t)(r.C * r.Kh * r.Kw);
    p.k_blocks = (p.K + 63) / 64;
    p.last_ksteps = (p.K - (p.k_blocks - 1) * 64 + 15) / 16;
    p.tiles_per_image = (p.HoWo + 127) / 128;
    p.w_per_sample = r.w_per_sample;
    p.bias_mode = r.bias ? r.bias_mode : NZB_BIAS_NONE;
    p.accumulate = r.accumulate; p.relu = r.relu;
    p.status = ds.status_dev;
    p.tiles_n = (p.Cout + Cfg::BN - 1) / Cfg::BN;
    CUtensorMap tmW;
    int rc = make_weight_map(&tmW, W16, p.K, Kp, p.Cout, wN, Cfg::BN);
    if (rc != NZB_OK) return rc;
    static std::atomic<uint64_t> smem_set[2];  // per kernel instantiation, one bit per device
    {
        int rc_attr = ensure_dynamic_smem(smem_set[0], reinterpret_cast<const void*>(conv2d_igemm_tcgen05_kernel<Cfg, false>), Cfg::SMEM_BYTES);
        if (rc_attr == NZB_OK)
            rc_attr = ensure_dynamic_smem(smem_set[1], reinterpret_cast<const void*>(conv2d_igemm_tcgen05_kernel<Cfg, true>), Cfg::SMEM_BYTES);
        if (rc_attr != NZB_OK) return rc_attr;
    }
    p.total_tiles = (int64_t)r.N * p.tiles_per_image * p.tiles_n;
    const int64_t grid = p.total_tiles < ds.sm_count ? p.total_tiles : ds.sm_count;
    if (p.accumulate)
        conv2d_igemm_tcgen05_kernel<Cfg, true><<<(unsigned)grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tmW, p);
    else
        conv2d_igemm_tcgen05_kernel<Cfg, false><<<(unsigned)grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tmW, p);
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}

template <class Cfg>
static int run_conv_rows_cfg(const ConvRun& r, const __half* W16, int64_t Kp, int64_t wN, const DeviceState& ds,
                             int tiles_per_row, int tile_px, int box_w, int box_c, cudaStream_t stream) {
    ConvParams p{};
    p.X = r.X; p.Y = r.Y; p.bias = r.bias;
    p.C = (int32_t)r.C; p.H = (int32_t)r.H; p.W = (int32_t)r.W; p.Cout = (int32_t)r.Cout;
    p.Kh = (int32_t)r.Kh; p.Kw = (int32_t)r.Kw; p.stride = (int32_t)r.stride; p.pad = (int32_t)r.pad;
    p.Ho = (int32_t)r.Ho; p.Wo = (int32_t)r.Wo; p.HoWo = (int32_t)(r.Ho * r.Wo);
    p.K = (int32_t)(r.C * r.Kh * r.Kw);
    p.k_blocks = (p.K + 63) / 64;
    p.last_ksteps = (p.K - (p.k_blocks - 1) * 64 + 15) / 16;
    p.w_per_sample = r.w_per_sample;
    p.bias_mode = r.bias ? r.bias_mode : NZB_BIAS_NONE;
    p.accumulate = r.accumulate; p.relu = r.relu;
    p.status = ds.status_dev;
    p.tiles_n = (p.Cout + Cfg::BN - 1) / Cfg::BN;
    p.tiles_per_row = tiles_per_row; p.tile_px = tile_px; p.win_pitch = box_w;
    p.win_bytes = (uint32_t)(box_w * r.Kh * box_c * 4);
    CUtensorMap tmW, tmX;
    int rc = make_weight_map(&tmW, W16, p.K, Kp, p.Cout, wN, Cfg::BN);
    if (rc != NZB_OK) return rc;
    {
        EncodeTiledFn enc;
        rc = get_encode_tiled(&enc);
        if (rc != NZB_OK) return rc;
        cuuint64_t dims[4] = {(cuuint64_t)r.W, (cuuint64_t)r.H, (cuuint64_t)r.C, (cuuint64_t)r.N};
        cuuint64_t strides[3] = {(cuuint64_t)r.W * 4, (cuuint64_t)r.H * r.W * 4, (cuuint64_t)r.C * r.H * r.W * 4};
        cuuint32_t box[4] = {(cuuint32_t)box_w, (cuuint32_t)r.Kh, (cuuint32_t)box_c, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        CUresult cr = enc(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(r.X), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled (image window) failed with CUresult %d", (int)cr);
    }
    static std::atomic<uint64_t> smem_set[2];  // per kernel instantiation, one bit per device
    {
        int rc_attr = ensure_dynamic_smem(smem_set[0], reinterpret_cast<const void*>(conv2d_rows_tcgen05_kernel<Cfg, false>), Cfg::SMEM_BYTES);
        if (rc_attr == NZB_OK)
            rc_attr = ensure_dynamic_smem(smem_set[1], reinterpret_cast<const void*>(conv2d_rows_tcgen05_kernel<Cfg, true>), Cfg::SMEM_BYTES);
        if (rc_attr != NZB_OK) return rc_attr;
    }
    p.total_tiles = (int64_t)r.N * r.Ho * tiles_per_row * p.tiles_n;
    const int64_t grid = p.total_tiles < ds.sm_count ? p.total_tiles : ds.sm_count;
    if (p.accumulate)
        conv2d_rows_tcgen05_kernel<Cfg, true><<<(unsigned)grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tmW, tmX, p);
    else
        conv2d_rows_tcgen05_kernel<Cfg, false><<<(unsigned)grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tmW, tmX, p);
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}

static int run_conv(const ConvRun& r, const __half* W16, int64_t Kp, int64_t wN, cudaStream_t stream) {
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    if (r.N <= 0 || r.Cout <= 0 || r.Ho <= 0 || r.Wo <= 0) return NZB_OK;
    if (r.Ho * r.Wo > INT32_MAX - 256 || r.C * r.Kh * r.Kw > INT32_MAX - 256 || r.C * r.H * r.W > INT32_MAX)
        return fail(NZB_ERR_UNSUPPORTED, "per-image extent exceeds 2^31");
    if (r.Kh > 31 || r.Kw > 31) return fail(NZB_ERR_UNSUPPORTED, "kernel extent above 31");
    if (r.Wo >= 32 && r.W % 4 == 0 && round_up(r.C * r.Kh * r.Kw, 64) <= ConvRowCfg<16, 4, 6>::KTAB_ENTRIES && (reinterpret_cast<uintptr_t>(r.X) & 15) == 0) {
        // row mode if the fp32 window of one k block (a TMA box) fits its shared-memory buffer
        const int tiles_per_row = (int)((r.Wo + 127) / 128);
        const int tile_px = (int)((r.Wo + tiles_per_row - 1) / tiles_per_row);
        // columns a tile touches, plus up to 3 for rounding the first column down to 16 bytes,
        // rounded up to a whole number of 16-byte units; unused tile rows (pixels past the
        // segment) still read inside the box row they start in or the rows after it
        int box_w = (int)((tile_px - 1) * r.stride + r.Kw) + 3;
        box_w = (box_w + 3) / 4 * 4;
        const int64_t khw = r.Kh * r.Kw;
        int64_t box_c = (63 + khw - 1) / khw + 1;
        if (box_c > r.C) box_c = r.C;
        const int64_t elems = (int64_t)box_w * r.Kh * box_c;
        const int64_t reach = elems + 128 * r.stride + r.Kw + 4;  // furthest element an unused tile row may read
        if (box_w <= 256 && r.Kh <= 256 && box_c <= 256 && reach * 4 <= ConvRowCfg<16, 4, 6>::WIN_BYTES * 2 &&
            elems * 4 <= ConvRowCfg<16, 4, 6>::WIN_BYTES) {
            if (r.Cout > 128) return run_conv_rows_cfg<ConvRowCfg<256, 2, 5>>(r, W16, Kp, wN, *ds, tiles_per_row, tile_px, box_w, (int)box_c, stream);
            if (r.Cout > 64) return run_conv_rows_cfg<ConvRowCfg<128, 3, 6>>(r, W16, Kp, wN, *ds, tiles_per_row, tile_px, box_w, (int)box_c, stream);
            if (r.Cout > 32) return run_conv_rows_cfg<ConvRowCfg<64, 4, 6>>(r, W16, Kp, wN, *ds, tiles_per_row, tile_px, box_w, (int)box_c, stream);
            if (r.Cout > 16) return run_conv_rows_cfg<ConvRowCfg<32, 4, 6>>(r, W16, Kp, wN, *ds, tiles_per_row, tile_px, box_w, (int)box_c, stream);
            return run_conv_rows_cfg<ConvRowCfg<16, 4, 6>>(r, W16, Kp, wN, *ds, tiles_per_row, tile_px, box_w, (int)box_c, stream);
        }
    }
    if (r.Cout > 128) return run_conv_cfg<ConvCfg<256, 4>>(r, W16, Kp, wN, *ds, stream);
    if (r.Cout > 64) return run_conv_cfg<ConvCfg<128, 6>>(r, W16, Kp, wN, *ds, stream);
    if (r.Cout > 32) return run_conv_cfg<ConvCfg<64, 8>>(r, W16, Kp, wN, *ds, stream);
    if (r.Cout > 16) return run_conv_cfg<ConvCfg<32, 8>>(r, W16, Kp, wN, *ds, stream);
    return run_conv_cfg<ConvCfg<16, 8>>(r, W16, Kp, wN, *ds, stream);
}

// Bytes of staged operands one pass may hold (images are processed in chunks that fit). The
// environment variable NZB_CONV_STAGE_BYTES overrides the default, which lets tests run the
// chunked path on small tensors.
static int64_t stage_budget(int64_t dflt) {
    static const int64_t env = [] {
        const char* e = getenv("NZB_CONV_STAGE_BYTES");
        return e ? atoll(e) : (long long)0;
    }();
    return env > 0 ? env : dflt;
}

// ---- TMA im2col mode: planning and launch ----------------------------------------------------
struct TmaPlan {
    bool ok;
    int64_t Kt;         // staged contraction length: Kw * ceil(Cin/16) blocks of 64 (16 * Kh used)
    int64_t Wp;         // row pitch of the shifted copies (elements)
    int64_t w_bytes;    // staged weights
    int64_t per_image;  // shifted copies of one image
    int64_t nchunk;     // images staged and convolved per pass
};
// Cin, Hin, Win: the tensor the taps slide over; R: output channels; Ho, Wo: output extent.
static TmaPlan tma_plan(int64_t N, int64_t Cin, int64_t Hin, int64_t Win, int64_t R, int64_t Kh, int64_t Kw,
                        int64_t stride, int64_t Ho, int64_t Wo, int64_t wN) {
    TmaPlan t{};
    t.ok = stride == 1 && Kh <= 4 && Kw <= 4 && Wo >= 32 && N > 0 && Hin < (int64_t(1) << 30) && Win < (int64_t(1) << 30);
    const int64_t cb = (Cin + 15) / 16;
    t.Kt = Kw * cb * 64;
    t.Wp = round_up(Wo, 64);  // rows start on 128-byte lines: one TMA request per box row
    t.w_bytes = round_up(wN * R * t.Kt * 2, 256);
    t.per_image = round_up(Kw * Cin * Hin * t.Wp * 2, 256);
    const int64_t budget = stage_budget(int64_t(1) << 30);
    int64_t n = budget / (t.per_image > 0 ? t.per_image : 1);
    if (n < 1) n = 1;
    if (n > N) n = N > 0 ? N : 1;
    if (N > 0) n = (N + (N + n - 1) / n - 1) / ((N + n - 1) / n);  // equal-sized passes
    t.nchunk = n;
    if (t.Kt > INT32_MAX - 256 || Cin > INT32_MAX || R > INT32_MAX) t.ok = false;
    return t;
}

// Y {N, R, Ho, Wo} (op)= conv(X {N, Cin, Hin, Win}, w) with stride 1; flip selects the backward-data form of
// the weights (w is always the layer's {wN, 1, C*Kh*Kw, Cout} tensor). ws holds plan.w_bytes + nchunk * per_image.
struct ConvTmaRun {
    const float* X;
    float* Y;
    const float* bias;
    const float* w;
    int64_t N, Cin, Hin, Win, R, Kh, Kw, pad, Ho, Wo;
    int64_t layerC, layerCout;  // the layer's own channel counts (weight tensor extents)
    int32_t w_per_sample, bias_mode, accumulate, relu, flip;
    const __half* staged;  // shifted copies of exactly these N images, already written (skips the staging pass)
    float* bias_t;         // scratch of Ho*Wo*R floats for the transposed bias matrix (null: read it as stored)
};

template <class Cfg>
static int run_conv_tma_cfg(const ConvTmaRun& r, const TmaPlan& pl, void* ws, const DeviceState& ds, cudaStream_t stream) {
    EncodeTiledFn enc;
    int rc = get_encode_tiled(&enc);
    if (rc != NZB_OK) return rc;
    const int64_t wN = r.w_per_sample ? r.N : 1;
    __half* W16 = reinterpret_cast<__half*>(ws);
    __half* XS = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(ws) + pl.w_bytes);
    {
        const int64_t total = wN * r.R * pl.Kt;
        int64_t blocks = (total + 255) / 256;
        if (blocks > (int64_t)ds.sm_count * 16) blocks = (int64_t)ds.sm_count * 16;
        tma_weights_kernel<<<(unsigned)blocks, 256, 0, stream>>>(W16, r.w, r.layerC, r.layerCout, r.Kh, r.Kw, wN, r.flip);
        NZB_CUDA_TRY(cudaGetLastError());
    }
    CUtensorMap tmW;
    {
        cuuint64_t dims[3] = {(cuuint64_t)pl.Kt, (cuuint64_t)r.R, (cuuint64_t)wN};
        cuuint64_t strides[2] = {(cuuint64_t)pl.Kt * 2, (cuuint64_t)r.R * pl.Kt * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)Cfg::BN, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult cr = enc(&tmW, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, W16, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled (weights) failed with CUresult %d", (int)cr);
    }
    static std::atomic<uint64_t> smem_set[2];  // per kernel instantiation, one bit per device
    {
        int rc_attr = ensure_dynamic_smem(smem_set[0], reinterpret_cast<const void*>(conv2d_tma_tcgen05_kernel<Cfg, false>), Cfg::SMEM_BYTES);
        if (rc_attr == NZB_OK)
            rc_attr = ensure_dynamic_smem(smem_set[1], reinterpret_cast<const void*>(conv2d_tma_tcgen05_kernel<Cfg, true>), Cfg::SMEM_BYTES);
        if (rc_attr != NZB_OK) return rc_attr;
    }
    ConvTmaParams p{};
    p.Y = r.Y; p.bias = r.bias;
    p.Cout = (int32_t)r.R; p.Kh = (int32_t)r.Kh; p.Kw = (int32_t)r.Kw; p.pad = (int32_t)r.pad;
    p.Ho = (int32_t)r.Ho; p.Wo = (int32_t)r.Wo; p.HoWo = (int32_t)(r.Ho * r.Wo);
    p.cblks = (int32_t)((r.Cin + 15) / 16);
    p.k_blocks = p.Kw * p.cblks;
    p.tiles_per_row = (int32_t)((r.Wo + 127) / 128);
    p.tiles_n = (p.Cout + Cfg::BN - 1) / Cfg::BN;
    p.w_per_sample = r.w_per_sample;
    p.bias_mode = r.bias ? r.bias_mode : NZB_BIAS_NONE;
    if (p.bias_mode == NZB_BIAS_MATRIX && r.bias_t && r.N >= 4 && r.R > 64) {  // pays once several images reuse it; up to 64 channels a lane reading its pixel's row as stored measured faster
        // [pixel][channel] as the reference stores it -> [channel][pixel], which the epilogue (lanes =
        // pixels) reads contiguously; 2 x Ho*Wo*Cout*4 bytes of traffic once per call
        const int64_t tiles = ((r.Ho * r.Wo + 31) / 32) * ((r.R + 31) / 32);
        const int64_t cap = (int64_t)ds.sm_count * 16;
        transpose_f32_kernel<<<(unsigned)(tiles < cap ? tiles : cap), 256, 0, stream>>>(r.bias_t, r.bias, r.Ho * r.Wo, r.R);
        NZB_CUDA_TRY(cudaGetLastError());
        p.bias = r.bias_t;
        p.bias_mode = kBiasMatrixT;
    }
    p.relu = r.relu;
    p.stage_tx = (uint32_t)(2 * 64 * r.Kh * 16 * 2 + Cfg::B_BYTES);
    p.status = ds.status_dev;
    const int64_t chunk = r.staged ? r.N : pl.nchunk;
    if (r.staged) XS = const_cast<__half*>(r.staged);
    for (int64_t img0 = 0; img0 < r.N; img0 += chunk) {
        const int64_t n = r.N - img0 < chunk ? r.N - img0 : chunk;
        const int64_t rows = n * r.Cin * r.Hin;
        if (!r.staged) {
            const int64_t total = rows * (pl.Wp / 8);
            int64_t blocks = (total + 255) / 256;
            if (blocks > (int64_t)ds.sm_count * 32) blocks = (int64_t)ds.sm_count * 32;
            const float* src = r.X + img0 * r.Cin * r.Hin * r.Win;
            switch (r.Kw) {
                case 1: shift_copies_kernel<1><<<(unsigned)blocks, 256, 0, stream>>>(XS, src, rows, (int)r.Win, (int)pl.Wp, (int)r.pad); break;
                case 2: shift_copies_kernel<2><<<(unsigned)blocks, 256, 0, stream>>>(XS, src, rows, (int)r.Win, (int)pl.Wp, (int)r.pad); break;
                case 3: shift_copies_kernel<3><<<(unsigned)blocks, 256, 0, stream>>>(XS, src, rows, (int)r.Win, (int)pl.Wp, (int)r.pad); break;
                default: shift_copies_kernel<4><<<(unsigned)blocks, 256, 0, stream>>>(XS, src, rows, (int)r.Win, (int)pl.Wp, (int)r.pad); break;
            }
            NZB_CUDA_TRY(cudaGetLastError());
        }
        CUtensorMap tmX;
        {
            const cuuint64_t row_b = (cuuint64_t)pl.Wp * 2;
            cuuint64_t dims[5] = {(cuuint64_t)pl.Wp, (cuuint64_t)r.Hin, (cuuint64_t)r.Cin, (cuuint64_t)n, (cuuint64_t)r.Kw};
            cuuint64_t strides[4] = {row_b, row_b * r.Hin, row_b * r.Hin * r.Cin, row_b * r.Hin * r.Cin * n};
            cuuint32_t box[5] = {64, (cuuint32_t)r.Kh, 16, 1, 1};
            cuuint32_t estr[5] = {1, 1, 1, 1, 1};
            CUresult cr = enc(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, XS, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (cr != CUDA_SUCCESS) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled (shifted copies) failed with CUresult %d", (int)cr);
        }
        p.img0 = (int32_t)img0;
        p.total_tiles = n * r.Ho * p.tiles_per_row * p.tiles_n;
        if (p.total_tiles > INT32_MAX) return fail(NZB_ERR_UNSUPPORTED, "more than 2^31 output tiles in one pass");
        const int64_t cap = (int64_t)ds.sm_count * Cfg::MIN_BLOCKS;
        const int64_t grid = p.total_tiles < cap ? p.total_tiles : cap;
        if (r.accumulate)
            conv2d_tma_tcgen05_kernel<Cfg, true><<<(unsigned)grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tmW, tmX, p);
        else
            conv2d_tma_tcgen05_kernel<Cfg, false><<<(unsigned)grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tmW, tmX, p);
        NZB_CUDA_TRY(cudaGetLastError());
    }
    return NZB_OK;
}

static int run_conv_tma(const ConvTmaRun& r, const TmaPlan& pl, void* ws, cudaStream_t stream) {
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    if (r.Ho * r.Wo > INT32_MAX - 256 || r.N * r.Ho > INT32_MAX) return fail(NZB_ERR_UNSUPPORTED, "per-image extent exceeds 2^31");
    if (r.R > 128) return run_conv_tma_cfg<ConvTmaCfg<256, 4, 1>>(r, pl, ws, *ds, stream);
    if (r.R > 64) return run_conv_tma_cfg<ConvTmaCfg<128, 3, 2>>(r, pl, ws, *ds, stream);
    if (r.R > 32) return run_conv_tma_cfg<ConvTmaCfg<64, 4, 2>>(r, pl, ws, *ds, stream);
    if (r.R > 16) return run_conv_tma_cfg<ConvTmaCfg<32, 5, 2>>(r, pl, ws, *ds, stream);
    return run_conv_tma_cfg<ConvTmaCfg<16, 4, 3>>(r, pl, ws, *ds, stream);
}

// ---- weight gradient in the TMA im2col mode: planning and launch --------------------------------
struct WgradPlan {
    bool ok;
    int64_t Wp, per_image, nchunk;
    int32_t cbw;
};
static WgradPlan wgrad_plan(const nzb_conv_desc* d, int64_t Ho, int64_t Wo) {
    WgradPlan t{};
    t.ok = d->stride == 1 && d->Kh <= 4 && d->Kw <= 4 && Wo >= 32 && d->N > 0 && d->C <= INT32_MAX &&
           d->Cout <= INT32_MAX;
    t.Wp = round_up(Wo, 64);
    t.cbw = (int32_t)((128 / d->Kh) / 16 * 16);
    t.per_image = round_up(d->Kw * d->C * d->H * t.Wp * 2, 256) + round_up(d->Cout * Ho * t.Wp * 2, 256);
    const int64_t budget = stage_budget(int64_t(3) << 29);  // 1.5 GiB of staged operands per pass
    int64_t n = budget / (t.per_image > 0 ? t.per_image : 1);
    if (n < 1) n = 1;
    if (n > d->N) n = d->N > 0 ? d->N : 1;
    if (d->N > 0) n = (d->N + (d->N + n - 1) / n - 1) / ((d->N + n - 1) / n);  // equal-sized passes
    t.nchunk = n;
    return t;
}

// Operands staged by the caller for all d->N images: the shifted copies of x (pitch pl.Wp) and one
// unshifted fp16 copy of dY with its own pitch.
struct WgradStaged {
    const __half* xs;
    const __half* dy16;
    int64_t dy_wp;
};

template <class Cfg>
static int run_wgrad_tma_cfg(const nzb_conv_desc* d, const WgradPlan& pl, const float* x, const float* dy, float* dw,
                             void* ws, int64_t Ho, int64_t Wo, const DeviceState& ds, cudaStream_t stream,
                             const WgradStaged* st = nullptr) {
    EncodeTiledFn enc;
    int rc = get_encode_tiled(&enc);
    if (rc != NZB_OK) return rc;
    static std::atomic<uint64_t> smem_set{0};  // per kernel instantiation, one bit per device
    {
        const int rc_attr = ensure_dynamic_smem(smem_set, reinterpret_cast<const void*>(conv2d_wgrad_tma_kernel<Cfg>), Cfg::SMEM_BYTES);
        if (rc_attr != NZB_OK) return rc_attr;
    }
    WgradParams p{};
    p.dW = dw;
    p.C = (int32_t)d->C; p.Cout = (int32_t)d->Cout; p.Kh = (int32_t)d->Kh; p.Kw = (int32_t)d->Kw; p.pad = (int32_t)d->pad;
    p.Ho = (int32_t)Ho; p.segs = (int32_t)((Wo + 127) / 128);
    p.cbw = pl.cbw;
    p.cblks = (int32_t)((d->C + pl.cbw - 1) / pl.cbw);
    p.tiles_n = (int32_t)((d->Cout + Cfg::BN - 1) / Cfg::BN);
    p.tiles = p.Kw * p.cblks * p.tiles_n;
    p.w_per_sample = d->weights_per_sample ? 1 : 0;
    p.stage_tx = (uint32_t)(2 * 64 * d->Kh * pl.cbw * 2 + 2 * 64 * Cfg::BN * 2);
    p.status = ds.status_dev;
    const int64_t chunk = st ? d->N : pl.nchunk;
    for (int64_t img0 = 0; img0 < d->N; img0 += chunk) {
        const int64_t n = d->N - img0 < chunk ? d->N - img0 : chunk;
        __half* XS = st ? const_cast<__half*>(st->xs) : reinterpret_cast<__half*>(ws);
        __half* DY = st ? const_cast<__half*>(st->dy16)
                        : reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(ws) + round_up(d->Kw * n * d->C * d->H * pl.Wp * 2, 256));
        const int64_t dy_wp = st ? st->dy_wp : pl.Wp;
        if (!st) {
            const int64_t rows = n * d->C * d->H;
            int64_t blocks = (rows * (pl.Wp / 8) + 255) / 256;
            if (blocks > (int64_t)ds.sm_count * 32) blocks = (int64_t)ds.sm_count * 32;
            const float* src = x + img0 * d->C * d->H * d->W;
            switch (d->Kw) {
                case 1: shift_copies_kernel<1><<<(unsigned)blocks, 256, 0, stream>>>(XS, src, rows, (int)d->W, (int)pl.Wp, (int)d->pad); break;
                case 2: shift_copies_kernel<2><<<(unsigned)blocks, 256, 0, stream>>>(XS, src, rows, (int)d->W, (int)pl.Wp, (int)d->pad); break;
                case 3: shift_copies_kernel<3><<<(unsigned)blocks, 256, 0, stream>>>(XS, src, rows, (int)d->W, (int)pl.Wp, (int)d->pad); break;
                default: shift_copies_kernel<4><<<(unsigned)blocks, 256, 0, stream>>>(XS, src, rows, (int)d->W, (int)pl.Wp, (int)d->pad); break;
            }
            NZB_CUDA_TRY(cudaGetLastError());
            // dY as one unshifted copy: columns [Wo, Wp) become zeros
            const int64_t rows2 = n * d->Cout * Ho;
            int64_t blocks2 = (rows2 * (pl.Wp / 8) + 255) / 256;
            if (blocks2 > (int64_t)ds.sm_count * 32) blocks2 = (int64_t)ds.sm_count * 32;
            shift_copies_kernel<1><<<(unsigned)blocks2, 256, 0, stream>>>(DY, dy + img0 * d->Cout * Ho * Wo, rows2, (int)Wo,
                                                                          (int)pl.Wp, 0);
            NZB_CUDA_TRY(cudaGetLastError());
        }
        CUtensorMap tmX, tmDY;
        {
            const cuuint64_t row_b = (cuuint64_t)pl.Wp * 2;
            cuuint64_t dims[5] = {(cuuint64_t)pl.Wp, (cuuint64_t)d->H, (cuuint64_t)d->C, (cuuint64_t)n, (cuuint64_t)d->Kw};
            cuuint64_t strides[4] = {row_b, row_b * d->H, row_b * d->H * d->C, row_b * d->H * d->C * n};
            cuuint32_t box[5] = {64, (cuuint32_t)d->Kh, (cuuint32_t)pl.cbw, 1, 1};
            cuuint32_t estr[5] = {1, 1, 1, 1, 1};
            CUresult cr = enc(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, XS, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (cr != CUDA_SUCCESS) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled (shifted copies) failed with CUresult %d", (int)cr);
            const cuuint64_t row_b2 = (cuuint64_t)dy_wp * 2;
            cuuint64_t dims2[4] = {(cuuint64_t)dy_wp, (cuuint64_t)Ho, (cuuint64_t)d->Cout, (cuuint64_t)n};
            cuuint64_t strides2[3] = {row_b2, row_b2 * Ho, row_b2 * Ho * d->Cout};
            cuuint32_t box2[4] = {64, 1, (cuuint32_t)Cfg::BN, 1};
            cuuint32_t estr2[4] = {1, 1, 1, 1};
            cr = enc(&tmDY, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, DY, dims2, strides2, box2, estr2,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (cr != CUDA_SUCCESS) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled (dY copy) failed with CUresult %d", (int)cr);
        }
        p.img0 = (int32_t)img0;
        p.groups = p.w_per_sample ? (int32_t)n : 1;
        p.imgs_per_group = p.w_per_sample ? 1 : (int32_t)n;
        p.kb_per_group = (int64_t)p.imgs_per_group * Ho * p.segs;
        if (p.kb_per_group > INT32_MAX) return fail(NZB_ERR_UNSUPPORTED, "contraction length exceeds 2^31 blocks");
        int64_t splits = (int64_t)ds.sm_count * Cfg::MIN_BLOCKS / ((int64_t)p.tiles * p.groups);
        if (splits < 1) splits = 1;
        if (splits > p.kb_per_group) splits = p.kb_per_group;
        p.splits = (int32_t)splits;
        p.total_items = (int64_t)p.tiles * p.groups * p.splits;
        if (p.total_items > INT32_MAX) return fail(NZB_ERR_UNSUPPORTED, "more than 2^31 work items");
        const int64_t cap = (int64_t)ds.sm_count * Cfg::MIN_BLOCKS;
        const int64_t grid = p.total_items < cap ? p.total_items : cap;
        conv2d_wgrad_tma_kernel<Cfg><<<(unsigned)grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tmX, tmDY, p);
        NZB_CUDA_TRY(cudaGetLastError());
    }
    return NZB_OK;
}

static int run_wgrad_tma(const nzb_conv_desc* d, const WgradPlan& pl, const float* x, const float* dy, float* dw, void* ws,
                         int64_t Ho, int64_t Wo, cudaStream_t stream, const WgradStaged* st = nullptr) {
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    if (d->Cout > 64) return run_wgrad_tma_cfg<WgradCfg<128, 3>>(d, pl, x, dy, dw, ws, Ho, Wo, *ds, stream, st);
    if (d->Cout > 32) return run_wgrad_tma_cfg<WgradCfg<64, 4>>(d, pl, x, dy, dw, ws, Ho, Wo, *ds, stream, st);
    if (d->Cout > 16) return run_wgrad_tma_cfg<WgradCfg<32, 5>>(d, pl, x, dy, dw, ws, Ho, Wo, *ds, stream, st);
    return run_wgrad_tma_cfg<WgradCfg<16, 3, 2>>(d, pl, x, dy, dw, ws, Ho, Wo, *ds, stream, st);
}

// ---- whole backward of one layer on shared staging ------------------------------------------------
// Weight gradient from ONE unshifted fp16 copy of x (pitch x_wp, a multiple of 64 covering the input width)
// and the Kw = 3 shifted copies of dY the data gradient uses (pitch dy_wp), for d->N images.
template <class Cfg>
static int run_wgrad_stacked_cfg(const nzb_conv_desc* d, const __half* x16, int64_t x_wp, const __half* dys, int64_t dy_wp,
                                 float* dw, int64_t Ho, int32_t img0, const DeviceState& ds, cudaStream_t stream) {
    EncodeTiledFn enc;
    int rc = get_encode_tiled(&enc);
    if (rc != NZB_OK) return rc;
    static std::atomic<uint64_t> smem_set{0};
    {
        const int rc_attr = ensure_dynamic_smem(smem_set, reinterpret_cast<const void*>(conv2d_wgrad_stacked_kernel<Cfg>), Cfg::SMEM_BYTES);
        if (rc_attr != NZB_OK) return rc_attr;
    }
    const int64_t n = d->N;
    WgradParams p{};
    p.dW = dw;
    p.C = (int32_t)d->C; p.Cout = (int32_t)d->Cout; p.Kh = (int32_t)d->Kh; p.Kw = (int32_t)d->Kw; p.pad = (int32_t)d->pad;
    p.Ho = (int32_t)Ho; p.segs = (int32_t)((d->W + 127) / 128);
    p.cbw = 16;
    p.cblks = (int32_t)((d->C + 15) / 16);
    p.tiles_n = (int32_t)((d->Cout + Cfg::BN - 1) / Cfg::BN);
    p.tiles = p.cblks * p.tiles_n;
    p.w_per_sample = d->weights_per_sample ? 1 : 0;
    p.stage_tx = (uint32_t)(2 * 64 * d->Kh * 16 * 2 + 2 * Cfg::B_HALF);
    p.status = ds.status_dev;
    CUtensorMap tmX, tmDY;
    {
        const cuuint64_t row_b = (cuuint64_t)x_wp * 2;
        cuuint64_t dims[4] = {(cuuint64_t)x_wp, (cuuint64_t)d->H, (cuuint64_t)d->C, (cuuint64_t)n};
        cuuint64_t strides[3] = {row_b, row_b * d->H, row_b * d->H * d->C};
        cuuint32_t box[4] = {64, (cuuint32_t)d->Kh, 16, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        CUresult cr = enc(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<__half*>(x16), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled (x copy) failed with CUresult %d", (int)cr);
        const cuuint64_t row_b2 = (cuuint64_t)dy_wp * 2;
        cuuint64_t dims2[5] = {(cuuint64_t)dy_wp, (cuuint64_t)Ho, (cuuint64_t)d->Cout, (cuuint64_t)n, (cuuint64_t)d->Kw};
        cuuint64_t strides2[4] = {row_b2, row_b2 * Ho, row_b2 * Ho * d->Cout, row_b2 * Ho * d->Cout * n};
        cuuint32_t box2[5] = {64, 1, (cuuint32_t)Cfg::BN, 1, (cuuint32_t)Cfg::NS};
        cuuint32_t estr2[5] = {1, 1, 1, 1, 1};
        cr = enc(&tmDY, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<__half*>(dys), dims2, strides2, box2, estr2,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled (dY copies) failed with CUresult %d", (int)cr);
    }
    p.img0 = img0;
    p.groups = p.w_per_sample ? (int32_t)n : 1;
    p.imgs_per_group = p.w_per_sample ? 1 : (int32_t)n;
    p.kb_per_group = (int64_t)p.imgs_per_group * Ho * p.segs;
    if (p.kb_per_group > INT32_MAX) return fail(NZB_ERR_UNSUPPORTED, "contraction length exceeds 2^31 blocks");
    int64_t splits = (int64_t)ds.sm_count * Cfg::MIN_BLOCKS / ((int64_t)p.tiles * p.groups);
    if (splits < 1) splits = 1;
    if (splits > p.kb_per_group) splits = p.kb_per_group;
    p.splits = (int32_t)splits;
    p.total_items = (int64_t)p.tiles * p.groups * p.splits;
    if (p.total_items > INT32_MAX) return fail(NZB_ERR_UNSUPPORTED, "more than 2^31 work items");
    const int64_t cap = (int64_t)ds.sm_count * Cfg::MIN_BLOCKS;
    const int64_t grid = p.total_items < cap ? p.total_items : cap;
    conv2d_wgrad_stacked_kernel<Cfg><<<(unsigned)grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tmX, tmDY, p);
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}

// The stacked form pays where instructions are narrow: three tap columns, at most 64 output channels.
static bool wgrad_stacked_ok(const nzb_conv_desc* d) {
    static const bool enabled = [] {
        const char* e = getenv("NZB_WGRAD_STACKED");
        return !(e && e[0] == '0');
    }();
    return enabled && d->Kw == 3 && d->Kh <= 4 && d->Cout <= 64 && d->stride == 1;
}

static int run_wgrad_stacked(const nzb_conv_desc* d, const __half* x16, int64_t x_wp, const __half* dys, int64_t dy_wp,
                             float* dw, int64_t Ho, int32_t img0, cudaStream_t stream) {
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    if (d->Cout > 32) return run_wgrad_stacked_cfg<WgradStackCfg<64, 3, 1>>(d, x16, x_wp, dys, dy_wp, dw, Ho, img0, *ds, stream);
    if (d->Cout > 16) return run_wgrad_stacked_cfg<WgradStackCfg<32, 4, 1>>(d, x16, x_wp, dys, dy_wp, dw, Ho, img0, *ds, stream);
    return run_wgrad_stacked_cfg<WgradStackCfg<16, 3, 2>>(d, x16, x_wp, dys, dy_wp, dw, Ho, img0, *ds, stream);
}

struct BackwardPlan {
    bool ok;
    TmaPlan dx;      // data-gradient plan for one chunk (N = nchunk)
    WgradPlan wg;
    int64_t wp_dy;   // pitch of the dY copies (= the data-gradient kernel's input pitch)
    int64_t x_bytes, dy_bytes;  // per image
    int64_t nchunk;
    int64_t total;
};
static BackwardPlan backward_plan(const nzb_conv_desc* d, int64_t Ho, int64_t Wo) {
    BackwardPlan b{};
    const int64_t wN1 = d->weights_per_sample ? 1 : 0;
    b.wg = wgrad_plan(d, Ho, Wo);
    b.ok = b.wg.ok && d->Kh == d->Kw && d->pad <= d->Kh - 1 && d->W >= 32 &&
           (d->bias_mode == NZB_BIAS_MATRIX || d->bias_mode == NZB_BIAS_NONE);
    // wide enough for the data gradient's rows (W) and for every column of dY itself (Wo > W when pad > (K-1)/2:
    // the bias gradient and the unshifted copy need them all)
    b.wp_dy = round_up(d->W > Wo ? d->W : Wo, 64);
    b.x_bytes = round_up(d->Kw * d->C * d->H * b.wg.Wp * 2, 256);
    b.dy_bytes = round_up(d->Kw * d->Cout * Ho * b.wp_dy * 2, 256);
    const int64_t budget = stage_budget(int64_t(3) << 29);
    int64_t n = budget / (b.x_bytes + b.dy_bytes);
    if (n < 1) n = 1;
    if (n > d->N) n = d->N > 0 ? d->N : 1;
    if (d->N > 0) n = (d->N + (d->N + n - 1) / n - 1) / ((d->N + n - 1) / n);
    b.nchunk = n;
    b.dx = tma_plan(n, d->Cout, Ho, Wo, d->C, d->Kh, d->Kw, d->stride, d->H, d->W, wN1 ? n : 1);
    b.dx.Wp = b.wp_dy;
    b.ok = b.ok && b.dx.ok;
    b.total = b.dx.w_bytes + n * (b.x_bytes + b.dy_bytes);
    return b;
}

static int check_conv_desc(const nzb_conv_desc* d, int64_t* Ho, int64_t* Wo) {
    if (!d) return fail(NZB_ERR_BAD_ARG, "descriptor is null");
    if (d->N < 0 || d->C < 1 || d->H < 1 || d->W < 1 || d->Cout < 1 || d->Kh < 1 || d->Kw < 1 || d->stride < 1 ||
        d->pad < 0)
        return fail(NZB_ERR_BAD_ARG, "bad convolution extent");
    if (d->H + 2 * d->pad < d->Kh || d->W + 2 * d->pad < d->Kw) return fail(NZB_ERR_BAD_ARG, "kernel larger than the padded input");
    if (d->bias_mode != NZB_BIAS_NONE && d->bias_mode != NZB_BIAS_ROW && d->bias_mode != NZB_BIAS_MATRIX)
        return fail(NZB_ERR_BAD_ARG, "bias_mode must be NONE, ROW ([Cout]) or MATRIX ([Ho*Wo][Cout])");
    *Ho = (d->H + 2 * d->pad - d->Kh) / d->stride + 1;
    *Wo = (d->W + 2 * d->pad - d->Kw) / d->stride + 1;
    return NZB_OK;
}

// Images per weight-gradient chunk and the staging bytes that chunk needs.
static int64_t weight_grad_stage_bytes(const nzb_conv_desc* d, int64_t HoWo, int64_t* nb_out) {
    const int64_t K = d->C * d->Kh * d->Kw;
    const int64_t per_image = (K + d->Cout) * round_up(HoWo, 64) * 2;
    const int64_t budget = stage_budget(int64_t(2) << 30);
    int64_t nb = 1;
    if (!d->weights_per_sample && d->N > 1) {
        int64_t nb_max = budget / (per_image > 0 ? per_image : 1);
        if (nb_max < 1) nb_max = 1;
        const int64_t chunks = (d->N + nb_max - 1) / nb_max;
        nb = (d->N + chunks - 1) / chunks;
    }
    if (nb_out) *nb_out = nb;
    const int64_t Qp = round_up(nb * HoWo, 64);
    return round_up(K * Qp * 2, 256) + round_up(d->Cout * Qp * 2, 256);
}

}  // namespace nzb

using namespace nzb;

extern "C" {

int nzb_conv2d_workspace_bytes(const nzb_conv_desc* d, size_t* bytes_out) {
    if (!bytes_out) return fail(NZB_ERR_BAD_ARG, "bytes_out is null");
    int64_t Ho, Wo;
    int rc = check_conv_desc(d, &Ho, &Wo);
    if (rc != NZB_OK) return rc;
    const int64_t wN = d->weights_per_sample ? d->N : 1;
    const int64_t Kf = round_up(d->C * d->Kh * d->Kw, kOperandKAlign);      // forward: [Cout][Kf]
    const int64_t Kb = round_up(d->Cout * d->Kh * d->Kw, kOperandKAlign);   // backward data: [C][Kb]
    const int64_t f = wN * d->Cout * Kf * 2, b = wN * d->C * Kb * 2;
    const int64_t g = weight_grad_stage_bytes(d, Ho * Wo, nullptr);
    int64_t m = f > b ? f : b;
    if (g > m) m = g;
    // TMA im2col mode: staged weights + the shifted fp16 copies of a chunk of images
    const TmaPlan tf = tma_plan(d->N, d->C, d->H, d->W, d->Cout, d->Kh, d->Kw, d->stride, Ho, Wo, wN);
    const NhwcPlan nf = nhwc_plan(d->N, d->C, d->H, d->W, d->Cout, d->Kh, d->Kw, d->stride, Ho, Wo, wN);
    if (nf.ok && nf.w_bytes + nf.nchunk * nf.per_image + nf.bias_bytes > m) m = nf.w_bytes + nf.nchunk * nf.per_image + nf.bias_bytes;
    // (+ the forward's transposed copy of the {Ho*Wo, Cout} bias matrix)
    const int64_t bias_t_bytes = round_up(Ho * Wo * d->Cout * 4, 256);
    if (tf.ok && tf.w_bytes + tf.nchunk * tf.per_image + bias_t_bytes > m) m = tf.w_bytes + tf.nchunk * tf.per_image + bias_t_bytes;
    const TmaPlan tb = tma_plan(d->N, d->Cout, Ho, Wo, d->C, d->Kh, d->Kw, d->stride, d->H, d->W, wN);
    if (tb.ok && tb.w_bytes + tb.nchunk * tb.per_image > m) m = tb.w_bytes + tb.nchunk * tb.per_image;
    const WgradPlan tg = wgrad_plan(d, Ho, Wo);
    if (tg.ok && tg.nchunk * tg.per_image > m) m = tg.nchunk * tg.per_image;
    *bytes_out = (size_t)round_up(m, 256);
    return NZB_OK;
}

int nzb_conv2d_forward(const nzb_conv_desc* d, const float* x, const float* w, const float* bias, float* y,
                       void* workspace, size_t workspace_bytes, void* stream) {
    int64_t Ho, Wo;
    int rc = check_conv_desc(d, &Ho, &Wo);
    if (rc != NZB_OK) return rc;
    if (d->N == 0) return NZB_OK;
    if (!x || !w || !y) return fail(NZB_ERR_BAD_ARG, "x, w and y must be non-null");
    if (d->bias_mode != NZB_BIAS_NONE && !bias) return fail(NZB_ERR_BAD_ARG, "bias_mode set but bias is null");
    size_t need;
    nzb_conv2d_workspace_bytes(d, &need);
    if (!workspace || workspace_bytes < need) return fail(NZB_ERR_WORKSPACE, "workspace of %zu bytes needed", need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(NZB_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t wN = d->weights_per_sample ? d->N : 1;
    {
        const NhwcPlan np = nhwc_plan(d->N, d->C, d->H, d->W, d->Cout, d->Kh, d->Kw, d->stride, Ho, Wo, wN);
        if (np.ok) {
            ConvNhwcRun r{x, y, bias, w, d->N, d->C, d->H, d->W, d->Cout, d->Kh, d->Kw, d->pad, Ho, Wo, d->C, d->Cout,
                          d->bias_mode, d->accumulate ? 1 : 0, d->relu ? 1 : 0, 0};
            return run_conv_nhwc(r, np, workspace, s);
        }
    }
    {
        const TmaPlan tp = tma_plan(d->N, d->C, d->H, d->W, d->Cout, d->Kh, d->Kw, d->stride, Ho, Wo, wN);
        if (tp.ok) {
            float* bias_t = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + tp.w_bytes + tp.nchunk * tp.per_image);
            ConvTmaRun r{x, y, bias, w, d->N, d->C, d->H, d->W, d->Cout, d->Kh, d->Kw, d->pad, Ho, Wo, d->C, d->Cout,
                         d->weights_per_sample ? 1 : 0, d->bias_mode, d->accumulate ? 1 : 0, d->relu ? 1 : 0, 0, nullptr,
                         bias_t};
            return run_conv_tma(r, tp, workspace, s);
        }
    }
    const int64_t K = d->C * d->Kh * d->Kw, Kp = round_up(K, kOperandKAlign);
    __half* W16 = reinterpret_cast<__half*>(workspace);
    // w is {wN, 1, K, Cout} row-major: stage as [wN][Cout][Kp] (transpose + round)
    rc = launch_cast(w, W16, d->Cout, K, d->Cout, Kp, 1, wN, 1, K * d->Cout, 0, s);
    if (rc != NZB_OK) return rc;
    ConvRun r{x, y, bias, d->N, d->C, d->H, d->W, d->Cout, d->Kh, d->Kw, d->stride, d->pad, Ho, Wo,
              d->weights_per_sample ? 1 : 0, d->bias_mode, d->accumulate ? 1 : 0, d->relu ? 1 : 0};
    return run_conv(r, W16, Kp, wN, s);
}

int nzb_conv2d_backward_data(const nzb_conv_desc* d, const float* dy, const float* w, float* dx, void* workspace,
                             size_t workspace_bytes, void* stream) {
    int64_t Ho, Wo;
    int rc = check_conv_desc(d, &Ho, &Wo);
    if (rc != NZB_OK) return rc;
    if (d->N == 0) return NZB_OK;
    if (!dy || !w || !dx) return fail(NZB_ERR_BAD_ARG, "dy, w and dx must be non-null");
    if (d->stride != 1) return fail(NZB_ERR_UNSUPPORTED, "the fused backward-data kernel handles stride 1; use nzb_gemm_backward + nzb_img2col_backward for other strides");
    if (d->Kh - 1 - d->pad < 0 || d->Kw - 1 - d->pad < 0) return fail(NZB_ERR_UNSUPPORTED, "pad larger than kernel - 1");
    if (d->Kh != d->Kw) return fail(NZB_ERR_UNSUPPORTED, "the fused backward-data kernel needs a square kernel (one pad value)");
    size_t need;
    nzb_conv2d_workspace_bytes(d, &need);
    if (!workspace || workspace_bytes < need) return fail(NZB_ERR_WORKSPACE, "workspace of %zu bytes needed", need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(NZB_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    DeviceState* ds;
    rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t wN = d->weights_per_sample ? d->N : 1;
    {
        // dX {N, C, H, W} += conv(dY {N, Cout, Ho, Wo}, flipped weights, pad' = Kh - 1 - pad, stride 1)
        const TmaPlan tp = tma_plan(d->N, d->Cout, Ho, Wo, d->C, d->Kh, d->Kw, d->stride, d->H, d->W, wN);
        if (tp.ok) {
            ConvTmaRun r{dy, dx, nullptr, w, d->N, d->Cout, Ho, Wo, d->C, d->Kh, d->Kw, d->Kh - 1 - d->pad, d->H, d->W,
                         d->C, d->Cout, d->weights_per_sample ? 1 : 0, NZB_BIAS_NONE, d->overwrite_dx ? 0 : 1, 0, 1, nullptr};
            return run_conv_tma(r, tp, workspace, s);
        }
    }
    const int64_t K2 = d->Cout * d->Kh * d->Kw, Kp2 = round_up(K2, kOperandKAlign);
    __half* W16 = reinterpret_cast<__half*>(workspace);
    {
        const int64_t total = wN * d->C * Kp2;
        int64_t blocks = (total + 255) / 256;
        if (blocks > (int64_t)ds->sm_count * 16) blocks = (int64_t)ds->sm_count * 16;
        flip_weights_kernel<<<(unsigned)blocks, 256, 0, s>>>(W16, w, d->C, d->Cout, d->Kh, d->Kw, Kp2, wN);
        NZB_CUDA_TRY(cudaGetLastError());
    }
    // dX {N, C, H, W} += conv(dY {N, Cout, Ho, Wo}, flipped weights, pad' = Kh - 1 - pad, stride 1)
    ConvRun r{dy, dx, nullptr, d->N, d->Cout, Ho, Wo, d->C, d->Kh, d->Kw, 1, d->Kh - 1 - d->pad, d->H, d->W,
              d->weights_per_sample ? 1 : 0, NZB_BIAS_NONE, d->overwrite_dx ? 0 : 1, 0};
    return run_conv(r, W16, Kp2, wN, s);
}

int nzb_conv2d_backward_weight(const nzb_conv_desc* d, const float* x, const float* dy, float* dw, void* workspace,
                               size_t workspace_bytes, void* stream) {
    int64_t Ho, Wo;
    int rc = check_conv_desc(d, &Ho, &Wo);
    if (rc != NZB_OK) return rc;
    if (d->N == 0) return NZB_OK;
    if (!x || !dy || !dw) return fail(NZB_ERR_BAD_ARG, "x, dy and dw must be non-null");
    size_t need;
    nzb_conv2d_workspace_bytes(d, &need);
    if (!workspace || workspace_bytes < need) return fail(NZB_ERR_WORKSPACE, "workspace of %zu bytes needed", need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(NZB_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    DeviceState* ds;
    rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    {
        const WgradPlan tg = wgrad_plan(d, Ho, Wo);
        if (tg.ok) return run_wgrad_tma(d, tg, x, dy, dw, workspace, Ho, Wo, s);
    }
    const int64_t HoWo = Ho * Wo, K = d->C * d->Kh * d->Kw;
    int64_t nb;
    weight_grad_stage_bytes(d, HoWo, &nb);
    if (nb * HoWo > INT32_MAX - 256) return fail(NZB_ERR_UNSUPPORTED, "contraction length exceeds 2^31");
    for (int64_t b0 = 0; b0 < d->N; b0 += nb) {
        const int64_t n = (d->N - b0 < nb) ? d->N - b0 : nb;
        const int64_t Q = n * HoWo, Qp = round_up(Q, 64);
        __half* colT = reinterpret_cast<__half*>(workspace);
        __half* dyT = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(workspace) + round_up(K * Qp * 2, 256));
        // grid.x covers the contraction in units of 8 per thread, grid.y = the row (k or channel)
        int64_t gx = (Q / 8 + 255) / 256;
        const int64_t capx = ((int64_t)ds->sm_count * 32 + K - 1) / K;
        if (gx > capx) gx = capx;
        if (gx < 1) gx = 1;
        if (K > 65535 || d->Cout > 65535) return fail(NZB_ERR_UNSUPPORTED, "more than 65535 weight rows or channels");
        im2col_f16_kmajor_kernel<<<dim3((unsigned)gx, (unsigned)K), 256, 0, s>>>(
            colT, x, (int)d->C, (int)d->H, (int)d->W, (int)d->Kh, (int)d->Kw, (int)d->stride, (int)d->pad, (int)Ho,
            (int)Wo, b0, (int)n, (int)K, Qp);
        NZB_CUDA_TRY(cudaGetLastError());
        int64_t gx2 = (Q / 8 + 255) / 256;
        const int64_t capx2 = ((int64_t)ds->sm_count * 32 + d->Cout - 1) / d->Cout;
        if (gx2 > capx2) gx2 = capx2;
        if (gx2 < 1) gx2 = 1;
        dy_f16_kmajor_kernel<<<dim3((unsigned)gx2, (unsigned)d->Cout), 256, 0, s>>>(dyT, dy, (int)d->Cout, (int)HoWo, b0,
                                                                                   (int)n, Qp);
        NZB_CUDA_TRY(cudaGetLastError());
        GemmLaunch g{};
        g.A16 = colT; g.B16 = dyT; g.nA = 1; g.nB = 1;
        g.M = K; g.N = d->Cout; g.K = Q; g.Kp = Qp;
        g.C = dw + (d->weights_per_sample ? b0 * K * d->Cout : 0);
        g.ldc = d->Cout;
        g.out_e[0] = g.out_e[1] = 1; g.red_e[0] = g.red_e[1] = 1;
        g.accumulate = 1;
        rc = launch_gemm(g, s);
        if (rc != NZB_OK) return rc;
    }
    return NZB_OK;
}

int nzb_conv2d_backward_workspace_bytes(const nzb_conv_desc* d, size_t* bytes_out) {
    if (!bytes_out) return fail(NZB_ERR_BAD_ARG, "bytes_out is null");
    int64_t Ho, Wo;
    int rc = check_conv_desc(d, &Ho, &Wo);
    if (rc != NZB_OK) return rc;
    const BackwardPlan b = backward_plan(d, Ho, Wo);
    if (!b.ok) return fail(NZB_ERR_UNSUPPORTED, "the one-pass backward needs stride 1, a square kernel of at most 4x4, pad <= K-1, rows of 32+ pixels and a matrix (or no) bias gradient; use the separate backward calls");
    *bytes_out = (size_t)round_up(b.total, 256);
    return NZB_OK;
}

int nzb_conv2d_backward(const nzb_conv_desc* d, const float* x, const float* w, const float* y, const float* dy,
                        float* dx, float* dw, float* dbias, void* workspace, size_t workspace_bytes, void* stream) {
    int64_t Ho, Wo;
    int rc = check_conv_desc(d, &Ho, &Wo);
    if (rc != NZB_OK) return rc;
    if (d->N == 0) return NZB_OK;
    if (!dy) return fail(NZB_ERR_BAD_ARG, "dy must be non-null");
    if ((dx && !w) || (dw && !x)) return fail(NZB_ERR_BAD_ARG, "dx needs w and dw needs x");
    if (d->relu && !y) return fail(NZB_ERR_BAD_ARG, "the ReLU mask needs the forward output y");
    if (dbias && d->bias_mode != NZB_BIAS_MATRIX) return fail(NZB_ERR_UNSUPPORTED, "the one-pass backward writes the {Ho*Wo, Cout} bias gradient; bias_mode must be NZB_BIAS_MATRIX");
    const BackwardPlan b = backward_plan(d, Ho, Wo);
    if (!b.ok) return fail(NZB_ERR_UNSUPPORTED, "shape not handled by the one-pass backward; use the separate backward calls");
    if (!workspace || workspace_bytes < (size_t)b.total) return fail(NZB_ERR_WORKSPACE, "workspace of %lld bytes needed", (long long)b.total);
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(NZB_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    DeviceState* ds;
    rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
    const int64_t K = d->C * d->Kh * d->Kw, padb = d->Kh - 1 - d->pad;
    for (int64_t img0 = 0; img0 < d->N; img0 += b.nchunk) {
        const int64_t n = d->N - img0 < b.nchunk ? d->N - img0 : b.nchunk;
        __half* XSdy = reinterpret_cast<__half*>(base + b.dx.w_bytes);
        __half* XSx = reinterpret_cast<__half*>(base + b.dx.w_bytes + n * b.dy_bytes);
        const float* dy_c = dy + img0 * d->Cout * Ho * Wo;
        const float* y_c = (d->relu && y) ? y + img0 * d->Cout * Ho * Wo : nullptr;
        const float* x_c = x ? x + img0 * d->C * d->H * d->W : nullptr;
        const float* w_c = (w && d->weights_per_sample) ? w + img0 * K * d->Cout : w;
        {
            // one pass over dY: mask, the Kw shifted copies, bias gradient
            // without a data gradient only the unshifted copy is needed, unless the weight gradient takes all of them
            const int only_kw = (dx || (dw && wgrad_stacked_ok(d))) ? -1 : (int)padb;
            const bool narrow = d->Cout <= 16;
            const int64_t blocks_all = narrow ? ((d->Cout + 15) / 16) * Ho * ((b.wp_dy + 127) / 128)
                                              : ((d->Cout + 31) / 32) * Ho * (b.wp_dy / 64);
            const int64_t blocks = blocks_all < (int64_t)ds->sm_count * 16 ? blocks_all : (int64_t)ds->sm_count * 16;
#define NZB_DY_PREPARE(KW)                                                                                          \
    if (narrow)                                                                                                     \
        dy_prepare_kernel<KW, 16><<<(unsigned)blocks, 256, 0, s>>>(XSdy, dy_c, y_c, dbias, (int)n, (int)d->Cout,      \
                                                                   (int)Ho, (int)Wo, (int)b.wp_dy, (int)padb, only_kw); \
    else                                                                                                            \
        dy_prepare_kernel<KW, 32><<<(unsigned)blocks, 256, 0, s>>>(XSdy, dy_c, y_c, dbias, (int)n, (int)d->Cout,      \
                                                                   (int)Ho, (int)Wo, (int)b.wp_dy, (int)padb, only_kw)
            switch (d->Kw) {
                case 1: NZB_DY_PREPARE(1); break;
                case 2: NZB_DY_PREPARE(2); break;
                case 3: NZB_DY_PREPARE(3); break;
                default: NZB_DY_PREPARE(4); break;
            }
#undef NZB_DY_PREPARE
            NZB_CUDA_TRY(cudaGetLastError());
        }
        nzb_conv_desc dc = *d;
        dc.N = n;
        if (dw && wgrad_stacked_ok(d)) {
            // one unshifted copy of x over its whole width; the tap shifts are in the dY copies
            const int64_t rows = n * d->C * d->H, x_wp = round_up(d->W, 64);
            int64_t blocks = (rows * (x_wp / 8) + 255) / 256;
            if (blocks > (int64_t)ds->sm_count * 32) blocks = (int64_t)ds->sm_count * 32;
            shift_copies_kernel<1><<<(unsigned)blocks, 256, 0, s>>>(XSx, x_c, rows, (int)d->W, (int)x_wp, 0);
            NZB_CUDA_TRY(cudaGetLastError());
            float* dw_c = dw + (d->weights_per_sample ? img0 * K * d->Cout : 0);
            rc = run_wgrad_stacked(&dc, XSx, x_wp, XSdy, b.wp_dy, dw_c, Ho, (int32_t)0, s);
            if (rc != NZB_OK) return rc;
        } else if (dw) {
            const int64_t rows = n * d->C * d->H;
            int64_t blocks = (rows * (b.wg.Wp / 8) + 255) / 256;
            if (blocks > (int64_t)ds->sm_count * 32) blocks = (int64_t)ds->sm_count * 32;
            switch (d->Kw) {
                case 1: shift_copies_kernel<1><<<(unsigned)blocks, 256, 0, s>>>(XSx, x_c, rows, (int)d->W, (int)b.wg.Wp, (int)d->pad); break;
                case 2: shift_copies_kernel<2><<<(unsigned)blocks, 256, 0, s>>>(XSx, x_c, rows, (int)d->W, (int)b.wg.Wp, (int)d->pad); break;
                case 3: shift_copies_kernel<3><<<(unsigned)blocks, 256, 0, s>>>(XSx, x_c, rows, (int)d->W, (int)b.wg.Wp, (int)d->pad); break;
                default: shift_copies_kernel<4><<<(unsigned)blocks, 256, 0, s>>>(XSx, x_c, rows, (int)d->W, (int)b.wg.Wp, (int)d->pad); break;
            }
            NZB_CUDA_TRY(cudaGetLastError());
            // copy number padb of the dY copies is the unshifted one
            WgradStaged st{XSx, XSdy + padb * (n * d->Cout * Ho * b.wp_dy), b.wp_dy};
            float* dw_c = dw + (d->weights_per_sample ? img0 * K * d->Cout : 0);
            rc = run_wgrad_tma(&dc, b.wg, x_c, dy_c, dw_c, nullptr, Ho, Wo, s, &st);
            if (rc != NZB_OK) return rc;
        }
        if (dx) {
            TmaPlan pl = tma_plan(n, d->Cout, Ho, Wo, d->C, d->Kh, d->Kw, d->stride, d->H, d->W,
                                  d->weights_per_sample ? n : 1);
            pl.Wp = b.wp_dy;  // the pitch the copies were written with
            ConvTmaRun r{dy_c, dx + img0 * d->C * d->H * d->W, nullptr, w_c, n, d->Cout, Ho, Wo, d->C, d->Kh, d->Kw, padb,
                         d->H, d->W, d->C, d->Cout, d->weights_per_sample ? 1 : 0, NZB_BIAS_NONE,
                         d->overwrite_dx ? 0 : 1, 0, 1, XSdy};
            rc = run_conv_tma(r, pl, base, s);
            if (rc != NZB_OK) return rc;
        }
    }
    return NZB_OK;
}

int nzb_conv2d_backward_bias(const nzb_conv_desc* d, const float* dy, float* dbias, void* stream) {
    int64_t Ho, Wo;
    int rc = check_conv_desc(d, &Ho, &Wo);
    if (rc != NZB_OK) return rc;
    if (!dy || !dbias) return fail(NZB_ERR_BAD_ARG, "null pointer");
    DeviceState* ds;
    rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    if (d->N == 0) return NZB_OK;
    const int64_t tiles = ((Ho * Wo + 31) / 32) * ((d->Cout + 31) / 32);
    int64_t blocks = tiles < (int64_t)ds->sm_count * 16 ? tiles : (int64_t)ds->sm_count * 16;
    conv_bias_grad_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(dbias, dy, d->N, d->Cout,
                                                                                        Ho * Wo);
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}

}  // extern "C"
