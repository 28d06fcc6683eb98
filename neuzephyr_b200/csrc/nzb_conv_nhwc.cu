// Stride-1 convolution on tcgen05 from ONE channels-last fp16 copy of the input.
//
// The im2col product Y[pixel][co] = sum_{kh,kw,c} X[h+kh-pad][w+kw-pad][c] * W[kh][kw][c][co] that the
// reference builds with img2col + GEMM + col2img (src/Model.cu:244-263, src/OperationKernels.cu:1308-1335)
// is computed here without materialising any tap copy:
//
//   * the input is staged once as XH[n][h][w][c] (fp16, channels contiguous). One pixel is then one
//     K-major operand row of Cb = 16, 32 or 64 channels (32, 64 or 128 bytes: the 32/64/128-byte swizzle
//     atoms of tcgen05), and an input row segment of 136 pixels is one TMA box;
//   * a tile is 128 consecutive output pixels of one output row. Its A operand for tap (kh, kw) is the
//     box of input row ho - pad + kh, read from operand row kw onward: the horizontal shift is a shared
//     memory offset of kw rows in the operand descriptor, the vertical one picks another ring slot.
//     Horizontal and vertical padding are TMA zero fill;
//   * a CTA walks consecutive output rows of one (image, column segment), so each new tile needs ONE new
//     input row in its ring; the other Kh - 1 are still there. L2 -> SM traffic per tile is one box
//     (17 KB for 64 channels) instead of Kh * Kw tap tiles;
//   * the weights of the CTA's output-channel tile, all taps, stay resident in shared memory.
//
// CTA: warp 0 TMA, warps 1-2 MMA issue (alternate instructions of a tile, one partial accumulator each),
// then one or two groups of four epilogue warps (lanes = pixels, one coalesced 128-byte store per output
// channel, straight into NCHW fp32).
//
// What bounds it (clock64 counters of the instrumented build, -DNZB_NHWC_PROFILE): a tcgen05.mma with
// both operands in shared memory costs about 107 clocks of an SM whatever its N up to 128 (operand fetch),
// and the epilogue's global loads and stores share that data path; the 36 instructions of a 3x3, 64-channel
// tile take 3 900 clocks against 2 300 of tensor work. Converting the fp32 input inside the kernel
// (converter warps writing the swizzled rows) was measured slower than the separate staging pass for
// that reason (0.56 against 0.53 ms), and loading the bias one chunk ahead did not help either. With
// 16-channel inputs an operand row is 32 bytes and a tap is a single K = 16 instruction; the SM then retires
// one instruction per 113 clocks even at N = 16 (one per 40 with 128-byte rows), so narrow layers stay on the
// shifted-copies kernel, whose operand tiles have the pixels contiguous whatever the channel count.
#include "nzb_internal.h"
#include "nzb_ptx.cuh"

namespace nzb {

namespace {

constexpr int kBoxPixels = 136;  // 128 output pixels + up to 8 tap columns, a multiple of the 8-row swizzle atom
constexpr int kBiasMatrixT = 4;  // internal: the {Ho*Wo, Cout} bias matrix transposed to {Cout, Ho*Wo}

struct NhwcParams {
    float* Y;
    const float* bias;
    int32_t Cout, Kh, Kw, pad;
    int32_t N, Ho, Wo, HoWo;
    int32_t CB;        // channel blocks of Cb channels
    int32_t rowb;      // bytes of one operand row: Cb * 2
    int32_t ksteps;    // Cb / 16
    int32_t layout;    // tcgen05 shared-memory layout code of the swizzle (2 = 128 B, 4 = 64 B, 6 = 32 B)
    int32_t sbo;       // bytes between 8-row groups: 8 * rowb
    int32_t segs, tiles_n;
    int32_t stages;
    int32_t nsplit;    // partial accumulators per tile: 2 unless a tile is a single instruction
    uint32_t slot_bytes;  // CB * kBoxPixels * rowb
    uint32_t bblk_bytes;  // BN * rowb: one (tap, channel block) weight tile
    uint32_t b_bytes;     // Kh * Kw * CB * bblk_bytes
    int32_t bias_mode, relu;
    int32_t img0;  // first image of this pass (Y index; XH is pass-local)
    int64_t total; // tiles_n * N * segs * Ho
    int* status;
};

// tcgen05.mma from the two 32-bit halves of the operand descriptors: the high half (stride, version,
// swizzle) is the same for every operand of a launch and the low half is a 32-bit running address, so
// the issuing thread spends one integer add per operand and instruction.
template <bool ACCUM>
__device__ __forceinline__ void mma_f16_lo(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
        "}" ::"r"(tmem_d),
        "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "n"(ACCUM ? 1 : 0)
        : "memory");
}
// One (tap, channel block): KS instructions of 16 channels each, of which this thread issues those whose
// running index i0 + k has parity `me`. `fresh` is true until the thread has issued its first instruction
// of the tile, which overwrites the accumulator.
template <int KS>
__device__ __forceinline__ void mma_block(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                          uint32_t i0, uint32_t me, bool& fresh) {
#pragma unroll
    for (int k = 0; k < KS; k++) {
        if (((i0 + k) & 1u) != me) continue;
        if (fresh) mma_f16_lo<false>(d, a_lo + 2 * k, b_lo + 2 * k, hi, idesc);
        else mma_f16_lo<true>(d, a_lo + 2 * k, b_lo + 2 * k, hi, idesc);
        fresh = false;
    }
}

#ifdef NZB_NHWC_PROFILE
// [role][counter] summed over CTAs: clocks spent in each wait / phase (debug builds only)
__device__ unsigned long long g_nhwc_prof[16];
#define PROF_T0() const long long _t0 = clock64()
#define PROF_ADD(i) if (lane == 0) atomicAdd(&g_nhwc_prof[i], (unsigned long long)(clock64() - _t0))
#else
#define PROF_T0()
#define PROF_ADD(i)
#endif

struct NhwcTile {
    int32_t nt, img, wo0, npx, ho;
    int32_t col;  // (nt, img, seg): tiles of one col are consecutive output rows
};
__device__ __forceinline__ NhwcTile decode_tile(const NhwcParams& p, int64_t idx) {
    // the host keeps `total` below 2^31
    NhwcTile t;
    const uint32_t i = static_cast<uint32_t>(idx);
    const uint32_t col = i / (uint32_t)p.Ho;
    t.col = static_cast<int32_t>(col);
    t.ho = static_cast<int32_t>(i - col * (uint32_t)p.Ho);
    const uint32_t r = col / (uint32_t)p.segs;
    const int32_t seg = static_cast<int32_t>(col - r * (uint32_t)p.segs);
    const uint32_t nt = r / (uint32_t)p.N;
    t.nt = static_cast<int32_t>(nt);
    t.img = static_cast<int32_t>(r - nt * (uint32_t)p.N);
    t.wo0 = seg * 128;
    t.npx = min(128, p.Wo - t.wo0);
    return t;
}

template <int BN_>
struct NhwcCfg {
    static constexpr int BN = BN_;
    static constexpr int EPI_GROUPS = BN >= 64 ? 2 : 1;     // column halves drained by separate warp groups
    static constexpr int COLS = BN / EPI_GROUPS;            // accumulator columns per epilogue warp
    static constexpr int CHUNK = COLS < 32 ? COLS : 32;
    static constexpr int THREADS = 96 + 128 * EPI_GROUPS;  // TMA warp, two MMA warps, epilogue groups
    static constexpr int TMEM_COLS = (4 * BN < 32) ? 32 : 4 * BN;  // two tiles in flight x one partial sum per MMA warp
    static constexpr int kMaxStages = 12;
    static constexpr int BAR_BYTES = 256;
};

template <class Cfg, bool ACC>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
conv2d_nhwc_tcgen05_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                           const NhwcParams p) {
    using namespace ptx;
    constexpr int BN = Cfg::BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smB = smem;                                            // resident weights
    uint8_t* smA = smem + ((p.b_bytes + 1023u) & ~1023u);           // ring of input rows
    uint64_t* bars = reinterpret_cast<uint64_t*>(smA + (size_t)p.stages * p.slot_bytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + Cfg::kMaxStages;
    uint64_t* tfull = bars + 2 * Cfg::kMaxStages;
    uint64_t* tempty = tfull + 2;
    uint64_t* bfull = tempty + 2;
    uint64_t* bempty = bfull + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bempty + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmW);
        prefetch_tensormap(&tmX);
        for (int s = 0; s < p.stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 2);  // one arrival per MMA warp
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tfull[a], 2);
            mbar_init(&tempty[a], 4 * Cfg::EPI_GROUPS);
        }
        mbar_init(bfull, 1);
        mbar_init(bempty, 2);
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

    // this CTA's share: a contiguous run of the tile sequence, so that consecutive tiles are
    // consecutive output rows of one column segment wherever possible
    const int64_t t_begin = p.total * blockIdx.x / gridDim.x;
    const int64_t t_end = p.total * (blockIdx.x + 1) / gridDim.x;
    const uint32_t stages = (uint32_t)p.stages;
#ifdef NZB_NHWC_PROFILE
    const long long _k0 = clock64();
#endif

    if (warp == 0) {
        // ---------------- TMA: weights when the channel tile changes, one input row per new tile ----------------
        uint32_t seq = 0, bgen = 0;
        int32_t cur_nt = -1, cur_col = -1, next_row = 0;
        bool ok = true;
        for (int64_t idx = t_begin; idx < t_end && ok; idx++) {
            const NhwcTile t = decode_tile(p, idx);
            if (t.nt != cur_nt) {
                if (!mbar_wait_warp(bempty, (bgen & 1) ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    mbar_arrive_expect_tx(bfull, p.b_bytes);
                    const int32_t taps = p.Kh * p.Kw;
                    uint8_t* dst = smB;
                    for (int32_t tap = 0; tap < taps; tap++)
                        for (int32_t cb = 0; cb < p.CB; cb++, dst += p.bblk_bytes)
                            tma_load_3d(dst, &tmW, cb * (p.rowb >> 1), t.nt * BN, tap, bfull);
                }
                __syncwarp();
                bgen++;
                cur_nt = t.nt;
            }
            if (t.col != cur_col) {
                cur_col = t.col;
                next_row = t.ho - p.pad;
            }
            const int32_t last_row = t.ho - p.pad + p.Kh - 1;
            for (; next_row <= last_row; next_row++, seq++) {
                const uint32_t s = seq % stages, ph = (seq / stages) & 1;
                {
                    PROF_T0();
                    if (!mbar_wait_warp(&empty[s], ph ^ 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    PROF_ADD(0);
                }
                if (elect_one()) {
                    uint8_t* dst = smA + (size_t)s * p.slot_bytes;
                    mbar_arrive_expect_tx(&full[s], p.slot_bytes);
                    const uint32_t blk = (uint32_t)kBoxPixels * (uint32_t)p.rowb;
                    for (int32_t cb = 0; cb < p.CB; cb++)
                        tma_load_4d(dst + cb * blk, &tmX, cb * (p.rowb >> 1), t.wo0 - p.pad, next_row, t.img, &full[s]);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) {
            // give the copies in flight a bounded time to land before the CTA retires
            const long long t0 = clock64();
            const uint32_t first = seq > stages ? seq - stages : 0;
            for (uint32_t j = first; j < seq; j++)
                while (!mbar_try_wait(&full[j % stages], (j / stages) & 1))
                    if (clock64() - t0 > kWaitCycleLimit) break;
            if (bgen)
                while (!mbar_try_wait(bfull, (bgen - 1) & 1))
                    if (clock64() - t0 > kWaitCycleLimit) break;
        }
    } else if (warp <= 2) {
        // ---------------- MMA issue: Kh * Kw * CB * ksteps instructions per tile, split over two warps ----------------
        // One thread issues a tcgen05.mma about every 120 clocks whatever its N, so a single issuing warp
        // keeps the tensor pipe at most half busy with 128-column tiles. The two warps take alternate
        // instructions of the SAME tile, each summing into its own accumulator (the epilogue adds the two),
        // so the ring needs no more rows than one tile reads. Every barrier the MMA side signals counts two
        // arrivals, one commit per warp.
        constexpr uint32_t idesc = make_idesc_f16_f32(128, BN);
        const uint32_t me = (uint32_t)(warp - 1);
        uint32_t seq = 0, bgen = 0, tcount = 0;
        int32_t cur_nt = -1, cur_col = -1, next_row = 0;
        const uint32_t blkA = (uint32_t)kBoxPixels * (uint32_t)p.rowb;
        for (int64_t idx = t_begin; idx < t_end; idx++, tcount++) {
            const NhwcTile t = decode_tile(p, idx);
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            {
                PROF_T0();
                if (!mbar_wait_warp(&tempty[acc], aph ^ 1, abort_flag)) break;
                if (me == 0) PROF_ADD(1);
            }
            if (t.nt != cur_nt) {
                if (!mbar_wait_warp(bfull, bgen & 1, abort_flag)) break;
                bgen++;
                cur_nt = t.nt;
            }
            if (t.col != cur_col) {
                cur_col = t.col;
                next_row = t.ho - p.pad;
            }
            const int32_t last_row = t.ho - p.pad + p.Kh - 1;
            const uint32_t fresh_rows = (uint32_t)(last_row + 1 - next_row);
            next_row = last_row + 1;
            bool ok = true;
            {
                PROF_T0();
                for (uint32_t i = 0; i < fresh_rows && ok; i++, seq++)
                    ok = mbar_wait_warp(&full[seq % stages], (seq / stages) & 1, abort_flag);
                if (me == 0) PROF_ADD(2);
            }
            if (!ok) break;
            tc_fence_after();
            PROF_T0();
            // is the next tile of this CTA the next output row of the same column?
            bool col_ends = idx + 1 >= t_end, nt_ends = col_ends;
            if (!col_ends) {
                const uint32_t ncol = static_cast<uint32_t>(idx + 1) / (uint32_t)p.Ho;
                col_ends = (int32_t)ncol != t.col;
                nt_ends = col_ends && (int32_t)(ncol / (uint32_t)(p.segs * p.N)) != t.nt;
            }
            const uint32_t d_tmem = tmem_base + acc * 2 * BN + me * BN;
            const uint32_t first = seq - (uint32_t)p.Kh;
            if (elect_one()) {
                // descriptor low words: (address >> 4) | leading-offset field; all offsets are multiples of 16 bytes
                const uint32_t hi = ((uint32_t)p.sbo >> 4) | (1u << 14) | ((uint32_t)p.layout << 29);
                const uint32_t a_base = ((smem_u32(smA) & 0x3ffff) >> 4) | (1u << 16);
                uint32_t b_lo = ((smem_u32(smB) & 0x3ffff) >> 4) | (1u << 16);
                const uint32_t slot_e = p.slot_bytes >> 4, blkA_e = blkA >> 4, row_e = (uint32_t)p.rowb >> 4,
                               bblk_e = p.bblk_bytes >> 4;
                bool fresh = true;
                uint32_t i0 = 0;
                for (int32_t kh = 0; kh < p.Kh; kh++) {
                    uint32_t a_row = a_base + ((first + kh) % stages) * slot_e;
                    for (int32_t kw = 0; kw < p.Kw; kw++, a_row += row_e) {
                        uint32_t a_lo = a_row;
                        for (int32_t cb = 0; cb < p.CB; cb++, a_lo += blkA_e, b_lo += bblk_e) {
                            if (p.ksteps == 4) mma_block<4>(d_tmem, a_lo, b_lo, hi, idesc, i0, me, fresh);
                            else if (p.ksteps == 2) mma_block<2>(d_tmem, a_lo, b_lo, hi, idesc, i0, me, fresh);
                            else mma_block<1>(d_tmem, a_lo, b_lo, hi, idesc, i0, me, fresh);
                            i0 += (uint32_t)p.ksteps;
                        }
                    }
                }
#ifdef NZB_NHWC_PROFILE
                if (me == 0) atomicAdd(&g_nhwc_prof[7], (unsigned long long)(clock64() - _t0));
#endif
                // free what no later tile of this CTA reads: the top row, or every row at the end of a column
                const int32_t nfree = col_ends ? p.Kh : 1;
                for (int32_t kh = 0; kh < nfree; kh++) mma_commit(&empty[(first + kh) % stages]);
                if (nt_ends) mma_commit(bempty);
                mma_commit(&tfull[acc]);
            }
            __syncwarp();
            if (me == 0) PROF_ADD(3);
        }
    } else {
        // ---------------- epilogue: lanes are pixels, one coalesced store per channel ----------------
        const int q = warp & 3;                // tensor-memory lane quarter this warp may read
        const int grp = (warp - 3) >> 2;       // which half of the channel tile
        constexpr int NCH = Cfg::COLS / Cfg::CHUNK;
        const int32_t m0 = q * 32;
        auto load_bias = [&](const NhwcTile& t, int c0, float (&a)[Cfg::CHUNK]) {
            const int32_t co0 = t.nt * BN + c0;
            const int32_t pix0 = t.ho * p.Wo + t.wo0 + m0;
            const int32_t pixc = m0 + lane < t.npx ? pix0 + lane : pix0;
            const bool whole = co0 + Cfg::CHUNK <= p.Cout;
            if (m0 >= t.npx || co0 >= p.Cout || p.bias_mode == NZB_BIAS_NONE) {
#pragma unroll
                for (int j = 0; j < Cfg::CHUNK; j++) a[j] = 0.f;
            } else if (p.bias_mode == kBiasMatrixT) {
                const float* bp = p.bias + static_cast<int64_t>(co0) * p.HoWo + pixc;
#pragma unroll
                for (int j = 0; j < Cfg::CHUNK; j++)
                    a[j] = (whole || co0 + j < p.Cout) ? __ldg(bp + static_cast<int64_t>(j) * p.HoWo) : 0.f;
            } else if (p.bias_mode == NZB_BIAS_MATRIX) {
                const float* bp = p.bias + static_cast<int64_t>(pixc) * p.Cout + co0;
#pragma unroll
                for (int j = 0; j < Cfg::CHUNK; j++) a[j] = (whole || co0 + j < p.Cout) ? __ldg(bp + j) : 0.f;
            } else {
#pragma unroll
                for (int j = 0; j < Cfg::CHUNK; j++) a[j] = __ldg(p.bias + min(co0 + j, p.Cout - 1));
            }
        };
        uint32_t tcount = 0;
        for (int64_t idx = t_begin; idx < t_end; idx++, tcount++) {
            const NhwcTile t = decode_tile(p, idx);
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            {
                PROF_T0();
                if (!mbar_wait_relaxed(&tfull[acc], aph, abort_flag)) break;
                if (warp == 3) PROF_ADD(4);
            }
            PROF_T0();
            tc_fence_after();
            const int32_t pix = t.ho * p.Wo + t.wo0 + m0 + lane;
            const bool pix_ok = m0 + lane < t.npx;
            const bool quarter_ok = m0 < t.npx;  // warp-uniform: this quarter of the tile holds pixels
            float* yb = p.Y + (static_cast<int64_t>(p.img0 + t.img) * p.Cout) * p.HoWo + pix;
#pragma unroll
            for (int ci = 0; ci < NCH; ci++) {
                const int c0 = grp * Cfg::COLS + ci * Cfg::CHUNK;
                const int32_t co0 = t.nt * BN + c0;
                float add[Cfg::CHUNK];
                if (!quarter_ok || co0 >= p.Cout) continue;
                load_bias(t, c0, add);  // before the accumulator load, so the two latencies overlap
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 2 * BN + c0;
                const bool whole = co0 + Cfg::CHUNK <= p.Cout;
                float* yg = yb + static_cast<int64_t>(co0) * p.HoWo;
                if constexpr (ACC) {
                    if (pix_ok) {
#pragma unroll
                        for (int j = 0; j < Cfg::CHUNK; j++)
                            if (whole || co0 + j < p.Cout) add[j] += yg[static_cast<int64_t>(j) * p.HoWo];
                    }
                }
                uint32_t v[Cfg::CHUNK];
                if constexpr (Cfg::CHUNK == 32) tmem_ld_32x32(taddr, v);
                else tmem_ld_32x16(taddr, v);
                if (p.nsplit == 2) {
                    // the second MMA warp's partial sum
                    uint32_t v2[Cfg::CHUNK];
                    if constexpr (Cfg::CHUNK == 32) tmem_ld_32x32(taddr + BN, v2);
                    else tmem_ld_32x16(taddr + BN, v2);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < Cfg::CHUNK; j++) add[j] += __uint_as_float(v2[j]);
                } else {
                    tmem_ld_wait();
                }
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[acc]);
            if (warp == 3) PROF_ADD(5);
        }
    }
#ifdef NZB_NHWC_PROFILE
    if (threadIdx.x == 0) atomicAdd(&g_nhwc_prof[6], (unsigned long long)(clock64() - _k0));
#endif

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

// ---- staging ---------------------------------------------------------------------------------------
// XH[n][pixel][c] = half(X[n][c][pixel]) for one pass of images: a CT x PT tile (CT * PT = 4096) goes
// through shared memory, read as float4 along pixels, written as 16-byte channel groups.
// The shared tile has a pitch of CT + 2 halves: lanes that differ in pixel and channel pair then write
// different banks, and the 4-byte reads of the store phase are conflict-free as well.
template <int CT>
__global__ void __launch_bounds__(256) nchw_to_nhwc_half_kernel(__half* __restrict__ out, const float* __restrict__ in,
                                                                int64_t HW, int32_t C, int32_t tiles_px, int vec_ok) {
    constexpr int PT = 4096 / CT, PITCH = CT + 2;
    __shared__ __align__(16) __half tile[PT * PITCH];
    const int32_t cblks = C / CT;
    uint32_t b = blockIdx.x;
    const uint32_t tp = b % (uint32_t)tiles_px;
    b /= (uint32_t)tiles_px;
    const uint32_t cbk = b % (uint32_t)cblks, n = b / (uint32_t)cblks;
    const int64_t px0 = (int64_t)tp * PT;
    const float* src = in + ((int64_t)n * C + cbk * CT) * HW + px0;
    const int64_t left = HW - px0;  // pixels of this tile that exist
#pragma unroll
    for (int it = 0; it < 2; it++) {
        const int t = threadIdx.x + it * 256;
        const int pxg = t & 7, cp = (t >> 3) & 3, rest = t >> 5;
        const int pb = rest % (PT / 32), cblk = rest / (PT / 32);
        const int px = pb * 32 + pxg * 4, c = cblk * 8 + cp * 2;
        float a[4], d[4];
        if (vec_ok && px + 4 <= left) {
            const float4 u = __ldg(reinterpret_cast<const float4*>(src + (int64_t)c * HW + px));
            const float4 w = __ldg(reinterpret_cast<const float4*>(src + (int64_t)(c + 1) * HW + px));
            a[0] = u.x; a[1] = u.y; a[2] = u.z; a[3] = u.w;
            d[0] = w.x; d[1] = w.y; d[2] = w.z; d[3] = w.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                a[i] = px + i < left ? __ldg(src + (int64_t)c * HW + px + i) : 0.f;
                d[i] = px + i < left ? __ldg(src + (int64_t)(c + 1) * HW + px + i) : 0.f;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++)
            *reinterpret_cast<__half2*>(&tile[(px + i) * PITCH + c]) = __floats2half2_rn(a[i], d[i]);
    }
    __syncthreads();
    __half* dst = out + ((int64_t)n * HW + px0) * C + cbk * CT;
#pragma unroll
    for (int it = 0; it < 2; it++) {
        const int u = threadIdx.x + it * 256;
        const int c8 = u % (CT / 8), px = u / (CT / 8);
        if (px < left) {
            const uint32_t* s = reinterpret_cast<const uint32_t*>(&tile[px * PITCH + c8 * 8]);
            uint4 v;
            v.x = s[0]; v.y = s[1]; v.z = s[2]; v.w = s[3];
            *reinterpret_cast<uint4*>(dst + (int64_t)px * C + c8 * 8) = v;
        }
    }
}

// Weights for the channels-last kernel: out[tap][r][cin], tap = kh * Kw + kw.
//   forward  (flip = 0): r = co, cin = c:  w[(c*Kh + kh)*Kw + kw][co]
//   backward (flip = 1): r = c, cin = co:  w[(c*Kh + Kh-1-kh)*Kw + Kw-1-kw][co]
// with w = {1, 1, C*Kh*Kw, Cout} as the reference stores it.
__global__ void __launch_bounds__(256) nhwc_weights_kernel(__half* __restrict__ out, const float* __restrict__ w,
                                                           int64_t C, int64_t Cout, int64_t Kh, int64_t Kw, int flip) {
    const int64_t Cin = flip ? Cout : C, R = flip ? C : Cout;
    const int64_t total = Kh * Kw * R * Cin;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t cin = i % Cin, r = (i / Cin) % R, tap = i / (Cin * R);
        const int64_t kh = tap / Kw, kw = tap % Kw;
        const int64_t c = flip ? r : cin, co = flip ? cin : r;
        const int64_t kh2 = flip ? Kh - 1 - kh : kh, kw2 = flip ? Kw - 1 - kw : kw;
        out[i] = __float2half_rn(__ldg(w + ((c * Kh + kh2) * Kw + kw2) * Cout + co));
    }
}

__global__ void __launch_bounds__(256) nhwc_transpose_f32_kernel(float* __restrict__ out, const float* __restrict__ in,
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

constexpr int kSmemLimit = 232448 - 1024;  // dynamic shared memory of one sm_100 CTA, less the alignment slack

static int64_t stage_budget_bytes() {
    static const int64_t env = [] {
        const char* e = getenv("NZB_CONV_STAGE_BYTES");
        return e ? atoll(e) : (long long)0;
    }();
    return env > 0 ? env : (int64_t(1) << 30);
}

template <class Cfg>
static int launch_nhwc(const ConvNhwcRun& r, const NhwcPlan& pl, void* ws, const DeviceState& ds, cudaStream_t stream) {
    EncodeTiledFn enc;
    int rc = get_encode_tiled(&enc);
    if (rc != NZB_OK) return rc;
    uint8_t* base = reinterpret_cast<uint8_t*>(ws);
    __half* W16 = reinterpret_cast<__half*>(base);
    __half* XH = reinterpret_cast<__half*>(base + pl.w_bytes);
    float* bias_t = reinterpret_cast<float*>(base + pl.w_bytes + pl.nchunk * pl.per_image);
    const int64_t taps = r.Kh * r.Kw;
    {
        const int64_t total = taps * r.R * r.Cin;
        int64_t blocks = (total + 255) / 256;
        if (blocks > (int64_t)ds.sm_count * 16) blocks = (int64_t)ds.sm_count * 16;
        nhwc_weights_kernel<<<(unsigned)blocks, 256, 0, stream>>>(W16, r.w, r.layerC, r.layerCout, r.Kh, r.Kw, r.flip);
        NZB_CUDA_TRY(cudaGetLastError());
    }
    const CUtensorMapSwizzle swz = pl.Cb == 64 ? CU_TENSOR_MAP_SWIZZLE_128B
                                   : pl.Cb == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    CUtensorMap tmW;
    {
        cuuint64_t dims[3] = {(cuuint64_t)r.Cin, (cuuint64_t)r.R, (cuuint64_t)taps};
        cuuint64_t strides[2] = {(cuuint64_t)r.Cin * 2, (cuuint64_t)r.R * r.Cin * 2};
        cuuint32_t box[3] = {(cuuint32_t)pl.Cb, (cuuint32_t)Cfg::BN, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult cr = enc(&tmW, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, W16, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled (channels-last weights) failed with CUresult %d", (int)cr);
    }
    NhwcParams p{};
    p.Y = r.Y;
    p.bias = r.bias;
    p.Cout = (int32_t)r.R; p.Kh = (int32_t)r.Kh; p.Kw = (int32_t)r.Kw; p.pad = (int32_t)r.pad;
    p.Ho = (int32_t)r.Ho; p.Wo = (int32_t)r.Wo; p.HoWo = (int32_t)(r.Ho * r.Wo);
    p.CB = (int32_t)(r.Cin / pl.Cb);
    p.rowb = pl.Cb * 2;
    p.ksteps = pl.Cb / 16;
    p.layout = pl.Cb == 64 ? 2 : pl.Cb == 32 ? 4 : 6;
    p.sbo = 8 * p.rowb;
    p.segs = (int32_t)((r.Wo + 127) / 128);
    p.tiles_n = (int32_t)((r.R + Cfg::BN - 1) / Cfg::BN);
    p.stages = pl.stages;
    p.nsplit = taps * p.CB * p.ksteps >= 2 ? 2 : 1;
    p.slot_bytes = (uint32_t)(p.CB * kBoxPixels * p.rowb);
    p.bblk_bytes = (uint32_t)(Cfg::BN * p.rowb);
    p.b_bytes = (uint32_t)(taps * p.CB) * p.bblk_bytes;
    p.bias_mode = r.bias ? r.bias_mode : NZB_BIAS_NONE;
    if (p.bias_mode == NZB_BIAS_MATRIX && r.N >= 4) {
        // [pixel][channel] as the reference stores it -> [channel][pixel], which lanes (= pixels) read contiguously
        const int64_t tiles = ((r.Ho * r.Wo + 31) / 32) * ((r.R + 31) / 32);
        const int64_t cap = (int64_t)ds.sm_count * 16;
        nhwc_transpose_f32_kernel<<<(unsigned)(tiles < cap ? tiles : cap), 256, 0, stream>>>(bias_t, r.bias, r.Ho * r.Wo, r.R);
        NZB_CUDA_TRY(cudaGetLastError());
        p.bias = bias_t;
        p.bias_mode = kBiasMatrixT;
    }
    p.relu = r.relu;
    p.status = ds.status_dev;
    const int smem_bytes = 1024 + (int)round_up(p.b_bytes, 1024) + p.stages * (int)p.slot_bytes + Cfg::BAR_BYTES;
    static std::atomic<uint64_t> smem_set[2];
    {
        // the attribute is raised to the largest size any plan can ask for, once per device
        int rc_attr = ensure_dynamic_smem(smem_set[0], reinterpret_cast<const void*>(conv2d_nhwc_tcgen05_kernel<Cfg, false>), kSmemLimit + 1024);
        if (rc_attr == NZB_OK)
            rc_attr = ensure_dynamic_smem(smem_set[1], reinterpret_cast<const void*>(conv2d_nhwc_tcgen05_kernel<Cfg, true>), kSmemLimit + 1024);
        if (rc_attr != NZB_OK) return rc_attr;
    }
    // resident CTAs per SM: what registers and shared memory allow, at most three, and no more than the
    // tensor memory holds (an allocation that does not fit would wait for a CTA to retire)
    int per_sm = 1;
    {
        const void* fn = r.accumulate ? reinterpret_cast<const void*>(conv2d_nhwc_tcgen05_kernel<Cfg, true>)
                                      : reinterpret_cast<const void*>(conv2d_nhwc_tcgen05_kernel<Cfg, false>);
        NZB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, Cfg::THREADS, smem_bytes));
    }
    if (per_sm > 512 / Cfg::TMEM_COLS) per_sm = 512 / Cfg::TMEM_COLS;
    if (per_sm > 3) per_sm = 3;
    if (per_sm < 1) per_sm = 1;
    const int64_t cap = (int64_t)ds.sm_count * per_sm;
    const int64_t HW = r.Hin * r.Win;
    for (int64_t img0 = 0; img0 < r.N; img0 += pl.nchunk) {
        const int64_t n = r.N - img0 < pl.nchunk ? r.N - img0 : pl.nchunk;
        {
            const float* src = r.X + img0 * r.Cin * HW;
            const int vec_ok = (HW % 4 == 0) && (reinterpret_cast<uintptr_t>(src) & 15) == 0;
            const int CT = r.Cin >= 64 ? 64 : (int)r.Cin;
            const int64_t tiles_px = (HW + 4096 / CT - 1) / (4096 / CT);
            const int64_t blocks = n * (r.Cin / CT) * tiles_px;
            if (blocks > INT32_MAX) return fail(NZB_ERR_UNSUPPORTED, "more than 2^31 staging tiles in one pass");
            if (CT == 64) nchw_to_nhwc_half_kernel<64><<<(unsigned)blocks, 256, 0, stream>>>(XH, src, HW, (int32_t)r.Cin, (int32_t)tiles_px, vec_ok);
            else if (CT == 32) nchw_to_nhwc_half_kernel<32><<<(unsigned)blocks, 256, 0, stream>>>(XH, src, HW, (int32_t)r.Cin, (int32_t)tiles_px, vec_ok);
            else nchw_to_nhwc_half_kernel<16><<<(unsigned)blocks, 256, 0, stream>>>(XH, src, HW, (int32_t)r.Cin, (int32_t)tiles_px, vec_ok);
            NZB_CUDA_TRY(cudaGetLastError());
        }
        CUtensorMap tmX;
        {
            const cuuint64_t px_b = (cuuint64_t)r.Cin * 2;
            cuuint64_t dims[4] = {(cuuint64_t)r.Cin, (cuuint64_t)r.Win, (cuuint64_t)r.Hin, (cuuint64_t)n};
            cuuint64_t strides[3] = {px_b, px_b * r.Win, px_b * r.Win * r.Hin};
            cuuint32_t box[4] = {(cuuint32_t)pl.Cb, (cuuint32_t)kBoxPixels, 1, 1};
            cuuint32_t estr[4] = {1, 1, 1, 1};
            CUresult cr = enc(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, XH, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (cr != CUDA_SUCCESS) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled (channels-last image) failed with CUresult %d", (int)cr);
        }
        p.N = (int32_t)n;
        p.img0 = (int32_t)img0;
        p.total = (int64_t)p.tiles_n * n * p.segs * r.Ho;
        if (p.total > INT32_MAX) return fail(NZB_ERR_UNSUPPORTED, "more than 2^31 output tiles in one pass");
        const int64_t grid = p.total < cap ? p.total : cap;
        if (r.accumulate)
            conv2d_nhwc_tcgen05_kernel<Cfg, true><<<(unsigned)grid, Cfg::THREADS, smem_bytes, stream>>>(tmW, tmX, p);
        else
            conv2d_nhwc_tcgen05_kernel<Cfg, false><<<(unsigned)grid, Cfg::THREADS, smem_bytes, stream>>>(tmW, tmX, p);
        NZB_CUDA_TRY(cudaGetLastError());
    }
    return NZB_OK;
}

}  // namespace

NhwcPlan nhwc_plan(int64_t N, int64_t Cin, int64_t Hin, int64_t Win, int64_t R, int64_t Kh, int64_t Kw, int64_t stride,
                   int64_t Ho, int64_t Wo, int64_t wN) {
    NhwcPlan t{};
    // NZB_CONV_NHWC: 0 = never, 2 = wherever the kernel can run (tests), default = where it wins
    static const int mode = [] {
        const char* e = getenv("NZB_CONV_NHWC");
        return e ? atoi(e) : 1;
    }();
    t.ok = mode != 0 && stride == 1 && wN == 1 && N > 0 && (Cin == 16 || Cin == 32 || (Cin % 64 == 0 && Cin > 0)) &&
           Kw <= 9 && Kh <= 9 && Wo >= 64 && Win >= 16 && Hin < (int64_t(1) << 30) && Win < (int64_t(1) << 30) &&
           R <= INT32_MAX && Ho * Wo <= INT32_MAX - 256;
    // Measured against the shifted-copies kernel on a B200: ahead where a 128-channel tile is mostly used and
    // its weights fit beside the ring (64 input channels, 65..128 output channels: 0.52 against 0.62 ms for
    // 32 x 64 x 224 x 224 -> 128), behind for narrow tiles (16 -> 16: 1.25 against 0.57 ms) and where that
    // kernel runs 256-column instructions (128 -> 256: 0.27 against 0.14 ms).
    if (t.ok && mode == 1) t.ok = Cin == 64 && R > 64 && R <= 128;
    if (!t.ok) return t;
    t.Cb = Cin >= 64 ? 64 : (int)Cin;
    const int64_t rowb = t.Cb * 2, CB = Cin / t.Cb;
    const int64_t slot = CB * kBoxPixels * rowb;
    int bn = 128;
    while (bn > 16 && bn / 2 >= R) bn /= 2;  // smallest tile that still covers R
    // The weights of one channel tile stay resident; the ring needs the Kh rows a tile reads plus at least
    // one in flight. The widest tile that fits wins: an instruction costs the issuing thread and the shared
    // memory operand fetch about the same whatever its N (128-column tiles with a ring of four measured
    // 0.52 ms on 32 x 64 x 224 x 224 -> 128, 64-column tiles with a ring of eight 0.74 ms).
    for (;; bn /= 2) {
        const int64_t b = round_up(Kh * Kw * CB * bn * rowb, 1024);
        const int64_t room = kSmemLimit - 1024 - 256 - b;
        const int64_t st = room > 0 ? room / slot : 0;
        if (st >= Kh + 1 && (mode == 2 || bn == 128)) {
            t.BN = bn;
            t.stages = (int)(st > 12 ? 12 : st);
            break;
        }
        if (bn == 16 || mode != 2) {
            t.ok = false;
            return t;
        }
    }
    t.w_bytes = round_up(Kh * Kw * R * Cin * 2, 256);
    t.per_image = round_up(Hin * Win * Cin * 2, 256);
    int64_t n = stage_budget_bytes() / t.per_image;
    if (n < 1) n = 1;
    if (n > N) n = N;
    n = (N + (N + n - 1) / n - 1) / ((N + n - 1) / n);  // equal-sized passes
    t.nchunk = n;
    t.bias_bytes = round_up(Ho * Wo * R * 4, 256);
    return t;
}

#ifdef NZB_NHWC_PROFILE
extern "C" __attribute__((visibility("default"))) int nzb_debug_nhwc_counters(unsigned long long* out, int reset) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, g_nhwc_prof, sizeof(unsigned long long) * 16);
    if (reset) {
        unsigned long long z[16] = {};
        cudaMemcpyToSymbol(g_nhwc_prof, z, sizeof(z));
    }
    return 0;
}
#endif

int run_conv_nhwc(const ConvNhwcRun& r, const NhwcPlan& pl, void* ws, cudaStream_t stream) {
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    switch (pl.BN) {
        case 128: return launch_nhwc<NhwcCfg<128>>(r, pl, ws, *ds, stream);
        case 64: return launch_nhwc<NhwcCfg<64>>(r, pl, ws, *ds, stream);
        case 32: return launch_nhwc<NhwcCfg<32>>(r, pl, ws, *ds, stream);
        default: return launch_nhwc<NhwcCfg<16>>(r, pl, ws, *ds, stream);
    }
}

}  // namespace nzb
