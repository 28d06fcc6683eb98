// fp16 x fp16 -> fp32 GEMM for sm_100a: TMA-fed shared-memory ring, tcgen05.mma into
// tensor memory, fused epilogue (accumulate / bias / ReLU / fp32 store).
//
// Stands in for GeneralMatrixMulTensorKernel and its Cutting / CuttingAndCompress
// passes (NeuZephyr src/OperationKernels.cu:821-883) behind the batched drivers
// (:914-1144). Operands arrive as fp16 copies, each either K-major (A' [nA][M][Kp],
// B' [nB][N][Kp]) or MN-major (A' [nA][K][Mp], B' [nB][K][Np], i.e. the source's own
// row-major layout when it is stored with the contraction along rows), so a transposed
// operand costs no transposing pass: the tensor core reads either layout.
//
// CTA layout (192 threads, persistent over a static round-robin tile list):
//   warp 0    TMA producer (one lane)
//   warp 1    tensor-memory allocator; one lane issues tcgen05.mma
//   warps 2-5 epilogue: tcgen05.ld -> shared staging -> coalesced global stores
// Two accumulators live in tensor memory so the epilogue of tile i overlaps the
// main loop of tile i+1. Every mbarrier wait is bounded; on expiry the CTA raises an
// abort flag, writes NZB_ERR_DEVICE_TIMEOUT to the status word, drains and returns.
#include <cuda_fp16.h>

#include "nzb_internal.h"
#include "nzb_ptx.cuh"

namespace nzb {

struct GemmParams {
    float* C;
    int64_t ldc;
    int32_t M, N, K;
    int32_t tiles_m, tiles_n;
    int32_t out_e0, out_e1, red_e0, red_e1;
    int32_t a_mul0, a_mul1, b_mul0, b_mul1;
    int64_t c_stride0, c_stride1;
    const float* bias;
    int64_t bias_ld;
    int32_t bias_mode;
    int32_t accumulate, relu;
    int32_t k_blocks;     // ceil(K / 64)
    int32_t last_ksteps;  // 16-wide MMA steps in the last k block (1..4)
    int32_t vec4;         // C (and bias) allow aligned float4 access
    int32_t group_m;      // m-tiles per rasterisation group
    int32_t splits;       // CTAs sharing one output tile along the contraction (results added atomically)
    int32_t a_mn, b_mn;   // operand copy is stored [k][m] / [k][n] (contiguous along the output dimension)
    int32_t trans_out;    // the kernel computes C^T (operands swapped by the host): element (r, c) goes to C[c][r]
    int64_t total_tiles;
    const float* alpha;   // device scalar multiplied into the product before accumulate / bias (null: 1)
    int* status;
};

template <int BN_, int STAGES_, int MINB_ = 1>
struct GemmCfg {
    static constexpr int BM = 128, BN = BN_, BK = 64, STAGES = STAGES_;
    static constexpr int MIN_BLOCKS = MINB_;  // CTAs per SM: narrow tiles are bound by per-k-block and per-tile
                                              // latencies, which a second resident CTA overlaps
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int EPI_STRIDE = 36;  // floats per staged row: 16-byte aligned, conflict-free
    static constexpr int EPI_BYTES = 4 * 32 * EPI_STRIDE * 4;
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES;
    static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
    static constexpr int CHUNK = (BN < 32) ? BN : 32;  // accumulator columns per tcgen05.ld
    static_assert(STAGE_BYTES % 1024 == 0, "operand tiles must stay 1024-byte aligned");
    static_assert((SMEM_BYTES + 1024) * MINB_ <= 233472, "exceeds the 228 KB shared memory of an sm_100 SM");
    static_assert(TMEM_COLS * MINB_ <= 512, "exceeds the tensor memory of an SM");
};


struct TileCoord {
    int32_t mt, nt, b0, b1;
};

__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int64_t tile) {
    const int64_t per_batch = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
    const int64_t ob = tile / per_batch;
    const int32_t rem = static_cast<int32_t>(tile - ob * per_batch);
    const int32_t group_size = p.group_m * p.tiles_n;
    const int32_t g = rem / group_size;
    const int32_t first_m = g * p.group_m;
    const int32_t gm = min(p.tiles_m - first_m, p.group_m);
    const int32_t within = rem - g * group_size;
    TileCoord t;
    t.mt = first_m + within % gm;
    t.nt = within / gm;
    t.b0 = static_cast<int32_t>(ob / p.out_e1);
    t.b1 = static_cast<int32_t>(ob % p.out_e1);
    return t;
}


// Operand tile loads for one k block. K-major: one box of `rows` x 64 k. MN-major: rows/64
// boxes of 64 (m or n) x 64 k, 8192 bytes apart, which is the layout the MN-major
// descriptor below walks (leading byte offset 8192, 1024 bytes per 8-k group).
template <int ROWS>
__device__ __forceinline__ void load_operand(uint8_t* dst, const CUtensorMap* tm, int32_t mn, int32_t k0, int32_t row0,
                                             int32_t z, uint64_t* bar) {
    using namespace ptx;
    if (mn) {
#pragma unroll
        for (int j = 0; j < ROWS / 64; j++) tma_load_3d(dst + j * 8192, tm, row0 + j * 64, k0, z, bar);
    } else {
        tma_load_3d(dst, tm, k0, row0, z, bar);
    }
}
template <int ROWS>
__device__ __forceinline__ void load_operand_pair(uint8_t* dst, const CUtensorMap* tm, int32_t mn, int32_t k0,
                                                  int32_t row0, int32_t z, uint32_t leader_bar) {
    using namespace ptx;
    if (mn) {
#pragma unroll
        for (int j = 0; j < ROWS / 64; j++) tma_load_3d_pair(dst + j * 8192, tm, row0 + j * 64, k0, z, leader_bar);
    } else {
        tma_load_3d_pair(dst, tm, k0, row0, z, leader_bar);
    }
}

// Descriptor bits above the start address for a SWIZZLE_128B operand tile.
//   K-major: rows of 128 bytes, 8-row groups 1024 bytes apart (leading offset unused: 1).
//   MN-major: 64-element blocks 8192 bytes apart (leading), 8-k groups 1024 bytes apart (stride).
__device__ __forceinline__ uint64_t desc_high_bits(int32_t mn) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>(mn ? (8192 >> 4) : 1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// Descriptor address units (16 bytes) per 16-wide k step: 32 bytes along a K-major row,
// 16 rows of 128 bytes in an MN-major tile.
__device__ __forceinline__ uint32_t desc_kstep(int32_t mn) { return mn ? 128u : 2u; }

// Drains one finished accumulator quarter (32 tensor-memory lanes x BN columns, owned by
// this warp) through the warp's shared staging buffer into coalesced global stores, applying
// accumulate / bias / ReLU. tmem_acc addresses lane quarter and first column.
template <class Cfg>
__device__ __forceinline__ void drain_accumulator(const GemmParams& p, uint32_t tmem_acc, float* stage, int lane,
                                                  float* Cb, int32_t row0, int32_t col_tile, bool first_split = true) {
    using namespace ptx;
    constexpr int BN = Cfg::BN;
    const float al = p.alpha ? __ldg(p.alpha) : 1.0f;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += Cfg::CHUNK) {
        const uint32_t taddr = tmem_acc + c0;
        if constexpr (Cfg::CHUNK == 32) {
            uint32_t v[32];
            tmem_ld_32x32(taddr, v);
            tmem_ld_wait();
            float4* dst = reinterpret_cast<float4*>(stage + lane * Cfg::EPI_STRIDE);
#pragma unroll
            for (int j = 0; j < 8; j++)
                dst[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                     __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
        } else {
            uint32_t v[16];
            tmem_ld_32x16(taddr, v);
            tmem_ld_wait();
            float4* dst = reinterpret_cast<float4*>(stage + lane * Cfg::EPI_STRIDE);
#pragma unroll
            for (int j = 0; j < 4; j++)
                dst[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                     __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
        }
        __syncwarp();
        const int32_t gc0 = col_tile + c0;
        if (p.vec4) {
            constexpr int LPR = Cfg::CHUNK / 4;  // lanes per staged row
            constexpr int RPI = 32 / LPR;        // rows per iteration
            const int cl = (lane % LPR) * 4;
            const int32_t gc = gc0 + cl;
#pragma unroll
            for (int rr = 0; rr < 32; rr += RPI) {
                const int r = rr + lane / LPR;
                const int32_t gr = row0 + r;
                if (gr < p.M && gc < p.N) {  // N % 4 == 0 on this path: the whole float4 is in range
                    float4 x = *reinterpret_cast<const float4*>(stage + r * Cfg::EPI_STRIDE + cl);
                    x.x *= al; x.y *= al; x.z *= al; x.w *= al;
                    float* cp = Cb + static_cast<int64_t>(gr) * p.ldc + gc;
                    if (p.accumulate) {
                        const float4 o = *reinterpret_cast<const float4*>(cp);
                        x.x += o.x; x.y += o.y; x.z += o.z; x.w += o.w;
                    }
                    if (p.bias_mode == NZB_BIAS_ROW) {
                        const float4 b = *reinterpret_cast<const float4*>(p.bias + gc);
                        x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w;
                    } else if (p.bias_mode == NZB_BIAS_COL) {
                        const float b = p.bias[gr];
                        x.x += b; x.y += b; x.z += b; x.w += b;
                    } else if (p.bias_mode == NZB_BIAS_MATRIX) {
                        const float4 b = *reinterpret_cast<const float4*>(
                            p.bias + static_cast<int64_t>(gr) * p.bias_ld + gc);
                        x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w;
                    }
                    if (p.relu) {
                        x.x = fmaxf(x.x, 0.f); x.y = fmaxf(x.y, 0.f);
                        x.z = fmaxf(x.z, 0.f); x.w = fmaxf(x.w, 0.f);
                    }
                    *reinterpret_cast<float4*>(cp) = x;
                }
            }
        } else {
            constexpr int RPI = 32 / Cfg::CHUNK;  // 1, or 2 when the chunk is 16 wide
            const int cl = lane % Cfg::CHUNK;
            const int32_t gc = gc0 + cl;
#pragma unroll 4
            for (int rr = 0; rr < 32; rr += RPI) {
                const int r = rr + lane / Cfg::CHUNK;
                const int32_t gr = row0 + r;
                if (gr < p.M && gc < p.N) {
                    float x = stage[r * Cfg::EPI_STRIDE + cl] * al;
                    float* cp = Cb + static_cast<int64_t>(gr) * p.ldc + gc;
                    if (p.splits > 1) {
                        // partial sum of one k slice; C was zeroed or holds the addend. The slice that
                        // starts the contraction also contributes the bias.
                        if (first_split) {
                            if (p.bias_mode == NZB_BIAS_ROW) x += p.bias[gc];
                            else if (p.bias_mode == NZB_BIAS_COL) x += p.bias[gr];
                            else if (p.bias_mode == NZB_BIAS_MATRIX)
                                x += p.bias[static_cast<int64_t>(gr) * p.bias_ld + gc];
                        }
                        atomicAdd(cp, x);
                        continue;
                    }
                    if (p.accumulate) x += *cp;
                    if (p.bias_mode == NZB_BIAS_ROW) x += p.bias[gc];
                    else if (p.bias_mode == NZB_BIAS_COL) x += p.bias[gr];
                    else if (p.bias_mode == NZB_BIAS_MATRIX)
                        x += p.bias[static_cast<int64_t>(gr) * p.bias_ld + gc];
                    if (p.relu) x = fmaxf(x, 0.f);
                    *cp = x;
                }
            }
        }
        __syncwarp();
    }
}


// Transposed drain for the swapped-operand form used when the caller's M is tiny: this
// kernel's rows are the caller's columns, so the 32 lanes of a warp (32 consecutive rows
// here) write 32 consecutive floats of one caller row -- coalesced without staging.
// p.M / p.N are this kernel's (swapped) extents; p.ldc, bias and bias_ld are the caller's.
template <class Cfg>
__device__ __forceinline__ void drain_accumulator_transposed(const GemmParams& p, uint32_t tmem_acc, int lane, float* Cb,
                                                             int32_t row0, int32_t col_tile, bool first_split) {
    using namespace ptx;
    constexpr int BN = Cfg::BN;
    constexpr int G = 16;
    const int32_t gr = row0 + lane;  // caller's column
    const bool row_ok = gr < p.M;
    const bool with_bias = p.bias_mode != NZB_BIAS_NONE && (p.splits == 1 || first_split);
    const float floor_v = (p.relu && p.splits == 1) ? 0.f : -INFINITY;
    const float bias_row = (with_bias && p.bias_mode == NZB_BIAS_ROW && row_ok) ? p.bias[gr] : 0.f;
    const float al = p.alpha ? __ldg(p.alpha) : 1.0f;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += G) {
        const int32_t gc0 = col_tile + c0;  // caller's first row of this group
        if (gc0 >= p.N) break;              // warp-uniform
        const bool whole = gc0 + G <= p.N;
        float* cg = Cb + static_cast<int64_t>(gc0) * p.ldc + gr;
        // addends first (their loads overlap the tensor-memory read); every mode decision is per
        // group of 16, the inner loops are straight-line code
        float add[G];
#pragma unroll
        for (int j = 0; j < G; j++) add[j] = bias_row;
        if (with_bias && p.bias_mode == NZB_BIAS_COL) {
#pragma unroll
            for (int j = 0; j < G; j++) add[j] = p.bias[min(gc0 + j, p.N - 1)];
        } else if (with_bias && p.bias_mode == NZB_BIAS_MATRIX && row_ok) {
#pragma unroll
            for (int j = 0; j < G; j++)
                add[j] = p.bias[static_cast<int64_t>(min(gc0 + j, p.N - 1)) * p.bias_ld + gr];
        }
        if (p.accumulate && p.splits == 1 && row_ok) {
#pragma unroll
            for (int j = 0; j < G; j++) add[j] += cg[static_cast<int64_t>(whole ? j : min(j, p.N - 1 - gc0)) * p.ldc];
        }
        uint32_t v[G];
        tmem_ld_32x16(tmem_acc + c0, v);
        tmem_ld_wait();
        if (!row_ok) continue;
        if (p.splits > 1) {
#pragma unroll
            for (int j = 0; j < G; j++)
                if (whole || gc0 + j < p.N) atomicAdd(cg + static_cast<int64_t>(j) * p.ldc, __uint_as_float(v[j]) * al + add[j]);
        } else if (whole) {
#pragma unroll
            for (int j = 0; j < G; j++) cg[static_cast<int64_t>(j) * p.ldc] = fmaxf(__uint_as_float(v[j]) * al + add[j], floor_v);
        } else {
#pragma unroll
            for (int j = 0; j < G; j++)
                if (gc0 + j < p.N) cg[static_cast<int64_t>(j) * p.ldc] = fmaxf(__uint_as_float(v[j]) * al + add[j], floor_v);
        }
    }
}

template <class Cfg>
__global__ void __launch_bounds__(192, Cfg::MIN_BLOCKS)
gemm_f16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const GemmParams p) {
    using namespace ptx;
    constexpr int BN = Cfg::BN, STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* epi = reinterpret_cast<float*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES + Cfg::EPI_BYTES);
    uint64_t* full = bars;                  // [STAGES] TMA landed
    uint64_t* empty = bars + STAGES;        // [STAGES] MMAs that read the stage retired
    uint64_t* tfull = bars + 2 * STAGES;    // [2] accumulator complete
    uint64_t* tempty = bars + 2 * STAGES + 2;  // [2] accumulator drained by the epilogue
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
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

    const int32_t k_iters = p.red_e0 * p.red_e1 * p.k_blocks;  // per tile

    const int64_t total_items = p.total_tiles * p.splits;
    if (warp == 0) {
        // ---------------- TMA producer (whole warp waits, one elected lane issues) ----------------
        uint32_t it = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
            const TileCoord t = decode_tile(p, item / p.splits);
            const int32_t split = static_cast<int32_t>(item % p.splits);
            const int32_t kk0 = static_cast<int32_t>(static_cast<int64_t>(k_iters) * split / p.splits);
            const int32_t kk1 = static_cast<int32_t>(static_cast<int64_t>(k_iters) * (split + 1) / p.splits);
            int32_t kb = kk0 % p.k_blocks;
            int32_t r = kk0 / p.k_blocks;
            int32_t r1 = r % p.red_e1, r0 = r / p.red_e1;
            for (int32_t kk = kk0; kk < kk1; kk++, it++) {
                const int32_t i0 = t.b0 + r0, i1 = t.b1 + r1;
                const int32_t za = i0 * p.a_mul0 + i1 * p.a_mul1;
                const int32_t zb = i0 * p.b_mul0 + i1 * p.b_mul1;
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&empty[s], ph ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
                    mbar_arrive_expect_tx(&full[s], Cfg::STAGE_BYTES);
                    load_operand<128>(sa, &tmA, p.a_mn, kb * 64, t.mt * 128, za, &full[s]);
                    load_operand<BN>(sa + Cfg::A_BYTES, &tmB, p.b_mn, kb * 64, t.nt * BN, zb, &full[s]);
                }
                __syncwarp();
                if (++kb == p.k_blocks) {
                    kb = 0;
                    if (++r1 == p.red_e1) {
                        r1 = 0;
                        r0++;
                    }
                }
            }
        }
        if (!ok && lane == 0) {
            // Wait (bounded) for the copies still in flight so none lands after exit.
            const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0;
            const long long t0 = clock64();
            for (uint32_t j = first; j < it; j++) {
                while (!mbar_try_wait(&full[j % STAGES], (j / STAGES) & 1)) {
                    if (clock64() - t0 > kWaitCycleLimit) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (whole warp runs the loop, one elected lane issues) ----------------
        const uint32_t idesc = make_idesc_f16_f32(128, BN) | (p.a_mn ? 1u << 15 : 0u) | (p.b_mn ? 1u << 16 : 0u);
        const uint64_t hi_a = desc_high_bits(p.a_mn), hi_b = desc_high_bits(p.b_mn);
        const uint32_t ka = desc_kstep(p.a_mn), kb_step = desc_kstep(p.b_mn);
        uint32_t it = 0, tcount = 0;
        bool ok = true;
        for (int64_t item = blockIdx.x; item < total_items && ok; item += gridDim.x, tcount++) {
            const int32_t split = static_cast<int32_t>(item % p.splits);
            const int32_t kk0 = static_cast<int32_t>(static_cast<int64_t>(k_iters) * split / p.splits);
            const int32_t kk1 = static_cast<int32_t>(static_cast<int64_t>(k_iters) * (split + 1) / p.splits);
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            if (!mbar_wait_warp(&tempty[acc], aph ^ 1, abort_flag)) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BN;
            int32_t kb = kk0 % p.k_blocks;
            for (int32_t kk = kk0; kk < kk1; kk++, it++) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(&full[s], ph, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
                const uint64_t da = hi_a | ((sa & 0x3ffff) >> 4);
                const uint64_t db = hi_b | (((sa + Cfg::A_BYTES) & 0x3ffff) >> 4);
                const int32_t ksteps = (kb == p.k_blocks - 1) ? p.last_ksteps : 4;
                if (++kb == p.k_blocks) kb = 0;
                if (elect_one()) {
                    mma_f16_ss(d_tmem, da, db, idesc, kk > kk0 ? 1u : 0u);
                    if (ksteps > 1) mma_f16_ss(d_tmem, da + ka, db + kb_step, idesc, 1u);
                    if (ksteps > 2) mma_f16_ss(d_tmem, da + 2 * ka, db + 2 * kb_step, idesc, 1u);
                    if (ksteps > 3) mma_f16_ss(d_tmem, da + 3 * ka, db + 3 * kb_step, idesc, 1u);
                    mma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (ok && elect_one()) mma_commit(&tfull[acc]);
            __syncwarp();
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int q = warp & 3;  // tensor-memory lane quarter this warp may read
        float* stage = epi + (warp - 2) * 32 * Cfg::EPI_STRIDE;
        uint32_t tcount = 0;
        for (int64_t item = blockIdx.x; item < total_items; item += gridDim.x, tcount++) {
            const TileCoord t = decode_tile(p, item / p.splits);
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            if (!mbar_wait_bounded(&tfull[acc], aph, abort_flag)) break;
            tc_fence_after();
            float* Cb = p.C + t.b0 * p.c_stride0 + t.b1 * p.c_stride1;
            const int32_t row0 = t.mt * 128 + q * 32;
            const int32_t col_tile = t.nt * BN;
            if (p.trans_out)
                drain_accumulator_transposed<Cfg>(p, tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN, lane,
                                                  Cb, row0, col_tile, item % p.splits == 0);
            else
                drain_accumulator<Cfg>(p, tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN, stage, lane, Cb,
                                       row0, col_tile, item % p.splits == 0);
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


// ---------------------------------------------------------------------------
// CTA-pair variant (cluster of 2, tcgen05 cta_group::2): one 256 x 256 output tile per
// pair and k block. Each CTA loads its own 128 rows of A and its own 128 rows of B
// (half of the tile's N) -- 32 KB per k block instead of 48 KB for the single-CTA
// 128 x 256 tile -- and the leader's single MMA thread drives both tensor cores, each
// accumulating its 128 rows x 256 columns in its own tensor memory. Loads are plain
// per-CTA TMA copies; only barrier arrivals cross between the CTAs.
// ---------------------------------------------------------------------------
// ---- in-kernel staging for the CTA-pair kernel ------------------------------------------------
constexpr int kFuseChunk = 8192;  // floats per unit of conversion work
constexpr int kFuseWarps = 14;    // converter warps per CTA: as many as the register file allows beside the GEMM roles
// One fp32 operand as stored (rows x cols, row-major) and its fp16 copy of the same layout. The
// tensor core consumes the copy in panels of 256 output rows / columns: for a K-major copy a panel
// is 256 storage rows, for an MN-major copy it is 256 storage columns over all rows.
struct FuseOperand {
    const float* src;
    __half* dst;
    int64_t ld_src, ld_dst;
    int32_t rows, cols;
    int32_t by_cols;            // panels are column ranges (MN-major copy)
    uint32_t segs;              // by rows: chunk-sized segments per storage row
    uint32_t chunks_per_panel;  // by rows: 256 * segs; by cols: ceil(rows / rows-per-chunk)
    uint32_t panels;
};
struct FuseParams {
    FuseOperand a, b;
    unsigned* sync;         // [0] next chunk; [8 + i] finished chunks of A panel i; [8 + a.panels + j] of B panel j
    uint32_t lead_a;        // A panels of the first rasterisation group: converted right after B panel 0
    uint32_t total_chunks;
};

// A chunk is kFuseChunk floats: one segment of a storage row (row panels) or kFuseChunk / 256 rows x 256
// columns (column panels), moved in rounds of 8 float4 loads followed by 8 half4 stores per lane. Large
// chunks amortise what every chunk pays once: the atomic that hands it out, the fences and the counter.
__device__ __forceinline__ void store_half4(__half* d, const float4& v) {
    const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(d) = u;
}
__device__ __forceinline__ void convert_chunk(const FuseOperand& o, uint32_t panel, uint32_t within, int lane) {
    if (!o.by_cols) {
        const int64_t row = static_cast<int64_t>(panel) * 256 + within / o.segs;
        if (row >= o.rows) return;
        const int32_t c0 = static_cast<int32_t>(within % o.segs) * kFuseChunk;
        const int32_t n = min(kFuseChunk, o.cols - c0);
        const float* s = o.src + row * o.ld_src + c0 + lane * 4;
        __half* d = o.dst + row * o.ld_dst + c0 + lane * 4;
#pragma unroll 1
        for (int h = 0; h < kFuseChunk / 1024; h++) {
            if (h * 1024 >= n) break;
            float4 v[8];
            const int base = h * 1024 + lane * 4;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (base + j * 128 < n) v[j] = __ldcs(reinterpret_cast<const float4*>(s + h * 1024 + j * 128));
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (base + j * 128 < n) store_half4(d + h * 1024 + j * 128, v[j]);
            }
        }
    } else {
        const int32_t k0 = static_cast<int32_t>(within) * (kFuseChunk / 256);
        const int32_t col = static_cast<int32_t>(panel) * 256 + lane * 4;
        const float* s = o.src + static_cast<int64_t>(k0) * o.ld_src + col;
        __half* d = o.dst + static_cast<int64_t>(k0) * o.ld_dst + col;
#pragma unroll 1
        for (int h = 0; h < kFuseChunk / 1024; h++) {
            if (k0 + h * 4 >= o.rows) break;
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int r = h * 4 + (j >> 1), c = (j & 1) * 128;
                if (k0 + r < o.rows && col + c < o.cols)
                    v[j] = __ldcs(reinterpret_cast<const float4*>(s + static_cast<int64_t>(r) * o.ld_src + c));
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int r = h * 4 + (j >> 1), c = (j & 1) * 128;
                if (k0 + r < o.rows && col + c < o.cols) store_half4(d + static_cast<int64_t>(r) * o.ld_dst + c, v[j]);
            }
        }
    }
}

// Whole-warp bounded wait until a global counter written by other CTAs reaches `target`, followed by
// the fence that orders the TMA (async proxy) reads after the generic-proxy writes the counter covers.
__device__ __forceinline__ bool wait_counter_warp(const unsigned* counter, unsigned target, volatile int* abort_flag) {
    bool ok = true;
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
    if (v < target) {
        const long long t0 = clock64();
        uint32_t spins = 0;
        do {
            __nanosleep(64);
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
            if ((++spins & 0x3f) == 0) {
                if (*abort_flag) {
                    ok = false;
                    break;
                }
                if (clock64() - t0 > ptx::kWaitCycleLimit) {
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
            }
        } while (v < target);
    }
    ok = __all_sync(0xffffffffu, ok);
    asm volatile("fence.proxy.async.global;" ::: "memory");
    return ok;
}

struct PairCfg {
    static constexpr int BN = 256, STAGES = 6;
    static constexpr int A_BYTES = 128 * 64 * 2;
    static constexpr int B_BYTES = 128 * 64 * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int EPI_STRIDE = 36;
    static constexpr int EPI_BYTES = 4 * 32 * EPI_STRIDE * 4;
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES;
    static constexpr int TMEM_COLS = 512;
    static constexpr int CHUNK = 32;
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared memory of an sm_100 CTA");
};

// FUSED adds kFuseWarps converter warps per CTA that stage the fp32 operands as fp16 while the
// GEMM runs: they take kFuseChunk-float chunks from one global counter, in the order the tile schedule needs
// the panels, and count finished chunks per panel; a producer warp starts a tile's loads only once the
// tile's A panel and B panel are complete. Converters never wait for anything, so the kernel cannot
// deadlock on itself; the producers' waits are bounded like every other wait.
template <bool FUSED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(FUSED ? 192 + 32 * kFuseWarps : 192, 1)
gemm_f16_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                             const GemmParams p, const FuseParams f) {
    using namespace ptx;
    using Cfg = PairCfg;
    constexpr int BN = Cfg::BN, STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* epi = reinterpret_cast<float*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES + Cfg::EPI_BYTES);
    uint64_t* full = bars;                     // [STAGES] leader's copy counts both CTAs' TMA bytes
    uint64_t* empty = bars + STAGES;           // [STAGES] per CTA, signalled by the leader's commits
    uint64_t* tfull = bars + 2 * STAGES;       // [2] per CTA, signalled by the leader's commits
    uint64_t* tempty = bars + 2 * STAGES + 2;  // [2] leader's copy: 8 epilogue warps arrive
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const int64_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], 8);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();  // both CTAs' barriers are initialised before anything crosses over
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int32_t k_iters = p.red_e0 * p.red_e1 * p.k_blocks;  // per tile

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs; whole warp waits, one elected lane issues) ----------------
        uint32_t it = 0;
        bool ok = true;
        for (int64_t tile = pair; tile < p.total_tiles && ok; tile += npairs) {
            const TileCoord t = decode_tile(p, tile);
            const int32_t row_a = t.mt * 256 + (int32_t)rank * 128;
            const int32_t row_b = t.nt * 256 + (int32_t)rank * 128;
            if constexpr (FUSED) {
                if (!wait_counter_warp(f.sync + 8 + t.mt, f.a.chunks_per_panel, abort_flag) ||
                    !wait_counter_warp(f.sync + 8 + f.a.panels + t.nt, f.b.chunks_per_panel, abort_flag)) {
                    ok = false;
                    break;
                }
            }
            for (int32_t r0 = 0; r0 < p.red_e0 && ok; r0++) {
                for (int32_t r1 = 0; r1 < p.red_e1 && ok; r1++) {
                    const int32_t i0 = t.b0 + r0, i1 = t.b1 + r1;
                    const int32_t za = i0 * p.a_mul0 + i1 * p.a_mul1;
                    const int32_t zb = i0 * p.b_mul0 + i1 * p.b_mul1;
                    for (int32_t kb = 0; kb < p.k_blocks; kb++, it++) {
                        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                        if (!mbar_wait_warp(&empty[s], ph ^ 1, abort_flag)) {
                            ok = false;
                            break;
                        }
                        if (elect_one()) {
                            uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
                            const uint32_t leader_full = map_to_cta(smem_u32(&full[s]), 0);
                            if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * Cfg::STAGE_BYTES);
                            load_operand_pair<128>(sa, &tmA, p.a_mn, kb * 64, row_a, za, leader_full);
                            load_operand_pair<128>(sa + Cfg::A_BYTES, &tmB, p.b_mn, kb * 64, row_b, zb, leader_full);
                        }
                        __syncwarp();
                    }
                }
            }
        }
        if (!ok && rank == 0 && lane == 0) {
            // Wait (bounded) for the copies still in flight so none lands after exit.
            const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0;
            for (uint32_t j = first; j < it; j++) {
                const long long t0 = clock64();
                while (!mbar_try_wait(&full[j % STAGES], (j / STAGES) & 1)) {
                    if (clock64() - t0 > kWaitCycleLimit) break;
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0) {
            // ---------------- MMA issuer (leader only; whole warp runs the loop) ----------------
            const uint32_t idesc = make_idesc_f16_f32(256, BN) | (p.a_mn ? 1u << 15 : 0u) | (p.b_mn ? 1u << 16 : 0u);
            const uint64_t hi_a = desc_high_bits(p.a_mn), hi_b = desc_high_bits(p.b_mn);
            const uint32_t ka = desc_kstep(p.a_mn), kb_step = desc_kstep(p.b_mn);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int64_t tile = pair; tile < p.total_tiles && ok; tile += npairs, tcount++) {
                const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
                if (!mbar_wait_warp(&tempty[acc], aph ^ 1, abort_flag)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                int32_t kb = 0;
                for (int32_t kk = 0; kk < k_iters; kk++, it++) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    if (!mbar_wait_warp(&full[s], ph, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
                    const uint64_t da = hi_a | ((sa & 0x3ffff) >> 4);
                    const uint64_t db = hi_b | (((sa + Cfg::A_BYTES) & 0x3ffff) >> 4);
                    const int32_t ksteps = (kb == p.k_blocks - 1) ? p.last_ksteps : 4;
                    if (++kb == p.k_blocks) kb = 0;
                    if (elect_one()) {
                        mma_f16_ss_pair(d_tmem, da, db, idesc, kk > 0 ? 1u : 0u);
                        if (ksteps > 1) mma_f16_ss_pair(d_tmem, da + ka, db + kb_step, idesc, 1u);
                        if (ksteps > 2) mma_f16_ss_pair(d_tmem, da + 2 * ka, db + 2 * kb_step, idesc, 1u);
                        if (ksteps > 3) mma_f16_ss_pair(d_tmem, da + 3 * ka, db + 3 * kb_step, idesc, 1u);
                        mma_commit_pair(&empty[s]);
                    }
                    __syncwarp();
                }
                if (ok && elect_one()) mma_commit_pair(&tfull[acc]);
                __syncwarp();
            }
        }
    } else if (FUSED && warp >= 6) {
        // ---------------- converter warps (both CTAs): fp32 -> fp16 staging ----------------
        const uint32_t c0 = f.b.chunks_per_panel;                          // B panel 0
        const uint32_t c1 = c0 + f.lead_a * f.a.chunks_per_panel;          // A panels of the first group
        const uint32_t c2 = c1 + (f.b.panels - 1) * f.b.chunks_per_panel;  // remaining B panels
        for (;;) {
            unsigned c = 0;
            if (lane == 0) c = atomicAdd(f.sync, 1u);
            c = __shfl_sync(0xffffffffu, c, 0);
            if (c >= f.total_chunks) break;
            uint32_t panel, within, slot;
            bool is_b;
            if (c < c0) {
                is_b = true; panel = 0; within = c;
            } else if (c < c1) {
                is_b = false; panel = (c - c0) / f.a.chunks_per_panel; within = (c - c0) % f.a.chunks_per_panel;
            } else if (c < c2) {
                is_b = true; panel = 1 + (c - c1) / f.b.chunks_per_panel; within = (c - c1) % f.b.chunks_per_panel;
            } else {
                is_b = false; panel = f.lead_a + (c - c2) / f.a.chunks_per_panel; within = (c - c2) % f.a.chunks_per_panel;
            }
            {
                FuseOperand o;  // one copy of the conversion code serves both operands (register budget)
                o.src = is_b ? f.b.src : f.a.src;
                o.dst = is_b ? f.b.dst : f.a.dst;
                o.ld_src = is_b ? f.b.ld_src : f.a.ld_src;
                o.ld_dst = is_b ? f.b.ld_dst : f.a.ld_dst;
                o.rows = is_b ? f.b.rows : f.a.rows;
                o.cols = is_b ? f.b.cols : f.a.cols;
                o.by_cols = is_b ? f.b.by_cols : f.a.by_cols;
                o.segs = is_b ? f.b.segs : f.a.segs;
                convert_chunk(o, panel, within, lane);
                slot = is_b ? 8 + f.a.panels + panel : 8 + panel;
            }
            // every lane's stores become visible (to the TMA engine too) before the chunk is counted
            asm volatile("fence.proxy.async.global;" ::: "memory");
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(f.sync + slot, 1u);
        }
    } else {
        // ---------------- epilogue warps (both CTAs) ----------------
        const int q = warp & 3;
        float* stage = epi + (warp - 2) * 32 * Cfg::EPI_STRIDE;
        uint32_t tcount = 0;
        for (int64_t tile = pair; tile < p.total_tiles; tile += npairs, tcount++) {
            const TileCoord t = decode_tile(p, tile);
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            if (!mbar_wait_bounded(&tfull[acc], aph, abort_flag)) break;
            tc_fence_after();
            float* Cb = p.C + t.b0 * p.c_stride0 + t.b1 * p.c_stride1;
            const int32_t row0 = t.mt * 256 + (int32_t)rank * 128 + q * 32;
            const int32_t col_tile = t.nt * BN;
            drain_accumulator<Cfg>(p, tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN, stage, lane, Cb,
                                   row0, col_tile);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[acc]), 0));
        }
    }

    __syncwarp();
    tc_fence_before();
    cluster_sync_all();  // neither CTA leaves while its pair may still touch its shared memory
    if (threadIdx.x == 0 && *abort_flag) {
        *p.status = NZB_ERR_DEVICE_TIMEOUT;
        __threadfence_system();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
static int make_operand_map(CUtensorMap* map, const __half* base, int64_t K, int64_t Kp, int64_t rows, int64_t nmat,
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

// MN-major operand copy [nmat][K][ld]: dimension 0 runs along m (or n), boxes are 64 x 64.
static int make_operand_map_mn(CUtensorMap* map, const __half* base, int64_t K, int64_t extent, int64_t ld,
                               int64_t nmat) {
    EncodeTiledFn enc;
    int rc = get_encode_tiled(&enc);
    if (rc != NZB_OK) return rc;
    cuuint64_t dims[3] = {(cuuint64_t)extent, (cuuint64_t)K, (cuuint64_t)nmat};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)K * (cuuint64_t)ld * 2};
    cuuint32_t box[3] = {64, 64, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NZB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return NZB_OK;
}

static int make_maps(const GemmLaunch& g, CUtensorMap* tmA, CUtensorMap* tmB, int box_n) {
    int rc = g.a_mn ? make_operand_map_mn(tmA, g.A16, g.K, g.M, g.lda16, g.nA)
                    : make_operand_map(tmA, g.A16, g.K, g.Kp, g.M, g.nA, 128);
    if (rc != NZB_OK) return rc;
    return g.b_mn ? make_operand_map_mn(tmB, g.B16, g.K, g.N, g.ldb16, g.nB)
                  : make_operand_map(tmB, g.B16, g.K, g.Kp, g.N, g.nB, box_n);
}

template <class Cfg>
static int launch_cfg(const GemmLaunch& g, GemmParams& p, const DeviceState& ds, cudaStream_t stream) {
    CUtensorMap tmA, tmB;
    int rc = make_maps(g, &tmA, &tmB, Cfg::BN);
    if (rc != NZB_OK) return rc;
    p.tiles_n = (int32_t)((g.N + Cfg::BN - 1) / Cfg::BN);
    p.total_tiles = (int64_t)p.tiles_m * p.tiles_n * p.out_e0 * p.out_e1;
    static std::atomic<uint64_t> smem_set{0};  // per kernel instantiation, one bit per device
    {
        const int rc_attr = ensure_dynamic_smem(smem_set, reinterpret_cast<const void*>(gemm_f16_tcgen05_kernel<Cfg>), Cfg::SMEM_BYTES);
        if (rc_attr != NZB_OK) return rc_attr;
    }
    // Few output tiles but a long contraction: share each tile among several CTAs along k and
    // add the partial sums atomically (the first slice adds the bias; not with ReLU, which needs
    // the full sum).
    p.splits = 1;
    const int64_t k_iters = (int64_t)p.red_e0 * p.red_e1 * p.k_blocks;
    const int64_t slots = (int64_t)ds.sm_count * Cfg::MIN_BLOCKS;
    if (p.total_tiles * 2 <= slots && k_iters >= 16 && !p.relu) {
        int64_t sp = slots / p.total_tiles;
        if (sp > k_iters / 8) sp = k_iters / 8;
        if (sp > 1) {
            p.splits = (int32_t)sp;
            p.vec4 = 0;
            if (!p.accumulate) {
                // partial sums are added into C: start from zero
                for (int32_t b0 = 0; b0 < p.out_e0; b0++)
                    for (int32_t b1 = 0; b1 < p.out_e1; b1++)
                        NZB_CUDA_TRY(cudaMemset2DAsync(p.C + b0 * p.c_stride0 + b1 * p.c_stride1, (size_t)p.ldc * 4, 0,
                                                       (size_t)(p.trans_out ? p.M : p.N) * 4,
                                                       (size_t)(p.trans_out ? p.N : p.M), stream));
            }
        }
    }
    const int64_t items = p.total_tiles * p.splits;
    const int64_t grid = items < slots ? items : slots;
    gemm_f16_tcgen05_kernel<Cfg><<<(unsigned)grid, 192, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, p);
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}


// Describes one operand for the converter warps: K-major copies are staged by row panels, MN-major by
// column panels. `out_extent` is the operand's extent along the output dimension (M for A, N for B).
static FuseOperand fuse_operand(const float* src, int64_t ld_src, const __half* dst, int32_t mn, int64_t out_extent,
                                int64_t K, int64_t Kp, int64_t ld_mn) {
    FuseOperand o{};
    o.src = src;
    o.dst = const_cast<__half*>(dst);
    o.ld_src = ld_src;
    o.by_cols = mn ? 1 : 0;
    o.panels = (uint32_t)((out_extent + 255) / 256);
    if (mn) {  // stored K x extent
        o.rows = (int32_t)K; o.cols = (int32_t)out_extent; o.ld_dst = ld_mn;
        o.segs = 1;
        o.chunks_per_panel = (uint32_t)((K + kFuseChunk / 256 - 1) / (kFuseChunk / 256));
    } else {  // stored extent x K
        o.rows = (int32_t)out_extent; o.cols = (int32_t)K; o.ld_dst = Kp;
        o.segs = (uint32_t)((K + kFuseChunk - 1) / kFuseChunk);
        o.chunks_per_panel = 256 * o.segs;
    }
    return o;
}

static int launch_pair(const GemmLaunch& g, GemmParams& p, const DeviceState& ds, cudaStream_t stream) {
    CUtensorMap tmA, tmB;
    int rc = make_maps(g, &tmA, &tmB, 128);
    if (rc != NZB_OK) return rc;
    p.tiles_m = (int32_t)((g.M + 255) / 256);
    p.tiles_n = (int32_t)((g.N + 255) / 256);
    p.group_m = 8;  // groups of 4 and 16 tile rows were measured slower (L2 fit)
    p.splits = 1;
    p.total_tiles = (int64_t)p.tiles_m * p.tiles_n * p.out_e0 * p.out_e1;
    static std::atomic<uint64_t> smem_set[2];  // per kernel instantiation, one bit per device
    int64_t pairs = ds.sm_count / 2;
    if (p.total_tiles < pairs) pairs = p.total_tiles;
    FuseParams f{};
    if (g.fuse_sync) {
        rc = ensure_dynamic_smem(smem_set[1], reinterpret_cast<const void*>(gemm_f16_tcgen05_pair_kernel<true>),
                                 PairCfg::SMEM_BYTES);
        if (rc != NZB_OK) return rc;
        f.a = fuse_operand(g.A32, g.lda32, g.A16, g.a_mn, g.M, g.K, g.Kp, g.lda16);
        f.b = fuse_operand(g.B32, g.ldb32, g.B16, g.b_mn, g.N, g.K, g.Kp, g.ldb16);
        f.sync = g.fuse_sync;
        f.lead_a = (uint32_t)(p.tiles_m < p.group_m ? p.tiles_m : p.group_m);
        const uint64_t total = (uint64_t)f.a.panels * f.a.chunks_per_panel + (uint64_t)f.b.panels * f.b.chunks_per_panel;
        if (total >= 0xffffffffull || f.a.panels + f.b.panels > (uint64_t)kFuseMaxPanels)
            return fail(NZB_ERR_UNSUPPORTED, "operands too large for in-kernel staging");
        f.total_chunks = (uint32_t)total;
        gemm_f16_tcgen05_pair_kernel<true><<<(unsigned)(2 * pairs), 192 + 32 * kFuseWarps, PairCfg::SMEM_BYTES, stream>>>(tmA, tmB, p, f);
    } else {
        rc = ensure_dynamic_smem(smem_set[0], reinterpret_cast<const void*>(gemm_f16_tcgen05_pair_kernel<false>),
                                 PairCfg::SMEM_BYTES);
        if (rc != NZB_OK) return rc;
        gemm_f16_tcgen05_pair_kernel<false><<<(unsigned)(2 * pairs), 192, PairCfg::SMEM_BYTES, stream>>>(tmA, tmB, p, f);
    }
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}

// True when launch_gemm_on() would take the CTA-pair kernel for this launch (the only kernel that can
// stage its own operands).
bool gemm_uses_pair_kernel(const GemmLaunch& g, int sm_count) {
    if (g.M <= 128 || g.N <= 128 || g.force_single_cta) return false;
    if (g.M <= 32 && g.N >= 4 * g.M && g.N > 64) return false;
    const int64_t tiles1 = ((g.M + 127) / 128) * ((g.N + 255) / 256) * g.out_e[0] * g.out_e[1];
    const int64_t k_iters = (int64_t)g.red_e[0] * g.red_e[1] * ((g.K + 63) / 64);
    const bool want_split = tiles1 * 2 <= sm_count && k_iters >= 64 && !g.relu;
    return !want_split;
}

int launch_gemm(const GemmLaunch& g, cudaStream_t stream) {
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    return launch_gemm_on(g, *ds, stream);
}

int launch_gemm_on(const GemmLaunch& g_in, const DeviceState& dstate, cudaStream_t stream) {
    const DeviceState* ds = &dstate;
    if (g_in.M <= 0 || g_in.N <= 0) return NZB_OK;
    // A tile is 128 rows tall: with a handful of rows and a wide output almost all of the tile
    // (and of the epilogue) would be padding. Compute C^T instead -- the operands trade places,
    // which costs nothing because either one may be K-major or MN-major -- and let the
    // epilogue write the transposed tile.
    GemmLaunch g = g_in;
    const bool swap = g_in.M <= 32 && g_in.N >= 4 * g_in.M && g_in.N > 64;
    if (swap) {
        g.A16 = g_in.B16; g.B16 = g_in.A16;
        g.nA = g_in.nB; g.nB = g_in.nA;
        g.M = g_in.N; g.N = g_in.M;
        g.a_mn = g_in.b_mn; g.b_mn = g_in.a_mn;
        g.lda16 = g_in.ldb16; g.ldb16 = g_in.lda16;
        for (int k = 0; k < 2; k++) {
            g.a_mul[k] = g_in.b_mul[k];
            g.b_mul[k] = g_in.a_mul[k];
        }
    }
    if (g.K <= 0) return fail(NZB_ERR_UNSUPPORTED, "K = 0 is not supported");
    if (g.M > INT32_MAX - 256 || g.N > INT32_MAX - 256 || g.K > INT32_MAX - 256 || g.nA > INT32_MAX ||
        g.nB > INT32_MAX)
        return fail(NZB_ERR_UNSUPPORTED, "extent exceeds 2^31");
    GemmParams p{};
    p.C = g.C;
    p.ldc = g.ldc;
    p.M = (int32_t)g.M;
    p.N = (int32_t)g.N;
    p.K = (int32_t)g.K;
    p.tiles_m = (int32_t)((g.M + 127) / 128);
    p.out_e0 = g.out_e[0]; p.out_e1 = g.out_e[1];
    p.red_e0 = g.red_e[0]; p.red_e1 = g.red_e[1];
    p.a_mul0 = (int32_t)g.a_mul[0]; p.a_mul1 = (int32_t)g.a_mul[1];
    p.b_mul0 = (int32_t)g.b_mul[0]; p.b_mul1 = (int32_t)g.b_mul[1];
    p.c_stride0 = g.c_stride[0]; p.c_stride1 = g.c_stride[1];
    p.bias = g.bias;
    p.bias_ld = g.bias_ld;
    p.bias_mode = g.bias ? g.bias_mode : NZB_BIAS_NONE;
    p.accumulate = g.accumulate;
    p.relu = g.relu;
    p.k_blocks = (int32_t)((g.K + 63) / 64);
    p.last_ksteps = (int32_t)((g.K - (int64_t)(p.k_blocks - 1) * 64 + 15) / 16);
    p.status = ds->status_dev;
    p.alpha = g.alpha;
    bool v4 = (g.N % 4 == 0) && (g.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(g.C) & 15) == 0) &&
              (g.c_stride[0] % 4 == 0) && (g.c_stride[1] % 4 == 0);
    if (p.bias_mode == NZB_BIAS_ROW) v4 = v4 && ((reinterpret_cast<uintptr_t>(g.bias) & 15) == 0);
    if (p.bias_mode == NZB_BIAS_MATRIX)
        v4 = v4 && ((reinterpret_cast<uintptr_t>(g.bias) & 15) == 0) && (g.bias_ld % 4 == 0);
    p.vec4 = v4 ? 1 : 0;
    p.group_m = 16;
    p.a_mn = g.a_mn ? 1 : 0;
    p.b_mn = g.b_mn ? 1 : 0;
    p.trans_out = swap ? 1 : 0;
    if (g.a_mn && (g.lda16 < g.M || g.lda16 % 8 != 0)) return fail(NZB_ERR_BAD_ARG, "MN-major A copy needs a leading dimension >= M and a multiple of 8");
    if (g.b_mn && (g.ldb16 < g.N || g.ldb16 % 8 != 0)) return fail(NZB_ERR_BAD_ARG, "MN-major B copy needs a leading dimension >= N and a multiple of 8");

    {
        // few tiles and a long contraction: the single-CTA kernel can split k across CTAs
        const int64_t tiles1 = (int64_t)p.tiles_m * ((g.N + 255) / 256) * p.out_e0 * p.out_e1;
        const int64_t k_iters = (int64_t)p.red_e0 * p.red_e1 * p.k_blocks;
        const bool want_split = tiles1 * 2 <= ds->sm_count && k_iters >= 64 && !p.relu;
        (void)want_split;
        if (!swap && gemm_uses_pair_kernel(g, ds->sm_count)) return launch_pair(g, p, *ds, stream);
    }
    if (g.fuse_sync) return fail(NZB_ERR_UNSUPPORTED, "in-kernel staging was requested for a shape the CTA-pair kernel does not take");

    if (g.N > 128) return launch_cfg<GemmCfg<256, 4>>(g, p, *ds, stream);
    if (g.N > 64) return launch_cfg<GemmCfg<128, 6>>(g, p, *ds, stream);
    // an MN-major B tile is loaded in boxes of 64 columns: narrower outputs use the 64-wide tile
    if (g.N > 32 || g.b_mn) return launch_cfg<GemmCfg<64, 8>>(g, p, *ds, stream);
    if (g.N > 16) return launch_cfg<GemmCfg<32, 4, 2>>(g, p, *ds, stream);
    return launch_cfg<GemmCfg<16, 5, 2>>(g, p, *ds, stream);
}

}  // namespace nzb
