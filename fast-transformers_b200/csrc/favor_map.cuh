// Positive random features of the softmax kernel (Favor) in one pass on the tensor cores:
//
//   xs = x * temp^(1/2);  u = xs omega;  off = |xs|^2 / 2 + log(n) / 2;  phi = [exp(u - off), exp(-u - off)]
//
// (fast_transformers/feature_maps/fourier_features.py:218-243, without `stabilize`), for rows of
// E = 64 values and n = 2 * HALF features (HALF = 64 or 128).  The reference runs it as six torch
// kernels over (rows x n)-sized tensors; here a row tile is read once (32 KB), u = x omega is one
// 128 x HALF x 64 tcgen05 product (TF32 operands, fp32 accumulation in tensor memory) and the
// epilogue writes the n features of every row once.
//
// A persistent CTA loops over tiles of 128 rows.  Warp 0: TMA producer (omega^T once, then x tiles
// into a two-stage ring); warp 1: one elected thread issues the product of a tile into one of two
// TMEM accumulators; warps 2-5: epilogue -- every thread first takes the squared norm of one row
// from the tile in shared memory, then the accumulator is read in the 16x256b shape so that a warp
// store writes 8 rows x 32 bytes (whole sectors).  99 KB of shared memory and 256 TMEM columns per
// CTA: two CTAs per SM.  Every wait is bounded (mbar_wait): on expiry the CTA records
// FTB_ERR_TIMEOUT in the device status word and leaves.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mma_scan.cuh"

namespace ftb {
namespace favor {

using namespace ftb::mma;

constexpr int kRows = 128;                 // rows per tile
constexpr int kE = 64;                     // input width
constexpr int kThreads = 192;              // producer, issuer, four epilogue warps
constexpr int kBlk = kRows * 128;          // one [128 rows][128 B] swizzled block
constexpr int kTile = 2 * kBlk;            // a 128 x 64 fp32 tile: two blocks
constexpr size_t kSmem = 1024 + 3 * kTile + 2 * kRows * sizeof(float) + 256;

struct Params {
    float *out;
    int64_t rows;
    int64_t out_stride;   // elements between output rows (>= 2 * HALF)
    float scale;          // temp^(1/2)
    float half_temp;      // temp / 2
    float log_term;       // log(n) / 2
    int pos_x[3], pos_w[3];   // TMA coordinate slots of {position, head, batch} (mma::make_map)
};

// AND of `ok` over the 128 epilogue threads (named barrier 1): they leave their loop together.
__device__ __forceinline__ bool epilogue_all(bool ok) {
    uint32_t r;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.u32 q, %1, 0;\n"
        "bar.red.and.pred p, 1, 128, q;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(r)
        : "r"((uint32_t)ok)
        : "memory");
    return r != 0;
}

template <int HALF>
__global__ void __launch_bounds__(kThreads, 2)
favor_map_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const Params p) {
    static_assert(HALF == 64 || HALF == 128, "one product of N = 64 or 128 columns");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sm_w = base, sm_x = base + kTile;
    float *s_off = reinterpret_cast<float *>(gen + 3 * kTile);           // [2][kRows]
    const uint32_t bars = base + 3 * kTile + 2 * kRows * sizeof(float);
    const uint32_t bar_w = bars, bar_full = bars + 8, bar_empty = bars + 24, bar_ufull = bars + 40,
                   bar_ufree = bars + 56;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + 3 * kTile + 2 * kRows * sizeof(float) + 128);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + 3 * kTile + 2 * kRows * sizeof(float) + 136);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t ntiles = (p.rows + kRows - 1) / kRows;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar_w, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1 + 128);   // the product has read the tile, and so have the norms
            mbar_init(bar_ufull + 8 * s, 1);
            mbar_init(bar_ufree + 8 * s, 128);
        }
        fence_barrier_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            mbar_expect_tx(bar_w, kTile);
            for (int b = 0; b < 2; ++b) tma_load_4d(sm_w + b * kBlk, &map_w, bar_w, b * 32, p.pos_w, 0, 0, 0);
            int it = 0;
            for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
                const int s = it & 1;
                if (!mbar_wait(bar_empty + 8 * s, ((it >> 1) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(bar_full + 8 * s, kTile);
                for (int b = 0; b < 2; ++b)
                    tma_load_4d(sm_x + s * kTile + b * kBlk, &map_x, bar_full + 8 * s, b * 32, p.pos_x,
                                (int)(t * kRows), 0, 0);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t ID = instr_desc(2 /* tf32 */, 0, 0, 128, HALF);
            const uint64_t dW = smem_desc(sm_w, 16, 1024);
            bool ok = mbar_wait(bar_w, 0, abort_flag);
            int it = 0;
            for (int64_t t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++it) {
                const int s = it & 1;
                ok = mbar_wait(bar_full + 8 * s, (it >> 1) & 1, abort_flag) &&
                     mbar_wait(bar_ufree + 8 * s, ((it >> 1) & 1) ^ 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint64_t dX = smem_desc(sm_x + s * kTile, 16, 1024);
#pragma unroll
                for (int b = 0; b < 2; ++b)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t off = (uint64_t)((b * kBlk + k * 32) >> 4);
                        mma_ss<false>(tmem + 128 * s, dX + off, dW + off, ID, (b | k) ? 1u : 0u);
                    }
                tc_commit(bar_ufull + 8 * s);
                tc_commit(bar_empty + 8 * s);
            }
        }
    } else {
        // ---- epilogue: thread i = row i of the tile for the norms; 16x256b fragments for the stores
        const int q = warp & 3;
        const int i = 32 * q + lane;
        const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
        uint32_t r[32];
        int it = 0;
        for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
            const int s = it & 1;
            bool ok = mbar_wait(bar_full + 8 * s, (it >> 1) & 1, abort_flag);
            if (ok) {
                // |x_i|^2 from the swizzled tile: 16-byte chunk c of row r sits at c ^ (r & 7)
                const uint8_t *xt = gen + kTile + s * kTile;
                float n2 = 0.f;
#pragma unroll
                for (int b = 0; b < 2; ++b)
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const float4 v = *reinterpret_cast<const float4 *>(xt + b * kBlk + i * 128 + ((c ^ (i & 7)) << 4));
                        n2 += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                    }
                s_off[s * kRows + i] = n2 * p.half_temp + p.log_term;
            }
            mbar_arrive(bar_empty + 8 * s);
            if (!epilogue_all(ok)) break;                 // (also: the offsets are visible to all four warps)
            ok = mbar_wait(bar_ufull + 8 * s, (it >> 1) & 1, abort_flag);
            if (ok) {
                tc_fence_after();
                const int64_t row0 = t * kRows;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const int ra = 32 * q + 16 * hf + (lane >> 2);
                    const float offa = s_off[s * kRows + ra], offb = s_off[s * kRows + ra + 8];
                    float *da = p.out + (row0 + ra) * p.out_stride + 2 * (lane & 3);
                    float *db = da + 8 * p.out_stride;
                    const bool oka = row0 + ra < p.rows, okb = row0 + ra + 8 < p.rows;
#pragma unroll
                    for (int cb = 0; cb < HALF / 64; ++cb) {
                        tmem_ld16x256(tlane + ((uint32_t)(16 * hf) << 16) + 128 * s + 64 * cb, r);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int col = 64 * cb + 8 * j;
                            const float u0 = p.scale * __uint_as_float(r[4 * j]), u1 = p.scale * __uint_as_float(r[4 * j + 1]);
                            const float u2 = p.scale * __uint_as_float(r[4 * j + 2]), u3 = p.scale * __uint_as_float(r[4 * j + 3]);
                            if (oka) {
                                *reinterpret_cast<float2 *>(da + col) = make_float2(__expf(u0 - offa), __expf(u1 - offa));
                                *reinterpret_cast<float2 *>(da + HALF + col) = make_float2(__expf(-u0 - offa), __expf(-u1 - offa));
                            }
                            if (okb) {
                                *reinterpret_cast<float2 *>(db + col) = make_float2(__expf(u2 - offb), __expf(u3 - offb));
                                *reinterpret_cast<float2 *>(db + HALF + col) = make_float2(__expf(-u2 - offb), __expf(-u3 - offb));
                            }
                        }
                    }
                }
                tc_fence_before();
            }
            mbar_arrive(bar_ufree + 8 * s);
            if (!epilogue_all(ok)) break;                 // (also: s_off[s] is rewritten two tiles from now)
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------
// The map's backward in one pass.  With phi = [p, m] (the forward's output) and g its gradient,
//
//   grad_u = g_p p - g_m m        grad_off = -sum(g phi)
//   grad_x = temp^(1/2) (grad_u omega^T) + temp grad_off x
//
// (the chain rule through fourier_features.py:218-243).  A persistent CTA loops over tiles of 128
// rows; a tile is HALF / 32 steps of 32 features.  Warp 0: TMA producer (omega once; per step the
// four blocks g_p | g_m | p | m of 128 rows x 32 columns into a two-stage ring; per tile the x
// tile); warps 2-5: element-wise workers -- grad_u of the step into an operand block (the swizzle
// of source and destination is the same, so a 16-byte piece keeps its place) and the row sums of
// g phi in registers; warp 1: one elected thread issues grad_u omega^T of the step (128 x 64 x 32,
// TF32, accumulated over the steps in one of two TMEM accumulators); after the last step the
// workers combine the accumulator, the row sums and x and store grad_x.  HBM-bound: (2 n + 128)
// floats per row.  Every wait is bounded.
constexpr int kBwdThreads = 192;
constexpr int kRingStage = 4 * kBlk;                       // g_p | g_m | p | m
constexpr int kUOff = 2 * kRingStage;                      // two grad_u operand blocks
constexpr int kWOff = kUOff + 2 * kBlk;                    // omega: HALF / 32 blocks of [64 rows][128 B]
constexpr int kWBlk = kE * 128;
constexpr int kXOff = kWOff + 4 * kWBlk;                   // the x tile
constexpr int kSumOff = kXOff + kTile;                     // 128 row sums
constexpr int kBwdBarOff = kSumOff + kRows * (int)sizeof(float);
constexpr size_t kSmemBwd = 1024 + kBwdBarOff + 256;

struct BwdParams {
    float *grad_x;
    int64_t rows;
    int64_t gx_stride;
    float scale;          // temp^(1/2)
    float temp;
    int pos_g[3], pos_p[3], pos_x[3];
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

template <int HALF>
__global__ void __launch_bounds__(kBwdThreads, 1)
favor_map_backward_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_p,
                          const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                          const BwdParams p) {
    static_assert(HALF == 64 || HALF == 128, "two or four steps of 32 features");
    constexpr int NKB = HALF / 32;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    float *s_sum = reinterpret_cast<float *>(gen + kSumOff);
    const uint32_t bars = base + kBwdBarOff;
    const uint32_t bar_full = bars, bar_empty = bars + 16, bar_ufull = bars + 32, bar_ufree = bars + 48,
                   bar_accfull = bars + 64, bar_accfree = bars + 80, bar_w = bars + 96, bar_xfull = bars + 104,
                   bar_xempty = bars + 112;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + kBwdBarOff + 128);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + kBwdBarOff + 136);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t ntiles = (p.rows + kRows - 1) / kRows;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 128);
            mbar_init(bar_ufull + 8 * s, 128);
            mbar_init(bar_ufree + 8 * s, 1);
            mbar_init(bar_accfull + 8 * s, 1);
            mbar_init(bar_accfree + 8 * s, 128);
        }
        mbar_init(bar_w, 1);
        mbar_init(bar_xfull, 1);
        mbar_init(bar_xempty, 128);
        fence_barrier_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), 128);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            mbar_expect_tx(bar_w, NKB * kWBlk);
            for (int kb = 0; kb < NKB; ++kb) tma_load_2d(base + kWOff + kb * kWBlk, &map_w, bar_w, 32 * kb, 0);
            int step = 0, it = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++it) {
                const int row = (int)(t * kRows);
                for (int kb = 0; kb < NKB && ok; ++kb, ++step) {
                    const int s = step & 1;
                    ok = mbar_wait(bar_empty + 8 * s, ((step >> 1) & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    const uint32_t st = base + s * kRingStage;
                    mbar_expect_tx(bar_full + 8 * s, kRingStage);
                    tma_load_4d(st, &map_g, bar_full + 8 * s, 32 * kb, p.pos_g, row, 0, 0);
                    tma_load_4d(st + kBlk, &map_g, bar_full + 8 * s, HALF + 32 * kb, p.pos_g, row, 0, 0);
                    tma_load_4d(st + 2 * kBlk, &map_p, bar_full + 8 * s, 32 * kb, p.pos_p, row, 0, 0);
                    tma_load_4d(st + 3 * kBlk, &map_p, bar_full + 8 * s, HALF + 32 * kb, p.pos_p, row, 0, 0);
                }
                // x is read after the last step only: requested last, so that the wait for the
                // previous tile's epilogue (which still reads the single x tile) holds up nothing
                if (!ok || !mbar_wait(bar_xempty, (it & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(bar_xfull, kTile);
                for (int b = 0; b < 2; ++b)
                    tma_load_4d(base + kXOff + b * kBlk, &map_x, bar_xfull, 32 * b, p.pos_x, row, 0, 0);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t ID = instr_desc(2 /* tf32 */, 0, 0, 128, kE);
            bool ok = mbar_wait(bar_w, 0, abort_flag);
            int step = 0, it = 0;
            for (int64_t t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++it) {
                const int ab = it & 1;
                ok = mbar_wait(bar_accfree + 8 * ab, ((it >> 1) & 1) ^ 1, abort_flag);
                for (int kb = 0; kb < NKB && ok; ++kb, ++step) {
                    const int ub = step & 1;
                    ok = mbar_wait(bar_ufull + 8 * ub, (step >> 1) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t dU = smem_desc(base + kUOff + ub * kBlk, 16, 1024);
                    const uint64_t dW = smem_desc(base + kWOff + kb * kWBlk, 16, 1024);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mma_ss<false>(tmem + 64 * ab, dU + (uint64_t)((k * 32) >> 4), dW + (uint64_t)((k * 32) >> 4), ID,
                                      (kb | k) ? 1u : 0u);
                    tc_commit(bar_ufree + 8 * ub);
                    if (kb + 1 == NKB) tc_commit(bar_accfull + 8 * ab);
                }
            }
        }
    } else {
        // ---- workers: 128 threads; piece idx = i * 128 + t of a block is 16 bytes of row idx / 8 ----
        const int t = threadIdx.x - 64;
        const int q = warp & 3;
        const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
        int step = 0, it = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++it) {
            float ssum[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) ssum[i] = 0.f;
            for (int kb = 0; kb < NKB && ok; ++kb, ++step) {
                const int s = step & 1;
                ok = mbar_wait(bar_full + 8 * s, (step >> 1) & 1, abort_flag) &&
                     mbar_wait(bar_ufree + 8 * s, ((step >> 1) & 1) ^ 1, abort_flag);
                if (!ok) break;
                const uint8_t *src = gen + s * kRingStage;
                uint8_t *dst = gen + kUOff + s * kBlk;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int off = (i * 128 + t) * 16;
                    const float4 gp = *reinterpret_cast<const float4 *>(src + off);
                    const float4 gm = *reinterpret_cast<const float4 *>(src + kBlk + off);
                    const float4 pp = *reinterpret_cast<const float4 *>(src + 2 * kBlk + off);
                    const float4 pm = *reinterpret_cast<const float4 *>(src + 3 * kBlk + off);
                    const float4 a = make_float4(gp.x * pp.x, gp.y * pp.y, gp.z * pp.z, gp.w * pp.w);
                    const float4 b = make_float4(gm.x * pm.x, gm.y * pm.y, gm.z * pm.z, gm.w * pm.w);
                    ssum[i] += (a.x + b.x) + (a.y + b.y) + (a.z + b.z) + (a.w + b.w);
                    *reinterpret_cast<float4 *>(dst + off) = make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w);
                }
                fence_proxy_async_smem();
                mbar_arrive(bar_ufull + 8 * s);
                mbar_arrive(bar_empty + 8 * s);
            }
            if (!epilogue_all(ok)) break;
            // row sums: the eight threads of a row are neighbours (t & 7 = position inside the row)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float v = ssum[i];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if ((t & 7) == 0) s_sum[i * 16 + (t >> 3)] = v;
            }
            const int ab = it & 1;
            ok = mbar_wait(bar_accfull + 8 * ab, (it >> 1) & 1, abort_flag) &&
                 mbar_wait(bar_xfull, it & 1, abort_flag);
            if (!epilogue_all(ok)) break;                  // (also: the row sums are visible to all four warps)
            tc_fence_after();
            const int64_t row0 = tile * kRows;
            const uint8_t *xt = gen + kXOff;
            uint32_t r[32];
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                tmem_ld16x256(tlane + ((uint32_t)(16 * hf) << 16) + 64 * ab, r);
                const int ra = 32 * q + 16 * hf + (lane >> 2), rb = ra + 8;
                const float ca = -p.temp * s_sum[ra], cb = -p.temp * s_sum[rb];
                float *da = p.grad_x + (row0 + ra) * p.gx_stride + 2 * (lane & 3);
                float *db = da + 8 * p.gx_stride;
                const bool oka = row0 + ra < p.rows, okb = row0 + rb < p.rows;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int col = 8 * j + 2 * (lane & 3);          // columns col, col + 1 of rows ra and rb
                    const int blk = col >> 5, cc = col & 31;
                    const float2 xa = *reinterpret_cast<const float2 *>(
                        xt + blk * kBlk + ra * 128 + (((cc >> 2) ^ (ra & 7)) << 4) + (cc & 3) * 4);
                    const float2 xb = *reinterpret_cast<const float2 *>(
                        xt + blk * kBlk + rb * 128 + (((cc >> 2) ^ (rb & 7)) << 4) + (cc & 3) * 4);
                    if (oka)
                        *reinterpret_cast<float2 *>(da + 8 * j) =
                            make_float2(p.scale * __uint_as_float(r[4 * j]) + ca * xa.x,
                                        p.scale * __uint_as_float(r[4 * j + 1]) + ca * xa.y);
                    if (okb)
                        *reinterpret_cast<float2 *>(db + 8 * j) =
                            make_float2(p.scale * __uint_as_float(r[4 * j + 2]) + cb * xb.x,
                                        p.scale * __uint_as_float(r[4 * j + 3]) + cb * xb.y);
                }
            }
            tc_fence_before();
            mbar_arrive(bar_accfree + 8 * ab);
            mbar_arrive(bar_xempty);
            if (!epilogue_all(true)) break;                // (s_sum is rewritten by the next tile)
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

}  // namespace favor
}  // namespace ftb
