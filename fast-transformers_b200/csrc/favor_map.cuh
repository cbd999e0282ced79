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

}  // namespace favor
}  // namespace ftb
