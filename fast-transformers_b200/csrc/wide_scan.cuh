// Tensor-core segment scan for a WIDE feature dimension on the a / b side: D = 64 nb (nb <= 4),
// 64 value columns, fp32 data with TF32 operands.  With (a, b, c) = (Q, K, V) -- or (K, Q, grad_out)
// walked downwards for grad_V --
//
//   out_c = sum_blk [ a_c,blk S_blk ] + mask( sum_blk a_c,blk b_c,blk^T ) c_c ;   S_blk += b_c,blk^T c_c
//
// so the sum over the nb 64-wide feature blocks is taken INSIDE the tensor cores: the scores and
// the output accumulate over the blocks in tensor memory, the mask runs once per chunk, c is
// loaded once per chunk and out is written once -- where nb separate scans of the blocks (the
// other way to run this shape) each read c and read-modify-write out.
//
// One CTA walks one segment of one (batch, head) pair; its unit of work is a "step" = (chunk of
// 128 rows, feature block): step v = chunk * nb + blk.
//
//   shared memory   two stages of {a_blk | b_blk} (64 KB each), two c tiles (32 KB each), two
//                   operand images of a 64 x 64 state block (16 KB each)
//   tensor memory   P: 128 columns; O: 2 x 64; S_0 .. S_3: 64 each, accumulated in place (fp32)
//
// Warp roles as in the 64-wide scan (mma_scan.cuh): 0 = TMA producer, 1 = output issuer
// (O += a S_blk every step, O += mask(P) c after the last block), 10 = score / state issuer
// (P += a b^T, S_blk += b^T c), 2-5 = state workers (S_blk -> operand image of the step that needs
// it next), 6-9 = output workers (MN-major image of b in place after the score product; O rows ->
// global memory), 11-14 = mask workers.  Every wait is bounded (mbar_wait): on expiry the CTA
// records FTB_ERR_TIMEOUT in the device status word, stops issuing work, frees its tensor memory
// and returns.
//
// Maths: fast_transformers/causal_product/causal_product_cpu.cpp:106-121 (forward) and :165-206
// (grad_V) in blocks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mma_scan.cuh"

namespace ftb {
namespace wide {

using namespace ftb::mma;

constexpr int MAXNB = 4;
constexpr int kBlk = C * 128;          // one [128 rows][128 B] swizzled block
constexpr int kTile = 2 * kBlk;        // 128 x 64 fp32
constexpr int kStage = 2 * kTile;      // a_blk | b_blk
constexpr int kImgBlk = 64 * 128;      // state operand: [64 rows][128 B] per 32 columns
constexpr int kImg = 2 * kImgBlk;
constexpr int kRing = 2 * kStage, kCOff = kRing, kImgOff = kRing + 2 * kTile, kBarOff = kImgOff + 2 * kImg;
constexpr size_t kSmem = 1024 + kBarOff + 512;
constexpr int TM_P = 0, TM_O = 128, TM_S = 256;

struct Params {
    float *out;
    Strides3 so;
    int H;
    int64_t L;
    int64_t seg_len;      // multiple of C
    int nseg;
    int nb;               // feature blocks (2 .. MAXNB)
    const float *states;  // per (bh, seg) blocks [64 nb rows of a / b][columns of c] (see state_ld,
                          // state_transposed), or nullptr
    int sum_mode;         // as mma::ScanParams
    int sub;
    int64_t state_blk;    // floats between consecutive (bh, seg) blocks
    int64_t state_ld;     // floats between consecutive rows of a stored block (its full width)
    int state_transposed; // the stored block holds [column of c][row of a / b] instead
    int reverse;
    int accumulate;       // add to what `out` holds
    int wait_first;       // programmatic launch: wait for the grid in front before any global access
    int pos_a[3], pos_b[3], pos_c[3];
};

// ---- pieces both kernels of this file share ------------------------------------------------------
// MN-major image of a 128 x 64 fp32 tile, in place: 16-byte chunk c of row r moves from its place in
// the 128-byte swizzle (c ^ (r & 7)) to its place in the 32-byte-atom swizzle.  `t`: 0..127 within
// the four warps that share the tile; a warp instruction covers four whole rows.
__device__ __forceinline__ void rearrange_tile_in_place(uint8_t *bt, int t) {
    for (int it0 = 0; it0 < 16; it0 += 4) {
        uint4 vv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int idx = (it0 + j) * 128 + t;
            vv[j] = reinterpret_cast<const uint4 *>(bt + (size_t)(idx >> 3) * 128)[idx & 7];
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int idx = (it0 + j) * 128 + t;
            const int pk = idx & 7, row = (idx >> 3) & 127;
            const int cc = pk ^ (row & 7);
            const int pm = ((((cc >> 1) ^ (row & 3)) << 1) | (cc & 1));
            reinterpret_cast<uint4 *>(bt + (size_t)(idx >> 3) * 128)[pm] = vv[j];
        }
        __syncwarp();
    }
    fence_proxy_async_smem();
}

// Causal mask on the 128 x 128 scores at `tP` (this warp's lane quarter q), in place: column blocks
// of 32 on the far side of the diagonal are zeroed, the diagonal block element by element.
__device__ __forceinline__ void mask_scores_in_place(uint32_t tP, int q, int lane, int reverse) {
    uint32_t r[32];
    const int nkeep = reverse ? 3 - q : q;
    tmem_zero_columns(tP + (reverse ? 0 : 32 * (q + 1)), 32 * (3 - nkeep));
    tmem_ld32(tP + 32 * q, r);
#pragma unroll
    for (int e = 0; e < 32; ++e) {
        const bool keep = reverse ? (e >= lane) : (e <= lane);
        r[e] = keep ? r[e] : 0u;
    }
    tmem_st32(tP + 32 * q, r);
    tmem_wait_st();
}

// The 64 x 64 state accumulator at `tS` (this warp's lane quarter) -> operand image `img` (read
// MN-major by "a S"): 64-row accumulators keep their rows in 16 lanes per quarter.
__device__ __forceinline__ void state_to_image(uint32_t tS, uint8_t *img, int lane, int q) {
    uint32_t r[32];
    const int srow = 16 * q + (lane & 15);
#pragma unroll
    for (int cb = 0; cb < 2; ++cb) {
        tmem_ld32(tS + 32 * cb, r);
        if (lane < 16) {
            uint8_t *rowp = img + cb * kImgBlk + srow * 128;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
                *reinterpret_cast<uint4 *>(rowp + (((ch >> 1) ^ (srow & 3)) * 32) + (ch & 1) * 16) =
                    make_uint4(r[4 * ch], r[4 * ch + 1], r[4 * ch + 2], r[4 * ch + 3]);
        }
    }
    fence_proxy_async_smem();
}

__global__ void __launch_bounds__(NTHREADS, 1)
wide_scan_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, const Params p) {
    if (!p.wait_first) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + kBarOff;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + kBarOff + 384);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + kBarOff + 392);
    // barriers (8 bytes each; [2] = one per stage / buffer, [4] = one per feature block)
    const uint32_t bar_full = bars, bar_empty = bars + 16, bar_sdone = bars + 32, bar_fullbmn = bars + 48,
                   bar_cfull = bars + 64, bar_cempty = bars + 80, bar_ofull = bars + 96, bar_ofree = bars + 112,
                   bar_smready = bars + 128, bar_smready2 = bars + 144, bar_smfree = bars + 160,
                   bar_pfull = bars + 176, bar_pready = bars + 184, bar_pfree = bars + 192,
                   bar_sfull = bars + 200;   // [4]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = p.nb;
    const int seg = (int)(blockIdx.x % (unsigned)p.nseg);
    const int64_t bh = blockIdx.x / (unsigned)p.nseg;
    const int bn = (int)(bh / p.H), bhh = (int)(bh % p.H);
    const int64_t seg_begin = (int64_t)seg * p.seg_len;
    const int64_t seg_end = min(p.L, seg_begin + p.seg_len);
    int nchunk = (int)((seg_end - seg_begin + C - 1) / C);
    if (nchunk < 0) nchunk = 0;
    const int nstep = nchunk * nb;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 2);      // both issuers
            mbar_init(bar_sdone + 8 * s, 1);
            mbar_init(bar_fullbmn + 8 * s, 128);
            mbar_init(bar_cfull + 8 * s, 1);
            mbar_init(bar_cempty + 8 * s, 2);     // both issuers
            mbar_init(bar_ofull + 8 * s, 1);
            mbar_init(bar_ofree + 8 * s, 128);
            mbar_init(bar_smready + 8 * s, 128);
            mbar_init(bar_smready2 + 8 * s, 128);
            mbar_init(bar_smfree + 8 * s, 1);
        }
        mbar_init(bar_pfull, 1);
        mbar_init(bar_pready, 128);
        mbar_init(bar_pfree, 1);
        for (int b = 0; b < MAXNB; ++b) mbar_init(bar_sfull + 8 * b, 1);
        fence_barrier_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (p.wait_first) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }

    if (nchunk > 0) {
        if (warp == 0) {
            // ================= TMA producer =====================================================
            if (elect_one()) {
                bool ok = true;
                for (int v = 0; v < nstep && ok; ++v) {
                    const int ci = v / nb, blk = v - ci * nb;
                    const int c = p.reverse ? nchunk - 1 - ci : ci;
                    const int row = (int)(seg_begin + (int64_t)c * C);
                    if (blk == 0) {
                        const int cb = ci & 1;
                        ok = mbar_wait(bar_cempty + 8 * cb, ((ci >> 1) & 1) ^ 1, abort_flag);
                        if (!ok) break;
                        mbar_expect_tx(bar_cfull + 8 * cb, kTile);
                        for (int b = 0; b < 2; ++b)
                            tma_load_4d(base + kCOff + cb * kTile + b * kBlk, &map_c, bar_cfull + 8 * cb, 32 * b,
                                        p.pos_c, row, bhh, bn);
                    }
                    const int s = v & 1;
                    ok = mbar_wait(bar_empty + 8 * s, ((v >> 1) & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    const uint32_t st = base + s * kStage;
                    mbar_expect_tx(bar_full + 8 * s, kStage);
                    for (int b = 0; b < 2; ++b) {
                        tma_load_4d(st + b * kBlk, &map_a, bar_full + 8 * s, 64 * blk + 32 * b, p.pos_a, row, bhh, bn);
                        tma_load_4d(st + kTile + b * kBlk, &map_b, bar_full + 8 * s, 64 * blk + 32 * b, p.pos_b, row,
                                    bhh, bn);
                    }
                }
            }
        } else if (warp == 1 || warp == 10) {
            // ================= MMA issuers ======================================================
            if (elect_one()) {
                constexpr uint32_t ID_P = instr_desc(2, 0, 0, 128, 128);
                constexpr uint32_t ID_AS = instr_desc(2, 0, 1, 128, 64);
                constexpr uint32_t ID_PC = instr_desc(2, 0, 1, 128, 64);
                constexpr uint32_t ID_ST = instr_desc(2, 1, 1, 64, 64);
                constexpr uint64_t STAGE_UNITS = (uint64_t)(kStage >> 4), TILE_UNITS = (uint64_t)(kTile >> 4),
                                   IMG_UNITS = (uint64_t)(kImg >> 4);
                const uint64_t dAk0 = smem_desc(base, 16, 1024);
                const uint64_t dBk0 = smem_desc(base + kTile, 16, 1024);
                const uint64_t dBmn0 = smem_desc(base + kTile, kBlk, 512, 1);
                const uint64_t dCmn0 = smem_desc(base + kCOff, kBlk, 512, 1);
                const uint64_t dSm0 = smem_desc(base + kImgOff, kImgBlk, 512, 1);
                bool ok = true;
                if (warp == 1) {
                    // ---- output issuer: O += a S_blk every step; O += mask(P) c after the last block
                    for (int v = 0; v < nstep && ok; ++v) {
                        const int ci = v / nb, blk = v - ci * nb;
                        const int s = v & 1, ob = ci & 1, cb = ci & 1;
                        const uint32_t tO = tmem + TM_O + 64 * ob;
                        ok = mbar_wait(bar_full + 8 * s, (v >> 1) & 1, abort_flag) &&
                             mbar_wait(bar_smready + 8 * s, (v >> 1) & 1, abort_flag) &&
                             (blk != 0 || mbar_wait(bar_ofree + 8 * ob, ((ci >> 1) & 1) ^ 1, abort_flag));
                        if (!ok) break;
                        tc_fence_after();
                        const uint64_t a0 = dAk0 + s * STAGE_UNITS, sm0 = dSm0 + s * IMG_UNITS;
#pragma unroll
                        for (int b = 0; b < 2; ++b)
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                mma_ss<false>(tO, a0 + (uint64_t)((b * kBlk + k * 32) >> 4),
                                              sm0 + (uint64_t)(((32 * b + 8 * k) * 128) >> 4), ID_AS,
                                              (blk | b | k) ? 1u : 0u);
                        tc_commit(bar_smfree + 8 * s);
                        if (blk + 1 < nb) {
                            tc_commit(bar_empty + 8 * s);
                            continue;
                        }
                        ok = mbar_wait(bar_pready, ci & 1, abort_flag) &&
                             mbar_wait(bar_cfull + 8 * cb, (ci >> 1) & 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        const uint64_t c0 = dCmn0 + cb * TILE_UNITS;
#pragma unroll
                        for (int k = 0; k < 16; ++k)
                            mma_ts<false>(tO, tmem + TM_P + k * 8, c0 + (uint64_t)((k * 1024) >> 4), ID_PC, 1u);
                        tc_commit(bar_ofull + 8 * ob);
                        tc_commit(bar_pfree);
                        tc_commit(bar_empty + 8 * s);
                        tc_commit(bar_cempty + 8 * cb);
                    }
                } else {
                    // ---- score / state issuer: two queues, served as their inputs arrive ----------
                    int sc = 0, ds = 0;
                    long long t0 = 0;
                    uint32_t idle = 0;
                    while (ds < nstep) {
                        if (sc < nstep && sc <= ds + 1) {
                            const int ci = sc / nb, blk = sc - ci * nb, s = sc & 1;
                            if (mbar_test(bar_full + 8 * s, (sc >> 1) & 1) &&
                                (blk != 0 || ci == 0 || mbar_test(bar_pfree, (ci - 1) & 1))) {
                                tc_fence_after();
                                const uint64_t a0 = dAk0 + s * STAGE_UNITS, b0 = dBk0 + s * STAGE_UNITS;
#pragma unroll
                                for (int b = 0; b < 2; ++b)
#pragma unroll
                                    for (int k = 0; k < 4; ++k) {
                                        const uint64_t off = (uint64_t)((b * kBlk + k * 32) >> 4);
                                        mma_ss<false>(tmem + TM_P, a0 + off, b0 + off, ID_P, (blk | b | k) ? 1u : 0u);
                                    }
                                tc_commit(bar_sdone + 8 * s);
                                if (blk + 1 == nb) tc_commit(bar_pfull);
                                ++sc;
                                idle = 0;
                                continue;
                            }
                        }
                        if (ds < sc) {
                            const int ci = ds / nb, blk = ds - ci * nb, s = ds & 1, cb = ci & 1;
                            if (mbar_test(bar_fullbmn + 8 * s, (ds >> 1) & 1) &&
                                mbar_test(bar_cfull + 8 * cb, (ci >> 1) & 1) &&
                                mbar_test(bar_smready2 + 8 * s, (ds >> 1) & 1)) {
                                tc_fence_after();
                                const uint64_t bmn0 = dBmn0 + s * STAGE_UNITS, c0 = dCmn0 + cb * TILE_UNITS;
#pragma unroll
                                for (int k = 0; k < 16; ++k) {
                                    const uint64_t off = (uint64_t)((k * 1024) >> 4);
                                    mma_ss<false>(tmem + TM_S + 64 * blk, bmn0 + off, c0 + off, ID_ST, 1u);
                                }
                                tc_commit(bar_sfull + 8 * blk);
                                tc_commit(bar_empty + 8 * s);
                                if (blk + 1 == nb) tc_commit(bar_cempty + 8 * cb);
                                ++ds;
                                idle = 0;
                                continue;
                            }
                        }
                        if (idle++ == 0) t0 = clock64();
                        if ((idle & 63u) == 0u) {
                            if (*abort_flag) break;
                            if (clock64() - t0 > 4000000000LL) {
                                *abort_flag = 1;
                                atomicExch(&g_device_status, 5 /* FTB_ERR_TIMEOUT */);
                                break;
                            }
                        }
                    }
                }
            }
        } else if (warp >= 11) {
            // ================= mask workers: once per chunk, in place =============================
            const int q = warp & 3;
            const uint32_t tP = tmem + ((uint32_t)(32 * q) << 16) + TM_P;
            for (int ci = 0; ci < nchunk; ++ci) {
                if (!mbar_wait(bar_pfull, ci & 1, abort_flag)) break;
                tc_fence_after();
                mask_scores_in_place(tP, q, lane, p.reverse);
                tc_fence_before();
                mbar_arrive(bar_pready);
            }
        } else if (warp >= 6 && warp < 10) {
            // ================= output workers ====================================================
            const int q = warp & 3;
            const int t = threadIdx.x - 192;
            const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
            uint32_t r[32];
            bool ok = true;
            float *O = p.out + (int64_t)bn * p.so.n + (int64_t)bhh * p.so.h;
            // the rows of chunk `ci` from accumulator ci & 1 to global memory
            auto write_chunk = [&](int ci) -> bool {
                const int c = p.reverse ? nchunk - 1 - ci : ci;
                const int64_t row0 = seg_begin + (int64_t)c * C;
                const int ob = ci & 1;
                float2 old[2][16];
                if (p.accumulate) {
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        const int64_t ra = row0 + 32 * q + 16 * hf + (lane >> 2);
                        const float *da = O + ra * p.so.l + 2 * (lane & 3);
                        const float *db = da + 8 * p.so.l;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            old[hf][2 * j] = ra < seg_end ? *reinterpret_cast<const float2 *>(da + 8 * j) : make_float2(0.f, 0.f);
                            old[hf][2 * j + 1] = ra + 8 < seg_end ? *reinterpret_cast<const float2 *>(db + 8 * j) : make_float2(0.f, 0.f);
                        }
                    }
                }
                if (!mbar_wait(bar_ofull + 8 * ob, (ci >> 1) & 1, abort_flag)) return false;
                tc_fence_after();
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    tmem_ld16x256(tlane + ((uint32_t)(16 * hf) << 16) + TM_O + 64 * ob, r);
                    const int64_t ra = row0 + 32 * q + 16 * hf + (lane >> 2);
                    float *da = O + ra * p.so.l + 2 * (lane & 3);
                    float *db = da + 8 * p.so.l;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float2 va = make_float2(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]));
                        float2 vb = make_float2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                        if (p.accumulate) {
                            va.x += old[hf][2 * j].x; va.y += old[hf][2 * j].y;
                            vb.x += old[hf][2 * j + 1].x; vb.y += old[hf][2 * j + 1].y;
                        }
                        if (ra < seg_end) *reinterpret_cast<float2 *>(da + 8 * j) = va;
                        if (ra + 8 < seg_end) *reinterpret_cast<float2 *>(db + 8 * j) = vb;
                    }
                }
                tc_fence_before();
                mbar_arrive(bar_ofree + 8 * ob);
                return true;
            };
            for (int v = 0; v < nstep && ok; ++v) {
                const int ci = v / nb, blk = v - ci * nb, s = v & 1;
                // MN-major image of b_blk, in place, once the score product has read the tile:
                // 16-byte chunk c of row r moves from c ^ (r & 7) to the 32-byte-atom position
                ok = mbar_wait(bar_sdone + 8 * s, (v >> 1) & 1, abort_flag);
                if (!ok) break;
                rearrange_tile_in_place(gen + s * kStage + kTile, t);
                mbar_arrive(bar_fullbmn + 8 * s);
                // the rows of the previous chunk (its accumulator completes a mask later than the
                // score product of its last block: written here, it does not hold up the image)
                if (blk == 0 && ci > 0) ok = write_chunk(ci - 1);
            }
            if (ok) write_chunk(nchunk - 1);
        } else if (warp >= 2 && warp < 6) {
            // ================= state workers ======================================================
            const int q = warp & 3;
            const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
            const bool srow_ok = lane < 16;                 // 64-row accumulators: 16 lanes per quarter
            const int srow = 16 * q + (lane & 15);
            uint32_t r[32];
            bool ok = true;
            // ---- segment-start states -> tensor memory ------------------------------------------
            {
                int s_lo = seg, s_hi = seg + 1, per_head = p.nseg;
                if (p.sum_mode) {
                    per_head = p.nseg * p.sub;
                    s_lo = p.reverse ? (seg + 1) * p.sub : 0;
                    s_hi = p.reverse ? per_head : seg * p.sub;
                }
                if (!p.states) s_hi = s_lo;
                if (s_hi > s_lo) asm volatile("griddepcontrol.wait;" ::: "memory");
                for (int blk = 0; blk < nb; ++blk)
#pragma unroll
                    for (int cb = 0; cb < 2; ++cb) {
                        float acc[32];
#pragma unroll
                        for (int e = 0; e < 32; ++e) acc[e] = 0.f;
                        if (srow_ok)
                            for (int sb = s_lo; sb < s_hi; ++sb) {
                                const float *src = p.states + ((int64_t)bh * per_head + sb) * p.state_blk;
                                if (p.state_transposed) {
                                    src += (int64_t)(32 * cb) * p.state_ld + 64 * blk + srow;
#pragma unroll
                                    for (int e = 0; e < 32; ++e) acc[e] += src[e * p.state_ld];
                                } else {
                                    const float4 *s4 = reinterpret_cast<const float4 *>(
                                        src + (int64_t)(64 * blk + srow) * p.state_ld + 32 * cb);
#pragma unroll
                                    for (int e = 0; e < 8; ++e) {
                                        const float4 x = s4[e];
                                        acc[4 * e] += x.x; acc[4 * e + 1] += x.y; acc[4 * e + 2] += x.z; acc[4 * e + 3] += x.w;
                                    }
                                }
                            }
#pragma unroll
                        for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(acc[e]);
                        tmem_st32(tlane + TM_S + 64 * blk + 32 * cb, r);
                    }
                tmem_wait_st();
            }
            // ---- S_blk -> operand image of every step ---------------------------------------------
            for (int v = 0; v < nstep && ok; ++v) {
                const int ci = v / nb, blk = v - ci * nb, s = v & 1;
                if (v >= 2) {
                    // the image buffer is free (a S of step v - 2 has read it), and the state update of
                    // step v - 2 has been issued past its own wait for that image
                    const int v2 = v - 2, ci2 = v2 / nb, blk2 = v2 - ci2 * nb;
                    ok = mbar_wait(bar_smfree + 8 * s, (v2 >> 1) & 1, abort_flag) &&
                         mbar_wait(bar_sfull + 8 * blk2, ci2 & 1, abort_flag);
                    if (!ok) break;
                }
                if (ci >= 1) {
                    ok = mbar_wait(bar_sfull + 8 * blk, (ci - 1) & 1, abort_flag);   // S_blk after chunk ci - 1
                    if (!ok) break;
                }
                tc_fence_after();
                state_to_image(tlane + TM_S + 64 * blk, gen + kImgOff + s * kImg, lane, q);
                tc_fence_before();
                mbar_arrive(bar_smready + 8 * s);
                mbar_arrive(bar_smready2 + 8 * s);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 512);
    if (threadIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// The same shape with the wide dimension on the c / out side: (a, b, c) = (grad_out, V, K) for
// grad_Q, (V, grad_out, Q) walked downwards for grad_K -- a and b rows of 64, c and out rows of
// 64 nb.  With the column blocks c_blk of c,
//
//   out_c,blk = a_c S_blk + mask(a_c b_c^T) c_c,blk ;   S_blk += b_c^T c_c,blk
//
// so the scores and their mask are made ONCE per chunk and a_c, b_c are loaded once; a step
// (chunk, blk) loads one column block of c (32 KB) and writes one of out.  Shared memory: two
// chunks of {a | b}, two c blocks, two operand images; tensor memory as above (P, two output
// accumulators, the nb states in place).  The states are stored as [64 nb][64] blocks (the
// forward's orientation), i.e. transposed to what this scan accumulates.
struct ParamsC {
    float *out;
    Strides3 so;
    int H;
    int64_t L;
    int64_t seg_len;
    int nseg;
    int nb;
    const float *states;  // per (bh, seg) blocks of [64 nb][64] floats ([column of c][row of b]), or nullptr
    int sum_mode;
    int sub;
    int64_t state_blk;
    int reverse;
    int wait_first;
    int pos_a[3], pos_b[3], pos_c[3];
};

__global__ void __launch_bounds__(NTHREADS, 1)
wide_c_scan_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_c, const ParamsC p) {
    if (!p.wait_first) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + kBarOff;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + kBarOff + 384);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + kBarOff + 392);
    const uint32_t bar_abfull = bars, bar_abempty = bars + 16, bar_fullbmn = bars + 32, bar_cfull = bars + 48,
                   bar_cempty = bars + 64, bar_ofull = bars + 80, bar_ofree = bars + 96, bar_smready = bars + 112,
                   bar_smready2 = bars + 128, bar_smfree = bars + 144, bar_pfull = bars + 160,
                   bar_pready = bars + 168, bar_pfree = bars + 176, bar_sfull = bars + 184;   // [4]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = p.nb;
    const int seg = (int)(blockIdx.x % (unsigned)p.nseg);
    const int64_t bh = blockIdx.x / (unsigned)p.nseg;
    const int bn = (int)(bh / p.H), bhh = (int)(bh % p.H);
    const int64_t seg_begin = (int64_t)seg * p.seg_len;
    const int64_t seg_end = min(p.L, seg_begin + p.seg_len);
    int nchunk = (int)((seg_end - seg_begin + C - 1) / C);
    if (nchunk < 0) nchunk = 0;
    const int nstep = nchunk * nb;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_abfull + 8 * s, 1);
            mbar_init(bar_abempty + 8 * s, 2);    // both issuers
            mbar_init(bar_fullbmn + 8 * s, 128);
            mbar_init(bar_cfull + 8 * s, 1);
            mbar_init(bar_cempty + 8 * s, 2);     // both issuers
            mbar_init(bar_ofull + 8 * s, 1);
            mbar_init(bar_ofree + 8 * s, 128);
            mbar_init(bar_smready + 8 * s, 128);
            mbar_init(bar_smready2 + 8 * s, 128);
            mbar_init(bar_smfree + 8 * s, 1);
        }
        mbar_init(bar_pfull, 1);
        mbar_init(bar_pready, 128);
        mbar_init(bar_pfree, 1);
        for (int b = 0; b < MAXNB; ++b) mbar_init(bar_sfull + 8 * b, 1);
        fence_barrier_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (p.wait_first) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }

    if (nchunk > 0) {
        if (warp == 0) {
            // ================= TMA producer =====================================================
            if (elect_one()) {
                bool ok = true;
                for (int v = 0; v < nstep && ok; ++v) {
                    const int ci = v / nb, blk = v - ci * nb;
                    const int c = p.reverse ? nchunk - 1 - ci : ci;
                    const int row = (int)(seg_begin + (int64_t)c * C);
                    if (blk == 0) {
                        const int sa = ci & 1;
                        ok = mbar_wait(bar_abempty + 8 * sa, ((ci >> 1) & 1) ^ 1, abort_flag);
                        if (!ok) break;
                        const uint32_t st = base + sa * kStage;
                        mbar_expect_tx(bar_abfull + 8 * sa, kStage);
                        for (int b = 0; b < 2; ++b) {
                            tma_load_4d(st + b * kBlk, &map_a, bar_abfull + 8 * sa, 32 * b, p.pos_a, row, bhh, bn);
                            tma_load_4d(st + kTile + b * kBlk, &map_b, bar_abfull + 8 * sa, 32 * b, p.pos_b, row, bhh, bn);
                        }
                    }
                    const int s = v & 1;
                    ok = mbar_wait(bar_cempty + 8 * s, ((v >> 1) & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(bar_cfull + 8 * s, kTile);
                    for (int b = 0; b < 2; ++b)
                        tma_load_4d(base + kCOff + s * kTile + b * kBlk, &map_c, bar_cfull + 8 * s, 64 * blk + 32 * b,
                                    p.pos_c, row, bhh, bn);
                }
            }
        } else if (warp == 1 || warp == 10) {
            // ================= MMA issuers ======================================================
            if (elect_one()) {
                constexpr uint32_t ID_P = instr_desc(2, 0, 0, 128, 128);
                constexpr uint32_t ID_AS = instr_desc(2, 0, 1, 128, 64);
                constexpr uint32_t ID_PC = instr_desc(2, 0, 1, 128, 64);
                constexpr uint32_t ID_ST = instr_desc(2, 1, 1, 64, 64);
                constexpr uint64_t STAGE_UNITS = (uint64_t)(kStage >> 4), TILE_UNITS = (uint64_t)(kTile >> 4),
                                   IMG_UNITS = (uint64_t)(kImg >> 4);
                const uint64_t dAk0 = smem_desc(base, 16, 1024);
                const uint64_t dBk0 = smem_desc(base + kTile, 16, 1024);
                const uint64_t dBmn0 = smem_desc(base + kTile, kBlk, 512, 1);
                const uint64_t dCmn0 = smem_desc(base + kCOff, kBlk, 512, 1);
                const uint64_t dSm0 = smem_desc(base + kImgOff, kImgBlk, 512, 1);
                bool ok = true;
                if (warp == 1) {
                    // ---- output issuer: O_v = a S_blk + mask(P) c_blk ---------------------------
                    for (int v = 0; v < nstep && ok; ++v) {
                        const int ci = v / nb, blk = v - ci * nb;
                        const int s = v & 1, sa = ci & 1;
                        const uint32_t tO = tmem + TM_O + 64 * s;
                        ok = (blk != 0 || mbar_wait(bar_abfull + 8 * sa, (ci >> 1) & 1, abort_flag)) &&
                             mbar_wait(bar_smready + 8 * s, (v >> 1) & 1, abort_flag) &&
                             mbar_wait(bar_ofree + 8 * s, ((v >> 1) & 1) ^ 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        const uint64_t a0 = dAk0 + sa * STAGE_UNITS, sm0 = dSm0 + s * IMG_UNITS;
#pragma unroll
                        for (int b = 0; b < 2; ++b)
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                mma_ss<false>(tO, a0 + (uint64_t)((b * kBlk + k * 32) >> 4),
                                              sm0 + (uint64_t)(((32 * b + 8 * k) * 128) >> 4), ID_AS, (b | k) ? 1u : 0u);
                        tc_commit(bar_smfree + 8 * s);
                        ok = (blk != 0 || mbar_wait(bar_pready, ci & 1, abort_flag)) &&
                             mbar_wait(bar_cfull + 8 * s, (v >> 1) & 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        const uint64_t c0 = dCmn0 + s * TILE_UNITS;
#pragma unroll
                        for (int k = 0; k < 16; ++k)
                            mma_ts<false>(tO, tmem + TM_P + k * 8, c0 + (uint64_t)((k * 1024) >> 4), ID_PC, 1u);
                        tc_commit(bar_ofull + 8 * s);
                        tc_commit(bar_cempty + 8 * s);
                        if (blk + 1 == nb) {
                            tc_commit(bar_pfree);
                            tc_commit(bar_abempty + 8 * sa);
                        }
                    }
                } else {
                    // ---- score / state issuer -------------------------------------------------------
                    int sc = 0, ds = 0;     // next chunk to score, next step to update
                    long long t0 = 0;
                    uint32_t idle = 0;
                    while (ds < nstep) {
                        if (sc < nchunk && mbar_test(bar_abfull + 8 * (sc & 1), (sc >> 1) & 1) &&
                            (sc == 0 || mbar_test(bar_pfree, (sc - 1) & 1))) {
                            tc_fence_after();
                            const uint64_t a0 = dAk0 + (sc & 1) * STAGE_UNITS, b0 = dBk0 + (sc & 1) * STAGE_UNITS;
#pragma unroll
                            for (int b = 0; b < 2; ++b)
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    const uint64_t off = (uint64_t)((b * kBlk + k * 32) >> 4);
                                    mma_ss<false>(tmem + TM_P, a0 + off, b0 + off, ID_P, (b | k) ? 1u : 0u);
                                }
                            tc_commit(bar_pfull);
                            ++sc;
                            idle = 0;
                            continue;
                        }
                        if (ds < sc * nb) {
                            const int ci = ds / nb, blk = ds - ci * nb, s = ds & 1, sa = ci & 1;
                            if (mbar_test(bar_fullbmn + 8 * sa, (ci >> 1) & 1) &&
                                mbar_test(bar_cfull + 8 * s, (ds >> 1) & 1) &&
                                mbar_test(bar_smready2 + 8 * s, (ds >> 1) & 1)) {
                                tc_fence_after();
                                const uint64_t bmn0 = dBmn0 + sa * STAGE_UNITS, c0 = dCmn0 + s * TILE_UNITS;
#pragma unroll
                                for (int k = 0; k < 16; ++k) {
                                    const uint64_t off = (uint64_t)((k * 1024) >> 4);
                                    mma_ss<false>(tmem + TM_S + 64 * blk, bmn0 + off, c0 + off, ID_ST, 1u);
                                }
                                tc_commit(bar_sfull + 8 * blk);
                                tc_commit(bar_cempty + 8 * s);
                                if (blk + 1 == nb) tc_commit(bar_abempty + 8 * sa);
                                ++ds;
                                idle = 0;
                                continue;
                            }
                        }
                        if (idle++ == 0) t0 = clock64();
                        if ((idle & 63u) == 0u) {
                            if (*abort_flag) break;
                            if (clock64() - t0 > 4000000000LL) {
                                *abort_flag = 1;
                                atomicExch(&g_device_status, 5 /* FTB_ERR_TIMEOUT */);
                                break;
                            }
                        }
                    }
                }
            }
        } else if (warp >= 11) {
            // ================= mask workers: once per chunk, in place =============================
            const int q = warp & 3;
            const uint32_t tP = tmem + ((uint32_t)(32 * q) << 16) + TM_P;
            for (int ci = 0; ci < nchunk; ++ci) {
                if (!mbar_wait(bar_pfull, ci & 1, abort_flag)) break;
                tc_fence_after();
                mask_scores_in_place(tP, q, lane, p.reverse);
                tc_fence_before();
                mbar_arrive(bar_pready);
            }
        } else if (warp >= 6 && warp < 10) {
            // ================= output workers ====================================================
            const int q = warp & 3;
            const int t = threadIdx.x - 192;
            const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
            uint32_t r[32];
            bool ok = true;
            float *O = p.out + (int64_t)bn * p.so.n + (int64_t)bhh * p.so.h;
            for (int v = 0; v < nstep && ok; ++v) {
                const int ci = v / nb, blk = v - ci * nb, s = v & 1;
                if (blk == 0) {
                    // MN-major image of b, in place, once the score product has read the tile
                    ok = mbar_wait(bar_pfull, ci & 1, abort_flag);
                    if (!ok) break;
                    rearrange_tile_in_place(gen + (ci & 1) * kStage + kTile, t);
                    mbar_arrive(bar_fullbmn + 8 * (ci & 1));
                }
                const int c = p.reverse ? nchunk - 1 - ci : ci;
                const int64_t row0 = seg_begin + (int64_t)c * C;
                ok = mbar_wait(bar_ofull + 8 * s, (v >> 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    tmem_ld16x256(tlane + ((uint32_t)(16 * hf) << 16) + TM_O + 64 * s, r);
                    const int64_t ra = row0 + 32 * q + 16 * hf + (lane >> 2);
                    float *da = O + ra * p.so.l + 64 * blk + 2 * (lane & 3);
                    float *db = da + 8 * p.so.l;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (ra < seg_end) *reinterpret_cast<uint2 *>(da + 8 * j) = make_uint2(r[4 * j], r[4 * j + 1]);
                        if (ra + 8 < seg_end) *reinterpret_cast<uint2 *>(db + 8 * j) = make_uint2(r[4 * j + 2], r[4 * j + 3]);
                    }
                }
                tc_fence_before();
                mbar_arrive(bar_ofree + 8 * s);
            }
        } else if (warp >= 2 && warp < 6) {
            // ================= state workers ======================================================
            const int q = warp & 3;
            const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
            const bool srow_ok = lane < 16;
            const int srow = 16 * q + (lane & 15);      // row of b^T c = column of the stored block
            uint32_t r[32];
            bool ok = true;
            {
                int s_lo = seg, s_hi = seg + 1, per_head = p.nseg;
                if (p.sum_mode) {
                    per_head = p.nseg * p.sub;
                    s_lo = p.reverse ? (seg + 1) * p.sub : 0;
                    s_hi = p.reverse ? per_head : seg * p.sub;
                }
                if (!p.states) s_hi = s_lo;
                if (s_hi > s_lo) asm volatile("griddepcontrol.wait;" ::: "memory");
                for (int blk = 0; blk < nb; ++blk)
#pragma unroll
                    for (int cb = 0; cb < 2; ++cb) {
                        float acc[32];
#pragma unroll
                        for (int e = 0; e < 32; ++e) acc[e] = 0.f;
                        if (srow_ok)
                            for (int sb = s_lo; sb < s_hi; ++sb) {
                                const float *src = p.states + ((int64_t)bh * per_head + sb) * p.state_blk +
                                                   (int64_t)(64 * blk + 32 * cb) * 64 + srow;
#pragma unroll
                                for (int e = 0; e < 32; ++e) acc[e] += src[e * 64];
                            }
#pragma unroll
                        for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(acc[e]);
                        tmem_st32(tlane + TM_S + 64 * blk + 32 * cb, r);
                    }
                tmem_wait_st();
            }
            for (int v = 0; v < nstep && ok; ++v) {
                const int ci = v / nb, blk = v - ci * nb, s = v & 1;
                if (v >= 2) {
                    const int v2 = v - 2, ci2 = v2 / nb, blk2 = v2 - ci2 * nb;
                    ok = mbar_wait(bar_smfree + 8 * s, (v2 >> 1) & 1, abort_flag) &&
                         mbar_wait(bar_sfull + 8 * blk2, ci2 & 1, abort_flag);
                    if (!ok) break;
                }
                if (ci >= 1) {
                    ok = mbar_wait(bar_sfull + 8 * blk, (ci - 1) & 1, abort_flag);
                    if (!ok) break;
                }
                tc_fence_after();
                state_to_image(tlane + TM_S + 64 * blk, gen + kImgOff + s * kImg, lane, q);
                tc_fence_before();
                mbar_arrive(bar_smready + 8 * s);
                mbar_arrive(bar_smready2 + 8 * s);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 512);
    if (threadIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace wide
}  // namespace ftb
