// fp32-accurate segment scan on the tensor cores: every fp32 operand x is split into
//
//   hi = x with the low 13 mantissa bits cleared   (exact in TF32)
//   lo = x - hi                                     (exact in fp32; TF32 keeps its leading 11 bits)
//
// and every product A B of the 64-wide scan (mma_scan.cuh) becomes A_hi B_hi + A_lo B_hi + A_hi B_lo
// with fp32 accumulation in tensor memory; the dropped term is below 2^-21 of the product.  Results
// match the fp64 oracle to ~1e-6 (the tier of the fp32 CUDA-core kernels, which this mode replaces
// for D = M = 64 fp32) at several times their speed.
//
// One CTA walks one segment in chunks of 128 rows.  The split doubles the operand tiles, so one
// chunk (a, b, c as hi | lo: 192 KB) and the two images of the state operand (32 KB) fill shared
// memory: ONE stage, no ring -- the next chunk's loads start when this chunk's products have
// retired.  Tensor memory: P_hi 128 columns (the scores, masked and truncated in place), P_lo 128,
// two output accumulators and two state-increment accumulators of 64.
//
// Warp roles: 0 = TMA producer; 1 = output issuer (O = a S, O += mask(P) c); 10 = score / state
// issuer (P = a b^T, T = b^T c); 2-5 = state workers (the running fp32 state in registers, one row
// per thread: += T, then its hi | lo operand images); 6-9 = output workers and 11-14 = mask workers:
// together they split the tiles that landed, then the output workers make the MN-major images of
// b in place and write O rows, the mask workers mask and split P.  Every wait is bounded
// (mbar_wait): on expiry the CTA records FTB_ERR_TIMEOUT, stops issuing work, frees its tensor
// memory and returns.
//
// Maths: fast_transformers/causal_product/causal_product_cpu.cpp:106-121, :165-206 in blocks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mma_scan.cuh"

namespace ftb {
namespace x3 {

using namespace ftb::mma;

constexpr int kBlk = C * 128;            // one [128 rows][128 B] swizzled block
constexpr int kTile = 2 * kBlk;          // 128 x 64 fp32
constexpr int kA = 0, kB = 2 * kTile, kC = 4 * kTile;   // hi tile; its lo tile follows at + kTile
constexpr int kImgBlk = 64 * 128;        // state operand: [64 rows][128 B] per 32 columns
constexpr int kImg = 2 * kImgBlk;
constexpr int kImgOff = 6 * kTile, kBarOff = kImgOff + 2 * kImg;
constexpr size_t kSmem = 1024 + kBarOff + 512;
constexpr int TM_P = 0, TM_PLO = 128, TM_O = 256, TM_T = 384;
constexpr uint32_t kHiMask = 0xFFFFE000u;

struct Params {
    float *out;
    Strides3 so;
    int H;
    int64_t L;
    int64_t seg_len;      // multiple of C
    int nseg;
    const float *states;  // per (bh, seg) [64][64] blocks, or nullptr
    int sum_mode;         // 0: the block of a segment is its start state; 1: raw totals, summed here
    int sub;              // sum_mode 1: `states` holds `sub` blocks per segment of this launch (the
                          // sweep ran on `sub` times finer segments, to fill more SMs)
    float *state_out;     // state-only: per (bh, seg) totals
    int skip_lo, skip_hi; // state-only: segments whose totals nobody reads
    int canon_is_DaDc;    // stored blocks are [DA][Dc] (1) or [Dc][DA] (0)
    int reverse;
    int state_only;
    int wait_first;       // programmatic launch: wait for the grid in front before any global access
                          // (0: that grid is this call's own; only its totals are waited for)
    int pos_a[3], pos_b[3], pos_c[3];
};

__device__ __forceinline__ void split4(const uint4 x, uint4 &hi, uint4 &lo) {
    hi = make_uint4(x.x & kHiMask, x.y & kHiMask, x.z & kHiMask, x.w & kHiMask);
    lo.x = __float_as_uint(__uint_as_float(x.x) - __uint_as_float(hi.x));
    lo.y = __float_as_uint(__uint_as_float(x.y) - __uint_as_float(hi.y));
    lo.z = __float_as_uint(__uint_as_float(x.z) - __uint_as_float(hi.z));
    lo.w = __float_as_uint(__uint_as_float(x.w) - __uint_as_float(hi.w));
}

__global__ void __launch_bounds__(NTHREADS, 1)
x3_scan_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_bmn, const __grid_constant__ CUtensorMap map_c,
               const Params p) {
    if (!p.wait_first) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + kBarOff;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + kBarOff + 256);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + kBarOff + 264);
    const uint32_t bar_full = bars, bar_split = bars + 8, bar_pfull = bars + 16, bar_fullbmn = bars + 24,
                   bar_pready = bars + 32, bar_smready = bars + 40, bar_smfree = bars + 48, bar_empty = bars + 56,
                   bar_ofull = bars + 64, bar_ofree = bars + 80, bar_tfull = bars + 96, bar_tfree = bars + 112;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = (int)(blockIdx.x % (unsigned)p.nseg);
    const int64_t bh = blockIdx.x / (unsigned)p.nseg;
    const int bn = (int)(bh / p.H), bhh = (int)(bh % p.H);
    const int64_t seg_begin = (int64_t)seg * p.seg_len;
    const int64_t seg_end = min(p.L, seg_begin + p.seg_len);
    int nchunk = (int)((seg_end - seg_begin + C - 1) / C);
    const bool skipped = p.state_only && seg >= p.skip_lo && seg < p.skip_hi;
    if (skipped || nchunk < 0) nchunk = 0;
    if (p.state_only && nchunk == 0 && !skipped) {
        // a segment without rows: its totals are zero, and they are read like any other block
        float *dst = p.state_out + ((int64_t)bh * p.nseg + seg) * 4096;
        if (p.wait_first) asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int e = threadIdx.x; e < 4096; e += NTHREADS) dst[e] = 0.f;
    }

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar_full, 1);
        mbar_init(bar_split, 256);
        mbar_init(bar_pfull, 1);
        mbar_init(bar_fullbmn, 128);
        mbar_init(bar_pready, 128);
        mbar_init(bar_smready, 128);
        mbar_init(bar_smfree, 1);
        mbar_init(bar_empty, p.state_only ? 1 : 2);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_ofull + 8 * s, 1);
            mbar_init(bar_ofree + 8 * s, 128);
            mbar_init(bar_tfull + 8 * s, 1);
            mbar_init(bar_tfree + 8 * s, 128);
        }
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

    // hi | lo of the tiles that landed: 16-byte pieces, shared by the 256 threads of warps 6-9 and
    // 11-14 (`t`: 0..255).  State-only launches have no a tile.
    auto split_tiles = [&](int t) {
        const int first = p.state_only ? 2048 : 0;
        for (int idx = first + t; idx < 3 * 2048; idx += 256) {
            uint8_t *hp = gen + (idx >> 11) * (2 * kTile) + (idx & 2047) * 16;
            uint4 hi, lo;
            split4(*reinterpret_cast<const uint4 *>(hp), hi, lo);
            *reinterpret_cast<uint4 *>(hp) = hi;
            *reinterpret_cast<uint4 *>(hp + kTile) = lo;
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_split);
    };

    if (nchunk > 0) {
        if (warp == 0) {
            // ================= TMA producer =====================================================
            if (elect_one()) {
                for (int ci = 0; ci < nchunk; ++ci) {
                    const int c = p.reverse ? nchunk - 1 - ci : ci;
                    const int row = (int)(seg_begin + (int64_t)c * C);
                    if (!mbar_wait(bar_empty, (ci & 1) ^ 1, abort_flag)) break;
                    mbar_expect_tx(bar_full, (p.state_only ? 2 : 3) * kTile);
                    for (int b = 0; b < 2; ++b) {
                        if (!p.state_only)
                            tma_load_4d(base + kA + b * kBlk, &map_a, bar_full, 32 * b, p.pos_a, row, bhh, bn);
                        tma_load_4d(base + kB + b * kBlk, p.state_only ? &map_bmn : &map_b, bar_full, 32 * b, p.pos_b,
                                    row, bhh, bn);
                        tma_load_4d(base + kC + b * kBlk, &map_c, bar_full, 32 * b, p.pos_c, row, bhh, bn);
                    }
                    // With one stage the next chunk cannot land in shared memory yet; pull it towards
                    // L2 meanwhile, so that its loads find it there (this kernel waits for latency, not
                    // for HBM bandwidth).
                    if (ci + 1 < nchunk) {
                        const int cn = p.reverse ? nchunk - 2 - ci : ci + 1;
                        const int rown = (int)(seg_begin + (int64_t)cn * C);
                        for (int b = 0; b < 2; ++b) {
                            if (!p.state_only) tma_prefetch_4d(&map_a, 32 * b, p.pos_a, rown, bhh, bn);
                            tma_prefetch_4d(&map_b, 32 * b, p.pos_b, rown, bhh, bn);
                            tma_prefetch_4d(&map_c, 32 * b, p.pos_c, rown, bhh, bn);
                        }
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
                constexpr uint64_t LO = (uint64_t)(kTile >> 4), IMG_LO = (uint64_t)(kImg >> 4);
                const uint64_t dAk = smem_desc(base + kA, 16, 1024);
                const uint64_t dBk = smem_desc(base + kB, 16, 1024);
                const uint64_t dBmn = smem_desc(base + kB, kBlk, 512, 1);
                const uint64_t dCmn = smem_desc(base + kC, kBlk, 512, 1);
                const uint64_t dSm = smem_desc(base + kImgOff, kImgBlk, 512, 1);
                bool ok = true;
                if (warp == 1) {
                    // ---- output issuer ---------------------------------------------------------
                    for (int ci = 0; ci < nchunk && ok && !p.state_only; ++ci) {
                        const int ob = ci & 1;
                        const uint32_t tO = tmem + TM_O + 64 * ob;
                        ok = mbar_wait(bar_split, ci & 1, abort_flag) && mbar_wait(bar_smready, ci & 1, abort_flag) &&
                             mbar_wait(bar_ofree + 8 * ob, ((ci >> 1) & 1) ^ 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        // The tensor cores add every product to the accumulator with truncation, an
                        // error of up to one unit in the last place of the ACCUMULATOR per instruction,
                        // all of one sign: the small terms (those with a low part) therefore go first,
                        // onto an accumulator that is still small, and the hi x hi terms last.
                        // O = a_lo S_hi + a_hi S_lo ...
#pragma unroll
                        for (int term = 1; term < 3; ++term) {
                            const uint64_t a0 = dAk + (term == 1 ? LO : 0), s0 = dSm + (term == 2 ? IMG_LO : 0);
#pragma unroll
                            for (int b = 0; b < 2; ++b)
#pragma unroll
                                for (int k = 0; k < 4; ++k)
                                    mma_ss<false>(tO, a0 + (uint64_t)((b * kBlk + k * 32) >> 4),
                                                  s0 + (uint64_t)(((32 * b + 8 * k) * 128) >> 4), ID_AS,
                                                  (term > 1 || b || k) ? 1u : 0u);
                        }
                        ok = mbar_wait(bar_pready, ci & 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        // ... + P_lo c_hi + P_hi c_lo ...
#pragma unroll
                        for (int term = 1; term < 3; ++term) {
                            const uint32_t tP = tmem + (term == 1 ? TM_PLO : TM_P);
                            const uint64_t c0 = dCmn + (term == 2 ? LO : 0);
#pragma unroll
                            for (int k = 0; k < 16; ++k)
                                mma_ts<false>(tO, tP + k * 8, c0 + (uint64_t)((k * 1024) >> 4), ID_PC, 1u);
                        }
                        // ... + a_hi S_hi + P_hi c_hi
#pragma unroll
                        for (int b = 0; b < 2; ++b)
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                mma_ss<false>(tO, dAk + (uint64_t)((b * kBlk + k * 32) >> 4),
                                              dSm + (uint64_t)(((32 * b + 8 * k) * 128) >> 4), ID_AS, 1u);
                        tc_commit(bar_smfree);
#pragma unroll
                        for (int k = 0; k < 16; ++k)
                            mma_ts<false>(tO, tmem + TM_P + k * 8, dCmn + (uint64_t)((k * 1024) >> 4), ID_PC, 1u);
                        tc_commit(bar_ofull + 8 * ob);
                        tc_commit(bar_empty);
                    }
                } else {
                    // ---- score / state issuer --------------------------------------------------
                    for (int ci = 0; ci < nchunk && ok; ++ci) {
                        const int tb = ci & 1;
                        ok = mbar_wait(bar_split, ci & 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        if (!p.state_only) {
                            // P = a_lo b_hi^T + a_hi b_lo^T + a_hi b_hi^T (small terms first)
#pragma unroll
                            for (int t3 = 0; t3 < 3; ++t3) {
                                const int term = (t3 + 1) % 3;
                                const uint64_t a0 = dAk + (term == 1 ? LO : 0), b0 = dBk + (term == 2 ? LO : 0);
#pragma unroll
                                for (int b = 0; b < 2; ++b)
#pragma unroll
                                    for (int k = 0; k < 4; ++k) {
                                        const uint64_t off = (uint64_t)((b * kBlk + k * 32) >> 4);
                                        mma_ss<false>(tmem + TM_P, a0 + off, b0 + off, ID_P, (t3 | b | k) ? 1u : 0u);
                                    }
                            }
                            tc_commit(bar_pfull);
                            ok = mbar_wait(bar_fullbmn, ci & 1, abort_flag);
                            if (!ok) break;
                        }
                        ok = mbar_wait(bar_tfree + 8 * tb, ((ci >> 1) & 1) ^ 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        // T = b_lo^T c_hi + b_hi^T c_lo + b_hi^T c_hi (small terms first)
#pragma unroll
                        for (int t3 = 0; t3 < 3; ++t3) {
                            const int term = (t3 + 1) % 3;
                            const uint64_t b0 = dBmn + (term == 1 ? LO : 0), c0 = dCmn + (term == 2 ? LO : 0);
#pragma unroll
                            for (int k = 0; k < 16; ++k) {
                                const uint64_t off = (uint64_t)((k * 1024) >> 4);
                                mma_ss<false>(tmem + TM_T + 64 * tb, b0 + off, c0 + off, ID_ST, (t3 | k) ? 1u : 0u);
                            }
                        }
                        tc_commit(bar_tfull + 8 * tb);
                        tc_commit(bar_empty);
                    }
                }
            }
        } else if (warp >= 11) {
            // ================= mask workers ======================================================
            const int q = warp & 3;
            const uint32_t tP = tmem + ((uint32_t)(32 * q) << 16) + TM_P;
            uint32_t r[32], lo[32];
            for (int ci = 0; ci < nchunk; ++ci) {
                if (!mbar_wait(bar_full, ci & 1, abort_flag)) break;
                split_tiles(128 + threadIdx.x - 352);
                if (p.state_only) continue;
                if (!mbar_wait(bar_pfull, ci & 1, abort_flag)) break;
                tc_fence_after();
                // rows 32q .. 32q+31; column blocks of 32: dropped ones are zeroed (hi and lo), kept
                // ones split, the diagonal one masked element by element first
                const int ndrop = p.reverse ? q : 3 - q;
                const uint32_t drop0 = p.reverse ? 0 : 32 * (q + 1);
                tmem_zero_columns(tP + drop0, 32 * ndrop);
                tmem_zero_columns(tP + TM_PLO + drop0, 32 * ndrop);
                const int kb0 = p.reverse ? q : 0, kb1 = p.reverse ? 3 : q;
                for (int cb = kb0; cb <= kb1; ++cb) {
                    tmem_ld32(tP + 32 * cb, r);
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const bool keep = cb != q || (p.reverse ? (e >= lane) : (e <= lane));
                        const uint32_t x = keep ? r[e] : 0u;
                        r[e] = x & kHiMask;
                        lo[e] = __float_as_uint(__uint_as_float(x) - __uint_as_float(r[e]));
                    }
                    tmem_st32(tP + 32 * cb, r);
                    tmem_st32(tP + TM_PLO + 32 * cb, lo);
                }
                tmem_wait_st();
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
            auto write_chunk = [&](int ci) -> bool {
                const int c = p.reverse ? nchunk - 1 - ci : ci;
                const int64_t row0 = seg_begin + (int64_t)c * C;
                const int ob = ci & 1;
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
                        if (ra < seg_end) *reinterpret_cast<uint2 *>(da + 8 * j) = make_uint2(r[4 * j], r[4 * j + 1]);
                        if (ra + 8 < seg_end) *reinterpret_cast<uint2 *>(db + 8 * j) = make_uint2(r[4 * j + 2], r[4 * j + 3]);
                    }
                }
                tc_fence_before();
                mbar_arrive(bar_ofree + 8 * ob);
                return true;
            };
            for (int ci = 0; ci < nchunk && ok; ++ci) {
                ok = mbar_wait(bar_full, ci & 1, abort_flag);
                if (!ok) break;
                split_tiles(t);
                if (p.state_only) continue;
                // MN-major images of b_hi and b_lo, in place, once the score product has read them:
                // 16-byte chunk c of row r moves from c ^ (r & 7) to the 32-byte-atom position
                ok = mbar_wait(bar_pfull, ci & 1, abort_flag);
                if (!ok) break;
                for (int it0 = 0; it0 < 32; it0 += 4) {
                    uint4 vv[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int idx = (it0 + j) * 128 + t;    // 16-byte chunk of b_hi | b_lo (contiguous)
                        vv[j] = reinterpret_cast<const uint4 *>(gen + kB + (size_t)(idx >> 3) * 128)[idx & 7];
                    }
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int idx = (it0 + j) * 128 + t;
                        const int pk = idx & 7, row = (idx >> 3) & 127;
                        const int cc = pk ^ (row & 7);
                        const int pm = ((((cc >> 1) ^ (row & 3)) << 1) | (cc & 1));
                        reinterpret_cast<uint4 *>(gen + kB + (size_t)(idx >> 3) * 128)[pm] = vv[j];
                    }
                    __syncwarp();
                }
                fence_proxy_async_smem();
                mbar_arrive(bar_fullbmn);
                if (ci > 0) ok = write_chunk(ci - 1);
            }
            if (ok && !p.state_only) write_chunk(nchunk - 1);
        } else if (warp >= 2 && warp < 6) {
            // ================= state workers: one state row per thread, fp32, in registers ========
            const int q = warp & 3;
            const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
            const bool srow_ok = lane < 16;                 // 64-row accumulators: 16 lanes per quarter
            const int srow = 16 * q + (lane & 15);
            uint32_t r[32];
            float stv[64];
            bool ok = true;
            auto store_images = [&]() {
                if (!srow_ok) return;
#pragma unroll
                for (int cb = 0; cb < 2; ++cb) {
                    uint8_t *rowp = gen + kImgOff + cb * kImgBlk + srow * 128;
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        uint4 x, hi, lo;
                        x = make_uint4(__float_as_uint(stv[32 * cb + 4 * ch]), __float_as_uint(stv[32 * cb + 4 * ch + 1]),
                                       __float_as_uint(stv[32 * cb + 4 * ch + 2]), __float_as_uint(stv[32 * cb + 4 * ch + 3]));
                        split4(x, hi, lo);
                        const int o = (((ch >> 1) ^ (srow & 3)) * 32) + (ch & 1) * 16;
                        *reinterpret_cast<uint4 *>(rowp + o) = hi;
                        *reinterpret_cast<uint4 *>(rowp + kImg + o) = lo;
                    }
                }
            };
#pragma unroll
            for (int e = 0; e < 64; ++e) stv[e] = 0.f;
            if (!p.state_only) {
                // ---- segment-start state ------------------------------------------------------------
                int s_lo = seg, s_hi = seg + 1, per_head = p.nseg;
                if (p.sum_mode) {
                    per_head = p.nseg * p.sub;
                    s_lo = p.reverse ? (seg + 1) * p.sub : 0;
                    s_hi = p.reverse ? per_head : seg * p.sub;
                }
                if (!p.states) s_hi = s_lo;
                // the totals come from the launch in front (a sweep of this call): wait for it here
                if (s_hi > s_lo) asm volatile("griddepcontrol.wait;" ::: "memory");
                if (srow_ok)
                    for (int sb = s_lo; sb < s_hi; ++sb) {
                        const float *src = p.states + ((int64_t)bh * per_head + sb) * 4096;
                        if (p.canon_is_DaDc) {
                            const float4 *s4 = reinterpret_cast<const float4 *>(src + srow * 64);
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                const float4 x = s4[e];
                                stv[4 * e] += x.x; stv[4 * e + 1] += x.y; stv[4 * e + 2] += x.z; stv[4 * e + 3] += x.w;
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 64; ++e) stv[e] += src[e * 64 + srow];
                        }
                    }
                store_images();
                fence_proxy_async_smem();
                mbar_arrive(bar_smready);
            }
            for (int ci = 0; ci < nchunk && ok; ++ci) {
                const int tb = ci & 1;
                ok = mbar_wait(bar_tfull + 8 * tb, (ci >> 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int cb = 0; cb < 2; ++cb) {
                    tmem_ld32(tlane + TM_T + 64 * tb + 32 * cb, r);
#pragma unroll
                    for (int e = 0; e < 32; ++e) stv[32 * cb + e] += __uint_as_float(r[e]);
                }
                tc_fence_before();
                mbar_arrive(bar_tfree + 8 * tb);
                if (p.state_only || ci + 1 == nchunk) continue;
                ok = mbar_wait(bar_smfree, ci & 1, abort_flag);   // a S of this chunk has read the images
                if (!ok) break;
                store_images();
                fence_proxy_async_smem();
                mbar_arrive(bar_smready);
            }
            if (p.state_only && ok && srow_ok) {
                float4 *d4 = reinterpret_cast<float4 *>(p.state_out + ((int64_t)bh * p.nseg + seg) * 4096 + srow * 64);
#pragma unroll
                for (int e = 0; e < 16; ++e) d4[e] = make_float4(stv[4 * e], stv[4 * e + 1], stv[4 * e + 2], stv[4 * e + 3]);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 512);
    // no block of a programmatically launched grid ends before the grid in front of it has
    if (threadIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace x3
}  // namespace ftb
