// The denominator of causal linear attention and its gradients:
//
//   den_l  = Q_l . C_l,          C_l = sum_{j<=l} K_j          (forward)
//   gQ_l   = g_l * C_l                                          (backward, ascending)
//   gK_j   = sum_{l>=j} g_l * Q_l                               (backward, descending)
//
// per (batch, head) sequence -- the reference's `torch.einsum("nlhi,nlhi->nlh", Q, K.cumsum(1))`
// (fast_transformers/attention/causal_linear_attention.py:95) and what autograd makes of it.
// All three are running sums of D-vectors along the sequence, so they stream every tensor once:
// fp32 accumulation, HBM-bound, no tensor cores (D multiply-adds per D elements read).
//
// A sequence is cut into segments; `norm_totals_kernel` sums the rows of every segment, and
// `norm_scan_kernel` walks a segment in tiles of 32 rows starting from the sum of the totals of
// the segments before (after) it.  Fixed summation order, no atomics.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "recurrent_step.cuh"   // step_load / step_store

namespace ftb {

constexpr int kNormThreads = 256;
constexpr int kNormRows = 32;     // rows per tile
constexpr int kNormMaxD = 256;    // feature width limit (shared-memory tiles)

struct Strides3n {
    int64_t n, h, l;   // element strides of batch, head, position; features contiguous
};

enum NormMode { NORM_FWD = 0, NORM_BWD_Q = 1, NORM_BWD_K = 2 };

struct NormParams {
    const void *q, *k, *g;      // g: gradient of den, (N,H,L) (backward modes)
    void *out;                  // FWD: den (N,H,L);  BWD_Q: gQ;  BWD_K: gK  (N,H,L,D)
    Strides3n qs, ks, gs, os;   // gs / os of (N,H,L) tensors use n, h, l only
    int H, D, nseg;
    int64_t L, seg_len;         // seg_len: multiple of kNormRows
    float *totals;              // (N*H, nseg, D) fp32: per-segment sums of K rows (FWD, BWD_Q)
                                // or of g * Q rows (BWD_K)
    int mode;
};

// ---- per-segment totals ---------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kNormThreads)
norm_totals_kernel(const NormParams p) {
    __shared__ float part[kNormThreads];
    const int t = threadIdx.x;
    const int seg = blockIdx.x % p.nseg;
    const int64_t bh = blockIdx.x / p.nseg;
    const int64_t n = bh / p.H, h = bh % p.H;
    const int64_t r0 = (int64_t)seg * p.seg_len, r1 = min(p.L, r0 + p.seg_len);
    const bool gq = p.mode == NORM_BWD_K;   // sum g * Q rows instead of K rows
    const T *x = reinterpret_cast<const T *>(gq ? p.q : p.k) + n * (gq ? p.qs.n : p.ks.n) +
                 h * (gq ? p.qs.h : p.ks.h);
    const int64_t xl = gq ? p.qs.l : p.ks.l;
    const T *gp = reinterpret_cast<const T *>(p.g) + n * p.gs.n + h * p.gs.h;
    float *dst = p.totals + (bh * p.nseg + seg) * p.D;
    // feature tiles of up to 256 columns; thread = (row group, feature)
    for (int d0 = 0; d0 < p.D; d0 += kNormThreads) {
        const int dt = min(p.D - d0, kNormThreads);
        const int groups = kNormThreads / dt;
        const int d = t % dt, rg = t / dt;
        float acc = 0.f;
        if (rg < groups) {
            for (int64_t r = r0 + rg; r < r1; r += groups) {
                float v = step_load(x + r * xl + d0 + d);
                if (gq) v *= step_load(gp + r * p.gs.l);
                acc += v;
            }
        }
        part[t] = acc;
        __syncthreads();
        if (t < dt) {
            float s = 0.f;
            for (int g2 = 0; g2 < groups; ++g2) s += part[g2 * dt + t];
            dst[d0 + t] = s;
        }
        __syncthreads();
    }
}

// ---- the scans --------------------------------------------------------------------------------
// One CTA per (batch, head, segment).  Tile = 32 rows x D features in shared memory (pitch D+1
// floats).  The running sums are kept by thread d < D in a register.
template <typename T>
__global__ void __launch_bounds__(kNormThreads)
norm_scan_kernel(const NormParams p) {
    extern __shared__ float sm[];
    const int D = p.D, PD = D + 1;
    float *sX = sm;                        // [32][PD]: the summed rows, then their running sums
    float *sY = sm + kNormRows * PD;       // [32][PD]: Q rows (FWD)
    __shared__ float sG[kNormRows];
    const int t = threadIdx.x;
    const int seg = blockIdx.x % p.nseg;
    const int64_t bh = blockIdx.x / p.nseg;
    const int64_t n = bh / p.H, h = bh % p.H;
    const int64_t r0 = (int64_t)seg * p.seg_len, r1 = min(p.L, r0 + p.seg_len);
    const bool rev = p.mode == NORM_BWD_K;
    const T *qp = reinterpret_cast<const T *>(p.q) + n * p.qs.n + h * p.qs.h;
    const T *kp = reinterpret_cast<const T *>(p.k) + n * p.ks.n + h * p.ks.h;
    const T *gp = reinterpret_cast<const T *>(p.g) + n * p.gs.n + h * p.gs.h;
    T *op = reinterpret_cast<T *>(p.out) + n * p.os.n + h * p.os.h;

    // start value of the running sums: totals of the segments before (after) this one
    float run = 0.f;
    if (t < D) {
        const float *tot = p.totals + bh * p.nseg * D;
        if (!rev)
            for (int s = 0; s < seg; ++s) run += tot[(int64_t)s * D + t];
        else
            for (int s = p.nseg - 1; s > seg; --s) run += tot[(int64_t)s * D + t];
    }

    const int64_t ntile = (r1 - r0 + kNormRows - 1) / kNormRows;
    for (int64_t ti = 0; ti < ntile; ++ti) {
        const int64_t tile = rev ? ntile - 1 - ti : ti;
        const int64_t row0 = r0 + tile * kNormRows;
        const int rows = (int)min((int64_t)kNormRows, r1 - row0);
        // ---- load (coalesced along features) ----
        if (p.mode != NORM_FWD && t < rows) sG[t] = step_load(gp + (row0 + t) * p.gs.l);
        __syncthreads();
        for (int e = t; e < rows * D; e += kNormThreads) {
            const int r = e / D, d = e % D;
            if (p.mode == NORM_BWD_K) {
                sX[r * PD + d] = sG[r] * step_load(qp + (row0 + r) * p.qs.l + d);
            } else {
                sX[r * PD + d] = step_load(kp + (row0 + r) * p.ks.l + d);
                if (p.mode == NORM_FWD) sY[r * PD + d] = step_load(qp + (row0 + r) * p.qs.l + d);
            }
        }
        __syncthreads();
        // ---- running sums down (up) the rows of the tile, one feature per thread ----
        if (t < D) {
            if (!rev) {
                for (int r = 0; r < rows; ++r) {
                    run += sX[r * PD + t];
                    sX[r * PD + t] = run;
                }
            } else {
                for (int r = rows - 1; r >= 0; --r) {
                    run += sX[r * PD + t];
                    sX[r * PD + t] = run;
                }
            }
        }
        __syncthreads();
        // ---- results ----
        if (p.mode == NORM_FWD) {
            // den_r = Q_r . C_r : 8 threads per row, combined with shuffles
            const int r = t >> 3, part = t & 7;
            float acc = 0.f;
            if (r < rows)
                for (int d = part; d < D; d += 8) acc += sX[r * PD + d] * sY[r * PD + d];
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            if (part == 0 && r < rows) step_store(op + (row0 + r) * p.os.l, acc);
        } else {
            for (int e = t; e < rows * D; e += kNormThreads) {
                const int r = e / D, d = e % D;
                const float v = p.mode == NORM_BWD_Q ? sG[r] * sX[r * PD + d] : sX[r * PD + d];
                step_store(op + (row0 + r) * p.os.l + d, v);
            }
        }
        __syncthreads();
    }
}

}  // namespace ftb
