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
    int accumulate;             // backward modes: add to what `out` holds instead of replacing it
    const void *elu_x;          // streaming backward kernels with `accumulate`: the sum is then taken
    Strides3n xs;               // through phi(x) = elu(x) + 1 of this raw input (same shape as out) and
    const float *elu_mask;      // a per-(batch, position) weight: out = (out + n) * w * phi'(x)
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
                float v = p.mode == NORM_BWD_Q ? sG[r] * sX[r * PD + d] : sX[r * PD + d];
                if (p.accumulate) v += step_load(op + (row0 + r) * p.os.l + d);
                step_store(op + (row0 + r) * p.os.l + d, v);
            }
        }
        __syncthreads();
    }
}

// ---- the fast path: D in {16, 32, 64, 128}, 16-byte (fp32) / 8-byte (bf16) aligned rows ------------
// A group of LPR = D / 4 lanes owns one (batch, head, segment); every lane keeps four features of
// the running sum in registers and streams down (up) the rows, U rows of loads in flight at a
// time.  No shared memory, no block-wide barriers; the per-row dot product of the forward is a
// shuffle reduction inside the group.
template <typename T>
__device__ __forceinline__ float4 norm_load4(const T *p);
template <>
__device__ __forceinline__ float4 norm_load4<float>(const float *p) {
    return *reinterpret_cast<const float4 *>(p);
}
template <>
__device__ __forceinline__ float4 norm_load4<__nv_bfloat16>(const __nv_bfloat16 *p) {
    const uint2 v = *reinterpret_cast<const uint2 *>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162 *>(&v.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162 *>(&v.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void norm_store4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void norm_store4(__nv_bfloat16 *p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t *>(&a);
    o.y = *reinterpret_cast<uint32_t *>(&b);
    *reinterpret_cast<uint2 *>(p) = o;
}

// totals == true: only the sum of the segment's rows is produced (into p.totals)
template <typename T, int LPR, int MODE, bool TOTALS>
__global__ void __launch_bounds__(kNormThreads, 2)
norm_stream_kernel(const NormParams p, int64_t ngroups) {
    constexpr int U = LPR < 8 ? 4 : 8;                 // rows in flight
    const int lane = threadIdx.x & 31;
    const int gl = lane % LPR;                         // lane inside the group
    const unsigned gmask = LPR == 32 ? 0xffffffffu : (((1u << LPR) - 1u) << (lane / LPR * LPR));
    const int64_t gid = (int64_t)blockIdx.x * (kNormThreads / LPR) + threadIdx.x / LPR;
    if (gid >= ngroups) return;
    const int seg = (int)(gid % p.nseg);
    const int64_t bh = gid / p.nseg;
    const int64_t n = bh / p.H, h = bh % p.H;
    const int64_t r0 = (int64_t)seg * p.seg_len, r1 = min(p.L, r0 + p.seg_len);
    constexpr int mode = MODE;
    constexpr bool rev = MODE == NORM_BWD_K;
    const int d = 4 * gl;
    const T *qp = reinterpret_cast<const T *>(p.q) + n * p.qs.n + h * p.qs.h + d;
    const T *kp = reinterpret_cast<const T *>(p.k) + n * p.ks.n + h * p.ks.h + d;
    const T *gp = reinterpret_cast<const T *>(p.g) + n * p.gs.n + h * p.gs.h;
    T *op = reinterpret_cast<T *>(p.out) + n * p.os.n + h * p.os.h;
    float *tot = p.totals + bh * p.nseg * p.D + d;

    float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!TOTALS && p.nseg > 1) {
        if (!rev) {
            for (int s = 0; s < seg; ++s) {
                const float4 v = *reinterpret_cast<const float4 *>(tot + (int64_t)s * p.D);
                run.x += v.x; run.y += v.y; run.z += v.z; run.w += v.w;
            }
        } else {
            for (int s = p.nseg - 1; s > seg; --s) {
                const float4 v = *reinterpret_cast<const float4 *>(tot + (int64_t)s * p.D);
                run.x += v.x; run.y += v.y; run.z += v.z; run.w += v.w;
            }
        }
    }

    const int64_t nrows = r1 - r0;
    for (int64_t b0 = 0; b0 < nrows; b0 += U) {
        float4 x[U], y[U];
        float gx[U];
        int64_t row[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            // ascending: rows r0 + b0 + u; descending: rows r1 - 1 - b0 - u
            row[u] = rev ? r1 - 1 - b0 - u : r0 + b0 + u;
            const bool ok = b0 + u < nrows;
            x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            y[u] = x[u];
            gx[u] = 0.f;
            if (ok) {
                if (mode == NORM_BWD_K) {
                    x[u] = norm_load4(qp + row[u] * p.qs.l);
                } else {
                    x[u] = norm_load4(kp + row[u] * p.ks.l);
                    if (mode == NORM_FWD && !TOTALS) y[u] = norm_load4(qp + row[u] * p.qs.l);
                }
                if (mode != NORM_FWD) gx[u] = step_load(gp + row[u] * p.gs.l);
            }
        }
        float keep = 0.f;   // forward: lane u of the group keeps the result of row u
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool ok = b0 + u < nrows;
            if (mode == NORM_BWD_K) {
                run.x += gx[u] * x[u].x; run.y += gx[u] * x[u].y;
                run.z += gx[u] * x[u].z; run.w += gx[u] * x[u].w;
            } else {
                run.x += x[u].x; run.y += x[u].y; run.z += x[u].z; run.w += x[u].w;
            }
            if (TOTALS) continue;
            if (mode == NORM_FWD) {
                float acc = y[u].x * run.x + y[u].y * run.y + y[u].z * run.z + y[u].w * run.w;
#pragma unroll
                for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(gmask, acc, o);
                if (gl == u) keep = acc;
            } else if (ok) {
                float4 v = mode == NORM_BWD_Q
                               ? make_float4(gx[u] * run.x, gx[u] * run.y, gx[u] * run.z, gx[u] * run.w)
                               : run;
                if (p.accumulate) {
                    const float4 o = norm_load4(op + row[u] * p.os.l + d);
                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                    if (p.elu_x) {
                        const float4 xv = norm_load4(reinterpret_cast<const T *>(p.elu_x) + n * p.xs.n + h * p.xs.h +
                                                     row[u] * p.xs.l + d);
                        const float w = p.elu_mask ? p.elu_mask[n * p.L + row[u]] : 1.f;
                        v.x *= w * (xv.x > 0.f ? 1.f : expf(xv.x));
                        v.y *= w * (xv.y > 0.f ? 1.f : expf(xv.y));
                        v.z *= w * (xv.z > 0.f ? 1.f : expf(xv.z));
                        v.w *= w * (xv.w > 0.f ? 1.f : expf(xv.w));
                    }
                }
                norm_store4(op + row[u] * p.os.l + d, v);
            }
        }
        if (!TOTALS && mode == NORM_FWD && gl < U && b0 + gl < nrows)
            step_store(op + (r0 + b0 + gl) * p.os.l, keep);
    }
    if (TOTALS) *reinterpret_cast<float4 *>(tot + (int64_t)seg * p.D) = run;
}

// ---- the layer's division, backward -----------------------------------------------------------
// With y = out * Z, Z = 1 / (den + eps) per row (fast_transformers/attention/
// causal_linear_attention.py:95-104):  grad_out = grad_y * Z,  grad_den = -Z * sum_m grad_y * y.
// One pass over grad_y and y (rows of M = 4 * LPR fp32 values, contiguous), LPR lanes per row.
template <int LPR>
__global__ void __launch_bounds__(256)
normalised_grads_kernel(const float *__restrict__ grad_y, const float *__restrict__ y,
                        const float *__restrict__ den, float *__restrict__ grad_out,
                        float *__restrict__ grad_den, int64_t rows, float eps) {
    const int lane = threadIdx.x & 31, gl = lane % LPR;
    const unsigned gmask = LPR == 32 ? 0xffffffffu : (((1u << LPR) - 1u) << (lane / LPR * LPR));
    const int64_t row = ((int64_t)blockIdx.x * 256 + threadIdx.x) / LPR;
    if (row >= rows) return;
    const int64_t off = row * (4 * LPR) + 4 * gl;
    const float4 g = *reinterpret_cast<const float4 *>(grad_y + off);
    const float4 v = *reinterpret_cast<const float4 *>(y + off);
    const float z = 1.f / (den[row] + eps);
    float s = g.x * v.x + g.y * v.y + g.z * v.z + g.w * v.w;
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(gmask, s, o);
    *reinterpret_cast<float4 *>(grad_out + off) = make_float4(g.x * z, g.y * z, g.z * z, g.w * z);
    if (gl == 0) grad_den[row] = -z * s;
}

}  // namespace ftb
