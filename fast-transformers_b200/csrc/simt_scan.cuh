// fp32 CUDA-core ("SIMT") kernels of the causal linear-attention product.
//
// The sequence of every (batch, head) pair is cut into SEGMENTS; one CTA walks one segment
// chunk by chunk (CH rows) carrying a slice of the running state in shared memory:
//
//   out_c  = a_c . S_prev  +  mask(a_c b_c^T) . c_c        S_prev += b_c^T c_c
//
// with (a, b, c) = (Q, K, V) for the forward product and the role permutations
// (G, V, K), (V, G, Q), (K, Q, G) for grad_Q, grad_K, grad_V (the last two walk the rows
// in descending order with the mask flipped).  The state a segment starts from is the
// exclusive prefix (suffix) of per-segment totals produced by state_sum_kernel and
// state_prefix_kernel, so all segments of all heads run concurrently.
//
// Maths: fast_transformers/causal_product/causal_product_cpu.cpp:106-121 (forward),
// :165-206 (backward), regrouped into blocks; every product is plain fp32 FMA.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ftb {

constexpr int CH = 32;        // rows per chunk
constexpr int KT = 64;        // tile of the contracted ("a") feature dimension
constexpr int NC = 64;        // output columns per CTA
constexpr int NTHR = 128;     // threads per CTA
constexpr int PA = KT + 4;    // shared-memory pitches (floats); +4 keeps float4 rows on
constexpr int PCC = NC + 4;   //   distinct banks for 8 consecutive rows
constexpr int PP = CH + 4;

struct Strides3 {
    int64_t n, h, l;
};

struct ScanArgs {
    const void *a, *b, *c;
    void *out;
    Strides3 sa, sb, sc, so;
    int H;
    int64_t L;
    int Da, Dc;          // a,b rows have Da features; c,out rows have Dc
    int64_t seg_len;     // rows per segment (multiple of CH)
    int nseg;
    const float *states; // [(bh*nseg + seg)] x (D*M) canonical blocks, or NULL (zeros)
    int canon_is_DaDc;   // canonical block is [Da][Dc] (1) or [Dc][Da] (0)
    int reverse;         // walk rows downwards, keep j >= i
    int va, vb, vc, vo;  // 4-element vector access allowed for a, b, c, out
};

__device__ __forceinline__ float4 ldg4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 ldg4(const __nv_bfloat16 *p) {
    uint2 u = *reinterpret_cast<const uint2 *>(p);
    __nv_bfloat162 lo = *reinterpret_cast<__nv_bfloat162 *>(&u.x);
    __nv_bfloat162 hi = *reinterpret_cast<__nv_bfloat162 *>(&u.y);
    float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float ldg1(const float *p) { return *p; }
__device__ __forceinline__ float ldg1(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stg4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void stg4(__nv_bfloat16 *p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t *>(&lo);
    u.y = *reinterpret_cast<uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(p) = u;
}
__device__ __forceinline__ void stg1(float *p, float v) { *p = v; }
__device__ __forceinline__ void stg1(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

// Four consecutive elements of a row, zero outside [0, ncols) or when the row is absent.
template <typename T>
__device__ __forceinline__ float4 load_quad(const T *row, int col, int ncols, bool row_ok, bool vec) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!row_ok) return v;
    if (vec && col + 3 < ncols) return ldg4(row + col);
    if (col < ncols) v.x = ldg1(row + col);
    if (col + 1 < ncols) v.y = ldg1(row + col + 1);
    if (col + 2 < ncols) v.z = ldg1(row + col + 2);
    if (col + 3 < ncols) v.w = ldg1(row + col + 3);
    return v;
}

// Copy a CH x 64 tile (rows row0.., columns col0..) of a global matrix into shared memory.
template <typename T>
__device__ __forceinline__ void load_tile(float *dst, int pitch, const T *base, int64_t sl,
                                          int64_t row0, int64_t row_end, int col0, int ncols,
                                          bool vec, int tid) {
#pragma unroll
    for (int it = 0; it < (CH * 16) / NTHR; ++it) {
        int u = tid + it * NTHR;
        int r = u >> 4, c4 = (u & 15) << 2;
        int64_t row = row0 + r;
        float4 v = load_quad(base + row * sl, col0 + c4, ncols, row < row_end, vec);
        *reinterpret_cast<float4 *>(dst + r * pitch + c4) = v;
    }
}

__device__ __forceinline__ float dot4(float4 a, float4 b, float acc) {
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    acc = fmaf(a.w, b.w, acc);
    return acc;
}

// Row of the shared state tile that holds output column n (0..63).  Columns owned by
// neighbouring threads (4 apart) land on consecutive rows, i.e. distinct banks.
__device__ __forceinline__ int state_row(int n) { return ((n & 3) << 4) + (n >> 2); }

inline size_t scan_smem_bytes(int Da) {
    int DaP = (Da + KT - 1) / KT * KT;
    return sizeof(float) * ((size_t)NC * (DaP + 4) + 2 * CH * PA + CH * PCC + CH * PP);
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(NTHR) simt_scan_kernel(ScanArgs p) {
    extern __shared__ __align__(16) float smem[];
    const int tid = threadIdx.x;
    const int DaP = (p.Da + KT - 1) / KT * KT;
    const int PS = DaP + 4;
    float *sSt = smem;                 // [NC][PS]   state slice, row = state_row(column)
    float *sA = sSt + NC * PS;         // [CH][PA]
    float *sB = sA + CH * PA;          // [CH][PA]
    float *sC = sB + CH * PA;          // [CH][PCC]
    float *sPt = sC + CH * PCC;        // [CH][PP]   masked scores, transposed: [j][i]

    const int ntile = (p.Dc + NC - 1) / NC;
    int64_t bid = blockIdx.x;
    const int tile = (int)(bid % ntile);
    bid /= ntile;
    const int seg = (int)(bid % p.nseg);
    const int64_t bh = bid / p.nseg;
    const int64_t bn = bh / p.H, bhh = bh % p.H;
    const int n0 = tile * NC;

    const TI *A = reinterpret_cast<const TI *>(p.a) + bn * p.sa.n + bhh * p.sa.h;
    const TI *B = reinterpret_cast<const TI *>(p.b) + bn * p.sb.n + bhh * p.sb.h;
    const TI *C = reinterpret_cast<const TI *>(p.c) + bn * p.sc.n + bhh * p.sc.h;
    TO *O = reinterpret_cast<TO *>(p.out) + bn * p.so.n + bhh * p.so.h;

    const int64_t seg_begin = (int64_t)seg * p.seg_len;
    const int64_t seg_end = min(p.L, seg_begin + p.seg_len);
    const int nchunk = (int)((seg_end - seg_begin + CH - 1) / CH);

    // ---- state slice this segment starts from ----------------------------------------
    if (p.states == nullptr) {
        for (int i = tid; i < NC * PS; i += NTHR) sSt[i] = 0.f;
    } else {
        const float *st = p.states + ((int64_t)bh * p.nseg + seg) * ((int64_t)p.Da * p.Dc);
        if (p.canon_is_DaDc) {   // st[k*Dc + n]
            for (int i = tid; i < NC * DaP; i += NTHR) {
                int n = i & (NC - 1), k = i >> 6;
                float v = (k < p.Da && n0 + n < p.Dc) ? st[(int64_t)k * p.Dc + n0 + n] : 0.f;
                sSt[state_row(n) * PS + k] = v;
            }
        } else {                 // st[n*Da + k]
            for (int i = tid; i < NC * DaP; i += NTHR) {
                int k = i % DaP, n = i / DaP;
                float v = (k < p.Da && n0 + n < p.Dc) ? st[(int64_t)(n0 + n) * p.Da + k] : 0.f;
                sSt[state_row(n) * PS + k] = v;
            }
        }
    }

    // thread coordinates of the three register tilings
    const int ti = tid >> 4, tn = tid & 15;   // out tile: rows 4ti.., cols 4tn..
    const int tj = tid >> 3, ti8 = tid & 7;   // score tile: j = 2tj+e, i = ti8+8a
    const int tn8 = tid >> 4, td = tid & 15;  // state tile: n = 8tn8+a, k = 4td..

    for (int ci = 0; ci < nchunk; ++ci) {
        const int c = p.reverse ? nchunk - 1 - ci : ci;
        const int64_t row0 = seg_begin + (int64_t)c * CH;

        load_tile(sC, PCC, C, p.sc.l, row0, seg_end, n0, p.Dc, p.vc, tid);

        float acc[4][4];
        float accP[2][4];
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) acc[x][y] = 0.f;
#pragma unroll
        for (int x = 0; x < 2; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) accP[x][y] = 0.f;

        for (int kt = 0; kt < DaP; kt += KT) {
            load_tile(sA, PA, A, p.sa.l, row0, seg_end, kt, p.Da, p.va, tid);
            load_tile(sB, PA, B, p.sb.l, row0, seg_end, kt, p.Da, p.vb, tid);
            __syncthreads();

            // scores (transposed): Pt[j][i] += b_j . a_i      and      out += a . S_prev
#pragma unroll 4
            for (int k4 = 0; k4 < KT; k4 += 4) {
                float4 b0 = *reinterpret_cast<const float4 *>(sB + (2 * tj) * PA + k4);
                float4 b1 = *reinterpret_cast<const float4 *>(sB + (2 * tj + 1) * PA + k4);
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    float4 av = *reinterpret_cast<const float4 *>(sA + (ti8 + 8 * a) * PA + k4);
                    accP[0][a] = dot4(b0, av, accP[0][a]);
                    accP[1][a] = dot4(b1, av, accP[1][a]);
                }
                float4 s[4];
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    s[b] = *reinterpret_cast<const float4 *>(sSt + (tn + 16 * b) * PS + kt + k4);
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    float4 av = *reinterpret_cast<const float4 *>(sA + (4 * ti + a) * PA + k4);
#pragma unroll
                    for (int b = 0; b < 4; ++b) acc[a][b] = dot4(av, s[b], acc[a][b]);
                }
            }
            __syncthreads();

            // S[n][kt+k] += sum_r c[r][n] * b[r][k]
            {
                float4 sacc[8];
#pragma unroll
                for (int a = 0; a < 8; ++a)
                    sacc[a] = *reinterpret_cast<const float4 *>(
                        sSt + state_row(8 * tn8 + a) * PS + kt + 4 * td);
#pragma unroll 4
                for (int r = 0; r < CH; ++r) {
                    float4 c0 = *reinterpret_cast<const float4 *>(sC + r * PCC + 8 * tn8);
                    float4 c1 = *reinterpret_cast<const float4 *>(sC + r * PCC + 8 * tn8 + 4);
                    float4 bv = *reinterpret_cast<const float4 *>(sB + r * PA + 4 * td);
                    const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
                    for (int a = 0; a < 8; ++a) {
                        sacc[a].x = fmaf(cc[a], bv.x, sacc[a].x);
                        sacc[a].y = fmaf(cc[a], bv.y, sacc[a].y);
                        sacc[a].z = fmaf(cc[a], bv.z, sacc[a].z);
                        sacc[a].w = fmaf(cc[a], bv.w, sacc[a].w);
                    }
                }
#pragma unroll
                for (int a = 0; a < 8; ++a)
                    *reinterpret_cast<float4 *>(sSt + state_row(8 * tn8 + a) * PS + kt + 4 * td) =
                        sacc[a];
            }
            __syncthreads();
        }

        // causal mask inside the chunk (the diagonal is kept), stored as Pt[j][i]
#pragma unroll
        for (int e = 0; e < 2; ++e)
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                int j = 2 * tj + e, i = ti8 + 8 * a;
                bool keep = p.reverse ? (j >= i) : (j <= i);
                sPt[j * PP + i] = keep ? accP[e][a] : 0.f;
            }
        __syncthreads();

#pragma unroll 4
        for (int j = 0; j < CH; ++j) {
            float4 pv = *reinterpret_cast<const float4 *>(sPt + j * PP + 4 * ti);
            float4 cv = *reinterpret_cast<const float4 *>(sC + j * PCC + 4 * tn);
            const float pp[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                acc[a][0] = fmaf(pp[a], cv.x, acc[a][0]);
                acc[a][1] = fmaf(pp[a], cv.y, acc[a][1]);
                acc[a][2] = fmaf(pp[a], cv.z, acc[a][2]);
                acc[a][3] = fmaf(pp[a], cv.w, acc[a][3]);
            }
        }

        const int col = n0 + 4 * tn;
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            int64_t row = row0 + 4 * ti + a;
            if (row < seg_end && col < p.Dc) {
                TO *dst = O + row * p.so.l + col;
                if (p.vo && col + 3 < p.Dc) {
                    stg4(dst, make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]));
                } else {
#pragma unroll
                    for (int b = 0; b < 4; ++b)
                        if (col + b < p.Dc) stg1(dst + b, acc[a][b]);
                }
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------
// per-segment totals  T[d][m] = sum_{rows of the segment} x[r][d] * y[r][m]
// ---------------------------------------------------------------------------------------
struct StateSumArgs {
    const void *x, *y;
    Strides3 sx, sy;
    int H;
    int64_t L;
    int D, M;
    int64_t seg_len;
    int nseg;
    float *states;   // [(bh*nseg + seg)][D][M]
    int vx, vy;
};

template <typename TI>
__global__ void __launch_bounds__(NTHR) simt_state_sum_kernel(StateSumArgs p) {
    __shared__ __align__(16) float sX[CH * PA];
    __shared__ __align__(16) float sY[CH * PCC];
    const int tid = threadIdx.x;
    const int dt = (p.D + KT - 1) / KT, mt = (p.M + NC - 1) / NC;
    int64_t bid = blockIdx.x;
    const int tm = (int)(bid % mt);
    bid /= mt;
    const int tdd = (int)(bid % dt);
    bid /= dt;
    const int seg = (int)(bid % p.nseg);
    const int64_t bh = bid / p.nseg;
    const int64_t bn = bh / p.H, bhh = bh % p.H;
    const int d0 = tdd * KT, m0 = tm * NC;

    const TI *X = reinterpret_cast<const TI *>(p.x) + bn * p.sx.n + bhh * p.sx.h;
    const TI *Y = reinterpret_cast<const TI *>(p.y) + bn * p.sy.n + bhh * p.sy.h;
    const int64_t seg_begin = (int64_t)seg * p.seg_len;
    const int64_t seg_end = min(p.L, seg_begin + p.seg_len);

    const int td8 = tid >> 4, tm4 = tid & 15;   // d = 8*td8 + a, m = 4*tm4 ..
    float4 acc[8];
#pragma unroll
    for (int a = 0; a < 8; ++a) acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);

    for (int64_t row0 = seg_begin; row0 < seg_end; row0 += CH) {
        load_tile(sX, PA, X, p.sx.l, row0, seg_end, d0, p.D, p.vx, tid);
        load_tile(sY, PCC, Y, p.sy.l, row0, seg_end, m0, p.M, p.vy, tid);
        __syncthreads();
#pragma unroll 4
        for (int r = 0; r < CH; ++r) {
            float4 x0 = *reinterpret_cast<const float4 *>(sX + r * PA + 8 * td8);
            float4 x1 = *reinterpret_cast<const float4 *>(sX + r * PA + 8 * td8 + 4);
            float4 yv = *reinterpret_cast<const float4 *>(sY + r * PCC + 4 * tm4);
            const float xx[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int a = 0; a < 8; ++a) {
                acc[a].x = fmaf(xx[a], yv.x, acc[a].x);
                acc[a].y = fmaf(xx[a], yv.y, acc[a].y);
                acc[a].z = fmaf(xx[a], yv.z, acc[a].z);
                acc[a].w = fmaf(xx[a], yv.w, acc[a].w);
            }
        }
        __syncthreads();
    }

    float *T = p.states + ((int64_t)bh * p.nseg + seg) * ((int64_t)p.D * p.M);
    const int m = m0 + 4 * tm4;
#pragma unroll
    for (int a = 0; a < 8; ++a) {
        int d = d0 + 8 * td8 + a;
        if (d < p.D) {
            float *dst = T + (int64_t)d * p.M + m;
            const float vv[4] = {acc[a].x, acc[a].y, acc[a].z, acc[a].w};
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (m + b < p.M) dst[b] = vv[b];
        }
    }
}

// ---------------------------------------------------------------------------------------
// exclusive prefix (suffix) of the per-segment totals along the segment axis, in place;
// `init` (per bh) is added to every entry, `total` (per bh) receives init + total_init + all
// segments (total_init lets a caller keep the entries free of an initial state it adds later).
// ---------------------------------------------------------------------------------------
__global__ void state_prefix_kernel(float *states, const float *init, float *total,
                                    const float *total_init, int64_t BH, int nseg, int64_t DM,
                                    int reverse) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= BH * DM) return;
    int64_t bh = idx / DM, e = idx % DM;
    float run = init ? init[idx] : 0.f;
    float *base = states + bh * nseg * DM + e;
    if (!reverse) {
        for (int s = 0; s < nseg; ++s) {
            float t = base[(int64_t)s * DM];
            base[(int64_t)s * DM] = run;
            run += t;
        }
    } else {
        for (int s = nseg - 1; s >= 0; --s) {
            float t = base[(int64_t)s * DM];
            base[(int64_t)s * DM] = run;
            run += t;
        }
    }
    if (total) total[idx] = run + (total_init ? total_init[idx] : 0.f);
}

// The same, four consecutive elements per thread (DM % 4 == 0, 16-byte aligned blocks) and the
// loads of eight segments in flight before the first store: the scalar form above walks the
// segments one dependent load-store pair at a time and took 28 us for nine 64 KB blocks per head.
__global__ void state_prefix4_kernel(float4 *states, const float4 *init, float4 *total,
                                     const float4 *total_init, int64_t BH, int nseg, int64_t DM4,
                                     int reverse) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= BH * DM4) return;
    int64_t bh = idx / DM4, e = idx % DM4;
    float4 run = init ? init[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 *base = states + bh * nseg * DM4 + e;
    for (int s0 = 0; s0 < nseg; s0 += 8) {
        float4 t[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int s = s0 + j;
            if (s < nseg) t[j] = base[(int64_t)(reverse ? nseg - 1 - s : s) * DM4];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int s = s0 + j;
            if (s < nseg) {
                base[(int64_t)(reverse ? nseg - 1 - s : s) * DM4] = run;
                run.x += t[j].x; run.y += t[j].y; run.z += t[j].z; run.w += t[j].w;
            }
        }
    }
    if (total) {
        if (total_init) {
            const float4 ti = total_init[idx];
            run.x += ti.x; run.y += ti.y; run.z += ti.z; run.w += ti.w;
        }
        total[idx] = run;
    }
}

// total[bh] = init[bh] + sum over all segments of the raw per-segment totals
__global__ void state_total_kernel(const float *states, const float *init, float *total,
                                   int64_t BH, int nseg, int64_t DM) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= BH * DM) return;
    int64_t bh = idx / DM, e = idx % DM;
    float run = init ? init[idx] : 0.f;
    const float *base = states + bh * nseg * DM + e;
    for (int s = 0; s < nseg; ++s) run += base[(int64_t)s * DM];
    total[idx] = run;
}

}  // namespace ftb
