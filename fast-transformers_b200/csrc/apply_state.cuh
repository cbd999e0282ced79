// out[n,h,l,:] = a[n,h,l,:] . S[n,h]  for one fixed state per (batch, head) pair -- fp32 FMA.
//
// The non-causal form of linear attention needs nothing else from a kernel: the state is the sum
// over ALL positions (ftb_causal_state_sum) and every position reads the same one
// (fast_transformers/attention/linear_attention.py:72-78: V = einsum(Q, KV) with KV = K^T V), and
// its gradients are the same two operations with the roles exchanged.  The tensor-core mode runs
// this as the APPLY instantiation of mma_scan_kernel; this file is the fp32 mode: a plain tiled
// product, 64 rows x 64 output columns per CTA, the state tile and the row tile staged in shared
// memory, a 4 x 4 register tile per thread.  Any Da, Dc; rows through strides.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "simt_scan.cuh"

namespace ftb {

constexpr int kApplyRows = 64, kApplyCols = 64, kApplyK = 32, kApplyThreads = 256;

struct ApplyArgs {
    const void *a;
    void *out;
    const float *state;   // (N*H) blocks of Da x Dc (canon) or Dc x Da (transposed)
    Strides3 sa, so;
    int H;
    int64_t L;
    int Da, Dc;
    int canon_is_DaDc;
    int vec_out;          // out rows start on 16-byte boundaries and Dc % 4 == 0 (fp32 only)
};

template <typename T>
__device__ __forceinline__ float apply_load(const T *p);
template <>
__device__ __forceinline__ float apply_load<float>(const float *p) { return *p; }
template <>
__device__ __forceinline__ float apply_load<__nv_bfloat16>(const __nv_bfloat16 *p) {
    return __bfloat162float(*p);
}
__device__ __forceinline__ void apply_store(float *p, float x) { *p = x; }
__device__ __forceinline__ void apply_store(__nv_bfloat16 *p, float x) { *p = __float2bfloat16(x); }

// grid: (row tiles, column tiles, N*H)
template <typename T>
__global__ void __launch_bounds__(kApplyThreads)
apply_state_kernel(ApplyArgs p) {
    __shared__ float sa[kApplyK][kApplyRows + 4];    // a tile, k-major so that row quads are float4s
    __shared__ float ss[kApplyK][kApplyCols + 4];    // state tile
    const int t = threadIdx.x;
    const int64_t bh = blockIdx.z;
    const int64_t n = bh / p.H, h = bh % p.H;
    const int64_t row0 = (int64_t)blockIdx.x * kApplyRows;
    const int col0 = blockIdx.y * kApplyCols;
    const T *A = reinterpret_cast<const T *>(p.a) + n * p.sa.n + h * p.sa.h;
    T *O = reinterpret_cast<T *>(p.out) + n * p.so.n + h * p.so.h;
    const float *S = p.state + bh * (int64_t)p.Da * p.Dc;
    const int tr = (t / 16) * 4, tc = (t % 16) * 4;   // this thread's 4 rows x 4 columns
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < p.Da; k0 += kApplyK) {
        // a tile: 64 rows x 32 features, consecutive threads along the feature axis
        for (int e = t; e < kApplyRows * kApplyK; e += kApplyThreads) {
            const int r = e / kApplyK, k = e % kApplyK;
            const int64_t row = row0 + r;
            float v = 0.f;
            if (row < p.L && k0 + k < p.Da) v = apply_load(A + row * p.sa.l + k0 + k);
            sa[k][r] = v;
        }
        // state tile: 32 features x 64 columns
        for (int e = t; e < kApplyK * kApplyCols; e += kApplyThreads) {
            int k, c;
            if (p.canon_is_DaDc) { k = e / kApplyCols; c = e % kApplyCols; }
            else { c = e / kApplyK; k = e % kApplyK; }      // consecutive threads along Da
            float v = 0.f;
            if (k0 + k < p.Da && col0 + c < p.Dc)
                v = p.canon_is_DaDc ? S[(int64_t)(k0 + k) * p.Dc + col0 + c]
                                    : S[(int64_t)(col0 + c) * p.Da + k0 + k];
            ss[k][c] = v;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < kApplyK; ++k) {
            const float4 av = *reinterpret_cast<const float4 *>(&sa[k][tr]);
            const float4 sv = *reinterpret_cast<const float4 *>(&ss[k][tc]);
            const float a4[4] = {av.x, av.y, av.z, av.w}, s4[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a4[i], s4[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t row = row0 + tr + i;
        if (row >= p.L) continue;
        if constexpr (sizeof(T) == 4) {
            if (p.vec_out && col0 + tc + 3 < p.Dc) {
                *reinterpret_cast<float4 *>(O + row * p.so.l + col0 + tc) =
                    make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
                continue;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (col0 + tc + j < p.Dc) apply_store(O + row * p.so.l + col0 + tc + j, acc[i][j]);
    }
}

}  // namespace ftb
