// One step of causal linear attention as a recurrent model:
//
//   Q = phi(q), K = phi(k);  z += K;  S += K (x) v;  y = (Q . S) / (Q . z + eps)
//
// for every (batch, head) pair, with the fp32 state S (D x M) and normaliser z (D) updated in
// place.  The reference does this with five torch einsum / add calls per step
// (fast_transformers/recurrent/attention/self_attention/linear_attention.py:78-87); here it is
// one launch: a CTA per (batch, head), S streamed through once (read, update, write back, and
// the column sums Q . S taken on the way), so a step moves the algorithmic 2 * D * M * 4 bytes
// per pair.  Sums run in a fixed order (no atomics): results are bit-identical run to run.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ftb {

constexpr int kStepThreads = 256;
constexpr int kStepMaxD = 512;

struct Strides2 {
    int64_t n, h;   // element strides of batch and head; the feature dimension is contiguous
};

template <typename T>
__device__ __forceinline__ float step_load(const T *p);
template <>
__device__ __forceinline__ float step_load<float>(const float *p) { return *p; }
template <>
__device__ __forceinline__ float step_load<__nv_bfloat16>(const __nv_bfloat16 *p) {
    return __bfloat162float(*p);
}
__device__ __forceinline__ void step_store(float *p, float x) { *p = x; }
__device__ __forceinline__ void step_store(__nv_bfloat16 *p, float x) { *p = __float2bfloat16(x); }

// feature: 0 = inputs are features already, 1 = phi(x) = elu(x) + 1 applied to q and k here
// (feature_maps/base.py:71-73)
// UPDATE = false: the state is only read -- y = (Q . S) / (Q . z + eps) with k and v unused: a
// step of cross attention over a fixed memory
// (fast_transformers/recurrent/attention/cross_attention/linear_attention.py:66-69).
template <typename T, bool UPDATE = true>
__global__ void __launch_bounds__(kStepThreads)
recurrent_step_kernel(const T *q, const T *k, const T *v, float *S, float *z, T *out, int H, int D,
                      int M, Strides2 qs, Strides2 ks, Strides2 vs, Strides2 os, int feature, float eps) {
    __shared__ float sq[kStepMaxD], sk[kStepMaxD];
    __shared__ float4 part4[kStepThreads];
    __shared__ float red[kStepThreads / 32];
    __shared__ float s_norm;
    const int t = threadIdx.x;
    const int64_t bh = blockIdx.x;
    const int64_t n = bh / H, h = bh % H;
    const T *qp = q + n * qs.n + h * qs.h;
    const T *kp = k + n * ks.n + h * ks.h;
    const T *vp = v + n * vs.n + h * vs.h;
    T *op = out + n * os.n + h * os.h;
    float *Sp = S + bh * (int64_t)D * M;
    float *zp = z + bh * (int64_t)D;

    // features, z += K, and the partial sums of Q . z
    float qz = 0.f;
    for (int d = t; d < D; d += kStepThreads) {
        float a = step_load(qp + d), b = UPDATE ? step_load(kp + d) : 0.f;
        if (feature == 1) {
            a = a > 0.f ? a + 1.f : expf(a);   // elu(x) + 1
            if (UPDATE) b = b > 0.f ? b + 1.f : expf(b);
        }
        const float zn = zp[d] + b;
        if (UPDATE) zp[d] = zn;
        sq[d] = a;
        sk[d] = b;
        qz += a * zn;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) qz += __shfl_xor_sync(0xffffffffu, qz, o);
    if ((t & 31) == 0) red[t >> 5] = qz;
    __syncthreads();
    if (t == 0) {
        float s = 0.f;
        for (int w = 0; w < kStepThreads / 32; ++w) s += red[w];
        s_norm = 1.f / (s + eps);
    }
    __syncthreads();
    const float Z = s_norm;

    // S += K (x) v and y = (Q . S) Z.  Thread = (row group, column group): consecutive threads
    // touch consecutive columns of a row, every thread walks its rows four at a time so that
    // several loads are in flight, and the row groups' partial column sums are added in a fixed
    // order at the end.
    if ((M & 3) == 0 && M <= 4 * kStepThreads) {
        // four columns per thread (16-byte accesses; S rows are 16-byte aligned when M % 4 == 0)
        const int cg = M >> 2;                       // column groups
        const int rg_count = kStepThreads / cg;      // row groups (>= 1 since M <= 1024)
        const int col4 = t % cg, rg = t / cg;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (rg < rg_count) {
            const float4 vm = UPDATE ? make_float4(step_load(vp + 4 * col4), step_load(vp + 4 * col4 + 1),
                                                   step_load(vp + 4 * col4 + 2), step_load(vp + 4 * col4 + 3))
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 *base = reinterpret_cast<float4 *>(Sp) + col4;
            int d = rg;
            for (; d + 3 * rg_count < D; d += 4 * rg_count) {
                float4 s[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) s[u] = base[(int64_t)(d + u * rg_count) * cg];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float kd = sk[d + u * rg_count], qd = sq[d + u * rg_count];
                    if (UPDATE) {
                        s[u].x += kd * vm.x; s[u].y += kd * vm.y; s[u].z += kd * vm.z; s[u].w += kd * vm.w;
                        base[(int64_t)(d + u * rg_count) * cg] = s[u];
                    }
                    acc.x += qd * s[u].x; acc.y += qd * s[u].y; acc.z += qd * s[u].z; acc.w += qd * s[u].w;
                }
            }
            for (; d < D; d += rg_count) {
                float4 s0 = base[(int64_t)d * cg];
                const float kd = sk[d], qd = sq[d];
                if (UPDATE) {
                    s0.x += kd * vm.x; s0.y += kd * vm.y; s0.z += kd * vm.z; s0.w += kd * vm.w;
                    base[(int64_t)d * cg] = s0;
                }
                acc.x += qd * s0.x; acc.y += qd * s0.y; acc.z += qd * s0.z; acc.w += qd * s0.w;
            }
        }
        part4[t] = acc;
        __syncthreads();
        if (t < cg) {
            float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int g = 0; g < rg_count; ++g) {
                const float4 a = part4[g * cg + t];
                y.x += a.x; y.y += a.y; y.z += a.z; y.w += a.w;
            }
            step_store(op + 4 * t, y.x * Z);
            step_store(op + 4 * t + 1, y.y * Z);
            step_store(op + 4 * t + 2, y.z * Z);
            step_store(op + 4 * t + 3, y.w * Z);
        }
        return;
    }
    // any M: one column per thread, a tile of up to 256 columns at a time
    float *part = reinterpret_cast<float *>(part4);
    for (int m0 = 0; m0 < M; m0 += kStepThreads) {
        const int mt = min(M - m0, kStepThreads);   // columns of this tile
        const int rg_count = kStepThreads / mt;     // row groups
        const int col = t % mt, rg = t / mt;
        float acc = 0.f;
        if (rg < rg_count) {
            const float vm = UPDATE ? step_load(vp + m0 + col) : 0.f;
            for (int d = rg; d < D; d += rg_count) {
                float *sp = Sp + (int64_t)d * M + m0 + col;
                const float s = *sp + sk[d] * vm;
                if (UPDATE) *sp = s;
                acc += sq[d] * s;
            }
        }
        part[t] = acc;
        __syncthreads();
        if (t < mt) {
            float y = 0.f;
            for (int g = 0; g < rg_count; ++g) y += part[g * mt + t];
            step_store(op + m0 + t, y * Z);
        }
        __syncthreads();
    }
}

}  // namespace ftb
