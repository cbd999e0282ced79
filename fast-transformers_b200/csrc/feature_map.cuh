// phi(x) = elu(x) + 1 (fast_transformers/feature_maps/base.py:71-73), optionally times a per-row
// 0/1 weight -- the key-length mask the layer multiplies K by
// (fast_transformers/attention/causal_linear_attention.py:83) -- and its gradient
// g * w * (x > 0 ? 1 : exp(x)).  One pass each over a contiguous (rows, inner) tensor whose mask
// (if any) has one entry per `inner_per_mask` consecutive elements; the reference spends an elu,
// an add and a multiply kernel forward and three more backward.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "normaliser.cuh"       // step_load / step_store, norm_load4 / norm_store4

namespace ftb {

// Aligned case: `total` and `inner_per_mask` multiples of 4, 16-byte (fp32) / 8-byte (bf16)
// aligned pointers -- one vector load and store per tensor and thread.
template <typename T, bool BACKWARD>
__global__ void __launch_bounds__(256)
elu1_vec_kernel(const T *x, const T *g, T *out, const float *mask, int64_t total, int64_t inner_per_mask) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= total) return;
    const float w = mask ? mask[i / inner_per_mask] : 1.f;
    const float4 v = norm_load4(x + i);
    float4 r;
    if (BACKWARD) {
        const float4 gv = norm_load4(g + i);
        r.x = gv.x * w * (v.x > 0.f ? 1.f : expf(v.x));
        r.y = gv.y * w * (v.y > 0.f ? 1.f : expf(v.y));
        r.z = gv.z * w * (v.z > 0.f ? 1.f : expf(v.z));
        r.w = gv.w * w * (v.w > 0.f ? 1.f : expf(v.w));
    } else {
        r.x = w * (v.x > 0.f ? v.x + 1.f : expf(v.x));
        r.y = w * (v.y > 0.f ? v.y + 1.f : expf(v.y));
        r.z = w * (v.z > 0.f ? v.z + 1.f : expf(v.z));
        r.w = w * (v.w > 0.f ? v.w + 1.f : expf(v.w));
    }
    norm_store4(out + i, r);
}

template <typename T, bool BACKWARD>
__global__ void __launch_bounds__(256)
elu1_kernel(const T *x, const T *g, T *out, const float *mask, int64_t total, int64_t inner_per_mask) {
    // four consecutive elements per thread; `total` and `inner_per_mask` are multiples of 4 when
    // this kernel is chosen with VEC, so a group of four never straddles two mask entries
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= total) return;
    const float w = mask ? mask[i / inner_per_mask] : 1.f;
    float v[4], gv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[j] = i + j < total ? step_load(x + i + j) : 0.f;
        gv[j] = BACKWARD && i + j < total ? step_load(g + i + j) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (i + j >= total) break;
        const float wj = (mask && (inner_per_mask & 3)) ? mask[(i + j) / inner_per_mask] : w;
        float r;
        if (BACKWARD)
            r = gv[j] * wj * (v[j] > 0.f ? 1.f : expf(v[j]));
        else
            r = wj * (v[j] > 0.f ? v[j] + 1.f : expf(v[j]));
        step_store(out + i + j, r);
    }
}

}  // namespace ftb
