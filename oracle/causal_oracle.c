/*
 * CPU restatement of the causal linear-attention product.  TEST INFRASTRUCTURE ONLY:
 * this file is the checker (and the "port" CPU baseline), never a product code path.
 *
 * It restates the recurrence of the reference's OpenMP kernel
 *   fast_transformers/causal_product/causal_product_cpu.cpp:82-124  (forward)
 *   fast_transformers/causal_product/causal_product_cpu.cpp:133-209 (backward)
 * for one (batch, head) pair at a time:
 *
 *   forward : S += k_l (x) v_l ;  out_l = q_l . S              (l ascending, :106-121)
 *   backward: S += k_l (x) v_l ;  gq_l  = S . g_l              (l ascending, :165-180)
 *             R += q_l (x) g_l ;  gk_l  = R . v_l ; gv_l = k_l . R   (l descending, :184-206)
 *
 * The state is updated BEFORE it is read, so position l attends to itself (j <= l).
 * Tensors are (N, H, L, dim) with the last dimension contiguous and arbitrary element
 * strides for the other three, like the reference's 4-D accessors.  The *_f32 entry
 * points keep every intermediate in fp32 in the reference's summation order; the *_f64
 * entry points take the same fp32 inputs and accumulate in double (the tolerance anchor).
 * (batch, head) pairs run in parallel under OpenMP exactly as in the reference (:101,:158).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    int64_t sn, sh, sl; /* element strides of batch, head and sequence position */
} strides_t;

#define ROW(p, s, n, h, l) ((p) + (n) * (s).sn + (h) * (s).sh + (l) * (s).sl)

#define DEFINE_ORACLE(SUFFIX, ACC)                                                          \
    void causal_oracle_forward_##SUFFIX(const float *q, const float *k, const float *v,     \
                                        ACC *out, int64_t N, int64_t H, int64_t L,          \
                                        int64_t D, int64_t M, const int64_t *qs,            \
                                        const int64_t *ks, const int64_t *vs,               \
                                        const int64_t *os) {                                \
        strides_t sq = {qs[0], qs[1], qs[2]}, sk = {ks[0], ks[1], ks[2]};                   \
        strides_t sv = {vs[0], vs[1], vs[2]}, so = {os[0], os[1], os[2]};                   \
        _Pragma("omp parallel for collapse(2)") for (int64_t n = 0; n < N; n++) {           \
            for (int64_t h = 0; h < H; h++) {                                               \
                ACC *S = (ACC *)calloc((size_t)(D * M), sizeof(ACC));                       \
                for (int64_t l = 0; l < L; l++) {                                           \
                    const float *ql = ROW(q, sq, n, h, l), *kl = ROW(k, sk, n, h, l);       \
                    const float *vl = ROW(v, sv, n, h, l);                                  \
                    ACC *ol = ROW(out, so, n, h, l);                                        \
                    for (int64_t d = 0; d < D; d++)                                         \
                        for (int64_t m = 0; m < M; m++)                                     \
                            S[d * M + m] += (ACC)kl[d] * (ACC)vl[m];                        \
                    for (int64_t m = 0; m < M; m++) ol[m] = 0;                              \
                    for (int64_t d = 0; d < D; d++)                                         \
                        for (int64_t m = 0; m < M; m++)                                     \
                            ol[m] += (ACC)ql[d] * S[d * M + m];                             \
                }                                                                           \
                free(S);                                                                    \
            }                                                                               \
        }                                                                                   \
    }                                                                                       \
                                                                                            \
    void causal_oracle_backward_##SUFFIX(                                                   \
        const float *q, const float *k, const float *v, const float *g, ACC *gq, ACC *gk,   \
        ACC *gv, int64_t N, int64_t H, int64_t L, int64_t D, int64_t M, const int64_t *qs,  \
        const int64_t *ks, const int64_t *vs, const int64_t *gs, const int64_t *gqs,        \
        const int64_t *gks, const int64_t *gvs) {                                           \
        strides_t sq = {qs[0], qs[1], qs[2]}, sk = {ks[0], ks[1], ks[2]};                   \
        strides_t sv = {vs[0], vs[1], vs[2]}, sg = {gs[0], gs[1], gs[2]};                   \
        strides_t sgq = {gqs[0], gqs[1], gqs[2]}, sgk = {gks[0], gks[1], gks[2]};           \
        strides_t sgv = {gvs[0], gvs[1], gvs[2]};                                           \
        _Pragma("omp parallel for collapse(2)") for (int64_t n = 0; n < N; n++) {           \
            for (int64_t h = 0; h < H; h++) {                                               \
                ACC *S = (ACC *)calloc((size_t)(D * M), sizeof(ACC));                       \
                for (int64_t l = 0; l < L; l++) {                                           \
                    const float *kl = ROW(k, sk, n, h, l), *vl = ROW(v, sv, n, h, l);       \
                    const float *gl = ROW(g, sg, n, h, l);                                  \
                    ACC *o = ROW(gq, sgq, n, h, l);                                         \
                    for (int64_t d = 0; d < D; d++)                                         \
                        for (int64_t m = 0; m < M; m++)                                     \
                            S[d * M + m] += (ACC)kl[d] * (ACC)vl[m];                        \
                    for (int64_t d = 0; d < D; d++) {                                       \
                        ACC s = 0;                                                          \
                        for (int64_t m = 0; m < M; m++) s += (ACC)gl[m] * S[d * M + m];     \
                        o[d] = s;                                                           \
                    }                                                                       \
                }                                                                           \
                memset(S, 0, (size_t)(D * M) * sizeof(ACC));                                \
                for (int64_t l = L - 1; l >= 0; l--) {                                      \
                    const float *ql = ROW(q, sq, n, h, l), *kl = ROW(k, sk, n, h, l);       \
                    const float *vl = ROW(v, sv, n, h, l), *gl = ROW(g, sg, n, h, l);       \
                    ACC *ok = ROW(gk, sgk, n, h, l), *ov = ROW(gv, sgv, n, h, l);           \
                    for (int64_t d = 0; d < D; d++)                                         \
                        for (int64_t m = 0; m < M; m++)                                     \
                            S[d * M + m] += (ACC)ql[d] * (ACC)gl[m];                        \
                    for (int64_t d = 0; d < D; d++) {                                       \
                        ACC s = 0;                                                          \
                        for (int64_t m = 0; m < M; m++) s += (ACC)vl[m] * S[d * M + m];     \
                        ok[d] = s;                                                          \
                    }                                                                       \
                    for (int64_t m = 0; m < M; m++) ov[m] = 0;                              \
                    for (int64_t d = 0; d < D; d++)                                         \
                        for (int64_t m = 0; m < M; m++)                                     \
                            ov[m] += (ACC)kl[d] * S[d * M + m];                             \
                }                                                                           \
                free(S);                                                                    \
            }                                                                               \
        }                                                                                   \
    }

DEFINE_ORACLE(f32, float)
DEFINE_ORACLE(f64, double)
