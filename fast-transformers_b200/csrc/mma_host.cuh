// Host-side launch logic of the tensor-core mode: TMA descriptors, segment plan, launches.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <utility>

#include "mma_scan.cuh"

namespace ftb {
namespace mma {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime, so the library carries no link
// dependency on libcuda and still loads on a machine without a driver.
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = (EncodeTiledFn)p;
    return fn;
}

// Tensor map over a (N, H, L, dim) view with element strides {n, h, l}.  The innermost
// dimension is the row; the other three are ordered by ascending stride (a permuted view such
// as (N, L, H, dim) storage has the head stride below the position stride), and `pos` receives
// the slot (1..3) of the position, head and batch coordinates.  One box is {128 bytes of the
// row, C positions}.  Returns FTB_OK, FTB_ERR_ALIGNMENT (TMA needs a 16-byte aligned base and
// strides that are positive multiples of 16 bytes) or FTB_ERR_CUDA.
static int make_map(CUtensorMap *map, int *pos, const void *base, int64_t N, int64_t H, int64_t L,
                    int64_t dim, const int64_t *s, int dtype, bool atom32 = false) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return FTB_ERR_CUDA;
    const int64_t es = dtype == FTB_F32 ? 4 : 2;
    if (((uintptr_t)base & 15) != 0) return FTB_ERR_ALIGNMENT;
    // extent, stride and role (0 = position, 1 = head, 2 = batch) of the three outer dimensions;
    // a dimension of extent 1 may carry any stride: give it one larger than everything else
    int64_t ext[3] = {L, H, N}, str[3] = {s[2], s[1], s[0]};
    int role[3] = {0, 1, 2};
    int64_t big = dim;
    for (int i = 0; i < 3; ++i)
        if (ext[i] > 1 && str[i] * ext[i] > big) big = str[i] * ext[i];
    big = (big + 7) / 8 * 8;
    for (int i = 0; i < 3; ++i) {
        if (ext[i] <= 1) str[i] = big * (i + 1);
        if (str[i] <= 0 || (str[i] * es) % 16) return FTB_ERR_ALIGNMENT;
    }
    for (int i = 0; i < 3; ++i)
        for (int j = i + 1; j < 3; ++j)
            if (str[j] < str[i]) {
                std::swap(str[i], str[j]);
                std::swap(ext[i], ext[j]);
                std::swap(role[i], role[j]);
            }
    cuuint64_t gdim[4] = {(cuuint64_t)dim, (cuuint64_t)ext[0], (cuuint64_t)ext[1], (cuuint64_t)ext[2]};
    cuuint64_t gstr[3] = {(cuuint64_t)(str[0] * es), (cuuint64_t)(str[1] * es), (cuuint64_t)(str[2] * es)};
    cuuint32_t box[4] = {(cuuint32_t)(128 / es), 1, 1, 1};
    for (int i = 0; i < 3; ++i) {
        pos[role[i]] = i;
        if (role[i] == 0) box[1 + i] = (cuuint32_t)C;
    }
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = CUDA_SUCCESS;
    for (int attempt = 0; attempt < 2; ++attempt) {
        r = enc(map, dtype == FTB_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                4, const_cast<void *>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_ERROR_INVALID_CONTEXT) break;
        // A thread that has made no runtime call yet (an autograd worker) has no context bound:
        // bind the device's primary context and try once more.
        cudaFree(nullptr);
    }
    if (r != CUDA_SUCCESS && std::getenv("FTB200_DEBUG"))
        fprintf(stderr, "[ftb200] cuTensorMapEncodeTiled failed: %d base=%p dim=%lld ext=(%lld,%lld,%lld) "
                        "stride_bytes=(%llu,%llu,%llu) box=(%u,%u,%u,%u)\n",
                (int)r, base, (long long)dim, (long long)ext[0], (long long)ext[1], (long long)ext[2],
                (unsigned long long)gstr[0], (unsigned long long)gstr[1], (unsigned long long)gstr[2],
                box[0], box[1], box[2], box[3]);
    return r == CUDA_SUCCESS ? FTB_OK : FTB_ERR_ALIGNMENT;
}

struct Plan {
    int64_t seg_len;
    int nseg;
};

// Number of SMs of the calling thread's current device (looked up once per device ordinal; 148, a
// whole B200, when no device can be asked -- a workspace query made on a machine without a GPU).
static int sm_count() {
    static std::atomic<int> cached[64];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        return 148;
    }
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return 148;
    }
    cached[dev].store(n, std::memory_order_relaxed);
    return n;
}

// Segments are whole chunks; one CTA walks one segment.  The count is chosen to minimise
// waves x (chunks per segment + a fixed per-CTA cost) over the device's SMs, with a small charge
// per segment for its state traffic.
constexpr int kSumInKernelMaxSegs = 16;  // the scan kernel adds up at most this many raw totals itself

static Plan plan(int64_t BH, int64_t L, int ntile) {
    Plan p;
    const int64_t chunks = (L + C - 1) / C;
    int64_t best = 1;
    if (chunks > 1 && BH > 0) {
        const int64_t sms = sm_count();
        double best_cost = 1e30;
        for (int64_t t = 1; t <= chunks && t <= 64; ++t) {
            const int64_t cps = (chunks + t - 1) / t;
            const int64_t n = (chunks + cps - 1) / cps;
            const int64_t ctas = BH * n * ntile;
            const int64_t waves = (ctas + sms - 1) / sms;
            const double cost = (double)waves * ((double)cps + 1.0) + 0.3 * (double)n;
            if (cost < best_cost - 1e-9) {
                best_cost = cost;
                best = n;
            }
        }
    }
    if (best < 1) best = 1;
    if (best > chunks) best = chunks > 0 ? chunks : 1;
    int64_t cps = (chunks + best - 1) / best;
    if (cps < 1) cps = 1;
    p.seg_len = cps * C;
    p.nseg = (int)((L + p.seg_len - 1) / p.seg_len);
    if (p.nseg < 1) p.nseg = 1;
    return p;
}

// Which (dtype, Da, Dc) combinations have a tensor-core kernel.
static bool supported(int dtype, int64_t Da, int64_t Dc) {
    if (dtype == FTB_F32) return Da == 64 && Dc % 64 == 0 && Dc >= 64;
    return (Da == 128 && Dc % 128 == 0 && Dc >= 128) || (Da == 64 && Dc % 64 == 0 && Dc >= 64);
}

// Every grid is started with programmatic stream serialisation: its blocks may be placed while
// the launch in front of it in the stream drains.  `after_own_launch`: that launch is this
// library's own, of the same call (the state-only sweep): the blocks wait for it only where they
// read what it wrote.  Otherwise they wait for it before they touch global memory at all
// (ScanBatch::wait_first), which is safe behind any kernel and overlaps the block set-up only.
// Environment (fault finding): FTB200_NO_PDL=1 ordinary launches throughout.
template <typename T, int DA, int DCT, bool APPLY = false>
static cudaError_t launch_t(ScanBatch &batch, cudaStream_t st, bool after_own_launch) {
    using K = Cfg<T, DA, DCT>;
    auto kern = mma_scan_kernel<T, DA, DCT, APPLY>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)K::SMEM);
    if (e != cudaSuccess) return e;
    static const char *no_pdl = std::getenv("FTB200_NO_PDL");
    batch.wait_first = 0;
    if (no_pdl) {
        kern<<<(unsigned)batch.first_block[batch.njobs], NTHREADS, K::SMEM, st>>>(batch);
        return cudaGetLastError();
    }
    batch.wait_first = after_own_launch ? 0 : 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)batch.first_block[batch.njobs]);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = K::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, batch);
    if (e == cudaSuccess) return e;
    // a context that does not take the attribute: the same grid as an ordinary launch
    (void)cudaGetLastError();
    batch.wait_first = 0;
    kern<<<(unsigned)batch.first_block[batch.njobs], NTHREADS, K::SMEM, st>>>(batch);
    return cudaGetLastError();
}

}  // namespace mma
}  // namespace ftb
