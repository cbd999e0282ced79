// C ABI of the B200 causal linear-attention kernels (see include/ftb200.h for the contract
// and for the reference functions each entry point replaces).
#include "ftb200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

#include "apply_state.cuh"
#include "favor_map.cuh"
#include "feature_map.cuh"
#include "mma_host.cuh"
#include "wide_scan.cuh"
#include "x3_scan.cuh"
#include "rank_exchange.cuh"
#include "recurrent_step.cuh"
#include "simt_scan.cuh"

namespace ftb {

static thread_local int g_last_cuda_error = 0;

static inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return FTB_ERR_CUDA;
}
#define FTB_CUDA(call)                                   \
    do {                                                 \
        cudaError_t e__ = (call);                        \
        if (e__ != cudaSuccess) return cuda_fail(e__);   \
    } while (0)

// ---- launch accounting --------------------------------------------------------------------
// A process-wide count of kernel launches, and an optional recorder that brackets every
// launch (of any host thread: autograd runs the backward on its own) with CUDA events on the
// launching stream so a caller can attribute device time to kernel kinds (FTB_KERNEL_*).
// Off by default; it changes nothing else.
static std::atomic<uint64_t> g_launches{0};

struct TimedSpan {
    int kind;
    cudaEvent_t beg, end;
};
static std::atomic<bool> g_timing{false};
static std::mutex g_spans_mutex;
static std::vector<TimedSpan> g_spans;

struct LaunchScope {
    cudaStream_t st;
    cudaEvent_t end = nullptr;
    LaunchScope(int kind, cudaStream_t s) : st(s) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (!g_timing.load(std::memory_order_relaxed)) return;
        TimedSpan sp;
        sp.kind = kind;
        if (cudaEventCreate(&sp.beg) != cudaSuccess) return;
        if (cudaEventCreate(&sp.end) != cudaSuccess) {
            cudaEventDestroy(sp.beg);
            return;
        }
        cudaEventRecord(sp.beg, st);
        end = sp.end;
        std::lock_guard<std::mutex> lock(g_spans_mutex);
        g_spans.push_back(sp);
    }
    ~LaunchScope() {
        if (end) cudaEventRecord(end, st);
    }
};

// ---- segment plan (pure function of the shape, so the workspace query needs no device) --
struct Plan {
    int64_t seg_len;
    int nseg;
    int64_t dm = 0;   // D * M: elements of one state block (set by choose_plan)
};

constexpr int64_t kMinSegRows = 4 * CH;
constexpr int kSimtMaxDim = 512;

static Plan simt_plan(int64_t BH, int64_t L) {
    Plan p;
    if (L <= 0 || BH <= 0) {
        p.seg_len = kMinSegRows;
        p.nseg = 1;
        return p;
    }
    int64_t want = ((int64_t)mma::sm_count() * 4 + BH - 1) / BH;
    if (want < 1) want = 1;
    int64_t len = (L + want - 1) / want;
    len = (len + CH - 1) / CH * CH;
    if (len < kMinSegRows) len = kMinSegRows;
    p.seg_len = len;
    p.nseg = (int)((L + len - 1) / len);
    return p;
}

static inline Strides3 S3(const int64_t *s) { return Strides3{s[0], s[1], s[2]}; }

static inline bool vec_ok(const void *ptr, const int64_t *s, int dtype) {
    uintptr_t a = (uintptr_t)ptr;
    size_t bytes = dtype == FTB_F32 ? 16 : 8;
    return (a % bytes == 0) && (s[0] % 4 == 0) && (s[1] % 4 == 0) && (s[2] % 4 == 0);
}

// ---- launches ---------------------------------------------------------------------------
static int simt_launch_state_sum(const void *x, const void *y, const int64_t *xs, const int64_t *ys,
                            int64_t N, int64_t H, int64_t L, int D, int M, int dtype, Plan pl,
                            float *states, cudaStream_t st) {
    StateSumArgs a;
    a.x = x; a.y = y; a.sx = S3(xs); a.sy = S3(ys);
    a.H = (int)H; a.L = L; a.D = D; a.M = M;
    a.seg_len = pl.seg_len; a.nseg = pl.nseg; a.states = states;
    a.vx = vec_ok(x, xs, dtype); a.vy = vec_ok(y, ys, dtype);
    int64_t blocks = N * H * pl.nseg * ((D + KT - 1) / KT) * ((M + NC - 1) / NC);
    if (blocks <= 0) return FTB_OK;
    if (blocks > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    LaunchScope scope(FTB_KERNEL_STATE_SUM, st);
    if (dtype == FTB_F32)
        simt_state_sum_kernel<float><<<(unsigned)blocks, NTHR, 0, st>>>(a);
    else
        simt_state_sum_kernel<__nv_bfloat16><<<(unsigned)blocks, NTHR, 0, st>>>(a);
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

static int launch_prefix(float *states, const float *init, float *total, const float *total_init,
                         int64_t BH, int nseg,
                         int64_t DM, int reverse, cudaStream_t st) {
    int64_t n = BH * DM;
    if (n <= 0) return FTB_OK;
    LaunchScope scope(FTB_KERNEL_STATE_PREFIX, st);
    auto aligned = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    if (DM % 4 == 0 && aligned(states) && aligned(init) && aligned(total) && aligned(total_init)) {
        const int64_t n4 = n / 4;
        state_prefix4_kernel<<<(unsigned)((n4 + 127) / 128), 128, 0, st>>>(
            (float4 *)states, (const float4 *)init, (float4 *)total, (const float4 *)total_init, BH, nseg,
            DM / 4, reverse);
    } else {
        state_prefix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(states, init, total, total_init, BH,
                                                                        nseg, DM, reverse);
    }
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

template <typename TI, typename TO>
static int launch_scan_t(const ScanArgs &a, int64_t blocks, size_t smem, cudaStream_t st) {
    if (smem > 48 * 1024)
        FTB_CUDA(cudaFuncSetAttribute(simt_scan_kernel<TI, TO>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LaunchScope scope(FTB_KERNEL_SIMT_SCAN, st);
    simt_scan_kernel<TI, TO><<<(unsigned)blocks, NTHR, smem, st>>>(a);
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

static int simt_launch_scan(const void *a, const void *b, const void *c, void *out, const int64_t *as,
                       const int64_t *bs, const int64_t *cs, const int64_t *os, int64_t N,
                       int64_t H, int64_t L, int Da, int Dc, int dtype, Plan pl,
                       const float *states, int nseg_states, int canon_is_DaDc, int reverse,
                       cudaStream_t st) {
    ScanArgs p;
    p.a = a; p.b = b; p.c = c; p.out = out;
    p.sa = S3(as); p.sb = S3(bs); p.sc = S3(cs); p.so = S3(os);
    p.H = (int)H; p.L = L; p.Da = Da; p.Dc = Dc;
    p.seg_len = pl.seg_len; p.nseg = pl.nseg;
    p.states = states; p.canon_is_DaDc = canon_is_DaDc; p.reverse = reverse;
    p.va = vec_ok(a, as, dtype); p.vb = vec_ok(b, bs, dtype);
    p.vc = vec_ok(c, cs, dtype); p.vo = vec_ok(out, os, dtype);
    (void)nseg_states;
    int64_t blocks = N * H * pl.nseg * ((Dc + NC - 1) / NC);
    if (blocks <= 0) return FTB_OK;
    if (blocks > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    size_t smem = scan_smem_bytes(Da);
    if (dtype == FTB_F32) return launch_scan_t<float, float>(p, blocks, smem, st);
    return launch_scan_t<__nv_bfloat16, __nv_bfloat16>(p, blocks, smem, st);
}

// Per-row normaliser of a scan's output: row i is multiplied by 1 / (den[i] + eps) as it is stored.
struct RowScale {
    const float *den;
    Strides3 s;      // element strides of {batch, head, position}
    float eps;
};

// ---- tensor-core launches -------------------------------------------------------------------
// A launch carries up to mma::MAX_JOBS independent jobs over one problem shape.
struct MmaBatch {
    mma::ScanBatch b;
    int dtype = FTB_F32;
    int da = 64;                     // width of the a / b rows (selects the instantiation)
    int kind = FTB_KERNEL_MMA_FWD;
    bool after_own_launch = false;   // see mma::launch_t
    bool apply = false;              // out = a S_init only (the APPLY instantiation)
    MmaBatch() { b.njobs = 0; b.first_block[0] = 0; b.interleave = 0; b.wait_first = 0; }
};

// Append one job (a scan, or a state-only sweep when `a` is null) to `batch`.
static int mma_add_job(MmaBatch &batch, const void *a, const void *b, const void *c, void *out,
                       const int64_t *as, const int64_t *bs, const int64_t *cs, const int64_t *os,
                       int64_t N, int64_t H, int64_t L, int Da, int Dc, int dtype, Plan pl,
                       const float *states, const float *init, int sum_mode, int sub, float *state_out,
                       int skip_lo, int skip_hi, int canon_is_DaDc, int reverse,
                       const RowScale *scale = nullptr, int64_t state_blk = 0) {
    const bool state_only = (a == nullptr);
    const bool apply_only = (b == nullptr);   // out = a S_init: only `a` is read
    const int DCT = (dtype == FTB_F32 || Da == 64) ? 64 : 128;
    // fp32 (TF32) operands read MN-major need the 32-byte-atom swizzle; bf16 uses one image
    const bool atom32 = dtype == FTB_F32;
    int64_t blocks = N * H * pl.nseg * (Dc / DCT);
    if (blocks <= 0) return FTB_OK;
    if (batch.b.njobs >= mma::MAX_JOBS) return FTB_ERR_INVALID;
    if (batch.b.first_block[batch.b.njobs] + blocks > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    mma::ScanJob &J = batch.b.job[batch.b.njobs];
    mma::ScanParams &p = J.p;
    int rc = FTB_OK;
    if (!apply_only) {
        rc = mma::make_map(&J.mb, p.pos_b, b, N, H, L, Da, bs, dtype, false);
        if (rc) return rc;
        rc = mma::make_map(&J.mbmn, p.pos_b, b, N, H, L, Da, bs, dtype, atom32);
        if (rc) return rc;
        rc = mma::make_map(&J.mc, p.pos_c, c, N, H, L, Dc, cs, dtype, atom32);
        if (rc) return rc;
    }
    if (state_only) {
        J.ma = J.mb;
        for (int i = 0; i < 3; ++i) p.pos_a[i] = p.pos_b[i];
    } else {
        rc = mma::make_map(&J.ma, p.pos_a, a, N, H, L, Da, as, dtype);
        if (rc) return rc;
        if (apply_only) {
            J.mb = J.mbmn = J.mc = J.ma;   // never dereferenced by the APPLY instantiation
            for (int i = 0; i < 3; ++i) p.pos_b[i] = p.pos_c[i] = p.pos_a[i];
            batch.apply = true;
        }
        const int64_t es = dtype == FTB_F32 ? 4 : 2;
        if (((uintptr_t)out & 15) || (os[0] * es) % 16 || (os[1] * es) % 16 || (os[2] * es) % 16) {
            if (std::getenv("FTB200_DEBUG"))
                fprintf(stderr, "[ftb200] output alignment: %p strides %lld %lld %lld\n", out,
                        (long long)os[0], (long long)os[1], (long long)os[2]);
            return FTB_ERR_ALIGNMENT;
        }
    }
    p.out = out;
    p.so = state_only ? Strides3{0, 0, 0} : S3(os);
    p.H = (int)H; p.L = L; p.Dc = Dc;
    p.seg_len = pl.seg_len; p.nseg = pl.nseg;
    p.states = states; p.state_out = state_out;
    p.init = init; p.sum_mode = sum_mode; p.sub = sub < 1 ? 1 : sub;
    p.skip_lo = skip_lo; p.skip_hi = skip_hi;
    p.canon_is_DaDc = canon_is_DaDc; p.reverse = reverse; p.state_only = state_only ? 1 : 0;
    p.row_den = scale ? scale->den : nullptr;
    p.sden = scale ? scale->s : Strides3{0, 0, 0};
    p.eps = scale ? scale->eps : 0.f;
    p.state_blk = state_blk;
    if (batch.b.njobs == 0) {
        batch.dtype = dtype;
        batch.da = Da;
        batch.kind = state_only ? FTB_KERNEL_MMA_STATE : (reverse ? FTB_KERNEL_MMA_BWD : FTB_KERNEL_MMA_FWD);
    }
    batch.b.first_block[batch.b.njobs + 1] = batch.b.first_block[batch.b.njobs] + (int)blocks;
    ++batch.b.njobs;
    return FTB_OK;
}

static int mma_launch_batch(MmaBatch &batch, cudaStream_t st) {
    if (batch.b.njobs == 0) return FTB_OK;
    for (int j = batch.b.njobs; j < mma::MAX_JOBS; ++j) batch.b.first_block[j + 1] = batch.b.first_block[j];
    // equal-sized scans are interleaved block by block (shared tiles meet in L2)
    bool equal = batch.b.njobs > 1;
    for (int j = 0; j < batch.b.njobs && equal; ++j)
        equal = batch.b.job[j].p.state_only == batch.b.job[0].p.state_only &&
                (!batch.b.job[j].p.state_only || batch.b.job[j].p.state_blk != 0) &&
                batch.b.first_block[j + 1] - batch.b.first_block[j] == batch.b.first_block[1];
    batch.b.interleave = equal ? 1 : 0;
    LaunchScope scope(batch.kind, st);
    cudaError_t e;
    if (batch.apply) {
        batch.b.interleave = 0;
        if (batch.dtype == FTB_F32)
            e = mma::launch_t<float, 64, 64, true>(batch.b, st, false);
        else if (batch.da == 64)
            e = mma::launch_t<__nv_bfloat16, 64, 64, true>(batch.b, st, false);
        else
            e = mma::launch_t<__nv_bfloat16, 128, 128, true>(batch.b, st, false);
    } else if (batch.dtype == FTB_F32)
        e = mma::launch_t<float, 64, 64>(batch.b, st, batch.after_own_launch);
    else if (batch.da == 64)
        e = mma::launch_t<__nv_bfloat16, 64, 64>(batch.b, st, batch.after_own_launch);
    else
        e = mma::launch_t<__nv_bfloat16, 128, 128>(batch.b, st, batch.after_own_launch);
    if (e != cudaSuccess) return cuda_fail(e);
    return FTB_OK;
}

static int mma_launch(const void *a, const void *b, const void *c, void *out, const int64_t *as,
                      const int64_t *bs, const int64_t *cs, const int64_t *os, int64_t N, int64_t H,
                      int64_t L, int Da, int Dc, int dtype, Plan pl, const float *states,
                      const float *init, int sum_mode, int sub, float *state_out, int skip_lo, int skip_hi,
                      int canon_is_DaDc, int reverse, cudaStream_t st, bool after_own_launch = false,
                      const RowScale *scale = nullptr) {
    MmaBatch batch;
    batch.after_own_launch = after_own_launch;
    int rc = mma_add_job(batch, a, b, c, out, as, bs, cs, os, N, H, L, Da, Dc, dtype, pl, states, init,
                         sum_mode, sub, state_out, skip_lo, skip_hi, canon_is_DaDc, reverse, scale);
    if (rc) return rc;
    return mma_launch_batch(batch, st);
}

static Plan choose_plan(int mode, int64_t BH, int64_t L, int64_t DM) {
    Plan p;
    if (mode == FTB_MODE_MMA) {
        mma::Plan m = mma::plan(BH, L, 1);
        p.seg_len = m.seg_len;
        p.nseg = m.nseg;
    } else {
        p = simt_plan(BH, L);
    }
    p.dm = DM;
    return p;
}

static int launch_state_sum(int mode, const void *x, const void *y, const int64_t *xs,
                            const int64_t *ys, int64_t N, int64_t H, int64_t L, int D, int M,
                            int dtype, Plan pl, float *states, int skip_lo, int skip_hi,
                            cudaStream_t st) {
    if (mode == FTB_MODE_MMA)
        return mma_launch(nullptr, x, y, nullptr, nullptr, xs, ys, nullptr, N, H, L, D, M, dtype, pl,
                          nullptr, nullptr, 0, 1, states, skip_lo, skip_hi, 1, 0, st);
    return simt_launch_state_sum(x, y, xs, ys, N, H, L, D, M, dtype, pl, states, st);
}

// Where a scan finds the state each of its segments starts from.
struct SegStates {
    const float *states;  // per (bh, seg) blocks, or nullptr
    const float *init;    // per bh block added on top, or nullptr
    int sum_mode;         // 1: `states` are raw totals the kernel adds up itself
    int sub;              // sum_mode 1: blocks per segment
    int fresh = 0;        // written by a launch of this call, directly in front of the scan's
};

static int launch_scan(int mode, const void *a, const void *b, const void *c, void *out,
                       const int64_t *as, const int64_t *bs, const int64_t *cs, const int64_t *os,
                       int64_t N, int64_t H, int64_t L, int Da, int Dc, int dtype, Plan pl,
                       SegStates ss, int canon_is_DaDc, int reverse, cudaStream_t st,
                       const RowScale *scale = nullptr) {
    if (mode == FTB_MODE_MMA)
        return mma_launch(a, b, c, out, as, bs, cs, os, N, H, L, Da, Dc, dtype, pl, ss.states, ss.init,
                          ss.sum_mode, ss.sub, nullptr, 0, 0, canon_is_DaDc, reverse, st, ss.fresh != 0,
                          scale);
    return simt_launch_scan(a, b, c, out, as, bs, cs, os, N, H, L, Da, Dc, dtype, pl,
                            ss.states ? ss.states : ss.init, pl.nseg, canon_is_DaDc, reverse, st);
}

// The tensor-core scan can add up raw segment totals itself (no prefix launch) -- worth it while
// the sum is short or the segments are long: every state-worker thread of a block walks the
// blocks in front of its segment row by row, batches of dependent loads that take ~13 us per grid
// for 8 blocks of 64 KB (config 4's shape) and are invisible for 3 blocks of 16 KB (config 2).
// Measured on config 4's recipe, one GPU, in-kernel sums against a prefix launch: 0.304 / 0.283 ms
// at L = 16384, 0.512 / 0.498 ms at 32768, 0.934 / 0.931 ms at 65536, 3.63 / 3.81 ms at 262144
// (there the prefix form also loses the sweep of (Q, grad_out) riding beside grad_Q).
constexpr int64_t kSumInKernelMaxBytes = 128 * 1024;
constexpr int64_t kSumInKernelAlwaysFromChunks = 64;   // segments this long amortise any sum
static inline bool sums_in_kernel(int mode, Plan pl) {
    if (mode != FTB_MODE_MMA || pl.nseg > mma::kSumInKernelMaxSegs) return false;
    return (int64_t)(pl.nseg - 1) * pl.dm * 4 <= kSumInKernelMaxBytes ||
           pl.seg_len / mma::C > kSumInKernelAlwaysFromChunks;
}

// The state-only launch reads (D+M)/(2D+2M) of what a scan reads, so on the scan's own segments it
// would leave most SMs idle: it runs on `sub` times finer segments (sub blocks per segment in the
// workspace).  `sub` is a function of the shape alone, so whoever wrote the states of a workspace
// (a forward call with or without final_state, ftb_causal_state_sum) and whoever reads them later
// (the scan of the same call, a backward call given `forward_workspace`) agree on the layout.
static int state_sub(int mode, Plan pl, int64_t BH) {
    if (!sums_in_kernel(mode, pl) || pl.nseg < 2) return 1;
    const int64_t cps = pl.seg_len / mma::C;
    for (int sub = 4; sub >= 2; --sub)
        if (cps % sub == 0 && BH * (pl.nseg - 1) * sub <= (int64_t)mma::sm_count() * 13 / 12 && pl.nseg * sub <= 16) return sub;
    return 1;
}

// Describe segment-start states that sit in `ws` (written by prepare_states).
static SegStates describe_states(int mode, Plan pl, const float *ws, const float *init, int64_t BH) {
    if (pl.nseg == 1) return SegStates{nullptr, init, 0, 1};
    if (sums_in_kernel(mode, pl)) return SegStates{ws, init, 1, state_sub(mode, pl, BH)};
    // exclusive prefixes: the tensor-core kernel adds `init` itself, the fp32 kernel reads one
    // block per segment, so there `init` is folded into the prefixes
    if (mode == FTB_MODE_MMA) return SegStates{ws, init, 0, 1};
    return SegStates{ws, nullptr, 0, 1};
}

// Per-segment totals of sum x (x) y into `ws`, turned into what the scans read; optionally the
// grand total (init + all segments) into `total`.
static int prepare_states(int mode, const void *x, const void *y, const int64_t *xs, const int64_t *ys,
                          int64_t N, int64_t H, int64_t L, int D, int M, int dtype, Plan pl, float *ws,
                          const float *init, float *total, int reverse, cudaStream_t st,
                          SegStates *out) {
    *out = describe_states(mode, pl, ws, init, N * H);
    if (pl.nseg == 1 && !total) return FTB_OK;
    int rc;
    if (sums_in_kernel(mode, pl)) {
        const int sub = out->sub;
        Plan fine = pl;
        fine.seg_len = pl.seg_len / sub;
        fine.nseg = pl.nseg * sub;
        int skip_lo = 0, skip_hi = 0;   // the segment nobody reads from: last (forward) / first
        if (!total) {
            skip_lo = reverse ? 0 : (pl.nseg - 1) * sub;
            skip_hi = skip_lo + sub;
        }
        rc = launch_state_sum(mode, x, y, xs, ys, N, H, L, D, M, dtype, fine, ws, skip_lo, skip_hi, st);
        out->fresh = 1;
        if (rc || !total) return rc;
        int64_t n = N * H * (int64_t)D * M;
        LaunchScope scope(FTB_KERNEL_STATE_PREFIX, st);
        state_total_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ws, init, total, N * H, fine.nseg,
                                                                       (int64_t)D * M);
        FTB_CUDA(cudaGetLastError());
        return FTB_OK;
    }
    rc = launch_state_sum(mode, x, y, xs, ys, N, H, L, D, M, dtype, pl, ws, 0, 0, st);
    if (rc) return rc;
    const bool fold = mode != FTB_MODE_MMA;
    rc = launch_prefix(ws, fold ? init : nullptr, total, fold ? nullptr : init, N * H, pl.nseg,
                       (int64_t)D * M, reverse, st);
    if (pl.nseg == 1) *out = SegStates{ws, fold ? nullptr : init, 0, 1};
    out->fresh = 1;
    return rc;
}

// Tensor-core mode, fp32, widths that are multiples of 64 with at least one of them above 64 (the
// Favor map gives D = 256 for M = 64): served by the wide scans (wide_scan.cuh), which take the sum
// over 64-wide feature blocks inside the tensor cores, one launch per 64 columns of the narrow side
// and per group of four feature blocks.  Returns the number of feature blocks D / 64, or 0.
static int wide_blocks(int mode, int dtype, int64_t D, int64_t M) {
    if (mode != FTB_MODE_MMA || dtype != FTB_F32 || D < 64 || M < 64 || D % 64 || M % 64) return 0;
    if (D == 64 && M == 64) return 0;
    return (int)(D / 64);
}

// Segments of the split-operand tensor-core mode (fp32, D = M = 64): one CTA per (pair, segment).
static Plan x3_plan(int64_t BH, int64_t L) {
    Plan p;
    mma::Plan m = mma::plan(BH, L, 1);
    p.seg_len = m.seg_len;
    p.nseg = m.nseg;
    p.dm = 4096;
    return p;
}

// The state-only sweep of the split-operand mode runs on `sub` times finer segments where that
// fills more SMs (a function of the shape alone: forward and backward agree on the layout).
static int x3_sub(Plan pl, int64_t BH) {
    if (pl.nseg < 2 || pl.nseg > mma::kSumInKernelMaxSegs) return 1;
    const int64_t cps = pl.seg_len / mma::C;
    for (int sub = 4; sub >= 2; --sub)
        if (cps % sub == 0 && BH * (pl.nseg - 1) * sub <= (int64_t)mma::sm_count() * 13 / 12 &&
            pl.nseg * sub <= mma::kSumInKernelMaxSegs)
            return sub;
    return 1;
}

// Segments of the wide form.  The scans that are wide on the a / b side walk all feature blocks of
// a segment in one CTA, so the plan counts one CTA per (pair, segment); the scans that are wide on
// the c side then run nb column tiles per segment side by side.  Whether the scans add up raw
// totals themselves is decided on what ONE 64-row block needs (a 64 x M block per segment).
struct WidePlan {
    Plan pl;      // pl.dm = 64 * M
    int sub;      // blocks per segment written by the state-only sweeps (state_sub)
};
static WidePlan wide_plan(int64_t BH, int64_t L, int nb, int64_t M) {
    WidePlan w;
    mma::Plan m = mma::plan(BH, L, 1);
    w.pl.seg_len = m.seg_len;
    w.pl.nseg = m.nseg;
    w.pl.dm = 64 * 64;
    w.sub = state_sub(FTB_MODE_MMA, w.pl, BH * nb * (M / 64));
    return w;
}

static int check_common(int64_t N, int64_t H, int64_t L, int64_t D, int64_t M, int dtype, int mode,
                        bool x3_ok = false) {
    if (N < 0 || H < 0 || L < 0 || D < 0 || M < 0) return FTB_ERR_INVALID;
    if (dtype != FTB_F32 && dtype != FTB_BF16) return FTB_ERR_INVALID;
    if (mode != FTB_MODE_FP32_SIMT && mode != FTB_MODE_MMA && mode != FTB_MODE_MMA_X3) return FTB_ERR_INVALID;
    // split-operand tensor-core mode: the product and its backward only, fp32, D = M = 64
    if (mode == FTB_MODE_MMA_X3 && D > 0 && M > 0 && (!x3_ok || dtype != FTB_F32 || D != 64 || M != 64))
        return FTB_ERR_UNSUPPORTED;
    if (mode == FTB_MODE_FP32_SIMT && (D > kSimtMaxDim || M > kSimtMaxDim)) return FTB_ERR_UNSUPPORTED;
    if (mode == FTB_MODE_MMA && D > 0 && M > 0 &&
        !(mma::supported(dtype, D, M) && mma::supported(dtype, M, D)) && !wide_blocks(mode, dtype, D, M))
        return FTB_ERR_UNSUPPORTED;
    return FTB_OK;
}

static inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace ftb

namespace ftb {
struct NormPlan {
    int nseg;
    int64_t seg_len;
};
constexpr int kNormMaxSegs = 64;
// `ctas_wanted`: how many (sequence, segment) work items should exist; segments are whole 32-row
// tiles, at least `min_rows` long, at most kNormMaxSegs per sequence
static NormPlan norm_plan(int64_t BH, int64_t L, int64_t items_wanted, int64_t min_rows) {
    int64_t want = (items_wanted + BH - 1) / BH;
    if (want < 1) want = 1;
    if (want > kNormMaxSegs) want = kNormMaxSegs;
    int64_t seg = (L + want - 1) / want;
    seg = (seg + kNormRows - 1) / kNormRows * kNormRows;
    if (seg < min_rows) seg = min_rows;
    NormPlan pl;
    pl.seg_len = seg;
    pl.nseg = (int)((L + seg - 1) / seg);
    if (pl.nseg < 1) pl.nseg = 1;
    return pl;
}
// The register-streaming kernels take D in {16, 32, 64, 128} with rows that start on 16-byte
// (fp32) / 8-byte (bf16) boundaries; everything else goes through the shared-memory kernels.
static bool norm_fast_ok(const NormParams &p, int dtype, bool vec_out) {
    if (p.D != 16 && p.D != 32 && p.D != 64 && p.D != 128) return false;
    const uintptr_t a = dtype == FTB_F32 ? 15 : 7;
    auto ok = [&](const void *ptr, const Strides3n &s) {
        return ((uintptr_t)ptr & a) == 0 && s.n % 4 == 0 && s.h % 4 == 0 && s.l % 4 == 0;
    };
    if (!ok(p.q, p.qs) || !ok(p.k, p.ks)) return false;
    if (vec_out && !ok(p.out, p.os)) return false;
    return true;
}
template <typename T, int LPR, int MODE>
static int norm_launch_fast_mode(const NormParams &p, int64_t groups, int64_t blocks, cudaStream_t st) {
    if (p.nseg > 1) {
        LaunchScope scope(FTB_KERNEL_NORMALISER, st);
        norm_stream_kernel<T, LPR, MODE, true><<<(unsigned)blocks, kNormThreads, 0, st>>>(p, groups);
        FTB_CUDA(cudaGetLastError());
    }
    LaunchScope scope(FTB_KERNEL_NORMALISER, st);
    norm_stream_kernel<T, LPR, MODE, false><<<(unsigned)blocks, kNormThreads, 0, st>>>(p, groups);
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}
template <typename T, int LPR>
static int norm_launch_fast(NormParams p, int64_t BH, cudaStream_t st) {
    constexpr int per_cta = kNormThreads / LPR;
    NormPlan pl = norm_plan(BH, p.L, (int64_t)mma::sm_count() * 4 * per_cta, 2 * kNormRows);
    p.nseg = pl.nseg;
    p.seg_len = pl.seg_len;
    const int64_t groups = BH * p.nseg;
    const int64_t blocks = (groups + per_cta - 1) / per_cta;
    if (blocks > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    if (p.mode == NORM_FWD) return norm_launch_fast_mode<T, LPR, NORM_FWD>(p, groups, blocks, st);
    if (p.mode == NORM_BWD_Q) return norm_launch_fast_mode<T, LPR, NORM_BWD_Q>(p, groups, blocks, st);
    return norm_launch_fast_mode<T, LPR, NORM_BWD_K>(p, groups, blocks, st);
}
template <typename T>
static int norm_launch(NormParams p, int64_t BH, int dtype, cudaStream_t st) {
    if (norm_fast_ok(p, dtype, p.mode != NORM_FWD)) {
        switch (p.D) {
            case 16: return norm_launch_fast<T, 4>(p, BH, st);
            case 32: return norm_launch_fast<T, 8>(p, BH, st);
            case 64: return norm_launch_fast<T, 16>(p, BH, st);
            default: return norm_launch_fast<T, 32>(p, BH, st);
        }
    }
    NormPlan pl = norm_plan(BH, p.L, (int64_t)mma::sm_count() * 8, 8 * kNormRows);
    p.nseg = pl.nseg;
    p.seg_len = pl.seg_len;
    const int64_t blocks = BH * p.nseg;
    if (blocks > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    if (p.nseg > 1) {
        LaunchScope scope(FTB_KERNEL_NORMALISER, st);
        norm_totals_kernel<T><<<(unsigned)blocks, kNormThreads, 0, st>>>(p);
        FTB_CUDA(cudaGetLastError());
    }
    const size_t smem = 2 * (size_t)kNormRows * (p.D + 1) * sizeof(float);
    if (smem > 48 * 1024)
        FTB_CUDA(cudaFuncSetAttribute(norm_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LaunchScope scope(FTB_KERNEL_NORMALISER, st);
    norm_scan_kernel<T><<<(unsigned)blocks, kNormThreads, smem, st>>>(p);
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}
static int norm_check(int64_t N, int64_t H, int64_t L, int64_t D, int dtype) {
    if (N < 0 || H < 0 || L < 0 || D < 0) return FTB_ERR_INVALID;
    if (dtype != FTB_F32 && dtype != FTB_BF16) return FTB_ERR_INVALID;
    if (D > kNormMaxD) return FTB_ERR_UNSUPPORTED;
    return FTB_OK;
}
}  // namespace ftb

using namespace ftb;

extern "C" {

int ftb_version(void) { return 1000; }

const char *ftb_status_string(int s) {
    switch (s) {
        case FTB_OK: return "ok";
        case FTB_ERR_UNSUPPORTED: return "unsupported shape, dtype or mode";
        case FTB_ERR_ALIGNMENT: return "pointer or stride alignment not met";
        case FTB_ERR_WORKSPACE: return "workspace missing or too small";
        case FTB_ERR_CUDA: return "CUDA runtime error";
        case FTB_ERR_TIMEOUT: return "device-side wait timed out";
        case FTB_ERR_INVALID: return "invalid argument";
        case FTB_ERR_STATIC_LIMIT:
            return "problem needs more scratch than the library's built-in static buffer holds";
        default: return "unknown status";
    }
}

int ftb_last_cuda_error(void) { return g_last_cuda_error; }

int ftb_device_status(int reset) {
    int v = 0;
    // every stream of the device, non-blocking ones included, has drained before the word is read
    if (cudaDeviceSynchronize() != cudaSuccess) return FTB_ERR_CUDA;
    if (cudaMemcpyFromSymbol(&v, mma::g_device_status, sizeof(int)) != cudaSuccess) return FTB_ERR_CUDA;
    if (reset && v) {
        int z = 0;
        cudaMemcpyToSymbol(mma::g_device_status, &z, sizeof(int));
    }
    return v;
}

uint64_t ftb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

void ftb_timing_enable(int enable) {
    std::lock_guard<std::mutex> lock(g_spans_mutex);
    if (!enable) {
        for (auto &sp : g_spans) {
            cudaEventDestroy(sp.beg);
            cudaEventDestroy(sp.end);
        }
        g_spans.clear();
    }
    g_timing.store(enable != 0);
}

int ftb_timing_read(float *ms_by_kind, int *launches_by_kind, int nkinds) {
    if (!ms_by_kind || !launches_by_kind || nkinds <= 0) return FTB_ERR_INVALID;
    for (int i = 0; i < nkinds; ++i) {
        ms_by_kind[i] = 0.f;
        launches_by_kind[i] = 0;
    }
    int rc = FTB_OK;
    std::lock_guard<std::mutex> lock(g_spans_mutex);
    for (auto &sp : g_spans) {
        float ms = 0.f;
        cudaError_t e = cudaEventSynchronize(sp.end);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, sp.beg, sp.end);
        if (e != cudaSuccess) rc = cuda_fail(e);
        if (sp.kind >= 0 && sp.kind < nkinds && e == cudaSuccess) {
            ms_by_kind[sp.kind] += ms;
            launches_by_kind[sp.kind] += 1;
        }
        cudaEventDestroy(sp.beg);
        cudaEventDestroy(sp.end);
    }
    g_spans.clear();
    return rc;
}

size_t ftb_causal_workspace_bytes(int64_t N, int64_t H, int64_t L, int64_t D, int64_t M,
                                  int dtype, int mode, int backward, int want_state) {
    if (N <= 0 || H <= 0 || L <= 0 || D <= 0 || M <= 0) return 0;
    if (const int nb = wide_blocks(mode, dtype, D, M)) {
        // per-segment states of the whole [D][M] width (a feature block is 64 of its rows)
        const WidePlan w = wide_plan(N * H, L, nb, M);
        const size_t one = align256((size_t)N * H * w.pl.nseg * w.sub * D * M * sizeof(float));
        if (backward) return 2 * one;
        return w.pl.nseg > 1 ? one : 0;
    }
    if (mode == FTB_MODE_MMA_X3) {
        if (check_common(N, H, L, D, M, dtype, mode, true) != FTB_OK) return 0;
        const Plan pl = x3_plan(N * H, L);
        const size_t one = align256((size_t)N * H * pl.nseg * x3_sub(pl, N * H) * 4096 * sizeof(float));
        if (backward) return 2 * one;
        return pl.nseg > 1 ? one : 0;
    }
    Plan pl = choose_plan(mode, N * H, L, (int64_t)D * M);
    size_t one = align256((size_t)N * H * pl.nseg * state_sub(mode, pl, N * H) * D * M * sizeof(float));
    if (backward) return 2 * one;
    return (pl.nseg > 1 || want_state) ? one : 0;
}

}  // extern "C"

#include "x3_host.cuh"
#include "wide_host.cuh"

static int forward_impl(const void *q, const void *k, const void *v, void *out, int64_t N,
                        int64_t H, int64_t L, int64_t D, int64_t M, const int64_t *qs,
                        const int64_t *ks, const int64_t *vs, const int64_t *os, int dtype,
                        int mode, const float *initial_state, float *final_state,
                        int workspace_has_states, void *workspace, size_t workspace_bytes,
                        void *stream, const RowScale *scale) {
    int rc = check_common(N, H, L, D, M, dtype, mode, true);
    // the normaliser rides in the tensor-core scans' epilogue only
    if (scale && (mode != FTB_MODE_MMA || wide_blocks(mode, dtype, D, M))) return FTB_ERR_UNSUPPORTED;
    if (rc != FTB_OK) return rc;
    if (mode == FTB_MODE_MMA_X3) {
        if (initial_state || final_state || workspace_has_states) return FTB_ERR_UNSUPPORTED;
        if (N == 0 || H == 0 || L == 0 || D == 0 || M == 0) return FTB_OK;
        if (!q || !k || !v || !out || !qs || !ks || !vs || !os) return FTB_ERR_INVALID;
        const size_t need = ftb_causal_workspace_bytes(N, H, L, D, M, dtype, mode, 0, 0);
        if (need && (!workspace || workspace_bytes < need)) return FTB_ERR_WORKSPACE;
        return x3_forward((const float *)q, (const float *)k, (const float *)v, (float *)out, N, H, L, qs, ks, vs,
                          os, (float *)workspace, (cudaStream_t)stream);
    }
    if (const int nb = wide_blocks(mode, dtype, D, M)) {
        if (initial_state || final_state || workspace_has_states) return FTB_ERR_UNSUPPORTED;
        if (N == 0 || H == 0 || L == 0) return FTB_OK;
        if (!q || !k || !v || !out || !qs || !ks || !vs || !os) return FTB_ERR_INVALID;
        const size_t need = ftb_causal_workspace_bytes(N, H, L, D, M, dtype, mode, 0, 0);
        if (need && (!workspace || workspace_bytes < need)) return FTB_ERR_WORKSPACE;
        return wide_forward((const float *)q, (const float *)k, (const float *)v, (float *)out, N, H, L, nb, (int)M,
                            qs, ks, vs, os, (float *)workspace, (cudaStream_t)stream);
    }
    if (!qs || !ks || !vs || !os) return FTB_ERR_INVALID;
    const bool empty = (N == 0 || H == 0 || L == 0 || M == 0);
    if (!empty && (!q || !k || !v || !out) && D > 0) return FTB_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    if (N == 0 || H == 0) return FTB_OK;
    if (D == 0 || M == 0 || L == 0) {
        // out has no columns, or is all zeros (D == 0); states are unchanged.
        if (L > 0 && M > 0 && D == 0) {
            for (int64_t n = 0; n < N; ++n)
                for (int64_t h = 0; h < H; ++h)
                    FTB_CUDA(cudaMemset2DAsync(
                        (char *)out + (n * os[0] + h * os[1]) * (dtype == FTB_F32 ? 4 : 2),
                        os[2] * (dtype == FTB_F32 ? 4 : 2), 0, M * (dtype == FTB_F32 ? 4 : 2), L, st));
        }
        if (final_state && D > 0 && M > 0) {
            if (initial_state)
                FTB_CUDA(cudaMemcpyAsync(final_state, initial_state, (size_t)N * H * D * M * 4,
                                         cudaMemcpyDeviceToDevice, st));
            else
                FTB_CUDA(cudaMemsetAsync(final_state, 0, (size_t)N * H * D * M * 4, st));
        }
        return FTB_OK;
    }

    Plan pl = choose_plan(mode, N * H, L, (int64_t)D * M);
    float *ws = (float *)workspace;
    if (pl.nseg > 1 || final_state) {
        size_t need = ftb_causal_workspace_bytes(N, H, L, D, M, dtype, mode, 0, final_state != nullptr);
        if (!workspace || workspace_bytes < need) return FTB_ERR_WORKSPACE;
    }
    SegStates ss;
    if (workspace_has_states && mode == FTB_MODE_MMA && !final_state) {
        // ftb_causal_state_sum(k, v, ...) already left the per-segment states in `workspace`
        ss = describe_states(mode, pl, ws, initial_state, N * H);
    } else {
        rc = prepare_states(mode, k, v, ks, vs, N, H, L, (int)D, (int)M, dtype, pl, ws, initial_state,
                            final_state, 0, st, &ss);
        if (rc) return rc;
    }
    return launch_scan(mode, q, k, v, out, qs, ks, vs, os, N, H, L, (int)D, (int)M, dtype, pl, ss,
                       /*canon_is_DaDc=*/1, /*reverse=*/0, st, scale);
}

extern "C" {

static int backward_impl(const void *q, const void *k, const void *v, const void *g, void *gq,
                         void *gk, void *gv, int64_t N, int64_t H, int64_t L, int64_t D,
                         int64_t M, const int64_t *qs, const int64_t *ks, const int64_t *vs,
                         const int64_t *gs, const int64_t *gqs, const int64_t *gks,
                         const int64_t *gvs, int dtype, int mode, const float *initial_state,
                         const float *initial_grad_state, const void *forward_workspace,
                         int workspace_has_grad_states, void *workspace, size_t workspace_bytes,
                         void *stream);

int ftb_causal_dot_product(const void *q, const void *k, const void *v, void *out, int64_t N,
                           int64_t H, int64_t L, int64_t D, int64_t M, const int64_t *qs,
                           const int64_t *ks, const int64_t *vs, const int64_t *os, int dtype,
                           int mode, const float *initial_state, float *final_state,
                           int workspace_has_states, void *workspace, size_t workspace_bytes,
                           void *stream) {
    return forward_impl(q, k, v, out, N, H, L, D, M, qs, ks, vs, os, dtype, mode, initial_state, final_state,
                        workspace_has_states, workspace, workspace_bytes, stream, nullptr);
}

int ftb_causal_dot_product_normalised(const void *q, const void *k, const void *v, const float *den, void *out,
                                      int64_t N, int64_t H, int64_t L, int64_t D, int64_t M, const int64_t *qs,
                                      const int64_t *ks, const int64_t *vs, const int64_t *dens,
                                      const int64_t *os, int dtype, int mode, float eps, void *workspace,
                                      size_t workspace_bytes, void *stream) {
    if (!den || !dens) return FTB_ERR_INVALID;
    RowScale sc{den, S3(dens), eps};
    return forward_impl(q, k, v, out, N, H, L, D, M, qs, ks, vs, os, dtype, mode, nullptr, nullptr, 0, workspace,
                        workspace_bytes, stream, &sc);
}

int ftb_causal_dot_backward(const void *q, const void *k, const void *v, const void *g, void *gq,
                            void *gk, void *gv, int64_t N, int64_t H, int64_t L, int64_t D,
                            int64_t M, const int64_t *qs, const int64_t *ks, const int64_t *vs,
                            const int64_t *gs, const int64_t *gqs, const int64_t *gks,
                            const int64_t *gvs, int dtype, int mode, const float *initial_state,
                            const float *initial_grad_state, const void *forward_workspace,
                            int workspace_has_grad_states, void *workspace, size_t workspace_bytes,
                            void *stream) {
    return backward_impl(q, k, v, g, gq, gk, gv, N, H, L, D, M, qs, ks, vs, gs, gqs, gks, gvs, dtype, mode,
                         initial_state, initial_grad_state, forward_workspace, workspace_has_grad_states,
                         workspace, workspace_bytes, stream);
}



static int backward_impl(const void *q, const void *k, const void *v, const void *g, void *gq,
                         void *gk, void *gv, int64_t N, int64_t H, int64_t L, int64_t D,
                         int64_t M, const int64_t *qs, const int64_t *ks, const int64_t *vs,
                         const int64_t *gs, const int64_t *gqs, const int64_t *gks,
                         const int64_t *gvs, int dtype, int mode, const float *initial_state,
                         const float *initial_grad_state, const void *forward_workspace,
                         int workspace_has_grad_states, void *workspace, size_t workspace_bytes,
                         void *stream) {
    int rc = check_common(N, H, L, D, M, dtype, mode, true);
    if (rc != FTB_OK) return rc;
    if (!qs || !ks || !vs || !gs || !gqs || !gks || !gvs) return FTB_ERR_INVALID;
    if (mode == FTB_MODE_MMA_X3) {
        if (initial_state || initial_grad_state || workspace_has_grad_states) return FTB_ERR_UNSUPPORTED;
        if (N == 0 || H == 0 || L == 0 || D == 0 || M == 0) return FTB_OK;
        if (!q || !k || !v || !g || (!gq && !gk && !gv)) return FTB_ERR_INVALID;
        const size_t need = ftb_causal_workspace_bytes(N, H, L, D, M, dtype, mode, 1, 0);
        if (need && (!workspace || workspace_bytes < need)) return FTB_ERR_WORKSPACE;
        return x3_backward((const float *)q, (const float *)k, (const float *)v, (const float *)g, (float *)gq,
                           (float *)gk, (float *)gv, N, H, L, qs, ks, vs, gs, gqs, gks, gvs,
                           (const float *)forward_workspace, (float *)workspace, need, (cudaStream_t)stream);
    }
    if (const int nb = wide_blocks(mode, dtype, D, M)) {
        if (initial_state || initial_grad_state || workspace_has_grad_states) return FTB_ERR_UNSUPPORTED;
        if (N == 0 || H == 0 || L == 0) return FTB_OK;
        if (!q || !k || !v || !g || (!gq && !gk && !gv)) return FTB_ERR_INVALID;
        const size_t need = ftb_causal_workspace_bytes(N, H, L, D, M, dtype, mode, 1, 0);
        if (need && (!workspace || workspace_bytes < need)) return FTB_ERR_WORKSPACE;
        return wide_backward((const float *)q, (const float *)k, (const float *)v, (const float *)g,
                             (float *)gq, (float *)gk, (float *)gv, N, H, L, nb, (int)M, qs, ks, vs, gs, gqs, gks, gvs,
                             (const float *)forward_workspace, (float *)workspace, need, (cudaStream_t)stream);
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (N == 0 || H == 0 || L == 0) return FTB_OK;
    const size_t es = dtype == FTB_F32 ? 4 : 2;
    if (D == 0 || M == 0) {
        // one operand has no features: every gradient that has columns is zero
        for (int64_t n = 0; n < N; ++n)
            for (int64_t h = 0; h < H; ++h) {
                if (D > 0 && gq)
                    FTB_CUDA(cudaMemset2DAsync((char *)gq + (n * gqs[0] + h * gqs[1]) * es,
                                               gqs[2] * es, 0, D * es, L, st));
                if (D > 0 && gk)
                    FTB_CUDA(cudaMemset2DAsync((char *)gk + (n * gks[0] + h * gks[1]) * es,
                                               gks[2] * es, 0, D * es, L, st));
                if (M > 0 && gv)
                    FTB_CUDA(cudaMemset2DAsync((char *)gv + (n * gvs[0] + h * gvs[1]) * es,
                                               gvs[2] * es, 0, M * es, L, st));
            }
        return FTB_OK;
    }
    if (!q || !k || !v || !g) return FTB_ERR_INVALID;
    // a null output pointer skips that gradient (and the states only it needs)
    const bool want_q = gq != nullptr, want_kv = gk != nullptr || gv != nullptr;
    if (!want_q && !want_kv) return FTB_ERR_INVALID;

    Plan pl = choose_plan(mode, N * H, L, (int64_t)D * M);
    size_t need = ftb_causal_workspace_bytes(N, H, L, D, M, dtype, mode, 1, 0);
    if (need && (!workspace || workspace_bytes < need)) return FTB_ERR_WORKSPACE;
    float *wsS = (float *)workspace;
    float *wsR = (float *)((char *)workspace + need / 2);

    // forward states: taken from the forward call's workspace when the caller kept it
    SegStates sS{nullptr, initial_state, 0, 1}, sR{nullptr, initial_grad_state, 0, 1};
    if (!want_q) {
        // grad_Q is the only reader of the forward states
    } else if (forward_workspace && pl.nseg > 1) {
        sS = describe_states(mode, pl, (const float *)forward_workspace, initial_state, N * H);
    } else {
        rc = prepare_states(mode, k, v, ks, vs, N, H, L, (int)D, (int)M, dtype, pl, wsS, initial_state,
                            nullptr, 0, st, &sS);
        if (rc) return rc;
    }
    // reverse states R = sum q (x) grad_out over the segments after each segment
    bool r_with_grad_q = false;   // tensor-core mode: the totals are swept in grad_Q's own launch
    // grad_K and grad_V may walk WHOLE sequences (one segment per pair) although the forward and
    // grad_Q use several: they then need no reverse totals at all -- no sweep of (q, grad_out) --
    // and it costs nothing where the two scans of all pairs fill the device once either way
    // (config 2: 128 blocks of 32 chunks instead of 256 blocks of 16 in 1.7 waves).
    Plan pl_kv = pl;
    if (mode == FTB_MODE_MMA && want_kv && gk && gv && pl.nseg > 1 && !workspace_has_grad_states) {
        const int64_t sms = mma::sm_count(), chunks = (L + mma::C - 1) / mma::C, cps = pl.seg_len / mma::C;
        const int64_t whole = (2 * N * H + sms - 1) / sms * (chunks + 1);
        const int64_t split = (2 * N * H * pl.nseg + sms - 1) / sms * (cps + 1);
        if (whole <= split) {
            pl_kv.nseg = 1;
            pl_kv.seg_len = chunks * mma::C;
        }
    }
    const bool kv_whole = pl_kv.nseg != pl.nseg;
    if (!want_kv || kv_whole) {
        // grad_K and grad_V are the only readers of the reverse states
    } else if (workspace_has_grad_states && mode == FTB_MODE_MMA) {
        // ftb_causal_state_sum(q, grad_out, ..., reverse=1, second half of `workspace`) ran before
        sR = describe_states(mode, pl, wsR, initial_grad_state, N * H);
    } else if (mode == FTB_MODE_MMA && pl.nseg > 1 && sums_in_kernel(mode, pl)) {
        sR = describe_states(mode, pl, wsR, initial_grad_state, N * H);
        r_with_grad_q = true;
    } else {
        rc = prepare_states(mode, q, g, qs, gs, N, H, L, (int)D, (int)M, dtype, pl, wsR,
                            initial_grad_state, nullptr, 1, st, &sR);
        if (rc) return rc;
    }

    if (mode == FTB_MODE_MMA) {
        // The three gradient scans are independent of each other; grad_Q does not read R.  They
        // go out as one grid -- or, when R's segment totals are still to be computed, as
        // {grad_Q scan + the state-only sweep of (q, grad_out)} followed by {grad_K, grad_V}:
        // the short sweep runs on the SMs the scan leaves idle, and consecutive scans overlap
        // where one's last CTAs would otherwise leave SMs empty.
        MmaBatch first;
        if (want_q) {
            rc = mma_add_job(first, g, v, k, gq, gs, vs, ks, gqs, N, H, L, (int)M, (int)D, dtype, pl,
                             sS.states, sS.init, sS.sum_mode, sS.sub, nullptr, 0, 0, 0, 0);
            if (rc) return rc;
            first.kind = FTB_KERNEL_MMA_BWD;
        }
        MmaBatch second;
        // (grad_K, grad_V on a plan of their own: a grid of their own, so that their blocks stay
        // side by side; it reads nothing the grad_Q grid writes)
        MmaBatch &kv = (r_with_grad_q || (kv_whole && want_q)) ? second : first;
        if (r_with_grad_q) {
            Plan fine = pl;
            fine.seg_len = pl.seg_len / sR.sub;
            fine.nseg = pl.nseg * sR.sub;
            rc = mma_add_job(first, nullptr, q, g, nullptr, nullptr, qs, gs, nullptr, N, H, L, (int)D, (int)M,
                             dtype, fine, nullptr, nullptr, 0, 1, wsR, 0, sR.sub, 1, 0);
            if (rc) return rc;
            first.kind = want_q ? FTB_KERNEL_MMA_BWD_QR : FTB_KERNEL_MMA_STATE;
        }
        if (gk) {
            rc = mma_add_job(kv, v, g, q, gk, vs, gs, qs, gks, N, H, L, (int)M, (int)D, dtype, pl_kv, sR.states,
                             sR.init, sR.sum_mode, sR.sub, nullptr, 0, 0, 0, 1);
            if (rc) return rc;
        }
        if (gv) {
            rc = mma_add_job(kv, k, q, g, gv, ks, qs, gs, gvs, N, H, L, (int)D, (int)M, dtype, pl_kv, sR.states,
                             sR.init, sR.sum_mode, sR.sub, nullptr, 0, 0, 1, 1);
            if (rc) return rc;
        }
        if (want_kv) kv.kind = (&kv == &first && want_q) || (gk && gv) ? FTB_KERNEL_MMA_BWD_MULTI
                                                                      : FTB_KERNEL_MMA_BWD;
        first.after_own_launch = sS.fresh || sR.fresh;   // a sweep of this call is directly in front
        rc = mma_launch_batch(first, st);
        if (rc || &kv == &first) return rc;
        second.after_own_launch = true;   // directly behind this call's grad_Q grid
        return mma_launch_batch(second, st);
    }

    // grad_Q_i = sum_{j<=i} (g_i . v_j) k_j + S_init g_i        state viewed as [M][D]
    if (gq) {
        rc = launch_scan(mode, g, v, k, gq, gs, vs, ks, gqs, N, H, L, (int)M, (int)D, dtype, pl, sS, 0, 0, st);
        if (rc) return rc;
    }
    // grad_K_j = sum_{i>=j} (v_j . g_i) q_i + R_init v_j        state viewed as [M][D]
    if (gk) {
        rc = launch_scan(mode, v, g, q, gk, vs, gs, qs, gks, N, H, L, (int)M, (int)D, dtype, pl, sR, 0, 1, st);
        if (rc) return rc;
    }
    // grad_V_j = sum_{i>=j} (k_j . q_i) g_i + R_init^T k_j      state viewed as [D][M]
    if (gv)
        rc = launch_scan(mode, k, q, g, gv, ks, qs, gs, gvs, N, H, L, (int)D, (int)M, dtype, pl, sR, 1, 1, st);
    return rc;
}

int ftb_causal_state_parts(int64_t N, int64_t H, int64_t L, int64_t D, int64_t M, int dtype, int mode) {
    if (check_common(N, H, L, D, M, dtype, mode) != FTB_OK) return 0;
    if (N <= 0 || H <= 0 || L <= 0 || D <= 0 || M <= 0) return 0;
    Plan pl = choose_plan(mode, N * H, L, (int64_t)D * M);
    if (pl.nseg == 1) return 1;
    if (!sums_in_kernel(mode, pl)) return 0;   // the workspace then holds prefixes, not raw totals
    return pl.nseg * state_sub(mode, pl, N * H);
}

int ftb_causal_state_sum(const void *x, const void *y, float *state, int64_t N, int64_t H,
                         int64_t L, int64_t D, int64_t M, const int64_t *xs, const int64_t *ys,
                         int dtype, int mode, int reverse, void *workspace, size_t workspace_bytes,
                         void *stream) {
    int rc = check_common(N, H, L, D, M, dtype, mode);
    if (rc != FTB_OK) return rc;
    if (!xs || !ys) return FTB_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    if (N == 0 || H == 0 || D == 0 || M == 0) return FTB_OK;
    if (!state) {
        // partial sums only: ftb_causal_state_parts(...) blocks per (batch, head) at the start of
        // `workspace`, for a caller that adds them up itself (ftb_exchange_push_parts)
        if (L == 0 || !x || !y) return FTB_ERR_INVALID;
        const int parts = ftb_causal_state_parts(N, H, L, D, M, dtype, mode);
        if (parts == 0) return FTB_ERR_UNSUPPORTED;
        size_t need = align256((size_t)N * H * parts * D * M * sizeof(float));
        if (!workspace || workspace_bytes < need) return FTB_ERR_WORKSPACE;
        Plan pl = choose_plan(mode, N * H, L, (int64_t)D * M);
        if (pl.nseg > 1) {
            const int sub = state_sub(mode, pl, N * H);
            pl.seg_len /= sub;
            pl.nseg *= sub;
        }
        return launch_state_sum(mode, x, y, xs, ys, N, H, L, (int)D, (int)M, dtype, pl, (float *)workspace,
                                0, 0, st);
    }
    if (L == 0) {
        FTB_CUDA(cudaMemsetAsync(state, 0, (size_t)N * H * D * M * 4, st));
        return FTB_OK;
    }
    if (!x || !y) return FTB_ERR_INVALID;
    Plan pl = choose_plan(mode, N * H, L, (int64_t)D * M);
    if (pl.nseg == 1)
        return launch_state_sum(mode, x, y, xs, ys, N, H, L, (int)D, (int)M, dtype, pl, state, 0, 0, st);
    size_t need = ftb_causal_workspace_bytes(N, H, L, D, M, dtype, mode, 0, 1);
    if (!workspace || workspace_bytes < need) return FTB_ERR_WORKSPACE;
    SegStates ss;
    return prepare_states(mode, x, y, xs, ys, N, H, L, (int)D, (int)M, dtype, pl, (float *)workspace,
                          nullptr, state, reverse ? 1 : 0, st, &ss);
}


// ---------------------------------------------------------------------------------------------
// The denominator Q_l . sum_{j<=l} K_j and its gradients.
// ---------------------------------------------------------------------------------------------
size_t ftb_causal_normaliser_workspace_bytes(int64_t N, int64_t H, int64_t L, int64_t D, int backward) {
    if (N <= 0 || H <= 0 || L <= 0 || D <= 0) return 0;
    // per-segment sums for the most segments either kernel family may use
    size_t one = align256((size_t)N * H * kNormMaxSegs * D * sizeof(float));
    return backward ? 2 * one : one;
}

int ftb_causal_normaliser(const void *q, const void *k, void *den, int64_t N, int64_t H, int64_t L,
                          int64_t D, const int64_t *qs, const int64_t *ks, const int64_t *dens,
                          int dtype, void *workspace, size_t workspace_bytes, void *stream) {
    int rc = norm_check(N, H, L, D, dtype);
    if (rc) return rc;
    if (!qs || !ks || !dens) return FTB_ERR_INVALID;
    if (N == 0 || H == 0 || L == 0) return FTB_OK;
    if (!den || (D > 0 && (!q || !k))) return FTB_ERR_INVALID;
    size_t need = ftb_causal_normaliser_workspace_bytes(N, H, L, D, 0);
    if (need && (!workspace || workspace_bytes < need)) return FTB_ERR_WORKSPACE;
    NormParams p{};
    p.q = q; p.k = k; p.g = nullptr; p.out = den;
    p.qs = Strides3n{qs[0], qs[1], qs[2]}; p.ks = Strides3n{ks[0], ks[1], ks[2]};
    p.gs = Strides3n{0, 0, 0}; p.os = Strides3n{dens[0], dens[1], dens[2]};
    p.H = (int)H; p.D = (int)D; p.L = L;
    p.totals = (float *)workspace; p.mode = NORM_FWD;
    cudaStream_t st = (cudaStream_t)stream;
    return dtype == FTB_F32 ? norm_launch<float>(p, N * H, dtype, st)
                            : norm_launch<__nv_bfloat16>(p, N * H, dtype, st);
}

// (elu: raw inputs and the key mask of the layer's feature map, or nullptr; see NormParams::elu_x)
struct NormElu {
    const void *xq, *xk;
    const int64_t *xqs, *xks;
    const float *key_mask;
};
static int normaliser_backward(const void *q, const void *k, const void *grad_den, void *gq, void *gk,
                               int64_t N, int64_t H, int64_t L, int64_t D, const int64_t *qs,
                               const int64_t *ks, const int64_t *gdens, const int64_t *gqs, const int64_t *gks,
                               int dtype, void *workspace, size_t workspace_bytes, void *stream, int accumulate,
                               const NormElu *elu = nullptr);

int ftb_causal_normaliser_backward(const void *q, const void *k, const void *grad_den, void *gq,
                                   void *gk, int64_t N, int64_t H, int64_t L, int64_t D,
                                   const int64_t *qs, const int64_t *ks, const int64_t *gdens,
                                   const int64_t *gqs, const int64_t *gks, int dtype, void *workspace,
                                   size_t workspace_bytes, void *stream) {
    return normaliser_backward(q, k, grad_den, gq, gk, N, H, L, D, qs, ks, gdens, gqs, gks, dtype, workspace,
                               workspace_bytes, stream, 0);
}

int ftb_causal_normaliser_backward_add(const void *q, const void *k, const void *grad_den, void *gq,
                                       void *gk, int64_t N, int64_t H, int64_t L, int64_t D,
                                       const int64_t *qs, const int64_t *ks, const int64_t *gdens,
                                       const int64_t *gqs, const int64_t *gks, int dtype, void *workspace,
                                       size_t workspace_bytes, void *stream) {
    return normaliser_backward(q, k, grad_den, gq, gk, N, H, L, D, qs, ks, gdens, gqs, gks, dtype, workspace,
                               workspace_bytes, stream, 1);
}

int ftb_causal_normaliser_backward_elu(const void *q, const void *k, const void *grad_den, void *gq,
                                       void *gk, const void *xq, const void *xk, const float *key_mask,
                                       int64_t N, int64_t H, int64_t L, int64_t D, const int64_t *qs,
                                       const int64_t *ks, const int64_t *gdens, const int64_t *gqs,
                                       const int64_t *gks, const int64_t *xqs, const int64_t *xks, int dtype,
                                       void *workspace, size_t workspace_bytes, void *stream) {
    if ((gq && (!xq || !xqs)) || (gk && (!xk || !xks))) return FTB_ERR_INVALID;
    NormElu elu{xq, xk, xqs, xks, key_mask};
    return normaliser_backward(q, k, grad_den, gq, gk, N, H, L, D, qs, ks, gdens, gqs, gks, dtype, workspace,
                               workspace_bytes, stream, 1, &elu);
}

static int normaliser_backward(const void *q, const void *k, const void *grad_den, void *gq, void *gk,
                               int64_t N, int64_t H, int64_t L, int64_t D, const int64_t *qs,
                               const int64_t *ks, const int64_t *gdens, const int64_t *gqs, const int64_t *gks,
                               int dtype, void *workspace, size_t workspace_bytes, void *stream, int accumulate,
                               const NormElu *elu) {
    int rc = norm_check(N, H, L, D, dtype);
    if (rc) return rc;
    if (!qs || !ks || !gdens || !gqs || !gks) return FTB_ERR_INVALID;
    if (N == 0 || H == 0 || L == 0 || D == 0) return FTB_OK;
    if (!q || !k || !grad_den || (!gq && !gk)) return FTB_ERR_INVALID;
    size_t need = ftb_causal_normaliser_workspace_bytes(N, H, L, D, 1);
    if (need && (!workspace || workspace_bytes < need)) return FTB_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    NormParams p{};
    p.q = q; p.k = k; p.g = grad_den;
    p.qs = Strides3n{qs[0], qs[1], qs[2]}; p.ks = Strides3n{ks[0], ks[1], ks[2]};
    p.gs = Strides3n{gdens[0], gdens[1], gdens[2]};
    p.H = (int)H; p.D = (int)D; p.L = L;
    p.accumulate = accumulate;
    auto with_elu = [&](const void *x, const int64_t *xs, const float *mask) -> int {
        p.elu_x = nullptr;
        p.elu_mask = nullptr;
        if (!elu) return FTB_OK;
        p.elu_x = x;
        p.xs = Strides3n{xs[0], xs[1], xs[2]};
        p.elu_mask = mask;
        // only the streaming kernels take the feature map's factor
        const uintptr_t a = dtype == FTB_F32 ? 15 : 7;
        if (!norm_fast_ok(p, dtype, true) || ((uintptr_t)x & a) || xs[0] % 4 || xs[1] % 4 || xs[2] % 4)
            return FTB_ERR_UNSUPPORTED;
        return FTB_OK;
    };
    if (gq) {   // gQ_l = g_l * sum_{j<=l} K_j
        p.out = gq; p.os = Strides3n{gqs[0], gqs[1], gqs[2]};
        if ((rc = with_elu(elu ? elu->xq : nullptr, elu ? elu->xqs : nullptr, nullptr))) return rc;
        p.totals = (float *)workspace; p.mode = NORM_BWD_Q;
        rc = dtype == FTB_F32 ? norm_launch<float>(p, N * H, dtype, st)
                              : norm_launch<__nv_bfloat16>(p, N * H, dtype, st);
        if (rc) return rc;
    }
    if (gk) {   // gK_j = sum_{l>=j} g_l * Q_l
        p.out = gk; p.os = Strides3n{gks[0], gks[1], gks[2]};
        if ((rc = with_elu(elu ? elu->xk : nullptr, elu ? elu->xks : nullptr, elu ? elu->key_mask : nullptr)))
            return rc;
        p.totals = (float *)((char *)workspace + need / 2); p.mode = NORM_BWD_K;
        rc = dtype == FTB_F32 ? norm_launch<float>(p, N * H, dtype, st)
                              : norm_launch<__nv_bfloat16>(p, N * H, dtype, st);
    }
    return rc;
}

int ftb_normalised_output_grads(const float *grad_y, const float *y, const float *den, float *grad_out,
                                float *grad_den, int64_t rows, int64_t M, float eps, void *stream) {
    if (rows < 0 || M <= 0) return FTB_ERR_INVALID;
    if (M != 16 && M != 32 && M != 64 && M != 128) return FTB_ERR_UNSUPPORTED;
    if (rows == 0) return FTB_OK;
    if (!grad_y || !y || !den || !grad_out || !grad_den) return FTB_ERR_INVALID;
    if ((((uintptr_t)grad_y | (uintptr_t)y | (uintptr_t)grad_out) & 15) != 0) return FTB_ERR_ALIGNMENT;
    const int lpr = (int)(M / 4);
    const int64_t blocks = (rows * lpr + 255) / 256;
    if (blocks > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    LaunchScope scope(FTB_KERNEL_NORMALISER, st);
    switch (lpr) {
        case 4: normalised_grads_kernel<4><<<(unsigned)blocks, 256, 0, st>>>(grad_y, y, den, grad_out, grad_den, rows, eps); break;
        case 8: normalised_grads_kernel<8><<<(unsigned)blocks, 256, 0, st>>>(grad_y, y, den, grad_out, grad_den, rows, eps); break;
        case 16: normalised_grads_kernel<16><<<(unsigned)blocks, 256, 0, st>>>(grad_y, y, den, grad_out, grad_den, rows, eps); break;
        default: normalised_grads_kernel<32><<<(unsigned)blocks, 256, 0, st>>>(grad_y, y, den, grad_out, grad_den, rows, eps); break;
    }
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

// ---------------------------------------------------------------------------------------------
// phi(x) = elu(x) + 1 with the key-length mask folded in, and its gradient.
// ---------------------------------------------------------------------------------------------
static int elu1_launch(const void *x, const void *g, void *out, const float *mask, int64_t total,
                       int64_t inner_per_mask, int dtype, bool backward, cudaStream_t st) {
    if (total < 0 || (dtype != FTB_F32 && dtype != FTB_BF16)) return FTB_ERR_INVALID;
    if (mask && inner_per_mask <= 0) return FTB_ERR_INVALID;
    if (total == 0) return FTB_OK;
    if (!x || !out || (backward && !g)) return FTB_ERR_INVALID;
    const int64_t blocks = (total + 1023) / 1024;
    if (blocks > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    LaunchScope scope(FTB_KERNEL_FEATURE_MAP, st);
    const uintptr_t am = dtype == FTB_F32 ? 15 : 7;
    const bool vec = total % 4 == 0 && (!mask || inner_per_mask % 4 == 0) && ((uintptr_t)x & am) == 0 &&
                     ((uintptr_t)out & am) == 0 && (!backward || ((uintptr_t)g & am) == 0);
    if (vec) {
        if (dtype == FTB_F32) {
            if (backward)
                elu1_vec_kernel<float, true><<<(unsigned)blocks, 256, 0, st>>>(
                    (const float *)x, (const float *)g, (float *)out, mask, total, inner_per_mask);
            else
                elu1_vec_kernel<float, false><<<(unsigned)blocks, 256, 0, st>>>(
                    (const float *)x, nullptr, (float *)out, mask, total, inner_per_mask);
        } else {
            using B = __nv_bfloat16;
            if (backward)
                elu1_vec_kernel<B, true><<<(unsigned)blocks, 256, 0, st>>>((const B *)x, (const B *)g, (B *)out,
                                                                          mask, total, inner_per_mask);
            else
                elu1_vec_kernel<B, false><<<(unsigned)blocks, 256, 0, st>>>((const B *)x, nullptr, (B *)out, mask,
                                                                           total, inner_per_mask);
        }
        FTB_CUDA(cudaGetLastError());
        return FTB_OK;
    }
    if (dtype == FTB_F32) {
        if (backward)
            elu1_kernel<float, true><<<(unsigned)blocks, 256, 0, st>>>((const float *)x, (const float *)g,
                                                                      (float *)out, mask, total, inner_per_mask);
        else
            elu1_kernel<float, false><<<(unsigned)blocks, 256, 0, st>>>((const float *)x, nullptr, (float *)out,
                                                                       mask, total, inner_per_mask);
    } else {
        using B = __nv_bfloat16;
        if (backward)
            elu1_kernel<B, true><<<(unsigned)blocks, 256, 0, st>>>((const B *)x, (const B *)g, (B *)out, mask,
                                                                  total, inner_per_mask);
        else
            elu1_kernel<B, false><<<(unsigned)blocks, 256, 0, st>>>((const B *)x, nullptr, (B *)out, mask, total,
                                                                   inner_per_mask);
    }
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

int ftb_elu_feature_map(const void *x, void *y, const float *row_mask, int64_t total,
                        int64_t elements_per_mask_entry, int dtype, void *stream) {
    return elu1_launch(x, nullptr, y, row_mask, total, elements_per_mask_entry, dtype, false,
                       (cudaStream_t)stream);
}

int ftb_elu_feature_map_backward(const void *x, const void *grad_y, void *grad_x, const float *row_mask,
                                 int64_t total, int64_t elements_per_mask_entry, int dtype,
                                 void *stream) {
    return elu1_launch(x, grad_y, grad_x, row_mask, total, elements_per_mask_entry, dtype, true,
                       (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// One recurrent step (the same attention as a fixed-state recurrent model).
// ---------------------------------------------------------------------------------------------
int ftb_recurrent_linear_step(const void *q, const void *k, const void *v, float *S, float *z,
                              void *out, int64_t N, int64_t H, int64_t D, int64_t M,
                              const int64_t *qs, const int64_t *ks, const int64_t *vs,
                              const int64_t *os, int dtype, int feature_map, float eps,
                              void *stream) {
    if (N < 0 || H < 0 || D < 0 || M < 0) return FTB_ERR_INVALID;
    if (dtype != FTB_F32 && dtype != FTB_BF16) return FTB_ERR_INVALID;
    if (feature_map != FTB_FEATURE_NONE && feature_map != FTB_FEATURE_ELU1) return FTB_ERR_INVALID;
    if (!qs || !ks || !vs || !os) return FTB_ERR_INVALID;
    if (D > kStepMaxD) return FTB_ERR_UNSUPPORTED;
    if (N == 0 || H == 0 || M == 0) return FTB_OK;
    if (N * H > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    if (!v || !out || (D > 0 && (!q || !k || !S || !z))) return FTB_ERR_INVALID;
    if (M % 4 == 0 && ((uintptr_t)S & 15)) return FTB_ERR_ALIGNMENT;   // rows of S are read 16 bytes wide
    cudaStream_t st = (cudaStream_t)stream;
    const Strides2 a{qs[0], qs[1]}, b{ks[0], ks[1]}, c{vs[0], vs[1]}, o{os[0], os[1]};
    LaunchScope scope(FTB_KERNEL_RECURRENT_STEP, st);
    if (dtype == FTB_F32)
        recurrent_step_kernel<float><<<(unsigned)(N * H), kStepThreads, 0, st>>>(
            (const float *)q, (const float *)k, (const float *)v, S, z, (float *)out, (int)H, (int)D, (int)M,
            a, b, c, o, feature_map, eps);
    else
        recurrent_step_kernel<__nv_bfloat16><<<(unsigned)(N * H), kStepThreads, 0, st>>>(
            (const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k, (const __nv_bfloat16 *)v, S, z,
            (__nv_bfloat16 *)out, (int)H, (int)D, (int)M, a, b, c, o, feature_map, eps);
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

// ---------------------------------------------------------------------------------------------
// Favor's positive random features, one pass on the tensor cores.
// ---------------------------------------------------------------------------------------------
int ftb_favor_feature_map(const float *x, const float *omega_t, float *out, int64_t rows, int64_t E,
                          int64_t half, int64_t x_row_stride, int64_t out_row_stride, float softmax_temp,
                          void *stream) {
    if (rows < 0 || E <= 0 || half <= 0 || !(softmax_temp > 0.f)) return FTB_ERR_INVALID;
    if (E != favor::kE || (half != 64 && half != 128)) return FTB_ERR_UNSUPPORTED;
    if (rows == 0) return FTB_OK;
    if (!x || !omega_t || !out) return FTB_ERR_INVALID;
    if (rows > 0x7fffffffLL - favor::kRows) return FTB_ERR_UNSUPPORTED;
    if (((uintptr_t)out & 7) || out_row_stride % 2 || out_row_stride < 2 * half) return FTB_ERR_ALIGNMENT;
    CUtensorMap mx, mw;
    favor::Params p;
    const int64_t xs[3] = {0, 0, x_row_stride}, ws[3] = {0, 0, E};
    int rc = mma::make_map(&mx, p.pos_x, x, 1, 1, rows, E, xs, FTB_F32);
    if (rc) return rc;
    rc = mma::make_map(&mw, p.pos_w, omega_t, 1, 1, half, E, ws, FTB_F32);
    if (rc) return rc;
    p.out = out;
    p.rows = rows;
    p.out_stride = out_row_stride;
    p.scale = sqrtf(softmax_temp);
    p.half_temp = 0.5f * softmax_temp;
    p.log_term = 0.5f * logf((float)(2 * half));
    const int64_t tiles = (rows + favor::kRows - 1) / favor::kRows;
    const unsigned grid = (unsigned)std::min<int64_t>(tiles, 2 * (int64_t)mma::sm_count());
    cudaStream_t st = (cudaStream_t)stream;
    LaunchScope scope(FTB_KERNEL_FEATURE_MAP, st);
    if (half == 64) {
        FTB_CUDA(cudaFuncSetAttribute(favor::favor_map_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)favor::kSmem));
        favor::favor_map_kernel<64><<<grid, favor::kThreads, favor::kSmem, st>>>(mx, mw, p);
    } else {
        FTB_CUDA(cudaFuncSetAttribute(favor::favor_map_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)favor::kSmem));
        favor::favor_map_kernel<128><<<grid, favor::kThreads, favor::kSmem, st>>>(mx, mw, p);
    }
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

int ftb_favor_feature_map_backward(const float *grad_phi, const float *phi, const float *x, const float *omega,
                                   float *grad_x, int64_t rows, int64_t E, int64_t half, int64_t grad_phi_row_stride,
                                   int64_t phi_row_stride, int64_t x_row_stride, int64_t grad_x_row_stride,
                                   float softmax_temp, void *stream) {
    if (rows < 0 || E <= 0 || half <= 0 || !(softmax_temp > 0.f)) return FTB_ERR_INVALID;
    if (E != favor::kE || (half != 64 && half != 128)) return FTB_ERR_UNSUPPORTED;
    if (rows == 0) return FTB_OK;
    if (!grad_phi || !phi || !x || !omega || !grad_x) return FTB_ERR_INVALID;
    if (rows > 0x7fffffffLL - favor::kRows) return FTB_ERR_UNSUPPORTED;
    if (((uintptr_t)grad_x & 7) || grad_x_row_stride % 2 || grad_x_row_stride < E) return FTB_ERR_ALIGNMENT;
    CUtensorMap mg, mp, mx, mw;
    favor::BwdParams p;
    const int64_t gs[3] = {0, 0, grad_phi_row_stride}, ps[3] = {0, 0, phi_row_stride}, xs[3] = {0, 0, x_row_stride};
    int rc = mma::make_map(&mg, p.pos_g, grad_phi, 1, 1, rows, 2 * half, gs, FTB_F32);
    if (rc) return rc;
    if ((rc = mma::make_map(&mp, p.pos_p, phi, 1, 1, rows, 2 * half, ps, FTB_F32))) return rc;
    if ((rc = mma::make_map(&mx, p.pos_x, x, 1, 1, rows, E, xs, FTB_F32))) return rc;
    {
        // omega (E rows of `half` floats): boxes of 32 features x all 64 rows
        mma::EncodeTiledFn enc = mma::encode_fn();
        if (!enc) return FTB_ERR_CUDA;
        if ((uintptr_t)omega & 15) return FTB_ERR_ALIGNMENT;
        cuuint64_t gdim[2] = {(cuuint64_t)half, (cuuint64_t)E};
        cuuint64_t gstr[1] = {(cuuint64_t)(half * 4)};
        cuuint32_t box[2] = {32, (cuuint32_t)E}, estr[2] = {1, 1};
        if (enc(&mw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(omega), gdim, gstr, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return FTB_ERR_ALIGNMENT;
    }
    p.grad_x = grad_x;
    p.rows = rows;
    p.gx_stride = grad_x_row_stride;
    p.scale = sqrtf(softmax_temp);
    p.temp = softmax_temp;
    const int64_t tiles = (rows + favor::kRows - 1) / favor::kRows;
    const unsigned grid = (unsigned)std::min<int64_t>(tiles, (int64_t)mma::sm_count());
    cudaStream_t st = (cudaStream_t)stream;
    LaunchScope scope(FTB_KERNEL_FEATURE_MAP, st);
    if (half == 64) {
        FTB_CUDA(cudaFuncSetAttribute(favor::favor_map_backward_kernel<64>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)favor::kSmemBwd));
        favor::favor_map_backward_kernel<64><<<grid, favor::kBwdThreads, favor::kSmemBwd, st>>>(mg, mp, mx, mw, p);
    } else {
        FTB_CUDA(cudaFuncSetAttribute(favor::favor_map_backward_kernel<128>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)favor::kSmemBwd));
        favor::favor_map_backward_kernel<128><<<grid, favor::kBwdThreads, favor::kSmemBwd, st>>>(mg, mp, mx, mw, p);
    }
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

// ---------------------------------------------------------------------------------------------
// One fixed state applied to every position (the non-causal form), and a read-only step.
// ---------------------------------------------------------------------------------------------
int ftb_linear_apply_state(const void *a, const float *state, void *out, int64_t N, int64_t H, int64_t L,
                           int64_t Da, int64_t Dc, const int64_t *as, const int64_t *os, int dtype,
                           int mode, int state_is_transposed, void *stream) {
    if (N < 0 || H < 0 || L < 0 || Da < 0 || Dc < 0) return FTB_ERR_INVALID;
    if (dtype != FTB_F32 && dtype != FTB_BF16) return FTB_ERR_INVALID;
    if (mode == FTB_MODE_MMA_X3) return FTB_ERR_UNSUPPORTED;
    if (mode != FTB_MODE_FP32_SIMT && mode != FTB_MODE_MMA) return FTB_ERR_INVALID;
    if (!as || !os) return FTB_ERR_INVALID;
    if (mode == FTB_MODE_MMA && Da > 0 && Dc > 0 && !mma::supported(dtype, Da, Dc)) return FTB_ERR_UNSUPPORTED;
    if (N == 0 || H == 0 || L == 0 || Dc == 0) return FTB_OK;
    if (!out || (Da > 0 && (!a || !state))) return FTB_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t es = dtype == FTB_F32 ? 4 : 2;
    if (Da == 0) {   // nothing to contract: zeros
        for (int64_t n = 0; n < N; ++n)
            for (int64_t h = 0; h < H; ++h)
                FTB_CUDA(cudaMemset2DAsync((char *)out + (n * os[0] + h * os[1]) * es, os[2] * es, 0,
                                           Dc * es, L, st));
        return FTB_OK;
    }
    if (mode == FTB_MODE_MMA) {
        Plan pl = choose_plan(mode, N * H, L, (int64_t)Da * Dc);
        MmaBatch batch;
        int rc = mma_add_job(batch, a, nullptr, nullptr, out, as, nullptr, nullptr, os, N, H, L, (int)Da,
                             (int)Dc, dtype, pl, nullptr, state, 0, 1, nullptr, 0, 0,
                             state_is_transposed ? 0 : 1, 0);
        if (rc) return rc;
        batch.kind = FTB_KERNEL_APPLY_STATE;
        return mma_launch_batch(batch, st);
    }
    if (N * H > 65535) return FTB_ERR_UNSUPPORTED;
    ApplyArgs p;
    p.a = a; p.out = out; p.state = state;
    p.sa = S3(as); p.so = S3(os);
    p.H = (int)H; p.L = L; p.Da = (int)Da; p.Dc = (int)Dc;
    p.canon_is_DaDc = state_is_transposed ? 0 : 1;
    p.vec_out = dtype == FTB_F32 && Dc % 4 == 0 && ((uintptr_t)out & 15) == 0 && os[0] % 4 == 0 &&
                os[1] % 4 == 0 && os[2] % 4 == 0;
    const dim3 grid((unsigned)((L + kApplyRows - 1) / kApplyRows), (unsigned)((Dc + kApplyCols - 1) / kApplyCols),
                    (unsigned)(N * H));
    if (grid.y > 65535) return FTB_ERR_UNSUPPORTED;
    LaunchScope scope(FTB_KERNEL_APPLY_STATE, st);
    if (dtype == FTB_F32)
        apply_state_kernel<float><<<grid, kApplyThreads, 0, st>>>(p);
    else
        apply_state_kernel<__nv_bfloat16><<<grid, kApplyThreads, 0, st>>>(p);
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

int ftb_recurrent_cross_linear_step(const void *q, const float *S, const float *z, void *out, int64_t N,
                                    int64_t H, int64_t D, int64_t M, const int64_t *qs, const int64_t *os,
                                    int dtype, int feature_map, float eps, void *stream) {
    if (N < 0 || H < 0 || D < 0 || M < 0) return FTB_ERR_INVALID;
    if (dtype != FTB_F32 && dtype != FTB_BF16) return FTB_ERR_INVALID;
    if (feature_map != FTB_FEATURE_NONE && feature_map != FTB_FEATURE_ELU1) return FTB_ERR_INVALID;
    if (!qs || !os) return FTB_ERR_INVALID;
    if (D > kStepMaxD) return FTB_ERR_UNSUPPORTED;
    if (N == 0 || H == 0 || M == 0) return FTB_OK;
    if (N * H > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    if (!out || (D > 0 && (!q || !S || !z))) return FTB_ERR_INVALID;
    if (M % 4 == 0 && ((uintptr_t)S & 15)) return FTB_ERR_ALIGNMENT;
    cudaStream_t st = (cudaStream_t)stream;
    const Strides2 a{qs[0], qs[1]}, o{os[0], os[1]}, none{0, 0};
    // the read-only instantiation never writes through its state pointers
    float *Sw = const_cast<float *>(S), *zw = const_cast<float *>(z);
    LaunchScope scope(FTB_KERNEL_RECURRENT_STEP, st);
    if (dtype == FTB_F32)
        recurrent_step_kernel<float, false><<<(unsigned)(N * H), kStepThreads, 0, st>>>(
            (const float *)q, nullptr, nullptr, Sw, zw, (float *)out, (int)H, (int)D, (int)M, a, none, none, o,
            feature_map, eps);
    else
        recurrent_step_kernel<__nv_bfloat16, false><<<(unsigned)(N * H), kStepThreads, 0, st>>>(
            (const __nv_bfloat16 *)q, nullptr, nullptr, Sw, zw, (__nv_bfloat16 *)out, (int)H, (int)D, (int)M, a,
            none, none, o, feature_map, eps);
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

// ---------------------------------------------------------------------------------------------
// Forward product for callers that must not allocate.
//
// Some callers cannot obtain device memory at call time: code running inside a memory pool it
// does not own, a real-time or serving loop whose allocator is frozen after start-up, a plugin
// host that forbids cudaMalloc from plugins.  For them the scratch of the forward product lives
// in this file-scope device array, part of the library image: every GPU that loads the library
// carries these FTB_STATIC_SCRATCH_BYTES until the process exits.
//
// In host code the array's name is only a stand-in symbol, not a device address, so its address
// is looked up with cudaGetSymbolAddress -- once per device, with that device current -- and the
// looked-up pointer is what the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[FTB_STATIC_SCRATCH_BYTES];

static std::atomic<void *> g_static_scratch_ptr[64];   // per device ordinal, filled at first use

int ftb_causal_dot_product_static(const void *q, const void *k, const void *v, void *out, int64_t N,
                                  int64_t H, int64_t L, int64_t D, int64_t M, const int64_t *qs,
                                  const int64_t *ks, const int64_t *vs, const int64_t *os, int dtype,
                                  int mode, void *stream) {
    int dev = -1;
    FTB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return FTB_ERR_UNSUPPORTED;
    // Set-up: the first call on a device resolves the symbol, with that device current.  It is a
    // synchronous lookup, so it should happen before any stream capture begins.  The address is
    // kept per device ordinal, so a host thread that alternates between GPUs looks nothing up again.
    void *scratch = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (scratch == nullptr) {
        void *p = nullptr;
        FTB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        if (p == nullptr) return FTB_ERR_CUDA;
        g_static_scratch_ptr[dev].store(p, std::memory_order_release);
        scratch = p;
    }
    const size_t need = ftb_causal_workspace_bytes(N, H, L, D, M, dtype, mode, 0, 0);
    if (need > (size_t)FTB_STATIC_SCRATCH_BYTES) return FTB_ERR_STATIC_LIMIT;
    // Nothing below allocates: tensor maps are encoded on the host stack, kernels are launched
    // on `stream`, the per-segment states go to the static array.  Every value read from the
    // array during a call was written earlier in the same call, so stale contents are harmless.
    return ftb_causal_dot_product(q, k, v, out, N, H, L, D, M, qs, ks, vs, os, dtype, mode, nullptr,
                                  nullptr, 0, scratch, (size_t)FTB_STATIC_SCRATCH_BYTES, stream);
}

// ---------------------------------------------------------------------------------------------
// Exchange of per-rank states between the GPUs of one node (csrc/rank_exchange.cuh).
// ---------------------------------------------------------------------------------------------
// Device address of the status word of the current device, looked up once per device ordinal (the
// lookup is a synchronous runtime call, so ftb_exchange_create makes it and the launches below,
// which may be issued while a stream is being captured, only read the cached value).
static std::atomic<int *> g_status_ptr[64];
static int device_status_ptr(int **out) {
    int dev = -1;
    FTB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return FTB_ERR_UNSUPPORTED;
    int *p = g_status_ptr[dev].load(std::memory_order_acquire);
    if (!p) {
        FTB_CUDA(cudaGetSymbolAddress((void **)&p, mma::g_device_status));
        if (!p) return FTB_ERR_CUDA;
        g_status_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return FTB_OK;
}

static std::atomic<long long> g_exchange_wait_ns{xchg::kDefaultWaitNs};

static int exchange_check(int world, int64_t elems) {
    if (world < 1 || elems < 0) return FTB_ERR_INVALID;
    if (world > xchg::kMaxRanks) return FTB_ERR_UNSUPPORTED;
    if (elems % 4) return FTB_ERR_ALIGNMENT;   // moved 16 bytes at a time
    return FTB_OK;
}

size_t ftb_exchange_bytes(int world, int64_t elems) {
    if (exchange_check(world, elems) != FTB_OK) return 0;
    return xchg::layout(world, elems).bytes;
}

int ftb_exchange_create(int world, int64_t elems, void **buffer, unsigned char *handle) {
    if (!buffer || !handle) return FTB_ERR_INVALID;
    int rc = exchange_check(world, elems);
    if (rc) return rc;
    static_assert(sizeof(cudaIpcMemHandle_t) == FTB_EXCHANGE_HANDLE_BYTES, "IPC handle size");
    int *status = nullptr;
    rc = device_status_ptr(&status);
    if (rc) return rc;
    const size_t bytes = xchg::layout(world, elems).bytes;
    void *p = nullptr;
    FTB_CUDA(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        FTB_CUDA(e);
    }
    std::memcpy(handle, &h, sizeof(h));
    *buffer = p;
    return FTB_OK;
}

int ftb_exchange_open(const unsigned char *handle, void **peer_buffer) {
    if (!handle || !peer_buffer) return FTB_ERR_INVALID;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    FTB_CUDA(cudaIpcOpenMemHandle(peer_buffer, h, cudaIpcMemLazyEnablePeerAccess));
    return FTB_OK;
}

int ftb_exchange_close(void *peer_buffer) {
    if (!peer_buffer) return FTB_ERR_INVALID;
    FTB_CUDA(cudaIpcCloseMemHandle(peer_buffer));
    return FTB_OK;
}

int ftb_exchange_destroy(void *buffer) {
    if (!buffer) return FTB_ERR_INVALID;
    FTB_CUDA(cudaFree(buffer));
    return FTB_OK;
}

int ftb_exchange_wait_limit_ms(int ms) {
    const long long before = g_exchange_wait_ns.load();
    if (ms > 0) g_exchange_wait_ns.store((long long)ms * 1000000LL);
    return (int)(before / 1000000LL);
}

static int exchange_push(const float *state, int64_t elems, int64_t unit_elems, int parts_per_unit,
                         void *const *buffers, int rank, int world, int reverse, void *stream) {
    int rc = exchange_check(world, elems);
    if (rc) return rc;
    if (!buffers || rank < 0 || rank >= world || (elems > 0 && !state)) return FTB_ERR_INVALID;
    if ((uintptr_t)state & 15) return FTB_ERR_ALIGNMENT;
    xchg::Peers peers;
    for (int r = 0; r < xchg::kMaxRanks; ++r) peers.buf[r] = r < world ? buffers[r] : nullptr;
    for (int r = 0; r < world; ++r)
        if (!peers.buf[r]) return FTB_ERR_INVALID;
    const int targets = reverse ? rank : world - 1 - rank;
    const int64_t n4 = elems / 4;
    int64_t per_target = (n4 + (int64_t)xchg::kThreads * 4 - 1) / ((int64_t)xchg::kThreads * 4);
    per_target = std::max<int64_t>(1, std::min<int64_t>(per_target, 32));
    const dim3 grid(targets ? (unsigned)per_target : 1u, targets ? (unsigned)targets : 1u);
    cudaStream_t st = (cudaStream_t)stream;
    int *status = nullptr;
    rc = device_status_ptr(&status);
    if (rc) return rc;
    LaunchScope scope(FTB_KERNEL_RANK_EXCHANGE, st);
    xchg::push_kernel<<<grid, xchg::kThreads, 0, st>>>(state, elems, unit_elems, parts_per_unit, peers, rank,
                                                       world, reverse ? 1 : 0, status, g_exchange_wait_ns.load());
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

int ftb_exchange_push(const float *state, int64_t elems, void *const *buffers, int rank, int world,
                      int reverse, void *stream) {
    return exchange_push(state, elems, elems, 1, buffers, rank, world, reverse, stream);
}

int ftb_exchange_push_parts(const float *parts, int64_t unit_elems, int parts_per_unit, int64_t units,
                            void *const *buffers, int rank, int world, int reverse, void *stream) {
    if (unit_elems < 0 || units < 0 || parts_per_unit < 1) return FTB_ERR_INVALID;
    if (unit_elems % 4) return FTB_ERR_ALIGNMENT;
    return exchange_push(parts, unit_elems * units, unit_elems, parts_per_unit, buffers, rank, world, reverse,
                         stream);
}

int ftb_exchange_receive(void *buffer, float *out, int64_t elems, int rank, int world, int reverse,
                         void *stream) {
    int rc = exchange_check(world, elems);
    if (rc) return rc;
    if (!buffer || rank < 0 || rank >= world || (elems > 0 && !out)) return FTB_ERR_INVALID;
    if ((uintptr_t)out & 15) return FTB_ERR_ALIGNMENT;
    int *status = nullptr;
    rc = device_status_ptr(&status);
    if (rc) return rc;
    const int64_t n4 = elems / 4;
    int64_t blocks = (n4 + (int64_t)xchg::kThreads * 2 - 1) / ((int64_t)xchg::kThreads * 2);
    blocks = std::max<int64_t>(1, std::min<int64_t>(blocks, mma::sm_count()));
    cudaStream_t st = (cudaStream_t)stream;
    LaunchScope scope(FTB_KERNEL_RANK_EXCHANGE, st);
    xchg::receive_kernel<<<(unsigned)blocks, xchg::kThreads, 0, st>>>(buffer, out, elems, rank, world,
                                                                      reverse ? 1 : 0, status,
                                                                      g_exchange_wait_ns.load());
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

}  // extern "C"
