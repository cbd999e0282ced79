// Host side of the wide scans (wide_scan.cuh): fp32 tensors in tensor-core mode whose widths are
// multiples of 64 with at least one above 64.  Part of ftb200.cu's translation unit: included
// there behind the launch helpers it uses (Plan, SegStates, MmaBatch, mma_add_job,
// mma_launch_batch, launch_prefix, LaunchScope, FTB_CUDA, WidePlan, wide_plan).
#pragma once

// ---- wide widths (D = 64 nb, M = 64 mt, fp32, tensor cores) ------------------------------------
// The states of a (pair, segment) are kept as one [D][M] block; feature block b is its rows
// 64 b .. 64 b + 63.  A scan that is wide on its a / b side (out and grad_V always; grad_Q and
// grad_K when M > 64) takes the sum over the 64-wide blocks of that side inside the tensor cores
// (wide_scan_kernel), up to four blocks per launch and one launch per 64 columns of its c side.
// With M = 64, grad_Q and grad_K are wide on the c / out side only: scores and mask once per chunk,
// the column blocks of K (Q) streamed (wide_c_scan_kernel).  The state-only sweeps of the feature
// blocks share one grid, block by block, so that V (grad_out) is read once there as well.

// Per-segment totals of sum x_b (x) y for every feature block b into `ws`; on return `ss`
// describes them for a scan over feature block 0 (block b: states + 64 b M).
static int wide_states(const float *x, const float *y, const int64_t *xs, const int64_t *ys, int64_t N,
                       int64_t H, int64_t L, int nb, int M, const WidePlan &w, float *ws, int reverse,
                       cudaStream_t st, SegStates *ss) {
    const int64_t DM = (int64_t)64 * nb * M;
    *ss = SegStates{nullptr, nullptr, 0, 1};
    if (w.pl.nseg == 1) return FTB_OK;
    const bool in_kernel = sums_in_kernel(FTB_MODE_MMA, w.pl);
    Plan fine = w.pl;
    int skip_lo = 0, skip_hi = 0;
    if (in_kernel) {
        fine.seg_len = w.pl.seg_len / w.sub;
        fine.nseg = w.pl.nseg * w.sub;
        skip_lo = reverse ? 0 : (w.pl.nseg - 1) * w.sub;
        skip_hi = skip_lo + w.sub;
    }
    MmaBatch sweep;
    for (int b = 0; b < nb; ++b) {
        if (sweep.b.njobs == mma::MAX_JOBS) {
            int rc = mma_launch_batch(sweep, st);
            if (rc) return rc;
            sweep = MmaBatch();
        }
        int rc = mma_add_job(sweep, nullptr, x + 64 * b, y, nullptr, nullptr, xs, ys, nullptr, N, H, L, 64, M,
                             FTB_F32, fine, nullptr, nullptr, 0, 1, ws + (int64_t)64 * b * M, skip_lo, skip_hi, 1, 0,
                             nullptr, DM);
        if (rc) return rc;
    }
    int rc = mma_launch_batch(sweep, st);
    if (rc) return rc;
    if (in_kernel) {
        *ss = SegStates{ws, nullptr, 1, w.sub, 1};
        return FTB_OK;
    }
    rc = launch_prefix(ws, nullptr, nullptr, nullptr, N * H, w.pl.nseg, DM, reverse, st);
    *ss = SegStates{ws, nullptr, 0, 1, 1};
    return rc;
}

static SegStates wide_describe(const WidePlan &w, const float *ws) {
    if (w.pl.nseg == 1) return SegStates{nullptr, nullptr, 0, 1};
    if (sums_in_kernel(FTB_MODE_MMA, w.pl)) return SegStates{ws, nullptr, 1, w.sub};
    return SegStates{ws, nullptr, 0, 1};
}

// One launch of the scan that sums over `cnt` (1 .. 4) feature blocks inside the tensor cores
// (wide_scan.cuh): a, b are rows of 64 cnt floats, c and out rows of 64.
static int wide_launch(const float *a, const float *b, const float *c, float *out, const int64_t *as,
                       const int64_t *bs, const int64_t *cs, const int64_t *os, int64_t N, int64_t H, int64_t L,
                       int cnt, const WidePlan &w, const float *states, int sum_mode, int sub, int64_t state_blk,
                       int64_t state_ld, int state_transposed, int reverse, int accumulate, bool after_own_launch,
                       int kind, cudaStream_t st) {
    const int64_t blocks = N * H * w.pl.nseg;
    if (blocks <= 0) return FTB_OK;
    if (blocks > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    CUtensorMap ma, mb, mc;
    wide::Params p;
    p.state_ld = state_ld;
    p.state_transposed = state_transposed;
    int rc = mma::make_map(&ma, p.pos_a, a, N, H, L, 64 * cnt, as, FTB_F32);
    if (rc) return rc;
    if ((rc = mma::make_map(&mb, p.pos_b, b, N, H, L, 64 * cnt, bs, FTB_F32))) return rc;
    if ((rc = mma::make_map(&mc, p.pos_c, c, N, H, L, 64, cs, FTB_F32, true))) return rc;
    if (((uintptr_t)out & 15) || (os[0] * 4) % 16 || (os[1] * 4) % 16 || (os[2] * 4) % 16) return FTB_ERR_ALIGNMENT;
    p.out = out;
    p.so = S3(os);
    p.H = (int)H; p.L = L;
    p.seg_len = w.pl.seg_len; p.nseg = w.pl.nseg; p.nb = cnt;
    p.states = states; p.sum_mode = sum_mode; p.sub = sub < 1 ? 1 : sub; p.state_blk = state_blk;
    p.reverse = reverse; p.accumulate = accumulate;
    static const char *no_pdl = std::getenv("FTB200_NO_PDL");
    p.wait_first = (no_pdl || after_own_launch) ? 0 : 1;
    FTB_CUDA(cudaFuncSetAttribute(wide::wide_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)wide::kSmem));
    LaunchScope scope(kind, st);
    if (!no_pdl) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)blocks);
        cfg.blockDim = dim3(mma::NTHREADS);
        cfg.dynamicSmemBytes = wide::kSmem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, wide::wide_scan_kernel, ma, mb, mc, p) == cudaSuccess) return FTB_OK;
        (void)cudaGetLastError();
        p.wait_first = 0;
    }
    wide::wide_scan_kernel<<<(unsigned)blocks, mma::NTHREADS, wide::kSmem, st>>>(ma, mb, mc, p);
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

// One launch of the scan that is wide on the c / out side (wide_c_scan_kernel): a, b rows of 64
// floats, c and out rows of 64 cnt (cnt = 2 .. 4).
static int wide_c_launch(const float *a, const float *b, const float *c, float *out, const int64_t *as,
                         const int64_t *bs, const int64_t *cs, const int64_t *os, int64_t N, int64_t H, int64_t L,
                         int cnt, const WidePlan &w, const float *states, int sum_mode, int sub, int64_t state_blk,
                         int reverse, bool after_own_launch, int kind, cudaStream_t st) {
    const int64_t blocks = N * H * w.pl.nseg;
    if (blocks <= 0) return FTB_OK;
    if (blocks > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    CUtensorMap ma, mb, mc;
    wide::ParamsC p;
    int rc = mma::make_map(&ma, p.pos_a, a, N, H, L, 64, as, FTB_F32);
    if (rc) return rc;
    if ((rc = mma::make_map(&mb, p.pos_b, b, N, H, L, 64, bs, FTB_F32))) return rc;
    if ((rc = mma::make_map(&mc, p.pos_c, c, N, H, L, 64 * cnt, cs, FTB_F32, true))) return rc;
    if (((uintptr_t)out & 15) || (os[0] * 4) % 16 || (os[1] * 4) % 16 || (os[2] * 4) % 16) return FTB_ERR_ALIGNMENT;
    p.out = out;
    p.so = S3(os);
    p.H = (int)H; p.L = L;
    p.seg_len = w.pl.seg_len; p.nseg = w.pl.nseg; p.nb = cnt;
    p.states = states; p.sum_mode = sum_mode; p.sub = sub < 1 ? 1 : sub; p.state_blk = state_blk;
    p.reverse = reverse;
    static const char *no_pdl = std::getenv("FTB200_NO_PDL");
    p.wait_first = (no_pdl || after_own_launch) ? 0 : 1;
    FTB_CUDA(cudaFuncSetAttribute(wide::wide_c_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)wide::kSmem));
    LaunchScope scope(kind, st);
    if (!no_pdl) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)blocks);
        cfg.blockDim = dim3(mma::NTHREADS);
        cfg.dynamicSmemBytes = wide::kSmem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, wide::wide_c_scan_kernel, ma, mb, mc, p) == cudaSuccess) return FTB_OK;
        (void)cudaGetLastError();
        p.wait_first = 0;
    }
    wide::wide_c_scan_kernel<<<(unsigned)blocks, mma::NTHREADS, wide::kSmem, st>>>(ma, mb, mc, p);
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

// One scan that is wide on the a / b side, as launches of up to four feature blocks per 64 columns
// of c / out: (a, b) rows of 64 na floats, c and out rows of 64 nc.  `states` as wide_states leaves
// them ([64 na][64 nc] per block) -- or transposed ([64 nc][64 na]) for the scans whose a / b side
// is the stored blocks' column side (grad_Q, grad_K).  `own`: whether the launch in front is one of
// this call's (updated).
static int wide_scan_ab(const float *a, const float *b, const float *c, float *out, const int64_t *as,
                        const int64_t *bs, const int64_t *cs, const int64_t *os, int64_t N, int64_t H, int64_t L,
                        int na, int nc, const WidePlan &w, const SegStates &ss, int64_t DM, int transposed,
                        int reverse, int kind, bool *own, cudaStream_t st) {
    const int64_t ld = transposed ? 64 * na : 64 * nc;     // row length of a stored block
    for (int t = 0; t < nc; ++t)
        for (int b0 = 0; b0 < na; b0 += wide::MAXNB) {
            // a later group of feature blocks adds to what the one before wrote and waits for that
            // whole grid; the first group of a column tile depends on nothing in front but totals
            const int cnt = na - b0 < wide::MAXNB ? na - b0 : wide::MAXNB;
            const float *st0 = nullptr;
            if (ss.states)
                st0 = transposed ? ss.states + (int64_t)64 * t * ld + 64 * b0 : ss.states + (int64_t)64 * b0 * ld + 64 * t;
            int rc = wide_launch(a + 64 * b0, b + 64 * b0, c + 64 * t, out + 64 * t, as, bs, cs, os, N, H, L, cnt, w, st0,
                                 ss.sum_mode, ss.sub, DM, ld, transposed, reverse, b0 > 0, b0 == 0 && *own, kind, st);
            if (rc) return rc;
            *own = true;
        }
    return FTB_OK;
}

static int wide_forward(const float *q, const float *k, const float *v, float *out, int64_t N, int64_t H,
                        int64_t L, int nb, int M, const int64_t *qs, const int64_t *ks, const int64_t *vs,
                        const int64_t *os, float *ws, cudaStream_t st) {
    const int64_t DM = (int64_t)64 * nb * M;
    const WidePlan w = wide_plan(N * H, L, nb, M);
    SegStates ss;
    int rc = wide_states(k, v, ks, vs, N, H, L, nb, M, w, ws, 0, st, &ss);
    if (rc) return rc;
    bool own = ss.fresh != 0;
    return wide_scan_ab(q, k, v, out, qs, ks, vs, os, N, H, L, nb, M / 64, w, ss, DM, 0, 0, FTB_KERNEL_MMA_FWD, &own, st);
}

static int wide_backward(const float *q, const float *k, const float *v, const float *g, float *gq, float *gk,
                         float *gv, int64_t N, int64_t H, int64_t L, int nb, int M, const int64_t *qs,
                         const int64_t *ks, const int64_t *vs, const int64_t *gs, const int64_t *gqs,
                         const int64_t *gks, const int64_t *gvs, const float *forward_workspace, float *workspace,
                         size_t workspace_bytes, cudaStream_t st) {
    const int D = 64 * nb, mt = M / 64;
    const int64_t DM = (int64_t)D * M;
    const WidePlan w = wide_plan(N * H, L, nb, M);
    float *wsS = workspace;
    float *wsR = (float *)((char *)workspace + workspace_bytes / 2);
    int rc;
    SegStates sS{nullptr, nullptr, 0, 1}, sR{nullptr, nullptr, 0, 1};
    if (gq) {
        if (forward_workspace && w.pl.nseg > 1) sS = wide_describe(w, forward_workspace);
        else if ((rc = wide_states(k, v, ks, vs, N, H, L, nb, M, w, wsS, 0, st, &sS))) return rc;
    }
    if ((gk || gv) && (rc = wide_states(q, g, qs, gs, N, H, L, nb, M, w, wsR, 1, st, &sR))) return rc;
    bool own = sS.fresh || sR.fresh;      // is the launch in front one of this call's?
    // grad_Q: (grad_out, V, K) and grad_K: (V, grad_out, Q) walked downwards.  Their a / b side is
    // the value side (64 mt wide), their c / out side the feature side (D wide).
    for (int which = 0; which < 2; ++which) {
        float *dst = which == 0 ? gq : gk;
        if (!dst) continue;
        const float *a = which == 0 ? g : v, *b = which == 0 ? v : g, *c = which == 0 ? k : q;
        const int64_t *as = which == 0 ? gs : vs, *bs = which == 0 ? vs : gs, *cs = which == 0 ? ks : qs;
        const int64_t *os = which == 0 ? gqs : gks;
        const SegStates &ss = which == 0 ? sS : sR;
        if (mt > 1) {
            // wide on both sides: the sum over the value blocks inside the tensor cores, one launch
            // per 64 feature columns (the stored [D][M] blocks read transposed)
            rc = wide_scan_ab(a, b, c, dst, as, bs, cs, os, N, H, L, mt, nb, w, ss, DM, 1, which, FTB_KERNEL_MMA_BWD,
                              &own, st);
            if (rc) return rc;
            continue;
        }
        // 64 value columns: wide on the c / out side only -- scores and mask once per chunk, the
        // column blocks of K (Q) streamed, up to four per launch (a single left-over block: the
        // 64-wide scan)
        for (int b0 = 0; b0 < nb; b0 += wide::MAXNB) {
            const int cnt = nb - b0 < wide::MAXNB ? nb - b0 : wide::MAXNB;
            const float *st0 = ss.states ? ss.states + (int64_t)64 * b0 * M : nullptr;
            if (cnt == 1) {
                MmaBatch one;
                one.after_own_launch = own;
                rc = mma_add_job(one, a, b, c + 64 * b0, dst + 64 * b0, as, bs, cs, os, N, H, L, M, 64, FTB_F32, w.pl,
                                 st0, nullptr, ss.sum_mode, ss.sub, nullptr, 0, 0, 0, which, nullptr, DM);
                if (rc) return rc;
                one.kind = FTB_KERNEL_MMA_BWD;
                rc = mma_launch_batch(one, st);
            } else {
                rc = wide_c_launch(a, b, c + 64 * b0, dst + 64 * b0, as, bs, cs, os, N, H, L, cnt, w, st0, ss.sum_mode,
                                   ss.sub, DM, which, own, FTB_KERNEL_MMA_BWD_MULTI, st);
            }
            if (rc) return rc;
            own = true;
        }
    }
    // grad_V: (K, Q, grad_out) walked downwards: the sum over the feature blocks
    if (gv)
        return wide_scan_ab(k, q, g, gv, ks, qs, gs, gvs, N, H, L, nb, mt, w, sR, DM, 0, 1, FTB_KERNEL_MMA_BWD, &own, st);
    return FTB_OK;
}
