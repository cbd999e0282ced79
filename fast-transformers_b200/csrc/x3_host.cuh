// Host side of the split-operand tensor-core mode (x3_scan.cuh): plans, launches, forward and
// backward.  Part of ftb200.cu's translation unit: included there behind the launch helpers it
// uses (Plan, LaunchScope, launch_prefix, FTB_CUDA, x3_plan, x3_sub).
#pragma once

// ---- split-operand tensor-core mode (x3_scan.cuh): fp32, D = M = 64 ------------------------------
// One scan (a, b, c) -> out, or, with a == nullptr, the state-only sweep of (b, c) -> state_out.
static int x3_launch(const float *a, const float *b, const float *c, float *out, const int64_t *as,
                     const int64_t *bs, const int64_t *cs, const int64_t *os, int64_t N, int64_t H, int64_t L,
                     Plan pl, const float *states, int sum_mode, int sub, float *state_out, int skip_lo, int skip_hi,
                     int canon_is_DaDc, int reverse, bool after_own_launch, int kind, cudaStream_t st) {
    const int64_t blocks = N * H * pl.nseg;
    if (blocks <= 0) return FTB_OK;
    if (blocks > 0x7fffffffLL) return FTB_ERR_UNSUPPORTED;
    CUtensorMap ma, mb, mbmn, mc;
    x3::Params p;
    int rc;
    if ((rc = mma::make_map(&mb, p.pos_b, b, N, H, L, 64, bs, FTB_F32))) return rc;
    if ((rc = mma::make_map(&mbmn, p.pos_b, b, N, H, L, 64, bs, FTB_F32, true))) return rc;
    if ((rc = mma::make_map(&mc, p.pos_c, c, N, H, L, 64, cs, FTB_F32, true))) return rc;
    if (a) {
        if ((rc = mma::make_map(&ma, p.pos_a, a, N, H, L, 64, as, FTB_F32))) return rc;
        if (((uintptr_t)out & 15) || (os[0] * 4) % 16 || (os[1] * 4) % 16 || (os[2] * 4) % 16) return FTB_ERR_ALIGNMENT;
    } else {
        ma = mb;
        for (int i = 0; i < 3; ++i) p.pos_a[i] = p.pos_b[i];
    }
    p.out = out;
    p.so = a ? S3(os) : Strides3{0, 0, 0};
    p.H = (int)H; p.L = L;
    p.seg_len = pl.seg_len; p.nseg = pl.nseg;
    p.states = states; p.sum_mode = sum_mode; p.sub = sub < 1 ? 1 : sub; p.state_out = state_out;
    p.skip_lo = skip_lo; p.skip_hi = skip_hi;
    p.canon_is_DaDc = canon_is_DaDc; p.reverse = reverse; p.state_only = a ? 0 : 1;
    static const char *no_pdl = std::getenv("FTB200_NO_PDL");
    p.wait_first = (no_pdl || after_own_launch) ? 0 : 1;
    FTB_CUDA(cudaFuncSetAttribute(x3::x3_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)x3::kSmem));
    LaunchScope scope(kind, st);
    if (!no_pdl) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)blocks);
        cfg.blockDim = dim3(mma::NTHREADS);
        cfg.dynamicSmemBytes = x3::kSmem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, x3::x3_scan_kernel, ma, mb, mbmn, mc, p) == cudaSuccess) return FTB_OK;
        (void)cudaGetLastError();
        p.wait_first = 0;
    }
    x3::x3_scan_kernel<<<(unsigned)blocks, mma::NTHREADS, x3::kSmem, st>>>(ma, mb, mbmn, mc, p);
    FTB_CUDA(cudaGetLastError());
    return FTB_OK;
}

// Where a split-operand scan finds its segment-start states.
struct X3States {
    const float *states = nullptr;
    int sum_mode = 0;     // 1: raw totals, `sub` blocks per segment, added up by the scan
    int sub = 1;
};

static X3States x3_describe(Plan pl, int64_t BH, const float *ws) {
    X3States s;
    if (pl.nseg == 1) return s;
    s.states = ws;
    s.sum_mode = pl.nseg <= mma::kSumInKernelMaxSegs ? 1 : 0;
    s.sub = s.sum_mode ? x3_sub(pl, BH) : 1;
    return s;
}

// Per-segment totals of sum x (x) y into `ws`, as what the scans read.
static int x3_states(const float *x, const float *y, const int64_t *xs, const int64_t *ys, int64_t N, int64_t H,
                     int64_t L, Plan pl, float *ws, int reverse, bool after_own_launch, cudaStream_t st,
                     X3States *out) {
    *out = x3_describe(pl, N * H, ws);
    if (pl.nseg == 1) return FTB_OK;
    Plan fine = pl;
    int skip_lo = 0, skip_hi = 0;
    if (out->sum_mode) {     // the scan adds up raw totals itself: the segment nobody reads from is skipped
        fine.seg_len = pl.seg_len / out->sub;
        fine.nseg = pl.nseg * out->sub;
        skip_lo = reverse ? 0 : (pl.nseg - 1) * out->sub;
        skip_hi = skip_lo + out->sub;
    }
    int rc = x3_launch(nullptr, x, y, nullptr, nullptr, xs, ys, nullptr, N, H, L, fine, nullptr, 0, 1, ws, skip_lo,
                       skip_hi, 1, 0, after_own_launch, FTB_KERNEL_MMA_STATE, st);
    if (rc || out->sum_mode) return rc;
    return launch_prefix(ws, nullptr, nullptr, nullptr, N * H, pl.nseg, 4096, reverse, st);
}

static int x3_forward(const float *q, const float *k, const float *v, float *out, int64_t N, int64_t H, int64_t L,
                      const int64_t *qs, const int64_t *ks, const int64_t *vs, const int64_t *os, float *ws,
                      cudaStream_t st) {
    const Plan pl = x3_plan(N * H, L);
    X3States ss;
    int rc = x3_states(k, v, ks, vs, N, H, L, pl, ws, 0, false, st, &ss);
    if (rc) return rc;
    // (behind a sweep of this call the scan waits only for the totals; a prefix launch in between
    // is not one of these kernels: then the scan waits for everything in front)
    const bool own = ss.states && ss.sum_mode == 1;
    return x3_launch(q, k, v, out, qs, ks, vs, os, N, H, L, pl, ss.states, ss.sum_mode, ss.sub, nullptr, 0, 0, 1, 0,
                     own, FTB_KERNEL_MMA_FWD, st);
}

static int x3_backward(const float *q, const float *k, const float *v, const float *g, float *gq, float *gk,
                       float *gv, int64_t N, int64_t H, int64_t L, const int64_t *qs, const int64_t *ks,
                       const int64_t *vs, const int64_t *gs, const int64_t *gqs, const int64_t *gks,
                       const int64_t *gvs, const float *forward_workspace, float *workspace, size_t workspace_bytes,
                       cudaStream_t st) {
    const Plan pl = x3_plan(N * H, L);
    float *wsS = workspace, *wsR = (float *)((char *)workspace + workspace_bytes / 2);
    X3States sS, sR;
    int rc;
    bool own = false;      // is the launch in front one of this call's scan kernels?
    if (gq) {
        if (forward_workspace && pl.nseg > 1) {
            sS = x3_describe(pl, N * H, forward_workspace);
        } else {
            if ((rc = x3_states(k, v, ks, vs, N, H, L, pl, wsS, 0, false, st, &sS))) return rc;
            own = sS.states && sS.sum_mode == 1;
        }
    }
    // grad_K and grad_V over WHOLE sequences where that takes fewer chunk times than a sweep of
    // (q, grad_out) and two grids over the segments: no reverse totals then, and the two grids run
    // side by side (the second is started programmatically while the first one runs; config 2:
    // two grids of 64 blocks x 32 chunks at once instead of three grids of 128 x 16 in a row)
    Plan pl_kv = pl;
    if (gk && gv && pl.nseg > 1) {
        const int64_t sms = mma::sm_count(), chunks = (L + mma::C - 1) / mma::C, cps = pl.seg_len / mma::C;
        const int64_t whole = (2 * N * H + sms - 1) / sms * (chunks + 1);
        const int64_t split = 3 * ((N * H * pl.nseg + sms - 1) / sms) * (cps + 1);
        if (whole <= split) {
            pl_kv.nseg = 1;
            pl_kv.seg_len = chunks * mma::C;
        }
    }
    if ((gk || gv) && pl_kv.nseg > 1) {
        if ((rc = x3_states(q, g, qs, gs, N, H, L, pl, wsR, 1, own, st, &sR))) return rc;
        own = sR.states ? sR.sum_mode == 1 : own;
    }
    // (a scan directly behind this call's own sweeps or scans waits only for the totals it reads:
    // everything else it reads is the caller's input)
    if (gq) {
        if ((rc = x3_launch(g, v, k, gq, gs, vs, ks, gqs, N, H, L, pl, sS.states, sS.sum_mode, sS.sub, nullptr, 0, 0, 0,
                            0, own, FTB_KERNEL_MMA_BWD, st)))
            return rc;
        own = true;
    }
    if (gk) {
        if ((rc = x3_launch(v, g, q, gk, vs, gs, qs, gks, N, H, L, pl_kv, sR.states, sR.sum_mode, sR.sub, nullptr, 0, 0,
                            0, 1, own, FTB_KERNEL_MMA_BWD, st)))
            return rc;
        own = true;
    }
    if (gv && (rc = x3_launch(k, q, g, gv, ks, qs, gs, gvs, N, H, L, pl_kv, sR.states, sR.sum_mode, sR.sub, nullptr, 0,
                              0, 1, 1, own, FTB_KERNEL_MMA_BWD, st)))
        return rc;
    return FTB_OK;
}
