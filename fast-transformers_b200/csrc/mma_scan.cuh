// Tensor-core (tcgen05 / TMEM / TMA) segment scan of the causal linear-attention product.
//
// One CTA walks one segment of one (batch, head) pair in chunks of C = 128 rows.  With the
// role triple (a, b, c) = (Q, K, V) -- and (G, V, K), (V, G, Q), (K, Q, G) for the three
// gradients, the last two with rows walked downwards and the mask flipped -- a chunk is
//
//   P   = a_c b_c^T                      tcgen05.mma  128 x 128, K = DA     (smem x smem)
//   O   = a_c S                          tcgen05.mma  128 x DCT, K = DA     (smem x smem)
//   O  += mask(P) c_c                    tcgen05.mma  128 x DCT, K = 128    (TMEM x smem)
//   S  += b_c^T c_c                      tcgen05.mma  DA  x DCT, K = 128    (smem x smem)
//
// P, O and the fp32 running state S live in tensor memory.  a_c, b_c, c_c arrive by TMA
// (128-byte swizzle) in a two-stage mbarrier ring; one tile layout serves as K-major operand
// (P, a S) and as MN-major operand (mask(P) c, b^T c).  Four worker warps own one TMEM lane
// (= one row) each: they apply the causal mask to P in place (only the diagonal 32x32 blocks
// need arithmetic), write O rows to global memory, and copy the updated state to shared
// memory where the next chunk's "a_c S" product reads it as an operand (TF32 reads the fp32
// bits; the bf16 variant rounds this operand copy only -- the accumulated state stays fp32).
//
// Warp roles: warp 0 = TMA producer (+ TMEM allocation), warps 1 and 10 = single-thread MMA
// issuers (outputs / scores and state; each elected with elect.sync), warps 2-5 = state workers
// (the loop-carried chain: state update -> operand copy -> next a S), warps 6-9 = output workers
// (O rows -> global memory; for TF32 they also make the MN-major image of b in place while the
// mask workers mask), warps 11-14 = mask workers.  Every wait is bounded: on expiry the CTA records
// FTB_ERR_TIMEOUT in a device status word, stops issuing work, releases its tensor memory and
// returns.
//
// Maths: fast_transformers/causal_product/causal_product_cpu.cpp:106-121, :165-206 in blocks.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "simt_scan.cuh"

namespace ftb {
namespace mma {

constexpr int C = 128;          // rows per chunk
// 15 warps: TMA (0), MMA issuers (1 and 10), state workers (2-5), output workers (6-9),
// mask workers (11-14)
constexpr int NTHREADS = 480;
constexpr int STAGES = 2;

__device__ int g_device_status = 0;   // 0 ok, else FTB_ERR_* recorded by a kernel


struct ScanParams {
    void *out;            // output tensor (scan) or nullptr (state only)
    Strides3 so;
    int H;
    int64_t L;
    int Dc;               // full width of c / out rows
    int64_t seg_len;      // multiple of C
    int nseg;
    const float *states;  // per (bh, seg) canonical [D][M] blocks, or nullptr (see sum_mode)
    const float *init;    // per bh state added to every segment's start, or nullptr
    int sum_mode;         // 0: states[bh][seg] is the state the segment starts from;
                          // 1: states holds raw per-segment totals: the start state is their sum
                          //    over the segments before (reverse: after) this one
    int skip_lo, skip_hi; // state-only mode: segments [skip_lo, skip_hi) whose totals nobody reads
    int sub;              // sum_mode 1: `states` holds `sub` blocks per segment of this launch (the
                          // state-only launch ran on `sub` times finer segments to fill more SMs)
    float *state_out;     // state-only mode: per (bh, seg) totals, canonical [DA][Dc]
    int canon_is_DaDc;    // canonical block is [DA][Dc] (1) or [Dc][DA] (0)
    int reverse;
    int state_only;
    const float *row_den; // scans: out row i is multiplied by 1 / (row_den[i] + eps) on its way to memory
    Strides3 sden;        // (the layer's normaliser, one fp32 value per (batch, head, position)); or nullptr
    float eps;
    int64_t state_blk;    // floats between consecutive (bh, seg) blocks of `states` / `state_out`; 0: DA * Dc
                          // (a 64-row feature block of a wider [D][M] state sits inside a block of D * M)
    int pos_a[3], pos_b[3], pos_c[3];   // TMA coordinate slot of {position, head, batch}
};

// One launch carries up to five independent jobs (scans or state-only sweeps over the same
// problem shape); job j owns the blocks [first_block[j], first_block[j+1]).  Independent scans
// in one grid keep every SM busy while the last CTAs of the previous scan finish, and a short
// state-only job rides on the SMs a 128-CTA scan leaves idle.
constexpr int MAX_JOBS = 5;
struct ScanJob {
    CUtensorMap ma, mb, mbmn, mc;   // a, b (K-major image), b (MN-major image), c
    ScanParams p;
};
struct ScanBatch {
    ScanJob job[MAX_JOBS];
    int first_block[MAX_JOBS + 1];
    int njobs;
    int interleave;   // jobs have equal block counts: block i belongs to job i % njobs
    // Programmatic stream serialisation.  0: the launch in front is this call's own (or the launch
    // is an ordinary one): blocks start at once and wait only where they read that launch's totals.
    // 1: the launch in front may be anybody's: every block waits for it before its first access to
    // global memory, and only its set-up (barriers, tensor memory) overlaps the other grid's tail.
    int wait_first;
};

// ---- small PTX wrappers -------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Non-blocking test of a phase (for a role that polls several barriers at once).
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait.  Returns false after ~2 s of polling or when another role has given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 63u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > 4000000000LL) {
                *abort_flag = 1;
                atomicExch(&g_device_status, 5 /* FTB_ERR_TIMEOUT */);
                return false;
            }
        }
    }
}
// One thread of a converged warp (the hardware picks it).  Code under this predicate is known to
// the compiler to run on a single thread, unlike code under `lane == 0`.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int c0, const int *pos, int row, int head, int batch) {
    int crd[3];
    crd[pos[0]] = row;
    crd[pos[1]] = head;
    crd[pos[2]] = batch;
    const int c1 = crd[0], c2 = crd[1], c3 = crd[2];
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
        : "memory");
}
// Pull one box towards L2 only (no shared-memory slot, no barrier).
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap *map, int c0, const int *pos, int row,
                                                int head, int batch) {
    int crd[3];
    crd[pos[0]] = row;
    crd[pos[1]] = head;
    crd[pos[2]] = batch;
    const int c1 = crd[0], c2 = crd[1], c3 = crd[2];
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
template <bool F16>
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
    if constexpr (F16) {
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n" ::"r"(d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
template <bool F16>
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
    if constexpr (F16) {
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d),
            "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d),
            "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16x256(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 64 columns of one lane quarter in one load (waits for the data).
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
}
// Zero `n` consecutive columns of this warp's lanes: one source register, named n times.
__device__ __forceinline__ void tmem_st_zero16(uint32_t taddr) {
    const uint32_t z = 0u;
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(z) : "memory");
}
__device__ __forceinline__ void tmem_st_zero32(uint32_t taddr) {
    const uint32_t z = 0u;
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(z) : "memory");
}
__device__ __forceinline__ void tmem_st_zero64(uint32_t taddr) {
    const uint32_t z = 0u;
    asm volatile("tcgen05.st.sync.aligned.32x32b.x64.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(z) : "memory");
}
// Zero `ncols` (a multiple of 16, at most 96) columns starting at `taddr`, in as few stores as possible.
__device__ __forceinline__ void tmem_zero_columns(uint32_t taddr, int ncols) {
    if (ncols >= 64) { tmem_st_zero64(taddr); taddr += 64; ncols -= 64; }
    if (ncols >= 32) { tmem_st_zero32(taddr); taddr += 32; ncols -= 32; }
    if (ncols >= 16) tmem_st_zero16(taddr);
}

// ---- descriptors ----------------------------------------------------------------------------
// Shared-memory matrix descriptor (descriptor version 1).  layout 2 = 128-byte swizzle with
// 16-byte atoms (K-major operands, and MN-major 16-bit operands); layout 1 = 128-byte swizzle
// with 32-byte atoms, the only layout MN-major 32-bit (TF32) operands may use.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout = 2) {
    uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)layout << 61;
    return d;
}
// Instruction descriptor: fp32 accumulate; fmt 1 = bf16, 2 = tf32; *_mn = 1 for MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int fmt, int a_mn, int b_mn, int M, int N) {
    return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)a_mn << 15) |
           ((uint32_t)b_mn << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

template <typename T, int DA, int DCT>
struct Cfg {
    static constexpr bool F16 = sizeof(T) == 2;
    static constexpr int EPB = 128 / sizeof(T);           // elements per 128-byte block
    static constexpr int KROWS = 32 / sizeof(T);          // K extent of one instruction
    static constexpr int A_BLKS = DA / EPB;               // 128-byte blocks per a/b row
    static constexpr int C_BLKS = DCT / EPB;
    static constexpr int BLK_BYTES = C * 128;             // one [C rows][128 B] block
    static constexpr int A_BYTES = A_BLKS * BLK_BYTES;
    static constexpr int C_BYTES = C_BLKS * BLK_BYTES;
    static constexpr int STAGE_BYTES = 2 * A_BYTES + C_BYTES;
    static constexpr int SM_BLK_BYTES = DA * 128;          // state operand: [DA rows][128 B]
    static constexpr int SM_BYTES = C_BLKS * SM_BLK_BYTES;
    static constexpr int NOBUF = (256 + 2 * DCT + DCT <= 512) ? 2 : 1;
    static constexpr int TM_P = 0;                         // two score buffers, 128 columns each
    static constexpr int TM_O = 256;
    static constexpr int TM_S = 256 + NOBUF * DCT;
    static constexpr int FMT = F16 ? 1 : 2;
    // MN-major operands: 16-bit types share the K-major tile image (layout 2, 8-row atoms);
    // TF32 needs the 32-byte-atom swizzle (layout 1, 4-row atoms), so the b tile -- read
    // K-major by the score product and MN-major by the state update -- needs a second image:
    // the mask workers rearrange the tile in place once the score product has consumed it
    // (a state-only launch loads the MN-major image directly).
    static constexpr bool RELOAD_B = !F16;
    // state-only launches: the same ring memory as slots of b | c
    static constexpr int SO_BYTES = A_BYTES + C_BYTES;
    static constexpr int SO_STAGES = (STAGES * STAGE_BYTES) / SO_BYTES;
    static_assert(SO_STAGES >= 2 && SO_STAGES <= 4, "state-only ring: barrier slots for up to 4 stages");
    static_assert(SO_BYTES % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
    // Where the running fp32 state lives.  REG_STATE: each chunk's increment b^T c goes to one of
    // two fresh TMEM accumulators and the state workers add it to the state they keep in
    // registers (one row per thread) -- the state update of chunk c+1 then does not wait for the
    // operand copy of chunk c.  Otherwise the increments accumulate in place in TMEM.
    static constexpr bool REG_STATE = !F16;
    static constexpr uint32_t MN_LAYOUT = F16 ? 2 : 1;
    static constexpr uint32_t MN_SBO = F16 ? 1024 : 512;
    static constexpr size_t SMEM = 1024 /* alignment slack */ + STAGES * STAGE_BYTES + SM_BYTES + 384;
    static_assert(DA % EPB == 0 && DCT % EPB == 0, "rows must be whole 128-byte blocks");
    static_assert(DA == 64 || DA == 128, "state rows map to 64 or 128 TMEM lanes");
    static_assert(TM_S + (REG_STATE ? 2 : 1) * DCT <= 512, "tensor memory budget");
};

// APPLY: the instantiation that computes out = a S_init only -- no scores, no state update; b and c
// are not read (a compile-time switch, so that the scan's own code is untouched by it).
template <typename T, int DA, int DCT, bool APPLY = false>
__global__ void __launch_bounds__(NTHREADS, 1)
mma_scan_kernel(const __grid_constant__ ScanBatch batch) {
    using K = Cfg<T, DA, DCT>;
    constexpr bool apply_only = APPLY;
    // which job this block belongs to (everything below is per job)
    int job = 0, job_block = 0;
    if (batch.interleave) {
        // equal-sized jobs: blocks of the same segment sit next to each other in the grid, are
        // dispatched together and walk their chunks at the same pace, so the tiles two gradient
        // scans share (grad_K and grad_V both read Q and grad_out) are fetched from HBM once
        // and found in L2 the second time
        job = (int)(blockIdx.x % (unsigned)batch.njobs);
        job_block = (int)(blockIdx.x / (unsigned)batch.njobs);
    } else {
        while (job + 1 < batch.njobs && (int)blockIdx.x >= batch.first_block[job + 1]) ++job;
        job_block = (int)blockIdx.x - batch.first_block[job];
    }
    // let a grid launched behind this one with programmatic stream serialisation start as SMs
    // become free (it waits for this grid's results where it needs them)
    if (!batch.wait_first) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const ScanJob &J = batch.job[job];
    const ScanParams &p = J.p;
    const CUtensorMap &map_a = J.ma, &map_b = J.mb, &map_bmn = J.mbmn, &map_c = J.mc;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t stage0 = smem_base;
    const uint32_t sm_state = smem_base + STAGES * K::STAGE_BYTES;
    uint8_t *sm_state_gen = smem_gen + STAGES * K::STAGE_BYTES;
    const uint32_t bars = sm_state + K::SM_BYTES;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm_state_gen + K::SM_BYTES + 256);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm_state_gen + K::SM_BYTES + 264);
    // barrier addresses (8 bytes each)
    const uint32_t bar_full = bars, bar_empty = bars + 16, bar_pfull = bars + 32,
                   bar_pready = bars + 48, bar_ofull = bars + 64, bar_ofree = bars + 80,
                   bar_sfull = bars + 96, bar_smready = bars + 104, bar_fullc = bars + 112,
                   bar_fullbmn = bars + 144, bar_pfree = bars + 160,
                   bar_smready2 = bars + 176, bar_smfree = bars + 184, bar_tfull = bars + 192,
                   bar_tfree = bars + 208, bar_so_full = bars + 272, bar_so_empty = bars + 304;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- work item ---------------------------------------------------------------------------
    const int ntile = p.Dc / DCT;
    int64_t bid = job_block;
    const int tile = (int)(bid % ntile);
    bid /= ntile;
    const int seg = (int)(bid % p.nseg);
    const int64_t bh = bid / p.nseg;
    const int bn = (int)(bh / p.H), bhh = (int)(bh % p.H);
    const int n0 = tile * DCT;
    const int64_t seg_begin = (int64_t)seg * p.seg_len;
    const int64_t seg_end = min(p.L, seg_begin + p.seg_len);
    int nchunk = (int)((seg_end - seg_begin + C - 1) / C);
    const bool skipped = p.state_only && seg >= p.skip_lo && seg < p.skip_hi;
    if (skipped || nchunk < 0) nchunk = 0;
    if (p.state_only && nchunk == 0 && !skipped) {
        // a segment without rows (the tail of a sequence that is not a whole number of
        // segments): its totals are zero, and they are read like any other block.  (Done here,
        // before the roles: at the end of the kernel it kept the block's coordinates alive
        // through every loop and cost the bf16 scan a tenth of its speed.)
        float *dst = p.state_out + ((int64_t)bh * p.nseg + seg) * (p.state_blk ? p.state_blk : (int64_t)DA * p.Dc);
        if (batch.wait_first) asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int e = threadIdx.x; e < DA * DCT; e += NTHREADS)
            dst[(int64_t)(e / DCT) * p.Dc + n0 + e % DCT] = 0.f;
    }

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, apply_only ? 1 : 2);   // released by both issuers
            mbar_init(bar_pfree + 8 * s, 1);
            mbar_init(bar_tfull + 8 * s, 1);
            mbar_init(bar_tfree + 8 * s, 128);
            mbar_init(bar_pfull + 8 * s, 1);
            mbar_init(bar_pready + 8 * s, 128);
            mbar_init(bar_ofull + 8 * s, 1);
            mbar_init(bar_ofree + 8 * s, 128);
            mbar_init(bar_fullc + 8 * s, 1);
            // the 128 threads that rearrange b in place
            mbar_init(bar_fullbmn + 8 * s, 128);
        }
        for (int s = 0; s < K::SO_STAGES; ++s) {
            mbar_init(bar_so_full + 8 * s, 1);
            mbar_init(bar_so_empty + 8 * s, 1);
        }
        mbar_init(bar_sfull, 1);
        mbar_init(bar_smready, 128);
        mbar_init(bar_smready2, 128);
        mbar_init(bar_smfree, 1);
        fence_barrier_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (batch.wait_first) {
        // Nothing above touched global memory.  From here on the grid in front has finished (and,
        // through its own last wait, every grid before it); only now may a grid behind this one
        // start, so that it never runs ahead of a launch that is not this library's.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }

    // The score product reads b K-major (128-byte swizzle: 16-byte chunk c of row r sits at
    // c ^ (r & 7)); the state update reads b MN-major, which for TF32 exists only in the
    // 32-byte-atom swizzle (32-byte unit u of row r at u ^ (r & 3)).  Both keep a tile row in the
    // same 128 bytes, so the second image is a permutation of the 8 chunks of every row, done in
    // place once the score product has retired: a warp instruction covers four whole rows (no
    // bank conflicts), reads them, then writes them back.  `t`: 0..127 within the four warps that
    // share the work.
    auto rearrange_b_in_place = [&](int ci, int t) {
        uint8_t *bt = smem_gen + (ci & 1) * K::STAGE_BYTES + K::A_BYTES;
        constexpr int NIT = K::A_BYTES / (128 * 16);   // 16-byte chunks per thread
        static_assert(NIT % 4 == 0, "chunks are moved four at a time");
        for (int it0 = 0; it0 < NIT; it0 += 4) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int idx = (it0 + j) * 128 + t;   // 16-byte chunk of the tile
                v[j] = reinterpret_cast<const uint4 *>(bt + (size_t)(idx >> 3) * 128)[idx & 7];
            }
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int idx = (it0 + j) * 128 + t;
                const int pk = idx & 7, row = (idx >> 3) & 127;
                const int c = pk ^ (row & 7);          // logical chunk held here
                const int pm = ((((c >> 1) ^ (row & 3)) << 1) | (c & 1));
                reinterpret_cast<uint4 *>(bt + (size_t)(idx >> 3) * 128)[pm] = v[j];
            }
            __syncwarp();
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_fullbmn + 8 * (ci & 1));
    };

    if (nchunk > 0) {
        if (warp == 0) {
            // ================= TMA producer =====================================================
            // bar_full[s]  : a and the K-major image of b have landed (score product, a S)
            // bar_fullc[s] : c has landed (mask(P) c, state update)
            // bar_fullbmn[s]: the MN-major image of b is in b's slot (state update): rearranged in
            //                place by the mask workers (scan), or loaded as such (state only)
            if (elect_one()) {
                // State-only launches: an L2 prefetch ahead of the loads into shared memory
                // (measured: ~8 % faster there; the scan, which already keeps HBM busy, runs
                // 3 % / 10 % SLOWER with its tiles prefetched one / two chunks ahead of the ring).
                auto prefetch_chunk = [&](int ci) {
                    if (ci >= nchunk) return;
                    const int c = p.reverse ? nchunk - 1 - ci : ci;
                    const int row = (int)(seg_begin + (int64_t)c * C);
#pragma unroll
                    for (int b = 0; b < K::A_BLKS; ++b)
                        tma_prefetch_4d(&map_b, b * K::EPB, p.pos_b, row, bhh, bn);
#pragma unroll
                    for (int b = 0; b < K::C_BLKS; ++b)
                        tma_prefetch_4d(&map_c, n0 + b * K::EPB, p.pos_c, row, bhh, bn);
                };
                // One tile = `nblk` boxes of 128 bytes x C rows.  (Shorter boxes, so that the
                // pieces of a row are requested closer together, were measured: 64 rows -2 %,
                // 32 rows -6 %, 8 rows -54 %.)
                auto load_tile = [&](uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0,
                                     const int *pos, int row, int nblk) {
                    for (int b = 0; b < nblk; ++b)
                        tma_load_4d(dst + b * K::BLK_BYTES, map, bar, c0 + b * K::EPB, pos, row, bhh, bn);
                };
                bool ok = true;
                if (p.state_only) {
                    // b and c only: the ring is cut into SO_STAGES slots of b | c (the a slots are
                    // not needed), so one more chunk is in flight -- these launches wait for
                    // loads and for little else
                    for (int ci = 0; ci < nchunk && ok; ++ci) {
                        const int c = p.reverse ? nchunk - 1 - ci : ci;
                        const int s = ci % K::SO_STAGES, use = ci / K::SO_STAGES;
                        ok = mbar_wait(bar_so_empty + 8 * s, (use & 1) ^ 1, abort_flag);
                        if (!ok) break;
                        const int row = (int)(seg_begin + (int64_t)c * C);
                        const uint32_t st = stage0 + s * K::SO_BYTES;
                        mbar_expect_tx(bar_so_full + 8 * s, K::A_BYTES + K::C_BYTES);
                        load_tile(st, &map_bmn, bar_so_full + 8 * s, 0, p.pos_b, row, K::A_BLKS);
                        load_tile(st + K::A_BYTES, &map_c, bar_so_full + 8 * s, n0, p.pos_c, row, K::C_BLKS);
                        prefetch_chunk(ci + K::SO_STAGES);
                    }
                }
                for (int ci = 0; ci < nchunk && ok && !p.state_only; ++ci) {
                    const int c = p.reverse ? nchunk - 1 - ci : ci;
                    const int s = ci & 1, use = ci >> 1;
                    ok = mbar_wait(bar_empty + 8 * s, (use & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    const int row = (int)(seg_begin + (int64_t)c * C);
                    const uint32_t st = stage0 + s * K::STAGE_BYTES;
                    if constexpr (apply_only) {
                        mbar_expect_tx(bar_full + 8 * s, K::A_BYTES);
                        load_tile(st, &map_a, bar_full + 8 * s, 0, p.pos_a, row, K::A_BLKS);
                        continue;
                    }
                    mbar_expect_tx(bar_full + 8 * s, 2 * K::A_BYTES);
                    load_tile(st, &map_a, bar_full + 8 * s, 0, p.pos_a, row, K::A_BLKS);
                    load_tile(st + K::A_BYTES, &map_b, bar_full + 8 * s, 0, p.pos_b, row, K::A_BLKS);
                    mbar_expect_tx(bar_fullc + 8 * s, K::C_BYTES);
                    load_tile(st + 2 * K::A_BYTES, &map_c, bar_fullc + 8 * s, n0, p.pos_c, row, K::C_BLKS);
                }
            }
        } else if (warp == 1 || warp == 10) {
            // ================= MMA issuers ======================================================
            // Two single-thread issuers, because a TF32 MMA covers only K = 8 and one thread
            // issuing all ~48 MMAs of a chunk is the pacing resource:
            //   warp 1  ("output" issuer): O = a S ; O += mask(P) c
            //   warp 10 ("state" issuer) : S += b^T c ; scores of the next chunk
            // They meet only through mbarriers; every barrier below has ONE waiting thread.
            if (elect_one()) {
                constexpr uint32_t ID_P = instr_desc(K::FMT, 0, 0, 128, 128);
                constexpr uint32_t ID_AS = instr_desc(K::FMT, 0, 1, 128, DCT);
                constexpr uint32_t ID_PC = instr_desc(K::FMT, 0, 1, 128, DCT);
                constexpr uint32_t ID_ST = instr_desc(K::FMT, 1, 1, DA, DCT);
                constexpr int KSTEP_BYTES = K::KROWS * 128;   // MN-major advance along K
                const uint32_t tS = tmem + K::TM_S;
                bool ok = true;
                // Descriptors are built once; each MMA then only adds a constant (the
                // start-address field counts 16-byte units and cannot carry into the next field).
                const uint64_t dAk0 = smem_desc(stage0, 16, 1024);
                const uint64_t dBk0 = smem_desc(stage0 + K::A_BYTES, 16, 1024);
                const uint64_t dBmn0 = smem_desc(stage0 + K::A_BYTES, K::BLK_BYTES, K::MN_SBO, K::MN_LAYOUT);
                const uint64_t dCmn0 = smem_desc(stage0 + 2 * K::A_BYTES, K::BLK_BYTES, K::MN_SBO, K::MN_LAYOUT);
                constexpr uint64_t STAGE_UNITS = (uint64_t)(K::STAGE_BYTES >> 4);
                const uint64_t dSm = smem_desc(sm_state, K::SM_BLK_BYTES, K::MN_SBO, K::MN_LAYOUT);

                if (p.state_only) {
                    if (warp == 1) {
                        const uint64_t dSOb = smem_desc(stage0, K::BLK_BYTES, K::MN_SBO, K::MN_LAYOUT);
                        const uint64_t dSOc = smem_desc(stage0 + K::A_BYTES, K::BLK_BYTES, K::MN_SBO, K::MN_LAYOUT);
                        constexpr uint64_t SO_UNITS = (uint64_t)(K::SO_BYTES >> 4);
                        for (int ci = 0; ci < nchunk && ok; ++ci) {
                            const int s = ci % K::SO_STAGES, use = ci / K::SO_STAGES;
                            ok = mbar_wait(bar_so_full + 8 * s, use & 1, abort_flag);
                            if (!ok) break;
                            tc_fence_after();
                            const uint64_t b0 = dSOb + s * SO_UNITS, c0 = dSOc + s * SO_UNITS;
#pragma unroll
                            for (int k = 0; k < C / K::KROWS; ++k) {
                                const uint64_t off = (uint64_t)((k * KSTEP_BYTES) >> 4);
                                mma_ss<K::F16>(tS, b0 + off, c0 + off, ID_ST, (ci | k) ? 1u : 0u);
                            }
                            tc_commit(bar_so_empty + 8 * s);
                        }
                        tc_commit(bar_sfull);
                    }
                } else if (warp == 1) {
                    // ---- output issuer -------------------------------------------------------
                    for (int ci = 0; ci < nchunk && ok; ++ci) {
                        const int s = ci & 1;
                        const uint64_t a0 = dAk0 + s * STAGE_UNITS, c0 = dCmn0 + s * STAGE_UNITS;
                        const int ob = ci % K::NOBUF, ouse = ci / K::NOBUF;
                        const uint32_t tO = tmem + K::TM_O + ob * DCT;
                        const uint32_t tP = tmem + K::TM_P + 128 * (ci & 1);
                        // O = a S: the a tile, the operand copy of the previous state, a free O
                        // (apply only: the state operand is written once, before the first chunk)
                        ok = mbar_wait(bar_full + 8 * s, (ci >> 1) & 1, abort_flag) &&
                             ((apply_only && ci > 0) || mbar_wait(bar_smready, ci & 1, abort_flag)) &&
                             mbar_wait(bar_ofree + 8 * ob, (ouse & 1) ^ 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        uint32_t acc = 0;
#pragma unroll
                        for (int b = 0; b < K::A_BLKS; ++b)
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const int krow = (b * K::EPB + k * K::KROWS);   // first state row
                                mma_ss<K::F16>(tO, a0 + (uint64_t)((b * K::BLK_BYTES + k * 32) >> 4),
                                               dSm + (uint64_t)((krow * 128) >> 4), ID_AS, acc);
                                acc = 1;
                            }
                        if constexpr (apply_only) {
                            tc_commit(bar_ofull + 8 * ob);   // output workers
                            tc_commit(bar_empty + 8 * s);    // the only release of the stage
                            continue;
                        }
                        // the state operand in shared memory may now be replaced by the next state
                        tc_commit(bar_smfree);
                        // O += mask(P) c
                        ok = mbar_wait(bar_pready + 8 * (ci & 1), (ci >> 1) & 1, abort_flag) &&
                             mbar_wait(bar_fullc + 8 * s, (ci >> 1) & 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int k = 0; k < C / K::KROWS; ++k) {
                            mma_ts<K::F16>(tO, tP + k * 8, c0 + (uint64_t)((k * KSTEP_BYTES) >> 4), ID_PC, acc);
                            acc = 1;
                        }
                        tc_commit(bar_ofull + 8 * ob);       // output workers
                        tc_commit(bar_pfree + 8 * (ci & 1)); // this score buffer may be overwritten
                        tc_commit(bar_empty + 8 * s);        // one of the two releases of the stage
                    }
                } else if (!apply_only) {
                    // ---- state issuer --------------------------------------------------------
                    auto issue_scores = [&](int ci) {
                        const int s = ci & 1;
                        const uint32_t tP = tmem + K::TM_P + 128 * (ci & 1);
                        const uint64_t a0 = dAk0 + s * STAGE_UNITS, b0 = dBk0 + s * STAGE_UNITS;
#pragma unroll
                        for (int b = 0; b < K::A_BLKS; ++b)
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const uint64_t off = (uint64_t)((b * K::BLK_BYTES + k * 32) >> 4);
                                mma_ss<K::F16>(tP, a0 + off, b0 + off, ID_P, (b | k) ? 1u : 0u);
                            }
                        tc_commit(bar_pfull + 8 * (ci & 1));
                    };
                    // Two job queues, served in whichever order their inputs arrive: the score
                    // product of chunk `sc` (a, K-major b, a free score buffer) and the state
                    // increment of chunk `ds` (c, MN-major b, a free accumulator).  The score
                    // product of chunk ds+1 must not sit behind the increment of chunk ds: the
                    // mask, the MN-major image of b and mask(P) c of chunk ds+1 all start from it.
                    int sc = 0, ds = 0;
                    long long t0 = 0;
                    uint32_t idle = 0;
                    while (ds < nchunk) {
                        if (sc < nchunk && sc <= ds + 1 &&
                            mbar_test(bar_full + 8 * (sc & 1), (sc >> 1) & 1) &&
                            (sc < 2 || mbar_test(bar_pfree + 8 * (sc & 1), ((sc - 2) >> 1) & 1))) {
                            tc_fence_after();
                            issue_scores(sc);
                            ++sc;
                            idle = 0;
                            continue;
                        }
                        const int s = ds & 1;
                        // fresh accumulator (REG_STATE): free once the increment of chunk ds-2 has
                        // been read out of it; in-place accumulation: the state workers must have
                        // finished reading the accumulator of the previous chunk
                        const bool acc_free =
                            K::REG_STATE ? mbar_test(bar_tfree + 8 * s, ((ds >> 1) & 1) ^ 1)
                                         : mbar_test(bar_smready2, ds & 1);
                        // (ds < sc: the score product of this chunk has been issued, so b has landed)
                        if (ds < sc && acc_free && mbar_test(bar_fullc + 8 * s, (ds >> 1) & 1) &&
                            (!K::RELOAD_B || mbar_test(bar_fullbmn + 8 * s, (ds >> 1) & 1))) {
                            const uint64_t bmn0 = dBmn0 + s * STAGE_UNITS, c0 = dCmn0 + s * STAGE_UNITS;
                            tc_fence_after();
                            const uint32_t tT = K::REG_STATE ? tS + s * DCT : tS;
#pragma unroll
                            for (int k = 0; k < C / K::KROWS; ++k) {
                                const uint64_t off = (uint64_t)((k * KSTEP_BYTES) >> 4);
                                mma_ss<K::F16>(tT, bmn0 + off, c0 + off, ID_ST, (K::REG_STATE && k == 0) ? 0u : 1u);
                            }
                            if constexpr (K::REG_STATE) tc_commit(bar_tfull + 8 * s);
                            else tc_commit(bar_sfull);
                            tc_commit(bar_empty + 8 * s);        // the other release of the stage
                            ++ds;
                            idle = 0;
                            continue;
                        }
                        // nothing ready: bounded polling, as in mbar_wait
                        if (idle++ == 0) t0 = clock64();
                        if ((idle & 63u) == 0u) {
                            if (*abort_flag) break;
                            if (clock64() - t0 > 4000000000LL) {
                                *abort_flag = 1;
                                atomicExch(&g_device_status, 5 /* FTB_ERR_TIMEOUT */);
                                break;
                            }
                        }
                    }
                }
            }
        } else if (warp >= 11) {
            // ================= mask workers: causal mask on the scores, in place ================
            // (warps 11-14 cover the four 32-lane quarters of tensor memory: q = 3, 0, 1, 2)
            if (!p.state_only && !apply_only) {
                const int q = warp & 3;
                const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
                uint32_t r[32];
                for (int ci = 0; ci < nchunk; ++ci) {
                    if (!mbar_wait(bar_pfull + 8 * (ci & 1), (ci >> 1) & 1, abort_flag)) break;
                    tc_fence_after();
                    const uint32_t tP = tlane + K::TM_P + 128 * (ci & 1);
                    // Rows of this warp are 32q..32q+31.  Column blocks of 32: those on one side of
                    // the diagonal are kept as they are, those on the other side are dropped
                    // (zeroed), the diagonal block is masked element by element.
                    const int nkeep = p.reverse ? 3 - q : q;      // whole blocks kept
                    const int ndrop = 3 - nkeep;                  // whole blocks dropped
                    if constexpr (!K::F16) {
                        // TF32: the product reads the fp32 scores in place.  The dropped columns
                        // are one range: zero them with the widest stores first (they do not
                        // depend on the load below and overlap its latency), then the diagonal.
                        tmem_zero_columns(tP + (p.reverse ? 0 : 32 * (q + 1)), 32 * ndrop);
                        tmem_ld32(tP + 32 * q, r);
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const bool keep = p.reverse ? (e >= lane) : (e <= lane);
                            r[e] = keep ? r[e] : 0u;
                        }
                        tmem_st32(tP + 32 * q, r);
                    } else {
                        // bf16: every kept block is rounded and packed in place (block cb: fp32
                        // columns 32cb.., packed columns 16cb..), blocks in ascending order so that
                        // a packed block never lands on scores that are still to be read; two
                        // blocks per load where there are two.  The dropped range is zeroed last
                        // (its packed columns overlap fp32 scores of kept blocks).
                        auto pack = [&](const uint32_t *src, uint32_t *dst, bool diag) {
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                float x0 = __uint_as_float(src[2 * e]), x1 = __uint_as_float(src[2 * e + 1]);
                                if (diag) {
                                    const bool k0 = p.reverse ? (2 * e >= lane) : (2 * e <= lane);
                                    const bool k1 = p.reverse ? (2 * e + 1 >= lane) : (2 * e + 1 <= lane);
                                    x0 = k0 ? x0 : 0.f;
                                    x1 = k1 ? x1 : 0.f;
                                }
                                __nv_bfloat162 hh = __floats2bfloat162_rn(x0, x1);
                                dst[e] = *reinterpret_cast<uint32_t *>(&hh);
                            }
                        };
                        const int kb0 = p.reverse ? q : 0, kb1 = p.reverse ? 3 : q;   // kept blocks, diagonal included
                        int cb = kb0;
                        for (; cb + 1 <= kb1; cb += 2) {
                            uint32_t w[64], h2[32];
                            tmem_ld64(tP + 32 * cb, w);
                            pack(w, h2, cb == q);
                            pack(w + 32, h2 + 16, cb + 1 == q);
                            tmem_st32(tP + 16 * cb, h2);
                        }
                        if (cb <= kb1) {
                            uint32_t h[16];
                            tmem_ld32(tP + 32 * cb, r);
                            pack(r, h, cb == q);
                            tmem_st16(tP + 16 * cb, h);
                        }
                        tmem_zero_columns(tP + (p.reverse ? 0 : 16 * (q + 1)), 16 * ndrop);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(bar_pready + 8 * (ci & 1));
                }
            }
        } else if (warp >= 6 && warp < 10) {
            // ================= output workers: O rows -> global memory ==========================
            if (!p.state_only) {
                const int q = warp & 3;
                const int i = 32 * q + lane;
                const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
                uint32_t r[32];
                bool ok = true;
                T *O = reinterpret_cast<T *>(p.out) + (int64_t)bn * p.so.n + (int64_t)bhh * p.so.h;
                const float *DEN = p.row_den ? p.row_den + (int64_t)bn * p.sden.n + (int64_t)bhh * p.sden.h : nullptr;
                // 1 / (row_den + eps) of a row (1 without a normaliser or past the segment)
                auto row_scale = [&](int64_t row) {
                    return (DEN && row < seg_end) ? 1.f / (DEN[row * p.sden.l] + p.eps) : 1.f;
                };
                for (int ci = 0; ci < nchunk && ok; ++ci) {
                    const int c = p.reverse ? nchunk - 1 - ci : ci;
                    const int64_t row0 = seg_begin + (int64_t)c * C;
                    const int ob = ci % K::NOBUF, ouse = ci / K::NOBUF;
                    if constexpr (K::RELOAD_B && !apply_only) {
                        // these warps are idle between two stores: they make the MN-major image
                        // of b while the mask workers mask the scores
                        ok = mbar_wait(bar_pfull + 8 * (ci & 1), (ci >> 1) & 1, abort_flag);
                        if (!ok) break;
                        rearrange_b_in_place(ci, threadIdx.x - 192);
                    }
                    // (the row scales are fetched before the wait for the accumulator)
                    float zs[(!K::F16 && DCT == 64) ? 4 : 1];
                    if constexpr (!K::F16 && DCT == 64) {
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            const int64_t ra = row0 + 32 * q + 16 * hf + (lane >> 2);
                            zs[2 * hf] = row_scale(ra);
                            zs[2 * hf + 1] = row_scale(ra + 8);
                        }
                    } else {
                        zs[0] = row_scale(row0 + i);
                    }
                    ok = mbar_wait(bar_ofull + 8 * ob, ouse & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    if constexpr (!K::F16 && DCT == 64) {
                        // fp32 rows: read the accumulator in the 16x256b shape (a thread gets
                        // column pairs of rows lane/4 and lane/4 + 8), so that one warp store
                        // writes 8 rows x 32 B -- whole sectors -- instead of 32 rows x 16 B
                        // (measured: ~6 % off the launch time)
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            tmem_ld16x256(tlane + ((uint32_t)(16 * hf) << 16) + K::TM_O + ob * DCT, r);
                            const int64_t ra = row0 + 32 * q + 16 * hf + (lane >> 2);
                            T *da = O + ra * p.so.l + n0 + 2 * (lane & 3);
                            T *db = da + 8 * p.so.l;
                            if (DEN) {
#pragma unroll
                                for (int e = 0; e < 32; ++e)
                                    r[e] = __float_as_uint(__uint_as_float(r[e]) * zs[2 * hf + ((e >> 1) & 1)]);
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                if (ra < seg_end)
                                    *reinterpret_cast<uint2 *>(da + 8 * j) = make_uint2(r[4 * j], r[4 * j + 1]);
                                if (ra + 8 < seg_end)
                                    *reinterpret_cast<uint2 *>(db + 8 * j) = make_uint2(r[4 * j + 2], r[4 * j + 3]);
                            }
                        }
                    } else {
                    const int64_t row = row0 + i;
                    T *dst = O + row * p.so.l + n0;
#pragma unroll
                    for (int cb = 0; cb < DCT / 32; ++cb) {
                        tmem_ld32(tlane + K::TM_O + ob * DCT + 32 * cb, r);
                        if (DEN) {
#pragma unroll
                            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * zs[0]);
                        }
                        if (row < seg_end) {
                            if constexpr (K::F16) {
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    uint4 v;
                                    __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r[8 * e + 0]), __uint_as_float(r[8 * e + 1]));
                                    __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r[8 * e + 2]), __uint_as_float(r[8 * e + 3]));
                                    __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[8 * e + 4]), __uint_as_float(r[8 * e + 5]));
                                    __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(r[8 * e + 6]), __uint_as_float(r[8 * e + 7]));
                                    v.x = *reinterpret_cast<uint32_t *>(&h0);
                                    v.y = *reinterpret_cast<uint32_t *>(&h1);
                                    v.z = *reinterpret_cast<uint32_t *>(&h2);
                                    v.w = *reinterpret_cast<uint32_t *>(&h3);
                                    *reinterpret_cast<uint4 *>(dst + 32 * cb + 8 * e) = v;
                                }
                            } else {
#pragma unroll
                                for (int e = 0; e < 8; ++e)
                                    *reinterpret_cast<uint4 *>(dst + 32 * cb + 4 * e) =
                                        make_uint4(r[4 * e], r[4 * e + 1], r[4 * e + 2], r[4 * e + 3]);
                            }
                        }
                    }
                    }
                    tc_fence_before();
                    mbar_arrive(bar_ofree + 8 * ob);
                }
            }
        } else if (warp >= 2 && warp < 6) {
            // ================= state workers: one TMEM lane (state row) per thread ===============
            const int q = warp & 3;
            const int i = 32 * q + lane;                       // row inside the chunk / lane
            const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
            // state row handled by this thread (DA == 64: 16 lanes per sub-partition hold rows)
            const bool srow_ok = (DA == 128) || (lane < 16);
            const int srow = (DA == 128) ? i : (16 * q + (lane & 15));
            uint32_t r[32];
            bool ok = true;
            float stv[K::REG_STATE ? DCT : 1];   // REG_STATE: this thread's state row, fp32

            auto store_state_operand = [&](int cb) {
                // r[] holds state row `srow`, columns 32*cb .. 32*cb+31 (fp32 bits)
                if (!srow_ok) return;
                if constexpr (K::F16) {
                    uint8_t *rowp = sm_state_gen + (cb >> 1) * K::SM_BLK_BYTES + srow * 128;
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        uint4 v;
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r[8 * ch + 0]), __uint_as_float(r[8 * ch + 1]));
                        __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
                        __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
                        v.x = *reinterpret_cast<uint32_t *>(&h0);
                        v.y = *reinterpret_cast<uint32_t *>(&h1);
                        v.z = *reinterpret_cast<uint32_t *>(&h2);
                        v.w = *reinterpret_cast<uint32_t *>(&h3);
                        const int chunk16 = ((cb & 1) * 4 + ch) ^ (srow & 7);
                        *reinterpret_cast<uint4 *>(rowp + chunk16 * 16) = v;
                    }
                } else {
                    uint8_t *rowp = sm_state_gen + cb * K::SM_BLK_BYTES + srow * 128;
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        uint4 v = make_uint4(r[4 * ch], r[4 * ch + 1], r[4 * ch + 2], r[4 * ch + 3]);
                        *reinterpret_cast<uint4 *>(rowp + (((ch >> 1) ^ (srow & 3)) * 32) + (ch & 1) * 16) = v;
                    }
                }
            };

            if (p.state_only) {
                ok = mbar_wait(bar_sfull, 0, abort_flag);
                if (ok) {
                    tc_fence_after();
                    float *dst = p.state_out + ((int64_t)bh * p.nseg + seg) * (p.state_blk ? p.state_blk : (int64_t)DA * p.Dc);
#pragma unroll
                    for (int cb = 0; cb < DCT / 32; ++cb) {
                        tmem_ld32(tlane + K::TM_S + 32 * cb, r);
                        if (srow_ok) {
                            float4 *d4 = reinterpret_cast<float4 *>(dst + (int64_t)srow * p.Dc + n0 + 32 * cb);
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                d4[e] = make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]),
                                                    __uint_as_float(r[4 * e + 2]), __uint_as_float(r[4 * e + 3]));
                        }
                    }
                }
            } else {
                // ---- initial state -> TMEM accumulator and shared-memory operand ---------------
                {
                    const int64_t blk = p.state_blk ? p.state_blk : (int64_t)DA * p.Dc;
                    // blocks to add up: the per-bh initial state and either this segment's own
                    // block or the raw totals of every segment before (after) it
                    int s_lo = seg, s_hi = seg + 1, per_head = p.nseg;
                    if (p.sum_mode) {
                        per_head = p.nseg * p.sub;
                        s_lo = p.reverse ? (seg + 1) * p.sub : 0;
                        s_hi = p.reverse ? per_head : seg * p.sub;
                    }
                    if (!p.states) s_hi = s_lo;
                    // Programmatic dependent launch: this grid may have been started before the
                    // launch in front of it (the state-only sweep that writes these totals) has
                    // finished -- its tiles, scores and masks do not depend on it.  The totals do:
                    // wait for that grid here (returns at once after an ordinary launch).
                    if (s_hi > s_lo) asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
                    for (int cb = 0; cb < DCT / 32; ++cb) {
                        float acc[32];
#pragma unroll
                        for (int e = 0; e < 32; ++e) acc[e] = 0.f;
                        if (srow_ok) {
                            for (int sb = s_lo - 1; sb < s_hi; ++sb) {
                                const float *src;
                                if (sb < s_lo) {
                                    if (!p.init) continue;
                                    src = p.init + (int64_t)bh * blk;
                                } else {
                                    src = p.states + ((int64_t)bh * per_head + sb) * blk;
                                }
                                const int dc0 = n0 + 32 * cb;
                                if (p.canon_is_DaDc) {
                                    const float4 *s4 = reinterpret_cast<const float4 *>(src + (int64_t)srow * p.Dc + dc0);
#pragma unroll
                                    for (int e = 0; e < 8; ++e) {
                                        float4 v = s4[e];
                                        acc[4 * e] += v.x; acc[4 * e + 1] += v.y;
                                        acc[4 * e + 2] += v.z; acc[4 * e + 3] += v.w;
                                    }
                                } else {
#pragma unroll
                                    for (int e = 0; e < 32; ++e) acc[e] += src[(int64_t)(dc0 + e) * DA + srow];
                                }
                            }
                        }
#pragma unroll
                        for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(acc[e]);
                        if constexpr (K::REG_STATE) {
#pragma unroll
                            for (int e = 0; e < 32; ++e) stv[32 * cb + e] = acc[e];
                        } else {
                            tmem_st32(tlane + K::TM_S + 32 * cb, r);
                        }
                        store_state_operand(cb);
                    }
                    if constexpr (!K::REG_STATE) tmem_wait_st();
                    fence_proxy_async_smem();
                    tc_fence_before();
                    mbar_arrive(bar_smready);
                    mbar_arrive(bar_smready2);
                }

                for (int ci = 0; ci + 1 < nchunk && ok && !apply_only; ++ci) {
                    // ---- updated state -> shared-memory operand of the next chunk ---------------
                    // the new state is complete, and "a S" of this chunk has finished reading the
                    // old operand copy (which also keeps the two issuers within one chunk of each
                    // other, as the parity waits require)
                    if constexpr (K::REG_STATE) {
                        // the increment is added to the register copy before the wait for the
                        // operand slot: its accumulator is handed back at once
                        ok = mbar_wait(bar_tfull + 8 * (ci & 1), (ci >> 1) & 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int cb = 0; cb < DCT / 32; ++cb) {
                            tmem_ld32(tlane + K::TM_S + (ci & 1) * DCT + 32 * cb, r);
#pragma unroll
                            for (int e = 0; e < 32; ++e) stv[32 * cb + e] += __uint_as_float(r[e]);
                        }
                        tc_fence_before();
                        mbar_arrive(bar_tfree + 8 * (ci & 1));
                        ok = mbar_wait(bar_smfree, ci & 1, abort_flag);
                        if (!ok) break;
#pragma unroll
                        for (int cb = 0; cb < DCT / 32; ++cb) {
#pragma unroll
                            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(stv[32 * cb + e]);
                            store_state_operand(cb);
                        }
                    } else {
                        ok = mbar_wait(bar_sfull, ci & 1, abort_flag);
                        if (ok) ok = mbar_wait(bar_smfree, ci & 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int cb = 0; cb < DCT / 32; ++cb) {
                            tmem_ld32(tlane + K::TM_S + 32 * cb, r);
                            store_state_operand(cb);
                        }
                    }
                    fence_proxy_async_smem();
                    tc_fence_before();
                    mbar_arrive(bar_smready);
                    mbar_arrive(bar_smready2);
                }
            }
        }
    }

    // ---- teardown: everyone meets here, tensor memory is returned ------------------------------
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 512);
    // no block of a programmatically launched grid ends before the grid in front of it has, so
    // that whatever is launched behind this grid is ordered after both
    if (threadIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace mma
}  // namespace ftb
