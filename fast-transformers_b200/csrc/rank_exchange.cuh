// Exchange of per-rank states between the GPUs of one node, without a library collective.
//
// A sequence split over P ranks needs, once per direction, the sum of the (N,H,D,M) fp32 totals
// of the ranks before (forward) or after (backward) each rank.  Here every rank owns one device
// buffer that its peers map through CUDA IPC:
//
//   [control block, 512 B, written by the owner only]
//       u64 [0]  exchanges pushed by the owner
//       u64 [1]  exchanges received by the owner (the peers read it before they reuse a slot)
//       u32 at byte 64 + 4 p   blocks that finished the push to rank p
//       u32 at byte 128        ranks the current push has finished with
//       u32 at byte 132        blocks that finished the current receive
//   [flags: 2 x P u64]         flag[parity][src] = number of the last exchange src has delivered
//   [slots: 2 x P x elems f32] slot[parity][src] = the state src delivered in that exchange
//
// push_kernel (rank r) stores its state (given whole, or as partial sums that it adds up on the
// way) into slot[e & 1][r] of every rank that needs it -- peer stores over NVLink -- and then releases flag[e & 1][r] = e at system scope; receive_kernel waits
// (bounded) until the flags of the ranks it needs have reached e and adds their slots up in rank
// order.  e comes from counters in the owner's control block, advanced by the kernels themselves,
// so the pair can be captured in a CUDA graph and replayed.  There are two slots per source,
// alternating with e, so a rank may deliver exchange e + 1 before a peer has read exchange e;
// before it overwrites a slot with exchange e, push_kernel checks that the target has finished
// its receive of e - 2 (the target's "received" counter, read through the mapping).  In a
// training step, where directions alternate, that is already true (a rank cannot get two
// exchanges ahead of a peer it also receives from); in a run of forward-only exchanges the first
// rank receives from nobody and would otherwise run away.
//
// No kernel here waits on another launch of the same GPU; the waits are on counters written by
// OTHER GPUs.  They give up after `wait_ns` nanoseconds of the global timer (a second by default,
// see ftb_exchange_wait_limit_ms), record FTB_ERR_TIMEOUT in the device status word, and a
// receive that gave up fills its result with NaN so that the failure cannot pass for data.
// Dependencies point from an exchange to the same or an earlier one only (receive e needs the
// peers' push e; push e needs the peers' receive e - 2), so the waits cannot form a cycle.
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_runtime.h>

namespace ftb {
namespace xchg {

constexpr int kMaxRanks = 16;
constexpr int kThreads = 256;
constexpr size_t kCtlBytes = 512;
constexpr long long kDefaultWaitNs = 1000000000LL;   // one second

struct Layout {
    size_t flags_off, slots_off, bytes;
};
__host__ __device__ inline Layout layout(int world, int64_t elems) {
    Layout l;
    l.flags_off = kCtlBytes;
    l.slots_off = kCtlBytes + (((size_t)2 * world * 8 + 255) / 256) * 256;
    l.bytes = l.slots_off + (size_t)2 * world * (size_t)elems * 4;
    return l;
}

struct Peers {
    void *buf[kMaxRanks];   // every rank's buffer as mapped on this GPU; [rank] is the own one
};

__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Poll *p (system scope) until it reaches `want`; false once `wait_ns` have passed.  The spin count
// is bounded as well, in case the timer does not advance.
__device__ __forceinline__ bool wait_reaches(const unsigned long long *p, unsigned long long want,
                                             long long wait_ns, unsigned long long add = 0) {
    if (ld_acquire_sys(p) + add >= want) return true;
    const long long t0 = global_ns();
    for (long long spins = 0; spins < 200000000LL; ++spins) {
        if (ld_acquire_sys(p) + add >= want) return true;
        if ((spins & 15) == 15 && global_ns() - t0 > wait_ns) return false;
        __nanosleep(200);
    }
    return false;
}

// grid (blocks per target, targets); targets = the ranks after this one (before it when reverse).
// A rank without targets launches one block, which only advances the counter.
__global__ void __launch_bounds__(kThreads)
push_kernel(const float *__restrict__ state, int64_t elems, int64_t unit_elems, int parts_per_unit,
            Peers peers, int rank, int world, int reverse, int *device_status, long long wait_ns) {
    char *own = static_cast<char *>(peers.buf[rank]);
    volatile unsigned long long *ctl = reinterpret_cast<volatile unsigned long long *>(own);
    const unsigned long long epoch = ctl[0] + 1;   // no block writes ctl[0] before all have read it
    const int ntargets = reverse ? rank : world - 1 - rank;
    if (ntargets == 0) {
        if (threadIdx.x == 0) ctl[0] = epoch;
        return;
    }
    const int p = reverse ? (int)blockIdx.y : rank + 1 + (int)blockIdx.y;
    const Layout l = layout(world, elems);
    const int parity = (int)(epoch & 1);
    char *peer = static_cast<char *>(peers.buf[p]);
    float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(peer + l.slots_off) +
                                             ((int64_t)parity * world + rank) * elems);
    const float4 *src = reinterpret_cast<const float4 *>(state);
    const int64_t n4 = elems / 4;
    // the slot still holds exchange e - 2 until the target has received it
    __shared__ int s_fail;
    if (threadIdx.x == 0) {
        const unsigned long long *received = reinterpret_cast<const unsigned long long *>(peer) + 1;
        const int fail = wait_reaches(received, epoch, wait_ns, 2) ? 0 : 1;
        if (fail) atomicExch(device_status, 5 /* FTB_ERR_TIMEOUT */);
        s_fail = fail;
    }
    __syncthreads();
    const bool deliver = !s_fail;
    if (deliver && parts_per_unit <= 1) {
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += (int64_t)gridDim.x * kThreads)
            dst[i] = src[i];
    } else if (deliver) {
        // the state arrives as `parts_per_unit` partial sums per unit of `unit_elems` floats (the
        // per-segment totals of one (batch, head) pair): they are added up on the way, in a fixed order
        const int64_t u4 = unit_elems / 4;
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += (int64_t)gridDim.x * kThreads) {
            const int64_t unit = i / u4, e = i - unit * u4;
            const float4 *part = src + unit * parts_per_unit * u4 + e;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < parts_per_unit; ++k) {
                const float4 v = part[(int64_t)k * u4];
                acc.x += v.x;
                acc.y += v.y;
                acc.z += v.z;
                acc.w += v.w;
            }
            dst[i] = acc;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned *blocks_done = reinterpret_cast<unsigned *>(own + 64) + p;
        unsigned *targets_done = reinterpret_cast<unsigned *>(own + 128);
        // low half: blocks done; high half: blocks that gave up waiting
        const unsigned mine = deliver ? 1u : 0x10001u;
        const unsigned before = atomicAdd(blocks_done, mine);
        if ((before & 0xffffu) == gridDim.x - 1) {
            // the last block of this target: every block's stores are fenced; publish them
            // (not after a time-out: the target's receive then times out as well)
            *blocks_done = 0;
            __threadfence_system();
            if (((before + mine) >> 16) == 0)
                st_release_sys(reinterpret_cast<unsigned long long *>(peer + l.flags_off) + parity * world + rank,
                               epoch);
            if (atomicAdd(targets_done, 1u) == gridDim.y - 1) {
                *targets_done = 0;
                ctl[0] = epoch;
            }
        }
    }
}

// out = sum of the states delivered by the ranks before this one (after it when reverse), zeros
// when there are none.  Any number of blocks; each waits for the flags itself.
__global__ void __launch_bounds__(kThreads)
receive_kernel(void *own_buf, float *__restrict__ out, int64_t elems, int rank, int world, int reverse,
               int *device_status, long long wait_ns) {
    char *own = static_cast<char *>(own_buf);
    volatile unsigned long long *ctl = reinterpret_cast<volatile unsigned long long *>(own);
    const unsigned long long epoch = ctl[1] + 1;
    const int parity = (int)(epoch & 1);
    const Layout l = layout(world, elems);
    const int lo = reverse ? rank + 1 : 0, hi = reverse ? world : rank;
    __shared__ int s_fail;
    if (threadIdx.x == 0) {
        int fail = 0;
        const unsigned long long *flags =
            reinterpret_cast<const unsigned long long *>(own + l.flags_off) + parity * world;
        for (int p = lo; p < hi && !fail; ++p)
            if (!wait_reaches(flags + p, epoch, wait_ns)) fail = 1;
        if (fail) atomicExch(device_status, 5 /* FTB_ERR_TIMEOUT */);
        s_fail = fail;
    }
    __syncthreads();
    if (s_fail) {
        // gave up: the result must not pass for data
        float4 *out4 = reinterpret_cast<float4 *>(out);
        const float nan = __int_as_float(0x7fc00000);
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < elems / 4; i += (int64_t)gridDim.x * kThreads)
            out4[i] = make_float4(nan, nan, nan, nan);
    } else {
        const float *slots = reinterpret_cast<const float *>(own + l.slots_off) + (int64_t)parity * world * elems;
        float4 *out4 = reinterpret_cast<float4 *>(out);
        const int64_t n4 = elems / 4;
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += (int64_t)gridDim.x * kThreads) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int p = lo; p < hi; ++p) {
                const float4 v = __ldcg(reinterpret_cast<const float4 *>(slots + (int64_t)p * elems) + i);
                acc.x += v.x;
                acc.y += v.y;
                acc.z += v.z;
                acc.w += v.w;
            }
            out4[i] = acc;
        }
    }
    __syncthreads();   // every thread of the block is done with the slots
    if (threadIdx.x == 0) {
        unsigned *blocks_done = reinterpret_cast<unsigned *>(own + 132);
        __threadfence_system();
        if (atomicAdd(blocks_done, 1u) == gridDim.x - 1) {
            // every block has read ctl[1] and the slots by now: the peers may reuse the slots
            *blocks_done = 0;
            __threadfence_system();
            st_release_sys(reinterpret_cast<unsigned long long *>(own) + 1, epoch);
        }
    }
}

}  // namespace xchg
}  // namespace ftb
