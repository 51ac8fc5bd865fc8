// Cross-GPU exchange of one fp32 maximum per rank over peer memory (NVLink / NVSwitch).  No counterpart in the
// reference, which runs on one GPU; it is what stands in for ncclAllReduce(MAX) of the per-shard amax when a
// row-sharded tensor needs a tensor-wide scale.
//
// Every rank owns a small "exchange state" in its own device memory (QCC_XCHG_STATE_BYTES, cleared once):
//
//   word 0   exchanges number of exchanges this rank has published
//   word 2   accum     running maximum of the producing calls since the last exchange (fp32 bits, non-negative)
//   word 3   abort     set when a wait ran out; later waits then return at once
//   word 4   timeout   limit of a wait in microseconds
//   byte 256 slots     uint64 [2][QCC_XCHG_MAX_RANKS]: slot [e & 1][r] = (e << 32) | amax bits of rank r in exchange e
//
// Producer (an amax kernel, or a cast that has every block maximum in registers anyway): each CTA merges its maximum
// into `accum` with one atomic max, skipped when accum already held as much when the CTA started; nothing else, so
// a CTA retires without waiting for an atomic to come back.  The kernel boundary completes the value; several
// producing calls (row chunks of one shard) accumulate.
// Resolve (one warp, a later launch on the stream): reads accum, stores (e << 32) | bits with e = exchanges + 1 into
// slot [e & 1][own rank] of EVERY rank's state (plain 8-byte peer stores over NVLink; value and tag travel in one
// word, so no flag or fence is needed), clears accum, then takes the maximum over the `world` slots of parity e in
// its own rank's memory, waiting (bounded) for tags that have not arrived, and writes the scale the casts read.
// Two slot sets suffice: a rank can publish exchange e + 1 while a slower peer still reads exchange e, but not
// e + 2, because that comes after resolving e + 1, which needs the slower peer's own e + 1.
// All ranks must resolve the same number of times; every resolve is preceded by this rank's producing calls.
// Waits are bounded by the state's timeout and report code QCC_DEVERR_XCHG.
#pragma once
#include "common.cuh"

namespace qcc {

constexpr unsigned int QCC_DEVERR_XCHG = 19u;   // a wait for a peer's amax ran out
constexpr int XCHG_W_EXCHANGES = 0, XCHG_W_ACCUM = 2, XCHG_W_ABORT = 3, XCHG_W_TIMEOUT = 4;
constexpr int XCHG_SLOT_BYTE_OFF = 256;
constexpr int AMAX_MAX_CTAS = 2048;              // partial maxima of the two-launch amax; its one-launch control words follow them

// slots[r] = address, valid on this GPU, of the slot array inside rank r's state
struct XchgPeers {
    unsigned long long *slots[QCC_XCHG_MAX_RANKS];
    int world, rank;
};

__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// The tag and the value travel in one 8-byte word, so neither side needs acquire / release ordering: a relaxed
// system-scope access that bypasses L1 is enough (an acquire at system scope would also drop the SM's L1 contents,
// which the streaming casts rely on between their 16-byte loads).
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long *p, unsigned long long v)
{
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// CTA-wide maximum of `m` merged into ctl[1]; true (for all threads of warp 0) in the CTA that finished last, with
// `m` then holding the kernel-wide maximum and ctl[] cleared.  `s` is shared scratch of blockDim.x / 32 words.
// Contains one __syncthreads(); threads outside warp 0 get false.  (The form for a kernel that must deliver the
// finished value itself; ctl[0] = ticket, ctl[1] = running maximum, both zero between calls.)
__device__ __forceinline__ bool cta_max_ticket(uint32_t &m, uint32_t *__restrict__ ctl, uint32_t *s)
{
    m = __reduce_max_sync(0xFFFFFFFFu, m);
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x >= 32) return false;
    const int nw = blockDim.x >> 5;
    m = (int)threadIdx.x < nw ? s[threadIdx.x] : 0u;
    m = __reduce_max_sync(0xFFFFFFFFu, m);
    uint32_t last = 0;
    if (threadIdx.x == 0) {
        if (m > ld_volatile_u32(ctl + 1)) atomicMax(ctl + 1, m);
        __threadfence();
        last = atomicAdd(ctl, 1u) == gridDim.x - 1 ? 1u : 0u;
        if (last) {
            __threadfence();
            m = atomicExch(ctl + 1, 0u);
            ctl[0] = 0u;
        }
    }
    last = __shfl_sync(0xFFFFFFFFu, last, 0);
    m = __shfl_sync(0xFFFFFFFFu, m, 0);
    return last != 0u;
}

// ---- producer side -------------------------------------------------------------------------------------------
// Call at the top of a producing kernel (all threads): returns, to thread 0 only, what accum held -- a lower bound
// of its final value that lets most CTAs skip their atomic (one L2 request per CTA; the same load from every warp
// makes the word's L2 slice a hot spot and cost 10 % of a streaming cast).
__device__ __forceinline__ uint32_t xchg_producer_begin(uint32_t *state)
{
    return threadIdx.x == 0 ? ld_volatile_u32(state + XCHG_W_ACCUM) : 0u;
}
// Call at the end (all threads; one __syncthreads()): the CTA's maximum of `m` goes into accum unless `seen`, the
// value xchg_producer_begin returned, already covers it.
__device__ __forceinline__ void xchg_producer_merge(uint32_t *state, uint32_t m, uint32_t seen, uint32_t *s)
{
    m = __reduce_max_sync(0xFFFFFFFFu, m);
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        m = (int)threadIdx.x < nw ? s[threadIdx.x] : 0u;
        m = __reduce_max_sync(0xFFFFFFFFu, m);
        if (threadIdx.x == 0 && m > seen) atomicMax(state + XCHG_W_ACCUM, m);
    }
}

// ---- resolve side --------------------------------------------------------------------------------------------
// Hands this rank's amax to every rank as the next exchange and returns that exchange's number; call with all 32
// lanes of one warp.  Waits for nothing.
__device__ __forceinline__ uint32_t xchg_publish(uint32_t *state, const XchgPeers &p)
{
    const int lane = threadIdx.x & 31;
    const uint32_t e = ld_volatile_u32(state + XCHG_W_EXCHANGES) + 1u;
    const uint32_t bits = ld_volatile_u32(state + XCHG_W_ACCUM);
    __syncwarp();
    if (lane < p.world) {
        unsigned long long *dst = p.slots[lane] + (size_t)(e & 1u) * QCC_XCHG_MAX_RANKS + p.rank;
        st_relaxed_sys_u64(dst, ((unsigned long long)e << 32) | bits);
    }
    if (lane == 0) {
        state[XCHG_W_ACCUM] = 0u;
        state[XCHG_W_EXCHANGES] = e;
    }
    return e;
}
// Number of the exchange this rank published last (for a reader that does not publish).
__device__ __forceinline__ uint32_t xchg_current(const uint32_t *state) { return ld_volatile_u32(state + XCHG_W_EXCHANGES); }

// The maximum over the `world` ranks of exchange `e`, to all lanes; call with all 32 lanes of a warp.
// On a timeout the value is the maximum of whatever the slots hold.
__device__ __forceinline__ float xchg_resolve(uint32_t *state, int world, uint32_t e)
{
    const int lane = threadIdx.x & 31;
    const unsigned long long *slots =
        reinterpret_cast<const unsigned long long *>(reinterpret_cast<const uint8_t *>(state) + XCHG_SLOT_BYTE_OFF) +
        (size_t)(e & 1u) * QCC_XCHG_MAX_RANKS;
    uint32_t bits = 0;
    if (lane < world) {
        unsigned long long v = ld_relaxed_sys_u64(slots + lane);
        if ((uint32_t)(v >> 32) != e) {
            const unsigned long long t0 = globaltimer_ns();
            const unsigned long long limit = (unsigned long long)ld_volatile_u32(state + XCHG_W_TIMEOUT) * 1000ull;
            for (;;) {
                v = ld_relaxed_sys_u64(slots + lane);
                if ((uint32_t)(v >> 32) == e) break;
                if (ld_volatile_u32(state + XCHG_W_ABORT) != 0u) break;
                if (globaltimer_ns() - t0 > limit) {
                    atomicMax(&g_qcc_error, QCC_DEVERR_XCHG);
                    atomicExch(state + XCHG_W_ABORT, 1u);
                    break;
                }
                __nanosleep(100);
            }
        }
        bits = (uint32_t)v;
    }
    return u2f(__reduce_max_sync(0xFFFFFFFFu, bits));
}

// Host side: the by-value peer table of a launch from the caller's array of state pointers.
inline int make_xchg_peers(XchgPeers *p, void *const *states, int world, int rank)
{
    if (!states || world < 1 || world > QCC_XCHG_MAX_RANKS || rank < 0 || rank >= world) return QCC_ERR_ARG;
    for (int r = 0; r < QCC_XCHG_MAX_RANKS; r++) p->slots[r] = nullptr;
    for (int r = 0; r < world; r++) {
        if (!states[r]) return QCC_ERR_ARG;
        p->slots[r] = reinterpret_cast<unsigned long long *>(static_cast<uint8_t *>(states[r]) + XCHG_SLOT_BYTE_OFF);
    }
    p->world = world;
    p->rank = rank;
    return 0;
}

}  // namespace qcc
