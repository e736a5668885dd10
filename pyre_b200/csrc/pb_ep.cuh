// Device side of the peer exchange between expert-parallel ranks: sequence-numbered flags in peer memory.
//
// flags[kind][src] in the receiver's memory = sequence number of the last exchange of `kind` that rank `src` completed.
// The writer orders its data stores before the flag with a system-scope fence and a release store; the reader polls
// with system-scope acquire loads.  Sequence numbers only grow, so a reader compares with >=.  Every wait is bounded:
// a rank whose peer never arrives records PB_DEV_PEER_TIMEOUT in the status word and carries on (its results are
// garbage; the host call that synchronises next returns PB_ERR_DEVICE).  The reference's CPU/GPU hand-shake gives up
// the same way (pyre_wait_flag, src/model/qwen4exp_gguf.rs:229-238).
// Only plain loads and stores touch peer memory.
#pragma once
#include "pb_common.cuh"
#include "pb_internal.h"

enum : int { PB_DEV_PEER_TIMEOUT = 5 };   // a peer did not announce an exchange in time

__device__ __forceinline__ unsigned long long pb_ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void pb_st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// one thread: tell rank p that this rank finished exchange `seq` of `kind`.  The data stores it covers must have been
// made visible to this thread first (a kernel boundary, or a barrier / ticket after the storing threads' own system
// fences); the fence here makes this thread's view of them the one the release store publishes.
__device__ __forceinline__ void pb_ep_post(const PbEpExch& x, int p, int kind, unsigned long long seq) {
    __threadfence_system();
    pb_st_release_sys(x.peer_flags[p] + (size_t)kind * x.world + x.rank, seq);
}
// one thread: wait (bounded) until rank p announced exchange `seq` of `kind`
__device__ __forceinline__ void pb_ep_wait(const PbEpExch& x, int p, int kind, unsigned long long seq) {
    const unsigned long long* mine = x.peer_flags[x.rank] + (size_t)kind * x.world + p;
    bool ok = false;
    for (unsigned int i = 0; i < x.spin_limit; i++) {
        if (pb_ld_acquire_sys(mine) >= seq) { ok = true; break; }
        if (i > 64) __nanosleep(200);
    }
    if (!ok) atomicExch(x.status, PB_DEV_PEER_TIMEOUT);
}
__device__ __forceinline__ void pb_ep_handshake(const PbEpExch& x, int p, int kind, unsigned long long seq) {
    const unsigned long long t0 = pb_globaltimer();
    pb_ep_post(x, p, kind, seq);
    pb_ep_wait(x, p, kind, seq);
    if (x.wait_ns) atomicAdd(x.wait_ns, pb_globaltimer() - t0);   // summed over the world's threads; the host divides
}
