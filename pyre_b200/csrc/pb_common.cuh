// Shared device/host helpers for the sm_100a kernels: status codes, bounded mbarrier
// waits, bulk (TMA 1-D) global->shared copies, f16 conversion.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/pyre_b200.h"

#define PB_WARP 32

// Device-side error word values (written to ctx->dev_status by kernels; never trap).
enum : int {
    PB_DEV_OK = 0,
    PB_DEV_WAIT_FULL_TIMEOUT = 1,   // consumer gave up waiting for a bulk copy to land
    PB_DEV_WAIT_EMPTY_TIMEOUT = 2,  // producer gave up waiting for a stage to be released
    PB_DEV_BAD_INDEX = 3,           // an expert id / position outside its range was skipped
};

// Upper bound for every spin on an mbarrier.  try_wait suspends for a hardware-defined
// interval per call, so this is seconds of wall time, after which the kernel records the
// failure in the status word and returns instead of hanging the GPU.
#define PB_SPIN_LIMIT (1u << 22)

__device__ __forceinline__ uint32_t pb_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void pb_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pb_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void pb_fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void pb_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void pb_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pb_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pb_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pb_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool pb_mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(pb_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and records `code` in *status) if the phase never completes.
__device__ __forceinline__ bool pb_mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
    for (uint32_t i = 0; i < PB_SPIN_LIMIT; i++) {
        if (pb_mbar_try_wait(bar, parity)) return true;
        if (i > 32) __nanosleep(96);
    }
    if (status) atomicExch(status, code);
    return false;
}
// The same for a waiter that is far ahead of the event (a producer waiting for a stage of its ring to be
// released): it sleeps between the polls from the start.  A bare polling loop issues an instruction every few
// cycles and takes a quarter of the issue slots of its SM sub-partition away from the warps that do the work.
__device__ __forceinline__ bool pb_mbar_wait_relaxed(uint64_t* bar, uint32_t parity, int* status, int code) {
    for (uint32_t i = 0; i < PB_SPIN_LIMIT; i++) {
        if (pb_mbar_try_wait(bar, parity)) return true;
        __nanosleep(256);
    }
    if (status) atomicExch(status, code);
    return false;
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
// Both addresses must be 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void pb_bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(pb_smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(pb_smem_u32(bar))
                 : "memory");
}

// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may
// start while its predecessor still runs.  pb_pdl_trigger lets the successor be scheduled;
// pb_pdl_wait blocks until every predecessor grid has completed and its writes are visible.  All
// reads of data produced by earlier kernels, and all global writes, come after pb_pdl_wait.
// Without the launch attribute both are no-ops.
__device__ __forceinline__ void pb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pb_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Phase stamps (tracing): when a launch was given a stamp slot, thread 0 of its first and of its last CTA record
// %globaltimer (ns) at fixed points of the kernel; the host reads the slots back after the step (pb_ctx_stamps_read).
// The reference traces its expert chain the same way (src/model/xchain.rs:1-111).  PB_STAMP_WORDS words per launch:
//   first CTA: 0 entry, 1 set-up done, 2 predecessor's data visible, 3 activations ready, 4 first stage landed, 5 last store
//   last CTA : 6 entry, 7 last store
#define PB_STAMP_WORDS 8
__device__ __forceinline__ unsigned long long pb_globaltimer() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ void pb_stamp(unsigned long long* slot, int phase, bool who) { if (slot && who) slot[phase] = pb_globaltimer(); }

__device__ __forceinline__ float pb_h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

__device__ __forceinline__ float pb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float pb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float pb_sigm(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float pb_silu(float x) { return x * pb_sigm(x); }
__device__ __forceinline__ float pb_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
