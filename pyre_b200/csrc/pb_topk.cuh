// Warp-level top-k over router logits with the reference's order: descending logit, ties to the lower
// expert id, NaN treated as -inf (top_k / nan_clean, src/model/qwen4exp_gguf.rs:3121-3139).
// A candidate is one 64-bit key: the logit mapped to an order-preserving unsigned in the high word and
// ~id in the low word, so one unsigned comparison decides both criteria and keys are unique.
#pragma once
#include "pb_common.cuh"

__device__ __forceinline__ unsigned long long pb_topk_key(float v, int e) {
    if (isnan(v)) v = -INFINITY;
    unsigned u = __float_as_uint(v);
    u ^= (u >> 31) ? 0xFFFFFFFFu : 0x80000000u;                      // monotonic: larger float -> larger unsigned
    return ((unsigned long long)u << 32) | (unsigned)(0xFFFFFFFFu - (unsigned)e);
}
__device__ __forceinline__ int pb_topk_id(unsigned long long k) { return (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFu)); }
__device__ __forceinline__ float pb_topk_val(unsigned long long k) {
    unsigned u = (unsigned)(k >> 32);
    u ^= (u >> 31) ? 0x80000000u : 0xFFFFFFFFu;
    return __uint_as_float(u);
}
__device__ __forceinline__ unsigned long long pb_warp_max64(unsigned long long k) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, k, o);
        k = other > k ? other : k;
    }
    return k;
}
// keys[N] per lane (0 = empty slot; real keys are never 0 because the low word of a real key is >= 0x7FFFFFFF).
// Returns in lane j (j < k) the j-th largest key of the warp's 32 * N keys; consumed keys are cleared.
template <int N>
__device__ __forceinline__ unsigned long long pb_warp_topk(unsigned long long (&keys)[N], int k, int lane) {
    unsigned long long mine = 0;
    for (int j = 0; j < k; j++) {
        unsigned long long m = keys[0];
#pragma unroll
        for (int i = 1; i < N; i++) m = keys[i] > m ? keys[i] : m;
        m = pb_warp_max64(m);
        if (lane == j) mine = m;
#pragma unroll
        for (int i = 0; i < N; i++) if (keys[i] == m) keys[i] = 0;
    }
    return mine;
}
