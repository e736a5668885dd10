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

// Second half of the routing of one token (one warp): lane j < top_k holds the j-th pick (descending logit, ties to the
// lower id, NaN as -inf) as a key; it ends up with the expert id, the softmax weight over the selection (summed in
// descending-logit order: top_k :3136-3138, soft_top :3126-3131; all-NaN / all -inf gives uniform weights) and `rank` =
// its position when the selection is sorted by ascending expert id, the order in which the expert outputs are
// accumulated (routed, f32 branch :1786).
__device__ __forceinline__ void pb_route_finish(unsigned long long pick, int top_k, int lane, int& my_e, float& w, int& rank) {
    my_e = pb_topk_id(pick);
    const float my_v = pb_topk_val(pick);
    float mx = lane < top_k ? my_v : -INFINITY;
    mx = pb_warp_max(mx);
    w = lane < top_k ? expf(my_v - mx) : 0.f;
    float sum = 0.f;
    for (int j = 0; j < top_k; j++) sum += __shfl_sync(0xffffffffu, w, j);
    w = isfinite(mx) ? w / sum : 1.0f / (float)(top_k > 0 ? top_k : 1);
    rank = 0;
    for (int j = 0; j < top_k; j++) { const int oe = __shfl_sync(0xffffffffu, my_e, j); if (oe < my_e) rank++; }
}

// Routing of one token by one warp.  lg: n_exp <= 1024 logits, read with L1-bypassing loads (they may have been written
// by other SMs of this launch).
__device__ __forceinline__ void pb_route_token(const float* lg, int n_exp, int top_k, int lane, int& my_e, float& w, int& rank) {
    unsigned long long pick;
    if (n_exp <= 512) {
        unsigned long long keys[16];
#pragma unroll
        for (int i = 0; i < 16; i++) { const int e = i * 32 + lane; keys[i] = e < n_exp ? pb_topk_key(__ldcg(lg + e), e) : 0ull; }
        pick = pb_warp_topk<16>(keys, top_k, lane);
    } else {
        unsigned long long keys[32];
#pragma unroll
        for (int i = 0; i < 32; i++) { const int e = i * 32 + lane; keys[i] = e < n_exp ? pb_topk_key(__ldcg(lg + e), e) : 0ull; }
        pick = pb_warp_topk<32>(keys, top_k, lane);
    }
    pb_route_finish(pick, top_k, lane, my_e, w, rank);
}
