// Router arithmetic shared by pb_router_kernel (pb_moe.cu) and the fused step kernel (pb_step.cu): both produce the
// same bits, so the expert selection of a token does not depend on which of them ran.
// Restates the router product of ffn (src/model/qwen4exp_gguf.rs:1675-1684) over rms(x) (:209).
#pragma once
#include "pb_common.cuh"

// 1 / sqrt(mean(x^2) + eps) of one row of `cols` values, computed by one warp (every lane gets the result).
// Every multiply-add is spelled out (fmaf): left to the compiler, the fusing of a*a + b*b + .. into multiply-adds may come
// out differently in the two kernels that inline this function, and their results would differ in the last bit.
__device__ __forceinline__ float pb_row_rms_scale(const float* x, int cols, float eps, int lane) {
    float ss = 0.f;
    for (int c = lane * 4; c < cols; c += 128) { const float4 v = *reinterpret_cast<const float4*>(x + c); ss += fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, __fmul_rn(v.w, v.w)))); }
    ss = pb_warp_sum(ss);
    return 1.0f / sqrtf(ss / (float)cols + eps);
}

// One router row of 2048 columns against one token, by one warp: the row times the norm weight is formed in registers,
// the token's scale is applied to the sum (w . (x s n) = s ((w n) . x) up to rounding).  norm_w may be null.
struct PbRouterRow2048 {
    float4 wr[16];
    __device__ __forceinline__ void load(const float* wrow, const float* norm_w, int lane) {
#pragma unroll
        for (int k = 0; k < 16; k++) {
            wr[k] = *reinterpret_cast<const float4*>(wrow + lane * 4 + 128 * k);
            if (norm_w) { const float4 n = *reinterpret_cast<const float4*>(norm_w + lane * 4 + 128 * k); wr[k].x *= n.x; wr[k].y *= n.y; wr[k].z *= n.z; wr[k].w *= n.w; }
        }
    }
    __device__ __forceinline__ float dot(const float* x, float scale, int lane) const {
        const float* xb = x + lane * 4;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int k = 0; k < 16; k++) {
            const float4 v = *reinterpret_cast<const float4*>(xb + 128 * k);
            a0 = fmaf(wr[k].x, v.x, a0); a1 = fmaf(wr[k].y, v.y, a1); a2 = fmaf(wr[k].z, v.z, a2); a3 = fmaf(wr[k].w, v.w, a3);
        }
        return pb_warp_sum((a0 + a1) + (a2 + a3)) * scale;
    }
};

// The same product for one token without keeping the row: (w n) is formed per element on the way (same roundings).
__device__ __forceinline__ float pb_router_row2048_dot1(const float* wrow, const float* norm_w, const float* x, float scale, int lane) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 4
    for (int k = 0; k < 16; k++) {
        float4 w = *reinterpret_cast<const float4*>(wrow + lane * 4 + 128 * k);
        if (norm_w) { const float4 n = *reinterpret_cast<const float4*>(norm_w + lane * 4 + 128 * k); w.x *= n.x; w.y *= n.y; w.z *= n.z; w.w *= n.w; }
        const float4 v = *reinterpret_cast<const float4*>(x + lane * 4 + 128 * k);
        a0 = fmaf(w.x, v.x, a0); a1 = fmaf(w.y, v.y, a1); a2 = fmaf(w.z, v.z, a2); a3 = fmaf(w.w, v.w, a3);
    }
    return pb_warp_sum((a0 + a1) + (a2 + a3)) * scale;
}

// any width (a multiple of 128): one accumulator chain over the normalized activations
__device__ __forceinline__ float pb_router_row_dot(const float* wrow, const float* norm_w, const float* x, float s, int cols, int lane) {
    float acc = 0.f;
#pragma unroll 4
    for (int c = lane * 4; c < cols; c += 128) {
        const float4 w = *reinterpret_cast<const float4*>(wrow + c);
        float4 v = *reinterpret_cast<const float4*>(x + c);
        if (norm_w) {
            const float4 n = *reinterpret_cast<const float4*>(norm_w + c);
            v.x = v.x * s * n.x; v.y = v.y * s * n.y; v.z = v.z * s * n.z; v.w = v.w * s * n.w;
        }
        acc = fmaf(w.x, v.x, acc); acc = fmaf(w.y, v.y, acc); acc = fmaf(w.z, v.z, acc); acc = fmaf(w.w, v.w, acc);
    }
    return pb_warp_sum(acc);
}
