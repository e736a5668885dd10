// Dequant-GEMM for 16 and more activation columns on the fifth-generation tensor cores (tcgen05), IQ3_S weights.
//
//   y[b][yoff_s + r] (+)= sum_c W_s[r][c] * act(x)[b][c]        b = 0 .. t-1,  t >= 16
//
// This is the path of prefill chunks, wide verify windows and batched decode: the reference switches to its tensor-core
// GEMM at 16 tokens as well (gmm, src/model/qwen4exp_gguf.rs:3264-3266; k_gemm_tc, src/model/qn_cube.rs:153, host side
// gemm_pfx :6559-6587).  One CTA owns a tile of 128 weight rows x up to 128 tokens and walks the contraction in steps of
// 64 columns through a ring of 6 stages (a weight tile in tensor memory + the activation tiles in shared memory):
//
//   producer warp       brings the activations of each step -- f16 high and low parts (x = hi + lo, 22 significant
//                       bits), prepared once per GEMM by pb_xt_prep_kernel in exactly the operand layout -- with 1-D
//                       bulk copies.
//   decoder warps (8)   stream the re-coded IQ3_S rows of the tile (4-bit codes, PB_T_IQ3S_N4: 136 bytes per row and 256
//                       columns) into a double buffer of raw bytes with 8-byte cp.async (all 256 threads share the
//                       copies), then one thread = one row x 64 columns per step: f16 weights stored with tcgen05.st
//                       into the thread's own lane of a weight tile in tensor memory (the A operand is read from
//                       there, behind the accumulator).  (2c - 15) * (1 + 2s) is
//                       exact in f16; the block scale d is folded in with one rounding (relative 2^-11), after a
//                       per-tile power-of-two shift that keeps d * 465 inside the f16 range and is undone at the end.
//   MMA warp            one elected thread issues tcgen05.mma (kind::f16, M = 128, N = tokens, K = 16) for the high and
//                       the low part into one f32 accumulator in tensor memory (128 lanes x N columns) and frees the
//                       stage with tcgen05.commit -> mbarrier.
//   epilogue            the decoder warps read the accumulator with tcgen05.ld (lane = row), undo the scales and store.
//
// Every wait is bounded; a wait that runs out records a status (the host call returns PB_ERR_DEVICE) and the CTA leaves
// through the common exit, which frees its tensor memory.  No cluster, nothing multicast, operands only from this GPU.
#include "pb_stream.cuh"
#include "pb_internal.h"

#include <cuda_fp16.h>
#include <stdio.h>

#define TC_ROWS 128                 // weight rows per tile = MMA M
#define TC_NBLK 128                 // tokens per CTA; the MMA's N is twice the (padded) token count: high and low parts side by side
#define TC_KSTEP 64                 // contraction columns per step
#define TC_STAGES 6                 // ring depth: a stage = a decoded weight tile in tensor memory (32 columns behind the accumulator's
                                    // 256) + the activation tiles of the same step in shared memory (32 KB at 128 tokens)
#define TC_ACC_COLS (2 * TC_NBLK)   // accumulator columns: high and low parts of up to 128 tokens
#define TC_A_COLS (TC_KSTEP / 2)    // a weight tile is 128 lanes x 32 columns: two f16 per 32-bit cell
#define TC_TMEM_COLS 512            // 256 + 6 x 32 = 448, rounded to the power of two: the whole tensor memory of the SM (one CTA per SM)
#define TC_RAW_STAGES 2             // raw double buffer: one block (256 columns = 4 steps) each
#define TC_RAW_BYTES (TC_ROWS * 136)
#define TC_DECODERS 8
#define TC_THREADS ((TC_DECODERS + 2) * 32)
#define TC_B_BYTES (2 * TC_NBLK * TC_KSTEP * 2)                   // high and low activation tiles: 32 KB
#define TC_XT_HEAD 4096             // bytes of per-token prescale inverses in front of the activation tiles

enum : int { PB_DEV_TC_TIMEOUT = 6 };

// ---------------------------------------------------------------- tcgen05 wrappers (cta_group::1)
__device__ __forceinline__ void tc_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pb_smem_u32(smem_dst)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D (tensor memory) (+)= A (tensor memory: lane = row, two f16 per cell along K) x B (shared memory, by descriptor)
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the mbarrier receives one arrival once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pb_smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive columns of 32-bit cells: thread l of the warp gets lane (base lane + l), columns c .. c+31
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory operand descriptor: K-major, 128-byte swizzle.  A row of the tile (one weight row or one token) is 128
// contiguous bytes = the 64 columns of a step; its 16-byte chunk c sits at chunk position c ^ (row & 7); groups of 8
// rows are 1024 bytes apart (the stride offset); the tile starts on a 1024-byte boundary.  A step of 16 columns along K
// is 32 bytes further into the row: the start address moves, the swizzle is applied by the hardware on the address bits.
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: f32 accumulator, f16 A and B, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t tc_idesc(int m, int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24); }

// ---------------------------------------------------------------- activations -> operand tiles

// byte offset of element (token n of its block, column c) inside the block's tiles; np = padded tokens of the block
__device__ __forceinline__ size_t pb_xt_off(int np, int n, int c, int lo) {
    const int ks = c >> 6, kk = c & 63;
    return (size_t)ks * (2 * (size_t)np * 128) + (lo ? (size_t)np * 128 : 0) + (size_t)n * 128 + (size_t)(((kk >> 3) ^ (n & 7)) * 16) + (size_t)(kk & 7) * 2;
}
__device__ __forceinline__ void pb_xt_store(uint8_t* blk, int np, int n, int c, float4 v) {
    const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
    const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
    const __half2 l01 = __floats2half2_rn(v.x - f01.x, v.y - f01.y), l23 = __floats2half2_rn(v.z - f23.x, v.w - f23.y);
    *reinterpret_cast<uint2*>(blk + pb_xt_off(np, n, c, 0)) = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
    *reinterpret_cast<uint2*>(blk + pb_xt_off(np, n, c, 1)) = make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
}
__host__ __device__ __forceinline__ int pb_xt_np(int t, int tb) { const int n = t - tb * TC_NBLK < TC_NBLK ? t - tb * TC_NBLK : TC_NBLK; return (n + 15) & ~15; }

// One CTA per token slot (the slots past t of the last block are written as zeros).  The activation function is the
// one of the other GEMV kernels: PLAIN (with an exact power-of-two prescale into [0.5, 1) so that f16 neither overflows
// nor loses small columns), NORM (RMS norm times weight), GNORM (per-head RMS norm times weight times sigmoid(z)).
// xbuf: TC_XT_HEAD bytes of prescale inverses [t], then per block of TC_NBLK tokens, per step of 64 columns, the high
// tile and the low tile, each np x 64 f16 as swizzled 128-byte rows.
__global__ void __launch_bounds__(256) pb_xt_prep_kernel(const PbGemvQParams p, uint8_t* __restrict__ xbuf) {
    constexpr int CT = 256;
    const int slot = (int)blockIdx.x;
    const int tb = slot / TC_NBLK, n = slot - tb * TC_NBLK;
    const int np = pb_xt_np(p.t, tb);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cols = p.bpr * 256;
    __shared__ float red0[8];
    pb_pdl_wait();
    pb_pdl_trigger();
    if (n >= np) return;
    const int tok = tb * TC_NBLK + n;
    const bool live = tok < p.t;
    const float* x = p.x + (size_t)tok * p.ldx;
    const float* z = p.z ? p.z + (size_t)tok * p.ldz : nullptr;
    uint8_t* blk = xbuf + TC_XT_HEAD + (size_t)tb * ((size_t)cols / 64) * (2 * (size_t)TC_NBLK * 128);
    float* xinv = reinterpret_cast<float*>(xbuf);
    if (tid == 0 && live) xinv[tok] = 1.0f;
    if (p.mode == PB_ACT_GNORM) {
        const int nheads = cols / p.head_dim;   // head_dim == 128 (checked on the host)
        for (int h = warp; h < nheads; h += 8) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live) {
                v = *reinterpret_cast<const float4*>(x + h * p.head_dim + 4 * lane);
                const float ss = pb_warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
                const float s = 1.0f / sqrtf(ss / (float)p.head_dim + p.eps);
                const float4 w = *reinterpret_cast<const float4*>(p.norm_w + 4 * lane);
                const float4 zz = *reinterpret_cast<const float4*>(z + h * p.head_dim + 4 * lane);
                v.x = v.x * (s * w.x) * pb_sigm(zz.x); v.y = v.y * (s * w.y) * pb_sigm(zz.y); v.z = v.z * (s * w.z) * pb_sigm(zz.z); v.w = v.w * (s * w.w) * pb_sigm(zz.w);
            }
            pb_xt_store(blk, np, n, h * p.head_dim + 4 * lane, v);
        }
        return;
    }
    float r = 0.f;
    if (live) for (int c = tid; c < cols; c += CT) { const float v = x[c]; r = p.mode == PB_ACT_NORM ? r + v * v : fmaxf(r, fabsf(v)); }
    r = p.mode == PB_ACT_NORM ? pb_warp_sum(r) : pb_warp_max(r);
    if (lane == 0) red0[warp] = r;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot = p.mode == PB_ACT_NORM ? tot + red0[i] : fmaxf(tot, red0[i]);
    float s = 1.0f;
    if (p.mode == PB_ACT_NORM) s = 1.0f / sqrtf(tot / (float)cols + p.eps);
    else if (tot > 0.f && tot <= 3.0e38f) {
        int e; (void)frexpf(tot, &e);
        s = ldexpf(1.0f, -e);
        if (tid == 0 && live) xinv[tok] = ldexpf(1.0f, e);
    }
    for (int c = tid * 4; c < cols; c += CT * 4) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
            v = *reinterpret_cast<const float4*>(x + c);
            if (p.mode == PB_ACT_NORM) { const float4 w = *reinterpret_cast<const float4*>(p.norm_w + c); v.x = v.x * s * w.x; v.y = v.y * s * w.y; v.z = v.z * s * w.z; v.w = v.w * s * w.w; }
            else { v.x *= s; v.y *= s; v.z *= s; v.w *= s; }
        }
        pb_xt_store(blk, np, n, c, v);
    }
}

// ---------------------------------------------------------------- weights -> operand tile

// raw bytes of one quarter (64 weights) of a re-coded block: {d (f16) | pad, four sub-scale bytes}, 32 bytes of codes
struct TcRaw { uint2 head; uint2 c[4]; };
// from the raw ring: `b` = shared-memory address of this row's block (rows 136 bytes apart: 8-byte loads of 16 lanes hit 32 banks)
__device__ __forceinline__ void tc_load_raw(TcRaw& r, uint32_t b, int qt, bool live) {
    if (!live) { r.head = make_uint2(0u, 0u); r.c[0] = r.c[1] = r.c[2] = r.c[3] = make_uint2(0x77777777u, 0x77777777u); return; }
    // volatile with a memory clobber: these loads must stay behind the wait for the block's copies
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(r.head.x), "=r"(r.head.y) : "r"(b) : "memory");
#pragma unroll
    for (int i = 0; i < 4; i++) asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(r.c[i].x), "=r"(r.c[i].y) : "r"(b + 8 + 32 * qt + 8 * i) : "memory");
}
__device__ __forceinline__ void tc_cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
// the mbarrier (initialised with one count per issuing thread) gets this thread's arrival once its copies so far have landed
__device__ __forceinline__ void tc_cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(pb_smem_u32(bar)) : "memory");
}
// 32 cells of this thread's lane, consecutive columns from taddr on (taddr carries the warp's first lane in bits 16+)
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
          "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
          "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// decode the 64 columns of step ks of this thread's row and store them as its lane of the weight tile at taddr
// (tensor memory: lane = row, cell j = columns 2j, 2j + 1 of the step)
__device__ __forceinline__ void tc_decode_store(const TcRaw& r, int ks, uint32_t taddr, float shift) {
    const int qt = ks & 3;
    const float d = pb_h2f((uint16_t)(r.head.x & 0xFFFF)) * shift;
    const uint32_t sc = (r.head.y >> (8 * qt)) & 0xFF;
    const float f0 = (float)(1 + 2 * (int)(sc & 0xF)), f1 = (float)(1 + 2 * (int)(sc >> 4));
    const __half2 a0 = __float2half2_rn(2.0f * f0), b0 = __float2half2_rn(-15.0f * f0);
    const __half2 a1 = __float2half2_rn(2.0f * f1), b1 = __float2half2_rn(-15.0f * f1);
    const __half2 k1024 = __float2half2_rn(1024.0f), d2 = __float2half2_rn(d);
    uint32_t cells[32];
#pragma unroll
    for (int i = 0; i < 4; i++) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int u = 2 * i + j;                      // word u = weights 8u .. 8u+7 of the quarter = core matrix u along K
            const uint32_t w = j ? r.c[i].y : r.c[i].x;
            const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
            const uint32_t c4[4] = {pb_prmt(lo, 0x64006400u, 0x7150u), pb_prmt(lo, 0x64006400u, 0x7352u), pb_prmt(hi, 0x64006400u, 0x7150u), pb_prmt(hi, 0x64006400u, 0x7352u)};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                // (1024 + c) - 1024 = c, c * 2m - 15m = (2c - 15) m: exact in f16; the product with d rounds once
                const __half2 v = __hmul2(__hfma2(__hsub2(*reinterpret_cast<const __half2*>(&c4[e]), k1024), u < 4 ? a0 : a1, u < 4 ? b0 : b1), d2);
                cells[4 * u + e] = *reinterpret_cast<const uint32_t*>(&v);
            }
        }
    }
    tc_st32(taddr, cells);
}

struct TcParams {
    PbGemvQSeg seg[4];      // chunk0 = first tile of the segment
    int nseg, ntiles;
    int row_bytes, cols, t;
    const uint8_t* xt;      // prepared activations (pb_xt_prep_kernel)
    float* y; int64_t ldy;
    int accumulate;
    int* status;
};

__global__ void __launch_bounds__(TC_THREADS, 1) pb_gemmtc_iq3s_kernel(const TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);             // [TC_STAGES] 128 decoder arrivals + the producer's, and the bulk-copy bytes
    uint64_t* empty = full + TC_STAGES;                             // [TC_STAGES] tcgen05.commit: the MMAs that read the stage are done
    uint64_t* raw_full = empty + TC_STAGES;                         // [TC_RAW_STAGES] 256 decoder threads (cp.async)
    uint64_t* raw_empty = raw_full + TC_RAW_STAGES;                 // [TC_RAW_STAGES] 256 decoder threads
    uint64_t* acc_full = raw_empty + TC_RAW_STAGES;                 // accumulator complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 384);
    float* red = reinterpret_cast<float*>(smem + 416);              // [8] per-warp maxima of d
    float* xinv = reinterpret_cast<float*>(smem + 512);             // [TC_NBLK]
    uint8_t* b_ring = smem + 1024;                                  // [TC_STAGES][high tile | low tile], swizzled 128-byte rows
    uint8_t* raw = b_ring + TC_STAGES * TC_B_BYTES;               // [TC_RAW_STAGES][128 rows][136 bytes]
    static_assert((TC_STAGES * 2 + TC_RAW_STAGES * 2 + 1) * 8 <= 384 && TC_ACC_COLS + TC_STAGES * TC_A_COLS <= TC_TMEM_COLS, "barriers fit in front of the TMEM slot");
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int tile = (int)blockIdx.x, tb = (int)blockIdx.y;
    int s = 0;
    while (s + 1 < p.nseg && tile >= p.seg[s + 1].chunk0) s++;
    const int r0 = (tile - p.seg[s].chunk0) * TC_ROWS;
    const int nr = min(TC_ROWS, p.seg[s].rows - r0);
    const int np = pb_xt_np(p.t, tb);                 // padded tokens of this block = MMA N
    const int nt = min(TC_NBLK, p.t - tb * TC_NBLK);  // live tokens
    const int nk = p.cols / TC_KSTEP;
    const uint32_t bbytes = 2u * (uint32_t)np * 128u;

    if (tid == 0) {
        for (int i = 0; i < TC_STAGES; i++) { pb_mbar_init(&full[i], 128 + 1); pb_mbar_init(&empty[i], 1); }
        for (int i = 0; i < TC_RAW_STAGES; i++) { pb_mbar_init(&raw_full[i], TC_DECODERS * 32); pb_mbar_init(&raw_empty[i], TC_DECODERS * 32); }
        pb_mbar_init(acc_full, 1);
        pb_fence_barrier_init();
    }
    if (warp == TC_DECODERS + 1) tc_alloc(tmem_slot, TC_TMEM_COLS);
    pb_pdl_trigger();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pb_pdl_wait();    // the activation tiles, and y when accumulating, come from earlier launches

    if (warp == TC_DECODERS) {
        // ------------------------------------------------------------ producer: activation tiles, TC_STAGES steps ahead
        if (lane == 0) {
            const uint8_t* src = p.xt + TC_XT_HEAD + (size_t)tb * (size_t)nk * (2 * (size_t)TC_NBLK * 128);
            int k = 0;
            for (; k < nk; k++) {
                const int st = k % TC_STAGES;
                if (k >= TC_STAGES && !pb_mbar_wait(&empty[st], ((k / TC_STAGES) - 1) & 1, p.status, PB_DEV_TC_TIMEOUT)) break;
                pb_mbar_expect_tx(&full[st], bbytes);
                pb_bulk_g2s(b_ring + (size_t)st * TC_B_BYTES, src + (size_t)k * bbytes, bbytes, &full[st]);
            }
            // error path: the copies in flight get a bounded chance to land before the CTA may exit
            // (a stage's barrier also counts the decoders' arrivals: on the error path it may never complete; the wait is bounded)
            if (k < nk) for (int j = max(0, k - TC_STAGES); j < k; j++) pb_mbar_wait(&full[j % TC_STAGES], (j / TC_STAGES) & 1, nullptr, 0);
        }
    } else if (warp == TC_DECODERS + 1) {
        // ------------------------------------------------------------ MMA issue
        // the high and the low tile are stacked along N: one instruction of N = 2 np columns per 16 columns of K reads the
        // weight tile once; the epilogue adds the two halves of the accumulator
        const uint32_t idesc = tc_idesc(TC_ROWS, 2 * np);
        bool ok = true;
        for (int k = 0; k < nk && ok; k++) {
            const int st = k % TC_STAGES;
            ok = pb_mbar_wait(&full[st], (k / TC_STAGES) & 1, p.status, PB_DEV_TC_TIMEOUT);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t a_t = tmem + TC_ACC_COLS + (uint32_t)st * TC_A_COLS;
                const uint32_t b_s = pb_smem_u32(b_ring + (size_t)st * TC_B_BYTES);
#pragma unroll
                for (int kk = 0; kk < TC_KSTEP / 16; kk++) tc_mma_f16_ts(tmem, a_t + kk * 8, tc_desc(b_s + kk * 32), idesc, (k | kk) ? 1u : 0u);
                tc_commit(&empty[st]);
            }
            __syncwarp();
        }
        if (ok && lane == 0) tc_commit(acc_full);
        __syncwarp();
    } else {
        // ------------------------------------------------------------ decoders, then epilogue
        const int grp = warp >> 2;                 // two groups of four warps take alternate steps
        const int row = (warp & 3) * 32 + lane;    // row of the tile
        const bool live = row < nr;
        const uint8_t* wbase = p.seg[s].w + (size_t)r0 * p.row_bytes;
        // raw bytes: block kb of the tile's rows (136 bytes per row) -> raw[kb % 2]; thread tid copies 8-byte words tid, tid + 256, ..
        const int nkb = p.cols / 256, nwords = nr * 17;
        auto issue_raw = [&](int kb) {
            const uint32_t dst = pb_smem_u32(raw + (size_t)(kb % TC_RAW_STAGES) * TC_RAW_BYTES);
            for (int i = tid; i < nwords; i += TC_DECODERS * 32) {
                const int r = i / 17, w = i - r * 17;
                tc_cp_async8(dst + (uint32_t)(r * 136 + w * 8), wbase + (size_t)r * p.row_bytes + (size_t)kb * 136 + w * 8);
            }
            tc_cp_async_arrive(&raw_full[kb % TC_RAW_STAGES]);
        };
        issue_raw(0);
        if (nkb > 1) issue_raw(1);
        // per-tile power-of-two shift: the largest |d| of the tile's rows times 465 lands in [2^14, 2^15)
        float dm = 0.f;
        if (grp == 0 && live) for (int b = 0; b < nkb; b++) dm = fmaxf(dm, fabsf(pb_h2f(__ldg(reinterpret_cast<const uint16_t*>(wbase + (size_t)row * p.row_bytes + (size_t)b * 136)))));
        dm = pb_warp_max(dm);
        if (lane == 0) red[warp] = dm;
        if (tid < TC_NBLK) xinv[tid] = tid < nt ? reinterpret_cast<const float*>(p.xt)[tb * TC_NBLK + tid] : 0.f;
        pb_named_barrier(1, TC_DECODERS * 32);
        dm = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
        int sh = 0;
        if (dm > 0.f && dm < 3.0e38f) { int e; (void)frexpf(dm * 465.0f, &e); sh = 15 - e; }   // dm * 465 * 2^sh in [2^14, 2^15)
        const float shift = ldexpf(1.0f, sh), unshift = ldexpf(1.0f, -sh);

        bool ok = true;
        for (int k = grp; k < nk; k += 2) {
            const int st = k % TC_STAGES, kb = k >> 2, rs = kb % TC_RAW_STAGES;
            // this group's steps of a block are quarters grp and grp + 2: wait for the bytes at the first; after the second,
            // release the buffer and -- once all 256 threads have released it -- refill it with the block after next
            if ((k & 3) == grp && !pb_mbar_wait(&raw_full[rs], (kb / TC_RAW_STAGES) & 1, p.status, PB_DEV_TC_TIMEOUT)) { ok = false; break; }
            TcRaw cur;
            tc_load_raw(cur, pb_smem_u32(raw + (size_t)rs * TC_RAW_BYTES) + (uint32_t)row * 136u, k & 3, live);
            if ((k & 3) == grp + 2) {
                pb_mbar_arrive(&raw_empty[rs]);
                if (kb + 2 < nkb) {
                    if (!pb_mbar_wait(&raw_empty[rs], (kb / TC_RAW_STAGES) & 1, p.status, PB_DEV_TC_TIMEOUT)) { ok = false; break; }
                    issue_raw(kb + 2);
                }
            }
            if (k >= TC_STAGES && !pb_mbar_wait(&empty[st], ((k / TC_STAGES) - 1) & 1, p.status, PB_DEV_TC_TIMEOUT)) { ok = false; break; }
            tc_decode_store(cur, k, tmem + ((uint32_t)((warp & 3) * 32) << 16) + TC_ACC_COLS + (uint32_t)st * TC_A_COLS, shift);
            tc_fence_before();                    // the stores are complete (wait::st); order them before the MMA warp's instructions
            pb_mbar_arrive(&full[st]);
        }
        // ---- epilogue: warp w reads lanes 32 (w % 4) .. + 31 (its rows); warps 0-3 take tokens below 64, 4-7 the rest; columns
        //      [0, np) hold the high parts' sums, [np, 2 np) the low parts'
        if (ok && pb_mbar_wait(acc_full, 0, p.status, PB_DEV_TC_TIMEOUT)) {
            tc_fence_after();
            for (int c0 = grp * (TC_NBLK / 2); c0 < (grp + 1) * (TC_NBLK / 2) && c0 < np; c0 += 32) {
                uint32_t v[32], vl[32];
                tc_ld32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)c0, v);
                tc_ld32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(np + c0), vl);
                if (live) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int b = c0 + j;
                        if (b < nt) {
                            float* dst = p.y + (size_t)(tb * TC_NBLK + b) * p.ldy + p.seg[s].yoff + r0 + row;
                            const float o = (__uint_as_float(v[j]) + __uint_as_float(vl[j])) * (unshift * xinv[b]);
                            *dst = p.accumulate ? *dst + o : o;
                        }
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");   // (error paths) no copy of this thread is still in flight when the CTA exits
    tc_fence_before();
    __syncthreads();
    if (warp == TC_DECODERS + 1) { tc_fence_after(); tc_dealloc(tmem, TC_TMEM_COLS); }
}

bool pb_gemmtc_supported(int type, int cols, int t) { return type == PB_T_IQ3_S && t >= 16 && cols % 256 == 0 && cols >= 256; }

// Fewest tokens the dispatchers send here.  The kernel works from 16 tokens on, but a CTA walks the whole contraction on
// its own (about 30 us for 2048 columns whatever the token count), so below ~32 tokens the warp-level kernel, which cuts
// the tokens into tiles of 16 over all SMs, is faster: measured 17 vs 36 us at 16 tokens and 42 vs 40 us at 64 tokens on
// a 4096 x 2048 matrix.  PYRE_B200_TC_MIN overrides (tests run the kernel at 16).
int pb_gemmtc_min_tokens() {
    const char* e = getenv("PYRE_B200_TC_MIN");
    const int v = e ? atoi(e) : 32;
    return v < 16 ? 16 : v;
}

int pb_gemmtc_max_tokens(int cols) {
    const size_t n = (PB_XH_BYTES - TC_XT_HEAD) / ((size_t)cols * 4) / TC_NBLK * TC_NBLK;
    return (int)(n < TC_XT_HEAD / 4 ? n : TC_XT_HEAD / 4);
}

int pb_launch_gemmtc(pb_ctx* ctx, const PbGemvQArgs& a) {
    if (!pb_gemmtc_supported(a.type, a.cols, a.t)) PB_FAIL(ctx, PB_UNSUPPORTED, "tensor-core gemm: type %d cols %d t %d", a.type, a.cols, a.t);
    if (a.mode == PB_ACT_PREQ) PB_FAIL(ctx, PB_UNSUPPORTED, "tensor-core gemm: pre-split activations are not accepted");
    if (a.mode == PB_ACT_GNORM && a.head_dim != 128) PB_FAIL(ctx, PB_UNSUPPORTED, "tensor-core gemm: gated norm over heads of %d (128 is built)", a.head_dim);
    if (((uintptr_t)a.x & 15) || (a.ldx & 3)) PB_FAIL(ctx, PB_ERR_ARG, "tensor-core gemm: activations must be 16-byte aligned");
    if (a.nseg < 1 || a.nseg > 4) PB_FAIL(ctx, PB_ERR_ARG, "tensor-core gemm: %d segments", a.nseg);
    for (int sg = 0; sg < a.nseg; sg++) if (!a.seg[sg].wr) PB_FAIL(ctx, PB_UNSUPPORTED, "tensor-core gemm: segment %d has no re-coded copy", sg);
    const int nblk = (a.t + TC_NBLK - 1) / TC_NBLK;
    const size_t need = TC_XT_HEAD + (size_t)nblk * TC_NBLK * a.cols * 4;
    if ((size_t)a.t * 4 > TC_XT_HEAD || need > PB_XH_BYTES) PB_FAIL(ctx, PB_UNSUPPORTED, "tensor-core gemm: %d tokens of %d columns exceed the %zu-byte operand buffer", a.t, a.cols, (size_t)PB_XH_BYTES);
    {
        PbGemvQParams q;
        memset(&q, 0, sizeof q);
        q.bpr = a.cols / 256; q.x = a.x; q.ldx = a.ldx; q.t = a.t; q.mode = a.mode; q.norm_w = a.norm_w; q.z = a.z; q.ldz = a.ldz; q.head_dim = a.head_dim; q.eps = a.eps;
        pb_launch_k(ctx, pb_xt_prep_kernel, dim3((nblk - 1) * TC_NBLK + pb_xt_np(a.t, nblk - 1)), dim3(256), (size_t)0, q, ctx->xh_buf);
        ctx->kernels_launched++;
        PB_CUDA(ctx, cudaGetLastError());
    }
    TcParams p;
    memset(&p, 0, sizeof p);
    p.nseg = a.nseg; p.row_bytes = a.cols / 256 * 136; p.cols = a.cols; p.t = a.t; p.xt = ctx->xh_buf; p.y = a.y; p.ldy = a.ldy; p.accumulate = a.accumulate; p.status = ctx->dev_status;
    int ntiles = 0;
    for (int sg = 0; sg < a.nseg; sg++) {
        p.seg[sg].w = a.seg[sg].wr; p.seg[sg].rows = (int)a.seg[sg].rows; p.seg[sg].yoff = (int)a.seg[sg].yoff; p.seg[sg].chunk0 = ntiles;
        ntiles += (int)((a.seg[sg].rows + TC_ROWS - 1) / TC_ROWS);
    }
    p.ntiles = ntiles;
    if (ntiles == 0) return PB_OK;
    const size_t smem = 1024 + (size_t)TC_STAGES * TC_B_BYTES + (size_t)TC_RAW_STAGES * TC_RAW_BYTES;
    auto kern = pb_gemmtc_iq3s_kernel;
    PB_TRY(pb_ensure_smem(ctx, kern, smem));
    pb_launch_k(ctx, kern, dim3(ntiles, nblk), dim3(TC_THREADS), smem, p);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
