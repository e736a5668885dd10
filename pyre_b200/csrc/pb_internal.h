// Internal definitions shared by the .cu files of libpyre_b200.so (not part of the C ABI).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>
#include <vector>

#include "../../include/pyre_b200.h"

struct pb_ctx {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;   // the stream every kernel of this context is launched on
    int* dev_status = nullptr;       // device status word (see PB_DEV_* in pb_common.cuh)
    int* host_status = nullptr;      // pinned host mirror, filled by an async copy before each sync
    int sm_count = 148;
    int max_smem_optin = 0;
    std::string err;
    // grow-only device scratch for host-buffer entry points
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    uint64_t kernels_launched = 0;
};

struct pb_qmat {
    pb_ctx* ctx = nullptr;
    int type = 0;
    int64_t rows = 0, cols = 0;
    int64_t row_bytes = 0;
    uint8_t* data = nullptr;   // device, 256-byte aligned, padded by >= 256 bytes past the last row
    size_t nbytes = 0;         // rows * row_bytes
    bool owns = true;          // false for row-range views into another matrix
};

#define PB_FAIL(ctx, code, ...)                                   \
    do {                                                          \
        char _b[512];                                             \
        snprintf(_b, sizeof _b, __VA_ARGS__);                     \
        if (ctx) (ctx)->err = _b;                                 \
        return (code);                                            \
    } while (0)

#define PB_CUDA(ctx, call)                                                                                   \
    do {                                                                                                     \
        cudaError_t _e = (call);                                                                             \
        if (_e != cudaSuccess) PB_FAIL(ctx, _e == cudaErrorMemoryAllocation ? PB_ERR_OOM : PB_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(_e)); \
    } while (0)

#define PB_TRY(call)                 \
    do {                             \
        int _s = (call);             \
        if (_s != PB_OK) return _s;  \
    } while (0)

int pb_scratch(pb_ctx* ctx, size_t bytes, void** out);
int pb_sync_check(pb_ctx* ctx, const char* who);

// pb_dequant.cu
int pb_launch_dequant(pb_ctx* ctx, int type, const uint8_t* w, int64_t nsteps, float* out);
int pb_launch_synth(pb_ctx* ctx, int type, uint8_t* w, int64_t nblocks, uint64_t seed, uint64_t tid);
int pb_launch_synth_normal(pb_ctx* ctx, float* out, int64_t n, uint64_t seed, uint64_t tid, float sigma);

// pb_gemv.cu
struct PbGemvArgs {
    const uint8_t* w;   // first row of the matrix (16-byte aligned)
    int type;
    int64_t rows;
    int cols;
    const float* x;     // [t][ldx]
    int64_t ldx;
    int t;              // 1..16 columns
    float* y;           // [t][ldy]
    int64_t ldy;
};
int pb_launch_gemv(pb_ctx* ctx, const PbGemvArgs& a);
