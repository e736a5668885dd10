// Expert-parallel exchange: one NCCL communicator per context, loaded lazily with dlopen so that
// single-GPU users need no NCCL at all.
//
// The reference splits experts between a VRAM cache and a CPU pool (XCache / routed_pool_ord,
// src/model/qwen4exp_gguf.rs:66-72, 1803-1922).  Here GPU r of N holds experts
// [r*n_exp/N, (r+1)*n_exp/N) of every layer, activations and dense weights are replicated, and
// one exchange per MoE block makes every rank's partial outputs part[token][slot][d] complete.
// Each (token, slot) element is produced by exactly one rank and is zero on the others, so an
// all-reduce(sum) is an exact gather: results are bit-identical for every GPU count.
// A state made with pb_state_create_sharded instead keeps only this rank's sequences (attention,
// DeltaNet and dense layers run on them alone); its MoE blocks all-gather the residual rows of all
// ranks, compute the local experts for every token, and reduce-scatter the partial rows back to
// the tokens' owners -- the same exact sum, 1/N of the dense work per rank.
#include "pb_internal.h"

#include <dlfcn.h>
#include <stdio.h>

typedef struct { char internal[128]; } pb_nccl_id;
typedef void* pb_nccl_comm;
typedef int (*fn_get_id)(pb_nccl_id*);
typedef int (*fn_init_rank)(pb_nccl_comm*, int, pb_nccl_id, int);
typedef int (*fn_destroy)(pb_nccl_comm);
typedef int (*fn_allreduce)(const void*, void*, size_t, int, int, pb_nccl_comm, cudaStream_t);
typedef int (*fn_allgather)(const void*, void*, size_t, int, pb_nccl_comm, cudaStream_t);
typedef int (*fn_reducescatter)(const void*, void*, size_t, int, int, pb_nccl_comm, cudaStream_t);
typedef const char* (*fn_errstr)(int);

static struct {
    void* lib = nullptr;
    fn_get_id get_id = nullptr; fn_init_rank init_rank = nullptr; fn_destroy destroy = nullptr; fn_allreduce allreduce = nullptr; fn_allgather allgather = nullptr; fn_reducescatter reducescatter = nullptr; fn_errstr errstr = nullptr;
} g_nccl;

static int load_nccl(pb_ctx* ctx) {
    if (g_nccl.lib) return PB_OK;
    // RTLD_NOLOAD first: reuse the NCCL a host program (e.g. torch) already mapped
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) PB_FAIL(ctx, PB_UNSUPPORTED, "expert parallelism needs libnccl.so.2: %s", dlerror());
    g_nccl.get_id = (fn_get_id)dlsym(h, "ncclGetUniqueId");
    g_nccl.init_rank = (fn_init_rank)dlsym(h, "ncclCommInitRank");
    g_nccl.destroy = (fn_destroy)dlsym(h, "ncclCommDestroy");
    g_nccl.allreduce = (fn_allreduce)dlsym(h, "ncclAllReduce");
    g_nccl.allgather = (fn_allgather)dlsym(h, "ncclAllGather");
    g_nccl.reducescatter = (fn_reducescatter)dlsym(h, "ncclReduceScatter");
    g_nccl.errstr = (fn_errstr)dlsym(h, "ncclGetErrorString");
    if (!g_nccl.get_id || !g_nccl.init_rank || !g_nccl.destroy || !g_nccl.allreduce || !g_nccl.allgather || !g_nccl.reducescatter) PB_FAIL(ctx, PB_UNSUPPORTED, "libnccl.so.2 lacks a required symbol");
    g_nccl.lib = h;
    return PB_OK;
}

#define PB_NCCL(ctx, call)                                                                                                   \
    do {                                                                                                                     \
        int _r = (call);                                                                                                     \
        if (_r != 0) PB_FAIL(ctx, PB_ERR_CUDA, "%s: %s", #call, g_nccl.errstr ? g_nccl.errstr(_r) : "nccl error");           \
    } while (0)

extern "C" {

int pb_ep_unique_id(pb_ctx* ctx, void* id128) {
    if (!ctx || !id128) return PB_ERR_ARG;
    PB_TRY(load_nccl(ctx));
    pb_nccl_id id;
    PB_NCCL(ctx, g_nccl.get_id(&id));
    memcpy(id128, &id, 128);
    return PB_OK;
}

int pb_ep_init(pb_ctx* ctx, const void* id128, int rank, int world) {
    if (!ctx || !id128) return PB_ERR_ARG;
    if (world < 1 || rank < 0 || rank >= world) PB_FAIL(ctx, PB_ERR_ARG, "pb_ep_init: rank %d of %d", rank, world);
    if (ctx->ep_comm) PB_FAIL(ctx, PB_ERR_STATE, "pb_ep_init: already initialised");
    PB_TRY(load_nccl(ctx));
    PB_CUDA(ctx, cudaSetDevice(ctx->device));
    pb_nccl_id id;
    memcpy(&id, id128, 128);
    pb_nccl_comm comm = nullptr;
    PB_NCCL(ctx, g_nccl.init_rank(&comm, world, id, rank));
    ctx->ep_comm = comm; ctx->ep_rank = rank; ctx->ep_world = world;
    return PB_OK;
}

int pb_ep_destroy(pb_ctx* ctx) {
    if (!ctx) return PB_ERR_ARG;
    if (ctx->ep_comm) { cudaStreamSynchronize(ctx->stream); g_nccl.destroy(ctx->ep_comm); ctx->ep_comm = nullptr; ctx->ep_world = 1; ctx->ep_rank = 0; }
    return PB_OK;
}

}  // extern "C"

// in-place sum of n floats over the expert-parallel group, on the context's stream
int pb_ep_allreduce(pb_ctx* ctx, float* buf, size_t n) {
    if (!ctx->ep_comm) PB_FAIL(ctx, PB_ERR_STATE, "expert-parallel model without pb_ep_init");
    PB_NCCL(ctx, g_nccl.allreduce(buf, buf, n, /*ncclFloat32*/ 7, /*ncclSum*/ 0, ctx->ep_comm, ctx->stream));
    return PB_OK;
}

// recv[r * n .. (r + 1) * n) = rank r's send[0 .. n), on the context's stream
int pb_ep_allgather(pb_ctx* ctx, const float* send, float* recv, size_t n) {
    if (!ctx->ep_comm) PB_FAIL(ctx, PB_ERR_STATE, "expert-parallel model without pb_ep_init");
    PB_NCCL(ctx, g_nccl.allgather(send, recv, n, /*ncclFloat32*/ 7, ctx->ep_comm, ctx->stream));
    return PB_OK;
}
// recv[0 .. n) = sum over ranks of their send[rank * n .. (rank + 1) * n)
int pb_ep_reduce_scatter(pb_ctx* ctx, const float* send, float* recv, size_t n) {
    if (!ctx->ep_comm) PB_FAIL(ctx, PB_ERR_STATE, "expert-parallel model without pb_ep_init");
    PB_NCCL(ctx, g_nccl.reducescatter(send, recv, n, /*ncclFloat32*/ 7, /*ncclSum*/ 0, ctx->ep_comm, ctx->stream));
    return PB_OK;
}
