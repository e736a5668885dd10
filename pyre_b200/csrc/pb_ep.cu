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
#include "pb_common.cuh"
#include "pb_internal.h"
#include "pb_ep.cuh"

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

// ------------------------------------------------------------------------------------ peer exchange inside kernels
//
// NCCL's all-gather + reduce-scatter cost about 25 us per call at these sizes (10 KB - 330 KB), twice per MoE block.  With
// every rank's exchange buffers mapped into every rank, the same hand-over is a few stores over NVLink and a flag:
//   rows     each rank stores the residual rows + router logits of its tokens into every rank's gathered-row buffer;
//   partials the expert-down kernel stores every finished (token, slot) row into the memory of the token's owner: each row has
//            exactly one producer, so what the owner sums is independent of the GPU count, as with the reduce-scatter;
//   flags    flags[kind][src] in the receiver's memory = sequence number of the last exchange that src completed.  The
//            writer orders its stores before the flag with a system-scope fence, the reader polls with system-scope acquire
//            loads.  Waits are bounded (about a second); a rank whose peer never arrives records PB_DEV_PEER_TIMEOUT and its
//            call returns PB_ERR_DEVICE (the reference's pyre_wait_flag does the same for its CPU/GPU hand-shake,
//            src/model/qwen4exp_gguf.rs:229-238).
// Only plain loads and stores touch peer memory (no bulk copy engine reads or writes it).

// grid = world CTAs of 256 threads: CTA p serves rank p
__global__ void __launch_bounds__(256) pb_ep_push_rows_kernel(const PbEpExch x, const float* __restrict__ rows, int64_t n, int64_t dst_off, int exch) {
    const int p = blockIdx.x;
    pb_pdl_wait();
    pb_pdl_trigger();
    float4* dst = reinterpret_cast<float4*>(x.peer_xg[p] + dst_off);
    const float4* src = reinterpret_cast<const float4*>(rows);
    for (int64_t i = threadIdx.x; i < n / 4; i += blockDim.x) dst[i] = src[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) pb_ep_handshake(x, p, 0, *x.seq_base + (unsigned long long)exch + 1);
}

__global__ void __launch_bounds__(32) pb_ep_signal_wait_kernel(const PbEpExch x, int kind, int exch) {
    pb_pdl_wait();      // the stores of the preceding kernel into peer memory are complete
    pb_pdl_trigger();
    if (threadIdx.x == 0) pb_ep_handshake(x, blockIdx.x, kind, *x.seq_base + (unsigned long long)exch + 1);
}

int pb_launch_ep_push_rows(pb_ctx* ctx, const PbEpExch& x, const float* rows, int64_t n, int64_t dst_off, int exch) {
    if ((n & 3) || (dst_off & 3)) PB_FAIL(ctx, PB_ERR_ARG, "peer exchange: row block of %lld floats at offset %lld is not 16-byte granular", (long long)n, (long long)dst_off);
    pb_launch_k(ctx, pb_ep_push_rows_kernel, dim3(x.world), dim3(256), (size_t)0, x, rows, n, dst_off, exch);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
int pb_launch_ep_signal_wait(pb_ctx* ctx, const PbEpExch& x, int kind, int exch) {
    pb_launch_k(ctx, pb_ep_signal_wait_kernel, dim3(x.world), dim3(32), (size_t)0, x, kind, exch);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

// One block of device memory per rank with the same layout everywhere, mapped into every rank of the node.  Collective:
// every rank of the group calls it at the same point (the handles travel through one NCCL all-gather).
int pb_ep_symm_alloc(pb_ctx* ctx, size_t bytes, PbEpSymm* out) {
    if (!ctx->ep_comm) PB_FAIL(ctx, PB_ERR_STATE, "peer exchange without pb_ep_init");
    if (ctx->ep_world > PB_EP_MAX_WORLD) PB_FAIL(ctx, PB_UNSUPPORTED, "peer exchange over %d ranks (at most %d)", ctx->ep_world, PB_EP_MAX_WORLD);
    const int world = ctx->ep_world, rank = ctx->ep_rank;
    PB_CUDA(ctx, cudaMalloc(&out->local, bytes));
    PB_CUDA(ctx, cudaMemsetAsync(out->local, 0, bytes, ctx->stream));
    out->bytes = bytes;
    cudaIpcMemHandle_t mine;
    PB_CUDA(ctx, cudaIpcGetMemHandle(&mine, out->local));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handles travel as 16 floats");
    float* hbuf = nullptr;
    PB_CUDA(ctx, cudaMalloc(&hbuf, (size_t)world * 64));
    PB_CUDA(ctx, cudaMemcpyAsync(reinterpret_cast<char*>(hbuf) + (size_t)rank * 64, &mine, 64, cudaMemcpyHostToDevice, ctx->stream));
    int rc = pb_ep_allgather(ctx, hbuf + (size_t)rank * 16, hbuf, 16);
    std::vector<cudaIpcMemHandle_t> all((size_t)world);
    if (rc == PB_OK && cudaMemcpyAsync(all.data(), hbuf, (size_t)world * 64, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess) rc = PB_ERR_CUDA;
    if (rc == PB_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = PB_ERR_CUDA;
    cudaFree(hbuf);
    if (rc != PB_OK) { cudaFree(out->local); out->local = nullptr; PB_FAIL(ctx, rc, "peer exchange: the memory handles could not be gathered"); }
    for (int p = 0; p < world; p++) {
        if (p == rank) { out->peer[p] = out->local; continue; }
        cudaError_t e = cudaIpcOpenMemHandle(&out->peer[p], all[p], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < p; q++) if (q != rank && out->peer[q]) cudaIpcCloseMemHandle(out->peer[q]);
            cudaFree(out->local); out->local = nullptr;
            PB_FAIL(ctx, PB_UNSUPPORTED, "peer exchange: rank %d's memory cannot be mapped (%s)", p, cudaGetErrorString(e));
        }
    }
    return PB_OK;
}
void pb_ep_symm_free(pb_ctx* ctx, PbEpSymm* m) {
    if (!m->local) return;
    for (int p = 0; p < ctx->ep_world && p < PB_EP_MAX_WORLD; p++) if (m->peer[p] && m->peer[p] != m->local) cudaIpcCloseMemHandle(m->peer[p]);
    cudaFree(m->local);
    m->local = nullptr;
}

extern "C" {
// Failure-detection probe: one hand-shake, with a limit of `spins` polls, whose partner never answers (the flag it waits for
// lives in a zeroed array that nobody writes).  The kernel must give up, the call must return PB_ERR_DEVICE, and the context
// must stay usable.  No GPU is faulted: the wait simply runs out.
int pb_ep_probe_wait_timeout(pb_ctx* ctx, unsigned int spins) {
    if (!ctx) return PB_ERR_ARG;
    PB_TRY(pb_enter(ctx));
    unsigned long long* mem = nullptr;
    PB_CUDA(ctx, cudaMalloc(&mem, 1024));
    PB_CUDA(ctx, cudaMemsetAsync(mem, 0, 1024, ctx->stream));
    PbEpExch x; memset(&x, 0, sizeof x);
    x.rank = 1; x.world = 2;                       // "rank 1 of 2": CTA 0 announces to rank 0 and waits for rank 0's flag
    x.peer_flags[0] = mem + 32; x.peer_flags[1] = mem + 64;   // both arrays are local; nothing ever writes mem[64 ..)
    x.seq_base = mem; x.spin_limit = spins; x.status = ctx->dev_status;
    pb_launch_k(ctx, pb_ep_signal_wait_kernel, dim3(1), dim3(32), (size_t)0, x, 0, 0);
    const int rc = pb_sync_check(ctx, "pb_ep_probe_wait_timeout");
    cudaFree(mem);
    return rc;
}
}
