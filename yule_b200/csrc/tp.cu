// tp.cu — output-row tensor parallelism: one process per GPU, NCCL all-gather over NVLink.
//
// Every quantized linear computes out[row] = dot(dequant(W[row, :]), x): rows are independent, so
// rank r of N holds rows [r*n/N, (r+1)*n/N) of every matrix (a byte slice of the raw GGUF tensor)
// and the activations a later stage needs in full are all-gathered.  Yule has no multi-device code
// (no collective anywhere in the reference), so this file has no counterpart there; parity is
// "N-rank logits equal 1-rank logits".
//
// NCCL is reached through dlopen (the library the process already loaded, e.g. PyTorch's, or the
// system one) and the handful of stable entry points declared below, so libyule_cuda.so itself
// has no link-time dependency on it.  The rendezvous id is created by rank 0 and carried to the
// other ranks by the caller (torch.distributed, MPI, a file — anything).

#include <dlfcn.h>

#include <cstring>

#include "internal.h"

namespace yule {
namespace {

struct NcclApi {
    void *lib = nullptr;
    int (*GetUniqueId)(void *id) = nullptr;
    int (*CommInitRank)(void **comm, int nranks, NcclId id, int rank) = nullptr;
    int (*AllGather)(const void *send, void *recv, size_t count, int dtype, void *comm, cudaStream_t s) = nullptr;
    int (*CommDestroy)(void *comm) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
};
NcclApi g_nccl;
std::mutex g_nccl_mu;

int32_t load_nccl() {
    std::lock_guard<std::mutex> lock(g_nccl_mu);
    if (g_nccl.lib) return YULE_OK;
    const char *env = getenv("YULE_NCCL_LIBRARY");
    const char *names[] = {env, "libnccl.so.2", "libnccl.so"};
    void *lib = nullptr;
    for (const char *n : names) {
        if (!n || !*n) continue;
        lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (lib) break;
    }
    if (!lib) return fail(YULE_ERR_CUDA, "NCCL not found (set YULE_NCCL_LIBRARY to libnccl.so.2): %s", dlerror());
    NcclApi a;
    a.lib = lib;
    a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(lib, "ncclGetUniqueId");
    a.CommInitRank = (decltype(a.CommInitRank))dlsym(lib, "ncclCommInitRank");
    a.AllGather = (decltype(a.AllGather))dlsym(lib, "ncclAllGather");
    a.CommDestroy = (decltype(a.CommDestroy))dlsym(lib, "ncclCommDestroy");
    a.GetErrorString = (decltype(a.GetErrorString))dlsym(lib, "ncclGetErrorString");
    if (!a.GetUniqueId || !a.CommInitRank || !a.AllGather || !a.CommDestroy || !a.GetErrorString)
        return fail(YULE_ERR_CUDA, "the NCCL library lacks an expected entry point");
    g_nccl = a;
    return YULE_OK;
}

int32_t nccl_fail(int rc, const char *what) {
    return fail(YULE_ERR_CUDA, "nccl: %s failed: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?");
}

}  // namespace

// In-place all-gather of fp32: every rank's slice of `count` floats already sits at
// buf + rank*count; afterwards all ranks hold all slices.  Enqueued on the context's stream
// (capturable into a CUDA graph).
cudaError_t tp_all_gather_inplace(yule_cuda_ctx *ctx, float *buf, size_t count) {
    if (ctx->tp_world <= 1) return cudaSuccess;
    int rc = g_nccl.AllGather(buf + (size_t)ctx->tp_rank * count, buf, count, /*ncclFloat*/ 7, ctx->tp_comm, ctx->stream);
    return rc == 0 ? cudaSuccess : cudaErrorUnknown;
}

void tp_destroy(yule_cuda_ctx *ctx) {
    if (ctx->tp_comm && g_nccl.CommDestroy) g_nccl.CommDestroy(ctx->tp_comm);
    ctx->tp_comm = nullptr;
}

}  // namespace yule

using namespace yule;

extern "C" {

int32_t yule_cuda_tp_unique_id(uint8_t *out_id128) {
    if (!out_id128) return fail(YULE_ERR_INVALID_ARGUMENT, "null id buffer");
    int32_t rc = load_nccl();
    if (rc) return rc;
    NcclId id;
    int n = g_nccl.GetUniqueId(&id);
    if (n != 0) return nccl_fail(n, "ncclGetUniqueId");
    memcpy(out_id128, id.internal, 128);
    return YULE_OK;
}

int32_t yule_cuda_tp_init(yule_cuda_ctx *ctx, uint32_t rank, uint32_t world, const uint8_t *id128) {
    if (!ctx || !id128) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    if (world == 0 || rank >= world) return fail(YULE_ERR_INVALID_ARGUMENT, "rank %u outside world %u", rank, world);
    if (ctx->tp_comm) return fail(YULE_ERR_INVALID_ARGUMENT, "tensor parallelism already initialised on this context");
    YULE_CUDA_TRY(cudaSetDevice(ctx->device));
    ctx->tp_rank = rank;
    ctx->tp_world = world;
    if (world == 1) return YULE_OK;
    int32_t rc = load_nccl();
    if (rc) return rc;
    NcclId id;
    memcpy(id.internal, id128, 128);
    void *comm = nullptr;
    int n = g_nccl.CommInitRank(&comm, (int)world, id, (int)rank);
    if (n != 0) return nccl_fail(n, "ncclCommInitRank");
    ctx->tp_comm = comm;
    return YULE_OK;
}

int32_t yule_cuda_tp_all_gather(yule_cuda_ctx *ctx, yule_buffer buffer, size_t count_per_rank) {
    if (!ctx) return fail(YULE_ERR_INVALID_ARGUMENT, "null context");
    YULE_CUDA_TRY(cudaSetDevice(ctx->device));
    Buffer b;
    if (!ctx->find(buffer, &b, "tp_all_gather")) return YULE_ERR_UNKNOWN_BUFFER;
    const uint32_t world = ctx->tp_world ? ctx->tp_world : 1;
    if (b.size < count_per_rank * world * sizeof(float))
        return fail(YULE_ERR_OUT_OF_BOUNDS, "all-gather of %zu floats x %u ranks exceeds the %zu-byte buffer", count_per_rank,
                    world, b.size);
    cudaError_t e = tp_all_gather_inplace(ctx, (float *)b.ptr, count_per_rank);
    if (e != cudaSuccess) return fail(YULE_ERR_CUDA, "nccl: ncclAllGather failed");
    return YULE_OK;
}

}  // extern "C"
