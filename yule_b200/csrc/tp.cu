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
#include <vector>

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

// ── peer-memory exchange ────────────────────────────────────────────────────────────────────
// NCCL's all-gather costs ~20 µs for the few KB a decode step exchanges, 4 times per layer; at batch
// 1 that is more than the matvecs it separates.  The runner therefore keeps the gathered activation
// buffers in one "exchange" allocation per rank that every peer maps (cudaIpc, over NVLink), and an
// all-gather becomes: each rank stores its slice straight into every peer's copy, fences, and
// publishes an epoch number in the peer's flag word; it then waits — for a bounded time — until its
// own flag words show the same epoch from every peer.  Plain stores and volatile loads only.
namespace {

constexpr int kMaxRanks = 8;
constexpr int kFlagSlots = 8;
constexpr int kXchgThreads = 256;

struct PeerTable {
    float *base[kMaxRanks];  // peer r's exchange region as mapped into this process (own region for r = rank)
};

// Flags live at the end of the exchange region: [slot][source rank] epochs, then one CTA counter.
__device__ __forceinline__ uint32_t *flags_of(float *base, size_t flag_offset_floats) {
    return reinterpret_cast<uint32_t *>(base + flag_offset_floats);
}

__global__ void __launch_bounds__(kXchgThreads)
tp_exchange_kernel(PeerTable peers, size_t buf_offset, uint32_t per_rank, uint32_t rank, uint32_t world,
                   size_t flag_offset, uint32_t slot, const uint32_t *__restrict__ tick, uint32_t epochs_per_tick,
                   uint32_t epoch_index, int *__restrict__ status, long long wait_cycles, uint32_t n_rows, size_t row_stride) {
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    // One epoch per (token, exchange): the token counter only changes in another kernel, so every
    // CTA of every rank computes the same number.
    const uint32_t epoch = *tick * epochs_per_tick + epoch_index + 1u;
    float *mine = peers.base[rank] + buf_offset + (size_t)rank * per_rank;
    // push this rank's slice into every peer's copy of the buffer; with n_rows > 1 the buffer is a matrix
    // [n_rows][row_stride] and the slice the column block [rank·per_rank, (rank+1)·per_rank) of every row
    const uint32_t n4 = per_rank / 4;
    const size_t total4 = (size_t)n4 * n_rows;
    for (uint32_t p = 0; p < world; p++) {
        if (p == rank) continue;
        float *dst_base = peers.base[p] + buf_offset + (size_t)rank * per_rank;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
            const size_t row = i / n4, c4 = i - row * n4;
            reinterpret_cast<float4 *>(dst_base + row * row_stride)[c4] = reinterpret_cast<const float4 *>(mine + row * row_stride)[c4];
        }
    }
    __threadfence_system();
    __syncthreads();
    __shared__ uint32_t s_last;
    uint32_t *my_flags = flags_of(peers.base[rank], flag_offset);
    uint32_t *counter = my_flags + kFlagSlots * kMaxRanks;
    if (threadIdx.x == 0) s_last = (atomicAdd(counter, 1u) == gridDim.x - 1) ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    // every CTA's stores are fenced: publish, then wait for the peers' slices
    __threadfence_system();
    if (threadIdx.x < world && threadIdx.x != rank) {
        volatile uint32_t *theirs = flags_of(peers.base[threadIdx.x], flag_offset) + slot * kMaxRanks + rank;
        *theirs = epoch;
    }
    if (threadIdx.x == 0) *counter = 0;
    if (threadIdx.x < world && threadIdx.x != rank) {
        volatile uint32_t *f = my_flags + slot * kMaxRanks + threadIdx.x;
        const long long t0 = clock64();
        // bounded: a peer that never arrives leaves a status word for the host instead of a hung GPU; once any
        // wait of this context has given up, later ones return at once
        while ((int32_t)(*f - epoch) < 0) {
            if (*reinterpret_cast<volatile int *>(status) != 0) break;
            if (clock64() - t0 > wait_cycles) {
                atomicCAS(status, 0, kStatusPeerTimeout);
                break;
            }
        }
    }
    __threadfence_system();
}

}  // namespace

cudaError_t tp_exchange(yule_cuda_ctx *ctx, size_t buf_offset_floats, uint32_t per_rank, uint32_t slot,
                        const uint32_t *tick, uint32_t epochs_per_tick, uint32_t epoch_index, bool pdl, uint64_t *launches,
                        uint32_t n_rows, size_t row_stride) {
    PeerTable pt;
    for (int i = 0; i < kMaxRanks; i++) pt.base[i] = ctx->tp_peer_base[i];
    // a few CTAs for a vector; a matrix of rows gets one CTA per 16 KB of payload, up to one per SM
    const size_t total4 = (size_t)(per_rank / 4) * n_rows;
    size_t want = (total4 + kXchgThreads * 4 - 1) / (kXchgThreads * 4);
    uint32_t grid = (uint32_t)(want < 1 ? 1 : (n_rows <= 1 ? (want > 8 ? 8 : want) : (want > 148 ? 148 : want)));
    const long long wait_cycles = ctx->wait_cycles;
    *launches += 1;
    return launch_kernel(tp_exchange_kernel, dim3(grid), dim3(kXchgThreads), 0, ctx->stream, pdl, pt, buf_offset_floats,
                         per_rank, ctx->tp_rank, ctx->tp_world, ctx->tp_flag_offset, slot, tick, epochs_per_tick,
                         epoch_index, ctx->device_status, wait_cycles, n_rows, row_stride);
}

// Allocates this rank's exchange region (n_floats of payload + flags), maps every peer's, and
// returns the local base.  Handles travel through one NCCL all-gather, so no other channel between
// the processes is needed.
int32_t tp_setup_exchange(yule_cuda_ctx *ctx, size_t n_floats, float **out_base) {
    if (ctx->tp_world <= 1 || !ctx->tp_comm) return fail(YULE_ERR_INVALID_ARGUMENT, "tensor parallelism is not initialised");
    if (ctx->tp_world > (uint32_t)kMaxRanks) return fail(YULE_ERR_INVALID_ARGUMENT, "at most %d ranks", kMaxRanks);
    if (ctx->tp_peer_base[ctx->tp_rank]) return fail(YULE_ERR_INVALID_ARGUMENT, "exchange region already set up on this context");
    const size_t payload = (n_floats + 63) & ~(size_t)63;
    const size_t bytes = payload * sizeof(float) + (kFlagSlots * kMaxRanks + 64) * sizeof(uint32_t);
    float *base = nullptr;
    YULE_CUDA_TRY(cudaMalloc((void **)&base, bytes));
    YULE_CUDA_TRY(cudaMemset(base, 0, bytes));
    cudaIpcMemHandle_t mine;
    YULE_CUDA_TRY(cudaIpcGetMemHandle(&mine, base));
    // all-gather the 64-byte handles on the device
    unsigned char *d_handles = nullptr;
    YULE_CUDA_TRY(cudaMalloc((void **)&d_handles, sizeof(mine) * ctx->tp_world));
    YULE_CUDA_TRY(cudaMemcpy(d_handles + sizeof(mine) * ctx->tp_rank, &mine, sizeof(mine), cudaMemcpyHostToDevice));
    int rc = g_nccl.AllGather(d_handles + sizeof(mine) * ctx->tp_rank, d_handles, sizeof(mine), /*ncclChar*/ 0, ctx->tp_comm,
                              ctx->stream);
    if (rc != 0) return nccl_fail(rc, "ncclAllGather of the exchange handles");
    YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    std::vector<cudaIpcMemHandle_t> all(ctx->tp_world);
    YULE_CUDA_TRY(cudaMemcpy(all.data(), d_handles, sizeof(mine) * ctx->tp_world, cudaMemcpyDeviceToHost));
    YULE_CUDA_TRY(cudaFree(d_handles));
    for (uint32_t p = 0; p < ctx->tp_world; p++) {
        if (p == ctx->tp_rank) {
            ctx->tp_peer_base[p] = base;
            continue;
        }
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return fail_cuda(e, "cudaIpcOpenMemHandle of a peer's exchange region");
        ctx->tp_peer_base[p] = (float *)ptr;
    }
    ctx->tp_flag_offset = payload;
    ctx->tp_xchg_floats = payload;
    *out_base = base;
    return YULE_OK;
}

// Gives the exchange region back when the runner that used it goes away, so that another runner can be created on
// the same context.  Collective: every rank unmaps its peers' regions, all ranks meet (a one-byte all-gather on
// the communicator), and only then does each free its own — a region must not be freed while a peer still has it
// mapped.  The caller has synchronised its stream, so nothing of this rank still touches the regions.
int32_t tp_release_exchange(yule_cuda_ctx *ctx) {
    if (!tp_has_exchange(ctx)) return YULE_OK;
    float *mine = ctx->tp_peer_base[ctx->tp_rank];
    for (uint32_t p = 0; p < (uint32_t)kMaxRanks; p++) {
        if (ctx->tp_peer_base[p] && p != ctx->tp_rank) cudaIpcCloseMemHandle(ctx->tp_peer_base[p]);
        ctx->tp_peer_base[p] = nullptr;
    }
    unsigned char *d = nullptr;
    if (ctx->tp_comm && cudaMalloc((void **)&d, ctx->tp_world) == cudaSuccess) {
        g_nccl.AllGather(d + ctx->tp_rank, d, 1, /*ncclChar*/ 0, ctx->tp_comm, ctx->stream);
        cudaStreamSynchronize(ctx->stream);
        cudaFree(d);
    }
    cudaFree(mine);
    ctx->tp_flag_offset = ctx->tp_xchg_floats = 0;
    return YULE_OK;
}

void tp_fuse_push(const yule_cuda_ctx *ctx, size_t pair_offset_floats, uint32_t per_rank, const uint32_t *tick,
                  uint32_t epochs_per_tick, uint32_t index, TpFuse *f) {
    f->world = ctx->tp_world;
    f->rank = ctx->tp_rank;
    f->tick = tick;
    f->epochs_per_tick = epochs_per_tick;
    f->status = ctx->device_status;
    f->wait_cycles = ctx->wait_cycles;
    f->push = true;
    f->push_index = index;
    for (uint32_t p = 0; p < (uint32_t)kMaxRanks; p++)
        f->pair_out[p] = p < ctx->tp_world
                             ? reinterpret_cast<uint2 *>(ctx->tp_peer_base[p] + pair_offset_floats) + (size_t)ctx->tp_rank * per_rank
                             : nullptr;
}

void tp_fuse_wait(const yule_cuda_ctx *ctx, size_t pair_offset_floats, const uint32_t *tick, uint32_t epochs_per_tick,
                  uint32_t index, TpFuse *f) {
    f->world = ctx->tp_world;
    f->rank = ctx->tp_rank;
    f->tick = tick;
    f->epochs_per_tick = epochs_per_tick;
    f->status = ctx->device_status;
    f->wait_cycles = ctx->wait_cycles;
    f->wait = true;
    f->wait_index = index;
    f->pair_in = reinterpret_cast<const uint2 *>(ctx->tp_peer_base[ctx->tp_rank] + pair_offset_floats);
}

bool tp_has_exchange(const yule_cuda_ctx *ctx) { return ctx->tp_world > 1 && ctx->tp_peer_base[ctx->tp_rank] != nullptr; }

// In-place all-gather of fp32: every rank's slice of `count` floats already sits at
// buf + rank*count; afterwards all ranks hold all slices.  Enqueued on the context's stream
// (capturable into a CUDA graph).
cudaError_t tp_all_gather_inplace(yule_cuda_ctx *ctx, float *buf, size_t count) {
    if (ctx->tp_world <= 1) return cudaSuccess;
    int rc = g_nccl.AllGather(buf + (size_t)ctx->tp_rank * count, buf, count, /*ncclFloat*/ 7, ctx->tp_comm, ctx->stream);
    return rc == 0 ? cudaSuccess : cudaErrorUnknown;
}

void tp_destroy(yule_cuda_ctx *ctx) {
    for (uint32_t p = 0; p < (uint32_t)kMaxRanks; p++) {
        if (!ctx->tp_peer_base[p]) continue;
        if (p == ctx->tp_rank)
            cudaFree(ctx->tp_peer_base[p]);
        else
            cudaIpcCloseMemHandle(ctx->tp_peer_base[p]);
        ctx->tp_peer_base[p] = nullptr;
    }
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

// Makes one bounded device-side wait run out on purpose, without a peer and without a fault: the waiting
// kernel polls memory that nothing ever writes, gives up after `budget_cycles`, records the status word and
// returns normally, and the synchronize at the end reports YULE_ERR_DEVICE_STATUS.  Single GPU.
//   which = 0  the Q4_K matvec as consumer of a gathered vector: its (value, epoch) pairs never arrive
//   which = 1  the exchange kernel: the stand-in peer (a second buffer on this GPU) never publishes its flag
int32_t yule_cuda_selftest_bounded_wait(yule_cuda_ctx *ctx, uint32_t which, uint64_t budget_cycles) {
    if (!ctx) return fail(YULE_ERR_INVALID_ARGUMENT, "null context");
    if (which > 1) return fail(YULE_ERR_INVALID_ARGUMENT, "unknown wait selector %u", which);
    if (ctx->tp_world > 1) return fail(YULE_ERR_INVALID_ARGUMENT, "the self-test runs on a context without tensor parallelism");
    YULE_CUDA_TRY(cudaSetDevice(ctx->device));
    YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    const uint32_t n_rows = 16, n_cols = 256, per_rank = 128;
    const size_t payload = 1024;  // floats: pairs of the 256-element vector, or the two 128-float slices
    const size_t region_bytes = payload * sizeof(float) + (kFlagSlots * kMaxRanks + 64) * sizeof(uint32_t);
    char *mem = nullptr;
    const size_t w_bytes = (size_t)n_rows * 144, total = 2 * region_bytes + w_bytes + 4096;
    YULE_CUDA_TRY(cudaMalloc((void **)&mem, total));
    cudaError_t e = cudaMemset(mem, 0, total);
    float *region_a = (float *)mem, *region_b = (float *)(mem + region_bytes);
    uint8_t *w = (uint8_t *)(mem + 2 * region_bytes);
    float *x = (float *)(mem + 2 * region_bytes + w_bytes), *out = x + n_cols;
    const uint32_t *tick = (const uint32_t *)(out + n_rows);  // stays 0: the awaited epoch is 1
    const long long budget = budget_cycles ? (long long)budget_cycles : ctx->wait_cycles;
    uint64_t launches = 0;
    if (e == cudaSuccess && which == 0) {
        Q4kFused f;
        f.w[0] = w;
        f.out[0] = out;
        f.rows[0] = n_rows;
        f.out_stride[0] = n_rows;
        f.x = x;
        f.x_stride = n_cols;
        f.n_cols = n_cols;
        f.status = ctx->device_status;
        f.wait_cycles = budget;
        f.tp.world = 2;
        f.tp.tick = tick;
        f.tp.epochs_per_tick = 1;
        f.tp.status = ctx->device_status;
        f.tp.wait_cycles = budget;
        f.tp.wait = true;
        f.tp.wait_index = 0;
        f.tp.pair_in = reinterpret_cast<const uint2 *>(region_a);
        e = launch_q4k_mma(f, ctx->prop.multiProcessorCount, ctx->stream, &launches);
    } else if (e == cudaSuccess) {
        const long long saved_budget = ctx->wait_cycles;
        ctx->tp_peer_base[0] = region_a;
        ctx->tp_peer_base[1] = region_b;
        ctx->tp_rank = 0;
        ctx->tp_world = 2;
        ctx->tp_flag_offset = payload;
        ctx->wait_cycles = budget;
        e = tp_exchange(ctx, 0, per_rank, 0, tick, 1, 0, false, &launches, 1, 0);
        ctx->tp_peer_base[0] = ctx->tp_peer_base[1] = nullptr;
        ctx->tp_world = 1;
        ctx->tp_flag_offset = 0;
        ctx->wait_cycles = saved_budget;
    }
    ctx->launches.fetch_add(launches);
    int32_t rc = e == cudaSuccess ? yule_cuda_synchronize(ctx) : fail_cuda(e, "bounded-wait self-test launch");
    cudaStreamSynchronize(ctx->stream);
    cudaFree(mem);
    return rc;
}

}  // extern "C"
