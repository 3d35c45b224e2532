// qmv_q6k_ring.cu — Q6_K fused dequantise + matvec on the tensor pipe, weights staged through a
// shared-memory ring by bulk copies from a row-planar copy of the tensor, plus the kernel that builds
// that copy.
//
// Contract: yule-core/src/dequant.rs:976-1009 — sum += d * sc[8h + l/16 + 2j] * (q − 32) * x for the
// weight at column 128h + 32j + l, q assembled from a nibble of ql and two bits of qh.
//
// Row-planar copy.  A Q6_K super-block is 210 bytes (ql[128] qh[64] scales[16] d[2]) and only 2-byte
// aligned in the GGUF stream, which rules out both wide loads and bulk copies (16-byte granular).  The
// device keeps, next to the raw tensor, the same bytes regrouped row by row: every block's ql of the
// row, then every block's qh, then the scales, then the d values (padded to a multiple of 16 bytes).
// Any run of blocks that starts at a multiple of eight is then four 16-byte-aligned contiguous pieces.
// Same values, 210 bytes per block plus at most 14 bytes per row; built once per tensor.
//
// Tensor-core formulation (batch 1):
//   A  the 6-bit q as an fp16 subnormal (q·2^-24, exact), assembled byte-parallel from ql/qh and
//      spread to 16-bit lanes with one PRMT per pair;
//   B  x·2^e split into hi/lo halves; column n = 4·part + t' carries x only at the k slots lane
//      t' feeds, so D[row][n] is the Σ q·x of one 16-column scale group whatever the k order;
//   −32 offset: Σ (q−32)·x = Σ q·x − 32·Σx, with the per-16-column Σx staged once per CTA;
//   scales and d applied in fp32.  Only the order of fp32 additions differs from the CPU code.
// Lane (g, t): rows g and g+8; t = (h, u) owns l ∈ [16u, 16u+16) of half h, i.e. columns
// 128h + 32j + 16u + [0,16) for j = 0..3: 16 bytes of ql for j ∈ {0,2}, 16 for j ∈ {1,3}, 16 of qh.
//
// Schedule: that of qmv_q4k_ring.cu — two groups of 8 warps per CTA, 16-row tiles dealt round-robin,
// a stage is 16 rows × up to 8 super-blocks (four planes in shared memory, each with a row pitch that
// keeps the 16-byte fragment reads of a quarter warp in distinct banks), copies issued before
// `griddepcontrol.wait`, slots refilled by the warp that releases them last, bounded waits.

#include <cuda.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace yule {

namespace {

#include "ring_common.cuh"
#include "q6k_ring_common.cuh"

constexpr int kMaxStages = 4;  // per group
constexpr size_t kFullSmSmem = 227 * 1024;
constexpr size_t kPreferredSmem = 140 * 1024;  // leaves room for a small neighbour kernel on the same SM

__global__ void repack_q6k_rows_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ planar, uint64_t n_rows, uint32_t bpr) {
    const size_t rec = row_record_bytes(bpr);
    const uint32_t dsec = d_section_bytes(bpr);
    const uint64_t per_row = (uint64_t)bpr * 104 + dsec / 2;  // 16-bit pieces of a row record (blocks are 2-byte aligned)
    const uint64_t total = n_rows * per_row;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = i / per_row;
        const uint32_t o = (uint32_t)(i - row * per_row) * 2;  // byte offset inside the record
        const uint8_t *src_row = raw + row * bpr * 210;
        unsigned short v = 0;
        if (o < bpr * 128) {
            v = *reinterpret_cast<const unsigned short *>(src_row + (size_t)(o / 128) * 210 + (o % 128));
        } else if (o < bpr * 192) {
            const uint32_t q = o - bpr * 128;
            v = *reinterpret_cast<const unsigned short *>(src_row + (size_t)(q / 64) * 210 + 128 + (q % 64));
        } else if (o < bpr * 208) {
            const uint32_t q = o - bpr * 192;
            v = *reinterpret_cast<const unsigned short *>(src_row + (size_t)(q / 16) * 210 + 192 + (q % 16));
        } else {
            const uint32_t q = (o - bpr * 208) / 2;  // block index; the tail of the section is padding
            if (q < bpr) v = *reinterpret_cast<const unsigned short *>(src_row + (size_t)q * 210 + 208);
        }
        *reinterpret_cast<unsigned short *>(planar + row * rec + o) = v;
    }
}

struct RingSmem {
    unsigned char *ring;
    XImage x;
    float *partial;  // [group][buffer][warp][row]
    uint64_t *bars;
    uint32_t *cnt;
};
constexpr size_t kPartialBytes = (size_t)kGroups * 2 * kWarps * 16 * sizeof(float);

__host__ __device__ inline size_t ring_fixed_bytes(uint32_t n_cols) {
    size_t off = 2 * (x_plane_bytes(n_cols) + 64) + (size_t)(n_cols / 16) * 4;
    off = (off + 15) & ~(size_t)15;
    off += 64 + 16 + 64 * sizeof(float) + kPartialBytes + (size_t)kGroups * kMaxStages * (8 + 4);
    return (off + 127) & ~(size_t)127;
}
__host__ __device__ inline size_t ring_smem_bytes(uint32_t n_cols, uint32_t stages) {
    return (size_t)kGroups * stages * kStageBytes + ring_fixed_bytes(n_cols);
}
__device__ __forceinline__ RingSmem carve(unsigned char *base, uint32_t n_cols, uint32_t stages) {
    RingSmem s;
    s.ring = base;
    size_t off = (size_t)kGroups * stages * kStageBytes;
    s.x.xh = reinterpret_cast<__half *>(base + off);
    off += x_plane_bytes(n_cols) + 64;
    s.x.xl = reinterpret_cast<__half *>(base + off);
    off += x_plane_bytes(n_cols) + 64;
    s.x.s32 = reinterpret_cast<float *>(base + off);
    off += (size_t)(n_cols / 16) * 4;
    off = (off + 15) & ~(size_t)15;
    s.x.zb = reinterpret_cast<uint4 *>(base + off);
    off += 64;
    s.x.inv_scale = reinterpret_cast<float *>(base + off);
    off += 16;
    s.x.red = reinterpret_cast<float *>(base + off);
    off += 64 * sizeof(float);
    s.partial = reinterpret_cast<float *>(base + off);
    off += kPartialBytes;
    s.bars = reinterpret_cast<uint64_t *>(base + off);
    off += (size_t)kGroups * kMaxStages * 8;
    s.cnt = reinterpret_cast<uint32_t *>(base + off);
    return s;
}

struct Q6kRingParams {
    // Tiled views of the four planes of the row records (8-byte elements, boxes = 16 rows x the shared-memory row
    // pitches): a stage is four copy instructions instead of sixty-four (which cost the issuing warp about 2.3 µs).
    CUtensorMap map[4];
    const uint8_t *planar;  // row-planar copy
    float *out;
    uint32_t n_rows, n_cols, n_tiles;
    const float *x;
    const float *norm_w;
    float eps;
    const float *residual;
    uint32_t stages, chunks;
    int *status;
    long long wait_cycles;
    uint32_t late_wait;  // inputs are not written by the previous kernel: only the stores wait for it
};

// Copies of stage (tile, chunk), by the first lane of a (converged) warp: one box per plane, as wide as the plane's
// shared-memory row pitch (what lies beyond the chunk's eight super-blocks is never read; rows past the end of the
// matrix arrive as zeros).
__device__ __forceinline__ void issue_stage(const Q6kRingParams &p, uint32_t tile, uint32_t chunk, uint32_t bpr, uint32_t dst,
                                            uint32_t bar, int lane) {
    (void)bpr;
    if (lane == 0) {
        const uint32_t row0 = tile * kStageRows, blk0 = chunk * kStageBlocks;
        mbar_arrive_expect_tx(bar, kStageBytes);
        auto box = [&](uint32_t off, const CUtensorMap *m, uint32_t x) {
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                             dst + off),
                         "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(row0)
                         : "memory");
        };
        box(kQlOff, &p.map[0], blk0 * 16u);
        box(kQhOff, &p.map[1], blk0 * 8u);
        box(kScOff, &p.map[2], blk0 * 2u);
        box(kDOff, &p.map[3], blk0 / 4u);
    }
    __syncwarp();
}

__device__ __forceinline__ void ring_group_barrier(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(kWarps * 32) : "memory");
}

__global__ void __launch_bounds__(kThreadsCta, 2)
qmv_q6k_ring_kernel(const __grid_constant__ Q6kRingParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    yule_pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int group = threadIdx.x >> 8, wid = (threadIdx.x >> 5) & (kWarps - 1);
    const int g = lane >> 2, t = lane & 3;
    const int h = t >> 1, u = t & 1;
    const uint32_t bpr = p.n_cols / 256;
    const uint32_t G = gridDim.x;
    const uint32_t first_tile = blockIdx.x + group * G, tile_stride = kGroups * G;
    const uint32_t my_tiles = p.n_tiles > first_tile ? (p.n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
    const uint32_t S = p.stages, chunks = p.chunks;
    const uint32_t total = my_tiles * chunks;

    const RingSmem sm = carve(smem_raw, p.n_cols, S);
    unsigned char *ring = sm.ring + (size_t)group * S * kStageBytes;
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t bar0 = smem_u32(sm.bars + group * kMaxStages);
    uint32_t *cnt = sm.cnt + group * kMaxStages;

    if (wid == 0) {
        if (lane == 0) {
            for (int i = 0; i < kMaxStages; i++) {
                mbar_init(bar0 + 8 * i, 1);
                cnt[i] = 0;
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
        uint32_t k = 0, c = 0;
        for (uint32_t n = 0; n < S && n < total; n++) {
            issue_stage(p, first_tile + k * tile_stride, c, bpr, ring_u32 + n * kStageBytes, bar0 + 8 * n, lane);
            if (++c == chunks) {
                c = 0;
                k++;
            }
        }
    }

    if (!p.late_wait) yule_pdl_wait();  // the activations (and the residual) come from the previous kernel
    stage_activations(
        sm.x,
        [&](uint32_t c, float(&a)[8]) {
            *reinterpret_cast<float4 *>(a) = *reinterpret_cast<const float4 *>(p.x + c);
            *reinterpret_cast<float4 *>(a + 4) = *reinterpret_cast<const float4 *>(p.x + c + 4);
        },
        p.n_cols, p.norm_w, p.eps);
    if (total == 0) return;

    // B source of this lane: column n = g is live only for g = t (hi) and g = t + 4 (lo)
    const bool feeds = (g & 3) == t;
    const __half *bx_base = feeds ? ((g >> 2) ? sm.x.xl : sm.x.xh) + (128 + 8) * h + 16 * u : reinterpret_cast<const __half *>(sm.x.zb);
    const uint32_t blk_stride = feeds ? 2 * (128 + 8) : 0u;  // halves per super-block (two padded 128-column runs)
    const uint32_t j_stride = feeds ? 32u : 0u;
    // −32·Σx: charged once, by the lanes whose output columns belong to the hi part (t < 2)
    const int u2 = t & 1;
    const bool charge = t < 2;
    const float *s32_base = charge ? sm.x.s32 + 8 * u2 : reinterpret_cast<const float *>(sm.x.zb);
    const uint32_t s32_stride = charge ? 16u : 0u;
    const uint32_t n_warps_used = bpr < (uint32_t)kWarps ? bpr : (uint32_t)kWarps;
    float *part_base = sm.partial + (size_t)group * (2 * kWarps * 16);

    uint32_t ck = 0, cc = 0;  // job and chunk of stage n
    float acc0 = 0.f, acc1 = 0.f;
    uint32_t slot = 0, phase = 0;
    for (uint32_t n = 0; n < total; n++) {
        const uint32_t bar = bar0 + 8 * slot;
        if (!ring_wait(bar, phase, p.status, p.wait_cycles)) return;  // all eight warps of the group wait on the same copy
        const uint32_t blk0 = cc * kStageBlocks;
        const uint32_t nblk = bpr - blk0 < (uint32_t)kStageBlocks ? bpr - blk0 : (uint32_t)kStageBlocks;
        if ((uint32_t)wid < nblk) {
            const unsigned char *st = ring + (size_t)slot * kStageBytes;
            const uint32_t blk = blk0 + wid;
            consume_block_smem(st + kQlOff + (uint32_t)g * kQlPitch + (uint32_t)wid * 128u + 64u * h + 16u * u,
                               st + kQhOff + (uint32_t)g * kQhPitch + (uint32_t)wid * 64u + 32u * h + 16u * u,
                               st + kScOff + (uint32_t)g * kScPitch + (uint32_t)wid * 16u, st + kDOff + (uint32_t)g * kDPitch + (uint32_t)wid * 2u,
                               bx_base + (size_t)blk * blk_stride, j_stride, s32_base + (size_t)blk * s32_stride, u2, acc0, acc1);
        }
        __syncwarp();
        uint32_t last = 0;
        if (lane == 0) {
            __threadfence_block();
            last = ((atomicAdd(&cnt[slot], 1u) & (kWarps - 1)) == kWarps - 1) ? 1u : 0u;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last && n + S < total) {
            uint32_t nk = ck, nc = cc + S;
            while (nc >= chunks) {
                nc -= chunks;
                nk++;
            }
            issue_stage(p, first_tile + nk * tile_stride, nc, bpr, ring_u32 + slot * kStageBytes, bar, lane);
        }
        if (cc + 1 == chunks) {
            float v0 = acc0, v1 = acc1;
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            float *part = part_base + (size_t)(ck & 1u) * (kWarps * 16);
            if (t == 0) {
                part[wid * 16 + g] = v0;
                part[wid * 16 + g + 8] = v1;
            }
            acc0 = acc1 = 0.f;
            if (p.late_wait) yule_pdl_wait();  // the previous kernel is settled before our stores
            ring_group_barrier(group);
            const uint32_t tid = threadIdx.x & (kWarps * 32 - 1);
            if (tid < (uint32_t)kStageRows) {
                const uint32_t row = (first_tile + ck * tile_stride) * kStageRows + tid;
                if (row < p.n_rows) {
                    float sacc = 0.f;  // fixed order over the warps: deterministic
                    for (uint32_t w2 = 0; w2 < n_warps_used; w2++) sacc += part[w2 * 16 + tid];
                    sacc *= sm.x.inv_scale[0];
                    if (p.residual) sacc += p.residual[row];
                    p.out[row] = sacc;
                }
            }
            cc = 0;
            ck++;
        } else {
            cc++;
        }
        if (++slot == S) {
            slot = 0;
            phase ^= 1u;
        }
    }
}

}  // namespace

size_t q6k_planar_bytes(uint64_t n_rows, uint32_t n_cols) { return (size_t)n_rows * row_record_bytes(n_cols / 256) + 256; }

cudaError_t launch_q6k_repack(const uint8_t *raw, uint8_t *planar, uint64_t n_rows, uint32_t n_cols, cudaStream_t s,
                              uint64_t *launches) {
    if (n_rows == 0) return cudaSuccess;
    repack_q6k_rows_kernel<<<148 * 8, 256, 0, s>>>(raw, planar, n_rows, n_cols / 256);
    *launches += 1;
    return cudaGetLastError();
}

bool q6k_mma_supported(uint32_t n_cols) { return n_cols != 0 && n_cols % 256 == 0 && ring_smem_bytes(n_cols, 1) <= kFullSmSmem; }

cudaError_t launch_q6k_mma(const Q6kPlanar &f, int sm_count, cudaStream_t s, uint64_t *launches) {
    if (f.n_rows == 0) return cudaSuccess;
    Q6kRingParams p = {};
    {
        const uint32_t bpr = f.n_cols / 256;
        const uint64_t rec = row_record_bytes(bpr);
        const uint64_t off[4] = {0, (uint64_t)bpr * 128, (uint64_t)bpr * 192, (uint64_t)bpr * 208};
        const uint64_t len[4] = {(uint64_t)bpr * 128, (uint64_t)bpr * 64, (uint64_t)bpr * 16, d_section_bytes(bpr)};
        const uint32_t pitch[4] = {kQlPitch, kQhPitch, kScPitch, kDPitch};
        for (int pl = 0; pl < 4; pl++) {
            cudaError_t me = cached_tensor_map_2d(f.planar + off[pl], 8, len[pl] / 8, f.n_rows, rec, pitch[pl] / 8, kStageRows, &p.map[pl]);
            if (me != cudaSuccess) return me;
        }
    }
    p.planar = f.planar;
    p.out = f.out;
    p.n_rows = f.n_rows;
    p.n_cols = f.n_cols;
    p.n_tiles = (f.n_rows + kStageRows - 1) / kStageRows;
    p.x = f.x;
    p.norm_w = f.norm_w;
    p.eps = f.eps;
    p.residual = f.residual;
    p.status = f.status;
    p.wait_cycles = f.wait_cycles;
    p.late_wait = (f.pdl && f.late_wait) ? 1u : 0u;
    const uint32_t bpr = f.n_cols / 256;
    p.chunks = (bpr + kStageBlocks - 1) / kStageBlocks;
    uint32_t max_ctas = (uint32_t)sm_count;  // one CTA per SM: the other half of the SM is for the neighbouring launches
    if (const char *k = knob("YULE_QMV_RING_CTAS")) max_ctas = (uint32_t)atoi(k) > 0 ? (uint32_t)atoi(k) : max_ctas;
    uint32_t grid = (p.n_tiles + kGroups - 1) / kGroups;
    if (grid > max_ctas) grid = max_ctas;
    // Ring depth: two stages per group when they fit next to the activation image without taking the whole SM,
    // more only up to what a group will consume; a very long x leaves room for one.
    const size_t fixed = ring_fixed_bytes(f.n_cols);
    uint32_t stages = fixed + 2 * (size_t)kGroups * kStageBytes <= kPreferredSmem
                          ? (uint32_t)((kPreferredSmem - fixed) / ((size_t)kGroups * kStageBytes))
                          : (uint32_t)((kFullSmSmem - fixed) / ((size_t)kGroups * kStageBytes));
    if (stages > (uint32_t)kMaxStages) stages = kMaxStages;
    const uint32_t jobs_per_group = (p.n_tiles + kGroups * grid - 1) / (kGroups * grid);
    const uint32_t need = jobs_per_group * p.chunks;
    if (stages > need) stages = need;
    if (stages < 1) return cudaErrorInvalidValue;
    p.stages = stages;
    const size_t smem = ring_smem_bytes(f.n_cols, stages);
    auto kern = qmv_q6k_ring_kernel;
    // the opt-in for large dynamic shared memory is a per-device attribute
    static bool attr_done[64] = {};
    static std::mutex mu;
    {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !attr_done[dev]) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFullSmSmem);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) attr_done[dev] = true;
        }
    }
    cudaError_t e = launch_kernel(kern, dim3(grid), dim3(kThreadsCta), smem, s, f.pdl, p);
    if (e != cudaSuccess) return e;
    *launches += 1;
    return cudaSuccess;
}

}  // namespace yule
