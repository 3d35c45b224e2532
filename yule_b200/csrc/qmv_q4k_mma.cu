// qmv_q4k_mma.cu — Q4_K fused dequantise + matvec on the tensor pipe, with the neighbouring
// element-wise ops of the decode step folded in.
//
// Why tensor cores for a matvec: at 0.5625 bytes per weight, HBM delivers ~11.6 T weights/s; the
// SIMT route (extract nibble, convert, FMA ≈ 3–4 issue slots per weight) needs more issue slots
// than the SMs have, so it is ALU-bound below the memory roofline.  `mma.sync.m16n8k16` takes the
// multiply-accumulate off the issue budget and leaves ~1.9 slots per weight (unpack + scale).
//
// Exactness.  The contract is yule-core/src/dequant.rs:929-972:
//     sum += (d*sc_s) * Σ_l q_l x_l − (dmin*mn_s) * Σ_l x_l        per 32-column sub-block s.
// Operands are fed to the tensor core without rounding:
//   A (weights)  q·sc_s as fp16 — an integer ≤ 15·63 = 945, exact.  Built from the packed nibbles
//                as (1024+q)·sc − 1024·sc in one fp16 FMA (exact: the product fits in the FMA's
//                internal precision and the result is an integer < 2048).
//   B (x)        x·2^e split into hi = fp16(x·2^e) and lo = fp16(x·2^e − hi): two columns of the
//                8-wide B tile, summed after the MMA.  2^e normalises max|x| to [2^13, 2^14) so
//                neither overflow nor fp16 subnormals cost precision (error ≤ 2^-22 relative).
//   accumulate   fp32 in the MMA; d, dmin and 2^-e are applied in fp32 afterwards.
//   mins         one extra MMA per super-block: A = mn_s, B = Σ_l x_l of each sub-block (hi/lo).
// What differs from the CPU code is only the order of the fp32 additions.
//
// Mapping.  A CTA of 8 warps owns ROWS (16 or 8) consecutive rows; warp w takes super-blocks
// w, w+8, … of those rows.  Lane (g = lane/4, t = lane%4) holds rows g and g+8 and the 64-column
// group t of the super-block: 32 bytes of qs per row plus the 16-byte header — all 16-byte
// loads, issued for the warp's first super-block before anything else, the next super-block's
// while the current one is being multiplied.  The k index of the MMA is a free permutation
// (A and B agree on it), so nibbles go straight from the loaded words into fragments.
// Cross-warp sums go through 2 KB of shared memory in a fixed order (deterministic).
//
// Fused around the matvec (each replaces a dispatch of yule-infer/src/gpu_runner.rs:296-695):
//   prologue  RMSNorm of x (rms_norm.cu) computed per CTA while the weight loads are in flight;
//   segments  up to three matrices sharing x in one launch (Q/K/V);
//   epilogue  + residual (add.cu), or SiLU(gate)·up (silu_mul.cu) for a gate/up pair.
// Programmatic dependent launch: weights do not depend on the previous kernel, so their loads are
// issued before `griddepcontrol.wait`; only the activation read waits.

#include <cstdlib>

#include <cuda_fp16.h>

#include "internal.h"

namespace yule {

namespace {

#include "q4k_mma_common.cuh"


struct Q4kMmaParams {
    const uint8_t *w[3];    // segment weight tensors (raw Q4_K blocks)
    float *out[3];          // segment outputs, [batch][out_stride[s]]
    uint32_t seg_tiles[3];  // row tiles per segment
    uint32_t seg_rows[3];
    uint32_t out_stride[3];
    uint32_t n_seg;
    uint32_t n_tiles;       // tiles over all segments (pair mode: tiles of one matrix)
    uint32_t pair;          // 1: w[0], w[1] are gate and up over the same rows → out[0] = SiLU(gate)·up
    const float *x;         // [batch][x_stride]
    uint32_t x_stride, n_cols, batch;
    const float *norm_w;    // RMSNorm weights for the prologue, or null
    float eps;
    const float *residual;  // added to segment 0's output, or null (same layout as out[0])
    const void *next_w[2];  // weights of the following kernel(s), prefetched into L2
    uint64_t next_bytes[2];
    TpFuse tp;              // tensor parallelism: push out[0] to the peers / wait for the gathered x
    uint32_t late_wait;     // inputs are not written by the previous kernel: only the stores wait for it
};

__device__ __forceinline__ void group_barrier(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(kWarps * 32) : "memory");
}

// Walks one warp's units in order: tile index k (of its group), matrix q (pair mode), super-block
// slot j; the row pointers are recomputed only when the tile or matrix changes.
template <int ROWS, bool Q5>
struct UnitCursor {
    static constexpr int NR = ROWS / 8;
    uint32_t k, q, j;
    const uint4 *rowp[NR];

    __device__ __forceinline__ void locate(const Q4kMmaParams &p, uint32_t first_tile, uint32_t tile_stride, uint32_t bpr,
                                           int g) {
        uint32_t tile = first_tile + k * tile_stride, seg = 0;
        if (p.pair) {
            seg = q;
        } else {
            while (seg + 1 < p.n_seg && tile >= p.seg_tiles[seg]) {
                tile -= p.seg_tiles[seg];
                seg++;
            }
        }
        const uint32_t n_rows = p.seg_rows[seg];
#pragma unroll
        for (int r = 0; r < NR; r++) {
            uint32_t row = tile * ROWS + g + 8 * r;
            row = row < n_rows ? row : n_rows - 1;  // clamp: the load stays in bounds, the result is dropped
            rowp[r] = reinterpret_cast<const uint4 *>(p.w[seg] + (size_t)row * bpr * (Q5 ? 176 : 144));
        }
    }
    __device__ __forceinline__ void advance(const Q4kMmaParams &p, uint32_t first_tile, uint32_t tile_stride, uint32_t bpr,
                                            int g, uint32_t nbw, uint32_t nq) {
        if (++j == nbw) {
            j = 0;
            if (++q == nq) {
                q = 0;
                k++;
            }
            locate(p, first_tile, tile_stride, bpr, g);
        }
    }
};

// Persistent kernel, one CTA per SM: CTA c owns tiles c, c+G, c+2G, … (G = gridDim.x), dealt
// alternately to its two 8-warp groups, so every SM gets the same number of tiles (±1) and at any
// moment the grid streams one contiguous region of the tensor.  Within a tile, warp w of the
// group multiplies super-blocks w, w+8, …; a warp's (tile, matrix, super-block) units form one
// sequence that is prefetched DEPTH units ahead.  In pair mode a tile is the gate rows followed by
// the same rows of up.  The activations are staged once per CTA.
// TP = true only for launches of a tensor-parallel runner that push or poll (value, epoch) pairs: the
// single-GPU instantiations carry none of that code.
template <int ROWS, int DEPTH, bool SUBCOL, bool TP, bool Q5>
__global__ void __launch_bounds__(kThreadsCta, 1)
qmv_q4k_mma_kernel(const __grid_constant__ Q4kMmaParams p) {
    constexpr int NR = ROWS / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    yule_pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int group = threadIdx.x >> 8, wid = (threadIdx.x >> 5) & (kWarps - 1);
    const int g = lane >> 2, t = lane & 3;
    const uint32_t bpr = p.n_cols / 256;
    const uint32_t nbw = bpr > (uint32_t)wid ? (bpr - wid + kWarps - 1) / kWarps : 0;  // super-blocks per tile for this warp
    const uint32_t nq = p.pair ? 2 : 1;
    const uint32_t G = gridDim.x;
    // tiles of this CTA: blockIdx.x + i*G; group takes i = group, group + 2, …
    const uint32_t first_tile = blockIdx.x + group * G, tile_stride = kGroups * G;
    const uint32_t my_tiles = p.n_tiles > first_tile ? (p.n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
    const uint32_t tiles_per_round = kRoundSlots / nq;

    const SmemLayout sm = carve(smem_raw, p.n_cols, p.batch);
    float *partial = sm.partial + (size_t)group * kRoundSlots * kWarps * 4 * 16;

    UnitCursor<ROWS, Q5> ld_cur;
    ld_cur.k = ld_cur.q = ld_cur.j = 0;
    const uint32_t total_units = my_tiles * nq * nbw;
    uint32_t issued = 0;
    BlockLoads buf[DEPTH][NR];
    if (total_units) {
        ld_cur.locate(p, first_tile, tile_stride, bpr, g);
#pragma unroll
        for (int i = 0; i < DEPTH; i++) {
            if (issued < total_units) {
                issue_loads<NR, Q5>(buf[i], ld_cur.rowp, wid + kWarps * ld_cur.j, t);
                issued++;
                if (issued < total_units) ld_cur.advance(p, first_tile, tile_stride, bpr, g, nbw, nq);
            }
        }
    }

    // Own weight loads are in flight; start HBM on the next kernel's weights too, then wait for
    // the kernel that produced the activations.
    yule_prefetch_l2_slice(p.next_w[0], p.next_bytes[0]);
    yule_prefetch_l2_slice(p.next_w[1], p.next_bytes[1]);
    if (!p.late_wait) yule_pdl_wait();
    // tensor parallelism: x may arrive as (value, epoch) pairs stored by all ranks
    if (TP)
        stage_activations<true>(sm, p.x, p.x_stride, p.n_cols, p.batch, p.norm_w, p.eps, p.tp.wait ? p.tp.pair_in : nullptr,
                                p.tp.wait ? *p.tp.tick * p.tp.epochs_per_tick + p.tp.wait_index + 1u : 0u, p.tp.status,
                                p.tp.wait_cycles);
    else
        stage_activations<false>(sm, p.x, p.x_stride, p.n_cols, p.batch, p.norm_w, p.eps);
    // B column n = g: vector n/2, part n%2.  Lanes whose vector does not exist read vector 0;
    // their output columns are never looked at.
    const uint32_t vec = (uint32_t)(g >> 1) < p.batch ? (g >> 1) : 0;
    const uint4 *xb_lane = sm.xb + (size_t)vec * (p.n_cols / 4) + (g & 1) * 4 + t;
    const uint32_t *sb_lane = sm.sb + (size_t)vec * (p.n_cols / 32) + (g & 1) * 4 + t;
    // batch-1 path: lane (g, t) feeds column g; that column is live only for g = t (hi part) and
    // g = t + 4 (lo part), every other lane reads zeros
    const bool feeds = (g & 3) == t;
    const uint4 *sub_base = feeds ? sm.xb + (g >> 2) * 4 + t : sm.zb;
    const uint32_t sub_stride = feeds ? 64u : 0u;
    const int u = t & 1;
    const bool charge_mins = t < 2;

    // Cross-warp sums of the tiles [k0, k0+kn) of this group, then the epilogue.  Every warp of
    // the group calls this once per round.
    auto finish_round = [&](uint32_t k0, uint32_t kn) {
        if (p.late_wait) yule_pdl_wait();  // everything the previous kernel wrote or read is settled before our stores
        group_barrier(group);
        const uint32_t n_warps_used = bpr < (uint32_t)kWarps ? bpr : kWarps;
        const uint32_t tid = threadIdx.x & (kWarps * 32 - 1);
        for (uint32_t idx = tid; idx < kn * 64; idx += kWarps * 32) {
            const uint32_t kk = idx >> 6, v = (idx >> 4) & 3, rr = idx & 15;
            if (v >= p.batch || rr >= ROWS) continue;
            uint32_t tile = first_tile + (k0 + kk) * tile_stride, seg = 0;
            if (!p.pair) {
                while (seg + 1 < p.n_seg && tile >= p.seg_tiles[seg]) {
                    tile -= p.seg_tiles[seg];
                    seg++;
                }
            }
            const uint32_t row = tile * ROWS + rr;
            if (row >= p.seg_rows[seg]) continue;
            const float inv_scale = sm.inv_scale[v];
            float sums[2] = {0.f, 0.f};
            for (uint32_t q = 0; q < nq; q++) {
                const uint32_t sl = kk * nq + q;
                float sacc = 0.f;  // fixed order over the warps: deterministic
                if (SUBCOL) {
                    // the four t lanes hold (hi, lo) × (sub-blocks 0..3, 4..7): one vector, four addends
                    for (uint32_t w2 = 0; w2 < n_warps_used; w2++)
#pragma unroll
                        for (int tt = 0; tt < 4; tt++) sacc += partial[((sl * kWarps + w2) * 4 + tt) * 16 + rr];
                } else {
                    for (uint32_t w2 = 0; w2 < n_warps_used; w2++) sacc += partial[((sl * kWarps + w2) * 4 + v) * 16 + rr];
                }
                sums[q] = sacc * inv_scale;
            }
            const size_t o = (size_t)v * p.out_stride[seg] + row;
            if (p.pair) {
                // silu_mul.cu: x / (1 + exp(−x)) * up
                sums[0] = (sums[0] / (1.0f + expf(-sums[0]))) * sums[1];
            } else if (seg == 0 && p.residual) {
                sums[0] += p.residual[o];
            }
            p.out[seg][o] = sums[0];
            if (TP && p.tp.push && seg == 0) tp_push_value(p.tp, o, sums[0]);  // the same row into every peer's copy
        }
        group_barrier(group);
    };

    if (nbw == 0) {
        // more warps than super-blocks per row: this warp only helps with the reductions
        for (uint32_t k0 = 0; k0 < my_tiles; k0 += tiles_per_round)
            finish_round(k0, (my_tiles - k0) < tiles_per_round ? (my_tiles - k0) : tiles_per_round);
    } else {

    float acc[NR][2];
#pragma unroll
    for (int r = 0; r < NR; r++) acc[r][0] = acc[r][1] = 0.f;
    uint32_t k0 = 0, kn = my_tiles < tiles_per_round ? my_tiles : tiles_per_round;
    uint32_t in_slot = 0, slot = 0;  // super-blocks done in the current (tile, matrix); slots done in the round
    // unit n lives in buf[n % DEPTH]; the loop is unrolled by DEPTH so the ring index is static
    for (uint32_t base = 0; base < total_units; base += DEPTH) {
#pragma unroll
        for (int i = 0; i < DEPTH; i++) {
            if (base + i < total_units) {
                if (SUBCOL) {
                    const uint32_t blk = wid + kWarps * in_slot;
                    consume_block_subcol<NR, Q5>(buf[i], sub_base + (size_t)blk * sub_stride, sm.sf + (size_t)blk * 8 + 4 * u,
                                                 u, t, charge_mins, acc);
                } else {
                    consume_block<NR, Q5>(buf[i], wid + kWarps * in_slot, t, xb_lane, sb_lane, acc);
                }
                if (issued < total_units) {
                    issue_loads<NR, Q5>(buf[i], ld_cur.rowp, wid + kWarps * ld_cur.j, t);
                    issued++;
                    if (issued < total_units) ld_cur.advance(p, first_tile, tile_stride, bpr, g, nbw, nq);
                }
                if (++in_slot == nbw) {
                    // lane (g, t) holds, for vector t, rows g (and g+8): hi-column + lo-column sums
#pragma unroll
                    for (int r = 0; r < NR; r++) {
                        partial[((slot * kWarps + wid) * 4 + t) * 16 + g + 8 * r] = acc[r][0] + acc[r][1];
                        acc[r][0] = acc[r][1] = 0.f;
                    }
                    in_slot = 0;
                    if (++slot == kn * nq) {
                        finish_round(k0, kn);
                        k0 += kn;
                        kn = (my_tiles - k0) < tiles_per_round ? (my_tiles - k0) : tiles_per_round;
                        slot = 0;
                    }
                }
            }
        }
    }
    }  // nbw != 0

}

template <int ROWS, int DEPTH, bool SUBCOL, bool Q5 = false, bool TP = false>
cudaError_t launch_variant(const Q4kMmaParams &p, int sm_count, size_t smem, bool pdl, cudaStream_t s) {
    if (!TP && !Q5 && (p.tp.push || p.tp.wait))
        return launch_variant<ROWS, DEPTH, SUBCOL, false, true>(p, sm_count, smem, pdl, s);
    auto kern = qmv_q4k_mma_kernel<ROWS, DEPTH, SUBCOL, TP, Q5>;
    // per instantiation: the opt-in for large dynamic shared memory
    // (the attribute belongs to the device, not the process: one flag per device ordinal)
    static bool attr_done[64] = {};
    static std::mutex mu;
    {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !attr_done[dev]) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) attr_done[dev] = true;
        }
    }
    // one CTA per SM; fewer when there are not enough tiles to give every group one
    uint32_t grid = (uint32_t)sm_count;
    const uint32_t want = (p.n_tiles + kGroups - 1) / kGroups;
    if (grid > want) grid = want;
    return launch_kernel(kern, dim3(grid), dim3(kThreadsCta), smem, s, pdl, p);
}

}  // namespace

bool q4k_mma_supported(uint32_t n_cols, uint32_t batch) {
    return n_cols % 256 == 0 && batch >= 1 && batch <= 4 && smem_bytes(n_cols, batch) <= 200 * 1024;
}

cudaError_t launch_q4k_mma(const Q4kFused &f, int sm_count, cudaStream_t s, uint64_t *launches) {
    // Two kernels, chosen by what the call depends on.  A call whose inputs do not come from the previous kernel
    // (late wait) goes to the shared-memory-ring kernel, which shares the SMs with its predecessor and overlaps
    // with it almost entirely; a link of a dependent chain, and any matrix long enough to hide a kernel's fixed
    // costs, goes to the register-streaming kernel below.  YULE_QMV_RING=1 / 0 forces one (timing aid).
    {
        uint32_t rows16 = 0;
        for (uint32_t i = 0; i < f.n_seg; i++) rows16 += (f.rows[i] + 15) / 16;
        bool ring = f.pdl && f.late_wait && rows16 <= 8u * (uint32_t)sm_count;
        if (const char *k = knob("YULE_QMV_RING")) ring = atoi(k) != 0;
        if (ring && q4k_ring_supported(f)) return launch_q4k_ring(f, sm_count, s, launches);
    }
    Q4kMmaParams p = {};
    const bool pair = f.swiglu_pair;
    uint32_t total_rows = 0;
    for (uint32_t i = 0; i < f.n_seg; i++) total_rows += f.rows[i];
    // 16-row tiles use the whole MMA; 8-row tiles (half of each MMA idle) only when 16-row tiles
    // would leave warp groups without work.
    const uint32_t rows_for_grid = pair ? 2 * f.rows[0] : total_rows;
    // Tile height.  16-row tiles use the whole MMA and half the instructions per byte of 8-row tiles; they win
    // as soon as they keep about 60 % of the warp groups busy (measured: 4096 rows, 256 tiles for 296 groups,
    // 10-25 % faster with 16; 2048 rows, 128 tiles, faster with 8).  YULE_QMV_ROWS forces one (timing aid).
    const uint32_t n_groups = (uint32_t)kGroups * (uint32_t)sm_count;
    int tile_rows = ((rows_for_grid / 16) * 10 >= n_groups * 6) ? 16 : 8;
    if (const char *force = knob("YULE_QMV_ROWS")) tile_rows = atoi(force) == 8 ? 8 : (atoi(force) == 16 ? 16 : tile_rows);
    uint32_t n_tiles = 0;
    for (uint32_t i = 0; i < f.n_seg; i++) {
        p.w[i] = f.w[i];
        p.out[i] = f.out[i];
        p.seg_rows[i] = f.rows[i];
        p.seg_tiles[i] = (f.rows[i] + tile_rows - 1) / tile_rows;
        p.out_stride[i] = f.out_stride[i];
        if (!pair || i == 0) n_tiles += p.seg_tiles[i];
    }
    p.n_seg = f.n_seg;
    p.n_tiles = n_tiles;
    p.pair = pair ? 1 : 0;
    p.x = f.x;
    p.x_stride = f.x_stride;
    p.n_cols = f.n_cols;
    p.batch = f.batch;
    p.norm_w = f.norm_w;
    p.eps = f.eps;
    p.residual = f.residual;
    p.tp = f.tp;
    p.late_wait = (f.pdl && f.late_wait) ? 1u : 0u;
    for (int i = 0; i < 2; i++) {
        p.next_w[i] = f.next_w[i];
        p.next_bytes[i] = f.next_bytes[i];
    }
    if (n_tiles == 0) return cudaSuccess;
    const size_t smem = smem_bytes(f.n_cols, f.batch);
    cudaError_t e;
    if (f.q5 && (f.tp.push || f.tp.wait)) return cudaErrorInvalidValue;  // the exchange is built for Q4_K only
    if (f.q5 && f.batch == 1)
        e = tile_rows == 8 ? launch_variant<8, 4, true, true>(p, sm_count, smem, f.pdl, s)
                           : launch_variant<16, 2, true, true>(p, sm_count, smem, f.pdl, s);
    else if (f.q5)
        e = tile_rows == 8 ? launch_variant<8, 4, false, true>(p, sm_count, smem, f.pdl, s)
                           : launch_variant<16, 2, false, true>(p, sm_count, smem, f.pdl, s);
    else if (f.batch == 1)
        e = tile_rows == 8 ? launch_variant<8, 4, true>(p, sm_count, smem, f.pdl, s)
                           : launch_variant<16, 2, true>(p, sm_count, smem, f.pdl, s);
    else
        e = tile_rows == 8 ? launch_variant<8, 4, false>(p, sm_count, smem, f.pdl, s)
                           : launch_variant<16, 2, false>(p, sm_count, smem, f.pdl, s);
    if (e != cudaSuccess) return e;
    *launches += 1;
    return cudaSuccess;
}

}  // namespace yule
