// qmv_q6k_mma.cu — Q6_K fused dequantise + matvec on the tensor pipe, weights streamed through registers
// from the row-planar copy of the tensor (built by qmv_q6k_ring.cu, which also describes the layout).
// This is the kernel of dependent chains (the token step of the runner): it keeps the first super-blocks of
// every warp in registers across the dependency wait.  qmv_q6k_ring.cu is the kernel of independent calls.
//
// Contract: yule-core/src/dequant.rs:976-1009 — sum += d * sc[8h + l/16 + 2j] * (q − 32) * x for the
// weight at column 128h + 32j + l, q assembled from a nibble of ql and two bits of qh.
//
// Row-planar copy: per row, every block's ql, then every block's qh, then the scales, then the d values — each
// piece a lane needs is one aligned 16-byte load.
//
// Tensor-core formulation (same ideas as qmv_q4k_mma.cu, batch 1):
//   A  the 6-bit q as an fp16 subnormal (q·2^-24, exact), assembled byte-parallel from ql/qh and
//      spread to 16-bit lanes with one PRMT per pair;
//   B  x·2^e split into hi/lo halves; column n = 4·part + t' carries x only at the k slots lane
//      t' feeds, so D[row][n] is the Σ q·x of one 16-column scale group whatever the k order;
//   −32 offset: Σ (q−32)·x = Σ q·x − 32·Σx, with the per-16-column Σx staged once per CTA;
//   scales and d applied in fp32.  Only the order of fp32 additions differs from the CPU code.
// Lane (g, t): rows g and g+8; t = (h, u) owns l ∈ [16u, 16u+16) of half h, i.e. columns
// 128h + 32j + 16u + [0,16) for j = 0..3: 16 bytes of ql for j ∈ {0,2}, 16 for j ∈ {1,3}, 16 of qh.

#include <cstdlib>

#include <cuda_fp16.h>

#include "internal.h"

namespace yule {

namespace {

constexpr int kWarps = 8;
constexpr int kGroups = 2;
constexpr int kThreadsCta = kGroups * kWarps * 32;
constexpr int kRoundSlots = 8;

__device__ __forceinline__ uint4 ld_stream_u4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::evict_first.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u16(const void *p) {
    unsigned short v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// Row record of the row-planar copy (same arithmetic as qmv_q6k_ring.cu).
__host__ __device__ inline size_t row_record_bytes(uint32_t bpr) { return (size_t)bpr * 208 + ((bpr * 2 + 15) & ~15u); }

// What one lane needs from one super-block of one row.
struct BlockLoads {
    uint4 qa, qb, qh, sc;  // ql for j ∈ {0,2}; ql for j ∈ {1,3}; qh; the 16 scales
    uint32_t d;            // f16 bits
};

template <int NR>
__device__ __forceinline__ void issue_loads(BlockLoads (&ld)[NR], const uint8_t *const (&rec)[NR], uint32_t bpr, uint32_t blk,
                                            int h, int u) {
#pragma unroll
    for (int r = 0; r < NR; r++) {
        const uint8_t *ql = rec[r] + (size_t)blk * 128, *qh = rec[r] + (size_t)bpr * 128 + (size_t)blk * 64;
        ld[r].qa = ld_stream_u4(ql + 64 * h + 16 * u);
        ld[r].qb = ld_stream_u4(ql + 64 * h + 32 + 16 * u);
        ld[r].qh = ld_stream_u4(qh + 32 * h + 16 * u);
        ld[r].sc = ld_stream_u4(rec[r] + (size_t)bpr * 192 + (size_t)blk * 16);
        ld[r].d = ld_stream_u16(rec[r] + (size_t)bpr * 208 + (size_t)blk * 2);
    }
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// Shared-memory image of the activation vector:
//   xh, xl   fp16 hi / lo of x·2^e in column order, 8 halves of padding after every 128 columns;
//            xl starts 64 bytes (mod 128) after xh, so the eight live lanes of a B load fall into
//            distinct banks;
//   s32      −32 · Σx over each 16-column scale group (fp32);
//   zb       zeros for lanes that feed an all-zero B column (and for the lanes that must not
//            charge the −32 term a second time).
struct SmemLayout {
    __half *xh, *xl;
    float *s32;
    uint4 *zb;
    float *inv_scale;
    float *partial;
    float *red;
};
__host__ __device__ inline uint32_t padded_cols(uint32_t n_cols) { return n_cols + 8 * (n_cols / 128); }
constexpr size_t kPartialBytes = (size_t)kGroups * kRoundSlots * kWarps * 4 * 16 * sizeof(float);

__host__ __device__ inline size_t x_plane_bytes(uint32_t n_cols) { return (((size_t)padded_cols(n_cols) * 2 + 127) / 128) * 128; }

__device__ __forceinline__ SmemLayout carve(unsigned char *base, uint32_t n_cols) {
    SmemLayout s;
    size_t off = 0;
    s.xh = reinterpret_cast<__half *>(base);
    off += x_plane_bytes(n_cols) + 64;
    s.xl = reinterpret_cast<__half *>(base + off);
    off += x_plane_bytes(n_cols) + 64;
    s.s32 = reinterpret_cast<float *>(base + off);
    off += (size_t)(n_cols / 16) * 4;
    off = (off + 15) & ~(size_t)15;
    s.zb = reinterpret_cast<uint4 *>(base + off);
    off += 64;
    s.inv_scale = reinterpret_cast<float *>(base + off);
    off += 16;
    s.partial = reinterpret_cast<float *>(base + off);
    off += kPartialBytes;
    s.red = reinterpret_cast<float *>(base + off);
    return s;
}
size_t smem_bytes(uint32_t n_cols) {
    size_t off = 2 * (x_plane_bytes(n_cols) + 64) + (size_t)(n_cols / 16) * 4;
    off = (off + 15) & ~(size_t)15;
    return off + 64 + 16 + kPartialBytes + 64 * sizeof(float) + 16;
}

__device__ __forceinline__ void stage_activations(const SmemLayout &sm, const float *__restrict__ x, uint32_t n_cols,
                                                  const float *__restrict__ norm_w, float eps) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    constexpr int NW = kThreadsCta / 32;
    constexpr int kCache = 4;
    if (threadIdx.x < 4) sm.zb[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);
    float cache[kCache][8];
    float ss = 0.f, mx = 0.f;
    auto load8 = [&](uint32_t c, float (&a)[8]) {
        *reinterpret_cast<float4 *>(a) = *reinterpret_cast<const float4 *>(x + c);
        *reinterpret_cast<float4 *>(a + 4) = *reinterpret_cast<const float4 *>(x + c + 4);
    };
    auto reduce8 = [&](uint32_t c, const float (&a)[8]) {
        float gw[8];
        if (norm_w) {
            *reinterpret_cast<float4 *>(gw) = *reinterpret_cast<const float4 *>(norm_w + c);
            *reinterpret_cast<float4 *>(gw + 4) = *reinterpret_cast<const float4 *>(norm_w + c + 4);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            ss = fmaf(a[i], a[i], ss);
            mx = fmaxf(mx, fabsf(norm_w ? a[i] * gw[i] : a[i]));
        }
    };
#pragma unroll
    for (int k = 0; k < kCache; k++) {
        const uint32_t c = (threadIdx.x + k * kThreadsCta) * 8;
        if (c < n_cols) {
            load8(c, cache[k]);
            reduce8(c, cache[k]);
        }
    }
    for (uint32_t c = (threadIdx.x + kCache * kThreadsCta) * 8; c < n_cols; c += kThreadsCta * 8) {
        float a[8];
        load8(c, a);
        reduce8(c, a);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0) {
        sm.red[wid] = ss;
        sm.red[32 + wid] = mx;
    }
    __syncthreads();
    ss = 0.f;
    mx = 0.f;
#pragma unroll
    for (int i = 0; i < NW; i++) {
        ss += sm.red[i];
        mx = fmaxf(mx, sm.red[32 + i]);
    }
    // RMSNorm scale as the CPU runner forms it: 1 / sqrt(ss / n + eps) (yule-infer/src/model_runner.rs:254-258)
    const float inv_rms = norm_w ? 1.0f / sqrtf(ss / (float)n_cols + eps) : 1.0f;
    mx *= inv_rms;
    int eb = (int)((__float_as_uint(mx) >> 23) & 0xFFu);
    if (mx == 0.f || eb == 0xFF) eb = 127 + 13;
    int se = 127 + 13 - (eb - 127);
    se = se < 1 ? 1 : (se > 253 ? 253 : se);
    const float scale = __uint_as_float((uint32_t)se << 23);
    if (threadIdx.x == 0) sm.inv_scale[0] = __uint_as_float((uint32_t)(254 - se) << 23);
    auto convert8 = [&](uint32_t c, float (&a)[8]) {
        if (norm_w) {
            float gw[8];
            *reinterpret_cast<float4 *>(gw) = *reinterpret_cast<const float4 *>(norm_w + c);
            *reinterpret_cast<float4 *>(gw + 4) = *reinterpret_cast<const float4 *>(norm_w + c + 4);
#pragma unroll
            for (int i = 0; i < 8; i++) a[i] = a[i] * inv_rms * gw[i];
        }
        __half hi[8], lo[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            a[i] *= scale;
            hi[i] = __float2half_rn(a[i]);
            lo[i] = __float2half_rn(a[i] - __half2float(hi[i]));
        }
        const uint32_t pc = c + 8 * (c >> 7);
        *reinterpret_cast<uint4 *>(sm.xh + pc) =
            make_uint4(h2_as_u32(__halves2half2(hi[0], hi[1])), h2_as_u32(__halves2half2(hi[2], hi[3])),
                       h2_as_u32(__halves2half2(hi[4], hi[5])), h2_as_u32(__halves2half2(hi[6], hi[7])));
        *reinterpret_cast<uint4 *>(sm.xl + pc) =
            make_uint4(h2_as_u32(__halves2half2(lo[0], lo[1])), h2_as_u32(__halves2half2(lo[2], lo[3])),
                       h2_as_u32(__halves2half2(lo[4], lo[5])), h2_as_u32(__halves2half2(lo[6], lo[7])));
        float s8 = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
        s8 += __shfl_xor_sync(0xffffffffu, s8, 1);  // two consecutive threads hold one 16-column group
        if ((lane & 1) == 0) sm.s32[c >> 4] = -32.0f * s8;
    };
#pragma unroll
    for (int k = 0; k < kCache; k++) {
        const uint32_t c = (threadIdx.x + k * kThreadsCta) * 8;
        if (c < n_cols) convert8(c, cache[k]);
    }
    for (uint32_t c = (threadIdx.x + kCache * kThreadsCta) * 8; c < n_cols; c += kThreadsCta * 8) {
        float a[8];
        load8(c, a);
        convert8(c, a);
    }
    __syncthreads();
}

// Multiply one super-block (this lane's rows, its 16 l-values, all four column groups j).
//   bx   this lane's B source for the block: xh/xl + padded column of (blk, h, u), or the zero region
//   s32  −32·Σx of the eight scale groups this lane applies (or zeros)
template <int NR>
__device__ __forceinline__ void consume_block(const BlockLoads (&ld)[NR], const __half *bx, uint32_t j_stride,
                                              const float *s32, int u2, float (&acc)[NR]) {
    float tmp[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) tmp[r] = 0.f;
    const float4 sa = *reinterpret_cast<const float4 *>(s32), sb = *reinterpret_cast<const float4 *>(s32 + 4);
    const float sg[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};  // index 2j + {0,1}
    // the eight scales this lane applies: sc[8·u2 + 2j + {0,1}], signed bytes → float
    float scf[NR][8];
#pragma unroll
    for (int r = 0; r < NR; r++) {
        const uint32_t w0 = (u2 ? ld[r].sc.z : ld[r].sc.x) ^ 0x80808080u, w1 = (u2 ? ld[r].sc.w : ld[r].sc.y) ^ 0x80808080u;
        const float k = 8388608.0f + 128.0f;
        scf[r][0] = __uint_as_float(__byte_perm(w0, 0x4B000000u, 0x7440)) - k;
        scf[r][1] = __uint_as_float(__byte_perm(w0, 0x4B000000u, 0x7441)) - k;
        scf[r][2] = __uint_as_float(__byte_perm(w0, 0x4B000000u, 0x7442)) - k;
        scf[r][3] = __uint_as_float(__byte_perm(w0, 0x4B000000u, 0x7443)) - k;
        scf[r][4] = __uint_as_float(__byte_perm(w1, 0x4B000000u, 0x7440)) - k;
        scf[r][5] = __uint_as_float(__byte_perm(w1, 0x4B000000u, 0x7441)) - k;
        scf[r][6] = __uint_as_float(__byte_perm(w1, 0x4B000000u, 0x7442)) - k;
        scf[r][7] = __uint_as_float(__byte_perm(w1, 0x4B000000u, 0x7443)) - k;
    }
    float dj[4][4];
#pragma unroll
    for (int j = 0; j < 4; j++) dj[j][0] = dj[j][1] = dj[j][2] = dj[j][3] = 0.f;

#pragma unroll
    for (int i4 = 0; i4 < 4; i4++) {
        // 6-bit values of the four column groups, four weights per word, one per byte
        uint32_t v[NR][4];
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const uint32_t qa = word_of(ld[r].qa, i4), qb = word_of(ld[r].qb, i4), qh = word_of(ld[r].qh, i4);
            v[r][0] = (qa & 0x0F0F0F0Fu) | ((qh << 4) & 0x30303030u);
            v[r][1] = (qb & 0x0F0F0F0Fu) | ((qh << 2) & 0x30303030u);
            v[r][2] = ((qa >> 4) & 0x0F0F0F0Fu) | (qh & 0x30303030u);
            v[r][3] = ((qb >> 4) & 0x0F0F0F0Fu) | ((qh >> 2) & 0x30303030u);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint2 b = *reinterpret_cast<const uint2 *>(bx + j * j_stride + 4 * i4);
            // bytes → 16-bit lanes: {b0, b1} and {b2, b3}; the value is q·2^-24 as an fp16 subnormal
            const uint32_t a0 = __byte_perm(v[0][j], 0u, 0x4140), a2 = __byte_perm(v[0][j], 0u, 0x4342);
            const uint32_t a1 = NR == 2 ? __byte_perm(v[NR - 1][j], 0u, 0x4140) : 0u;
            const uint32_t a3 = NR == 2 ? __byte_perm(v[NR - 1][j], 0u, 0x4342) : 0u;
            mma_16816(dj[j], a0, a1, a2, a3, b.x, b.y);
        }
    }
    const float k24 = 16777216.0f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
#pragma unroll
        for (int r = 0; r < NR; r++) {
            // columns 2t and 2t+1 of D are scale groups (h = u2, u = 0) and (h = u2, u = 1) of group j
            tmp[r] = fmaf(scf[r][2 * j], fmaf(dj[j][2 * r], k24, sg[2 * j]), tmp[r]);
            tmp[r] = fmaf(scf[r][2 * j + 1], fmaf(dj[j][2 * r + 1], k24, sg[2 * j + 1]), tmp[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < NR; r++)
        acc[r] = fmaf(__half2float(__ushort_as_half((unsigned short)ld[r].d)), tmp[r], acc[r]);
}

struct Q6kMmaParams {
    const uint8_t *planar;
    float *out;
    uint32_t n_rows, n_cols, n_tiles;
    const float *x;
    const float *norm_w;
    float eps;
    const float *residual;
    const void *next_w[2];  // weights of the following kernel(s), prefetched into L2
    uint64_t next_bytes[2];
};

__device__ __forceinline__ void group_barrier(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(kWarps * 32) : "memory");
}

// Same schedule as qmv_q4k_mma_kernel: persistent, one 512-thread CTA per SM, tiles dealt
// alternately to two 8-warp groups, warp w takes super-blocks w, w+8, …, DEPTH units prefetched.
template <int ROWS, int DEPTH>
__global__ void __launch_bounds__(kThreadsCta, 1)
qmv_q6k_mma_kernel(const Q6kMmaParams p) {
    constexpr int NR = ROWS / 8;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    yule_pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int group = threadIdx.x >> 8, wid = (threadIdx.x >> 5) & (kWarps - 1);
    const int g = lane >> 2, t = lane & 3;
    const int h = t >> 1, u = t & 1;
    const uint32_t bpr = p.n_cols / 256;
    const uint32_t nbw = bpr > (uint32_t)wid ? (bpr - wid + kWarps - 1) / kWarps : 0;
    const uint32_t G = gridDim.x;
    const uint32_t first_tile = blockIdx.x + group * G, tile_stride = kGroups * G;
    const uint32_t my_tiles = p.n_tiles > first_tile ? (p.n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
    const size_t rec_bytes = row_record_bytes(bpr);

    const SmemLayout sm = carve(smem_raw, p.n_cols);
    float *partial = sm.partial + (size_t)group * kRoundSlots * kWarps * 4 * 16;

    // load cursor: tile k, super-block slot j
    uint32_t lk = 0, lj = 0;
    const uint8_t *rowrec[NR];
    auto locate = [&]() {
        const uint32_t tile = first_tile + lk * tile_stride;
#pragma unroll
        for (int r = 0; r < NR; r++) {
            uint32_t row = tile * ROWS + g + 8 * r;
            row = row < p.n_rows ? row : p.n_rows - 1;  // clamp: the load stays in bounds, the result is dropped
            rowrec[r] = p.planar + (size_t)row * rec_bytes;
        }
    };
    auto advance = [&]() {
        if (++lj == nbw) {
            lj = 0;
            lk++;
            locate();
        }
    };
    const uint32_t total_units = my_tiles * nbw;
    uint32_t issued = 0;
    BlockLoads buf[DEPTH][NR];
    if (total_units) {
        locate();
#pragma unroll
        for (int i = 0; i < DEPTH; i++) {
            if (issued < total_units) {
                issue_loads<NR>(buf[i], rowrec, bpr, wid + kWarps * lj, h, u);
                issued++;
                if (issued < total_units) advance();
            }
        }
    }

    // own weights are in flight; start HBM on the next kernel's weights too
    yule_prefetch_l2_slice(p.next_w[0], p.next_bytes[0]);
    yule_prefetch_l2_slice(p.next_w[1], p.next_bytes[1]);
    yule_pdl_wait();  // the activations come from the previous kernel
    stage_activations(sm, p.x, p.n_cols, p.norm_w, p.eps);

    // B source of this lane: column n = g is live only for g = t (hi) and g = t + 4 (lo)
    const bool feeds = (g & 3) == t;
    const __half *bx_base = feeds ? ((g >> 2) ? sm.xl : sm.xh) + (128 + 8) * h + 16 * u : reinterpret_cast<const __half *>(sm.zb);
    const uint32_t blk_stride = feeds ? 2 * (128 + 8) : 0u;  // halves per super-block (two padded 128-column runs)
    const uint32_t j_stride = feeds ? 32u : 0u;
    // −32·Σx: charged once, by the lanes whose output columns belong to the hi part (t < 2)
    const int u2 = t & 1;
    const bool charge = t < 2;
    const float *s32_base = charge ? sm.s32 + 8 * u2 : reinterpret_cast<const float *>(sm.zb);
    const uint32_t s32_stride = charge ? 16u : 0u;

    auto finish_round = [&](uint32_t k0, uint32_t kn) {
        group_barrier(group);
        const uint32_t n_warps_used = bpr < (uint32_t)kWarps ? bpr : kWarps;
        const uint32_t tid = threadIdx.x & (kWarps * 32 - 1);
        for (uint32_t idx = tid; idx < kn * 16; idx += kWarps * 32) {
            const uint32_t kk = idx >> 4, rr = idx & 15;
            if (rr >= ROWS) continue;
            const uint32_t row = (first_tile + (k0 + kk) * tile_stride) * ROWS + rr;
            if (row >= p.n_rows) continue;
            float sacc = 0.f;  // fixed order: deterministic
            for (uint32_t w2 = 0; w2 < n_warps_used; w2++)
#pragma unroll
                for (int tt = 0; tt < 4; tt++) sacc += partial[((kk * kWarps + w2) * 4 + tt) * 16 + rr];
            sacc *= sm.inv_scale[0];
            if (p.residual) sacc += p.residual[row];
            p.out[row] = sacc;
        }
        group_barrier(group);
    };

    if (nbw == 0) {
        for (uint32_t k0 = 0; k0 < my_tiles; k0 += kRoundSlots)
            finish_round(k0, (my_tiles - k0) < kRoundSlots ? (my_tiles - k0) : kRoundSlots);
        return;
    }

    float acc[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) acc[r] = 0.f;
    uint32_t k0 = 0, kn = my_tiles < kRoundSlots ? my_tiles : kRoundSlots;
    uint32_t in_slot = 0, slot = 0;
    for (uint32_t base = 0; base < total_units; base += DEPTH) {
#pragma unroll
        for (int i = 0; i < DEPTH; i++) {
            if (base + i < total_units) {
                const uint32_t blk = wid + kWarps * in_slot;
                consume_block<NR>(buf[i], bx_base + (size_t)blk * blk_stride, j_stride, s32_base + (size_t)blk * s32_stride, u2,
                                  acc);
                if (issued < total_units) {
                    issue_loads<NR>(buf[i], rowrec, bpr, wid + kWarps * lj, h, u);
                    issued++;
                    if (issued < total_units) advance();
                }
                if (++in_slot == nbw) {
#pragma unroll
                    for (int r = 0; r < NR; r++) {
                        partial[((slot * kWarps + wid) * 4 + t) * 16 + g + 8 * r] = acc[r];
                        acc[r] = 0.f;
                    }
                    in_slot = 0;
                    if (++slot == kn) {
                        finish_round(k0, kn);
                        k0 += kn;
                        kn = (my_tiles - k0) < kRoundSlots ? (my_tiles - k0) : kRoundSlots;
                        slot = 0;
                    }
                }
            }
        }
    }
}

template <int ROWS, int DEPTH>
cudaError_t launch_variant(const Q6kMmaParams &p, int sm_count, size_t smem, bool pdl, cudaStream_t s) {
    auto kern = qmv_q6k_mma_kernel<ROWS, DEPTH>;
    // the attribute belongs to the device, not the process: one flag per device ordinal
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
    uint32_t grid = (uint32_t)sm_count;
    const uint32_t want = (p.n_tiles + kGroups - 1) / kGroups;
    if (grid > want) grid = want;
    return launch_kernel(kern, dim3(grid), dim3(kThreadsCta), smem, s, pdl, p);
}

}  // namespace

bool q6k_stream_supported(uint32_t n_cols) { return n_cols % 256 == 0 && smem_bytes(n_cols) <= 200 * 1024; }

cudaError_t launch_q6k_stream(const Q6kPlanar &f, int sm_count, cudaStream_t s, uint64_t *launches) {
    if (f.n_rows == 0) return cudaSuccess;
    Q6kMmaParams p = {};
    // Tile height.  16-row tiles use the whole MMA and half the instructions per byte of 8-row tiles; they win
    // as soon as they keep about 60 % of the warp groups busy (measured: 4096 rows, 256 tiles for 296 groups,
    // 10-25 % faster with 16; 2048 rows, 128 tiles, faster with 8).  YULE_QMV_ROWS forces one (timing aid).
    const uint32_t n_groups = (uint32_t)kGroups * (uint32_t)sm_count;
    int tile_rows = ((f.n_rows / 16) * 10 >= n_groups * 6) ? 16 : 8;
    if (const char *force = knob("YULE_QMV_ROWS")) tile_rows = atoi(force) == 8 ? 8 : (atoi(force) == 16 ? 16 : tile_rows);
    p.planar = f.planar;
    p.out = f.out;
    p.n_rows = f.n_rows;
    p.n_cols = f.n_cols;
    p.n_tiles = (f.n_rows + tile_rows - 1) / tile_rows;
    p.x = f.x;
    p.norm_w = f.norm_w;
    p.eps = f.eps;
    p.residual = f.residual;
    for (int i = 0; i < 2; i++) {
        p.next_w[i] = f.next_w[i];
        p.next_bytes[i] = f.next_bytes[i];
    }
    const size_t smem = smem_bytes(f.n_cols);
    cudaError_t e = tile_rows == 8 ? launch_variant<8, 2>(p, sm_count, smem, f.pdl, s)
                                   : launch_variant<16, 2>(p, sm_count, smem, f.pdl, s);
    if (e != cudaSuccess) return e;
    *launches += 1;
    return cudaSuccess;
}

}  // namespace yule
