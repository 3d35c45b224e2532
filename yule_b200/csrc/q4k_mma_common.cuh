// q4k_mma_common.cuh — device code shared by the Q4_K / Q5_K tensor-pipe matvec kernels
// (qmv_q4k_mma.cu: weights streamed through registers; qmv_q4k_ring.cu: weights staged in shared memory):
// fragment construction from packed nibbles, the 6-bit scale unpack, the shared-memory image of the
// activations and the tensor-parallel (value, epoch) pair helpers.  Include inside namespace yule { namespace { … } }.
#pragma once

constexpr int kWarps = 8;  // warps per group: one per super-block slot of a tile

__device__ __forceinline__ uint4 ld_stream_u4(const uint4 *p) {
    uint4 v;
    // L1-allocating on purpose: neighbouring 16-byte pieces share 32-byte sectors, and the second
    // request then merges with the first in L1 instead of going to L2 again.
    asm volatile("ld.global.nc.L1::evict_first.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_u2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::evict_first.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
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
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

// The three 16-byte pieces one lane needs from one super-block of one row.
// Q5_K (dequant.rs:297-338) adds the 32 bytes of fifth bits that sit between header and nibbles:
// bit s of byte l belongs to sub-block s, column l.  All four lanes of a row need all 32 bytes;
// each keeps a quarter (bytes 8t..8t+7) and hands words out by shuffle when the block is used.
struct BlockLoads {
    uint4 hdr, qa, qb;
    uint2 f;  // Q5_K only
};

template <int NR, bool Q5>  // rows per lane: 2 (ROWS = 16) or 1 (ROWS = 8)
__device__ __forceinline__ void issue_loads(BlockLoads (&ld)[NR], const uint4 *const (&rowp)[NR], uint32_t blk, int t) {
#pragma unroll
    for (int r = 0; r < NR; r++) {
        const uint4 *bp = rowp[r] + (size_t)blk * (Q5 ? 11 : 9);
        ld[r].hdr = ld_stream_u4(bp);
        if (Q5) ld[r].f = ld_stream_u2(reinterpret_cast<const uint2 *>(bp + 1) + t);
        ld[r].qa = ld_stream_u4(bp + (Q5 ? 3 : 1) + 2 * t);
        ld[r].qb = ld_stream_u4(bp + (Q5 ? 4 : 2) + 2 * t);
    }
}

// Fifth bits of the four columns of word wi for this lane's group t, moved to bit 0 of each byte:
// `.x` for the low-nibble sub-block 2t, `.y` for the high-nibble sub-block 2t+1.
// Word wi of the 32 bytes of fifth bits: it lives in lane (wi >> 1) of this row's quad; every lane of
// the warp takes part in the shuffle.
template <bool Q5>
__device__ __forceinline__ uint32_t fifth_word(const BlockLoads &b, int wi) {
    if (!Q5) return 0u;
    return __shfl_sync(0xFFFFFFFFu, (wi & 1) ? b.f.y : b.f.x, wi >> 1, 4);
}
template <bool Q5>
__device__ __forceinline__ uint2 fifth_of(const BlockLoads &b, int wi, int t) {
    if (!Q5) return make_uint2(0u, 0u);
    const uint32_t f = fifth_word<Q5>(b, wi) >> (2 * t);
    return make_uint2(f & 0x01010101u, (f >> 1) & 0x01010101u);
}

// Word wi (0..7) of the lane's 32 bytes of qs; wi is a compile-time constant after unrolling.
__device__ __forceinline__ uint32_t word_of(const BlockLoads &b, int wi) {
    switch (wi) {
        case 0: return b.qa.x;
        case 1: return b.qa.y;
        case 2: return b.qa.z;
        case 3: return b.qa.w;
        case 4: return b.qb.x;
        case 5: return b.qb.y;
        case 6: return b.qb.z;
        default: return b.qb.w;
    }
}

// Per-row constants of one super-block for this lane's 64-column group t.
struct RowScales {
    __half2 sc_lo, c_lo;  // low nibbles:  (1024+q)*sc_lo + c_lo          = q*sc[2t]
    __half2 sc_hi, c_hi;  // high nibbles: (1024+16q)*(sc/16) + (−64 sc)  = q*sc[2t+1]
    uint32_t mn;          // half2 {mn[2t], mn[2t+1]}
    float d, dmin;  // dmin carries the 2^6 that the stored column sums lack
};

// 6-bit scale/min unpack of yule-core/src/dequant.rs:176-190 for sub-blocks 2t and 2t+1, two
// bytes at a time.
__device__ __forceinline__ RowScales unpack_scales(const uint4 &hdr, int t) {
    const int sh = 16 * (t & 1);
    const uint32_t a0 = (hdr.y >> sh) & 0xFFFFu, a1 = (hdr.z >> sh) & 0xFFFFu, a2 = (hdr.w >> sh) & 0xFFFFu;
    uint32_t sc2, mn2;
    if (t < 2) {
        sc2 = a0 & 0x3F3Fu;
        mn2 = a1 & 0x3F3Fu;
    } else {
        sc2 = (a2 & 0x0F0Fu) | ((a0 >> 2) & 0x3030u);
        mn2 = ((a2 >> 4) & 0x0F0Fu) | ((a1 >> 2) & 0x3030u);
    }
    // bytes {v0, v1} → half2 {1024+v0, 1024+v1} → minus 1024
    const __half2 k1024 = __float2half2_rn(1024.0f);
    const __half2 sc = __hsub2(u32_as_h2(__byte_perm(sc2, 0x64u, 0x4140)), k1024);
    const __half2 mn = __hsub2(u32_as_h2(__byte_perm(mn2, 0x64u, 0x4140)), k1024);
    RowScales r;
    r.sc_lo = __low2half2(sc);
    r.c_lo = __hmul2(r.sc_lo, __float2half2_rn(-1024.0f));
    const __half2 sch = __high2half2(sc);
    r.sc_hi = __hmul2(sch, __float2half2_rn(0.0625f));
    r.c_hi = __hmul2(sch, __float2half2_rn(-64.0f));
    r.mn = h2_as_u32(mn);
    r.d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
    r.dmin = 64.0f * __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));  // sums are stored as Σ·2^-6
    return r;
}

// One word = 4 bytes = 4 low-nibble weights (columns c..c+3) + 4 high-nibble weights (c+32..).
// Fragment halves pair bytes (0,2) and (1,3); B is laid out to match.
// A fifth bit (Q5_K) is +16: mantissa bit 4 of 1024+q, bit 8 of 1024+16q; 31·63 < 2048 stays exact.
__device__ __forceinline__ void word_to_frags(uint32_t w, const RowScales &s, uint2 fifth, uint32_t &lo02, uint32_t &lo13,
                                              uint32_t &hi02, uint32_t &hi13) {
    const uint32_t magic = 0x64006400u;
    const uint32_t w8 = w >> 8;
    const uint32_t f_lo02 = (fifth.x & 0x00010001u) << 4, f_lo13 = ((fifth.x >> 8) & 0x00010001u) << 4;
    const uint32_t f_hi02 = (fifth.y & 0x00010001u) << 8, f_hi13 = ((fifth.y >> 8) & 0x00010001u) << 8;
    lo02 = h2_as_u32(__hfma2(u32_as_h2((w & 0x000F000Fu) | magic | f_lo02), s.sc_lo, s.c_lo));
    lo13 = h2_as_u32(__hfma2(u32_as_h2((w8 & 0x000F000Fu) | magic | f_lo13), s.sc_lo, s.c_lo));
    hi02 = h2_as_u32(__hfma2(u32_as_h2((w & 0x00F000F0u) | magic | f_hi02), s.sc_hi, s.c_hi));
    hi13 = h2_as_u32(__hfma2(u32_as_h2((w8 & 0x00F000F0u) | magic | f_hi13), s.sc_hi, s.c_hi));
}

// Shared-memory image of the activations for one CTA.  Per vector v:
//   xb[v]  uint4 index ((blk*2 + h)*4 + wp)*8 + part*4 + t  — for super-block blk, nibble half h
//          (0 = columns of the low nibbles), word pair wp, part (0 = hi, 1 = lo) and 64-column
//          group t: the B fragments of words 2wp and 2wp+1, i.e. halves
//          {x[c], x[c+2], x[c+1], x[c+3], x[c+4], x[c+6], x[c+5], x[c+7]}, c = 256 blk + 64 t + 32 h + 8 wp.
//          The eight (part, t) combinations a warp reads at once are 128 contiguous bytes.
//   sb[v]  half2 index (blk*2 + part)*4 + t = 2^-6 · {Σ sub-block 2t, Σ sub-block 2t+1}
//   inv_scale[v] = 2^-e
//   sf[v]  float index c/32 = Σ of the 32 columns (scaled by 2^e), for the batch-1 path
//   zb     64 zeroed uint4: B fragments of lanes that feed an all-zero column
struct SmemLayout {
    uint4 *xb;
    uint32_t *sb;
    float *sf;
    uint4 *zb;
    float *inv_scale;
    float *partial;  // [2 groups][kRoundSlots][kWarps][4 vectors][16 rows]
    float *red;      // reduction scratch, 2 × 32 floats
};

constexpr int kGroups = 2;       // independent 8-warp groups per CTA
constexpr int kRoundSlots = 8;   // (tile, matrix) slots whose partial sums a group holds at once

__host__ __device__ inline size_t xb_bytes(uint32_t n_cols, uint32_t nb) { return (size_t)nb * n_cols * 4; }
__host__ __device__ inline size_t sb_bytes(uint32_t n_cols, uint32_t nb) { return (size_t)nb * (n_cols / 32) * 4; }
constexpr size_t kZeroBytes = 64 * sizeof(uint4);
constexpr size_t kPartialBytes = (size_t)kGroups * kRoundSlots * kWarps * 4 * 16 * sizeof(float);

__device__ __forceinline__ SmemLayout carve(unsigned char *base, uint32_t n_cols, uint32_t nb) {
    SmemLayout s;
    size_t off = 0;
    s.xb = reinterpret_cast<uint4 *>(base);
    off += xb_bytes(n_cols, nb);
    s.sb = reinterpret_cast<uint32_t *>(base + off);
    off += sb_bytes(n_cols, nb);
    s.sf = reinterpret_cast<float *>(base + off);
    off += sb_bytes(n_cols, nb);
    off = (off + 15) & ~(size_t)15;
    s.zb = reinterpret_cast<uint4 *>(base + off);
    off += kZeroBytes;
    s.inv_scale = reinterpret_cast<float *>(base + off);
    off += 4 * sizeof(float);
    s.partial = reinterpret_cast<float *>(base + off);
    off += kPartialBytes;
    s.red = reinterpret_cast<float *>(base + off);
    return s;
}

size_t smem_bytes(uint32_t n_cols, uint32_t nb) {
    size_t off = xb_bytes(n_cols, nb) + 2 * sb_bytes(n_cols, nb);
    off = (off + 15) & ~(size_t)15;
    return off + kZeroBytes + 4 * sizeof(float) + kPartialBytes + 64 * sizeof(float) + 16;
}

constexpr int kThreadsCta = kGroups * kWarps * 32;  // 512

// Kept out of line: the tensor-parallel path must not cost the single-GPU kernels registers.
__device__ __noinline__ void tp_push_value(const TpFuse &tp, size_t o, float v) {
    const uint2 pair = make_uint2(__float_as_uint(v), *tp.tick * tp.epochs_per_tick + tp.push_index + 1u);
    for (uint32_t pp = 0; pp < tp.world; pp++)  // one 8-byte store each
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(tp.pair_out[pp] + o), "r"(pair.x), "r"(pair.y) : "memory");
}
// Eight consecutive elements of a gathered vector from its (value, epoch) pairs: polls until all eight
// carry `epoch`.  Bounded, and bounded once per failure: the first wait that runs out of `budget` cycles
// writes the status word, and every wait that starts (or polls) after that returns at once, so a lost peer
// costs one budget per kernel in flight, not one per wait.  The values returned after a give-up are
// whatever the buffer held; the host reads the status word and discards the step.
__device__ __forceinline__ void tp_load8(const uint2 *pairs, uint32_t epoch, int *status, long long budget, float (&a)[8]) {
    long long t0 = 0;
    for (uint32_t it = 0;; it++) {
        uint4 q[4];
        // one 16-byte load per two pairs: value and epoch of a pair must come from the same access
#pragma unroll
        for (int i = 0; i < 4; i++)
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(q[i].x), "=r"(q[i].y), "=r"(q[i].z), "=r"(q[i].w)
                         : "l"(pairs + 2 * i)
                         : "memory");
        bool ok = true;
#pragma unroll
        for (int i = 0; i < 4; i++) ok = ok && q[i].y == epoch && q[i].w == epoch;
        if (!ok) {
            if (it == 0) t0 = clock64();
            if (it != 0 && (it & 63u) != 63u) continue;
            if (*reinterpret_cast<volatile int *>(status) == 0) {
                if (clock64() - t0 < budget) continue;
                atomicCAS(status, 0, kStatusPeerTimeout);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            a[2 * i] = __uint_as_float(q[i].x);
            a[2 * i + 1] = __uint_as_float(q[i].z);
        }
        return;
    }
}

// Stage NB activation vectors: optional RMSNorm, power-of-two normalisation, hi/lo split,
// fragment order, per-32-column sums.  Each thread owns groups of 8 consecutive columns; the first
// kCache groups (16 K columns per CTA) stay in registers between the reduction pass and the
// conversion pass, so x is fetched from L2 only once; longer vectors re-read the remainder.
constexpr int kCache = 4;

template <bool TP, int KC = kCache>
__device__ __forceinline__ void stage_activations(const SmemLayout &sm, const float *__restrict__ x, uint32_t x_stride,
                                                  uint32_t n_cols, uint32_t nb, const float *__restrict__ norm_w,
                                                  float eps, const uint2 *pairs = nullptr, uint32_t pair_epoch = 0,
                                                  int *status = nullptr, long long budget = 0,
                                                  unsigned long long *prof = nullptr) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    constexpr int NW = kThreadsCta / 32;
    if (threadIdx.x < 64) sm.zb[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);
    for (uint32_t v = 0; v < nb; v++) {
        const float *xv = x + (size_t)v * x_stride;
        float cache[KC][8];
        float ss = 0.f, mx = 0.f;
        auto load8 = [&](uint32_t c, float (&a)[8]) {
            if (TP && pairs) {  // tensor parallelism: the vector arrives as (value, epoch) pairs stored by all ranks
                tp_load8(pairs + c, pair_epoch, status, budget, a);
                return;
            }
            *reinterpret_cast<float4 *>(a) = *reinterpret_cast<const float4 *>(xv + c);
            *reinterpret_cast<float4 *>(a + 4) = *reinterpret_cast<const float4 *>(xv + c + 4);
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
        for (int k = 0; k < KC; k++) {
            const uint32_t c = (threadIdx.x + k * kThreadsCta) * 8;
            if (c < n_cols) {
                load8(c, cache[k]);
                reduce8(c, cache[k]);
            }
        }
        for (uint32_t c = (threadIdx.x + KC * kThreadsCta) * 8; c < n_cols; c += kThreadsCta * 8) {
            float a[8];
            load8(c, a);
            reduce8(c, a);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        if (prof && (threadIdx.x & 255) == 0) prof[0] = clock64();
        __syncthreads();  // previous vector's readers of `red` are done
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
        // RMSNorm scale exactly as the CPU runner forms it: 1 / sqrt(ss / n + eps)
        const float inv_rms = norm_w ? 1.0f / sqrtf(ss / (float)n_cols + eps) : 1.0f;
        mx *= inv_rms;
        // 2^e with max|x|·2^e in [2^13, 2^14); exponent clamped so both 2^e and 2^-e stay finite normals
        int eb = (int)((__float_as_uint(mx) >> 23) & 0xFFu);
        if (mx == 0.f || eb == 0xFF) eb = 127 + 13;
        int se = 127 + 13 - (eb - 127);
        se = se < 1 ? 1 : (se > 253 ? 253 : se);
        const float scale = __uint_as_float((uint32_t)se << 23);
        const float inv_scale = __uint_as_float((uint32_t)(254 - se) << 23);
        if (threadIdx.x == 0) sm.inv_scale[v] = inv_scale;
        if (prof && (threadIdx.x & 255) == 0) prof[1] = clock64();
        uint4 *xb = sm.xb + (size_t)v * (n_cols / 4);
        __half *sbh = reinterpret_cast<__half *>(sm.sb + (size_t)v * (n_cols / 32));
        float *sf = sm.sf + (size_t)v * (n_cols / 32);
        auto convert8 = [&](uint32_t c, float (&a)[8]) {
            if (norm_w) {
                float gw[8];
                *reinterpret_cast<float4 *>(gw) = *reinterpret_cast<const float4 *>(norm_w + c);
                *reinterpret_cast<float4 *>(gw + 4) = *reinterpret_cast<const float4 *>(norm_w + c + 4);
                // x * inv * w, rounded in that order (yule-infer/src/model_runner.rs:273)
#pragma unroll
                for (int i = 0; i < 8; i++) a[i] = a[i] * inv_rms * gw[i];
            }
            __half hi[8], lo[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                a[i] *= scale;  // exact (power of two)
                hi[i] = __float2half_rn(a[i]);
                lo[i] = __float2half_rn(a[i] - __half2float(hi[i]));
            }
            float s8 = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
            const uint32_t blk = c >> 8, t = (c >> 6) & 3, h = (c >> 5) & 1, wp = (c >> 3) & 3;
            const uint32_t idx = ((blk * 2 + h) * 4 + wp) * 8 + t;
            xb[idx] = make_uint4(h2_as_u32(__halves2half2(hi[0], hi[2])), h2_as_u32(__halves2half2(hi[1], hi[3])),
                                 h2_as_u32(__halves2half2(hi[4], hi[6])), h2_as_u32(__halves2half2(hi[5], hi[7])));
            xb[idx + 4] = make_uint4(h2_as_u32(__halves2half2(lo[0], lo[2])), h2_as_u32(__halves2half2(lo[1], lo[3])),
                                     h2_as_u32(__halves2half2(lo[4], lo[6])), h2_as_u32(__halves2half2(lo[5], lo[7])));
            // Σ over 32 columns: 4 consecutive threads hold one sub-block
            s8 += __shfl_xor_sync(0xffffffffu, s8, 1);
            s8 += __shfl_xor_sync(0xffffffffu, s8, 2);
            if ((lane & 3) == 0) {
                sf[c >> 5] = s8;
                // 32 values below 2^14 can sum to 2^19: keep Σ·2^-6 (exact) so fp16 cannot overflow;
                // unpack_scales folds the 2^6 back into dmin
                s8 *= 0.015625f;
                const __half sh = __float2half_rn(s8);
                const uint32_t sub = (c >> 5) & 7;  // sub-block within the super-block
                const uint32_t hidx = ((blk * 2 + 0) * 4 + (sub >> 1)) * 2 + (sub & 1);
                sbh[hidx] = sh;
                sbh[hidx + 8] = __float2half_rn(s8 - __half2float(sh));  // part 1 sits 4 half2 further on
            }
        };
        // n_cols is a multiple of 256, so whole warps are in or out of every step (the shuffles are safe)
#pragma unroll
        for (int k = 0; k < KC; k++) {
            const uint32_t c = (threadIdx.x + k * kThreadsCta) * 8;
            if (c < n_cols) convert8(c, cache[k]);
        }
        for (uint32_t c = (threadIdx.x + KC * kThreadsCta) * 8; c < n_cols; c += kThreadsCta * 8) {
            float a[8];
            load8(c, a);
            convert8(c, a);
        }
    }
    __syncthreads();
}

// Multiply one super-block (this lane's rows × 64-column group) into the running sums.
template <int NR, bool Q5>
__device__ __forceinline__ void consume_block(const BlockLoads (&ld)[NR], uint32_t blk, int t, const uint4 *xb_lane,
                                              const uint32_t *sb_lane, float (&acc)[NR][2]) {
    RowScales rs[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) rs[r] = unpack_scales(ld[r].hdr, t);

    // two independent accumulator chains (low-nibble and high-nibble MMAs)
    float dl[4] = {0.f, 0.f, 0.f, 0.f}, dh[4] = {0.f, 0.f, 0.f, 0.f}, dm[4] = {0.f, 0.f, 0.f, 0.f};
    const uint4 *bp = xb_lane + (size_t)blk * 64;  // 2 halves × 4 word pairs × 8 lanes-groups
#pragma unroll
    for (int wp = 0; wp < 4; wp++) {
        const uint4 bl = bp[wp * 8], bh = bp[32 + wp * 8];
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int wi = 2 * wp + e;
            uint32_t lo02[2], lo13[2], hi02[2], hi13[2];
#pragma unroll
            for (int r = 0; r < NR; r++) {
                const uint32_t w = word_of(ld[r], wi);
                word_to_frags(w, rs[r], fifth_of<Q5>(ld[r], wi, t), lo02[r], lo13[r], hi02[r], hi13[r]);
            }
            if (NR == 1) lo02[1] = lo13[1] = hi02[1] = hi13[1] = 0u;
            mma_16816(dl, lo02[0], lo02[1], lo13[0], lo13[1], e ? bl.z : bl.x, e ? bl.w : bl.y);
            mma_16816(dh, hi02[0], hi02[1], hi13[0], hi13[1], e ? bh.z : bh.x, e ? bh.w : bh.y);
        }
    }
    // mins: k slots 2t, 2t+1 carry sub-blocks 2t, 2t+1; the other slots are zero
    const uint32_t sx = sb_lane[(size_t)blk * 8];
    mma_16816(dm, rs[0].mn, NR == 2 ? rs[NR - 1].mn : 0u, 0u, 0u, sx, 0u);
    acc[0][0] = fmaf(rs[0].d, dl[0] + dh[0], acc[0][0]);
    acc[0][0] = fmaf(-rs[0].dmin, dm[0], acc[0][0]);
    acc[0][1] = fmaf(rs[0].d, dl[1] + dh[1], acc[0][1]);
    acc[0][1] = fmaf(-rs[0].dmin, dm[1], acc[0][1]);
    if (NR == 2) {
        acc[NR - 1][0] = fmaf(rs[NR - 1].d, dl[2] + dh[2], acc[NR - 1][0]);
        acc[NR - 1][0] = fmaf(-rs[NR - 1].dmin, dm[2], acc[NR - 1][0]);
        acc[NR - 1][1] = fmaf(rs[NR - 1].d, dl[3] + dh[3], acc[NR - 1][1]);
        acc[NR - 1][1] = fmaf(-rs[NR - 1].dmin, dm[3], acc[NR - 1][1]);
    }
}

// ── batch-1 path: sub-blocks in the N dimension ─────────────────────────────────────────────
// B column n = 4·part + t' carries x (part 0 = hi, 1 = lo) only at the k slots that lane t' feeds,
// zeros elsewhere.  Those slots belong to one sub-block (2t' for the low-nibble MMA, 2t'+1 for the
// high-nibble one), so D[row][n] is that sub-block's Σ q·x whatever the k order — and the weights
// go in unscaled: the nibble's bits are used as an fp16 subnormal (q·2^-24, or 16q·2^-24 for a
// high nibble), one AND per pair of weights.  Lane (g, t) ends up with columns 2t, 2t+1 =
// groups 2u, 2u+1 (u = t&1) of part t>>1, i.e. sub-blocks 4u..4u+3, and applies their scales.
struct RowScalesF {
    float sc[4];  // sc[4u + i] · d · 2^24 (i even: low-nibble MMAs) or · d · 2^20 (i odd)
    float mn[4];  // mn[4u + i] · dmin, zero in the lanes of the lo part (mins are charged once)
};

template <bool Q5>
__device__ __forceinline__ RowScalesF unpack_scales_f(const uint4 &hdr, int u, bool charge_mins) {
    uint32_t sc4, mn4;  // four 6-bit values each, one per byte (dequant.rs:176-190)
    if (u == 0) {
        sc4 = hdr.y & 0x3F3F3F3Fu;
        mn4 = hdr.z & 0x3F3F3F3Fu;
    } else {
        sc4 = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
        mn4 = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
    }
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
    const float dmin = charge_mins ? __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16))) : 0.f;
    // Q5_K operands carry q·2^-24 in both halves; Q4_K's high nibbles stay in place (16q·2^-24)
    const float d24 = d * 16777216.0f, d20 = Q5 ? d24 : d * 1048576.0f;
    const float k23 = 8388608.0f;
    RowScalesF r;
    r.sc[0] = (__uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7440)) - k23) * d24;
    r.sc[1] = (__uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7441)) - k23) * d20;
    r.sc[2] = (__uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7442)) - k23) * d24;
    r.sc[3] = (__uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7443)) - k23) * d20;
    r.mn[0] = (__uint_as_float(__byte_perm(mn4, 0x4B000000u, 0x7440)) - k23) * dmin;
    r.mn[1] = (__uint_as_float(__byte_perm(mn4, 0x4B000000u, 0x7441)) - k23) * dmin;
    r.mn[2] = (__uint_as_float(__byte_perm(mn4, 0x4B000000u, 0x7442)) - k23) * dmin;
    r.mn[3] = (__uint_as_float(__byte_perm(mn4, 0x4B000000u, 0x7443)) - k23) * dmin;
    return r;
}

template <int NR, bool Q5>
__device__ __forceinline__ void consume_block_subcol(const BlockLoads (&ld)[NR], const uint4 *bp, const float *sfp, int u,
                                                     int t, bool charge_mins, float (&acc)[NR][2]) {
    float dl[4] = {0.f, 0.f, 0.f, 0.f}, dh[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int wp = 0; wp < 4; wp++) {
        const uint4 bl = bp[wp * 8], bh = bp[32 + wp * 8];
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int wi = 2 * wp + e;
            uint32_t lo02[2], lo13[2], hi02[2], hi13[2];
#pragma unroll
            for (int r = 0; r < NR; r++) {
                const uint32_t w = word_of(ld[r], wi), w8 = w >> 8;
                if (Q5) {
                    // four 5-bit values per register first (nibble | fifth bit << 4), then one byte
                    // permute per operand: both halves of the word are q·2^-24 (no factor 16 on the
                    // high nibbles, see unpack_scales_f)
                    const uint32_t f = fifth_word<Q5>(ld[r], wi) >> (2 * t);
                    const uint32_t cl = (w & 0x0F0F0F0Fu) | ((f << 4) & 0x10101010u);
                    const uint32_t ch = ((w >> 4) & 0x0F0F0F0Fu) | ((f << 3) & 0x10101010u);
                    lo02[r] = __byte_perm(cl, 0u, 0x4240);
                    lo13[r] = __byte_perm(cl, 0u, 0x4341);
                    hi02[r] = __byte_perm(ch, 0u, 0x4240);
                    hi13[r] = __byte_perm(ch, 0u, 0x4341);
                } else {
                    lo02[r] = w & 0x000F000Fu;
                    lo13[r] = w8 & 0x000F000Fu;
                    hi02[r] = w & 0x00F000F0u;
                    hi13[r] = w8 & 0x00F000F0u;
                }
            }
            if (NR == 1) lo02[1] = lo13[1] = hi02[1] = hi13[1] = 0u;
            mma_16816(dl, lo02[0], lo02[1], lo13[0], lo13[1], e ? bl.z : bl.x, e ? bl.w : bl.y);
            mma_16816(dh, hi02[0], hi02[1], hi13[0], hi13[1], e ? bh.z : bh.x, e ? bh.w : bh.y);
        }
    }
    const float4 sx = *reinterpret_cast<const float4 *>(sfp);  // Σx of sub-blocks 4u..4u+3
#pragma unroll
    for (int r = 0; r < NR; r++) {
        const RowScalesF rs = unpack_scales_f<Q5>(ld[r].hdr, u, charge_mins);
        float a = acc[r][0];
        a = fmaf(rs.sc[0], dl[2 * r + 0], a);
        a = fmaf(rs.sc[1], dh[2 * r + 0], a);
        a = fmaf(rs.sc[2], dl[2 * r + 1], a);
        a = fmaf(rs.sc[3], dh[2 * r + 1], a);
        float m = rs.mn[0] * sx.x;
        m = fmaf(rs.mn[1], sx.y, m);
        m = fmaf(rs.mn[2], sx.z, m);
        m = fmaf(rs.mn[3], sx.w, m);
        acc[r][0] = a - m;
    }
}
