// q6k_ring_common.cuh — the Q6_K stage layout in shared memory, the activation image and the multiplication of one
// staged super-block, shared by qmv_q6k_ring.cu and decode_mega.cu.  Include inside namespace yule { namespace { … } }
// (decode_mega.cu wraps it in a namespace of its own: the names mirror those of the Q4_K headers).
#pragma once

constexpr int kWarps = 8;
constexpr int kGroups = 2;
constexpr int kThreadsCta = kGroups * kWarps * 32;
constexpr int kStageRows = 16;
constexpr int kStageBlocks = kWarps;
// planes of a stage: row pitches ≡ 32, 64, 16, 16 (mod 128) for the 16-byte reads at 64h+16u, 32h+16u, 0, 0
constexpr uint32_t kQlPitch = kStageBlocks * 128 + 32, kQhPitch = kStageBlocks * 64 + 64, kScPitch = kStageBlocks * 16 + 16,
                   kDPitch = 16;
constexpr uint32_t kQlOff = 0, kQhOff = kQlOff + kStageRows * kQlPitch, kScOff = kQhOff + kStageRows * kQhPitch,
                   kDOff = kScOff + kStageRows * kScPitch, kStageBytes = kDOff + kStageRows * kDPitch;  // 28 672
static_assert(kStageBytes % 128 == 0, "stages stay 128-byte aligned");

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// Row record of the row-planar copy.
__host__ __device__ inline uint32_t d_section_bytes(uint32_t bpr) { return (bpr * 2 + 15) & ~15u; }
__host__ __device__ inline size_t row_record_bytes(uint32_t bpr) { return (size_t)bpr * 208 + d_section_bytes(bpr); }

// Shared-memory image of the activation vector:
//   xh, xl   fp16 hi / lo of x·2^e in column order, 8 halves of padding after every 128 columns;
//            xl starts 64 bytes (mod 128) after xh, so the eight live lanes of a B load fall into
//            distinct banks;
//   s32      −32 · Σx over each 16-column scale group (fp32);
//   zb       zeros for lanes that feed an all-zero B column (and for the lanes that must not
//            charge the −32 term a second time).
struct XImage {
    __half *xh, *xl;
    float *s32;
    uint4 *zb;
    float *inv_scale;
    float *red;
};

__host__ __device__ inline uint32_t padded_cols(uint32_t n_cols) { return n_cols + 8 * (n_cols / 128); }
__host__ __device__ inline size_t x_plane_bytes(uint32_t n_cols) { return (((size_t)padded_cols(n_cols) * 2 + 127) / 128) * 128; }

// RMSNorm (optional), power-of-two normalisation, fp16 hi/lo split and per-16-column sums of x, by the
// whole CTA.  Each thread keeps its first kCache groups of 8 columns in registers between the reduction
// pass and the conversion pass; longer vectors re-read the remainder from L2.
// `load8(c, a)` fetches columns c..c+7 (plain loads in the matvec kernel, polled (value, epoch) pairs in the
// persistent decode kernel).
template <class Load8>
__device__ __forceinline__ void stage_activations(const XImage &sm, Load8 load8, uint32_t n_cols, const float *__restrict__ norm_w,
                                                  float eps) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    constexpr int NW = kThreadsCta / 32;
    constexpr int kCache = 2;
    if (threadIdx.x < 4) sm.zb[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);
    float cache[kCache][8];
    float ss = 0.f, mx = 0.f;
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

__device__ __forceinline__ uint32_t word4(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// One super-block of rows g and g+8 from the stage (`st`: stage base, `rb`: this lane's first row and the
// block slot already folded into the plane offsets) times this lane's 16 l-values of all four column groups.
//   bx   this lane's B source for the block: xh/xl + padded column of (blk, h, u), or the zero region
//   s32  −32·Σx of the eight scale groups this lane applies (or zeros)
__device__ __forceinline__ void consume_block_smem(const unsigned char *ql0, const unsigned char *qh0, const unsigned char *sc0,
                                                   const unsigned char *d0, const __half *bx, uint32_t j_stride, const float *s32,
                                                   int u2, float &acc0, float &acc1) {
    float dj[4][4];
#pragma unroll
    for (int j = 0; j < 4; j++) dj[j][0] = dj[j][1] = dj[j][2] = dj[j][3] = 0.f;
    {
        // rows g (index 0) and g + 8 (index 1) sit 8 row pitches apart in every plane
        const uint4 qa0 = *reinterpret_cast<const uint4 *>(ql0), qa1 = *reinterpret_cast<const uint4 *>(ql0 + 8 * kQlPitch);
        const uint4 qb0 = *reinterpret_cast<const uint4 *>(ql0 + 32), qb1 = *reinterpret_cast<const uint4 *>(ql0 + 8 * kQlPitch + 32);
        const uint4 h0 = *reinterpret_cast<const uint4 *>(qh0), h1 = *reinterpret_cast<const uint4 *>(qh0 + 8 * kQhPitch);
#pragma unroll
        for (int i4 = 0; i4 < 4; i4++) {
            // 6-bit values of the four column groups, four weights per word, one per byte
            uint32_t v[2][4];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const uint32_t qa = word4(r ? qa1 : qa0, i4), qb = word4(r ? qb1 : qb0, i4), qh = word4(r ? h1 : h0, i4);
                v[r][0] = (qa & 0x0F0F0F0Fu) | ((qh << 4) & 0x30303030u);
                v[r][1] = (qb & 0x0F0F0F0Fu) | ((qh << 2) & 0x30303030u);
                v[r][2] = ((qa >> 4) & 0x0F0F0F0Fu) | (qh & 0x30303030u);
                v[r][3] = ((qb >> 4) & 0x0F0F0F0Fu) | ((qh >> 2) & 0x30303030u);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint2 b = *reinterpret_cast<const uint2 *>(bx + j * j_stride + 4 * i4);
                // bytes → 16-bit lanes: {b0, b1} and {b2, b3}; the value is q·2^-24 as an fp16 subnormal
                mma_16816(dj[j], __byte_perm(v[0][j], 0u, 0x4140), __byte_perm(v[1][j], 0u, 0x4140),
                          __byte_perm(v[0][j], 0u, 0x4342), __byte_perm(v[1][j], 0u, 0x4342), b.x, b.y);
            }
        }
    }
    const float4 sa = *reinterpret_cast<const float4 *>(s32), sb = *reinterpret_cast<const float4 *>(s32 + 4);
    const float sg[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};  // index 2j + {0,1}
    const float k24 = 16777216.0f;
#pragma unroll
    for (int r = 0; r < 2; r++) {
        // the eight scales this lane applies: sc[8·u2 + 2j + {0,1}], signed bytes → float
        const uint2 scw = *reinterpret_cast<const uint2 *>(sc0 + r * 8 * kScPitch + 8 * u2);
        const uint32_t w0 = scw.x ^ 0x80808080u, w1 = scw.y ^ 0x80808080u;
        const float k = 8388608.0f + 128.0f;
        float scf[8];
        scf[0] = __uint_as_float(__byte_perm(w0, 0x4B000000u, 0x7440)) - k;
        scf[1] = __uint_as_float(__byte_perm(w0, 0x4B000000u, 0x7441)) - k;
        scf[2] = __uint_as_float(__byte_perm(w0, 0x4B000000u, 0x7442)) - k;
        scf[3] = __uint_as_float(__byte_perm(w0, 0x4B000000u, 0x7443)) - k;
        scf[4] = __uint_as_float(__byte_perm(w1, 0x4B000000u, 0x7440)) - k;
        scf[5] = __uint_as_float(__byte_perm(w1, 0x4B000000u, 0x7441)) - k;
        scf[6] = __uint_as_float(__byte_perm(w1, 0x4B000000u, 0x7442)) - k;
        scf[7] = __uint_as_float(__byte_perm(w1, 0x4B000000u, 0x7443)) - k;
        float tmp = 0.f;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // columns 2t and 2t+1 of D are scale groups (h = u2, u = 0) and (h = u2, u = 1) of group j
            tmp = fmaf(scf[2 * j], fmaf(dj[j][2 * r], k24, sg[2 * j]), tmp);
            tmp = fmaf(scf[2 * j + 1], fmaf(dj[j][2 * r + 1], k24, sg[2 * j + 1]), tmp);
        }
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(d0 + r * 8 * kDPitch)));
        if (r)
            acc1 = fmaf(d, tmp, acc1);
        else
            acc0 = fmaf(d, tmp, acc0);
    }
}
