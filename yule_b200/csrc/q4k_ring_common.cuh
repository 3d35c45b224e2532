// q4k_ring_common.cuh — the Q4_K stage layout in shared memory and the multiplication of one staged super-block,
// shared by qmv_q4k_ring.cu and decode_mega.cu.  Include after q4k_mma_common.cuh, inside the same namespace.
#pragma once

constexpr int kStageRows = 16;
constexpr int kStageBlocks = kWarps;                                // super-blocks per row in a stage
constexpr uint32_t kRowPitch = kStageBlocks * 144 + 16;             // ≡ 16 (mod 128)
constexpr uint32_t kStageBytes = kStageRows * kRowPitch;            // 18 688

__device__ __forceinline__ uint32_t word4(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// One super-block of rows g and g+8 (r0, r1: the block's bytes in the ring) times this lane's 64-column
// group, in the sub-block-per-column formulation of consume_block_subcol — same MMA order, so the same
// bits — with the nibbles fetched from shared memory 16 bytes at a time, just before they are used.
__device__ __forceinline__ void consume_block_smem(const unsigned char *r0, const unsigned char *r1, const uint4 *bp,
                                                   const float *sfp, int u, int t, bool charge_mins, float &acc0, float &acc1) {
    float dl[4] = {0.f, 0.f, 0.f, 0.f}, dh[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const uint4 q0 = *reinterpret_cast<const uint4 *>(r0 + 16 + 32 * t + 16 * half);
        const uint4 q1 = *reinterpret_cast<const uint4 *>(r1 + 16 + 32 * t + 16 * half);
#pragma unroll
        for (int w2 = 0; w2 < 2; w2++) {
            const int wp = 2 * half + w2;
            const uint4 bl = bp[wp * 8], bh = bp[32 + wp * 8];
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const uint32_t a = word4(q0, 2 * w2 + e), b = word4(q1, 2 * w2 + e);
                const uint32_t a8 = a >> 8, b8 = b >> 8;
                mma_16816(dl, a & 0x000F000Fu, b & 0x000F000Fu, a8 & 0x000F000Fu, b8 & 0x000F000Fu, e ? bl.z : bl.x,
                          e ? bl.w : bl.y);
                mma_16816(dh, a & 0x00F000F0u, b & 0x00F000F0u, a8 & 0x00F000F0u, b8 & 0x00F000F0u, e ? bh.z : bh.x,
                          e ? bh.w : bh.y);
            }
        }
    }
    const float4 sx = *reinterpret_cast<const float4 *>(sfp);  // Σx of sub-blocks 4u..4u+3
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const uint4 hdr = *reinterpret_cast<const uint4 *>(r ? r1 : r0);
        const RowScalesF rs = unpack_scales_f<false>(hdr, u, charge_mins);
        float a = r ? acc1 : acc0;
        a = fmaf(rs.sc[0], dl[2 * r + 0], a);
        a = fmaf(rs.sc[1], dh[2 * r + 0], a);
        a = fmaf(rs.sc[2], dl[2 * r + 1], a);
        a = fmaf(rs.sc[3], dh[2 * r + 1], a);
        float m = rs.mn[0] * sx.x;
        m = fmaf(rs.mn[1], sx.y, m);
        m = fmaf(rs.mn[2], sx.z, m);
        m = fmaf(rs.mn[3], sx.w, m);
        if (r)
            acc1 = a - m;
        else
            acc0 = a - m;
    }
}
