// synth.cpp — seeded synthetic GGUF tensors for tests and benchmarks (host only, no CUDA).
//
// Yule ships dequantisers but no quantiser (yule-core/src/dequant.rs), and no model file is
// available offline, so benchmarks and tests need (a) blocks with random fields of the right
// distributions and (b) a quantiser that turns N(0, σ) weights into valid Q4_K / Q6_K / Q4_0 /
// Q8_0 blocks.  Both sides of every comparison consume the same bytes, so the quantiser's
// quality does not enter parity; it only has to produce realistic, valid blocks.
//
// Every value is a pure function of (seed, element index) — SplitMix64 of a counter — so the
// output does not depend on the number of threads.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
inline uint64_t rnd(uint64_t seed, uint64_t idx) { return splitmix64(seed * 0xD1342543DE82EF95ull + idx); }
inline double uniform01(uint64_t r) { return ((r >> 11) + 0.5) * (1.0 / 9007199254740992.0); }
// Standard normal from two counters (Box–Muller).
inline float normal(uint64_t seed, uint64_t idx) {
    double u1 = uniform01(rnd(seed, 2 * idx)), u2 = uniform01(rnd(seed, 2 * idx + 1));
    return (float)(std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
}

// f32 → f16 bits, round to nearest even, subnormals kept, overflow to inf.
inline uint16_t f32_to_f16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    int32_t e = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    uint32_t m = x & 0x7FFFFFu;
    if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (m ? 0x200u : 0));
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        m |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)e << 10) | (m >> 13);
    uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
    return (uint16_t)(sign | half);
}
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1F, m = h & 0x3FFu, out;
    if (e == 0) {
        if (m == 0) {
            out = sign;
        } else {
            int sh = 0;
            while (!(m & 0x400u)) {
                m <<= 1;
                sh++;
            }
            out = sign | ((uint32_t)(113 - sh) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (e == 31) {
        out = sign | 0x7F800000u | (m << 13);
    } else {
        out = sign | ((e + 112) << 23) | (m << 13);
    }
    float f;
    std::memcpy(&f, &out, 4);
    return f;
}
inline void put_f16(uint8_t *p, uint16_t h) {
    p[0] = (uint8_t)(h & 0xFF);
    p[1] = (uint8_t)(h >> 8);
}

int block_size(int t) {
    switch (t) {
        case 2: case 3: case 6: case 7: case 8: case 9: return 32;
        case 10: case 11: case 12: case 13: case 14: return 256;
        default: return 0;
    }
}
int block_bytes(int t) {
    switch (t) {
        case 2: return 18;
        case 3: return 20;
        case 6: return 22;
        case 7: return 24;
        case 8: return 34;
        case 9: return 36;
        case 10: return 84;
        case 11: return 110;
        case 12: return 144;
        case 13: return 176;
        case 14: return 210;
        default: return 0;
    }
}

template <class F>
void parallel_for(uint64_t n, int n_threads, F fn) {
    if (n_threads <= 0) n_threads = (int)std::max(1u, std::thread::hardware_concurrency());
    n_threads = (int)std::min<uint64_t>((uint64_t)n_threads, std::max<uint64_t>(1, n / 64));
    if (n_threads <= 1) {
        fn(0, n);
        return;
    }
    std::vector<std::thread> th;
    uint64_t chunk = (n + n_threads - 1) / n_threads;
    for (int t = 0; t < n_threads; t++) {
        uint64_t b = t * chunk, e = std::min(n, b + chunk);
        if (b >= e) break;
        th.emplace_back([=] { fn(b, e); });
    }
    for (auto &t : th) t.join();
}

// ── random-field blocks (matvec sweeps): scales f16(|N(0, scale_std)|), every other byte uniform ──
void random_block(int type, uint64_t seed, uint64_t blk, float scale_std, uint8_t *out) {
    const int bb = block_bytes(type);
    const uint64_t base = blk * 64;  // 64 counters per block: 0..1 normals, 2.. raw bytes
    for (int i = 0; i < bb; i += 8) {
        uint64_t r = rnd(seed ^ 0xA5A5A5A5ull, base * 8 + (uint64_t)i);
        for (int k = 0; k < 8 && i + k < bb; k++) out[i + k] = (uint8_t)(r >> (8 * k));
    }
    uint16_t d = f32_to_f16(std::fabs(normal(seed, 2 * blk)) * scale_std);
    uint16_t dm = f32_to_f16(std::fabs(normal(seed, 2 * blk + 1)) * scale_std);
    switch (type) {
        case 3: case 7: case 9: case 12: case 13:  // d then m / s / dmin
            put_f16(out, d);
            put_f16(out + 2, dm);
            break;
        case 10:
            put_f16(out + 80, d);
            put_f16(out + 82, dm);
            break;
        case 11: put_f16(out + 108, d); break;
        case 14: put_f16(out + 208, d); break;
        default: put_f16(out, d); break;
    }
}

// ── quantisers (this project's own; simple min/max encoders) ──────────────────────────────────
inline int nearest(float v) { return (int)std::lrintf(v); }

void quantize_q8_0(const float *x, uint8_t *out) {
    float amax = 0.f;
    for (int i = 0; i < 32; i++) amax = std::max(amax, std::fabs(x[i]));
    uint16_t dh = f32_to_f16(amax / 127.0f);
    float d = f16_to_f32(dh), id = d > 0 ? 1.0f / d : 0.f;
    put_f16(out, dh);
    for (int i = 0; i < 32; i++) out[2 + i] = (uint8_t)(int8_t)std::clamp(nearest(x[i] * id), -127, 127);
}

// Yule's Q4_0 nibble order: weight i in byte i/2, even i in the low nibble (dequant.rs:77-86).
void quantize_q4_0(const float *x, uint8_t *out) {
    float amax = 0.f;
    for (int i = 0; i < 32; i++) amax = std::max(amax, std::fabs(x[i]));
    uint16_t dh = f32_to_f16(amax / 7.0f);
    float d = f16_to_f32(dh), id = d > 0 ? 1.0f / d : 0.f;
    put_f16(out, dh);
    std::memset(out + 2, 0, 16);
    for (int i = 0; i < 32; i++) {
        int q = std::clamp(nearest(x[i] * id) + 8, 0, 15);
        out[2 + i / 2] |= (uint8_t)(q << (4 * (i & 1)));
    }
}

// Q4_K (levels 15) and Q5_K (levels 31): same scales, Q5_K keeps bit 4 of weight (s, l) in bit s of qh[l].
void quantize_q45_k(const float *x, uint8_t *out, int levels) {
    float scale[8], mn[8], max_scale = 0.f, max_min = 0.f;
    for (int s = 0; s < 8; s++) {
        float lo = x[32 * s], hi = x[32 * s];
        for (int i = 1; i < 32; i++) {
            lo = std::min(lo, x[32 * s + i]);
            hi = std::max(hi, x[32 * s + i]);
        }
        mn[s] = std::max(0.f, -lo);
        scale[s] = (hi + mn[s]) / (float)levels;
        max_scale = std::max(max_scale, scale[s]);
        max_min = std::max(max_min, mn[s]);
    }
    uint16_t dh = f32_to_f16(max_scale / 63.0f), dmh = f32_to_f16(max_min / 63.0f);
    float d = f16_to_f32(dh), dmin = f16_to_f32(dmh);
    uint8_t sc[8], m[8];
    for (int s = 0; s < 8; s++) {
        sc[s] = (uint8_t)std::clamp(d > 0 ? nearest(scale[s] / d) : 0, 0, 63);
        m[s] = (uint8_t)std::clamp(dmin > 0 ? nearest(mn[s] / dmin) : 0, 0, 63);
    }
    put_f16(out, dh);
    put_f16(out + 2, dmh);
    // inverse of the 6-bit unpack of dequant.rs:176-190
    uint8_t *q = out + 4;
    for (int j = 0; j < 4; j++) {
        q[j] = (uint8_t)(sc[j] | ((sc[j + 4] >> 4) << 6));
        q[j + 4] = (uint8_t)(m[j] | ((m[j + 4] >> 4) << 6));
        q[j + 8] = (uint8_t)((sc[j + 4] & 0xF) | ((m[j + 4] & 0xF) << 4));
    }
    for (int g = 0; g < 4; g++) {
        for (int l = 0; l < 32; l++) {
            int qs[2];
            for (int h = 0; h < 2; h++) {
                int s = 2 * g + h;
                float ds = d * (float)sc[s], ms = dmin * (float)m[s];
                qs[h] = ds > 0 ? std::clamp(nearest((x[64 * g + 32 * h + l] + ms) / ds), 0, levels) : 0;
            }
            if (levels == 15) {
                out[16 + 32 * g + l] = (uint8_t)(qs[0] | (qs[1] << 4));
            } else {
                if (g == 0) out[16 + l] = 0;
                out[16 + l] |= (uint8_t)(((qs[0] >> 4) << (2 * g)) | ((qs[1] >> 4) << (2 * g + 1)));
                out[48 + 32 * g + l] = (uint8_t)((qs[0] & 15) | ((qs[1] & 15) << 4));
            }
        }
    }
}

// Legacy 5-bit and asymmetric formats (dequant.rs:91-138): qh bit i is bit 4 of weight i.
void quantize_q5_0(const float *x, uint8_t *out) {
    float amax = 0.f;
    for (int i = 0; i < 32; i++) amax = std::max(amax, std::fabs(x[i]));
    uint16_t dh = f32_to_f16(amax / 15.0f);
    float d = f16_to_f32(dh), id = d > 0 ? 1.0f / d : 0.f;
    put_f16(out, dh);
    std::memset(out + 2, 0, 20);
    for (int i = 0; i < 32; i++) {
        int q = std::clamp(nearest(x[i] * id) + 16, 0, 31);
        out[2 + i / 8] |= (uint8_t)((q >> 4) << (i & 7));
        out[6 + i / 2] |= (uint8_t)((q & 15) << (4 * (i & 1)));
    }
}
void quantize_q45_1(const float *x, uint8_t *out, int levels) {
    float lo = x[0], hi = x[0];
    for (int i = 1; i < 32; i++) {
        lo = std::min(lo, x[i]);
        hi = std::max(hi, x[i]);
    }
    uint16_t dh = f32_to_f16((hi - lo) / (float)levels), mh = f32_to_f16(lo);
    float d = f16_to_f32(dh), m = f16_to_f32(mh), id = d > 0 ? 1.0f / d : 0.f;
    put_f16(out, dh);
    put_f16(out + 2, mh);
    const int qs_off = levels == 15 ? 4 : 8;
    std::memset(out + 4, 0, levels == 15 ? 16 : 20);
    for (int i = 0; i < 32; i++) {
        int q = std::clamp(nearest((x[i] - m) * id), 0, levels);
        if (levels == 31) out[4 + i / 8] |= (uint8_t)((q >> 4) << (i & 7));
        out[qs_off + i / 2] |= (uint8_t)((q & 15) << (4 * (i & 1)));
    }
}

void quantize_q6_k(const float *x, uint8_t *out) {
    float scale[16], max_abs_scale = 0.f;
    for (int s = 0; s < 16; s++) {
        float amax = 0.f;
        for (int i = 0; i < 16; i++) amax = std::max(amax, std::fabs(x[16 * s + i]));
        scale[s] = amax / 31.0f;
        max_abs_scale = std::max(max_abs_scale, scale[s]);
    }
    uint16_t dh = f32_to_f16(max_abs_scale / 127.0f);
    float d = f16_to_f32(dh);
    int8_t sc[16];
    for (int s = 0; s < 16; s++) sc[s] = (int8_t)std::clamp(d > 0 ? nearest(scale[s] / d) : 0, 0, 127);
    std::memset(out, 0, 192);
    for (int s = 0; s < 16; s++) out[192 + s] = (uint8_t)sc[s];
    put_f16(out + 208, dh);
    // column c = 128h + 32g + l uses scale index 8h + l/16 + 2g = c/16 (dequant.rs:346-372)
    for (int c = 0; c < 256; c++) {
        float ds = d * (float)sc[c / 16];
        int q = ds > 0 ? std::clamp(nearest(x[c] / ds), -32, 31) + 32 : 32;
        int h = c / 128, r = c % 128, g = r / 32, l = r % 32;
        out[64 * h + l + 32 * (g & 1)] |= (uint8_t)((q & 0xF) << (4 * (g >> 1)));
        out[128 + 32 * h + l] |= (uint8_t)((q >> 4) << (2 * g));
    }
}

void quantize_block(int type, const float *x, uint8_t *out) {
    switch (type) {
        case 2: quantize_q4_0(x, out); break;
        case 8: quantize_q8_0(x, out); break;
        case 3: quantize_q45_1(x, out, 15); break;
        case 6: quantize_q5_0(x, out); break;
        case 7: quantize_q45_1(x, out, 31); break;
        case 12: quantize_q45_k(x, out, 15); break;
        case 13: quantize_q45_k(x, out, 31); break;
        case 14: quantize_q6_k(x, out); break;
    }
}

bool has_quantizer(int t) { return t == 2 || t == 3 || t == 6 || t == 7 || t == 8 || t == 12 || t == 13 || t == 14; }

}  // namespace

extern "C" {

// n floats ~ N(mean, std), element i a function of (seed, i) only.
void ys_fill_normal(uint64_t seed, float mean, float std_, float *out, uint64_t n, int n_threads) {
    parallel_for(n, n_threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; i++) out[i] = mean + std_ * normal(seed, i);
    });
}

// n uniform integers in [0, bound).
void ys_fill_tokens(uint64_t seed, uint32_t bound, uint32_t *out, uint64_t n) {
    for (uint64_t i = 0; i < n; i++) out[i] = (uint32_t)(rnd(seed, i) % bound);
}

// n_blocks blocks with random fields: f16 scales |N(0, scale_std)|, all other bytes uniform.
int ys_random_blocks(int type, uint64_t seed, float scale_std, uint8_t *out, uint64_t n_blocks, int n_threads) {
    const int bb = block_bytes(type);
    if (!bb) return -1;
    parallel_for(n_blocks, n_threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; i++) random_block(type, seed, i, scale_std, out + i * (uint64_t)bb);
    });
    return 0;
}

// Quantise n floats (a multiple of the block size) into blocks.
int ys_quantize(int type, const float *x, uint64_t n, uint8_t *out, int n_threads) {
    const int bs = block_size(type), bb = block_bytes(type);
    if (!bs || !has_quantizer(type) || n % (uint64_t)bs) return -1;
    parallel_for(n / bs, n_threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; i++) quantize_block(type, x + i * (uint64_t)bs, out + i * (uint64_t)bb);
    });
    return 0;
}

// N(0, std) weights generated and quantised block by block without an f32 copy of the tensor.  The weights
// are those at positions [first_weight, first_weight + n_weights) of the tensor's stream (a function of seed
// and position only), so a row shard can be generated on its own and equals the same rows of the whole tensor.
int ys_random_quantized_at(int type, uint64_t seed, float std_, uint8_t *out, uint64_t first_weight, uint64_t n_weights,
                           int n_threads) {
    const int bs = block_size(type), bb = block_bytes(type);
    if (!bs || !has_quantizer(type) || n_weights % (uint64_t)bs || first_weight % (uint64_t)bs) return -1;
    parallel_for(n_weights / bs, n_threads, [=](uint64_t b, uint64_t e) {
        float tmp[256];
        for (uint64_t i = b; i < e; i++) {
            for (int k = 0; k < bs; k++) tmp[k] = std_ * normal(seed, first_weight + i * (uint64_t)bs + k);
            quantize_block(type, tmp, out + i * (uint64_t)bb);
        }
    });
    return 0;
}
int ys_random_quantized(int type, uint64_t seed, float std_, uint8_t *out, uint64_t n_weights, int n_threads) {
    return ys_random_quantized_at(type, seed, std_, out, 0, n_weights, n_threads);
}

uint16_t ys_f32_to_f16(float f) { return f32_to_f16(f); }

}  // extern "C"
