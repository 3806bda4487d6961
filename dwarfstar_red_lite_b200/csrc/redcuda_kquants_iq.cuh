// Value decode of five further codebook types, kept in their file layout. IQ3_XXS (18, 98-byte blocks), IQ2_S (22, 82 bytes),
// IQ4_XS (23, 136 bytes): the float operations and their order are those of the reference's rl_iq3_group8
// (native/redlite_native_iq3.c:53-110): the scale product is rounded factor by factor, the magnitude product once, and the
// sign is an exact factor. IQ2_XS (17, 74 bytes) and IQ1_M (29, 56 bytes): the reference forms these weights in double inside
// its row dot (native/redlite_native_reference.c:116-176); every factor is a short integer or a power of two (at most 22
// significant bits in all), so the same products in float are exact and equal the double value. Host and device compile the
// same function, so the decode can be checked against the CPU checker without a GPU. The tables are data of the formats
// and are handed in by the caller.
#pragma once
#include <stdint.h>

namespace rc {

// iq3xxs: 256 x 4 packed bytes, iq2s: 1024 x 8 packed bytes, iq4nl: 16 values, iq2xs: 512 x 8 magnitudes, iq1m: 2048 x 8 values
struct KqIqTabs { const uint32_t *iq3xxs; const uint64_t *iq2s; const int8_t *iq4nl; const int8_t *iq2xs; const int8_t *iq1m; };

#if defined(__CUDA_ARCH__)
#define RC_KQ_MUL(a, b) __fmul_rn((a), (b))
#else
#define RC_KQ_MUL(a, b) ((a) * (b))
#endif

__host__ __device__ inline bool kq_iq_type(uint32_t t) { return t == 17u || t == 18u || t == 22u || t == 23u || t == 29u; }
__host__ __device__ inline bool kq_iq_family3(uint32_t t) { return t == 18u || t == 22u || t == 23u; }       // tables of redcuda_set_codebooks_ext
__host__ __device__ inline uint32_t kq_iq_block_bytes(uint32_t t) { return t == 17u ? 74u : t == 18u ? 98u : t == 22u ? 82u : t == 23u ? 136u : 56u; }

// exact binary16 -> binary32, subnormals included
__host__ __device__ inline float kq_iq_f16(const uint8_t *p) {
    const uint32_t h = (uint32_t)p[0] | ((uint32_t)p[1] << 8), sign = (h >> 15) << 31, e = (h >> 10) & 31u, m = h & 1023u;
    union { uint32_t u; float f; } v;
    if (e == 0u) { v.f = (float)m * 5.9604644775390625e-08f; v.u |= sign; return v.f; }      // m * 2^-24, exact
    v.u = sign | ((e == 31u ? 255u : e + 112u) << 23) | (m << 13);
    return v.f;
}
// the eighth sign bit of a 7-bit sign index is its odd parity (iq3.c:28-29)
__host__ __device__ inline uint32_t kq_iq_sign8(uint32_t s7) {
    uint32_t p = s7 ^ (s7 >> 4);
    p ^= p >> 2; p ^= p >> 1;
    return s7 | ((p & 1u) << 7);
}

// value j in [0, 256) of the block at bp
__host__ __device__ inline float kq_iq_value(uint32_t t, const uint8_t *bp, uint32_t j, const KqIqTabs &T) {
    if (t == 17u) {
        const float d = kq_iq_f16(bp);
        const uint32_t group = j >> 4, part = (j >> 3) & 1u, jj = j & 7u;
        const uint32_t scale = ((uint32_t)bp[66u + (group >> 1)] >> (4u * (group & 1u))) & 0xfu;
        const float db = RC_KQ_MUL(RC_KQ_MUL(d, 0.5f + (float)scale), 0.25f);
        const uint8_t *qp = bp + 2u + 2u * (2u * group + part);
        const uint32_t q = (uint32_t)qp[0] | ((uint32_t)qp[1] << 8);
        const float v = RC_KQ_MUL(db, (float)T.iq2xs[(q & 0x1ffu) * 8u + jj]);
        return ((kq_iq_sign8((q >> 9) & 127u) >> jj) & 1u) ? -v : v;
    }
    if (t == 29u) {
        uint32_t sc[4];
#pragma unroll
        for (uint32_t i = 0; i < 4u; ++i) sc[i] = (uint32_t)bp[48u + 2u * i] | ((uint32_t)bp[49u + 2u * i] << 8);
        const uint32_t d_bits = (sc[0] >> 12) | ((sc[1] >> 8) & 0x00f0u) | ((sc[2] >> 4) & 0x0f00u) | (sc[3] & 0xf000u);
        const uint8_t db2[2] = {(uint8_t)(d_bits & 255u), (uint8_t)(d_bits >> 8)};
        const float d = kq_iq_f16(db2);
        const uint32_t group = j >> 3, jj = j & 7u;
        const uint32_t nibble = ((uint32_t)bp[32u + (group >> 1)] >> (4u * (group & 1u))) & 0xfu;
        const uint32_t grid_index = (uint32_t)bp[group] | ((nibble & 7u) << 8);
        const uint32_t scale_index = group >> 1;
        const uint32_t scale = (sc[scale_index >> 2] >> (3u * (scale_index & 3u))) & 7u;
        const float dl = RC_KQ_MUL(d, (float)(2u * scale + 1u));
        return RC_KQ_MUL(dl, (float)T.iq1m[grid_index * 8u + jj] + ((nibble & 8u) ? -0.125f : 0.125f));
    }
    const float d = kq_iq_f16(bp);
    const uint32_t g = j >> 3, jj = j & 7u, ib32 = g >> 2, l = g & 3u;
    float v; uint32_t neg;
    if (t == 18u) {
        const uint8_t *qs = bp + 2u + 8u * ib32, *ap = bp + 66u + 4u * ib32;
        const uint32_t aux = (uint32_t)ap[0] | ((uint32_t)ap[1] << 8) | ((uint32_t)ap[2] << 16) | ((uint32_t)ap[3] << 24);
        const float db = RC_KQ_MUL(RC_KQ_MUL(d, 0.5f + (float)(aux >> 28)), 0.5f);
        const uint32_t grid = T.iq3xxs[qs[2u * l + (jj >> 2)]];
        v = RC_KQ_MUL(db, (float)((grid >> (8u * (jj & 3u))) & 255u));
        neg = (kq_iq_sign8((aux >> (7u * l)) & 127u) >> jj) & 1u;
    } else if (t == 22u) {
        const uint8_t *qs = bp + 2u, *signs = bp + 34u, *qh = bp + 66u, *scales = bp + 74u;
        const uint32_t nib = (l < 2u ? (uint32_t)scales[ib32] : (uint32_t)scales[ib32] >> 4) & 0xfu;
        const float dl = RC_KQ_MUL(RC_KQ_MUL(d, 0.5f + (float)nib), 0.25f);
        const uint32_t idx = (uint32_t)qs[4u * ib32 + l] | (((uint32_t)qh[ib32] << (8u - 2u * l)) & 0x300u);
        v = RC_KQ_MUL(dl, (float)(uint32_t)((T.iq2s[idx] >> (8u * jj)) & 255u));
        neg = ((uint32_t)signs[4u * ib32 + l] >> jj) & 1u;
    } else {
        const uint32_t scales_h = (uint32_t)bp[2] | ((uint32_t)bp[3] << 8);
        const uint8_t *scales_l = bp + 4u, *qs = bp + 8u + 16u * ib32;
        const int ls = (int)(((uint32_t)scales_l[ib32 >> 1] >> (4u * (ib32 & 1u))) & 0xfu) | (int)(((scales_h >> (2u * ib32)) & 3u) << 4);
        const float dl = RC_KQ_MUL(d, (float)(ls - 32));
        const uint32_t q = qs[8u * (l & 1u) + jj];
        v = RC_KQ_MUL(dl, (float)T.iq4nl[l < 2u ? (q & 0xfu) : (q >> 4)]);
        neg = 0u;
    }
    return neg ? -v : v;
}

}  // namespace rc
