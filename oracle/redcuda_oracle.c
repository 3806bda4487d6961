/*
 * TEST INFRASTRUCTURE — CPU restatement of the reference's CPU arithmetic (see redcuda_oracle.h).
 * Never linked into or loaded by the product library.
 *
 * The order of floating-point operations follows the cited reference lines exactly, so that the restatement
 * agrees with the reference library to the last bit wherever both compute the same thing; the build uses
 * -ffp-contract=off so that the compiler cannot fuse multiply-adds the reference (built with -O2, no
 * contraction across statements in these expressions) does not fuse.
 */
#define _POSIX_C_SOURCE 200809L
#include "redcuda_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#define QK 256u
#define Q6_K_BLOCK 210u
#define IQ2_XXS_BLOCK 66u
#define IQ3_S_BLOCK 110u

static const uint8_t *g_iq2xxs_grid = NULL;   /* 256 entries x 8 bytes */
static const uint32_t *g_iq3s_grid = NULL;    /* 512 entries x 4 packed bytes */

int ro_set_codebooks(const uint8_t *iq2xxs_grid_2048, const uint32_t *iq3s_grid_512) {
    g_iq2xxs_grid = iq2xxs_grid_2048;
    g_iq3s_grid = iq3s_grid_512;
    return 1;
}

/* tables of the further types of the IQ3 family (iq3.c:53-110): IQ3_XXS grid (256 x 4 packed bytes), IQ2_S grid (1024 x 8
 * packed bytes), IQ4_NL values (16 x int8) */
static const uint32_t *g_iq3xxs_grid = NULL;
static const uint64_t *g_iq2s_grid = NULL;
static const int8_t *g_iq4nl = NULL;
int ro_set_codebooks_ext(const uint32_t *iq3xxs_grid_256, const uint64_t *iq2s_grid_1024, const int8_t *iq4nl_16) {
    g_iq3xxs_grid = iq3xxs_grid_256;
    g_iq2s_grid = iq2s_grid_1024;
    g_iq4nl = iq4nl_16;
    return 1;
}
/* grids of IQ2_XS (512 x 8 magnitudes) and IQ1_M (2048 x 8 values), the two types of reference.c:116-176 */
static const int8_t *g_iq2xs_grid = NULL, *g_iq1m_grid = NULL;
int ro_set_codebooks_xs(const int8_t *iq2xs_grid_4096, const int8_t *iq1m_grid_16384) {
    g_iq2xs_grid = iq2xs_grid_4096;
    g_iq1m_grid = iq1m_grid_16384;
    return 1;
}

static uint16_t rd16(const uint8_t *p) { return (uint16_t)((uint16_t)p[0] | ((uint16_t)p[1] << 8)); }
static uint32_t rd32(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }

/* quant_cpu.c:20-38 — exact binary16 -> binary32, subnormals included */
float ro_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu, bits;
    if (e == 0u) {
        if (m == 0u) bits = sign;
        else {
            int shift = 0;
            while (!(m & 0x400u)) { m <<= 1; ++shift; }
            bits = sign | ((uint32_t)(113 - shift) << 23) | ((m & 0x3ffu) << 13);
        }
    } else if (e == 31u) bits = sign | 0x7f800000u | (m << 13);
    else bits = sign | ((e + 112u) << 23) | (m << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* engine_cpu.c:29-38 — float rounded to the nearest binary16 (ties to even), returned as float */
float ro_round_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t a = x & 0x7fffffffu, sign = x & 0x80000000u;
    if (a >= 0x7f800000u) return f;
    if (a < 0x38800000u) return ldexpf(rintf(ldexpf(f, 24)), -24);
    uint32_t r = (a + 0x00000fffu + ((a >> 13) & 1u)) & ~0x1fffu;
    if (r >= 0x47800000u) r = 0x7f800000u;
    r |= sign;
    memcpy(&f, &r, 4);
    return f;
}

size_t ro_row_bytes(uint32_t type, uint32_t ncols) {
    if (!ncols) return 0;
    switch (type) {
        case 0: return (size_t)ncols * 4u;
        case 1: return (size_t)ncols * 2u;
        case 8: return ncols % 32u ? 0 : (size_t)(ncols / 32u) * 34u;           /* Q8_0 */
        case 10: return ncols % QK ? 0 : (size_t)(ncols / QK) * 84u;            /* Q2_K */
        case 12: return ncols % QK ? 0 : (size_t)(ncols / QK) * 144u;           /* Q4_K */
        case 13: return ncols % QK ? 0 : (size_t)(ncols / QK) * 176u;           /* Q5_K */
        case 14: return ncols % QK ? 0 : (size_t)(ncols / QK) * Q6_K_BLOCK;
        case 16: return ncols % QK ? 0 : (size_t)(ncols / QK) * IQ2_XXS_BLOCK;
        case 17: return ncols % QK ? 0 : (size_t)(ncols / QK) * 74u;            /* IQ2_XS */
        case 18: return ncols % QK ? 0 : (size_t)(ncols / QK) * 98u;            /* IQ3_XXS */
        case 21: return ncols % QK ? 0 : (size_t)(ncols / QK) * IQ3_S_BLOCK;
        case 22: return ncols % QK ? 0 : (size_t)(ncols / QK) * 82u;            /* IQ2_S */
        case 23: return ncols % QK ? 0 : (size_t)(ncols / QK) * 136u;           /* IQ4_XS */
        case 29: return ncols % QK ? 0 : (size_t)(ncols / QK) * 56u;            /* IQ1_M */
        default: return 0;
    }
}

/* sign byte of the IQ2/IQ3 "ksigns" convention: 7 stored bits + odd-parity eighth (quant_cpu.c:182-183, iq3.c:29) */
static uint32_t sign8_of(uint32_t s7) { return s7 | (((uint32_t)__builtin_popcount(s7) & 1u) << 7); }

/* iq3.c:82-91 — eight consecutive IQ3_S values, group g in [0,32) of a 110-byte block */
static void iq3s_group8(const uint8_t *bp, uint32_t g, float out[8]) {
    const float d = ro_f16_to_f32(rd16(bp));
    const uint32_t ib32 = g / 4u, l = g % 4u;
    const uint8_t *qs = bp + 2u + 8u * ib32, *qh = bp + 66u, *signs = bp + 74u + 4u * ib32, *scales = bp + 106u;
    const float db = d * (float)(1 + 2 * ((scales[ib32 / 2u] >> (4u * (ib32 % 2u))) & 0xf));
    const uint32_t i1 = qs[2u * l + 0u] | (((uint32_t)qh[ib32] << (8u - 2u * l)) & 256u);
    const uint32_t i2 = qs[2u * l + 1u] | (((uint32_t)qh[ib32] << (7u - 2u * l)) & 256u);
    const uint32_t g1 = g_iq3s_grid[i1], g2 = g_iq3s_grid[i2];
    for (uint32_t j = 0; j < 4u; ++j) {
        out[j + 0u] = db * (float)((g1 >> (8u * j)) & 255u) * ((signs[l] & (1u << (j + 0u))) ? -1.f : 1.f);
        out[j + 4u] = db * (float)((g2 >> (8u * j)) & 255u) * ((signs[l] & (1u << (j + 4u))) ? -1.f : 1.f);
    }
}

/* iq3.c:70-81, 92-109 — eight consecutive values of group g in [0,32) of an IQ3_XXS (18, 98 bytes), IQ2_S (22, 82 bytes) or
 * IQ4_XS (23, 136 bytes) block. The magnitude product is rounded once, the sign is an exact factor. */
static uint32_t iq3fam_block(uint32_t type) { return type == 18u ? 98u : type == 22u ? 82u : 136u; }
static int iq3fam_ready(uint32_t type) { return type == 18u ? g_iq3xxs_grid != NULL : type == 22u ? g_iq2s_grid != NULL : g_iq4nl != NULL; }
static void iq3fam_group8(uint32_t type, const uint8_t *bp, uint32_t g, float out[8]) {
    const float d = ro_f16_to_f32(rd16(bp));
    const uint32_t ib32 = g / 4u, l = g % 4u;
    if (type == 18u) {
        const uint8_t *qs = bp + 2u + 8u * ib32;
        const uint32_t aux = rd32(bp + 66u + 4u * ib32);
        const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
        const uint32_t s8 = sign8_of((aux >> (7u * l)) & 127u);
        const uint32_t g1 = g_iq3xxs_grid[qs[2u * l]], g2 = g_iq3xxs_grid[qs[2u * l + 1u]];
        for (uint32_t j = 0; j < 4u; ++j) {
            out[j] = db * (float)((g1 >> (8u * j)) & 255u) * ((s8 & (1u << j)) ? -1.f : 1.f);
            out[j + 4u] = db * (float)((g2 >> (8u * j)) & 255u) * ((s8 & (1u << (j + 4u))) ? -1.f : 1.f);
        }
    } else if (type == 22u) {
        const uint8_t *qs = bp + 2u, *signs = bp + 34u, *qh = bp + 66u, *scales = bp + 74u;
        const uint32_t nib = (l < 2u ? scales[ib32] : (uint32_t)(scales[ib32] >> 4)) & 0xfu;
        const float dl = d * (0.5f + (float)nib) * 0.25f;
        const uint32_t idx = qs[4u * ib32 + l] | (((uint32_t)qh[ib32] << (8u - 2u * l)) & 0x300u);
        const uint64_t gv = g_iq2s_grid[idx];
        const uint32_t sg = signs[4u * ib32 + l];
        for (uint32_t j = 0; j < 8u; ++j) out[j] = dl * (float)((gv >> (8u * j)) & 255u) * ((sg & (1u << j)) ? -1.f : 1.f);
    } else {
        const uint32_t scales_h = rd16(bp + 2u);
        const uint8_t *scales_l = bp + 4u, *qs = bp + 8u + 16u * ib32;
        const int ls = (int)((scales_l[ib32 / 2u] >> (4u * (ib32 % 2u))) & 0xfu) | (int)(((scales_h >> (2u * ib32)) & 3u) << 4);
        const float dl = d * (float)(ls - 32);
        const uint32_t base = 8u * (l % 2u);
        for (uint32_t j = 0; j < 8u; ++j) out[j] = dl * (float)g_iq4nl[l < 2u ? (qs[base + j] & 0xfu) : (qs[base + j] >> 4)];
    }
}

/* reference.c:116-176 — weight j in [0,256) of an IQ2_XS (17, 74 bytes) or IQ1_M (29, 56 bytes) block, formed in double as the
 * reference's row dot forms it (it has no dequantiser for these two types) */
static double xs_weight(uint32_t type, const uint8_t *bp, uint32_t j) {
    if (type == 17u) {
        const double d = (double)ro_f16_to_f32(rd16(bp));
        const uint32_t group = j >> 4, part = (j >> 3) & 1u, jj = j & 7u;
        const uint32_t scale = (bp[66u + (group >> 1)] >> (4u * (group & 1u))) & 0x0fu;
        const double db = d * (0.5 + (double)scale) * 0.25;
        const uint32_t q = rd16(bp + 2u + 2u * (2u * group + part));
        const uint32_t s8 = sign8_of((q >> 9) & 127u);
        const double sign = (s8 & (1u << jj)) ? -1.0 : 1.0;
        return db * (double)g_iq2xs_grid[(q & 0x1ffu) * 8u + jj] * sign;
    }
    uint16_t sc[4];
    for (uint32_t i = 0; i < 4u; ++i) sc[i] = rd16(bp + 48u + 2u * i);
    const uint16_t d_bits = (uint16_t)((sc[0] >> 12) | ((sc[1] >> 8) & 0x00f0u) | ((sc[2] >> 4) & 0x0f00u) | (sc[3] & 0xf000u));
    const double d = (double)ro_f16_to_f32(d_bits);
    const uint32_t group = j >> 3, jj = j & 7u;
    const uint32_t nibble = (bp[32u + (group >> 1)] >> (4u * (group & 1u))) & 0x0fu;
    const uint32_t grid_index = (uint32_t)bp[group] | ((nibble & 7u) << 8);
    const double delta = (nibble & 8u) ? -0.125 : 0.125;
    const uint32_t scale_index = group >> 1;
    const uint32_t scale = (sc[scale_index >> 2] >> (3u * (scale_index & 3u))) & 7u;
    const double dl = d * (double)(2u * scale + 1u);
    return dl * ((double)g_iq1m_grid[grid_index * 8u + jj] + delta);
}
static uint32_t xs_block(uint32_t type) { return type == 17u ? 74u : 56u; }
static int xs_ready(uint32_t type) { return type == 17u ? g_iq2xs_grid != NULL : g_iq1m_grid != NULL; }

/* ---- the GGUF types beyond the decode path's three (quant_cpu.c:40-129): value j of one block, the float operations in
 * the reference's order. Used by the dequantiser and (widened to double as the reference does) by the row dot. ---- */
/* quant_cpu.c:40-46 — the packed 6-bit scale / min pairs of Q4_K and Q5_K */
static void k4_scale_min(uint32_t j, const uint8_t *q, uint32_t *d, uint32_t *m) {
    if (j < 4u) { *d = q[j] & 63u; *m = q[j + 4u] & 63u; }
    else { *d = (q[j + 4u] & 0x0fu) | ((uint32_t)(q[j - 4u] >> 6) << 4); *m = (uint32_t)(q[j + 4u] >> 4) | ((uint32_t)(q[j] >> 6) << 4); }
}
/* integer code, scale and min factors of value j of a block: w = dscale * sc * q - dmin * mn  (Q8_0: mn = 0, sc = 1) */
typedef struct { float d, dmin; uint32_t sc, mn; int q; } kq_parts;
static kq_parts kq_split(uint32_t type, const uint8_t *bp, uint32_t j) {
    kq_parts r = {0.f, 0.f, 1u, 0u, 0};
    if (type == 8u) {                    /* quant_cpu.c:50-57: [d f16][32 x int8] */
        r.d = ro_f16_to_f32(rd16(bp)); r.q = (int)(int8_t)bp[2u + j];
    } else if (type == 10u) {            /* quant_cpu.c:59-82: [16 scale/min nibbles][64 x 2-bit quads][d][dmin] */
        const uint32_t half = j / 128u, r128 = j % 128u, sub = r128 / 32u, l32 = r128 % 32u;
        const uint8_t scb = bp[half * 8u + sub * 2u + l32 / 16u];
        r.d = ro_f16_to_f32(rd16(bp + 80u)); r.dmin = ro_f16_to_f32(rd16(bp + 82u));
        r.sc = scb & 0xFu; r.mn = scb >> 4;
        r.q = (int)((bp[16u + half * 32u + l32] >> (2u * sub)) & 3u);
    } else if (type == 12u) {            /* quant_cpu.c:84-103: [d][dmin][12 scale bytes][128 nibble bytes] */
        const uint32_t g = j / 32u, l = j % 32u;
        r.d = ro_f16_to_f32(rd16(bp)); r.dmin = ro_f16_to_f32(rd16(bp + 2u));
        k4_scale_min(g, bp + 4u, &r.sc, &r.mn);
        const uint8_t b = bp[16u + (g / 2u) * 32u + l];
        r.q = (int)((g & 1u) ? (b >> 4) : (b & 0x0fu));
    } else {                             /* 13, quant_cpu.c:105-128: [d][dmin][12 scale bytes][32 high-bit bytes][128 nibble bytes] */
        const uint32_t g = j / 32u, l = j % 32u;
        r.d = ro_f16_to_f32(rd16(bp)); r.dmin = ro_f16_to_f32(rd16(bp + 2u));
        k4_scale_min(g, bp + 4u, &r.sc, &r.mn);
        const uint8_t b = bp[48u + (g / 2u) * 32u + l];
        const uint32_t hi = (bp[16u + l] >> g) & 1u;
        r.q = (int)(((g & 1u) ? (b >> 4) : (b & 0x0fu)) + (hi ? 16u : 0u));
    }
    return r;
}
static uint32_t kq_block_values(uint32_t type) { return type == 8u ? 32u : QK; }
static uint32_t kq_block_bytes(uint32_t type) { return type == 8u ? 34u : type == 10u ? 84u : type == 12u ? 144u : 176u; }

int ro_dequant_row(uint32_t type, const uint8_t *row, uint32_t ncols, float *out) {
    if (!row || !out || !ncols) return 0;
    switch (type) {
        case 0: memcpy(out, row, (size_t)ncols * 4u); return 1;
        case 1: for (uint32_t i = 0; i < ncols; ++i) out[i] = ro_f16_to_f32(rd16(row + 2u * i)); return 1;
        case 8: case 10: case 12: case 13: {
            const uint32_t bv = kq_block_values(type);
            if (ncols % bv) return 0;
            for (uint32_t i = 0; i < ncols; ++i) {
                const kq_parts p = kq_split(type, row + (size_t)(i / bv) * kq_block_bytes(type), i % bv);
                if (type == 8u) out[i] = p.d * (float)p.q;                                    /* d * q */
                else out[i] = p.d * (float)p.sc * (float)p.q - p.dmin * (float)p.mn;          /* (d * sc) * q - (dmin * mn), float */
            }
            return 1;
        }
        case 14: {   /* quant_cpu.c:130-153 */
            if (ncols % QK) return 0;
            for (uint32_t ib = 0; ib < ncols / QK; ++ib) {
                const uint8_t *bp = row + (size_t)ib * Q6_K_BLOCK;
                const uint8_t *ql = bp, *qh = bp + 128u;
                const int8_t *sc = (const int8_t *)(bp + 192u);
                const float d = ro_f16_to_f32(rd16(bp + 208u));
                float *y = out + (size_t)ib * QK;
                for (uint32_t n = 0; n < QK; n += 128u) {
                    for (uint32_t l = 0; l < 32u; ++l) {
                        const int is = (int)(l / 16u);
                        const int8_t q1 = (int8_t)((ql[l] & 0xFu) | (((qh[l] >> 0) & 3u) << 4)) - 32;
                        const int8_t q2 = (int8_t)((ql[l + 32u] & 0xFu) | (((qh[l] >> 2) & 3u) << 4)) - 32;
                        const int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3u) << 4)) - 32;
                        const int8_t q4 = (int8_t)((ql[l + 32u] >> 4) | (((qh[l] >> 6) & 3u) << 4)) - 32;
                        y[l] = d * (float)sc[is + 0] * (float)q1;
                        y[l + 32u] = d * (float)sc[is + 2] * (float)q2;
                        y[l + 64u] = d * (float)sc[is + 4] * (float)q3;
                        y[l + 96u] = d * (float)sc[is + 6] * (float)q4;
                    }
                    y += 128u; ql += 64u; qh += 32u; sc += 8;
                }
            }
            return 1;
        }
        case 16: {   /* quant_cpu.c:166-191 */
            if (ncols % QK || !g_iq2xxs_grid) return 0;
            for (uint32_t ib = 0; ib < ncols / QK; ++ib) {
                const uint8_t *bp = row + (size_t)ib * IQ2_XXS_BLOCK;
                const float d = ro_f16_to_f32(rd16(bp));
                float *y = out + (size_t)ib * QK;
                for (uint32_t g = 0; g < 8u; ++g) {
                    const uint32_t auxg = rd32(bp + 2u + 8u * g), auxs = rd32(bp + 6u + 8u * g);
                    const float db = d * (0.5f + (float)(auxs >> 28)) * 0.25f;
                    for (uint32_t l = 0; l < 4u; ++l) {
                        const uint8_t *gv = g_iq2xxs_grid + ((auxg >> (8u * l)) & 255u) * 8u;
                        const uint32_t s8 = sign8_of((auxs >> (7u * l)) & 127u);
                        for (uint32_t j = 0; j < 8u; ++j)
                            y[g * 32u + l * 8u + j] = db * (float)gv[j] * ((s8 & (1u << j)) ? -1.0f : 1.0f);
                    }
                }
            }
            return 1;
        }
        case 21: {   /* iq3.c:112-118 */
            if (ncols % QK || !g_iq3s_grid) return 0;
            for (uint32_t b = 0; b < ncols / QK; ++b)
                for (uint32_t g = 0; g < 32u; ++g) iq3s_group8(row + (size_t)b * IQ3_S_BLOCK, g, out + (size_t)b * QK + 8u * g);
            return 1;
        }
        case 18: case 22: case 23: {   /* iq3.c:112-118 */
            if (ncols % QK || !iq3fam_ready(type)) return 0;
            for (uint32_t b = 0; b < ncols / QK; ++b)
                for (uint32_t g = 0; g < 32u; ++g) iq3fam_group8(type, row + (size_t)b * iq3fam_block(type), g, out + (size_t)b * QK + 8u * g);
            return 1;
        }
        case 17: case 29: {   /* the double weight of reference.c:116-176, rounded to float (it is exact there: at most 22 significant bits) */
            if (ncols % QK || !xs_ready(type)) return 0;
            for (uint32_t i = 0; i < ncols; ++i) out[i] = (float)xs_weight(type, row + (size_t)(i / QK) * xs_block(type), i % QK);
            return 1;
        }
        default: return 0;
    }
}

/* x is float (xd == NULL) or double (xf == NULL) */
static double xin(const float *xf, const double *xd, uint32_t i) { return xd ? xd[i] : (double)xf[i]; }

static int row_dot_any(uint32_t type, const uint8_t *row, const float *xf, const double *xd, uint32_t ncols, double *out) {
    if (!row || (!xf && !xd) || !out || !ncols) return 0;
    double acc = 0.0;
    switch (type) {
        case 0: { const float *w = (const float *)row; for (uint32_t i = 0; i < ncols; ++i) acc += (double)w[i] * xin(xf, xd, i); break; }
        case 1: for (uint32_t i = 0; i < ncols; ++i) acc += (double)ro_f16_to_f32(rd16(row + 2u * i)) * xin(xf, xd, i); break;
        case 8:      /* quant_cpu.c:205-214: x * d * q in double */
            if (ncols % 32u) return 0;
            for (uint32_t i = 0; i < ncols; ++i) {
                const kq_parts p = kq_split(8u, row + (size_t)(i / 32u) * 34u, i % 32u);
                acc += xin(xf, xd, i) * (double)p.d * (double)p.q;
            }
            break;
        case 12: case 13:   /* quant_cpu.c:215-256: x * (d * sc * q - dmin * mn), the weight formed in double */
            if (ncols % QK) return 0;
            for (uint32_t i = 0; i < ncols; ++i) {
                const kq_parts p = kq_split(type, row + (size_t)(i / QK) * kq_block_bytes(type), i % QK);
                acc += xin(xf, xd, i) * ((double)p.d * p.sc * (double)p.q - (double)p.dmin * p.mn);
            }
            break;
        case 10:     /* quant_cpu.c:257-265: the fp32 dequantised value times x */
            if (ncols % QK) return 0;
            for (uint32_t i = 0; i < ncols; ++i) {
                const kq_parts p = kq_split(10u, row + (size_t)(i / QK) * 84u, i % QK);
                acc += (double)(p.d * (float)p.sc * (float)p.q - p.dmin * (float)p.mn) * xin(xf, xd, i);
            }
            break;
        case 14: {   /* shared_exec.c:78-112 — weight formed in double */
            if (ncols % QK) return 0;
            for (uint32_t ib = 0; ib < ncols / QK; ++ib) {
                const uint8_t *bp = row + (size_t)ib * Q6_K_BLOCK;
                const int8_t *sc0 = (const int8_t *)(bp + 192u);
                const float d = ro_f16_to_f32(rd16(bp + 208u));
                for (uint32_t n = 0; n < 256u; n += 128u) {
                    const uint8_t *ql = bp + n / 2u, *qh = bp + 128u + n / 4u;
                    const int8_t *sc = sc0 + n / 16u;
                    for (uint32_t l = 0; l < 32u; ++l) {
                        const uint32_t is = l / 16u;
                        const int q1 = (int)((ql[l] & 0x0fu) | (((qh[l] >> 0) & 3u) << 4)) - 32;
                        const int q2 = (int)((ql[l + 32u] & 0x0fu) | (((qh[l] >> 2) & 3u) << 4)) - 32;
                        const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3u) << 4)) - 32;
                        const int q4 = (int)((ql[l + 32u] >> 4) | (((qh[l] >> 6) & 3u) << 4)) - 32;
                        const uint32_t xb = ib * 256u + n;
                        acc += xin(xf, xd, xb + l) * ((double)d * sc[is + 0u] * q1);
                        acc += xin(xf, xd, xb + l + 32u) * ((double)d * sc[is + 2u] * q2);
                        acc += xin(xf, xd, xb + l + 64u) * ((double)d * sc[is + 4u] * q3);
                        acc += xin(xf, xd, xb + l + 96u) * ((double)d * sc[is + 6u] * q4);
                    }
                }
            }
            break;
        }
        case 16: {   /* shared_exec.c:114-151 — weight formed in double */
            if (ncols % QK || !g_iq2xxs_grid) return 0;
            for (uint32_t ib = 0; ib < ncols / QK; ++ib) {
                const uint8_t *bp = row + (size_t)ib * IQ2_XXS_BLOCK;
                const float d = ro_f16_to_f32(rd16(bp));
                for (uint32_t g = 0; g < 8u; ++g) {
                    const uint32_t auxg = rd32(bp + 2u + 8u * g), auxs = rd32(bp + 6u + 8u * g);
                    const double db = (double)d * (0.5 + (double)(auxs >> 28)) * 0.25;
                    for (uint32_t l = 0; l < 4u; ++l) {
                        const uint8_t *gv = g_iq2xxs_grid + ((auxg >> (8u * l)) & 255u) * 8u;
                        const uint32_t s8 = sign8_of((auxs >> (7u * l)) & 127u);
                        const uint32_t xb = ib * 256u + g * 32u + l * 8u;
                        for (uint32_t j = 0; j < 8u; ++j) {
                            const double s = (s8 & (1u << j)) ? -1.0 : 1.0;
                            acc += xin(xf, xd, xb + j) * (db * (double)gv[j] * s);
                        }
                    }
                }
            }
            break;
        }
        case 21: {   /* iq3.c:120-148 — fp32 dequantised group, double products */
            if (ncols % QK || !g_iq3s_grid) return 0;
            float v[8];
            for (uint32_t b = 0; b < ncols / QK; ++b)
                for (uint32_t g = 0; g < 32u; ++g) {
                    iq3s_group8(row + (size_t)b * IQ3_S_BLOCK, g, v);
                    const uint32_t xb = b * QK + 8u * g;
                    for (uint32_t j = 0; j < 8u; ++j) acc += (double)v[j] * xin(xf, xd, xb + j);
                }
            break;
        }
        case 17: case 29:   /* reference.c:116-176: x * weight, the weight formed in double */
            if (ncols % QK || !xs_ready(type)) return 0;
            for (uint32_t i = 0; i < ncols; ++i) acc += xin(xf, xd, i) * xs_weight(type, row + (size_t)(i / QK) * xs_block(type), i % QK);
            break;
        case 18: case 22: case 23: {   /* iq3.c:120-148 — fp32 dequantised group, double products */
            if (ncols % QK || !iq3fam_ready(type)) return 0;
            float v[8];
            for (uint32_t b = 0; b < ncols / QK; ++b)
                for (uint32_t g = 0; g < 32u; ++g) {
                    iq3fam_group8(type, row + (size_t)b * iq3fam_block(type), g, v);
                    const uint32_t xb = b * QK + 8u * g;
                    for (uint32_t j = 0; j < 8u; ++j) acc += (double)v[j] * xin(xf, xd, xb + j);
                }
            break;
        }
        default: return 0;
    }
    *out = acc;
    return 1;
}

int ro_row_dot(uint32_t type, const uint8_t *row, const float *x, uint32_t ncols, double *out) {
    return row_dot_any(type, row, x, NULL, ncols, out);
}
int ro_row_dot_d(uint32_t type, const uint8_t *row, const double *x, uint32_t ncols, double *out) {
    return row_dot_any(type, row, NULL, x, ncols, out);
}

/* ---- row-parallel helper (engine_cpu.c:54-92) ---- */
typedef struct {
    uint32_t type, ncols, begin, end;
    const uint8_t *w; size_t rb;
    const float *xf; const double *xd;
    float *outf; double *outd;
    int ok;
} rows_job;

static void *rows_worker(void *arg) {
    rows_job *j = (rows_job *)arg;
    j->ok = 1;
    for (uint32_t r = j->begin; r < j->end; ++r) {
        double d = 0.0;
        if (!row_dot_any(j->type, j->w + (size_t)r * j->rb, j->xf, j->xd, j->ncols, &d)) { j->ok = 0; return NULL; }
        if (j->outf) j->outf[r] = (float)d;
        if (j->outd) j->outd[r] = d;
    }
    return NULL;
}

static int rows_parallel(uint32_t type, const uint8_t *w, uint32_t nrows, uint32_t ncols, const float *xf, const double *xd,
                         float *outf, double *outd, int threads) {
    const size_t rb = ro_row_bytes(type, ncols);
    if (!rb || !w) return 0;
    if (threads > 64) threads = 64;
    if ((uint32_t)threads > nrows) threads = (int)nrows;
    if (threads < 1) threads = 1;
    rows_job jobs[64]; pthread_t tids[64]; int spawned[64] = {0};
    const uint32_t chunk = (nrows + (uint32_t)threads - 1u) / (uint32_t)threads;
    for (int i = 0; i < threads; ++i) {
        rows_job *j = &jobs[i];
        j->type = type; j->ncols = ncols; j->w = w; j->rb = rb; j->xf = xf; j->xd = xd; j->outf = outf; j->outd = outd; j->ok = 1;
        j->begin = (uint32_t)i * chunk; if (j->begin > nrows) j->begin = nrows;
        j->end = j->begin + chunk > nrows ? nrows : j->begin + chunk;
        if (i > 0) spawned[i] = pthread_create(&tids[i], NULL, rows_worker, j) == 0;
    }
    rows_worker(&jobs[0]);
    for (int i = 1; i < threads; ++i) if (!spawned[i]) rows_worker(&jobs[i]);
    int ok = jobs[0].ok;
    for (int i = 1; i < threads; ++i) { if (spawned[i]) pthread_join(tids[i], NULL); ok = ok && jobs[i].ok; }
    return ok;
}

int ro_matvec(uint32_t type, const uint8_t *w, uint32_t nrows, uint32_t ncols, const float *x, float *out, int threads) {
    return rows_parallel(type, w, nrows, ncols, x, NULL, out, NULL, threads);
}

/* ---- router ---- */
int ro_router_logits(const float *w, const float *x, uint32_t n_expert, uint32_t hidden, float *logits) {   /* engine_cpu.c:347-355 */
    for (uint32_t e = 0; e < n_expert; ++e) {
        double acc = 0.0;
        const float *row = w + (size_t)e * hidden;
        for (uint32_t i = 0; i < hidden; ++i) acc += (double)row[i] * x[i];
        logits[e] = (float)acc;
    }
    return 1;
}

int ro_router_select(const float *logits, uint32_t n, uint32_t top_k, uint32_t *ids, float *weights, float *probs_out) {   /* router_exec.c:102-184 */
    if (!logits || !ids || !weights || !n || !top_k || top_k > n) return 0;
    float *p = probs_out ? probs_out : (float *)malloc((size_t)n * sizeof(float));
    unsigned char *used = (unsigned char *)calloc(n, 1);
    if (!p || !used) { if (!probs_out) free(p); free(used); return 0; }
    float mx = logits[0];
    for (uint32_t i = 1; i < n; ++i) if (logits[i] > mx) mx = logits[i];
    double denom = 0.0;
    for (uint32_t i = 0; i < n; ++i) { const float v = expf(logits[i] - mx); p[i] = v; denom += (double)v; }
    int ok = denom > 0.0 && isfinite(denom);
    if (ok) {
        const float inv = (float)(1.0 / denom);
        for (uint32_t i = 0; i < n; ++i) p[i] *= inv;
        double sel = 0.0;
        for (uint32_t k = 0; k < top_k; ++k) {
            uint32_t best = UINT32_MAX; float bp = -INFINITY;
            for (uint32_t i = 0; i < n; ++i) {
                if (used[i]) continue;
                if (best == UINT32_MAX || p[i] > bp || (p[i] == bp && i < best)) { best = i; bp = p[i]; }
            }
            if (best == UINT32_MAX) { ok = 0; break; }   /* only NaN probabilities can get here */
            used[best] = 1; ids[k] = best; weights[k] = bp; sel += (double)bp;
        }
        if (ok && sel > 0.0 && isfinite(sel)) {
            const float invs = (float)(1.0 / sel);
            for (uint32_t k = 0; k < top_k; ++k) weights[k] *= invs;
        } else ok = 0;
    }
    if (!probs_out) free(p);
    free(used);
    return ok;
}

/* ---- routed experts ---- */
static double silu_mul(double gate, double up) {   /* reference.c:251-259 */
    double sig;
    if (gate >= 0.0) sig = 1.0 / (1.0 + exp(-gate));
    else { const double eg = exp(gate); sig = eg / (1.0 + eg); }
    return (gate * sig) * up;
}

int ro_routed_experts(uint32_t type_gu, uint32_t type_down, const uint8_t *gate_all, const uint8_t *up_all, const uint8_t *down_all,
                      const uint32_t *ids, const float *weights, uint32_t top_k, uint32_t hidden, uint32_t ffn,
                      const float *x, double *out, int threads) {   /* reference.c:267-382 */
    const size_t gu_bytes = ro_row_bytes(type_gu, hidden) * ffn, down_bytes = ro_row_bytes(type_down, ffn) * hidden;
    if (!gu_bytes || !down_bytes) return 0;
    double *gate = (double *)malloc(sizeof(double) * ffn), *up = (double *)malloc(sizeof(double) * ffn);
    double *act = (double *)malloc(sizeof(double) * ffn), *eo = (double *)malloc(sizeof(double) * hidden);
    int ok = gate && up && act && eo;
    for (uint32_t r = 0; ok && r < hidden; ++r) out[r] = 0.0;
    for (uint32_t i = 0; ok && i < top_k; ++i) {
        const size_t e = ids[i];
        ok = rows_parallel(type_gu, gate_all + e * gu_bytes, ffn, hidden, x, NULL, NULL, gate, threads) &&
             rows_parallel(type_gu, up_all + e * gu_bytes, ffn, hidden, x, NULL, NULL, up, threads);
        if (!ok) break;
        for (uint32_t j = 0; j < ffn; ++j) act[j] = silu_mul(gate[j], up[j]);
        ok = rows_parallel(type_down, down_all + e * down_bytes, hidden, ffn, NULL, act, NULL, eo, threads);
        if (!ok) break;
        for (uint32_t r = 0; r < hidden; ++r) out[r] += (double)weights[i] * eo[r];
    }
    free(gate); free(up); free(act); free(eo);
    return ok;
}

int ro_moe_ffn(const ro_moe_layer *L, const float *x, float *out, uint32_t *ids_out, float *weights_out, float *logits_out, int threads) {
    return ro_moe_ffn2(L, x, NULL, out, ids_out, weights_out, logits_out, threads);
}

int ro_moe_ffn2(const ro_moe_layer *L, const float *x, const float *logits_in, float *out, uint32_t *ids_out, float *weights_out,
                float *logits_out, int threads) {   /* engine_cpu.c:329-386 */
    const uint32_t hidden = L->hidden, ne = L->n_expert, k = L->top_k;
    if (k > RO_MAX_TOPK) return 0;
    float *logits = (float *)malloc(sizeof(float) * ne), *probs = (float *)malloc(sizeof(float) * ne);
    float *shg = (float *)malloc(sizeof(float) * L->ffn_sh), *shu = (float *)malloc(sizeof(float) * L->ffn_sh);
    float *act = (float *)malloc(sizeof(float) * L->ffn_sh), *sho = (float *)malloc(sizeof(float) * hidden);
    double *routed = (double *)malloc(sizeof(double) * hidden);
    uint32_t ids[RO_MAX_TOPK]; float w[RO_MAX_TOPK];
    int ok = logits && probs && shg && shu && act && sho && routed;
    if (ok && logits_in) memcpy(logits, logits_in, sizeof(float) * ne);
    else ok = ok && ro_router_logits(L->router, x, ne, hidden, logits);
    ok = ok && ro_router_select(logits, ne, k, ids, w, probs);
    ok = ok && ro_routed_experts(L->type_gu, L->type_down, L->gate_all, L->up_all, L->down_all, ids, w, k, hidden, L->ffn, x, routed, threads);
    ok = ok && ro_matvec(L->type_sh, L->sh_gate, L->ffn_sh, hidden, x, shg, threads) && ro_matvec(L->type_sh, L->sh_up, L->ffn_sh, hidden, x, shu, threads);
    if (ok) {
        for (uint32_t i = 0; i < L->ffn_sh; ++i) { const double g = shg[i]; act[i] = (float)((g / (1.0 + exp(-g))) * (double)shu[i]); }
        ok = ro_matvec(L->type_sh, L->sh_down, hidden, L->ffn_sh, act, sho, threads);
    }
    if (ok) {
        double acc = 0.0;
        for (uint32_t i = 0; i < hidden; ++i) acc += (double)L->sh_gate_inp[i] * x[i];
        const double scalar = 1.0 / (1.0 + exp(-acc));
        for (uint32_t i = 0; i < hidden; ++i) out[i] = (float)(routed[i] + (double)sho[i] * scalar);
        if (ids_out) memcpy(ids_out, ids, sizeof(uint32_t) * k);
        if (weights_out) memcpy(weights_out, w, sizeof(float) * k);
        if (logits_out) memcpy(logits_out, logits, sizeof(float) * ne);
    }
    free(logits); free(probs); free(shg); free(shu); free(act); free(sho); free(routed);
    return ok;
}

/* ---- DeltaNet ---- */
static double sigmoid_stable(double x) { if (x >= 0.0) { const double z = exp(-x); return 1.0 / (1.0 + z); } const double z = exp(x); return z / (1.0 + z); }
static double softplus_stable(double x) { if (x > 20.0) return x; if (x < -20.0) return exp(x); return log1p(exp(x)); }

int ro_deltanet_mid(const ro_deltanet_params *P, const float *qkv, const float *z, const float *ba,
                    float *conv_state, float *rec_state, float *ng) {   /* engine_cpu.c:148-230 */
    const uint32_t channels = P->channels, rank = P->dt_rank, groups = P->n_group, S = P->d_state, d_conv = P->d_conv;
    const uint32_t qk_each = S * groups, ns = d_conv - 1u, head_v = P->d_inner / rank;
    if (head_v != S || rank % groups) return 0;
    float *beta = (float *)malloc(sizeof(float) * rank), *gate = (float *)malloc(sizeof(float) * rank);
    float *cs = (float *)malloc(sizeof(float) * channels), *q = (float *)malloc(sizeof(float) * qk_each), *k = (float *)malloc(sizeof(float) * qk_each);
    float *core = (float *)malloc(sizeof(float) * P->d_inner), *next = (float *)malloc(sizeof(float) * (size_t)channels * ns);
    float *delta = (float *)malloc(sizeof(float) * S);
    if (!beta || !gate || !cs || !q || !k || !core || !next || !delta) { free(beta); free(gate); free(cs); free(q); free(k); free(core); free(next); free(delta); return 0; }
    {
        const uint32_t width = rank / groups, stride = 2u * width;
        for (uint32_t h = 0; h < rank; ++h) {
            const uint32_t g = h / width, l = h - g * width;
            const double b = ba[g * stride + l];
            const double a = (double)ba[g * stride + width + l] + P->dt_bias[h];
            beta[h] = (float)sigmoid_stable(b);
            gate[h] = (float)(softplus_stable(a) * (double)P->ssm_a[h]);
        }
    }
    for (uint32_t c = 0; c < channels; ++c) {
        double acc = 0.0;
        for (uint32_t j = 0; j < ns; ++j) acc += (double)conv_state[(size_t)c * ns + j] * P->conv_kernel[(size_t)c * d_conv + j];
        acc += (double)qkv[c] * P->conv_kernel[(size_t)c * d_conv + ns];
        cs[c] = (float)(acc / (1.0 + exp(-acc)));
    }
    for (uint32_t c = 0; c < channels; ++c) {
        const size_t b = (size_t)c * ns;
        for (uint32_t j = 0; j + 1u < ns; ++j) next[b + j] = conv_state[b + j + 1u];
        next[b + ns - 1u] = qkv[c];
    }
    for (uint32_t which = 0; which < 2u; ++which) {
        float *dst = which ? k : q;
        const uint32_t offset = which ? qk_each : 0u;
        for (uint32_t h = 0; h < groups; ++h) {
            const uint32_t b = offset + h * S;
            double ss = 0.0;
            for (uint32_t j = 0; j < S; ++j) ss += (double)cs[b + j] * cs[b + j];
            const double inv = 1.0 / fmax(sqrt(ss), (double)P->rms_eps);
            for (uint32_t j = 0; j < S; ++j) dst[(size_t)h * S + j] = (float)((double)cs[b + j] * inv);
        }
    }
    const float *v = cs + 2u * qk_each;
    {
        const size_t matrix = (size_t)S * S;
        const float scale = 1.0f / sqrtf((float)S);
        const uint32_t ratio = rank / groups;
        for (uint32_t h = 0; h < rank; ++h) {
            const uint32_t kh = h / ratio;
            const float *qh = q + (size_t)kh * S, *khv = k + (size_t)kh * S, *vh = v + (size_t)h * S;
            float *mh = rec_state + (size_t)h * matrix, *oh = core + (size_t)h * S;
            const float decay = expf(gate[h]);
            for (uint32_t j = 0; j < S; ++j) { float *row = mh + (size_t)j * S; for (uint32_t i = 0; i < S; ++i) row[i] *= decay; }
            for (uint32_t j = 0; j < S; ++j) {
                float sum = 0.0f; const float *row = mh + (size_t)j * S;
                for (uint32_t i = 0; i < S; ++i) sum += row[i] * khv[i];
                delta[j] = (vh[j] - sum) * beta[h];
            }
            for (uint32_t j = 0; j < S; ++j) { float *row = mh + (size_t)j * S; const float d = delta[j]; for (uint32_t i = 0; i < S; ++i) row[i] += khv[i] * d; }
            for (uint32_t j = 0; j < S; ++j) {
                float sum = 0.0f; const float *row = mh + (size_t)j * S;
                for (uint32_t i = 0; i < S; ++i) sum += row[i] * qh[i];
                oh[j] = sum * scale;
            }
        }
    }
    for (uint32_t h = 0; h < rank; ++h) {
        const float *x = core + (size_t)h * head_v, *g = z + (size_t)h * head_v;
        float *y = ng + (size_t)h * head_v;
        double ss = 0.0;
        for (uint32_t i = 0; i < head_v; ++i) ss += (double)x[i] * x[i];
        const float inv = 1.0f / sqrtf((float)(ss / head_v) + P->rms_eps);
        for (uint32_t i = 0; i < head_v; ++i) { const float silu = g[i] / (1.0f + expf(-g[i])); y[i] = x[i] * inv * P->ssm_norm[i] * silu; }
    }
    memcpy(conv_state, next, sizeof(float) * (size_t)channels * ns);
    free(beta); free(gate); free(cs); free(q); free(k); free(core); free(next); free(delta);
    return 1;
}

/* ---- whole model ---- */
struct ro_state {
    const ro_model *m;
    uint32_t position, n_rec, n_att;
    float *conv, *rec, *kcache, *vcache, *layer_out, *final_norm;
    uint32_t *router_ids;
    float *router_logits;       /* [layer][n_expert] of the last step: lets a test measure the margin of a selection */
    size_t conv_count, rec_count, kv_layer;
};

ro_state *ro_state_create(const ro_model *m) {
    ro_state *s = (ro_state *)calloc(1, sizeof(*s));
    if (!s) return NULL;
    s->m = m;
    for (uint32_t l = 0; l < m->n_layer; ++l) { if (m->layers[l].recurrent) s->n_rec++; else s->n_att++; }
    s->conv_count = (size_t)(m->d_conv - 1u) * m->channels;
    s->rec_count = (size_t)m->dt_rank * m->d_state * m->d_state;
    s->kv_layer = (size_t)m->context * m->n_head_kv * m->head_dim;
    s->conv = (float *)calloc(s->conv_count * s->n_rec + 1u, sizeof(float));
    s->rec = (float *)calloc(s->rec_count * s->n_rec + 1u, sizeof(float));
    s->kcache = (float *)calloc(s->kv_layer * s->n_att + 1u, sizeof(float));
    s->vcache = (float *)calloc(s->kv_layer * s->n_att + 1u, sizeof(float));
    s->layer_out = (float *)calloc((size_t)m->n_layer * m->hidden, sizeof(float));
    s->final_norm = (float *)calloc(m->hidden, sizeof(float));
    s->router_ids = (uint32_t *)calloc((size_t)m->n_layer * RO_MAX_TOPK, sizeof(uint32_t));
    s->router_logits = (float *)calloc((size_t)m->n_layer * m->n_expert, sizeof(float));
    if (!s->conv || !s->rec || !s->kcache || !s->vcache || !s->layer_out || !s->final_norm || !s->router_ids || !s->router_logits) { ro_state_free(s); return NULL; }
    return s;
}
void ro_state_free(ro_state *s) {
    if (!s) return;
    free(s->conv); free(s->rec); free(s->kcache); free(s->vcache); free(s->layer_out); free(s->final_norm); free(s->router_ids); free(s->router_logits); free(s);
}
void ro_state_reset(ro_state *s) {
    s->position = 0;
    memset(s->conv, 0, sizeof(float) * s->conv_count * s->n_rec);
    memset(s->rec, 0, sizeof(float) * s->rec_count * s->n_rec);
    memset(s->kcache, 0, sizeof(float) * s->kv_layer * s->n_att);
    memset(s->vcache, 0, sizeof(float) * s->kv_layer * s->n_att);
}
uint32_t ro_state_position(const ro_state *s) { return s->position; }
const float *ro_state_layer_out(const ro_state *s, uint32_t layer) { return s->layer_out + (size_t)layer * s->m->hidden; }
const uint32_t *ro_state_router_ids(const ro_state *s, uint32_t layer) { return s->router_ids + (size_t)layer * RO_MAX_TOPK; }
const float *ro_state_final_norm(const ro_state *s) { return s->final_norm; }
const float *ro_state_router_logits(const ro_state *s, uint32_t layer) { return s->router_logits + (size_t)layer * s->m->n_expert; }
float *ro_state_rec(ro_state *s, uint32_t i) { return s->rec + s->rec_count * i; }
float *ro_state_conv(ro_state *s, uint32_t i) { return s->conv + s->conv_count * i; }

static void rmsnorm_d(const float *x, const float *w, uint32_t n, float eps, float *out) {   /* engine_cpu.c:96-101 */
    double ss = 0.0;
    for (uint32_t i = 0; i < n; ++i) ss += (double)x[i] * x[i];
    const double inv = 1.0 / sqrt(ss / n + (double)eps);
    for (uint32_t i = 0; i < n; ++i) out[i] = (float)((double)x[i] * inv * w[i]);
}

static void rope_neox(float *x, uint32_t rope_dims, uint32_t position, float freq_base) {   /* engine_cpu.c:242-251 */
    const uint32_t half = rope_dims / 2u;
    for (uint32_t i = 0; i < half; ++i) {
        const float theta = (float)position * powf(freq_base, -2.0f * (float)i / (float)rope_dims);
        const float c = cosf(theta), s = sinf(theta);
        const float x0 = x[i], x1 = x[half + i];
        x[i] = x0 * c - x1 * s;
        x[half + i] = x0 * s + x1 * c;
    }
}

static int tmatvec(const ro_tensor *t, const float *x, float *out, int threads) {
    return ro_matvec(t->type, t->data, t->nrows, t->ncols, x, out, threads);
}

static int deltanet_branch(const ro_model *m, ro_state *s, const ro_layer *L, uint32_t ridx, const float *normed, float *out, int threads) {   /* engine_cpu.c:120-238 */
    float *qkv = (float *)malloc(sizeof(float) * m->channels), *z = (float *)malloc(sizeof(float) * m->d_inner);
    float *ba = (float *)malloc(sizeof(float) * 2u * m->dt_rank), *ng = (float *)malloc(sizeof(float) * m->d_inner);
    int ok = qkv && z && ba && ng;
    ok = ok && tmatvec(&L->qkv, normed, qkv, threads) && tmatvec(&L->z, normed, z, threads) && tmatvec(&L->ba, normed, ba, threads);
    if (ok) {
        ro_deltanet_params P;
        P.d_conv = m->d_conv; P.d_state = m->d_state; P.n_group = m->n_group; P.dt_rank = m->dt_rank; P.d_inner = m->d_inner; P.channels = m->channels;
        P.rms_eps = m->rms_eps;
        P.conv_kernel = (const float *)L->conv.data; P.dt_bias = (const float *)L->dt.data; P.ssm_a = (const float *)L->a.data; P.ssm_norm = (const float *)L->ssm_norm.data;
        ok = ro_deltanet_mid(&P, qkv, z, ba, s->conv + s->conv_count * ridx, s->rec + s->rec_count * ridx, ng);
    }
    ok = ok && tmatvec(&L->ssm_out, ng, out, threads);
    free(qkv); free(z); free(ba); free(ng);
    return ok;
}

static int attention_branch(const ro_model *m, ro_state *s, const ro_layer *L, uint32_t aidx, const float *normed, float *out, int threads) {   /* engine_cpu.c:253-325 */
    const uint32_t hd = m->head_dim, nq = m->n_head, nkv = m->n_head_kv, qcount = nq * hd, kvcount = nkv * hd;
    const uint32_t position = s->position, seq_len = position + 1u;
    if (position >= m->context) return 0;
    float *kc = s->kcache + s->kv_layer * aidx, *vc = s->vcache + s->kv_layer * aidx;
    float *qg = (float *)malloc(sizeof(float) * 2u * qcount), *kraw = (float *)malloc(sizeof(float) * kvcount), *val = (float *)malloc(sizeof(float) * kvcount);
    float *query = (float *)malloc(sizeof(float) * qcount), *gate = (float *)malloc(sizeof(float) * qcount), *key = (float *)malloc(sizeof(float) * kvcount);
    float *gated = (float *)malloc(sizeof(float) * qcount);
    double *scores = (double *)malloc(sizeof(double) * seq_len);
    int ok = qg && kraw && val && query && gate && key && gated && scores;
    ok = ok && tmatvec(&L->q, normed, qg, threads) && tmatvec(&L->k, normed, kraw, threads) && tmatvec(&L->v, normed, val, threads);
    if (ok) {
        const float *qn = (const float *)L->q_norm.data, *kn = (const float *)L->k_norm.data;
        for (uint32_t h = 0; h < nq; ++h) {
            const float *src = qg + (size_t)h * hd * 2u;
            rmsnorm_d(src, qn, hd, m->rms_eps, query + (size_t)h * hd);
            memcpy(gate + (size_t)h * hd, src + hd, sizeof(float) * hd);
            rope_neox(query + (size_t)h * hd, m->rope_dims, position, m->rope_freq_base);
        }
        for (uint32_t h = 0; h < nkv; ++h) {
            rmsnorm_d(kraw + (size_t)h * hd, kn, hd, m->rms_eps, key + (size_t)h * hd);
            rope_neox(key + (size_t)h * hd, m->rope_dims, position, m->rope_freq_base);
        }
        for (uint32_t i = 0; i < kvcount; ++i) {
            kc[(size_t)position * kvcount + i] = m->kv_f16 ? ro_round_half(key[i]) : key[i];
            vc[(size_t)position * kvcount + i] = m->kv_f16 ? ro_round_half(val[i]) : val[i];
        }
        const double scale = 1.0 / sqrt((double)hd);
        for (uint32_t h = 0; h < nq; ++h) {
            const uint32_t kvh = h / (nq / nkv);
            const float *qv = query + (size_t)h * hd;
            double mx = -INFINITY;
            for (uint32_t p = 0; p < seq_len; ++p) {
                const float *kv = kc + ((size_t)p * nkv + kvh) * hd;
                double dot = 0.0;
                for (uint32_t i = 0; i < hd; ++i) dot += (double)qv[i] * kv[i];
                scores[p] = dot * scale;
                if (scores[p] > mx) mx = scores[p];
            }
            double denom = 0.0;
            for (uint32_t p = 0; p < seq_len; ++p) { scores[p] = exp(scores[p] - mx); denom += scores[p]; }
            for (uint32_t i = 0; i < hd; ++i) {
                double acc = 0.0;
                for (uint32_t p = 0; p < seq_len; ++p) acc += (scores[p] / denom) * vc[((size_t)p * nkv + kvh) * hd + i];
                const size_t idx = (size_t)h * hd + i;
                gated[idx] = (float)(acc / (1.0 + exp(-(double)gate[idx])));
            }
        }
        ok = tmatvec(&L->o, gated, out, threads);
    }
    free(qg); free(kraw); free(val); free(query); free(gate); free(key); free(gated); free(scores);
    return ok;
}

int ro_model_step(const ro_model *m, ro_state *s, uint32_t token, float *logits, int threads) {   /* engine_cpu.c:390-441 */
    const uint32_t hidden = m->hidden;
    if (token >= m->vocab) return 0;
    float *x = (float *)malloc(sizeof(float) * hidden), *normed = (float *)malloc(sizeof(float) * hidden);
    float *branch = (float *)malloc(sizeof(float) * hidden), *resid = (float *)malloc(sizeof(float) * hidden), *ffn_out = (float *)malloc(sizeof(float) * hidden);
    int ok = x && normed && branch && resid && ffn_out;
    /* embedding row: dequantised (engine.c:740-749) */
    ok = ok && ro_dequant_row(m->tok_embd.type, m->tok_embd.data + (size_t)token * ro_row_bytes(m->tok_embd.type, hidden), hidden, x);
    uint32_t ridx = 0, aidx = 0;
    for (uint32_t l = 0; ok && l < m->n_layer; ++l) {
        const ro_layer *L = &m->layers[l];
        rmsnorm_d(x, (const float *)L->attn_norm.data, hidden, m->rms_eps, normed);
        if (L->recurrent) ok = deltanet_branch(m, s, L, ridx++, normed, branch, threads);
        else ok = attention_branch(m, s, L, aidx++, normed, branch, threads);
        if (!ok) break;
        {
            double ss = 0.0;
            const float *pw = (const float *)L->post_norm.data;
            for (uint32_t i = 0; i < hidden; ++i) { resid[i] = x[i] + branch[i]; ss += (double)resid[i] * resid[i]; }
            const double inv = 1.0 / sqrt(ss / (double)hidden + (double)m->rms_eps);
            for (uint32_t i = 0; i < hidden; ++i) normed[i] = (float)((double)resid[i] * inv * pw[i]);
        }
        ro_moe_layer M;
        M.hidden = hidden; M.n_expert = m->n_expert; M.top_k = m->top_k; M.ffn = L->gate_exps.nrows; M.ffn_sh = L->sh_gate.nrows;
        M.type_gu = L->gate_exps.type; M.type_down = L->down_exps.type; M.type_sh = L->sh_gate.type;
        M.router = (const float *)L->router.data; M.gate_all = L->gate_exps.data; M.up_all = L->up_exps.data; M.down_all = L->down_exps.data;
        M.sh_gate_inp = (const float *)L->sh_gate_inp.data; M.sh_gate = L->sh_gate.data; M.sh_up = L->sh_up.data; M.sh_down = L->sh_down.data;
        if (L->sh_up.type != M.type_sh || L->sh_down.type != M.type_sh || L->up_exps.type != M.type_gu) { ok = 0; break; }
        ok = ro_moe_ffn(&M, normed, ffn_out, s->router_ids + (size_t)l * RO_MAX_TOPK, NULL, s->router_logits + (size_t)l * m->n_expert, threads);
        if (!ok) break;
        for (uint32_t i = 0; i < hidden; ++i) x[i] = resid[i] + ffn_out[i];
        memcpy(s->layer_out + (size_t)l * hidden, x, sizeof(float) * hidden);
    }
    if (ok) {
        rmsnorm_d(x, (const float *)m->output_norm.data, hidden, m->rms_eps, s->final_norm);
        if (logits) ok = tmatvec(&m->output, s->final_norm, logits, threads);
        if (ok) s->position++;
    }
    free(x); free(normed); free(branch); free(resid); free(ffn_out);
    return ok;
}
