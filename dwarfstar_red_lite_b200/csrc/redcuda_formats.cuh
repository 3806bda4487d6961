// GGML block formats of the decode hot path: planar repacking and exact decoders, usable from host and device.
//
// Weights arrive as GGUF rows (blocks of 256 values: IQ2_XXS 66 B, IQ3_S 110 B, Q6_K 210 B; layouts as decoded by
// native/redlite_native_quant_cpu.c:130-191 and native/redlite_native_iq3.c:82-91 of the reference). None of those
// block sizes is a multiple of 16 bytes, so a GGUF row cannot be read with aligned 128-bit loads. At load time every
// matrix is therefore re-laid out "planar": each field of all blocks becomes one contiguous array (a plane), every
// plane starts on a 16-byte boundary, and a lane fetches 64 values' worth of one field with a single 128-bit load.
// The byte count in HBM is unchanged (66 / 110 / 210 bytes per block) and no value is altered: the decoders below
// reproduce the reference's float operations in the same order, so dequantised values are bit-identical.
//
//   IQ2_XXS  [qs: nb x 64][d: nb x 2]                              qs = 8 x (4 grid-index bytes, u32 signs+scale)
//   IQ3_S    [qs: nb x 64][signs: nb x 32][qh: nb x 8][scales: nb x 4][d: nb x 2]
//   Q6_K     [ql: nb x 128][qh: nb x 64][sc: nb x 16][d: nb x 2]
//
// nb = number of blocks of the matrix = nrows * ncols / 256; block index = row * (ncols/256) + block-in-row.
// With a 16-byte aligned matrix base, every plane that is read with vector loads starts on a 16-byte boundary for
// any nb (plane offsets are nb x 64, 96, 128, 192, 208); the 2-byte d planes only need 2-byte alignment.
#pragma once
#include <stdint.h>
#include <string.h>
#ifdef __CUDACC__
#include <cuda_fp16.h>
#define RC_HD __host__ __device__ __forceinline__
#else
#define RC_HD static inline      /* plain C++ build: the host unit test of the layout and the decoders */
#endif

enum RcType : uint32_t { RC_F32 = 0u, RC_F16 = 1u, RC_Q6_K = 14u, RC_IQ2_XXS = 16u, RC_IQ3_S = 21u,
                         RC_Q8_0 = 8u, RC_Q2_K = 10u, RC_Q4_K = 12u, RC_Q5_K = 13u };      // the last four: kept in file layout (redcuda_kquants.cuh), dense matrices only

RC_HD uint32_t rc_block_bytes(uint32_t t) { return t == RC_Q6_K ? 210u : t == RC_IQ2_XXS ? 66u : t == RC_IQ3_S ? 110u : 0u; }
RC_HD bool rc_is_quant(uint32_t t) { return rc_block_bytes(t) != 0u; }
RC_HD bool rc_is_file_layout_quant(uint32_t t) { return t == RC_Q8_0 || t == RC_Q2_K || t == RC_Q4_K || t == RC_Q5_K; }
RC_HD bool rc_type_supported(uint32_t t) { return t == RC_F32 || t == RC_F16 || rc_is_quant(t) || rc_is_file_layout_quant(t); }
RC_HD uint64_t rc_row_bytes(uint32_t t, uint32_t ncols) {
    if (t == RC_F32) return (uint64_t)ncols * 4u;
    if (t == RC_F16) return (uint64_t)ncols * 2u;
    if (t == RC_Q8_0) return (ncols % 32u) ? 0u : (uint64_t)(ncols / 32u) * 34u;
    if (rc_is_file_layout_quant(t)) return (ncols % 256u) ? 0u : (uint64_t)(ncols / 256u) * (t == RC_Q2_K ? 84u : t == RC_Q4_K ? 144u : 176u);
    return (ncols % 256u) ? 0u : (uint64_t)(ncols / 256u) * rc_block_bytes(t);
}
RC_HD uint64_t rc_matrix_bytes(uint32_t t, uint32_t nrows, uint32_t ncols) { return rc_row_bytes(t, ncols) * nrows; }

// ---- plane offsets (bytes from the matrix base) ----
RC_HD uint64_t rc_iq2_d(uint64_t nb) { return nb * 64u; }
RC_HD uint64_t rc_iq3_signs(uint64_t nb) { return nb * 64u; }
RC_HD uint64_t rc_iq3_qh(uint64_t nb) { return nb * 96u; }
RC_HD uint64_t rc_iq3_scales(uint64_t nb) { return nb * 104u; }
RC_HD uint64_t rc_iq3_d(uint64_t nb) { return nb * 108u; }
RC_HD uint64_t rc_q6_qh(uint64_t nb) { return nb * 128u; }
RC_HD uint64_t rc_q6_sc(uint64_t nb) { return nb * 192u; }
RC_HD uint64_t rc_q6_d(uint64_t nb) { return nb * 208u; }

// Destination of byte `off` of raw block `b` inside the planar matrix.
RC_HD uint64_t rc_planar_dst(uint32_t t, uint64_t nb, uint64_t b, uint32_t off) {
    if (t == RC_IQ2_XXS) return off < 2u ? rc_iq2_d(nb) + b * 2u + off : b * 64u + (off - 2u);
    if (t == RC_IQ3_S) {
        if (off < 2u) return rc_iq3_d(nb) + b * 2u + off;
        if (off < 66u) return b * 64u + (off - 2u);
        if (off < 74u) return rc_iq3_qh(nb) + b * 8u + (off - 66u);
        if (off < 106u) return rc_iq3_signs(nb) + b * 32u + (off - 74u);
        return rc_iq3_scales(nb) + b * 4u + (off - 106u);
    }
    /* Q6_K */
    if (off < 128u) return b * 128u + off;
    if (off < 192u) return rc_q6_qh(nb) + b * 64u + (off - 128u);
    if (off < 208u) return rc_q6_sc(nb) + b * 16u + (off - 192u);
    return rc_q6_d(nb) + b * 2u + (off - 208u);
}

// Host-side repack of a whole matrix (raw GGUF rows -> planar). dst and src must not overlap.
static inline void rc_repack_host(uint32_t t, const uint8_t *src, uint8_t *dst, uint64_t nb) {
    const uint32_t bb = rc_block_bytes(t);
    if (!bb) { return; }
    for (uint64_t b = 0; b < nb; ++b) {
        const uint8_t *s = src + b * bb;
        if (t == RC_IQ2_XXS) {
            memcpy(dst + b * 64u, s + 2u, 64u); memcpy(dst + rc_iq2_d(nb) + b * 2u, s, 2u);
        } else if (t == RC_IQ3_S) {
            memcpy(dst + b * 64u, s + 2u, 64u); memcpy(dst + rc_iq3_qh(nb) + b * 8u, s + 66u, 8u);
            memcpy(dst + rc_iq3_signs(nb) + b * 32u, s + 74u, 32u); memcpy(dst + rc_iq3_scales(nb) + b * 4u, s + 106u, 4u);
            memcpy(dst + rc_iq3_d(nb) + b * 2u, s, 2u);
        } else {
            memcpy(dst + b * 128u, s, 128u); memcpy(dst + rc_q6_qh(nb) + b * 64u, s + 128u, 64u);
            memcpy(dst + rc_q6_sc(nb) + b * 16u, s + 192u, 16u); memcpy(dst + rc_q6_d(nb) + b * 2u, s + 208u, 2u);
        }
    }
}

// ---- exact scalar helpers ----
RC_HD float rc_h2f(uint16_t h) {
#ifdef __CUDA_ARCH__
    return __half2float(__ushort_as_half(h));      // exact, subnormals included
#else
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu, bits;
    if (e == 0u) {
        if (!m) bits = sign;
        else { int sh = 0; while (!(m & 0x400u)) { m <<= 1; ++sh; } bits = sign | ((uint32_t)(113 - sh) << 23) | ((m & 0x3ffu) << 13); }
    } else if (e == 31u) bits = sign | 0x7f800000u | (m << 13);
    else bits = sign | ((e + 112u) << 23) | (m << 13);
    float f; memcpy(&f, &bits, 4); return f;
#endif
}
RC_HD uint32_t rc_popc(uint32_t x) {
#ifdef __CUDA_ARCH__
    return (uint32_t)__popc(x);
#else
    return (uint32_t)__builtin_popcount(x);
#endif
}
// 7 stored sign bits -> 8 with the odd-parity bit on top (the "ksigns" table of the IQ2/IQ3 formats)
RC_HD uint32_t rc_sign8(uint32_t s7) { return s7 | ((rc_popc(s7) & 1u) << 7); }
RC_HD uint16_t rc_ld16(const uint8_t *p) { return (uint16_t)((uint16_t)p[0] | ((uint16_t)p[1] << 8)); }
RC_HD uint32_t rc_ld32(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }

// Codebooks as the decoders see them: iq2 = 256 entries x 8 magnitude bytes, iq3s = 512 entries x 4 packed bytes.
struct RcBooks { const uint8_t *iq2; const uint32_t *iq3s; };

// Exact dequantisation of the 8 consecutive values [8*g8, 8*g8+8) of block b of a PLANAR matrix.
// Same float operations, in the same order, as rl_quant_dequant_row / rl_iq3_group8 of the reference.
RC_HD void rc_decode8(uint32_t t, const uint8_t *base, uint64_t nb, uint64_t b, uint32_t g8, const RcBooks &bk, float out[8]) {
    if (t == RC_IQ2_XXS) {
        const float d = rc_h2f(rc_ld16(base + rc_iq2_d(nb) + b * 2u));
        const uint32_t ib32 = g8 >> 2, l = g8 & 3u;
        const uint32_t auxg = rc_ld32(base + b * 64u + ib32 * 8u), auxs = rc_ld32(base + b * 64u + ib32 * 8u + 4u);
        const float db = d * (0.5f + (float)(auxs >> 28)) * 0.25f;
        const uint8_t *gv = bk.iq2 + ((auxg >> (8u * l)) & 255u) * 8u;
        const uint32_t s8 = rc_sign8((auxs >> (7u * l)) & 127u);
        for (uint32_t j = 0; j < 8u; ++j) { const float v = db * (float)gv[j]; out[j] = (s8 >> j) & 1u ? -v : v; }
    } else if (t == RC_IQ3_S) {
        const float d = rc_h2f(rc_ld16(base + rc_iq3_d(nb) + b * 2u));
        const uint32_t ib32 = g8 >> 2, l = g8 & 3u;
        const uint8_t *qs = base + b * 64u + 8u * ib32;
        const uint32_t qh = base[rc_iq3_qh(nb) + b * 8u + ib32];
        const uint32_t sg = base[rc_iq3_signs(nb) + b * 32u + 4u * ib32 + l];
        const uint32_t scb = base[rc_iq3_scales(nb) + b * 4u + (ib32 >> 1)];
        const float db = d * (float)(1 + 2 * (int)((scb >> (4u * (ib32 & 1u))) & 0xfu));
        const uint32_t i1 = qs[2u * l] | ((qh << (8u - 2u * l)) & 256u), i2 = qs[2u * l + 1u] | ((qh << (7u - 2u * l)) & 256u);
        const uint32_t g1 = bk.iq3s[i1], g2 = bk.iq3s[i2];
        for (uint32_t j = 0; j < 4u; ++j) {
            const float v1 = db * (float)((g1 >> (8u * j)) & 255u), v2 = db * (float)((g2 >> (8u * j)) & 255u);
            out[j] = (sg >> j) & 1u ? -v1 : v1;
            out[j + 4u] = (sg >> (j + 4u)) & 1u ? -v2 : v2;
        }
    } else {   /* Q6_K: values k = 8*g8 .. +7; half n = k/128, quarter = (k%128)/32, l = k%32 */
        const float d = rc_h2f(rc_ld16(base + rc_q6_d(nb) + b * 2u));
        const uint32_t k = g8 * 8u, half = k >> 7, quarter = (k & 127u) >> 5, l0 = k & 31u;
        const uint8_t *ql = base + b * 128u + half * 64u + (quarter & 1u) * 32u + l0;
        const uint8_t *qh = base + rc_q6_qh(nb) + b * 64u + half * 32u + l0;
        const int8_t sc = (int8_t)base[rc_q6_sc(nb) + b * 16u + half * 8u + (l0 >> 4) + 2u * quarter];
        const float ds = d * (float)sc;
        for (uint32_t j = 0; j < 8u; ++j) {
            const uint32_t nib = quarter < 2u ? (ql[j] & 0xFu) : (uint32_t)(ql[j] >> 4);
            const int q = (int)(int8_t)(nib | (((qh[j] >> (2u * quarter)) & 3u) << 4)) - 32;
            out[j] = ds * (float)q;
        }
    }
}
