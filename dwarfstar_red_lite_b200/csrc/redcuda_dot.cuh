// Device-side dot-product building blocks over planar quantised matrices.
//
// Unit of work: a CHUNK of 64 values of one row (a quarter of a 256-value block), fetched with 128-bit loads:
//   IQ2_XXS  one uint4 = two (grid indices, signs+scale) groups of 32 values
//   IQ3_S    one uint4 of grid-index bytes + one uint2 of sign bytes + 2 high-bit bytes + 1 scale byte
//   Q6_K     two uint4 of low nibbles + one uint4 of high bit pairs + 4 int8 scales (4 runs of 16 values)
//   F32/F16  64 consecutive values
// Lanes of a warp take consecutive chunks of a row, so a warp's load is one contiguous, fully coalesced segment.
//
// Activations live in shared memory, one padded row per token: value k sits at index k + 4*(k/64), so that lanes
// working on different chunks hit different bank groups with their float4 reads.
#pragma once
#include "redcuda_formats.cuh"
#include "redcuda_kquants.cuh"

namespace rc {

__device__ __forceinline__ uint32_t xi(uint32_t k) { return k + ((k >> 6) << 2); }
__host__ __device__ __forceinline__ uint32_t x_padded(uint32_t ncols) { return ncols + ((ncols >> 6) << 2); }

struct SBooks { const uint2 *iq2; const uint32_t *iq3s; };   // shared-memory copies of the codebooks

// float4 loads of 8 consecutive activations of every token, multiplied into s[t]
template <int NT>
__device__ __forceinline__ void fma8(const float (&w)[8], const float *xs, uint32_t xstride, uint32_t idx, float (&s)[NT]) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const float4 a = *reinterpret_cast<const float4 *>(xs + t * xstride + idx);
        const float4 b = *reinterpret_cast<const float4 *>(xs + t * xstride + idx + 4);
        s[t] += w[0] * a.x + w[1] * a.y + w[2] * a.z + w[3] * a.w + w[4] * b.x + w[5] * b.y + w[6] * b.z + w[7] * b.w;
    }
}

// ---- IQ2_XXS: chunk cc (0..3) of block blk; kblk = column of the block's first value within the row ----
template <int NT>
__device__ __forceinline__ void chunk_iq2xxs(const uint8_t *base, uint64_t nb, uint64_t blk, uint32_t cc, uint32_t kblk,
                                             const float *xs, uint32_t xstride, const SBooks &sb, float (&acc)[NT]) {
    const uint4 q = __ldg(reinterpret_cast<const uint4 *>(base) + blk * 4u + cc);
    const float d = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(base + rc_iq2_d(nb)) + blk)));
    const uint32_t x0 = xi(kblk + cc * 64u);
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
        const uint32_t auxg = grp ? q.z : q.x, auxs = grp ? q.w : q.y;
        const float db = d * (0.5f + (float)(auxs >> 28)) * 0.25f;
        float s[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) s[t] = 0.f;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint2 gv = sb.iq2[(auxg >> (8 * l)) & 255u];
            const uint32_t s8 = rc_sign8((auxs >> (7 * l)) & 127u);
            float w[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w[j] = (float)((gv.x >> (8 * j)) & 255u);
                w[j + 4] = (float)((gv.y >> (8 * j)) & 255u);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = __uint_as_float(__float_as_uint(w[j]) ^ (((s8 >> j) & 1u) << 31));
            fma8<NT>(w, xs, xstride, x0 + grp * 32 + l * 8, s);
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] += db * s[t];
    }
}

// ---- IQ3_S ----
template <int NT>
__device__ __forceinline__ void chunk_iq3s(const uint8_t *base, uint64_t nb, uint64_t blk, uint32_t cc, uint32_t kblk,
                                           const float *xs, uint32_t xstride, const SBooks &sb, float (&acc)[NT]) {
    const uint4 qs = __ldg(reinterpret_cast<const uint4 *>(base) + blk * 4u + cc);
    const uint2 sg = __ldg(reinterpret_cast<const uint2 *>(base + rc_iq3_signs(nb)) + blk * 4u + cc);
    const uint32_t qh2 = __ldg(reinterpret_cast<const unsigned short *>(base + rc_iq3_qh(nb)) + blk * 4u + cc);
    const uint32_t scb = __ldg(base + rc_iq3_scales(nb) + blk * 4u + cc);
    const float d = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(base + rc_iq3_d(nb)) + blk)));
    const uint32_t x0 = xi(kblk + cc * 64u);
#pragma unroll
    for (int sub = 0; sub < 2; ++sub) {
        const uint32_t w0 = sub ? qs.z : qs.x, w1 = sub ? qs.w : qs.y;
        const uint32_t qh = (qh2 >> (8 * sub)) & 255u, signs = sub ? sg.y : sg.x;
        const float db = d * (float)(1 + 2 * (int)((scb >> (4 * sub)) & 15u));
        float s[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) s[t] = 0.f;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t word = l < 2 ? w0 : w1;
            const uint32_t b0 = (word >> (16 * (l & 1))) & 255u, b1 = (word >> (16 * (l & 1) + 8)) & 255u;
            const uint32_t g1 = sb.iq3s[b0 | ((qh << (8 - 2 * l)) & 256u)], g2 = sb.iq3s[b1 | ((qh << (7 - 2 * l)) & 256u)];
            const uint32_t s8 = (signs >> (8 * l)) & 255u;
            float w[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w[j] = (float)((g1 >> (8 * j)) & 255u);
                w[j + 4] = (float)((g2 >> (8 * j)) & 255u);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = __uint_as_float(__float_as_uint(w[j]) ^ (((s8 >> j) & 1u) << 31));
            fma8<NT>(w, xs, xstride, x0 + sub * 32 + l * 8, s);
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] += db * s[t];
    }
}

// ---- Q6_K: chunk cc = (half, 16-wide l range); its 64 values are 4 runs of 16 at k = half*128 + 32*quarter + l0 ----
template <int NT>
__device__ __forceinline__ void chunk_q6k(const uint8_t *base, uint64_t nb, uint64_t blk, uint32_t cc, uint32_t kblk,
                                          const float *xs, uint32_t xstride, float (&acc)[NT]) {
    const uint32_t half = cc >> 1, l0 = (cc & 1u) * 16u;
    const uint4 qa = __ldg(reinterpret_cast<const uint4 *>(base + blk * 128u + half * 64u + l0));
    const uint4 qb = __ldg(reinterpret_cast<const uint4 *>(base + blk * 128u + half * 64u + 32u + l0));
    const uint4 hh = __ldg(reinterpret_cast<const uint4 *>(base + rc_q6_qh(nb) + blk * 64u + half * 32u + l0));
    const signed char *sc = reinterpret_cast<const signed char *>(base + rc_q6_sc(nb) + blk * 16u + half * 8u + (cc & 1u));
    const float d = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(base + rc_q6_d(nb)) + blk)));
    const float ds[4] = {d * (float)__ldg(sc), d * (float)__ldg(sc + 2), d * (float)__ldg(sc + 4), d * (float)__ldg(sc + 6)};
    const uint32_t a4[4] = {qa.x, qa.y, qa.z, qa.w}, b4[4] = {qb.x, qb.y, qb.z, qb.w}, h4[4] = {hh.x, hh.y, hh.z, hh.w};
    float s[4][NT];
#pragma unroll
    for (int qd = 0; qd < 4; ++qd)
#pragma unroll
        for (int t = 0; t < NT; ++t) s[qd][t] = 0.f;
    const uint32_t kbase = kblk + half * 128u + l0;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const uint32_t a = a4[w], b = b4[w], h = h4[w];
        const uint32_t v[4] = {(a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u), (b & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u),
                               ((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u), ((b >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u)};
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            const uint32_t idx = xi(kbase + 32u * qd + 4u * w);
            const float w0 = (float)((int)(v[qd] & 255u) - 32), w1 = (float)((int)((v[qd] >> 8) & 255u) - 32);
            const float w2 = (float)((int)((v[qd] >> 16) & 255u) - 32), w3 = (float)((int)(v[qd] >> 24) - 32);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const float4 x4 = *reinterpret_cast<const float4 *>(xs + t * xstride + idx);
                s[qd][t] += w0 * x4.x + w1 * x4.y + w2 * x4.z + w3 * x4.w;
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] += ds[0] * s[0][t] + ds[1] * s[1][t] + ds[2] * s[2][t] + ds[3] * s[3][t];
}

// ---- F32 / F16 rows, accumulated in double (router logits and the shared-expert gate decide discrete outcomes) ----
template <int NT>
__device__ __forceinline__ void chunk_plain(uint32_t type, const uint8_t *base, uint64_t row, uint32_t ncols, uint32_t c,
                                            const float *xs, uint32_t xstride, double (&acc)[NT]) {
    const uint32_t k0 = c * 64u, x0 = xi(k0);
    if (type == RC_F32) {
        const float4 *wp = reinterpret_cast<const float4 *>(base + (row * ncols + k0) * 4u);
#pragma unroll 8              // eight 16-byte loads in flight per lane: a lane's 256 bytes arrive in two round trips, not four
        for (int i = 0; i < 16; ++i) {
            const float4 w = __ldg(wp + i);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const float4 x4 = *reinterpret_cast<const float4 *>(xs + t * xstride + x0 + 4 * i);
                acc[t] += (double)w.x * x4.x + (double)w.y * x4.y + (double)w.z * x4.z + (double)w.w * x4.w;
            }
        }
    } else {
        const uint2 *wp = reinterpret_cast<const uint2 *>(base + (row * ncols + k0) * 2u);
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
            const uint2 r = __ldg(wp + i);
            const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&r.x)), hi = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const float4 x4 = *reinterpret_cast<const float4 *>(xs + t * xstride + x0 + 4 * i);
                acc[t] += (double)lo.x * x4.x + (double)lo.y * x4.y + (double)hi.x * x4.z + (double)hi.y * x4.w;
            }
        }
    }
}

// Dot products of one row with NT activation rows, spread over LPR lanes (LPR = power of two <= 32, lanes of one row
// are adjacent). cpr = chunks per row = ncols / 64. After the call every lane of the row's group holds the full sums.
template <int TYPE, int NT>
__device__ __forceinline__ void row_dot(const uint8_t *base, uint64_t nb, uint64_t row, uint32_t ncols, uint32_t lpr, uint32_t sub,
                                        const float *xs, uint32_t xstride, const SBooks &sb, float (&out)[NT]) {
    const uint32_t cpr = ncols >> 6;
    if (TYPE == RC_Q8_0 || TYPE == RC_Q2_K || TYPE == RC_Q4_K || TYPE == RC_Q5_K) {
        // rows in file layout, a value at a time: correct for every type of the family, not tuned
        float acc[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = 0.f;
        const uint8_t *rp = base + row * rc_row_bytes(TYPE, ncols);
        for (uint32_t c = sub; c < cpr; c += lpr)
            for (uint32_t j = 0; j < 64u; ++j) {
                const uint32_t k = c * 64u + j;
                const float w = kq_row_value(TYPE, rp, k);
#pragma unroll
                for (int t = 0; t < NT; ++t) acc[t] = fmaf(w, xs[t * xstride + xi(k)], acc[t]);
            }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            for (uint32_t o = lpr >> 1; o; o >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
            out[t] = acc[t];
        }
    } else if (TYPE == RC_F32 || TYPE == RC_F16) {
        double acc[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = 0.0;
        for (uint32_t c = sub; c < cpr; c += lpr) chunk_plain<NT>(TYPE, base, row, ncols, c, xs, xstride, acc);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            for (uint32_t o = lpr >> 1; o; o >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
            out[t] = (float)acc[t];
        }
    } else {
        float acc[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = 0.f;
        const uint64_t blk0 = row * (uint64_t)(ncols >> 8);
        for (uint32_t c = sub; c < cpr; c += lpr) {
            const uint64_t blk = blk0 + (c >> 2);
            const uint32_t cc = c & 3u, kblk = (c >> 2) << 8;
            if (TYPE == RC_IQ2_XXS) chunk_iq2xxs<NT>(base, nb, blk, cc, kblk, xs, xstride, sb, acc);
            else if (TYPE == RC_IQ3_S) chunk_iq3s<NT>(base, nb, blk, cc, kblk, xs, xstride, sb, acc);
            else chunk_q6k<NT>(base, nb, blk, cc, kblk, xs, xstride, acc);
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            for (uint32_t o = lpr >> 1; o; o >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
            out[t] = acc[t];
        }
    }
}

__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

// Cooperative copy of the codebooks into shared memory (whole block; caller syncs).
__device__ __forceinline__ void load_books(uint2 *s_iq2, uint32_t *s_iq3s, const uint8_t *g_iq2, const uint32_t *g_iq3s, uint32_t type_mask) {
    if (type_mask & (1u << RC_IQ2_XXS)) for (uint32_t i = threadIdx.x; i < 256u; i += blockDim.x) s_iq2[i] = reinterpret_cast<const uint2 *>(g_iq2)[i];
    if (type_mask & (1u << RC_IQ3_S)) for (uint32_t i = threadIdx.x; i < 512u; i += blockDim.x) s_iq3s[i] = g_iq3s[i];
}

// Stage `nt` activation rows (global, row stride src_stride, row picked by rows[t] when rows != nullptr) into padded
// shared rows; rows beyond nt are zero-filled so that fixed-width inner loops read defined values.
template <int NT>
__device__ __forceinline__ void stage_x(float *xs, uint32_t xstride, const float *src, size_t src_stride, const uint32_t *rows,
                                        uint32_t first, uint32_t nt, uint32_t ncols) {
    const uint32_t n4 = ncols >> 2;
    for (uint32_t i = threadIdx.x; i < NT * n4; i += blockDim.x) {
        const uint32_t t = i / n4, k = (i - t * n4) << 2;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < nt) {
            const size_t r = rows ? rows[first + t] : (size_t)(first + t);
            v = *reinterpret_cast<const float4 *>(src + r * src_stride + k);
        }
        *reinterpret_cast<float4 *>(xs + t * xstride + xi(k)) = v;
    }
}

}  // namespace rc
