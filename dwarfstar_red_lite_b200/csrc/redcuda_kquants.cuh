// Value decode of the GGUF types kept in their file layout (Q8_0, Q2_K, Q4_K, Q5_K): shared by the stage kernels
// (redcuda_kquants.cu), the GEMV and the embedding lookup. The float operations and their order are the reference's
// (native/redlite_native_quant_cpu.c:40-128); every multiply and subtract is rounded on its own, so no fused
// multiply-add changes a bit.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace rc {

__host__ __device__ __forceinline__ bool kq_type(uint32_t t) { return t == 8u || t == 10u || t == 12u || t == 13u; }
__host__ __device__ __forceinline__ uint32_t kq_block_values(uint32_t t) { return t == 8u ? 32u : 256u; }
__host__ __device__ __forceinline__ uint32_t kq_block_bytes(uint32_t t) { return t == 8u ? 34u : t == 10u ? 84u : t == 12u ? 144u : 176u; }

#ifdef __CUDACC__
__device__ __forceinline__ float kq_f16(const uint8_t *p) { return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8)))); }
// the packed 6-bit scale / min pairs of Q4_K and Q5_K (quant_cpu.c:40-46)
__device__ __forceinline__ void kq_scale_min(uint32_t j, const uint8_t *q, uint32_t &d, uint32_t &m) {
    if (j < 4u) { d = q[j] & 63u; m = q[j + 4u] & 63u; }
    else { d = (q[j + 4u] & 0x0fu) | ((uint32_t)(q[j - 4u] >> 6) << 4); m = (uint32_t)(q[j + 4u] >> 4) | ((uint32_t)(q[j] >> 6) << 4); }
}
// value j of the block at bp: (d * sc) * q - (dmin * mn); Q8_0: d * q
__device__ __forceinline__ float kq_value(uint32_t t, const uint8_t *bp, uint32_t j) {
    if (t == 8u) return __fmul_rn(kq_f16(bp), (float)(int)(int8_t)bp[2u + j]);
    float d, dmin; uint32_t sc, mn, q;
    if (t == 10u) {
        const uint32_t half = j >> 7, r = j & 127u, sub = r >> 5, l = r & 31u;
        const uint32_t scb = bp[half * 8u + sub * 2u + (l >> 4)];
        d = kq_f16(bp + 80u); dmin = kq_f16(bp + 82u); sc = scb & 0xFu; mn = scb >> 4;
        q = (bp[16u + half * 32u + l] >> (2u * sub)) & 3u;
    } else {
        const uint32_t g = j >> 5, l = j & 31u;
        d = kq_f16(bp); dmin = kq_f16(bp + 2u);
        kq_scale_min(g, bp + 4u, sc, mn);
        if (t == 12u) {
            const uint32_t b = bp[16u + (g >> 1) * 32u + l];
            q = (g & 1u) ? (b >> 4) : (b & 0x0fu);
        } else {
            const uint32_t b = bp[48u + (g >> 1) * 32u + l];
            q = ((g & 1u) ? (b >> 4) : (b & 0x0fu)) + (((bp[16u + l] >> g) & 1u) ? 16u : 0u);
        }
    }
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
}
// column c of a row in file layout
__device__ __forceinline__ float kq_row_value(uint32_t t, const uint8_t *row, uint32_t c) {
    const uint32_t bv = kq_block_values(t);
    return kq_value(t, row + (uint64_t)(c / bv) * kq_block_bytes(t), c % bv);
}
#endif

}  // namespace rc
