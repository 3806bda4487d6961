// Prefill projections on the 5th-generation tensor cores (tcgen05): out[t][r] = sum_k W[r][k] * x[t][k] for a chunk of
// tokens, W a quantised matrix (Q6_K / IQ2_XXS / IQ3_S rows, planar layout) that is decoded on the fly.
//
// The batched form of rl_quant_row_dot over every row (native/redlite_native_quant_cpu.c:247-266); the reference's GPU
// prefill dequantises to f32 and runs an f32 GEMM (native/redmetal_engine_prefill.m:205-227, 889-909). Results have to
// stay at fp32 accuracy (the 48-layer model amplifies rounding noise by orders of magnitude), so neither operand is
// rounded to one 16-bit value: both are split into two fp16 digits, v * 2^e = hi + lo (|error| <= 2^-22 |v|), and
// three products are accumulated in fp32 in tensor memory: hi*hi + hi*lo + lo*hi. The power-of-two scales (per row
// tile for the weights, per token for the activations) keep hi in the normal fp16 range and are undone in the epilogue.
// The tensor core adds into its fp32 accumulator without rounding to nearest, so a long chain of accumulations drifts
// (measured: 2e-5 of the result over 2048 columns, a hundred times the error of an fp32 sum). Two measures keep the
// result at fp32 accuracy: the small cross products (hi*lo, lo*hi) have an accumulator of their own, so their
// truncation is relative to their own size, and the accumulators only ever cover one 256-column block (16 MMAs for
// hi*hi): they are double-buffered in tensor memory, read back with tcgen05.ld while the next block multiplies, and
// summed over the blocks in fp32 registers with ordinary rounding.
//
// Two kernels per launch. k_tc_decode_w turns the launch's weights into fp16 digit tiles once (the exact decoder of the
// GEMV path on raw blocks staged by cp.async, canonical K-major core-matrix layout, no swizzle; 4 bytes per weight in a
// scratch that the caller sizes for its widest launch), so that the GEMM decodes nothing: before, every token tile of a
// 2048-token chunk decoded the whole matrix again behind a block barrier per stage. k_tc_gemm then streams a stage's
// weight digits and activation digits (laid out for the MMA by k_tc_prep_x) with two bulk copies on one mbarrier and is
// split into roles (producer thread, MMA thread, drain warps) that meet only on mbarriers; see the kernel's own header.
// Every wait on an mbarrier is bounded; on a timeout the kernel raises a flag, frees its tensor memory and returns.
#define RC_PDL_DEFAULT 0
#include "redcuda_common.cuh"
#include "redcuda_formats.cuh"
#include "redcuda_dot.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_tc_gemm.cuh"

#include <cuda_fp16.h>

namespace rc {

__device__ __forceinline__ uint32_t tc_d_plane(uint32_t type, uint64_t nb) {
    return (uint32_t)(type == RC_Q6_K ? rc_q6_d(nb) : type == RC_IQ2_XXS ? rc_iq2_d(nb) : rc_iq3_d(nb));
}

__device__ __forceinline__ void cp_async_n(uint32_t dst, const void *src, uint32_t bytes) {
    if (bytes == 8u) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" :: "r"(dst), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(dst), "l"(src) : "memory");
}

// ---- raw staging area: the quant blocks of one 256-column block of the tile's 128 rows, one plane per block field.
// Row pitches are padded so that the 32 rows a warp decodes at once fall into distinct banks (8-byte reads: two
// wavefronts, the minimum). Offsets in bytes from the start of the area:
//   Q6_K     ql pitch 136 @0, qh pitch 72 @17408, scales pitch 20 @26624, d (fp16) @29184           -> 29440
//   IQ2_XXS  qs pitch 72 @0, d @9216                                                                -> 9472
//   IQ3_S    qs pitch 72 @0, signs pitch 40 @9216, qh pitch 12 @14336, scales pitch 4 @15872, d @16384 -> 16640
__host__ __device__ __forceinline__ uint32_t tc_raw_bytes(uint32_t type) { return type == RC_Q6_K ? 29440u : type == RC_IQ2_XXS ? 9472u : 16640u; }
__device__ __forceinline__ uint32_t tc_raw_d(uint32_t type) { return type == RC_Q6_K ? 29184u : type == RC_IQ2_XXS ? 9216u : 16384u; }

// Request block column c of rows [row0, row0 + 128) into `raw` (cp.async, one commit group). The 2-byte block scales
// come back in a register of the threads that own a row (tid < 128) and are stored by tc_put_d.
__device__ __forceinline__ unsigned short tc_stage_raw(uint32_t type, const uint8_t *w, uint64_t nb, uint32_t bpr, uint32_t row0, uint32_t nrows,
                                                       uint32_t c, uint8_t *raw, uint32_t tid) {
    const uint32_t raw_s = smem_u32(raw);
    auto plane = [&](uint64_t off_g, uint32_t off_s, uint32_t piece, uint32_t pitch, uint32_t unit) {
        const uint32_t per_row = piece / unit;
        for (uint32_t i = tid; i < TC_M * per_row; i += TC_THREADS) {
            const uint32_t r = i / per_row, u = i - r * per_row;
            if (row0 + r < nrows) cp_async_n(raw_s + off_s + r * pitch + u * unit, w + off_g + ((uint64_t)(row0 + r) * bpr + c) * piece + u * unit, unit);
        }
    };
    if (type == RC_Q6_K) {
        plane(0u, 0u, 128u, 136u, 8u); plane(rc_q6_qh(nb), 17408u, 64u, 72u, 8u); plane(rc_q6_sc(nb), 26624u, 16u, 20u, 4u);
    } else if (type == RC_IQ2_XXS) {
        plane(0u, 0u, 64u, 72u, 8u);
    } else {
        plane(0u, 0u, 64u, 72u, 8u); plane(rc_iq3_signs(nb), 9216u, 32u, 40u, 8u); plane(rc_iq3_qh(nb), 14336u, 8u, 12u, 4u);
        plane(rc_iq3_scales(nb), 15872u, 4u, 4u, 4u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    unsigned short d = 0;
    if (tid < TC_M && row0 + tid < nrows) d = __ldg(reinterpret_cast<const unsigned short *>(w + tc_d_plane(type, nb)) + (uint64_t)(row0 + tid) * bpr + c);
    return d;
}

__device__ __forceinline__ void tc_put_d(uint32_t type, uint8_t *raw, uint32_t tid, unsigned short d) {
    if (tid < TC_M) reinterpret_cast<unsigned short *>(raw + tc_raw_d(type))[tid] = d;
}

// byte j of w as a float without a conversion instruction: one PRMT builds the bits of 2^23 + byte
__device__ __forceinline__ float tc_byte_f(uint32_t w, int j) { return __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7540u | (uint32_t)j)); }

// two scaled values -> their fp16 digits: hi = the top 11 significant bits (the low 13 mantissa bits cleared, so the
// conversion is exact in the normal fp16 range), lo = the rounded remainder; packed conversions, two values each
__device__ __forceinline__ void tc_split2(float a, float b, uint32_t &hi, uint32_t &lo) {
    const float ah = __uint_as_float(__float_as_uint(a) & 0xffffe000u), bh = __uint_as_float(__float_as_uint(b) & 0xffffe000u);
    const __half2 hh = __floats2half2_rn(ah, bh), ll = __floats2half2_rn(a - ah, b - bh);
    hi = *reinterpret_cast<const uint32_t *>(&hh); lo = *reinterpret_cast<const uint32_t *>(&ll);
}

// The 8 consecutive values [8*g8, 8*g8 + 8) of row r's block from the staging area, times the tile's power-of-two
// scale, as two fp16 digits. The float operations are those of rc_decode8 with d replaced by d * scale (a power of two
// commutes with every rounding), read with 8-byte shared-memory loads.
template <uint32_t TYPE>
__device__ __forceinline__ void tc_decode_split(const uint8_t *raw, uint32_t r, uint32_t g8, float scale, const RcBooks &bk, uint4 &hi, uint4 &lo) {
    const float d = __half2float(__ushort_as_half(reinterpret_cast<const unsigned short *>(raw + tc_raw_d(TYPE))[r])) * scale;
    float v[8];
    if (TYPE == RC_Q6_K) {
        const uint32_t k = g8 * 8u, half = k >> 7, quarter = (k & 127u) >> 5, l0 = k & 31u;
        const uint2 ql = *reinterpret_cast<const uint2 *>(raw + r * 136u + half * 64u + (quarter & 1u) * 32u + l0);
        const uint2 qh = *reinterpret_cast<const uint2 *>(raw + 17408u + r * 72u + half * 32u + l0);
        const int sc = (int)(int8_t)raw[26624u + r * 20u + half * 8u + (l0 >> 4) + 2u * quarter];
        const float ds = d * (float)sc;
        const uint32_t nsh = quarter < 2u ? 0u : 4u, hsh = 2u * quarter;
        const uint32_t w0 = ((ql.x >> nsh) & 0x0f0f0f0fu) | (((qh.x >> hsh) & 0x03030303u) << 4);
        const uint32_t w1 = ((ql.y >> nsh) & 0x0f0f0f0fu) | (((qh.y >> hsh) & 0x03030303u) << 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {      // 6-bit value 0..63: (2^23 + value) - (2^23 + 32) = value - 32, exactly
            v[j] = ds * (tc_byte_f(w0, j) - 8388640.f);
            v[j + 4] = ds * (tc_byte_f(w1, j) - 8388640.f);
        }
    } else if (TYPE == RC_IQ2_XXS) {
        const uint32_t ib32 = g8 >> 2, l = g8 & 3u;
        const uint2 aux = *reinterpret_cast<const uint2 *>(raw + r * 72u + ib32 * 8u);
        const float db = d * (0.5f + (float)(aux.y >> 28)) * 0.25f;
        const uint2 gv = __ldg(reinterpret_cast<const uint2 *>(bk.iq2 + ((aux.x >> (8u * l)) & 255u) * 8u));
        const uint32_t s8 = rc_sign8((aux.y >> (7u * l)) & 127u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float m = db * (tc_byte_f(j < 4 ? gv.x : gv.y, j & 3) - 8388608.f);
            v[j] = __uint_as_float(__float_as_uint(m) ^ ((s8 << (31 - j)) & 0x80000000u));
        }
    } else {
        const uint32_t ib32 = g8 >> 2, l = g8 & 3u;
        const uint8_t *qs = raw + r * 72u + 8u * ib32;
        const uint32_t qh = raw[14336u + r * 12u + ib32];
        const uint32_t sg = raw[9216u + r * 40u + 4u * ib32 + l];
        const uint32_t scb = raw[15872u + r * 4u + (ib32 >> 1)];
        const float db = d * (float)(1 + 2 * (int)((scb >> (4u * (ib32 & 1u))) & 0xfu));
        const uint32_t i1 = qs[2u * l] | ((qh << (8u - 2u * l)) & 256u), i2 = qs[2u * l + 1u] | ((qh << (7u - 2u * l)) & 256u);
        const uint32_t g1 = __ldg(bk.iq3s + i1), g2 = __ldg(bk.iq3s + i2);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float m1 = db * (tc_byte_f(g1, j) - 8388608.f), m2 = db * (tc_byte_f(g2, j) - 8388608.f);
            v[j] = __uint_as_float(__float_as_uint(m1) ^ ((sg << (31 - j)) & 0x80000000u));
            v[j + 4] = __uint_as_float(__float_as_uint(m2) ^ ((sg << (27 - j)) & 0x80000000u));
        }
    }
    tc_split2(v[0], v[1], hi.x, lo.x); tc_split2(v[2], v[3], hi.y, lo.y);
    tc_split2(v[4], v[5], hi.z, lo.z); tc_split2(v[6], v[7], hi.w, lo.w);
}

// the weight digits of one stage: thread -> (row, k-chunk of 8), 32 consecutive rows per warp pass (padded pitches: no
// bank conflicts on the reads, and the 16-byte digit stores of a warp are contiguous)
template <uint32_t TYPE>
__device__ __forceinline__ void tc_decode_stage(const uint8_t *raw, uint8_t *abuf, uint32_t g8_0, uint32_t rows_live, float scale, const RcBooks &bk, uint32_t tid) {
#pragma unroll
    for (uint32_t it = 0; it < (TC_M * 8u) / TC_THREADS; ++it) {
        const uint32_t item = it * TC_THREADS + tid, r = item & (TC_M - 1u), kc = item >> 7;
        uint4 hi = make_uint4(0u, 0u, 0u, 0u), lo = hi;
        if (r < rows_live) tc_decode_split<TYPE>(raw, r, g8_0 + kc, scale, bk, hi, lo);
        const uint32_t off = kc * (TC_M * 16u) + r * 16u;          // [k chunk][row group][row in group][16 B]
        *reinterpret_cast<uint4 *>(abuf + off) = hi;
        *reinterpret_cast<uint4 *>(abuf + TC_A_DIGIT + off) = lo;
    }
}

// the same for a plain fp32 matrix (router weights): rows of ncols floats, stage = columns [col0, col0 + 64)
__device__ __forceinline__ void tc_decode_stage_f32(const float *w, uint32_t ncols, uint32_t row0, uint32_t col0, uint8_t *abuf, uint32_t rows_live, float scale, uint32_t tid) {
#pragma unroll
    for (uint32_t it = 0; it < (TC_M * 8u) / TC_THREADS; ++it) {
        const uint32_t item = it * TC_THREADS + tid, kc = item & 7u, r = item >> 3;      // 8 lanes read 256 contiguous bytes of a row
        uint4 hi = make_uint4(0u, 0u, 0u, 0u), lo = hi;
        if (r < rows_live) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(w + (size_t)(row0 + r) * ncols + col0 + kc * 8u));
            const float4 b = __ldg(reinterpret_cast<const float4 *>(w + (size_t)(row0 + r) * ncols + col0 + kc * 8u + 4u));
            tc_split2(a.x * scale, a.y * scale, hi.x, lo.x); tc_split2(a.z * scale, a.w * scale, hi.y, lo.y);
            tc_split2(b.x * scale, b.y * scale, hi.z, lo.z); tc_split2(b.z * scale, b.w * scale, hi.w, lo.w);
        }
        const uint32_t off = kc * (TC_M * 16u) + r * 16u;
        *reinterpret_cast<uint4 *>(abuf + off) = hi;
        *reinterpret_cast<uint4 *>(abuf + TC_A_DIGIT + off) = lo;
    }
}

// x [ntok][ncols] fp32 (or SiLU(x) * x2 when x2 is given) -> fp16 digits in the order the GEMM stages consume them:
// xs[token tile][k stage][k chunk of 8 (8)][digit hi/lo][token group of 8 (TN/8)][token in group (8)][8 halves];
// x_inv[t] = 2^-e_t undoes the per-token scale. Tokens beyond ntok are zero. grid = token tiles * TN, block = 256
__global__ void k_tc_prep_x(const float *__restrict__ x, const float *__restrict__ x2, uint32_t x_stride, uint32_t ntok, uint32_t ncols, uint32_t tn,
                            __half *__restrict__ xs, float *__restrict__ x_inv) {
    pdl_prologue();
    __shared__ float red[8];
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    const bool live = t < ntok;
    float mx = 0.f;
    auto val = [&](uint32_t k) { const size_t i = (size_t)t * x_stride + k; return x2 ? silu_mul(x[i], x2[i]) : x[i]; };
    if (live) for (uint32_t k = tid; k < ncols; k += blockDim.x) mx = fmaxf(mx, fabsf(val(k)));
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((tid & 31u) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = 0.f;
    for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
    int e = 0;
    if (mx > 0.f && mx < INFINITY) { int ex; frexpf(mx, &ex); e = 14 - ex; }     // max |x| * 2^e in [2^13, 2^14)
    e = e > 100 ? 100 : e < -100 ? -100 : e;
    const float sc = exp2f((float)e);
    if (tid == 0) x_inv[t] = exp2f((float)-e);
    const uint32_t tile = t / tn, tt = t - tile * tn, nstage = ncols / TC_KS;
    const size_t digit = (size_t)tn * TC_KS;                   // halves of one digit of one stage
    for (uint32_t c = tid; c < ncols / 8u; c += blockDim.x) {  // one 16-byte k-chunk per iteration
        const uint32_t stage = c >> 3, kc = c & 7u;
        __half hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float v = live ? val(c * 8u + j) * sc : 0.f;
            hi[j] = __float2half_rn(v);
            lo[j] = __float2half_rn(v - __half2float(hi[j]));
        }
        // inside a stage: [k chunk][2 tn rows: the hi digits of the tn tokens, then their lo digits][8 halves], so that one MMA
        // of N = 2 tn takes both digits and one of N = tn the hi digits alone
        __half *dst = xs + ((size_t)tile * nstage + stage) * 2u * digit + ((size_t)kc * (tn >> 2) + (tt >> 3)) * 64u + (tt & 7u) * 8u;
        *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(hi);
        *reinterpret_cast<uint4 *>(dst + (size_t)tn * 8u) = *reinterpret_cast<const uint4 *>(lo);
    }
}

// ---- weights of a launch -> fp16 digit tiles, once per launch -----------------------------------------------------------
// wd[row tile][stage][hi 16 KB | lo 16 KB] in the layout an MMA stage reads (tc_decode_stage), w_inv[row tile] = the inverse
// of the tile's power-of-two scale. grid = (row tiles of the launch, 256-column blocks), block = TC_THREADS.
__global__ void __launch_bounds__(TC_THREADS) k_tc_decode_w(const __grid_constant__ TcArgs A) {
    pdl_prologue();
    __shared__ __align__(16) uint8_t raw[29440];          // tc_raw_bytes of the widest format
    __shared__ float red[TC_WARPS];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    uint32_t ji = 0;
    for (uint32_t j = 1; j < A.njobs; ++j) if (blockIdx.x >= A.job[j].tile0) ji = j;
    const TcJob &J = A.job[ji];
    const uint32_t row0 = (blockIdx.x - J.tile0) * TC_M, c = blockIdx.y, bpr = A.ncols >> 8, nstage = A.ncols / TC_KS;
    const RcBooks bk{A.iq2, A.iq3s};
    const bool f32 = J.type == RC_F32;
    const unsigned short d = f32 ? (unsigned short)0 : tc_stage_raw(J.type, J.w, J.nb, bpr, row0, J.nrows, c, raw, tid);
    // power-of-two scale of the tile: the largest block scale d times the largest integer factor of the format (fp32 rows:
    // the largest magnitude of the tile itself)
    float dmax = 0.f;
    if (f32) {
        const float *wf = reinterpret_cast<const float *>(J.w);
        const uint32_t rows = J.nrows - row0 < TC_M ? J.nrows - row0 : TC_M;
        for (uint32_t i = tid; i < rows * (A.ncols >> 2); i += TC_THREADS) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(wf + (size_t)row0 * A.ncols) + i);
            dmax = fmaxf(fmaxf(dmax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
        for (int o = 16; o; o >>= 1) dmax = fmaxf(dmax, __shfl_xor_sync(0xffffffffu, dmax, o));
        if (lane == 0) red[warp] = dmax;
    } else {
        const unsigned short *dp = reinterpret_cast<const unsigned short *>(J.w + tc_d_plane(J.type, J.nb));
        for (uint32_t i = tid; i < TC_M * bpr; i += TC_THREADS) {
            const uint32_t r = row0 + i / bpr;
            if (r < J.nrows) dmax = fmaxf(dmax, fabsf(__half2float(__ushort_as_half(__ldg(dp + (size_t)r * bpr + (i % bpr))))));
        }
        for (int o = 16; o; o >>= 1) dmax = fmaxf(dmax, __shfl_xor_sync(0xffffffffu, dmax, o));
        if (lane == 0) red[warp] = dmax;
    }
    if (!f32) tc_put_d(J.type, raw, tid, d);
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    dmax = 0.f;
    for (uint32_t w = 0; w < TC_WARPS; ++w) dmax = fmaxf(dmax, red[w]);
    int we = 0;
    {
        const float bound = dmax * (f32 ? 1.f : J.type == RC_Q6_K ? 4096.f : J.type == RC_IQ2_XXS ? 256.f : 512.f);
        if (bound > 0.f && bound < INFINITY) { int ex; frexpf(bound, &ex); we = 15 - ex; }       // |w| * 2^we < 2^15
        we = we > 100 ? 100 : we < -100 ? -100 : we;
    }
    const float w_scale = exp2f((float)we);
    if (c == 0u && tid == 0) A.w_inv[blockIdx.x] = exp2f((float)-we);
    const uint32_t rows_live = J.nrows - row0 < TC_M ? J.nrows - row0 : TC_M;
#pragma unroll 1
    for (uint32_t st = 0; st < 256u / TC_KS; ++st) {
        uint8_t *dst = A.wd + ((size_t)blockIdx.x * nstage + c * (256u / TC_KS) + st) * (2u * TC_A_DIGIT);
        if (f32) tc_decode_stage_f32(reinterpret_cast<const float *>(J.w), A.ncols, row0, c * 256u + st * TC_KS, dst, rows_live, w_scale, tid);
        else if (J.type == RC_Q6_K) tc_decode_stage<RC_Q6_K>(raw, dst, st * (TC_KS / 8u), rows_live, w_scale, bk, tid);
        else if (J.type == RC_IQ2_XXS) tc_decode_stage<RC_IQ2_XXS>(raw, dst, st * (TC_KS / 8u), rows_live, w_scale, bk, tid);
        else tc_decode_stage<RC_IQ3_S>(raw, dst, st * (TC_KS / 8u), rows_live, w_scale, bk, tid);
    }
}

// ---- the GEMM proper: one CTA = 128 weight rows (MMA M) x TN tokens (MMA N) x all columns, K in stages of 64 -------------
//   warp 0, one thread   producer: per stage ONE mbarrier transaction of two bulk copies (the stage's weight digits from wd,
//                        its activation digits from xs), NS stages ahead of the MMAs
//   warp 1, one thread   issues 4 k-steps x 2 tcgen05.mma per stage (A_hi x [B_hi | B_lo], N = 2 TN; A_lo x B_hi, N = TN), a
//                        tcgen05.commit that frees the stage's buffers, and after every fourth stage one that hands the
//                        256-column block's accumulator pair to the drain warps
//   warps 2..9           tcgen05.ld of a finished block's two accumulators into fp32 register sums while the next block
//                        multiplies into the other pair; scaling and stores at the end
// No block-wide barrier inside the loop; every wait on an mbarrier is bounded, and a wait that gives up raises a flag that
// every role reads before its next wait, so the CTA winds down, frees its tensor memory and reports the timeout.
constexpr uint32_t TCG_THREADS = 320u, TCG_DRAIN_WARPS = 8u;
template <int TN> struct TcCfg { static constexpr uint32_t NS = TN >= 128 ? 3u : 4u; };

template <int TN>
__global__ void __launch_bounds__(TCG_THREADS, 1) k_tc_gemm(const __grid_constant__ TcArgs A) {
    pdl_prologue();
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t NS = TcCfg<TN>::NS;
    constexpr uint32_t B_DIGIT = (uint32_t)TN * TC_KS * 2u, A_BUF = 2u * TC_A_DIGIT, B_BUF = 2u * B_DIGIT, STAGE = A_BUF + B_BUF;
    constexpr uint32_t TMEM_COLS = 4u * (uint32_t)TN;     // two blocks in flight x (hi*hi accumulator, cross-product accumulator)
    static_assert(TMEM_COLS >= 32u && TMEM_COLS <= 512u && (TMEM_COLS & (TMEM_COLS - 1u)) == 0u, "tensor-memory allocation must be a power of two in [32, 512]");
    __shared__ __align__(8) uint64_t full[NS];       // both operands of a stage have landed
    __shared__ __align__(8) uint64_t empty[NS];      // the MMAs that read a stage's buffers are done
    __shared__ __align__(8) uint64_t acc_full[2];    // every MMA of a 256-column block has landed in accumulator pair b
    __shared__ __align__(8) uint64_t acc_empty[2];   // the drain warps have read accumulator pair b
    __shared__ uint32_t tmem_slot;
    __shared__ volatile uint32_t fail;               // a bounded wait ran out
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;

    // token tile = blockIdx.x (fastest: the CTAs that share a weight tile run together and read it from L2), row tile = blockIdx.y
    const uint32_t rt = blockIdx.y;
    uint32_t ji = 0;
    for (uint32_t j = 1; j < A.njobs; ++j) if (rt >= A.job[j].tile0) ji = j;
    const TcJob &J = A.job[ji];
    const uint32_t row0 = (rt - J.tile0) * TC_M, t0 = blockIdx.x * (uint32_t)TN;
    const uint32_t nstage = A.ncols / TC_KS, nblk = A.ncols >> 8;
    const __half *xs_tile = A.xs + (size_t)blockIdx.x * nstage * (B_BUF / 2u);
    const uint8_t *wd_tile = A.wd + (size_t)rt * nstage * A_BUF;

    if (tid == 0) {
        fail = 0u;
        auto init = [](uint64_t *bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count)); };
        for (uint32_t i = 0; i < NS; ++i) { init(&full[i], 1u); init(&empty[i], 1u); }
        for (uint32_t i = 0; i < 2u; ++i) { init(&acc_full[i], 1u); init(&acc_empty[i], TCG_DRAIN_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    auto wait = [&](uint64_t *bar, uint32_t parity) -> bool {
        if (fail) return false;
        if (mbar_wait(smem_u32(bar), parity)) return true;
        fail = 1u;
        return false;
    };
    // for the roles that are far ahead of their producer: longer sleeps between polls, so that their spinning takes no issue
    // slots from the MMA thread
    auto wait_idle = [&](uint64_t *bar, uint32_t parity) -> bool {
        if (fail) return false;
        const uint32_t addr = smem_u32(bar);
        for (uint32_t i = 0; i < TC_SPIN_LIMIT / 8u; ++i) {
            uint32_t done;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                         : "=r"(done) : "r"(addr), "r"(parity) : "memory");
            if (done) return true;
            __nanosleep(256);
        }
        fail = 1u;
        return false;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            uint32_t issued = 0u;
            for (uint32_t s = 0; s < nstage; ++s) {
                const uint32_t j = s % NS;
                if (s >= NS && !wait_idle(&empty[j], ((s / NS) - 1u) & 1u)) break;
                const uint32_t bar = smem_u32(&full[j]), dst = smem_u32(smem + j * STAGE);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(STAGE) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             :: "r"(dst), "l"(wd_tile + (size_t)s * A_BUF), "r"(A_BUF), "r"(bar) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             :: "r"(dst + A_BUF), "l"(xs_tile + (size_t)s * (B_BUF / 2u)), "r"(B_BUF), "r"(bar) : "memory");
                issued = s + 1u;
            }
            // after a timeout elsewhere, copies that nobody waits for may still be writing into this CTA's shared memory
            if (fail) for (uint32_t s = issued >= NS ? issued - NS : 0u; s < issued; ++s) mbar_wait(smem_u32(&full[s % NS]), (s / NS) & 1u);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc = tc_idesc((uint32_t)TN), idesc2 = tc_idesc(2u * (uint32_t)TN);
            constexpr uint32_t A_LBO = TC_M * 16u, B_LBO = 2u * (uint32_t)TN * 16u, SBO = 128u;
            const uint64_t da0 = tc_smem_desc(0u, A_LBO, SBO), db0 = tc_smem_desc(0u, B_LBO, SBO);
            for (uint32_t s = 0; s < nstage; ++s) {
                const uint32_t j = s % NS, c = s >> 2;
                if (!wait(&full[j], (s / NS) & 1u)) break;
                if ((s & 3u) == 0u && c >= 2u && !wait(&acc_empty[c & 1u], ((c >> 1) - 1u) & 1u)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // Two MMAs per k-step: A_hi x [B_hi | B_lo] (N = 2 TN: the hi*hi sums land in the first TN accumulator
                // columns, hi*lo in the next TN) and A_lo x B_hi (N = TN, added to the cross-product columns).
                const uint32_t a_st = smem_u32(smem + j * STAGE);
                const uint32_t a_hi = a_st >> 4, a_lo = (a_st + TC_A_DIGIT) >> 4, b_st = (a_st + A_BUF) >> 4;
                const uint32_t d_main = tmem + (c & 1u) * 2u * (uint32_t)TN, d_cross = d_main + (uint32_t)TN;
#pragma unroll
                for (uint32_t kk = 0; kk < TC_KS / 16u; ++kk) {
                    const uint64_t dah = da0 + ((a_hi + kk * (2u * A_LBO >> 4)) & 0x3fffu), dal = da0 + ((a_lo + kk * (2u * A_LBO >> 4)) & 0x3fffu);
                    const uint64_t db = db0 + ((b_st + kk * (2u * B_LBO >> 4)) & 0x3fffu);
                    tc_mma(d_main, dah, db, idesc2, ((s & 3u) | kk) ? 1u : 0u);      // a block's first MMA overwrites its accumulators
                    tc_mma(d_cross, dal, db, idesc, 1u);
                }
                tc_commit(smem_u32(&empty[j]));
                if ((s & 3u) == 3u) tc_commit(smem_u32(&acc_full[c & 1u]));
            }
        }
    } else {
        // ------------------------------------------------------------------ accumulator drain and epilogue (256 threads)
        // warp w reads the tensor-memory lanes of its quarter (32 * (w % 4)) and PER of the TN token columns
        constexpr uint32_t PER = (uint32_t)TN / (TCG_DRAIN_WARPS / 4u);
        const uint32_t qlane = (warp & 3u) * 32u, c_begin = ((warp - 2u) >> 2) * PER;
        float acc[PER];
#pragma unroll
        for (uint32_t j = 0; j < PER; ++j) acc[j] = 0.f;
        bool ok = true;
        for (uint32_t blk = 0; blk < nblk && ok; ++blk) {
            ok = wait_idle(&acc_full[blk & 1u], (blk >> 1) & 1u);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t base = tmem + (qlane << 16) + (blk & 1u) * 2u * (uint32_t)TN + c_begin;
#pragma unroll
            for (uint32_t c = 0; c < PER; c += 8u) {
                uint32_t m[8], x[8];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                             : "=r"(m[0]), "=r"(m[1]), "=r"(m[2]), "=r"(m[3]), "=r"(m[4]), "=r"(m[5]), "=r"(m[6]), "=r"(m[7]) : "r"(base + c));
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                             : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]), "=r"(x[4]), "=r"(x[5]), "=r"(x[6]), "=r"(x[7]) : "r"(base + (uint32_t)TN + c));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[c + j] += __uint_as_float(m[j]) + __uint_as_float(x[j]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(&acc_empty[blk & 1u])) : "memory");
        }
        if (ok && !fail) {
            const uint32_t row = row0 + qlane + lane;
            const float w_inv = A.w_inv[rt];
#pragma unroll
            for (uint32_t j = 0; j < PER; ++j) {
                const uint32_t t = t0 + c_begin + j;
                if (t < A.ntok && row < J.nrows) J.out[(size_t)t * J.out_stride + row] = acc[j] * w_inv * A.x_inv[t];
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (fail && tid == 0) atomicExch(A.err, 1u);
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(TMEM_COLS) : "memory");
}

size_t tc_xs_halves(uint32_t ntok, uint32_t ncols, uint32_t tn) { return (size_t)((ntok + tn - 1u) / tn) * tn * ncols * 2u; }

// Token tile (MMA N) of a launch: the largest of 32 / 64 / 128 that the chunk fills, halved while the grid would leave
// most SMs idle (a CTA per 128 rows x tile; a smaller tile repeats the weight decode in more CTAs, which idle SMs absorb).
uint32_t tc_token_tile(uint32_t ntok, uint32_t row_tiles) {
    uint32_t tn = ntok <= 32u ? 32u : ntok <= 64u ? 64u : 128u;
    while (tn > 32u && row_tiles * ((ntok + tn - 1u) / tn) < 96u) tn >>= 1;
    return tn;
}
uint32_t tc_row_tiles(uint32_t nrows) { return (nrows + TC_M - 1u) / TC_M; }

static size_t tc_smem_bytes(uint32_t tn) {
    const uint32_t ns = tn >= 128u ? 3u : 4u;
    return (size_t)ns * (2u * (size_t)TC_A_DIGIT + 2u * (size_t)tn * TC_KS * 2u);
}
// bytes of the weight digit scratch (TcArgs::wd) and floats of TcArgs::w_inv for a launch of row_tiles tiles
size_t tc_wd_bytes(uint32_t row_tiles, uint32_t ncols) { return (size_t)row_tiles * TC_M * ncols * 4u; }

int launch_tc_prep_x(const float *x, const float *x2, uint32_t x_stride, uint32_t ntok, uint32_t ncols, uint32_t tn, __half *xs, float *x_inv, cudaStream_t s) {
    RC_REQUIRE(ncols % TC_KS == 0, "tc gemm: %u columns is not a multiple of %u", ncols, TC_KS);
    RC_REQUIRE(tn == 32u || tn == 64u || tn == 128u, "tc gemm: token tile %u is not 32, 64 or 128", tn);
    const uint32_t tiles = (ntok + tn - 1u) / tn;
    prof_begin("tc_prep_x", s);
    RC_LAUNCH((k_tc_prep_x), tiles * tn, 256, 0, s, x, x2, x_stride, ntok, ncols, tn, xs, x_inv);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

int launch_tc_gemm(TcArgs &A, uint32_t tn, const char *tag, cudaStream_t s) {
    RC_REQUIRE(tn == 32u || tn == 64u || tn == 128u, "tc gemm: token tile %u is not 32, 64 or 128", tn);
    RC_REQUIRE(A.njobs >= 1 && A.njobs <= TC_MAX_JOBS && A.ntok >= 1, "tc gemm: bad job count or no tokens");
    RC_REQUIRE(A.ncols % 256u == 0, "tc gemm: %u columns is not a multiple of 256", A.ncols);
    uint32_t tiles = 0;
    for (uint32_t j = 0; j < A.njobs; ++j) {
        RC_REQUIRE(rc_is_quant(A.job[j].type) || A.job[j].type == RC_F32, "tc gemm: matrix type %u is neither a block-quantised format nor fp32", A.job[j].type);
        A.job[j].tile0 = tiles;
        tiles += (A.job[j].nrows + TC_M - 1u) / TC_M;
    }
    RC_REQUIRE(A.wd && A.w_inv, "tc gemm: no scratch for the weight digits");
    A.iq2 = books_iq2(); A.iq3s = books_iq3s();
    prof_begin("tc_decode_w", s);
    RC_LAUNCH((k_tc_decode_w), dim3(tiles, A.ncols >> 8), TC_THREADS, 0, s, A);
    prof_end(s);
    RC_LAUNCHED();
    const dim3 grid((A.ntok + tn - 1u) / tn, tiles);
    RC_REQUIRE(tiles <= 65535u, "tc gemm: %u row tiles exceed the grid", tiles);
    const size_t smem = tc_smem_bytes(tn);
    prof_begin(tag, s);
#define RC_TC_LAUNCH(TN_) do { \
        RC_CUDA(cudaFuncSetAttribute(k_tc_gemm<TN_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        RC_LAUNCH((k_tc_gemm<TN_>), grid, TCG_THREADS, smem, s, A); } while (0)
    if (tn == 32u) RC_TC_LAUNCH(32); else if (tn == 64u) RC_TC_LAUNCH(64); else RC_TC_LAUNCH(128);
#undef RC_TC_LAUNCH
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

}  // namespace rc

using namespace rc;

// Host-buffer form for tests and one-off use: rows = nrows raw GGUF rows of `type`, x = [ntok][ncols] fp32,
// out = [ntok][nrows]. Same contract as redcuda_quant_matvec, computed by the tensor-core path.
extern "C" int redcuda_quant_matmul_tc(uint32_t type, const uint8_t *w, uint32_t nrows, uint32_t ncols, const float *x, uint32_t ntok, float *out) {
    if (!require_device() || !require_books(type)) return 0;
    RC_REQUIRE(w && x && out && nrows && ncols && ntok, "matmul_tc: null or empty argument");
    RC_REQUIRE(rc_is_quant(type), "matmul_tc: type %u is not a block-quantised format", type);
    RC_REQUIRE(ncols % 256u == 0, "matmul_tc: %u columns is not a multiple of 256", ncols);
    const uint64_t bytes = rc_matrix_bytes(type, nrows, ncols);
    const uint32_t tn = tc_token_tile(ntok, tc_row_tiles(nrows));
    DevMem raw, planar, xd, od, xs, xinv, err, wd, winv;
    if (!raw.alloc(bytes) || !planar.alloc(bytes) || !xd.alloc((size_t)ntok * ncols * 4u) || !od.alloc((size_t)ntok * nrows * 4u) ||
        !xs.alloc(tc_xs_halves(ntok, ncols, tn) * 2u) || !xinv.alloc((size_t)((ntok + tn - 1u) / tn) * tn * 4u) || !err.alloc(4u) ||
        !wd.alloc(tc_wd_bytes(tc_row_tiles(nrows), ncols)) || !winv.alloc((size_t)tc_row_tiles(nrows) * 4u)) return 0;
    cudaStream_t s = 0;
    if (!upload_matrix(type, nrows, ncols, w, false, planar.as<uint8_t>(), raw.as<uint8_t>(), s)) return 0;
    RC_CUDA(cudaMemcpyAsync(xd.p, x, (size_t)ntok * ncols * 4u, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemsetAsync(err.p, 0, 4u, s));
    if (!launch_tc_prep_x(xd.as<float>(), nullptr, ncols, ntok, ncols, tn, xs.as<__half>(), xinv.as<float>(), s)) return 0;
    TcArgs A{};
    A.njobs = 1; A.ncols = ncols; A.ntok = ntok; A.xs = xs.as<__half>(); A.x_inv = xinv.as<float>(); A.err = err.as<uint32_t>();
    A.wd = wd.as<uint8_t>(); A.w_inv = winv.as<float>();
    A.job[0] = TcJob{planar.as<uint8_t>(), (uint64_t)nrows * (ncols / 256u), type, nrows, od.as<float>(), nrows, 0u};
    if (!launch_tc_gemm(A, tn, "tc_gemm", s)) return 0;
    uint32_t flag = 0;
    RC_CUDA(cudaMemcpyAsync(&flag, err.p, 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaMemcpyAsync(out, od.p, (size_t)ntok * nrows * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    RC_REQUIRE(flag == 0u, "matmul_tc: a tensor-core stage never signalled completion (bounded wait ran out)");
    return 1;
}
