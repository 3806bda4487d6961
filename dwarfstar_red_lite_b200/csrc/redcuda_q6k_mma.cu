// Q6_K matrix x many activation rows on the integer tensor-core path (mma.sync m16n8k16, s8 x s8 -> s32).
//
// Used when one Q6_K matrix meets a batch of tokens (the shared expert of a ragged decode batch): the CUDA-core GEMV
// re-decodes the weights for every four tokens, whereas here a lane rebuilds two operand registers (4 weights of rows
// g and g+8) per 16-column scale group with ~14 integer instructions and then serves 8 tokens per three MMAs.
//
//   weight      w = d * sc * q,  q = 6-bit value - 32 in [-32, 31] (one int8), sc the int8 scale of the 16-group
//   activation  x = sx * (65536*q2 + 256*q1 + q0), balanced 8-bit digits (k_quant_act)
//   per group   the three digit products of a (row, token) are exact s32 (|.| <= 2^16); digits 1 and 2 are recombined
//               exactly in s32 (|.| < 2^25), the result and digit 0 converted to fp32 and accumulated with the fp32
//               scale d*sc
//
// Block = 8 warps = MS matrices x KS column splits x TGB groups of 8 tokens, for one tile of 16 rows; partial sums meet
// in shared memory, where the epilogue (plain store or SiLU(gate)*up) is applied.
#define RC_PDL_DEFAULT 0
#include "redcuda_common.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_moe_mma.cuh"

namespace rc {

// z: a quad of registers holding zero for the whole kernel (a literal 0 costs four moves in front of every MMA)
__device__ __forceinline__ void mma_s8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, const int (&z)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};\n"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(z[0]), "r"(z[1]), "r"(z[2]), "r"(z[3]));
}

struct Q6Args {
    const uint8_t *w[2];
    uint64_t nb;
    uint32_t nrows, ncols, ntok;
    const int8_t *xq; const float *sx;      // digits [ntok][3][ncols], scale per token
    float *out; uint32_t out_stride;        // out[token * out_stride + row]
    uint32_t pair_silu;                     // 1: out = SiLU(w[0].x) * (w[1].x)
    uint32_t MS, KS;                        // matrices and column splits per block (8 % (MS*KS) == 0)
    uint32_t bits; float dw1;               // digit width and 2^bits
};

__global__ void __launch_bounds__(256) k_q6k_mma(const __grid_constant__ Q6Args A) {
    pdl_prologue();
    __shared__ float part[8][16][8];        // per warp: 16 rows x 8 tokens
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t MS = A.MS, KS = A.KS, TGB = 8u / (MS * KS);
    const uint32_t mat = warp % MS, ks = (warp / MS) % KS, tgl = warp / (MS * KS);
    const uint32_t tg = blockIdx.y * TGB + tgl;                 // group of 8 tokens
    const uint32_t row0 = blockIdx.x * 16u, bpr = A.ncols >> 8, nsteps = A.ncols >> 4;
    const uint32_t s_begin = ks * (nsteps / KS), s_end = s_begin + nsteps / KS;
    const uint8_t *base = A.w[mat];
    const uint64_t nb = A.nb;
    const uint32_t tok = tg * 8u + g;                           // this lane's B column
    const bool tok_ok = tok < A.ntok;
    const int8_t *xrow = A.xq + (size_t)(tok_ok ? tok : 0u) * 3u * A.ncols + 4u * t;
    float out[4] = {0.f, 0.f, 0.f, 0.f};
    int z[4];
    asm volatile("mov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;" : "=r"(z[0]), "=r"(z[1]), "=r"(z[2]), "=r"(z[3]));
    if (tg * 8u < A.ntok) {
#pragma unroll 8
        for (uint32_t s = s_begin; s < s_end; ++s) {
            const uint32_t b = s >> 4, grp = s & 15u, h = grp >> 3, q = (grp >> 1) & 3u, i = grp & 1u;
            uint32_t a[2];
            float scl[2];
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
                const uint64_t blk = (uint64_t)(row0 + hr * 8u + g) * bpr + b;
                const uint32_t ql = __ldg(reinterpret_cast<const uint32_t *>(base + blk * 128u + 64u * h + 32u * (q & 1u) + 16u * i + 4u * t));
                const uint32_t qh = __ldg(reinterpret_cast<const uint32_t *>(base + rc_q6_qh(nb) + blk * 64u + 32u * h + 16u * i + 4u * t));
                const int sc = (int)(signed char)__ldg(base + rc_q6_sc(nb) + blk * 16u + grp);
                const float d = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(base + rc_q6_d(nb)) + blk)));
                const uint32_t v = ((ql >> (4u * (q >> 1))) & 0x0F0F0F0Fu) | (((qh >> (2u * q)) & 0x03030303u) << 4);
                const uint32_t u = v ^ 0x20202020u;            // 6-bit two's complement of (value - 32)
                a[hr] = u + (u & 0x20202020u) * 6u;             // sign-extend every byte to 8 bits (bits 6,7 were clear: no carry)
                scl[hr] = d * (float)sc;
            }
            int d0[4], d1[4], d2[4];
            const uint32_t b0 = tok_ok ? __ldg(reinterpret_cast<const uint32_t *>(xrow + 16u * s)) : 0u;
            const uint32_t b1 = tok_ok ? __ldg(reinterpret_cast<const uint32_t *>(xrow + A.ncols + 16u * s)) : 0u;
            const uint32_t b2 = tok_ok ? __ldg(reinterpret_cast<const uint32_t *>(xrow + 2u * A.ncols + 16u * s)) : 0u;
            mma_s8_k16(d0, a[0], a[1], b0, z);
            mma_s8_k16(d1, a[0], a[1], b1, z);
            mma_s8_k16(d2, a[0], a[1], b2, z);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int hi = d1[c] + (d2[c] << A.bits);                 // 8-bit digits: the full recombination would leave s32
                out[c] += scl[c >> 1] * fmaf(A.dw1, (float)hi, (float)d0[c]);
            }
        }
        // accumulator columns 2t, 2t+1 of this lane are tokens tg*8 + 2t, +1
        const uint32_t tk0 = tg * 8u + 2u * t;
        const float s0 = tk0 < A.ntok ? A.sx[tk0] : 0.f, s1 = tk0 + 1u < A.ntok ? A.sx[tk0 + 1u] : 0.f;
        out[0] *= s0; out[1] *= s1; out[2] *= s0; out[3] *= s1;
    }
    part[warp][g][2u * t] = out[0]; part[warp][g][2u * t + 1u] = out[1];
    part[warp][g + 8u][2u * t] = out[2]; part[warp][g + 8u][2u * t + 1u] = out[3];
    __syncthreads();
    // epilogue: TGB token groups x 16 rows x 8 tokens
    for (uint32_t idx = tid; idx < TGB * 128u; idx += 256u) {
        const uint32_t tl = idx >> 7, row = (idx >> 3) & 15u, c = idx & 7u;
        const uint32_t tkn = (blockIdx.y * TGB + tl) * 8u + c;
        if (tkn >= A.ntok || row0 + row >= A.nrows) continue;
        float val[2] = {0.f, 0.f};
        for (uint32_t m = 0; m < MS; ++m)
            for (uint32_t k = 0; k < KS; ++k) val[m] += part[(tl * KS + k) * MS + m][row][c];
        float v = val[0];
        if (A.pair_silu) v = (val[0] / (1.0f + expf(-val[0]))) * val[1];
        A.out[(size_t)tkn * A.out_stride + row0 + row] = v;
    }
}

// out[t][r] = W0[r].x[t]   or   SiLU(W0[r].x[t]) * (W1[r].x[t]) for Q6_K matrices and activations already in digit form.
int launch_q6k_mma(const uint8_t *w0, const uint8_t *w1, uint64_t nb, uint32_t nrows, uint32_t ncols, uint32_t ntok,
                   const int8_t *xq, const float *sx, float *out, uint32_t out_stride, const char *tag, cudaStream_t s) {
    RC_REQUIRE(nrows % 16u == 0 && ncols % 256u == 0, "q6k mma: matrix %ux%u must be a multiple of 16 rows x 256 columns", nrows, ncols);
    if (!ntok) return 1;
    Q6Args A{};
    A.w[0] = w0; A.w[1] = w1 ? w1 : w0; A.nb = nb; A.nrows = nrows; A.ncols = ncols; A.ntok = ntok; A.xq = xq; A.sx = sx;
    A.out = out; A.out_stride = out_stride; A.pair_silu = w1 ? 1u : 0u;
    A.MS = w1 ? 2u : 1u;
    A.bits = act_digit_bits(); A.dw1 = (float)(1u << A.bits);
    const uint32_t nsteps = ncols / 16u, tgroups = (ntok + 7u) / 8u, tiles = nrows / 16u;
    // column splits while the launch would leave SMs idle and every split keeps >= 16 steps
    uint32_t KS = 1u;
    while (A.MS * KS * 2u <= 8u && (nsteps / (KS * 2u)) >= 16u && nsteps % (KS * 2u) == 0 &&
           (uint64_t)tiles * ((tgroups + 8u / (A.MS * KS) - 1u) / (8u / (A.MS * KS))) < 148u * 2u) KS <<= 1;
    A.KS = KS;
    const uint32_t TGB = 8u / (A.MS * KS);
    const dim3 grid(tiles, (tgroups + TGB - 1u) / TGB);
    prof_begin(tag, s);
    RC_LAUNCH((k_q6k_mma), grid, 256, 0, s, A);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

}  // namespace rc
