// Expert-grouped IQ2_XXS FFN matrices on the integer tensor-core path (mma.sync m16n8k32, s8 x s8 -> s32).
//
// Why: IQ2_XXS packs 2.06 bits per weight, so at HBM speed a B200 must decode ~25e12 weights/s. A CUDA-core GEMV
// spends >= 5 instructions per weight (grid byte -> float, sign, FMA per token) and tops out near a quarter of that;
// here a lane turns 8 weights into two operand registers with two shared-memory table lookups and six integer
// instructions, and every further token of the same expert costs one more MMA instead of 8 FMAs per weight.
//
// Arithmetic (exact integers, then fp32 scaling):
//   weight          w = d/8 * (2s+1) * (+-g),  g in {8,25,43} from the codebook, s the 4-bit scale of the 32-group
//   activation      x = sx * (16384*q2 + 128*q1 + q0), q_i balanced 7-bit digits (k_quant_act): 21-bit fixed point
//                   per row, error <= 2^-21 max|x| per element
//   per 32-group    one MMA per 8 columns gives sum(+-g * q) exactly in s32; multiplied by the integer (2s+1) and
//                   summed over the 8 groups of a block still in s32 (|.| < 2^25)
//   per block       converted to fp32 once and scaled by d/8; fp32 accumulation over the row's blocks only
//   per row,token   out = sx * (16384*o2 + 128*o1 + o0)
//
// Operand layout: lane (g = lane/4, t = lane%4) owns grid entry t (8 consecutive weights) of rows g and g+8 of the
// current 32-group, i.e. MMA k-slots {4t..4t+3, 16+4t..16+4t+3} stand for columns 8t..8t+7 of the group; the B
// fragment of a lane is then simply the 8 consecutive activation digits at 32*group + 8t of column g.
//
// Weights are streamed with cp.async (16 B per lane, fully coalesced: a warp copies whole 128-byte row segments)
// into per-warp double-buffered staging, rows padded to 144 B so that the 8-byte operand reads are conflict free.
// Both lookup tables are replicated 16x in shared memory (entry stride 128 B, replica = lane%16) for the same reason.
#include "redcuda_common.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_moe_mma.cuh"

namespace rc {

__device__ __align__(16) uint2 d_lut_grid[256];   // codebook magnitudes, 8 bytes per entry
__device__ __align__(16) uint2 d_lut_sign[128];   // 0xFF in every byte whose weight is negative (parity bit included)
static const uint2 *g_lut_grid_ptr[64] = {nullptr};
static const uint2 *g_lut_sign_ptr[64] = {nullptr};

int mma_set_luts(const uint8_t *iq2_grid_host) {
    uint2 hg[256], hs[128];
    for (int e = 0; e < 256; ++e) {
        uint32_t lo = 0, hi = 0;
        for (int j = 0; j < 4; ++j) { lo |= (uint32_t)iq2_grid_host[e * 8 + j] << (8 * j); hi |= (uint32_t)iq2_grid_host[e * 8 + 4 + j] << (8 * j); }
        hg[e] = make_uint2(lo, hi);
    }
    for (uint32_t s7 = 0; s7 < 128; ++s7) {
        const uint32_t s8 = rc_sign8(s7);
        uint32_t lo = 0, hi = 0;
        for (int j = 0; j < 4; ++j) { if ((s8 >> j) & 1u) lo |= 0xFFu << (8 * j); if ((s8 >> (j + 4)) & 1u) hi |= 0xFFu << (8 * j); }
        hs[s7] = make_uint2(lo, hi);
    }
    int dev = 0;
    RC_CUDA(cudaGetDevice(&dev));
    RC_CUDA(cudaMemcpyToSymbol(d_lut_grid, hg, sizeof(hg)));
    RC_CUDA(cudaMemcpyToSymbol(d_lut_sign, hs, sizeof(hs)));
    void *pg = nullptr, *ps = nullptr;
    RC_CUDA(cudaGetSymbolAddress(&pg, d_lut_grid));
    RC_CUDA(cudaGetSymbolAddress(&ps, d_lut_sign));
    g_lut_grid_ptr[dev & 63] = (const uint2 *)pg;
    g_lut_sign_ptr[dev & 63] = (const uint2 *)ps;
    return 1;
}

// ---- activation rows -> three balanced 7-bit digit planes + one fp32 scale per row ----
// grid = rows, block = 256. xq[row][3][ncols] (digit 0 = least significant), sx[row].
__global__ void __launch_bounds__(256) k_quant_act(const float *__restrict__ x, uint32_t x_stride, uint32_t ncols,
                                                   int8_t *__restrict__ xq, float *__restrict__ sx) {
    __shared__ float red[8];
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const float *xr = x + (size_t)row * x_stride;
    float mx = 0.f;
    for (uint32_t k = tid * 4u; k < ncols; k += 1024u) {
        const float4 v = *reinterpret_cast<const float4 *>(xr + k);
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((tid & 31u) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
    const float QMAX = 1040000.0f;
    const float scale = (mx > 0.f && mx < INFINITY) ? mx / QMAX : 1.0f;
    const float inv = 1.0f / scale;
    if (tid == 0) sx[row] = scale;
    int8_t *q = xq + (size_t)row * 3u * ncols;
    for (uint32_t k = tid * 4u; k < ncols; k += 1024u) {
        const float4 v = *reinterpret_cast<const float4 *>(xr + k);
        const float f[4] = {v.x, v.y, v.z, v.w};
        uint32_t p0 = 0, p1 = 0, p2 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int iv = __float2int_rn(fminf(fmaxf(f[i] * inv, -QMAX), QMAX));
            const int d0 = ((iv + 64) & 127) - 64; iv = (iv - d0) >> 7;
            const int d1 = ((iv + 64) & 127) - 64; iv = (iv - d1) >> 7;
            p0 |= (uint32_t)(d0 & 255) << (8 * i); p1 |= (uint32_t)(d1 & 255) << (8 * i); p2 |= (uint32_t)(iv & 255) << (8 * i);
        }
        *reinterpret_cast<uint32_t *>(q + k) = p0;
        *reinterpret_cast<uint32_t *>(q + ncols + k) = p1;
        *reinterpret_cast<uint32_t *>(q + 2u * ncols + k) = p2;
    }
}

int launch_quant_act(const float *x, uint32_t x_stride, uint32_t rows, uint32_t ncols, int8_t *xq, float *sx, cudaStream_t s) {
    RC_REQUIRE(ncols % 16u == 0, "quant_act: %u columns is not a multiple of 16", ncols);
    if (!rows) return 1;
    prof_begin("moe_quant_act", s);
    k_quant_act<<<rows, 256, 0, s>>>(x, x_stride, ncols, xq, sx);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

// ---- small PTX wrappers ----
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gsrc));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void mma_s8_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// shared-memory geometry
#define MMA_ROW_PITCH 144u                 // staged row segment: 128 B of qs (two blocks) + 16 B pad
#define MMA_STAGES 2u
#define MMA_CHUNK_COLS 512u                // columns per staged unit (two 256-blocks)
__host__ __device__ __forceinline__ uint32_t mma_b_pitch(uint32_t ncols) { return ncols + 32u; }   // == 32 (mod 128)

// One warp: 16 rows x one 512-column chunk of `NMAT` matrices against NTILE*8 activation columns. Each of the two
// 256-blocks of the chunk is closed inside (integer accumulation over its 8 groups, then one fp32 scaling), so only
// the fp32 accumulators out[m][tile][4] live across calls.
template <int NMAT, int NTILE>
__device__ __forceinline__ void mma_unit(const uint8_t *stage, const float (&dsc)[NMAT][2][2], const int8_t *Bs, uint32_t bpitch, uint32_t kbase,
                                         const uint8_t *lutg, const uint8_t *luts, uint32_t lane, float (&out)[NMAT][NTILE][4]) {
    const uint32_t g = lane >> 2, t = lane & 3u, rep8 = (lane & 15u) * 8u;
    const uint32_t sel = 0x4440u + t, sh7 = 7u * t;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
        int blk[NMAT][NTILE][4];
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
#pragma unroll
            for (int n = 0; n < NTILE; ++n) { blk[m][n][0] = blk[m][n][1] = blk[m][n][2] = blk[m][n][3] = 0; }
#pragma unroll 2
        for (int kg = 0; kg < 8; ++kg) {
            const uint32_t goff = (uint32_t)(b * 8 + kg) * 8u;
            uint32_t a[NMAT][4];
            int sc[NMAT][2];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint2 q = *reinterpret_cast<const uint2 *>(stage + (uint32_t)(m * 16 + h * 8 + g) * MMA_ROW_PITCH + goff);
                    const uint32_t gi = __byte_perm(q.x, 0u, sel);
                    const uint32_t s7 = (q.y >> sh7) & 127u;
                    const uint2 P = *reinterpret_cast<const uint2 *>(lutg + gi * 128u + rep8);
                    const uint2 M = *reinterpret_cast<const uint2 *>(luts + s7 * 128u + rep8);
                    a[m][h] = (P.x ^ M.x) + (M.x & 0x01010101u);         // bytes: +g or -g (no carry between bytes: g >= 1)
                    a[m][2 + h] = (P.y ^ M.y) + (M.y & 0x01010101u);
                    sc[m][h] = (int)(2u * (q.y >> 28) + 1u);
                }
            }
#pragma unroll
            for (int n = 0; n < NTILE; ++n) {
                const uint2 bf = *reinterpret_cast<const uint2 *>(Bs + (uint32_t)(n * 8 + g) * bpitch + kbase + (uint32_t)(b * 8 + kg) * 32u + 8u * t);
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                    int d[4];
                    mma_s8_k32(d, a[m][0], a[m][1], a[m][2], a[m][3], bf.x, bf.y);
                    blk[m][n][0] += sc[m][0] * d[0]; blk[m][n][1] += sc[m][0] * d[1];
                    blk[m][n][2] += sc[m][1] * d[2]; blk[m][n][3] += sc[m][1] * d[3];
                }
            }
        }
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
#pragma unroll
            for (int n = 0; n < NTILE; ++n) {
                out[m][n][0] += dsc[m][b][0] * (float)blk[m][n][0]; out[m][n][1] += dsc[m][b][0] * (float)blk[m][n][1];
                out[m][n][2] += dsc[m][b][1] * (float)blk[m][n][2]; out[m][n][3] += dsc[m][b][1] * (float)blk[m][n][3];
            }
    }
}

// Block = 8 warps = R row tiles x S column splits (R*S == 8). Warp (r, ks) works on `tiles_per_warp` 16-row tiles
// and on the 512-column chunks c with c % S == ks. grid = (row-tile groups, experts that received a pair).
template <int NMAT, int NTILE>
__global__ void __launch_bounds__(256, 1) k_moe_mma(const __grid_constant__ MmaArgs A) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr uint32_t NCOL = NTILE * 8u, TOK = NCOL / 3u;
    // one work item = up to TOK pairs of one expert (k_group_pairs cuts every expert's pairs into such items, so that
    // all blocks carry the same amount of work whatever the routing skew)
    if (blockIdx.y >= *A.n_items) return;
    const uint32_t u = A.item_u[blockIdx.y], p0 = A.item_p0[blockIdx.y];
    const uint32_t e = A.uexp[u] - A.expert_begin, pe = A.ustart[u + 1u];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t S = A.S, R = 8u / S, r = warp / S, ks = warp % S;
    const uint32_t bpr = A.ncols >> 8, nchunks = A.ncols / MMA_CHUNK_COLS, bpitch = mma_b_pitch(A.ncols);
    // carve shared memory
    uint8_t *lutg = smem;                                   // 256 x 128 B
    uint8_t *luts = lutg + 256u * 128u;                     // 128 x 128 B
    int8_t *Bs = reinterpret_cast<int8_t *>(luts + 128u * 128u);                       // NCOL x bpitch
    float *sxs = reinterpret_cast<float *>(Bs + (size_t)NCOL * bpitch);                // TOK (+pad) floats
    uint8_t *stage0 = reinterpret_cast<uint8_t *>(sxs + 16);                           // 8 warps x STAGES x NMAT*16 rows x pitch
    const uint32_t stage_bytes = NMAT * 16u * MMA_ROW_PITCH;
    float *scratch0 = reinterpret_cast<float *>(stage0 + 8u * MMA_STAGES * stage_bytes);   // 8 warps x NMAT x 16 x NCOL floats
    uint8_t *my_stage = stage0 + warp * MMA_STAGES * stage_bytes;
    float *my_scratch = scratch0 + (size_t)warp * NMAT * 16u * NCOL;

    for (uint32_t i = tid; i < 256u * 16u; i += 256u) reinterpret_cast<uint2 *>(lutg)[i] = A.lut_grid[i >> 4];
    for (uint32_t i = tid; i < 128u * 16u; i += 256u) reinterpret_cast<uint2 *>(luts)[i] = A.lut_sign[i >> 4];

    const uint8_t *w[2] = {A.w0 + (size_t)e * A.mat_bytes, A.w1 ? A.w1 + (size_t)e * A.mat_bytes : nullptr};
    const uint32_t tile_first = (blockIdx.x * R + r) * A.tiles_per_warp;            // in units of 16 rows
    uint32_t my_chunks = 0;
    for (uint32_t c = ks; c < nchunks; c += S) ++my_chunks;
    const uint32_t ntile_rows = A.nrows >> 4;
    uint32_t my_tiles = 0;
    for (uint32_t i = 0; i < A.tiles_per_warp; ++i) if (tile_first + i < ntile_rows) ++my_tiles;
    const uint32_t nunits = my_tiles * my_chunks;

    {
        const uint32_t nt = min(TOK, pe - p0);
        // ---- stage the activation digits of pairs [p0, p0 + nt): column = 3 * token + digit
        {
            const uint32_t v16 = A.ncols >> 4;
            for (uint32_t i = tid; i < NCOL * v16; i += 256u) {
                const uint32_t col = i / v16, k = (i - col * v16) << 4, tk = col / 3u, dg = col - tk * 3u;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (tk < nt) {
                    const size_t xr = A.sorted[p0 + tk] / A.x_div;
                    v = *reinterpret_cast<const uint4 *>(A.xq + (xr * 3u + dg) * A.ncols + k);
                }
                *reinterpret_cast<uint4 *>(Bs + (size_t)col * bpitch + k) = v;
            }
            if (tid < TOK) sxs[tid] = tid < nt ? A.sx[A.sorted[p0 + tid] / A.x_div] : 0.f;
        }
        __syncthreads();

        auto issue = [&](uint32_t unit, uint32_t buf) {
            const uint32_t ti = unit / my_chunks, c = ks + (unit - ti * my_chunks) * S;
            const uint32_t row0 = (tile_first + ti) << 4;
            uint8_t *dst = my_stage + buf * stage_bytes;
#pragma unroll
            for (uint32_t i = 0; i < NMAT * 4u; ++i) {
                const uint32_t p = lane + 32u * i, rr = p >> 3, piece = p & 7u, m = rr >> 4, row = row0 + (rr & 15u);
                cp_async16(dst + rr * MMA_ROW_PITCH + piece * 16u, w[m] + ((size_t)row * bpr + c * 2u) * 64u + piece * 16u);
            }
        };

        float out[NMAT][NTILE][4];
        if (nunits) { issue(0u, 0u); }
        cp_async_commit();
        for (uint32_t unit = 0; unit < nunits; ++unit) {
            const uint32_t ti = unit / my_chunks, ci = unit - ti * my_chunks, c = ks + ci * S;
            const uint32_t row0 = (tile_first + ti) << 4;
            if (unit + 1u < nunits) issue(unit + 1u, (unit + 1u) & 1u);
            cp_async_commit();
            // block scales d/8 of rows g, g+8 for the two blocks of this chunk (plain loads, 2 B each)
            float dsc[NMAT][2][2];
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
                for (int b = 0; b < 2; ++b)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const size_t bi = (size_t)(row0 + h * 8u + g) * bpr + c * 2u + b;
                        dsc[m][b][h] = 0.125f * __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(w[m] + A.nb * 64u) + bi)));
                    }
            if (ci == 0u) {
#pragma unroll
                for (int m = 0; m < NMAT; ++m)
#pragma unroll
                    for (int n = 0; n < NTILE; ++n) { out[m][n][0] = out[m][n][1] = out[m][n][2] = out[m][n][3] = 0.f; }
            }
            cp_async_wait<1>();
            __syncwarp();
            mma_unit<NMAT, NTILE>(my_stage + (unit & 1u) * stage_bytes, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, out);
            __syncwarp();
            if (ci + 1u == my_chunks) {
                // ---- tile finished for this warp: fragments -> scratch[m][row][col]
#pragma unroll
                for (int m = 0; m < NMAT; ++m)
#pragma unroll
                    for (int n = 0; n < NTILE; ++n) {
                        float *sp = my_scratch + (size_t)m * 16u * NCOL + n * 8u + 2u * t;
                        sp[(size_t)g * NCOL] = out[m][n][0]; sp[(size_t)g * NCOL + 1u] = out[m][n][1];
                        sp[(size_t)(g + 8u) * NCOL] = out[m][n][2]; sp[(size_t)(g + 8u) * NCOL + 1u] = out[m][n][3];
                    }
                if (S > 1u) __syncthreads(); else __syncwarp();       // S > 1 implies one tile per warp: every warp gets here once
                if (ks == 0u) {
                    for (uint32_t idx = lane; idx < 16u * nt; idx += 32u) {
                        const uint32_t row = idx & 15u, tk = idx >> 4;
                        float val[NMAT];
#pragma unroll
                        for (int m = 0; m < NMAT; ++m) {
                            float o0 = 0.f, o1 = 0.f, o2 = 0.f;
                            for (uint32_t s = 0; s < S; ++s) {
                                const float *sp = scratch0 + ((size_t)(warp + s) * NMAT + m) * 16u * NCOL + (size_t)row * NCOL + 3u * tk;
                                o0 += sp[0]; o1 += sp[1]; o2 += sp[2];
                            }
                            val[m] = sxs[tk] * (16384.f * o2 + 128.f * o1 + o0);
                        }
                        const uint32_t p = A.sorted[p0 + tk];
                        float v = val[0];
                        if (NMAT == 2) { const float gte = val[0]; v = (gte / (1.0f + expf(-gte))) * val[NMAT - 1]; }
                        A.out[(size_t)p * A.out_stride + row0 + row] = v;
                    }
                }
                if (S > 1u) __syncthreads(); else __syncwarp();
            }
        }
        cp_async_wait<0>();
        if (S > 1u && nunits == 0u) { __syncthreads(); __syncthreads(); }   // keep barrier counts equal for warps without work
    }
}

size_t mma_smem_bytes(uint32_t nmat, uint32_t ntile, uint32_t ncols) {
    const size_t ncol = ntile * 8u;
    return 256u * 128u + 128u * 128u + ncol * mma_b_pitch(ncols) + 64u + 8u * MMA_STAGES * nmat * 16u * MMA_ROW_PITCH + 8u * nmat * 16u * ncol * 4u;
}

int launch_moe_mma(MmaArgs &A, uint32_t groups, bool few_tokens, cudaStream_t s) {
    int dev = 0;
    RC_CUDA(cudaGetDevice(&dev));
    A.lut_grid = g_lut_grid_ptr[dev & 63];
    A.lut_sign = g_lut_sign_ptr[dev & 63];
    RC_REQUIRE(A.lut_grid && A.lut_sign, "IQ2_XXS tensor-core tables not set on device %d: call redcuda_set_codebooks first", dev);
    RC_REQUIRE(A.ncols % MMA_CHUNK_COLS == 0 && A.nrows % 16u == 0, "moe mma: matrix %ux%u is not a multiple of 16 rows x 512 columns", A.nrows, A.ncols);
    const uint32_t nmat = A.w1 ? 2u : 1u, nchunks = A.ncols / MMA_CHUNK_COLS, ntile_rows = A.nrows / 16u;
    // Single-token decode: few row tiles in total, so the wide matrices are also split along the columns (S warps
    // share a row tile); batches: about four blocks per expert so that the tables and the activation tile of a block
    // are staged once per 2^17..2^19 weights.
    uint32_t S = 1u, tpw = 1u;
    if (few_tokens) {
        while (S < 8u && S * 2u <= nchunks && nchunks % (S * 2u) == 0 && (uint64_t)ntile_rows * groups * S < 148u * 8u) S <<= 1;
    } else {
        while (tpw < 8u && ntile_rows / (8u * tpw * 2u) >= 4u && ntile_rows % (8u * tpw * 2u) == 0) tpw <<= 1;
    }
    const uint32_t R = 8u / S;
    A.S = S; A.tiles_per_warp = tpw;
    const dim3 grid((ntile_rows + R * tpw - 1u) / (R * tpw), groups);
    const uint32_t ntile = few_tokens ? 1u : 3u;
    const size_t smem = mma_smem_bytes(nmat, ntile, A.ncols);
    RC_REQUIRE(smem <= 227u * 1024u, "moe mma: %zu bytes of shared memory needed for %u columns", smem, A.ncols);
    prof_begin(nmat == 2u ? "moe_gateup" : "moe_down", s);
#define RC_MMA_LAUNCH(NM, NT) do { \
        RC_CUDA(cudaFuncSetAttribute(k_moe_mma<NM, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        k_moe_mma<NM, NT><<<grid, 256, smem, s>>>(A); } while (0)
    if (nmat == 2u) { if (ntile == 1u) RC_MMA_LAUNCH(2, 1); else RC_MMA_LAUNCH(2, 3); }
    else { if (ntile == 1u) RC_MMA_LAUNCH(1, 1); else RC_MMA_LAUNCH(1, 3); }
#undef RC_MMA_LAUNCH
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

}  // namespace rc
