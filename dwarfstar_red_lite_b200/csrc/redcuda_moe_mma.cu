// Expert-grouped IQ2_XXS FFN matrices on the integer tensor-core path (mma.sync m16n8k32, s8 x s8 -> s32).
//
// Why: IQ2_XXS packs 2.06 bits per weight, so at HBM speed a B200 must decode ~25e12 weights/s. A CUDA-core GEMV
// spends >= 5 instructions per weight (grid byte -> float, sign, FMA per token) and tops out near a quarter of that;
// here a lane turns 8 weights into two operand registers with two shared-memory table lookups and six integer
// instructions, and every further token of the same expert costs one more MMA instead of 8 FMAs per weight.
//
// Arithmetic (exact integers, then fp32 scaling):
//   weight          w = d/8 * (2s+1) * (+-g),  g in {8,25,43} from the codebook, s the 4-bit scale of the 32-group
//   activation      x = sx * (65536*q2 + 256*q1 + q0), q_i balanced 8-bit digits (k_quant_act): 24-bit fixed point
//                   per row, error <= 2^-24 max|x| per element (an fp32 mantissa for the row's largest elements)
//   per 32-group    one MMA per 8 columns gives sum(+-g * q) exactly in s32; multiplied by the integer (2s+1) and
//                   summed over the 8 groups of a block still in s32 (|.| < 2^25)
//   per block       converted to fp32 once and scaled by d/8; fp32 accumulation over the row's blocks only
//   per row,token   out = sx * (65536*o2 + 256*o1 + o0)
//
// Operand layout: lane (g = lane/4, t = lane%4) owns grid entry t (8 consecutive weights) of rows g and g+8 of the
// current 32-group, i.e. MMA k-slots {4t..4t+3, 16+4t..16+4t+3} stand for columns 8t..8t+7 of the group; the B
// fragment of a lane is then simply the 8 consecutive activation digits at 32*group + 8t of column g.
//
// Weights are streamed with cp.async (16 B per lane; a warp copies the 64-byte block segments of its 16 or 32 rows) into
// per-warp staging, three 256-column units in flight, rows padded to 80 B so that the 8-byte operand reads are conflict
// free. The activation digits of a work item (<= 8 pairs, or <= 16 when experts see many pairs each) sit in shared memory,
// column-major with a pitch that spreads the 8 columns of a tile over the banks.
// Both lookup tables are replicated 8x in shared memory (magnitudes: 8 copies of 8 B, entry stride 64 B; signs: 8 copies
// of 16 B holding the byte mask and its +1 carry term, entry stride 128 B; replica = lane % 8), since a lane's entry index
// is data dependent.
// Kernels: k_moe_mma<NMAT, NTILE> (8 warps; NMAT = 2 fuses gate and up with SiLU * mul, used for one or two tokens;
// NMAT = 1 is the down projection) and k_moe_gateup16<NTILE> (16 warps: gate warps + up warps, used for batches).
#define RC_PDL_DEFAULT 0
#include "redcuda_common.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_moe_mma.cuh"

#include <stdlib.h>

namespace rc {

__device__ __align__(16) uint2 d_lut_grid[256];   // codebook magnitudes, 8 bytes per entry
__device__ __align__(16) uint4 d_lut_sign[128];   // x,y: 0xFF in every byte whose weight is negative (parity bit included); z,w: 0x01 there
static const uint2 *g_lut_grid_ptr[64] = {nullptr};
static const uint4 *g_lut_sign_ptr[64] = {nullptr};

int mma_set_luts(const uint8_t *iq2_grid_host) {
    uint2 hg[256];
    uint4 hs[128];
    for (int e = 0; e < 256; ++e) {
        uint32_t lo = 0, hi = 0;
        for (int j = 0; j < 4; ++j) { lo |= (uint32_t)iq2_grid_host[e * 8 + j] << (8 * j); hi |= (uint32_t)iq2_grid_host[e * 8 + 4 + j] << (8 * j); }
        hg[e] = make_uint2(lo, hi);
    }
    for (uint32_t s7 = 0; s7 < 128; ++s7) {
        const uint32_t s8 = rc_sign8(s7);
        uint32_t lo = 0, hi = 0;
        for (int j = 0; j < 4; ++j) { if ((s8 >> j) & 1u) lo |= 0xFFu << (8 * j); if ((s8 >> (j + 4)) & 1u) hi |= 0xFFu << (8 * j); }
        hs[s7] = make_uint4(lo, hi, lo & 0x01010101u, hi & 0x01010101u);
    }
    int dev = 0;
    RC_CUDA(cudaGetDevice(&dev));
    RC_CUDA(cudaMemcpyToSymbol(d_lut_grid, hg, sizeof(hg)));
    RC_CUDA(cudaMemcpyToSymbol(d_lut_sign, hs, sizeof(hs)));
    void *pg = nullptr, *ps = nullptr;
    RC_CUDA(cudaGetSymbolAddress(&pg, d_lut_grid));
    RC_CUDA(cudaGetSymbolAddress(&ps, d_lut_sign));
    g_lut_grid_ptr[dev & 63] = (const uint2 *)pg;
    g_lut_sign_ptr[dev & 63] = (const uint4 *)ps;
    return 1;
}

uint32_t act_digit_bits() {
    static const uint32_t bits = (getenv("RC_ACT_BITS") && atoi(getenv("RC_ACT_BITS")) == 7) ? 7u : 8u;
    return bits;
}

// ---- activation rows -> three balanced digit planes of `bits` bits + one fp32 scale per row ----
// grid = rows, block = 256. xq[row][3][ncols] (digit 0 = least significant), sx[row]. Digits lie in [-2^(bits-1), 2^(bits-1)).
__global__ void __launch_bounds__(256) k_quant_act(const float *__restrict__ x, uint32_t x_stride, uint32_t ncols,
                                                   int8_t *__restrict__ xq, float *__restrict__ sx, uint32_t bits) {
    pdl_prologue();
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
    const float QMAX = act_qmax(bits);
    const float scale = act_scale(mx, QMAX);
    const float inv = 1.0f / scale;
    if (tid == 0) sx[row] = scale;
    int8_t *q = xq + (size_t)row * 3u * ncols;
    for (uint32_t k = tid * 4u; k < ncols; k += 1024u) {
        const float4 v = *reinterpret_cast<const float4 *>(xr + k);
        const float f[4] = {v.x, v.y, v.z, v.w};
        uint32_t p0 = 0, p1 = 0, p2 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int d0, d1, d2;
            act_digits(f[i], inv, QMAX, bits, d0, d1, d2);
            p0 |= (uint32_t)(d0 & 255) << (8 * i); p1 |= (uint32_t)(d1 & 255) << (8 * i); p2 |= (uint32_t)(d2 & 255) << (8 * i);
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
    RC_LAUNCH((k_quant_act), rows, 256, 0, s, x, x_stride, ncols, xq, sx, act_digit_bits());
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

// The accumulator input is a quad of registers that hold zero for the whole kernel (zero_quad): given a literal 0 the
// compiler writes four moves in front of every MMA.
__device__ __forceinline__ void mma_s8_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, const int (&z)[4]) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z[0]), "r"(z[1]), "r"(z[2]), "r"(z[3]));
}
__device__ __forceinline__ void zero_quad(int (&z)[4]) {
    asm volatile("mov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;" : "=r"(z[0]), "=r"(z[1]), "=r"(z[2]), "=r"(z[3]));
}
// byte permute with the selector as it is (the intrinsic first masks bit 3 of every selector nibble: one more instruction)
__device__ __forceinline__ uint32_t prmt_raw(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// shared-memory geometry
#define MMA_ROW_PITCH 80u                  // staged row segment: 64 B of qs (one 256-block) + 16 B pad (8-byte reads of 8 rows hit 8 bank pairs)
#define MMA_STAGES 3u                      // units in flight per warp: two ahead of the one being multiplied (HBM latency ~ one unit of work)
#define MMA_CHUNK_COLS 256u                // columns per staged unit (one block)
#ifndef MMA_MINB
#define MMA_MINB 2                         // blocks per SM the register allocation aims at
#endif
#ifndef MMA_KG_UNROLL
#define MMA_KG_UNROLL 2                    // 32-column groups in flight per warp
#endif
// copies of the magnitude table in shared memory (replica = lane % copies): 16 in the 16-warp gate/up kernel (measured
// 9 % faster there: two lanes per replica, always the minimum of two wavefronts per lookup), 8 where shared memory
// decides how many blocks fit an SM
#define MMA_GREP 8u
#define MMA_GREP_GU16 16u
#define RC_PRAGMA_(x) _Pragma(#x)
#define RC_UNROLL(n) RC_PRAGMA_(unroll n)

// One warp: 16 rows x one 256-column block of `NMAT` matrices against the first `ntiles` of NTILE 8-column tiles.
// Integer accumulation over the 8 groups of the block, then one fp32 scaling by d/8 into out[m][tile][4].
// Bs: activation digits of the work item in shared memory, column-major with pitch bpitch (== 32 mod 128: the 8-byte
// fragment reads of the 8 columns of a tile fall into 8 different bank groups).
// NUSED > 0: the number of column tiles in use is a compile-time constant (no per-tile tests in the loop).
template <int NMAT, int NTILE, int NUSED = 0, uint32_t GREP = MMA_GREP>
__device__ __forceinline__ void mma_unit(const uint8_t *stage, const float (&dsc)[NMAT][2], const int8_t *Bs, uint32_t bpitch, uint32_t kbase,
                                         const uint8_t *lutg, const uint8_t *luts, uint32_t lane, uint32_t ntiles, float (&out)[NMAT][NTILE][4]) {
    if (NUSED > 0) ntiles = NUSED;
    int z[4];
    zero_quad(z);
    const uint32_t g = lane >> 2, t = lane & 3u, rep8 = (lane & (GREP - 1u)) * 8u, rep16 = (lane & 7u) * 16u;
    const uint32_t sel = 0x4440u + t, sh7 = 7u * t;
    int blk[NMAT][NTILE][4];
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
        for (int n = 0; n < NTILE; ++n) { blk[m][n][0] = blk[m][n][1] = blk[m][n][2] = blk[m][n][3] = 0; }
    RC_UNROLL(MMA_KG_UNROLL)
    for (int kg = 0; kg < 8; ++kg) {
        uint32_t a[NMAT][4];
        int sc[NMAT][2];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint2 q = *reinterpret_cast<const uint2 *>(stage + (uint32_t)(m * 16 + h * 8 + g) * MMA_ROW_PITCH + (uint32_t)kg * 8u);
                const uint32_t gi = prmt_raw(q.x, 0u, sel);
                const uint32_t s7 = (q.y >> sh7) & 127u;
                const uint2 P = *reinterpret_cast<const uint2 *>(lutg + gi * (GREP * 8u) + rep8);
                if (GREP == 16u) {      // 16 copies of the 8-byte sign mask; the +1 carry term is recomputed from it
                    const uint2 M = *reinterpret_cast<const uint2 *>(luts + s7 * 128u + rep8);
                    a[m][h] = (P.x ^ M.x) + (M.x & 0x01010101u);
                    a[m][2 + h] = (P.y ^ M.y) + (M.y & 0x01010101u);
                } else {
                    const uint4 M = *reinterpret_cast<const uint4 *>(luts + s7 * 128u + rep16);
                    a[m][h] = (P.x ^ M.x) + M.z;         // bytes: +g, or ~g + 1 = -g (no carry between bytes: g >= 1)
                    a[m][2 + h] = (P.y ^ M.y) + M.w;
                }
                sc[m][h] = (int)(2u * (q.y >> 28) + 1u);
            }
        }
#pragma unroll
        for (int n = 0; n < NTILE; ++n) {
            if (NUSED > 0 ? n >= NUSED : (uint32_t)n >= ntiles) break;        // column tiles beyond the item's tokens hold zeros: skip them
            const uint2 bf = *reinterpret_cast<const uint2 *>(Bs + (uint32_t)(n * 8 + g) * bpitch + kbase + (uint32_t)kg * 32u + 8u * t);
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                int d[4];
                mma_s8_k32(d, a[m][0], a[m][1], a[m][2], a[m][3], bf.x, bf.y, z);
                blk[m][n][0] += sc[m][0] * d[0]; blk[m][n][1] += sc[m][0] * d[1];
                blk[m][n][2] += sc[m][1] * d[2]; blk[m][n][3] += sc[m][1] * d[3];
            }
        }
    }
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
        for (int n = 0; n < NTILE; ++n) {
            if (NUSED > 0 ? n >= NUSED : (uint32_t)n >= ntiles) break;
            out[m][n][0] += dsc[m][0] * (float)blk[m][n][0]; out[m][n][1] += dsc[m][0] * (float)blk[m][n][1];
            out[m][n][2] += dsc[m][1] * (float)blk[m][n][2]; out[m][n][3] += dsc[m][1] * (float)blk[m][n][3];
        }
}

// Block = 8 warps = R row tiles x S column splits (R*S == 8). The NTILE == 1 instance (work items of one or two pairs:
// four fifths of a Zipf-routed batch, and all of single-token decode) fits two blocks per SM (<= 128 registers, ~105 KB
// shared memory), so that one block's table fill, first weight load and epilogue overlap the other's MMA loop.
// item_class: 0 = take every item, 1 = only items of at most 2 pairs, 2 = only larger items (a batch is served by one
// NTILE == 1 launch for the small items and one NTILE == 3 launch for the rest).
// Warp (r, ks) works on `tiles_per_warp` 16-row tiles and on the 256-column blocks c with c % S == ks.
// grid = (row-tile groups, work items); one work item = up to TOK pairs of one expert (k_group_pairs cuts every
// expert's pairs into such items, so that all blocks carry the same amount of work whatever the routing skew).
template <int NMAT, int NTILE>
__global__ void __launch_bounds__(256, NTILE == 1 ? MMA_MINB : (NMAT == 1 && NTILE == 6 ? 2 : 1)) k_moe_mma(const __grid_constant__ MmaArgs A) {
    pdl_prologue();
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr uint32_t NCOL = NTILE * 8u;
    if (blockIdx.y >= *A.n_items) return;
    const uint32_t u = A.item_u[blockIdx.y], p0 = A.item_p0[blockIdx.y];
    const uint32_t e = A.uexp[u] - A.expert_begin, pe = A.ustart[u + 1u], nt = min(A.item_tok, pe - p0);
    if (e >= A.n_local) { if (A.status && threadIdx.x == 0) A.status[ST_EXPERT_RANGE] = 1u; return; }     // never index the arena with a foreign id
    if ((A.item_class == 1u && nt > 2u) || (A.item_class == 2u && nt <= 2u)) return;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t S = A.S, R = 8u / S, r = warp / S, ks = warp % S;
    const uint32_t bpr = A.ncols >> 8, nchunks = bpr;
    // carve shared memory: tables, per-warp staging, per-warp epilogue scratch (aliased onto the staging when NMAT == 2)
    uint8_t *lutg = smem;                                   // 256 x 64 B
    uint8_t *luts = lutg + 256u * MMA_GREP * 8u;            // 128 x 128 B
    uint8_t *stage0 = luts + 128u * 128u;                   // 8 warps x STAGES x NMAT*16 rows x pitch
    constexpr uint32_t stage_bytes = NMAT * 16u * MMA_ROW_PITCH, warp_stage = MMA_STAGES * stage_bytes;
    constexpr uint32_t scratch_bytes = NMAT * 16u * NCOL * 4u;
    static_assert(NMAT == 1 || scratch_bytes <= warp_stage, "the epilogue scratch of a gate/up warp must fit its staging area");
    uint8_t *my_stage = stage0 + warp * warp_stage;
    uint8_t *scratch_base = NMAT == 2 ? stage0 : stage0 + 8u * warp_stage;
    const uint32_t bpitch = A.ncols + 32u;
    int8_t *Bs = reinterpret_cast<int8_t *>(stage0 + 8u * warp_stage + (NMAT == 2 ? 0u : 8u * scratch_bytes));   // NCOL x bpitch
    constexpr uint32_t scratch_pitch = NMAT == 2 ? warp_stage : scratch_bytes;
    float *my_scratch = reinterpret_cast<float *>(scratch_base + warp * scratch_pitch);

    for (uint32_t i = tid; i < 256u * MMA_GREP; i += 256u) reinterpret_cast<uint2 *>(lutg)[i] = A.lut_grid[i / MMA_GREP];
    for (uint32_t i = tid; i < 128u * 8u; i += 256u) reinterpret_cast<uint4 *>(luts)[i] = A.lut_sign[i >> 3];

    const uint8_t *w[2] = {A.w0 + (size_t)e * A.mat_bytes, A.w1 ? A.w1 + (size_t)e * A.mat_bytes : nullptr};
    const uint32_t tile_first = (blockIdx.x * R + r) * A.tiles_per_warp;            // in units of 16 rows
    uint32_t my_chunks = 0;
    for (uint32_t c = ks; c < nchunks; c += S) ++my_chunks;
    const uint32_t ntile_rows = A.nrows >> 4;
    uint32_t my_tiles = 0;
    for (uint32_t i = 0; i < A.tiles_per_warp; ++i) if (tile_first + i < ntile_rows) ++my_tiles;
    const uint32_t nunits = my_tiles * my_chunks;

    const uint32_t ntiles = (3u * nt + 7u) >> 3;

    auto issue = [&](uint32_t unit, uint32_t buf) {
        const uint32_t ti = unit / my_chunks, c = ks + (unit - ti * my_chunks) * S;
        const uint32_t row0 = (tile_first + ti) << 4;
        uint8_t *dst = my_stage + buf * stage_bytes;
#pragma unroll
        for (uint32_t i = 0; i < NMAT * 2u; ++i) {
            const uint32_t p = lane + 32u * i, rr = p >> 2, piece = p & 3u, m = rr >> 4, row = row0 + (rr & 15u);
            cp_async16(dst + rr * MMA_ROW_PITCH + piece * 16u, w[m] + ((size_t)row * bpr + c) * 64u + piece * 16u);
        }
    };

    for (uint32_t i = 0; i + 1u < MMA_STAGES; ++i) {     // weights start streaming while the tables and the activations settle
        if (i < nunits) issue(i, i);
        cp_async_commit();
    }
    {   // activation digits of pairs [p0, p0 + nt): column = 3 * token + digit; only the tiles in use are filled
        const uint32_t v16 = A.ncols >> 4;
        for (uint32_t i = tid; i < ntiles * 8u * v16; i += 256u) {
            const uint32_t col = i / v16, k = (i - col * v16) << 4, tk = col / 3u, dg = col - tk * 3u;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (tk < nt) v = *reinterpret_cast<const uint4 *>(A.xq + ((size_t)(A.sorted[p0 + tk] / A.x_div) * 3u + dg) * A.ncols + k);
            *reinterpret_cast<uint4 *>(Bs + (size_t)col * bpitch + k) = v;
        }
    }
    __syncthreads();

    float out[NMAT][NTILE][4];
    for (uint32_t unit = 0; unit < nunits; ++unit) {
        const uint32_t ti = unit / my_chunks, ci = unit - ti * my_chunks, c = ks + ci * S;
        const uint32_t row0 = (tile_first + ti) << 4;
        if (unit + MMA_STAGES - 1u < nunits) issue(unit + MMA_STAGES - 1u, (unit + MMA_STAGES - 1u) % MMA_STAGES);
        cp_async_commit();
        float dsc[NMAT][2];              // d/8 of rows g, g+8 for this block (plain loads, 2 B each)
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const size_t bi = (size_t)(row0 + h * 8u + g) * bpr + c;
                dsc[m][h] = 0.125f * __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(w[m] + A.nb * 64u) + bi)));
            }
        if (ci == 0u) {
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
                for (int n = 0; n < NTILE; ++n) { out[m][n][0] = out[m][n][1] = out[m][n][2] = out[m][n][3] = 0.f; }
        }
        cp_async_wait<MMA_STAGES - 1>();
        __syncwarp();
        {
            const uint8_t *st = my_stage + (unit % MMA_STAGES) * stage_bytes;
            if (NTILE >= 3 && ntiles == 1u) mma_unit<NMAT, NTILE, 1>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
            else if (NTILE >= 3 && ntiles == 2u) mma_unit<NMAT, NTILE, 2>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
            else if (NTILE >= 3 && ntiles == 3u) mma_unit<NMAT, NTILE, (NTILE >= 3 ? 3 : 0)>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
            else if (NTILE == 6 && ntiles == 4u) mma_unit<NMAT, NTILE, (NTILE == 6 ? 4 : 0)>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
            else if (NTILE == 6 && ntiles == 5u) mma_unit<NMAT, NTILE, (NTILE == 6 ? 5 : 0)>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
            else mma_unit<NMAT, NTILE, (NTILE >= 3 ? NTILE : 0)>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);   // NTILE == 1: the tested form measured faster
        }
        __syncwarp();
        if (ci + 1u == my_chunks) {
            // ---- tile finished for this warp: fragments -> scratch[m][row][col]. With NMAT == 2 the scratch is the warp's own
            // staging area: a gate/up warp has one tile (launcher), so nothing is in flight into it any more.
            if (NMAT == 2) { cp_async_wait<0>(); __syncwarp(); }
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
                for (int n = 0; n < NTILE; ++n) {
                    float *sp = my_scratch + (size_t)m * 16u * NCOL + n * 8u + 2u * t;
                    const bool live = (uint32_t)n < ntiles;
                    sp[(size_t)g * NCOL] = live ? out[m][n][0] : 0.f; sp[(size_t)g * NCOL + 1u] = live ? out[m][n][1] : 0.f;
                    sp[(size_t)(g + 8u) * NCOL] = live ? out[m][n][2] : 0.f; sp[(size_t)(g + 8u) * NCOL + 1u] = live ? out[m][n][3] : 0.f;
                }
            if (S > 1u) __syncthreads(); else __syncwarp();       // S > 1 implies one tile per warp: every warp gets here once
            if (ks == 0u) {
                for (uint32_t idx = lane; idx < 16u * nt; idx += 32u) {
                    const uint32_t row = idx & 15u, tk = idx >> 4;
                    const uint32_t p = A.sorted[p0 + tk];
                    const float sxv = A.sx[p / A.x_div];
                    float val[NMAT];
#pragma unroll
                    for (int m = 0; m < NMAT; ++m) {
                        float o0 = 0.f, o1 = 0.f, o2 = 0.f;
                        for (uint32_t s = 0; s < S; ++s) {
                            const float *sp = reinterpret_cast<const float *>(scratch_base + (warp + s) * scratch_pitch) + (size_t)m * 16u * NCOL + (size_t)row * NCOL + 3u * tk;
                            o0 += sp[0]; o1 += sp[1]; o2 += sp[2];
                        }
                        val[m] = sxv * (A.dw2 * o2 + A.dw1 * o1 + o0);
                    }
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

// Gate/up of a batch with 16 warps per block: warps 0-7 take the gate rows of eight 16-row tiles, warps 8-15 the up rows
// of the same tiles, each with the single-matrix MMA loop (92 registers instead of the 142 of the fused two-matrix loop),
// so twice as many warps hide the dependent table lookups. A block-wide barrier hands the up values to the gate warps,
// which apply SiLU(gate) * up. Same shared-memory budget as the 8-warp kernel (the staging is per 16 rows).
template <int NTILE>
__global__ void __launch_bounds__(512, 1) k_moe_gateup16(const __grid_constant__ MmaArgs A) {
    pdl_prologue();
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr uint32_t NCOL = NTILE * 8u;
    if (blockIdx.y >= *A.n_items) return;
    const uint32_t u = A.item_u[blockIdx.y], p0 = A.item_p0[blockIdx.y];
    const uint32_t e = A.uexp[u] - A.expert_begin, pe = A.ustart[u + 1u], nt = min(A.item_tok, pe - p0);
    if (e >= A.n_local) { if (A.status && threadIdx.x == 0) A.status[ST_EXPERT_RANGE] = 1u; return; }     // never index the arena with a foreign id
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t bpr = A.ncols >> 8;
    uint8_t *lutg = smem, *luts = lutg + 256u * MMA_GREP_GU16 * 8u, *stage0 = luts + 128u * 128u;
    constexpr uint32_t stage_bytes = 16u * MMA_ROW_PITCH, warp_stage = MMA_STAGES * stage_bytes;
    static_assert(16u * NCOL * 4u <= warp_stage, "the epilogue scratch of a warp must fit its staging area");
    uint8_t *my_stage = stage0 + warp * warp_stage;
    const uint32_t bpitch = A.ncols + 32u;
    int8_t *Bs = reinterpret_cast<int8_t *>(stage0 + 16u * warp_stage);

    for (uint32_t i = tid; i < 256u * MMA_GREP_GU16; i += 512u) reinterpret_cast<uint2 *>(lutg)[i] = A.lut_grid[i / MMA_GREP_GU16];
    for (uint32_t i = tid; i < 128u * 16u; i += 512u) { const uint4 e4 = A.lut_sign[i >> 4]; reinterpret_cast<uint2 *>(luts)[i] = make_uint2(e4.x, e4.y); }

    const uint32_t is_up = warp >> 3;
    const uint8_t *w = (is_up ? A.w1 : A.w0) + (size_t)e * A.mat_bytes;
    const uint32_t tile = blockIdx.x * 8u + (warp & 7u), row0 = tile << 4;
    const bool live_tile = tile < (A.nrows >> 4);
    const uint32_t nunits = live_tile ? bpr : 0u;
    const uint32_t ntiles = (3u * nt + 7u) >> 3;

    auto issue = [&](uint32_t c, uint32_t buf) {
        uint8_t *dst = my_stage + buf * stage_bytes;
#pragma unroll
        for (uint32_t i = 0; i < 2u; ++i) {
            const uint32_t p = lane + 32u * i, rr = p >> 2, piece = p & 3u;
            cp_async16(dst + rr * MMA_ROW_PITCH + piece * 16u, w + ((size_t)(row0 + rr) * bpr + c) * 64u + piece * 16u);
        }
    };
    for (uint32_t i = 0; i + 1u < MMA_STAGES; ++i) {
        if (i < nunits) issue(i, i);
        cp_async_commit();
    }
    {
        const uint32_t v16 = A.ncols >> 4;
        for (uint32_t i = tid; i < ntiles * 8u * v16; i += 512u) {
            const uint32_t col = i / v16, k = (i - col * v16) << 4, tk = col / 3u, dg = col - tk * 3u;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (tk < nt) v = *reinterpret_cast<const uint4 *>(A.xq + ((size_t)(A.sorted[p0 + tk] / A.x_div) * 3u + dg) * A.ncols + k);
            *reinterpret_cast<uint4 *>(Bs + (size_t)col * bpitch + k) = v;
        }
    }
    __syncthreads();

    float out[1][NTILE][4];
#pragma unroll
    for (int n = 0; n < NTILE; ++n) { out[0][n][0] = out[0][n][1] = out[0][n][2] = out[0][n][3] = 0.f; }
    for (uint32_t c = 0; c < nunits; ++c) {
        if (c + MMA_STAGES - 1u < nunits) issue(c + MMA_STAGES - 1u, (c + MMA_STAGES - 1u) % MMA_STAGES);
        cp_async_commit();
        float dsc[1][2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const size_t bi = (size_t)(row0 + h * 8u + g) * bpr + c;
            dsc[0][h] = 0.125f * __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(w + A.nb * 64u) + bi)));
        }
        cp_async_wait<MMA_STAGES - 1>();
        __syncwarp();
        const uint8_t *st = my_stage + (c % MMA_STAGES) * stage_bytes;
        if (NTILE >= 3 && ntiles == 1u) mma_unit<1, NTILE, 1, MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        else if (NTILE >= 3 && ntiles == 2u) mma_unit<1, NTILE, 2, MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        else if (NTILE >= 3 && ntiles == 3u) mma_unit<1, NTILE, 3, MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        else if (NTILE == 6 && ntiles == 4u) mma_unit<1, NTILE, (NTILE == 6 ? 4 : NTILE), MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        else if (NTILE == 6 && ntiles == 5u) mma_unit<1, NTILE, (NTILE == 6 ? 5 : NTILE), MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        else mma_unit<1, NTILE, NTILE, MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        __syncwarp();
    }
    cp_async_wait<0>();
    __syncwarp();
    float *my_scratch = reinterpret_cast<float *>(my_stage);          // nothing is in flight into the staging any more
#pragma unroll
    for (int n = 0; n < NTILE; ++n) {
        float *sp = my_scratch + n * 8u + 2u * t;
        const bool live = (uint32_t)n < ntiles;
        sp[(size_t)g * NCOL] = live ? out[0][n][0] : 0.f; sp[(size_t)g * NCOL + 1u] = live ? out[0][n][1] : 0.f;
        sp[(size_t)(g + 8u) * NCOL] = live ? out[0][n][2] : 0.f; sp[(size_t)(g + 8u) * NCOL + 1u] = live ? out[0][n][3] : 0.f;
    }
    __syncthreads();
    if (!is_up && live_tile) {
        const float *gs = my_scratch, *us = reinterpret_cast<const float *>(my_stage + 8u * warp_stage);
        for (uint32_t idx = lane; idx < 16u * nt; idx += 32u) {
            const uint32_t row = idx & 15u, tk = idx >> 4;
            const uint32_t p = A.sorted[p0 + tk];
            const float sxv = A.sx[p / A.x_div];
            const float *a = gs + (size_t)row * NCOL + 3u * tk, *b = us + (size_t)row * NCOL + 3u * tk;
            const float gte = sxv * (A.dw2 * a[2] + A.dw1 * a[1] + a[0]), upv = sxv * (A.dw2 * b[2] + A.dw1 * b[1] + b[0]);
            A.out[(size_t)p * A.out_stride + row0 + row] = (gte / (1.0f + expf(-gte))) * upv;
        }
    }
}

// Down projection of a batch with 16 warps per block sharing one set of tables (16 copies of both, as in the gate/up
// kernel): warp w of block x takes the `tiles_per_warp` 16-row tiles starting at (16 x + w) * tiles_per_warp, one after
// the other, each over all 256-column blocks of the row. The epilogue scratch is separate from the staging (the next
// tile's weights are already in flight when a tile finishes).
template <int NTILE>
__global__ void __launch_bounds__(512, 1) k_moe_down16(const __grid_constant__ MmaArgs A) {
    pdl_prologue();
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr uint32_t NCOL = NTILE * 8u;
    if (blockIdx.y >= *A.n_items) return;
    const uint32_t u = A.item_u[blockIdx.y], p0 = A.item_p0[blockIdx.y];
    const uint32_t e = A.uexp[u] - A.expert_begin, pe = A.ustart[u + 1u], nt = min(A.item_tok, pe - p0);
    if (e >= A.n_local) { if (A.status && threadIdx.x == 0) A.status[ST_EXPERT_RANGE] = 1u; return; }     // never index the arena with a foreign id
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t bpr = A.ncols >> 8;
    uint8_t *lutg = smem, *luts = lutg + 256u * MMA_GREP_GU16 * 8u, *stage0 = luts + 128u * 128u;
    constexpr uint32_t stage_bytes = 16u * MMA_ROW_PITCH, warp_stage = MMA_STAGES * stage_bytes, scratch_bytes = 16u * NCOL * 4u;
    uint8_t *my_stage = stage0 + warp * warp_stage;
    float *my_scratch = reinterpret_cast<float *>(stage0 + 16u * warp_stage + warp * scratch_bytes);
    const uint32_t bpitch = A.ncols + 32u;
    int8_t *Bs = reinterpret_cast<int8_t *>(stage0 + 16u * warp_stage + 16u * scratch_bytes);

    for (uint32_t i = tid; i < 256u * MMA_GREP_GU16; i += 512u) reinterpret_cast<uint2 *>(lutg)[i] = A.lut_grid[i / MMA_GREP_GU16];
    for (uint32_t i = tid; i < 128u * 16u; i += 512u) { const uint4 e4 = A.lut_sign[i >> 4]; reinterpret_cast<uint2 *>(luts)[i] = make_uint2(e4.x, e4.y); }

    const uint8_t *w = A.w0 + (size_t)e * A.mat_bytes;
    const uint32_t tile_first = (blockIdx.x * 16u + warp) * A.tiles_per_warp, ntile_rows = A.nrows >> 4;
    uint32_t my_tiles = 0;
    for (uint32_t i = 0; i < A.tiles_per_warp; ++i) if (tile_first + i < ntile_rows) ++my_tiles;
    const uint32_t nunits = my_tiles * bpr;
    const uint32_t ntiles = (3u * nt + 7u) >> 3;

    auto issue = [&](uint32_t unit, uint32_t buf) {
        const uint32_t ti = unit / bpr, c = unit - ti * bpr, row0 = (tile_first + ti) << 4;
        uint8_t *dst = my_stage + buf * stage_bytes;
#pragma unroll
        for (uint32_t i = 0; i < 2u; ++i) {
            const uint32_t p = lane + 32u * i, rr = p >> 2, piece = p & 3u;
            cp_async16(dst + rr * MMA_ROW_PITCH + piece * 16u, w + ((size_t)(row0 + rr) * bpr + c) * 64u + piece * 16u);
        }
    };
    for (uint32_t i = 0; i + 1u < MMA_STAGES; ++i) {
        if (i < nunits) issue(i, i);
        cp_async_commit();
    }
    {
        const uint32_t v16 = A.ncols >> 4;
        for (uint32_t i = tid; i < ntiles * 8u * v16; i += 512u) {
            const uint32_t col = i / v16, k = (i - col * v16) << 4, tk = col / 3u, dg = col - tk * 3u;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (tk < nt) v = *reinterpret_cast<const uint4 *>(A.xq + ((size_t)(A.sorted[p0 + tk] / A.x_div) * 3u + dg) * A.ncols + k);
            *reinterpret_cast<uint4 *>(Bs + (size_t)col * bpitch + k) = v;
        }
    }
    __syncthreads();

    float out[1][NTILE][4];
    for (uint32_t unit = 0; unit < nunits; ++unit) {
        const uint32_t ti = unit / bpr, c = unit - ti * bpr, row0 = (tile_first + ti) << 4;
        if (unit + MMA_STAGES - 1u < nunits) issue(unit + MMA_STAGES - 1u, (unit + MMA_STAGES - 1u) % MMA_STAGES);
        cp_async_commit();
        float dsc[1][2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const size_t bi = (size_t)(row0 + h * 8u + g) * bpr + c;
            dsc[0][h] = 0.125f * __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(w + A.nb * 64u) + bi)));
        }
        if (c == 0u) {
#pragma unroll
            for (int n = 0; n < NTILE; ++n) { out[0][n][0] = out[0][n][1] = out[0][n][2] = out[0][n][3] = 0.f; }
        }
        cp_async_wait<MMA_STAGES - 1>();
        __syncwarp();
        const uint8_t *st = my_stage + (unit % MMA_STAGES) * stage_bytes;
        if (NTILE >= 3 && ntiles == 1u) mma_unit<1, NTILE, 1, MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        else if (NTILE >= 3 && ntiles == 2u) mma_unit<1, NTILE, 2, MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        else if (NTILE >= 3 && ntiles == 3u) mma_unit<1, NTILE, 3, MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        else if (NTILE == 6 && ntiles == 4u) mma_unit<1, NTILE, (NTILE == 6 ? 4 : NTILE), MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        else if (NTILE == 6 && ntiles == 5u) mma_unit<1, NTILE, (NTILE == 6 ? 5 : NTILE), MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        else mma_unit<1, NTILE, NTILE, MMA_GREP_GU16>(st, dsc, Bs, bpitch, c * MMA_CHUNK_COLS, lutg, luts, lane, ntiles, out);
        __syncwarp();
        if (c + 1u == bpr) {      // tile finished: fragments -> the warp's scratch -> rows of the pairs
#pragma unroll
            for (int n = 0; n < NTILE; ++n) {
                float *sp = my_scratch + n * 8u + 2u * t;
                const bool live = (uint32_t)n < ntiles;
                sp[(size_t)g * NCOL] = live ? out[0][n][0] : 0.f; sp[(size_t)g * NCOL + 1u] = live ? out[0][n][1] : 0.f;
                sp[(size_t)(g + 8u) * NCOL] = live ? out[0][n][2] : 0.f; sp[(size_t)(g + 8u) * NCOL + 1u] = live ? out[0][n][3] : 0.f;
            }
            __syncwarp();
            for (uint32_t idx = lane; idx < 16u * nt; idx += 32u) {
                const uint32_t row = idx & 15u, tk = idx >> 4;
                const uint32_t p = A.sorted[p0 + tk];
                const float *a = my_scratch + (size_t)row * NCOL + 3u * tk;
                A.out[(size_t)p * A.out_stride + row0 + row] = A.sx[p / A.x_div] * (A.dw2 * a[2] + A.dw1 * a[1] + a[0]);
            }
            __syncwarp();
        }
    }
    cp_async_wait<0>();
}

size_t mma_smem_bytes(uint32_t nmat, uint32_t ntile, uint32_t ncols) {
    const size_t stages = 8u * MMA_STAGES * nmat * 16u * MMA_ROW_PITCH;
    return 256u * MMA_GREP * 8u + 128u * 128u + stages + (nmat == 2u ? 0u : 8u * 16u * ntile * 8u * 4u) + (size_t)ntile * 8u * (ncols + 32u);
}

uint32_t mma_item_tokens(bool few_tokens, uint32_t npairs, uint32_t n_experts) {
    static const bool allow16 = !(getenv("RC_MMA_ITEM16") && atoi(getenv("RC_MMA_ITEM16")) == 0);   // A/B switch
    return few_tokens ? 2u : (allow16 && npairs >= 6u * n_experts ? 16u : 8u);
}

int launch_moe_mma(MmaArgs &A, uint32_t groups, uint32_t item_tok, cudaStream_t s) {
    const bool few_tokens = item_tok <= 2u, big_items = item_tok > 8u;
    RC_REQUIRE(item_tok == 2u || item_tok == 8u || item_tok == 16u, "moe mma: work items of %u pairs are not built", item_tok);
    int dev = 0;
    RC_CUDA(cudaGetDevice(&dev));
    A.lut_grid = g_lut_grid_ptr[dev & 63];
    A.dw1 = (float)(1u << act_digit_bits()); A.dw2 = A.dw1 * A.dw1;
    A.lut_sign = g_lut_sign_ptr[dev & 63];
    RC_REQUIRE(A.lut_grid && A.lut_sign, "IQ2_XXS tensor-core tables not set on device %d: call redcuda_set_codebooks first", dev);
    RC_REQUIRE(A.ncols % MMA_CHUNK_COLS == 0 && A.nrows % 16u == 0, "moe mma: matrix %ux%u is not a multiple of 16 rows x 256 columns", A.nrows, A.ncols);
    const uint32_t nmat = A.w1 ? 2u : 1u, nchunks = A.ncols / MMA_CHUNK_COLS, ntile_rows = A.nrows / 16u;
    // Single-token decode: few row tiles in total, so the wide matrices are also split along the columns (S warps
    // share a row tile); batches: about four blocks per expert for the down projection (one tile per warp for gate/up,
    // whose epilogue scratch lives in the warp's staging area).
    uint32_t S = 1u, tpw = 1u;
    if (few_tokens) {
        while (S < 8u && S * 2u <= nchunks && nchunks % (S * 2u) == 0 && (uint64_t)ntile_rows * groups * S < 148u * 16u) S <<= 1;
    } else if (nmat == 1u) {
        while (tpw < 8u && ntile_rows / (8u * tpw * 2u) >= 4u && ntile_rows % (8u * tpw * 2u) == 0) tpw <<= 1;
    }
    const uint32_t R = 8u / S;
    A.S = S; A.tiles_per_warp = tpw;
    A.item_tok = item_tok;
    const dim3 grid((ntile_rows + R * tpw - 1u) / (R * tpw), groups);
    prof_begin(nmat == 2u ? "moe_gateup" : "moe_down", s);
#define RC_MMA_LAUNCH(NM, NT, CLS) do { \
        const size_t smem = mma_smem_bytes(NM, NT, A.ncols); \
        RC_REQUIRE(smem <= 227u * 1024u, "moe mma: %zu bytes of shared memory needed for %u columns", smem, A.ncols); \
        A.item_class = CLS; \
        RC_CUDA(cudaFuncSetAttribute(k_moe_mma<NM, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        RC_LAUNCH((k_moe_mma<NM, NT>), grid, 256, smem, s, A); g_launches.fetch_add(1, std::memory_order_relaxed); } while (0)
    if (few_tokens) { if (nmat == 2u) RC_MMA_LAUNCH(2, 1, 0u); else RC_MMA_LAUNCH(1, 1, 0u); }
    else {
        static const bool split = getenv("RC_MMA_SPLIT") && atoi(getenv("RC_MMA_SPLIT")) != 0;   // A/B switch; measured: one launch for all items is faster (no serialised tails)
        if (split && !big_items) {      // large items first: they are the long blocks
            if (nmat == 2u) { RC_MMA_LAUNCH(2, 3, 2u); RC_MMA_LAUNCH(2, 1, 1u); } else { RC_MMA_LAUNCH(1, 3, 2u); RC_MMA_LAUNCH(1, 1, 1u); }
        } else if (nmat == 2u) {
            static const bool gu16 = !(getenv("RC_MMA_GU16") && atoi(getenv("RC_MMA_GU16")) == 0);   // A/B switch
            RC_REQUIRE(!big_items || (gu16 && tpw == 1u && S == 1u), "moe mma: work items of 16 pairs need the 16-warp gate/up kernel");
            if (gu16 && tpw == 1u && S == 1u) {
                const size_t smem = 256u * MMA_GREP_GU16 * 8u + 128u * 128u + 16u * MMA_STAGES * 16u * MMA_ROW_PITCH + (size_t)(big_items ? 48u : 24u) * (A.ncols + 32u);
                RC_REQUIRE(smem <= 227u * 1024u, "moe mma: %zu bytes of shared memory needed for %u columns", smem, A.ncols);
                A.item_class = 0u;
                if (big_items) {
                    RC_CUDA(cudaFuncSetAttribute(k_moe_gateup16<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                    RC_LAUNCH((k_moe_gateup16<6>), dim3((ntile_rows + 7u) / 8u, groups), 512, smem, s, A);
                } else {
                    RC_CUDA(cudaFuncSetAttribute(k_moe_gateup16<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                    RC_LAUNCH((k_moe_gateup16<3>), dim3((ntile_rows + 7u) / 8u, groups), 512, smem, s, A);
                }
                g_launches.fetch_add(1, std::memory_order_relaxed);
            } else RC_MMA_LAUNCH(2, 3, 0u);
        } else {
            // down projection: 16 warps per block when the tiles divide evenly (2 tiles per warp at the usual 2048 rows)
            static const bool down16 = !(getenv("RC_MMA_DOWN16") && atoi(getenv("RC_MMA_DOWN16")) == 0);   // A/B switch
            uint32_t tpw16 = 1u;
            while (tpw16 < 8u && ntile_rows / (16u * tpw16 * 2u) >= 4u && ntile_rows % (16u * tpw16 * 2u) == 0) tpw16 <<= 1;
            const uint32_t ncol = big_items ? 48u : 24u;
            const size_t smem16 = 256u * MMA_GREP_GU16 * 8u + 128u * 128u + 16u * MMA_STAGES * 16u * MMA_ROW_PITCH + 16u * 16u * ncol * 4u + (size_t)ncol * (A.ncols + 32u);
            if (down16 && ntile_rows % (16u * tpw16) == 0 && smem16 <= 227u * 1024u) {
                A.tiles_per_warp = tpw16; A.item_class = 0u;
                const dim3 grid16(ntile_rows / (16u * tpw16), groups);
                if (big_items) {
                    RC_CUDA(cudaFuncSetAttribute(k_moe_down16<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem16));
                    RC_LAUNCH((k_moe_down16<6>), grid16, 512, smem16, s, A);
                } else {
                    RC_CUDA(cudaFuncSetAttribute(k_moe_down16<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem16));
                    RC_LAUNCH((k_moe_down16<3>), grid16, 512, smem16, s, A);
                }
                g_launches.fetch_add(1, std::memory_order_relaxed);
            } else if (big_items) RC_MMA_LAUNCH(1, 6, 0u);
            else RC_MMA_LAUNCH(1, 3, 0u);
        }
    }
#undef RC_MMA_LAUNCH
    g_launches.fetch_sub(1, std::memory_order_relaxed);     // RC_LAUNCHED below counts one of them
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

}  // namespace rc
