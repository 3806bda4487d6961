// Routed IQ2_XXS experts in the "nibble" layout: a load-time re-coding whose decode needs no table in shared memory.
//
// Why: IQ2_XXS stores 8 weights as one codebook index (8 bits) plus 7 sign bits; turning them into tensor-core operands
// costs two dependent shared-memory lookups and ~10 integer instructions per 8 weights, and the expert kernels were
// bound by instruction issue at a sixth of HBM speed (57 M warp instructions per gate/up launch of a 64-token batch).
// Here every weight is re-coded once, at load, as a 4-bit code (bits 1:0 = which of the three codebook magnitudes
// 8 / 25 / 43, bit 2 = sign); a lane then expands 4 weights into an int8 operand register with ONE instruction
// (prmt against an 8-byte table held in two registers). Dequantised values are unchanged bit for bit
// (redcuda_nib_dequant_rows against rl_quant_dequant_row, native/redlite_native_quant_cpu.c:166-191). The price is bytes:
// 138 per 256 weights instead of 66, i.e. 2.09x the HBM footprint and traffic of the routed experts.
//
// Layout of one expert matrix [nrows][ncols], bpr = ncols / 256 blocks per row: one contiguous RECORD of 2208 bytes per
// (16-row tile, 256-column block), records ordered [tile][block], so that a warp fetches everything it needs for one
// block of its tile with a single bulk copy:
//   codes  @0     16 rows x 128 B; logical byte 32 t + 4 kg of a row = u32 word (t, kg) = the 8 weights 32 kg + 8 t .. +7
//                 of the block, weight j in bits 4j+3..4j (a lane's 8 words are 32 contiguous bytes). The 16-byte
//                 pieces of odd rows are stored pairwise swapped (piece p at p ^ 1): a record lands in shared memory
//                 as it is, and with the swap the 16-byte reads of a quarter warp hit eight different bank groups
//   scales @2048  16 rows x 8 B, byte kg = 2 s + 1, s the 4-bit scale of the 32-weight group
//   d      @2176  16 fp16 block scales
// Arithmetic is the integer tensor-core scheme of redcuda_moe_mma.cu (mma.sync m16n8k32 s8, activations as three
// balanced digits per value, s32 sums per 32-weight group scaled by the integer 2s+1, fp32 scaling by d/8 per block).
//
// Kernel: persistent CTAs of 8 warps, two per SM. A unit of work = one work item (<= 8 pairs of one expert, cut by
// k_group_pairs) x a block of rows; CTAs draw units from an atomic counter, so the routing skew never leaves SMs idle
// and nothing is set up per unit except the item's activation digits in shared memory. Every warp streams its 16-row
// tiles through a private ring of three records (one cp.async.bulk and one mbarrier each; the ring runs on across unit
// boundaries). Waits on the mbarriers are bounded: a warp that gives up raises the status word and the CTA winds down.
// Column layout of the digits: items of one or two pairs pack (pair, digit) into one 8-column tile (cols 3*pair+digit);
// larger items use one tile per digit (col = 8*digit + pair), so a lane holds all three digits of its two pairs and the
// epilogue needs no exchange.
#define RC_PDL_DEFAULT 0
#include "redcuda_common.cuh"
#include "redcuda_dot.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_moe_mma.cuh"
#include "../../include/redcuda.h"

#include <stdlib.h>

namespace rc {

uint64_t nib_matrix_bytes(uint32_t nrows, uint32_t ncols) { return (uint64_t)nrows * (ncols / 256u) * NIB_BLOCK_BYTES; }
bool nib_shape_ok(uint32_t nrows, uint32_t ncols) { return nrows % 16u == 0 && (ncols == 256u || ncols == 512u || ncols == 1024u || ncols == 2048u); }

// ---- planar IQ2_XXS -> nibble layout: one thread per (block, group kg, quarter t) ----
__global__ void k_nib_repack(const uint8_t *__restrict__ planar, uint64_t nb, uint32_t nrows, uint32_t bpr, const uint8_t *__restrict__ iq2,
                             uint8_t *__restrict__ dst) {
    pdl_prologue();
    const uint64_t total = nb * 32u;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t b = i >> 5;
        const uint32_t kg = ((uint32_t)i >> 2) & 7u, t = (uint32_t)i & 3u;
        const uint32_t row = (uint32_t)(b / bpr), blk = (uint32_t)(b - (uint64_t)row * bpr);
        const uint32_t auxg = *reinterpret_cast<const uint32_t *>(planar + b * 64u + kg * 8u), auxs = *reinterpret_cast<const uint32_t *>(planar + b * 64u + kg * 8u + 4u);
        const uint8_t *gv = iq2 + ((auxg >> (8u * t)) & 255u) * 8u;
        const uint32_t s8 = rc_sign8((auxs >> (7u * t)) & 127u);
        uint32_t word = 0u;
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) {
            const uint32_t m = gv[j] == 0x19u ? 1u : gv[j] == 0x2bu ? 2u : 0u;
            word |= (m | (((s8 >> j) & 1u) << 2)) << (4u * j);
        }
        uint8_t *rec = dst + ((uint64_t)(row >> 4) * bpr + blk) * NIB_REC;
        const uint32_t rr = row & 15u;
        *reinterpret_cast<uint32_t *>(rec + nib_code_off(rr, t, kg)) = word;
        if (t == 0u) {
            rec[NIB_SC_OFF + rr * 8u + kg] = (uint8_t)(2u * (auxs >> 28) + 1u);
            if (kg == 0u) *reinterpret_cast<unsigned short *>(rec + NIB_D_OFF + rr * 2u) = *reinterpret_cast<const unsigned short *>(planar + rc_iq2_d(nb) + b * 2u);
        }
    }
}

int launch_nib_repack(const uint8_t *planar, uint32_t nrows, uint32_t ncols, uint8_t *dst, cudaStream_t s) {
    RC_REQUIRE(nib_shape_ok(nrows, ncols), "nibble layout: matrix %ux%u is not tileable (16 rows, 256/512/1024/2048 columns)", nrows, ncols);
    RC_REQUIRE(((uintptr_t)dst & 15u) == 0 && ((uintptr_t)planar & 15u) == 0, "nibble layout: unaligned matrix");
    const uint64_t nb = (uint64_t)nrows * (ncols / 256u), total = nb * 32u;
    const uint32_t grid = (uint32_t)((total + 255u) / 256u < 148u * 16u ? (total + 255u) / 256u : 148u * 16u);
    prof_begin("nib_repack", s);
    RC_LAUNCH((k_nib_repack), grid ? grid : 1u, 256, 0, s, planar, nb, nrows, ncols / 256u, books_iq2(), dst);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

// ---- nibble layout -> fp32, the float operations of rl_quant_dequant_row in the same order (exact) ----
__global__ void k_nib_dequant(const uint8_t *__restrict__ nib, uint64_t nb, uint32_t nrows, uint32_t bpr, float *__restrict__ out) {
    pdl_prologue();
    const uint64_t total = nb * 32u;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t b = i >> 5;
        const uint32_t kg = ((uint32_t)i >> 2) & 7u, t = (uint32_t)i & 3u;
        const uint32_t row = (uint32_t)(b / bpr), blk = (uint32_t)(b - (uint64_t)row * bpr);
        const uint8_t *rec = nib + ((uint64_t)(row >> 4) * bpr + blk) * NIB_REC;
        const uint32_t rr = row & 15u;
        const uint32_t word = *reinterpret_cast<const uint32_t *>(rec + nib_code_off(rr, t, kg));
        const uint32_t scb = rec[NIB_SC_OFF + rr * 8u + kg];
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rec + NIB_D_OFF + rr * 2u)));
        const float db = d * (0.5f + (float)((scb - 1u) >> 1)) * 0.25f;
        float *o = out + ((uint64_t)row * bpr + blk) * 256u + kg * 32u + t * 8u;
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) {
            const uint32_t code = (word >> (4u * j)) & 7u, m = code & 3u;
            const float v = db * (m == 0u ? 8.0f : m == 1u ? 25.0f : 43.0f);
            o[j] = (code & 4u) ? -v : v;
        }
    }
}

// ---- small PTX wrappers ----
__device__ __forceinline__ uint32_t nb_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
// z: four registers that hold zero for the whole kernel, the accumulator input of every MMA (each 32-weight group gets
// its own exact s32 product sum, scaled by the group's integer scale afterwards)
__device__ __forceinline__ void nb_mma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, const int (&z)[4]) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z[0]), "r"(z[1]), "r"(z[2]), "r"(z[3]));
}
// byte permute with the selector taken as it is (the intrinsic masks bit 3 of every selector nibble first, one more
// instruction per use; the 4-bit codes never set it)
__device__ __forceinline__ uint32_t nb_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// one record into a ring slot: the copy engine signals the slot's mbarrier with the bytes it delivered
__device__ __forceinline__ void nb_fetch(uint32_t dst, const void *src, uint32_t bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(NIB_REC) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(NIB_REC), "r"(bar) : "memory");
}
constexpr uint32_t NIB_SPIN_LIMIT = 1u << 22;      // polls of the (itself time-limited) try_wait: far beyond any real wait
__device__ __forceinline__ bool nb_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < NIB_SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

constexpr uint32_t NIB_WARPS = 8u;
// records in flight per warp: 3 for batches (two blocks per SM), 8 for a single token (few units, one block per SM: a
// warp requests its whole tile at once, one HBM round trip instead of three)
constexpr uint32_t NIB_STAGES_BATCH = 3u, NIB_STAGES_ONE = 8u;
constexpr uint32_t NIB_TAB_POS = 0x002b1908u, NIB_TAB_NEG = 0x00d5e7f8u;      // bytes 8, 25, 43, 0 and -8, -25, -43, 0

// One warp: 16 rows x one 256-column block (a record in shared memory) against NT 8-column tiles of activation digits.
// Bl: digits of column g of tile 0 at this block's first column + 8 t (tile n is n * 8 * BPITCH further).
template <int NT, uint32_t BPITCH>
__device__ __forceinline__ void nib_chunk(const uint8_t *st, const int8_t *Bl, uint32_t g, uint32_t t, const int (&z)[4], float (&out)[3][4]) {
    const uint32_t o0 = g * 128u + ((2u * t) ^ (g & 1u)) * 16u, o1 = g * 128u + ((2u * t + 1u) ^ (g & 1u)) * 16u;   // rows g and g + 8 have the same parity
    const uint4 qa0 = *reinterpret_cast<const uint4 *>(st + o0), qa1 = *reinterpret_cast<const uint4 *>(st + o1);
    const uint4 qb0 = *reinterpret_cast<const uint4 *>(st + 1024u + o0), qb1 = *reinterpret_cast<const uint4 *>(st + 1024u + o1);
    const uint2 sa = *reinterpret_cast<const uint2 *>(st + NIB_SC_OFF + g * 8u), sb = *reinterpret_cast<const uint2 *>(st + NIB_SC_OFF + (g + 8u) * 8u);
    const float da = 0.125f * __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(st + NIB_D_OFF + g * 2u)));
    const float db = 0.125f * __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(st + NIB_D_OFF + (g + 8u) * 2u)));
    const uint32_t wa[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
    const uint32_t wb[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
    int blk[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { blk[n][0] = blk[n][1] = blk[n][2] = blk[n][3] = 0; }
#pragma unroll
    for (int kg = 0; kg < 8; ++kg) {
        const uint32_t a0 = nb_prmt(NIB_TAB_POS, NIB_TAB_NEG, wa[kg]), a2 = nb_prmt(NIB_TAB_POS, NIB_TAB_NEG, wa[kg] >> 16);
        const uint32_t a1 = nb_prmt(NIB_TAB_POS, NIB_TAB_NEG, wb[kg]), a3 = nb_prmt(NIB_TAB_POS, NIB_TAB_NEG, wb[kg] >> 16);
        const int sca = (int)nb_prmt(kg < 4 ? sa.x : sa.y, 0u, 0x4440u + (uint32_t)(kg & 3));
        const int scb = (int)nb_prmt(kg < 4 ? sb.x : sb.y, 0u, 0x4440u + (uint32_t)(kg & 3));
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const uint2 bf = *reinterpret_cast<const uint2 *>(Bl + (uint32_t)n * 8u * BPITCH + (uint32_t)kg * 32u);
            int d[4];
            nb_mma(d, a0, a1, a2, a3, bf.x, bf.y, z);
            blk[n][0] += sca * d[0]; blk[n][1] += sca * d[1];
            blk[n][2] += scb * d[2]; blk[n][3] += scb * d[3];
        }
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        out[n][0] += da * (float)blk[n][0]; out[n][1] += da * (float)blk[n][1];
        out[n][2] += db * (float)blk[n][2]; out[n][3] += db * (float)blk[n][3];
    }
}

struct NibUnit {
    const uint8_t *rec;        // first record of this warp's tiles in the unit (records of a tile, then of the next tile, are contiguous)
    uint32_t item, p0, nt;     // work item, its first pair in sorted[], its pairs
    uint32_t tile0, n;         // first 16-row tile of this warp and the number of records it streams in the unit
};

// A warp's private ring of STAGES record slots. Records are requested in stream order: first the rest of the
// current unit (cur_*), then the first ones of the next unit (nxt_*), so the ring never drains at a unit boundary.
// Between two reads exactly one request is made, which keeps STAGES - 1 records in flight behind the one being read.
struct NibRing {
    uint32_t stage_s, bar_s;           // shared-memory addresses of slot 0 and of its mbarrier
    uint32_t prod, cons, phase;        // next slot to fill / to read; bit s = parity the next read of slot s waits for
    const uint8_t *cur_src, *nxt_src;
    uint32_t cur_rem, nxt_rem, nxt_taken;
    uint32_t timed_out;
};
template <uint32_t STAGES>
__device__ __forceinline__ void nib_request(NibRing &R, uint32_t lane) {
    const uint8_t *src;
    if (R.cur_rem) { src = R.cur_src; R.cur_src += NIB_REC; --R.cur_rem; }
    else if (R.nxt_rem) { src = R.nxt_src; R.nxt_src += NIB_REC; --R.nxt_rem; ++R.nxt_taken; }
    else return;
    if (lane == 0) nb_fetch(R.stage_s + R.prod * NIB_REC, src, R.bar_s + 8u * R.prod);
    R.prod = R.prod + 1u == STAGES ? 0u : R.prod + 1u;
}
// waits for the oldest record; returns its slot. After a wait ran out no further wait is attempted (the results of the
// launch are void: the caller raises the status word).
__device__ __forceinline__ uint32_t nib_acquire(NibRing &R) {
    const uint32_t slot = R.cons;
    if (!R.timed_out && !nb_wait(R.bar_s + 8u * slot, (R.phase >> slot) & 1u)) R.timed_out = 1u;
    return slot;
}
template <uint32_t STAGES>
__device__ __forceinline__ void nib_release(NibRing &R) {
    __syncwarp();                      // every lane has read the slot: it may be refilled
    R.phase ^= 1u << R.cons;
    R.cons = R.cons + 1u == STAGES ? 0u : R.cons + 1u;
}

// All tiles of one unit for one warp, NT column tiles of digits in use (1: pairs packed into one tile, 3: a tile per digit).
// vals[ti][.] = (row g, pair slot 0), (row g, pair slot 1), (row g + 8, slot 0), (row g + 8, slot 1), times the pair's scale.
template <int NT, uint32_t BPR, uint32_t BPITCH, uint32_t TPW, uint32_t STAGES>
__device__ __forceinline__ void nib_tiles(NibRing &R, const uint8_t *my_stage, const int8_t *Bbase, uint32_t tiles, uint32_t lane, uint32_t g, uint32_t t,
                                          const int (&z)[4], float dw1, float dw2, const float (&sxv)[2], float (&vals)[TPW][4]) {
    for (uint32_t ti = 0; ti < tiles; ++ti) {
        float out[3][4];
#pragma unroll
        for (int n = 0; n < 3; ++n) { out[n][0] = out[n][1] = out[n][2] = out[n][3] = 0.f; }
        for (uint32_t c = 0; c < BPR; ++c) {
            nib_request<STAGES>(R, lane);
            const uint32_t slot = nib_acquire(R);
            nib_chunk<NT, BPITCH>(my_stage + slot * NIB_REC, Bbase + c * 256u, g, t, z, out);
            nib_release<STAGES>(R);
        }
        float v[2][2];                 // [row half][pair slot]
        if (NT == 1) {
            const uint32_t src = (lane & ~3u) + 1u;
            const float x0 = __shfl_sync(0xffffffffu, out[0][0], src), y0 = __shfl_sync(0xffffffffu, out[0][1], src);
            const float x1 = __shfl_sync(0xffffffffu, out[0][2], src), y1 = __shfl_sync(0xffffffffu, out[0][3], src);
            // t == 0: pair 0 = cols 0, 1 (own) and 2 (lane t = 1); t == 2: pair 1 = col 3 (lane t = 1) and cols 4, 5 (own)
            v[0][0] = t == 0u ? out[0][0] + dw1 * out[0][1] + dw2 * x0 : y0 + dw1 * out[0][0] + dw2 * out[0][1];
            v[1][0] = t == 0u ? out[0][2] + dw1 * out[0][3] + dw2 * x1 : y1 + dw1 * out[0][2] + dw2 * out[0][3];
            v[0][1] = v[1][1] = 0.f;
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 2; ++j) v[h][j] = out[0][2 * h + j] + dw1 * out[1][2 * h + j] + dw2 * out[2][2 * h + j];
        }
        vals[ti][0] = v[0][0] * sxv[0]; vals[ti][1] = v[0][1] * sxv[1]; vals[ti][2] = v[1][0] * sxv[0]; vals[ti][3] = v[1][1] * sxv[1];
    }
}

// GATEUP: warps 0-3 take the gate rows of 4 x TPW tiles, warps 4-7 the up rows of the same tiles; the up values cross a
// small shared buffer and the gate warps store SiLU(gate) * up. Otherwise (down projection) 8 x TPW tiles per unit.
template <bool GATEUP, uint32_t NCOLS, uint32_t STAGES>
__global__ void __launch_bounds__(NIB_WARPS * 32u, STAGES == NIB_STAGES_BATCH ? 2 : 1) k_nib_experts(const __grid_constant__ MmaArgs A) {
    pdl_prologue();
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr uint32_t BPR = NCOLS / 256u, TPW = BPR >= 8u ? 1u : 8u / BPR, WSLOTS = GATEUP ? 4u : 8u, UNIT_TILES = WSLOTS * TPW;
    constexpr uint32_t BPITCH = NCOLS + 32u, V16 = NCOLS / 16u;
    __shared__ uint32_t s_unit[2];
    __shared__ volatile uint32_t s_fail;
    __shared__ __align__(8) uint64_t s_bar[NIB_WARPS][STAGES];
    __shared__ __align__(16) float4 s_ex[GATEUP ? TPW : 1u][4][32];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    uint8_t *my_stage = smem + warp * (STAGES * NIB_REC);
    int8_t *Bs = reinterpret_cast<int8_t *>(smem + NIB_WARPS * STAGES * NIB_REC);
    const uint32_t ntile_rows = A.nrows >> 4, U = (ntile_rows + UNIT_TILES - 1u) / UNIT_TILES;
    const uint32_t total = *A.n_items * U;
    const bool is_up = GATEUP && warp >= 4u;
    const uint32_t wslot = GATEUP ? (warp & 3u) : warp;
    const uint8_t *wmat = is_up ? A.w1 : A.w0;
    NibRing R{};
    R.stage_s = nb_smem(my_stage); R.bar_s = nb_smem(&s_bar[warp][0]);

    auto decode = [&](uint32_t unit, NibUnit &I) {
        const uint32_t item = unit / U, rb = unit - item * U;
        const uint32_t u = A.item_u[item], p0 = A.item_p0[item];
        uint32_t e = A.uexp[u] - A.expert_begin, nt = min(A.item_tok, A.ustart[u + 1u] - p0);
        if (e >= A.n_local) { if (A.status && tid == 0) A.status[ST_EXPERT_RANGE] = 1u; e = 0u; nt = 0u; }     // never index the arena with a foreign id
        I.item = item; I.p0 = p0; I.nt = nt;
        I.tile0 = rb * UNIT_TILES + wslot * TPW;
        const uint32_t tiles = I.tile0 >= ntile_rows ? 0u : min(TPW, ntile_rows - I.tile0);
        I.n = nt ? tiles * BPR : 0u;
        I.rec = wmat + (size_t)e * A.mat_bytes + (size_t)I.tile0 * BPR * NIB_REC;
    };

    if (tid == 0) { s_unit[0] = atomicAdd(A.work, 1u); s_fail = 0u; }
    if (lane == 0) {
        for (uint32_t i = 0; i < STAGES; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(R.bar_s + 8u * i));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    __shared__ float s_red[NIB_WARPS], s_sx;
    if (A.x_raw) {
        // single token: every unit multiplies the same activation row, so the block turns it into digits itself (the
        // arithmetic of k_quant_act) — columns 0..2 of the one tile in use, columns 3..7 zero
        float mx = 0.f;
        for (uint32_t k = tid * 4u; k < NCOLS; k += NIB_WARPS * 128u) {
            const float4 v = *reinterpret_cast<const float4 *>(A.x_raw + k);
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) s_red[warp] = mx;
        __syncthreads();
        mx = s_red[0];
        for (uint32_t w = 1; w < NIB_WARPS; ++w) mx = fmaxf(mx, s_red[w]);
        const float qmax = act_qmax(A.act_bits), scale = act_scale(mx, qmax), inv = 1.0f / scale;
        if (tid == 0) s_sx = scale;
        for (uint32_t k = tid * 4u; k < NCOLS; k += NIB_WARPS * 128u) {
            const float4 v = *reinterpret_cast<const float4 *>(A.x_raw + k);
            const float f[4] = {v.x, v.y, v.z, v.w};
            uint32_t p0 = 0, p1 = 0, p2 = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int d0, d1, d2;
                act_digits(f[i], inv, qmax, A.act_bits, d0, d1, d2);
                p0 |= (uint32_t)(d0 & 255) << (8 * i); p1 |= (uint32_t)(d1 & 255) << (8 * i); p2 |= (uint32_t)(d2 & 255) << (8 * i);
            }
            *reinterpret_cast<uint32_t *>(Bs + k) = p0;
            *reinterpret_cast<uint32_t *>(Bs + BPITCH + k) = p1;
            *reinterpret_cast<uint32_t *>(Bs + 2u * BPITCH + k) = p2;
#pragma unroll
            for (uint32_t col = 3u; col < 8u; ++col) *reinterpret_cast<uint32_t *>(Bs + col * BPITCH + k) = 0u;
        }
        __syncthreads();
    }
    uint32_t cur = s_unit[0], par = 0u, cur_item = 0xffffffffu;
    uint32_t ahead = 0u;             // records of the CURRENT unit already requested (while the previous unit was multiplying)
    int zero[4];                     // opaque to the compiler: four registers that stay zero, the accumulator input of every MMA
    asm volatile("mov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;" : "=r"(zero[0]), "=r"(zero[1]), "=r"(zero[2]), "=r"(zero[3]));
    NibUnit I{}, N{};
    if (cur < total) decode(cur, I);
    while (cur < total) {
        if (tid == 0) s_unit[par ^ 1u] = atomicAdd(A.work, 1u);
        // this unit's stream; STAGES - 1 of its records are put in flight before the first read
        R.cur_src = I.rec + (size_t)ahead * NIB_REC; R.cur_rem = I.n - ahead; R.nxt_rem = 0u; R.nxt_taken = 0u;
        for (uint32_t i = ahead; i + 1u < STAGES; ++i) nib_request<STAGES>(R, lane);
        const bool packed = I.nt <= 2u;
        if (!A.x_raw && I.item != cur_item) {    // activation digits of the item (every warp passed the barrier that ended the last unit)
            const uint32_t ncolb = packed ? 8u : 24u;
            for (uint32_t i = tid; i < ncolb * V16; i += NIB_WARPS * 32u) {
                const uint32_t col = i / V16, k = (i - col * V16) << 4;
                const uint32_t tk = packed ? col / 3u : (col & 7u), dg = packed ? col - 3u * (col / 3u) : (col >> 3);
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (tk < I.nt) v = *reinterpret_cast<const uint4 *>(A.xq + ((size_t)(A.sorted[I.p0 + tk] / A.x_div) * 3u + dg) * NCOLS + k);
                *reinterpret_cast<uint4 *>(Bs + (size_t)col * BPITCH + k) = v;
            }
            cur_item = I.item;
        }
        // the pairs this lane stores: packed -> pair t/2 on even t; one tile per digit -> pairs 2t, 2t+1
        uint32_t prow[2] = {0u, 0u};
        float sxv[2] = {0.f, 0.f};
        bool ok[2];
#pragma unroll
        for (uint32_t j = 0; j < 2u; ++j) {
            const uint32_t tk = packed ? (t >> 1) : 2u * t + j;
            ok[j] = packed ? (j == 0u && (t & 1u) == 0u && tk < I.nt) : tk < I.nt;
            if (ok[j]) { prow[j] = A.sorted[I.p0 + tk]; sxv[j] = A.x_raw ? s_sx : A.sx[prow[j] / A.x_div]; }
        }
        __syncthreads();             // digits and the next unit's number are in shared memory
        const uint32_t nxt = s_unit[par ^ 1u];
        const bool nv = nxt < total;
        if (nv) { decode(nxt, N); if (I.n + 1u >= STAGES) { R.nxt_src = N.rec; R.nxt_rem = N.n; } }     // a unit shorter than the ring does not look ahead

        float vals[TPW][4];
        const uint32_t tiles = I.n / BPR;
        const int8_t *Bbase = Bs + (size_t)g * BPITCH + 8u * t;
        if (packed) nib_tiles<1, BPR, BPITCH, TPW, STAGES>(R, my_stage, Bbase, tiles, lane, g, t, zero, A.dw1, A.dw2, sxv, vals);
        else nib_tiles<3, BPR, BPITCH, TPW, STAGES>(R, my_stage, Bbase, tiles, lane, g, t, zero, A.dw1, A.dw2, sxv, vals);
        if (R.timed_out && lane == 0) { s_fail = 1u; if (A.status) A.status[ST_TIMEOUT] = 1u; }
        if (GATEUP) {
            if (is_up) for (uint32_t ti = 0; ti < tiles; ++ti) s_ex[ti][wslot][lane] = make_float4(vals[ti][0], vals[ti][1], vals[ti][2], vals[ti][3]);
        } else {
            for (uint32_t ti = 0; ti < tiles; ++ti) {
                const uint32_t row = ((I.tile0 + ti) << 4) + g;
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    if (ok[j]) {
                        A.out[(size_t)prow[j] * A.out_stride + row] = vals[ti][j];
                        A.out[(size_t)prow[j] * A.out_stride + row + 8u] = vals[ti][2 + j];
                    }
            }
        }
        __syncthreads();             // the unit is done in every warp: up values are in s_ex, the digits may be replaced
        const bool fail = s_fail != 0u;      // written only between the two barriers of a unit, read only here: every warp sees the same value
        if (GATEUP && !is_up) {
            for (uint32_t ti = 0; ti < tiles; ++ti) {
                const float4 up = s_ex[ti][wslot][lane];
                const float uv[4] = {up.x, up.y, up.z, up.w};
                const uint32_t row = ((I.tile0 + ti) << 4) + g;
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    if (ok[j]) {
                        const float g0 = vals[ti][j], g1 = vals[ti][2 + j];
                        A.out[(size_t)prow[j] * A.out_stride + row] = (g0 / (1.0f + expf(-g0))) * uv[j];
                        A.out[(size_t)prow[j] * A.out_stride + row + 8u] = (g1 / (1.0f + expf(-g1))) * uv[2 + j];
                    }
            }
        }
        if (fail) break;             // some warp's copy never arrived (status word raised): stop drawing units
        ahead = R.nxt_taken;
        cur = nxt; I = N; par ^= 1u;
    }
}

// ---- single token: down projection of the selected experts + shared expert's down rows + weighted sum + residual ----
// grid = nrows / 16 (one 16-row tile per block), block = top_k + 2 warps: warp k < top_k takes expert k (its tile's
// records arrive by bulk copy while the warp quantises expert k's activation row), the last two warps take the shared
// expert's 16 rows (Q6_K, CUDA cores). Partial rows meet in shared memory and are summed in router order.
constexpr uint32_t NIB_TAIL_MAX_K = 14u;
template <uint32_t NCOLS>
__global__ void __launch_bounds__((NIB_TAIL_MAX_K + 2u) * 32u) k_nib_down_tail(const __grid_constant__ NibTailArgs A) {
    pdl_prologue();
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr uint32_t BPR = NCOLS / 256u, BPITCH = NCOLS + 32u, PER_LANE = NCOLS / 32u;
    __shared__ __align__(8) uint64_t s_bar[NIB_TAIL_MAX_K];
    __shared__ float s_part[NIB_TAIL_MAX_K][16], s_sh[16];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u, K = A.top_k;
    uint8_t *recs = smem;                                                    // [K][BPR] records
    int8_t *digits = reinterpret_cast<int8_t *>(smem + K * BPR * NIB_REC);   // [K][3][BPITCH]
    int8_t *zrow = digits + K * 3u * BPITCH;                                 // one row of zeros: digit columns 3..7 of every tile
    float *xs = reinterpret_cast<float *>(zrow + BPITCH);                    // shared expert's activation, padded rows of redcuda_dot.cuh
    const uint32_t row0 = blockIdx.x * 16u;

    for (uint32_t k = tid * 4u; k < BPITCH; k += blockDim.x * 4u) *reinterpret_cast<uint32_t *>(zrow + k) = 0u;
    if (A.sh_down) for (uint32_t k = tid * 4u; k < NCOLS; k += blockDim.x * 4u) *reinterpret_cast<float4 *>(xs + xi(k)) = *reinterpret_cast<const float4 *>(A.sh_act + k);
    if (tid < 16u) s_sh[tid] = 0.f;
    if (warp < K && lane == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(nb_smem(&s_bar[warp])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (warp < K) {
        uint32_t e = A.ids[warp] - A.expert_begin;
        bool live = true;
        if (e >= A.n_local) { if (A.status && lane == 0) A.status[ST_EXPERT_RANGE] = 1u; e = 0u; live = false; }      // never index the arena with a foreign id
        uint8_t *my_rec = recs + warp * BPR * NIB_REC;
        const uint32_t bar = nb_smem(&s_bar[warp]);
        if (lane == 0) {
            const uint8_t *src = A.w_down + (size_t)e * A.mat_bytes + (size_t)blockIdx.x * BPR * NIB_REC;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(BPR * NIB_REC) : "memory");
            for (uint32_t c = 0; c < BPR; ++c)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             :: "r"(nb_smem(my_rec + c * NIB_REC)), "l"(src + (size_t)c * NIB_REC), "r"(NIB_REC), "r"(bar) : "memory");
        }
        // this expert's activation row -> digits (the arithmetic of k_quant_act), while the records are in flight
        const float *ar = A.act + (size_t)warp * A.act_stride;
        float v[PER_LANE];
        float mx = 0.f;
#pragma unroll
        for (uint32_t i = 0; i < PER_LANE / 4u; ++i) {
            const float4 q = *reinterpret_cast<const float4 *>(ar + lane * 4u + 128u * i);
            v[4 * i] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(q.x), fabsf(q.y)), fmaxf(fabsf(q.z), fabsf(q.w))));
        }
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float qmax = act_qmax(A.bits), sx = act_scale(mx, qmax), inv = 1.0f / sx;
        int8_t *mine = digits + warp * 3u * BPITCH;
#pragma unroll
        for (uint32_t i = 0; i < PER_LANE / 4u; ++i) {
            uint32_t p0 = 0, p1 = 0, p2 = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int d0, d1, d2;
                act_digits(v[4 * i + j], inv, qmax, A.bits, d0, d1, d2);
                p0 |= (uint32_t)(d0 & 255) << (8 * j); p1 |= (uint32_t)(d1 & 255) << (8 * j); p2 |= (uint32_t)(d2 & 255) << (8 * j);
            }
            const uint32_t k = lane * 4u + 128u * i;
            *reinterpret_cast<uint32_t *>(mine + k) = p0;
            *reinterpret_cast<uint32_t *>(mine + BPITCH + k) = p1;
            *reinterpret_cast<uint32_t *>(mine + 2u * BPITCH + k) = p2;
        }
        __syncwarp();
        if (!__all_sync(0xffffffffu, nb_wait(bar, 0u))) { live = false; if (A.status && lane == 0) A.status[ST_TIMEOUT] = 1u; }
        float out[3][4];
#pragma unroll
        for (int n = 0; n < 3; ++n) { out[n][0] = out[n][1] = out[n][2] = out[n][3] = 0.f; }
        int zero[4];
        asm volatile("mov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;" : "=r"(zero[0]), "=r"(zero[1]), "=r"(zero[2]), "=r"(zero[3]));
        const int8_t *Bl = (g < 3u ? mine + g * BPITCH : zrow) + 8u * t;       // columns 0..2 = the pair's three digits, the rest of the tile is zero
        if (live) for (uint32_t c = 0; c < BPR; ++c) nib_chunk<1, BPITCH>(my_rec + c * NIB_REC, Bl + c * 256u, g, t, zero, out);
        const uint32_t src = (lane & ~3u) + 1u;
        const float x0 = __shfl_sync(0xffffffffu, out[0][0], src), x1 = __shfl_sync(0xffffffffu, out[0][2], src);
        if (t == 0u) {
            s_part[warp][g] = (out[0][0] + A.dw1 * out[0][1] + A.dw2 * x0) * sx;
            s_part[warp][g + 8u] = (out[0][2] + A.dw1 * out[0][3] + A.dw2 * x1) * sx;
        }
    } else if (A.sh_down) {
        const uint32_t sw = warp - K;                                       // 0 or 1: rows 8 sw .. 8 sw + 7 of the tile
        uint32_t lpr = 32u;
        while (lpr > (NCOLS >> 6)) lpr >>= 1;
        const uint32_t rw = 32u / lpr, slot = lane / lpr, sub = lane % lpr;
        const SBooks sb{nullptr, nullptr};
        for (uint32_t r = 0; r < 8u; r += rw) {
            const uint32_t rr = 8u * sw + r + slot;                         // rw <= 8 for every row length from 256 up
            float a[1];
            row_dot<RC_Q6_K, 1>(A.sh_down, A.sh_nb, (uint64_t)(row0 + rr), NCOLS, lpr, sub, xs, x_padded(NCOLS), sb, a);
            if (sub == 0u) s_sh[rr] = a[0];
        }
    }
    __syncthreads();
    if (tid < 16u) {
        const uint32_t row = row0 + tid;
        float acc = 0.f;
        for (uint32_t k = 0; k < K; ++k) { const float wk = A.wk[k]; if (wk != 0.f) acc += wk * s_part[k][tid]; }
        if (A.sh_down) acc += s_sh[tid] * (A.scalar ? A.scalar[0] : 1.0f);
        if (A.resid) acc += A.resid[row];
        A.out[row] = acc;
    }
}

bool nib_tail_ok(uint32_t top_k, uint32_t nrows, uint32_t ncols) {
    return top_k >= 1u && top_k <= NIB_TAIL_MAX_K && nrows % 16u == 0 && (ncols == 256u || ncols == 512u || ncols == 1024u);
}

int launch_nib_down_tail(NibTailArgs &A, cudaStream_t s) {
    RC_REQUIRE(nib_tail_ok(A.top_k, A.nrows, A.ncols), "nibble down tail: top_k %u, %ux%u is not a shape it serves", A.top_k, A.nrows, A.ncols);
    A.bits = act_digit_bits(); A.dw1 = (float)(1u << A.bits); A.dw2 = A.dw1 * A.dw1;
    const uint32_t bpr = A.ncols / 256u, bpitch = A.ncols + 32u;
    const size_t smem = (size_t)A.top_k * bpr * NIB_REC + (size_t)A.top_k * 3u * bpitch + bpitch + (size_t)x_padded(A.ncols) * 4u + 16u;
    const uint32_t threads = (A.top_k + 2u) * 32u, grid = A.nrows / 16u;
    prof_begin("moe_down_tail", s);
#define RC_TAIL_LAUNCH(NC) do { \
        RC_CUDA(cudaFuncSetAttribute(k_nib_down_tail<NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        RC_LAUNCH((k_nib_down_tail<NC>), grid, threads, smem, s, A); } while (0)
    if (A.ncols == 256u) RC_TAIL_LAUNCH(256u); else if (A.ncols == 512u) RC_TAIL_LAUNCH(512u); else RC_TAIL_LAUNCH(1024u);
#undef RC_TAIL_LAUNCH
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

static size_t nib_smem_bytes(uint32_t ncols, uint32_t stages) { return (size_t)NIB_WARPS * stages * NIB_REC + 24u * (size_t)(ncols + 32u); }

// A.w0 / A.w1: nibble-layout expert matrices (gate and up, or down and nullptr); A.work: the unit counter of this launch
// (zeroed by the grouping kernel); items are cut with at most 8 pairs. max_items bounds the number of work items.
int launch_nib_experts(MmaArgs &A, uint32_t max_items, cudaStream_t s) {
    const bool gateup = A.w1 != nullptr;
    RC_REQUIRE(nib_shape_ok(A.nrows, A.ncols), "nibble experts: matrix %ux%u is not tileable", A.nrows, A.ncols);
    RC_REQUIRE(A.work != nullptr && A.item_tok >= 1u && A.item_tok <= 8u, "nibble experts: work counter missing or items of %u pairs", A.item_tok);
    A.act_bits = act_digit_bits(); A.dw1 = (float)(1u << A.act_bits); A.dw2 = A.dw1 * A.dw1;
    RC_REQUIRE(!A.x_raw || (gateup && A.item_tok == 1u), "nibble experts: in-kernel quantisation serves the gate/up of a single token");
    static int sm_count = 0;
    if (!sm_count) { int dev = 0; RC_CUDA(cudaGetDevice(&dev)); RC_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev)); }
    const uint32_t bpr = A.ncols / 256u, tpw = bpr >= 8u ? 1u : 8u / bpr, unit_tiles = (gateup ? 4u : 8u) * tpw;
    const uint64_t units = (uint64_t)max_items * ((A.nrows / 16u + unit_tiles - 1u) / unit_tiles);
    const bool one = A.x_raw != nullptr;          // single token: deep rings, one block per SM
    const uint32_t per_sm = one ? 1u : 2u, stages = one ? NIB_STAGES_ONE : NIB_STAGES_BATCH;
    const uint32_t grid = (uint32_t)(units < per_sm * (uint64_t)sm_count ? (units ? units : 1u) : per_sm * (uint64_t)sm_count);
    const size_t smem = nib_smem_bytes(A.ncols, stages);
    prof_begin(gateup ? "moe_gateup" : "moe_down", s);
#define RC_NIB_LAUNCH(GU, NC, ST) do { \
        RC_CUDA(cudaFuncSetAttribute(k_nib_experts<GU, NC, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        RC_LAUNCH((k_nib_experts<GU, NC, ST>), grid, NIB_WARPS * 32u, smem, s, A); } while (0)
    if (one) {
        if (A.ncols == 2048u) RC_NIB_LAUNCH(true, 2048u, NIB_STAGES_ONE); else if (A.ncols == 1024u) RC_NIB_LAUNCH(true, 1024u, NIB_STAGES_ONE);
        else if (A.ncols == 512u) RC_NIB_LAUNCH(true, 512u, NIB_STAGES_ONE); else RC_NIB_LAUNCH(true, 256u, NIB_STAGES_ONE);
    } else if (gateup) {
        if (A.ncols == 2048u) RC_NIB_LAUNCH(true, 2048u, NIB_STAGES_BATCH); else if (A.ncols == 1024u) RC_NIB_LAUNCH(true, 1024u, NIB_STAGES_BATCH);
        else if (A.ncols == 512u) RC_NIB_LAUNCH(true, 512u, NIB_STAGES_BATCH); else RC_NIB_LAUNCH(true, 256u, NIB_STAGES_BATCH);
    } else {
        if (A.ncols == 2048u) RC_NIB_LAUNCH(false, 2048u, NIB_STAGES_BATCH); else if (A.ncols == 1024u) RC_NIB_LAUNCH(false, 1024u, NIB_STAGES_BATCH);
        else if (A.ncols == 512u) RC_NIB_LAUNCH(false, 512u, NIB_STAGES_BATCH); else RC_NIB_LAUNCH(false, 256u, NIB_STAGES_BATCH);
    }
#undef RC_NIB_LAUNCH
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

}  // namespace rc

using namespace rc;

// Host-buffer check of the layout: raw IQ2_XXS GGUF rows -> planar -> nibble layout -> fp32. Must equal
// redcuda_quant_dequant_rows (and rl_quant_dequant_row) bit for bit.
extern "C" int redcuda_nib_dequant_rows(const uint8_t *rows, uint32_t nrows, uint32_t ncols, float *out) {
    if (!require_device() || !require_books(RC_IQ2_XXS)) return 0;
    RC_REQUIRE(rows && out, "nib dequant: null argument");
    RC_REQUIRE(nib_shape_ok(nrows, ncols), "nib dequant: matrix %ux%u is not tileable (16 rows, 256/512/1024/2048 columns)", nrows, ncols);
    const uint64_t bytes = rc_matrix_bytes(RC_IQ2_XXS, nrows, ncols), nb = (uint64_t)nrows * (ncols / 256u);
    DevMem raw, planar, nib, o;
    if (!raw.alloc(bytes) || !planar.alloc(bytes) || !nib.alloc(nib_matrix_bytes(nrows, ncols)) || !o.alloc((size_t)nrows * ncols * 4u)) return 0;
    cudaStream_t s = 0;
    if (!upload_matrix(RC_IQ2_XXS, nrows, ncols, rows, false, planar.as<uint8_t>(), raw.as<uint8_t>(), s)) return 0;
    if (!launch_nib_repack(planar.as<uint8_t>(), nrows, ncols, nib.as<uint8_t>(), s)) return 0;
    const uint64_t total = nb * 32u;
    RC_LAUNCH((k_nib_dequant), (unsigned)((total + 255u) / 256u < 4096u ? (total + 255u) / 256u : 4096u), 256, 0, s, nib.as<uint8_t>(), nb, nrows, ncols / 256u, o.as<float>());
    RC_LAUNCHED();
    RC_CUDA(cudaMemcpyAsync(out, o.p, (size_t)nrows * ncols * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    return 1;
}
