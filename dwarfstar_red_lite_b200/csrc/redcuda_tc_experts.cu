// Routed experts of a prefill chunk on the 5th-generation tensor cores (tcgen05): for every work item (up to 64 pairs of
// one expert) and every 128-row tile of the expert's matrix, out[pair][row] = sum_k W_e[row][k] * x[pair][k].
//
// The batched form of the expert GEMV (rl_quant_row_dot per row, native/redlite_native_quant_cpu.c:247-266, called per
// selected expert by the MoE layer, native/redlite_native_moe.c); the reference's chunked prefill groups the chunk's
// tokens by expert and runs one matrix product per expert (native/redmetal_engine_prefill.m:889-909).
//
// Operands. The experts are held in the nibble layout (redcuda_moe_mma.cuh): a weight is d/8 * (2s+1) * (+-8|25|43) with
// d the fp16 scale of its 256-block and s the 4-bit scale of its 32-group. The integer (2s+1) * (+-m) is at most 1333, so
// it is ONE exact fp16 value: the weight operand needs a single digit, built with two byte permutes and one half2 FMA
// per pair of weights, and d/8 multiplies the fp32 sum of each 256-column block when it is drained. Activations are two
// fp16 digits (hi + lo, 22 significant bits, power-of-two scale per row), prepared once per row by k_tc_prep_rows; the
// digit rows of an item's pairs are gathered straight into the MMA's core-matrix layout with 16-byte cp.async pieces, so
// a token that goes to ten experts is stored once.
// Accumulation follows k_tc_gemm: the tensor core adds into fp32 without rounding to nearest, so the accumulators cover
// one 256-column block only (one for A*hi, one for A*lo), double-buffered in tensor memory and summed in fp32 registers.
//
// One CTA = one item x one 128-row tile of one matrix, K in stages of 64 columns:
//   thread 0      requests the 8 records (16 rows x 256 columns each) of the next block with cp.async.bulk on an mbarrier
//   all 16 warps  gather the next stage's activation pieces, decode 128 x 64 weights of this stage from the records
//   thread 0      issues 4 k-steps x 2 tcgen05.mma (128 x 64 x 16, kind::f16) and commits on the stage's mbarrier
// Blocks beyond the item count leave at once. Every wait is bounded: on a timeout the CTA stops issuing, waits (bounded)
// for its own copies, frees its tensor memory, raises the launch's flag and the sticky status word, and returns.
#define RC_PDL_DEFAULT 0
#include "redcuda_common.cuh"
#include "redcuda_dot.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_moe_mma.cuh"
#include "redcuda_tc_gemm.cuh"

#include <cuda_fp16.h>
#include <stdlib.h>

namespace rc {

constexpr uint32_t TCX_RAW = 8u * NIB_REC;                // records of one 256-column block of a 128-row tile
constexpr uint32_t TCX_DEAD = 0xffffffffu;
// biased byte tables of the 4-bit codes: 128 + (8, 25, 43, 0) and 128 - (8, 25, 43, 0)
constexpr uint32_t TCX_TAB_POS = 0x80ab9988u, TCX_TAB_NEG = 0x80556778u;

__device__ __forceinline__ uint32_t tcx_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// 8 codes (one word) times the group's integer scale -> 8 exact fp16 values. A code selects a biased byte u = 128 + w;
// 0x6400 | u is the fp16 number 1024 + u, and (1024 + u) * sc - 1152 * sc = w * sc with one rounding of an exact integer.
__device__ __forceinline__ uint4 tcx_decode8(uint32_t word, uint32_t sc) {
    const __half2 hs = __half2half2(__ushort2half_rn((unsigned short)sc));
    const __half2 hb = __hmul2(hs, __float2half2_rn(-1152.0f));
    const uint32_t b0 = tcx_prmt(TCX_TAB_POS, TCX_TAB_NEG, word), b1 = tcx_prmt(TCX_TAB_POS, TCX_TAB_NEG, word >> 16);
    uint32_t h[4] = {tcx_prmt(b0, 0x64646464u, 0x5140u), tcx_prmt(b0, 0x64646464u, 0x5342u), tcx_prmt(b1, 0x64646464u, 0x5140u), tcx_prmt(b1, 0x64646464u, 0x5342u)};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __half2 v = __hfma2(*reinterpret_cast<const __half2 *>(&h[j]), hs, hb);
        h[j] = *reinterpret_cast<const uint32_t *>(&v);
    }
    return make_uint4(h[0], h[1], h[2], h[3]);
}

// v[r][k] (optionally SiLU(a) * b) -> two fp16 digits per value, rows kept row-major: xd[r][digit][ncols]; x_inv[r]
// undoes the row's power-of-two scale. grid = rows, block = 256
__global__ void __launch_bounds__(256) k_tc_prep_rows(const float *__restrict__ a, const float *__restrict__ b, uint32_t stride, uint32_t ncols,
                                                      __half *__restrict__ xd, float *__restrict__ x_inv) {
    pdl_prologue();
    __shared__ float red[8];
    const uint32_t r = blockIdx.x, tid = threadIdx.x;
    const float *ar = a + (size_t)r * stride, *br = b ? b + (size_t)r * stride : nullptr;
    float mx = 0.f;
    for (uint32_t k = tid; k < ncols; k += 256u) mx = fmaxf(mx, fabsf(br ? silu_mul(ar[k], br[k]) : ar[k]));
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((tid & 31u) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = 0.f;
    for (uint32_t w = 0; w < 8u; ++w) mx = fmaxf(mx, red[w]);
    int e = 0;
    if (mx > 0.f && mx < INFINITY) { int ex; frexpf(mx, &ex); e = 14 - ex; }     // max |v| * 2^e in [2^13, 2^14)
    e = e > 100 ? 100 : e < -100 ? -100 : e;
    const float sc = exp2f((float)e);
    if (tid == 0) x_inv[r] = exp2f((float)-e);
    __half *hi = xd + (size_t)r * 2u * ncols, *lo = hi + ncols;
    for (uint32_t c = tid; c < ncols / 8u; c += 256u) {
        __half h[8], l[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t k = c * 8u + j;
            const float v = (br ? silu_mul(ar[k], br[k]) : ar[k]) * sc;
            h[j] = __float2half_rn(v);
            l[j] = __float2half_rn(v - __half2float(h[j]));
        }
        *reinterpret_cast<uint4 *>(hi + c * 8u) = *reinterpret_cast<const uint4 *>(h);
        *reinterpret_cast<uint4 *>(lo + c * 8u) = *reinterpret_cast<const uint4 *>(l);
    }
}

// LA = how many stages ahead the activation pieces are requested (LA + 2 stage buffers)
template <int TN, int LA>
__global__ void __launch_bounds__(TC_THREADS, 1) k_tc_experts(const __grid_constant__ TcxArgs A) {
    pdl_prologue();
    const uint32_t item = blockIdx.y;
    if (item >= *A.n_items) return;                       // the grid covers the largest possible item count
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t NB = (uint32_t)LA + 2u;
    constexpr uint32_t B_DIGIT = (uint32_t)TN * TC_KS * 2u, A_BUF = TC_A_DIGIT, B_BUF = 2u * B_DIGIT;
    constexpr uint32_t TMEM_COLS = 4u * (uint32_t)TN;     // two blocks in flight x (A*hi accumulator, A*lo accumulator)
    static_assert(TMEM_COLS >= 32u && TMEM_COLS <= 512u && (TMEM_COLS & (TMEM_COLS - 1u)) == 0u, "tensor-memory allocation must be a power of two in [32, 512]");
    __shared__ __align__(8) uint64_t mbar[2];        // MMAs that read A buffer b (and the activation buffer of the same stage) are done
    __shared__ __align__(8) uint64_t accfull[2];     // every MMA of a 256-column block has landed in accumulator pair b
    __shared__ __align__(8) uint64_t rawfull[2];     // the records of a 256-column block have landed in raw buffer b
    __shared__ uint32_t tmem_slot;
    __shared__ volatile uint32_t fail;               // a bounded wait ran out: no more MMAs are issued, later waits are skipped
    __shared__ uint32_t s_row[TN], s_pair[TN];       // activation row and pair of every token slot of the item (TCX_DEAD beyond its pairs)
    __shared__ float s_xinv[TN], s_d[2][TC_M];       // inverse activation scales; d/8 of every row for the two blocks in flight
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;

    const uint32_t u = A.item_u[item], p0 = A.item_p0[item], pe = A.ustart[u + 1u];
    const uint32_t nt = pe - p0 < (uint32_t)TN ? pe - p0 : (uint32_t)TN;
    uint32_t e = A.uexp[u] - A.expert_begin;
    if (e >= A.n_local) {                                 // cannot happen with k_group_pairs' output; never an address
        if (tid == 0 && A.status) A.status[ST_EXPERT_RANGE] = 1u;
        return;
    }
    const uint32_t rtiles = A.nrows / TC_M, mat = blockIdx.x / rtiles, rt = blockIdx.x - mat * rtiles;
    const uint32_t bpr = A.ncols >> 8, nstage = A.ncols / TC_KS;
    const uint8_t *wrec = A.w[mat] + (uint64_t)e * A.mat_bytes + (uint64_t)(rt * 8u) * bpr * NIB_REC;     // record (tile 8 rt + j, block c) at (j * bpr + c) * NIB_REC
    uint8_t *a_base = smem, *b_base = smem + 2u * A_BUF, *raw_base = b_base + NB * B_BUF;

    if (tid < (uint32_t)TN) {
        uint32_t row = TCX_DEAD, pair = TCX_DEAD; float inv = 0.f;
        if (tid < nt) { pair = A.sorted[p0 + tid]; row = pair / A.x_div; inv = A.x_inv[row]; }
        s_row[tid] = row; s_pair[tid] = pair; s_xinv[tid] = inv;
    }
    // the 8 records of block column c -> raw buffer c & 1 (thread 0)
    auto issue_raw = [&](uint32_t c) {
        const uint32_t bar = smem_u32(&rawfull[c & 1u]), dst = smem_u32(raw_base + (c & 1u) * TCX_RAW);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(TCX_RAW) : "memory");
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         :: "r"(dst + j * NIB_REC), "l"(wrec + ((uint64_t)j * bpr + c) * NIB_REC), "r"(NIB_REC), "r"(bar) : "memory");
    };
    if (tid == 0) {
        fail = 0u;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&mbar[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&mbar[1])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&accfull[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&accfull[1])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&rawfull[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&rawfull[1])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue_raw(0u);
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    const uint32_t idesc = tc_idesc((uint32_t)TN);

    // the activation digits of a stage: 16-byte pieces of the item's rows into the core-matrix layout
    // [digit][k chunk of 8][token group of 8][token in group][8 halves]; slots beyond the item's pairs are zero-filled
    auto issue_b = [&](uint32_t stage) {
        const uint32_t bb = smem_u32(b_base + (stage % NB) * B_BUF);
#pragma unroll
        for (uint32_t i = tid; i < 16u * (uint32_t)TN; i += TC_THREADS) {
            const uint32_t kc = i & 7u, tt = (i >> 3) & ((uint32_t)TN - 1u), dg = i / (8u * (uint32_t)TN);
            const uint32_t row = s_row[tt], live = row != TCX_DEAD ? 16u : 0u;
            const __half *src = A.xd + ((size_t)(live ? row : 0u) * 2u + dg) * A.ncols + stage * TC_KS + kc * 8u;
            const uint32_t dst = bb + dg * B_DIGIT + (kc * ((uint32_t)TN >> 3) + (tt >> 3)) * 128u + (tt & 7u) * 16u;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(live) : "memory");
        }
    };
#pragma unroll
    for (uint32_t st = 0; st < (uint32_t)LA; ++st) {
        if (st < nstage) issue_b(st);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    // fp32 sums over the 256-column blocks: warp w owns TMEM lanes 32*(w%4)..+31 (its quarter) and PER token columns
    constexpr uint32_t PER = (uint32_t)TN / (TC_WARPS / 4u);
    const uint32_t qlane = (warp & 3u) * 32u, c_begin = (warp >> 2) * PER;
    float acc[PER];
#pragma unroll
    for (uint32_t j = 0; j < PER; ++j) acc[j] = 0.f;
    auto drain = [&](uint32_t blk) {
        if (fail) return;
        if (!mbar_wait(smem_u32(&accfull[blk & 1u]), (blk >> 1) & 1u)) { fail = 1u; return; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float dsc = s_d[blk & 1u][qlane + lane];
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
            for (int j = 0; j < 8; ++j) acc[c + j] = fmaf(dsc, __uint_as_float(m[j]) + __uint_as_float(x[j]), acc[c + j]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");     // the pair is overwritten two blocks later, after barriers
    };

    uint32_t raw_issued = 1u, raw_waited = 0u;           // thread 0's count of block requests; every thread's count of completed waits
    for (uint32_t s = 0; s < nstage; ++s) {
        const uint32_t b = s & 1u, c = s >> 2;
        uint8_t *abuf = a_base + b * A_BUF;
        const uint8_t *raw = raw_base + (c & 1u) * TCX_RAW;
        if ((s & 3u) == 0u) {
            // new block column. Its records were requested a block ago; the other raw buffer was last read in the stage
            // before this one, which ended with a barrier, so the next block can be requested into it now
            if (!fail) { if (!mbar_wait(smem_u32(&rawfull[c & 1u]), (c >> 1) & 1u)) fail = 1u; else raw_waited = c + 1u; }
            if (tid == 0 && c + 1u < bpr && !fail) { issue_raw(c + 1u); raw_issued = c + 2u; }
            if (tid < TC_M) s_d[c & 1u][tid] = 0.125f * __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(raw + (tid >> 4) * NIB_REC + NIB_D_OFF + (tid & 15u) * 2u)));
        }
        // the MMAs of stage s - 2 read this A buffer and the activation buffer that stage s + LA will use
        if (s >= 2u && !fail) {
            if (!mbar_wait(smem_u32(&mbar[b]), ((s >> 1) - 1u) & 1u)) fail = 1u;
        }
        if (s + (uint32_t)LA < nstage) issue_b(s + (uint32_t)LA);
        asm volatile("cp.async.commit_group;" ::: "memory");                 // one group per stage, empty at the end
        if ((s & 3u) == 1u && s >= 4u) drain((s >> 2) - 1u);                  // the previous block's MMAs were issued more than a stage ago
        // ---- weights of the stage: thread -> row 8 * warp + lane / 4, code words (t, kg0) and (t, kg0 + 1), t = lane % 4
        if (!fail) {
            const uint32_t r = warp * 8u + (lane >> 2), t = lane & 3u, kg0 = 2u * (s & 3u);
            const uint8_t *rec = raw + (r >> 4) * NIB_REC;
            const uint32_t rr = r & 15u;
            const uint2 wd = *reinterpret_cast<const uint2 *>(rec + nib_code_off(rr, t, kg0));
            const uint32_t sc2 = *reinterpret_cast<const unsigned short *>(rec + NIB_SC_OFF + rr * 8u + kg0);
            // k chunk of 8 inside the stage: columns 32 (kg - kg0) + 8 t  ->  chunk 4 (kg - kg0) + t
            *reinterpret_cast<uint4 *>(abuf + t * (TC_M * 16u) + r * 16u) = tcx_decode8(wd.x, sc2 & 255u);
            *reinterpret_cast<uint4 *>(abuf + (t + 4u) * (TC_M * 16u) + r * 16u) = tcx_decode8(wd.y, sc2 >> 8);
        }
        asm volatile("cp.async.wait_group %0;" :: "n"(LA) : "memory");       // this stage's activation pieces (those of the next LA stages may be in flight)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");         // generic-proxy writes -> visible to the tensor core
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && !fail) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_d = smem_u32(abuf), b_hi = smem_u32(b_base + (s % NB) * B_BUF), b_lo = b_hi + B_DIGIT;
            constexpr uint32_t A_LBO = TC_M * 16u, B_LBO = (uint32_t)TN * 16u, SBO = 128u;
            const uint32_t d_main = tmem + (c & 1u) * 2u * (uint32_t)TN, d_cross = d_main + (uint32_t)TN;
#pragma unroll
            for (uint32_t kk = 0; kk < TC_KS / 16u; ++kk) {
                const uint64_t da = tc_smem_desc(a_d + 2u * kk * A_LBO, A_LBO, SBO);
                const uint64_t dbh = tc_smem_desc(b_hi + 2u * kk * B_LBO, B_LBO, SBO), dbl = tc_smem_desc(b_lo + 2u * kk * B_LBO, B_LBO, SBO);
                const uint32_t first = ((s & 3u) | kk) ? 1u : 0u;       // a block's first MMA overwrites its accumulators
                tc_mma(d_main, da, dbh, idesc, first);
                tc_mma(d_cross, da, dbl, idesc, first);
            }
            tc_commit(smem_u32(&mbar[b]));
            if ((s & 3u) == 3u) tc_commit(smem_u32(&accfull[c & 1u]));
        }
    }
    __syncthreads();
    drain((nstage >> 2) - 1u);
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    if (!fail) {
        const uint32_t row = rt * TC_M + qlane + lane;
        float *out = A.out[mat];
#pragma unroll
        for (uint32_t j = 0; j < PER; ++j) {
            const uint32_t pair = s_pair[c_begin + j];
            if (pair != TCX_DEAD) out[(size_t)pair * A.out_stride + row] = acc[j] * s_xinv[c_begin + j];
        }
    } else {
        if (tid == 0) {
            // a block request that was never waited for may still be writing into this CTA's shared memory
            for (uint32_t c = raw_waited; c < raw_issued; ++c) mbar_wait(smem_u32(&rawfull[c & 1u]), (c >> 1) & 1u);
            atomicExch(A.err, 1u);
            if (A.status) A.status[ST_TIMEOUT] = 1u;
        }
        __syncthreads();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(TMEM_COLS) : "memory");
}

bool tcx_shape_ok(uint32_t nrows, uint32_t ncols) { return nrows % TC_M == 0 && nrows && (ncols == 256u || ncols == 512u || ncols == 1024u || ncols == 2048u); }

int launch_tc_prep_rows(const float *a, const float *b, uint32_t stride, uint32_t nrows, uint32_t ncols, __half *xd, float *x_inv, cudaStream_t s) {
    RC_REQUIRE(ncols % TC_KS == 0 && nrows, "tc experts: %u columns is not a multiple of %u, or no rows", ncols, TC_KS);
    prof_begin(b ? "tcx_prep_act" : "tcx_prep_x", s);
    RC_LAUNCH((k_tc_prep_rows), nrows, 256, 0, s, a, b, stride, ncols, xd, x_inv);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

int launch_tc_experts(TcxArgs &A, uint32_t max_items, const char *tag, cudaStream_t s) {
    RC_REQUIRE(tcx_shape_ok(A.nrows, A.ncols), "tc experts: matrix %ux%u is not tileable (128 rows, 256/512/1024/2048 columns)", A.nrows, A.ncols);
    RC_REQUIRE((A.nmat == 1u || A.nmat == 2u) && A.w[0] && (A.nmat == 1u || A.w[1]) && max_items && A.x_div, "tc experts: bad matrix count or empty launch");
    RC_REQUIRE(max_items <= 65535u, "tc experts: %u work items exceed the grid", max_items);
    constexpr uint32_t TN = TCX_TN;
    static const int la = getenv("RC_TCX_LA") ? atoi(getenv("RC_TCX_LA")) : 2;      // A/B switch: 1 or 2 stages of lookahead
    const size_t smem = 2u * (size_t)TC_A_DIGIT + (size_t)(la == 1 ? 3u : 4u) * 2u * TN * TC_KS * 2u + 2u * (size_t)TCX_RAW;
    const dim3 grid(A.nmat * (A.nrows / TC_M), max_items);
    prof_begin(tag, s);
    if (la == 1) {
        RC_CUDA(cudaFuncSetAttribute(k_tc_experts<(int)TN, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        RC_LAUNCH((k_tc_experts<(int)TN, 1>), grid, TC_THREADS, smem, s, A);
    } else {
        RC_CUDA(cudaFuncSetAttribute(k_tc_experts<(int)TN, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        RC_LAUNCH((k_tc_experts<(int)TN, 2>), grid, TC_THREADS, smem, s, A);
    }
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

}  // namespace rc
