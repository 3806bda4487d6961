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
// One CTA = one item x one 128-row tile of one matrix, K in stages of 128 columns, the warps split into roles that hand
// tiles to each other through mbarriers (see k_tc_experts). Blocks beyond the item count leave at once. Every wait is
// bounded: on a timeout the role raises a flag that stops the other roles at their next wait; the CTA waits (bounded) for
// its own copies, frees its tensor memory, raises the launch's flag and the sticky status word, and returns.
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

// shared-memory matrix descriptor, K-major rows of 128 bytes (64 halves) with the 128-byte swizzle: the 16-byte chunk c of
// row r sits at r * 128 + ((c ^ (r % 8)) * 16) of a 1024-byte aligned tile; 8-row groups are 1024 bytes apart. A k-step
// of 16 halves is addressed by advancing the start address by 32 bytes.
__device__ __forceinline__ uint64_t tcx_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint32_t tcx_sw128(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }
// 128-row tiles one CTA works through: as many as keep it at 8 blocks of 256 columns (and divide the matrix)
__host__ __device__ uint32_t tcx_tiles_per_cta(uint32_t nrows, uint32_t ncols) {
    uint32_t tpc = 2048u / ncols;
    const uint32_t rtiles = nrows / 128u;
    tpc = tpc < 1u ? 1u : tpc;
    while (tpc > 1u && rtiles % tpc) tpc >>= 1;
    return tpc;
}

__device__ __forceinline__ void tcx_arrive(uint32_t mbar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(mbar) : "memory"); }

// Roles of the 16 warps (no block-wide barrier inside the K loop; the roles meet on mbarriers):
//   warp 0          lane 0 issues the 8 MMAs of a stage once its weight tiles and its activation tiles are full, and commits
//                   their completion to the "empty" barriers of both tiles (and, at the end of a 256-column block, to the
//                   block's "accumulators full" barrier)
//   warps 1-2       gather the activation pieces of stage after stage (cp.async, up to NB stages ahead of the MMAs)
//   warp 3          lane 0 requests the records of block after block (cp.async.bulk, one block ahead of the decoders)
//   warps 4-11      decode the weights of a stage into the fp16 tile (two (row, 8-column-pair) items per thread)
//   warps 12-15     read a finished block's accumulators out of tensor memory (warp w owns lanes 32 (w % 4) ..) and add
//                   them, scaled by d / 8, to their fp32 register sums; at the end they store the results
constexpr uint32_t TCX_NB = 3u;               // activation stage buffers
// A stage is 128 columns: two 64-column operand tiles (the 128-byte swizzle spans 64 halves) side by side in one buffer, so the
// issuing thread's waits, fence and commits - which, not the tensor pipe, bound this kernel - are paid once per 8 MMAs.
constexpr uint32_t TCX_KS = 128u, TCX_SUBS = TCX_KS / TC_KS, TCX_SPB = 256u / TCX_KS;      // stage width, tiles per stage, stages per 256-column block
constexpr uint32_t TCX_W_GATHER = 1u, TCX_N_GATHER = 2u, TCX_W_RAW = 3u, TCX_W_DECODE = 4u, TCX_N_DECODE = 8u, TCX_W_DRAIN = 12u;

template <int TN>
__global__ void __launch_bounds__(TC_THREADS, 1) k_tc_experts(const __grid_constant__ TcxArgs A) {
    pdl_prologue();
    const uint32_t item = blockIdx.y;
    if (item >= *A.n_items) return;                       // the grid covers the largest possible item count
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr uint32_t NB = TCX_NB;
    constexpr uint32_t B_DIGIT = (uint32_t)TN * TC_KS * 2u, A_SUB = TC_A_DIGIT, B_SUB = 2u * B_DIGIT, A_BUF = TCX_SUBS * A_SUB, B_BUF = TCX_SUBS * B_SUB;
    constexpr uint32_t TMEM_COLS = 4u * (uint32_t)TN;     // two blocks in flight x (A*hi accumulator, A*lo accumulator)
    static_assert(TN == 64, "the role split below is laid out for 64-token items");
    __shared__ __align__(8) uint64_t a_full[2], a_empty[2], b_full[NB], b_empty[NB], acc_full[2], acc_empty[2], raw_full[2], raw_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile uint32_t fail;               // a bounded wait ran out: every role stops at its next wait
    __shared__ uint32_t s_row[TN], s_pair[TN];       // activation row and pair of every token slot of the item (TCX_DEAD beyond its pairs)
    __shared__ float s_xinv[TN];
    __shared__ float s_d[8][TC_M];                   // d / 8 of every row for every 256-column block (at most 8 blocks)
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;

    const uint32_t u = A.item_u[item], p0 = A.item_p0[item], pe = A.ustart[u + 1u];
    const uint32_t nt = pe - p0 < (uint32_t)TN ? pe - p0 : (uint32_t)TN;
    const uint32_t e = A.uexp[u] - A.expert_begin;
    if (e >= A.n_local) {                                 // cannot happen with k_group_pairs' output; never an address
        if (tid == 0 && A.status) A.status[ST_EXPERT_RANGE] = 1u;
        return;
    }
    // A CTA takes tpc consecutive 128-row tiles of one matrix, one after the other, so that 8 blocks of 256 columns pass
    // through it whatever the row length: the set-up and the pipeline fill are paid once per CTA, not once per short row.
    const uint32_t bpr = A.ncols >> 8, kstage = A.ncols / TCX_KS, tpc = tcx_tiles_per_cta(A.nrows, A.ncols);
    const uint32_t groups = A.nrows / TC_M / tpc, mat = blockIdx.x / groups, rt0 = (blockIdx.x - mat * groups) * tpc;
    const uint32_t nstage = tpc * kstage, nblk = tpc * bpr;           // stages and 256-column blocks of the whole CTA
    const uint8_t *wrec = A.w[mat] + (uint64_t)e * A.mat_bytes + (uint64_t)(rt0 * 8u) * bpr * NIB_REC;    // record (16-row tile 8 rt0 + j, block c) at (j * bpr + c) * NIB_REC
    uint8_t *a_base = smem, *b_base = smem + 2u * A_BUF, *raw_base = b_base + NB * B_BUF;

    if (tid < (uint32_t)TN) {
        uint32_t row = TCX_DEAD, pair = TCX_DEAD; float inv = 0.f;
        if (tid < nt) { pair = A.sorted[p0 + tid]; row = pair / A.x_div; inv = A.x_inv[row]; }
        s_row[tid] = row; s_pair[tid] = pair; s_xinv[tid] = inv;
    }
    for (uint32_t i = tid; i < TC_M * nblk; i += TC_THREADS) {     // block scales of the CTA's rows: s_d[tile * bpr + block][row of the tile]
        const uint32_t cb = i / TC_M, r = i - cb * TC_M, tile = cb / bpr, c = cb - tile * bpr;
        s_d[cb][r] = 0.125f * __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(wrec + ((uint64_t)(tile * 8u + (r >> 4)) * bpr + c) * NIB_REC + NIB_D_OFF + (r & 15u) * 2u))));
    }
    if (tid == 0) {
        fail = 0u;
        auto init = [](uint64_t *bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count)); };
        for (uint32_t i = 0; i < 2u; ++i) {
            init(&a_full[i], TCX_N_DECODE); init(&a_empty[i], 1u); init(&acc_full[i], 1u); init(&acc_empty[i], 4u);
            init(&raw_full[i], 1u); init(&raw_empty[i], TCX_N_DECODE);
        }
        for (uint32_t i = 0; i < NB; ++i) { init(&b_full[i], TCX_N_GATHER); init(&b_empty[i], 1u); }
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
    // a wait that gives up raises the flag; every role checks it before each wait, so the CTA winds down within a few waits
    auto wait = [&](uint64_t *bar, uint32_t parity) -> bool {
        if (fail) return false;
        if (mbar_wait(smem_u32(bar), parity)) return true;
        fail = 1u;
        return false;
    };
    // the same for roles that are far ahead of their producer (drain, record fetch, gather): they sleep longer between polls,
    // so that their spinning does not take issue slots from the decode warps and the MMA thread
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
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            // One MMA per k-step: the hi and lo digit rows of a stage are one 128-row operand (hi rows, then lo rows), so the
            // product lands as [A*hi | A*lo] in 2 TN accumulator columns. Descriptors differ from stage to stage only in
            // their start address, so the loop adds a constant to a precomputed low word. This thread's latency per stage
            // is what bounds the pipeline, so its waits are kept to the bare polls.
            const uint32_t idesc = tc_idesc(2u * (uint32_t)TN);
            const uint64_t desc0 = tcx_desc_sw128(0u);
            auto ready = [&](uint64_t *bar, uint32_t parity) -> bool {
                const uint32_t addr = smem_u32(bar);
                uint32_t done;
                asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                             : "=r"(done) : "r"(addr), "r"(parity) : "memory");
                return done ? true : wait(bar, parity);
            };
            for (uint32_t s = 0; s < nstage; ++s) {
                const uint32_t b = s & 1u, jb = s % NB, c = s / TCX_SPB, sb = s % TCX_SPB;
                if (!ready(&a_full[b], (s >> 1) & 1u) || !ready(&b_full[jb], (s / NB) & 1u)) break;
                if (sb == 0u && c >= 2u && !ready(&acc_empty[c & 1u], ((c >> 1) - 1u) & 1u)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = desc0 + ((smem_u32(a_base + b * A_BUF) >> 4) & 0x3fffu), db = desc0 + ((smem_u32(b_base + jb * B_BUF) >> 4) & 0x3fffu);
                const uint32_t d_acc = tmem + (c & 1u) * 2u * (uint32_t)TN;
#pragma unroll
                for (uint32_t kk = 0; kk < TCX_KS / 16u; ++kk) {     // + 32 bytes per k-step inside a tile, the next tile after four; a block's first MMA overwrites
                    const uint32_t sub = kk >> 2, k4 = kk & 3u;
                    tc_mma(d_acc, da + sub * (A_SUB >> 4) + 2u * k4, db + sub * (B_SUB >> 4) + 2u * k4, idesc, (sb | kk) ? 1u : 0u);
                }
                tc_commit(smem_u32(&a_empty[b]));
                tc_commit(smem_u32(&b_empty[jb]));
                if (sb == TCX_SPB - 1u) tc_commit(smem_u32(&acc_full[c & 1u]));
            }
        }
    } else if (warp < TCX_W_RAW) {
        // ------------------------------------------------------------------ activation gather (64 threads)
        // thread g: k chunk g % 8 of the token slots g / 8 + 8 m (m < 8), both digits, both tiles of the stage: 32 pieces of 16 bytes per stage
        const uint32_t g = tid - TCX_W_GATHER * 32u, kc = g & 7u, ttb = g >> 3;
        const __half *src[8]; uint32_t live = 0u;
#pragma unroll
        for (uint32_t m = 0; m < 8u; ++m) {
            const uint32_t row = s_row[ttb + 8u * m];
            if (row != TCX_DEAD) live |= 1u << m;
            src[m] = A.xd + (size_t)(row != TCX_DEAD ? row : 0u) * 2u * A.ncols + kc * 8u;
        }
        const uint32_t dst0 = tcx_sw128(ttb, kc);         // token slot ttb + 8 m: the same swizzle phase, 1024 bytes further per m
        auto issue = [&](uint32_t s) {
            const uint32_t bb = smem_u32(b_base + (s % NB) * B_BUF) + dst0;
#pragma unroll
            for (uint32_t sub = 0; sub < TCX_SUBS; ++sub)
#pragma unroll
                for (uint32_t m = 0; m < 8u; ++m) {
                    const uint32_t sz = (live >> m) & 1u ? 16u : 0u;
                    const __half *sp = src[m] + (s % kstage) * TCX_KS + sub * TC_KS;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(bb + sub * B_SUB + m * 1024u), "l"(sp), "r"(sz) : "memory");
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(bb + sub * B_SUB + B_DIGIT + m * 1024u), "l"(sp + A.ncols), "r"(sz) : "memory");
                }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        // stage s is requested AHEAD stages before it is handed over; AHEAD <= NB - 2, so that handing over stage s - AHEAD never
        // waits for the MMAs of the stage just before it (the wait at the top of an iteration is for stage s - NB)
        constexpr uint32_t AHEAD = NB - 2u;
        bool ok = true;
        for (uint32_t s = 0; s < nstage + AHEAD && ok; ++s) {
            if (s < nstage) {
                if (s >= NB) ok = wait_idle(&b_empty[s % NB], ((s / NB) - 1u) & 1u);
                if (ok) issue(s); else asm volatile("cp.async.commit_group;" ::: "memory");
            } else asm volatile("cp.async.commit_group;" ::: "memory");
            if (s >= AHEAD) {
                asm volatile("cp.async.wait_group %0;" :: "n"(AHEAD) : "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) tcx_arrive(smem_u32(&b_full[(s - AHEAD) % NB]));
                
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp == TCX_W_RAW) {
        // ------------------------------------------------------------------ weight records, one block ahead
        if (lane == 0) {
            uint32_t issued = 0u;
            for (uint32_t c = 0; c < nblk; ++c) {       // c counts the CTA's blocks: tile c / bpr, block column c % bpr
                if (c >= 2u && !wait_idle(&raw_empty[c & 1u], ((c >> 1) - 1u) & 1u)) break;
                const uint32_t tile = c / bpr, col = c - tile * bpr;
                const uint32_t bar = smem_u32(&raw_full[c & 1u]), dst = smem_u32(raw_base + (c & 1u) * TCX_RAW);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(TCX_RAW) : "memory");
#pragma unroll
                for (uint32_t j = 0; j < 8u; ++j)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 :: "r"(dst + j * NIB_REC), "l"(wrec + ((uint64_t)(tile * 8u + j) * bpr + col) * NIB_REC), "r"(NIB_REC), "r"(bar) : "memory");
                issued = c + 1u;
            }
            // a copy that nobody waited for may still be writing into this CTA's shared memory: wait for the last two (bounded)
            for (uint32_t c = issued >= 2u ? issued - 2u : 0u; c < issued; ++c) mbar_wait(smem_u32(&raw_full[c & 1u]), (c >> 1) & 1u);
        }
    } else if (warp < TCX_W_DRAIN) {
        // ------------------------------------------------------------------ weight decode (256 threads)
        const uint32_t dw = warp - TCX_W_DECODE, t = lane & 3u;
        for (uint32_t s = 0; s < nstage; ++s) {
            const uint32_t b = s & 1u, c = s / TCX_SPB, sb = s % TCX_SPB;
            if (sb == 0u && !wait(&raw_full[c & 1u], (c >> 1) & 1u)) break;
            if (s >= 2u && !wait(&a_empty[b], ((s >> 1) - 1u) & 1u)) break;
            const uint8_t *raw = raw_base + (c & 1u) * TCX_RAW;
            uint8_t *abuf = a_base + b * A_BUF;
            const uint32_t kg0 = 4u * sb;                 // the stage's four 32-column groups
            
#pragma unroll
            for (uint32_t q = 0; q < 2u; ++q) {
                // rows 8 dw + lane / 4 and + 64; code words (t, kg0 .. kg0 + 3) of the row (one 16-byte piece): columns
                // 32 (kg - kg0) + 8 t of the stage, i.e. chunk t or t + 4 of tile (kg - kg0) / 2
                const uint32_t r = q * 64u + dw * 8u + (lane >> 2), rr = r & 15u;
                const uint8_t *rec = raw + (r >> 4) * NIB_REC;
                const uint4 wd = *reinterpret_cast<const uint4 *>(rec + nib_code_off(rr, t, kg0));
                const uint32_t sc4 = *reinterpret_cast<const uint32_t *>(rec + NIB_SC_OFF + rr * 8u + kg0);
                *reinterpret_cast<uint4 *>(abuf + tcx_sw128(r, t)) = tcx_decode8(wd.x, sc4 & 255u);
                *reinterpret_cast<uint4 *>(abuf + tcx_sw128(r, t + 4u)) = tcx_decode8(wd.y, (sc4 >> 8) & 255u);
                *reinterpret_cast<uint4 *>(abuf + A_SUB + tcx_sw128(r, t)) = tcx_decode8(wd.z, (sc4 >> 16) & 255u);
                *reinterpret_cast<uint4 *>(abuf + A_SUB + tcx_sw128(r, t + 4u)) = tcx_decode8(wd.w, sc4 >> 24);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy writes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) {
                tcx_arrive(smem_u32(&a_full[b]));
                if (sb == TCX_SPB - 1u) tcx_arrive(smem_u32(&raw_empty[c & 1u]));     // this warp has read the block's records for the last time
                
            }
        }
    } else {
        // ------------------------------------------------------------------ accumulator drain and epilogue (128 threads)
        const uint32_t qlane = (warp & 3u) * 32u;
        float acc[TN];
#pragma unroll
        for (uint32_t j = 0; j < (uint32_t)TN; ++j) acc[j] = 0.f;
        bool ok = true;
        for (uint32_t blk = 0; blk < nblk && ok; ++blk) {
            ok = wait_idle(&acc_full[blk & 1u], (blk >> 1) & 1u);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            
            const float dsc = s_d[blk][qlane + lane];
            const uint32_t base = tmem + (qlane << 16) + (blk & 1u) * 2u * (uint32_t)TN;
#pragma unroll
            for (uint32_t cc = 0; cc < (uint32_t)TN; cc += 16u) {
                uint32_t m[16], x[16];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                             : "=r"(m[0]), "=r"(m[1]), "=r"(m[2]), "=r"(m[3]), "=r"(m[4]), "=r"(m[5]), "=r"(m[6]), "=r"(m[7]),
                               "=r"(m[8]), "=r"(m[9]), "=r"(m[10]), "=r"(m[11]), "=r"(m[12]), "=r"(m[13]), "=r"(m[14]), "=r"(m[15]) : "r"(base + cc));
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                             : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]), "=r"(x[4]), "=r"(x[5]), "=r"(x[6]), "=r"(x[7]),
                               "=r"(x[8]), "=r"(x[9]), "=r"(x[10]), "=r"(x[11]), "=r"(x[12]), "=r"(x[13]), "=r"(x[14]), "=r"(x[15]) : "r"(base + (uint32_t)TN + cc));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[cc + j] = fmaf(dsc, __uint_as_float(m[j]) + __uint_as_float(x[j]), acc[cc + j]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tcx_arrive(smem_u32(&acc_empty[blk & 1u]));
            if ((blk + 1u) % bpr == 0u) {            // the last block of a row tile: store it and start the next tile from zero
                const uint32_t row = (rt0 + blk / bpr) * TC_M + qlane + lane;
                float *out = A.out[mat];
#pragma unroll
                for (uint32_t j = 0; j < (uint32_t)TN; ++j) {
                    const uint32_t pair = s_pair[j];
                    if (pair != TCX_DEAD) out[(size_t)pair * A.out_stride + row] = acc[j] * s_xinv[j];
                    acc[j] = 0.f;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (fail && tid == 0) {
        atomicExch(A.err, 1u);
        if (A.status) A.status[ST_TIMEOUT] = 1u;
    }
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
    const size_t smem = 2u * (size_t)TCX_SUBS * TC_A_DIGIT + (size_t)TCX_NB * TCX_SUBS * 2u * TN * TC_KS * 2u + 2u * (size_t)TCX_RAW;
    const dim3 grid(A.nmat * (A.nrows / TC_M / tcx_tiles_per_cta(A.nrows, A.ncols)), max_items);
    prof_begin(tag, s);
    RC_CUDA(cudaFuncSetAttribute(k_tc_experts<(int)TN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    RC_LAUNCH((k_tc_experts<(int)TN>), grid, TC_THREADS, smem, s, A);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

}  // namespace rc
