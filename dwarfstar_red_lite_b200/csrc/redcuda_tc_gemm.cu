// Prefill projections on the 5th-generation tensor cores (tcgen05): out[t][r] = sum_k W[r][k] * x[t][k] for a chunk of
// tokens, W a quantised matrix (Q6_K / IQ2_XXS / IQ3_S rows, planar layout) that is decoded on the fly.
//
// The batched form of rl_quant_row_dot over every row (native/redlite_native_quant_cpu.c:247-266); the reference's GPU
// prefill dequantises to f32 and runs an f32 GEMM (native/redmetal_engine_prefill.m:205-227, 889-909). Results have to
// stay at fp32 accuracy (the 48-layer model amplifies rounding noise by orders of magnitude), so neither operand is
// rounded to one 16-bit value: both are split into two fp16 digits, v * 2^e = hi + lo (|error| <= 2^-22 |v|), and
// three products are accumulated in fp32 in tensor memory: hi*hi + hi*lo + lo*hi. The power-of-two scales (per row
// tile for the weights, per token for the activations) keep hi in the normal fp16 range and are undone in the epilogue.
//
// One CTA = 128 weight rows (MMA M) x TN tokens (MMA N) x all columns, K in stages of 64:
//   all 8 warps   stage the raw quant blocks of the 128 rows one 256-column block ahead (cp.async, 16-byte pieces, the
//                 planar layout kept, so the exact decoder of the GEMV path reads them unchanged), decode 128 x 64
//                 weights from shared memory into the two fp16 digit tiles of the stage (canonical K-major core-matrix
//                 layout, no swizzle) and copy the stage's activation digits (laid out for the MMA by k_tc_prep_x)
//   one thread    issues 4 k-steps x 3 tcgen05.mma (128 x TN x 16, kind::f16, fp32 accumulate) and a tcgen05.commit
//                 on the stage buffer's mbarrier; the MMAs of a stage run while the warps decode the next one
//   epilogue      tcgen05.ld of the accumulator (lane = weight row, column = token), scaling, coalesced stores
// Every wait on an mbarrier is bounded; on a timeout the kernel raises a flag, frees its tensor memory and returns.
#define RC_PDL_DEFAULT 0
#include "redcuda_common.cuh"
#include "redcuda_formats.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_tc_gemm.cuh"

#include <cuda_fp16.h>

namespace rc {

constexpr uint32_t TC_M = 128u, TC_KS = 64u, TC_THREADS = 256u;
constexpr uint32_t TC_A_DIGIT = TC_M * TC_KS * 2u;            // bytes of one weight digit tile of a stage (16 KB)
constexpr uint32_t TC_SPIN_LIMIT = 4u * 1000u * 1000u;        // polls of ~50 ns: far beyond any legitimate wait

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// shared-memory matrix descriptor: K-major, no swizzle, core matrix = 8 rows x 16 bytes stored as 128 contiguous bytes;
// lbo = byte distance between the two 16-byte k-chunks of one MMA, sbo = byte distance between 8-row groups
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) | ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}

// instruction descriptor, kind::f16: D = f32, A = B = f16, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t tc_idesc(uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((TC_M >> 4) << 24); }

__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(mbar) : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(mbar), "r"(parity) : "memory");
        if (done) return true;
        __nanosleep(32);
    }
    return false;
}

__device__ __forceinline__ uint32_t tc_d_plane(uint32_t type, uint64_t nb) {
    return (uint32_t)(type == RC_Q6_K ? rc_q6_d(nb) : type == RC_IQ2_XXS ? rc_iq2_d(nb) : rc_iq3_d(nb));
}

__device__ __forceinline__ void cp_async_n(uint32_t dst, const void *src, uint32_t bytes) {
    if (bytes == 16u) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(src) : "memory");
    else if (bytes == 8u) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" :: "r"(dst), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(dst), "l"(src) : "memory");
}

// bytes of the raw staging area: the planar layout of a 128-block matrix of the type
__host__ __device__ __forceinline__ uint32_t tc_raw_bytes(uint32_t type) { return TC_M * rc_block_bytes(type); }

// Copy block column c of rows [row0, row0 + 128) into `raw`, laid out as a planar matrix of 128 blocks (block r = row r).
// Every plane piece of 4 bytes or more goes by cp.async; the 2-byte block scales are returned in a register by the
// threads that own a row (tid < 128) and stored by tc_put_d once the previous block column is no longer read.
__device__ __forceinline__ unsigned short tc_stage_raw(uint32_t type, const uint8_t *w, uint64_t nb, uint32_t bpr, uint32_t row0, uint32_t nrows,
                                                       uint32_t c, uint8_t *raw, uint32_t tid) {
    const uint32_t raw_s = smem_u32(raw);
    auto plane = [&](uint64_t off_g, uint32_t off_s, uint32_t piece) {
        const uint32_t unit = piece >= 16u ? 16u : piece, per_row = piece / unit;
        for (uint32_t i = tid; i < TC_M * per_row; i += TC_THREADS) {
            const uint32_t r = i / per_row, u = i - r * per_row;
            if (row0 + r < nrows) cp_async_n(raw_s + off_s + r * piece + u * unit, w + off_g + ((uint64_t)(row0 + r) * bpr + c) * piece + u * unit, unit);
        }
    };
    if (type == RC_Q6_K) {
        plane(0u, 0u, 128u); plane(rc_q6_qh(nb), (uint32_t)rc_q6_qh(TC_M), 64u); plane(rc_q6_sc(nb), (uint32_t)rc_q6_sc(TC_M), 16u);
    } else if (type == RC_IQ2_XXS) {
        plane(0u, 0u, 64u);
    } else {
        plane(0u, 0u, 64u); plane(rc_iq3_signs(nb), (uint32_t)rc_iq3_signs(TC_M), 32u); plane(rc_iq3_qh(nb), (uint32_t)rc_iq3_qh(TC_M), 8u);
        plane(rc_iq3_scales(nb), (uint32_t)rc_iq3_scales(TC_M), 4u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    unsigned short d = 0;
    if (tid < TC_M && row0 + tid < nrows) d = __ldg(reinterpret_cast<const unsigned short *>(w + tc_d_plane(type, nb)) + (uint64_t)(row0 + tid) * bpr + c);
    return d;
}

__device__ __forceinline__ void tc_put_d(uint32_t type, uint8_t *raw, uint32_t tid, unsigned short d) {
    if (tid < TC_M) reinterpret_cast<unsigned short *>(raw + tc_d_plane(type, TC_M))[tid] = d;
}

// x [ntok][ncols] fp32 -> fp16 digits in the order the GEMM stages consume them:
// xs[token tile][k stage][digit hi/lo][k chunk of 8 (8)][token group of 8 (TN/8)][token in group (8)][8 halves];
// x_inv[t] = 2^-e_t undoes the per-token scale. Tokens beyond ntok are zero. grid = token tiles * TN, block = 256
__global__ void k_tc_prep_x(const float *__restrict__ x, uint32_t x_stride, uint32_t ntok, uint32_t ncols, uint32_t tn,
                            __half *__restrict__ xs, float *__restrict__ x_inv) {
    pdl_prologue();
    __shared__ float red[8];
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    const bool live = t < ntok;
    float mx = 0.f;
    if (live) for (uint32_t k = tid; k < ncols; k += blockDim.x) mx = fmaxf(mx, fabsf(x[(size_t)t * x_stride + k]));
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
            const float v = live ? x[(size_t)t * x_stride + c * 8u + j] * sc : 0.f;
            hi[j] = __float2half_rn(v);
            lo[j] = __float2half_rn(v - __half2float(hi[j]));
        }
        __half *dst = xs + ((size_t)tile * nstage + stage) * 2u * digit + ((size_t)kc * (tn >> 3) + (tt >> 3)) * 64u + (tt & 7u) * 8u;
        *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(hi);
        *reinterpret_cast<uint4 *>(dst + digit) = *reinterpret_cast<const uint4 *>(lo);
    }
}

template <int TN>
__global__ void __launch_bounds__(TC_THREADS, 1) k_tc_gemm(const __grid_constant__ TcArgs A) {
    pdl_prologue();
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t B_DIGIT = (uint32_t)TN * TC_KS * 2u, BUF = 2u * TC_A_DIGIT + 2u * B_DIGIT;
    constexpr uint32_t TMEM_COLS = TN < 32 ? 32u : (uint32_t)TN;
    __shared__ __align__(8) uint64_t mbar[2];
    __shared__ uint32_t tmem_slot, fail;
    __shared__ float red[8];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;

    // which matrix of the launch this row tile belongs to
    uint32_t ji = 0;
    for (uint32_t j = 1; j < A.njobs; ++j) if (blockIdx.x >= A.job[j].tile0) ji = j;
    const TcJob &J = A.job[ji];
    const uint32_t row0 = (blockIdx.x - J.tile0) * TC_M, t0 = blockIdx.y * (uint32_t)TN;
    const uint32_t bpr = A.ncols >> 8, nstage = A.ncols / TC_KS;
    const RcBooks bk{A.iq2, A.iq3s};

    if (tid == 0) {
        fail = 0u;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&mbar[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&mbar[1])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // power-of-two scale of the tile: the largest block scale d times the largest integer factor of the format
    float dmax = 0.f;
    {
        const unsigned short *dp = reinterpret_cast<const unsigned short *>(J.w + tc_d_plane(J.type, J.nb));
        for (uint32_t i = tid; i < TC_M * bpr; i += TC_THREADS) {
            const uint32_t r = row0 + i / bpr;
            if (r < J.nrows) dmax = fmaxf(dmax, fabsf(__half2float(__ushort_as_half(dp[(size_t)r * bpr + (i % bpr)]))));
        }
        for (int o = 16; o; o >>= 1) dmax = fmaxf(dmax, __shfl_xor_sync(0xffffffffu, dmax, o));
        if (lane == 0) red[warp] = dmax;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    dmax = 0.f;
    for (int w = 0; w < 8; ++w) dmax = fmaxf(dmax, red[w]);
    int we = 0;
    {
        const float bound = dmax * (J.type == RC_Q6_K ? 4096.f : J.type == RC_IQ2_XXS ? 256.f : 512.f);
        if (bound > 0.f && bound < INFINITY) { int ex; frexpf(bound, &ex); we = 15 - ex; }       // |w| * 2^we < 2^15
        we = we > 100 ? 100 : we < -100 ? -100 : we;
    }
    const float w_scale = exp2f((float)we), w_inv = exp2f((float)-we);

    const __half *xs_tile = A.xs + (size_t)blockIdx.y * nstage * (2u * B_DIGIT / 2u);
    const uint32_t idesc = tc_idesc((uint32_t)TN);

    uint8_t *raw_buf[2] = {smem + 2u * BUF, smem + 2u * BUF + tc_raw_bytes(J.type)};
    unsigned short d_next = tc_stage_raw(J.type, J.w, J.nb, bpr, row0, J.nrows, 0u, raw_buf[0], tid);

    for (uint32_t s = 0; s < nstage; ++s) {
        const uint32_t b = s & 1u;
        uint8_t *buf = smem + b * BUF;
        const uint32_t c = (s * TC_KS) >> 8;                      // 256-column block of this stage
        if (((s * TC_KS) & 255u) == 0u) {
            // new block column: its raw bytes were requested one column ago; request the next one
            tc_put_d(J.type, raw_buf[c & 1u], tid, d_next);
            asm volatile("cp.async.wait_all;" ::: "memory");
            __syncthreads();                                       // raw[c & 1] complete, raw[(c + 1) & 1] no longer read
            if (c + 1u < bpr) d_next = tc_stage_raw(J.type, J.w, J.nb, bpr, row0, J.nrows, c + 1u, raw_buf[(c + 1u) & 1u], tid);
        }
        const uint8_t *raw = raw_buf[c & 1u];
        // the MMAs that read this buffer two stages ago must have finished
        if (s >= 2u) {
            if (!mbar_wait(smem_u32(&mbar[b]), ((s >> 1) - 1u) & 1u)) fail = 1u;
        }
        // ---- weights: thread -> (row, k-chunk of 8), 4 rows x 8 chunks per warp pass
        const uint32_t g8_0 = ((s * TC_KS) & 255u) >> 3;
#pragma unroll
        for (uint32_t it = 0; it < (TC_M * 8u) / TC_THREADS; ++it) {
            const uint32_t item = it * TC_THREADS + tid, r = item >> 3, kc = item & 7u;
            __half hi[8], lo[8];
            if (row0 + r < J.nrows) {
                float v[8];
                rc_decode8(J.type, raw, TC_M, r, g8_0 + kc, bk, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float vs = v[j] * w_scale;
                    hi[j] = __float2half_rn(vs);
                    lo[j] = __float2half_rn(vs - __half2float(hi[j]));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) { hi[j] = __float2half_rn(0.f); lo[j] = hi[j]; }
            }
            const uint32_t off = kc * (TC_M * 16u) + r * 16u;          // [k chunk][row group][row in group][16 B]
            *reinterpret_cast<uint4 *>(buf + off) = *reinterpret_cast<const uint4 *>(hi);
            *reinterpret_cast<uint4 *>(buf + TC_A_DIGIT + off) = *reinterpret_cast<const uint4 *>(lo);
        }
        // ---- activations: the stage's two digit tiles are one contiguous run in xs
        {
            const uint4 *src = reinterpret_cast<const uint4 *>(xs_tile + (size_t)s * (2u * B_DIGIT / 2u));
            uint4 *dst = reinterpret_cast<uint4 *>(buf + 2u * TC_A_DIGIT);
            for (uint32_t i = tid; i < 2u * B_DIGIT / 16u; i += TC_THREADS) dst[i] = __ldg(src + i);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy writes -> visible to the tensor core
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && !fail) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = smem_u32(buf), a_lo = a_hi + TC_A_DIGIT, b_hi = a_hi + 2u * TC_A_DIGIT, b_lo = b_hi + B_DIGIT;
            constexpr uint32_t A_LBO = TC_M * 16u, B_LBO = (uint32_t)TN * 16u, SBO = 128u;
#pragma unroll
            for (uint32_t kk = 0; kk < TC_KS / 16u; ++kk) {
                const uint64_t dah = tc_smem_desc(a_hi + 2u * kk * A_LBO, A_LBO, SBO), dal = tc_smem_desc(a_lo + 2u * kk * A_LBO, A_LBO, SBO);
                const uint64_t dbh = tc_smem_desc(b_hi + 2u * kk * B_LBO, B_LBO, SBO), dbl = tc_smem_desc(b_lo + 2u * kk * B_LBO, B_LBO, SBO);
                tc_mma(tmem, dah, dbh, idesc, (s | kk) ? 1u : 0u);
                tc_mma(tmem, dah, dbl, idesc, 1u);
                tc_mma(tmem, dal, dbh, idesc, 1u);
            }
            tc_commit(smem_u32(&mbar[b]));
        }
    }
    // ---- all MMAs done? (the last commit of each buffer covers everything issued before it)
    {
        const uint32_t last = nstage - 1u;
        if (!mbar_wait(smem_u32(&mbar[last & 1u]), (last >> 1) & 1u)) fail = 1u;
        if (nstage >= 2u && !mbar_wait(smem_u32(&mbar[(last - 1u) & 1u]), ((last - 1u) >> 1) & 1u)) fail = 1u;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    if (!fail) {
        // warp w reads TMEM lanes 32*(w%4)..+31 (its quarter); warps w and w+4 share a quarter and split the columns
        const uint32_t q = warp & 3u, row = row0 + q * 32u + lane;
        constexpr uint32_t HALF = (uint32_t)TN / 2u < 16u ? 16u : (uint32_t)TN / 2u;
        const uint32_t c_begin = (warp >> 2) * HALF, c_end = c_begin + HALF > (uint32_t)TN ? (uint32_t)TN : c_begin + HALF;
        for (uint32_t c = c_begin; c < c_end; c += 16u) {
            uint32_t v[16];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                         : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                           "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                         : "r"(tmem + ((q * 32u) << 16) + c));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t t = t0 + c + j;
                if (t < A.ntok && row < J.nrows) J.out[(size_t)t * J.out_stride + row] = __uint_as_float(v[j]) * w_inv * A.x_inv[t];
            }
        }
    } else if (tid == 0) atomicExch(A.err, 1u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(TMEM_COLS) : "memory");
}

size_t tc_xs_halves(uint32_t ntok, uint32_t ncols, uint32_t tn) { return (size_t)((ntok + tn - 1u) / tn) * tn * ncols * 2u; }

uint32_t tc_token_tile(uint32_t ntok) { return ntok <= 32u ? 32u : ntok <= 64u ? 64u : 128u; }

int launch_tc_prep_x(const float *x, uint32_t x_stride, uint32_t ntok, uint32_t ncols, __half *xs, float *x_inv, cudaStream_t s) {
    RC_REQUIRE(ncols % TC_KS == 0, "tc gemm: %u columns is not a multiple of %u", ncols, TC_KS);
    const uint32_t tn = tc_token_tile(ntok), tiles = (ntok + tn - 1u) / tn;
    prof_begin("tc_prep_x", s);
    RC_LAUNCH((k_tc_prep_x), tiles * tn, 256, 0, s, x, x_stride, ntok, ncols, tn, xs, x_inv);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

int launch_tc_gemm(TcArgs &A, const char *tag, cudaStream_t s) {
    RC_REQUIRE(A.njobs >= 1 && A.njobs <= TC_MAX_JOBS && A.ntok >= 1, "tc gemm: bad job count or no tokens");
    RC_REQUIRE(A.ncols % 256u == 0, "tc gemm: %u columns is not a multiple of 256", A.ncols);
    uint32_t tiles = 0;
    for (uint32_t j = 0; j < A.njobs; ++j) {
        RC_REQUIRE(rc_is_quant(A.job[j].type), "tc gemm: matrix type %u is not a block-quantised format", A.job[j].type);
        A.job[j].tile0 = tiles;
        tiles += (A.job[j].nrows + TC_M - 1u) / TC_M;
    }
    A.iq2 = books_iq2(); A.iq3s = books_iq3s();
    const uint32_t tn = tc_token_tile(A.ntok);
    const dim3 grid(tiles, (A.ntok + tn - 1u) / tn);
    uint32_t raw_max = 0;
    for (uint32_t j = 0; j < A.njobs; ++j) raw_max = raw_max > tc_raw_bytes(A.job[j].type) ? raw_max : tc_raw_bytes(A.job[j].type);
    const size_t smem = 2u * (2u * TC_A_DIGIT + 2u * (size_t)tn * TC_KS * 2u) + 2u * (size_t)raw_max;
    prof_begin(tag, s);
#define RC_TC_LAUNCH(TN_) do { \
        RC_CUDA(cudaFuncSetAttribute(k_tc_gemm<TN_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        RC_LAUNCH((k_tc_gemm<TN_>), grid, TC_THREADS, smem, s, A); } while (0)
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
    const uint32_t tn = tc_token_tile(ntok);
    DevMem raw, planar, xd, od, xs, xinv, err;
    if (!raw.alloc(bytes) || !planar.alloc(bytes) || !xd.alloc((size_t)ntok * ncols * 4u) || !od.alloc((size_t)ntok * nrows * 4u) ||
        !xs.alloc(tc_xs_halves(ntok, ncols, tn) * 2u) || !xinv.alloc((size_t)((ntok + tn - 1u) / tn) * tn * 4u) || !err.alloc(4u)) return 0;
    cudaStream_t s = 0;
    if (!upload_matrix(type, nrows, ncols, w, false, planar.as<uint8_t>(), raw.as<uint8_t>(), s)) return 0;
    RC_CUDA(cudaMemcpyAsync(xd.p, x, (size_t)ntok * ncols * 4u, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemsetAsync(err.p, 0, 4u, s));
    if (!launch_tc_prep_x(xd.as<float>(), ncols, ntok, ncols, xs.as<__half>(), xinv.as<float>(), s)) return 0;
    TcArgs A{};
    A.njobs = 1; A.ncols = ncols; A.ntok = ntok; A.xs = xs.as<__half>(); A.x_inv = xinv.as<float>(); A.err = err.as<uint32_t>();
    A.job[0] = TcJob{planar.as<uint8_t>(), (uint64_t)nrows * (ncols / 256u), type, nrows, od.as<float>(), nrows, 0u};
    if (!launch_tc_gemm(A, "tc_gemm", s)) return 0;
    uint32_t flag = 0;
    RC_CUDA(cudaMemcpyAsync(&flag, err.p, 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaMemcpyAsync(out, od.p, (size_t)ntok * nrows * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    RC_REQUIRE(flag == 0u, "matmul_tc: a tensor-core stage never signalled completion (bounded wait ran out)");
    return 1;
}
