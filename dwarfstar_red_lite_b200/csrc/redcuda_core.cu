// redcuda core: error state, codebooks, matrix upload/repack, dequantisation, generic multi-job GEMV, router top-k.
#include "redcuda_common.cuh"
#include "redcuda_dot.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_moe_mma.cuh"
#include "../../include/redcuda.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <map>
#include <mutex>
#include <vector>

namespace rc {

static thread_local std::string t_err;
std::atomic<uint64_t> g_launches{0};

void set_error(const char *fmt, ...) {
    char buf[1024];
    va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof(buf), fmt, ap); va_end(ap);
    t_err = buf;
}

// ---- per-kernel event timing ----
struct ProfRec { const char *tag; cudaEvent_t a, b; };
static bool g_prof_on = false;
static std::vector<ProfRec> g_prof;
static std::mutex g_prof_mu;

void prof_begin(const char *tag, cudaStream_t s) {
    if (!g_prof_on) return;
    ProfRec r{tag, nullptr, nullptr};
    if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
    cudaEventRecord(r.a, s);
    std::lock_guard<std::mutex> lk(g_prof_mu);
    g_prof.push_back(r);
}
bool prof_active() { return g_prof_on; }
void prof_end(cudaStream_t s) {
    if (!g_prof_on) return;
    std::lock_guard<std::mutex> lk(g_prof_mu);
    if (!g_prof.empty()) cudaEventRecord(g_prof.back().b, s);
}

int pdl_mode() {
    static const int mode = getenv("RC_PDL") ? (atoi(getenv("RC_PDL")) != 0) : -1;
    return mode;
}

static uint32_t *g_status = nullptr;
static std::once_flag g_status_once;
uint32_t *status_words() {
    std::call_once(g_status_once, [] {
        void *p = nullptr;
        if (cudaHostAlloc(&p, ST_WORDS * sizeof(uint32_t), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) { cudaGetLastError(); return; }
        memset(p, 0, ST_WORDS * sizeof(uint32_t));
        g_status = (uint32_t *)p;      // unified addressing: the host pointer is valid on every device
    });
    return g_status;
}
int status_failed() {
    volatile uint32_t *st = g_status;
    if (!st) return 0;
    const uint32_t a = st[ST_ROUTER_NONFINITE], b = st[ST_TOKEN_RANGE], c = st[ST_EXPERT_RANGE], d = st[ST_TIMEOUT];
    if (!(a | b | c | d)) return 0;
    st[ST_ROUTER_NONFINITE] = 0; st[ST_TOKEN_RANGE] = 0; st[ST_EXPERT_RANGE] = 0; st[ST_TIMEOUT] = 0;
    if (a) set_error("invalid router softmax denominator (non-finite router logits)");
    else if (b) set_error("token id out of range on the device (non-finite logits in the argmax?)");
    else if (c) set_error("an expert id outside this shard reached an expert kernel");
    else set_error("an expert kernel gave up waiting for a weight copy (bounded wait ran out); its outputs are incomplete");
    return 1;
}

int require_device() {
    int n = 0;
    const cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        set_error("no usable CUDA device (%s); redcuda has no CPU path", e == cudaSuccess ? "device count 0" : cudaGetErrorString(e));
        return 0;
    }
    return 1;
}

int DevMem::alloc(size_t n) {
    release();
    if (!n) n = 16;
    RC_CUDA(cudaMalloc(&p, n));
    bytes = n;
    return 1;
}
void DevMem::release() { if (p) { cudaFree(p); p = nullptr; bytes = 0; } }

// ---- codebooks: one copy per device, in global memory; kernels stage them into shared memory ----
__device__ __align__(16) uint8_t d_iq2_grid[2048];
__device__ __align__(16) uint32_t d_iq3s_grid[512];
static std::mutex g_books_mu;
static bool g_books_set[64] = {false};
static const uint8_t *g_iq2_ptr[64] = {nullptr};
static const uint32_t *g_iq3s_ptr[64] = {nullptr};

int require_books(uint32_t t) {
    if (t != RC_IQ2_XXS && t != RC_IQ3_S) return 1;
    int dev = 0;
    RC_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_books_mu);
    RC_REQUIRE(dev < 64 && g_books_set[dev], "codebooks not set on device %d: call redcuda_set_codebooks first", dev);
    return 1;
}
const uint8_t *books_iq2() { int dev = 0; cudaGetDevice(&dev); return g_iq2_ptr[dev & 63]; }
const uint32_t *books_iq3s() { int dev = 0; cudaGetDevice(&dev); return g_iq3s_ptr[dev & 63]; }

// ---- raw GGUF blocks -> planar ----
__global__ void k_repack(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, uint32_t type, uint64_t nb, uint32_t units_per_block) {
    pdl_prologue();
    // one thread per 2-byte unit of the raw matrix (every field of the three formats starts on an even offset)
    const uint64_t total = nb * units_per_block;
    for (uint64_t u = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; u < total; u += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t b = u / units_per_block;
        const uint32_t off = (uint32_t)(u - b * units_per_block) * 2u;
        const unsigned short v = reinterpret_cast<const unsigned short *>(src)[u];
        *reinterpret_cast<unsigned short *>(dst + rc_planar_dst(type, nb, b, off)) = v;
    }
}

int upload_matrix(uint32_t type, uint32_t nrows, uint32_t ncols, const void *src, bool src_on_device, uint8_t *dst,
                  uint8_t *scratch, cudaStream_t stream) {
    RC_REQUIRE(rc_type_supported(type), "unsupported ggml type %u", type);
    const uint64_t bytes = rc_matrix_bytes(type, nrows, ncols);
    RC_REQUIRE(bytes != 0, "matrix %ux%u of type %u has no valid row size", nrows, ncols, type);
    RC_REQUIRE(((uintptr_t)dst & 15u) == 0, "matrix destination is not 16-byte aligned");
    if (!rc_is_quant(type)) {
        RC_REQUIRE(ncols % 64u == 0, "F32 / F16 / file-layout matrices need a row length that is a multiple of 64 (got %u)", ncols);
        RC_CUDA(cudaMemcpyAsync(dst, src, bytes, src_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, stream));
        return 1;
    }
    const uint8_t *raw = (const uint8_t *)src;
    if (!src_on_device) {
        RC_REQUIRE(scratch != nullptr, "upload_matrix needs scratch for host sources");
        RC_CUDA(cudaMemcpyAsync(scratch, src, bytes, cudaMemcpyHostToDevice, stream));
        raw = scratch;
    }
    RC_REQUIRE(((uintptr_t)raw & 1u) == 0, "raw matrix source is not 2-byte aligned");
    const uint64_t nb = (uint64_t)nrows * (ncols / 256u);
    const uint32_t upb = rc_block_bytes(type) / 2u;
    const uint64_t total = nb * upb;
    const uint32_t grid = (uint32_t)((total + 255u) / 256u < 148u * 16u ? (total + 255u) / 256u : 148u * 16u);
    prof_begin("repack", stream);
    RC_LAUNCH((k_repack), grid ? grid : 1u, 256, 0, stream, raw, dst, type, nb, upb);
    prof_end(stream);
    RC_LAUNCHED();
    return 1;
}

// ---- dequantisation: one thread per group of 8 values ----
__global__ void k_dequant(const uint8_t *__restrict__ base, uint32_t type, uint64_t nb, const uint8_t *iq2, const uint32_t *iq3s, float *__restrict__ out) {
    pdl_prologue();
    const RcBooks bk{iq2, iq3s};
    const uint64_t total = nb * 32u;
    for (uint64_t g = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; g < total; g += (uint64_t)gridDim.x * blockDim.x) {
        float v[8];
        rc_decode8(type, base, nb, g >> 5, (uint32_t)(g & 31u), bk, v);
        float4 *o = reinterpret_cast<float4 *>(out + g * 8u);
        o[0] = make_float4(v[0], v[1], v[2], v[3]);
        o[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}
__global__ void k_dequant_f16(const unsigned short *__restrict__ src, uint64_t n, float *__restrict__ out) {
    pdl_prologue();
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        out[i] = __half2float(__ushort_as_half(src[i]));
}

// Softmax + top-k of one token's logits by one warp; NPL = probabilities per lane (expert i sits in lane i % 32, slot
// i / 32). CG: the logits were written by other blocks of the same launch (read past L1).
// A single warp runs this alone while the rest of the layer waits, so what counts is the length of the dependent chain,
// not the instruction count: every round finds each lane's best slot with a pairwise tree (depth log2 NPL instead of a
// scan of NPL dependent compares), then the warp's best with five shuffle steps; ties go to the lower expert id in both.
template <bool CG, int NPL>
__device__ __forceinline__ void route_one_token_n(const float *__restrict__ l, uint32_t n_expert, uint32_t top_k, uint32_t *__restrict__ ids_row,
                                                  float *__restrict__ weights_row, float *__restrict__ probs_row, const RouteGroup1 &G,
                                                  uint32_t *__restrict__ status, uint32_t lane) {
    float p[NPL];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < NPL; ++j) { const uint32_t i = lane + 32u * j; p[j] = i < n_expert ? (CG ? __ldcg(l + i) : l[i]) : -INFINITY; mx = fmaxf(mx, p[j]); }
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    double den = 0.0;
#pragma unroll
    for (int j = 0; j < NPL; ++j) { const uint32_t i = lane + 32u * j; const float e = i < n_expert ? expf(p[j] - mx) : 0.f; p[j] = e; den += (double)e; }
    for (int o = 16; o; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
    const float inv = (float)(1.0 / den);
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const uint32_t i = lane + 32u * j;
        p[j] = i < n_expert ? p[j] * inv : -2.0f;
        if (probs_row && i < n_expert) probs_row[i] = p[j];
    }
    double sel = 0.0;
    float myw = 0.f;                   // lane k keeps the weight of selection k (top_k <= 64: two per lane)
    float myw2 = 0.f;
    for (uint32_t k = 0; k < top_k; ++k) {
        // lane-local best: a tree over the slots; on equal values the lower slot (= lower expert id) wins
        float tv[NPL]; uint32_t tj[NPL];
#pragma unroll
        for (int j = 0; j < NPL; ++j) { tv[j] = p[j]; tj[j] = (uint32_t)j; }
#pragma unroll
        for (int w = 1; w < NPL; w <<= 1)
#pragma unroll
            for (int j = 0; j + w < NPL; j += 2 * w)
                if (tv[j + w] > tv[j]) { tv[j] = tv[j + w]; tj[j] = tj[j + w]; }
        float bv = tv[0]; uint32_t bi = tv[0] > -3.0f ? lane + 32u * tj[0] : 0xffffffffu;      // NaN compares false: no index
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi >= n_expert) { bi = k; if (status && lane == 0) status[ST_ROUTER_NONFINITE] = 1u; }   // NaN probabilities: nothing compared greater
#pragma unroll
        for (int j = 0; j < NPL; ++j) if (lane + 32u * j == bi) p[j] = -1.0f;
        if (lane == 0) {
            ids_row[k] = bi;
            if (G.sorted) { G.sorted[k] = k; G.uexp[k] = bi; G.ustart[k] = k; G.item_u[k] = k; G.item_p0[k] = k; }      // single token: pair k = group k = item k
            if (G.ids_mirror) G.ids_mirror[k] = bi;
        }
        if (lane == (k & 31u)) { if (k < 32u) myw = bv; else myw2 = bv; }
        sel += (double)bv;
    }
    if (!(sel > 0.0 && sel < (double)INFINITY) && status && lane == 0) status[ST_ROUTER_NONFINITE] = 1u;
    const float invs = (float)(1.0 / sel);
    if (lane < top_k) weights_row[lane] = myw * invs;
    if (lane + 32u < top_k) weights_row[lane + 32u] = myw2 * invs;
    if (G.sorted && lane == 0) { G.ustart[top_k] = top_k; *G.n_unique = top_k; *G.n_items = top_k; if (G.work) { G.work[0] = 0u; G.work[1] = 0u; } }
}
template <bool CG>
__device__ __forceinline__ void route_one_token(const float *__restrict__ l, uint32_t n_expert, uint32_t top_k, uint32_t *__restrict__ ids_row,
                                                float *__restrict__ weights_row, float *__restrict__ probs_row, const RouteGroup1 &G,
                                                uint32_t *__restrict__ status, uint32_t lane) {
    if (n_expert <= 128u) route_one_token_n<CG, 4>(l, n_expert, top_k, ids_row, weights_row, probs_row, G, status, lane);
    else if (n_expert <= 512u) route_one_token_n<CG, 16>(l, n_expert, top_k, ids_row, weights_row, probs_row, G, status, lane);
    else route_one_token_n<CG, 32>(l, n_expert, top_k, ids_row, weights_row, probs_row, G, status, lane);
}

// ---- generic multi-job GEMV ----
// Each block takes one tile (a run of rows) of one job. All jobs of a launch read the same activation rows.
template <int TYPE, int NT>
__device__ __forceinline__ void gemv_tile(const GemvJob &J, uint32_t row0, uint32_t ntok_here, uint32_t tok0, uint32_t ntok,
                                          const float *xs, uint32_t xstride, const SBooks &sb) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, nwarps = blockDim.x >> 5;
    const uint32_t cpr = J.ncols >> 6;
    uint32_t lpr = 32u;
    while (lpr > cpr) lpr >>= 1;
    const uint32_t rw = 32u / lpr, slot = lane / lpr, sub = lane % lpr;
    const uint32_t row_end = min(row0 + J.rows_per_tile, J.nrows);
    (void)ntok;
    for (uint32_t r = row0 + warp * rw; r < row_end; r += nwarps * rw) {
        const uint32_t row = r + slot;
        const bool live = row < row_end;
        const uint64_t rr = live ? row : (uint64_t)(row_end - 1u);   // idle slots recompute a valid row, never store
        float a0[NT], a1[NT];
        row_dot<TYPE, NT>(J.w0, J.nb, rr, J.ncols, lpr, sub, xs, xstride, sb, a0);
        if (J.epi == GEMV_PAIR_SILU) row_dot<TYPE, NT>(J.w1, J.nb, rr, J.ncols, lpr, sub, xs, xstride, sb, a1);
        if (live && sub == 0u) {
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                if ((uint32_t)t >= ntok_here) break;
                float v = a0[t];
                if (J.epi == GEMV_PAIR_SILU) v = silu_mul(a0[t], a1[t]);
                else if (J.epi == GEMV_SIGMOID) v = 1.0f / (1.0f + expf(-v));
                J.out[(size_t)(tok0 + t) * J.out_stride + row] = v;
            }
        }
    }
}

template <int NT>
__global__ void __launch_bounds__(256) k_gemv(const __grid_constant__ GemvArgs A) {
    pdl_prologue();
    extern __shared__ __align__(16) float xs[];
    __shared__ uint2 s_iq2[256];
    __shared__ uint32_t s_iq3s[512];
    uint32_t j = 0;
    while (j + 1u < A.njobs && blockIdx.x >= A.job[j + 1u].tile_begin) ++j;
    const GemvJob &J = A.job[j];
    const uint32_t row0 = (blockIdx.x - J.tile_begin) * J.rows_per_tile;
    load_books(s_iq2, s_iq3s, A.iq2, A.iq3s, 1u << J.type);
    const SBooks sb{s_iq2, s_iq3s};
    const uint32_t xstride = x_padded(J.ncols);
    for (uint32_t tok0 = 0; tok0 < A.ntok; tok0 += NT) {
        const uint32_t nt = min((uint32_t)NT, A.ntok - tok0);
        __syncthreads();
        stage_x<NT>(xs, xstride, A.x, A.x_stride, nullptr, tok0, nt, J.ncols);
        __syncthreads();
        switch (J.type) {
            case RC_F32: gemv_tile<RC_F32, NT>(J, row0, nt, tok0, A.ntok, xs, xstride, sb); break;
            case RC_F16: gemv_tile<RC_F16, NT>(J, row0, nt, tok0, A.ntok, xs, xstride, sb); break;
            case RC_Q6_K: gemv_tile<RC_Q6_K, NT>(J, row0, nt, tok0, A.ntok, xs, xstride, sb); break;
            case RC_IQ2_XXS: gemv_tile<RC_IQ2_XXS, NT>(J, row0, nt, tok0, A.ntok, xs, xstride, sb); break;
            case RC_IQ3_S: gemv_tile<RC_IQ3_S, NT>(J, row0, nt, tok0, A.ntok, xs, xstride, sb); break;
            case RC_Q8_0: gemv_tile<RC_Q8_0, NT>(J, row0, nt, tok0, A.ntok, xs, xstride, sb); break;
            case RC_Q2_K: gemv_tile<RC_Q2_K, NT>(J, row0, nt, tok0, A.ntok, xs, xstride, sb); break;
            case RC_Q4_K: gemv_tile<RC_Q4_K, NT>(J, row0, nt, tok0, A.ntok, xs, xstride, sb); break;
            case RC_Q5_K: gemv_tile<RC_Q5_K, NT>(J, row0, nt, tok0, A.ntok, xs, xstride, sb); break;
            default: break;
        }
    }
    if (NT == 1 && A.tail.ticket) {
        // the block that draws the last ticket sees every block's logits (fence before the ticket, fence after it) and
        // runs the selection for the launch's single token
        __shared__ uint32_t s_last;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_last = atomicAdd(A.tail.ticket, 1u) == gridDim.x - 1u ? 1u : 0u;
        __syncthreads();
        if (s_last) {
            __threadfence();
            if (threadIdx.x == 0) *A.tail.ticket = 0u;
            if (threadIdx.x < 32u) route_one_token<true>(A.tail.logits, A.tail.n_expert, A.tail.top_k, A.tail.ids, A.tail.weights, nullptr, A.tail.G, A.tail.status, threadIdx.x);
        }
    }
}

// Fill tile_begin / rows_per_tile of every job and launch. Jobs must share ncols (they read the same x rows).
int launch_gemv(GemvArgs &A, cudaStream_t stream) {
    RC_REQUIRE(A.njobs >= 1 && A.njobs <= RC_MAX_JOBS, "gemv: bad job count %u", A.njobs);
    RC_REQUIRE(!A.tail.ticket || (A.ntok == 1u && A.tail.n_expert <= 1024u), "gemv: the routing tail serves one token and at most 1024 experts");
    const uint32_t ncols = A.job[0].ncols;
    RC_REQUIRE(ncols % 64u == 0 && ncols >= 64u, "gemv: row length %u is not a multiple of 64", ncols);
    uint64_t total_rows = 0;
    for (uint32_t j = 0; j < A.njobs; ++j) {
        RC_REQUIRE(A.job[j].ncols == ncols, "gemv: jobs of one launch must share the row length");
        RC_REQUIRE(rc_type_supported(A.job[j].type), "gemv: unsupported type %u", A.job[j].type);
        RC_REQUIRE(!rc_is_quant(A.job[j].type) || ncols % 256u == 0, "gemv: quantised rows need a multiple of 256 columns");
        total_rows += A.job[j].nrows;
    }
    uint32_t lpr = 32u;
    while (lpr > (ncols >> 6)) lpr >>= 1;
    const uint32_t rows_per_pass = 8u * (32u / lpr);                 // rows one block covers per sweep of its 8 warps
    // aim at >= 4 blocks per SM when the work allows it, at most 8 sweeps per block
    uint32_t sweeps = (uint32_t)(total_rows / ((uint64_t)rows_per_pass * 148u * 4u));
    sweeps = sweeps < 1u ? 1u : sweeps > 8u ? 8u : sweeps;
    uint32_t tiles = 0;
    for (uint32_t j = 0; j < A.njobs; ++j) {
        A.job[j].rows_per_tile = rows_per_pass * sweeps;
        A.job[j].tile_begin = tiles;
        tiles += (A.job[j].nrows + A.job[j].rows_per_tile - 1u) / A.job[j].rows_per_tile;
    }
    A.iq2 = books_iq2();
    A.iq3s = books_iq3s();
    const int nt = A.ntok <= 1u ? 1 : 4;
    const size_t smem = (size_t)nt * x_padded(ncols) * sizeof(float);
    RC_REQUIRE(smem <= 200u * 1024u, "gemv: row length %u too large for the shared-memory staging", ncols);
    prof_begin(A.tag ? A.tag : "gemv", stream);
    if (nt == 1) {
        if (smem > 48u * 1024u) RC_CUDA(cudaFuncSetAttribute(k_gemv<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        RC_LAUNCH((k_gemv<1>), tiles, 256, smem, stream, A);
    } else {
        if (smem > 48u * 1024u) RC_CUDA(cudaFuncSetAttribute(k_gemv<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        RC_LAUNCH((k_gemv<4>), tiles, 256, smem, stream, A);
    }
    prof_end(stream);
    RC_LAUNCHED();
    return 1;
}

// ---- router: softmax + top-k, one block per token (router_exec.c:102-184 semantics, ties -> lower id) ----
__global__ void __launch_bounds__(256) k_route(const float *__restrict__ logits, uint32_t n_expert, uint32_t top_k,
                                               uint32_t *__restrict__ ids, float *__restrict__ weights, float *__restrict__ probs_out,
                                               uint32_t *__restrict__ status) {
    pdl_prologue();
    extern __shared__ float p[];                 // n_expert probabilities
    __shared__ float s_redf[8];
    __shared__ double s_redd[8];
    __shared__ float s_bv[8];
    __shared__ uint32_t s_bi[8];
    __shared__ float s_selw[REDCUDA_MAX_TOPK];
    const uint32_t tok = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const float *l = logits + (size_t)tok * n_expert;
    float mx = -INFINITY;
    for (uint32_t i = tid; i < n_expert; i += 256u) mx = fmaxf(mx, l[i]);
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (!lane) s_redf[warp] = mx;
    __syncthreads();
    mx = s_redf[0];
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, s_redf[w]);
    double den = 0.0;
    for (uint32_t i = tid; i < n_expert; i += 256u) { const float e = expf(l[i] - mx); p[i] = e; den += (double)e; }
    for (int o = 16; o; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
    if (!lane) s_redd[warp] = den;
    __syncthreads();
    den = 0.0;
    for (int w = 0; w < 8; ++w) den += s_redd[w];
    const float inv = (float)(1.0 / den);
    for (uint32_t i = tid; i < n_expert; i += 256u) { p[i] *= inv; if (probs_out) probs_out[(size_t)tok * n_expert + i] = p[i]; }
    __syncthreads();
    for (uint32_t k = 0; k < top_k; ++k) {
        float bv = -INFINITY; uint32_t bi = 0xffffffffu;
        for (uint32_t i = tid; i < n_expert; i += 256u) { const float v = p[i]; if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; } }
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (!lane) { s_bv[warp] = bv; s_bi[warp] = bi; }
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < 8; ++w) if (s_bv[w] > bv || (s_bv[w] == bv && s_bi[w] < bi)) { bv = s_bv[w]; bi = s_bi[w]; }
            if (bi >= n_expert) { bi = k; if (status) status[ST_ROUTER_NONFINITE] = 1u; }   // NaN probabilities compare false everywhere: no index was chosen
            ids[(size_t)tok * top_k + k] = bi;
            s_selw[k] = bv;
            p[bi] = -1.0f;   // selected: below every probability from now on
        }
        __syncthreads();
    }
    if (tid == 0) {
        double sel = 0.0;
        for (uint32_t k = 0; k < top_k; ++k) sel += (double)s_selw[k];
        if (!(sel > 0.0 && sel < (double)INFINITY) && status) status[ST_ROUTER_NONFINITE] = 1u;
        const float invs = (float)(1.0 / sel);
        for (uint32_t k = 0; k < top_k; ++k) weights[(size_t)tok * top_k + k] = s_selw[k] * invs;
    }
}

// Warp-per-token variant for n_expert <= 1024: the probabilities of a token live in the warp's registers (32 per lane
// at most), every selection round is a register scan plus a 5-step shuffle argmax — no block barriers, so the k rounds
// cost a few hundred dependent instructions instead of 2k barriers. Same arithmetic and tie rule as k_route.
__global__ void __launch_bounds__(256) k_route_warp(const float *__restrict__ logits, uint32_t ntok, uint32_t n_expert, uint32_t top_k,
                                                    uint32_t *__restrict__ ids, float *__restrict__ weights, float *__restrict__ probs_out,
                                                    RouteGroup1 G, uint32_t *__restrict__ status) {
    pdl_prologue();
    const uint32_t lane = threadIdx.x & 31u, tok = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (tok >= ntok) return;
    route_one_token<false>(logits + (size_t)tok * n_expert, n_expert, top_k, ids + (size_t)tok * top_k, weights + (size_t)tok * top_k,
                           probs_out ? probs_out + (size_t)tok * n_expert : nullptr, G, status, lane);
}

int launch_route(const float *logits_dev, uint32_t ntok, uint32_t n_expert, uint32_t top_k, uint32_t *ids_dev, float *weights_dev,
                 float *probs_dev, cudaStream_t stream, const RouteGroup1 *group1) {
    RC_REQUIRE(!group1 || (ntok == 1u && n_expert <= 1024u), "router: the fused grouping serves one token and at most 1024 experts");
    const RouteGroup1 G = group1 ? *group1 : RouteGroup1{};
    RC_REQUIRE(top_k >= 1 && top_k <= REDCUDA_MAX_TOPK && top_k <= n_expert, "router: top_k %u out of range", top_k);
    RC_REQUIRE(n_expert <= 8192u, "router: too many experts (%u)", n_expert);
    if (!ntok) return 1;
    prof_begin("route", stream);
    uint32_t *st = status_words();
    if (n_expert <= 1024u) RC_LAUNCH((k_route_warp), (ntok + 7u) / 8u, 256, 0, stream, logits_dev, ntok, n_expert, top_k, ids_dev, weights_dev, probs_dev, G, st);
    else RC_LAUNCH((k_route), ntok, 256, n_expert * sizeof(float), stream, logits_dev, n_expert, top_k, ids_dev, weights_dev, probs_dev, st);
    prof_end(stream);
    RC_LAUNCHED();
    return 1;
}

// out[t] = sigmoid(w . x[t]) for one F32 row w (the shared-expert gate), fp64 accumulation; one block per token.
__global__ void __launch_bounds__(256) k_vec_sigmoid(const float *__restrict__ w, const float *__restrict__ x, uint32_t x_stride, uint32_t ncols,
                                                     float *__restrict__ out) {
    pdl_prologue();
    __shared__ double red[8];
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    const float *xr = x + (size_t)t * x_stride;
    double acc = 0.0;
    for (uint32_t k = tid * 4u; k < ncols; k += 1024u) {
        const float4 a = *reinterpret_cast<const float4 *>(w + k), b = *reinterpret_cast<const float4 *>(xr + k);
        acc += (double)a.x * b.x + (double)a.y * b.y + (double)a.z * b.z + (double)a.w * b.w;
    }
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((tid & 31u) == 0) red[tid >> 5] = acc;
    __syncthreads();
    if (tid == 0) {
        double tot = 0.0;
        for (int i = 0; i < 8; ++i) tot += red[i];
        out[t] = (float)(1.0 / (1.0 + exp(-tot)));
    }
}

// Router logits of a batch: logits[t][e] = (float) sum_k (double) x[t][k] * (double) w[e][k], F32 weights
// (rl_quant_row_dot on an F32 row accumulates in double, native/redlite_native_quant_cpu.c:198-212, and the top-k that
// follows must not depend on a summation order). The multi-token GEMV re-reads the matrix for every four tokens; this
// is a small tiled fp64 GEMM instead: block = 32 tokens x 64 experts, K in tiles of 64 staged as doubles in shared
// memory (the next tile is fetched into registers while the current one is multiplied); each of the 8 warps owns a
// 16 x 16 tile of the result as 2 x 2 fragments of the fp64 tensor-core instruction (mma.sync.m8n8k4.f64: four 8-byte
// shared loads per four instructions; the row pitch of 68 doubles keeps those loads conflict-free). Batches that do
// not fill half of that tile take a block of 16 tokens x 32 experts with one fragment per warp.
constexpr uint32_t RL_KT = 64u, RL_PITCH = RL_KT + 4u;
template <uint32_t FR>            // fragments per warp and direction: block = 16 FR tokens x 32 FR experts
__global__ void __launch_bounds__(256) k_router_logits(const float *__restrict__ w, const float *__restrict__ x, uint32_t x_stride, uint32_t ntok,
                                                       uint32_t n_expert, uint32_t ncols, float *__restrict__ logits) {
    pdl_prologue();
    constexpr uint32_t TT = 16u * FR, TE = 32u * FR;
    extern __shared__ __align__(16) double rl_smem[];
    double *xs = rl_smem, *ws = rl_smem + TT * RL_PITCH;
    const uint32_t tid = threadIdx.x;
    const uint32_t t0 = blockIdx.x * TT, e0 = blockIdx.y * TE;
    // staging roles: a tile row is 64 floats = 16 float4; thread -> (row tid / 16 + 16 i, float4 tid % 16)
    const uint32_t sr = tid >> 4, sc = (tid & 15u) * 4u;
    constexpr uint32_t NW = TE / 16u, NX = TT / 16u;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 rw[NW], rx[NX];
    auto fetch = [&](uint32_t k0) {
#pragma unroll
        for (uint32_t i = 0; i < NW; ++i) rw[i] = e0 + sr + 16u * i < n_expert ? __ldg(reinterpret_cast<const float4 *>(w + (size_t)(e0 + sr + 16u * i) * ncols + k0 + sc)) : zero;
#pragma unroll
        for (uint32_t i = 0; i < NX; ++i) rx[i] = t0 + sr + 16u * i < ntok ? *reinterpret_cast<const float4 *>(x + (size_t)(t0 + sr + 16u * i) * x_stride + k0 + sc) : zero;
    };
    fetch(0u);
    // warp -> (token group of 8 FR, expert group of 8 FR); lane -> A element (row lane/4, k lane%4), B element (k lane%4,
    // column lane/4), C elements (row lane/4, columns 2*(lane%4), +1)
    const uint32_t warp = tid >> 5, lane = tid & 31u, th = warp >> 2, eq = warp & 3u, fr = lane >> 2, fk = lane & 3u;
    double acc[FR][FR][2];
#pragma unroll
    for (uint32_t i = 0; i < FR; ++i)
#pragma unroll
        for (uint32_t j = 0; j < FR; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;
    for (uint32_t k0 = 0; k0 < ncols; k0 += RL_KT) {
        __syncthreads();                                   // the previous tile is no longer read
#pragma unroll
        for (uint32_t i = 0; i < NW; ++i) { double *d = ws + (sr + 16u * i) * RL_PITCH + sc; d[0] = rw[i].x; d[1] = rw[i].y; d[2] = rw[i].z; d[3] = rw[i].w; }
#pragma unroll
        for (uint32_t i = 0; i < NX; ++i) { double *d = xs + (sr + 16u * i) * RL_PITCH + sc; d[0] = rx[i].x; d[1] = rx[i].y; d[2] = rx[i].z; d[3] = rx[i].w; }
        __syncthreads();
        if (k0 + RL_KT < ncols) fetch(k0 + RL_KT);
        const double *a = xs + (th * 8u * FR + fr) * RL_PITCH + fk, *b = ws + (eq * 8u * FR + fr) * RL_PITCH + fk;
#pragma unroll
        for (uint32_t kk = 0; kk < RL_KT; kk += 4u) {
            double av[FR], bv[FR];
#pragma unroll
            for (uint32_t i = 0; i < FR; ++i) { av[i] = a[i * 8u * RL_PITCH + kk]; bv[i] = b[i * 8u * RL_PITCH + kk]; }
#pragma unroll
            for (uint32_t i = 0; i < FR; ++i)
#pragma unroll
                for (uint32_t j = 0; j < FR; ++j)
                    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};" : "+d"(acc[i][j][0]), "+d"(acc[i][j][1]) : "d"(av[i]), "d"(bv[j]));
        }
    }
#pragma unroll
    for (uint32_t i = 0; i < FR; ++i)
#pragma unroll
        for (uint32_t j = 0; j < FR; ++j) {
            const uint32_t t = t0 + (th * FR + i) * 8u + fr, e = e0 + (eq * FR + j) * 8u + 2u * fk;
            if (t < ntok) {
                if (e < n_expert) logits[(size_t)t * n_expert + e] = (float)acc[i][j][0];
                if (e + 1u < n_expert) logits[(size_t)t * n_expert + e + 1u] = (float)acc[i][j][1];
            }
        }
}

int launch_router_logits(const float *w, const float *x, uint32_t x_stride, uint32_t ntok, uint32_t n_expert, uint32_t ncols, float *logits, cudaStream_t stream) {
    RC_REQUIRE(ncols % RL_KT == 0 && x_stride % 4u == 0, "router logits: %u columns (stride %u) is not a multiple of %u", ncols, x_stride, RL_KT);
    if (!ntok) return 1;
    prof_begin("moe_router_logits", stream);
    if (ntok >= 256u && n_expert >= 64u) {
        const size_t smem = (size_t)(32u + 64u) * RL_PITCH * sizeof(double);
        RC_CUDA(cudaFuncSetAttribute(k_router_logits<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        RC_LAUNCH((k_router_logits<2>), dim3((ntok + 31u) / 32u, (n_expert + 63u) / 64u), 256, smem, stream, w, x, x_stride, ntok, n_expert, ncols, logits);
    } else {
        const size_t smem = (size_t)(16u + 32u) * RL_PITCH * sizeof(double);
        RC_LAUNCH((k_router_logits<1>), dim3((ntok + 15u) / 16u, (n_expert + 31u) / 32u), 256, smem, stream, w, x, x_stride, ntok, n_expert, ncols, logits);
    }
    prof_end(stream);
    RC_LAUNCHED();
    return 1;
}

int launch_vec_sigmoid(const float *w, const float *x, uint32_t x_stride, uint32_t ncols, uint32_t ntok, float *out, cudaStream_t stream) {
    RC_REQUIRE(ncols % 4u == 0, "vec_sigmoid: %u columns is not a multiple of 4", ncols);
    if (!ntok) return 1;
    prof_begin("moe_shared_gate", stream);
    RC_LAUNCH((k_vec_sigmoid), ntok, 256, 0, stream, w, x, x_stride, ncols, out);
    prof_end(stream);
    RC_LAUNCHED();
    return 1;
}

}  // namespace rc

using namespace rc;

// ================================================================================================= C ABI
extern "C" {

uint32_t redcuda_abi_version(void) { return REDCUDA_ABI_VERSION; }
const char *redcuda_last_error(void) { return rc::t_err.c_str(); }
uint64_t redcuda_launch_count(void) { return rc::g_launches.load(); }

int redcuda_profile_enable(int on) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    for (auto &r : g_prof) { if (r.a) cudaEventDestroy(r.a); if (r.b) cudaEventDestroy(r.b); }
    g_prof.clear();
    g_prof_on = on != 0;
    return 1;
}

int redcuda_profile_report(char *buf, size_t cap) {
    if (!buf || !cap) return 0;
    cudaDeviceSynchronize();
    std::lock_guard<std::mutex> lk(g_prof_mu);
    std::map<std::string, std::pair<uint64_t, double>> agg;
    for (auto &r : g_prof) {
        float ms = 0.f;
        if (r.a && r.b && cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) { auto &e = agg[r.tag]; e.first += 1; e.second += ms; }
    }
    cudaGetLastError();
    size_t pos = 0; int n = 0;
    buf[0] = 0;
    for (auto &kv : agg) {
        const int w = snprintf(buf + pos, cap - pos, "%s %llu %.6f\n", kv.first.c_str(), (unsigned long long)kv.second.first, kv.second.second);
        if (w < 0 || (size_t)w >= cap - pos) break;
        pos += (size_t)w; ++n;
    }
    return n;
}

int redcuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

int redcuda_set_device(int device) {
    if (!require_device()) return 0;
    RC_CUDA(cudaSetDevice(device));
    return 1;
}

int redcuda_set_codebooks(const uint8_t *iq2xxs_grid, uint32_t iq2xxs_bytes, const uint32_t *iq3s_grid, uint32_t iq3s_count) {
    if (!require_device()) return 0;
    RC_REQUIRE(iq2xxs_grid && iq2xxs_bytes == 2048u, "IQ2_XXS grid must be 256 x 8 bytes");
    RC_REQUIRE(iq3s_grid && iq3s_count == 512u, "IQ3_S grid must be 512 entries");
    for (uint32_t i = 0; i < 2048u; ++i) RC_REQUIRE(iq2xxs_grid[i] == 0x08 || iq2xxs_grid[i] == 0x19 || iq2xxs_grid[i] == 0x2b, "IQ2_XXS grid byte %u is not one of 0x08/0x19/0x2b", i);
    int dev = 0;
    RC_CUDA(cudaGetDevice(&dev));
    RC_REQUIRE(dev < 64, "device index %d out of range", dev);
    RC_CUDA(cudaMemcpyToSymbol(d_iq2_grid, iq2xxs_grid, 2048));
    RC_CUDA(cudaMemcpyToSymbol(d_iq3s_grid, iq3s_grid, 2048));
    void *p2 = nullptr, *p3 = nullptr;
    RC_CUDA(cudaGetSymbolAddress(&p2, d_iq2_grid));
    RC_CUDA(cudaGetSymbolAddress(&p3, d_iq3s_grid));
    if (!mma_set_luts(iq2xxs_grid)) return 0;
    std::lock_guard<std::mutex> lk(g_books_mu);
    g_iq2_ptr[dev] = (const uint8_t *)p2;
    g_iq3s_ptr[dev] = (const uint32_t *)p3;
    g_books_set[dev] = true;
    return 1;
}

int redcuda_set_codebooks_ext(const uint32_t *iq3xxs_grid, uint32_t iq3xxs_count, const uint64_t *iq2s_grid, uint32_t iq2s_count,
                              const int8_t *iq4nl_values, uint32_t iq4nl_count) {
    if (!require_device()) return 0;
    RC_REQUIRE(iq3xxs_grid && iq3xxs_count == 256u, "IQ3_XXS grid must be 256 entries");
    RC_REQUIRE(iq2s_grid && iq2s_count == 1024u, "IQ2_S grid must be 1024 entries");
    RC_REQUIRE(iq4nl_values && iq4nl_count == 16u, "IQ4_NL values must be 16 entries");
    return kq_set_iq_tables(iq3xxs_grid, iq2s_grid, iq4nl_values);
}

int redcuda_set_codebooks_xs(const int8_t *iq2xs_grid, uint32_t iq2xs_count, const int8_t *iq1m_grid, uint32_t iq1m_count) {
    if (!require_device()) return 0;
    RC_REQUIRE(iq2xs_grid && iq2xs_count == 4096u, "IQ2_XS grid must be 512 x 8 values");
    RC_REQUIRE(iq1m_grid && iq1m_count == 16384u, "IQ1_M grid must be 2048 x 8 values");
    return kq_set_xs_tables(iq2xs_grid, iq1m_grid);
}

int redcuda_quant_dequant_rows(uint32_t type, const uint8_t *rows, uint32_t nrows, uint32_t ncols, float *out) {
    if (!require_device()) return 0;
    RC_REQUIRE(rows && out && nrows && ncols, "dequant: null or empty argument");
    if (kq_supported(type)) return kq_dequant_rows(type, rows, nrows, ncols, out);      // Q8_0 / Q2_K / Q4_K / Q5_K: redcuda_kquants.cu
    if (!require_books(type)) return 0;
    RC_REQUIRE(rc_type_supported(type), "dequant: unsupported ggml type %u", type);
    const uint64_t bytes = rc_matrix_bytes(type, nrows, ncols);
    RC_REQUIRE(bytes, "dequant: %u columns is not a valid row length for type %u", ncols, type);
    const size_t n = (size_t)nrows * ncols;
    if (type == RC_F32) { memcpy(out, rows, n * 4u); return 1; }   // a copy, as in the reference (quant_cpu.c:159)
    DevMem raw, planar, o;
    if (!raw.alloc(bytes) || !planar.alloc(bytes) || !o.alloc(n * 4u)) return 0;
    cudaStream_t s = 0;
    if (type == RC_F16) {
        RC_CUDA(cudaMemcpyAsync(raw.p, rows, bytes, cudaMemcpyHostToDevice, s));
        RC_LAUNCH((k_dequant_f16), (unsigned)((n + 255u) / 256u < 4096u ? (n + 255u) / 256u : 4096u), 256, 0, s, raw.as<unsigned short>(), n, o.as<float>());
        RC_LAUNCHED();
    } else {
        if (!upload_matrix(type, nrows, ncols, rows, false, planar.as<uint8_t>(), raw.as<uint8_t>(), s)) return 0;
        const uint64_t nb = (uint64_t)nrows * (ncols / 256u), groups = nb * 32u;
        RC_LAUNCH((k_dequant), (unsigned)((groups + 255u) / 256u < 4096u ? (groups + 255u) / 256u : 4096u), 256, 0, s, planar.as<uint8_t>(), type, nb, books_iq2(), books_iq3s(), o.as<float>());
        RC_LAUNCHED();
    }
    RC_CUDA(cudaMemcpyAsync(out, o.p, n * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    return 1;
}

int redcuda_quant_matvec(uint32_t type, const uint8_t *w, uint32_t nrows, uint32_t ncols, const float *x, uint32_t ntok, float *out) {
    if (!require_device()) return 0;
    RC_REQUIRE(w && x && out && nrows && ncols && ntok, "matvec: null or empty argument");
    if (kq_supported(type)) return kq_matvec(type, w, nrows, ncols, x, ntok, out);
    if (!require_books(type)) return 0;
    RC_REQUIRE(rc_type_supported(type), "matvec: unsupported ggml type %u", type);
    const uint64_t bytes = rc_matrix_bytes(type, nrows, ncols);
    RC_REQUIRE(bytes, "matvec: %u columns is not a valid row length for type %u", ncols, type);
    DevMem raw, planar, xd, od;
    if (!raw.alloc(bytes) || !planar.alloc(bytes) || !xd.alloc((size_t)ntok * ncols * 4u) || !od.alloc((size_t)ntok * nrows * 4u)) return 0;
    cudaStream_t s = 0;
    if (!upload_matrix(type, nrows, ncols, w, false, planar.as<uint8_t>(), raw.as<uint8_t>(), s)) return 0;
    RC_CUDA(cudaMemcpyAsync(xd.p, x, (size_t)ntok * ncols * 4u, cudaMemcpyHostToDevice, s));
    GemvArgs A{};
    A.njobs = 1; A.ntok = ntok; A.x = xd.as<float>(); A.x_stride = ncols;
    A.job[0].w0 = planar.as<uint8_t>(); A.job[0].w1 = nullptr; A.job[0].out = od.as<float>(); A.job[0].nb = (uint64_t)nrows * (ncols / 256u);
    A.job[0].type = type; A.job[0].nrows = nrows; A.job[0].ncols = ncols; A.job[0].out_stride = nrows; A.job[0].epi = GEMV_STORE;
    if (!launch_gemv(A, s)) return 0;
    RC_CUDA(cudaMemcpyAsync(out, od.p, (size_t)ntok * nrows * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    return 1;
}

int redcuda_router_select_softmax_topk(const float *logits, uint32_t ntok, uint32_t n_expert, uint32_t top_k,
                                       uint32_t *ids, float *weights, float *probs) {
    if (!require_device()) return 0;
    RC_REQUIRE(logits && ids && weights && n_expert && top_k && top_k <= n_expert, "invalid router top-k selection arguments");
    if (!ntok) return 1;
    DevMem l, i, w, p;
    if (!l.alloc((size_t)ntok * n_expert * 4u) || !i.alloc((size_t)ntok * top_k * 4u) || !w.alloc((size_t)ntok * top_k * 4u)) return 0;
    if (probs && !p.alloc((size_t)ntok * n_expert * 4u)) return 0;
    cudaStream_t s = 0;
    RC_CUDA(cudaMemcpyAsync(l.p, logits, (size_t)ntok * n_expert * 4u, cudaMemcpyHostToDevice, s));
    if (!launch_route(l.as<float>(), ntok, n_expert, top_k, i.as<uint32_t>(), w.as<float>(), probs ? p.as<float>() : nullptr, s)) return 0;
    RC_CUDA(cudaMemcpyAsync(ids, i.p, (size_t)ntok * top_k * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaMemcpyAsync(weights, w.p, (size_t)ntok * top_k * 4u, cudaMemcpyDeviceToHost, s));
    if (probs) RC_CUDA(cudaMemcpyAsync(probs, p.p, (size_t)ntok * n_expert * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    return status_failed() ? 0 : 1;
}

}  // extern "C"
