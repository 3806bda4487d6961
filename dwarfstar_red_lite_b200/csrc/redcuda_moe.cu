// Resident MoE layer: router, expert-grouped routed FFN, sigmoid-gated shared expert.
//
// Pass structure (one stream, no host round trip; the reference's GPU path needs the same dependency chain,
// native/redmetal_engine.m:1733-1863):
//   1. one multi-job GEMV over the token activations: router logits (F32 rows, fp64 accumulation), shared gate/up with
//      SiLU*mul fused, shared-expert scalar gate with the sigmoid fused
//   2. softmax + top-k per token (ties -> lower id)
//   3. (token, expert) pairs grouped by expert on the device — the layout the reference builds on the CPU for its
//      batched path (expert_start / pair_token, native/redmetal_topk.h:182-190)
//   4. gate/up of every selected expert over the tokens routed to it (weights decoded once per pass of up to 4 tokens)
//   5. shared down projection
//   6. down projection per pair
//   7. per-token combine in router order: out = resid + sum_k w_k * expert_k + shared * scalar
#define RC_PDL_DEFAULT 0
#include "redcuda_common.cuh"
#include "redcuda_dot.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_moe_mma.cuh"
#include "redcuda_tc_gemm.cuh"
#include "../../include/redcuda.h"

#include <new>
#include <type_traits>
#include <stdlib.h>

namespace rc {

struct MoeArgs {
    const uint8_t *w0, *w1;        // expert matrices of the shard, back to back (gate / up, or down / unused)
    uint64_t mat_bytes, nb;        // bytes and blocks of one expert matrix
    uint32_t type, nrows, ncols;   // per expert matrix
    uint32_t expert_begin, rows_per_tile, n_local;
    uint32_t *status;
    const uint32_t *sorted, *uexp, *ustart, *n_unique;
    const float *x; uint32_t x_stride, x_div;   // activation row of pair p = x + (p / x_div) * x_stride
    float *out; uint32_t out_stride;            // result row of pair p = out + p * out_stride
    uint32_t pair_silu;                         // 1: out = SiLU(w0.x) * (w1.x); 0: out = w0.x
    const uint8_t *iq2; const uint32_t *iq3s;
};

template <int TYPE, int NT>
__device__ __forceinline__ void moe_tile(const MoeArgs &A, const uint8_t *m0, const uint8_t *m1, uint32_t row0, uint32_t p0, uint32_t nt,
                                         const float *xs, uint32_t xstride, const SBooks &sb) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, nwarps = blockDim.x >> 5;
    const uint32_t cpr = A.ncols >> 6;
    uint32_t lpr = 32u;
    while (lpr > cpr) lpr >>= 1;
    const uint32_t rw = 32u / lpr, slot = lane / lpr, sub = lane % lpr;
    const uint32_t row_end = min(row0 + A.rows_per_tile, A.nrows);
    for (uint32_t r = row0 + warp * rw; r < row_end; r += nwarps * rw) {
        const uint32_t row = r + slot;
        const bool live = row < row_end;
        const uint64_t rr = live ? row : (uint64_t)(row_end - 1u);
        float a0[NT], a1[NT];
        row_dot<TYPE, NT>(m0, A.nb, rr, A.ncols, lpr, sub, xs, xstride, sb, a0);
        if (A.pair_silu) row_dot<TYPE, NT>(m1, A.nb, rr, A.ncols, lpr, sub, xs, xstride, sb, a1);
        if (live && sub == 0u) {
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                if ((uint32_t)t >= nt) break;
                const uint32_t p = A.sorted[p0 + t];
                A.out[(size_t)p * A.out_stride + row] = A.pair_silu ? silu_mul(a0[t], a1[t]) : a0[t];
            }
        }
    }
}

template <int NT>
__global__ void __launch_bounds__(256) k_moe_experts(const __grid_constant__ MoeArgs A) {
    pdl_prologue();
    extern __shared__ __align__(16) float xs[];
    __shared__ uint2 s_iq2[256];
    __shared__ uint32_t s_iq3s[512];
    const uint32_t u = blockIdx.y;
    if (u >= *A.n_unique) return;
    const uint32_t e = A.uexp[u] - A.expert_begin, ps = A.ustart[u], pe = A.ustart[u + 1u];
    if (e >= A.n_local) { if (A.status && threadIdx.x == 0) A.status[ST_EXPERT_RANGE] = 1u; return; }     // never index the arena with a foreign id
    const uint8_t *m0 = A.w0 + (size_t)e * A.mat_bytes, *m1 = A.w1 ? A.w1 + (size_t)e * A.mat_bytes : nullptr;
    const uint32_t row0 = blockIdx.x * A.rows_per_tile;
    load_books(s_iq2, s_iq3s, A.iq2, A.iq3s, 1u << A.type);
    const SBooks sb{s_iq2, s_iq3s};
    const uint32_t xstride = x_padded(A.ncols);
    for (uint32_t p0 = ps; p0 < pe; p0 += NT) {
        const uint32_t nt = min((uint32_t)NT, pe - p0);
        __syncthreads();
        {   // stage the activation rows of pairs [p0, p0 + nt)
            const uint32_t n4 = A.ncols >> 2;
            for (uint32_t i = threadIdx.x; i < NT * n4; i += blockDim.x) {
                const uint32_t t = i / n4, k = (i - t * n4) << 2;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t < nt) v = *reinterpret_cast<const float4 *>(A.x + (size_t)(A.sorted[p0 + t] / A.x_div) * A.x_stride + k);
                *reinterpret_cast<float4 *>(xs + t * xstride + xi(k)) = v;
            }
        }
        __syncthreads();
        switch (A.type) {
            case RC_IQ2_XXS: moe_tile<RC_IQ2_XXS, NT>(A, m0, m1, row0, p0, nt, xs, xstride, sb); break;
            case RC_IQ3_S: moe_tile<RC_IQ3_S, NT>(A, m0, m1, row0, p0, nt, xs, xstride, sb); break;
            case RC_Q6_K: moe_tile<RC_Q6_K, NT>(A, m0, m1, row0, p0, nt, xs, xstride, sb); break;
            default: break;
        }
    }
}

// Group pairs by expert: sorted[] = pair ids, expert by expert (ascending expert id); uexp / ustart list the experts
// that received at least one pair; n_unique their count. Every expert's pairs are also cut into work items of at most
// item_tok pairs (item_u = slot in uexp, item_p0 = first position in sorted[]), so that kernels which take one item
// per block see equal-sized work whatever the routing skew. One block of 1024 threads, expert_count <= 1024.
// Ownership: expert g belongs to the shard when g = expert_begin + i * expert_stride for some i < expert_count (i is the
// index of its matrices in the shard; uexp holds expert_begin + i). Pairs of other shards are counted in *bad, or just
// left out when skip_foreign is set (the all-gather form of expert parallelism hands every rank every pair).
__device__ __forceinline__ uint32_t shard_local(uint32_t g, uint32_t begin, uint32_t stride, uint32_t count) {
    const uint32_t d = g - begin;
    if (g < begin || d % stride) return 0xffffffffu;
    const uint32_t i = d / stride;
    return i < count ? i : 0xffffffffu;
}

__global__ void __launch_bounds__(1024) k_group_pairs(const uint32_t *__restrict__ pair_expert, uint32_t npairs, uint32_t expert_begin, uint32_t expert_stride,
                                                      uint32_t skip_foreign, uint32_t expert_count, uint32_t item_tok, uint32_t *__restrict__ sorted, uint32_t *__restrict__ uexp,
                                                      uint32_t *__restrict__ ustart, uint32_t *__restrict__ n_unique, uint32_t *__restrict__ item_u,
                                                      uint32_t *__restrict__ item_p0, uint32_t *__restrict__ n_items, uint32_t *__restrict__ bad, uint32_t *__restrict__ work, const EpWait wait) {
    pdl_prologue();
    ep_wait_all(wait);         // peer-memory exchange: the pairs' ids are written by the other ranks; wait until every rank's rows have landed
    if (work && threadIdx.x < 2u) work[threadIdx.x] = 0u;      // unit counters of the persistent expert kernels that follow
    __shared__ uint32_t cnt[1024], start[1024], wsum[32], wsum2[32], wsum3[32];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    cnt[tid] = 0;
    __syncthreads();
    for (uint32_t p = tid; p < npairs; p += 1024u) {
        const uint32_t e = shard_local(pair_expert[p], expert_begin, expert_stride, expert_count);
        if (e != 0xffffffffu) atomicAdd(&cnt[e], 1u); else if (!skip_foreign) atomicAdd(bad, 1u);   // a pair outside the shard is reported, not run
    }
    __syncthreads();
    // exclusive scans over experts of (count), (count > 0) and (items)
    const uint32_t c = tid < expert_count ? cnt[tid] : 0u, f = c ? 1u : 0u, it = (c + item_tok - 1u) / item_tok;
    uint32_t sc = c, sf = f, si = it;
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t a = __shfl_up_sync(0xffffffffu, sc, o), b = __shfl_up_sync(0xffffffffu, sf, o), d = __shfl_up_sync(0xffffffffu, si, o);
        if ((int)lane >= o) { sc += a; sf += b; si += d; }
    }
    if (lane == 31u) { wsum[warp] = sc; wsum2[warp] = sf; wsum3[warp] = si; }
    __syncthreads();
    if (warp == 0) {
        uint32_t a = wsum[lane], b = wsum2[lane], d = wsum3[lane];
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t ua = __shfl_up_sync(0xffffffffu, a, o), ub = __shfl_up_sync(0xffffffffu, b, o), ud = __shfl_up_sync(0xffffffffu, d, o);
            if ((int)lane >= o) { a += ua; b += ub; d += ud; }
        }
        wsum[lane] = a; wsum2[lane] = b; wsum3[lane] = d;
    }
    __syncthreads();
    const uint32_t basec = warp ? wsum[warp - 1u] : 0u, basef = warp ? wsum2[warp - 1u] : 0u, basei = warp ? wsum3[warp - 1u] : 0u;
    const uint32_t exc = basec + sc - c, exf = basef + sf - f, exi = basei + si - it;
    start[tid] = exc;
    if (f) { uexp[exf] = expert_begin + tid; ustart[exf] = exc; }
    for (uint32_t j = 0; j < it; ++j) { item_u[exi + j] = exf; item_p0[exi + j] = exc + j * item_tok; }
    if (tid == 1023u) { const uint32_t nu = exf + f; *n_unique = nu; ustart[nu] = exc + c; *n_items = exi + it; }
    cnt[tid] = 0;
    __syncthreads();
    for (uint32_t p = tid; p < npairs; p += 1024u) {
        const uint32_t e = shard_local(pair_expert[p], expert_begin, expert_stride, expert_count);
        if (e != 0xffffffffu) sorted[start[e] + atomicAdd(&cnt[e], 1u)] = p;
    }
}

// Single-token case: the k selected experts are distinct, so every pair is its own group and its own work item.
__global__ void k_group_trivial(const uint32_t *__restrict__ pair_expert, uint32_t npairs, uint32_t *__restrict__ sorted,
                                uint32_t *__restrict__ uexp, uint32_t *__restrict__ ustart, uint32_t *__restrict__ n_unique,
                                uint32_t *__restrict__ item_u, uint32_t *__restrict__ item_p0, uint32_t *__restrict__ n_items, uint32_t *__restrict__ work) {
    pdl_prologue();
    const uint32_t i = threadIdx.x;
    if (work && i < 2u) work[i] = 0u;
    if (i < npairs) { sorted[i] = i; uexp[i] = pair_expert[i]; ustart[i] = i; item_u[i] = i; item_p0[i] = i; }
    if (i == 0) { ustart[npairs] = npairs; *n_unique = npairs; *n_items = npairs; }
}

// out[t] = resid[t] + (sum_k w[t][k] * pair_out[t*k + kk] + shared[t] * scalar[t]); k may be 0 (shared part only).
__global__ void __launch_bounds__(256) k_moe_combine(const float *__restrict__ pair_out, const float *__restrict__ w, uint32_t top_k,
                                                     const float *__restrict__ shared, const float *__restrict__ scalar,
                                                     const float *__restrict__ resid, float *__restrict__ out, uint32_t hidden,
                                                     const uint32_t *__restrict__ pair_row) {
    pdl_prologue();
    const uint32_t t = blockIdx.y;
    const uint32_t r = (blockIdx.x * 256u + threadIdx.x) * 4u;
    if (r >= hidden) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t k = 0; k < top_k; ++k) {
        const float wk = w[(size_t)t * top_k + k];
        if (wk == 0.f) continue;           // also the mark of a pair that another shard computes: its row was never written
        const size_t prow = pair_row ? pair_row[(size_t)t * top_k + k] : (size_t)t * top_k + k;   // where the pair's expert output sits
        const float4 v = *reinterpret_cast<const float4 *>(pair_out + prow * hidden + r);
        acc.x += wk * v.x; acc.y += wk * v.y; acc.z += wk * v.z; acc.w += wk * v.w;
    }
    if (shared) {
        const float s = scalar ? scalar[t] : 1.0f;
        const float4 v = *reinterpret_cast<const float4 *>(shared + (size_t)t * hidden + r);
        acc.x += v.x * s; acc.y += v.y * s; acc.z += v.z * s; acc.w += v.w * s;
    }
    if (resid) {
        const float4 v = *reinterpret_cast<const float4 *>(resid + (size_t)t * hidden + r);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4 *>(out + (size_t)t * hidden + r) = acc;
}

// Combine of the all-gather form of expert parallelism: every rank holds every token's ids / weights;
// out[t] = sum over the pairs of token t whose expert THIS shard holds of w * pair_out[t * top_k + k], plus add[t - add_begin]
// for the add_count tokens from add_begin on (the rank's own tokens: their shared-expert part rides along in the
// reduce-scatter). A token without local pairs gets zeros (or its add row).
__global__ void __launch_bounds__(256) k_ep_combine(const float *__restrict__ pair_out, const uint32_t *__restrict__ ids, const float *__restrict__ w, uint32_t top_k,
                                                    uint32_t begin, uint32_t stride, uint32_t count, const float *__restrict__ add, uint32_t add_begin, uint32_t add_count,
                                                    float *__restrict__ out, uint32_t hidden) {
    pdl_prologue();
    const uint32_t t = blockIdx.y;
    const uint32_t r = (blockIdx.x * 256u + threadIdx.x) * 4u;
    if (r >= hidden) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t k = 0; k < top_k; ++k) {
        const size_t p = (size_t)t * top_k + k;
        if (shard_local(ids[p], begin, stride, count) == 0xffffffffu) continue;       // another shard computes this pair; its row here was never written
        const float wk = w[p];
        const float4 v = *reinterpret_cast<const float4 *>(pair_out + p * hidden + r);
        acc.x += wk * v.x; acc.y += wk * v.y; acc.z += wk * v.z; acc.w += wk * v.w;
    }
    if (add && t >= add_begin && t - add_begin < add_count) {
        const float4 v = *reinterpret_cast<const float4 *>(add + (size_t)(t - add_begin) * hidden + r);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4 *>(out + (size_t)t * hidden + r) = acc;
}

// The same sum delivered through peer memory: token t's row is stored into the slot its owner keeps for this rank
// (NVLink stores; zeros when no local expert served the token, so that the owner can add all slots), then the flag.
__global__ void __launch_bounds__(256) k_ep_combine_push(const float *__restrict__ pair_out, const uint32_t *__restrict__ ids, const float *__restrict__ w, uint32_t top_k,
                                                         uint32_t begin, uint32_t stride, uint32_t count, const __grid_constant__ EpPush P, uint32_t hidden) {
    pdl_prologue();
    const uint32_t t = blockIdx.y;
    const uint32_t r = (blockIdx.x * 256u + threadIdx.x) * 4u;
    if (r < hidden) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t k = 0; k < top_k; ++k) {
            const size_t p = (size_t)t * top_k + k;
            if (shard_local(ids[p], begin, stride, count) == 0xffffffffu) continue;
            const float wk = w[p];
            const float4 v = *reinterpret_cast<const float4 *>(pair_out + p * hidden + r);
            acc.x += wk * v.x; acc.y += wk * v.y; acc.z += wk * v.z; acc.w += wk * v.w;
        }
        const uint32_t owner = t / P.tokens, tl = t - owner * P.tokens;
        float *dst = reinterpret_cast<float *>(P.peers.base[owner] + P.off_part) + ((size_t)P.peers.rank * P.tokens + tl) * hidden + r;
        *reinterpret_cast<float4 *>(dst) = acc;
    }
    ep_signal_all(P.peers, P.off_flag, P.seq, P.ticket, gridDim.x * gridDim.y);
}

}  // namespace rc

using namespace rc;

struct redcuda_moe {
    redcuda_moe_desc d;
    int device = 0;
    DevMem wmem, ws;
    DMat router, sh_gate_inp, sh_gate, sh_up, sh_down;
    uint8_t *gate = nullptr, *up = nullptr, *down = nullptr;
    uint64_t gu_bytes = 0, down_bytes = 0, gu_nb = 0, down_nb = 0;
    // workspace
    float *x = nullptr, *logits = nullptr, *wk = nullptr, *scalar = nullptr, *sh_act = nullptr, *sh_out = nullptr, *act = nullptr, *tmp = nullptr, *out = nullptr;
    uint32_t *ids = nullptr, *sorted = nullptr, *uexp = nullptr, *ustart = nullptr, *n_unique = nullptr, *bad = nullptr;
    uint32_t *item_u = nullptr, *item_p0 = nullptr, *n_items = nullptr;
    uint32_t *ids_mirror = nullptr;       // optional: a single token's ids are also written here (the engine's per-layer view)
    int8_t *xq_x = nullptr, *xq_act = nullptr, *xq_sh = nullptr;      // activation digits for the tensor-core paths
    float *sx_x = nullptr, *sx_act = nullptr, *sx_sh = nullptr;
    // digits of the token rows for redcuda_moe_shared_device alone: under expert parallelism it runs on another stream
    // than redcuda_moe_partial_device, which fills xq_x / sx_x with the gathered rows of every rank at the same time
    int8_t *xq_own = nullptr; float *sx_own = nullptr;
    EpWait wait{};             // set for one call by rc::moe_partial_gathered: the grouping kernel first waits for the other ranks' rows
    const int8_t *xq_ext = nullptr; const float *sx_ext = nullptr;   // digits of the gate/up input supplied by the caller for one call (rc::moe_partial_gathered)
    uint32_t max_pairs = 0;
    bool use_mma = false;      // IQ2_XXS experts (and the Q6_K shared expert of a batch) on the integer tensor-core path
    bool nib = false;          // routed experts held in the nibble layout (redcuda_moe_nib.cu) instead of planar IQ2_XXS
    uint32_t *work = nullptr;  // two unit counters of the persistent expert kernels (gate/up, down)
    uint32_t *ticket = nullptr; // ticket counter of the single-token GEMV's routing tail (zero between launches)
    uint32_t *tc_err = nullptr; // timeout flag of the tcgen05 kernels
    __half *sh_xs = nullptr; float *sh_xinv = nullptr;   // shared expert on the tcgen05 GEMM: activation digits and inverse scales
    uint8_t *sh_wd = nullptr; float *sh_winv = nullptr;  // and the weight digits of one launch (gate + up, or down)
    __half *rt_xs = nullptr; float *rt_xinv = nullptr; uint8_t *rt_wd = nullptr; float *rt_winv = nullptr;   // the same for the router logits of a large chunk
    bool tc_ok = false;         // the tcgen05 expert kernel can serve this layer's shapes
    bool tc_now = false;        // ... and serves the call in progress (set by moe_choose_path, read by the grouping and the launches)
    bool ws_shared = false;     // the workspace belongs to the caller (rc::moe_create_shared)
    cudaStream_t stream = nullptr;
    cudaStream_t side = nullptr;                    // the shared expert runs here, beside the routed experts
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_quant = nullptr;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// tensor-core path of the routed experts: IQ2_XXS gate/up/down with tile-able shapes
static bool moe_experts_mma(const redcuda_moe *m) {
    return m->nib || (m->use_mma && m->d.type_gu == RC_IQ2_XXS && m->d.type_down == RC_IQ2_XXS && m->d.hidden % 512u == 0 && m->d.ffn % 512u == 0);
}
// pairs per work item: the nibble-layout kernels take at most 8
static uint32_t moe_item_tokens(const redcuda_moe *m, bool single_token, uint32_t npairs) {
    if (m->tc_now && !single_token) return TCX_TN;
    if (m->nib) return single_token ? 1u : 8u;
    return mma_item_tokens(single_token, npairs, m->d.expert_count);
}
// Which expert kernels serve a call of npairs pairs (all_local: every pair belongs to this shard; otherwise the share
// expert_count / n_expert of them): the tcgen05 kernel works on items of up to 64 pairs of one expert and decodes an
// expert's weights once per item, so it needs experts that see many pairs each (prefill chunks of 2048 tokens: 40 pairs
// per expert). RC_MOE_TC_MIN = pairs per expert from which it is used (default 32; 0 = never). Measured on 2048-token
// chunks: gate/up 0.86 ms against 1.00 ms for the mma.sync kernels with items of 8 pairs, down 0.45 against 0.41 ms.
static void moe_choose_path(redcuda_moe *m, uint32_t npairs, bool all_local) {
    const char *v = getenv("RC_MOE_TC_MIN");
    const uint32_t min_avg = v ? (uint32_t)atoi(v) : 32u;
    const uint64_t local = all_local ? npairs : (uint64_t)npairs * m->d.expert_count / m->d.n_expert;
    m->tc_now = m->tc_ok && min_avg && local >= (uint64_t)min_avg * m->d.expert_count;
}
// tensor-core path of the shared expert: Q6_K and at least 3 tokens (below that the CUDA-core GEMV wins)
static bool moe_shared_mma(const redcuda_moe *m, uint32_t ntok) {
    return m->use_mma && m->d.type_sh == RC_Q6_K && ntok >= 3u && m->d.ffn_sh % 16u == 0 && m->d.hidden % 16u == 0;
}

// tcgen05 GEMM for the shared expert: from RC_SH_TC_MIN tokens on (default 128; 0 = never). Needs room for the "up"
// half of the gate/up pair in sh_out (ffn_sh <= hidden).
static bool moe_shared_tc(const redcuda_moe *m, uint32_t ntok) {
    const char *v = getenv("RC_SH_TC_MIN");
    const uint32_t min_tok = v ? (uint32_t)atoi(v) : 128u;
    return min_tok && ntok >= min_tok && rc_is_quant(m->d.type_sh) && m->d.ffn_sh <= m->d.hidden && m->d.hidden % 256u == 0 && m->d.ffn_sh % 256u == 0;
}
// Router logits on the tcgen05 GEMM: only with RC_ROUTER_TC_MIN=<tokens> (off by default). Measured on 2048-token chunks it
// takes 78 us instead of the fp64 GEMM's 242 us, but the softmax turns the ABSOLUTE error of a logit into a RELATIVE error of
// the expert weights: a split-fp16 product is good to about 1e-6 of sum |w x|, i.e. some 5e-5 of the weights, and the layer-48
// error of a 64-token chunk of the deep test model rose from 4.4e-5 to 2.0e-4. The double-precision sums stay the default.
static bool moe_router_tc(const redcuda_moe *m, uint32_t ntok) {
    const char *v = getenv("RC_ROUTER_TC_MIN");
    const uint32_t min_tok = v ? (uint32_t)atoi(v) : 0u;
    return min_tok && ntok >= min_tok && m->router.type == RC_F32 && m->d.hidden % 256u == 0 && m->rt_wd;
}
// out[j][t][row] = W_j x[t] for one or two matrices that share x (x2: the input is SiLU(x) * x2)
static int moe_shared_tc_gemm(redcuda_moe *m, uint32_t ntok, const float *x, const float *x2, uint32_t ncols, const DMat *w0, float *out0, const DMat *w1, float *out1,
                              const char *tag, cudaStream_t s) {
    const uint32_t tn = tc_token_tile(ntok, tc_row_tiles(w0->nrows) + (w1 ? tc_row_tiles(w1->nrows) : 0u));
    if (!launch_tc_prep_x(x, x2, ncols, ntok, ncols, tn, m->sh_xs, m->sh_xinv, s)) return 0;
    TcArgs A{};
    A.njobs = w1 ? 2u : 1u; A.ncols = ncols; A.ntok = ntok; A.xs = m->sh_xs; A.x_inv = m->sh_xinv; A.err = m->tc_err;
    A.wd = m->sh_wd; A.w_inv = m->sh_winv;
    A.job[0] = TcJob{w0->base, w0->nb, w0->type, w0->nrows, out0, w0->nrows, 0u};
    if (w1) A.job[1] = TcJob{w1->base, w1->nb, w1->type, w1->nrows, out1, w1->nrows, 0u};
    return launch_tc_gemm(A, tn, tag, s);
}

// x_quantised: xq_x / sx_x already hold the digits of x
static int moe_gemv_pre(redcuda_moe *m, uint32_t ntok, const float *x, bool with_router, bool with_shared, bool x_quantised, cudaStream_t s,
                        const int8_t *xq = nullptr, const float *sx = nullptr, const RouteTail *tail = nullptr) {
    if (!xq) { xq = m->xq_x; sx = m->sx_x; }
    GemvArgs A{};
    A.ntok = ntok; A.x = x; A.x_stride = m->d.hidden;
    uint32_t j = 0;
    auto add = [&](const DMat &w0, const DMat *w1, float *out, uint32_t stride, uint32_t epi) {
        GemvJob &J = A.job[j++];
        J.w0 = w0.base; J.w1 = w1 ? w1->base : nullptr; J.out = out; J.nb = w0.nb; J.type = w0.type; J.nrows = w0.nrows; J.ncols = w0.ncols;
        J.out_stride = stride; J.epi = epi;
    };
    if (with_router) {
        // batches: the tiled fp64 GEMM (one pass over the router matrix per 16 tokens of a block, from shared memory)
        if (moe_router_tc(m, ntok)) {
            // opt-in: the logits as a split-fp16 product on the tcgen05 GEMM (see moe_router_tc)
            const uint32_t tn = tc_token_tile(ntok, tc_row_tiles(m->d.n_expert));
            if (!launch_tc_prep_x(x, nullptr, m->d.hidden, ntok, m->d.hidden, tn, m->rt_xs, m->rt_xinv, s)) return 0;
            TcArgs T{};
            T.njobs = 1u; T.ncols = m->d.hidden; T.ntok = ntok; T.xs = m->rt_xs; T.x_inv = m->rt_xinv; T.err = m->tc_err;
            T.wd = m->rt_wd; T.w_inv = m->rt_winv;
            T.job[0] = TcJob{m->router.base, 0u, RC_F32, m->d.n_expert, m->logits, m->d.n_expert, 0u};
            if (!launch_tc_gemm(T, tn, "moe_router_logits_tc", s)) return 0;
        } else if (ntok >= 8u && m->router.type == RC_F32 && m->d.hidden % 64u == 0) {
            if (!launch_router_logits((const float *)m->router.base, x, m->d.hidden, ntok, m->d.n_expert, m->d.hidden, m->logits, s)) return 0;
        } else add(m->router, nullptr, m->logits, m->d.n_expert, GEMV_STORE);
    }
    if (with_shared) {
        if (moe_shared_tc(m, ntok)) {       // gate -> sh_act, up -> sh_out; moe_shared_down applies SiLU(gate) * up
            if (!moe_shared_tc_gemm(m, ntok, x, nullptr, m->d.hidden, &m->sh_gate, m->sh_act, &m->sh_up, m->sh_out, "moe_shared_gateup_tc", s)) return 0;
        } else if (moe_shared_mma(m, ntok) && x_quantised) {
            if (!launch_q6k_mma(m->sh_gate.base, m->sh_up.base, m->sh_gate.nb, m->d.ffn_sh, m->d.hidden, ntok, xq, sx, m->sh_act, m->d.ffn_sh,
                                "moe_shared_gateup_mma", s)) return 0;
        } else add(m->sh_gate, &m->sh_up, m->sh_act, m->d.ffn_sh, GEMV_PAIR_SILU);
        // the scalar gate is a single row: as a GEMV job it would be one block sweeping every token
        if (ntok >= 3u) { if (!launch_vec_sigmoid((const float *)m->sh_gate_inp.base, x, m->d.hidden, m->d.hidden, ntok, m->scalar, s)) return 0; }
        else add(m->sh_gate_inp, nullptr, m->scalar, 1u, GEMV_SIGMOID);
    }
    if (!j) return 1;
    A.njobs = j;
    A.tag = "moe_pre_gemv";
    if (tail) A.tail = *tail;
    return launch_gemv(A, s);
}

static int moe_shared_down(redcuda_moe *m, uint32_t ntok, cudaStream_t s) {
    if (moe_shared_tc(m, ntok)) return moe_shared_tc_gemm(m, ntok, m->sh_act, m->sh_out, m->d.ffn_sh, &m->sh_down, m->sh_out, nullptr, nullptr, "moe_shared_down_tc", s);
    if (moe_shared_mma(m, ntok)) {
        if (!launch_quant_act(m->sh_act, m->d.ffn_sh, ntok, m->d.ffn_sh, m->xq_sh, m->sx_sh, s)) return 0;
        return launch_q6k_mma(m->sh_down.base, nullptr, m->sh_down.nb, m->d.hidden, m->d.ffn_sh, ntok, m->xq_sh, m->sx_sh, m->sh_out, m->d.hidden,
                              "moe_shared_down_mma", s);
    }
    GemvArgs A{};
    A.ntok = ntok; A.x = m->sh_act; A.x_stride = m->d.ffn_sh; A.njobs = 1;
    GemvJob &J = A.job[0];
    J.w0 = m->sh_down.base; J.out = m->sh_out; J.nb = m->sh_down.nb; J.type = m->sh_down.type; J.nrows = m->sh_down.nrows; J.ncols = m->sh_down.ncols;
    J.out_stride = m->d.hidden; J.epi = GEMV_STORE;
    A.tag = "moe_shared_down_gemv";
    return launch_gemv(A, s);
}

// gate/up (x = token or pair activations) or down (x = act) of the grouped pairs. x_quantised: digits already in place.
static int moe_launch_experts(redcuda_moe *m, bool gateup, uint32_t npairs, bool single_token, const float *x, uint32_t x_stride, uint32_t x_div,
                              bool x_quantised, float *out, uint32_t out_stride, cudaStream_t s) {
    const uint32_t nrows = gateup ? m->d.ffn : m->d.hidden, ncols = gateup ? m->d.hidden : m->d.ffn;
    if (m->tc_now && !single_token) {
        // gate and up land in two plain [pair][ffn] buffers (out, and tmp as the second); the down launch's preparation
        // reads both, applies SiLU(gate) * up and splits the product into digits
        __half *xd = reinterpret_cast<__half *>(gateup ? m->xq_x : m->xq_act);
        float *xinv = gateup ? m->sx_x : m->sx_act;
        if (gateup) { if (!launch_tc_prep_rows(x, nullptr, x_stride, (npairs + x_div - 1u) / x_div, ncols, xd, xinv, s)) return 0; }
        else if (!launch_tc_prep_rows(x, m->tmp, x_stride, npairs, ncols, xd, xinv, s)) return 0;
        TcxArgs T{};
        T.w[0] = gateup ? m->gate : m->down; T.w[1] = gateup ? m->up : nullptr; T.nmat = gateup ? 2u : 1u;
        T.mat_bytes = gateup ? m->gu_bytes : m->down_bytes; T.nrows = nrows; T.ncols = ncols;
        T.expert_begin = m->d.expert_begin; T.n_local = m->d.expert_count;
        T.sorted = m->sorted; T.uexp = m->uexp; T.ustart = m->ustart; T.item_u = m->item_u; T.item_p0 = m->item_p0; T.n_items = m->n_items;
        T.xd = xd; T.x_inv = xinv; T.x_div = gateup ? x_div : 1u;
        T.out[0] = out; T.out[1] = gateup ? m->tmp : nullptr; T.out_stride = out_stride;
        T.err = m->tc_err; T.status = status_words();
        const uint32_t live = npairs < m->d.expert_count ? npairs : m->d.expert_count;
        return launch_tc_experts(T, npairs / TCX_TN + live, gateup ? "moe_gateup_tc" : "moe_down_tc", s);
    }
    if (moe_experts_mma(m)) {
        int8_t *xq = gateup ? m->xq_x : m->xq_act;
        float *sx = gateup ? m->sx_x : m->sx_act;
        if (!x_quantised && !launch_quant_act(x, x_stride, (npairs + x_div - 1u) / x_div, ncols, xq, sx, s)) return 0;
        const int8_t *xq_in = gateup && m->xq_ext ? m->xq_ext : xq;
        const float *sx_in = gateup && m->sx_ext ? m->sx_ext : sx;
        MmaArgs M{};
        M.w0 = gateup ? m->gate : m->down; M.w1 = gateup ? m->up : nullptr;
        M.mat_bytes = gateup ? m->gu_bytes : m->down_bytes; M.nb = gateup ? m->gu_nb : m->down_nb;
        M.nrows = nrows; M.ncols = ncols; M.expert_begin = m->d.expert_begin; M.n_local = m->d.expert_count; M.status = status_words();
        M.sorted = m->sorted; M.uexp = m->uexp; M.ustart = m->ustart; M.item_u = m->item_u; M.item_p0 = m->item_p0; M.n_items = m->n_items;
        M.xq = xq_in; M.sx = sx_in; M.x_div = x_div; M.out = out; M.out_stride = out_stride;
        const uint32_t tok = moe_item_tokens(m, single_token, npairs);
        const uint32_t live = npairs < m->d.expert_count ? npairs : m->d.expert_count;
        const uint32_t max_items = single_token ? npairs : (npairs / tok + live < npairs ? npairs / tok + live : npairs);
        if (m->nib) { M.item_tok = tok; M.work = m->work + (gateup ? 0 : 1); return launch_nib_experts(M, max_items, s); }
        return launch_moe_mma(M, max_items, tok, s);
    }
    MoeArgs A{};
    A.w0 = gateup ? m->gate : m->down; A.w1 = gateup ? m->up : nullptr;
    A.mat_bytes = gateup ? m->gu_bytes : m->down_bytes; A.nb = gateup ? m->gu_nb : m->down_nb;
    A.type = gateup ? m->d.type_gu : m->d.type_down;
    A.nrows = nrows; A.ncols = ncols;
    A.expert_begin = m->d.expert_begin; A.n_local = m->d.expert_count; A.status = status_words();
    A.sorted = m->sorted; A.uexp = m->uexp; A.ustart = m->ustart; A.n_unique = m->n_unique;
    A.x = x; A.x_stride = x_stride; A.x_div = x_div; A.out = out; A.out_stride = out_stride; A.pair_silu = gateup ? 1u : 0u;
    A.iq2 = books_iq2(); A.iq3s = books_iq3s();
    uint32_t lpr = 32u;
    while (lpr > (A.ncols >> 6)) lpr >>= 1;
    const uint32_t rows_per_pass = 8u * (32u / lpr);
    const uint32_t groups = npairs < m->d.expert_count ? npairs : m->d.expert_count;   // upper bound of experts that got a pair
    // >= 2 blocks per SM when the row count allows, at most 8 sweeps per block
    uint32_t sweeps = (uint32_t)(((uint64_t)A.nrows * groups) / ((uint64_t)rows_per_pass * 148u * 2u));
    sweeps = sweeps < 1u ? 1u : sweeps > 8u ? 8u : sweeps;
    A.rows_per_tile = rows_per_pass * sweeps;
    const dim3 grid((A.nrows + A.rows_per_tile - 1u) / A.rows_per_tile, groups);
    const int nt = single_token ? 1 : 4;
    const size_t smem = (size_t)nt * x_padded(A.ncols) * sizeof(float);
    RC_REQUIRE(smem <= 200u * 1024u, "moe: row length %u too large for the shared-memory staging", A.ncols);
    prof_begin(gateup ? "moe_gateup" : "moe_down", s);
    if (nt == 1) {
        if (smem > 48u * 1024u) RC_CUDA(cudaFuncSetAttribute(k_moe_experts<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        RC_LAUNCH((k_moe_experts<1>), grid, 256, smem, s, A);
    } else {
        if (smem > 48u * 1024u) RC_CUDA(cudaFuncSetAttribute(k_moe_experts<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        RC_LAUNCH((k_moe_experts<4>), grid, 256, smem, s, A);
    }
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

static int moe_group(redcuda_moe *m, const uint32_t *pair_expert, uint32_t npairs, bool distinct, cudaStream_t s, bool skip_foreign = false) {
    RC_REQUIRE(npairs <= m->max_pairs, "moe: %u pairs exceed the workspace (%u)", npairs, m->max_pairs);
    prof_begin("moe_group", s);
    if (distinct && npairs <= 64u && !skip_foreign) {
        RC_LAUNCH((k_group_trivial), 1, 64, 0, s, pair_expert, npairs, m->sorted, m->uexp, m->ustart, m->n_unique, m->item_u, m->item_p0, m->n_items, m->work);
    } else {
        RC_LAUNCH((k_group_pairs), 1, 1024, 0, s, pair_expert, npairs, m->d.expert_begin, m->d.expert_stride, skip_foreign ? 1u : 0u, m->d.expert_count, moe_item_tokens(m, false, npairs), m->sorted, m->uexp, m->ustart,
                                         m->n_unique, m->item_u, m->item_p0, m->n_items, m->bad, m->work, m->wait);
    }
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

static int moe_combine(redcuda_moe *m, uint32_t ntok, const float *pair_out, const float *wk, uint32_t top_k, bool shared, const float *resid,
                       float *out, cudaStream_t s) {
    const dim3 grid((m->d.hidden / 4u + 255u) / 256u, ntok);
    prof_begin("moe_combine", s);
    RC_LAUNCH((k_moe_combine), grid, 256, 0, s, pair_out, wk, top_k, shared ? m->sh_out : nullptr, m->scalar, resid, out, m->d.hidden, nullptr);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

// One token in three launches (the dependency chain of the layer, nothing else): (1) router logits + shared gate/up +
// scalar gate in one multi-job GEMV whose last block also runs the softmax / top-k; (2) gate/up of the selected experts,
// the token quantised inside the kernel; (3) down of the selected experts + shared down + weighted sum + residual.
// The reference fuses the same tail (redmetal_topk_down_tail, native/redmetal_topk.m:254-280).
static bool moe_fused1_ok(const redcuda_moe *m) {
    static const bool want = !(getenv("RC_MOE_FUSE1") && atoi(getenv("RC_MOE_FUSE1")) == 0);     // A/B switch
    return want && m->nib && m->d.type_sh == RC_Q6_K && m->d.n_expert <= 1024u && nib_tail_ok(m->d.top_k, m->d.hidden, m->d.ffn) &&
           m->d.ffn_sh == m->d.ffn;
}
static int moe_forward_fused1(redcuda_moe *m, const float *x, const float *logits_in, const float *resid, float *out, cudaStream_t s) {
    const uint32_t k = m->d.top_k;
    RouteTail T{};
    T.ticket = m->ticket; T.logits = logits_in ? logits_in : m->logits; T.n_expert = m->d.n_expert; T.top_k = k; T.ids = m->ids; T.weights = m->wk;
    T.G = RouteGroup1{m->sorted, m->uexp, m->ustart, m->n_unique, m->item_u, m->item_p0, m->n_items, m->ids_mirror, m->work};
    T.status = status_words();
    if (!moe_gemv_pre(m, 1u, x, logits_in == nullptr, true, false, s, nullptr, nullptr, &T)) return 0;
    MmaArgs M{};
    M.w0 = m->gate; M.w1 = m->up; M.mat_bytes = m->gu_bytes; M.nb = m->gu_nb; M.nrows = m->d.ffn; M.ncols = m->d.hidden;
    M.expert_begin = m->d.expert_begin; M.n_local = m->d.expert_count; M.status = status_words();
    M.sorted = m->sorted; M.uexp = m->uexp; M.ustart = m->ustart; M.item_u = m->item_u; M.item_p0 = m->item_p0; M.n_items = m->n_items;
    M.xq = nullptr; M.sx = nullptr; M.x_div = k; M.out = m->act; M.out_stride = m->d.ffn; M.item_tok = 1u; M.work = m->work; M.x_raw = x;
    if (!launch_nib_experts(M, k, s)) return 0;
    NibTailArgs D{};
    D.w_down = m->down; D.mat_bytes = m->down_bytes; D.nrows = m->d.hidden; D.ncols = m->d.ffn; D.expert_begin = m->d.expert_begin; D.n_local = m->d.expert_count;
    D.top_k = k; D.ids = m->ids; D.wk = m->wk; D.act = m->act; D.act_stride = m->d.ffn;
    D.sh_down = m->sh_down.base; D.sh_nb = m->sh_down.nb; D.sh_act = m->sh_act; D.scalar = m->scalar; D.resid = resid; D.out = out; D.status = status_words();
    return launch_nib_down_tail(D, s);
}

static int moe_forward_on(redcuda_moe *m, uint32_t ntok, const float *x, const float *logits_in, const float *resid, float *out, cudaStream_t s) {
    RC_REQUIRE(m->d.expert_begin == 0 && m->d.expert_count == m->d.n_expert && m->d.expert_stride == 1u, "moe forward needs every expert on this device; use the route/experts/shared pieces under expert parallelism");
    RC_REQUIRE(ntok >= 1 && ntok <= m->d.max_tokens, "moe forward: ntok %u outside [1, %u]", ntok, m->d.max_tokens);
    if (ntok == 1u && moe_fused1_ok(m)) return moe_forward_fused1(m, x, logits_in, resid, out, s);
    const uint32_t k = m->d.top_k, npairs = ntok * k;
    moe_choose_path(m, npairs, true);
    // one quantisation of the token activations serves the routed gate/up and the shared gate/up
    const bool xq = moe_experts_mma(m) || moe_shared_mma(m, ntok);
    // The shared expert needs nothing from the router, so it runs on a side stream next to the routed
    // experts and joins before the combine (both edges are events, so the fork is kept when the caller captures a graph).
    // With profiling on, everything stays on one stream so that per-kernel times are not overlapped.
    const bool fork = !prof_active();
    // The quantisation of x leaves the critical path too: it opens the side stream (the shared expert's tensor-core
    // kernels, which read the digits as well, follow it there) and the main stream waits for it only before the
    // gate/up launch, behind the router GEMV, the selection and the grouping.
    const bool quant_aside = fork && xq;
    // the tcgen05 expert path keeps its fp16 digits where the int8 digits of the routed experts would go, so the int8
    // digits that the shared expert still reads move to the buffer of the stand-alone shared-expert call
    int8_t *xqd = m->tc_now ? m->xq_own : m->xq_x;
    float *sxd = m->tc_now ? m->sx_own : m->sx_x;
    if (xq && !quant_aside && !launch_quant_act(x, m->d.hidden, ntok, m->d.hidden, xqd, sxd, s)) return 0;
    if (fork) {
        RC_CUDA(cudaEventRecord(m->ev_fork, s));
        RC_CUDA(cudaStreamWaitEvent(m->side, m->ev_fork, 0));
        if (quant_aside) {
            if (!launch_quant_act(x, m->d.hidden, ntok, m->d.hidden, xqd, sxd, m->side)) return 0;
            RC_CUDA(cudaEventRecord(m->ev_quant, m->side));
        }
        if (!moe_gemv_pre(m, ntok, x, false, true, xq, m->side, xqd, sxd) || !moe_shared_down(m, ntok, m->side)) return 0;
        RC_CUDA(cudaEventRecord(m->ev_join, m->side));
        if (!moe_gemv_pre(m, ntok, x, logits_in == nullptr, false, xq, s, xqd, sxd)) return 0;
    } else if (!moe_gemv_pre(m, ntok, x, logits_in == nullptr, true, xq, s, xqd, sxd)) return 0;
    if (ntok == 1u && m->d.n_expert <= 1024u) {      // one token: the router kernel also writes the (trivial) grouping
        const RouteGroup1 G{m->sorted, m->uexp, m->ustart, m->n_unique, m->item_u, m->item_p0, m->n_items, m->ids_mirror, m->work};
        if (!launch_route(logits_in ? logits_in : m->logits, ntok, m->d.n_expert, k, m->ids, m->wk, nullptr, s, &G)) return 0;
    } else {
        if (!launch_route(logits_in ? logits_in : m->logits, ntok, m->d.n_expert, k, m->ids, m->wk, nullptr, s)) return 0;
        if (!moe_group(m, m->ids, npairs, ntok == 1u, s)) return 0;
    }
    if (quant_aside && !m->tc_now) RC_CUDA(cudaStreamWaitEvent(s, m->ev_quant, 0));
    if (!moe_launch_experts(m, true, npairs, ntok == 1u, x, m->d.hidden, k, xq && moe_experts_mma(m), m->act, m->d.ffn, s)) return 0;
    if (!fork && !moe_shared_down(m, ntok, s)) return 0;
    if (!moe_launch_experts(m, false, npairs, ntok == 1u, m->act, m->d.ffn, 1u, false, m->tmp, m->d.hidden, s)) return 0;
    if (fork) RC_CUDA(cudaStreamWaitEvent(s, m->ev_join, 0));
    return moe_combine(m, ntok, m->tmp, m->wk, k, true, resid, out, s);
}

// Carves the workspace of a layer out of B (m and B null: only the size is computed). Every piece is 256-byte aligned.
static size_t moe_ws_layout(const redcuda_moe_desc &d, redcuda_moe *m, uint8_t *B) {
    const size_t T = d.max_tokens, P = T * d.top_k;
    size_t w = 0;
    auto put = [&](auto &ptr, size_t bytes) {
        if (m) ptr = reinterpret_cast<std::remove_reference_t<decltype(ptr)>>(B + w);
        w = align_up(w + bytes, 256);
    };
    redcuda_moe scratch_names;            // pointer members to aim at when only the size is wanted
    redcuda_moe &r = m ? *m : scratch_names;
    put(r.x, T * d.hidden * 4u); put(r.logits, T * d.n_expert * 4u); put(r.wk, P * 4u); put(r.scalar, T * 4u);
    put(r.sh_act, T * d.ffn_sh * 4u); put(r.sh_out, T * d.hidden * 4u); put(r.act, P * d.ffn * 4u); put(r.tmp, P * d.hidden * 4u);
    put(r.out, T * d.hidden * 4u); put(r.ids, P * 4u); put(r.sorted, P * 4u); put(r.uexp, (size_t)(d.expert_count + 1u) * 4u);
    put(r.ustart, (size_t)(d.expert_count + 2u) * 4u); put(r.n_unique, 16); put(r.bad, 16);
    // digits of the routed experts' inputs: three int8 digits per value (mma.sync kernels) or two fp16 digits (tcgen05 kernel)
    put(r.xq_x, P * 4u * d.hidden); put(r.sx_x, P * 4u); put(r.xq_act, P * 4u * d.ffn); put(r.sx_act, P * 4u);
    put(r.xq_sh, T * 3u * d.ffn_sh); put(r.sx_sh, T * 4u); put(r.xq_own, T * 3u * d.hidden); put(r.sx_own, T * 4u);
    put(r.item_u, (P + 8u) * 4u); put(r.item_p0, (P + 8u) * 4u); put(r.n_items, 16); put(r.work, 16);
    put(r.sh_xs, tc_xs_halves((uint32_t)T, d.hidden > d.ffn_sh ? d.hidden : d.ffn_sh, 128u) * 2u); put(r.sh_xinv, (T + 128u) * 4u);
    {
        const uint32_t t_up = 2u * tc_row_tiles(d.ffn_sh), t_down = tc_row_tiles(d.hidden);
        put(r.sh_wd, std::max(tc_wd_bytes(t_up, d.hidden), tc_wd_bytes(t_down, d.ffn_sh))); put(r.sh_winv, (size_t)std::max(t_up, t_down) * 4u);
    }
    if (d.hidden % 256u == 0) {
        put(r.rt_xs, tc_xs_halves((uint32_t)T, d.hidden, 128u) * 2u); put(r.rt_xinv, (T + 128u) * 4u);
        put(r.rt_wd, tc_wd_bytes(tc_row_tiles(d.n_expert), d.hidden)); put(r.rt_winv, (size_t)tc_row_tiles(d.n_expert) * 4u);
    }
    if (m) { m->ticket = m->work + 2; m->tc_err = m->work + 3; }
    return w;
}

namespace rc {
const uint32_t *moe_last_ids_device(const redcuda_moe *m) { return m->ids; }
void moe_set_ids_mirror(redcuda_moe *m, uint32_t *dev_ptr) { m->ids_mirror = dev_ptr; }
}
namespace rc {
// true when the routed experts read int8 activation digits (so a caller may quantise before an exchange and hand the digits in)
// (for a call over ntok gathered tokens: the tcgen05 kernel of large chunks prepares its own fp16 digits from the fp32 rows)
bool moe_takes_digits(redcuda_moe *m, uint32_t ntok) {
    moe_choose_path(m, ntok * m->d.top_k, false);
    return moe_experts_mma(m) && !m->tc_now;
}
// The shard's experts over gathered tokens: x [ntok][hidden] fp32, or (when xq is given) its digits xq [ntok][3][hidden] with
// scales sx [ntok]; ids / w [ntok][top_k] contiguous. out [ntok][hidden] as k_ep_combine defines it.
// wait (may be null): the grouping kernel first waits for the other ranks' rows (peer-memory exchange). push (may be
// null): the sums go to their owners' slots in peer memory instead of out (add is then left to the owner).
int moe_partial_gathered(redcuda_moe *m, uint32_t ntok, const float *x, const int8_t *xq, const float *sx, const uint32_t *ids, const float *w,
                         const float *add, uint32_t add_begin, uint32_t add_count, float *out, cudaStream_t s, const EpWait *wait, const EpPush *push) {
    RC_REQUIRE(m && (x || (xq && sx)) && ids && w && (out || push), "moe partial: null argument");
    RC_REQUIRE(ntok >= 1 && ntok <= m->d.max_tokens, "moe partial: ntok %u outside [1, %u]", ntok, m->d.max_tokens);
    const uint32_t k = m->d.top_k, npairs = ntok * k;
    moe_choose_path(m, npairs, false);
    const bool digits = xq && moe_experts_mma(m) && !m->tc_now;
    RC_REQUIRE(digits || x, "moe partial: this layer's expert kernels need the fp32 rows");
    if (wait) m->wait = *wait;
    const int grouped = moe_group(m, ids, npairs, false, s, true);
    m->wait = EpWait{};
    if (!grouped) return 0;
    if (digits) { m->xq_ext = xq; m->sx_ext = sx; }
    const int ok = moe_launch_experts(m, true, npairs, false, x, m->d.hidden, k, digits, m->act, m->d.ffn, s);
    m->xq_ext = nullptr; m->sx_ext = nullptr;
    if (!ok) return 0;
    if (!moe_launch_experts(m, false, npairs, false, m->act, m->d.ffn, 1u, false, m->tmp, m->d.hidden, s)) return 0;
    const dim3 grid((m->d.hidden / 4u + 255u) / 256u, ntok);
    prof_begin(push ? "ep_combine_push" : "ep_combine", s);
    if (push) RC_LAUNCH((k_ep_combine_push), grid, 256, 0, s, m->tmp, ids, w, k, m->d.expert_begin, m->d.expert_stride, m->d.expert_count, *push, m->d.hidden);
    else RC_LAUNCH((k_ep_combine), grid, 256, 0, s, m->tmp, ids, w, k, m->d.expert_begin, m->d.expert_stride, m->d.expert_count, add, add_begin, add_count, out, m->d.hidden);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}
}
static redcuda_moe *moe_create_impl(const redcuda_moe_desc *desc, void *shared_ws);
namespace rc {
// One workspace for many layers: legal when the calls of those layers are ordered on one stream (the engine's are), and
// what keeps a 2048-token prefill chunk affordable (the workspace grows with max_tokens * top_k * hidden).
size_t moe_workspace_bytes(const redcuda_moe_desc *d) { return moe_ws_layout(*d, nullptr, nullptr); }
redcuda_moe *moe_create_shared(const redcuda_moe_desc *d, void *workspace) { return moe_create_impl(d, workspace); }
}

static redcuda_moe *moe_create_impl(const redcuda_moe_desc *desc, void *shared_ws) {
    if (!require_device()) return nullptr;
    if (!desc) { set_error("moe create: null descriptor"); return nullptr; }
    const redcuda_moe_desc &d = *desc;
    auto fail = [](const char *msg) -> redcuda_moe * { set_error("moe create: %s", msg); return nullptr; };
    if (!d.hidden || !d.n_expert || !d.top_k || !d.ffn || !d.ffn_sh || !d.max_tokens) return fail("zero dimension");
    if (d.top_k > REDCUDA_MAX_TOPK || d.top_k > d.n_expert) return fail("top_k out of range");
    if (d.hidden % 256u || d.ffn % 256u || d.ffn_sh % 256u) return fail("hidden / ffn sizes must be multiples of 256");
    if (!rc_is_quant(d.type_gu) || !rc_is_quant(d.type_down) || !rc_is_quant(d.type_sh)) return fail("expert matrices must be IQ2_XXS, IQ3_S or Q6_K");
    const uint32_t stride = d.expert_stride ? d.expert_stride : 1u;
    if (d.expert_count == 0 || d.expert_count > 1024u || (uint64_t)d.expert_begin + (uint64_t)(d.expert_count - 1u) * stride >= d.n_expert) return fail("bad expert shard");
    if (!d.router || !d.gate_exps || !d.up_exps || !d.down_exps || !d.sh_gate_inp || !d.sh_gate || !d.sh_up || !d.sh_down) return fail("null weight pointer");
    if (!require_books(d.type_gu) || !require_books(d.type_down) || !require_books(d.type_sh)) return nullptr;

    status_words();        // allocated here, never inside a stream capture
    redcuda_moe *m = new (std::nothrow) redcuda_moe();
    if (!m) return fail("out of host memory");
    m->d = d;
    m->d.expert_stride = stride;
    cudaGetDevice(&m->device);
    auto bail = [&]() -> redcuda_moe * { redcuda_moe_destroy(m); return nullptr; };
    if (cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess || cudaStreamCreateWithFlags(&m->side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming) != cudaSuccess || cudaEventCreateWithFlags(&m->ev_join, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&m->ev_quant, cudaEventDisableTiming) != cudaSuccess) {
        set_error("moe create: stream / event creation failed"); return bail();
    }

    {   // RC_EXPERT_FMT: "nib4" keeps IQ2_XXS experts in the nibble layout (table-free decode, 2.09x the bytes), "iq2" in the
        // planar GGUF bytes; unset = nib4 where the shapes allow it (measured on the 64-token batch: gate/up 105 -> 69 us,
        // down 74 -> 39 us per layer)
        const char *fmt = getenv("RC_EXPERT_FMT");
        const bool want = !(fmt && fmt[0] == 'i');
        m->nib = want && d.type_gu == RC_IQ2_XXS && d.type_down == RC_IQ2_XXS && nib_shape_ok(d.ffn, d.hidden) && nib_shape_ok(d.hidden, d.ffn);
    }
    m->gu_bytes = m->nib ? nib_matrix_bytes(d.ffn, d.hidden) : rc_matrix_bytes(d.type_gu, d.ffn, d.hidden);
    m->down_bytes = m->nib ? nib_matrix_bytes(d.hidden, d.ffn) : rc_matrix_bytes(d.type_down, d.hidden, d.ffn);
    m->gu_nb = (uint64_t)d.ffn * (d.hidden / 256u);
    m->down_nb = (uint64_t)d.hidden * (d.ffn / 256u);
    if (m->gu_bytes % 16u || m->down_bytes % 16u) { set_error("moe create: expert matrix size is not a multiple of 16 bytes"); return bail(); }
    const size_t router_b = (size_t)d.n_expert * d.hidden * 4u, gvec_b = (size_t)d.hidden * 4u;
    const size_t shgu_b = rc_matrix_bytes(d.type_sh, d.ffn_sh, d.hidden), shd_b = rc_matrix_bytes(d.type_sh, d.hidden, d.ffn_sh);
    size_t off = 0;
    const size_t o_router = off; off = align_up(off + router_b, 256);
    const size_t o_gate = off; off = align_up(off + m->gu_bytes * d.expert_count, 256);
    const size_t o_up = off; off = align_up(off + m->gu_bytes * d.expert_count, 256);
    const size_t o_down = off; off = align_up(off + m->down_bytes * d.expert_count, 256);
    const size_t o_gvec = off; off = align_up(off + gvec_b, 256);
    const size_t o_shg = off; off = align_up(off + shgu_b, 256);
    const size_t o_shu = off; off = align_up(off + shgu_b, 256);
    const size_t o_shd = off; off = align_up(off + shd_b, 256);
    if (!m->wmem.alloc(off)) return bail();
    uint8_t *W = m->wmem.as<uint8_t>();
    m->gate = W + o_gate; m->up = W + o_up; m->down = W + o_down;
    m->router = DMat{W + o_router, RC_F32, d.n_expert, d.hidden, 0};
    m->sh_gate_inp = DMat{W + o_gvec, RC_F32, 1u, d.hidden, 0};
    m->sh_gate = DMat{W + o_shg, d.type_sh, d.ffn_sh, d.hidden, (uint64_t)d.ffn_sh * (d.hidden / 256u)};
    m->sh_up = DMat{W + o_shu, d.type_sh, d.ffn_sh, d.hidden, (uint64_t)d.ffn_sh * (d.hidden / 256u)};
    m->sh_down = DMat{W + o_shd, d.type_sh, d.hidden, d.ffn_sh, (uint64_t)d.hidden * (d.ffn_sh / 256u)};

    // upload + planar repack; host sources go through a bounded staging buffer, expert by expert
    const bool dev = d.weights_on_device != 0;
    DevMem scratch, planar_tmp;
    const size_t raw_gu = rc_matrix_bytes(d.type_gu, d.ffn, d.hidden), raw_down = rc_matrix_bytes(d.type_down, d.hidden, d.ffn);
    if (m->nib && !planar_tmp.alloc(raw_gu > raw_down ? raw_gu : raw_down)) return bail();
    const size_t big = raw_gu > raw_down ? raw_gu : raw_down;
    const size_t sc_b = big > shgu_b ? (big > shd_b ? big : shd_b) : (shgu_b > shd_b ? shgu_b : shd_b);
    if (!dev && !scratch.alloc(sc_b)) return bail();
    cudaStream_t s = m->stream;
    int ok = upload_matrix(RC_F32, d.n_expert, d.hidden, d.router, dev, W + o_router, nullptr, s) &&
             upload_matrix(RC_F32, 1u, d.hidden, d.sh_gate_inp, dev, W + o_gvec, nullptr, s) &&
             upload_matrix(d.type_sh, d.ffn_sh, d.hidden, d.sh_gate, dev, W + o_shg, scratch.as<uint8_t>(), s) &&
             upload_matrix(d.type_sh, d.ffn_sh, d.hidden, d.sh_up, dev, W + o_shu, scratch.as<uint8_t>(), s) &&
             upload_matrix(d.type_sh, d.hidden, d.ffn_sh, d.sh_down, dev, W + o_shd, scratch.as<uint8_t>(), s);
    // one expert matrix: raw GGUF rows -> planar (in place in the arena, or in a temporary when the arena holds the nibble layout)
    auto put = [&](uint32_t type, uint32_t nrows, uint32_t ncols, const uint8_t *src, uint8_t *dst) -> int {
        if (!m->nib) return upload_matrix(type, nrows, ncols, src, dev, dst, scratch.as<uint8_t>(), s);
        return upload_matrix(type, nrows, ncols, src, dev, planar_tmp.as<uint8_t>(), scratch.as<uint8_t>(), s) &&
               launch_nib_repack(planar_tmp.as<uint8_t>(), nrows, ncols, dst, s);
    };
    for (uint32_t e = 0; ok && e < d.expert_count; ++e) {
        ok = put(d.type_gu, d.ffn, d.hidden, d.gate_exps + (size_t)e * raw_gu, m->gate + (size_t)e * m->gu_bytes) &&
             put(d.type_gu, d.ffn, d.hidden, d.up_exps + (size_t)e * raw_gu, m->up + (size_t)e * m->gu_bytes) &&
             put(d.type_down, d.hidden, d.ffn, d.down_exps + (size_t)e * raw_down, m->down + (size_t)e * m->down_bytes);
    }
    if (!ok) return bail();

    // workspace: this layer's own, or the caller's (shared by layers whose calls are ordered on one stream)
    m->max_pairs = d.max_tokens * d.top_k;
    const size_t w = moe_ws_layout(d, nullptr, nullptr);
    uint8_t *B = static_cast<uint8_t *>(shared_ws);
    if (B) m->ws_shared = true;
    else { if (!m->ws.alloc(w)) return bail(); B = m->ws.as<uint8_t>(); }
    moe_ws_layout(d, m, B);
    m->tc_ok = m->nib && tcx_shape_ok(d.ffn, d.hidden) && tcx_shape_ok(d.hidden, d.ffn);
    {   // RC_MOE_PATH=cuda keeps the IQ2_XXS experts on the CUDA-core kernels (A/B switch for profiling)
        const char *pth = getenv("RC_MOE_PATH");
        m->use_mma = !(pth && pth[0] == 'c');
    }
    if (cudaMemsetAsync(B, 0, w, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) {
        set_error("moe create: weight upload failed: %s", cudaGetErrorString(cudaGetLastError()));
        return bail();
    }
    m->d.router = nullptr; m->d.gate_exps = m->d.up_exps = m->d.down_exps = nullptr; m->d.sh_gate_inp = nullptr; m->d.sh_gate = m->d.sh_up = m->d.sh_down = nullptr;
    return m;
}

extern "C" {

redcuda_moe *redcuda_moe_create(const redcuda_moe_desc *desc) { return moe_create_impl(desc, nullptr); }

void redcuda_moe_destroy(redcuda_moe *m) {
    if (!m) return;
    if (m->stream) { cudaStreamSynchronize(m->stream); cudaStreamDestroy(m->stream); }
    if (m->side) { cudaStreamSynchronize(m->side); cudaStreamDestroy(m->side); }
    if (m->ev_fork) cudaEventDestroy(m->ev_fork);
    if (m->ev_join) cudaEventDestroy(m->ev_join);
    if (m->ev_quant) cudaEventDestroy(m->ev_quant);
    delete m;
}

uint64_t redcuda_moe_resident_bytes(const redcuda_moe *m) { return m ? m->wmem.bytes : 0; }

int redcuda_moe_forward_device(redcuda_moe *m, uint32_t ntok, const float *x_dev, const float *logits_in_dev, const float *resid_dev,
                               float *out_dev, void *stream) {
    RC_REQUIRE(m && x_dev && out_dev, "moe forward: null argument");
    return moe_forward_on(m, ntok, x_dev, logits_in_dev, resid_dev, out_dev, (cudaStream_t)stream);
}

int redcuda_moe_forward(redcuda_moe *m, uint32_t ntok, const float *x, const float *logits_in, float *out,
                        uint32_t *ids_out, float *weights_out, float *logits_out) {
    RC_REQUIRE(m && x && out, "moe forward: null argument");
    RC_REQUIRE(ntok >= 1 && ntok <= m->d.max_tokens, "moe forward: ntok %u outside [1, %u]", ntok, m->d.max_tokens);
    RC_CUDA(cudaSetDevice(m->device));
    cudaStream_t s = m->stream;
    const size_t xb = (size_t)ntok * m->d.hidden * 4u, lb = (size_t)ntok * m->d.n_expert * 4u, kb = (size_t)ntok * m->d.top_k * 4u;
    RC_CUDA(cudaMemcpyAsync(m->x, x, xb, cudaMemcpyHostToDevice, s));
    if (logits_in) RC_CUDA(cudaMemcpyAsync(m->logits, logits_in, lb, cudaMemcpyHostToDevice, s));
    if (!moe_forward_on(m, ntok, m->x, logits_in ? m->logits : nullptr, nullptr, m->out, s)) return 0;
    RC_CUDA(cudaMemcpyAsync(out, m->out, xb, cudaMemcpyDeviceToHost, s));
    if (ids_out) RC_CUDA(cudaMemcpyAsync(ids_out, m->ids, kb, cudaMemcpyDeviceToHost, s));
    if (weights_out) RC_CUDA(cudaMemcpyAsync(weights_out, m->wk, kb, cudaMemcpyDeviceToHost, s));
    if (logits_out) RC_CUDA(cudaMemcpyAsync(logits_out, m->logits, lb, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    return status_failed() ? 0 : 1;
}

int redcuda_moe_route_device(redcuda_moe *m, uint32_t ntok, const float *x_dev, const float *logits_in_dev, uint32_t *ids_dev, float *weights_dev, void *stream) {
    RC_REQUIRE(m && ids_dev && weights_dev && (x_dev || logits_in_dev), "moe route: null argument");
    RC_REQUIRE(ntok >= 1 && ntok <= m->d.max_tokens, "moe route: ntok %u outside [1, %u]", ntok, m->d.max_tokens);
    cudaStream_t s = (cudaStream_t)stream;
    if (!logits_in_dev && !moe_gemv_pre(m, ntok, x_dev, true, false, false, s)) return 0;
    return launch_route(logits_in_dev ? logits_in_dev : m->logits, ntok, m->d.n_expert, m->d.top_k, ids_dev, weights_dev, nullptr, s);
}

int redcuda_moe_experts_device(redcuda_moe *m, uint32_t npairs, const float *pair_x_dev, const uint32_t *pair_expert_dev, float *pair_out_dev, void *stream) {
    RC_REQUIRE(m && pair_x_dev && pair_expert_dev && pair_out_dev, "moe experts: null argument");
    if (!npairs) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    RC_REQUIRE(npairs <= m->max_pairs, "moe experts: %u pairs exceed the workspace (%u)", npairs, m->max_pairs);
    moe_choose_path(m, npairs, true);
    if (!moe_group(m, pair_expert_dev, npairs, false, s)) return 0;
    if (!moe_launch_experts(m, true, npairs, false, pair_x_dev, m->d.hidden, 1u, false, m->act, m->d.ffn, s)) return 0;
    return moe_launch_experts(m, false, npairs, false, m->act, m->d.ffn, 1u, false, pair_out_dev, m->d.hidden, s);
}

// Contiguous copies of the pairs' expert ids and of their router weights, the weight zeroed when the expert lives on
// another shard (ids / w rows are meta_stride elements apart)
__global__ void k_mask_weights(const uint32_t *__restrict__ ids, const float *__restrict__ w, uint32_t ntok, uint32_t top_k, uint32_t meta_stride,
                               uint32_t begin, uint32_t stride, uint32_t count, uint32_t *__restrict__ ids_out, float *__restrict__ w_local) {
    pdl_prologue();
    const uint32_t p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= ntok * top_k) return;
    const uint32_t t = p / top_k, k = p - t * top_k;
    const uint32_t g = ids[(size_t)t * meta_stride + k];
    ids_out[p] = g;
    w_local[p] = shard_local(g, begin, stride, count) != 0xffffffffu ? w[(size_t)t * meta_stride + k] : 0.f;
}

int redcuda_moe_partial_device(redcuda_moe *m, uint32_t ntok, const float *x_dev, uint32_t x_stride, const uint32_t *ids_dev, const float *weights_dev,
                               uint32_t meta_stride, float *out_dev, void *stream) {
    RC_REQUIRE(m && x_dev && ids_dev && weights_dev && out_dev, "moe partial: null argument");
    RC_REQUIRE(ntok >= 1 && ntok <= m->d.max_tokens, "moe partial: ntok %u outside [1, %u]", ntok, m->d.max_tokens);
    RC_REQUIRE(x_stride >= m->d.hidden && x_stride % 4u == 0 && meta_stride >= m->d.top_k, "moe partial: bad row strides (%u, %u)", x_stride, meta_stride);
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t k = m->d.top_k, npairs = ntok * k;
    moe_choose_path(m, npairs, false);
    const bool xq = moe_experts_mma(m) && !m->tc_now;
    if (xq && !launch_quant_act(x_dev, x_stride, ntok, m->d.hidden, m->xq_x, m->sx_x, s)) return 0;
    prof_begin("moe_mask_weights", s);
    RC_LAUNCH((k_mask_weights), (npairs + 255u) / 256u, 256, 0, s, ids_dev, weights_dev, ntok, k, meta_stride, m->d.expert_begin, m->d.expert_stride, m->d.expert_count, m->ids, m->wk);
    prof_end(s);
    RC_LAUNCHED();
    if (!moe_group(m, m->ids, npairs, false, s, true)) return 0;
    if (!moe_launch_experts(m, true, npairs, false, x_dev, x_stride, k, xq, m->act, m->d.ffn, s)) return 0;
    if (!moe_launch_experts(m, false, npairs, false, m->act, m->d.ffn, 1u, false, m->tmp, m->d.hidden, s)) return 0;
    return moe_combine(m, ntok, m->tmp, m->wk, k, false, nullptr, out_dev, s);
}

int redcuda_moe_combine_device(redcuda_moe *m, uint32_t ntok, const float *pair_out_dev, const uint32_t *pair_row_dev, const float *weights_dev,
                               const float *add_dev, const float *resid_dev, float *out_dev, void *stream) {
    RC_REQUIRE(m && pair_out_dev && weights_dev && out_dev && ntok, "moe combine: null or empty argument");
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((m->d.hidden / 4u + 255u) / 256u, ntok);
    prof_begin("moe_combine", s);
    RC_LAUNCH((k_moe_combine), grid, 256, 0, s, pair_out_dev, weights_dev, m->d.top_k, add_dev, nullptr, resid_dev, out_dev, m->d.hidden, pair_row_dev);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

int redcuda_moe_shared_device(redcuda_moe *m, uint32_t ntok, const float *x_dev, float *out_dev, void *stream) {
    RC_REQUIRE(m && x_dev && out_dev, "moe shared: null argument");
    RC_REQUIRE(ntok >= 1 && ntok <= m->d.max_tokens, "moe shared: ntok %u outside [1, %u]", ntok, m->d.max_tokens);
    cudaStream_t s = (cudaStream_t)stream;
    const bool xq = moe_shared_mma(m, ntok);
    if (xq && !launch_quant_act(x_dev, m->d.hidden, ntok, m->d.hidden, m->xq_own, m->sx_own, s)) return 0;
    if (!moe_gemv_pre(m, ntok, x_dev, false, true, xq, s, m->xq_own, m->sx_own) || !moe_shared_down(m, ntok, s)) return 0;
    return moe_combine(m, ntok, nullptr, nullptr, 0u, true, nullptr, out_dev, s);
}

}  // extern "C"

// =====================================================================================================================
// Expert-pool ABI v1 of the reference (include/redmetal_topk.h): a resident arena with the reference's bookkeeping kept
// as counters. Slots hold raw GGUF bytes (the reference loads byte ranges without knowing their type); execute re-lays
// the selected experts out planar into a scratch area and runs the CUDA-core expert kernel, which serves every
// supported type — this is the parity entry point, not the decode path (that is redcuda_moe_*).
// =====================================================================================================================
#include "../../include/redmetal_topk.h"

#include <fcntl.h>
#include <unistd.h>
#include <chrono>
#include <vector>

namespace {

struct TopkPool {
    int fd = -1, device = 0;
    uint64_t slot_bytes = 0, bytes_read = 0, read_calls = 0;
    double read_ms = 0.0;
    uint32_t capacity = 0;
    DevMem arena, scratch, table;
    std::vector<uint32_t> generation, inflight;
    std::vector<uint64_t> table_h;
    uint32_t layers = 0, experts = 0;
    uint8_t *pin = nullptr; size_t pin_bytes = 0;
    cudaStream_t stream = nullptr;
};

double pool_now_ms() { return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

int pool_arena(TopkPool *p) {
    if (p->arena.p) return 1;
    RC_CUDA(cudaSetDevice(p->device));
    return p->arena.alloc((size_t)p->capacity * p->slot_bytes);
}

// gate/up + down + weighted sum of the selected slots on `s`; x_dev [hidden], out_dev [row_count]
int pool_run(TopkPool *p, const uint32_t *slot_ids, const uint64_t *gate_bytes, const uint64_t *up_bytes, const uint64_t *down_bytes,
             const float *router_weights, uint32_t top_k, uint32_t type_word, uint32_t hidden, uint32_t ffn, uint32_t row_start, uint32_t row_count,
             const float *x_dev, float *out_dev, cudaStream_t s) {
    const uint32_t tg = type_word & 255u, td = (type_word >> 8) & 255u ? (type_word >> 8) & 255u : tg;
    RC_REQUIRE(rc_is_quant(tg) && rc_is_quant(td), "expert pool: ggml types %u / %u are not served (16, 14, 21)", tg, td);
    RC_REQUIRE(top_k >= 1 && top_k <= REDCUDA_MAX_TOPK && hidden % 256u == 0 && ffn % 256u == 0, "expert pool: bad top_k or shape");
    RC_REQUIRE(row_start + (uint64_t)row_count <= hidden && row_count, "expert pool: output rows outside the matrix");
    if (!require_books(tg) || !require_books(td)) return 0;
    const uint64_t gu_b = rc_matrix_bytes(tg, ffn, hidden), dn_b = rc_matrix_bytes(td, hidden, ffn);
    RC_REQUIRE(gu_b % 16u == 0 && dn_b % 16u == 0, "expert pool: matrix sizes must be multiples of 16 bytes");
    for (uint32_t k = 0; k < top_k; ++k) {
        RC_REQUIRE(slot_ids[k] < p->capacity && p->generation[slot_ids[k]] != 0u, "expert pool: slot %u is empty or out of range", slot_ids[k]);
        RC_REQUIRE(gate_bytes[k] == gu_b && up_bytes[k] == gu_b && down_bytes[k] == dn_b && gu_b * 2u + dn_b <= p->slot_bytes,
                   "expert pool: slot %u byte counts do not match the type and shape", slot_ids[k]);
    }
    // scratch: planar copies of the selected experts, the grouping arrays, activations
    const size_t a16 = 256;
    size_t off = 0;
    auto take = [&](size_t n) { const size_t o = off; off = (off + n + a16 - 1) / a16 * a16; return o; };
    const size_t o_g = take(gu_b * top_k), o_u = take(gu_b * top_k), o_d = take(dn_b * top_k), o_idx = take((size_t)(3u * top_k + 8u) * 4u), o_w = take(top_k * 4u),
                 o_act = take((size_t)top_k * ffn * 4u), o_tmp = take((size_t)top_k * hidden * 4u), o_out = take((size_t)hidden * 4u);
    if (p->scratch.bytes < off && !p->scratch.alloc(off)) return 0;
    uint8_t *S = p->scratch.as<uint8_t>();
    const uint8_t *A0 = p->arena.as<uint8_t>();
    for (uint32_t k = 0; k < top_k; ++k) {
        const uint8_t *slot = A0 + (size_t)slot_ids[k] * p->slot_bytes;
        if (!upload_matrix(tg, ffn, hidden, slot, true, S + o_g + k * gu_b, nullptr, s) || !upload_matrix(tg, ffn, hidden, slot + gu_b, true, S + o_u + k * gu_b, nullptr, s) ||
            !upload_matrix(td, hidden, ffn, slot + 2u * gu_b, true, S + o_d + k * dn_b, nullptr, s)) return 0;
    }
    // grouping of a single token: pair k = group k = scratch expert k
    uint32_t *hidx = reinterpret_cast<uint32_t *>(p->pin);
    for (uint32_t k = 0; k < top_k; ++k) { hidx[k] = k; hidx[top_k + k] = k; hidx[2u * top_k + k] = k; }      // sorted | uexp | ustart
    hidx[3u * top_k] = top_k; hidx[3u * top_k + 1u] = top_k;                                                  // ustart[top_k] | n_unique
    memcpy(hidx + 3u * top_k + 8u, router_weights, top_k * 4u);
    RC_CUDA(cudaMemcpyAsync(S + o_idx, hidx, (3u * top_k + 2u) * 4u, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemcpyAsync(S + o_w, hidx + 3u * top_k + 8u, top_k * 4u, cudaMemcpyHostToDevice, s));
    uint32_t *d_idx = reinterpret_cast<uint32_t *>(S + o_idx);
    MoeArgs A{};
    A.expert_begin = 0; A.n_local = top_k; A.status = status_words();
    A.sorted = d_idx; A.uexp = d_idx + top_k; A.ustart = d_idx + 2u * top_k; A.n_unique = d_idx + 3u * top_k + 1u;
    A.iq2 = books_iq2(); A.iq3s = books_iq3s();
    for (int pass = 0; pass < 2; ++pass) {
        const bool gu = pass == 0;
        A.w0 = S + (gu ? o_g : o_d); A.w1 = gu ? S + o_u : nullptr; A.mat_bytes = gu ? gu_b : dn_b;
        A.type = gu ? tg : td; A.nrows = gu ? ffn : hidden; A.ncols = gu ? hidden : ffn; A.nb = (uint64_t)A.nrows * (A.ncols / 256u);
        A.x = gu ? x_dev : reinterpret_cast<const float *>(S + o_act); A.x_stride = gu ? hidden : ffn; A.x_div = gu ? top_k : 1u;
        A.out = reinterpret_cast<float *>(S + (gu ? o_act : o_tmp)); A.out_stride = gu ? ffn : hidden; A.pair_silu = gu ? 1u : 0u;
        uint32_t lpr = 32u;
        while (lpr > (A.ncols >> 6)) lpr >>= 1;
        A.rows_per_tile = 8u * (32u / lpr);
        const dim3 grid((A.nrows + A.rows_per_tile - 1u) / A.rows_per_tile, top_k);
        const size_t smem = (size_t)x_padded(A.ncols) * sizeof(float);
        RC_REQUIRE(smem <= 200u * 1024u, "expert pool: row length %u too large", A.ncols);
        if (smem > 48u * 1024u) RC_CUDA(cudaFuncSetAttribute(k_moe_experts<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        RC_LAUNCH((k_moe_experts<1>), grid, 256, smem, s, A);
        RC_LAUNCHED();
    }
    RC_LAUNCH((k_moe_combine), dim3((hidden / 4u + 255u) / 256u, 1), 256, 0, s, reinterpret_cast<const float *>(S + o_tmp), reinterpret_cast<const float *>(S + o_w), top_k,
              (const float *)nullptr, (const float *)nullptr, (const float *)nullptr, reinterpret_cast<float *>(S + o_out), hidden, (const uint32_t *)nullptr);
    RC_LAUNCHED();
    RC_CUDA(cudaMemcpyAsync(out_dev, S + o_out + (size_t)row_start * 4u, (size_t)row_count * 4u, cudaMemcpyDeviceToDevice, s));
    return 1;
}

}  // namespace

extern "C" {

uint32_t redmetal_topk_abi_version(void) { return 1u; }
const char *redmetal_topk_last_error(void) { return redcuda_last_error(); }

redmetal_topk_pool_t redmetal_topk_pool_create(const char *model_path, uint64_t budget_bytes, uint64_t slot_bytes, uint32_t slots_per_slab,
                                               const int8_t *, uint32_t, const int8_t *, uint32_t) {
    (void)slots_per_slab;
    if (!require_device()) return nullptr;
    if (!model_path || !slot_bytes || slot_bytes % 16u || budget_bytes < slot_bytes) { set_error("expert pool: model path, a slot size that is a multiple of 16 and a budget of at least one slot are required"); return nullptr; }
    TopkPool *p = new (std::nothrow) TopkPool();
    if (!p) { set_error("expert pool: out of host memory"); return nullptr; }
    p->fd = open(model_path, O_RDONLY);
    if (p->fd < 0) { set_error("expert pool: cannot open %s", model_path); delete p; return nullptr; }
    cudaGetDevice(&p->device);
    p->slot_bytes = slot_bytes;
    const uint64_t cap = budget_bytes / slot_bytes;
    p->capacity = cap > 0xffffffffull ? 0xffffffffu : (uint32_t)cap;
    p->generation.assign(p->capacity, 0u); p->inflight.assign(p->capacity, 0u);
    p->pin_bytes = (size_t)slot_bytes > (1u << 16) ? (size_t)slot_bytes : (1u << 16);
    if (cudaMallocHost((void **)&p->pin, p->pin_bytes) != cudaSuccess || cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking) != cudaSuccess) {
        set_error("expert pool: staging buffer or stream creation failed"); redmetal_topk_pool_destroy(p); return nullptr;
    }
    status_words();
    return p;
}

void redmetal_topk_pool_destroy(redmetal_topk_pool_t h) {
    TopkPool *p = (TopkPool *)h;
    if (!p) return;
    if (p->stream) { cudaStreamSynchronize(p->stream); cudaStreamDestroy(p->stream); }
    if (p->pin) cudaFreeHost(p->pin);
    if (p->fd >= 0) close(p->fd);
    delete p;
}

int redmetal_topk_pool_set_classes(redmetal_topk_pool_t h, uint32_t n, const uint64_t *slot_bytes, const uint32_t *capacity) {
    TopkPool *p = (TopkPool *)h;
    RC_REQUIRE(p && n >= 1 && n <= 8u && slot_bytes && capacity, "expert pool: bad size classes");
    uint64_t total = 0;
    for (uint32_t i = 0; i < n; ++i) { RC_REQUIRE(slot_bytes[i] && slot_bytes[i] <= p->slot_bytes, "expert pool: class %u does not fit a slot", i); total += capacity[i]; }
    RC_REQUIRE(total <= p->capacity && !p->arena.p, "expert pool: classes exceed the capacity, or slots are already in use");
    return 1;       // one arena of full-size slots serves every class: nothing to re-partition
}
uint32_t redmetal_topk_pool_capacity(redmetal_topk_pool_t h) { return h ? ((TopkPool *)h)->capacity : 0u; }
uint32_t redmetal_topk_pool_slab_count(redmetal_topk_pool_t h) { return h && ((TopkPool *)h)->arena.p ? 1u : 0u; }
uint64_t redmetal_topk_pool_allocated_bytes(redmetal_topk_pool_t h) { return h ? ((TopkPool *)h)->arena.bytes : 0u; }
uint64_t redmetal_topk_pool_bytes_read(redmetal_topk_pool_t h) { return h ? ((TopkPool *)h)->bytes_read : 0u; }
uint64_t redmetal_topk_pool_read_calls(redmetal_topk_pool_t h) { return h ? ((TopkPool *)h)->read_calls : 0u; }
double redmetal_topk_pool_read_ms(redmetal_topk_pool_t h) { return h ? ((TopkPool *)h)->read_ms : 0.0; }
uint32_t redmetal_topk_pool_slot_generation(redmetal_topk_pool_t h, uint32_t slot) { TopkPool *p = (TopkPool *)h; return p && slot < p->capacity ? p->generation[slot] : 0u; }
int redmetal_topk_pool_slot_inflight(redmetal_topk_pool_t h, uint32_t slot) { TopkPool *p = (TopkPool *)h; return p && slot < p->capacity ? (int)p->inflight[slot] : 0; }
int redmetal_topk_pool_allocate_all(redmetal_topk_pool_t h) { RC_REQUIRE(h, "expert pool: null pool"); return pool_arena((TopkPool *)h); }

int redmetal_topk_pool_load_expert(redmetal_topk_pool_t h, uint32_t slot, uint64_t g_off, uint64_t g_bytes, uint64_t u_off, uint64_t u_bytes, uint64_t d_off, uint64_t d_bytes,
                                   uint64_t *bytes_read, double *elapsed_ms) {
    TopkPool *p = (TopkPool *)h;
    RC_REQUIRE(p && slot < p->capacity, "expert pool: slot %u out of range", slot);
    RC_REQUIRE(g_bytes + u_bytes + d_bytes <= p->slot_bytes && g_bytes + u_bytes + d_bytes <= p->pin_bytes, "expert pool: expert of %llu bytes does not fit a slot",
               (unsigned long long)(g_bytes + u_bytes + d_bytes));
    RC_REQUIRE(p->inflight[slot] == 0u, "expert pool: slot %u is in flight", slot);
    if (!pool_arena(p)) return 0;
    const double t0 = pool_now_ms();
    RC_CUDA(cudaStreamSynchronize(p->stream));          // the staging buffer is reused
    const uint64_t offs[3] = {g_off, u_off, d_off}, lens[3] = {g_bytes, u_bytes, d_bytes};
    size_t at = 0;
    for (int i = 0; i < 3; ++i) {
        size_t done = 0;
        while (done < lens[i]) {
            const ssize_t r = pread(p->fd, p->pin + at + done, lens[i] - done, (off_t)(offs[i] + done));
            RC_REQUIRE(r > 0, "expert pool: short read at offset %llu", (unsigned long long)(offs[i] + done));
            done += (size_t)r;
        }
        at += lens[i];
    }
    RC_CUDA(cudaMemcpyAsync(p->arena.as<uint8_t>() + (size_t)slot * p->slot_bytes, p->pin, at, cudaMemcpyHostToDevice, p->stream));
    RC_CUDA(cudaStreamSynchronize(p->stream));
    const double ms = pool_now_ms() - t0;
    p->generation[slot] += 1u; p->bytes_read += at; p->read_calls += 3u; p->read_ms += ms;
    if (bytes_read) *bytes_read = at;
    if (elapsed_ms) *elapsed_ms = ms;
    return 1;
}

int redmetal_topk_pool_slot_addresses(redmetal_topk_pool_t h, uint32_t slot, uint64_t g_bytes, uint64_t u_bytes, uint64_t d_bytes, uint64_t *ga, uint64_t *ua, uint64_t *da) {
    TopkPool *p = (TopkPool *)h;
    RC_REQUIRE(p && slot < p->capacity && ga && ua && da && g_bytes + u_bytes + d_bytes <= p->slot_bytes, "expert pool: bad slot or sizes");
    if (!pool_arena(p)) return 0;
    const uint64_t base = (uint64_t)(uintptr_t)(p->arena.as<uint8_t>() + (size_t)slot * p->slot_bytes);
    *ga = base; *ua = base + g_bytes; *da = base + g_bytes + u_bytes;
    return 1;
}

int redmetal_topk_pool_execute(redmetal_topk_pool_t h, const uint32_t *slot_ids, const uint64_t *gate_bytes, const uint64_t *up_bytes, const uint64_t *down_bytes,
                               const float *router_weights, uint32_t top_k, uint32_t ggml_type, uint32_t hidden, uint32_t ffn, uint32_t row_start, uint32_t row_count,
                               const float *input, uint32_t input_count, float *output, uint32_t output_count, double *elapsed_ms) {
    TopkPool *p = (TopkPool *)h;
    RC_REQUIRE(p && slot_ids && gate_bytes && up_bytes && down_bytes && router_weights && input && output, "expert pool: null argument");
    RC_REQUIRE(input_count == hidden && output_count == row_count, "expert pool: input / output counts do not match the shape");
    RC_REQUIRE(p->arena.p, "expert pool: no expert has been loaded");
    RC_CUDA(cudaSetDevice(p->device));
    const double t0 = pool_now_ms();
    DevMem x, o;
    if (!x.alloc((size_t)hidden * 4u) || !o.alloc((size_t)row_count * 4u)) return 0;
    cudaStream_t s = p->stream;
    RC_CUDA(cudaMemcpyAsync(x.p, input, (size_t)hidden * 4u, cudaMemcpyHostToDevice, s));
    if (!pool_run(p, slot_ids, gate_bytes, up_bytes, down_bytes, router_weights, top_k, ggml_type, hidden, ffn, row_start, row_count, x.as<float>(), o.as<float>(), s)) return 0;
    RC_CUDA(cudaMemcpyAsync(output, o.p, (size_t)row_count * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    if (status_failed()) return 0;
    if (elapsed_ms) *elapsed_ms = pool_now_ms() - t0;
    return 1;
}

int redmetal_topk_pool_encode(redmetal_topk_pool_t h, void *stream, const uint32_t *slot_ids, const uint64_t *gate_bytes, const uint64_t *up_bytes, const uint64_t *down_bytes,
                              const float *router_weights, uint32_t top_k, uint32_t ggml_type, uint32_t hidden, uint32_t ffn, uint32_t row_start, uint32_t row_count,
                              void *in_dev, uint64_t in_off, void *out_dev, uint64_t out_off) {
    TopkPool *p = (TopkPool *)h;
    RC_REQUIRE(p && slot_ids && gate_bytes && up_bytes && down_bytes && router_weights && in_dev && out_dev, "expert pool: null argument");
    RC_REQUIRE(p->arena.p, "expert pool: no expert has been loaded");
    RC_CUDA(cudaStreamSynchronize((cudaStream_t)stream));        // the pinned grouping words and the scratch are shared by the pool's calls
    if (!pool_run(p, slot_ids, gate_bytes, up_bytes, down_bytes, router_weights, top_k, ggml_type, hidden, ffn, row_start, row_count,
                  reinterpret_cast<const float *>((const uint8_t *)in_dev + in_off), reinterpret_cast<float *>((uint8_t *)out_dev + out_off), (cudaStream_t)stream)) return 0;
    for (uint32_t k = 0; k < top_k; ++k) p->inflight[slot_ids[k]] += 1u;
    return 1;
}

void redmetal_topk_pool_release(redmetal_topk_pool_t h, const uint32_t *slot_ids, uint32_t top_k) {
    TopkPool *p = (TopkPool *)h;
    if (!p || !slot_ids) return;
    for (uint32_t k = 0; k < top_k; ++k) if (slot_ids[k] < p->capacity && p->inflight[slot_ids[k]]) p->inflight[slot_ids[k]] -= 1u;
}

int redmetal_topk_pool_residency_table_init(redmetal_topk_pool_t h, uint32_t layers, uint32_t experts) {
    TopkPool *p = (TopkPool *)h;
    RC_REQUIRE(p && layers && experts, "expert pool: bad residency table shape");
    RC_CUDA(cudaSetDevice(p->device));
    if (!p->table.alloc((size_t)layers * experts * 8u)) return 0;
    RC_CUDA(cudaMemset(p->table.p, 0, (size_t)layers * experts * 8u));
    p->table_h.assign((size_t)layers * experts, 0u); p->layers = layers; p->experts = experts;
    return 1;
}
void *redmetal_topk_pool_residency_table(redmetal_topk_pool_t h) { return h ? ((TopkPool *)h)->table.p : nullptr; }
int redmetal_topk_pool_residency_set(redmetal_topk_pool_t h, uint32_t layer, uint32_t expert, uint32_t slot) {
    TopkPool *p = (TopkPool *)h;
    RC_REQUIRE(p && p->table.p && layer < p->layers && expert < p->experts && slot < p->capacity, "expert pool: residency entry out of range");
    if (!pool_arena(p)) return 0;
    const size_t i = (size_t)layer * p->experts + expert;
    p->table_h[i] = (uint64_t)(uintptr_t)(p->arena.as<uint8_t>() + (size_t)slot * p->slot_bytes);
    RC_CUDA(cudaMemcpy(p->table.as<uint64_t>() + i, &p->table_h[i], 8u, cudaMemcpyHostToDevice));
    return 1;
}
void redmetal_topk_pool_residency_clear(redmetal_topk_pool_t h, uint32_t layer, uint32_t expert) {
    TopkPool *p = (TopkPool *)h;
    if (!p || !p->table.p || layer >= p->layers || expert >= p->experts) return;
    const size_t i = (size_t)layer * p->experts + expert;
    p->table_h[i] = 0u;
    cudaMemcpy(p->table.as<uint64_t>() + i, &p->table_h[i], 8u, cudaMemcpyHostToDevice);
}

}  // extern "C"
