// rl_engine_* on CUDA: the persistent Qwen3-Next decode engine (every weight and every routed expert resident in HBM).
//
// One token (rl_engine_cpu_step, native/redlite_native_engine_cpu.c:390-441, is the arithmetic being reproduced):
//   embedding row -> 48 x { RMSNorm -> Gated DeltaNet or gated GQA attention -> residual + RMSNorm -> MoE FFN + residual }
//   -> final RMSNorm -> LM head.
// Everything runs on one stream without a host round trip; the host mirrors the reference keeps for parity checks
// (embedding, per-layer outputs, final norm, router ids, native/redlite_native_engine_internal.h:35-47) are copied back
// at the end of the step together with the logits.
#include "redcuda_common.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_kquants.cuh"
#include "redcuda_moe_mma.cuh"
#include "redcuda_tc_gemm.cuh"
#include "redcuda_gguf.h"
#include "../../include/redcuda.h"
#include "../../include/rl_engine.h"

#include <math.h>
#include <stdlib.h>
#include <algorithm>
#include <chrono>
#include <new>
#include <vector>

namespace rc {

const uint32_t *moe_last_ids_device(const redcuda_moe *m);   // redcuda_moe.cu
void moe_set_ids_mirror(redcuda_moe *m, uint32_t *dev_ptr);   // a single token's router ids are also written to dev_ptr
size_t moe_workspace_bytes(const redcuda_moe_desc *d);
// expert parallelism: which contiguous share of every layer's experts the engines opened next will hold
static thread_local int g_shard_rank = 0, g_shard_world = 1;
redcuda_moe *moe_create_shared(const redcuda_moe_desc *d, void *workspace);   // workspace shared by layers that run on one stream

static double now_ms() { return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

// ---- small kernels ----
// out[b] = dequantised embedding row of token[b] (grid = tokens, block = 256 threads)
__global__ void k_embed_row(const uint8_t *__restrict__ base, uint32_t type, uint64_t nb, uint32_t ncols, uint32_t nrows, const uint32_t *__restrict__ token,
                            const uint8_t *iq2, const uint32_t *iq3s, float *__restrict__ out, uint32_t *__restrict__ status) {
    pdl_prologue();
    uint64_t row = token[blockIdx.x];
    if (row >= nrows) { row = 0; if (status && threadIdx.x == 0) status[ST_TOKEN_RANGE] = 1u; }   // never index the table with an id the argmax could not form
    out += (size_t)blockIdx.x * ncols;
    if (type == RC_F32) { for (uint32_t i = threadIdx.x; i < ncols; i += blockDim.x) out[i] = reinterpret_cast<const float *>(base)[row * ncols + i]; return; }
    if (type == RC_F16) { for (uint32_t i = threadIdx.x; i < ncols; i += blockDim.x) out[i] = __half2float(__ushort_as_half(reinterpret_cast<const unsigned short *>(base)[row * ncols + i])); return; }
    if (rc_is_file_layout_quant(type)) {
        const uint8_t *rp = base + row * rc_row_bytes(type, ncols);
        for (uint32_t i = threadIdx.x; i < ncols; i += blockDim.x) out[i] = kq_row_value(type, rp, i);
        return;
    }
    const RcBooks bk{iq2, iq3s};
    const uint32_t bpr = ncols >> 8;
    for (uint32_t g = threadIdx.x; g < bpr * 32u; g += blockDim.x) {
        float v[8];
        rc_decode8(type, base, nb, row * bpr + (g >> 5), g & 31u, bk, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) out[g * 8u + j] = v[j];
    }
}

__device__ __forceinline__ double block_sum_d(double v, double *red) {
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0.0;
    for (uint32_t w = 0; w < (blockDim.x + 31u) / 32u; ++w) t += red[w];
    __syncthreads();
    return t;
}

// normed = RMSNorm(x [+ branch]) * w (engine_cpu.c:96-101, 418-424); resid_out (optional) = x + branch. One block per token.
__global__ void __launch_bounds__(1024) k_rmsnorm(const float *__restrict__ x, const float *__restrict__ branch, const float *__restrict__ w,
                                                  uint32_t n, float eps, float *__restrict__ resid_out, float *__restrict__ normed) {
    pdl_prologue();
    __shared__ double red[32];
    const size_t tok_off = (size_t)blockIdx.x * n;
    x += tok_off; normed += tok_off;
    if (branch) branch += tok_off;
    if (resid_out) resid_out += tok_off;
    double ss = 0.0;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v = x[i];
        if (branch) v = v + branch[i];
        if (resid_out) resid_out[i] = v;
        ss += (double)v * (double)v;
    }
    const double tot = block_sum_d(ss, red);
    const double inv = 1.0 / sqrt(tot / (double)n + (double)eps);
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v = x[i];
        if (branch) v = v + branch[i];
        normed[i] = (float)((double)v * inv * (double)w[i]);
    }
}

template <typename KV> __device__ __forceinline__ KV to_kv(float v);
template <> __device__ __forceinline__ float to_kv<float>(float v) { return v; }
template <> __device__ __forceinline__ __half to_kv<__half>(float v) { return __float2half_rn(v); }
__device__ __forceinline__ float from_kv(float v) { return v; }
__device__ __forceinline__ float from_kv(__half v) { return __half2float(v); }

// Per-head RMSNorm of q and k, NeoX RoPE on the first rope_dims, K/V rows appended to the cache (engine_cpu.c:277-296).
// grid = (n_head + 2 * n_kv, tokens) blocks of head_dim threads; token z sits at position pos_p[z].
template <typename KV>
__global__ void k_attn_prep(const float *__restrict__ qg, const float *__restrict__ kraw, const float *__restrict__ vraw,
                            const float *__restrict__ qn, const float *__restrict__ kn, uint32_t n_head, uint32_t n_kv, uint32_t hd,
                            uint32_t rope_dims, float freq_base, float eps, const uint32_t *__restrict__ pos_p, float *__restrict__ query, float *__restrict__ gate,
                            KV *__restrict__ kcache, KV *__restrict__ vcache) {
    pdl_prologue();
    extern __shared__ float sh[];
    __shared__ double red[32];
    const uint32_t b = blockIdx.x, tid = threadIdx.x, z = blockIdx.y, pos = pos_p[z];   // the position lives in device memory: a captured graph replays for every token
    qg += (size_t)z * n_head * 2u * hd; kraw += (size_t)z * n_kv * hd; vraw += (size_t)z * n_kv * hd;
    query += (size_t)z * n_head * hd; gate += (size_t)z * n_head * hd;
    if (b >= n_head + n_kv) {      // value head: plain append
        const uint32_t kh = b - n_head - n_kv;
        vcache[((size_t)pos * n_kv + kh) * hd + tid] = to_kv<KV>(vraw[(size_t)kh * hd + tid]);
        return;
    }
    const bool is_q = b < n_head;
    const uint32_t h = is_q ? b : b - n_head;
    const float src = is_q ? qg[(size_t)h * 2u * hd + tid] : kraw[(size_t)h * hd + tid];
    if (is_q) gate[(size_t)h * hd + tid] = qg[(size_t)h * 2u * hd + hd + tid];
    const double tot = block_sum_d((double)src * (double)src, red);
    const double inv = 1.0 / sqrt(tot / (double)hd + (double)eps);
    const float val = (float)((double)src * inv * (double)(is_q ? qn[tid] : kn[tid]));
    sh[tid] = val;
    __syncthreads();
    float outv = val;
    if (tid < rope_dims) {
        const uint32_t half = rope_dims >> 1, i = tid < half ? tid : tid - half;
        const float fr = (float)pow((double)freq_base, (double)(-2.0f * (float)i / (float)rope_dims));
        const float theta = __fmul_rn((float)pos, fr);
        const float c = (float)cos((double)theta), s = (float)sin((double)theta);
        const float x0 = sh[i], x1 = sh[half + i];
        outv = tid < half ? __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)) : __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
    if (is_q) query[(size_t)h * hd + tid] = outv;
    else kcache[((size_t)pos * n_kv + h) * hd + tid] = to_kv<KV>(outv);
}

// Split-K decode attention. grid = (n_kv, nsplit, tokens), block = 256 (8 warps); token z attends to positions <= pos_p[z]
// (the K/V rows of a whole prefill chunk are appended before this runs, so the mask is the sequence length alone). Every block serves the G query heads of one
// K/V head over a slice of positions (K and V rows are read once for all G heads); a warp takes every 8th position,
// a lane VPL = head_dim/32 consecutive dimensions; online softmax per head. Partials: m, l and the accumulator.
template <typename KV, int VPL, int G>
__global__ void __launch_bounds__(256) k_attn_decode(const float *__restrict__ query, const KV *__restrict__ kcache, const KV *__restrict__ vcache,
                                                     uint32_t n_kv, const uint32_t *__restrict__ pos_p, uint32_t nsplit, float scale,
                                                     float *__restrict__ part_m, float *__restrict__ part_l, float *__restrict__ part_acc) {
    pdl_prologue();
    extern __shared__ float sm[];            // [8][G][hd] accumulators, then [8][G] m, [8][G] l
    constexpr uint32_t hd = VPL * 32u;
    const uint32_t kvh = blockIdx.x, split = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t n_head = n_kv * G;
    const uint32_t seq_len = pos_p[blockIdx.z] + 1u;
    query += (size_t)blockIdx.z * n_head * hd;
    part_m += (size_t)blockIdx.z * n_head * nsplit; part_l += (size_t)blockIdx.z * n_head * nsplit; part_acc += (size_t)blockIdx.z * n_head * nsplit * hd;
    // slices of at least 32 positions; at short sequences the trailing blocks find an empty slice and report m = -inf
    const uint32_t per = max((seq_len + nsplit - 1u) / nsplit, 32u), p_begin = min(split * per, seq_len), p_end = min(seq_len, p_begin + per);
    float q[G][VPL], acc[G][VPL], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) { q[g][i] = query[((size_t)kvh * G + g) * hd + lane * VPL + i] * scale; acc[g][i] = 0.f; }
    }
    for (uint32_t p = p_begin + warp; p < p_end; p += 8u) {
        const KV *kp = kcache + ((size_t)p * n_kv + kvh) * hd + lane * VPL, *vp = vcache + ((size_t)p * n_kv + kvh) * hd + lane * VPL;
        float kx[VPL], vx[VPL];
#pragma unroll
        for (int i = 0; i < VPL; ++i) { kx[i] = from_kv(kp[i]); vx[i] = from_kv(vp[i]); }
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < VPL; ++i) d += q[g][i] * kx[i];
            s[g] = d;
        }
#pragma unroll
        for (int o = 16; o; o >>= 1)
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float mn = fmaxf(m[g], s[g]);
            const float c = expf(m[g] - mn), pe = expf(s[g] - mn);
            l[g] = l[g] * c + pe;
#pragma unroll
            for (int i = 0; i < VPL; ++i) acc[g][i] = acc[g][i] * c + pe * vx[i];
            m[g] = mn;
        }
    }
    float *s_acc = sm, *s_m = sm + 8u * G * hd, *s_l = s_m + 8u * G;
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int i = 0; i < VPL; ++i) s_acc[((size_t)warp * G + g) * hd + lane * VPL + i] = acc[g][i];
        if (lane == 0) { s_m[warp * G + g] = m[g]; s_l[warp * G + g] = l[g]; }
    }
    __syncthreads();
    for (uint32_t idx = threadIdx.x; idx < G * hd; idx += 256u) {
        const uint32_t g = idx / hd, d = idx - g * hd;
        float M = -INFINITY;
        for (int w = 0; w < 8; ++w) M = fmaxf(M, s_m[w * G + g]);
        float L = 0.f, A = 0.f;
        if (M > -INFINITY) {
            for (int w = 0; w < 8; ++w) {
                const float e = expf(s_m[w * G + g] - M);
                L += s_l[w * G + g] * e; A += s_acc[((size_t)w * G + g) * hd + d] * e;
            }
        }
        const size_t head = (size_t)kvh * G + g;
        part_acc[(head * nsplit + split) * hd + d] = A;
        if (d == 0) { part_m[head * nsplit + split] = M; part_l[head * nsplit + split] = L; }
    }
}

// merge the split partials, normalise, apply the sigmoid output gate (engine_cpu.c:312-317). grid = (n_head, tokens), block = hd
__global__ void k_attn_merge(const float *__restrict__ part_m, const float *__restrict__ part_l, const float *__restrict__ part_acc,
                             const float *__restrict__ gate, uint32_t nsplit, uint32_t hd, float *__restrict__ gated) {
    pdl_prologue();
    const uint32_t h = blockIdx.x, d = threadIdx.x;
    const size_t zoff = (size_t)blockIdx.y * gridDim.x;
    part_m += zoff * nsplit; part_l += zoff * nsplit; part_acc += zoff * nsplit * hd; gate += zoff * hd; gated += zoff * hd;
    float M = -INFINITY;
    for (uint32_t s = 0; s < nsplit; ++s) M = fmaxf(M, part_m[(size_t)h * nsplit + s]);
    float L = 0.f, A = 0.f;
    for (uint32_t s = 0; s < nsplit; ++s) {
        const float pm = part_m[(size_t)h * nsplit + s];
        if (pm == -INFINITY) continue;
        const float e = expf(pm - M);
        L += part_l[(size_t)h * nsplit + s] * e; A += part_acc[((size_t)h * nsplit + s) * hd + d] * e;
    }
    const double o = (double)A / (double)L;
    gated[(size_t)h * hd + d] = (float)(o / (1.0 + exp(-(double)gate[(size_t)h * hd + d])));
}

// argmax of n floats, ties to the lowest index; one block of 1024
__global__ void k_advance(uint32_t *pos) {
    pdl_prologue(); if (threadIdx.x == 0 && blockIdx.x == 0) *pos += 1u; }

// gen_log / gen_count (optional): the chosen id is also appended to gen_log[*gen_count]
__global__ void __launch_bounds__(1024) k_argmax(const float *__restrict__ v, uint32_t n, uint32_t *__restrict__ out, uint32_t *__restrict__ gen_log,
                                                 uint32_t *__restrict__ gen_count, uint32_t *__restrict__ status) {
    pdl_prologue();
    __shared__ float bv[32];
    __shared__ uint32_t bi[32];
    float best = -INFINITY; uint32_t idx = 0xffffffffu;
    for (uint32_t i = threadIdx.x; i < n; i += 1024u) { const float x = v[i]; if (x > best || (x == best && i < idx)) { best = x; idx = i; } }
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o); const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31u) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 32; ++w) if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
        if (idx >= n) { idx = 0; if (status) status[ST_TOKEN_RANGE] = 1u; }      // every logit NaN: nothing compared greater
        *out = idx;
        if (gen_log) { gen_log[*gen_count] = idx; *gen_count += 1u; }
    }
}

struct EngLayer {
    bool recurrent = false;
    uint32_t ridx = 0, aidx = 0;
    const float *attn_norm = nullptr, *post_norm = nullptr;
    DMat qkv, z, ba, ssm_out, q, k, v, o;
    const float *conv_k = nullptr, *dt = nullptr, *a = nullptr, *ssm_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    redcuda_moe *moe = nullptr;
};

}  // namespace rc

using namespace rc;

struct rl_engine {
    rl_engine_config cfg;
    rl_engine_info info;
    GgufFile gguf;
    std::vector<EngLayer> layers;
    DMat tok_embd, output;
    const float *output_norm = nullptr;
    int ep_rank = 0, ep_world = 1;       // expert shard of this engine (contiguous: experts [rank * E / world, (rank + 1) * E / world))
    redcuda_ep *ep = nullptr;            // attached exchange context (not owned); required before the first step when ep_world > 1
    DevMem dense, state, scratch, moe_ws;      // moe_ws: the expert workspace shared by every layer
    bool kv_half = false;
    uint32_t position = 0, ffn = 0, ffn_sh = 0;
    uint64_t expert_bytes = 0, dense_step_bytes = 0;
    double preload_ms = 0.0;
    // state
    float *conv = nullptr, *rec = nullptr;
    void *kcache = nullptr, *vcache = nullptr;
    // scratch (device)
    float *x0 = nullptr, *normed = nullptr, *branch = nullptr, *resid = nullptr, *qkv = nullptr, *z = nullptr, *ba = nullptr, *ng = nullptr;
    float *dn_qk = nullptr, *dn_v = nullptr, *dn_beta = nullptr, *dn_gate = nullptr, *dn_core = nullptr;
    float *qg = nullptr, *kraw = nullptr, *vraw = nullptr, *query = nullptr, *gate = nullptr, *gated = nullptr, *part_m = nullptr, *part_l = nullptr, *part_acc = nullptr;
    float *embed_d = nullptr, *layer_out_d = nullptr, *final_norm_d = nullptr, *logits_d = nullptr;
    uint32_t *router_ids_d = nullptr, *token_d = nullptr, *gen_tokens_d = nullptr, *pos_d = nullptr, *gen_count_d = nullptr;
    cudaGraphExec_t graph_greedy = nullptr;      // one greedy token (step + LM head + argmax), captured after the first eager token
    bool graph_failed = false;
    uint64_t graph_launches = 0;
    uint32_t max_split = 64, pf_split = 8;
    uint32_t pb = 1;                             // tokens per prefill chunk; every per-token scratch buffer holds pb rows
    float *bx[2] = {nullptr, nullptr};           // layer input / output of a chunk (ping-pong)
    int8_t *xq = nullptr; float *sx = nullptr;   // chunk activations as digit planes for the Q6_K tensor-core projections
    uint32_t *tok_chunk_d = nullptr, *pos_chunk_d = nullptr;
    float *dn_pd = nullptr;          // DeltaNet prefill: the 16 pair products of every group of four tokens and key head
    __half *tc_xs = nullptr; float *tc_xinv = nullptr; uint32_t *tc_err = nullptr;   // tcgen05 GEMM: activation digits, per-token inverse scales, timeout flag
    uint8_t *tc_wd = nullptr; float *tc_winv = nullptr; size_t tc_wd_cap = 0;        // and the weight digits of one launch (widest projection group)
    // host mirrors
    std::vector<float> embed_h, layer_out_h, final_norm_h;
    std::vector<uint32_t> router_ids_h;
    uint32_t *token_pin = nullptr;
    cudaStream_t stream = nullptr;
    int device = 0;
};

static void eng_err(char *error, size_t cap, const char *msg) { if (error && cap) snprintf(error, cap, "%s", msg ? msg : "unknown engine error"); }
#define ENG_FAIL(...) do { char b_[512]; snprintf(b_, sizeof(b_), __VA_ARGS__); eng_err(error, cap, b_); return 0; } while (0)
#define ENG_RC(call) do { if (!(call)) { eng_err(error, cap, redcuda_last_error()); return 0; } } while (0)
#define ENG_CUDA(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) { ENG_FAIL("%s failed: %s", #expr, cudaGetErrorString(e_)); } } while (0)

static int eng_gemv(rl_engine *e, const DMat *mats, float *const *outs, uint32_t n, const float *x, const char *tag) {
    GemvArgs A{};
    A.njobs = n; A.ntok = 1; A.x = x; A.x_stride = mats[0].ncols; A.tag = tag;
    for (uint32_t j = 0; j < n; ++j) {
        GemvJob &J = A.job[j];
        J.w0 = mats[j].base; J.w1 = nullptr; J.out = outs[j]; J.nb = mats[j].nb; J.type = mats[j].type; J.nrows = mats[j].nrows; J.ncols = mats[j].ncols;
        J.out_stride = mats[j].nrows; J.epi = GEMV_STORE;
    }
    return launch_gemv(A, e->stream);
}

// ntok tokens at positions pos[0..ntok): decode passes e->pos_d (one token), a prefill chunk its position list
template <typename KV>
static int eng_attention(rl_engine *e, const EngLayer &L, uint32_t ntok, const uint32_t *pos, char *error, size_t cap) {
    const rl_engine_info &in = e->info;
    const uint32_t hd = in.head_dim, nq = in.n_head, nkv = in.n_head_kv, G = nq / nkv;
    const size_t kv_layer = (size_t)in.context * nkv * hd;
    KV *kc = (KV *)e->kcache + kv_layer * L.aidx, *vc = (KV *)e->vcache + kv_layer * L.aidx;
    cudaStream_t s = e->stream;
    prof_begin("attn_prep", s);
    RC_LAUNCH((k_attn_prep<KV>), dim3(nq + 2u * nkv, ntok), hd, hd * sizeof(float), s, e->qg, e->kraw, e->vraw, L.q_norm, L.k_norm, nq, nkv, hd, in.rope_dims, in.rope_freq_base,
                                                                 in.rms_eps, pos, e->query, e->gate, kc, vc);
    prof_end(s);
    const float scale = (float)(1.0 / sqrt((double)hd));
    {   // a chunk of tokens: the tiled tensor-core kernel (RC_ATTN_CHUNK=0 keeps the per-token kernel, for A/B runs)
        static const bool want = !(getenv("RC_ATTN_CHUNK") && atoi(getenv("RC_ATTN_CHUNK")) == 0);
        if (want && ntok >= 8u && attn_chunk_ok<KV>(hd, G)) {
            ENG_RC(launch_attn_chunk<KV>(e->query, kc, vc, nkv, G, hd, pos, ntok, scale, e->gate, e->gated, s));
            g_launches.fetch_add(1);
            return 1;
        }
    }
    uint32_t nsplit = (in.context + 31u) / 32u;                 // fixed per engine (graph replay): enough slices for a full context
    nsplit = nsplit < 1u ? 1u : nsplit > e->max_split ? e->max_split : nsplit;
    if (ntok > 1u && nsplit > e->pf_split) nsplit = e->pf_split;     // a chunk brings its own parallelism (and the partials are per token)
    const size_t smem = (size_t)(8u * G * hd + 16u * G) * sizeof(float);
    const dim3 grid(nkv, nsplit, ntok);
    prof_begin("attn_decode", s);
#define ENG_ATTN(VPL_, G_) do { \
        if (smem > 48u * 1024u) ENG_CUDA(cudaFuncSetAttribute(k_attn_decode<KV, VPL_, G_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        RC_LAUNCH((k_attn_decode<KV, VPL_, G_>), grid, 256, smem, s, e->query, kc, vc, nkv, pos, nsplit, scale, e->part_m, e->part_l, e->part_acc); } while (0)
    if (hd == 256u && G == 8u) ENG_ATTN(8, 8);
    else if (hd == 128u && G == 8u) ENG_ATTN(4, 8);
    else if (hd == 128u && G == 4u) ENG_ATTN(4, 4);
    else if (hd == 64u && G == 2u) ENG_ATTN(2, 2);
    else if (hd == 64u && G == 4u) ENG_ATTN(2, 4);
    else if (hd == 256u && G == 4u) ENG_ATTN(8, 4);
    else ENG_FAIL("attention shape head_dim %u with %u query heads per KV head is not built", hd, G);
#undef ENG_ATTN
    prof_end(s);
    prof_begin("attn_merge", s);
    RC_LAUNCH((k_attn_merge), dim3(nq, ntok), hd, 0, s, e->part_m, e->part_l, e->part_acc, e->gate, nsplit, hd, e->gated);
    prof_end(s);
    g_launches.fetch_add(3);
    ENG_CUDA(cudaGetLastError());
    return 1;
}

// One token on the device; the token id is already in e->token_d. want_logits: run the LM head.
static int eng_step_device(rl_engine *e, bool want_logits, char *error, size_t cap) {
    const rl_engine_info &in = e->info;
    cudaStream_t s = e->stream;
    if (e->ep_world > 1 && !e->ep) ENG_FAIL("this engine holds an expert shard: attach the exchange context first (redcuda_engine_attach_ep)");
    if (e->position >= in.context) ENG_FAIL("context of %u positions is full", in.context);
    prof_begin("embed", s);
    RC_LAUNCH((k_embed_row), 1, 256, 0, s, e->tok_embd.base, e->tok_embd.type, e->tok_embd.nb, in.hidden, in.vocab, e->token_d, books_iq2(), books_iq3s(), e->embed_d, status_words());
    prof_end(s);
    g_launches.fetch_add(1);
    const float *x = e->embed_d;
    const DnDims D{in.d_conv, in.d_state, in.n_group, in.dt_rank, in.d_inner, in.channels, in.rms_eps};
    for (uint32_t l = 0; l < in.n_layer; ++l) {
        const EngLayer &L = e->layers[l];
        prof_begin("rmsnorm", s);
        RC_LAUNCH((k_rmsnorm), 1, 1024, 0, s, x, nullptr, L.attn_norm, in.hidden, in.rms_eps, nullptr, e->normed);
        prof_end(s);
        g_launches.fetch_add(1);
        if (L.recurrent) {
            const DMat mats[3] = {L.qkv, L.z, L.ba};
            float *outs[3] = {e->qkv, e->z, e->ba};
            ENG_RC(eng_gemv(e, mats, outs, 3, e->normed, "dn_proj_gemv"));
            ENG_RC(launch_deltanet(D, 1u, L.conv_k, L.dt, L.a, L.ssm_norm, e->qkv, e->z, e->ba, e->conv + (size_t)L.ridx * (in.d_conv - 1u) * in.channels,
                                   e->rec + (size_t)L.ridx * in.dt_rank * in.d_state * in.d_state, e->dn_qk, e->dn_v, e->dn_beta, e->dn_gate, e->dn_core, e->ng, s));
            float *o1[1] = {e->branch};
            ENG_RC(eng_gemv(e, &L.ssm_out, o1, 1, e->ng, "dn_out_gemv"));
        } else {
            const DMat mats[3] = {L.q, L.k, L.v};
            float *outs[3] = {e->qg, e->kraw, e->vraw};
            ENG_RC(eng_gemv(e, mats, outs, 3, e->normed, "attn_proj_gemv"));
            if (e->kv_half) { if (!eng_attention<__half>(e, L, 1u, e->pos_d, error, cap)) return 0; }
            else { if (!eng_attention<float>(e, L, 1u, e->pos_d, error, cap)) return 0; }
            float *o1[1] = {e->branch};
            ENG_RC(eng_gemv(e, &L.o, o1, 1, e->gated, "attn_out_gemv"));
        }
        prof_begin("resid_rmsnorm", s);
        RC_LAUNCH((k_rmsnorm), 1, 1024, 0, s, x, e->branch, L.post_norm, in.hidden, in.rms_eps, e->resid, e->normed);
        prof_end(s);
        g_launches.fetch_add(1);
        float *xo = e->layer_out_d + (size_t)l * in.hidden;
        if (e->ep_world > 1) {
            ENG_RC(redcuda_ep_layer_forward_n(e->ep, L.moe, 1u, e->normed, nullptr, e->resid, xo, s));
            ENG_CUDA(cudaMemcpyAsync(e->router_ids_d + (size_t)l * RL_ENGINE_MAX_TOPK, redcuda_ep_last_ids_device(e->ep), in.top_k * sizeof(uint32_t), cudaMemcpyDeviceToDevice, s));
        } else
        ENG_RC(redcuda_moe_forward_device(L.moe, 1u, e->normed, nullptr, e->resid, xo, s));      // its router kernel also fills router_ids_d (mirror set at open)
        if (e->ep_world == 1 && in.n_expert > 1024u) ENG_CUDA(cudaMemcpyAsync(e->router_ids_d + (size_t)l * RL_ENGINE_MAX_TOPK, moe_last_ids_device(L.moe), in.top_k * sizeof(uint32_t), cudaMemcpyDeviceToDevice, s));
        x = xo;
    }
    prof_begin("rmsnorm", s);
    RC_LAUNCH((k_rmsnorm), 1, 1024, 0, s, x, nullptr, e->output_norm, in.hidden, in.rms_eps, nullptr, e->final_norm_d);
    prof_end(s);
    g_launches.fetch_add(1);
    if (want_logits) {
        float *o1[1] = {e->logits_d};
        ENG_RC(eng_gemv(e, &e->output, o1, 1, e->final_norm_d, "lm_head_gemv"));
    }
    RC_LAUNCH((k_advance), 1, 32, 0, s, e->pos_d);
    g_launches.fetch_add(1);
    ENG_CUDA(cudaGetLastError());
    e->position++;
    return 1;
}

// Projections of a chunk. From 8 tokens on, block-quantised matrices run on the tcgen05 GEMM (the matrices of one call
// share the input, so its fp16 digits are prepared once and one launch covers them all); below that, or with
// RL_PREFILL_TC=0, Q6_K matrices with >= 3 tokens take the mma.sync kernel on int8 digit planes and the rest the GEMV.
static int eng_proj(rl_engine *e, const DMat *mats, float *const *outs, uint32_t n, const float *x, uint32_t ntok, const char *tag) {
    static const bool want_mma = !(getenv("RC_MOE_PATH") && getenv("RC_MOE_PATH")[0] == 'c');
    static const bool want_tc = !(getenv("RL_PREFILL_TC") && atoi(getenv("RL_PREFILL_TC")) == 0);
    bool all_quant = true;
    for (uint32_t i = 0; i < n; ++i) all_quant = all_quant && rc_is_quant(mats[i].type) && mats[i].ncols == mats[0].ncols;
    if (want_tc && all_quant && ntok >= 8u && n <= TC_MAX_JOBS && mats[0].ncols % 256u == 0) {
        uint32_t row_tiles = 0;
        for (uint32_t i = 0; i < n; ++i) row_tiles += tc_row_tiles(mats[i].nrows);
        const uint32_t tn = tc_token_tile(ntok, row_tiles);
        if (!launch_tc_prep_x(x, nullptr, mats[0].ncols, ntok, mats[0].ncols, tn, e->tc_xs, e->tc_xinv, e->stream)) return 0;
        TcArgs A{};
        A.njobs = n; A.ncols = mats[0].ncols; A.ntok = ntok; A.xs = e->tc_xs; A.x_inv = e->tc_xinv; A.err = e->tc_err;
        A.wd = e->tc_wd; A.w_inv = e->tc_winv;
        RC_REQUIRE(tc_wd_bytes(row_tiles, mats[0].ncols) <= e->tc_wd_cap, "projection group %s: %u row tiles x %u columns exceed the weight-digit scratch", tag, row_tiles, mats[0].ncols);
        for (uint32_t i = 0; i < n; ++i) A.job[i] = TcJob{mats[i].base, mats[i].nb, mats[i].type, mats[i].nrows, outs[i], mats[i].nrows, 0u};
        return launch_tc_gemm(A, tn, tag, e->stream);
    }
    GemvArgs A{};
    A.ntok = ntok; A.x = x; A.x_stride = mats[0].ncols; A.tag = tag;
    uint32_t j = 0;
    bool quantised = false;
    for (uint32_t i = 0; i < n; ++i) {
        const DMat &M = mats[i];
        if (want_mma && ntok >= 3u && M.type == RC_Q6_K && M.nrows % 16u == 0 && M.ncols % 256u == 0) {
            if (!quantised) { if (!launch_quant_act(x, M.ncols, ntok, M.ncols, e->xq, e->sx, e->stream)) return 0; quantised = true; }
            if (!launch_q6k_mma(M.base, nullptr, M.nb, M.nrows, M.ncols, ntok, e->xq, e->sx, outs[i], M.nrows, tag, e->stream)) return 0;
            continue;
        }
        GemvJob &J = A.job[j++];
        J.w0 = M.base; J.w1 = nullptr; J.out = outs[i]; J.nb = M.nb; J.type = M.type; J.nrows = M.nrows; J.ncols = M.ncols; J.out_stride = M.nrows; J.epi = GEMV_STORE;
    }
    if (!j) return 1;
    A.njobs = j;
    return launch_gemv(A, e->stream);
}

// A chunk of n consecutive tokens (ids in e->tok_chunk_d, positions in e->pos_chunk_d) through every layer at once:
// projections, router and experts see the n tokens as a batch (each weight byte is read once per chunk); the DeltaNet
// recurrence runs over the tokens inside one kernel with the state in registers; attention appends the chunk's K/V
// rows and masks by position. The mirrors are left holding the last token's rows, as after n single steps
// (the reference's chunked prefill, native/redlite_native_engine.c:600-640).
static int eng_prefill_chunk(rl_engine *e, uint32_t n, bool want_logits, char *error, size_t cap) {
    if (e->ep_world > 1 && !e->ep) ENG_FAIL("this engine holds an expert shard: attach the exchange context first (redcuda_engine_attach_ep)");
    const rl_engine_info &in = e->info;
    cudaStream_t s = e->stream;
    if (e->position + n > in.context) ENG_FAIL("context of %u positions is full", in.context);
    const DnDims D{in.d_conv, in.d_state, in.n_group, in.dt_rank, in.d_inner, in.channels, in.rms_eps};
    const size_t last = (size_t)(n - 1u);
    prof_begin("embed", s);
    RC_LAUNCH((k_embed_row), n, 256, 0, s, e->tok_embd.base, e->tok_embd.type, e->tok_embd.nb, in.hidden, in.vocab, e->tok_chunk_d, books_iq2(), books_iq3s(), e->bx[0], status_words());
    prof_end(s);
    g_launches.fetch_add(1);
    ENG_CUDA(cudaMemcpyAsync(e->embed_d, e->bx[0] + last * in.hidden, in.hidden * 4u, cudaMemcpyDeviceToDevice, s));
    const float *x = e->bx[0];
    for (uint32_t l = 0; l < in.n_layer; ++l) {
        const EngLayer &L = e->layers[l];
        prof_begin("rmsnorm", s);
        RC_LAUNCH((k_rmsnorm), n, 1024, 0, s, x, nullptr, L.attn_norm, in.hidden, in.rms_eps, nullptr, e->normed);
        prof_end(s);
        g_launches.fetch_add(1);
        if (L.recurrent) {
            const DMat mats[3] = {L.qkv, L.z, L.ba};
            float *outs[3] = {e->qkv, e->z, e->ba};
            ENG_RC(eng_proj(e, mats, outs, 3, e->normed, n, "dn_proj"));
            ENG_RC(launch_deltanet_seq(D, n, L.conv_k, L.dt, L.a, L.ssm_norm, e->qkv, e->z, e->ba, e->conv + (size_t)L.ridx * (in.d_conv - 1u) * in.channels,
                                       e->rec + (size_t)L.ridx * in.dt_rank * in.d_state * in.d_state, e->dn_qk, e->dn_v, e->dn_beta, e->dn_gate, e->dn_core, e->ng, e->dn_pd, s));
            float *o1[1] = {e->branch};
            ENG_RC(eng_proj(e, &L.ssm_out, o1, 1, e->ng, n, "dn_out"));
        } else {
            const DMat mats[3] = {L.q, L.k, L.v};
            float *outs[3] = {e->qg, e->kraw, e->vraw};
            ENG_RC(eng_proj(e, mats, outs, 3, e->normed, n, "attn_proj"));
            if (e->kv_half) { if (!eng_attention<__half>(e, L, n, e->pos_chunk_d, error, cap)) return 0; }
            else { if (!eng_attention<float>(e, L, n, e->pos_chunk_d, error, cap)) return 0; }
            float *o1[1] = {e->branch};
            ENG_RC(eng_proj(e, &L.o, o1, 1, e->gated, n, "attn_out"));
        }
        prof_begin("resid_rmsnorm", s);
        RC_LAUNCH((k_rmsnorm), n, 1024, 0, s, x, e->branch, L.post_norm, in.hidden, in.rms_eps, e->resid, e->normed);
        prof_end(s);
        g_launches.fetch_add(1);
        float *xo = e->bx[(l + 1u) & 1u];
        if (e->ep_world > 1) ENG_RC(redcuda_ep_layer_forward_n(e->ep, L.moe, n, e->normed, nullptr, e->resid, xo, s));
        else ENG_RC(redcuda_moe_forward_device(L.moe, n, e->normed, nullptr, e->resid, xo, s));
        ENG_CUDA(cudaMemcpyAsync(e->router_ids_d + (size_t)l * RL_ENGINE_MAX_TOPK, (e->ep_world > 1 ? redcuda_ep_last_ids_device(e->ep) : moe_last_ids_device(L.moe)) + last * in.top_k, in.top_k * sizeof(uint32_t), cudaMemcpyDeviceToDevice, s));
        ENG_CUDA(cudaMemcpyAsync(e->layer_out_d + (size_t)l * in.hidden, xo + last * in.hidden, in.hidden * 4u, cudaMemcpyDeviceToDevice, s));
        x = xo;
    }
    prof_begin("rmsnorm", s);
    RC_LAUNCH((k_rmsnorm), 1, 1024, 0, s, x + last * in.hidden, nullptr, e->output_norm, in.hidden, in.rms_eps, nullptr, e->final_norm_d);
    prof_end(s);
    g_launches.fetch_add(1);
    if (want_logits) {
        float *o1[1] = {e->logits_d};
        ENG_RC(eng_gemv(e, &e->output, o1, 1, e->final_norm_d, "lm_head_gemv"));
    }
    ENG_CUDA(cudaGetLastError());
    e->position += n;
    return 1;
}

static int eng_set_position(rl_engine *e, uint32_t position, char *error, size_t cap) {
    ENG_CUDA(cudaStreamSynchronize(e->stream));
    e->token_pin[2] = position;
    ENG_CUDA(cudaMemcpyAsync(e->pos_d, e->token_pin + 2, 4, cudaMemcpyHostToDevice, e->stream));
    ENG_CUDA(cudaStreamSynchronize(e->stream));
    e->position = position;
    return 1;
}

static int eng_copy_mirrors(rl_engine *e, float *logits, char *error, size_t cap) {
    const rl_engine_info &in = e->info;
    cudaStream_t s = e->stream;
    ENG_CUDA(cudaMemcpyAsync(e->embed_h.data(), e->embed_d, in.hidden * 4u, cudaMemcpyDeviceToHost, s));
    ENG_CUDA(cudaMemcpyAsync(e->layer_out_h.data(), e->layer_out_d, (size_t)in.n_layer * in.hidden * 4u, cudaMemcpyDeviceToHost, s));
    ENG_CUDA(cudaMemcpyAsync(e->final_norm_h.data(), e->final_norm_d, in.hidden * 4u, cudaMemcpyDeviceToHost, s));
    ENG_CUDA(cudaMemcpyAsync(e->router_ids_h.data(), e->router_ids_d, (size_t)in.n_layer * RL_ENGINE_MAX_TOPK * 4u, cudaMemcpyDeviceToHost, s));
    if (logits) ENG_CUDA(cudaMemcpyAsync(logits, e->logits_d, (size_t)in.vocab * 4u, cudaMemcpyDeviceToHost, s));
    ENG_CUDA(cudaStreamSynchronize(s));
    if (status_failed()) ENG_FAIL("%s", redcuda_last_error());
    return 1;
}

static int eng_reset_state(rl_engine *e, char *error, size_t cap) {
    ENG_CUDA(cudaMemsetAsync(e->state.p, 0, e->state.bytes, e->stream));
    if (e->tc_err) ENG_CUDA(cudaMemsetAsync(e->tc_err, 0, 4, e->stream));
    ENG_CUDA(cudaStreamSynchronize(e->stream));
    return eng_set_position(e, 0u, error, cap);
}

// upload one dense GGUF matrix [ncols = shape[0], nrows = shape[1]] into the arena at *off
static int eng_upload(rl_engine *e, const GgufTensor *t, const char *name, uint8_t *arena, size_t *off, uint8_t *scratch, DMat *out, char *error, size_t cap) {
    if (!t) ENG_FAIL("missing tensor %s", name);
    if (t->n_dims != 2u || !t->bytes) ENG_FAIL("tensor %s has an unsupported type (%u) or rank (%u)", name, t->type, t->n_dims);
    const uint32_t ncols = (uint32_t)t->shape[0], nrows = (uint32_t)t->shape[1];
    uint8_t *dst = arena + *off;
    ENG_RC(upload_matrix(t->type, nrows, ncols, e->gguf.data(t), false, dst, scratch, e->stream));
    *out = DMat{dst, t->type, nrows, ncols, rc_is_quant(t->type) ? (uint64_t)nrows * (ncols / 256u) : 0u};
    *off += (t->bytes + 255u) / 256u * 256u;
    return 1;
}

static int eng_upload_f32(rl_engine *e, const GgufTensor *t, const char *name, uint64_t count, uint8_t *arena, size_t *off, const float **out, char *error, size_t cap) {
    if (!t) ENG_FAIL("missing tensor %s", name);
    uint64_t n = 1;
    for (uint32_t d = 0; d < t->n_dims; ++d) n *= t->shape[d];
    if (t->type != 0u || n != count) ENG_FAIL("tensor %s must be F32 with %llu values", name, (unsigned long long)count);
    ENG_CUDA(cudaMemcpyAsync(arena + *off, e->gguf.data(t), count * 4u, cudaMemcpyHostToDevice, e->stream));
    *out = (const float *)(arena + *off);
    *off += (count * 4u + 255u) / 256u * 256u;
    return 1;
}

static int eng_open(rl_engine *e, const char *path, char *error, size_t cap) {
    const double t_open = now_ms();
    if (!require_device()) ENG_FAIL("%s", redcuda_last_error());
    if (!e->gguf.open_file(path)) ENG_FAIL("%s", e->gguf.error.c_str());
    const GgufFile &g = e->gguf;
    if (g.architecture != "qwen3next") ENG_FAIL("GGUF architecture is not qwen3next");
    rl_engine_info &in = e->info;
    memset(&in, 0, sizeof(in));
    in.n_layer = g.u32("qwen3next.block_count"); in.hidden = g.u32("qwen3next.embedding_length"); in.vocab = (uint32_t)g.vocab;
    in.n_expert = g.u32("qwen3next.expert_count"); in.top_k = e->cfg.top_k ? e->cfg.top_k : g.u32("qwen3next.expert_used_count");
    in.context = e->cfg.context ? e->cfg.context : 4096u;
    in.d_conv = g.u32("qwen3next.ssm.conv_kernel"); in.d_inner = g.u32("qwen3next.ssm.inner_size"); in.d_state = g.u32("qwen3next.ssm.state_size");
    in.n_group = g.u32("qwen3next.ssm.group_count"); in.dt_rank = g.u32("qwen3next.ssm.time_step_rank");
    in.n_head = g.u32("qwen3next.attention.head_count"); in.n_head_kv = g.u32("qwen3next.attention.head_count_kv");
    in.head_dim = g.u32("qwen3next.attention.key_length"); in.rope_dims = g.u32("qwen3next.rope.dimension_count");
    in.rope_freq_base = g.f32("qwen3next.rope.freq_base"); in.rms_eps = g.f32("qwen3next.attention.layer_norm_rms_epsilon");
    e->ffn_sh = g.u32("qwen3next.expert_shared_feed_forward_length");
    // the same consistency checks as the reference applies (native/redlite_native_engine.c:213-243)
    if (!in.n_layer || !in.hidden || !in.n_head || !in.n_head_kv || !in.head_dim || !in.rope_dims || !in.n_expert || !in.top_k || in.d_conv < 2u ||
        !in.d_state || !in.n_group || !in.dt_rank || !in.d_inner || !e->ffn_sh || in.rms_eps <= 0.f || in.rope_freq_base <= 0.f ||
        in.head_dim != g.u32("qwen3next.attention.value_length") || in.n_head % in.n_head_kv || in.dt_rank % in.n_group || in.d_inner % in.dt_rank || !in.vocab)
        ENG_FAIL("incomplete or inconsistent qwen3next metadata");
    in.head_v = in.d_inner / in.dt_rank;
    in.channels = 2u * in.d_state * in.n_group + in.d_inner;
    if (in.head_v != in.d_state) ENG_FAIL("DeltaNet head_v != state size");
    if (in.top_k > RL_ENGINE_MAX_TOPK || in.top_k > in.n_expert) ENG_FAIL("top-k out of range");
    if (in.rope_dims > in.head_dim || in.rope_dims % 2u) ENG_FAIL("unsupported RoPE dims");
    if (in.head_dim > 1024u || in.head_dim % 32u) ENG_FAIL("unsupported head_dim %u", in.head_dim);
    {
        const char *v = getenv("RL_KV_F16");      // same switch as the reference (native/redlite_native_engine.c:43-47)
        e->kv_half = v && atoi(v) != 0;
    }
    ENG_CUDA(cudaGetDevice(&e->device));
    ENG_CUDA(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
    // Prefill chunk: the reference defaults to 2048 tokens per batched dispatch (native/redlite_native_engine.h:37), and so
    // does this engine (2048 is also the ceiling). The chunk sizes the expert workspace (about 0.5 GB at 2048), which all
    // layers share: they run one after the other on the engine's stream. 1 = token by token.
    e->pb = e->cfg.prefill_batch ? std::min(e->cfg.prefill_batch, 2048u) : 2048u;
    e->ep_rank = g_shard_rank; e->ep_world = g_shard_world;
    if (e->ep_world > 1 && in.n_expert % (uint32_t)e->ep_world) ENG_FAIL("%u experts do not divide over %d ranks", in.n_expert, e->ep_world);
    if (e->pb > in.context) e->pb = in.context;

    // ---- layer kinds from tensor names (native/redlite_native_layer_map.c:114-124), sizes of the dense arena
    e->layers.resize(in.n_layer);
    size_t dense_total = 0, scratch_max = 0;
    auto account = [&](const GgufTensor *t) { if (t) { dense_total += (t->bytes + 255u) / 256u * 256u + 256u; if (t->bytes > scratch_max) scratch_max = t->bytes; } };
    const char *rec_names[] = {"attn_qkv.weight", "attn_gate.weight", "ssm_ba.weight", "ssm_conv1d.weight", "ssm_dt.bias", "ssm_a", "ssm_norm.weight", "ssm_out.weight"};
    const char *att_names[] = {"attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_q_norm.weight", "attn_k_norm.weight", "attn_output.weight"};
    const char *common[] = {"attn_norm.weight", "post_attention_norm.weight", "ffn_gate_inp.weight", "ffn_gate_inp_shexp.weight"};
    for (uint32_t l = 0; l < in.n_layer; ++l) {
        bool rec = false, att = false;
        for (const char *n : rec_names) { const GgufTensor *t = g.find_layer(l, n); if (t) { rec = true; account(t); } }
        for (const char *n : att_names) { const GgufTensor *t = g.find_layer(l, n); if (t) { att = true; account(t); } }
        for (const char *n : common) account(g.find_layer(l, n));
        if (rec == att) ENG_FAIL("layer %u has an unknown/mixed structure", l);
        e->layers[l].recurrent = rec;
        if (rec) e->layers[l].ridx = in.n_recurrent++; else e->layers[l].aidx = in.n_attention++;
    }
    const GgufTensor *t_embd = g.find("token_embd.weight"), *t_onorm = g.find("output_norm.weight"), *t_out = g.find("output.weight");
    if (!t_out) t_out = t_embd;      // tied embeddings (native/redlite_native_engine.c:253)
    account(t_embd); account(t_onorm); if (t_out != t_embd) account(t_out);
    if (!e->dense.alloc(dense_total + 4096u)) ENG_FAIL("%s", redcuda_last_error());
    DevMem up_scratch;
    if (!up_scratch.alloc(scratch_max + 256u)) ENG_FAIL("%s", redcuda_last_error());
    uint8_t *arena = e->dense.as<uint8_t>(), *sc = up_scratch.as<uint8_t>();
    size_t off = 0;
    if (!eng_upload(e, t_embd, "token_embd.weight", arena, &off, sc, &e->tok_embd, error, cap)) return 0;
    if (e->tok_embd.ncols != in.hidden || e->tok_embd.nrows != in.vocab) ENG_FAIL("token_embd.weight shape does not match (hidden, vocab)");
    if (t_out != t_embd) { if (!eng_upload(e, t_out, "output.weight", arena, &off, sc, &e->output, error, cap)) return 0; }
    else e->output = e->tok_embd;
    if (e->output.ncols != in.hidden || e->output.nrows != in.vocab) ENG_FAIL("output.weight shape does not match (hidden, vocab)");
    if (!eng_upload_f32(e, t_onorm, "output_norm.weight", in.hidden, arena, &off, &e->output_norm, error, cap)) return 0;
    in.dense_bytes = 0;

    for (uint32_t l = 0; l < in.n_layer; ++l) {
        EngLayer &L = e->layers[l];
        auto T = [&](const char *n) { return g.find_layer(l, n); };
        if (!eng_upload_f32(e, T("attn_norm.weight"), "attn_norm", in.hidden, arena, &off, &L.attn_norm, error, cap) ||
            !eng_upload_f32(e, T("post_attention_norm.weight"), "post_attention_norm", in.hidden, arena, &off, &L.post_norm, error, cap)) return 0;
        if (L.recurrent) {
            if (!eng_upload(e, T("attn_qkv.weight"), "attn_qkv", arena, &off, sc, &L.qkv, error, cap) || !eng_upload(e, T("attn_gate.weight"), "attn_gate", arena, &off, sc, &L.z, error, cap) ||
                !eng_upload(e, T("ssm_ba.weight"), "ssm_ba", arena, &off, sc, &L.ba, error, cap) || !eng_upload(e, T("ssm_out.weight"), "ssm_out", arena, &off, sc, &L.ssm_out, error, cap) ||
                !eng_upload_f32(e, T("ssm_conv1d.weight"), "ssm_conv1d", (uint64_t)in.d_conv * in.channels, arena, &off, &L.conv_k, error, cap) ||
                !eng_upload_f32(e, T("ssm_dt.bias"), "ssm_dt", in.dt_rank, arena, &off, &L.dt, error, cap) || !eng_upload_f32(e, T("ssm_a"), "ssm_a", in.dt_rank, arena, &off, &L.a, error, cap) ||
                !eng_upload_f32(e, T("ssm_norm.weight"), "ssm_norm", in.head_v, arena, &off, &L.ssm_norm, error, cap)) return 0;
            if (L.qkv.ncols != in.hidden || L.qkv.nrows != in.channels || L.z.nrows != in.d_inner || L.ba.nrows != 2u * in.dt_rank || L.ssm_out.ncols != in.d_inner || L.ssm_out.nrows != in.hidden)
                ENG_FAIL("layer %u: DeltaNet tensor shapes do not match the metadata", l);
            e->dense_step_bytes += rc_matrix_bytes(L.qkv.type, L.qkv.nrows, L.qkv.ncols) + rc_matrix_bytes(L.z.type, L.z.nrows, L.z.ncols) +
                                   rc_matrix_bytes(L.ba.type, L.ba.nrows, L.ba.ncols) + rc_matrix_bytes(L.ssm_out.type, L.ssm_out.nrows, L.ssm_out.ncols);
        } else {
            const uint32_t qc = in.n_head * in.head_dim, kvc = in.n_head_kv * in.head_dim;
            if (!eng_upload(e, T("attn_q.weight"), "attn_q", arena, &off, sc, &L.q, error, cap) || !eng_upload(e, T("attn_k.weight"), "attn_k", arena, &off, sc, &L.k, error, cap) ||
                !eng_upload(e, T("attn_v.weight"), "attn_v", arena, &off, sc, &L.v, error, cap) || !eng_upload(e, T("attn_output.weight"), "attn_output", arena, &off, sc, &L.o, error, cap) ||
                !eng_upload_f32(e, T("attn_q_norm.weight"), "attn_q_norm", in.head_dim, arena, &off, &L.q_norm, error, cap) ||
                !eng_upload_f32(e, T("attn_k_norm.weight"), "attn_k_norm", in.head_dim, arena, &off, &L.k_norm, error, cap)) return 0;
            if (L.q.nrows != 2u * qc || L.k.nrows != kvc || L.v.nrows != kvc || L.o.ncols != qc || L.o.nrows != in.hidden) ENG_FAIL("layer %u: attention tensor shapes do not match the metadata", l);
            e->dense_step_bytes += rc_matrix_bytes(L.q.type, L.q.nrows, L.q.ncols) + 2u * rc_matrix_bytes(L.k.type, L.k.nrows, L.k.ncols) + rc_matrix_bytes(L.o.type, L.o.nrows, L.o.ncols);
        }
        // ---- MoE: router, shared expert, every routed expert of the layer
        const GgufTensor *tr = T("ffn_gate_inp.weight"), *tg = T("ffn_gate_inp_shexp.weight"), *sg = T("ffn_gate_shexp.weight"), *su = T("ffn_up_shexp.weight"),
                         *sd = T("ffn_down_shexp.weight"), *ge = T("ffn_gate_exps.weight"), *ue = T("ffn_up_exps.weight"), *de = T("ffn_down_exps.weight");
        if (!tr || !tg || !sg || !su || !sd || !ge || !ue || !de) ENG_FAIL("layer %u: missing MoE tensor", l);
        if (tr->type != 0u || tg->type != 0u || ge->n_dims != 3u || ue->n_dims != 3u || de->n_dims != 3u || ge->shape[2] != in.n_expert || de->shape[2] != in.n_expert ||
            ge->shape[0] != in.hidden || de->shape[1] != in.hidden || ge->type != ue->type || sg->type != su->type || sg->type != sd->type || !ge->bytes || !de->bytes || !sg->bytes)
            ENG_FAIL("layer %u: MoE tensor types or shapes are not supported", l);
        redcuda_moe_desc d;
        memset(&d, 0, sizeof(d));
        d.hidden = in.hidden; d.n_expert = in.n_expert; d.top_k = in.top_k; d.ffn = (uint32_t)ge->shape[1]; d.ffn_sh = (uint32_t)sg->shape[1];
        d.type_gu = ge->type; d.type_down = de->type; d.type_sh = sg->type; d.weights_on_device = 0;
        // under expert parallelism the engine holds a contiguous share of the experts and sees the tokens of every rank
        const uint32_t ec = in.n_expert / (uint32_t)e->ep_world, eb = (uint32_t)e->ep_rank * ec;
        d.expert_begin = eb; d.expert_count = ec; d.max_tokens = e->pb * (uint32_t)e->ep_world;
        d.router = (const float *)g.data(tr);
        d.gate_exps = g.data(ge) + (size_t)eb * (ge->bytes / in.n_expert); d.up_exps = g.data(ue) + (size_t)eb * (ue->bytes / in.n_expert);
        d.down_exps = g.data(de) + (size_t)eb * (de->bytes / in.n_expert);
        d.sh_gate_inp = (const float *)g.data(tg); d.sh_gate = g.data(sg); d.sh_up = g.data(su); d.sh_down = g.data(sd);
        e->ffn = d.ffn;
        {
            const size_t need = moe_workspace_bytes(&d);
            if (!e->moe_ws.p && !e->moe_ws.alloc(need)) ENG_FAIL("%s", redcuda_last_error());
            L.moe = need <= e->moe_ws.bytes ? moe_create_shared(&d, e->moe_ws.p) : redcuda_moe_create(&d);
        }
        if (!L.moe) ENG_FAIL("layer %u: %s", l, redcuda_last_error());
        e->expert_bytes += ge->bytes + ue->bytes + de->bytes;
        e->dense_step_bytes += tr->bytes + tg->bytes + sg->bytes + su->bytes + sd->bytes;
    }
    e->dense_step_bytes += rc_matrix_bytes(e->output.type, e->output.nrows, e->output.ncols);
    in.dense_bytes = off;
    ENG_CUDA(cudaStreamSynchronize(e->stream));
    up_scratch.release();

    // ---- state: conv windows, recurrent states, KV cache (one allocation so that reset is one memset)
    const size_t conv_b = (size_t)(in.d_conv - 1u) * in.channels * in.n_recurrent * 4u, rec_b = (size_t)in.dt_rank * in.d_state * in.d_state * in.n_recurrent * 4u;
    const size_t kv_b = (size_t)in.context * in.n_head_kv * in.head_dim * in.n_attention * (e->kv_half ? 2u : 4u);
    const size_t o_conv = 0, o_rec = (conv_b + 255u) / 256u * 256u, o_k = o_rec + (rec_b + 255u) / 256u * 256u, o_v = o_k + (kv_b + 255u) / 256u * 256u;
    if (!e->state.alloc(o_v + kv_b + 256u)) ENG_FAIL("%s", redcuda_last_error());
    uint8_t *S = e->state.as<uint8_t>();
    e->conv = (float *)(S + o_conv); e->rec = (float *)(S + o_rec); e->kcache = S + o_k; e->vcache = S + o_v;
    in.state_bytes = conv_b + rec_b + 2u * kv_b;

    // ---- scratch
    size_t w = 0;
    auto take = [&](size_t bytes) { const size_t o = w; w = (w + bytes + 255u) / 256u * 256u; return o; };
    const uint32_t qc = in.n_head * in.head_dim, kvc = in.n_head_kv * in.head_dim;
    const size_t T = e->pb;          // rows of every per-token buffer (decode uses row 0)
    const size_t parts = std::max<size_t>(e->max_split, T * e->pf_split);
    const uint32_t widest = std::max(std::max(in.hidden, in.d_inner), qc);
    // weight digits of the widest projection group that the tcgen05 GEMM may be given (4 bytes per weight, rows in tiles of 128)
    size_t wd_bytes = 0, wd_tiles = 0;
    for (uint32_t l = 0; l < in.n_layer; ++l) {
        const EngLayer &L = e->layers[l];
        const DMat *groups[2][3] = {{L.recurrent ? &L.qkv : &L.q, L.recurrent ? &L.z : &L.k, L.recurrent ? &L.ba : &L.v}, {L.recurrent ? &L.ssm_out : &L.o, nullptr, nullptr}};
        for (auto &g : groups) {
            uint32_t tiles = 0;
            for (const DMat *m : g) if (m) tiles += tc_row_tiles(m->nrows);
            wd_bytes = std::max(wd_bytes, tc_wd_bytes(tiles, g[0]->ncols));
            wd_tiles = std::max<size_t>(wd_tiles, tiles);
        }
    }
    const size_t o_twd = take(wd_bytes), o_twi = take(wd_tiles * 4u);
    const size_t o_norm = take(T * in.hidden * 4u), o_br = take(T * in.hidden * 4u), o_res = take(T * in.hidden * 4u), o_qkv = take(T * in.channels * 4u), o_z = take(T * in.d_inner * 4u),
                 o_ba = take(T * 2u * in.dt_rank * 4u), o_ng = take(T * in.d_inner * 4u), o_dqk = take(T * 2u * in.n_group * in.d_state * 4u), o_dv = take(T * in.d_inner * 4u),
                 o_db = take(T * in.dt_rank * 4u), o_dg = take(T * in.dt_rank * 4u), o_dc = take(T * in.d_inner * 4u), o_qg = take(T * 2u * qc * 4u), o_kr = take(T * kvc * 4u), o_vr = take(T * kvc * 4u),
                 o_qu = take(T * qc * 4u), o_ga = take(T * qc * 4u), o_gd = take(T * qc * 4u), o_pm = take((size_t)in.n_head * parts * 4u), o_pl = take((size_t)in.n_head * parts * 4u),
                 o_pa = take((size_t)in.n_head * parts * in.head_dim * 4u), o_em = take(in.hidden * 4u), o_lo = take((size_t)in.n_layer * in.hidden * 4u),
                 o_fn = take(in.hidden * 4u), o_lg = take((size_t)in.vocab * 4u), o_ri = take((size_t)in.n_layer * RL_ENGINE_MAX_TOPK * 4u), o_tk = take(16), o_gt = take(4096u * 4u),
                 o_bx0 = take(T * in.hidden * 4u), o_bx1 = take(T * in.hidden * 4u), o_xq = take(T * 3u * widest), o_sx = take(T * 4u), o_tc = take(T * 4u), o_pc = take(T * 4u),
                 o_txs = take(tc_xs_halves((uint32_t)T, widest, 128u) * 2u), o_txi = take((T + 128u) * 4u), o_ter = take(16),
                 o_pd = take((T + 4u) * in.n_group * 4u * 4u);
    if (!e->scratch.alloc(w)) ENG_FAIL("%s", redcuda_last_error());
    uint8_t *B = e->scratch.as<uint8_t>();
    ENG_CUDA(cudaMemsetAsync(B, 0, w, e->stream));
    e->normed = (float *)(B + o_norm); e->branch = (float *)(B + o_br); e->resid = (float *)(B + o_res); e->qkv = (float *)(B + o_qkv); e->z = (float *)(B + o_z);
    e->ba = (float *)(B + o_ba); e->ng = (float *)(B + o_ng); e->dn_qk = (float *)(B + o_dqk); e->dn_v = (float *)(B + o_dv); e->dn_beta = (float *)(B + o_db);
    e->dn_gate = (float *)(B + o_dg); e->dn_core = (float *)(B + o_dc); e->qg = (float *)(B + o_qg); e->kraw = (float *)(B + o_kr); e->vraw = (float *)(B + o_vr);
    e->query = (float *)(B + o_qu); e->gate = (float *)(B + o_ga); e->gated = (float *)(B + o_gd); e->part_m = (float *)(B + o_pm); e->part_l = (float *)(B + o_pl);
    e->part_acc = (float *)(B + o_pa); e->embed_d = (float *)(B + o_em); e->layer_out_d = (float *)(B + o_lo); e->final_norm_d = (float *)(B + o_fn);
    e->logits_d = (float *)(B + o_lg); e->router_ids_d = (uint32_t *)(B + o_ri); e->token_d = (uint32_t *)(B + o_tk); e->gen_tokens_d = (uint32_t *)(B + o_gt);
    e->pos_d = e->token_d + 2; e->gen_count_d = e->token_d + 3;
    e->bx[0] = (float *)(B + o_bx0); e->bx[1] = (float *)(B + o_bx1); e->xq = (int8_t *)(B + o_xq); e->sx = (float *)(B + o_sx);
    e->tok_chunk_d = (uint32_t *)(B + o_tc); e->pos_chunk_d = (uint32_t *)(B + o_pc);
    for (uint32_t l = 0; l < in.n_layer; ++l) moe_set_ids_mirror(e->layers[l].moe, e->router_ids_d + (size_t)l * RL_ENGINE_MAX_TOPK);
    e->tc_xs = (__half *)(B + o_txs); e->tc_xinv = (float *)(B + o_txi); e->tc_err = (uint32_t *)(B + o_ter);
    e->dn_pd = (float *)(B + o_pd);
    e->tc_wd = B + o_twd; e->tc_winv = (float *)(B + o_twi); e->tc_wd_cap = wd_bytes;
    e->embed_h.assign(in.hidden, 0.f); e->layer_out_h.assign((size_t)in.n_layer * in.hidden, 0.f); e->final_norm_h.assign(in.hidden, 0.f);
    e->router_ids_h.assign((size_t)in.n_layer * RL_ENGINE_MAX_TOPK, 0u);
    ENG_CUDA(cudaMallocHost((void **)&e->token_pin, 64u + 2u * T * 4u));      // [16 words][chunk tokens][chunk positions]
    if (!eng_reset_state(e, error, cap)) return 0;
    e->preload_ms = now_ms() - t_open;
    return 1;
}

extern "C" {

void rl_engine_config_default(rl_engine_config *cfg) {
    if (!cfg) return;
    memset(cfg, 0, sizeof(*cfg));
    cfg->context = 4096u; cfg->cache_mib = 4096u; cfg->enable_gpu = 1;
}

rl_engine *rl_engine_open(const char *model_path, const rl_engine_config *cfg, char *error, size_t cap) {
    if (!model_path) { eng_err(error, cap, "model path required"); return nullptr; }
    rl_engine *e = new (std::nothrow) rl_engine();
    if (!e) { eng_err(error, cap, "engine allocation failed"); return nullptr; }
    if (cfg) e->cfg = *cfg; else rl_engine_config_default(&e->cfg);
    if (e->cfg.enable_cpu) { eng_err(error, cap, "this library has no CPU backend (enable_cpu must be 0)"); delete e; return nullptr; }
    if (e->cfg.mtp_path && e->cfg.mtp_path[0]) { eng_err(error, cap, "multi-token prediction is not part of the CUDA backend"); delete e; return nullptr; }
    if (!eng_open(e, model_path, error, cap)) { rl_engine_close(e); return nullptr; }
    if (error && cap) error[0] = '\0';
    return e;
}

void rl_engine_close(rl_engine *e) {
    if (!e) return;
    if (e->stream) cudaStreamSynchronize(e->stream);
    if (e->graph_greedy) cudaGraphExecDestroy(e->graph_greedy);
    for (auto &L : e->layers) if (L.moe) redcuda_moe_destroy(L.moe);
    if (e->token_pin) cudaFreeHost(e->token_pin);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
}

const rl_engine_info *rl_engine_info_get(const rl_engine *e) { return e ? &e->info : nullptr; }

int rl_engine_reset(rl_engine *e, rl_engine_backend backend, char *error, size_t cap) {
    if (!e || backend != RL_BACKEND_GPU) { eng_err(error, cap, "backend not enabled"); return 0; }
    return eng_reset_state(e, error, cap);
}

uint32_t rl_engine_position(const rl_engine *e, rl_engine_backend backend) { return e && backend == RL_BACKEND_GPU ? e->position : 0u; }

int rl_engine_bench_set_position(rl_engine *e, rl_engine_backend backend, uint32_t position, char *error, size_t cap) {
    if (!e || backend != RL_BACKEND_GPU) { eng_err(error, cap, "backend not enabled"); return 0; }
    if (position >= e->info.context) { eng_err(error, cap, "position beyond the context"); return 0; }
    return eng_set_position(e, position, error, cap);
}

int rl_engine_step(rl_engine *e, rl_engine_backend backend, uint32_t token, float *logits, rl_engine_step_stats *stats, char *error, size_t cap) {
    if (!e) { eng_err(error, cap, "null engine"); return 0; }
    if (backend != RL_BACKEND_GPU) { eng_err(error, cap, "the CPU backend is not part of this library"); return 0; }
    if (token >= e->info.vocab) { eng_err(error, cap, "token id out of range"); return 0; }
    if (e->ep_world > 1) { eng_err(error, cap, "greedy generation on the device is not served under expert parallelism (the exchange's step counter cannot live in a replayed graph); use rl_engine_step"); return 0; }
    const double t0 = now_ms();
    if (stats) memset(stats, 0, sizeof(*stats));
    ENG_CUDA(cudaSetDevice(e->device));
    e->token_pin[0] = token;
    ENG_CUDA(cudaMemcpyAsync(e->token_d, e->token_pin, 4, cudaMemcpyHostToDevice, e->stream));
    if (!eng_step_device(e, logits != nullptr, error, cap)) return 0;
    if (!eng_copy_mirrors(e, logits, error, cap)) return 0;
    if (stats) { stats->total_ms = now_ms() - t0; stats->gpu_ms = stats->total_ms; stats->speculative = 1; stats->resident_slots = stats->slot_capacity = e->info.n_layer * e->info.n_expert; }
    if (error && cap) error[0] = '\0';
    return 1;
}

int rl_engine_prefill(rl_engine *e, rl_engine_backend backend, const uint32_t *tokens, uint32_t count, float *logits, rl_engine_step_stats *stats,
                      char *error, size_t cap) {
    // chunks of prefill_batch tokens (native/redlite_native_engine.c:600-640); a chunk of one token, and prefill_batch = 1,
    // take the single-token path. Only the last token runs the LM head.
    if (!e || !tokens || !count) { eng_err(error, cap, "invalid prefill arguments"); return 0; }
    if (backend != RL_BACKEND_GPU) { eng_err(error, cap, "the CPU backend is not part of this library"); return 0; }
    const double t0 = now_ms();
    if (stats) memset(stats, 0, sizeof(*stats));
    ENG_CUDA(cudaSetDevice(e->device));
    for (uint32_t i = 0; i < count; ++i) if (tokens[i] >= e->info.vocab) { eng_err(error, cap, "token id out of range"); return 0; }
    if (e->position + (uint64_t)count > e->info.context) { eng_err(error, cap, "prompt does not fit the context"); return 0; }
    uint32_t *tok_pin = e->token_pin + 16, *pos_pin = tok_pin + e->pb;
    ENG_CUDA(cudaMemsetAsync(e->tc_err, 0, 4, e->stream));     // a timeout of an earlier call must not fail this one
    for (uint32_t i = 0; i < count;) {
        const uint32_t n = std::min(e->pb, count - i);
        const bool last = i + n == count;
        ENG_CUDA(cudaStreamSynchronize(e->stream));      // the pinned staging words are reused
        if (n == 1u) {
            e->token_pin[0] = tokens[i];
            ENG_CUDA(cudaMemcpyAsync(e->token_d, e->token_pin, 4, cudaMemcpyHostToDevice, e->stream));
            if (!eng_step_device(e, logits != nullptr && last, error, cap)) return 0;
        } else {
            for (uint32_t t = 0; t < n; ++t) { tok_pin[t] = tokens[i + t]; pos_pin[t] = e->position + t; }
            e->token_pin[2] = e->position + n;
            ENG_CUDA(cudaMemcpyAsync(e->tok_chunk_d, tok_pin, n * 4u, cudaMemcpyHostToDevice, e->stream));
            ENG_CUDA(cudaMemcpyAsync(e->pos_chunk_d, pos_pin, n * 4u, cudaMemcpyHostToDevice, e->stream));
            if (!eng_prefill_chunk(e, n, logits != nullptr && last, error, cap)) return 0;
            ENG_CUDA(cudaMemcpyAsync(e->pos_d, e->token_pin + 2, 4, cudaMemcpyHostToDevice, e->stream));
        }
        i += n;
    }
    ENG_CUDA(cudaMemcpyAsync(e->token_pin + 3, e->tc_err, 4, cudaMemcpyDeviceToHost, e->stream));
    if (!eng_copy_mirrors(e, logits, error, cap)) return 0;
    if (e->token_pin[3]) ENG_FAIL("prefill: a tensor-core stage never signalled completion (bounded wait ran out); the engine state holds partial results: call rl_engine_reset before the next use");
    if (stats) { stats->total_ms = now_ms() - t0; stats->gpu_ms = stats->total_ms; }
    if (error && cap) error[0] = '\0';
    return 1;
}

uint32_t rl_engine_prefill_batch(const rl_engine *e) { return e ? e->pb : 0u; }

int redcuda_engine_shard(int rank, int world) {
    if (world < 1 || rank < 0 || rank >= world) { set_error("engine shard: rank %d of %d", rank, world); return 0; }
    g_shard_rank = rank; g_shard_world = world;
    return 1;
}

int redcuda_engine_attach_ep(rl_engine *e, redcuda_ep *ep) {
    if (!e || !ep) { set_error("engine attach: null argument"); return 0; }
    e->ep = ep;
    return 1;
}

int rl_engine_generate_greedy(rl_engine *e, uint32_t token, uint32_t n_new, uint32_t *out_tokens, rl_engine_step_stats *stats, char *error, size_t cap) {
    if (!e || !out_tokens || !n_new || n_new > 4096u) { eng_err(error, cap, "invalid generate arguments (1..4096 new tokens)"); return 0; }
    if (token >= e->info.vocab) { eng_err(error, cap, "token id out of range"); return 0; }
    const double t0 = now_ms();
    if (stats) memset(stats, 0, sizeof(*stats));
    ENG_CUDA(cudaSetDevice(e->device));
    e->token_pin[0] = token;
    ENG_CUDA(cudaMemcpyAsync(e->token_d, e->token_pin, 4, cudaMemcpyHostToDevice, e->stream));
    if (e->position + n_new > e->info.context) { eng_err(error, cap, "not enough context left for the requested tokens"); return 0; }
    ENG_CUDA(cudaMemsetAsync(e->gen_count_d, 0, 4, e->stream));
    auto one_token = [&]() -> int {
        if (!eng_step_device(e, true, error, cap)) return 0;
        RC_LAUNCH((k_argmax), 1, 1024, 0, e->stream, e->logits_d, e->info.vocab, e->token_d, e->gen_tokens_d, e->gen_count_d, status_words());
        g_launches.fetch_add(1);
        return 1;
    };
    for (uint32_t i = 0; i < n_new; ++i) {
        // The first token of an engine runs eagerly (it also sets every kernel attribute); then one token is captured
        // into a CUDA graph — position, token and output slot are read from device memory, so the same graph serves
        // every later token. RL_CUDA_GRAPH=0 keeps everything eager.
        static const bool want_graph = !(getenv("RL_CUDA_GRAPH") && atoi(getenv("RL_CUDA_GRAPH")) == 0);
        if (e->graph_greedy) {
            const uint64_t per_token = e->graph_launches;
            ENG_CUDA(cudaGraphLaunch(e->graph_greedy, e->stream));
            g_launches.fetch_add(per_token);
            e->position++;
            continue;
        }
        if (i >= 1u && want_graph && !e->graph_failed) {
            cudaGraph_t g = nullptr;
            const uint64_t before = g_launches.load();
            const uint32_t pos_before = e->position;
            bool ok = cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
            if (ok) {
                const int rc_ = one_token();
                const cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
                ok = rc_ && ce == cudaSuccess && g;
                e->position = pos_before;                     // capturing ran nothing
            }
            if (ok) ok = cudaGraphInstantiate(&e->graph_greedy, g, 0) == cudaSuccess;
            if (g) cudaGraphDestroy(g);
            if (!ok) { cudaGetLastError(); e->graph_failed = true; e->graph_greedy = nullptr; g_launches.store(before); }
            else { e->graph_launches = g_launches.load() - before; g_launches.store(before); --i; continue; }
        }
        if (!one_token()) return 0;
    }
    ENG_CUDA(cudaMemcpyAsync(out_tokens, e->gen_tokens_d, (size_t)n_new * 4u, cudaMemcpyDeviceToHost, e->stream));
    if (!eng_copy_mirrors(e, nullptr, error, cap)) return 0;
    if (stats) { stats->total_ms = now_ms() - t0; stats->gpu_ms = stats->total_ms; }
    if (error && cap) error[0] = '\0';
    return 1;
}

const float *rl_engine_last_embedding(const rl_engine *e, rl_engine_backend b) { return e && b == RL_BACKEND_GPU ? e->embed_h.data() : nullptr; }
const float *rl_engine_last_layer_output(const rl_engine *e, rl_engine_backend b, uint32_t layer) {
    return e && b == RL_BACKEND_GPU && layer < e->info.n_layer ? e->layer_out_h.data() + (size_t)layer * e->info.hidden : nullptr;
}
const float *rl_engine_last_final_norm(const rl_engine *e, rl_engine_backend b) { return e && b == RL_BACKEND_GPU ? e->final_norm_h.data() : nullptr; }
const uint32_t *rl_engine_last_router_ids(const rl_engine *e, rl_engine_backend b, uint32_t layer) {
    return e && b == RL_BACKEND_GPU && layer < e->info.n_layer ? e->router_ids_h.data() + (size_t)layer * RL_ENGINE_MAX_TOPK : nullptr;
}
int rl_engine_experts_preloaded(const rl_engine *e, double *preload_ms) { if (!e) return 0; if (preload_ms) *preload_ms = e->preload_ms; return 1; }
uint64_t rl_engine_full_residency_mib(const rl_engine *e) { return e ? (e->expert_bytes + (1u << 20) - 1u) >> 20 : 0u; }

int rl_engine_embed_token(const rl_engine *ce, uint32_t token, float *out, char *error, size_t cap) {
    rl_engine *e = const_cast<rl_engine *>(ce);
    if (!e || !out) { eng_err(error, cap, "invalid embed arguments"); return 0; }
    if (token >= e->info.vocab) { eng_err(error, cap, "token id out of range"); return 0; }
    ENG_CUDA(cudaStreamSynchronize(e->stream));
    e->token_pin[1] = token;
    ENG_CUDA(cudaMemcpyAsync(e->token_d + 1, e->token_pin + 1, 4, cudaMemcpyHostToDevice, e->stream));
    RC_LAUNCH((k_embed_row), 1, 256, 0, e->stream, e->tok_embd.base, e->tok_embd.type, e->tok_embd.nb, e->info.hidden, e->info.vocab, e->token_d + 1, books_iq2(), books_iq3s(), e->normed, status_words());
    g_launches.fetch_add(1);
    ENG_CUDA(cudaMemcpyAsync(out, e->normed, e->info.hidden * 4u, cudaMemcpyDeviceToHost, e->stream));
    ENG_CUDA(cudaStreamSynchronize(e->stream));
    return 1;
}

uint64_t rl_engine_step_bytes(const rl_engine *e) {
    if (!e) return 0;
    const rl_engine_info &in = e->info;
    const uint64_t per_expert = e->expert_bytes / ((uint64_t)in.n_layer * in.n_expert);
    const uint64_t states = 2ull * ((uint64_t)in.dt_rank * in.d_state * in.d_state + (uint64_t)(in.d_conv - 1u) * in.channels) * 4u * in.n_recurrent;
    const uint64_t kv = 2ull * (uint64_t)(e->position + 1u) * in.n_head_kv * in.head_dim * (e->kv_half ? 2u : 4u) * in.n_attention;
    return e->dense_step_bytes + per_expert * in.top_k * in.n_layer + states + kv + (uint64_t)in.hidden * rc_row_bytes(e->tok_embd.type, in.hidden) / in.hidden;
}

}  // extern "C"
