// Gated DeltaNet decode step between the projections (deltanet_branch, native/redlite_native_engine_cpu.c:148-230).
//
//   k_dn_prep   beta = sigmoid(b), gate = softplus(a + dt_bias) * A; causal depthwise conv over [conv state, new
//               sample] + SiLU; conv window shifted in place; q and k L2-normalised per key head (fp64 for the small
//               reductions, as the CPU path)
//   k_dn_state  the fp32 delta rule, one warp per state row: the row (d_state floats) is loaded once into the warp's
//               registers, decayed, corrected and read out, then stored — one read and one write of the state,
//               where the CPU path sweeps it four times
//   k_dn_tail   per value head RMSNorm(core) * w * SiLU(z)
#include "redcuda_common.cuh"
#include "redcuda_kernels.cuh"
#include "../../include/redcuda.h"

#include <stdlib.h>
#include <mutex>
#include <new>
#include <type_traits>

namespace rc {

__device__ __forceinline__ double sigmoid_stable(double x) { if (x >= 0.0) { const double z = exp(-x); return 1.0 / (1.0 + z); } const double z = exp(x); return z / (1.0 + z); }
__device__ __forceinline__ double softplus_stable(double x) { if (x > 20.0) return x; if (x < -20.0) return exp(x); return log1p(exp(x)); }

// grid.x = 2*groups (q/k heads) + d_inner/S (v runs) + 1 (beta/gate); grid.y = batch; block = S threads
__global__ void k_dn_prep(DnDims D, const float *__restrict__ conv_kernel, const float *__restrict__ dt_bias, const float *__restrict__ ssm_a,
                          const float *__restrict__ qkv, const float *__restrict__ ba, float *__restrict__ conv_state,
                          float *__restrict__ qk, float *__restrict__ v, float *__restrict__ beta, float *__restrict__ gate) {
    pdl_prologue();
    __shared__ double red[32];
    const uint32_t seq = blockIdx.y, tid = threadIdx.x, S = D.S, ns = D.d_conv - 1u;
    const uint32_t n_qk = 2u * D.groups, n_v = D.d_inner / S;
    if (blockIdx.x == n_qk + n_v) {   // beta / gate of every value head
        const uint32_t width = D.rank / D.groups, stride = 2u * width;
        for (uint32_t h = tid; h < D.rank; h += blockDim.x) {
            const uint32_t g = h / width, l = h - g * width;
            const float *b = ba + (size_t)seq * 2u * D.rank;
            beta[(size_t)seq * D.rank + h] = (float)sigmoid_stable((double)b[g * stride + l]);
            gate[(size_t)seq * D.rank + h] = (float)(softplus_stable((double)b[g * stride + width + l] + (double)dt_bias[h]) * (double)ssm_a[h]);
        }
        return;
    }
    const uint32_t c = blockIdx.x * S + tid;          // channel: q heads, then k heads, then v
    float *cs = conv_state + ((size_t)seq * D.channels + c) * ns;
    const float *kr = conv_kernel + (size_t)c * D.d_conv;
    const float xnew = qkv[(size_t)seq * D.channels + c];
    double acc = 0.0;
    for (uint32_t j = 0; j < ns; ++j) acc += (double)cs[j] * (double)kr[j];
    acc += (double)xnew * (double)kr[ns];
    for (uint32_t j = 0; j + 1u < ns; ++j) cs[j] = cs[j + 1u];
    cs[ns - 1u] = xnew;
    const float y = (float)(acc / (1.0 + exp(-acc)));
    if (blockIdx.x >= n_qk) { v[(size_t)seq * D.d_inner + (c - n_qk * S)] = y; return; }
    // L2 normalisation over the head (block)
    double ss = (double)y * (double)y;
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31u) == 0) red[tid >> 5] = ss;
    __syncthreads();
    double tot = 0.0;
    for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
    const double inv = 1.0 / fmax(sqrt(tot), (double)D.eps);
    qk[(size_t)seq * n_qk * S + c] = (float)((double)y * inv);
}

// one warp per (seq, value head, state row); VPL = S / 32 values per lane, element i = lane + 32 * v
template <int VPL>
__global__ void __launch_bounds__(256) k_dn_state(DnDims D, uint32_t batch, const float *__restrict__ qk, const float *__restrict__ v,
                                                  const float *__restrict__ beta, const float *__restrict__ gate,
                                                  float *__restrict__ state, float *__restrict__ core) {
    pdl_prologue();
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t gw = (blockIdx.x * (uint64_t)blockDim.x + threadIdx.x) >> 5;
    const uint32_t S = D.S;
    const uint64_t rows = (uint64_t)batch * D.rank * S;
    if (gw >= rows) return;
    const uint32_t j = (uint32_t)(gw % S), h = (uint32_t)((gw / S) % D.rank), seq = (uint32_t)(gw / ((uint64_t)S * D.rank));
    const uint32_t kh = h / (D.rank / D.groups);
    const float *q = qk + ((size_t)seq * 2u * D.groups + kh) * S;
    const float *k = qk + ((size_t)seq * 2u * D.groups + D.groups + kh) * S;
    float *row = state + (((size_t)seq * D.rank + h) * S + j) * S;
    const float decay = expf(gate[(size_t)seq * D.rank + h]);
    float m[VPL], kv[VPL];
    float sum = 0.f;
#pragma unroll
    for (int t = 0; t < VPL; ++t) { kv[t] = k[lane + 32 * t]; m[t] = row[lane + 32 * t] * decay; sum += m[t] * kv[t]; }
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float delta = (v[(size_t)seq * D.d_inner + (size_t)h * S + j] - sum) * beta[(size_t)seq * D.rank + h];
    float o_acc = 0.f;
#pragma unroll
    for (int t = 0; t < VPL; ++t) { m[t] += kv[t] * delta; o_acc += m[t] * q[lane + 32 * t]; row[lane + 32 * t] = m[t]; }
    for (int o = 16; o; o >>= 1) o_acc += __shfl_xor_sync(0xffffffffu, o_acc, o);
    if (lane == 0) core[(size_t)seq * D.d_inner + (size_t)h * S + j] = o_acc * (1.0f / sqrtf((float)S));
}

// grid (rank, batch), block S threads
__global__ void k_dn_tail(DnDims D, const float *__restrict__ core, const float *__restrict__ z, const float *__restrict__ norm_w, float *__restrict__ out) {
    pdl_prologue();
    __shared__ double red[32];
    const uint32_t h = blockIdx.x, seq = blockIdx.y, i = threadIdx.x, S = D.S;
    const size_t idx = (size_t)seq * D.d_inner + (size_t)h * S + i;
    const float x = core[idx], g = z[idx];
    double ss = (double)x * (double)x;
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((i & 31u) == 0) red[i >> 5] = ss;
    __syncthreads();
    double tot = 0.0;
    for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
    const float inv = 1.0f / sqrtf((float)(tot / (double)S) + D.eps);
    const float silu = g / (1.0f + expf(-g));
    out[idx] = x * inv * norm_w[i] * silu;
}

// Delta rule + gated RMSNorm of one value head in one block: grid (rank, batch), 8 warps, warp w owns the S / 8
// consecutive state rows w * S / 8 ... Every lane first requests ALL of its rows (S / 8 rows x VPL floats: 64 registers
// at S = 128), so a block has its whole 64 KB of state in flight at once — at batch 1 only `rank` blocks exist and each
// must cover the memory latency by itself — then the rows are decayed, corrected, read out and stored one after the
// other; q and k of the head are loaded once per lane instead of once per row. The head's S outputs meet in shared
// memory, where the tail (k_dn_tail's arithmetic, unchanged) normalises and gates them: one launch less, and the
// un-normalised outputs never travel through global memory.
template <int VPL>
__global__ void __launch_bounds__(256) k_dn_state_tail(DnDims D, const float *__restrict__ qk, const float *__restrict__ v,
                                                       const float *__restrict__ beta, const float *__restrict__ gate, float *__restrict__ state,
                                                       const float *__restrict__ z, const float *__restrict__ norm_w, float *__restrict__ out) {
    pdl_prologue();
    constexpr uint32_t S = VPL * 32u, RPW = S / 8u;
    __shared__ float s_core[S];
    __shared__ double red[8];
    const uint32_t h = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t kh = h / (D.rank / D.groups);
    const float *q = qk + ((size_t)seq * 2u * D.groups + kh) * S;
    const float *k = qk + ((size_t)seq * 2u * D.groups + D.groups + kh) * S;
    float *rows = state + (((size_t)seq * D.rank + h) * S + (size_t)warp * RPW) * S;
    float m[RPW][VPL];
    // volatile asm keeps these loads where they are written: all of them are issued before the first row is worked on
    // (left to itself the compiler fetches each row just before its use, with one row in flight per warp)
#pragma unroll
    for (uint32_t r = 0; r < RPW; ++r)
#pragma unroll
        for (int t = 0; t < VPL; ++t) asm volatile("ld.global.f32 %0, [%1];" : "=f"(m[r][t]) : "l"(rows + (size_t)r * S + lane + 32 * t));
    __syncwarp();                      // a fixed point between the requests above and the shuffles below
    float qv[VPL], kv[VPL];
#pragma unroll
    for (int t = 0; t < VPL; ++t) { qv[t] = q[lane + 32 * t]; kv[t] = k[lane + 32 * t]; }
    const float decay = expf(gate[(size_t)seq * D.rank + h]), bh = beta[(size_t)seq * D.rank + h], scale = 1.0f / sqrtf((float)S);
    const float *vh = v + (size_t)seq * D.d_inner + (size_t)h * S + warp * RPW;
#pragma unroll
    for (uint32_t r = 0; r < RPW; ++r) {
        float sum = 0.f;
#pragma unroll
        for (int t = 0; t < VPL; ++t) { m[r][t] = m[r][t] * decay; sum += m[r][t] * kv[t]; }
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float delta = (vh[r] - sum) * bh;
        float o_acc = 0.f;
#pragma unroll
        for (int t = 0; t < VPL; ++t) { m[r][t] += kv[t] * delta; o_acc += m[r][t] * qv[t]; rows[(size_t)r * S + lane + 32 * t] = m[r][t]; }
        for (int o = 16; o; o >>= 1) o_acc += __shfl_xor_sync(0xffffffffu, o_acc, o);
        if (lane == 0) s_core[warp * RPW + r] = o_acc * scale;
    }
    __syncthreads();
    // gated RMSNorm over the head (the arithmetic of k_dn_tail)
    const size_t idx = (size_t)seq * D.d_inner + (size_t)h * S + tid;
    float x = 0.f, g = 0.f;
    double ss = 0.0;
    if (tid < S) { x = s_core[tid]; g = z[idx]; ss = (double)x * (double)x; }
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (tid < S) {
        double tot = 0.0;
        for (uint32_t w = 0; w < S / 32u; ++w) tot += red[w];
        const float inv = 1.0f / sqrtf((float)(tot / (double)S) + D.eps);
        const float silu = g / (1.0f + expf(-g));
        out[idx] = x * inv * norm_w[tid] * silu;
    }
}

// ---- sequence form: T consecutive tokens of ONE sequence (a prefill chunk) ----
// k_dn_prep_seq   grid (2*groups + d_inner/S + 1, T / 8): token t's conv window is the d_conv-1 samples before it (the conv
//                 state for times before the chunk, chunk rows after); the state itself is rolled by k_dn_conv_roll
// k_dn_state_seq  the delta rule over the T tokens with the state row held in registers: one read and one write of
//                 the state per chunk instead of per token; the next token's q/k/v/beta/gate are fetched while the
//                 current one is reduced
// the tail kernel is k_dn_tail with the token as its batch index
// a block serves DN_PREP_TOK consecutive tokens of its channel group (one token per block left the kernel bound by block
// scheduling: 133,000 blocks of 128 threads for a 2048-token chunk)
constexpr uint32_t DN_PREP_TOK = 8u;
__global__ void k_dn_prep_seq(DnDims D, uint32_t T, const float *__restrict__ conv_kernel, const float *__restrict__ dt_bias, const float *__restrict__ ssm_a,
                              const float *__restrict__ qkv, const float *__restrict__ ba, const float *__restrict__ conv_state,
                              float *__restrict__ qk, float *__restrict__ v, float *__restrict__ beta, float *__restrict__ gate) {
    pdl_prologue();
    __shared__ double red[2][32];
    const uint32_t tid = threadIdx.x, S = D.S, ns = D.d_conv - 1u;
    const uint32_t n_qk = 2u * D.groups, n_v = D.d_inner / S;
    const uint32_t t_begin = blockIdx.y * DN_PREP_TOK, t_end = min(T, t_begin + DN_PREP_TOK);
    if (blockIdx.x == n_qk + n_v) {
        const uint32_t width = D.rank / D.groups, stride = 2u * width;
        for (uint32_t ti = t_begin; ti < t_end; ++ti)
            for (uint32_t h = tid; h < D.rank; h += blockDim.x) {
                const uint32_t g = h / width, l = h - g * width;
                const float *b = ba + (size_t)ti * 2u * D.rank;
                beta[(size_t)ti * D.rank + h] = (float)sigmoid_stable((double)b[g * stride + l]);
                gate[(size_t)ti * D.rank + h] = (float)(softplus_stable((double)b[g * stride + width + l] + (double)dt_bias[h]) * (double)ssm_a[h]);
            }
        return;
    }
    const uint32_t c = blockIdx.x * S + tid;
    const float *cs = conv_state + (size_t)c * ns;
    const float *kr = conv_kernel + (size_t)c * D.d_conv;
    for (uint32_t ti = t_begin; ti < t_end; ++ti) {
        double acc = 0.0;
        for (uint32_t j = 0; j < ns; ++j) {
            const int tau = (int)ti + (int)j - (int)ns;        // time of tap j relative to the chunk start
            const float smp = tau < 0 ? cs[(int)ns + tau] : qkv[(size_t)tau * D.channels + c];
            acc += (double)smp * (double)kr[j];
        }
        acc += (double)qkv[(size_t)ti * D.channels + c] * (double)kr[ns];
        const float y = (float)(acc / (1.0 + exp(-acc)));
        if (blockIdx.x >= n_qk) { v[(size_t)ti * D.d_inner + (c - n_qk * S)] = y; continue; }
        double ss = (double)y * (double)y;
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        double *rd = red[ti & 1u];                             // alternating buffers: one barrier per token
        if ((tid & 31u) == 0) rd[tid >> 5] = ss;
        __syncthreads();
        double tot = 0.0;
        for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) tot += rd[w];
        const double inv = 1.0 / fmax(sqrt(tot), (double)D.eps);
        qk[(size_t)ti * n_qk * S + c] = (float)((double)y * inv);
    }
}

// conv state <- the last d_conv-1 samples of [state, chunk]; one thread per channel
__global__ void k_dn_conv_roll(DnDims D, uint32_t T, const float *__restrict__ qkv, float *__restrict__ conv_state) {
    pdl_prologue();
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x, ns = D.d_conv - 1u;
    if (c >= D.channels) return;
    float *cs = conv_state + (size_t)c * ns;
    for (uint32_t j = 0; j < ns; ++j) {                     // ascending: a kept sample moves down, so its source is still intact
        const int tau = (int)T + (int)j - (int)ns;
        cs[j] = tau < 0 ? cs[(int)ns + tau] : qkv[(size_t)tau * D.channels + c];
    }
}

// Block = 8 warps = 8 consecutive state rows of ONE value head, so the eight warps need the same q / k rows and the same
// beta / gate of every token: they are staged in shared memory TB tokens at a time by cp.async, one token block ahead
// of the one being applied (a warp that fetched them itself waited for L2 on every token of its sequential chain).
constexpr uint32_t DN_TB = 8u;          // tokens per staged block
template <int VPL>
__global__ void __launch_bounds__(256) k_dn_state_seq(DnDims D, uint32_t T, const float *__restrict__ qk, const float *__restrict__ v,
                                                      const float *__restrict__ beta, const float *__restrict__ gate,
                                                      float *__restrict__ state, float *__restrict__ core) {
    pdl_prologue();
    constexpr uint32_t S = VPL * 32u;
    __shared__ __align__(16) float s_q[2][DN_TB][S], s_k[2][DN_TB][S];
    __shared__ __align__(16) float s_v[2][DN_TB][8];
    __shared__ float s_b[2][DN_TB], s_g[2][DN_TB];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t row0 = blockIdx.x * 8u;                       // first of the block's 8 rows, counted over (head, j)
    const uint32_t h = row0 / S, j0 = row0 - h * S, j = j0 + warp;
    const uint32_t kh = h / (D.rank / D.groups);
    const size_t tok_qk = (size_t)2u * D.groups * S;
    const float *q = qk + (size_t)kh * S, *k = qk + (size_t)(D.groups + kh) * S;
    float *row = state + ((size_t)h * S + j) * S;
    const float scale = 1.0f / sqrtf((float)S);

    auto stage = [&](uint32_t tb, uint32_t buf) {               // tokens [tb * DN_TB, ...) -> buffer buf
        const uint32_t t0 = tb * DN_TB, n = min(DN_TB, T - t0);
        constexpr uint32_t V4 = S / 4u;                          // float4 per q or k row
        for (uint32_t i = tid; i < 2u * n * V4; i += 256u) {
            const uint32_t which = i / (n * V4), r = i - which * n * V4, tt = r / V4, c = (r - tt * V4) * 4u;
            const float *src = (which ? k : q) + (size_t)(t0 + tt) * tok_qk + c;
            float *dst = (which ? &s_k[buf][tt][0] : &s_q[buf][tt][0]) + c;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
        }
        for (uint32_t i = tid; i < n * 2u; i += 256u) {          // v of the block's 8 rows: 32 bytes per token
            const uint32_t tt = i >> 1, c = (i & 1u) * 4u;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(&s_v[buf][tt][c])),
                         "l"(v + (size_t)(t0 + tt) * D.d_inner + (size_t)h * S + j0 + c) : "memory");
        }
        for (uint32_t i = tid; i < n * 2u; i += 256u) {
            const uint32_t tt = i >> 1;
            const float *src = (i & 1u ? gate : beta) + (size_t)(t0 + tt) * D.rank + h;
            float *dst = i & 1u ? &s_g[buf][tt] : &s_b[buf][tt];
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float m[VPL];
#pragma unroll
    for (int t = 0; t < VPL; ++t) m[t] = row[lane + 32 * t];
    const uint32_t nblk = (T + DN_TB - 1u) / DN_TB;
    stage(0u, 0u);
    for (uint32_t tb = 0; tb < nblk; ++tb) {
        const uint32_t buf = tb & 1u, n = min(DN_TB, T - tb * DN_TB);
        if (tb + 1u < nblk) stage(tb + 1u, buf ^ 1u); else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();                                         // block tb has landed for every warp
        // Off the token-to-token dependency chain: the block's eight decays are computed once (lane l holds token l % 8's) and
        // the output dot products are only reduced after the eight tokens, all together.
        const float dec_l = expf(s_g[buf][lane & (DN_TB - 1u)]);
        float op[DN_TB];
#pragma unroll
        for (uint32_t tt = 0; tt < DN_TB; ++tt) {
            op[tt] = 0.f;
            if (tt < n) {
                const float decay = __shfl_sync(0xffffffffu, dec_l, (int)tt);
                float kc[VPL];
                float sum = 0.f;
#pragma unroll
                for (int t = 0; t < VPL; ++t) { kc[t] = s_k[buf][tt][lane + 32 * t]; m[t] = m[t] * decay; sum += m[t] * kc[t]; }
                for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                const float delta = (s_v[buf][tt][warp] - sum) * s_b[buf][tt];
                float o_acc = 0.f;
#pragma unroll
                for (int t = 0; t < VPL; ++t) { m[t] += kc[t] * delta; o_acc += m[t] * s_q[buf][tt][lane + 32 * t]; }
                op[tt] = o_acc;
            }
        }
        {   // eight sums across the warp with the pairing of the plain butterfly (16, 8, 4, 2, 1), but each exchange halves the
            // values a lane carries: 4 + 2 + 1 + 1 + 1 shuffles instead of 8 x 5. Value i ends up in the lanes whose bits 4, 3, 2 spell i.
            const bool hi4 = lane & 16u, hi3 = lane & 8u, hi2 = lane & 4u;
            float a4[4], a2[2], a1;
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float keep = hi4 ? op[4 + i] : op[i], send = hi4 ? op[i] : op[4 + i]; a4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16); }
#pragma unroll
            for (int i = 0; i < 2; ++i) { const float keep = hi3 ? a4[2 + i] : a4[i], send = hi3 ? a4[i] : a4[2 + i]; a2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8); }
            { const float keep = hi2 ? a2[1] : a2[0], send = hi2 ? a2[0] : a2[1]; a1 = keep + __shfl_xor_sync(0xffffffffu, send, 4); }
            a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
            a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
            const uint32_t ti = ((lane >> 4) & 1u) * 4u + ((lane >> 3) & 1u) * 2u + ((lane >> 2) & 1u);
            if ((lane & 3u) == 0u && ti < n) core[(size_t)(tb * DN_TB + ti) * D.d_inner + (size_t)h * S + j] = a1 * scale;
        }
        __syncthreads();                                         // buffer buf may be refilled by the next stage() call
    }
#pragma unroll
    for (int t = 0; t < VPL; ++t) row[lane + 32 * t] = m[t];
}

// ---- the same token-by-token recurrence with a lane group per row (the default scan) -----------------------------------
// k_dn_state_seq spreads ONE row over the 32 lanes of a warp: per token a warp issues about 50 instructions for 4 x 128
// multiply-adds, ten of them the two five-step reductions, and every SM carries 32 such warps. Here LPR = S / CPT lanes
// share a row (CPT columns each, as float4 pieces interleaved over the lanes so that a quarter warp reads 128 contiguous
// bytes of k or q), a thread carries RPT rows (k and q, read from shared memory once, serve all of them: the shared-memory
// pipe delivers 128 bytes per cycle whether or not lanes read the same address, and with one row per thread it was busier
// than the fp32 pipe), the row's partial sums meet in ONE exchange step, and the arithmetic is packed fp32 (two columns
// per instruction). Per element it is the reference's (decay the row, dot with k, add k * delta, dot with q:
// native/redlite_native_engine_cpu.c:198-216); only the order of the sums inside a dot product differs. Whole blocks of
// eight tokens run through a branch-free unrolled body; the block's decays, betas and v are fetched before its first
// token, a token's q and the next token's k before the exchange that the chain waits for, and the eight output sums are
// reduced together after the block. RC_DN_SCAN=warp selects k_dn_state_seq for comparison.
template <uint32_t S, uint32_t CPT, uint32_t RPT, uint32_t WARPS>
__global__ void __launch_bounds__(WARPS * 32u) k_dn_scan(DnDims D, uint32_t T, const float *__restrict__ qk, const float *__restrict__ v,
                                                         const float *__restrict__ beta, const float *__restrict__ gate,
                                                         float *__restrict__ state, float *__restrict__ core) {
    pdl_prologue();
    constexpr uint32_t LPR = S / CPT, RPW = 32u / LPR, RB = RPW * RPT * WARPS, NP = CPT / 4u, NT = WARPS * 32u, V4 = S / 4u;
    static_assert(LPR == 2u || LPR == 4u || LPR == 8u || LPR == 16u || LPR == 32u, "lanes per row");
    static_assert(S % RB == 0u && RB % 4u == 0u && DN_TB == 8u, "rows per block");
    __shared__ __align__(16) float s_q[2][DN_TB][S], s_k[2][DN_TB][S];
    __shared__ __align__(16) float s_v[2][RB][DN_TB];            // v by (row, token): a thread reads its row's eight values as two float4
    __shared__ __align__(16) float s_b[2][DN_TB], s_g[2][DN_TB];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, p = lane % LPR, r = lane / LPR;
    const uint32_t h = blockIdx.x / (S / RB), j0 = (blockIdx.x % (S / RB)) * RB;     // head, first of the block's RB rows
    const uint32_t jr = (warp * RPW + r) * RPT;                                      // this thread's first row inside the block
    const uint32_t kh = h / (D.rank / D.groups);
    const size_t tok_qk = (size_t)2u * D.groups * S;
    const float *q = qk + (size_t)kh * S, *k = qk + (size_t)(D.groups + kh) * S;
    float *rows = state + ((size_t)h * S + j0 + jr) * S;
    const float scale = 1.0f / sqrtf((float)S);

    auto stage = [&](uint32_t tb, uint32_t buf) {               // tokens [tb * DN_TB, ...) -> buffer buf
        const uint32_t t0 = tb * DN_TB, n = min(DN_TB, T - t0);
        for (uint32_t i = tid; i < 2u * DN_TB * V4; i += NT) {
            const uint32_t which = i / (DN_TB * V4), tt = (i / V4) % DN_TB, c = (i % V4) * 4u;
            if (tt < n) {
                const float *src = (which ? k : q) + (size_t)(t0 + tt) * tok_qk + c;
                float *dst = (which ? &s_k[buf][tt][0] : &s_q[buf][tt][0]) + c;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
            }
        }
        for (uint32_t i = tid; i < DN_TB * RB; i += NT) {
            const uint32_t tt = i / RB, rr = i % RB;
            if (tt < n)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"((uint32_t)__cvta_generic_to_shared(&s_v[buf][rr][tt])),
                             "l"(v + (size_t)(t0 + tt) * D.d_inner + (size_t)h * S + j0 + rr) : "memory");
        }
        for (uint32_t i = tid; i < DN_TB * 2u; i += NT) {
            const uint32_t tt = i >> 1;
            if (tt < n) {
                const float *src = (i & 1u ? gate : beta) + (size_t)(t0 + tt) * D.rank + h;
                float *dst = i & 1u ? &s_g[buf][tt] : &s_b[buf][tt];
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float2 m[RPT][CPT / 2u];                                     // the rows as register pairs: the arithmetic is packed fp32 (two lanes per instruction)
#pragma unroll
    for (uint32_t a = 0; a < RPT; ++a)
#pragma unroll
        for (uint32_t i = 0; i < NP; ++i) {
            const float4 x = *reinterpret_cast<const float4 *>(rows + (size_t)a * S + 4u * (i * LPR + p));
            m[a][2u * i] = make_float2(x.x, x.y); m[a][2u * i + 1u] = make_float2(x.z, x.w);
        }

    auto body = [&](auto full_c, uint32_t buf, uint32_t n, uint32_t t0) {
        constexpr bool FULL = decltype(full_c)::value;
        // the block's scalars first, off the token-to-token chain: eight decays (lane l computes token l % 8's), betas and this
        // thread's v (entries of tokens >= n are stale and never used)
        float dec[DN_TB], bt[DN_TB], vv[RPT][DN_TB];
        {
            const float dec_l = expf(s_g[buf][lane & (DN_TB - 1u)]);
#pragma unroll
            for (uint32_t tt = 0; tt < DN_TB; ++tt) dec[tt] = __shfl_sync(0xffffffffu, dec_l, (int)tt);
            const float4 b0 = *reinterpret_cast<const float4 *>(&s_b[buf][0]), b1 = *reinterpret_cast<const float4 *>(&s_b[buf][4]);
            bt[0] = b0.x; bt[1] = b0.y; bt[2] = b0.z; bt[3] = b0.w; bt[4] = b1.x; bt[5] = b1.y; bt[6] = b1.z; bt[7] = b1.w;
#pragma unroll
            for (uint32_t a = 0; a < RPT; ++a) {
                const float4 v0 = *reinterpret_cast<const float4 *>(&s_v[buf][jr + a][0]), v1 = *reinterpret_cast<const float4 *>(&s_v[buf][jr + a][4]);
                vv[a][0] = v0.x; vv[a][1] = v0.y; vv[a][2] = v0.z; vv[a][3] = v0.w; vv[a][4] = v1.x; vv[a][5] = v1.y; vv[a][6] = v1.z; vv[a][7] = v1.w;
            }
        }
        float op[RPT][DN_TB];
        float4 kc[NP], kn[NP], qc[NP];
#pragma unroll
        for (uint32_t i = 0; i < NP; ++i) kc[i] = *reinterpret_cast<const float4 *>(&s_k[buf][0][4u * (i * LPR + p)]);
#pragma unroll
        for (uint32_t tt = 0; tt < DN_TB; ++tt) {
#pragma unroll
            for (uint32_t a = 0; a < RPT; ++a) op[a][tt] = 0.f;
            if (FULL || tt < n) {
                // this token's q and the next token's k are requested before the reduction that the chain waits for
#pragma unroll
                for (uint32_t i = 0; i < NP; ++i) {
                    qc[i] = *reinterpret_cast<const float4 *>(&s_q[buf][tt][4u * (i * LPR + p)]);
                    if (tt + 1u < DN_TB) kn[i] = *reinterpret_cast<const float4 *>(&s_k[buf][tt + 1u][4u * (i * LPR + p)]);
                }
                const float2 d2 = make_float2(dec[tt], dec[tt]);
                float delta[RPT];
#pragma unroll
                for (uint32_t a = 0; a < RPT; ++a) {
#pragma unroll
                    for (uint32_t i = 0; i < 2u * NP; ++i) m[a][i] = __fmul2_rn(m[a][i], d2);
                    float2 s2 = __fmul2_rn(m[a][0], make_float2(kc[0].x, kc[0].y));
                    if constexpr (NP == 1u) {
                        s2 = __ffma2_rn(m[a][1], make_float2(kc[0].z, kc[0].w), s2);
                    } else {
                        float2 pb = __fmul2_rn(m[a][1], make_float2(kc[0].z, kc[0].w));
#pragma unroll
                        for (uint32_t i = 1; i < NP; ++i) {
                            s2 = __ffma2_rn(m[a][2u * i], make_float2(kc[i].x, kc[i].y), s2);
                            pb = __ffma2_rn(m[a][2u * i + 1u], make_float2(kc[i].z, kc[i].w), pb);
                        }
                        s2 = __fadd2_rn(s2, pb);
                    }
                    float sum = s2.x + s2.y;
                    if constexpr (LPR <= 8u) {
                        // one exchange step instead of log2(LPR) dependent ones: every lane of the row fetches all LPR partial sums
                        // and adds them in the same order (so the row's lanes agree to the bit)
                        float x[LPR];
#pragma unroll
                        for (uint32_t l = 0; l < LPR; ++l) x[l] = __shfl_sync(0xffffffffu, sum, (int)((lane & ~(LPR - 1u)) + l));
#pragma unroll
                        for (uint32_t w = LPR; w > 1u; w >>= 1)
#pragma unroll
                            for (uint32_t l = 0; l < w / 2u; ++l) x[l] = x[2u * l] + x[2u * l + 1u];
                        sum = x[0];
                    } else {
#pragma unroll
                        for (uint32_t o = LPR / 2u; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, (int)o);
                    }
                    delta[a] = (vv[a][tt] - sum) * bt[tt];
                }
#pragma unroll
                for (uint32_t a = 0; a < RPT; ++a) {
                    const float2 e2 = make_float2(delta[a], delta[a]);
#pragma unroll
                    for (uint32_t i = 0; i < NP; ++i) {
                        m[a][2u * i] = __ffma2_rn(make_float2(kc[i].x, kc[i].y), e2, m[a][2u * i]);
                        m[a][2u * i + 1u] = __ffma2_rn(make_float2(kc[i].z, kc[i].w), e2, m[a][2u * i + 1u]);
                    }
                    float2 s2 = __fmul2_rn(m[a][0], make_float2(qc[0].x, qc[0].y));
                    if constexpr (NP == 1u) {
                        s2 = __ffma2_rn(m[a][1], make_float2(qc[0].z, qc[0].w), s2);
                    } else {
                        float2 pb = __fmul2_rn(m[a][1], make_float2(qc[0].z, qc[0].w));
#pragma unroll
                        for (uint32_t i = 1; i < NP; ++i) {
                            s2 = __ffma2_rn(m[a][2u * i], make_float2(qc[i].x, qc[i].y), s2);
                            pb = __ffma2_rn(m[a][2u * i + 1u], make_float2(qc[i].z, qc[i].w), pb);
                        }
                        s2 = __fadd2_rn(s2, pb);
                    }
                    op[a][tt] = s2.x + s2.y;
                }
                if (tt + 1u < DN_TB) {
#pragma unroll
                    for (uint32_t i = 0; i < NP; ++i) kc[i] = kn[i];
                }
            }
        }
        // the eight output sums over the row's LPR lanes: while a lane carries more than one value each exchange halves them,
        // so a lane ends with max(1, 8 / LPR) finished tokens (first token `tok`) instead of every lane reducing all eight
        constexpr uint32_t LOW = LPR > DN_TB ? LPR / DN_TB - 1u : 0u;     // lane bits below the halving exchanges: those lanes hold copies
#pragma unroll
        for (uint32_t a = 0; a < RPT; ++a) {
            uint32_t tok = 0u, cnt = DN_TB;
#pragma unroll
            for (uint32_t o = LPR / 2u; o; o >>= 1) {
                if (cnt > 1u) {
                    cnt >>= 1;
                    const bool hi = p & o;
#pragma unroll
                    for (uint32_t i = 0; i < DN_TB / 2u; ++i)
                        if (i < cnt) {
                            const float keep = hi ? op[a][cnt + i] : op[a][i], send = hi ? op[a][i] : op[a][cnt + i];
                            op[a][i] = keep + __shfl_xor_sync(0xffffffffu, send, (int)o);
                        }
                    if (hi) tok += cnt;
                } else {
                    op[a][0] += __shfl_xor_sync(0xffffffffu, op[a][0], (int)o);
                }
            }
#pragma unroll
            for (uint32_t i = 0; i < (LPR < DN_TB ? DN_TB / LPR : 1u); ++i)
                if ((p & LOW) == 0u && (FULL || tok + i < n)) core[(size_t)(t0 + tok + i) * D.d_inner + (size_t)h * S + j0 + jr + a] = op[a][i] * scale;
        }
    };

    const uint32_t nblk = (T + DN_TB - 1u) / DN_TB;
    stage(0u, 0u);
    for (uint32_t tb = 0; tb < nblk; ++tb) {
        const uint32_t buf = tb & 1u, n = min(DN_TB, T - tb * DN_TB);
        if (tb + 1u < nblk) stage(tb + 1u, buf ^ 1u); else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();                                         // block tb has landed for every warp
        if (n == DN_TB) body(std::true_type{}, buf, n, tb * DN_TB); else body(std::false_type{}, buf, n, tb * DN_TB);
        __syncthreads();                                         // buffer buf may be refilled by the next stage() call
    }
#pragma unroll
    for (uint32_t a = 0; a < RPT; ++a)
#pragma unroll
        for (uint32_t i = 0; i < NP; ++i)
            *reinterpret_cast<float4 *>(rows + (size_t)a * S + 4u * (i * LPR + p)) =
                make_float4(m[a][2u * i].x, m[a][2u * i].y, m[a][2u * i + 1u].x, m[a][2u * i + 1u].y);
}

// ---- the same recurrence four tokens at a time -------------------------------------------------------------------
// Inside a group of four tokens the corrections delta_t depend on each other only through the scalars k_s . k_t, which are
// the same for every state row of a head. With d_t the per-token decay, g_t = d_1 ... d_t, r(t,s) = d_{s+1} ... d_t and
// m the row before the group:
//   delta_t = beta_t (v_t - g_t (m . k_t) - sum_{s<t} r(t,s) (k_s . k_t) delta_s)
//   out_t   = scale (g_t (m . q_t) + sum_{s<=t} r(t,s) (k_s . q_t) delta_s)
//   m      <- g_4 m + sum_s r(4,s) delta_s k_s
// (the delta rule of native/redlite_native_engine_cpu.c:198-216 unrolled over four steps; the sums are reassociated,
// nothing else changes). A warp therefore needs ONE round of reductions per four tokens — the eight dot products of the
// row with k_1..k_4 and q_1..q_4, reduced together — instead of two dependent reductions per token, which is what bounded
// the token-by-token kernel (a chain of about 1100 cycles per token and row).
// k_dn_pairdots  the 16 scalars of a group per key head: k_s . k_t (s < t) and k_s . q_t (s <= t); grid (groups of 4, key heads)
constexpr uint32_t DN_MC = 4u;
__global__ void __launch_bounds__(32) k_dn_pairdots(DnDims D, uint32_t T, const float *__restrict__ qk, float *__restrict__ pd) {
    pdl_prologue();
    const uint32_t c = blockIdx.x, kh = blockIdx.y, lane = threadIdx.x, S = D.S;
    const size_t tok_qk = (size_t)2u * D.groups * S;
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (uint32_t i = lane; i < S; i += 32u) {
        float q[4], k[4];
#pragma unroll
        for (uint32_t a = 0; a < 4u; ++a) {
            const uint32_t t = c * 4u + a;
            q[a] = t < T ? qk[(size_t)t * tok_qk + (size_t)kh * S + i] : 0.f;
            k[a] = t < T ? qk[(size_t)t * tok_qk + (size_t)(D.groups + kh) * S + i] : 0.f;
        }
        acc[0] += k[0] * k[1]; acc[1] += k[0] * k[2]; acc[2] += k[1] * k[2]; acc[3] += k[0] * k[3]; acc[4] += k[1] * k[3]; acc[5] += k[2] * k[3];
        acc[6] += k[0] * q[0]; acc[7] += k[0] * q[1]; acc[8] += k[1] * q[1]; acc[9] += k[0] * q[2]; acc[10] += k[1] * q[2]; acc[11] += k[2] * q[2];
        acc[12] += k[0] * q[3]; acc[13] += k[1] * q[3]; acc[14] += k[2] * q[3]; acc[15] += k[3] * q[3];
    }
#pragma unroll
    for (int i = 0; i < 16; ++i)
        for (int o = 16; o; o >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
    if (lane < 16u) {
        float v = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) if ((int)lane == i) v = acc[i];
        pd[((size_t)c * D.groups + kh) * 16u + lane] = v;
    }
}

// Block and staging as k_dn_state_seq (8 warps = 8 rows of one head, eight tokens staged at a time); T4 = the tokens that
// form whole groups of four (the caller runs the rest through k_dn_state_seq).
template <int VPL>
__global__ void __launch_bounds__(256) k_dn_state_seq4(DnDims D, uint32_t T4, const float *__restrict__ qk, const float *__restrict__ v,
                                                       const float *__restrict__ beta, const float *__restrict__ gate, const float *__restrict__ pd,
                                                       float *__restrict__ state, float *__restrict__ core) {
    pdl_prologue();
    constexpr uint32_t S = VPL * 32u;
    __shared__ __align__(16) float s_q[2][DN_TB][S], s_k[2][DN_TB][S];
    __shared__ __align__(16) float s_v[2][DN_TB][8];
    __shared__ __align__(16) float s_pd[2][DN_TB / DN_MC][16];
    __shared__ float s_b[2][DN_TB], s_g[2][DN_TB];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t row0 = blockIdx.x * 8u;
    const uint32_t h = row0 / S, j0 = row0 - h * S, j = j0 + warp;
    const uint32_t kh = h / (D.rank / D.groups);
    const size_t tok_qk = (size_t)2u * D.groups * S;
    const float *q = qk + (size_t)kh * S, *k = qk + (size_t)(D.groups + kh) * S;
    float *row = state + ((size_t)h * S + j) * S;
    const float scale = 1.0f / sqrtf((float)S);

    auto stage = [&](uint32_t tb, uint32_t buf) {               // tokens [tb * DN_TB, ...) -> buffer buf (T4 is a multiple of 4, so n is 4 or 8)
        const uint32_t t0 = tb * DN_TB, n = min(DN_TB, T4 - t0);
        constexpr uint32_t V4 = S / 4u;
        for (uint32_t i = tid; i < 2u * n * V4; i += 256u) {
            const uint32_t which = i / (n * V4), r = i - which * n * V4, tt = r / V4, c = (r - tt * V4) * 4u;
            const float *src = (which ? k : q) + (size_t)(t0 + tt) * tok_qk + c;
            float *dst = (which ? &s_k[buf][tt][0] : &s_q[buf][tt][0]) + c;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
        }
        for (uint32_t i = tid; i < n * 2u; i += 256u) {
            const uint32_t tt = i >> 1, c = (i & 1u) * 4u;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(&s_v[buf][tt][c])),
                         "l"(v + (size_t)(t0 + tt) * D.d_inner + (size_t)h * S + j0 + c) : "memory");
        }
        for (uint32_t i = tid; i < n * 2u; i += 256u) {
            const uint32_t tt = i >> 1;
            const float *src = (i & 1u ? gate : beta) + (size_t)(t0 + tt) * D.rank + h;
            float *dst = i & 1u ? &s_g[buf][tt] : &s_b[buf][tt];
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
        }
        for (uint32_t i = tid; i < (n / DN_MC) * 4u; i += 256u) {     // the groups' 16 scalars, 16 bytes per copy
            const uint32_t g = i >> 2, c = (i & 3u) * 4u;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(&s_pd[buf][g][c])),
                         "l"(pd + ((size_t)(t0 / DN_MC + g) * D.groups + kh) * 16u + c) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float m[VPL];
#pragma unroll
    for (int t = 0; t < VPL; ++t) m[t] = row[lane + 32 * t];
    const uint32_t nblk = (T4 + DN_TB - 1u) / DN_TB;
    if (nblk) stage(0u, 0u);
    for (uint32_t tb = 0; tb < nblk; ++tb) {
        const uint32_t buf = tb & 1u, n = min(DN_TB, T4 - tb * DN_TB);
        if (tb + 1u < nblk) stage(tb + 1u, buf ^ 1u); else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        for (uint32_t g4 = 0; g4 < n / DN_MC; ++g4) {
            const uint32_t t0 = g4 * DN_MC;
            // ---- the row's eight dot products with k_1..k_4 (p[0..3]) and q_1..q_4 (p[4..7]), this lane's share
            float kc[4][VPL], p[8];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                float sk = 0.f, sq = 0.f;
#pragma unroll
                for (int t = 0; t < VPL; ++t) { kc[a][t] = s_k[buf][t0 + a][lane + 32 * t]; sk += m[t] * kc[a][t]; sq += m[t] * s_q[buf][t0 + a][lane + 32 * t]; }
                p[a] = sk; p[4 + a] = sq;
            }
            // ---- reduce the eight values together: each exchange halves the values a lane carries (4 + 2 + 1 shuffles), two
            // more finish the one that is left; value i ends up complete in the lanes whose bits 4, 3, 2 spell i
            {
                const bool hi4 = lane & 16u, hi3 = lane & 8u, hi2 = lane & 4u;
                float a4[4], a2[2], a1;
#pragma unroll
                for (int i = 0; i < 4; ++i) { const float keep = hi4 ? p[4 + i] : p[i], send = hi4 ? p[i] : p[4 + i]; a4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16); }
#pragma unroll
                for (int i = 0; i < 2; ++i) { const float keep = hi3 ? a4[2 + i] : a4[i], send = hi3 ? a4[i] : a4[2 + i]; a2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8); }
                { const float keep = hi2 ? a2[1] : a2[0], send = hi2 ? a2[0] : a2[1]; a1 = keep + __shfl_xor_sync(0xffffffffu, send, 4); }
                a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
                a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
#pragma unroll
                for (int i = 0; i < 8; ++i) p[i] = __shfl_sync(0xffffffffu, a1, ((i >> 2) & 1) * 16 + ((i >> 1) & 1) * 8 + (i & 1) * 4);
            }
            // ---- the four corrections and outputs (every lane computes them; they are scalars of the row)
            const float d0 = expf(s_g[buf][t0]), d1 = expf(s_g[buf][t0 + 1u]), d2 = expf(s_g[buf][t0 + 2u]), d3 = expf(s_g[buf][t0 + 3u]);
            const float g0 = d0, g1 = g0 * d1, g2 = g1 * d2, g3 = g2 * d3;
            const float r10 = d1, r21 = d2, r32 = d3, r20 = d1 * d2, r31 = d2 * d3, r30 = r20 * d3;
            const float4 pa = *reinterpret_cast<const float4 *>(&s_pd[buf][g4][0]), pb = *reinterpret_cast<const float4 *>(&s_pd[buf][g4][4]),
                         pc = *reinterpret_cast<const float4 *>(&s_pd[buf][g4][8]), pe = *reinterpret_cast<const float4 *>(&s_pd[buf][g4][12]);
            // pa = (k0.k1, k0.k2, k1.k2, k0.k3), pb = (k1.k3, k2.k3, k0.q0, k0.q1), pc = (k1.q1, k0.q2, k1.q2, k2.q2), pe = (k0.q3, k1.q3, k2.q3, k3.q3)
            const float e0 = (s_v[buf][t0][warp] - g0 * p[0]) * s_b[buf][t0];
            const float e1 = (s_v[buf][t0 + 1u][warp] - g1 * p[1] - r10 * pa.x * e0) * s_b[buf][t0 + 1u];
            const float e2 = (s_v[buf][t0 + 2u][warp] - g2 * p[2] - r20 * pa.y * e0 - r21 * pa.z * e1) * s_b[buf][t0 + 2u];
            const float e3 = (s_v[buf][t0 + 3u][warp] - g3 * p[3] - r30 * pa.w * e0 - r31 * pb.x * e1 - r32 * pb.y * e2) * s_b[buf][t0 + 3u];
            if (lane == 0) {
                const size_t o = (size_t)(tb * DN_TB + t0) * D.d_inner + (size_t)h * S + j;
                core[o] = (g0 * p[4] + pb.z * e0) * scale;
                core[o + D.d_inner] = (g1 * p[5] + r10 * pb.w * e0 + pc.x * e1) * scale;
                core[o + 2u * (size_t)D.d_inner] = (g2 * p[6] + r20 * pc.y * e0 + r21 * pc.z * e1 + pc.w * e2) * scale;
                core[o + 3u * (size_t)D.d_inner] = (g3 * p[7] + r30 * pe.x * e0 + r31 * pe.y * e1 + r32 * pe.z * e2 + pe.w * e3) * scale;
            }
            // ---- the row after the group
            const float c0 = r30 * e0, c1 = r31 * e1, c2 = r32 * e2;
#pragma unroll
            for (int t = 0; t < VPL; ++t) m[t] = g3 * m[t] + c0 * kc[0][t] + c1 * kc[1][t] + c2 * kc[2][t] + e3 * kc[3][t];
        }
        __syncthreads();
    }
#pragma unroll
    for (int t = 0; t < VPL; ++t) row[lane + 32 * t] = m[t];
}

int launch_deltanet_seq(const DnDims &D, uint32_t T, const float *conv_kernel, const float *dt_bias, const float *ssm_a, const float *norm_w,
                        const float *qkv, const float *z, const float *ba, float *conv_state, float *rec_state,
                        float *qk, float *v, float *beta, float *gate, float *core, float *out, float *pairdots, cudaStream_t s) {
    RC_REQUIRE(D.S == 32u || D.S == 64u || D.S == 128u || D.S == 256u, "deltanet: state size %u not in {32,64,128,256}", D.S);
    RC_REQUIRE(D.rank && D.groups && D.rank % D.groups == 0 && D.d_inner == D.rank * D.S && D.channels == 2u * D.S * D.groups + D.d_inner && D.d_conv >= 2u,
               "deltanet: inconsistent dimensions");
    if (!T) return 1;
    prof_begin("dn_prep_seq", s);
    RC_LAUNCH((k_dn_prep_seq), dim3(2u * D.groups + D.d_inner / D.S + 1u, (T + DN_PREP_TOK - 1u) / DN_PREP_TOK), D.S, 0, s, D, T, conv_kernel, dt_bias, ssm_a, qkv, ba, (const float *)conv_state, qk, v, beta, gate);
    prof_end(s);
    RC_LAUNCHED();
    prof_begin("dn_conv_roll", s);
    RC_LAUNCH((k_dn_conv_roll), (D.channels + 255u) / 256u, 256, 0, s, D, T, qkv, conv_state);
    prof_end(s);
    RC_LAUNCHED();
    const uint32_t blocks = (D.rank * D.S + 7u) / 8u;
    // RC_DN_SCAN=grouped sends whole groups of four tokens through the grouped recurrence (the token-by-token kernel takes
    // the up to three tokens left over). Off by default: measured on 2048-token chunks it is 1.19x faster (0.98 against
    // 1.16 ms per layer — both forms execute about the same number of instructions) and its reassociated sums leave three
    // times the rounding noise at the 48th layer (1.8e-4 against 5.4e-5 of the layer output), which the full-depth router
    // comparison notices.
    const char *scan = getenv("RC_DN_SCAN");
    const bool grouped = scan && scan[0] == 'g';
    const uint32_t T4 = grouped && pairdots && D.S <= 128u ? T / DN_MC * DN_MC : 0u;
    if (T4) {
        prof_begin("dn_pairdots", s);
        RC_LAUNCH((k_dn_pairdots), dim3(T4 / DN_MC, D.groups), 32, 0, s, D, T4, (const float *)qk, pairdots);
        prof_end(s);
        RC_LAUNCHED();
        prof_begin("dn_state_seq4", s);
        switch (D.S) {
            case 32: RC_LAUNCH((k_dn_state_seq4<1>), blocks, 256, 0, s, D, T4, qk, v, beta, gate, (const float *)pairdots, rec_state, core); break;
            case 64: RC_LAUNCH((k_dn_state_seq4<2>), blocks, 256, 0, s, D, T4, qk, v, beta, gate, (const float *)pairdots, rec_state, core); break;
            default: RC_LAUNCH((k_dn_state_seq4<4>), blocks, 256, 0, s, D, T4, qk, v, beta, gate, (const float *)pairdots, rec_state, core); break;
        }
        prof_end(s);
        RC_LAUNCHED();
    }
    const bool per_warp = scan && scan[0] == 'w';                 // RC_DN_SCAN=warp: the one-row-per-warp kernel, for comparison
    if (T4 < T && !per_warp) {
        const uint32_t Tr = T - T4;
        const size_t tok_qk = (size_t)2u * D.groups * D.S;
        const float *qk_r = qk + (size_t)T4 * tok_qk, *v_r = v + (size_t)T4 * D.d_inner, *b_r = beta + (size_t)T4 * D.rank, *g_r = gate + (size_t)T4 * D.rank;
        float *core_r = core + (size_t)T4 * D.d_inner;
        prof_begin("dn_state_seq", s);
        switch (D.S) {
            case 32: RC_LAUNCH((k_dn_scan<32, 16, 1, 2>), D.rank, 64, 0, s, D, Tr, qk_r, v_r, b_r, g_r, rec_state, core_r); break;
            case 64: RC_LAUNCH((k_dn_scan<64, 16, 1, 8>), D.rank, 256, 0, s, D, Tr, qk_r, v_r, b_r, g_r, rec_state, core_r); break;
            // 128-wide states: two rows per thread halve the shared-memory reads of k and q per multiply-add; measured on 2048-token
            // chunks this tile took 0.50 ms, one row per thread 0.53-0.54 ms, wider lane groups (4 or 8 columns per thread) 0.58-0.70 ms
            case 128: RC_LAUNCH((k_dn_scan<128, 16, 2, 4>), D.rank * 4u, 128, 0, s, D, Tr, qk_r, v_r, b_r, g_r, rec_state, core_r); break;
            default: RC_LAUNCH((k_dn_scan<256, 32, 1, 8>), D.rank * 8u, 256, 0, s, D, Tr, qk_r, v_r, b_r, g_r, rec_state, core_r); break;
        }
        prof_end(s);
        RC_LAUNCHED();
    } else if (T4 < T) {
        const uint32_t Tr = T - T4;
        const size_t tok_qk = (size_t)2u * D.groups * D.S;
        const float *qk_r = qk + (size_t)T4 * tok_qk, *v_r = v + (size_t)T4 * D.d_inner, *b_r = beta + (size_t)T4 * D.rank, *g_r = gate + (size_t)T4 * D.rank;
        float *core_r = core + (size_t)T4 * D.d_inner;
        prof_begin("dn_state_seq", s);
        switch (D.S) {
            case 32: RC_LAUNCH((k_dn_state_seq<1>), blocks, 256, 0, s, D, Tr, qk_r, v_r, b_r, g_r, rec_state, core_r); break;
            case 64: RC_LAUNCH((k_dn_state_seq<2>), blocks, 256, 0, s, D, Tr, qk_r, v_r, b_r, g_r, rec_state, core_r); break;
            case 128: RC_LAUNCH((k_dn_state_seq<4>), blocks, 256, 0, s, D, Tr, qk_r, v_r, b_r, g_r, rec_state, core_r); break;
            default: RC_LAUNCH((k_dn_state_seq<8>), blocks, 256, 0, s, D, Tr, qk_r, v_r, b_r, g_r, rec_state, core_r); break;
        }
        prof_end(s);
        RC_LAUNCHED();
    }
    prof_begin("dn_tail", s);
    RC_LAUNCH((k_dn_tail), dim3(D.rank, T), D.S, 0, s, D, core, z, norm_w, out);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

int launch_deltanet(const DnDims &D, uint32_t batch, const float *conv_kernel, const float *dt_bias, const float *ssm_a, const float *norm_w,
                    const float *qkv, const float *z, const float *ba, float *conv_state, float *rec_state,
                    float *qk, float *v, float *beta, float *gate, float *core, float *out, cudaStream_t s) {
    RC_REQUIRE(D.S >= 32u && D.S <= 256u && D.S % 32u == 0 && (D.S == 32u || D.S == 64u || D.S == 128u || D.S == 256u), "deltanet: state size %u not in {32,64,128,256}", D.S);
    RC_REQUIRE(D.rank && D.groups && D.rank % D.groups == 0 && D.d_inner == D.rank * D.S && D.channels == 2u * D.S * D.groups + D.d_inner && D.d_conv >= 2u,
               "deltanet: inconsistent dimensions");
    if (!batch) return 1;
    const dim3 gp(2u * D.groups + D.d_inner / D.S + 1u, batch);
    prof_begin("dn_prep", s);
    RC_LAUNCH((k_dn_prep), gp, D.S, 0, s, D, conv_kernel, dt_bias, ssm_a, qkv, ba, conv_state, qk, v, beta, gate);
    prof_end(s);
    RC_LAUNCHED();
    // One block per (head, sequence) for state update + tail. Measured (16/32 heads of 128): batch 8 12.8 us against 16.5 us
    // for the two-kernel form; a single sequence fills only 32 SMs that way and stays on the two-kernel form (7.3 against
    // 7.9 us). RC_DN_FUSE=0 / 1 forces one or the other.
    static const int fuse_env = getenv("RC_DN_FUSE") ? atoi(getenv("RC_DN_FUSE")) : -1;
    const bool fuse = fuse_env < 0 ? batch >= 2u : fuse_env != 0;
    if (fuse && D.S <= 128u) {
        prof_begin("dn_state_tail", s);
        const dim3 gs(D.rank, batch);
        switch (D.S) {
            case 32: RC_LAUNCH((k_dn_state_tail<1>), gs, 256, 0, s, D, qk, v, beta, gate, rec_state, z, norm_w, out); break;
            case 64: RC_LAUNCH((k_dn_state_tail<2>), gs, 256, 0, s, D, qk, v, beta, gate, rec_state, z, norm_w, out); break;
            default: RC_LAUNCH((k_dn_state_tail<4>), gs, 256, 0, s, D, qk, v, beta, gate, rec_state, z, norm_w, out); break;
        }
        prof_end(s);
        RC_LAUNCHED();
        return 1;
    }
    prof_begin("dn_state", s);
    const uint64_t warps = (uint64_t)batch * D.rank * D.S;
    const uint32_t blocks = (uint32_t)((warps + 7u) / 8u);
    switch (D.S) {
        case 32: RC_LAUNCH((k_dn_state<1>), blocks, 256, 0, s, D, batch, qk, v, beta, gate, rec_state, core); break;
        case 64: RC_LAUNCH((k_dn_state<2>), blocks, 256, 0, s, D, batch, qk, v, beta, gate, rec_state, core); break;
        case 128: RC_LAUNCH((k_dn_state<4>), blocks, 256, 0, s, D, batch, qk, v, beta, gate, rec_state, core); break;
        default: RC_LAUNCH((k_dn_state<8>), blocks, 256, 0, s, D, batch, qk, v, beta, gate, rec_state, core); break;
    }
    prof_end(s);
    RC_LAUNCHED();
    prof_begin("dn_tail", s);
    RC_LAUNCH((k_dn_tail), dim3(D.rank, batch), D.S, 0, s, D, core, z, norm_w, out);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

}  // namespace rc

using namespace rc;

extern "C" int redcuda_deltanet_step(const redcuda_deltanet_params *p, uint32_t batch, const float *qkv, const float *z, const float *ba,
                                     float *conv_state, float *rec_state, float *out) {
    if (!require_device()) return 0;
    RC_REQUIRE(p && qkv && z && ba && conv_state && rec_state && out && batch, "deltanet step: null or empty argument");
    RC_REQUIRE(p->conv_kernel && p->dt_bias && p->ssm_a && p->ssm_norm, "deltanet step: null parameter array");
    const DnDims D{p->d_conv, p->d_state, p->n_group, p->dt_rank, p->d_inner, p->channels, p->rms_eps};
    RC_REQUIRE(D.rank && D.S && D.groups && D.d_conv >= 2u, "deltanet step: zero dimension");
    const size_t ns = D.d_conv - 1u, nqk = 2u * (size_t)D.groups * D.S;
    const size_t b_ck = (size_t)D.channels * D.d_conv * 4u, b_r = (size_t)D.rank * 4u, b_nw = (size_t)D.S * 4u;
    const size_t b_qkv = (size_t)batch * D.channels * 4u, b_z = (size_t)batch * D.d_inner * 4u, b_ba = (size_t)batch * 2u * D.rank * 4u;
    const size_t b_cs = (size_t)batch * D.channels * ns * 4u, b_rs = (size_t)batch * D.rank * D.S * D.S * 4u;
    DevMem ck, dt, sa, nw, dq, dz, dba, cs, rs, qk, v, beta, gate, core, o;
    if (!ck.alloc(b_ck) || !dt.alloc(b_r) || !sa.alloc(b_r) || !nw.alloc(b_nw) || !dq.alloc(b_qkv) || !dz.alloc(b_z) || !dba.alloc(b_ba) ||
        !cs.alloc(b_cs) || !rs.alloc(b_rs) || !qk.alloc(batch * nqk * 4u) || !v.alloc(b_z) || !beta.alloc(batch * b_r) || !gate.alloc(batch * b_r) ||
        !core.alloc(b_z) || !o.alloc(b_z)) return 0;
    cudaStream_t s = 0;
    RC_CUDA(cudaMemcpyAsync(ck.p, p->conv_kernel, b_ck, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemcpyAsync(dt.p, p->dt_bias, b_r, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemcpyAsync(sa.p, p->ssm_a, b_r, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemcpyAsync(nw.p, p->ssm_norm, b_nw, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemcpyAsync(dq.p, qkv, b_qkv, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemcpyAsync(dz.p, z, b_z, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemcpyAsync(dba.p, ba, b_ba, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemcpyAsync(cs.p, conv_state, b_cs, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemcpyAsync(rs.p, rec_state, b_rs, cudaMemcpyHostToDevice, s));
    if (!launch_deltanet(D, batch, ck.as<float>(), dt.as<float>(), sa.as<float>(), nw.as<float>(), dq.as<float>(), dz.as<float>(), dba.as<float>(),
                         cs.as<float>(), rs.as<float>(), qk.as<float>(), v.as<float>(), beta.as<float>(), gate.as<float>(), core.as<float>(), o.as<float>(), s)) return 0;
    RC_CUDA(cudaMemcpyAsync(conv_state, cs.p, b_cs, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaMemcpyAsync(rec_state, rs.p, b_rs, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaMemcpyAsync(out, o.p, b_z, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    return 1;
}

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free variant of the DeltaNet step.
//
// The step needs scratch between its three kernels (normalised q/k, conv output v, beta, gate, un-normalised head
// outputs). redcuda_deltanet_step allocates that scratch per call, which a caller cannot afford when it runs inside a
// serving loop that must never block on the allocator (cudaMalloc / cudaFree synchronise the whole device), or when
// another runtime owns the device memory budget. For those callers the scratch lives in the array below, part of the
// library image: every GPU that loads the library holds these 512 KiB until the process exits.
#define RC_DN_SCRATCH_FLOATS (128u * 1024u)
static __device__ __align__(256) float g_dn_scratch[RC_DN_SCRATCH_FLOATS];

// In host code g_dn_scratch is only a handle for the runtime, not an address a kernel may use; the device address is
// asked for once per device (with that device current) and cached here.
static std::mutex g_dn_scratch_mu;
static float *g_dn_scratch_dev[64] = {nullptr};

extern "C" int redcuda_deltanet_step_noalloc(const redcuda_deltanet_params *p, uint32_t batch, const float *qkv_dev, const float *z_dev,
                                             const float *ba_dev, float *conv_state_dev, float *rec_state_dev, float *out_dev, void *stream) {
    if (!require_device()) return 0;
    RC_REQUIRE(p && qkv_dev && z_dev && ba_dev && conv_state_dev && rec_state_dev && out_dev && batch, "deltanet step (no-alloc): null or empty argument");
    RC_REQUIRE(p->conv_kernel && p->dt_bias && p->ssm_a && p->ssm_norm, "deltanet step (no-alloc): null parameter array");
    const DnDims D{p->d_conv, p->d_state, p->n_group, p->dt_rank, p->d_inner, p->channels, p->rms_eps};
    const uint64_t n_qk = (uint64_t)batch * 2u * D.groups * D.S, n_v = (uint64_t)batch * D.d_inner, n_r = (uint64_t)batch * D.rank;
    const uint64_t need = n_qk + 2u * n_v + 2u * n_r;
    RC_REQUIRE(need <= RC_DN_SCRATCH_FLOATS,
               "deltanet step (no-alloc): batch %u with these dimensions needs %llu scratch floats, the built-in scratch holds %u; "
               "use a smaller batch or redcuda_deltanet_step", batch, (unsigned long long)need, RC_DN_SCRATCH_FLOATS);
    int dev = 0;
    RC_CUDA(cudaGetDevice(&dev));
    RC_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
    float *scr = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_dn_scratch_mu);
        if (!g_dn_scratch_dev[dev]) {      // first call on this device: resolve the symbol (not during stream capture)
            void *sym = nullptr;
            RC_CUDA(cudaGetSymbolAddress(&sym, g_dn_scratch));
            g_dn_scratch_dev[dev] = (float *)sym;
        }
        scr = g_dn_scratch_dev[dev];
    }
    // every scratch region is fully written by k_dn_prep / k_dn_state before it is read, so nothing has to be cleared
    float *qk = scr, *v = qk + n_qk, *core = v + n_v, *beta = core + n_v, *gate = beta + n_r;
    return launch_deltanet(D, batch, p->conv_kernel, p->dt_bias, p->ssm_a, p->ssm_norm, qkv_dev, z_dev, ba_dev, conv_state_dev, rec_state_dev,
                           qk, v, beta, gate, core, out_dev, (cudaStream_t)stream);
}
