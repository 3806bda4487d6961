// Causal attention of a prefill chunk on the tensor cores: every token of the chunk against the K/V cache up to its own
// position (the chunk's K/V rows are appended first), grouped-query heads, online softmax, sigmoid output gate.
//
// What it computes is the per-token attention of native/redlite_native_engine_cpu.c:297-317 (scores q.k / sqrt(d),
// softmax over positions <= the token's, weighted V sum, output gate); the reference's batched form is
// native/redmetal_engine_prefill.m:536-605. The decode kernel of this library (k_attn_decode) does the same per token on
// CUDA cores; for a chunk that reads every K/V row once per token. Here a block of 64 query rows shares each K/V tile.
//
// Tiling. One CTA = one K/V head x 64 query rows = 64 / G consecutive tokens x the G query heads that share the K/V
// head; 4 warps of 16 rows. Positions are visited in tiles of 32: S = Q K^T with mma.sync m16n8k16 (fp16 operands, fp32
// accumulation), online softmax in registers, O += P V. K/V tiles are double-buffered in shared memory (cp.async when the
// cache is fp16). All shared-memory tiles are swizzled (16-byte chunk index xor row % 8) so that ldmatrix is conflict-free.
//
// Accuracy. The activations are fp32 and the 48-layer model amplifies rounding noise, so no operand is rounded to one
// fp16 value: Q and P are split into two fp16 digits (hi + lo, 22 significant bits); an fp16 cache supplies K and V
// exactly, an fp32 cache is split as well (then hi*hi + lo*hi + hi*lo, the lo*lo term is below fp32 resolution).
// The tensor core's fp32 accumulation is kept short: the scores of a tile are one accumulation of 2 * head_dim / 16
// MMAs, and every tile's P V product starts from zero and is added to the running output with ordinary fp32 FMAs (which
// also apply the online-softmax rescale), so no accumulator lives longer than a tile.
#define RC_PDL_DEFAULT 1
#include "redcuda_common.cuh"
#include "redcuda_kernels.cuh"

#include <cuda_fp16.h>

namespace rc {

constexpr uint32_t AC_ROWS = 64u, AC_TILE = 32u, AC_THREADS = 128u;

__device__ __forceinline__ uint32_t ac_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
// byte offset of 16-byte chunk c of row r in a swizzled tile with `pitch` bytes per row
__device__ __forceinline__ uint32_t ac_off(uint32_t r, uint32_t c, uint32_t pitch) { return r * pitch + ((c ^ (r & 7u)) << 4); }

__device__ __forceinline__ void ac_ldsm4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ac_ldsm4t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ac_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// two fp32 values -> their fp16 digits, packed: hi = round(v), lo = round(v - hi)
__device__ __forceinline__ void ac_split2(float a, float b, uint32_t &hi, uint32_t &lo) {
    const __half2 h = __floats2half2_rn(a, b);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(a - hf.x, b - hf.y);
    hi = *reinterpret_cast<const uint32_t *>(&h); lo = *reinterpret_cast<const uint32_t *>(&l);
}

// KV = __half: K/V tiles are copied as they are (one digit). KV = float: split into hi / lo tiles on the way in.
template <typename KV, int HD, int G>
__global__ void __launch_bounds__(AC_THREADS, 1) k_attn_chunk(const float *__restrict__ query, const KV *__restrict__ kcache, const KV *__restrict__ vcache,
                                                               uint32_t n_kv, const uint32_t *__restrict__ pos_p, uint32_t ntok, float scale,
                                                               const float *__restrict__ gate, float *__restrict__ gated) {
    pdl_prologue();
    constexpr bool HALF = sizeof(KV) == 2;
    constexpr uint32_t PITCH = HD * 2u, CH = HD / 8u;                 // bytes and 16-byte chunks per row of a tile
    constexpr uint32_t Q_BYTES = AC_ROWS * PITCH, KV_BYTES = AC_TILE * PITCH;
    constexpr uint32_t TPB = AC_ROWS / G;                             // tokens per block
    constexpr uint32_t ND = HALF ? 1u : 2u;                           // digits of K and V
    extern __shared__ __align__(128) uint8_t sm[];
    // layout: Q hi, Q lo, then two K/V buffer sets; a set = K digits then V digits. The fp32 cache uses one set (no copy engine to overlap with).
    uint8_t *q_hi = sm, *q_lo = sm + Q_BYTES, *kv0 = sm + 2u * Q_BYTES;
    constexpr uint32_t SET = 2u * ND * KV_BYTES;
    __shared__ uint32_t s_lim[AC_ROWS];                               // last position every row may attend to
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t qb = gridDim.x - 1u - blockIdx.x, kvh = blockIdx.y;    // the longest rows first
    const uint32_t n_head = n_kv * G, tok0 = qb * TPB;

    // ---- Q rows of the block -> two fp16 digit tiles; row r = (token tok0 + r / G, head kvh * G + r % G)
    for (uint32_t i = tid; i < AC_ROWS * CH; i += AC_THREADS) {
        const uint32_t r = i / CH, c = i - r * CH, z = tok0 + r / G, h = kvh * G + r % G;
        uint4 hi = make_uint4(0u, 0u, 0u, 0u), lo = hi;
        if (z < ntok) {
            const float4 *src = reinterpret_cast<const float4 *>(query + ((size_t)z * n_head + h) * HD + c * 8u);
            const float4 a = src[0], b = src[1];
            ac_split2(a.x, a.y, hi.x, lo.x); ac_split2(a.z, a.w, hi.y, lo.y); ac_split2(b.x, b.y, hi.z, lo.z); ac_split2(b.z, b.w, hi.w, lo.w);
        }
        *reinterpret_cast<uint4 *>(q_hi + ac_off(r, c, PITCH)) = hi;
        *reinterpret_cast<uint4 *>(q_lo + ac_off(r, c, PITCH)) = lo;
    }
    if (tid < AC_ROWS) { const uint32_t z = tok0 + tid / G; s_lim[tid] = z < ntok ? pos_p[z] : 0u; }
    const uint32_t z_last = min(tok0 + TPB, ntok) - 1u;
    const uint32_t p_max = pos_p[z_last], n_tiles = p_max / AC_TILE + 1u;      // positions grow with the token index

    // ---- K/V tile j -> buffer set (rows beyond p_max are zero-filled and masked)
    auto load_tile = [&](uint32_t j, uint8_t *set) {
        for (uint32_t i = tid; i < AC_TILE * CH; i += AC_THREADS) {
            const uint32_t r = i / CH, c = i - r * CH, p = j * AC_TILE + r;
            const bool live = p <= p_max;
            const size_t row = ((size_t)(live ? p : 0u) * n_kv + kvh) * HD + c * 8u;
            if (HALF) {
                const uint32_t sz = live ? 16u : 0u;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(ac_smem(set + ac_off(r, c, PITCH))), "l"(kcache + row), "r"(sz) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(ac_smem(set + KV_BYTES + ac_off(r, c, PITCH))), "l"(vcache + row), "r"(sz) : "memory");
            } else {
                uint4 kh = make_uint4(0u, 0u, 0u, 0u), kl = kh, vh = kh, vl = kh;
                if (live) {
                    const float4 *ks = reinterpret_cast<const float4 *>(kcache + row), *vs = reinterpret_cast<const float4 *>(vcache + row);
                    const float4 a = ks[0], b = ks[1], e = vs[0], f = vs[1];
                    ac_split2(a.x, a.y, kh.x, kl.x); ac_split2(a.z, a.w, kh.y, kl.y); ac_split2(b.x, b.y, kh.z, kl.z); ac_split2(b.z, b.w, kh.w, kl.w);
                    ac_split2(e.x, e.y, vh.x, vl.x); ac_split2(e.z, e.w, vh.y, vl.y); ac_split2(f.x, f.y, vh.z, vl.z); ac_split2(f.z, f.w, vh.w, vl.w);
                }
                const uint32_t o = ac_off(r, c, PITCH);
                *reinterpret_cast<uint4 *>(set + o) = kh; *reinterpret_cast<uint4 *>(set + KV_BYTES + o) = kl;
                *reinterpret_cast<uint4 *>(set + 2u * KV_BYTES + o) = vh; *reinterpret_cast<uint4 *>(set + 3u * KV_BYTES + o) = vl;
            }
        }
        if (HALF) asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // ---- per-warp state: 16 rows; a lane holds rows lane / 4 and lane / 4 + 8, columns 2 * (lane % 4) + {0, 1} of every 8-wide tile
    constexpr uint32_t NT_O = HD / 8u;                                // 8-wide output tiles
    float o_acc[NT_O][4];
#pragma unroll
    for (uint32_t n = 0; n < NT_O; ++n) { o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const uint32_t r_base = warp * 16u;
    if (HALF) load_tile(0u, kv0);
    __syncthreads();                                                  // Q tiles and s_lim written
    const uint32_t lim0 = s_lim[r_base + (lane >> 2)], lim1 = s_lim[r_base + (lane >> 2) + 8u];

    for (uint32_t j = 0; j < n_tiles; ++j) {
        uint8_t *set = HALF ? kv0 + (j & 1u) * SET : kv0;
        if (HALF) {
            if (j + 1u < n_tiles) { load_tile(j + 1u, kv0 + ((j + 1u) & 1u) * SET); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
            else asm volatile("cp.async.wait_group 0;" ::: "memory");
        } else load_tile(j, set);
        __syncthreads();
        const uint8_t *k_hi = set, *k_lo = set + KV_BYTES, *v_hi = set + ND * KV_BYTES, *v_lo = v_hi + KV_BYTES;

        // ---- S = Q K^T for 16 rows x 32 positions
        float s[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll 4
        for (uint32_t kk = 0; kk < HD / 16u; ++kk) {
            uint32_t ah[4], al[4];
            {   // A fragments: matrices (rows 0-7 | 8-15) x (k chunk 2 kk | 2 kk + 1)
                const uint32_t r = r_base + (lane & 7u) + ((lane >> 3) & 1u) * 8u, c = 2u * kk + (lane >> 4);
                ac_ldsm4(ac_smem(q_hi + ac_off(r, c, PITCH)), ah[0], ah[1], ah[2], ah[3]);
                ac_ldsm4(ac_smem(q_lo + ac_off(r, c, PITCH)), al[0], al[1], al[2], al[3]);
            }
#pragma unroll
            for (uint32_t np = 0; np < 2u; ++np) {     // two position tiles of 8 per ldmatrix.x4
                const uint32_t r = np * 16u + (lane & 7u) + (lane >> 4) * 8u, c = 2u * kk + ((lane >> 3) & 1u);
                uint32_t b0, b1, b2, b3;
                ac_ldsm4(ac_smem(k_hi + ac_off(r, c, PITCH)), b0, b1, b2, b3);
                ac_mma(s[2 * np], ah[0], ah[1], ah[2], ah[3], b0, b1); ac_mma(s[2 * np + 1], ah[0], ah[1], ah[2], ah[3], b2, b3);
                ac_mma(s[2 * np], al[0], al[1], al[2], al[3], b0, b1); ac_mma(s[2 * np + 1], al[0], al[1], al[2], al[3], b2, b3);
                if (!HALF) {
                    ac_ldsm4(ac_smem(k_lo + ac_off(r, c, PITCH)), b0, b1, b2, b3);
                    ac_mma(s[2 * np], ah[0], ah[1], ah[2], ah[3], b0, b1); ac_mma(s[2 * np + 1], ah[0], ah[1], ah[2], ah[3], b2, b3);
                }
            }
        }
        // ---- mask, online softmax (rows lane / 4 and + 8; a row's 32 scores sit in the 4 lanes of a quad)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            const uint32_t p = j * AC_TILE + n * 8u + 2u * (lane & 3u);
            s[n][0] = p <= lim0 ? s[n][0] * scale : -INFINITY; s[n][1] = p + 1u <= lim0 ? s[n][1] * scale : -INFINITY;
            s[n][2] = p <= lim1 ? s[n][2] * scale : -INFINITY; s[n][3] = p + 1u <= lim1 ? s[n][3] * scale : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1])); mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        // position 0 is open to every row, so after the first tile no maximum is -inf; inside the first tile m_run is
        const float c0 = m_run[0] == -INFINITY ? 0.f : expf(m_run[0] - mn0), c1 = m_run[1] == -INFINITY ? 0.f : expf(m_run[1] - mn1);
        m_run[0] = mn0; m_run[1] = mn1;
        uint32_t ph[2][4], pl[2][4];              // P as A fragments of the two k-steps (16 positions each), hi and lo digits
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            const float e0 = expf(s[n][0] - mn0), e1 = expf(s[n][1] - mn0), e2 = expf(s[n][2] - mn1), e3 = expf(s[n][3] - mn1);
            sum0 += e0 + e1; sum1 += e2 + e3;
            // accumulator tile n -> A fragment registers: tile 2q gives a0 (row) and a1 (row + 8), tile 2q + 1 gives a2 and a3
            ac_split2(e0, e1, ph[n >> 1][(n & 1) * 2], pl[n >> 1][(n & 1) * 2]);
            ac_split2(e2, e3, ph[n >> 1][(n & 1) * 2 + 1], pl[n >> 1][(n & 1) * 2 + 1]);
        }
        l_run[0] = l_run[0] * c0 + sum0; l_run[1] = l_run[1] * c1 + sum1;      // per-lane partial sums; the quad is added up at the end
        // ---- O = O * c + P V, the product of this tile accumulated from zero, two 8-wide output tiles per ldmatrix
#pragma unroll
        for (uint32_t np = 0; np < NT_O / 2u; ++np) {
            float t0[4] = {0.f, 0.f, 0.f, 0.f}, t1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (uint32_t ks = 0; ks < 2u; ++ks) {
                // B fragments from V [position][dim], transposed on load: matrices (positions 0-7 | 8-15 of the k-step) x (dim chunk 2 np | 2 np + 1)
                const uint32_t r = ks * 16u + (lane & 7u) + ((lane >> 3) & 1u) * 8u, c = 2u * np + (lane >> 4);
                uint32_t b0, b1, b2, b3;
                ac_ldsm4t(ac_smem(v_hi + ac_off(r, c, PITCH)), b0, b1, b2, b3);
                ac_mma(t0, ph[ks][0], ph[ks][1], ph[ks][2], ph[ks][3], b0, b1); ac_mma(t1, ph[ks][0], ph[ks][1], ph[ks][2], ph[ks][3], b2, b3);
                ac_mma(t0, pl[ks][0], pl[ks][1], pl[ks][2], pl[ks][3], b0, b1); ac_mma(t1, pl[ks][0], pl[ks][1], pl[ks][2], pl[ks][3], b2, b3);
                if (!HALF) {
                    ac_ldsm4t(ac_smem(v_lo + ac_off(r, c, PITCH)), b0, b1, b2, b3);
                    ac_mma(t0, ph[ks][0], ph[ks][1], ph[ks][2], ph[ks][3], b0, b1); ac_mma(t1, ph[ks][0], ph[ks][1], ph[ks][2], ph[ks][3], b2, b3);
                }
            }
            o_acc[2 * np][0] = fmaf(o_acc[2 * np][0], c0, t0[0]); o_acc[2 * np][1] = fmaf(o_acc[2 * np][1], c0, t0[1]);
            o_acc[2 * np][2] = fmaf(o_acc[2 * np][2], c1, t0[2]); o_acc[2 * np][3] = fmaf(o_acc[2 * np][3], c1, t0[3]);
            o_acc[2 * np + 1][0] = fmaf(o_acc[2 * np + 1][0], c0, t1[0]); o_acc[2 * np + 1][1] = fmaf(o_acc[2 * np + 1][1], c0, t1[1]);
            o_acc[2 * np + 1][2] = fmaf(o_acc[2 * np + 1][2], c1, t1[2]); o_acc[2 * np + 1][3] = fmaf(o_acc[2 * np + 1][3], c1, t1[3]);
        }
        __syncthreads();          // every warp is done with this buffer set before the next iteration refills it
    }
    // ---- normalise, gate, store (the arithmetic of k_attn_merge: division and sigmoid in double)
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1); l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1); l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const uint32_t r = r_base + (lane >> 2) + half * 8u, z = tok0 + r / G, h = kvh * G + r % G;
        if (z >= ntok) continue;
        const size_t base = ((size_t)z * n_head + h) * HD;
        const double L = (double)l_run[half];
#pragma unroll
        for (uint32_t n = 0; n < NT_O; ++n) {
            const uint32_t d = n * 8u + 2u * (lane & 3u);
            const float2 g = *reinterpret_cast<const float2 *>(gate + base + d);
            const double a0 = (double)o_acc[n][half * 2] / L, a1 = (double)o_acc[n][half * 2 + 1] / L;
            float2 o;
            o.x = (float)(a0 / (1.0 + exp(-(double)g.x))); o.y = (float)(a1 / (1.0 + exp(-(double)g.y)));
            *reinterpret_cast<float2 *>(gated + base + d) = o;
        }
    }
}

template <typename KV>
bool attn_chunk_ok(uint32_t hd, uint32_t G) { return (hd == 64u || hd == 128u || hd == 256u) && (G == 1u || G == 2u || G == 4u || G == 8u || G == 16u); }

template <typename KV, int HD, int G>
static int attn_chunk_launch(const float *query, const KV *kc, const KV *vc, uint32_t n_kv, const uint32_t *pos, uint32_t ntok, float scale, const float *gate, float *gated, cudaStream_t s) {
    constexpr uint32_t nd = sizeof(KV) == 2 ? 1u : 2u;
    const size_t smem = 2u * (size_t)AC_ROWS * HD * 2u + (sizeof(KV) == 2 ? 2u : 1u) * 2u * nd * (size_t)AC_TILE * HD * 2u;
    const uint32_t tpb = AC_ROWS / G;
    const dim3 grid((ntok + tpb - 1u) / tpb, n_kv);
    RC_CUDA(cudaFuncSetAttribute(k_attn_chunk<KV, HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    RC_LAUNCH((k_attn_chunk<KV, HD, G>), grid, AC_THREADS, smem, s, query, kc, vc, n_kv, pos, ntok, scale, gate, gated);
    return 1;
}

// query [ntok][n_kv * G][hd] fp32, K/V cache [position][n_kv][hd], pos[z] = position of token z (increasing); gate as
// query; gated receives out * sigmoid(gate). Returns 0 with an error for shapes that are not built.
template <typename KV>
int launch_attn_chunk(const float *query, const KV *kc, const KV *vc, uint32_t n_kv, uint32_t G, uint32_t hd, const uint32_t *pos, uint32_t ntok, float scale,
                      const float *gate, float *gated, cudaStream_t s) {
    RC_REQUIRE(attn_chunk_ok<KV>(hd, G), "chunk attention: head_dim %u with %u query heads per K/V head is not built", hd, G);
    prof_begin("attn_chunk", s);
    int ok = 0;
#define AC_CASE(HD_, G_) if (hd == HD_ && G == G_) ok = attn_chunk_launch<KV, HD_, G_>(query, kc, vc, n_kv, pos, ntok, scale, gate, gated, s);
#define AC_HD(HD_) AC_CASE(HD_, 1) AC_CASE(HD_, 2) AC_CASE(HD_, 4) AC_CASE(HD_, 8) AC_CASE(HD_, 16)
    AC_HD(64) AC_HD(128) AC_HD(256)
#undef AC_HD
#undef AC_CASE
    prof_end(s);
    if (!ok) return 0;
    RC_LAUNCHED();
    return 1;
}

template int launch_attn_chunk<__half>(const float *, const __half *, const __half *, uint32_t, uint32_t, uint32_t, const uint32_t *, uint32_t, float, const float *, float *, cudaStream_t);
template int launch_attn_chunk<float>(const float *, const float *, const float *, uint32_t, uint32_t, uint32_t, const uint32_t *, uint32_t, float, const float *, float *, cudaStream_t);
template bool attn_chunk_ok<__half>(uint32_t, uint32_t);
template bool attn_chunk_ok<float>(uint32_t, uint32_t);

}  // namespace rc
