// Launch-level interfaces shared between the translation units of the redcuda library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace rc {

enum GemvEpilogue : uint32_t {
    GEMV_STORE = 0,       // out[t][row] = W0[row] . x[t]
    GEMV_PAIR_SILU = 1,   // out[t][row] = SiLU(W0[row] . x[t]) * (W1[row] . x[t])   (gate/up pair of an FFN)
    GEMV_SIGMOID = 2,     // out[t][row] = sigmoid(W0[row] . x[t])                    (shared-expert scalar gate)
};

struct GemvJob {
    const uint8_t *w0, *w1;
    float *out;
    uint64_t nb;
    uint32_t type, nrows, ncols, out_stride, epi;
    uint32_t tile_begin, rows_per_tile;     // filled by launch_gemv
};

// Where a single token's selection is also written as the (trivial) expert grouping the expert kernels read: every
// selected expert is distinct, so pair k is its own group and its own work item.
struct RouteGroup1 { uint32_t *sorted, *uexp, *ustart, *n_unique, *item_u, *item_p0, *n_items, *ids_mirror, *work; };   // work (may be null): two unit counters to zero
// Optional tail of a single-token GEMV launch: the block that finishes last (an atomic ticket) also runs the router's
// softmax / top-k over the logits the launch produced, so the selection costs no launch of its own.
struct RouteTail {
    uint32_t *ticket;          // null = no tail; zero before the launch, left at zero by the last block
    const float *logits;
    uint32_t n_expert, top_k;
    uint32_t *ids; float *weights;
    RouteGroup1 G;
    uint32_t *status;
};

#define RC_MAX_JOBS 6u
struct GemvArgs {
    GemvJob job[RC_MAX_JOBS];
    uint32_t njobs, ntok;
    const float *x;            // [ntok][x_stride] device
    uint32_t x_stride;
    const uint8_t *iq2;        // filled by launch_gemv
    const uint32_t *iq3s;
    const char *tag;           // name under which the launch is timed when profiling is on (host side only)
    RouteTail tail;
};

int launch_gemv(GemvArgs &A, cudaStream_t stream);
// group1 (ntok == 1 only, may be null): fill the grouping arrays in the same kernel; ids_mirror (may be null) gets a copy of the ids
int launch_route(const float *logits_dev, uint32_t ntok, uint32_t n_expert, uint32_t top_k, uint32_t *ids_dev, float *weights_dev,
                 float *probs_dev, cudaStream_t stream, const RouteGroup1 *group1 = nullptr);

// Gated DeltaNet step between the projections (redcuda_deltanet.cu). All pointers are device memory; qk, v, beta,
// gate, core are scratch of batch * {2*groups*S, d_inner, rank, rank, d_inner} floats.
struct DnDims { uint32_t d_conv, S, groups, rank, d_inner, channels; float eps; };
int launch_deltanet(const DnDims &D, uint32_t batch, const float *conv_kernel, const float *dt_bias, const float *ssm_a, const float *norm_w,
                    const float *qkv, const float *z, const float *ba, float *conv_state, float *rec_state,
                    float *qk, float *v, float *beta, float *gate, float *core, float *out, cudaStream_t s);
// T consecutive tokens of one sequence (prefill chunk): rows of qkv / z / ba / out and of the scratch are per token;
// pairdots: scratch of T * groups * 4 floats (null: the recurrence runs token by token)
int launch_deltanet_seq(const DnDims &D, uint32_t T, const float *conv_kernel, const float *dt_bias, const float *ssm_a, const float *norm_w,
                    const float *qkv, const float *z, const float *ba, float *conv_state, float *rec_state,
                    float *qk, float *v, float *beta, float *gate, float *core, float *out, float *pairdots, cudaStream_t s);

// Cross-GPU flags of the peer-memory exchange (redcuda_ep.cu): a flag word holds the sequence number of the last step its
// writer completed. ep_wait_flag spins (system-scope acquire loads, at most EP_WAIT_NS) until *flag has reached seq;
// on a timeout, or when an earlier wait already failed (*dead != 0), it returns false at once, sets *dead and the sticky
// ST_TIMEOUT status word.
struct EpWait { const uint32_t *flags; uint32_t n, seq; uint32_t *dead, *status; };     // flags[i * 32] for i < n; flags == nullptr: no wait
constexpr uint32_t EP_MAX_WORLD = 8u;
// The exchange areas of every rank (this rank's own included) as mapped into this process, all with the same layout.
struct EpPeers { uint8_t *base[EP_MAX_WORLD]; uint32_t world, rank; };
// Where the combine of the all-gather form delivers: token t's partial row goes to its owner's slot
// base[t / tokens] + off_part + ((rank * tokens + t % tokens) * hidden) * 4, and when every block has written, the flag word
// base[p] + off_flag + rank * 128 of every rank p is set to seq. ticket: a zeroed device word, left at zero.
struct EpPush { EpPeers peers; size_t off_part, off_flag; uint32_t tokens, seq; uint32_t *ticket; };
#ifdef __CUDACC__
// after a block's stores to peer memory: the last block of the grid (by ticket) publishes seq to every rank
__device__ __forceinline__ void ep_signal_all(const EpPeers &P, size_t off_flag, uint32_t seq, uint32_t *ticket, uint32_t nblocks) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(ticket, 1u) == nblocks - 1u) {
            *ticket = 0u;
            __threadfence_system();
            for (uint32_t p = 0; p < P.world; ++p)
                asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(P.base[p] + off_flag + (size_t)P.rank * 128u), "r"(seq) : "memory");
        }
    }
}
#endif
#ifdef __CUDACC__
constexpr unsigned long long EP_WAIT_NS = 2000000000ull;
__device__ __forceinline__ bool ep_wait_flag(const uint32_t *flag, uint32_t seq, uint32_t *dead, uint32_t *status) {
    if (*reinterpret_cast<volatile uint32_t *>(dead)) return false;
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if ((int32_t)(v - seq) >= 0) return true;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 > EP_WAIT_NS) break;
        __nanosleep(64);
    }
    *reinterpret_cast<volatile uint32_t *>(dead) = 1u;
    if (status) status[3] = 1u;       // ST_TIMEOUT
    return false;
}
// the first W.n threads of a block wait for one flag each; every thread of the block must call it
__device__ __forceinline__ void ep_wait_all(const EpWait &W) {
    if (!W.flags) return;
    if (threadIdx.x < W.n) ep_wait_flag(W.flags + threadIdx.x * 32u, W.seq, W.dead, W.status);
    __syncthreads();
}
#endif

// Causal attention of a prefill chunk on the tensor cores (redcuda_attn_chunk.cu); KV = __half or float
template <typename KV> bool attn_chunk_ok(uint32_t hd, uint32_t G);
template <typename KV>
int launch_attn_chunk(const float *query, const KV *kc, const KV *vc, uint32_t n_kv, uint32_t G, uint32_t hd, const uint32_t *pos, uint32_t ntok, float scale,
                      const float *gate, float *gated, cudaStream_t s);

// Q8_0 / Q2_K / Q4_K / Q5_K rows in their GGUF layout (redcuda_kquants.cu): host-pointer dequantisation and matvec
bool kq_supported(uint32_t ggml_type);
int kq_set_iq_tables(const uint32_t *iq3xxs_grid_256, const uint64_t *iq2s_grid_1024, const int8_t *iq4nl_16);     // current device
int kq_set_xs_tables(const int8_t *iq2xs_grid_4096, const int8_t *iq1m_grid_16384);                                 // current device
int kq_dequant_rows(uint32_t type, const uint8_t *rows, uint32_t nrows, uint32_t ncols, float *out);
int kq_matvec(uint32_t type, const uint8_t *w, uint32_t nrows, uint32_t ncols, const float *x, uint32_t ntok, float *out);

int launch_vec_sigmoid(const float *w, const float *x, uint32_t x_stride, uint32_t ncols, uint32_t ntok, float *out, cudaStream_t stream);
// logits[t][e] = dot(w[e], x[t]) accumulated in double, F32 weights [n_expert][ncols]; for batches (tiled fp64 GEMM)
int launch_router_logits(const float *w, const float *x, uint32_t x_stride, uint32_t ntok, uint32_t n_expert, uint32_t ncols, float *logits, cudaStream_t stream);

}  // namespace rc
