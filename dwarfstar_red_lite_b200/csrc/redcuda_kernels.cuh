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
// T consecutive tokens of one sequence (prefill chunk): rows of qkv / z / ba / out and of the scratch are per token
int launch_deltanet_seq(const DnDims &D, uint32_t T, const float *conv_kernel, const float *dt_bias, const float *ssm_a, const float *norm_w,
                    const float *qkv, const float *z, const float *ba, float *conv_state, float *rec_state,
                    float *qk, float *v, float *beta, float *gate, float *core, float *out, cudaStream_t s);

int launch_vec_sigmoid(const float *w, const float *x, uint32_t x_stride, uint32_t ncols, uint32_t ntok, float *out, cudaStream_t stream);
// logits[t][e] = dot(w[e], x[t]) accumulated in double, F32 weights [n_expert][ncols]; for batches (tiled fp64 GEMM)
int launch_router_logits(const float *w, const float *x, uint32_t x_stride, uint32_t ntok, uint32_t n_expert, uint32_t ncols, float *logits, cudaStream_t stream);

}  // namespace rc
