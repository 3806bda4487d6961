/*
 * redcuda — C ABI of the B200 (sm_100a) backend for Red Lite's Qwen3-Next decode hot path.
 *
 * Plain C linkage, plain pointers and sizes; no C++ or torch types cross this boundary. Conventions follow the
 * reference (native/redlite_native_engine.h:89-93, native/redmetal_topk.h:13-14): functions return 1 on success and
 * 0 on failure; the message of the last failure on the calling thread is read with redcuda_last_error(). Output
 * buffers are caller-owned. Unless a function says "device", pointers are HOST pointers and the call is synchronous
 * (it returns after the results are in the caller's buffer), like redmetal_topk_pool_execute. "Device" variants take
 * CUDA device pointers and a cudaStream_t passed as void*, return right after the launches, and never allocate.
 *
 * ggml type ids: 0 F32, 1 F16, 14 Q6_K, 16 IQ2_XXS, 21 IQ3_S. Matrices are GGUF rows (row-major, the row length is
 * the input dimension), exactly the bytes of the GGUF tensor; the library re-lays them out in HBM at load.
 *
 * There is no CPU fallback: every entry point fails with a message when no CUDA device is usable.
 */
#ifndef REDCUDA_H
#define REDCUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define REDCUDA_ABI_VERSION 1u
#define REDCUDA_MAX_TOPK 64u          /* RL_ENGINE_MAX_TOPK, native/redlite_native_engine_internal.h:19 */

/* replaces redmetal_topk_abi_version / redmetal_topk_last_error (native/redmetal_topk.h:13-14) */
uint32_t redcuda_abi_version(void);
const char *redcuda_last_error(void);
/* number of usable CUDA devices (0 when none); selects the device for every later call on this thread's objects */
int redcuda_device_count(void);
int redcuda_set_device(int device);

/*
 * Codebooks of the IQ formats, supplied by the host exactly as the reference supplies its grids to the Metal pool
 * (iq2_xs_grid / iq1_m_grid arguments of redmetal_topk_pool_create, native/redmetal_topk.h:16-24):
 * iq2xxs_grid = 256 entries x 8 magnitude bytes (rl_native_iq2_xxs_build_grid, native/redlite_native_iq2_xxs.c:39),
 * iq3s_grid = 512 packed entries (rl_iq3s_grid, native/redlite_native_iq3_tables.h). Must be called once per
 * device before any IQ2_XXS / IQ3_S data is decoded.
 */
int redcuda_set_codebooks(const uint8_t *iq2xxs_grid, uint32_t iq2xxs_bytes, const uint32_t *iq3s_grid, uint32_t iq3s_count);

/*
 * Tables of three further types of the same family (rl_iq3_group8, native/redlite_native_iq3.c:53-110): iq3xxs_grid =
 * 256 packed entries (rl_iq3xxs_grid), iq2s_grid = 1024 packed entries (rl_iq2s_grid), iq4nl_values = 16 values
 * (rl_kvalues_iq4nl), all of native/redlite_native_iq3_tables.h. Once per device before IQ3_XXS (18), IQ2_S (22) or
 * IQ4_XS (23) rows are handed to redcuda_quant_dequant_rows / redcuda_quant_matvec.
 */
int redcuda_set_codebooks_ext(const uint32_t *iq3xxs_grid, uint32_t iq3xxs_count, const uint64_t *iq2s_grid, uint32_t iq2s_count,
                              const int8_t *iq4nl_values, uint32_t iq4nl_count);

/*
 * The two grids the reference hands to its Metal pool (iq2_xs_grid / iq1_m_grid of redmetal_topk_pool_create,
 * native/redmetal_topk.h:16-24; built by rl_native_quant_tables_init, native/redlite_native_tables.c:229): 512 x 8 and
 * 2048 x 8 int8 values (RL_IQ2_XS_GRID_COUNT, RL_IQ1_M_GRID_COUNT). Once per device before IQ2_XS (17) or IQ1_M (29) rows
 * are handed to redcuda_quant_dequant_rows / redcuda_quant_matvec.
 */
int redcuda_set_codebooks_xs(const int8_t *iq2xs_grid, uint32_t iq2xs_count, const int8_t *iq1m_grid, uint32_t iq1m_count);

/* ------------------------------------------------------------------------------------------------------------
 * Stage entry points (host pointers, synchronous). Each replaces one CPU reference function of the path.
 * ---------------------------------------------------------------------------------------------------------- */

/* rl_quant_dequant_row (native/redlite_native_quant_cpu.c:155-196) for nrows rows at once: out[nrows][ncols].
 * ggml types: 0 F32, 1 F16, 14 Q6_K, 16 IQ2_XXS, 21 IQ3_S (the types of the decode path), and 8 Q8_0, 10 Q2_K, 12 Q4_K,
 * 13 Q5_K (cases 8 / 10 / 12 / 13 of the same reference function, :50-128) and 18 IQ3_XXS, 22 IQ2_S, 23 IQ4_XS (its
 * rl_iq3_dequant_row branch, :193; native/redlite_native_iq3.c:53-118), which this entry point and redcuda_quant_matvec
 * serve but the engine and the expert kernels do not yet. Values are bit-identical to the reference's. Also 17 IQ2_XS and
 * 29 IQ1_M, for which the reference has no dequantiser: the value is the weight its row dot forms in double
 * (native/redlite_native_reference.c:116-176), which is exactly a float. */
int redcuda_quant_dequant_rows(uint32_t ggml_type, const uint8_t *rows, uint32_t nrows, uint32_t ncols, float *out);

/* The same values through the layout the routed IQ2_XXS experts are kept in (4-bit magnitude/sign codes, byte scales;
 * dwarfstar_red_lite_b200/csrc/redcuda_moe_nib.cu): raw IQ2_XXS GGUF rows -> that layout -> fp32. The re-coding must not
 * change a single value: out equals redcuda_quant_dequant_rows(16, ...) and rl_quant_dequant_row
 * (native/redlite_native_quant_cpu.c:166-191) bit for bit. nrows a multiple of 16, ncols one of 256 / 512 / 1024 / 2048. */
int redcuda_nib_dequant_rows(const uint8_t *rows, uint32_t nrows, uint32_t ncols, float *out);

/* rl_quant_row_dot over every row and ntok input vectors (native/redlite_native_quant_cpu.c:198-280; the row-parallel
 * matvec of native/redlite_native_engine_cpu.c:54-92): out[t][r] = dot(W[r], x[t]). x[ntok][ncols], out[ntok][nrows]. */
int redcuda_quant_matvec(uint32_t ggml_type, const uint8_t *w, uint32_t nrows, uint32_t ncols,
                         const float *x, uint32_t ntok, float *out);

/* The same contract as redcuda_quant_matvec for a chunk of tokens, computed on the tcgen05 tensor cores (block-quantised
 * types only, ncols a multiple of 256): weights and activations are split into two fp16 digits each, products are
 * accumulated in fp32 in tensor memory. This is the prefill form of the projections; the reference's counterpart is the
 * dequantise + f32 GEMM pair of its batched prefill (native/redmetal_engine_prefill.m:205-227, 889-909). */
int redcuda_quant_matmul_tc(uint32_t ggml_type, const uint8_t *w, uint32_t nrows, uint32_t ncols,
                            const float *x, uint32_t ntok, float *out);

/* rl_native_router_select_softmax_topk (native/redlite_native_router_exec.c:102-184) for ntok rows of logits:
 * ids[ntok][top_k], weights[ntok][top_k] (renormalised over the selection), probs[ntok][n_expert] (may be NULL).
 * Ties go to the lower expert id. */
int redcuda_router_select_softmax_topk(const float *logits, uint32_t ntok, uint32_t n_expert, uint32_t top_k,
                                       uint32_t *ids, float *weights, float *probs);

/* Gated DeltaNet decode step between the projections, for `batch` independent sequences
 * (deltanet_branch, native/redlite_native_engine_cpu.c:148-230; stage tools native/redmetal_deltanet_state.m,
 * native/redmetal_deltanet_tail.m). Per sequence: qkv[channels], z[d_inner], ba[2*dt_rank] in,
 * conv_state[channels][d_conv-1] and rec_state[dt_rank][d_state][d_state] updated in place, out[d_inner]. */
typedef struct {
    uint32_t d_conv, d_state, n_group, dt_rank, d_inner, channels;
    float rms_eps;
    const float *conv_kernel;   /* [channels][d_conv] */
    const float *dt_bias;       /* [dt_rank] */
    const float *ssm_a;         /* [dt_rank] */
    const float *ssm_norm;      /* [d_state] */
} redcuda_deltanet_params;
int redcuda_deltanet_step(const redcuda_deltanet_params *p, uint32_t batch, const float *qkv, const float *z, const float *ba,
                          float *conv_state, float *rec_state, float *out);

/* No counterpart in the reference. The same DeltaNet step for callers that must not allocate device memory at call
 * time: a serving loop with a latency budget (cudaMalloc / cudaFree stall the whole device), or a process in which
 * another runtime owns the device's memory budget and hands this library only the buffers it passes in. Every pointer
 * — the four arrays inside *p included — is DEVICE memory; the launches go to `stream` (cudaStream_t) and the call
 * returns without synchronising. The scratch between the kernels is a fixed array of 131,072 floats (512 KiB) inside
 * the library image, held by every GPU that loads the library until the process exits. A call needs
 * batch * (2 * n_group * d_state + 2 * d_inner + 2 * dt_rank) of them: 12,352 per sequence at the Qwen3-Next shape
 * (16 key / 32 value heads of 128), i.e. at most batch 10 there; larger requests fail with a message and launch
 * nothing. The call never calls cudaMalloc, cudaFree or any allocating routine. The first call on a device looks up
 * the array's device address (once, cached): make that first call before any stream capture begins. All calls share
 * the one array: two calls whose kernels overlap on the GPU (different streams, no ordering) race on it. Nothing in it
 * needs clearing between calls — each call overwrites every value it later reads. */
int redcuda_deltanet_step_noalloc(const redcuda_deltanet_params *p_device_arrays, uint32_t batch, const float *qkv_dev, const float *z_dev,
                                  const float *ba_dev, float *conv_state_dev, float *rec_state_dev, float *out_dev, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Resident MoE layer: router + routed experts + sigmoid-gated shared expert of one layer, every expert in HBM.
 * Replaces ffn() of native/redlite_native_engine_cpu.c:329-386 and, on the GPU side, the expert pool with its LRU
 * (native/redmetal_topk.h, native/redlite_native_cache.h): with every expert resident, residency bookkeeping is a
 * no-op and the expert id is the slot id.
 * ---------------------------------------------------------------------------------------------------------- */
typedef struct redcuda_moe redcuda_moe;

typedef struct {
    uint32_t hidden, n_expert, top_k, ffn, ffn_sh;
    uint32_t type_gu, type_down, type_sh;  /* routed gate/up, routed down, shared-expert matrices */
    uint32_t expert_begin, expert_count;   /* experts held by this object: [expert_begin, expert_begin + expert_count);
                                              (0, n_expert) on one GPU, one shard per rank under expert parallelism */
    uint32_t max_tokens;                   /* largest ntok of a forward call (workspace is sized once, at create) */
    uint32_t weights_on_device;            /* 0: the pointers below are host memory; 1: CUDA device memory */
    const float *router;                   /* [n_expert][hidden] F32 */
    const uint8_t *gate_exps, *up_exps;    /* expert_count matrices [ffn][hidden], back to back (GGUF expert-major) */
    const uint8_t *down_exps;              /* expert_count matrices [hidden][ffn] */
    const float *sh_gate_inp;              /* [hidden] F32 */
    const uint8_t *sh_gate, *sh_up;        /* [ffn_sh][hidden] */
    const uint8_t *sh_down;                /* [hidden][ffn_sh] */
    uint32_t expert_stride;                /* 0 or 1: the shard is the contiguous range above. s > 1: the shard holds experts
                                              expert_begin + i * s, i < expert_count (interleaved placement, which spreads the
                                              hot experts of a skewed routing over the ranks); matrix i belongs to that expert */
} redcuda_moe_desc;

redcuda_moe *redcuda_moe_create(const redcuda_moe_desc *desc);
void redcuda_moe_destroy(redcuda_moe *m);
uint64_t redcuda_moe_resident_bytes(const redcuda_moe *m);

/* Expert parallelism, all-gather form (no reference counterpart: the reference is single-device; the pair layout is its
 * expert_start / pair_token / pair_weight of native/redmetal_topk.h:182-190). Every rank holds every token of the step
 * (x rows x_stride floats apart) with its router ids / weights (rows meta_stride elements apart) and computes
 * out[t] = sum over the pairs of token t whose expert lives on THIS shard of weight * expert(x[t]); pairs of other shards
 * are skipped, a token without local pairs gets zeros. The sum of the ranks' outputs (a reduce-scatter) is the routed
 * part of the layer. Device pointers, asynchronous on `stream`; ntok <= max_tokens. */
int redcuda_moe_partial_device(redcuda_moe *m, uint32_t ntok, const float *x_dev, uint32_t x_stride, const uint32_t *ids_dev,
                               const float *weights_dev, uint32_t meta_stride, float *out_dev, void *stream);

/* The all-gather form of expert parallelism as one host call per layer or per step (redcuda_ep.cu; no reference
 * counterpart). One process per GPU; every rank keeps `tokens` tokens and a shard of every layer's experts (a redcuda_moe
 * created with expert_begin / expert_count / expert_stride and max_tokens >= world * tokens). Rank 0 draws a unique id
 * (128 bytes) and hands it to the other ranks by any means; create is collective (ncclCommInitRank). NCCL is loaded
 * with dlopen("libnccl.so.2") on first use; world = 1 needs none.
 *   layer_forward: out[t] = routed(x[t]) over all ranks' experts + shared(x[t]) * sigmoid(g.x[t]) for the rank's own
 *                  tokens (device pointers [tokens][hidden], asynchronous on `stream`; logits_in_dev may be NULL)
 *   step:          layer_forward for n_layers layers in order; x_dev[l] / out_dev[l] per layer (a caller that chains
 *                  layers passes out_dev[l - 1] as x_dev[l]), logits_in_dev NULL or one pointer (or NULL) per layer
 *   ipc_handle / attach_peers: optional, for ranks that are processes on one node (2 to 8). Every rank exports the CUDA IPC
 *                  handle (64 bytes) of its exchange area; attach_peers takes all ranks' handles in rank order (world x 64
 *                  bytes) and switches the exchange from NCCL to stores into peer memory with flag words (bounded waits:
 *                  a missing rank ends the step with the "timeout" status, not a hang). Ranks must not destroy the
 *                  context while others may still be stepping. */
typedef struct redcuda_ep redcuda_ep;
int redcuda_ep_unique_id(void *out128);
int redcuda_ep_ipc_handle(redcuda_ep *ep, void *out64);
int redcuda_ep_attach_peers(redcuda_ep *ep, const void *handles);
int redcuda_ep_detach_peers(redcuda_ep *ep);      /* back to NCCL; every rank must do the same between steps */
redcuda_ep *redcuda_ep_create(int rank, int world, const void *unique_id128, uint32_t tokens, uint32_t hidden, uint32_t top_k);
void redcuda_ep_destroy(redcuda_ep *ep);
int redcuda_ep_layer_forward(redcuda_ep *ep, redcuda_moe *layer, const float *x_dev, const float *logits_in_dev, float *out_dev, void *stream);
/* The same for ntok <= tokens tokens (the same ntok on every rank) with an optional residual: out = resid + routed + shared.
 * last_ids_device: the router ids [ntok][top_k] of the rank's own tokens from the last call (device memory). */
int redcuda_ep_layer_forward_n(redcuda_ep *ep, redcuda_moe *layer, uint32_t ntok, const float *x_dev, const float *logits_in_dev, const float *resid_dev,
                               float *out_dev, void *stream);
const uint32_t *redcuda_ep_last_ids_device(const redcuda_ep *ep);
/* The engine under expert parallelism (config 4 across GPUs; no reference counterpart): every rank runs its own sequences
 * through its own engine, which holds the dense weights and a contiguous share of every layer's experts.
 * redcuda_engine_shard(rank, world) sets that share for the engines this thread opens next (rank 0 of 1 = everything);
 * redcuda_engine_attach_ep hands the engine an exchange context created with tokens >= the prefill chunk (not owned by the
 * engine; every rank must make the same sequence of prefill / step calls with the same token counts).
 * rl_engine_generate_greedy is refused on a sharded engine. */
struct rl_engine;
int redcuda_engine_shard(int rank, int world);
int redcuda_engine_attach_ep(struct rl_engine *e, redcuda_ep *ep);
int redcuda_ep_step(redcuda_ep *ep, redcuda_moe *const *layers, uint32_t n_layers, const float *const *x_dev, const float *const *logits_in_dev,
                    float *const *out_dev, void *stream);

/* One MoE FFN pass over ntok tokens (host pointers, synchronous): out[t] = routed(x[t]) + shared(x[t]) * sigmoid(g.x[t]).
 * logits_in, when not NULL, replaces the router matvec ([ntok][n_expert], the "drawn logits" of the ragged-batch
 * workload). ids_out [ntok][top_k], weights_out [ntok][top_k], logits_out [ntok][n_expert] may be NULL. */
int redcuda_moe_forward(redcuda_moe *m, uint32_t ntok, const float *x, const float *logits_in, float *out,
                        uint32_t *ids_out, float *weights_out, float *logits_out);

/* Same pass with device pointers on `stream` (cudaStream_t). Never allocates or synchronises, so it can be captured
 * in a CUDA graph. resid_dev, when not NULL, is added to the output (x_out = resid + ffn). */
int redcuda_moe_forward_device(redcuda_moe *m, uint32_t ntok, const float *x_dev, const float *logits_in_dev,
                               const float *resid_dev, float *out_dev, void *stream);

/* Expert-parallel pieces (device pointers, `stream`), the two halves either side of the all-to-all exchange:
 *   route:   ids_dev[ntok][top_k], weights_dev[ntok][top_k] from x_dev (or logits_in_dev)
 *   experts: routed experts of THIS shard over (token, expert) pairs already grouped by the caller:
 *            pair_x_dev[npairs][hidden] activations, pair_expert_dev[npairs] global expert ids (all within the
 *            shard), result pair_out_dev[npairs][hidden] (unweighted expert outputs)
 *   shared:  out_dev[t] = shared(x[t]) * sigmoid(g.x[t]) */
int redcuda_moe_route_device(redcuda_moe *m, uint32_t ntok, const float *x_dev, const float *logits_in_dev,
                             uint32_t *ids_dev, float *weights_dev, void *stream);
int redcuda_moe_experts_device(redcuda_moe *m, uint32_t npairs, const float *pair_x_dev, const uint32_t *pair_expert_dev,
                               float *pair_out_dev, void *stream);
int redcuda_moe_shared_device(redcuda_moe *m, uint32_t ntok, const float *x_dev, float *out_dev, void *stream);
/*   combine: out_dev[t] = resid[t] + add[t] + sum_k weights[t][k] * pair_out[row(t,k)] in router order, the per-token sum of
 *            redmetal_topk_sum_b (native/redmetal_topk.m:626-640); row(t,k) = pair_row_dev[t*top_k+k], or t*top_k+k when
 *            pair_row_dev is NULL; add_dev (the shared-expert part) and resid_dev may be NULL */
int redcuda_moe_combine_device(redcuda_moe *m, uint32_t ntok, const float *pair_out_dev, const uint32_t *pair_row_dev, const float *weights_dev,
                               const float *add_dev, const float *resid_dev, float *out_dev, void *stream);

/* Per-kernel timing for benchmarks: while enabled, every kernel launch is bracketed by CUDA events on its stream
 * (do not enable while capturing a CUDA graph). report() waits for the device and writes one line per kernel name,
 * "name launches total_ms\n", into buf; returns the number of lines. enable(0/1) clears the records. */
int redcuda_profile_enable(int on);
int redcuda_profile_report(char *buf, size_t cap);

/* number of kernel launches the library has issued on this thread's device since load (for bench accounting) */
uint64_t redcuda_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
