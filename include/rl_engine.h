/*
 * rl_engine_* — the persistent Qwen3-Next engine entry points, served by the CUDA backend ("redcuda").
 *
 * This header restates the subset of the reference's engine ABI (native/redlite_native_engine.h:22-209) that the
 * decode path needs, with the same names, argument order, struct layouts and conventions (1 = ok / 0 = failure with
 * the message copied into error[error_cap]; outputs caller-owned; one caller thread; a step returns after the logits
 * are on the host). A program written against the reference header links against libredcuda.so unchanged for these
 * symbols; RL_BACKEND_GPU is the CUDA backend. RL_BACKEND_CPU is not served here (there is no CPU path in this
 * library): calls with it fail with a message.
 *
 * With every routed expert resident in HBM, cfg.cache_mib is accepted and ignored, rl_engine_experts_preloaded()
 * is always 1, and the cache counters of rl_engine_step_stats stay 0 (cache_misses = 0 after open).
 */
#ifndef RL_ENGINE_H
#define RL_ENGINE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rl_engine rl_engine;

typedef enum { RL_BACKEND_CPU = 0, RL_BACKEND_GPU = 1 } rl_engine_backend;     /* redlite_native_engine.h:24-27 */

typedef struct {                                                               /* redlite_native_engine.h:29-40 */
    uint32_t context;        /* KV-cache capacity in positions (0 -> 4096) */
    uint64_t cache_mib;      /* ignored: every expert is resident */
    uint32_t top_k;          /* 0 -> model expert_used_count */
    int enable_cpu;          /* must be 0 */
    int enable_gpu;          /* create the CUDA backend */
    int cpu_threads;         /* ignored */
    uint32_t prefill_batch;  /* tokens per prefill chunk (0 -> default) */
    const char *mtp_path;    /* must be NULL (multi-token prediction is outside this backend) */
} rl_engine_config;

typedef struct {                                                               /* redlite_native_engine.h:42-60 */
    uint32_t n_layer, n_recurrent, n_attention, hidden, vocab, n_expert, top_k, context;
    uint32_t d_conv, d_inner, d_state, n_group, dt_rank, channels, head_v;
    uint32_t n_head, n_head_kv, head_dim, rope_dims;
    float rope_freq_base, rms_eps;
    uint64_t dense_bytes, state_bytes;
} rl_engine_info;

typedef struct {                                                               /* redlite_native_engine.h:62-87 */
    double embed_ms, layers_ms, recurrent_ms, attention_ms, router_ms, routed_ms, shared_ms, output_ms, total_ms;
    double routed_load_ms, routed_gpu_ms, gpu_ms;
    uint64_t expert_loads, cache_hits, cache_misses, ssd_bytes, ssd_reads;
    uint32_t resident_slots, slot_capacity, expert_plans;
    double prep_lru_ms, prep_load_ms, prep_commit_ms, expert_wait_ms, prefetch_ms;
    uint32_t speculative, speculative_fallback;
} rl_engine_step_stats;

#define RL_ENGINE_CACHE_FULL UINT64_MAX
#define RL_ENGINE_MAX_TOPK 64u

void rl_engine_config_default(rl_engine_config *cfg);                                                    /* :89 */
rl_engine *rl_engine_open(const char *model_path, const rl_engine_config *cfg, char *error, size_t error_cap);   /* :91 */
void rl_engine_close(rl_engine *engine);                                                                 /* :92 */
const rl_engine_info *rl_engine_info_get(const rl_engine *engine);                                       /* :94 */
int rl_engine_reset(rl_engine *engine, rl_engine_backend backend, char *error, size_t error_cap);        /* :97 */
uint32_t rl_engine_position(const rl_engine *engine, rl_engine_backend backend);                         /* :99 */
int rl_engine_bench_set_position(rl_engine *engine, rl_engine_backend backend, uint32_t position, char *error, size_t error_cap);   /* :105 */
/* one token at the current position; logits = vocab floats or NULL (skips the LM head)  — :111-112 */
int rl_engine_step(rl_engine *engine, rl_engine_backend backend, uint32_t token, float *logits, rl_engine_step_stats *stats,
                   char *error, size_t error_cap);
/* a token sequence from the current position; logits (may be NULL) are those of the last token — :120-121 */
int rl_engine_prefill(rl_engine *engine, rl_engine_backend backend, const uint32_t *tokens, uint32_t count, float *logits,
                      rl_engine_step_stats *stats, char *error, size_t error_cap);
/* effective prefill chunk: cfg.prefill_batch (capped at 512), or the default of 512; 1 = token by token — :146 */
uint32_t rl_engine_prefill_batch(const rl_engine *engine);
/* host views of the last step's intermediates (hidden floats each; router ids: top_k entries) — :124-129 */
const float *rl_engine_last_embedding(const rl_engine *engine, rl_engine_backend backend);
const float *rl_engine_last_layer_output(const rl_engine *engine, rl_engine_backend backend, uint32_t layer);
const float *rl_engine_last_final_norm(const rl_engine *engine, rl_engine_backend backend);
const uint32_t *rl_engine_last_router_ids(const rl_engine *engine, rl_engine_backend backend, uint32_t layer);
int rl_engine_experts_preloaded(const rl_engine *engine, double *preload_ms);                            /* :132 */
uint64_t rl_engine_full_residency_mib(const rl_engine *engine);                                          /* :144 */
int rl_engine_embed_token(const rl_engine *engine, uint32_t token, float *out, char *error, size_t error_cap);   /* :198 */

/* Not in the reference: greedy decoding without moving the logits to the host. Feeds `token`, then n_new - 1 further
 * steps each fed with the argmax of the previous logits; out_tokens receives the n_new argmax ids. */
int rl_engine_generate_greedy(rl_engine *engine, uint32_t token, uint32_t n_new, uint32_t *out_tokens, rl_engine_step_stats *stats,
                              char *error, size_t error_cap);
/* Not in the reference: HBM bytes one decode step reads/writes at the current position (weights touched + states +
 * KV), for roofline accounting. */
uint64_t rl_engine_step_bytes(const rl_engine *engine);

#ifdef __cplusplus
}
#endif
#endif
