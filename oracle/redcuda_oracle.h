/*
 * TEST INFRASTRUCTURE — CPU restatement of the reference's CPU arithmetic for the Qwen3-Next decode hot path.
 *
 * This is the checker the CUDA library is compared with. It is never linked into or loaded by the product
 * library; only the test-suite, the smoke check and the benchmark's CPU-baseline leg use it.
 *
 * Parity pin: every function here is checked in tests/ against the reference's own code compiled unchanged
 * (oracle/_ref/libredlite_ref.so: rl_quant_dequant_row, rl_quant_row_dot, rl_iq3_*,
 * rl_native_router_select_softmax_topk, rl_engine_step on the CPU backend) and against the known-answer vectors of
 * the reference's offline tests. Each function cites the reference file:line it restates.
 *
 * All matrices are row-major "GGUF rows": a row of ncols values is ro_row_bytes(type, ncols) bytes.
 * ggml type ids: 0 F32, 1 F16, 14 Q6_K, 16 IQ2_XXS, 21 IQ3_S.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RO_MAX_TOPK 64u

/* Codebooks are supplied by the caller (the reference keeps them in native/redlite_native_iq2_xxs.c:6-22 and
 * native/redlite_native_iq3_tables.h); the pointers are borrowed and must outlive every later call. */
int ro_set_codebooks(const uint8_t *iq2xxs_grid_2048, const uint32_t *iq3s_grid_512);
/* tables of IQ3_XXS (18), IQ2_S (22) and IQ4_XS (23); the pointers must stay valid */
int ro_set_codebooks_ext(const uint32_t *iq3xxs_grid_256, const uint64_t *iq2s_grid_1024, const int8_t *iq4nl_16);
/* grids of IQ2_XS (17) and IQ1_M (29); the pointers must stay valid */
int ro_set_codebooks_xs(const int8_t *iq2xs_grid_4096, const int8_t *iq1m_grid_16384);

float ro_f16_to_f32(uint16_t h);                                   /* quant_cpu.c:20-38 */
float ro_round_half(float f);                                      /* engine_cpu.c:29-38 */
size_t ro_row_bytes(uint32_t type, uint32_t ncols);
int ro_dequant_row(uint32_t type, const uint8_t *row, uint32_t ncols, float *out);                /* quant_cpu.c:155-196 */
int ro_row_dot(uint32_t type, const uint8_t *row, const float *x, uint32_t ncols, double *out);   /* quant_cpu.c:198-280 */
int ro_row_dot_d(uint32_t type, const uint8_t *row, const double *x, uint32_t ncols, double *out);/* reference.c:82-176, iq3.c:135-148 */
/* out[r] = (float) dot(W[r], x), rows spread over `threads` pthreads (engine_cpu.c:54-92) */
int ro_matvec(uint32_t type, const uint8_t *w, uint32_t nrows, uint32_t ncols, const float *x, float *out, int threads);

/* router (engine_cpu.c:347-355, router_exec.c:102-184) */
int ro_router_logits(const float *w, const float *x, uint32_t n_expert, uint32_t hidden, float *logits);
int ro_router_select(const float *logits, uint32_t n_expert, uint32_t top_k, uint32_t *ids, float *weights, float *probs);

/* routed experts (reference.c:251-382): gate_all/up_all/down_all hold n_expert matrices back to back */
int ro_routed_experts(uint32_t type_gu, uint32_t type_down,
                      const uint8_t *gate_all, const uint8_t *up_all, const uint8_t *down_all,
                      const uint32_t *ids, const float *weights, uint32_t top_k,
                      uint32_t hidden, uint32_t ffn, const float *x, double *out, int threads);

typedef struct {
    uint32_t hidden, n_expert, top_k, ffn, ffn_sh;
    uint32_t type_gu, type_down, type_sh;      /* routed gate/up, routed down, shared expert matrices */
    const float *router;                        /* [n_expert][hidden] */
    const uint8_t *gate_all, *up_all, *down_all;
    const float *sh_gate_inp;                   /* [hidden] */
    const uint8_t *sh_gate, *sh_up, *sh_down;   /* [ffn_sh][hidden], [ffn_sh][hidden], [hidden][ffn_sh] */
} ro_moe_layer;

/* whole MoE FFN of one token: router + routed + sigmoid-gated shared expert (engine_cpu.c:329-386).
 * ids_out/weights_out (top_k entries) and logits_out (n_expert) may be NULL. */
int ro_moe_ffn(const ro_moe_layer *L, const float *x, float *out, uint32_t *ids_out, float *weights_out,
               float *logits_out, int threads);
/* same, with the router matvec replaced by given logits when logits_in is not NULL (drawn-logits workloads) */
int ro_moe_ffn2(const ro_moe_layer *L, const float *x, const float *logits_in, float *out, uint32_t *ids_out, float *weights_out,
                float *logits_out, int threads);

typedef struct {
    uint32_t d_conv, d_state, n_group, dt_rank, d_inner, channels;
    float rms_eps;
    const float *conv_kernel;   /* [channels][d_conv] */
    const float *dt_bias;       /* [dt_rank] */
    const float *ssm_a;         /* [dt_rank] */
    const float *ssm_norm;      /* [d_state] */
} ro_deltanet_params;

/* The part of deltanet_branch between the projections (engine_cpu.c:148-230): beta/gate, causal conv + SiLU,
 * L2-normalised q/k, fp32 gated delta rule on the state in place, gated RMSNorm. conv_state [channels][d_conv-1]
 * and rec_state [dt_rank][d_state][d_state] are updated in place. out_ng: [d_inner]. */
int ro_deltanet_mid(const ro_deltanet_params *P, const float *qkv, const float *z, const float *ba,
                    float *conv_state, float *rec_state, float *out_ng);

/* ---- whole model (engine_cpu.c:390-441) over in-memory tensors ---- */
typedef struct { uint32_t type, nrows, ncols; const uint8_t *data; } ro_tensor;

typedef struct {
    int recurrent;                                   /* 1 DeltaNet, 0 full attention */
    ro_tensor attn_norm, post_norm;
    ro_tensor qkv, z, ba, conv, dt, a, ssm_norm, ssm_out;
    ro_tensor q, k, v, q_norm, k_norm, o;
    ro_tensor router, sh_gate_inp, sh_gate, sh_up, sh_down;
    ro_tensor gate_exps, up_exps, down_exps;         /* nrows = rows per expert, data = expert 0 */
} ro_layer;

typedef struct {
    uint32_t n_layer, hidden, vocab, n_expert, top_k, context;
    uint32_t d_conv, d_inner, d_state, n_group, dt_rank, channels;
    uint32_t n_head, n_head_kv, head_dim, rope_dims;
    float rope_freq_base, rms_eps;
    int kv_f16;                                      /* round K/V rows to fp16 like RL_KV_F16=1 */
    ro_tensor tok_embd, output_norm, output;
    const ro_layer *layers;
} ro_model;

typedef struct ro_state ro_state;
ro_state *ro_state_create(const ro_model *m);
void ro_state_free(ro_state *s);
void ro_state_reset(ro_state *s);
uint32_t ro_state_position(const ro_state *s);
const float *ro_state_layer_out(const ro_state *s, uint32_t layer);
const uint32_t *ro_state_router_ids(const ro_state *s, uint32_t layer);
const float *ro_state_final_norm(const ro_state *s);
const float *ro_state_router_logits(const ro_state *s, uint32_t layer);   /* [n_expert] router logits of the last step */
float *ro_state_rec(ro_state *s, uint32_t recurrent_index);
float *ro_state_conv(ro_state *s, uint32_t recurrent_index);
/* one token; logits (vocab floats) may be NULL */
int ro_model_step(const ro_model *m, ro_state *s, uint32_t token, float *logits, int threads);

#ifdef __cplusplus
}
#endif
