/*
 * Expert-pool ABI, version 1, of the reference (native/redmetal_topk.h:11-245), served by the CUDA backend.
 *
 * These are the symbols the reference's portable expert runtime links (native/redlite_native_metal.c:63-79, 121, 316,
 * 361, 570, 602, 645). Names, argument order and meaning are the reference's; what was an opaque Metal handle is a
 * CUDA one: `mtl_command_buffer` is a cudaStream_t, `mtl_*_buffer` are device pointers. Functions return 1 on success
 * and 0 on failure (message from redmetal_topk_last_error, per thread), as in native/redmetal_topk.m:56-63.
 *
 * On a B200 every routed expert fits in HBM, so the pool is one resident arena: slot s lives at arena + s * slot_bytes
 * (gate | up | down contiguous, native/redmetal_topk.m:1241-1247), a load is one read + one host-to-device copy, and the
 * bookkeeping that guarded eviction on the Mac (slot generations, in-flight counts, the residency table) is kept as
 * constant-time counters so that the plan / prepare / release logic above it runs unchanged and never finds a miss it
 * has to wait for.
 */
#ifndef REDMETAL_TOPK_H
#define REDMETAL_TOPK_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *redmetal_topk_pool_t;

/* native/redmetal_topk.h:11-12 */
uint32_t redmetal_topk_abi_version(void);
const char *redmetal_topk_last_error(void);

/* native/redmetal_topk.h:14-22. The two grids are the IQ2_XS / IQ1_M codebooks of the reference's expert types; the CUDA
 * backend's expert types (IQ2_XXS 16, Q6_K 14, IQ3_S 21) take their codebooks from redcuda_set_codebooks, so the
 * arguments may be NULL / 0. capacity = budget_bytes / slot_bytes slots. */
redmetal_topk_pool_t redmetal_topk_pool_create(const char *model_path, uint64_t budget_bytes, uint64_t slot_bytes, uint32_t slots_per_slab,
                                               const int8_t *iq2_xs_grid, uint32_t iq2_xs_grid_count, const int8_t *iq1_m_grid, uint32_t iq1_m_grid_count);
void redmetal_topk_pool_destroy(redmetal_topk_pool_t pool);                                                   /* :24 */
/* :27 — slot size classes: accepted when every class fits a slot (one arena of the largest class serves them all) */
int redmetal_topk_pool_set_classes(redmetal_topk_pool_t pool, uint32_t n, const uint64_t *slot_bytes, const uint32_t *capacity);
uint32_t redmetal_topk_pool_capacity(redmetal_topk_pool_t pool);                                             /* :28 */
uint32_t redmetal_topk_pool_slab_count(redmetal_topk_pool_t pool);                                           /* :29 — 1 once the arena exists */
uint64_t redmetal_topk_pool_allocated_bytes(redmetal_topk_pool_t pool);                                      /* :30 */
uint64_t redmetal_topk_pool_bytes_read(redmetal_topk_pool_t pool);                                           /* :31 */
uint64_t redmetal_topk_pool_read_calls(redmetal_topk_pool_t pool);                                           /* :32 */
double redmetal_topk_pool_read_ms(redmetal_topk_pool_t pool);                                                /* :33 */
uint32_t redmetal_topk_pool_slot_generation(redmetal_topk_pool_t pool, uint32_t slot_id);                    /* :35 */
int redmetal_topk_pool_slot_inflight(redmetal_topk_pool_t pool, uint32_t slot_id);                           /* :36 */

/* :38-48 — read the three byte ranges of model_path and copy them into the slot (gate | up | down) */
int redmetal_topk_pool_load_expert(redmetal_topk_pool_t pool, uint32_t slot_id, uint64_t gate_file_offset, uint64_t gate_bytes,
                                   uint64_t up_file_offset, uint64_t up_bytes, uint64_t down_file_offset, uint64_t down_bytes,
                                   uint64_t *bytes_read, double *elapsed_ms);
/* :50-58 — device addresses of the three matrices of a slot */
int redmetal_topk_pool_slot_addresses(redmetal_topk_pool_t pool, uint32_t slot_id, uint64_t gate_bytes, uint64_t up_bytes, uint64_t down_bytes,
                                      uint64_t *gate_address, uint64_t *up_address, uint64_t *down_address);

/* :60-77 — host pointers, synchronous: output[r - row_start] = sum_k w_k * down_k[r] . (SiLU(gate_k x) * (up_k x)) for the
 * output rows [row_start, row_start + row_count). ggml_type: gate/up type in bits 0-7, down type in bits 8-15 when it
 * differs (native/redlite_native_metal.h:69-73); types 16, 14 and 21. */
int redmetal_topk_pool_execute(redmetal_topk_pool_t pool, const uint32_t *slot_ids, const uint64_t *gate_bytes, const uint64_t *up_bytes,
                               const uint64_t *down_bytes, const float *router_weights, uint32_t top_k, uint32_t ggml_type, uint32_t hidden_size,
                               uint32_t ffn_size, uint32_t output_row_start, uint32_t output_row_count, const float *input, uint32_t input_count,
                               float *output, uint32_t output_count, double *elapsed_ms);

/* :86-103 — the same work queued on a stream (mtl_command_buffer = cudaStream_t, the two buffers = device pointers, offsets
 * in bytes); marks the slots in flight until redmetal_topk_pool_release. */
int redmetal_topk_pool_encode(redmetal_topk_pool_t pool, void *mtl_command_buffer, const uint32_t *slot_ids, const uint64_t *gate_bytes,
                              const uint64_t *up_bytes, const uint64_t *down_bytes, const float *router_weights, uint32_t top_k, uint32_t ggml_type,
                              uint32_t hidden_size, uint32_t ffn_size, uint32_t output_row_start, uint32_t output_row_count, void *mtl_input_buffer,
                              uint64_t input_offset, void *mtl_output_buffer, uint64_t output_offset);
void redmetal_topk_pool_release(redmetal_topk_pool_t pool, const uint32_t *slot_ids, uint32_t top_k);       /* :105 */

/* :112-116 — table of layers x experts slot addresses (0 = not resident) in device memory, kept for GPU-side routing */
int redmetal_topk_pool_residency_table_init(redmetal_topk_pool_t pool, uint32_t layers, uint32_t experts);
void *redmetal_topk_pool_residency_table(redmetal_topk_pool_t pool);      /* device pointer, uint64_t[layers][experts] */
int redmetal_topk_pool_residency_set(redmetal_topk_pool_t pool, uint32_t layer, uint32_t expert, uint32_t slot_id);
void redmetal_topk_pool_residency_clear(redmetal_topk_pool_t pool, uint32_t layer, uint32_t expert);
int redmetal_topk_pool_allocate_all(redmetal_topk_pool_t pool);           /* :121 — create the arena now */

#ifdef __cplusplus
}
#endif
#endif
