// Launch interface of the integer tensor-core path for IQ2_XXS expert matrices (redcuda_moe_mma.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace rc {

struct MmaArgs {
    const uint8_t *w0, *w1;        // planar IQ2_XXS expert matrices of the shard, back to back (gate/up, or down/nullptr)
    uint64_t mat_bytes, nb;        // bytes and 256-blocks of one expert matrix
    uint32_t nrows, ncols;         // per expert matrix
    uint32_t expert_begin, n_local;  // first expert id of the shard and the number of experts it holds (slot = id - expert_begin)
    uint32_t *status;              // sticky status words (redcuda_common.cuh), may be null
    const uint32_t *sorted, *uexp, *ustart;              // pairs grouped by expert (k_group_pairs)
    const uint32_t *item_u, *item_p0, *n_items;          // work items: expert slot and first pair of up to `TOK` pairs
    const int8_t *xq;              // activation digits [row][3][ncols]; row of pair p = p / x_div
    const float *sx;               // activation scale per row
    uint32_t x_div;
    float *out; uint32_t out_stride;                     // result row of pair p = out + p * out_stride
    const uint2 *lut_grid; const uint4 *lut_sign;        // filled by launch_moe_mma
    uint32_t S, tiles_per_warp, item_tok, item_class;    // filled by launch_moe_mma
    float dw1, dw2;                // weights of digits 1 and 2 (2^bits, 4^bits), filled by launch_moe_mma
    uint32_t *work;                // nibble-layout kernels: the launch's unit counter, zeroed by the grouping kernel
    const float *x_raw;            // nibble-layout gate/up of a single token: its fp32 activation row, quantised inside the kernel (xq / sx unused)
    uint32_t act_bits;             // digit width, filled by the launcher
};

// Builds the magnitude and sign tables of the tensor-core path from the IQ2_XXS codebook (current device).
int mma_set_luts(const uint8_t *iq2_grid_host);
// Width of one balanced activation digit: 8 bits (24-bit fixed point per row, the default) or 7 (RC_ACT_BITS=7, the
// earlier 21-bit form, kept for A/B runs).
uint32_t act_digit_bits();
// x[rows][x_stride] (first ncols of each row) -> digits xq[rows][3][ncols] and scales sx[rows]
int launch_quant_act(const float *x, uint32_t x_stride, uint32_t rows, uint32_t ncols, int8_t *xq, float *sx, cudaStream_t s);
// Pairs one work item of the tensor-core expert kernel covers: 2 in the few-token configuration, 8 for a decode batch,
// 16 when the experts see many pairs each (prefill chunks, expert-parallel shards): an expert's weights are decoded
// once per item, so larger items halve that work where most experts would otherwise need two.
uint32_t mma_item_tokens(bool few_tokens, uint32_t npairs = 0u, uint32_t n_experts = 1u);
// max_items = upper bound of work items (grid.y); item_tok: the size the items were cut with (2, 8 or 16)
int launch_moe_mma(MmaArgs &A, uint32_t max_items, uint32_t item_tok, cudaStream_t s);
// ---- nibble layout of IQ2_XXS expert matrices (redcuda_moe_nib.cu): 138 bytes per 256 weights, table-free decode ----
constexpr uint32_t NIB_BLOCK_BYTES = 138u;
// one record = one 16-row tile x one 256-column block
constexpr uint32_t NIB_SC_OFF = 2048u, NIB_D_OFF = 2176u, NIB_REC = 2208u;
// byte offset of code word (t, kg) of row rr inside a record (16-byte pieces of odd rows pairwise swapped)
__host__ __device__ __forceinline__ uint32_t nib_code_off(uint32_t rr, uint32_t t, uint32_t kg) {
    const uint32_t piece = (2u * t + (kg >> 2)) ^ (rr & 1u);
    return rr * 128u + piece * 16u + (kg & 3u) * 4u;
}
uint64_t nib_matrix_bytes(uint32_t nrows, uint32_t ncols);
bool nib_shape_ok(uint32_t nrows, uint32_t ncols);
// planar IQ2_XXS matrix -> nibble layout (dst: nib_matrix_bytes, 16-byte aligned)
int launch_nib_repack(const uint8_t *planar, uint32_t nrows, uint32_t ncols, uint8_t *dst, cudaStream_t s);
// gate/up (A.w1 set) or down projection of the grouped pairs, work items of at most 8 pairs; persistent kernel
int launch_nib_experts(MmaArgs &A, uint32_t max_items, cudaStream_t s);
// Single token, nibble layout: down projection of the token's top_k experts for one 16-row tile per block, the shared
// expert's down rows, and the tail out = resid + sum_k w_k * expert_k + shared * scalar, in router order — the fusion of
// redmetal_topk_down_tail (native/redmetal_topk.m:254-280). The act rows are quantised inside the kernel.
struct NibTailArgs {
    const uint8_t *w_down; uint64_t mat_bytes;       // nibble-layout down matrices of the shard, bytes of one
    uint32_t nrows, ncols, expert_begin, n_local, top_k;
    const uint32_t *ids; const float *wk;            // the token's experts and router weights [top_k]
    const float *act; uint32_t act_stride;            // act[k][ncols]: SiLU(gate) * up of expert k
    const uint8_t *sh_down; uint64_t sh_nb;           // shared expert's down matrix (planar Q6_K), or null
    const float *sh_act, *scalar, *resid;             // shared activation [ncols], its scalar gate [1], residual [nrows] or null
    float *out;
    float dw1, dw2; uint32_t bits;                    // filled by the launcher
    uint32_t *status;
};
bool nib_tail_ok(uint32_t top_k, uint32_t nrows, uint32_t ncols);
int launch_nib_down_tail(NibTailArgs &A, cudaStream_t s);

#ifdef __CUDACC__
// the three balanced digits of one activation and the row scale: the arithmetic of k_quant_act, shared with the kernels
// that quantise a row themselves
__device__ __forceinline__ float act_qmax(uint32_t bits) { return bits == 8u ? 8355711.0f : 1040000.0f; }    // largest value three digits hold: 127 * (65536 + 256 + 1), or just below 63.5 * 16384
__device__ __forceinline__ float act_scale(float mx, float qmax) { return (mx > 0.f && mx < INFINITY) ? mx / qmax : 1.0f; }
__device__ __forceinline__ void act_digits(float f, float inv, float qmax, uint32_t bits, int &d0, int &d1, int &d2) {
    const int half = 1 << (bits - 1u), mask = (1 << bits) - 1;
    int iv = __float2int_rn(fminf(fmaxf(f * inv, -qmax), qmax));
    d0 = ((iv + half) & mask) - half; iv = (iv - d0) >> bits;
    d1 = ((iv + half) & mask) - half; iv = (iv - d1) >> bits;
    d2 = iv;
}
#endif

// Q6_K matrix (or gate/up pair with SiLU*mul when w1 != nullptr) x ntok activation rows given as digits (redcuda_q6k_mma.cu)
int launch_q6k_mma(const uint8_t *w0, const uint8_t *w1, uint64_t nb, uint32_t nrows, uint32_t ncols, uint32_t ntok,
                   const int8_t *xq, const float *sx, float *out, uint32_t out_stride, const char *tag, cudaStream_t s);

}  // namespace rc
