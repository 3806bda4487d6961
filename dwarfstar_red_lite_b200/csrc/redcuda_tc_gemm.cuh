// Tensor-core (tcgen05) GEMM of quantised weight matrices against a chunk of tokens: launch interface (redcuda_tc_gemm.cu)
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rc {

constexpr uint32_t TC_MAX_JOBS = 4u;

struct TcJob {
    const uint8_t *w;        // planar quantised matrix
    uint64_t nb;             // its blocks of 256
    uint32_t type, nrows;
    float *out;              // out[t * out_stride + row]
    uint32_t out_stride;
    uint32_t tile0;          // first 128-row tile of this matrix in grid.x (set by the launcher)
};

struct TcArgs {
    TcJob job[TC_MAX_JOBS];  // matrices that share the input x (same column count)
    uint32_t njobs, ncols, ntok;
    const __half *xs;        // activation digits from launch_tc_prep_x
    const float *x_inv;      // per-token inverse scale from launch_tc_prep_x
    const uint8_t *iq2; const uint32_t *iq3s;
    uint32_t *err;           // device flag: set to 1 when a bounded wait ran out
    uint8_t *wd;             // scratch for the launch's weight digits: tc_wd_bytes(row tiles of the launch, ncols)
    float *w_inv;            // scratch: one float per row tile of the launch
};

// halves of the digit buffer for ntok tokens of ncols columns with token tile tn (x_inv needs ntok rounded up to tn floats)
size_t tc_xs_halves(uint32_t ntok, uint32_t ncols, uint32_t tn);
uint32_t tc_row_tiles(uint32_t nrows);
size_t tc_wd_bytes(uint32_t row_tiles, uint32_t ncols);
uint32_t tc_token_tile(uint32_t ntok, uint32_t row_tiles);     // row_tiles = sum of tc_row_tiles over the launch's matrices
// x2 (may be null): the digits are those of SiLU(x) * x2, both with rows x_stride apart
int launch_tc_prep_x(const float *x, const float *x2, uint32_t x_stride, uint32_t ntok, uint32_t ncols, uint32_t tn, __half *xs, float *x_inv, cudaStream_t s);
int launch_tc_gemm(TcArgs &A, uint32_t tn, const char *tag, cudaStream_t s);   // tn: the tile the digits were prepared with

// ---- routed experts of a prefill chunk on the tensor cores (redcuda_tc_experts.cu) ----
// Nibble-layout IQ2_XXS expert matrices against the pairs grouped by expert. One work item = up to TCX_TN pairs of one
// expert (k_group_pairs cut with item_tok = TCX_TN).
constexpr uint32_t TCX_TN = 64u;
struct TcxArgs {
    const uint8_t *w[2];            // nibble-layout matrices of the shard: (gate, up) or (down, null)
    uint64_t mat_bytes;             // bytes of one expert matrix
    uint32_t nmat, nrows, ncols;    // matrices in this launch (1 or 2), rows / columns of one expert matrix
    uint32_t expert_begin, n_local;
    const uint32_t *sorted, *uexp, *ustart, *item_u, *item_p0, *n_items;    // grouping (k_group_pairs)
    const __half *xd;               // activation digits [row][hi / lo][ncols] from launch_tc_prep_rows
    const float *x_inv;             // per-row inverse scale
    uint32_t x_div;                 // activation row of pair p = p / x_div
    float *out[2];                  // out[m][p * out_stride + row]
    uint32_t out_stride;
    uint32_t *err, *status;         // timeout flag of the launch; sticky status words (may be null)
};
// v[r][k] = b ? SiLU(a[r][k]) * b[r][k] : a[r][k]  ->  fp16 digits xd[r][2][ncols] and x_inv[r]
int launch_tc_prep_rows(const float *a, const float *b, uint32_t stride, uint32_t nrows, uint32_t ncols, __half *xd, float *x_inv, cudaStream_t s);
bool tcx_shape_ok(uint32_t nrows, uint32_t ncols);
int launch_tc_experts(TcxArgs &A, uint32_t max_items, const char *tag, cudaStream_t s);

#ifdef __CUDACC__
// ---- device helpers shared by the tcgen05 kernels ----
constexpr uint32_t TC_M = 128u, TC_KS = 64u, TC_THREADS = 512u, TC_WARPS = TC_THREADS / 32u;
constexpr uint32_t TC_A_DIGIT = TC_M * TC_KS * 2u;            // bytes of one weight digit tile of a stage (16 KB)
constexpr uint32_t TC_SPIN_LIMIT = 4u * 1000u * 1000u;        // polls of ~50 ns: far beyond any legitimate wait

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// shared-memory matrix descriptor: K-major, no swizzle, core matrix = 8 rows x 16 bytes stored as 128 contiguous bytes;
// lbo = byte distance between the two 16-byte k-chunks of one MMA, sbo = byte distance between 8-row groups
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) | ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}

// instruction descriptor, kind::f16: D = f32, A = B = f16, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t tc_idesc(uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((TC_M >> 4) << 24); }

__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(mbar) : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(mbar), "r"(parity) : "memory");
        if (done) return true;
        __nanosleep(32);
    }
    return false;
}
#endif

}  // namespace rc
