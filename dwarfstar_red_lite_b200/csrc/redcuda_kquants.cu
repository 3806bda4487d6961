// Further GGUF block types behind the stage entry points: Q8_0, Q2_K, Q4_K, Q5_K (the reference's
// rl_quant_dequant_row / rl_quant_row_dot cases 8, 10, 12, 13: native/redlite_native_quant_cpu.c:40-128, 198-265).
// Rows stay in their GGUF layout; values are decoded with the reference's float operations in the reference's order
// (explicit round-to-nearest multiplies and subtractions, so that no fused multiply-add changes a bit). These types are
// not on the decode path of the Qwen3-Next model files this library was built for (those use Q6_K / IQ2_XXS / IQ3_S);
// they are served for dequantisation and matrix-vector products, not yet by the engine or the expert kernels.
#include "redcuda_common.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_kquants.cuh"

#include <cuda_fp16.h>

namespace rc {

bool kq_supported(uint32_t t) { return kq_type(t); }
uint64_t kq_row_bytes(uint32_t t, uint32_t ncols) { return ncols % kq_block_values(t) ? 0u : (uint64_t)(ncols / kq_block_values(t)) * kq_block_bytes(t); }

// out[r][c] for GGUF rows; one thread per value
__global__ void __launch_bounds__(256) k_kq_dequant(const uint8_t *__restrict__ rows, uint32_t type, uint64_t row_bytes, uint32_t ncols, uint64_t total, float *__restrict__ out) {
    pdl_prologue();
    const uint32_t bv = kq_block_values(type), bb = kq_block_bytes(type);
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / ncols; const uint32_t c = (uint32_t)(i - r * ncols);
        out[i] = kq_value(type, rows + r * row_bytes + (uint64_t)(c / bv) * bb, c % bv);
    }
}

// out[t][row] = sum_c W[row][c] * x[t][c]; one warp per (row, token), fp32 products and sums
__global__ void __launch_bounds__(256) k_kq_gemv(const uint8_t *__restrict__ w, uint32_t type, uint64_t row_bytes, uint32_t nrows, uint32_t ncols,
                                                 const float *__restrict__ x, uint32_t ntok, float *__restrict__ out) {
    pdl_prologue();
    const uint32_t warp = (blockIdx.x * 256u + threadIdx.x) >> 5, lane = threadIdx.x & 31u;
    if (warp >= nrows * ntok) return;
    const uint32_t row = warp % nrows, t = warp / nrows;
    const uint32_t bv = kq_block_values(type), bb = kq_block_bytes(type);
    const uint8_t *rp = w + (uint64_t)row * row_bytes;
    const float *xr = x + (size_t)t * ncols;
    float acc = 0.f;
    for (uint32_t c = lane; c < ncols; c += 32u) acc = fmaf(kq_value(type, rp + (uint64_t)(c / bv) * bb, c % bv), xr[c], acc);
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[(size_t)t * nrows + row] = acc;
}

int kq_dequant_rows(uint32_t type, const uint8_t *rows, uint32_t nrows, uint32_t ncols, float *out) {
    const uint64_t rb = kq_row_bytes(type, ncols), bytes = rb * nrows;
    RC_REQUIRE(rb, "dequant: %u columns is not a valid row length for type %u", ncols, type);
    const uint64_t n = (uint64_t)nrows * ncols;
    DevMem raw, o;
    if (!raw.alloc(bytes) || !o.alloc(n * 4u)) return 0;
    cudaStream_t s = 0;
    RC_CUDA(cudaMemcpyAsync(raw.p, rows, bytes, cudaMemcpyHostToDevice, s));
    RC_LAUNCH((k_kq_dequant), (unsigned)((n + 255u) / 256u < 4096u ? (n + 255u) / 256u : 4096u), 256, 0, s, raw.as<uint8_t>(), type, rb, ncols, n, o.as<float>());
    RC_LAUNCHED();
    RC_CUDA(cudaMemcpyAsync(out, o.p, n * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    return 1;
}

int kq_matvec(uint32_t type, const uint8_t *w, uint32_t nrows, uint32_t ncols, const float *x, uint32_t ntok, float *out) {
    const uint64_t rb = kq_row_bytes(type, ncols), bytes = rb * nrows;
    RC_REQUIRE(rb, "matvec: %u columns is not a valid row length for type %u", ncols, type);
    RC_REQUIRE((uint64_t)nrows * ntok < (1ull << 26), "matvec: %u rows x %u tokens exceed the grid", nrows, ntok);
    DevMem raw, xd, od;
    if (!raw.alloc(bytes) || !xd.alloc((size_t)ntok * ncols * 4u) || !od.alloc((size_t)ntok * nrows * 4u)) return 0;
    cudaStream_t s = 0;
    RC_CUDA(cudaMemcpyAsync(raw.p, w, bytes, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemcpyAsync(xd.p, x, (size_t)ntok * ncols * 4u, cudaMemcpyHostToDevice, s));
    const uint32_t warps = nrows * ntok;
    RC_LAUNCH((k_kq_gemv), (warps + 7u) / 8u, 256, 0, s, raw.as<uint8_t>(), type, rb, nrows, ncols, xd.as<float>(), ntok, od.as<float>());
    RC_LAUNCHED();
    RC_CUDA(cudaMemcpyAsync(out, od.p, (size_t)ntok * nrows * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    return 1;
}

}  // namespace rc
