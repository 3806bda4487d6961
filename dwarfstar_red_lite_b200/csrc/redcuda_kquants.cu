// Further GGUF block types behind the stage entry points: Q8_0, Q2_K, Q4_K, Q5_K (the reference's
// rl_quant_dequant_row / rl_quant_row_dot cases 8, 10, 12, 13: native/redlite_native_quant_cpu.c:40-128, 198-265) and the
// codebook types IQ3_XXS, IQ2_S, IQ4_XS (cases 18, 22, 23 through rl_iq3_group8: native/redlite_native_iq3.c:53-148) and
// IQ2_XS, IQ1_M (17, 29: the weights of rl_native_quant_row_dot, native/redlite_native_reference.c:116-176).
// Rows stay in their GGUF layout; values are decoded with the reference's float operations in the reference's order
// (explicit round-to-nearest multiplies and subtractions, so that no fused multiply-add changes a bit). These types are
// not on the decode path of the Qwen3-Next model files this library was built for (those use Q6_K / IQ2_XXS / IQ3_S);
// they are served for dequantisation and matrix-vector products, not yet by the engine or the expert kernels.
#include "redcuda_common.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_kquants.cuh"
#include "redcuda_kquants_iq.cuh"

#include <cuda_fp16.h>
#include <mutex>

namespace rc {

bool kq_supported(uint32_t t) { return kq_type(t) || kq_iq_type(t); }
static uint32_t kq_any_block_values(uint32_t t) { return kq_iq_type(t) ? 256u : kq_block_values(t); }
static uint32_t kq_any_block_bytes(uint32_t t) { return kq_iq_type(t) ? kq_iq_block_bytes(t) : kq_block_bytes(t); }
uint64_t kq_row_bytes(uint32_t t, uint32_t ncols) { return ncols % kq_any_block_values(t) ? 0u : (uint64_t)(ncols / kq_any_block_values(t)) * kq_any_block_bytes(t); }

// tables of the IQ3-family types, one copy per device (module globals), set by redcuda_set_codebooks_ext
__device__ uint32_t d_iq3xxs_grid[256];
__device__ uint64_t d_iq2s_grid[1024];
__device__ int8_t d_iq4nl[16];
__device__ int8_t d_iq2xs_grid[4096];
__device__ int8_t d_iq1m_grid[16384];
static bool g_iq_tabs_set[64], g_xs_tabs_set[64];
static KqIqTabs g_iq_tabs[64];
static std::mutex g_iq_mu;

int kq_set_iq_tables(const uint32_t *iq3xxs, const uint64_t *iq2s, const int8_t *iq4nl) {
    int dev = 0;
    RC_CUDA(cudaGetDevice(&dev));
    RC_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
    RC_CUDA(cudaMemcpyToSymbol(d_iq3xxs_grid, iq3xxs, sizeof(d_iq3xxs_grid)));
    RC_CUDA(cudaMemcpyToSymbol(d_iq2s_grid, iq2s, sizeof(d_iq2s_grid)));
    RC_CUDA(cudaMemcpyToSymbol(d_iq4nl, iq4nl, sizeof(d_iq4nl)));
    void *a = nullptr, *b = nullptr, *c = nullptr;
    RC_CUDA(cudaGetSymbolAddress(&a, d_iq3xxs_grid));
    RC_CUDA(cudaGetSymbolAddress(&b, d_iq2s_grid));
    RC_CUDA(cudaGetSymbolAddress(&c, d_iq4nl));
    std::lock_guard<std::mutex> lk(g_iq_mu);
    g_iq_tabs[dev].iq3xxs = (const uint32_t *)a; g_iq_tabs[dev].iq2s = (const uint64_t *)b; g_iq_tabs[dev].iq4nl = (const int8_t *)c;
    g_iq_tabs_set[dev] = true;
    return 1;
}
int kq_set_xs_tables(const int8_t *iq2xs, const int8_t *iq1m) {
    int dev = 0;
    RC_CUDA(cudaGetDevice(&dev));
    RC_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
    RC_CUDA(cudaMemcpyToSymbol(d_iq2xs_grid, iq2xs, sizeof(d_iq2xs_grid)));
    RC_CUDA(cudaMemcpyToSymbol(d_iq1m_grid, iq1m, sizeof(d_iq1m_grid)));
    void *a = nullptr, *b = nullptr;
    RC_CUDA(cudaGetSymbolAddress(&a, d_iq2xs_grid));
    RC_CUDA(cudaGetSymbolAddress(&b, d_iq1m_grid));
    std::lock_guard<std::mutex> lk(g_iq_mu);
    g_iq_tabs[dev].iq2xs = (const int8_t *)a; g_iq_tabs[dev].iq1m = (const int8_t *)b;
    g_xs_tabs_set[dev] = true;
    return 1;
}
// the current device's tables; fails (with a message) for an IQ3-family type before they were set
static int kq_tabs_for(uint32_t type, KqIqTabs &T) {
    T = KqIqTabs{nullptr, nullptr, nullptr, nullptr, nullptr};
    if (!kq_iq_type(type)) return 1;
    int dev = 0;
    RC_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_iq_mu);
    RC_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
    if (kq_iq_family3(type)) RC_REQUIRE(g_iq_tabs_set[dev], "type %u needs the IQ3-family tables on device %d: call redcuda_set_codebooks_ext first", type, dev);
    else RC_REQUIRE(g_xs_tabs_set[dev], "type %u needs the IQ2_XS / IQ1_M grids on device %d: call redcuda_set_codebooks_xs first", type, dev);
    T = g_iq_tabs[dev];
    return 1;
}
__device__ __forceinline__ float kq_any_value(uint32_t type, const uint8_t *bp, uint32_t j, const KqIqTabs &T) {
    return kq_iq_type(type) ? kq_iq_value(type, bp, j, T) : kq_value(type, bp, j);
}

// out[r][c] for GGUF rows; one thread per value
__global__ void __launch_bounds__(256) k_kq_dequant(const uint8_t *__restrict__ rows, uint32_t type, uint64_t row_bytes, uint32_t ncols, uint64_t total, KqIqTabs T, float *__restrict__ out) {
    pdl_prologue();
    const uint32_t bv = kq_iq_type(type) ? 256u : kq_block_values(type), bb = kq_iq_type(type) ? kq_iq_block_bytes(type) : kq_block_bytes(type);
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / ncols; const uint32_t c = (uint32_t)(i - r * ncols);
        out[i] = kq_any_value(type, rows + r * row_bytes + (uint64_t)(c / bv) * bb, c % bv, T);
    }
}

// out[t][row] = sum_c W[row][c] * x[t][c]; one warp per (row, token), fp32 products and sums
__global__ void __launch_bounds__(256) k_kq_gemv(const uint8_t *__restrict__ w, uint32_t type, uint64_t row_bytes, uint32_t nrows, uint32_t ncols,
                                                 const float *__restrict__ x, uint32_t ntok, KqIqTabs T, float *__restrict__ out) {
    pdl_prologue();
    const uint32_t warp = (blockIdx.x * 256u + threadIdx.x) >> 5, lane = threadIdx.x & 31u;
    if (warp >= nrows * ntok) return;
    const uint32_t row = warp % nrows, t = warp / nrows;
    const uint32_t bv = kq_iq_type(type) ? 256u : kq_block_values(type), bb = kq_iq_type(type) ? kq_iq_block_bytes(type) : kq_block_bytes(type);
    const uint8_t *rp = w + (uint64_t)row * row_bytes;
    const float *xr = x + (size_t)t * ncols;
    float acc = 0.f;
    for (uint32_t c = lane; c < ncols; c += 32u) acc = fmaf(kq_any_value(type, rp + (uint64_t)(c / bv) * bb, c % bv, T), xr[c], acc);
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[(size_t)t * nrows + row] = acc;
}

int kq_dequant_rows(uint32_t type, const uint8_t *rows, uint32_t nrows, uint32_t ncols, float *out) {
    const uint64_t rb = kq_row_bytes(type, ncols), bytes = rb * nrows;
    RC_REQUIRE(rb, "dequant: %u columns is not a valid row length for type %u", ncols, type);
    const uint64_t n = (uint64_t)nrows * ncols;
    KqIqTabs T;
    if (!kq_tabs_for(type, T)) return 0;
    DevMem raw, o;
    if (!raw.alloc(bytes) || !o.alloc(n * 4u)) return 0;
    cudaStream_t s = 0;
    RC_CUDA(cudaMemcpyAsync(raw.p, rows, bytes, cudaMemcpyHostToDevice, s));
    RC_LAUNCH((k_kq_dequant), (unsigned)((n + 255u) / 256u < 4096u ? (n + 255u) / 256u : 4096u), 256, 0, s, raw.as<uint8_t>(), type, rb, ncols, n, T, o.as<float>());
    RC_LAUNCHED();
    RC_CUDA(cudaMemcpyAsync(out, o.p, n * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    return 1;
}

int kq_matvec(uint32_t type, const uint8_t *w, uint32_t nrows, uint32_t ncols, const float *x, uint32_t ntok, float *out) {
    const uint64_t rb = kq_row_bytes(type, ncols), bytes = rb * nrows;
    RC_REQUIRE(rb, "matvec: %u columns is not a valid row length for type %u", ncols, type);
    RC_REQUIRE((uint64_t)nrows * ntok < (1ull << 26), "matvec: %u rows x %u tokens exceed the grid", nrows, ntok);
    KqIqTabs T;
    if (!kq_tabs_for(type, T)) return 0;
    DevMem raw, xd, od;
    if (!raw.alloc(bytes) || !xd.alloc((size_t)ntok * ncols * 4u) || !od.alloc((size_t)ntok * nrows * 4u)) return 0;
    cudaStream_t s = 0;
    RC_CUDA(cudaMemcpyAsync(raw.p, w, bytes, cudaMemcpyHostToDevice, s));
    RC_CUDA(cudaMemcpyAsync(xd.p, x, (size_t)ntok * ncols * 4u, cudaMemcpyHostToDevice, s));
    const uint32_t warps = nrows * ntok;
    RC_LAUNCH((k_kq_gemv), (warps + 7u) / 8u, 256, 0, s, raw.as<uint8_t>(), type, rb, nrows, ncols, xd.as<float>(), ntok, T, od.as<float>());
    RC_LAUNCHED();
    RC_CUDA(cudaMemcpyAsync(out, od.p, (size_t)ntok * nrows * 4u, cudaMemcpyDeviceToHost, s));
    RC_CUDA(cudaStreamSynchronize(s));
    return 1;
}

}  // namespace rc
