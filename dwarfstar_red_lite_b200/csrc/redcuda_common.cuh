// Shared host-side plumbing of the redcuda library: error reporting, launch accounting, device buffers, codebooks.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <atomic>
#include <string>

#include "redcuda_formats.cuh"

namespace rc {

void set_error(const char *fmt, ...);
extern std::atomic<uint64_t> g_launches;

#define RC_CUDA(expr) do { cudaError_t rc_e_ = (expr); if (rc_e_ != cudaSuccess) { \
    rc::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(rc_e_), __FILE__, __LINE__); return 0; } } while (0)
// after a kernel launch: count it and surface launch-configuration errors at once
#define RC_LAUNCHED() do { rc::g_launches.fetch_add(1, std::memory_order_relaxed); cudaError_t rc_e_ = cudaGetLastError(); \
    if (rc_e_ != cudaSuccess) { rc::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(rc_e_), __FILE__, __LINE__); return 0; } } while (0)
#define RC_REQUIRE(cond, ...) do { if (!(cond)) { rc::set_error(__VA_ARGS__); return 0; } } while (0)

// Optional per-kernel timing: while enabled, every launch site brackets its kernel with a pair of CUDA events on the
// launching stream (not usable while a stream is being captured into a graph).
void prof_begin(const char *tag, cudaStream_t s);
void prof_end(cudaStream_t s);
bool prof_active();

// Sticky status words written by kernels that met data they must not act on (a non-finite router softmax, a token id
// beyond the vocabulary, an expert id outside the shard). They live in mapped pinned host memory: a kernel stores to
// them only in the failing case, and the host reads them after its next synchronisation without a copy. The kernels
// clamp the offending index to a valid one, so nothing is read out of bounds; the synchronous entry points turn a set
// word into an error, as the reference's CPU path does ("invalid router softmax denominator").
enum StatusWord : uint32_t { ST_ROUTER_NONFINITE = 0, ST_TOKEN_RANGE = 1, ST_EXPERT_RANGE = 2, ST_TIMEOUT = 3, ST_WORDS = 4 };
uint32_t *status_words();          // device-visible pointer to ST_WORDS words (nullptr when the allocation failed)
// Reads and clears the words; returns 0 when none was set, else writes a message with set_error and returns 1.
int status_failed();

// Fails (with a message) unless a CUDA device is usable: the library has no CPU path.
int require_device();
// Fails unless the codebooks have been set on the current device.
int require_books(uint32_t ggml_type);
// device pointers of the codebooks on the current device
const uint8_t *books_iq2();
const uint32_t *books_iq3s();

// Programmatic dependent launch: every kernel of the library is launched with the stream-serialisation attribute, so the
// next kernel's blocks are scheduled (and run their prologue up to pdl_prologue's wait) while the previous kernel drains.
// Every kernel calls pdl_prologue() first: it lets its own dependents start launching once all of its blocks have begun,
// then waits until the kernels before it have completed and their writes are visible. RC_PDL=0 launches plainly.
// Programmatic dependent launch: RC_PDL=0 never, RC_PDL=1 every kernel, unset = per source file (RC_PDL_DEFAULT:
// on for the short latency-bound kernels, off for the expert kernels, where early-resident blocks measured slower).
int pdl_mode();
#ifndef RC_PDL_DEFAULT
#define RC_PDL_DEFAULT 1
#endif
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_prologue() {
    asm volatile("griddepcontrol.launch_dependents;" ::);
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <typename K, typename... Args>
inline cudaError_t launch_kernel(int file_default, K kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = (pdl_mode() < 0 ? file_default : pdl_mode()) ? 1 : 0;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}
#define RC_LAUNCH(kernel, grid, block, smem, stream, ...) rc::launch_kernel(RC_PDL_DEFAULT, kernel, dim3(grid), dim3(block), (size_t)(smem), stream, __VA_ARGS__)
#endif

struct DevMem {
    void *p = nullptr; size_t bytes = 0;
    int alloc(size_t n);
    void release();
    ~DevMem() { release(); }
    DevMem() = default;
    DevMem(const DevMem &) = delete;
    DevMem &operator=(const DevMem &) = delete;
    template <class T> T *as() const { return reinterpret_cast<T *>(p); }
};

// A weight matrix resident in HBM in planar layout (F32/F16 matrices stay plain row-major).
struct DMat {
    const uint8_t *base = nullptr;
    uint32_t type = 0, nrows = 0, ncols = 0;
    uint64_t nb = 0;       // blocks of 256 (quantised types)
};

// Upload one matrix of raw GGUF rows (host or device memory) into dst (device, 16-byte aligned, matrix_bytes long)
// and re-lay it out planar. scratch must hold matrix_bytes when the type is quantised and the source is host memory.
int upload_matrix(uint32_t type, uint32_t nrows, uint32_t ncols, const void *src, bool src_on_device, uint8_t *dst,
                  uint8_t *scratch, cudaStream_t stream);

}  // namespace rc
