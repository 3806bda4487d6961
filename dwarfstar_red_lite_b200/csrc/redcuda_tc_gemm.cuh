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
};

// halves of the digit buffer for ntok tokens of ncols columns with token tile tn (x_inv needs ntok rounded up to tn floats)
size_t tc_xs_halves(uint32_t ntok, uint32_t ncols, uint32_t tn);
uint32_t tc_row_tiles(uint32_t nrows);
uint32_t tc_token_tile(uint32_t ntok, uint32_t row_tiles);     // row_tiles = sum of tc_row_tiles over the launch's matrices
int launch_tc_prep_x(const float *x, uint32_t x_stride, uint32_t ntok, uint32_t ncols, uint32_t tn, __half *xs, float *x_inv, cudaStream_t s);
int launch_tc_gemm(TcArgs &A, uint32_t tn, const char *tag, cudaStream_t s);   // tn: the tile the digits were prepared with

}  // namespace rc
