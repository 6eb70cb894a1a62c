// Batched GEMM descriptors of Muon's Newton-Schulz chain (shared by muon.cu and the
// GEMM kernels).  One launch runs the same contraction for every matrix of the optimizer:
// a tile list (problem, m0, n0) is walked by a persistent grid.
#pragma once

#include "vb_internal.h"

namespace vb {

struct GemmTile {
    int32_t problem;
    int32_t m0;
    int32_t n0;
    int32_t pad;
};

enum F32Epilogue { F32_EPI_NONE = 0, F32_EPI_THREE_I_MINUS = 1, F32_EPI_HALF = 2 };

// C[M,N] = epilogue( A[M,K] * B[K,N] ), row-major C and B.  A is row-major [M,K]
// (trans_a = 0) or stored as [K,M] (trans_a = 1, i.e. A = transpose of a row-major matrix).
struct F32GemmProblem {
    const float *A;
    const float *B;
    float *C;
    int32_t M, N, K;
    int32_t lda, ldb, ldc;
    int32_t trans_a;
    int32_t epilogue;
    int32_t tensor;  // index into the optimizer's gradient-presence bytes
    int32_t pad;
};

int launch_ns_gemm_f32(const F32GemmProblem *d_problems, const GemmTile *d_tiles, int n_tiles,
                       const uint8_t *d_present, int sm_count, cudaStream_t stream);
void f32_gemm_tile_shape(int *bm, int *bn);

}  // namespace vb
