// Batched GEMM descriptors of Muon's Newton-Schulz chain (shared by muon.cu and the
// GEMM kernels).  One launch runs the same contraction for every matrix of the optimizer:
// a tile list (problem, m0, n0) is walked by a persistent grid.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "vb_internal.h"

namespace vb {

// The f32-accurate tensor-core path holds every operand as two f16 planes of the value
// scaled by 2^15 (see ns_gemm_tc.cu); the 16-bit words travel in the same buffers and tensor
// maps as the bf16 operands of the plain path.
constexpr float kSplitScale = 32768.0f;            // 2^15
constexpr float kSplitInvScale = 1.0f / 32768.0f;  // 2^-15
constexpr int kSplitPlanes = 2;
constexpr int kSplitTerms = 3;  // plane products per product

#ifdef __CUDACC__
__device__ __forceinline__ float f16_bits_to_float(uint32_t bits16)
{
    return __half2float(__ushort_as_half((unsigned short)bits16));
}
// Exponent e <= 0 of the power of two that bounds every Newton-Schulz iterate of a matrix whose
// update has the sequential sum of squares `sumsq`: the normalised update x = u / sqrt(sumsq + 1e-8)
// has Frobenius norm phi <= 1, every singular value of an iterate is at most min(1, 1.5^it phi)
// (sigma' = 1.5 sigma - 0.5 sigma^3), and 8 phi covers five iterations.  X is then held scaled by
// 2^(15 - e) and the Gram by 2^(15 - 2e), which keeps both planes in the normal f16 range also for
// updates far smaller than sqrt(1e-8).  e = 0 whenever phi >= 1/16, i.e. for every update whose
// norm is not dwarfed by the 1e-8 under the root.  Same inputs, same result, wherever it is called.
__device__ __forceinline__ int split_exponent(float sumsq)
{
    const float root = __fsqrt_rn(sumsq);
    const float norm = __fsqrt_rn(__fadd_rn(sumsq, 1e-8f));
    const float phi = norm > 1e-8f ? __fdiv_rn(root, norm) : root;
    const float b = fminf(1.0f, 8.0f * phi);
    if (!(b > 0.0f)) return -40;
    int ex;
    (void)frexpf(b, &ex);  // b = m * 2^ex with m in [0.5, 1): b < 2^ex
    return ex > 0 ? 0 : (ex < -40 ? -40 : ex);
}
// scaled value -> its two f16 planes: h0 = f16(xs), h1 = f16(xs - h0) (the difference is exact)
__device__ __forceinline__ void split_f16(float xs, unsigned short &h0, unsigned short &h1)
{
    const __half a = __float2half_rn(xs);
    const __half b = __float2half_rn(xs - __half2float(a));
    h0 = __half_as_ushort(a);
    h1 = __half_as_ushort(b);
}
#endif

enum GemmTileFlags {
    GEMM_TILE_MIRROR = 1,  // symmetric output: also store this tile transposed
    GEMM_TILE_B_IS_A = 2,  // diagonal tile of X^T X (or X X^T): the rows of B are the rows of A, staged once
    // 256 x 512 tiles (two 256-column halves at n0 and n0 + 256):
    GEMM_TILE_SINGLE = 4,     // only the first half exists
    GEMM_TILE_SYMMETRIC = 8   // tile of a symmetric product on or above the diagonal: a half right of the diagonal
                              // is also stored transposed, the half on the diagonal reads A's rows as its B
};

struct GemmTile {
    int32_t problem;
    int32_t m0;
    int32_t n0;
    int32_t flags;
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

enum TcEpilogue {
    TC_EPI_THREE_I_MINUS = 0,  // D = 3I - acc
    TC_EPI_HALF = 1,           // D = 0.5 acc
    TC_EPI_IDENTITY = 2,       // D = acc
    TC_EPI_NS_COMBINE = 3      // D = 1.5 X - 0.5 acc, X read from in_bf16 at the output position
};

// How an operand of the tensor-core GEMM is laid out in memory and fetched by TMA.
enum TcOperandMode {
    TC_OP_K_MAJOR = 0,   // row-major [rows][k]: rows indexed by m (or n)
    TC_OP_MN_BOXES = 1,  // row-major [k][rows]: rows indexed by k ("MN-major"), fetched as 64 x 64 boxes
    TC_OP_MN_3D = 2      // the same, fetched through a 3-D view (row length a multiple of 64)
};

// D[M,N] = epilogue( sum_k A[m,k] * B[n,k] ) on the tensor cores, bf16 operands.
// Each operand is a row-major bf16 matrix described by a TMA tensor map built for its mode.
struct alignas(128) TcGemmProblem {
    CUtensorMap map_a;
    CUtensorMap map_b;
    int32_t M, N, K;
    int32_t a_mode, b_mode;  // TcOperandMode
    int32_t epilogue;
    int32_t ld_out;
    int32_t tensor;          // index into the optimizer's gradient-presence bytes
    int32_t withhold_loads;  // test hook: the producer stages nothing, so the consumers' bounded waits expire
    int32_t transpose_out;   // plain kernel: D[m][n] is stored at out[n * ld_out + m] (the output matrix is D^T)
    int32_t n_terms;         // 1: plain bf16 operands; 3: operands held as two f16 planes (f32-accurate)
    int32_t n_out_planes;    // planes written to out_bf16: 1 (bf16 rounding) or 3 (split)
    int64_t out_plane_stride;  // elements between output planes
    const float *split_sumsq;      // split kernel, update problems: the matrix's sum of squares (see split_exponent)
    const float *scale_sumsq;      // if set: the accumulator is scaled by s^scale_power, s = 1/sqrt(*scale_sumsq + 1e-8)
                                   // (the Frobenius normalisation of muon.rs:59-64 folded into the first iteration)
    int32_t scale_power;           // 1 or 2
    float extra_scale;             // plain kernel: a further factor on the accumulator (0 = none)
    const __nv_bfloat16 *in_bf16;  // TC_EPI_NS_COMBINE only: planes of X (same ld and plane stride as the output)
    __nv_bfloat16 *out_bf16; // may be null
    // plain kernel, TC_EPI_THREE_I_MINUS only: if set, the scaled accumulator itself (G, where out_bf16
    // receives 3I - G), same leading dimension
    __nv_bfloat16 *out2_bf16;
    float *out_f32;          // may be null
    // Launches with TcApplyArgs::enabled: the weights of this matrix (row-major, ld_out) and the
    // arena position of their first element; the epilogue applies the update to them in place.
    float *apply_w;
    int64_t apply_arena_pos;
};

// The last update launch of a step can apply its result instead of (or besides) storing it:
//     w -= (lr * u) * 0.1                                            (src/nn/optim/muon.rs:158-160)
// with u the f32 value the epilogue would have written, so the weights are those the separate
// apply kernel computes, bit for bit.  With peer arenas in `pt` the new weights (and their bf16
// copies) are also stored into every peer, as that kernel does.
struct TcApplyArgs {
    int enabled;      // 0: an ordinary launch
    int keep_update;  // also store the f32 update (for vb_muon_download_update)
    float lr;
    PeerTable pt;
};

// wait_limit: mbarrier polls before a role gives up (0 = the default, about a second).
int launch_ns_gemm_tc(const TcGemmProblem *d_problems, const GemmTile *d_tiles, int n_tiles,
                      const uint8_t *d_present, int *d_error_flag, int sm_count, cudaStream_t stream,
                      uint32_t wait_limit = 0, bool split = false, const TcApplyArgs *apply = nullptr, bool wide = false,
                      bool dual = false);  // dual: the launch's 3I - G problems also store G (out2_bf16)
void tc_gemm_tile_shape(int *bm, int *bn);
int tc_gemm_wide_cols();       // columns of the wide tile (512) of the update products, 0 if not in use
int tc_gemm_wide_gram_cols();  // the same for the Gram products
int make_bf16_tensor_map(void *map_out, const void *base, int64_t inner, int64_t outer, int mode, int planes = 1,
                         int64_t plane_stride = 0);
int tc_mn_major_mode(int64_t inner);

int launch_ns_gemm_f32(const F32GemmProblem *d_problems, const GemmTile *d_tiles, int n_tiles,
                       const uint8_t *d_present, int sm_count, cudaStream_t stream);
void f32_gemm_tile_shape(int *bm, int *bn);

}  // namespace vb
