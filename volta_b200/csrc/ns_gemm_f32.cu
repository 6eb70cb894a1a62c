// f32 Newton-Schulz contractions on the CUDA cores (the VB_NS_F32 path of Muon).
//
// The reference forms, per iteration (src/nn/optim/muon.rs:67-100),
//     xt_x = matmul_raw(transpose(X), X)      [cols x cols]
//     C    = 3I - xt_x
//     X    = 0.5 * matmul_raw(X, C)           [rows x cols]
// with matmul_raw = matrixmultiply::sgemm (src/ops/matmul.rs:104-121).  That crate cuts
// the contraction index in blocks of 256, runs one fused-multiply-add chain per output
// element inside a block and adds the block results.  The kernel below keeps exactly
// that summation order (k ascending, fmaf chain per 256-block, blocks added in order),
// so its result does not depend on tiling or thread count.  The transpose is folded into
// the operand addressing; "3I - G" and "* 0.5" are fused into the epilogues.
//
// One launch handles the same contraction of every matrix of the optimizer: the grid
// strides over a tile list (matrix, tile row, tile column).
#include "ns_gemm.h"

namespace vb {

namespace {

constexpr int BM = 128, BN = 128, BK = 16;
constexpr int TM = 8, TN = 8;
constexpr int kThreads = 256;
constexpr int kKBlock = 256;  // matrixmultiply's kc

// As[k][m], Bs[k][n]
struct Smem {
    float a[2][BK][BM];
    float b[2][BK][BN];
};

__device__ __forceinline__ float load_a(const F32GemmProblem &p, int m, int k)
{
    if (m >= p.M || k >= p.K) return 0.0f;
    return p.trans_a ? p.A[(int64_t)k * p.lda + m] : p.A[(int64_t)m * p.lda + k];
}

__device__ __forceinline__ float load_b(const F32GemmProblem &p, int k, int n)
{
    if (n >= p.N || k >= p.K) return 0.0f;
    return p.B[(int64_t)k * p.ldb + n];
}

__device__ __forceinline__ void load_tiles(const F32GemmProblem &p, int m0, int n0, int k0, Smem &s, int buf,
                                           bool fast)
{
    const int tid = threadIdx.x;
    if (fast) {
        // 128 x 16 floats per operand = 512 float4, two per thread
        if (p.trans_a) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int idx = tid + i * kThreads;       // 0..511
                const int k = idx >> 5, m4 = (idx & 31) << 2;
                const float4 v = *reinterpret_cast<const float4 *>(p.A + (int64_t)(k0 + k) * p.lda + m0 + m4);
                *reinterpret_cast<float4 *>(&s.a[buf][k][m4]) = v;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int idx = tid + i * kThreads;
                const int m = idx >> 2, k4 = (idx & 3) << 2;
                const float4 v = *reinterpret_cast<const float4 *>(p.A + (int64_t)(m0 + m) * p.lda + k0 + k4);
                s.a[buf][k4 + 0][m] = v.x;
                s.a[buf][k4 + 1][m] = v.y;
                s.a[buf][k4 + 2][m] = v.z;
                s.a[buf][k4 + 3][m] = v.w;
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + i * kThreads;
            const int k = idx >> 5, n4 = (idx & 31) << 2;
            const float4 v = *reinterpret_cast<const float4 *>(p.B + (int64_t)(k0 + k) * p.ldb + n0 + n4);
            *reinterpret_cast<float4 *>(&s.b[buf][k][n4]) = v;
        }
    } else {
        for (int idx = tid; idx < BK * BM; idx += kThreads) {
            const int k = idx / BM, m = idx % BM;
            s.a[buf][k][m] = load_a(p, m0 + m, k0 + k);
        }
        for (int idx = tid; idx < BK * BN; idx += kThreads) {
            const int k = idx / BN, n = idx % BN;
            s.b[buf][k][n] = load_b(p, k0 + k, n0 + n);
        }
    }
}

__global__ void __launch_bounds__(kThreads)
ns_gemm_f32_kernel(const F32GemmProblem *__restrict__ problems, const GemmTile *__restrict__ tiles, int n_tiles,
                   const uint8_t *__restrict__ present)
{
    __shared__ Smem s;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each an 8 x 8 block of C

    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const GemmTile tile = tiles[t];
        const F32GemmProblem p = problems[tile.problem];
        if (present[p.tensor] == 0) continue;
        const int m0 = tile.m0, n0 = tile.n0;
        const bool aligned = ((p.lda & 3) == 0) && ((p.ldb & 3) == 0) &&
                             ((reinterpret_cast<uintptr_t>(p.A) & 15) == 0) &&
                             ((reinterpret_cast<uintptr_t>(p.B) & 15) == 0);
        const bool full_mn = aligned && (m0 + BM <= p.M) && (n0 + BN <= p.N);

        float total[TM][TN];
        float acc[TM][TN];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) total[i][j] = acc[i][j] = 0.0f;

        const int k_tiles = (p.K + BK - 1) / BK;
        __syncthreads();  // previous tile's readers are done with smem
        load_tiles(p, m0, n0, 0, s, 0, full_mn && BK <= p.K);
        __syncthreads();
        for (int kt = 0; kt < k_tiles; ++kt) {
            const int buf = kt & 1;
            if (kt + 1 < k_tiles)
                load_tiles(p, m0, n0, (kt + 1) * BK, s, buf ^ 1, full_mn && (kt + 2) * BK <= p.K);
            const int k0 = kt * BK;
            // a new 256-block starts: fold the finished chain into the running result
            if (k0 > 0 && (k0 % kKBlock) == 0) {
                const bool first = (k0 == kKBlock);
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) {
                        total[i][j] = first ? acc[i][j] : __fadd_rn(total[i][j], acc[i][j]);
                        acc[i][j] = 0.0f;
                    }
            }
#pragma unroll
            for (int k = 0; k < BK; ++k) {
                float av[TM], bv[TN];
                const float4 a0 = *reinterpret_cast<const float4 *>(&s.a[buf][k][ty * 4]);
                const float4 a1 = *reinterpret_cast<const float4 *>(&s.a[buf][k][64 + ty * 4]);
                const float4 b0 = *reinterpret_cast<const float4 *>(&s.b[buf][k][tx * 4]);
                const float4 b1 = *reinterpret_cast<const float4 *>(&s.b[buf][k][64 + tx * 4]);
                av[0] = a0.x; av[1] = a0.y; av[2] = a0.z; av[3] = a0.w;
                av[4] = a1.x; av[5] = a1.y; av[6] = a1.z; av[7] = a1.w;
                bv[0] = b0.x; bv[1] = b0.y; bv[2] = b0.z; bv[3] = b0.w;
                bv[4] = b1.x; bv[5] = b1.y; bv[6] = b1.z; bv[7] = b1.w;
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) acc[i][j] = __fmaf_rn(av[i], bv[j], acc[i][j]);
            }
            __syncthreads();
        }
        const bool single_block = (p.K <= kKBlock);

        // epilogue
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
            if (m >= p.M) continue;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
                if (n >= p.N) continue;
                // zero-padded k beyond K adds fma(0, 0, acc) = acc: no effect on the chain
                float r = single_block ? acc[i][j] : __fadd_rn(total[i][j], acc[i][j]);
                if (p.K == 0) r = 0.0f;
                if (p.epilogue == F32_EPI_THREE_I_MINUS)
                    r = (m == n) ? __fsub_rn(3.0f, r) : -r;  // muon.rs:76-89
                else if (p.epilogue == F32_EPI_HALF)
                    r = __fmul_rn(r, 0.5f);                  // muon.rs:95-99
                p.C[(int64_t)m * p.ldc + n] = r;
            }
        }
    }
}

}  // namespace

int launch_ns_gemm_f32(const F32GemmProblem *d_problems, const GemmTile *d_tiles, int n_tiles,
                       const uint8_t *d_present, int sm_count, cudaStream_t stream)
{
    if (n_tiles <= 0) return VB_OK;
    int grid = sm_count * 2;
    if (grid > n_tiles) grid = n_tiles;
    ns_gemm_f32_kernel<<<grid, kThreads, 0, stream>>>(d_problems, d_tiles, n_tiles, d_present);
    VB_CUDA(cudaGetLastError());
    return VB_OK;
}

void f32_gemm_tile_shape(int *bm, int *bn)
{
    *bm = BM;
    *bn = BN;
}

}  // namespace vb
