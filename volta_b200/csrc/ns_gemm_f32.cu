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

// Register-staged copy of the next k tile on the aligned interior path: the global loads are
// issued before the multiply-add block of the current tile and written to shared memory
// after it, so their latency overlaps the arithmetic.
struct Staged {
    float4 a[2], b[2];
};

__device__ __forceinline__ void fetch_tiles(const F32GemmProblem &p, int m0, int n0, int k0, Staged &r)
{
    const int tid = threadIdx.x;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int idx = tid + i * kThreads;  // 0..511
        if (p.trans_a) {
            const int k = idx >> 5, m4 = (idx & 31) << 2;
            r.a[i] = __ldg(reinterpret_cast<const float4 *>(p.A + (int64_t)(k0 + k) * p.lda + m0 + m4));
        } else {
            const int m = idx >> 2, k4 = (idx & 3) << 2;
            r.a[i] = __ldg(reinterpret_cast<const float4 *>(p.A + (int64_t)(m0 + m) * p.lda + k0 + k4));
        }
        const int k = idx >> 5, n4 = (idx & 31) << 2;
        r.b[i] = __ldg(reinterpret_cast<const float4 *>(p.B + (int64_t)(k0 + k) * p.ldb + n0 + n4));
    }
}

__device__ __forceinline__ void commit_tiles(const F32GemmProblem &p, const Staged &r, Smem &s, int buf)
{
    const int tid = threadIdx.x;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int idx = tid + i * kThreads;
        if (p.trans_a) {
            const int k = idx >> 5, m4 = (idx & 31) << 2;
            *reinterpret_cast<float4 *>(&s.a[buf][k][m4]) = r.a[i];
        } else {
            const int m = idx >> 2, k4 = (idx & 3) << 2;
            s.a[buf][k4 + 0][m] = r.a[i].x;
            s.a[buf][k4 + 1][m] = r.a[i].y;
            s.a[buf][k4 + 2][m] = r.a[i].z;
            s.a[buf][k4 + 3][m] = r.a[i].w;
        }
        const int k = idx >> 5, n4 = (idx & 31) << 2;
        *reinterpret_cast<float4 *>(&s.b[buf][k][n4]) = r.b[i];
    }
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

// Dynamic shared memory: the staging buffers, then one running total per accumulator and
// thread ([i][j][thread]: conflict free).  The totals live there because they are touched
// once per 256 values of k, while keeping them in registers would halve the occupancy.
constexpr size_t kSmemBytes = sizeof(Smem) + (size_t)TM * TN * kThreads * sizeof(float);

__global__ void __launch_bounds__(kThreads, 2)
ns_gemm_f32_kernel(const F32GemmProblem *__restrict__ problems, const GemmTile *__restrict__ tiles, int n_tiles,
                   const uint8_t *__restrict__ present)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    Smem &s = *reinterpret_cast<Smem *>(smem_raw);
    float *total = reinterpret_cast<float *>(smem_raw + sizeof(Smem)) + threadIdx.x;  // [(i * TN + j) * kThreads]
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

        float acc[TM][TN];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

        const int k_tiles = (p.K + BK - 1) / BK;
        __syncthreads();  // previous tile's readers are done with smem
        load_tiles(p, m0, n0, 0, s, 0, full_mn && BK <= p.K);
        __syncthreads();
        for (int kt = 0; kt < k_tiles; ++kt) {
            const int buf = kt & 1;
            const bool has_next = kt + 1 < k_tiles;
            const bool next_fast = has_next && full_mn && (kt + 2) * BK <= p.K;
            Staged staged;
            if (next_fast) fetch_tiles(p, m0, n0, (kt + 1) * BK, staged);  // lands while this tile is multiplied
            else if (has_next) load_tiles(p, m0, n0, (kt + 1) * BK, s, buf ^ 1, false);
            const int k0 = kt * BK;
            // a new 256-block starts: fold the finished chain into the running result
            if (k0 > 0 && (k0 % kKBlock) == 0) {
                const bool first = (k0 == kKBlock);
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) {
                        float *slot = total + (i * TN + j) * kThreads;
                        *slot = first ? acc[i][j] : __fadd_rn(*slot, acc[i][j]);
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
            if (next_fast) commit_tiles(p, staged, s, buf ^ 1);
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
                float r = single_block ? acc[i][j] : __fadd_rn(total[(i * TN + j) * kThreads], acc[i][j]);
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
    // the attribute is per device; setting it again is cheap next to a launch of this size
    VB_CUDA(cudaFuncSetAttribute(ns_gemm_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    ns_gemm_f32_kernel<<<grid, kThreads, kSmemBytes, stream>>>(d_problems, d_tiles, n_tiles, d_present);
    VB_CUDA(cudaGetLastError());
    return VB_OK;
}

void f32_gemm_tile_shape(int *bm, int *bn)
{
    *bm = BM;
    *bn = BN;
}

}  // namespace vb
