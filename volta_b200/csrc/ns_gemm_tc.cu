// bf16 Newton-Schulz contractions on the 5th-generation tensor cores (sm_100a):
// tcgen05.mma with operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte
// swizzle), f32 accumulators in tensor memory (TMEM), epilogue from TMEM with tcgen05.ld.
//
// Per iteration Muon needs (src/nn/optim/muon.rs:67-100)
//     C  = 3I - X^T X          X' = 0.5 * X C            (rows >= cols), or the equal
//     C  = 3I - X X^T          X' = 0.5 * C X            (rows <  cols: the short-side Gram)
// Both are D[M,N] = sum_k A[m,k] B[n,k] with operands read straight from the row-major X and
// from the symmetric C: an operand whose contraction index is its row index is described to
// the tensor core as "MN-major" (instruction-descriptor transpose bits), so no transposed
// copy of X is ever written.  The polynomial pieces (3I - G, * 0.5, bf16 rounding of the next
// operand, f32 copy of the final update) are fused into the epilogues.
//
// One persistent launch handles one contraction of every matrix: a tile list
// (problem, m0, n0) is walked by 148 CTAs.  Each CTA is warp specialised:
//   warp 0     TMA producer  (kStages-deep ring of {A 128x64, B 256x64} bf16 tiles)
//   warp 1     MMA issuer    (one thread; 4 x tcgen05.mma 128x256x16 per ring slot)
//   warps 2-5  epilogue      (TMEM -> registers -> global), overlapped with the next tile's
//                             main loop through two TMEM accumulator buffers
// Every mbarrier wait is bounded: on expiry the CTA raises an abort flag that all roles
// poll, records an error code for the host, releases its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include <stdlib.h>

#include "ns_gemm.h"

namespace vb {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;            // bf16 elements = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kBoxRows = 64;      // every TMA box is 64 x 64 bf16 = 8 KiB
constexpr int kBoxBytes = kBoxRows * BK * 2;
constexpr int kABytes = BM * BK * 2;                    // 16 KiB
constexpr int kBBytes = BN * BK * 2;                    // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;          // 48 KiB
constexpr int kAccCols = BN;                            // f32 columns per accumulator
constexpr int kTmemCols = 2 * kAccCols;                 // 512: two accumulators
constexpr int kThreads = 192;
constexpr int kEpiWarps = 4;
constexpr uint32_t kWaitLimit = 1u << 22;               // mbarrier polls before giving up

struct alignas(8) Barriers {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort;
};
constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + (size_t)kStages * kStageBytes + sizeof(Barriers);

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if the barrier did not flip in time or another role aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag)
{
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u && *abort_flag != 0u) return false;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format): start address, leading/stride byte offsets
// (all >> 4), version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3fffu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}

// Instruction descriptor for kind::f16 with bf16 operands and f32 accumulation.
__device__ __forceinline__ uint32_t make_idesc(int a_mn_major, int b_mn_major)
{
    uint32_t d = 0;
    d |= 1u << 4;                    // D format: f32
    d |= 1u << 7;                    // A format: bf16
    d |= 1u << 10;                   // B format: bf16
    d |= (uint32_t)(a_mn_major & 1) << 15;
    d |= (uint32_t)(b_mn_major & 1) << 16;
    d |= (uint32_t)(BN >> 3) << 17;  // N
    d |= (uint32_t)(BM >> 4) << 24;  // M
    return d;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b)
{
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

__global__ void __launch_bounds__(kThreads, 1)
ns_gemm_tc_kernel(const TcGemmProblem *__restrict__ problems, const GemmTile *__restrict__ tiles, int n_tiles,
                  const uint8_t *__restrict__ present, int *__restrict__ error_flag)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    Barriers *bars = reinterpret_cast<Barriers *>(smem + (size_t)kStages * kStageBytes);
    volatile uint32_t *abort_flag = &bars->abort;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&bars->tmem_full[a], 1);
            mbar_init(&bars->tmem_empty[a], kEpiWarps);
        }
        bars->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // TMEM allocation is warp-wide
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&bars->tmem_base)),
                     "r"((uint32_t)kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const GemmTile tile = tiles[t];
                const TcGemmProblem *p = problems + tile.problem;
                if (present[p->tensor] == 0) continue;
                const int k_blocks = (p->K + BK - 1) / BK;
                const int a_mn = p->a_mn_major, b_mn = p->b_mn_major;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&bars->empty[stage], phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t *sa = smem + (size_t)stage * kStageBytes;
                    uint8_t *sb = sa + kABytes;
                    mbar_expect_tx(&bars->full[stage], kStageBytes);
                    const int k0 = kb * BK;
#pragma unroll
                    for (int j = 0; j < BM / kBoxRows; ++j) {
                        const int r0 = tile.m0 + j * kBoxRows;
                        if (a_mn) tma_load_2d(sa + j * kBoxBytes, &p->map_a, r0, k0, &bars->full[stage]);
                        else      tma_load_2d(sa + j * kBoxBytes, &p->map_a, k0, r0, &bars->full[stage]);
                    }
#pragma unroll
                    for (int j = 0; j < BN / kBoxRows; ++j) {
                        const int r0 = tile.n0 + j * kBoxRows;
                        if (b_mn) tma_load_2d(sb + j * kBoxBytes, &p->map_b, r0, k0, &bars->full[stage]);
                        else      tma_load_2d(sb + j * kBoxBytes, &p->map_b, k0, r0, &bars->full[stage]);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                bars->abort = 1;
                atomicExch(error_flag, 1);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const GemmTile tile = tiles[t];
                const TcGemmProblem *p = problems + tile.problem;
                if (present[p->tensor] == 0) continue;
                const int k_blocks = (p->K + BK - 1) / BK;
                const int a_mn = p->a_mn_major, b_mn = p->b_mn_major;
                const uint32_t idesc = make_idesc(a_mn, b_mn);
                // the epilogue must have drained this accumulator
                if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * kAccCols);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&bars->full[stage], phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)stage * kStageBytes);
                    const uint32_t sb = sa + kABytes;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        // K-major: 16 bf16 = 32 bytes further along the swizzled 128-byte row.
                        // MN-major: 16 k-rows = two 8-row groups of 1 KiB further down the box.
                        const uint64_t da = a_mn ? make_smem_desc(sa + kk * 2048, kBoxBytes, 1024)
                                                 : make_smem_desc(sa + kk * 32, 16, 1024);
                        const uint64_t db = b_mn ? make_smem_desc(sb + kk * 2048, kBoxBytes, 1024)
                                                 : make_smem_desc(sb + kk * 32, 16, 1024);
                        tcgen05_mma_bf16(tmem_d, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(&bars->empty[stage]);  // slot reusable once these MMAs have read it
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                tcgen05_commit(&bars->tmem_full[acc]);  // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
            if (!ok) {
                bars->abort = 1;
                atomicExch(error_flag, 2);
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int quarter = warp & 3;  // the TMEM lane quarter this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            const GemmTile tile = tiles[t];
            const TcGemmProblem *p = problems + tile.problem;
            if (present[p->tensor] == 0) continue;
            const int M = p->M, N = p->N;
            const int epi = p->epilogue;
            __nv_bfloat16 *out_bf16 = p->out_bf16;
            float *out_f32 = p->out_f32;
            const int64_t ld = p->ld_out;
            if (!mbar_wait(&bars->tmem_full[acc], acc_phase, abort_flag)) {
                ok = false;
                break;
            }
            tcgen05_fence_after();
            const int row = tile.m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * kAccCols);
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; ++cc) {
                const int col0 = tile.n0 + cc * 32;
                if (col0 >= N) break;  // uniform across the warp
                uint32_t v[32];
                tmem_ld_32x32(taddr + (uint32_t)(cc * 32), v);
                tmem_ld_wait();
                if (row < M) {
                    float f[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float a = __uint_as_float(v[j]);
                        if (epi == TC_EPI_THREE_I_MINUS) f[j] = (row == col0 + j) ? 3.0f - a : -a;  // muon.rs:76-89
                        else f[j] = 0.5f * a;                                                       // muon.rs:95-99
                    }
#pragma unroll
                    for (int g8 = 0; g8 < 4; ++g8) {  // groups of 8 columns: N is a multiple of 8
                        const int col = col0 + g8 * 8;
                        if (col >= N) break;
                        if (out_bf16) {
                            uint4 q;
                            q.x = pack_bf16(f[g8 * 8 + 0], f[g8 * 8 + 1]);
                            q.y = pack_bf16(f[g8 * 8 + 2], f[g8 * 8 + 3]);
                            q.z = pack_bf16(f[g8 * 8 + 4], f[g8 * 8 + 5]);
                            q.w = pack_bf16(f[g8 * 8 + 6], f[g8 * 8 + 7]);
                            *reinterpret_cast<uint4 *>(out_bf16 + (int64_t)row * ld + col) = q;
                        }
                        if (out_f32) {
                            float4 *dst = reinterpret_cast<float4 *>(out_f32 + (int64_t)row * ld + col);
                            dst[0] = make_float4(f[g8 * 8 + 0], f[g8 * 8 + 1], f[g8 * 8 + 2], f[g8 * 8 + 3]);
                            dst[1] = make_float4(f[g8 * 8 + 4], f[g8 * 8 + 5], f[g8 * 8 + 6], f[g8 * 8 + 7]);
                        }
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        if (!ok && lane == 0) {
            bars->abort = 1;
            atomicExch(error_flag, 3);
        }
        __syncwarp();
    }

    // ---------------- teardown ----------------
    tcgen05_fence_before();
    __syncthreads();
    if (bars->abort != 0 && threadIdx.x == 0) {
        // give copies that may still be in flight a bounded time to land before smem is released
        for (int s = 0; s < kStages; ++s)
            for (uint32_t i = 0; i < 4096u; ++i)
                if (mbar_try_wait(&bars->full[s], 0) || mbar_try_wait(&bars->full[s], 1)) break;
    }
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                     : "memory");
    }
}

// =============================================================================================
// Two-CTA variant: a cluster of two CTAs (the two SMs of a TPC) computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and its own 128 rows of B
// (32 KiB per ring slot instead of 48 KiB for half as many FLOPs again), which cuts the
// L2 -> shared-memory traffic per FLOP by a third -- the limiter of the one-CTA kernel -- and
// holds its own 128 x 256 half of the accumulator in its TMEM.
//   * the MMA is issued by the leader CTA (cluster rank 0) only;
//   * both producers credit their bytes to the leader's `full` barrier (loads carry
//     .cta_group::2; every CTA fetches its own rows, no load is shared between CTAs);
//   * tcgen05.commit with .multicast::cluster releases ring slots / publishes accumulators to
//     both CTAs; the peer's epilogue warps arrive remotely on the leader's `tmem_empty`.
// =============================================================================================
constexpr int BM2 = 256;               // cluster tile rows (128 per CTA)
constexpr int kStages2 = 6;
constexpr int kBHalfBytes = (BN / 2) * BK * 2;           // 16 KiB: this CTA's half of B
constexpr int kStageBytes2 = kABytes + kBHalfBytes;      // 32 KiB
struct alignas(8) Barriers2 {
    uint64_t full[kStages2];
    uint64_t empty[kStages2];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort;
};
constexpr size_t kSmemBytes2 = 1024 + (size_t)kStages2 * kStageBytes2 + sizeof(Barriers2);

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (an address in this CTA's shared memory) in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_remote_expect_tx(uint32_t cluster_addr, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_remote_arrive(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory, completion bytes credited to a barrier that may live
// in the peer CTA.  Every CTA fetches its own rows.
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *map, int c0, int c1,
                                                 uint32_t bar_cluster_addr)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
        : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t *bar)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(smem_u32(bar)), "h"((uint16_t)3)
        : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                      uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ uint32_t make_idesc_pair(int a_mn_major, int b_mn_major)
{
    uint32_t d = 0;
    d |= 1u << 4;
    d |= 1u << 7;
    d |= 1u << 10;
    d |= (uint32_t)(a_mn_major & 1) << 15;
    d |= (uint32_t)(b_mn_major & 1) << 16;
    d |= (uint32_t)(BN >> 3) << 17;   // N = 256
    d |= (uint32_t)(BM2 >> 4) << 24;  // M = 256 across the pair
    return d;
}

__global__ void __launch_bounds__(kThreads, 1)
ns_gemm_tc2_kernel(const TcGemmProblem *__restrict__ problems, const GemmTile *__restrict__ tiles, int n_tiles,
                   const uint8_t *__restrict__ present, int *__restrict__ error_flag)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    Barriers2 *bars = reinterpret_cast<Barriers2 *>(smem + (size_t)kStages2 * kStageBytes2);
    volatile uint32_t *abort_flag = &bars->abort;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();       // 0 = leader
    const int cluster_id = blockIdx.x >> 1;
    const int n_clusters = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s) {
            mbar_init(&bars->full[s], 2);              // one arrive.expect_tx from each CTA's producer
            mbar_init(&bars->empty[s], 1);             // one multicast commit from the leader's MMA thread
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&bars->tmem_full[a], 1);
            mbar_init(&bars->tmem_empty[a], 2 * kEpiWarps);  // epilogue warps of both CTAs
        }
        bars->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // the same warp of both CTAs allocates the pair's tensor memory
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&bars->tmem_base)),
                     "r"((uint32_t)kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = cluster_id; t < n_tiles && ok; t += n_clusters) {
                const GemmTile tile = tiles[t];
                const TcGemmProblem *p = problems + tile.problem;
                if (present[p->tensor] == 0) continue;
                const int k_blocks = (p->K + BK - 1) / BK;
                const int a_mn = p->a_mn_major, b_mn = p->b_mn_major;
                const int a_row0 = tile.m0 + (int)cta_rank * BM;        // this CTA's rows of A
                const int b_row0 = tile.n0 + (int)cta_rank * (BN / 2);  // this CTA's rows of B
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&bars->empty[stage], phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t *sa = smem + (size_t)stage * kStageBytes2;
                    uint8_t *sb = sa + kABytes;
                    const uint32_t full_leader = map_to_cta(smem_u32(&bars->full[stage]), 0);
                    mbar_remote_expect_tx(full_leader, kStageBytes2);
                    const int k0 = kb * BK;
#pragma unroll
                    for (int j = 0; j < BM / kBoxRows; ++j) {
                        const int r0 = a_row0 + j * kBoxRows;
                        if (a_mn) tma_load_2d_pair(sa + j * kBoxBytes, &p->map_a, r0, k0, full_leader);
                        else      tma_load_2d_pair(sa + j * kBoxBytes, &p->map_a, k0, r0, full_leader);
                    }
#pragma unroll
                    for (int j = 0; j < (BN / 2) / kBoxRows; ++j) {
                        const int r0 = b_row0 + j * kBoxRows;
                        if (b_mn) tma_load_2d_pair(sb + j * kBoxBytes, &p->map_b, r0, k0, full_leader);
                        else      tma_load_2d_pair(sb + j * kBoxBytes, &p->map_b, k0, r0, full_leader);
                    }
                    if (++stage == kStages2) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                bars->abort = 1;
                atomicExch(error_flag, 11);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && cta_rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = cluster_id; t < n_tiles && ok; t += n_clusters) {
                const GemmTile tile = tiles[t];
                const TcGemmProblem *p = problems + tile.problem;
                if (present[p->tensor] == 0) continue;
                const int k_blocks = (p->K + BK - 1) / BK;
                const int a_mn = p->a_mn_major, b_mn = p->b_mn_major;
                const uint32_t idesc = make_idesc_pair(a_mn, b_mn);
                if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * kAccCols);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&bars->full[stage], phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)stage * kStageBytes2);
                    const uint32_t sb = sa + kABytes;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint64_t da = a_mn ? make_smem_desc(sa + kk * 2048, kBoxBytes, 1024)
                                                 : make_smem_desc(sa + kk * 32, 16, 1024);
                        const uint64_t db = b_mn ? make_smem_desc(sb + kk * 2048, kBoxBytes, 1024)
                                                 : make_smem_desc(sb + kk * 32, 16, 1024);
                        tcgen05_mma_bf16_pair(tmem_d, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    tcgen05_commit_pair(&bars->empty[stage]);  // frees the slot in both CTAs
                    if (++stage == kStages2) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                tcgen05_commit_pair(&bars->tmem_full[acc]);  // both CTAs' epilogues may read their halves
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
            if (!ok) {
                bars->abort = 1;
                atomicExch(error_flag, 12);
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
        const int quarter = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int t = cluster_id; t < n_tiles && ok; t += n_clusters) {
            const GemmTile tile = tiles[t];
            const TcGemmProblem *p = problems + tile.problem;
            if (present[p->tensor] == 0) continue;
            const int M = p->M, N = p->N;
            const int epi = p->epilogue;
            __nv_bfloat16 *out_bf16 = p->out_bf16;
            float *out_f32 = p->out_f32;
            const int64_t ld = p->ld_out;
            if (!mbar_wait(&bars->tmem_full[acc], acc_phase, abort_flag)) {
                ok = false;
                break;
            }
            tcgen05_fence_after();
            const int row = tile.m0 + (int)cta_rank * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * kAccCols);
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; ++cc) {
                const int col0 = tile.n0 + cc * 32;
                if (col0 >= N) break;
                uint32_t v[32];
                tmem_ld_32x32(taddr + (uint32_t)(cc * 32), v);
                tmem_ld_wait();
                if (row < M) {
                    float f[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float a = __uint_as_float(v[j]);
                        if (epi == TC_EPI_THREE_I_MINUS) f[j] = (row == col0 + j) ? 3.0f - a : -a;
                        else f[j] = 0.5f * a;
                    }
#pragma unroll
                    for (int g8 = 0; g8 < 4; ++g8) {
                        const int col = col0 + g8 * 8;
                        if (col >= N) break;
                        if (out_bf16) {
                            uint4 q;
                            q.x = pack_bf16(f[g8 * 8 + 0], f[g8 * 8 + 1]);
                            q.y = pack_bf16(f[g8 * 8 + 2], f[g8 * 8 + 3]);
                            q.z = pack_bf16(f[g8 * 8 + 4], f[g8 * 8 + 5]);
                            q.w = pack_bf16(f[g8 * 8 + 6], f[g8 * 8 + 7]);
                            *reinterpret_cast<uint4 *>(out_bf16 + (int64_t)row * ld + col) = q;
                        }
                        if (out_f32) {
                            float4 *dst = reinterpret_cast<float4 *>(out_f32 + (int64_t)row * ld + col);
                            dst[0] = make_float4(f[g8 * 8 + 0], f[g8 * 8 + 1], f[g8 * 8 + 2], f[g8 * 8 + 3]);
                            dst[1] = make_float4(f[g8 * 8 + 4], f[g8 * 8 + 5], f[g8 * 8 + 6], f[g8 * 8 + 7]);
                        }
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_remote_arrive(map_to_cta(smem_u32(&bars->tmem_empty[acc]), 0));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        if (!ok && lane == 0) {
            bars->abort = 1;
            atomicExch(error_flag, 13);
        }
        __syncwarp();
    }

    // ---------------- teardown ----------------
    tcgen05_fence_before();
    __syncthreads();
    if (bars->abort != 0 && threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s)
            for (uint32_t i = 0; i < 4096u; ++i)
                if (mbar_try_wait(&bars->full[s], 0) || mbar_try_wait(&bars->full[s], 1)) break;
    }
    cluster_sync_all();  // neither CTA leaves while its peer may still signal it or read its operands
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                     : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

}  // namespace

// The two-CTA kernel is the default; VB_TC_ONE_CTA=1 selects the one-CTA kernel (128 x 256 tiles).
bool tc_use_pair()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("VB_TC_ONE_CTA");
        v = (e && *e == '1') ? 0 : 1;
    }
    return v == 1;
}

void tc_gemm_tile_shape(int *bm, int *bn)
{
    *bm = tc_use_pair() ? BM2 : BM;
    *bn = BN;
}

// Tensor map over a row-major bf16 matrix [outer][inner] with 64 x 64 boxes and 128-byte
// swizzle; out-of-range elements read as zero.
int make_bf16_tensor_map(void *map_out, const void *base, int64_t inner, int64_t outer)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(VB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((inner % 8) != 0 || (reinterpret_cast<uintptr_t>(base) & 15u) != 0)
        return fail(VB_ERR_UNSUPPORTED, "TMA needs 16-byte aligned rows (inner extent %lld)", (long long)inner);
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)inner * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)kBoxRows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(reinterpret_cast<CUtensorMap *>(map_out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(VB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return VB_OK;
}

int launch_ns_gemm_tc(const TcGemmProblem *d_problems, const GemmTile *d_tiles, int n_tiles,
                      const uint8_t *d_present, int *d_error_flag, int sm_count, cudaStream_t stream)
{
    if (n_tiles <= 0) return VB_OK;
    static bool attr_set = false;
    if (!attr_set) {
        VB_CUDA(cudaFuncSetAttribute(ns_gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kSmemBytes));
        attr_set = true;
    }
    if (tc_use_pair()) {
        static bool attr2_set = false;
        if (!attr2_set) {
            VB_CUDA(cudaFuncSetAttribute(ns_gemm_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemBytes2));
            attr2_set = true;
        }
        int clusters = sm_count / 2;  // one CTA pair per TPC
        if (clusters > n_tiles) clusters = n_tiles;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(clusters * 2));
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSmemBytes2;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        VB_CUDA(cudaLaunchKernelEx(&cfg, ns_gemm_tc2_kernel, d_problems, d_tiles, n_tiles, d_present, d_error_flag));
        return VB_OK;
    }
    int grid = sm_count;  // one persistent CTA per SM (it owns all 512 TMEM columns)
    if (grid > n_tiles) grid = n_tiles;
    ns_gemm_tc_kernel<<<grid, kThreads, kSmemBytes, stream>>>(d_problems, d_tiles, n_tiles, d_present,
                                                              d_error_flag);
    VB_CUDA(cudaGetLastError());
    return VB_OK;
}

}  // namespace vb
