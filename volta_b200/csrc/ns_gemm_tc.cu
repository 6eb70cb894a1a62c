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
// (problem, m0, n0) is walked by the whole GPU.  The kernel is warp specialised:
//   warp 0     TMA producer  (ring of {A 128 x 64, B rows x 64} bf16 slots)
//   warp 1     MMA issuer    (one thread; 4 x tcgen05.mma ...x16 per ring slot)
//   warps 2-9  epilogue      (TMEM -> registers -> global), overlapped with the next tile's
//                             main loop through two TMEM accumulator buffers.  Warp w reads
//                             lane quarter w % 4 and half of the 256 columns, one 32-column
//                             tcgen05.ld ahead of the stores, 256-bit global stores
//
// Two shapes of the same kernel (template parameter kCtas):
//   kCtas = 2 (default)  a cluster of two CTAs -- the two SMs of a TPC -- computes a 256 x 256
//       tile with tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and its own
//       128 rows of B (32 KiB per slot, 6 slots) and keeps its 128 x 256 half of the
//       accumulator in its own TMEM.  The leader CTA issues the MMAs; both producers credit
//       their bytes to the leader's `full` barrier (loads carry .cta_group::2; every CTA
//       fetches its own rows, no load is shared between CTAs); tcgen05.commit with
//       .multicast::cluster frees ring slots and publishes accumulators in both CTAs; the
//       peer's epilogue warps arrive remotely on the leader's `tmem_empty`.
//   kCtas = 1            one CTA per 128 x 256 tile (48 KiB per slot, 4 slots).  It needs 1.5x
//       the shared-memory fill traffic per FLOP and is limited by it (measured 0.85 vs 1.0+
//       PFLOP/s); kept selectable (VB_TC_ONE_CTA=1) for comparison.
//
// Every mbarrier wait is bounded: on expiry the CTA raises an abort flag that all roles
// poll, records an error code for the host, releases its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>

#include "ns_gemm.h"

namespace vb {

namespace {

constexpr int BM = 128;           // rows of A per CTA
constexpr int BN = 256;           // tile columns
constexpr int BK = 64;            // bf16 elements = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kBoxRows = 64;
constexpr int kBoxBytes = kBoxRows * BK * 2;             // 8 KiB: a 64 x 64 bf16 box
constexpr int kRows128Bytes = 128 * BK * 2;              // 16 KiB: 128 operand rows of one slot
constexpr int kAccCols = BN;                             // f32 columns per accumulator
constexpr int kTmemCols = 2 * kAccCols;                  // 512: two accumulators
constexpr int kEpiWarps = 8;                             // two per TMEM lane quarter, 128 columns each
constexpr int kThreads = 64 + kEpiWarps * 32;            // producer warp + MMA warp + epilogue warps
constexpr uint32_t kDefaultWaitLimit = 1u << 22;         // mbarrier polls before giving up

// Staging of the plain kernel's epilogue: each epilogue warp owns 32 rows of 128 bytes.  A lane
// holds one accumulator row, so a direct global store would touch 32 different rows per
// instruction, one 32-byte sector each; through this buffer the warp writes 8 whole 128-byte
// lines per instruction instead.  The 16-byte pieces of row r sit at position (piece ^ (r & 7)),
// which makes both the row-per-lane writes and the four-lanes-per-row reads free of bank
// conflicts without padding.
constexpr int kStageRowBytes = 128;
constexpr int kStageWarpBytes = 32 * kStageRowBytes;
constexpr int kMaxStages = 6;

// kWide (CTA pairs, plain bf16 operands only): the tile is 256 x 512.  The two 256-column halves of
// the accumulator fill all 512 TMEM columns and share the staged rows of A, so a tile fetches
// 256 + 512 operand rows per k block instead of 2 x (256 + 256) for the same work: a quarter less
// traffic from L2, which is what bounds the k = 1024 update products.  There is no second
// accumulator to drain into while the next tile runs; instead each half has its own full / empty
// barriers, the ring keeps filling during the drain, and the MMA thread starts a half as soon as
// that half has been drained.
template <int kCtas, bool kSplit, bool kWide = false>
struct Cfg {
    static_assert(!kWide || (kCtas == 2 && !kSplit), "the wide tile exists for the plain pair kernel");
    // ring slots: 4..7 measure the same on the plain pair kernel (operand bandwidth, not latency, is
    // the limit); the one-CTA kernel gives one up for the epilogue staging
    static constexpr int kStages = kWide ? 4 : (kCtas == 2 ? 6 : (kSplit ? 4 : 3));
    static constexpr int kHalves = kWide ? 2 : 1;                     // 256-column accumulator halves per tile
    static constexpr int kBRows = BN * kHalves / kCtas;               // rows of B staged by one CTA
    static constexpr int kStageBytes = kRows128Bytes + kBRows * BK * 2;
    static constexpr int kTileM = BM * kCtas;
    // Split kernel: one ring slot holds both planes of A and of B for one k block (two images of
    // the plain slot, plane 0 then plane 1), so that each plane crosses from L2 once per k block
    // although it enters two of the three plane products.
    static constexpr int kSplitStages = kStages / 2;
    static constexpr int kSplitStageBytes = 2 * kStageBytes;
    static constexpr int kEpiStageBytes = kSplit ? 0 : kEpiWarps * kStageWarpBytes;
};

struct alignas(8) Barriers {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort;
    uint32_t skip;  // the error flag was already set when this CTA started: do nothing
};
template <int kCtas, bool kSplit, bool kWide>
constexpr size_t smem_bytes()
{
    using C = Cfg<kCtas, kSplit, kWide>;
    return 1024 /*alignment slack*/ + (size_t)C::kStages * C::kStageBytes + C::kEpiStageBytes + sizeof(Barriers);
}
static_assert(smem_bytes<2, false, true>() <= 232448 && smem_bytes<2, false, false>() <= 232448 &&
                  smem_bytes<2, true, false>() <= 232448,
              "a CTA has 227 KiB of shared memory");

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
__device__ __forceinline__ void mbar_remote_arrive(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t wait_limit)
{
    for (uint32_t i = 0; i < wait_limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u && *abort_flag != 0u) return false;
    }
    return false;
}

// Compile-time diagnostic (-DVB_TC_TIMING): cycles the first CTA pair spends in each kind of
// wait, accumulated in g_wait_cycles[site + 4 * (blockIdx.x & 1)]; not built by default.
#ifdef VB_TC_TIMING
__device__ unsigned long long g_wait_cycles[16];
__device__ __forceinline__ bool mbar_wait_timed(int site, uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag)
{
    const long long t0 = clock64();
    const bool ok = mbar_wait(bar, parity, abort_flag, kDefaultWaitLimit);
    if (blockIdx.x < 2) atomicAdd(&g_wait_cycles[site + 4 * (blockIdx.x & 1)], (unsigned long long)(clock64() - t0));
    return ok;
}
#define MBAR_WAIT(site, bar, parity) mbar_wait_timed(site, bar, parity, abort_flag)
#else
#define MBAR_WAIT(site, bar, parity) mbar_wait(bar, parity, abort_flag, wait_limit)
#endif

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

// TMA loads into this CTA's shared memory.  `bar` is a shared::cluster address: this CTA's own
// barrier, or (kCtas == 2, .cta_group::2) the leader's.  Every CTA fetches its own rows.
template <int kCtas>
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int c0, int c1, uint32_t bar)
{
    if (kCtas == 2)
        asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
            "[%0], [%1, {%2, %3}], [%4];"
            ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
            : "memory");
    else
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
            ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
            : "memory");
}
template <int kCtas>
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *map, int c0, int c1, int c2,
                                            uint32_t bar)
{
    if (kCtas == 2)
        asm volatile(
            "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
            "[%0], [%1, {%2, %3, %4}], [%5];"
            ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
            : "memory");
    else
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
            "[%0], [%1, {%2, %3, %4}], [%5];"
            ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
            : "memory");
}
template <int kCtas>
__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *map, int c0, int c1, int c2, int c3,
                                            uint32_t bar)
{
    if (kCtas == 2)
        asm volatile(
            "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
            "[%0], [%1, {%2, %3, %4, %5}], [%6];"
            ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
            "r"(bar)
            : "memory");
    else
        asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
            "[%0], [%1, {%2, %3, %4, %5}], [%6];"
            ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
            "r"(bar)
            : "memory");
}
// Stages 128 operand rows x 64 k (16 KiB) of plane `plane` with as few TMA instructions as the
// layout allows: the issuing thread is the scarce resource (every instruction costs it a few
// hundred cycles).  The outermost tensor-map dimension selects the plane (one plane for plain
// bf16 operands, three for operands split into bf16 pieces).
//   TC_OP_K_MAJOR   one 64 x 128 box of a [rows][k] matrix
//   TC_OP_MN_BOXES  two 64 x 64 boxes of a [k][rows] matrix (any row count)
//   TC_OP_MN_3D     one 64 x 64 x 2 box of the same matrix viewed as [rows/64][k][64]
// All three leave the same image in shared memory.
template <int kCtas, bool kSplit>
__device__ __forceinline__ void load_rows128(uint8_t *dst, const CUtensorMap *map, int mode, int row0, int k0,
                                             int plane, uint32_t bar)
{
    if (kSplit) {  // tensor maps with a plane dimension
        if (mode == TC_OP_K_MAJOR) {
            tma_load_3d<kCtas>(dst, map, k0, row0, plane, bar);
        } else if (mode == TC_OP_MN_3D) {
            tma_load_4d<kCtas>(dst, map, 0, k0, row0 >> 6, plane, bar);
        } else {
            tma_load_3d<kCtas>(dst, map, row0, k0, plane, bar);
            tma_load_3d<kCtas>(dst + kBoxBytes, map, row0 + kBoxRows, k0, plane, bar);
        }
    } else {
        if (mode == TC_OP_K_MAJOR) {
            tma_load_2d<kCtas>(dst, map, k0, row0, bar);
        } else if (mode == TC_OP_MN_3D) {
            tma_load_3d<kCtas>(dst, map, 0, k0, row0 >> 6, bar);
        } else {
            tma_load_2d<kCtas>(dst, map, row0, k0, bar);
            tma_load_2d<kCtas>(dst + kBoxBytes, map, row0 + kBoxRows, k0, bar);
        }
    }
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Arrive on `bar` (same offset in every CTA of the group) once all MMAs issued so far are done.
template <int kCtas>
__device__ __forceinline__ void tcgen05_commit(uint64_t *bar)
{
    if (kCtas == 2)
        asm volatile(
            "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
            ::"r"(smem_u32(bar)), "h"((uint16_t)3)
            : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                     : "memory");
}
template <int kCtas>
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate)
{
    if (kCtas == 2)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    else
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
// Load and wait in one statement: the values are final when the statement ends.
__device__ __forceinline__ void tmem_ld_32x32_sync(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

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
// Descriptor of the 16-wide k slice `kk` of a staged operand.
//   K-major : rows of 128 bytes, 8-row groups 1 KiB apart; 16 bf16 = 32 bytes along the row.
//   MN-major: [k][64 rows] blocks of 8 KiB; 8-k groups 1 KiB apart (SBO), 64-row blocks 8 KiB
//             apart (LBO); 16 k = 2 KiB further down the block.
__device__ __forceinline__ uint64_t operand_desc(uint32_t base, int mode, int kk)
{
    return mode == TC_OP_K_MAJOR ? make_smem_desc(base + kk * 32, 16, 1024)
                                 : make_smem_desc(base + kk * 2048, kBoxBytes, 1024);
}

// Instruction descriptor for kind::f16 with bf16 operands and f32 accumulation.
__device__ __forceinline__ uint32_t make_idesc(int a_mode, int b_mode, int m, bool fp16)
{
    uint32_t d = 0;
    d |= 1u << 4;                    // D format: f32
    d |= (fp16 ? 0u : 1u) << 7;      // A format: f16 (0) or bf16 (1)
    d |= (fp16 ? 0u : 1u) << 10;     // B format
    d |= (uint32_t)(a_mode != TC_OP_K_MAJOR) << 15;  // A is MN-major
    d |= (uint32_t)(b_mode != TC_OP_K_MAJOR) << 16;  // B is MN-major
    d |= (uint32_t)(BN >> 3) << 17;  // N
    d |= (uint32_t)(m >> 4) << 24;   // M (across the CTA group)
    return d;
}

// One 32-byte (sector-sized) global store.  The address must be 32-byte aligned.
__device__ __forceinline__ void st_global_256(void *p, const uint32_t (&q)[8])
{
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(q[0]), "r"(q[1]), "r"(q[2]),
                 "r"(q[3]), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7])
                 : "memory");
}

__device__ __forceinline__ void ld_global_256(const void *p, uint32_t (&q)[8])
{
    asm volatile("ld.global.L1::no_allocate.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7])
                 : "l"(p));
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b)
{
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

// Muon's apply on 8 consecutive weights of one row (32-byte aligned): w -= (lr * u) * 0.1 with the
// reference's order of operations (src/nn/optim/muon.rs:158-160, each product and the difference
// rounded once), then the stores the apply kernel would do: the local arena, every peer's arena,
// the bf16 copy and the peers' bf16 copies.  `wq` holds the old weights and receives the new ones.
__device__ __forceinline__ void apply_octet(uint32_t (&wq)[8], const uint32_t (&u)[8], float lr, float *w_dst,
                                            int64_t arena_pos, const PeerTable &pt)
{
#pragma unroll
    for (int j = 0; j < 8; ++j)
        wq[j] = __float_as_uint(__fsub_rn(__uint_as_float(wq[j]), __fmul_rn(__fmul_rn(lr, __uint_as_float(u[j])), 0.1f)));
    st_global_256(w_dst, wq);
    if (pt.n > 0) {
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
            if (r < pt.n) st_global_256(pt.base[r] + arena_pos, wq);
    }
    if (pt.half_local != nullptr) {
        const uint4 h = make_uint4(pack_bf16(__uint_as_float(wq[0]), __uint_as_float(wq[1])),
                                   pack_bf16(__uint_as_float(wq[2]), __uint_as_float(wq[3])),
                                   pack_bf16(__uint_as_float(wq[4]), __uint_as_float(wq[5])),
                                   pack_bf16(__uint_as_float(wq[6]), __uint_as_float(wq[7])));
        *reinterpret_cast<uint4 *>(pt.half_local + arena_pos) = h;
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
            if (r < pt.n_half) *reinterpret_cast<uint4 *>(pt.half_base[r] + arena_pos) = h;
    }
}

// The f32-accurate path: every operand is held as two f16 planes of the value scaled by 2^15,
//     x * 2^15 = h0 + h1,   h0 = f16(x * 2^15),   h1 = f16(x * 2^15 - h0),
// 22 significand bits in all (Newton-Schulz operands are bounded by 1 in magnitude once the
// update is normalised, so the scaled values stay below the f16 maximum and the small plane
// stays out of the f16 subnormals for every element that matters to the Frobenius norm).
// Three plane products, smallest first, are accumulated into the same f32 accumulator:
// (plane of A, plane of B) = (0,1) (1,0) (0,0); the dropped h1*h1 is below 2^-22 relative.
// The accumulator then holds 2^30 times the product.  One nibble per term, term 0 lowest.
__device__ __forceinline__ int term_plane_a(int n_terms, int term) { return n_terms == 1 ? 0 : ((0x010 >> (4 * term)) & 15); }
__device__ __forceinline__ int term_plane_b(int n_terms, int term) { return n_terms == 1 ? 0 : ((0x001 >> (4 * term)) & 15); }

// What a role needs to know about a tile, fetched one tile ahead so that the dependent global
// loads (tile -> problem -> fields) never sit between two tiles' main loops.
// The common path of the plain bf16 kernel (the warp's 128 columns lie inside the matrix, output
// rows start on 32-byte boundaries): one multiply per element, the 3I of the Gram epilogue added
// only by the one warp piece that holds the diagonal, bf16 rounding.  The epilogue warps share
// their schedulers with the producer and the MMA thread, so the instruction count here decides
// how much the drain disturbs the main loop.
//
// A lane owns one accumulator row (TMEM lane = row), so direct stores would hit 32 rows per
// instruction with one 32-byte sector each.  Row-major outputs therefore go through the warp's
// staging buffer in shared memory: every lane writes its row piece, then the warp reads the
// buffer back with four lanes per row and stores 8 whole 128-byte lines per instruction (bf16:
// two 32-column pieces make one line; f32: one piece is one line).  The fused apply reads and
// writes the weights in the same line-per-four-lanes pattern.  Outputs at the transposed position
// (the mirror of a symmetric tile, the transposed update) are contiguous along the rows the 32
// lanes hold and are stored directly, 64 or 128 bytes per instruction.
__device__ __forceinline__ void st_shared_128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void ld_shared_128(uint32_t addr, uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d)
{
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr) : "memory");
}

// kIn: the bf16 tile of `in_bf16` at the output position enters the result, f = 1.5 in + mult acc
// (TC_EPI_NS_COMBINE on the plain path, with mult = -0.5 times the accumulator's scale).
template <int EPI, bool kIn = false>
__device__ __forceinline__ void drain_fast(uint32_t taddr, int row0, int tile_col0, int M, float mult, int lane,
                                           __nv_bfloat16 *out_bf16, float *out_f32, bool mirror, bool transpose,
                                           int64_t ld, float *apply_w, int64_t apply_pos, const TcApplyArgs &ap,
                                           uint32_t stage, const __nv_bfloat16 *in_bf16 = nullptr)
{
    constexpr int kPieces = (BN / 2) / 32;
    const int row = row0 + lane;  // the accumulator row this lane holds
    const bool row_ok = row < M;
    const bool direct_bf16 = out_bf16 != nullptr && !transpose;
    const bool direct_f32 = (out_f32 != nullptr && !transpose) || apply_w != nullptr;
    // read-back mapping: four lanes per row (32 bytes each), eight rows per pass, four passes
    const int r_sub = lane >> 2, seg = lane & 3;
    const uint32_t my_row = stage + (uint32_t)(lane * kStageRowBytes);
    const uint32_t my_sw = (uint32_t)(lane & 7);
    const uint32_t rd_row = stage + (uint32_t)(r_sub * kStageRowBytes);  // row r_sub + 8 * pass: (row & 7) == r_sub
    const uint32_t rd_c0 = (uint32_t)(((2 * seg) ^ r_sub) << 4), rd_c1 = (uint32_t)(((2 * seg + 1) ^ r_sub) << 4);
    uint32_t v[2][32];
    tmem_ld_32x32(taddr, v[0]);
#pragma unroll
    for (int cc = 0; cc < kPieces; ++cc) {
        const int col0 = tile_col0 + cc * 32;
        tmem_ld_wait();
        if (cc + 1 < kPieces) tmem_ld_32x32(taddr + (uint32_t)((cc + 1) * 32), v[(cc + 1) & 1]);
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[cc & 1][j]) * mult;
        if (kIn && row_ok) {  // the lane's 32 bf16 of the input tile: four 16-byte loads (rows start on 32-byte boundaries)
            const uint4 *src = reinterpret_cast<const uint4 *>(in_bf16 + (int64_t)row * ld + col0);
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
                const uint4 q = src[g8];
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    f[g8 * 8 + 2 * h] = fmaf(1.5f, __uint_as_float(w[h] << 16), f[g8 * 8 + 2 * h]);
                    f[g8 * 8 + 2 * h + 1] = fmaf(1.5f, __uint_as_float(w[h] & 0xffff0000u), f[g8 * 8 + 2 * h + 1]);
                }
            }
        }
        if (EPI == TC_EPI_THREE_I_MINUS && row - col0 == lane) {  // warp-uniform: the piece that holds the diagonal
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = (j == lane) ? 3.0f + f[j] : f[j];
        }
        if (row_ok) {
            const int64_t at_t = (int64_t)col0 * ld + row;  // element (row, col0) of the transposed matrix
            if (out_f32 != nullptr && transpose) {
                float *t = out_f32 + at_t;
#pragma unroll
                for (int j = 0; j < 32; ++j) t[(int64_t)j * ld] = f[j];
            }
            if (out_bf16 != nullptr && (mirror || transpose)) {
                __nv_bfloat16 *t = out_bf16 + at_t;
#pragma unroll
                for (int j = 0; j < 32; ++j) t[(int64_t)j * ld] = __float2bfloat16_rn(f[j]);
            }
        }
        if (direct_bf16) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
                st_shared_128(my_row + ((((uint32_t)((cc & 1) * 4 + q)) ^ my_sw) << 4), pack_bf16(f[8 * q], f[8 * q + 1]),
                              pack_bf16(f[8 * q + 2], f[8 * q + 3]), pack_bf16(f[8 * q + 4], f[8 * q + 5]),
                              pack_bf16(f[8 * q + 6], f[8 * q + 7]));
            if (cc & 1) {  // two pieces = 64 columns = one 128-byte line per row
                __syncwarp();
                const int colp = col0 - 32;
#pragma unroll
                for (int pass = 0; pass < 4; ++pass) {
                    uint32_t q[8];
                    const uint32_t src = rd_row + (uint32_t)(pass * 8 * kStageRowBytes);
                    ld_shared_128(src + rd_c0, q[0], q[1], q[2], q[3]);
                    ld_shared_128(src + rd_c1, q[4], q[5], q[6], q[7]);
                    const int r = row0 + r_sub + 8 * pass;
                    if (r < M) st_global_256(out_bf16 + (int64_t)r * ld + colp + seg * 16, q);
                }
                __syncwarp();
            }
        }
        if (direct_f32) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
                st_shared_128(my_row + ((((uint32_t)q) ^ my_sw) << 4), __float_as_uint(f[4 * q]), __float_as_uint(f[4 * q + 1]),
                              __float_as_uint(f[4 * q + 2]), __float_as_uint(f[4 * q + 3]));
            __syncwarp();
            uint32_t u[4][8], wq[4][8];
#pragma unroll
            for (int pass = 0; pass < 4; ++pass) {  // all loads of the old weights first: their latency overlaps
                const int r = row0 + r_sub + 8 * pass;
                if (apply_w != nullptr && r < M) ld_global_256(apply_w + (int64_t)r * ld + col0 + seg * 8, wq[pass]);
                const uint32_t src = rd_row + (uint32_t)(pass * 8 * kStageRowBytes);
                ld_shared_128(src + rd_c0, u[pass][0], u[pass][1], u[pass][2], u[pass][3]);
                ld_shared_128(src + rd_c1, u[pass][4], u[pass][5], u[pass][6], u[pass][7]);
            }
#pragma unroll
            for (int pass = 0; pass < 4; ++pass) {
                const int r = row0 + r_sub + 8 * pass;
                if (r < M) {
                    const int64_t at = (int64_t)r * ld + col0 + seg * 8;
                    if (apply_w != nullptr) apply_octet(wq[pass], u[pass], ap.lr, apply_w + at, apply_pos + at, ap.pt);
                    if (out_f32 != nullptr && !transpose) st_global_256(out_f32 + at, u[pass]);
                }
            }
            __syncwarp();
        }
    }
}

// Every other case: ragged edges (columns beyond N, unaligned output rows), and all of the
// split (f32-accurate) kernel's epilogues.  Element-wise code with the bounds checks inside.
struct DrainArgs {
    uint32_t taddr;
    int row, tile_col0, M, N, epi, lane, split_e;
    float acc_scale;
    int64_t ld, plane_stride;
    int out_planes, out_planes_in;
    bool bf16_rows_32b, mirror, transpose;
    __nv_bfloat16 *out_bf16;
    float *out_f32;
    const __nv_bfloat16 *in_bf16;
    float *apply_w;        // fused apply: the matrix's weights (null: none), see TcApplyArgs
    int64_t apply_pos;     // arena position of the matrix's first element
    const TcApplyArgs *ap;
};
// 16-bit output formats: bf16 on the plain path, f16 planes on the split path.
template <bool kHalf>
__device__ __forceinline__ uint32_t pack16(float a, float b)
{
    if (kHalf) {
        const __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
    return pack_bf16(a, b);
}
template <bool kHalf>
__device__ __forceinline__ unsigned short round16(float a)
{
    if (kHalf) return __half_as_ushort(__float2half_rn(a));
    return __bfloat16_as_ushort(__float2bfloat16_rn(a));
}
template <bool kHalf>
__device__ __forceinline__ float rounded16(float a)
{
    if (kHalf) return __half2float(__float2half_rn(a));
    return __bfloat162float(__float2bfloat16_rn(a));
}

// kInRead: TC_EPI_NS_COMBINE (the output position of `in_bf16` enters the result) is compiled in; always
// on the split path, on the plain path only in the instantiation kept for the rarer launches.
template <bool kSplit, bool kInRead>
__device__ __forceinline__ void drain_generic(const DrainArgs &a)
{
    constexpr int kChunks = (BN / 2) / 32;
    const uint32_t taddr = a.taddr;
    const int row = a.row, tile_col0 = a.tile_col0, M = a.M, N = a.N, epi = a.epi;
    const float acc_scale = a.acc_scale;
    const int64_t ld = a.ld, plane_stride = a.plane_stride;
    const int out_planes = a.out_planes, out_planes_in = a.out_planes_in;
    const bool bf16_rows_32b = a.bf16_rows_32b, transpose = a.transpose;
    const bool mirror = a.mirror || transpose;  // the transposed position is written in both cases
    __nv_bfloat16 *out_bf16 = a.out_bf16;
    float *out_f32 = a.out_f32;
    const __nv_bfloat16 *in_bf16 = a.in_bf16;
    // One load in flight at a time, waited for in the same statement: the registers a
    // tcgen05.ld targets are written asynchronously, so nothing may touch or move them before
    // the wait; this path is off the critical path (ragged edges; the split kernel's main loop is
    // three times longer), so it does not pipeline its loads.
    uint32_t v[32];
    for (int cc = 0; cc < kChunks; ++cc) {
        const int col0 = tile_col0 + cc * 32;
        if (col0 >= N) break;  // uniform across the warp
        tmem_ld_32x32_sync(taddr + (uint32_t)(cc * 32), v);
        if (row < M) {
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float a = __uint_as_float(v[j]) * acc_scale;
                if (epi == TC_EPI_THREE_I_MINUS) f[j] = (row == col0 + j) ? 3.0f - a : -a;  // muon.rs:76-89
                else if (epi == TC_EPI_HALF) f[j] = 0.5f * a;                               // muon.rs:95-99
                else f[j] = a;  // TC_EPI_IDENTITY, or TC_EPI_NS_COMBINE (finished below)
            }
            if (kInRead && epi == TC_EPI_NS_COMBINE) {
                // X' = 0.5 X (3I - G) evaluated as 1.5 X - 0.5 (X G): the accumulator holds only
                // the small product X G, so the tensor core's truncating f32 accumulation acts on
                // a term that is a few percent of the result instead of on the result itself.
                const __nv_bfloat16 *src = in_bf16 + (int64_t)row * ld + col0;
                float x[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) x[j] = 0.0f;
                for (int pl = out_planes_in - 1; pl >= 0; --pl) {  // smallest piece first: the sum is exact
#pragma unroll
                    for (int g8 = 0; g8 < 4; ++g8) {               // 8 columns = one 16-byte load
                        if (col0 + g8 * 8 < N) {
                            const uint4 q = *reinterpret_cast<const uint4 *>(src + pl * plane_stride + g8 * 8);
                            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                            for (int h = 0; h < 4; ++h) {
                                if (kSplit) {
                                    x[g8 * 8 + 2 * h] += f16_bits_to_float(w[h] & 0xffffu);
                                    x[g8 * 8 + 2 * h + 1] += f16_bits_to_float(w[h] >> 16);
                                } else {  // bf16: the upper half of an f32
                                    x[g8 * 8 + 2 * h] += __uint_as_float(w[h] << 16);
                                    x[g8 * 8 + 2 * h + 1] += __uint_as_float(w[h] & 0xffff0000u);
                                }
                            }
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] = fmaf(1.5f, x[j], -0.5f * f[j]);  // X' scaled by 2^(15 - e)
            }
            // the update of the split kernel is in the scaled domain: what goes out in f32 is scaled back
            const bool scaled = kSplit && epi == TC_EPI_NS_COMBINE;
            if (scaled && (out_f32 != nullptr || a.apply_w != nullptr)) {
                const float back = ldexpf(1.0f, a.split_e - 15);
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] *= back;
            }
            if (a.apply_w != nullptr) {  // never combined with a transposed output
                const int64_t at = (int64_t)row * ld + col0;
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {  // N and ld are multiples of 8: whole octets, 32-byte aligned
                    if (col0 + g8 * 8 >= N) break;
                    uint32_t wq[8], uq[8];
                    ld_global_256(a.apply_w + at + g8 * 8, wq);
#pragma unroll
                    for (int j = 0; j < 8; ++j) uq[j] = __float_as_uint(f[g8 * 8 + j]);
                    apply_octet(wq, uq, a.ap->lr, a.apply_w + at + g8 * 8, a.apply_pos + at + g8 * 8, a.ap->pt);
                }
            }
            if (out_f32 && transpose) {
                float *tdst = out_f32 + (int64_t)col0 * ld + row;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < N) tdst[(int64_t)j * ld] = f[j];
            }
            if (out_f32 && !transpose) {
                float *dst = out_f32 + (int64_t)row * ld + col0;
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {  // 8 columns = one 32-byte sector per store
                    if (col0 + g8 * 8 >= N) break;
                    uint32_t q[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) q[j] = __float_as_uint(f[g8 * 8 + j]);
                    st_global_256(dst + g8 * 8, q);
                }
            }
            if (out_bf16) {
                if (kSplit && !scaled) {  // the planes hold the value times 2^15 (the update is scaled already)
#pragma unroll
                    for (int j = 0; j < 32; ++j) f[j] *= kSplitScale;
                }
                for (int pl = 0; pl < out_planes; ++pl) {
                    __nv_bfloat16 *dst = out_bf16 + pl * plane_stride + (int64_t)row * ld + col0;
#pragma unroll
                    for (int g16 = 0; g16 < 2; ++g16) {  // 16 columns = one 32-byte sector per store
                        if (transpose) break;            // only the transposed position is written
                        const int col = col0 + g16 * 16;
                        if (col + 16 <= N && bf16_rows_32b) {
                            uint32_t q[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                q[j] = pack16<kSplit>(f[g16 * 16 + 2 * j], f[g16 * 16 + 2 * j + 1]);
                            st_global_256(dst + g16 * 16, q);
                        } else {  // 16-byte pieces (N and ld are multiples of 8)
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                if (col + h * 8 >= N) break;
                                uint4 q;
                                q.x = pack16<kSplit>(f[g16 * 16 + h * 8 + 0], f[g16 * 16 + h * 8 + 1]);
                                q.y = pack16<kSplit>(f[g16 * 16 + h * 8 + 2], f[g16 * 16 + h * 8 + 3]);
                                q.z = pack16<kSplit>(f[g16 * 16 + h * 8 + 4], f[g16 * 16 + h * 8 + 5]);
                                q.w = pack16<kSplit>(f[g16 * 16 + h * 8 + 6], f[g16 * 16 + h * 8 + 7]);
                                *reinterpret_cast<uint4 *>(dst + g16 * 16 + h * 8) = q;
                            }
                        }
                    }
                    if (mirror) {
                        // D is symmetric and only its upper tiles are computed: element (row, col)
                        // also goes to (col, row).  For a fixed column the 32 lanes of the warp
                        // hold 32 consecutive rows, i.e. one contiguous 64-byte run of the mirror.
                        __nv_bfloat16 *mdst = out_bf16 + pl * plane_stride + (int64_t)col0 * ld + row;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < N)
                                reinterpret_cast<unsigned short *>(mdst)[(int64_t)j * ld] = round16<kSplit>(f[j]);
                    }
                    if (pl + 1 < out_planes) {  // what this plane's rounding left over goes to the next
#pragma unroll
                        for (int j = 0; j < 32; ++j) f[j] -= rounded16<kSplit>(f[j]);
                    }
                }
            }
        }
    }
}

struct TileInfo {
    const TcGemmProblem *p;
    int m0, n0, k_blocks, a_mode, b_mode, n_terms;
    bool mirror;    // symmetric product: this off-diagonal tile is also stored transposed
    bool b_is_a;    // diagonal tile of a symmetric product: B's rows are A's rows, staged once
    bool single;    // wide tile with one half only
    bool symmetric; // wide tile of a symmetric product (mirror / operand sharing decided per half)
    bool skipped;   // gradient absent: nothing to do
    bool withhold;  // test hook (TcGemmProblem::withhold_loads): the producer stages nothing
};
__device__ __forceinline__ TileInfo fetch_tile(const TcGemmProblem *problems, const GemmTile *tiles, int n_tiles,
                                               const uint8_t *present, int t)
{
    TileInfo ti;
    ti.p = problems;
    ti.m0 = ti.n0 = ti.k_blocks = ti.a_mode = ti.b_mode = 0;
    ti.n_terms = 1;
    ti.skipped = true;
    ti.withhold = false;
    ti.mirror = false;
    ti.b_is_a = false;
    ti.single = false;
    ti.symmetric = false;
    if (t < n_tiles) {
        const GemmTile tile = tiles[t];
        const TcGemmProblem *p = problems + tile.problem;
        ti.p = p;
        ti.m0 = tile.m0;
        ti.n0 = tile.n0;
        ti.mirror = (tile.flags & GEMM_TILE_MIRROR) != 0;
        ti.b_is_a = (tile.flags & GEMM_TILE_B_IS_A) != 0;
        ti.single = (tile.flags & GEMM_TILE_SINGLE) != 0;
        ti.symmetric = (tile.flags & GEMM_TILE_SYMMETRIC) != 0;
        ti.k_blocks = (p->K + BK - 1) / BK;
        ti.a_mode = p->a_mode;
        ti.b_mode = p->b_mode;
        ti.n_terms = p->n_terms;
        ti.skipped = present[p->tensor] == 0;
        ti.withhold = p->withhold_loads != 0;
    }
    return ti;
}

// kSplit: the operands are two f16 planes (f32-accurate path); the plain bf16 instantiation
// carries none of that code.
// kDual: launches whose 3I - G problems also store G itself (TcGemmProblem::out2_bf16) drain every
// accumulator twice; the code for that lives in an instantiation of its own so that the register
// allocation of every other launch is not touched by it.
template <int kCtas, bool kSplit, bool kWide, bool kDual>
__global__ void __launch_bounds__(kThreads, 1)
ns_gemm_tc_kernel(const TcGemmProblem *__restrict__ problems, const GemmTile *__restrict__ tiles, int n_tiles,
                  const uint8_t *__restrict__ present, int *__restrict__ error_flag, uint32_t wait_limit,
                  const __grid_constant__ TcApplyArgs ap)
{
    using C = Cfg<kCtas, kSplit, kWide>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *epi_stage = smem + (size_t)C::kStages * C::kStageBytes;
    Barriers *bars = reinterpret_cast<Barriers *>(epi_stage + C::kEpiStageBytes);
    volatile uint32_t *abort_flag = &bars->abort;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = kCtas == 2 ? cluster_ctarank() : 0u;  // 0 = leader
    const int group_id = blockIdx.x / kCtas;                        // CTA pair (or CTA) index
    const int n_groups = gridDim.x / kCtas;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(&bars->full[s], 1);   // the (leader's) producer arrives; bytes come from every CTA
            mbar_init(&bars->empty[s], 1);  // one commit from the MMA thread
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&bars->tmem_full[a], 1);
            mbar_init(&bars->tmem_empty[a], kCtas * kEpiWarps);  // epilogue warps of every CTA of the group
        }
        bars->abort = 0;
        // An earlier kernel of the chain gave up a wait: its output is half written, so this
        // launch computes and stores nothing (read once per CTA: every role sees the same value).
        bars->skip = *reinterpret_cast<const volatile int *>(error_flag) != 0 ? 1u : 0u;
        // a launch that stores into peer GPUs also stays idle when the fence before it gave up
        if (ap.enabled && (ap.pt.n > 0 || ap.pt.n_half > 0) && fence_failed(ap.pt.fence_error)) bars->skip = 1u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // TMEM allocation is warp-wide; with two CTAs the same warp of both allocates
        if (kCtas == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(&bars->tmem_base)),
                         "r"((uint32_t)kTmemCols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(&bars->tmem_base)),
                         "r"((uint32_t)kTmemCols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (kCtas == 2) cluster_sync_all();  // the peer's barriers exist before anything signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    if (bars->skip != 0u) n_tiles = 0;

    if (warp == 0) {
        // ---------------- TMA producer (every CTA) ----------------
        // Two lanes share the issue work: lane 0 fetches A (and posts the byte count), lane 1
        // fetches B.  Both wait on the same `empty` barrier.
        if (lane < 2) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            TileInfo next = fetch_tile(problems, tiles, n_tiles, present, group_id);
            for (int t = group_id; t < n_tiles && ok; t += n_groups) {
                const TileInfo ti = next;
                next = fetch_tile(problems, tiles, n_tiles, present, t + n_groups);
                if (ti.skipped) continue;
                const int a_row0 = ti.m0 + (int)cta_rank * BM;         // this CTA's rows of A
                const int b_row0 = ti.n0 + (int)cta_rank * C::kBRows;  // this CTA's rows of B
                // diagonal tile of a symmetric product (pair kernel, plain bf16): each CTA's 128 rows of
                // B are its 128 rows of A, so they are fetched once and the MMA reads A's slot twice
                const bool alias_b = kCtas == 2 && !kSplit && !kWide && ti.b_is_a;
                // wide tile: the half on the diagonal of a symmetric product reads A's rows as its B
                const bool alias_h0 = kWide && ti.symmetric && ti.n0 == ti.m0;
                const int wide_b_loads = (ti.single ? 1 : 2) - (alias_h0 ? 1 : 0);
                constexpr int kRing = kSplit ? C::kSplitStages : C::kStages;
                constexpr int kSlotBytes = kSplit ? C::kSplitStageBytes : C::kStageBytes;
                const int n_slots = ti.k_blocks;  // one ring slot per k block
                for (int slot = 0; slot < n_slots; ++slot) {
                    // both producer lanes act on one decision: if either saw the wait run out (or
                    // the abort flag), both stop here
                    if (!__all_sync(0x3u, MBAR_WAIT(0, &bars->empty[stage], phase ^ 1u))) {
                        ok = false;
                        break;
                    }
                    uint8_t *sa = smem + (size_t)stage * kSlotBytes;
                    uint8_t *sb = sa + kRows128Bytes;
                    // Only the leader posts the expected byte count (for all CTAs' loads): a remote
                    // arrive from the peer would put a cluster round trip into every ring slot.
                    // The peer's bytes may land before the leader's expect_tx; the phase cannot
                    // complete until the leader has arrived.
                    const uint32_t full_bar =
                        kCtas == 2 ? map_to_cta(smem_u32(&bars->full[stage]), 0) : smem_u32(&bars->full[stage]);
                    const int k0 = slot * BK;
                    if (ti.withhold) {
                        // Nothing is staged and no bytes are announced: the consumers' bounded waits
                        // (and, a ring later, this thread's own) run out.  Used by the expiry test.
                    } else if (lane == 0) {
                        if (cta_rank == 0)
                            mbar_expect_tx(&bars->full[stage], kWide     ? kCtas * kRows128Bytes * (1 + wide_b_loads)
                                                               : alias_b ? kCtas * kRows128Bytes
                                                                         : kCtas * kSlotBytes);
#pragma unroll
                        for (int pl = 0; pl < (kSplit ? kSplitPlanes : 1); ++pl)
                            load_rows128<kCtas, kSplit>(sa + pl * C::kStageBytes, &ti.p->map_a, ti.a_mode, a_row0, k0, pl,
                                                        full_bar);
                    } else if (!alias_b) {
#pragma unroll
                        for (int pl = 0; pl < (kSplit ? kSplitPlanes : 1); ++pl)
#pragma unroll
                            for (int j = 0; j < C::kBRows / 128; ++j) {  // wide tile: this CTA's 128 rows of each half
                                if (kWide && ((j == 1 && ti.single) || (j == 0 && alias_h0))) continue;
                                load_rows128<kCtas, kSplit>(sb + pl * C::kStageBytes + j * kRows128Bytes, &ti.p->map_b,
                                                            ti.b_mode,
                                                            kWide ? ti.n0 + j * BN + (int)cta_rank * 128 : b_row0 + j * 128,
                                                            k0, pl, full_bar);
                            }
                    }
                    if (++stage == kRing) {
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
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && cta_rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            uint32_t half_phase[2] = {0u, 0u};  // wide tile: each half's barriers advance only when the half is used
            bool ok = true;
            TileInfo next = fetch_tile(problems, tiles, n_tiles, present, group_id);
            for (int t = group_id; t < n_tiles && ok; t += n_groups) {
                const TileInfo ti = next;
                next = fetch_tile(problems, tiles, n_tiles, present, t + n_groups);
                if (ti.skipped) continue;
                const uint32_t idesc = make_idesc(ti.a_mode, ti.b_mode, C::kTileM, kSplit);
                // the epilogue(s) must have drained this accumulator (wide tile: each half is waited
                // for right before its first MMA, see below)
                if (!kWide) {
                    if (!MBAR_WAIT(1, &bars->tmem_empty[acc], acc_phase ^ 1u)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                }
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * kAccCols);
                constexpr int kRing = kSplit ? C::kSplitStages : C::kStages;
                constexpr int kSlotBytes = kSplit ? C::kSplitStageBytes : C::kStageBytes;
                const int n_slots = ti.k_blocks;
                for (int slot = 0; slot < n_slots; ++slot) {
                    if (!MBAR_WAIT(2, &bars->full[stage], phase)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t base = smem_u32(smem + (size_t)stage * kSlotBytes);
                    if (kSplit) {
                        // three plane products per k block, smallest first, from the two staged planes
#pragma unroll
                        for (int term = 0; term < kSplitTerms; ++term) {
                            const uint32_t sa = base + (uint32_t)(term_plane_a(kSplitTerms, term) * C::kStageBytes);
                            const uint32_t sb = base + (uint32_t)(term_plane_b(kSplitTerms, term) * C::kStageBytes) +
                                                kRows128Bytes;
#pragma unroll
                            for (int kk = 0; kk < BK / UMMA_K; ++kk)
                                tcgen05_mma_bf16<kCtas>(tmem_d, operand_desc(sa, ti.a_mode, kk),
                                                        operand_desc(sb, ti.b_mode, kk), idesc,
                                                        (slot > 0 || term > 0 || kk > 0) ? 1u : 0u);
                        }
                    } else if (kWide) {
                        // both halves of the 512 accumulator columns read the same staged rows of A
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (h == 1 && ti.single) continue;
                            if (slot == 0) {  // this half must have been drained by the previous tile's epilogue
                                if (!MBAR_WAIT(1, &bars->tmem_empty[h], half_phase[h] ^ 1u)) {
                                    ok = false;
                                    break;
                                }
                                tcgen05_fence_after();
                            }
                            const bool alias = h == 0 && ti.symmetric && ti.n0 == ti.m0;  // B's rows are A's
                            const uint32_t sb = alias ? base : base + kRows128Bytes + (uint32_t)(h * kRows128Bytes);
#pragma unroll
                            for (int kk = 0; kk < BK / UMMA_K; ++kk)
                                tcgen05_mma_bf16<kCtas>(tmem_base + (uint32_t)(h * kAccCols), operand_desc(base, ti.a_mode, kk),
                                                        operand_desc(sb, ti.b_mode, kk), idesc, (slot > 0 || kk > 0) ? 1u : 0u);
                        }
                        if (!ok) break;
                    } else {
                        const uint32_t sa = base;
                        const uint32_t sb = (kCtas == 2 && ti.b_is_a) ? sa : sa + kRows128Bytes;
#pragma unroll
                        for (int kk = 0; kk < BK / UMMA_K; ++kk)
                            tcgen05_mma_bf16<kCtas>(tmem_d, operand_desc(sa, ti.a_mode, kk),
                                                    operand_desc(sb, ti.b_mode, kk), idesc, (slot > 0 || kk > 0) ? 1u : 0u);
                    }
                    tcgen05_commit<kCtas>(&bars->empty[stage]);  // slot reusable once these MMAs have read it
                    if (++stage == kRing) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                if (kWide) {  // the halves this tile used are complete (in every CTA)
                    tcgen05_commit<kCtas>(&bars->tmem_full[0]);
                    half_phase[0] ^= 1u;
                    if (!ti.single) {
                        tcgen05_commit<kCtas>(&bars->tmem_full[1]);
                        half_phase[1] ^= 1u;
                    }
                } else {
                    tcgen05_commit<kCtas>(&bars->tmem_full[acc]);  // accumulator complete (in every CTA)
                    if (++acc == 2) {
                        acc = 0;
                        acc_phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                bars->abort = 1;
                atomicExch(error_flag, 2);
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue (warps 2..9 of every CTA) ----------------
        const int quarter = warp & 3;          // the TMEM lane quarter this warp may read
        const int col_half = (warp - 2) >> 2;  // which 128 of the 256 accumulator columns
        const uint32_t my_stage = smem_u32(epi_stage) + (uint32_t)((warp - 2) * kStageWarpBytes);  // plain kernel only
        int acc = 0;
        uint32_t acc_phase = 0;
        uint32_t half_phase[2] = {0u, 0u};
        bool ok = true;
        TileInfo next = fetch_tile(problems, tiles, n_tiles, present, group_id);
        for (int t = group_id; t < n_tiles && ok; t += n_groups) {
            const TileInfo ti = next;
            next = fetch_tile(problems, tiles, n_tiles, present, t + n_groups);
            if (ti.skipped) continue;
            const TcGemmProblem *p = ti.p;
            const int M = p->M, N = p->N;
            const int epi = p->epilogue;
            __nv_bfloat16 *out_bf16 = p->out_bf16;
            // a launch that applies its result keeps the f32 update only on request
            float *apply_w = ap.enabled ? p->apply_w : nullptr;
            const int64_t apply_pos = p->apply_arena_pos;
            float *out_f32 = (apply_w != nullptr && !ap.keep_update) ? nullptr : p->out_f32;
            const __nv_bfloat16 *in_bf16 = p->in_bf16;  // TC_EPI_NS_COMBINE: the planes of X at the output position
            // Frobenius normalisation folded into the first iteration (plain bf16 path): the operand is
            // the unnormalised update u, the accumulator is scaled by 1/norm (or its square)
            // split operands carry 2^15 each (Gram: acc = 2^30 G, the exponent of tiny updates cancels
            // in what is stored); the update works in the scaled domain, see drain_generic
            float acc_scale = kSplit ? kSplitInvScale * kSplitInvScale : 1.0f;
            int split_e = 0;
            if (kSplit && epi == TC_EPI_NS_COMBINE) {
                if (p->split_sumsq) split_e = split_exponent(*p->split_sumsq);
                acc_scale = ldexpf(1.0f, 2 * split_e - 15);  // acc = 2^(30 - 3e) (X G)  ->  2^(15 - e) (X G)
            }
            if (!kSplit && p->scale_sumsq) {
                const float norm = sqrtf(*p->scale_sumsq + 1e-8f);  // muon.rs:59
                const float inv = norm > 1e-8f ? 1.0f / norm : 1.0f;  // muon.rs:60
                acc_scale = p->scale_power == 2 ? inv * inv : inv;
            }
            if (kSplit && epi == TC_EPI_IDENTITY && p->split_sumsq) {
                // the last product of the chain form: one operand is X_0 at 2^(15 - e), the other a square
                // whose power-of-two scale the host folded into extra_scale
                split_e = split_exponent(*p->split_sumsq);
                acc_scale = ldexpf(acc_scale, split_e);
            }
            if (p->extra_scale != 0.0f) acc_scale *= p->extra_scale;
            // a second output of a 3I - G launch: G itself (drained by a second pass over the accumulator)
            __nv_bfloat16 *out2_bf16 = (kDual && !kSplit && epi == TC_EPI_THREE_I_MINUS) ? p->out2_bf16 : nullptr;
            const int64_t ld = p->ld_out;
            const int out_planes = kSplit ? p->n_out_planes : 1;  // 1: bf16 rounding; 2: the two f16 planes
            const int out_planes_in = kSplit ? kSplitPlanes : 1;  // planes of the operands (and of in_bf16)
            const int64_t plane_stride = p->out_plane_stride;
            const bool bf16_rows_32b = (ld % 16) == 0;  // every bf16 output row starts on a 32-byte boundary
            const bool transpose = !kSplit && p->transpose_out != 0;
            // One accumulator of 256 columns per tile, alternating between the two TMEM buffers; or
            // (wide tile) both buffers in every tile, as the two halves of its 512 columns.
#pragma unroll 1
            for (int h = 0; h < C::kHalves && ok; ++h) {
            if (kWide && h == 1 && ti.single) break;
            const int buf = kWide ? h : acc;
            // a half of a symmetric wide tile is mirrored when it lies right of the diagonal
            const bool mirror = (kWide && ti.symmetric) ? (ti.n0 + h * BN > ti.m0) : ti.mirror;
            // warp-uniform: near expiry some lanes could see the barrier flip and others give up;
            // the whole warp must take the same branch before the aligned tcgen05.ld below
            if (!__all_sync(0xffffffffu, MBAR_WAIT(3, &bars->tmem_full[buf], kWide ? half_phase[h] : acc_phase))) {
                ok = false;
                break;
            }
#ifdef VB_TC_TIMING
            const long long t_body0 = clock64();
#endif
            tcgen05_fence_after();
            const int row = ti.m0 + (int)cta_rank * BM + quarter * 32 + lane;
            const int tile_col0 = ti.n0 + h * BN + col_half * (BN / 2);
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) +
                                   (uint32_t)(buf * kAccCols + col_half * (BN / 2));
            // Common case of the plain bf16 kernel: the warp's 128 columns lie inside the matrix and
            // output rows start on 32-byte boundaries.
            // (one staging buffer per warp: a launch writes its result row-major either as bf16 or as f32)
            const bool fast = !kSplit && tile_col0 + BN / 2 <= N && bf16_rows_32b &&
                              (out_bf16 == nullptr || transpose || (out_f32 == nullptr && apply_w == nullptr)) &&
                              (epi == TC_EPI_HALF || epi == TC_EPI_THREE_I_MINUS || epi == TC_EPI_IDENTITY ||
                               (kDual && epi == TC_EPI_NS_COMBINE));
            // one pass over the accumulator per output: 3I - G, then (if asked for) G itself
            const int n_pass = (kDual && out2_bf16 != nullptr) ? 2 : 1;
#pragma unroll 1
            for (int pass = 0; pass < n_pass; ++pass) {
                const int epi_p = pass == 0 ? epi : (int)TC_EPI_IDENTITY;
                __nv_bfloat16 *const out_p = pass == 0 ? out_bf16 : out2_bf16;
                if (fast) {
                    // (a * s) * 0.5 == a * (s * 0.5) and -(a * s) == a * (-s) exactly
                    if (epi_p == TC_EPI_HALF)
                        drain_fast<TC_EPI_HALF>(taddr, row - lane, tile_col0, M, 0.5f * acc_scale, lane, out_p, out_f32,
                                                mirror, transpose, ld, apply_w, apply_pos, ap, my_stage);
                    else if (epi_p == TC_EPI_THREE_I_MINUS)
                        drain_fast<TC_EPI_THREE_I_MINUS>(taddr, row - lane, tile_col0, M, -acc_scale, lane, out_p,
                                                         out_f32, mirror, transpose, ld, nullptr, 0, ap, my_stage);
                    else if (kDual && epi_p == TC_EPI_NS_COMBINE)
                        drain_fast<TC_EPI_IDENTITY, kDual>(taddr, row - lane, tile_col0, M, -0.5f * acc_scale, lane, out_p,
                                                           nullptr, mirror, false, ld, nullptr, 0, ap, my_stage, in_bf16);
                    else
                        drain_fast<TC_EPI_IDENTITY>(taddr, row - lane, tile_col0, M, acc_scale, lane, out_p, out_f32,
                                                    mirror, transpose, ld, nullptr, 0, ap, my_stage);
                } else {
                    DrainArgs da;
                    da.taddr = taddr; da.row = row; da.tile_col0 = tile_col0; da.M = M; da.N = N; da.epi = epi_p;
                    da.lane = lane; da.acc_scale = acc_scale; da.split_e = split_e; da.ld = ld; da.plane_stride = plane_stride;
                    da.out_planes = out_planes; da.out_planes_in = out_planes_in; da.bf16_rows_32b = bf16_rows_32b;
                    da.mirror = mirror; da.transpose = transpose; da.out_bf16 = out_p; da.out_f32 = out_f32; da.in_bf16 = in_bf16;
                    da.apply_w = apply_w; da.apply_pos = apply_pos; da.ap = &ap;
                    drain_generic<kSplit, kSplit || kDual>(da);
                }
            }
            tcgen05_fence_before();
            __syncwarp();
#ifdef VB_TC_TIMING
            if (blockIdx.x == 0 && warp == 2 && lane == 0) {
                atomicAdd(&g_wait_cycles[8], (unsigned long long)(clock64() - t_body0));
                atomicAdd(&g_wait_cycles[10], 1ull);
            }
#endif
            if (lane == 0) {
                if (kCtas == 2) mbar_remote_arrive(map_to_cta(smem_u32(&bars->tmem_empty[buf]), 0));
                else mbar_arrive(&bars->tmem_empty[buf]);
            }
            if (kWide) half_phase[h] ^= 1u;
            }  // halves
            if (!kWide && ++acc == 2) {
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
        for (int s = 0; s < C::kStages; ++s)
            for (uint32_t i = 0; i < 4096u; ++i)
                if (mbar_try_wait(&bars->full[s], 0) || mbar_try_wait(&bars->full[s], 1)) break;
    }
    __syncthreads();
    if (kCtas == 2) cluster_sync_all();  // neither CTA leaves while its peer may still signal it or read its operands
    if (warp == 1) {
        tcgen05_fence_after();
        if (kCtas == 2)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                         "r"((uint32_t)kTmemCols)
                         : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                         "r"((uint32_t)kTmemCols)
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

}  // namespace

void tc_gemm_tile_shape(int *bm, int *bn)
{
    *bm = tc_use_pair() ? 2 * BM : BM;
    *bn = BN;
}

// How an operand whose rows are indexed by k (an "MN-major" operand) is best staged: through
// the 3-D view when its row length is a multiple of 64 elements, else as 64 x 64 boxes.
int tc_mn_major_mode(int64_t inner) { return (inner % 64) == 0 ? TC_OP_MN_3D : TC_OP_MN_BOXES; }

// Tensor map over `planes` row-major bf16 matrices [outer][inner] that lie `plane_stride`
// elements apart (planes = 1 for plain operands, 3 for split ones), 128-byte swizzle,
// out-of-range elements read as zero.  `mode` selects the box the kernel will ask for (see
// load_rows128); the plane is the outermost coordinate.
int make_bf16_tensor_map(void *map_out, const void *base, int64_t inner, int64_t outer, int mode, int planes,
                         int64_t plane_stride)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(VB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((inner % 8) != 0 || (reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (plane_stride % 8) != 0)
        return fail(VB_ERR_UNSUPPORTED, "TMA needs 16-byte aligned rows (inner extent %lld)", (long long)inner);
    // plain operands (planes <= 1) get maps without a plane dimension; split operands get one
    // more, outermost, dimension
    const bool with_planes = planes > 1;
    const cuuint64_t pstride = (cuuint64_t)plane_stride * 2;
    CUresult r;
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (mode == TC_OP_MN_3D) {
        if ((inner % 64) != 0) return fail(VB_ERR_INVALID_ARG, "the 3-D operand view needs rows of a multiple of 64");
        cuuint64_t dims[4] = {64, (cuuint64_t)outer, (cuuint64_t)(inner / 64), (cuuint64_t)planes};
        cuuint64_t strides[3] = {(cuuint64_t)inner * 2, 128, pstride};
        cuuint32_t box[4] = {64, 64, 2, 1};
        r = fn(reinterpret_cast<CUtensorMap *>(map_out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, with_planes ? 4 : 3,
               const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)planes};
        cuuint64_t strides[2] = {(cuuint64_t)inner * 2, pstride};
        cuuint32_t box[3] = {(cuuint32_t)BK, mode == TC_OP_K_MAJOR ? 128u : (cuuint32_t)kBoxRows, 1};
        r = fn(reinterpret_cast<CUtensorMap *>(map_out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, with_planes ? 3 : 2,
               const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return fail(VB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return VB_OK;
}

template <int kCtas, bool kSplit, bool kWide, bool kDual = false>
static int launch_variant(const TcGemmProblem *d_problems, const GemmTile *d_tiles, int n_tiles,
                          const uint8_t *d_present, int *d_error_flag, int sm_count, cudaStream_t stream,
                          uint32_t wait_limit, const TcApplyArgs &ap)
{
    static bool attr_set = false;
    if (!attr_set) {
        VB_CUDA(cudaFuncSetAttribute(ns_gemm_tc_kernel<kCtas, kSplit, kWide, kDual>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem_bytes<kCtas, kSplit, kWide>()));
        attr_set = true;
    }
    if (kCtas == 1) {
        int grid = sm_count;  // one persistent CTA per SM (it owns all 512 TMEM columns)
        if (grid > n_tiles) grid = n_tiles;
        ns_gemm_tc_kernel<kCtas, kSplit, kWide, kDual><<<grid, kThreads, smem_bytes<kCtas, kSplit, kWide>(), stream>>>(
            d_problems, d_tiles, n_tiles, d_present, d_error_flag, wait_limit, ap);
        VB_CUDA(cudaGetLastError());
        return VB_OK;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes<kCtas, kSplit, kWide>();
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // A persistent grid must be fully resident: ask how many CTA pairs the device holds at once.
    static int max_clusters = 0;
    if (max_clusters == 0) {
        cfg.gridDim = dim3((unsigned)(sm_count / 2 * 2));
        int n = 0;
        VB_CUDA(cudaOccupancyMaxActiveClusters(&n, ns_gemm_tc_kernel<kCtas, kSplit, kWide, kDual>, &cfg));
        if (n < 1) return fail(VB_ERR_CUDA, "the device cannot hold a 2-CTA cluster of the GEMM kernel");
        max_clusters = n;
    }
    int clusters = max_clusters;
    if (clusters > n_tiles) clusters = n_tiles;
    cfg.gridDim = dim3((unsigned)(clusters * 2));
    VB_CUDA(cudaLaunchKernelEx(&cfg, ns_gemm_tc_kernel<kCtas, kSplit, kWide, kDual>, d_problems, d_tiles, n_tiles, d_present,
                               d_error_flag, wait_limit, ap));
    return VB_OK;
}

// split: the problems' operands are two f16 planes (all problems of a launch are alike).
int launch_ns_gemm_tc(const TcGemmProblem *d_problems, const GemmTile *d_tiles, int n_tiles,
                      const uint8_t *d_present, int *d_error_flag, int sm_count, cudaStream_t stream,
                      uint32_t wait_limit, bool split, const TcApplyArgs *apply, bool wide, bool dual)
{
    if (n_tiles <= 0) return VB_OK;
    if (wait_limit == 0) wait_limit = kDefaultWaitLimit;
    const TcApplyArgs ap = apply ? *apply : TcApplyArgs{};
    if (dual) {
        if (split || wide) return fail(VB_ERR_INVALID_ARG, "a second output exists for the plain kernel");
        return tc_use_pair() ? launch_variant<2, false, false, true>(d_problems, d_tiles, n_tiles, d_present, d_error_flag,
                                                                     sm_count, stream, wait_limit, ap)
                             : launch_variant<1, false, false, true>(d_problems, d_tiles, n_tiles, d_present, d_error_flag,
                                                                     sm_count, stream, wait_limit, ap);
    }
    if (wide) {
        if (split || !tc_use_pair()) return fail(VB_ERR_INVALID_ARG, "the wide tile exists for the plain pair kernel");
        return launch_variant<2, false, true>(d_problems, d_tiles, n_tiles, d_present, d_error_flag, sm_count, stream,
                                              wait_limit, ap);
    }
    if (tc_use_pair())
        return split ? launch_variant<2, true, false>(d_problems, d_tiles, n_tiles, d_present, d_error_flag, sm_count,
                                                      stream, wait_limit, ap)
                     : launch_variant<2, false, false>(d_problems, d_tiles, n_tiles, d_present, d_error_flag, sm_count,
                                                       stream, wait_limit, ap);
    return split ? launch_variant<1, true, false>(d_problems, d_tiles, n_tiles, d_present, d_error_flag, sm_count, stream,
                                                  wait_limit, ap)
                 : launch_variant<1, false, false>(d_problems, d_tiles, n_tiles, d_present, d_error_flag, sm_count, stream,
                                                   wait_limit, ap);
}

// Columns of a wide tile, or 0 where the wide kernel is not in use.  It is off unless
// VB_TC_WIDE=1: measured on the 96-matrix configuration it fetches a quarter less from L2 but
// cannot hide its drain (all 512 TMEM columns belong to one tile), and the update products end up
// 10 % slower than with 256 x 256 tiles and two accumulators (Newton-Schulz chain 5.14 ms against
// 4.87 ms per step).  Kept selectable, and covered by the parity tests when selected.
int tc_gemm_wide_cols()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("VB_TC_WIDE");
        v = (tc_use_pair() && e && *e == '1') ? 2 * BN : 0;
    }
    return v;
}

// The same tile for the Gram products: rows of tiles on and above the diagonal, one or two halves
// each.  Off unless VB_TC_WIDE_GRAM=1: although the contraction is four times longer (the exposed
// drain weighs less) and a quarter less is fetched from L2, the mixed tile costs balance worse over
// the 74 CTA pairs and the chain measured 5.12 ms against 4.88 ms per step.
int tc_gemm_wide_gram_cols()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("VB_TC_WIDE_GRAM");
        v = (tc_use_pair() && e && *e == '1') ? 2 * BN : 0;
    }
    return v;
}

}  // namespace vb
