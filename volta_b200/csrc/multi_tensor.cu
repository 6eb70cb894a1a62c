// Fused multi-tensor Adam / SGD update for sm_100a.
//
// One launch updates every tensor of an optimizer: the grid strides over a chunk table
// (fixed-length pieces of tensors, so ragged tensor lists load-balance), each chunk is
// streamed with 256-bit (else 128-bit) loads/stores of param / grad / state, and every element is
// touched exactly once (HBM traffic = 28 B/param for Adam, 20 B/param for SGD with
// momentum, 12 B/param for plain SGD).
//
// Arithmetic contract: bit-identical to Volta's CPU optimizers
// (src/nn/optim/adam.rs:139-205, src/nn/optim/sgd.rs:189-238).  Rust never contracts
// a*b+c, so every operation below is an explicitly rounded intrinsic (__fmul_rn,
// __fadd_rn, ... are never fused by nvcc) and __fmaf_rn appears only where the
// reference writes mul_add.  Division and square root are the IEEE-rounded forms.
#include <cuda_bf16.h>
#include <stdlib.h>

#include <mutex>

#include "vb_internal.h"

namespace vb {

namespace {

constexpr int kThreads = 256;
// Launch shape found by sweeping on a B200 with realistic (non-zero) data: 256-bit accesses,
// one vector per array per thread in flight, and exactly 512 resident threads per SM
// (2 CTAs x 256).  The step runs under the board's power cap: more resident threads or
// deeper unrolling put more requests in flight than the memory system sustains and cost
// 5-15 % (768 threads/SM: -7 %, 1024: -6 %, 2048: -15 %).
constexpr int kCtasPerSm = 2;            // Adam (launch bound of the kernel template: up to kCtasPerSmMax)
constexpr int kCtasPerSmMax = 3;
constexpr int kSgdMomentumCtasPerSm = 2;
constexpr int kSgdCtasPerSm = 3;           // measured on C3-sized lists: SGD 3 (6.77 TB/s), SGD+momentum 2 (6.72), Adam 2 (6.69)
constexpr int kVecElems = 8;  // floats per 256-bit access

struct alignas(32) Vec8 {
    float4 lo, hi;
};

// 256-bit global accesses (sm_100: ld/st.global.v8.f32).  Loads bypass L1: every byte is
// touched once per step.
__device__ __forceinline__ Vec8 ld_vec8(const Vec8 *p)
{
    Vec8 r;
    asm volatile("ld.global.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.lo.x), "=f"(r.lo.y), "=f"(r.lo.z), "=f"(r.lo.w), "=f"(r.hi.x), "=f"(r.hi.y),
                   "=f"(r.hi.z), "=f"(r.hi.w)
                 : "l"(p));
    return r;
}

__device__ __forceinline__ void st_vec8(Vec8 *p, const Vec8 &r)
{
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(r.lo.x), "f"(r.lo.y),
                 "f"(r.lo.z), "f"(r.lo.w), "f"(r.hi.x), "f"(r.hi.y), "f"(r.hi.z), "f"(r.hi.w)
                 : "memory");
}

// Division and square root are the IEEE-rounded forms.  Their quick hardware sequence covers
// operands inside the normal range; a subnormal numerator or quotient sends the warp through a
// long fallback and the kernel turns from HBM-bound into ALU-bound (measured: 6.7 -> 4.5 TB/s when
// most elements are affected, e.g. after thousands of steps on one constant gradient, which trains
// every parameter to the fixed point g + wd * theta = 0 where the effective gradient and the first
// moment underflow).  Routing those cases around the fallback by exact power-of-two scaling was
// tried: the extra compares cost 5-8 % on ordinary values, because the kernel already sits at the
// edge of the issue rate, and a subnormal quotient needs the fallback anyway.  Exactness wins.
template <int OP>
__device__ __forceinline__ void update_one(float &p, float g, float &s1, float &s2,
                                           const StepScalars &s)
{
    // adam.rs:150-154 / sgd.rs:201-205: weight decay folded into a copy of the gradient
    if (s.weight_decay != 0.0f) g = __fadd_rn(g, __fmul_rn(s.weight_decay, p));
    if (OP == OP_ADAM) {
        // adam.rs:172-185
        s1 = __fmaf_rn(s.beta1, s1, __fmul_rn(s.one_minus_beta1, g));
        s2 = __fmaf_rn(s.beta2, s2, __fmul_rn(s.one_minus_beta2, __fmul_rn(g, g)));
        // adam.rs:196-204: theta -= lr * m_hat / (sqrt(v_hat) + eps)
        const float m_hat = __fmul_rn(s1, s.m_hat_scale);
        const float v_hat = __fmul_rn(s2, s.v_hat_scale);
        p = __fsub_rn(p, __fdiv_rn(__fmul_rn(s.lr, m_hat), __fadd_rn(__fsqrt_rn(v_hat), s.eps)));
    } else if (OP == OP_SGD_MOMENTUM) {
        // sgd.rs:216-218, 225-227
        s1 = __fmaf_rn(s.beta1, s1, -__fmul_rn(s.lr, g));
        p = __fadd_rn(p, s1);
    } else {
        // sgd.rs:234-236
        p = __fsub_rn(p, __fmul_rn(s.lr, g));
    }
}

template <int OP>
__device__ __forceinline__ void update_vec(float4 &p, const float4 &g, float4 &a, float4 &b,
                                           const StepScalars &s)
{
    update_one<OP>(p.x, g.x, a.x, b.x, s);
    update_one<OP>(p.y, g.y, a.y, b.y, s);
    update_one<OP>(p.z, g.z, a.z, b.z, s);
    update_one<OP>(p.w, g.w, a.w, b.w, s);
}

__device__ __forceinline__ FatChunk load_chunk(const FatChunk *c)
{
    // 48 bytes as three 128-bit read-only loads
    const uint4 *q = reinterpret_cast<const uint4 *>(c);
    union {
        uint4 v[3];
        FatChunk f;
    } u;
    u.v[0] = __ldg(q);
    u.v[1] = __ldg(q + 1);
    u.v[2] = __ldg(q + 2);
    return u.f;
}

// f32 -> bf16, round to nearest even (the conversion Volta's storage uses for its bf16
// dtype, src/storage.rs:499-505), two per 32-bit word, low element in the low half.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

__device__ __forceinline__ uint16_t bf16_bits(float x)
{
    const __nv_bfloat16 v = __float2bfloat16_rn(x);
    return *reinterpret_cast<const uint16_t *>(&v);
}

// Gradient of one element under data parallelism: the sum of every rank's gradient at the
// same arena position, added in rank order (one rounded f32 add per rank, so the result does
// not depend on which rank computes it), then scaled.  The peers' values come over NVLink as
// plain loads; the loop is unrolled so that the table stays in the constant bank.
__device__ __forceinline__ const float *grad_source(const PeerTable &pt, const float *local, ptrdiff_t arena_pos, int k)
{
    // rank k's gradient arena at this position: peers are stored in rank order without this rank
    const float *arena = k == pt.rank ? local : (k < pt.rank ? pt.grad_base[k < kMaxPeers ? k : 0] : pt.grad_base[k > 0 ? k - 1 : 0]);
    return arena + arena_pos;
}

__device__ __forceinline__ Vec8 sum_grads8(const PeerTable &pt, const float *local, ptrdiff_t arena_pos, uint32_t i)
{
    Vec8 term[kMaxPeers + 1];
#pragma unroll
    for (int k = 0; k <= kMaxPeers; ++k)  // all loads first: NVLink latency overlaps
        if (k <= pt.n_grad) term[k] = ld_vec8(reinterpret_cast<const Vec8 *>(grad_source(pt, local, arena_pos, k)) + i);
    Vec8 acc = term[0];
#pragma unroll
    for (int k = 1; k <= kMaxPeers; ++k) {
        if (k <= pt.n_grad) {
            acc.lo.x = __fadd_rn(acc.lo.x, term[k].lo.x); acc.lo.y = __fadd_rn(acc.lo.y, term[k].lo.y);
            acc.lo.z = __fadd_rn(acc.lo.z, term[k].lo.z); acc.lo.w = __fadd_rn(acc.lo.w, term[k].lo.w);
            acc.hi.x = __fadd_rn(acc.hi.x, term[k].hi.x); acc.hi.y = __fadd_rn(acc.hi.y, term[k].hi.y);
            acc.hi.z = __fadd_rn(acc.hi.z, term[k].hi.z); acc.hi.w = __fadd_rn(acc.hi.w, term[k].hi.w);
        }
    }
    const float sc = pt.grad_scale;
    acc.lo.x = __fmul_rn(acc.lo.x, sc); acc.lo.y = __fmul_rn(acc.lo.y, sc); acc.lo.z = __fmul_rn(acc.lo.z, sc);
    acc.lo.w = __fmul_rn(acc.lo.w, sc); acc.hi.x = __fmul_rn(acc.hi.x, sc); acc.hi.y = __fmul_rn(acc.hi.y, sc);
    acc.hi.z = __fmul_rn(acc.hi.z, sc); acc.hi.w = __fmul_rn(acc.hi.w, sc);
    return acc;
}

__device__ __forceinline__ float sum_grads1(const PeerTable &pt, const float *local, ptrdiff_t arena_pos, uint32_t i)
{
    float acc = 0.0f;
#pragma unroll
    for (int k = 0; k <= kMaxPeers; ++k) {
        if (k <= pt.n_grad) {
            const float t = grad_source(pt, local, arena_pos, k)[i];
            acc = k == 0 ? t : __fadd_rn(acc, t);
        }
    }
    return __fmul_rn(acc, pt.grad_scale);
}

// PEERS: besides the local arena, every updated parameter is stored into the same arena
// position on every peer GPU (plain st.global to peer-mapped memory over NVLink), so the
// all-gather of updated parameters rides along with the update, piece by piece.
// HALF: 1 = the new parameter is also written, rounded to bf16, into the local bf16 copy of the
// arena; 2 = and into every peer's bf16 copy (2 bytes per parameter over NVLink instead of 4
// when PEERS is off).
// GSUM: the gradient is summed over the ranks' gradient arenas (see sum_grads8).
template <int OP, bool PEERS, int HALF, bool GSUM>
__device__ __forceinline__ void update_chunk(const FatChunk &ch, const StepScalars &s, const PeerTable &pt)
{
    constexpr bool kHasS1 = (OP != OP_SGD);
    constexpr bool kHasS2 = (OP == OP_ADAM);
    float *__restrict__ p = ch.p;
    const float *__restrict__ g = ch.g;
    float *__restrict__ s1 = kHasS1 ? ch.s1 : nullptr;
    float *__restrict__ s2 = kHasS2 ? ch.s2 : nullptr;
    const uint32_t n = ch.len;

    const ptrdiff_t arena_pos = (PEERS || HALF || GSUM) ? (p - pt.local_base) : 0;  // element offset inside the arena
    // peers to store to: none for a chunk of the replicated tail, which every rank computes itself
    const int n_peers = (PEERS && ch.local_only == 0) ? pt.n : 0;
    const int n_half_peers = (HALF == 2 && ch.local_only == 0) ? pt.n_half : 0;
    const float *g_arena = g - arena_pos;  // this rank's gradient arena (same layout as the parameters)

    uintptr_t align_bits = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g);
    if (kHasS1) align_bits |= reinterpret_cast<uintptr_t>(s1);
    if (kHasS2) align_bits |= reinterpret_cast<uintptr_t>(s2);

    uint32_t done = 0;
    if ((align_bits & 31u) == 0) {
        const uint32_t n8 = n >> 3;
        Vec8 *__restrict__ p8 = reinterpret_cast<Vec8 *>(p);
        const Vec8 *__restrict__ g8 = reinterpret_cast<const Vec8 *>(g);
        Vec8 *__restrict__ a8 = reinterpret_cast<Vec8 *>(s1);
        Vec8 *__restrict__ b8 = reinterpret_cast<Vec8 *>(s2);
        for (uint32_t i = threadIdx.x; i < n8; i += kThreads) {
            Vec8 vp = ld_vec8(p8 + i), va, vb;
            const Vec8 vg = GSUM ? sum_grads8(pt, g_arena, arena_pos, i) : ld_vec8(g8 + i);
            if (kHasS1) va = ld_vec8(a8 + i);
            if (kHasS2) vb = ld_vec8(b8 + i);
            update_vec<OP>(vp.lo, vg.lo, va.lo, vb.lo, s);
            update_vec<OP>(vp.hi, vg.hi, va.hi, vb.hi, s);
            st_vec8(p8 + i, vp);
            if (PEERS) {
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r)  // unrolled: the table stays in the constant bank
                    if (r < n_peers) st_vec8(reinterpret_cast<Vec8 *>(pt.base[r] + arena_pos) + i, vp);
            }
            if (HALF) {  // arena_pos is a multiple of 8 here: 16-byte aligned bf16 octets
                const uint4 h = make_uint4(pack_bf16x2(vp.lo.x, vp.lo.y), pack_bf16x2(vp.lo.z, vp.lo.w),
                                           pack_bf16x2(vp.hi.x, vp.hi.y), pack_bf16x2(vp.hi.z, vp.hi.w));
                reinterpret_cast<uint4 *>(pt.half_local + arena_pos)[i] = h;
                if (HALF == 2) {
#pragma unroll
                    for (int r = 0; r < kMaxPeers; ++r)
                        if (r < n_half_peers) reinterpret_cast<uint4 *>(pt.half_base[r] + arena_pos)[i] = h;
                }
            }
            if (kHasS1) st_vec8(a8 + i, va);
            if (kHasS2) st_vec8(b8 + i, vb);
        }
        done = n8 << 3;
    } else if ((align_bits & 15u) == 0) {
        const uint32_t n4 = n >> 2;
        float4 *__restrict__ p4 = reinterpret_cast<float4 *>(p);
        const float4 *__restrict__ g4 = reinterpret_cast<const float4 *>(g);
        float4 *__restrict__ a4 = reinterpret_cast<float4 *>(s1);
        float4 *__restrict__ b4 = reinterpret_cast<float4 *>(s2);
        for (uint32_t i = threadIdx.x; i < n4; i += kThreads) {
            float4 vp = __ldcs(p4 + i), va, vb;
            float4 vg;
            if (GSUM) {
                vg.x = sum_grads1(pt, g_arena, arena_pos, 4 * i);
                vg.y = sum_grads1(pt, g_arena, arena_pos, 4 * i + 1);
                vg.z = sum_grads1(pt, g_arena, arena_pos, 4 * i + 2);
                vg.w = sum_grads1(pt, g_arena, arena_pos, 4 * i + 3);
            } else {
                vg = __ldcs(g4 + i);
            }
            if (kHasS1) va = __ldcs(a4 + i);
            if (kHasS2) vb = __ldcs(b4 + i);
            update_vec<OP>(vp, vg, va, vb, s);
            __stcs(p4 + i, vp);
            if (PEERS) {
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r)
                    if (r < n_peers) reinterpret_cast<float4 *>(pt.base[r] + arena_pos)[i] = vp;
            }
            if (HALF) {
                const uint2 h = make_uint2(pack_bf16x2(vp.x, vp.y), pack_bf16x2(vp.z, vp.w));
                reinterpret_cast<uint2 *>(pt.half_local + arena_pos)[i] = h;
                if (HALF == 2) {
#pragma unroll
                    for (int r = 0; r < kMaxPeers; ++r)
                        if (r < n_half_peers) reinterpret_cast<uint2 *>(pt.half_base[r] + arena_pos)[i] = h;
                }
            }
            if (kHasS1) __stcs(a4 + i, va);
            if (kHasS2) __stcs(b4 + i, vb);
        }
        done = n4 << 2;
    }
    // ragged tail (n mod 8 / n mod 4) or a chunk whose pointers are not 16-byte aligned
    for (uint32_t i = done + threadIdx.x; i < n; i += kThreads) {
        float vp = p[i], va = 0.0f, vb = 0.0f;
        const float vg = GSUM ? sum_grads1(pt, g_arena, arena_pos, i) : g[i];
        if (kHasS1) va = s1[i];
        if (kHasS2) vb = s2[i];
        update_one<OP>(vp, vg, va, vb, s);
        p[i] = vp;
        if (PEERS) {
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
                if (r < n_peers) pt.base[r][arena_pos + i] = vp;
        }
        if (HALF) {
            const uint16_t h = bf16_bits(vp);
            pt.half_local[arena_pos + i] = h;
            if (HALF == 2) {
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r)
                    if (r < n_half_peers) pt.half_base[r][arena_pos + i] = h;
            }
        }
        if (kHasS1) s1[i] = va;
        if (kHasS2) s2[i] = vb;
    }
}

// CHECK_PRESENT = false is the common case (every tensor has a gradient): the descriptor of
// the next chunk is fetched while the current one streams, so no dependent-load latency
// sits between chunks.  With CHECK_PRESENT the per-tensor flag is looked up as well.
template <int OP, bool CHECK_PRESENT, bool PEERS, int HALF, bool GSUM>
__global__ void __launch_bounds__(kThreads, GSUM ? 2 : kCtasPerSmMax)  // GSUM holds up to 8 vectors of gradients
multi_tensor_update_kernel(const FatChunk *__restrict__ chunks, int64_t n_chunks,
                           const uint8_t *__restrict__ present, const StepScalars s, const PeerTable pt)
{
    int64_t c = blockIdx.x;
    if (c >= n_chunks) return;
    if ((PEERS || HALF == 2 || GSUM) && fence_failed(pt.fence_error)) return;  // the fence before this launch gave up
    FatChunk cur = load_chunk(chunks + c);
    for (;;) {
        const int64_t cn = c + gridDim.x;
        const bool has_next = cn < n_chunks;
        FatChunk nxt = cur;
        if (has_next) nxt = load_chunk(chunks + cn);  // in flight while `cur` is processed
        // `grad == None` -> skip: adam.rs:81-84, sgd.rs:75-78
        if (!CHECK_PRESENT || present[cur.tensor] != 0) update_chunk<OP, PEERS, HALF, GSUM>(cur, s, pt);
        if (!has_next) break;
        cur = nxt;
        c = cn;
    }
}

}  // namespace

float powi_f32(float a, int b)
{
    const bool recip = b < 0;
    volatile float r = 1.0f;  // volatile: keep every product rounded to f32
    volatile float x = a;
    for (;;) {
        if (b & 1) r = r * x;
        b /= 2;
        if (b == 0) break;
        x = x * x;
    }
    return recip ? 1.0f / r : r;
}

StepScalars make_scalars(int op, float lr, float beta1, float beta2, float eps, float wd, int64_t t)
{
    StepScalars s{};
    s.lr = lr;
    s.beta1 = beta1;
    s.beta2 = beta2;
    s.eps = eps;
    s.weight_decay = wd;
    if (op == OP_ADAM) {
        volatile float omb1 = 1.0f - beta1, omb2 = 1.0f - beta2;
        s.one_minus_beta1 = omb1;
        s.one_minus_beta2 = omb2;
        // adam.rs:188-189: `self.t as i32`
        volatile float d1 = 1.0f - powi_f32(beta1, (int)t);
        volatile float d2 = 1.0f - powi_f32(beta2, (int)t);
        s.m_hat_scale = 1.0f / d1;
        s.v_hat_scale = 1.0f / d2;
    }
    return s;
}

int64_t pick_chunk_len(int64_t total_elements, int sm_count)
{
    // One or two passes of a CTA (256 threads x 8 floats = 2048 elements per pass): short
    // enough that every CTA walks >100 chunks of a large model (static round-robin then
    // balances to <1 %), long enough to amortise the 48-byte descriptor.  Measured on B200:
    // 2 Ki .. 8 Ki elements stream equally fast, longer chunks lose a few percent.
    const int64_t quantum = kThreads * kVecElems;
    int64_t len = total_elements / ((int64_t)sm_count * 64);
    len = (len + quantum - 1) / quantum * quantum;
    if (len < quantum) len = quantum;
    if (len > 2 * quantum) len = 2 * quantum;
    return len;
}

// Resident CTAs per SM by operation (fewer arrays per element -> fewer bytes in flight per
// thread -> one more CTA to reach the same total); VB_CTAS_PER_SM overrides for experiments.
static int ctas_per_sm(int op)
{
    static int override_v = -1;
    if (override_v < 0) {
        const char *e = getenv("VB_CTAS_PER_SM");
        override_v = e ? atoi(e) : 0;
    }
    if (override_v >= 1 && override_v <= kCtasPerSmMax) return override_v;
    return op == OP_ADAM ? 2 : op == OP_SGD_MOMENTUM ? kSgdMomentumCtasPerSm : kSgdCtasPerSm;
}

template <int OP, bool PEERS, int HALF, bool GSUM>
static void launch_variant(unsigned grid, const FatChunk *d_chunks, int64_t n_chunks, const uint8_t *d_present,
                           bool all_present, const StepScalars &s, const PeerTable &pt, cudaStream_t stream)
{
    if (all_present)
        multi_tensor_update_kernel<OP, false, PEERS, HALF, GSUM><<<grid, kThreads, 0, stream>>>(d_chunks, n_chunks,
                                                                                               d_present, s, pt);
    else
        multi_tensor_update_kernel<OP, true, PEERS, HALF, GSUM><<<grid, kThreads, 0, stream>>>(d_chunks, n_chunks,
                                                                                              d_present, s, pt);
}

template <int OP>
static void launch_op(unsigned grid, const FatChunk *d_chunks, int64_t n_chunks, const uint8_t *d_present,
                      bool all_present, const StepScalars &s, const PeerTable *peers, cudaStream_t stream)
{
    const PeerTable pt = peers ? *peers : PeerTable{};
    const bool f32_peers = pt.n > 0;
    const int half = pt.half_local == nullptr ? 0 : pt.n_half > 0 ? 2 : 1;
#define VB_LAUNCH(P, H, G) launch_variant<OP, P, H, G>(grid, d_chunks, n_chunks, d_present, all_present, s, pt, stream)
    if (pt.n_grad > 0) {
        // gradients summed over the ranks: built for the exchanges a data-parallel step uses
        if (half == 2 && !f32_peers) VB_LAUNCH(false, 2, true);
        else if (half == 2) VB_LAUNCH(true, 2, true);
        else if (half == 1 && f32_peers) VB_LAUNCH(true, 1, true);
        else if (half == 1) VB_LAUNCH(false, 1, true);
        else if (f32_peers) VB_LAUNCH(true, 0, true);
        else VB_LAUNCH(false, 0, true);
    } else if (half == 0) {
        if (f32_peers) VB_LAUNCH(true, 0, false);
        else VB_LAUNCH(false, 0, false);
    } else if (half == 1) {
        if (f32_peers) VB_LAUNCH(true, 1, false);
        else VB_LAUNCH(false, 1, false);
    } else {
        if (f32_peers) VB_LAUNCH(true, 2, false);
        else VB_LAUNCH(false, 2, false);
    }
#undef VB_LAUNCH
}

int launch_multi_tensor(int op, const FatChunk *d_chunks, int64_t n_chunks, const uint8_t *d_present,
                        bool all_present, const StepScalars &s, int sm_count, cudaStream_t stream,
                        const PeerTable *peers)
{
    if (n_chunks <= 0) return VB_OK;
    if (op != OP_ADAM && op != OP_SGD_MOMENTUM && op != OP_SGD)
        return fail(VB_ERR_INVALID_ARG, "unknown multi-tensor op %d", op);
    int64_t grid = (int64_t)sm_count * ctas_per_sm(op);  // whole waves: a multiple of the SM count
    if (grid > n_chunks) grid = n_chunks;
    switch (op) {
        case OP_ADAM:
            launch_op<OP_ADAM>((unsigned)grid, d_chunks, n_chunks, d_present, all_present, s, peers, stream);
            break;
        case OP_SGD_MOMENTUM:
            launch_op<OP_SGD_MOMENTUM>((unsigned)grid, d_chunks, n_chunks, d_present, all_present, s, peers, stream);
            break;
        default: launch_op<OP_SGD>((unsigned)grid, d_chunks, n_chunks, d_present, all_present, s, peers, stream); break;
    }
    VB_CUDA(cudaGetLastError());
    return VB_OK;
}

// ---- bf16 copy of a run of parameters (after an upload) ---------------------------------------------
__global__ void __launch_bounds__(256)
f32_to_bf16_kernel(uint16_t *__restrict__ dst, const float *__restrict__ src, int64_t n)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t done = 0;
    if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
        const int64_t n4 = n >> 2;
        for (int64_t i = tid; i < n4; i += stride) {
            const float4 v = __ldcs(reinterpret_cast<const float4 *>(src) + i);
            reinterpret_cast<uint2 *>(dst)[i] = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
        }
        done = n4 << 2;
    }
    for (int64_t i = done + tid; i < n; i += stride) dst[i] = bf16_bits(src[i]);
}

int launch_f32_to_bf16(uint16_t *dst, const float *src, int64_t n, int sm_count, cudaStream_t stream)
{
    if (n <= 0) return VB_OK;
    int64_t grid = (n / 4 + 255) / 256;
    if (grid > (int64_t)sm_count * 8) grid = (int64_t)sm_count * 8;
    if (grid < 1) grid = 1;
    f32_to_bf16_kernel<<<(unsigned)grid, 256, 0, stream>>>(dst, src, n);
    VB_CUDA(cudaGetLastError());
    return VB_OK;
}

// ---- gradient accumulation (src/autograd.rs:140-148,158-184) -------------------------------------
// grad = present ? grad + contribution : contribution, element by element (one rounded add).
__global__ void __launch_bounds__(256)
accumulate_grad_kernel(float *__restrict__ grad, const float *__restrict__ src, int64_t n, int add)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (((reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0) {
        const int64_t n4 = n >> 2;
        for (int64_t i = tid; i < n4; i += stride) {
            float4 s4 = __ldcs(reinterpret_cast<const float4 *>(src) + i);
            if (add) {
                const float4 g4 = reinterpret_cast<const float4 *>(grad)[i];
                s4.x = __fadd_rn(g4.x, s4.x);
                s4.y = __fadd_rn(g4.y, s4.y);
                s4.z = __fadd_rn(g4.z, s4.z);
                s4.w = __fadd_rn(g4.w, s4.w);
            }
            reinterpret_cast<float4 *>(grad)[i] = s4;
        }
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride) grad[i] = add ? __fadd_rn(grad[i], src[i]) : src[i];
    } else {
        for (int64_t i = tid; i < n; i += stride) grad[i] = add ? __fadd_rn(grad[i], src[i]) : src[i];
    }
}

int launch_accumulate_grad(float *grad, const float *src, int64_t n, bool add, int sm_count, cudaStream_t stream)
{
    if (n <= 0) return VB_OK;
    int64_t blocks = (n / 4 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > (int64_t)sm_count * 8) blocks = (int64_t)sm_count * 8;
    accumulate_grad_kernel<<<(unsigned)blocks, 256, 0, stream>>>(grad, src, n, add ? 1 : 0);
    VB_CUDA(cudaGetLastError());
    return VB_OK;
}

// ---------------------------------------------------------------------------------------------
// vb_multi_tensor_step_static: the fused step for callers that must not allocate.
//
// vb_multi_tensor_step keeps its chunk table in device and pinned host memory that it
// allocates (and grows) on demand.  Some hosts cannot tolerate that inside their step: a
// runtime that has handed all device memory to its own pool, a loop that must not touch the
// allocator's locks once training has started, a plugin host that forbids allocation after
// initialisation.  This variant keeps the chunk table in a fixed array that is part of the
// library image, so a call performs no cudaMalloc / cudaHostAlloc / cudaFree at all: it
// writes the table into a fixed host array, copies it to the fixed device array on the
// engine's stream and launches the same kernel as vb_multi_tensor_step.
//
// Consequences of the fixed array, all documented in the header:
//  * capacity: VB_STATIC_MAX_CHUNKS chunks (the chunk length grows with the problem up to
//    VB_STATIC_MAX_CHUNK_ELEMS elements); larger tensor lists are rejected;
//  * every GPU that loads the library carries the array (384 KiB) until the process exits;
//  * all calls on a device share it: two calls that overlap on the GPU (different engines
//    or streams) race; calls on one engine are ordered by its stream and are safe;
//  * the host staging array is shared by every device and host thread of the process; a lock
//    around filling it and handing it to the copy keeps concurrent callers apart on the host;
//  * the first call on a device looks the array's address up (cudaGetSymbolAddress), so
//    make that first call before starting a stream capture.
// ---------------------------------------------------------------------------------------------

#define VB_STATIC_MAX_CHUNKS 8192
#define VB_STATIC_MAX_CHUNK_ELEMS (1 << 17)
#define VB_STATIC_MAX_DEVICES 64

// The scratch itself.  In host code `g_static_chunk_table` is only a handle for the runtime,
// not a device address: the address is resolved per device below.
static __device__ __align__(256) unsigned char g_static_chunk_table[VB_STATIC_MAX_CHUNKS * sizeof(FatChunk)];

namespace {

FatChunk g_static_host_table[VB_STATIC_MAX_CHUNKS];       // staging on the host, equally fixed, one per process
std::mutex g_static_host_mutex;                           // serialises host threads filling it
FatChunk *g_static_dev_ptr[VB_STATIC_MAX_DEVICES] = {};   // resolved device address, per device

// Once per device, with that device current.
int static_table_address(int device, FatChunk **out)
{
    if (device < 0 || device >= VB_STATIC_MAX_DEVICES)
        return fail(VB_ERR_UNSUPPORTED, "device %d is beyond the %d devices the static table supports", device,
                    VB_STATIC_MAX_DEVICES);
    if (!g_static_dev_ptr[device]) {
        void *ptr = nullptr;
        VB_CUDA(cudaSetDevice(device));
        VB_CUDA(cudaGetSymbolAddress(&ptr, g_static_chunk_table));
        if (!ptr) return fail(VB_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        g_static_dev_ptr[device] = static_cast<FatChunk *>(ptr);
    }
    *out = g_static_dev_ptr[device];
    return VB_OK;
}

}  // namespace
}  // namespace vb

extern "C" int vb_multi_tensor_step_static(vb_engine *engine, const vb_optimizer_step_params *hp, int64_t n_tensors,
                                           const int64_t *sizes, void *const *params, const void *const *grads,
                                           void *const *state1, void *const *state2)
{
    using namespace vb;
    int device = 0, sm_count = 0;
    cudaStream_t stream = nullptr;
    if (!hp) return fail(VB_ERR_INVALID_ARG, "null argument");
    int64_t total = 0;
    VB_TRY(check_caller_buffers(hp, n_tensors, sizes, params, grads, state1, state2, &total));
    if (!engine) return fail(VB_ERR_INVALID_ARG, "engine is null");
    if (engine_launch_info(engine, &device, &sm_count, &stream) != VB_OK) return VB_ERR_INVALID_ARG;
    if (n_tensors > VB_STATIC_MAX_CHUNKS)
        return fail(VB_ERR_UNSUPPORTED, "%lld tensors exceed the static table (%d chunks); use vb_multi_tensor_step",
                    (long long)n_tensors, VB_STATIC_MAX_CHUNKS);
    if (total == 0) return VB_OK;
    // smallest chunk length (doubling from the usual one) whose table fits the fixed array
    int64_t chunk_len = pick_chunk_len(total, sm_count);
    int64_t n_chunks = 0;
    for (;;) {
        n_chunks = 0;
        for (int64_t i = 0; i < n_tensors; ++i) n_chunks += (sizes[i] + chunk_len - 1) / chunk_len;
        if (n_chunks <= VB_STATIC_MAX_CHUNKS) break;
        if (chunk_len * 2 > VB_STATIC_MAX_CHUNK_ELEMS)
            return fail(VB_ERR_UNSUPPORTED,
                        "%lld elements in %lld tensors need %lld chunks of %lld elements; the static table holds %d "
                        "(use vb_multi_tensor_step, which allocates its table)",
                        (long long)total, (long long)n_tensors, (long long)n_chunks, (long long)chunk_len,
                        VB_STATIC_MAX_CHUNKS);
        chunk_len *= 2;
    }
    VB_CUDA(cudaSetDevice(device));
    VB_TRY(check_caller_memory(engine, hp, n_tensors, sizes, params, grads, state1, state2));
    // The host staging array is one per process: the lock keeps two host threads (driving two
    // engines, on the same or on different devices) from interleaving their tables in it.  It is
    // held until cudaMemcpyAsync returns; the source is ordinary (pageable) host memory, so by
    // then the runtime has taken its copy and the array can be refilled.
    std::lock_guard<std::mutex> lock(g_static_host_mutex);
    FatChunk *d_table = nullptr;
    VB_TRY(static_table_address(device, &d_table));  // first call on this device: resolves the address
    int64_t c = 0;
    for (int64_t i = 0; i < n_tensors; ++i) {
        for (int64_t b = 0; b < sizes[i]; b += chunk_len) {
            FatChunk &f = g_static_host_table[c++];
            f.p = (float *)params[i] + b;
            f.g = (const float *)grads[i] + b;
            f.s1 = (state1 && state1[i]) ? (float *)state1[i] + b : nullptr;
            f.s2 = (state2 && state2[i]) ? (float *)state2[i] + b : nullptr;
            f.len = (uint32_t)(sizes[i] - b < chunk_len ? sizes[i] - b : chunk_len);
            f.tensor = (uint32_t)i;
            f.local_only = 0;
        }
    }
    // The used prefix of the device table is rewritten on every call; nothing in it has to
    // start at zero and entries beyond n_chunks are never read.
    VB_CUDA(cudaMemcpyAsync(d_table, g_static_host_table, (size_t)n_chunks * sizeof(FatChunk), cudaMemcpyHostToDevice,
                            stream));
    const StepScalars s =
        make_scalars((int)hp->op, hp->lr, hp->beta1, hp->beta2, hp->eps, hp->weight_decay, (int64_t)hp->t);
    VB_TRY(launch_multi_tensor((int)hp->op, d_table, n_chunks, nullptr, /*all_present=*/true, s, sm_count, stream));
    engine_count_launch(engine);
    return VB_OK;
}
