// Muon::step on the GPU (src/nn/optim/muon.rs:108-163): ownership of matrices, the
// elementwise kernels (momentum / Nesterov, sum of squares, normalise, apply) and the
// orchestration of the Newton-Schulz GEMM chain.
//
//   K3a  momentum_kernel      v = fma(mu, v, g); u = nesterov ? mu*v + g : v      muon.rs:133-150
//   K3s  sumsq_ordered_kernel sum of u*u in the reference's left-to-right f32 order muon.rs:58
//        (VB_NS_F32), or per-chunk partial sums + ordered reduce (VB_NS_BF16)
//   K3b  normalise_kernel     x = u / sqrt(sumsq + 1e-8)                            muon.rs:59-64
//   K4/5 Newton-Schulz GEMMs  ns_gemm_f32.cu (f32) / ns_gemm_tc.cu (bf16, tcgen05)     muon.rs:67-100
//   K6   apply_kernel         w -= (lr * u) * 0.1                                   muon.rs:158-160
//
// Every kernel walks a chunk or tile table over all matrices this rank owns, so a step
// is a fixed, small number of launches whatever the number of parameters.
#include <cuda_bf16.h>

#include <math.h>
#include <stddef.h>
#include <stdlib.h>

#include <algorithm>
#include <numeric>

#include "engine.h"
#include "ns_gemm.h"

namespace vb {

namespace {

constexpr int kEwThreads = 256;

// ---- K3a: momentum (+ Nesterov), optional per-chunk sum of squares ------------------------
// TensorDesc fields here: p = weights, g = gradient, s1 = velocity, s2 = update buffer.
// `direct_bf16` (may be null): tensors flagged there feed the tensor-core chain with the
// *unnormalised* update (the 1/norm factors are applied by the first iteration's epilogues), so
// this kernel writes the bf16 operand itself and the separate normalise pass is skipped.
// Data-parallel gradients (GSUM): the gradient of an element is the sum of every rank's value at
// the same position of its gradient arena, added in rank order, then scaled (see PeerTable).
struct GradPeers {
    const float *base[kMaxPeers];  // peers' gradient arenas in rank order, without this rank
    const float *local_base;       // this rank's gradient arena
    int n, rank;
    float scale;
    const uint32_t *fence_error;   // see PeerTable::fence_error
};
__device__ __forceinline__ const float *grad_source(const GradPeers &gp, const float *local, ptrdiff_t pos, int k)
{
    const float *arena = k == gp.rank ? local : (k < gp.rank ? gp.base[k < kMaxPeers ? k : 0] : gp.base[k > 0 ? k - 1 : 0]);
    return arena + pos;
}
__device__ __forceinline__ float4 sum_grads4(const GradPeers &gp, const float *local, ptrdiff_t pos, uint32_t i)
{
    float4 term[kMaxPeers + 1];
#pragma unroll
    for (int k = 0; k <= kMaxPeers; ++k)
        if (k <= gp.n) term[k] = __ldcs(reinterpret_cast<const float4 *>(grad_source(gp, local, pos, k)) + i);
    float4 acc = term[0];
#pragma unroll
    for (int k = 1; k <= kMaxPeers; ++k) {
        if (k <= gp.n) {
            acc.x = __fadd_rn(acc.x, term[k].x); acc.y = __fadd_rn(acc.y, term[k].y);
            acc.z = __fadd_rn(acc.z, term[k].z); acc.w = __fadd_rn(acc.w, term[k].w);
        }
    }
    acc.x = __fmul_rn(acc.x, gp.scale); acc.y = __fmul_rn(acc.y, gp.scale);
    acc.z = __fmul_rn(acc.z, gp.scale); acc.w = __fmul_rn(acc.w, gp.scale);
    return acc;
}
__device__ __forceinline__ float sum_grads1(const GradPeers &gp, const float *local, ptrdiff_t pos, uint32_t i)
{
    float acc = 0.0f;
#pragma unroll
    for (int k = 0; k <= kMaxPeers; ++k) {
        if (k <= gp.n) {
            const float t = grad_source(gp, local, pos, k)[i];
            acc = k == 0 ? t : __fadd_rn(acc, t);
        }
    }
    return __fmul_rn(acc, gp.scale);
}

template <bool PARTIALS, bool GSUM>
__global__ void __launch_bounds__(kEwThreads)
momentum_kernel(const TensorDesc *__restrict__ tensors, const ChunkDesc *__restrict__ chunks, int64_t n_chunks,
                const uint8_t *__restrict__ present, float momentum, int nesterov, float *__restrict__ partials,
                const uint8_t *__restrict__ direct_bf16, const float *upd_base, __nv_bfloat16 *__restrict__ xb_base,
                const GradPeers gp)
{
    __shared__ float warp_sums[kEwThreads / 32];
    if (GSUM && fence_failed(gp.fence_error)) return;  // the peers' gradients may not be there
    for (int64_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        const ChunkDesc ch = chunks[c];
        if (present[ch.tensor] == 0) continue;
        const TensorDesc td = tensors[ch.tensor];
        const float *__restrict__ g = td.g + ch.offset;
        float *__restrict__ v = td.s1 + ch.offset;
        float *__restrict__ u = td.s2 + ch.offset;
        const bool to_bf16 = direct_bf16 != nullptr && direct_bf16[ch.tensor] != 0;
        __nv_bfloat16 *__restrict__ xb = to_bf16 ? xb_base + (u - upd_base) : nullptr;
        const uint32_t n = ch.len;
        const ptrdiff_t gpos = GSUM ? (g - gp.local_base) : 0;  // position inside the gradient arena
        const float *g_arena = g - gpos;
        float local = 0.0f;
        const uint32_t n4 = n >> 2;  // chunk starts are 16-byte aligned by construction
        for (uint32_t i = threadIdx.x; i < n4; i += kEwThreads) {
            const float4 g4 = GSUM ? sum_grads4(gp, g_arena, gpos, i) : __ldcs(reinterpret_cast<const float4 *>(g) + i);
            float4 v4 = __ldcs(reinterpret_cast<const float4 *>(v) + i);
            float4 u4;
            v4.x = __fmaf_rn(momentum, v4.x, g4.x);
            v4.y = __fmaf_rn(momentum, v4.y, g4.y);
            v4.z = __fmaf_rn(momentum, v4.z, g4.z);
            v4.w = __fmaf_rn(momentum, v4.w, g4.w);
            if (nesterov) {
                u4.x = __fadd_rn(__fmul_rn(momentum, v4.x), g4.x);
                u4.y = __fadd_rn(__fmul_rn(momentum, v4.y), g4.y);
                u4.z = __fadd_rn(__fmul_rn(momentum, v4.z), g4.z);
                u4.w = __fadd_rn(__fmul_rn(momentum, v4.w), g4.w);
            } else {
                u4 = v4;
            }
            __stcs(reinterpret_cast<float4 *>(v) + i, v4);
            if (to_bf16) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(u4.x, u4.y), hi = __floats2bfloat162_rn(u4.z, u4.w);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t *>(&lo);
                packed.y = *reinterpret_cast<uint32_t *>(&hi);
                reinterpret_cast<uint2 *>(xb)[i] = packed;
            } else {
                reinterpret_cast<float4 *>(u)[i] = u4;  // read again soon: keep it in L2
            }
            if (PARTIALS) local += u4.x * u4.x + u4.y * u4.y + u4.z * u4.z + u4.w * u4.w;
        }
        for (uint32_t i = (n4 << 2) + threadIdx.x; i < n; i += kEwThreads) {
            const float gv = GSUM ? sum_grads1(gp, g_arena, gpos, i) : g[i];
            const float vv = __fmaf_rn(momentum, v[i], gv);
            const float uv = nesterov ? __fadd_rn(__fmul_rn(momentum, vv), gv) : vv;
            v[i] = vv;
            if (to_bf16) xb[i] = __float2bfloat16_rn(uv);
            else u[i] = uv;
            if (PARTIALS) local += uv * uv;
        }
        if (PARTIALS) {
            // fixed-shape tree: the result does not depend on timing
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) local += __shfl_down_sync(0xffffffffu, local, d);
            if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = local;
            __syncthreads();
            if (threadIdx.x == 0) {
                float s = 0.0f;
#pragma unroll
                for (int w = 0; w < kEwThreads / 32; ++w) s += warp_sums[w];
                partials[c] = s;
            }
            __syncthreads();
        }
    }
}

// Adds each tensor's chunk partials in chunk order (one warp per tensor, lane-strided then
// a fixed tree: deterministic).  Tensors without chunks keep sumsq = 0.
__global__ void reduce_partials_kernel(const float *__restrict__ partials, const int64_t *__restrict__ first_chunk,
                                       const int32_t *__restrict__ ns_tensors, int n_ns, float *__restrict__ sumsq)
{
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= n_ns) return;
    const int t = ns_tensors[w];
    const int64_t lo = first_chunk[t], hi = first_chunk[t + 1];
    float s = 0.0f;
    for (int64_t c = lo + (threadIdx.x & 31); c < hi; c += 32) s += partials[c];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_down_sync(0xffffffffu, s, d);
    if ((threadIdx.x & 31) == 0) sumsq[t] = s;
}

// ---- K3s: order-faithful sum of squares ------------------------------------------------------
// The identity times 2^scale_log2 as the first of two f16 planes, or as bf16 (chain forms that start from P_0 = I).
__global__ void set_identity_planes_kernel(__nv_bfloat16 *__restrict__ plane0, int n, int scale_log2, int as_bf16)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = ldexpf(1.0f, scale_log2);
    reinterpret_cast<unsigned short *>(plane0)[(int64_t)i * n + i] =
        as_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}

// The reference adds x*x left to right in f32 (muon.rs:58).  With millions of addends that
// differs from the exact sum by up to a few 1e-3 relative, far more than the 1e-5 parity
// bound of the f32 path, so the GPU must reproduce the *sequence of roundings*.
//
// All addends are >= 0, so the running sum s never decreases.  While s stays inside one
// binade [2^e, 2^(e+1)) it is k * ulp with ulp = 2^(e-23) and integer k in [2^23, 2^24), and
//     fl(s + a) = (k + rne(a / ulp)) * ulp,
// where the round-to-nearest-even of a/ulp = q + f depends on s only through the parity of k
// (and only when f is exactly 1/2).  So every element is a map  parity -> integer increment,
// i.e. two numbers, and the composition of such maps is associative: a block composes the
// maps of thousands of consecutive elements with an ordered tree and applies the result to
// k in one go.  If the result would leave the binade (k + inc >= 2^24), or s is not a normal
// number yet, one thread walks the elements with real f32 additions until the exponent of s
// changes and the block resumes from there; this happens about once per doubling of s.  The
// per-warp and per-thread maps localise the crossing to one thread's 16 elements, so a walk is short.
struct IncMap {
    uint32_t even;  // increment (in ulps) when k is even
    uint32_t odd;   // increment when k is odd
};
constexpr uint32_t kIncSat = 1u << 25;  // ">= 2^24": leaves the binade for certain

__device__ __forceinline__ IncMap compose(IncMap a, IncMap b)  // a first, then b
{
    IncMap c;
    const uint32_t b_after_even = (a.even & 1u) ? b.odd : b.even;
    const uint32_t b_after_odd = ((a.odd + 1u) & 1u) ? b.odd : b.even;
    c.even = min(a.even + b_after_even, kIncSat);
    c.odd = min(a.odd + b_after_odd, kIncSat);
    return c;
}

// Map of one addend a >= 0: x = a / ulp = q + f is exact (power-of-two scaling; inv_ulp =
// 2^(23 - e)).  Unless f is exactly 1/2 the increment is rne(x) whatever the parity of k, read
// off the low bits of x + 2^23; x is clamped to 2^23, an increment that leaves the binade for
// certain (k >= 2^23), which also catches inf and NaN.  On a tie the even-k increment is the even
// one of {q, q + 1} (what the addition above rounds to) and the odd-k increment the other one.
struct ElementInc {
    uint32_t r;  // rne(x), ties to even; 2^23 when x was clamped
    float d;     // x - rne(x), exact: +-0.5 on a tie
};
__device__ __forceinline__ ElementInc element_inc(float a, float inv_ulp)
{
    ElementInc e;
    const float x = fminf(__fmul_rn(a, inv_ulp), 8388608.0f);
    const float y = __fadd_rn(x, 8388608.0f);
    e.r = __float_as_uint(y) - 0x4B000000u;
    e.d = __fsub_rn(x, __fsub_rn(y, 8388608.0f));
    return e;
}
// Composed map of 16 consecutive addends (not saturated: below 2^28).  Ties are rare (the addend
// must end exactly half an ulp of the running sum), so the sixteen increments are simply added and
// the parity-dependent composition is only run when one of them was a tie.
__device__ __forceinline__ IncMap compose16(const float *a, float inv_ulp)
{
    uint32_t sum = 0u;
    bool any_tie = false;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const ElementInc e = element_inc(a[i], inv_ulp);
        sum += e.r;
        any_tie |= fabsf(e.d) == 0.5f;
    }
    IncMap m = {sum, sum};
    if (any_tie) {
        m.even = m.odd = 0u;
#pragma unroll 1
        for (int i = 0; i < 16; ++i) {
            const ElementInc e = element_inc(a[i], inv_ulp);
            const uint32_t k_odd_even = m.even & 1u, k_odd_odd = (m.odd & 1u) ^ 1u;  // parity of k + increment so far
            m.even += e.r;
            m.odd += e.r;
            if (fabsf(e.d) == 0.5f) {
                const uint32_t other = e.d > 0.0f ? 1u : 0xffffffffu;  // the odd neighbour is r + 1 or r - 1
                if (k_odd_even) m.even += other;
                if (k_odd_odd) m.odd += other;
            }
        }
    }
    m.even = min(m.even, kIncSat);
    m.odd = min(m.odd, kIncSat);
    return m;
}

__device__ __forceinline__ bool binade_ok(float s)
{
    // positive, finite, and large enough (>= 2^-100) that 1/ulp = 2^(23-e) is a normal float;
    // smaller running sums are simply added one element at a time
    const uint32_t e = (__float_as_uint(s) >> 23) & 0xffu;
    return s > 0.0f && e >= 27u && e != 0xffu;
}

constexpr int kSeqThreads = 512;
constexpr int kSeqPerThread = 16;  // compose16 and load_block16 take sixteen elements per thread
constexpr int kSeqChunk = kSeqThreads * kSeqPerThread;       // 8192 elements per pass
constexpr int kSeqWarpSpan = 32 * kSeqPerThread;             // elements one warp covers

__device__ __forceinline__ float float_from_k(uint32_t bits_of_s, uint32_t k)
{
    return __uint_as_float((bits_of_s & 0x7f800000u) | (k & 0x7fffffu));
}

// The chain above is sequential per matrix, but almost all of its work can be done ahead of it
// in parallel.  A block of 8192 consecutive elements is one composed map once the binade of the
// running sum at the block's start is known, and that binade can be guessed from an ordinary
// (tree) prefix sum, which differs from the sequential sum by parts in 10^3 only:
//   1. momentum_kernel          also leaves the tree sum of squares of every block (its chunks are
//                               these blocks when the ordered sum is in use)   (parallel)
//   2. block_guess_kernel       prefix over a matrix's blocks -> guessed exponent per block
//   3. block_map_kernel         composed map of every block under its guess   (parallel)
//   4. sumsq_ordered_kernel     walks the blocks: a guessed map is used when the running sum
//                               really is in the guessed binade and stays there (one integer
//                               add per block); any other block (the first ones, the ~25 binade
//                               crossings, a wrong guess) is redone exactly by the whole CTA.
// The result is the same sequence of roundings either way.
struct SeqBlock {
    int32_t tensor;  // index into the optimizer's tensors
    int32_t index;   // block number inside the tensor
};

__device__ __forceinline__ void load_block16(const float *__restrict__ x, int64_t n, int64_t base, int tid, float *dst)
{
    const int64_t i0 = base + (int64_t)tid * 16;
    if (i0 + 16 <= n) {  // tensors start 128-byte aligned: vector loads are aligned
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 v = *reinterpret_cast<const float4 *>(x + i0 + 4 * q);
            dst[4 * q + 0] = v.x; dst[4 * q + 1] = v.y; dst[4 * q + 2] = v.z; dst[4 * q + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i] = (i0 + i < n) ? x[i0 + i] : 0.0f;
    }
}

// One warp per matrix: biased exponent of the (approximate) sum of everything before each block.
// The block sums are the momentum kernel's per-chunk sums: with the ordered sum in use the
// element-wise chunks are the 8192-element blocks (block b of a tensor is its chunk b).
__global__ void block_guess_kernel(const float *__restrict__ chunk_sum, const int64_t *__restrict__ first_chunk,
                                   const int64_t *__restrict__ first_block,
                                   const int32_t *__restrict__ ns_tensors, int n_ns,
                                   const uint8_t *__restrict__ present, int32_t *__restrict__ guess)
{
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= n_ns) return;
    if (present[ns_tensors[w]] == 0) return;
    const int lane = threadIdx.x & 31;
    const int64_t lo = first_block[w], hi = first_block[w + 1];
    const float *__restrict__ block_sum = chunk_sum + first_chunk[ns_tensors[w]] - lo;
    double carry = 0.0;
    for (int64_t base = lo; base < hi; base += 32) {
        const int64_t i = base + lane;
        const double mine = i < hi ? (double)block_sum[i] : 0.0;
        double incl = mine;  // inclusive prefix over the 32 lanes
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const double o = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += o;
        }
        if (i < hi) guess[i] = (int32_t)((__float_as_uint((float)(carry + incl - mine)) >> 23) & 0xffu);
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
}

__global__ void __launch_bounds__(512)
block_map_kernel(const TensorDesc *__restrict__ tensors, const SeqBlock *__restrict__ blocks, int n_blocks,
                 const int64_t *__restrict__ sizes, const uint8_t *__restrict__ present,
                 const int32_t *__restrict__ guess, IncMap *__restrict__ block_map)
{
    __shared__ IncMap warp_maps[16];
    for (int b = blockIdx.x; b < n_blocks; b += gridDim.x) {
        const SeqBlock sb = blocks[b];
        if (present[sb.tensor] == 0) continue;
        const uint32_t biased = (uint32_t)guess[b];
        if (biased < 27u || biased == 0xffu) {  // no usable guess (empty prefix, tiny sums): the chain redoes it
            if (threadIdx.x == 0) block_map[b] = IncMap{kIncSat, kIncSat};
            continue;
        }
        float v[16];
        load_block16(tensors[sb.tensor].s2, sizes[sb.tensor], (int64_t)sb.index * 8192, threadIdx.x, v);
        const float inv_ulp = __uint_as_float((277u - biased) << 23);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = __fmul_rn(v[i], v[i]);
        IncMap m = compose16(v, inv_ulp);
        const int lane = threadIdx.x & 31;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            IncMap o;
            o.even = __shfl_down_sync(0xffffffffu, m.even, d);
            o.odd = __shfl_down_sync(0xffffffffu, m.odd, d);
            if ((lane & (2 * d - 1)) == 0) m = compose(m, o);
        }
        if (lane == 0) warp_maps[threadIdx.x >> 5] = m;
        __syncthreads();
        if (threadIdx.x == 0) {
            IncMap t = warp_maps[0];
#pragma unroll
            for (int w = 1; w < 16; ++w) t = compose(t, warp_maps[w]);
            block_map[b] = t;
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kSeqThreads)
sumsq_ordered_kernel(const TensorDesc *__restrict__ tensors, const int32_t *__restrict__ ns_tensors,
                     const int64_t *__restrict__ sizes, const uint8_t *__restrict__ present,
                     float *__restrict__ sumsq, const int64_t *__restrict__ first_block,
                     const IncMap *__restrict__ block_map, const int32_t *__restrict__ guess)
{
    constexpr int kWindow = 512;  // blocks whose guessed maps are staged in shared memory at a time
    __shared__ float sq[kSeqChunk];
    __shared__ IncMap warp_maps[kSeqThreads / 32];
    __shared__ IncMap thread_maps[kSeqThreads];
    __shared__ IncMap win_map[kWindow];
    __shared__ int32_t win_guess[kWindow];
    __shared__ float sh_s;
    __shared__ int sh_start;
    __shared__ int sh_next;

    const int t = ns_tensors[blockIdx.x];
    if (present[t] == 0) return;
    const float *__restrict__ x = tensors[t].s2;  // the update buffer
    const int64_t n = sizes[t];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t n_blocks = (n + kSeqChunk - 1) / kSeqChunk;
    const int64_t fb = block_map ? first_block[blockIdx.x] : 0;

    if (tid == 0) sh_s = 0.0f;
    __syncthreads();

    for (int64_t win = 0; win < n_blocks; win += kWindow) {
        const int wn = (int)min((int64_t)kWindow, n_blocks - win);
        if (block_map != nullptr && tid < wn) {
            win_map[tid] = block_map[fb + win + tid];
            win_guess[tid] = guess[fb + win + tid];
        }
        __syncthreads();
        int b = 0;
        for (;;) {
            if (tid == 0) {
                // take the guessed maps while the running sum is in the guessed binade and stays there
                float s = sh_s;
                int bb = b;
                if (block_map != nullptr) {
                    while (bb < wn) {
                        const uint32_t bits = __float_as_uint(s);
                        if (!binade_ok(s) || (int32_t)((bits >> 23) & 0xffu) != win_guess[bb]) break;
                        const IncMap m = win_map[bb];
                        const uint32_t k = (bits & 0x7fffffu) | 0x800000u;
                        const uint32_t inc = (k & 1u) ? m.odd : m.even;
                        if (k + inc >= (1u << 24)) break;  // would leave the binade (or the map is saturated)
                        s = float_from_k(bits, k + inc);
                        ++bb;
                    }
                }
                sh_s = s;
                sh_next = bb;
            }
            __syncthreads();
            b = sh_next;
            if (b >= wn) break;

            // ---- block win + b exactly, by the whole CTA --------------------------------------
            const int64_t base = (win + b) * kSeqChunk;
            const int cnt = (int)min((int64_t)kSeqChunk, n - base);
            float a[kSeqPerThread];
            load_block16(x, n, base, tid, a);
#pragma unroll
            for (int i = 0; i < kSeqPerThread; ++i) {
                a[i] = __fmul_rn(a[i], a[i]);      // `x * x`, muon.rs:58 (padding squares to 0)
                sq[i * kSeqThreads + tid] = a[i];  // element tid*16+i, stored bank-conflict free
            }
            if (tid == 0) sh_start = 0;
            __syncthreads();
            for (;;) {
                const int start = sh_start;
                const float s = sh_s;
                if (start >= cnt) break;
                const bool ok = binade_ok(s);
                if (ok && (warp + 1) * kSeqWarpSpan > start) {  // warps wholly before `start` have nothing to add
                    // 1/ulp(s) = 2^(23 - e) with e the unbiased exponent of s: biased exponent 150 - e - 127 + 127
                    const uint32_t biased = (__float_as_uint(s) >> 23) & 0xffu;
                    const float inv_ulp = __uint_as_float((277u - biased) << 23);
                    float rest[kSeqPerThread];  // the addends from `start` on (past cnt: squares of the zero padding)
#pragma unroll
                    for (int i = 0; i < kSeqPerThread; ++i) rest[i] = tid * kSeqPerThread + i >= start ? a[i] : 0.0f;
                    IncMap m = compose16(rest, inv_ulp);
                    thread_maps[tid] = m;
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        IncMap o;
                        o.even = __shfl_down_sync(0xffffffffu, m.even, d);
                        o.odd = __shfl_down_sync(0xffffffffu, m.odd, d);
                        if ((lane & (2 * d - 1)) == 0) m = compose(m, o);
                    }
                    if (lane == 0) warp_maps[warp] = m;
                }
                __syncthreads();
                if (tid == 0) {
                    float s_new = s;
                    int walk_from = start;
                    bool done = false;
                    if (ok) {
                        // apply the warps' maps in order; stop at the first that would leave the binade
                        const uint32_t bits = __float_as_uint(s);
                        uint32_t k = (bits & 0x7fffffu) | 0x800000u;
                        int w = start / kSeqWarpSpan;
                        const int w_end = (cnt + kSeqWarpSpan - 1) / kSeqWarpSpan;
                        for (; w < w_end; ++w) {
                            const IncMap wm = warp_maps[w];
                            const uint32_t inc = (k & 1u) ? wm.odd : wm.even;
                            if (k + inc >= (1u << 24)) break;
                            k += inc;
                        }
                        s_new = float_from_k(bits, k);
                        if (w == w_end) {
                            sh_start = cnt;
                            done = true;
                        } else {
                            // the crossing is inside warp w's span: take its threads' maps up to the one that crosses
                            int th = max(start / kSeqPerThread, w * 32);
                            const int th_end = (w + 1) * 32;
                            for (; th < th_end; ++th) {
                                const IncMap tm = thread_maps[th];
                                const uint32_t inc = (k & 1u) ? tm.odd : tm.even;
                                if (k + inc >= (1u << 24)) break;
                                k += inc;
                            }
                            s_new = float_from_k(bits, k);
                            walk_from = max(start, min(th, th_end - 1) * kSeqPerThread);
                        }
                    }
                    if (!done) {
                        // walk with real additions until s enters a new binade (or the block ends)
                        int j = walk_from;
                        while (j < cnt) {
                            const float nx = __fadd_rn(s_new, sq[(j % kSeqPerThread) * kSeqThreads + j / kSeqPerThread]);
                            const bool changed = ((__float_as_uint(nx) ^ __float_as_uint(s_new)) >> 23) != 0u;
                            s_new = nx;
                            ++j;
                            if (changed && binade_ok(s_new)) break;
                        }
                        sh_start = j;
                    }
                    sh_s = s_new;
                }
                __syncthreads();
            }
            __syncthreads();  // everyone has left the loop before sq / sh_start / sh_s are touched again
            b += 1;
        }
        __syncthreads();  // the staged window is rewritten next
    }
    if (tid == 0) sumsq[t] = sh_s;
}

// ---- K3b: normalise ----------------------------------------------------------------------------
// x = u / sqrt(sumsq + 1e-8) where the norm exceeds 1e-8 (muon.rs:59-64).  Per tensor
// (ns_kind): 1 = rewrite the f32 update buffer in place (operand of the f32 GEMMs, and the
// final update when ns_steps == 0), 2 = write the bf16 operand of the first tensor-core GEMM,
// 3 = write that operand as two f16 planes of x * 2^15 (f32-accurate tensor-core path).
__global__ void __launch_bounds__(kEwThreads)
normalise_kernel(const TensorDesc *__restrict__ tensors, const ChunkDesc *__restrict__ chunks, int64_t n_chunks,
                 const uint8_t *__restrict__ present, const uint8_t *__restrict__ ns_kind,
                 const float *__restrict__ sumsq, const float *upd_base, __nv_bfloat16 *__restrict__ xb_base,
                 int64_t plane_stride, const uint8_t *__restrict__ skip)
{
    for (int64_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        const ChunkDesc ch = chunks[c];
        const int kind = ns_kind[ch.tensor];
        if (present[ch.tensor] == 0 || kind == 0) continue;
        if (skip != nullptr && skip[ch.tensor] != 0) continue;  // normalisation folded into the GEMM epilogues
        float *u = tensors[ch.tensor].s2 + ch.offset;
        const float norm = __fsqrt_rn(__fadd_rn(sumsq[ch.tensor], 1e-8f));
        const bool scale = norm > 1e-8f;
        const uint32_t n = ch.len;
        const uint32_t n4 = n >> 2;
        if (kind == 3) {
            __nv_bfloat16 *xb = xb_base + (u - upd_base);
            unsigned short *xh = reinterpret_cast<unsigned short *>(xb);
            const float kScale = ldexpf(1.0f, 15 - split_exponent(sumsq[ch.tensor]));  // 2^15 unless the update is tiny
            for (uint32_t i = threadIdx.x; i < n4; i += kEwThreads) {
                float4 v = reinterpret_cast<const float4 *>(u)[i];
                if (scale) {
                    v.x = __fdiv_rn(v.x, norm); v.y = __fdiv_rn(v.y, norm);
                    v.z = __fdiv_rn(v.z, norm); v.w = __fdiv_rn(v.w, norm);
                }
                unsigned short p[2][4];
                split_f16(v.x * kScale, p[0][0], p[1][0]);
                split_f16(v.y * kScale, p[0][1], p[1][1]);
                split_f16(v.z * kScale, p[0][2], p[1][2]);
                split_f16(v.w * kScale, p[0][3], p[1][3]);
#pragma unroll
                for (int pl = 0; pl < kSplitPlanes; ++pl) {
                    uint2 packed;
                    packed.x = (uint32_t)p[pl][0] | ((uint32_t)p[pl][1] << 16);
                    packed.y = (uint32_t)p[pl][2] | ((uint32_t)p[pl][3] << 16);
                    reinterpret_cast<uint2 *>(xh + pl * plane_stride)[i] = packed;
                }
            }
            for (uint32_t i = (n4 << 2) + threadIdx.x; i < n; i += kEwThreads) {
                unsigned short h0, h1;
                split_f16((scale ? __fdiv_rn(u[i], norm) : u[i]) * kScale, h0, h1);
                xh[i] = h0;
                xh[plane_stride + i] = h1;
            }
        } else if (kind == 2) {
            __nv_bfloat16 *xb = xb_base + (u - upd_base);
            for (uint32_t i = threadIdx.x; i < n4; i += kEwThreads) {
                float4 v = reinterpret_cast<const float4 *>(u)[i];
                if (scale) {
                    v.x = __fdiv_rn(v.x, norm); v.y = __fdiv_rn(v.y, norm);
                    v.z = __fdiv_rn(v.z, norm); v.w = __fdiv_rn(v.w, norm);
                }
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t *>(&lo);
                packed.y = *reinterpret_cast<uint32_t *>(&hi);
                reinterpret_cast<uint2 *>(xb)[i] = packed;
            }
            for (uint32_t i = (n4 << 2) + threadIdx.x; i < n; i += kEwThreads)
                xb[i] = __float2bfloat16_rn(scale ? __fdiv_rn(u[i], norm) : u[i]);
        } else {
            if (!scale) continue;
            for (uint32_t i = threadIdx.x; i < n4; i += kEwThreads) {
                float4 v = reinterpret_cast<const float4 *>(u)[i];
                v.x = __fdiv_rn(v.x, norm); v.y = __fdiv_rn(v.y, norm);
                v.z = __fdiv_rn(v.z, norm); v.w = __fdiv_rn(v.w, norm);
                reinterpret_cast<float4 *>(u)[i] = v;
            }
            for (uint32_t i = (n4 << 2) + threadIdx.x; i < n; i += kEwThreads) u[i] = __fdiv_rn(u[i], norm);
        }
    }
}

// ---- K6: apply -----------------------------------------------------------------------------------
// w -= lr * u * 0.1 (muon.rs:158-160; Rust evaluates (lr * u) * 0.1).  TensorDesc.g here points
// at the buffer that holds the final update of the tensor.
template <bool PEERS, int HALF>
__global__ void __launch_bounds__(kEwThreads)
apply_kernel(const TensorDesc *__restrict__ tensors, const ChunkDesc *__restrict__ chunks, int64_t n_chunks,
             const uint8_t *__restrict__ present, float lr, const PeerTable pt, const int *__restrict__ error_flag)
{
    // A Newton-Schulz kernel of this step gave up a wait: its update buffers are half written.
    // Nothing is applied, so the weights (here and on the peers) keep their pre-step values.
    if (error_flag != nullptr && *reinterpret_cast<const volatile int *>(error_flag) != 0) return;
    if ((PEERS || HALF == 2) && fence_failed(pt.fence_error)) return;  // the fence before this launch gave up
    for (int64_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        const ChunkDesc ch = chunks[c];
        if (present[ch.tensor] == 0) continue;
        float *__restrict__ w = tensors[ch.tensor].p + ch.offset;
        const float *__restrict__ u = tensors[ch.tensor].g + ch.offset;
        const ptrdiff_t arena_pos = (PEERS || HALF) ? (w - pt.local_base) : 0;
        const uint32_t n = ch.len;
        const uint32_t n4 = n >> 2;
        for (uint32_t i = threadIdx.x; i < n4; i += kEwThreads) {
            float4 wv = __ldcs(reinterpret_cast<const float4 *>(w) + i);
            const float4 uv = __ldcs(reinterpret_cast<const float4 *>(u) + i);
            wv.x = __fsub_rn(wv.x, __fmul_rn(__fmul_rn(lr, uv.x), 0.1f));
            wv.y = __fsub_rn(wv.y, __fmul_rn(__fmul_rn(lr, uv.y), 0.1f));
            wv.z = __fsub_rn(wv.z, __fmul_rn(__fmul_rn(lr, uv.z), 0.1f));
            wv.w = __fsub_rn(wv.w, __fmul_rn(__fmul_rn(lr, uv.w), 0.1f));
            __stcs(reinterpret_cast<float4 *>(w) + i, wv);
            if (PEERS) {  // the owner's new weights go straight into every peer's arena (NVLink stores)
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r)
                    if (r < pt.n) reinterpret_cast<float4 *>(pt.base[r] + arena_pos)[i] = wv;
            }
            if (HALF) {  // bf16 copy of the new weights: local, and (HALF == 2) on every peer
                const __nv_bfloat162 lo = __floats2bfloat162_rn(wv.x, wv.y), hi = __floats2bfloat162_rn(wv.z, wv.w);
                const uint2 h = make_uint2(*reinterpret_cast<const uint32_t *>(&lo),
                                           *reinterpret_cast<const uint32_t *>(&hi));
                reinterpret_cast<uint2 *>(pt.half_local + arena_pos)[i] = h;
                if (HALF == 2) {
#pragma unroll
                    for (int r = 0; r < kMaxPeers; ++r)
                        if (r < pt.n_half) reinterpret_cast<uint2 *>(pt.half_base[r] + arena_pos)[i] = h;
                }
            }
        }
        for (uint32_t i = (n4 << 2) + threadIdx.x; i < n; i += kEwThreads) {
            const float wv = __fsub_rn(w[i], __fmul_rn(__fmul_rn(lr, u[i]), 0.1f));
            w[i] = wv;
            if (PEERS) {
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r)
                    if (r < pt.n) pt.base[r][arena_pos + i] = wv;
            }
            if (HALF) {
                const __nv_bfloat16 hb = __float2bfloat16_rn(wv);
                const uint16_t h = *reinterpret_cast<const uint16_t *>(&hb);
                pt.half_local[arena_pos + i] = h;
                if (HALF == 2) {
#pragma unroll
                    for (int r = 0; r < kMaxPeers; ++r)
                        if (r < pt.n_half) pt.half_base[r][arena_pos + i] = h;
                }
            }
        }
    }
}

template <typename T>
int upload(T **d, const std::vector<T> &h, cudaStream_t stream)
{
    *d = nullptr;
    const size_t bytes = std::max<size_t>(h.size(), 1) * sizeof(T);
    VB_CUDA(cudaMalloc((void **)d, bytes));
    if (!h.empty()) VB_CUDA(cudaMemcpyAsync(*d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice, stream));
    return VB_OK;
}

}  // namespace

// VB_TC_NO_TRANSPOSE=1 keeps the direct form X' = X C for tall matrices (for comparison).
static bool use_transposed_update()
{
    const char *e = getenv("VB_TC_NO_TRANSPOSE");
    return !(e && *e == '1');
}

struct MuonState {
    std::vector<int> owner;           // per tensor
    std::vector<int64_t> local_off;   // per tensor: offset into this rank's buffers, -1 if not owned
    std::vector<uint8_t> ns_kind;     // per tensor: 0 no Newton-Schulz, 1 f32 CUDA-core path, 2 bf16 tensor-core
                                      // path, 3 split-bf16 (f32-accurate) tensor-core path
    int planes = 1;                   // 16-bit planes per tensor-core operand (2 on the split path)
    int64_t cb_elems = 0;             // elements of one plane of the C buffer
    int64_t owned_elems = 0;
    float *d_upd = nullptr;           // update buffer u / X (f32), owned tensors
    float *d_xnext = nullptr;         // f32 path: the other Newton-Schulz buffer
    float *d_gram = nullptr;          // f32 path: C = 3I - X^T X per matrix
    __nv_bfloat16 *d_xb[2] = {nullptr, nullptr};  // bf16 path: X ping-pong
    __nv_bfloat16 *d_cb = nullptr;                // bf16 path: C = 3I - Gram per matrix (short side squared)
    float *d_sumsq = nullptr;         // per tensor
    float *d_partials = nullptr;      // per chunk: sum of squares of the update (tree order)
    uint8_t *d_ns_kind = nullptr;
    int64_t *d_sizes = nullptr;
    int32_t *d_ns_tensors = nullptr;  // owned tensors that run Newton-Schulz
    int n_ns = 0;
    int64_t *d_first_chunk = nullptr;
    // ordered sum of squares (f32 modes): 8192-element blocks of the Newton-Schulz tensors, their
    // tree sums, guessed exponents and guessed maps (see block_map_kernel)
    SeqBlock *d_seq_blocks = nullptr;
    int64_t *d_first_block = nullptr;  // per Newton-Schulz tensor (n_ns + 1)
    int32_t *d_block_guess = nullptr;
    IncMap *d_block_map = nullptr;
    int n_seq_blocks = 0;
    TensorDesc *d_desc = nullptr;        // p = w, g = grad, s1 = velocity, s2 = update buffer
    TensorDesc *d_desc_apply = nullptr;  // p = w, g = final update
    ChunkDesc *d_chunks = nullptr;
    int64_t n_chunks = 0;
    std::vector<float *> final_update;   // per tensor: device pointer of the last step's update
    // f32 GEMM schedules: [parity] -> gram problems, update problems
    F32GemmProblem *d_gram_prob[2] = {nullptr, nullptr};
    F32GemmProblem *d_upd_prob[2] = {nullptr, nullptr};
    GemmTile *d_gram_tiles = nullptr, *d_upd_tiles = nullptr;
    int n_gram_tiles = 0, n_upd_tiles = 0;
    // tensor-core GEMM schedules: [parity]; the last iteration's update writes the f32 result
    // tensor-core GEMM schedules, one problem array per Newton-Schulz iteration (the first may
    // fold the normalisation in, the last writes the f32 result)
    std::vector<TcGemmProblem *> d_tc_gram, d_tc_upd;
    uint8_t *d_fold_norm = nullptr;    // per tensor: normalisation folded into the first iteration
    bool fold_norm = false;
    GemmTile *d_tc_gram_tiles = nullptr, *d_tc_upd_tiles = nullptr;
    GemmTile *d_tc_upd_tiles_last = nullptr;  // the last iteration's update is always in the direct form
    int n_tc_gram_tiles = 0, n_tc_upd_tiles = 0, n_tc_upd_tiles_last = 0;
    // update products whose output width is a multiple of 512 run on 256 x 512 tiles (a quarter
    // less operand traffic from L2); the lists above then hold only the other matrices
    GemmTile *d_tc_upd_tiles_wide = nullptr, *d_tc_upd_tiles_last_wide = nullptr, *d_tc_gram_tiles_wide = nullptr;
    int n_tc_upd_tiles_wide = 0, n_tc_upd_tiles_last_wide = 0, n_tc_gram_tiles_wide = 0;
    // The chain form of the plain bf16 path (see build of chain_launches): launches in order, the
    // last one is the product that yields the update
    struct TcLaunch {
        TcGemmProblem *d_problems = nullptr;
        const GemmTile *d_tiles = nullptr;
        int n_tiles = 0;
        bool final_product = false;
        bool dual = false;  // its problems store G beside 3I - G
    };
    bool chain = false;
    bool chain_g_only = false;  // only G, T, P are stored; C = 1.5 I - 0.5 G is applied in the epilogues
    std::vector<TcLaunch> chain_launches;
    __nv_bfloat16 *d_chain = nullptr;    // per matrix six short-side squares: G, T, C'[2], P'[2]
    GemmTile *d_small_tiles = nullptr, *d_small_tiles2 = nullptr;
    int n_small_tiles = 0, n_small_tiles2 = 0;
    int *d_error = nullptr;
    int *h_error = nullptr;              // pinned mirror of d_error, refreshed after every step
    // The last update launch applies its result to the weights itself (tensor-core matrices); the
    // apply kernel then covers only the other tensors.  VB_MUON_UNFUSED_APPLY=1 keeps the separate
    // pass for all (for comparison).  keep_update: the f32 update is stored as well.
    bool fuse_apply = false;
    bool keep_update = false;
    bool last_step_fused = false;
    ChunkDesc *d_chunks_apply = nullptr;
    int64_t n_chunks_apply = 0;
    bool debug_withhold = false;         // test hook: the next step's first Gram launch stages nothing
    uint32_t debug_wait_limit = 0;
    double flops_per_step = 0.0;
    double last_flops = 0.0;
};

void destroy_muon_state(MuonState *s)
{
    if (!s) return;
    cudaFree(s->d_upd);
    cudaFree(s->d_xnext);
    cudaFree(s->d_gram);
    cudaFree(s->d_xb[0]);
    cudaFree(s->d_xb[1]);
    cudaFree(s->d_cb);
    cudaFree(s->d_chain);
    cudaFree(s->d_small_tiles);
    cudaFree(s->d_small_tiles2);
    for (auto &l : s->chain_launches) cudaFree(l.d_problems);
    cudaFree(s->d_sumsq);
    cudaFree(s->d_partials);
    cudaFree(s->d_ns_kind);
    cudaFree(s->d_sizes);
    cudaFree(s->d_ns_tensors);
    cudaFree(s->d_first_chunk);
    cudaFree(s->d_seq_blocks);
    cudaFree(s->d_first_block);
    cudaFree(s->d_block_guess);
    cudaFree(s->d_block_map);
    cudaFree(s->d_desc);
    cudaFree(s->d_desc_apply);
    cudaFree(s->d_chunks);
    cudaFree(s->d_chunks_apply);
    for (int i = 0; i < 2; ++i) {
        cudaFree(s->d_gram_prob[i]);
        cudaFree(s->d_upd_prob[i]);
    }
    for (TcGemmProblem *p : s->d_tc_gram) cudaFree(p);
    for (TcGemmProblem *p : s->d_tc_upd) cudaFree(p);
    cudaFree(s->d_fold_norm);
    cudaFree(s->d_gram_tiles);
    cudaFree(s->d_upd_tiles);
    cudaFree(s->d_tc_gram_tiles);
    cudaFree(s->d_tc_upd_tiles);
    cudaFree(s->d_tc_upd_tiles_last);
    cudaFree(s->d_tc_upd_tiles_wide);
    cudaFree(s->d_tc_gram_tiles_wide);
    cudaFree(s->d_tc_upd_tiles_last_wide);
    cudaFree(s->d_error);
    if (s->h_error) cudaFreeHost(s->h_error);
    delete s;
}

// Estimated device time of one tensor's share of a step, in seconds, under the arithmetic the
// mode really executes: the bit-faithful f32 kernels run the reference's formulation,
// 4 * rows * cols^2 FLOPs per iteration whatever the orientation (muon.rs:73: always cols x cols),
// on the CUDA cores; the tensor-core modes run the short-side form with the symmetric Gram
// computed on and above the diagonal (three plane products per product in the f32-accurate
// mode); every tensor also pays its element-wise passes.  Only the ratios matter.
double muon_tensor_cost(int64_t rows, int64_t cols, int ns_mode, int ns_steps)
{
    const double r = (double)rows, c = (double)cols;
    const double elementwise = r * c * 40.0 / 6.5e12;  // momentum, normalise, apply: ~40 B per element from HBM
    if (!(rows > 1 && cols > 1) || ns_steps <= 0) return elementwise;
    const bool tc = ns_mode != VB_NS_F32 && (rows % 8) == 0 && (cols % 8) == 0;
    if (!tc) return elementwise + 4.0 * r * c * c * (double)ns_steps / 45e12;
    const double L = std::max(r, c), S = std::min(r, c);
    const double t = std::ceil(S / 256.0);                  // 256 x 256 tiles per side of the Gram
    const double upper = (t * (t + 1.0) / 2.0) / (t * t);   // share of the Gram that is computed
    // the chain form: the first Gram (upper tiles), the short-side squares (upper tiles), the last product;
    // three plane products per product on the f32-accurate path, which also forms P_1 by a product
    const bool split = ns_mode == VB_NS_F32_TC;
    const double squares = split ? 3.0 * (double)ns_steps - 2.0 : 3.0 * (double)(ns_steps - 1);
    const double work = 2.0 * L * S * S * (1.0 + upper) + squares * 2.0 * S * S * S * upper;
    return elementwise + (split ? 3.0 * work / 0.95e15 : work / 0.8e15);
}

// Whole matrices are owned by one rank: tensors are taken in order of decreasing estimated
// cost (muon_tensor_cost) and each goes to the rank with the least work so far (ties: lowest
// rank).
void plan_muon_owners(int64_t n, const int64_t *rows, const int64_t *cols, int world, int ns_mode, int ns_steps,
                      int *owner_out)
{
    std::vector<int64_t> order((size_t)n);
    std::iota(order.begin(), order.end(), 0);
    auto cost = [&](int64_t i) -> double { return muon_tensor_cost(rows[i], cols[i], ns_mode, ns_steps); };
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return cost(a) > cost(b); });
    std::vector<double> load((size_t)world, 0.0);
    for (int64_t i : order) {
        int best = 0;
        for (int r = 1; r < world; ++r)
            if (load[(size_t)r] < load[(size_t)best]) best = r;
        owner_out[i] = best;
        load[(size_t)best] += cost(i);
    }
}

int muon_owner(vb_optimizer *opt, int64_t tensor) { return opt->muon ? opt->muon->owner[(size_t)tensor] : 0; }

float *muon_velocity_ptr(vb_optimizer *opt, int64_t tensor)
{
    if (!opt->muon || opt->muon->local_off[(size_t)tensor] < 0) return nullptr;
    return opt->d_s1 + opt->muon->local_off[(size_t)tensor];
}

int muon_check_error(vb_optimizer *opt)
{
    MuonState *s = opt->muon;
    if (s && s->h_error && *s->h_error != 0) {
        const int code = *s->h_error;
        return fail(VB_ERR_TIMEOUT, "a Newton-Schulz GEMM kernel gave up waiting on a pipeline barrier (role %d)", code);
    }
    return VB_OK;
}

int muon_init(vb_optimizer *opt)
{
    vb_engine *e = opt->eng;
    MuonState *s = new MuonState();
    opt->muon = s;
    const int64_t nt = opt->n_tensors;
    s->owner.assign((size_t)nt, 0);
    plan_muon_owners(nt, opt->rows.data(), opt->cols.data(), e->world, opt->ns_mode, opt->ns_steps, s->owner.data());
    s->local_off.assign((size_t)nt, -1);
    s->ns_kind.assign((size_t)std::max<int64_t>(nt, 1), 0);
    s->final_update.assign((size_t)nt, nullptr);
    int64_t off = 0, gram_elems = 0, cb_elems = 0;
    std::vector<int32_t> ns_tensors, f32_tensors, tc_tensors;
    std::vector<int64_t> gram_off((size_t)nt, -1), cb_off((size_t)nt, -1);
    for (int64_t i = 0; i < nt; ++i) {
        const int64_t r = opt->rows[i], c = opt->cols[i];
        const bool ns = r > 1 && c > 1;  // muon.rs:153
        if (ns) {
            // The tensor-core path needs 16-byte aligned bf16 rows for TMA; other shapes of a
            // bf16-mode optimizer run the (more accurate) f32 path.
            const bool tc = opt->ns_mode != VB_NS_F32 && opt->ns_steps > 0 && (r % 8) == 0 && (c % 8) == 0;
            s->ns_kind[(size_t)i] = !tc ? 1 : (opt->ns_mode == VB_NS_F32_TC ? 3 : 2);
        }
        if (s->owner[(size_t)i] != e->rank) continue;
        s->local_off[(size_t)i] = off;
        off += (opt->sizes[i] + 31) / 32 * 32;
        if (ns && opt->sizes[i] > 0) {
            if (r > 0x7fffffff || c > 0x7fffffff) return fail(VB_ERR_UNSUPPORTED, "matrix %lld is too large", (long long)i);
            ns_tensors.push_back((int32_t)i);
            if (s->ns_kind[(size_t)i] >= 2) {
                tc_tensors.push_back((int32_t)i);
                const int64_t sh = std::min(r, c);
                cb_off[(size_t)i] = cb_elems;
                cb_elems += (sh * sh + 63) / 64 * 64;
            } else {
                f32_tensors.push_back((int32_t)i);
                gram_off[(size_t)i] = gram_elems;
                gram_elems += (c * c + 31) / 32 * 32;
            }
        }
    }
    s->owned_elems = off;
    s->n_ns = (int)ns_tensors.size();
    const size_t owned_bytes = (size_t)std::max<int64_t>(off, 1) * sizeof(float);
    // velocity (muon.rs:26-29) and the update buffer, for owned tensors only
    VB_CUDA(cudaMalloc(&opt->d_s1, owned_bytes));
    VB_CUDA(cudaMemsetAsync(opt->d_s1, 0, owned_bytes, e->stream));
    VB_CUDA(cudaMalloc(&s->d_upd, owned_bytes));
    VB_CUDA(cudaMemsetAsync(s->d_upd, 0, owned_bytes, e->stream));
    VB_CUDA(cudaMalloc(&s->d_sumsq, (size_t)std::max<int64_t>(nt, 1) * sizeof(float)));
    VB_CUDA(cudaMemsetAsync(s->d_sumsq, 0, (size_t)std::max<int64_t>(nt, 1) * sizeof(float), e->stream));
    VB_CUDA(cudaMalloc(&s->d_error, sizeof(int)));
    VB_CUDA(cudaMemsetAsync(s->d_error, 0, sizeof(int), e->stream));
    VB_CUDA(cudaHostAlloc((void **)&s->h_error, sizeof(int), cudaHostAllocDefault));
    *s->h_error = 0;

    // element-wise chunk table over owned tensors
    // with the ordered sum of squares in use a chunk is one of its 8192-element blocks, so that the
    // momentum kernel's chunk sums serve as the block sums of the binade guess
    const int64_t chunk_len = opt->ns_mode != VB_NS_BF16 ? (int64_t)kSeqChunk : pick_chunk_len(off, e->sm_count);
    std::vector<TensorDesc> desc((size_t)std::max<int64_t>(nt, 1));
    std::vector<ChunkDesc> chunks;
    std::vector<int64_t> first_chunk((size_t)nt + 1, 0);
    for (int64_t i = 0; i < nt; ++i) {
        first_chunk[(size_t)i] = (int64_t)chunks.size();
        TensorDesc &td = desc[(size_t)i];
        td.p = opt->d_param + opt->offsets[(size_t)i];
        td.g = opt->d_grad + opt->offsets[(size_t)i];
        td.s1 = td.s2 = nullptr;
        if (s->local_off[(size_t)i] < 0) continue;
        td.s1 = opt->d_s1 + s->local_off[(size_t)i];
        td.s2 = s->d_upd + s->local_off[(size_t)i];
        for (int64_t b = 0; b < opt->sizes[i]; b += chunk_len) {
            ChunkDesc c;
            c.offset = b;
            c.tensor = (uint32_t)i;
            c.len = (uint32_t)std::min(chunk_len, opt->sizes[i] - b);
            chunks.push_back(c);
        }
    }
    first_chunk[(size_t)nt] = (int64_t)chunks.size();
    s->n_chunks = (int64_t)chunks.size();
    {
        const char *unfused = getenv("VB_MUON_UNFUSED_APPLY");
        s->fuse_apply = !(unfused && *unfused == '1');
        std::vector<ChunkDesc> apply_chunks;
        for (const ChunkDesc &c : chunks)
            if (!(s->fuse_apply && s->ns_kind[c.tensor] >= 2)) apply_chunks.push_back(c);
        s->n_chunks_apply = (int64_t)apply_chunks.size();
        VB_TRY(upload(&s->d_chunks_apply, apply_chunks, e->stream));
    }
    VB_TRY(upload(&s->d_desc, desc, e->stream));
    VB_TRY(upload(&s->d_chunks, chunks, e->stream));
    VB_TRY(upload(&s->d_first_chunk, first_chunk, e->stream));
    VB_TRY(upload(&s->d_ns_kind, s->ns_kind, e->stream));
    VB_TRY(upload(&s->d_sizes, opt->sizes, e->stream));
    VB_TRY(upload(&s->d_ns_tensors, ns_tensors, e->stream));
    VB_CUDA(cudaMalloc(&s->d_partials, (size_t)std::max<int64_t>(s->n_chunks, 1) * sizeof(float)));
    if (opt->ns_mode != VB_NS_BF16 && !ns_tensors.empty()) {
        // block tables of the ordered sum of squares; VB_SUMSQ_SERIAL=1 keeps the one-CTA-per-matrix
        // chain without the parallel pre-pass (for comparison)
        const char *serial = getenv("VB_SUMSQ_SERIAL");
        if (!(serial && *serial == '1')) {
            std::vector<SeqBlock> blocks;
            std::vector<int64_t> first_block(ns_tensors.size() + 1, 0);
            for (size_t j = 0; j < ns_tensors.size(); ++j) {
                first_block[j] = (int64_t)blocks.size();
                const int64_t nb = (opt->sizes[(size_t)ns_tensors[j]] + kSeqChunk - 1) / kSeqChunk;
                for (int64_t b = 0; b < nb; ++b) blocks.push_back(SeqBlock{ns_tensors[j], (int32_t)b});
            }
            first_block[ns_tensors.size()] = (int64_t)blocks.size();
            if (blocks.size() < (size_t)0x7fffffff) {
                s->n_seq_blocks = (int)blocks.size();
                VB_TRY(upload(&s->d_seq_blocks, blocks, e->stream));
                VB_TRY(upload(&s->d_first_block, first_block, e->stream));
                const size_t nb = std::max<size_t>(blocks.size(), 1);
                VB_CUDA(cudaMalloc(&s->d_block_guess, nb * sizeof(int32_t)));
                VB_CUDA(cudaMalloc(&s->d_block_map, nb * sizeof(IncMap)));
            }
        }
    }

    const bool odd = (opt->ns_steps & 1) != 0;
    if (!f32_tensors.empty()) {
        VB_CUDA(cudaMalloc(&s->d_xnext, owned_bytes));
        VB_CUDA(cudaMalloc(&s->d_gram, (size_t)std::max<int64_t>(gram_elems, 1) * sizeof(float)));
    }
    s->planes = opt->ns_mode == VB_NS_F32_TC ? kSplitPlanes : 1;
    s->cb_elems = cb_elems;
    if (!tc_tensors.empty()) {
        const size_t xb_bytes = (size_t)s->planes * (size_t)std::max<int64_t>(off, 1) * sizeof(__nv_bfloat16);
        for (int i = 0; i < 2; ++i) {
            VB_CUDA(cudaMalloc(&s->d_xb[i], xb_bytes));
            VB_CUDA(cudaMemsetAsync(s->d_xb[i], 0, xb_bytes, e->stream));
        }
        VB_CUDA(cudaMalloc(&s->d_cb, (size_t)s->planes * (size_t)std::max<int64_t>(cb_elems, 1) *
                                         sizeof(__nv_bfloat16)));
        // plain bf16 path: the chain form (below) unless VB_NS_CHAIN=0 asks for one Gram and one update
        // product per iteration
        const char *chain_env = getenv("VB_NS_CHAIN");
        s->chain = opt->ns_steps >= 1 && !(chain_env && *chain_env == '0');
        // VB_NS_CHAIN=2: the plain bf16 path also keeps only G, T and P (as the f32-accurate path does)
        s->chain_g_only = s->planes > 1 || (chain_env && *chain_env == '2');
        if (s->chain) {
            // six short-side squares per matrix (of `planes` planes each)
            const size_t chain_bytes = 6 * (size_t)s->planes * (size_t)std::max<int64_t>(cb_elems, 1) * sizeof(__nv_bfloat16);
            VB_CUDA(cudaMalloc(&s->d_chain, chain_bytes));
            VB_CUDA(cudaMemsetAsync(s->d_chain, 0, chain_bytes, e->stream));
        }
    }
    // where the final update of each tensor lives after a step
    std::vector<TensorDesc> desc_apply = desc;
    for (int64_t i = 0; i < nt; ++i) {
        if (s->local_off[(size_t)i] < 0) continue;
        float *fin = s->d_upd + s->local_off[(size_t)i];
        if (s->ns_kind[(size_t)i] == 1 && odd) fin = s->d_xnext + s->local_off[(size_t)i];
        s->final_update[(size_t)i] = fin;
        desc_apply[(size_t)i].g = fin;
    }
    VB_TRY(upload(&s->d_desc_apply, desc_apply, e->stream));

    // ---- Newton-Schulz schedules ----
    s->flops_per_step = 0.0;
    auto by_size = [&](int32_t a, int32_t b) { return opt->sizes[(size_t)a] > opt->sizes[(size_t)b]; };
    if (!f32_tensors.empty()) {
        int bm, bn;
        f32_gemm_tile_shape(&bm, &bn);
        std::vector<F32GemmProblem> gram[2], upd[2];
        std::vector<GemmTile> gram_tiles, upd_tiles;
        // largest matrices first so the tail of the persistent grid is short
        std::stable_sort(f32_tensors.begin(), f32_tensors.end(), by_size);
        for (int32_t t : f32_tensors) {
            const int r = (int)opt->rows[t], c = (int)opt->cols[t];
            float *buf[2] = {s->d_upd + s->local_off[(size_t)t], s->d_xnext + s->local_off[(size_t)t]};
            float *gm = s->d_gram + gram_off[(size_t)t];
            const int pidx = (int)gram[0].size();
            for (int par = 0; par < 2; ++par) {
                F32GemmProblem g{};  // xt_x = X^T X, then C = 3I - xt_x   (muon.rs:69-89)
                g.A = buf[par]; g.B = buf[par]; g.C = gm;
                g.M = c; g.N = c; g.K = r; g.lda = c; g.ldb = c; g.ldc = c;
                g.trans_a = 1; g.epilogue = F32_EPI_THREE_I_MINUS; g.tensor = t;
                gram[par].push_back(g);
                F32GemmProblem u{};  // X <- 0.5 * (X C)                  (muon.rs:93-99)
                u.A = buf[par]; u.B = gm; u.C = buf[par ^ 1];
                u.M = r; u.N = c; u.K = c; u.lda = c; u.ldb = c; u.ldc = c;
                u.trans_a = 0; u.epilogue = F32_EPI_HALF; u.tensor = t;
                upd[par].push_back(u);
            }
            for (int m0 = 0; m0 < c; m0 += bm)
                for (int n0 = 0; n0 < c; n0 += bn) gram_tiles.push_back(GemmTile{pidx, m0, n0, 0});
            for (int m0 = 0; m0 < r; m0 += bm)
                for (int n0 = 0; n0 < c; n0 += bn) upd_tiles.push_back(GemmTile{pidx, m0, n0, 0});
            s->flops_per_step += 4.0 * (double)r * (double)c * (double)c * (double)opt->ns_steps;
        }
        for (int par = 0; par < 2; ++par) {
            VB_TRY(upload(&s->d_gram_prob[par], gram[par], e->stream));
            VB_TRY(upload(&s->d_upd_prob[par], upd[par], e->stream));
        }
        VB_TRY(upload(&s->d_gram_tiles, gram_tiles, e->stream));
        VB_TRY(upload(&s->d_upd_tiles, upd_tiles, e->stream));
        s->n_gram_tiles = (int)gram_tiles.size();
        s->n_upd_tiles = (int)upd_tiles.size();
    }
    if (!tc_tensors.empty()) {
        int bm, bn;
        tc_gemm_tile_shape(&bm, &bn);
        const int iters = opt->ns_steps;
        std::vector<std::vector<TcGemmProblem>> gram((size_t)iters), upd((size_t)iters);
        std::vector<GemmTile> gram_tiles, upd_tiles, upd_tiles_last, upd_tiles_wide, upd_tiles_last_wide, gram_tiles_wide;
        const int wide_cols = (s->planes == 1 && !s->chain) ? tc_gemm_wide_cols() : 0;  // the chain form keeps to square tiles
        const int wide_gram_cols = (s->planes == 1 && !s->chain) ? tc_gemm_wide_gram_cols() : 0;
        // The chain form.  With C' = 3I - G every iterate is X_k = X_0 P_k with P_k a polynomial in
        // G_0 = X_0^T X_0, and all of G_k, C'_k, P_k commute and are symmetric:
        //     T_k = G_k C'_k,   G_{k+1} = C'_k T_k / 4,   C'_{k+1} = 3I - G_{k+1},   P'_{k+1} = P'_k C'_k  (P'_1 = C'_0)
        //     X_K = 2^-K X_0 P'_K
        // so only the first Gram and the last product touch the long side of the matrix; everything
        // in between is short-side squares, computed on and above the diagonal and mirrored.  For a
        // 4096 x 1024 matrix (n = 1024, 10 of 16 tiles on or above the diagonal) and K = 5 that is
        // 5 n^3 (first Gram) + 8 n^3 (last product) + 12 x 1.25 n^3 (squares) = 28 n^3 FLOP against
        // 5 x (5 + 8) n^3 = 65 n^3 for one Gram and one update product per iteration.  In exact
        // arithmetic the result is the reference's (tests/test_ns_chain_identity.py); in bf16 the
        // distance from the f32 oracle stays what the per-iteration form has (a few 1e-3, bound 2e-2).
        // G is stored from the accumulator itself, beside 3I - G (out2_bf16): deriving it from the
        // rounded C' loses its diagonal as G approaches I, and the chain diverges.
        const int n_chain_mid = std::max(iters - 1, 0);
        std::vector<TcGemmProblem> chain_l0, chain_final;
        std::vector<std::vector<TcGemmProblem>> chain_a((size_t)n_chain_mid), chain_b((size_t)n_chain_mid),
            chain_c((size_t)iters);  // chain_c[k], k = 1 .. iters - 1
        std::vector<std::vector<TcGemmProblem>> split_p((size_t)iters);  // f32-accurate path: the P products
        std::vector<GemmTile> small_tiles;
        std::stable_sort(tc_tensors.begin(), tc_tensors.end(), by_size);
        // plain bf16 path: the momentum kernel writes the unnormalised bf16 operand and the first
        // iteration's epilogues apply 1/norm; the split path keeps the reference's true division
        s->fold_norm = s->planes == 1;
        std::vector<uint8_t> fold((size_t)std::max<int64_t>(nt, 1), 0);
        for (int32_t t : tc_tensors) fold[(size_t)t] = s->fold_norm ? 1 : 0;
        VB_TRY(upload(&s->d_fold_norm, fold, e->stream));
        for (int32_t t : tc_tensors) {
            const int r = (int)opt->rows[t], c = (int)opt->cols[t];
            const bool tall = r >= c;
            const int sh = std::min(r, c);
            __nv_bfloat16 *xb[2] = {s->d_xb[0] + s->local_off[(size_t)t], s->d_xb[1] + s->local_off[(size_t)t]};
            __nv_bfloat16 *cb = s->d_cb + cb_off[(size_t)t];
            // X is fetched K-major (rows = m or n) or MN-major (rows = k) depending on the product
            const int mn_mode = tc_mn_major_mode(c);
            CUtensorMap map_x_k[2], map_x_mn[2], map_c, map_c_mn;
            const int c_mn_mode = tc_mn_major_mode(sh);
            const int planes = s->planes;
            const int n_terms = planes > 1 ? kSplitTerms : 1;
            for (int par = 0; par < 2; ++par) {
                VB_TRY(make_bf16_tensor_map(&map_x_k[par], xb[par], c, r, TC_OP_K_MAJOR, planes, s->owned_elems));
                VB_TRY(make_bf16_tensor_map(&map_x_mn[par], xb[par], c, r, mn_mode, planes, s->owned_elems));
            }
            VB_TRY(make_bf16_tensor_map(&map_c, cb, sh, sh, TC_OP_K_MAJOR, planes, s->cb_elems));
            VB_TRY(make_bf16_tensor_map(&map_c_mn, cb, sh, sh, c_mn_mode, planes, s->cb_elems));
            const int pidx = (int)gram[0].size();
            for (int it = 0; it < iters; ++it) {
                const int par = it & 1;
                const bool first = it == 0, last = it == iters - 1;
                // C = 3I - X^T X (tall: both operands are X read with k = row index, "MN-major")
                // C = 3I - X X^T (wide: both operands are X, K-major)
                TcGemmProblem g{};
                g.map_a = tall ? map_x_mn[par] : map_x_k[par];
                g.map_b = g.map_a;
                g.M = sh; g.N = sh; g.K = tall ? r : c;
                g.a_mode = tall ? mn_mode : TC_OP_K_MAJOR;
                g.b_mode = g.a_mode;
                // split path: keep the Gram itself and form 1.5 X - 0.5 X G in the update's epilogue
                g.epilogue = planes > 1 ? TC_EPI_IDENTITY : TC_EPI_THREE_I_MINUS; g.ld_out = sh; g.tensor = t;
                g.n_terms = n_terms; g.n_out_planes = planes; g.out_plane_stride = s->cb_elems;
                g.out_bf16 = cb; g.out_f32 = nullptr;
                if (first && s->fold_norm) {  // operands are u, not u/norm: G = (u^T u) / norm^2
                    g.scale_sumsq = s->d_sumsq + t;
                    g.scale_power = 2;
                }
                gram[(size_t)it].push_back(g);
                // X' = 0.5 X C (tall: A = X K-major, B = C which is symmetric)
                // X' = 0.5 C X (wide: A = C, B = X read with k = row index)
                // C is symmetric, so it can be staged either way round; the tensor core reads an
                // MN-major A operand measurably faster than a K-major one (wide update: +7.6 %), so
                // as the A operand C is staged MN-major.
                // Tall matrices on the plain bf16 path go one step further and compute the transposed
                // product (X C)^T = C X^T: A = C (MN-major), B = X with its rows as the n index
                // (K-major), and the epilogue stores each element at the transposed position, which is
                // X' in its ordinary row-major layout (+5 % on the tall update GEMMs).
                // (not in the last iteration, whose f32 result would go out in 4-byte pieces)
                const bool upd_t = tall && planes == 1 && !last && use_transposed_update();
                TcGemmProblem u{};
                u.map_a = upd_t ? map_c_mn : (tall ? map_x_k[par] : map_c_mn);
                u.map_b = upd_t ? map_x_k[par] : (tall ? map_c : map_x_mn[par]);
                u.M = upd_t ? sh : r; u.N = upd_t ? r : c; u.K = sh;
                u.a_mode = (upd_t || !tall) ? c_mn_mode : TC_OP_K_MAJOR;
                u.b_mode = tall ? TC_OP_K_MAJOR : mn_mode;
                u.transpose_out = upd_t ? 1 : 0;
                u.epilogue = planes > 1 ? TC_EPI_NS_COMBINE : TC_EPI_HALF; u.ld_out = c; u.tensor = t;
                u.in_bf16 = xb[par];
                if (planes > 1) u.split_sumsq = s->d_sumsq + t;
                u.n_terms = n_terms; u.n_out_planes = planes; u.out_plane_stride = s->owned_elems;
                u.out_bf16 = xb[par ^ 1]; u.out_f32 = nullptr;
                if (first && s->fold_norm) {  // X1 = 0.5 (u C) / norm
                    u.scale_sumsq = s->d_sumsq + t;
                    u.scale_power = 1;
                }
                if (last) {
                    u.out_bf16 = nullptr;  // last iteration: the f32 update is the result
                    u.out_f32 = s->d_upd + s->local_off[(size_t)t];
                    u.apply_w = opt->d_param + opt->offsets[(size_t)t];  // used when the launch applies it
                    u.apply_arena_pos = opt->offsets[(size_t)t];
                }
                upd[(size_t)it].push_back(u);
            }
            if (s->chain && s->chain_g_only) {
                // f32-accurate path: the chain with only G, T and P stored (two f16 planes each) and
                // C = 1.5 I - 0.5 G applied in the epilogues, which all have the form 1.5 Y - 0.5 (Y G)
                // of the per-iteration update (TC_EPI_NS_COMBINE):
                //     T_k = 1.5 G_k - 0.5 G_k G_k,   G_{k+1} = 1.5 T_k - 0.5 G_k T_k,   P_{k+1} = 1.5 P_k - 0.5 P_k G_k  (P_0 = I)
                //     X_K = X_0 P_K
                // G and T carry the scale of the Gram (2^(15 - 2e), see split_exponent), P is held at
                // 2^p_log2 with 1.5^K 2^p_log2 inside the f16 range; every product has G as one operand, so
                // the accumulator returns to the scale of Y by the same factor as in the update product.
                const int p_log2 = planes > 1 ? std::min(15, (int)std::floor(std::log2(60000.0 / std::pow(1.5, (double)iters)))) : 0;
                enum { kG0 = 0, kG1 = 1, kT = 2, kPI = 3, kPa = 4, kPb = 5 };
                __nv_bfloat16 *sq[6];
                CUtensorMap sq_k[6], sq_mn[6];
                const int64_t buf_stride = (int64_t)planes * cb_elems;
                for (int b = 0; b < 6; ++b) {
                    sq[b] = s->d_chain + (int64_t)b * buf_stride + cb_off[(size_t)t];
                    VB_TRY(make_bf16_tensor_map(&sq_k[b], sq[b], sh, sh, TC_OP_K_MAJOR, planes, cb_elems));
                    VB_TRY(make_bf16_tensor_map(&sq_mn[b], sq[b], sh, sh, c_mn_mode, planes, cb_elems));
                }
                set_identity_planes_kernel<<<(sh + 255) / 256, 256, 0, e->stream>>>(sq[kPI], sh, p_log2, planes == 1);
                VB_CUDA(cudaGetLastError());
                auto combine = [&](int y, int g, int out) {  // out = 1.5 Y - 0.5 (Y G)
                    TcGemmProblem q{};
                    q.map_a = sq_mn[y]; q.map_b = sq_k[g];
                    q.M = sh; q.N = sh; q.K = sh;
                    q.a_mode = c_mn_mode; q.b_mode = TC_OP_K_MAJOR;
                    q.epilogue = TC_EPI_NS_COMBINE; q.ld_out = sh; q.tensor = t;
                    q.n_terms = n_terms; q.n_out_planes = planes; q.out_plane_stride = cb_elems;
                    q.in_bf16 = sq[y];
                    q.split_sumsq = s->d_sumsq + t;
                    q.out_bf16 = sq[out];
                    return q;
                };
                TcGemmProblem l0 = gram[0].back();  // G_0 = X_0^T X_0 (plain path: of u, scaled by 1 / norm^2)
                l0.epilogue = TC_EPI_IDENTITY;
                l0.out_bf16 = sq[kG0];
                chain_l0.push_back(l0);
                auto p_buf = [&](int j) { return j == 0 ? (int)kPI : (j & 1) ? (int)kPa : (int)kPb; };
                for (int k = 0; k < iters; ++k) {
                    const int g_now = kG0 + (k & 1), g_next = kG0 + ((k + 1) & 1);
                    if (k + 1 < iters) {
                        chain_a[(size_t)k].push_back(combine(g_now, g_now, kT));   // T_k
                        chain_b[(size_t)k].push_back(combine(kT, g_now, g_next));  // G_{k+1}
                    }
                    split_p[(size_t)k].push_back(combine(p_buf(k), g_now, p_buf(k + 1)));  // P_{k+1}
                }
                TcGemmProblem fin = upd[(size_t)iters - 1].back();  // X_K = X_0 P_K, in the direct form of the update product
                const int pk = p_buf(iters);
                if (tall) {
                    fin.map_a = map_x_k[0];
                    fin.map_b = sq_k[pk];
                } else {
                    fin.map_a = sq_mn[pk];
                    fin.map_b = map_x_mn[0];
                }
                fin.in_bf16 = nullptr;
                if (planes > 1) {
                    fin.epilogue = TC_EPI_IDENTITY;  // the accumulator is X_K 2^(15 - e + p_log2)
                    fin.split_sumsq = s->d_sumsq + t;
                    fin.extra_scale = ldexpf(1.0f, 15 - p_log2);
                } else {
                    fin.epilogue = TC_EPI_HALF;  // X_K = (u P_K) / norm: 0.5 * 2
                    fin.scale_sumsq = s->d_sumsq + t;
                    fin.scale_power = 1;
                    fin.extra_scale = 2.0f;
                }
                chain_final.push_back(fin);
                for (int m0 = 0; m0 < sh; m0 += bm)
                    for (int n0 = m0; n0 < sh; n0 += bn)
                        small_tiles.push_back(GemmTile{pidx, m0, n0, n0 > m0 ? GEMM_TILE_MIRROR : 0});
            }
            if (s->chain && !s->chain_g_only) {
                __nv_bfloat16 *sq[6];  // G, T, C'[0], C'[1], P'[0], P'[1]
                CUtensorMap sq_k[6], sq_mn[6];
                for (int b = 0; b < 6; ++b) {
                    sq[b] = s->d_chain + (int64_t)b * cb_elems + cb_off[(size_t)t];
                    VB_TRY(make_bf16_tensor_map(&sq_k[b], sq[b], sh, sh, TC_OP_K_MAJOR, 1, 0));
                    VB_TRY(make_bf16_tensor_map(&sq_mn[b], sq[b], sh, sh, c_mn_mode, 1, 0));
                }
                enum { kG = 0, kT = 1, kC0 = 2, kP0 = 4 };
                auto small = [&](int a, int b, int out, int epi) {
                    TcGemmProblem q{};
                    q.map_a = sq_mn[a]; q.map_b = sq_k[b];  // both symmetric: A staged MN-major (the faster way)
                    q.M = sh; q.N = sh; q.K = sh;
                    q.a_mode = c_mn_mode; q.b_mode = TC_OP_K_MAJOR;
                    q.epilogue = epi; q.ld_out = sh; q.tensor = t;
                    q.n_terms = 1; q.n_out_planes = 1; q.out_plane_stride = 0;
                    q.out_bf16 = sq[out];
                    return q;
                };
                TcGemmProblem l0 = gram[0].back();  // G_0 = (u^T u) / norm^2 and C'_0 = 3I - G_0
                l0.out_bf16 = sq[kC0];
                l0.out2_bf16 = sq[kG];
                chain_l0.push_back(l0);
                for (int k = 0; k + 1 < iters; ++k) {
                    const int c_now = kC0 + (k & 1), c_next = kC0 + ((k + 1) & 1);
                    chain_a[(size_t)k].push_back(small(kG, c_now, kT, TC_EPI_IDENTITY));            // T_k = G_k C'_k
                    TcGemmProblem lb = small(c_now, kT, c_next, TC_EPI_THREE_I_MINUS);              // C'_{k+1} = 3I - C'_k T_k / 4
                    lb.extra_scale = 0.25f;
                    lb.out2_bf16 = sq[kG];                                                          // G_{k+1}
                    chain_b[(size_t)k].push_back(lb);
                }
                // P'_1 = C'_0 lives in C'[0]; P'_j (j >= 2) in P'[j & 1]
                auto p_buf = [&](int j) { return j == 1 ? (int)kC0 : kP0 + (j & 1); };
                for (int k = 1; k < iters; ++k)
                    chain_c[(size_t)k].push_back(small(p_buf(k), kC0 + (k & 1), p_buf(k + 1), TC_EPI_IDENTITY));
                // X_K = 2^-K (u P'_K) / norm, in the direct form of the last update product
                TcGemmProblem fin = upd[(size_t)iters - 1].back();
                const int pk = p_buf(iters);
                if (tall) {
                    fin.map_a = map_x_k[0];
                    fin.map_b = sq_k[pk];
                } else {
                    fin.map_a = sq_mn[pk];
                    fin.map_b = map_x_mn[0];
                }
                fin.in_bf16 = nullptr;
                fin.epilogue = TC_EPI_HALF;  // 0.5 * 2^(1 - K) = 2^-K
                fin.scale_sumsq = s->d_sumsq + t;
                fin.scale_power = 1;
                fin.extra_scale = ldexpf(1.0f, 1 - iters);
                chain_final.push_back(fin);
                for (int m0 = 0; m0 < sh; m0 += bm)
                    for (int n0 = m0; n0 < sh; n0 += bn)
                        small_tiles.push_back(GemmTile{pidx, m0, n0, n0 > m0 ? GEMM_TILE_MIRROR : 0});
            }
            // The Gram is symmetric: with square tiles only those on or above the diagonal are
            // computed; off-diagonal ones are also stored transposed by the epilogue.
            int gram_all = 0, gram_used = 0;
            const bool gram_wide = wide_gram_cols == 2 * bn && bm == bn && sh % bn == 0;
            if (gram_wide) {
                // rows of tiles on and above the diagonal, two 256-column halves per tile where a
                // partner exists: the halves share the staged rows of A, and the half on the
                // diagonal reads them as its B as well
                gram_all = (sh / bm) * (sh / bn);
                for (int m0 = 0; m0 < sh; m0 += bm) {
                    int n0 = m0;
                    while (n0 < sh) {
                        if (n0 + bn < sh) {
                            gram_tiles_wide.push_back(GemmTile{pidx, m0, n0, GEMM_TILE_SYMMETRIC});
                            n0 += 2 * bn;
                            gram_used += 2;
                        } else {
                            gram_tiles_wide.push_back(GemmTile{pidx, m0, n0, GEMM_TILE_SYMMETRIC | GEMM_TILE_SINGLE});
                            n0 += bn;
                            gram_used += 1;
                        }
                    }
                }
            }
            for (int m0 = 0; m0 < sh && !gram_wide; m0 += bm)
                for (int n0 = 0; n0 < sh; n0 += bn) {
                    ++gram_all;
                    if (bm == bn && n0 < m0) continue;
                    ++gram_used;
                    int flags = 0;
                    if (bm == bn && n0 > m0) flags |= GEMM_TILE_MIRROR;
                    if (bm == bn && n0 == m0 && planes == 1) flags |= GEMM_TILE_B_IS_A;
                    gram_tiles.push_back(GemmTile{pidx, m0, n0, flags});
                }
            const bool upd_t = tall && planes == 1 && use_transposed_update();  // as above: the update computes (X C)^T
            {
                const int um = upd_t ? sh : r, un = upd_t ? r : c;
                const bool wide = wide_cols > 0 && un % wide_cols == 0;
                for (int m0 = 0; m0 < um; m0 += bm)
                    for (int n0 = 0; n0 < un; n0 += wide ? wide_cols : bn)
                        (wide ? upd_tiles_wide : upd_tiles).push_back(GemmTile{pidx, m0, n0, 0});
            }
            {
                const bool wide = wide_cols > 0 && c % wide_cols == 0;
                for (int m0 = 0; m0 < r; m0 += bm)
                    for (int n0 = 0; n0 < c; n0 += wide ? wide_cols : bn)
                        (wide ? upd_tiles_last_wide : upd_tiles_last).push_back(GemmTile{pidx, m0, n0, 0});
            }
            // executed tensor-core FLOPs: three plane products per product on the split path; the
            // Gram counts only the tiles that are computed
            const double prod = 2.0 * (double)std::max(r, c) * (double)sh * (double)sh;
            if (s->chain) {
                const double upper = (double)gram_used / (double)gram_all;
                const double square = 2.0 * (double)sh * (double)sh * (double)sh * upper;
                const double n_squares = s->chain_g_only ? 3.0 * (double)iters - 2.0 : 3.0 * (double)(iters - 1);
                s->flops_per_step += (double)n_terms * (prod * upper + n_squares * square + prod);
            } else {
                s->flops_per_step += (double)n_terms * (double)opt->ns_steps *
                                     (prod * (double)gram_used / (double)gram_all + prod);
            }
        }
        if (s->chain) {
            if (bm != bn) return fail(VB_ERR_STATE, "the chain form needs square tiles");
            const int n_tc = (int)chain_l0.size();
            std::vector<GemmTile> small_tiles2 = small_tiles;  // two problem sets in one launch
            for (const GemmTile &tl : small_tiles) small_tiles2.push_back(GemmTile{tl.problem + n_tc, tl.m0, tl.n0, tl.flags});
            VB_TRY(upload(&s->d_small_tiles, small_tiles, e->stream));
            VB_TRY(upload(&s->d_small_tiles2, small_tiles2, e->stream));
            s->n_small_tiles = (int)small_tiles.size();
            s->n_small_tiles2 = (int)small_tiles2.size();
            auto add = [&](const std::vector<TcGemmProblem> &probs, const GemmTile *tiles, int n_tiles, bool fin,
                           bool dual = false) -> int {
                MuonState::TcLaunch l;
                VB_TRY(upload(&l.d_problems, probs, e->stream));
                l.d_tiles = tiles;
                l.n_tiles = n_tiles;
                l.final_product = fin;
                l.dual = dual;
                s->chain_launches.push_back(l);
                return VB_OK;
            };
            // the tile lists of the first Gram and of the last product are uploaded below; their
            // pointers are filled in once they exist
            if (s->chain_g_only) {
                // on the plain path the epilogue that reads a tile back lives in the kernel's second instantiation
                const bool aux = s->planes == 1;
                VB_TRY(add(chain_l0, nullptr, 0, false));
                for (int k = 0; k + 1 < iters; ++k) {  // T_k and P_{k+1} need only G_k: one launch
                    std::vector<TcGemmProblem> both = chain_a[(size_t)k];
                    both.insert(both.end(), split_p[(size_t)k].begin(), split_p[(size_t)k].end());
                    VB_TRY(add(both, s->d_small_tiles2, s->n_small_tiles2, false, aux));
                    VB_TRY(add(chain_b[(size_t)k], s->d_small_tiles, s->n_small_tiles, false, aux));
                }
                VB_TRY(add(split_p[(size_t)iters - 1], s->d_small_tiles, s->n_small_tiles, false, aux));
                VB_TRY(add(chain_final, nullptr, 0, true));
            }
            if (!s->chain_g_only) VB_TRY(add(chain_l0, nullptr, 0, false, /*dual=*/true));
            for (int k = 0; !s->chain_g_only && k + 1 < iters; ++k) {
                std::vector<TcGemmProblem> both = chain_a[(size_t)k];
                if (k >= 1) both.insert(both.end(), chain_c[(size_t)k].begin(), chain_c[(size_t)k].end());
                VB_TRY(add(both, k >= 1 ? s->d_small_tiles2 : s->d_small_tiles,
                           k >= 1 ? s->n_small_tiles2 : s->n_small_tiles, false));
                VB_TRY(add(chain_b[(size_t)k], s->d_small_tiles, s->n_small_tiles, false, /*dual=*/true));
            }
            if (!s->chain_g_only) {
                if (iters >= 2) VB_TRY(add(chain_c[(size_t)iters - 1], s->d_small_tiles, s->n_small_tiles, false));
                VB_TRY(add(chain_final, nullptr, 0, true));
            }
        }
        s->d_tc_gram.assign((size_t)iters, nullptr);
        s->d_tc_upd.assign((size_t)iters, nullptr);
        for (int it = 0; it < iters; ++it) {
            VB_TRY(upload(&s->d_tc_gram[(size_t)it], gram[(size_t)it], e->stream));
            VB_TRY(upload(&s->d_tc_upd[(size_t)it], upd[(size_t)it], e->stream));
        }
        VB_TRY(upload(&s->d_tc_gram_tiles, gram_tiles, e->stream));
        VB_TRY(upload(&s->d_tc_upd_tiles, upd_tiles, e->stream));
        VB_TRY(upload(&s->d_tc_upd_tiles_last, upd_tiles_last, e->stream));
        VB_TRY(upload(&s->d_tc_upd_tiles_wide, upd_tiles_wide, e->stream));
        VB_TRY(upload(&s->d_tc_gram_tiles_wide, gram_tiles_wide, e->stream));
        s->n_tc_gram_tiles_wide = (int)gram_tiles_wide.size();
        VB_TRY(upload(&s->d_tc_upd_tiles_last_wide, upd_tiles_last_wide, e->stream));
        s->n_tc_upd_tiles_wide = (int)upd_tiles_wide.size();
        s->n_tc_upd_tiles_last_wide = (int)upd_tiles_last_wide.size();
        s->n_tc_upd_tiles_last = (int)upd_tiles_last.size();
        s->n_tc_gram_tiles = (int)gram_tiles.size();
        s->n_tc_upd_tiles = (int)upd_tiles.size();
        if (s->chain) {
            s->chain_launches.front().d_tiles = s->d_tc_gram_tiles;
            s->chain_launches.front().n_tiles = s->n_tc_gram_tiles;
            s->chain_launches.back().d_tiles = s->d_tc_upd_tiles_last;
            s->chain_launches.back().n_tiles = s->n_tc_upd_tiles_last;
        }
    }
    VB_CUDA(cudaStreamSynchronize(e->stream));
    return VB_OK;
}

int muon_step(vb_optimizer *opt, uint32_t flags)
{
    vb_engine *e = opt->eng;
    MuonState *s = opt->muon;
    ExchangePlan xp;
    VB_TRY(plan_exchange(opt, flags, &xp));  // the same outcome on every rank: nothing is enqueued on a refusal
    // A GEMM kernel of an earlier step gave up a wait on this rank: the optimizer is fail-stop,
    // but this rank still takes every fence and collective of the step (its kernels skip their
    // work), so that no other rank is left waiting for it; the fence tells the peers.
    const int local_status = muon_check_error(opt);
    const bool compute = local_status == VB_OK;
    VB_TRY(sync_present(opt));
    xp.fence.local_error = s->d_error;
    const int ew_grid = (int)std::min<int64_t>(std::max<int64_t>(s->n_chunks, 1), (int64_t)e->sm_count * 8);
    const bool fast_norm = opt->ns_mode == VB_NS_BF16;  // both f32 modes need the reference's ordered sum
    const bool gsum = xp.pt.n_grad > 0;
    // peers' gradients are read by the first kernel: every rank must have reached its step
    // The last update launch applies its result itself (and stores the new weights into the peers
    // when their arenas are open: measured at 2 GPUs 3.37 ms per step against 3.57 ms with the
    // separate apply pass, since the NVLink stores then overlap the launch's tensor work).
    const bool fuse_now = s->fuse_apply && s->n_tc_upd_tiles_last + s->n_tc_upd_tiles_last_wide > 0;
    s->last_step_fused = fuse_now;
    bool fence1_done = false;
    if (gsum) {
        VB_TRY(exchange_fence(opt, xp, 1));
        fence1_done = true;
    }
    const uint32_t gemm_wait_limit = s->debug_wait_limit;  // 0 = the default; set by the expiry test hook
    TcGemmProblem *first_tc_problems = s->chain ? s->chain_launches.front().d_problems
                                                : (s->d_tc_gram.empty() ? nullptr : s->d_tc_gram[0]);
    if (s->debug_withhold && compute && first_tc_problems != nullptr) {
        const int32_t one = 1;
        VB_CUDA(cudaMemcpyAsync(reinterpret_cast<char *>(first_tc_problems) + offsetof(TcGemmProblem, withhold_loads), &one,
                                sizeof(one), cudaMemcpyHostToDevice, e->stream));
    }
    prof_begin(e, VB_PHASE_MUON_PRE);
    if (s->n_chunks > 0 && compute) {
        const uint8_t *direct = s->fold_norm ? s->d_fold_norm : nullptr;
        GradPeers gp{};
        gp.local_base = opt->d_grad;
        gp.n = xp.pt.n_grad;
        gp.rank = xp.pt.rank;
        gp.scale = xp.pt.grad_scale;
        gp.fence_error = xp.pt.fence_error;
        for (int r = 0; r < gp.n; ++r) gp.base[r] = xp.pt.grad_base[r];
        // a one-rank engine asked for the mean or the sum of gradients: scale 1, nothing to add
#define VB_MOMENTUM(P, G)                                                                                      \
    momentum_kernel<P, G><<<ew_grid, kEwThreads, 0, e->stream>>>(s->d_desc, s->d_chunks, s->n_chunks,      \
                                                                opt->d_present, opt->momentum, opt->nesterov, \
                                                                s->d_partials, direct, s->d_upd, s->d_xb[0], gp)
        if (fast_norm || s->n_seq_blocks > 0) {  // chunk sums: the sum itself (bf16 mode) or the binade guesses
            if (gsum) VB_MOMENTUM(true, true); else VB_MOMENTUM(true, false);
        } else {
            if (gsum) VB_MOMENTUM(false, true); else VB_MOMENTUM(false, false);
        }
#undef VB_MOMENTUM
        VB_CUDA(cudaGetLastError());
        e->launches += 1;
    }
    if (s->n_ns > 0 && compute) {
        if (fast_norm)
            reduce_partials_kernel<<<(s->n_ns + 3) / 4, 128, 0, e->stream>>>(s->d_partials, s->d_first_chunk,
                                                                            s->d_ns_tensors, s->n_ns, s->d_sumsq);
        else {
            if (s->n_seq_blocks > 0) {
                const int grid = std::min(s->n_seq_blocks, e->sm_count * 4);
                block_guess_kernel<<<(s->n_ns + 3) / 4, 128, 0, e->stream>>>(s->d_partials, s->d_first_chunk,
                                                                            s->d_first_block, s->d_ns_tensors, s->n_ns,
                                                                            opt->d_present, s->d_block_guess);
                block_map_kernel<<<grid, 512, 0, e->stream>>>(s->d_desc, s->d_seq_blocks, s->n_seq_blocks, s->d_sizes,
                                                              opt->d_present, s->d_block_guess, s->d_block_map);
                e->launches += 2;
            }
            sumsq_ordered_kernel<<<s->n_ns, kSeqThreads, 0, e->stream>>>(
                s->d_desc, s->d_ns_tensors, s->d_sizes, opt->d_present, s->d_sumsq, s->d_first_block,
                s->n_seq_blocks > 0 ? s->d_block_map : nullptr, s->d_block_guess);
        }
        VB_CUDA(cudaGetLastError());
        normalise_kernel<<<ew_grid, kEwThreads, 0, e->stream>>>(s->d_desc, s->d_chunks, s->n_chunks, opt->d_present,
                                                               s->d_ns_kind, s->d_sumsq, s->d_upd, s->d_xb[0],
                                                               s->owned_elems, s->fold_norm ? s->d_fold_norm : nullptr);
        VB_CUDA(cudaGetLastError());
        e->launches += 2;
        prof_end(e, VB_PHASE_MUON_PRE);
        prof_begin(e, VB_PHASE_MUON_NS);
        // the launch that yields the update applies it itself when fused (see TcApplyArgs)
        auto final_apply_args = [&](TcApplyArgs &ap) -> int {
            if (!fuse_now) return VB_OK;
            // this launch writes the new weights (also into the peers): nobody is written to
            // before it has reached its step
            if (!fence1_done) {
                prof_end(e, VB_PHASE_MUON_NS);
                VB_TRY(exchange_fence(opt, xp, 1));
                prof_begin(e, VB_PHASE_MUON_NS);
                fence1_done = true;
            }
            ap.enabled = 1;
            ap.keep_update = s->keep_update ? 1 : 0;
            ap.lr = opt->lr;
            ap.pt = xp.pt;
            // phase timing: this launch counts as Newton-Schulz and, on its own, as "apply"
            prof_begin(e, VB_PHASE_MUON_APPLY);
            return VB_OK;
        };
        if (s->chain) {
            for (const MuonState::TcLaunch &l : s->chain_launches) {
                TcApplyArgs ap{};
                if (l.final_product) VB_TRY(final_apply_args(ap));
                VB_TRY(launch_ns_gemm_tc(l.d_problems, l.d_tiles, l.n_tiles, opt->d_present, s->d_error, e->sm_count,
                                         e->stream, gemm_wait_limit, s->planes > 1, ap.enabled ? &ap : nullptr, false, l.dual));
                if (ap.enabled) prof_end(e, VB_PHASE_MUON_APPLY);
                e->launches += l.n_tiles > 0;
            }
        }
        for (int it = 0; it < opt->ns_steps; ++it) {
            const int par = it & 1;
            if (!s->chain && s->n_tc_gram_tiles + s->n_tc_gram_tiles_wide > 0) {
                const bool split = s->planes > 1;
                VB_TRY(launch_ns_gemm_tc(s->d_tc_gram[(size_t)it], s->d_tc_gram_tiles, s->n_tc_gram_tiles,
                                         opt->d_present, s->d_error, e->sm_count, e->stream, gemm_wait_limit, split));
                VB_TRY(launch_ns_gemm_tc(s->d_tc_gram[(size_t)it], s->d_tc_gram_tiles_wide, s->n_tc_gram_tiles_wide,
                                         opt->d_present, s->d_error, e->sm_count, e->stream, gemm_wait_limit, split, nullptr,
                                         /*wide=*/true));
                const bool last_it = it == opt->ns_steps - 1;
                TcApplyArgs ap{};
                if (last_it) VB_TRY(final_apply_args(ap));
                VB_TRY(launch_ns_gemm_tc(s->d_tc_upd[(size_t)it], last_it ? s->d_tc_upd_tiles_last : s->d_tc_upd_tiles,
                                         last_it ? s->n_tc_upd_tiles_last : s->n_tc_upd_tiles,
                                         opt->d_present, s->d_error, e->sm_count, e->stream, gemm_wait_limit, split,
                                         ap.enabled ? &ap : nullptr));
                const int n_wide = last_it ? s->n_tc_upd_tiles_last_wide : s->n_tc_upd_tiles_wide;
                VB_TRY(launch_ns_gemm_tc(s->d_tc_upd[(size_t)it],
                                         last_it ? s->d_tc_upd_tiles_last_wide : s->d_tc_upd_tiles_wide, n_wide,
                                         opt->d_present, s->d_error, e->sm_count, e->stream, gemm_wait_limit, split,
                                         ap.enabled ? &ap : nullptr, /*wide=*/true));
                if (ap.enabled) prof_end(e, VB_PHASE_MUON_APPLY);
                e->launches += (s->n_tc_gram_tiles > 0) + (s->n_tc_gram_tiles_wide > 0) +
                               ((last_it ? s->n_tc_upd_tiles_last : s->n_tc_upd_tiles) > 0) + (n_wide > 0);
            }
            if (s->n_gram_tiles > 0) {
                VB_TRY(launch_ns_gemm_f32(s->d_gram_prob[par], s->d_gram_tiles, s->n_gram_tiles, opt->d_present,
                                          e->sm_count, e->stream));
                VB_TRY(launch_ns_gemm_f32(s->d_upd_prob[par], s->d_upd_tiles, s->n_upd_tiles, opt->d_present,
                                          e->sm_count, e->stream));
                e->launches += 2;
            }
        }
        prof_end(e, VB_PHASE_MUON_NS);
        s->last_flops = s->flops_per_step;
        if (s->n_tc_gram_tiles + s->n_tc_gram_tiles_wide > 0)
            VB_CUDA(cudaMemcpyAsync(s->h_error, s->d_error, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    }
    prof_end(e, VB_PHASE_MUON_PRE);  // no-op if already closed (no Newton-Schulz matrices)
    if (s->debug_withhold && compute && first_tc_problems != nullptr) {
        const int32_t zero = 0;
        VB_CUDA(cudaMemcpyAsync(reinterpret_cast<char *>(first_tc_problems) + offsetof(TcGemmProblem, withhold_loads), &zero,
                                sizeof(zero), cudaMemcpyHostToDevice, e->stream));
        s->debug_withhold = false;
        s->debug_wait_limit = 0;
    }
    // see vb_optimizer_step_ex: nobody is written to before it has reached its step
    if (!fence1_done) VB_TRY(exchange_fence(opt, xp, 1));
    const ChunkDesc *apply_chunks = fuse_now ? s->d_chunks_apply : s->d_chunks;
    const int64_t n_apply_chunks = fuse_now ? s->n_chunks_apply : s->n_chunks;
    if (n_apply_chunks > 0 && compute) {
        if (!fuse_now) prof_begin(e, VB_PHASE_MUON_APPLY);  // fused: the phase is the last GEMM launch
        const bool f32_peers = xp.pt.n > 0;
        const int half = xp.pt.half_local == nullptr ? 0 : xp.pt.n_half > 0 ? 2 : 1;
        const int apply_grid = (int)std::min<int64_t>(n_apply_chunks, (int64_t)e->sm_count * 8);
#define VB_APPLY(P, H)                                                                                      \
    apply_kernel<P, H><<<apply_grid, kEwThreads, 0, e->stream>>>(s->d_desc_apply, apply_chunks, n_apply_chunks, \
                                                                opt->d_present, opt->lr, xp.pt, s->d_error)
        if (half == 0) {
            if (f32_peers) VB_APPLY(true, 0); else VB_APPLY(false, 0);
        } else if (half == 1) {
            if (f32_peers) VB_APPLY(true, 1); else VB_APPLY(false, 1);
        } else {
            if (f32_peers) VB_APPLY(true, 2); else VB_APPLY(false, 2);
        }
#undef VB_APPLY
        VB_CUDA(cudaGetLastError());
        if (!fuse_now) prof_end(e, VB_PHASE_MUON_APPLY);
        e->launches += 1;
    }
    VB_TRY(exchange_fence(opt, xp, 2));
    if (xp.nccl_f32 || xp.nccl_half) {
        // every matrix from its owner; all ranks must hold the same gradient-presence flags
        std::vector<BcastItem> items;
        for (int64_t i = 0; i < opt->n_tensors; ++i) {
            if (!opt->present[(size_t)i] || opt->sizes[(size_t)i] == 0) continue;
            if (xp.nccl_f32)
                items.push_back(BcastItem{opt->d_param + opt->offsets[(size_t)i], opt->sizes[(size_t)i],
                                          s->owner[(size_t)i], 4});
            if (xp.nccl_half)
                items.push_back(BcastItem{opt->d_param_bf16 + opt->offsets[(size_t)i], opt->sizes[(size_t)i] * 2,
                                          s->owner[(size_t)i], 1});
        }
        prof_begin(e, VB_PHASE_EXCHANGE);
        VB_TRY(comm_group_broadcast(e, items.data(), (int64_t)items.size()));
        prof_end(e, VB_PHASE_EXCHANGE);
    }
    if (!compute) return muon_check_error(opt);  // sets the message again
    return VB_OK;
}

int muon_reset_velocity(vb_optimizer *opt)
{
    const size_t bytes = (size_t)std::max<int64_t>(opt->muon->owned_elems, 1) * sizeof(float);
    VB_CUDA(cudaMemsetAsync(opt->d_s1, 0, bytes, opt->eng->stream));
    return VB_OK;
}

int muon_set_keep_update(vb_optimizer *opt, int keep)
{
    opt->muon->keep_update = keep != 0;
    return VB_OK;
}

int muon_debug_withhold(vb_optimizer *opt, uint32_t wait_limit)
{
    MuonState *s = opt->muon;
    if (!s || s->d_tc_gram.empty())
        return fail(VB_ERR_STATE, "the optimizer runs no tensor-core Newton-Schulz kernel on this rank");
    s->debug_withhold = true;
    s->debug_wait_limit = wait_limit;
    return VB_OK;
}

int muon_download_update(vb_optimizer *opt, int64_t tensor, float *host, int64_t n)
{
    MuonState *s = opt->muon;
    if (s->local_off[(size_t)tensor] < 0)
        return fail(VB_ERR_STATE, "tensor %lld is owned by rank %d", (long long)tensor, s->owner[(size_t)tensor]);
    if (n == 0) return VB_OK;
    if (!host) return fail(VB_ERR_INVALID_ARG, "host pointer is null");
    if (s->last_step_fused && s->ns_kind[(size_t)tensor] >= 2 && opt->ns_steps > 0 && !s->keep_update)
        return fail(VB_ERR_STATE, "the update of a tensor-core matrix is applied inside the last GEMM and not stored; "
                                  "call vb_muon_set_keep_update(opt, 1) before the step");
    VB_CUDA(cudaMemcpyAsync(host, s->final_update[(size_t)tensor], (size_t)n * sizeof(float),
                            cudaMemcpyDeviceToHost, opt->eng->stream));
    VB_CUDA(cudaStreamSynchronize(opt->eng->stream));
    return muon_check_error(opt);
}

// Launches the tensor-core GEMM on a small synthetic problem whose producer withholds its
// loads, so every role's bounded wait expires, and reports what the kernel recorded.
int debug_gemm_wait_expiry(vb_engine *e, uint32_t wait_limit, int *role_code)
{
    const int n = 256;
    __nv_bfloat16 *x = nullptr, *c = nullptr;
    TcGemmProblem *d_prob = nullptr;
    GemmTile *d_tile = nullptr;
    uint8_t *d_present = nullptr;
    int *d_err = nullptr;
    int status = VB_OK, code = 0;
    auto cleanup = [&]() {
        cudaFree(x); cudaFree(c); cudaFree(d_prob); cudaFree(d_tile); cudaFree(d_present); cudaFree(d_err);
    };
#define VB_DBG_CUDA(expr)                                                                        \
    do {                                                                                         \
        cudaError_t _e = (expr);                                                                 \
        if (_e != cudaSuccess) {                                                                 \
            cleanup();                                                                           \
            return fail(VB_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e));            \
        }                                                                                        \
    } while (0)
    VB_DBG_CUDA(cudaMalloc(&x, (size_t)n * n * 2));
    VB_DBG_CUDA(cudaMalloc(&c, (size_t)n * n * 2));
    VB_DBG_CUDA(cudaMemsetAsync(x, 0, (size_t)n * n * 2, e->stream));
    VB_DBG_CUDA(cudaMalloc(&d_prob, sizeof(TcGemmProblem)));
    VB_DBG_CUDA(cudaMalloc(&d_tile, sizeof(GemmTile)));
    VB_DBG_CUDA(cudaMalloc(&d_present, 1));
    VB_DBG_CUDA(cudaMalloc(&d_err, sizeof(int)));
    VB_DBG_CUDA(cudaMemsetAsync(d_present, 1, 1, e->stream));
    VB_DBG_CUDA(cudaMemsetAsync(d_err, 0, sizeof(int), e->stream));
    TcGemmProblem p{};
    status = make_bf16_tensor_map(&p.map_a, x, n, n, TC_OP_K_MAJOR);
    if (status == VB_OK) status = make_bf16_tensor_map(&p.map_b, x, n, n, TC_OP_K_MAJOR);
    if (status != VB_OK) {
        cleanup();
        return status;
    }
    p.M = p.N = p.K = n;
    p.a_mode = p.b_mode = TC_OP_K_MAJOR;
    p.epilogue = TC_EPI_HALF;
    p.ld_out = n;
    p.tensor = 0;
    p.n_terms = 1;
    p.n_out_planes = 1;
    p.withhold_loads = 1;
    p.out_bf16 = c;
    const GemmTile t{0, 0, 0, 0};
    VB_DBG_CUDA(cudaMemcpyAsync(d_prob, &p, sizeof(p), cudaMemcpyHostToDevice, e->stream));
    VB_DBG_CUDA(cudaMemcpyAsync(d_tile, &t, sizeof(t), cudaMemcpyHostToDevice, e->stream));
    status = launch_ns_gemm_tc(d_prob, d_tile, 1, d_present, d_err, e->sm_count, e->stream, wait_limit);
    if (status == VB_OK) {
        VB_DBG_CUDA(cudaMemcpyAsync(&code, d_err, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
        VB_DBG_CUDA(cudaStreamSynchronize(e->stream));
    }
#undef VB_DBG_CUDA
    cleanup();
    if (status != VB_OK) return status;
    if (role_code) *role_code = code;
    if (code != 0)
        return fail(VB_ERR_TIMEOUT, "a Newton-Schulz GEMM kernel gave up waiting on a pipeline barrier (role %d)", code);
    return VB_OK;
}

int muon_last_flops(vb_optimizer *opt, double *flops)
{
    *flops = opt->muon->last_flops;
    return VB_OK;
}

}  // namespace vb
