// Fused multi-tensor Adam / SGD update for sm_100a.
//
// One launch updates every tensor of an optimizer: the grid strides over a chunk table
// (fixed-length pieces of tensors, so ragged tensor lists load-balance), each chunk is
// streamed with 128-bit loads/stores of param / grad / state, and every element is
// touched exactly once (HBM traffic = 28 B/param for Adam, 20 B/param for SGD with
// momentum, 12 B/param for plain SGD).
//
// Arithmetic contract: bit-identical to Volta's CPU optimizers
// (src/nn/optim/adam.rs:139-205, src/nn/optim/sgd.rs:189-238).  Rust never contracts
// a*b+c, so every operation below is an explicitly rounded intrinsic (__fmul_rn,
// __fadd_rn, ... are never fused by nvcc) and __fmaf_rn appears only where the
// reference writes mul_add.  Division and square root are the IEEE-rounded forms.
#include "vb_internal.h"

namespace vb {

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 2;  // independent 128-bit transactions per array per thread in flight

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

template <int OP>
__global__ void __launch_bounds__(kThreads)
multi_tensor_update_kernel(const TensorDesc *__restrict__ tensors,
                           const ChunkDesc *__restrict__ chunks, int64_t n_chunks,
                           const uint8_t *__restrict__ present, const StepScalars s)
{
    constexpr bool kHasS1 = (OP != OP_SGD);
    constexpr bool kHasS2 = (OP == OP_ADAM);

    for (int64_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        const ChunkDesc ch = chunks[c];
        if (present[ch.tensor] == 0) continue;  // `grad == None`: adam.rs:81-84, sgd.rs:75-78
        const TensorDesc td = tensors[ch.tensor];
        float *__restrict__ p = td.p + ch.offset;
        const float *__restrict__ g = td.g + ch.offset;
        float *__restrict__ s1 = kHasS1 ? td.s1 + ch.offset : nullptr;
        float *__restrict__ s2 = kHasS2 ? td.s2 + ch.offset : nullptr;
        const uint32_t n = ch.len;

        uintptr_t align_bits = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g);
        if (kHasS1) align_bits |= reinterpret_cast<uintptr_t>(s1);
        if (kHasS2) align_bits |= reinterpret_cast<uintptr_t>(s2);

        uint32_t done = 0;
        if ((align_bits & 15u) == 0) {
            const uint32_t n4 = n >> 2;
            float4 *__restrict__ p4 = reinterpret_cast<float4 *>(p);
            const float4 *__restrict__ g4 = reinterpret_cast<const float4 *>(g);
            float4 *__restrict__ a4 = reinterpret_cast<float4 *>(s1);
            float4 *__restrict__ b4 = reinterpret_cast<float4 *>(s2);
            for (uint32_t base = 0; base < n4; base += kThreads * kUnroll) {
                float4 vp[kUnroll], vg[kUnroll], va[kUnroll], vb[kUnroll];
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const uint32_t i = base + u * kThreads + threadIdx.x;
                    if (i < n4) {
                        vp[u] = __ldcs(p4 + i);
                        vg[u] = __ldcs(g4 + i);
                        if (kHasS1) va[u] = __ldcs(a4 + i);
                        if (kHasS2) vb[u] = __ldcs(b4 + i);
                    }
                }
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const uint32_t i = base + u * kThreads + threadIdx.x;
                    if (i < n4) {
                        update_vec<OP>(vp[u], vg[u], va[u], vb[u], s);
                        __stcs(p4 + i, vp[u]);
                        if (kHasS1) __stcs(a4 + i, va[u]);
                        if (kHasS2) __stcs(b4 + i, vb[u]);
                    }
                }
            }
            done = n4 << 2;
        }
        // ragged tail (n mod 4) or a chunk whose pointers are not 16-byte aligned
        for (uint32_t i = done + threadIdx.x; i < n; i += kThreads) {
            float vp = p[i], va = 0.0f, vb = 0.0f;
            const float vg = g[i];
            if (kHasS1) va = s1[i];
            if (kHasS2) vb = s2[i];
            update_one<OP>(vp, vg, va, vb, s);
            p[i] = vp;
            if (kHasS1) s1[i] = va;
            if (kHasS2) s2[i] = vb;
        }
    }
}

template <int OP>
int occupancy_ctas_per_sm()
{
    static int cached = 0;
    if (cached == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, multi_tensor_update_kernel<OP>,
                                                          kThreads, 0) != cudaSuccess || n < 1)
            n = 4;
        cached = n;
    }
    return cached;
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
    // Enough chunks that every SM sees dozens (small tail), but each long enough to
    // amortise the descriptor fetch: between 2 Ki and 16 Ki elements, a multiple of
    // kThreads * 4 * kUnroll so full chunks have no partial vector iteration.
    const int64_t quantum = kThreads * 4 * kUnroll;
    int64_t len = total_elements / ((int64_t)sm_count * 64);
    len = (len + quantum - 1) / quantum * quantum;
    if (len < quantum) len = quantum;
    if (len > 8 * quantum) len = 8 * quantum;
    return len;
}

int launch_multi_tensor(int op, const TensorDesc *d_tensors, const ChunkDesc *d_chunks,
                        int64_t n_chunks, const uint8_t *d_present, const StepScalars &s,
                        int sm_count, cudaStream_t stream)
{
    if (n_chunks <= 0) return VB_OK;
    int per_sm;
    switch (op) {
        case OP_ADAM: per_sm = occupancy_ctas_per_sm<OP_ADAM>(); break;
        case OP_SGD_MOMENTUM: per_sm = occupancy_ctas_per_sm<OP_SGD_MOMENTUM>(); break;
        case OP_SGD: per_sm = occupancy_ctas_per_sm<OP_SGD>(); break;
        default: return fail(VB_ERR_INVALID_ARG, "unknown multi-tensor op %d", op);
    }
    int64_t grid = (int64_t)sm_count * per_sm;  // whole waves: a multiple of the SM count
    if (grid > n_chunks) grid = n_chunks;
    switch (op) {
        case OP_ADAM:
            multi_tensor_update_kernel<OP_ADAM><<<(unsigned)grid, kThreads, 0, stream>>>(
                d_tensors, d_chunks, n_chunks, d_present, s);
            break;
        case OP_SGD_MOMENTUM:
            multi_tensor_update_kernel<OP_SGD_MOMENTUM><<<(unsigned)grid, kThreads, 0, stream>>>(
                d_tensors, d_chunks, n_chunks, d_present, s);
            break;
        default:
            multi_tensor_update_kernel<OP_SGD><<<(unsigned)grid, kThreads, 0, stream>>>(
                d_tensors, d_chunks, n_chunks, d_present, s);
            break;
    }
    VB_CUDA(cudaGetLastError());
    return VB_OK;
}

}  // namespace vb
