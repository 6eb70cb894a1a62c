// Internal declarations shared by the translation units of libvolta_b200.so.
// Nothing here is part of the C ABI (include/volta_b200.h).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/volta_b200.h"

namespace vb {

// ---- error plumbing -------------------------------------------------------------------
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);

#define VB_CUDA(expr)                                                                       \
    do {                                                                                    \
        cudaError_t _e = (expr);                                                            \
        if (_e != cudaSuccess)                                                              \
            return ::vb::fail(VB_ERR_CUDA, "%s failed: %s (%d) at %s:%d", #expr,            \
                              cudaGetErrorString(_e), (int)_e, __FILE__, __LINE__);         \
    } while (0)

#define VB_TRY(expr)                 \
    do {                             \
        int _s = (expr);             \
        if (_s != VB_OK) return _s;  \
    } while (0)

// ---- descriptors read by the multi-tensor kernels ------------------------------------
// One entry per tensor.  For a sharded optimizer s1/s2 are biased so that s1 + i is the
// state of element i of the tensor for every i this rank owns.
struct TensorDesc {
    float *p;
    const float *g;
    float *s1;
    float *s2;
};
// One entry per unit of work: `len` consecutive elements of one tensor from `offset`.
// A chunk never crosses a tensor boundary, so ragged tensor lists load-balance.
struct ChunkDesc {
    int64_t offset;
    uint32_t tensor;
    uint32_t len;
};

// Unit of work of the fused Adam/SGD kernel: `len` consecutive elements of one tensor with
// the four array addresses resolved on the host, so the kernel needs one 48-byte fetch per
// chunk and no dependent lookups.
struct alignas(16) FatChunk {
    float *p;
    const float *g;
    float *s1;
    float *s2;
    uint32_t len;
    uint32_t tensor;
    uint32_t local_only;  // 1: a chunk of the replicated tail: the new values stay on this GPU
    uint32_t pad;
};
static_assert(sizeof(FatChunk) == 48, "FatChunk is fetched as three 16-byte words");

// Peer GPUs' parameter arenas (same layout as the local one), mapped into this process, and
// the optional bf16 copies of the parameters (one 16-bit word per arena element, local and
// on the peers).  A launch stores f32 to `n` peers, bf16 locally when `half_local` is set and
// bf16 to `n_half` peers.
constexpr int kMaxPeers = 7;
struct PeerTable {
    float *base[kMaxPeers];
    uint16_t *half_base[kMaxPeers];
    const float *grad_base[kMaxPeers];  // peers' gradient arenas, in rank order without this rank
    const float *local_base;
    uint16_t *half_local;
    int n;
    int n_half;
    int n_grad;        // > 0: the gradient of an element is the sum over all ranks, in rank order
    int rank;          // this rank's place in that order
    float grad_scale;  // the sum is multiplied by this (1, or 1 / world for the mean)
    // The error words of this rank's fence block (kSyncError, one per rank), or null when the step
    // touches no peer memory.  A kernel that finds one set does nothing: the fence before it gave
    // up (a peer never reached the step, or failed), so peers must not be written to or read from.
    const uint32_t *fence_error;
};

#ifdef __CUDACC__
__device__ __forceinline__ bool fence_failed(const uint32_t *fence_error)
{
    if (fence_error == nullptr) return false;
    uint32_t any = 0;
#pragma unroll
    for (int r = 0; r <= 7; ++r) any |= reinterpret_cast<const volatile uint32_t *>(fence_error)[r];
    return any != 0u;
}
#endif

// Flag words that order the ranks around a step that touches peer memory.  Every arena that can
// be opened by the peers (parameters, bf16 copies, gradients) carries one block of kSyncWords
// 32-bit words behind its last element, so a peer that maps the arena maps the block as well.
// Rank r writes word [r] of a group in every rank's block; a rank polls only its own block.
constexpr int kSyncWords = 256;       // 1 KiB
constexpr int kSyncArrive = 0;        // [r]: epoch of the last step rank r has reached
constexpr int kSyncDone = 32;         // [r]: epoch of the last step whose peer accesses rank r has finished
constexpr int kSyncError = 64;        // [r]: non-zero once rank r gave up a wait (sticky)
struct FenceArgs {
    uint32_t *local;                  // this rank's block
    uint32_t *peer[kMaxPeers];        // the peers' blocks, in rank order without this rank
    uint32_t *host_error;             // mapped pinned word the host reads without a copy (may be null)
    const int *local_error;           // if set and non-zero: a kernel of this rank failed during the step; the
                                      // fence reports it to every rank as if a wait had run out
    int n_peers;
    int rank;
    uint32_t epoch;
    uint64_t wait_ns;                 // bound of each wait
};
// phase 1: tell every peer "rank has reached step `epoch`" and wait until all peers have;
// phase 2: tell every peer "rank's accesses of step `epoch` are complete" and wait for theirs.
// A wait that runs out stores an error code for every rank and for the host and returns; later
// waits on any rank then give up at once, so all ranks fail together.
int launch_exchange_fence(const FenceArgs &args, int phase, cudaStream_t stream);

// Scalars of one step, computed on the host in f32 exactly as the reference does.
struct StepScalars {
    float lr;
    float beta1;            // Adam beta1 / SGD momentum
    float beta2;
    float one_minus_beta1;  // 1.0f - beta1   (src/nn/optim/adam.rs:176)
    float one_minus_beta2;  // 1.0f - beta2   (adam.rs:183)
    float m_hat_scale;      // 1/(1 - beta1.powi(t))  (adam.rs:188)
    float v_hat_scale;      // 1/(1 - beta2.powi(t))  (adam.rs:189)
    float eps;
    float weight_decay;
};

enum MultiTensorOp { OP_SGD = 0, OP_SGD_MOMENTUM = 1, OP_ADAM = 2 };

// f32::powi as compiler-rt's __powisf2 computes it (square-and-multiply, exponent bits
// least significant first, each product rounded to f32).
float powi_f32(float a, int b);
StepScalars make_scalars(int op, float lr, float beta1, float beta2, float eps, float wd, int64_t t);

// Launches the fused multi-tensor update over `n_chunks` chunks.  `present` holds one
// byte per tensor (0 = gradient absent, skip).
int launch_multi_tensor(int op, const FatChunk *d_chunks, int64_t n_chunks, const uint8_t *d_present,
                        bool all_present, const StepScalars &s, int sm_count, cudaStream_t stream,
                        const PeerTable *peers = nullptr);

// Checks shared by the two caller-buffer entry points, all on the host and before any launch:
// null pointers, 4-byte alignment of every array the op touches (a misaligned pointer would
// fault the scalar path of the kernel), Adam's t, and -- once per distinct pointer set -- that
// every pointer is device (or managed) memory of the engine's device.  Allocates nothing.
// *total receives the number of elements.
int check_caller_buffers(const vb_optimizer_step_params *hp, int64_t n_tensors, const int64_t *sizes,
                         void *const *params, const void *const *grads, void *const *state1, void *const *state2,
                         int64_t *total);
int check_caller_memory(vb_engine *e, const vb_optimizer_step_params *hp, int64_t n_tensors, const int64_t *sizes,
                        void *const *params, const void *const *grads, void *const *state1, void *const *state2);

// Device, SM count and stream of an engine / launch bookkeeping, for translation units that
// do not see the engine's definition (api.cu).
int engine_launch_info(vb_engine *e, int *device, int *sm_count, cudaStream_t *stream);
void engine_count_launch(vb_engine *e);

// bf16[i] = round-to-nearest-even(src[i]) for i in [0, n)
int launch_f32_to_bf16(uint16_t *dst, const float *src, int64_t n, int sm_count, cudaStream_t stream);

int launch_accumulate_grad(float *grad, const float *src, int64_t n, bool add, int sm_count, cudaStream_t stream);

// Splits [begin, end) of each tensor into chunks.
int64_t pick_chunk_len(int64_t total_elements, int sm_count);

}  // namespace vb
