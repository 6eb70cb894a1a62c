// Stream-ordered barrier between the ranks of a sharded optimizer, in peer-mapped memory.
//
// A step whose kernels store into (or load from) other GPUs' arenas must not start before
// every rank has reached its step (the peers' earlier readers of the parameters are done,
// their gradients are written) and must not end before every rank's peer accesses have
// completed.  Both conditions are flags: one 32-bit epoch per rank and condition, written with
// a system-scope release store into every rank's block and polled locally with acquire loads.
// One tiny kernel per phase sits in the engine's stream on either side of the update kernel, so
// kernel boundaries order the flags against the data (a kernel's stores are performed system
// wide before the next kernel of the stream starts).  No collective library call is involved.
//
// Every wait is bounded (wall time from %globaltimer plus an iteration cap).  A rank that
// gives up writes its error word on every rank and in a mapped host word; waits on any rank end
// as soon as they see an error word, so one stuck rank makes all ranks return in bounded time
// with the GPU context intact.  Each GPU runs only its own fence kernel: nothing here needs two
// kernels to be resident on one GPU at the same time.
#include "vb_internal.h"

namespace vb {

namespace {

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

constexpr uint32_t kMaxPolls = 1u << 30;

// One warp; lane j < n_peers talks to peer j.
__global__ void __launch_bounds__(32) exchange_fence_kernel(const FenceArgs a, int phase)
{
    const int j = threadIdx.x;
    const int group = phase == 1 ? kSyncArrive : kSyncDone;
    bool ok = true;
    if (j < a.n_peers) {
        uint32_t *peer = nullptr;
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
            if (r == j) peer = a.peer[r];
        const int peer_rank = j < a.rank ? j : j + 1;
        st_release_sys(peer + group + a.rank, a.epoch);
        const uint32_t *flag = a.local + group + peer_rank;
        const uint64_t t0 = globaltimer_ns();
        for (uint32_t it = 0;; ++it) {
            if ((int32_t)(ld_acquire_sys(flag) - a.epoch) >= 0) break;
            if ((it & 7u) == 7u) {
                bool failed = it >= kMaxPolls || globaltimer_ns() - t0 > a.wait_ns;
#pragma unroll
                for (int r = 0; r <= kMaxPeers; ++r) failed |= ld_acquire_sys(a.local + kSyncError + r) != 0u;  // any rank gave up
                if (failed) {
                    ok = false;
                    break;
                }
                __nanosleep(100);
            }
        }
    }
    // One lane giving up ends the step for the whole rank: every peer is told, not only the one
    // that was waited for, so that all ranks stop together.
    if (a.local_error != nullptr && *reinterpret_cast<const volatile int *>(a.local_error) != 0) ok = false;
    // A rank that gave up earlier has written its error word here: this rank fails with it even if
    // the flags it was waiting for are all there (the failed rank publishes its flags before it
    // waits), so that no rank goes on alone.
    if (j == 0) {
#pragma unroll
        for (int r = 0; r <= kMaxPeers; ++r)
            if (ld_acquire_sys(a.local + kSyncError + r) != 0u) ok = false;
    }
    const bool bad = __any_sync(0xffffffffu, !ok);
    if (bad) {
        const uint32_t code = (uint32_t)phase;  // names the phase that ran out
        if (j < a.n_peers) {
            uint32_t *peer = nullptr;
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
                if (r == j) peer = a.peer[r];
            st_release_sys(peer + kSyncError + a.rank, code);
        }
        if (j == 0) {
            st_release_sys(a.local + kSyncError + a.rank, code);
            if (a.host_error) *reinterpret_cast<volatile uint32_t *>(a.host_error) = code;
        }
    }
    __syncwarp();
}

}  // namespace

int launch_exchange_fence(const FenceArgs &args, int phase, cudaStream_t stream)
{
    if (args.n_peers <= 0 || args.local == nullptr) return VB_OK;
    if (phase != 1 && phase != 2) return fail(VB_ERR_INVALID_ARG, "fence phase %d", phase);
    exchange_fence_kernel<<<1, 32, 0, stream>>>(args, phase);
    VB_CUDA(cudaGetLastError());
    return VB_OK;
}

}  // namespace vb
