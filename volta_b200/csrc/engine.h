// Engine and optimizer objects behind the opaque handles of include/volta_b200.h.
#pragma once

#include <memory>

#include "vb_internal.h"

namespace vb {
struct Comm;       // comm.cpp: NCCL communicator (library resolved at run time)
struct MuonState;  // muon.cu: matrices, work buffers and GEMM schedules of a Muon optimizer
void destroy_muon_state(MuonState *);
}  // namespace vb

struct vb_optimizer;

struct vb_engine {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    uint64_t launches = 0;
    int rank = 0;
    int world = 1;
    vb::Comm *comm = nullptr;
    // staging for vb_multi_tensor_step (caller-owned buffers): descriptors are written to
    // pinned host memory and copied to the device on the stream, double buffered.
    void *h_stage[2] = {nullptr, nullptr};
    void *d_stage[2] = {nullptr, nullptr};
    size_t stage_bytes[2] = {0, 0};
    cudaEvent_t stage_done[2] = {nullptr, nullptr};
    int stage_next = 0;
    // copy streams and events of the pipelined host step (vb_optimizer_step_host)
    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
    std::vector<cudaEvent_t> pipe_events;
    cudaStream_t peer_streams[vb::kMaxPeers] = {};  // vb_optimizer_peer_copy_probe: one copy stream per peer
    cudaEvent_t peer_events[vb::kMaxPeers + 3] = {};
    float *d_accum_scratch = nullptr;  // staging for host contributions to vb_optimizer_accumulate_grad
    size_t accum_scratch_elems = 0;
    // caller-buffer entry points: hashes of the pointer sets whose memory type and device were
    // already checked (cudaPointerGetAttributes costs about a microsecond per pointer)
    uint64_t checked_sets[4] = {0, 0, 0, 0};
    int checked_next = 0;
    std::vector<vb_optimizer *> optimizers;  // alive optimizers of this engine (their error words are read on synchronize)
    cudaEvent_t deadline_event = nullptr;  // vb_engine_synchronize_deadline
    uint32_t wait_limit_ms = 5000;         // bound of every device-side wait on another rank
    double replicated_fraction = 0.0;      // Adam/SGD optimizers created from now on: share of the arena every rank updates itself
    // optional phase timing (vb_engine_set_profiling): event pairs per phase, summed on query
    bool profiling = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof_pairs[VB_PHASE_COUNT];
    std::vector<cudaEvent_t> prof_free;
    cudaEvent_t prof_open[VB_PHASE_COUNT] = {};
};

enum OptimizerKind { KIND_ADAM = 0, KIND_SGD = 1, KIND_MUON = 2 };

struct vb_optimizer {
    vb_engine *eng = nullptr;
    int kind = KIND_ADAM;
    int64_t n_tensors = 0;
    std::vector<int64_t> sizes;    // elements per tensor
    std::vector<int64_t> offsets;  // element offset of each tensor in the arenas
    std::vector<int64_t> rows, cols;  // Muon's 2-D view
    int64_t total = 0;             // sum of sizes
    int64_t arena = 0;             // arena length in elements (padded)
    // this rank's slice of the arena (Adam/SGD state lives only here)
    int64_t shard_begin = 0, shard_end = 0;
    int64_t tail_begin = 0;  // [tail_begin, arena): updated by every rank itself, never exchanged (== arena: none)
    // index into the state arrays of an arena position this rank updates (slice first, then the tail)
    int64_t state_pos(int64_t pos) const
    {
        return pos < tail_begin ? pos - shard_begin : (shard_end - shard_begin) + (pos - tail_begin);
    }

    float *d_param = nullptr;
    float *d_grad = nullptr;
    float *d_s1 = nullptr;  // Adam m / SGD velocity / Muon velocity
    float *d_s2 = nullptr;  // Adam v
    int64_t state_elems = 0;

    // hyper-parameters
    float lr = 0, beta1 = 0, beta2 = 0, eps = 0, weight_decay = 0, momentum = 0;
    int nesterov = 0, ns_steps = 0, ns_mode = 0;
    int64_t t = 0;

    // descriptors
    vb::FatChunk *d_chunks = nullptr;
    std::vector<int64_t> chunk_pos;  // arena position of each chunk's first element (ascending)
    int64_t n_chunks = 0;
    uint8_t *d_present = nullptr;
    std::vector<uint8_t> present;        // host truth
    std::vector<uint8_t> present_on_dev; // last copy sent to d_present

    vb::MuonState *muon = nullptr;

    // bf16 copy of the parameter arena (vb_optimizer_enable_bf16_params), one word per element
    uint16_t *d_param_bf16 = nullptr;

    // peer GPUs' parameter arenas (f32, and bf16 copies) opened through CUDA IPC
    // (vb_optimizer_open_peers / vb_optimizer_open_peers_bf16)
    vb::PeerTable peers{};
    std::vector<void *> peer_mappings;  // what cudaIpcOpenMemHandle returned, to close on destroy

    // device-side fence around steps that touch peer memory (exchange_fence.cu): epoch of the
    // last fenced step and a mapped pinned word a fence kernel writes when a wait runs out
    uint32_t fence_epoch = 0;
    uint32_t *h_fence_error = nullptr;
    uint32_t *d_fence_error = nullptr;  // device alias of h_fence_error
    int sticky_status = 0;              // fail-stop: set once a step reported VB_ERR_TIMEOUT
};

namespace vb {

// api.cu: phase timing; no-ops unless profiling is on
void prof_begin(vb_engine *e, int phase, cudaStream_t stream = nullptr);  // stream: default the engine's
void prof_end(vb_engine *e, int phase, cudaStream_t stream = nullptr);

// muon.cu
int muon_init(vb_optimizer *opt);
int muon_step(vb_optimizer *opt, uint32_t flags);
int muon_download_update(vb_optimizer *opt, int64_t tensor, float *host, int64_t n);
int muon_last_flops(vb_optimizer *opt, double *flops);
int muon_owner(vb_optimizer *opt, int64_t tensor);
int debug_gemm_wait_expiry(vb_engine *e, uint32_t wait_limit, int *role_code);
int muon_set_keep_update(vb_optimizer *opt, int keep);
int muon_reset_velocity(vb_optimizer *opt);
int muon_debug_withhold(vb_optimizer *opt, uint32_t wait_limit);  // test hook, see vb_debug_muon_withhold_loads
int muon_check_error(vb_optimizer *opt);  // VB_ERR_TIMEOUT if a GEMM kernel reported a bounded wait expiring
float *muon_velocity_ptr(vb_optimizer *opt, int64_t tensor);  // nullptr if not owned
void plan_muon_owners(int64_t n, const int64_t *rows, const int64_t *cols, int world, int ns_mode, int ns_steps,
                      int *owner_out);
double muon_tensor_cost(int64_t rows, int64_t cols, int ns_mode, int ns_steps);  // estimated seconds per step

// comm.cpp
int comm_unique_id(void *id128);
int comm_init(vb_engine *eng, const void *id128, int rank, int world);
void comm_destroy(vb_engine *eng);
int comm_all_gather_inplace(vb_engine *eng, float *base, int64_t elems_per_rank);
int comm_all_gather_inplace_bytes(vb_engine *eng, void *base, int64_t bytes_per_rank);
int comm_barrier(vb_engine *eng);  // stream-ordered: completes once every rank's stream has reached it
struct BcastItem {
    void *ptr;
    int64_t count;  // elements of `elem_bytes` bytes (4: f32, 1: raw bytes)
    int root;
    int elem_bytes;
};
int comm_group_broadcast(vb_engine *eng, const BcastItem *items, int64_t n_items);

// What one step writes besides the local f32 parameters, from the step flags, the bf16 copy
// and the peers that are open: the table handed to the update / apply kernel, whether the
// two stream-ordered barriers are needed around it, and which copies NCCL still has to move.
struct ExchangePlan {
    PeerTable pt{};
    FenceArgs fence{};       // the flag barrier around a fused step (n_peers == 0: none needed)
    bool nccl_fence = false; // VB_EXCHANGE_FENCE=nccl: one-float all-reduces instead (for comparison)
    bool fused = false;      // the kernel stores into peers: fence it with barriers
    bool nccl_f32 = false;   // f32 parameters go by all-gather / broadcast after the kernel
    bool nccl_half = false;  // bf16 copies go by all-gather / broadcast after the kernel
};
int plan_exchange(vb_optimizer *opt, uint32_t flags, ExchangePlan *plan);
// The two halves of the barrier around a fused step; no-ops when the plan needs none.
int exchange_fence(vb_optimizer *opt, const ExchangePlan &plan, int phase);
// VB_ERR_TIMEOUT once a fence wait of this optimizer ran out on any rank (fail-stop).
int fence_check_error(vb_optimizer *opt);

inline int sync_present(vb_optimizer *opt)
{
    if (opt->present != opt->present_on_dev) {
        VB_CUDA(cudaMemcpyAsync(opt->d_present, opt->present.data(), opt->present.size(),
                                cudaMemcpyHostToDevice, opt->eng->stream));
        opt->present_on_dev = opt->present;
    }
    return VB_OK;
}

}  // namespace vb
