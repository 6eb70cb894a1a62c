// C ABI entry points (include/volta_b200.h): engine, optimizer construction, tensor
// access, step().  The arithmetic lives in multi_tensor.cu (Adam/SGD) and muon.cu.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <chrono>
#include <new>
#include <thread>

#include "engine.h"

namespace vb {

static thread_local char g_err[1024] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int engine_launch_info(vb_engine *e, int *device, int *sm_count, cudaStream_t *stream)
{
    if (!e) return fail(VB_ERR_INVALID_ARG, "engine is null");
    *device = e->device;
    *sm_count = e->sm_count;
    *stream = e->stream;
    return VB_OK;
}

void engine_count_launch(vb_engine *e) { e->launches += 1; }

constexpr int64_t kTensorAlign = 32;   // elements: every tensor starts on a 128-byte boundary
constexpr int64_t kShardAlign = 256;   // elements: every rank's slice starts on a 1 KiB boundary

static int64_t round_up(int64_t x, int64_t q) { return (x + q - 1) / q * q; }

static cudaEvent_t prof_event(vb_engine *e)
{
    cudaEvent_t ev = nullptr;
    if (!e->prof_free.empty()) {
        ev = e->prof_free.back();
        e->prof_free.pop_back();
    } else if (cudaEventCreate(&ev) != cudaSuccess) {
        return nullptr;
    }
    return ev;
}

void prof_begin(vb_engine *e, int phase, cudaStream_t stream)
{
    if (!e->profiling) return;
    cudaEvent_t ev = prof_event(e);
    if (!ev) return;
    cudaEventRecord(ev, stream ? stream : e->stream);
    e->prof_open[phase] = ev;
}

void prof_end(vb_engine *e, int phase, cudaStream_t stream)
{
    if (!e->profiling || !e->prof_open[phase]) return;
    cudaEvent_t ev = prof_event(e);
    if (!ev) return;
    cudaEventRecord(ev, stream ? stream : e->stream);
    e->prof_pairs[phase].emplace_back(e->prof_open[phase], ev);
    e->prof_open[phase] = nullptr;
}

static int check_opt(const vb_optimizer *opt)
{
    if (!opt || !opt->eng) return fail(VB_ERR_INVALID_ARG, "optimizer handle is null");
    return VB_OK;
}

static int check_tensor(const vb_optimizer *opt, int64_t tensor, int64_t n, bool check_n)
{
    VB_TRY(check_opt(opt));
    if (tensor < 0 || tensor >= opt->n_tensors)
        return fail(VB_ERR_INVALID_ARG, "tensor index %lld out of range [0, %lld)", (long long)tensor,
                    (long long)opt->n_tensors);
    if (check_n && n != opt->sizes[tensor])
        return fail(VB_ERR_INVALID_ARG, "tensor %lld has %lld elements, caller passed %lld",
                    (long long)tensor, (long long)opt->sizes[tensor], (long long)n);
    return VB_OK;
}

static int set_device(const vb_engine *e)
{
    VB_CUDA(cudaSetDevice(e->device));
    return VB_OK;
}

// ---- pure host planning (no CUDA call): arena layout, rank slices, chunk table ------------

struct Layout {
    std::vector<int64_t> offsets;
    int64_t total = 0, arena = 0, shard_begin = 0, shard_end = 0, chunk_len = 0;
    int64_t tail_begin = 0;  // [tail_begin, arena) is updated by every rank itself and never exchanged
    std::vector<ChunkDesc> chunks;
    std::vector<uint8_t> chunk_local;  // per chunk: 1 = part of the replicated tail
};

// Sharded engines: the arena positions [0, tail_begin) are cut into one slice per rank (updated by
// its owner, exchanged afterwards); with replicated_fraction > 0 the last part of the arena,
// [tail_begin, arena), is instead updated by every rank from its own copy of the gradients and
// never crosses NVLink.  The chunks of the two parts are interleaved in the table so that a launch
// mixes link-bound and HBM-bound work all along.
static void plan_layout(int64_t n_tensors, const int64_t *sizes, int world, int rank, int sm_count,
                        bool shard, double replicated_fraction, Layout *L)
{
    L->offsets.resize((size_t)n_tensors);
    int64_t off = 0;
    L->total = 0;
    for (int64_t i = 0; i < n_tensors; ++i) {
        L->offsets[(size_t)i] = off;
        off += round_up(sizes[i], kTensorAlign);
        L->total += sizes[i];
    }
    L->arena = round_up(std::max<int64_t>(off, 1), kShardAlign * world);
    L->tail_begin = L->arena;
    if (shard) {
        if (world > 1 && replicated_fraction > 0.0) {
            const double keep = replicated_fraction >= 1.0 ? 0.0 : 1.0 - replicated_fraction;
            L->tail_begin = std::min(L->arena, round_up((int64_t)((double)L->arena * keep), kShardAlign * world));
        }
        const int64_t per = L->tail_begin / world;
        L->shard_begin = per * rank;
        L->shard_end = L->shard_begin + per;
    } else {
        L->shard_begin = 0;
        L->shard_end = L->arena;
    }
    // the two owned ranges of this rank: its slice and the tail
    const int64_t range_lo[2] = {L->shard_begin, L->tail_begin};
    const int64_t range_hi[2] = {L->shard_end, L->arena};
    int64_t owned = 0;
    for (int part = 0; part < 2; ++part)
        for (int64_t i = 0; i < n_tensors; ++i) {
            const int64_t lo = std::max(L->offsets[(size_t)i], range_lo[part]);
            const int64_t hi = std::min(L->offsets[(size_t)i] + sizes[i], range_hi[part]);
            if (hi > lo) owned += hi - lo;
        }
    L->chunk_len = pick_chunk_len(owned, sm_count);
    std::vector<ChunkDesc> part_chunks[2];
    for (int part = 0; part < 2; ++part)
        for (int64_t i = 0; i < n_tensors; ++i) {
            const int64_t o = L->offsets[(size_t)i];
            const int64_t lo = std::max(o, range_lo[part]);
            const int64_t hi = std::min(o + sizes[i], range_hi[part]);
            for (int64_t b = lo; b < hi; b += L->chunk_len) {
                ChunkDesc c;
                c.offset = b - o;
                c.tensor = (uint32_t)i;
                c.len = (uint32_t)std::min(L->chunk_len, hi - b);
                part_chunks[part].push_back(c);
            }
        }
    // merge in proportion (each part keeps its order): position k of the table is a tail chunk
    // whenever the tail is behind its share of the first k chunks
    const size_t n_s = part_chunks[0].size(), n_t = part_chunks[1].size();
    L->chunks.clear();
    L->chunk_local.clear();
    L->chunks.reserve(n_s + n_t);
    L->chunk_local.reserve(n_s + n_t);
    size_t i_s = 0, i_t = 0;
    while (i_s < n_s || i_t < n_t) {
        const bool take_tail = i_s == n_s || (i_t < n_t && (i_t + 1) * n_s <= (i_s + 1) * n_t);
        if (take_tail) L->chunks.push_back(part_chunks[1][i_t++]);
        else L->chunks.push_back(part_chunks[0][i_s++]);
        L->chunk_local.push_back(take_tail ? 1 : 0);
    }
}

// Allocates the arenas of an optimizer from its layout.
static int build_arena(vb_optimizer *opt, int n_state_buffers, bool shard_states, Layout *L)
{
    vb_engine *e = opt->eng;
    VB_TRY(set_device(e));
    plan_layout(opt->n_tensors, opt->sizes.data(), e->world, e->rank, e->sm_count, shard_states,
                shard_states ? e->replicated_fraction : 0.0, L);
    opt->offsets = L->offsets;
    opt->total = L->total;
    opt->arena = L->arena;
    opt->shard_begin = L->shard_begin;
    opt->shard_end = L->shard_end;
    opt->tail_begin = L->tail_begin;
    // each arena a peer can map ends with the flag block of the exchange fence (vb_internal.h)
    const size_t arena_bytes = (size_t)opt->arena * sizeof(float) + kSyncWords * sizeof(uint32_t);
    VB_CUDA(cudaMalloc(&opt->d_param, arena_bytes));
    VB_CUDA(cudaMalloc(&opt->d_grad, arena_bytes));
    VB_CUDA(cudaMemsetAsync(opt->d_param, 0, arena_bytes, e->stream));
    VB_CUDA(cudaMemsetAsync(opt->d_grad, 0, arena_bytes, e->stream));
    VB_CUDA(cudaHostAlloc((void **)&opt->h_fence_error, sizeof(uint32_t), cudaHostAllocMapped));
    *opt->h_fence_error = 0;
    VB_CUDA(cudaHostGetDevicePointer((void **)&opt->d_fence_error, opt->h_fence_error, 0));
    // state: this rank's slice, then the replicated tail
    opt->state_elems = (opt->shard_end - opt->shard_begin) + (opt->arena - opt->tail_begin);
    const size_t state_bytes = (size_t)std::max<int64_t>(opt->state_elems, 1) * sizeof(float);
    if (n_state_buffers >= 1) {  // Storage::new_zeros, adam.rs:26-47 / sgd.rs:30-41
        VB_CUDA(cudaMalloc(&opt->d_s1, state_bytes));
        VB_CUDA(cudaMemsetAsync(opt->d_s1, 0, state_bytes, e->stream));
    }
    if (n_state_buffers >= 2) {
        VB_CUDA(cudaMalloc(&opt->d_s2, state_bytes));
        VB_CUDA(cudaMemsetAsync(opt->d_s2, 0, state_bytes, e->stream));
    }
    opt->present.assign((size_t)std::max<int64_t>(opt->n_tensors, 1), 0);
    opt->present_on_dev = opt->present;
    VB_CUDA(cudaMalloc(&opt->d_present, opt->present.size()));
    VB_CUDA(cudaMemsetAsync(opt->d_present, 0, opt->present.size(), e->stream));
    return VB_OK;
}

static int build_chunk_table(vb_optimizer *opt, const Layout &L)
{
    vb_engine *e = opt->eng;
    std::vector<FatChunk> fat(L.chunks.size());
    for (size_t c = 0; c < L.chunks.size(); ++c) {
        const ChunkDesc &ch = L.chunks[c];
        const int64_t pos = opt->offsets[ch.tensor] + ch.offset;  // arena element of the chunk start
        FatChunk &f = fat[c];
        f.p = opt->d_param + pos;
        f.g = opt->d_grad + pos;
        // state arrays cover only what this rank updates: its slice, then the replicated tail
        f.s1 = opt->d_s1 ? opt->d_s1 + opt->state_pos(pos) : nullptr;
        f.s2 = opt->d_s2 ? opt->d_s2 + opt->state_pos(pos) : nullptr;
        f.len = ch.len;
        f.tensor = ch.tensor;
        f.local_only = L.chunk_local[c];
    }
    opt->n_chunks = (int64_t)fat.size();
    opt->chunk_pos.resize(L.chunks.size());
    for (size_t c = 0; c < L.chunks.size(); ++c) opt->chunk_pos[c] = opt->offsets[L.chunks[c].tensor] + L.chunks[c].offset;
    if (!fat.empty()) {
        VB_CUDA(cudaMalloc(&opt->d_chunks, fat.size() * sizeof(FatChunk)));
        VB_CUDA(cudaMemcpyAsync(opt->d_chunks, fat.data(), fat.size() * sizeof(FatChunk),
                                cudaMemcpyHostToDevice, e->stream));
    }
    VB_CUDA(cudaStreamSynchronize(e->stream));  // the host vector goes out of scope
    return VB_OK;
}

static int validate_sizes(int64_t n_tensors, const int64_t *sizes)
{
    if (n_tensors < 0) return fail(VB_ERR_INVALID_ARG, "n_tensors is negative");
    if (n_tensors > 0 && !sizes) return fail(VB_ERR_INVALID_ARG, "sizes is null");
    if (n_tensors > (int64_t)1 << 30) return fail(VB_ERR_INVALID_ARG, "too many tensors");
    for (int64_t i = 0; i < n_tensors; ++i) {
        if (sizes[i] < 0) return fail(VB_ERR_INVALID_ARG, "sizes[%lld] is negative", (long long)i);
        // a chunk's offset/len and Volta's own cap (1e8 elements, src/tensor.rs:125-129)
        if (sizes[i] > ((int64_t)1 << 40))
            return fail(VB_ERR_INVALID_ARG, "sizes[%lld] is too large", (long long)i);
    }
    return VB_OK;
}

static void free_optimizer(vb_optimizer *opt)
{
    if (!opt) return;
    if (opt->eng) {
        cudaSetDevice(opt->eng->device);
        auto &list = opt->eng->optimizers;
        list.erase(std::remove(list.begin(), list.end(), opt), list.end());
    }
    if (opt->muon) destroy_muon_state(opt->muon);
    for (void *m : opt->peer_mappings) cudaIpcCloseMemHandle(m);
    cudaFree(opt->d_param);
    cudaFree(opt->d_param_bf16);
    cudaFree(opt->d_grad);
    cudaFree(opt->d_s1);
    cudaFree(opt->d_s2);
    cudaFree(opt->d_chunks);
    cudaFree(opt->d_present);
    if (opt->h_fence_error) cudaFreeHost(opt->h_fence_error);
    delete opt;
}

static int create_elementwise(vb_engine *engine, int kind, int64_t n_tensors, const int64_t *sizes,
                              int n_states, vb_optimizer **out, vb_optimizer **tmp)
{
    if (!engine) return fail(VB_ERR_INVALID_ARG, "engine is null");
    if (!out) return fail(VB_ERR_INVALID_ARG, "out is null");
    *out = nullptr;
    VB_TRY(validate_sizes(n_tensors, sizes));
    vb_optimizer *opt = new (std::nothrow) vb_optimizer();
    if (!opt) return fail(VB_ERR_STATE, "out of host memory");
    *tmp = opt;
    opt->eng = engine;
    opt->kind = kind;
    opt->n_tensors = n_tensors;
    opt->sizes.assign(sizes, sizes + n_tensors);
    Layout L;
    VB_TRY(build_arena(opt, n_states, /*shard_states=*/true, &L));
    VB_TRY(build_chunk_table(opt, L));
    return VB_OK;
}


int check_caller_buffers(const vb_optimizer_step_params *hp, int64_t n_tensors, const int64_t *sizes,
                         void *const *params, const void *const *grads, void *const *state1, void *const *state2,
                         int64_t *total)
{
    *total = 0;
    if (hp->op > 2u) return fail(VB_ERR_INVALID_ARG, "op %u is not 0 (SGD), 1 (SGD+momentum) or 2 (Adam)", hp->op);
    VB_TRY(validate_sizes(n_tensors, sizes));
    if (n_tensors == 0) return VB_OK;
    if (!params || !grads) return fail(VB_ERR_INVALID_ARG, "params/grads is null");
    if (hp->op >= 1 && !state1) return fail(VB_ERR_INVALID_ARG, "state1 is null for op %u", hp->op);
    if (hp->op == 2 && !state2) return fail(VB_ERR_INVALID_ARG, "state2 is null for Adam");
    if (hp->op == 2 && !(hp->t >= 1.0f && hp->t <= 2147483648.0f))
        return fail(VB_ERR_INVALID_ARG, "Adam needs t >= 1");
    for (int64_t i = 0; i < n_tensors; ++i) {
        if (sizes[i] == 0) continue;
        if (!params[i] || !grads[i])
            return fail(VB_ERR_INVALID_ARG, "params[%lld] or grads[%lld] is null", (long long)i, (long long)i);
        if (hp->op >= 1 && !state1[i]) return fail(VB_ERR_INVALID_ARG, "state1[%lld] is null", (long long)i);
        if (hp->op == 2 && !state2[i]) return fail(VB_ERR_INVALID_ARG, "state2[%lld] is null", (long long)i);
        // every array the kernel's scalar path touches must hold aligned f32 values
        uintptr_t bits = (uintptr_t)params[i] | (uintptr_t)grads[i];
        if (hp->op >= 1) bits |= (uintptr_t)state1[i];
        if (hp->op == 2) bits |= (uintptr_t)state2[i];
        if (bits & 3u)
            return fail(VB_ERR_INVALID_ARG, "tensor %lld: params, grads and state pointers must be 4-byte aligned",
                        (long long)i);
        *total += sizes[i];
    }
    return VB_OK;
}

static uint64_t fnv1a(uint64_t h, const void *data, size_t n)
{
    const unsigned char *p = static_cast<const unsigned char *>(data);
    for (size_t i = 0; i < n; ++i) h = (h ^ p[i]) * 0x100000001b3ull;
    return h;
}

int check_caller_memory(vb_engine *e, const vb_optimizer_step_params *hp, int64_t n_tensors, const int64_t *sizes,
                        void *const *params, const void *const *grads, void *const *state1, void *const *state2)
{
    uint64_t h = 0xcbf29ce484222325ull;
    h = fnv1a(h, &hp->op, sizeof(hp->op));
    h = fnv1a(h, sizes, (size_t)n_tensors * sizeof(int64_t));
    h = fnv1a(h, params, (size_t)n_tensors * sizeof(void *));
    h = fnv1a(h, grads, (size_t)n_tensors * sizeof(void *));
    if (hp->op >= 1) h = fnv1a(h, state1, (size_t)n_tensors * sizeof(void *));
    if (hp->op == 2) h = fnv1a(h, state2, (size_t)n_tensors * sizeof(void *));
    if (h == 0) h = 1;
    for (uint64_t seen : e->checked_sets)
        if (seen == h) return VB_OK;
    const void *const *arrays[4] = {(const void *const *)params, grads, hp->op >= 1 ? (const void *const *)state1 : nullptr,
                                    hp->op == 2 ? (const void *const *)state2 : nullptr};
    const char *names[4] = {"params", "grads", "state1", "state2"};
    for (int a = 0; a < 4; ++a) {
        if (!arrays[a]) continue;
        for (int64_t i = 0; i < n_tensors; ++i) {
            if (sizes[i] == 0) continue;
            cudaPointerAttributes attr;
            const cudaError_t err = cudaPointerGetAttributes(&attr, arrays[a][i]);
            if (err != cudaSuccess) {
                cudaGetLastError();
                return fail(VB_ERR_INVALID_ARG, "%s[%lld] is not a pointer CUDA knows: %s", names[a], (long long)i,
                            cudaGetErrorString(err));
            }
            if (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)
                return fail(VB_ERR_INVALID_ARG, "%s[%lld] is not device memory", names[a], (long long)i);
            if (attr.type == cudaMemoryTypeDevice && attr.device != e->device)
                return fail(VB_ERR_INVALID_ARG, "%s[%lld] lives on device %d, the engine runs on device %d", names[a],
                            (long long)i, attr.device, e->device);
        }
    }
    e->checked_sets[e->checked_next] = h;
    e->checked_next = (e->checked_next + 1) & 3;
    return VB_OK;
}
}  // namespace vb

using namespace vb;

#define VB_API_BEGIN try {
#define VB_API_END                                                         \
    }                                                                      \
    catch (const std::bad_alloc &) { return fail(VB_ERR_STATE, "out of host memory"); } \
    catch (const std::exception &ex) { return fail(VB_ERR_STATE, "exception: %s", ex.what()); } \
    catch (...) { return fail(VB_ERR_STATE, "unknown exception"); }

namespace vb {

int plan_exchange(vb_optimizer *opt, uint32_t flags, ExchangePlan *plan)
{
    vb_engine *e = opt->eng;
    if (flags & ~(VB_STEP_NO_EXCHANGE | VB_STEP_EXCHANGE_BF16 | VB_STEP_REDUCE_GRADS | VB_STEP_MEAN_GRADS))
        return fail(VB_ERR_INVALID_ARG, "unknown step flags 0x%x", flags);
    const bool half = opt->d_param_bf16 != nullptr;
    const bool half_only = (flags & VB_STEP_EXCHANGE_BF16) != 0;
    if (half_only && !half)
        return fail(VB_ERR_STATE, "VB_STEP_EXCHANGE_BF16 needs vb_optimizer_enable_bf16_params first");
    ExchangePlan xp;
    xp.pt.local_base = opt->d_param;
    xp.pt.half_local = opt->d_param_bf16;
    const bool exchange = e->world > 1 && !(flags & VB_STEP_NO_EXCHANGE);
    if (exchange) {
        if (!half_only) {
            if (opt->peers.n > 0) {
                xp.pt.n = opt->peers.n;
                for (int r = 0; r < opt->peers.n; ++r) xp.pt.base[r] = opt->peers.base[r];
            } else {
                xp.nccl_f32 = true;
            }
        }
        if (half) {
            if (opt->peers.n_half > 0) {
                xp.pt.n_half = opt->peers.n_half;
                for (int r = 0; r < opt->peers.n_half; ++r) xp.pt.half_base[r] = opt->peers.half_base[r];
            } else {
                xp.nccl_half = true;
            }
        }
        xp.fused = xp.pt.n > 0 || xp.pt.n_half > 0;
    }
    if (flags & (VB_STEP_REDUCE_GRADS | VB_STEP_MEAN_GRADS)) {
        if (e->world > 1) {
            if (opt->peers.n_grad != e->world - 1)
                return fail(VB_ERR_STATE, "VB_STEP_REDUCE_GRADS needs vb_optimizer_open_peers_grads first");
            xp.pt.n_grad = opt->peers.n_grad;
            for (int r = 0; r < opt->peers.n_grad; ++r) xp.pt.grad_base[r] = opt->peers.grad_base[r];
            xp.fused = true;  // peers' gradients are read: fence the step on both sides
        }
        xp.pt.rank = e->rank;
    }
    xp.pt.grad_scale = (flags & VB_STEP_MEAN_GRADS) ? 1.0f / (float)e->world : 1.0f;
    if (xp.fused) {
        // The flag blocks sit behind whichever arena every rank has opened on every other rank:
        // parameters first, then the bf16 copies, then the gradients (all ranks open the same set).
        FenceArgs &f = xp.fence;
        const size_t arena = (size_t)opt->arena;
        if (xp.pt.n > 0) {
            f.local = reinterpret_cast<uint32_t *>(opt->d_param + arena);
            f.n_peers = xp.pt.n;
            for (int r = 0; r < f.n_peers; ++r) f.peer[r] = reinterpret_cast<uint32_t *>(xp.pt.base[r] + arena);
        } else if (xp.pt.n_half > 0) {
            f.local = reinterpret_cast<uint32_t *>(opt->d_param_bf16 + arena);
            f.n_peers = xp.pt.n_half;
            for (int r = 0; r < f.n_peers; ++r) f.peer[r] = reinterpret_cast<uint32_t *>(xp.pt.half_base[r] + arena);
        } else {
            f.local = reinterpret_cast<uint32_t *>(opt->d_grad + arena);
            f.n_peers = xp.pt.n_grad;
            for (int r = 0; r < f.n_peers; ++r)
                f.peer[r] = reinterpret_cast<uint32_t *>(const_cast<float *>(xp.pt.grad_base[r]) + arena);
        }
        f.host_error = opt->d_fence_error;
        xp.pt.fence_error = f.local + kSyncError;
        f.rank = e->rank;
        f.wait_ns = (uint64_t)e->wait_limit_ms * 1000000ull;
        static const bool nccl_fence = [] {
            const char *v = getenv("VB_EXCHANGE_FENCE");
            return v && strcmp(v, "nccl") == 0;
        }();
        xp.nccl_fence = nccl_fence;
    }
    *plan = xp;
    return VB_OK;
}

int exchange_fence(vb_optimizer *opt, const ExchangePlan &plan, int phase)
{
    if (!plan.fused) return VB_OK;
    vb_engine *e = opt->eng;
    prof_begin(e, VB_PHASE_EXCHANGE);
    int st;
    if (plan.nccl_fence) {
        st = comm_barrier(e);
    } else {
        FenceArgs f = plan.fence;
        if (phase == 1) opt->fence_epoch += 1;  // both halves of a step carry the same epoch
        f.epoch = opt->fence_epoch;
        st = launch_exchange_fence(f, phase, e->stream);
        e->launches += 1;
    }
    prof_end(e, VB_PHASE_EXCHANGE);
    return st;
}

int fence_check_error(vb_optimizer *opt)
{
    if (opt->sticky_status != 0)
        return fail(opt->sticky_status, "an earlier step of this optimizer timed out; it is fail-stop (destroy it)");
    if (opt->h_fence_error && *reinterpret_cast<volatile uint32_t *>(opt->h_fence_error) != 0) {
        const unsigned code = *reinterpret_cast<volatile uint32_t *>(opt->h_fence_error);
        opt->sticky_status = VB_ERR_TIMEOUT;
        return fail(VB_ERR_TIMEOUT,
                    "a rank did not reach the %s of a sharded step within %u ms: the optimizer is fail-stop on every "
                    "rank", code == 1 ? "start" : "end", opt->eng->wait_limit_ms);
    }
    return VB_OK;
}

}  // namespace vb

extern "C" {

int vb_abi_version(void) { return 1002; }

const char *vb_last_error(void) { return g_err; }

int vb_device_count(int *count)
{
    if (!count) return fail(VB_ERR_INVALID_ARG, "count is null");
    *count = 0;
    VB_CUDA(cudaGetDeviceCount(count));
    return VB_OK;
}

int vb_plan_layout(int64_t n_tensors, const int64_t *sizes, int world_size, int rank, int sm_count,
                   int64_t *offsets_out, int64_t *arena_elements, int64_t *shard_begin, int64_t *shard_end,
                   int64_t *n_chunks, int64_t chunk_capacity, int64_t *chunk_tensor, int64_t *chunk_offset,
                   int64_t *chunk_len)
{
    return vb_plan_layout_replicated(n_tensors, sizes, world_size, rank, sm_count, 0.0, offsets_out, arena_elements,
                                     shard_begin, shard_end, nullptr, n_chunks, chunk_capacity, chunk_tensor,
                                     chunk_offset, chunk_len, nullptr);
}

int vb_plan_layout_replicated(int64_t n_tensors, const int64_t *sizes, int world_size, int rank, int sm_count,
                              double replicated_fraction, int64_t *offsets_out, int64_t *arena_elements,
                              int64_t *shard_begin, int64_t *shard_end, int64_t *tail_begin, int64_t *n_chunks,
                              int64_t chunk_capacity, int64_t *chunk_tensor, int64_t *chunk_offset,
                              int64_t *chunk_len, int32_t *chunk_local_only)
{
    VB_API_BEGIN
    VB_TRY(validate_sizes(n_tensors, sizes));
    if (world_size < 1 || rank < 0 || rank >= world_size || sm_count < 1)
        return fail(VB_ERR_INVALID_ARG, "rank %d / world_size %d / sm_count %d is not valid", rank, world_size,
                    sm_count);
    if (!(replicated_fraction >= 0.0 && replicated_fraction <= 1.0))
        return fail(VB_ERR_INVALID_ARG, "the replicated fraction must be in [0, 1]");
    Layout L;
    plan_layout(n_tensors, sizes, world_size, rank, sm_count, true, replicated_fraction, &L);
    if (tail_begin) *tail_begin = L.tail_begin;
    if (offsets_out)
        for (int64_t i = 0; i < n_tensors; ++i) offsets_out[i] = L.offsets[(size_t)i];
    if (arena_elements) *arena_elements = L.arena;
    if (shard_begin) *shard_begin = L.shard_begin;
    if (shard_end) *shard_end = L.shard_end;
    if (n_chunks) *n_chunks = (int64_t)L.chunks.size();
    if (chunk_tensor || chunk_offset || chunk_len || chunk_local_only) {
        if (chunk_capacity < (int64_t)L.chunks.size())
            return fail(VB_ERR_INVALID_ARG, "chunk_capacity %lld is less than the %lld chunks of the plan",
                        (long long)chunk_capacity, (long long)L.chunks.size());
        for (size_t c = 0; c < L.chunks.size(); ++c) {
            if (chunk_tensor) chunk_tensor[c] = L.chunks[c].tensor;
            if (chunk_offset) chunk_offset[c] = L.chunks[c].offset;
            if (chunk_len) chunk_len[c] = L.chunks[c].len;
            if (chunk_local_only) chunk_local_only[c] = L.chunk_local[c];
        }
    }
    return VB_OK;
    VB_API_END
}

int vb_plan_muon_owners(int64_t n_tensors, const int64_t *rows, const int64_t *cols, int world_size, int ns_mode,
                        int ns_steps, int32_t *owner_out, double *rank_cost_out)
{
    VB_API_BEGIN
    if (n_tensors < 0 || world_size < 1) return fail(VB_ERR_INVALID_ARG, "n_tensors or world_size is not valid");
    if (n_tensors > 0 && (!rows || !cols || !owner_out)) return fail(VB_ERR_INVALID_ARG, "null argument");
    if (ns_mode != VB_NS_F32 && ns_mode != VB_NS_BF16 && ns_mode != VB_NS_F32_TC)
        return fail(VB_ERR_INVALID_ARG, "unknown ns_mode %d", ns_mode);
    std::vector<int> owners((size_t)n_tensors);
    plan_muon_owners(n_tensors, rows, cols, world_size, ns_mode, ns_steps, owners.data());
    if (rank_cost_out)
        for (int r = 0; r < world_size; ++r) rank_cost_out[r] = 0.0;
    for (int64_t i = 0; i < n_tensors; ++i) {
        owner_out[i] = owners[(size_t)i];
        if (rank_cost_out) rank_cost_out[owners[(size_t)i]] += muon_tensor_cost(rows[i], cols[i], ns_mode, ns_steps);
    }
    return VB_OK;
    VB_API_END
}

// ---- plan fingerprints: do all ranks describe the same optimizer? -----------------------------

static uint64_t plan_hash(int kind, int64_t n, const int64_t *a, const int64_t *b, const float *hyper, int n_hyper,
                          const int32_t *ints, int n_ints, int world)
{
    uint64_t h = 0xcbf29ce484222325ull;
    const int32_t head[3] = {vb_abi_version(), kind, world};
    h = fnv1a(h, head, sizeof(head));
    h = fnv1a(h, &n, sizeof(n));
    if (a) h = fnv1a(h, a, (size_t)n * sizeof(int64_t));
    if (b) h = fnv1a(h, b, (size_t)n * sizeof(int64_t));
    if (hyper) h = fnv1a(h, hyper, (size_t)n_hyper * sizeof(float));
    if (ints) h = fnv1a(h, ints, (size_t)n_ints * sizeof(int32_t));
    return h;
}

int vb_plan_fingerprint(int kind, int64_t n_tensors, const int64_t *sizes_or_rows, const int64_t *cols,
                        const float *hyper, int n_hyper, const int32_t *ints, int n_ints, int world_size,
                        uint64_t *fingerprint)
{
    if (!fingerprint) return fail(VB_ERR_INVALID_ARG, "fingerprint is null");
    if (n_tensors < 0 || (n_tensors > 0 && !sizes_or_rows) || n_hyper < 0 || n_ints < 0 || (n_hyper > 0 && !hyper) ||
        (n_ints > 0 && !ints) || world_size < 1)
        return fail(VB_ERR_INVALID_ARG, "invalid argument");
    *fingerprint = plan_hash(kind, n_tensors, sizes_or_rows, cols, hyper, n_hyper, ints, n_ints, world_size);
    return VB_OK;
}

int vb_optimizer_plan_fingerprint(vb_optimizer *opt, uint64_t *fingerprint)
{
    VB_TRY(check_opt(opt));
    if (!fingerprint) return fail(VB_ERR_INVALID_ARG, "fingerprint is null");
    const float hyper[6] = {opt->lr, opt->beta1, opt->beta2, opt->eps, opt->weight_decay, opt->momentum};
    // a replicated tail is part of the plan: ranks that cut the arena differently must not step together
    const bool tail = opt->kind != KIND_MUON && opt->tail_begin < opt->arena;
    const int32_t ints[6] = {opt->nesterov, opt->ns_steps, opt->ns_mode, opt->d_param_bf16 ? 1 : 0,
                             (int32_t)(opt->tail_begin & 0x7fffffff), (int32_t)(opt->tail_begin >> 31)};
    const bool muon = opt->kind == KIND_MUON;
    *fingerprint = plan_hash(opt->kind, opt->n_tensors, muon ? opt->rows.data() : opt->sizes.data(),
                             muon ? opt->cols.data() : nullptr, hyper, 6, ints, tail ? 6 : 4, opt->eng->world);
    return VB_OK;
}

int vb_plan_fingerprints_agree(const uint64_t *fingerprints, int n_ranks, int *first_mismatch)
{
    if (!fingerprints || n_ranks < 1) return fail(VB_ERR_INVALID_ARG, "invalid argument");
    if (first_mismatch) *first_mismatch = -1;
    for (int r = 1; r < n_ranks; ++r) {
        if (fingerprints[r] != fingerprints[0]) {
            if (first_mismatch) *first_mismatch = r;
            return fail(VB_ERR_STATE,
                        "rank %d describes a different optimizer than rank 0 (tensor list, hyper-parameters, mode or "
                        "world size): fingerprint %016llx against %016llx; no sharded step may be launched",
                        r, (unsigned long long)fingerprints[r], (unsigned long long)fingerprints[0]);
        }
    }
    return VB_OK;
}

int vb_engine_create(int device, vb_engine **out)
{
    VB_API_BEGIN
    if (!out) return fail(VB_ERR_INVALID_ARG, "out is null");
    *out = nullptr;
    int count = 0;
    VB_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count)
        return fail(VB_ERR_INVALID_ARG, "device %d out of range (%d visible)", device, count);
    VB_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    VB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(VB_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only",
                    device, prop.major, prop.minor);
    vb_engine *e = new vb_engine();
    e->device = device;
    e->sm_count = prop.multiProcessorCount;
    cudaError_t err = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking);
    if (err != cudaSuccess) {
        delete e;
        return fail(VB_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(err));
    }
    *out = e;
    return VB_OK;
    VB_API_END
}

int vb_engine_destroy(vb_engine *e)
{
    if (!e) return VB_OK;
    cudaSetDevice(e->device);
    if (e->stream) cudaStreamSynchronize(e->stream);
    comm_destroy(e);
    for (int ph = 0; ph < VB_PHASE_COUNT; ++ph) {
        for (auto &pr : e->prof_pairs[ph]) {
            cudaEventDestroy(pr.first);
            cudaEventDestroy(pr.second);
        }
        if (e->prof_open[ph]) cudaEventDestroy(e->prof_open[ph]);
    }
    for (cudaEvent_t ev : e->prof_free) cudaEventDestroy(ev);
    if (e->deadline_event) cudaEventDestroy(e->deadline_event);
    for (cudaStream_t st : e->peer_streams)
        if (st) cudaStreamDestroy(st);
    for (cudaEvent_t ev : e->peer_events)
        if (ev) cudaEventDestroy(ev);
    if (e->d_accum_scratch) cudaFree(e->d_accum_scratch);
    for (cudaEvent_t ev : e->pipe_events) cudaEventDestroy(ev);
    if (e->h2d_stream) cudaStreamDestroy(e->h2d_stream);
    if (e->d2h_stream) cudaStreamDestroy(e->d2h_stream);
    for (int i = 0; i < 2; ++i) {
        if (e->h_stage[i]) cudaFreeHost(e->h_stage[i]);
        if (e->d_stage[i]) cudaFree(e->d_stage[i]);
        if (e->stage_done[i]) cudaEventDestroy(e->stage_done[i]);
    }
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
    return VB_OK;
}

// After the stream has drained: the first error any optimizer of the engine recorded on the
// device (a fence wait or a GEMM wait that ran out).
static int engine_device_errors(vb_engine *e)
{
    for (vb_optimizer *opt : e->optimizers) {
        VB_TRY(fence_check_error(opt));
        if (opt->kind == KIND_MUON) VB_TRY(muon_check_error(opt));
    }
    return VB_OK;
}

int vb_engine_synchronize(vb_engine *e)
{
    if (!e) return fail(VB_ERR_INVALID_ARG, "engine is null");
    VB_CUDA(cudaStreamSynchronize(e->stream));
    return engine_device_errors(e);
}

int vb_engine_synchronize_deadline(vb_engine *e, double timeout_ms)
{
    VB_API_BEGIN
    if (!e) return fail(VB_ERR_INVALID_ARG, "engine is null");
    if (!(timeout_ms >= 0.0)) return fail(VB_ERR_INVALID_ARG, "timeout_ms must be >= 0");
    VB_TRY(set_device(e));
    if (!e->deadline_event) VB_CUDA(cudaEventCreateWithFlags(&e->deadline_event, cudaEventDisableTiming));
    VB_CUDA(cudaEventRecord(e->deadline_event, e->stream));
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const cudaError_t q = cudaEventQuery(e->deadline_event);
        if (q == cudaSuccess) break;
        if (q != cudaErrorNotReady)
            return fail(VB_ERR_CUDA, "cudaEventQuery failed: %s (%d)", cudaGetErrorString(q), (int)q);
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        if (ms > timeout_ms)
            return fail(VB_ERR_TIMEOUT, "the engine's stream did not drain within %.3f ms (work is still queued; the "
                                        "engine stays usable and a later synchronize can wait for it)", timeout_ms);
        std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
    return engine_device_errors(e);
    VB_API_END
}

int vb_engine_set_wait_limit_ms(vb_engine *e, uint32_t ms)
{
    if (!e) return fail(VB_ERR_INVALID_ARG, "engine is null");
    if (ms == 0) return fail(VB_ERR_INVALID_ARG, "the wait limit must be at least 1 ms");
    e->wait_limit_ms = ms;
    return VB_OK;
}

int vb_engine_set_replicated_fraction(vb_engine *e, double fraction)
{
    if (!e) return fail(VB_ERR_INVALID_ARG, "engine is null");
    if (!(fraction >= 0.0 && fraction <= 1.0)) return fail(VB_ERR_INVALID_ARG, "the replicated fraction must be in [0, 1]");
    e->replicated_fraction = fraction;
    return VB_OK;
}

int vb_plan_replicated_fraction(double bytes_per_element, int world_size, double hbm_gb_per_s, double link_gb_per_s,
                                double *fraction)
{
    if (!fraction) return fail(VB_ERR_INVALID_ARG, "fraction is null");
    if (!(bytes_per_element > 0.0) || world_size < 1 || !(hbm_gb_per_s > 0.0) || !(link_gb_per_s > 0.0))
        return fail(VB_ERR_INVALID_ARG, "bytes_per_element, world_size and both rates must be positive");
    *fraction = 0.0;
    if (world_size == 1) return VB_OK;
    // per arena element: t_local = time to update it here, t_link = time its 4 bytes take into every GPU
    // when everything is exchanged.  With a fraction f replicated the launch moves
    //     HBM:  t_local * ((1 - f) / N + f)        NVLink:  t_link * (1 - f)
    // at the same time; the two are equal at the fraction returned.
    const double n = (double)world_size;
    const double t_local = bytes_per_element / hbm_gb_per_s;
    const double t_link = 4.0 * (n - 1.0) / n / link_gb_per_s;
    const double exchanged = t_local / (t_link + t_local * (1.0 - 1.0 / n));
    *fraction = exchanged >= 1.0 ? 0.0 : 1.0 - exchanged;
    return VB_OK;
}

int vb_engine_stream(vb_engine *e, void **cuda_stream)
{
    if (!e || !cuda_stream) return fail(VB_ERR_INVALID_ARG, "null argument");
    *cuda_stream = (void *)e->stream;
    return VB_OK;
}

int vb_engine_launch_count(vb_engine *e, uint64_t *count)
{
    if (!e || !count) return fail(VB_ERR_INVALID_ARG, "null argument");
    *count = e->launches;
    return VB_OK;
}

int vb_engine_set_profiling(vb_engine *e, int enabled)
{
    if (!e) return fail(VB_ERR_INVALID_ARG, "engine is null");
    e->profiling = enabled != 0;
    return VB_OK;
}

int vb_engine_profile(vb_engine *e, int phase, double *total_ms, int64_t *count)
{
    VB_API_BEGIN
    if (!e || !total_ms || !count) return fail(VB_ERR_INVALID_ARG, "null argument");
    if (phase < 0 || phase >= VB_PHASE_COUNT) return fail(VB_ERR_INVALID_ARG, "unknown phase %d", phase);
    VB_CUDA(cudaSetDevice(e->device));
    VB_CUDA(cudaStreamSynchronize(e->stream));
    if (e->h2d_stream) VB_CUDA(cudaStreamSynchronize(e->h2d_stream));
    if (e->d2h_stream) VB_CUDA(cudaStreamSynchronize(e->d2h_stream));
    double total = 0.0;
    for (auto &pr : e->prof_pairs[phase]) {
        float ms = 0.0f;
        VB_CUDA(cudaEventElapsedTime(&ms, pr.first, pr.second));
        total += ms;
        e->prof_free.push_back(pr.first);
        e->prof_free.push_back(pr.second);
    }
    *total_ms = total;
    *count = (int64_t)e->prof_pairs[phase].size();
    e->prof_pairs[phase].clear();
    return VB_OK;
    VB_API_END
}

int vb_debug_gemm_wait_expiry(vb_engine *e, uint32_t wait_limit, int *role_code)
{
    VB_API_BEGIN
    if (!e) return fail(VB_ERR_INVALID_ARG, "engine is null");
    if (role_code) *role_code = 0;
    VB_TRY(set_device(e));
    return debug_gemm_wait_expiry(e, wait_limit, role_code);
    VB_API_END
}

int vb_debug_muon_withhold_loads(vb_optimizer *opt, uint32_t wait_limit)
{
    VB_TRY(check_opt(opt));
    if (opt->kind != KIND_MUON) return fail(VB_ERR_INVALID_ARG, "not a Muon optimizer");
    return muon_debug_withhold(opt, wait_limit);
}

int vb_debug_fence_wait_expiry(vb_engine *e, uint32_t timeout_ms, int phase, int *code)
{
    VB_API_BEGIN
    if (!e) return fail(VB_ERR_INVALID_ARG, "engine is null");
    if (phase != 1 && phase != 2) return fail(VB_ERR_INVALID_ARG, "phase must be 1 or 2");
    if (code) *code = 0;
    VB_TRY(set_device(e));
    // two flag blocks in this GPU's own memory: "this rank" and a peer that never shows up
    uint32_t *blocks = nullptr, *h_err = nullptr, *d_err = nullptr;
    VB_CUDA(cudaMalloc((void **)&blocks, 2 * kSyncWords * sizeof(uint32_t)));
    cudaError_t err = cudaMemsetAsync(blocks, 0, 2 * kSyncWords * sizeof(uint32_t), e->stream);
    if (err == cudaSuccess) err = cudaHostAlloc((void **)&h_err, sizeof(uint32_t), cudaHostAllocMapped);
    if (err == cudaSuccess) {
        *h_err = 0;
        err = cudaHostGetDevicePointer((void **)&d_err, h_err, 0);
    }
    int st = VB_OK;
    if (err == cudaSuccess) {
        FenceArgs f{};
        f.local = blocks;
        f.peer[0] = blocks + kSyncWords;
        f.host_error = d_err;
        f.n_peers = 1;
        f.rank = 0;
        f.epoch = 1;
        f.wait_ns = (uint64_t)(timeout_ms ? timeout_ms : 1u) * 1000000ull;
        st = launch_exchange_fence(f, phase, e->stream);
        if (st == VB_OK) err = cudaStreamSynchronize(e->stream);
    }
    const uint32_t got = (err == cudaSuccess && h_err) ? *reinterpret_cast<volatile uint32_t *>(h_err) : 0u;
    cudaFree(blocks);
    if (h_err) cudaFreeHost(h_err);
    if (err != cudaSuccess) return fail(VB_ERR_CUDA, "fence self-test: %s", cudaGetErrorString(err));
    if (st != VB_OK) return st;
    if (code) *code = (int)got;
    if (got != 0)
        return fail(VB_ERR_TIMEOUT, "the exchange fence gave up waiting for a peer in phase %u after %u ms", got,
                    timeout_ms);
    return VB_OK;
    VB_API_END
}

int vb_comm_unique_id(void *id128)
{
    VB_API_BEGIN
    if (!id128) return fail(VB_ERR_INVALID_ARG, "id128 is null");
    return comm_unique_id(id128);
    VB_API_END
}

int vb_engine_comm_init(vb_engine *e, const void *id128, int rank, int world_size)
{
    VB_API_BEGIN
    if (!e || !id128) return fail(VB_ERR_INVALID_ARG, "null argument");
    if (world_size < 1 || rank < 0 || rank >= world_size)
        return fail(VB_ERR_INVALID_ARG, "rank %d / world_size %d is not valid", rank, world_size);
    if (e->comm) return fail(VB_ERR_STATE, "engine already has a communicator");
    VB_TRY(set_device(e));
    return comm_init(e, id128, rank, world_size);
    VB_API_END
}

int vb_engine_rank(vb_engine *e, int *rank, int *world_size)
{
    if (!e) return fail(VB_ERR_INVALID_ARG, "engine is null");
    if (rank) *rank = e->rank;
    if (world_size) *world_size = e->world;
    return VB_OK;
}

int vb_host_alloc_pinned(void **ptr, size_t bytes)
{
    if (!ptr) return fail(VB_ERR_INVALID_ARG, "ptr is null");
    *ptr = nullptr;
    VB_CUDA(cudaHostAlloc(ptr, bytes ? bytes : 1, cudaHostAllocDefault));
    return VB_OK;
}

int vb_host_free_pinned(void *ptr)
{
    if (ptr) VB_CUDA(cudaFreeHost(ptr));
    return VB_OK;
}

int vb_adam_create(vb_engine *engine, int64_t n_tensors, const int64_t *sizes, float lr, float beta1,
                   float beta2, float eps, float weight_decay, vb_optimizer **out)
{
    VB_API_BEGIN
    vb_optimizer *opt = nullptr;
    int st = create_elementwise(engine, KIND_ADAM, n_tensors, sizes, 2, out, &opt);
    if (st != VB_OK) {
        free_optimizer(opt);
        return st;
    }
    opt->lr = lr;
    opt->beta1 = beta1;
    opt->beta2 = beta2;
    opt->eps = eps;
    opt->weight_decay = weight_decay;
    engine->optimizers.push_back(opt);
    *out = opt;
    return VB_OK;
    VB_API_END
}

int vb_sgd_create(vb_engine *engine, int64_t n_tensors, const int64_t *sizes, float lr, float momentum,
                  float weight_decay, vb_optimizer **out)
{
    VB_API_BEGIN
    vb_optimizer *opt = nullptr;
    // sgd.rs:30: velocity only if momentum > 0.0
    int st = create_elementwise(engine, KIND_SGD, n_tensors, sizes, momentum > 0.0f ? 1 : 0, out, &opt);
    if (st != VB_OK) {
        free_optimizer(opt);
        return st;
    }
    opt->lr = lr;
    opt->momentum = momentum;
    opt->weight_decay = weight_decay;
    engine->optimizers.push_back(opt);
    *out = opt;
    return VB_OK;
    VB_API_END
}

int vb_muon_create(vb_engine *engine, int64_t n_tensors, const int64_t *rows, const int64_t *cols,
                   float lr, float momentum, int nesterov, int ns_steps, int ns_mode, vb_optimizer **out)
{
    VB_API_BEGIN
    if (!engine) return fail(VB_ERR_INVALID_ARG, "engine is null");
    if (!out) return fail(VB_ERR_INVALID_ARG, "out is null");
    *out = nullptr;
    if (n_tensors < 0 || (n_tensors > 0 && (!rows || !cols)))
        return fail(VB_ERR_INVALID_ARG, "rows/cols is null or n_tensors negative");
    if (ns_steps < 0) return fail(VB_ERR_INVALID_ARG, "ns_steps is negative");
    if (ns_mode != VB_NS_F32 && ns_mode != VB_NS_BF16 && ns_mode != VB_NS_F32_TC)
        return fail(VB_ERR_INVALID_ARG, "unknown ns_mode %d", ns_mode);
    std::vector<int64_t> sizes((size_t)n_tensors);
    for (int64_t i = 0; i < n_tensors; ++i) {
        if (rows[i] < 0 || cols[i] < 0 || (cols[i] > 0 && rows[i] > ((int64_t)1 << 40) / cols[i]))
            return fail(VB_ERR_INVALID_ARG, "rows/cols of tensor %lld are not valid", (long long)i);
        sizes[(size_t)i] = rows[i] * cols[i];
    }
    vb_optimizer *opt = new vb_optimizer();
    opt->eng = engine;
    opt->kind = KIND_MUON;
    opt->n_tensors = n_tensors;
    opt->sizes = sizes;
    opt->rows.assign(rows, rows + n_tensors);
    opt->cols.assign(cols, cols + n_tensors);
    opt->lr = lr;
    opt->momentum = momentum;
    opt->nesterov = nesterov ? 1 : 0;
    opt->ns_steps = ns_steps;
    opt->ns_mode = ns_mode;
    // Parameters and gradients are whole on every rank; velocity is allocated by
    // muon_init for the matrices this rank owns.
    Layout L;
    int st = build_arena(opt, 0, /*shard_states=*/false, &L);
    if (st == VB_OK) st = muon_init(opt);
    if (st != VB_OK) {
        free_optimizer(opt);
        return st;
    }
    engine->optimizers.push_back(opt);
    *out = opt;
    return VB_OK;
    VB_API_END
}

int vb_optimizer_destroy(vb_optimizer *opt)
{
    if (!opt) return VB_OK;
    if (opt->eng && opt->eng->stream) {
        cudaSetDevice(opt->eng->device);
        cudaStreamSynchronize(opt->eng->stream);
    }
    free_optimizer(opt);
    return VB_OK;
}

int vb_optimizer_num_tensors(vb_optimizer *opt, int64_t *n)
{
    VB_TRY(check_opt(opt));
    if (!n) return fail(VB_ERR_INVALID_ARG, "null argument");
    *n = opt->n_tensors;
    return VB_OK;
}

int vb_optimizer_tensor_size(vb_optimizer *opt, int64_t tensor, int64_t *n)
{
    VB_TRY(check_tensor(opt, tensor, 0, false));
    if (!n) return fail(VB_ERR_INVALID_ARG, "null argument");
    *n = opt->sizes[tensor];
    return VB_OK;
}

int vb_optimizer_total_size(vb_optimizer *opt, int64_t *n)
{
    VB_TRY(check_opt(opt));
    if (!n) return fail(VB_ERR_INVALID_ARG, "null argument");
    *n = opt->total;
    return VB_OK;
}

// Keeps the bf16 copy (if enabled) equal to the rounded f32 parameters after they were
// written by an upload: arena elements [begin, begin + n).
static int refresh_bf16(vb_optimizer *opt, int64_t begin, int64_t n)
{
    if (!opt->d_param_bf16 || n <= 0) return VB_OK;
    return launch_f32_to_bf16(opt->d_param_bf16 + begin, opt->d_param + begin, n, opt->eng->sm_count,
                              opt->eng->stream);
}

static int copy_tensor(vb_optimizer *opt, int64_t tensor, float *dev_base, void *host, int64_t n,
                       bool to_device)
{
    VB_TRY(check_tensor(opt, tensor, n, true));
    if (n > 0 && !host) return fail(VB_ERR_INVALID_ARG, "host pointer is null");
    VB_TRY(set_device(opt->eng));
    if (n == 0) return VB_OK;
    float *dev = dev_base + opt->offsets[tensor];
    if (to_device) {
        VB_CUDA(cudaMemcpyAsync(dev, host, (size_t)n * sizeof(float), cudaMemcpyHostToDevice,
                                opt->eng->stream));
        if (dev_base == opt->d_param) VB_TRY(refresh_bf16(opt, opt->offsets[tensor], n));
    } else {
        VB_CUDA(cudaMemcpyAsync(host, dev, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost,
                                opt->eng->stream));
        VB_CUDA(cudaStreamSynchronize(opt->eng->stream));
        if (opt->kind == KIND_MUON) return muon_check_error(opt);
    }
    return VB_OK;
}

int vb_optimizer_upload_params(vb_optimizer *opt, int64_t tensor, const float *host, int64_t n)
{
    VB_TRY(check_opt(opt));
    return copy_tensor(opt, tensor, opt->d_param, (void *)host, n, true);
}

int vb_optimizer_download_params(vb_optimizer *opt, int64_t tensor, float *host, int64_t n)
{
    VB_TRY(check_opt(opt));
    return copy_tensor(opt, tensor, opt->d_param, host, n, false);
}

int vb_optimizer_upload_grad(vb_optimizer *opt, int64_t tensor, const float *host, int64_t n)
{
    VB_TRY(check_opt(opt));
    VB_TRY(copy_tensor(opt, tensor, opt->d_grad, (void *)host, n, true));
    opt->present[(size_t)tensor] = 1;
    return VB_OK;
}

// `p.grad = match p.grad { None => Some(g), Some(e) => Some(e + g) }` (src/autograd.rs:140-148,158-184)
static int accumulate(vb_optimizer *opt, int64_t tensor, const float *dev_src, int64_t n)
{
    float *grad = opt->d_grad + opt->offsets[tensor];
    const bool add = opt->present[(size_t)tensor] != 0;
    VB_TRY(launch_accumulate_grad(grad, dev_src, n, add, opt->eng->sm_count, opt->eng->stream));
    opt->eng->launches += 1;
    opt->present[(size_t)tensor] = 1;
    return VB_OK;
}

int vb_optimizer_accumulate_grad_device(vb_optimizer *opt, int64_t tensor, const void *device_src, int64_t n)
{
    VB_API_BEGIN
    VB_TRY(check_tensor(opt, tensor, n, true));
    if (n > 0 && !device_src) return fail(VB_ERR_INVALID_ARG, "device_src is null");
    if (((uintptr_t)device_src & 3u) != 0) return fail(VB_ERR_INVALID_ARG, "device_src is not 4-byte aligned");
    VB_TRY(set_device(opt->eng));
    return accumulate(opt, tensor, (const float *)device_src, n);
    VB_API_END
}

int vb_optimizer_accumulate_grad(vb_optimizer *opt, int64_t tensor, const float *host, int64_t n)
{
    VB_API_BEGIN
    VB_TRY(check_tensor(opt, tensor, n, true));
    if (n > 0 && !host) return fail(VB_ERR_INVALID_ARG, "host pointer is null");
    vb_engine *e = opt->eng;
    VB_TRY(set_device(e));
    if (n == 0) {
        opt->present[(size_t)tensor] = 1;
        return VB_OK;
    }
    if (!opt->present[(size_t)tensor]) {  // first contribution: it simply becomes the gradient
        VB_CUDA(cudaMemcpyAsync(opt->d_grad + opt->offsets[tensor], host, (size_t)n * sizeof(float),
                                cudaMemcpyHostToDevice, e->stream));
        opt->present[(size_t)tensor] = 1;
        return VB_OK;
    }
    if (e->accum_scratch_elems < (size_t)n) {
        if (e->d_accum_scratch) VB_CUDA(cudaFree(e->d_accum_scratch));  // waits for earlier users
        e->d_accum_scratch = nullptr;
        e->accum_scratch_elems = 0;
        VB_CUDA(cudaMalloc(&e->d_accum_scratch, (size_t)n * sizeof(float)));
        e->accum_scratch_elems = (size_t)n;
    }
    VB_CUDA(cudaMemcpyAsync(e->d_accum_scratch, host, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, e->stream));
    return accumulate(opt, tensor, e->d_accum_scratch, n);
    VB_API_END
}

int vb_optimizer_download_grad(vb_optimizer *opt, int64_t tensor, float *host, int64_t n)
{
    VB_TRY(check_opt(opt));
    return copy_tensor(opt, tensor, opt->d_grad, host, n, false);
}

int vb_optimizer_param_ptr(vb_optimizer *opt, int64_t tensor, void **p)
{
    VB_TRY(check_tensor(opt, tensor, 0, false));
    if (!p) return fail(VB_ERR_INVALID_ARG, "null argument");
    *p = opt->d_param + opt->offsets[tensor];
    return VB_OK;
}

int vb_optimizer_grad_ptr(vb_optimizer *opt, int64_t tensor, void **p)
{
    VB_TRY(check_tensor(opt, tensor, 0, false));
    if (!p) return fail(VB_ERR_INVALID_ARG, "null argument");
    *p = opt->d_grad + opt->offsets[tensor];
    return VB_OK;
}

int vb_optimizer_arena(vb_optimizer *opt, void **param_arena, void **grad_arena, int64_t *arena_elements,
                       int64_t *offsets_out)
{
    VB_TRY(check_opt(opt));
    if (param_arena) *param_arena = opt->d_param;
    if (grad_arena) *grad_arena = opt->d_grad;
    if (arena_elements) *arena_elements = opt->arena;
    if (offsets_out)
        for (int64_t i = 0; i < opt->n_tensors; ++i) offsets_out[i] = opt->offsets[i];
    return VB_OK;
}

int vb_optimizer_upload_arena(vb_optimizer *opt, int which, const float *host, int64_t n)
{
    VB_TRY(check_opt(opt));
    if (which != 0 && which != 1) return fail(VB_ERR_INVALID_ARG, "which must be 0 (params) or 1 (grads)");
    if (n != opt->arena)
        return fail(VB_ERR_INVALID_ARG, "arena has %lld elements, caller passed %lld", (long long)opt->arena,
                    (long long)n);
    if (!host) return fail(VB_ERR_INVALID_ARG, "host pointer is null");
    VB_TRY(set_device(opt->eng));
    VB_CUDA(cudaMemcpyAsync(which == 0 ? opt->d_param : opt->d_grad, host, (size_t)n * sizeof(float),
                            cudaMemcpyHostToDevice, opt->eng->stream));
    if (which == 1) std::fill(opt->present.begin(), opt->present.end(), (uint8_t)1);
    else VB_TRY(refresh_bf16(opt, 0, n));
    return VB_OK;
}

int vb_optimizer_download_arena(vb_optimizer *opt, int which, float *host, int64_t n)
{
    VB_TRY(check_opt(opt));
    if (which != 0 && which != 1) return fail(VB_ERR_INVALID_ARG, "which must be 0 (params) or 1 (grads)");
    if (n != opt->arena)
        return fail(VB_ERR_INVALID_ARG, "arena has %lld elements, caller passed %lld", (long long)opt->arena,
                    (long long)n);
    if (!host) return fail(VB_ERR_INVALID_ARG, "host pointer is null");
    VB_TRY(set_device(opt->eng));
    VB_CUDA(cudaMemcpyAsync(host, which == 0 ? opt->d_param : opt->d_grad, (size_t)n * sizeof(float),
                            cudaMemcpyDeviceToHost, opt->eng->stream));
    VB_CUDA(cudaStreamSynchronize(opt->eng->stream));
    return VB_OK;
}

static int arena_range_copy(vb_optimizer *opt, int which, void *host, int64_t begin, int64_t n, bool to_device)
{
    VB_TRY(check_opt(opt));
    if (which != 0 && which != 1) return fail(VB_ERR_INVALID_ARG, "which must be 0 (params) or 1 (grads)");
    if (begin < 0 || n < 0 || begin + n > opt->arena)
        return fail(VB_ERR_INVALID_ARG, "range [%lld, %lld) is outside the arena of %lld elements", (long long)begin,
                    (long long)(begin + n), (long long)opt->arena);
    if (n == 0) return VB_OK;
    if (!host) return fail(VB_ERR_INVALID_ARG, "host pointer is null");
    VB_TRY(set_device(opt->eng));
    float *dev = (which == 0 ? opt->d_param : opt->d_grad) + begin;
    if (to_device) {
        VB_CUDA(cudaMemcpyAsync(dev, host, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, opt->eng->stream));
        if (which == 1) std::fill(opt->present.begin(), opt->present.end(), (uint8_t)1);
        else VB_TRY(refresh_bf16(opt, begin, n));
    } else {
        VB_CUDA(cudaMemcpyAsync(host, dev, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost, opt->eng->stream));
        VB_CUDA(cudaStreamSynchronize(opt->eng->stream));
    }
    return VB_OK;
}

int vb_optimizer_upload_arena_range(vb_optimizer *opt, int which, const float *host, int64_t begin, int64_t n)
{
    return arena_range_copy(opt, which, (void *)host, begin, n, true);
}

int vb_optimizer_download_arena_range(vb_optimizer *opt, int which, float *host, int64_t begin, int64_t n)
{
    return arena_range_copy(opt, which, host, begin, n, false);
}

int vb_optimizer_owned_range(vb_optimizer *opt, int64_t *begin, int64_t *end)
{
    VB_TRY(check_opt(opt));
    if (begin) *begin = opt->shard_begin;
    if (end) *end = opt->shard_end;
    return VB_OK;
}

int vb_optimizer_replicated_range(vb_optimizer *opt, int64_t *begin, int64_t *end)
{
    VB_TRY(check_opt(opt));
    if (begin) *begin = opt->kind == KIND_MUON ? opt->arena : opt->tail_begin;
    if (end) *end = opt->arena;
    return VB_OK;
}

int vb_optimizer_set_grad_present(vb_optimizer *opt, int64_t tensor, int present)
{
    VB_TRY(check_tensor(opt, tensor, 0, false));
    opt->present[(size_t)tensor] = present ? 1 : 0;
    return VB_OK;
}

int vb_optimizer_zero_grad(vb_optimizer *opt)
{
    VB_TRY(check_opt(opt));
    std::fill(opt->present.begin(), opt->present.end(), (uint8_t)0);
    return VB_OK;
}

int vb_optimizer_set_lr(vb_optimizer *opt, float lr)
{
    VB_TRY(check_opt(opt));
    opt->lr = lr;
    return VB_OK;
}

int vb_optimizer_step_ex(vb_optimizer *opt, uint32_t flags)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    vb_engine *e = opt->eng;
    VB_TRY(set_device(e));
    VB_TRY(fence_check_error(opt));
    if (opt->kind == KIND_MUON) return muon_step(opt, flags);

    // everything that can refuse the step comes before any state changes (a refused step must
    // not advance Adam's t: the retry would no longer match the reference)
    ExchangePlan xp;
    VB_TRY(plan_exchange(opt, flags, &xp));
    VB_TRY(sync_present(opt));
    int op;
    StepScalars s;
    if (opt->kind == KIND_ADAM) {
        opt->t += 1;  // adam.rs:71: before looking at any gradient
        op = OP_ADAM;
        s = make_scalars(op, opt->lr, opt->beta1, opt->beta2, opt->eps, opt->weight_decay, opt->t);
    } else {
        op = opt->momentum > 0.0f ? OP_SGD_MOMENTUM : OP_SGD;  // sgd.rs:207
        s = make_scalars(op, opt->lr, opt->momentum, 0.0f, 0.0f, opt->weight_decay, 0);
    }
    // With peer arenas mapped, the exchange is fused into the update: the kernel stores
    // every new parameter locally and into each peer's arena.  A flag barrier in peer-mapped
    // memory fences it on both sides: no rank is written to before it has reached its step (its
    // earlier readers of the parameters are done), and no rank continues before all writes have
    // landed.  Every rank takes part, also one whose slice holds no tensor element.
    VB_TRY(exchange_fence(opt, xp, 1));
    if (opt->n_chunks > 0) {
        bool all_present = true;
        for (int64_t i = 0; i < opt->n_tensors && all_present; ++i) all_present = opt->present[(size_t)i] != 0;
        prof_begin(e, VB_PHASE_UPDATE);
        VB_TRY(launch_multi_tensor(op, opt->d_chunks, opt->n_chunks, opt->d_present, all_present, s,
                                   e->sm_count, e->stream, &xp.pt));
        prof_end(e, VB_PHASE_UPDATE);
        e->launches += 1;
    }
    VB_TRY(exchange_fence(opt, xp, 2));
    if (xp.nccl_f32 || xp.nccl_half) {
        prof_begin(e, VB_PHASE_EXCHANGE);
        if (xp.nccl_f32) VB_TRY(comm_all_gather_inplace(e, opt->d_param, opt->tail_begin / e->world));
        if (xp.nccl_half)
            VB_TRY(comm_all_gather_inplace_bytes(e, opt->d_param_bf16, opt->tail_begin / e->world * (int64_t)sizeof(uint16_t)));
        prof_end(e, VB_PHASE_EXCHANGE);
    }
    return VB_OK;
    VB_API_END
}

int vb_optimizer_step(vb_optimizer *opt) { return vb_optimizer_step_ex(opt, VB_STEP_DEFAULT); }

int vb_optimizer_step_host(vb_optimizer *opt, const float *grads_host, float *params_host, int pieces)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    vb_engine *e = opt->eng;
    if (opt->kind == KIND_MUON) return fail(VB_ERR_UNSUPPORTED, "the pipelined host step is implemented for Adam and SGD");
    if (!grads_host || !params_host) return fail(VB_ERR_INVALID_ARG, "host arena pointer is null");
    if (opt->tail_begin < opt->arena)
        return fail(VB_ERR_UNSUPPORTED, "the pipelined host step moves one contiguous owned range: create the optimizer "
                                        "with no replicated part (vb_engine_set_replicated_fraction 0)");
    if (pieces < 1) pieces = 1;
    if (pieces > 64) pieces = 64;
    VB_TRY(set_device(e));
    if (!e->h2d_stream) VB_CUDA(cudaStreamCreateWithFlags(&e->h2d_stream, cudaStreamNonBlocking));
    if (!e->d2h_stream) VB_CUDA(cudaStreamCreateWithFlags(&e->d2h_stream, cudaStreamNonBlocking));
    while ((int)e->pipe_events.size() < 2 * pieces + 2) {
        cudaEvent_t ev;
        VB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        e->pipe_events.push_back(ev);
    }
    VB_TRY(fence_check_error(opt));
    ExchangePlan xp;
    VB_TRY(plan_exchange(opt, VB_STEP_DEFAULT, &xp));
    int op;
    StepScalars s;
    if (opt->kind == KIND_ADAM) {
        opt->t += 1;
        op = OP_ADAM;
        s = make_scalars(op, opt->lr, opt->beta1, opt->beta2, opt->eps, opt->weight_decay, opt->t);
    } else {
        op = opt->momentum > 0.0f ? OP_SGD_MOMENTUM : OP_SGD;
        s = make_scalars(op, opt->lr, opt->momentum, 0.0f, 0.0f, opt->weight_decay, 0);
    }
    std::fill(opt->present.begin(), opt->present.end(), (uint8_t)1);  // a whole gradient arena arrives
    opt->present_on_dev = opt->present;
    VB_CUDA(cudaMemsetAsync(opt->d_present, 1, opt->present.size(), e->stream));
    VB_TRY(exchange_fence(opt, xp, 1));
    // everything enqueued so far (earlier steps, uploads) precedes the first copy of this step
    cudaEvent_t ev_start = e->pipe_events[2 * pieces];
    VB_CUDA(cudaEventRecord(ev_start, e->stream));
    VB_CUDA(cudaStreamWaitEvent(e->h2d_stream, ev_start, 0));
    VB_CUDA(cudaStreamWaitEvent(e->d2h_stream, ev_start, 0));
    // phase timing (when on): the span of each stream's part of the step; the three overlap
    prof_begin(e, VB_PHASE_HOST_H2D, e->h2d_stream);
    prof_begin(e, VB_PHASE_UPDATE);
    prof_begin(e, VB_PHASE_HOST_D2H, e->d2h_stream);
    const int64_t nc = opt->n_chunks;
    for (int j = 0; j < pieces; ++j) {
        const int64_t c_lo = nc * j / pieces, c_hi = nc * (j + 1) / pieces;
        if (c_hi <= c_lo) continue;
        // the arena range the chunks [c_lo, c_hi) cover (gaps between tensors travel along)
        const int64_t a_lo = j == 0 ? opt->shard_begin : opt->chunk_pos[(size_t)c_lo];
        const int64_t a_hi = c_hi == nc ? opt->shard_end : opt->chunk_pos[(size_t)c_hi];
        const size_t bytes = (size_t)(a_hi - a_lo) * sizeof(float);
        VB_CUDA(cudaMemcpyAsync(opt->d_grad + a_lo, grads_host + a_lo, bytes, cudaMemcpyHostToDevice, e->h2d_stream));
        VB_CUDA(cudaEventRecord(e->pipe_events[2 * j], e->h2d_stream));
        VB_CUDA(cudaStreamWaitEvent(e->stream, e->pipe_events[2 * j], 0));
        VB_TRY(launch_multi_tensor(op, opt->d_chunks + c_lo, c_hi - c_lo, opt->d_present, /*all_present=*/true, s,
                                   e->sm_count, e->stream, &xp.pt));
        e->launches += 1;
        VB_CUDA(cudaEventRecord(e->pipe_events[2 * j + 1], e->stream));
        VB_CUDA(cudaStreamWaitEvent(e->d2h_stream, e->pipe_events[2 * j + 1], 0));
        VB_CUDA(cudaMemcpyAsync(params_host + a_lo, opt->d_param + a_lo, bytes, cudaMemcpyDeviceToHost, e->d2h_stream));
    }
    prof_end(e, VB_PHASE_HOST_H2D, e->h2d_stream);
    prof_end(e, VB_PHASE_UPDATE);
    prof_end(e, VB_PHASE_HOST_D2H, e->d2h_stream);
    VB_TRY(exchange_fence(opt, xp, 2));
    if (xp.nccl_f32) VB_TRY(comm_all_gather_inplace(e, opt->d_param, opt->tail_begin / e->world));
    if (xp.nccl_half)
        VB_TRY(comm_all_gather_inplace_bytes(e, opt->d_param_bf16, opt->tail_begin / e->world * (int64_t)sizeof(uint16_t)));
    VB_CUDA(cudaStreamSynchronize(e->d2h_stream));
    VB_CUDA(cudaStreamSynchronize(e->stream));
    return fence_check_error(opt);
    VB_API_END
}

int vb_optimizer_export_state(vb_optimizer *opt, int64_t tensor, int which, float *host, int64_t n,
                              int64_t *owned_begin, int64_t *owned_end)
{
    VB_API_BEGIN
    VB_TRY(check_tensor(opt, tensor, n, true));
    if (n > 0 && !host) return fail(VB_ERR_INVALID_ARG, "host pointer is null");
    float *state = which == 0 ? opt->d_s1 : which == 1 ? opt->d_s2 : nullptr;
    if (which != 0 && which != 1) return fail(VB_ERR_INVALID_ARG, "which must be 0 or 1");
    VB_TRY(set_device(opt->eng));
    int64_t lo = 0, hi = 0;
    if (opt->kind == KIND_MUON) {
        if (which != 0) return fail(VB_ERR_INVALID_ARG, "Muon has one state buffer (velocity)");
        if (muon_owner(opt, tensor) == opt->eng->rank) hi = n;
    } else {
        // Every element is reported by exactly one rank: its slice by its owner, the replicated tail
        // (identical on all ranks) by the last rank, whose slice ends where the tail begins, so
        // that the reported range stays one interval.
        const int64_t off = opt->offsets[tensor];
        const bool with_tail = opt->eng->rank == opt->eng->world - 1;
        lo = std::max(off, opt->shard_begin) - off;
        hi = std::min(off + n, with_tail ? opt->arena : opt->shard_end) - off;
        if (hi < lo) lo = hi = 0;
    }
    if (!state && hi > lo)
        return fail(VB_ERR_STATE, "this optimizer has no state buffer %d (e.g. SGD without momentum)", which);
    if (n > 0) memset(host, 0, (size_t)n * sizeof(float));
    if (hi > lo) {
        if (opt->kind == KIND_MUON) {
            VB_CUDA(cudaMemcpyAsync(host + lo, muon_velocity_ptr(opt, tensor) + lo, (size_t)(hi - lo) * sizeof(float),
                                    cudaMemcpyDeviceToHost, opt->eng->stream));
        } else {
            // the slice part and the tail part are two runs of the state arrays
            const int64_t off = opt->offsets[tensor];
            const int64_t mid = std::min(std::max(opt->tail_begin - off, lo), hi);
            if (mid > lo)
                VB_CUDA(cudaMemcpyAsync(host + lo, state + opt->state_pos(off + lo), (size_t)(mid - lo) * sizeof(float),
                                        cudaMemcpyDeviceToHost, opt->eng->stream));
            if (hi > mid)
                VB_CUDA(cudaMemcpyAsync(host + mid, state + opt->state_pos(off + mid), (size_t)(hi - mid) * sizeof(float),
                                        cudaMemcpyDeviceToHost, opt->eng->stream));
        }
        VB_CUDA(cudaStreamSynchronize(opt->eng->stream));
    }
    if (owned_begin) *owned_begin = lo;
    if (owned_end) *owned_end = hi;
    return VB_OK;
    VB_API_END
}

int vb_optimizer_import_state(vb_optimizer *opt, int64_t tensor, int which, const float *host, int64_t n)
{
    VB_API_BEGIN
    VB_TRY(check_tensor(opt, tensor, n, true));
    if (n > 0 && !host) return fail(VB_ERR_INVALID_ARG, "host pointer is null");
    if (which != 0 && which != 1) return fail(VB_ERR_INVALID_ARG, "which must be 0 or 1");
    float *state = which == 0 ? opt->d_s1 : opt->d_s2;
    VB_TRY(set_device(opt->eng));
    int64_t lo = 0, hi = 0;
    if (opt->kind == KIND_MUON) {
        if (which != 0) return fail(VB_ERR_INVALID_ARG, "Muon has one state buffer (velocity)");
        if (muon_owner(opt, tensor) == opt->eng->rank) hi = n;
    } else {
        const int64_t off = opt->offsets[tensor];
        lo = std::max(off, opt->shard_begin) - off;
        hi = std::min(off + n, opt->shard_end) - off;
        if (hi < lo) lo = hi = 0;
    }
    // every rank keeps the part of the replicated tail this tensor reaches into as well
    int64_t t_lo = 0, t_hi = 0;
    if (opt->kind != KIND_MUON) {
        const int64_t off = opt->offsets[tensor];
        t_lo = std::max(off, opt->tail_begin) - off;
        t_hi = std::min(off + n, opt->arena) - off;
        if (t_hi < t_lo) t_lo = t_hi = 0;
    }
    if (!state && (hi > lo || t_hi > t_lo)) return fail(VB_ERR_STATE, "this optimizer has no state buffer %d", which);
    if (hi > lo) {
        float *dst = opt->kind == KIND_MUON ? muon_velocity_ptr(opt, tensor) + lo
                                            : state + opt->state_pos(opt->offsets[tensor] + lo);
        VB_CUDA(cudaMemcpyAsync(dst, host + lo, (size_t)(hi - lo) * sizeof(float), cudaMemcpyHostToDevice,
                                opt->eng->stream));
    }
    if (t_hi > t_lo)
        VB_CUDA(cudaMemcpyAsync(state + opt->state_pos(opt->offsets[tensor] + t_lo), host + t_lo,
                                (size_t)(t_hi - t_lo) * sizeof(float), cudaMemcpyHostToDevice, opt->eng->stream));
    if (hi > lo || t_hi > t_lo) VB_CUDA(cudaStreamSynchronize(opt->eng->stream));
    return VB_OK;
    VB_API_END
}

int vb_optimizer_ipc_handle(vb_optimizer *opt, void *handle64)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    if (!handle64) return fail(VB_ERR_INVALID_ARG, "handle64 is null");
    static_assert(sizeof(cudaIpcMemHandle_t) == VB_IPC_HANDLE_BYTES, "CUDA IPC handles are 64 bytes");
    VB_TRY(set_device(opt->eng));
    cudaIpcMemHandle_t h;
    VB_CUDA(cudaIpcGetMemHandle(&h, opt->d_param));
    memcpy(handle64, &h, sizeof(h));
    return VB_OK;
    VB_API_END
}

static int open_peer_handles(vb_optimizer *opt, const void *handles, int n_handles, void **mapped_out)
{
    vb_engine *e = opt->eng;
    if (!handles) return fail(VB_ERR_INVALID_ARG, "handles is null");
    if (n_handles != e->world)
        return fail(VB_ERR_INVALID_ARG, "expected %d handles (one per rank), got %d", e->world, n_handles);
    if (e->world - 1 > kMaxPeers) return fail(VB_ERR_UNSUPPORTED, "at most %d peers", kMaxPeers);
    VB_TRY(set_device(e));
    int n = 0;
    for (int r = 0; r < e->world; ++r) {
        if (r == e->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + (size_t)r * VB_IPC_HANDLE_BYTES, sizeof(h));
        void *mapped = nullptr;
        VB_CUDA(cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess));
        opt->peer_mappings.push_back(mapped);
        mapped_out[n++] = mapped;
    }
    return VB_OK;
}

int vb_optimizer_enable_bf16_params(vb_optimizer *opt)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    if (opt->d_param_bf16) return VB_OK;
    VB_TRY(set_device(opt->eng));
    uint16_t *buf = nullptr;
    const size_t bytes = (size_t)opt->arena * sizeof(uint16_t) + kSyncWords * sizeof(uint32_t);
    VB_CUDA(cudaMalloc((void **)&buf, bytes));
    VB_CUDA(cudaMemsetAsync(buf, 0, bytes, opt->eng->stream));
    opt->d_param_bf16 = buf;
    return refresh_bf16(opt, 0, opt->arena);
    VB_API_END
}

int vb_optimizer_refresh_bf16_params(vb_optimizer *opt)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    if (!opt->d_param_bf16) return fail(VB_ERR_STATE, "the bf16 copy is not enabled");
    VB_TRY(set_device(opt->eng));
    return refresh_bf16(opt, 0, opt->arena);
    VB_API_END
}

int vb_optimizer_param_bf16_ptr(vb_optimizer *opt, int64_t tensor, void **out)
{
    VB_TRY(check_tensor(opt, tensor, 0, false));
    if (!out) return fail(VB_ERR_INVALID_ARG, "out is null");
    if (!opt->d_param_bf16) return fail(VB_ERR_STATE, "the bf16 copy is not enabled");
    *out = opt->d_param_bf16 + opt->offsets[tensor];
    return VB_OK;
}

int vb_optimizer_download_params_bf16(vb_optimizer *opt, int64_t tensor, uint16_t *host, int64_t n)
{
    VB_API_BEGIN
    VB_TRY(check_tensor(opt, tensor, n, true));
    if (!opt->d_param_bf16) return fail(VB_ERR_STATE, "the bf16 copy is not enabled");
    if (n == 0) return VB_OK;
    if (!host) return fail(VB_ERR_INVALID_ARG, "host pointer is null");
    VB_TRY(set_device(opt->eng));
    VB_CUDA(cudaMemcpyAsync(host, opt->d_param_bf16 + opt->offsets[tensor], (size_t)n * sizeof(uint16_t),
                            cudaMemcpyDeviceToHost, opt->eng->stream));
    VB_CUDA(cudaStreamSynchronize(opt->eng->stream));
    if (opt->kind == KIND_MUON) return muon_check_error(opt);
    return VB_OK;
    VB_API_END
}

int vb_optimizer_ipc_handle_bf16(vb_optimizer *opt, void *handle64)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    if (!handle64) return fail(VB_ERR_INVALID_ARG, "handle64 is null");
    if (!opt->d_param_bf16) return fail(VB_ERR_STATE, "the bf16 copy is not enabled");
    VB_TRY(set_device(opt->eng));
    cudaIpcMemHandle_t h;
    VB_CUDA(cudaIpcGetMemHandle(&h, opt->d_param_bf16));
    memcpy(handle64, &h, sizeof(h));
    return VB_OK;
    VB_API_END
}

int vb_optimizer_open_peers_bf16(vb_optimizer *opt, const void *handles, int n_handles)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    if (!opt->d_param_bf16) return fail(VB_ERR_STATE, "the bf16 copy is not enabled");
    if (opt->peers.n_half > 0) return fail(VB_ERR_STATE, "bf16 peers are already open");
    void *mapped[kMaxPeers] = {};
    VB_TRY(open_peer_handles(opt, handles, n_handles, mapped));
    for (int r = 0; r < opt->eng->world - 1; ++r) opt->peers.half_base[r] = (uint16_t *)mapped[r];
    opt->peers.n_half = opt->eng->world - 1;
    return VB_OK;
    VB_API_END
}

int vb_optimizer_open_peers(vb_optimizer *opt, const void *handles, int n_handles)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    if (opt->peers.n > 0) return fail(VB_ERR_STATE, "peers are already open");
    void *mapped[kMaxPeers] = {};
    VB_TRY(open_peer_handles(opt, handles, n_handles, mapped));
    for (int r = 0; r < opt->eng->world - 1; ++r) opt->peers.base[r] = (float *)mapped[r];
    opt->peers.local_base = opt->d_param;
    opt->peers.n = opt->eng->world - 1;
    return VB_OK;
    VB_API_END
}

int vb_optimizer_peer_copy_probe(vb_optimizer *opt, int reps, double *ms_per_rep)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    if (!ms_per_rep || reps < 1) return fail(VB_ERR_INVALID_ARG, "reps must be >= 1 and ms_per_rep non-null");
    vb_engine *e = opt->eng;
    if (opt->peers.n <= 0) return fail(VB_ERR_STATE, "vb_optimizer_open_peers first");
    if (opt->kind == KIND_MUON) return fail(VB_ERR_UNSUPPORTED, "the probe copies arena slices (Adam, SGD)");
    VB_TRY(set_device(e));
    VB_TRY(fence_check_error(opt));
    const int np = opt->peers.n;
    for (int k = 0; k < np; ++k)
        if (!e->peer_streams[k]) VB_CUDA(cudaStreamCreateWithFlags(&e->peer_streams[k], cudaStreamNonBlocking));
    for (int k = 0; k < np + 3; ++k)
        if (!e->peer_events[k]) VB_CUDA(cudaEventCreateWithFlags(&e->peer_events[k], k < np + 1 ? cudaEventDisableTiming : cudaEventDefault));
    cudaEvent_t ev_fork = e->peer_events[np], t0 = e->peer_events[np + 1], t1 = e->peer_events[np + 2];
    ExchangePlan xp;
    VB_TRY(plan_exchange(opt, VB_STEP_DEFAULT, &xp));
    const size_t bytes = (size_t)(opt->shard_end - opt->shard_begin) * sizeof(float);
    VB_TRY(exchange_fence(opt, xp, 1));  // every rank is here: all start sending together
    VB_CUDA(cudaEventRecord(t0, e->stream));
    for (int rep = 0; rep < reps; ++rep) {
        VB_CUDA(cudaEventRecord(ev_fork, e->stream));
        for (int k = 0; k < np; ++k) {
            VB_CUDA(cudaStreamWaitEvent(e->peer_streams[k], ev_fork, 0));
            VB_CUDA(cudaMemcpyAsync(opt->peers.base[k] + opt->shard_begin, opt->d_param + opt->shard_begin, bytes,
                                    cudaMemcpyDeviceToDevice, e->peer_streams[k]));
            VB_CUDA(cudaEventRecord(e->peer_events[k], e->peer_streams[k]));
            VB_CUDA(cudaStreamWaitEvent(e->stream, e->peer_events[k], 0));
        }
    }
    VB_TRY(exchange_fence(opt, xp, 2));  // ... and every rank's copies into this arena have landed
    VB_CUDA(cudaEventRecord(t1, e->stream));
    VB_CUDA(cudaStreamSynchronize(e->stream));
    float ms = 0.0f;
    VB_CUDA(cudaEventElapsedTime(&ms, t0, t1));
    *ms_per_rep = (double)ms / (double)reps;
    return fence_check_error(opt);
    VB_API_END
}

int vb_optimizer_ipc_handle_grads(vb_optimizer *opt, void *handle64)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    if (!handle64) return fail(VB_ERR_INVALID_ARG, "handle64 is null");
    VB_TRY(set_device(opt->eng));
    cudaIpcMemHandle_t h;
    VB_CUDA(cudaIpcGetMemHandle(&h, opt->d_grad));
    memcpy(handle64, &h, sizeof(h));
    return VB_OK;
    VB_API_END
}

int vb_optimizer_open_peers_grads(vb_optimizer *opt, const void *handles, int n_handles)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    if (opt->peers.n_grad > 0) return fail(VB_ERR_STATE, "gradient peers are already open");
    void *mapped[kMaxPeers] = {};
    VB_TRY(open_peer_handles(opt, handles, n_handles, mapped));
    for (int r = 0; r < opt->eng->world - 1; ++r) opt->peers.grad_base[r] = (const float *)mapped[r];
    opt->peers.n_grad = opt->eng->world - 1;
    return VB_OK;
    VB_API_END
}

int vb_optimizer_reset_state(vb_optimizer *opt)
{
    VB_API_BEGIN
    VB_TRY(check_opt(opt));
    vb_engine *e = opt->eng;
    VB_TRY(set_device(e));
    if (opt->kind == KIND_MUON) {
        VB_TRY(muon_reset_velocity(opt));
    } else {
        const size_t bytes = (size_t)opt->state_elems * sizeof(float);
        if (opt->d_s1) VB_CUDA(cudaMemsetAsync(opt->d_s1, 0, bytes, e->stream));
        if (opt->d_s2) VB_CUDA(cudaMemsetAsync(opt->d_s2, 0, bytes, e->stream));
    }
    opt->t = 0;
    return VB_OK;
    VB_API_END
}

int vb_optimizer_get_t(vb_optimizer *opt, int64_t *t)
{
    VB_TRY(check_opt(opt));
    if (!t) return fail(VB_ERR_INVALID_ARG, "null argument");
    *t = opt->t;
    return VB_OK;
}

int vb_optimizer_set_t(vb_optimizer *opt, int64_t t)
{
    VB_TRY(check_opt(opt));
    if (t < 0 || t > 0x7fffffff) return fail(VB_ERR_INVALID_ARG, "t out of range");
    opt->t = t;
    return VB_OK;
}

int vb_muon_download_update(vb_optimizer *opt, int64_t tensor, float *host, int64_t n)
{
    VB_API_BEGIN
    VB_TRY(check_tensor(opt, tensor, n, true));
    if (opt->kind != KIND_MUON) return fail(VB_ERR_INVALID_ARG, "not a Muon optimizer");
    VB_TRY(set_device(opt->eng));
    return muon_download_update(opt, tensor, host, n);
    VB_API_END
}

int vb_muon_set_keep_update(vb_optimizer *opt, int keep)
{
    VB_TRY(check_opt(opt));
    if (opt->kind != KIND_MUON) return fail(VB_ERR_INVALID_ARG, "not a Muon optimizer");
    return muon_set_keep_update(opt, keep);
}

int vb_muon_last_ns_flops(vb_optimizer *opt, double *flops)
{
    VB_TRY(check_opt(opt));
    if (!flops) return fail(VB_ERR_INVALID_ARG, "null argument");
    if (opt->kind != KIND_MUON) return fail(VB_ERR_INVALID_ARG, "not a Muon optimizer");
    return muon_last_flops(opt, flops);
}

// ---- caller-owned buffers ----------------------------------------------------------------

static int ensure_stage(vb_engine *e, int slot, size_t bytes)
{
    if (e->stage_bytes[slot] >= bytes) return VB_OK;
    size_t cap = std::max<size_t>(bytes, 1 << 16);
    cap = (cap + 4095) / 4096 * 4096;
    if (e->h_stage[slot]) VB_CUDA(cudaFreeHost(e->h_stage[slot]));
    if (e->d_stage[slot]) VB_CUDA(cudaFree(e->d_stage[slot]));
    e->h_stage[slot] = e->d_stage[slot] = nullptr;
    e->stage_bytes[slot] = 0;
    VB_CUDA(cudaHostAlloc(&e->h_stage[slot], cap, cudaHostAllocDefault));
    VB_CUDA(cudaMalloc(&e->d_stage[slot], cap));
    if (!e->stage_done[slot]) VB_CUDA(cudaEventCreateWithFlags(&e->stage_done[slot], cudaEventDisableTiming));
    e->stage_bytes[slot] = cap;
    return VB_OK;
}

int vb_multi_tensor_step(vb_engine *e, const vb_optimizer_step_params *hp, int64_t n_tensors,
                         const int64_t *sizes, void *const *params, const void *const *grads,
                         void *const *state1, void *const *state2)
{
    VB_API_BEGIN
    if (!hp) return fail(VB_ERR_INVALID_ARG, "null argument");
    int64_t total = 0;
    VB_TRY(check_caller_buffers(hp, n_tensors, sizes, params, grads, state1, state2, &total));
    if (!e) return fail(VB_ERR_INVALID_ARG, "engine is null");
    if (total == 0) return VB_OK;
    VB_TRY(set_device(e));
    VB_TRY(check_caller_memory(e, hp, n_tensors, sizes, params, grads, state1, state2));
    const int64_t chunk_len = pick_chunk_len(total, e->sm_count);
    int64_t n_chunks = 0;
    for (int64_t i = 0; i < n_tensors; ++i) n_chunks += (sizes[i] + chunk_len - 1) / chunk_len;
    if (n_chunks == 0) return VB_OK;

    // staging block: one FatChunk per chunk, built in pinned memory and copied on the stream
    const size_t bytes = (size_t)n_chunks * sizeof(FatChunk);
    const int slot = e->stage_next;
    e->stage_next ^= 1;
    if (e->stage_done[slot]) VB_CUDA(cudaEventSynchronize(e->stage_done[slot]));  // previous user of this slot
    VB_TRY(ensure_stage(e, slot, bytes));
    FatChunk *chs = (FatChunk *)e->h_stage[slot];
    int64_t c = 0;
    for (int64_t i = 0; i < n_tensors; ++i) {
        for (int64_t b = 0; b < sizes[i]; b += chunk_len) {
            FatChunk &f = chs[c++];
            f.p = (float *)params[i] + b;
            f.g = (const float *)grads[i] + b;
            f.s1 = (state1 && state1[i]) ? (float *)state1[i] + b : nullptr;
            f.s2 = (state2 && state2[i]) ? (float *)state2[i] + b : nullptr;
            f.len = (uint32_t)std::min(chunk_len, sizes[i] - b);
            f.tensor = (uint32_t)i;
            f.local_only = 0;
        }
    }
    FatChunk *d = (FatChunk *)e->d_stage[slot];
    VB_CUDA(cudaMemcpyAsync(d, chs, bytes, cudaMemcpyHostToDevice, e->stream));
    VB_CUDA(cudaEventRecord(e->stage_done[slot], e->stream));
    const StepScalars s = make_scalars((int)hp->op, hp->lr, hp->beta1, hp->beta2, hp->eps, hp->weight_decay,
                                       (int64_t)hp->t);
    VB_TRY(launch_multi_tensor((int)hp->op, d, n_chunks, nullptr, /*all_present=*/true, s, e->sm_count,
                               e->stream));
    e->launches += 1;
    return VB_OK;
    VB_API_END
}

}  // extern "C"
