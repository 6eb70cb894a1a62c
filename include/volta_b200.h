/*
 * volta_b200 — C ABI of the B200 (sm_100a) optimizer-step engine for Volta.
 *
 * This is the whole boundary between Volta's optimizer types (Adam / SGD / Muon with
 * step() and zero_grad()) and the CUDA implementation: plain pointers, sizes and
 * scalars, no C++ or torch types.  A Rust, C++ or Python host binds exactly these
 * symbols.  Each declaration names the reference interface (path:line inside
 * rlarson20/Volta 0.3.0) it stands in for.
 *
 * Conventions
 *  - Every function returns a vb_status (0 = ok).  Nothing aborts, throws or prints;
 *    vb_last_error() gives the message of the calling thread's last failure.  (Volta's
 *    own step() panics on invariant violations and silently drops a failed GPU
 *    dispatch, src/nn/optim/adam.rs:127-129,164; here the caller gets a code.)
 *  - One engine = one CUDA device + one stream.  All work of an engine is enqueued on
 *    that stream in call order; calls return without waiting unless stated.  An engine
 *    and its optimizers are used from one host thread at a time (Volta is single
 *    threaded: Tensor = Rc<RefCell<_>>, src/tensor.rs:16-23).
 *  - All tensors are contiguous row-major f32, as Volta's optimizers require
 *    (src/storage.rs:269-281).
 *  - There is no CPU fallback: without a usable CUDA device every call fails with
 *    VB_ERR_CUDA.
 */
#ifndef VOLTA_B200_H
#define VOLTA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum vb_status {
    VB_OK = 0,
    VB_ERR_INVALID_ARG = 1, /* null pointer, bad index, size mismatch, bad hyper-parameter */
    VB_ERR_CUDA = 2,        /* a CUDA runtime/driver call failed (message has the code) */
    VB_ERR_NCCL = 3,        /* NCCL missing or a collective failed */
    VB_ERR_TIMEOUT = 4,     /* a bounded device-side wait gave up */
    VB_ERR_STATE = 5,       /* call not valid in the object's current state */
    VB_ERR_UNSUPPORTED = 6  /* shape or mode this build does not implement */
} vb_status;

typedef struct vb_engine vb_engine;
typedef struct vb_optimizer vb_optimizer;

/* Same field order, types and size (32 bytes) as Volta's OptimizerStepParams
 * (src/gpu/kernels.rs:42-54), the uniform its WGSL kernel reads
 * (src/gpu/shaders/optimizer_step.wgsl:8-17).  op: 0 SGD, 1 SGD+momentum, 2 Adam.
 * beta1 doubles as the momentum coefficient for op 1; t is the time step as f32. */
typedef struct vb_optimizer_step_params {
    uint32_t op;
    float lr;
    float beta1;
    float beta2;
    float t;
    float eps;
    float weight_decay;
    float padding;
} vb_optimizer_step_params;

/* Newton-Schulz arithmetic of a Muon optimizer. */
typedef enum vb_ns_mode {
    /* f32-faithful: sum of squares in the reference's sequential order
     * (src/nn/optim/muon.rs:58), contraction accurate to f32, operations in the
     * reference's order.  Target: relative Frobenius error <= 1e-5 per matrix. */
    VB_NS_F32 = 0,
    /* bf16 operands on the tcgen05 tensor cores, f32 accumulation in TMEM.
     * Target: relative Frobenius error <= 2e-2 per matrix.
     * Both tensor-core modes evaluate the iteration (src/nn/optim/muon.rs:67-100) in an
     * algebraically equal chain form: every Gram matrix of the iteration is a polynomial in the
     * first one, so one Gram and one product on the long side of the matrix frame a chain of
     * short-side symmetric squares.  VB_NS_CHAIN=0 in the environment at creation selects one
     * Gram and one update product per iteration instead; the targets hold for both. */
    VB_NS_BF16 = 1,
    /* f32-accurate on the tensor cores: every operand is held as two f16 pieces of the value
     * scaled by 2^15 (22 significand bits; Newton-Schulz operands are bounded by 1 once the
     * update is normalised) and each product is three tcgen05 f16 products accumulated in f32;
     * the sum of squares keeps the reference's sequential order.  Same target as VB_NS_F32
     * (<= 1e-5) at tensor-core speed, but not bit-identical to the CPU arithmetic.  Updates far
     * smaller than sqrt(1e-8), whose normalised form is tiny (src/nn/optim/muon.rs:59), are held
     * with a larger power of two so that the bound covers them as well. */
    VB_NS_F32_TC = 2
} vb_ns_mode;

/* Flags of vb_optimizer_step_ex. */
#define VB_STEP_DEFAULT 0u
#define VB_STEP_NO_EXCHANGE 1u /* sharded engines: update the owned part only, skip the all-gather / broadcast */
#define VB_STEP_REDUCE_GRADS 4u /* sharded engines, after vb_optimizer_open_peers_grads: the gradient of every element a
                                   rank updates is the sum of all ranks' gradients (a reduce-scatter fused into the
                                   update kernel's loads) */
#define VB_STEP_MEAN_GRADS 8u   /* as VB_STEP_REDUCE_GRADS, the sum multiplied by 1 / world_size */
#define VB_STEP_EXCHANGE_BF16 2u /* sharded engines with the bf16 copy enabled: exchange only the bf16 copies (half the
                                    bytes); f32 parameters other ranks own are left as they were */

/* ---- library ---------------------------------------------------------------------- */

/* ABI version of this header (major*1000 + minor). */
int vb_abi_version(void);
/* Message of the calling thread's most recent failing call ("" if none). */
const char *vb_last_error(void);
/* Number of CUDA devices visible (replaces is_gpu_available(), src/gpu/mod.rs:50-60). */
int vb_device_count(int *count);

/* Pure host planning, no CUDA call: the arena layout (element offset of every tensor,
 * each on a 128-byte boundary), the arena slice [shard_begin, shard_end) that `rank` of
 * `world_size` owns, and the chunk table (tensor, offset within tensor, length) that
 * rank's fused Adam/SGD launch walks on a device with `sm_count` SMs.  Every output
 * pointer may be NULL; chunk arrays need chunk_capacity >= *n_chunks (query first).
 * This is exactly the plan vb_adam_create / vb_sgd_create use; it exists so that hosts
 * and tests can check coverage (every element owned by exactly one rank and one chunk)
 * without a GPU.  No counterpart in the reference (one dispatch per tensor,
 * src/gpu/kernels.rs:2077-2078). */
int vb_plan_layout(int64_t n_tensors, const int64_t *sizes, int world_size, int rank, int sm_count,
                   int64_t *offsets_out, int64_t *arena_elements, int64_t *shard_begin,
                   int64_t *shard_end, int64_t *n_chunks, int64_t chunk_capacity,
                   int64_t *chunk_tensor, int64_t *chunk_offset, int64_t *chunk_len);
/* The same plan with a replicated tail (see vb_engine_set_replicated_fraction): the positions
 * [0, *tail_begin) are cut into the ranks' slices, [*tail_begin, *arena_elements) is updated by
 * every rank; chunk_local_only[c] = 1 marks the chunks of the tail, which the table interleaves
 * with those of the slice.  replicated_fraction = 0 gives vb_plan_layout's plan. */
int vb_plan_layout_replicated(int64_t n_tensors, const int64_t *sizes, int world_size, int rank, int sm_count,
                              double replicated_fraction, int64_t *offsets_out, int64_t *arena_elements,
                              int64_t *shard_begin, int64_t *shard_end, int64_t *tail_begin,
                              int64_t *n_chunks, int64_t chunk_capacity, int64_t *chunk_tensor,
                              int64_t *chunk_offset, int64_t *chunk_len, int32_t *chunk_local_only);
/* The replicated fraction at which a sharded step's HBM time and NVLink time are equal, from
 * the bytes one element's update moves through HBM (Adam 28, SGD with momentum 20, plain SGD
 * 12), the HBM rate of the update kernel and the NVLink rate per direction of the fused exchange
 * with both directions busy (GB/s; measure them, e.g. from a step with VB_STEP_NO_EXCHANGE and a
 * whole step without replication).  0 when exchanging everything is not the bottleneck. */
int vb_plan_replicated_fraction(double bytes_per_element, int world_size, double hbm_gb_per_s,
                                double link_gb_per_s, double *fraction);

/* Pure host planning, no CUDA call: which rank owns each Muon tensor.  Whole tensors are
 * taken in order of decreasing estimated cost per step under the arithmetic `ns_mode` really
 * executes and given to the least-loaded rank; this is the assignment vb_muon_create uses.
 * Cost: VB_NS_F32 runs the reference's formulation, 4 * rows * cols^2 FLOPs per iteration
 * whatever the orientation (src/nn/optim/muon.rs:73 forms cols x cols), on the CUDA cores; the
 * tensor-core modes run the chain form: the first Gram (tiles on and above the diagonal) and the
 * last product on the long side, 2 * long * short^2 each in full, and 3 K - 3 (VB_NS_F32_TC:
 * 3 K - 2) short-side squares on their upper tiles (three plane products each in VB_NS_F32_TC);
 * shapes that a tensor-core mode hands to the f32 kernels (a side not a multiple of 8) are
 * charged as such; every tensor also pays its element-wise passes.  rank_cost_out (world_size
 * entries, may be NULL) receives each rank's summed estimate in seconds.  No counterpart in the
 * reference (single process). */
int vb_plan_muon_owners(int64_t n_tensors, const int64_t *rows, const int64_t *cols, int world_size,
                        int ns_mode, int ns_steps, int32_t *owner_out, double *rank_cost_out);

/* Plan fingerprints: do all ranks describe the same optimizer?  A sharded step is a collective;
 * ranks that disagree on the tensor list, the hyper-parameters, the mode or the world size would
 * write into each other's arenas at wrong offsets or wait for each other for ever.  The
 * fingerprint is a 64-bit hash of exactly those inputs (not of the rank).  The host gathers the
 * ranks' fingerprints over its own transport before vb_optimizer_open_peers or the first step and
 * hands them to vb_plan_fingerprints_agree, which returns VB_ERR_STATE (on every rank, since every
 * rank sees the same list) naming the first rank that differs from rank 0.  vb_plan_fingerprint is
 * the pure host form (no CUDA call, usable before any engine exists): kind 0 Adam, 1 SGD, 2 Muon;
 * sizes_or_rows / cols as in the create calls (cols NULL for Adam and SGD); hyper and ints are
 * the scalar arguments of the create call in order.  Counterpart in the reference: none (single
 * process); its own pre-flight check is check_system_resources, src/gpu/monitor.rs:58-100. */
int vb_plan_fingerprint(int kind, int64_t n_tensors, const int64_t *sizes_or_rows, const int64_t *cols,
                        const float *hyper, int n_hyper, const int32_t *ints, int n_ints, int world_size,
                        uint64_t *fingerprint);
int vb_plan_fingerprints_agree(const uint64_t *fingerprints, int n_ranks, int *first_mismatch);

/* ---- engine (replaces the process-global wgpu context, src/gpu/mod.rs:30-47) ----- */

int vb_engine_create(int device, vb_engine **out);
int vb_engine_destroy(vb_engine *engine);
/* Blocks until everything enqueued so far has run (GpuContext::sync, src/gpu/context.rs:342-382). */
int vb_engine_synchronize(vb_engine *engine);
/* The same with a deadline on the host: polls the stream for at most timeout_ms and returns
 * VB_ERR_TIMEOUT if work is still queued (sync_checked()'s timeout path,
 * src/gpu/context.rs:448-505).  Nothing is cancelled: the engine stays usable and a later
 * synchronize can wait for the rest.  Both forms also report, as VB_ERR_TIMEOUT, a device-side
 * wait of one of the engine's optimizers that ran out (see vb_engine_set_wait_limit_ms). */
int vb_engine_synchronize_deadline(vb_engine *engine, double timeout_ms);
/* Bound, in milliseconds of device wall time, of every wait of this engine's kernels on another
 * rank (the flag barrier around sharded steps).  Default 5000.  A wait that runs out ends the
 * step on every rank: each rank's next call on the optimizer (or synchronize) returns
 * VB_ERR_TIMEOUT, the optimizer is fail-stop from then on, the CUDA context stays usable.
 * No counterpart in the reference (single process; its own waits are bounded by
 * sync_checked(), src/gpu/context.rs:448-505). */
int vb_engine_set_wait_limit_ms(vb_engine *engine, uint32_t milliseconds);
/* Sharded engines, Adam and SGD optimizers created after the call: the last `fraction` of the
 * arena is not sharded.  Every rank keeps optimizer state for that tail and updates it itself in
 * the same launch that updates (and sends to the peers) its slice of the rest, so that part of
 * the parameters never crosses NVLink: when the exchange bounds the step (it does from two B200s
 * on: 4 B/param into every GPU against 28 B/param of HBM traffic shared by N GPUs) the launch
 * overlaps link-bound and HBM-bound work, see vb_plan_replicated_fraction.  The price: state
 * memory for the tail on every rank, and every rank needs the complete, identical gradients of
 * the tail (the default when gradients were all-reduced; with VB_STEP_REDUCE_GRADS every rank
 * sums the tail's gradients itself, which multiplies that NVLink traffic).  Results are
 * unchanged: all ranks run the same arithmetic on the same inputs.  All ranks must set the same
 * fraction (vb_optimizer_plan_fingerprint covers it).  Default 0: plain ZeRO-1 slices.  No
 * counterpart in the reference (single device). */
int vb_engine_set_replicated_fraction(vb_engine *engine, double fraction);
/* The engine's cudaStream_t, for callers that enqueue their own producers of gradients. */
int vb_engine_stream(vb_engine *engine, void **cuda_stream);
/* Kernels launched by this engine since creation (bookkeeping for benchmarks). */
int vb_engine_launch_count(vb_engine *engine, uint64_t *count);

/* Phase timing for benchmarks (no counterpart in the reference; its SystemMonitor counts
 * operations with host clocks, src/gpu/system_monitor.rs:31-150).  While profiling is on,
 * every step brackets its phases with CUDA events on the engine stream.
 * vb_engine_profile waits for the stream, returns the summed device time and the number
 * of brackets of one phase since the last query, and clears them. */
#define VB_PHASE_UPDATE 0    /* fused Adam / SGD launch */
#define VB_PHASE_MUON_PRE 1  /* Muon momentum, sum of squares, normalise */
#define VB_PHASE_MUON_NS 2   /* Muon Newton-Schulz GEMM chain */
#define VB_PHASE_MUON_APPLY 3 /* the separate apply pass, or the last update launch when it applies its result itself
                                (that launch is then counted under VB_PHASE_MUON_NS as well) */
#define VB_PHASE_EXCHANGE 4  /* fences of a fused exchange; NCCL all-gather / broadcast */
#define VB_PHASE_HOST_H2D 5  /* vb_optimizer_step_host: gradient uploads (first to last, on their own stream) */
#define VB_PHASE_HOST_D2H 6  /* vb_optimizer_step_host: parameter downloads (first to last, on their own stream) */
#define VB_PHASE_COUNT 7
int vb_engine_set_profiling(vb_engine *engine, int enabled);
int vb_engine_profile(vb_engine *engine, int phase, double *total_ms, int64_t *count);

/* Failure-detection self-test (the reference's counterpart is sync_checked()'s timeout path,
 * src/gpu/context.rs:448-505).  Runs the tensor-core GEMM kernel on a small problem whose
 * loads are withheld, so that every bounded wait inside the kernel expires after
 * `wait_limit` polls (0 = default).  The kernel must then record which role gave up, free
 * its tensor memory and return; this call reports VB_ERR_TIMEOUT with that role in
 * *role_code, and the engine stays usable.  Nothing faults or hangs. */
int vb_debug_gemm_wait_expiry(vb_engine *engine, uint32_t wait_limit, int *role_code);
/* The same inside a real optimizer: the next step of this Muon optimizer withholds the loads of
 * its first tensor-core launch, with `wait_limit` polls per wait (0 = default).  That launch
 * records the expiry; every later kernel of the step sees the record and stores nothing, so the
 * weights keep their pre-step values (the velocity has advanced).  The step itself returns
 * VB_OK (work is enqueued); the next call that waits for the stream returns VB_ERR_TIMEOUT and
 * the optimizer is fail-stop from then on. */
int vb_debug_muon_withhold_loads(vb_optimizer *opt, uint32_t wait_limit);
/* Self-test of the flag barrier that fences sharded steps (a rank that never arrives, simulated
 * on one GPU by a flag nobody sets): runs one fence kernel of the given phase (1 start, 2 end)
 * against a peer block in this GPU's own memory with a bound of timeout_ms.  Reports
 * VB_ERR_TIMEOUT with the phase in *code; the engine stays usable.  Nothing faults or hangs. */
int vb_debug_fence_wait_expiry(vb_engine *engine, uint32_t timeout_ms, int phase, int *code);

/* Page-locked host memory for upload/download buffers (pinned buffers make the copies
 * asynchronous and full speed; a pinned upload buffer must stay unchanged until the next
 * vb_engine_synchronize or download).  Counterpart: the staging buffer pool,
 * src/gpu/staging_pool.rs. */
int vb_host_alloc_pinned(void **ptr, size_t bytes);
int vb_host_free_pinned(void *ptr);

/* Multi-GPU (no counterpart in the reference, which is single-process, README.md:61-62):
 * one process per GPU; rank 0 makes an id, the host shares its 128 bytes with the other
 * ranks by any means, every rank calls vb_engine_comm_init.  Optimizers created
 * afterwards shard their state over the ranks (Adam/SGD: equal slices of the flat
 * parameter arena; Muon: whole matrices by FLOPs) and exchange updated parameters with
 * NCCL at the end of step(). */
int vb_comm_unique_id(void *id128);
int vb_engine_comm_init(vb_engine *engine, const void *id128, int rank, int world_size);
int vb_engine_rank(vb_engine *engine, int *rank, int *world_size);

/* ---- optimizer construction ------------------------------------------------------- */

/* Adam::new(params, lr, betas, eps, weight_decay), src/nn/optim/adam.rs:18-60.
 * sizes[i] = element count of parameter i.  The engine allocates flat device arenas for
 * parameters, gradients and the moments m, v (zero-initialised, adam.rs:26-47), every
 * tensor starting on a 128-byte boundary.  t starts at 0. */
int vb_adam_create(vb_engine *engine, int64_t n_tensors, const int64_t *sizes, float lr,
                   float beta1, float beta2, float eps, float weight_decay, vb_optimizer **out);

/* SGD::new(params, lr, momentum, weight_decay), src/nn/optim/sgd.rs:28-52.  Velocity is
 * allocated only when momentum > 0.0 (sgd.rs:30). */
int vb_sgd_create(vb_engine *engine, int64_t n_tensors, const int64_t *sizes, float lr,
                  float momentum, float weight_decay, vb_optimizer **out);

/* Muon::new(params, lr, momentum, nesterov, ns_steps), src/nn/optim/muon.rs:19-38.
 * rows[i], cols[i] are the 2-D view of parameter i that Muon::step derives from its
 * shape (muon.rs:117-130): (shape[0], product of the rest), or (n, 1) for 1-D.
 * Newton-Schulz runs only where rows > 1 and cols > 1 (muon.rs:153). */
int vb_muon_create(vb_engine *engine, int64_t n_tensors, const int64_t *rows, const int64_t *cols,
                   float lr, float momentum, int nesterov, int ns_steps, int ns_mode,
                   vb_optimizer **out);

int vb_optimizer_destroy(vb_optimizer *opt);
/* The fingerprint of this optimizer's plan (see vb_plan_fingerprint). */
int vb_optimizer_plan_fingerprint(vb_optimizer *opt, uint64_t *fingerprint);

/* ---- tensors of an optimizer ------------------------------------------------------ */

int vb_optimizer_num_tensors(vb_optimizer *opt, int64_t *n_tensors);
int vb_optimizer_tensor_size(vb_optimizer *opt, int64_t tensor, int64_t *n_elements);
/* Sum of all tensor sizes. */
int vb_optimizer_total_size(vb_optimizer *opt, int64_t *n_elements);

/* Host <-> device copies of one parameter tensor (its `data`, src/tensor.rs:38-46).
 * n must equal the tensor's size.  Uploads/downloads are enqueued on the engine stream;
 * download blocks until the data is in `host`. `host` may be pageable or pinned. */
int vb_optimizer_upload_params(vb_optimizer *opt, int64_t tensor, const float *host, int64_t n);
int vb_optimizer_download_params(vb_optimizer *opt, int64_t tensor, float *host, int64_t n);

/* Sets the gradient of one tensor from host memory and marks it present
 * (`p.grad = Some(..)`, src/autograd.rs:140-148). */
int vb_optimizer_upload_grad(vb_optimizer *opt, int64_t tensor, const float *host, int64_t n);
int vb_optimizer_download_grad(vb_optimizer *opt, int64_t tensor, float *host, int64_t n);

/* Adds one gradient contribution on the device, as backward() does for a parameter that is
 * reached along several paths or over several micro-batches (RawTensor::accumulate_grad,
 * src/autograd.rs:140-148,158-184): the first contribution after zero_grad() becomes the
 * gradient, later ones are added element by element (one rounded f32 add each).  The source
 * is host memory or a device buffer on the engine's device. */
int vb_optimizer_accumulate_grad(vb_optimizer *opt, int64_t tensor, const float *host, int64_t n);
int vb_optimizer_accumulate_grad_device(vb_optimizer *opt, int64_t tensor, const void *device_src, int64_t n);

/* Device addresses (f32, 128-byte aligned) so producers can write gradients / read
 * parameters in place without staging.  Valid until the optimizer is destroyed. */
int vb_optimizer_param_ptr(vb_optimizer *opt, int64_t tensor, void **device_ptr);
int vb_optimizer_grad_ptr(vb_optimizer *opt, int64_t tensor, void **device_ptr);

/* Whole-arena access: all tensors in index order, each padded to a 128-byte boundary.
 * offsets_out (n_tensors entries, may be NULL) receives each tensor's element offset. */
int vb_optimizer_arena(vb_optimizer *opt, void **param_arena, void **grad_arena,
                       int64_t *arena_elements, int64_t *offsets_out);
/* Copies whole arenas between a host buffer of arena_elements floats and the device
 * (one transfer instead of one per tensor).  which: 0 params, 1 grads.  Uploading grads
 * marks every tensor's gradient present. */
int vb_optimizer_upload_arena(vb_optimizer *opt, int which, const float *host, int64_t n);
int vb_optimizer_download_arena(vb_optimizer *opt, int which, float *host, int64_t n);

/* The same for a slice [begin, begin + n) of the arena: a rank of a sharded engine needs only
 * the gradients of its own slice (what a reduce-scatter would deliver) and publishes only the
 * parameters it updated.  Uploading a gradient slice marks every tensor's gradient present. */
int vb_optimizer_upload_arena_range(vb_optimizer *opt, int which, const float *host, int64_t begin, int64_t n);
int vb_optimizer_download_arena_range(vb_optimizer *opt, int which, float *host, int64_t begin, int64_t n);
/* The slice of the arena whose state this rank owns (Adam/SGD; the whole arena for Muon). */
int vb_optimizer_owned_range(vb_optimizer *opt, int64_t *begin, int64_t *end);
/* The tail of the arena every rank updates itself (empty, begin == end == arena size, unless
 * vb_engine_set_replicated_fraction was set when the optimizer was created). */
int vb_optimizer_replicated_range(vb_optimizer *opt, int64_t *begin, int64_t *end);

/* Presence of a gradient: step() skips tensors whose gradient is absent
 * (src/nn/optim/adam.rs:81-84, sgd.rs:75-78, muon.rs:110). */
int vb_optimizer_set_grad_present(vb_optimizer *opt, int64_t tensor, int present);

/* ---- the hot path ----------------------------------------------------------------- */

/* Adam::step / SGD::step / Muon::step (src/nn/optim/adam.rs:70-95, sgd.rs:69-90,
 * muon.rs:108-163).  One call updates every tensor whose gradient is present: Adam and
 * SGD in one fused multi-tensor launch, Muon as momentum/normalise -> Newton-Schulz GEMM
 * chain -> apply.  Adam's t advances by one per call whether or not any gradient is
 * present (adam.rs:71).  On a sharded engine the call ends with the parameter exchange.
 * Work is enqueued; use vb_engine_synchronize or a download to wait. */
int vb_optimizer_step(vb_optimizer *opt);
int vb_optimizer_step_ex(vb_optimizer *opt, uint32_t flags);

/* The whole step for a host-resident model in one call (Adam, SGD): `grads_host` and
 * `params_host` are host images of the arena (vb_optimizer_arena gives its length and the
 * tensor offsets).  The owned part of the arena is cut into `pieces` (1..64); for each piece
 * the gradients are copied to the device, updated, and the new parameters copied back, on
 * three streams so that the upload of piece j+1, the update of piece j and the download of
 * piece j-1 overlap (PCIe is full duplex).  Every gradient counts as present.  Returns when
 * the parameters are in `params_host`.  Use pinned host memory (vb_host_alloc_pinned):
 * pageable buffers work but serialise the copies.  This is what Volta's step() costs a
 * CPU-resident model (src/nn/optim/adam.rs:70-95), minus the two gradient clones. */
int vb_optimizer_step_host(vb_optimizer *opt, const float *grads_host, float *params_host, int pieces);

/* zero_grad(): marks every gradient absent (`grad = None`, src/nn/optim/adam.rs:62-66,
 * sgd.rs:58-62, muon.rs:40-44).  The gradient arena itself is left as is. */
int vb_optimizer_zero_grad(vb_optimizer *opt);

/* Hyper-parameters can change between steps (learning-rate schedules). */
int vb_optimizer_set_lr(vb_optimizer *opt, float lr);

/* Fused exchange over NVLink peer memory (sharded engines; no counterpart in the reference).  Every rank exports a CUDA IPC handle of its parameter arena, the host
 * gathers the world_size handles in rank order (any transport) and hands them to every
 * rank.  From then on step() no longer runs an all-gather / broadcast after the update: the
 * update kernel (Adam, SGD) or the apply kernel (Muon, for the matrices a rank owns) stores
 * each new parameter into the local arena and into the same position of every peer's arena,
 * fenced on both sides by a flag barrier in the same peer-mapped memory (one epoch word per rank,
 * system-scope release stores and acquire polls by a one-warp kernel; every wait is bounded by
 * vb_engine_set_wait_limit_ms).  All ranks must make the same sequence of step calls.
 * All ranks must be processes on one node whose GPUs can reach each other (NVLink/NVSwitch). */
#define VB_IPC_HANDLE_BYTES 64
int vb_optimizer_ipc_handle(vb_optimizer *opt, void *handle64);
int vb_optimizer_open_peers(vb_optimizer *opt, const void *handles, int n_handles);
/* Measures, in the running job, what the NVLink fabric gives the parameter exchange: every rank
 * copies the slice of the parameter arena it owns to the same position of every peer's arena
 * with the copy engines (one cudaMemcpyAsync per peer, all in flight together, `reps` times),
 * between the two halves of the exchange fence, so all ranks send and receive at once and the
 * time covers the arrival of everybody's data.  The copies rewrite values the peers already hold
 * after a step, so the parameters are unchanged.  *ms_per_rep is this rank's device time per
 * repetition; bytes in and out per repetition are (world - 1) slices each.  Needs
 * vb_optimizer_open_peers; all ranks must call it together.  Benchmarks use the result as the
 * measured ceiling of a sharded step's exchange.  No counterpart in the reference. */
int vb_optimizer_peer_copy_probe(vb_optimizer *opt, int reps, double *ms_per_rep);

/* Data-parallel gradients (no counterpart in the reference, which has one process and one
 * device).  Every rank holds its own gradient of the whole model in its gradient arena; after
 * vb_optimizer_open_peers_grads was given every rank's vb_optimizer_ipc_handle_grads,
 * step_ex(VB_STEP_REDUCE_GRADS) makes the update kernel (Adam, SGD) or the momentum kernel
 * (Muon) of the owning rank read the element's gradient from every rank over NVLink and add
 * the values in rank order, one rounded f32 addition per rank (VB_STEP_MEAN_GRADS: then multiply
 * by 1 / world_size): the reduce-scatter rides in the kernel's loads, gradients are read once,
 * and no reduced gradient is ever written.  The step is fenced by the same two stream-ordered
 * barriers as the fused parameter exchange, so work enqueued on the engine's stream after
 * step() (uploads through this API included) cannot overtake the peers' reads; a producer that
 * writes gradients from another stream must first wait for the engine's stream.  All ranks must
 * hold the same presence flags. */
int vb_optimizer_ipc_handle_grads(vb_optimizer *opt, void *handle64);
int vb_optimizer_open_peers_grads(vb_optimizer *opt, const void *handles, int n_handles);

/* bf16 copies of the parameters, written by the update kernel next to the f32 master (no
 * counterpart in the reference's optimizers; the rounding is the one its bf16 storage type
 * uses, round to nearest even, src/storage.rs:499-505).  After enabling, the library keeps a
 * second arena of one 16-bit word per parameter with bf16[i] == rne(param[i]): it is filled
 * from the current parameters, refreshed by every upload of parameters through this API and
 * written by every step for the parameters the step updates (call
 * vb_optimizer_refresh_bf16_params after writing parameters through vb_optimizer_param_ptr).
 * On a sharded engine the default step() exchanges both the f32 parameters and the copies;
 * VB_STEP_EXCHANGE_BF16 exchanges only the copies: 2 instead of 4 bytes per parameter cross
 * NVLink, every rank ends the step with the complete bf16 arena and with exact f32 values
 * for the part it owns only.  The copies travel by NCCL, or by peer stores fused into the
 * update / apply kernel once vb_optimizer_open_peers_bf16 was given every rank's
 * vb_optimizer_ipc_handle_bf16 (same protocol as vb_optimizer_open_peers).
 * Gradient-less parameters keep their value and their copy. */
int vb_optimizer_enable_bf16_params(vb_optimizer *opt);
int vb_optimizer_refresh_bf16_params(vb_optimizer *opt);
/* Device address of tensor i's copy (valid until destroy). */
int vb_optimizer_param_bf16_ptr(vb_optimizer *opt, int64_t tensor, void **out);
/* Copies tensor i's bf16 words to the host (blocking). */
int vb_optimizer_download_params_bf16(vb_optimizer *opt, int64_t tensor, uint16_t *host, int64_t n);
int vb_optimizer_ipc_handle_bf16(vb_optimizer *opt, void *handle64);
int vb_optimizer_open_peers_bf16(vb_optimizer *opt, const void *handles, int n_handles);

/* ---- optimizer state (private in the reference, src/nn/optim/adam.rs:5-14) -------- */

/* which: 0 = first state (Adam m, SGD velocity, Muon velocity), 1 = Adam v.
 * On a sharded engine only the owning rank holds a tensor's state: export returns the
 * owned elements and zeros elsewhere, and reports the owned range.  Every element is reported
 * by exactly one rank: the state of a replicated tail (vb_engine_set_replicated_fraction),
 * identical on all ranks, by the last rank, whose slice the tail follows.  Import takes the whole
 * tensor and keeps every element whose state the rank holds, the tail's on every rank. */
int vb_optimizer_export_state(vb_optimizer *opt, int64_t tensor, int which, float *host, int64_t n,
                              int64_t *owned_begin, int64_t *owned_end);
int vb_optimizer_import_state(vb_optimizer *opt, int64_t tensor, int which, const float *host,
                              int64_t n);
/* Puts the optimizer's state back to what the constructor leaves (moments / velocity zero,
 * src/nn/optim/adam.rs:26-47, sgd.rs:30-41, muon.rs:26-29; t = 0), on the device, without
 * touching parameters or gradients.  Benchmarks use it to replay a configuration from its
 * start; a training loop that restarts a schedule can too. */
int vb_optimizer_reset_state(vb_optimizer *opt);
int vb_optimizer_get_t(vb_optimizer *opt, int64_t *t);
int vb_optimizer_set_t(vb_optimizer *opt, int64_t t);

/* Muon only: copies the orthogonalised update of the last step for one tensor (the
 * reference's local `update`, src/nn/optim/muon.rs:139-155) to the host.  In the reference the
 * update is a temporary of step(); here the last Newton-Schulz launch of a tensor-core mode
 * applies it to the weights in its epilogue and does not store it unless
 * vb_muon_set_keep_update(opt, 1) was called before the step (VB_ERR_STATE otherwise; matrices
 * on the f32 kernels and vectors are always available).  Keeping it costs 4 bytes of HBM
 * writes per parameter and step. */
int vb_muon_set_keep_update(vb_optimizer *opt, int keep);
int vb_muon_download_update(vb_optimizer *opt, int64_t tensor, float *host, int64_t n);
/* Muon only: tensor-core FLOPs executed by the last step's Newton-Schulz chain. */
int vb_muon_last_ns_flops(vb_optimizer *opt, double *flops);

/* ---- caller-owned device buffers -------------------------------------------------- */

/* Replaces n_tensors calls of RawTensor::gpu_optimizer_step(params, grads, state1,
 * state2, &OptimizerStepParams) (src/ops/gpu_ops.rs:495-508, one wgpu dispatch per
 * tensor, src/gpu/kernels.rs:2016-2086) by one fused launch over caller-owned device
 * buffers.  params/grads/state1/state2 are host arrays of n_tensors device pointers;
 * state2 entries (and, for op 0, state1 entries) may be NULL where the op does not use
 * them.  hp->t is the step number the bias correction uses; it is computed on the host
 * with the reference's CPU arithmetic (powi, src/nn/optim/adam.rs:188-189), not the
 * shader's per-thread pow().  Before anything is launched every pointer the op touches is
 * checked on the host: non-null, 4-byte aligned and, the first time a pointer set is seen,
 * device memory of the engine's device; a violation returns VB_ERR_INVALID_ARG. */
int vb_multi_tensor_step(vb_engine *engine, const vb_optimizer_step_params *hp, int64_t n_tensors,
                         const int64_t *sizes, void *const *params, const void *const *grads,
                         void *const *state1, void *const *state2);

/* The same fused step for callers that cannot allocate: no counterpart in the reference.
 *
 * vb_multi_tensor_step builds its chunk table in device and pinned host memory that it
 * allocates, and re-allocates when a larger tensor list arrives.  A host that has given all
 * device memory to its own pool, that must keep the allocator's locks out of its training
 * loop, or that forbids allocation after start-up cannot make that call.  This entry point
 * performs no cudaMalloc, cudaHostAlloc, cudaFree or any other allocating call: the chunk
 * table lives in a fixed 384 KiB device array that is part of the library image (every GPU
 * that loads the library holds it until the process exits) and is staged through an equally
 * fixed host array.  Arguments, arithmetic and results are those of vb_multi_tensor_step.
 *
 * Limits and rules that follow from the fixed array:
 *  - at most 8192 chunks: n_tensors <= 8192, and the list must fit in 8192 pieces of at most
 *    131072 elements (about 1.07e9 elements for large tensors; fewer for many ragged ones).
 *    Anything larger returns VB_ERR_UNSUPPORTED with a message that says so;
 *  - all calls on one device share the array and it keeps the last call's table.  The part a
 *    call uses is rewritten by that call (nothing in it must start at zero).  Calls issued on
 *    one engine are ordered by its stream; calls from different engines or streams that
 *    overlap on the GPU race on the table and must be serialised by the caller;
 *  - the host array the table is staged through is one per process, shared by all devices and
 *    host threads; the library holds a lock while it fills the array and hands it to the copy,
 *    so concurrent callers on different devices are safe on the host side (they serialise);
 *  - the first call on a device also looks up the array's device address; make that first
 *    call before any stream capture begins. */
int vb_multi_tensor_step_static(vb_engine *engine, const vb_optimizer_step_params *hp,
                                int64_t n_tensors, const int64_t *sizes, void *const *params,
                                const void *const *grads, void *const *state1,
                                void *const *state2);

#ifdef __cplusplus
}
#endif
#endif /* VOLTA_B200_H */
