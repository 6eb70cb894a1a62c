#!/usr/bin/env python
"""Benchmark of the optimizer-step hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one optimizer step() over the whole parameter set of the workload with
the gradients already resident in HBM.  Headline workload: Adam (weight decay 0.01) on
the 12-layer d=768 transformer parameter set, 109 602 816 f32 parameters (28 B/param of
HBM traffic).  Rank 0 prints ONE JSON line.

N > 1 is launched by torch.distributed.run, one rank per GPU: the arena is sharded
ZeRO-1 style (each rank updates arena/N elements) and step() ends with the NCCL
all-gather of updated parameters, so `value` is total params / (update + gather) time.

`--impl reference` times the CPU restatement of Volta's own optimizer (oracle/) on the
host cores on the same workload; Volta is single threaded by construction, so it uses
one core.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import workloads  # noqa: E402

ADAM_BYTES_PER_PARAM = 28  # read theta, g, m, v (16) + write theta, m, v (12)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        deadline = time.time() + 10.0  # nvidia-smi takes a moment to print its first sample
        while not self.rows and time.time() < deadline:
            time.sleep(0.02)
        self.rows.clear()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()  # the exact child we started
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": len(self.rows)}
        if not self.rows:
            return out
        sm = []
        reasons = set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                out["sm_max_mhz"] = float(r[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # "under load": the upper half of the samples (idle samples sit at low clocks)
        if sm:
            sm.sort()
            out["sm_mhz"] = statistics.median(sm[len(sm) // 2:])
        out["reasons"] = sorted(reasons)
        return out


def fill_arena(wl, offsets, arena, arrays):
    host = np.zeros(arena, np.float32)
    for o, a in zip(offsets, arrays):
        host[o:o + a.size] = a.reshape(-1)
    return host


# ---------------------------------------------------------------------------------------------
# CPU arm: the restatement of Volta's CPU optimizer, one thread (Volta is single threaded)
# ---------------------------------------------------------------------------------------------

def time_cpu_adam(wl, steps, warmup, max_seconds=25.0):
    import oracle
    oracle.build()
    oracle.set_threads(1)
    params = wl.make_params()
    grads = wl.make_grads(1)
    h = wl.hyper
    opt = oracle.Adam(params, h["lr"], h["betas"], h["eps"], h["weight_decay"])
    for _ in range(warmup):
        opt.step(grads)
    times = []
    t_begin = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        opt.step(grads)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > max_seconds:
            break
    return times


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    wl = workloads.c3_transformer_adam()
    times = time_cpu_adam(wl, args.steps, min(args.warmup, 1), max_seconds=120.0)
    sec = sum(times) / len(times)
    value = wl.total / sec
    cores = 1
    line = {
        "impl": "reference", "metric": "adam_params_per_s", "value": value, "unit": "params/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": C3_WORKLOAD,
                   "host_cores_available": os.cpu_count()},
        "cpu_baseline": {"value": value, "unit": "params/s", "cores": cores, "kind": "port",
                         "sample": f"{len(times)} full steps of the whole workload, 1 thread "
                                   "(Volta's optimizer is single threaded)"},
        "e2e": {"value": value, "unit": "params/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

C3_WORKLOAD = ("c3_transformer_adam: Adam lr=1e-3 betas=(0.9,0.999) eps=1e-8 wd=0.01, 157 tensors, "
               "109602816 f32 params")


def bind_near_gpu(local_rank: int):
    """Runs this rank on the CPUs of its GPU's NUMA node, so that the pinned host buffers it allocates
    afterwards (first touch) and its copy threads sit next to the GPU's PCIe root.  Best effort: returns
    the node, or None where the topology is not exposed."""
    try:
        import torch
        pr = torch.cuda.get_device_properties(local_rank)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf.lower()}/numa_node").read().strip())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except (OSError, ValueError, AttributeError, TypeError):
        return None


def gather_handles(mine: bytes, world: int, dev):
    """Every rank's 64-byte CUDA IPC handle, in rank order (torch.distributed is the transport)."""
    import torch
    t = torch.frombuffer(bytearray(mine), dtype=torch.uint8).to(dev)
    allh = torch.zeros(world * 64, dtype=torch.uint8, device=dev)
    torch.distributed.all_gather_into_tensor(allh, t)
    blob = allh.cpu().numpy().tobytes()
    return [blob[r * 64:(r + 1) * 64] for r in range(world)]


def run_ours(args):
    import torch
    import torch.distributed as dist

    import volta_b200
    from volta_b200 import VB_STEP_NO_EXCHANGE, Adam, Engine, PinnedBuffer, Tensor

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa_node = bind_near_gpu(local_rank) if world > 1 else None
    eng = Engine(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        idt = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            idt.copy_(torch.frombuffer(bytearray(Engine.unique_id()), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        eng.init_comm(bytes(idt.cpu().numpy().tobytes()), rank, world)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        eng.synchronize()

    peaks = load_peaks()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.only_muon:
        muon = run_muon(args, eng, world, rank, dev, barrier, max_over_ranks, peaks)
        if rank == 0:
            print(json.dumps({"metric": "muon_ns_tflops", "muon": muon}), flush=True)
        return 0

    wl = workloads.c3_transformer_adam()
    h = wl.hyper
    params = wl.make_params()
    tensors = [Tensor(p, p.shape) for p in params]
    opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=eng)
    if world > 1 and args.exchange == "peer":
        opt.open_peers(gather_handles(opt.ipc_handle(), world, dev))
    _, _, arena, offsets = opt.arena_layout()
    grads_pinned = PinnedBuffer(arena)
    grads_pinned.array[:] = fill_arena(wl, offsets, arena, wl.make_grads(1))
    params_pinned = PinnedBuffer(arena)
    opt.upload_arena(1, grads_pinned.array)
    eng.synchronize()

    stream = torch.cuda.ExternalStream(eng.stream, device=dev)

    def timed_steps(n, flags=0, per_step=False):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
        evs[0].record(stream)
        for i in range(n):
            opt.step(flags)
            if per_step or i == n - 1:
                evs[i + 1].record(stream)
        eng.synchronize()
        total = evs[0].elapsed_time(evs[n])
        steps_ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(n)] if per_step else None
        return total, steps_ms

    # ---- device-resident timing: W warm-up steps, then exactly K steps ----
    for _ in range(args.warmup):
        opt.step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = eng.launch_count
    barrier()
    total_ms, _ = timed_steps(args.steps)
    barrier()
    launches = eng.launch_count - launches0

    # the update kernel alone (no exchange), per-launch durations, for the roofline
    barrier()
    _, kernel_ms = timed_steps(args.steps, VB_STEP_NO_EXCHANGE, per_step=True)
    barrier()
    clocks = sampler.stop() if rank == 0 else None

    total_ms = max_over_ranks(total_ms)
    kernel_avg_ms = max_over_ranks(sum(kernel_ms) / len(kernel_ms))
    ms_per_step = total_ms / args.steps
    value = wl.total / (ms_per_step * 1e-3)

    # ---- end to end through the public API with host buffers ----
    e2e_steps = 0 if args.skip_e2e else max(3, min(args.steps, 10))
    barrier()
    t0 = time.perf_counter()
    # One public call per step: gradients up from pinned host memory, update, parameters back down
    # (blocks until they are in host memory).  N > 1: a rank moves only its own slice over PCIe
    # (what a reduce-scatter would hand it, and the parameters it updated).
    for _ in range(e2e_steps):
        opt.step_host(grads_pinned.array, params_pinned.array, pieces=max(4, 32 // world))  # ~14 MB per piece
    barrier()
    e2e_s = max_over_ranks((time.perf_counter() - t0) / max(e2e_steps, 1))

    # ---- N > 1: data-parallel step, the reduce-scatter of gradients fused into the kernel's loads ----
    # (These extra sections must never cost the headline: a library error in one of them, which every
    # rank would raise at the same call, is recorded instead of ending the run.)
    dp_step = None
    if world > 1 and args.exchange == "peer":
        try:
            from volta_b200 import VB_STEP_MEAN_GRADS
            opt.open_peers_grads(gather_handles(opt.ipc_handle_grads(), world, dev))
            for _ in range(3):
                opt.step(VB_STEP_MEAN_GRADS)
            barrier()
            dp_ms, _ = timed_steps(args.steps, VB_STEP_MEAN_GRADS)
            barrier()
            dp_ms = max_over_ranks(dp_ms) / args.steps
            dp_step = {"value": wl.total / (dp_ms * 1e-3), "unit": "params/s", "ms_per_step": dp_ms,
                       "note": "step(VB_STEP_MEAN_GRADS): every rank holds its own gradient of the whole model; the "
                               "owner's update kernel reads all ranks' gradients over NVLink, adds them in rank "
                               "order, updates and stores the new parameters to every rank (reduce-scatter + Adam + "
                               "all-gather in one kernel)"}
        except volta_b200.VoltaB200Error as exc:
            dp_step = {"error": str(exc)}

    # ---- N > 1: the same step exchanging bf16 copies of the parameters instead of f32 ----
    bf16_exchange = None
    if world > 1:
        try:
            from volta_b200 import VB_STEP_EXCHANGE_BF16
            opt.enable_bf16_params()
            if args.exchange == "peer":
                opt.open_peers_bf16(gather_handles(opt.ipc_handle_bf16(), world, dev))
            for _ in range(3):
                opt.step(VB_STEP_EXCHANGE_BF16)
            barrier()
            half_ms, _ = timed_steps(args.steps, VB_STEP_EXCHANGE_BF16)
            barrier()
            half_ms = max_over_ranks(half_ms) / args.steps
            bf16_exchange = {"value": wl.total / (half_ms * 1e-3), "unit": "params/s", "ms_per_step": half_ms,
                             "note": "step(VB_STEP_EXCHANGE_BF16): the update kernel also writes bf16 copies of the "
                                     "new parameters and only those cross NVLink (2 B/param instead of 4); f32 "
                                     "masters stay exact on their owners"}
        except volta_b200.VoltaB200Error as exc:
            bf16_exchange = {"error": str(exc)}

    opt.close()
    grads_pinned.free()
    params_pinned.free()
    del params, tensors

    # ---- Muon (second headline: Newton-Schulz tensor TFLOP/s), on every rank ----
    muon = None if args.skip_muon else run_muon(args, eng, world, rank, dev, barrier, max_over_ranks, peaks)

    c5 = None if args.skip_c5 else run_c5(args, eng, world, rank, dev, barrier, max_over_ranks, peaks)

    if rank != 0:
        return 0

    achieved_gbs = ADAM_BYTES_PER_PARAM * (wl.total / world) / (kernel_avg_ms * 1e-3) / 1e9
    line = {
        "metric": "adam_params_per_s", "value": value, "unit": "params/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": C3_WORKLOAD,
                   "l2": "inputs larger than L2 (1.75 GB of theta/g/m/v per step vs 126 MB)",
                   "parallelism": f"zero1x{world}" if world > 1 else "single",
                   "exchange": ("none" if world == 1 else
                                "peer stores over NVLink fused into the update kernel, fenced by two one-float "
                                "NCCL all-reduces" if args.exchange == "peer" else
                                "nccl all-gather of updated params after the update kernel")},
        "update_only": {"value": wl.total / (kernel_avg_ms * 1e-3), "unit": "params/s",
                        "ms_per_step": kernel_avg_ms,
                        "note": "fused update kernel alone, max over ranks"},
        "roofline": {"bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved_gbs / peaks["hbm_gbs"], "traffic": None,
                     "peak_source": peaks["source"], "frac_of_nominal_8tbs": achieved_gbs / 8000.0,
                     "kernel": "multi_tensor_update_kernel<ADAM>",
                     "algorithmic_bytes_per_launch": ADAM_BYTES_PER_PARAM * (wl.total // world),
                     "launch_ms": kernel_avg_ms},
        "e2e": {"value": wl.total / e2e_s, "unit": "params/s", "h2d_bytes_per_step": arena * 4,
                "d2h_bytes_per_step": arena * 4, "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                "note": "bytes are totals over all ranks; each rank moves its own 1/N slice of the arena",
                "rank0_numa_node": numa_node},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    line["roofline"]["traffic"] = traffic_from_profile()

    if world == 1 and not args.no_cpu_baseline:
        times = time_cpu_adam(wl, 12, 1, max_seconds=20.0)
        sec = sum(times) / len(times)
        line["cpu_baseline"] = {"value": wl.total / sec, "unit": "params/s", "cores": 1, "kind": "port",
                                "sample": f"{len(times)} full steps of the same workload, 1 thread of "
                                          f"{os.cpu_count()} host cores (Volta's optimizer is single threaded)",
                                "ms_per_step": sec * 1e3}
    if world > 1:
        # Every rank must receive the (N-1)/N of the updated parameters it does not own: NVLink
        # ingress bounds the whole step whatever the update costs.  770 GB/s is the peer-copy rate
        # measured per direction per GPU on this pool (900 nominal).
        ingress = 4.0 * wl.total * (world - 1) / world
        floor_ms = ingress / 770e9 * 1e3
        line["exchange_roofline"] = {"bound": "nvlink ingress per GPU", "bytes_in_per_gpu": ingress, "peak": 770.0,
                                     "unit": "GB/s", "floor_ms": floor_ms,
                                     "achieved": ingress / (ms_per_step * 1e-3) / 1e9,
                                     "frac": floor_ms / ms_per_step,
                                     "note": "strong scaling of the whole step is capped by this floor; the update "
                                             "kernel itself scales with 1/N (update_only)"}
    if dp_step is not None:
        line["data_parallel_step"] = dp_step
    if bf16_exchange is not None:
        line["bf16_exchange"] = bf16_exchange
    if muon is not None:
        line["muon"] = muon
    if c5 is not None:
        line["c5_ragged_adam"] = c5
    print(json.dumps(line), flush=True)
    return 0


def run_c5(args, eng, world, rank, dev, barrier, max_over_ranks, peaks):
    """Ragged multi-tensor Adam (4096 tensors, sizes log-uniform in [1, 2^22], ~1.13e9 params):
    the same kernel must hold its HBM fraction when the tensor list is ragged."""
    import torch

    from volta_b200 import VB_STEP_NO_EXCHANGE, Adam, Tensor
    from volta_b200.interop import device_array

    wl = workloads.c5_ragged_adam()
    h = wl.hyper
    tensors = [Tensor(np.zeros(n, np.float32)) for n in wl.sizes]
    opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=eng)
    p_ptr, g_ptr, arena, offsets = opt.arena_layout()
    theta = torch.as_tensor(device_array(p_ptr, arena, opt), device=dev)
    grad = torch.as_tensor(device_array(g_ptr, arena, opt), device=dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234)
    theta.normal_(0.0, 1.0, generator=gen)
    grad.normal_(0.0, 1e-3, generator=gen)
    opt.mark_all_grads_present()
    torch.cuda.synchronize()
    steps = max(3, min(args.steps, 10))
    for _ in range(3):
        opt.step(VB_STEP_NO_EXCHANGE)
    barrier()
    eng.set_profiling(True)
    eng.profile("update")
    for _ in range(steps):
        opt.step(VB_STEP_NO_EXCHANGE)
    ms = max_over_ranks(eng.profile("update")[0] / steps)
    eng.set_profiling(False)
    barrier()
    del theta, grad
    opt.close()
    gbs = ADAM_BYTES_PER_PARAM * (wl.total / world) / (ms * 1e-3) / 1e9
    return {"workload": f"c5_ragged_adam: {len(wl.sizes)} tensors, {wl.total} f32 params, sizes in "
                        f"[{min(wl.sizes)}, {max(wl.sizes)}], lr=3e-4 wd=0.1", "steps": steps,
            "update_ms_per_step": ms, "params_per_s": wl.total / (ms * 1e-3), "achieved_gbs_per_gpu": gbs,
            "frac_of_measured_hbm_peak": gbs / peaks["hbm_gbs"], "note": "update kernel only (no exchange)"}


def time_cpu_muon_sample(ns_steps=5):
    """Oracle Muon step on one 1024 x 1024 matrix, one thread; returns (seconds, flops)."""
    import oracle
    oracle.build()
    oracle.set_threads(1)
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((1024, 1024)) * 0.02).astype(np.float32)
    g = (rng.standard_normal((1024, 1024)) * 1e-3).astype(np.float32)
    opt = oracle.Muon([w], 0.1, 0.9, True, ns_steps)
    t0 = time.perf_counter()
    opt.step([g])
    return time.perf_counter() - t0, 4.0 * 1024 ** 3 * ns_steps


def run_muon(args, eng, world, rank, dev, barrier, max_over_ranks, peaks):
    """Muon on the 96 matrices of the 24-layer d=1024 configuration: NS TFLOP/s."""
    import torch

    from volta_b200 import VB_NS_BF16, VB_NS_F32, VB_NS_F32_TC, Muon, Tensor

    wl = workloads.c4_muon(layers=args.muon_layers)
    h = wl.hyper
    params = wl.make_params()
    grads = wl.make_grads(1)
    out = {}
    for mode_name, mode, steps in (("bf16", VB_NS_BF16, max(3, min(args.steps, 20))),
                                   ("f32_tc", VB_NS_F32_TC, max(3, min(args.steps, 5))), ("f32", VB_NS_F32, 2)):
        if mode_name == "f32" and (args.skip_muon_f32 or (args.only_muon and not args.muon_f32)):
            continue
        if mode_name == "f32_tc" and args.only_muon and not args.muon_f32_tc:
            continue
        tensors = [Tensor(p, p.shape) for p in params]
        opt = Muon(tensors, h["lr"], h["momentum"], h["nesterov"], h["ns_steps"], ns_mode=mode, engine=eng)
        if world > 1 and args.exchange == "peer":
            opt.open_peers(gather_handles(opt.ipc_handle(), world, dev))
        _, _, arena, offsets = opt.arena_layout()
        host = fill_arena(wl, offsets, arena, grads)
        opt.upload_arena(1, host)
        del host
        eng.synchronize()
        warm = 1 if mode_name == "f32" else 3
        for _ in range(warm):
            opt.step()
        barrier()
        eng.set_profiling(True)
        for ph in ("muon_pre", "muon_ns", "muon_apply", "exchange"):
            eng.profile(ph)
        stream = torch.cuda.ExternalStream(eng.stream, device=dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = eng.launch_count
        sampler = ClockSampler(dev.index) if rank == 0 and mode_name == "bf16" else None
        if sampler is not None:
            sampler.start()
        barrier()
        e0.record(stream)
        for _ in range(steps):
            opt.step()
        e1.record(stream)
        eng.synchronize()
        barrier()
        muon_clocks = sampler.stop() if sampler is not None else None
        step_ms = max_over_ranks(e0.elapsed_time(e1) / steps)
        ns_ms = max_over_ranks(eng.profile("muon_ns")[0] / steps)
        pre_ms = eng.profile("muon_pre")[0] / steps
        apply_ms = eng.profile("muon_apply")[0] / steps
        exch_ms = eng.profile("exchange")[0] / steps
        eng.set_profiling(False)
        flops_rank = opt.last_ns_flops
        if world > 1:
            t = torch.tensor([flops_rank], dtype=torch.float64, device=dev)
            torch.distributed.all_reduce(t)
            flops_total = float(t.item())
        else:
            flops_total = flops_rank
        tflops = flops_total / (ns_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops_sustained"] * world
        out[mode_name] = {
            "ns_tflops": tflops, "ns_ms_per_step": ns_ms, "ms_per_step": step_ms,
            "pre_ms": pre_ms, "apply_ms": apply_ms, "exchange_ms": exch_ms,
            "params_per_s": wl.total / (step_ms * 1e-3), "steps": steps,
            "executed_flops_per_step": flops_total,
            "note": {"bf16": "tcgen05 bf16, short-side Gram, symmetric Gram computed on and above the diagonal only", "f32": "CUDA-core FFMA, bit-identical to the CPU arithmetic",
                     "f32_tc": "tcgen05, operands held as two f16 planes (three products per product); "
                               "ns_tflops counts executed f16 tensor FLOPs"}[mode_name],
            "reference_formulation_flops_per_step": sum(4.0 * r * c * c * h["ns_steps"] for r, c in wl.shapes),
            "gpu_launches": int(eng.launch_count - launches0),
        }
        if muon_clocks is not None:
            out[mode_name]["clocks"] = muon_clocks
        if mode_name == "bf16" and world > 1:
            from volta_b200 import VB_STEP_EXCHANGE_BF16
            opt.enable_bf16_params()
            if args.exchange == "peer":
                opt.open_peers_bf16(gather_handles(opt.ipc_handle_bf16(), world, dev))
            for _ in range(2):
                opt.step(VB_STEP_EXCHANGE_BF16)
            barrier()
            e0.record(stream)
            for _ in range(steps):
                opt.step(VB_STEP_EXCHANGE_BF16)
            e1.record(stream)
            eng.synchronize()
            barrier()
            half_ms = max_over_ranks(e0.elapsed_time(e1) / steps)
            out[mode_name]["bf16_exchange"] = {"ms_per_step": half_ms, "params_per_s": wl.total / (half_ms * 1e-3),
                                               "note": "step(VB_STEP_EXCHANGE_BF16): owners send bf16 copies only"}
        if mode_name == "bf16":
            out[mode_name]["roofline"] = {
                "bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
                "peak_source": peaks["source"] + " (cuBLAS bf16 sustained)",
                "frac_of_burst_peak": tflops / (peaks["bf16_tflops"] * world),
                "frac_of_nominal_2250": tflops / (2250.0 * world),
                "traffic": NCU_MUON_4LAYER_DRAM_BYTES_PER_LAUNCH * args.muon_layers / 4.0 / world,
                "traffic_note": "ncu capture of the 4-layer case (mean of a Gram and an update launch), scaled by "
                                "layers / 4: per-launch traffic grows with the number of matrices",
                "kernel": "ns_gemm_tc_kernel (tcgen05 bf16, 10 launches per step)"}
        opt.close()
    out["config"] = {"workload": f"c4_muon: {len(wl.shapes)} matrices ({args.muon_layers} x {{3072x1024, 1024x1024, "
                                 f"4096x1024, 1024x4096}}), {wl.total} f32 params, lr=0.1 momentum=0.9 nesterov "
                                 "ns_steps=5"}
    if world == 1 and not args.no_cpu_baseline and "bf16" in out:
        sec, fl = time_cpu_muon_sample(h["ns_steps"])
        ref_flops = out["bf16"]["reference_formulation_flops_per_step"]
        out["cpu_baseline"] = {"value": fl / sec / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
                               "sample": "one Muon step of one 1024x1024 matrix (21.5 GFLOP), 1 thread; a whole "
                                         f"step of the workload is {ref_flops / 1e12:.2f} TFLOP in the reference's "
                                         f"formulation, i.e. ~{ref_flops / fl * sec:.0f} s at this rate (extrapolated)"}
    return out



# dram__bytes_read.sum + dram__bytes_write.sum per launch of multi_tensor_update_kernel<ADAM>
# on this workload, from the ncu capture summarised in profiles/adam_c3_multi_tensor_update.md
NCU_ADAM_C3_DRAM_BYTES_PER_LAUNCH = 3.0164e9


# dram__bytes_read.sum + dram__bytes_write.sum per launch of ns_gemm_tc_kernel<2, 0> on 4 layers of the Muon
# workload (16 matrices): mean of a Gram launch (110.4 MB) and an update launch (206.8 MB), from the ncu
# capture summarised in profiles/muon_c4_ns_gemm_tc.md
NCU_MUON_4LAYER_DRAM_BYTES_PER_LAUNCH = 158.6e6


def traffic_from_profile():
    return NCU_ADAM_C3_DRAM_BYTES_PER_LAUNCH


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: device-resident timing only")
    ap.add_argument("--skip-muon", action="store_true", help="Adam only")
    ap.add_argument("--skip-muon-f32", action="store_true", help="skip the (slow) f32 Newton-Schulz timing")
    ap.add_argument("--only-muon", action="store_true", help="profiling runs: Muon bf16 only")
    ap.add_argument("--skip-c5", action="store_true", help="skip the ragged 4096-tensor Adam section")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: updated parameters reach the other ranks by NVLink peer stores fused into the "
                         "update kernel (default) or by an NCCL all-gather after it")
    ap.add_argument("--muon-f32-tc", action="store_true", help="with --only-muon: also time the f32-accurate TC path")
    ap.add_argument("--muon-f32", action="store_true", help="with --only-muon: also time the bit-faithful f32 path")
    ap.add_argument("--muon-layers", type=int, default=24, help="profiling runs: fewer layers of the Muon set")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
