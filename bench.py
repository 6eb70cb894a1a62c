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
import datetime
import json
import math
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
C3_WORKLOAD = ("c3_transformer_adam: Adam lr=1e-3 betas=(0.9,0.999) eps=1e-8 wd=0.01, 157 tensors, "
               "109602816 f32 params")
MIN_TIMED_SECONDS = 0.5   # every headline number is the median of K-step blocks that together run at least this long


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
                 "-i", str(self.gpu_index), "-lms", "10"],
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


def bench_config(n_gpus: int):
    """The workload description both arms print (identical for the same N)."""
    return {"workload": C3_WORKLOAD,
            "inputs_vs_l2": "inputs larger than L2 (1.75 GB of theta/g/m/v per step vs 126 MB): no flush needed",
            "sharding": "single GPU" if n_gpus == 1 else f"parameter arena sharded by ownership over {n_gpus} ranks (ZeRO-1), one rank per GPU"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    wl = workloads.c3_transformer_adam()
    times = time_cpu_adam(wl, args.steps, args.warmup, max_seconds=240.0)
    sec = sum(times) / len(times)
    value = wl.total / sec
    cores = 1
    line = {
        "impl": "reference", "metric": "adam_params_per_s", "value": value, "unit": "params/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": bench_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "params/s", "cores": cores, "kind": "port",
                         "host_cores_available": os.cpu_count(),
                         "sample": f"{len(times)} full steps of the whole workload, 1 thread "
                                   "(Volta's optimizer is single threaded: Tensor = Rc<RefCell<_>>)"},
        "e2e": {"value": value, "unit": "params/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

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


def timed_blocks(run_block, barrier, max_over_ranks, min_seconds=MIN_TIMED_SECONDS, max_blocks=400):
    """Runs `run_block()` (which enqueues one K-step block and returns its device milliseconds after
    waiting for it) again and again, each block between a barrier + synchronize on both sides, until
    the blocks together cover `min_seconds`.  Every rank runs the same number of blocks (decided from
    the first block's max-over-ranks time).  Returns the per-block times, max over ranks."""
    min_seconds = min(min_seconds, timed_blocks.cap_seconds)
    barrier()
    mine = [run_block()]
    first = max_over_ranks(mine[0])
    barrier()
    n = int(min(max_blocks, max(3, math.ceil(min_seconds * 1e3 / max(first, 1e-3)))))
    out = [first]
    for _ in range(n - 1):
        ms = run_block()
        barrier()
        mine.append(ms)
        out.append(max_over_ranks(ms))
    timed_blocks.last_local = mine   # this rank's own times of the same blocks
    return out


timed_blocks.cap_seconds = MIN_TIMED_SECONDS   # lowered by --min-seconds


def block_stats(blocks_ms, steps):
    return {"count": len(blocks_ms), "steps_per_block": steps, "median_ms": statistics.median(blocks_ms),
            "min_ms": min(blocks_ms), "max_ms": max(blocks_ms), "timed_seconds": sum(blocks_ms) * 1e-3}


def run_parity(eng, world, rank, dev, exchange):
    """Outside every timed region: small Adam, SGD and Muon workloads sharded over all ranks with the
    benchmark's exchange, three steps each; rank 0 runs the CPU oracle and every rank compares its WHOLE
    parameter set with it.  Returns the `parity` object; any mismatch makes the run exit non-zero."""
    import torch
    import torch.distributed as dist

    import oracle
    import volta_b200
    from volta_b200 import SGD, VB_NS_BF16, VB_NS_F32, Adam, Muon, Tensor

    muon_shapes = [(256, 128), (128, 384), (64, 36), (100,), (512, 256), (256, 256), (384, 384), (128, 512),
                   (768, 256), (3, 3)]
    muon_wl = workloads.Workload("muon_parity", "muon", muon_shapes, [("normal", 0.02)] * len(muon_shapes), 1e-3,
                                 dict(lr=0.1, momentum=0.9, nesterov=True, ns_steps=5), 3)
    cases = [("adam", workloads.c5_ragged_adam(n_tensors=96, max_log2=16, seed=11), None),
             ("sgd", workloads.c2_cnn_sgd(), None),
             ("muon_f32", muon_wl, VB_NS_F32), ("muon_bf16", muon_wl, VB_NS_BF16)]
    if world > 1:  # the same Adam list with 45 % of the arena updated by every rank itself instead of exchanged
        cases.insert(1, ("adam_replicated_tail", workloads.c5_ragged_adam(n_tensors=96, max_log2=16, seed=11), None))
    out = {"n_ranks": world, "steps": 3, "exchange": exchange if world > 1 else "none"}
    all_equal = True
    for name, wl, mode in cases:
        h = wl.hyper
        tensors = [Tensor(p, p.shape) for p in wl.make_params()]
        if name.startswith("adam"):
            eng.set_replicated_fraction(0.45 if name == "adam_replicated_tail" else 0.0)
            opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=eng)
            eng.set_replicated_fraction(0.0)
        elif name == "sgd":
            opt = SGD(tensors, h["lr"], h["momentum"], h["weight_decay"], engine=eng)
        else:
            opt = Muon(tensors, h["lr"], h["momentum"], h["nesterov"], h["ns_steps"], ns_mode=mode, engine=eng)
        if world > 1:
            fps = torch.zeros(world, dtype=torch.int64, device=dev)
            mine = torch.tensor([opt.plan_fingerprint() & 0x7fffffffffffffff], dtype=torch.int64, device=dev)
            dist.all_gather_into_tensor(fps, mine)
            volta_b200.verify_plan([int(x) for x in fps.cpu().tolist()])   # all ranks describe the same optimizer
            if exchange == "peer":
                opt.open_peers(gather_handles(opt.ipc_handle(), world, dev))
        for s in (1, 2, 3):
            opt.zero_grad()
            for t, g in zip(tensors, wl.make_grads(s)):
                t.grad = g
            opt.step()
        eng.synchronize()
        got = np.concatenate([t.data.reshape(-1) for t in tensors])
        opt.close()
        # the oracle's result, computed once on rank 0 and handed to every rank
        want = torch.zeros(got.size, dtype=torch.float32, device=dev)
        if rank == 0:
            oracle.build()
            ref = wl.make_params()
            if name.startswith("adam"):
                o = oracle.Adam(ref, h["lr"], h["betas"], h["eps"], h["weight_decay"])
            elif name == "sgd":
                o = oracle.SGD(ref, h["lr"], h["momentum"], h["weight_decay"])
            else:
                o = oracle.Muon(ref, h["lr"], h["momentum"], h["nesterov"], h["ns_steps"])
            for s in (1, 2, 3):
                o.step(wl.make_grads(s))
            want.copy_(torch.from_numpy(np.concatenate([r.reshape(-1) for r in ref])))
        if world > 1:
            dist.broadcast(want, 0)
        want = want.cpu().numpy()
        exact = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
        # parameters moved by lr * 0.1 * update per step: relate the difference to the distance travelled
        start = np.concatenate([p.reshape(-1) for p in wl.make_params()])
        rel = float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want.astype(np.float64) - start), 1e-300))
        digest = int(np.bitwise_xor.reduce(got.view(np.uint32).astype(np.uint64) * np.uint64(0x9E3779B97F4A7C15)
                                           + np.arange(got.size, dtype=np.uint64)) & np.uint64(0x7fffffffffffffff))
        stats = torch.tensor([1.0 if exact else 0.0, -rel], dtype=torch.float64, device=dev)
        dig = torch.tensor([digest], dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(stats, op=dist.ReduceOp.MIN)   # all ranks exact; the largest relative error
            digs = torch.zeros(world, dtype=torch.int64, device=dev)
            dist.all_gather_into_tensor(digs, dig)
            all_equal = all_equal and len(set(digs.cpu().tolist())) == 1
        if name == "muon_bf16":
            out["muon_bf16_rel_fro_max"] = -float(stats[1].item())
        else:
            out[f"{name}_bit_identical"] = bool(stats[0].item() == 1.0)
    out["all_ranks_equal"] = all_equal
    out["ok"] = bool(out["adam_bit_identical"] and out["sgd_bit_identical"] and out["muon_f32_bit_identical"]
                     and out.get("adam_replicated_tail_bit_identical", True)
                     and out["muon_bf16_rel_fro_max"] <= 2e-2 and all_equal)
    return out


def pcie_floor(opt, grads_pinned, params_pinned, dev, barrier, max_over_ranks, reps=5):
    """Plain pinned copies of this rank's slice up (gradients) and down (parameters), issued together on two
    streams by all ranks at once, no kernel: what the host side gives one end-to-end step."""
    import torch

    from volta_b200.interop import device_array
    p_ptr, g_ptr, arena, _ = opt.arena_layout()
    lo, hi = opt.owned_range()
    theta = torch.as_tensor(device_array(p_ptr, arena, opt), device=dev)
    grad = torch.as_tensor(device_array(g_ptr, arena, opt), device=dev)
    host_g = torch.from_numpy(grads_pinned.array)
    host_p = torch.from_numpy(params_pinned.array)
    up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    times = []
    for _ in range(reps):
        barrier()
        t0 = time.perf_counter()
        with torch.cuda.stream(up):
            grad[lo:hi].copy_(host_g[lo:hi], non_blocking=True)
        with torch.cuda.stream(down):
            host_p[lo:hi].copy_(theta[lo:hi], non_blocking=True)
        up.synchronize()
        down.synchronize()
        times.append(time.perf_counter() - t0)
    barrier()
    del theta, grad
    return max_over_ranks(statistics.median(times)) * 1e3, bool(host_g.is_pinned())


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
    numa_node = bind_near_gpu(local_rank)
    cpu_set = sorted(os.sched_getaffinity(0))
    eng = Engine(local_rank)
    if world > 1:
        # a rank that fails must not leave the others waiting in a collective for the default ten minutes
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
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

    # ---- parity first (outside every timed region): all ranks against the CPU oracle ----
    parity = None if args.skip_parity else run_parity(eng, world, rank, dev, args.exchange)
    if parity is not None and not parity["ok"]:
        if rank == 0:
            print(json.dumps({"metric": "adam_params_per_s", "value": None, "n_gpus": world, "parity": parity,
                              "error": "parity against the CPU oracle failed; nothing was timed"}), flush=True)
        return 3

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
    params0_pinned = PinnedBuffer(arena)
    opt.download_arena(0, params0_pinned.array)

    def restart(o=None):
        """Back to the start of the configuration (seeded parameters, zero moments, t = 0), outside every
        timed region.  The configuration is 50 steps; replaying one resident gradient for thousands of steps
        instead would train every parameter to the fixed point g + wd * theta = 0, where parameters' effective
        gradients and moments underflow -- values no 50-step run ever sees."""
        o = opt if o is None else o
        o.reset_state()
        o.upload_arena(0, params0_pinned.array)
        eng.synchronize()

    def make_block(flags=0, o=None):
        def run_block():
            target = opt if o is None else o
            restart(target)
            for _ in range(args.warmup):
                target.step(flags)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            lc0 = eng.launch_count
            e0.record(stream)
            for _ in range(args.steps):
                target.step(flags)
            e1.record(stream)
            eng.synchronize()
            timed_launches[0] += eng.launch_count - lc0
            return e0.elapsed_time(e1)
        return run_block

    timed_launches = [0]

    # ---- device-resident timing: W warm-up steps, then blocks of exactly K steps ----
    for _ in range(args.warmup):
        opt.step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    blocks = timed_blocks(make_block(0), barrier, max_over_ranks)
    launches = timed_launches[0]
    # the update kernel alone (no exchange): at N = 1 that is the same launch sequence
    if world > 1:
        kernel_blocks = timed_blocks(make_block(VB_STEP_NO_EXCHANGE), barrier, max_over_ranks, min_seconds=0.3)
    else:
        kernel_blocks = blocks
    per_rank_update_ms = [statistics.median(timed_blocks.last_local) / args.steps]

    # ---- N > 1: part of the arena replicated instead of exchanged ----
    # When everything is exchanged the step is bound by NVLink while HBM idles; with the last fraction f of
    # the arena updated by every rank itself the same launch mixes link-bound and HBM-bound chunks.  f comes
    # from the two rates just measured (vb_plan_replicated_fraction), the result must equal the plain one.
    tail = None
    if world > 1 and args.exchange == "peer" and args.replicated_fraction != 0.0:
        try:
            k_ms = statistics.median(kernel_blocks) / args.steps
            hbm_gbs = ADAM_BYTES_PER_PARAM * (wl.total / world) / (k_ms * 1e-3) / 1e9
            # the update launch with its peer stores, apart from the fences around it: a short profiled pass
            restart(opt)
            for _ in range(args.warmup):
                opt.step()
            barrier()
            eng.set_profiling(True)
            for ph in ("update", "exchange"):
                eng.profile(ph)
            for _ in range(args.steps):
                opt.step()
            eng.synchronize()
            upd_ms = max_over_ranks(eng.profile("update")[0] / args.steps)
            fence_ms = max_over_ranks(eng.profile("exchange")[0] / args.steps)
            eng.set_profiling(False)
            link_gbs = 4.0 * arena * (world - 1) / world / (upd_ms * 1e-3) / 1e9
            frac = args.replicated_fraction if args.replicated_fraction > 0.0 else \
                volta_b200.plan_replicated_fraction(ADAM_BYTES_PER_PARAM, world, hbm_gbs, link_gbs)
            ft = torch.tensor([frac], dtype=torch.float64, device=dev)
            dist.broadcast(ft, 0)    # one value on every rank
            frac = float(ft.item())
            def measure_tail(fr):
                eng.set_replicated_fraction(fr)
                tensors_t = [Tensor(p, p.shape) for p in params]
                opt_t = Adam(tensors_t, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=eng)
                eng.set_replicated_fraction(0.0)
                fps = torch.zeros(world, dtype=torch.int64, device=dev)
                dist.all_gather_into_tensor(fps, torch.tensor([opt_t.plan_fingerprint() & 0x7fffffffffffffff],
                                                              dtype=torch.int64, device=dev))
                volta_b200.verify_plan([int(x) for x in fps.cpu().tolist()])
                opt_t.open_peers(gather_handles(opt_t.ipc_handle(), world, dev))
                opt_t.upload_arena(1, grads_pinned.array)
                eng.synchronize()
                launches_before = timed_launches[0]
                t_blocks = timed_blocks(make_block(0, opt_t), barrier, max_over_ranks)
                t_launches = timed_launches[0] - launches_before
                timed_launches[0] = launches_before
                # same number of steps from the same start on both optimizers: the parameters must agree bit for bit
                restart(opt)
                restart(opt_t)
                for _ in range(args.steps):
                    opt.step()
                    opt_t.step()
                eng.synchronize()
                opt.download_arena(0, params_pinned.array)
                plain_bits = params_pinned.array.view(np.uint32).copy()
                opt_t.download_arena(0, params_pinned.array)
                same = bool(np.array_equal(plain_bits, params_pinned.array.view(np.uint32)))
                del plain_bits
                st = torch.tensor([1.0 if same else 0.0], dtype=torch.float64, device=dev)
                dist.all_reduce(st, op=dist.ReduceOp.MIN)
                t_lo, t_hi = opt_t.replicated_range()
                t_ms = statistics.median(t_blocks) / args.steps
                opt_t.close()
                del tensors_t
                return {"fraction": fr, "replicated_elements": t_hi - t_lo, "ms_per_step": t_ms,
                        "value": wl.total / (t_ms * 1e-3), "unit": "params/s",
                        "blocks": block_stats(t_blocks, args.steps), "launches": int(t_launches),
                        "equals_the_fully_exchanged_result_bit_for_bit": bool(st.item() == 1.0),
                        "extra_state_bytes_per_gpu": 8 * (t_hi - t_lo)}, t_blocks

            if frac > 0.0:
                # the model assumes the two kinds of traffic overlap perfectly; they do not quite, and the best
                # cut lies a little to either side of the model's (below at N = 2, above at N = 4): three
                # fractions around it are measured and the fastest kept
                candidates = [frac] if args.replicated_fraction > 0.0 else [frac, 0.8 * frac, min(1.15 * frac, 0.95)]
                tried = []
                for fr in candidates:
                    res, res_blocks = measure_tail(fr)
                    tried.append({"fraction": fr, "ms_per_step": res["ms_per_step"]})
                    if res["equals_the_fully_exchanged_result_bit_for_bit"] and \
                            (tail is None or res["ms_per_step"] < tail["ms_per_step"]):
                        tail, tail_blocks = res, res_blocks
                if tail is None:
                    tail, tail_blocks = res, res_blocks
                tail["fractions_tried"] = tried
                tail["rates_used"] = {"hbm_gbs": hbm_gbs, "nvlink_gbs_per_direction": link_gbs,
                                      "all_exchanged_update_launch_ms": upd_ms, "fences_ms_per_step": fence_ms,
                                      "model_fraction": frac,
                                      "how": "HBM: the update kernel alone on a slice (update_only); NVLink: bytes into "
                                             "a GPU over the duration of the update launch that stores every parameter "
                                             "to every peer (CUDA events around the launch, a separate pass)"}
                tail["note"] = ("the last `fraction` of the arena is updated by every rank itself (its moments live "
                                "on every rank; every rank holds the complete gradients) and never crosses NVLink; "
                                "the rest is sliced ZeRO-1 style and exchanged by the same launch")
        except volta_b200.VoltaB200Error as exc:
            tail = {"error": str(exc)}
            eng.set_replicated_fraction(0.0)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.zeros(world, dtype=torch.float64, device=dev)
        dist.all_gather_into_tensor(t, torch.tensor(per_rank_update_ms, dtype=torch.float64, device=dev))
        per_rank_update_ms = [float(x) for x in t.cpu().tolist()]

    ms_per_step = statistics.median(blocks) / args.steps
    kernel_avg_ms = statistics.median(kernel_blocks) / args.steps
    all_exchanged = None
    if tail is not None and tail.get("equals_the_fully_exchanged_result_bit_for_bit") and tail["ms_per_step"] < ms_per_step:
        # the headline is the faster of the two shardings of the same step; the other one stays in the line
        all_exchanged = {"ms_per_step": ms_per_step, "value": wl.total / (ms_per_step * 1e-3), "unit": "params/s",
                         "blocks": block_stats(blocks, args.steps),
                         "note": "plain ZeRO-1: every parameter is updated by one rank and sent to all others"}
        zero1_ms_per_step = ms_per_step
        ms_per_step = tail["ms_per_step"]
        headline_blocks = tail_blocks
        launches = tail["launches"]
    else:
        zero1_ms_per_step = ms_per_step
        headline_blocks = blocks
    value = wl.total / (ms_per_step * 1e-3)

    # ---- the fabric's own rate for the exchange, measured in this run (N > 1, peer exchange) ----
    nvlink = None
    if world > 1 and args.exchange == "peer":
        opt.peer_copy_probe(2)
        barrier()
        probe_ms = max_over_ranks(opt.peer_copy_probe(6))
        barrier()
        ingress = 4.0 * arena * (world - 1) / world
        nvlink = {"ms": probe_ms, "bytes_in_per_gpu": ingress, "gbs_in_per_gpu": ingress / (probe_ms * 1e-3) / 1e9,
                  "how": "every rank copies its slice of the parameter arena into every peer's arena with the copy "
                         "engines, all ranks at once, between the two halves of the exchange fence (6 repetitions)"}

    # ---- end to end through the public API with host buffers ----
    e2e = None
    if not args.skip_e2e:
        e2e_steps = args.steps
        pieces = max(4, 24 // world)   # ~18 MB per piece: 20-24 pieces measured best at N=1 (9.85 ms; 9.95 with 32, 10.3 with 12)
        restart()
        for _ in range(2):
            opt.step_host(grads_pinned.array, params_pinned.array, pieces=pieces)
        barrier()
        t0 = time.perf_counter()
        # One public call per step: gradients up from pinned host memory, update, parameters back down
        # (blocks until they are in host memory).  N > 1: a rank moves only its own slice over PCIe
        # (what a reduce-scatter would hand it, and the parameters it updated).
        for _ in range(e2e_steps):
            opt.step_host(grads_pinned.array, params_pinned.array, pieces=pieces)
        barrier()
        e2e_s = max_over_ranks((time.perf_counter() - t0) / e2e_steps)
        # phases of the same call (a separate short pass: the extra events are not in the number above)
        eng.set_profiling(True)
        for ph in ("host_h2d", "update", "host_d2h", "exchange"):
            eng.profile(ph)
        n_ph = 5
        for _ in range(n_ph):
            opt.step_host(grads_pinned.array, params_pinned.array, pieces=pieces)
        phases = {ph: max_over_ranks(eng.profile(ph)[0] / n_ph) for ph in ("host_h2d", "update", "host_d2h", "exchange")}
        eng.set_profiling(False)
        floor_ms, pinned_seen = pcie_floor(opt, grads_pinned, params_pinned, dev, barrier, max_over_ranks)
        e2e = {"value": wl.total / e2e_s, "unit": "params/s", "h2d_bytes_per_step": arena * 4,
               "d2h_bytes_per_step": arena * 4, "ms_per_step": e2e_s * 1e3, "steps": e2e_steps, "pieces": pieces,
               "phases_ms": {"h2d_span": phases["host_h2d"], "update_span": phases["update"],
                             "d2h_span": phases["host_d2h"], "fences": phases["exchange"],
                             "note": "device time from the first to the last operation of each of the three streams of "
                                     "one call (they overlap), max over ranks, from a separate 5-call pass"},
               "pcie_floor_ms": floor_ms,
               "pcie_floor_note": "plain pinned copies of every rank's slice up and down, issued together by all ranks, no "
                                  "kernel (median of 5, max over ranks); pinned memory recognised: " + str(pinned_seen),
               "frac_of_pcie_floor": floor_ms / (e2e_s * 1e3),
               "note": "bytes are totals over all ranks; each rank moves its own 1/N slice of the arena",
               "rank0_numa_node": numa_node, "rank0_cpus": f"{len(cpu_set)} CPUs {cpu_set[0]}-{cpu_set[-1]}"}

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
            dp_blocks = timed_blocks(make_block(VB_STEP_MEAN_GRADS), barrier, max_over_ranks, min_seconds=0.2)
            dp_ms = statistics.median(dp_blocks) / args.steps
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
            half_blocks = timed_blocks(make_block(VB_STEP_EXCHANGE_BF16), barrier, max_over_ranks, min_seconds=0.2)
            half_ms = statistics.median(half_blocks) / args.steps
            bf16_exchange = {"value": wl.total / (half_ms * 1e-3), "unit": "params/s", "ms_per_step": half_ms,
                             "note": "step(VB_STEP_EXCHANGE_BF16): the update kernel also writes bf16 copies of the "
                                     "new parameters and only those cross NVLink (2 B/param instead of 4); f32 "
                                     "masters stay exact on their owners"}
        except volta_b200.VoltaB200Error as exc:
            bf16_exchange = {"error": str(exc)}

    opt.close()
    grads_pinned.free()
    params_pinned.free()
    params0_pinned.free()
    del params, tensors

    # ---- Muon (second headline: Newton-Schulz tensor TFLOP/s), on every rank ----
    muon = None if args.skip_muon else run_muon(args, eng, world, rank, dev, barrier, max_over_ranks, peaks)

    c5 = None if args.skip_c5 else run_c5(args, eng, world, rank, dev, barrier, max_over_ranks, peaks,
                                          tail["fraction"] if tail and "fraction" in tail else 0.0)

    if rank != 0:
        return 0

    achieved_gbs = ADAM_BYTES_PER_PARAM * (wl.total / world) / (kernel_avg_ms * 1e-3) / 1e9
    config = bench_config(world)
    line = {
        "metric": "adam_params_per_s", "value": value, "unit": "params/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "data_note": "seeded synthetic parameters and one seeded gradient set resident in HBM; every timed block "
                     "restarts from the seeded parameters with zero moments and t = 0, runs the warm-up steps and "
                     "then exactly `steps` timed steps (the configuration itself is 50 steps)",
        "config": config,
        "arm_details": {"sharding": ("none" if world == 1 else
                                     f"ZeRO-1 slices of the first {1.0 - tail['fraction']:.3f} of the arena, the rest updated "
                                     "by every rank (replicated_tail)" if all_exchanged is not None else
                                     "ZeRO-1 slices of the whole arena"),
                        "exchange": ("none" if world == 1 else
                                     "peer stores over NVLink fused into the update kernel, fenced by a flag barrier in "
                                     "peer-mapped memory" if args.exchange == "peer" else
                                     "nccl all-gather of updated params after the update kernel")},
        "blocks": block_stats(headline_blocks, args.steps),
        "update_only": {"value": wl.total / (kernel_avg_ms * 1e-3), "unit": "params/s",
                        "ms_per_step": kernel_avg_ms, "blocks": block_stats(kernel_blocks, args.steps),
                        "per_rank_ms_per_step": per_rank_update_ms,
                        "note": "fused update kernel alone, max over ranks"},
        "roofline": {"bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved_gbs / peaks["hbm_gbs"], "traffic": NCU_ADAM_C3_DRAM_BYTES_PER_LAUNCH / world,
                     "traffic_note": "ncu capture of a whole-arena launch" + ("" if world == 1 else
                                     f", divided by {world}: a launch covers this rank's slice and traffic is "
                                     "proportional to the elements updated"),
                     "peak_source": peaks["source"], "frac_of_nominal_8tbs": achieved_gbs / 8000.0,
                     "kernel": "multi_tensor_update_kernel<ADAM>",
                     "algorithmic_bytes_per_launch": ADAM_BYTES_PER_PARAM * (wl.total // world),
                     "launch_ms": kernel_avg_ms},
        "gpu_launches": int(launches),
        "gpu_launches_note": f"update and fence kernels launched inside the timed regions of the {len(headline_blocks)} blocks "
                             f"({launches // max(len(headline_blocks) * args.steps, 1)} per step)",
        "clocks": clocks,
    }
    if clocks and clocks.get("sm_mhz"):
        line["ms_per_step_x_sm_mhz"] = ms_per_step * clocks["sm_mhz"]
    if e2e is not None:
        line["e2e"] = e2e
    if parity is not None:
        line["parity"] = parity

    if not args.no_cpu_baseline:
        n_cpu = 12 if world == 1 else 3
        times = time_cpu_adam(wl, n_cpu, 1, max_seconds=20.0 if world == 1 else 4.0)
        sec = sum(times) / len(times)
        line["cpu_baseline"] = {"value": wl.total / sec, "unit": "params/s", "cores": 1, "kind": "port",
                                "sample": f"{len(times)} full steps of the same workload, 1 thread of "
                                          f"{os.cpu_count()} host cores (Volta's optimizer is single threaded)"
                                          + ("" if world == 1 else "; a shorter sample than at N=1"),
                                "ms_per_step": sec * 1e3}
    if world > 1:
        # Every rank must receive the (N-1)/N of the updated parameters it does not own: NVLink
        # ingress bounds the whole step whatever the update costs.
        ingress = 4.0 * arena * (world - 1) / world
        if nvlink is not None:
            peak, src = nvlink["gbs_in_per_gpu"], "measured in this run (copy engines, all ranks sending at once)"
        else:
            peak, src = 770.0, "peer-copy rate of an earlier measurement (900 GB/s nominal)"
        floor_ms = ingress / (peak * 1e9) * 1e3
        line["exchange_roofline"] = {"bound": "nvlink ingress per GPU", "bytes_in_per_gpu": ingress, "peak": peak,
                                     "peak_source": src, "unit": "GB/s", "floor_ms": floor_ms,
                                     "achieved": ingress / (zero1_ms_per_step * 1e-3) / 1e9,
                                     "frac": floor_ms / zero1_ms_per_step,
                                     "strong_scaling_efficiency_bound": (wl.total / (floor_ms * 1e-3)) / world,
                                     "note": "for the step that exchanges every parameter (all_exchanged when the headline "
                                             "is the replicated-tail sharding): its strong scaling is capped by "
                                             "this floor; the update kernel itself scales with 1/N (update_only); "
                                             "strong_scaling_efficiency_bound is params/s per GPU at the floor"}
        if nvlink is not None:
            line["exchange_roofline"]["probe"] = nvlink
    if tail is not None:
        line["replicated_tail"] = tail
    if all_exchanged is not None:
        line["all_exchanged"] = all_exchanged
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


def run_c5(args, eng, world, rank, dev, barrier, max_over_ranks, peaks, replicated_fraction=0.0):
    """Ragged multi-tensor Adam (4096 tensors, sizes log-uniform in [1, 2^22], ~1.13e9 params):
    the same kernel must hold its HBM fraction when the tensor list is ragged.  At N > 1 also the
    whole step with the fused exchange, every parameter exchanged and with the replicated tail the
    C3 measurement chose."""
    import torch

    from volta_b200 import VB_STEP_NO_EXCHANGE, Adam, Tensor
    from volta_b200.interop import device_array

    wl = workloads.c5_ragged_adam()
    h = wl.hyper
    steps = max(3, min(args.steps, 10))

    def build(fraction):
        eng.set_replicated_fraction(fraction)
        tensors = [Tensor(np.zeros(n, np.float32)) for n in wl.sizes]
        opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=eng)
        eng.set_replicated_fraction(0.0)
        p_ptr, g_ptr, arena, _ = opt.arena_layout()
        theta = torch.as_tensor(device_array(p_ptr, arena, opt), device=dev)
        grad = torch.as_tensor(device_array(g_ptr, arena, opt), device=dev)
        gen = torch.Generator(device=dev)
        gen.manual_seed(1234)   # the same values on every rank
        theta.normal_(0.0, 1.0, generator=gen)
        grad.normal_(0.0, 1e-3, generator=gen)
        opt.mark_all_grads_present()
        torch.cuda.synchronize()
        del theta, grad
        return opt, tensors

    def whole_steps(opt):
        stream = torch.cuda.ExternalStream(eng.stream, device=dev)
        for _ in range(2):
            opt.step()
        times = []
        for _ in range(3):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                opt.step()
            e1.record(stream)
            eng.synchronize()
            times.append(max_over_ranks(e0.elapsed_time(e1) / steps))
        barrier()
        return statistics.median(times)

    opt, tensors = build(0.0)
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
    gbs = ADAM_BYTES_PER_PARAM * (wl.total / world) / (ms * 1e-3) / 1e9
    out = {"workload": f"c5_ragged_adam: {len(wl.sizes)} tensors, {wl.total} f32 params, sizes in "
                       f"[{min(wl.sizes)}, {max(wl.sizes)}], lr=3e-4 wd=0.1", "steps": steps,
           "update_ms_per_step": ms, "params_per_s": wl.total / (ms * 1e-3), "achieved_gbs_per_gpu": gbs,
           "frac_of_measured_hbm_peak": gbs / peaks["hbm_gbs"], "note": "update kernel only (no exchange)"}
    if world > 1 and args.exchange == "peer":
        try:
            import volta_b200
            opt.open_peers(gather_handles(opt.ipc_handle(), world, dev))
            full_ms = whole_steps(opt)
            out["whole_step"] = {"ms_per_step": full_ms, "params_per_s": wl.total / (full_ms * 1e-3),
                                 "note": "fused peer exchange of every parameter"}
            opt.close()
            del tensors
            opt = None
            if replicated_fraction > 0.0:
                opt, tensors = build(replicated_fraction)
                opt.open_peers(gather_handles(opt.ipc_handle(), world, dev))
                tail_ms = whole_steps(opt)
                out["whole_step_replicated_tail"] = {"fraction": replicated_fraction, "ms_per_step": tail_ms,
                                                     "params_per_s": wl.total / (tail_ms * 1e-3)}
        except volta_b200.VoltaB200Error as exc:
            out["whole_step_error"] = str(exc)
            eng.set_replicated_fraction(0.0)
    if opt is not None:
        opt.close()
    return out


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


def time_library_chain(shapes, ns_steps, dev, min_seconds):
    """The Newton-Schulz chain's products alone through torch.bmm (cuBLAS, bf16): the library baseline.

    Same matrices per shape batched into one call, the short-side Gram as in the product path, but
    whole products (no symmetry), no polynomial pieces, no normalisation and no apply: what a
    chain of library GEMMs costs before anything is fused into it.  Returns (ms, flops) per chain."""
    import torch

    by_shape = {}
    for r, c in shapes:
        by_shape[(r, c)] = by_shape.get((r, c), 0) + 1
    gen = torch.Generator(device=dev).manual_seed(7)
    xs = [torch.randn(n, r, c, device=dev, dtype=torch.bfloat16, generator=gen) * 0.01 for (r, c), n in by_shape.items()]

    def chain():
        flops = 0.0
        for x in xs:
            n, r, c = x.shape
            y = x
            for _ in range(ns_steps):
                if r >= c:
                    y = torch.bmm(y, torch.bmm(y.transpose(1, 2), y))
                else:
                    y = torch.bmm(torch.bmm(y, y.transpose(1, 2)), y)
                flops += 4.0 * n * min(r, c) ** 2 * max(r, c)
        return flops

    for _ in range(3):
        flops = chain()
    torch.cuda.synchronize(dev)
    blocks = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    while len(blocks) < 3 or (time.perf_counter() - t0 < min_seconds and len(blocks) < 40):
        e0.record()
        for _ in range(10):
            chain()
        e1.record()
        e1.synchronize()
        blocks.append(e0.elapsed_time(e1) / 10)
    return statistics.median(blocks), flops


def run_muon(args, eng, world, rank, dev, barrier, max_over_ranks, peaks):
    """Muon on the 96 matrices of the 24-layer d=1024 configuration: NS TFLOP/s."""
    import torch

    from volta_b200 import VB_NS_BF16, VB_NS_F32, VB_NS_F32_TC, Muon, Tensor

    wl = workloads.c4_muon(layers=args.muon_layers)
    h = wl.hyper
    params = wl.make_params()
    grads = wl.make_grads(1)
    out = {}
    # "bf16" is the library's default (the chain form of Newton-Schulz); "bf16_per_iteration_form" runs the
    # same kernel on one Gram and one update product per iteration (VB_NS_CHAIN=0): twice the FLOPs in long
    # main loops, the like-for-like measure of the kernel against the dense-GEMM peak
    for mode_name, mode, steps in (("bf16", VB_NS_BF16, max(3, min(args.steps, 20))),
                                   ("bf16_per_iteration_form", VB_NS_BF16, max(3, min(args.steps, 20))),
                                   ("f32_tc", VB_NS_F32_TC, max(3, min(args.steps, 5))), ("f32", VB_NS_F32, 2)):
        if mode_name == "f32" and (args.skip_muon_f32 or (args.only_muon and not args.muon_f32)):
            continue
        if mode_name == "f32_tc" and args.only_muon and not args.muon_f32_tc:
            continue
        tensors = [Tensor(p, p.shape) for p in params]
        chain_env = os.environ.get("VB_NS_CHAIN")
        if mode_name == "bf16_per_iteration_form":
            os.environ["VB_NS_CHAIN"] = "0"   # read when the optimizer is created
        try:
            opt = Muon(tensors, h["lr"], h["momentum"], h["nesterov"], h["ns_steps"], ns_mode=mode, engine=eng)
        finally:
            if mode_name == "bf16_per_iteration_form":
                if chain_env is None:
                    del os.environ["VB_NS_CHAIN"]
                else:
                    os.environ["VB_NS_CHAIN"] = chain_env
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

        def run_block():
            e0.record(stream)
            for _ in range(steps):
                opt.step()
            e1.record(stream)
            eng.synchronize()
            return e0.elapsed_time(e1)

        # blocks of `steps` steps until the timed region is long enough for the clocks to settle
        # (the bit-faithful f32 mode is slow enough as it is)
        blocks = timed_blocks(run_block, barrier, max_over_ranks,
                              min_seconds=MIN_TIMED_SECONDS if mode_name == "bf16" else
                              0.25 if mode_name in ("f32_tc", "bf16_per_iteration_form") else 0.0,
                              max_blocks=40)
        muon_clocks = sampler.stop() if sampler is not None else None
        n_steps_total = steps * len(blocks)
        step_ms = statistics.median(blocks) / steps
        ns_ms = max_over_ranks(eng.profile("muon_ns")[0] / n_steps_total)
        pre_ms = eng.profile("muon_pre")[0] / n_steps_total
        apply_ms = eng.profile("muon_apply")[0] / n_steps_total
        exch_ms = eng.profile("exchange")[0] / n_steps_total
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
            "params_per_s": wl.total / (step_ms * 1e-3), "steps": steps, "blocks": block_stats(blocks, steps),
            "executed_flops_per_step": flops_total,
            "apply_note": "apply_ms is the last update launch, which applies its result to the weights in its epilogue "
                          "(8 B/param of HBM traffic on top of the product); it is part of ns_ms_per_step as well"
                          if mode_name != "f32" else "separate apply pass",
            "note": {"bf16_per_iteration_form": "tcgen05 bf16, one short-side Gram (computed on and above the diagonal) "
                                                "and one update product per iteration (VB_NS_CHAIN=0): the form whose "
                                                "launches are long dense products",
                     "bf16": "tcgen05 bf16, chain form: one long-side Gram, 3 (K - 1) short-side symmetric squares (computed "
                             "on and above the diagonal) and one long-side product per matrix instead of K Gram and K "
                             "update products; same result within the bf16 bound (VB_NS_CHAIN=0 selects the "
                             "per-iteration form)", "f32": "CUDA-core FFMA, bit-identical to the CPU arithmetic",
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
        if mode_name in ("bf16", "bf16_per_iteration_form"):
            out[mode_name]["roofline"] = {
                "bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
                "peak_source": peaks["source"] + " (cuBLAS bf16 sustained)",
                "frac_of_burst_peak": tflops / (peaks["bf16_tflops"] * world),
                "frac_of_nominal_2250": tflops / (2250.0 * world),
                "traffic": NCU_MUON_4LAYER_DRAM_BYTES_PER_LAUNCH * args.muon_layers / 4.0 / world,
                "traffic_note": "ncu capture of the 4-layer case (mean over the eleven launches of a step), scaled by "
                                "layers / 4: per-launch traffic grows with the number of matrices",
                "kernel": "ns_gemm_tc_kernel (tcgen05 bf16, 11 launches per step in the chain form)"
                          if mode_name == "bf16" else "ns_gemm_tc_kernel (tcgen05 bf16, 10 launches per step)"}
            if mode_name == "bf16_per_iteration_form":
                out[mode_name]["roofline"]["traffic"] = 158.6e6 * args.muon_layers / 4.0 / world
                out[mode_name]["roofline"]["traffic_note"] = ("ncu capture of the 4-layer case (mean of a Gram and an "
                                                              "update launch), scaled by layers / 4")
                if "bf16" in out:
                    out["bf16"]["roofline"]["note"] = (
                        "the chain form executes about half the FLOPs of the per-iteration form, in short (k = S) "
                        "symmetric squares that run at a lower rate, and ends sooner: "
                        f"{out['bf16']['ns_ms_per_step']:.3f} ms against {ns_ms:.3f} ms for the GEMM launches of a step; "
                        "the kernel's rate on long dense products is bf16_per_iteration_form.roofline")
        opt.close()
    out["config"] = {"workload": f"c4_muon: {len(wl.shapes)} matrices ({args.muon_layers} x {{3072x1024, 1024x1024, "
                                 f"4096x1024, 1024x4096}}), {wl.total} f32 params, lr=0.1 momentum=0.9 nesterov "
                                 "ns_steps=5"}
    if world == 1 and not args.no_library_baseline and "bf16" in out:
        lib_ms, lib_flops = time_library_chain(wl.shapes, h["ns_steps"], dev, timed_blocks.cap_seconds)
        out["bf16"]["library_baseline"] = {
            "ms_per_chain": lib_ms, "tflops": lib_flops / (lib_ms * 1e-3) / 1e12, "flops_per_chain": lib_flops,
            "ours_ms": out["bf16"]["ns_ms_per_step"],
            "ours_tflops_on_whole_products": lib_flops / (out["bf16"]["ns_ms_per_step"] * 1e-3) / 1e12,
            "note": "the reference's ten products per matrix (a Gram and an update product per iteration) through "
                    "torch.bmm (cuBLAS bf16, one batched call per shape), whole products, nothing fused: no "
                    "polynomial pieces, normalisation or apply, which ns_ms_per_step includes"}
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


# dram__bytes_read.sum + dram__bytes_write.sum per launch of ns_gemm_tc_kernel on 4 layers of the Muon workload
# (16 matrices): mean over the eleven launches of one step of the chain form (133, 71, 4 x 89, 3 x 158, 71 and
# 488 MB), from the ncu capture summarised in profiles/muon_c4_ns_gemm_tc.md
NCU_MUON_4LAYER_DRAM_BYTES_PER_LAUNCH = 144.8e6


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
    ap.add_argument("--replicated-fraction", type=float, default=-1.0,
                    help="N > 1: share of the arena every rank updates itself instead of receiving it "
                         "(-1 = from the measured HBM and NVLink rates, 0 = off)")
    ap.add_argument("--only-muon", action="store_true", help="profiling runs: Muon bf16 only")
    ap.add_argument("--no-library-baseline", action="store_true",
                    help="skip timing the Newton-Schulz products through torch.bmm beside the Muon numbers")
    ap.add_argument("--skip-c5", action="store_true", help="skip the ragged 4096-tensor Adam section")
    ap.add_argument("--skip-parity", action="store_true", help="profiling runs: skip the parity block")
    ap.add_argument("--min-seconds", type=float, default=MIN_TIMED_SECONDS,
                    help="each headline number is the median of K-step blocks that together run at least this long "
                         "(profiling runs: 0 = three blocks)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: updated parameters reach the other ranks by NVLink peer stores fused into the "
                         "update kernel (default) or by an NCCL all-gather after it")
    ap.add_argument("--muon-f32-tc", action="store_true", help="with --only-muon: also time the f32-accurate TC path")
    ap.add_argument("--muon-f32", action="store_true", help="with --only-muon: also time the bit-faithful f32 path")
    ap.add_argument("--muon-layers", type=int, default=24, help="profiling runs: fewer layers of the Muon set")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    timed_blocks.cap_seconds = args.min_seconds
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
