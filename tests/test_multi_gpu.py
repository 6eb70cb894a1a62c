"""Sharded optimizers on 2 and 4 GPUs (skipped with fewer): one child process per GPU, the library's
own NCCL communicator, results compared with the unsharded CPU oracle.

Adam/SGD: ZeRO-1 slices of the arena + in-place all-gather.  Muon: whole matrices per owner +
grouped broadcast.  Every rank must end with the full, bit-identical parameter set."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpu_count():
    import torch
    return torch.cuda.device_count()


def _worker(rank, world, shared, kind):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import time

    import workloads
    from volta_b200 import SGD, VB_NS_BF16, VB_NS_F32, Adam, Engine, Muon, Tensor
    eng = Engine(rank)
    if rank == 0:
        shared["id"] = Engine.unique_id()
    while "id" not in shared:
        time.sleep(0.01)
    eng.init_comm(shared["id"], rank, world)
    assert (eng.rank, eng.world_size) == (rank, world)
    peer = kind.endswith("_peer")  # exchange fused into the update kernel (NVLink peer stores)
    kind = kind.replace("_peer", "")
    if kind.endswith("_tail"):     # part of the arena is updated by every rank itself and never exchanged
        eng.set_replicated_fraction(0.45)
        kind = kind.replace("_tail", "")
    if kind == "adam":
        wl = workloads.c5_ragged_adam(n_tensors=96, max_log2=16, seed=11)
    elif kind == "sgd":
        wl = workloads.c2_cnn_sgd()
    else:
        shapes = [(256, 128), (128, 384), (64, 36), (100,), (512, 256), (256, 256)]
        wl = workloads.Workload("muon_small", "muon", shapes, [("normal", 0.02)] * len(shapes), 1e-3,
                                dict(lr=0.1, momentum=0.9, nesterov=True, ns_steps=5), 3)
    h = wl.hyper
    tensors = [Tensor(p, p.shape) for p in wl.make_params()]
    if kind == "adam":
        opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=eng)
    elif kind == "sgd":
        opt = SGD(tensors, h["lr"], h["momentum"], h["weight_decay"], engine=eng)
    else:
        opt = Muon(tensors, h["lr"], h["momentum"], h["nesterov"], h["ns_steps"],
                   ns_mode=VB_NS_F32 if kind == "muon_f32" else VB_NS_BF16, engine=eng)
    if peer:
        shared[f"ipc{rank}"] = opt.ipc_handle()
        while any(f"ipc{r}" not in shared for r in range(world)):
            time.sleep(0.01)
        opt.open_peers([shared[f"ipc{r}"] for r in range(world)])
    owned = 0
    for s in (1, 2, 3):
        opt.zero_grad()
        for t, g in zip(tensors, wl.make_grads(s)):
            t.grad = g
        opt.step()
    for i in range(len(tensors)):
        lo, hi = opt.state_owned_range(i, 0)
        owned += hi - lo
    shared[f"params{rank}"] = [t.data.copy() for t in tensors]
    shared[f"owned{rank}"] = owned
    shared[f"ranges{rank}"] = (opt.owned_range(), opt.replicated_range()) if kind in ("adam", "sgd") else None
    opt.close()
    eng.close()


@pytest.mark.parametrize("world,kind", [(2, k) for k in ("adam", "sgd", "adam_peer", "sgd_peer", "muon_f32", "muon_bf16",
                                                         "muon_f32_peer", "muon_bf16_peer")] +
                         [(2, k) for k in ("adam_tail", "adam_tail_peer", "sgd_tail_peer")] +
                         [(4, k) for k in ("adam", "adam_peer", "sgd_peer", "muon_f32_peer", "muon_bf16_peer",
                                           "adam_tail_peer")])
def test_sharded_step_matches_oracle(oracle, world, kind):
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    import workloads
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        shared = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, shared, kind)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0
        res = dict(shared)
    kind = kind.replace("_peer", "")
    tail = kind.endswith("_tail")
    kind = kind.replace("_tail", "")
    if kind in ("adam", "sgd"):
        (lo0, hi0), (t_lo, t_hi) = res["ranges0"]
        assert (t_hi - t_lo > 0) == tail and all(res[f"ranges{r}"][1] == (t_lo, t_hi) for r in range(world))
        assert (hi0 - lo0) * world == t_lo  # the slices cut up what the tail leaves
    if kind == "adam":
        wl = workloads.c5_ragged_adam(n_tensors=96, max_log2=16, seed=11)
    elif kind == "sgd":
        wl = workloads.c2_cnn_sgd()
    else:
        shapes = [(256, 128), (128, 384), (64, 36), (100,), (512, 256), (256, 256)]
        wl = workloads.Workload("muon_small", "muon", shapes, [("normal", 0.02)] * len(shapes), 1e-3,
                                dict(lr=0.1, momentum=0.9, nesterov=True, ns_steps=5), 3)
    h = wl.hyper
    ref = wl.make_params()
    if kind == "adam":
        o = oracle.Adam(ref, h["lr"], h["betas"], h["eps"], h["weight_decay"])
    elif kind == "sgd":
        o = oracle.SGD(ref, h["lr"], h["momentum"], h["weight_decay"])
    else:
        o = oracle.Muon(ref, h["lr"], h["momentum"], h["nesterov"], h["ns_steps"])
    for s in (1, 2, 3):
        o.step(wl.make_grads(s))
    for i, r in enumerate(ref):
        a = res["params0"][i]
        for rank in range(1, world):   # every rank holds the same parameters
            assert np.array_equal(a.view(np.uint32), res[f"params{rank}"][i].view(np.uint32)), (rank, i)
        if kind == "muon_bf16":
            assert np.max(np.abs(a - r)) <= 2e-2 * 0.1 * 0.1 * 3 * max(1.0, float(np.max(np.abs(r))))
        else:
            assert np.array_equal(a.view(np.uint32), r.view(np.uint32))
    # state is partitioned: the ranks' owned element counts add up to the whole
    owned = [res[f"owned{rank}"] for rank in range(world)]
    assert sum(owned) == wl.total and min(owned) > 0


def _worker_tail_resume(rank, world, shared):
    """Two steps, export the state, a new optimizer with the merged state, a third step on both."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import time

    import workloads
    from volta_b200 import Adam, Engine, Tensor, VoltaB200Error
    eng = Engine(rank)
    if rank == 0:
        shared["id"] = Engine.unique_id()
    while "id" not in shared:
        time.sleep(0.01)
    eng.init_comm(shared["id"], rank, world)
    eng.set_replicated_fraction(0.45)
    wl = workloads.c5_ragged_adam(n_tensors=96, max_log2=16, seed=11)
    h = wl.hyper

    def gather(key, value):
        shared[f"{key}{rank}"] = value
        while any(f"{key}{r}" not in shared for r in range(world)):
            time.sleep(0.01)
        return [shared[f"{key}{r}"] for r in range(world)]

    def make():
        tensors = [Tensor(p, p.shape) for p in wl.make_params()]
        return tensors, Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=eng)

    def step(tensors, opt, s):
        opt.zero_grad()
        for t, g in zip(tensors, wl.make_grads(s)):
            t.grad = g
        opt.step()

    tensors, opt = make()
    opt.open_peers(gather("ipc_a", opt.ipc_handle()))
    # the pipelined host step moves one contiguous owned range: refused (before anything is enqueued)
    _, _, arena, _ = opt.arena_layout()
    try:
        opt.step_host(np.zeros(arena, np.float32), np.zeros(arena, np.float32), pieces=2)
        raise AssertionError("step_host accepted an optimizer with a replicated tail")
    except VoltaB200Error as exc:
        assert "replicated" in str(exc)
    for s in (1, 2):
        step(tensors, opt, s)
    # every element of the state is reported by exactly one rank
    mine = [[(opt.state(i, w), opt.state_owned_range(i, w)) for i in range(len(tensors))] for w in (0, 1)]
    everyone = gather("state", mine)
    tensors2, opt2 = make()
    opt2.open_peers(gather("ipc_b", opt2.ipc_handle()))
    covered = 0
    for w in (0, 1):
        for i in range(len(tensors)):
            full = np.zeros(tensors[i].data.size, np.float32)
            for r in range(world):
                arr, (lo, hi) = everyone[r][w][i]
                assert not full[lo:hi].any()
                full[lo:hi] = arr[lo:hi]
                covered += (hi - lo) if w == 0 else 0
            opt2.load_state(i, w, full)
    assert covered == wl.total
    for t2, t1 in zip(tensors2, tensors):
        t2.data = t1.data.copy()
    opt2.t = opt.t
    step(tensors, opt, 3)
    step(tensors2, opt2, 3)
    shared[f"a{rank}"] = [t.data.copy() for t in tensors]
    shared[f"b{rank}"] = [t.data.copy() for t in tensors2]
    gather("done", 1)
    opt.close()
    opt2.close()
    eng.close()


def test_state_round_trip_with_a_replicated_tail(oracle):
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    import workloads
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        shared = mgr.dict()
        procs = [ctx.Process(target=_worker_tail_resume, args=(r, 2, shared)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0
        res = dict(shared)
    wl = workloads.c5_ragged_adam(n_tensors=96, max_log2=16, seed=11)
    h = wl.hyper
    ref = wl.make_params()
    o = oracle.Adam(ref, h["lr"], h["betas"], h["eps"], h["weight_decay"])
    for s in (1, 2, 3):
        o.step(wl.make_grads(s))
    for i, r in enumerate(ref):
        for key in ("a0", "a1", "b0", "b1"):
            assert np.array_equal(res[key][i].view(np.uint32), r.view(np.uint32)), (key, i)


def _bf16_rne(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def _small_workload(kind):
    import workloads
    if kind == "adam":
        return workloads.c5_ragged_adam(n_tensors=96, max_log2=16, seed=11)
    if kind == "sgd":
        return workloads.c2_cnn_sgd()
    shapes = [(256, 128), (128, 384), (64, 36), (100,), (512, 256), (256, 256), (3, 3)]
    return workloads.Workload("muon_small", "muon", shapes, [("normal", 0.02)] * len(shapes), 1e-3,
                              dict(lr=0.1, momentum=0.9, nesterov=True, ns_steps=5), 3)


def _worker_bf16(rank, world, shared, kind, transport, what):
    """`what` = "half": step(VB_STEP_EXCHANGE_BF16), only the bf16 copies cross; "both": default step with
    the copies enabled.  `transport` = "nccl" or "peer" (stores fused into the kernel)."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import time

    from volta_b200 import SGD, VB_NS_F32, VB_STEP_EXCHANGE_BF16, Adam, Engine, Muon, Tensor
    eng = Engine(rank)
    if rank == 0:
        shared["id"] = Engine.unique_id()
    while "id" not in shared:
        time.sleep(0.01)
    eng.init_comm(shared["id"], rank, world)
    wl = _small_workload(kind)
    h = wl.hyper
    tensors = [Tensor(p, p.shape) for p in wl.make_params()]
    if kind == "adam":
        opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=eng)
    elif kind == "sgd":
        opt = SGD(tensors, h["lr"], h["momentum"], h["weight_decay"], engine=eng)
    else:
        opt = Muon(tensors, h["lr"], h["momentum"], h["nesterov"], h["ns_steps"], ns_mode=VB_NS_F32, engine=eng)
    opt.enable_bf16_params()

    def gather(key, value):
        shared[f"{key}{rank}"] = value
        while any(f"{key}{r}" not in shared for r in range(world)):
            time.sleep(0.01)
        return [shared[f"{key}{r}"] for r in range(world)]

    if transport == "peer":
        opt.open_peers_bf16(gather("ipch", opt.ipc_handle_bf16()))
        if what == "both":
            opt.open_peers(gather("ipc", opt.ipc_handle()))
    for s in (1, 2, 3):
        opt.zero_grad()
        for t, g in zip(tensors, wl.make_grads(s)):
            t.grad = g
        opt.step(VB_STEP_EXCHANGE_BF16 if what == "half" else 0)
    shared[f"params{rank}"] = [t.data.copy() for t in tensors]
    shared[f"half{rank}"] = [opt.bf16_params(i) for i in range(len(tensors))]
    shared[f"owned{rank}"] = [opt.state_owned_range(i, 0) for i in range(len(tensors))]
    opt.close()
    eng.close()


@pytest.mark.parametrize("kind,transport,what", [
    ("adam", "nccl", "half"), ("adam", "peer", "half"), ("adam", "peer", "both"), ("adam", "nccl", "both"),
    ("sgd", "peer", "half"), ("muon_f32", "nccl", "half"), ("muon_f32", "peer", "half"), ("muon_f32", "peer", "both")])
def test_two_gpu_bf16_copies_exchange(oracle, kind, transport, what):
    """bf16 copies of the parameters written by the update / apply kernel: every rank ends with
    rne(theta) for ALL parameters; with the bf16-only exchange the f32 values are exact on the
    part a rank owns (the rest keeps its old value), with the default step everywhere."""
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        shared = mgr.dict()
        procs = [ctx.Process(target=_worker_bf16, args=(r, 2, shared, kind, transport, what)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0
        res = dict(shared)
    wl = _small_workload(kind)
    h = wl.hyper
    ref = wl.make_params()
    start = [p.copy() for p in ref]
    if kind == "adam":
        o = oracle.Adam(ref, h["lr"], h["betas"], h["eps"], h["weight_decay"])
    elif kind == "sgd":
        o = oracle.SGD(ref, h["lr"], h["momentum"], h["weight_decay"])
    else:
        o = oracle.Muon(ref, h["lr"], h["momentum"], h["nesterov"], h["ns_steps"])
    for s in (1, 2, 3):
        o.step(wl.make_grads(s))
    owned_total = 0
    for rank in (0, 1):
        for i, r in enumerate(ref):
            want = _bf16_rne(r).reshape(r.shape)
            assert np.array_equal(res[f"half{rank}"][i], want), (rank, i)
            got = res[f"params{rank}"][i].reshape(-1).view(np.uint32)
            exact = r.reshape(-1).view(np.uint32)
            if what == "both":
                assert np.array_equal(got, exact)
            else:
                lo, hi = res[f"owned{rank}"][i]
                owned_total += hi - lo
                assert np.array_equal(got[lo:hi], exact[lo:hi])
                stale = start[i].reshape(-1).view(np.uint32)
                assert np.array_equal(got[:lo], stale[:lo]) and np.array_equal(got[hi:], stale[hi:])
    if what == "half":
        assert owned_total == wl.total


def _rank_grads(wl, step, rank):
    """Rank-specific gradients of the whole model (what data parallelism gives each rank)."""
    return [(g * np.float32(1.0 + 0.25 * rank) + np.float32(1e-4 * rank)).astype(np.float32)
            for g in wl.make_grads(step * 7 + rank)]


def _worker_reduce(rank, world, shared, kind, transport, mean):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import time

    from volta_b200 import (SGD, VB_NS_F32, VB_STEP_MEAN_GRADS, VB_STEP_REDUCE_GRADS, Adam, Engine, Muon, Tensor)
    eng = Engine(rank)
    if rank == 0:
        shared["id"] = Engine.unique_id()
    while "id" not in shared:
        time.sleep(0.01)
    eng.init_comm(shared["id"], rank, world)
    wl = _small_workload(kind)
    h = wl.hyper
    tensors = [Tensor(p, p.shape) for p in wl.make_params()]
    if kind == "adam":
        opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=eng)
    elif kind == "sgd":
        opt = SGD(tensors, h["lr"], h["momentum"], h["weight_decay"], engine=eng)
    else:
        opt = Muon(tensors, h["lr"], h["momentum"], h["nesterov"], h["ns_steps"], ns_mode=VB_NS_F32, engine=eng)

    def gather(key, value):
        shared[f"{key}{rank}"] = value
        while any(f"{key}{r}" not in shared for r in range(world)):
            time.sleep(0.01)
        return [shared[f"{key}{r}"] for r in range(world)]

    opt.open_peers_grads(gather("ipcg", opt.ipc_handle_grads()))
    if transport == "peer":
        opt.open_peers(gather("ipc", opt.ipc_handle()))
    for s in (1, 2, 3):
        for t, g in zip(tensors, _rank_grads(wl, s, rank)):
            t.grad = g
        opt.step(VB_STEP_MEAN_GRADS if mean else VB_STEP_REDUCE_GRADS)
        eng.synchronize()   # the next upload overwrites gradients the peers read during this step
    shared[f"params{rank}"] = [t.data.copy() for t in tensors]
    opt.close()
    eng.close()


@pytest.mark.parametrize("kind,transport,mean", [("adam", "peer", False), ("adam", "nccl", True), ("sgd", "peer", True),
                                                 ("muon_f32", "peer", False), ("muon_f32", "nccl", True)])
def test_two_gpu_gradient_reduction_fused_into_the_update(oracle, kind, transport, mean):
    """Data-parallel step: each rank holds its own gradient of the whole model; the owning rank's
    kernel adds the ranks' values in rank order while it loads them.  Bit-identical to the oracle
    stepping with the gradients summed the same way on the host."""
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        shared = mgr.dict()
        procs = [ctx.Process(target=_worker_reduce, args=(r, 2, shared, kind, transport, mean)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0
        res = dict(shared)
    wl = _small_workload(kind)
    h = wl.hyper
    ref = wl.make_params()
    if kind == "adam":
        o = oracle.Adam(ref, h["lr"], h["betas"], h["eps"], h["weight_decay"])
    elif kind == "sgd":
        o = oracle.SGD(ref, h["lr"], h["momentum"], h["weight_decay"])
    else:
        o = oracle.Muon(ref, h["lr"], h["momentum"], h["nesterov"], h["ns_steps"])
    for s in (1, 2, 3):
        g0, g1 = _rank_grads(wl, s, 0), _rank_grads(wl, s, 1)
        summed = [(a + b).astype(np.float32) for a, b in zip(g0, g1)]          # one rounded add, rank order
        if mean:
            summed = [(x * np.float32(0.5)).astype(np.float32) for x in summed]
        o.step(summed)
    for a, b, r in zip(res["params0"], res["params1"], ref):
        assert np.array_equal(a.view(np.uint32), r.view(np.uint32))
        assert np.array_equal(b.view(np.uint32), r.view(np.uint32))


def _worker_absent_rank(rank, world, shared):
    """Rank 1 takes part in the first step and then stops stepping (it stays alive and idle: nothing
    of it is in flight).  Rank 0's next step must give up its wait in bounded time, and rank 1, when
    it steps again later, must fail as well: no rank goes on alone."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, ROOT)
    import time

    import workloads
    from volta_b200 import VB_STEP_NO_EXCHANGE, Adam, Engine, Tensor, VoltaB200Error
    eng = Engine(rank)
    if rank == 0:
        shared["id"] = Engine.unique_id()
    while "id" not in shared:
        time.sleep(0.01)
    eng.init_comm(shared["id"], rank, world)
    eng.set_wait_limit_ms(300)
    wl = workloads.c5_ragged_adam(n_tensors=32, max_log2=14, seed=3)
    h = wl.hyper

    def make():
        ts = [Tensor(p, p.shape) for p in wl.make_params()]
        return ts, Adam(ts, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=eng)

    tensors, opt = make()
    shared[f"ipc{rank}"] = opt.ipc_handle()
    while any(f"ipc{r}" not in shared for r in range(world)):
        time.sleep(0.01)
    opt.open_peers([shared[f"ipc{r}"] for r in range(world)])
    for t, g in zip(tensors, wl.make_grads(1)):
        t.grad = g
    opt.step()                       # both ranks: an ordinary sharded step
    eng.synchronize()
    shared[f"stepped{rank}"] = True
    while any(f"stepped{r}" not in shared for r in range(world)):
        time.sleep(0.01)
    out = {}
    if rank == 0:
        t0 = time.perf_counter()
        opt.step()                   # rank 1 never comes: the fence's bounded wait runs out
        try:
            eng.synchronize()
            out["status"] = 0
        except VoltaB200Error as exc:
            out["status"], out["message"] = exc.status, exc.message
        out["seconds"] = time.perf_counter() - t0
        shared["rank0_reported"] = True
    else:
        while "rank0_reported" not in shared:
            time.sleep(0.01)
        opt.step()                   # late, after rank 0 gave up: must not go on alone
        try:
            eng.synchronize()
            out["status"] = 0
        except VoltaB200Error as exc:
            out["status"], out["message"] = exc.status, exc.message
    try:                             # fail-stop: the optimizer refuses further steps ...
        opt.step()
        out["again"] = 0
    except VoltaB200Error as exc:
        out["again"] = exc.status
    shared[f"late{rank}"] = True     # nobody frees an arena a peer's kernels may still write flags into
    while any(f"late{r}" not in shared for r in range(world)):
        time.sleep(0.01)
    import ctypes as C
    from volta_b200 import _lib
    _lib.load().vb_optimizer_destroy(opt._h)
    opt._h = C.c_void_p()
    # ... while the engine and its context are intact: a new optimizer works (no exchange asked for)
    tensors2, opt2 = make()
    for t, g in zip(tensors2, wl.make_grads(2)):
        t.grad = g
    opt2.step(VB_STEP_NO_EXCHANGE)
    eng.synchronize()
    lo, hi = opt2.owned_range()
    out["alive"] = bool(hi > lo and all(np.all(np.isfinite(t.data)) for t in tensors2))
    shared[f"out{rank}"] = out
    shared[f"finished{rank}"] = True
    while any(f"finished{r}" not in shared for r in range(world)):   # leave together: peers' memory stays mapped
        time.sleep(0.01)
    _lib.load().vb_optimizer_destroy(opt2._h)
    opt2._h = C.c_void_p()
    eng.close()


def test_a_rank_that_stops_stepping_ends_the_step_on_every_rank():
    """Failure detection between ranks on real GPUs, without faulting anything: the absent rank is
    alive and idle, the others' waits are bounded (300 ms here), every rank gets VB_ERR_TIMEOUT, the
    optimizer is fail-stop and the CUDA context stays usable."""
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        shared = mgr.dict()
        procs = [ctx.Process(target=_worker_absent_rank, args=(r, 2, shared)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        res = dict(shared)
    r0, r1 = res["out0"], res["out1"]
    assert r0["status"] == 4 and "did not reach" in r0["message"], r0
    assert 0.25 <= r0["seconds"] < 10.0, r0
    assert r1["status"] == 4, r1
    assert r0["again"] == 4 and r1["again"] == 4
    assert r0["alive"] and r1["alive"]
