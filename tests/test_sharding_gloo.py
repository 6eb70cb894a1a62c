"""The multi-rank path on CPU: two gloo ranks, the library's own sharding plans, the oracle as
the arithmetic.  Checks that ZeRO-1 slicing of the arena (Adam/SGD) and whole-matrix ownership
(Muon) followed by the exchange step reproduce the unsharded result bit for bit, i.e. that
the host-side plan is a partition and the exchange layout (in-place all-gather of equal
slices; broadcast of each matrix from its owner) is consistent between ranks."""
import ctypes as C
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _plan(sizes, world, rank):
    from volta_b200 import _lib
    n = len(sizes)
    arr = (C.c_int64 * n)(*sizes)
    offs = (C.c_int64 * n)()
    arena, lo, hi, nch = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64()
    _lib.call("vb_plan_layout", n, arr, world, rank, 148, offs, C.byref(arena), C.byref(lo), C.byref(hi),
              C.byref(nch), 0, None, None, None)
    return [offs[i] for i in range(n)], arena.value, lo.value, hi.value


def _adam_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import oracle
    import workloads
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        wl = workloads.c5_ragged_adam(n_tensors=64, max_log2=14, seed=7)
        h = wl.hyper
        offsets, arena, lo, hi = _plan(wl.sizes, world, rank)
        theta = np.zeros(arena, np.float32)
        for o, p in zip(offsets, wl.make_params()):
            theta[o:o + p.size] = p.reshape(-1)
        # this rank's slice only: m, v exist for [lo, hi)
        mine = theta[lo:hi]
        opt = oracle.Adam([mine], h["lr"], h["betas"], h["eps"], h["weight_decay"])
        for s in (1, 2, 3):
            g = np.zeros(arena, np.float32)
            for o, gi in zip(offsets, wl.make_grads(s)):
                g[o:o + gi.size] = gi.reshape(-1)
            opt.step([np.ascontiguousarray(g[lo:hi])])
            # exchange: in-place all-gather of equal slices
            t = torch.from_numpy(theta)
            dist.all_gather_into_tensor(t, t[lo:hi].clone())
        ret[rank] = theta.copy()
    finally:
        dist.destroy_process_group()


def _adam_tail_worker(rank, world, port, ret, fraction):
    """ZeRO-1 slices of [0, tail) plus a tail every rank updates itself from its own gradients."""
    sys.path.insert(0, ROOT)
    import oracle
    import workloads
    from volta_b200 import _lib
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        wl = workloads.c5_ragged_adam(n_tensors=64, max_log2=14, seed=7)
        h = wl.hyper
        n = len(wl.sizes)
        arr = (C.c_int64 * n)(*wl.sizes)
        offs = (C.c_int64 * n)()
        arena, lo, hi, tail, nch = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64()
        _lib.call("vb_plan_layout_replicated", n, arr, world, rank, 148, fraction, offs, C.byref(arena), C.byref(lo),
                  C.byref(hi), C.byref(tail), C.byref(nch), 0, None, None, None, None)
        offsets, arena, lo, hi, tail = [offs[i] for i in range(n)], arena.value, lo.value, hi.value, tail.value
        assert 0 < tail < arena
        theta = np.zeros(arena, np.float32)
        for o, p in zip(offsets, wl.make_params()):
            theta[o:o + p.size] = p.reshape(-1)
        mine, shared = theta[lo:hi], theta[tail:]
        opt = oracle.Adam([mine, shared], h["lr"], h["betas"], h["eps"], h["weight_decay"])
        for s in (1, 2, 3):
            g = np.zeros(arena, np.float32)
            for o, gi in zip(offsets, wl.make_grads(s)):
                g[o:o + gi.size] = gi.reshape(-1)
            opt.step([np.ascontiguousarray(g[lo:hi]), np.ascontiguousarray(g[tail:])])
            t = torch.from_numpy(theta)
            dist.all_gather_into_tensor(t[:tail], t[lo:hi].clone())  # only the sliced part is exchanged
        ret[rank] = theta.copy()
    finally:
        dist.destroy_process_group()


def _free_port():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _spawn(fn, world, *extra):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=fn, args=(r, world, port, ret, *extra)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        return dict(ret)


def test_zero1_adam_two_ranks_matches_unsharded():
    import oracle
    import workloads
    res = _spawn(_adam_worker, 2)
    wl = workloads.c5_ragged_adam(n_tensors=64, max_log2=14, seed=7)
    h = wl.hyper
    params = wl.make_params()
    opt = oracle.Adam(params, h["lr"], h["betas"], h["eps"], h["weight_decay"])
    for s in (1, 2, 3):
        opt.step(wl.make_grads(s))
    offsets, arena, _, _ = _plan(wl.sizes, 2, 0)
    assert np.array_equal(res[0], res[1])
    for o, p in zip(offsets, params):
        assert np.array_equal(res[0][o:o + p.size].view(np.uint32), p.reshape(-1).view(np.uint32))


def test_adam_with_a_replicated_tail_two_ranks_matches_unsharded():
    import oracle
    import workloads
    res = _spawn(_adam_tail_worker, 2, 0.4)
    wl = workloads.c5_ragged_adam(n_tensors=64, max_log2=14, seed=7)
    h = wl.hyper
    params = wl.make_params()
    opt = oracle.Adam(params, h["lr"], h["betas"], h["eps"], h["weight_decay"])
    for s in (1, 2, 3):
        opt.step(wl.make_grads(s))
    offsets, arena, _, _ = _plan(wl.sizes, 2, 0)
    assert np.array_equal(res[0], res[1])
    for o, p in zip(offsets, params):
        assert np.array_equal(res[0][o:o + p.size].view(np.uint32), p.reshape(-1).view(np.uint32))


def _muon_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import oracle
    from volta_b200 import _lib
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shapes = [(48, 32), (32, 96), (64, 64), (40,), (16, 16)]
        rows = (C.c_int64 * len(shapes))(*[oracle.muon_dims(s)[0] for s in shapes])
        cols = (C.c_int64 * len(shapes))(*[oracle.muon_dims(s)[1] for s in shapes])
        owners = (C.c_int32 * len(shapes))()
        _lib.call("vb_plan_muon_owners", len(shapes), rows, cols, world, 0, 5, owners, None)
        rng = np.random.default_rng(0)
        params = [(rng.standard_normal(s) * 0.02).astype(np.float32) for s in shapes]
        owned = [i for i in range(len(shapes)) if owners[i] == rank]
        opt = oracle.Muon([params[i] for i in owned], 0.1, 0.9, True, 5)
        for _ in range(2):
            grads = [(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in shapes]
            opt.step([grads[i] for i in owned])
            for i in range(len(shapes)):  # every matrix from its owner
                t = torch.from_numpy(params[i])
                dist.broadcast(t, src=int(owners[i]))
        ret[rank] = ([p.copy() for p in params], list(owners))
    finally:
        dist.destroy_process_group()


def test_muon_ownership_two_ranks_matches_unsharded():
    import oracle
    res = _spawn(_muon_worker, 2)
    shapes = [(48, 32), (32, 96), (64, 64), (40,), (16, 16)]
    rng = np.random.default_rng(0)
    params = [(rng.standard_normal(s) * 0.02).astype(np.float32) for s in shapes]
    opt = oracle.Muon(params, 0.1, 0.9, True, 5)
    for _ in range(2):
        opt.step([(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in shapes])
    assert res[0][1] == res[1][1] and set(res[0][1]) == {0, 1}  # both ranks own something
    for a, b, c in zip(res[0][0], res[1][0], params):
        assert np.array_equal(a, b) and np.array_equal(a.view(np.uint32), c.view(np.uint32))


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_muon_owner_plan_balances_c4_under_the_executed_cost(mode):
    """Ownership is planned with the cost the mode executes: the bit-faithful f32 kernels run
    4 * rows * cols^2 FLOPs per iteration (4x more for 1024 x 4096 than for 4096 x 1024), the
    tensor-core modes the short-side form.  The heaviest rank stays within 5 % of the mean."""
    import workloads
    from volta_b200 import _lib
    wl = workloads.c4_muon()
    n = len(wl.shapes)
    rows = (C.c_int64 * n)(*[s[0] for s in wl.shapes])
    cols = (C.c_int64 * n)(*[s[1] for s in wl.shapes])

    def executed(shape):
        r, c = shape
        if mode == 0:
            return 4.0 * r * c * c                      # src/nn/optim/muon.rs:73: always cols x cols
        long_, short = max(r, c), min(r, c)
        t = -(-short // 256)
        upper = (t * (t + 1) / 2) / (t * t)
        return 2.0 * long_ * short * short * (1.0 + upper)

    for world in (2, 4, 8):
        owners = (C.c_int32 * n)()
        est = (C.c_double * world)()
        _lib.call("vb_plan_muon_owners", n, rows, cols, world, mode, 5, owners, est)
        load = np.zeros(world)
        for i, s in enumerate(wl.shapes):
            load[owners[i]] += executed(s)
        assert load.max() / load.mean() <= 1.05, (mode, world, load)
        assert max(est) / (sum(est) / world) <= 1.05


def _fingerprint_worker(rank, world, port, ret, odd_rank):
    """Every rank hashes its own description of the optimizer, the ranks all-gather the hashes over
    gloo (the host's transport) and each checks the list before anything would be launched."""
    sys.path.insert(0, ROOT)
    from volta_b200 import VoltaB200Error, plan_fingerprint, verify_plan
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sizes = [4096, 12, 777]
        if rank == odd_rank:
            sizes = [4096, 12, 778]   # this rank built its model differently
        fp = plan_fingerprint("adam", sizes, [1e-3, 0.9, 0.999, 1e-8, 0.01], world_size=world)
        mine = torch.tensor([fp & 0x7fffffffffffffff, fp >> 63], dtype=torch.int64)
        gathered = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(gathered, mine)
        fps = [int(g[0]) | (int(g[1]) << 63) for g in gathered]
        try:
            verify_plan(fps)
            ret[rank] = "ok"
        except VoltaB200Error as exc:
            ret[rank] = (exc.status, exc.message)
    finally:
        dist.destroy_process_group()


def test_ranks_with_different_tensor_lists_are_caught_before_the_first_step():
    """Host-side failure detection between ranks (no GPU involved): a size mismatch is found by
    comparing plan fingerprints, and every rank gets the same VB_ERR_STATE."""
    res = _spawn(_fingerprint_worker, 2, -1)
    assert res[0] == "ok" and res[1] == "ok"
    res = _spawn(_fingerprint_worker, 2, 1)
    for rank in (0, 1):
        status, message = res[rank]
        assert status == 5 and "rank 1" in message
