"""Failure detection without faulting the GPU.

Every spin-wait inside the tensor-core GEMM kernel is bounded.  `vb_debug_gemm_wait_expiry`
runs the kernel on a problem whose producer withholds its loads, so the waits run out: the
kernel must report which role gave up, release its tensor memory and return, the host must
see VB_ERR_TIMEOUT, and the engine must keep working afterwards (a following Muon step on the
same engine reproduces the oracle, which it could not if TMEM had leaked or the context had
been lost)."""
import ctypes as C

import numpy as np
import pytest

from helpers import rel_frobenius


@pytest.mark.gpu
def test_bounded_wait_expiry_is_reported_and_engine_survives(oracle, engine):
    from volta_b200 import VB_NS_BF16, Muon, Tensor, VoltaB200Error, _lib
    role = C.c_int(0)
    with pytest.raises(VoltaB200Error) as ei:
        _lib.call("vb_debug_gemm_wait_expiry", engine._h, 1 << 12, C.byref(role))
    assert ei.value.status == 4  # VB_ERR_TIMEOUT
    assert role.value in (1, 2, 3) and "gave up waiting" in ei.value.message
    # the engine is still healthy: run a real tensor-core step on it
    rng = np.random.default_rng(0)
    g = (rng.standard_normal((256, 384)) * 1e-3).astype(np.float32)
    w = Tensor(np.zeros((256, 384), np.float32))
    opt = Muon([w], 0.1, 0.0, False, 5, ns_mode=VB_NS_BF16, engine=engine, keep_update=True)
    w.grad = g
    opt.step()
    assert rel_frobenius(opt.last_update(0), oracle.newton_schulz(g, 5)) <= 2e-2
    opt.close()


@pytest.mark.gpu
def test_muon_step_whose_gemm_gives_up_leaves_the_weights_untouched(engine):
    """The bounded waits run out inside a real optimizer step (the first tensor-core launch
    withholds its loads; nothing faults or hangs).  Every later kernel of the step sees the
    record and stores nothing: the weights keep their pre-step values, the error reaches the host
    as VB_ERR_TIMEOUT at the next call that waits, and the optimizer is fail-stop afterwards
    while the engine keeps working for other optimizers."""
    from volta_b200 import VB_NS_BF16, Muon, Tensor, VoltaB200Error, _lib
    rng = np.random.default_rng(3)
    shapes = [(256, 384), (128, 128), (40,)]
    start = [(rng.standard_normal(s) * 0.02).astype(np.float32) for s in shapes]
    tensors = [Tensor(p.copy()) for p in start]
    opt = Muon(tensors, 0.1, 0.9, True, 5, ns_mode=VB_NS_BF16, engine=engine)
    for t in tensors:
        t.grad = (rng.standard_normal(t.shape) * 1e-3).astype(np.float32)
    _lib.call("vb_debug_muon_withhold_loads", opt._h, 1 << 12)
    opt.step()   # enqueues; the expiry is found when the stream is waited for
    lib = _lib.load()
    for i, p in enumerate(start):
        out = np.full(p.size, np.nan, np.float32)
        status = lib.vb_optimizer_download_params(opt._h, i, out.ctypes.data_as(C.c_void_p), out.size)
        assert status == 4    # VB_ERR_TIMEOUT, reported by the call that waited
        assert np.array_equal(out.view(np.uint32), p.reshape(-1).view(np.uint32)), i   # ... data untouched
    with pytest.raises(VoltaB200Error) as ei:
        opt.step()
    assert ei.value.status == 4
    lib.vb_optimizer_destroy(opt._h)
    opt._h = C.c_void_p()
    # the engine itself is fine
    w = Tensor(np.zeros((256, 384), np.float32))
    opt2 = Muon([w], 0.1, 0.0, False, 5, ns_mode=VB_NS_BF16, engine=engine)
    w.grad = (rng.standard_normal((256, 384)) * 1e-3).astype(np.float32)
    opt2.step()
    engine.synchronize()
    assert np.all(np.isfinite(w.data)) and np.any(w.data != 0)
    opt2.close()


@pytest.mark.gpu
@pytest.mark.parametrize("phase", [1, 2])
def test_fence_wait_on_a_rank_that_never_arrives_runs_out(engine, phase):
    """The flag barrier around sharded steps, on one GPU: the "peer" is a flag block nobody ever
    writes.  The wait must end after its bound, name the phase, and leave the engine usable."""
    import time
    from volta_b200 import VoltaB200Error, _lib
    code = C.c_int(0)
    t0 = time.perf_counter()
    with pytest.raises(VoltaB200Error) as ei:
        _lib.call("vb_debug_fence_wait_expiry", engine._h, 20, phase, C.byref(code))
    dt = time.perf_counter() - t0
    assert ei.value.status == 4 and code.value == phase and "gave up waiting" in ei.value.message
    assert 0.015 <= dt < 5.0, dt
    engine.synchronize()


@pytest.mark.gpu
def test_synchronize_with_a_host_deadline(engine):
    """sync_checked()'s timeout path (src/gpu/context.rs:448-505): a long but finite queue of
    kernels and a deadline far shorter than the queue -> VB_ERR_TIMEOUT; nothing is cancelled, a
    plain synchronize then waits for the rest and the results are the ordinary ones."""
    from volta_b200 import Adam, Tensor, VoltaB200Error
    n = 1 << 24
    t = Tensor(np.ones(n, np.float32))
    opt = Adam([t], 1e-3, (0.9, 0.999), 1e-8, 0.0, engine=engine)
    t.grad = np.full(n, 0.5, np.float32)
    engine.synchronize()
    for _ in range(400):       # ~70 us each on a B200: tens of milliseconds of queued work
        opt.step()
    with pytest.raises(VoltaB200Error) as ei:
        engine.synchronize(timeout_ms=0.05)
    assert ei.value.status == 4 and "did not drain" in ei.value.message
    engine.synchronize()                      # the queue still completes
    engine.synchronize(timeout_ms=1000.0)     # and an idle stream meets any deadline
    assert opt.t == 400 and np.all(t.data < 1.0)
    opt.close()


def test_host_side_faults_return_codes():
    """Invalid descriptors and states are refused on the host, before any launch."""
    from volta_b200 import _lib
    lib = _lib.load()
    hp = _lib.StepParams(7, 1e-3, 0.9, 0.999, 1.0, 1e-8, 0.0, 0.0)
    assert lib.vb_multi_tensor_step(None, C.byref(hp), 0, None, None, None, None, None) == 1
    assert lib.vb_multi_tensor_step_static(None, C.byref(hp), 0, None, None, None, None, None) == 1
    assert lib.vb_debug_gemm_wait_expiry(None, 0, None) == 1
    assert lib.vb_engine_comm_init(None, None, 0, 1) == 1
    assert lib.vb_optimizer_open_peers(None, None, 0) == 1


def _step_args(op, p, g, a, b, n=8):
    from volta_b200 import _lib
    hp = _lib.StepParams(op, 1e-3, 0.9, 0.999, 1.0, 1e-8, 0.0, 0.0)
    arr = lambda v: (C.c_void_p * 1)(v)  # noqa: E731
    return C.byref(hp), 1, (C.c_int64 * 1)(n), arr(p), arr(g), arr(a), arr(b)


@pytest.mark.parametrize("entry", ["vb_multi_tensor_step", "vb_multi_tensor_step_static"])
def test_misaligned_state_pointers_are_refused_before_any_launch(entry):
    """A state pointer that is 2 bytes off would reach the kernel's scalar loads and raise a
    misaligned-address fault on the GPU.  Both caller-buffer entry points refuse it on the host
    (the check needs no device, so it also runs where there is none): every array the op reads
    must be 4-byte aligned; arrays the op does not read are not looked at."""
    from volta_b200 import _lib
    lib = _lib.load()
    fn = getattr(lib, entry)
    ok = 0x10000
    for op, p, g, a, b in ((2, ok, ok, ok + 2, ok), (2, ok, ok, ok, ok + 2), (1, ok, ok, ok + 1, ok),
                           (0, ok + 2, ok, ok, ok), (2, ok, ok + 3, ok, ok)):
        assert fn(None, *_step_args(op, p, g, a, b)) == 1
        assert b"4-byte aligned" in lib.vb_last_error(), (op, lib.vb_last_error())
    # op 1 never reads state2, op 0 reads neither state: those pointers may be anything
    for op, a, b in ((1, ok, ok + 2), (0, ok + 2, ok + 1)):
        assert fn(None, *_step_args(op, ok, ok, a, b)) == 1
        assert b"engine is null" in lib.vb_last_error()   # got past the pointer checks


def test_plan_fingerprints_expose_a_rank_with_a_different_plan():
    """Pure host: same plan -> same fingerprint whatever the rank; a different tensor list,
    hyper-parameter, mode or world size -> VB_ERR_STATE naming the first rank that differs."""
    from volta_b200 import VoltaB200Error, plan_fingerprint, verify_plan
    base = plan_fingerprint("adam", [1024, 7, 300], [1e-3, 0.9, 0.999, 1e-8, 0.01], world_size=4)
    assert base == plan_fingerprint("adam", [1024, 7, 300], [1e-3, 0.9, 0.999, 1e-8, 0.01], world_size=4)
    verify_plan([base] * 4)
    others = [plan_fingerprint("adam", [1024, 7, 301], [1e-3, 0.9, 0.999, 1e-8, 0.01], world_size=4),
              plan_fingerprint("adam", [1024, 7, 300], [2e-3, 0.9, 0.999, 1e-8, 0.01], world_size=4),
              plan_fingerprint("adam", [1024, 7, 300], [1e-3, 0.9, 0.999, 1e-8, 0.01], world_size=2),
              plan_fingerprint("sgd", [1024, 7, 300], [1e-3, 0.9, 0.999, 1e-8, 0.01], world_size=4),
              plan_fingerprint("muon", [(32, 32), (7,), (10, 30)], [0.1, 0.9], [1, 5, 1], world_size=4),
              plan_fingerprint("muon", [(32, 32), (7,), (30, 10)], [0.1, 0.9], [1, 5, 1], world_size=4),
              plan_fingerprint("muon", [(32, 32), (7,), (10, 30)], [0.1, 0.9], [1, 5, 2], world_size=4)]
    assert len(set(others + [base])) == len(others) + 1
    with pytest.raises(VoltaB200Error) as ei:
        verify_plan([base, base, others[0], base])
    assert ei.value.status == 5 and "rank 2" in ei.value.message
