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
    opt = Muon([w], 0.1, 0.0, False, 5, ns_mode=VB_NS_BF16, engine=engine)
    w.grad = g
    opt.step()
    assert rel_frobenius(opt.last_update(0), oracle.newton_schulz(g, 5)) <= 2e-2
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
