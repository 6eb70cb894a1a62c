"""ctypes binding of the CPU oracle (``volta_cpu_oracle.c``).

TEST INFRASTRUCTURE ONLY: the checker for the CUDA path and the timed CPU baseline.
Nothing in the ``volta_b200`` package imports this module; only the tests, the smoke
check and the benchmark's CPU-baseline / reference arm do.

The arithmetic lives in C (see the header of ``volta_cpu_oracle.c`` for the reference
file:line each function restates); this module only marshals numpy float32 arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "volta_cpu_oracle.c")
_SO = os.path.join(_HERE, "libvolta_cpu_oracle.so")

# -ffp-contract=off: Rust never fuses a*b+c on its own; fmaf() appears in the source only
# where the reference writes mul_add.  -mfma lets fmaf() compile to one instruction
# (same result as libm's fmaf, which is correctly rounded either way).
CFLAGS = ["-O3", "-ffp-contract=off", "-fno-fast-math", "-mavx2", "-mfma", "-fopenmp",
          "-shared", "-fPIC", "-std=c11"]


def build(force: bool = False) -> str:
    """Compile the oracle with gcc if the shared object is missing or stale."""
    if (not force and os.path.exists(_SO)
            and os.path.getmtime(_SO) >= os.path.getmtime(_SRC)):
        return _SO
    tmp = _SO + f".tmp{os.getpid()}"
    subprocess.run(["gcc", *CFLAGS, "-o", tmp, _SRC, "-lm"], check=True)
    os.replace(tmp, _SO)
    return _SO


_lib = None
_f32p = C.POINTER(C.c_float)


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.vo_powi_f32.restype = C.c_float
        L.vo_powi_f32.argtypes = [C.c_float, C.c_int]
        L.vo_adam_bias_scales.argtypes = [C.c_float, C.c_float, C.c_int, _f32p, _f32p]
        L.vo_adam_step.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_size_t, C.c_float, C.c_float,
                                   C.c_float, C.c_float, C.c_float, C.c_int, _f32p]
        L.vo_sgd_step.argtypes = [_f32p, _f32p, _f32p, C.c_size_t, C.c_float, C.c_float,
                                  C.c_float, _f32p]
        L.vo_wgsl_optimizer_step.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_size_t, C.c_uint32,
                                             C.c_float, C.c_float, C.c_float, C.c_float,
                                             C.c_float, C.c_float]
        L.vo_transpose_2d.argtypes = [_f32p, _f32p, C.c_size_t, C.c_size_t]
        for name in ("vo_sgemm", "vo_sgemm_f64acc"):
            getattr(L, name).argtypes = [_f32p, _f32p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t]
        L.vo_sum_sq_sequential.restype = C.c_float
        L.vo_sum_sq_sequential.argtypes = [_f32p, C.c_size_t]
        L.vo_newton_schulz.argtypes = [_f32p, C.c_size_t, C.c_size_t, C.c_int, C.c_int]
        L.vo_muon_step.argtypes = [_f32p, _f32p, _f32p, C.c_size_t, C.c_size_t, C.c_float,
                                   C.c_float, C.c_int, C.c_int, C.c_int, _f32p]
        L.vo_max_threads.restype = C.c_int
        L.vo_set_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _p(a):
    if a is None:
        return None
    assert isinstance(a, np.ndarray) and a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_f32p)


def powi(a: float, b: int) -> np.float32:
    return np.float32(lib().vo_powi_f32(np.float32(a), int(b)))


def adam_bias_scales(beta1, beta2, t):
    s1, s2 = C.c_float(), C.c_float()
    lib().vo_adam_bias_scales(beta1, beta2, t, C.byref(s1), C.byref(s2))
    return np.float32(s1.value), np.float32(s2.value)


def set_threads(n: int) -> None:
    lib().vo_set_threads(n)


def max_threads() -> int:
    return lib().vo_max_threads()


class Adam:
    """Volta's ``Adam`` on CPU tensors (src/nn/optim/adam.rs:5-95).

    ``params`` is a list of float32 numpy arrays updated in place; ``grads[i] is None``
    reproduces the skip rule of adam.rs:81-84 (``t`` still advances, adam.rs:71).
    """

    def __init__(self, params, lr, betas, eps, weight_decay):
        self.params = params
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.m = [np.zeros(p.size, np.float32) for p in params]
        self.v = [np.zeros(p.size, np.float32) for p in params]
        self.t = 0
        self._scratch = np.empty(max([p.size for p in params] + [1]), np.float32)

    def step(self, grads):
        self.t += 1
        L = lib()
        for p, g, m, v in zip(self.params, grads, self.m, self.v):
            if g is None:
                continue
            L.vo_adam_step(_p(p.reshape(-1)), _p(g.reshape(-1)), _p(m), _p(v), p.size, self.lr,
                           self.betas[0], self.betas[1], self.eps, self.weight_decay, self.t,
                           _p(self._scratch))


class SGD:
    """Volta's ``SGD`` on CPU tensors (src/nn/optim/sgd.rs:11-90,189-238)."""

    def __init__(self, params, lr, momentum, weight_decay):
        self.params = params
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        # sgd.rs:30: velocity buffers exist only when momentum > 0.0
        self.velocity = [np.zeros(p.size, np.float32) for p in params] if momentum > 0.0 else []
        self._scratch = np.empty(max([p.size for p in params] + [1]), np.float32)

    def step(self, grads):
        L = lib()
        for i, (p, g) in enumerate(zip(self.params, grads)):
            if g is None:
                continue
            vel = self.velocity[i] if self.velocity else None
            L.vo_sgd_step(_p(p.reshape(-1)), _p(g.reshape(-1)), _p(vel), p.size, self.lr,
                          self.momentum, self.weight_decay, _p(self._scratch))


def muon_dims(shape):
    """(rows, cols) flattening of src/nn/optim/muon.rs:117-130."""
    shape = tuple(int(s) for s in shape)
    if len(shape) < 2:
        return (shape[0] if shape else 1), 1
    cols = 1
    for s in shape[1:]:
        cols *= s
    return shape[0], cols


class Muon:
    """Volta's ``Muon`` (src/nn/optim/muon.rs:8-163).  ``gemm_mode`` 0 = f32 blocked
    fused-multiply-add SGEMM, 1 = f64-accumulating SGEMM.  ``last_update[i]`` holds the
    orthogonalised update of the most recent step."""

    def __init__(self, params, lr, momentum, nesterov, ns_steps, gemm_mode=0):
        self.params = params
        self.lr, self.momentum, self.nesterov, self.ns_steps = lr, momentum, nesterov, ns_steps
        self.gemm_mode = gemm_mode
        self.velocity = [np.zeros(p.size, np.float32) for p in params]
        self.last_update = [None] * len(params)

    def step(self, grads):
        L = lib()
        for i, (p, g) in enumerate(zip(self.params, grads)):
            if g is None:
                continue
            rows, cols = muon_dims(p.shape)
            upd = np.empty(p.size, np.float32)
            L.vo_muon_step(_p(p.reshape(-1)), _p(g.reshape(-1)), _p(self.velocity[i]), rows, cols,
                           self.lr, self.momentum, int(self.nesterov), self.ns_steps,
                           self.gemm_mode, _p(upd))
            self.last_update[i] = upd.reshape(p.shape)


def newton_schulz(x: np.ndarray, steps: int, gemm_mode: int = 0) -> np.ndarray:
    """Muon::newton_schulz on a copy of the 2-D array ``x``."""
    rows, cols = x.shape
    out = np.ascontiguousarray(x, np.float32).copy()
    lib().vo_newton_schulz(_p(out.reshape(-1)), rows, cols, steps, gemm_mode)
    return out


def sgemm(a, b, f64acc=False):
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), np.float32)
    fn = lib().vo_sgemm_f64acc if f64acc else lib().vo_sgemm
    fn(_p(np.ascontiguousarray(a)), _p(np.ascontiguousarray(b)), _p(c), m, k, n)
    return c


def sum_sq_sequential(x) -> np.float32:
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    return np.float32(lib().vo_sum_sq_sequential(_p(x), x.size))


def wgsl_optimizer_step(params, grads, state1, state2, op, lr, beta1, beta2, t, eps, wd):
    lib().vo_wgsl_optimizer_step(_p(params), _p(grads), _p(state1), _p(state2), params.size, op,
                                 lr, beta1, beta2, float(t), eps, wd)
