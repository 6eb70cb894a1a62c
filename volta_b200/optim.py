"""Host-side mirror of Volta's optimizer API over the C ABI.

Same names, argument order and meaning as the reference
(``Adam::new(params, lr, betas, eps, weight_decay)`` src/nn/optim/adam.rs:18-24,
``SGD::new(params, lr, momentum, weight_decay)`` src/nn/optim/sgd.rs:28,
``Muon::new(params, lr, momentum, nesterov, ns_steps)`` src/nn/optim/muon.rs:19-25;
each with ``step()`` and ``zero_grad()``), so a training loop written against Volta reads
the same here:

    opt = Adam(model_parameters, 1e-3, (0.9, 0.999), 1e-8, 0.0)
    opt.zero_grad(); ...set p.grad...; opt.step()

All arithmetic runs in the CUDA library; this module only moves bytes and keeps handles.
"""
from __future__ import annotations

import ctypes as C
from typing import Iterable, List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import (VB_NS_BF16, VB_NS_F32, VB_NS_F32_TC, VB_STEP_DEFAULT, VB_STEP_EXCHANGE_BF16, VB_STEP_MEAN_GRADS,
                   VB_STEP_NO_EXCHANGE, VB_STEP_REDUCE_GRADS,
                   VoltaB200Error, call)

__all__ = ["Engine", "Tensor", "Adam", "SGD", "Muon", "default_engine", "multi_tensor_step", "accumulate_grad", "plan_replicated_fraction",
           "verify_plan", "plan_fingerprint",
           "VoltaB200Error", "VB_NS_F32", "VB_NS_BF16", "VB_NS_F32_TC", "VB_STEP_NO_EXCHANGE", "VB_STEP_EXCHANGE_BF16", "VB_STEP_REDUCE_GRADS", "VB_STEP_MEAN_GRADS"]


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class Engine:
    """One CUDA device + stream (the role of Volta's global GPU context,
    src/gpu/mod.rs:30-47).  Optionally one rank of a multi-GPU group."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        call("vb_engine_create", int(device), C.byref(self._h))
        self.device = int(device)

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h:
            call("vb_engine_destroy", self._h)
            self._h = C.c_void_p()

    def synchronize(self, timeout_ms: Optional[float] = None) -> None:
        """Waits for the engine's stream.  With ``timeout_ms`` the wait has a deadline on the host
        (the counterpart of ``sync_checked()``, src/gpu/context.rs:448-505): ``VB_ERR_TIMEOUT`` is
        raised if work is still queued when it passes; nothing is cancelled."""
        if timeout_ms is None:
            call("vb_engine_synchronize", self._h)
        else:
            call("vb_engine_synchronize_deadline", self._h, float(timeout_ms))

    def set_wait_limit_ms(self, ms: int) -> None:
        """Bound of every device-side wait on another rank (default 5000 ms)."""
        call("vb_engine_set_wait_limit_ms", self._h, int(ms))

    def set_replicated_fraction(self, fraction: float) -> None:
        """Adam/SGD optimizers created from now on keep the last ``fraction`` of their arena out of
        the sharding: every rank updates that tail itself (state for it on every rank, complete
        gradients needed on every rank) and it never crosses NVLink.  0 = plain ZeRO-1 slices."""
        call("vb_engine_set_replicated_fraction", self._h, float(fraction))

    @property
    def stream(self) -> int:
        """The engine's ``cudaStream_t`` as an integer."""
        s = C.c_void_p()
        call("vb_engine_stream", self._h, C.byref(s))
        return int(s.value or 0)

    @property
    def launch_count(self) -> int:
        n = C.c_uint64()
        call("vb_engine_launch_count", self._h, C.byref(n))
        return int(n.value)

    PHASES = {"update": 0, "muon_pre": 1, "muon_ns": 2, "muon_apply": 3, "exchange": 4, "host_h2d": 5, "host_d2h": 6}

    def set_profiling(self, enabled: bool) -> None:
        call("vb_engine_set_profiling", self._h, int(bool(enabled)))

    def profile(self, phase: str):
        """(total device ms, number of brackets) of one phase since the last query."""
        ms, n = C.c_double(), C.c_int64()
        call("vb_engine_profile", self._h, self.PHASES[phase], C.byref(ms), C.byref(n))
        return float(ms.value), int(n.value)

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        call("vb_comm_unique_id", buf)
        return buf.raw

    def init_comm(self, unique_id: bytes, rank: int, world_size: int) -> None:
        if len(unique_id) != 128:
            raise ValueError("unique_id must be 128 bytes")
        call("vb_engine_comm_init", self._h, C.c_char_p(unique_id), int(rank), int(world_size))

    @property
    def rank(self) -> int:
        r, w = C.c_int(), C.c_int()
        call("vb_engine_rank", self._h, C.byref(r), C.byref(w))
        return r.value

    @property
    def world_size(self) -> int:
        r, w = C.c_int(), C.c_int()
        call("vb_engine_rank", self._h, C.byref(r), C.byref(w))
        return w.value


_default_engine: Optional[Engine] = None


def default_engine() -> Engine:
    """Process-wide engine on device 0, created on first use."""
    global _default_engine
    if _default_engine is None:
        _default_engine = Engine(0)
    return _default_engine


class PinnedBuffer:
    """Page-locked float32 host array (``vb_host_alloc_pinned``)."""

    def __init__(self, n: int):
        self._p = C.c_void_p()
        call("vb_host_alloc_pinned", C.byref(self._p), max(int(n), 1) * 4)
        self.array = np.ctypeslib.as_array(C.cast(self._p, C.POINTER(C.c_float)), shape=(int(n),))

    def free(self) -> None:
        if self._p:
            self.array = None
            call("vb_host_free_pinned", self._p)
            self._p = C.c_void_p()


class Tensor:
    """What Volta's optimizers see of a ``Tensor`` (src/tensor.rs:38-46): a shape, f32
    ``data`` and an optional ``grad``.  Before an optimizer takes it, the values live in
    host memory; afterwards they live in the optimizer's device arena, ``data`` reads them
    back and assigning ``grad`` uploads (``None`` = no gradient)."""

    def __init__(self, data, shape: Optional[Sequence[int]] = None, requires_grad: bool = True):
        arr = _f32(data)
        self.shape = tuple(int(s) for s in (shape if shape is not None else arr.shape))
        if int(np.prod(self.shape, dtype=np.int64)) != arr.size:
            raise ValueError("shape does not match data")
        self.requires_grad = requires_grad
        self._host = arr.reshape(-1).copy()
        self._host_grad: Optional[np.ndarray] = None
        self._opt: Optional["_Optimizer"] = None
        self._index = -1

    @property
    def size(self) -> int:
        return int(self._host.size)

    @property
    def data(self) -> np.ndarray:
        if self._opt is not None:
            self._opt._download_params(self._index, self._host)
        return self._host.reshape(self.shape)

    @data.setter
    def data(self, value) -> None:
        arr = _f32(value).reshape(-1)
        if arr.size != self._host.size:
            raise ValueError("size mismatch")
        self._host[:] = arr
        if self._opt is not None:
            self._opt._upload_params(self._index, self._host)

    @property
    def grad(self) -> Optional[np.ndarray]:
        if self._opt is not None:
            return self._opt._download_grad(self._index, self.shape)
        return None if self._host_grad is None else self._host_grad.reshape(self.shape)

    @grad.setter
    def grad(self, value) -> None:
        if value is None:
            self._host_grad = None
            if self._opt is not None:
                self._opt._set_present(self._index, False)
            return
        arr = _f32(value).reshape(-1)
        if arr.size != self._host.size:
            raise ValueError("gradient size mismatch")
        if self._opt is not None:
            self._opt._upload_grad(self._index, arr)
        else:
            self._host_grad = arr.copy()


def accumulate_grad(tensor: "Tensor", contribution) -> None:
    """``RawTensor::accumulate_grad`` (src/autograd.rs:140-148,158-184) for a tensor held by an
    optimizer: the first contribution becomes the gradient, later ones are added on the device."""
    arr = _f32(contribution).reshape(-1)
    if tensor._opt is None:
        tensor._host_grad = arr.copy() if tensor._host_grad is None else (tensor._host_grad + arr).astype(np.float32)
        return
    if arr.size != tensor.size:
        raise ValueError("gradient size mismatch")
    call("vb_optimizer_accumulate_grad", tensor._opt._h, tensor._index, arr.ctypes.data_as(C.c_void_p), arr.size)
    tensor._opt._present[tensor._index] = True


class _Optimizer:
    def __init__(self, params: Iterable[Tensor], engine: Optional[Engine]):
        self.params: List[Tensor] = list(params)
        for p in self.params:
            if not isinstance(p, Tensor):
                raise TypeError("params must be volta_b200.Tensor objects")
            if p._opt is not None:
                raise ValueError("a Tensor can belong to one optimizer")
        self.engine = engine if engine is not None else default_engine()
        self._h = C.c_void_p()
        self._present = [False] * len(self.params)

    # -- construction helpers --------------------------------------------------------------
    def _sizes(self):
        n = len(self.params)
        return n, (C.c_int64 * max(n, 1))(*[p.size for p in self.params])

    def _adopt(self) -> None:
        for i, p in enumerate(self.params):
            p._opt, p._index = self, i
            self._upload_params(i, p._host)
            if p._host_grad is not None:
                self._upload_grad(i, p._host_grad)
                p._host_grad = None

    def close(self) -> None:
        if self._h:
            for p in self.params:
                if p._opt is self:
                    self._download_params(p._index, p._host)
                    p._opt, p._index = None, -1
            call("vb_optimizer_destroy", self._h)
            self._h = C.c_void_p()

    # -- tensor traffic --------------------------------------------------------------------
    def _upload_params(self, i, arr):
        call("vb_optimizer_upload_params", self._h, i, arr.ctypes.data_as(C.c_void_p), arr.size)

    def _download_params(self, i, out):
        call("vb_optimizer_download_params", self._h, i, out.ctypes.data_as(C.c_void_p), out.size)

    def _upload_grad(self, i, arr):
        call("vb_optimizer_upload_grad", self._h, i, arr.ctypes.data_as(C.c_void_p), arr.size)
        self._present[i] = True

    def _download_grad(self, i, shape):
        if not self._present[i]:
            return None
        out = np.empty(self.params[i].size, np.float32)
        call("vb_optimizer_download_grad", self._h, i, out.ctypes.data_as(C.c_void_p), out.size)
        return out.reshape(shape)

    def _set_present(self, i, present: bool):
        call("vb_optimizer_set_grad_present", self._h, i, int(present))
        self._present[i] = bool(present)

    # -- the reference API -----------------------------------------------------------------
    def step(self, flags: int = VB_STEP_DEFAULT) -> None:
        """``step()``: one fused update of every parameter that has a gradient."""
        call("vb_optimizer_step_ex", self._h, int(flags))

    def step_host(self, grads_arena: np.ndarray, params_arena: np.ndarray, pieces: int = 8) -> None:
        """One step of a host-resident model: gradients in, parameters out, both as host images of
        the arena (``arena_layout()``); upload, update and download are pipelined piece by piece."""
        assert grads_arena.dtype == np.float32 and params_arena.dtype == np.float32
        assert grads_arena.flags.c_contiguous and params_arena.flags.c_contiguous
        assert grads_arena.size == params_arena.size
        call("vb_optimizer_step_host", self._h, grads_arena.ctypes.data_as(C.c_void_p),
             params_arena.ctypes.data_as(C.c_void_p), int(pieces))
        self._present = [True] * len(self.params)

    def zero_grad(self) -> None:
        """``zero_grad()``: every ``grad`` becomes ``None`` (adam.rs:62-66)."""
        call("vb_optimizer_zero_grad", self._h)
        self._present = [False] * len(self.params)

    # -- extras (state is private in the reference; exposed for parity checks/resume) ------
    def set_lr(self, lr: float) -> None:
        call("vb_optimizer_set_lr", self._h, float(lr))

    def state(self, i: int, which: int = 0) -> np.ndarray:
        out = np.empty(self.params[i].size, np.float32)
        lo, hi = C.c_int64(), C.c_int64()
        call("vb_optimizer_export_state", self._h, i, which, out.ctypes.data_as(C.c_void_p), out.size,
             C.byref(lo), C.byref(hi))
        return out

    def state_owned_range(self, i: int, which: int = 0):
        out = np.empty(self.params[i].size, np.float32)
        lo, hi = C.c_int64(), C.c_int64()
        call("vb_optimizer_export_state", self._h, i, which, out.ctypes.data_as(C.c_void_p), out.size,
             C.byref(lo), C.byref(hi))
        return int(lo.value), int(hi.value)

    def load_state(self, i: int, which: int, values) -> None:
        arr = _f32(values).reshape(-1)
        call("vb_optimizer_import_state", self._h, i, which, arr.ctypes.data_as(C.c_void_p), arr.size)

    def reset_state(self) -> None:
        """Moments / velocity back to zero and ``t`` to 0, as a newly constructed optimizer has them."""
        call("vb_optimizer_reset_state", self._h)

    @property
    def t(self) -> int:
        t = C.c_int64()
        call("vb_optimizer_get_t", self._h, C.byref(t))
        return int(t.value)

    @t.setter
    def t(self, value: int) -> None:
        call("vb_optimizer_set_t", self._h, int(value))

    # -- do all ranks describe the same optimizer? -------------------------------------------
    def plan_fingerprint(self) -> int:
        """64-bit hash of the tensor list, hyper-parameters, mode and world size (not of the
        rank).  Gather it from every rank and pass the list to ``verify_plan``."""
        fp = C.c_uint64()
        call("vb_optimizer_plan_fingerprint", self._h, C.byref(fp))
        return int(fp.value)

    # -- fused exchange over NVLink peer memory (sharded Adam / SGD) -------------------------
    def ipc_handle(self) -> bytes:
        """CUDA IPC handle (64 bytes) of this rank's parameter arena."""
        buf = C.create_string_buffer(64)
        call("vb_optimizer_ipc_handle", self._h, buf)
        return buf.raw

    def open_peers(self, handles: Sequence[bytes]) -> None:
        """``handles[r]`` = rank r's ``ipc_handle()``.  Afterwards ``step()`` stores updated
        parameters straight into the peers' arenas instead of running an all-gather."""
        blob = b"".join(handles)
        if len(blob) != 64 * len(handles):
            raise ValueError("every handle must be 64 bytes")
        call("vb_optimizer_open_peers", self._h, C.c_char_p(blob), len(handles))

    def peer_copy_probe(self, reps: int = 4) -> float:
        """Device milliseconds per repetition of "every rank copies its slice to every peer with
        the copy engines, all at once" (``vb_optimizer_peer_copy_probe``): the fabric's own rate
        for the parameter exchange, measured in the running job.  All ranks call it together."""
        ms = C.c_double()
        call("vb_optimizer_peer_copy_probe", self._h, int(reps), C.byref(ms))
        return float(ms.value)

    # -- data-parallel gradients: reduce-scatter fused into the update kernel's loads -------
    def ipc_handle_grads(self) -> bytes:
        buf = C.create_string_buffer(64)
        call("vb_optimizer_ipc_handle_grads", self._h, buf)
        return buf.raw

    def open_peers_grads(self, handles: Sequence[bytes]) -> None:
        """``handles[r]`` = rank r's ``ipc_handle_grads()``; afterwards ``step(VB_STEP_REDUCE_GRADS)``
        (or ``VB_STEP_MEAN_GRADS``) updates with the sum (mean) of all ranks' gradients."""
        blob = b"".join(handles)
        if len(blob) != 64 * len(handles):
            raise ValueError("every handle must be 64 bytes")
        call("vb_optimizer_open_peers_grads", self._h, C.c_char_p(blob), len(handles))

    # -- bf16 copies of the parameters, written next to the f32 master ----------------------
    def enable_bf16_params(self) -> None:
        """Keeps ``bf16[i] == round_to_nearest_even(param[i])`` in a second arena from now on;
        ``step(VB_STEP_EXCHANGE_BF16)`` then exchanges only these copies between ranks."""
        call("vb_optimizer_enable_bf16_params", self._h)

    def refresh_bf16_params(self) -> None:
        call("vb_optimizer_refresh_bf16_params", self._h)

    def bf16_params(self, i: int) -> np.ndarray:
        """Parameter ``i``'s bf16 copy as raw 16-bit words (``uint16``) in the tensor's shape."""
        shape = self.params[i].shape
        n = int(np.prod(shape, dtype=np.int64))
        out = np.empty(n, np.uint16)
        call("vb_optimizer_download_params_bf16", self._h, i, out.ctypes.data_as(C.c_void_p), n)
        return out.reshape(shape)

    def bf16_param_ptr(self, i: int) -> int:
        p = C.c_void_p()
        call("vb_optimizer_param_bf16_ptr", self._h, i, C.byref(p))
        return int(p.value or 0)

    def ipc_handle_bf16(self) -> bytes:
        buf = C.create_string_buffer(64)
        call("vb_optimizer_ipc_handle_bf16", self._h, buf)
        return buf.raw

    def open_peers_bf16(self, handles: Sequence[bytes]) -> None:
        """``handles[r]`` = rank r's ``ipc_handle_bf16()``: the copies then reach the peers by
        stores fused into the update / apply kernel instead of an NCCL call."""
        blob = b"".join(handles)
        if len(blob) != 64 * len(handles):
            raise ValueError("every handle must be 64 bytes")
        call("vb_optimizer_open_peers_bf16", self._h, C.c_char_p(blob), len(handles))

    # -- whole-arena access (one transfer for all tensors) ---------------------------------
    def arena_layout(self):
        """(param_ptr, grad_ptr, arena_elements, offsets[n_tensors])."""
        n = len(self.params)
        p, g, e = C.c_void_p(), C.c_void_p(), C.c_int64()
        offs = (C.c_int64 * max(n, 1))()
        call("vb_optimizer_arena", self._h, C.byref(p), C.byref(g), C.byref(e), offs)
        return int(p.value or 0), int(g.value or 0), int(e.value), [int(offs[i]) for i in range(n)]

    def upload_arena(self, which: int, host: np.ndarray) -> None:
        assert host.dtype == np.float32 and host.flags.c_contiguous
        call("vb_optimizer_upload_arena", self._h, which, host.ctypes.data_as(C.c_void_p), host.size)
        if which == 1:
            self._present = [True] * len(self.params)

    def download_arena(self, which: int, host: np.ndarray) -> None:
        assert host.dtype == np.float32 and host.flags.c_contiguous
        call("vb_optimizer_download_arena", self._h, which, host.ctypes.data_as(C.c_void_p), host.size)

    def owned_range(self):
        """[begin, end) of the arena whose state this rank owns."""
        lo, hi = C.c_int64(), C.c_int64()
        call("vb_optimizer_owned_range", self._h, C.byref(lo), C.byref(hi))
        return int(lo.value), int(hi.value)

    def replicated_range(self):
        """[begin, end) of the arena every rank updates itself (empty unless the engine had a
        replicated fraction set when the optimizer was created)."""
        lo, hi = C.c_int64(), C.c_int64()
        call("vb_optimizer_replicated_range", self._h, C.byref(lo), C.byref(hi))
        return int(lo.value), int(hi.value)

    def upload_arena_range(self, which: int, host: np.ndarray, begin: int) -> None:
        assert host.dtype == np.float32 and host.flags.c_contiguous
        call("vb_optimizer_upload_arena_range", self._h, which, host.ctypes.data_as(C.c_void_p), int(begin), host.size)
        if which == 1:
            self._present = [True] * len(self.params)

    def download_arena_range(self, which: int, host: np.ndarray, begin: int) -> None:
        assert host.dtype == np.float32 and host.flags.c_contiguous
        call("vb_optimizer_download_arena_range", self._h, which, host.ctypes.data_as(C.c_void_p), int(begin),
             host.size)

    def mark_all_grads_present(self) -> None:
        for i in range(len(self.params)):
            if not self._present[i]:
                self._set_present(i, True)


class Adam(_Optimizer):
    """``Adam::new(params, lr, betas, eps, weight_decay)`` (src/nn/optim/adam.rs:18-60):
    bias-corrected Adam with L2 weight decay folded into the gradient."""

    def __init__(self, params, lr: float, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, engine: Optional[Engine] = None):
        super().__init__(params, engine)
        n, sizes = self._sizes()
        call("vb_adam_create", self.engine._h, n, sizes, lr, betas[0], betas[1], eps, weight_decay,
             C.byref(self._h))
        self._adopt()


class SGD(_Optimizer):
    """``SGD::new(params, lr, momentum, weight_decay)`` (src/nn/optim/sgd.rs:28-52)."""

    def __init__(self, params, lr: float, momentum: float = 0.0, weight_decay: float = 0.0,
                 engine: Optional[Engine] = None):
        super().__init__(params, engine)
        n, sizes = self._sizes()
        call("vb_sgd_create", self.engine._h, n, sizes, lr, momentum, weight_decay, C.byref(self._h))
        self._adopt()


def muon_dims(shape):
    """(rows, cols) as Muon::step flattens a shape (src/nn/optim/muon.rs:117-130)."""
    shape = tuple(int(s) for s in shape)
    if len(shape) < 2:
        return (shape[0] if shape else 1), 1
    cols = 1
    for s in shape[1:]:
        cols *= s
    return shape[0], cols


class Muon(_Optimizer):
    """``Muon::new(params, lr, momentum, nesterov, ns_steps)`` (src/nn/optim/muon.rs:19-38).
    ``ns_mode`` picks the Newton-Schulz arithmetic: ``VB_NS_F32`` (bit-faithful, CUDA cores),
    ``VB_NS_BF16`` (tcgen05 bf16 tensor cores) or ``VB_NS_F32_TC`` (f32-accurate on the tensor
    cores through three-way bf16 splitting)."""

    def __init__(self, params, lr: float, momentum: float, nesterov: bool, ns_steps: int,
                 ns_mode: int = VB_NS_F32, engine: Optional[Engine] = None, keep_update: bool = False):
        """``keep_update``: also store the orthogonalised update of every step so that
        ``last_update(i)`` can return it (the tensor-core modes otherwise apply it to the weights
        inside their last launch and never write it; the reference's ``update`` is a temporary too)."""
        super().__init__(params, engine)
        n = len(self.params)
        dims = [muon_dims(p.shape) for p in self.params]
        rows = (C.c_int64 * max(n, 1))(*[d[0] for d in dims])
        cols = (C.c_int64 * max(n, 1))(*[d[1] for d in dims])
        call("vb_muon_create", self.engine._h, n, rows, cols, lr, momentum, int(bool(nesterov)),
             int(ns_steps), int(ns_mode), C.byref(self._h))
        if keep_update:
            call("vb_muon_set_keep_update", self._h, 1)
        self._adopt()

    def last_update(self, i: int) -> np.ndarray:
        """The orthogonalised update of the last step for parameter ``i``."""
        out = np.empty(self.params[i].size, np.float32)
        call("vb_muon_download_update", self._h, i, out.ctypes.data_as(C.c_void_p), out.size)
        return out.reshape(self.params[i].shape)

    @property
    def last_ns_flops(self) -> float:
        f = C.c_double()
        call("vb_muon_last_ns_flops", self._h, C.byref(f))
        return float(f.value)


def verify_plan(fingerprints: Sequence[int]) -> None:
    """Raises ``VoltaB200Error`` (``VB_ERR_STATE``) on every rank if the ranks' plan fingerprints
    (gathered in rank order over the host's own transport) differ: a sharded step is a collective
    and must not be launched by ranks that describe different optimizers."""
    n = len(fingerprints)
    arr = (C.c_uint64 * max(n, 1))(*[int(f) for f in fingerprints])
    bad = C.c_int(-1)
    call("vb_plan_fingerprints_agree", arr, n, C.byref(bad))


def plan_replicated_fraction(bytes_per_element: float, world_size: int, hbm_gb_per_s: float,
                             link_gb_per_s: float) -> float:
    """The replicated fraction at which a sharded step's HBM time and NVLink time are equal
    (``vb_plan_replicated_fraction``): Adam moves 28 B per element through HBM, SGD with momentum
    20, plain SGD 12; the rates are those of the update kernel and of the fused exchange."""
    out = C.c_double()
    call("vb_plan_replicated_fraction", float(bytes_per_element), int(world_size), float(hbm_gb_per_s),
         float(link_gb_per_s), C.byref(out))
    return float(out.value)


def plan_fingerprint(kind: str, sizes_or_shapes, hyper: Sequence[float], ints: Sequence[int] = (),
                     world_size: int = 1) -> int:
    """The same fingerprint without a device (``vb_plan_fingerprint``): ``kind`` "adam" | "sgd" |
    "muon"; element counts for Adam / SGD, shapes for Muon."""
    k = {"adam": 0, "sgd": 1, "muon": 2}[kind]
    if k == 2:
        dims = [muon_dims(s) for s in sizes_or_shapes]
        a, b = [d[0] for d in dims], [d[1] for d in dims]
    else:
        a, b = [int(x) for x in sizes_or_shapes], None
    n = len(a)
    arr_a = (C.c_int64 * max(n, 1))(*a)
    arr_b = (C.c_int64 * max(n, 1))(*b) if b is not None else None
    hy = (C.c_float * max(len(hyper), 1))(*[float(x) for x in hyper])
    it = (C.c_int32 * max(len(ints), 1))(*[int(x) for x in ints])
    fp = C.c_uint64()
    call("vb_plan_fingerprint", k, n, arr_a, arr_b, hy, len(hyper), it, len(ints), int(world_size), C.byref(fp))
    return int(fp.value)


def multi_tensor_step(engine: Engine, op: int, sizes: Sequence[int], params: Sequence[int],
                      grads: Sequence[int], state1: Optional[Sequence[int]] = None,
                      state2: Optional[Sequence[int]] = None, *, lr: float, beta1: float = 0.0,
                      beta2: float = 0.0, t: float = 0.0, eps: float = 0.0,
                      weight_decay: float = 0.0, static_table: bool = False) -> None:
    """One fused launch over caller-owned device buffers (device addresses as integers):
    the replacement of per-tensor ``gpu_optimizer_step`` calls (src/ops/gpu_ops.rs:495-508).

    ``static_table=True`` takes the entry point that allocates nothing
    (``vb_multi_tensor_step_static``): same results, but the chunk table sits in a fixed array
    inside the library, so the tensor list is limited to 8192 chunks and overlapping calls on
    one GPU must be serialised by the caller."""
    n = len(sizes)
    hp = _lib.StepParams(op, lr, beta1, beta2, float(t), eps, weight_decay, 0.0)
    arr_sizes = (C.c_int64 * max(n, 1))(*sizes)

    def ptrs(seq):
        if seq is None:
            return None
        return (C.c_void_p * max(n, 1))(*[(int(x) if x else None) for x in seq])

    call("vb_multi_tensor_step_static" if static_table else "vb_multi_tensor_step", engine._h, C.byref(hp), n,
         arr_sizes, ptrs(params), ptrs(grads), ptrs(state1), ptrs(state2))
