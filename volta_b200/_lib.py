"""ctypes binding of ``libvolta_b200.so`` (the C ABI of ``include/volta_b200.h``).

There is no fallback of any kind: if the shared library is missing or a call fails,
an exception is raised.  Nothing here computes optimizer arithmetic on the host.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libvolta_b200.so")

STATUS_NAMES = {
    0: "VB_OK", 1: "VB_ERR_INVALID_ARG", 2: "VB_ERR_CUDA", 3: "VB_ERR_NCCL",
    4: "VB_ERR_TIMEOUT", 5: "VB_ERR_STATE", 6: "VB_ERR_UNSUPPORTED",
}

VB_NS_F32 = 0
VB_NS_BF16 = 1
VB_NS_F32_TC = 2
VB_STEP_DEFAULT = 0
VB_STEP_NO_EXCHANGE = 1
VB_STEP_EXCHANGE_BF16 = 2
VB_STEP_REDUCE_GRADS = 4
VB_STEP_MEAN_GRADS = 8


class VoltaB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.message = message


class StepParams(C.Structure):
    """Mirror of ``vb_optimizer_step_params`` (Volta's ``OptimizerStepParams``)."""

    _fields_ = [("op", C.c_uint32), ("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float),
                ("t", C.c_float), ("eps", C.c_float), ("weight_decay", C.c_float),
                ("padding", C.c_float)]


_vp = C.c_void_p
_i64 = C.c_int64
_i64p = C.POINTER(C.c_int64)
_f32p = C.POINTER(C.c_float)
_vpp = C.POINTER(C.c_void_p)

# name -> argtypes; every function returns int (vb_status) except where noted below.
SIGNATURES = {
    "vb_device_count": [C.POINTER(C.c_int)],
    "vb_plan_layout": [_i64, _i64p, C.c_int, C.c_int, C.c_int, _i64p, _i64p, _i64p, _i64p, _i64p, _i64,
                       _i64p, _i64p, _i64p],
    "vb_plan_layout_replicated": [_i64, _i64p, C.c_int, C.c_int, C.c_int, C.c_double, _i64p, _i64p, _i64p, _i64p, _i64p,
                                  _i64p, _i64, _i64p, _i64p, _i64p, C.POINTER(C.c_int32)],
    "vb_plan_replicated_fraction": [C.c_double, C.c_int, C.c_double, C.c_double, C.POINTER(C.c_double)],
    "vb_plan_muon_owners": [_i64, _i64p, _i64p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int32),
                            C.POINTER(C.c_double)],
    "vb_plan_fingerprint": [C.c_int, _i64, _i64p, _i64p, _f32p, C.c_int, C.POINTER(C.c_int32), C.c_int, C.c_int,
                            C.POINTER(C.c_uint64)],
    "vb_plan_fingerprints_agree": [C.POINTER(C.c_uint64), C.c_int, C.POINTER(C.c_int)],
    "vb_optimizer_plan_fingerprint": [_vp, C.POINTER(C.c_uint64)],
    "vb_engine_synchronize_deadline": [_vp, C.c_double],
    "vb_engine_set_wait_limit_ms": [_vp, C.c_uint32],
    "vb_engine_set_replicated_fraction": [_vp, C.c_double],
    "vb_debug_muon_withhold_loads": [_vp, C.c_uint32],
    "vb_debug_fence_wait_expiry": [_vp, C.c_uint32, C.c_int, C.POINTER(C.c_int)],
    "vb_engine_create": [C.c_int, _vpp],
    "vb_engine_destroy": [_vp],
    "vb_engine_synchronize": [_vp],
    "vb_engine_stream": [_vp, _vpp],
    "vb_engine_launch_count": [_vp, C.POINTER(C.c_uint64)],
    "vb_engine_set_profiling": [_vp, C.c_int],
    "vb_engine_profile": [_vp, C.c_int, C.POINTER(C.c_double), _i64p],
    "vb_debug_gemm_wait_expiry": [_vp, C.c_uint32, C.POINTER(C.c_int)],
    "vb_host_alloc_pinned": [_vpp, C.c_size_t],
    "vb_host_free_pinned": [_vp],
    "vb_comm_unique_id": [_vp],
    "vb_engine_comm_init": [_vp, _vp, C.c_int, C.c_int],
    "vb_engine_rank": [_vp, C.POINTER(C.c_int), C.POINTER(C.c_int)],
    "vb_adam_create": [_vp, _i64, _i64p, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, _vpp],
    "vb_sgd_create": [_vp, _i64, _i64p, C.c_float, C.c_float, C.c_float, _vpp],
    "vb_muon_create": [_vp, _i64, _i64p, _i64p, C.c_float, C.c_float, C.c_int, C.c_int, C.c_int, _vpp],
    "vb_optimizer_destroy": [_vp],
    "vb_optimizer_num_tensors": [_vp, _i64p],
    "vb_optimizer_tensor_size": [_vp, _i64, _i64p],
    "vb_optimizer_total_size": [_vp, _i64p],
    "vb_optimizer_upload_params": [_vp, _i64, _vp, _i64],
    "vb_optimizer_download_params": [_vp, _i64, _vp, _i64],
    "vb_optimizer_upload_grad": [_vp, _i64, _vp, _i64],
    "vb_optimizer_download_grad": [_vp, _i64, _vp, _i64],
    "vb_optimizer_accumulate_grad": [_vp, _i64, _vp, _i64],
    "vb_optimizer_accumulate_grad_device": [_vp, _i64, _vp, _i64],
    "vb_optimizer_param_ptr": [_vp, _i64, _vpp],
    "vb_optimizer_grad_ptr": [_vp, _i64, _vpp],
    "vb_optimizer_arena": [_vp, _vpp, _vpp, _i64p, _i64p],
    "vb_optimizer_upload_arena": [_vp, C.c_int, _vp, _i64],
    "vb_optimizer_download_arena": [_vp, C.c_int, _vp, _i64],
    "vb_optimizer_upload_arena_range": [_vp, C.c_int, _vp, _i64, _i64],
    "vb_optimizer_download_arena_range": [_vp, C.c_int, _vp, _i64, _i64],
    "vb_optimizer_owned_range": [_vp, _i64p, _i64p],
    "vb_optimizer_replicated_range": [_vp, _i64p, _i64p],
    "vb_optimizer_set_grad_present": [_vp, _i64, C.c_int],
    "vb_optimizer_step": [_vp],
    "vb_optimizer_step_ex": [_vp, C.c_uint32],
    "vb_optimizer_step_host": [_vp, _vp, _vp, C.c_int],
    "vb_optimizer_zero_grad": [_vp],
    "vb_optimizer_set_lr": [_vp, C.c_float],
    "vb_optimizer_export_state": [_vp, _i64, C.c_int, _vp, _i64, _i64p, _i64p],
    "vb_optimizer_import_state": [_vp, _i64, C.c_int, _vp, _i64],
    "vb_optimizer_ipc_handle": [_vp, _vp],
    "vb_optimizer_open_peers": [_vp, _vp, C.c_int],
    "vb_optimizer_peer_copy_probe": [_vp, C.c_int, C.POINTER(C.c_double)],
    "vb_optimizer_ipc_handle_grads": [_vp, _vp],
    "vb_optimizer_open_peers_grads": [_vp, _vp, C.c_int],
    "vb_optimizer_enable_bf16_params": [_vp],
    "vb_optimizer_refresh_bf16_params": [_vp],
    "vb_optimizer_param_bf16_ptr": [_vp, C.c_int64, C.POINTER(C.c_void_p)],
    "vb_optimizer_download_params_bf16": [_vp, C.c_int64, _vp, C.c_int64],
    "vb_optimizer_ipc_handle_bf16": [_vp, _vp],
    "vb_optimizer_open_peers_bf16": [_vp, _vp, C.c_int],
    "vb_optimizer_reset_state": [_vp],
    "vb_optimizer_get_t": [_vp, _i64p],
    "vb_optimizer_set_t": [_vp, _i64],
    "vb_muon_set_keep_update": [_vp, C.c_int],
    "vb_muon_download_update": [_vp, _i64, _vp, _i64],
    "vb_muon_last_ns_flops": [_vp, C.POINTER(C.c_double)],
    "vb_multi_tensor_step": [_vp, C.POINTER(StepParams), _i64, _i64p, _vpp, _vpp, _vpp, _vpp],
    "vb_multi_tensor_step_static": [_vp, C.POINTER(StepParams), _i64, _i64p, _vpp, _vpp, _vpp, _vpp],
}
OTHER_SYMBOLS = ["vb_abi_version", "vb_last_error"]

_lib = None


def load() -> C.CDLL:
    """Loads the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python volta_b200/build.py` "
            "(nvcc, sm_100a).  volta_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = C.c_int
    lib.vb_abi_version.restype = C.c_int
    lib.vb_abi_version.argtypes = []
    lib.vb_last_error.restype = C.c_char_p
    lib.vb_last_error.argtypes = []
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != 0:
        raise VoltaB200Error(status, load().vb_last_error().decode("utf-8", "replace"))


def call(name: str, *args) -> None:
    check(getattr(load(), name)(*args))
