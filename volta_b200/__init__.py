"""volta_b200: a B200 (sm_100a) optimizer-step engine behind Volta's optimizer API.

``Adam``, ``SGD`` and ``Muon`` mirror ``volta::nn::{Adam, SGD, Muon}``; everything runs in
``libvolta_b200.so`` (hand-written CUDA behind the C ABI of ``include/volta_b200.h``).
Importing this package needs the built library; there is no CPU or PyTorch fallback.
"""
from . import _lib
from .optim import (VB_NS_BF16, VB_NS_F32, VB_NS_F32_TC, VB_STEP_EXCHANGE_BF16, VB_STEP_MEAN_GRADS, VB_STEP_NO_EXCHANGE,
                    VB_STEP_REDUCE_GRADS, Adam, Engine, Muon, PinnedBuffer,
                    SGD, Tensor, VoltaB200Error, accumulate_grad, default_engine, multi_tensor_step, plan_fingerprint,
                    plan_replicated_fraction, verify_plan)

_lib.load()  # fail loudly at import time if the CUDA library has not been built

__all__ = ["Adam", "SGD", "Muon", "Tensor", "Engine", "PinnedBuffer", "default_engine",
           "multi_tensor_step", "accumulate_grad", "plan_fingerprint", "plan_replicated_fraction", "verify_plan", "VoltaB200Error", "VB_NS_F32", "VB_NS_BF16", "VB_NS_F32_TC", "VB_STEP_NO_EXCHANGE", "VB_STEP_EXCHANGE_BF16", "VB_STEP_REDUCE_GRADS", "VB_STEP_MEAN_GRADS"]
