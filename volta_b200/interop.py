"""Views of the engine's device memory for array libraries (no copies).

``device_array(ptr, n)`` wraps ``n`` float32 values at device address ``ptr`` in an object
that exposes ``__cuda_array_interface__`` (version 3), which torch, cupy and numba accept:

    theta = torch.as_tensor(device_array(param_ptr, arena_elements), device="cuda:0")

This is plumbing for producers of gradients that already live on the GPU (and for the
benchmark, which fills arenas on the device); the optimizer arithmetic never goes through it.
"""
from __future__ import annotations


class device_array:
    def __init__(self, ptr: int, n: int, owner=None):
        self._owner = owner  # keeps the optimizer alive while the view exists
        self.__cuda_array_interface__ = {
            "shape": (int(n),), "typestr": "<f4", "data": (int(ptr), False), "version": 3, "strides": None,
        }
