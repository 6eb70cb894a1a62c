"""The allocation-free entry point, checked against the allocating one.

Some hosts cannot let the optimizer allocate: all device memory already belongs to their own
pool, or allocation is forbidden once their loop has started.  ``vb_multi_tensor_step_static``
keeps its chunk table in a fixed array inside the library instead of allocating one.  This
test drives both entry points through the C ABI on identical device buffers, twice in a row
(the second call reuses the array that still holds the first call's table, with a different
tensor list), and requires bit-identical parameters and state: the same bar the other
Adam/SGD tests use.  It lives in a file of its own that pytest collects last, so a run that
stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _buffers(torch, rng, sizes, dev):
    host = {k: [] for k in "pgab"}
    for n in sizes:
        host["p"].append(rng.standard_normal(n).astype(np.float32))
        host["g"].append((rng.standard_normal(n) * 0.1).astype(np.float32))
        host["a"].append((rng.standard_normal(n) * 0.01).astype(np.float32))
        host["b"].append((np.abs(rng.standard_normal(n)) * 1e-3).astype(np.float32))
    make = lambda: {k: [torch.from_numpy(x).to(dev) for x in v] for k, v in host.items()}  # noqa: E731
    return make(), make()


def _call(name, engine, op, sizes, bufs, t):
    from volta_b200 import _lib
    n = len(sizes)
    hp = _lib.StepParams(op, 1e-2, 0.9, 0.999, float(t), 1e-8, 0.01, 0.0)
    arr = (C.c_int64 * n)(*sizes)
    ptrs = lambda k: (C.c_void_p * n)(*[x.data_ptr() if x.numel() else None for x in bufs[k]])  # noqa: E731
    _lib.call(name, engine._h, C.byref(hp), n, arr, ptrs("p"), ptrs("g"),
              ptrs("a") if op >= 1 else None, ptrs("b") if op == 2 else None)


@pytest.mark.parametrize("op", [2, 1, 0])
def test_static_entry_point_matches_allocating_one_twice(engine, op):
    import torch
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(100 + op)
    for call_no, sizes in enumerate(([1, 7, 2048, 70001, 0, 333, 1 << 20], [5000, 3, 129, 1 << 18])):
        ref, got = _buffers(torch, rng, sizes, dev)
        torch.cuda.synchronize()
        _call("vb_multi_tensor_step", engine, op, sizes, ref, t=3 + call_no)
        _call("vb_multi_tensor_step_static", engine, op, sizes, got, t=3 + call_no)
        engine.synchronize()
        for k in "pgab":
            for r, g in zip(ref[k], got[k]):
                assert torch.equal(r.view(torch.int32), g.view(torch.int32)), (call_no, k)


def test_static_entry_point_rejects_lists_beyond_its_table(engine):
    from volta_b200 import VoltaB200Error, _lib
    n = 8193
    hp = _lib.StepParams(0, 1e-2, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0)
    sizes = (C.c_int64 * n)(*([4] * n))
    fake = (C.c_void_p * n)(*([0x1000] * n))  # never dereferenced: the size check comes first
    with pytest.raises(VoltaB200Error) as ei:
        _lib.call("vb_multi_tensor_step_static", engine._h, C.byref(hp), n, sizes, fake, fake, None, None)
    assert ei.value.status == 6 and "static table" in ei.value.message
