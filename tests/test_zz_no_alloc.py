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


def test_static_entry_point_matches_the_cpu_oracle_and_allocates_nothing(oracle, engine):
    """Directly against the reference arithmetic (not only against the allocating entry point),
    with the free device memory read before and after the calls: it must not move."""
    import torch
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(77)
    sizes = [4097, 1, 250000, 33]
    host_p = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    host_g = [[(rng.standard_normal(n) * 0.1).astype(np.float32) for n in sizes] for _ in range(2)]
    bufs = {"p": [torch.from_numpy(x).to(dev) for x in host_p],
            "g": [torch.empty(n, dtype=torch.float32, device=dev) for n in sizes],
            "a": [torch.zeros(n, dtype=torch.float32, device=dev) for n in sizes],
            "b": [torch.zeros(n, dtype=torch.float32, device=dev) for n in sizes]}
    ref_p = [x.copy() for x in host_p]
    ref = oracle.Adam(ref_p, 1e-2, (0.9, 0.999), 1e-8, 0.01)
    _call("vb_multi_tensor_step_static", engine, 2, sizes, bufs, t=1)  # warm: first call resolves the address
    for x, h in zip(bufs["p"], host_p):
        x.copy_(torch.from_numpy(h))
    for k in "ab":
        for x in bufs[k]:
            x.zero_()
    staged = [[torch.from_numpy(g).to(dev) for g in gs] for gs in host_g]
    torch.cuda.synchronize()
    engine.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for step in (1, 2):
        for dst, src in zip(bufs["g"], staged[step - 1]):
            dst.copy_(src)
        torch.cuda.synchronize()
        _call("vb_multi_tensor_step_static", engine, 2, sizes, bufs, t=step)
        engine.synchronize()
        ref.step(host_g[step - 1])
    assert torch.cuda.mem_get_info()[0] == free_before
    for got, want in zip(bufs["p"], ref_p):
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    for got, want in zip(bufs["a"], ref.m):
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    for got, want in zip(bufs["b"], ref.v):
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_static_entry_point_grows_its_chunks_for_lists_beyond_8192_pieces(engine):
    """40 M elements would need 9766 pieces of the usual 4096 elements: the fixed table holds 8192,
    so the entry point doubles the piece length instead.  Same result as the allocating one."""
    import torch
    dev = torch.device("cuda:0")
    sizes = [40_000_003, 11]
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    ref = {"p": [torch.randn(n, device=dev, generator=gen) for n in sizes],
           "g": [torch.randn(n, device=dev, generator=gen) * 0.1 for n in sizes],
           "a": [torch.randn(n, device=dev, generator=gen) * 0.01 for n in sizes], "b": []}
    got = {k: [x.clone() for x in v] for k, v in ref.items()}
    torch.cuda.synchronize()
    _call("vb_multi_tensor_step", engine, 1, sizes, ref, t=1)
    _call("vb_multi_tensor_step_static", engine, 1, sizes, got, t=1)
    engine.synchronize()
    for k in "pga":
        for r, g in zip(ref[k], got[k]):
            assert torch.equal(r.view(torch.int32), g.view(torch.int32)), k


def test_static_entry_point_rejects_lists_beyond_its_table(engine):
    from volta_b200 import VoltaB200Error, _lib
    n = 8193
    hp = _lib.StepParams(0, 1e-2, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0)
    sizes = (C.c_int64 * n)(*([4] * n))
    fake = (C.c_void_p * n)(*([0x1000] * n))  # never dereferenced: the size check comes first
    with pytest.raises(VoltaB200Error) as ei:
        _lib.call("vb_multi_tensor_step_static", engine._h, C.byref(hp), n, sizes, fake, fake, None, None)
    assert ei.value.status == 6 and "static table" in ei.value.message
    # one tensor beyond 8192 pieces of the largest piece length (131072 elements)
    sizes = (C.c_int64 * 1)(8192 * 131072 + 1)
    fake = (C.c_void_p * 1)(0x1000)
    with pytest.raises(VoltaB200Error) as ei:
        _lib.call("vb_multi_tensor_step_static", engine._h, C.byref(hp), 1, sizes, fake, fake, None, None)
    assert ei.value.status == 6 and "static table" in ei.value.message


@pytest.mark.parametrize("entry", ["vb_multi_tensor_step", "vb_multi_tensor_step_static"])
def test_caller_buffers_must_be_device_memory_of_the_engine(engine, entry):
    """A host pointer handed in by mistake would fault the kernel; it is refused on the host."""
    import torch
    from volta_b200 import VoltaB200Error, _lib
    n = 1000
    good = torch.zeros(n, dtype=torch.float32, device="cuda:0")
    host = np.zeros(n, np.float32)
    hp = _lib.StepParams(0, 1e-2, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0)
    sizes = (C.c_int64 * 1)(n)
    with pytest.raises(VoltaB200Error) as ei:
        _lib.call(entry, engine._h, C.byref(hp), 1, sizes, (C.c_void_p * 1)(good.data_ptr()),
                  (C.c_void_p * 1)(host.ctypes.data), None, None)
    assert ei.value.status == 1 and "grads[0]" in ei.value.message
    engine.synchronize()
