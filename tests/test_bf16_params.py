"""bf16 copies of the parameters kept by the update kernels next to the f32 master (one GPU):
after every step and every upload bf16[i] == round-to-nearest-even(param[i]), bit for bit, on
all three code paths of the kernel (256-bit, 128-bit, scalar) and for every optimizer."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def bf16_rne(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def _check(opt, tensors):
    for i, t in enumerate(tensors):
        assert np.array_equal(opt.bf16_params(i), bf16_rne(t.data).reshape(t.shape)), i


@pytest.mark.parametrize("kind", ["adam", "sgd_momentum", "sgd"])
def test_copies_follow_every_step_and_upload(engine, oracle, kind):
    from volta_b200 import SGD, Adam, Tensor
    rng = np.random.default_rng(5)
    sizes = list(range(1, 71)) + [4096, 8191, 20000, 0]
    params = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    tensors = [Tensor(p.copy()) for p in params]
    ref = [p.copy() for p in params]
    if kind == "adam":
        opt, o = Adam(tensors, 1e-2, (0.9, 0.999), 1e-8, 0.01, engine=engine), oracle.Adam(ref, 1e-2, (0.9, 0.999), 1e-8, 0.01)
    else:
        mom = 0.9 if kind == "sgd_momentum" else 0.0
        opt, o = SGD(tensors, 0.05, mom, 5e-4, engine=engine), oracle.SGD(ref, 0.05, mom, 5e-4)
    opt.enable_bf16_params()
    _check(opt, tensors)                       # filled from the current parameters
    for step in range(3):
        grads = [(rng.standard_normal(n) * 0.1).astype(np.float32) for n in sizes]
        if step == 1:
            grads[7] = None                    # a parameter without gradient keeps value and copy
            grads[71] = None
        for t, g in zip(tensors, grads):
            t.grad = g
        opt.step()
        o.step(grads)
        for t, r in zip(tensors, ref):
            assert np.array_equal(t.data.view(np.uint32), r.view(np.uint32))
        _check(opt, tensors)
    tensors[3].data = np.array([1.00390625, -3.0e-39, 65504.0, 1.01171875], np.float32)   # ties, subnormal, large
    _check(opt, tensors)
    opt.close()


def test_muon_copies(engine, oracle):
    from volta_b200 import VB_NS_F32, Muon, Tensor
    rng = np.random.default_rng(6)
    shapes = [(64, 48), (33, 7), (5,), (128, 128), (1, 9)]
    params = [(rng.standard_normal(s) * 0.02).astype(np.float32) for s in shapes]
    tensors = [Tensor(p.copy()) for p in params]
    opt = Muon(tensors, 0.1, 0.9, True, 5, ns_mode=VB_NS_F32, engine=engine)
    opt.enable_bf16_params()
    for _ in range(2):
        for t in tensors:
            t.grad = (rng.standard_normal(t.shape) * 1e-3).astype(np.float32)
        opt.step()
        _check(opt, tensors)
    opt.close()


def test_bf16_only_exchange_needs_the_copies(engine):
    from volta_b200 import VB_STEP_EXCHANGE_BF16, Adam, Tensor, VoltaB200Error
    t = Tensor(np.ones(8, np.float32))
    opt = Adam([t], 1e-3, (0.9, 0.999), 1e-8, 0.0, engine=engine)
    t.grad = np.ones(8, np.float32)
    with pytest.raises(VoltaB200Error):
        opt.step(VB_STEP_EXCHANGE_BF16)
    with pytest.raises(VoltaB200Error):
        opt.bf16_params(0)
    opt.close()


def test_copies_follow_the_pipelined_host_step(engine):
    """vb_optimizer_step_host with the copies enabled: every piece's update kernel writes them too."""
    import workloads
    from volta_b200 import Adam, PinnedBuffer, Tensor
    wl = workloads.c5_ragged_adam(n_tensors=120, max_log2=15, seed=31)
    h = wl.hyper
    tensors = [Tensor(p, p.shape) for p in wl.make_params()]
    opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=engine)
    opt.enable_bf16_params()
    _, _, arena, offsets = opt.arena_layout()
    gbuf, pbuf = PinnedBuffer(arena), PinnedBuffer(arena)
    gbuf.array[:] = 0
    for s in (1, 2):
        for o, g in zip(offsets, wl.make_grads(s)):
            gbuf.array[o:o + g.size] = g.reshape(-1)
        opt.step_host(gbuf.array, pbuf.array, pieces=5)
        for i, (o, t) in enumerate(zip(offsets, tensors)):
            assert np.array_equal(opt.bf16_params(i).reshape(-1), bf16_rne(pbuf.array[o:o + t.size]))
    opt.close()
    gbuf.free()
    pbuf.free()
