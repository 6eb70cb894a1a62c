"""GPU parity of the fused multi-tensor Adam / SGD path against the CPU oracle.

Tolerances: max relative error on params, m and v <= 1e-6 after one
step and <= 1e-5 after 100 steps.  The kernels are written to be bit-identical to the
reference's CPU arithmetic, so most cases assert exact equality, which implies both.
Everything goes through the C ABI (the ctypes mirror in volta_b200.optim).
"""
import json
import os

import numpy as np
import pytest

from helpers import bits_equal, max_rel_err

pytestmark = pytest.mark.gpu

TOL_ONE_STEP = 1e-6
TOL_MANY_STEPS = 1e-5

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "volta_optimizer_kats.json")
with open(GOLDEN) as fh:
    KATS = json.load(fh)


def _scalar(t):
    return float(t.data.reshape(-1)[0])


# ---- the reference's own optimizer tests, replayed through the drop-in API ----------------

@pytest.mark.parametrize("case", [c for c in KATS if c["kind"] in ("adam", "sgd")], ids=lambda c: c["name"])
def test_reference_known_answers(engine, case):
    """tests/test_optimizers.rs / tests/coverage_fill.rs / src/lib.rs:3102-3119."""
    from volta_b200 import SGD, Adam, Tensor
    t = Tensor([case["theta0"]], (1,), True)
    t.grad = [case["grad"]]
    if case["kind"] == "adam":
        opt = Adam([t], case["lr"], tuple(case["betas"]), case["eps"], case["weight_decay"], engine=engine)
    else:
        opt = SGD([t], case["lr"], case["momentum"], case["weight_decay"], engine=engine)
    for step in range(case["steps"]):
        opt.step()  # the gradient persists across steps, as in test_sgd_no_momentum_simple
        actual, expected = _scalar(t), case["expected"][step]
        if "tol_rel" in case:
            assert abs(actual - expected) <= case["tol_rel"] * abs(expected)
        else:
            assert abs(actual - expected) < case["tol_abs"], (actual, expected)
    opt.close()


def test_adam_convergence_convex(engine):
    """tests/test_optimizers.rs:142-162: minimise (x-3)^2, lr 0.05, 500 steps."""
    from volta_b200 import Adam, Tensor
    x = Tensor([0.0], (1,))
    opt = Adam([x], 0.05, (0.9, 0.999), 1e-8, 0.0, engine=engine)
    for _ in range(500):
        opt.zero_grad()
        x.grad = 2.0 * (x.data - 3.0)
        opt.step()
    assert abs(_scalar(x) - 3.0) < 0.05
    opt.close()


def test_sgd_convergence_convex(engine):
    """tests/test_optimizers.rs:225-245: momentum 0.9, lr 0.05, 500 steps."""
    from volta_b200 import SGD, Tensor
    x = Tensor([0.0], (1,))
    opt = SGD([x], 0.05, 0.9, 0.0, engine=engine)
    for _ in range(500):
        opt.zero_grad()
        x.grad = 2.0 * (x.data - 3.0)
        opt.step()
    assert abs(_scalar(x) - 3.0) < 0.05
    opt.close()


# ---- configuration-level parity ------------------------------------------------------------

def _run_both(oracle, engine, wl, steps, check_at=(1,), drop=None):
    """Runs `steps` steps of workload `wl` on the oracle and on the GPU with identical
    inputs; returns max relative errors of (params, state1, state2) at the checked steps."""
    from volta_b200 import SGD, Adam, Tensor
    params = wl.make_params()
    ref_params = [p.copy() for p in params]
    tensors = [Tensor(p, p.shape) for p in params]
    h = wl.hyper
    if wl.optimizer == "adam":
        ref = oracle.Adam(ref_params, h["lr"], h["betas"], h["eps"], h["weight_decay"])
        opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=engine)
    else:
        ref = oracle.SGD(ref_params, h["lr"], h["momentum"], h["weight_decay"])
        opt = SGD(tensors, h["lr"], h["momentum"], h["weight_decay"], engine=engine)
    out = {}
    for s in range(1, steps + 1):
        grads = wl.make_grads(s)
        if drop is not None:
            grads = [None if drop(i, s) else g for i, g in enumerate(grads)]
        opt.zero_grad()
        for t, g in zip(tensors, grads):
            if g is not None:
                t.grad = g
        opt.step()
        ref.step(grads)
        if s in check_at or s == steps:
            ep = max(max_rel_err(t.data, r) for t, r in zip(tensors, ref_params))
            exact = all(bits_equal(t.data, r) for t, r in zip(tensors, ref_params))
            es1 = es2 = 0.0
            if wl.optimizer == "adam":
                es1 = max(max_rel_err(opt.state(i, 0), ref.m[i]) for i in range(len(tensors)))
                es2 = max(max_rel_err(opt.state(i, 1), ref.v[i]) for i in range(len(tensors)))
                exact = exact and all(bits_equal(opt.state(i, 0), ref.m[i]) and
                                      bits_equal(opt.state(i, 1), ref.v[i]) for i in range(len(tensors)))
            elif ref.velocity:
                es1 = max(max_rel_err(opt.state(i, 0), ref.velocity[i]) for i in range(len(tensors)))
                exact = exact and all(bits_equal(opt.state(i, 0), ref.velocity[i]) for i in range(len(tensors)))
            out[s] = (ep, es1, es2, exact)
    if wl.optimizer == "adam":
        assert opt.t == ref.t == steps
    opt.close()
    return out


def test_c1_mlp_adam_100_steps(oracle, engine):
    import workloads
    wl = workloads.c1_mlp_adam()
    res = _run_both(oracle, engine, wl, 100, check_at=(1, 3, 10))
    assert max(res[1][:3]) <= TOL_ONE_STEP
    assert max(res[100][:3]) <= TOL_MANY_STEPS
    assert all(r[3] for r in res.values()), res  # in fact bit-identical at every checked step


def test_c2_cnn_sgd_200_steps(oracle, engine):
    import workloads
    wl = workloads.c2_cnn_sgd()
    res = _run_both(oracle, engine, wl, 200, check_at=(1, 100))
    assert max(res[1][:3]) <= TOL_ONE_STEP
    assert max(res[200][:3]) <= TOL_MANY_STEPS
    assert all(r[3] for r in res.values()), res


@pytest.mark.parametrize("kind,momentum,wd", [("adam", 0.0, 0.0), ("adam", 0.0, 0.1),
                                              ("sgd", 0.0, 0.0), ("sgd", 0.0, 0.05),
                                              ("sgd", 0.9, 0.0), ("sgd", 0.9, 5e-4)])
def test_ragged_sizes_every_length_1_to_70(oracle, engine, kind, momentum, wd):
    """Tiny tensors of every length (vector body + scalar tail), all in one launch."""
    import workloads
    shapes = [(n,) for n in range(1, 71)] + [(0,), (257,), (4099,), (3, 5, 7)]
    hyper = dict(lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=wd, momentum=momentum)
    wl = workloads.Workload("ragged_small", kind, shapes, [("normal", 1.0)] * len(shapes), 1e-1, hyper, 5)
    res = _run_both(oracle, engine, wl, 5)
    assert all(r[3] for r in res.values()), res


def test_missing_gradients_are_skipped_and_t_advances(oracle, engine):
    """adam.rs:71,81-84: a parameter without a gradient keeps theta, m and v; t still counts."""
    import workloads
    shapes = [(1000,), (33,), (5000,), (7,)]
    hyper = dict(lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    wl = workloads.Workload("skip", "adam", shapes, [("normal", 1.0)] * 4, 1e-1, hyper, 6)
    res = _run_both(oracle, engine, wl, 6, check_at=(1, 2, 3), drop=lambda i, s: (i + s) % 3 == 0)
    assert all(r[3] for r in res.values()), res


def test_c5_ragged_reduced(oracle, engine):
    """The ragged stress shape law (log-uniform sizes) at a size the oracle finishes quickly:
    512 tensors in [1, 2^18], lr 3e-4, wd 0.1, 10 steps."""
    import workloads
    wl = workloads.c5_ragged_adam(n_tensors=512, max_log2=18, seed=4096)
    res = _run_both(oracle, engine, wl, 10, check_at=(1,))
    assert max(res[1][:3]) <= TOL_ONE_STEP and max(res[10][:3]) <= TOL_MANY_STEPS
    assert all(r[3] for r in res.values()), res


def test_c3_full_size_two_steps(oracle, engine):
    """The 109 602 816-parameter Adam set at full size: two steps, whole-arena comparison."""
    import workloads
    from volta_b200 import Adam, Tensor
    wl = workloads.c3_transformer_adam()
    assert wl.total == 109_602_816 and len(wl.shapes) == 157
    params = wl.make_params()
    ref_params = [p.copy() for p in params]
    tensors = [Tensor(p, p.shape) for p in params]
    h = wl.hyper
    opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=engine)
    ref = oracle.Adam(ref_params, h["lr"], h["betas"], h["eps"], h["weight_decay"])
    _, _, arena, offsets = opt.arena_layout()
    host = np.zeros(arena, np.float32)
    for s in (1, 2):
        grads = wl.make_grads(s)
        for o, g in zip(offsets, grads):
            host[o:o + g.size] = g.reshape(-1)
        opt.upload_arena(1, host)
        opt.step()
        ref.step(grads)
    opt.download_arena(0, host)
    for o, r in zip(offsets, ref_params):
        assert bits_equal(host[o:o + r.size], r)
    for i in (0, 1, 5, 156):
        assert bits_equal(opt.state(i, 0), ref.m[i]) and bits_equal(opt.state(i, 1), ref.v[i])
    # linearity-free size-independent property: padding between tensors stays zero
    mask = np.ones(arena, bool)
    for o, r in zip(offsets, ref_params):
        mask[o:o + r.size] = False
    assert not host[mask].any()
    opt.close()


def test_state_import_export_and_t(engine, oracle):
    """Resume: exported m, v, t imported into a fresh optimizer continue bit-identically."""
    from volta_b200 import Adam, Tensor
    rng = np.random.default_rng(7)
    p0 = rng.standard_normal(5000).astype(np.float32)
    grads = [(rng.standard_normal(5000) * 0.01).astype(np.float32) for _ in range(4)]
    a = Tensor(p0.copy())
    opt_a = Adam([a], 1e-3, (0.9, 0.999), 1e-8, 0.01, engine=engine)
    for g in grads[:2]:
        a.grad = g
        opt_a.step()
    b = Tensor(a.data.copy())
    opt_b = Adam([b], 1e-3, (0.9, 0.999), 1e-8, 0.01, engine=engine)
    opt_b.load_state(0, 0, opt_a.state(0, 0))
    opt_b.load_state(0, 1, opt_a.state(0, 1))
    opt_b.t = opt_a.t
    for g in grads[2:]:
        a.grad = g
        b.grad = g
        opt_a.step()
        opt_b.step()
    assert bits_equal(a.data, b.data)
    opt_a.close()
    opt_b.close()


# ---- caller-owned buffers: the per-tensor gpu_optimizer_step seam, fused -------------------

@pytest.mark.parametrize("op", [0, 1, 2])
def test_multi_tensor_step_on_caller_buffers(oracle, engine, op):
    """vb_multi_tensor_step on torch-allocated device buffers, including tensors whose
    addresses are only 4-byte aligned (scalar path)."""
    import torch
    from volta_b200 import multi_tensor_step
    rng = np.random.default_rng(op)
    sizes = [1, 5, 1024, 4097, 70001, 333]
    dev = torch.device("cuda:0")
    pool = torch.zeros(4 * (sum(sizes) + 64 * len(sizes)), device=dev)  # carve misaligned views
    cursor = 0
    views = {k: [] for k in "pgab"}
    host = {k: [] for k in "pgab"}
    for i, n in enumerate(sizes):
        for k in "pgab":
            start = cursor + (i % 4 if k in "pg" else (i + 1) % 4)  # different misalignments
            v = pool[start:start + n]
            cursor = start + n + 16
            cursor += (-cursor) % 4
            if k == "p":
                x = rng.standard_normal(n).astype(np.float32)
            elif k == "g":
                x = (rng.standard_normal(n) * 0.1).astype(np.float32)
            else:
                x = (np.abs(rng.standard_normal(n)) * 0.01).astype(np.float32)
            v.copy_(torch.from_numpy(x))
            views[k].append(v)
            host[k].append(x)
    torch.cuda.synchronize()
    lr, b1, b2, eps, wd, t = 1e-2, 0.9, 0.999, 1e-8, 0.01, 7
    multi_tensor_step(engine, op, sizes, [v.data_ptr() for v in views["p"]],
                      [v.data_ptr() for v in views["g"]],
                      [v.data_ptr() for v in views["a"]] if op >= 1 else None,
                      [v.data_ptr() for v in views["b"]] if op == 2 else None,
                      lr=lr, beta1=b1, beta2=b2, t=t, eps=eps, weight_decay=wd)
    engine.synchronize()
    for i, n in enumerate(sizes):
        p, g, a, b = (host[k][i].copy() for k in "pgab")
        if op == 2:
            o = oracle.Adam([p], lr, (b1, b2), eps, wd)
            o.m[0][:], o.v[0][:], o.t = a, b, t - 1
            o.step([g])
            assert bits_equal(views["a"][i].cpu().numpy(), o.m[0])
            assert bits_equal(views["b"][i].cpu().numpy(), o.v[0])
        else:
            o = oracle.SGD([p], lr, b1 if op == 1 else 0.0, wd)
            if op == 1:
                o.velocity[0][:] = a
            o.step([g])
            if op == 1:
                assert bits_equal(views["a"][i].cpu().numpy(), o.velocity[0])
        assert bits_equal(views["p"][i].cpu().numpy(), p)
        assert bits_equal(views["g"][i].cpu().numpy(), host["g"][i])  # gradients are read-only


def test_errors_are_reported_not_fatal(engine):
    from volta_b200 import Adam, Tensor, VoltaB200Error, multi_tensor_step
    t = Tensor(np.zeros(8, np.float32))
    opt = Adam([t], 1e-3, engine=engine)
    with pytest.raises(ValueError):
        t.grad = np.zeros(9, np.float32)
    with pytest.raises(VoltaB200Error) as ei:
        opt.load_state(0, 5, np.zeros(8, np.float32))
    assert ei.value.status == 1
    with pytest.raises(VoltaB200Error):
        multi_tensor_step(engine, 2, [8], [0], [0], [0], [0], lr=1e-3, t=1)
    opt.close()


def test_c5_full_size_ragged_properties(oracle, engine):
    """The ragged stress configuration at full size (4096 tensors, sizes log-uniform in
    [1, 2^22], 1.13e9 parameters, lr 3e-4, wd 0.1), two steps.  The arenas are filled on the
    device; a sample of tensors (largest, smallest, random) is checked bit for bit against the
    oracle, and size-independent properties are checked on everything: padding between tensors
    stays zero, every parameter moves, m and v are finite and v >= 0."""
    import torch
    import workloads
    from volta_b200 import Adam, Tensor
    from volta_b200.interop import device_array
    wl = workloads.c5_ragged_adam()
    assert len(wl.sizes) == 4096 and wl.total == 1_129_164_500 and min(wl.sizes) >= 1 and max(wl.sizes) <= 2 ** 22
    h = wl.hyper
    tensors = [Tensor(np.zeros(n, np.float32)) for n in wl.sizes]
    opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=engine)
    p_ptr, g_ptr, arena, offsets = opt.arena_layout()
    theta = torch.as_tensor(device_array(p_ptr, arena, opt), device="cuda:0")
    grad = torch.as_tensor(device_array(g_ptr, arena, opt), device="cuda:0")
    gen = torch.Generator(device="cuda:0")
    gen.manual_seed(1234)
    mask = torch.zeros(arena, dtype=torch.bool, device="cuda:0")
    for o, n in zip(offsets, wl.sizes):
        mask[o:o + n] = True
    theta.normal_(0.0, 1.0, generator=gen)
    theta.mul_(mask)  # padding must start (and stay) zero
    order = np.argsort(wl.sizes)
    rng = np.random.default_rng(0)
    sample = sorted(set(order[:8].tolist() + order[-4:].tolist() + rng.choice(4096, 24, replace=False).tolist()))
    ref_p = {i: theta[offsets[i]:offsets[i] + wl.sizes[i]].cpu().numpy().copy() for i in sample}
    ref = oracle.Adam([ref_p[i] for i in sample], h["lr"], h["betas"], h["eps"], h["weight_decay"])
    before = theta.clone()
    opt.mark_all_grads_present()
    for s in (1, 2):
        grad.normal_(0.0, 1e-3, generator=gen)
        grad.mul_(mask)
        torch.cuda.synchronize()
        gs = [grad[offsets[i]:offsets[i] + wl.sizes[i]].cpu().numpy().copy() for i in sample]
        opt.step()
        engine.synchronize()
        ref.step(gs)
    for k, i in enumerate(sample):
        got = theta[offsets[i]:offsets[i] + wl.sizes[i]].cpu().numpy()
        assert bits_equal(got, ref_p[i]), i
        assert bits_equal(opt.state(i, 0), ref.m[k]) and bits_equal(opt.state(i, 1), ref.v[k])
    assert not bool(theta[~mask].any())                      # padding untouched
    assert bool(((theta != before) | ~mask).all())           # every parameter moved (wd 0.1, N(0,1) data)
    assert bool(torch.isfinite(theta).all())
    del theta, grad, before, mask
    opt.close()


def test_gradient_accumulation_on_device(oracle, engine):
    """RawTensor::accumulate_grad (src/autograd.rs:158-184): contributions are summed in arrival
    order with one rounded add each; after zero_grad the next contribution replaces."""
    import torch
    from volta_b200 import Adam, Tensor, _lib
    from volta_b200.optim import accumulate_grad
    rng = np.random.default_rng(9)
    n = 10007
    p = Tensor(rng.standard_normal(n).astype(np.float32))
    opt = Adam([p], 1e-3, (0.9, 0.999), 1e-8, 0.0, engine=engine)
    parts = [(rng.standard_normal(n) * 0.01).astype(np.float32) for _ in range(3)]
    accumulate_grad(p, parts[0])
    accumulate_grad(p, parts[1])
    dev = torch.from_numpy(parts[2]).to("cuda:0")
    torch.cuda.synchronize()
    _lib.call("vb_optimizer_accumulate_grad_device", opt._h, 0, dev.data_ptr(), n)
    opt._present[0] = True
    expect = ((parts[0] + parts[1]).astype(np.float32) + parts[2]).astype(np.float32)
    assert bits_equal(p.grad, expect)
    ref_p = p.data.copy()
    ref = oracle.Adam([ref_p], 1e-3, (0.9, 0.999), 1e-8, 0.0)
    opt.step()
    ref.step([expect])
    assert bits_equal(p.data, ref_p)
    opt.zero_grad()
    accumulate_grad(p, parts[1])          # first contribution after zero_grad replaces the old gradient
    assert bits_equal(p.grad, parts[1])
    opt.close()


@pytest.mark.parametrize("pieces", [1, 3, 8])
def test_pipelined_host_step_matches_oracle(oracle, engine, pieces):
    """vb_optimizer_step_host: upload / update / download overlapped piece by piece must give the
    same bits as the plain step (and as the oracle), whatever the number of pieces."""
    import workloads
    from volta_b200 import Adam, PinnedBuffer, Tensor
    wl = workloads.c5_ragged_adam(n_tensors=200, max_log2=16, seed=21)
    h = wl.hyper
    params = wl.make_params()
    ref_params = [p.copy() for p in params]
    tensors = [Tensor(p, p.shape) for p in params]
    opt = Adam(tensors, h["lr"], h["betas"], h["eps"], h["weight_decay"], engine=engine)
    ref = oracle.Adam(ref_params, h["lr"], h["betas"], h["eps"], h["weight_decay"])
    _, _, arena, offsets = opt.arena_layout()
    gbuf, pbuf = PinnedBuffer(arena), PinnedBuffer(arena)
    gbuf.array[:] = 0
    for s in (1, 2, 3):
        grads = wl.make_grads(s)
        for o, g in zip(offsets, grads):
            gbuf.array[o:o + g.size] = g.reshape(-1)
        opt.step_host(gbuf.array, pbuf.array, pieces=pieces)
        ref.step(grads)
        for o, r in zip(offsets, ref_params):
            assert bits_equal(pbuf.array[o:o + r.size], r)
    assert opt.t == 3
    for t, r in zip(tensors, ref_params):
        assert bits_equal(t.data, r)
    opt.close()
    gbuf.free()
    pbuf.free()


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["adam", "sgd_momentum"])
def test_special_values_follow_ieee_like_the_cpu(oracle, engine, kind):
    """Zeros of both signs, subnormals, the largest finite numbers, infinities and NaN in parameters
    and gradients: the kernels use IEEE division / square root / fused multiply-add without flushing
    subnormals, so every finite or infinite result has the CPU's bits and NaN appears exactly where
    the CPU produces one (NaN payloads are not compared)."""
    from volta_b200 import SGD, Adam, Tensor
    specials = np.array([0.0, -0.0, 1e-45, -1e-45, 1e-39, 1.1754944e-38, 3.4028235e38, -3.4028235e38,
                         np.inf, -np.inf, np.nan, 1.0, -1.0, 1e-20, 1e20, 65504.0], np.float32)
    p0 = np.repeat(specials, specials.size)           # every parameter value ...
    g0 = np.tile(specials, specials.size)             # ... against every gradient value
    t = Tensor(p0.copy())
    ref = [p0.copy()]
    if kind == "adam":
        opt, o = Adam([t], 1e-3, (0.9, 0.999), 1e-8, 0.01, engine=engine), oracle.Adam(ref, 1e-3, (0.9, 0.999), 1e-8, 0.01)
    else:
        opt, o = SGD([t], 0.01, 0.9, 5e-4, engine=engine), oracle.SGD(ref, 0.01, 0.9, 5e-4)
    with np.errstate(all="ignore"):
        for step in range(3):
            t.grad = g0
            opt.step()
            o.step([g0])
            got, want = t.data.reshape(-1), ref[0].reshape(-1)
            nan_g, nan_w = np.isnan(got), np.isnan(want)
            assert np.array_equal(nan_g, nan_w), step
            assert np.array_equal(got[~nan_g].view(np.uint32), want[~nan_w].view(np.uint32)), step
            for which in range(2 if kind == "adam" else 1):
                cpu_state = ([o.m, o.v] if kind == "adam" else [o.velocity])[which][0]
                sg, sw = opt.state(0, which).reshape(-1), cpu_state.reshape(-1)
                assert np.array_equal(np.isnan(sg), np.isnan(sw))
                m = ~np.isnan(sg)
                assert np.array_equal(sg[m].view(np.uint32), sw[m].view(np.uint32)), (step, which)
    opt.close()


@pytest.mark.gpu
@pytest.mark.parametrize("lr,eps,wd", [(1e-3, 1e-8, 0.01), (1e-3, 0.0, 0.0), (1e-20, 1e-30, 0.1), (1.0, 1e-8, 0.0)])
def test_adam_across_the_whole_exponent_range(oracle, engine, lr, eps, wd):
    """Parameters and gradients with magnitudes from the smallest subnormal to 1e3 in every
    combination: subnormal moments, subnormal numerators over ordinary denominators, tiny
    denominators, subnormal quotients.  Every result must carry the CPU's bits
    (src/nn/optim/adam.rs:172-204): nothing is flushed to zero, division and square root are the
    IEEE-rounded forms also where the hardware has to take its long fallback."""
    from volta_b200 import Adam, Tensor
    rng = np.random.default_rng(99)
    n = 1 << 16
    mag = np.exp2(rng.uniform(-149.0, 10.0, n)).astype(np.float32)
    p0 = (mag * rng.choice([-1.0, 1.0], n)).astype(np.float32)
    gmag = np.exp2(rng.uniform(-149.0, 10.0, n)).astype(np.float32)
    g0 = (gmag * rng.choice([-1.0, 1.0], n)).astype(np.float32)
    g0[::17] = 0.0   # gradient-free elements: only weight decay acts
    t = Tensor(p0.copy())
    ref = [p0.copy()]
    opt, o = Adam([t], lr, (0.9, 0.999), eps, wd, engine=engine), oracle.Adam(ref, lr, (0.9, 0.999), eps, wd)
    with np.errstate(all="ignore"):
        for step in range(4):
            t.grad = g0
            opt.step()
            o.step([g0])
            got, want = t.data.reshape(-1), ref[0].reshape(-1)
            nan_g, nan_w = np.isnan(got), np.isnan(want)
            assert np.array_equal(nan_g, nan_w), step
            assert np.array_equal(got[~nan_g].view(np.uint32), want[~nan_w].view(np.uint32)), step
            for which, cpu in enumerate((o.m[0], o.v[0])):
                sg = opt.state(0, which).reshape(-1)
                keep = ~np.isnan(sg)
                assert np.array_equal(sg[keep].view(np.uint32), cpu[keep].view(np.uint32)), (step, which)
    opt.close()
