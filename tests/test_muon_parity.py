"""GPU parity of Muon (momentum, normalisation, Newton-Schulz, apply) against the oracle.

Tolerances, per matrix, on the Newton-Schulz output ("update"):
relative Frobenius error <= 1e-5 on the f32 path and <= 2e-2 on the bf16 tensor-core path.
The oracle's contraction restates matrixmultiply's blocking; the reference itself holds no
numeric test for Muon, so these compare against the restatement (and, for context, against
the f64-accumulating variant of the oracle).
"""
import numpy as np
import pytest

from helpers import bits_equal, max_rel_err, rel_frobenius

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_BF16 = 2e-2


def _run(oracle, engine, shapes, steps, ns_mode, lr=0.1, momentum=0.9, nesterov=True, ns_steps=5,
         grad_std=1e-3, param_std=0.02, seed=0, drop=None, gemm_mode=0):
    from volta_b200 import Muon, Tensor
    rng = np.random.default_rng(seed)
    params = [(rng.standard_normal(s) * param_std).astype(np.float32) for s in shapes]
    ref_params = [p.copy() for p in params]
    tensors = [Tensor(p, p.shape) for p in params]
    opt = Muon(tensors, lr, momentum, nesterov, ns_steps, ns_mode=ns_mode, engine=engine, keep_update=True)
    ref = oracle.Muon(ref_params, lr, momentum, nesterov, ns_steps, gemm_mode=gemm_mode)
    out = []
    for s in range(1, steps + 1):
        grads = [(rng.standard_normal(sh) * grad_std).astype(np.float32) for sh in shapes]
        if drop is not None:
            grads = [None if drop(i, s) else g for i, g in enumerate(grads)]
        opt.zero_grad()
        for t, g in zip(tensors, grads):
            if g is not None:
                t.grad = g
        opt.step()
        ref.step(grads)
        errs = []
        for i, g in enumerate(grads):
            if g is None:
                continue
            errs.append(rel_frobenius(opt.last_update(i), ref.last_update[i]))
        out.append(dict(update=max(errs) if errs else 0.0,
                        weights=max(max_rel_err(t.data, r) for t, r in zip(tensors, ref_params)),
                        velocity_exact=all(bits_equal(opt.state(i, 0), ref.velocity[i]) for i in range(len(shapes))),
                        weights_exact=all(bits_equal(t.data, r) for t, r in zip(tensors, ref_params))))
    opt.close()
    return out


def test_reference_muon_test(engine):
    """src/nn/optim/muon.rs:172-192: 2x2 parameter, values change and stay below 2.0."""
    from volta_b200 import VB_NS_F32, Muon, Tensor
    x = Tensor([1.0, -1.0, 0.5, 0.5], (2, 2), True)
    x.grad = [0.1, 0.1, -0.1, -0.1]
    opt = Muon([x], 0.1, 0.9, True, 5, ns_mode=VB_NS_F32, engine=engine, keep_update=True)
    before = x.data.copy()
    opt.step()
    after = x.data.copy()
    assert not np.array_equal(before, after)
    assert np.all(np.abs(after) < 2.0)
    opt.close()


@pytest.mark.parametrize("shapes", [
    [(2, 2)], [(48, 32), (32, 48)], [(257, 130), (64, 288), (32, 9)], [(300, 520), (1, 64), (64, 1), (40,)],
    [(32, 1, 3, 3), (64, 32, 3, 3), (128, 10)],
])
def test_f32_path_small_shapes(oracle, engine, shapes):
    """Odd sizes, conv-shaped 4-D tensors flattened to (out, in*k*k), vectors that skip
    Newton-Schulz (muon.rs:117-130,153).  The f32 path keeps the oracle's summation order, so
    beyond the 1e-5 bound the results are expected to be bit-identical."""
    from volta_b200 import VB_NS_F32
    res = _run(oracle, engine, shapes, 3, VB_NS_F32)
    for r in res:
        assert r["update"] <= TOL_F32, res
        assert r["velocity_exact"]
    assert all(r["weights_exact"] for r in res), res


@pytest.mark.parametrize("nesterov,ns_steps", [(False, 5), (True, 0), (True, 1), (True, 4)])
def test_f32_path_variants(oracle, engine, nesterov, ns_steps):
    from volta_b200 import VB_NS_F32
    res = _run(oracle, engine, [(96, 160), (200, 72)], 2, VB_NS_F32, nesterov=nesterov, ns_steps=ns_steps)
    assert all(r["update"] <= TOL_F32 and r["weights_exact"] for r in res), res


def test_f32_path_missing_gradients(oracle, engine):
    from volta_b200 import VB_NS_F32
    res = _run(oracle, engine, [(64, 64), (100, 30), (17,)], 4, VB_NS_F32, drop=lambda i, s: (i + s) % 2 == 0)
    assert all(r["weights_exact"] and r["velocity_exact"] for r in res), res


def test_f32_path_large_matrix_ordered_norm(oracle, engine):
    """A 1024 x 1024 matrix: the sequential f32 sum of a million squares is ~5e-4 below the
    exact sum, so a tree reduction would land ~2.5e-4 away from the reference, 25x outside
    the 1e-5 bound.  The ordered-sum kernel must reproduce the reference's norm exactly."""
    from volta_b200 import VB_NS_F32
    res = _run(oracle, engine, [(1024, 1024)], 1, VB_NS_F32, ns_steps=2)
    assert res[0]["update"] <= TOL_F32, res
    assert res[0]["weights_exact"], res


def test_ordered_sum_adversarial_values(oracle, engine):
    """Ties, huge dynamic range, zeros and denormals in the sum of squares: ns_steps = 0 makes
    the update exactly u / sqrt(sumsq + 1e-8), so equality of the update pins the sum."""
    from volta_b200 import VB_NS_F32, Muon, Tensor
    rng = np.random.default_rng(5)
    n_r, n_c = 96, 512
    cases = []
    cases.append(np.full((n_r, n_c), 2.0 ** -6, np.float32))                      # constant: many exact ties
    x = np.exp2(rng.integers(-20, 3, (n_r, n_c))).astype(np.float32)              # powers of two
    cases.append(x)
    x = (rng.standard_normal((n_r, n_c)) * 1e-3).astype(np.float32)
    x[::7, ::3] = 0.0
    x[5, 5] = 30.0                                                                 # one huge addend mid-stream
    cases.append(x)
    x = (rng.standard_normal((n_r, n_c)) * 1e-20).astype(np.float32)              # squares are denormal / zero
    cases.append(x)
    x = np.sort(np.abs(rng.standard_normal((n_r, n_c)).astype(np.float32)).reshape(-1))[::-1].reshape(n_r, n_c).copy()
    cases.append(x)                                                                # big first, then tiny
    for g in cases:
        w = Tensor(np.zeros((n_r, n_c), np.float32))
        opt = Muon([w], 0.1, 0.0, False, 0, ns_mode=VB_NS_F32, engine=engine, keep_update=True)
        w.grad = g
        opt.step()
        wr = np.zeros((n_r, n_c), np.float32)
        ref = oracle.Muon([wr], 0.1, 0.0, False, 0)
        ref.step([g])
        assert bits_equal(opt.last_update(0), ref.last_update[0])
        opt.close()


@pytest.mark.gpu
def test_ordered_sum_ties_on_large_matrices(oracle, engine):
    """4 M addends drawn from a few powers of two: once the running sum passes 1 the smallest square
    (2^-24) is exactly half an ulp of it, so about a third of the additions are ties whose rounding
    depends on the parity of the running sum; the blocks then run under guessed binades.  A second
    matrix mixes such values with ordinary ones so that ties and inexact addends alternate."""
    from volta_b200 import VB_NS_F32, Muon, Tensor
    rng = np.random.default_rng(11)
    n_r, n_c = 2048, 2048
    cases = [np.exp2(-rng.integers(10, 13, (n_r, n_c))).astype(np.float32)]
    x = (rng.standard_normal((n_r, n_c)) * 6e-4).astype(np.float32)
    pick = rng.random((n_r, n_c)) < 0.5
    x[pick] = np.exp2(-rng.integers(11, 14, int(pick.sum()))).astype(np.float32)
    cases.append(x)
    for g in cases:
        w = Tensor(np.zeros((n_r, n_c), np.float32))
        opt = Muon([w], 0.1, 0.0, False, 0, ns_mode=VB_NS_F32, engine=engine, keep_update=True)
        w.grad = g
        opt.step()
        wr = np.zeros((n_r, n_c), np.float32)
        ref = oracle.Muon([wr], 0.1, 0.0, False, 0)
        ref.step([g])
        assert bits_equal(opt.last_update(0), ref.last_update[0])
        opt.close()


# ---- bf16 tensor-core path (tcgen05) ----------------------------------------------------------

def _bf16_round(x):
    """float32 -> bfloat16 -> float32, round to nearest even (what the kernels store)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def _ns_bf16_model(u, steps):
    """numpy model of the bf16 path: the unnormalised update rounded to bf16 is the first operand
    and the first iteration's epilogues apply 1/norm (squared for the Gram); operands rounded to
    bf16, f32-or-better accumulation, short-side Gram.  Used to tell a wrong descriptor (O(1)
    error) from rounding (1e-3)."""
    r, c = u.shape
    inv = 1.0 / np.sqrt(np.sum(u.astype(np.float64) ** 2) + 1e-8)
    x = _bf16_round(u).astype(np.float64)
    for it in range(steps):
        s2, s1 = (inv * inv, inv) if it == 0 else (1.0, 1.0)
        if r >= c:
            cm = _bf16_round((3.0 * np.eye(c) - s2 * (x.T @ x)).astype(np.float32)).astype(np.float64)
            nx = 0.5 * s1 * (x @ cm)
        else:
            cm = _bf16_round((3.0 * np.eye(r) - s2 * (x @ x.T)).astype(np.float32)).astype(np.float64)
            nx = 0.5 * s1 * (cm @ x)
        x = nx if it == steps - 1 else _bf16_round(nx.astype(np.float32)).astype(np.float64)
    return x.astype(np.float32)


def _ns_bf16_chain_model(u, steps):
    """numpy model of the chain form of the bf16 path: with C' = 3I - G the iterate is X_0 P_k, and
    G, C', T = G C' and P' = C'_0 ... C'_{k-1} are short-side squares stored in bf16:
    T_k = G_k C'_k, G_{k+1} = C'_k T_k / 4, C'_{k+1} = 3I - G_{k+1}, P'_{k+1} = P'_k C'_k,
    X_K = 2^-K X_0 P'_K / norm."""
    if u.shape[0] < u.shape[1]:
        return _ns_bf16_chain_model(np.ascontiguousarray(u.T), steps).T
    n = u.shape[1]
    inv = 1.0 / np.sqrt(np.sum(u.astype(np.float64) ** 2) + 1e-8)
    rnd = lambda a: _bf16_round(a.astype(np.float32)).astype(np.float64)
    x0 = _bf16_round(u).astype(np.float64)
    g32 = inv * inv * (x0.T @ x0)
    g, c = rnd(g32), rnd(3.0 * np.eye(n) - g32)
    p = None
    for it in range(steps):
        if it < steps - 1:
            t = rnd(g @ c)
            a = 0.25 * (c @ t)
            g_next, c_next = rnd(a), rnd(3.0 * np.eye(n) - a)
        p = c if p is None else rnd(p @ c)
        if it < steps - 1:
            g, c = g_next, c_next
    return (inv * 0.5 ** steps * (x0 @ p)).astype(np.float32)


@pytest.mark.parametrize("form", ["chain", "chain_g_only", "per_iteration"])
@pytest.mark.parametrize("shape", [(128, 256), (256, 128), (512, 512), (384, 1024), (1024, 384), (200, 72), (72, 200),
                                   (1032, 264)])
def test_bf16_path_single_matrix(oracle, engine, shape, form, monkeypatch):
    """One matrix per launch, tall / wide / square, full and ragged tiles (dims are multiples
    of 8 but not of the 128 x 256 tile or the 64-wide k block), in both forms of the bf16 path:
    the chain of short-side squares (the default) and one Gram and one update product per
    iteration (VB_NS_CHAIN=0).  The numpy model of the form tells a wrong descriptor (O(1) error)
    from rounding (1e-3)."""
    from volta_b200 import VB_NS_BF16, Muon, Tensor
    # chain_g_only (VB_NS_CHAIN=2): the chain that stores only G, T and P, as the f32-accurate mode runs it
    monkeypatch.setenv("VB_NS_CHAIN", {"chain": "1", "chain_g_only": "2", "per_iteration": "0"}[form])
    rng = np.random.default_rng(sum(shape))
    g = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
    w = Tensor(np.zeros(shape, np.float32))
    opt = Muon([w], 0.1, 0.0, False, 5, ns_mode=VB_NS_BF16, engine=engine, keep_update=True)
    w.grad = g
    opt.step()
    got = opt.last_update(0)
    ref = oracle.newton_schulz(g, 5)
    if form != "chain_g_only":
        model = _ns_bf16_chain_model(g, 5) if form == "chain" else _ns_bf16_model(g, 5)
        assert rel_frobenius(got, model) < 3e-3, (rel_frobenius(got, model), rel_frobenius(got, ref))
    assert rel_frobenius(got, ref) <= TOL_BF16
    assert np.allclose(w.data, -(np.float32(0.1) * got) * np.float32(0.1), rtol=0, atol=1e-9)
    opt.close()


@pytest.mark.parametrize("ns_steps", [1, 2, 3, 7])
def test_bf16_chain_form_iteration_counts_and_spectra(oracle, engine, ns_steps):
    """The chain form across iteration counts, on a matrix whose singular values span e^-10."""
    from volta_b200 import VB_NS_BF16, Muon, Tensor
    rng = np.random.default_rng(ns_steps)
    m, n = 768, 256
    q1, _ = np.linalg.qr(rng.standard_normal((m, n)))
    q2, _ = np.linalg.qr(rng.standard_normal((n, n)))
    g = ((q1 * np.exp(-10.0 * np.arange(n) / n)) @ q2.T).astype(np.float32) * np.float32(1e-3)
    w = Tensor(np.zeros((m, n), np.float32))
    opt = Muon([w], 0.1, 0.0, False, ns_steps, ns_mode=VB_NS_BF16, engine=engine, keep_update=True)
    w.grad = g
    opt.step()
    err = rel_frobenius(opt.last_update(0), oracle.newton_schulz(g, ns_steps))
    assert err <= TOL_BF16, err
    opt.close()


def test_bf16_path_mixed_list_three_steps(oracle, engine):
    """Several matrices in one optimizer (tensor-core shapes, a shape that falls back to the
    f32 kernels because its rows are not 16-byte aligned in bf16, and a vector), momentum and
    Nesterov on, three steps."""
    from volta_b200 import VB_NS_BF16
    shapes = [(256, 256), (768, 256), (256, 1024), (64, 36), (100,), (512, 128)]
    res = _run(oracle, engine, shapes, 3, VB_NS_BF16)
    for r in res:
        assert r["update"] <= TOL_BF16, res
        assert r["velocity_exact"]


def test_bf16_path_missing_gradients(oracle, engine):
    from volta_b200 import VB_NS_BF16
    res = _run(oracle, engine, [(256, 256), (128, 384), (384, 128)], 4, VB_NS_BF16,
               drop=lambda i, s: (i + s) % 2 == 0)
    assert all(r["update"] <= TOL_BF16 and r["velocity_exact"] for r in res), res


def test_bf16_path_c4_layer_shapes(oracle, engine):
    """The four matrix shapes of one layer of the Muon benchmark configuration (3072x1024,
    1024x1024, 4096x1024, 1024x4096) at full size, one step, against the f32 oracle."""
    from volta_b200 import VB_NS_BF16, Muon, Tensor
    oracle.set_threads(oracle.max_threads())
    shapes = [(3072, 1024), (1024, 1024), (4096, 1024), (1024, 4096)]
    rng = np.random.default_rng(11)
    grads = [(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in shapes]
    tensors = [Tensor((rng.standard_normal(s) * 0.02).astype(np.float32)) for s in shapes]
    opt = Muon(tensors, 0.1, 0.9, True, 5, ns_mode=VB_NS_BF16, engine=engine, keep_update=True)
    for t, g in zip(tensors, grads):
        t.grad = g
    opt.step()
    # executed FLOPs: symmetric products only on and above the diagonal (10 of 16 tiles of 256 x 256
    # for a 1024 x 1024 square)
    # chain form: the first Gram and 3 (K - 1) short-side squares on the upper tiles, the last product in full
    assert opt.last_ns_flops == sum(2.0 * max(s) * min(s) ** 2 * (1 + 10 / 16) + 12 * 2.0 * min(s) ** 3 * (10 / 16)
                                    for s in shapes)
    for i, (s, g) in enumerate(zip(shapes, grads)):
        u = np.float32(0.9) * g + g  # first step: v = g, Nesterov update = mu*v + g
        # short-side form of the reference iteration on the oracle (same mathematics, 4x less
        # CPU work for the 1024x4096 matrix): NS(X)^T == NS(X^T)
        ref = oracle.newton_schulz(u, 5) if s[0] >= s[1] else oracle.newton_schulz(np.ascontiguousarray(u.T), 5).T
        err = rel_frobenius(opt.last_update(i), ref)
        assert err <= TOL_BF16, (s, err)
    opt.close()


# ---- f32-accurate tensor-core path (two f16 planes per operand) ----------------------------------

@pytest.mark.parametrize("form", ["chain", "per_iteration"])
@pytest.mark.parametrize("shapes", [[(256, 128)], [(128, 384), (512, 512)], [(200, 72), (64, 36), (50,)], [(1032, 264)]])
def test_f32_tc_path_meets_f32_tolerance(oracle, engine, shapes, form, monkeypatch):
    """VB_NS_F32_TC: operands held as two f16 planes, three tensor-core products per product,
    ordered sum of squares.  Same 1e-5 bound as the bit-faithful path (shapes whose rows are
    not 16-byte aligned in bf16 run the bit-faithful kernels inside the same optimizer).  Both
    forms: the chain of short-side squares (default) and one Gram and one update product per
    iteration (VB_NS_CHAIN=0)."""
    from volta_b200 import VB_NS_F32_TC
    monkeypatch.setenv("VB_NS_CHAIN", "1" if form == "chain" else "0")
    res = _run(oracle, engine, shapes, 3, VB_NS_F32_TC)
    for r in res:
        assert r["update"] <= TOL_F32, res
        assert r["velocity_exact"]


def test_f32_tc_path_c4_layer_shapes(oracle, engine):
    """One layer of the benchmark configuration at full size on the f32-accurate tensor-core
    path, against the f32 oracle and its f64-accumulating variant."""
    from volta_b200 import VB_NS_F32_TC, Muon, Tensor
    oracle.set_threads(oracle.max_threads())
    shapes = [(3072, 1024), (1024, 1024), (4096, 1024)]
    rng = np.random.default_rng(12)
    grads = [(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in shapes]
    tensors = [Tensor((rng.standard_normal(s) * 0.02).astype(np.float32)) for s in shapes]
    opt = Muon(tensors, 0.1, 0.9, True, 5, ns_mode=VB_NS_F32_TC, engine=engine, keep_update=True)
    for t, g in zip(tensors, grads):
        t.grad = g
    opt.step()
    for i, g in enumerate(grads):
        u = np.float32(0.9) * g + g
        got = opt.last_update(i)
        assert rel_frobenius(got, oracle.newton_schulz(u, 5)) <= TOL_F32
        assert rel_frobenius(got, oracle.newton_schulz(u, 5, gemm_mode=1)) <= TOL_F32
    opt.close()


def test_f32_tc_tiny_updates(oracle, engine):
    """Updates far smaller than sqrt(1e-8): the 1e-8 under the root dominates the norm
    (muon.rs:59), the normalised update is tiny and the f16 pieces are held with a larger power of
    two so that they stay in the normal f16 range.  Same 1e-5 bound; zero gradients give zero."""
    from volta_b200 import VB_NS_F32_TC, Muon, Tensor
    rng = np.random.default_rng(21)
    for scale in (1e-15, 1e-13, 1e-11, 1e-9, 1e-7, 1e-5):
        g = (rng.standard_normal((128, 64)) * scale).astype(np.float32)
        w = Tensor(np.ones((128, 64), np.float32))
        opt = Muon([w], 0.1, 0.0, False, 5, ns_mode=VB_NS_F32_TC, engine=engine, keep_update=True)
        w.grad = g
        opt.step()
        got = opt.last_update(0)
        assert np.all(np.isfinite(got))
        assert rel_frobenius(got, oracle.newton_schulz(g, 5)) <= TOL_F32, scale
        opt.close()
    w = Tensor(np.ones((128, 64), np.float32))
    opt = Muon([w], 0.1, 0.0, False, 5, ns_mode=VB_NS_F32_TC, engine=engine, keep_update=True)
    w.grad = np.zeros((128, 64), np.float32)
    opt.step()
    assert not np.any(opt.last_update(0)) and np.array_equal(w.data, np.ones((128, 64), np.float32))
    opt.close()


@pytest.mark.parametrize("mode_name", ["bf16", "f32_tc"])
def test_tensor_core_paths_across_gradient_scales(oracle, engine, mode_name):
    """Gradient magnitudes from 1e-15 to 1e15: the tensor-core paths stay finite and inside their
    bounds (bf16 operands have f32's range; the f16 pieces carry a per-matrix power of two)."""
    from volta_b200 import VB_NS_BF16, VB_NS_F32_TC, Muon, Tensor
    mode, tol = (VB_NS_BF16, TOL_BF16) if mode_name == "bf16" else (VB_NS_F32_TC, TOL_F32)
    rng = np.random.default_rng(5)
    for scale in (1e-15, 1e-10, 1e-6, 1.0, 1e4, 1e8, 1e15):
        g = (rng.standard_normal((256, 128)) * scale).astype(np.float32)
        w = Tensor(np.ones((256, 128), np.float32))
        opt = Muon([w], 0.1, 0.0, False, 5, ns_mode=mode, engine=engine, keep_update=True)
        w.grad = g
        opt.step()
        got = opt.last_update(0)
        assert np.all(np.isfinite(got)), scale
        assert rel_frobenius(got, oracle.newton_schulz(g, 5)) <= tol, scale
        opt.close()


@pytest.mark.parametrize("ns_steps", [0, 1, 2, 3, 6])
@pytest.mark.parametrize("mode_name", ["bf16", "f32_tc", "f32"])
def test_iteration_counts(oracle, engine, mode_name, ns_steps):
    """First == last iteration, odd and even counts, none at all: tall, wide and square matrices
    (the tall update changes form between the last iteration and the others)."""
    from volta_b200 import VB_NS_BF16, VB_NS_F32, VB_NS_F32_TC, Muon, Tensor
    mode, tol = {"bf16": (VB_NS_BF16, TOL_BF16), "f32_tc": (VB_NS_F32_TC, TOL_F32), "f32": (VB_NS_F32, 0.0)}[mode_name]
    rng = np.random.default_rng(100 + ns_steps)
    shapes = [(512, 256), (256, 512), (256, 256), (264, 72)]
    grads = [(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in shapes]
    tensors = [Tensor(np.zeros(s, np.float32)) for s in shapes]
    opt = Muon(tensors, 0.1, 0.0, False, ns_steps, ns_mode=mode, engine=engine, keep_update=True)
    for t, g in zip(tensors, grads):
        t.grad = g
    opt.step()
    for i, g in enumerate(grads):
        got, ref = opt.last_update(i), oracle.newton_schulz(g, ns_steps)
        if mode_name == "f32" or ns_steps == 0:
            # no iteration: the result is the normalised update itself, exact on every path
            assert bits_equal(got, ref) or rel_frobenius(got, ref) <= tol, (shapes[i], rel_frobenius(got, ref))
        else:
            assert rel_frobenius(got, ref) <= tol, (shapes[i], rel_frobenius(got, ref))
    opt.close()


@pytest.mark.parametrize("mode_name", ["f32", "f32_tc"])
def test_f32_paths_hold_their_bound_whatever_the_summation_order(oracle, engine, mode_name):
    """The reference's contraction is a third-party SGEMM whose exact order of f32 additions is not
    part of the reference tree, so the oracle's f32 order is a restatement.  The 1e-5 bound must
    not hinge on that order: both f32 paths are also compared with the oracle accumulating every
    dot product in f64 (the correctly rounded contraction, from which any f32 order deviates by a
    few 1e-7 at these sizes), and the two oracles with each other."""
    from volta_b200 import VB_NS_F32, VB_NS_F32_TC, Muon, Tensor
    oracle.set_threads(oracle.max_threads())
    mode = VB_NS_F32 if mode_name == "f32" else VB_NS_F32_TC
    rng = np.random.default_rng(77)
    for shape in ((1024, 512), (512, 1024), (768, 768)):
        g = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
        w = Tensor(np.zeros(shape, np.float32))
        opt = Muon([w], 0.1, 0.0, False, 5, ns_mode=mode, engine=engine, keep_update=True)
        w.grad = g
        opt.step()
        got = opt.last_update(0)
        f32_order, f64_acc = oracle.newton_schulz(g, 5), oracle.newton_schulz(g, 5, gemm_mode=1)
        assert rel_frobenius(got, f64_acc) <= TOL_F32, (shape, rel_frobenius(got, f64_acc))
        assert rel_frobenius(got, f32_order) <= TOL_F32
        assert rel_frobenius(f32_order, f64_acc) <= TOL_F32 / 3
        opt.close()
    oracle.set_threads(1)


# ---- one whole layer of the benchmark configuration, three consecutive steps, all three modes --------

C4_LAYER = [(3072, 1024), (1024, 1024), (4096, 1024), (1024, 4096)]


@pytest.fixture(scope="module")
def c4_layer_reference(oracle):
    """The CPU oracle on one full layer (3072x1024, 1024x1024, 4096x1024 and the wide 1024x4096, the
    latter in the reference's own cols x cols formulation, src/nn/optim/muon.rs:73), momentum 0.9 with
    Nesterov, five Newton-Schulz iterations, three consecutive steps: ~1.5 TFLOP of CPU work on all
    host threads.  Computed once for the three modes."""
    oracle.set_threads(oracle.max_threads())
    rng = np.random.default_rng(2024)
    start = [(rng.standard_normal(s) * 0.02).astype(np.float32) for s in C4_LAYER]
    grads = [[(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in C4_LAYER] for _ in range(3)]
    params = [p.copy() for p in start]
    ref = oracle.Muon(params, 0.1, 0.9, True, 5)
    updates, weights, velocity = [], [], []
    for gs in grads:
        ref.step(gs)
        updates.append([u.copy() for u in ref.last_update])
        weights.append([p.copy() for p in params])
        velocity.append([v.copy() for v in ref.velocity])
    oracle.set_threads(1)
    return dict(start=start, grads=grads, updates=updates, weights=weights, velocity=velocity)


@pytest.mark.parametrize("mode_name", ["f32", "f32_tc", "bf16"])
def test_c4_layer_three_steps_with_momentum(engine, c4_layer_reference, mode_name):
    """Momentum carried through Newton-Schulz at full size: per step the update of every matrix
    (the wide one included) against the oracle, the velocity bit for bit, and the weights, whose
    distance travelled since the start must agree to the mode's bound (bit for bit on the f32 path)."""
    from volta_b200 import VB_NS_BF16, VB_NS_F32, VB_NS_F32_TC, Muon, Tensor
    mode, tol = {"f32": (VB_NS_F32, 0.0), "f32_tc": (VB_NS_F32_TC, TOL_F32), "bf16": (VB_NS_BF16, TOL_BF16)}[mode_name]
    ref = c4_layer_reference
    tensors = [Tensor(p.copy()) for p in ref["start"]]
    opt = Muon(tensors, 0.1, 0.9, True, 5, ns_mode=mode, engine=engine, keep_update=True)
    for step in range(3):
        opt.zero_grad()
        for t, g in zip(tensors, ref["grads"][step]):
            t.grad = g
        opt.step()
        for i, shape in enumerate(C4_LAYER):
            got = opt.last_update(i)
            want = ref["updates"][step][i]
            assert bits_equal(opt.state(i, 0), ref["velocity"][step][i]), (step, shape)
            if mode_name == "f32":
                assert bits_equal(got, want), (step, shape, rel_frobenius(got, want))
                assert bits_equal(tensors[i].data, ref["weights"][step][i]), (step, shape)
            else:
                assert rel_frobenius(got, want) <= tol, (step, shape, rel_frobenius(got, want))
                moved = tensors[i].data.astype(np.float64) - ref["start"][i]
                moved_ref = ref["weights"][step][i].astype(np.float64) - ref["start"][i]
                # f32 weights of size 0.02 carry ~1e-8 of rounding per step of size ~1e-5: allow for it
                assert rel_frobenius(moved, moved_ref) <= tol + 2e-3 * (mode_name == "f32_tc"), (step, shape)
    opt.close()


def test_f32_path_tall_c4_matrix_five_iterations(oracle, engine):
    """The bit-faithful kernels at the benchmark's tall shape with all five iterations."""
    from volta_b200 import VB_NS_F32, Muon, Tensor
    oracle.set_threads(oracle.max_threads())
    rng = np.random.default_rng(8)
    g = (rng.standard_normal((4096, 1024)) * 1e-3).astype(np.float32)
    w = Tensor(np.zeros((4096, 1024), np.float32))
    opt = Muon([w], 0.1, 0.0, False, 5, ns_mode=VB_NS_F32, engine=engine, keep_update=True)
    w.grad = g
    opt.step()
    assert bits_equal(opt.last_update(0), oracle.newton_schulz(g, 5))
    oracle.set_threads(1)
    opt.close()


@pytest.mark.parametrize("mode_name", ["bf16", "f32_tc"])
def test_apply_fused_into_the_last_launch_gives_the_same_weights(oracle, engine, mode_name):
    """By default the tensor-core modes apply the update inside their last launch and never store
    it; with keep_update it is stored as well.  The weights must be the same bit for bit either way
    (and they are compared with the oracle wherever the update is: every test above keeps it), over
    full and ragged tiles, a matrix on the f32 kernels, a vector, missing gradients and momentum."""
    from volta_b200 import VB_NS_BF16, VB_NS_F32_TC, Muon, Tensor, VoltaB200Error
    mode = VB_NS_BF16 if mode_name == "bf16" else VB_NS_F32_TC
    shapes = [(512, 256), (256, 768), (264, 72), (1032, 264), (64, 36), (50,), (256, 256)]
    rng = np.random.default_rng(17)
    start = [(rng.standard_normal(s) * 0.02).astype(np.float32) for s in shapes]
    grads = [[(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in shapes] for _ in range(3)]
    results = []
    for keep in (True, False):
        tensors = [Tensor(p.copy()) for p in start]
        opt = Muon(tensors, 0.1, 0.9, True, 5, ns_mode=mode, engine=engine, keep_update=keep)
        for step, gs in enumerate(grads):
            opt.zero_grad()
            for i, (t, g) in enumerate(zip(tensors, gs)):
                if (i + step) % 4 != 3:      # some gradients are missing in every step
                    t.grad = g
            opt.step()
        if not keep:
            with pytest.raises(VoltaB200Error) as ei:
                opt.last_update(0)
            assert ei.value.status == 5           # not stored: VB_ERR_STATE
            assert opt.last_update(4).shape == (64, 36)   # the f32-kernel matrix always is
        results.append([t.data.copy() for t in tensors])
        opt.close()
    for a, b, p0 in zip(results[0], results[1], start):
        assert bits_equal(a, b)
        assert not bits_equal(a, p0)


WIDE_TILE_CHECK = r"""
import sys
import numpy as np
sys.path.insert(0, {root!r})
import oracle
import volta_b200
from volta_b200 import VB_NS_BF16, Engine, Muon, Tensor
oracle.build()
eng = Engine(0)
rng = np.random.default_rng(31)
shapes = [(1024, 512), (512, 1024), (1024, 1024), (1536, 512), (384, 256), (264, 72)]
start = [(rng.standard_normal(s) * 0.02).astype(np.float32) for s in shapes]
tensors = [Tensor(p.copy()) for p in start]
opt = Muon(tensors, 0.1, 0.9, True, 5, ns_mode=VB_NS_BF16, engine=eng, keep_update=True)
ref_p = [p.copy() for p in start]
ref = oracle.Muon(ref_p, 0.1, 0.9, True, 5)
worst = 0.0
for step in range(2):
    gs = [(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in shapes]
    for t, g in zip(tensors, gs):
        t.grad = g
    opt.step()
    ref.step(gs)
    for i in range(len(shapes)):
        a, b = opt.last_update(i).astype(np.float64), ref.last_update[i].astype(np.float64)
        worst = max(worst, float(np.linalg.norm(a - b) / np.linalg.norm(b)))
moved = max(float(np.linalg.norm(t.data.astype(np.float64) - r) / np.linalg.norm(r.astype(np.float64) - p0))
            for t, r, p0 in zip(tensors, ref_p, start))
opt.close()
eng.close()
print("WORST", worst, moved)
assert worst <= 2e-2 and moved <= 2e-2
"""


def test_wide_tiles_when_selected():
    """VB_TC_WIDE=1 / VB_TC_WIDE_GRAM=1 run the update products whose width is a multiple of 512, and
    the symmetric Gram products, on 256 x 512 tiles (both accumulator halves share the staged rows
    of A; Gram tiles come with one or two halves and the half on the diagonal reads A's rows as
    its B).  The variants are off by default because they measured slower; selected, they must
    meet the same bound.  The switches are read once per process, hence the child process."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, VB_TC_WIDE="1", VB_TC_WIDE_GRAM="1", VB_NS_CHAIN="0")  # the wide tiles belong to the per-iteration form
    r = subprocess.run([sys.executable, "-c", WIDE_TILE_CHECK.format(root=root)], env=env, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "WORST" in r.stdout
