"""The oracle against the reference's own known-answer tests (CPU only).

The expected values in tests/golden/volta_optimizer_kats.json are the hand computations
the reference's tests assert against (see tests/golden/make_kats.py for the file:line of
each); tolerances are the reference's.
"""
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "volta_optimizer_kats.json")
with open(GOLDEN) as fh:
    KATS = json.load(fh)


def _close(actual, expected, case):
    if "tol_rel" in case:
        assert abs(actual - expected) <= case["tol_rel"] * max(abs(expected), abs(actual)), (actual, expected)
    else:
        assert abs(actual - expected) < case["tol_abs"], (actual, expected)


@pytest.mark.parametrize("case", [c for c in KATS if c["kind"] in ("adam", "sgd")], ids=lambda c: c["name"])
def test_oracle_matches_reference_kat(oracle, case):
    theta = np.array([case["theta0"]], np.float32)
    grad = np.array([case["grad"]], np.float32)
    if case["kind"] == "adam":
        opt = oracle.Adam([theta], case["lr"], tuple(case["betas"]), case["eps"], case["weight_decay"])
    else:
        opt = oracle.SGD([theta], case["lr"], case["momentum"], case["weight_decay"])
    for step in range(case["steps"]):
        opt.step([grad])
        _close(float(theta[0]), case["expected"][step], case)


def test_oracle_muon_property(oracle):
    case = next(c for c in KATS if c["kind"] == "muon")
    w = np.array(case["theta0"], np.float32).reshape(case["shape"])
    before = w.copy()
    opt = oracle.Muon([w], case["lr"], case["momentum"], case["nesterov"], case["ns_steps"])
    opt.step([np.array(case["grad"], np.float32).reshape(case["shape"])])
    assert not np.array_equal(before, w)
    assert np.all(np.abs(w) < case["bound_abs"])


def test_powi_is_square_and_multiply(oracle):
    """f32::powi differs from a correctly rounded pow from small t on (beta2 = 0.999), and
    the difference is amplified in 1/(1 - beta^t): the bias correction must use powi."""
    beta = np.float32(0.999)
    differing = 0
    for t in range(1, 201):
        exact = np.float32(float(beta) ** t)  # f64 pow of the f32 value, rounded once
        if oracle.powi(beta, t) != exact:
            differing += 1
    assert differing > 50
    # structure: powi(a, 5) = (a * (a^2)^2) with every product rounded
    a = np.float32(0.9)
    a2 = np.float32(a * a)
    a4 = np.float32(a2 * a2)
    assert oracle.powi(a, 5) == np.float32(a * a4)
    assert oracle.powi(a, 1) == a
    assert oracle.powi(a, 0) == np.float32(1.0)
    assert oracle.powi(a, 2) == a2


def test_adam_uses_fused_multiply_add_where_reference_does(oracle):
    """m = beta1.mul_add(m, (1-beta1)*g) (adam.rs:176): a single rounding of beta1*m + c."""
    rng = np.random.default_rng(0)
    n = 4096
    theta = rng.standard_normal(n).astype(np.float32)
    g = (rng.standard_normal(n) * 0.01).astype(np.float32)
    opt = oracle.Adam([theta], 1e-3, (0.9, 0.999), 1e-8, 0.0)
    opt.m[0][:] = rng.standard_normal(n).astype(np.float32)
    m0 = opt.m[0].copy()
    opt.step([g])
    b1 = np.float32(0.9)
    c = (np.float32(1.0) - b1) * g
    fused = (b1.astype(np.float64) * m0.astype(np.float64) + c.astype(np.float64)).astype(np.float32)
    assert np.array_equal(opt.m[0], fused)  # f64 holds the f32 product exactly: one rounding
    unfused = (b1 * m0).astype(np.float32) + c
    assert not np.array_equal(opt.m[0], unfused)


def test_adam_skip_rule_and_t(oracle):
    """Parameters without a gradient are skipped but t still advances (adam.rs:71,81-84)."""
    a = np.ones(8, np.float32)
    b = np.ones(8, np.float32)
    opt = oracle.Adam([a, b], 1e-2, (0.9, 0.999), 1e-8, 0.0)
    g = np.full(8, 0.5, np.float32)
    opt.step([g, None])
    assert opt.t == 1 and np.all(b == 1.0) and np.all(a != 1.0)
    opt.step([None, g])
    assert opt.t == 2
    # b's first update uses t = 2 bias correction with m, v from a single accumulation
    s1, s2 = oracle.adam_bias_scales(0.9, 0.999, 2)
    m = np.float32(np.float32(0.1) * np.float32(0.5))
    assert np.float32(0.1) != np.float32(1.0) - np.float32(0.9)  # (1 - beta1) is computed in f32
    m = np.float32((np.float32(1.0) - np.float32(0.9)) * np.float32(0.5))
    v = np.float32((np.float32(1.0) - np.float32(0.999)) * np.float32(0.25))
    expect = np.float32(1.0) - np.float32(np.float32(np.float32(1e-2) * np.float32(m * s1)) /
                                          np.float32(np.sqrt(np.float32(v * s2)) + np.float32(1e-8)))
    assert np.all(b == expect)


def test_sgd_variants(oracle):
    p = np.array([1.0, -2.0, 3.0], np.float32)
    g = np.array([0.5, 0.25, -1.0], np.float32)
    opt = oracle.SGD([p], 0.1, 0.0, 0.0)
    assert opt.velocity == []  # sgd.rs:30
    opt.step([g])
    assert np.array_equal(p, np.array([1.0, -2.0, 3.0], np.float32) - np.float32(0.1) * g)


def test_sequential_sum_is_not_the_true_norm(oracle):
    """muon.rs:58 is a left-to-right f32 fold; at Muon sizes it is far from the exact sum."""
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(1 << 20) * 1e-3).astype(np.float32)
    seq = float(oracle.sum_sq_sequential(x))
    exact = float(np.sum(x.astype(np.float64) ** 2))
    manual = np.float32(0)
    for v in x[:1000]:
        manual = np.float32(manual + np.float32(v * v))
    assert float(oracle.sum_sq_sequential(x[:1000])) == float(manual)
    assert 1e-5 < abs(seq - exact) / exact < 1e-2


def test_sgemm_blocking_and_accuracy(oracle):
    rng = np.random.default_rng(2)
    a = rng.standard_normal((37, 600)).astype(np.float32)
    b = rng.standard_normal((600, 29)).astype(np.float32)
    c = oracle.sgemm(a, b)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert np.max(np.abs(c - ref)) / np.max(np.abs(ref)) < 1e-5
    c64 = oracle.sgemm(a, b, f64acc=True)
    assert np.array_equal(c64, ref.astype(np.float32))
    # k <= 256: a single fused chain per element, in k order
    a1, b1 = a[:1, :5], b[:5, :1]
    acc = np.float64(0)
    chain = np.float32(0)
    for k in range(5):
        chain = np.float32(np.float64(a1[0, k]) * np.float64(b1[k, 0]) + np.float64(chain))
    assert oracle.sgemm(a1, b1)[0, 0] == chain


def test_newton_schulz_moves_singular_values_towards_one(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((48, 32)).astype(np.float32)
    y = oracle.newton_schulz(x, 5)
    s_before = np.linalg.svd(x / np.linalg.norm(x), compute_uv=False)
    s_after = np.linalg.svd(y.astype(np.float64), compute_uv=False)
    assert np.all(s_after > s_before - 1e-6) and np.all(s_after < 1.0 + 1e-4)
    y64 = oracle.newton_schulz(x, 5, gemm_mode=1)
    assert np.linalg.norm(y - y64) / np.linalg.norm(y64) < 1e-5


def test_muon_skips_ns_for_vectors(oracle):
    """rows == 1 or cols == 1: plain momentum update scaled by 0.1 (muon.rs:153,159)."""
    w = np.ones(16, np.float32)
    g = np.full(16, 0.25, np.float32)
    opt = oracle.Muon([w], 0.1, 0.9, False, 5)
    opt.step([g])
    assert np.array_equal(w, np.float32(1.0) - np.float32(np.float32(0.1) * g) * np.float32(0.1))


def test_wgsl_restatement_within_reference_tolerance(oracle):
    """The shader math agrees with the CPU path to the 1e-4 the reference asks of it
    (src/lib.rs:3872-3877)."""
    rng = np.random.default_rng(4)
    n = 1000
    p = rng.standard_normal(n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    p_cpu = p.copy()
    opt = oracle.Adam([p_cpu], 1e-3, (0.9, 0.999), 1e-8, 0.01)
    opt.step([g])
    p_gpu, m, v = p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    oracle.wgsl_optimizer_step(p_gpu, g, m, v, 2, 1e-3, 0.9, 0.999, 1.0, 1e-8, 0.01)
    assert np.max(np.abs(p_gpu - p_cpu)) < 1e-4
