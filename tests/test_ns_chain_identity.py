"""The algebra behind the chain forms of Newton-Schulz, checked on the CPU against the oracle's
restatement of the reference's iteration (src/nn/optim/muon.rs:49-104).

The tensor-core modes do not run `C = 3I - X^T X; X = 0.5 X C` iteration by iteration.  All the
Gram matrices of the iteration are polynomials in the first one, hence symmetric and commuting,
and the iterate is the first operand times a short-side square:

* bf16 mode:          T_k = G_k C'_k, G_{k+1} = C'_k T_k / 4, C'_{k+1} = 3I - G_{k+1},
                      P'_{k+1} = P'_k C'_k (P'_1 = C'_0), X_K = 2^-K X_0 P'_K
* f32-accurate mode:  T_k = 1.5 G_k - 0.5 G_k G_k, G_{k+1} = 1.5 T_k - 0.5 G_k T_k,
                      P_{k+1} = 1.5 P_k - 0.5 P_k G_k (P_0 = I), X_K = X_0 P_K

In float64 both must reproduce the iteration to rounding."""
import numpy as np
import pytest


def _reference_iteration(u, steps):
    x = u.astype(np.float64)
    x = x / np.sqrt(np.sum(x * x) + 1e-8)
    for _ in range(steps):
        g = x.T @ x
        x = 0.5 * (x @ (3.0 * np.eye(g.shape[0]) - g))
    return x


def _chain_bf16_mode(u, steps):
    x0 = u.astype(np.float64)
    inv = 1.0 / np.sqrt(np.sum(x0 * x0) + 1e-8)
    n = x0.shape[1]
    g = inv * inv * (x0.T @ x0)
    c = 3.0 * np.eye(n) - g
    p = None
    for k in range(steps):
        if k + 1 < steps:
            t = g @ c
            g_next = 0.25 * (c @ t)
            c_next = 3.0 * np.eye(n) - g_next
        p = c if p is None else p @ c
        if k + 1 < steps:
            g, c = g_next, c_next
    return inv * 0.5 ** steps * (x0 @ p)


def _chain_f32_accurate_mode(u, steps):
    x0 = u.astype(np.float64)
    x0 = x0 / np.sqrt(np.sum(x0 * x0) + 1e-8)
    g = x0.T @ x0
    p = np.eye(x0.shape[1])
    for k in range(steps):
        p_next = 1.5 * p - 0.5 * (p @ g)
        if k + 1 < steps:
            t = 1.5 * g - 0.5 * (g @ g)
            g = 1.5 * t - 0.5 * (g @ t)
        p = p_next
    return x0 @ p


@pytest.mark.parametrize("shape", [(96, 32), (64, 64), (200, 72)])
@pytest.mark.parametrize("steps", [1, 2, 5, 7])
def test_chain_forms_equal_the_iteration_in_exact_arithmetic(shape, steps):
    rng = np.random.default_rng(shape[0] + steps)
    u = rng.standard_normal(shape) * 1e-3
    want = _reference_iteration(u, steps)
    scale = np.linalg.norm(want)
    assert np.linalg.norm(_chain_bf16_mode(u, steps) - want) <= 1e-12 * scale
    assert np.linalg.norm(_chain_f32_accurate_mode(u, steps) - want) <= 1e-12 * scale


def test_the_float64_iteration_is_the_oracles(oracle):
    """The float64 iteration used above agrees with the oracle's f32 restatement of the reference
    to f32 rounding, so the identities are statements about the reference's iteration."""
    rng = np.random.default_rng(5)
    u = (rng.standard_normal((96, 32)) * 1e-3).astype(np.float32)
    got = oracle.newton_schulz(u, 5)
    want = _reference_iteration(u, 5)
    assert np.linalg.norm(got - want) <= 1e-5 * np.linalg.norm(want)
