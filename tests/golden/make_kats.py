"""Regenerates ``volta_optimizer_kats.json``: the known-answer tests the reference holds
for its optimizers, written down as (inputs, expected values, tolerance).

Each case restates the *hand computation the reference test itself performs* (in numpy
float32, independent of the oracle's C code), so the expected values are the ones the
reference's own assertions compare against:

* adam_bias_correction        tests/test_optimizers.rs:13-48
* adam_mv_accumulation        tests/test_optimizers.rs:50-89
* adam_weight_decay(+no_wd)   tests/test_optimizers.rs:91-140
* sgd_no_momentum_simple      tests/test_optimizers.rs:168-196
* sgd_weight_decay            tests/test_optimizers.rs:198-223
* sgd_momentum_logic          tests/coverage_fill.rs:45-67
* weight_decay_sgd            src/lib.rs:3102-3119

Run:  python tests/golden/make_kats.py
"""
import json
import os

import numpy as np

f = np.float32


def adam_hand(theta0, grad, lr, b1, b2, eps, wd, steps):
    """The reference tests' hand formula: unfused EMA, division by (1 - beta^t)."""
    theta0, grad, lr, b1, b2, eps, wd = map(f, (theta0, grad, lr, b1, b2, eps, wd))
    m = f(0)
    v = f(0)
    theta = theta0
    out = []
    for t in range(1, steps + 1):
        g = grad + wd * theta if wd != 0 else grad
        m = b1 * m + (f(1) - b1) * g
        v = b2 * v + (f(1) - b2) * (g * g)
        b1t = f(1)
        b2t = f(1)
        for _ in range(t):  # powi by repeated product is exact enough for the 1e-6/1e-7 bound
            b1t = b1t * b1
            b2t = b2t * b2
        m_hat = m / (f(1) - b1t)
        v_hat = v / (f(1) - b2t)
        theta = theta - lr * m_hat / (np.sqrt(v_hat) + eps)
        out.append(float(theta))
    return out


def main():
    cases = []
    cases.append(dict(name="adam_bias_correction", kind="adam", theta0=1.0, grad=0.5, lr=0.01,
                      betas=[0.9, 0.999], eps=1e-8, weight_decay=0.0, steps=1,
                      expected=adam_hand(1.0, 0.5, 0.01, 0.9, 0.999, 1e-8, 0.0, 1), tol_abs=1e-7,
                      ref="tests/test_optimizers.rs:13-48"))
    cases.append(dict(name="adam_mv_accumulation_multi_step", kind="adam", theta0=2.0, grad=0.5,
                      lr=0.01, betas=[0.9, 0.999], eps=1e-8, weight_decay=0.0, steps=3,
                      expected=adam_hand(2.0, 0.5, 0.01, 0.9, 0.999, 1e-8, 0.0, 3), tol_abs=1e-6,
                      ref="tests/test_optimizers.rs:50-89"))
    cases.append(dict(name="adam_weight_decay", kind="adam", theta0=2.0, grad=0.0, lr=0.01,
                      betas=[0.9, 0.999], eps=1e-8, weight_decay=0.01, steps=1,
                      expected=adam_hand(2.0, 0.0, 0.01, 0.9, 0.999, 1e-8, 0.01, 1), tol_abs=1e-7,
                      ref="tests/test_optimizers.rs:91-140"))
    cases.append(dict(name="adam_no_weight_decay_zero_grad", kind="adam", theta0=2.0, grad=0.0,
                      lr=0.01, betas=[0.9, 0.999], eps=1e-8, weight_decay=0.0, steps=1,
                      expected=[2.0], tol_abs=1e-8, ref="tests/test_optimizers.rs:112-116"))
    e1 = f(5.0) - f(0.1) * f(2.0)
    e2 = e1 - f(0.1) * f(2.0)
    cases.append(dict(name="sgd_no_momentum_simple", kind="sgd", theta0=5.0, grad=2.0, lr=0.1,
                      momentum=0.0, weight_decay=0.0, steps=2, expected=[float(e1), float(e2)],
                      tol_abs=1e-7, ref="tests/test_optimizers.rs:168-196"))
    eff = f(1.0) + f(0.1) * f(4.0)
    cases.append(dict(name="sgd_weight_decay", kind="sgd", theta0=4.0, grad=1.0, lr=0.1,
                      momentum=0.0, weight_decay=0.1, steps=1,
                      expected=[float(f(4.0) - f(0.1) * eff)], tol_abs=1e-7,
                      ref="tests/test_optimizers.rs:198-223"))
    cases.append(dict(name="sgd_momentum_logic", kind="sgd", theta0=1.0, grad=0.1, lr=0.1,
                      momentum=0.9, weight_decay=0.0, steps=2, expected=[0.99, 0.971],
                      tol_abs=1e-6, ref="tests/coverage_fill.rs:45-67"))
    cases.append(dict(name="weight_decay_sgd", kind="sgd", theta0=1.0, grad=0.0, lr=0.1,
                      momentum=0.0, weight_decay=0.1, steps=1, expected=[0.99], tol_rel=1e-6,
                      ref="src/lib.rs:3102-3119"))
    # src/nn/optim/muon.rs:172-192 holds no numbers: only "changed" and "|w| < 2.0".
    cases.append(dict(name="muon_step_property", kind="muon", shape=[2, 2],
                      theta0=[1.0, -1.0, 0.5, 0.5], grad=[0.1, 0.1, -0.1, -0.1], lr=0.1,
                      momentum=0.9, nesterov=True, ns_steps=5, steps=1, bound_abs=2.0,
                      ref="src/nn/optim/muon.rs:172-192"))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "volta_optimizer_kats.json")
    with open(path, "w") as fh:
        json.dump(cases, fh, indent=1)
    print("wrote", path, len(cases), "cases")


if __name__ == "__main__":
    main()
