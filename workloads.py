"""The benchmark configurations as tensor lists plus seeded synthetic data.

No dataset is involved in the optimizer path: a configuration is a list of parameter
shapes, an initialisation law and a gradient distribution.  The same generator feeds the
CPU oracle and the GPU engine, so both see bit-identical inputs.  Seeds: parameters 1234,
gradients of step s 5678 + s.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import numpy as np

PARAM_SEED = 1234
GRAD_SEED = 5678


@dataclass
class Workload:
    name: str
    optimizer: str                       # "adam" | "sgd" | "muon"
    shapes: List[Tuple[int, ...]]
    init: List[Tuple[str, float]]        # per tensor: ("uniform", bound) | ("normal", std) | ("const", value)
    grad_std: float
    hyper: Dict[str, object]
    steps: int
    notes: str = ""
    sizes: List[int] = field(init=False)

    def __post_init__(self):
        self.sizes = [int(np.prod(s, dtype=np.int64)) for s in self.shapes]

    @property
    def total(self) -> int:
        return int(sum(self.sizes))

    def make_params(self, seed: int = PARAM_SEED) -> List[np.ndarray]:
        rng = np.random.default_rng(seed)
        out = []
        for shape, (law, a) in zip(self.shapes, self.init):
            n = int(np.prod(shape, dtype=np.int64))
            if law == "uniform":
                x = rng.random(n, dtype=np.float32)
                x = (x * np.float32(2.0 * a) - np.float32(a)).astype(np.float32)
            elif law == "normal":
                x = rng.standard_normal(n, dtype=np.float32) * np.float32(a)
            else:
                x = np.full(n, a, np.float32)
            out.append(np.ascontiguousarray(x, np.float32).reshape(shape))
        return out

    def make_grads(self, step: int, seed: int = GRAD_SEED) -> List[np.ndarray]:
        rng = np.random.default_rng(seed + step)
        return [np.ascontiguousarray(
            rng.standard_normal(int(np.prod(s, dtype=np.int64)), dtype=np.float32) * np.float32(self.grad_std),
            np.float32).reshape(s) for s in self.shapes]


def c1_mlp_adam() -> Workload:
    """Adam on MLP 784->256->128->10: weights [in, out] Kaiming-uniform, biases 0."""
    shapes, init = [], []
    for fin, fout in ((784, 256), (256, 128), (128, 10)):
        shapes += [(fin, fout), (fout,)]
        init += [("uniform", math.sqrt(6.0 / fin)), ("const", 0.0)]
    return Workload("c1_mlp_adam", "adam", shapes, init, 1e-2,
                    dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0), 100)


def c2_cnn_sgd() -> Workload:
    """SGD momentum 0.9, wd 5e-4 on the MNIST CNN parameter set (weights He-normal)."""
    shapes = [(32, 1, 3, 3), (32,), (64, 32, 3, 3), (64,), (9216, 128), (128,), (128, 10), (10,)]
    fan_in = [9, None, 288, None, 9216, None, 128, None]
    init = [("normal", math.sqrt(2.0 / f)) if f else ("const", 0.0) for f in fan_in]
    return Workload("c2_cnn_sgd", "sgd", shapes, init, 1e-3,
                    dict(lr=0.01, momentum=0.9, weight_decay=5e-4), 200)


def c3_transformer_adam(layers: int = 12, d: int = 768, ffn: int = 3072, vocab: int = 32000) -> Workload:
    """Adam wd 0.01 on a 12-layer d=768 transformer parameter set (109 602 816 params):
    embedding, per layer q/k/v (no bias), out (+bias), FFN up/down (+bias), two LayerNorms."""
    shapes: List[Tuple[int, ...]] = [(vocab, d)]
    init: List[Tuple[str, float]] = [("normal", 0.02)]
    for _ in range(layers):
        for shp, ini in (((d, d), ("normal", 0.02)), ((d, d), ("normal", 0.02)), ((d, d), ("normal", 0.02)),
                         ((d, d), ("normal", 0.02)), ((d,), ("const", 0.0)),
                         ((d, ffn), ("normal", 0.02)), ((ffn,), ("const", 0.0)),
                         ((ffn, d), ("normal", 0.02)), ((d,), ("const", 0.0)),
                         ((d,), ("const", 1.0)), ((d,), ("const", 0.0)),
                         ((d,), ("const", 1.0)), ((d,), ("const", 0.0))):
            shapes.append(shp)
            init.append(ini)
    return Workload("c3_transformer_adam", "adam", shapes, init, 1e-3,
                    dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01), 50)


def c4_muon(layers: int = 24, d: int = 1024) -> Workload:
    """Muon on the 2-D matrices of a 24-layer d=1024 transformer: qkv 3d x d, o d x d,
    ffn 4d x d and d x 4d.  Hyper-parameters of the reference's only instantiation
    (src/nn/optim/muon.rs:179): lr 0.1, momentum 0.9, nesterov, 5 Newton-Schulz steps."""
    shapes, init = [], []
    for _ in range(layers):
        for shp in ((3 * d, d), (d, d), (4 * d, d), (d, 4 * d)):
            shapes.append(shp)
            init.append(("normal", 0.02))
    return Workload("c4_muon", "muon", shapes, init, 1e-3,
                    dict(lr=0.1, momentum=0.9, nesterov=True, ns_steps=5), 20)


def c5_ragged_adam(n_tensors: int = 4096, max_log2: int = 22, seed: int = 4096) -> Workload:
    """Ragged multi-tensor Adam: sizes floor(2^(22 U)), U ~ U[0,1), clamped to [1, 2^22]."""
    rng = np.random.default_rng(seed)
    u = rng.random(n_tensors)
    sizes = np.clip(np.floor(np.exp2(max_log2 * u)), 1, 2 ** max_log2).astype(np.int64)
    shapes = [(int(s),) for s in sizes]
    init = [("normal", 1.0)] * n_tensors
    return Workload("c5_ragged_adam", "adam", shapes, init, 1e-3,
                    dict(lr=3e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1), 10)


ALL = {"c1": c1_mlp_adam, "c2": c2_cnn_sgd, "c3": c3_transformer_adam, "c4": c4_muon, "c5": c5_ragged_adam}
