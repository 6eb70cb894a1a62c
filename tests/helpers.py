"""Shared helpers of the parity tests."""
import numpy as np

TINY = np.float32(1e-30)


def max_rel_err(actual: np.ndarray, expected: np.ndarray) -> float:
    """max |a - e| / max(|e|, tiny) over all elements (the Adam/SGD parity measure)."""
    a = np.asarray(actual, np.float64).reshape(-1)
    e = np.asarray(expected, np.float64).reshape(-1)
    if a.size == 0:
        return 0.0
    return float(np.max(np.abs(a - e) / np.maximum(np.abs(e), float(TINY))))


def rel_frobenius(actual: np.ndarray, expected: np.ndarray) -> float:
    a = np.asarray(actual, np.float64)
    e = np.asarray(expected, np.float64)
    return float(np.linalg.norm(a - e) / max(np.linalg.norm(e), 1e-300))


def bits_equal(a: np.ndarray, b: np.ndarray) -> bool:
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32).reshape(-1),
                          np.asarray(b, np.float32).view(np.uint32).reshape(-1))
