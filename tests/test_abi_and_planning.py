"""CPU-only checks of the C-ABI library: it loads, exports every symbol the header
declares, validates arguments, and plans arena layouts / rank slices / chunk tables that
cover every element exactly once.  No CUDA call is made here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "volta_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from volta_b200 import _lib
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 40
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/volta_b200.h but not exported"
    bound = set(_lib.SIGNATURES) | set(_lib.OTHER_SYMBOLS)
    assert set(names) == bound, set(names) ^ bound
    assert lib.vb_abi_version() == 1002


def test_python_constants_match_the_header():
    """Flags, modes and sizes are written twice (header and ctypes module): they must agree."""
    from volta_b200 import _lib
    text = open(HEADER).read()
    defines = {k: int(v.rstrip("u"), 0) for k, v in re.findall(r"#define\s+(VB_[A-Z0-9_]+)\s+(\d+u?)\b", text)}
    for name in ("VB_STEP_DEFAULT", "VB_STEP_NO_EXCHANGE", "VB_STEP_EXCHANGE_BF16", "VB_STEP_REDUCE_GRADS",
                 "VB_STEP_MEAN_GRADS"):
        assert defines[name] == getattr(_lib, name), name
    assert defines["VB_IPC_HANDLE_BYTES"] == 64
    enums = dict(re.findall(r"\b(VB_NS_[A-Z0-9_]+)\s*=\s*(\d+)", text))
    for name in ("VB_NS_F32", "VB_NS_BF16", "VB_NS_F32_TC"):
        assert int(enums[name]) == getattr(_lib, name), name
    flags = [defines[n] for n in defines if n.startswith("VB_STEP_") and defines[n]]
    assert len(set(flags)) == len(flags) and all(f & (f - 1) == 0 for f in flags)   # distinct single bits


def test_step_params_mirror_layout():
    """32-byte, same field order as Volta's OptimizerStepParams (src/gpu/kernels.rs:42-54)."""
    from volta_b200._lib import StepParams
    assert C.sizeof(StepParams) == 32
    assert [f[0] for f in StepParams._fields_] == ["op", "lr", "beta1", "beta2", "t", "eps",
                                                   "weight_decay", "padding"]


def test_null_and_invalid_arguments_return_codes_not_crashes():
    from volta_b200 import _lib
    lib = _lib.load()
    assert lib.vb_engine_synchronize(None) == 1
    assert b"null" in lib.vb_last_error()
    assert lib.vb_optimizer_step(None) == 1
    assert lib.vb_optimizer_zero_grad(None) == 1
    assert lib.vb_engine_destroy(None) == 0 and lib.vb_optimizer_destroy(None) == 0
    out = C.c_void_p()
    assert lib.vb_adam_create(None, 0, None, 1e-3, 0.9, 0.999, 1e-8, 0.0, C.byref(out)) == 1
    sizes = (C.c_int64 * 1)(-5)
    n = C.c_int64()
    assert lib.vb_plan_layout(1, sizes, 1, 0, 148, None, None, None, None, C.byref(n), 0, None, None, None) == 1
    assert lib.vb_plan_layout(1, sizes, 2, 2, 148, None, None, None, None, C.byref(n), 0, None, None, None) == 1


def plan(sizes, world, rank, sm=148):
    from volta_b200 import _lib
    n = len(sizes)
    arr = (C.c_int64 * max(n, 1))(*sizes)
    offs = (C.c_int64 * max(n, 1))()
    arena, lo, hi, nch = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64()
    _lib.call("vb_plan_layout", n, arr, world, rank, sm, offs, C.byref(arena), C.byref(lo), C.byref(hi),
              C.byref(nch), 0, None, None, None)
    k = nch.value
    ct, co, cl = (C.c_int64 * max(k, 1))(), (C.c_int64 * max(k, 1))(), (C.c_int64 * max(k, 1))()
    _lib.call("vb_plan_layout", n, arr, world, rank, sm, offs, C.byref(arena), C.byref(lo), C.byref(hi),
              C.byref(nch), k, ct, co, cl)
    return dict(offsets=[offs[i] for i in range(n)], arena=arena.value, lo=lo.value, hi=hi.value,
                chunks=[(ct[i], co[i], cl[i]) for i in range(k)])


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_plan_covers_every_element_exactly_once(world):
    rng = np.random.default_rng(world)
    sizes = [int(s) for s in np.floor(np.exp2(18 * rng.random(200))).astype(np.int64)] + [0, 1, 3, 31, 32, 33]
    total = sum(sizes)
    cover = None
    prev_hi = 0
    for rank in range(world):
        p = plan(sizes, world, rank)
        if cover is None:
            cover = np.zeros(p["arena"], np.int32)
            offsets = p["offsets"]
            for i, (o, s) in enumerate(zip(offsets, sizes)):
                assert o % 32 == 0  # 128-byte aligned tensor starts
                if i + 1 < len(sizes):
                    assert offsets[i + 1] >= o + s
        assert p["offsets"] == offsets
        assert p["lo"] == prev_hi and (p["hi"] - p["lo"]) * world == p["arena"] and p["lo"] % 256 == 0
        prev_hi = p["hi"]
        for t, off, ln in p["chunks"]:
            assert ln > 0 and off >= 0 and off + ln <= sizes[t]
            a = offsets[t] + off
            assert p["lo"] <= a and a + ln <= p["hi"]  # a rank only touches its own slice
            assert a % 4 == 0  # 16-byte aligned chunk starts -> vector path
            cover[a:a + ln] += 1
    assert prev_hi == cover.size
    assert cover.sum() == total and cover.max() == 1
    for o, s in zip(offsets, sizes):
        assert np.all(cover[o:o + s] == 1)


def plan_replicated(sizes, world, rank, fraction, sm=148):
    from volta_b200 import _lib
    n = len(sizes)
    arr = (C.c_int64 * max(n, 1))(*sizes)
    offs = (C.c_int64 * max(n, 1))()
    arena, lo, hi, tail, nch = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64()
    _lib.call("vb_plan_layout_replicated", n, arr, world, rank, sm, fraction, offs, C.byref(arena), C.byref(lo),
              C.byref(hi), C.byref(tail), C.byref(nch), 0, None, None, None, None)
    k = nch.value
    ct, co, cl = (C.c_int64 * max(k, 1))(), (C.c_int64 * max(k, 1))(), (C.c_int64 * max(k, 1))()
    local = (C.c_int32 * max(k, 1))()
    _lib.call("vb_plan_layout_replicated", n, arr, world, rank, sm, fraction, offs, C.byref(arena), C.byref(lo),
              C.byref(hi), C.byref(tail), C.byref(nch), k, ct, co, cl, local)
    return dict(offsets=[offs[i] for i in range(n)], arena=arena.value, lo=lo.value, hi=hi.value, tail=tail.value,
                chunks=[(ct[i], co[i], cl[i], local[i]) for i in range(k)])


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("fraction", [0.0, 0.2, 0.55, 1.0])
def test_plan_with_a_replicated_tail(world, fraction):
    """[0, tail) is cut into the ranks' slices, [tail, arena) belongs to every rank; a rank's chunks
    cover its slice and the tail exactly once, flagged by part and mixed in proportion."""
    rng = np.random.default_rng(world)
    sizes = [int(s) for s in np.floor(np.exp2(18 * rng.random(150))).astype(np.int64)] + [1 << 21, 0, 1, 33]
    plain = [plan(sizes, world, r) for r in range(world)]
    cover_slices = None
    prev_hi = 0
    for rank in range(world):
        p = plan_replicated(sizes, world, rank, fraction)
        if fraction == 0.0:
            assert p["tail"] == p["arena"] and (p["lo"], p["hi"]) == (plain[rank]["lo"], plain[rank]["hi"])
            assert [c[:3] for c in p["chunks"]] == plain[rank]["chunks"] and not any(c[3] for c in p["chunks"])
        if cover_slices is None:
            cover_slices = np.zeros(p["arena"], np.int32)
            tail = p["tail"]
            offsets = p["offsets"]
            assert tail % (256 * world) == 0 and 0 <= tail <= p["arena"]
            assert abs((p["arena"] - tail) - fraction * p["arena"]) <= 256 * world
        assert p["tail"] == tail and p["offsets"] == offsets
        assert p["lo"] == prev_hi and (p["hi"] - p["lo"]) * world == tail
        prev_hi = p["hi"]
        cover_tail = np.zeros(p["arena"], np.int32)
        for t, off, ln, local in p["chunks"]:
            assert ln > 0 and off + ln <= sizes[t]
            a = offsets[t] + off
            assert a % 4 == 0
            if local:
                assert tail <= a and a + ln <= p["arena"]
                cover_tail[a:a + ln] += 1
            else:
                assert p["lo"] <= a and a + ln <= p["hi"]
                cover_slices[a:a + ln] += 1
        for o, s in zip(offsets, sizes):  # every rank covers the whole tail once
            assert np.all(cover_tail[max(o, tail):max(o + s, tail)] == 1)
        assert cover_tail[:tail].sum() == 0
        flags = np.array([c[3] for c in p["chunks"]], np.int64)
        if 0 < flags.sum() < flags.size:  # the two kinds are spread evenly over the table
            share = flags.mean()
            running = np.cumsum(flags) - share * np.arange(1, flags.size + 1)
            assert np.abs(running).max() <= 2.0
    assert prev_hi == tail
    for o, s in zip(offsets, sizes):
        assert np.all(cover_slices[o:min(o + s, max(o, tail))] == 1)
    assert cover_slices[tail:].sum() == 0 and cover_slices.max() <= 1


def test_replicated_fraction_balances_hbm_and_link_time():
    from volta_b200 import plan_replicated_fraction
    assert plan_replicated_fraction(28, 1, 6700, 630) == 0.0
    for world in (2, 4, 8):
        f = plan_replicated_fraction(28, world, 6700, 630)
        assert 0.0 < f < 1.0
        hbm = 28 / 6700 * ((1 - f) / world + f)
        link = 4 * (world - 1) / world / 630 * (1 - f)
        assert abs(hbm - link) < 1e-9 * hbm + 1e-15
    # a link as fast as needed: nothing to replicate
    assert plan_replicated_fraction(28, 2, 1000, 1e6) == 0.0


def test_plan_chunk_lengths_scale_with_problem_size():
    small = plan([235146 // 6] * 6, 1, 0)
    big = plan([1 << 22] * 64, 1, 0)
    assert len(small["chunks"]) >= 100          # a 235k-parameter model still spreads over the SMs
    assert max(c[2] for c in big["chunks"]) <= 16384
    assert len(big["chunks"]) >= 148 * 64


def test_plan_empty_and_tiny():
    p = plan([], 1, 0)
    assert p["chunks"] == [] and p["arena"] >= 1
    p = plan([0, 0], 2, 1)
    assert p["chunks"] == []
    p = plan([1], 1, 0)
    assert p["chunks"] == [(0, 0, 1)]
