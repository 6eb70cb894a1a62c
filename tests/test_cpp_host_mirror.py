"""The C++ host mirror (include/volta_b200.hpp: volta::nn::{Adam, SGD, Muon} over the C ABI)
replaying the reference's own optimizer tests (tests/cpp/test_optimizers.cpp)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "test_optimizers.bin")


def test_cpp_test_binary_is_built():
    """CPU check: the binary exists (built by build()) and links against the library."""
    assert os.path.exists(BIN), "run `python volta_b200/build.py` (or __graft_entry__.build())"
    out = subprocess.run(["ldd", BIN], capture_output=True, text=True).stdout
    assert "libvolta_b200.so" in out and "not found" not in out.split("libvolta_b200.so")[1].splitlines()[0]


@pytest.mark.gpu
def test_reference_tests_pass_through_cpp_mirror():
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    print(r.stdout[-2000:])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-500:]
    assert "0 failure(s)" in r.stdout and r.stdout.count(" ... ok") == 11
