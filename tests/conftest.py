import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def refcpu():
    """The reference's own qwasar_cpu.c (bf16 cache build), when oracle/_ref holds it."""
    from oracle.oracle import RefCpu
    if not RefCpu.available("bf16"):
        pytest.skip("oracle/_ref not built (needs the reference checkout at build time)")
    return RefCpu("bf16")


@pytest.fixture(scope="session")
def be():
    """The initialised CUDA backend.  Fails (does not skip) when the library or the
    device is missing: GPU tests must never pass on a fallback."""
    import qwasar_b200
    return qwasar_b200.Backend()


def xorshift_fill(n, seed):
    """The generator the reference's tests fill their inputs with
    (tests/test_attn.c:27-33): xorshift32, top 24 bits mapped to [-1, 1)."""
    out = np.empty(n, np.float32)
    s = np.uint32(seed | 1)
    with np.errstate(over="ignore"):
        for i in range(n):
            s ^= np.uint32(s << np.uint32(13))
            s ^= np.uint32(s >> np.uint32(17))
            s ^= np.uint32(s << np.uint32(5))
            out[i] = np.float32((np.int64(s >> np.uint32(8)) - 8388608) / 8388608.0)
    return out


def rel_l2(a, b):
    """The reference tests' error measure (tests/test_attn.c:35-43)."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    den = float(np.sum(b * b))
    num = float(np.sum((a - b) ** 2))
    return (num / den) ** 0.5 if den > 0 else num ** 0.5


def max_rel_err(got, want):
    """Max relative error per output vector: max_i |got_i - want_i| / max_i |want_i|,
    maximised over the (row, head) vectors (last axis = head_dim).  An element-wise
    ratio on a softmax average of zero-mean values would measure the cancellation
    in the reference value, not the kernel (the reference's tests make the same
    point, tests/test_ops.c:31-33)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    num = np.max(np.abs(got - want), axis=-1)
    den = np.maximum(np.max(np.abs(want), axis=-1), 1e-30)
    return float(np.max(num / den))
