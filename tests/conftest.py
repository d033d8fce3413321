import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")
REL_L2_TOL = 2.0 ** -8      # per-row relative L2 after bf16 rounding (the op's parity bar)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def lib():
    from mimfer_b200.build import build
    build()
    import mimfer_b200
    return mimfer_b200.lib()


@pytest.fixture(scope="session")
def oracle():
    from oracle.pyoracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle.pyoracle import Reference
    return Reference()


@pytest.fixture(scope="session")
def rt(lib):
    import mimfer_b200
    r = mimfer_b200.Runtime.get(0)
    for kv in os.environ.get("MIMFER_TUNE", "").split(","):      # e.g. MIMFER_TUNE=2=1 for experiments
        if "=" in kv:
            k, v = kv.split("=")
            r.lib.mm_f4_tune(int(k), int(v))
    return r


@pytest.fixture
def stream_kernel(rt):
    """Decode ops on the CUDA-core streaming kernel for the duration of a test (the
    block-scaled tensor kernel is the default)."""
    rt.lib.mm_f4_tune(5, 0)
    yield rt
    rt.lib.mm_f4_tune(5, 1)


def bf16_bits_to_f32(bits):
    return (np.ascontiguousarray(bits).astype(np.uint32) << 16).view(np.float32)


def row_rel_l2(y_bits, ref_bits):
    """max over rows of ||y - ref|| / ||ref||, on bf16-rounded outputs."""
    y = bf16_bits_to_f32(y_bits).astype(np.float64)
    r = bf16_bits_to_f32(ref_bits).astype(np.float64)
    num = np.sqrt(((y - r) ** 2).sum(axis=1))
    den = np.sqrt((r ** 2).sum(axis=1))
    den = np.where(den == 0, 1.0, den)
    return float((num / den).max())


def fnv1a64(a):
    h = 1469598103934665603
    for b in np.ascontiguousarray(a).view(np.uint8).ravel().tolist():
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h
