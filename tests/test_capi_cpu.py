"""CPU-side checks of the C ABI: libelb.so builds, loads, exports every function include/elb.h declares, and refuses
compute loudly (no CPU fallback) when no CUDA device is present."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from exactinfer_b200 import build, capi
    build.build()
    return capi.lib()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "elb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(elb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_functions()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/elb.h but not exported"


def test_binding_covers_header():
    from exactinfer_b200 import capi
    assert sorted(capi.SIGNATURES) == declared_functions()


def test_no_cpu_fallback_without_device(lib):
    import exactinfer_b200 as e
    ok, why = e.cuda_available()
    if ok:
        pytest.skip("a CUDA device is present")
    assert why
    with pytest.raises(e.ElbError):
        e.Weight(12, 16, 256, np.zeros((16, 144), np.uint8))
    with pytest.raises(e.ElbError):
        e.rmsnorm(np.ones(8, np.float32), np.ones(8, np.float32), 1e-6)
    cfg = e.Config(1, 256, 256, 2, 1, 128, 64, 128, 1e6, 1e-6, 0)
    h = C.c_void_p()
    assert lib.elb_model_create(C.byref(cfg), 8, 0, C.byref(h)) == 1  # ELB_ERR_CUDA
    assert b"CUDA" in lib.elb_last_error()


def test_status_to_exception_mapping(lib):
    from exactinfer_b200 import capi
    for rc, exc in ((capi.ERR_INVALID, ValueError), (capi.ERR_RANGE, IndexError), (capi.ERR_MEMORY, MemoryError),
                    (capi.ERR_CUDA, capi.ElbError), (capi.ERR_UNSUPPORTED, capi.ElbError)):
        with pytest.raises(exc):
            capi.check(rc)
    capi.check(capi.OK)


def test_lcg_tokens_match_reference_stream():
    from exactinfer_b200 import synth
    s, want = 12345, []
    for _ in range(5):
        s = (s * 1664525 + 1013904223) % 2 ** 32
        want.append((s >> 8) % 150000)
    assert list(synth.lcg_tokens(5, 151936)) == want
    assert synth.lcg_tokens(100, 640).max() < 640
