"""The allocation-free matvec (elb_matvec_static): for hosts that cannot call cudaMalloc at the point where they need
the product — a thread that must not block on the driver's allocation lock, a process whose device memory is already
owned by a pool. Its working memory is a static device array, so this test checks, through the C ABI, that it gives
exactly what the ordinary entry point (elb_matvec_dev, per-weight allocated scratch) gives, twice in a row with
different inputs (the array keeps the previous call's contents), that repeated calls leave the device's free memory
unchanged (what the entry point is for), and that weights beyond the static limits are refused with a message naming
the limit. Collected last on purpose: it must pass after every other test and alone."""
import ctypes as C

import numpy as np
import pytest

from exactinfer_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def elb():
    import exactinfer_b200 as e
    ok, why = e.cuda_available()
    assert ok, f"CUDA path unavailable: {why}"
    return e


def both(elb, w, x):
    from exactinfer_b200 import capi
    dx = elb.DeviceBuffer.from_array(x)
    dy0, dy1 = elb.DeviceBuffer(w.rows * 4), elb.DeviceBuffer(w.rows * 4)
    capi.check(capi.lib().elb_matvec_dev(w._h, dx.ptr, dy0.ptr, 4))
    capi.check(capi.lib().elb_matvec_static(w._h, dx.ptr, dy1.ptr, 4))
    return dy0.to_array(np.float32, w.rows), dy1.to_array(np.float32, w.rows)


@pytest.mark.parametrize("t", (synth.Q4_K, synth.Q6_K, synth.Q8_0, synth.F16))
def test_static_matvec_equals_allocating_matvec_twice(elb, t):
    rng = np.random.default_rng(77 + t)
    rows, n = 1000, 2560
    w = elb.Weight(t, rows, n, synth.rand_weight(rng, t, rows, n))
    for scale in (1.0, 37.5):  # two calls in a row; the second finds the first one's data in the array
        x = (rng.normal(size=n) * scale).astype(np.float32)
        ref, got = both(elb, w, x)
        assert np.array_equal(ref.view(np.uint32), got.view(np.uint32))  # same kernels: bit-identical
    # and across weights of another shape sharing the array
    w2 = elb.Weight(t, 130, 1024, synth.rand_weight(rng, t, 130, 1024))
    ref, got = both(elb, w2, rng.normal(size=1024).astype(np.float32))
    assert np.array_equal(ref.view(np.uint32), got.view(np.uint32))


def test_static_matvec_refuses_oversize(elb):
    from exactinfer_b200 import capi
    rng = np.random.default_rng(5)
    n = 16384 + 256
    w = elb.Weight(synth.Q8_0, 16, n, synth.rand_weight(rng, synth.Q8_0, 16, n))
    dx, dy = elb.DeviceBuffer(n * 4), elb.DeviceBuffer(16 * 4)
    rc = capi.lib().elb_matvec_static(w._h, dx.ptr, dy.ptr, 4)
    assert rc == capi.ERR_UNSUPPORTED
    assert b"16384" in capi.lib().elb_last_error()
    w.close()
    # too many rows: 262144 is the limit
    rows = 262144 + 16
    w = elb.Weight(synth.Q8_0, rows, 128, synth.rand_weight(rng, synth.Q8_0, rows, 128))
    dx, dy = elb.DeviceBuffer(128 * 4), elb.DeviceBuffer(rows * 4)
    rc = capi.lib().elb_matvec_static(w._h, dx.ptr, dy.ptr, 4)
    assert rc == capi.ERR_UNSUPPORTED
    assert b"262144" in capi.lib().elb_last_error()
    w.close()


def free_bytes():
    from exactinfer_b200 import capi
    f, t = C.c_size_t(), C.c_size_t()
    capi.check(capi.lib().elb_device_mem_info(0, C.byref(f), C.byref(t)))
    return f.value


@pytest.mark.parametrize("t", (synth.Q4_K, synth.F16))
def test_static_matvec_allocates_nothing(elb, t):
    """After the first call (which looks up the array's address), repeated calls must leave the amount of free device
    memory exactly as they found it: no cudaMalloc / cudaFree hides in the path."""
    from exactinfer_b200 import capi
    rng = np.random.default_rng(9)
    rows, n = 512, 1024
    w = elb.Weight(t, rows, n, synth.rand_weight(rng, t, rows, n))
    dx = elb.DeviceBuffer.from_array(rng.normal(size=n).astype(np.float32))
    dy = elb.DeviceBuffer(rows * 4)
    capi.check(capi.lib().elb_matvec_static(w._h, dx.ptr, dy.ptr, 4))  # first call on the device
    before = free_bytes()
    for _ in range(50):
        capi.check(capi.lib().elb_matvec_static(w._h, dx.ptr, dy.ptr, 4))
        assert free_bytes() == before
    w.close()
