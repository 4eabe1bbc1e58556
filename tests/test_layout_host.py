"""The tiled weight layouts are pure permutations: building a tile on the CPU with the index functions the kernels
use and decoding it back must reproduce the oracle's decoded rows bit for bit (no GPU needed)."""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest

import oracle_lib as ol
from exactinfer_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def helper(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    so = str(tmp_path_factory.mktemp("layout") / "liblayout_host.so")
    subprocess.run([nvcc, "-O1", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-o", so,
                    os.path.join(ROOT, "tests", "layout_host.cu")], check=True, capture_output=True)
    L = C.CDLL(so)
    L.layout_roundtrip.argtypes = [C.c_int, C.c_longlong, C.c_longlong, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    return L


@pytest.mark.parametrize("t", (synth.Q4_K, synth.Q6_K, synth.Q8_0))
@pytest.mark.parametrize("rows", (16, 37))
def test_roundtrip_matches_oracle(helper, t, rows):
    rng = np.random.default_rng(rows + t)
    n = 512
    w = synth.rand_weight(rng, t, rows, n)
    want = ol.dequant_rows(t, rows, n, w)
    rows16 = (rows + 15) // 16 * 16
    out = np.empty((rows16, n), dtype=np.float32)
    assert helper.layout_roundtrip(t, rows, n, w.ctypes.data, 0, out.ctypes.data, None) == 0
    assert np.array_equal(out[:rows].view(np.uint32), want.view(np.uint32))
    assert not out[rows:].any()  # padding rows decode to zero


@pytest.mark.parametrize("t", (synth.Q4_K, synth.Q6_K, synth.Q8_0))
def test_paired_layout_interleaves_gate_and_up(helper, t):
    rng = np.random.default_rng(t)
    half, n = 24, 256
    gate, up = synth.rand_weight(rng, t, half, n), synth.rand_weight(rng, t, half, n)
    both = np.concatenate([gate, up])
    out = np.empty((48, n), dtype=np.float32)
    assert helper.layout_roundtrip(t, 2 * half, n, both.ctypes.data, 1, out.ctypes.data, None) == 0
    dg, du = ol.dequant_rows(t, half, n, gate), ol.dequant_rows(t, half, n, up)
    for T in range(3):
        assert np.array_equal(out[16 * T:16 * T + 8].view(np.uint32), dg[8 * T:8 * T + 8].view(np.uint32))
        assert np.array_equal(out[16 * T + 8:16 * T + 16].view(np.uint32), du[8 * T:8 * T + 8].view(np.uint32))
