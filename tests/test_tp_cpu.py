"""Tensor-parallel host logic on CPU: two gloo ranks cut one layer with the library's shard functions (host arithmetic
of libelb.so, no GPU), run their shares through the oracle and exchange over gloo (tp_cpu_worker.py)."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

import exactinfer_b200 as e
from exactinfer_b200 import synth

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gloo_ranks_match_whole_tensors():
    port = free_port()
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_cpu_worker.py"), str(r), "2", str(port)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{out[-3000:]}"
        assert f"rank {r}: ok" in out


@pytest.mark.parametrize("name,size", [("qwen3-4b-q4_k_m", 2), ("qwen3-4b-q4_k_m", 4), ("qwen3-4b-q4_k_m", 8),
                                       ("qwen3-32b-q4_k_m", 8), ("qwen3-0.6b-f16", 8), ("qwen3-1.7b-q8_0", 4)])
def test_dims_tile_the_model(name, size):
    spec = synth.SPECS[name]
    dims = [e.tp_dims(spec, r, size) for r in range(size)]
    assert sum(d["n_head"] for d in dims) == spec.n_head and sum(d["n_head_kv"] for d in dims) == spec.n_head_kv
    assert dims[0]["f0"] == 0 and dims[-1]["f1"] == spec.n_ff
    assert dims[0]["v0"] == 0 and dims[-1]["v1"] == spec.n_vocab
    for a, b in zip(dims, dims[1:]):
        assert a["f1"] == b["f0"] and a["v1"] == b["v0"]
    assert all((d["f1"] - d["f0"]) % 256 == 0 and d["f1"] > d["f0"] and d["v0"] % 16 == 0 for d in dims)


def test_rejects_cuts_that_split_a_head_or_a_block():
    spec = synth.SPECS["qwen3-4b-q4_k_m"]
    with pytest.raises(Exception, match="divide"):
        e.tp_dims(spec, 0, 3)
    with pytest.raises(ValueError):
        e.tp_dims(spec, 2, 2)
    odd = synth.Spec("odd", n_layer=1, n_embd=256, n_ff=256, n_head=2, n_head_kv=2, n_vocab=64, layout="q4_k")
    with pytest.raises(Exception, match="256"):
        e.tp_dims(odd, 0, 2)  # one query head per rank: its 128 columns of attn_output are half a Q4_K block


def test_column_cut_copies_whole_blocks():
    spec = synth.Spec("cut", n_layer=1, n_embd=256, n_ff=512, n_head=4, n_head_kv=2, n_vocab=64, layout="q4_k")
    rng = np.random.default_rng(3)
    w = synth.rand_q4_k(rng, 256, 512)  # ffn_down: E x F
    raw = np.ascontiguousarray(w).reshape(256, 2, 144)
    for r in range(2):
        rows, n, b = e.tp_shard(spec, r, 2, "ffn_down", synth.Q4_K, 256, 512, w)
        assert (rows, n) == (256, 256)
        assert np.array_equal(b.reshape(256, 144), raw[:, r, :])


@pytest.mark.parametrize("layout,t", [("f16", synth.F16), ("q8_0", synth.Q8_0), ("q6_k", synth.Q6_K)])
def test_cuts_reassemble_the_tensor(layout, t):
    """Row cuts concatenated, and column cuts interleaved row by row, give back the whole tensor for every type."""
    spec = synth.Spec("cut", n_layer=1, n_embd=256, n_ff=768, n_head=4, n_head_kv=2, n_vocab=100, layout=layout)
    rng = np.random.default_rng(11)
    F, E = spec.n_ff, spec.n_embd
    gate = synth.rand_weight(rng, t, F, E)   # row cut
    down = synth.rand_weight(rng, t, E, F)   # column cut
    gate_b = np.ascontiguousarray(gate).reshape(F, -1)
    down_b = np.ascontiguousarray(down).reshape(E, -1)
    rows, cols = [], []
    for r in range(2):
        n_r, n_c, b = e.tp_shard(spec, r, 2, "ffn_gate", t, F, E, gate)
        assert n_c == E
        rows.append(b.reshape(n_r, -1))
        n_r, n_c, b = e.tp_shard(spec, r, 2, "ffn_down", t, E, F, down)
        assert n_r == E
        cols.append(b.reshape(E, -1))
    assert np.array_equal(np.concatenate(rows, axis=0), gate_b)
    assert np.array_equal(np.concatenate(cols, axis=1), down_b)
    d0, d1 = e.tp_dims(spec, 0, 2), e.tp_dims(spec, 1, 2)
    assert (d0["f1"] - d0["f0"], d1["f1"] - d1["f0"]) == (256, 512)  # three 256-blocks cut 1 + 2
