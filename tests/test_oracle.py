"""Pins the CPU oracle (oracle/oracle.c): against golden vectors made by the reference's own CPU code, against the
reference library itself when it is present, and against the `gguf` package's independent decoders (the check the
reference's tests/parity_dequant.py makes)."""
import hashlib
import os

import numpy as np
import pytest

import oracle_lib as ol
from exactinfer_b200 import synth

TYPES = (synth.Q8_0, synth.Q4_K, synth.Q6_K, synth.F16, synth.F32)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.fixture(scope="module")
def ops(golden_dir):
    return np.load(os.path.join(golden_dir, "ops.npz"))


@pytest.mark.parametrize("t", TYPES)
def test_decode_and_matvec_match_golden(ops, t):
    name = synth.TYPE_NAMES[t]
    w, x = ops[f"{name}_w"], ops[f"{name}_x"]
    rows, n = w.shape[0], x.size
    assert np.array_equal(bits(ol.dequant_rows(t, rows, n, w)), bits(ops[f"{name}_deq"]))
    assert np.array_equal(bits(ol.matvec(t, rows, n, w, x)), bits(ops[f"{name}_y"]))


def test_f16_corner_values(ops):
    h = ops["f16_bits"]
    got = np.array([ol.oracle().orc_f16_to_f32(int(v)) for v in h], dtype=np.float32)
    assert np.array_equal(bits(got), bits(ops["f16_vals"]))
    assert np.array_equal(bits(got), bits(h.view(np.float16).astype(np.float32)))


@pytest.mark.parametrize("n", (128, 1000))
def test_rmsnorm_matches_golden(ops, n):
    got = ol.rmsnorm(ops[f"rms{n}_x"], ops[f"rms{n}_w"], 1e-6)
    assert np.array_equal(bits(got), bits(ops[f"rms{n}_y"]))


@pytest.mark.parametrize("t", (synth.Q8_0, synth.Q4_K, synth.Q6_K))
def test_decoders_match_gguf_package(t):
    gguf = pytest.importorskip("gguf")
    qt = {synth.Q8_0: gguf.GGMLQuantizationType.Q8_0, synth.Q4_K: gguf.GGMLQuantizationType.Q4_K,
          synth.Q6_K: gguf.GGMLQuantizationType.Q6_K}[t]
    rng = np.random.default_rng(5)
    rows, n = 16, 1024
    w = synth.rand_weight(rng, t, rows, n)
    want = gguf.quants.dequantize(w, qt).astype(np.float32).reshape(rows, n)
    assert np.array_equal(bits(ol.dequant_rows(t, rows, n, w)), bits(want))


def test_q4k_scale_min_all_bytes():
    import ctypes as C
    rng = np.random.default_rng(9)
    for _ in range(200):
        q = rng.integers(0, 256, size=12, dtype=np.uint8)
        for j in range(8):
            sc, m = C.c_int(), C.c_int()
            ol.oracle().orc_q4k_scale_min(j, q.ctypes.data_as(C.POINTER(C.c_uint8)), C.byref(sc), C.byref(m))
            if j < 4:
                want = (q[j] & 63, q[j + 4] & 63)
            else:
                want = ((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4), (q[j + 4] >> 4) | ((q[j] >> 6) << 4))
            assert (sc.value, m.value) == (int(want[0]), int(want[1]))
            assert 0 <= sc.value < 64 and 0 <= m.value < 64


def _digest(tensors):
    h = hashlib.sha256()
    for role, layer, t, rows, n, data in tensors:
        h.update(f"{role}:{layer}:{t}:{rows}:{n}".encode())
        h.update(np.ascontiguousarray(data).tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("layout", ("f16", "q8_0", "q4_k_m"))
def test_tiny_model_logits_match_golden(golden_dir, layout):
    g = np.load(os.path.join(golden_dir, "tiny_model.npz"))
    spec = synth.Spec(name="tiny", n_layer=2, n_embd=256, n_ff=512, n_head=4, n_head_kv=2, n_vocab=640,
                      layout=layout, head_sigma=2e-5)
    tens = list(synth.generate(spec, seed=11))
    assert _digest(tens) == bytes(g[f"{layout}_sha"]).decode(), "synthetic weight generator drifted"
    toks = g["tokens"]
    assert np.array_equal(toks, synth.lcg_tokens(12, spec.n_vocab))
    m = ol.OracleModel(spec, tens, 32)
    outs = [m.eval(toks[:8], 0)]
    for i in range(8, 12):
        outs.append(m.eval(toks[i:i + 1], i))
    assert np.array_equal(bits(np.stack(outs)), bits(g[f"{layout}_logits"]))


def test_eval_rejects_bad_token_and_position():
    spec = synth.Spec(name="tiny", n_layer=1, n_embd=256, n_ff=256, n_head=2, n_head_kv=1, n_vocab=64, layout="q8_0")
    m = ol.OracleModel(spec, list(synth.generate(spec, 3)), 4)
    with pytest.raises(IndexError):
        m.eval([64], 0)
    with pytest.raises(IndexError):
        m.eval([1], 4)


@pytest.mark.skipif(not ol.have_ref(), reason="reference library not built (oracle/_ref)")
@pytest.mark.parametrize("t", TYPES)
def test_against_reference_library(t):
    rng = np.random.default_rng(100 + t)
    rows = 19
    n = 768 if t in (synth.Q4_K, synth.Q6_K) else 417 if t in (synth.F16, synth.F32) else 416
    w = synth.rand_weight(rng, t, rows, n)
    x = rng.normal(size=n).astype(np.float32)
    assert np.array_equal(bits(ol.dequant_rows(t, rows, n, w)), bits(ol.dequant_rows(t, rows, n, w, lib="ref")))
    assert np.array_equal(bits(ol.matvec(t, rows, n, w, x)), bits(ol.matvec(t, rows, n, w, x, lib="ref")))


# ---------------------------------------------------------------- limbs (integer restatement; properties)

@pytest.mark.parametrize("nl", (2, 3, 4))
def test_limb_split_reconstructs_rounded_fixed_point(nl):
    rng = np.random.default_rng(nl)
    for scale in (1.0, 1e-20, 3e7, 2.0 ** -100):
        x = (rng.normal(size=777) * scale).astype(np.float32)
        x[5] = 0.0
        limbs, inv, k = ol.split_limbs(x, nl)
        m = np.abs(x).max()
        e = int(np.frexp(m)[1])
        assert k == 8 * nl - 2 - e and inv == np.float32(2.0 ** -k)
        X = np.rint(np.ldexp(x.astype(np.float64), k)).astype(np.int64)
        rec = sum(limbs[l].astype(np.int64) << (8 * l) for l in range(nl))
        assert np.array_equal(rec, X)
        assert np.abs(X).max() < 2 ** (8 * nl - 2) + 1 and np.abs(X).max() >= 2 ** (8 * nl - 3)
        assert np.abs(limbs[nl - 1].astype(int)).max() <= 65
    limbs, inv, k = ol.split_limbs(np.zeros(64, np.float32), nl)
    assert k == 0 and inv == 1.0 and not limbs.any()


def test_limb_split_ties_to_even():
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, 32.0], dtype=np.float32)  # max 32 = 0.5*2^6 -> k = 8*2-2-6 = 8
    limbs, inv, k = ol.split_limbs(x * 2.0 ** -8, 2)
    assert k == 16 - 2 - (6 - 8)
    rec = limbs[0].astype(int) + 256 * limbs[1].astype(int)
    assert list(rec) == [int(np.rint(v * 2.0 ** (k - 8))) for v in x]


@pytest.mark.parametrize("t", (synth.Q8_0, synth.Q4_K, synth.Q6_K))
def test_limb_sums_agree_with_decoded_weights(t):
    """sum over sub-blocks of scale*P (and the min term) must reproduce the dot product of the fixed-point
    activation with the decoded weights, computed independently in float64."""
    rng = np.random.default_rng(40 + t)
    rows, n, nl = 5, 512, 4
    w = synth.rand_weight(rng, t, rows, n)
    x = rng.normal(size=n).astype(np.float32)
    limbs, inv, k = ol.split_limbs(x, nl)
    X = sum(limbs[l].astype(np.int64) << (8 * l) for l in range(nl))
    P = ol.limb_partials(t, rows, n, w, limbs)
    I, J = ol.limb_block_sums(t, rows, n, w, limbs)
    deq = ol.dequant_rows(t, rows, n, w).astype(np.float64)
    want = deq @ X.astype(np.float64)
    wb = w.reshape(rows, -1)
    for r in range(rows):
        if t == synth.Q8_0:
            d = wb[r].reshape(-1, 34)[:, :2].copy().view(np.float16).astype(np.float64)[:, 0]
            got = sum(d * (I[r, :, l].astype(np.float64) * 256.0 ** l) for l in range(nl)).sum()
            assert np.array_equal(I[r], P[r])
        elif t == synth.Q4_K:
            blk = wb[r].reshape(-1, 144)
            d = blk[:, 0:2].copy().view(np.float16).astype(np.float64)[:, 0]
            dmin = blk[:, 2:4].copy().view(np.float16).astype(np.float64)[:, 0]
            got = sum((d * I[r, :, l] - dmin * J[r, :, l]) * 256.0 ** l for l in range(nl)).sum()
        else:
            d = wb[r].reshape(-1, 210)[:, 208:210].copy().view(np.float16).astype(np.float64)[:, 0]
            got = sum(d * I[r, :, l] * 256.0 ** l for l in range(nl)).sum()
        assert abs(got - want[r]) <= 1e-9 * max(1.0, abs(want[r]))
