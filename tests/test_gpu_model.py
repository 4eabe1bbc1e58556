"""GPU parity of the whole forward pass (Backend.eval through the C ABI) against the CPU oracle's restated
CpuModel on the same seeded synthetic weights: prompt chunk, then single-token steps (the captured decode graph).

Bars (written here): max |delta logprob| <= 3e-5 over the generated tokens (double-precision log-softmax as in the
reference's generate command), logits and the residual stream within 2e-4 of the oracle relative to their largest
magnitude (errors of the order of fp32 rounding compound over the layers), and the golden logits of the reference's own
CPU build within the same bar.
"""
import os

import numpy as np
import pytest

import oracle_lib as ol
from exactinfer_b200 import synth

pytestmark = pytest.mark.gpu
LOGPROB_TOL = 3e-5
REL_TOL = 2e-4


@pytest.fixture(scope="module")
def elb():
    import exactinfer_b200 as e
    ok, why = e.cuda_available()
    assert ok, f"CUDA path unavailable: {why}"
    return e


def logprobs(logits):
    return logits.astype(np.float64) - ol.logsumexp(logits)


def rel(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(np.abs(b).max(), 1e-30))


def run_pair(elb, spec, seed, n_prompt, n_decode, max_batch=0):
    tens = list(synth.generate(spec, seed))
    n_ctx = n_prompt + n_decode + 1
    gpu = elb.Backend(spec, tens, n_ctx, max_batch=max_batch)
    cpu = ol.OracleModel(spec, tens, n_ctx)
    toks = synth.lcg_tokens(n_prompt, spec.n_vocab)
    lg, lc = gpu.eval(toks, 0), cpu.eval(toks, 0)
    worst_lp, worst_rel = 0.0, rel(lg, lc)
    assert rel(gpu.hidden(), cpu.hidden()) <= REL_TOL
    pos = n_prompt
    for _ in range(n_decode):
        nxt = int(np.argmax(lc))  # teacher-forced on the oracle's greedy token
        pg, pc = logprobs(lg), logprobs(lc)
        worst_lp = max(worst_lp, abs(pg[nxt] - pc[nxt]))
        top = np.argsort(lc)[-8:]
        worst_lp = max(worst_lp, float(np.abs(pg[top] - pc[top]).max()))
        lg, lc = gpu.eval([nxt], pos), cpu.eval([nxt], pos)
        worst_rel = max(worst_rel, rel(lg, lc))
        pos += 1
    gpu.close()
    cpu.close()
    return worst_lp, worst_rel


@pytest.mark.parametrize("layout", ("q4_k_m", "q8_0", "f16", "q6_k"))
def test_small_model_prefill_and_decode(elb, layout):
    spec = synth.Spec(name="small", n_layer=3, n_embd=512, n_ff=1024, n_head=8, n_head_kv=2, n_vocab=2048, layout=layout,
                      head_sigma=2e-5)
    lp, r = run_pair(elb, spec, seed=21, n_prompt=40, n_decode=6)
    assert lp <= LOGPROB_TOL, lp
    assert r <= REL_TOL, r


def test_chunked_prompt_equals_oracle(elb):
    """A prompt longer than the chunk length goes through several chunks (eval's internal chunking)."""
    spec = synth.Spec(name="small", n_layer=2, n_embd=256, n_ff=512, n_head=4, n_head_kv=2, n_vocab=640, layout="q4_k_m",
                      head_sigma=2e-5)
    lp, r = run_pair(elb, spec, seed=5, n_prompt=75, n_decode=3, max_batch=32)
    assert lp <= LOGPROB_TOL and r <= REL_TOL, (lp, r)


def test_wide_group_and_odd_shapes(elb):
    """8 query heads per KV head (the 32B grouping) and a vocabulary that is not a multiple of 16."""
    spec = synth.Spec(name="wide", n_layer=2, n_embd=1024, n_ff=768, n_head=8, n_head_kv=1, n_vocab=1003, layout="q4_k_m",
                      head_sigma=2e-5)
    lp, r = run_pair(elb, spec, seed=9, n_prompt=33, n_decode=4)
    assert lp <= LOGPROB_TOL and r <= REL_TOL, (lp, r)


@pytest.mark.parametrize("layout", ("f16", "q8_0", "q4_k_m"))
def test_golden_logits_of_reference_build(elb, golden_dir, layout):
    g = np.load(os.path.join(golden_dir, "tiny_model.npz"))
    spec = synth.Spec(name="tiny", n_layer=2, n_embd=256, n_ff=512, n_head=4, n_head_kv=2, n_vocab=640, layout=layout,
                      head_sigma=2e-5)
    m = elb.Backend(spec, list(synth.generate(spec, seed=11)), 32)
    toks = g["tokens"]
    outs = [m.eval(toks[:8], 0)]
    for i in range(8, 12):
        outs.append(m.eval(toks[i:i + 1], i))
    want = g[f"{layout}_logits"]
    for a, b in zip(outs, want):
        assert rel(a, b) <= REL_TOL
        assert np.abs(logprobs(a) - logprobs(b))[np.argsort(b)[-8:]].max() <= LOGPROB_TOL


def test_decode_only_from_position_zero_and_prefix_rewrite(elb):
    """Single-token evals from position 0, then re-evaluating a suffix (the serve loop's prefix reuse relies on eval
    touching only the KV rows it is given)."""
    spec = synth.Spec(name="small", n_layer=2, n_embd=256, n_ff=512, n_head=4, n_head_kv=2, n_vocab=640, layout="q8_0")
    tens = list(synth.generate(spec, 13))
    gpu, cpu = elb.Backend(spec, tens, 16), ol.OracleModel(spec, tens, 16)
    toks = synth.lcg_tokens(10, spec.n_vocab)
    for i in range(6):
        lg, lc = gpu.eval(toks[i:i + 1], i), cpu.eval(toks[i:i + 1], i)
        assert rel(lg, lc) <= REL_TOL
    # rewind to position 3 with other tokens: rows 3.. are overwritten, rows 0..2 are reused
    lg, lc = gpu.eval(toks[6:10], 3), cpu.eval(toks[6:10], 3)
    assert rel(lg, lc) <= REL_TOL
    assert gpu.eval(toks[:2], 7, want_logits=False) is None


def test_eval_argument_errors(elb):
    spec = synth.Spec(name="small", n_layer=1, n_embd=256, n_ff=256, n_head=2, n_head_kv=1, n_vocab=64, layout="q8_0")
    m = elb.Backend(spec, list(synth.generate(spec, 3)), 8)
    with pytest.raises(ValueError):
        m.eval(np.zeros(0, np.int32), 0)
    with pytest.raises(IndexError):
        m.eval([64], 0)
    with pytest.raises(IndexError):
        m.eval([-1], 0)
    with pytest.raises(IndexError):
        m.eval([1, 2, 3], 6)
    with pytest.raises(IndexError):
        m.eval([1], -1)
    assert m.eval([1, 2, 3], 5).shape == (64,)
    assert m.name() == "cuda-b200" and m.n_ctx() == 8 and m.cfg().n_vocab == 64


def test_benchmark_distribution_within_logit_resolution(elb):
    """With the benchmark's block-scale spread (1e-3 everywhere) logits reach 10^2..10^3, where one fp32 ulp is itself
    3e-5..6e-5: there the log-probability error is bounded by the resolution of the logits, 3e-5 + 2 ulp(max |logit|)."""
    spec = synth.Spec(name="small", n_layer=3, n_embd=512, n_ff=1024, n_head=8, n_head_kv=2, n_vocab=2048, layout="q4_k_m")
    tens = list(synth.generate(spec, 21))
    gpu, cpu = elb.Backend(spec, tens, 48), ol.OracleModel(spec, tens, 48)
    toks = synth.lcg_tokens(40, spec.n_vocab)
    lg, lc = gpu.eval(toks, 0), cpu.eval(toks, 0)
    tol = LOGPROB_TOL + 2 * float(np.spacing(np.float32(np.abs(lc).max())))
    top = np.argsort(lc)[-8:]
    assert np.abs(logprobs(lg) - logprobs(lc))[top].max() <= tol
    assert rel(lg, lc) <= REL_TOL


def test_ffn_activation_in_global_memory(elb, monkeypatch):
    """Shapes whose FFN activation does not fit in shared memory next to the weight rings keep its limbs in global
    memory (one more grid barrier per layer); forced here on a small model."""
    monkeypatch.setenv("ELB_DK_GACT", "1")
    spec = synth.Spec(name="small", n_layer=3, n_embd=512, n_ff=1536, n_head=8, n_head_kv=2, n_vocab=2048, layout="q4_k_m",
                      head_sigma=2e-5)
    lp, r = run_pair(elb, spec, seed=23, n_prompt=24, n_decode=6)
    assert lp <= LOGPROB_TOL and r <= REL_TOL, (lp, r)


def test_long_context(elb):
    """A prompt of several chunks deep into the context (the chunked prompt attention cuts the keys of a query tile into
    up to eight chunks) and a single-token step whose key splits take more than one pass over their keys. On this
    sequence the reference's fp32 CPU path is itself ~1.6e-5 (relative) away from a float64 evaluation, so the bars
    are taken against float64: the CUDA path may be at most as far from it as the CPU path (with a factor 1.5 of slack),
    or within the usual bars."""
    from f64_model import f64_logits
    spec = synth.Spec(name="long", n_layer=1, n_embd=256, n_ff=512, n_head=4, n_head_kv=2, n_vocab=300, layout="q4_k_m",
                      head_sigma=2e-5)
    tens = list(synth.generate(spec, 9))
    n = 2500
    toks = list(synth.lcg_tokens(n, spec.n_vocab))
    gpu = elb.Backend(spec, tens, n + 2)
    cpu = ol.OracleModel(spec, tens, n + 2)
    for step in range(2):  # the prompt, then one more token
        if step == 0:
            lg, lc = gpu.eval(toks, 0), cpu.eval(toks, 0)
        else:
            toks.append(int(np.argmax(lc)))
            lg, lc = gpu.eval(toks[-1:], n), cpu.eval(toks[-1:], n)
        exact = f64_logits(spec, tens, np.asarray(toks))
        lp_exact = exact - (np.log(np.sum(np.exp(exact - exact.max()))) + exact.max())
        top = np.argsort(exact)[-8:]
        e_gpu, e_cpu = rel(lg, exact), rel(lc, exact)
        d_gpu = float(np.abs(logprobs(lg)[top] - lp_exact[top]).max())
        d_cpu = float(np.abs(logprobs(lc)[top] - lp_exact[top]).max())
        assert e_gpu <= max(REL_TOL, 1.5 * e_cpu), (step, e_gpu, e_cpu)
        assert d_gpu <= max(LOGPROB_TOL, 1.5 * d_cpu), (step, d_gpu, d_cpu)
    gpu.close()
    cpu.close()


def test_device_side_top_and_logsumexp(elb):
    """elb_model_eval_top: the k best tokens by (logit descending, id ascending) and the double-precision log-sum-exp,
    computed on the device, equal what the host computes from the full logits of the same evaluation."""
    spec = synth.Spec(name="small", n_layer=2, n_embd=256, n_ff=512, n_head=4, n_head_kv=2, n_vocab=3001, layout="q4_k_m",
                      head_sigma=2e-5)
    tens = list(synth.generate(spec, 4))
    gpu = elb.Backend(spec, tens, 40)
    toks = synth.lcg_tokens(12, spec.n_vocab)
    full = gpu.eval(toks, 0)
    for k, (t, pos) in ((5, (toks, 0)), (1, ([7], 12)), (64, ([9], 13))):  # prompt chunk, then single-token steps
        if len(t) == 1:
            full = gpu.eval(t, pos)
        ids, vals, lse = gpu.eval_top(t, pos, k)  # the same tokens at the same positions again: same logits
        order = np.lexsort((np.arange(spec.n_vocab), -full.astype(np.float64)))[:k]
        assert np.array_equal(ids, order)
        assert np.array_equal(vals, full[order])
        assert abs(lse - ol.logsumexp(full)) <= 1e-12 * max(1.0, abs(lse))
    # constrained pick: only every third token allowed; the log-sum-exp is still over all tokens
    full = gpu.eval([3], 14)
    allowed = np.arange(spec.n_vocab) % 3 == 1
    ids, vals, lse = gpu.eval_top([3], 14, 4, allowed=allowed)
    cand = np.where(allowed)[0]
    order = cand[np.lexsort((cand, -full[cand].astype(np.float64)))[:4]]
    assert np.array_equal(ids, order) and np.array_equal(vals, full[order])
    assert abs(lse - ol.logsumexp(full)) <= 1e-12 * max(1.0, abs(lse))
    only = np.zeros(spec.n_vocab, bool)
    only[[17, 2999]] = True
    ids, vals, _ = gpu.eval_top([3], 14, 3, allowed=only)  # fewer allowed than asked for
    assert set(ids[:2]) == {17, 2999} and ids[2] == -1
    with pytest.raises(ValueError):
        gpu.eval_top([1], 15, 65)
    gpu.close()


@pytest.mark.parametrize("layout", ("q4_k_m", "f16"))
def test_model_loaded_from_gguf_equals_tensor_fed_model(elb, layout, tmp_path):
    """elb_model_load_gguf (file mapped and parsed by the library) gives bit-identical logits to the model built from the
    same tensors through elb_model_set_tensor, and reports the file's configuration."""
    spec = synth.Spec(name="small", n_layer=2, n_embd=256, n_ff=512, n_head=4, n_head_kv=2, n_vocab=640, layout=layout,
                      head_sigma=2e-5)
    tens = list(synth.generate(spec, 6))
    path = os.path.join(tmp_path, "model.gguf")
    synth.write_gguf(path, spec, tens)
    a = elb.Backend(spec, tens, 32)
    b = elb.Backend.from_gguf(path, 32)
    c = b.cfg()
    assert (c.n_layer, c.n_embd, c.n_ff, c.n_head, c.n_head_kv, c.n_vocab, c.head_dim) == (2, 256, 512, 4, 2, 640, 128)
    toks = synth.lcg_tokens(9, spec.n_vocab)
    assert np.array_equal(a.eval(toks, 0), b.eval(toks, 0))
    assert np.array_equal(a.eval([5], 9), b.eval([5], 9))
    a.close()
    b.close()
