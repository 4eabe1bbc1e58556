"""Several sequences in one model (elb_model_eval_batch) against the CPU oracle, which evaluates every sequence on its
own: prompts as rows of one sequence, batched single-token steps as one row per sequence, and a batch that mixes a
two-row continuation of one sequence with single rows of others. Bars as in test_gpu_model.py."""
import numpy as np
import pytest

import oracle_lib as ol
from exactinfer_b200 import synth

pytestmark = pytest.mark.gpu
LOGPROB_TOL = 3e-5  # max |delta logprob| against the CPU path
REL_TOL = 2e-4      # logits relative to their largest magnitude


@pytest.fixture(scope="module")
def elb():
    import exactinfer_b200 as e
    ok, why = e.cuda_available()
    assert ok, f"CUDA path unavailable: {why}"
    return e


def rel(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(np.abs(b).max(), 1e-30))


def logprobs(l):
    return l.astype(np.float64) - ol.logsumexp(l)


@pytest.mark.parametrize("layout", ("q8_0", "q4_k_m", "f16"))
def test_sequences_match_oracle(elb, layout):
    spec = synth.Spec(name="batch", n_layer=2, n_embd=512, n_ff=1024, n_head=8, n_head_kv=2, n_vocab=1200, layout=layout,
                      head_sigma=2e-5)
    tens = list(synth.generate(spec, 17))
    n_seq, n_ctx = 3, 48
    gpu = elb.Backend(spec, tens, n_ctx, max_batch=16, n_seq=n_seq)
    cpus = [ol.OracleModel(spec, tens, n_ctx) for _ in range(n_seq)]
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, spec.n_vocab, size=k).astype(np.int32) for k in (10, 7, 13)]
    last_g, last_c = [None] * n_seq, [None] * n_seq
    for s, toks in enumerate(prompts):  # prompts: rows of one sequence, only the last row's logits wanted
        want = np.zeros(len(toks), np.uint8)
        want[-1] = 1
        last_g[s] = gpu.eval_batch(toks, np.full(len(toks), s), np.arange(len(toks)), want)[0]
        last_c[s] = cpus[s].eval(toks, 0)
        assert rel(last_g[s], last_c[s]) <= REL_TOL
    pos = [len(t) for t in prompts]
    worst_rel = worst_lp = 0.0
    for step in range(4):  # batched decode: one row per sequence, teacher-forced on the oracle's greedy token
        nxt = [int(np.argmax(l)) for l in last_c]
        for s in range(n_seq):
            top = np.argsort(last_c[s])[-8:]
            worst_lp = max(worst_lp, float(np.abs(logprobs(last_g[s])[top] - logprobs(last_c[s])[top]).max()))
        order = [2, 0, 1] if step % 2 else [0, 1, 2]  # row order is free
        out = gpu.eval_batch([nxt[s] for s in order], order, [pos[s] for s in order])
        for r, s in enumerate(order):
            last_g[s] = out[r]
            last_c[s] = cpus[s].eval([nxt[s]], pos[s])
            worst_rel = max(worst_rel, rel(last_g[s], last_c[s]))
            pos[s] += 1
    # a mixed batch: two more rows of sequence 1 and one row each of sequences 0 and 2; logits of three of the rows
    t1 = rng.integers(0, spec.n_vocab, size=2).astype(np.int32)
    t0, t2 = int(np.argmax(last_c[0])), int(np.argmax(last_c[2]))
    out = gpu.eval_batch([t1[0], t0, t1[1], t2], [1, 0, 1, 2], [pos[1], pos[0], pos[1] + 1, pos[2]], want=[0, 1, 1, 1])
    c1 = cpus[1].eval(t1, pos[1])
    c0 = cpus[0].eval([t0], pos[0])
    c2 = cpus[2].eval([t2], pos[2])
    for g, c in zip(out, (c0, c1, c2)):
        worst_rel = max(worst_rel, rel(g, c))
    gpu.close()
    for c in cpus:
        c.close()
    assert worst_rel <= REL_TOL and worst_lp <= LOGPROB_TOL, (worst_rel, worst_lp)


def test_argument_errors(elb):
    spec = synth.Spec(name="batch", n_layer=1, n_embd=256, n_ff=512, n_head=4, n_head_kv=2, n_vocab=300, layout="q8_0")
    gpu = elb.Backend(spec, list(synth.generate(spec, 3)), 16, max_batch=8, n_seq=2)
    with pytest.raises(IndexError):
        gpu.eval_batch([1], [2], [0])          # sequence index out of range
    with pytest.raises(IndexError):
        gpu.eval_batch([1], [0], [16])         # context window full
    with pytest.raises(ValueError):
        gpu.eval_batch([1, 2], [0, 0], [0, 2])  # rows of a sequence must be consecutive
    with pytest.raises(IndexError):
        gpu.eval_batch(list(range(9)), [0] * 9, list(range(9)))  # more rows than max_batch
    gpu.close()


def test_batch_top_equals_host_reduction_of_the_same_logits(elb):
    """elb_model_eval_batch_top: the k best tokens (logit descending, id ascending) and the double-precision log-sum-exp
    of every wanted row, computed on the device, against the host's reduction of the logits elb_model_eval_batch returns
    for the same rows (two models with the same weights and the same history, so both see the same step)."""
    spec = synth.Spec(name="batch-top", n_layer=2, n_embd=512, n_ff=1024, n_head=8, n_head_kv=2, n_vocab=1200, layout="q4_k_m",
                      head_sigma=2e-5)
    tens = list(synth.generate(spec, 19))
    n_seq, n_ctx, k = 4, 32, 5
    a = elb.Backend(spec, tens, n_ctx, max_batch=16, n_seq=n_seq)
    b = elb.Backend(spec, tens, n_ctx, max_batch=16, n_seq=n_seq)
    rng = np.random.default_rng(8)
    for s in range(n_seq):  # prompts of different lengths, one sequence each
        p = rng.integers(0, spec.n_vocab, size=4 + 2 * s).astype(np.int32)
        for m in (a, b):
            m.eval_batch(p, np.full(p.size, s, np.int32), np.arange(p.size, dtype=np.int32), want_logits=False)
    toks = rng.integers(0, spec.n_vocab, size=n_seq).astype(np.int32)
    seq = np.arange(n_seq, dtype=np.int32)
    pos = np.array([4 + 2 * s for s in range(n_seq)], np.int32)
    want = np.array([1, 0, 1, 1], np.uint8)
    logits = a.eval_batch(toks, seq, pos, want=want)  # [3][V]
    ids, vals, lse = b.eval_batch_top(toks, seq, pos, k=k, want=want)
    assert ids.shape == (3, k) and vals.shape == (3, k) and lse.shape == (3,)
    for r in range(3):
        order = np.lexsort((np.arange(spec.n_vocab), -logits[r].astype(np.float64)))[:k]
        assert np.array_equal(ids[r], order), r
        assert np.array_equal(vals[r].view(np.uint32), logits[r][order].view(np.uint32)), r
        assert abs(lse[r] - ol.logsumexp(logits[r])) <= 1e-9 * max(1.0, abs(lse[r])), r
    with pytest.raises(ValueError):
        b.eval_batch_top(toks, seq, pos + 1, k=0)
    a.close()
    b.close()
