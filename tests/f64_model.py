"""float64 restatement of the forward pass in numpy, for adjudication only: where the reference's fp32 CPU path is itself
many units of fp32 rounding away from exact arithmetic (long contexts), a parity test compares both the CUDA path and
the CPU path with this one instead of asking the two fp32 computations to agree more closely than either is accurate.
Follows CpuModel::forward of the reference (src/model.cpp:157-234) with every operation in double."""
import numpy as np

import oracle_lib as ol
from exactinfer_b200 import synth


def f64_logits(spec, tens, toks):
    """float64 forward pass of a 1-layer model (last token's logits)."""
    T = {(r, l): (t, rows, n, w) for r, l, t, rows, n, w in tens}
    def W(role, l=0):
        t, rows, n, w = T[(role, l)]
        if t == synth.F32: return np.ascontiguousarray(w).view(np.float32).reshape(rows, n).astype(np.float64)
        return ol.dequant_rows(t, rows, n, w).astype(np.float64)
    E, H, HKV, D = spec.n_embd, spec.n_head, spec.n_head_kv, spec.head_dim
    emb = W("token_embd", -1)
    x = emb[toks]                                   # [n, E]
    def rms(v, w): return v / np.sqrt((v * v).mean(-1, keepdims=True) + spec.eps) * w
    n = len(toks)
    for l in range(spec.n_layer):
        h = rms(x, W("attn_norm", l)[0])
        q = (h @ W("attn_q", l).T).reshape(n, H, D); k = (h @ W("attn_k", l).T).reshape(n, HKV, D); v = (h @ W("attn_v", l).T).reshape(n, HKV, D)
        q = rms(q, W("attn_q_norm", l)[0]); k = rms(k, W("attn_k_norm", l)[0])
        half = D // 2
        inv = spec.rope_base ** (-2.0 * np.arange(half) / D)
        th = np.arange(n)[:, None] * inv[None, :]
        c, s = np.cos(th)[:, None, :], np.sin(th)[:, None, :]
        def rope(a): return np.concatenate([a[..., :half] * c - a[..., half:] * s, a[..., :half] * s + a[..., half:] * c], -1)
        q, k = rope(q), rope(k)
        out = np.zeros((n, H, D))
        g = H // HKV
        for hd in range(H):
            sc = q[:, hd] @ k[:, hd // g].T / np.sqrt(D)
            sc = np.where(np.tril(np.ones((n, n), bool)), sc, -np.inf)
            p = np.exp(sc - sc.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
            out[:, hd] = p @ v[:, hd // g]
        x = x + out.reshape(n, H * D) @ W("attn_output", l).T
        h = rms(x, W("ffn_norm", l)[0])
        a = h @ W("ffn_gate", l).T; u = h @ W("ffn_up", l).T
        x = x + (a / (1 + np.exp(-a)) * u) @ W("ffn_down", l).T
    h = rms(x[-1], W("output_norm", -1)[0])
    return h @ emb.T


def f64_last_token(spec, tens, toks, chunk=2048):
    """float64 forward pass of a model of any size: the last token's residual stream (before the final norm) and
    logits. Matrices are decoded `chunk` rows at a time, so that the float64 copy of a large weight never exists whole."""
    T = {(r, l): (t, rows, n, w) for r, l, t, rows, n, w in tens}
    toks = np.asarray(toks)

    def vec(role, l):
        t, rows, n, w = T[(role, l)]
        return np.ascontiguousarray(w).view(np.float32).reshape(-1).astype(np.float64)

    def mm(x, role, l):  # x [n, K] -> [n, rows]
        t, rows, n, w = T[(role, l)]
        out = np.empty((x.shape[0], rows))
        for r0 in range(0, rows, chunk):
            r1 = min(rows, r0 + chunk)
            out[:, r0:r1] = x @ ol.dequant_rows(t, rows, n, w, r0, r1 - r0).astype(np.float64).T
        return out

    H, HKV, D = spec.n_head, spec.n_head_kv, spec.head_dim
    t, rows, n_, w = T[("token_embd", -1)]
    x = np.stack([ol.dequant_rows(t, rows, n_, w, int(tok), 1)[0] for tok in toks]).astype(np.float64)
    def rms(v, wt): return v / np.sqrt((v * v).mean(-1, keepdims=True) + spec.eps) * wt
    n = len(toks)
    half = D // 2
    inv = spec.rope_base ** (-2.0 * np.arange(half) / D)
    th = np.arange(n)[:, None] * inv[None, :]
    c, sn = np.cos(th)[:, None, :], np.sin(th)[:, None, :]
    def rope(a): return np.concatenate([a[..., :half] * c - a[..., half:] * sn, a[..., :half] * sn + a[..., half:] * c], -1)
    causal = np.tril(np.ones((n, n), bool))
    for l in range(spec.n_layer):
        h = rms(x, vec("attn_norm", l))
        q = mm(h, "attn_q", l).reshape(n, H, D); k = mm(h, "attn_k", l).reshape(n, HKV, D); v = mm(h, "attn_v", l).reshape(n, HKV, D)
        q, k = rope(rms(q, vec("attn_q_norm", l))), rope(rms(k, vec("attn_k_norm", l)))
        out = np.zeros((n, H, D)); g = H // HKV
        for hd in range(H):
            sc = np.where(causal, q[:, hd] @ k[:, hd // g].T / np.sqrt(D), -np.inf)
            p = np.exp(sc - sc.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
            out[:, hd] = p @ v[:, hd // g]
        x = x + mm(out.reshape(n, H * D), "attn_output", l)
        h = rms(x, vec("ffn_norm", l))
        a = mm(h, "ffn_gate", l); u = mm(h, "ffn_up", l)
        with np.errstate(over="ignore"):
            x = x + mm(a / (1 + np.exp(-a)) * u, "ffn_down", l)
    head = ("output", -1) if ("output", -1) in T else ("token_embd", -1)
    return x[-1], mm(rms(x[-1:], vec("output_norm", -1)), head[0], -1)[0]
