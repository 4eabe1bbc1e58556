"""One rank of the CPU tensor-parallel check (started by test_tp_cpu.py): cut the tensors of one layer with the library's
host-side shard functions, run this rank's share through the oracle's operators, exchange over gloo, and compare with
the whole-tensor result on every rank.  usage: tp_cpu_worker.py RANK SIZE PORT"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

import exactinfer_b200 as e  # noqa: E402
from exactinfer_b200 import synth  # noqa: E402
import oracle_lib as ol  # noqa: E402


def all_reduce(v):
    t = torch.from_numpy(v.copy())
    dist.all_reduce(t)
    return t.numpy()


def main():
    rank, size, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=size)
    # F = 3 blocks of 256: an uneven cut over 2 ranks; 4 query / 2 KV heads
    spec = synth.Spec("tp-tiny", n_layer=1, n_embd=512, n_ff=768, n_head=4, n_head_kv=2, n_vocab=1000, layout="q4_k_m")
    tens = {(role, layer): (t, rows, n, w) for role, layer, t, rows, n, w in synth.generate(spec, 7)}
    d = e.tp_dims(spec, rank, size)
    E, F, QD = spec.n_embd, spec.n_ff, spec.qd
    rng = np.random.default_rng(99)  # same stream on every rank
    x = rng.normal(size=E).astype(np.float32)
    att = rng.normal(size=QD).astype(np.float32)

    def full(role, v):
        t, rows, n, w = tens[(role, 0 if role != "token_embd" else -1)]
        return ol.matvec(t, rows, n, w, v)

    def mine(role, v, as_role=None):
        t, rows, n, w = tens[(role, 0 if role != "token_embd" else -1)]
        r, c, b = e.tp_shard(spec, rank, size, as_role or role, t, rows, n, w)
        return ol.matvec(t, r, c, b, v), r, c

    # the cuts tile the whole dimension
    dims = [e.tp_dims(spec, r, size) for r in range(size)]
    assert dims[0]["f0"] == 0 and dims[-1]["f1"] == F and all(dims[i]["f1"] == dims[i + 1]["f0"] for i in range(size - 1))
    assert dims[0]["v0"] == 0 and dims[-1]["v1"] == spec.n_vocab
    assert all(dims[i]["v1"] == dims[i + 1]["v0"] and dims[i]["v0"] % 16 == 0 for i in range(size - 1))
    assert all(dd["f0"] % 256 == 0 for dd in dims) and len({dd["f1"] - dd["f0"] for dd in dims}) == 2  # uneven

    # column-parallel: a rank's rows are bit-identical to the same rows of the whole product
    q_full, (q_mine, r, c) = full("attn_q", x), mine("attn_q", x)
    assert c == E and r == d["n_head"] * 128
    assert np.array_equal(q_mine, q_full[rank * r:(rank + 1) * r])
    k_full, (k_mine, r, _) = full("attn_k", x), mine("attn_k", x)
    assert np.array_equal(k_mine, k_full[rank * r:(rank + 1) * r])

    # row-parallel attention output: partial sums over this rank's heads, all-reduced
    o_full = full("attn_output", att)
    o_mine, r, c = mine("attn_output", att[rank * d["n_head"] * 128:(rank + 1) * d["n_head"] * 128])
    assert r == E and c == d["n_head"] * 128
    o_sum = all_reduce(o_mine)
    assert np.max(np.abs(o_sum - o_full)) <= 2e-6 * np.max(np.abs(o_full)), "attn_output all-reduce"

    # MLP block: gate/up by rows, SwiGLU locally, down by columns, all-reduce
    g, u = full("ffn_gate", x), full("ffn_up", x)
    act = (g / (1.0 + np.exp(-g))).astype(np.float32) * u
    y_full = full("ffn_down", act)
    (g_m, r, _), (u_m, _, _) = mine("ffn_gate", x), mine("ffn_up", x)
    assert r == d["f1"] - d["f0"] and np.array_equal(g_m, g[d["f0"]:d["f1"]]) and np.array_equal(u_m, u[d["f0"]:d["f1"]])
    act_m = (g_m / (1.0 + np.exp(-g_m))).astype(np.float32) * u_m
    y_m, r, c = mine("ffn_down", act_m)
    assert r == E and c == d["f1"] - d["f0"]
    y_sum = all_reduce(y_m)
    assert np.max(np.abs(y_sum - y_full)) <= 2e-6 * np.max(np.abs(y_full)), "ffn_down all-reduce"

    # head by vocabulary rows (tied table cut with the role of the output tensor), all-gather of padded chunks
    l_full = full("token_embd", x)
    l_m, r, _ = mine("token_embd", x, as_role="output")
    assert r == d["v1"] - d["v0"]
    chunk = dims[0]["v1"] - dims[0]["v0"]
    pad = np.zeros(chunk, np.float32)
    pad[:r] = l_m
    parts = [torch.zeros(chunk) for _ in range(size)]
    dist.all_gather(parts, torch.from_numpy(pad))
    l_all = torch.cat(parts).numpy()[:spec.n_vocab]
    assert np.array_equal(l_all, l_full), "head all-gather"

    # replicated tensors come back whole
    t, rows, n, w = tens[("attn_norm", 0)]
    r, c, b = e.tp_shard(spec, rank, size, "attn_norm", t, rows, n, w)
    assert (r, c) == (rows, n) and np.array_equal(b, np.ascontiguousarray(w).reshape(-1))
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: ok")


if __name__ == "__main__":
    main()
