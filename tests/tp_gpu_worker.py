"""One rank of the 2-GPU tensor-parallel parity check (started by test_gpu_tp.py): Backend(tp=...) on GPU `rank`, a prompt
chunk then single-token steps, every rank compares the gathered logits with the CPU oracle's whole-model result.
usage: tp_gpu_worker.py RANK SIZE ID_FILE LAYOUT [gguf|fail]   (gguf: every rank loads the same GGUF file itself;
fail: one rank's set-up is made to fail on the host (ELB_TEST_FAIL_FINALIZE_RANK) and EVERY rank must get an error)"""
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

import exactinfer_b200 as e  # noqa: E402
from exactinfer_b200 import synth  # noqa: E402
import oracle_lib as ol  # noqa: E402

LOGPROB_TOL = 3e-5  # max |delta logprob| against the CPU path
REL_TOL = 2e-4      # logits and residual stream relative to their largest magnitude


def main():
    rank, size, id_file, layout = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    if rank == 0:
        ident = e.tp_unique_id()
        with open(id_file + ".tmp", "wb") as f:
            f.write(ident)
        os.replace(id_file + ".tmp", id_file)
    else:
        t0 = time.time()
        while not os.path.exists(id_file):
            if time.time() - t0 > 120:
                raise SystemExit("rank 0 never published the communicator id")
            time.sleep(0.05)
        ident = open(id_file, "rb").read()
    # F = 5 blocks of 256 (uneven cut), vocabulary not a multiple of 16
    spec = synth.Spec(name="tp-small", n_layer=3, n_embd=512, n_ff=1280, n_head=8, n_head_kv=2, n_vocab=2043,
                      layout=layout, head_sigma=2e-5)
    tens = list(synth.generate(spec, 33))
    n_prompt, n_decode = 40, 5
    if len(sys.argv) > 5 and sys.argv[5] == "gguf":  # the library maps the file and uploads this rank's cuts
        path = id_file + ".gguf"
        if rank == 0:
            synth.write_gguf(path + ".tmp", spec, tens)
            os.replace(path + ".tmp", path)
        t0 = time.time()
        while not os.path.exists(path):
            if time.time() - t0 > 120:
                raise SystemExit("rank 0 never wrote the model file")
            time.sleep(0.05)
        gpu = e.Backend.from_gguf(path, n_prompt + n_decode + 1, device=rank, tp=(rank, size, ident))
    elif len(sys.argv) > 5 and sys.argv[5] == "fail":
        try:
            e.Backend(spec, tens, n_prompt + n_decode + 1, device=rank, tp=(rank, size, ident))
        except (MemoryError, RuntimeError) as exc:
            print(f"rank {rank}: set-up failed as it must: {exc}")
            return
        raise SystemExit(f"rank {rank}: the model came up although a rank of the group failed")
    else:
        gpu = e.Backend(spec, tens, n_prompt + n_decode + 1, device=rank, tp=(rank, size, ident))
    cpu = ol.OracleModel(spec, tens, n_prompt + n_decode + 1)
    toks = synth.lcg_tokens(n_prompt, spec.n_vocab)

    def rel(a, b):
        return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(np.abs(b).max(), 1e-30))

    def logprobs(l):
        return l.astype(np.float64) - ol.logsumexp(l)

    # a short chunk first (5 rows: the all-reduce of a small batch of rows goes through peer memory), then the prompt
    l5g, l5c = gpu.eval(toks[:5], 0), cpu.eval(toks[:5], 0)
    assert rel(l5g, l5c) <= REL_TOL, rel(l5g, l5c)
    assert rel(gpu.hidden(), cpu.hidden()) <= REL_TOL
    lg, lc = gpu.eval(toks, 0), cpu.eval(toks, 0)
    worst_rel, worst_lp = max(rel(lg, lc), rel(l5g, l5c)), 0.0
    assert rel(gpu.hidden(), cpu.hidden()) <= REL_TOL
    pos = n_prompt
    for _ in range(n_decode):
        nxt = int(np.argmax(lc))
        top = np.argsort(lc)[-8:]
        worst_lp = max(worst_lp, float(np.abs(logprobs(lg)[top] - logprobs(lc)[top]).max()))
        lg, lc = gpu.eval([nxt], pos), cpu.eval([nxt], pos)
        worst_rel = max(worst_rel, rel(lg, lc))
        pos += 1
    ms, launches = gpu.last_eval_stats()
    gpu.close()
    cpu.close()
    print(f"rank {rank}: rel {worst_rel:.3e} logprob {worst_lp:.3e} launches/step {launches}")
    assert worst_rel <= REL_TOL and worst_lp <= LOGPROB_TOL, (worst_rel, worst_lp)
    print(f"rank {rank}: ok")


if __name__ == "__main__":
    main()
