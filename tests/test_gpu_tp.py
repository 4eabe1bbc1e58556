"""Tensor parallelism on two GPUs against the CPU oracle (needs 2 devices; skipped on a single-GPU box): one process per
GPU, NCCL all-reduce after attn_output and ffn_down, all-gather of the logits. NVLS is switched off for the test."""
import os
import subprocess
import sys
import tempfile

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def device_count():
    import exactinfer_b200 as e
    from exactinfer_b200 import capi
    ok, _ = e.cuda_available()
    return capi.lib().elb_device_count() if ok else 0


@pytest.mark.parametrize("layout,source", (("q4_k_m", ""), ("q8_0", ""), ("f16", ""), ("q4_k_m", "gguf")))
def test_two_ranks_match_oracle(layout, source):
    if device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    with tempfile.TemporaryDirectory() as tmp:
        idf = os.path.join(tmp, "nccl_id")
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_gpu_worker.py"), str(r), "2", idf, layout, source],
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env) for r in range(2)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=300)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
            outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r}: ok" in out, f"rank {r}:\n{out[-3000:]}"


def test_rank_failure_at_setup_reaches_every_rank():
    """A rank whose set-up fails on the host (injected after its local allocations) still joins the set-up collectives
    with "failed" as its answer: rank 1 reports its own error, rank 0 learns that another rank failed, nobody waits in a
    collective for a rank that left (the test would time out). No GPU work is in flight when the rank gives up."""
    if device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", ELB_TEST_FAIL_FINALIZE_RANK="1")
    with tempfile.TemporaryDirectory() as tmp:
        idf = os.path.join(tmp, "nccl_id")
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_gpu_worker.py"), str(r), "2", idf, "q4_k_m", "fail"],
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env) for r in range(2)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=120)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
                out += "\n(timed out: a rank was left waiting)"
            outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r}: set-up failed as it must" in out, f"rank {r}:\n{out[-3000:]}"
    assert "injected failure" in outs[1] and "another rank" in outs[0], outs
