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
