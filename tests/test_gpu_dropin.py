"""The reference's own CLI, linked with this repository's backend in place of its CUDA translation unit
(oracle/_ref/el_b200, built by oracle/Makefile where the reference tree is available), runs its benchmark command on a
synthetic GGUF with --backend cuda: the drop-in boundary (el::cuda_available / el::make_cuda_backend / Backend::eval)
works end to end from the reference's main.cpp."""
import json
import os
import subprocess

import pytest

from exactinfer_b200 import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EL = os.path.join(ROOT, "oracle", "_ref", "el_b200")


@pytest.mark.skipif(not os.path.exists(EL), reason="oracle/_ref/el_b200 not built (needs the reference tree at build time)")
def test_reference_cli_runs_on_the_b200_backend(tmp_path):
    spec = synth.Spec(name="tiny", n_layer=2, n_embd=256, n_ff=512, n_head=4, n_head_kv=2, n_vocab=640, layout="q4_k_m")
    path = str(tmp_path / "tiny.gguf")
    synth.write_gguf(path, spec, list(synth.generate(spec, 4)))
    r = subprocess.run([EL, "bench", path, "--backend", "cuda", "--pp", "24", "--tg", "8", "--reps", "1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["backend"] == "cuda" and out["pp"] == 24 and out["tg"] == 8
    assert out["pp_tps"] > 0 and out["tg_tps"] > 0
    # a token id outside the vocabulary must surface as the reference's error exit, not a crash
    r = subprocess.run([EL, "bench", path, "--backend", "cuda", "--pp", "0", "--tg", "0"], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode != 0
