"""Generate tests/golden/*.npz from the reference's own CPU code (oracle/_ref/libelref.so, built from the
unmodified reference sources by oracle/Makefile). Run where the reference tree is available:

    make -C oracle ref && python tests/golden/make_golden.py

The fixtures are small seeded cases: raw block bytes with the reference's decoded rows and matvec results,
RMSNorm inputs/outputs, and the logits of a tiny Qwen3-shaped model (weights regenerated from the seed by
exactinfer_b200.synth; a SHA-256 of the weight bytes guards against generator drift).
"""
import hashlib
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle_lib as ol  # noqa: E402
from exactinfer_b200 import synth  # noqa: E402

TINY = dict(name="tiny", n_layer=2, n_embd=256, n_ff=512, n_head=4, n_head_kv=2, n_vocab=640, head_sigma=2e-5)


def weights_digest(tensors):
    h = hashlib.sha256()
    for role, layer, t, rows, n, data in tensors:
        h.update(f"{role}:{layer}:{t}:{rows}:{n}".encode())
        h.update(np.ascontiguousarray(data).tobytes())
    return h.hexdigest()


def main():
    assert ol.have_ref(), "build oracle/_ref first (make -C oracle ref)"
    ol.ref().ref_set_threads(1)
    rng = np.random.default_rng(20251125)
    ops = {}
    for t, rows, n in ((synth.Q8_0, 6, 512), (synth.Q4_K, 6, 512), (synth.Q6_K, 6, 512), (synth.F16, 6, 200),
                       (synth.F32, 3, 100)):
        w = synth.rand_weight(rng, t, rows, n)
        x = rng.normal(size=n).astype(np.float32)
        name = synth.TYPE_NAMES[t]
        ops[f"{name}_w"] = w
        ops[f"{name}_x"] = x
        ops[f"{name}_deq"] = ol.dequant_rows(t, rows, n, w, lib="ref")
        ops[f"{name}_y"] = ol.matvec(t, rows, n, w, x, lib="ref")
    # fp16 corner values: zero, subnormals, smallest/largest normals, both signs
    h = np.array([0x0000, 0x8000, 0x0001, 0x03ff, 0x0400, 0x3c00, 0x7bff, 0xfbff, 0x8001, 0x3555], dtype=np.uint16)
    ops["f16_bits"] = h
    ops["f16_vals"] = ol.dequant_rows(synth.F16, 1, h.size, h.view(np.uint8).reshape(1, -1), lib="ref")[0]
    for n in (128, 1000):
        x = (rng.normal(size=n) * 3).astype(np.float32)
        w = synth.rand_norm(rng, n)
        ops[f"rms{n}_x"], ops[f"rms{n}_w"] = x, w
        ops[f"rms{n}_y"] = ol.rmsnorm(x, w, 1e-6, lib="ref")
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **ops)

    model = {}
    for layout in ("f16", "q8_0", "q4_k_m"):
        spec = synth.Spec(layout=layout, **TINY)
        tens = list(synth.generate(spec, seed=11))
        path = os.path.join(tempfile.mkdtemp(), "tiny.gguf")
        synth.write_gguf(path, spec, tens)
        rm = ol.RefModel(path, 32)
        toks = synth.lcg_tokens(12, spec.n_vocab)
        outs = [rm.eval(toks[:8], 0)]
        for i in range(8, 12):
            outs.append(rm.eval(toks[i:i + 1], i))
        model[f"{layout}_logits"] = np.stack(outs)
        model[f"{layout}_sha"] = np.frombuffer(weights_digest(tens).encode(), dtype=np.uint8)
        rm.close()
        os.remove(path)
    model["tokens"] = synth.lcg_tokens(12, TINY["n_vocab"])
    np.savez_compressed(os.path.join(HERE, "tiny_model.npz"), **model)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
