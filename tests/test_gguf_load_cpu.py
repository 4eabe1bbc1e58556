"""elb_model_load_gguf checks the file before it touches a device: the rejections of the reference's loader
(src/gguf.cpp, read_config / read_tensors in src/model.cpp:38-103) are testable without a GPU."""
import os
import struct

import numpy as np
import pytest

import exactinfer_b200 as e
from exactinfer_b200 import synth


def tiny(tmp_path):
    spec = synth.Spec(name="tiny", n_layer=1, n_embd=256, n_ff=256, n_head=2, n_head_kv=2, n_vocab=64, layout="q8_0")
    path = os.path.join(tmp_path, "m.gguf")
    synth.write_gguf(path, spec, list(synth.generate(spec, 1)))
    return path


def test_missing_file(tmp_path):
    with pytest.raises(ValueError, match="cannot open"):
        e.Backend.from_gguf(os.path.join(tmp_path, "nope.gguf"), 8)


def test_not_a_gguf_file(tmp_path):
    p = os.path.join(tmp_path, "x.gguf")
    open(p, "wb").write(b"GGML" + bytes(64))
    with pytest.raises(ValueError, match="not a GGUF"):
        e.Backend.from_gguf(p, 8)
    open(p, "wb").write(b"GGUF" + struct.pack("<I", 1) + bytes(64))
    with pytest.raises(e.ElbError, match="version"):
        e.Backend.from_gguf(p, 8)


def test_tensor_parallel_load_checks_the_file_first(tmp_path):
    """elb_model_load_gguf_tp: the same checks before any device or communicator is touched."""
    p = os.path.join(tmp_path, "x.gguf")
    open(p, "wb").write(b"GGML" + bytes(64))
    with pytest.raises(ValueError, match="not a GGUF"):
        e.Backend.from_gguf(p, 8, tp=(1, 2, bytes(128)))


def test_truncated_directory(tmp_path):
    path = tiny(tmp_path)
    data = open(path, "rb").read()
    cut = os.path.join(tmp_path, "cut.gguf")
    open(cut, "wb").write(data[:200])
    with pytest.raises(ValueError, match="damaged|missing|past the end"):
        e.Backend.from_gguf(cut, 8)


def test_other_architecture_rejected(tmp_path):
    path = tiny(tmp_path)
    data = open(path, "rb").read().replace(b"qwen3", b"qwen9")  # same length: offsets stay valid
    bad = os.path.join(tmp_path, "arch.gguf")
    open(bad, "wb").write(data)
    with pytest.raises(e.ElbError, match="architecture"):
        e.Backend.from_gguf(bad, 8)


def test_short_norm_vector_rejected(tmp_path):
    """A norm vector shorter than the embedding would make every kernel read past its allocation: refused while the
    file is checked, as the reference's expect_shape does (src/model.cpp:76,92-95)."""
    spec = synth.Spec(name="tiny", n_layer=1, n_embd=256, n_ff=256, n_head=2, n_head_kv=2, n_vocab=64, layout="q8_0")
    tens = []
    for role, layer, t, rows, n, data in synth.generate(spec, 1):
        if role == "attn_norm":
            n -= 32
            data = np.ascontiguousarray(data.view(np.float32).reshape(-1)[:n]).view(np.uint8).reshape(1, -1)
        tens.append((role, layer, t, rows, n, data))
    path = os.path.join(tmp_path, "short.gguf")
    synth.write_gguf(path, spec, tens)
    with pytest.raises(e.ElbError, match="shape of blk.0.attn_norm"):
        e.Backend.from_gguf(path, 8)


def test_tensor_offset_near_2_to_64_rejected(tmp_path):
    """The offset of a tensor comes from the file: a value close to 2^64 must not wrap the bounds check around."""
    path = tiny(tmp_path)
    data = bytearray(open(path, "rb").read())
    name = b"output_norm.weight"
    at = data.index(name) + len(name)
    (nd,) = struct.unpack_from("<I", data, at)
    off_at = at + 4 + 8 * nd + 4
    struct.pack_into("<Q", data, off_at, 2 ** 64 - 64)
    bad = os.path.join(tmp_path, "wrap.gguf")
    open(bad, "wb").write(bytes(data))
    with pytest.raises(ValueError, match="past the end"):
        e.Backend.from_gguf(bad, 8)
