"""The algorithmic work that the roofline fractions of bench.py are computed from, checked on the host: quantized weight
bytes per decoded token of the four benchmark shapes (block sizes of src/quant.h:23-41 of the reference: 34 B per 32
values for Q8_0, 144 B and 210 B per 256 for Q4_K and Q6_K), the microbenchmark matrix, and the multiply-accumulates
per token that the prompt figures use."""
import importlib.util
import os

import pytest

from exactinfer_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)  # only definitions run: the benchmark itself sits under __main__
    return mod


def test_row_bytes_follow_the_block_layouts():
    assert synth.row_bytes(synth.Q8_0, 256) == 8 * 34
    assert synth.row_bytes(synth.Q4_K, 256) == 144
    assert synth.row_bytes(synth.Q6_K, 256) == 210
    assert synth.row_bytes(synth.F16, 256) == 512


@pytest.mark.parametrize("name,gigabytes", (("qwen3-0.6b-f16", 1.192), ("qwen3-1.7b-q8_0", 1.828),
                                             ("qwen3-4b-q4_k_m", 2.503), ("qwen3-32b-q4_k_m", 19.36)))
def test_decode_weight_bytes_of_the_benchmark_shapes(name, gigabytes):
    got = synth.decode_weight_bytes(synth.SPECS[name]) / 1e9
    assert abs(got - gigabytes) <= 0.0006 * gigabytes + 0.0005, got


def test_q4_k_m_layout_mixes_the_types_as_the_file_format_does():
    s = synth.SPECS["qwen3-4b-q4_k_m"]
    assert s.weight_type("attn_v", 3) == synth.Q6_K and s.weight_type("token_embd", -1) == synth.Q6_K
    assert s.weight_type("ffn_down", 0) == synth.Q6_K and s.weight_type("ffn_down", 1) == synth.Q4_K
    assert s.weight_type("attn_q", 0) == synth.Q4_K and s.weight_type("ffn_gate", 5) == synth.Q4_K


def test_bench_constants():
    b = load_bench()
    assert b.MICRO_BYTES == 14_008_320 == 2560 * synth.row_bytes(synth.Q4_K, 9728)
    # 4.02 G multiply-accumulates per token for the 4B shape with the head, 3.63 G without it (a prompt chunk runs the
    # head once, for its last token only)
    s4 = synth.SPECS["qwen3-4b-q4_k_m"]
    assert abs(b.spec_macs_per_token(s4) / 1e9 - 3.633) < 0.001
    assert abs((b.spec_macs_per_token(s4) + s4.n_vocab * s4.n_embd) / 1e9 - 4.02) < 0.01
    # the ncu-derived traffic of the decode kernel stays within 1 % of the algorithmic bytes at the bench's positions
    s = synth.SPECS["qwen3-4b-q4_k_m"]
    kv_row = 2 * s.n_layer * s.kd * 4
    algorithmic = synth.decode_weight_bytes(s) + kv_row * 530
    assert abs(b.decode_traffic(s) / algorithmic - 1.0) < 0.01
    assert b.decode_traffic(synth.SPECS["qwen3-32b-q4_k_m"]) is None
