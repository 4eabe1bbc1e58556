"""Seeded synthetic Qwen3-shaped weights in ggml block formats (numpy only).

Real Qwen3 files are not available offline, so every test and benchmark draws raw quantization blocks from a
seed with the value distributions below and feeds the same bytes to the CUDA backend and to the CPU oracle.

Block layouts follow the reference's structs (src/quant.h:23-41):
  Q8_0  34 B / 32 values : fp16 d, int8 qs[32]
  Q4_K 144 B / 256 values: fp16 d, fp16 dmin, u8 scales[12] (6-bit scale and min of 8 sub-blocks), u8 qs[128]
  Q6_K 210 B / 256 values: u8 ql[128], u8 qh[64], int8 scales[16], fp16 d
Distributions: nibbles / 6-bit fields / int8 values uniform over their range, fp16 scales |N(0, 1e-3)|,
F16 weights N(0, 0.02), norm weights 1 + N(0, 0.01) as fp32. No fp16 NaN/Inf is ever produced.
"""
from __future__ import annotations

import dataclasses

import numpy as np

F32, F16, Q8_0, Q4_K, Q6_K, BF16 = 0, 1, 8, 12, 14, 30  # ggml type ids (src/gguf.h:22-25)
TYPE_NAMES = {F32: "F32", F16: "F16", Q8_0: "Q8_0", Q4_K: "Q4_K", Q6_K: "Q6_K", BF16: "BF16"}
BLOCK = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210)}


def row_bytes(t: int, n: int) -> int:
    blk, nb = BLOCK[t]
    if n % blk:
        raise ValueError(f"row length {n} is not a multiple of the {TYPE_NAMES[t]} block ({blk})")
    return n // blk * nb


def _scale_f16(rng: np.random.Generator, shape, sigma=1e-3) -> np.ndarray:
    return np.abs(rng.normal(0.0, sigma, size=shape)).astype(np.float16)


def rand_q8_0(rng, rows: int, n: int, sigma=1e-3) -> np.ndarray:
    nb = n // 32
    out = np.empty((rows, nb, 34), dtype=np.uint8)
    out[:, :, 0:2] = _scale_f16(rng, (rows, nb), sigma).view(np.uint8).reshape(rows, nb, 2)
    out[:, :, 2:] = rng.integers(-127, 128, size=(rows, nb, 32), dtype=np.int8).view(np.uint8)
    return out.reshape(rows, nb * 34)


def rand_q4_k(rng, rows: int, n: int, sigma=1e-3) -> np.ndarray:
    nb = n // 256
    out = np.empty((rows, nb, 144), dtype=np.uint8)
    out[:, :, 0:2] = _scale_f16(rng, (rows, nb), sigma).view(np.uint8).reshape(rows, nb, 2)
    out[:, :, 2:4] = _scale_f16(rng, (rows, nb), sigma).view(np.uint8).reshape(rows, nb, 2)
    out[:, :, 4:] = rng.integers(0, 256, size=(rows, nb, 140), dtype=np.uint8)
    return out.reshape(rows, nb * 144)


def rand_q6_k(rng, rows: int, n: int, sigma=1e-3) -> np.ndarray:
    nb = n // 256
    out = np.empty((rows, nb, 210), dtype=np.uint8)
    out[:, :, 0:208] = rng.integers(0, 256, size=(rows, nb, 208), dtype=np.uint8)
    out[:, :, 208:210] = _scale_f16(rng, (rows, nb), sigma).view(np.uint8).reshape(rows, nb, 2)
    return out.reshape(rows, nb * 210)


def rand_f16(rng, rows: int, n: int, sigma=0.02) -> np.ndarray:
    return rng.normal(0.0, sigma, size=(rows, n)).astype(np.float16).view(np.uint8).reshape(rows, n * 2)


def rand_weight(rng, t: int, rows: int, n: int, sigma=1e-3) -> np.ndarray:
    """Raw bytes of a (rows x n) weight of ggml type t, as a C-contiguous uint8 array (rows, row_bytes).
    sigma is the spread of the fp16 block scales of the quantized types."""
    if t == Q8_0:
        return rand_q8_0(rng, rows, n, sigma)
    if t == Q4_K:
        return rand_q4_k(rng, rows, n, sigma)
    if t == Q6_K:
        return rand_q6_k(rng, rows, n, sigma)
    if t == F16:
        return rand_f16(rng, rows, n)
    if t == F32:
        return rng.normal(0.0, 0.02, size=(rows, n)).astype(np.float32).view(np.uint8).reshape(rows, n * 4)
    raise ValueError(f"no generator for ggml type {t}")


def rand_norm(rng, n: int) -> np.ndarray:
    return (1.0 + rng.normal(0.0, 0.01, size=n)).astype(np.float32)


@dataclasses.dataclass
class Spec:
    """Shape of a Qwen3 dense decoder plus the weight-type layout ('f16', 'q8_0', 'q4_k', 'q6_k', 'q4_k_m')."""

    name: str
    n_layer: int
    n_embd: int
    n_ff: int
    n_head: int
    n_head_kv: int
    n_vocab: int
    layout: str
    head_dim: int = 128
    rope_base: float = 1e6
    eps: float = 1e-6
    tied: bool = True
    # spread of the block scales of token_embd / output. The benchmark configurations keep 1e-3 like every other
    # tensor, which makes logits of magnitude 10^2..10^3 (one fp32 ulp there is already 3e-5..6e-5); parity tests that
    # hold the absolute log-probability bar use a smaller head so that logits are O(10) as in a trained model.
    head_sigma: float = 1e-3

    @property
    def qd(self):
        return self.n_head * self.head_dim

    @property
    def kd(self):
        return self.n_head_kv * self.head_dim

    def weight_type(self, role: str, layer: int) -> int:
        """Q4_K_M: Q4_K everywhere except Q6_K for attn_v, every other layer's ffn_down, and the head / embedding."""
        lay = self.layout
        if lay == "f16":
            return F16
        if lay == "q8_0":
            return Q8_0
        if lay == "q4_k":
            return Q4_K
        if lay == "q6_k":
            return Q6_K
        if lay == "q4_k_m":
            if role in ("token_embd", "output", "attn_v"):
                return Q6_K
            if role == "ffn_down" and layer % 2 == 0:
                return Q6_K
            return Q4_K
        raise ValueError(lay)


V_FULL = 151936
SPECS = {
    "qwen3-0.6b-f16": Spec("qwen3-0.6b-f16", 28, 1024, 3072, 16, 8, V_FULL, "f16"),
    "qwen3-1.7b-q8_0": Spec("qwen3-1.7b-q8_0", 28, 2048, 6144, 16, 8, V_FULL, "q8_0"),
    "qwen3-4b-q4_k_m": Spec("qwen3-4b-q4_k_m", 36, 2560, 9728, 32, 8, V_FULL, "q4_k_m"),
    "qwen3-32b-q4_k_m": Spec("qwen3-32b-q4_k_m", 64, 5120, 25600, 64, 8, V_FULL, "q4_k_m"),
}

# tensor roles, in the order and with the ggml names the reference's loader uses (src/model.cpp:66-103)
GLOBAL_ROLES = ("token_embd", "output", "output_norm")
LAYER_ROLES = ("attn_norm", "ffn_norm", "attn_q_norm", "attn_k_norm", "attn_q", "attn_k", "attn_v", "attn_output",
               "ffn_gate", "ffn_up", "ffn_down")
ROLE_ID = {r: i for i, r in enumerate(GLOBAL_ROLES + LAYER_ROLES)}


def layer_shapes(s: Spec) -> dict:
    """role -> (rows, n) as (out, in), i.e. ggml ne = [in, out]"""
    return {"attn_q": (s.qd, s.n_embd), "attn_k": (s.kd, s.n_embd), "attn_v": (s.kd, s.n_embd),
            "attn_output": (s.n_embd, s.qd), "ffn_gate": (s.n_ff, s.n_embd), "ffn_up": (s.n_ff, s.n_embd),
            "ffn_down": (s.n_embd, s.n_ff)}


def decode_weight_bytes(spec: Spec) -> int:
    """Quantized weight bytes a single-token step has to read once: every matrix of every layer plus the head (the
    tied embedding table when there is no output tensor); norm vectors and the one embedding row are left out. This is
    the algorithmic traffic of decode before the KV rows are added."""
    total = spec.n_vocab * row_bytes(spec.weight_type("output" if not spec.tied else "token_embd", -1), spec.n_embd)
    for l in range(spec.n_layer):
        for role, (rows, n) in layer_shapes(spec).items():
            total += rows * row_bytes(spec.weight_type(role, l), n)
    return total


def generate(spec: Spec, seed: int, share_layers: bool = False):
    """Yield (role, layer, ggml_type, rows, n, bytes) for every tensor of the model (layer = -1 for globals).

    share_layers=True reuses layer 0's and layer 1's random blocks for the later layers of the same parity
    (keeps every tensor's type and shape; only for timing runs where host generation time matters).
    """
    rng = np.random.default_rng(seed)
    E, V = spec.n_embd, spec.n_vocab
    yield ("token_embd", -1, spec.weight_type("token_embd", -1), V, E,
           rand_weight(rng, spec.weight_type("token_embd", -1), V, E, spec.head_sigma))
    if not spec.tied:
        yield ("output", -1, spec.weight_type("output", -1), V, E,
               rand_weight(rng, spec.weight_type("output", -1), V, E, spec.head_sigma))
    yield "output_norm", -1, F32, 1, E, rand_norm(rng, E).view(np.uint8).reshape(1, -1)
    cache = {}
    for l in range(spec.n_layer):
        for role in ("attn_norm", "ffn_norm"):
            yield role, l, F32, 1, E, rand_norm(rng, E).view(np.uint8).reshape(1, -1)
        for role in ("attn_q_norm", "attn_k_norm"):
            yield role, l, F32, 1, spec.head_dim, rand_norm(rng, spec.head_dim).view(np.uint8).reshape(1, -1)
        for role, (rows, n) in layer_shapes(spec).items():
            t = spec.weight_type(role, l)
            key = (role, l % 2)
            if share_layers and key in cache and cache[key][0] == t:
                w = cache[key][1]
            else:
                w = rand_weight(rng, t, rows, n)
                cache[key] = (t, w)
            yield role, l, t, rows, n, w


def lcg_tokens(count: int, n_vocab: int, seed: int = 12345) -> np.ndarray:
    """The reference benchmark's token stream (src/main.cpp:629-630)."""
    out = np.empty(count, dtype=np.int32)
    s = seed & 0xFFFFFFFF
    lim = min(n_vocab, 150000)
    for i in range(count):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = (s >> 8) % lim
    return out


def write_gguf(path: str, spec: Spec, tensors) -> None:
    """Write a GGUF file that the reference's loader accepts (metadata keys of src/model.cpp:44-55)."""
    import gguf

    qt = {F32: None, F16: None, Q8_0: gguf.GGMLQuantizationType.Q8_0, Q4_K: gguf.GGMLQuantizationType.Q4_K,
          Q6_K: gguf.GGMLQuantizationType.Q6_K}
    w = gguf.GGUFWriter(path, "qwen3")
    w.add_block_count(spec.n_layer)
    w.add_embedding_length(spec.n_embd)
    w.add_feed_forward_length(spec.n_ff)
    w.add_head_count(spec.n_head)
    w.add_head_count_kv(spec.n_head_kv)
    w.add_key_length(spec.head_dim)
    w.add_value_length(spec.head_dim)
    w.add_rope_freq_base(spec.rope_base)
    w.add_layer_norm_rms_eps(spec.eps)
    w.add_context_length(40960)
    for role, layer, t, rows, n, data in tensors:
        name = f"{role}.weight" if layer < 0 else f"blk.{layer}.{role}.weight"
        if t == F32:
            arr = data.view(np.float32).reshape(-1) if rows == 1 else data.view(np.float32).reshape(rows, n)
            w.add_tensor(name, arr)
        elif t == F16:
            w.add_tensor(name, data.view(np.float16).reshape(rows, n))
        else:
            w.add_tensor(name, np.ascontiguousarray(data).reshape(rows, -1), raw_dtype=qt[t])
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
