"""exactinfer forward pass on B200 (sm_100a): Python host side over the C ABI of libelb.so.

`Weight` and the free functions mirror the reference's operator interface (src/ops.h:11-29: matvec, get_row, rmsnorm);
`Backend` mirrors el::Backend (src/model.h:42-51: cfg, n_ctx, name, eval). All arithmetic runs in the CUDA library.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import capi, synth
from .capi import Config, ElbError, check, lib

__all__ = ["Weight", "Backend", "cuda_available", "matvec", "get_row", "rmsnorm", "split_limbs", "synth", "Config",
           "ElbError"]


def cuda_available():
    """el::cuda_available (src/model.h:56): (ok, why)"""
    n = lib().elb_device_count()
    return (True, "") if n > 0 else (False, lib().elb_last_error().decode(errors="replace"))


class DeviceBuffer:
    def __init__(self, nbytes: int, device: int = 0):
        p = C.c_void_p()
        check(lib().elb_malloc(device, nbytes, C.byref(p)))
        self.ptr, self.nbytes = p, nbytes

    @classmethod
    def from_array(cls, a: np.ndarray, device: int = 0):
        a = np.ascontiguousarray(a)
        b = cls(a.nbytes, device)
        check(lib().elb_memcpy_h2d(b.ptr, a.ctypes.data_as(C.c_void_p), a.nbytes))
        return b

    def to_array(self, dtype, shape):
        out = np.empty(shape, dtype=dtype)
        check(lib().elb_memcpy_d2h(out.ctypes.data_as(C.c_void_p), self.ptr, out.nbytes))
        return out

    def free(self):
        if self.ptr:
            lib().elb_free(self.ptr)
            self.ptr = None

    def __del__(self):
        self.free()


class Weight:
    """One weight matrix in a ggml block format on the device (el::Tensor + upload_group of the reference)."""

    def __init__(self, ggml_type: int, rows: int, n: int, data: np.ndarray, planes: bool = False, pair: bool = False,
                 device: int = 0):
        data = np.ascontiguousarray(data, dtype=np.uint8)
        h = C.c_void_p()
        flags = (capi.W_PLANES if planes else 0) | (capi.W_PAIR if pair else 0)
        check(lib().elb_weight_create(device, ggml_type, rows, n, data.ctypes.data_as(C.c_void_p), data.nbytes, flags,
                                      C.byref(h)))
        self._h, self.type, self.device = h, ggml_type, device
        self.rows, self.n = lib().elb_weight_rows(h), lib().elb_weight_cols(h)

    @property
    def device_bytes(self):
        return lib().elb_weight_device_bytes(self._h)

    def get_rows(self, row0: int, count: int = 1) -> np.ndarray:
        out = np.empty((count, self.n), dtype=np.float32)
        check(lib().elb_get_rows(self._h, row0, count, capi.fptr(out)))
        return out

    def matvec(self, x: np.ndarray, nl: int = 4) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.size != self.n:
            raise ValueError("matvec: x has the wrong length")
        y = np.empty(self.rows, dtype=np.float32)
        check(lib().elb_matvec(self._h, capi.fptr(x), capi.fptr(y), nl))
        return y

    def matmul(self, x: np.ndarray, nl: int = 4) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        b = x.shape[0]
        y = np.empty((b, self.rows), dtype=np.float32)
        check(lib().elb_matmul(self._h, capi.fptr(x), b, capi.fptr(y), nl))
        return y

    def limb_sums(self, x: np.ndarray, nl: int = 4):
        x = np.ascontiguousarray(x, dtype=np.float32)
        sub = 16 if self.type == synth.Q6_K else 32
        blk = 32 if self.type == synth.Q8_0 else 256
        P = np.empty((self.rows, self.n // sub, nl), dtype=np.int32)
        I = np.empty((self.rows, self.n // blk, nl), dtype=np.int32)
        J = np.empty_like(I)
        ip = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
        check(lib().elb_limb_sums(self._h, capi.fptr(x), nl, ip(P), ip(I), ip(J)))
        return P, I, J

    def matmul_acc(self, x: np.ndarray, nl: int = 4) -> np.ndarray:
        """The int32 accumulator columns of the tensor-core limb GEMM, A[b][n/256][nl + 1][rows] (elb_matmul_acc)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        b = x.shape[0]
        A = np.empty((b, self.n // 256, nl + 1, self.rows), dtype=np.int32)
        check(lib().elb_matmul_acc(self._h, capi.fptr(x), b, nl, A.ctypes.data_as(C.POINTER(C.c_int32))))
        return A

    def close(self):
        if getattr(self, '_h', None):
            lib().elb_weight_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()


def matvec(w: Weight, x: np.ndarray, nl: int = 4) -> np.ndarray:
    """el::matvec (src/ops.h:23)"""
    return w.matvec(x, nl)


def get_row(w: Weight, row: int) -> np.ndarray:
    """el::get_row (src/ops.h:20)"""
    return w.get_rows(row, 1)[0]


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """el::rmsnorm (src/ops.h:26) over the last axis"""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    n = x.shape[-1]
    out = np.empty_like(x)
    check(lib().elb_rmsnorm(capi.fptr(out), capi.fptr(x), capi.fptr(w), n, eps, x.size // n))
    return out


def split_limbs(x: np.ndarray, nl: int, device: int = 0):
    """k_split8 of the reference: returns (limbs[nl][b][n] int8, inv_scale[b])"""
    x = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
    b, n = x.shape
    limbs = np.empty((nl, b, n), dtype=np.int8)
    inv = np.empty(b, dtype=np.float32)
    check(lib().elb_split_limbs(device, capi.fptr(x), b, n, nl, limbs.ctypes.data_as(C.POINTER(C.c_int8)), capi.fptr(inv)))
    return limbs, inv


def spec_config(spec: "synth.Spec", max_batch: int = 0, n_seq: int = 0) -> Config:
    return Config(spec.n_layer, spec.n_embd, spec.n_ff, spec.n_head, spec.n_head_kv, spec.head_dim, spec.n_vocab,
                  spec.head_dim, spec.rope_base, spec.eps, max_batch, n_seq)


def tp_unique_id() -> bytes:
    """128-byte NCCL id for Backend(tp=...): make it on one rank, hand it to the others."""
    buf = C.create_string_buffer(128)
    check(lib().elb_tp_unique_id(buf))
    return buf.raw


def tp_dims(spec: "synth.Spec", rank: int, size: int) -> dict:
    """This rank's share of the model: heads, FFN range [f0, f1), vocabulary rows [v0, v1). Host arithmetic only."""
    cfg = spec_config(spec)
    h, hkv = C.c_int(), C.c_int()
    f0, f1, v0, v1 = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64()
    check(lib().elb_tp_dims(C.byref(cfg), rank, size, C.byref(h), C.byref(hkv), C.byref(f0), C.byref(f1), C.byref(v0),
                            C.byref(v1)))
    return {"n_head": h.value, "n_head_kv": hkv.value, "f0": f0.value, "f1": f1.value, "v0": v0.value, "v1": v1.value}


def tp_shard(spec: "synth.Spec", rank: int, size: int, role: str, t: int, rows: int, n: int, data: np.ndarray):
    """Rank `rank`'s cut of one tensor of the whole model: (rows, n, bytes). Host arithmetic only."""
    cfg = spec_config(spec)
    data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    orows, on, nb = C.c_int64(), C.c_int64(), C.c_size_t()
    rid = synth.ROLE_ID[role]
    check(lib().elb_tp_shard_shape(C.byref(cfg), rank, size, rid, t, rows, n, C.byref(orows), C.byref(on), C.byref(nb)))
    out = np.empty(nb.value, dtype=np.uint8)
    check(lib().elb_tp_shard_copy(C.byref(cfg), rank, size, rid, t, rows, n, data.ctypes.data_as(C.c_void_p), data.nbytes,
                                  out.ctypes.data_as(C.c_void_p), out.nbytes))
    return orows.value, on.value, out


class Backend:
    """el::Backend (src/model.h:42-51) on the CUDA library: cfg(), n_ctx(), name(), eval(tokens, pos0) -> logits."""

    def __init__(self, spec: "synth.Spec", tensors, n_ctx: int, device: int = 0, max_batch: int = 0, tp=None,
                 n_seq: int = 0):
        """tp = (rank, size, id) makes this process rank `rank` of a tensor-parallel group of `size` GPUs; `id` is the
        128-byte value of tp_unique_id() made on one rank and given to all. `tensors` are the whole model's on every
        rank; eval must then be called by all ranks with the same arguments."""
        self.spec = spec
        self._cfg = spec_config(spec, max_batch, n_seq)
        self._n_ctx = n_ctx
        h = C.c_void_p()
        if tp is None or tp[1] == 1:
            check(lib().elb_model_create(C.byref(self._cfg), n_ctx, device, C.byref(h)))
        else:
            rank, size, ident = tp
            buf = C.create_string_buffer(bytes(ident), 128)
            check(lib().elb_model_create_tp(C.byref(self._cfg), n_ctx, device, rank, size, buf, C.byref(h)))
        self._h = h
        try:
            keep = []
            for role, layer, t, rows, n, data in tensors:
                data = np.ascontiguousarray(data, dtype=np.uint8)
                keep.append(data)  # bytes must stay valid until finalize
                check(lib().elb_model_set_tensor(h, synth.ROLE_ID[role], max(layer, 0), t, rows, n,
                                                 data.ctypes.data_as(C.c_void_p), data.nbytes))
            check(lib().elb_model_finalize(h))
        except Exception:
            self.close()
            raise
        self._logits_host = None

    @classmethod
    def from_gguf(cls, path: str, n_ctx: int, device: int = 0, max_batch: int = 0, n_seq: int = 0, tp=None):
        """The model of a GGUF file, read and uploaded by the library itself (elb_model_load_gguf); tp = (rank, size,
        id) makes this process one rank of a tensor-parallel group that loads the same file (elb_model_load_gguf_tp)."""
        h = C.c_void_p()
        if tp is None:
            check(lib().elb_model_load_gguf(os.fsencode(path), n_ctx, device, max_batch, n_seq, C.byref(h)))
        else:
            rank, size, ident = tp
            buf = C.create_string_buffer(bytes(ident), 128)
            check(lib().elb_model_load_gguf_tp(os.fsencode(path), n_ctx, device, max_batch, n_seq, rank, size, buf, C.byref(h)))
        self = cls.__new__(cls)
        self._h, self._n_ctx, self._logits_host = h, n_ctx, None
        self._cfg = Config()
        check(lib().elb_model_config(h, C.byref(self._cfg)))
        c = self._cfg
        self.spec = synth.Spec(name=os.path.basename(path), n_layer=c.n_layer, n_embd=c.n_embd, n_ff=c.n_ff, n_head=c.n_head,
                               n_head_kv=c.n_head_kv, n_vocab=c.n_vocab, layout="gguf", head_dim=c.head_dim,
                               rope_base=c.rope_base, eps=c.eps)
        return self

    def cfg(self):
        return self._cfg

    def n_ctx(self):
        return self._n_ctx

    def name(self):
        return "cuda-b200"

    def eval(self, tokens, pos0: int, want_logits: bool = True, out: np.ndarray | None = None):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = None
        if want_logits:
            logits = out if out is not None else np.empty(self.spec.n_vocab, dtype=np.float32)
        check(lib().elb_model_eval(self._h, tokens.ctypes.data_as(C.POINTER(C.c_int32)), tokens.size, pos0,
                                   logits.ctypes.data_as(C.c_void_p) if want_logits else None))
        return logits

    def eval_top(self, tokens, pos0: int, k: int = 1, allowed=None):
        """eval with the logits reduced on the device: (ids[k], logits[k], log-sum-exp) of the last token, ids ordered by
        (logit descending, id ascending); logprob of ids[i] = logits[i] - lse. allowed: boolean mask over the vocabulary
        (constrained decoding): only allowed tokens are picked, the log-sum-exp still covers all."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        ids, vals, lse = np.empty(k, np.int32), np.empty(k, np.float32), C.c_double()
        i32 = C.POINTER(C.c_int32)
        if allowed is None:
            check(lib().elb_model_eval_top(self._h, tokens.ctypes.data_as(i32), tokens.size, pos0, k, ids.ctypes.data_as(i32),
                                           capi.fptr(vals), C.byref(lse)))
        else:
            bits = np.packbits(np.asarray(allowed, dtype=bool), bitorder="little")
            words = np.zeros((self.spec.n_vocab + 31) // 32 * 4, np.uint8)
            words[:bits.size] = bits
            check(lib().elb_model_eval_top_masked(self._h, tokens.ctypes.data_as(i32), tokens.size, pos0, k,
                                                  words.ctypes.data_as(C.c_void_p), ids.ctypes.data_as(i32), capi.fptr(vals),
                                                  C.byref(lse)))
        return ids, vals, lse.value

    def eval_batch(self, tokens, seq, pos, want=None, want_logits: bool = True):
        """Rows of several sequences in one pass: row i is tokens[i] at position pos[i] of sequence seq[i] (n_seq given at
        construction). Returns one row of logits per wanted row (want: boolean mask, default all rows), or None."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        seq = np.ascontiguousarray(seq, dtype=np.int32)
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        n = tokens.size
        w = None if want is None else np.ascontiguousarray(want, dtype=np.uint8)
        n_out = n if w is None else int(np.count_nonzero(w))
        out = np.empty((n_out, self.spec.n_vocab), dtype=np.float32) if want_logits else None
        i32 = C.POINTER(C.c_int32)
        check(lib().elb_model_eval_batch(self._h, n, tokens.ctypes.data_as(i32), seq.ctypes.data_as(i32), pos.ctypes.data_as(i32),
                                         w.ctypes.data_as(C.c_void_p) if w is not None else None,
                                         out.ctypes.data_as(C.c_void_p) if want_logits else None))
        return out

    def eval_batch_top(self, tokens, seq, pos, k: int = 1, want=None):
        """eval_batch with every wanted row reduced on the device: (ids[R][k], logits[R][k], lse[R])."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        seq = np.ascontiguousarray(seq, dtype=np.int32)
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        n = tokens.size
        w = None if want is None else np.ascontiguousarray(want, dtype=np.uint8)
        R = n if w is None else int(np.count_nonzero(w))
        ids, vals, lse = np.empty((R, k), np.int32), np.empty((R, k), np.float32), np.empty(R, np.float64)
        i32 = C.POINTER(C.c_int32)
        check(lib().elb_model_eval_batch_top(self._h, n, tokens.ctypes.data_as(i32), seq.ctypes.data_as(i32), pos.ctypes.data_as(i32),
                                             w.ctypes.data_as(C.c_void_p) if w is not None else None, k, ids.ctypes.data_as(i32),
                                             capi.fptr(vals), lse.ctypes.data_as(C.POINTER(C.c_double))))
        return ids, vals, lse

    def eval_steps(self, tokens, pos0: int) -> float:
        """Single-token steps back to back, logits left on the device; returns the device time in ms."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        ms = C.c_float()
        check(lib().elb_model_eval_steps(self._h, tokens.ctypes.data_as(C.POINTER(C.c_int32)), tokens.size, pos0,
                                         C.byref(ms)))
        return ms.value

    def last_eval_stats(self):
        ms, n = C.c_float(), C.c_int64()
        check(lib().elb_model_last_eval_stats(self._h, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def hidden(self):
        out = np.empty(self.spec.n_embd, dtype=np.float32)
        check(lib().elb_model_hidden(self._h, capi.fptr(out)))
        return out

    @property
    def weight_bytes(self):
        return lib().elb_model_weight_bytes(self._h)

    @property
    def kv_bytes_per_token(self):
        return lib().elb_model_kv_bytes_per_token(self._h)

    def close(self):
        if getattr(self, "_h", None):
            lib().elb_model_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()
