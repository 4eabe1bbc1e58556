"""ctypes access to the CPU oracle (oracle/liboracle.so) and, when present, to the reference's own CPU path
compiled unmodified (oracle/_ref/libelref.so). Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
_f32p = C.POINTER(C.c_float)
_i8p = C.POINTER(C.c_int8)
_i32p = C.POINTER(C.c_int32)
_u8p = C.POINTER(C.c_uint8)


def _ptr(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def build_oracle() -> str:
    so = os.path.join(ORACLE_DIR, "liboracle.so")
    src = os.path.join(ORACLE_DIR, "oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", ORACLE_DIR, "oracle"], check=True, capture_output=True)
    return so


_oracle = None
_ref = None


def oracle():
    global _oracle
    if _oracle is None:
        L = C.CDLL(build_oracle())
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_dequant_rows.argtypes = [C.c_int, C.c_int64, C.c_int64, _u8p, C.c_int64, C.c_int64, _f32p]
        L.orc_matvec.argtypes = [C.c_int, C.c_int64, C.c_int64, _u8p, _f32p, _f32p]
        L.orc_rmsnorm.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_float]
        L.orc_rope.argtypes = [_f32p, C.c_int, C.c_int, C.c_double]
        L.orc_rope_table.argtypes = [_f32p, C.c_int, C.c_int, C.c_double]
        L.orc_q4k_scale_min.argtypes = [C.c_int, _u8p, C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.orc_model_create.restype = C.c_void_p
        L.orc_model_create.argtypes = [C.POINTER(C.c_int), C.c_double, C.c_float, C.c_int]
        L.orc_model_set_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, _u8p]
        L.orc_model_eval.argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int, _f32p]
        L.orc_model_hidden.restype = _f32p
        L.orc_model_hidden.argtypes = [C.c_void_p]
        L.orc_model_destroy.argtypes = [C.c_void_p]
        L.orc_logsumexp.restype = C.c_double
        L.orc_logsumexp.argtypes = [_f32p, C.c_int]
        L.orc_split_limbs.argtypes = [_f32p, C.c_int64, C.c_int, _i8p, _f32p, C.POINTER(C.c_int)]
        L.orc_limb_partials.argtypes = [C.c_int, C.c_int64, C.c_int64, _u8p, _i8p, C.c_int, _i32p]
        L.orc_limb_block_sums.argtypes = [C.c_int, C.c_int64, C.c_int64, _u8p, _i8p, C.c_int, _i32p, _i32p]
        L.orc_set_threads.argtypes = [C.c_int]
        L.orc_threads.restype = C.c_int
        _oracle = L
    return _oracle


def ref_path() -> str:
    return os.path.join(ORACLE_DIR, "_ref", "libelref.so")


def have_ref() -> bool:
    return os.path.exists(ref_path())


def ref():
    global _ref
    if _ref is None:
        L = C.CDLL(ref_path())
        L.ref_last_error.restype = C.c_char_p
        L.ref_dequant_rows.argtypes = [C.c_int, C.c_int64, C.c_int64, _u8p, C.c_uint64, C.c_int64, C.c_int64, _f32p]
        L.ref_matvec.argtypes = [C.c_int, C.c_int64, C.c_int64, _u8p, C.c_uint64, _f32p, _f32p]
        L.ref_rmsnorm.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_float]
        L.ref_q4k_scale_min.argtypes = [C.c_int, _u8p, C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.ref_model_open.restype = C.c_void_p
        L.ref_model_open.argtypes = [C.c_char_p, C.c_int]
        L.ref_model_config.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
        L.ref_model_eval.argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int, _f32p]
        L.ref_model_close.argtypes = [C.c_void_p]
        L.ref_set_threads.argtypes = [C.c_int]
        L.ref_threads.restype = C.c_int
        _ref = L
    return _ref


# ---------------------------------------------------------------- numpy-level helpers (oracle)

def _bytes2d(w: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(w, dtype=np.uint8)


def dequant_rows(t, rows_total, n, w, row0=0, rows=None, lib="oracle"):
    w = _bytes2d(w)
    rows = rows_total - row0 if rows is None else rows
    out = np.empty((rows, n), dtype=np.float32)
    if lib == "oracle":
        rc = oracle().orc_dequant_rows(t, rows_total, n, _ptr(w, _u8p), row0, rows, _ptr(out, _f32p))
    else:
        rc = ref().ref_dequant_rows(t, rows_total, n, _ptr(w, _u8p), w.nbytes, row0, rows, _ptr(out, _f32p))
    if rc:
        raise RuntimeError(f"dequant_rows rc={rc}")
    return out


def matvec(t, rows, n, w, x, lib="oracle"):
    w = _bytes2d(w)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(rows, dtype=np.float32)
    if lib == "oracle":
        rc = oracle().orc_matvec(t, rows, n, _ptr(w, _u8p), _ptr(x, _f32p), _ptr(y, _f32p))
    else:
        rc = ref().ref_matvec(t, rows, n, _ptr(w, _u8p), w.nbytes, _ptr(x, _f32p), _ptr(y, _f32p))
    if rc:
        raise RuntimeError(f"matvec rc={rc}")
    return y


def rmsnorm(x, w, eps, lib="oracle"):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty_like(x)
    f = oracle().orc_rmsnorm if lib == "oracle" else ref().ref_rmsnorm
    f(_ptr(out, _f32p), _ptr(x, _f32p), _ptr(w, _f32p), x.size, eps)
    return out


def rope(v, pos, dim, base):
    v = np.array(v, dtype=np.float32, copy=True)
    oracle().orc_rope(_ptr(v, _f32p), pos, dim, base)
    return v


def split_limbs(x, nl):
    x = np.ascontiguousarray(x, dtype=np.float32)
    limbs = np.empty((nl, x.size), dtype=np.int8)
    inv = C.c_float()
    k = C.c_int()
    oracle().orc_split_limbs(_ptr(x, _f32p), x.size, nl, _ptr(limbs, _i8p), C.byref(inv), C.byref(k))
    return limbs, inv.value, k.value


def limb_partials(t, rows, n, w, limbs):
    w = _bytes2d(w)
    nl = limbs.shape[0]
    sub = 16 if t == 14 else 32
    P = np.empty((rows, n // sub, nl), dtype=np.int32)
    rc = oracle().orc_limb_partials(t, rows, n, _ptr(w, _u8p), _ptr(np.ascontiguousarray(limbs), _i8p), nl,
                                    _ptr(P, _i32p))
    if rc:
        raise RuntimeError("limb_partials: unsupported type")
    return P


def limb_block_sums(t, rows, n, w, limbs):
    w = _bytes2d(w)
    nl = limbs.shape[0]
    blk = 32 if t == 8 else 256
    I = np.empty((rows, n // blk, nl), dtype=np.int32)
    J = np.empty_like(I)
    rc = oracle().orc_limb_block_sums(t, rows, n, _ptr(w, _u8p), _ptr(np.ascontiguousarray(limbs), _i8p), nl,
                                      _ptr(I, _i32p), _ptr(J, _i32p))
    if rc:
        raise RuntimeError("limb_block_sums: unsupported type")
    return I, J


def logsumexp(logits):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    return oracle().orc_logsumexp(_ptr(logits, _f32p), logits.size)


class OracleModel:
    """The restated CpuModel (src/model.cpp:115-234) fed with raw tensors."""

    def __init__(self, spec, tensors, n_ctx):
        from exactinfer_b200 import synth

        self.spec, self.n_ctx = spec, n_ctx
        cfg = (C.c_int * 8)(spec.n_layer, spec.n_embd, spec.n_ff, spec.n_head, spec.n_head_kv, spec.head_dim,
                            spec.n_vocab, spec.head_dim)
        self._h = oracle().orc_model_create(cfg, spec.rope_base, spec.eps, n_ctx)
        self._keep = []
        for role, layer, t, rows, n, data in tensors:
            data = _bytes2d(data)
            self._keep.append(data)
            rc = oracle().orc_model_set_tensor(self._h, synth.ROLE_ID[role], max(layer, 0), t, rows, n,
                                               _ptr(data, _u8p))
            assert rc == 0, (role, layer)

    def eval(self, tokens, pos0, want_logits=True):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.spec.n_vocab, dtype=np.float32) if want_logits else None
        rc = oracle().orc_model_eval(self._h, _ptr(tokens, _i32p), tokens.size, pos0,
                                     _ptr(logits, _f32p) if want_logits else None)
        if rc:
            raise IndexError(f"oracle eval rc={rc}")
        return logits

    def hidden(self):
        return np.ctypeslib.as_array(oracle().orc_model_hidden(self._h), shape=(self.spec.n_embd,)).copy()

    def close(self):
        if self._h:
            oracle().orc_model_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()


class RefModel:
    """The reference's make_cpu_backend over a GGUF file (needs oracle/_ref/libelref.so)."""

    def __init__(self, gguf_path, n_ctx):
        self._h = ref().ref_model_open(gguf_path.encode(), n_ctx)
        if not self._h:
            raise RuntimeError(ref().ref_last_error().decode(errors="replace"))
        cfg = (C.c_int * 10)()
        ref().ref_model_config(self._h, cfg)
        self.n_vocab = cfg[6]

    def eval(self, tokens, pos0, want_logits=True):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.n_vocab, dtype=np.float32) if want_logits else None
        rc = ref().ref_model_eval(self._h, _ptr(tokens, _i32p), tokens.size, pos0,
                                  _ptr(logits, _f32p) if want_logits else None)
        if rc:
            raise IndexError(f"reference eval rc={rc}: {ref().ref_last_error().decode(errors='replace')}")
        return logits

    def close(self):
        if self._h:
            ref().ref_model_close(self._h)
            self._h = None

    def __del__(self):
        self.close()
