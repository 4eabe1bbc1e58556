"""ctypes binding of libelb.so (include/elb.h). The library is built in-tree by exactinfer_b200.build; loading it
fails loudly when it is missing — there is no CPU fallback."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libelb.so")

OK, ERR_CUDA, ERR_INVALID, ERR_RANGE, ERR_UNSUPPORTED, ERR_MEMORY, ERR_STATE = range(7)
W_PLANES, W_PAIR = 1, 2


class Config(C.Structure):
    """elb_config (mirrors el::Config of the reference, src/model.h:17-23)"""
    _fields_ = [("n_layer", C.c_int32), ("n_embd", C.c_int32), ("n_ff", C.c_int32), ("n_head", C.c_int32),
                ("n_head_kv", C.c_int32), ("head_dim", C.c_int32), ("n_vocab", C.c_int32), ("rope_dim", C.c_int32),
                ("rope_base", C.c_double), ("eps", C.c_float), ("max_batch", C.c_int32), ("n_seq", C.c_int32)]


_f32p, _i8p, _i32p = C.POINTER(C.c_float), C.POINTER(C.c_int8), C.POINTER(C.c_int32)
_vp = C.c_void_p
_i64p = C.POINTER(C.c_int64)

SIGNATURES = {
    "elb_last_error": (C.c_char_p, []),
    "elb_device_count": (C.c_int, []),
    "elb_malloc": (C.c_int, [C.c_int, C.c_size_t, C.POINTER(_vp)]),
    "elb_free": (C.c_int, [_vp]),
    "elb_host_alloc": (C.c_int, [C.c_size_t, C.POINTER(_vp)]),
    "elb_host_free": (C.c_int, [_vp]),
    "elb_memcpy_h2d": (C.c_int, [_vp, _vp, C.c_size_t]),
    "elb_memcpy_d2h": (C.c_int, [_vp, _vp, C.c_size_t]),
    "elb_device_sync": (C.c_int, [C.c_int]),
    "elb_device_mem_info": (C.c_int, [C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "elb_selftest_wait_expiry": (C.c_int, [C.c_int]),
    "elb_weight_create": (C.c_int, [C.c_int, C.c_int, C.c_int64, C.c_int64, _vp, C.c_size_t, C.c_int, C.POINTER(_vp)]),
    "elb_weight_destroy": (None, [_vp]),
    "elb_weight_rows": (C.c_int64, [_vp]),
    "elb_weight_cols": (C.c_int64, [_vp]),
    "elb_weight_device_bytes": (C.c_size_t, [_vp]),
    "elb_get_rows": (C.c_int, [_vp, C.c_int64, C.c_int64, _f32p]),
    "elb_get_rows_dev": (C.c_int, [_vp, C.c_int64, C.c_int64, _vp]),
    "elb_matvec": (C.c_int, [_vp, _f32p, _f32p, C.c_int]),
    "elb_matvec_dev": (C.c_int, [_vp, _vp, _vp, C.c_int]),
    "elb_matvec_static": (C.c_int, [_vp, _vp, _vp, C.c_int]),
    "elb_matmul": (C.c_int, [_vp, _f32p, C.c_int64, _f32p, C.c_int]),
    "elb_matmul_dev": (C.c_int, [_vp, _vp, C.c_int64, _vp, C.c_int]),
    "elb_rmsnorm": (C.c_int, [_f32p, _f32p, _f32p, C.c_int, C.c_float, C.c_int]),
    "elb_split_limbs": (C.c_int, [C.c_int, _f32p, C.c_int64, C.c_int64, C.c_int, _i8p, _f32p]),
    "elb_limb_sums": (C.c_int, [_vp, _f32p, C.c_int, _i32p, _i32p, _i32p]),
    "elb_matmul_acc": (C.c_int, [_vp, _f32p, C.c_int64, C.c_int, _i32p]),
    "elb_model_create": (C.c_int, [C.POINTER(Config), C.c_int, C.c_int, C.POINTER(_vp)]),
    "elb_model_set_tensor": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, _vp, C.c_size_t]),
    "elb_model_finalize": (C.c_int, [_vp]),
    "elb_model_load_gguf": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(_vp)]),
    "elb_model_config": (C.c_int, [_vp, C.POINTER(Config)]),
    "elb_model_destroy": (None, [_vp]),
    "elb_model_eval": (C.c_int, [_vp, _i32p, C.c_int, C.c_int, _vp]),
    "elb_model_eval_top": (C.c_int, [_vp, _i32p, C.c_int, C.c_int, C.c_int, _i32p, _f32p, C.POINTER(C.c_double)]),
    "elb_model_eval_top_masked": (C.c_int, [_vp, _i32p, C.c_int, C.c_int, C.c_int, _vp, _i32p, _f32p, C.POINTER(C.c_double)]),
    "elb_model_eval_batch": (C.c_int, [_vp, C.c_int, _i32p, _i32p, _i32p, _vp, _vp]),
    "elb_model_eval_batch_top": (C.c_int, [_vp, C.c_int, _i32p, _i32p, _i32p, _vp, C.c_int, _i32p, _f32p, C.POINTER(C.c_double)]),
    "elb_model_eval_steps": (C.c_int, [_vp, _i32p, C.c_int, C.c_int, _f32p]),
    "elb_model_last_eval_stats": (C.c_int, [_vp, _f32p, C.POINTER(C.c_int64)]),
    "elb_model_hidden": (C.c_int, [_vp, _f32p]),
    "elb_model_weight_bytes": (C.c_size_t, [_vp]),
    "elb_model_kv_bytes_per_token": (C.c_size_t, [_vp]),
    "elb_tp_dims": (C.c_int, [C.POINTER(Config), C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), _i64p, _i64p,
                              _i64p, _i64p]),
    "elb_tp_shard_shape": (C.c_int, [C.POINTER(Config), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, _i64p,
                                     _i64p, C.POINTER(C.c_size_t)]),
    "elb_tp_shard_copy": (C.c_int, [C.POINTER(Config), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, _vp,
                                    C.c_size_t, _vp, C.c_size_t]),
    "elb_tp_unique_id": (C.c_int, [_vp]),
    "elb_model_create_tp": (C.c_int, [C.POINTER(Config), C.c_int, C.c_int, C.c_int, C.c_int, _vp, C.POINTER(_vp)]),
    "elb_model_load_gguf_tp": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, C.POINTER(_vp)]),
    "elb_bench_matvec": (C.c_int, [C.POINTER(_vp), C.c_int, _vp, _vp, C.c_int, C.c_int, _f32p]),
    "elb_bench_matmul": (C.c_int, [C.POINTER(_vp), C.c_int, _vp, C.c_int64, _vp, C.c_int, C.c_int, _f32p]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m exactinfer_b200.build` "
                               "(there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


class ElbError(RuntimeError):
    pass


def check(rc: int):
    """Status code -> the exception type the reference throws for the same condition (src/cuda/model_cuda.cu:1649-1652)."""
    if rc == OK:
        return
    msg = lib().elb_last_error().decode(errors="replace")
    if rc == ERR_INVALID:
        raise ValueError(msg)           # std::invalid_argument
    if rc == ERR_RANGE:
        raise IndexError(msg)           # std::out_of_range
    if rc == ERR_MEMORY:
        raise MemoryError(msg)
    raise ElbError(f"[{rc}] {msg}")     # std::runtime_error


def fptr(a: np.ndarray):
    return a.ctypes.data_as(_f32p)
