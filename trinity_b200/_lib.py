"""ctypes binding of libtrinity_b200.so (include/trinity_b200.h).  There is no fallback: if the
library is missing or does not load, importing this module raises."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtrinity_b200.so")

F16, BF16, F32 = 0, 1, 2
ATTN_PRENORM, ATTN_QKNORM, ATTN_CAUSAL, ATTN_KEYFORMER, ATTN_ROCO, ATTN_ROCO_VARIANCE, ATTN_NORM_FOLDED = 1, 2, 4, 8, 16, 32, 64
FFN_SWIGLU, FFN_GELU = 0, 1
FFN_NORM, FFN_FALCON_TAIL, FFN_NORM_FOLDED = 1, 2, 4


class GemmArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("act", C.c_int),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("a", C.c_void_p), ("b", C.c_void_p), ("b2", C.c_void_p), ("c", C.c_void_p),
        ("row_scale", C.c_void_p), ("residual", C.c_void_p),
        ("split_k", C.c_int), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class AttnArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("flags", C.c_int),
        ("batch", C.c_int), ("seq", C.c_int), ("hidden", C.c_int),
        ("n_q_heads", C.c_int), ("n_kv_heads", C.c_int), ("head_dim", C.c_int),
        ("past", C.c_int), ("cache_len", C.c_int),
        ("sm_scale", C.c_float), ("norm_eps", C.c_float), ("qk_eps", C.c_float), ("tau", C.c_float),
        ("x", C.c_void_p), ("wq", C.c_void_p), ("wk", C.c_void_p), ("wv", C.c_void_p),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("o2", C.c_void_p),
        ("norm_weight", C.c_void_p), ("q_norm_weight", C.c_void_p), ("k_norm_weight", C.c_void_p),
        ("noise", C.c_void_p), ("c_out", C.c_void_p), ("c_out1", C.c_void_p), ("c_out2", C.c_void_p),
        ("aux_dtype", C.c_int), ("topk", C.c_int), ("topk_idx", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class FfnArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("act", C.c_int), ("flags", C.c_int),
        ("tokens", C.c_int64), ("hidden", C.c_int64), ("inner", C.c_int64),
        ("norm_eps", C.c_float), ("tail_divisor", C.c_int),
        ("x", C.c_void_p), ("o2", C.c_void_p), ("wo", C.c_void_p), ("norm_weight", C.c_void_p),
        ("w_gate", C.c_void_p), ("w_up", C.c_void_p), ("w_down", C.c_void_p),
        ("ff2", C.c_void_p), ("attn_o2", C.c_void_p), ("ff1", C.c_void_p), ("o_ff_norm", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class PeerGemmArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("world", C.c_int), ("rank", C.c_int),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("a", C.c_void_p), ("b", C.c_void_p), ("residual", C.c_void_p),
        ("stage", C.c_void_p * 8), ("out", C.c_void_p * 8), ("sync", C.c_void_p * 8),
        ("epoch", C.c_uint32),
    ]


class KvCompactArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("rows", C.c_int), ("head_dim", C.c_int), ("kv_len", C.c_int),
        ("src_cache_len", C.c_int), ("dst_cache_len", C.c_int), ("n_idx", C.c_int), ("keep_recent", C.c_int),
        ("idx", C.c_void_p), ("k_src", C.c_void_p), ("v_src", C.c_void_p), ("k_dst", C.c_void_p), ("v_dst", C.c_void_p),
        ("kept_pos", C.c_void_p), ("new_len", C.c_void_p),
    ]


# every symbol include/trinity_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "tb200_strerror": (C.c_char_p, [C.c_int]),
    "tb200_version": (C.c_int, []),
    "tb200_device_status": (C.c_int, [C.POINTER(C.c_int)]),
    "tb200_set_wait_limit_cycles": (C.c_int, [C.c_longlong]),
    "tb200_get_wait_limit_cycles": (C.c_longlong, []),
    "tb200_set_chained_launch": (C.c_int, [C.c_int]),
    "tb200_selftest_wait_timeout": (C.c_int, [C.c_longlong, C.c_void_p]),
    "tb200_gemm_check": (C.c_int, [C.POINTER(GemmArgs)]),
    "tb200_attn_check": (C.c_int, [C.POINTER(AttnArgs)]),
    "tb200_ffn_check": (C.c_int, [C.POINTER(FfnArgs)]),
    "tb200_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_int, C.c_void_p]),
    "tb200_fold_norm_weight": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "tb200_gemm_workspace_bytes": (C.c_size_t, [C.POINTER(GemmArgs)]),
    "tb200_gemm": (C.c_int, [C.POINTER(GemmArgs), C.c_void_p]),
    "tb200_gemm_static_scratch": (C.c_int, [C.POINTER(GemmArgs), C.c_void_p]),
    "tb200_peer_stage_bytes": (C.c_size_t, [C.c_int64, C.c_int64]),
    "tb200_peer_sync_bytes": (C.c_size_t, [C.c_int64, C.c_int]),
    "tb200_gemm_peer_reduce": (C.c_int, [C.POINTER(PeerGemmArgs), C.c_void_p]),
    "tb200_ipc_export": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]),
    "tb200_ipc_open": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_void_p)]),
    "tb200_ipc_close": (C.c_int, [C.c_void_p, C.c_int64]),
    "tb200_attn_workspace_bytes": (C.c_size_t, [C.POINTER(AttnArgs)]),
    "tb200_attn_forward": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "tb200_attn_forward_timed": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p, C.POINTER(C.c_float)]),
    "tb200_ffn_workspace_bytes": (C.c_size_t, [C.POINTER(FfnArgs)]),
    "tb200_ffn_forward": (C.c_int, [C.POINTER(FfnArgs), C.c_void_p]),
    "tb200_layer_forward": (C.c_int, [C.POINTER(AttnArgs), C.POINTER(FfnArgs), C.c_void_p]),
    "tb200_topk": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "tb200_kv_compact_max_keep": (C.c_int64, [C.POINTER(KvCompactArgs)]),
    "tb200_kv_compact": (C.c_int, [C.POINTER(KvCompactArgs), C.c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m trinity_b200.build` (nvcc, sm_100a). "
                "trinity_b200 has no CPU or PyTorch fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class Tb200Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = load().tb200_strerror(status).decode()
        super().__init__(f"{where}: {msg} (status {status})")


def check(status: int, where: str) -> None:
    if status != 0:
        raise Tb200Error(status, where)
