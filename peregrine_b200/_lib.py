"""ctypes binding of libperegrine_b200.so (the declarations of include/peregrine_b200.h).

There is no fallback of any kind: if the library is missing, cannot be loaded, or a call
fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libperegrine_b200.so")

PG_OK = 0
PG_ERR_INVALID = -1
PG_ERR_CUDA = -2
PG_ERR_NOMEM = -3
PG_ERR_UNSUPPORTED = -4
PG_ERR_DEVICE_TIMEOUT = -5

GGUF_Q4_0, GGUF_Q4_1, GGUF_Q8_0 = 2, 3, 8
ALGO_AUTO, ALGO_NAIVE, ALGO_STREAM, ALGO_TCGEN05, ALGO_WSTREAM = 0, 1, 2, 3, 4


class PeregrineError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[pg status {code}] {message}")
        self.code = code


class InvalidArgument(PeregrineError, AssertionError):
    """Raised where the reference `assert!`s / panics on a shape or argument."""


_vp = C.c_void_p
_i64 = C.c_int64
_i32 = C.c_int32
_sz = C.c_size_t

# name -> (restype, argtypes); every symbol include/peregrine_b200.h declares
SIGNATURES = {
    "pg_last_error": (C.c_char_p, []),
    "pg_version": (_i32, []),
    "pg_launch_count": (C.c_uint64, []),
    "pg_ctx_create": (_i32, [_i32, _vp, C.POINTER(_vp)]),
    "pg_ctx_destroy": (_i32, [_vp]),
    "pg_ctx_sync": (_i32, [_vp]),
    "pg_ctx_stream": (_vp, [_vp]),
    "pg_ctx_device_status": (_i32, [_vp, C.POINTER(_i32)]),
    "pg_ctx_set_wait_limit_ns": (_i32, [_vp, C.c_uint64]),
    "pg_ctx_scratch_bytes": (C.c_uint64, [_vp]),
    "pg_graph_begin": (_i32, [_vp]),
    "pg_graph_end": (_i32, [_vp, C.POINTER(_vp)]),
    "pg_graph_launch": (_i32, [_vp, _vp]),
    "pg_graph_free": (_i32, [_vp, _vp]),
    "pg_mem_alloc": (_i32, [_vp, _sz, C.POINTER(_vp)]),
    "pg_mem_free": (_i32, [_vp, _vp]),
    "pg_mem_upload": (_i32, [_vp, _vp, _vp, _sz]),
    "pg_mem_download": (_i32, [_vp, _vp, _vp, _sz]),
    "pg_quantize_activations": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "pg_quantize_activations_host": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "pg_quantize_weights": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "pg_quantize_weights_host": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "pg_dequantize": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "pg_qtensor_upload": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, C.POINTER(_vp)]),
    "pg_qtensor_wrap": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, C.POINTER(_vp)]),
    "pg_qtensor_from_f32": (_i32, [_vp, _vp, _i64, _i64, _i32, C.POINTER(_vp)]),
    "pg_qtensor_download": (_i32, [_vp, _vp, _vp, _vp, _vp]),
    "pg_qtensor_free": (_i32, [_vp, _vp]),
    "pg_qtensor_rows": (_i64, [_vp]),
    "pg_qtensor_cols": (_i64, [_vp]),
    "pg_qtensor_data_i8_t": (_vp, [_vp]),
    "pg_qtensor_scales": (_vp, [_vp]),
    "pg_matmul_quantized": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "pg_matmul_quantized_ex": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i32]),
    "pg_matmul_quantized_host": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "pg_matmul_dequant_w8a32": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _i32]),
    "pg_matmul_quantized_static": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "pg_static_scratch_bytes": (_i64, []),
    "pg_gemm_i8": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _i32]),
    "pg_dequant_blocks": (_i32, [_vp, _i32, _vp, _sz, _i64, _vp]),
    "pg_dequant_blocks_host": (_i32, [_vp, _i32, _vp, _sz, _i64, _vp]),
    "pg_f16_to_f32": (_i32, [_vp, _vp, _i64, _vp]),
    "pg_gguf_upload": (_i32, [_vp, _i32, _vp, _sz, _i64, _i64, _i64, _i64, C.POINTER(_vp)]),
    "pg_gguf_free": (_i32, [_vp, _vp]),
    "pg_gguf_rows": (_i64, [_vp]),
    "pg_gguf_cols": (_i64, [_vp]),
    "pg_matmul_gguf": (_i32, [_vp, _vp, _i64, _vp, _vp]),
    "pg_matmul_gguf_host": (_i32, [_vp, _vp, _i64, _vp, _vp]),
    "pg_qtensor_from_q8_0": (_i32, [_vp, _vp, _sz, _i64, _i64, C.POINTER(_vp)]),
    "pg_qtensor_from_i8": (_i32, [_vp, _vp, _vp, _i64, _i64, C.POINTER(_vp)]),
    "pg_huffman_decode_host": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _vp]),
    "pg_qtensor_from_huffman": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, C.POINTER(_vp)]),
    "pg_exchange_create": (_i32, [_vp, _i32, _i32, _sz, _vp, C.POINTER(_vp)]),
    "pg_exchange_connect": (_i32, [_vp, _vp, _vp]),
    "pg_exchange_result": (_vp, [_vp]),
    "pg_exchange_allgather": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64]),
    "pg_exchange_store": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64]),
    "pg_exchange_wait": (_i32, [_vp, _vp]),
    "pg_exchange_destroy": (_i32, [_vp, _vp]),
    "pg_exchange_connect_local": (_i32, [_vp, _vp, C.POINTER(_vp)]),
    "pg_exchange_gather": (_i32, [_vp, _vp, _i64, _i64, _vp]),
    "pg_exchange_gather_many": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32]),
    "pg_matmul_quantized_exchange": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _i64, _i64, _vp]),
    "pg_exchange_store_cells": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64]),
    "pg_gemm_i8_exchange": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp, _vp, _i64, _i64, _vp]),
    "pg_quantize_activations_exchange": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "pg_add_rmsnorm_quantize_exchange": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, C.c_float, _vp, _vp, _vp]),
    "pg_gqa_attention_decode_fused_exchange": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _i32, _vp, _i64, _i64]),
    "pg_swiglu_exchange": (_i32, [_vp, _vp, _i64, _i64, _vp, _i64, _i64]),
    "pg_argmax_exchange": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp]),
    "pg_pick_embed": (_i32, [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _i64, _vp]),
    "pg_add_rmsnorm_quantize": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, C.c_float, _vp, _vp, _vp]),
    "pg_swiglu_quantize": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "pg_rope_kv_append": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp]),
    "pg_gqa_decode_splits": (_i32, [_vp, _i64, _i64, _i64, _i64]),
    "pg_gqa_attention_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp]),
    "pg_gqa_attention_decode_fused": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp]),
    "pg_embedding": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "pg_argmax_advance": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _i64]),
    "pg_matmul_f32": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _vp]),
}

# the knobs of include/peregrine_b200_tune.h (tests and profiling runs; process-wide, not thread-safe)
_int = C.c_int
TUNE_SIGNATURES = {
    "pg_tune_stream_ng": (None, [_int]),
    "pg_tune_stream_depth": (None, [_int]),
    "pg_tune_stream_carveout": (None, [_int]),
    "pg_tune_stream_split": (None, [_int]),
    "pg_tune_wstream_kw": (None, [_int]),
    "pg_tune_wstream_cluster": (None, [_int]),
    "pg_tune_tcgen05_bn": (None, [_int]),
    "pg_tune_tcgen05_pair": (None, [_int]),
    "pg_tune_tcgen05_split": (None, [_int]),
    "pg_tune_gguf_simple": (None, [_int]),
    "pg_tune_host_direct": (None, [_int, _int]),
    "pg_tune_host_push": (None, [_int]),
    "pg_tune_host_graph": (None, [_int]),
    "pg_tune_exchange_solo": (None, [_int]),
    "pg_huffman_last_sweeps": (_int, []),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library (building it first if the sources are newer and nvcc exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        from . import build as _build

        _build.build()
    try:
        lib = C.CDLL(LIB_PATH)
    except OSError as e:  # loud, never silent
        raise ImportError(f"cannot load {LIB_PATH}: {e}. Build it with `python -m peregrine_b200.build`.") from e
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    for name, (res, args) in TUNE_SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int) -> None:
    if code == PG_OK:
        return
    msg = load().pg_last_error().decode("utf-8", "replace")
    if code == PG_ERR_INVALID:
        raise InvalidArgument(code, msg)
    raise PeregrineError(code, msg)
