"""ctypes loader for libnemotron_b200.so: one prototype per symbol in include/nemotron_b200.h.

There is no fallback: if the library is missing or a symbol is absent, loading
raises, and every operator in this package goes through this module.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libnemotron_b200.so")

_p = C.c_void_p
_i64 = C.c_int64
_f = C.c_float
_int = C.c_int

# name -> (restype, argtypes); mirrors include/nemotron_b200.h declaration by declaration.
PROTOTYPES = {
    "nmt_version": (C.c_char_p, []),
    "nmt_status_string": (C.c_char_p, [_int]),
    "nmt_last_cuda_error": (C.c_char_p, []),
    "nmt_set_device": (_int, [_int]),
    "nmt_device_synchronize": (_int, []),
    "nmt_rmsnorm_f32": (_int, [_p, _p, _p, _i64, _i64, _f, _p]),
    "nmt_rmsnorm_bf16": (_int, [_p, _p, _p, _i64, _i64, _f, _p]),
    "nmt_add_rmsnorm_bf16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _f, _p]),
    "nmt_fuse_next_norm": (_int, [_p, _f]),
    "nmt_fusion_reset": (_int, []),
    "nmt_fusion_counters": (_int, [C.POINTER(_i64), C.POINTER(_i64)]),
    "nmt_block_head_rmsnorm_bf16": (_int, [_p, _p, _p, _i64, _i64, _f, _p]),
    "nmt_block_tail_add_bf16": (_int, [_p, _p, _p, _i64, _p]),
    "nmt_rmsnorm_gated_bf16": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _f, _p]),
    "nmt_rmsnorm_gated_f32": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _f, _p]),
    "nmt_relu2_bf16": (_int, [_p, _p, _i64, _p]),
    "nmt_gemv_w8a16_fused_conv_step": (_int, [_p, _p, _f, _p, _p, _p, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _p]),
    "nmt_gemv_w8a16_gated": (_int, [_p, _p, _p, _f, _i64, _p, _p, _p, _p, _i64, _i64, _p]),
    "nmt_sdpa_decode_workspace_bytes": (_i64, [_i64, _i64]),
    "nmt_sdpa_decode_bf16": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p, _p]),
    "nmt_ssm_decode_step_bf16": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _f, _f, _p]),
    "nmt_relu2_f32": (_int, [_p, _p, _i64, _p]),
    "nmt_add_bf16": (_int, [_p, _p, _p, _i64, _p]),
    "nmt_add_f32": (_int, [_p, _p, _p, _i64, _p]),
    "nmt_embedding_bf16_i64": (_int, [_p, _p, _p, _i64, _i64, _i64, _p, _p]),
    "nmt_embedding_bf16_i32": (_int, [_p, _p, _p, _i64, _i64, _i64, _p, _p]),
    "nmt_causal_conv1d_silu_split_bf16": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _i64, _i64, _p]),
    "nmt_causal_conv1d_silu_decode_split_bf16": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _i64, _p]),
    "nmt_causal_conv1d_silu_f32": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p]),
    "nmt_gemv_w8a16": (_int, [_p, _p, _p, _p, _i64, _i64, _p]),
    "nmt_gemv_w8a16_fused": (_int, [_p, _p, _f, _p, _p, _int, _p, _p, _i64, _i64, _p]),
    "nmt_quantize_fp8": (_int, [_p, _p, _p, _p, _i64, _p]),
    "nmt_relu2_quant_fp8": (_int, [_p, _p, _p, _p, _i64, _p]),
    "nmt_fp8_workspace_bytes": (_i64, [_i64]),
    "nmt_rmsnorm_quant_fp8": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _f, _p]),
    "nmt_add_rmsnorm_quant_fp8": (_int, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _f, _p]),
    "nmt_rmsnorm_gated_quant_fp8": (_int, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _f, _p]),
    "nmt_add_rmsnorm_quant_fp8_static": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _f, _p]),
    "nmt_tune_set": (_int, [C.c_char_p, _int]),
    "nmt_tune_get": (_int, [C.c_char_p, C.POINTER(_int)]),
    "nmt_selftest_wait_runs_out": (_int, [_int, _p, _p]),
    "nmt_launch_count": (_i64, []),
    "nmt_device_wait_timeouts": (_i64, []),
}

_lock = threading.Lock()
_lib = None


class NemotronB200Error(RuntimeError):
    """Raised when a C-ABI call returns a non-zero nmt_status."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def load() -> C.CDLL:
    """Loads the library once and binds every prototype; raises if anything is missing."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: run `python -m nemotron_infer_b200.build` "
                "(the package has no CPU or PyTorch fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)          # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib


def check(status: int, what: str) -> None:
    if status != 0:
        lib = load()
        msg = lib.nmt_status_string(status).decode()
        if status == 4:
            msg += ": " + lib.nmt_last_cuda_error().decode()
        raise NemotronB200Error(status, f"{what}: {msg}")
