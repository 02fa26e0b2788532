"""ctypes binding of the C ABI in ``include/mk36.h`` (libmk36.so).

The PyTorch extension ``_C`` is the normal way into the kernels; this module binds the same
entry points without any torch type in between, for callers that only have device pointers and
for tests that want to exercise the C ABI itself.  Structure layouts mirror mk36.h field by field.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

MK36_BF16, MK36_F16, MK36_F32 = 0, 1, 2
MK36_OK = 0
MK36_ERR_INVALID_ARG, MK36_ERR_UNSUPPORTED, MK36_ERR_LAUNCH = -1, -2, -3
MK36_ERR_WORKSPACE, MK36_ERR_BARRIER_TIMEOUT = -4, -5

LIBRARY_NAME = "libmk36.so"


class MoeArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("norm_weight", C.c_void_p), ("router_weight", C.c_void_p),
        ("expert_gate", C.c_void_p), ("expert_up", C.c_void_p), ("expert_down", C.c_void_p),
        ("shared_gate", C.c_void_p), ("shared_up", C.c_void_p), ("shared_down", C.c_void_p),
        ("out", C.c_void_p), ("indices", C.c_void_p), ("route_weights", C.c_void_p),
        ("partial_out", C.c_void_p),
        ("dtype", C.c_int32), ("batch", C.c_int32), ("hidden", C.c_int32), ("experts", C.c_int32),
        ("top_k", C.c_int32), ("intermediate", C.c_int32), ("shared_intermediate", C.c_int32),
        ("expert_base", C.c_int32), ("local_experts", C.c_int32), ("add_residual", C.c_int32),
        ("eps", C.c_float),
    ]


class DenseFfnArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("norm_weight", C.c_void_p), ("gate_weight", C.c_void_p),
        ("up_weight", C.c_void_p), ("down_weight", C.c_void_p), ("out", C.c_void_p),
        ("partial_out", C.c_void_p),
        ("dtype", C.c_int32), ("batch", C.c_int32), ("hidden", C.c_int32), ("intermediate", C.c_int32),
        ("add_residual", C.c_int32), ("eps", C.c_float),
    ]


class LinearArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("norm_weight", C.c_void_p), ("weight", C.c_void_p), ("residual", C.c_void_p),
        ("out", C.c_void_p), ("argmax", C.c_void_p),
        ("dtype", C.c_int32), ("batch", C.c_int32), ("in_features", C.c_int32), ("out_features", C.c_int32),
        ("eps", C.c_float),
    ]


class AttentionArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("out", C.c_void_p),
        ("dtype", C.c_int32), ("batch", C.c_int32), ("query_heads", C.c_int32), ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("seq_len", C.c_int32), ("scale", C.c_float),
    ]


class LinearAttentionArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("state", C.c_void_p),
        ("out", C.c_void_p), ("new_state", C.c_void_p), ("decay_per_head", C.c_void_p),
        ("beta_per_head", C.c_void_p),
        ("dtype", C.c_int32), ("batch", C.c_int32), ("key_heads", C.c_int32), ("value_heads", C.c_int32),
        ("key_dim", C.c_int32), ("value_dim", C.c_int32), ("decay", C.c_float),
    ]


class LinearAttentionStepsArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("state", C.c_void_p),
        ("out", C.c_void_p), ("new_state", C.c_void_p), ("decay_per_step", C.c_void_p),
        ("beta_per_step", C.c_void_p),
        ("dtype", C.c_int32), ("steps", C.c_int32), ("batch", C.c_int32), ("key_heads", C.c_int32),
        ("value_heads", C.c_int32), ("key_dim", C.c_int32), ("value_dim", C.c_int32), ("decay", C.c_float),
    ]


MK36_MAX_RANKS = 8
MK36_IPC_HANDLE_BYTES = 64


class Comm(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("buffers", C.c_void_p * MK36_MAX_RANKS)]


# symbol -> (restype, argtypes); every function declared in mk36.h appears here
SIGNATURES = {
    "mk36_version": (C.c_int, []),
    "mk36_last_error": (C.c_char_p, []),
    "mk36_workspace_bytes": (C.c_size_t, []),
    "mk36_workspace_init": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "mk36_workspace_status": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]),
    "mk36_set_option": (C.c_int, [C.c_char_p, C.c_int]),
    "mk36_workspace_trace": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_ulonglong), C.c_int]),
    "mk36_workspace_cta_trace": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_ulonglong), C.c_int]),
    "mk36_selftest_bounded_wait": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_int]),
    "mk36_moe_workspace_bytes": (C.c_size_t, [C.POINTER(MoeArgs)]),
    "mk36_moe_decode": (C.c_int, [C.POINTER(MoeArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mk36_dense_ffn_workspace_bytes": (C.c_size_t, [C.POINTER(DenseFfnArgs)]),
    "mk36_dense_ffn_decode": (C.c_int, [C.POINTER(DenseFfnArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mk36_linear_workspace_bytes": (C.c_size_t, [C.POINTER(LinearArgs)]),
    "mk36_linear_decode": (C.c_int, [C.POINTER(LinearArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mk36_attention_workspace_bytes": (C.c_size_t, [C.POINTER(AttentionArgs)]),
    "mk36_full_attention_decode": (C.c_int, [C.POINTER(AttentionArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mk36_full_attention_decode_static": (C.c_int, [C.POINTER(AttentionArgs), C.c_void_p]),
    "mk36_static_scratch_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "mk36_linear_attention_decode": (C.c_int, [C.POINTER(LinearAttentionArgs), C.c_void_p]),
    "mk36_linear_attention_decode_steps": (C.c_int, [C.POINTER(LinearAttentionStepsArgs), C.c_void_p]),
    "mk36_comm_buffer_bytes": (C.c_size_t, []),
    "mk36_comm_buffer_alloc": (C.c_int, [C.POINTER(C.c_void_p)]),
    "mk36_comm_buffer_reset": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mk36_comm_buffer_free": (C.c_int, [C.c_void_p]),
    "mk36_ipc_export": (C.c_int, [C.c_void_p, C.POINTER(C.c_ubyte)]),
    "mk36_ipc_open": (C.c_int, [C.POINTER(C.c_ubyte), C.POINTER(C.c_void_p)]),
    "mk36_ipc_close": (C.c_int, [C.c_void_p]),
    "mk36_moe_decode_ep": (C.c_int, [C.POINTER(MoeArgs), C.POINTER(Comm), C.c_void_p, C.c_size_t, C.c_void_p]),
    "mk36_dense_ffn_decode_tp": (C.c_int, [C.POINTER(DenseFfnArgs), C.POINTER(Comm), C.c_void_p, C.c_size_t, C.c_void_p]),
}


def library_path() -> Path:
    override = os.environ.get("MK36_LIBRARY")
    return Path(override) if override else Path(__file__).resolve().parent / LIBRARY_NAME


_lib = None


def load() -> C.CDLL:
    """Loads libmk36.so and attaches the signatures above.  Raises OSError when it is not built."""
    global _lib
    if _lib is None:
        lib = C.CDLL(str(library_path()))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class Mk36Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{message} (mk36 status {status})")
        self.status = status


def check(status: int) -> None:
    if status != MK36_OK:
        raise Mk36Error(status, load().mk36_last_error().decode())
