"""ctypes binding of libdejavu_b200.so (declared in include/dejavu_b200.h).

The library is the only compute path of this package: if it is missing the import of any operator
raises, there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libdejavu_b200.so"

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_SCRATCH, ERR_TIMEOUT = 0, -1, -2, -3, -4, -5
ACT = {"id": 0, "relu": 1, "gelu": 2, "gelu_approx": 3, "squared_relu": 4}
MAX_BATCH = 32
KV_WINDOW = 16
EXCHANGE_REFILL = 1
ATTN_STATE_HDR = 8


class DejavuKernelError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, fn: str, status: int, message: str):
        super().__init__(f"{fn} failed with status {status}: {message}")
        self.status = status


_vp, _i, _ll, _sz, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_size_t, C.c_float

# name -> (restype, argtypes); mirrors include/dejavu_b200.h one to one
SIGNATURES = {
    "djv_version": (_i, []),
    "djv_last_error": (C.c_char_p, []),
    "djv_status_string": (C.c_char_p, [_i]),
    "djv_launch_count": (C.c_ulonglong, []),
    "djv_gather_gemv": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _i, _i, _vp]),
    "djv_gather_transposed_gemv_scratch_bytes": (_sz, [_i, _i, _i]),
    "djv_gather_transposed_gemv": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _i, _vp, _sz, _vp]),
    "djv_gather_transposed_gemv_static": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _i, _vp]),
    "djv_mlp_sparse": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _i, _vp, _sz, _vp]),
    "djv_topk": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "djv_qkv_proj_sparse": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "djv_out_proj_sparse": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "djv_k_cache_copy_sparse": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _ll, _ll, _vp]),
    "djv_v_cache_copy_sparse": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _ll, _ll, _vp]),
    "djv_attn_state_reset": (_i, [_vp, _i, _i, _vp]),
    "djv_attn_step_scratch_bytes": (_sz, [_i, _i, _i]),
    "djv_attn_step": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp]),
    "djv_attn_step_project": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "djv_topk_attn_prep": (_i, [_vp, _vp, _i, _i, _i, _vp, _i, _vp]),
    "djv_attn_step_attend": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp, _sz, _vp]),
    "djv_attn_step_project_batch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "djv_attn_step_attend_batch": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp, _sz, _vp]),
    "djv_attn_step_finish": (_i, [_vp, _i, _vp]),
    "djv_decode_attn_scratch_bytes": (_sz, [_i, _i, _i, _i]),
    "djv_decode_attn": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp]),
    "djv_add_layernorm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "djv_ipc_alloc": (_i, [_sz, C.POINTER(_vp)]),
    "djv_ipc_free": (_i, [_vp]),
    "djv_ipc_get_handle": (_i, [_vp, C.c_char_p]),
    "djv_ipc_open": (_i, [C.c_char_p, C.POINTER(_vp)]),
    "djv_ipc_close": (_i, [_vp]),
    "djv_comm_buffer_bytes": (_sz, [_i, _sz]),
    "djv_comm_create": (_i, [C.POINTER(_vp), _i, _i, C.POINTER(_vp), _sz]),
    "djv_gather_transposed_gemv_push": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _i, _vp, _sz, _vp]),
    "djv_out_proj_sparse_push": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "djv_comm_end_step": (_i, [_vp, _i, _vp]),
    "djv_prefetch_rows_l2": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _vp]),
    "djv_prefetch_segments_l2": (_i, [_vp, _vp, _i, _i, _i, _ll, _i, _vp]),
    "djv_mlp_sparse_fused_supported": (_i, [_i, _i, _i]),
    "djv_mlp_sparse_fused_single_batch": (_i, [_i, _i, _i]),
    "djv_mlp_sparse_fused_scratch_bytes": (_sz, [_i, _i, _i]),
    "djv_mlp_ring_timeouts": (C.c_uint, []),
    "djv_mlp_ring_bad_indices": (C.c_uint, []),
    "djv_mlp_sparse_fused": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _i, _vp, _sz, _vp]),
    "djv_mlp_sparse_fused_exchange": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp,
                                           _i, _i, _i, _i, _ll, _ll, _i, _vp, _sz, _vp]),
    "djv_set_early_weight_prefetch": (None, [_i]),
    "djv_set_programmatic_launch": (None, [_i]),
    "djv_batch_sum": (_i, [_vp, _vp, _i, _i, _vp]),
    "djv_comm_destroy": (_i, [_vp]),
    "djv_comm_status": (_i, [_vp]),
    "djv_allreduce_add_layernorm": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library (once). Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m dejavu_b200.build` "
                "(there is no fallback path)"
            )
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(fn_name: str, status: int) -> None:
    if status != OK:
        msg = load().djv_last_error().decode(errors="replace")
        raise DejavuKernelError(fn_name, status, msg)


def call(fn_name: str, *args) -> None:
    check(fn_name, getattr(load(), fn_name)(*args))


def launch_count() -> int:
    return int(load().djv_launch_count())
