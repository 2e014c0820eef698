"""ctypes binding of ``libttq.so``: the same C ABI a Nim ``{.importc.}`` block binds (include/ttq.h).

Loading fails loudly when the shared object is missing; there is no alternative implementation.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libttq.so")

# enums of include/ttq.h
FMT_Q8_0, FMT_Q4_K, FMT_Q6_K, FMT_TQ3 = 0, 1, 2, 3
DT_BF16, DT_F16, DT_F32 = 0, 1, 2
SHARD_NONE, SHARD_COLUMN, SHARD_COLUMN_GATED, SHARD_ROW = 0, 1, 2, 3
OK = 0
STATUS_NAMES = {0: "TTQ_OK", 1: "TTQ_ERR_INVALID_ARG", 2: "TTQ_ERR_SHAPE", 3: "TTQ_ERR_UNSUPPORTED",
                4: "TTQ_ERR_CUDA", 5: "TTQ_ERR_OOM", 6: "TTQ_ERR_DEVICE", 7: "TTQ_ERR_LIMIT",
                8: "TTQ_ERR_TIMEOUT"}

# Every symbol include/ttq.h declares, with its signature.
_i64, _vp, _ci, _sz = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
_pp = ctypes.POINTER(ctypes.c_void_p)


class Shard(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("rank", ctypes.c_int32), ("world", ctypes.c_int32)]


class HostLinear(ctypes.Structure):
    """``ttq_host_linear``: one host-buffer linear of a recorded batch."""
    _fields_ = [("w", ctypes.c_void_p), ("x_host", ctypes.c_void_p), ("x_dt", ctypes.c_int32), ("M", ctypes.c_int64),
                ("ldx", ctypes.c_int64), ("bias_host", ctypes.c_void_p), ("bias_dt", ctypes.c_int32), ("y_host", ctypes.c_void_p),
                ("y_dt", ctypes.c_int32), ("ldy", ctypes.c_int64)]


SIGNATURES = {
    "ttq_init": (_ci, [_ci, _pp]),
    "ttq_destroy": (_ci, [_vp]),
    "ttq_last_error": (ctypes.c_char_p, [_vp]),
    "ttq_status_string": (ctypes.c_char_p, [_ci]),
    "ttq_version": (ctypes.c_char_p, []),
    "ttq_block_elems": (_i64, [_ci]),
    "ttq_block_bytes": (_i64, [_ci]),
    "ttq_packed_bytes": (_i64, [_ci, _i64, _i64]),
    "ttq_weight_create": (_ci, [_vp, _ci, _i64, _i64, _vp, _sz, ctypes.POINTER(Shard), _pp]),
    "ttq_weight_create_device": (_ci, [_vp, _ci, _i64, _i64, _vp, _sz, _vp, _pp]),
    "ttq_weight_destroy": (_ci, [_vp]),
    "ttq_weight_info": (_ci, [_vp, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(_i64), ctypes.POINTER(_i64)]),
    "ttq_weight_bytes": (_i64, [_vp]),
    "ttq_dequantize": (_ci, [_vp, _vp, _vp, _i64, _vp]),
    "ttq_linear_forward": (_ci, [_vp, _vp, _vp, _ci, _i64, _i64, _vp, _ci, _vp, _ci, _i64, _vp]),
    "ttq_linear_forward_host": (_ci, [_vp, _vp, _vp, _ci, _i64, _i64, _vp, _ci, _vp, _ci, _i64]),
    "ttq_linear_forward_host_async": (_ci, [_vp, _vp, _vp, _ci, _i64, _i64, _vp, _ci, _vp, _ci, _i64]),
    "ttq_host_sync": (_ci, [_vp]),
    "ttq_host_batch_create": (_ci, [_vp, ctypes.POINTER(HostLinear), _ci, _pp]),
    "ttq_host_batch_run": (_ci, [_vp]),
    "ttq_host_batch_destroy": (_ci, [_vp]),
    "ttq_linear_forward_static": (_ci, [_vp, _vp, _ci, _i64, _i64, _vp, _ci, _vp, _ci, _i64, _vp, ctypes.c_char_p, _sz]),
    "ttq_static_status": (_ci, [_vp, ctypes.c_char_p, _sz]),
    "ttq_linear_forward_gated": (_ci, [_vp, _vp, _vp, _ci, _i64, _i64, _vp, _ci, _vp, _ci, _i64, _vp]),
    "ttq_comm_create": (_ci, [_vp, _ci, _ci, _i64, _ci, _pp, _vp]),
    "ttq_comm_connect": (_ci, [_vp, _vp]),
    "ttq_comm_local_buffer": (_ci, [_vp, _pp, ctypes.POINTER(_sz)]),
    "ttq_comm_connect_pointers": (_ci, [_vp, _pp]),
    "ttq_comm_set_wait_limit": (_ci, [_vp, _i64]),
    "ttq_comm_destroy": (_ci, [_vp]),
    "ttq_linear_forward_allreduce": (_ci, [_vp, _vp, _vp, _ci, _i64, _i64, _vp, _ci, _vp, _ci, _i64, _vp, _vp]),
    "ttq_silu_and_mul": (_ci, [_vp, _vp, _ci, _i64, _i64, _i64, _vp, _i64, _vp]),
    "ttq_moe_create": (_ci, [_vp, ctypes.c_int32, _vp, _vp, _i64, ctypes.c_int32, _pp]),
    "ttq_moe_destroy": (_ci, [_vp]),
    "ttq_moe_forward": (_ci, [_vp, _vp, _vp, _ci, _i64, _i64, _vp, _vp, _vp, _ci, _i64, _vp]),
    "ttq_add_rmsnorm": (_ci, [_vp, _vp, _vp, _vp, _ci, _i64, _i64, _i64, _i64, ctypes.c_float, _vp, _i64, _vp]),
    "ttq_add_rmsnorm_prepare": (_ci, [_vp, _vp, _vp, _vp, _ci, _i64, _i64, _i64, _i64, ctypes.c_float, _vp, _i64, _vp]),
    "ttq_linear_forward_prepared": (_ci, [_vp, _vp, _i64, _vp, _ci, _vp, _ci, _i64, _vp]),
    "ttq_rope_kv_append": (_ci, [_vp, _vp, _ci, _i64, _i64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, _vp, _vp, _vp, _vp, _vp,
                                 _i64, _i64, _vp]),
    "ttq_decode_attention": (_ci, [_vp, _vp, _vp, _vp, _ci, _i64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, _i64, _i64, _vp, _vp]),
    "ttq_launch_count": (_i64, [_vp]),
    "ttq_device_status": (_ci, [_vp, _vp]),
    "ttq_trace_read": (_ci, [_vp, _vp, _i64, ctypes.POINTER(_i64)]),
}

_lib = None


class TtqError(RuntimeError):
    """Raised for every non-zero ttq_status (the Nim wrapper raises ValueError the same way)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m tattletale_b200.build` "
                "(there is no non-CUDA implementation of this path)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here = header and library out of sync
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(ctx_handle, status: int) -> None:
    if status != OK:
        lib = load()
        msg = lib.ttq_last_error(ctx_handle).decode() if ctx_handle else ""
        if not msg:
            msg = lib.ttq_status_string(status).decode()
        raise TtqError(status, msg)
