"""ctypes binding of libfswiglu.so (the C ABI declared in include/fswiglu.h).

Every compute entry point of this package goes through the functions below; there
is no PyTorch or CPU fallback.  If the shared library has not been built, importing
this module raises, so a missing CUDA build can never pass silently.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libfswiglu.so")

OK = 0
ERR_BAD_ARG = -1
ERR_ALIGNMENT = -2
ERR_SHAPE = -3
ERR_CUDA = -4
ERR_WATCHDOG = -5
ERR_WORKSPACE = -6
ERR_NO_DEVICE = -7
ERR_TOO_LARGE = -8

OUT_BF16 = 0
OUT_F32 = 1

# name -> (restype, argtypes); mirrors include/fswiglu.h one to one.
_vp, _i64, _int, _sz, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t, ctypes.c_float
SIGNATURES = {
    "fswiglu_gateup_bf16": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp]),
    "fswiglu_gateup_bf16_ex": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp, _sz, _vp]),
    "fswiglu_gemm_scratch_bytes": (_sz, []),
    "fswiglu_down_bf16": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _int, _vp]),
    "fswiglu_down_bf16_ex": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _int, _vp, _i64, _vp, _sz, _vp]),
    "fswiglu_mlp_bf16_ex": (_int, [_vp, _i64, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _int, _i64, _i64,
                                   _i64, _vp, _sz, _vp]),
    "fswiglu_rms_scale_f32": (_int, [_vp, _i64, _i64, _i64, _f32, _vp, _vp]),
    "fswiglu_static_status": (_int, [ctypes.POINTER(ctypes.c_uint32), _vp]),
    "fswiglu_mlp_bf16": (_int, [_vp, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _int, _i64, _i64, _i64,
                                _vp, _sz, _vp]),
    "fswiglu_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "fswiglu_mlp_bf16_host": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _sz, _vp]),
    "fswiglu_host_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "fswiglu_mlp_bf16_static": (_int, [_vp, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _int, _i64, _i64, _i64, _vp]),
    "fswiglu_backward_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "fswiglu_mlp_backward_bf16": (_int, [_vp, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _vp,
                                         _i64, _int, _i64, _i64, _i64, _vp, _sz, _vp]),
    "fswiglu_gemm_tn_bf16": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "fswiglu_transpose_bf16": (_int, [_vp, _i64, _vp, _i64, _i64, _i64, _vp]),
    "fswiglu_cast_f32_to_bf16": (_int, [_vp, _vp, _i64, _vp]),
    "fswiglu_down_scatter_bf16": (_int, [_vp, _i64, _vp, _i64, ctypes.POINTER(ctypes.c_void_p), _int, _int, _i64, _i64,
                                         _i64, _i64, _vp, _sz, _vp]),
    "fswiglu_reduce_bcast_bf16": (_int, [_vp, ctypes.POINTER(ctypes.c_void_p), _int, _i64, _i64, _int, _vp]),
    "fswiglu_set_max_ctas": (_int, [_int]),
    "fswiglu_device_status": (_int, [ctypes.POINTER(ctypes.c_uint32), _vp]),
    "fswiglu_set_wait_limit_us": (_i64, [_i64]),
    "fswiglu_test_expire_next_wait": (None, [_int]),
    "fswiglu_set_decode_trace": (None, [_vp]),
    "fswiglu_status_string": (ctypes.c_char_p, [_int]),
    "fswiglu_plan_kernel": (ctypes.c_int, [ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int]),
    "fswiglu_version": (ctypes.c_char_p, []),
    "fswiglu_launch_count": (ctypes.c_uint64, []),
}


class FswigluError(RuntimeError):
    """A libfswiglu call returned a negative status."""

    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {status_string(status)} (status {status})")


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()' "
            "or python fused-swiglu_b200/build.py). There is no fallback path."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def status_string(status: int) -> str:
    return lib.fswiglu_status_string(int(status)).decode()


def version() -> str:
    return lib.fswiglu_version().decode()


def launch_count() -> int:
    return int(lib.fswiglu_launch_count())


def check(status: int, where: str) -> None:
    if status != OK:
        raise FswigluError(status, where)


def static_status(stream_ptr: int = 0) -> int:
    """Watchdog word of the allocation-free entry point on the current device (0 = healthy)."""
    word = ctypes.c_uint32(0)
    rc = lib.fswiglu_static_status(ctypes.byref(word), ctypes.c_void_p(stream_ptr))
    if rc not in (OK, ERR_WATCHDOG):
        raise FswigluError(rc, "fswiglu_static_status")
    return int(word.value)


def device_status(stream_ptr: int = 0) -> int:
    """Synchronise the stream and return the device watchdog word (0 = healthy)."""
    word = ctypes.c_uint32(0)
    rc = lib.fswiglu_device_status(ctypes.byref(word), ctypes.c_void_p(stream_ptr))
    if rc not in (OK, ERR_WATCHDOG):
        raise FswigluError(rc, "fswiglu_device_status")
    return int(word.value)
