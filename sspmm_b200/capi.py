"""ctypes binding of libsspmm_b200.so (the C ABI in include/sspmm_b200.h).

The library is the product: nothing here computes on the CPU, and importing
this module raises if the shared object is missing (build it with
``python -m sspmm_b200.build``)."""
from __future__ import annotations

import ctypes as C
import os

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libsspmm_b200.so")

c_int_p = C.POINTER(C.c_int)
_vp = C.c_void_p

# name -> (restype, argtypes); mirrors include/sspmm_b200.h one to one
SIGNATURES = {
    "sspmm_f16_f32": (C.c_int, [C.c_int] * 4 + [_vp] * 7),
    "sspmm_f16_f16": (C.c_int, [C.c_int] * 4 + [_vp] * 7),
    "sspmm_f16_f16_batched": (C.c_int, [C.c_int] * 5 + [_vp, _vp, _vp, _vp, C.c_int64, _vp, C.c_int64, _vp, C.c_int64, _vp]),
    "sspmm_f16_f16_noalloc": (C.c_int, [C.c_int] * 4 + [_vp] * 7),
    "sspmm_workspace_bytes": (C.c_int, [C.c_int] * 4 + [C.c_int64, C.c_int, C.POINTER(C.c_int64)]),
    "sspmm_f16_f16_ws": (C.c_int, [C.c_int] * 4 + [_vp] * 6 + [C.c_int64, _vp, C.c_int64, _vp]),
    "sspmm_plan_create": (C.c_int, [C.c_int] * 3 + [_vp, _vp, _vp, C.POINTER(_vp)]),
    "sspmm_plan_destroy": (C.c_int, [_vp]),
    "sspmm_plan_info": (C.c_int, [_vp, C.POINTER(C.c_int64), c_int_p, c_int_p, C.POINTER(C.c_int64)]),
    "sspmm_planned": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, _vp]),
    "sspmm_group_create": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, C.POINTER(_vp)]),
    "sspmm_group_run": (C.c_int, [_vp, _vp]),
    "sspmm_group_info": (C.c_int, [_vp, c_int_p, c_int_p, c_int_p, c_int_p, C.POINTER(C.c_int64)]),
    "sspmm_group_destroy": (C.c_int, [_vp]),
    "sspmm_set_kernel": (C.c_int, [C.c_int]),
    "sspmm_device_status": (C.c_int, [c_int_p]),
    "sspmm_selftest_wait_expiry": (C.c_int, [C.c_longlong, c_int_p]),
    "svc_begin": (C.c_int, [C.c_int] * 3 + [_vp, _vp, _vp, _vp, C.POINTER(_vp), C.POINTER(C.c_int64)]),
    "svc_finish": (C.c_int, [_vp, _vp, _vp, _vp, _vp]),
    "svc_free": (C.c_int, [_vp]),
    "svc_batch_begin": (C.c_int, [C.c_int, C.c_int, c_int_p, c_int_p, c_int_p, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _vp,
                                  C.POINTER(_vp), C.POINTER(C.c_int64)]),
    "svc_batch_finish": (C.c_int, [_vp, _vp, _vp, _vp, _vp]),
    "svc_batch_free": (C.c_int, [_vp]),
    "svc_batch_replayed_rows": (C.c_int, [_vp, C.POINTER(C.c_int64)]),
    "svc_reorder": (C.c_int, [C.c_int] * 3 + [_vp] * 4),
    "svc_replayed_rows": (C.c_int, [_vp, C.POINTER(C.c_int64)]),
    "sspmm_sorted_row_swizzle": (C.c_int, [C.c_int, _vp, _vp, _vp]),
    "smtx_read_header": (C.c_int, [C.c_char_p, c_int_p, c_int_p, c_int_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "smtx_read": (C.c_int, [C.c_char_p, _vp, C.c_int64, _vp, C.c_int64]),
    "smtx_write": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_int, _vp, C.c_int64, _vp, C.c_int64]),
    "sspmm_last_error_string": (C.c_char_p, []),
    "sspmm_version": (C.c_char_p, []),
}


class GroupItem(C.Structure):
    """struct sspmm_group_item of include/sspmm_b200.h."""
    _fields_ = [("plan", _vp), ("values_f16", _vp), ("rhs_f16", _vp), ("out", _vp), ("N", C.c_int)]


class SspmmError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"sspmm_b200 error {code}: {message}")
        self.code = code


def load(path: str = _LIB_PATH) -> C.CDLL:
    if not os.path.exists(path):
        raise ImportError(f"{path} not found: build it with `python -m sspmm_b200.build`")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = load()
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise SspmmError(rc, lib().sspmm_last_error_string().decode())
