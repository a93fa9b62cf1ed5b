"""ctypes binding of include/mononn.h -- the stub a Python host would add.

The CUDA library is the product: importing this module fails loudly when
libmononn_b200.so is missing, and there is no CPU path behind it.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmononn_b200.so")

EXPORTS = [
    "mononn_compile_hlo_text", "mononn_compile_encoder_json", "mononn_module_args",
    "mononn_module_launch_config", "mononn_set_constant", "mononn_constant_count",
    "mononn_constant_info", "mononn_launch", "mononn_last_status", "mononn_tune",
    "mononn_save_spec", "mononn_spec_json", "mononn_profile_stages", "mononn_module_cost",
    "mononn_destroy", "mononn_strerror", "mononn_last_error", "mononn_enabled",
    "mononn_trace_stages", "mononn_plan_json", "mononn_describe", "mononn_free_string", "mononn_launch_stages", "mononn_debug_skew_barrier", "mononn_attention_noalloc",
    "mononn_infer_host", "mononn_debug_mma_issue", "mononn_attention_noalloc_status",
]


class Options(C.Structure):
    _fields_ = [("device", C.c_int), ("dump_dir", C.c_char_p), ("spec_dir", C.c_char_p),
                ("threadpool_size", C.c_int), ("tuning_level", C.c_int),
                ("barrier_timeout_us", C.c_uint)]


class ArgDesc(C.Structure):
    _fields_ = [("index", C.c_int), ("bytes", C.c_size_t), ("kind", C.c_int),
                ("param_number", C.c_int)]


class MononnError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"mononn error {code}: {message}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m mononn_b200.build` "
                "(there is no fallback implementation)")
        l = C.CDLL(LIB_PATH)
        vp, cp, ip = C.c_void_p, C.c_char_p, C.POINTER(C.c_int)
        l.mononn_compile_hlo_text.argtypes = [cp, C.c_size_t, cp, C.POINTER(Options), C.POINTER(vp)]
        l.mononn_compile_encoder_json.argtypes = [cp, cp, C.POINTER(Options), C.POINTER(vp)]
        l.mononn_module_args.argtypes = [vp, C.POINTER(C.POINTER(ArgDesc)), ip]
        l.mononn_module_launch_config.argtypes = [vp, C.POINTER(C.c_uint * 3), C.POINTER(C.c_uint * 3),
                                                  C.POINTER(C.c_uint)]
        l.mononn_set_constant.argtypes = [vp, cp, vp, C.c_size_t]
        l.mononn_constant_count.argtypes = [vp, ip]
        l.mononn_constant_info.argtypes = [vp, C.c_int, C.POINTER(cp), C.POINTER(C.c_size_t)]
        l.mononn_launch.argtypes = [vp, C.POINTER(vp), C.c_int, vp]
        l.mononn_last_status.argtypes = [vp, ip, ip]
        l.mononn_infer_host.argtypes = [vp, C.POINTER(vp), C.c_int, C.POINTER(vp), C.c_int, C.POINTER(vp), C.c_int, vp]
        l.mononn_tune.argtypes = [vp, C.POINTER(vp), C.c_int, vp]
        l.mononn_save_spec.argtypes = [vp, cp]
        l.mononn_spec_json.argtypes = [vp, C.POINTER(cp)]
        l.mononn_profile_stages.argtypes = [vp, C.POINTER(vp), C.c_int, vp, C.POINTER(C.c_double),
                                            C.POINTER(cp), C.c_int, ip]
        l.mononn_module_cost.argtypes = [vp, C.POINTER(C.c_double), C.POINTER(C.c_double)]
        l.mononn_trace_stages.argtypes = [vp, C.POINTER(vp), C.c_int, vp, C.POINTER(C.c_double), C.c_size_t, ip, ip]
        l.mononn_plan_json.argtypes = [vp, C.POINTER(cp)]
        l.mononn_describe.argtypes = [cp, cp, C.c_size_t, cp, C.c_uint, C.POINTER(vp)]
        l.mononn_free_string.argtypes = [vp]
        l.mononn_free_string.restype = None
        l.mononn_launch_stages.argtypes = [vp, C.POINTER(vp), C.c_int, vp, C.c_uint, C.c_uint]
        l.mononn_debug_skew_barrier.argtypes = [vp, C.c_uint]
        l.mononn_attention_noalloc.argtypes = [vp, vp, vp, vp, vp, C.c_uint, C.c_uint, C.c_uint, C.c_uint,
                                               C.c_uint, C.c_uint, C.c_float, C.c_float, C.c_int, vp]
        l.mononn_attention_noalloc_status.argtypes = [vp]
        dp = C.POINTER(C.c_double)
        l.mononn_debug_mma_issue.argtypes = [C.c_int, C.c_uint, C.c_uint, C.c_uint, C.c_uint, C.c_uint, dp, dp, dp]
        l.mononn_destroy.argtypes = [vp]
        l.mononn_destroy.restype = None
        l.mononn_strerror.argtypes = [C.c_int]
        l.mononn_strerror.restype = cp
        l.mononn_last_error.restype = cp
        l.mononn_enabled.restype = C.c_int
        _lib = l
    return _lib


def check(code: int) -> None:
    if code != 0:
        l = lib()
        msg = (l.mononn_last_error() or b"").decode() or l.mononn_strerror(code).decode()
        raise MononnError(code, msg)
