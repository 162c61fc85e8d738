"""ctypes binding of ``libjabas_b200.so`` (declarations: ``include/jabas_b200.h``).

The library is the only implementation of the gradient path: if it cannot be loaded
this module raises, and nothing in the package substitutes a PyTorch or CPU path.
"""
from __future__ import annotations

import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libjabas_b200.so")

MAX_VSW = 16
MAX_GROUPS = 16

#: every symbol ``include/jabas_b200.h`` declares
EXPORTS = (
    "jabas_version", "jabas_last_error", "jabas_ctx_create", "jabas_ctx_destroy",
    "jabas_layout_create", "jabas_layout_destroy", "jabas_vsw_aggregate_f32", "jabas_div_f32",
    "jabas_sgd_momentum_f32", "jabas_adam_f32", "jabas_dot_norms_f32", "jabas_cosine_finalize",
    "jabas_replicate_f32", "jabas_dot_norms_static_f32", "jabas_vsw_sgd_momentum_f32",
    "jabas_vsw_adam_f32", "jabas_sumsq_f32", "jabas_clip_coef", "jabas_dynhp_create",
    "jabas_dynhp_destroy", "jabas_dynhp_push_sgd", "jabas_dynhp_push_adam",
    "jabas_ctx_set_staging", "jabas_ctx_staging_timeouts", "jabas_ctx_set_wait_limits",
    "jabas_ctx_inject_staging_stall", "jabas_exchange_flag_words", "jabas_exchange_create",
    "jabas_exchange_destroy", "jabas_exchange_reset", "jabas_exchange_status", "jabas_exchange_step_f32",
    "jabas_exchange_cosine", "jabas_exchange_set_trace", "jabas_exchange_set_grid_limit", "jabas_exchange_set_ctas_per_sm",
)

EXCHANGE_PIECE = 8192          # JABAS_EXCHANGE_PIECE


class Seg(ctypes.Structure):
    _fields_ = [("begin", ctypes.c_uint64), ("end", ctypes.c_uint64),
                ("group", ctypes.c_uint32), ("reserved", ctypes.c_uint32)]


class Group(ctypes.Structure):
    _fields_ = [("lr", ctypes.c_double), ("weight_decay", ctypes.c_double),
                ("step", ctypes.c_int64), ("reserved", ctypes.c_int64)]


class SgdHp(ctypes.Structure):
    _fields_ = [("momentum", ctypes.c_double), ("dampening", ctypes.c_double),
                ("nesterov", ctypes.c_int), ("first_step", ctypes.c_int),
                ("grad_scale", ctypes.c_void_p), ("dynamic", ctypes.c_void_p),
                ("remote_sources", ctypes.c_int), ("reserved", ctypes.c_int)]


class AdamHp(ctypes.Structure):
    _fields_ = [("beta1", ctypes.c_double), ("beta2", ctypes.c_double), ("eps", ctypes.c_double),
                ("decoupled", ctypes.c_int), ("reserved", ctypes.c_int),
                ("grad_scale", ctypes.c_void_p), ("dynamic", ctypes.c_void_p),
                ("remote_sources", ctypes.c_int), ("reserved2", ctypes.c_int)]


class ExchangeDesc(ctypes.Structure):
    _fields_ = [("nranks", ctypes.c_int), ("rank", ctypes.c_int),
                ("px", ctypes.POINTER(ctypes.c_void_p)), ("pg", ctypes.POINTER(ctypes.c_void_p)),
                ("flags", ctypes.POINTER(ctypes.c_void_p)), ("max_slots", ctypes.c_uint32),
                ("window_pieces", ctypes.c_uint32), ("piece_elems", ctypes.c_uint32),
                ("update_lag", ctypes.c_uint32)]


class ExchangeBufs(ctypes.Structure):
    _fields_ = [("grads", ctypes.POINTER(ctypes.c_void_p)), ("Kg", ctypes.c_int), ("K", ctypes.c_int),
                ("w", ctypes.POINTER(ctypes.c_void_p)), ("m", ctypes.c_void_p), ("v", ctypes.c_void_p),
                ("stat3", ctypes.c_void_p)]


class JabasError(RuntimeError):
    """A libjabas_b200 call returned a negative status."""


_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once and declare every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m jabas_b200.build` "
            "(nvcc, sm_100a). There is no fallback implementation.")
    lib = ctypes.CDLL(LIB_PATH)
    vp, u64, f32, i32, f64 = (ctypes.c_void_p, ctypes.c_uint64, ctypes.c_float, ctypes.c_int,
                              ctypes.c_double)
    pvp = ctypes.POINTER(ctypes.c_void_p)
    lib.jabas_version.argtypes = []
    lib.jabas_last_error.argtypes = []
    lib.jabas_last_error.restype = ctypes.c_char_p
    lib.jabas_ctx_create.argtypes = [i32, pvp]
    lib.jabas_ctx_destroy.argtypes = [vp]
    lib.jabas_ctx_set_staging.argtypes = [vp, i32]
    lib.jabas_ctx_staging_timeouts.argtypes = [vp, ctypes.POINTER(ctypes.c_uint32)]
    lib.jabas_ctx_set_wait_limits.argtypes = [vp, f64, f64]
    lib.jabas_ctx_inject_staging_stall.argtypes = [vp, i32]
    u32 = ctypes.c_uint32
    lib.jabas_exchange_flag_words.argtypes = [u32]
    lib.jabas_exchange_create.argtypes = [vp, ctypes.POINTER(ExchangeDesc), pvp]
    lib.jabas_exchange_destroy.argtypes = [vp]
    lib.jabas_exchange_reset.argtypes = [vp]
    lib.jabas_exchange_status.argtypes = [vp, ctypes.POINTER(u32), ctypes.POINTER(u32)]
    lib.jabas_exchange_step_f32.argtypes = [pvp, ctypes.POINTER(ExchangeBufs), i32, u64, u64, u32, f32, f32, vp,
                                            ctypes.POINTER(Group), i32, ctypes.POINTER(SgdHp),
                                            ctypes.POINTER(AdamHp), vp]
    lib.jabas_exchange_set_trace.argtypes = [vp, vp, u64]
    lib.jabas_exchange_set_grid_limit.argtypes = [vp, u32]
    lib.jabas_exchange_set_ctas_per_sm.argtypes = [vp, i32]
    lib.jabas_exchange_cosine.argtypes = [pvp, pvp, pvp, i32, f64, vp]
    lib.jabas_layout_create.argtypes = [vp, ctypes.POINTER(Seg), i32, u64, pvp]
    lib.jabas_layout_destroy.argtypes = [vp]
    lib.jabas_vsw_aggregate_f32.argtypes = [vp, pvp, i32, vp, vp, u64, f32, f32, vp, vp]
    lib.jabas_div_f32.argtypes = [vp, vp, u64, f32, vp]
    lib.jabas_sgd_momentum_f32.argtypes = [vp, vp, pvp, i32, vp, u64, u64, vp,
                                           ctypes.POINTER(Group), i32, ctypes.POINTER(SgdHp),
                                           vp, f32, vp, vp]
    lib.jabas_adam_f32.argtypes = [vp, vp, pvp, i32, vp, vp, u64, u64, vp,
                                   ctypes.POINTER(Group), i32, ctypes.POINTER(AdamHp),
                                   vp, f32, vp, vp]
    lib.jabas_vsw_sgd_momentum_f32.argtypes = [vp, pvp, i32, f32, vp, pvp, i32, vp, u64, u64, vp,
                                               ctypes.POINTER(Group), i32, ctypes.POINTER(SgdHp),
                                               f32, vp, vp]
    lib.jabas_vsw_adam_f32.argtypes = [vp, pvp, i32, f32, vp, pvp, i32, vp, vp, u64, u64, vp,
                                       ctypes.POINTER(Group), i32, ctypes.POINTER(AdamHp), f32, vp, vp]
    lib.jabas_dot_norms_f32.argtypes = [vp, vp, vp, u64, vp, vp]
    lib.jabas_dynhp_create.argtypes = [vp, pvp]
    lib.jabas_dynhp_destroy.argtypes = [vp]
    lib.jabas_dynhp_push_sgd.argtypes = [vp, ctypes.POINTER(Group), i32, ctypes.POINTER(SgdHp), vp]
    lib.jabas_dynhp_push_adam.argtypes = [vp, ctypes.POINTER(Group), i32, ctypes.POINTER(AdamHp), vp]
    lib.jabas_sumsq_f32.argtypes = [vp, vp, u64, vp, vp]
    lib.jabas_clip_coef.argtypes = [vp, vp, f64, vp, vp]
    lib.jabas_cosine_finalize.argtypes = [vp, vp, f64, vp, vp]
    lib.jabas_replicate_f32.argtypes = [vp, vp, pvp, i32, u64, vp]
    lib.jabas_dot_norms_static_f32.argtypes = [vp, vp, u64, vp, vp]
    for name in EXPORTS:
        if name not in ("jabas_last_error", "jabas_exchange_flag_words"):
            getattr(lib, name).restype = i32
    lib.jabas_exchange_flag_words.restype = ctypes.c_size_t
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != 0:
        msg = load().jabas_last_error()
        raise JabasError(f"libjabas_b200 error {rc}: {msg.decode() if msg else '?'}")
