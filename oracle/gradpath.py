"""TEST INFRASTRUCTURE — numpy front-end of the C oracle in ``gradpath_oracle.c``.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
module.  Parity of the arithmetic is UNPINNED by the reference (it ships no tests and
the code that owns the arithmetic is an absent submodule); see the header of the C file.

Every function takes C-contiguous ``numpy.float32`` arrays and mutates its outputs in
place, mirroring the in-place PyTorch ops of the reference path.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` next to its source if it is missing or stale."""
    src = os.path.join(_HERE, "gradpath_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)
             or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src))
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(_LIB_PATH)
        sz = ctypes.c_size_t
        pp = ctypes.POINTER(_f32p)
        lib.oracle_vsw_aggregate_f32.argtypes = [pp, ctypes.c_int, _f32p, _f32p, sz, ctypes.c_float]
        lib.oracle_div_f32.argtypes = [_f32p, sz, ctypes.c_float]
        lib.oracle_dot_norms_f32.argtypes = [_f32p, _f32p, sz, _f64p]
        lib.oracle_half_stat_f32.argtypes = [_f32p, _f32p, sz, ctypes.c_float, _f64p]
        lib.oracle_vsw_parity_stat_f32.argtypes = [pp, ctypes.c_int, sz, ctypes.c_float, _f64p]
        lib.oracle_cosine_from_stat.argtypes = [_f64p, ctypes.c_double]
        lib.oracle_cosine_from_stat.restype = ctypes.c_float
        lib.oracle_sgd_momentum_f32.argtypes = [_f32p, _f32p, _f32p, sz] + [ctypes.c_double] * 4 + [ctypes.c_int] * 2
        lib.oracle_adam_f32.argtypes = ([_f32p] * 4 + [sz] + [ctypes.c_double] * 5
                                        + [ctypes.c_longlong, ctypes.c_int])
        lib.oracle_replicate_f32.argtypes = [_f32p, pp, ctypes.c_int, sz]
        lib.oracle_sumsq_f32.argtypes = [_f32p, sz]
        lib.oracle_sumsq_f32.restype = ctypes.c_double
        lib.oracle_clip_grad_norm_f32.argtypes = [_f32p, sz, ctypes.c_double, _f32p]
        lib.oracle_clip_grad_norm_f32.restype = ctypes.c_float
        for name in ("oracle_vsw_aggregate_f32", "oracle_div_f32", "oracle_dot_norms_f32",
                     "oracle_half_stat_f32", "oracle_vsw_parity_stat_f32",
                     "oracle_sgd_momentum_f32", "oracle_adam_f32", "oracle_replicate_f32"):
            getattr(lib, name).restype = None
        _lib = lib
    return _lib


def _chk(a: np.ndarray) -> np.ndarray:
    if a.dtype != np.float32 or not a.flags["C_CONTIGUOUS"]:
        raise TypeError("oracle arrays must be C-contiguous float32")
    return a


def _p(a: Optional[np.ndarray]):
    return None if a is None else _chk(a).ctypes.data_as(_f32p)


def _pp(arrs: Sequence[np.ndarray]):
    return (_f32p * len(arrs))(*[_p(a) for a in arrs])


def vsw_aggregate(grads: Sequence[np.ndarray], out: np.ndarray, divisor: float,
                  half_out: Optional[np.ndarray] = None) -> None:
    """out = (g_0 + g_1 + ... + g_{K-1}) / divisor, ascending k; half_out = the sum."""
    n = out.size
    assert all(g.size == n for g in grads)
    _load().oracle_vsw_aggregate_f32(_pp(grads), len(grads), _p(out), _p(half_out), n, divisor)


def div_(x: np.ndarray, divisor: float) -> None:
    _load().oracle_div_f32(_p(x), x.size, divisor)


def dot_norms(a: np.ndarray, b: np.ndarray, stat: Optional[np.ndarray] = None) -> np.ndarray:
    """stat += (<a,b>, |a|^2, |b|^2) in fp64."""
    stat = np.zeros(3, np.float64) if stat is None else stat
    _load().oracle_dot_norms_f32(_p(a), _p(b), a.size, stat.ctypes.data_as(_f64p))
    return stat


def half_stat(g: np.ndarray, half: np.ndarray, half_divisor: float,
              stat: Optional[np.ndarray] = None) -> np.ndarray:
    """stat += (<e,o>, |e|^2, |o|^2) with e = half/half_divisor, o = 2g - e."""
    stat = np.zeros(3, np.float64) if stat is None else stat
    _load().oracle_half_stat_f32(_p(g), _p(half), g.size, half_divisor, stat.ctypes.data_as(_f64p))
    return stat


def vsw_parity_stat(grads: Sequence[np.ndarray], half_divisor: float,
                    stat: Optional[np.ndarray] = None) -> np.ndarray:
    """Single-GPU statistic: halves are the even-index and the odd-index VSWs."""
    stat = np.zeros(3, np.float64) if stat is None else stat
    _load().oracle_vsw_parity_stat_f32(_pp(grads), len(grads), grads[0].size, half_divisor,
                                       stat.ctypes.data_as(_f64p))
    return stat


def cosine_from_stat(stat: np.ndarray, eps: float = 1e-8) -> float:
    stat = np.ascontiguousarray(stat, np.float64)
    return float(_load().oracle_cosine_from_stat(stat.ctypes.data_as(_f64p), eps))


def sgd_momentum(g: np.ndarray, p: np.ndarray, m: np.ndarray, *, lr: float,
                 weight_decay: float = 0.0, momentum: float = 0.0, dampening: float = 0.0,
                 nesterov: bool = False, first_step: bool = False) -> None:
    _load().oracle_sgd_momentum_f32(_p(g), _p(p), _p(m), p.size, lr, weight_decay, momentum,
                                    dampening, int(nesterov), int(first_step))


def adam(g: np.ndarray, p: np.ndarray, m: np.ndarray, v: np.ndarray, *, lr: float,
         weight_decay: float, beta1: float, beta2: float, eps: float, step: int,
         decoupled: bool) -> None:
    """``decoupled=True`` is AdamW, ``False`` is Adam with coupled L2."""
    _load().oracle_adam_f32(_p(g), _p(p), _p(m), _p(v), p.size, lr, weight_decay, beta1, beta2,
                            eps, step, int(decoupled))


def replicate(src: np.ndarray, dsts: Sequence[np.ndarray]) -> None:
    _load().oracle_replicate_f32(_p(src), _pp(dsts), len(dsts), src.size)


def sumsq(x: np.ndarray) -> float:
    return float(_load().oracle_sumsq_f32(_p(x), x.size))


def clip_grad_norm(g: np.ndarray, max_norm: float):
    """In-place L2-norm clipping of a flat gradient; returns (coefficient, norm)."""
    norm = ctypes.c_float()
    coef = _load().oracle_clip_grad_norm_f32(_p(g), g.size, max_norm, ctypes.byref(norm))
    return float(coef), float(norm.value)


def update_segments(kind: str, g, p, m, v, segments, groups, **common) -> None:
    """Apply ``sgd_momentum`` or ``adam`` range by range.

    ``segments`` is a list of ``(begin, end, group_index)`` over the flat buffer and
    ``groups`` a list of dicts of per-parameter-group hyper-parameters (``lr``,
    ``weight_decay`` and, for Adam, ``step``) — the flat-bucket form of the
    param-group lists built at examples/resnet50/main.py:340-349.
    """
    for begin, end, gi in segments:
        hp = dict(common)
        hp.update(groups[gi])
        sl = slice(begin, end)
        if kind == "sgd":
            sgd_momentum(g[sl], p[sl], m[sl], **hp)
        else:
            adam(g[sl], p[sl], m[sl], v[sl], **hp)
