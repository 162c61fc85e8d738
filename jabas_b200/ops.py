"""Host-side launchers: torch tensors in, C-ABI calls out.

PyTorch is used here only for device memory and streams.  Every function enqueues one
kernel of ``libjabas_b200.so`` on the given (default: current) CUDA stream and returns
immediately.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import MAX_GROUPS, MAX_VSW, JabasError


def _stream_handle(device: torch.device, stream: Optional[torch.cuda.Stream]) -> int:
    s = stream if stream is not None else torch.cuda.current_stream(device)
    return s.cuda_stream


def _dev_f32(t, device: torch.device, name: str) -> int:
    if isinstance(t, int):            # a raw device pointer (e.g. a peer mapping of another rank's buffer)
        if t == 0:
            raise JabasError(f"{name} is a null pointer")
        return t
    if not t.is_cuda or t.device != device:
        raise JabasError(f"{name} must live on {device} (got {t.device}); there is no CPU path")
    if t.dtype != torch.float32 or not t.is_contiguous():
        raise JabasError(f"{name} must be a contiguous float32 tensor")
    return t.data_ptr()


def _stat_ptr(stat: Optional[torch.Tensor], device: torch.device) -> Optional[int]:
    if stat is None:
        return None
    if (not stat.is_cuda or stat.device != device or stat.dtype != torch.float64
            or stat.numel() != 3 or not stat.is_contiguous()):
        raise JabasError("stat must be a contiguous float64 tensor of 3 elements on the context's device")
    return stat.data_ptr()


def _scale_ptr(t: Optional[torch.Tensor], device: torch.device) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda or t.device != device or t.dtype != torch.float32 or t.numel() < 1:
        raise JabasError("grad_scale must be a float32 tensor on the context's device")
    return t.data_ptr()


def _dyn_ptr(d) -> Optional[int]:
    return None if d is None else d._h


def _ptr_array(ptrs: Sequence[int]):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


class Context:
    """Owns a ``jabas_ctx_t``: device id, SM count, per-stream reduction workspaces."""

    def __init__(self, device=None):
        if not torch.cuda.is_available():
            raise JabasError("jabas_b200 needs a CUDA device (B200, sm_100a); there is no CPU fallback")
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None
                                   else torch.device(device).index or 0)
        self._lib = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(self._lib.jabas_ctx_create(self.device.index, ctypes.byref(h)))
        self._h = h
        self.staging = "register"

    STAGING = {"register": 0, "bulk": 1}

    def set_staging(self, mode: str) -> None:
        """How the update kernels fetch their tiles: ``"register"`` (per-thread 128-bit
        loads, default) or ``"bulk"`` (TMA bulk copies into a shared-memory ring)."""
        if mode not in self.STAGING:
            raise ValueError("staging must be 'register' or 'bulk'")
        _lib.check(self._lib.jabas_ctx_set_staging(self._h, self.STAGING[mode]))
        self.staging = mode

    def staging_timeouts(self) -> int:
        """Bulk staging: number of CTAs whose bounded wait for a copy ran out since the
        context was created (synchronises the device; 0 when all is well)."""
        c = ctypes.c_uint32(0)
        _lib.check(self._lib.jabas_ctx_staging_timeouts(self._h, ctypes.byref(c)))
        return int(c.value)

    def set_wait_limits(self, staging_ms: float = 50.0, peer_ms: float = 5000.0) -> None:
        """Wall-time limits of the device-side waits: for a bulk copy into the shared-memory ring
        and for another GPU's progress inside the pipelined exchange.  A wait that runs out is
        reported (``staging_timeouts`` / ``Exchange.status``), never trapped."""
        _lib.check(self._lib.jabas_ctx_set_wait_limits(self._h, float(staging_ms), float(peer_ms)))

    def inject_staging_stall(self, on: bool) -> None:
        """Test seam: the bulk-staged kernels' stage barriers expect more bytes than are copied."""
        _lib.check(self._lib.jabas_ctx_inject_staging_stall(self._h, int(bool(on))))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.jabas_ctx_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover - interpreter shutdown order
        try:
            self.close()
        except Exception:
            pass


class Layout:
    """Device copy of a segment table ``[(begin, end, group), ...]`` over a flat buffer."""

    def __init__(self, ctx: Context, segments: Sequence[Sequence[int]], total: int):
        self.ctx = ctx
        self.segments = [tuple(int(x) for x in s) for s in segments]
        self.total = int(total)
        arr = (_lib.Seg * len(self.segments))()
        for i, (b, e, g) in enumerate(self.segments):
            arr[i].begin, arr[i].end, arr[i].group = b, e, g
        h = ctypes.c_void_p()
        _lib.check(ctx._lib.jabas_layout_create(ctx._h, arr, len(self.segments), self.total,
                                                ctypes.byref(h)))
        self._h = h

    def close(self) -> None:
        if getattr(self, "_h", None):
            self.ctx._lib.jabas_layout_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


class DynHp:
    """Device-resident hyper-parameters for update launches captured in a CUDA graph: pass
    it as ``dynamic=`` when capturing, then call ``push_sgd`` / ``push_adam`` before every
    replay (outside the graph) with the values of that iteration."""

    def __init__(self, ctx: Context):
        self.ctx = ctx
        h = ctypes.c_void_p()
        _lib.check(ctx._lib.jabas_dynhp_create(ctx._h, ctypes.byref(h)))
        self._h = h

    def push_sgd(self, groups: Sequence[dict], *, momentum: float = 0.0, dampening: float = 0.0,
                 nesterov: bool = False, first_step: bool = False, stream=None) -> None:
        hp = _lib.SgdHp(momentum, dampening, int(nesterov), int(first_step), None, None, 0, 0)
        _lib.check(self.ctx._lib.jabas_dynhp_push_sgd(self._h, _groups_array(groups), len(groups),
                                                      ctypes.byref(hp), _stream_handle(self.ctx.device, stream)))

    def push_adam(self, groups: Sequence[dict], *, beta1: float, beta2: float, eps: float,
                  decoupled: bool, stream=None) -> None:
        hp = _lib.AdamHp(beta1, beta2, eps, int(decoupled), 0, None, None, 0, 0)
        _lib.check(self.ctx._lib.jabas_dynhp_push_adam(self._h, _groups_array(groups), len(groups),
                                                       ctypes.byref(hp), _stream_handle(self.ctx.device, stream)))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self.ctx._lib.jabas_dynhp_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


def _groups_array(groups: Sequence[dict]):
    if not 1 <= len(groups) <= MAX_GROUPS:
        raise JabasError(f"between 1 and {MAX_GROUPS} param groups per launch")
    arr = (_lib.Group * len(groups))()
    for i, g in enumerate(groups):
        arr[i].lr = float(g["lr"])
        arr[i].weight_decay = float(g.get("weight_decay", 0.0))
        arr[i].step = int(g.get("step", 0))
    return arr


def vsw_aggregate(ctx: Context, grads: Sequence[torch.Tensor], out: torch.Tensor, divisor: float, *,
                  half_out: Optional[torch.Tensor] = None, half_divisor: float = 1.0,
                  stat: Optional[torch.Tensor] = None, n: Optional[int] = None,
                  stream: Optional[torch.cuda.Stream] = None) -> None:
    """out = (sum_k grads[k]) / divisor; half_out = the sum; stat += VSW-parity statistic."""
    n = out.numel() if n is None else n
    gp = _ptr_array([_dev_f32(g, ctx.device, "grads[k]") for g in grads])
    _lib.check(ctx._lib.jabas_vsw_aggregate_f32(
        ctx._h, gp, len(grads), _dev_f32(out, ctx.device, "out"),
        None if half_out is None else _dev_f32(half_out, ctx.device, "half_out"),
        n, divisor, half_divisor, _stat_ptr(stat, ctx.device), _stream_handle(ctx.device, stream)))


def div_(ctx: Context, x: torch.Tensor, divisor: float, *, stream=None) -> None:
    _lib.check(ctx._lib.jabas_div_f32(ctx._h, _dev_f32(x, ctx.device, "x"), x.numel(), divisor,
                                      _stream_handle(ctx.device, stream)))


def sgd_momentum(ctx: Context, g: torch.Tensor, weights: Sequence[torch.Tensor],
                 m: Optional[torch.Tensor], groups: Sequence[dict], *, momentum: float = 0.0,
                 dampening: float = 0.0, nesterov: bool = False, first_step: bool = False,
                 layout: Optional[Layout] = None, base: int = 0,
                 half: Optional[torch.Tensor] = None, half_divisor: float = 1.0,
                 stat: Optional[torch.Tensor] = None, grad_scale: Optional[torch.Tensor] = None,
                 dynamic: Optional["DynHp"] = None, stream=None) -> None:
    """Fused SGD-momentum update of ``weights[0]`` with write-back to every replica."""
    hp = _lib.SgdHp(momentum, dampening, int(nesterov), int(first_step), _scale_ptr(grad_scale, ctx.device), _dyn_ptr(dynamic), 0, 0)
    wp = _ptr_array([_dev_f32(w, ctx.device, "weights[k]") for w in weights])
    _lib.check(ctx._lib.jabas_sgd_momentum_f32(
        ctx._h, None if g is None else _dev_f32(g, ctx.device, "g"), wp, len(weights),
        None if m is None else _dev_f32(m, ctx.device, "m"), weights[0].numel(), base,
        None if layout is None else layout._h, _groups_array(groups), len(groups), ctypes.byref(hp),
        None if half is None else _dev_f32(half, ctx.device, "half"), half_divisor,
        _stat_ptr(stat, ctx.device), _stream_handle(ctx.device, stream)))


def adam(ctx: Context, g: torch.Tensor, weights: Sequence[torch.Tensor], m: torch.Tensor,
         v: torch.Tensor, groups: Sequence[dict], *, beta1: float, beta2: float, eps: float,
         decoupled: bool, layout: Optional[Layout] = None, base: int = 0,
         half: Optional[torch.Tensor] = None, half_divisor: float = 1.0,
         stat: Optional[torch.Tensor] = None, grad_scale: Optional[torch.Tensor] = None,
         dynamic: Optional["DynHp"] = None, stream=None) -> None:
    """Fused Adam (``decoupled=False``) / AdamW (``True``) update with write-back."""
    hp = _lib.AdamHp(beta1, beta2, eps, int(decoupled), 0, _scale_ptr(grad_scale, ctx.device), _dyn_ptr(dynamic), 0, 0)
    wp = _ptr_array([_dev_f32(w, ctx.device, "weights[k]") for w in weights])
    _lib.check(ctx._lib.jabas_adam_f32(
        ctx._h, None if g is None else _dev_f32(g, ctx.device, "g"), wp, len(weights),
        _dev_f32(m, ctx.device, "m"), _dev_f32(v, ctx.device, "v"), weights[0].numel(), base,
        None if layout is None else layout._h,
        _groups_array(groups), len(groups), ctypes.byref(hp),
        None if half is None else _dev_f32(half, ctx.device, "half"), half_divisor,
        _stat_ptr(stat, ctx.device), _stream_handle(ctx.device, stream)))


MAX_FUSED_VSW = 8


def vsw_sgd_momentum(ctx: Context, grads: Sequence[torch.Tensor], divisor: float,
                     weights: Sequence[torch.Tensor], m: Optional[torch.Tensor], groups: Sequence[dict], *,
                     momentum: float = 0.0, dampening: float = 0.0, nesterov: bool = False,
                     first_step: bool = False, layout: Optional[Layout] = None, base: int = 0,
                     grad_out: Optional[torch.Tensor] = None, half_divisor: float = 1.0,
                     stat: Optional[torch.Tensor] = None, grad_scale: Optional[torch.Tensor] = None,
                     dynamic: Optional["DynHp"] = None, stream=None) -> None:
    """Single-GPU path in one launch: aggregate the VSW gradients, update, write back."""
    hp = _lib.SgdHp(momentum, dampening, int(nesterov), int(first_step), _scale_ptr(grad_scale, ctx.device), _dyn_ptr(dynamic), int(any(isinstance(g, int) for g in grads)), 0)
    gp = _ptr_array([_dev_f32(g, ctx.device, "grads[k]") for g in grads])
    wp = _ptr_array([_dev_f32(w, ctx.device, "weights[k]") for w in weights])
    _lib.check(ctx._lib.jabas_vsw_sgd_momentum_f32(
        ctx._h, gp, len(grads), divisor,
        None if grad_out is None else _dev_f32(grad_out, ctx.device, "grad_out"), wp, len(weights),
        None if m is None else _dev_f32(m, ctx.device, "m"), weights[0].numel(), base,
        None if layout is None else layout._h, _groups_array(groups), len(groups), ctypes.byref(hp),
        half_divisor, _stat_ptr(stat, ctx.device), _stream_handle(ctx.device, stream)))


def vsw_adam(ctx: Context, grads: Sequence[torch.Tensor], divisor: float,
             weights: Sequence[torch.Tensor], m: torch.Tensor, v: torch.Tensor, groups: Sequence[dict], *,
             beta1: float, beta2: float, eps: float, decoupled: bool, layout: Optional[Layout] = None,
             base: int = 0, grad_out: Optional[torch.Tensor] = None, half_divisor: float = 1.0,
             stat: Optional[torch.Tensor] = None, grad_scale: Optional[torch.Tensor] = None,
             dynamic: Optional["DynHp"] = None, stream=None) -> None:
    """Adam / AdamW counterpart of :func:`vsw_sgd_momentum`."""
    hp = _lib.AdamHp(beta1, beta2, eps, int(decoupled), 0, _scale_ptr(grad_scale, ctx.device), _dyn_ptr(dynamic), int(any(isinstance(g, int) for g in grads)), 0)
    gp = _ptr_array([_dev_f32(g, ctx.device, "grads[k]") for g in grads])
    wp = _ptr_array([_dev_f32(w, ctx.device, "weights[k]") for w in weights])
    _lib.check(ctx._lib.jabas_vsw_adam_f32(
        ctx._h, gp, len(grads), divisor,
        None if grad_out is None else _dev_f32(grad_out, ctx.device, "grad_out"), wp, len(weights),
        _dev_f32(m, ctx.device, "m"), _dev_f32(v, ctx.device, "v"), weights[0].numel(), base,
        None if layout is None else layout._h, _groups_array(groups), len(groups), ctypes.byref(hp),
        half_divisor, _stat_ptr(stat, ctx.device), _stream_handle(ctx.device, stream)))


def dot_norms(ctx: Context, a: torch.Tensor, b: torch.Tensor, stat: torch.Tensor, *, stream=None) -> None:
    _lib.check(ctx._lib.jabas_dot_norms_f32(ctx._h, _dev_f32(a, ctx.device, "a"),
                                            _dev_f32(b, ctx.device, "b"), a.numel(),
                                            _stat_ptr(stat, ctx.device),
                                            _stream_handle(ctx.device, stream)))


def sumsq(ctx: Context, x: torch.Tensor, stat: torch.Tensor, *, stream=None) -> None:
    """stat[0..2] += sum of squares of x (fp64)."""
    _lib.check(ctx._lib.jabas_sumsq_f32(ctx._h, _dev_f32(x, ctx.device, "x"), x.numel(),
                                        _stat_ptr(stat, ctx.device), _stream_handle(ctx.device, stream)))


def clip_coef(ctx: Context, sumsq_stat: torch.Tensor, max_norm: float, coef_out: torch.Tensor, *,
              stream=None) -> None:
    """coef_out[0] = max_norm / (sqrt(sumsq) + 1e-6), coef_out[1] = the norm (fp32, 2 elements)."""
    if coef_out.numel() < 2:
        raise JabasError("coef_out needs two float32 elements (coefficient, norm)")
    _lib.check(ctx._lib.jabas_clip_coef(ctx._h, _stat_ptr(sumsq_stat, ctx.device), max_norm,
                                        _dev_f32(coef_out, ctx.device, "coef_out"),
                                        _stream_handle(ctx.device, stream)))


EXCHANGE_PIECE = _lib.EXCHANGE_PIECE


def exchange_flag_words(max_slots: int) -> int:
    """uint32 words of one rank's flag block for an exchange with ``max_slots`` piece slots."""
    return int(_lib.load().jabas_exchange_flag_words(int(max_slots)))


class Exchange:
    """One rank's handle on the pipelined cross-GPU exchange (``jabas_exchange_*``).

    ``px``, ``pg`` and ``flags`` are lists of raw device pointers, one per rank in rank order, all
    addressable from this GPU (peer mappings for the other ranks); the flag blocks must be zero
    before the first launch on any rank."""

    def __init__(self, ctx: Context, nranks: int, rank: int, px: Sequence[int], pg: Sequence[int],
                 flags: Sequence[int], max_slots: int, window_pieces: int = 0, piece_elems: int = EXCHANGE_PIECE,
                 update_lag: int = 0):
        self.ctx, self.nranks, self.rank = ctx, int(nranks), int(rank)
        self.max_slots, self.window, self.piece = int(max_slots), int(window_pieces), int(piece_elems)
        self._px, self._pg, self._fl = _ptr_array(px), _ptr_array(pg), _ptr_array(flags)
        desc = _lib.ExchangeDesc(self.nranks, self.rank, self._px, self._pg, self._fl, self.max_slots, self.window,
                                 self.piece, int(update_lag))
        h = ctypes.c_void_p()
        _lib.check(ctx._lib.jabas_exchange_create(ctx._h, ctypes.byref(desc), ctypes.byref(h)))
        self._h = h

    def slots_for(self, n: int) -> int:
        """Piece slots a launch over ``n`` elements occupies."""
        return -(-int(n) // self.piece)

    def status(self):
        """(status word, completed launches); synchronises the device.  Status 0: no wait ran out."""
        st, la = ctypes.c_uint32(0), ctypes.c_uint32(0)
        _lib.check(self.ctx._lib.jabas_exchange_status(self._h, ctypes.byref(st), ctypes.byref(la)))
        return int(st.value), int(la.value)

    def reset(self) -> None:
        _lib.check(self.ctx._lib.jabas_exchange_reset(self._h))

    def set_ctas_per_sm(self, ctas: int) -> None:
        """Kernel variant: 2 resident CTAs per SM (96 KB ring, default) or 3 (64 KB ring)."""
        _lib.check(self.ctx._lib.jabas_exchange_set_ctas_per_sm(self._h, int(ctas)))

    def set_grid_limit(self, max_ctas: int) -> None:
        """Largest grid of the following launches (0: the whole GPU)."""
        _lib.check(self.ctx._lib.jabas_exchange_set_grid_limit(self._h, int(max_ctas)))

    def set_trace(self, buf: Optional[torch.Tensor]) -> None:
        """Timeline tracing: ``buf`` is an int64 CUDA tensor of 6 words per ticket (None: off)."""
        if buf is None:
            _lib.check(self.ctx._lib.jabas_exchange_set_trace(self._h, None, 0))
        else:
            assert buf.dtype == torch.int64 and buf.is_cuda and buf.is_contiguous()
            _lib.check(self.ctx._lib.jabas_exchange_set_trace(self._h, buf.data_ptr(), buf.numel() // 6))
        self._trace = buf

    def close(self) -> None:
        if getattr(self, "_h", None):
            self.ctx._lib.jabas_exchange_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


def _exchange_bufs(ctx, grads, weights, m, v, stat):
    gp = _ptr_array([_dev_f32(g, ctx.device, "grads[k]") for g in grads])
    wp = _ptr_array([_dev_f32(w, ctx.device, "weights[k]") for w in weights])
    b = _lib.ExchangeBufs(gp, len(grads), len(weights), wp,
                          None if m is None else _dev_f32(m, ctx.device, "m"),
                          None if v is None else _dev_f32(v, ctx.device, "v"), _stat_ptr(stat, ctx.device))
    return b, (gp, wp)


def exchange_step(exs: Sequence[Exchange], bufs: Sequence[dict], n: int, base: int, slot_base: int,
                  divisor: float, half_divisor: float, groups: Sequence[dict], *, kind: str,
                  layout: Optional[Layout] = None, momentum: float = 0.0, dampening: float = 0.0,
                  nesterov: bool = False, first_step: bool = False, beta1: float = 0.9, beta2: float = 0.999,
                  eps: float = 1e-8, dynamic: Optional["DynHp"] = None, stream=None) -> None:
    """One launch of the pipelined exchange over elements ``[base, base + n)`` of the flat buffers.

    ``exs`` / ``bufs`` hold ONE entry in production (this GPU's rank; ``bufs[i]`` is a dict with
    ``grads`` (K flat VSW gradient buffers), ``weights`` (replicas), ``m``, ``v``, ``stat``) or
    one entry per rank when all ranks live on this GPU (single-GPU tests of the protocol).
    ``kind`` is ``"sgd"``, ``"adam"`` or ``"adamw"``."""
    ctx = exs[0].ctx
    keep, arr = [], (_lib.ExchangeBufs * len(exs))()
    for i, b in enumerate(bufs):
        arr[i], k = _exchange_bufs(ctx, b["grads"], b["weights"], b.get("m"), b.get("v"), b.get("stat"))
        keep.append(k)
    hs = _ptr_array([e._h.value for e in exs])
    sgd = adam = None
    if kind == "sgd":
        sgd = ctypes.pointer(_lib.SgdHp(momentum, dampening, int(nesterov), int(first_step), None, _dyn_ptr(dynamic), 0, 0))
    else:
        adam = ctypes.pointer(_lib.AdamHp(beta1, beta2, eps, int(kind == "adamw"), 0, None, _dyn_ptr(dynamic), 0, 0))
    _lib.check(ctx._lib.jabas_exchange_step_f32(
        hs, arr, len(exs), int(n), int(base), int(slot_base), float(divisor), float(half_divisor),
        None if layout is None else layout._h, _groups_array(groups), len(groups), sgd, adam,
        _stream_handle(ctx.device, stream)))


def exchange_cosine(exs: Sequence[Exchange], stats: Sequence[torch.Tensor], cos_outs: Sequence[torch.Tensor], *,
                    eps: float = 1e-8, stream=None) -> None:
    """Sum the ranks' three statistic sums (rank order, identical everywhere) and finalize the cosine."""
    ctx = exs[0].ctx
    hs = _ptr_array([e._h.value for e in exs])
    sp = _ptr_array([_stat_ptr(s, ctx.device) for s in stats])
    cp = _ptr_array([_dev_f32(c, ctx.device, "cos_out") for c in cos_outs])
    _lib.check(ctx._lib.jabas_exchange_cosine(hs, sp, cp, len(exs), eps, _stream_handle(ctx.device, stream)))


STATIC_MAX_ELEMS = 1 << 31


def dot_norms_static(a: torch.Tensor, b: torch.Tensor, stat: torch.Tensor, *, stream=None) -> None:
    """``stat += (<a,b>, |a|^2, |b|^2)`` without a context and without any device allocation.

    For callers that cannot allocate when they need the statistic (the process's allocator
    already owns the device, or a synchronising ``cudaMalloc`` is not acceptable where they
    are): the reduction scratch is a static array inside the library.  At most
    ``STATIC_MAX_ELEMS`` elements per call; all calls share the scratch, so calls that can
    overlap on the GPU (different streams) must be ordered by the caller.  The first call on
    a device resolves the scratch address and should come before any stream capture."""
    dev = a.device
    _lib.check(_lib.load().jabas_dot_norms_static_f32(
        _dev_f32(a, dev, "a"), _dev_f32(b, dev, "b"), a.numel(), _stat_ptr(stat, dev),
        _stream_handle(dev, stream)))


def cosine_finalize(ctx: Context, stat: torch.Tensor, cos_out: torch.Tensor, *, eps: float = 1e-8,
                    stream=None) -> None:
    _lib.check(ctx._lib.jabas_cosine_finalize(ctx._h, _stat_ptr(stat, ctx.device), eps,
                                              _dev_f32(cos_out, ctx.device, "cos_out"),
                                              _stream_handle(ctx.device, stream)))


def replicate(ctx: Context, src: torch.Tensor, dsts: Sequence[torch.Tensor], *, stream=None) -> None:
    dp = _ptr_array([_dev_f32(d, ctx.device, "dsts[k]") for d in dsts])
    _lib.check(ctx._lib.jabas_replicate_f32(ctx._h, _dev_f32(src, ctx.device, "src"), dp, len(dsts),
                                            src.numel(), _stream_handle(ctx.device, stream)))


__all__ = ["Context", "Layout", "DynHp", "Exchange", "exchange_step", "exchange_cosine", "exchange_flag_words", "EXCHANGE_PIECE", "JabasError", "MAX_VSW", "MAX_GROUPS", "vsw_aggregate", "div_",
           "sgd_momentum", "adam", "vsw_sgd_momentum", "vsw_adam", "MAX_FUSED_VSW", "sumsq", "clip_coef", "dot_norms", "dot_norms_static", "cosine_finalize", "replicate"]
