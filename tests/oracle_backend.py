"""A stand-in for ``jabas_b200.ops`` that runs the CPU oracle on CPU tensors.

TEST DOUBLE ONLY: it lets the host-side logic (bucket readiness, hook ordering, interval
gating, process-group construction) run as gloo ranks on a machine without a GPU.  The
product has no such path — ``jabas_b200.ops`` refuses anything that is not a CUDA tensor.
"""
import numpy as np
import torch

from oracle import gradpath as O


class Context:
    def __init__(self, device=None):
        self.device = torch.device("cpu")

    def close(self):
        pass


class Layout:
    def __init__(self, ctx, segments, total):
        self.segments, self.total = [tuple(s) for s in segments], total

    def close(self):
        pass


def _np(t):
    return t.detach().numpy()


def vsw_aggregate(ctx, grads, out, divisor, *, half_out=None, half_divisor=1.0, stat=None, n=None, stream=None):
    gs = [_np(g) for g in grads]
    if stat is not None:
        O.vsw_parity_stat(gs, half_divisor, _np(stat))
    O.vsw_aggregate(gs, _np(out), divisor, None if half_out is None else _np(half_out))


def div_(ctx, x, divisor, *, stream=None):
    O.div_(_np(x), divisor)


def _segments(layout, base, n):
    if layout is None:
        return [(0, n, 0)]
    out = []
    for b, e, g in layout.segments:
        lo, hi = max(b, base), min(e, base + n)
        if lo < hi:
            out.append((lo - base, hi - base, g))
    return out


def _replicate(weights):
    for w in weights[1:]:
        w.copy_(weights[0])


def sgd_momentum(ctx, g, weights, m, groups, *, momentum=0.0, dampening=0.0, nesterov=False,
                 first_step=False, layout=None, base=0, half=None, half_divisor=1.0, stat=None, grad_scale=None,
                 dynamic=None, stream=None):
    if stat is not None:
        O.half_stat(_np(g), _np(half), half_divisor, _np(stat))
    g = _scaled(g, grad_scale)
    mm = _np(m) if m is not None else np.zeros(g.numel(), np.float32)
    O.update_segments("sgd", _np(g), _np(weights[0]), mm, None, _segments(layout, base, g.numel()),
                      [dict(lr=x["lr"], weight_decay=x.get("weight_decay", 0.0)) for x in groups],
                      momentum=momentum, dampening=dampening, nesterov=nesterov, first_step=first_step)
    _replicate(weights)


def adam(ctx, g, weights, m, v, groups, *, beta1, beta2, eps, decoupled, layout=None, base=0,
         half=None, half_divisor=1.0, stat=None, grad_scale=None, dynamic=None, stream=None):
    if stat is not None:
        O.half_stat(_np(g), _np(half), half_divisor, _np(stat))
    g = _scaled(g, grad_scale)
    O.update_segments("adam", _np(g), _np(weights[0]), _np(m), _np(v), _segments(layout, base, g.numel()),
                      [dict(lr=x["lr"], weight_decay=x.get("weight_decay", 0.0), step=x["step"]) for x in groups],
                      beta1=beta1, beta2=beta2, eps=eps, decoupled=decoupled)
    _replicate(weights)


def sumsq(ctx, x, stat, *, stream=None):
    _np(stat)[:] += O.sumsq(_np(x))


def clip_coef(ctx, sumsq_stat, max_norm, coef_out, *, stream=None):
    total = np.float32(np.sqrt(_np(sumsq_stat)[0]))
    coef_out[0] = float(np.float32(max_norm) / (total + np.float32(1e-6)))
    coef_out[1] = float(total)


def _scaled(g, grad_scale):
    if grad_scale is None or float(grad_scale[0]) >= 1.0:
        return g
    return (g * grad_scale[0]).to(torch.float32)


def dot_norms(ctx, a, b, stat, *, stream=None):
    O.dot_norms(_np(a), _np(b), _np(stat))


def cosine_finalize(ctx, stat, cos_out, *, eps=1e-8, stream=None):
    cos_out[0] = O.cosine_from_stat(_np(stat), eps)


def replicate(ctx, src, dsts, *, stream=None):
    for d in dsts:
        if d.data_ptr() != src.data_ptr():
            d.copy_(src)


MAX_FUSED_VSW = 8


def vsw_sgd_momentum(ctx, grads, divisor, weights, m, groups, *, grad_out=None, half_divisor=1.0, stat=None,
                     **kw):
    g = torch.empty_like(weights[0]) if grad_out is None else grad_out
    vsw_aggregate(ctx, grads, g, divisor, half_divisor=half_divisor, stat=stat)
    sgd_momentum(ctx, g, weights, m, groups, **kw)


def vsw_adam(ctx, grads, divisor, weights, m, v, groups, *, grad_out=None, half_divisor=1.0, stat=None, **kw):
    g = torch.empty_like(weights[0]) if grad_out is None else grad_out
    vsw_aggregate(ctx, grads, g, divisor, half_divisor=half_divisor, stat=stat)
    adam(ctx, g, weights, m, v, groups, **kw)
