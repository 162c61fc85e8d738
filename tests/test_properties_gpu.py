"""Property tests of the kernels against the oracle: random K, sizes, alignments, segment
tables, sub-range launches."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from oracle import gradpath as O

pytestmark = pytest.mark.gpu
_CTX = {}


def _ctx():
    from jabas_b200 import ops
    if "c" not in _CTX:
        _CTX["c"] = ops.Context(0)
    return _CTX["c"]


def _dev(a, offset):
    t = torch.empty(a.size + offset, dtype=torch.float32, device="cuda")
    v = t[offset:]
    v.copy_(torch.from_numpy(a))
    return v


@settings(max_examples=40, deadline=None)
@given(K=st.integers(1, 16), n=st.integers(1, 70000), off=st.integers(0, 3), seed=st.integers(0, 2 ** 16),
       T=st.sampled_from([1.0, 2.0, 3.0, 6.0, 8.0, 48.0]))
def test_aggregate_any_shape(K, n, off, seed, T):
    from jabas_b200 import ops
    rng = np.random.default_rng(seed)
    grads = [(rng.standard_normal(n) * 1e-3).astype(np.float32) for _ in range(K)]
    out_o, half_o = np.empty(n, np.float32), np.empty(n, np.float32)
    O.vsw_aggregate(grads, out_o, T, half_o)
    dg = [_dev(g, off) for g in grads]
    out, half = _dev(np.zeros(n, np.float32), off), _dev(np.zeros(n, np.float32), off)
    ops.vsw_aggregate(_ctx(), dg, out, T, half_out=half)
    assert np.array_equal(out.cpu().numpy(), out_o) and np.array_equal(half.cpu().numpy(), half_o)


@settings(max_examples=40, deadline=None)
@given(K=st.integers(1, 8), Kw=st.integers(1, 5), n=st.integers(4, 60000), off=st.integers(0, 1),
       seed=st.integers(0, 2 ** 16), opt=st.sampled_from(["sgd", "adamw", "adam"]), nseg=st.integers(1, 30),
       split=st.floats(0.0, 1.0), fused=st.booleans())
def test_update_any_shape(K, Kw, n, off, seed, opt, nseg, split, fused):
    """Two launches over [0, cut) and [cut, n) of a flat buffer with a random segment table,
    in the two-kernel form or the fused single-launch form; bit-exact against the oracle."""
    from jabas_b200 import ops
    ctx = _ctx()
    rng = np.random.default_rng(seed)
    cuts = sorted(set(int(c) for c in rng.integers(1, n, size=nseg - 1))) if nseg > 1 else []
    edges = [0] + cuts + [n]
    segs = [(edges[i], edges[i + 1], int(rng.integers(0, 3))) for i in range(len(edges) - 1)]
    groups = [dict(lr=0.1, weight_decay=0.0, step=3), dict(lr=0.03, weight_decay=1e-2, step=3),
              dict(lr=0.2, weight_decay=1e-4, step=7)]
    layout = ops.Layout(ctx, segs, n)
    grads = [(rng.standard_normal(n) * 1e-3).astype(np.float32) for _ in range(K)]
    p = rng.standard_normal(n).astype(np.float32)
    m = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    v = np.abs(rng.standard_normal(n) * 1e-6).astype(np.float32)
    T = float(2 * K)
    g = np.empty(n, np.float32)
    O.vsw_aggregate(grads, g, T)
    po, mo, vo = p.copy(), m.copy(), v.copy()
    if opt == "sgd":
        O.update_segments("sgd", g, po, mo, None, segs,
                          [dict(lr=x["lr"], weight_decay=x["weight_decay"]) for x in groups], momentum=0.9, nesterov=True)
    else:
        O.update_segments("adam", g, po, mo, vo, segs, groups, beta1=0.9, beta2=0.999, eps=1e-8,
                          decoupled=(opt == "adamw"))
    dg = [_dev(x, off) for x in grads]
    w = [_dev(p, off)] + [_dev(np.zeros(n, np.float32), off) for _ in range(Kw - 1)]
    dm, dv, davg = _dev(m, off), _dev(v, off), _dev(np.zeros(n, np.float32), off)
    cut = int(split * n)
    if off == 0:
        cut &= ~3                                   # keep the second launch 16-byte aligned
    for b, e in ((0, cut), (cut, n)):
        if e == b:
            continue
        ws = [x[b:e] for x in w]
        if fused:
            if opt == "sgd":
                ops.vsw_sgd_momentum(ctx, [x[b:e] for x in dg], T, ws, dm[b:e], groups, momentum=0.9, nesterov=True,
                                     layout=layout, base=b)
            else:
                ops.vsw_adam(ctx, [x[b:e] for x in dg], T, ws, dm[b:e], dv[b:e], groups, beta1=0.9, beta2=0.999,
                             eps=1e-8, decoupled=(opt == "adamw"), layout=layout, base=b)
        else:
            ops.vsw_aggregate(ctx, [x[b:e] for x in dg], davg[b:e], T)
            if opt == "sgd":
                ops.sgd_momentum(ctx, davg[b:e], ws, dm[b:e], groups, momentum=0.9, nesterov=True, layout=layout, base=b)
            else:
                ops.adam(ctx, davg[b:e], ws, dm[b:e], dv[b:e], groups, beta1=0.9, beta2=0.999, eps=1e-8,
                         decoupled=(opt == "adamw"), layout=layout, base=b)
    for k in range(Kw):
        assert np.array_equal(w[k].cpu().numpy(), po), k
    assert np.array_equal(dm.cpu().numpy(), mo)
    if opt != "sgd":
        assert np.array_equal(dv.cpu().numpy(), vo)
    layout.close()
