"""Parity of every CUDA kernel with the CPU oracle, called through the C ABI.

Bit-exact (``array_equal``) wherever the summation order is fixed: aggregation,
division, the optimizer updates, the write-back.  The statistic sums are compared to
the oracle's fp64 sums at 1e-6 relative and the cosine at 1e-5 absolute (the stated
tolerance of the path).
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import gradpath as O

pytestmark = pytest.mark.gpu

SIZES = [1, 3, 4, 5, 1023, 1025, 2 ** 20 + 1, 3 * 2 ** 20 + 2]


@pytest.fixture(scope="module", params=["register", "bulk"])
def ctx(request):
    """Every test of this module runs twice: with the update kernels loading their tiles
    straight into registers, and through the bulk-copy (TMA) shared-memory ring."""
    from jabas_b200 import ops
    c = ops.Context(0)
    c.set_staging(request.param)
    yield c
    assert c.staging_timeouts() == 0          # no bounded wait for a bulk copy ever ran out
    c.close()


def _rand(rng, n, scale=1.0):
    return (rng.standard_normal(n) * scale).astype(np.float32)


def _dev(a, offset=0):
    """Copy a numpy array to the device; ``offset`` elements of slack give a pointer
    that is only 4-byte aligned, which takes the scalar kernels."""
    t = torch.empty(a.size + offset, dtype=torch.from_numpy(a).dtype, device="cuda")
    v = t[offset:]
    v.copy_(torch.from_numpy(a))
    return v


def _host(t):
    return t.detach().cpu().numpy()


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("K", [1, 2, 3, 4, 5, 8, 9, 16])
def test_aggregate_bit_exact(ctx, n, K):
    from jabas_b200 import ops
    rng = np.random.default_rng(1000 * K + n % 997)
    grads = [_rand(rng, n, 1e-3) for _ in range(K)]
    T = float(2 * K + (K % 3))                       # includes divisors that are not powers of two
    out_o, half_o = np.empty(n, np.float32), np.empty(n, np.float32)
    O.vsw_aggregate(grads, out_o, T, half_o)
    dg = [_dev(g) for g in grads]
    out, half = torch.empty(n, device="cuda"), torch.empty(n, device="cuda")
    ops.vsw_aggregate(ctx, dg, out, T, half_out=half)
    assert np.array_equal(_host(out), out_o)
    assert np.array_equal(_host(half), half_o)
    ops.vsw_aggregate(ctx, dg, dg[0], T)             # in place into the main replica's bucket
    assert np.array_equal(_host(dg[0]), out_o)


@pytest.mark.parametrize("n", [5, 1025, 2 ** 20 + 3])
@pytest.mark.parametrize("K", [2, 3, 4, 8])
def test_aggregate_unaligned_pointers(ctx, n, K):
    from jabas_b200 import ops
    rng = np.random.default_rng(n + K)
    grads = [_rand(rng, n, 1e-3) for _ in range(K)]
    out_o = np.empty(n, np.float32)
    st_o = O.vsw_parity_stat(grads, K / 2)
    O.vsw_aggregate(grads, out_o, float(K))
    dg = [_dev(g, offset=1 + (k % 3)) for k, g in enumerate(grads)]
    out = torch.empty(n + 1, device="cuda")[1:]
    stat = torch.zeros(3, dtype=torch.float64, device="cuda")
    ops.vsw_aggregate(ctx, dg, out, float(K), half_divisor=K / 2, stat=stat)
    assert np.array_equal(_host(out), out_o)
    assert np.allclose(_host(stat), st_o, rtol=1e-6, atol=0)


@pytest.mark.parametrize("n", [4, 1023, 2 ** 20 + 1, 5 * 2 ** 20])
@pytest.mark.parametrize("K", [2, 3, 4, 7, 8, 16])
def test_aggregate_vsw_parity_statistic(ctx, n, K):
    from jabas_b200 import ops
    rng = np.random.default_rng(77 * K + n % 1013)
    common = _rand(rng, n, 1e-3)
    grads = [(_rand(rng, n, 1e-3) + 0.5 * common).astype(np.float32) for _ in range(K)]
    st_o = O.vsw_parity_stat(grads, K / 2)
    dg = [_dev(g) for g in grads]
    out = torch.empty(n, device="cuda")
    stat = torch.zeros(3, dtype=torch.float64, device="cuda")
    cos = torch.zeros(1, device="cuda")
    ops.vsw_aggregate(ctx, dg, out, float(K), half_divisor=K / 2, stat=stat)
    ops.cosine_finalize(ctx, stat, cos)
    first = _host(stat).copy()
    assert np.allclose(first, st_o, rtol=1e-6, atol=0)
    assert abs(float(cos) - O.cosine_from_stat(st_o)) < 1e-5
    stat.zero_()
    ops.vsw_aggregate(ctx, dg, out, float(K), half_divisor=K / 2, stat=stat)
    assert np.array_equal(_host(stat), first)          # run-to-run deterministic
    ops.vsw_aggregate(ctx, dg, out, float(K), half_divisor=K / 2, stat=stat)
    assert np.allclose(_host(stat), 2 * first, rtol=1e-15)   # accumulates across buckets


def _segments(rng, n, ngroups, nseg):
    if n < 2 or nseg < 2:
        return [(0, n, 0)]
    cuts = sorted(set(int(c) for c in rng.integers(1, n, size=nseg - 1)))
    edges = [0] + cuts + [n]
    return [(edges[i], edges[i + 1], int(rng.integers(0, ngroups))) for i in range(len(edges) - 1)]


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("K", [1, 4])
@pytest.mark.parametrize("variant", ["plain", "wd", "nesterov", "dampening", "no_momentum"])
def test_sgd_bit_exact(ctx, n, K, variant):
    from jabas_b200 import ops
    rng = np.random.default_rng(n % 991 + K)
    hp = dict(momentum=0.9, dampening=0.0, nesterov=False)
    wd = 0.0
    if variant == "wd":
        wd = 1e-4
    elif variant == "nesterov":
        hp["nesterov"], wd = True, 5e-5
    elif variant == "dampening":
        hp["dampening"] = 0.1
    elif variant == "no_momentum":
        hp["momentum"] = 0.0
    p, m = _rand(rng, n), np.zeros(n, np.float32)
    w = [_dev(p)] + [torch.full((n,), 7.0, device="cuda") for _ in range(K - 1)]
    dm = None if variant == "no_momentum" else torch.zeros(n, device="cuda")
    for it in range(3):
        g = _rand(rng, n, 1e-3)
        lr = 0.1 / (it + 1)
        O.sgd_momentum(g, p, m, lr=lr, weight_decay=wd, first_step=(it == 0), **hp)
        ops.sgd_momentum(ctx, _dev(g), w, dm, [dict(lr=lr, weight_decay=wd)], first_step=(it == 0), **hp)
        for k in range(K):
            assert np.array_equal(_host(w[k]), p), (it, k)
        if dm is not None:
            assert np.array_equal(_host(dm), m)


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("decoupled", [True, False])
@pytest.mark.parametrize("K", [1, 8])
def test_adam_bit_exact(ctx, n, decoupled, K):
    from jabas_b200 import ops
    rng = np.random.default_rng(n % 983 + K)
    p, m, v = _rand(rng, n), np.zeros(n, np.float32), np.zeros(n, np.float32)
    w = [_dev(p)] + [torch.empty(n, device="cuda") for _ in range(K - 1)]
    dm, dv = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    hp = dict(beta1=0.9, beta2=0.999, eps=1e-8)
    for it in range(3):
        g = _rand(rng, n, 1e-3)
        O.adam(g, p, m, v, lr=2e-3, weight_decay=0.05, step=it + 1, decoupled=decoupled, **hp)
        ops.adam(ctx, _dev(g), w, dm, dv, [dict(lr=2e-3, weight_decay=0.05, step=it + 1)],
                 decoupled=decoupled, **hp)
        assert np.array_equal(_host(dm), m)
        assert np.array_equal(_host(dv), v)
        for k in range(K):
            assert np.array_equal(_host(w[k]), p), (it, k)


@pytest.mark.parametrize("n,nseg", [(7, 3), (1025, 9), (2 ** 20 + 1, 161), (2 ** 20 + 1, 2000)])
@pytest.mark.parametrize("opt", ["sgd", "adamw", "adam"])
@pytest.mark.parametrize("offset", [0, 1])
def test_update_with_segment_table_and_base(ctx, n, nseg, opt, offset):
    """Param-group runs inside a flat buffer, updated in two launches (two 'buckets')
    addressed by ``base``; ``offset=1`` takes the scalar kernels."""
    from jabas_b200 import ops
    rng = np.random.default_rng(n + nseg)
    segs = _segments(rng, n, 3, nseg)
    groups = [dict(lr=0.1, weight_decay=0.0, step=2), dict(lr=0.05, weight_decay=1e-2, step=2),
              dict(lr=0.2, weight_decay=1e-4, step=5)]
    layout = ops.Layout(ctx, segs, n)
    g, p = _rand(rng, n, 1e-3), _rand(rng, n)
    m, v = _rand(rng, n, 1e-3), np.abs(_rand(rng, n, 1e-6))
    dg, dm, dv = _dev(g, offset), _dev(m, offset), _dev(v, offset)
    w = [_dev(p, offset), torch.empty(n + offset, device="cuda")[offset:]]
    if opt == "sgd":
        O.update_segments("sgd", g, p, m, None, segs, [dict(lr=x["lr"], weight_decay=x["weight_decay"]) for x in groups], momentum=0.9)
    else:
        O.update_segments("adam", g, p, m, v, segs, groups, beta1=0.9, beta2=0.999, eps=1e-8,
                          decoupled=(opt == "adamw"))
    cut = (n // 3) & ~3 if offset == 0 else n // 3
    for b, e in ((0, cut), (cut, n)):
        if e == b:
            continue
        ws = [x[b:e] for x in w]
        if opt == "sgd":
            ops.sgd_momentum(ctx, dg[b:e], ws, dm[b:e], groups, momentum=0.9, layout=layout, base=b)
        else:
            ops.adam(ctx, dg[b:e], ws, dm[b:e], dv[b:e], groups, beta1=0.9, beta2=0.999, eps=1e-8,
                     decoupled=(opt == "adamw"), layout=layout, base=b)
    assert np.array_equal(_host(w[0]), p)
    assert np.array_equal(_host(w[1]), p)
    assert np.array_equal(_host(dm), m)
    if opt != "sgd":
        assert np.array_equal(_host(dv), v)
    layout.close()


@pytest.mark.parametrize("n", [3, 1025, 2 ** 20 + 1, 6 * 2 ** 20])
@pytest.mark.parametrize("opt", ["sgd", "adamw"])
def test_update_fused_half_statistic(ctx, n, opt):
    from jabas_b200 import ops
    rng = np.random.default_rng(n % 977)
    T = 8.0
    sum_e, sum_o = _rand(rng, n, 1e-3), _rand(rng, n, 1e-3)
    sum_o += 0.4 * sum_e
    g = ((sum_e + sum_o) / np.float32(T)).astype(np.float32)
    st_o = O.half_stat(g, sum_e, T / 2)
    p = _rand(rng, n)
    w = [_dev(p)]
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    stat = torch.zeros(3, dtype=torch.float64, device="cuda")
    cos = torch.zeros(1, device="cuda")
    if opt == "sgd":
        po, mo = p.copy(), np.zeros(n, np.float32)
        O.sgd_momentum(g, po, mo, lr=0.1, momentum=0.9, first_step=True)
        ops.sgd_momentum(ctx, _dev(g), w, m, [dict(lr=0.1)], momentum=0.9, first_step=True,
                         half=_dev(sum_e), half_divisor=T / 2, stat=stat)
    else:
        po, mo, vo = p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
        O.adam(g, po, mo, vo, lr=1e-3, weight_decay=0.05, beta1=0.9, beta2=0.999, eps=1e-8, step=1,
               decoupled=True)
        ops.adam(ctx, _dev(g), w, m, v, [dict(lr=1e-3, weight_decay=0.05, step=1)], beta1=0.9,
                 beta2=0.999, eps=1e-8, decoupled=True, half=_dev(sum_e), half_divisor=T / 2, stat=stat)
    ops.cosine_finalize(ctx, stat, cos)
    assert np.array_equal(_host(w[0]), po)              # the statistic does not disturb the update
    assert np.allclose(_host(stat), st_o, rtol=1e-6, atol=0)
    assert abs(float(cos) - O.cosine_from_stat(st_o)) < 1e-5
    # and it agrees with the pair-exchange form of the reference (E on rank 0, O on rank 1)
    e, o = sum_e / np.float32(T / 2), sum_o / np.float32(T / 2)
    assert abs(float(cos) - O.cosine_from_stat(O.dot_norms(e, o))) < 1e-5


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("offset", [0, 1])
def test_dot_norms_div_replicate(ctx, n, offset):
    from jabas_b200 import ops
    rng = np.random.default_rng(n % 971)
    a, b = _rand(rng, n, 1e-3), _rand(rng, n, 1e-3)
    da, db = _dev(a, offset), _dev(b, offset)
    stat = torch.zeros(3, dtype=torch.float64, device="cuda")
    ops.dot_norms(ctx, da, db, stat)
    assert np.allclose(_host(stat), O.dot_norms(a, b), rtol=1e-6, atol=1e-30)
    ops.div_(ctx, da, 6.0)
    O.div_(a, 6.0)
    assert np.array_equal(_host(da), a)
    d1, d2 = torch.zeros(n + offset, device="cuda")[offset:], torch.zeros(n, device="cuda")
    ops.replicate(ctx, da, [d1, da, d2])
    assert np.array_equal(_host(d1), a) and np.array_equal(_host(d2), a)


def test_cosine_finalize_known_answers(ctx):
    from jabas_b200 import ops
    cos = torch.zeros(1, device="cuda")
    for st in ([1.0, 1.0, 1.0], [-2.0, 4.0, 1.0], [0.0, 3.0, 5.0], [1e-12, 1e-12, 1e-12], [0.0, 0.0, 0.0]):
        ops.cosine_finalize(ctx, torch.tensor(st, dtype=torch.float64, device="cuda"), cos)
        assert float(cos) == O.cosine_from_stat(np.array(st))


def test_argument_errors_are_reported_not_launched(ctx):
    """Bad arguments come back as JABAS_EINVAL with a message; nothing reaches the GPU."""
    from jabas_b200 import ops, JabasError
    x = torch.zeros(8, device="cuda")
    with pytest.raises(JabasError, match="K must be"):
        ops.vsw_aggregate(ctx, [x] * 17, x, 1.0)
    with pytest.raises(JabasError, match="divisor"):
        ops.vsw_aggregate(ctx, [x], x, 0.0)
    with pytest.raises(JabasError, match="K >= 2"):
        ops.vsw_aggregate(ctx, [x], x, 1.0, stat=torch.zeros(3, dtype=torch.float64, device="cuda"))
    with pytest.raises(JabasError, match="momentum buffer"):
        ops.sgd_momentum(ctx, x, [x], None, [dict(lr=0.1)], momentum=0.9)
    with pytest.raises(JabasError, match="both"):
        ops.sgd_momentum(ctx, x, [x], x.clone(), [dict(lr=0.1)], momentum=0.9, half=x)
    with pytest.raises(JabasError, match="step"):
        ops.adam(ctx, x, [x], x.clone(), x.clone(), [dict(lr=0.1, step=0)], beta1=0.9, beta2=0.999,
                 eps=1e-8, decoupled=True)
    with pytest.raises(JabasError, match="contiguous"):
        ops.div_(ctx, torch.zeros(8, 2, device="cuda")[:, 0], 2.0)
    with pytest.raises(JabasError, match="no CPU path"):
        ops.div_(ctx, torch.zeros(8), 2.0)
    with pytest.raises(JabasError, match="contiguous from 0"):
        ops.Layout(ctx, [(0, 4, 0), (5, 8, 1)], 8)
    with pytest.raises(JabasError, match="cover"):
        ops.Layout(ctx, [(0, 4, 0)], 8)
    lay = ops.Layout(ctx, [(0, 8, 0)], 8)
    with pytest.raises(JabasError, match="exceeds"):
        ops.sgd_momentum(ctx, x, [x], x.clone(), [dict(lr=0.1)], momentum=0.9, layout=lay, base=4)
    ops.vsw_aggregate(ctx, [x], x, 1.0, n=0)            # empty input: accepted, no launch
    torch.cuda.synchronize()


def test_streams_have_independent_statistic_workspaces(ctx):
    from jabas_b200 import ops
    rng = np.random.default_rng(9)
    n = 2 ** 21 + 5
    a, b = _rand(rng, n), _rand(rng, n)
    da, db = _dev(a), _dev(b)
    ref = O.dot_norms(a, b)
    streams = [torch.cuda.Stream() for _ in range(4)]
    stats = [torch.zeros(3, dtype=torch.float64, device="cuda") for _ in streams]
    torch.cuda.synchronize()
    for _ in range(5):
        for s, st in zip(streams, stats):
            ops.dot_norms(ctx, da, db, st, stream=s)
    torch.cuda.synchronize()
    for st in stats:
        assert np.allclose(_host(st), 5 * ref, rtol=1e-6)
        assert np.array_equal(_host(st), _host(stats[0]))


@pytest.mark.parametrize("n", [3, 1025, 2 ** 20 + 1, 5 * 2 ** 20 + 2])
@pytest.mark.parametrize("K", [1, 2, 4, 5, 8])
@pytest.mark.parametrize("opt", ["sgd", "adamw", "adam"])
@pytest.mark.parametrize("offset", [0, 1])
def test_fused_aggregate_update_equals_two_kernel_path(ctx, n, K, opt, offset):
    """Single-GPU form: one launch must reproduce aggregate -> update bit for bit, with
    param-group segments, write-back to all replicas and the VSW-parity statistic."""
    from jabas_b200 import ops
    if offset and n > 2 ** 20 + 1:
        pytest.skip("scalar kernels are covered by the smaller sizes")
    rng = np.random.default_rng(n % 953 + 7 * K)
    segs = _segments(rng, n, 2, 40)
    layout = ops.Layout(ctx, segs, n)
    groups = [dict(lr=0.1, weight_decay=0.0, step=3), dict(lr=0.05, weight_decay=1e-2, step=3)]
    common = _rand(rng, n, 1e-3)
    grads = [(_rand(rng, n, 1e-3) + 0.5 * common).astype(np.float32) for _ in range(K)]
    p, m, v = _rand(rng, n), _rand(rng, n, 1e-3), np.abs(_rand(rng, n, 1e-6))
    T = float(2 * K)
    g = np.empty(n, np.float32)
    O.vsw_aggregate(grads, g, T)
    st_o = O.vsw_parity_stat(grads, T / 2) if K >= 2 else None
    if opt == "sgd":
        O.update_segments("sgd", g, p_o := p.copy(), m_o := m.copy(), None, segs,
                          [dict(lr=x["lr"], weight_decay=x["weight_decay"]) for x in groups], momentum=0.9)
        v_o = v
    else:
        O.update_segments("adam", g, p_o := p.copy(), m_o := m.copy(), v_o := v.copy(), segs, groups,
                          beta1=0.9, beta2=0.999, eps=1e-8, decoupled=(opt == "adamw"))
    dg = [_dev(x, offset) for x in grads]
    w = [_dev(p, offset)] + [torch.empty(n + offset, device="cuda")[offset:] for _ in range(2)]
    dm, dv = _dev(m, offset), _dev(v, offset)
    gout = torch.empty(n + offset, device="cuda")[offset:]
    stat = torch.zeros(3, dtype=torch.float64, device="cuda") if K >= 2 else None
    kw = dict(layout=layout, grad_out=gout, half_divisor=T / 2, stat=stat)
    if opt == "sgd":
        ops.vsw_sgd_momentum(ctx, dg, T, w, dm, groups, momentum=0.9, **kw)
    else:
        ops.vsw_adam(ctx, dg, T, w, dm, dv, groups, beta1=0.9, beta2=0.999, eps=1e-8,
                     decoupled=(opt == "adamw"), **kw)
    assert np.array_equal(_host(gout), g)
    for k in range(3):
        assert np.array_equal(_host(w[k]), p_o), k
    assert np.array_equal(_host(dm), m_o)
    assert np.array_equal(_host(dv), v_o)
    if K >= 2:
        assert np.allclose(_host(stat), st_o, rtol=1e-6, atol=0)
    layout.close()


def test_fused_form_argument_errors(ctx):
    from jabas_b200 import ops, JabasError
    x = torch.zeros(64, device="cuda")
    with pytest.raises(JabasError, match="1..8"):
        ops.vsw_sgd_momentum(ctx, [x] * 9, 9.0, [x.clone()], x.clone(), [dict(lr=0.1)], momentum=0.9)
    with pytest.raises(JabasError, match="divisor"):
        ops.vsw_sgd_momentum(ctx, [x] * 2, 0.0, [x.clone()], x.clone(), [dict(lr=0.1)], momentum=0.9)
    with pytest.raises(JabasError, match="K >= 2"):
        ops.vsw_sgd_momentum(ctx, [x], 1.0, [x.clone()], x.clone(), [dict(lr=0.1)], momentum=0.9,
                             stat=torch.zeros(3, dtype=torch.float64, device="cuda"))


@pytest.mark.parametrize("n", [5, 1025, 2 ** 20 + 3])
@pytest.mark.parametrize("opt", ["sgd", "adam"])
@pytest.mark.parametrize("max_norm", [0.01, 1e6])
def test_gradient_norm_clipping(ctx, n, opt, max_norm):
    """sumsq -> clip_coef -> update(grad_scale): the clip of clip_grad_norm_ (active for the
    small max_norm, inactive for the large one) folded into the update kernel."""
    from jabas_b200 import ops
    rng = np.random.default_rng(n)
    g, p = _rand(rng, n, 1e-2), _rand(rng, n)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    dg, w, dm, dv = _dev(g), [_dev(p), torch.empty(n, device="cuda")], _dev(m), _dev(v)
    st = torch.zeros(3, dtype=torch.float64, device="cuda")
    coef = torch.zeros(2, device="cuda")
    ops.sumsq(ctx, dg, st)
    ops.clip_coef(ctx, st, max_norm, coef)
    gc = g.copy()
    coef_o, norm_o = O.clip_grad_norm(gc, max_norm)
    assert np.allclose(_host(st), O.sumsq(g), rtol=1e-6)
    assert abs(float(coef[1]) - norm_o) <= 1e-6 * norm_o
    assert (coef_o < 1.0) == (max_norm < 1.0)
    if opt == "sgd":
        O.sgd_momentum(gc, p, m, lr=0.1, weight_decay=1e-4, momentum=0.9, first_step=True)
        ops.sgd_momentum(ctx, dg, w, dm, [dict(lr=0.1, weight_decay=1e-4)], momentum=0.9, first_step=True,
                         grad_scale=coef)
    else:
        O.adam(gc, p, m, v, lr=1e-3, weight_decay=0.0, beta1=0.9, beta2=0.999, eps=1e-8, step=1, decoupled=False)
        ops.adam(ctx, dg, w, dm, dv, [dict(lr=1e-3, step=1)], beta1=0.9, beta2=0.999, eps=1e-8,
                 decoupled=False, grad_scale=coef)
    if float(coef[0]) == np.float32(coef_o):
        assert np.array_equal(_host(w[0]), p) and np.array_equal(_host(w[1]), p)
        assert np.array_equal(_host(dm), m)
    else:                                               # the two fp64 sums rounded to neighbouring fp32 norms
        assert np.allclose(_host(w[0]), p, rtol=1e-6, atol=1e-9)
    assert np.array_equal(_host(dg), g)                 # the gradient buffer itself is not rewritten


def test_layout_group_must_be_provided(ctx):
    from jabas_b200 import ops, JabasError
    x = torch.zeros(64, device="cuda")
    lay = ops.Layout(ctx, [(0, 32, 0), (32, 64, 2)], 64)
    with pytest.raises(JabasError, match="param group"):
        ops.sgd_momentum(ctx, x, [x.clone()], x.clone(), [dict(lr=0.1), dict(lr=0.1)], momentum=0.9, layout=lay)
    lay.close()


def test_bulk_staging_wait_runs_out_and_is_reported():
    """Host-side fault injection: the stage barriers of the bulk-staged update kernel expect 16
    bytes more than are copied, so every CTA's first wait runs out after the (lowered) wall-time
    limit.  All copies that were issued complete, the kernel returns, the context counts the
    time-outs and stays usable; with the injection off the same launch is bit-exact again."""
    from jabas_b200 import ops
    c = ops.Context(0)
    c.set_staging("bulk")
    c.set_wait_limits(staging_ms=2.0)
    n, K = 2 ** 20 + 8, 2
    rng = np.random.default_rng(12)
    g, p = _rand(rng, n, 1e-3), _rand(rng, n)
    dg, dm = _dev(g), torch.zeros(n, device="cuda")
    dw = [_dev(p) for _ in range(K)]
    groups = [dict(lr=0.1, weight_decay=1e-4)]
    c.inject_staging_stall(True)
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    ops.sgd_momentum(c, dg, dw, dm, groups, momentum=0.9, first_step=True)
    z.record()
    torch.cuda.synchronize()
    assert c.staging_timeouts() > 0
    assert a.elapsed_time(z) < 1000.0                      # bounded by time: a few waits of 2 ms per CTA
    c.inject_staging_stall(False)
    c.set_wait_limits(staging_ms=50.0)
    before = c.staging_timeouts()
    for w in dw:
        w.copy_(torch.from_numpy(p))
    dm.zero_()
    ops.sgd_momentum(c, dg, dw, dm, groups, momentum=0.9, first_step=True)
    torch.cuda.synchronize()
    assert c.staging_timeouts() == before                  # no new time-out
    m_o = np.zeros(n, np.float32)
    O.sgd_momentum(g, p, m_o, lr=0.1, weight_decay=1e-4, momentum=0.9, first_step=True)
    for w in dw:
        assert np.array_equal(_host(w), p)
    assert np.array_equal(_host(dm), m_o)
    c.close()
