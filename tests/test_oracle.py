"""The CPU oracle against hand-made known answers and against stock torch ops.

The reference ships no golden vectors for this arithmetic, so the oracle is pinned as
far as it can be: bit-exact against the installed ``torch.optim.SGD`` on CPU, bit-exact
against a torch-op restatement of the PyTorch v1.8.1 ``adam``/``adamw`` functional form
(device-kernel operand order), and within 1e-5 relative of the installed
``torch.optim.Adam/AdamW`` (which moved to ``lerp_`` after v1.8.1).
"""
import math

import numpy as np
import pytest
import torch

from oracle import gradpath as O

SIZES = [1, 3, 4, 1023, 1025, 2 ** 16 + 1]


def _rand(rng, n, scale=1.0):
    return (rng.standard_normal(n) * scale).astype(np.float32)


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("K", [1, 2, 3, 4, 8])
def test_aggregate_matches_sequential_torch_adds(n, K):
    rng = np.random.default_rng(n * 31 + K)
    grads = [_rand(rng, n, 1e-3) for _ in range(K)]
    T = float(2 * K)
    out, half = np.empty(n, np.float32), np.empty(n, np.float32)
    O.vsw_aggregate(grads, out, T, half)
    buf = torch.from_numpy(grads[0].copy())
    for k in range(1, K):
        buf.add_(torch.from_numpy(grads[k]))
    assert np.array_equal(half, buf.numpy())
    buf.div_(T)
    assert np.array_equal(out, buf.numpy())


def test_aggregate_known_answers():
    g0 = np.array([1.0, -2.0, 3.5, 1e-8], np.float32)
    out = np.empty_like(g0)
    O.vsw_aggregate([g0], out, 1.0)                     # K = 1, T = 1: identity
    assert np.array_equal(out, g0)
    O.vsw_aggregate([g0, -g0], out, 2.0)                # g1 = -g0: exact zeros
    assert np.array_equal(out, np.zeros_like(g0))
    a = g0.copy()
    O.vsw_aggregate([a, g0, g0], a, 3.0)                # out aliases grads[0]
    assert np.array_equal(a, (g0 + g0 + g0) / np.float32(3.0))


def test_cosine_known_answers():
    rng = np.random.default_rng(5)
    e = _rand(rng, 4099)
    assert O.cosine_from_stat(O.dot_norms(e, e)) == pytest.approx(1.0, abs=1e-7)
    assert O.cosine_from_stat(O.dot_norms(e, -e)) == pytest.approx(-1.0, abs=1e-7)
    a = np.zeros(8, np.float32); b = np.zeros(8, np.float32)
    a[:4] = 1.0; b[4:] = 2.0                            # orthogonal halves
    assert O.cosine_from_stat(O.dot_norms(a, b)) == 0.0
    tiny = np.full(4, 1e-6, np.float32)                 # |E||O| < eps: clamped denominator
    st = O.dot_norms(tiny, tiny)
    assert O.cosine_from_stat(st) == pytest.approx(st[0] / 1e-8, rel=1e-6)
    assert O.cosine_from_stat(np.zeros(3)) == 0.0


@pytest.mark.parametrize("n", [7, 4096, 100003])
def test_cosine_matches_torch_cosine_similarity(n):
    rng = np.random.default_rng(n)
    a, b = _rand(rng, n, 1e-3), _rand(rng, n, 1e-3)
    b += 0.3 * a
    ref = torch.nn.functional.cosine_similarity(torch.from_numpy(a), torch.from_numpy(b), dim=0)
    assert abs(O.cosine_from_stat(O.dot_norms(a, b)) - float(ref)) < 1e-5


def test_half_stat_equals_pair_exchange_form():
    """o = 2g - e reproduces the other sub-group's mean to within fp32 rounding."""
    rng = np.random.default_rng(11)
    n, hd = 50001, 4.0
    sum_e, sum_o = _rand(rng, n, 1e-3), _rand(rng, n, 1e-3)
    e, o = sum_e / np.float32(hd), sum_o / np.float32(hd)
    g = ((sum_e + sum_o) / np.float32(2 * hd)).astype(np.float32)
    c_local = O.cosine_from_stat(O.half_stat(g, sum_e, hd))
    c_pair = O.cosine_from_stat(O.dot_norms(e, o))
    assert abs(c_local - c_pair) < 1e-5


@pytest.mark.parametrize("K", [2, 3, 4, 8])
def test_vsw_parity_stat(K):
    rng = np.random.default_rng(K)
    n = 10007
    grads = [_rand(rng, n, 1e-3) for _ in range(K)]
    hd = np.float32(K / 2)
    e = sum(grads[k] for k in range(2, K, 2)) + grads[0] if K > 2 else grads[0]
    e = grads[0].copy()
    for k in range(2, K, 2):
        e = e + grads[k]
    o = grads[1].copy()
    for k in range(3, K, 2):
        o = o + grads[k]
    st = O.vsw_parity_stat(grads, float(hd))
    ref = O.dot_norms((e / hd).astype(np.float32), (o / hd).astype(np.float32))
    assert np.allclose(st, ref, rtol=1e-14, atol=0)


@pytest.mark.parametrize("wd", [0.0, 1e-4])
@pytest.mark.parametrize("nesterov", [False, True])
def test_sgd_bit_exact_vs_installed_torch_optim(wd, nesterov):
    rng = np.random.default_rng(3)
    n = 100003
    p0 = _rand(rng, n)
    P = torch.nn.Parameter(torch.from_numpy(p0.copy()))
    opt = torch.optim.SGD([P], lr=0.1, momentum=0.9, weight_decay=wd, nesterov=nesterov,
                          foreach=False)
    p, m = p0.copy(), np.zeros_like(p0)
    for it in range(4):
        g = _rand(rng, n, 1e-3)
        P.grad = torch.from_numpy(g.copy())
        opt.step()
        O.sgd_momentum(g, p, m, lr=0.1, weight_decay=wd, momentum=0.9, nesterov=nesterov,
                       first_step=(it == 0))
        assert np.array_equal(P.detach().numpy(), p)
        assert np.array_equal(opt.state[P]["momentum_buffer"].numpy(), m)


def test_sgd_first_step_and_dampening_known_answer():
    g = np.array([1.0, 2.0], np.float32)
    p = np.array([10.0, 20.0], np.float32)
    m = np.array([99.0, 99.0], np.float32)              # ignored on the first step
    O.sgd_momentum(g, p, m, lr=0.5, momentum=0.5, dampening=0.5, first_step=True)
    assert np.array_equal(m, g) and np.array_equal(p, np.array([9.5, 19.0], np.float32))
    O.sgd_momentum(g, p, m, lr=0.5, momentum=0.5, dampening=0.5)
    assert np.array_equal(m, np.array([1.0, 2.0], np.float32))      # .5*m + .5*g
    assert np.array_equal(p, np.array([9.0, 18.0], np.float32))


def _adam_v181_device_form(param, grad, m, v, step, beta1, beta2, lr, wd, eps, decoupled):
    """torch/optim/_functional.py of v1.8.1 with addcdiv in its device-kernel operand
    order a + alpha*(b/c) (the CPU kernel of the installed torch evaluates (alpha*b)/c)."""
    if decoupled:
        param.mul_(1 - lr * wd)
    elif wd != 0:
        grad = grad.add(param, alpha=wd)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    m.mul_(beta1).add_(grad, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)
    # The installed torch's vectorised CPU sqrt is off by one ulp on ~0.7 % of inputs
    # (checked against a float64 square root); numpy's is correctly rounded, like the
    # device's sqrt.rn, so the square root alone is taken through numpy.
    root = torch.from_numpy(np.sqrt(v.numpy()))
    denom = (root / math.sqrt(bc2)).add_(eps)
    param.add_(m / denom, alpha=-(lr / bc1))


@pytest.mark.parametrize("decoupled", [True, False])
def test_adam_bit_exact_vs_v181_functional_form(decoupled):
    rng = np.random.default_rng(4)
    n = 100003
    p0 = _rand(rng, n)
    P, M, V = torch.from_numpy(p0.copy()), torch.zeros(n), torch.zeros(n)
    p, m, v = p0.copy(), np.zeros_like(p0), np.zeros_like(p0)
    hp = dict(lr=1e-3, weight_decay=0.05, beta1=0.9, beta2=0.999, eps=1e-8)
    for it in range(4):
        g = _rand(rng, n, 1e-3)
        _adam_v181_device_form(P, torch.from_numpy(g.copy()), M, V, it + 1, 0.9, 0.999, 1e-3,
                               0.05, 1e-8, decoupled)
        O.adam(g, p, m, v, step=it + 1, decoupled=decoupled, **hp)
        assert np.array_equal(M.numpy(), m)
        assert np.array_equal(V.numpy(), v)
        assert np.array_equal(P.numpy(), p)


@pytest.mark.parametrize("decoupled", [True, False])
def test_adam_close_to_installed_torch_optim(decoupled):
    rng = np.random.default_rng(6)
    n = 50001
    p0 = _rand(rng, n)
    P = torch.nn.Parameter(torch.from_numpy(p0.copy()))
    cls = torch.optim.AdamW if decoupled else torch.optim.Adam
    opt = cls([P], lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.05, foreach=False)
    p, m, v = p0.copy(), np.zeros_like(p0), np.zeros_like(p0)
    for it in range(5):
        g = _rand(rng, n, 1e-3)
        P.grad = torch.from_numpy(g.copy())
        opt.step()
        O.adam(g, p, m, v, lr=1e-3, weight_decay=0.05, beta1=0.9, beta2=0.999, eps=1e-8,
               step=it + 1, decoupled=decoupled)
    assert np.abs(P.detach().numpy() - p).max() < 1e-6
    assert np.allclose(opt.state[P]["exp_avg"].numpy(), m, rtol=1e-5, atol=1e-9)
    assert np.allclose(opt.state[P]["exp_avg_sq"].numpy(), v, rtol=1e-5, atol=1e-12)


def test_update_segments_two_groups():
    rng = np.random.default_rng(8)
    n = 1000
    g, p0 = _rand(rng, n, 1e-3), _rand(rng, n)
    segs = [(0, 130, 0), (130, 131, 1), (131, 777, 0), (777, 1000, 1)]
    groups = [dict(lr=0.1, weight_decay=0.0), dict(lr=0.05, weight_decay=1e-2)]
    p, m = p0.copy(), np.zeros_like(p0)
    O.update_segments("sgd", g, p, m, None, segs, groups, momentum=0.9, first_step=True)
    for b, e, gi in segs:
        pe, me = p0[b:e].copy(), np.zeros(e - b, np.float32)
        O.sgd_momentum(g[b:e].copy(), pe, me, momentum=0.9, first_step=True, **groups[gi])
        assert np.array_equal(pe, p[b:e])


def test_replicate_and_sumsq():
    src = np.arange(10, dtype=np.float32)
    d1, d2 = np.zeros(10, np.float32), np.zeros(10, np.float32)
    O.replicate(src, [d1, d2, src])
    assert np.array_equal(d1, src) and np.array_equal(d2, src)
    assert O.sumsq(src) == float((np.arange(10.0) ** 2).sum())
