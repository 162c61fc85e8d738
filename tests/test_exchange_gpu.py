"""The pipelined cross-GPU exchange (``jabas_exchange_*``) on ONE GPU: all ranks' buffers live
on the device and all ranks run as one launch (``nlocal == nranks``), because kernels that wait
on one another may not run as separate launches on a GPU.  Expected values: the C oracle applied
in the exchange's fixed order — VSWs ascending, then ranks ascending with each rank's sum divided
by T first (the reference's ``div_(T)`` before the SUM allreduce,
jabas/ddp_comm_hooks/similarity_allreduce.py:42), E / O = even / odd ranks over T/2
(jabas/train/trainer.py:427-445).  Weights, state and averaged gradient are bit-exact; the
cosine is within 1e-5.
"""
import numpy as np
import pytest
import torch

from oracle import gradpath as O

pytestmark = pytest.mark.gpu

PIECE = 8192          # a small work item keeps the multi-chunk cases small


def _setup(ops, ctx, n_ranks, K, total, window, max_slots=None, seed=0, kw=2, lag=0):
    rng = np.random.default_rng(seed)
    max_slots = max_slots or max(1, -(-total // PIECE)) + 4
    words = ops.exchange_flag_words(max_slots)
    dev = ctx.device
    f32 = dict(dtype=torch.float32, device=dev)
    px = [torch.zeros(total, **f32) for _ in range(n_ranks)]
    pg = [torch.zeros(total, **f32) for _ in range(n_ranks)]
    fl = [torch.zeros(words, dtype=torch.int32, device=dev) for _ in range(n_ranks)]
    exs = [ops.Exchange(ctx, n_ranks, r, [t.data_ptr() for t in px], [t.data_ptr() for t in pg],
                        [t.data_ptr() for t in fl], max_slots, window, PIECE, lag) for r in range(n_ranks)]
    w0 = rng.standard_normal(total).astype(np.float32)
    ranks = []
    for r in range(n_ranks):
        ranks.append(dict(
            grads=[torch.zeros(total, **f32) for _ in range(K)],
            weights=[torch.from_numpy(w0).to(dev) for _ in range(kw)],
            m=torch.zeros(total, **f32), v=torch.zeros(total, **f32),
            stat=torch.zeros(3, dtype=torch.float64, device=dev), cos=torch.zeros(1, **f32)))
    return exs, ranks, (px, pg, fl), w0, rng


def _fill_grads(ranks, rng, total):
    host = []
    for r, rk in enumerate(ranks):
        gs = [(rng.standard_normal(total) * 1e-3).astype(np.float32) for _ in rk["grads"]]
        for t, g in zip(rk["grads"], gs):
            t.copy_(torch.from_numpy(g))
        host.append(gs)
    return host


def _expected(host, T, kind, hp_common, groups, segments, w, m, v):
    """One step of the fixed-order contract on the host; mutates w, m, v; returns (g, stat)."""
    n_ranks, total = len(host), w.size
    sums = []
    for gs in host:
        s = np.empty(total, np.float32)
        O.vsw_aggregate(gs, s, 1.0)
        sums.append(s)
    g = sums[0] / np.float32(T)
    for r in range(1, n_ranks):
        g = g + sums[r] / np.float32(T)
    e, o = sums[0].copy(), sums[1].copy()
    for r in range(2, n_ranks):
        if r & 1:
            o = o + sums[r]
        else:
            e = e + sums[r]
    half = np.float32(T / 2)
    stat = O.dot_norms(e / half, o / half)
    O.update_segments(kind, g, w, m, v, segments, groups, **hp_common)
    return g, stat


def _close_stat(got, want):
    """Norms to 1e-6 relative; the dot product, which may be small against them, to 1e-6 of
    their geometric mean (its weight in the cosine)."""
    assert np.allclose(got[1:], want[1:], rtol=1e-6), (got, want)
    assert abs(got[0] - want[0]) <= 1e-6 * np.sqrt(want[1] * want[2]), (got, want)


def _run(ops, exs, ranks, total, base, slot_base, T, kind, groups, layout, step, with_stat=True):
    bufs = [dict(grads=r["grads"], weights=r["weights"], m=r["m"], v=r["v"],
                 stat=r["stat"] if with_stat else None) for r in ranks]
    if kind == "sgd":
        ops.exchange_step(exs, bufs, total, base, slot_base, float(T), T / 2, groups, kind="sgd", layout=layout,
                          momentum=0.9, first_step=(step == 0))
    else:
        gs = [dict(g, step=step + 1) for g in groups]
        ops.exchange_step(exs, bufs, total, base, slot_base, float(T), T / 2, gs, kind=kind, layout=layout,
                          beta1=0.9, beta2=0.999, eps=1e-8)


@pytest.fixture(scope="module")
def ctx():
    from jabas_b200 import ops
    c = ops.Context(0)
    c.set_wait_limits(peer_ms=2000.0)
    yield c
    c.close()


@pytest.mark.parametrize("lag", [1, 2])             # steps between a piece's reduce and update items
@pytest.mark.parametrize("n_ranks,K,kind,total,window", [
    (2, 4, "sgd", 3 * 2 * 8192 + 4096 + 8, 2),      # 4 steps of one group, ragged last piece
    (2, 1, "adamw", 40, 4),                         # less than one piece
    (4, 2, "sgd", 5 * 4 * 2 * 8192 + 12, 8),        # 5 full windows of two groups + 12 elements
    (4, 3, "adamw", 2 * 4 * 8192 + 8192 * 3, 4),    # generic K, last window holds three pieces only
    (8, 4, "sgd", 4 * 8 * 8192 + 5 * 8192 + 100, 8),
    (8, 8, "adamw", 2 * 8 * 2 * 8192 + 4, 16),
    (8, 2, "adam", 8 * 8192, 0),                    # window sized from the grid: one step
    (6, 2, "sgd", 3 * 6 * 8192 + 64, 6),            # generic rank count
    (2, 7, "sgd", 2 * 8192 + 256, 2),               # odd K
    (4, 4, "sgd", 150 * 8192 + 1024, 0),            # many pieces, automatic window
])
def test_exchange_single_gpu_all_ranks_bit_exact(ctx, n_ranks, K, kind, total, window, lag):
    from jabas_b200 import ops
    exs, ranks, keep, w0, rng = _setup(ops, ctx, n_ranks, K, total, window, seed=n_ranks * 100 + K, lag=lag)
    T = n_ranks * K
    # two param groups in alternating runs of odd length: tiles straddle segment boundaries
    segments, pos, gi = [], 0, 0
    while pos < total:
        end = min(total, pos + 7001 + 13 * len(segments))
        segments.append((pos, end, gi))
        pos, gi = end, 1 - gi
    layout = ops.Layout(ctx, segments, total) if len(segments) > 1 else None
    if kind == "sgd":
        groups = [dict(lr=0.1, weight_decay=0.0), dict(lr=0.05, weight_decay=1e-4)]
        common = dict(momentum=0.9)
    else:
        groups = [dict(lr=1e-3, weight_decay=0.0), dict(lr=2e-3, weight_decay=0.05)]
        common = dict(beta1=0.9, beta2=0.999, eps=1e-8, decoupled=(kind == "adamw"))
    w, m, v = w0.copy(), np.zeros(total, np.float32), np.zeros(total, np.float32)
    for step in range(3):
        host = _fill_grads(ranks, rng, total)
        for r in ranks:
            r["stat"].zero_()
        _run(ops, exs, ranks, total, 0, 0, T, kind, groups, layout, step)
        ops.exchange_cosine(exs, [r["stat"] for r in ranks], [r["cos"] for r in ranks])
        torch.cuda.synchronize()
        for ex in exs:
            status, launches = ex.status()
            assert status == 0 and launches == step + 1
        if kind == "sgd":
            hp = dict(common, first_step=(step == 0))
            g_exp, stat = _expected(host, T, "sgd", hp, groups, segments, w, m, v)
        else:
            gs = [dict(g, step=step + 1) for g in groups]
            g_exp, stat = _expected(host, T, "adam", common, gs, segments, w, m, v)
        cos_exp = O.cosine_from_stat(stat)
        px, pg, _ = keep
        for r, rk in enumerate(ranks):
            for k, wt in enumerate(rk["weights"]):
                assert np.array_equal(wt.cpu().numpy(), w), (step, r, k)
            assert np.array_equal(rk["m"].cpu().numpy(), m), (step, r)
            if kind != "sgd":
                assert np.array_equal(rk["v"].cpu().numpy(), v), (step, r)
            # the pieces of the averaged gradient that this rank reduces (dealt in turn)
            got = pg[r].cpu().numpy()
            for P in range(r, -(-total // PIECE), n_ranks):
                lo, hi = P * PIECE, min(total, (P + 1) * PIECE)
                assert np.array_equal(got[lo:hi], g_exp[lo:hi]), (step, r, P)
            st = rk["stat"].cpu().numpy()
            _close_stat(st, stat)
            assert abs(float(rk["cos"]) - cos_exp) <= 1e-5
        # every rank holds the same bits of the statistic and the cosine
        assert len({r["stat"].cpu().numpy().tobytes() for r in ranks}) == 1
        assert len({float(r["cos"]) for r in ranks}) == 1
    for ex in exs:
        ex.close()


def test_exchange_per_bucket_launches_share_one_statistic(ctx):
    """Launches over disjoint ranges with disjoint slots, as the comm hooks issue them per DDP
    bucket, followed by one statistic exchange: same result as one launch over everything."""
    from jabas_b200 import ops
    n_ranks, K = 4, 2
    chunk = n_ranks * PIECE
    spans = [(0, chunk + 4096), (chunk + 4096, 3 * chunk + 32), (4 * chunk + 4128, 512)]
    total = spans[-1][0] + spans[-1][1]
    exs, ranks, keep, w0, rng = _setup(ops, ctx, n_ranks, K, total, 4, max_slots=32, seed=9)
    T = n_ranks * K
    groups = [dict(lr=0.1, weight_decay=1e-4)]
    w, m, v = w0.copy(), np.zeros(total, np.float32), np.zeros(total, np.float32)
    for step in range(2):
        host = _fill_grads(ranks, rng, total)
        for r in ranks:
            r["stat"].zero_()
        slot = 0
        for base, length in spans:
            _run(ops, exs, ranks, length, base, slot, T, "sgd", groups, None, step)
            slot += -(-length // PIECE)
        ops.exchange_cosine(exs, [r["stat"] for r in ranks], [r["cos"] for r in ranks])
        torch.cuda.synchronize()
        assert all(ex.status()[0] == 0 for ex in exs)
        g_exp, stat = _expected(host, T, "sgd", dict(momentum=0.9, first_step=(step == 0)), groups,
                                [(0, total, 0)], w, m, v)
        for r, rk in enumerate(ranks):
            assert np.array_equal(rk["weights"][1].cpu().numpy(), w), (step, r)
            _close_stat(rk["stat"].cpu().numpy(), stat)
            assert abs(float(rk["cos"]) - O.cosine_from_stat(stat)) <= 1e-5
    for ex in exs:
        ex.close()


def test_exchange_wait_runs_out_when_a_rank_never_signals():
    """Host-side fault injection: only rank 0 of two is ever launched, so its reduce pieces wait
    for flags that nothing sets.  With a 5 ms limit the kernel gives up, records where, returns,
    and the context stays usable; after a reset the same exchange works again."""
    from jabas_b200 import ops
    c = ops.Context(0)
    c.set_wait_limits(peer_ms=5.0)
    n_ranks, K, total = 2, 2, 3 * 2 * 8192
    exs, ranks, keep, w0, rng = _setup(ops, c, n_ranks, K, total, 2, seed=3)
    _fill_grads(ranks, rng, total)
    groups = [dict(lr=0.1, weight_decay=0.0)]
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    _run(ops, exs[:1], ranks[:1], total, 0, 0, 4, "sgd", groups, None, 0)        # rank 1 never runs
    t1.record()
    torch.cuda.synchronize()
    status, launches = exs[0].status()
    # gave up: in a reduce piece (rank 1's sums never arrive) or in an update piece whose wait for
    # the reduced shard ran out at the same moment — whichever CTA recorded first
    assert status >> 31 == 1 and (status >> 24) & 0xf in (2, 3)
    assert launches == 1
    assert t0.elapsed_time(t1) < 2000.0                               # bounded by time, not a hang
    # nothing was updated past the point of giving up, and the device still answers
    x = torch.arange(8, device="cuda").sum().item()
    assert x == 28
    # recovery: clear local counters and flags, then both ranks run and agree with the oracle
    for ex in exs:
        ex.reset()
    for t in keep[2]:
        t.zero_()
    c.set_wait_limits(peer_ms=2000.0)
    for r in ranks:
        r["weights"][0].copy_(torch.from_numpy(w0)); r["weights"][1].copy_(torch.from_numpy(w0))
        r["m"].zero_()
    host = _fill_grads(ranks, rng, total)
    _run(ops, exs, ranks, total, 0, 0, 4, "sgd", groups, None, 0)
    torch.cuda.synchronize()
    assert all(ex.status()[0] == 0 for ex in exs)
    w, m, v = w0.copy(), np.zeros(total, np.float32), np.zeros(total, np.float32)
    _expected(host, 4, "sgd", dict(momentum=0.9, first_step=True), groups, [(0, total, 0)], w, m, v)
    for rk in ranks:
        assert np.array_equal(rk["weights"][0].cpu().numpy(), w)
    for ex in exs:
        ex.close()
    c.close()


def test_exchange_rejects_bad_arguments(ctx):
    from jabas_b200 import ops
    exs, ranks, keep, w0, rng = _setup(ops, ctx, 2, 2, 4096, 2, max_slots=1)
    groups = [dict(lr=0.1, weight_decay=0.0)]
    with pytest.raises(ops.JabasError):                      # n not a multiple of 4
        _run(ops, exs, ranks, 4094, 0, 0, 4, "sgd", groups, None, 0)
    with pytest.raises(ops.JabasError):                      # more slots than the exchange owns
        _run(ops, exs, ranks, 4096, 0, 1, 4, "sgd", groups, None, 0)
    with pytest.raises(ops.JabasError):                      # more VSW gradients than a ring stage has slots
        many = [dict(grads=[r["grads"][0]] * 9, weights=r["weights"], m=r["m"], v=r["v"], stat=None) for r in ranks]
        ops.exchange_step(exs, many, 4096, 0, 0, 18.0, 9.0, groups, kind="sgd", momentum=0.9)
    with pytest.raises(ops.JabasError):                      # neither one rank nor all of them
        bad = ops.Exchange(ctx, 4, 0, [t.data_ptr() for t in keep[0]] * 2, [t.data_ptr() for t in keep[1]] * 2,
                           [t.data_ptr() for t in keep[2]] * 2, 1, 0, PIECE)
        _run(ops, [bad, bad], ranks, 4096, 0, 0, 4, "sgd", groups, None, 0)
    for ex in exs:
        ex.close()
