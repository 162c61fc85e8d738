"""Golden vectors produced by the reference's OWN comm hook and cosine code
(``tests/golden/make_golden.py``: two gloo ranks, K = 2 VSWs each, three ragged buckets).

The CPU test pins the oracle on them; the GPU test runs the CUDA kernels through the C ABI
on the same inputs.  With two ranks every collective is a single fp32 addition, which is
commutative, so everything except the cosine must match bit for bit."""
import os

import numpy as np
import pytest
import torch

from oracle import gradpath as O

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "similarity_hook_ws2.npz"))
K, WORLD, T = (int(x) for x in G["meta_K_world_T"])
NB = 3


def _grads(r, b):
    return [np.ascontiguousarray(G[f"grad_r{r}_k{k}_b{b}"]) for k in range(K)]


def test_fixture_shape():
    assert (K, WORLD, T) == (2, 2, 4)
    assert float(G["cos_r0"]) == float(G["cos_r1"])          # broadcast from the first rank
    for b in range(NB):
        assert np.array_equal(G[f"avg_r0_b{b}"], G[f"avg_r1_b{b}"])


def test_oracle_reproduces_reference_hook_chain():
    stat_pair, stat_fused = np.zeros(3), [np.zeros(3), np.zeros(3)]
    for b in range(NB):
        outs, halves = [], []
        for r in range(WORLD):
            g = _grads(r, b)
            out, half = np.empty_like(g[0]), np.empty_like(g[0])
            O.vsw_aggregate(g, out, float(T), half)
            outs.append(out); halves.append(half)
        avg = outs[0] + outs[1]                               # world SUM of the already divided buckets
        assert np.array_equal(avg, G[f"avg_r0_b{b}"])
        E = []
        for r in range(WORLD):                                # each parity sub-group has one rank
            e = halves[r].copy()
            O.div_(e, T / 2)
            assert np.array_equal(e, G[f"half_r{r}_b{b}"])
            E.append(e)
            O.half_stat(avg, halves[r], T / 2, stat_fused[r])
        O.dot_norms(E[0], E[1], stat_pair)
    cos_ref = float(G["cos_r0"])
    assert abs(O.cosine_from_stat(stat_pair) - cos_ref) < 1e-5
    for r in range(WORLD):                                    # o = 2g - e form, from either rank
        assert abs(O.cosine_from_stat(stat_fused[r]) - cos_ref) < 1e-5


@pytest.mark.gpu
def test_cuda_kernels_reproduce_reference_hook_chain():
    from jabas_b200 import ops
    ctx = ops.Context(0)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    stat_pair = torch.zeros(3, dtype=torch.float64, device="cuda")
    stat_fused = [torch.zeros(3, dtype=torch.float64, device="cuda") for _ in range(WORLD)]
    cos = torch.zeros(1, device="cuda")
    for b in range(NB):
        outs, halves = [], []
        for r in range(WORLD):
            g = [dev(x) for x in _grads(r, b)]
            half = torch.empty_like(g[0])
            ops.vsw_aggregate(ctx, g, g[0], float(T), half_out=half)
            outs.append(g[0]); halves.append(half)
        avg = outs[0] + outs[1]                               # stands for the 2-rank NCCL SUM
        assert np.array_equal(avg.cpu().numpy(), G[f"avg_r0_b{b}"])
        n = avg.numel()
        for r in range(WORLD):
            # fused form: the SGD update kernel accumulates the statistic while it streams g
            w, m = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
            ops.sgd_momentum(ctx, avg, [w], m, [dict(lr=0.1)], momentum=0.9, first_step=True,
                             half=halves[r], half_divisor=T / 2, stat=stat_fused[r])
        E = []
        for r in range(WORLD):                                # pair-exchange form: materialised E
            ops.div_(ctx, halves[r], T / 2)
            assert np.array_equal(halves[r].cpu().numpy(), G[f"half_r{r}_b{b}"])
            E.append(halves[r])
        ops.dot_norms(ctx, E[0], E[1], stat_pair)
    cos_ref = float(G["cos_r0"])
    for st in [stat_pair] + stat_fused:
        ops.cosine_finalize(ctx, st, cos)
        assert abs(float(cos) - cos_ref) < 1e-5
    ctx.close()
