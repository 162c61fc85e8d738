"""Parity of the CUDA path on the benchmark configurations that the small kernel tests do not
reach: the ViT-B/16 layout (152 tensors, K = 8, AdamW, two param groups), the GNMT-8 layout
(244 M elements, K = 2, Adam, buckets up to 125 MiB) and flat buffers of 2^27 and 2^29 elements
(and one just past 2^29, where byte offsets cross 2^31).  Model-shaped layouts are compared
whole against ``ReferencePath(arith="c")``; the large flat buffers by windows — the oracle is
element-wise, so windows at the head, the tail and around the power-of-two offsets prove the
index arithmetic — plus whole-buffer properties (replicas identical, statistic against an fp64
reduction by torch).
"""
import numpy as np
import pytest
import torch

from oracle import gradpath as O

pytestmark = pytest.mark.gpu


def _spec(opt):
    from jabas_b200.gradient_path import OptimizerSpec
    return OptimizerSpec(kind=opt["kind"], groups=opt["groups"], momentum=opt.get("momentum", 0.0),
                         betas=opt.get("betas", (0.9, 0.999)), eps=opt.get("eps", 1e-8))


@pytest.mark.parametrize("model,K,opt", [
    ("vit_b_16", 8, dict(kind="adamw", groups=[dict(lr=1e-3, weight_decay=0.0), dict(lr=1e-3, weight_decay=0.05)],
                         betas=(0.9, 0.999), eps=1e-8)),
    ("gnmt8", 2, dict(kind="adam", groups=[dict(lr=2e-3, weight_decay=0.0)], betas=(0.9, 0.999), eps=1e-8)),
])
@pytest.mark.parametrize("form", ["fused", "per_bucket"])
def test_model_layouts_match_reference_path(model, K, opt, form):
    from jabas_b200.gradient_path import GradientPath
    from jabas_b200.layout import build_layout, model_zoo_shapes
    from oracle.reference_path import ReferencePath
    names, shapes, groups = model_zoo_shapes(model)
    layout = build_layout(names, shapes, groups)
    if model == "vit_b_16":
        assert layout.num_params == 86567656 and len(names) == 152 and layout.num_buckets == 14
    else:
        assert layout.num_params == 243967233 and max(layout.bucket_sizes_mib()) > 120
    dev = torch.device("cuda", 0)
    eng = GradientPath(layout, K, dev, _spec(opt), total_num_decoupled_workers=K)
    ref = ReferencePath(layout, K, opt, total_num_decoupled_workers=K, arith="c")
    gen = torch.Generator(device=dev).manual_seed(11)
    pad = torch.ones(layout.total, dtype=torch.bool, device=dev)
    for b, e in layout.buckets:
        pad[b:e] = False
    eng.weights[0].normal_(generator=gen)
    eng.weights[0][pad] = 0.0                    # padding between buckets is zero and stays zero
    for k in range(K):
        if k:
            eng.weights[k].copy_(eng.weights[0])
        ref.weights[k].copy_(eng.weights[0].cpu())
    how = dict() if form == "fused" else dict(per_bucket=True, fuse_local=False)
    for it in range(2):
        for k in range(K):
            eng.grads[k].normal_(0.0, 1e-3, generator=gen)
            eng.grads[k][pad] = 0.0
            ref.grads[k].copy_(eng.grads[k].cpu())
        cos = float(eng.run_iteration(**how))
        torch.cuda.synchronize()
        cos_ref = ref.run_iteration()
        assert abs(cos - cos_ref) <= 1e-5, (it, cos, cos_ref)
        wr = ref.weights[0]
        for k in (0, K - 1):
            assert torch.equal(eng.weights[k].cpu(), wr), (it, k)           # bit-exact: the order is fixed
        assert torch.equal(eng.m.cpu(), ref.m)
        assert torch.equal(eng.v.cpu(), ref.v)
    for k in range(1, K):
        assert torch.equal(eng.weights[k], eng.weights[0])
    eng.close()


def _windows(n):
    w = 4096
    marks = [0, n - w, n // 2 - w // 2, (1 << 27) - w // 2, (1 << 28) - w // 2, (1 << 29) - w, (1 << 29) - w // 2,
             n // 3, 5 * (n // 7) + 1]
    out = []
    for lo in marks:
        lo = max(0, min(n - w, lo))
        out.append((lo, lo + w))
    return sorted(set(out))


@pytest.mark.parametrize("log2n,extra,kind", [(27, 0, "sgd"), (27, 0, "adamw"), (29, 0, "sgd"), (29, 0, "adamw"),
                                              (29, 4100, "sgd")])
def test_flat_buffers_by_windows(log2n, extra, kind):
    from jabas_b200.gradient_path import GradientPath
    from jabas_b200.layout import build_layout
    n = (1 << log2n) + extra
    K = T = 2
    layout = build_layout(["flat"], [(n,)], [0], bucket_cap_mb=1 << 30, first_bucket_bytes=1 << 62)
    if kind == "sgd":
        opt = dict(kind="sgd", groups=[dict(lr=0.1, weight_decay=1e-4)], momentum=0.9)
    else:
        opt = dict(kind="adamw", groups=[dict(lr=1e-3, weight_decay=0.05)], betas=(0.9, 0.999), eps=1e-8)
    dev = torch.device("cuda", 0)
    eng = GradientPath(layout, K, dev, _spec(opt), total_num_decoupled_workers=T)
    gen = torch.Generator(device=dev).manual_seed(log2n + extra)
    eng.weights[0].normal_(generator=gen)
    eng.weights[1].copy_(eng.weights[0])
    wins = _windows(n)
    hw = {w: eng.weights[0][w[0]:w[1]].cpu().numpy().copy() for w in wins}
    hm = {w: np.zeros(w[1] - w[0], np.float32) for w in wins}
    hv = {w: np.zeros(w[1] - w[0], np.float32) for w in wins}
    for it in range(2):
        for k in range(K):
            eng.grads[k].normal_(0.0, 1e-3, generator=gen)
        hg = {w: [eng.grads[k][w[0]:w[1]].cpu().numpy().copy() for k in range(K)] for w in wins}
        # the statistic over the WHOLE buffer in fp64 (K = 2: E = g_0 / (T/2), O = g_1 / (T/2), T = 2)
        e, o = eng.grads[0].double(), eng.grads[1].double()
        stat64 = [float((e * o).sum()), float((e * e).sum()), float((o * o).sum())]
        del e, o
        cos = float(eng.run_iteration())
        torch.cuda.synchronize()
        st = eng.stat.cpu().numpy()
        assert np.allclose(st[1:], stat64[1:], rtol=1e-6), (st, stat64)
        # the dot product can be small against the norms: bound its error on the cosine's scale
        assert abs(st[0] - stat64[0]) <= 1e-6 * np.sqrt(stat64[1] * stat64[2]), (st, stat64)
        assert abs(cos - stat64[0] / max(np.sqrt(stat64[1] * stat64[2]), 1e-8)) <= 1e-5
        assert torch.equal(eng.weights[1], eng.weights[0])
        for w in wins:
            g = np.empty(w[1] - w[0], np.float32)
            O.vsw_aggregate(hg[w], g, float(T))
            if kind == "sgd":
                O.sgd_momentum(g, hw[w], hm[w], lr=0.1, weight_decay=1e-4, momentum=0.9, first_step=(it == 0))
            else:
                O.adam(g, hw[w], hm[w], hv[w], lr=1e-3, weight_decay=0.05, beta1=0.9, beta2=0.999, eps=1e-8,
                       step=it + 1, decoupled=True)
            assert np.array_equal(eng.weights[0][w[0]:w[1]].cpu().numpy(), hw[w]), (it, w)
            assert np.array_equal(eng.weights[1][w[0]:w[1]].cpu().numpy(), hw[w]), (it, w)
            assert np.array_equal(eng.m[w[0]:w[1]].cpu().numpy(), hm[w]), (it, w)
            if kind != "sgd":
                assert np.array_equal(eng.v[w[0]:w[1]].cpu().numpy(), hv[w]), (it, w)
    eng.close()
    del eng
    torch.cuda.empty_cache()


@pytest.mark.parametrize("log2n", [27, 29])
def test_two_kernel_form_by_windows(log2n):
    """Aggregate kernel + update kernel (the form used between collectives) at the large sizes."""
    from jabas_b200 import ops
    n, K, T = 1 << log2n, 2, 4
    dev = torch.device("cuda", 0)
    ctx = ops.Context(0)
    gen = torch.Generator(device=dev).manual_seed(log2n)
    gs = [torch.empty(n, device=dev).normal_(0.0, 1e-3, generator=gen) for _ in range(K)]
    w = [torch.empty(n, device=dev).normal_(generator=gen)]
    w.append(w[0].clone())
    m, half, out = torch.zeros(n, device=dev), torch.empty(n, device=dev), torch.empty(n, device=dev)
    wins = _windows(n)
    hg = {x: [g[x[0]:x[1]].cpu().numpy().copy() for g in gs] for x in wins}
    hw = {x: w[0][x[0]:x[1]].cpu().numpy().copy() for x in wins}
    stat = torch.zeros(3, dtype=torch.float64, device=dev)
    ops.vsw_aggregate(ctx, gs, out, float(T), half_out=half)
    # what the world allreduce would add: the other rank's (already divided) contribution
    other = torch.empty(n, device=dev).normal_(0.0, 2.5e-4, generator=gen)
    hother = {x: other[x[0]:x[1]].cpu().numpy().copy() for x in wins}
    hout = {x: out[x[0]:x[1]].cpu().numpy().copy() for x in wins}
    out.add_(other)
    del other
    ops.sgd_momentum(ctx, out, w, m, [dict(lr=0.1, weight_decay=1e-4)], momentum=0.9, first_step=True,
                     half=half, half_divisor=T / 2, stat=stat)
    torch.cuda.synchronize()
    for x in wins:
        g, h = np.empty(x[1] - x[0], np.float32), np.empty(x[1] - x[0], np.float32)
        O.vsw_aggregate(hg[x], g, float(T), h)
        assert np.array_equal(hout[x], g)
        assert np.array_equal(half[x[0]:x[1]].cpu().numpy(), h)
        g = g + hother[x]
        mm = np.zeros_like(g)
        O.sgd_momentum(g, hw[x], mm, lr=0.1, weight_decay=1e-4, momentum=0.9, first_step=True)
        assert np.array_equal(w[1][x[0]:x[1]].cpu().numpy(), hw[x])
    e = half.double() / (T / 2)
    o = 2.0 * out.double() - e
    ref = [float((e * o).sum()), float((e * e).sum()), float((o * o).sum())]
    st = stat.cpu().numpy()
    assert np.allclose(st[1:], ref[1:], rtol=1e-5), (st, ref)
    assert abs(st[0] - ref[0]) <= 1e-6 * np.sqrt(ref[1] * ref[2]), (st, ref)
    ctx.close()
    del gs, w, m, half, out, e, o
    torch.cuda.empty_cache()
