"""CUDA-graph mode of the gradient path: one graph launch per iteration must give the
same bits as the eager launches, including hyper-parameters that change between replays
(they live in a device block refreshed before each replay)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(kind, K, per_bucket, staging="register"):
    from jabas_b200.gradient_path import GradientPath, OptimizerSpec
    from jabas_b200.layout import build_layout
    shapes = [(64, 3, 7, 7), (64,), (64,), (256, 64, 3, 3), (1000, 257), (1000,)]
    names = ["conv1.weight", "bn1.weight", "bn1.bias", "conv2.weight", "fc.weight", "fc.bias"]
    layout = build_layout(names, shapes, [1, 0, 0, 1, 1, 1], bucket_cap_mb=0.5, first_bucket_bytes=64 * 1024)
    if kind == "sgd":
        spec = OptimizerSpec("sgd", [dict(lr=0.1, weight_decay=0.0), dict(lr=0.1, weight_decay=1e-4)], momentum=0.9)
    else:
        spec = OptimizerSpec("adamw", [dict(lr=1e-3, weight_decay=0.0), dict(lr=1e-3, weight_decay=0.05)])
    eng = GradientPath(layout, K, torch.device("cuda", 0), spec, total_num_decoupled_workers=K,
                       staging=staging)
    g = torch.Generator(device="cuda").manual_seed(3)
    eng.weights[0].normal_(generator=g)
    for b, e in zip([0] + [x[1] for x in layout.buckets], [x[0] for x in layout.buckets] + [layout.total]):
        eng.weights[0][b:e] = 0
    for k in range(1, K):
        eng.weights[k].copy_(eng.weights[0])
    return eng, dict(per_bucket=per_bucket, fuse_local=None if not per_bucket else False)


def _fill_grads(eng, it):
    for k in range(eng.K):
        g = torch.Generator(device="cuda").manual_seed(100 * it + k)
        eng.grads[k].normal_(0.0, 1e-3, generator=g)


@pytest.mark.parametrize("kind", ["sgd", "adamw"])
@pytest.mark.parametrize("per_bucket", [False, True])
@pytest.mark.parametrize("staging", ["register", "bulk"])
def test_graph_replay_is_bit_identical_to_eager(kind, per_bucket, staging):
    eager, how = _engine(kind, 4, per_bucket)
    graphed, _ = _engine(kind, 4, per_bucket, staging)
    lrs = [0.1, 0.1, 0.05, 0.2, 0.01]
    cos_e = []
    for it, lr in enumerate(lrs):
        for gr in eager.opt.groups:
            gr["lr"] = lr
        _fill_grads(eager, it)
        cos_e.append(float(eager.run_iteration(**how)))
    # graph engine: the two warm-up iterations of capture() are iterations 0 and 1
    it_box = [0]
    orig_body = graphed._iteration_body

    def body(*a, **k):                       # feed the warm-up iterations with the same gradients
        if it_box[0] < 2:                    # not under capture: RNG kernels must stay out of the graph
            _fill_grads(graphed, it_box[0])
        it_box[0] += 1
        return orig_body(*a, **k)
    for gr in graphed.opt.groups:
        gr["lr"] = lrs[0]
    graphed._iteration_body = body
    graphed.capture(warmup=2, **how)         # also runs body once more under capture (no side effect on steps)
    graphed._iteration_body = orig_body
    assert graphed.steps == 2
    cos_g = []
    for it in range(2, len(lrs)):
        for gr in graphed.opt.groups:
            gr["lr"] = lrs[it]
        _fill_grads(graphed, it)
        cos_g.append(float(graphed.replay()))
    torch.cuda.synchronize()
    assert graphed.steps == eager.steps == len(lrs)
    for k in range(4):
        assert torch.equal(graphed.weights[k], eager.weights[0]), k
    assert torch.equal(graphed.m, eager.m)
    if staging == "register":
        assert cos_g == cos_e[2:]
    else:                                    # other tile-to-thread map: fp64 sums in another order
        assert np.allclose(cos_g, cos_e[2:], rtol=0, atol=1e-6)
        assert graphed.ctx.staging_timeouts() == 0
    assert graphed.launches_per_replay >= 2
    eager.close(); graphed.close()
