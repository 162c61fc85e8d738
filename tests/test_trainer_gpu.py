"""The trainer / comm-hook / optimizer mirrors on a real GPU: K VSWs on K streams, hooks
fired from backward, fused kernels through the C ABI.  Expected values: the reference-path
restatement (C oracle arithmetic) fed with per-VSW gradients taken by plain autograd."""
import copy

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = dict(similarity_target=0.1, batch_size_adjust_interval=1, enable_adjust=False)


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(
        torch.nn.Conv2d(3, 16, 3, padding=1, bias=False), torch.nn.BatchNorm2d(16), torch.nn.ReLU(),
        torch.nn.Conv2d(16, 32, 3, padding=1, stride=2, bias=False), torch.nn.BatchNorm2d(32), torch.nn.ReLU(),
        torch.nn.AdaptiveAvgPool2d(4), torch.nn.Flatten(), torch.nn.Linear(512, 100), torch.nn.ReLU(),
        torch.nn.Linear(100, 10)).cuda()


def _groups(model):
    params = list(model.named_parameters())
    return [{"params": [p for n, p in params if p.dim() == 1], "weight_decay": 0.0},
            {"params": [p for n, p in params if p.dim() != 1], "weight_decay": 1e-3}]


def _opt_dict(kind):
    if kind == "sgd":
        return dict(kind="sgd", groups=[dict(lr=0.1, weight_decay=0.0), dict(lr=0.1, weight_decay=1e-3)],
                    momentum=0.9)
    return dict(kind="adamw", groups=[dict(lr=1e-2, weight_decay=0.0), dict(lr=1e-2, weight_decay=1e-3)],
                betas=(0.9, 0.999), eps=1e-8)


def _capture_vsw_gradients(tr):
    """Wrap every VSW's comm hook so that it first copies that VSW's raw gradient bucket:
    the exact inputs of the gradient path (two separate backward passes would differ by
    the rounding noise of non-deterministic convolution kernels)."""
    captured = {}
    for k, lm in enumerate(tr.local_models):
        def hook(state, bucket, k=k, orig=lm._hook):
            captured[(k, bucket.index())] = bucket.buffer(materialize=False).clone()
            return orig(state, bucket)
        lm.register_comm_hook(lm._hook_state, hook)
    return captured


@pytest.mark.parametrize("wsm,kind,K,threaded,staging", [
    ("sequential", "sgd", 2, False, "register"), ("overlap", "sgd", 2, False, "register"),
    ("sequential", "adamw", 2, False, "register"), ("overlap", "adamw", 2, False, "register"),
    ("sequential", "sgd", 4, False, "register"), ("overlap", "sgd", 4, False, "register"),
    ("sequential", "adamw", 4, False, "register"), ("overlap", "adamw", 4, False, "register"),
    ("overlap", "sgd", 4, True, "register"), ("sequential", "adamw", 4, True, "register"),
    ("sequential", "sgd", 4, False, "bulk"), ("overlap", "adamw", 2, False, "bulk")])
def test_trainer_on_gpu_matches_reference_path(wsm, kind, K, threaded, staging):
    import jabas_b200
    from jabas_b200.iidp.optim import ShardAdamW, ShardSGD
    from oracle.reference_path import ReferencePath
    tr = jabas_b200.JABASTrainer(0, 8, K, 0, wsm, dict(CFG))
    tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss().cuda(), bucket_cap_mb=0.05,
                               first_bucket_bytes=4096, staging=staging)
    assert tr.reducer.layout.num_buckets >= 3
    groups = _groups(tr.main_model)
    if kind == "sgd":
        opt = (ShardSGD if wsm == "overlap" else torch.optim.SGD)(groups, lr=0.1, momentum=0.9)
    else:
        opt = (ShardAdamW if wsm == "overlap" else torch.optim.AdamW)(groups, lr=1e-2)
    tr.prepare_weight_sync_method(opt, None, _groups)
    tr.set_model_train()
    tr.threaded_compute = threaded                      # K forward/backward passes from K threads
    ref = ReferencePath(tr.reducer.layout, K, _opt_dict(kind), total_num_decoupled_workers=K, arith="c")
    for k in range(K):
        ref.weights[k].copy_(tr.reducer.engine.weights[k].cpu())
    g = torch.Generator().manual_seed(1)
    launches0 = tr.reducer.engine.launches
    captured = _capture_vsw_gradients(tr)
    lay = tr.reducer.layout
    for it in range(3):
        x = torch.randn(8 * K, 3, 16, 16, generator=g).cuda()
        y = torch.randint(0, 10, (8 * K,), generator=g).cuda()
        tr.compute((x, y))
        assert tr.step() is True
        torch.cuda.synchronize()
        assert len(captured) == K * lay.num_buckets
        for (k, b), t in captured.items():
            ref.grads[k][lay.buckets[b][0]:lay.buckets[b][1]].copy_(t.cpu())
        captured.clear()
        cos_ref = ref.run_iteration()
        assert abs(float(tr.cos_placeholder) - cos_ref) < 1e-5
        wr = ref.weights[0]
        for k in range(K):
            assert torch.equal(tr.reducer.engine.weights[k].cpu(), wr), (it, k)   # bit-exact on one GPU
        for p0, pk in zip(tr.local_models[0].parameters(), tr.local_models[K - 1].parameters()):
            assert torch.equal(p0, pk)
    assert tr.reducer.engine.launches > launches0          # the CUDA library did the work
    if staging == "bulk":
        assert tr.reducer.engine.ctx.staging_timeouts() == 0


def test_runtime_change_of_vsw_count_on_gpu():
    """K: 2 -> 4 -> 2 between iterations on the device: surviving flat buffers keep their
    addresses, new replicas are filled by the replicate kernel, steps keep all replicas equal."""
    import jabas_b200
    from jabas_b200.iidp.optim import ShardSGD
    tr = jabas_b200.JABASTrainer(0, 8, 2, 0, "overlap", dict(CFG))
    tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss().cuda(), bucket_cap_mb=0.05,
                               first_bucket_bytes=4096)
    tr.prepare_weight_sync_method(ShardSGD(_groups(tr.main_model), lr=0.1, momentum=0.9), None, _groups)
    tr.set_model_train()
    eng = tr.reducer.engine
    g = torch.Generator().manual_seed(2)

    def one_step(K):
        before = eng.weights[0].clone()
        x = torch.randn(8 * K, 3, 16, 16, generator=g).cuda()
        y = torch.randint(0, 10, (8 * K,), generator=g).cuda()
        tr.compute((x, y))
        assert tr.step() is True
        torch.cuda.synchronize()
        assert not torch.equal(before, eng.weights[0])
        for k in range(1, K):
            assert torch.equal(eng.weights[k], eng.weights[0]), k
        assert -1.0 <= float(tr.cos_placeholder) <= 1.0

    one_step(2)
    ptrs = (eng.weights[0].data_ptr(), eng.grads[1].data_ptr(), eng.m.data_ptr())
    tr.change_num_models(4)
    torch.cuda.synchronize()
    assert eng.K == 4 and tr.total_num_decoupled_workers == 4
    assert (eng.weights[0].data_ptr(), eng.grads[1].data_ptr(), eng.m.data_ptr()) == ptrs
    assert torch.equal(eng.weights[3], eng.weights[0])
    one_step(4)
    tr.change_num_models(2)
    assert eng.K == 2 and eng.weights[0].data_ptr() == ptrs[0]
    one_step(2)


def test_resnet50_two_vsws_five_iterations():
    """The CPU-runnable configuration of the reference (ResNet-50, 2 VSWs, local batch 8,
    SGD momentum 0.9 lr 0.1 wd 1e-4, 25 MB buckets, 5 iterations, statistic every iteration)
    on one GPU through the trainer mirror; bit-exact against the reference-path restatement
    fed with the gradients captured from the run."""
    import torchvision
    import jabas_b200
    from jabas_b200.iidp.optim import ShardSGD
    from oracle.reference_path import ReferencePath
    torch.manual_seed(0)
    model = torchvision.models.resnet50().cuda()
    K = 2
    tr = jabas_b200.JABASTrainer(0, 8, K, 0, "overlap", dict(CFG))
    tr.prepare_stream_parallel(model, torch.nn.CrossEntropyLoss().cuda())
    lay = tr.reducer.layout
    assert lay.num_params == 25557032 and lay.bucket_sizes_mib() == [7.82, 30.04, 25.04, 25.32, 9.27]

    def groups(m):
        named = list(m.named_parameters())
        return [{"params": [p for n, p in named if "bn" in n], "weight_decay": 0},
                {"params": [p for n, p in named if "bn" not in n], "weight_decay": 1e-4}]
    tr.prepare_weight_sync_method(ShardSGD(groups(tr.main_model), 0.1, momentum=0.9, weight_decay=1e-4),
                                  None, groups)
    assert len(lay.segments) == 99
    tr.set_model_train()
    opt = dict(kind="sgd", groups=[dict(lr=0.1, weight_decay=0.0), dict(lr=0.1, weight_decay=1e-4)], momentum=0.9)
    ref = ReferencePath(lay, K, opt, total_num_decoupled_workers=K, arith="c")
    for k in range(K):
        ref.weights[k].copy_(tr.reducer.engine.weights[k].cpu())
    captured = _capture_vsw_gradients(tr)
    for it in range(5):
        g = torch.Generator().manual_seed(10 * it)
        x = torch.randn(8 * K, 3, 224, 224, generator=g).cuda()
        y = torch.randint(0, 1000, (8 * K,), generator=g).cuda()
        tr.compute((x, y))
        assert tr.step() is True
        torch.cuda.synchronize()
        for (k, b), t in captured.items():
            ref.grads[k][lay.buckets[b][0]:lay.buckets[b][1]].copy_(t.cpu())
        captured.clear()
        cos_ref = ref.run_iteration()
        assert abs(float(tr.cos_placeholder) - cos_ref) < 1e-5, it
        for k in range(K):
            assert torch.equal(tr.reducer.engine.weights[k].cpu(), ref.weights[0]), (it, k)
        assert torch.isfinite(tr.losses[0]).item()
