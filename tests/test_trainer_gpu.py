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


def _feed(ref, captured, lay):
    for (k, b), t in captured.items():
        ref.grads[k][lay.buckets[b][0]:lay.buckets[b][1]].copy_(t.cpu())
    captured.clear()


def _ref_with_vsws(ref, new_k, T):
    """The oracle after a change of the VSW count: a fresh ``ReferencePath`` with ``new_k``
    replicas that carries over the main weights, the optimizer state and the step count."""
    from oracle.reference_path import ReferencePath
    out = ReferencePath(ref.layout, new_k, ref.opt, total_num_decoupled_workers=T, arith="c")
    for k in range(new_k):
        out.weights[k].copy_(ref.weights[0])
    out.m.copy_(ref.m); out.v.copy_(ref.v)
    out.steps = ref.steps
    return out


@pytest.mark.parametrize("wsm", ["overlap", "sequential"])
def test_runtime_change_of_vsw_count_on_gpu(wsm):
    """K: 2 -> 4 -> 2 between iterations on the device (jabas/train/trainer.py:485-575):
    surviving flat buffers keep their addresses, new replicas are filled by the replicate
    kernel, and after every change the weights of all replicas and the cosine follow the
    oracle fed with the gradients captured from the run (T and T/2 change with K)."""
    import jabas_b200
    from jabas_b200.iidp.optim import ShardSGD
    from oracle.reference_path import ReferencePath
    tr = jabas_b200.JABASTrainer(0, 8, 2, 0, wsm, dict(CFG))
    tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss().cuda(), bucket_cap_mb=0.05,
                               first_bucket_bytes=4096)
    opt = (ShardSGD if wsm == "overlap" else torch.optim.SGD)(_groups(tr.main_model), lr=0.1, momentum=0.9)
    tr.prepare_weight_sync_method(opt, None, _groups)
    tr.set_model_train()
    eng, lay = tr.reducer.engine, tr.reducer.layout
    ref = ReferencePath(lay, 2, _opt_dict("sgd"), total_num_decoupled_workers=2, arith="c")
    for k in range(2):
        ref.weights[k].copy_(eng.weights[k].cpu())
    g = torch.Generator().manual_seed(2)
    state = {"ref": ref, "captured": _capture_vsw_gradients(tr)}

    def one_step(K):
        x = torch.randn(8 * K, 3, 16, 16, generator=g).cuda()
        y = torch.randint(0, 10, (8 * K,), generator=g).cuda()
        tr.compute((x, y))
        assert tr.step() is True
        torch.cuda.synchronize()
        assert len(state["captured"]) == K * lay.num_buckets
        _feed(state["ref"], state["captured"], lay)
        cos_ref = state["ref"].run_iteration()
        assert abs(float(tr.cos_placeholder) - cos_ref) < 1e-5
        for k in range(K):
            assert torch.equal(eng.weights[k].cpu(), state["ref"].weights[0]), k
        assert torch.equal(eng.m.cpu(), state["ref"].m)

    one_step(2)
    ptrs = (eng.weights[0].data_ptr(), eng.grads[1].data_ptr(), eng.m.data_ptr())
    tr.change_num_models(4)
    torch.cuda.synchronize()
    assert eng.K == 4 and tr.total_num_decoupled_workers == 4
    assert (eng.weights[0].data_ptr(), eng.grads[1].data_ptr(), eng.m.data_ptr()) == ptrs
    assert torch.equal(eng.weights[3], eng.weights[0])
    state["ref"] = _ref_with_vsws(state["ref"], 4, 4)
    state["captured"] = _capture_vsw_gradients(tr)          # the new VSWs' hooks are wrapped too
    one_step(4)
    one_step(4)
    tr.change_num_models(2)
    assert eng.K == 2 and eng.weights[0].data_ptr() == ptrs[0]
    state["ref"] = _ref_with_vsws(state["ref"], 2, 2)
    state["captured"] = _capture_vsw_gradients(tr)
    one_step(2)


def test_module_buffers_follow_the_main_replica():
    """BatchNorm running statistics and step counters of all K VSWs are views of one flat buffer
    per VSW and are overwritten with VSW 0's at the start of every iteration (the
    ``broadcast_buffers`` step of DistributedDataParallel that the reference keeps through
    ``sync_buffer_barrier``, jabas/train/trainer.py:515-528), by ONE replicate kernel."""
    import jabas_b200
    from jabas_b200.iidp.optim import ShardSGD
    K = 4
    tr = jabas_b200.JABASTrainer(0, 8, K, 0, "overlap", dict(CFG))
    tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss().cuda(), bucket_cap_mb=0.05,
                               first_bucket_bytes=4096)
    tr.prepare_weight_sync_method(ShardSGD(_groups(tr.main_model), lr=0.1, momentum=0.9), None, _groups)
    tr.set_model_train()
    red = tr.reducer
    assert red.num_module_buffers == 6 and len(red.buffers_flat) == K      # 2 BatchNorm layers x 3 buffers
    assert [f.dtype for f in red.buffers_flat[0]] == [torch.float32, torch.int64]
    for k in range(K):                        # the modules' buffers ARE the flat storage (one per dtype)
        spans = [(f.data_ptr(), f.data_ptr() + f.numel() * f.element_size()) for f in red.buffers_flat[k]]
        for b in tr.local_models[k].module.buffers():
            assert any(lo <= b.data_ptr() < hi for lo, hi in spans)
    torch.save(tr.main_model.module.state_dict(), "/dev/null")          # still saveable as it is
    g = torch.Generator().manual_seed(3)
    x = torch.randn(8 * K, 3, 16, 16, generator=g).cuda()
    y = torch.randint(0, 10, (8 * K,), generator=g).cuda()
    tr.compute((x, y)); tr.step()
    torch.cuda.synchronize()
    bufs = [[b.clone().cpu() for b in lm.module.buffers()] for lm in tr.local_models]
    assert any(not torch.equal(a, b) for a, b in zip(bufs[0], bufs[1]))     # different data, different statistics
    launches = red.engine.launches
    red.sync_buffers()
    torch.cuda.synchronize()
    assert red.engine.launches == launches + 2          # one bit-copy kernel per dtype
    for lm in tr.local_models:                # CPU restatement: every buffer <- VSW 0's
        for b, want in zip(lm.module.buffers(), bufs[0]):
            assert b.dtype == want.dtype and torch.equal(b.cpu(), want)
    # the next iteration starts from the synchronised statistics and training goes on
    tr.compute((x, y)); tr.step()
    torch.cuda.synchronize()
    nbt = [int(lm.module[1].num_batches_tracked) for lm in tr.local_models]
    assert nbt == [2] * K


@pytest.mark.parametrize("wsm,kind", [("sequential", "sgd"), ("overlap", "adamw")])
def test_gradient_accumulation_on_gpu(wsm, kind):
    """accum_step = 1 (jabas/train/trainer.py:572-575, 604-612): the first micro-step only
    accumulates into the flat gradient views (no hook fires, no kernel of the path runs), the
    second one synchronises; T = K * (accum_step + 1).  Oracle: fed with the accumulated buckets."""
    import jabas_b200
    from jabas_b200.iidp.optim import ShardAdamW, ShardSGD
    from oracle.reference_path import ReferencePath
    K, accum = 2, 1
    tr = jabas_b200.JABASTrainer(0, 8, K, accum, wsm, dict(CFG))
    tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss().cuda(), bucket_cap_mb=0.05,
                               first_bucket_bytes=4096)
    groups = _groups(tr.main_model)
    if kind == "sgd":
        opt = (ShardSGD if wsm == "overlap" else torch.optim.SGD)(groups, lr=0.1, momentum=0.9)
    else:
        opt = (ShardAdamW if wsm == "overlap" else torch.optim.AdamW)(groups, lr=1e-2)
    tr.prepare_weight_sync_method(opt, None, _groups)
    tr.set_model_train()
    T = tr.total_num_decoupled_workers
    assert T == K * (accum + 1) and tr.is_accum_mode
    eng, lay = tr.reducer.engine, tr.reducer.layout
    ref = ReferencePath(lay, K, _opt_dict(kind), total_num_decoupled_workers=T, arith="c")
    for k in range(K):
        ref.weights[k].copy_(eng.weights[k].cpu())
    captured = _capture_vsw_gradients(tr)
    g = torch.Generator().manual_seed(4)
    for it in range(3):
        launches = eng.launches
        for micro in range(accum + 1):
            x = torch.randn(8 * K, 3, 16, 16, generator=g).cuda()
            y = torch.randint(0, 10, (8 * K,), generator=g).cuda()
            tr.compute((x, y))
            done = tr.step()
            assert done is (micro == accum)
            if micro < accum:
                torch.cuda.synchronize()
                # no hook fired; the only launch is the module-buffer synchronisation that opens an iteration
                assert not captured and eng.launches == launches + len(tr.reducer.buffers_flat[0])
        torch.cuda.synchronize()
        assert len(captured) == K * lay.num_buckets
        _feed(ref, captured, lay)
        cos_ref = ref.run_iteration()
        assert abs(float(tr.cos_placeholder) - cos_ref) < 1e-5
        for k in range(K):
            assert torch.equal(eng.weights[k].cpu(), ref.weights[0]), (it, k)
        # the flat gradients were zeroed for the next accumulation
        assert float(eng.grads[1].abs().max()) == 0.0


@pytest.mark.parametrize("kind", ["sgd", "adamw"])
def test_checkpoint_round_trip_on_gpu(kind, tmp_path):
    """save() after two iterations, load() into a FRESH trainer on the GPU, run iteration 3 in
    both: bit-equal weights, optimizer state, Adam step, similarity step and LR modifier
    (jabas/train/trainer.py:105-169, 748-799).  Also: a checkpoint whose optimizer entry is a
    stock ``torch.optim`` state dict (the reference's format) loads into the flat buffers."""
    import jabas_b200
    from jabas_b200.iidp.optim import ShardAdamW, ShardSGD
    # two trainers must compute the same bits from the same batch: deterministic convolutions
    monkey_prev = torch.backends.cudnn.deterministic
    torch.backends.cudnn.deterministic = True

    def make(K=2):
        tr = jabas_b200.JABASTrainer(0, 8, K, 0, "overlap", dict(CFG, enable_adjust=True))
        tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss().cuda(), bucket_cap_mb=0.05,
                                   first_bucket_bytes=4096)
        groups = _groups(tr.main_model)
        opt = ShardSGD(groups, lr=0.1, momentum=0.9) if kind == "sgd" else ShardAdamW(groups, lr=1e-2)
        tr.prepare_weight_sync_method(opt, None, _groups)
        tr.set_model_train()
        return tr

    def batch(seed, K=2):
        g = torch.Generator().manual_seed(seed)
        return (torch.randn(8 * K, 3, 16, 16, generator=g).cuda(), torch.randint(0, 10, (8 * K,), generator=g).cuda())

    a = make()
    a.config_params["global_lr_modifier"] = 1.25
    for it in range(2):
        a.compute(batch(it)); a.step()
    torch.cuda.synchronize()
    path = a.save(str(tmp_path / "ckpt"))
    b = make()
    b.load(path)
    assert b.similarity_state.step == a.similarity_state.step == 3
    assert b.config_params["global_lr_modifier"] == 1.25
    assert b.sync_step == a.sync_step == 2
    ea, eb = a.reducer.engine, b.reducer.engine
    assert eb.steps == ea.steps == 2
    assert torch.equal(eb.weights[0], ea.weights[0]) and torch.equal(eb.weights[1], ea.weights[0])
    assert torch.equal(eb.m, ea.m)
    if kind != "sgd":
        assert torch.equal(eb.v, ea.v)
    # BatchNorm running statistics travel with the model state dict
    for (na, ba), (nb_, bb) in zip(a.main_model.module.named_buffers(), b.main_model.module.named_buffers()):
        assert na == nb_ and torch.equal(ba, bb)
    for tr in (a, b):
        tr.compute(batch(7)); tr.step()
    torch.cuda.synchronize()
    assert torch.equal(eb.weights[0], ea.weights[0]) and torch.equal(eb.weights[1], ea.weights[1])
    assert torch.equal(eb.m, ea.m)
    if kind != "sgd":
        assert torch.equal(eb.v, ea.v)
        pa, pb = a.main_model._params[0], b.main_model._params[0]
        assert float(a.main_optimizer.state[pa]["step"]) == float(b.main_optimizer.state[pb]["step"]) == 3.0
    assert float(a.cos_placeholder) == float(b.cos_placeholder)
    assert a.similarity_state.step == b.similarity_state.step == 4

    # the reference's format: model + a stock torch.optim state dict, trained without this library
    torch.manual_seed(0)
    stock = _model()
    sgroups = _groups(stock)
    sopt = torch.optim.SGD(sgroups, lr=0.1, momentum=0.9) if kind == "sgd" else torch.optim.AdamW(sgroups, lr=1e-2)
    for it in range(2):
        x, y = batch(it, K=1)
        sopt.zero_grad()
        torch.nn.functional.cross_entropy(stock(x), y).backward()
        sopt.step()
    sd = {"epoch": 1, "total_epoch_time": 0.0, "step": 2, "model": stock.state_dict(),
          "optimizer": sopt.state_dict(), "scheduler": None, "global_batch_size": 16, "local_batch_size": 8}
    p2 = str(tmp_path / "stock.pth")
    torch.save(sd, p2)
    c = make()
    c.load(p2)
    ec = c.reducer.engine
    lay = c.reducer.layout
    for p_stock, slot in zip(stock.parameters(), lay.slots):
        sl = slice(slot.offset, slot.offset + slot.numel)
        assert torch.equal(ec.weights[0][sl], p_stock.detach().reshape(-1))
        assert torch.equal(ec.weights[1][sl], p_stock.detach().reshape(-1))
        st = sopt.state[p_stock]
        key = "momentum_buffer" if kind == "sgd" else "exp_avg"
        assert torch.equal(ec.m[sl], st[key].reshape(-1))
        if kind != "sgd":
            assert torch.equal(ec.v[sl], st["exp_avg_sq"].reshape(-1))
    assert ec.steps == 2
    c.compute(batch(9)); c.step()                         # and training goes on from there
    torch.cuda.synchronize()
    assert torch.isfinite(ec.weights[0]).all()
    torch.backends.cudnn.deterministic = monkey_prev


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


@pytest.mark.parametrize("wsm,kind,K,interval,lr_step", [
    ("overlap", "sgd", 2, 1, False), ("sequential", "adamw", 4, 1, True), ("overlap", "adamw", 2, 2, True),
    ("sequential", "sgd", 4, 3, False)])
def test_iteration_graph_matches_reference_path(wsm, kind, K, interval, lr_step):
    """compute() + step() as ONE CUDA-graph launch per iteration (K forward/backward passes on K
    streams, the hooks' launches, the update, the statistic, zeroed gradients): the weights after
    every replay are bit-equal to the reference path fed with the gradients of that replay; the
    lr may change between replays (device-resident hyper-parameters), and iterations with and
    without the statistic replay their own graphs."""
    import jabas_b200
    from jabas_b200.iidp.optim import ShardAdamW, ShardSGD
    from oracle.reference_path import ReferencePath
    tr = jabas_b200.JABASTrainer(0, 8, K, 0, wsm, dict(CFG, batch_size_adjust_interval=interval))
    tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss().cuda(), bucket_cap_mb=0.05,
                               first_bucket_bytes=4096)
    groups = _groups(tr.main_model)
    if kind == "sgd":
        opt = (ShardSGD if wsm == "overlap" else torch.optim.SGD)(groups, lr=0.1, momentum=0.9)
    else:
        opt = (ShardAdamW if wsm == "overlap" else torch.optim.AdamW)(groups, lr=1e-2)
    tr.prepare_weight_sync_method(opt, None, _groups)
    tr.set_model_train()
    od = _opt_dict(kind)
    ref = ReferencePath(tr.reducer.layout, K, od, total_num_decoupled_workers=K, arith="c")
    for k in range(K):
        ref.weights[k].copy_(tr.reducer.engine.weights[k].cpu())
    captured = _capture_vsw_gradients(tr)
    lay = tr.reducer.layout
    tr.enable_iteration_graph(warmup=2)
    G = tr._iter_graph
    g = torch.Generator().manual_seed(3)
    static_copies = {}            # per graph: the clones made while capturing, refilled by every replay
    replays = 0
    for it in range(9):
        x = torch.randn(8 * K, 3, 16, 16, generator=g).cuda()
        y = torch.randint(0, 10, (8 * K,), generator=g).cuda()
        if lr_step and it in (4, 7):
            for gr, go in zip(opt.param_groups, od["groups"]):
                gr["lr"] *= 0.5
                go["lr"] *= 0.5
        sim = tr._is_similarity_step()
        ngraphs, launches = len(G["graphs"]), tr.reducer.engine.launches
        tr.compute((x, y))
        replayed = G["replayed"]
        assert tr.step() is True
        torch.cuda.synchronize()
        assert tr.reducer.engine.launches > launches
        if len(G["graphs"]) > ngraphs:
            static_copies[sim] = dict(captured)
        src = static_copies[sim] if replayed else captured
        replays += bool(replayed)
        assert len(src) == K * lay.num_buckets
        for (k, b), t in src.items():
            ref.grads[k][lay.buckets[b][0]:lay.buckets[b][1]].copy_(t.cpu())
        cos_ref = ref.run_iteration(similarity_step=sim)
        if sim:
            assert abs(float(tr.cos_placeholder) - cos_ref) < 1e-5, it
        for k in range(K):
            assert torch.equal(tr.reducer.engine.weights[k].cpu(), ref.weights[0]), (it, k, replayed)
        assert all(float(tr.reducer.engine.grads[k].abs().max()) == 0.0 for k in range(K))
        assert torch.isfinite(torch.stack([tr.losses[k].detach() for k in range(K)])).all()
    assert len(G["graphs"]) == (1 if interval == 1 else 2)
    assert replays == {1: 7, 2: 5, 3: 5}[interval]        # two eager iterations of each kind come first
    with pytest.raises(ValueError, match="shape"):
        tr.compute((torch.randn(4 * K, 3, 16, 16).cuda(), torch.zeros(4 * K, dtype=torch.long).cuda()))
    # a change of the VSW count drops the graphs; they are captured again for the new set
    tr.change_num_models(K + 2)
    assert not G["graphs"] and not G["seen"]
    x = torch.randn(8 * (K + 2), 3, 16, 16, generator=g).cuda()
    y = torch.randint(0, 10, (8 * (K + 2),), generator=g).cuda()
    for it in range(8):
        tr.compute((x, y))
        tr.step()
    torch.cuda.synchronize()
    assert len(G["graphs"]) >= 1
    for k in range(1, K + 2):
        assert torch.equal(tr.reducer.engine.weights[k], tr.reducer.engine.weights[0])
    tr.reducer.engine.close()


def test_iteration_graph_can_be_switched_off():
    """After ``disable_iteration_graph`` the trainer runs eagerly again and a changed lr reaches the
    kernels through the launch arguments (the device-resident block is gone)."""
    import jabas_b200
    from jabas_b200.iidp.optim import ShardSGD
    from oracle.reference_path import ReferencePath
    K = 2
    tr = jabas_b200.JABASTrainer(0, 8, K, 0, "overlap", dict(CFG))
    tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss().cuda(), bucket_cap_mb=0.05,
                               first_bucket_bytes=4096)
    opt = ShardSGD(_groups(tr.main_model), lr=0.1, momentum=0.9)
    tr.prepare_weight_sync_method(opt, None, _groups)
    tr.set_model_train()
    od = _opt_dict("sgd")
    ref = ReferencePath(tr.reducer.layout, K, od, total_num_decoupled_workers=K, arith="c")
    for k in range(K):
        ref.weights[k].copy_(tr.reducer.engine.weights[k].cpu())
    captured = _capture_vsw_gradients(tr)
    lay, eng = tr.reducer.layout, tr.reducer.engine
    g = torch.Generator().manual_seed(9)
    tr.enable_iteration_graph(warmup=1)
    static = None
    for it in range(6):
        if it == 4:
            tr.disable_iteration_graph()
            assert tr._iter_graph is None and eng._dyn is None
            for gr, go in zip(opt.param_groups, od["groups"]):
                gr["lr"] *= 0.25
                go["lr"] *= 0.25
        x = torch.randn(8 * K, 3, 16, 16, generator=g).cuda()
        y = torch.randint(0, 10, (8 * K,), generator=g).cuda()
        tr.compute((x, y))
        replayed = tr._iter_graph is not None and tr._iter_graph["replayed"]
        tr.step()
        torch.cuda.synchronize()
        if replayed and static is None:
            static = dict(captured)
        for (k, b), t in (static if replayed else captured).items():
            ref.grads[k][lay.buckets[b][0]:lay.buckets[b][1]].copy_(t.cpu())
        ref.run_iteration()
        assert torch.equal(eng.weights[K - 1].cpu(), ref.weights[0]), (it, replayed)
    assert static is not None
    eng.close()
