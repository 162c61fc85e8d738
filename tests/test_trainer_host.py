"""Host-side logic of the trainer / comm-hook / optimizer mirrors, on CPU.

The device kernels are replaced by the oracle-backed double of ``tests/oracle_backend.py``
(the product itself has no CPU path), so what is under test here is the plumbing: flat
views of parameters and gradients, bucket readiness and hook order over K VSWs, interval
gating, gradient accumulation, param-group segment tables, world_size-2 gloo collectives
and the parity sub-groups.  Expected values come from ``oracle.reference_path``: the
op-by-op restatement of the reference path, fed with the same per-VSW gradients.
"""
import copy
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import oracle_backend  # noqa: E402

import jabas_b200  # noqa: E402
from jabas_b200.iidp.optim import ShardAdamW, ShardSGD  # noqa: E402
from oracle.reference_path import ReferencePath  # noqa: E402

CFG = dict(similarity_target=0.1, batch_size_adjust_interval=1, enable_adjust=False)


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(20, 64), torch.nn.LayerNorm(64), torch.nn.ReLU(),
                               torch.nn.Linear(64, 48), torch.nn.ReLU(), torch.nn.Linear(48, 10))


def _groups(model):
    params = list(model.named_parameters())
    return [{"params": [p for n, p in params if p.dim() == 1], "weight_decay": 0.0},
            {"params": [p for n, p in params if p.dim() != 1], "weight_decay": 1e-2}]


def _make_trainer(K, wsm, kind, cfg=CFG, accum=0, mode="fused", cls=None):
    cls = cls or jabas_b200.JABASTrainer
    if cls is jabas_b200.JABASTrainer:
        tr = cls("cpu", 8, K, accum, wsm, dict(cfg), similarity_mode=mode)
    else:
        tr = cls("cpu", 8, K, accum, wsm)
    tr._backend = oracle_backend
    tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss(), bucket_cap_mb=0.01,
                               first_bucket_bytes=2048)
    groups = _groups(tr.main_model)
    if kind == "sgd":
        opt = (ShardSGD if wsm == "overlap" else torch.optim.SGD)(groups, lr=0.1, momentum=0.9)
    else:
        opt = (ShardAdamW if wsm == "overlap" else torch.optim.AdamW)(groups, lr=1e-2, betas=(0.9, 0.999),
                                                                       eps=1e-8)
    tr.prepare_weight_sync_method(opt, None, _groups)
    return tr


def _opt_dict(kind):
    if kind == "sgd":
        return dict(kind="sgd", groups=[dict(lr=0.1, weight_decay=0.0), dict(lr=0.1, weight_decay=1e-2)],
                    momentum=0.9)
    return dict(kind="adamw", groups=[dict(lr=1e-2, weight_decay=0.0), dict(lr=1e-2, weight_decay=1e-2)],
                betas=(0.9, 0.999), eps=1e-8)


def _reference_for(tr, kind, similarity=True):
    ref = ReferencePath(tr.reducer.layout, tr.num_models, _opt_dict(kind),
                        total_num_decoupled_workers=tr.total_num_decoupled_workers,
                        similarity=similarity, arith="c")
    for k in range(tr.num_models):
        ref.weights[k].copy_(tr.reducer.engine.weights[k])
    return ref


def _vsw_gradients(tr, x, y, scale=1.0):
    """Per-VSW flat gradients of the trainer's CURRENT weights, by plain autograd."""
    lay = tr.reducer.layout
    out = []
    for k, (xs, ys) in enumerate(zip(torch.chunk(x, tr.num_models), torch.chunk(y, tr.num_models))):
        m = copy.deepcopy(tr.original_local_models[k])
        for p in m.parameters():
            p.grad = None
        torch.nn.functional.cross_entropy(m(xs), ys).backward()
        flat = torch.zeros(lay.total)
        for p, s in zip(m.parameters(), lay.slots):
            flat[s.offset:s.offset + s.numel] = p.grad.reshape(-1)
        out.append(flat)
    return out


@pytest.mark.parametrize("wsm", ["sequential", "overlap"])
@pytest.mark.parametrize("kind", ["sgd", "adamw"])
@pytest.mark.parametrize("K", [2, 4])
def test_single_rank_trainer_matches_reference_path(wsm, kind, K):
    tr = _make_trainer(K, wsm, kind)
    assert tr.reducer.layout.num_buckets >= 3
    ref = _reference_for(tr, kind)
    g = torch.Generator().manual_seed(1)
    for it in range(3):
        x, y = torch.randn(8 * K, 20, generator=g), torch.randint(0, 10, (8 * K,), generator=g)
        for k, flat in enumerate(_vsw_gradients(tr, x, y)):
            ref.grads[k].copy_(flat)
        cos_ref = ref.run_iteration()
        tr.compute((x, y))
        assert tr.step() is True
        assert abs(float(tr.cos_placeholder) - cos_ref) < 1e-5
        for k in range(K):
            assert torch.equal(tr.reducer.engine.weights[k], ref.weights[0]), (it, k)
        # the modules see the new weights through their views, in every replica
        for p0, pk in zip(tr.local_models[0].parameters(), tr.local_models[K - 1].parameters()):
            assert torch.equal(p0, pk)
    assert tr.sync_step == 3 and tr.similarity_state.step == 4


def test_optimizer_state_is_exposed_per_parameter():
    tr = _make_trainer(2, "sequential", "sgd")
    x, y = torch.randn(16, 20), torch.randint(0, 10, (16,))
    tr.compute((x, y)); tr.step()
    sd = tr.main_optimizer.state_dict()
    assert len(sd["state"]) == len(list(tr.main_model.parameters()))
    for p in tr.main_model.parameters():
        buf = tr.main_optimizer.state[p]["momentum_buffer"]
        assert buf.shape == p.shape and buf.abs().sum() > 0
    tr2 = _make_trainer(2, "sequential", "adamw")
    tr2.compute((x, y)); tr2.step()
    st = tr2.main_optimizer.state[next(tr2.main_model.parameters())]
    assert float(st["step"]) == 1.0 and st["exp_avg"].abs().sum() > 0


def test_lr_changes_between_iterations_reach_the_kernel():
    tr = _make_trainer(2, "overlap", "sgd")
    ref = _reference_for(tr, "sgd")
    g = torch.Generator().manual_seed(3)
    for it, lr in enumerate([0.1, 0.05, 0.2]):
        for pg in tr.main_optimizer.param_groups:           # what an lr scheduler does
            pg["lr"] = lr
        for gr in ref.opt["groups"]:
            gr["lr"] = lr
        x, y = torch.randn(16, 20, generator=g), torch.randint(0, 10, (16,), generator=g)
        for k, flat in enumerate(_vsw_gradients(tr, x, y)):
            ref.grads[k].copy_(flat)
        ref.run_iteration()
        tr.compute((x, y)); tr.step()
        assert torch.equal(tr.reducer.engine.weights[0], ref.weights[0])


def test_interval_gates_the_statistic():
    cfg = dict(CFG, batch_size_adjust_interval=3)
    tr = _make_trainer(2, "sequential", "sgd", cfg)
    seen = []
    for it in range(6):
        x, y = torch.randn(16, 20), torch.randint(0, 10, (16,))
        before = float(tr.cos_placeholder)
        tr.compute((x, y)); tr.step()
        seen.append(float(tr.cos_placeholder) != before)
    # state.step starts at 1 (jabas/ddp_comm_hooks/similarity_allreduce.py:17): steps 3 and 6 qualify
    assert seen == [False, False, True, False, False, True]


def test_gradient_accumulation_defers_the_hooks():
    K, accum = 2, 1
    tr = _make_trainer(K, "sequential", "sgd", accum=accum)
    assert tr.total_num_decoupled_workers == K * (accum + 1)
    ref = _reference_for(tr, "sgd")
    g = torch.Generator().manual_seed(5)
    x1, y1 = torch.randn(16, 20, generator=g), torch.randint(0, 10, (16,), generator=g)
    x2, y2 = torch.randn(16, 20, generator=g), torch.randint(0, 10, (16,), generator=g)
    g1, g2 = _vsw_gradients(tr, x1, y1), _vsw_gradients(tr, x2, y2)
    for k in range(K):
        ref.grads[k].copy_(g1[k] + g2[k])                 # accumulated in place in the bucket views
    ref.run_iteration()
    tr.compute((x1, y1))
    assert tr.step() is False and tr.reducer.engine.launches == 0
    tr.compute((x2, y2))
    assert tr.step() is True
    assert torch.equal(tr.reducer.engine.weights[0], ref.weights[0])


def test_iidp_trainer_without_similarity_and_foreign_hook():
    tr = _make_trainer(3, "sequential", "sgd", cls=jabas_b200.IIDPTrainer)
    ref = _reference_for(tr, "sgd", similarity=False)
    x, y = torch.randn(24, 20), torch.randint(0, 10, (24,))
    for k, flat in enumerate(_vsw_gradients(tr, x, y)):
        ref.grads[k].copy_(flat)
    ref.run_iteration()
    tr.compute((x, y)); tr.step()
    assert torch.equal(tr.reducer.engine.weights[2], ref.weights[0])

    # a caller-supplied hook in the PyTorch 1.8 form sees the plain local sum
    tr2 = _make_trainer(3, "sequential", "sgd", cls=jabas_b200.IIDPTrainer)
    ref2 = _reference_for(tr2, "sgd", similarity=False)
    T = tr2.total_num_decoupled_workers

    def my_hook(state, bucket):
        t = bucket.get_tensors()[0]
        t.div_(T)
        fut = torch.futures.Future()
        fut.set_result([t])
        return fut
    tr2.local_models[0].register_comm_hook(None, my_hook)
    for k, flat in enumerate(_vsw_gradients(tr2, x, y)):
        ref2.grads[k].copy_(flat)
    ref2.run_iteration()
    tr2.compute((x, y)); tr2.step()
    assert torch.equal(tr2.reducer.engine.weights[0], ref2.weights[0])


def test_constructor_contract():
    with pytest.raises(ValueError):
        jabas_b200.JABASTrainer("cpu", 8, 2, 0, "sequential", None)
    with pytest.raises(AssertionError):                      # T must be even for the two halves
        tr = jabas_b200.JABASTrainer("cpu", 8, 3, 0, "sequential", dict(CFG))
        tr._backend = oracle_backend
        tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss())
    tr = _make_trainer(2, "sequential", "sgd")
    assert tr.global_batch_size == 16 and tr.batch_size_per_gpu == 16
    assert len(tr.hooks) == 2 and tr.hooks[1] is jabas_b200.iidp.ddp_comm_hooks.dummy_hook
    assert tr.states[0] is tr.similarity_state and tr.states[1] is None
    with pytest.raises(ValueError, match="Shard"):
        t2 = jabas_b200.IIDPTrainer("cpu", 8, 2, 0, "overlap")
        t2._backend = oracle_backend
        t2.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss())
        t2.prepare_weight_sync_method(torch.optim.SGD(t2.main_model.parameters(), lr=0.1))


# ---------------------------------------------------------------------------------------
# world_size 2 on gloo
# ---------------------------------------------------------------------------------------

def _rank_main(rank, world, port, mode, kind, wsm, q):
    try:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        torch.set_num_threads(1)
        K = 2
        tr = _make_trainer(K, wsm, kind, mode=mode)
        assert tr.total_num_decoupled_workers == world * K
        assert tr.sub_groups_idx == [[0], [1]] and (tr.first_subgroup_src_rank, tr.second_subgroup_src_rank) == (0, 1)
        ref = _reference_for(tr, kind)
        g = torch.Generator().manual_seed(100 + rank)
        worst_w, worst_c = 0.0, 0.0
        for it in range(3):
            x, y = torch.randn(8 * K, 20, generator=g), torch.randint(0, 10, (8 * K,), generator=g)
            for k, flat in enumerate(_vsw_gradients(tr, x, y)):
                ref.grads[k].copy_(flat)
            cos_ref = ref.run_iteration()
            tr.compute((x, y)); tr.step()
            w, wr = tr.reducer.engine.weights[K - 1], ref.weights[0]
            worst_w = max(worst_w, float(((w - wr).abs() / wr.abs().clamp_min(1e-3)).max()))
            worst_c = max(worst_c, abs(float(tr.cos_placeholder) - cos_ref))
        both = [None, None]
        dist.all_gather_object(both, float(tr.cos_placeholder))
        q.put((rank, worst_w, worst_c, both[0] == both[1]))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc(), False))


@pytest.mark.parametrize("mode,kind,wsm", [("fused", "sgd", "overlap"), ("pair_exchange", "sgd", "sequential"),
                                           ("fused", "adamw", "sequential"), ("pair_exchange", "adamw", "overlap")])
def test_two_gloo_ranks_match_reference_path(mode, kind, wsm):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + hash((mode, kind, wsm))) % 400
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, mode, kind, wsm, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, w, c, same in res:
        assert w != "error", c
        assert w <= 1e-6, (rank, w)          # fp32 weights within 1e-6 relative after the allreduce
        assert c <= 1e-5, (rank, c)          # cosine within 1e-5 absolute
        assert same                          # every rank holds rank 0's value


def test_gradient_norm_clipping_sequential_and_overlap():
    """Whole-model clipping (sequential mode, clip_grad_norm_ between compute and step) and
    per-bucket clipping (overlap mode, ShardAdam(grad_clip=...)) against the oracle."""
    from jabas_b200.iidp.optim import ShardAdam
    from jabas_b200.iidp.utils.clip_grad import clip_grad_norm_
    from oracle import gradpath as O
    K, clip = 2, 0.05
    for wsm in ("sequential", "overlap"):
        tr = jabas_b200.JABASTrainer("cpu", 8, K, 0, wsm, dict(CFG))
        tr._backend = oracle_backend
        tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss(), bucket_cap_mb=0.01,
                                   first_bucket_bytes=2048)
        params = list(tr.main_model.parameters())
        if wsm == "overlap":
            opt = ShardAdam(params, lr=1e-2, grad_clip=clip)
        else:
            opt = torch.optim.Adam(params, lr=1e-2)
        tr.prepare_weight_sync_method(opt)
        lay = tr.reducer.layout
        ref = ReferencePath(lay, K, dict(kind="adam", groups=[dict(lr=1e-2, weight_decay=0.0)],
                                         betas=(0.9, 0.999), eps=1e-8),
                            total_num_decoupled_workers=K, arith="c")
        for k in range(K):
            ref.weights[k].copy_(tr.reducer.engine.weights[k])
        x, y = torch.randn(16, 20), torch.randint(0, 10, (16,))
        for k, flat in enumerate(_vsw_gradients(tr, x, y)):
            ref.grads[k].copy_(flat)
        for b in range(lay.num_buckets):
            ref.reduce_bucket(b, True)
        g = ref.grads[0].numpy()
        if wsm == "overlap":
            norms = [O.clip_grad_norm(g[bb:be], clip)[1] for bb, be in lay.buckets]
            assert max(norms) > clip                          # the clip is active
        else:
            coef, norm = O.clip_grad_norm(g, clip)
            assert coef < 1.0
        ref.optimizer_step(); ref.copy_weights(); ref.compute_cosine_similarity()
        tr.compute((x, y))
        if wsm == "sequential":
            total = clip_grad_norm_(tr.main_model.parameters(), clip)
        tr.step()
        assert torch.equal(tr.reducer.engine.weights[K - 1], ref.weights[0]), wsm
        if wsm == "sequential":
            assert abs(float(total) - norm) < 1e-6 * norm


def test_runtime_change_of_vsw_count():
    """K: 2 -> 4 -> 2 between iterations: buffers that stay are not reallocated, the new
    replicas start from the main weights, T reaches the hook state and the kernels."""
    tr = _make_trainer(2, "overlap", "sgd")
    eng = tr.reducer.engine
    g = torch.Generator().manual_seed(9)

    def one_step(K):
        ref = _reference_for(tr, "sgd")
        ref.steps = eng.steps
        ref.m.copy_(eng.m)
        x, y = torch.randn(8 * K, 20, generator=g), torch.randint(0, 10, (8 * K,), generator=g)
        for k, flat in enumerate(_vsw_gradients(tr, x, y)):
            ref.grads[k].copy_(flat)
        cos_ref = ref.run_iteration()
        tr.compute((x, y)); tr.step()
        for k in range(K):
            assert torch.equal(eng.weights[k], ref.weights[0]), k
        assert abs(float(tr.cos_placeholder) - cos_ref) < 1e-5

    one_step(2)
    ptr_w0, ptr_g1, ptr_m = eng.weights[0].data_ptr(), eng.grads[1].data_ptr(), eng.m.data_ptr()
    tr.change_num_models(4)
    assert tr.num_models == 4 and eng.K == 4 and len(tr.local_models) == 4 and len(tr.hooks) == 4
    assert tr.total_num_decoupled_workers == 4 and tr.similarity_state.total_num_decoupled_workers == 4
    assert tr.similarity_state.subgroup_total_num_decoupled_workers == 2
    assert tr.batch_size_per_gpu == 32 and tr.global_batch_size == 32
    assert (eng.weights[0].data_ptr(), eng.grads[1].data_ptr(), eng.m.data_ptr()) == (ptr_w0, ptr_g1, ptr_m)
    assert torch.equal(eng.weights[3], eng.weights[0])
    one_step(4)
    tr.change_num_models(2)
    assert eng.K == 2 and len(tr.local_models) == 2 and len(tr.model_streams) == 2
    assert eng.weights[0].data_ptr() == ptr_w0
    one_step(2)


@pytest.mark.parametrize("kind", ["sgd", "adamw"])
def test_checkpoint_round_trip(kind, tmp_path):
    """save -> new trainer -> load -> both take the same next step (weights, optimizer state,
    step counters, similarity step); the keys are those of the reference's checkpoints."""
    a = _make_trainer(2, "sequential", kind)
    g = torch.Generator().manual_seed(21)
    batches = [(torch.randn(16, 20, generator=g), torch.randint(0, 10, (16,), generator=g)) for _ in range(3)]
    for x, y in batches[:2]:
        a.compute((x, y)); a.step()
    path = a.save(str(tmp_path))
    sd = torch.load(path, weights_only=False)
    for key in ("epoch", "total_epoch_time", "step", "model", "optimizer", "scheduler", "gbs_trajectory",
                "similarity_step", "global_lr_modifier", "global_batch_size", "local_batch_size"):
        assert key in sd, key
    assert len(sd["optimizer"]["state"]) == len(list(a.main_model.parameters()))
    b = _make_trainer(2, "sequential", kind)
    b.load(str(tmp_path), restrict_saved_config=True)
    assert b.sync_step == 2 and b.similarity_state.step == a.similarity_state.step
    assert b.reducer.engine.steps == a.reducer.engine.steps
    for k in range(2):
        assert torch.equal(b.reducer.engine.weights[k], a.reducer.engine.weights[0])
    assert torch.equal(b.reducer.engine.m, a.reducer.engine.m)
    x, y = batches[2]
    a.compute((x, y)); a.step()
    b.compute((x, y)); b.step()
    assert torch.equal(b.reducer.engine.weights[1], a.reducer.engine.weights[0])
    # a stock torch optimizer can read the same optimizer state (it is per parameter)
    params = [torch.nn.Parameter(p.detach().clone()) for p in a.main_model.parameters()]
    named = list(zip([n for n, _ in a.main_model.named_parameters()], params))
    groups = [{"params": [p for n, p in named if p.dim() == 1], "weight_decay": 0.0},
              {"params": [p for n, p in named if p.dim() != 1], "weight_decay": 1e-2}]
    stock = torch.optim.SGD(groups, lr=0.1, momentum=0.9) if kind == "sgd" else torch.optim.AdamW(groups, lr=1e-2)
    stock.load_state_dict(a.main_optimizer.state_dict())


@pytest.mark.parametrize("wsm", ["sequential", "overlap"])
def test_replicas_may_share_one_weight_buffer(wsm):
    """share_weights=True: every replica's parameters are views of the same flat buffer, the
    update writes it once, and results are those of K separate replicas."""
    K = 4
    tr = jabas_b200.JABASTrainer("cpu", 8, K, 0, wsm, dict(CFG))
    tr._backend = oracle_backend
    tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss(), bucket_cap_mb=0.01,
                               first_bucket_bytes=2048, share_weights=True)
    groups = _groups(tr.main_model)
    opt = (ShardSGD if wsm == "overlap" else torch.optim.SGD)(groups, lr=0.1, momentum=0.9)
    tr.prepare_weight_sync_method(opt, None, _groups)
    eng = tr.reducer.engine
    assert all(w.data_ptr() == eng.weights[0].data_ptr() for w in eng.weights)
    p0 = next(tr.local_models[0].parameters()); p3 = next(tr.local_models[3].parameters())
    assert p0.data_ptr() == p3.data_ptr() and p0 is not p3
    ref = _reference_for(tr, "sgd")
    g = torch.Generator().manual_seed(1)
    for it in range(3):
        x, y = torch.randn(8 * K, 20, generator=g), torch.randint(0, 10, (8 * K,), generator=g)
        for k, flat in enumerate(_vsw_gradients(tr, x, y)):
            ref.grads[k].copy_(flat)
        cos_ref = ref.run_iteration()
        tr.compute((x, y)); tr.step()
        assert torch.equal(eng.weights[0], ref.weights[0])
        assert abs(float(tr.cos_placeholder) - cos_ref) < 1e-5
    tr.change_num_models(2); tr.change_num_models(4)
    assert eng.weights[3].data_ptr() == eng.weights[0].data_ptr()


def test_groups_may_differ_only_in_lr_and_weight_decay():
    tr = jabas_b200.IIDPTrainer("cpu", 8, 2, 0, "sequential")
    tr._backend = oracle_backend
    tr.prepare_stream_parallel(_model(), torch.nn.CrossEntropyLoss())
    groups = _groups(tr.main_model)
    groups[0]["momentum"] = 0.5
    with pytest.raises(NotImplementedError, match="momentum"):
        tr.prepare_weight_sync_method(torch.optim.SGD(groups, lr=0.1, momentum=0.9))


@pytest.mark.parametrize("wsm", ["sequential", "overlap"])
def test_threaded_compute_gives_the_same_result(wsm):
    """K forward/backward passes from K threads: hooks still fire one bucket at a time, in
    bucket order, and the result equals the single-threaded one bit for bit."""
    K = 4
    a, b = _make_trainer(K, wsm, "sgd"), _make_trainer(K, wsm, "sgd")
    b.threaded_compute = True
    g = torch.Generator().manual_seed(31)
    for it in range(4):
        x, y = torch.randn(8 * K, 20, generator=g), torch.randint(0, 10, (8 * K,), generator=g)
        a.compute((x, y)); a.step()
        b.compute((x, y)); b.step()
        assert torch.equal(a.reducer.engine.weights[0], b.reducer.engine.weights[K - 1]), it
        assert float(a.cos_placeholder) == float(b.cos_placeholder)


def test_module_buffers_are_flat_views_and_follow_vsw0():
    """Host logic of the buffer synchronisation: every module buffer of every VSW is a view of
    that VSW's flat byte buffer (dtype and shape kept), and ``sync_buffers`` gives all VSWs the
    main replica's values — the DistributedDataParallel ``broadcast_buffers`` step."""
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(20, 32), torch.nn.BatchNorm1d(32), torch.nn.ReLU(),
                                torch.nn.Linear(32, 10))
    K = 3
    tr = jabas_b200.IIDPTrainer("cpu", 8, K, 0, "sequential")
    tr._backend = oracle_backend
    tr.prepare_stream_parallel(model, torch.nn.CrossEntropyLoss(), bucket_cap_mb=0.01, first_bucket_bytes=2048)
    tr.prepare_weight_sync_method(torch.optim.SGD(tr.main_model.parameters(), lr=0.1, momentum=0.9))
    tr.set_model_train()
    red = tr.reducer
    assert red.num_module_buffers == 3 and len(red.buffers_flat) == K
    for k in range(K):
        bn = tr.local_models[k].module[1]
        assert bn.running_mean.dtype == torch.float32 and bn.num_batches_tracked.dtype == torch.int64
        assert bn.running_mean.shape == (32,) and bn.num_batches_tracked.shape == ()
        spans = [(f.data_ptr(), f.data_ptr() + f.numel() * f.element_size()) for f in red.buffers_flat[k]]
        for b in bn.buffers():
            assert any(lo <= b.data_ptr() < hi and (b.data_ptr() - lo) % 16 == 0 for lo, hi in spans)
    x, y = torch.randn(8 * K, 20), torch.randint(0, 10, (8 * K,))
    tr.compute((x, y)); tr.step()
    means = [lm.module[1].running_mean.clone() for lm in tr.local_models]
    assert not torch.equal(means[0], means[1])
    tr.compute((x, y)); tr.step()              # the next forward starts from VSW 0's statistics
    for k in range(K):
        assert int(tr.local_models[k].module[1].num_batches_tracked) == 2
    red.sync_buffers()
    for lm in tr.local_models[1:]:
        for a, b in zip(lm.module.buffers(), tr.local_models[0].module.buffers()):
            assert torch.equal(a, b)


# ---------------------------------------------------------------------------------------
# the reference's CPU-runnable configuration: ResNet-50, gloo world_size 2, K = 2, LBS 8
# ---------------------------------------------------------------------------------------

def _config1_rank(rank, world, port, iters, q):
    try:
        import torchvision
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        torch.set_num_threads(max(1, (os.cpu_count() or 2) // world))
        K, lbs = 2, 8
        tr = jabas_b200.JABASTrainer("cpu", lbs, K, 0, "overlap", dict(CFG))
        tr._backend = oracle_backend
        torch.manual_seed(0)
        tr.prepare_stream_parallel(torchvision.models.resnet50(), torch.nn.CrossEntropyLoss())   # 25 MiB buckets

        def groups(m):
            named = list(m.named_parameters())
            return [{"params": [p for n, p in named if "bn" in n], "weight_decay": 0},
                    {"params": [p for n, p in named if "bn" not in n], "weight_decay": 1e-4}]
        tr.prepare_weight_sync_method(ShardSGD(groups(tr.main_model), 0.1, momentum=0.9, weight_decay=1e-4),
                                      None, groups)
        tr.set_model_train()
        lay = tr.reducer.layout
        assert lay.num_params == 25557032 and lay.bucket_sizes_mib() == [7.82, 30.04, 25.04, 25.32, 9.27]
        assert tr.total_num_decoupled_workers == world * K
        opt = dict(kind="sgd", groups=[dict(lr=0.1, weight_decay=0.0), dict(lr=0.1, weight_decay=1e-4)], momentum=0.9)
        # two executions of the reference path's op sequence: stock torch CPU ops (weights), and the
        # C oracle, whose cosine sums are fp64 — stock fp32 reductions over 25.6 M elements of real
        # gradients (|g| ~ 200 at random init) are themselves off by up to ~1e-3 in the cosine
        ref = ReferencePath(lay, K, opt, total_num_decoupled_workers=world * K, arith="torch")
        ref64 = ReferencePath(lay, K, opt, total_num_decoupled_workers=world * K, arith="c")
        for k in range(K):
            ref.weights[k].copy_(tr.reducer.engine.weights[k])
            ref64.weights[k].copy_(tr.reducer.engine.weights[k])
        captured = {}
        for k, lm in enumerate(tr.local_models):
            def hook(state, bucket, k=k, orig=lm._hook):
                captured[(k, bucket.index())] = bucket.buffer(materialize=False).clone()
                return orig(state, bucket)
            lm.register_comm_hook(lm._hook_state, hook)
        worst_w = worst_c = 0.0
        cosines = []
        for it in range(iters):
            xs, ys = [], []
            for k in range(K):                               # seed = 1000 * rank + 10 * k + iteration
                g = torch.Generator().manual_seed(1000 * rank + 10 * k + it)
                xs.append(torch.randn(lbs, 3, 224, 224, generator=g))
                ys.append(torch.randint(0, 1000, (lbs,), generator=g))
            tr.compute((torch.cat(xs), torch.cat(ys)))
            assert tr.step() is True
            assert len(captured) == K * lay.num_buckets
            for (k, b), t in captured.items():
                ref.grads[k][lay.buckets[b][0]:lay.buckets[b][1]].copy_(t)
                ref64.grads[k][lay.buckets[b][0]:lay.buckets[b][1]].copy_(t)
            captured.clear()
            cos_torch = ref.run_iteration()
            cos_ref = ref64.run_iteration()
            w = tr.reducer.engine.weights[K - 1]
            for wr in (ref.weights[0], ref64.weights[0]):
                worst_w = max(worst_w, float(((w - wr).abs() / wr.abs().clamp_min(1e-3)).max()))
            worst_c = max(worst_c, abs(float(tr.cos_placeholder) - cos_ref))
            assert abs(cos_torch - cos_ref) < 5e-3               # the stock fp32 reduction's own rounding
            cosines.append(float(tr.cos_placeholder))
        chk = int(tr.reducer.engine.weights[0].view(torch.int32).to(torch.int64).sum())
        both = [None] * world
        dist.all_gather_object(both, (chk, cosines))
        q.put((rank, worst_w, worst_c, both[0] == both[1], cosines))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc(), False, []))


def test_config1_resnet50_two_gloo_ranks_five_iterations():
    """ResNet-50 (seed 0), CPU, gloo world_size 2, 2 VSWs per rank with local batch 8, N(0,1)
    images, SGD momentum 0.9 lr 0.1 wd 1e-4 (BN parameters without decay), 25 MiB buckets,
    statistic every iteration, 5 iterations: the trainer / hook / optimizer mirrors (device kernels
    replaced by the oracle-backed double) against the reference path's op sequence executed with
    stock torch CPU ops on the same ranks, fed with the gradients captured from the run."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + 77) % 400
    procs = [ctx.Process(target=_config1_rank, args=(r, 2, port, 5, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=900) for _ in procs]
    for p in procs:
        p.join(timeout=120)
    for rank, w, c, same, cosines in res:
        assert w != "error", c
        assert w <= 1e-6, (rank, w)
        assert c <= 1e-5, (rank, c)
        assert same                                           # both ranks: same weights, same cosines
        assert len(cosines) == 5 and all(-1.0 <= x <= 1.0 for x in cosines)


class _Branchy(torch.nn.Module):
    """A model with a head that the forward pass never uses."""

    def __init__(self):
        super().__init__()
        self.body = torch.nn.Sequential(torch.nn.Linear(20, 32), torch.nn.ReLU(), torch.nn.Linear(32, 10))
        self.unused = torch.nn.Linear(32, 7)

    def forward(self, x):
        return self.body(x)


def test_find_unused_parameters():
    """Parameters outside the graph: with the flag their buckets complete with zero gradients at
    the end of each VSW's backward (weights stay, momentum stays zero, the rest matches the
    reference path fed with zeros there); without it the incomplete bucket is an error."""
    def make(flag):
        torch.manual_seed(0)
        tr = jabas_b200.JABASTrainer("cpu", 8, 2, 0, "overlap", dict(CFG))
        tr._backend = oracle_backend
        tr.prepare_stream_parallel(_Branchy(), torch.nn.CrossEntropyLoss(), bucket_cap_mb=0.002, first_bucket_bytes=512,
                                   find_unused_parameters=flag)
        tr.prepare_weight_sync_method(ShardSGD(tr.main_model.parameters(), lr=0.1, momentum=0.9))
        return tr
    x, y = torch.randn(16, 20), torch.randint(0, 10, (16,))
    tr = make(False)
    with pytest.raises(RuntimeError, match="find_unused_parameters"):
        tr.compute((x, y))
    tr = make(True)
    lay, eng = tr.reducer.layout, tr.reducer.engine
    ref = ReferencePath(lay, 2, dict(kind="sgd", groups=[dict(lr=0.1, weight_decay=0.0)], momentum=0.9),
                        total_num_decoupled_workers=2, arith="c")
    for k in range(2):
        ref.weights[k].copy_(eng.weights[k])
    w_unused = tr.main_model.module.unused.weight.detach().clone()
    for it in range(2):
        xs, ys = torch.chunk(x, 2), torch.chunk(y, 2)
        for k in range(2):                                   # per-VSW gradients by plain autograd
            m = copy.deepcopy(tr.local_models[k].module)
            m.zero_grad()
            torch.nn.functional.cross_entropy(m(xs[k]), ys[k]).backward()
            flat = torch.zeros(lay.total)
            for p, slot in zip(m.parameters(), lay.slots):
                if p.grad is not None:
                    flat[slot.offset:slot.offset + slot.numel] = p.grad.reshape(-1)
            ref.grads[k].copy_(flat)
        ref.run_iteration()
        tr.compute((x, y))
        assert tr.step() is True
        assert torch.equal(eng.weights[1], ref.weights[0])
    assert torch.equal(tr.main_model.module.unused.weight, w_unused)


def test_iteration_graph_needs_a_cuda_device():
    """The whole-iteration CUDA graph is a device feature: on the CPU double it refuses."""
    tr = _make_trainer(2, "overlap", "sgd")
    with pytest.raises(RuntimeError, match="CUDA"):
        tr.enable_iteration_graph()
    assert tr._iter_graph is None
