"""Two NCCL ranks on two GPUs (skipped on a box with fewer): the whole path through the
trainer mirror — K VSWs, hooks fired from backward, sub-group + world allreduce, fused
update and statistic — against the reference-path restatement run on the same ranks over
gloo with the gradients captured from the GPU run."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _rank_main(rank, world, port, mode, kind, wsm, q, collective="nccl", graph=False):
    try:
        sys.path.insert(0, HERE)
        sys.path.insert(0, os.path.dirname(HERE))
        import torch.distributed as dist
        import jabas_b200
        from jabas_b200.iidp.optim import ShardAdamW, ShardSGD
        from oracle.reference_path import ReferencePath
        import test_trainer_gpu as T
        torch.cuda.set_device(rank)
        dist.init_process_group("cpu:gloo,cuda:nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                                world_size=world)
        K = 2
        tr = jabas_b200.JABASTrainer(rank, 8, K, 0, wsm, dict(T.CFG), similarity_mode=mode)
        tr.prepare_stream_parallel(T._model(), torch.nn.CrossEntropyLoss().cuda(), bucket_cap_mb=0.05,
                                   first_bucket_bytes=4096, collective=collective)
        groups = T._groups(tr.main_model)
        if kind == "sgd":
            opt = (ShardSGD if wsm == "overlap" else torch.optim.SGD)(groups, lr=0.1, momentum=0.9)
        else:
            opt = (ShardAdamW if wsm == "overlap" else torch.optim.AdamW)(groups, lr=1e-2)
        tr.prepare_weight_sync_method(opt, None, T._groups)
        tr.set_model_train()
        ref = ReferencePath(tr.reducer.layout, K, T._opt_dict(kind),
                            total_num_decoupled_workers=tr.total_num_decoupled_workers, arith="c")
        for k in range(K):
            ref.weights[k].copy_(tr.reducer.engine.weights[k].cpu())
        captured = T._capture_vsw_gradients(tr)
        lay = tr.reducer.layout
        g = torch.Generator().manual_seed(50 + rank)
        worst_w = worst_c = 0.0
        static_copies = None
        for it in range(9 if graph else 3):
            if graph and it == 3:
                # from here on compute() + step() are ONE graph launch per iteration (collectives or
                # exchange kernels included); two more eager iterations on the capture stream first
                tr.enable_iteration_graph(warmup=2)
            x = torch.randn(8 * K, 3, 16, 16, generator=g).cuda()
            y = torch.randint(0, 10, (8 * K,), generator=g).cuda()
            tr.compute((x, y))
            replayed = graph and it >= 3 and tr._iter_graph["replayed"]
            tr.step()
            torch.cuda.synchronize()
            if replayed and static_copies is None:
                static_copies = dict(captured)      # clones made during capture: every replay refills them
            for (k, b), t in (static_copies if replayed else captured).items():
                ref.grads[k][lay.buckets[b][0]:lay.buckets[b][1]].copy_(t.cpu())
            if not replayed:
                captured.clear()
            cos_ref = ref.run_iteration()
            wr = ref.weights[0]
            w = tr.reducer.engine.weights[K - 1].cpu()
            worst_w = max(worst_w, float(((w - wr).abs() / wr.abs().clamp_min(1e-3)).max()))
            worst_c = max(worst_c, abs(float(tr.cos_placeholder) - cos_ref))
        if tr.reducer.engine.exchange is not None:
            tr.reducer.engine.check_exchange()
        # module buffers: after a synchronisation every VSW on every rank holds rank 0's
        tr.reducer.sync_buffers()
        torch.cuda.synchronize()
        sums = [None] * world
        dist.all_gather_object(sums, [sum(int(f.view(torch.uint8).to(torch.int64).sum()) for f in fs)
                                      for fs in tr.reducer.buffers_flat])
        if len({tuple(s) for s in sums}) != 1 or len(set(sums[0])) != 1:
            worst_w = float("inf")
        if graph and not tr._iter_graph["graphs"]:
            worst_w = float("inf")
        tr.disable_iteration_graph()
        q.put((rank, worst_w, worst_c, tr.reducer.engine.launches))
        dist.barrier()
        torch.cuda.synchronize()
        tr.reducer.engine.close()
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc(), 0))


@pytest.mark.parametrize("mode,kind,wsm,collective,graph", [
    ("fused", "sgd", "overlap", "nccl", False), ("pair_exchange", "sgd", "sequential", "nccl", False),
    ("fused", "adamw", "overlap", "nccl", False), ("fused", "adamw", "sequential", "nccl", False),
    ("fused", "sgd", "sequential", "peer", False), ("fused", "adamw", "sequential", "peer", False),
    ("fused", "sgd", "overlap", "peer", False), ("fused", "adamw", "overlap", "peer", False),
    ("fused", "sgd", "overlap", "peer", True), ("fused", "adamw", "overlap", "nccl", True)])
def test_two_nccl_ranks_match_reference_path(mode, kind, wsm, collective, graph):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + hash((mode, kind, wsm, collective, graph))) % 400
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, mode, kind, wsm, q, collective, graph))
             for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, w, c, launches in res:
        assert w != "error", c
        assert w <= 1e-6, (rank, w)
        assert c <= 1e-5, (rank, c)
        assert launches > 0


def _engine_rank(rank, world, port, collective, kind, K, q, direct=None):
    try:
        sys.path.insert(0, os.path.dirname(HERE))
        import datetime
        import numpy as np
        import torch.distributed as dist
        from jabas_b200.gradient_path import GradientPath, OptimizerSpec
        from jabas_b200.layout import build_layout
        from oracle.reference_path import ReferencePath
        torch.cuda.set_device(rank)
        dist.init_process_group("cpu:gloo,cuda:nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                                world_size=world, timeout=datetime.timedelta(seconds=120))
        shapes = [(64, 3, 7, 7), (64,), (64,), (256, 64, 3, 3), (1000, 257), (1000,), (333,)]
        names = ["c1.w", "bn1.w", "bn1.b", "c2.w", "fc.w", "fc.b", "odd"]
        layout = build_layout(names, shapes, [1, 0, 0, 1, 1, 1, 0], bucket_cap_mb=0.5, first_bucket_bytes=64 * 1024)
        if kind == "sgd":
            opt = dict(kind="sgd", groups=[dict(lr=0.1, weight_decay=0.0), dict(lr=0.1, weight_decay=1e-4)], momentum=0.9)
        else:
            opt = dict(kind=kind, groups=[dict(lr=1e-3, weight_decay=0.0), dict(lr=1e-3, weight_decay=0.05)],
                       betas=(0.9, 0.999), eps=1e-8)
        spec = OptimizerSpec(opt["kind"], opt["groups"], momentum=opt.get("momentum", 0.0))
        idx = [[r for r in range(world) if r % 2 == p] for p in (0, 1)]
        groups = [dist.new_group(ix) for ix in idx]
        pair = dist.new_group([idx[0][0], idx[1][0]])
        T = world * K
        form = direct or "pipeline"
        if form == "direct" and world != 2:
            form = "pipeline"                              # the direct form exists for two ranks only
        eng = GradientPath(layout, K, torch.device("cuda", rank), spec, total_num_decoupled_workers=T,
                           sub_group=groups[rank % 2], pair_group=pair, collective=collective, peer_form=form)
        ref = ReferencePath(layout, K, opt, total_num_decoupled_workers=T, arith="c")
        rng = np.random.default_rng(5)
        w0 = rng.standard_normal(layout.total).astype(np.float32)
        pads = list(zip([0] + [x[1] for x in layout.buckets], [x[0] for x in layout.buckets] + [layout.total]))
        for b, e in pads:
            w0[b:e] = 0
        for k in range(K):
            eng.weights[k].copy_(torch.from_numpy(w0)); ref.weights[k].copy_(torch.from_numpy(w0))
        worst_w = worst_c = 0.0
        graph = collective == "peer"
        for it in range(4):
            rg = np.random.default_rng(1000 * rank + it)
            for k in range(K):
                # mean-shifted so that the sum over ranks never cancels to ~0: with more than two
                # ranks the summation order of an allreduce is not fixed, and Adam's
                # g / (|g| + eps) turns an order-dependent last bit of a near-zero gradient into
                # a visible weight difference (in the reference just as here)
                g = ((rg.standard_normal(layout.total) + 3.0) * 1e-3).astype(np.float32)
                for b, e in pads:
                    g[b:e] = 0
                eng.grads[k].copy_(torch.from_numpy(g)); ref.grads[k].copy_(torch.from_numpy(g))
            if graph and it == 2:
                eng.capture(warmup=1)                      # iteration 2 is the warm-up, 3 is replayed
                cos = float(eng.cos)
            elif graph and it == 3:
                cos = float(eng.replay())
            else:
                cos = float(eng.run_iteration())
            torch.cuda.synchronize()
            cos_ref = ref.run_iteration()
            wr = ref.weights[0]
            for k in range(K):
                w = eng.weights[k].cpu()
                worst_w = max(worst_w, float(((w - wr).abs() / wr.abs().clamp_min(1e-3)).max()))
            worst_c = max(worst_c, abs(cos - cos_ref))
        # every rank must hold the same bits (no drift between data-parallel replicas)
        chk = int(eng.weights[0].view(torch.int32).to(torch.int64).sum())
        sums = [None] * world
        dist.all_gather_object(sums, chk)
        if len(set(sums)) != 1:
            worst_w = float("inf")
        if eng.exchange is not None:
            eng.check_exchange()                           # no bounded wait ever ran out
        q.put((rank, worst_w, worst_c, eng.launches))
        # orderly exit: the captured graph and the peer mappings go before the process group
        dist.barrier()
        torch.cuda.synchronize()
        eng.close()
        del eng
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc(), 0))


@pytest.mark.parametrize("collective,kind,K,direct", [
    ("peer", "sgd", 4, "pipeline"), ("peer", "adamw", 2, "pipeline"), ("peer", "adam", 1, "pipeline"),
    ("peer", "sgd", 4, "direct"), ("peer", "sgd", 3, "direct"), ("peer", "adamw", 1, "direct"),
    ("nccl", "sgd", 2, None)])
def test_engine_exchange_modes_match_reference_path(collective, kind, K, direct):
    """The gradient path at engine level on 2 (or, when visible, 4) GPUs: the peer-memory
    exchange in its forms (``pipeline``: one persistent kernel with flag-ordered aggregate /
    reduce / update pieces; ``direct``, two ranks: the update kernel reads both ranks' sums, T = 6
    included, where dividing before or after the addition differs in the last bit), eager and as a
    replayed CUDA graph, and the NCCL exchange, against the reference path over gloo."""
    world = 2 if torch.cuda.device_count() < 4 else 4
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + hash((collective, kind, K))) % 400
    procs = [ctx.Process(target=_engine_rank, args=(r, world, port, collective, kind, K, q, direct))
             for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, w, c, launches in res:
        assert w != "error", c
        assert w <= 1e-6, (rank, w)
        assert c <= 1e-5, (rank, c)
        assert launches > 0
