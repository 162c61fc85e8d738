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


def _rank_main(rank, world, port, mode, kind, wsm, q):
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
                                   first_bucket_bytes=4096)
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
        for it in range(3):
            x = torch.randn(8 * K, 3, 16, 16, generator=g).cuda()
            y = torch.randint(0, 10, (8 * K,), generator=g).cuda()
            tr.compute((x, y))
            tr.step()
            torch.cuda.synchronize()
            for (k, b), t in captured.items():
                ref.grads[k][lay.buckets[b][0]:lay.buckets[b][1]].copy_(t.cpu())
            captured.clear()
            cos_ref = ref.run_iteration()
            wr = ref.weights[0]
            w = tr.reducer.engine.weights[K - 1].cpu()
            worst_w = max(worst_w, float(((w - wr).abs() / wr.abs().clamp_min(1e-3)).max()))
            worst_c = max(worst_c, abs(float(tr.cos_placeholder) - cos_ref))
        q.put((rank, worst_w, worst_c, tr.reducer.engine.launches))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc(), 0))


@pytest.mark.parametrize("mode,kind,wsm", [("fused", "sgd", "overlap"), ("pair_exchange", "sgd", "sequential"),
                                           ("fused", "adamw", "overlap"), ("fused", "adamw", "sequential")])
def test_two_nccl_ranks_match_reference_path(mode, kind, wsm):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + hash((mode, kind, wsm))) % 400
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, mode, kind, wsm, q)) for r in range(2)]
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
