"""Mirror of ``iidp.train.trainer.IIDPTrainer`` as far as the gradient path needs it: the
constructor, ``prepare_stream_parallel``, ``prepare_weight_sync_method``, ``compute``,
``step`` and the profiling entry points, with the attribute names the reference reads
(jabas/train/trainer.py:40-43, 82-98, 171-197, 327-337; examples/resnet50/main.py:230-446).

K virtual stream workers (VSWs) are K copies of the model on K CUDA streams of ONE GPU.
Their parameters, gradients and the optimizer state live in flat HBM buffers owned by a
``VSWReducer``; backward fires one comm hook per DDP bucket; the optimizer update writes
the new weights to all K replicas in the same kernel, so there is no separate copy stage.
"""
from __future__ import annotations

import copy
from typing import List, Optional

import torch
import torch.distributed as dist

from ...nn.parallel import IndependentIdenticalDataParallel, VSWReducer
from ..ddp_comm_hooks import IIDPState, dummy_hook, iidp_allreduce_hook
from ..optim import FusedBinding

WEIGHT_SYNC_METHODS = ("recommend", "overlap", "sequential")


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized()


class _ReplicaOptimizer:
    """Stands where the reference keeps one optimizer clone per VSW
    (jabas/train/trainer.py:501-510): the replicas have no optimizer state of their own —
    their weights are written by the main update — so only ``zero_grad`` means anything."""

    def __init__(self, main, reducer: VSWReducer, k: int):
        self._main, self._reducer, self._k = main, reducer, k
        self.param_groups, self.defaults = main.param_groups, main.defaults

    def zero_grad(self, set_to_none: bool = False) -> None:
        self._reducer.engine.grads[self._k].zero_()

    def state_dict(self):
        return self._main.state_dict()

    def load_state_dict(self, sd) -> None:
        pass


class IIDPTrainer(object):
    def __init__(self, gpu, local_batch_size, num_models, accum_step, weight_sync_method="recommend"):
        if weight_sync_method not in WEIGHT_SYNC_METHODS:
            raise ValueError(f"weight_sync_method must be one of {WEIGHT_SYNC_METHODS}")
        self.gpu = gpu
        self.device = torch.device("cuda", gpu) if isinstance(gpu, int) else torch.device(gpu)
        self.local_batch_size = int(local_batch_size)
        self.num_models = self.num_local_models = int(num_models)
        self.accum_step = self.max_accum_step = int(accum_step)
        self.is_accum_mode = self.accum_step > 0
        self.weight_sync_method = "overlap" if weight_sync_method == "recommend" else weight_sync_method
        self.batch_size_per_gpu = self.local_batch_size * self.num_models
        self._get_total_num_decoupled_workers()
        self.global_batch_size = self.local_batch_size * self.total_num_decoupled_workers
        self.local_accum_step = -1
        self.sync_step = 0
        self.epoch = 0
        self.total_epoch_time = 0.0
        self.prepared_for_ddp = False
        self.local_models: List[IndependentIdenticalDataParallel] = []
        self.original_local_models: List[torch.nn.Module] = []
        self.model_streams: List[Optional[torch.cuda.Stream]] = []
        self.local_optimizers, self.local_schedulers = [], []
        self.main_optimizer = self.main_scheduler = None
        self.states, self.hooks = [], []
        self.losses = {}
        self.param_groups_func = None
        self.reducer: Optional[VSWReducer] = None
        self.binding: Optional[FusedBinding] = None
        self._backend = None            # tests on CPU inject an oracle-backed double here
        #: issue the K forward/backward passes from K Python threads (as the reference does,
        #: jabas/train/trainer.py:584-588) instead of one after the other from the calling thread
        self.threaded_compute = False
        self._iter_graph = None         # whole-iteration CUDA graphs, see enable_iteration_graph

    # -- helpers -----------------------------------------------------------------------
    def trainer_print(self, message, status="info"):
        rank = dist.get_rank() if _dist_on() else 0
        if rank == 0:
            print(f"[{status.upper()}] {message}")

    def _get_total_num_decoupled_workers(self):
        """T = sum over ranks of VSWs x (accumulation steps + 1) (jabas/train/trainer.py:152)."""
        mine = self.num_models * (self.accum_step + 1)
        if _dist_on() and dist.get_world_size() > 1:
            gathered = [None] * dist.get_world_size()
            dist.all_gather_object(gathered, mine)
            self.all_partition_size_in_process_group = gathered
            self.total_num_decoupled_workers = int(sum(gathered))
        else:
            self.all_partition_size_in_process_group = [mine]
            self.total_num_decoupled_workers = mine
        return self.total_num_decoupled_workers

    def _similarity_enabled(self) -> bool:
        return False

    def _similarity_mode(self) -> str:
        return "fused"

    def _is_similarity_step(self) -> bool:
        return False

    @property
    def _cuda(self) -> bool:
        return self.device.type == "cuda"

    # -- set-up --------------------------------------------------------------------------
    def prepare_stream_parallel(self, model, criterion, **kwargs):
        """K streams, K model copies, K DDP wrappers over one shared flat storage."""
        kwargs.setdefault("gradient_as_bucket_view", True)
        bucket_cap_mb = kwargs.pop("bucket_cap_mb", 25)
        first_bucket_bytes = kwargs.pop("first_bucket_bytes", None)
        # share_weights=True: the K replicas' parameters are views of ONE flat weight buffer
        # (they are only read between updates), which removes the write-back to K-1 replicas
        share_weights = kwargs.pop("share_weights", False)
        # collective="peer": several GPUs exchange gradients through this library's kernels over
        # NVLink peer memory.  peer_form="pipeline" (default): one pipelined kernel per bucket, fired
        # by the bucket's hook chain during backward ('overlap'), or one over the whole model at step
        # time ('sequential'); peer_form="direct" (two GPUs) runs once per iteration at step time only
        collective = kwargs.pop("collective", "nccl")
        peer_form = kwargs.pop("peer_form", "pipeline")
        if collective == "peer" and peer_form != "pipeline" and self.weight_sync_method != "sequential":
            raise NotImplementedError(f"peer_form={peer_form!r} works on the whole model at step time: "
                                      "use weight_sync_method='sequential'")
        # staging="bulk": the update kernels fetch their tiles by TMA bulk copies (same results)
        staging = kwargs.pop("staging", "register")
        # as in DistributedDataParallel: module buffers follow rank 0's main replica at every forward
        self.broadcast_buffers = kwargs.pop("broadcast_buffers", True)
        self.criterion = criterion
        K = self.num_models
        self.model_streams = [torch.cuda.Stream(self.device) if self._cuda else None for _ in range(K)]
        self.main_stream = self.model_streams[0]
        self.original_local_models = [model] + [copy.deepcopy(model) for _ in range(K - 1)]
        self.reducer = VSWReducer(self.device, K, self.total_num_decoupled_workers, bucket_cap_mb,
                                  similarity=self._similarity_enabled(),
                                  similarity_mode=self._similarity_mode(), backend=self._backend,
                                  first_bucket_bytes=first_bucket_bytes, share_weights=share_weights,
                                  collective=collective, staging=staging, peer_form=peer_form)
        self._sync_buffer_barrier = [None, None]
        self.local_models = [
            IndependentIdenticalDataParallel(
                m, device_ids=[self.gpu], output_device=[self.gpu], model_index=i, num_local_models=K,
                total_num_models=self.total_num_decoupled_workers, reducer=self.reducer, **kwargs)
            for i, m in enumerate(self.original_local_models)]
        self.main_model = self.local_models[0]
        self.eval_model = self.main_model.module
        self.prepared_for_ddp = True
        if self._cuda:
            torch.cuda.current_stream(self.device).synchronize()

    def set_original_local_models(self, models):
        self.original_local_models = list(models)

    def _set_local_optimizers(self, optimizer, param_groups_func=None):
        self.param_groups_func = param_groups_func
        self.main_optimizer = optimizer
        self.binding = FusedBinding(optimizer, self.reducer.engine, self.main_model._params)
        # one GPU: let the update kernel aggregate the VSW gradients itself (one launch per bucket)
        eng = self.reducer.engine
        eng.defer_local = eng.can_fuse_local() or eng.collective == "peer"
        if hasattr(optimizer, "bind"):
            optimizer.bind(self.binding)
        self.local_optimizers = [optimizer] + [_ReplicaOptimizer(optimizer, self.reducer, k)
                                               for k in range(1, self.num_models)]

    def _set_local_schedulers(self, scheduler=None):
        self.main_scheduler = scheduler
        self.local_schedulers = [scheduler] + [None] * (self.num_models - 1)

    def _prepare_hooks(self):
        self.states = [IIDPState(None, self.total_num_decoupled_workers)] + [None] * (self.num_models - 1)
        self.hooks = [iidp_allreduce_hook] + [dummy_hook] * (self.num_models - 1)

    def prepare_weight_sync_method(self, optimizer, scheduler=None, param_groups_func=None):
        self._set_local_optimizers(optimizer, param_groups_func)
        self._set_local_schedulers(scheduler)
        self._prepare_hooks()
        if not self.prepared_for_ddp:
            raise RuntimeError("prepare_stream_parallel() must be called first")
        if self.weight_sync_method == "overlap":
            self._prepare_overlap_optimizer_with_ddp()
        else:
            self._register_comm_hook()

    def _create_stream_for_optimizer(self):
        self.optimizer_stream = self.reducer.path_stream

    def _check_overlap_with_ddp(self):
        if not hasattr(self.main_optimizer, "bind"):
            raise ValueError("weight_sync_method='overlap' needs a Shard optimizer (ShardSGD, ShardAdam, "
                             "ShardAdamW); use 'sequential' with a stock torch.optim optimizer")

    def _create_optimizer_hook(self, hook):
        """Chain the sharded optimizer step of a bucket behind its comm hook: the update of
        bucket b is enqueued as soon as its allreduce is, and overlaps the rest of backward."""
        def hook_with_optimizer_step(state, bucket):
            fut = hook(state, bucket)

            def optimizer_step(f):
                grads = bucket.gradients()
                for g, i in zip(grads, self.reducer.layout.bucket_indices[bucket.index()]):
                    g.index = i
                    g._jabas_binding = self.binding
                with self.reducer.stream_scope():
                    self.main_optimizer.step(grads)
                return f.value()
            return fut.then(optimizer_step)
        return hook_with_optimizer_step

    def _prepare_overlap_optimizer_with_ddp(self):                 # jabas/train/trainer.py:327-333
        self._create_stream_for_optimizer()
        self._check_overlap_with_ddp()
        for i, (local_model, state, hook) in enumerate(zip(self.local_models, self.states, self.hooks)):
            if i == 0:
                hook = self._create_optimizer_hook(hook)
            local_model.register_comm_hook(state=state, hook=hook)

    def _register_comm_hook(self):                                 # jabas/train/trainer.py:335-337
        for local_model, state, hook in zip(self.local_models, self.states, self.hooks):
            local_model.register_comm_hook(state=state, hook=hook)

    # -- run-time reconfiguration (jabas/train/trainer.py:485-600) ----------------------------
    def _change_local_trainer_state(self, new_num_models, new_accum_step):
        """Deltas, as in the reference: ``new_num_models`` VSWs and ``new_accum_step``
        accumulation steps are ADDED to the current values."""
        self.prev_num_models = self.num_models
        if new_num_models != 0:
            self.num_models = self.prev_num_models + new_num_models
            assert self.num_models > 0, "self.num_models must be > 0"
            self.num_local_models = self.num_models
        if new_accum_step != 0:
            self.accum_step = self.accum_step + new_accum_step
            self.is_accum_mode = self.accum_step > 0
        self.batch_size_per_gpu = self.local_batch_size * self.num_models
        if getattr(self, "data_loader", None) is not None and hasattr(self.data_loader, "update_local_state"):
            self.data_loader.update_local_state(self.batch_size_per_gpu, self.num_models, self.accum_step)

    def _change_global_trainer_state(self, solved_iidp_config_map=None):
        self._get_total_num_decoupled_workers()
        self.global_batch_size = self.local_batch_size * self.total_num_decoupled_workers

    def _change_local_models_state(self, adjust_num_models_diff):
        """Add or remove VSWs between two iterations.  The flat buffers of the VSWs that
        stay are not reallocated; new replicas get their weights from the main replica by
        one kernel; T reaches the hook states and the kernels' divisors."""
        K_old, K_new = self.prev_num_models, self.num_models
        assert K_new == K_old + adjust_num_models_diff
        if self._cuda:
            torch.cuda.current_stream(self.device).synchronize()
        self._drop_iteration_graphs()            # captured for the old set of VSWs
        T = self.total_num_decoupled_workers
        self.reducer.resize(K_new, T)
        if adjust_num_models_diff > 0:
            for idx in range(K_old, K_new):
                self.model_streams.append(torch.cuda.Stream(self.device) if self._cuda else None)
                copied = copy.deepcopy(self.main_model.module)
                self.original_local_models.append(copied)
                wrapper = IndependentIdenticalDataParallel(
                    copied, device_ids=[self.gpu], output_device=[self.gpu], model_index=idx,
                    num_local_models=K_new, total_num_models=T, reducer=self.reducer,
                    find_unused_parameters=self.main_model.find_unused_parameters)
                wrapper.train(self.main_model.training)
                self.local_models.append(wrapper)
                self.local_optimizers.append(_ReplicaOptimizer(self.main_optimizer, self.reducer, idx))
                self.local_schedulers.append(None)
                self.states.append(None)
                self.hooks.append(dummy_hook)
                wrapper.register_comm_hook(state=None, hook=dummy_hook)
        else:
            for _ in range(K_new, K_old):
                for lst in (self.local_models, self.original_local_models, self.local_optimizers,
                            self.local_schedulers, self.model_streams, self.states, self.hooks):
                    del lst[-1]
        assert len(self.local_models) == self.num_models == len(self.local_optimizers)
        for m in self.local_models:
            m.reconfigure(self.num_models, T, self._sync_buffer_barrier)
        if self.states and self.states[0] is not None:
            self.states[0].total_num_decoupled_workers = T
            if hasattr(self.states[0], "subgroup_total_num_decoupled_workers"):
                assert T % 2 == 0
                self.states[0].subgroup_total_num_decoupled_workers = T / 2

    def change_num_models(self, new_num_models: int, new_accum_step=None):
        """Convenience over the three reference-named steps: set K (and optionally the
        accumulation steps) on THIS rank, re-derive T over all ranks, rebuild local state.
        Collective: every rank must call it (T is all-gathered)."""
        d_models = int(new_num_models) - self.num_models
        d_accum = 0 if new_accum_step is None else int(new_accum_step) - self.accum_step
        self._change_local_trainer_state(d_models, d_accum)
        self._change_global_trainer_state()
        self._change_local_models_state(d_models)

    # -- per iteration ---------------------------------------------------------------------
    def set_model_train(self):
        for m in self.local_models:
            m.train()

    def is_sync_step(self) -> bool:
        return self.local_accum_step == self.accum_step

    def compute(self, data):
        inputs, targets = data[0], data[1]
        if self._iter_graph is not None:
            return self._graphed_compute(inputs, targets)
        K = self.num_models
        self.parallel_compute(torch.chunk(inputs, K), torch.chunk(targets, K))

    # -- one CUDA-graph launch per iteration ---------------------------------------------
    def enable_iteration_graph(self, warmup: int = 3) -> None:
        """From now on a synchronising iteration (``compute`` then ``step``) is ONE CUDA-graph
        launch: the K VSWs' forward and backward passes on their K streams, every launch the comm
        hooks make from backward (aggregation, exchange or collectives, fused update, statistic)
        and the zeroing of the gradients.  ``compute`` copies the batch into static input
        buffers and replays the graph; ``step`` keeps the host-side bookkeeping.  What changes
        between iterations (lr, weight decay, Adam step, first-step flag) is read by the kernels
        from a device block refreshed before each replay.

        The first ``warmup`` iterations of each kind (with and without the statistic) run eagerly
        on the capture stream (they bring up cuDNN / cuBLAS work spaces, the per-stream reduction
        work spaces and the communicators); that kind's graph is captured at its next iteration.  Needs
        ``accum_step == 0``, a fixed batch shape and the single-threaded issue order; a change of
        the VSW count drops the graphs, which are then captured again."""
        if not self._cuda:
            raise RuntimeError("iteration graphs need a CUDA device")
        if self.binding is None:
            raise RuntimeError("prepare_weight_sync_method() must be called first")
        eng = self.reducer.engine
        own_block = eng._dyn is None
        if own_block:
            eng._dyn = eng.ops.DynHp(eng.ctx)
        self._iter_graph = dict(own_block=own_block, warmup=max(1, int(warmup)), seen={}, stream=torch.cuda.Stream(self.device),
                                graphs={}, launches={}, losses={}, static=None, pool=None, replayed=False)

    def disable_iteration_graph(self) -> None:
        """Back to eager iterations: the graphs go, and the kernels take their hyper-parameters
        from the launch arguments again."""
        G = self._iter_graph
        if G is None:
            return
        torch.cuda.synchronize(self.device)
        self._iter_graph = None
        eng = self.reducer.engine
        if G["own_block"] and eng._dyn is not None and getattr(eng, "_graph", None) is None:
            eng._dyn.close()
            eng._dyn = None

    def _drop_iteration_graphs(self) -> None:
        G = self._iter_graph
        if G is not None:
            torch.cuda.synchronize(self.device)
            G.update(graphs={}, launches={}, losses={}, static=None, pool=None, seen={}, replayed=False)

    def _graphed_compute(self, inputs, targets):
        G, K, eng = self._iter_graph, self.num_models, self.reducer.engine
        if self.accum_step != 0 or self.threaded_compute:
            raise RuntimeError("iteration graphs need accum_step == 0 and threaded_compute == False")
        if G["static"] is None:
            G["static"] = (torch.empty(inputs.shape, dtype=inputs.dtype, device=self.device),
                           torch.empty(targets.shape, dtype=targets.dtype, device=self.device))
        xin, tin = G["static"]
        if inputs.shape != xin.shape or targets.shape != tin.shape:
            raise ValueError(f"the iteration graph takes batches of shape {tuple(xin.shape)} / {tuple(tin.shape)}, "
                             f"got {tuple(inputs.shape)} / {tuple(targets.shape)}")
        sim = bool(self._is_similarity_step())
        cur, s = torch.cuda.current_stream(self.device), G["stream"]
        s.wait_stream(cur)
        with torch.cuda.stream(s):
            xin.copy_(inputs, non_blocking=True)
            tin.copy_(targets, non_blocking=True)
            self.binding.sync_hyperparams()
            if G["seen"].get(sim, 0) < G["warmup"]:    # each kind of iteration warms up before its capture
                G["seen"][sim] = G["seen"].get(sim, 0) + 1
                eng.push_hyperparams()
                self.parallel_compute(torch.chunk(xin, K), torch.chunk(tin, K))
                cur.wait_stream(s)
                return
            if sim not in G["graphs"]:
                self._capture_iteration(sim)
            self.local_accum_step += 1
            eng.push_hyperparams()
            G["graphs"][sim].replay()
        cur.wait_stream(s)
        eng._sim_step = sim and eng.similarity
        eng.launches += G["launches"][sim]
        self.losses = dict(G["losses"][sim])
        G["replayed"] = True

    def _capture_iteration(self, sim: bool) -> None:
        """Capture ``parallel_compute`` + the device part of ``step`` on the capture stream (the
        caller has made it current).  Nothing runs and no host counter moves: the replay that
        follows is the iteration."""
        G, K, eng = self._iter_graph, self.num_models, self.reducer.engine
        xin, tin = G["static"]
        graph = torch.cuda.CUDAGraph()
        keep = (self.local_accum_step, eng.launches)
        with torch.cuda.graph(graph, pool=G["pool"], stream=G["stream"]):
            self.parallel_compute(torch.chunk(xin, K), torch.chunk(tin, K))
            self._step_device()
        if G["pool"] is None:
            G["pool"] = graph.pool()
        G["graphs"][sim] = graph
        G["launches"][sim] = eng.launches - keep[1]
        G["losses"][sim] = dict(self.losses)
        self.local_accum_step, eng.launches = keep

    def parallel_compute(self, scatter_inputs, scatter_targets, accum_step=0):
        """Forward + backward of the K VSWs, each on its own stream.  On the synchronising
        micro-step the comm hooks fire bucket by bucket during the backward passes."""
        self.local_accum_step += 1
        sync = self.is_sync_step()
        self.reducer.require_sync = sync
        if self.binding is not None:
            self.binding.sync_hyperparams()
        if sync:
            self.reducer.prepare_for_backward(self._is_similarity_step())
        if getattr(self, "broadcast_buffers", True) and self.local_accum_step == 0:
            self.reducer.sync_buffers()              # before the K streams fork off the current one
        cur = torch.cuda.current_stream(self.device) if self._cuda else None

        def run(k):
            if self._cuda:
                torch.cuda.set_device(self.device)
                with torch.cuda.stream(self.model_streams[k]):
                    self._forward_backward(k, scatter_inputs[k], scatter_targets[k])
            else:
                self._forward_backward(k, scatter_inputs[k], scatter_targets[k])

        for k in range(self.num_models):
            self.reducer.install_grad_views(k)
            if self._cuda:
                self.model_streams[k].wait_stream(cur)
        if self.threaded_compute and self.num_models > 1:
            import threading
            errors = []

            def guarded(k):
                try:
                    run(k)
                except BaseException as e:     # re-raised in the calling thread
                    errors.append(e)
            threads = [threading.Thread(target=guarded, args=(k,)) for k in range(self.num_models)]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
            if errors:
                raise errors[0]
        else:
            for k in range(self.num_models):
                run(k)

    def _forward_backward(self, k, inputs, targets):
        out = self.local_models[k](inputs)
        loss = self.criterion(out, targets)
        self.losses[k] = loss
        loss.backward()
        self.reducer.finish_backward(k, self.local_models[k].find_unused_parameters)

    def step(self) -> bool:
        if not self.is_sync_step():
            return False
        G = self._iter_graph
        if G is not None and G["replayed"]:
            G["replayed"] = False                # the graph launched by compute() held the device part
        elif G is not None:
            cur, s = torch.cuda.current_stream(self.device), G["stream"]
            s.wait_stream(cur)
            with torch.cuda.stream(s):           # warm-up iterations run where the capture will
                self._step_device()
            cur.wait_stream(s)
        else:
            self._step_device()
        self.binding.finish_step()
        self.local_accum_step = -1
        self.sync_step += 1
        return True

    def _step_device(self) -> None:
        """Everything of ``step`` that is work on the GPU: join the K streams, wait for the hook
        chains, the whole-model update of the sequential mode, the statistic, zeroed gradients."""
        if self._cuda:
            cur = torch.cuda.current_stream(self.device)
            for s in self.model_streams:
                cur.wait_stream(s)
        self.reducer.wait()
        if self.weight_sync_method == "sequential":
            with self.reducer.stream_scope():
                self.binding.step(None)          # one fused launch over the whole flat model
        self._after_update()
        self.reducer.engine.zero_grads()

    def _after_update(self):
        """Hook for subclasses: runs after the update is enqueued, before gradients are zeroed."""

    def scheduler_step(self):
        if self.main_scheduler is not None:
            self.main_scheduler.step()

    def remaining_epochs(self, final_epochs):
        while self.epoch < final_epochs:
            yield self.epoch
            self.epoch += 1

    # -- checkpoints (keys of jabas/train/trainer.py:747-799) -----------------------------------
    CHECKPOINT_FILE_NAME = "checkpoint.pth"

    def _state_dict_for_ckpt_based_restart(self):
        sched = self.main_scheduler.state_dict() if self.main_scheduler is not None else None
        sd = {"epoch": self.epoch, "total_epoch_time": self.total_epoch_time, "step": self.sync_step,
              "model": self.main_model.module.state_dict(), "optimizer": self.main_optimizer.state_dict(),
              "scheduler": sched}
        loader = getattr(self, "data_loader", None)
        if loader is not None and hasattr(loader, "state_dict"):
            sd["data"] = loader.state_dict()
        return sd

    def _load_state_dict_for_ckpt_based_restart(self, state_dict):
        if self._cuda:
            torch.cuda.current_stream(self.device).synchronize()
        for local_model in self.local_models:              # in place: the parameters stay views of the flat buffers
            local_model.module.load_state_dict(state_dict["model"])
        self.binding.load_state_dict(state_dict["optimizer"], sync_step=state_dict.get("step"))
        if self.main_scheduler is not None and state_dict.get("scheduler") is not None:
            self.main_scheduler.load_state_dict(state_dict["scheduler"])
        loader = getattr(self, "data_loader", None)
        if loader is not None and "data" in state_dict and hasattr(loader, "load_state_dict"):
            loader.load_state_dict(state_dict["data"])
        self.epoch = state_dict["epoch"]
        self.total_epoch_time = state_dict["total_epoch_time"]
        self.sync_step = state_dict["step"]

    def _checkpoint_file(self, checkpoint_path, create=False):
        import os
        if os.path.isdir(checkpoint_path) or not os.path.splitext(checkpoint_path)[1]:
            if create:
                os.makedirs(checkpoint_path, exist_ok=True)
            return os.path.join(checkpoint_path, self.CHECKPOINT_FILE_NAME)
        return checkpoint_path

    def save(self, checkpoint_path):
        sd = self._state_dict_for_ckpt_based_restart()
        sd["global_batch_size"], sd["local_batch_size"] = self.global_batch_size, self.local_batch_size
        path = self._checkpoint_file(checkpoint_path, create=True)
        torch.save(sd, path)
        return path

    def load(self, checkpoint_path, restrict_saved_config=False):
        import os
        if not os.path.exists(checkpoint_path):
            raise FileExistsError(f"Checkpoint path: {checkpoint_path} does not exist")
        sd = torch.load(self._checkpoint_file(checkpoint_path), map_location=self.device, weights_only=False)
        self._load_state_dict_for_ckpt_based_restart(sd)
        if restrict_saved_config:
            assert self.global_batch_size == sd["global_batch_size"], \
                f"self.global_batch_size: {self.global_batch_size} | state_dict['global_batch_size']: {sd['global_batch_size']}"
            assert self.local_batch_size == sd["local_batch_size"]

    # -- profiling entry points (examples/resnet50/profiler/comp/comp_profiler.py:61-62) ------
    def profile_parallel_compute(self, scatter_inputs, scatter_targets):
        """(forward+backward ms, 0.0): the two phases are not separated here."""
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        self.parallel_compute(scatter_inputs, scatter_targets)
        for s in self.model_streams:
            torch.cuda.current_stream(self.device).wait_stream(s)
        z.record()
        z.synchronize()
        return a.elapsed_time(z), 0.0

    def profile_step(self):
        """(update ms, copy ms).  The weight copy is part of the update kernel: copy is 0."""
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        self.step()
        z.record()
        z.synchronize()
        return a.elapsed_time(z), 0.0
