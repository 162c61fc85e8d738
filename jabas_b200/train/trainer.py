"""Drop-in for the gradient-path part of ``jabas.train.trainer.JABASTrainer``
(jabas/train/trainer.py:40-98, 171-197, 327-337, 421-483, 693-700): same constructor,
same configuration keys, same hook / state attributes, same ``compute`` / ``step`` flow.

What differs is where the work happens.  The reference materialises the sub-group mean
gradient E of the whole model, ships it between the first ranks of the two parity
sub-groups with ``all_gather`` and reduces it on one rank (jabas/train/trainer.py:470-483).
Here the three sums of the cosine are accumulated by the optimizer-update kernel while it
streams the gradient anyway (``similarity_mode="fused"``, default), or, on request
(``"pair_exchange"``), by one reduction kernel after the reference's own exchange.  On a
single GPU, which the reference rejects (world size must be even, :430), the two halves
are the even-index and the odd-index VSWs.

Everything that only CONSUMES the cosine — batch-size adaptation, configuration solver,
elastic restart — is outside this package; ``step()`` records the decision the reference
would take (``last_decision``) and leaves the reconfiguration to the caller.
"""
from __future__ import annotations

import json
import math
import os
from collections import defaultdict

import torch
import torch.distributed as dist

from .. import ddp_comm_hooks as jabas_hooks
from ..iidp.ddp_comm_hooks import dummy_hook
from ..iidp.train.trainer import IIDPTrainer, _dist_on


class JABASTrainer(IIDPTrainer):
    def __init__(self, gpu, local_batch_size, num_models, accum_step,
                 weight_sync_method="recommend", config_params=None,
                 checkpoint_dir_for_elastic=None, restart_timer_for_elastic=None,
                 similarity_mode="fused"):
        super().__init__(gpu, local_batch_size, num_models, accum_step, weight_sync_method)
        if checkpoint_dir_for_elastic is not None:
            raise NotImplementedError("elastic (checkpoint-restart) training is outside this package")
        self.data_loader = None
        self.is_elastic_training = False
        self._sim_mode = similarity_mode
        self.config_params = config_params
        self._init_config_params()
        self.prev_max_num_models = self.num_models
        self.global_batch_size_trajectory = []
        self.cos_placeholder = None
        self.last_decision = None

    # -- configuration (jabas/train/trainer.py:272-321, jabas/docs/CONFIG.md) ---------------
    def _init_config_params(self):
        cp = self.config_params
        if cp is None:
            raise ValueError("JABAS configuration parameters must be configured")
        if isinstance(cp, (str, os.PathLike)):
            if not os.path.isfile(cp):
                raise ValueError(f"Adaptive config param file: {cp} must exist")
            with open(cp) as f:
                cp = json.load(f)
        cp = defaultdict(lambda: None, cp)
        cp["original_batch_size"] = self.global_batch_size
        if cp["batch_size_lower_bound"] is None:
            cp["batch_size_lower_bound"] = cp["original_batch_size"]
        if cp["batch_size_upper_bound"] is not None:
            assert cp["batch_size_upper_bound"] >= cp["batch_size_lower_bound"]
        cp["global_lr_modifier"] = 1.0
        if cp["enable_adjust"] is None:
            cp["enable_adjust"] = True
        elif isinstance(cp["enable_adjust"], str):
            cp["enable_adjust"] = cp["enable_adjust"] == "True"
        if cp["metric"] is None:
            cp["metric"] = "similarity"
        if cp["batch_size_adjust_rate"] is None:
            cp["batch_size_adjust_rate"] = 0.1
        if cp["batch_size_adjust_interval"] is None:
            cp["batch_size_adjust_interval"] = 100
        else:
            cp["batch_size_adjust_interval"] = int(cp["batch_size_adjust_interval"])
        if cp["similarity_target"] is None:
            cp["similarity_target"] = 0.1
        self.config_params = cp

    def _similarity_enabled(self) -> bool:
        return self.config_params["metric"] == "similarity"

    def _similarity_mode(self) -> str:
        return self._sim_mode

    def _is_similarity_step(self) -> bool:
        st = getattr(self, "similarity_state", None)
        return st is not None and st.step % st.interval == 0

    # -- set-up ----------------------------------------------------------------------------
    def prepare_stream_parallel(self, model, criterion, **kwargs):
        if not kwargs.get("gradient_as_bucket_view"):
            kwargs["gradient_as_bucket_view"] = True
            self.trainer_print("gradient_as_bucket_view must be True")
        super().prepare_stream_parallel(model, criterion, **kwargs)

    def prepare_weight_sync_method(self, optimizer, scheduler=None, param_groups_func=None):
        self._set_local_optimizers(optimizer, param_groups_func)
        self._set_local_schedulers(scheduler)
        self._prepare_gradient_based_metric()
        if self.prepared_for_ddp:
            if self.weight_sync_method == "overlap":
                self._prepare_overlap_optimizer_with_ddp()
            if self.weight_sync_method == "sequential":
                self._register_comm_hook()
        else:
            raise RuntimeError("[ERROR] Without DDP, AdaptiveIIDPTrainer cannot work")

    def prepare_adaptive_data_loader(self, data_loader):
        self.data_loader = data_loader

    def _prepare_gradient_based_metric(self):
        if self.config_params["metric"] == "similarity":
            self._prepare_cosine_similarity()
        else:
            raise ValueError("Not support other gradient-based metric except similarity: "
                             f"{self.config_params['metric']}")

    def _build_subgroup(self):
        world = dist.get_world_size() if _dist_on() else 1
        if world == 1:
            self.sub_groups_idx = [[0], [0]]
            return
        assert world % 2 == 0
        for i in range(world):
            self.sub_groups_idx[i % 2].append(i)

    def _prepare_cosine_similarity(self):
        num_sub_groups = 2            # SimiGrad: two allreduce sub-groups
        self.sub_groups_idx = [[] for _ in range(num_sub_groups)]
        self.sub_groups = []
        self._build_subgroup()
        multi = _dist_on() and dist.get_world_size() > 1
        if multi:
            for idx in self.sub_groups_idx:
                self.sub_groups.append(dist.new_group(idx))
            self.first_subgroup_src_rank = self.sub_groups_idx[0][0]
            self.second_subgroup_src_rank = self.sub_groups_idx[1][0]
            self.sub_groups.append(dist.new_group([self.first_subgroup_src_rank,
                                                   self.second_subgroup_src_rank]))
        else:
            self.sub_groups = [None, None, None]
            self.first_subgroup_src_rank = self.second_subgroup_src_rank = 0
        eng = self.reducer.engine
        eng.sub_group = self.sub_groups[self._rank() % 2]
        eng.pair_group = self.sub_groups[-1]
        eng.src0, eng.src1 = self.first_subgroup_src_rank, self.second_subgroup_src_rank
        self.grad_placeholders = [[] for _ in range(num_sub_groups)]
        self.cos_placeholder = eng.cos
        self._prepare_similarity_allreduce_hooks()

    def _rank(self) -> int:
        return dist.get_rank() if _dist_on() else 0

    def _prepare_similarity_allreduce_hooks(self):
        self.states, self.hooks = [], []
        self.similarity_state = jabas_hooks.GradientSimilarityState(
            None, self.total_num_decoupled_workers, self.sub_groups[self._rank() % 2],
            self.grad_placeholders[self._rank() % 2], self.config_params["batch_size_adjust_interval"])
        main_hook = jabas_hooks.similimarity_allreduce_hook(jabas_hooks.subgroup_allreduce_hook)
        for i in range(self.num_models):
            if i == 0:
                self.states.append(self.similarity_state)
                self.hooks.append(main_hook)
            else:
                self.states.append(None)
                self.hooks.append(dummy_hook)

    # -- per iteration ------------------------------------------------------------------------
    def compute(self, data):
        if self.config_params["enable_adjust"] and self.local_accum_step == -1:
            self._adjust_adaptive_lr()
        super().compute(data)

    def _after_update(self):
        # the statistic of this iteration, while the sub-group sums are still in place
        if self.config_params["metric"] == "similarity" and self._is_similarity_step():
            self._compute_cosine_similarity()

    def step(self):
        if super().step() is False:
            return False
        if self.config_params["enable_adjust"]:
            self._adjust_adaptive_lr(intialize=True)
        sim_step = self.config_params["metric"] == "similarity" and self._is_similarity_step()
        if self.config_params["enable_adjust"] and sim_step:
            self._adjust_adaptive_global_batch_size()
        if self.config_params["metric"] == "similarity":
            self.similarity_state.step += 1
        return True

    def _compute_cosine_similarity(self):
        """Finishes the statistic: a 1-thread fp64 kernel (fused mode), or the reference's
        cat-free pair exchange + one reduction kernel; rank 0's value is broadcast."""
        with self.reducer.stream_scope():
            self.cos_placeholder = self.reducer.engine.finish_similarity()
        self.similarity_state.grad_placeholder.clear()

    def _adjust_adaptive_lr(self, intialize=False):                # jabas/train/trainer.py:693-700
        if self.config_params["metric"] == "similarity":
            mod = self.config_params["global_lr_modifier"]
            for param_group in self.main_optimizer.param_groups:
                if not intialize:
                    param_group["lr"] *= mod
                else:
                    param_group["lr"] /= mod

    def _adjust_adaptive_global_batch_size(self):
        """The SimiGrad rule of jabas/train/trainer.py:702-718, decision only: reading the
        cosine synchronises the host with the GPU, as it does in the reference."""
        cos = float(self.cos_placeholder)
        target, rate = self.config_params["similarity_target"], self.config_params["batch_size_adjust_rate"]
        if cos < target:
            self.last_decision = ("increase", self.global_batch_size * (1 + rate))
        elif cos > target and self.global_batch_size > 1:
            self.last_decision = ("decrease", self.global_batch_size * (1 - rate))
        else:
            self.last_decision = ("keep", self.global_batch_size)
        self.global_batch_size_trajectory.append([self.similarity_state.step, self.global_batch_size])

    def _state_dict_for_ckpt_based_restart(self):                  # jabas/train/trainer.py:747-776
        sd = super()._state_dict_for_ckpt_based_restart()
        sd["total_epoch_cost"] = getattr(self, "total_epoch_cost", 0)
        sd["gbs_trajectory"] = self.global_batch_size_trajectory
        if self.config_params["metric"] == "similarity":
            sd["similarity_step"] = self.similarity_state.step
            sd["global_lr_modifier"] = self.config_params["global_lr_modifier"]
        return sd

    def _load_state_dict_for_ckpt_based_restart(self, state_dict):  # jabas/train/trainer.py:778-799
        super()._load_state_dict_for_ckpt_based_restart(state_dict)
        self.total_epoch_cost = state_dict.get("total_epoch_cost", 0)
        self.global_batch_size_trajectory = state_dict.get("gbs_trajectory", [])
        if self.config_params["metric"] == "similarity" and "similarity_step" in state_dict:
            self.similarity_state.step = state_dict["similarity_step"]
            self.config_params["global_lr_modifier"] = state_dict["global_lr_modifier"]

    def _scale_lr(self, new_global_batch_size):                    # square-root scaling, :676-691
        initial = max(self.config_params["original_batch_size"], self.config_params["batch_size_lower_bound"])
        self.config_params["global_lr_modifier"] = math.sqrt(new_global_batch_size / initial)
