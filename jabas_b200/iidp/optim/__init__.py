"""Mirror of ``iidp.optim``: ``ShardSGD``, ``ShardAdam``, ``ShardAdamW`` — optimizers whose
``step(gradients)`` updates only the parameters of one DDP bucket, so that the update of
bucket b overlaps the allreduce of bucket b+1 (contract visible at
examples/gnmt/seq2seq/train/shard_optimizer.py:30-50 and examples/resnet50/main.py:351-359).

Here every optimizer, sharded or stock (``torch.optim.SGD/Adam/AdamW``), is bound to the
flat HBM storage by ``FusedBinding`` and stepped by ONE fused kernel per bucket (or per
model): gradient, weight and state are read once, the new weights are written to all K
VSW replicas in the same pass.  ``optimizer.param_groups`` stays the source of truth for
``lr`` / ``weight_decay`` (they are re-read at every step), and ``optimizer.state`` holds
views of the flat state buffers, so ``state_dict()`` keeps its per-parameter shape.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

import torch

from ...gradient_path import GradientPath, OptimizerSpec


class FusedBinding:
    """Ties a ``torch.optim.Optimizer`` over the MAIN replica's parameters to a
    ``GradientPath``."""

    def __init__(self, optimizer: torch.optim.Optimizer, engine: GradientPath,
                 main_params: Sequence[torch.nn.Parameter]):
        self.optimizer, self.engine = optimizer, engine
        self.params = list(main_params)
        group_of = {}
        for gi, g in enumerate(optimizer.param_groups):
            for p in g["params"]:
                group_of[id(p)] = gi
        missing = [i for i, p in enumerate(self.params) if id(p) not in group_of]
        if missing:
            raise ValueError(f"{len(missing)} parameters of the main model are not in the optimizer")
        engine.layout.set_groups([group_of[id(p)] for p in self.params])
        for i, p in enumerate(self.params):
            p.index = i                              # the matching key of ShardOptimizer.step
            p._jabas_binding = self
        self.kind = self._kind(optimizer)
        engine.set_optimizer(self._spec())
        self._install_state_views()

    @staticmethod
    def _kind(opt) -> str:
        d = opt.defaults
        if isinstance(opt, torch.optim.AdamW):       # AdamW subclasses Adam in current torch
            kind = "adamw"
        elif isinstance(opt, torch.optim.Adam):
            kind = "adamw" if d.get("decoupled_weight_decay", False) else "adam"
        elif isinstance(opt, torch.optim.SGD):
            kind = "sgd"
        else:
            raise NotImplementedError(f"no fused update for {type(opt).__name__}: use SGD, Adam or AdamW")
        if d.get("amsgrad", False) or d.get("maximize", False):
            raise NotImplementedError("amsgrad / maximize are not supported by the fused update")
        return kind

    def _spec(self) -> OptimizerSpec:
        o, d = self.optimizer, self.optimizer.defaults
        # the kernels take lr and weight decay per group; everything else is per launch
        shared = ("momentum", "dampening", "nesterov") if self.kind == "sgd" else ("betas", "eps")
        for key in shared:
            vals = {repr(g.get(key, d.get(key))) for g in o.param_groups}
            if len(vals) > 1:
                raise NotImplementedError(f"param groups with different {key!r} are not supported by the "
                                          f"fused update (only lr and weight_decay may differ)")
        groups = [dict(lr=float(g["lr"]), weight_decay=float(g.get("weight_decay", 0.0)))
                  for g in o.param_groups]
        if self.kind == "sgd":
            g0 = o.param_groups[0]
            return OptimizerSpec("sgd", groups, momentum=float(g0.get("momentum", 0.0)),
                                 dampening=float(g0.get("dampening", 0.0)),
                                 nesterov=bool(g0.get("nesterov", False)))
        g0 = o.param_groups[0]
        return OptimizerSpec(self.kind, groups, betas=tuple(g0.get("betas", d["betas"])),
                             eps=float(g0.get("eps", d["eps"])))

    def _install_state_views(self) -> None:
        eng, lay = self.engine, self.engine.layout
        for p, slot in zip(self.params, lay.slots):
            sl = slice(slot.offset, slot.offset + slot.numel)
            st = self.optimizer.state[p]
            if self.kind == "sgd":
                if eng.m is not None:
                    st["momentum_buffer"] = eng.m[sl].view(slot.shape)
            else:
                st["step"] = torch.tensor(float(eng.steps))
                st["exp_avg"] = eng.m[sl].view(slot.shape)
                st["exp_avg_sq"] = eng.v[sl].view(slot.shape)

    def sync_hyperparams(self) -> None:
        """Copy the (possibly rescheduled) lr / weight decay of every group to the engine."""
        spec = self.engine.opt
        for g, dst in zip(self.optimizer.param_groups, spec.groups):
            dst["lr"], dst["weight_decay"] = float(g["lr"]), float(g.get("weight_decay", 0.0))

    def request_model_clip(self, max_norm: float) -> torch.Tensor:
        """Whole-model norm clipping for the NEXT whole-model step (sequential mode): the
        reduction runs inside that step, once every bucket's allreduce has been waited for.
        Returns the device scalar that will hold the norm."""
        self.model_clip = float(max_norm)
        return self.engine.clip_coef[self.engine.layout.num_buckets][1]

    def step(self, buckets: Optional[Iterable[int]] = None) -> None:
        self.sync_hyperparams()
        if buckets is None:
            if getattr(self, "model_clip", None) is not None:
                self.engine.clip_grad_norm(None, self.model_clip)
                self.model_clip = None
            self.engine.step_buckets(None)
        else:
            self.engine.step_buckets(buckets)

    def clip(self, buckets: Optional[Iterable[int]], max_norm: float):
        """Norm clipping of the given buckets' gradients (None: one norm over the model)."""
        if buckets is None:
            return self.engine.clip_grad_norm(None, max_norm)
        return [self.engine.clip_grad_norm(b, max_norm) for b in buckets]

    def finish_step(self) -> None:
        """Once per iteration, after every bucket was updated."""
        self.engine.end_iteration()
        if self.kind != "sgd":
            for p in self.params:
                self.optimizer.state[p]["step"] = torch.tensor(float(self.engine.steps))

    def load_state_dict(self, sd: dict, sync_step: Optional[int] = None) -> None:
        """Load a ``torch.optim.Optimizer.state_dict()`` (per-parameter ``momentum_buffer`` /
        ``exp_avg`` / ``exp_avg_sq`` / ``step``, as the reference checkpoints hold it,
        jabas/train/trainer.py:764,783) into the flat state buffers, and the groups'
        hyper-parameters into ``param_groups``."""
        eng, lay = self.engine, self.engine.layout
        id_map = {}
        for sg, cg in zip(sd["param_groups"], self.optimizer.param_groups):
            if len(sg["params"]) != len(cg["params"]):
                raise ValueError("the checkpoint's param groups do not match this optimizer")
            for pid, p in zip(sg["params"], cg["params"]):
                id_map[pid] = p
            for k, v in sg.items():
                if k != "params":
                    cg[k] = v
        adam_step, has_state = None, False
        with torch.no_grad():
            for pid, st in sd["state"].items():
                slot = lay.slots[id_map[pid].index]
                sl = slice(slot.offset, slot.offset + slot.numel)
                if st.get("momentum_buffer") is not None:
                    eng.m[sl].copy_(st["momentum_buffer"].reshape(-1))
                    has_state = True
                if "exp_avg" in st:
                    eng.m[sl].copy_(st["exp_avg"].reshape(-1))
                    eng.v[sl].copy_(st["exp_avg_sq"].reshape(-1))
                    adam_step = int(st["step"])
        if self.kind == "sgd":
            eng.steps = int(sync_step) if sync_step is not None else (1 if has_state else 0)
            if not has_state:
                eng.steps = 0                      # the momentum buffers are created by the next step
        else:
            eng.steps = adam_step or 0
        self._install_state_views()
        self.sync_hyperparams()

    def buckets_of(self, gradients: Sequence[torch.Tensor]) -> List[int]:
        """Buckets covered by a list of gradient tensors carrying ``.index``."""
        lay = self.engine.layout
        idx = sorted(int(g.index) for g in gradients)
        buckets = sorted({lay.slots[i].bucket for i in idx})
        want = sorted(i for b in buckets for i in lay.bucket_indices[b])
        if want != idx:
            raise ValueError("step(gradients) must receive the gradients of whole buckets")
        return buckets


class _ShardMixin:
    """``step(gradients)`` of the overlap mode; ``step()`` updates the whole model."""
    _binding: Optional[FusedBinding] = None

    def bind(self, binding: FusedBinding) -> None:
        self._binding = binding

    @torch.no_grad()
    def step(self, gradients=None, closure=None):
        if self._binding is None:
            raise RuntimeError(f"{type(self).__name__} is not bound to the flat gradient storage: "
                               "pass it to IIDPTrainer.prepare_weight_sync_method first")
        clip = getattr(self, "grad_clip", float("inf"))
        if gradients is None:
            if clip != float("inf"):
                self._binding.request_model_clip(clip)
            self._binding.step(None)
        else:
            buckets = self._binding.buckets_of(gradients)
            if clip != float("inf") and len(gradients) > 0:      # shard_optimizer.py:75-76
                self._binding.clip(buckets, clip)
            self._binding.step(buckets)


class ShardSGD(_ShardMixin, torch.optim.SGD):
    def __init__(self, params, lr=1e-3, momentum=0, dampening=0, weight_decay=0, nesterov=False):
        torch.optim.SGD.__init__(self, params, lr=lr, momentum=momentum, dampening=dampening,
                                 weight_decay=weight_decay, nesterov=nesterov)


class ShardAdam(_ShardMixin, torch.optim.Adam):
    """``grad_clip`` clips the L2 norm of each bucket's gradient before its update, as
    ``ShardGNMTAdam`` does (examples/gnmt/seq2seq/train/shard_optimizer.py:8-29, 75-76)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, amsgrad=False,
                 grad_clip=float("inf")):
        torch.optim.Adam.__init__(self, params, lr=lr, betas=betas, eps=eps,
                                  weight_decay=weight_decay, amsgrad=amsgrad)
        self.grad_clip = grad_clip
        if grad_clip != float("inf") and len(self.param_groups) > 1:
            raise ValueError("Length of self.param_groups must not be > 1 "
                             "because of applying gradient clipping")


class ShardAdamW(_ShardMixin, torch.optim.AdamW):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, amsgrad=False):
        torch.optim.AdamW.__init__(self, params, lr=lr, betas=betas, eps=eps,
                                   weight_decay=weight_decay, amsgrad=amsgrad)


__all__ = ["FusedBinding", "ShardSGD", "ShardAdam", "ShardAdamW"]
