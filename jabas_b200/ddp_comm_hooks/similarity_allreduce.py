"""Drop-in for ``jabas.ddp_comm_hooks.similarity_allreduce`` (same names, arguments and
error behaviour as jabas/ddp_comm_hooks/similarity_allreduce.py:8-45), on top of the
fused CUDA kernels.

Per bucket, on a similarity step, the reference does
``clone -> sub-group SUM -> div_(T/2) -> append`` and then the world allreduce averaged
over T.  Here the clone, the K-VSW aggregation and the division by T are one kernel, the
division by T/2 is folded into the update kernel that consumes the sub-group sum (or is
one in-place kernel in ``pair_exchange`` mode), and both collectives stay asynchronous
``torch.distributed`` calls so the comm-hook future protocol is unchanged.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..iidp.ddp_comm_hooks.default_hooks import _allreduce_sum_fut
from ..iidp.ddp_comm_hooks.iidp_allreduce import IIDPState, iidp_allreduce_hook

__all__ = ["GradientSimilarityState", "subgroup_allreduce_hook", "similimarity_allreduce_hook"]


class GradientSimilarityState(IIDPState):
    def __init__(self, process_group, total_num_decoupled_workers, sub_group, grad_placeholder, interval):
        super().__init__(process_group, total_num_decoupled_workers)
        self.sub_group = sub_group
        self.grad_placeholder = grad_placeholder
        assert self.total_num_decoupled_workers % 2 == 0, \
            f"self.total_num_decoupled_workers must be power of 2, but {self.total_num_decoupled_workers}"
        self.subgroup_total_num_decoupled_workers = self.total_num_decoupled_workers / 2
        self.interval = interval
        self.step = 1  # the first step is skipped, as in the reference (bucket rebuild)


def subgroup_allreduce_hook(state: GradientSimilarityState, bucket) -> torch.futures.Future:
    if state.step % state.interval != 0:
        fut = torch.futures.Future()
        fut.set_result(bucket.get_tensors(materialize=False) if hasattr(bucket, "engine")
                       else bucket.get_tensors())
        return fut
    if hasattr(bucket, "engine"):
        # one kernel: local sum of the K VSW buckets -> main bucket / T and undivided copy
        tensor = bucket.aggregate_with_half(state.total_num_decoupled_workers)
        if bucket.deferred:                    # one GPU, or the peer-memory exchange: nothing to send here
            fut = torch.futures.Future()
            fut.set_result([tensor])
            return fut
    else:
        tensor = bucket.get_tensors()[0].detach().clone()
    future_work = _allreduce_sum_fut(state.sub_group, tensor)

    def append_to_grad_placeholder(fut):
        t = fut.value()[0]
        if hasattr(bucket, "engine"):
            state.grad_placeholder.append(bucket.half_entry(t, state.subgroup_total_num_decoupled_workers))
        else:
            state.grad_placeholder.append(t.div_(state.subgroup_total_num_decoupled_workers))
        return [t]

    return future_work.then(append_to_grad_placeholder)


def similimarity_allreduce_hook(hook):
    def hook_with_allreduce(state, bucket):
        future_work = hook(state, bucket)

        def allgroup_allreduce(fut):
            iidp_allreduce_hook(state, bucket).wait()
            return bucket.get_tensors(materialize=False) if hasattr(bucket, "engine") \
                else bucket.get_tensors()
        return future_work.then(allgroup_allreduce)
    return hook_with_allreduce
