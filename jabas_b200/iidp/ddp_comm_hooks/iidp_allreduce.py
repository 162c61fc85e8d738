"""Mirror of ``iidp.ddp_comm_hooks.iidp_allreduce``: ``IIDPState`` and
``iidp_allreduce_hook``, imported by the reference at
jabas/ddp_comm_hooks/similarity_allreduce.py:5 and used at :42.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .default_hooks import _allreduce_sum_fut


class IIDPState(object):
    """Process group plus T, the number of decoupled workers over all ranks
    (sum over ranks of VSWs x (accumulation steps + 1), jabas/train/trainer.py:152)."""

    def __init__(self, process_group, total_num_decoupled_workers):
        self.process_group = process_group
        self.total_num_decoupled_workers = total_num_decoupled_workers


def iidp_allreduce_hook(state: IIDPState, bucket) -> torch.futures.Future:
    """World allreduce of a bucket averaged over T.

    The bucket handed over by ``IndependentIdenticalDataParallel`` aggregates lazily: if
    no earlier hook of the chain has produced the local sum yet, this call launches the
    K-VSW aggregation kernel with the division by T fused in; if the bucket already holds
    the plain sum it is divided in place.  A foreign bucket (stock ``dist.GradBucket``) is
    divided and reduced with stock ops — those are collectives' plumbing, not a fallback
    of the kernels: such a bucket has no VSWs to aggregate."""
    if hasattr(bucket, "engine"):
        bucket.ensure_averaged(state.total_num_decoupled_workers)
        tensor = bucket.buffer(materialize=False)
        if bucket.deferred:                    # aggregation and exchange happen in the optimizer step
            fut = torch.futures.Future()
            fut.set_result([tensor])
            return fut
    else:
        tensor = bucket.buffer() if hasattr(bucket, "buffer") else bucket.get_tensors()[0]
        tensor.div_(state.total_num_decoupled_workers)
    return _allreduce_sum_fut(state.process_group, tensor)
