"""Mirror of ``iidp.ddp_comm_hooks.default_hooks`` — the two helpers the reference
imports from the (absent) IIDP package at
jabas/ddp_comm_hooks/similarity_allreduce.py:4 and jabas/train/trainer.py:461.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _allreduce_sum_fut(process_group, tensor: torch.Tensor) -> torch.futures.Future:
    """Asynchronous SUM allreduce of ``tensor`` in place.  The future's ``value()[0]`` is
    the reduced tensor, the form jabas/ddp_comm_hooks/similarity_allreduce.py:30-33 reads.
    For NCCL the future completes on the stream level: waiting on it never blocks the host."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(process_group) == 1:
        fut = torch.futures.Future()
        fut.set_result([tensor])
        return fut
    return dist.all_reduce(tensor, group=process_group, async_op=True).get_future().then(
        lambda f: [tensor])


def dummy_hook(state, bucket) -> torch.futures.Future:
    """Comm hook of VSWs 1..K-1: no communication (jabas/train/trainer.py:461-468); their
    gradient buckets are consumed by VSW 0's hook through the local aggregation."""
    fut = torch.futures.Future()
    fut.set_result(bucket.get_tensors(materialize=False) if hasattr(bucket, "engine")
                   else bucket.get_tensors())
    return fut
