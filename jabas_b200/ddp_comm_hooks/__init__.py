"""Comm hooks of the adaptive-batching statistic, under the names the reference exports from
``jabas.ddp_comm_hooks`` (used at jabas/train/trainer.py:452-460)."""
from .similarity_allreduce import (GradientSimilarityState, similimarity_allreduce_hook,
                                   subgroup_allreduce_hook)

__all__ = ["GradientSimilarityState", "subgroup_allreduce_hook", "similimarity_allreduce_hook"]
