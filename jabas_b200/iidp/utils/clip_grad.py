"""Mirror of ``iidp.utils.clip_grad`` (imported at
examples/gnmt/seq2seq/train/shard_optimizer.py:4) and of the ``clip_grad_norm_`` call of the
sequential mode (examples/gnmt/seq2seq/train/trainer.py:157-161).

Both compute the L2 norm with one reduction kernel over the flat averaged gradient and
leave the coefficient on the device; the optimizer-update kernel that follows applies it in
registers.  ``.grad`` itself is not rewritten: it is consumed by that update and zeroed
afterwards, so the scaled copy would never be read.
"""
from __future__ import annotations

from typing import Iterable

import torch


def _binding_of(tensors):
    for t in tensors:
        b = getattr(t, "_jabas_binding", None)
        if b is not None:
            return b
    raise RuntimeError("these tensors are not bound to the flat gradient storage of an IIDPTrainer")


def clip_grad_norm_for_overlap(gradients: Iterable[torch.Tensor], max_norm: float):
    """Per-bucket clipping for the overlap mode: ``gradients`` are the gradient views of
    whole buckets (each carries ``.index``).  Returns the list of per-bucket norms."""
    gradients = list(gradients)
    binding = _binding_of(gradients)
    return binding.clip(binding.buckets_of(gradients), max_norm)


def clip_grad_norm_(parameters: Iterable[torch.nn.Parameter], max_norm: float):
    """Whole-model clipping for the sequential mode; call it between ``compute`` and
    ``step`` on the main model's parameters.  The reduction itself runs inside ``step``,
    after the last bucket's allreduce; the returned device scalar holds the norm from then on."""
    binding = _binding_of(list(parameters))
    return binding.request_model_clip(max_norm)
