"""jabas_b200 — the JABAS/IIDP per-iteration gradient path on B200 (sm_100a).

K-VSW gradient aggregation, comm-hook bucket allreduce, two-half cosine statistic and
fused SGD-momentum / Adam / AdamW update with weight write-back, as hand-written CUDA
behind a C ABI (``include/jabas_b200.h``), with a Python mirror of the reference's
comm-hook, trainer and optimizer interfaces on top.
"""
from . import _lib, ops  # noqa: F401
from ._lib import JabasError  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    # the trainer mirrors import torch.distributed; keep `import jabas_b200` light
    if name in ("JABASTrainer",):
        from .train.trainer import JABASTrainer
        return JABASTrainer
    if name in ("IIDPTrainer",):
        from .iidp.train.trainer import IIDPTrainer
        return IIDPTrainer
    if name in ("ddp_comm_hooks", "iidp", "gradient_path", "layout"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
