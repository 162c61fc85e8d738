"""Mirror of the parts of the ``iidp`` package (an absent git submodule of the reference)
that the gradient path of JABAS reaches: comm hooks, sharded optimizers, ``IIDPTrainer``."""
from . import ddp_comm_hooks, optim, utils  # noqa: F401
from .train.trainer import IIDPTrainer  # noqa: F401
