from .default_hooks import _allreduce_sum_fut, dummy_hook  # noqa: F401
from .iidp_allreduce import IIDPState, iidp_allreduce_hook  # noqa: F401
