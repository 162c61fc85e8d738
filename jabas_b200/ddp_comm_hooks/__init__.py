from .similarity_allreduce import *  # noqa: F401,F403
