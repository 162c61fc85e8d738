from . import clip_grad  # noqa: F401
