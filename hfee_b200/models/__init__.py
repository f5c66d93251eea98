"""Architectures: each module registers itself in ``hfee_b200.config.registry``."""
from . import dobelix, llama  # noqa: F401
