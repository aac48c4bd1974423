"""Architectures: each module registers itself in ``hfee_b200.config.registry``."""
from . import bamipel, dobelix, llama, muvetar, pupinex  # noqa: F401
