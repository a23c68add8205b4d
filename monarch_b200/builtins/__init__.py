"""Small remote functions that programs commonly need on the workers.

Parity: python/monarch/builtins/{log,random}.py (``log_remote``, ``set_manual_seed_remote``,
``get_rng_state_remote`` ...): each is a resolvable function path usable with ``remote``."""
from . import log, random  # noqa: F401
