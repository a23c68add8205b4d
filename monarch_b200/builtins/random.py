"""Random-state helpers as remote functions (see :mod:`monarch_b200.random`)."""
from ..random import (_get_state as get_rng_state, _manual_seed as set_manual_seed,  # noqa: F401
                      _set_state as set_rng_state, get_state as get_rng_state_remote,
                      manual_seed as set_manual_seed_remote, set_state as set_rng_state_remote)
