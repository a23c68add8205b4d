"""Simulated time (monarch_extension/src/simulation_tools.rs).
"""
from ..._native import sim_clock_advance_us, use_real_clock, use_sim_clock

_active = False


def start_event_loop() -> None:
    global _active
    use_sim_clock()
    _active = True


def is_simulator_active() -> bool:
    return _active


def sleep(seconds: float) -> None:
    """Advance simulated time (no wall-clock wait)."""
    sim_clock_advance_us(int(seconds * 1e6))


def stop() -> None:
    global _active
    use_real_clock()
    _active = False
