"""Runtime helpers (monarch_hyperactor/src/runtime.rs:36-155).
"""
import time


def sleep_indefinitely_for_unit_tests() -> None:
    """Block the calling thread until the process is killed (signals still arrive)."""
    while True:
        time.sleep(3600)
