"""Device-side timers: CUDA-event timing with running statistics.

Parity: python/monarch/timer/execution_timer.py (``ExecutionTimer``: named timers as
context managers, start/stop, ``summary`` with mean/std/min/max, ``reset``) and
example_monarch.py's remote use.  On a machine without CUDA the timers fall back to
``time.perf_counter`` so host-side code keeps working."""
from .execution_timer import CudaTimer, ExecutionTimer, execution_timer_start, \
    execution_timer_stop, get_execution_timer_average_ms, get_latest_timer_measurement

__all__ = ["CudaTimer", "ExecutionTimer", "execution_timer_start", "execution_timer_stop",
           "get_execution_timer_average_ms", "get_latest_timer_measurement"]
