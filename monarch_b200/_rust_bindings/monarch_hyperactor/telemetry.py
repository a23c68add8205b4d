"""Telemetry (monarch_hyperactor/src/telemetry.rs; hyperactor_telemetry).
"""
from ...telemetry import Counter as PyCounter  # noqa: F401
from ...telemetry import Histogram as PyHistogram  # noqa: F401
from ...telemetry import Span as PySpan  # noqa: F401
from ...telemetry import SqliteTracing as PySqliteTracing  # noqa: F401
from ...telemetry import UpDownCounter as PyUpDownCounter  # noqa: F401
from ...telemetry import (forward_to_tracing, get_current_span_id, get_execution_id,  # noqa: F401
                          use_real_clock, use_sim_clock)
