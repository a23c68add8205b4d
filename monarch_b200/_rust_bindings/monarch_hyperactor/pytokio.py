"""Tasks on the native runtime (monarch_hyperactor/src/pytokio.rs:61-295).
"""
from ...actor.pytokio import PythonTask, Shared, is_tokio_thread  # noqa: F401
