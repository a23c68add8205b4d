"""Logging from the controller into the workers' logs.

Parity: python/monarch/builtins/log.py (``log_remote(*args, level=WARNING)``,
``set_logging_level_remote(level)``)."""
import logging

logger = logging.getLogger("monarch_b200.worker")


def log(*args, level: int = logging.WARNING, **kwargs) -> None:
    logger.log(level, *args, **kwargs)


def set_logging_level(level: int) -> None:
    logger.setLevel(level)
    logging.getLogger().setLevel(level)


def log_remote(*args, level: int = logging.WARNING, **kwargs) -> None:
    """``logger.log(level, *args)`` on every worker of the active mesh."""
    from ..tensor_engine import remote
    remote("monarch_b200.builtins.log.log", propagate=None)(*args, level=level, **kwargs)


def set_logging_level_remote(level: int) -> None:
    from ..tensor_engine import remote
    remote("monarch_b200.builtins.log.set_logging_level", propagate=None)(level)
