"""Logging from the controller into the workers' logs."""
import logging

logger = logging.getLogger("monarch_b200.worker")


def log(fmt: str, *args) -> None:
    logger.info(fmt, *args)


def set_logging_level(level: int) -> None:
    logging.getLogger().setLevel(level)


def log_remote(fmt: str, *args) -> None:
    """Emit ``fmt % args`` at INFO level on every worker of the active mesh."""
    from ..tensor_engine import remote
    remote("monarch_b200.builtins.log.log", propagate=None)(fmt, *args)


def set_logging_level_remote(level: int) -> None:
    from ..tensor_engine import remote
    remote("monarch_b200.builtins.log.set_logging_level", propagate=None)(level)
