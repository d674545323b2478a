"""Package logger (counterpart of vllm/logger.py:66-150): level from ``TW_LOGGING_LEVEL``, one-shot
helpers, and a per-process prefix for worker processes."""
from __future__ import annotations

import logging
import os
import sys
from functools import lru_cache

_FORMAT = "%(levelname)s %(asctime)s [%(name)s:%(lineno)d] %(message)s"
_configured = False
_prefix = ""


def _configure() -> None:
    global _configured
    if _configured:
        return
    root = logging.getLogger("tokenweave_b200")
    handler = logging.StreamHandler(sys.stderr)
    handler.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d %H:%M:%S"))
    root.addHandler(handler)
    root.setLevel(os.getenv("TW_LOGGING_LEVEL", "INFO").upper())
    root.propagate = False
    _configured = True


def init_logger(name: str) -> logging.Logger:
    _configure()
    return logging.getLogger(name if name.startswith("tokenweave_b200") else f"tokenweave_b200.{name}")


def set_process_prefix(prefix: str) -> None:
    """Prefix every log line of this process (workers use ``(Worker_TPn pid=...)``)."""
    global _prefix
    _prefix = prefix
    _configure()
    for h in logging.getLogger("tokenweave_b200").handlers:
        h.setFormatter(logging.Formatter(f"{prefix} {_FORMAT}", datefmt="%m-%d %H:%M:%S"))


@lru_cache(maxsize=None)
def _once(level: int, logger_name: str, msg: str) -> None:
    logging.getLogger(logger_name).log(level, msg)


def info_once(logger: logging.Logger, msg: str) -> None:
    _once(logging.INFO, logger.name, msg)


def warning_once(logger: logging.Logger, msg: str) -> None:
    _once(logging.WARNING, logger.name, msg)
