"""Logging helpers with once-only and rank-filtered variants
(parity with rl_engine/utils/logger.py:16-77; stream chosen by ``RL_KERNEL_LOG_STREAM``)."""
from __future__ import annotations

import logging
import os
import sys

_ONCE: set[tuple[str, str]] = set()
_FORMAT = "[%(asctime)s][%(name)s][%(levelname)s] %(message)s"


def init_logger(name: str = "rl_kernel_b200", level: int | str | None = None) -> logging.Logger:
    logger = logging.getLogger(name)
    if not logger.handlers:
        stream = sys.stdout if os.environ.get("RL_KERNEL_LOG_STREAM", "stderr") == "stdout" else sys.stderr
        handler = logging.StreamHandler(stream)
        handler.setFormatter(logging.Formatter(_FORMAT, datefmt="%H:%M:%S"))
        logger.addHandler(handler)
        logger.propagate = False
    lvl = level if level is not None else os.environ.get("RL_KERNEL_LOG_LEVEL", "INFO")
    logger.setLevel(lvl)
    return logger


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


def info_once(logger: logging.Logger, msg: str) -> None:
    key = (logger.name, msg)
    if key not in _ONCE:
        _ONCE.add(key)
        logger.info(msg)


def warn_once(logger: logging.Logger, msg: str) -> None:
    key = (logger.name, "W:" + msg)
    if key not in _ONCE:
        _ONCE.add(key)
        logger.warning(msg)


def info_on_rank(logger: logging.Logger, msg: str, rank: int = 0) -> None:
    if _rank() == rank:
        logger.info(msg)


# the package-wide logger (the reference exposes the same name: ``from rl_engine.utils.logger import logger``)
logger = init_logger("rl_kernel_b200", os.environ.get("RL_KERNEL_LOG_LEVEL", "WARNING"))
