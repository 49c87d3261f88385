"""Rank-aware logging (loguru when present, stdlib logging otherwise).

Messages from ranks other than 0 are dropped unless ``rank0_only=False``. Parity target:
cosmos_predict2/_src/imaginaire/utils/log.py:56-162.
"""

from __future__ import annotations

import logging
import os
import sys

try:
    from loguru import logger as _logger
    _HAVE_LOGURU = True
except Exception:  # pragma: no cover
    _logger = logging.getLogger("cosmos_b200")
    _HAVE_LOGURU = False

_LEVEL = os.environ.get("COSMOS_B200_LOG", "INFO")


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


def init_loguru_stdout():
    if _HAVE_LOGURU:
        _logger.remove()
        _logger.add(sys.stdout, level=_LEVEL, format="[{time:MM-DD HH:mm:ss}|{level}|rank" + str(_rank()) + "] {message}")
    else:
        logging.basicConfig(level=getattr(logging, _LEVEL, logging.INFO))


def init_loguru_file(path: str):
    if _HAVE_LOGURU:
        _logger.add(path, level=_LEVEL, encoding="utf8")
    else:
        _logger.addHandler(logging.FileHandler(path))


def _emit(fn, msg, rank0_only):
    if rank0_only and _rank() != 0:
        return
    fn(msg)


def info(msg, rank0_only: bool = True): _emit(_logger.info, msg, rank0_only)
def debug(msg, rank0_only: bool = True): _emit(_logger.debug, msg, rank0_only)
def warning(msg, rank0_only: bool = True): _emit(_logger.warning, msg, rank0_only)
def error(msg, rank0_only: bool = False): _emit(_logger.error, msg, rank0_only)
def critical(msg, rank0_only: bool = False): _emit(_logger.critical, msg, rank0_only)
def success(msg, rank0_only: bool = True): _emit(getattr(_logger, "success", _logger.info), msg, rank0_only)


init_loguru_stdout()
