"""Rank-aware logging helpers (reference: ``extras/logging.py:34-159``)."""
from __future__ import annotations

import logging
import os
import sys
from functools import lru_cache

_FORMAT = "[%(levelname)s|%(asctime)s] %(name)s:%(lineno)s >> %(message)s"


def _rank() -> int:
    return int(os.environ.get("RANK", os.environ.get("LOCAL_RANK", "0")))


def _level() -> int:
    name = os.environ.get("HMF_VERBOSITY", "INFO").upper()
    return getattr(logging, name, logging.INFO)


def get_logger(name: str = "hmf") -> logging.Logger:
    logger = logging.getLogger(name)
    root = logging.getLogger("hybrid_model_factory_b200")
    if not root.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter(_FORMAT, datefmt="%Y-%m-%d %H:%M:%S"))
        root.addHandler(h)
        root.setLevel(_level())
        root.propagate = False
    return logger


def add_file_handler(path: str) -> None:
    h = logging.FileHandler(path)
    h.setFormatter(logging.Formatter(_FORMAT, datefmt="%Y-%m-%d %H:%M:%S"))
    logging.getLogger("hybrid_model_factory_b200").addHandler(h)


def info_rank0(logger: logging.Logger, msg: str, *args) -> None:
    if _rank() == 0:
        logger.info(msg, *args)


def warning_rank0(logger: logging.Logger, msg: str, *args) -> None:
    if _rank() == 0:
        logger.warning(msg, *args)


@lru_cache(None)
def warning_rank0_once(msg: str) -> None:
    if _rank() == 0:
        get_logger().warning(msg)
