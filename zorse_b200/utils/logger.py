"""Process logger: messages from local rank 0 only unless `leader_only=False`
(reference utils/logger.py:21-34)."""
from __future__ import annotations

import logging
import os
import sys

_logger = None


class LoggerUtility:
    def __init__(self, level: str = "INFO", name: str = "zorse"):
        self.log = logging.getLogger(name)
        if not self.log.handlers:
            h = logging.StreamHandler(sys.stdout)
            h.setFormatter(logging.Formatter("%(asctime)s [%(levelname)s] %(message)s"))
            self.log.addHandler(h)
        self.log.setLevel(getattr(logging, level.upper(), logging.INFO))
        self.log.propagate = False
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    def _emit(self, fn, msg, leader_only):
        if leader_only and self.local_rank != 0:
            return
        fn(msg)

    def debug(self, msg, leader_only=True):
        self._emit(self.log.debug, msg, leader_only)

    def info(self, msg, leader_only=True):
        self._emit(self.log.info, msg, leader_only)

    def warning(self, msg, leader_only=True):
        self._emit(self.log.warning, msg, leader_only)

    def error(self, msg, leader_only=False):
        self._emit(self.log.error, msg, leader_only)


def init_logger(level: str = "INFO") -> LoggerUtility:
    global _logger
    _logger = LoggerUtility(level)
    return _logger


def get_logger() -> LoggerUtility:
    return _logger or init_logger()
