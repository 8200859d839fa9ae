"""Logging helpers (reference: vllm/logger.py): ``init_logger`` with ``info_once``/``warning_once``."""
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
    _configured = True
    root = logging.getLogger("onecat_vllm")
    root.setLevel(os.environ.get("ONECAT_LOGGING_LEVEL", "INFO").upper())
    if not root.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d %H:%M:%S"))
        root.addHandler(h)
    root.propagate = False


class _Logger(logging.LoggerAdapter):
    def process(self, msg, kwargs):
        return (_prefix + msg if _prefix else msg), kwargs

    @lru_cache(maxsize=None)
    def _once(self, level: int, msg: str) -> None:
        self.log(level, msg)

    def info_once(self, msg: str) -> None:
        self._once(logging.INFO, msg)

    def warning_once(self, msg: str) -> None:
        self._once(logging.WARNING, msg)


def init_logger(name: str) -> _Logger:
    _configure()
    return _Logger(logging.getLogger(name if name.startswith("onecat_vllm") else "onecat_vllm." + name), {})


def decorate_logs(process_name: str) -> None:
    """Prefix every record of this process, e.g. ``(Worker_TP1) `` (reference: vllm/utils/system_utils.py decorate_logs)."""
    global _prefix
    _prefix = f"({process_name} pid={os.getpid()}) "
