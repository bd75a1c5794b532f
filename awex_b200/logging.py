"""Process-local stdout logger.

Output line format (same as the reference's `awex/logging.py:39-52`):
``<timestamp>\\t<LEVEL> <file>:<line> -- <pid> -- <message>``.  The logger does
not go through the stdlib ``logging`` tree, so inference engines that
reconfigure stdlib logging cannot silence or duplicate weight-exchange lines.

A default level can be set with the environment variable ``AWEX_LOG_LEVEL``.
"""

from __future__ import annotations

import os
import sys
import time
import traceback
from enum import IntEnum


class LogLevel(IntEnum):
    """The levels as an enumeration (`awex/logging.py:25-30`); the module
    constants below are the same numbers."""

    DEBUG = 10
    INFO = 20
    WARNING = 30
    ERROR = 40
    CRITICAL = 50


DEBUG, INFO, WARNING, ERROR, CRITICAL = (int(level) for level in LogLevel)
_NAMES = {DEBUG: "DEBUG", INFO: "INFO", WARNING: "WARNING", ERROR: "ERROR", CRITICAL: "CRITICAL"}
_BY_NAME = {v: k for k, v in _NAMES.items()}
_BY_NAME["WARN"] = WARNING


def _coerce_level(level) -> int:
    if isinstance(level, str):
        return _BY_NAME.get(level.upper(), INFO)
    return int(level)


_registry: dict = {}
_default_level = _coerce_level(os.environ.get("AWEX_LOG_LEVEL", "INFO"))


class Logger:
    __slots__ = ("name", "level")

    def __init__(self, name: str, level: int):
        self.name = name
        self.level = level

    def isEnabledFor(self, level: int) -> bool:
        return level >= self.level

    def _emit(self, level: int, msg, args) -> None:
        if level < self.level:
            return
        if args:
            try:
                msg = msg % args
            except (TypeError, ValueError):
                msg = f"{msg} {args}"
        frame = sys._getframe(2)
        now = time.time()
        stamp = time.strftime("%Y-%m-%d %H:%M:%S", time.localtime(now)) + f".{int(now * 1000) % 1000:03d}"
        fname = os.path.basename(frame.f_code.co_filename)
        sys.stdout.write(f"{stamp}\t{_NAMES.get(level, level)} {fname}:{frame.f_lineno} -- {os.getpid()} -- {msg}\n")
        sys.stdout.flush()

    def debug(self, msg, *args, **_kw):
        self._emit(DEBUG, msg, args)

    def info(self, msg, *args, **_kw):
        self._emit(INFO, msg, args)

    def warning(self, msg, *args, **_kw):
        self._emit(WARNING, msg, args)

    warn = warning

    def error(self, msg, *args, **_kw):
        self._emit(ERROR, msg, args)

    def critical(self, msg, *args, **_kw):
        self._emit(CRITICAL, msg, args)

    def exception(self, msg, *args, **_kw):
        self._emit(ERROR, msg, args)
        if sys.exc_info()[0] is not None:
            sys.stdout.write(traceback.format_exc())
            sys.stdout.flush()

    def setLevel(self, level) -> None:
        self.level = _coerce_level(level)


def getLogger(name: str | None = None) -> Logger:
    name = name or "root"
    logger = _registry.get(name)
    if logger is None:
        logger = _registry[name] = Logger(name, _default_level)
    return logger


def setLevel(level) -> None:
    """Set the level of every existing logger and the default for new ones."""
    global _default_level
    _default_level = _coerce_level(level)
    for logger in _registry.values():
        logger.level = _default_level


def basicConfig(level=INFO, **_ignored) -> None:
    """stdlib-compatible shim: only ``level`` is honoured."""
    setLevel(level)
