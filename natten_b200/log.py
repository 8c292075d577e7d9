"""Logging for natten_b200, driven by the same two environment variables the reference uses
(src/natten/utils/log.py:43-134), so a user who sets them for one library gets the other too:

* ``NATTEN_LOG_LEVEL`` = debug | info | warning | error | critical (default: info)
* ``NATTEN_LOG_PIPE``  = stdout (default) | stderr | /dev/null | a writable file path

At DEBUG every attention call says which kernel it took (tensor cores on the caller's layout,
tensor cores on token-permuted copies, CUDA cores), with which tile shapes, how many key/value
tiles a query tile walks on average and whether the head dim was padded; the multi-GPU and
host-streaming helpers say how they partitioned the work. Nothing is logged while torch.compile
is tracing (a log call would be traced into the graph or break it).
"""
from __future__ import annotations

import logging
import os
import sys

_LEVELS = {"debug": logging.DEBUG, "info": logging.INFO, "warning": logging.WARNING,
           "error": logging.ERROR, "critical": logging.CRITICAL}
_FORMAT = "| %(asctime)s | [[ %(name)s ]] [ %(levelname)s ]: %(message)s"


def _level() -> int:
    return _LEVELS.get(os.environ.get("NATTEN_LOG_LEVEL", "").strip().lower(), logging.INFO)


def _handler() -> logging.Handler:
    pipe = os.environ.get("NATTEN_LOG_PIPE", "stdout").strip()
    low = pipe.lower()
    if low == "stderr":
        return logging.StreamHandler(sys.stderr)
    if low in ("stdout", ""):
        return logging.StreamHandler(sys.stdout)
    if pipe == "/dev/null":
        return logging.NullHandler()
    try:
        return logging.FileHandler(pipe)
    except OSError:
        return logging.NullHandler()


def _tracing() -> bool:
    try:
        import torch
        return bool(torch.compiler.is_compiling())
    except Exception:
        return False


class Logger:
    """A named logger; the level and the pipe are read from the environment when it is made."""

    def __init__(self, name: str):
        self._log = logging.getLogger(name)
        self._log.setLevel(_level())
        self._log.propagate = False
        if not self._log.handlers:
            h = _handler()
            h.setLevel(_level())
            h.setFormatter(logging.Formatter(_FORMAT))
            self._log.addHandler(h)

    @property
    def debug_enabled(self) -> bool:
        return self._log.isEnabledFor(logging.DEBUG)

    def debug(self, msg: str, *args) -> None:
        if self.debug_enabled and not _tracing():
            self._log.debug(msg, *args)

    def info(self, msg: str, *args) -> None:
        if not _tracing():
            self._log.info(msg, *args)

    def warning(self, msg: str, *args) -> None:
        if not _tracing():
            self._log.warning(msg, *args)


def get_logger(name: str) -> Logger:
    return Logger(name)
