"""Logging setup: one colourised stream handler, limited to this package's loggers."""

from __future__ import annotations

import logging
import sys

_COLORS = {"DEBUG": "\033[36m", "INFO": "\033[32m", "WARNING": "\033[33m", "ERROR": "\033[31m",
           "CRITICAL": "\033[35m"}
_RESET = "\033[0m"
_PREFIXES = ("parallax_b200", "__main__", "bench")
_configured = False


class _Formatter(logging.Formatter):
    def __init__(self, color: bool):
        super().__init__("%(asctime)s %(levelname)-7s %(name)s: %(message)s", "%H:%M:%S")
        self.color = color

    def format(self, record: logging.LogRecord) -> str:
        s = super().format(record)
        if self.color:
            return f"{_COLORS.get(record.levelname, '')}{s}{_RESET}"
        return s


class _PackageFilter(logging.Filter):
    def filter(self, record: logging.LogRecord) -> bool:
        return record.name.startswith(_PREFIXES) or record.levelno >= logging.WARNING


def set_log_level(level: str = "INFO") -> None:
    global _configured
    root = logging.getLogger()
    if not _configured:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(_Formatter(sys.stderr.isatty()))
        h.addFilter(_PackageFilter())
        root.addHandler(h)
        _configured = True
    root.setLevel(getattr(logging, level.upper(), logging.INFO))


def get_logger(name: str) -> logging.Logger:
    return logging.getLogger(name)
