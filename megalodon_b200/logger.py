"""Process-wide logging set-up: stdout gets everything, stderr gets warnings
and above, every record is prefixed `LEVEL date - elapsed - ` (same line
format as the reference, megalodon/logger.py:8-60)."""
from __future__ import annotations

import logging
import sys
import time
from datetime import timedelta


class LogFormatter(logging.Formatter):
    def __init__(self):
        super().__init__()
        self._t0 = time.time()

    def format(self, record: logging.LogRecord) -> str:
        whole = int(record.created)
        micros = int((record.created - whole) * 1e6)
        stamp = time.strftime("%y-%m-%d %H:%M:%S", time.localtime(whole)) + f".{micros:06d}"
        elapsed = timedelta(seconds=round(record.created - self._t0))
        prefix = f"{record.levelname:<7} {stamp} - {elapsed} - "
        body = record.getMessage().replace("\n", "\n" + " " * len(prefix))
        return prefix + body


def _stream(stream, level):
    h = logging.StreamHandler(stream)
    h.setLevel(level)
    h.setFormatter(LogFormatter())
    return h


def initialize_logger() -> logging.Logger:
    root = logging.getLogger()
    root.setLevel(logging.NOTSET)
    root.handlers.clear()
    root.addHandler(_stream(sys.stdout, logging.NOTSET))
    root.addHandler(_stream(sys.stderr, logging.WARNING))
    return root


def add_logger_file_handler(filepath: str) -> None:
    h = logging.FileHandler(filepath, "a")
    h.setLevel(logging.INFO)
    h.setFormatter(LogFormatter())
    logging.getLogger().addHandler(h)
