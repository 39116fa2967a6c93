"""Loggers with timestamps relative to process start (reference: disagmoe/utils/logger.py)."""
import logging
import os
import sys
import time

_T0 = time.time()
_LEVEL = os.environ.get("DMOE_LOG_LEVEL", "WARNING").upper()


class _RelFormatter(logging.Formatter):
    def format(self, record):
        record.rel = f"{record.created - _T0:9.3f}"
        return super().format(record)


_handler = None


def get_logger(name: str) -> logging.Logger:
    global _handler
    if _handler is None:
        _handler = logging.StreamHandler(sys.stderr)
        _handler.setFormatter(_RelFormatter("[%(rel)ss %(levelname).1s %(name)s pid=%(process)d] %(message)s"))
    lg = logging.getLogger("dmoe." + name)
    if not lg.handlers:
        lg.addHandler(_handler)
        lg.propagate = False
        lg.setLevel(getattr(logging, _LEVEL, logging.WARNING))
    return lg
