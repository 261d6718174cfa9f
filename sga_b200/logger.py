"""The ``sga`` logger; level from ``SGA_LOG_LEVEL`` (default INFO). ``sga/logger.py:1-27``."""
import logging
import os

_LOGGER = None


def get_logger() -> logging.Logger:
    global _LOGGER
    if _LOGGER is None:
        lg = logging.getLogger("sga")
        level = os.environ.get("SGA_LOG_LEVEL", "INFO").upper()
        lg.setLevel(getattr(logging, level, logging.INFO))
        if not lg.handlers:
            h = logging.StreamHandler()
            h.setFormatter(logging.Formatter("[%(asctime)s %(name)s %(levelname)s] %(message)s"))
            lg.addHandler(h)
        lg.propagate = False
        _LOGGER = lg
    return _LOGGER
