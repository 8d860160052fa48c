"""Process-wide logging set-up with a rank prefix (reference: ``astrai/logging.py:5-35``)."""

import logging as _logging
import os

LOGGER_NAME = "astrai_b200"
_FORMAT = "%(asctime)s | %(levelname)-8s | rank=%(rank)2s/%(world_size)-2s | %(name)-32s | %(message)s"


class _RankFilter(_logging.Filter):
    def filter(self, record):
        record.rank = os.environ.get("RANK", "0")
        record.world_size = os.environ.get("WORLD_SIZE", "1")
        return True


def setup_logging(level: str = "INFO"):
    """Install one stream handler on the package logger; ``ASTR_LOG_LEVEL`` overrides *level*."""
    logger = _logging.getLogger(LOGGER_NAME)
    if logger.handlers:
        return logger
    name = os.environ.get("ASTR_LOG_LEVEL", level).upper()
    logger.setLevel(getattr(_logging, name, _logging.INFO))
    handler = _logging.StreamHandler()
    handler.addFilter(_RankFilter())
    handler.setFormatter(_logging.Formatter(_FORMAT, datefmt="%Y-%m-%d %H:%M:%S"))
    logger.addHandler(handler)
    return logger
