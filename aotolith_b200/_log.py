"""Package logger: ``logging.getLogger("aotolith_b200")`` with a NullHandler.

``AOTOLITH_LOG=<level>`` (or :func:`configure_logging`) attaches a stderr
handler, as the reference's ``src/aotolith/_log.py`` does for its logger.
"""

from __future__ import annotations

import logging
import os

LOGGER_NAME = "aotolith_b200"
logger = logging.getLogger(LOGGER_NAME)
logger.addHandler(logging.NullHandler())


def configure_logging(level: str | int = "INFO") -> logging.Logger:
    if isinstance(level, str):
        level = getattr(logging, level.upper(), logging.INFO)
    if not any(isinstance(h, logging.StreamHandler) and not isinstance(h, logging.NullHandler) for h in logger.handlers):
        handler = logging.StreamHandler()
        handler.setFormatter(logging.Formatter("%(asctime)s %(name)s %(levelname)s %(message)s"))
        logger.addHandler(handler)
    logger.setLevel(level)
    return logger


if os.environ.get("AOTOLITH_LOG"):
    configure_logging(os.environ["AOTOLITH_LOG"])
