"""``logging.getLogger("cosmos")`` with the level taken from COSMOS_LOG_LEVEL (cosmos_rl/utils/logging.py:1-40)."""
import logging
import os
import sys

logger = logging.getLogger("cosmos")
if not logger.handlers:
    _h = logging.StreamHandler(sys.stderr)
    _h.setFormatter(logging.Formatter("[cosmos] %(asctime)s %(levelname)s %(message)s", "%H:%M:%S"))
    logger.addHandler(_h)
    logger.setLevel(os.environ.get("COSMOS_LOG_LEVEL", "INFO").upper())
    logger.propagate = False
