"""Rank-prefixed logging (the reference only has printf-style macros, examples/utils/utils.h:11-13)."""
from __future__ import annotations

import logging
import os

_configured = False


def get_logger(name: str = "catcoc") -> logging.Logger:
    global _configured
    if not _configured:
        rank = os.environ.get("RANK", "0")
        level = os.environ.get("CATCOC_LOG", "WARNING").upper()
        logging.basicConfig(level=getattr(logging, level, logging.WARNING),
                            format="[%(asctime)s rank " + rank + " %(levelname)s %(name)s] %(message)s")
        _configured = True
    return logging.getLogger(name)
