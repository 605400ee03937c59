"""Logging.  The reference's host side prints through OP_LOGE/OP_LOGW macros that map to printf,
with info/debug compiled out (ascend_kernels/utils/op_host/error_log.h:15-26).  Here it is the
standard ``logging`` module; ``UMDK_CAM_LOG`` (debug|info|warning|error) sets the level."""
from __future__ import annotations

import logging
import os

_CONFIGURED = False


def get_logger(name: str = "umdk_cam") -> logging.Logger:
    global _CONFIGURED
    logger = logging.getLogger(name)
    if not _CONFIGURED:
        level = os.environ.get("UMDK_CAM_LOG", "warning").upper()
        root = logging.getLogger("umdk_cam")
        if not root.handlers:
            h = logging.StreamHandler()
            h.setFormatter(logging.Formatter("[%(asctime)s %(name)s %(levelname)s] %(message)s"))
            root.addHandler(h)
        root.setLevel(getattr(logging, level, logging.WARNING))
        _CONFIGURED = True
    return logger
