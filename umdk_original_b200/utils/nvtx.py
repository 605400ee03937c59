"""NVTX ranges around the Python-level steps, for timelines taken with an external profiler.

Off unless ``UMDK_CAM_NVTX=1`` (or ``enable(True)``): a disabled range costs one attribute test.  The
reference links a profiling API but places no ranges of its own (src/cam/comm_operator/pybind/setup.py:64,78).
"""
from __future__ import annotations

import contextlib
import os

import torch

_ON = [os.environ.get("UMDK_CAM_NVTX", "0") not in ("", "0", "false", "False")]


def enable(on: bool = True) -> None:
    _ON[0] = bool(on)


def enabled() -> bool:
    return _ON[0]


@contextlib.contextmanager
def nvtx_range(name: str):
    if not _ON[0] or not torch.cuda.is_available():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
