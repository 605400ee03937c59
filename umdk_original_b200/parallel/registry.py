"""Name / id registry of CPU (gloo) groups.  CUDA buffers are registered inside the native
extension; this is the same lookup for the CPU path (``group_ep`` is a name, ``extInfo`` an id)."""
from __future__ import annotations

from typing import Dict

from .gloo_backend import CpuGroup

_BY_NAME: Dict[str, CpuGroup] = {}
_BY_ID: Dict[int, CpuGroup] = {}
_NEXT = [1 << 20]  # ids of CPU groups live far from the native ids, which start at 1


def register(g: CpuGroup, name: str) -> int:
    g.name = name
    g.ident = _NEXT[0]
    _NEXT[0] += 1
    _BY_NAME[name] = g
    _BY_ID[g.ident] = g
    return g.ident


def unregister(g: CpuGroup) -> None:
    _BY_NAME.pop(g.name, None)
    _BY_ID.pop(g.ident, None)


def by_name(name: str) -> CpuGroup:
    if name not in _BY_NAME:
        raise KeyError(f"umdk_cam_op_lib: no CPU Buffer is registered under the group name '{name}'")
    return _BY_NAME[name]


def by_id(ident: int) -> CpuGroup:
    if ident not in _BY_ID:
        raise KeyError(f"umdk_cam_op_lib: extInfo {ident} is not the id of a live CPU Buffer")
    return _BY_ID[ident]
