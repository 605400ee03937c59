"""Exceptions raised from device status words.

The reference's kernels spin without a limit (moe_dispatch_normal.h:463-469,
moe_combine_normal.h:289-296); the only bounded wait in its tree returns a stale flag value
instead of an error (sync_collectives.h:375-416).  Here every device wait has a budget and
reports {code, who, detail, block}; this module turns that record into a Python exception.
"""
from __future__ import annotations

STATUS_TEXT = {
    0: "ok",
    1: "timeout waiting for a peer's per-expert counts",
    2: "timeout waiting for a peer's dispatch completion flag",
    3: "timeout waiting for a peer's combine completion flag",
    4: "rows routed to one rank or cell exceed the buffer capacity",
    5: "timeout inside the GEMM pipeline (mbarrier wait)",
    6: "timeout waiting for a low-latency count cell",
    7: "timeout in the cross-rank barrier",
    8: "index out of range recorded by a device-side check",
    9: "timeout waiting for the rows of one local expert to arrive (fused layer)",
    10: "timeout waiting for the first GEMM of a row block (fused layer)",
}
TIMEOUT_CODES = {1, 2, 3, 5, 6, 7, 9, 10}


class CamError(RuntimeError):
    """Base class: carries the raw status record."""

    def __init__(self, code: int, who: int, detail: int, block: int, text: str | None = None):
        self.code, self.who, self.detail, self.block = int(code), int(who), int(detail), int(block)
        msg = text or STATUS_TEXT.get(self.code, "unknown status")
        super().__init__(f"{msg} (code={self.code}, who={self.who}, detail={self.detail}, block={self.block})")


class MoeCommTimeout(CamError):
    """A bounded device wait ran out: a peer did not arrive.  Call ``Buffer.reset()`` on every
    surviving rank before the buffer is used again."""


class RecvOverflow(CamError):
    """More rows were routed to a rank than its receive buffer holds; nothing was written out of
    bounds, the surplus destination was skipped."""


def raise_for_status(code: int, who: int = -1, detail: int = 0, block: int = -1, text: str | None = None) -> None:
    if code == 0:
        return
    if code in TIMEOUT_CODES:
        raise MoeCommTimeout(code, who, detail, block, text)
    if code == 4:
        raise RecvOverflow(code, who, detail, block, text)
    raise CamError(code, who, detail, block, text)
