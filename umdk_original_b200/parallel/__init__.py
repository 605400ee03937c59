"""Expert-parallel plumbing: symmetric Buffers, the gloo backend and the virtual-rank harness."""
from .buffer import (PHASE_ALL, PHASE_COUNT, PHASE_FINAL, PHASE_RECV, PHASE_SEND, PHASE_TP_RECV,  # noqa: F401
                     PHASE_TP_SEND, Buffer, phases, run_virtual)
from .gloo_backend import CpuGroup  # noqa: F401
