"""Expert-parallel plumbing: symmetric Buffers, the gloo backend and the virtual-rank harness."""
from .buffer import (PHASE_ALL, PHASE_COUNT, PHASE_FINAL, PHASE_RECV, PHASE_SEND, Buffer, phases,  # noqa: F401
                     run_virtual)
from .gloo_backend import CpuGroup  # noqa: F401
