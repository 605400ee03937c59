"""umdk_original_b200 -- a B200-native MoE expert-parallel communication library with the op
surface of UMDK's CAM component (``torch.ops.umdk_cam_op_lib``): normal and low-latency
dispatch/combine, a fused dispatch -> grouped GEMM -> SwiGLU -> grouped GEMM -> combine layer and
explicit symmetric buffers.  Hot paths are hand-written sm_100a CUDA (csrc/)."""
from . import ops, utils  # noqa: F401
from .ops import cam_ops  # noqa: F401
from . import parallel, models  # noqa: F401
from .parallel import Buffer  # noqa: F401
from .utils import CamConfig, CamError, MoeCommTimeout, RecvOverflow  # noqa: F401

__version__ = "0.1.0"
