"""Ops of ``torch.ops.umdk_cam_op_lib`` (same six names as the reference) and the CPU oracle."""
from . import reference  # noqa: F401
from .cam_ops import native_loaded, native_module, ops  # noqa: F401

fused_deep_moe = ops.fused_deep_moe
get_dispatch_layout = ops.get_dispatch_layout
moe_dispatch_prefill = ops.moe_dispatch_prefill
moe_combine_prefill = ops.moe_combine_prefill
moe_dispatch_shmem = ops.moe_dispatch_shmem
moe_combine_shmem = ops.moe_combine_shmem
moe_dispatch_prefill_quant = ops.moe_dispatch_prefill_quant
grouped_gemm_fp8 = ops.grouped_gemm_fp8
grouped_gemm_fp8_swiglu = ops.grouped_gemm_fp8_swiglu
