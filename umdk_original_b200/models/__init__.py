"""Model-level pieces: layer shapes, routing, expert weights and the FusedMoE layer."""
from .configs import (BY_NAME, CPU_PLUMBING, DEEPSEEK_V3, LOW_LATENCY, QWEN3_MOE, REFERENCE_UT_4RANK, TINY,  # noqa: F401
                      MoEConfig)
from .fused_moe import FusedMoE, MoEStepRunner, make_buffer_for  # noqa: F401
from .router import grouped_topk, route, topk_softmax, zipf_bias  # noqa: F401
from .weights import (ExpertWeights, from_reference_w8a8, quantize_fp8_block, random_fp8_experts,  # noqa: F401
                      random_w8a8_experts, stack_tensor_list)
