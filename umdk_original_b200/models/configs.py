"""Model / benchmark shapes.  The reference ships no model code: the shapes it exercises are the
4-rank unit-test case (test/cam/ut/fused_deep_moe/test_fused_deep_moe.py:339-348) and the 16-rank
example (src/cam/examples/fused_deep_moe_sample.py:30-43).  The DeepSeek-V3 and Qwen3-MoE rows are
the layer shapes the benchmarks of this library are quoted on."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class MoEConfig:
    name: str
    hidden: int
    intermediate: int
    num_experts: int
    topk: int
    tokens_per_rank: int
    num_groups: int = 1          # expert groups for group-limited routing (1 = plain top-k)
    topk_groups: int = 1
    weight_format: str = "fp8_block"   # fp8_block | w8a8 | float

    def flops_per_token(self) -> int:
        """Tensor-core FLOPs of the expert MLPs for one token (top-k experts, gate+up and down)."""
        return 2 * self.topk * 3 * self.hidden * self.intermediate


DEEPSEEK_V3 = MoEConfig("deepseek-v3-moe", 7168, 2048, 256, 8, 4096, num_groups=8, topk_groups=4)
QWEN3_MOE = MoEConfig("qwen3-moe-w8a8", 4096, 1536, 128, 8, 8192, weight_format="w8a8")
CPU_PLUMBING = MoEConfig("cpu-plumbing", 1024, 512, 8, 2, 128, weight_format="float")
REFERENCE_UT_4RANK = MoEConfig("reference-ut-4rank", 7168, 2048, 16, 8, 16, weight_format="w8a8")
LOW_LATENCY = MoEConfig("deepseek-v3-decode", 7168, 2048, 256, 8, 128)
TINY = MoEConfig("tiny", 256, 128, 8, 2, 32)

BY_NAME = {c.name: c for c in (DEEPSEEK_V3, QWEN3_MOE, CPU_PLUMBING, REFERENCE_UT_4RANK, LOW_LATENCY, TINY)}
