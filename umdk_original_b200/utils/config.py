"""Run-time configuration.

The reference has three tiers: build-time switches (build/cam/comm_operator/build.sh:35-76),
environment variables such as HCCL_BUFFSIZE (moe_dispatch_normal_tiling.cc:37-58) and per-call
attributes.  Here the per-call attributes stay on the ops, and everything else is this dataclass
with environment overrides (``UMDK_CAM_<FIELD>``)."""
from __future__ import annotations

import os
from dataclasses import dataclass, fields


@dataclass
class CamConfig:
    num_experts: int = 256
    max_tokens: int = 4096          # tokens per rank, normal mode
    hidden: int = 7168
    topk: int = 8
    capacity: int = 0               # receive rows per rank; 0 = worst case min(R*T*min(K,E_l), ...)
    capacity_factor: float = 0.0    # >0: capacity = factor * T * K (mean load per rank is T*K)
    ll_max_tokens: int = 0          # tokens per rank, low-latency mode (0 = disabled)
    timeout_ms: float = 10000.0     # budget of every device-side wait
    copy_outputs: bool = False      # prefill dispatch returns private copies instead of views of the buffer

    @classmethod
    def from_env(cls, **overrides) -> "CamConfig":
        cfg = cls(**overrides)
        for f in fields(cls):
            v = os.environ.get("UMDK_CAM_" + f.name.upper())
            if v is not None and f.name not in overrides:
                kind = type(getattr(cfg, f.name))
                setattr(cfg, f.name, v.strip().lower() in ("1", "true", "yes", "on") if kind is bool else kind(v))
        return cfg

    def resolve_capacity(self, num_ranks: int) -> int:
        if self.capacity > 0:
            return self.capacity
        el = max(1, self.num_experts // num_ranks)
        worst = num_ranks * self.max_tokens * min(self.topk, el)
        if self.capacity_factor > 0:
            return min(worst, max(128, int(self.capacity_factor * self.max_tokens * self.topk)))
        return worst
