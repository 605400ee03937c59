"""Top-k routing.  Routing is outside the reference's ops (callers pass expert ids and weights);
the benchmarks need it to produce ids of the right distribution."""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def topk_softmax(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Plain top-k with a softmax over the selected logits."""
    vals, idx = torch.topk(logits.float(), k, dim=-1)
    return idx.to(torch.int64), torch.softmax(vals, dim=-1)


def grouped_topk(logits: torch.Tensor, k: int, num_groups: int, topk_groups: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Group-limited routing: keep the `topk_groups` groups with the largest per-group maximum,
    then top-k among their experts (a token reaches at most `topk_groups` groups of experts)."""
    t, e = logits.shape
    lf = logits.float()
    g = lf.view(t, num_groups, e // num_groups)
    group_score = g.max(dim=-1).values
    keep = torch.topk(group_score, topk_groups, dim=-1).indices
    mask = torch.zeros(t, num_groups, dtype=torch.bool, device=logits.device)
    mask.scatter_(1, keep, True)
    masked = lf.masked_fill(~mask.unsqueeze(-1).expand(-1, -1, e // num_groups).reshape(t, e), float("-inf"))
    return topk_softmax(masked, k)


def zipf_bias(num_experts: int, s: float = 1.2, scale: float = 1.0, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Additive gate bias log(rank^-s) over a random permutation of experts: hot experts draw a
    multiple of the mean load."""
    ranks = torch.arange(1, num_experts + 1, dtype=torch.float32)
    bias = -s * torch.log(ranks) * scale
    perm = torch.randperm(num_experts, generator=generator)
    return bias[perm]


def route(logits: torch.Tensor, k: int, num_groups: int = 1, topk_groups: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    if num_groups > 1 and topk_groups < num_groups:
        return grouped_topk(logits, k, num_groups, topk_groups)
    return topk_softmax(logits, k)
