"""CPU oracle for every op of the library (pure PyTorch, fp32 arithmetic, deterministic).

The reference has no CPU implementation: its only oracle is a chain of stock NPU ops
(test/cam/ut/fused_deep_moe/test_fused_deep_moe.py:126-197).  This module restates the
contracts of the six ops and the kernel math so that GPU kernels, the gloo backend and the
multi-rank protocols can all be checked against one source of truth:

* quantisation formulas (identical, operation for operation, to csrc/common/quant.cuh)
* ``get_dispatch_layout`` (dispatch_layout.h:108-124)
* the receive-row order of dispatch: local expert major, source rank ascending, sender scan
  order (pybind/moe_dispatch_prefill.cpp:103-145), for any number of simulated ranks
* combine: ``out[t] = rint_bf16(sum_k w[t,k] * row(t,k))`` in k order (moe_combine_normal.h:312-337)
* the dense MoE layer and the block-scaled fp8 / int8 W8A8 expert MLPs (fused_deep_moe math,
  GMM1.h:781-818, block_epilogue_per_token_dequant_swiglu.h:236-264, GMM1.h:193-265).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

FP8_MAX = 448.0
FP8 = torch.float8_e4m3fn


# ----------------------------------------------------------------------------------------------
# Quantisation
# ----------------------------------------------------------------------------------------------
def ue8m0_round_up(scale: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= scale (fp32, positive, normal): what a UE8M0 scale factor can hold.
    Same bit arithmetic as ue8m0_scale() in csrc/common/quant.cuh."""
    bits = scale.float().contiguous().view(torch.int32)
    e = (bits >> 23) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return (e << 23).view(torch.float32)


def is_power_of_two(scale: torch.Tensor) -> bool:
    bits = scale.float().contiguous().view(torch.int32)
    return bool(((bits & 0x7FFFFF) == 0).all()) and bool((scale > 0).all())


def quant_fp8_1x128(x: torch.Tensor, ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """e4m3 with one fp32 scale per 128 contiguous elements of the last dim.  With ``ue8m0`` the
    scale is rounded up to a power of two (the form the tensor core's block scaling takes)."""
    n, h = x.shape
    assert h % 128 == 0
    xf = x.float().view(n, h // 128, 128)
    amax = xf.abs().amax(dim=-1).clamp_min(1e-4)
    if ue8m0:
        scale = ue8m0_round_up(amax / torch.tensor(FP8_MAX, dtype=torch.float32))
        q = (xf * (1.0 / scale).unsqueeze(-1)).to(FP8).view(n, h)
        return q, scale
    inv = (torch.tensor(FP8_MAX, dtype=torch.float32) / amax).unsqueeze(-1)
    q = (xf * inv).to(FP8).view(n, h)
    return q, amax / FP8_MAX


def dequant_fp8_1x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    n, h = q.shape
    return (q.float().view(n, h // 128, 128) * s.float().unsqueeze(-1)).view(n, h)


def quant_fp8_128x128(w: torch.Tensor, ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Weights [..., N, K] -> e4m3 with one fp32 scale per 128x128 block (scale = amax/448, rounded
    up to a power of two with ``ue8m0``)."""
    *lead, n, k = w.shape
    assert n % 128 == 0 and k % 128 == 0
    wf = w.float().reshape(*lead, n // 128, 128, k // 128, 128)
    amax = wf.abs().amax(dim=(-3, -1)).clamp_min(1e-4)  # [..., n/128, k/128]
    scale = amax / FP8_MAX
    if ue8m0:
        scale = ue8m0_round_up(scale)
    q = (wf / scale.unsqueeze(-1).unsqueeze(-3)).to(FP8).reshape(*lead, n, k)
    return q, scale


def dequant_fp8_128x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    *lead, n, k = q.shape
    qf = q.float().reshape(*lead, n // 128, 128, k // 128, 128)
    return (qf * s.float().unsqueeze(-1).unsqueeze(-3)).reshape(*lead, n, k)


def quant_int8_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """int8 with one fp32 scale per 128 contiguous elements (the wire format of combine's comm quant)."""
    n, h = x.shape
    xf = x.float().view(n, h // 128, 128)
    amax = xf.abs().amax(dim=-1).clamp_min(1e-12)
    inv = (torch.tensor(127.0, dtype=torch.float32) / amax).unsqueeze(-1)
    q = torch.round(xf * inv).clamp_(-127, 127).to(torch.int8).view(n, h)
    return q, amax / 127.0


def dequant_int8_1x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    n, h = q.shape
    return (q.float().view(n, h // 128, 128) * s.float().unsqueeze(-1)).view(n, h)


def quant_int8_token(x: torch.Tensor, smooth: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token dynamic int8 (moe_dispatch_normal.h:289-315): q = rint(x*127/(amax+1e-12))."""
    xf = x.float()
    if smooth is not None:
        xf = xf * smooth.float()
    amax = xf.abs().amax(dim=-1, keepdim=True)
    inv = torch.tensor(127.0, dtype=torch.float32) / (amax + 1e-12)
    q = torch.round(xf * inv).clamp_(-127, 127).to(torch.int8)
    return q, (1.0 / inv).squeeze(-1)


# ----------------------------------------------------------------------------------------------
# Shared-expert ranks
# ----------------------------------------------------------------------------------------------
def remap_for_shared_ranks(ids: torch.Tensor, weights: Optional[torch.Tensor], num_ranks: int, moe_expert_num: int,
                           shared_rank_num: int):
    """Routing over "virtual" experts when the first ``shared_rank_num`` ranks hold a replica of the
    shared expert (moe_dispatch_shmem.h:408-489): with E_l = moe_expert_num / (R - S) local experts per
    routed rank, routed expert e becomes e + S * E_l, the replica on rank s is virtual expert s * E_l,
    and every token gets one more pair (weight 1) to replica min(S - 1, t * S / T).
    Returns (ids [T, K+1], weights [T, K+1] or None, virtual expert count, E_l)."""
    assert 0 < shared_rank_num < num_ranks and moe_expert_num % (num_ranks - shared_rank_num) == 0
    el = moe_expert_num // (num_ranks - shared_rank_num)
    t = ids.shape[0]
    routed = torch.where(ids >= 0, ids + shared_rank_num * el, torch.full_like(ids, -1))
    tok = torch.arange(t, dtype=ids.dtype, device=ids.device)
    replica = torch.clamp(torch.div(tok * shared_rank_num, max(t, 1), rounding_mode="floor"), max=shared_rank_num - 1)
    new_ids = torch.cat([routed, (replica * el).unsqueeze(1)], dim=1).contiguous()
    new_w = None
    if weights is not None:
        new_w = torch.cat([weights.float(), torch.ones(t, 1, dtype=torch.float32, device=weights.device)], dim=1).contiguous()
    return new_ids, new_w, el * num_ranks, el


# ----------------------------------------------------------------------------------------------
# Layout and dispatch order
# ----------------------------------------------------------------------------------------------
def get_dispatch_layout(topk_idx: torch.Tensor, num_experts: int, num_ranks: int):
    t, k = topk_idx.shape
    el = num_experts // num_ranks
    idx = topk_idx.long()
    valid = (idx >= 0) & (idx < num_experts)
    per_expert = torch.zeros(num_experts, dtype=torch.int32)
    flat = idx[valid]
    if flat.numel():
        per_expert += torch.bincount(flat, minlength=num_experts).to(torch.int32)
    in_rank = torch.zeros(t, num_ranks, dtype=torch.bool)
    if t:
        rank_of = torch.where(valid, idx // el, torch.zeros_like(idx))
        for kk in range(k):
            rows = torch.nonzero(valid[:, kk]).squeeze(-1)
            in_rank[rows, rank_of[rows, kk]] = True
    per_rank = in_rank.sum(dim=0).to(torch.int32)
    return per_rank, per_expert, in_rank


@dataclass
class DispatchPlan:
    """Receive side of one rank after a dispatch among `num_ranks` simulated ranks."""
    src: torch.Tensor          # [N, 3] (src rank, src token, src k) per received row
    recv_count: torch.Tensor   # [E_local * R] inclusive cumsum, expert major / source minor
    per_expert: torch.Tensor   # [E_local] rows per local expert
    expert_offsets: torch.Tensor  # [E_local + 1]


def slots_in_expert(topk_idx: torch.Tensor, num_experts: int, active_tokens: Optional[int] = None) -> torch.Tensor:
    """expandIdx of the reference (moe_dispatch_shmem.h:629-638): for every (t, k) pair in scan
    order, the number of earlier pairs of this rank routed to the same expert; -1 if skipped."""
    t, k = topk_idx.shape
    flat = topk_idx.reshape(-1).long().clone()
    if active_tokens is not None:
        flat[active_tokens * k:] = -1
    out = torch.full((t * k,), -1, dtype=torch.int32)
    seen = [0] * num_experts
    for i, e in enumerate(flat.tolist()):
        if 0 <= e < num_experts:
            out[i] = seen[e]
            seen[e] += 1
    return out


def plan_dispatch(topk_per_rank: Sequence[torch.Tensor], num_experts: int) -> List[DispatchPlan]:
    """Row order every rank must observe after dispatch (same for normal and low-latency)."""
    r = len(topk_per_rank)
    el = num_experts // r
    plans = []
    for dst in range(r):
        rows, counts = [], torch.zeros(el, r, dtype=torch.int64)
        for le in range(el):
            e = dst * el + le
            for src in range(r):
                idx = topk_per_rank[src].long()
                hits = torch.nonzero(idx.reshape(-1) == e).squeeze(-1)
                k = idx.shape[1]
                for i in hits.tolist():
                    rows.append((src, i // k, i % k))
                counts[le, src] = hits.numel()
        src_t = torch.tensor(rows, dtype=torch.int32).reshape(-1, 3)
        cum = counts.reshape(-1).cumsum(0).to(torch.int32)
        per_e = counts.sum(dim=1)
        off = torch.cat([torch.zeros(1, dtype=torch.int64), per_e.cumsum(0)]).to(torch.int32)
        plans.append(DispatchPlan(src_t, cum, per_e, off))
    return plans


def combine_reference(rows_by_pair: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                      num_experts: int) -> torch.Tensor:
    """rows_by_pair [T, K, h] (bf16 expert outputs per pair) -> [T, h] bf16, fp32 sum in k order."""
    t, k, h = rows_by_pair.shape
    acc = torch.zeros(t, h, dtype=torch.float32)
    idx = topk_idx.long()
    for kk in range(k):
        ok = ((idx[:, kk] >= 0) & (idx[:, kk] < num_experts)).float().unsqueeze(-1)
        acc = torch.addcmul(acc, rows_by_pair[:, kk].float() * ok, topk_weights[:, kk].float().unsqueeze(-1))
    return acc.to(torch.bfloat16)


# ----------------------------------------------------------------------------------------------
# Expert MLPs
# ----------------------------------------------------------------------------------------------
def swiglu_mlp_fp32(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """x [n,h], w1 [2I,h] (gate rows first: 'activate_left'), w2 [h,I] -> [n,h], all fp32."""
    y = x.float() @ w1.float().t()
    i = w1.shape[0] // 2
    g, u = y[:, :i], y[:, i:]
    return (torch.nn.functional.silu(g) * u) @ w2.float().t()


def dense_moe_fp32(x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, w1: torch.Tensor,
                   w2: torch.Tensor) -> torch.Tensor:
    """Single-process dense MoE: w1 [E,2I,h], w2 [E,h,I]; out[t] = sum_k w[t,k] * MLP_e(x[t])."""
    t, h = x.shape
    out = torch.zeros(t, h, dtype=torch.float32)
    e_total = w1.shape[0]
    idx = topk_idx.long()
    for e in range(e_total):
        tok, kk = torch.nonzero(idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        y = swiglu_mlp_fp32(x[tok], w1[e], w2[e])
        out.index_add_(0, tok, y * topk_weights[tok, kk].float().unsqueeze(-1))
    return out


def expert_mlp_fp8(xq: torch.Tensor, xs: torch.Tensor, w1q: torch.Tensor, w1s: torch.Tensor, w2q: torch.Tensor,
                   w2s: torch.Tensor, return_act: bool = False, ue8m0: bool = False):
    """Block-scaled fp8 expert MLP exactly as the two grouped GEMMs compute it (one expert).
    xq [n,h] e4m3 + xs [n,h/128]; w1q [2I,h] + w1s [2I/128,h/128]; w2q [h,I] + w2s [h/128,I/128].
    Returns bf16 [n,h]."""
    x = dequant_fp8_1x128(xq, xs)
    y = x @ dequant_fp8_128x128(w1q, w1s).t()
    i = w1q.shape[0] // 2
    g, u = y[:, :i], y[:, i:]
    a = (g / (1.0 + torch.exp(-g))) * u
    aq, a_s = quant_fp8_1x128(a, ue8m0)
    z = dequant_fp8_1x128(aq, a_s) @ dequant_fp8_128x128(w2q, w2s).t()
    if return_act:
        return z.to(torch.bfloat16), aq, a_s
    return z.to(torch.bfloat16)


def fused_moe_fp8_reference(x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, w1q: torch.Tensor,
                            w1s: torch.Tensor, w2q: torch.Tensor, w2s: torch.Tensor,
                            ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Whole fp8 MoE layer for one rank's tokens with all experts visible (w*: [E, ...]).
    Returns (out [T,h] bf16, tokens per expert [E] int64)."""
    t, h = x.shape
    k = topk_idx.shape[1]
    e_total = w1q.shape[0]
    xq, xs = quant_fp8_1x128(x, ue8m0)
    rows = torch.zeros(t, k, h, dtype=torch.bfloat16)
    counts = torch.zeros(e_total, dtype=torch.int64)
    idx = topk_idx.long()
    for e in range(e_total):
        tok, kk = torch.nonzero(idx == e, as_tuple=True)
        counts[e] = tok.numel()
        if tok.numel() == 0:
            continue
        rows[tok, kk] = expert_mlp_fp8(xq[tok], xs[tok], w1q[e], w1s[e], w2q[e], w2s[e], ue8m0=ue8m0)
    return combine_reference(rows, topk_idx, topk_weights, e_total), counts


def expert_mlp_w8a8(x: torch.Tensor, w1: torch.Tensor, s1: torch.Tensor, w2: torch.Tensor, s2: torch.Tensor) -> torch.Tensor:
    """int8 W8A8 expert MLP of the reference (fused_deep_moe): x [n,h] bf16; w1 [2I,h] int8 with
    per-output-channel scale s1 [2I]; w2 [h,I] int8 with s2 [h].  Exact int32 accumulation."""
    xf = x.float()
    sx = xf.abs().amax(dim=-1, keepdim=True).clamp_min(1e-12) / 127.0
    xq = torch.round(xf / sx).clamp_(-127, 127)
    acc1 = xq.double() @ w1.double().t()
    y = acc1.float() * s1.float().unsqueeze(0) * sx
    i = w1.shape[0] // 2
    g, u = y[:, :i], y[:, i:]
    a = (g / (1.0 + torch.exp(-g))) * u
    sa = a.abs().amax(dim=-1, keepdim=True).clamp_min(1e-12) / 127.0
    aq = torch.round(a / sa).clamp_(-127, 127)
    acc2 = aq.double() @ w2.double().t()
    return (acc2.float() * s2.float().unsqueeze(0) * sa).to(torch.bfloat16)
