"""CPU / gloo implementation of the op contracts (world_size >= 1, one process per rank).

Same Python surface and the same row-order contracts as the CUDA kernels, built from
``torch.distributed.all_gather`` / ``all_to_all_single`` on CPU tensors.  It is the plumbing
check that runs without a GPU and the timed CPU baseline; the reference has no such path (its
tests need >= 4 NPUs, test/cam/ut/fused_deep_moe/test_fused_deep_moe.py:361-423).

Failure detection: every collective uses the group's timeout, so a rank that never joins makes
the others raise ``MoeCommTimeout`` instead of hanging.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import reference as ref
from ..utils.errors import MoeCommTimeout


@dataclass
class CpuGroup:
    """State a CUDA Buffer keeps in symmetric memory, kept here as plain tensors."""
    group: Optional[object]
    rank: int
    world: int
    num_experts: int
    name: str = ""
    ident: int = 0
    stats: Dict[str, int] = field(default_factory=lambda: {"dispatch_calls": 0, "combine_calls": 0, "rows_sent": 0})
    ll_src: Optional[torch.Tensor] = None      # [N,3] rows of the last low-latency dispatch
    last_src: Optional[torch.Tensor] = None    # [N,3] rows of the last normal dispatch
    drop_next_send: bool = False               # host-side fault injection: skip the next exchange
    tp_group: Optional[object] = None          # two ranks: this one and its tensor-parallel partner
    tp_rank: int = 0
    tp_counts: Optional[torch.Tensor] = None   # [2] rows each TP rank received in the last low-latency dispatch

    # ------------------------------------------------------------------ collectives
    def _guard(self, fn, *a, **kw):
        try:
            return fn(*a, **kw)
        except RuntimeError as e:  # gloo reports a timeout / dead peer as RuntimeError
            raise MoeCommTimeout(2, -1, 0, -1, f"gloo collective failed or timed out: {e}") from e

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t.unsqueeze(0).clone()
        out = [torch.empty_like(t) for _ in range(self.world)]
        self._guard(dist.all_gather, out, t.contiguous(), group=self.group)
        return torch.stack(out)

    def all_to_all(self, send: torch.Tensor, send_splits: List[int], recv_splits: List[int]) -> torch.Tensor:
        if self.world == 1:
            return send.clone()
        out = send.new_empty((sum(recv_splits),) + tuple(send.shape[1:]))
        self._guard(dist.all_to_all_single, out, send.contiguous(), output_split_sizes=recv_splits,
                    input_split_sizes=send_splits, group=self.group)
        return out


    def tp_exchange(self, mine: torch.Tensor, counts: List[int]) -> torch.Tensor:
        """Rows of the tensor-parallel partner: this rank contributes ``mine`` (counts[tp_rank] rows), the
        partner counts[1 - tp_rank] rows.  Both sides pad to the larger count, since gloo's all_gather wants
        equal shapes; fp8 rows travel as bytes."""
        me = self.tp_rank
        n_max = max(counts)
        as_bytes = mine.dtype == ref.FP8
        t = mine.view(torch.uint8) if as_bytes else mine
        pad = t.new_zeros((n_max,) + tuple(t.shape[1:]))
        pad[:counts[me]] = t[:counts[me]]
        out = [torch.empty_like(pad), torch.empty_like(pad)]
        self._guard(dist.all_gather, out, pad, group=self.tp_group)
        got = out[1 - me][:counts[1 - me]]
        return got.view(ref.FP8) if as_bytes else got

    def tp_all_gather_counts(self, n: int) -> List[int]:
        out = [torch.zeros(1, dtype=torch.long), torch.zeros(1, dtype=torch.long)]
        self._guard(dist.all_gather, out, torch.tensor([n], dtype=torch.long), group=self.tp_group)
        return [int(out[0]), int(out[1])]


def _send_order(topk_idx: torch.Tensor, num_experts: int, world: int, active: Optional[int] = None):
    """Pairs of this rank ordered (destination rank, local expert, scan order)."""
    t, k = topk_idx.shape
    flat = topk_idx.reshape(-1).long().clone()
    if active is not None:
        flat[active * k:] = -1
    valid = (flat >= 0) & (flat < num_experts)
    pair = torch.nonzero(valid).squeeze(-1)
    order = torch.argsort(flat[pair], stable=True)  # expert-major keeps scan order inside an expert
    pair = pair[order]
    counts = torch.bincount(flat[pair], minlength=num_experts) if pair.numel() else torch.zeros(num_experts, dtype=torch.long)
    return pair, counts


def dispatch(g: CpuGroup, x: torch.Tensor, topk_idx: torch.Tensor, quant_mode: int = 0,
             active: Optional[int] = None, smooth: Optional[torch.Tensor] = None):
    """Returns (recv_x, recv_scales|None, src [N,3] int32, recv_count [E_l*R] int32, per_expert [E_l] int64,
    slots [T*K] int32)."""
    e_total, r = g.num_experts, g.world
    el = e_total // r
    t, k = topk_idx.shape
    pair, counts = _send_order(topk_idx, e_total, r, active)
    cm = g.all_gather(counts)  # [R, E]
    tok = pair // k
    rows = x[tok]
    scales = None
    if quant_mode in (3, 4):
        rows, scales = ref.quant_fp8_1x128(rows, quant_mode == 4) if rows.numel() else (rows.to(ref.FP8), rows.new_zeros((0, x.shape[1] // 128), dtype=torch.float32))
    elif quant_mode == 2:
        if smooth is not None and rows.numel():
            ids = topk_idx.reshape(-1).long()[pair]
            q, s = ref.quant_int8_token(rows, smooth[ids])
        else:
            q, s = ref.quant_int8_token(rows) if rows.numel() else (rows.to(torch.int8), rows.new_zeros((0,), dtype=torch.float32))
        rows, scales = q, s.reshape(-1, 1)
    triple = torch.stack([torch.full_like(tok, g.rank), tok, pair % k], dim=1).to(torch.int32)
    send_splits = [int(counts[d * el:(d + 1) * el].sum()) for d in range(r)]
    recv_splits = [int(cm[s, g.rank * el:(g.rank + 1) * el].sum()) for s in range(r)]
    if g.drop_next_send:
        g.drop_next_send = False
        raise MoeCommTimeout(2, g.rank, 0, -1, "fault injection: this rank withheld its dispatch")
    if rows.dtype == ref.FP8:  # gloo has no fp8: ship the bytes
        recv_rows = g.all_to_all(rows.view(torch.uint8), send_splits, recv_splits).view(ref.FP8)
    else:
        recv_rows = g.all_to_all(rows, send_splits, recv_splits)
    recv_tri = g.all_to_all(triple, send_splits, recv_splits)
    recv_sc = g.all_to_all(scales, send_splits, recv_splits) if scales is not None else None
    # received chunks are source-major / expert-minor; the contract is expert-major / source-minor
    mine = cm[:, g.rank * el:(g.rank + 1) * el]  # [R, E_l]
    starts = torch.zeros(r, el, dtype=torch.long)
    run = 0
    for s in range(r):
        for le in range(el):
            starts[s, le] = run
            run += int(mine[s, le])
    perm = []
    for le in range(el):
        for s in range(r):
            n = int(mine[s, le])
            perm.append(torch.arange(starts[s, le], starts[s, le] + n))
    perm = torch.cat(perm) if perm else torch.zeros(0, dtype=torch.long)
    recv_rows, recv_tri = recv_rows[perm], recv_tri[perm]
    if recv_sc is not None:
        recv_sc = recv_sc[perm]
    recv_count = mine.t().reshape(-1).cumsum(0).to(torch.int32)
    per_expert = mine.sum(dim=0).to(torch.int64)
    g.stats["dispatch_calls"] += 1
    g.stats["rows_sent"] += int(pair.numel())
    g.last_src = recv_tri
    return recv_rows, recv_sc, recv_tri, recv_count, per_expert, ref.slots_in_expert(topk_idx, e_total, active)


def combine(g: CpuGroup, y: torch.Tensor, src: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
            out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y [N,h] expert outputs in receive order, src [N,3] -> out [T,h] (fp32 sum in k order)."""
    r = g.world
    t, k = topk_idx.shape
    n = src.shape[0]
    y = y[:n]
    order = torch.argsort(src[:, 0].long(), stable=True)
    send_splits = torch.bincount(src[:, 0].long(), minlength=r).tolist() if n else [0] * r
    splits_all = g.all_gather(torch.tensor(send_splits, dtype=torch.long))  # [R(src of y), R(dest)]
    recv_splits = splits_all[:, g.rank].tolist()
    rows = g.all_to_all(y[order], send_splits, recv_splits)
    meta = g.all_to_all(src[order][:, 1:].contiguous(), send_splits, recv_splits)
    buf = torch.zeros(t, k, y.shape[1], dtype=y.dtype)
    if rows.shape[0]:
        buf[meta[:, 0].long(), meta[:, 1].long()] = rows
    g.stats["combine_calls"] += 1
    if y.dtype == torch.bfloat16:
        return ref.combine_reference(buf, topk_idx, topk_weights, g.num_experts)
    idx = topk_idx.long()
    ok = ((idx >= 0) & (idx < g.num_experts)).to(torch.float32)
    out = (buf.float() * (topk_weights.float() * ok).unsqueeze(-1)).sum(dim=1)
    return out.to(out_dtype or y.dtype)
