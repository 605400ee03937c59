"""``FusedMoE``: an expert-parallel MoE layer on top of ``fused_deep_moe``.

What a user of the reference writes by hand around ``torch.ops.umdk_cam_op_lib.fused_deep_moe``
(the FusionOp class of test/cam/ut/fused_deep_moe/test_fused_deep_moe.py:199-267): keep the
local experts' quantised weights, route, call the op.  ``MoEStepRunner`` adds the host side of a
serving step: inputs arrive in pinned host memory, are copied to the device on a side stream
while the previous step computes, and a small result record is read back.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..ops import cam_ops
from ..parallel.buffer import Buffer
from ..utils.config import CamConfig
from ..utils.nvtx import nvtx_range
from .configs import MoEConfig
from .router import route
from .weights import ExpertWeights, from_reference_w8a8, random_fp8_experts, random_w8a8_experts


class FusedMoE(torch.nn.Module):
    def __init__(self, cfg: MoEConfig, buffer: Buffer, weights: Optional[ExpertWeights] = None, seed: int = 0,
                 gate_weight: Optional[torch.Tensor] = None, exact_w8a8: bool = False,
                 convert_scales: bool = False):
        """``convert_scales``: fp8 weights that arrive with arbitrary fp32 block scales are moved onto
        power-of-two scales once here (``ExpertWeights.with_power_of_two_scales``), so that the layer runs the
        tensor-core block-scaled GEMMs (``quantMode=4``) instead of the software-scaled ones (``quantMode=3``)."""
        super().__init__()
        self.cfg, self.buffer = cfg, buffer
        self.rank, self.num_ranks = buffer.rank, buffer.num_ranks
        assert cfg.num_experts % self.num_ranks == 0
        self.num_local = cfg.num_experts // self.num_ranks
        dev = buffer.device
        if weights is None and cfg.weight_format == "w8a8" and exact_w8a8:
            # the reference's own arithmetic: int8 weights [E_l, h, 2I] / [E_l, I, h] with per-channel scales,
            # per-token int8 activations, int32 accumulation on the tensor cores (quantMode 0)
            parts = [random_w8a8_experts(min(8, self.num_local - i), cfg.hidden, cfg.intermediate, device=dev,
                                         seed=seed * 1000 + self.rank * 64 + i) for i in range(0, self.num_local, 8)]
            weights = ExpertWeights(*[torch.cat([p[j] for p in parts]) for j in range(4)])
        if weights is None and cfg.weight_format == "w8a8":
            # int8-range weights with per-output-channel scales in the reference's layout, computed as
            # block-scaled fp8 (weights in [-16, 16] are exact in e4m3; the channel scales fold into
            # the 128x128 block scales)
            parts = []
            for i in range(0, self.num_local, 8):
                n = min(8, self.num_local - i)
                parts.append(from_reference_w8a8(*random_w8a8_experts(n, cfg.hidden, cfg.intermediate, device=dev,
                                                                      seed=seed * 1000 + self.rank * 64 + i)))
            weights = ExpertWeights(*[torch.cat([getattr(p, f) for p in parts]) for f in ("w1", "s1", "w2", "s2")])
        if weights is None:
            weights = random_fp8_experts(self.num_local, cfg.hidden, cfg.intermediate, device=dev,
                                         seed=seed * 1000 + self.rank)
        self.weights = weights.to(dev)
        if convert_scales and self.weights.w1.dtype != torch.int8 and not self.weights.power_of_two_scales:
            self.weights = self.weights.with_power_of_two_scales()
        # 0: int8 W8A8 in the reference's layout; 4: fp8 with power-of-two scales -> tcgen05 block-scaled
        # GEMMs; 3: fp8 with arbitrary fp32 scales
        if self.weights.w1.dtype == torch.int8:
            self.quant_mode = 0
        else:
            self.quant_mode = 4 if self.weights.power_of_two_scales else 3
        if gate_weight is None:
            g = torch.Generator(device="cpu")
            g.manual_seed(seed + 17)
            gate_weight = torch.randn(cfg.num_experts, cfg.hidden, generator=g) * 0.02
        self.register_buffer("gate_weight", gate_weight.to(dev, torch.bfloat16))

    def route(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        logits = x @ self.gate_weight.t()
        return route(logits, self.cfg.topk, self.cfg.num_groups, self.cfg.topk_groups)

    def forward(self, x: torch.Tensor, topk_idx: Optional[torch.Tensor] = None,
                topk_weights: Optional[torch.Tensor] = None, x_active_mask: Optional[torch.Tensor] = None):
        """x [T, h] bf16 -> (out [T, h] bf16, tokens per local expert [E_l] int64)."""
        if topk_idx is None:
            topk_idx, topk_weights = self.route(x)
        w = self.weights
        with nvtx_range("umdk_cam.fused_deep_moe"):
            out, nums = cam_ops.ops.fused_deep_moe(
                x, topk_idx, [w.w1], [w.s1], [w.w2], [w.s2], topk_weights.float(), None, x_active_mask,
                self.buffer.name, self.num_ranks, self.rank, self.cfg.num_experts, 0, 0, self.quant_mode, 0)
        return out, nums


class MoEStepRunner:
    """End-to-end step: pinned host inputs -> H2D -> FusedMoE -> D2H of the step's result.

    Two device input slots and two host result slots alternate; the copy of step i+1 runs on a side
    stream while step i computes, the result of step i leaves on a third stream while step i+1 computes,
    and the host may launch step i+1 before it reads the result of step i (``run`` returns a ticket,
    ``result(ticket)`` waits for that step only), so the device does not idle while the host reads a
    result and prepares the next launch.  What is read back each step is the layer's output ``[T, h]``
    in bf16 (``copy_output=False``: nothing of it) plus a small record: the per-expert token counts and
    the sum of the output in fp32 (a checksum a caller can log); ``h2d_bytes`` / ``d2h_bytes`` are what
    moves per step."""

    def __init__(self, layer: FusedMoE, tokens: int, copy_output: bool = True, time_copies: bool = False):
        self.layer = layer
        # time_copies: CUDA events round every host<->device copy (on the copy streams, so they cost the
        # pipeline nothing); ``copy_times()`` then says how long this rank's copies took per step
        self.time_copies = time_copies
        self._copy_events = {"h2d": [], "d2h": []}
        cfg, dev = layer.cfg, layer.buffer.device
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.d2h_stream = torch.cuda.Stream(device=dev)
        self.copy_output = copy_output
        self.slots = []
        for _ in range(2):
            self.slots.append({
                "x": torch.empty(tokens, cfg.hidden, dtype=torch.bfloat16, device=dev),
                "idx": torch.empty(tokens, cfg.topk, dtype=torch.int64, device=dev),
                "w": torch.empty(tokens, cfg.topk, dtype=torch.float32, device=dev),
                "ready": torch.cuda.Event(), "free": torch.cuda.Event(),
            })
        self.result_dev = [torch.zeros(layer.num_local + 1, dtype=torch.float32, device=dev) for _ in range(2)]
        self.result_host = [torch.zeros(layer.num_local + 1, dtype=torch.float32).pin_memory() for _ in range(2)]
        self.out_host = [torch.empty(tokens, cfg.hidden, dtype=torch.bfloat16).pin_memory() if copy_output else None
                         for _ in range(2)]
        self.computed = [torch.cuda.Event(), torch.cuda.Event()]
        self.result_done = [torch.cuda.Event(), torch.cuda.Event()]
        self.h2d_bytes = tokens * (cfg.hidden * 2 + cfg.topk * 8 + cfg.topk * 4)
        self.d2h_bytes = (layer.num_local + 1) * 4 + (tokens * cfg.hidden * 2 if copy_output else 0)
        self._step = 0
        self._staged = None

    def stage(self, x_host: torch.Tensor, idx_host: torch.Tensor, w_host: torch.Tensor) -> None:
        """Starts the host->device copy of the next step's inputs (pinned tensors)."""
        slot = self.slots[self._step % 2]
        with nvtx_range("umdk_cam.step.h2d"), torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(slot["free"])
            ev = self._timed("h2d", self.copy_stream)
            slot["x"].copy_(x_host, non_blocking=True)
            slot["idx"].copy_(idx_host, non_blocking=True)
            slot["w"].copy_(w_host, non_blocking=True)
            if ev is not None:
                ev[1].record(self.copy_stream)
            slot["ready"].record(self.copy_stream)
        self._staged = slot

    def run(self) -> int:
        """Launches the staged step (nothing here waits for the device) and returns its ticket.  At most
        two steps may be outstanding: collect ``result(ticket)`` of a step before launching the step after
        the next one, whose result takes the same place."""
        slot = self._staged
        cur = torch.cuda.current_stream()
        cur.wait_event(slot["ready"])
        out, nums = self.layer(slot["x"], slot["idx"], slot["w"])
        slot["free"].record(cur)
        r = self._step % 2
        self.result_dev[r][:-1] = nums.float()
        self.result_dev[r][-1] = out.sum(dtype=torch.float32)
        self.computed[r].record(cur)
        with nvtx_range("umdk_cam.step.result_d2h"), torch.cuda.stream(self.d2h_stream):
            self.d2h_stream.wait_event(self.computed[r])
            ev = self._timed("d2h", self.d2h_stream)
            if self.copy_output:
                self.out_host[r].copy_(out, non_blocking=True)
                out.record_stream(self.d2h_stream)
            self.result_host[r].copy_(self.result_dev[r], non_blocking=True)
            if ev is not None:
                ev[1].record(self.d2h_stream)
            self.result_done[r].record(self.d2h_stream)
        ticket = self._step
        self._step += 1
        self.last_out = out
        return ticket

    def _timed(self, kind: str, stream):
        if not self.time_copies:
            return None
        pair = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        pair[0].record(stream)
        self._copy_events[kind].append(pair)
        return pair

    def copy_times(self, reset: bool = True) -> dict:
        """Mean milliseconds per step of this rank's host->device and device->host copies since the last call
        (``time_copies=True``); synchronises both copy streams."""
        self.copy_stream.synchronize()
        self.d2h_stream.synchronize()
        out = {}
        for kind, pairs in self._copy_events.items():
            out[kind + "_ms"] = sum(a.elapsed_time(b) for a, b in pairs) / len(pairs) if pairs else 0.0
        if reset:
            self._copy_events = {"h2d": [], "d2h": []}
        return out

    def result(self, ticket: int) -> torch.Tensor:
        """Host record of the step with this ticket (waits for that step only); the step's output is then
        in ``output(ticket)``."""
        assert self._step - 2 <= ticket < self._step, "the result of this step has been overwritten or not produced"
        self.result_done[ticket % 2].synchronize()
        return self.result_host[ticket % 2]

    def output(self, ticket: int) -> Optional[torch.Tensor]:
        """Pinned host copy of the step's output (valid after ``result(ticket)``, until two steps later)."""
        return self.out_host[ticket % 2]

    def finish(self) -> torch.Tensor:
        """Waits for everything launched and returns the record of the last step."""
        torch.cuda.current_stream().synchronize()
        self.d2h_stream.synchronize()
        return self.result_host[(self._step - 1) % 2]


def make_buffer_for(cfg: MoEConfig, group=None, tokens: Optional[int] = None, capacity_factor: float = 0.0,
                    ll_max_tokens: int = 0, name: Optional[str] = None, device=None, timeout_ms: float = 10000.0) -> Buffer:
    cam_cfg = CamConfig(num_experts=cfg.num_experts, max_tokens=tokens or cfg.tokens_per_rank, hidden=cfg.hidden,
                        topk=cfg.topk, capacity_factor=capacity_factor, ll_max_tokens=ll_max_tokens,
                        timeout_ms=timeout_ms)
    return Buffer(group, cam_cfg, name=name, device=device)
