"""Expert weights: random initialisation, quantisation and pre-packing.

Layouts used by the kernels (K-major = the reduction dim is contiguous, what TMA + tcgen05 want):
  w1 [E_local, 2I, h]  gate rows first ("activate_left", test_fused_deep_moe.py:165), e4m3,
                       scales [E_local, 2I/128, h/128]
  w2 [E_local, h, I]   e4m3, scales [E_local, h/128, I/128]
The reference stores int8 weights as [E_local, h, 2I] / [E_local, I, h] in the Ascend NZ fractal
layout with per-output-channel scales (fused_deep_moe.h:59,182; pybind/fused_deep_moe.cpp:26-79);
``from_reference_w8a8`` converts that form.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple, Union

import torch

from ..ops import reference as ref


@dataclass
class ExpertWeights:
    """Local experts of one rank, ready for ``fused_deep_moe(quantMode=3)``."""
    w1: torch.Tensor   # [E_l, 2I, h] e4m3
    s1: torch.Tensor   # [E_l, 2I/128, h/128] fp32
    w2: torch.Tensor   # [E_l, h, I] e4m3
    s2: torch.Tensor   # [E_l, h/128, I/128] fp32

    def to(self, device) -> "ExpertWeights":
        return ExpertWeights(self.w1.to(device), self.s1.to(device), self.w2.to(device), self.s2.to(device))

    @property
    def power_of_two_scales(self) -> bool:
        """True when both scale tensors hold exact powers of two: the layer then runs the
        tensor-core block-scaled path (``quantMode=4``)."""
        return ref.is_power_of_two(self.s1) and ref.is_power_of_two(self.s2)

    def with_power_of_two_scales(self, chunk: int = 4) -> "ExpertWeights":
        """The same experts with every block scale rounded up to a power of two and the e4m3 values
        re-rounded to match (value = q * s is kept up to one more e4m3 rounding; blocks whose scale is a
        power of two already are unchanged).  Checkpoints with arbitrary fp32 block scales run on the
        software-scaled GEMM (``quantMode=3``); after this conversion they take the tensor-core
        block-scaled path (``quantMode=4``)."""
        def convert(q: torch.Tensor, sc: torch.Tensor):
            qs, ss = [], []
            for i in range(0, q.shape[0], chunk):
                s_old = sc[i:i + chunk].float()
                s_new = ref.ue8m0_round_up(s_old)
                ratio = (s_old / s_new).unsqueeze(-1).unsqueeze(-3)          # in (0.5, 1]: no overflow
                e, n, k = q[i:i + chunk].shape
                v = q[i:i + chunk].float().reshape(e, n // 128, 128, k // 128, 128) * ratio
                qs.append(v.to(ref.FP8).reshape(e, n, k))
                ss.append(s_new)
            return torch.cat(qs), torch.cat(ss)
        w1, s1 = convert(self.w1, self.s1)
        w2, s2 = convert(self.w2, self.s2)
        return ExpertWeights(w1, s1, w2, s2)

    @property
    def num_local_experts(self) -> int:
        return self.w1.shape[0]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w1, self.s1, self.w2, self.s2))


def quantize_fp8_block(w: torch.Tensor, chunk: int = 8, ue8m0: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """[E, N, K] float -> (e4m3, fp32 128x128 scales); processed in expert chunks to bound memory.
    ``ue8m0`` rounds the scales up to powers of two (needed by the tensor-core block-scaled path)."""
    qs, ss = [], []
    for i in range(0, w.shape[0], chunk):
        q, s = ref.quant_fp8_128x128(w[i:i + chunk], ue8m0)
        qs.append(q)
        ss.append(s)
    return torch.cat(qs), torch.cat(ss)


def random_fp8_experts(num_local: int, hidden: int, inter: int, device="cpu", std: float = 0.02, seed: int = 0,
                       chunk: int = 4, ue8m0: bool = True) -> ExpertWeights:
    """Random-init N(0, std) experts, quantised to e4m3 with 128x128 block scales (powers of two
    unless ``ue8m0=False``), generated on `device` in chunks so that 256 DeepSeek-sized experts
    never exist in fp32 at once."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w1q, s1, w2q, s2 = [], [], [], []
    for i in range(0, num_local, chunk):
        n = min(chunk, num_local - i)
        a = torch.randn(n, 2 * inter, hidden, device=device, generator=g) * std
        q, s = ref.quant_fp8_128x128(a, ue8m0)
        w1q.append(q)
        s1.append(s)
        b = torch.randn(n, hidden, inter, device=device, generator=g) * std
        q, s = ref.quant_fp8_128x128(b, ue8m0)
        w2q.append(q)
        s2.append(s)
        del a, b
    return ExpertWeights(torch.cat(w1q), torch.cat(s1), torch.cat(w2q), torch.cat(s2))


def random_w8a8_experts(num_local: int, hidden: int, inter: int, device="cpu", seed: int = 0):
    """int8-range weights with per-output-channel scales in the reference's layout
    (randint(-16, 16), scales rand*0.003+0.0015: test_fused_deep_moe.py:290-319)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w1 = torch.randint(-16, 16, (num_local, hidden, 2 * inter), device=device, generator=g, dtype=torch.int8)
    w2 = torch.randint(-16, 16, (num_local, inter, hidden), device=device, generator=g, dtype=torch.int8)
    s1 = torch.rand(num_local, 2 * inter, device=device, generator=g) * 0.003 + 0.0015
    s2 = torch.rand(num_local, hidden, device=device, generator=g) * 0.003 + 0.0015
    return w1, s1, w2, s2


def from_reference_w8a8(w1: torch.Tensor, s1: torch.Tensor, w2: torch.Tensor, s2: torch.Tensor,
                        ue8m0: bool = True) -> ExpertWeights:
    """Reference-format int8 W8A8 weights (w1 [E,h,2I] + s1 [E,2I], w2 [E,I,h] + s2 [E,h]) to the
    block-scaled fp8 form the tensor-core path computes in: dequantise per output channel, then
    requantise per 128x128 block."""
    qs1, ss1, qs2, ss2 = [], [], [], []
    for e in range(w1.shape[0]):
        a = w1[e].t().float() * s1[e].float().unsqueeze(-1)   # [2I, h]
        q, s = ref.quant_fp8_128x128(a, ue8m0)
        qs1.append(q)
        ss1.append(s)
        b = w2[e].t().float() * s2[e].float().unsqueeze(-1)   # [h, I]
        q, s = ref.quant_fp8_128x128(b, ue8m0)
        qs2.append(q)
        ss2.append(s)
    return ExpertWeights(torch.stack(qs1), torch.stack(ss1), torch.stack(qs2), torch.stack(ss2))


def stack_tensor_list(ws: Union[torch.Tensor, Sequence[torch.Tensor]]) -> torch.Tensor:
    """Accepts one stacked tensor or a list of per-expert tensors (the reference's "tensor list"
    form for dynamic expert load balancing, fused_deep_moe_tiling.cpp:83-127)."""
    if isinstance(ws, torch.Tensor):
        return ws
    ws = list(ws)
    if len(ws) == 1 and ws[0].dim() == 3:
        return ws[0]
    return torch.stack(ws).contiguous()
