"""What rounding block scales up to powers of two costs.

The tensor cores' block scaling takes only the exponent of a scale (UE8M0), so the fast path of the fused layer
quantises activations with power-of-two 1x128 scales and expects weights with power-of-two 128x128 scales;
checkpoints that carry arbitrary fp32 scales are converted once (ExpertWeights.with_power_of_two_scales).  A
rounded-up scale wastes at most one bit of the e4m3 range, so the error against the dense fp32 layer may grow,
but only by a bounded factor.  This test pins that factor on the CPU oracle for the whole expert MLP."""
import torch

from umdk_original_b200.models.weights import ExpertWeights
from umdk_original_b200.ops import reference as ref


def _dense(x, w1, w2):
    return ref.swiglu_mlp_fp32(x, w1, w2)


def test_power_of_two_scales_cost_less_than_a_factor_of_two_in_error():
    g = torch.Generator().manual_seed(0)
    n, h, inter = 96, 1024, 512
    x = torch.randn(n, h, generator=g).to(torch.bfloat16)
    w1 = torch.randn(2 * inter, h, generator=g) * 0.02
    w2 = torch.randn(h, inter, generator=g) * 0.02
    want = _dense(x.float(), w1, w2)
    errs = {}
    for ue8m0 in (False, True):
        w1q, s1 = ref.quant_fp8_128x128(w1, ue8m0)
        w2q, s2 = ref.quant_fp8_128x128(w2, ue8m0)
        xq, xs = ref.quant_fp8_1x128(x, ue8m0)
        got = ref.expert_mlp_fp8(xq, xs, w1q, s1, w2q, s2, ue8m0=ue8m0).float()
        errs[ue8m0] = ((got - want).norm() / want.norm()).item()
    # both formats keep the layer within a few percent of the dense result (measured: 6.3 % with fp32 scales, 6.6 % with
    # power-of-two scales: two e4m3 quantisations of the activations and one of each weight matrix) ...
    assert errs[False] < 0.08 and errs[True] < 0.085, errs
    # ... and the power-of-two form costs a few percent of that error, never a multiple
    assert errs[True] <= 1.25 * errs[False], errs


def test_converting_fp32_scales_to_powers_of_two_adds_one_rounding():
    """A checkpoint with fp32 block scales moved onto power-of-two scales: the dequantised weights change by at most
    one e4m3 rounding step (2^-4 relative to a block's largest value) and the layer output moves accordingly."""
    g = torch.Generator().manual_seed(1)
    e, h, inter = 2, 512, 256
    w1 = torch.randn(e, 2 * inter, h, generator=g) * 0.02
    w2 = torch.randn(e, h, inter, generator=g) * 0.02
    w1q, s1 = ref.quant_fp8_128x128(w1, False)
    w2q, s2 = ref.quant_fp8_128x128(w2, False)
    a = ExpertWeights(w1q, s1, w2q, s2)
    b = a.with_power_of_two_scales()
    assert ref.is_power_of_two(b.s1) and ref.is_power_of_two(b.s2)
    d1a, d1b = ref.dequant_fp8_128x128(a.w1, a.s1), ref.dequant_fp8_128x128(b.w1, b.s1)
    blk = d1a.abs().reshape(e, 2 * inter // 128, 128, h // 128, 128).amax(dim=(2, 4), keepdim=True)
    rel = ((d1a - d1b).abs().reshape(e, 2 * inter // 128, 128, h // 128, 128) / blk).max().item()
    assert rel <= 2 ** -4 + 1e-6, rel
    x = torch.randn(64, h, generator=g).to(torch.bfloat16)
    xq, xs = ref.quant_fp8_1x128(x, True)
    ya = ref.expert_mlp_fp8(*ref.quant_fp8_1x128(x, False), a.w1[0], a.s1[0], a.w2[0], a.s2[0], ue8m0=False).float()
    yb = ref.expert_mlp_fp8(xq, xs, b.w1[0], b.s1[0], b.w2[0], b.s2[0], ue8m0=True).float()
    dense = _dense(x.float(), w1[0], w2[0])
    ea, eb = ((ya - dense).norm() / dense.norm()).item(), ((yb - dense).norm() / dense.norm()).item()
    assert eb <= 2.0 * ea + 1e-3, (ea, eb)
