"""The CPU oracle itself: quantisation round trips, layout and dispatch-order contracts."""
import torch
from hypothesis import given, settings, strategies as st

from umdk_original_b200.ops import reference as ref


def test_fp8_1x128_roundtrip():
    torch.manual_seed(0)
    x = torch.randn(16, 512)
    q, s = ref.quant_fp8_1x128(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (16, 4)
    back = ref.dequant_fp8_1x128(q, s)
    assert (back - x).abs().max() <= x.abs().max() * 0.07
    # all-zero rows stay finite (the reference divides by the row max without a guard: GMM1.h:804)
    q0, s0 = ref.quant_fp8_1x128(torch.zeros(2, 128))
    assert torch.isfinite(s0).all() and (q0.float() == 0).all()


def test_fp8_128x128_roundtrip():
    torch.manual_seed(1)
    w = torch.randn(2, 256, 384) * 0.02
    q, s = ref.quant_fp8_128x128(w)
    assert s.shape == (2, 2, 3)
    assert (ref.dequant_fp8_128x128(q, s) - w).abs().max() <= w.abs().max() * 0.07


def test_int8_token_matches_formula():
    x = torch.tensor([[1.0, -2.0, 0.5, 4.0]])
    q, s = ref.quant_int8_token(x)
    assert q.tolist() == [[32, -64, 16, 127]]
    assert abs(s.item() - 4.0 / 127) < 1e-6


def test_layout_counts_and_negative_ids():
    idx = torch.tensor([[0, 5], [5, 6], [-1, 7], [1, 1]])
    per_rank, per_expert, in_rank = ref.get_dispatch_layout(idx, 8, 2)
    assert per_expert.tolist() == [1, 2, 0, 0, 0, 2, 1, 1]
    assert per_rank.tolist() == [2, 3]
    assert in_rank.tolist() == [[True, True], [False, True], [False, True], [True, False]]


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 3), st.integers(1, 12), st.integers(1, 4), st.integers(0, 10 ** 6))
def test_plan_dispatch_properties(log_r, tokens, k, seed):
    r = 1 << (log_r - 1)
    e = r * 3
    g = torch.Generator().manual_seed(seed)
    topk = [torch.randint(-1, e, (tokens, k), generator=g) for _ in range(r)]
    plans = ref.plan_dispatch(topk, e)
    el = e // r
    total_valid = sum(int(((t >= 0) & (t < e)).sum()) for t in topk)
    assert sum(p.src.shape[0] for p in plans) == total_valid
    for dst, p in enumerate(plans):
        assert p.recv_count.numel() == el * r
        assert int(p.expert_offsets[-1]) == p.src.shape[0]
        # every row's expert id really lives on dst, rows are expert-major then source-minor
        keys = []
        for s, t, kk in p.src.tolist():
            eid = int(topk[s][t, kk])
            assert eid // el == dst
            keys.append((eid % el, s, t * k + kk))
        assert keys == sorted(keys)


def test_slots_in_expert_scan_order():
    idx = torch.tensor([[2, 0], [2, 2], [0, -1]])
    assert ref.slots_in_expert(idx, 4).tolist() == [0, 0, 1, 2, 1, -1]
    assert ref.slots_in_expert(idx, 4, active_tokens=1).tolist() == [0, 0, -1, -1, -1, -1]


def test_dense_vs_fp8_layer_close():
    torch.manual_seed(3)
    t, h, i, e, k = 24, 256, 128, 4, 2
    x = torch.randn(t, h).to(torch.bfloat16)
    w1 = torch.randn(e, 2 * i, h) * 0.05
    w2 = torch.randn(e, h, i) * 0.05
    idx = torch.stack([torch.randperm(e)[:k] for _ in range(t)])
    wt = torch.softmax(torch.randn(t, k), -1)
    w1q, s1 = ref.quant_fp8_128x128(w1)
    w2q, s2 = ref.quant_fp8_128x128(w2)
    out, counts = ref.fused_moe_fp8_reference(x, idx, wt, w1q, s1, w2q, s2)
    dense = ref.dense_moe_fp32(x.float(), idx, wt, w1, w2)
    assert counts.sum() == t * k
    assert (out.float() - dense).abs().max() <= 0.1 * dense.abs().max() + 1e-3
