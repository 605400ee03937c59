"""Property tests (hypothesis) of the routing / layout contracts on the CPU oracle and the CPU ops:
random token counts, expert counts, rank counts, top-k, skipped (-1) ids, empty experts and
everything-to-one-expert routing."""
import torch
from hypothesis import given, settings, strategies as st

import umdk_original_b200 as u  # noqa: F401  (registers the ops)
from umdk_original_b200.ops import reference as ref

ops = torch.ops.umdk_cam_op_lib


@st.composite
def routing(draw):
    ranks = draw(st.sampled_from([1, 2, 4]))
    el = draw(st.integers(1, 4))
    e = ranks * el
    k = draw(st.integers(1, min(4, e)))
    t = draw(st.integers(0, 24))
    mode = draw(st.sampled_from(["random", "one_expert", "with_skips"]))
    seed = draw(st.integers(0, 2 ** 16))
    g = torch.Generator().manual_seed(seed)
    per_rank = []
    for _ in range(ranks):
        if mode == "one_expert":
            ids = torch.full((t, k), e - 1, dtype=torch.int64)
        else:
            ids = torch.randint(-1 if mode == "with_skips" else 0, e, (t, k), generator=g)
        per_rank.append(ids)
    return ranks, e, k, t, per_rank


@settings(max_examples=60, deadline=None)
@given(routing())
def test_layout_counts_are_consistent(case):
    ranks, e, k, t, per_rank = case
    for ids in per_rank:
        per_rank_cnt, per_expert, in_rank = ops.get_dispatch_layout(ids, e, ranks)
        valid = (ids >= 0) & (ids < e)
        assert int(per_expert.sum()) == int(valid.sum())
        assert torch.equal(per_rank_cnt, in_rank.sum(dim=0).to(torch.int32))
        el = e // ranks
        for r in range(ranks):
            want = ((ids // el == r) & valid).any(dim=1)
            assert torch.equal(in_rank[:, r], want)


@settings(max_examples=60, deadline=None)
@given(routing())
def test_dispatch_plan_is_a_permutation_of_the_valid_pairs(case):
    ranks, e, k, t, per_rank = case
    plans = ref.plan_dispatch(per_rank, e)
    el = e // ranks
    seen = set()
    for dst, plan in enumerate(plans):
        # counts: inclusive cumsum, expert major / source minor; rows grouped accordingly
        assert plan.recv_count.numel() == el * ranks
        assert int(plan.per_expert.sum()) == plan.src.shape[0]
        if plan.recv_count.numel():
            assert int(plan.recv_count[-1]) == plan.src.shape[0]
        prev = (-1, -1, -1, -1)
        for row, (s, tok, kk) in enumerate(plan.src.tolist()):
            ex = int(per_rank[s][tok, kk])
            assert ex // el == dst
            key = (ex % el, s, tok, kk)
            assert key > prev  # local expert, then source rank, then scan order
            prev = key
            seen.add((s, tok, kk))
    total_valid = sum(int(((ids >= 0) & (ids < e)).sum()) for ids in per_rank)
    assert len(seen) == total_valid


@settings(max_examples=40, deadline=None)
@given(routing())
def test_slots_count_earlier_pairs_of_the_same_expert(case):
    ranks, e, k, t, per_rank = case
    ids = per_rank[0]
    slots = ref.slots_in_expert(ids, e).view(t, k) if t else torch.zeros(0, k, dtype=torch.int32)
    flat = ids.reshape(-1).tolist()
    for i, ex in enumerate(flat):
        want = -1 if not (0 <= ex < e) else sum(1 for j in range(i) if flat[j] == ex)
        assert int(slots.reshape(-1)[i]) == want


@settings(max_examples=30, deadline=None)
@given(st.integers(1, 6), st.integers(1, 3), st.integers(0, 2 ** 16))
def test_ue8m0_scales_bound_the_block(rows, blocks, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, blocks * 128, generator=g) * torch.exp(torch.randn(rows, 1, generator=g) * 3)
    q, s = ref.quant_fp8_1x128(x, ue8m0=True)
    assert ref.is_power_of_two(s)
    amax = x.view(rows, blocks, 128).abs().amax(-1).clamp_min(1e-4)
    assert (s * 448.0 >= amax * (1 - 1e-6)).all() and (s * 448.0 < 2.0 * amax * (1 + 1e-6)).all()
    back = ref.dequant_fp8_1x128(q, s)
    assert ((back - x).abs() <= 0.0725 * amax.unsqueeze(-1).expand(rows, blocks, 128).reshape(rows, -1) + 1e-6).all()


def test_power_of_two_scale_conversion_keeps_values_within_one_e4m3_rounding():
    """Arbitrary fp32 block scales -> powers of two: dequantised weights move by at most one e4m3
    half-ulp (2^-4 relative for normal numbers), already-converted weights do not move at all."""
    import torch
    from umdk_original_b200.models.weights import random_fp8_experts
    from umdk_original_b200.ops import reference as ref
    w = random_fp8_experts(2, 256, 128, ue8m0=False, seed=3)
    assert not w.power_of_two_scales
    c = w.with_power_of_two_scales()
    assert c.power_of_two_scales
    for (q0, s0), (q1, s1) in (((w.w1, w.s1), (c.w1, c.s1)), ((w.w2, w.s2), (c.w2, c.s2))):
        assert bool((s1 >= s0).all()) and bool((s1 < 2 * s0).all())
        a, b = ref.dequant_fp8_128x128(q0, s0), ref.dequant_fp8_128x128(q1, s1)
        # e4m3: 3 mantissa bits -> half an ulp is 2^-4 of the value; subnormals of the new grid are absolute
        tol = a.abs() * 2.0 ** -4 + (s1 * 2.0 ** -10).repeat_interleave(128, -2).repeat_interleave(128, -1)
        assert bool(((a - b).abs() <= tol).all())
    again = c.with_power_of_two_scales()
    assert torch.equal(again.w1.view(torch.uint8), c.w1.view(torch.uint8)) and torch.equal(again.s1, c.s1)
    assert torch.equal(again.w2.view(torch.uint8), c.w2.view(torch.uint8)) and torch.equal(again.s2, c.s2)
