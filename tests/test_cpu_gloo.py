"""CPU plumbing on gloo (world_size 2): the op surface end to end, checked against the oracle.
Covers the first benchmark configuration: 128 tokens/rank, hidden 1024, 8 experts top-2, SwiGLU
with intermediate 512, against a single-process dense MoE with seed 0."""
import pytest
import torch

from conftest import run_gloo

pytestmark = pytest.mark.multi_process_test


def _make_inputs(seed, world, t, h, e, k, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn(t, h, generator=g).to(dtype) for _ in range(world)]
    logits = [torch.randn(t, e, generator=g) for _ in range(world)]
    return xs, logits, g


def _config1_rank(rank, world):
    import torch
    import umdk_original_b200 as u
    from umdk_original_b200.models import topk_softmax
    from umdk_original_b200.ops import reference as ref
    t, h, e, k, inter = 128, 1024, 8, 2, 512
    xs, logits, g = _make_inputs(0, world, t, h, e, k)
    w1 = torch.randn(e, 2 * inter, h, generator=g) * 0.02
    w2 = torch.randn(e, h, inter, generator=g) * 0.02
    buf = u.Buffer(None, u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k), name="cfg1",
                   device=torch.device("cpu"))
    idx, wt = topk_softmax(logits[rank], k)
    el = e // world
    lo = rank * el
    out, nums = torch.ops.umdk_cam_op_lib.fused_deep_moe(
        xs[rank], idx, [w1[lo:lo + el]], [torch.empty(0)], [w2[lo:lo + el]], [torch.empty(0)], wt, None, None,
        "cfg1", world, rank, e, 0, 0, 0, 0)
    dense = ref.dense_moe_fp32(xs[rank], idx, wt, w1, w2)
    # tokens per local expert counted over all ranks' routing
    want = torch.zeros(el, dtype=torch.int64)
    for r in range(world):
        ir, _ = topk_softmax(logits[r], k)
        for le in range(el):
            want[le] += int((ir == lo + le).sum())
    return float((out - dense).abs().max()), nums.tolist(), want.tolist()


def test_config1_dense_equivalence():
    res = run_gloo(_config1_rank, 2)
    assert len(res) == 2
    for r, (st, val) in res.items():
        assert st == "ok", val
        err, nums, want = val
        assert err < 1e-4, f"rank {r}: max abs err {err}"
        assert nums == want


def _dispatch_combine_rank(rank, world, quant_mode):
    import torch
    import umdk_original_b200 as u
    from umdk_original_b200.ops import reference as ref
    t, h, e, k = 40, 256, 8, 3
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(t, h, generator=g).to(torch.bfloat16) for _ in range(world)]
    topk = [torch.randint(-1, e, (t, k), generator=g) for _ in range(world)]
    wts = [torch.rand(t, k, generator=g) for _ in range(world)]
    buf = u.Buffer(None, u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k), name="dc", device=torch.device("cpu"))
    ops = torch.ops.umdk_cam_op_lib
    nr, ne, inr = ops.get_dispatch_layout(topk[rank], e, world)
    rx, src, cnt, per_e, rs = ops.moe_dispatch_prefill_quant(xs[rank], topk[rank], wts[rank], 0, "dc", rank, world, quant_mode)
    plan = ref.plan_dispatch(topk, e)[rank]
    assert torch.equal(src.reshape(-1, 3), plan.src)
    assert torch.equal(cnt, plan.recv_count)
    assert torch.equal(per_e, plan.per_expert)
    rows = torch.stack([xs[s][tt] for s, tt, _ in plan.src.tolist()]) if plan.src.shape[0] else rx
    if quant_mode == 0:
        assert torch.equal(rx, rows)
        y = rx
    else:
        q, s = ref.quant_fp8_1x128(rows)
        assert torch.equal(rx.view(torch.uint8), q.view(torch.uint8)) and torch.equal(rs, s)
        y = ref.dequant_fp8_1x128(rx, rs).to(torch.bfloat16)
    out = ops.moe_combine_prefill(y, topk[rank], wts[rank], src, cnt, "dc", rank, world)
    pair_rows = y.new_zeros(t, k, h)
    idx = topk[rank]
    xin = xs[rank] if quant_mode == 0 else ref.dequant_fp8_1x128(*ref.quant_fp8_1x128(xs[rank])).to(torch.bfloat16)
    for kk in range(k):
        pair_rows[:, kk] = xin
    want = ref.combine_reference(pair_rows, idx, wts[rank], e)
    return float((out.float() - want.float()).abs().max())


@pytest.mark.parametrize("quant_mode", [0, 3])
def test_dispatch_combine_contract(quant_mode):
    res = run_gloo(_dispatch_combine_rank, 2, args=(quant_mode,))
    assert len(res) == 2
    for r, (st, val) in res.items():
        assert st == "ok", val
        assert val == 0.0


def _ll_rank(rank, world):
    import torch
    import umdk_original_b200 as u
    from umdk_original_b200.ops import reference as ref
    t, h, e, k = 16, 128, 4, 2
    g = torch.Generator().manual_seed(9)
    xs = [torch.randn(t, h, generator=g).to(torch.bfloat16) for _ in range(world)]
    topk = [torch.randint(0, e, (t, k), generator=g).to(torch.int32) for _ in range(world)]
    wts = [torch.rand(t, k, generator=g) for _ in range(world)]
    buf = u.Buffer(None, u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, ll_max_tokens=t), name="ll",
                   device=torch.device("cpu"))
    ops = torch.ops.umdk_cam_op_lib
    mask = torch.zeros(t, dtype=torch.bool)
    mask[:12] = True
    outs = ops.moe_dispatch_shmem(xs[rank], topk[rank], None, mask, world, rank, e, 1, 0, 0, 0, 0, 0, 0, 1, buf.handle)
    expand, dyn, eidx, nums, ep_cnt, tp_cnt = outs
    masked = [tk.clone() for tk in topk]
    for m in masked:
        m[12:] = -1
    plan = ref.plan_dispatch(masked, e)[rank]
    n = plan.src.shape[0]
    assert expand.shape[0] == t * world * min(e // world, k)
    assert torch.equal(ep_cnt, plan.recv_count) and torch.equal(nums, plan.per_expert)
    assert torch.equal(eidx, ref.slots_in_expert(topk[rank], e, 12))
    rows = torch.stack([xs[s][tt] for s, tt, _ in plan.src.tolist()])
    assert torch.equal(expand[:n], rows)
    out = ops.moe_combine_shmem(expand, topk[rank], eidx, ep_cnt, wts[rank], None, mask, None, None, None, None,
                                world, rank, e, 1, 0, 0, 0, 0, 0, 0, buf.handle, 0, 0)
    pair_rows = xs[rank].unsqueeze(1).expand(t, k, h).contiguous()
    want = ref.combine_reference(pair_rows, masked[rank], wts[rank], e)
    return float((out.float() - want.float()).abs().max())


def test_low_latency_ops_with_active_mask():
    res = run_gloo(_ll_rank, 2)
    assert len(res) == 2
    for r, (st, val) in res.items():
        assert st == "ok", val
        assert val == 0.0


def _fault_rank(rank, world):
    """Rank 1 raises before its dispatch; rank 0 must get MoeCommTimeout, not hang."""
    import torch
    import umdk_original_b200 as u
    t, h, e, k = 8, 128, 4, 2
    buf = u.Buffer(None, u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k), name="flt", device=torch.device("cpu"))
    x = torch.randn(t, h).to(torch.bfloat16)
    idx = torch.randint(0, e, (t, k))
    w = torch.rand(t, k)
    if rank == 1:
        buf.inject_drop_flags(True)
    try:
        torch.ops.umdk_cam_op_lib.moe_dispatch_prefill_quant(x, idx, w, 0, "flt", rank, world, 0)
    except u.MoeCommTimeout as e2:
        return "timeout:" + str(e2.code)
    return "completed"


def test_fault_injection_rank_withholds_dispatch():
    res = run_gloo(_fault_rank, 2, timeout_s=8)
    assert len(res) == 2
    for r, (st, val) in res.items():
        assert st == "ok", val
        assert val.startswith("timeout"), f"rank {r}: {val}"


def _shared_rank_fused(rank, world):
    """2 ranks: rank 0 holds the shared expert, rank 1 the 4 routed experts (float weights, CPU path)."""
    import torch
    import umdk_original_b200 as u
    from umdk_original_b200.models import topk_softmax
    from umdk_original_b200.ops import reference as ref
    t, h, e, k, inter, shared = 32, 256, 4, 2, 128, 1
    xs, logits, g = _make_inputs(3, world, t, h, e, k)
    w1 = torch.randn(e, 2 * inter, h, generator=g) * 0.05
    w2 = torch.randn(e, h, inter, generator=g) * 0.05
    sw1 = torch.randn(1, 2 * inter, h, generator=g) * 0.05
    sw2 = torch.randn(1, h, inter, generator=g) * 0.05
    el = e // (world - shared)
    buf = u.Buffer(None, u.CamConfig(num_experts=el * world, max_tokens=t, hidden=h, topk=k + 1), name="shf",
                   device=torch.device("cpu"))
    idx, wt = topk_softmax(logits[rank], k)
    mine1, mine2 = (sw1, sw2) if rank < shared else (w1, w2)
    out, nums = torch.ops.umdk_cam_op_lib.fused_deep_moe(
        xs[rank], idx, [mine1], [torch.empty(0)], [mine2], [torch.empty(0)], wt, None, None, "shf", world, rank, e,
        1, shared, 0, 0)
    want = ref.dense_moe_fp32(xs[rank], idx, wt, w1, w2) + ref.swiglu_mlp_fp32(xs[rank], sw1[0], sw2[0])
    return float((out - want).abs().max()), nums.tolist()


def test_fused_with_shared_expert_rank():
    res = run_gloo(_shared_rank_fused, 2)
    assert len(res) == 2
    for r, (st, val) in res.items():
        assert st == "ok", val
        err, nums = val
        assert err < 1e-4, f"rank {r}: max abs err {err}"
        assert len(nums) == (1 if r == 0 else 4)
    assert res[0][1][1][0] == 64  # the replica sees every token of both ranks once


def _tp_rank(rank, world):
    """EP 2 x TP 2 on four gloo ranks (rank = tp * 2 + ep): dispatch appends the TP partner's rows,
    combine adds both partial outputs of every row before sending it home."""
    import torch
    import torch.distributed as dist
    import umdk_original_b200 as u
    from umdk_original_b200.ops import reference as ref
    ops = torch.ops.umdk_cam_op_lib
    ep, t, h, e, k = 2, 16, 256, 4, 2
    tp, r = divmod(rank, ep)
    ep_groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]
    tp_groups = [dist.new_group([0, 2]), dist.new_group([1, 3])]
    g = torch.Generator().manual_seed(123)
    xs = [torch.randn(t, h, generator=g).to(torch.bfloat16) for _ in range(world)]
    topk = [torch.randint(0, e, (t, k), generator=g).to(torch.int32) for _ in range(world)]
    wts = [torch.rand(t, k, generator=g) for _ in range(world)]
    buf = u.Buffer(ep_groups[tp], u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, ll_max_tokens=t),
                   name="tp", device=torch.device("cpu"), tp_group=tp_groups[r])
    expand, dyn, eidx, nums, ep_cnt, tp_cnt = ops.moe_dispatch_shmem(
        xs[rank], topk[rank], None, None, ep, r, e, 2, tp, 0, 0, 0, 3, 0, 1, buf.handle)
    plans = [ref.plan_dispatch([topk[p * ep + q] for q in range(ep)], e) for p in range(2)]
    own, other = plans[tp][r], plans[1 - tp][r]
    n, m = own.src.shape[0], other.src.shape[0]
    assert tp_cnt.tolist() == ([n, m] if tp == 0 else [m, n]), (tp_cnt.tolist(), n, m)
    assert expand.shape[0] == 2 * t * ep * min(e // ep, k) and dyn.shape == (expand.shape[0], h // 128)
    own_rows = torch.stack([xs[tp * ep + s][tt] for s, tt, _ in own.src.tolist()])
    oth_rows = torch.stack([xs[(1 - tp) * ep + s][tt] for s, tt, _ in other.src.tolist()])
    for rows, lo in ((own_rows, 0), (oth_rows, n)):
        q, s = ref.quant_fp8_1x128(rows)
        assert torch.equal(expand[lo:lo + rows.shape[0]].view(torch.uint8), q.view(torch.uint8))
        assert torch.equal(dyn[lo:lo + rows.shape[0]], s)
    # a TP-sharded expert: this rank's partial output of every row it holds is (1 + tp) * row
    both = torch.cat([own_rows, oth_rows])
    y = torch.zeros(expand.shape[0], h, dtype=torch.bfloat16)
    y[:n + m] = (both.float() * (1.0 + tp)).to(torch.bfloat16)
    out = ops.moe_combine_shmem(y, topk[rank], eidx, ep_cnt, wts[rank], tp_cnt, None, None, None, None, None,
                                ep, r, e, 2, tp, 0, 0, 0, 0, 0, buf.handle, 0, 0)
    rows3 = (xs[rank].float() * 1.0).to(torch.bfloat16).float() + (xs[rank].float() * 2.0).to(torch.bfloat16).float()
    want = ref.combine_reference(rows3.to(torch.bfloat16).unsqueeze(1).expand(t, k, h).contiguous(), topk[rank],
                                 wts[rank], e)
    return float((out.float() - want.float()).abs().max())


def test_low_latency_ops_with_tensor_parallel_pair():
    res = run_gloo(_tp_rank, 4)
    assert len(res) == 4
    for r, (st, val) in res.items():
        assert st == "ok", val
        assert val == 0.0


def test_fp16_activations_are_accepted_and_returned_as_fp16():
    """The reference's fused op and low-latency ops take bf16 or fp16 rows (fused_deep_moe.cpp:17-19).  One rank on
    the CPU: fp16 input gives fp16 output equal to the bf16 path's result (the layer computes on bf16 rows)."""
    import torch
    import umdk_original_b200 as u
    from umdk_original_b200.ops import reference as ref
    ops = torch.ops.umdk_cam_op_lib
    t, h, e, k, inter = 16, 256, 4, 2, 128
    g = torch.Generator().manual_seed(0)
    buf = u.Buffer(None, u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, ll_max_tokens=t), name="h16",
                   device=torch.device("cpu"))
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)   # values both 16-bit formats hold exactly after this cast
    x = (x.float() * 0.5).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)])
    w = torch.softmax(torch.randn(t, k, generator=g), -1)
    w1q, s1 = ref.quant_fp8_128x128(torch.randn(e, 2 * inter, h, generator=g) * 0.05, True)
    w2q, s2 = ref.quant_fp8_128x128(torch.randn(e, h, inter, generator=g) * 0.05, True)
    outs = {}
    for dt in (torch.bfloat16, torch.float16):
        out, nums = ops.fused_deep_moe(x.to(dt), idx, [w1q], [s1], [w2q], [s2], w, None, None, "h16", 1, 0, e, 0, 0, 4, 0)
        assert out.dtype == dt and out.shape == (t, h)
        outs[dt] = out.float()
        idx32 = idx.to(torch.int32)
        r = ops.moe_dispatch_shmem(x.to(dt), idx32, None, None, 1, 0, e, 1, 0, 0, 0, 0, 0, 0, 1, buf.handle)
        o = ops.moe_combine_shmem(r[0], idx32, r[2], r[4], w, None, None, None, None, None, None, 1, 0, e, 1, 0, 0, 0, 0,
                                  0, 0, buf.handle, 0, 0)
        assert r[0].dtype == dt and o.dtype == dt
    # bf16 rows survive the trip through fp16 here (|x| < 4, 8 mantissa bits fit in fp16's 11), so both runs saw the
    # same rows; the fp16 result is the bf16 result rounded once more
    assert (outs[torch.float16] - outs[torch.bfloat16]).abs().max() <= 1e-2 * outs[torch.bfloat16].abs().max()
    buf.destroy()
