"""GPU tests of the communication kernels: layout, normal dispatch/combine, low-latency
dispatch/combine.  Multi-rank protocols run as R virtual ranks on one GPU, phase by phase, so no
launch ever waits for another launch.  Every check is against the CPU oracle."""
import pytest
import torch

import umdk_original_b200 as u
from umdk_original_b200.ops import reference as ref
from umdk_original_b200.parallel import PHASE_COUNT, PHASE_RECV, PHASE_SEND, run_virtual

pytestmark = pytest.mark.gpu
ops = torch.ops.umdk_cam_op_lib


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32])
def test_layout_kernel(dtype):
    g = torch.Generator().manual_seed(0)
    idx = torch.randint(-1, 64, (777, 8), generator=g).to(dtype)
    got = ops.get_dispatch_layout(idx.to(_dev()), 64, 8)
    want = ref.get_dispatch_layout(idx, 64, 8)
    for a, b in zip(got, want):
        assert torch.equal(a.cpu(), b)


def _inputs(world, t, h, e, k, seed, lo=-1):
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn(t, h, generator=g).to(torch.bfloat16) for _ in range(world)]
    topk = [torch.randint(lo, e, (t, k), generator=g) for _ in range(world)]
    wts = [torch.rand(t, k, generator=g) for _ in range(world)]
    return xs, topk, wts


@pytest.mark.parametrize("world,quant_mode", [(1, 0), (1, 3), (2, 3), (4, 0), (4, 2), (8, 3)])
def test_dispatch_combine_normal(world, quant_mode):
    t, h, e, k = 61, 512, 16, 4
    xs, topk, wts = _inputs(world, t, h, e, k, seed=world * 10 + quant_mode)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=2000.0)
    bufs = u.Buffer.virtual(world, cfg, _dev(), name=f"n{world}q{quant_mode}_")
    dx = [x.to(_dev()) for x in xs]
    dk = [x.to(_dev()) for x in topk]
    dw = [x.to(_dev()) for x in wts]

    def disp(r):
        return ops.moe_dispatch_prefill_quant(dx[r], dk[r], dw[r], 0, bufs[r].name, r, world, quant_mode)

    res = run_virtual(disp, world, masks=(PHASE_COUNT, PHASE_SEND, PHASE_RECV))
    plans = ref.plan_dispatch(topk, e)
    ys = []
    for r in range(world):
        bufs[r].check()
        rx, src, cnt, per_e, rs = res[r]
        plan = plans[r]
        assert torch.equal(src.cpu().reshape(-1, 3), plan.src)
        assert torch.equal(cnt.cpu(), plan.recv_count)
        assert torch.equal(per_e.cpu(), plan.per_expert)
        rows = torch.stack([xs[s][tt] for s, tt, _ in plan.src.tolist()])
        if quant_mode == 0:
            assert torch.equal(rx.cpu(), rows)
            ys.append(rx.clone())
        elif quant_mode == 3:
            q, s = ref.quant_fp8_1x128(rows)
            assert torch.equal(rs.cpu(), s)
            assert torch.equal(rx.cpu().view(torch.uint8), q.view(torch.uint8))
            ys.append(ref.dequant_fp8_1x128(rx.cpu(), rs.cpu()).to(torch.bfloat16).to(_dev()))
        else:
            q, s = ref.quant_int8_token(rows)
            assert torch.allclose(rs.cpu().reshape(-1), s, rtol=1e-6)
            assert (rx.cpu().int() - q.int()).abs().max() <= 1
            ys.append((rx.float() * rs).to(torch.bfloat16))

    def comb(r):
        rx, src, cnt, per_e, rs = res[r]
        return ops.moe_combine_prefill(ys[r], dk[r], dw[r], src, cnt, bufs[r].name, r, world)

    outs = run_virtual(comb, world, masks=(PHASE_SEND, PHASE_RECV))
    for r in range(world):
        bufs[r].check()
        if quant_mode == 0:
            xin = xs[r]
        elif quant_mode == 3:
            xin = ref.dequant_fp8_1x128(*ref.quant_fp8_1x128(xs[r])).to(torch.bfloat16)
        else:
            q, s = ref.quant_int8_token(xs[r])
            xin = (q.float() * s.unsqueeze(-1)).to(torch.bfloat16)
        want = ref.combine_reference(xin.unsqueeze(1).expand(t, k, h).contiguous(), topk[r], wts[r], e)
        tol = 0.0 if quant_mode != 2 else 0.1
        assert (outs[r].cpu().float() - want.float()).abs().max() <= tol
    for b in bufs:
        b.destroy()


def test_dispatch_padded_mode_no_host_sync():
    t, h, e, k = 32, 256, 8, 2
    xs, topk, wts = _inputs(1, t, h, e, k, seed=3, lo=0)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=2000.0)
    buf = u.Buffer(None, cfg, name="pad", device=_dev(), rank=0, num_ranks=1)
    rx, src, cnt, per_e, rs = ops.moe_dispatch_prefill_quant(xs[0].to(_dev()), topk[0].to(_dev()), wts[0].to(_dev()),
                                                              t * k, "pad", 0, 1, 3)
    assert rx.shape[0] == t * k and per_e.is_cuda
    assert int(per_e.sum()) == t * k
    buf.check()
    buf.destroy()


@pytest.mark.parametrize("world,quant_mode", [(1, 3), (2, 0), (4, 3), (4, 2)])
def test_low_latency_dispatch_combine(world, quant_mode):
    t, h, e, k = 24, 256, 8, 2
    xs, topk, wts = _inputs(world, t, h, e, k, seed=40 + world, lo=-1)
    topk = [x.to(torch.int32) for x in topk]
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, ll_max_tokens=t, timeout_ms=2000.0)
    bufs = u.Buffer.virtual(world, cfg, _dev(), name=f"l{world}q{quant_mode}_")
    dx = [x.to(_dev()) for x in xs]
    dk = [x.to(_dev()) for x in topk]
    dw = [x.to(_dev()) for x in wts]
    active = t - 5
    mask = torch.zeros(t, dtype=torch.bool, device=_dev())
    mask[:active] = True

    def disp(r):
        return ops.moe_dispatch_shmem(dx[r], dk[r], None, mask, world, r, e, 1, 0, 0, 0, 0, quant_mode, 0, 1,
                                      bufs[r].handle)

    both = run_virtual(disp, world, masks=(PHASE_SEND, PHASE_RECV), return_all=True)
    res = both[PHASE_RECV]
    masked = [x.clone() for x in topk]
    for m in masked:
        m[active:] = -1
    plans = ref.plan_dispatch(masked, e)
    ys = []
    for r in range(world):
        bufs[r].check()
        expand, dyn, eidx, nums, ep_cnt, tp_cnt = res[r]
        plan = plans[r]
        n = plan.src.shape[0]
        assert expand.shape[0] == t * world * min(e // world, k)
        assert torch.equal(ep_cnt.cpu(), plan.recv_count)
        assert torch.equal(nums.cpu(), plan.per_expert)
        eidx = both[PHASE_SEND][r][2]  # expandIdx is produced by the send phase
        assert torch.equal(eidx.cpu(), ref.slots_in_expert(topk[r], e, active))
        rows = torch.stack([xs[s][tt] for s, tt, _ in plan.src.tolist()]) if n else None
        if n and quant_mode == 0:
            assert torch.equal(expand[:n].cpu(), rows)
        elif n and quant_mode == 3:
            q, s = ref.quant_fp8_1x128(rows)
            assert torch.equal(expand[:n].cpu().view(torch.uint8), q.view(torch.uint8))
            assert torch.equal(dyn[:n].cpu(), s)
        elif n:
            q, s = ref.quant_int8_token(rows)
            assert (expand[:n].cpu().int() - q.int()).abs().max() <= 1
        y = torch.zeros(expand.shape[0], h, dtype=torch.bfloat16, device=_dev())
        if n:
            y[:n] = rows.to(_dev())
        ys.append(y)

    def comb(r):
        expand, dyn, eidx, nums, ep_cnt, tp_cnt = res[r]
        return ops.moe_combine_shmem(ys[r], dk[r], eidx, ep_cnt, dw[r], None, mask, None, None, None, None, world, r, e,
                                     1, 0, 0, 0, 0, 0, 0, bufs[r].handle, 0, 0)

    # the combine of virtual rank r must use rank r's own dispatch state, which the Buffer keeps
    outs = run_virtual(comb, world, masks=(PHASE_SEND, PHASE_RECV))
    for r in range(world):
        bufs[r].check()
        want = ref.combine_reference(xs[r].unsqueeze(1).expand(t, k, h).contiguous(), masked[r], wts[r], e)
        assert (outs[r].cpu().float() - want.float()).abs().max() == 0.0
    for b in bufs:
        b.destroy()


def test_bounded_wait_reports_timeout_and_buffer_recovers():
    """Rank 1 withholds its flags (host-side injection); rank 0's wait runs out after 50 ms, the
    kernel returns a status record, and after reset() the same buffers work again."""
    world, t, h, e, k = 2, 16, 256, 4, 2
    xs, topk, wts = _inputs(world, t, h, e, k, seed=77, lo=0)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=50.0)
    bufs = u.Buffer.virtual(world, cfg, _dev(), name="to_")
    dx = [x.to(_dev()) for x in xs]
    dk = [x.to(_dev()) for x in topk]
    dw = [x.to(_dev()) for x in wts]

    def disp(r):
        return ops.moe_dispatch_prefill_quant(dx[r], dk[r], dw[r], t * k * world, bufs[r].name, r, world, 0)

    bufs[1].inject_drop_flags(True)
    run_virtual(disp, world, masks=(PHASE_COUNT, PHASE_SEND))
    with pytest.raises(u.MoeCommTimeout) as ei:
        bufs[0].check()
    assert ei.value.code == 1 and ei.value.who == 1
    bufs[1].inject_drop_flags(False)
    for b in bufs:
        try:
            b.check()
        except u.CamError:
            pass
        b.reset()
    res = run_virtual(disp, world, masks=(PHASE_COUNT, PHASE_SEND, PHASE_RECV))
    plans = ref.plan_dispatch(topk, e)
    for r in range(world):
        bufs[r].check()
        n = plans[r].src.shape[0]
        assert torch.equal(res[r][1].cpu().reshape(-1, 3)[:n], plans[r].src)
    for b in bufs:
        b.destroy()


def test_low_latency_combine_int8_on_the_wire():
    """commQuantMode 2: rows travel as int8 with one scale per 128 elements; the result is the
    weighted sum of the dequantised rows."""
    world, t, h, e, k = 2, 24, 512, 8, 2
    xs, topk, wts = _inputs(world, t, h, e, k, seed=91, lo=0)
    topk = [x.to(torch.int32) for x in topk]
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, ll_max_tokens=t, timeout_ms=2000.0)
    bufs = u.Buffer.virtual(world, cfg, _dev(), name="cq_")
    dx = [x.to(_dev()) for x in xs]
    dk = [x.to(_dev()) for x in topk]
    dw = [x.to(_dev()) for x in wts]

    def disp(r):
        return ops.moe_dispatch_shmem(dx[r], dk[r], None, None, world, r, e, 1, 0, 0, 0, 0, 0, 0, 1, bufs[r].handle)

    res = run_virtual(disp, world, masks=(PHASE_SEND, PHASE_RECV))

    def comb(r):
        expand, dyn, eidx, nums, ep_cnt, tp_cnt = res[r]
        return ops.moe_combine_shmem(expand, dk[r], eidx, ep_cnt, dw[r], None, None, None, None, None, None, world, r, e,
                                     1, 0, 0, 0, 0, 0, 2, bufs[r].handle, 0, 0)

    outs = run_virtual(comb, world, masks=(PHASE_SEND, PHASE_RECV))
    for r in range(world):
        bufs[r].check()
        xin = ref.dequant_int8_1x128(*ref.quant_int8_1x128(xs[r])).unsqueeze(1).expand(t, k, h)
        want = (xin * wts[r].unsqueeze(-1)).sum(dim=1)
        got = outs[r].cpu().float()
        assert (got - want).abs().max() <= 2e-2 * want.abs().max() + 1e-3
        # and it is close to the unquantised combine (int8 per 128 keeps about 2 decimal digits)
        exact = (xs[r].float().unsqueeze(1).expand(t, k, h) * wts[r].unsqueeze(-1)).sum(dim=1)
        assert (got - exact).abs().max() <= 3e-2 * exact.abs().max()
    for b in bufs:
        b.destroy()


@pytest.mark.parametrize("world,shared", [(2, 1), (4, 2)])
def test_low_latency_shared_expert_ranks(world, shared):
    """The first `shared` ranks hold a replica of the shared expert: every token also reaches one of
    them, each replica gets an equal slice of every rank's batch, and combine adds that row unweighted."""
    t, h, k = 16, 256, 2
    routed = 4 * (world - shared)           # 4 routed experts per routed-expert rank
    el = routed // (world - shared)
    xs, topk, wts = _inputs(world, t, h, routed, k, seed=60 + world, lo=0)
    topk = [x.to(torch.int32) for x in topk]
    cfg = u.CamConfig(num_experts=el * world, max_tokens=t, hidden=h, topk=k + 1, ll_max_tokens=t, timeout_ms=2000.0)
    bufs = u.Buffer.virtual(world, cfg, _dev(), name=f"sh{world}_")
    dx = [x.to(_dev()) for x in xs]
    dk = [x.to(_dev()) for x in topk]
    dw = [x.to(_dev()) for x in wts]

    def disp(r):
        return ops.moe_dispatch_shmem(dx[r], dk[r], None, None, world, r, routed, 1, 0, 0, 1, shared, 0, 0, 1,
                                      bufs[r].handle)

    res = run_virtual(disp, world, masks=(PHASE_SEND, PHASE_RECV))
    virt = [ref.remap_for_shared_ranks(topk[r], wts[r], world, routed, shared) for r in range(world)]
    plans = ref.plan_dispatch([v[0] for v in virt], el * world)
    ys = []
    for r in range(world):
        bufs[r].check()
        expand, dyn, eidx, nums, ep_cnt, tp_cnt = res[r]
        plan = plans[r]
        n = plan.src.shape[0]
        if r < shared:
            assert expand.shape[0] == t * world // shared and nums.numel() == 1 and ep_cnt.numel() == world
            assert n == t * world // shared and int(nums[0]) == n
        else:
            assert expand.shape[0] == t * world * min(el, k) and nums.numel() == el
            assert torch.equal(nums.cpu(), plan.per_expert)
        rows = torch.stack([xs[s][tt] for s, tt, _ in plan.src.tolist()])
        assert torch.equal(expand[:n].cpu(), rows)
        # "expert" = multiply by (1 + virtual expert id) so that the combine result shows who computed what
        scale = torch.repeat_interleave(torch.arange(el), plan.per_expert).float() + 1.0 + r * el
        y = torch.zeros(expand.shape[0], h, dtype=torch.bfloat16, device=_dev())
        y[:n] = (rows.float() * scale.unsqueeze(-1)).to(torch.bfloat16).to(_dev())
        ys.append(y)

    def comb(r):
        expand, dyn, eidx, nums, ep_cnt, tp_cnt = res[r]
        return ops.moe_combine_shmem(ys[r], dk[r], eidx, ep_cnt, dw[r], None, None, None, None, None, None, world, r,
                                     routed, 1, 0, 0, 1, shared, 0, 0, bufs[r].handle, 0, 0)

    outs = run_virtual(comb, world, masks=(PHASE_SEND, PHASE_RECV))
    for r in range(world):
        bufs[r].check()
        vid, vw, _, _ = virt[r]
        rows_by_pair = (xs[r].float().unsqueeze(1) * (vid.float() + 1.0).unsqueeze(-1)).to(torch.bfloat16)
        want = ref.combine_reference(rows_by_pair, vid, vw, el * world)
        assert (outs[r].cpu().float() - want.float()).abs().max() == 0.0
    for b in bufs:
        b.destroy()


def test_device_barrier_and_its_timeout():
    """Every rank flags every peer and waits for all of them; a rank that withholds its flags makes
    the others report a barrier timeout instead of hanging."""
    world = 4
    cfg = u.CamConfig(num_experts=8, max_tokens=8, hidden=256, topk=2, timeout_ms=50.0)
    bufs = u.Buffer.virtual(world, cfg, _dev(), name="bar_")
    for _ in range(3):
        run_virtual(lambda r: bufs[r].barrier(), world, masks=(PHASE_SEND, PHASE_RECV))
        for b in bufs:
            b.check()
    bufs[2].inject_drop_flags(True)
    run_virtual(lambda r: bufs[r].barrier(), world, masks=(PHASE_SEND, PHASE_RECV))
    with pytest.raises(u.CamError) as ei:
        bufs[0].check()
    assert ei.value.code == 7 and ei.value.who == 2
    for b in bufs:
        try:
            b.check()
        except u.CamError:
            pass
        b.inject_drop_flags(False)
        b.reset()
    run_virtual(lambda r: bufs[r].barrier(), world, masks=(PHASE_SEND, PHASE_RECV))
    for b in bufs:
        b.check()
        b.destroy()


def test_low_latency_with_tensor_parallel_pair():
    """EP 2 x TP 2 as four virtual ranks: after dispatch every rank also holds its TP partner's rows
    (all-gather); before combine the partial outputs are exchanged and added (reduce-scatter)."""
    from umdk_original_b200.parallel import PHASE_TP_RECV, PHASE_TP_SEND
    ep, t, h, e, k = 2, 16, 256, 4, 2
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, ll_max_tokens=t, timeout_ms=2000.0)
    groups = []  # groups[tp][ep_rank]
    for tp in range(2):
        groups.append([u.Buffer(None, cfg, name=f"tp{tp}_{r}", device=_dev(), rank=r, num_ranks=ep, tp_world_size=2,
                                _connect=False) for r in range(ep)])
        for b in groups[tp]:
            b._native.set_local_peers([x._native for x in groups[tp]])
    for r in range(ep):
        groups[0][r].connect_local_tp_peer(groups[1][r], 0)
        groups[1][r].connect_local_tp_peer(groups[0][r], 1)
    flat = [groups[tp][r] for tp in range(2) for r in range(ep)]  # virtual rank v = tp * ep + r
    g = torch.Generator().manual_seed(123)
    xs = [torch.randn(t, h, generator=g).to(torch.bfloat16) for _ in flat]
    topk = [torch.randint(0, e, (t, k), generator=g).to(torch.int32) for _ in flat]
    wts = [torch.rand(t, k, generator=g) for _ in flat]
    dx = [x.to(_dev()) for x in xs]
    dk = [x.to(_dev()) for x in topk]
    dw = [x.to(_dev()) for x in wts]

    def disp(v):
        tp, r = divmod(v, ep)
        return ops.moe_dispatch_shmem(dx[v], dk[v], None, None, ep, r, e, 2, tp, 0, 0, 0, 0, 0, 1, flat[v].handle)

    res = run_virtual(disp, len(flat), masks=(PHASE_SEND, PHASE_RECV, PHASE_TP_SEND, PHASE_TP_RECV))
    plans = [ref.plan_dispatch([topk[tp * ep + r] for r in range(ep)], e) for tp in range(2)]
    ys = []
    for v, b in enumerate(flat):
        b.check()
        tp, r = divmod(v, ep)
        expand, dyn, eidx, nums, ep_cnt, tp_cnt = res[v]
        own, other = plans[tp][r], plans[1 - tp][r]
        n, m = own.src.shape[0], other.src.shape[0]
        assert tp_cnt.cpu().tolist() == ([n, m] if tp == 0 else [m, n])
        own_rows = torch.stack([xs[tp * ep + s][tt] for s, tt, _ in own.src.tolist()])
        oth_rows = torch.stack([xs[(1 - tp) * ep + s][tt] for s, tt, _ in other.src.tolist()])
        assert torch.equal(expand[:n].cpu(), own_rows) and torch.equal(expand[n:n + m].cpu(), oth_rows)
        # "TP-sharded expert": each TP rank produces a partial output, here (1 + tp) * row for every row it holds
        y = torch.zeros_like(expand)
        y[:n + m] = (expand[:n + m].float() * (1.0 + tp)).to(torch.bfloat16)
        ys.append(y)

    def comb(v):
        tp, r = divmod(v, ep)
        expand, dyn, eidx, nums, ep_cnt, tp_cnt = res[v]
        return ops.moe_combine_shmem(ys[v], dk[v], eidx, ep_cnt, dw[v], tp_cnt, None, None, None, None, None, ep, r, e, 2,
                                     tp, 0, 0, 0, 0, 0, flat[v].handle, 0, 0)

    outs = run_virtual(comb, len(flat), masks=(PHASE_TP_SEND, PHASE_TP_RECV, PHASE_SEND, PHASE_RECV))
    for v, b in enumerate(flat):
        b.check()
        # both partial outputs of every row: 1 * row + 2 * row
        rows3 = (xs[v].float() * 1.0).to(torch.bfloat16).float() + (xs[v].float() * 2.0).to(torch.bfloat16).float()
        want = ref.combine_reference(rows3.to(torch.bfloat16).unsqueeze(1).expand(t, k, h).contiguous(), topk[v], wts[v], e)
        assert (outs[v].cpu().float() - want.float()).abs().max() == 0.0
    for b in flat:
        b.destroy()


def test_receive_overflow_publishes_no_rows_and_writes_nothing():
    """More rows are routed to rank 0 than its buffer holds: the status word says so, every sender skips that
    rank, the counts rank 0 publishes are zero (so the kernels that follow touch no row at or past the capacity)
    and its receive region stays as it was.  The fused layer on the same routing returns the same status."""
    world, t, h, e, k, cap = 2, 64, 256, 4, 2, 32
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(t, h, generator=g).to(torch.bfloat16) for _ in range(world)]
    topk = [torch.stack([torch.randperm(2, generator=g)[:k] for _ in range(t)]) for _ in range(world)]  # experts 0, 1: rank 0
    wts = [torch.rand(t, k, generator=g) for _ in range(world)]
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, capacity=cap, timeout_ms=2000.0)
    bufs = u.Buffer.virtual(world, cfg, _dev(), name="ovf_")
    dx, dk, dw = ([v.to(_dev()) for v in part] for part in (xs, topk, wts))
    region = bufs[0].native.recv_x(cap, h, 0)
    region.fill_(7.0)
    canary = region.clone()

    def disp(r):
        return ops.moe_dispatch_prefill_quant(dx[r], dk[r], dw[r], cap, bufs[r].name, r, world, 0)

    res = run_virtual(disp, world, masks=(PHASE_COUNT, PHASE_SEND, PHASE_RECV))
    with pytest.raises(u.RecvOverflow) as ei:
        bufs[0].check()
    assert ei.value.who == 0 and ei.value.detail == world * t * k
    assert int(bufs[0].native.total_recv().item()) == 0
    assert int(bufs[0].native.expert_offsets(e // world + 1).abs().sum().item()) == 0
    assert int(res[0][3].sum().item()) == 0          # rows per local expert
    assert torch.equal(region, canary)
    for r in range(world):                            # no sender assigned a row on the overflowing rank
        assert bool((bufs[r].native.send_row(t * k) == -1).all())
    for b in bufs:
        try:
            b.check()
        except u.CamError:
            pass
        b.reset()

    from umdk_original_b200.models import random_fp8_experts
    w = random_fp8_experts(e // world, h, 128, device=_dev(), seed=1)

    def fused(r):
        return ops.fused_deep_moe(dx[r], dk[r], [w.w1], [w.s1], [w.w2], [w.s2], dw[r], None, None, bufs[r].name, world, r,
                                  e, 0, 0, 4, 0)

    every = run_virtual(fused, world, return_all=True)
    with pytest.raises(u.RecvOverflow):
        bufs[0].check()
    assert int(every[PHASE_RECV][0][1].sum().item()) == 0
    assert torch.equal(region, canary)
    for b in bufs:
        try:
            b.check()
        except u.CamError:
            pass
        b.destroy()


def test_dispatch_outputs_are_views_until_the_next_dispatch_or_copies_on_request():
    """Default: the outputs of the prefill dispatch view the Buffer's receive region, so the next dispatch on the
    same Buffer replaces their contents.  With set_copy_outputs(True) every call returns tensors of its own (what
    the reference does, pybind/moe_dispatch_prefill.cpp:166-191)."""
    t, h, e, k = 24, 256, 4, 2
    g = torch.Generator().manual_seed(9)
    x1 = torch.randn(t, h, generator=g).to(torch.bfloat16).to(_dev())
    x2 = torch.randn(t, h, generator=g).to(torch.bfloat16).to(_dev())
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(_dev())
    w = torch.rand(t, k, generator=g).to(_dev())
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=2000.0)
    buf = u.Buffer(None, cfg, name="life", device=_dev(), rank=0, num_ranks=1)
    a = ops.moe_dispatch_prefill_quant(x1, idx, w, 0, "life", 0, 1, 0)
    first = a[0].clone()
    b = ops.moe_dispatch_prefill_quant(x2, idx, w, 0, "life", 0, 1, 0)
    assert a[0].data_ptr() == b[0].data_ptr() and torch.equal(a[0], b[0]) and not torch.equal(a[0], first)
    buf.set_copy_outputs(True)
    c = ops.moe_dispatch_prefill_quant(x1, idx, w, 0, "life", 0, 1, 0)
    d = ops.moe_dispatch_prefill_quant(x2, idx, w, 0, "life", 0, 1, 0)
    assert c[0].data_ptr() != d[0].data_ptr()
    assert torch.equal(c[0], first) and torch.equal(d[0], b[0]) and torch.equal(c[1], d[1])
    buf.check()
    # a view that outlives destroy() keeps the memory mapped: reading it afterwards is still defined
    buf.destroy()
    assert torch.equal(b[0], d[0])


def test_stats_name_rows_per_peer_and_waits_and_guards_catch_an_overrun():
    """Buffer.stats(): pairs routed to every peer and the longest wait per peer; Buffer.check(guards=True): the guard
    words behind the receive regions are intact after normal use and an overwritten one is reported by name."""
    world, t, h, e, k = 2, 40, 256, 8, 2
    xs, topk, wts = _inputs(world, t, h, e, k, seed=123, lo=0)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=2000.0)
    bufs = u.Buffer.virtual(world, cfg, _dev(), name="stats_")
    dx, dk, dw = ([v.to(_dev()) for v in part] for part in (xs, topk, wts))

    def disp(r):
        return ops.moe_dispatch_prefill_quant(dx[r], dk[r], dw[r], 0, bufs[r].name, r, world, 0)

    res = run_virtual(disp, world, masks=(PHASE_COUNT, PHASE_SEND, PHASE_RECV))

    def comb(r):
        rx, src, cnt, per_e, rs = res[r]
        return ops.moe_combine_prefill(rx.clone(), dk[r], dw[r], src, cnt, bufs[r].name, r, world)

    run_virtual(comb, world, masks=(PHASE_SEND, PHASE_RECV))
    el = e // world
    for r in range(world):
        bufs[r].check(guards=True)
        st = bufs[r].stats()
        want = [int(((topk[r] // el) == d).sum()) for d in range(world)]
        assert st["rows_routed_to_peer"] == want and st["dispatch_calls"] == 1 and st["combine_calls"] == 1
        assert all(len(v) == world for v in st["max_wait_us"].values())
        assert st["kernel_launches"] >= 5          # three dispatch phases, two combine phases
        assert bufs[r].stats(reset=True)["dispatch_calls"] == 1 and bufs[r].stats()["dispatch_calls"] == 0
    bufs[0].native.guard(2).zero_()                # as if something had written past the end of recv_src
    with pytest.raises(u.CamError) as ei:
        bufs[0].check(guards=True)
    assert ei.value.code == 8 and "recv_src" in str(ei.value)
    bufs[0].check(guards=True)                     # reported once, then restored
    for b in bufs:
        b.destroy()
