"""GPU tests of the deep-fused MoE layer (kernels/fused_moe_mx.cu): the rows of a local expert are
multiplied as soon as they have all arrived, the second GEMM of a row block follows the first one
through a counter, and the combine rows leave from the second GEMM's epilogue.

The reference gates its first GEMM the same way (per-expert token counters,
grouped_matmul_slice_m_per_token_dequant_swiglu_quant_multistage_workspace.h:558-574) and tests
the fused op only against its unfused chain (test_fused_deep_moe.py:361-423); here the oracle is
the fp32 CPU restatement of the layer, and the unfused launches of this library."""
import pytest
import torch

import umdk_original_b200 as u
from umdk_original_b200.models import ExpertWeights
from umdk_original_b200.ops import reference as ref
from umdk_original_b200.parallel import PHASE_COUNT, PHASE_FINAL, PHASE_RECV, PHASE_SEND, phases, run_virtual

pytestmark = pytest.mark.gpu
ops = torch.ops.umdk_cam_op_lib
DEV = torch.device("cuda", 0)


def _case(world, t, h, inter, e, k, seed, holes=False):
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn(t, h, generator=g).to(torch.bfloat16) for _ in range(world)]
    topk = [torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]) for _ in range(world)]
    if holes:
        for tk in topk:
            tk[::5, 0] = -1
    wts = [torch.softmax(torch.randn(t, k, generator=g), -1) for _ in range(world)]
    w1 = torch.randn(e, 2 * inter, h, generator=g) * 0.05
    w2 = torch.randn(e, h, inter, generator=g) * 0.05
    w1q, s1 = ref.quant_fp8_128x128(w1, True)
    w2q, s2 = ref.quant_fp8_128x128(w2, True)
    return xs, topk, wts, (w1q, s1, w2q, s2)


def _local_weights(w, world, e):
    w1q, s1, w2q, s2 = w
    el = e // world
    return [ExpertWeights(w1q[r * el:(r + 1) * el].contiguous(), s1[r * el:(r + 1) * el].contiguous(),
                          w2q[r * el:(r + 1) * el].contiguous(), s2[r * el:(r + 1) * el].contiguous()).to(DEV)
            for r in range(world)]


def _run_layer(monkeypatch, deep, world, cfg, name, dx, dk, dw, local, e):
    monkeypatch.setenv("UMDK_CAM_DEEP_FUSE", str(int(deep)))  # 0: four launches, 1: deep-fused, 2: fused GEMMs only
    bufs = u.Buffer.virtual(world, cfg, DEV, name=name)

    def step(r):
        w = local[r]
        return ops.fused_deep_moe(dx[r], dk[r], [w.w1], [w.s1], [w.w2], [w.s2], dw[r], None, None, bufs[r].name, world, r,
                                  e, 0, 0, 4, 0)

    every = run_virtual(step, world, return_all=True)
    for b in bufs:
        b.check()
    outs = [every[PHASE_FINAL][r][0].cpu().float() for r in range(world)]
    nums = [every[PHASE_RECV][r][1].cpu() for r in range(world)]
    return bufs, step, outs, nums


@pytest.mark.parametrize("world,holes,route", [(1, False, 1), (2, True, 1), (4, False, 1), (1, False, 2), (2, True, 2)])
def test_deep_fused_layer_matches_oracle_and_unfused(world, holes, route, monkeypatch):
    """Virtual ranks on one GPU: every expert spans more than one 256-row tile on some rank and the
    tile walk interleaves the two GEMMs; results against the fp32 oracle (row-relative) and against
    the four-launch route.  Route 1 sends the dispatch rows from inside the fused kernel, route 2 runs the
    normal dispatch first and the fused kernel for the two GEMMs only."""
    t, h, inter, e, k = 384, 1024, 512, 8, 4
    xs, topk, wts, w = _case(world, t, h, inter, e, k, seed=300 + world, holes=holes)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=3000.0)
    local = _local_weights(w, world, e)
    dx, dk, dw = ([v.to(DEV) for v in part] for part in (xs, topk, wts))
    bufs, step, outs, nums = _run_layer(monkeypatch, route, world, cfg, f"deep{world}_{route}_", dx, dk, dw, local, e)
    # a second call on the same buffers: epochs, counters and parities roll over
    every2 = run_virtual(step, world, return_all=True)
    outs2 = [every2[PHASE_FINAL][r][0].cpu().float() for r in range(world)]
    for b in bufs:
        b.check()
        b.destroy()
    bufs_u, _, outs_u, nums_u = _run_layer(monkeypatch, 0, world, cfg, f"flat{world}_{route}_", dx, dk, dw, local, e)
    for b in bufs_u:
        b.destroy()
    el = e // world
    total = torch.zeros(e, dtype=torch.int64)
    for r in range(world):
        want, counts = ref.fused_moe_fp8_reference(xs[r], topk[r], wts[r], *w, ue8m0=True)
        total += counts
        wf = want.float()
        row_scale = wf.abs().amax(dim=1, keepdim=True) + 1e-6
        err = ((outs[r] - wf).abs() / row_scale).max().item()
        assert err <= 0.04, f"rank {r}: row-relative error {err} against the oracle"
        assert torch.equal(outs[r], outs2[r]), "the second call on the same buffers differs"
        # same quantisation and same tile arithmetic as the unfused launches
        assert ((outs[r] - outs_u[r]).abs() / row_scale).max().item() <= 0.02
    for r in range(world):
        assert torch.equal(nums[r], total[r * el:(r + 1) * el])
        assert torch.equal(nums[r], nums_u[r])


def test_deep_fused_layer_production_shape_one_gpu(monkeypatch):
    """h = 7168, I = 2048 (56 K-blocks, 16 + 28 column tiles per row block), 8 local experts of about 1000 rows:
    every CTA pair walks several tiles of both GEMMs, and sends overlap the GEMMs inside one real (not
    phase-split) launch.  Checked on a sample of tokens against the fp32 oracle."""
    monkeypatch.setenv("UMDK_CAM_DEEP_FUSE", "1")
    t, h, inter, e, k = 2048, 7168, 2048, 8, 4
    g = torch.Generator().manual_seed(11)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)])
    wt = torch.softmax(torch.randn(t, k, generator=g), -1)
    w1q, s1, w2q, s2 = [], [], [], []
    for i in range(e):  # expert by expert keeps the fp32 temporaries small
        a, b = ref.quant_fp8_128x128(torch.randn(1, 2 * inter, h, generator=g) * 0.03, True)
        c, d = ref.quant_fp8_128x128(torch.randn(1, h, inter, generator=g) * 0.03, True)
        w1q.append(a); s1.append(b); w2q.append(c); s2.append(d)
    w1q, s1, w2q, s2 = (torch.cat(v) for v in (w1q, s1, w2q, s2))
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=5000.0)
    buf = u.Buffer(None, cfg, name="deep_prod", device=DEV, rank=0, num_ranks=1)
    w = ExpertWeights(w1q, s1, w2q, s2).to(DEV)
    buf.set_fused_trace(True)
    for _ in range(2):
        out, nums = ops.fused_deep_moe(x.to(DEV), idx.to(DEV), [w.w1], [w.s1], [w.w2], [w.s2], wt.to(DEV), None, None,
                                       "deep_prod", 1, 0, e, 0, 0, 4, 0)
    buf.check()
    released = buf.read_fused_trace(e)
    assert all(v is not None for v in released), released
    assert released == sorted(released), f"experts were not released in order: {released}"
    sample = torch.arange(0, t, 37)[:48]
    want, _ = ref.fused_moe_fp8_reference(x[sample], idx[sample], wt[sample], w1q, s1, w2q, s2, ue8m0=True)
    got = out.cpu().float()[sample]
    wf = want.float()
    row_scale = wf.abs().amax(dim=1, keepdim=True) + 1e-6
    err = ((got - wf).abs() / row_scale).max().item()
    assert err <= 0.04, f"row-relative error {err}"
    assert torch.equal(nums.cpu(), torch.bincount(idx.reshape(-1), minlength=e))
    buf.destroy()


def test_deep_fused_layer_runs_complete_experts_and_reports_a_held_back_rank(monkeypatch):
    """Rank 1 sends its rows but never counts them on the arrival counters (host-side injection).  Its tokens use
    the second local expert of every rank only, so on rank 0 the first local expert is complete and its GEMM is
    released (trace stamp), while the second one runs into the time limit: the kernel returns a status record,
    and after reset() the same buffers compute the right result."""
    monkeypatch.setenv("UMDK_CAM_DEEP_FUSE", "1")
    world, t, h, inter, e, k = 2, 256, 512, 256, 4, 2
    xs, topk, wts, w = _case(world, t, h, inter, e, k, seed=41)
    topk[1] = torch.tensor([1, 3]).repeat(t, 1)          # rank 1: local expert 1 of rank 0 and of rank 1
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=200.0)
    bufs = u.Buffer.virtual(world, cfg, DEV, name="held_")
    local = _local_weights(w, world, e)
    dx, dk, dw = ([v.to(DEV) for v in part] for part in (xs, topk, wts))

    def step(r):
        lw = local[r]
        return ops.fused_deep_moe(dx[r], dk[r], [lw.w1], [lw.s1], [lw.w2], [lw.s2], dw[r], None, None, bufs[r].name,
                                  world, r, e, 0, 0, 4, 0)

    bufs[0].set_fused_trace(True)
    run_virtual(step, world, masks=(PHASE_COUNT,))
    bufs[1].inject_drop_flags(True)      # the counts were exchanged; from here on rank 1's rows are never counted
    run_virtual(step, world, masks=(PHASE_SEND,))
    with phases(PHASE_RECV):
        step(0)
    with pytest.raises(u.MoeCommTimeout) as ei:
        bufs[0].check()
    assert ei.value.code == 9 and ei.value.who == 1, (ei.value.code, ei.value.who)
    released = bufs[0].read_fused_trace(e // world)
    assert released[0] is not None and released[1] is None, released
    bufs[1].inject_drop_flags(False)
    for b in bufs:
        try:
            b.check()
        except u.CamError:
            pass
        b.reset()
    every = run_virtual(step, world, return_all=True)
    for r in range(world):
        bufs[r].check()
        want, _ = ref.fused_moe_fp8_reference(xs[r], topk[r], wts[r], *w, ue8m0=True)
        wf = want.float()
        row_scale = wf.abs().amax(dim=1, keepdim=True) + 1e-6
        assert ((every[PHASE_FINAL][r][0].cpu().float() - wf).abs() / row_scale).max().item() <= 0.04
    for b in bufs:
        b.destroy()


def test_route_follows_rank_count_expert_size_and_the_switch(monkeypatch):
    """Unset, the deep-fused route is taken on 8 ranks or more when experts get 768 rows or more on average; the switch
    forces any route.  The layer gives the same answer on every route (8 virtual ranks on one GPU)."""
    world, t, h, inter, e, k = 8, 192, 512, 256, 8, 4   # 192 * 4 * 8 / 8 = 768 rows per expert
    xs, topk, wts, w = _case(world, t, h, inter, e, k, seed=77, holes=False)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=3000.0)
    local = _local_weights(w, world, e)
    dx, dk, dw = ([v.to(DEV) for v in part] for part in (xs, topk, wts))
    monkeypatch.delenv("UMDK_CAM_DEEP_FUSE", raising=False)
    bufs = u.Buffer.virtual(world, cfg, DEV, name="route_auto_")
    assert bufs[0].fused_route(t, inter) == "deep-fused"
    assert bufs[0].fused_route(t // 2, inter) == "four launches"          # 384 rows per expert
    assert bufs[0].fused_route(t, inter, hidden=640) == "four launches"    # scale rows not whole 16-byte pieces

    def step(r):
        wl = local[r]
        return ops.fused_deep_moe(dx[r], dk[r], [wl.w1], [wl.s1], [wl.w2], [wl.s2], dw[r], None, None, bufs[r].name, world,
                                  r, e, 0, 0, 4, 0)

    every = run_virtual(step, world, return_all=True)
    outs = [every[PHASE_FINAL][r][0].cpu().float() for r in range(world)]
    for b in bufs:
        b.check()
        b.destroy()
    small = u.Buffer.virtual(2, cfg, DEV, name="route_two_")
    assert small[0].fused_route(t * 4, inter) == "four launches"           # two ranks: never by default
    for b in small:
        b.destroy()
    bufs_u, _, outs_u, _ = _run_layer(monkeypatch, 0, world, cfg, "route_flat_", dx, dk, dw, local, e)
    assert bufs_u[0].fused_route(t, inter) == "four launches"
    for b in bufs_u:
        b.destroy()
    for r in range(world):
        scale = outs_u[r].abs().amax(dim=1, keepdim=True) + 1e-6
        assert ((outs[r] - outs_u[r]).abs() / scale).max().item() <= 0.02
