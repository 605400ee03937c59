"""GPU tests of the tcgen05 grouped GEMM and of the fused MoE layer, against the fp32 oracle."""
import pytest
import torch

import umdk_original_b200 as u
from umdk_original_b200.models import ExpertWeights
from umdk_original_b200.ops import reference as ref
from umdk_original_b200.parallel import PHASE_FINAL, PHASE_RECV, run_virtual

pytestmark = pytest.mark.gpu
ops = torch.ops.umdk_cam_op_lib
DEV = torch.device("cuda", 0)


@pytest.fixture(params=["single", "pair", "swap"])
def gemm_variant(request, monkeypatch):
    """Runs a block-scaled GEMM test on the one-CTA kernel, on the CTA-pair (cta_group::2) kernel and on the
    one-CTA kernel with its operands exchanged (weights as the M operand, for small experts)."""
    monkeypatch.setenv("UMDK_CAM_GEMM_PAIR", "1" if request.param == "pair" else "0")
    monkeypatch.setenv("UMDK_CAM_GEMM_SWAP", "1" if request.param == "swap" else "0")
    return request.param


def _ragged_problem(counts, n, k, seed, ue8m0=False):
    g = torch.Generator().manual_seed(seed)
    m = sum(counts)
    # rows and weight blocks of very different magnitude, so that a misplaced scale factor shows
    a = torch.randn(m, k, generator=g) * torch.exp(torch.randn(m, 1, generator=g) * 2.0)
    w = torch.randn(len(counts), n, k, generator=g) * 0.05
    w = w * torch.exp(torch.randn(len(counts), n // 128, 1, k // 128, 1, generator=g)).expand(
        -1, -1, 128, -1, 128).reshape(len(counts), n, k)
    aq, a_s = ref.quant_fp8_1x128(a, ue8m0)
    wq, w_s = ref.quant_fp8_128x128(w, ue8m0)
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32)
    return aq, a_s, wq, w_s, off


@pytest.mark.parametrize("ue8m0", [False, True])
@pytest.mark.parametrize("counts,n,k", [([128], 256, 128), ([128], 256, 512), ([5, 0, 130, 257], 512, 384),
                                         ([300, 1, 77], 384, 256), ([40, 512, 129], 512, 1024)])
def test_grouped_gemm_plain(counts, n, k, ue8m0, gemm_variant):
    if not ue8m0 and gemm_variant != "single":
        pytest.skip("the fp32-scale kernel has one form only")
    aq, a_s, wq, w_s, off = _ragged_problem(counts, n, k, seed=len(counts) * 7 + n, ue8m0=ue8m0)
    got = ops.grouped_gemm_fp8(aq.to(DEV), a_s.to(DEV), wq.to(DEV), w_s.to(DEV), off.to(DEV), ue8m0).cpu().float()
    want = ops.grouped_gemm_fp8(aq, a_s, wq, w_s, off).float()  # CPU oracle
    torch.cuda.synchronize()
    # per-row tolerance: rows differ in magnitude by orders
    row_scale = want.abs().amax(dim=1, keepdim=True)
    err = ((got - want).abs() / (row_scale + 1e-6)).max().item()
    assert err <= 2e-2, f"max row-relative err {err}"


@pytest.mark.parametrize("ue8m0", [False, True])
@pytest.mark.parametrize("counts,inter,k", [([128], 128, 256), ([70, 200, 0, 3], 256, 384)])
def test_grouped_gemm_swiglu_requant(counts, inter, k, ue8m0, gemm_variant):
    if not ue8m0 and gemm_variant != "single":
        pytest.skip("the fp32-scale kernel has one form only")
    aq, a_s, wq, w_s, off = _ragged_problem(counts, 2 * inter, k, seed=inter + k, ue8m0=ue8m0)
    q, s = ops.grouped_gemm_fp8_swiglu(aq.to(DEV), a_s.to(DEV), wq.to(DEV), w_s.to(DEV), off.to(DEV), ue8m0)
    qc, sc = ops.grouped_gemm_fp8_swiglu(aq, a_s, wq, w_s, off, ue8m0)
    got = ref.dequant_fp8_1x128(q.cpu(), s.cpu())
    want = ref.dequant_fp8_1x128(qc, sc)
    row_scale = want.abs().amax(dim=1, keepdim=True) + 1e-6
    # one e4m3 step (2^-3 relative) where a value sits on a rounding boundary
    assert ((got - want).abs() / row_scale).max().item() <= 0.14
    assert ((got - want).abs() / row_scale).mean().item() <= 0.01
    if ue8m0:
        assert ref.is_power_of_two(s.cpu()[: sum(counts)])
        # a block whose amax/448 sits within rounding of a power of two may land one step apart
        ratio = s.cpu()[: sum(counts)] / sc[: sum(counts)]
        assert ((ratio == 1.0) | (ratio == 2.0) | (ratio == 0.5)).all() and (ratio == 1.0).float().mean() > 0.98
    else:
        assert torch.allclose(s.cpu(), sc, rtol=2e-2, atol=1e-6)


def _fused_case(world, t, h, inter, e, k, seed, lo=0, ue8m0=False):
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn(t, h, generator=g).to(torch.bfloat16) for _ in range(world)]
    topk = [torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]) for _ in range(world)]
    if lo < 0:
        for tk in topk:
            tk[::7, 0] = -1
    wts = [torch.softmax(torch.randn(t, k, generator=g), -1) for _ in range(world)]
    w1 = torch.randn(e, 2 * inter, h, generator=g) * 0.05
    w2 = torch.randn(e, h, inter, generator=g) * 0.05
    w1q, s1 = ref.quant_fp8_128x128(w1, ue8m0)
    w2q, s2 = ref.quant_fp8_128x128(w2, ue8m0)
    return xs, topk, wts, (w1q, s1, w2q, s2)


@pytest.mark.parametrize("ue8m0", [False, True])
@pytest.mark.parametrize("world,lo", [(1, 0), (1, -1), (2, 0), (4, -1)])
def test_fused_moe_fp8(world, lo, ue8m0, gemm_variant):
    if not ue8m0 and gemm_variant != "single":
        pytest.skip("the fp32-scale kernel has one form only")
    t, h, inter, e, k = 48, 512, 256, 8, 2
    xs, topk, wts, (w1q, s1, w2q, s2) = _fused_case(world, t, h, inter, e, k, seed=100 + world, lo=lo, ue8m0=ue8m0)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=3000.0)
    bufs = u.Buffer.virtual(world, cfg, DEV, name=f"f{world}_{-lo}_{int(ue8m0)}_")
    el = e // world
    local = [ExpertWeights(w1q[r * el:(r + 1) * el].contiguous(), s1[r * el:(r + 1) * el].contiguous(),
                           w2q[r * el:(r + 1) * el].contiguous(), s2[r * el:(r + 1) * el].contiguous()).to(DEV)
             for r in range(world)]
    dx = [x.to(DEV) for x in xs]
    dk = [x.to(DEV) for x in topk]
    dw = [x.to(DEV) for x in wts]

    def step(r):
        w = local[r]
        return ops.fused_deep_moe(dx[r], dk[r], [w.w1], [w.s1], [w.w2], [w.s2], dw[r], None, None, bufs[r].name, world, r,
                                  e, 0, 0, 4 if ue8m0 else 3, 0)

    every = run_virtual(step, world, return_all=True)
    res = every[PHASE_FINAL]
    total_counts = torch.zeros(e, dtype=torch.int64)
    for r in range(world):
        bufs[r].check()
        want, counts = ref.fused_moe_fp8_reference(xs[r], topk[r], wts[r], w1q, s1, w2q, s2, ue8m0=ue8m0)
        total_counts += counts
        got = res[r][0].cpu().float()
        scale = want.float().abs().max().item()
        err = (got - want.float()).abs().max().item()
        assert err <= 0.06 * scale + 1e-3, f"rank {r}: max err {err} vs scale {scale}"
    for r in range(world):
        assert torch.equal(every[PHASE_RECV][r][1].cpu(), total_counts[r * el:(r + 1) * el])
    for b in bufs:
        b.destroy()


def test_fused_moe_x_active_mask():
    t, h, inter, e, k = 32, 256, 128, 4, 2
    xs, topk, wts, (w1q, s1, w2q, s2) = _fused_case(1, t, h, inter, e, k, seed=5)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=3000.0)
    buf = u.Buffer(None, cfg, name="mask", device=DEV, rank=0, num_ranks=1)
    w = ExpertWeights(w1q, s1, w2q, s2).to(DEV)
    mask = torch.zeros(t, dtype=torch.bool, device=DEV)
    mask[:20] = True
    out, nums = ops.fused_deep_moe(xs[0].to(DEV), topk[0].to(DEV), [w.w1], [w.s1], [w.w2], [w.s2], wts[0].to(DEV), None,
                                   mask, "mask", 1, 0, e, 0, 0, 3, 0)
    buf.check()
    masked = topk[0].clone()
    masked[20:] = -1
    want, counts = ref.fused_moe_fp8_reference(xs[0], masked, wts[0], w1q, s1, w2q, s2)
    assert torch.equal(nums.cpu(), counts)
    assert (out.cpu().float() - want.float()).abs().max() <= 0.06 * want.float().abs().max() + 1e-3
    assert (out[20:].float().abs().max() == 0)
    buf.destroy()


def test_fused_moe_tensor_list_matches_stacked():
    """Weights as a list of per-expert tensors (dynamic expert placement) give the stacked result,
    and replacing one expert's tensor is picked up on the next call."""
    t, h, inter, e, k = 32, 256, 128, 4, 2
    xs, topk, wts, (w1q, s1, w2q, s2) = _fused_case(1, t, h, inter, e, k, seed=9, ue8m0=True)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=3000.0)
    buf = u.Buffer(None, cfg, name="tl", device=DEV, rank=0, num_ranks=1)
    w = ExpertWeights(w1q, s1, w2q, s2).to(DEV)
    x, ids, sc = xs[0].to(DEV), topk[0].to(DEV), wts[0].to(DEV)

    def call(a, b, c, d):
        out, nums = ops.fused_deep_moe(x, ids, a, b, c, d, sc, None, None, "tl", 1, 0, e, 0, 0, 4, 0)
        buf.check()
        return out.clone(), nums.clone()

    want, n0 = call([w.w1], [w.s1], [w.w2], [w.s2])
    lists = [list(v.unbind(0)) for v in (w.w1, w.s1, w.w2, w.s2)]
    lists = [[v.clone() for v in l] for l in lists]
    got, n1 = call(*lists)
    assert torch.equal(got, want) and torch.equal(n0, n1)
    got2, _ = call(*lists)  # cached stack
    assert torch.equal(got2, want)
    # swap experts 0 and 1 in the list: the result must change like the stacked form does
    for l in lists:
        l[0], l[1] = l[1], l[0]
    perm = torch.tensor([1, 0, 2, 3], device=DEV)
    want_sw, _ = call([w.w1[perm].contiguous()], [w.s1[perm].contiguous()], [w.w2[perm].contiguous()],
                      [w.s2[perm].contiguous()])
    got_sw, _ = call(*lists)
    assert torch.equal(got_sw, want_sw)
    buf.destroy()


def test_fused_moe_shared_expert_rank():
    """2 virtual ranks: rank 0 holds the shared expert (one local expert), rank 1 the 4 routed experts."""
    world, shared, t, h, inter, e, k = 2, 1, 32, 256, 128, 4, 2
    xs, topk, wts, (w1q, s1, w2q, s2) = _fused_case(world, t, h, inter, e, k, seed=21, ue8m0=True)
    g = torch.Generator().manual_seed(22)
    sw1q, ss1 = ref.quant_fp8_128x128(torch.randn(1, 2 * inter, h, generator=g) * 0.05, True)
    sw2q, ss2 = ref.quant_fp8_128x128(torch.randn(1, h, inter, generator=g) * 0.05, True)
    el = e // (world - shared)
    cfg = u.CamConfig(num_experts=el * world, max_tokens=t, hidden=h, topk=k + 1, timeout_ms=3000.0)
    bufs = u.Buffer.virtual(world, cfg, DEV, name="fsh_")
    local = [ExpertWeights(sw1q, ss1, sw2q, ss2).to(DEV), ExpertWeights(w1q, s1, w2q, s2).to(DEV)]
    dx = [x.to(DEV) for x in xs]
    dk = [x.to(DEV) for x in topk]
    dw = [x.to(DEV) for x in wts]

    def step(r):
        w = local[r]
        return ops.fused_deep_moe(dx[r], dk[r], [w.w1], [w.s1], [w.w2], [w.s2], dw[r], None, None, bufs[r].name, world, r,
                                  e, 1, shared, 4, 0)

    every = run_virtual(step, world, return_all=True)
    res = every[PHASE_FINAL]
    for r in range(world):
        bufs[r].check()
        routed, counts = ref.fused_moe_fp8_reference(xs[r], topk[r], wts[r], w1q, s1, w2q, s2, ue8m0=True)
        xq, xsc = ref.quant_fp8_1x128(xs[r], True)
        shared_row = ref.expert_mlp_fp8(xq, xsc, sw1q[0], ss1[0], sw2q[0], ss2[0], ue8m0=True)
        want = routed.float() + shared_row.float()
        got = res[r][0].cpu().float()
        assert (got - want).abs().max() <= 0.06 * want.abs().max() + 1e-3
    assert every[PHASE_RECV][0][1].numel() == 1 and int(every[PHASE_RECV][0][1][0]) == t * world
    assert every[PHASE_RECV][1][1].numel() == el
    for b in bufs:
        b.destroy()


@pytest.mark.parametrize("counts,n,k", [([128], 256, 128), ([5, 0, 130, 257], 512, 384), ([300, 1, 77], 384, 1024)])
def test_grouped_gemm_w8a8_exact(counts, n, k):
    """int8 x int8 -> int32 on the tensor cores: the result is the exact integer product times the scales."""
    g = torch.Generator().manual_seed(n + k)
    m = sum(counts)
    a_q = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8)
    a_s = torch.rand(m, generator=g) * 0.01 + 0.001
    w_q = torch.randint(-127, 128, (len(counts), n, k), generator=g, dtype=torch.int8)
    w_s = torch.rand(len(counts), n, generator=g) * 0.003 + 0.0015
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32)
    got = ops.grouped_gemm_w8a8(a_q.to(DEV), a_s.to(DEV), w_q.to(DEV), w_s.to(DEV), off.to(DEV)).cpu().float()
    want = ops.grouped_gemm_w8a8(a_q, a_s, w_q, w_s, off).float()
    # same integer sum, same two fp32 multiplications, one bf16 rounding
    assert (got - want).abs().max().item() <= 2 ** -7 * want.abs().max().item()
    assert ((got - want).abs() > 0).float().mean().item() < 1e-3


@pytest.mark.parametrize("world", [1, 2])
def test_fused_moe_w8a8_reference_layout(world):
    """quantMode 0 with int8 weights in the reference's layout ([E_l, h, 2I] / [E_l, I, h], per-channel
    scales) runs the exact W8A8 path; data recipe of the reference's unit test
    (test_fused_deep_moe.py:290-319: weights randint(-16, 16), scales rand * 0.003 + 0.0015)."""
    from umdk_original_b200.models import random_w8a8_experts
    t, h, inter, e, k = 48, 512, 256, 8, 2
    g = torch.Generator().manual_seed(300 + world)
    xs = [(torch.rand(t, h, generator=g) * 10 - 5).to(torch.bfloat16) for _ in range(world)]
    topk = [torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]) for _ in range(world)]
    wts = [torch.softmax(torch.randn(t, k, generator=g), -1) for _ in range(world)]
    w1, s1, w2, s2 = random_w8a8_experts(e, h, inter, seed=7)   # [E, h, 2I], [E, 2I], [E, I, h], [E, h]
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=3000.0)
    bufs = u.Buffer.virtual(world, cfg, DEV, name=f"w8_{world}_")
    el = e // world
    dev_w = [[v[r * el:(r + 1) * el].contiguous().to(DEV) for v in (w1, s1, w2, s2)] for r in range(world)]
    dx = [x.to(DEV) for x in xs]
    dk = [x.to(DEV) for x in topk]
    dw = [x.to(DEV) for x in wts]

    def step(r):
        a, b, c, d = dev_w[r]
        return ops.fused_deep_moe(dx[r], dk[r], [a], [b], [c], [d], dw[r], None, None, bufs[r].name, world, r, e, 0, 0, 0, 0)

    every = run_virtual(step, world, return_all=True)
    res = every[PHASE_FINAL]
    for r in range(world):
        bufs[r].check()
        rows = torch.zeros(t, k, h, dtype=torch.bfloat16)
        for ex in range(e):
            tok, kk = torch.nonzero(topk[r] == ex, as_tuple=True)
            if tok.numel():
                rows[tok, kk] = ref.expert_mlp_w8a8(xs[r][tok], w1[ex].t(), s1[ex], w2[ex].t(), s2[ex])
        want = ref.combine_reference(rows, topk[r], wts[r], e).float()
        got = res[r][0].cpu().float()
        # the reference's own gate for this operator is atol 2.0, rtol 0.02; the exact path is much closer
        assert torch.allclose(got, want, atol=0.02 * want.abs().max().item(), rtol=0.02), (got - want).abs().max()
    for b in bufs:
        b.destroy()


def test_fused_layer_stage_profile():
    """Buffer.set_profile() records events around the four launches of a full fused call."""
    t, h, inter, e, k = 32, 256, 128, 4, 2
    xs, topk, wts, (w1q, s1, w2q, s2) = _fused_case(1, t, h, inter, e, k, seed=11, ue8m0=True)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=3000.0)
    buf = u.Buffer(None, cfg, name="prof", device=DEV, rank=0, num_ranks=1)
    w = ExpertWeights(w1q, s1, w2q, s2).to(DEV)
    buf.set_profile(True)
    ops.fused_deep_moe(xs[0].to(DEV), topk[0].to(DEV), [w.w1], [w.s1], [w.w2], [w.s2], wts[0].to(DEV), None, None, "prof",
                       1, 0, e, 0, 0, 4, 0)
    parts = buf.read_profile()
    assert set(parts) == {"dispatch_ms", "gemm1_ms", "gemm2_send_ms", "combine_ms"} and all(v > 0 for v in parts.values())
    buf.set_profile(False)
    buf.check()
    buf.destroy()
