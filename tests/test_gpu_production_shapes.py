"""GPU tests at the shapes the library is benchmarked on, where every persistent loop runs many times:
K = 7168 (56 K-blocks), thousands of output tiles for 148 CTAs, thousands of tokens per rank.
The small-shape tests cover the contracts; these cover the carry-over of pipeline state from tile
to tile and the multi-round paths of the communication kernels.

Inputs are produced on the GPU; the fp32 oracle runs on the CPU for a sample of rows per expert
(plain matrix products of the dequantised operands).  The last group repeats the only cases the
reference's own unit test defines (test/cam/ut/fused_deep_moe/test_fused_deep_moe.py:339-359,
data recipe :290-319) under its gate, atol 2.0 / rtol 0.02 (:416-422), and under a tight one."""
import pytest
import torch

import umdk_original_b200 as u
from umdk_original_b200.ops import reference as ref
from umdk_original_b200.parallel import PHASE_COUNT, PHASE_FINAL, PHASE_RECV, PHASE_SEND, run_virtual

pytestmark = pytest.mark.gpu
ops = torch.ops.umdk_cam_op_lib
DEV = torch.device("cuda", 0)


def _ragged_counts(num_experts, hi, seed):
    g = torch.Generator().manual_seed(seed)
    c = torch.randint(0, hi + 1, (num_experts,), generator=g)
    c[1] = 0          # an empty expert
    c[2] = hi         # a full one
    c[3] = 129        # one row into a second 128-row tile
    return c.tolist()


def _big_fp8_problem(counts, n, k, seed, ue8m0):
    """Operands made on the GPU: rows and weight blocks of very different magnitude."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    m = sum(counts)
    a = torch.randn(m, k, device=DEV, generator=g) * torch.exp(torch.randn(m, 1, device=DEV, generator=g) * 1.5)
    aq, a_s = ref.quant_fp8_1x128(a, ue8m0)
    del a
    wq, w_s = [], []
    for _ in counts:  # expert by expert keeps the fp32 temporaries small
        w = torch.randn(n, k, device=DEV, generator=g) * 0.05
        w = (w.view(n // 128, 128, k // 128, 128) *
             torch.exp(torch.randn(n // 128, 1, k // 128, 1, device=DEV, generator=g))).view(1, n, k)
        q, s = ref.quant_fp8_128x128(w, ue8m0)
        wq.append(q)
        w_s.append(s)
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    return aq, a_s.contiguous(), torch.cat(wq), torch.cat(w_s).contiguous(), off


def _sample_rows(counts, per_expert, seed):
    g = torch.Generator().manual_seed(seed)
    picks, start = [], 0
    for e, c in enumerate(counts):
        if c:
            r = torch.unique(torch.cat([torch.tensor([0, c - 1]), torch.randint(0, c, (per_expert,), generator=g)]))
            picks.append((e, start + r))
        start += c
    return picks


@pytest.fixture(params=["fp32_scales", "mx_single", "mx_pair"])
def big_variant(request, monkeypatch):
    monkeypatch.setenv("UMDK_CAM_GEMM_PAIR", "1" if request.param == "mx_pair" else "0")
    monkeypatch.setenv("UMDK_CAM_GEMM_SWAP", "0")
    return request.param


def test_grouped_gemm_plain_many_tiles_per_cta(big_variant):
    """24 ragged experts x N = 2048 x K = 7168: about 700 (one-CTA kernels) / 400 (CTA pairs) output tiles."""
    ue8m0 = big_variant != "fp32_scales"
    counts = _ragged_counts(24, 700, seed=5)
    n, k = 2048, 7168
    aq, a_s, wq, w_s, off = _big_fp8_problem(counts, n, k, seed=17, ue8m0=ue8m0)
    got = ops.grouped_gemm_fp8(aq, a_s, wq, w_s, off, ue8m0)
    torch.cuda.synchronize()
    worst = 0.0
    for e, rows in _sample_rows(counts, 6, seed=3):
        a = ref.dequant_fp8_1x128(aq[rows.to(DEV)].cpu(), a_s[rows.to(DEV)].cpu())
        w = ref.dequant_fp8_128x128(wq[e].cpu(), w_s[e].cpu())
        want = a @ w.t()
        g = got[rows.to(DEV)].cpu().float()
        worst = max(worst, ((g - want).abs() / (want.abs().amax(dim=1, keepdim=True) + 1e-6)).max().item())
    assert worst <= 2e-2, f"max row-relative error {worst}"


def test_grouped_gemm_swiglu_requant_many_tiles_per_cta(big_variant):
    """GEMM1 flavour at the production shape: 2I = 4096, K = 7168, SwiGLU + 1x128 requantisation in the epilogue."""
    ue8m0 = big_variant != "fp32_scales"
    counts = _ragged_counts(16, 600, seed=9)
    inter, k = 2048, 7168
    aq, a_s, wq, w_s, off = _big_fp8_problem(counts, 2 * inter, k, seed=23, ue8m0=ue8m0)
    q, s = ops.grouped_gemm_fp8_swiglu(aq, a_s, wq, w_s, off, ue8m0)
    torch.cuda.synchronize()
    worst, mean_acc, nrow = 0.0, 0.0, 0
    for e, rows in _sample_rows(counts, 5, seed=4):
        a = ref.dequant_fp8_1x128(aq[rows.to(DEV)].cpu(), a_s[rows.to(DEV)].cpu())
        w = ref.dequant_fp8_128x128(wq[e].cpu(), w_s[e].cpu())
        y = a @ w.t()
        want = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
        g = ref.dequant_fp8_1x128(q[rows.to(DEV)].cpu(), s[rows.to(DEV)].cpu())
        rel = (g - want).abs() / (want.abs().amax(dim=1, keepdim=True) + 1e-6)
        worst = max(worst, rel.max().item())
        mean_acc += rel.mean().item() * rows.numel()
        nrow += rows.numel()
    # one e4m3 step (2^-3 relative) where a value sits on a rounding boundary
    assert worst <= 0.14 and mean_acc / nrow <= 0.01, (worst, mean_acc / nrow)
    if ue8m0:
        assert ref.is_power_of_two(s[: sum(counts)].cpu())


def test_grouped_gemm_w8a8_many_tiles_per_cta():
    """int8 x int8 -> int32 at K = 7168: the integer sums are exact, so sampled rows must agree to bf16 rounding."""
    counts = _ragged_counts(16, 600, seed=13)
    n, k = 2048, 7168
    g = torch.Generator(device=DEV).manual_seed(2)
    m = sum(counts)
    a_q = torch.randint(-127, 128, (m, k), device=DEV, generator=g, dtype=torch.int8)
    a_s = torch.rand(m, device=DEV, generator=g) * 0.01 + 0.001
    w_q = torch.randint(-127, 128, (len(counts), n, k), device=DEV, generator=g, dtype=torch.int8)
    w_s = torch.rand(len(counts), n, device=DEV, generator=g) * 0.003 + 0.0015
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    got = ops.grouped_gemm_w8a8(a_q, a_s, w_q, w_s, off)
    torch.cuda.synchronize()
    for e, rows in _sample_rows(counts, 5, seed=6):
        acc = a_q[rows.to(DEV)].cpu().double() @ w_q[e].cpu().double().t()
        want = (acc.float() * w_s[e].cpu().unsqueeze(0) * a_s[rows.to(DEV)].cpu().unsqueeze(1)).to(torch.bfloat16).float()
        gg = got[rows.to(DEV)].cpu().float()
        assert (gg - want).abs().max().item() <= 2 ** -7 * want.abs().max().item()


@pytest.mark.parametrize("world,quant_mode", [(1, 4), (4, 0)])
def test_dispatch_combine_normal_production_shape(world, quant_mode):
    """T = 4096 tokens per rank, top-8 of 256 experts, h = 7168: about 28 tokens per CTA, so the count phase makes
    several passes per CTA and the replicate lists hold thousands of entries.  Row order, source triples and counts
    against ref.plan_dispatch; bf16 rows bit for bit, fp8 rows bit for bit on a sample; combine against the
    weighted sum."""
    t, h, e, k = 4096, 7168, 256, 8
    g = torch.Generator().manual_seed(world + quant_mode)
    topk = [torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]) for _ in range(world)]
    for tk in topk:
        tk[::97, 3] = -1
    gd = torch.Generator(device=DEV).manual_seed(8)
    dx = [torch.randn(t, h, device=DEV, generator=gd).to(torch.bfloat16) for _ in range(world)]
    dw = [torch.rand(t, k, device=DEV, generator=gd) for _ in range(world)]
    dk = [v.to(DEV) for v in topk]
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=5000.0)
    bufs = u.Buffer.virtual(world, cfg, DEV, name=f"prod{world}q{quant_mode}_")

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
        psrc = plan.src.to(DEV).long()
        if quant_mode == 0:
            want_rows = torch.stack(dx)[psrc[:, 0], psrc[:, 1]]
            assert torch.equal(rx, want_rows)
            ys.append(rx.clone())
        else:
            pick = torch.arange(0, psrc.shape[0], 61, device=DEV)
            rows = torch.stack(dx)[psrc[pick, 0], psrc[pick, 1]].cpu()
            q, s = ref.quant_fp8_1x128(rows, quant_mode == 4)
            assert torch.equal(rs[pick].cpu(), s)
            assert torch.equal(rx[pick].cpu().view(torch.uint8), q.view(torch.uint8))
            ys.append(ref.dequant_fp8_1x128(rx, rs).to(torch.bfloat16))

    def comb(r):
        rx, src, cnt, per_e, rs = res[r]
        return ops.moe_combine_prefill(ys[r], dk[r], dw[r], src, cnt, bufs[r].name, r, world)

    outs = run_virtual(comb, world, masks=(PHASE_SEND, PHASE_RECV))
    for r in range(world):
        bufs[r].check()
        if quant_mode == 0:
            xin = dx[r].float()
        else:
            xin = ref.dequant_fp8_1x128(*ref.quant_fp8_1x128(dx[r], quant_mode == 4)).to(torch.bfloat16).float()
        wsum = torch.zeros(t, 1, device=DEV)
        acc = torch.zeros(t, h, device=DEV)
        for kk in range(k):
            ok = (dk[r][:, kk] >= 0).float().unsqueeze(-1)
            acc = acc + xin * (dw[r][:, kk:kk + 1] * ok)
            wsum += dw[r][:, kk:kk + 1] * ok
        got = outs[r].float()
        # fp32 sums in k order on both sides; a fused multiply-add may differ from mul + add in the last bit before the
        # bf16 rounding
        assert ((got - acc).abs() <= 2 ** -7 * acc.abs() + 1e-6).all()
    del res, ys, outs
    for b in bufs:
        b.destroy()


# ---------------------------------------------------------------------------------------------------------------
# The reference's own cases
# ---------------------------------------------------------------------------------------------------------------
def _reference_case(world, bs, e, k, h, inter, seed):
    """Data recipe of the reference's unit test: x in [-5, 5), expert ids arange % E (every expert hit uniformly),
    int8 weights randint(-16, 16), scales rand * 0.003 + 0.0015 rounded through bfloat16, expert scales rand."""
    g = torch.Generator().manual_seed(seed)
    xs = [(torch.rand(bs, h, generator=g) * 10 - 5).to(torch.bfloat16) for _ in range(world)]
    ids = [(torch.arange(r * bs * k, (r + 1) * bs * k) % e).to(torch.int32).view(bs, k) for r in range(world)]
    wts = [torch.rand(bs, k, generator=g) for _ in range(world)]
    w1 = torch.randint(-16, 16, (e, h, 2 * inter), generator=g, dtype=torch.int8)
    w2 = torch.randint(-16, 16, (e, inter, h), generator=g, dtype=torch.int8)
    s1 = (torch.rand(e, 2 * inter, generator=g) * 0.003 + 0.0015).bfloat16().float()
    s2 = (torch.rand(e, h, generator=g) * 0.003 + 0.0015).bfloat16().float()
    return xs, ids, wts, (w1, s1, w2, s2)


@pytest.mark.parametrize("world,bs,tensor_list", [(4, 16, False), (8, 32, True)])
def test_reference_unit_test_cases(world, bs, tensor_list):
    """CASE_4RANK (E = 16, K = 8, bs = 16, h = 7168, I = 2048, stacked weights) and CASE_8RANK (bs = 32, one weight
    tensor per expert) of the reference's unit test, as virtual ranks on one GPU, W8A8 with int32 accumulation."""
    e, k, h, inter = 16, 8, 7168, 2048
    xs, ids, wts, (w1, s1, w2, s2) = _reference_case(world, bs, e, k, h, inter, seed=1000 + world)
    cfg = u.CamConfig(num_experts=e, max_tokens=bs, hidden=h, topk=k, timeout_ms=5000.0)
    bufs = u.Buffer.virtual(world, cfg, DEV, name=f"refut{world}_")
    el = e // world
    dev_w = []
    for r in range(world):
        part = [v[r * el:(r + 1) * el].contiguous().to(DEV) for v in (w1, s1, w2, s2)]
        dev_w.append([list(p.unbind(0)) for p in part] if tensor_list else [[p] for p in part])
    dx, dk, dw = ([v.to(DEV) for v in part] for part in (xs, ids, wts))

    def step(r):
        a, b, c, d = dev_w[r]
        return ops.fused_deep_moe(dx[r], dk[r], a, b, c, d, dw[r], None, None, bufs[r].name, world, r, e, 0, 0, 0, 0)

    every = run_virtual(step, world, return_all=True)
    counts = torch.zeros(e, dtype=torch.int64)
    for r in range(world):
        counts += torch.bincount(ids[r].reshape(-1).long(), minlength=e)
    rows = [torch.zeros(bs, k, h, dtype=torch.bfloat16) for _ in range(world)]
    for ex in range(e):  # one oracle call per expert over the tokens of all ranks
        hits = [torch.nonzero(ids[r] == ex, as_tuple=True) for r in range(world)]
        xcat = torch.cat([xs[r][tok] for r, (tok, _) in enumerate(hits)])
        if xcat.shape[0] == 0:
            continue
        y = ref.expert_mlp_w8a8(xcat, w1[ex].t(), s1[ex], w2[ex].t(), s2[ex])
        pos = 0
        for r, (tok, kk) in enumerate(hits):
            rows[r][tok, kk] = y[pos:pos + tok.numel()]
            pos += tok.numel()
    for r in range(world):
        bufs[r].check()
        want = ref.combine_reference(rows[r], ids[r], wts[r], e).float()
        got = every[PHASE_FINAL][r][0].cpu().float()
        assert torch.allclose(got, want, atol=2.0, rtol=0.02), "outside the reference's own gate"
        assert torch.allclose(got, want, atol=0.01 * want.abs().max().item(), rtol=0.02), (got - want).abs().max()
        assert torch.equal(every[PHASE_RECV][r][1].cpu(), counts[r * el:(r + 1) * el])   # token counts exact
    for b in bufs:
        b.destroy()
