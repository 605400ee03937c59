"""CUDA-graph capture of the ops: epochs live on the device and masks are applied on the device,
so a captured decode step (low-latency dispatch + combine) or a whole fused layer can be replayed
with new inputs written into the captured tensors."""
import pytest
import torch

import umdk_original_b200 as u
from umdk_original_b200.models import ExpertWeights
from umdk_original_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
ops = torch.ops.umdk_cam_op_lib
DEV = torch.device("cuda", 0)


def _capture(fn, warmup=2):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = fn()
    return g, out


def test_low_latency_pair_replays_in_a_graph():
    t, h, e, k = 32, 512, 8, 2
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, ll_max_tokens=t, timeout_ms=2000.0)
    buf = u.Buffer(None, cfg, name="graph_ll", device=DEV, rank=0, num_ranks=1)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(t, h, generator=gen).to(torch.bfloat16).to(DEV)
    ids = torch.randint(0, e, (t, k), generator=gen).to(torch.int32).to(DEV)
    w = torch.rand(t, k, generator=gen).to(DEV)
    mask = torch.ones(t, dtype=torch.bool, device=DEV)

    def step():
        d = ops.moe_dispatch_shmem(x, ids, None, mask, 1, 0, e, 1, 0, 0, 0, 0, 0, 0, 1, buf.handle)
        return ops.moe_combine_shmem(d[0], ids, d[2], d[4], w, None, mask, None, None, None, None, 1, 0, e, 1, 0, 0, 0,
                                     0, 0, 0, buf.handle, 0, 0)

    graph, out = _capture(step)
    for it in range(4):
        x.copy_(torch.randn(t, h, generator=gen).to(torch.bfloat16))
        ids.copy_(torch.randint(0, e, (t, k), generator=gen).to(torch.int32))
        m = torch.ones(t, dtype=torch.bool)
        m[t - 3 * it:] = False
        mask.copy_(m)
        graph.replay()
        torch.cuda.synchronize()
        buf.check()
        masked = ids.cpu().clone()
        masked[~m] = -1
        want = ref.combine_reference(x.cpu().unsqueeze(1).expand(t, k, h).contiguous(), masked, w.cpu(), e)
        assert (out.cpu().float() - want.float()).abs().max() == 0.0
    buf.destroy()


def test_fused_layer_replays_in_a_graph():
    t, h, inter, e, k = 32, 256, 128, 4, 2
    gen = torch.Generator().manual_seed(1)
    w1q, s1 = ref.quant_fp8_128x128(torch.randn(e, 2 * inter, h, generator=gen) * 0.05, True)
    w2q, s2 = ref.quant_fp8_128x128(torch.randn(e, h, inter, generator=gen) * 0.05, True)
    wts = ExpertWeights(w1q, s1, w2q, s2).to(DEV)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=3000.0)
    buf = u.Buffer(None, cfg, name="graph_fused", device=DEV, rank=0, num_ranks=1)
    x = torch.randn(t, h, generator=gen).to(torch.bfloat16).to(DEV)
    ids = torch.stack([torch.randperm(e, generator=gen)[:k] for _ in range(t)]).to(DEV)
    sc = torch.softmax(torch.randn(t, k, generator=gen), -1).to(DEV)

    def step():
        return ops.fused_deep_moe(x, ids, [wts.w1], [wts.s1], [wts.w2], [wts.s2], sc, None, None, "graph_fused", 1, 0, e,
                                  0, 0, 4, 0)

    graph, (out, nums) = _capture(step)
    for _ in range(3):
        x.copy_(torch.randn(t, h, generator=gen).to(torch.bfloat16))
        ids.copy_(torch.stack([torch.randperm(e, generator=gen)[:k] for _ in range(t)]))
        graph.replay()
        torch.cuda.synchronize()
        buf.check()
        want, counts = ref.fused_moe_fp8_reference(x.cpu(), ids.cpu(), sc.cpu(), w1q, s1, w2q, s2, ue8m0=True)
        assert torch.equal(nums.cpu(), counts)
        assert (out.cpu().float() - want.float()).abs().max() <= 0.06 * want.float().abs().max() + 1e-3
    buf.destroy()
