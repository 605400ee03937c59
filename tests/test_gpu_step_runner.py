"""MoEStepRunner: pinned host inputs -> device -> fused layer -> host record, with launches running one
step ahead of the reads.  Every step's record must equal what a direct call of the layer gives."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_pipelined_steps_return_each_steps_own_record():
    import umdk_original_b200 as u
    from umdk_original_b200.models import TINY, FusedMoE, MoEStepRunner
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = TINY
    t = cfg.tokens_per_rank
    buf = u.Buffer(None, u.CamConfig(num_experts=cfg.num_experts, max_tokens=t, hidden=cfg.hidden, topk=cfg.topk,
                                     timeout_ms=2000.0), name="runner", device=dev, rank=0, num_ranks=1)
    layer = FusedMoE(cfg, buf, seed=0)
    g = torch.Generator().manual_seed(5)
    host, want, want_out = [], [], []
    for _ in range(5):
        x = torch.randn(t, cfg.hidden, generator=g).to(torch.bfloat16)
        idx, w = layer.route(x.to(dev))
        host.append((x.pin_memory(), idx.cpu().pin_memory(), w.float().cpu().pin_memory()))
        out, nums = layer(x.to(dev), idx, w)
        want.append(torch.cat([nums.float(), out.sum(dtype=torch.float32).reshape(1)]).cpu())
        want_out.append(out.cpu())
    runner = MoEStepRunner(layer, t, time_copies=True)
    assert runner.h2d_bytes == t * (cfg.hidden * 2 + cfg.topk * 12)
    assert runner.d2h_bytes == 4 * (layer.num_local + 1) + t * cfg.hidden * 2     # the record and the output itself
    got, got_out = [], []
    runner.stage(*host[0])
    pending = None
    for i in range(len(host)):
        ticket = runner.run()
        if i + 1 < len(host):
            runner.stage(*host[i + 1])
        if pending is not None:
            got.append(runner.result(pending).clone())
            got_out.append(runner.output(pending).clone())
        pending = ticket
    got.append(runner.result(pending).clone())
    got_out.append(runner.output(pending).clone())
    assert torch.equal(runner.finish(), got[-1])
    buf.check()
    times = runner.copy_times()
    assert times["h2d_ms"] > 0.0 and times["d2h_ms"] > 0.0 and runner.copy_times() == {"h2d_ms": 0.0, "d2h_ms": 0.0}
    for i, (a, b) in enumerate(zip(got, want)):
        assert torch.equal(a[:-1], b[:-1]), f"step {i}: token counts differ"
        assert abs(float(a[-1]) - float(b[-1])) <= 1e-3 * max(1.0, abs(float(b[-1]))), f"step {i}: checksum differs"
        assert torch.equal(got_out[i], want_out[i]), f"step {i}: the output read back on the host differs"
    with pytest.raises(AssertionError):
        runner.result(0)  # long overwritten
    buf.destroy()


def test_layer_converts_fp32_block_scales_on_request():
    """Weights with arbitrary fp32 block scales: the layer runs quantMode 3 as they are and quantMode 4 after the
    one-time conversion; both agree with the oracle of their own weights."""
    import umdk_original_b200 as u
    from umdk_original_b200.models import TINY, FusedMoE
    from umdk_original_b200.models.weights import random_fp8_experts
    from umdk_original_b200.ops import reference as ref
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = TINY
    t = cfg.tokens_per_rank
    w = random_fp8_experts(cfg.num_experts, cfg.hidden, cfg.intermediate, ue8m0=False, seed=11)
    x = (torch.randn(t, cfg.hidden, generator=torch.Generator().manual_seed(2))).to(torch.bfloat16)
    for convert, mode in ((False, 3), (True, 4)):
        buf = u.Buffer(None, u.CamConfig(num_experts=cfg.num_experts, max_tokens=t, hidden=cfg.hidden, topk=cfg.topk,
                                         timeout_ms=2000.0), name=f"conv{mode}", device=dev, rank=0, num_ranks=1)
        layer = FusedMoE(cfg, buf, weights=w, convert_scales=convert)
        assert layer.quant_mode == mode
        idx, wt = layer.route(x.to(dev))
        out, nums = layer(x.to(dev), idx, wt)
        buf.check()
        lw = layer.weights
        want, counts = ref.fused_moe_fp8_reference(x, idx.cpu(), wt.cpu(), lw.w1.cpu(), lw.s1.cpu(), lw.w2.cpu(),
                                                   lw.s2.cpu(), ue8m0=mode == 4)
        assert torch.equal(nums.cpu(), counts)
        scale = want.float().abs().max().item()
        assert (out.cpu().float() - want.float()).abs().max().item() <= 0.05 * scale + 1e-3
        buf.destroy()
