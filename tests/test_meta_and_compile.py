"""Shape inference (Meta key) and graph capture of the four ops whose output shapes do not depend on data:
fused_deep_moe, get_dispatch_layout, moe_dispatch_shmem, moe_combine_shmem.

The reference registers Meta implementations for its fused and shmem ops so that they can be traced in graph
mode (pybind/fused_deep_moe.cpp:87-122, 220-235), parametrises its unit test over graph and eager mode
(test_fused_deep_moe.py:365) and compiles its example with torchair (examples/fused_deep_moe_sample.py:30-43).
Here the Meta kernels are checked with tensors on the "meta" device (no GPU needed) and, on a GPU, the ops are
traced by torch.compile(fullgraph=True) and must return what the eager call returns."""
import pytest
import torch

import umdk_original_b200 as u  # noqa: F401  (registers the op library)
from umdk_original_b200.ops import cam_ops

ops = torch.ops.umdk_cam_op_lib
needs_native = pytest.mark.skipif(not cam_ops.native_loaded(), reason="native extension not built")


def _m(*shape, dtype=torch.float32):
    return torch.empty(*shape, dtype=dtype, device="meta")


@needs_native
def test_meta_fused_deep_moe_shapes():
    bs, h, k, e, r, inter = 16, 7168, 8, 16, 4, 2048
    el = e // r
    x = _m(bs, h, dtype=torch.bfloat16)
    ids = _m(bs, k, dtype=torch.int32)
    w1 = [_m(el, h, 2 * inter, dtype=torch.int8)]
    s1 = [_m(el, 2 * inter)]
    w2 = [_m(el, inter, h, dtype=torch.int8)]
    s2 = [_m(el, h)]
    out, nums = ops.fused_deep_moe(x, ids, w1, s1, w2, s2, _m(bs, k), None, None, "g", r, 1, e, 0, 0, 0, 0)
    assert out.shape == (bs, h) and out.dtype == torch.bfloat16 and out.device.type == "meta"
    assert nums.shape == (el,) and nums.dtype == torch.int64
    # a shared-expert rank holds one expert (pybind/fused_deep_moe.cpp:26-79)
    out, nums = ops.fused_deep_moe(x, ids, w1, s1, w2, s2, _m(bs, k), None, None, "g", r, 0, 12, 1, 1, 0, 0)
    assert nums.shape == (1,)


@needs_native
def test_meta_layout_and_low_latency_shapes():
    t, k, e, r, h = 48, 8, 64, 8, 1024
    a, b, c = ops.get_dispatch_layout(_m(t, k, dtype=torch.int64), e, r)
    assert a.shape == (r,) and b.shape == (e,) and c.shape == (t, r) and c.dtype == torch.bool
    el = e // r
    outs = ops.moe_dispatch_shmem(_m(t, h, dtype=torch.bfloat16), _m(t, k, dtype=torch.int32), None, None, r, 0, e, 1, 0, 0,
                                  0, 0, 3, 0, 1, 1)
    rows = t * r * min(el, k)          # worst-case rows, as in pybind/moe_dispatch_shmem.cpp:50-62
    assert outs[0].shape == (rows, h) and outs[0].dtype == torch.float8_e4m3fn
    assert outs[2].shape == (t * k,) and outs[3].shape == (el,) and outs[4].shape == (r * el,)
    y = ops.moe_combine_shmem(_m(rows, h, dtype=torch.bfloat16), _m(t, k, dtype=torch.int32), outs[2], outs[4], _m(t, k),
                              None, None, None, None, None, None, r, 0, e, 1, 0, 0, 0, 0, 0, 0, 1, 0, 0)
    assert y.shape == (t, h) and y.dtype == torch.bfloat16


@pytest.mark.gpu
def test_compiled_fused_layer_and_low_latency_ops_match_eager():
    from umdk_original_b200.models import TINY, FusedMoE
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = TINY
    t = cfg.tokens_per_rank
    buf = u.Buffer(None, u.CamConfig(num_experts=cfg.num_experts, max_tokens=t, hidden=cfg.hidden, topk=cfg.topk,
                                     ll_max_tokens=t, timeout_ms=2000.0), name="compiled", device=dev, rank=0, num_ranks=1)
    layer = FusedMoE(cfg, buf, seed=0)
    x = torch.randn(t, cfg.hidden, device=dev).to(torch.bfloat16)
    idx, w = layer.route(x)
    wts = layer.weights

    def fused(x, idx, w):
        out, nums = ops.fused_deep_moe(x, idx, [wts.w1], [wts.s1], [wts.w2], [wts.s2], w, None, None, "compiled", 1, 0,
                                       cfg.num_experts, 0, 0, layer.quant_mode, 0)
        return out * 2, nums

    def low_latency(x, idx32, w):
        d = ops.moe_dispatch_shmem(x, idx32, None, None, 1, 0, cfg.num_experts, 1, 0, 0, 0, 0, 0, 0, 1, buf.handle)
        lay = ops.get_dispatch_layout(idx32.long(), cfg.num_experts, 1)
        return ops.moe_combine_shmem(d[0], idx32, d[2], d[4], w, None, None, None, None, None, None, 1, 0, cfg.num_experts,
                                     1, 0, 0, 0, 0, 0, 0, buf.handle, 0, 0), lay[1]

    want = fused(x, idx, w.float())
    got = torch.compile(fused, fullgraph=True, backend="aot_eager")(x, idx, w.float())
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    idx32 = idx.to(torch.int32)
    want = low_latency(x, idx32, w.float())
    got = torch.compile(low_latency, fullgraph=True, backend="aot_eager")(x, idx32, w.float())
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    buf.check()
    buf.destroy()
