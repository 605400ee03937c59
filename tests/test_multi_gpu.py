"""Real multi-GPU runs (one process per GPU, buffers connected over CUDA IPC, bootstrap on gloo):
normal dispatch/combine, the fused layer and the low-latency pair against the CPU oracle.
Skipped when fewer than two GPUs are visible."""
import datetime
import os
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import free_port

pytestmark = pytest.mark.gpu


def _case(rank, world):
    import umdk_original_b200 as u
    from umdk_original_b200.models import ExpertWeights
    from umdk_original_b200.ops import reference as ref
    ops = torch.ops.umdk_cam_op_lib
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    t, h, inter, e, k = 96, 512, 256, 16, 4
    g = torch.Generator().manual_seed(2024)
    xs = [torch.randn(t, h, generator=g).to(torch.bfloat16) for _ in range(world)]
    topk = [torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]) for _ in range(world)]
    for tk in topk:
        tk[::9, 1] = -1
    wts = [torch.softmax(torch.randn(t, k, generator=g), -1) for _ in range(world)]
    w1q, s1 = ref.quant_fp8_128x128(torch.randn(e, 2 * inter, h, generator=g) * 0.05)
    w2q, s2 = ref.quant_fp8_128x128(torch.randn(e, h, inter, generator=g) * 0.05)
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, ll_max_tokens=t, timeout_ms=5000.0)
    buf = u.Buffer(None, cfg, name="mg", device=dev)
    x, idx, w = xs[rank].to(dev), topk[rank].to(dev), wts[rank].to(dev)
    report = {}
    # normal dispatch (fp8) + combine, three rounds to exercise epochs
    plan = ref.plan_dispatch(topk, e)[rank]
    for _ in range(3):
        rx, src, cnt, per_e, rs = ops.moe_dispatch_prefill_quant(x, idx, w, 0, "mg", rank, world, 3)
        buf.check()
        assert torch.equal(src.cpu().reshape(-1, 3), plan.src)
        assert torch.equal(cnt.cpu(), plan.recv_count)
        rows = torch.stack([xs[s][tt] for s, tt, _ in plan.src.tolist()])
        q, s = ref.quant_fp8_1x128(rows)
        assert torch.equal(rx.cpu().view(torch.uint8), q.view(torch.uint8)) and torch.equal(rs.cpu(), s)
        y = ref.dequant_fp8_1x128(rx.cpu(), rs.cpu()).to(torch.bfloat16).to(dev)
        out = ops.moe_combine_prefill(y, idx, w, src, cnt, "mg", rank, world)
        buf.check()
        xin = ref.dequant_fp8_1x128(*ref.quant_fp8_1x128(xs[rank])).to(torch.bfloat16)
        want = ref.combine_reference(xin.unsqueeze(1).expand(t, k, h).contiguous(), topk[rank], wts[rank], e)
        assert (out.cpu().float() - want.float()).abs().max() == 0
    # fused layer
    el = e // world
    sl = slice(rank * el, (rank + 1) * el)
    lw = ExpertWeights(w1q[sl].contiguous(), s1[sl].contiguous(), w2q[sl].contiguous(), s2[sl].contiguous()).to(dev)
    for _ in range(2):
        out, nums = ops.fused_deep_moe(x, idx, [lw.w1], [lw.s1], [lw.w2], [lw.s2], w, None, None, "mg", world, rank, e,
                                       0, 0, 3, 0)
        buf.check()
    want, _ = ref.fused_moe_fp8_reference(xs[rank], topk[rank], wts[rank], w1q, s1, w2q, s2)
    err = (out.cpu().float() - want.float()).abs().max().item()
    assert err <= 0.06 * want.float().abs().max().item() + 1e-3, err
    assert torch.equal(nums.cpu(), plan.per_expert)
    report["fused_err"] = err
    # the same layer with power-of-two scales: tensor-core block-scaled GEMMs (quantMode 4)
    p1q, p1s = ref.quant_fp8_128x128(ref.dequant_fp8_128x128(w1q, s1), True)
    p2q, p2s = ref.quant_fp8_128x128(ref.dequant_fp8_128x128(w2q, s2), True)
    pw = ExpertWeights(p1q[sl].contiguous(), p1s[sl].contiguous(), p2q[sl].contiguous(), p2s[sl].contiguous()).to(dev)
    for _ in range(2):
        out, nums = ops.fused_deep_moe(x, idx, [pw.w1], [pw.s1], [pw.w2], [pw.s2], w, None, None, "mg", world, rank, e,
                                       0, 0, 4, 0)
        buf.check()
    want, _ = ref.fused_moe_fp8_reference(xs[rank], topk[rank], wts[rank], p1q, p1s, p2q, p2s, ue8m0=True)
    err = (out.cpu().float() - want.float()).abs().max().item()
    assert err <= 0.06 * want.float().abs().max().item() + 1e-3, err
    assert torch.equal(nums.cpu(), plan.per_expert)
    report["fused_mx_err"] = err
    # the same layer through the fused kernels (route 1: the kernel sends the dispatch rows itself over NVLink and starts
    # an expert when its arrival counter is complete; route 2: normal dispatch, then the two GEMMs in one kernel).  The
    # route is chosen when a Buffer is created, so each gets a Buffer of its own.
    for route in (1, 2):
        os.environ["UMDK_CAM_DEEP_FUSE"] = str(route)
        bd = u.Buffer(None, cfg, name=f"mgd{route}", device=dev)
        os.environ["UMDK_CAM_DEEP_FUSE"] = "0"
        for _ in range(3):
            out_d, nums_d = ops.fused_deep_moe(x, idx, [pw.w1], [pw.s1], [pw.w2], [pw.s2], w, None, None, f"mgd{route}",
                                               world, rank, e, 0, 0, 4, 0)
            bd.check()
        assert torch.equal(nums_d.cpu(), plan.per_expert)
        diff = (out_d.float() - out.float()).abs().max().item()
        assert diff <= 0.01 * want.float().abs().max().item() + 1e-3, (route, diff)
        report[f"fused_route{route}_diff"] = diff
        dist.barrier()
        bd.destroy()
    # low-latency pair
    idx32 = idx.to(torch.int32)
    for _ in range(3):
        expand, dyn, eidx, tn, ep_cnt, _tp = ops.moe_dispatch_shmem(x, idx32, None, None, world, rank, e, 1, 0, 0, 0, 0,
                                                                    0, 0, 1, buf.handle)
        buf.check()
        n = plan.src.shape[0]
        assert torch.equal(ep_cnt.cpu(), plan.recv_count)
        assert torch.equal(eidx.cpu(), ref.slots_in_expert(topk[rank], e))
        rows = torch.stack([xs[s][tt] for s, tt, _ in plan.src.tolist()])
        assert torch.equal(expand[:n].cpu(), rows)
        out = ops.moe_combine_shmem(expand, idx32, eidx, ep_cnt, w, None, None, None, None, None, None, world, rank, e,
                                    1, 0, 0, 0, 0, 0, 0, buf.handle, 0, 0)
        buf.check()
        want = ref.combine_reference(xs[rank].unsqueeze(1).expand(t, k, h).contiguous(), topk[rank], wts[rank], e)
        assert (out.cpu().float() - want.float()).abs().max() == 0
    # device barrier across the real GPUs, then flag ping-pong and a peer write between ranks 0 and 1
    for _ in range(3):
        buf.barrier()
    buf.check()
    if rank < 2:
        buf.native.p2p_pingpong(1 - rank, 0, 200, rank == 0)
        buf.native.p2p_write(1 - rank, 512 * 64, 8)
        buf.check()
    dist.barrier()
    buf.destroy()
    return report


def _worker(rank, world, port, q):
    try:
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=120))
        q.put((rank, "ok", _case(rank, world)))
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_gpu_end_to_end(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        r, st, val = q.get(timeout=300)
        res[r] = (st, val)
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    for r, (st, val) in sorted(res.items()):
        assert st == "ok", f"rank {r}: {val}"
