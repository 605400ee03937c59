"""Dispatch / combine micro-benchmarks: latency in microseconds and GB/s per GPU, device-timed,
maximum over ranks.

Two workloads:

``--mode normal``  prefill shapes: 4096 tokens per rank, hidden 7168, 256 experts, top-8 with
    group-limited routing (8 groups, at most 4 per token), dispatch quantised to e4m3 with 1x128
    scales, combine in bf16.
``--mode ll``      decode shapes: 128 tokens per rank, Zipf(s=1.2) bias on the gate logits so that hot
    experts draw several times the mean load, p50 / p99 over ``--iters`` iterations.

``--impl nccl`` times the library-call comparison (quantise + permute kernels of PyTorch and
``all_to_all_single`` over NCCL) on the same routing.  The reference publishes no such numbers
and ships no tool for them (its perftest tools cover URMA verbs only:
src/urma/tools/urma_perftest/perftest_run_test.c:521-595 for the percentile report this follows).

    python -m umdk_original_b200.bench.comm --mode normal --gpus 1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29560 -m umdk_original_b200.bench.comm --mode normal --gpus 8
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

NVLINK_NOMINAL_GBS = 900.0   # per direction per GPU
NVLINK_MEASURED_GBS = 770.0  # peer copy measured on this pool
HBM_FALLBACK_GBS = 6650.0


def _measured_hbm() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:  # noqa: BLE001
        return HBM_FALLBACK_GBS


def _init(n: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n:
        raise SystemExit(f"--gpus {n} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def _barrier(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def _max(v: float, world: int) -> float:
    if world == 1:
        return v
    t = torch.tensor([v], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _time_ops_queued(fns, iters, warmup, world, chunk=50):
    """Device time with the host kept out of the measurement: every chunk starts with a spin kernel
    of a few milliseconds, behind which the host enqueues `chunk` iterations with an event after
    every op; the intervals between events are then pure device time (kernel + waits on peers)."""
    for _ in range(warmup):
        for f in fns:
            f()
    out = [[] for _ in fns]
    done = 0
    while done < iters:
        n = min(chunk, iters - done)
        _barrier(world)
        torch.cuda._sleep(20_000_000)  # about 10 ms of spinning on the device
        evs = []
        for _ in range(n):
            row = [torch.cuda.Event(enable_timing=True) for _ in range(len(fns) + 1)]
            row[0].record()
            for i, f in enumerate(fns):
                f()
                row[i + 1].record()
            evs.append(row)
        torch.cuda.synchronize()
        for row in evs:
            for i in range(len(fns)):
                out[i].append(row[i].elapsed_time(row[i + 1]))
        done += n
    return out


def _time_ops(fns, iters, warmup, world, flush):
    """fns: list of callables run back to back every iteration; returns per-fn lists of ms."""
    from ..utils.timing import flush_l2
    for _ in range(warmup):
        for f in fns:
            f()
    out = [[] for _ in fns]
    for _ in range(iters):
        if flush:
            flush_l2()
        _barrier(world)
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(fns) + 1)]
        evs[0].record()
        for i, f in enumerate(fns):
            f()
            evs[i + 1].record()
        torch.cuda.synchronize()
        for i in range(len(fns)):
            out[i].append(evs[i].elapsed_time(evs[i + 1]))
    return out


def _pct(v, q):
    s = sorted(v)
    return s[min(len(s) - 1, int(q * len(s)))]


def _remote_rows(idx: torch.Tensor, num_experts: int, world: int, rank: int):
    """(pairs, pairs whose expert lives on another rank, distinct (token, other rank) combinations).  The last
    number is what the normal dispatch of this library puts on NVLink: a token crosses once per destination rank
    and is replicated there; the NCCL arm and both combines move one row per pair."""
    el = num_experts // world
    dst = torch.where(idx >= 0, idx // el, torch.full_like(idx, -1))
    total = int((dst >= 0).sum())
    remote = int(((dst >= 0) & (dst != rank)).sum())
    hit = torch.zeros(idx.shape[0], world + 1, dtype=torch.bool, device=idx.device)
    hit.scatter_(1, torch.where(dst >= 0, dst, torch.full_like(dst, world)), True)
    hit[:, rank] = False
    unique_remote = int(hit[:, :world].sum())
    return total, remote, unique_remote


def run(args):
    import umdk_original_b200 as u
    from ..models import BY_NAME, route, zipf_bias

    rank, world, local = _init(args.gpus)
    dev = torch.device("cuda", local)
    ll = args.mode == "ll"
    cfg = BY_NAME["deepseek-v3-decode" if ll else "deepseek-v3-moe"]
    tokens = args.tokens or cfg.tokens_per_rank
    e, k, h = cfg.num_experts, cfg.topk, cfg.hidden
    g = torch.Generator(device=dev)
    g.manual_seed(4321 + rank)
    x = torch.randn(tokens, h, device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn(tokens, e, device=dev, generator=g)
    if ll:
        gb = torch.Generator().manual_seed(7)  # the same hot experts on every rank
        logits = logits + zipf_bias(e, 1.2, generator=gb).to(dev)
        idx, w = route(logits, k)
    else:
        idx, w = route(logits, k, 8, 4)
    idx = idx.contiguous()
    w = w.float().contiguous()
    total_rows, remote_rows, unique_remote_rows = _remote_rows(idx, e, world, rank)
    nscale = h // 128
    disp_row_bytes = h + nscale * 4 + 12
    comb_row_bytes = h * 2
    group = dist.group.WORLD if world > 1 else None
    result = {"mode": args.mode, "impl": args.impl, "n_gpus": world, "tokens_per_rank": tokens, "hidden": h,
              "num_experts": e, "topk": k, "iters": args.iters, "dispatch_dtype": "e4m3 + fp32 1x128 scales",
              "combine_dtype": "bf16", "timing": "CUDA events per op, barrier before every iteration, max over ranks",
              "l2": "flushed before every iteration" if args.flush else "not flushed (decode loop reuses buffers)"}

    if args.impl == "ours":
        cam = u.CamConfig(num_experts=e, max_tokens=tokens if not ll else 128, hidden=h, topk=k,
                          ll_max_tokens=tokens if ll else 0, timeout_ms=20000.0)
        buf = u.Buffer(group, cam, name="commbench", device=dev)
        ops = torch.ops.umdk_cam_op_lib
        state = {}
        if ll:
            idx32 = idx.to(torch.int32)

            def disp():
                state["d"] = ops.moe_dispatch_shmem(x, idx32, None, None, world, rank, e, 1, 0, 0, 0, 0, 3, 0, 1,
                                                    buf.handle)

            disp()
            y = torch.randn(state["d"][0].shape[0], h, device=dev, generator=g).to(torch.bfloat16)

            def comb():
                d = state["d"]
                state["o"] = ops.moe_combine_shmem(y, idx32, d[2], d[4], w, None, None, None, None, None, None, world,
                                                   rank, e, 1, 0, 0, 0, 0, 0, 0, buf.handle, 0, 0)
        else:
            cap = buf.capacity

            def disp():
                state["d"] = ops.moe_dispatch_prefill_quant(x, idx, w, cap, "commbench", rank, world, 3)

            y = torch.randn(cap, h, device=dev, generator=g).to(torch.bfloat16)

            def comb():
                d = state["d"]
                state["o"] = ops.moe_combine_prefill(y, idx, w, d[1], d[2], "commbench", rank, world)

        if ll and args.graph:
            # one CUDA graph per op (epochs live on the device, so replays stay in step across ranks)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    disp()
                    comb()
            torch.cuda.current_stream().wait_stream(side)
            _barrier(world)
            g_disp, g_comb = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_disp):
                disp()
            with torch.cuda.graph(g_comb, pool=g_disp.pool()):
                comb()
            t_disp, t_comb = _time_ops_queued([g_disp.replay, g_comb.replay], args.iters, args.warmup, world)
            result["timing"] = ("each op captured in a CUDA graph; CUDA events after every replay, iterations enqueued "
                                "behind a device spin, max over ranks")
        elif ll:
            t_disp, t_comb = _time_ops_queued([disp, comb], args.iters, args.warmup, world)
            result["timing"] = ("CUDA events after every op, iterations enqueued behind a device spin so that host "
                                "launch latency is outside the intervals, max over ranks")
        else:
            t_disp, t_comb = _time_ops([disp, comb], args.iters, args.warmup, world, args.flush)
        buf.check()
        buf.destroy()
    else:
        el = e // world
        flat = idx.reshape(-1)

        def disp():
            # quantise, sort pairs by expert, exchange counts (host sync for the split sizes), exchange rows
            xf = x.float().view(tokens, nscale, 128)
            amax = xf.abs().amax(dim=-1).clamp_min(1e-4)
            q = (xf * (448.0 / amax).unsqueeze(-1)).to(torch.float8_e4m3fn).view(tokens, h)
            sc = amax / 448.0
            order = torch.argsort(flat, stable=True)
            counts = torch.bincount(flat, minlength=e)
            recv_counts = torch.empty_like(counts)
            if world > 1:
                dist.all_to_all_single(recv_counts, counts)
            else:
                recv_counts.copy_(counts)
            rc = recv_counts.view(world, el).sum(dim=1).tolist()
            scn = counts.view(world, el).sum(dim=1).tolist()
            send_q = q[order // k].view(torch.uint8)
            send_s = sc[order // k]
            recv_q = send_q.new_empty((sum(rc), h))
            recv_s = send_s.new_empty((sum(rc), nscale))
            if world > 1:
                dist.all_to_all_single(recv_q, send_q, output_split_sizes=rc, input_split_sizes=scn)
                dist.all_to_all_single(recv_s, send_s, output_split_sizes=rc, input_split_sizes=scn)
            else:
                recv_q.copy_(send_q)
                recv_s.copy_(send_s)
            state_b["rc"], state_b["sc"], state_b["order"], state_b["n"] = rc, scn, order, sum(rc)

        state_b = {}
        disp()
        yb = torch.randn(state_b["n"], h, device=dev, generator=g).to(torch.bfloat16)

        def comb():
            ret = yb.new_empty((tokens * k, h))
            if world > 1:
                dist.all_to_all_single(ret, yb, output_split_sizes=state_b["sc"], input_split_sizes=state_b["rc"])
            else:
                ret.copy_(yb)
            rows = torch.empty_like(ret)
            rows[state_b["order"]] = ret
            state_b["o"] = (rows.view(tokens, k, h).float() * w.unsqueeze(-1)).sum(dim=1).to(torch.bfloat16)

        if ll:
            t_disp, t_comb = _time_ops_queued([disp, comb], args.iters, args.warmup, world)
        else:
            t_disp, t_comb = _time_ops([disp, comb], args.iters, args.warmup, world, args.flush)

    hbm = _measured_hbm()
    for name, ts, row_bytes in (("dispatch", t_disp, disp_row_bytes), ("combine", t_comb, comb_row_bytes)):
        p50 = _max(_pct(ts, 0.5), world) * 1e3
        p99 = _max(_pct(ts, 0.99), world) * 1e3
        mean = _max(statistics.fmean(ts), world) * 1e3
        # bytes that actually cross NVLink: this library's normal dispatch sends a token once per destination rank
        # (12 bytes of source triple per pair still travel); everything else moves one row per remote pair
        dedup = name == "dispatch" and args.impl == "ours" and not ll
        wire_rows = unique_remote_rows if dedup else remote_rows
        nv_bytes = wire_rows * row_bytes + (remote_rows - wire_rows) * 20
        all_bytes = total_rows * row_bytes
        result[name] = {
            "p50_us": p50, "p99_us": p99, "mean_us": mean,
            "rows": total_rows, "remote_rows": remote_rows, "rows_on_the_wire": wire_rows,
            "nvlink_bytes_per_gpu": nv_bytes, "payload_bytes_per_gpu": all_bytes,
            "nvlink_gbs_per_gpu": nv_bytes / (p50 * 1e-6) / 1e9 if world > 1 else 0.0,
            "payload_gbs_per_gpu": all_bytes / (p50 * 1e-6) / 1e9,
        }
        if world > 1:
            result[name]["frac_of_nvlink_nominal_900"] = result[name]["nvlink_gbs_per_gpu"] / NVLINK_NOMINAL_GBS
            result[name]["frac_of_nvlink_measured_770"] = result[name]["nvlink_gbs_per_gpu"] / NVLINK_MEASURED_GBS
        else:
            # one GPU: a local permutation, bounded by HBM (read + write of every row)
            result[name]["frac_of_hbm_measured"] = 2 * all_bytes / (p50 * 1e-6) / 1e9 / hbm
    if rank == 0:
        print(json.dumps(result))
    _barrier(world)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--mode", default="normal", choices=["normal", "ll"])
    ap.add_argument("--impl", default="ours", choices=["ours", "nccl"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--iters", type=int, default=0)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--flush", action="store_true", help="flush L2 before every iteration")
    ap.add_argument("--graph", action="store_true", help="low-latency mode: replay the ops from CUDA graphs")
    a = ap.parse_args()
    if a.iters <= 0:
        a.iters = 1000 if a.mode == "ll" else 30
    if a.mode == "normal":
        a.flush = True
    run(a)


if __name__ == "__main__":
    main()
