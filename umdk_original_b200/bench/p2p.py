"""One-sided P2P microbenchmark on the symmetric buffer: write bandwidth to one peer and flag
round-trip latency, the two quantities the dispatch / combine rooflines are built from.
Needs at least two GPUs (one rank per GPU).  The part of ``urma_perftest write_bw / write_lat``
(src/urma/tools/urma_perftest/perftest_parameters.c:57-64) for NVLink peer memory.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29570 -m umdk_original_b200.bench.p2p --gpus 2
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--mbytes", type=int, default=512)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--pingpongs", type=int, default=2000)
    a = ap.parse_args()
    import umdk_original_b200 as u

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    assert world == a.gpus and world >= 2, "run with torch.distributed.run on at least 2 GPUs"
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    nbytes = a.mbytes << 20
    rows = nbytes // (7168 * 2) + 1
    cfg = u.CamConfig(num_experts=world, max_tokens=rows, hidden=7168, topk=1, capacity=rows, timeout_ms=20000.0)
    buf = u.Buffer(dist.group.WORLD, cfg, name="p2p", device=torch.device("cuda", local))
    nat = buf.native
    peer = (rank + 1) % world
    out = {"n_gpus": world, "bytes": nbytes}
    # every rank writes to its right neighbour at the same time (each link direction carries one stream)
    for grid, key in ((0, "write_all_sms"), (32, "write_32_ctas")):
        for _ in range(3):
            nat.p2p_write(peer, nbytes, grid)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            nat.p2p_write(peer, nbytes, grid)
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / a.iters], device="cuda", dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        out[key + "_gbs"] = nbytes / (ms.item() * 1e-3) / 1e9
    # flag round trips between ranks 0 and 1
    if rank < 2:
        other = 1 - rank
        base = 0
        for rep in range(3):
            dist.barrier(group=None) if False else None
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            nat.p2p_pingpong(other, base, a.pingpongs, rank == 0)
            e1.record()
            torch.cuda.synchronize()
            base += a.pingpongs
            rtt = e0.elapsed_time(e1) * 1e3 / a.pingpongs
        out["flag_round_trip_us"] = rtt
    buf.check()
    dist.barrier()
    if rank == 0:
        out["frac_of_nvlink_measured_770"] = out["write_all_sms_gbs"] / 770.0
        print(json.dumps(out))
    buf.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
