"""Example: the fused MoE op against the same layer built from the library's separate ops.

It plays the part of the reference's ``src/cam/examples/fused_deep_moe_sample.py`` (``run_once``,
lines 366-443: a ``DecodeMoeOps`` chain of dispatch + two grouped matmuls + combine against the
fused operator) on GPUs: every rank owns ``moe_expert_num / ep_world_size`` experts, routes its
own tokens, and the two paths must agree.  Three variants, as there:

* base                      all tokens active, one stacked weight tensor per argument
* ``--with-mask``           an ``x_active_mask`` prefix of the tokens takes part
* ``--dynamic-eplb``        weights passed as a list of per-expert tensors

    python -m umdk_original_b200.examples.fused_deep_moe_sample --world 1
    python -m umdk_original_b200.examples.fused_deep_moe_sample --world 4 --with-mask

On a machine without GPUs the same script runs its ranks as gloo processes on the CPU
implementation of the ops (slow; use the small default sizes).
"""
from __future__ import annotations

import argparse
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

BASE_KWARGS = {
    "batch_size": 64,
    "token_hidden_size": 1024,
    "moe_intermediate_size": 512,
    "ep_world_size": 1,
    "moe_expert_num": 16,
    "top_k": 4,
    "with_mask": False,
    "dynamic_eplb": False,
}


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class SmallOps(torch.nn.Module):
    """Unfused chain: dispatch (fp8 1x128) -> grouped GEMM + SwiGLU + requant -> grouped GEMM -> combine."""

    def __init__(self, weights, group_name, rank, world, num_experts, ue8m0):
        super().__init__()
        self.w, self.name, self.rank, self.world, self.e, self.ue8m0 = weights, group_name, rank, world, num_experts, ue8m0

    def forward(self, x, expert_ids, expert_scales, x_active_mask=None):
        ops = torch.ops.umdk_cam_op_lib
        ids = expert_ids
        if x_active_mask is not None:
            ids = expert_ids.clone()
            ids[int(x_active_mask.sum()):] = -1
        rx, src, cnt, per_e, rs = ops.moe_dispatch_prefill_quant(x, ids, expert_scales, 0, self.name, self.rank,
                                                                 self.world, 4 if self.ue8m0 else 3)
        off = torch.cat([per_e.new_zeros(1), per_e.cumsum(0)]).to(torch.int32).to(x.device)
        if rx.shape[0] == 0:
            y = torch.zeros(0, x.shape[1], dtype=torch.bfloat16, device=x.device)
        else:
            aq, a_s = ops.grouped_gemm_fp8_swiglu(rx, rs, self.w.w1, self.w.s1, off, self.ue8m0)
            y = ops.grouped_gemm_fp8(aq, a_s, self.w.w2, self.w.s2, off, self.ue8m0)
        out = ops.moe_combine_prefill(y, ids, expert_scales, src, cnt, self.name, self.rank, self.world)
        return out, per_e.to(torch.int64)


class FusionOp(torch.nn.Module):
    """One call of ``fused_deep_moe``."""

    def __init__(self, weights, group_name, rank, world, num_experts, ue8m0, as_list=False):
        super().__init__()
        self.w, self.name, self.rank, self.world, self.e, self.ue8m0 = weights, group_name, rank, world, num_experts, ue8m0
        self.as_list = as_list

    def forward(self, x, expert_ids, expert_scales, x_active_mask=None):
        w = self.w
        if self.as_list:  # one tensor per local expert ("tensor list", used with dynamic expert placement)
            args = [list(w.w1.unbind(0)), list(w.s1.unbind(0)), list(w.w2.unbind(0)), list(w.s2.unbind(0))]
        else:
            args = [[w.w1], [w.s1], [w.w2], [w.s2]]
        out, nums = torch.ops.umdk_cam_op_lib.fused_deep_moe(
            x, expert_ids, *args, expert_scales, None, x_active_mask, self.name, self.world, self.rank, self.e, 0, 0,
            4 if self.ue8m0 else 3, 0)
        return out, nums


def run_once(rank: int, world: int, port: int, kw: dict, results):
    import umdk_original_b200 as u
    from umdk_original_b200.models import random_fp8_experts

    use_gpu = torch.cuda.is_available()
    if use_gpu:
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
    else:
        dev = torch.device("cpu")
    if world > 1:
        dist.init_process_group("nccl" if use_gpu else "gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                                world_size=world)
    t, h, inter = kw["batch_size"], kw["token_hidden_size"], kw["moe_intermediate_size"]
    e, k = kw["moe_expert_num"], kw["top_k"]
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=10000.0)
    buf = u.Buffer(dist.group.WORLD if world > 1 else None, cfg, name="sample", device=dev, rank=rank, num_ranks=world)
    torch.manual_seed(42 + rank)
    weights = random_fp8_experts(e // world, h, inter, device=dev, std=0.05, seed=1000 + rank)
    x = torch.randn(t, h, device=dev).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(e, device=dev)[:k] for _ in range(t)]).to(torch.int64)
    scales = torch.softmax(torch.randn(t, k, device=dev), dim=-1)
    mask = None
    if kw["with_mask"]:
        mask = torch.zeros(t, dtype=torch.bool, device=dev)
        mask[: max(1, (3 * t) // 4)] = True
    small = SmallOps(weights, "sample", rank, world, e, True)
    fused = FusionOp(weights, "sample", rank, world, e, True, as_list=kw["dynamic_eplb"])
    out_s, n_s = small(x, ids, scales, mask)
    out_f, n_f = fused(x, ids, scales, mask)
    buf.check()
    err = (out_s.float() - out_f.float()).abs().max().item()
    ok = bool(torch.equal(n_s.cpu(), n_f.cpu())) and err <= 2e-2 * out_s.float().abs().max().item() + 1e-3
    print(f"[rank {rank}] tokens per local expert {n_f.tolist()}  max |fused - small| = {err:.3e}  {'OK' if ok else 'MISMATCH'}")
    if results is not None:
        results[rank] = ok
    buf.destroy()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return ok


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--world", type=int, default=BASE_KWARGS["ep_world_size"])
    ap.add_argument("--batch-size", type=int, default=BASE_KWARGS["batch_size"])
    ap.add_argument("--hidden", type=int, default=BASE_KWARGS["token_hidden_size"])
    ap.add_argument("--intermediate", type=int, default=BASE_KWARGS["moe_intermediate_size"])
    ap.add_argument("--experts", type=int, default=BASE_KWARGS["moe_expert_num"])
    ap.add_argument("--top-k", type=int, default=BASE_KWARGS["top_k"])
    ap.add_argument("--with-mask", action="store_true")
    ap.add_argument("--dynamic-eplb", action="store_true")
    a = ap.parse_args()
    kw = dict(BASE_KWARGS, batch_size=a.batch_size, token_hidden_size=a.hidden, moe_intermediate_size=a.intermediate,
              ep_world_size=a.world, moe_expert_num=a.experts, top_k=a.top_k, with_mask=a.with_mask,
              dynamic_eplb=a.dynamic_eplb)
    if a.world == 1:
        ok = run_once(0, 1, 0, kw, None)
    else:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        mgr = mp.Manager()
        results = mgr.dict()
        mp.spawn(run_once, args=(a.world, _free_port(), kw, results), nprocs=a.world, join=True)
        ok = all(results.get(r, False) for r in range(a.world))
    print("fused_deep_moe sample:", "PASS" if ok else "FAIL")
    raise SystemExit(0 if ok else 1)


if __name__ == "__main__":
    main()
