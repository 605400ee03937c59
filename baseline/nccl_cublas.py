"""Comparison arm: the same MoE layer built from library calls only --
``torch.distributed.all_to_all_single`` over NCCL for dispatch and combine, cuBLAS GEMMs for the
experts (``torch._scaled_mm`` with row-wise fp8 scales per expert, or ``torch._grouped_mm`` in
bf16 when that is not available), PyTorch elementwise kernels for permutation, SwiGLU and the
weighted sum.  It is what the product has to beat; nothing here is imported by the package."""
from __future__ import annotations

import json
import time

import torch
import torch.distributed as dist


class BaselineMoE:
    def __init__(self, cfg, rank, world, dev, seed=0, gemm="fp8_per_expert"):
        """gemm: "fp8_per_expert" (cuBLAS fp8 torch._scaled_mm, one call per local expert) or "bf16_grouped"
        (the library's bf16 grouped GEMM torch._grouped_mm: no per-expert loop, twice the bytes per weight)."""
        self.cfg, self.rank, self.world, self.dev = cfg, rank, world, dev
        self.want_gemm = gemm
        self.el = cfg.num_experts // world
        g = torch.Generator(device=dev)
        g.manual_seed(seed * 1000 + rank)
        h, i = cfg.hidden, cfg.intermediate
        self.mode = None
        w1, w2 = [], []
        for _ in range(self.el):
            w1.append((torch.randn(2 * i, h, device=dev, generator=g) * 0.02).to(torch.bfloat16))
            w2.append((torch.randn(h, i, device=dev, generator=g) * 0.02).to(torch.bfloat16))
        self.w1 = torch.stack(w1)  # [El, 2I, h]
        self.w2 = torch.stack(w2)  # [El, h, I]
        del w1, w2
        self._pick_mode()

    def _pick_mode(self):
        if self.want_gemm == "bf16_grouped":
            self.mode = "bf16_grouped_mm"
            self.w1t = self.w1.transpose(1, 2).contiguous()  # [El, h, 2I]
            self.w2t = self.w2.transpose(1, 2).contiguous()  # [El, I, h]
            del self.w1, self.w2
            return
        try:
            self.w1q, self.s1 = self._quant_rows(self.w1)
            self.w2q, self.s2 = self._quant_rows(self.w2)
            a = torch.randn(64, self.cfg.hidden, device=self.dev).to(torch.bfloat16)
            self._mlp_fp8(a, 0)
            torch.cuda.synchronize()
            self.mode = "cublas_fp8_rowwise_scaled_mm_per_expert"
            del self.w1, self.w2
        except Exception:  # noqa: BLE001
            self.mode = "bf16_grouped_mm"
            self.w1t = self.w1.transpose(1, 2).contiguous()  # [El, h, 2I]
            self.w2t = self.w2.transpose(1, 2).contiguous()  # [El, I, h]

    @staticmethod
    def _quant_rows(w):
        amax = w.float().abs().amax(dim=-1, keepdim=True).clamp_min(1e-4)
        s = amax / 448.0
        return (w.float() / s).to(torch.float8_e4m3fn), s.squeeze(-1).contiguous()

    def _mlp_fp8(self, rows, le):
        amax = rows.float().abs().amax(dim=-1, keepdim=True).clamp_min(1e-4)
        sa = amax / 448.0
        q = (rows.float() / sa).to(torch.float8_e4m3fn)
        y = torch._scaled_mm(q, self.w1q[le].t(), scale_a=sa, scale_b=self.s1[le].unsqueeze(0), out_dtype=torch.bfloat16)
        i = self.cfg.intermediate
        act = torch.nn.functional.silu(y[:, :i]) * y[:, i:]
        amax2 = act.float().abs().amax(dim=-1, keepdim=True).clamp_min(1e-4)
        sb = amax2 / 448.0
        q2 = (act.float() / sb).to(torch.float8_e4m3fn)
        return torch._scaled_mm(q2, self.w2q[le].t(), scale_a=sb, scale_b=self.s2[le].unsqueeze(0), out_dtype=torch.bfloat16)

    def forward(self, x, idx, w):
        cfg, world, el = self.cfg, self.world, self.el
        t, k = idx.shape
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=cfg.num_experts)
        if world > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts)  # [src, le] for my experts
            # one host sync: NCCL needs the split sizes on the host
            both = torch.stack([recv_counts.view(world, el).sum(dim=1), counts.view(world, el).sum(dim=1)]).cpu()
            recv_split, send_split = both[0].tolist(), both[1].tolist()
        else:
            recv_counts = counts
        send = x[order // k]
        if world > 1:
            recv = send.new_empty((sum(recv_split), cfg.hidden))
            dist.all_to_all_single(recv, send, output_split_sizes=recv_split, input_split_sizes=send_split)
            # source-major -> expert-major
            seg_expert = torch.arange(el, device=self.dev).repeat(world)
            row_expert = torch.repeat_interleave(seg_expert, recv_counts.view(-1), output_size=recv.shape[0])
            perm = torch.argsort(row_expert, stable=True)
            rows = recv[perm]
        else:
            rows, perm = send, None          # one rank: already expert-major, nothing reaches the host
        per_e = recv_counts.view(world, el).sum(dim=0)
        if self.mode == "bf16_grouped_mm":
            offs = per_e.cumsum(0).to(torch.int32)
            y = torch._grouped_mm(rows, self.w1t, offs=offs)
            i = cfg.intermediate
            act = torch.nn.functional.silu(y[:, :i]) * y[:, i:]
            z = torch._grouped_mm(act, self.w2t, offs=offs)
        else:
            z = torch.empty_like(rows)
            a = 0
            per_e_host = per_e.tolist()
            for le in range(el):
                n = int(per_e_host[le])
                if n:
                    z[a:a + n] = self._mlp_fp8(rows[a:a + n], le)
                a += n
        if world > 1:
            back = torch.empty_like(z)
            back[perm] = z
            ret = back.new_empty((t * k, cfg.hidden))
            dist.all_to_all_single(ret, back, output_split_sizes=send_split, input_split_sizes=recv_split)
        else:
            ret = z
        pair_rows = torch.empty_like(ret)
        pair_rows[order] = ret
        out = (pair_rows.view(t, k, cfg.hidden).float() * w.unsqueeze(-1)).sum(dim=1)
        return out.to(torch.bfloat16)


def time_baseline(cfg, tokens, rank, world, local, steps, warmup, gemm="bf16_grouped", sets=None):
    """Device time per step (ms, max over ranks) of the comparison layer on the given inputs, and the GEMM it used."""
    from bench import barrier, make_inputs, max_over_ranks
    dev = torch.device("cuda", local)
    layer = BaselineMoE(cfg, rank, world, dev, gemm=gemm)
    if sets is None:
        sets = make_inputs(cfg, tokens, rank, 4, dev)
    for i in range(max(warmup, 3)):
        layer.forward(*sets[i % len(sets)])
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        layer.forward(*sets[i % len(sets)])
    e1.record()
    barrier(world)
    ms = max_over_ranks(e0.elapsed_time(e1), world) / steps
    mode = layer.mode
    del layer
    torch.cuda.empty_cache()
    return ms, mode


def run_baseline(args, cfg, rank, world, local, metric):
    tokens = args.tokens or cfg.tokens_per_rank
    ms, mode = time_baseline(cfg, tokens, rank, world, local, args.steps, args.warmup,
                             gemm=getattr(args, "baseline_gemm", "bf16_grouped"))
    if rank == 0:
        print(json.dumps({
            "metric": metric, "value": tokens * world / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "impl": "baseline", "dtype": mode, "data": "synthetic",
            "config": {"model": cfg.name, "tokens_per_rank": tokens, "num_experts": cfg.num_experts,
                       "parallelism": f"ep{world}", "comm": "nccl all_to_all_single", "gemm": mode}}))
