"""Headline benchmark: tokens/s of one fused MoE layer (dispatch -> fp8 quantise -> grouped GEMM ->
SwiGLU -> grouped GEMM -> combine) on DeepSeek-V3 shapes: hidden 7168, intermediate 2048,
256 routed experts, top-8, 4096 tokens per rank, e4m3 weights with 128x128 scales, e4m3
activations with 1x128 scales, fp32 accumulation, bf16 in/out.  Weak scaling: tokens per rank are
fixed, the 256 experts are spread over the N ranks.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29555 bench.py --gpus 8 --steps 20 --warmup 5

Rank 0 prints one JSON line.  `value` is device-timed (CUDA events around exactly `steps` steps,
barrier + synchronize on both sides, max over ranks); `e2e` is the same layer driven through
MoEStepRunner with a pinned-host -> device copy of every step's inputs and a device -> host read
of the step's result record (the host launches step i+1 before it waits for the record of step i, so
every record is read inside the timed region, one step behind the launches).  `--impl reference` reports why the Ascend-only reference cannot
run here; `--impl baseline` times the NCCL all_to_all_single + cuBLAS comparison layer.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

METRIC = "moe_layer_tokens_per_s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"])
    ap.add_argument("--model", default="deepseek-v3-moe")
    ap.add_argument("--tokens", type=int, default=0, help="tokens per rank (0 = the model's default)")
    ap.add_argument("--experts", type=int, default=0, help="override the number of routed experts (smaller smoke runs)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-baseline", action="store_true",
                    help="skip the NCCL + cuBLAS comparison layer that fills vs_baseline (it runs after the timed regions)")
    ap.add_argument("--no-verify", action="store_true",
                    help="skip the check of one step's output against the unfused ops of this library")
    ap.add_argument("--baseline-gemm", default="bf16_grouped", choices=["fp8_per_expert", "bf16_grouped"],
                    help="--impl baseline: cuBLAS fp8 per expert, or the library's bf16 grouped GEMM")
    ap.add_argument("--fp32-scales", action="store_true",
                    help="fp8 weights with arbitrary fp32 block scales: the software-scaled GEMM (quantMode 3) instead of "
                         "tensor-core block scaling (not the headline configuration)")
    ap.add_argument("--w8a8-exact", action="store_true",
                    help="W8A8 models: int8 x int8 -> int32 tensor-core path instead of computing in block-scaled fp8")
    return ap.parse_args()


def reference_unavailable() -> None:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference (UMDK CAM) is AscendC for Ascend 910 NPUs behind CANN/torch_npu and has no CUDA "
                       "path; its repository root is not pip-installable (no setup.py/pyproject.toml), and building "
                       "its pybind sub-package was refused by a safety check",
    }))


def init_dist(n: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n:
        raise SystemExit(f"--gpus {n} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n}")
    torch.cuda.set_device(local)
    if world > 1:
        # pinned staging buffers of the end-to-end path should sit on the GPU's own NUMA node
        from umdk_original_b200.utils.host import bind_to_gpu_numa_node
        bind_to_gpu_numa_node(local)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier(world: int) -> None:
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(v: float, world: int) -> float:
    if world == 1:
        return v
    t = torch.tensor([v], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def make_inputs(cfg, tokens: int, rank: int, nsets: int, dev):
    """Synthetic N(0,1) tokens and top-k routing from N(0,1) gate logits (group-limited for
    DeepSeek-V3: 8 groups, 4 kept), several independent sets so steps do not reuse data."""
    from umdk_original_b200.models import route
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    sets = []
    for _ in range(nsets):
        x = torch.randn(tokens, cfg.hidden, device=dev, generator=g).to(torch.bfloat16)
        logits = torch.randn(tokens, cfg.num_experts, device=dev, generator=g)
        idx, w = route(logits, cfg.topk, cfg.num_groups, cfg.topk_groups)
        sets.append((x, idx.contiguous(), w.float().contiguous()))
    return sets


def verify_against_unfused_ops(layer, buf, x, idx, w, rank, world):
    """One step of the fused layer against the same layer built from the stand-alone ops of this library
    (dispatch with fp8 quantisation -> grouped GEMM + SwiGLU + requantisation -> grouped GEMM -> combine).
    Every rank calls it (the ops are collective).  Returns (max abs difference, max abs of the output)."""
    ops = torch.ops.umdk_cam_op_lib
    out, _ = layer(x, idx, w)
    out = out.clone()
    wts = layer.weights
    el = layer.num_local
    rx, src, cnt, per_e, rs = ops.moe_dispatch_prefill_quant(x, idx, w, 0, buf.name, rank, world, 4)
    off = buf.native.expert_offsets(el + 1).clone()
    q, s = ops.grouped_gemm_fp8_swiglu(rx, rs, wts.w1, wts.s1, off, True)
    y = ops.grouped_gemm_fp8(q, s, wts.w2, wts.s2, off, True)
    want = ops.moe_combine_prefill(y, idx, w, src, cnt, buf.name, rank, world)
    torch.cuda.synchronize()
    return float((out.float() - want.float()).abs().max()), float(want.float().abs().max())


def run_ours(args, cfg, rank, world, local):
    import umdk_original_b200 as u
    from umdk_original_b200.models import FusedMoE, MoEStepRunner, make_buffer_for
    from umdk_original_b200.utils import ClockSampler

    dev = torch.device("cuda", local)
    tokens = args.tokens or cfg.tokens_per_rank
    group = dist.group.WORLD if world > 1 else None
    buf = make_buffer_for(cfg, group, tokens=tokens, name="bench", device=dev, timeout_ms=20000.0)
    weights = None
    if args.fp32_scales:
        from umdk_original_b200.models.weights import random_fp8_experts
        weights = random_fp8_experts(cfg.num_experts // world, cfg.hidden, cfg.intermediate, device=dev, seed=rank,
                                     ue8m0=False)
    layer = FusedMoE(cfg, buf, weights=weights, seed=0, exact_w8a8=args.w8a8_exact)
    sets = make_inputs(cfg, tokens, rank, 4, dev)

    def step(i):
        x, idx, w = sets[i % len(sets)]
        return layer(x, idx, w)

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier(world)
    buf.check()

    launches0 = buf.native.launch_count()
    with ClockSampler(local) as clocks:
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            step(i)
        e1.record()
        barrier(world)
        ms = max_over_ranks(e0.elapsed_time(e1), world) / args.steps
        time.sleep(0.3)
    launches = buf.native.launch_count() - launches0   # kernels of this library launched inside the timed region
    buf.check()
    clock_summary = clocks.summary()

    max_err = None
    if not args.no_verify and layer.quant_mode == 4:
        err, scale = verify_against_unfused_ops(layer, buf, *sets[0], rank, world)
        max_err = {"max_abs_err_vs_unfused_ops": max_over_ranks(err, world), "output_max_abs": max_over_ranks(scale, world)}
        buf.check()

    # per-stage breakdown from a separate, untimed pass (events between the four launches)
    buf.set_profile(True)
    parts = []
    for i in range(5):
        step(i)
        parts.append(buf.read_profile())
        barrier(world)
    buf.set_profile(False)
    breakdown = {k: max_over_ranks(sorted(p[k] for p in parts)[len(parts) // 2], world) for k in parts[0]}

    e2e = None
    e2e_record = None
    if not args.no_e2e:
        host = [(x.cpu().pin_memory(), idx.cpu().pin_memory(), w.cpu().pin_memory()) for x, idx, w in sets]

        def run_e2e(copy_output: bool):
            runner = MoEStepRunner(layer, tokens, copy_output=copy_output, time_copies=True)
            runner.stage(*host[0])
            for i in range(3):  # warm-up of the pipelined path
                runner.run()
                runner.stage(*host[(i + 1) % len(host)])
                runner.finish()
            runner.copy_times()  # forget the warm-up copies
            barrier(world)
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            pending = None
            for i in range(args.steps):
                ticket = runner.run()                         # step i is launched ...
                runner.stage(*host[(i + 1) % len(host)])      # ... step i+1's inputs are copied in meanwhile ...
                if pending is not None:
                    runner.result(pending)                    # ... and the record of step i-1 is read on the host
                pending = ticket
            runner.result(pending)                            # every step's record has reached the host
            t1.record()
            barrier(world)
            ms = max_over_ranks(t0.elapsed_time(t1), world) / args.steps
            copies = {k: max_over_ranks(v, world) for k, v in runner.copy_times().items()}
            buf.check()
            return {"value": tokens * world / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
                    "h2d_bytes_per_step": runner.h2d_bytes, "d2h_bytes_per_step": runner.d2h_bytes,
                    # how long the slowest rank's copies of one step take by themselves (they overlap the compute of
                    # the neighbouring steps; a value near ms_per_step means the host link, not the GPU, sets the pace)
                    "h2d_ms_max_over_ranks": copies["h2d_ms"], "d2h_ms_max_over_ranks": copies["d2h_ms"]}

        e2e = run_e2e(True)
        e2e["d2h"] = "the layer output [tokens, hidden] bf16 and a record of token counts + checksum, every step"
        # the same with only the record read back (what a training step that keeps its activations on the device reads)
        e2e_record = run_e2e(False)
        e2e_record["d2h"] = "a record of token counts + checksum, every step; the output stays on the device"
        del host

    # the comparison layer (NCCL all_to_all_single + library GEMMs) at the same N on the same inputs, after the timed regions
    base = None
    if not args.no_baseline:
        from baseline.nccl_cublas import time_baseline
        try:
            base_ms, base_mode = time_baseline(cfg, tokens, rank, world, local, max(5, args.steps // 2), 3,
                                               gemm=args.baseline_gemm, sets=sets)
            base = {"ms_per_step": base_ms, "value": tokens * world / (base_ms * 1e-3), "gemm": base_mode,
                    "comm": "nccl all_to_all_single" if world > 1 else "none (one rank)"}
        except Exception as exc:  # noqa: BLE001 - the comparison must not take the product's number down with it
            base = {"error": f"{type(exc).__name__}: {exc}"[:200]}

    if rank == 0:
        value = tokens * world / (ms * 1e-3)
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / base["value"]) if base and "value" in base else None,
            "dtype": ("fp8_e4m3 block-scaled (fp32 accumulate, bf16 in/out)" if cfg.weight_format != "w8a8" else
                      "int8 W8A8 (per-token x per-channel scales, int32 accumulate, bf16 in/out)" if args.w8a8_exact else
                      "int8-range weights + per-channel scales computed as fp8_e4m3 block-scaled (fp32 accumulate, bf16 in/out)"),
            "data": "synthetic",
            "impl": "ours",
            "config": {"model": cfg.name, "global_batch": tokens * world, "seq_len": tokens, "tokens_per_rank": tokens,
                       "hidden": cfg.hidden, "moe_intermediate": cfg.intermediate, "num_experts": cfg.num_experts,
                       "topk": cfg.topk, "parallelism": f"ep{world}",
                       "scales": ("per token x per channel (int8)" if (cfg.weight_format == "w8a8" and args.w8a8_exact) else
                                  "fp32 (software-scaled GEMM)" if args.fp32_scales else
                                  "power of two (tensor-core block scaling)"),
                       "cache": "expert weights per rank exceed the 126 MB L2 and 4 input sets rotate; no explicit flush"},
            "clocks": {k: clock_summary[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "gpu_launches": int(launches),
            "launches_per_step": launches / args.steps,
            "tflops_per_gpu": cfg.flops_per_token() * tokens / (ms * 1e-3) / 1e12,
            "stage_ms_max_over_ranks": breakdown,
        }
        # three launches per step = a fused route: "gemm1_ms" is then the one kernel that runs both GEMMs and the combine
        # send (and, when "dispatch_ms" is only the count exchange and quantisation, the dispatch rows too)
        line["route"] = "fused kernel (3 launches)" if round(launches / args.steps) == 3 else "four launches"
        if e2e is not None:
            line["e2e"] = e2e
            line["e2e_record_only"] = e2e_record
        if base is not None:
            line["baseline"] = base
        if max_err is not None:
            line["verify"] = max_err
        print(json.dumps(line))
    barrier(world)
    buf.destroy()


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_unavailable()
        return
    from umdk_original_b200.models import BY_NAME
    import dataclasses
    cfg = BY_NAME[args.model]
    if args.experts:
        cfg = dataclasses.replace(cfg, num_experts=args.experts, num_groups=1, topk_groups=1)
    rank, world, local = init_dist(args.gpus)
    try:
        if args.impl == "baseline":
            from baseline.nccl_cublas import run_baseline
            run_baseline(args, cfg, rank, world, local, METRIC)
        else:
            run_ours(args, cfg, rank, world, local)
    finally:
        if world > 1 and dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
