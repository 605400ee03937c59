"""``Buffer``: the registered symmetric memory every op works on.

The reference has no such object: peers' "windows" come from the HCCL group named by
``group_ep`` (pybind/fused_deep_moe.cpp:65-77) or from the Ascend-SHMEM heap pointer passed as
``extInfo`` (pybind/moe_dispatch_shmem.cpp:143-150), and the ping-pong state hides inside the
window.  Here one Buffer per rank owns

* one symmetric allocation, exported with CUDA IPC and mapped into every peer of the group
  (bootstrap over the caller's ``torch.distributed`` group: NCCL or gloo, never in the hot path);
* a device table of every peer's base address, per-op epoch counters and a status word;
* a name (what ops take as ``group_ep`` / ``groupEp``) and an integer id (``extInfo``).

On CPU tensors the same class wraps a gloo group, so the op surface is identical.
``Buffer.virtual`` builds R buffers on ONE GPU whose peer tables point at each other; with
``phases()`` the ops then run phase by phase over all virtual ranks, which exercises the whole
multi-rank protocol without any launch waiting for another launch.
"""
from __future__ import annotations

import contextlib
from typing import Iterator, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import cam_ops
from ..utils.config import CamConfig
from ..utils.errors import raise_for_status
from ..utils.log import get_logger
from . import registry
from .gloo_backend import CpuGroup

log = get_logger("umdk_cam.buffer")

PHASE_COUNT, PHASE_SEND, PHASE_RECV, PHASE_FINAL = 1, 2, 4, 8
PHASE_TP_SEND, PHASE_TP_RECV = 16, 32   # exchange inside a tensor-parallel pair (tpWorldSize = 2)
PHASE_ALL = 63
_AUTO = [0]


class Buffer:
    def __init__(self, group=None, config: Optional[CamConfig] = None, *, name: Optional[str] = None,
                 device: Optional[torch.device] = None, rank: Optional[int] = None, num_ranks: Optional[int] = None,
                 tp_group=None, tp_world_size: int = 1, _connect: bool = True):
        """``group`` is the expert-parallel group.  ``tp_group`` (two ranks: this one and the rank at the
        same expert-parallel position of the other tensor-parallel group) enables ``tpWorldSize=2`` in the
        low-latency ops; ``tp_world_size=2`` without a group only reserves the exchange region (the
        single-process test harness then connects partners with ``connect_local_tp_peer``)."""
        self.config = config or CamConfig.from_env()
        self.group = group
        if rank is None:
            rank = dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0
        if num_ranks is None:
            num_ranks = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank, self.num_ranks = int(rank), int(num_ranks)
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        _AUTO[0] += 1
        self.name = name or f"umdk_cam_group_{_AUTO[0]}"
        self._native = None
        self._cpu: Optional[CpuGroup] = None
        cfg = self.config
        if cfg.num_experts % self.num_ranks != 0:
            raise ValueError(f"num_experts {cfg.num_experts} must be a multiple of num_ranks {self.num_ranks}")
        self.capacity = cfg.resolve_capacity(self.num_ranks)
        if self.device.type == "cuda":
            C = cam_ops.native_module()
            tp_rows = 0
            if tp_group is not None or tp_world_size == 2:
                el = cfg.num_experts // self.num_ranks
                tp_rows = max(1, cfg.ll_max_tokens * self.num_ranks * min(el, cfg.topk))
            self._native = C.Buffer(self.device.index or 0, self.rank, self.num_ranks, cfg.num_experts, cfg.max_tokens,
                                    cfg.hidden, cfg.topk, self.capacity, cfg.ll_max_tokens, tp_rows)
            self._native.set_timeout_ms(cfg.timeout_ms)
            self._native.set_copy_outputs(bool(cfg.copy_outputs))
            self._native.register_name(self.name)
            self.handle = int(self._native.id)
            if _connect:
                self._connect_ipc()
                if tp_group is not None:
                    self._connect_tp(tp_group)
        else:
            self._cpu = CpuGroup(group, self.rank, self.num_ranks, cfg.num_experts)
            if tp_group is not None:
                assert dist.get_world_size(tp_group) == 2, "tensor parallelism inside the ops is limited to 2 ranks"
                self._cpu.tp_group = tp_group
                self._cpu.tp_rank = self.tp_rank = dist.get_rank(tp_group)
            self.handle = registry.register(self._cpu, self.name)
        log.info("Buffer %s rank %d/%d on %s: %.1f MiB symmetric", self.name, self.rank, self.num_ranks, self.device,
                 self.total_bytes / 2 ** 20)

    # ------------------------------------------------------------------ construction helpers
    def _connect_ipc(self) -> None:
        if self.num_ranks == 1:
            self._native.set_local_peers([self._native])
            return
        handles: List[Optional[bytes]] = [None] * self.num_ranks
        dist.all_gather_object(handles, self._native.ipc_handle(), group=self.group)
        self._native.open_ipc_peers([bytes(h) for h in handles])
        dist.barrier(group=self.group)

    def _connect_tp(self, tp_group) -> None:
        assert dist.get_world_size(tp_group) == 2, "tensor parallelism inside the ops is limited to 2 ranks"
        tp_rank = dist.get_rank(tp_group)
        handles: List[Optional[bytes]] = [None, None]
        dist.all_gather_object(handles, self._native.ipc_handle(), group=tp_group)
        self._native.open_ipc_tp_peer(bytes(handles[1 - tp_rank]), tp_rank)
        self.tp_rank = tp_rank
        dist.barrier(group=tp_group)

    def connect_local_tp_peer(self, partner: "Buffer", tp_rank: int) -> None:
        """Single-process harness: the partner is another Buffer of this process on the same GPU."""
        self._native.set_local_tp_peer(partner._native, tp_rank)
        self.tp_rank = tp_rank

    @classmethod
    def virtual(cls, num_ranks: int, config: CamConfig, device: Optional[torch.device] = None,
                name: str = "virt") -> List["Buffer"]:
        """R ranks as R buffers of this process on one GPU (peer tables point at each other)."""
        device = device or torch.device("cuda", torch.cuda.current_device())
        bufs = [cls(None, config, name=f"{name}{r}", device=device, rank=r, num_ranks=num_ranks, _connect=False)
                for r in range(num_ranks)]
        natives = [b._native for b in bufs]
        for b in bufs:
            b._native.set_local_peers(natives)
        return bufs

    @staticmethod
    def get_size_hint(config: CamConfig, num_ranks: int) -> int:
        """Bytes of symmetric memory a Buffer of this configuration allocates per rank."""
        cap = config.resolve_capacity(num_ranks)
        h, e, k = config.hidden, config.num_experts, config.topk
        total = 5 * 4 * 72 + 8 * num_ranks * e + 16 * e
        total += cap * h * 2 + cap * (h // 128) * 4 + cap * 12 + config.max_tokens * k * h * 2
        total += 2 * num_ranks * config.max_tokens * k * 8  # replicate lists of normal dispatch
        if config.ll_max_tokens:
            cells = 2 * e
            total += cells * config.ll_max_tokens * (h * 2 + (h // 128) * 4 + 8) + config.ll_max_tokens * k * h * 2
        return int(total + 16 * 1024)

    # ------------------------------------------------------------------ properties / state
    @property
    def total_bytes(self) -> int:
        return int(self._native.total_bytes) if self._native is not None else 0

    @property
    def native(self):
        return self._native

    @property
    def cpu_group(self) -> Optional[CpuGroup]:
        return self._cpu

    GUARDED_REGIONS = ("recv_x", "recv_scales", "recv_src", "combine_buf")

    def check(self, guards: bool = False) -> None:
        """Synchronises the current stream, reads the device status word and raises on an error.  With ``guards``
        it also reads the guard words that sit directly behind the four regions peers write rows into and raises
        ``CamError`` (code 8) naming every region something has written past."""
        if self._native is None:
            return
        code, who, detail, block, text = self._native.poll_status()
        raise_for_status(code, who, detail, block, text)
        if guards:
            damaged = int(self._native.check_guards())
            if damaged:
                names = [n for i, n in enumerate(self.GUARDED_REGIONS) if damaged & (1 << i)]
                raise_for_status(8, -1, damaged, -1, "guard words overwritten behind " + ", ".join(names))

    def reset(self) -> None:
        """Zeroes flags and epochs after an error (every surviving rank must call it).  Handles and
        tensors returned by earlier dispatch calls are void afterwards.  With a process group the call ends with a
        host-side barrier over the group, so that no rank's first flags of the next op can be wiped by a rank that
        is still zeroing."""
        if self._native is not None:
            self._native.reset()
            if self.num_ranks > 1 and self.group is not None and dist.is_available() and dist.is_initialized():
                dist.barrier(group=self.group)
        elif self._cpu is not None:
            self._cpu.ll_src = None
            self._cpu.last_src = None

    def set_copy_outputs(self, on: bool = True) -> None:
        """What ``moe_dispatch_prefill`` / ``moe_dispatch_prefill_quant`` return.  Off (default): views of this
        Buffer's receive region, valid until the next dispatch on the Buffer (this rank's, or a peer's that has
        moved on to its next call), ``reset()`` or ``destroy()``; the memory itself stays allocated for as long as
        such a view is alive.  On: private copies, as the reference returns
        (pybind/moe_dispatch_prefill.cpp:166-191), for callers that keep a layer's rows across the next dispatch."""
        if self._native is not None:
            self._native.set_copy_outputs(on)

    def set_timeout_ms(self, ms: float) -> None:
        if self._native is not None:
            self._native.set_timeout_ms(ms)

    def inject_drop_flags(self, on: bool = True) -> None:
        """Host-side fault injection: this rank withholds its completion flags / its next send."""
        if self._native is not None:
            self._native.set_debug_drop_flags(on)
        else:
            self._cpu.drop_next_send = on

    def barrier(self) -> None:
        """Device barrier over all ranks of the Buffer, enqueued on the current stream (every rank must
        call it).  On CPU it is the group's gloo barrier."""
        if self._native is not None:
            self._native.barrier()
        elif self._cpu is not None and self.num_ranks > 1:
            dist.barrier(group=self.group)

    LL_DISPATCH_TRACE = ("start", "slot_table", "rows_issued", "system_fence", "grid_barrier", "cells_arrived",
                         "rows_packed", "last_cta_out")
    COMBINE_TRACE = ("start", "rows_issued", "system_fence", "flags_arrived", "reduced", "last_cta_out")

    def set_trace(self, on: bool = True) -> None:
        """In-kernel timeline of the low-latency dispatch and of combine: CTA 0 stamps ``%globaltimer`` at
        the phase boundaries of the kernels (off by default; one predicated branch per point)."""
        if self._native is not None:
            self._native.set_trace(on)

    def read_trace(self) -> dict:
        """Microseconds since kernel start of every trace point of the last traced launches
        (synchronises the device)."""
        t = self._native.read_trace()
        def rel(vals, names):
            t0 = vals[0]
            return {n: (v - t0) / 1e3 for n, v in zip(names, vals) if v}
        return {"dispatch_ll": rel(t[:8], self.LL_DISPATCH_TRACE), "combine": rel(t[8:14], self.COMBINE_TRACE)}

    def set_fused_trace(self, on: bool = True) -> None:
        """Timeline of the deep-fused layer (off by default): the kernel notes when the first GEMM of every local
        expert was released, i.e. when all rows of that expert had arrived."""
        if self._native is not None:
            self._native.set_fused_trace(on)

    def read_fused_trace(self, num_local_experts: Optional[int] = None) -> List[Optional[float]]:
        """Microseconds after the start of the last fused kernel at which each local expert's first GEMM was
        released; ``None`` for an expert that never was (its rows did not all arrive).  Synchronises the device."""
        n = num_local_experts or self.config.num_experts // self.num_ranks
        return [None if v < 0 else v / 1e3 for v in self._native.read_fused_trace(n)]

    def read_fused_waits(self, num_local_experts: Optional[int] = None) -> dict:
        """What the MMA-issuing thread of the first CTA pair waited for in the last traced fused kernel (clock
        cycles): the whole loop, and inside it the waits for a drained accumulator, for scale factors and for
        operand tiles; also the K-blocks and tiles it issued.  Tells which producer limits the tensor cores."""
        n = num_local_experts or self.config.num_experts // self.num_ranks
        v = self._native.read_fused_waits(n)
        return dict(zip(("loop_cycles", "wait_accumulator", "wait_scale_factors", "wait_operands", "k_blocks", "tiles", "issue_cycles"), v))

    def fused_route(self, tokens: int, intermediate: int, hidden: Optional[int] = None, topk: Optional[int] = None,
                    num_experts: Optional[int] = None) -> str:
        """Which route ``fused_deep_moe`` takes on this Buffer for block-scaled fp8 weights with power-of-two scales
        and these shapes: ``"four launches"``, ``"deep-fused"`` (one kernel sends the dispatch rows, runs both GEMMs
        and pushes the combine rows) or ``"dispatch + fused GEMMs"``.  The choice follows ``UMDK_CAM_DEEP_FUSE`` as it
        was when the Buffer was created, else the rank count and the mean rows per expert."""
        cfg = self.config
        r = self._native.fused_route(tokens, topk or cfg.topk, hidden or cfg.hidden, intermediate,
                                     num_experts or cfg.num_experts) if self._native is not None else 0
        return ("four launches", "deep-fused", "dispatch + fused GEMMs")[int(r)]

    def set_profile(self, on: bool = True) -> None:
        """Per-stage device timing of ``fused_deep_moe`` (CUDA events around its four launches)."""
        if self._native is not None:
            self._native.set_profile(on)

    def read_profile(self) -> dict:
        """Milliseconds of the last profiled fused layer: dispatch, GEMM1 (+SwiGLU+requant), GEMM2
        (+combine send), combine reduce.  On the deep-fused route the first entry is the count exchange and local
        quantisation, the second the one kernel that sends, runs both GEMMs and pushes the combine rows, the third
        is zero.  Synchronises on the last event."""
        d, g1, g2, c = self._native.read_profile()
        return {"dispatch_ms": d, "gemm1_ms": g1, "gemm2_send_ms": g2, "combine_ms": c}

    def stats(self, reset: bool = False) -> dict:
        """Counters of this rank since the Buffer was created (or since the last ``stats(reset=True)``); synchronises
        the device.  Besides the row counts of the last dispatch: per peer, the (token, k) pairs routed to it by the
        normal-mode dispatches and the longest time this rank waited for that peer's dispatch counts, dispatch rows
        and combine rows (microseconds) -- the peer with the largest wait is the one that was late."""
        if self._cpu is not None:
            return dict(self._cpu.stats)
        el = self.config.num_experts // self.num_ranks
        waits, rows, calls = self._native.read_stats(reset)
        r = self.num_ranks
        return {"total_recv": int(self._native.total_recv().item()),
                "recv_per_expert": self._native.num_recv_per_expert(el).tolist(),
                "symmetric_bytes": self.total_bytes,
                "dispatch_calls": calls[0], "combine_calls": calls[1],
                "rows_routed_to_peer": list(rows),
                "max_wait_us": {"dispatch_counts": [w / 1e3 for w in waits[0:r]],
                                "dispatch_rows": [w / 1e3 for w in waits[r:2 * r]],
                                "combine_rows": [w / 1e3 for w in waits[2 * r:3 * r]]},
                "kernel_launches": int(self._native.launch_count())}

    def destroy(self) -> None:
        if self._native is not None:
            self._native.destroy()
            self._native = None
        if self._cpu is not None:
            registry.unregister(self._cpu)
            self._cpu = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.destroy()
        except Exception:  # noqa: BLE001
            pass


@contextlib.contextmanager
def phases(mask: int) -> Iterator[None]:
    """Restricts the CUDA ops to the given phases (virtual-rank harness); restores all phases."""
    C = cam_ops.native_module()
    old = C.get_phase_mask()
    C.set_phase_mask(mask)
    try:
        yield
    finally:
        C.set_phase_mask(old)


def run_virtual(fn, num_ranks: int, masks: Sequence[int] = (PHASE_COUNT, PHASE_SEND, PHASE_RECV, PHASE_FINAL),
                return_all: bool = False):
    """Calls ``fn(rank)`` for every virtual rank once per phase and returns the results of the last
    phase (with ``return_all`` a dict phase -> results, since an op allocates fresh outputs on every
    call and fills each of them in one particular phase).  ``fn`` issues the same op call(s) each
    time; the phase mask decides what the kernels do."""
    out = [None] * num_ranks
    every = {}
    for m in masks:
        with phases(m):
            for r in range(num_ranks):
                out[r] = fn(r)
        every[m] = list(out)
    torch.cuda.synchronize()
    return every if return_all else out
