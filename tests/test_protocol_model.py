"""Model check of the epoch-flag protocol on the CPU: two ranks as interleaved step lists, every
interleaving explored, no GPU involved.

The device protocol being modelled (csrc/kernels/dispatch_ll.cu, combine.cu): a sender stores its
payload into the receiver's memory, then release-stores the call's epoch into a flag of the receiver;
the receiver waits until the flag equals its own epoch and then reads.  Nothing is cleared between
calls.  Low-latency dispatch slabs and cells are double-buffered on the parity of the epoch; combine
slots are single-buffered and rely on the data dependency "a rank sends its combine rows only after
it has received the dispatch of the same step".

The reference has no such test: its waits are unbounded spins on the device
(src/cam/comm_operator/ascend_kernels/moe_dispatch_shmem/op_kernel/moe_dispatch_shmem.h:766-776).
"""
from typing import Dict, List, Tuple

RANKS = 2


def _program(ops: str, buffers: int, comb_buffers: int = 1) -> List[Tuple]:
    """Step list of one rank for a call sequence such as "DCDC" (D = dispatch, C = combine).
    `buffers` is the number of dispatch slabs (1 = single-buffered, 2 = parity double buffering),
    `comb_buffers` the same for the combine slots (1 in the kernels)."""
    steps: List[Tuple] = []
    d_epoch = c_epoch = 0
    for op in ops:
        if op == "D":
            d_epoch += 1
            slab = d_epoch % buffers
            steps += [("store", "slab", slab, d_epoch), ("flag", "cell", slab, d_epoch),
                      ("wait", "cell", slab, d_epoch), ("load", "slab", slab, d_epoch)]
        else:
            c_epoch += 1
            slot = c_epoch % comb_buffers
            steps += [("store", "slot", slot, c_epoch), ("flag", "cflag", slot, c_epoch),
                      ("wait", "cflag", slot, c_epoch), ("load", "slot", slot, c_epoch)]
    return steps


def _explore(ops: str, buffers: int, comb_buffers: int = 1) -> List[str]:
    """Depth-first search over all interleavings.  Memory: mem[(owner, region, index)] = value, where a
    payload value is the epoch its writer was in.  Returns the violations found (empty = protocol holds).
    A wait that can never be satisfied shows up as a deadlock."""
    prog = _program(ops, buffers, comb_buffers)
    n = len(prog)
    violations: List[str] = []
    seen = set()
    stack: List[Tuple[Tuple[int, ...], Tuple]] = [((0,) * RANKS, ())]
    while stack:
        pcs, mem_items = stack.pop()
        if (pcs, mem_items) in seen:
            continue
        seen.add((pcs, mem_items))
        mem: Dict = dict(mem_items)
        progressed = False
        for r in range(RANKS):
            if pcs[r] >= n:
                continue
            kind, region, idx, epoch = prog[pcs[r]]
            peer = 1 - r
            new_mem = mem
            if kind in ("store", "flag"):
                new_mem = dict(mem)
                new_mem[(peer, region, idx)] = epoch
            elif kind == "wait":
                # flags are monotonic per index: a flag that has moved past the awaited epoch means the
                # sender has already started overwriting, which the load below reports
                if mem.get((r, region, idx), 0) < epoch:
                    continue
            elif kind == "load":
                got = mem.get((r, region, idx), 0)
                if got != epoch:
                    violations.append(f"rank {r} read {region}[{idx}] of epoch {got} while in epoch {epoch} ({ops})")
                    continue
            progressed = True
            nxt = tuple(p + 1 if i == r else p for i, p in enumerate(pcs))
            stack.append((nxt, tuple(sorted(new_mem.items()))))
        if not progressed and any(p < n for p in pcs) and not violations:
            violations.append(f"deadlock at {pcs} ({ops})")
    return violations


def test_alternating_dispatch_combine_is_safe_even_single_buffered():
    # combine k cannot be sent before dispatch k was received, so the receiver of dispatch k + 1 has
    # finished reading dispatch k long before the slab is written again
    assert _explore("DCDCDC", buffers=1) == []
    assert _explore("DCDCDC", buffers=2) == []


def test_two_dispatches_in_flight_need_the_parity_double_buffer():
    # two micro-batches on one Buffer: D D C C.  One slab: the second dispatch can overwrite rows the peer
    # has not read.  Two slabs (the kernels' layout): every dispatch read is safe.
    assert any("slab" in v for v in _explore("DDCC", buffers=1))
    assert all("slab" not in v for v in _explore("DDCCDDCC", buffers=2))


def test_back_to_back_combines_overrun_the_single_combine_slot():
    # ... but the second combine may overwrite combine slots whose origin has not reduced the first one yet:
    # nothing orders "peer finished reducing combine 1" before "this rank sends combine 2".  Hence the rule of
    # the bindings: one dispatch -> combine pair in flight per Buffer; overlapped micro-batches take a Buffer
    # each.  A second set of combine slots would lift it.
    assert any("slot" in v for v in _explore("DDCC", buffers=2, comb_buffers=1))
    assert _explore("DDCCDDCC", buffers=2, comb_buffers=2) == []


def test_two_buffers_suffice_for_any_run_of_dispatches():
    # a rank leaves dispatch k only after it has seen its peer's flag of dispatch k, and the peer raises that flag
    # after it has read dispatch k - 1: so dispatch k + 1 never meets an unread slab of dispatch k - 1
    assert _explore("DDDDCCCC", buffers=2, comb_buffers=2) == []
    assert any("slab" in v for v in _explore("DDD", buffers=1))
