"""Model check of the arrival-counter protocol of the deep-fused layer on the CPU: two ranks as
interleaved step lists, every interleaving explored, no GPU involved.

The device protocol being modelled (csrc/kernels/dispatch_normal.cu with defer_push, csrc/kernels/fused_moe_mx.cu):
per layer a rank (1) zeroes its own arrival counter of the layer's parity, (2) release-stores the layer's epoch
into a count flag of every peer, (3) waits for the peer's count flag of the same epoch, (4) writes its rows into the
peer's receive buffer and adds their number to the peer's arrival counter with a release, (5) waits until its own
counter has reached the number of rows it expects and then reads them (the first GEMM), (6) pushes combine rows,
raises the combine flag, waits for the peer's.  Nothing but the counter is cleared between layers.

What the model shows: the order zero -> count flag -> wait for the peer's count flag -> send is what makes the
counter safe (a sender that does not wait for the count flag can have its rows wiped, whatever the number of counter
sets); the receive buffer is safe because a rank sends layer n + 1 only after the peer has raised the count flag of
n + 1, which the peer does after it has read layer n.

The reference spins without bound on a per-expert token counter
(fused_deep_moe/gemm/kernel/grouped_matmul_slice_m_per_token_dequant_swiglu_quant_multistage_workspace.h:558-574)
and has no such test.
"""
from typing import Dict, List, Tuple

RANKS = 2
ROWS = 2   # rows every rank sends to its peer per layer (each its own step, so adds can interleave)


def _program(layers: int, counter_sets: int, wait_for_count_flag: bool) -> List[Tuple]:
    steps: List[Tuple] = []
    for n in range(1, layers + 1):
        p = n % counter_sets
        steps.append(("zero", "arrival", p, n))            # own memory
        steps.append(("flag", "count_flag", 0, n))         # into the peer's memory
        if wait_for_count_flag:
            steps.append(("wait_flag", "count_flag", 0, n))
        for i in range(ROWS):
            steps.append(("store", "recv_row", i, n))      # into the peer's memory
            steps.append(("add", "arrival", p, 1))         # peer's counter, release
        steps.append(("wait_count", "arrival", p, ROWS))   # own counter
        for i in range(ROWS):
            steps.append(("load", "recv_row", i, n))       # first GEMM reads the rows
        steps.append(("flag", "combine_flag", 0, n))       # combine rows pushed (not modelled), flag raised
        steps.append(("wait_flag", "combine_flag", 0, n))  # reduce waits for the peer's rows
    return steps


def _explore(layers: int, counter_sets: int, wait_for_count_flag: bool = True) -> List[str]:
    """Depth-first search over all interleavings of the two ranks' step lists.  Returns the violations found
    (a stale or future row read by a GEMM, a counter that ran past what the layer expects, a deadlock)."""
    prog = _program(layers, counter_sets, wait_for_count_flag)
    n = len(prog)
    violations: List[str] = []
    seen = set()
    stack: List[Tuple[Tuple[int, ...], Tuple]] = [((0,) * RANKS, ())]
    while stack and len(violations) < 8:
        pcs, mem_items = stack.pop()
        if (pcs, mem_items) in seen:
            continue
        seen.add((pcs, mem_items))
        mem: Dict = dict(mem_items)
        progressed = False
        for r in range(RANKS):
            if pcs[r] >= n:
                continue
            kind, region, idx, val = prog[pcs[r]]
            peer = 1 - r
            new_mem = mem
            if kind == "zero":
                new_mem = dict(mem)
                new_mem[(r, region, idx)] = 0
            elif kind in ("store", "flag"):
                new_mem = dict(mem)
                new_mem[(peer, region, idx)] = val
            elif kind == "add":
                new_mem = dict(mem)
                new_mem[(peer, region, idx)] = mem.get((peer, region, idx), 0) + val
                if new_mem[(peer, region, idx)] > ROWS:
                    violations.append(f"counter {idx} of rank {peer} reached {new_mem[(peer, region, idx)]} > {ROWS}")
                    continue
            elif kind == "wait_flag":
                if mem.get((r, region, idx), 0) < val:
                    continue
            elif kind == "wait_count":
                if mem.get((r, region, idx), 0) < val:
                    continue
            elif kind == "load":
                got = mem.get((r, region, idx), 0)
                layer = val
                if got != layer:
                    violations.append(f"rank {r} read row {idx} of layer {got} while in layer {layer}")
                    continue
            progressed = True
            nxt = tuple(p + 1 if i == r else p for i, p in enumerate(pcs))
            stack.append((nxt, tuple(sorted(new_mem.items()))))
        if not progressed and any(p < n for p in pcs) and not violations:
            violations.append(f"deadlock at {pcs}")
    return violations


def test_counter_protocol_holds_with_the_handshake_for_any_number_of_counter_sets():
    # the kernels use two sets (parity of the dispatch epoch); one would do as long as the handshake is kept
    assert _explore(layers=3, counter_sets=2) == []
    assert _explore(layers=3, counter_sets=1) == []


def test_sending_before_the_peers_count_flag_loses_rows():
    # without step (3) a fast rank's rows of layer n can land before the slow rank has zeroed its counter for layer n:
    # the rows are wiped (the slow rank then waits forever: a bounded wait on the device, a deadlock here), or a row
    # of layer n + 1 lands while the slow rank's first GEMM still reads layer n
    for sets in (1, 2):
        found = _explore(layers=2, counter_sets=sets, wait_for_count_flag=False)
        assert found, f"the model missed the race with {sets} counter set(s)"
