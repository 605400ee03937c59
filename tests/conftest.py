"""Shared fixtures.  GPU tests carry ``@pytest.mark.gpu``; everything else runs on CPU, the
multi-rank cases as gloo child processes (the reference's harness needs real NPUs and torchrun:
test/cam/ut/conftest.py:17-32)."""
import os
import socket
import sys
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multi_process_test: spawns gloo ranks on CPU")


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, args, timeout_s, q):
    import datetime
    try:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s))
        res = fn(rank, world, *args)
        q.put((rank, "ok", res))
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
    finally:
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def run_gloo(fn, world: int, args=(), timeout_s: int = 60):
    """Runs fn(rank, world, *args) in `world` gloo processes; returns {rank: (status, value)}."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, timeout_s, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    for _ in range(world):
        try:
            r, st, val = q.get(timeout=timeout_s * 3)
            out[r] = (st, val)
        except Exception:  # noqa: BLE001
            break
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()
    return out


@pytest.fixture
def gloo_runner():
    return run_gloo
