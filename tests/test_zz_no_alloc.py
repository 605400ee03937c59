"""The allocation-free single-rank dispatch, called the way its users call it: through the
exported C symbol of libumdk_cam.so (ctypes here, no PyTorch binding in between), with inputs and
outputs the caller owns.  Its rows, scales, source triples and expert offsets must equal what
dispatch on a one-rank Buffer produces, on two calls in a row that share the built-in scratch.

Collected last on purpose: a failure here cannot hide the result of any other test."""
import ctypes
import os

import pytest
import torch

import umdk_original_b200 as u

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _lib():
    path = os.path.join(os.path.dirname(u.__file__), "lib", "libumdk_cam.so")
    lib = ctypes.CDLL(path)
    fn = lib.cam_dispatch_local_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p]
    lib.cam_dispatch_local_noalloc_status.restype = ctypes.c_int
    lib.cam_dispatch_local_noalloc_status.argtypes = [ctypes.c_void_p]
    lib.cam_dispatch_local_noalloc_error.restype = ctypes.c_char_p
    return lib


def _call(lib, x, idx, e, quant_mode, capacity):
    t, h = x.shape
    k = idx.shape[1]
    esize = 2 if quant_mode == 0 else 1
    nscale = h // 128 if quant_mode in (3, 4) else 1
    rx = torch.zeros(capacity, h * esize, dtype=torch.uint8, device=DEV)
    rs = torch.zeros(capacity, nscale, dtype=torch.float32, device=DEV)
    src = torch.full((capacity, 3), -7, dtype=torch.int32, device=DEV)
    off = torch.zeros(e + 1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.cam_dispatch_local_noalloc(x.data_ptr(), idx.data_ptr(), 1 if idx.dtype == torch.int64 else 0, t, k, h, e,
                                        quant_mode, capacity, rx.data_ptr(), rs.data_ptr(), src.data_ptr(),
                                        off.data_ptr(), stream)
    assert rc == 0, lib.cam_dispatch_local_noalloc_error().decode()
    return rx, rs, src, off, lib.cam_dispatch_local_noalloc_status(stream)


@pytest.mark.parametrize("quant_mode", [3, 0, 4])
def test_noalloc_dispatch_matches_buffer_dispatch_twice(quant_mode):
    lib = _lib()
    t, h, e, k = 150, 512, 24, 4
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=2000.0)
    buf = u.Buffer(None, cfg, name=f"na{quant_mode}", device=DEV, rank=0, num_ranks=1)
    g = torch.Generator().manual_seed(11 + quant_mode)
    for call in range(2):  # second call: other routing, other token count -> stale scratch would show
        tt = t if call == 0 else t - 37
        x = torch.randn(tt, h, generator=g).to(torch.bfloat16).to(DEV)
        idx = torch.randint(-1, e, (tt, k), generator=g).to(DEV)
        w = torch.rand(tt, k, generator=g).to(DEV)
        rx0, src0, cnt0, per_e0, rs0 = torch.ops.umdk_cam_op_lib.moe_dispatch_prefill_quant(x, idx, w, 0, buf.name, 0, 1,
                                                                                            quant_mode)
        buf.check()
        n = rx0.shape[0]
        want_off = buf.native.expert_offsets(e + 1).cpu()
        rx, rs, src, off, status = _call(lib, x, idx, e, quant_mode, capacity=tt * k)
        assert status == 0, lib.cam_dispatch_local_noalloc_error().decode()
        assert torch.equal(off.cpu(), want_off) and int(off[-1]) == n
        assert torch.equal(src[:n].cpu().reshape(-1), src0.cpu())
        assert torch.equal(rx[:n].cpu(), rx0.contiguous().view(torch.uint8).reshape(n, -1).cpu())
        if quant_mode in (3, 4):
            assert torch.equal(rs[:n].cpu(), rs0.cpu())
        assert (src[n:] == -7).all()  # nothing beyond the last row was touched
    buf.destroy()


@pytest.mark.parametrize("quant_mode", [2, 3])
def test_noalloc_dispatch_many_pairs_per_cta(quant_mode):
    """8192 tokens x 16 pairs at hidden 128: every CTA makes several passes over its pairs (more pairs per CTA than
    it has threads), with per-token int8 and with fp8 rows; compared with the Buffer dispatch row for row."""
    lib = _lib()
    t, h, e, k = 8192, 128, 64, 16
    cfg = u.CamConfig(num_experts=e, max_tokens=t, hidden=h, topk=k, timeout_ms=4000.0)
    buf = u.Buffer(None, cfg, name=f"na_big{quant_mode}", device=DEV, rank=0, num_ranks=1)
    g = torch.Generator().manual_seed(3 + quant_mode)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16).to(DEV)
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)])
    idx[::11, 5] = -1
    idx[7, 0] = 2 ** 32 + 3          # must be skipped, not taken for expert 3
    idx = idx.to(DEV)
    w = torch.rand(t, k, generator=g).to(DEV)
    rx0, src0, cnt0, per_e0, rs0 = torch.ops.umdk_cam_op_lib.moe_dispatch_prefill_quant(x, idx, w, 0, buf.name, 0, 1,
                                                                                        quant_mode)
    buf.check()
    n = rx0.shape[0]
    assert n == int(((idx >= 0) & (idx < e)).sum())
    rx, rs, src, off, status = _call(lib, x, idx, e, quant_mode, capacity=t * k)
    assert status == 0, lib.cam_dispatch_local_noalloc_error().decode()
    assert int(off[-1]) == n and torch.equal(off.cpu(), buf.native.expert_offsets(e + 1).cpu())
    assert torch.equal(src[:n].cpu().reshape(-1), src0.cpu())
    assert torch.equal(rx[:n].cpu(), rx0.contiguous().view(torch.uint8).reshape(n, -1).cpu())
    assert torch.equal(rs[:n].cpu().reshape(-1), rs0.cpu().reshape(-1))
    buf.destroy()


def test_noalloc_rejects_oversize_and_reports_overflow():
    lib = _lib()
    x = torch.zeros(8, 128, dtype=torch.bfloat16, device=DEV)
    idx = torch.zeros(8, 2, dtype=torch.int64, device=DEV)
    out = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    # more pairs than the built-in scratch holds: refused before any launch
    rc = lib.cam_dispatch_local_noalloc(x.data_ptr(), idx.data_ptr(), 1, 8192 * 16 + 1, 1, 128, 4, 0, 16, out.data_ptr(),
                                        None, out.data_ptr(), out.data_ptr(), stream)
    assert rc == -1 and b"scratch limit" in lib.cam_dispatch_local_noalloc_error()
    rc = lib.cam_dispatch_local_noalloc(x.data_ptr(), idx.data_ptr(), 1, 8, 2, 128, 4096, 0, 16, out.data_ptr(), None,
                                        out.data_ptr(), out.data_ptr(), stream)
    assert rc == -1
    # a pointer the 16-byte row accesses cannot use: refused with a message, nothing is launched
    rc = lib.cam_dispatch_local_noalloc(x.data_ptr() + 2, idx.data_ptr(), 1, 4, 2, 128, 4, 0, 16, out.data_ptr(), None,
                                        out.data_ptr(), out.data_ptr(), stream)
    assert rc == -1 and b"aligned" in lib.cam_dispatch_local_noalloc_error()
    rc = lib.cam_dispatch_local_noalloc(x.data_ptr(), idx.data_ptr(), 1, 4, 2, 128, 4, 0, 16, out.data_ptr() + 8, None,
                                        out.data_ptr(), out.data_ptr(), stream)
    assert rc == -1 and b"aligned" in lib.cam_dispatch_local_noalloc_error()
    # outputs too small for the rows: the kernel writes no row and the status says so
    rx, rs, src, off, status = _call(lib, x, idx, 4, 0, capacity=5)
    assert status == -3 and int(off[-1]) == 16
    assert (src == -7).all()
