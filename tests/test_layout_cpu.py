"""Symmetric-memory layout (CamLayout) checked on the CPU through the C runtime: regions are aligned, ordered,
disjoint and large enough for what the kernels put there.  The reference sizes its windows from
globalBs = maxBs * R with fixed flag / data areas (src/cam/comm_operator/ascend_kernels/utils/op_kernel/comm_args.h:17-80)."""
import ctypes
import os

import pytest

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "umdk_original_b200", "lib",
                   "libumdk_cam.so")
CAM_MAX_RANKS = 72  # flag arrays are sized for this many ranks (cam_types.h)

OFFSETS = ["off_count_flag", "off_data_flag", "off_combine_flag", "off_barrier_flag", "off_ll_combine_flag",
           "off_count_matrix", "off_ll_cells", "off_recv_x", "off_recv_scales", "off_recv_src", "off_combine_buf",
           "off_ll_x", "off_ll_scales", "off_ll_meta", "off_ll_combine_buf", "off_tp_flag", "off_tp_cnt", "off_tp_x",
           "off_tp_scales", "off_dup_cnt", "off_dup_list", "off_arrival", "off_guard0", "off_guard1", "off_guard2", "off_guard3", "total_bytes"]


class CamLayout(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("num_ranks", "num_experts", "max_tokens", "hidden", "topk", "capacity",
                                              "ll_max_tokens", "tp_rows")] + [(n, ctypes.c_uint64) for n in OFFSETS]


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        pytest.skip("native library not built")
    handle = ctypes.CDLL(LIB)
    handle.cam_layout_compute_tp.argtypes = [ctypes.POINTER(CamLayout)] + [ctypes.c_int] * 8
    handle.cam_layout_compute_tp.restype = ctypes.c_int
    return handle


def _layout(lib, r, e, t, h, k, cap, ll, tp_rows=0):
    lay = CamLayout()
    assert lib.cam_layout_compute_tp(ctypes.byref(lay), r, e, t, h, k, cap, ll, tp_rows) == 0
    return lay


@pytest.mark.parametrize("r,e,t,h,k,ll,tp_rows", [(1, 8, 64, 256, 2, 0, 0), (8, 256, 4096, 7168, 8, 128, 0),
                                                  (2, 4, 16, 256, 2, 16, 64), (4, 128, 8192, 4096, 8, 0, 0)])
def test_regions_are_aligned_ordered_and_big_enough(lib, r, e, t, h, k, ll, tp_rows):
    cap = t * min(k, e // r) * r
    lay = _layout(lib, r, e, t, h, k, cap, ll, tp_rows)
    el = e // r
    need = {
        "off_count_flag": 4 * CAM_MAX_RANKS, "off_data_flag": 4 * CAM_MAX_RANKS, "off_combine_flag": 4 * CAM_MAX_RANKS,
        "off_barrier_flag": 4 * CAM_MAX_RANKS, "off_ll_combine_flag": 4 * CAM_MAX_RANKS,
        "off_count_matrix": 4 * 2 * r * e, "off_ll_cells": 8 * 2 * e,  # one cell per (source, local expert), two parities
        "off_recv_x": cap * h * 2, "off_recv_scales": 4 * cap * (h // 128), "off_recv_src": 12 * cap,
        "off_combine_buf": 2 * t * k * h,
        "off_ll_x": 2 * (r * el) * ll * h * 2, "off_ll_scales": 4 * 2 * (r * el) * ll * (h // 128),
        "off_ll_meta": 8 * 2 * (r * el) * ll, "off_ll_combine_buf": 2 * ll * k * h,
        "off_tp_flag": 8, "off_tp_cnt": 8,
        "off_tp_x": tp_rows * h * 2, "off_tp_scales": 4 * tp_rows * (h // 128),
        "off_dup_cnt": 4 * 2 * CAM_MAX_RANKS, "off_dup_list": 8 * 2 * r * t * k,
        "off_arrival": 4 * 2 * e,  # rows landed per local expert of the fused layer, two parities
        "off_guard0": 64, "off_guard1": 64, "off_guard2": 64, "off_guard3": 64,
    }
    # regions that this configuration does not have (no low-latency mode, no TP partner) keep offset 0
    offs = sorted((getattr(lay, n), n) for n in OFFSETS if n != "total_bytes" and need[n] > 0)
    assert all(getattr(lay, n) == 0 for n in OFFSETS if n != "total_bytes" and need[n] == 0)
    total = lay.total_bytes
    assert total % 16 == 0 and total > 0
    for (off, name), nxt in zip(offs, [o for o, _ in offs[1:]] + [total]):
        assert off % 16 == 0, f"{name} is not 16-byte aligned (bulk copies and vector stores need it)"
        assert nxt - off >= need[name], f"{name}: {nxt - off} bytes before the next region, needs {need[name]}"
    assert lay.capacity == cap and lay.num_ranks == r and lay.tp_rows == tp_rows


def test_rejects_what_the_kernels_cannot_handle(lib):
    lay = CamLayout()
    for args in ((0, 8, 64, 256, 2, 128, 0, 0),        # no ranks
                 (3, 8, 64, 256, 2, 128, 0, 0),        # experts not divisible by ranks
                 (2, 8, 64, 200, 2, 128, 0, 0),        # hidden not a multiple of 128
                 (2, 8, 64, 256, 0, 128, 0, 0)):       # top-k of zero
        assert lib.cam_layout_compute_tp(ctypes.byref(lay), *args) != 0, args


def test_size_hint_matches_the_layout(lib):
    import umdk_original_b200 as u
    cfg = u.CamConfig(num_experts=256, max_tokens=4096, hidden=7168, topk=8, ll_max_tokens=128)
    lay = _layout(lib, 8, 256, 4096, 7168, 8, cfg.resolve_capacity(8), 128)
    hint = u.Buffer.get_size_hint(cfg, 8)
    assert abs(hint - lay.total_bytes) <= 0.02 * lay.total_bytes, (hint, lay.total_bytes)


def _gemm_args(lib, **over):
    """Argument list of cam_grouped_gemm_mxfp8 with dummy non-null pointers (validation runs before any CUDA call)."""
    lib.cam_grouped_gemm_mxfp8.restype = ctypes.c_int
    lib.cam_last_error.restype = ctypes.c_char_p
    ptr = ctypes.c_void_p(0x1000)
    a = dict(b=None, a_q=ptr, a_scales=ptr, a_rows=128, w_q=ptr, w_scales=ptr, offs=ptr, num_experts=1, n_dim=256,
             k_dim=128, mode=0, out=ptr, act_q=None, act_s=None, row_src=None, topk=0, ll=0, stream=None)
    a.update(over)
    return [a["b"], a["a_q"], a["a_scales"], ctypes.c_int(a["a_rows"]), a["w_q"], a["w_scales"], a["offs"],
            ctypes.c_int(a["num_experts"]), ctypes.c_int(a["n_dim"]), ctypes.c_int(a["k_dim"]), ctypes.c_int(a["mode"]),
            a["out"], a["act_q"], a["act_s"], a["row_src"], ctypes.c_int(a["topk"]), ctypes.c_int(a["ll"]), a["stream"]]


@pytest.mark.parametrize("over,word", [
    (dict(a_q=None), "null operand"),
    (dict(k_dim=100), "multiple of 128"),
    (dict(mode=7), "mode"),
    (dict(mode=1, n_dim=384, act_q=ctypes.c_void_p(0x1000), act_s=ctypes.c_void_p(0x1000)), "multiple of 256"),
    (dict(mode=1), "act_q"),
    (dict(mode=0, out=None), "output"),
    (dict(mode=2), "row_src"),
    (dict(num_experts=0), "empty problem"),
])
def test_grouped_gemm_rejects_bad_shapes_before_any_launch(lib, over, word):
    rc = lib.cam_grouped_gemm_mxfp8(*_gemm_args(lib, **over))
    assert rc != 0
    assert word in lib.cam_last_error().decode(), lib.cam_last_error()


def test_status_strings_cover_every_code(lib):
    lib.cam_status_string.restype = ctypes.c_char_p
    texts = [lib.cam_status_string(c).decode() for c in range(0, 11)]
    assert texts[0] == "ok" and len(set(texts)) == len(texts) and "unknown status" not in texts
    assert lib.cam_status_string(999).decode() == "unknown status"
