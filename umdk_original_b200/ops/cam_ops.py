"""``torch.ops.umdk_cam_op_lib``: loading of the native extension and the CPU implementations.

The schemas, the CUDA implementations, the Meta implementations and the Autograd wrappers are
registered by the native extension (csrc/bindings.cpp), mirroring the reference's
pybind/pybind.cpp:23-42.  This module

* imports the extension (or, where it has not been built and there is no GPU, defines the same
  schemas from Python so that the CPU path still works);
* registers the ``CPU`` dispatch key of every op on the gloo backend;
* refuses to run on a machine with a GPU when the extension is missing, instead of silently
  falling back.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import reference as ref

_C = None
_IMPORT_ERROR: Optional[BaseException] = None
try:  # the native extension registers the library on import
    from .. import _C as _C  # type: ignore
except Exception as e:  # noqa: BLE001
    _IMPORT_ERROR = e

SCHEMAS = [
    "fused_deep_moe(Tensor x, Tensor expertIds, Tensor[] gmm1PermutedWeight, Tensor[] gmm1PermutedWeightScale, "
    "Tensor[] gmm2Weight, Tensor[] gmm2WeightScale, Tensor expertScales, Tensor? expertSmoothScales, "
    "Tensor? xActiveMask, str groupEp, int epRankSize, int epRankId, int moeExpertNum, int sharedExpertNum, "
    "int sharedExpertRankNum, int quantMode, int globalBs) -> Tensor[]",
    "get_dispatch_layout(Tensor topk_idx, int num_experts, int num_ranks) -> (Tensor, Tensor, Tensor)",
    "moe_dispatch_prefill(Tensor x, Tensor topk_idx, Tensor topk_weights, Tensor num_tokens_per_rank, "
    "Tensor is_token_in_rank, Tensor num_tokens_per_expert, int num_worst_tokens, str group_ep, int rank, "
    "int num_ranks) -> (Tensor, Tensor, Tensor, Tensor)",
    "moe_combine_prefill(Tensor x, Tensor topk_idx, Tensor topk_weights, Tensor src_idx, Tensor send_head, "
    "str group_ep, int rank, int num_ranks) -> Tensor",
    "moe_dispatch_shmem(Tensor x, Tensor expertIds, Tensor? scales, Tensor? xActiveMask, int epWorldSize, "
    "int epRankId, int moeExpertNum, int tpWorldSize, int tpRankId, int expertShardType, int sharedExpertNum, "
    "int sharedExpertRankNum, int quantMode, int globalBS, int expertTokenNumsType, int extInfo) -> Tensor[]",
    "moe_combine_shmem(Tensor expandX, Tensor expertIds, Tensor expandIdx, Tensor epSendCounts, "
    "Tensor expertScales, Tensor? tpSendCounts, Tensor? xActiveMask, Tensor? activationScale, "
    "Tensor? weightScale, Tensor? groupList, Tensor? expandScales, int epWorldSize, int epRankId, "
    "int moeExpertNum, int tpWorldSize, int tpRankId, int expertShardType, int sharedExpertNum, "
    "int sharedExpertRankNum, int globalBS, int commQuantMode, int extInfo, int outDtype, int groupListType) "
    "-> Tensor",
    "moe_dispatch_prefill_quant(Tensor x, Tensor topk_idx, Tensor topk_weights, int num_worst_tokens, "
    "str group_ep, int rank, int num_ranks, int quant_mode) -> (Tensor, Tensor, Tensor, Tensor, Tensor)",
    "grouped_gemm_fp8(Tensor a_q, Tensor a_s, Tensor w_q, Tensor w_s, Tensor expert_offsets, "
    "bool ue8m0=False) -> Tensor",
    "grouped_gemm_fp8_swiglu(Tensor a_q, Tensor a_s, Tensor w_q, Tensor w_s, Tensor expert_offsets, "
    "bool ue8m0=False) -> (Tensor, Tensor)",
    "grouped_gemm_w8a8(Tensor a_q, Tensor a_s, Tensor w_q, Tensor w_s, Tensor expert_offsets) -> Tensor",
]

if _C is None:
    if torch.cuda.is_available():
        raise ImportError(
            "umdk_original_b200: the native extension is not built but a GPU is present; run "
            "`python -m umdk_original_b200._build` (refusing to fall back to the CPU path)") from _IMPORT_ERROR
    _DEF = torch.library.Library("umdk_cam_op_lib", "DEF")
    for _s in SCHEMAS:
        _DEF.define(_s)

_CPU = torch.library.Library("umdk_cam_op_lib", "IMPL", "CPU")


def native_loaded() -> bool:
    return _C is not None


def native_module():
    if _C is None:
        raise RuntimeError(f"umdk_original_b200: native extension not available: {_IMPORT_ERROR}")
    return _C


# ------------------------------------------------------------------------------------------------
# CPU implementations (gloo)
# ------------------------------------------------------------------------------------------------
def _reg():
    from ..parallel import registry
    return registry


def _backend():
    from ..parallel import gloo_backend
    return gloo_backend


def _get_dispatch_layout_cpu(topk_idx, num_experts, num_ranks):
    return ref.get_dispatch_layout(topk_idx, num_experts, num_ranks)


def _dispatch_prefill_common(x, topk_idx, group_ep, rank, num_ranks, quant_mode, num_worst_tokens):
    g = _reg().by_name(group_ep)
    assert g.rank == rank and g.world == num_ranks, "rank/num_ranks do not match the registered Buffer"
    rx, rs, src, cnt, per_e, _ = _backend().dispatch(g, x, topk_idx, quant_mode)
    if num_worst_tokens > 0:
        pad = num_worst_tokens - rx.shape[0]
        assert pad >= 0, "num_worst_tokens is smaller than the rows received"
        rx = torch.cat([rx, rx.new_zeros((pad, rx.shape[1]))]) if rx.dtype != ref.FP8 else torch.cat(
            [rx.view(torch.uint8), torch.zeros((pad, rx.shape[1]), dtype=torch.uint8)]).view(ref.FP8)
        src = torch.cat([src, src.new_full((pad, 3), -1)])
        if rs is not None:
            rs = torch.cat([rs, rs.new_zeros((pad, rs.shape[1]))])
    if rs is None:
        rs = torch.empty(0, dtype=torch.float32)
    return rx, src.reshape(-1), cnt, per_e, rs


def _moe_dispatch_prefill_cpu(x, topk_idx, topk_weights, num_tokens_per_rank, is_token_in_rank,
                              num_tokens_per_expert, num_worst_tokens, group_ep, rank, num_ranks):
    r = _dispatch_prefill_common(x, topk_idx, group_ep, rank, num_ranks, 0, num_worst_tokens)
    return r[0], r[1], r[2], r[3]


def _moe_dispatch_prefill_quant_cpu(x, topk_idx, topk_weights, num_worst_tokens, group_ep, rank, num_ranks, quant_mode):
    return _dispatch_prefill_common(x, topk_idx, group_ep, rank, num_ranks, quant_mode, num_worst_tokens)


def _moe_combine_prefill_cpu(x, topk_idx, topk_weights, src_idx, send_head, group_ep, rank, num_ranks):
    g = _reg().by_name(group_ep)
    src = src_idx.reshape(-1, 3)
    src = src[src[:, 0] >= 0]
    return _backend().combine(g, x, src, topk_idx, topk_weights)


def _moe_dispatch_shmem_cpu(x, expertIds, scales, xActiveMask, epWorldSize, epRankId, moeExpertNum, tpWorldSize,
                            tpRankId, expertShardType, sharedExpertNum, sharedExpertRankNum, quantMode, globalBS,
                            expertTokenNumsType, extInfo):
    g = _reg().by_id(extInfo)
    if quantMode == 1:
        raise RuntimeError("umdk_cam_op_lib: static quantisation (quantMode 1) is rejected, as in the reference")
    if tpWorldSize not in (0, 1, 2) or (tpWorldSize == 2 and g.tp_group is None):
        raise RuntimeError("umdk_cam_op_lib: tpWorldSize must be 1 or 2 (as in the reference), and 2 needs a Buffer "
                           "created with tp_group")
    t, k = expertIds.shape
    ids = expertIds
    el = moeExpertNum // epWorldSize
    shared_rank = epRankId < sharedExpertRankNum
    if sharedExpertRankNum > 0:
        ids, _, e_virtual, el = ref.remap_for_shared_ranks(expertIds, None, epWorldSize, moeExpertNum, sharedExpertRankNum)
        assert g.num_experts == e_virtual, "the Buffer must be created for R * E_local virtual experts"
    a = max(1, -(-t * epWorldSize // sharedExpertRankNum) if shared_rank else t * epWorldSize * min(el, k))
    active = int(xActiveMask.sum()) if xActiveMask is not None else None
    rx, rs, src, cnt, per_e, slots = _backend().dispatch(g, x, ids, quantMode, active, scales)
    if sharedExpertRankNum > 0:
        slots = slots.view(t, k + 1)[:, :k].contiguous().view(-1)
        if shared_rank:
            per_e, cnt = per_e[:1], cnt[:epWorldSize]
    n = rx.shape[0]
    tp_counts = torch.zeros(max(tpWorldSize, 1), dtype=torch.int32)
    if tpWorldSize == 2:
        # all-gather inside the TP pair (moe_dispatch_shmem.h:936-1018): the partner's rows follow this rank's own
        counts = g.tp_all_gather_counts(n)
        rx = torch.cat([rx.view(torch.uint8), g.tp_exchange(rx, counts).view(torch.uint8)]).view(rx.dtype) \
            if rx.dtype == ref.FP8 else torch.cat([rx, g.tp_exchange(rx, counts)])
        if rs is not None:
            rs = torch.cat([rs, g.tp_exchange(rs, counts)])
        tp_counts = torch.tensor(counts, dtype=torch.int32)
        g.tp_counts = tp_counts
        n, a = rx.shape[0], 2 * a
    pad = a - n
    if rx.dtype == ref.FP8:
        expand = torch.cat([rx.view(torch.uint8), torch.zeros((pad, rx.shape[1]), dtype=torch.uint8)]).view(ref.FP8)
    else:
        expand = torch.cat([rx, rx.new_zeros((pad, rx.shape[1]))])
    if quantMode in (3, 4):
        dyn = torch.cat([rs, rs.new_zeros((pad, rs.shape[1]))])
    elif quantMode == 2:
        dyn = torch.cat([rs.reshape(-1), rs.new_zeros(pad)])
    else:
        dyn = torch.zeros(a, dtype=torch.float32)
    g.ll_src = src
    nums = per_e if expertTokenNumsType == 1 else per_e.cumsum(0)
    return [expand, dyn, slots, nums.to(torch.int64), cnt, tp_counts]


def _moe_combine_shmem_cpu(expandX, expertIds, expandIdx, epSendCounts, expertScales, tpSendCounts, xActiveMask,
                           activationScale, weightScale, groupList, expandScales, epWorldSize, epRankId,
                           moeExpertNum, tpWorldSize, tpRankId, expertShardType, sharedExpertNum,
                           sharedExpertRankNum, globalBS, commQuantMode, extInfo, outDtype, groupListType):
    g = _reg().by_id(extInfo)
    if g.ll_src is None:
        raise RuntimeError("umdk_cam_op_lib: moe_combine_shmem needs a preceding moe_dispatch_shmem on the same Buffer")
    ids, w = expertIds, expertScales
    if sharedExpertRankNum > 0:
        ids, w, _, _ = ref.remap_for_shared_ranks(expertIds, expertScales, epWorldSize, moeExpertNum, sharedExpertRankNum)
    if xActiveMask is not None:
        ids = ids.clone()
        ids[int(xActiveMask.sum()):] = -1
    y = expandX
    if tpWorldSize == 2:
        # reduce-scatter inside the TP pair (moe_combine_shmem.h:438-470): the partner gets this rank's partial outputs
        # of the partner's rows and this rank adds the partner's partial outputs of its own rows
        if g.tp_group is None or g.tp_counts is None:
            raise RuntimeError("umdk_cam_op_lib: tpWorldSize 2 needs a Buffer created with tp_group and a preceding "
                               "moe_dispatch_shmem")
        counts = g.tp_counts.tolist()
        n_own, n_other = counts[g.tp_rank], counts[1 - g.tp_rank]
        swapped = [0, 0]  # what each TP rank contributes: its partial outputs of the OTHER rank's rows
        swapped[g.tp_rank], swapped[1 - g.tp_rank] = n_other, n_own
        partner = g.tp_exchange(expandX[n_own:n_own + n_other].contiguous(), swapped)
        y = (expandX[:n_own].float() + partner.float()).to(expandX.dtype)
    if commQuantMode == 2:  # int8 on the wire, one scale per 128 elements
        q, s = ref.quant_int8_1x128(y)
        y = ref.dequant_int8_1x128(q, s)
    return _backend().combine(g, y, g.ll_src, ids, w)


def _stack(ws) -> torch.Tensor:
    ws = list(ws)
    return ws[0] if len(ws) == 1 and ws[0].dim() == 3 else torch.stack([w for w in ws])


def _fused_deep_moe_cpu(x, expertIds, gmm1PermutedWeight, gmm1PermutedWeightScale, gmm2Weight, gmm2WeightScale,
                        expertScales, expertSmoothScales, xActiveMask, groupEp, epRankSize, epRankId, moeExpertNum,
                        sharedExpertNum, sharedExpertRankNum, quantMode, globalBs):
    if expertSmoothScales is not None:
        raise RuntimeError("expertSmoothScales is not supported by fused_deep_moe (pass None; moe_dispatch_shmem "
                           "applies smooth scales)")
    g = _reg().by_name(groupEp)
    be = _backend()
    # fp16 activations are accepted like bf16 ones (fused_deep_moe.cpp:17-19 of the reference): the layer computes on
    # bf16 rows, as the CUDA implementation does, and the result comes back in the caller's dtype
    in_dtype = x.dtype
    if x.dtype == torch.float16:
        x = x.to(torch.bfloat16)
    w1, s1 = _stack(gmm1PermutedWeight), _stack(gmm1PermutedWeightScale)
    w2, s2 = _stack(gmm2Weight), _stack(gmm2WeightScale)
    el = moeExpertNum // epRankSize
    active = int(xActiveMask.sum()) if xActiveMask is not None else None
    ids = expertIds
    if sharedExpertRankNum > 0:
        ids, expertScales, e_virtual, _ = ref.remap_for_shared_ranks(expertIds, expertScales, epRankSize, moeExpertNum,
                                                                     sharedExpertRankNum)
        assert g.num_experts == e_virtual, "the Buffer must be created for R * E_local virtual experts"
        el = w1.shape[0]  # 1 on a shared-expert rank
    if active is not None:
        ids = ids.clone()
        ids[active:] = -1
    if w1.dtype == ref.FP8:  # block-scaled fp8 (quantMode 3; 4 = power-of-two scales)
        po2 = quantMode == 4
        rx, rs, src, cnt, per_e, _ = be.dispatch(g, x, ids, 4 if po2 else 3)
        y = torch.zeros(rx.shape[0], x.shape[1], dtype=torch.bfloat16)
        off = torch.cat([torch.zeros(1, dtype=torch.long), per_e.cumsum(0)])
        for le in range(el):
            a, b = int(off[le]), int(off[le + 1])
            if b > a:
                y[a:b] = ref.expert_mlp_fp8(rx[a:b], rs[a:b], w1[le], s1[le], w2[le], s2[le], ue8m0=po2)
    elif w1.dtype == torch.int8:  # reference layout: w1 [E_l, h, 2I], s1 [E_l, 2I], w2 [E_l, I, h], s2 [E_l, h]
        rx, rs, src, cnt, per_e, _ = be.dispatch(g, x, ids, 0)
        y = torch.zeros(rx.shape[0], x.shape[1], dtype=torch.bfloat16)
        off = torch.cat([torch.zeros(1, dtype=torch.long), per_e.cumsum(0)])
        for le in range(el):
            a, b = int(off[le]), int(off[le + 1])
            if b > a:
                y[a:b] = ref.expert_mlp_w8a8(rx[a:b], w1[le].t(), s1[le], w2[le].t(), s2[le])
    else:  # floating-point weights: plain SwiGLU MLP, w1 [E_l, 2I, h], w2 [E_l, h, I]
        rx, rs, src, cnt, per_e, _ = be.dispatch(g, x, ids, 0)
        y = torch.zeros(rx.shape[0], x.shape[1], dtype=x.dtype)
        off = torch.cat([torch.zeros(1, dtype=torch.long), per_e.cumsum(0)])
        for le in range(el):
            a, b = int(off[le]), int(off[le + 1])
            if b > a:
                y[a:b] = ref.swiglu_mlp_fp32(rx[a:b], w1[le], w2[le]).to(x.dtype)
    out = be.combine(g, y, src, ids, expertScales, out_dtype=x.dtype)
    return [out.to(in_dtype), per_e[:el].to(torch.int64)]


def _grouped_gemm_fp8_cpu(a_q, a_s, w_q, w_s, expert_offsets, ue8m0=False):
    out = torch.zeros(a_q.shape[0], w_q.shape[1], dtype=torch.bfloat16)
    off = expert_offsets.tolist()
    for e in range(w_q.shape[0]):
        a, b = off[e], off[e + 1]
        if b > a:
            out[a:b] = (ref.dequant_fp8_1x128(a_q[a:b], a_s[a:b]) @ ref.dequant_fp8_128x128(w_q[e], w_s[e]).t()).to(torch.bfloat16)
    return out


def _grouped_gemm_fp8_swiglu_cpu(a_q, a_s, w_q, w_s, expert_offsets, ue8m0=False):
    i = w_q.shape[1] // 2
    q = torch.zeros(a_q.shape[0], i, dtype=torch.uint8).view(ref.FP8)
    s = torch.zeros(a_q.shape[0], i // 128, dtype=torch.float32)
    off = expert_offsets.tolist()
    for e in range(w_q.shape[0]):
        a, b = off[e], off[e + 1]
        if b > a:
            y = ref.dequant_fp8_1x128(a_q[a:b], a_s[a:b]) @ ref.dequant_fp8_128x128(w_q[e], w_s[e]).t()
            act = (y[:, :i] / (1.0 + torch.exp(-y[:, :i]))) * y[:, i:]
            qq, ss = ref.quant_fp8_1x128(act, ue8m0)
            q.view(torch.uint8)[a:b] = qq.view(torch.uint8)
            s[a:b] = ss
    return q, s


_CPU.impl("get_dispatch_layout", _get_dispatch_layout_cpu)
_CPU.impl("moe_dispatch_prefill", _moe_dispatch_prefill_cpu)
_CPU.impl("moe_dispatch_prefill_quant", _moe_dispatch_prefill_quant_cpu)
_CPU.impl("moe_combine_prefill", _moe_combine_prefill_cpu)
_CPU.impl("moe_dispatch_shmem", _moe_dispatch_shmem_cpu)
_CPU.impl("moe_combine_shmem", _moe_combine_shmem_cpu)
_CPU.impl("fused_deep_moe", _fused_deep_moe_cpu)
_CPU.impl("grouped_gemm_fp8", _grouped_gemm_fp8_cpu)
def _grouped_gemm_w8a8_cpu(a_q, a_s, w_q, w_s, expert_offsets):
    """Exact int32 accumulation: out = (a_q @ w_q^T) * a_s[row] * w_s[expert, col]."""
    out = torch.zeros(a_q.shape[0], w_q.shape[1], dtype=torch.bfloat16)
    off = expert_offsets.tolist()
    for e in range(w_q.shape[0]):
        a, b = off[e], off[e + 1]
        if b > a:
            acc = a_q[a:b].double() @ w_q[e].double().t()
            out[a:b] = (acc.float() * a_s[a:b].float().unsqueeze(-1) * w_s[e].float().unsqueeze(0)).to(torch.bfloat16)
    return out


_CPU.impl("grouped_gemm_fp8_swiglu", _grouped_gemm_fp8_swiglu_cpu)
_CPU.impl("grouped_gemm_w8a8", _grouped_gemm_w8a8_cpu)

ops = torch.ops.umdk_cam_op_lib
