// Normal-mode (prefill) dispatch for sm_100a: ONE kernel that builds the routing layout,
// all-gathers the per-expert counts through peer memory, quantises every token once and pushes
// each (token, k) row with plain P2P stores into its final, expert-grouped position in the
// destination rank's receive buffer, then raises a completion flag in every peer's memory.
//
// It replaces, in the reference, the chain dispatch_layout + notify_dispatch + two host loops +
// moe_dispatch_normal (pybind/moe_dispatch_prefill.cpp:96-160 and
// ascend_kernels/moe_dispatch_normal/op_kernel/moe_dispatch_normal.h:331-535): there a row is
// staged in the sender's window, flagged, pulled by the receiver and copied again; the slot of a
// row inside its expert and the receive offsets are computed on the host after two device->host
// copies.  Here the slot arithmetic runs on the device and a row crosses NVLink exactly once.
//
// Receive-buffer row order (same contract as the reference): local expert major, then source
// rank ascending, then the sender's (token, k) scan order.
#include <cooperative_groups.h>
#include "../common/cam_types.h"
#include "../common/ptx.cuh"
#include "../common/quant.cuh"
#include "launch.h"

namespace cg = cooperative_groups;

namespace cam {

constexpr int kDispThreads = 512;
constexpr int kDispWarps = kDispThreads / 32;

__device__ __forceinline__ void record_status(CamStatus* st, int code, int who, int detail) {
    if (atomicCAS(&st->code, 0, code) == 0) {
        st->who = who;
        st->detail = detail;
        st->block = static_cast<int>(blockIdx.x);
    }
}

__global__ void __launch_bounds__(kDispThreads, 1)
dispatch_normal_kernel(const DispatchNormalParams p) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    __shared__ int s_hist[CAM_MAX_EXPERTS];     // running per-expert count of this CTA's chunk
    __shared__ int s_aux[CAM_MAX_EXPERTS];      // prefix over earlier CTAs / totals / bases
    __shared__ int s_tot[CAM_MAX_EXPERTS];      // rows per expert summed over all sources
    __shared__ int s_ids[kDispThreads];
    __shared__ int s_rank_ok[CAM_MAX_RANKS];
    __shared__ uint32_t s_abort;
    __shared__ int s_dup_pre[CAM_MAX_RANKS + 1];

    const int tid = static_cast<int>(threadIdx.x);
    const int nb = static_cast<int>(gridDim.x);
    const int b = static_cast<int>(blockIdx.x);
    const int E = p.E, R = p.R, K = p.K, El = p.E / p.R;
    const int tpc = (p.T + nb - 1) / nb;  // tokens per CTA (contiguous chunk keeps scan order)
    const int t0 = min(p.T, b * tpc);
    const int t1 = min(p.T, t0 + tpc);
    const int npairs = (t1 - t0) * K;
    // epochs of this call, one per phase (equal when a call runs all phases in one launch)
    const uint32_t ep_count = p.epochs[0] + 1u, ep_send = p.epochs[1] + 1u, ep_recv = p.epochs[2] + 1u;
    uint8_t* const my_base = p.peer_base[p.rank];

    if (tid == 0) s_abort = 0u;

    // ------------------------------------------------------------------ phase COUNT
    if (p.phase_mask & CAM_PHASE_COUNT) {
        const int parity = static_cast<int>(ep_count & 1u);
        for (int e = tid; e < E; e += kDispThreads) s_hist[e] = 0;
        __syncthreads();
        // Slot of every (token, k) pair inside its expert, in scan order, chunk-local first.
        for (int sub = 0; sub < npairs; sub += kDispThreads) {
            const int i = sub + tid;
            int id = -1;
            if (i < npairs) {
                id = load_expert_id(p.topk_idx, p.idx_is_i64, static_cast<size_t>(t0) * K + i);
                if (id < 0 || id >= E) id = -1;
            }
            s_ids[tid] = id;
            __syncthreads();
            if (id >= 0) {
                int r = 0;
                for (int j = 0; j < tid; ++j) r += (s_ids[j] == id) ? 1 : 0;
                p.slot_in_expert[static_cast<size_t>(t0) * K + i] = s_hist[id] + r;
            } else if (i < npairs) {
                p.slot_in_expert[static_cast<size_t>(t0) * K + i] = -1;
            }
            __syncthreads();
            if (id >= 0) atomicAdd(&s_hist[id], 1);
            __syncthreads();
        }
        for (int e = tid; e < E; e += kDispThreads) p.cta_hist[static_cast<size_t>(b) * E + e] = s_hist[e];
        if (p.g1_done != nullptr && b == nb - 1) {
            // Counters of the fused kernel start at zero.  Peers add to this call's arrival counters only after they
            // have seen this rank's count flag, which is raised after the grid-wide barrier below.
            if (p.defer_push) {
                uint32_t* arr = reinterpret_cast<uint32_t*>(my_base + p.off_arrival) + static_cast<size_t>(parity) * E;
                for (int e = tid; e < E; e += kDispThreads) arr[e] = 0u;
            }
            for (int i = tid; i < p.g1_done_len; i += kDispThreads) p.g1_done[i] = 0u;
            __threadfence_system();
        }
        __threadfence();
        cg::this_grid().sync();

        // Exclusive prefix over earlier CTAs (s_aux) and grand total (s_tot) per expert.
        for (int e = tid; e < E; e += kDispThreads) {
            int pre = 0, tot = 0;
            for (int bb = 0; bb < nb; ++bb) {
                const int c = __ldcg(&p.cta_hist[static_cast<size_t>(bb) * E + e]);
                pre += (bb < b) ? c : 0;
                tot += c;
            }
            s_aux[e] = pre;
            s_tot[e] = tot;
        }
        __syncthreads();
        for (int i = tid; i < npairs; i += kDispThreads) {
            const size_t g = static_cast<size_t>(t0) * K + i;
            const int id = load_expert_id(p.topk_idx, p.idx_is_i64, g);
            if (id >= 0 && id < E) p.slot_in_expert[g] += s_aux[id];
        }
        // Count all-gather: CTA d writes this rank's full count vector into peer d's matrix.
        for (int d = b; d < R; d += nb) {
            int* dst = reinterpret_cast<int*>(p.peer_base[d] + p.off_count_matrix) +
                       (static_cast<size_t>(parity) * R + p.rank) * E;
            for (int e = tid; e < E; e += kDispThreads) dst[e] = s_tot[e];
            __syncthreads();
            if (tid == 0 && p.dbg_drop_flags == 0) {
                __threadfence_system();
                st_release_sys_u32(reinterpret_cast<uint32_t*>(p.peer_base[d] + p.off_count_flag) + p.rank,
                                   ep_count);
            }
        }
        if (p.num_tokens_per_expert_out != nullptr && b == 0) {
            for (int e = tid; e < E; e += kDispThreads) p.num_tokens_per_expert_out[e] = s_tot[e];
        }
        __syncthreads();
    }

    // ------------------------------------------------------------------ phase SEND
    if (p.phase_mask & CAM_PHASE_SEND) {
        const int parity = static_cast<int>(ep_send & 1u);
        if (tid < R) {
            const uint32_t* f = reinterpret_cast<const uint32_t*>(my_base + p.off_count_flag) + tid;
            const uint64_t t_wait = (b == 0 && p.stats != nullptr) ? globaltimer_ns() : 0ull;
            if (!wait_flag_eq_sys(f, ep_send, p.timeout_ns)) {
                record_status(p.status, CAM_ERR_TIMEOUT_COUNT_FLAG, tid, static_cast<int>(ld_acquire_sys_u32(f)));
                s_abort = 1u;
            }
            if (b == 0 && p.stats != nullptr) atomicMax(&p.stats->max_wait_ns[0][tid], globaltimer_ns() - t_wait);
        }
        __syncthreads();
        if (s_abort) goto done;  // no grid-wide sync follows, so leaving here cannot strand another CTA

        const int* cm = reinterpret_cast<const int*>(my_base + p.off_count_matrix) +
                        static_cast<size_t>(parity) * R * E;
        for (int e = tid; e < E; e += kDispThreads) {
            int tot = 0;
            for (int s = 0; s < R; ++s) tot += __ldcg(&cm[static_cast<size_t>(s) * E + e]);
            s_tot[e] = tot;
        }
        __syncthreads();
        // Base row, at the owner of expert e, of the block of rows that come from this rank.
        for (int e = tid; e < E; e += kDispThreads) {
            const int d = e / El, le = e - d * El;
            int base = 0;
            for (int l = 0; l < le; ++l) base += s_tot[d * El + l];
            for (int s = 0; s < p.rank; ++s) base += __ldcg(&cm[static_cast<size_t>(s) * E + e]);
            s_aux[e] = base;
        }
        for (int d = tid; d < R; d += kDispThreads) {
            int tot = 0;
            for (int l = 0; l < El; ++l) tot += s_tot[d * El + l];
            s_rank_ok[d] = (tot <= p.capacity) ? 1 : 0;
            if (tot > p.capacity) record_status(p.status, CAM_ERR_RECV_OVERFLOW, d, tot);
            if (b == 0 && p.stats != nullptr) {
                int mine = 0;
                for (int l = 0; l < El; ++l) mine += __ldcg(&cm[static_cast<size_t>(p.rank) * E + d * El + l]);
                atomicAdd(&p.stats->rows_routed[d], static_cast<unsigned long long>(mine));
                if (d == 0) atomicAdd(&p.stats->calls[0], 1ull);
            }
        }
        __syncthreads();
        // Receiver-side bookkeeping for this rank's own experts (one CTA is enough).  When more rows are routed
        // here than the buffer holds, every sender skips this rank (s_rank_ok) and the counts published below are
        // zero, so that the kernels that follow touch no row at or past the capacity; the status word says why.
        if (b == 0) {
            const bool fits = s_rank_ok[p.rank] != 0;
            for (int le = tid; le < El; le += kDispThreads) {
                int start = 0;
                for (int l = 0; l < le; ++l) start += s_tot[p.rank * El + l];
                if (!fits) start = 0;
                p.expert_offsets[le] = start;
                int run = start;
                for (int s = 0; s < R; ++s) {
                    if (fits) run += __ldcg(&cm[static_cast<size_t>(s) * E + p.rank * El + le]);
                    p.recv_count[le * R + s] = run;  // inclusive cumsum, expert major / source minor
                }
                p.num_recv_per_expert[le] = fits ? static_cast<long long>(s_tot[p.rank * El + le]) : 0ll;
                if (le == El - 1) {
                    p.expert_offsets[El] = run;
                    p.total_recv[0] = run;
                }
            }
        }
        __syncthreads();

        // Push.  One warp per token: quantise once into the warp's staging area, then store the
        // row, its scales and its (src rank, token, k) triple to every destination.
        const int warp = tid >> 5;
        const uint32_t lane = lane_id();
        const int nscale = CAM_QUANT_IS_FP8(p.quant_mode) ? (p.h >> 7)
                           : (p.quant_mode == CAM_QUANT_INT8_TOKEN) ? 1 : 0;
        const int row_bytes = (p.quant_mode == CAM_QUANT_NONE) ? p.h * 2 : p.h;
        const int stage_bytes = (p.quant_mode == CAM_QUANT_NONE) ? 0 : ((p.h + nscale * 4 + 15) & ~15);
        uint8_t* stage_q = dyn_smem + static_cast<size_t>(warp) * stage_bytes;
        float* stage_s = reinterpret_cast<float*>(stage_q + p.h);

        // Quantised rows leave the staging area as bulk copies (one 7 KB transfer per destination
        // instead of 14 rounds of 16-byte stores per lane): lane k issues the copies of pair (t, k).
        //
        // A token crosses to a destination rank ONCE.  Lane k handles pair (t, k); lanes whose experts
        // live on the same rank find each other with match.any: the lowest of them sends the row, the
        // others append (row that arrives, row to copy it to) to the replicate list of that rank, which
        // the receiver works off locally after the data flags (RECV phase below).
        const bool bulk_rows = (p.quant_mode != CAM_QUANT_NONE) && (row_bytes % 16 == 0);
        const bool bulk_scales = bulk_rows && ((nscale * 4) % 16 == 0);
        if (p.defer_push) {
            // Nothing is pushed here.  Position of every pair in the send list: pairs are ordered by (local expert
            // at the destination, destination rank counted from this rank on, scan order), so expert 0 of every rank is
            // served first and, at any one time, the ranks of the group send to different destinations.
            int* s_mine = reinterpret_cast<int*>(dyn_smem);  // the staging area is unused in this mode
            for (int e = tid; e < E; e += kDispThreads)
                s_mine[e] = s_rank_ok[e / El] ? __ldcg(&cm[static_cast<size_t>(p.rank) * E + e]) : 0;
            __syncthreads();
            for (int e = tid; e < E; e += kDispThreads) {
                const int d = e / El, le = e - d * El;
                const int turn = (d - p.rank + R) % R;  // place of destination d in this rank's order
                int pre = 0;
                for (int l2 = 0; l2 < le; ++l2)
                    for (int d2 = 0; d2 < R; ++d2) pre += s_mine[d2 * El + l2];
                for (int t2 = 0; t2 < turn; ++t2) pre += s_mine[((p.rank + t2) % R) * El + le];
                s_hist[e] = pre;
                // the last key: the last local expert of the destination this rank serves last
                if (b == 0 && le == El - 1 && turn == R - 1) p.send_list_len[0] = pre + s_mine[e];
            }
            __syncthreads();
            for (int t = t0 + warp; t < t1; t += kDispWarps) {
                const __nv_bfloat16* xrow = p.x + static_cast<size_t>(t) * p.h;
                uint8_t* q = p.xq + static_cast<size_t>(t) * p.h;
                float* sc = p.xs + static_cast<size_t>(t) * nscale;
                if (p.quant_mode == CAM_QUANT_FP8_1x128_UE8M0) warp_quant_fp8_1x128<true>(xrow, p.h, q, sc);
                else warp_quant_fp8_1x128<false>(xrow, p.h, q, sc);
                if (lane < static_cast<uint32_t>(K)) {
                    const size_t g = static_cast<size_t>(t) * K + lane;
                    const int id = load_expert_id(p.topk_idx, p.idx_is_i64, g);
                    int row = -1;
                    if (id >= 0 && id < E && s_rank_ok[id / El]) {
                        const int d = id / El, slot = p.slot_in_expert[g];
                        row = s_aux[id] + slot;
                        p.send_list[s_hist[id] + slot] = make_int4(t, d, row, (id - d * El) | (static_cast<int>(lane) << 16));
                    }
                    p.send_row[g] = row;
                }
            }
        } else {
        for (int t = t0 + warp; t < t1; t += kDispWarps) {
            const __nv_bfloat16* xrow = p.x + static_cast<size_t>(t) * p.h;
            if (bulk_rows) {
                if (lane < static_cast<uint32_t>(K)) bulk_wait_group_read<0>();  // staging is free again
                __syncwarp();
            }
            if (p.quant_mode == CAM_QUANT_FP8_1x128) {
                warp_quant_fp8_1x128<false>(xrow, p.h, stage_q, stage_s);
            } else if (p.quant_mode == CAM_QUANT_FP8_1x128_UE8M0) {
                warp_quant_fp8_1x128<true>(xrow, p.h, stage_q, stage_s);
            } else if (p.quant_mode == CAM_QUANT_INT8_TOKEN) {
                warp_quant_int8_token(xrow, p.h, stage_q, stage_s);
            }
            __syncwarp();
            // pair of this lane
            int d = -1, row = -1;
            if (lane < static_cast<uint32_t>(K)) {
                const size_t g = static_cast<size_t>(t) * K + lane;
                const int id = load_expert_id(p.topk_idx, p.idx_is_i64, g);
                if (id >= 0 && id < E && s_rank_ok[id / El]) {
                    d = id / El;
                    row = s_aux[id] + p.slot_in_expert[g];
                }
                p.send_row[g] = row;
            }
            // rows for this rank's own experts are written directly (local stores cost less than a copy pass)
            const uint32_t peers =
                __match_any_sync(0xFFFFFFFFu, (d >= 0 && d != p.rank) ? d : -1 - static_cast<int>(lane));
            const int first = __ffs(static_cast<int>(peers)) - 1;
            const int first_row = __shfl_sync(0xFFFFFFFFu, row, first);
            const bool sends = d >= 0 && static_cast<int>(lane) == first;
            if (d >= 0) {
                uint8_t* pb = p.peer_base[d];
                int* tri = reinterpret_cast<int*>(pb + p.off_recv_src) + static_cast<size_t>(row) * 3;
                tri[0] = p.rank;
                tri[1] = t;
                tri[2] = static_cast<int>(lane);
                if (!sends) {
                    const unsigned int idx = atomicAdd(&p.dup_ctr[d], 1u);
                    int* ent = reinterpret_cast<int*>(pb + p.off_dup_list) +
                               ((static_cast<size_t>(parity) * R + p.rank) * p.dup_cap + idx) * 2;
                    st_na_v2(ent, make_uint2(static_cast<uint32_t>(first_row), static_cast<uint32_t>(row)));
                }
            }
            if (bulk_rows) {
                fence_proxy_async_smem();  // the staged row is read by the async proxy
                __syncwarp();
                if (sends) {
                    uint8_t* pb = p.peer_base[d];
                    bulk_store_s2g(pb + p.off_recv_x + static_cast<size_t>(row) * row_bytes, stage_q,
                                   static_cast<uint32_t>(row_bytes));
                    float* sdst = reinterpret_cast<float*>(pb + p.off_recv_scales) + static_cast<size_t>(row) * nscale;
                    if (bulk_scales) {
                        bulk_store_s2g(sdst, stage_s, static_cast<uint32_t>(nscale * 4));
                    } else {
                        for (int o = 0; o < nscale; ++o) sdst[o] = stage_s[o];
                    }
                }
                if (lane < static_cast<uint32_t>(K)) bulk_commit_group();
                __syncwarp();
                continue;
            }
            const uint32_t senders = __ballot_sync(0xFFFFFFFFu, sends);
            for (uint32_t m = senders; m != 0u; m &= m - 1u) {
                const int k = __ffs(static_cast<int>(m)) - 1;
                const int dk = __shfl_sync(0xFFFFFFFFu, d, k);
                const int rk = __shfl_sync(0xFFFFFFFFu, row, k);
                uint8_t* pb = p.peer_base[dk];
                uint8_t* dst = pb + p.off_recv_x + static_cast<size_t>(rk) * row_bytes;
                if (p.quant_mode == CAM_QUANT_NONE) {
                    warp_copy_row<false>(dst, reinterpret_cast<const uint8_t*>(xrow), row_bytes, lane);
                } else {
                    for (int o = static_cast<int>(lane) * 16; o < row_bytes; o += 512)
                        st_na_v4(dst + o, *reinterpret_cast<const uint4*>(stage_q + o));
                    float* sdst = reinterpret_cast<float*>(pb + p.off_recv_scales) + static_cast<size_t>(rk) * nscale;
                    for (int o = static_cast<int>(lane); o < nscale; o += 32) sdst[o] = stage_s[o];
                }
            }
            __syncwarp();
        }

        // Completion: the last CTA to finish raises this rank's data flag in every peer.
        if (bulk_rows && lane < static_cast<uint32_t>(K)) bulk_wait_group<0>();  // this lane's copies are written
        __syncthreads();
        if (tid == 0) {
            __threadfence_system();
            const unsigned int old = atomicAdd(p.done_ctr, 1u);
            if (old == static_cast<unsigned int>(nb - 1)) {
                p.done_ctr[0] = 0u;
                __threadfence_system();
                for (int d = 0; d < R; ++d) {  // length of the replicate list this rank wrote at d, then reset the cursor
                    const unsigned int n = atomicExch(&p.dup_ctr[d], 0u);
                    reinterpret_cast<uint32_t*>(p.peer_base[d] + p.off_dup_cnt)[parity * CAM_MAX_RANKS + p.rank] = n;
                }
                __threadfence_system();
                if (p.dbg_drop_flags == 0) {
                    for (int d = 0; d < R; ++d)
                        st_release_sys_u32(reinterpret_cast<uint32_t*>(p.peer_base[d] + p.off_data_flag) + p.rank,
                                           ep_send);
                }
            }
        }
        }  // !defer_push
    }

    // ------------------------------------------------------------------ phase RECV
    if (p.phase_mask & CAM_PHASE_RECV) {
        const int parity = static_cast<int>(ep_recv & 1u);
        if (tid < R) {
            const uint32_t* f = reinterpret_cast<const uint32_t*>(my_base + p.off_data_flag) + tid;
            const uint64_t t_wait = (b == 0 && p.stats != nullptr) ? globaltimer_ns() : 0ull;
            if (!wait_flag_eq_sys(f, ep_recv, p.timeout_ns)) {
                record_status(p.status, CAM_ERR_TIMEOUT_DATA_FLAG, tid, static_cast<int>(ld_acquire_sys_u32(f)));
                s_abort = 1u;
            }
            if (b == 0 && p.stats != nullptr) atomicMax(&p.stats->max_wait_ns[1][tid], globaltimer_ns() - t_wait);
        }
        __syncthreads();
        if (s_abort) goto done;
        // Replicate: rows that several local experts need arrived once; copy them to the other rows.
        if (tid == 0) {
            const uint32_t* cnt = reinterpret_cast<const uint32_t*>(my_base + p.off_dup_cnt) + parity * CAM_MAX_RANKS;
            int run = 0;
            for (int s = 0; s < R; ++s) {
                s_dup_pre[s] = run;
                run += static_cast<int>(min(__ldcg(cnt + s), static_cast<uint32_t>(p.dup_cap)));
            }
            s_dup_pre[R] = run;
        }
        __syncthreads();
        const int nscale = CAM_QUANT_IS_FP8(p.quant_mode) ? (p.h >> 7) : (p.quant_mode == CAM_QUANT_INT8_TOKEN) ? 1 : 0;
        const int row_bytes = (p.quant_mode == CAM_QUANT_NONE) ? p.h * 2 : p.h;
        const int warp = tid >> 5;
        const uint32_t lane = lane_id();
        const int total = s_dup_pre[R];
        uint8_t* rx = my_base + p.off_recv_x;
        float* rs = reinterpret_cast<float*>(my_base + p.off_recv_scales);
        for (int i = b * kDispWarps + warp; i < total; i += nb * kDispWarps) {
            int s = 0;
            while (s + 1 < R && s_dup_pre[s + 1] <= i) ++s;
            const int* ent = reinterpret_cast<const int*>(my_base + p.off_dup_list) +
                             ((static_cast<size_t>(parity) * R + s) * p.dup_cap + (i - s_dup_pre[s])) * 2;
            const int from = __ldcg(ent), to = __ldcg(ent + 1);
            if (from < 0 || to < 0 || from >= p.capacity || to >= p.capacity) {  // never copy out of range
                if (lane == 0) record_status(p.status, CAM_ERR_BAD_INDEX, 2, i);
                continue;
            }
            warp_copy_row<true>(rx + static_cast<size_t>(to) * row_bytes, rx + static_cast<size_t>(from) * row_bytes,
                                row_bytes, lane);
            for (int o = static_cast<int>(lane); o < nscale; o += 32)
                rs[static_cast<size_t>(to) * nscale + o] = __ldcg(rs + static_cast<size_t>(from) * nscale + o);
        }
    }

done:
    // the CTA that leaves last advances the epochs of the phases this launch ran
    __syncthreads();
    if (tid == 0 && last_cta_out(p.exit_ctr, static_cast<unsigned int>(nb))) {
        if (p.phase_mask & CAM_PHASE_COUNT) p.epochs[0] = ep_count;
        if (p.phase_mask & CAM_PHASE_SEND) p.epochs[1] = ep_send;
        if (p.phase_mask & CAM_PHASE_RECV) p.epochs[2] = ep_recv;
        // a deferred push has no receive phase of its own: keep the three counters in step for the next plain dispatch
        if (p.defer_push && (p.phase_mask & CAM_PHASE_SEND)) p.epochs[2] = ep_send;
    }
}

// ----------------------------------------------------------------------------------------
// Stand-alone layout kernel (the reference's dispatch_layout op,
// ascend_kernels/dispatch_layout/op_kernel/dispatch_layout.h:83-134).  Negative ids are skipped.
// ----------------------------------------------------------------------------------------
__global__ void layout_kernel(const void* topk_idx, int idx_is_i64, int T, int K, int E, int R,
                              int* num_tokens_per_rank, int* num_tokens_per_expert,
                              uint8_t* is_token_in_rank) {
    static_assert(CAM_MAX_RANKS <= 128, "the ranks a token goes to are tracked in two 64-bit masks");
    __shared__ int s_rank[CAM_MAX_RANKS];
    __shared__ int s_exp[CAM_MAX_EXPERTS];
    for (int i = threadIdx.x; i < R; i += blockDim.x) s_rank[i] = 0;
    for (int i = threadIdx.x; i < E; i += blockDim.x) s_exp[i] = 0;
    __syncthreads();
    const int El = E / R;
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x) {
        unsigned long long seen_lo = 0ull, seen_hi = 0ull;  // ranks 0..63 and 64..127
        for (int k = 0; k < K; ++k) {
            const int id = load_expert_id(topk_idx, idx_is_i64, static_cast<size_t>(t) * K + k);
            if (id < 0 || id >= E) continue;
            atomicAdd(&s_exp[id], 1);
            const int r = id / El;
            if (r < 64) seen_lo |= 1ull << r; else seen_hi |= 1ull << (r - 64);
        }
        for (int r = 0; r < R; ++r) {
            const bool in = (r < 64) ? ((seen_lo >> r) & 1ull) : ((seen_hi >> (r - 64)) & 1ull);
            is_token_in_rank[static_cast<size_t>(t) * R + r] = in ? 1 : 0;
            if (in) atomicAdd(&s_rank[r], 1);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < R; i += blockDim.x) if (s_rank[i]) atomicAdd(&num_tokens_per_rank[i], s_rank[i]);
    for (int i = threadIdx.x; i < E; i += blockDim.x) if (s_exp[i]) atomicAdd(&num_tokens_per_expert[i], s_exp[i]);
}

}  // namespace cam

// ----------------------------------------------------------------------------------------
// Launchers (C ABI)
// ----------------------------------------------------------------------------------------
extern "C" int cam_dispatch_normal_smem_bytes(int h, int quant_mode) {
    if (quant_mode == CAM_QUANT_NONE) return 0;
    const int nscale = CAM_QUANT_IS_FP8(quant_mode) ? h / 128 : 1;
    return cam::kDispWarps * ((h + nscale * 4 + 15) & ~15);
}

extern "C" int cam_dispatch_normal_max_grid(int device, int h, int quant_mode) {
    int sms = 0, per_sm = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
    const int smem = cam_dispatch_normal_smem_bytes(h, quant_mode);
    cudaFuncSetAttribute(cam::dispatch_normal_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, cam::dispatch_normal_kernel, cam::kDispThreads,
                                                      smem) != cudaSuccess)
        return -1;
    return sms * (per_sm > 0 ? 1 : 0);
}

extern "C" int cam_launch_dispatch_normal(const cam::DispatchNormalParams* p, int grid, cudaStream_t stream) {
    const int smem = cam_dispatch_normal_smem_bytes(p->h, p->quant_mode);
    static cam::SmemLimitCache limit;
    cudaError_t e = limit.ensure(cam::dispatch_normal_kernel, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    void* args[] = {const_cast<cam::DispatchNormalParams*>(p)};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(cam::dispatch_normal_kernel), dim3(grid),
                                    dim3(cam::kDispThreads), args, smem, stream);
    return static_cast<int>(e);
}

extern "C" int cam_launch_layout(const void* topk_idx, int idx_is_i64, int T, int K, int E, int R,
                                 int* num_tokens_per_rank, int* num_tokens_per_expert,
                                 uint8_t* is_token_in_rank, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = 256;
    int blocks = (T + threads - 1) / threads;
    const int cap = 4 * cam::sm_count_of_current_device();  // the kernel strides over the tokens
    if (blocks > cap) blocks = cap;
    cam::layout_kernel<<<blocks, threads, 0, stream>>>(topk_idx, idx_is_i64, T, K, E, R, num_tokens_per_rank,
                                                       num_tokens_per_expert, is_token_in_rank);
    return static_cast<int>(cudaGetLastError());
}
