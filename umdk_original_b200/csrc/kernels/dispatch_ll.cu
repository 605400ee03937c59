// Low-latency (decode) dispatch for sm_100a.  No count exchange precedes the data: every
// (source rank, local expert) pair owns a fixed slab of `max_tokens` rows in the destination's
// symmetric memory, so a sender knows the address of every row without asking.
//
// SEND  every CTA computes the slot of each (token, k) pair inside its expert (scan order) in
//       shared memory; then the pairs are spread over ALL warps of the grid, one row per warp at a
//       time, so a hot expert does not serialise on one CTA: quantise, push the row, its scales
//       and its (token, k) with P2P stores.  After a grid-wide barrier {epoch, count} goes out as
//       one 64-bit release store per (destination, local expert) cell.
// RECV  wait for the cells of all sources, prefix-sum the counts, and pack the slabs into the
//       contiguous expert-major / source-minor layout that the grouped GEMM consumes, again one
//       row per warp over the whole grid.
//
// Counterpart of the reference's moe_dispatch_shmem kernel
// (ascend_kernels/moe_dispatch_shmem/op_kernel/moe_dispatch_shmem.h: AlltoAllDispatch 551-652,
// SetStatus 655-690, WaitDispatch 736-778, LocalWindowCopy 840-933, UpdateTokenNumsOut
// 1056-1086).  expandIdx keeps the reference meaning: the number of earlier pairs of this rank
// routed to the same expert.  Float flags summed by a vector reduce become one integer cell.
#include <cooperative_groups.h>
#include "../common/cam_types.h"
#include "../common/ptx.cuh"
#include "../common/quant.cuh"
#include "launch.h"

namespace cg = cooperative_groups;

namespace cam {

constexpr int kLLThreads = 512;
constexpr int kLLWarps = kLLThreads / 32;

__device__ __forceinline__ void ll_record_status(CamStatus* st, int code, int who, int detail) {
    if (atomicCAS(&st->code, 0, code) == 0) {
        st->who = who;
        st->detail = detail;
        st->block = static_cast<int>(blockIdx.x);
    }
}

__global__ void __launch_bounds__(kLLThreads, 1) dispatch_ll_kernel(const DispatchLLParams p) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    __shared__ int s_run[CAM_MAX_EXPERTS];   // SEND: pairs per expert / RECV: rows per cell (local expert, source)
    __shared__ int s_cum[CAM_MAX_EXPERTS];   // RECV: inclusive cumsum in the same order
    __shared__ uint32_t s_abort;

    const int tid = static_cast<int>(threadIdx.x);
    const int warp = tid >> 5;
    const uint32_t lane = lane_id();
    const int nb = static_cast<int>(gridDim.x);
    const int gwarp = static_cast<int>(blockIdx.x) * kLLWarps + warp;
    const int nwarps = nb * kLLWarps;
    const int E = p.E, R = p.R, K = p.K, El = p.E / p.R;
    const int npairs = p.T * K;
    const uint32_t ep_send = p.epochs[0] + 1u, ep_recv = p.epochs[1] + 1u;
    const int nscale = CAM_QUANT_IS_FP8(p.quant_mode) ? (p.h >> 7)
                       : (p.quant_mode == CAM_QUANT_INT8_TOKEN) ? 1 : 0;
    const int row_bytes = (p.quant_mode == CAM_QUANT_NONE) ? p.h * 2 : p.h;
    const size_t cell_rows = static_cast<size_t>(p.max_tokens);
    // dynamic smem: ids [npairs] | slots [npairs] | per-warp staging
    int* s_ids = reinterpret_cast<int*>(dyn_smem);
    int* s_slot = s_ids + npairs;
    const int stage_bytes = (p.quant_mode == CAM_QUANT_NONE) ? 0 : ((p.h + nscale * 4 + 15) & ~15);
    uint8_t* stage0 = dyn_smem + ((static_cast<size_t>(npairs) * 8 + 15) & ~static_cast<size_t>(15));
    uint8_t* stage_q = stage0 + static_cast<size_t>(warp) * stage_bytes;
    float* stage_s = reinterpret_cast<float*>(stage_q + p.h);

    if (tid == 0) s_abort = 0u;

    // ------------------------------------------------------------------ SEND
    trace_point(p.trace, 0);  // kernel start
    if (p.phase_mask & CAM_PHASE_SEND) {
        const int parity = static_cast<int>(ep_send & 1u);
        for (int i = tid; i < npairs; i += kLLThreads) {
            int id = load_expert_id(p.expert_ids, p.idx_is_i64, i);
            if (id < 0 || id >= E || (i / K) >= p.active_tokens) id = -1;
            s_ids[i] = id;
        }
        for (int e = tid; e < E; e += kLLThreads) s_run[e] = 0;
        __syncthreads();
        // Slot of every pair inside its expert, in scan order.  Lanes of a 32-pair chunk that share an
        // expert find each other with match.any, which gives the rank inside the chunk and the chunk's
        // count for that expert.  Fast path (the chunk x expert table fits in shared memory): all warps
        // take chunks in parallel, one thread per expert turns the counts into exclusive prefixes over
        // the chunks, and a last pass adds them.  Otherwise one warp walks the chunks in order.
        if (p.slot_table_bytes > 0) {
            uint16_t* tab = reinterpret_cast<uint16_t*>(stage0 + stage_bytes);  // [chunks][E]
            const int nchunks = (npairs + 31) >> 5;
            for (int o = tid * 8; o < nchunks * E; o += kLLThreads * 8)  // table bytes are a multiple of 16
                *reinterpret_cast<uint4*>(tab + o) = make_uint4(0, 0, 0, 0);
            __syncthreads();
            for (int c = warp; c < nchunks; c += kLLWarps) {
                const int i = c * 32 + static_cast<int>(lane);
                const int id = (i < npairs) ? s_ids[i] : -1;
                const uint32_t peers = __match_any_sync(0xFFFFFFFFu, id);
                const int before = __popc(peers & ((1u << lane) - 1u));
                if (id >= 0) {
                    s_slot[i] = before;
                    if (before == 0) tab[c * E + id] = static_cast<uint16_t>(__popc(peers));
                } else if (i < npairs) {
                    s_slot[i] = -1;
                }
            }
            __syncthreads();
            for (int e = tid; e < E; e += kLLThreads) {
                int run = 0;
                for (int c = 0; c < nchunks; ++c) {
                    const int v = tab[c * E + e];
                    tab[c * E + e] = static_cast<uint16_t>(run);
                    run += v;
                }
                s_run[e] = run;
            }
            __syncthreads();
            for (int i = tid; i < npairs; i += kLLThreads) {
                const int id = s_ids[i];
                if (id >= 0) s_slot[i] += tab[(i >> 5) * E + id];
            }
        } else if (warp == 0) {
            for (int c = 0; c < npairs; c += 32) {
                const int i = c + static_cast<int>(lane);
                const int id = (i < npairs) ? s_ids[i] : -1;
                const uint32_t peers = __match_any_sync(0xFFFFFFFFu, id);
                if (id >= 0) {
                    const int before = __popc(peers & ((1u << lane) - 1u));
                    s_slot[i] = s_run[id] + before;
                }
                __syncwarp();
                if (id >= 0 && (peers & ((1u << lane) - 1u)) == 0u) s_run[id] += __popc(peers);
                if (id < 0 && i < npairs) s_slot[i] = -1;
                __syncwarp();
            }
        }
        __syncthreads();
        if (blockIdx.x == 0)
            for (int i = tid; i < npairs; i += kLLThreads) p.expand_idx[i] = s_slot[i];
        trace_point(p.trace, 1);  // slot table done

        if (p.quant_mode != CAM_QUANT_INT8_TOKEN) {
            // Token-major: the CTA quantises a token once (all threads load together, so a row costs one
            // memory latency), then its warps push the staged row to the token's K destinations, the row
            // cut into `parts` pieces so that all warps have work.
            const int parts = max(1, kLLWarps / K);
            const int part_bytes = ((row_bytes + parts - 1) / parts + 511) & ~511;
            const int t_end = min(p.T, p.active_tokens);
            for (int t = static_cast<int>(blockIdx.x); t < t_end; t += nb) {
                const __nv_bfloat16* xrow = p.x + static_cast<size_t>(t) * p.h;
                if (p.quant_mode == CAM_QUANT_FP8_1x128)
                    block_quant_fp8_1x128<false>(xrow, p.h, stage0, reinterpret_cast<float*>(stage0 + p.h));
                else if (p.quant_mode == CAM_QUANT_FP8_1x128_UE8M0)
                    block_quant_fp8_1x128<true>(xrow, p.h, stage0, reinterpret_cast<float*>(stage0 + p.h));
                __syncthreads();
                for (int item = warp; item < K * parts; item += kLLWarps) {
                    const int k = item / parts, part = item - k * parts;
                    const int i = t * K + k;
                    const int e = s_ids[i];
                    const int j = s_slot[i];
                    if (e < 0 || j >= p.max_tokens) continue;  // skipped pair, or beyond the slab (reported below)
                    const int d = e / El, le = e - d * El;
                    const size_t cell = static_cast<size_t>(parity) * E + static_cast<size_t>(p.rank) * El + le;
                    uint8_t* pb = p.peer_base[d];
                    uint8_t* dst = pb + p.off_ll_x + (cell * cell_rows + j) * static_cast<size_t>(row_bytes);
                    const int b0 = part * part_bytes, b1 = min(row_bytes, b0 + part_bytes);
                    if (p.quant_mode == CAM_QUANT_NONE) {
                        if (b1 > b0)
                            warp_copy_row<false>(dst + b0, reinterpret_cast<const uint8_t*>(xrow) + b0, b1 - b0, lane);
                    } else {
                        for (int o = b0 + static_cast<int>(lane) * 16; o < b1; o += 512)
                            st_na_v4(dst + o, *reinterpret_cast<const uint4*>(stage0 + o));
                        if (part == 0) {
                            const float* ssrc = reinterpret_cast<const float*>(stage0 + p.h);
                            float* sdst = reinterpret_cast<float*>(pb + p.off_ll_scales) + (cell * cell_rows + j) * nscale;
                            for (int o = static_cast<int>(lane); o < nscale; o += 32) sdst[o] = ssrc[o];
                        }
                    }
                    if (part == 0 && lane < 2) {
                        int* m = reinterpret_cast<int*>(pb + p.off_ll_meta) + (cell * cell_rows + j) * 2;
                        m[lane] = (lane == 0) ? t : k;
                    }
                }
                __syncthreads();  // the staged row is overwritten by the next token
            }
        } else {
            // Per-token int8 with an expert-specific smooth scale: the quantised row depends on the
            // destination expert, so every (token, k) pair is quantised by the warp that sends it.
            for (int i = gwarp; i < npairs; i += nwarps) {
                const int e = s_ids[i];
                const int j = s_slot[i];
                if (e < 0 || j >= p.max_tokens) continue;
                const int t = i / K, k = i - t * K;
                const int d = e / El, le = e - d * El;
                const size_t cell = static_cast<size_t>(parity) * E + static_cast<size_t>(p.rank) * El + le;
                uint8_t* pb = p.peer_base[d];
                const __nv_bfloat16* xrow = p.x + static_cast<size_t>(t) * p.h;
                uint8_t* dst = pb + p.off_ll_x + (cell * cell_rows + j) * static_cast<size_t>(row_bytes);
                warp_quant_int8_token(xrow, p.h, stage_q, stage_s,
                                      p.smooth ? p.smooth + static_cast<size_t>(e) * p.h : nullptr);
                __syncwarp();
                for (int o = static_cast<int>(lane) * 16; o < row_bytes; o += 512)
                    st_na_v4(dst + o, *reinterpret_cast<const uint4*>(stage_q + o));
                if (lane == 0)
                    reinterpret_cast<float*>(pb + p.off_ll_scales)[(cell * cell_rows + j) * nscale] = stage_s[0];
                __syncwarp();
                if (lane < 2) {
                    int* m = reinterpret_cast<int*>(pb + p.off_ll_meta) + (cell * cell_rows + j) * 2;
                    m[lane] = (lane == 0) ? t : k;
                }
            }
        }
        trace_point(p.trace, 2);  // this CTA's rows are issued
        // every row of this CTA is visible to every GPU before the barrier: the CTA barrier orders the
        // other threads' stores before thread 0's fence, which is cumulative
        __syncthreads();
        if (tid == 0) __threadfence_system();
        trace_point(p.trace, 3);  // system fence done
        cg::this_grid().sync();
        trace_point(p.trace, 4);  // grid barrier done
        // Every CTA knows every count; CTA b publishes the cells of experts b, b + grid, ...
        for (int e = static_cast<int>(blockIdx.x) * kLLThreads + tid; e < E; e += nb * kLLThreads) {
            int cnt = s_run[e];
            if (cnt > p.max_tokens) {
                ll_record_status(p.status, CAM_ERR_RECV_OVERFLOW, e, cnt);
                cnt = p.max_tokens;
            }
            const int d = e / El, le = e - d * El;
            const size_t cell = static_cast<size_t>(parity) * E + static_cast<size_t>(p.rank) * El + le;
            if (p.dbg_drop_flags == 0)
                st_release_sys_u64(reinterpret_cast<uint64_t*>(p.peer_base[d] + p.off_ll_cells) + cell,
                                   (static_cast<uint64_t>(ep_send) << 32) | static_cast<uint32_t>(cnt));
        }
        __syncthreads();
    }

    // ------------------------------------------------------------------ RECV
    if (p.phase_mask & CAM_PHASE_RECV) {
        const int parity = static_cast<int>(ep_recv & 1u);
        uint8_t* const my_base = p.peer_base[p.rank];
        const uint64_t* cells = reinterpret_cast<const uint64_t*>(my_base + p.off_ll_cells) +
                                static_cast<size_t>(parity) * E;
        for (int o = tid; o < E; o += kLLThreads) {  // o = le * R + src
            const int le = o / R, src = o - le * R;
            const uint64_t* c = cells + static_cast<size_t>(src) * El + le;
            uint64_t v = ld_acquire_sys_u64(c);
            if (static_cast<uint32_t>(v >> 32) != ep_recv) {
                const uint64_t t0 = globaltimer_ns();
                uint32_t spins = 0;
                while (true) {
                    v = ld_acquire_sys_u64(c);
                    if (static_cast<uint32_t>(v >> 32) == ep_recv) break;
                    if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > p.timeout_ns) {
                        ll_record_status(p.status, CAM_ERR_TIMEOUT_LL_CELL, src, le);
                        s_abort = 1u;
                        break;
                    }
                }
            }
            s_run[o] = static_cast<int>(static_cast<uint32_t>(v));
        }
        __syncthreads();
        trace_point(p.trace, 5);  // all cells have arrived
        if (s_abort) goto done;
        if (warp == 0) {  // inclusive scan of the counts in (local expert, source) order
            const int per = (E + 31) / 32;
            const int lo = static_cast<int>(lane) * per, hi = min(E, lo + per);
            int sum = 0;
            for (int o = lo; o < hi; ++o) sum += s_run[o];
            int incl = sum;
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                const int n = __shfl_up_sync(0xFFFFFFFFu, incl, s);
                if (static_cast<int>(lane) >= s) incl += n;
            }
            int run = incl - sum;
            for (int o = lo; o < hi; ++o) { run += s_run[o]; s_cum[o] = run; }
        }
        __syncthreads();
        if (blockIdx.x == 0) {
            for (int o = tid; o < E; o += kLLThreads) p.ep_send_counts[o] = s_cum[o];
            for (int le = tid; le < El; le += kLLThreads) {
                const int end = s_cum[le * R + R - 1];
                const int begin = (le == 0) ? 0 : s_cum[le * R - 1];
                p.expert_token_nums[le] = (p.count_type == 1) ? static_cast<long long>(end - begin)
                                                              : static_cast<long long>(end);
            }
            if (tid == 0) p.total_rows[0] = s_cum[E - 1];
        }
        // pack the slabs into the contiguous output: output row r belongs to the cell o with
        // s_cum[o-1] <= r < s_cum[o]
        const int total = s_cum[E - 1];
        for (int r = gwarp; r < total; r += nwarps) {
            int lo = 0, hi = E - 1;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (s_cum[mid] > r) hi = mid; else lo = mid + 1;
            }
            const int o = lo;
            const int le = o / R, src = o - le * R;
            const int j = r - (s_cum[o] - s_run[o]);
            const size_t cell = static_cast<size_t>(parity) * E + static_cast<size_t>(src) * El + le;
            const uint8_t* s = my_base + p.off_ll_x + (cell * cell_rows + j) * static_cast<size_t>(row_bytes);
            uint8_t* dx = p.expand_x + static_cast<size_t>(r) * row_bytes;
            warp_copy_row<true>(dx, s, row_bytes, lane);
            const float* ss = reinterpret_cast<const float*>(my_base + p.off_ll_scales) + (cell * cell_rows + j) * nscale;
            for (int b = static_cast<int>(lane); b < nscale; b += 32)
                p.expand_scales[static_cast<size_t>(r) * nscale + b] = __ldcg(ss + b);
            if (lane < 3) {
                const int* sm = reinterpret_cast<const int*>(my_base + p.off_ll_meta) + (cell * cell_rows + j) * 2;
                const int v = (lane == 0) ? src : __ldcg(sm + (lane - 1));
                p.expand_src[static_cast<size_t>(r) * 3 + lane] = v;
            }
        }
    }

done:
    __syncthreads();
    trace_point(p.trace, 6);  // CTA 0 packed its rows
    if (tid == 0 && last_cta_out(p.exit_ctr, static_cast<unsigned int>(nb))) {
        if (p.trace != nullptr) p.trace[7] = globaltimer_ns();  // the last CTA leaves
        if (p.phase_mask & CAM_PHASE_SEND) p.epochs[0] = ep_send;
        if (p.phase_mask & CAM_PHASE_RECV) p.epochs[1] = ep_recv;
    }
}

}  // namespace cam

// Bytes of the chunk x expert slot table when it is worth having (0: the kernel walks the chunks with one warp).
extern "C" int cam_dispatch_ll_slot_table_bytes(int T, int K, int E) {
    const long long bytes = (static_cast<long long>((T * K + 31) / 32) * E * 2 + 15) & ~15ll;
    return (T * K > 64 && T * K <= 65535 && bytes <= 64 * 1024) ? static_cast<int>(bytes) : 0;
}

extern "C" int cam_dispatch_ll_smem_bytes(int h, int quant_mode, int T, int K, int E) {
    const int nscale = CAM_QUANT_IS_FP8(quant_mode) ? h / 128 : (quant_mode == CAM_QUANT_INT8_TOKEN) ? 1 : 0;
    const int stage = (quant_mode == CAM_QUANT_NONE) ? 0 : ((h + nscale * 4 + 15) & ~15);
    const int table = cam_dispatch_ll_slot_table_bytes(T, K, E);
    const int per_warp = cam::kLLWarps * stage;          // the int8 path stages one row per warp
    const int shared_row = stage + table;                 // the other paths stage one row per CTA, then the table
    return ((T * K * 8 + 15) & ~15) + (per_warp > shared_row ? per_warp : shared_row);
}

extern "C" int cam_dispatch_ll_max_grid(int device, int h, int quant_mode, int T, int K, int E) {
    int sms = 0, per_sm = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
    const int smem = cam_dispatch_ll_smem_bytes(h, quant_mode, T, K, E);
    cudaFuncSetAttribute(cam::dispatch_ll_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, cam::dispatch_ll_kernel, cam::kLLThreads, smem) !=
        cudaSuccess)
        return -1;
    return sms * per_sm;
}

extern "C" int cam_launch_dispatch_ll(const cam::DispatchLLParams* p, int grid, cudaStream_t stream) {
    const int smem = cam_dispatch_ll_smem_bytes(p->h, p->quant_mode, p->T, p->K, p->E);
    static cam::SmemLimitCache limit;
    cudaError_t e = limit.ensure(cam::dispatch_ll_kernel, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    void* args[] = {const_cast<cam::DispatchLLParams*>(p)};
    return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(cam::dispatch_ll_kernel), dim3(grid),
                                                        dim3(cam::kLLThreads), args, smem, stream));
}
