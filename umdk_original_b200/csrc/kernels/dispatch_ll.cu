// Low-latency (decode) dispatch for sm_100a.  No count exchange precedes the data: every
// (source rank, local expert) pair owns a fixed slab of `max_tokens` rows in the destination's
// symmetric memory, so a sender knows the address of every row without asking.  One CTA owns one
// expert: it finds that expert's (token, k) pairs in scan order, quantises and pushes each row
// with P2P stores, then publishes {epoch, count} as one 64-bit release store into the
// destination's cell.  The receive phase waits for its cells, packs the slabs into the
// contiguous expert-major / source-minor layout that the grouped GEMM consumes and emits the
// cumulative counts.
//
// Counterpart of the reference's moe_dispatch_shmem kernel
// (ascend_kernels/moe_dispatch_shmem/op_kernel/moe_dispatch_shmem.h: AlltoAllDispatch 551-652,
// SetStatus 655-690, WaitDispatch 736-778, LocalWindowCopy 840-933, UpdateTokenNumsOut
// 1056-1086).  expandIdx keeps the reference meaning: the number of earlier pairs of this rank
// routed to the same expert.  Float flags summed by a vector reduce become one integer cell.
#include "../common/cam_types.h"
#include "../common/ptx.cuh"
#include "../common/quant.cuh"
#include "launch.h"

namespace cam {

constexpr int kLLThreads = 256;
constexpr int kLLWarps = kLLThreads / 32;

__device__ __forceinline__ void ll_record_status(CamStatus* st, int code, int who, int detail) {
    if (atomicCAS(&st->code, 0, code) == 0) {
        st->who = who;
        st->detail = detail;
        st->block = static_cast<int>(blockIdx.x);
    }
}

__device__ __forceinline__ int ll_expert_id(const void* idx, int is_i64, size_t i) {
    return is_i64 ? static_cast<int>(reinterpret_cast<const long long*>(idx)[i])
                  : reinterpret_cast<const int*>(idx)[i];
}

__global__ void __launch_bounds__(kLLThreads, 1) dispatch_ll_kernel(const DispatchLLParams p) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    __shared__ int s_warp_cnt[kLLWarps];
    __shared__ int s_cnt[CAM_MAX_EXPERTS];   // RECV: rows per cell, ordered (local expert, source)
    __shared__ int s_cum[CAM_MAX_EXPERTS];   // RECV: inclusive cumsum in the same order
    __shared__ int s_running;
    __shared__ uint32_t s_abort;

    const int tid = static_cast<int>(threadIdx.x);
    const int warp = tid >> 5;
    const uint32_t lane = lane_id();
    const int nb = static_cast<int>(gridDim.x);
    const int E = p.E, R = p.R, K = p.K, El = p.E / p.R;
    const int npairs = p.T * K;
    const int parity = static_cast<int>(p.epoch & 1u);
    const int nscale = CAM_QUANT_IS_FP8(p.quant_mode) ? (p.h >> 7)
                       : (p.quant_mode == CAM_QUANT_INT8_TOKEN) ? 1 : 0;
    const int row_bytes = (p.quant_mode == CAM_QUANT_NONE) ? p.h * 2 : p.h;
    const size_t cell_rows = static_cast<size_t>(p.max_tokens);
    // dynamic smem: ids [npairs] | list [npairs] | per-warp staging
    int* s_ids = reinterpret_cast<int*>(dyn_smem);
    int* s_list = s_ids + npairs;
    const int stage_bytes = (p.quant_mode == CAM_QUANT_NONE) ? 0 : ((p.h + nscale * 4 + 15) & ~15);
    uint8_t* stage0 = dyn_smem + ((static_cast<size_t>(npairs) * 8 + 15) & ~static_cast<size_t>(15));
    uint8_t* stage_q = stage0 + static_cast<size_t>(warp) * stage_bytes;
    float* stage_s = reinterpret_cast<float*>(stage_q + p.h);

    if (tid == 0) s_abort = 0u;

    // ------------------------------------------------------------------ SEND
    if (p.phase_mask & CAM_PHASE_SEND) {
        for (int i = tid; i < npairs; i += kLLThreads) {
            int id = ll_expert_id(p.expert_ids, p.idx_is_i64, i);
            if (id < 0 || id >= E || (i / K) >= p.active_tokens) id = -1;
            s_ids[i] = id;
            if (id < 0 && blockIdx.x == 0) p.expand_idx[i] = -1;
        }
        __syncthreads();
        for (int e = static_cast<int>(blockIdx.x); e < E; e += nb) {
            // ordered compaction of the pairs routed to expert e
            if (tid == 0) s_running = 0;
            __syncthreads();
            for (int sub = 0; sub < npairs; sub += kLLThreads) {
                const int i = sub + tid;
                const bool hit = (i < npairs) && (s_ids[i] == e);
                const uint32_t m = __ballot_sync(0xFFFFFFFFu, hit);
                if (lane == 0) s_warp_cnt[warp] = __popc(m);
                __syncthreads();
                int before = s_running;
                for (int w2 = 0; w2 < warp; ++w2) before += s_warp_cnt[w2];
                if (hit) {
                    const int pos = before + __popc(m & ((1u << lane) - 1u));
                    s_list[pos] = i;
                    p.expand_idx[i] = pos;
                }
                __syncthreads();
                if (tid == 0) {
                    int tot = 0;
                    for (int w2 = 0; w2 < kLLWarps; ++w2) tot += s_warp_cnt[w2];
                    s_running += tot;
                }
                __syncthreads();
            }
            int cnt = s_running;
            if (cnt > p.max_tokens) {
                if (tid == 0) ll_record_status(p.status, CAM_ERR_RECV_OVERFLOW, e, cnt);
                cnt = p.max_tokens;
            }
            const int d = e / El, le = e - d * El;
            const size_t cell = static_cast<size_t>(parity) * E + static_cast<size_t>(p.rank) * El + le;
            uint8_t* pb = p.peer_base[d];
            for (int j = warp; j < cnt; j += kLLWarps) {
                const int pair = s_list[j];
                const int t = pair / K, k = pair - t * K;
                const __nv_bfloat16* xrow = p.x + static_cast<size_t>(t) * p.h;
                uint8_t* dst = pb + p.off_ll_x + (cell * cell_rows + j) * static_cast<size_t>(row_bytes);
                if (p.quant_mode == CAM_QUANT_NONE) {
                    const uint8_t* src = reinterpret_cast<const uint8_t*>(xrow);
                    for (int o = static_cast<int>(lane) * 16; o < row_bytes; o += 512)
                        st_na_v4(dst + o, ld_nc_v4(src + o));
                } else {
                    if (p.quant_mode == CAM_QUANT_FP8_1x128)
                        warp_quant_fp8_1x128<false>(xrow, p.h, stage_q, stage_s);
                    else if (p.quant_mode == CAM_QUANT_FP8_1x128_UE8M0)
                        warp_quant_fp8_1x128<true>(xrow, p.h, stage_q, stage_s);
                    else
                        warp_quant_int8_token(xrow, p.h, stage_q, stage_s,
                                              p.smooth ? p.smooth + static_cast<size_t>(e) * p.h : nullptr);
                    __syncwarp();
                    for (int o = static_cast<int>(lane) * 16; o < row_bytes; o += 512)
                        st_na_v4(dst + o, *reinterpret_cast<const uint4*>(stage_q + o));
                    float* sdst = reinterpret_cast<float*>(pb + p.off_ll_scales) + (cell * cell_rows + j) * nscale;
                    for (int o = static_cast<int>(lane); o < nscale; o += 32) sdst[o] = stage_s[o];
                    __syncwarp();
                }
                if (lane < 2) {
                    int* m = reinterpret_cast<int*>(pb + p.off_ll_meta) + (cell * cell_rows + j) * 2;
                    m[lane] = (lane == 0) ? t : k;
                }
            }
            __syncthreads();
            if (tid == 0 && p.dbg_drop_flags == 0) {
                __threadfence_system();
                st_release_sys_u64(reinterpret_cast<uint64_t*>(pb + p.off_ll_cells) + cell,
                                   (static_cast<uint64_t>(p.epoch) << 32) | static_cast<uint32_t>(cnt));
            }
            __syncthreads();
        }
    }

    // ------------------------------------------------------------------ RECV
    if (p.phase_mask & CAM_PHASE_RECV) {
        uint8_t* const my_base = p.peer_base[p.rank];
        const uint64_t* cells = reinterpret_cast<const uint64_t*>(my_base + p.off_ll_cells) +
                                static_cast<size_t>(parity) * E;
        for (int o = tid; o < E; o += kLLThreads) {  // o = le * R + src
            const int le = o / R, src = o - le * R;
            const uint64_t* c = cells + static_cast<size_t>(src) * El + le;
            uint64_t v = ld_acquire_sys_u64(c);
            if (static_cast<uint32_t>(v >> 32) != p.epoch) {
                const uint64_t t0 = globaltimer_ns();
                uint32_t spins = 0;
                while (true) {
                    v = ld_acquire_sys_u64(c);
                    if (static_cast<uint32_t>(v >> 32) == p.epoch) break;
                    if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > p.timeout_ns) {
                        ll_record_status(p.status, CAM_ERR_TIMEOUT_LL_CELL, src, le);
                        s_abort = 1u;
                        break;
                    }
                }
            }
            s_cnt[o] = static_cast<int>(static_cast<uint32_t>(v));
        }
        __syncthreads();
        if (s_abort) return;
        if (warp == 0) {  // inclusive scan of s_cnt in (local expert, source) order
            const int per = (E + 31) / 32;
            const int lo = static_cast<int>(lane) * per, hi = min(E, lo + per);
            int sum = 0;
            for (int o = lo; o < hi; ++o) sum += s_cnt[o];
            int incl = sum;
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                const int n = __shfl_up_sync(0xFFFFFFFFu, incl, s);
                if (static_cast<int>(lane) >= s) incl += n;
            }
            int run = incl - sum;
            for (int o = lo; o < hi; ++o) { run += s_cnt[o]; s_cum[o] = run; }
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
        // pack the slabs into the contiguous output
        for (int o = static_cast<int>(blockIdx.x); o < E; o += nb) {
            const int le = o / R, src = o - le * R;
            const int n = s_cnt[o];
            const int start = s_cum[o] - n;
            const size_t cell = static_cast<size_t>(parity) * E + static_cast<size_t>(src) * El + le;
            const uint8_t* sx = my_base + p.off_ll_x + cell * cell_rows * row_bytes;
            const float* ss = reinterpret_cast<const float*>(my_base + p.off_ll_scales) + cell * cell_rows * nscale;
            const int* sm = reinterpret_cast<const int*>(my_base + p.off_ll_meta) + cell * cell_rows * 2;
            for (int j = warp; j < n; j += kLLWarps) {
                const uint8_t* s = sx + static_cast<size_t>(j) * row_bytes;
                uint8_t* dx = p.expand_x + static_cast<size_t>(start + j) * row_bytes;
                for (int b = static_cast<int>(lane) * 16; b < row_bytes; b += 512) st_na_v4(dx + b, ld_cg_v4(s + b));
                for (int b = static_cast<int>(lane); b < nscale; b += 32)
                    p.expand_scales[static_cast<size_t>(start + j) * nscale + b] =
                        __ldcg(ss + static_cast<size_t>(j) * nscale + b);
                if (lane < 3) {
                    const int v = (lane == 0) ? src : __ldcg(sm + static_cast<size_t>(j) * 2 + (lane - 1));
                    p.expand_src[static_cast<size_t>(start + j) * 3 + lane] = v;
                }
            }
        }
    }
}

}  // namespace cam

extern "C" int cam_dispatch_ll_smem_bytes(int h, int quant_mode, int T, int K) {
    const int nscale = CAM_QUANT_IS_FP8(quant_mode) ? h / 128 : (quant_mode == CAM_QUANT_INT8_TOKEN) ? 1 : 0;
    const int stage = (quant_mode == CAM_QUANT_NONE) ? 0 : ((h + nscale * 4 + 15) & ~15);
    return ((T * K * 8 + 15) & ~15) + cam::kLLWarps * stage;
}

extern "C" int cam_dispatch_ll_max_grid(int device, int h, int quant_mode, int T, int K) {
    int sms = 0, per_sm = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
    const int smem = cam_dispatch_ll_smem_bytes(h, quant_mode, T, K);
    cudaFuncSetAttribute(cam::dispatch_ll_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, cam::dispatch_ll_kernel, cam::kLLThreads, smem) !=
        cudaSuccess)
        return -1;
    return sms * per_sm;
}

extern "C" int cam_launch_dispatch_ll(const cam::DispatchLLParams* p, int grid, cudaStream_t stream) {
    const int smem = cam_dispatch_ll_smem_bytes(p->h, p->quant_mode, p->T, p->K);
    cudaError_t e = cudaFuncSetAttribute(cam::dispatch_ll_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    void* args[] = {const_cast<cam::DispatchLLParams*>(p)};
    return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(cam::dispatch_ll_kernel), dim3(grid),
                                                        dim3(cam::kLLThreads), args, smem, stream));
}
