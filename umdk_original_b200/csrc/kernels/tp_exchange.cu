// Tensor-parallel pair exchange for the low-latency ops (tpWorldSize = 2): the two TP ranks that sit
// at the same expert-parallel position hold differently sharded expert weights, so after dispatch
// each needs the other's received tokens as well (all-gather), and before combine each returns the
// partial outputs it computed for the other's tokens and adds what comes back (reduce-scatter).
//
// Counterpart of the TP branches of the reference's shmem kernels
// (moe_dispatch_shmem.h:936-1018 AllGatherSetStatusAndWait / AllgatherProcessOut and
// moe_combine_shmem.h:438-470, 594-620 ReduceScatterTrans): rows are pushed into a region of the
// partner's symmetric buffer, a count and an epoch flag follow, the partner copies or adds.
#include "../common/cam_types.h"
#include "../common/ptx.cuh"
#include "../common/quant.cuh"
#include "launch.h"

namespace cam {

constexpr int kTpThreads = 512;
constexpr int kTpWarps = kTpThreads / 32;

__global__ void __launch_bounds__(kTpThreads, 1) tp_exchange_kernel(const TpExchangeParams p) {
    __shared__ uint32_t s_abort;
    const int tid = static_cast<int>(threadIdx.x);
    const int warp = tid >> 5;
    const uint32_t lane = lane_id();
    const int nb = static_cast<int>(gridDim.x);
    const int gwarp = static_cast<int>(blockIdx.x) * kTpWarps + warp;
    const int nwarps = nb * kTpWarps;
    const uint32_t ep_send = p.epochs[0] + 1u, ep_recv = p.epochs[1] + 1u;
    if (tid == 0) s_abort = 0u;
    __syncthreads();

    if (p.phase_mask & CAM_PHASE_SEND) {
        // all-gather: my own rows [0, n_own); reduce-scatter: the partner's rows [n_own, n_own + n_peer)
        const int n_own = min(p.n_own[0], p.max_rows);
        const int first = p.reduce ? n_own : 0;
        const int count = p.reduce ? min(p.n_peer[0], p.max_rows) : n_own;
        uint8_t* dst_rows = p.peer_base + p.off_tp_x;
        for (int i = gwarp; i < count; i += nwarps) {
            warp_copy_row<false>(dst_rows + static_cast<size_t>(i) * p.row_bytes,
                                 p.rows + static_cast<size_t>(first + i) * p.row_bytes, p.row_bytes, lane);
            if (p.scales != nullptr) {
                float* sd = reinterpret_cast<float*>(p.peer_base + p.off_tp_scales) + static_cast<size_t>(i) * p.nscale;
                for (int o = static_cast<int>(lane); o < p.nscale; o += 32)
                    sd[o] = p.scales[static_cast<size_t>(first + i) * p.nscale + o];
            }
        }
        __syncthreads();
        if (tid == 0) {
            __threadfence_system();
            const unsigned int old = atomicAdd(p.done_ctr, 1u);
            if (old == static_cast<unsigned int>(nb - 1)) {
                p.done_ctr[0] = 0u;
                __threadfence_system();
                reinterpret_cast<uint32_t*>(p.peer_base + p.off_tp_cnt)[p.reduce] = static_cast<uint32_t>(count);
                __threadfence_system();
                if (p.dbg_drop_flags == 0)
                    st_release_sys_u32(reinterpret_cast<uint32_t*>(p.peer_base + p.off_tp_flag) + p.reduce, ep_send);
            }
        }
    }

    if (p.phase_mask & CAM_PHASE_RECV) {
        if (tid == 0) {
            const uint32_t* f = reinterpret_cast<const uint32_t*>(p.my_base + p.off_tp_flag) + p.reduce;
            if (!wait_flag_eq_sys(f, ep_recv, p.timeout_ns)) {
                if (atomicCAS(&p.status->code, 0, CAM_ERR_TIMEOUT_BARRIER) == 0) {
                    p.status->who = p.tp_rank ^ 1;
                    p.status->detail = static_cast<int>(ld_acquire_sys_u32(f));
                    p.status->block = static_cast<int>(blockIdx.x);
                }
                s_abort = 1u;
            }
        }
        __syncthreads();
        if (!s_abort) {
            const int got = static_cast<int>(min(__ldcg(reinterpret_cast<const uint32_t*>(p.my_base + p.off_tp_cnt) + p.reduce),
                                                 static_cast<uint32_t>(p.max_rows)));
            const int n_own = min(p.n_own[0], p.max_rows);
            const uint8_t* src_rows = p.my_base + p.off_tp_x;
            if (!p.reduce) {
                // append the partner's rows after my own
                for (int i = gwarp; i < got; i += nwarps) {
                    if (n_own + i >= p.out_rows) break;
                    warp_copy_row<true>(p.out + static_cast<size_t>(n_own + i) * p.row_bytes,
                                        src_rows + static_cast<size_t>(i) * p.row_bytes, p.row_bytes, lane);
                    if (p.scales_out != nullptr) {
                        const float* ss = reinterpret_cast<const float*>(p.my_base + p.off_tp_scales) + static_cast<size_t>(i) * p.nscale;
                        for (int o = static_cast<int>(lane); o < p.nscale; o += 32)
                            p.scales_out[static_cast<size_t>(n_own + i) * p.nscale + o] = __ldcg(ss + o);
                    }
                }
                if (blockIdx.x == 0 && tid == 0) {
                    p.tp_counts[p.tp_rank] = n_own;
                    p.tp_counts[p.tp_rank ^ 1] = got;
                }
            } else {
                // out[i] = my partial + the partner's partial for my rows (bf16, fp32 add, round to nearest)
                const int n = min(n_own, got);
                for (int i = gwarp; i < n_own; i += nwarps) {
                    const uint8_t* a = p.rows + static_cast<size_t>(i) * p.row_bytes;
                    const uint8_t* b2 = src_rows + static_cast<size_t>(i) * p.row_bytes;
                    uint8_t* o8 = p.out + static_cast<size_t>(i) * p.row_bytes;
                    for (int o = static_cast<int>(lane) * 16; o < p.row_bytes; o += 512) {
                        const uint4 va = ld_nc_v4(a + o);
                        if (i >= n) { st_na_v4(o8 + o, va); continue; }
                        const uint4 vb = ld_cg_v4(b2 + o);
                        const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
                        uint32_t r[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            __nv_bfloat162 t = __floats2bfloat162_rn(bf16_lo(wa[j]) + bf16_lo(wb[j]), bf16_hi(wa[j]) + bf16_hi(wb[j]));
                            r[j] = *reinterpret_cast<uint32_t*>(&t);
                        }
                        st_na_v4(o8 + o, make_uint4(r[0], r[1], r[2], r[3]));
                    }
                }
            }
        }
    }

    __syncthreads();
    if (tid == 0 && last_cta_out(p.exit_ctr, static_cast<unsigned int>(nb))) {
        if (p.phase_mask & CAM_PHASE_SEND) p.epochs[0] = ep_send;
        if (p.phase_mask & CAM_PHASE_RECV) p.epochs[1] = ep_recv;
    }
}

}  // namespace cam

extern "C" int cam_launch_tp_exchange(const cam::TpExchangeParams* p, int grid, cudaStream_t stream) {
    void* args[] = {const_cast<cam::TpExchangeParams*>(p)};
    return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(cam::tp_exchange_kernel), dim3(grid),
                                                        dim3(cam::kTpThreads), args, 0, stream));
}
