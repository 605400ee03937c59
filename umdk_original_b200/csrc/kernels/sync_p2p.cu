// Small cross-rank kernels on the symmetric buffer: a device barrier over all ranks of the group and
// the two measurement kernels of the P2P microbenchmark (bulk write to one peer, flag ping-pong).
//
// The barrier plays the part of the reference's SyncCollectives (ascend_kernels/utils/op_kernel/
// sync_collectives.h:26-433: every rank sets a flag in every peer's window and waits for all of its
// own, with a timeout-capable wait at :375-416); flags are epochs, so nothing is reset between uses.
// The microbenchmark covers what urma_perftest measures for one-sided writes (bandwidth and
// latency, src/urma/tools/urma_perftest/perftest_run_test.c:2413-2480) on NVLink peer memory.
#include "../common/cam_types.h"
#include "../common/ptx.cuh"
#include "launch.h"

namespace cam {

// One CTA.  SEND: thread d raises this rank's barrier flag at rank d.  RECV: thread s waits for rank s.
__global__ void barrier_kernel(uint8_t* const* peer_base, uint64_t off_barrier_flag, uint32_t* epochs, int R, int rank,
                               int phase_mask, int dbg_drop_flags, uint64_t timeout_ns, CamStatus* status) {
    const int tid = static_cast<int>(threadIdx.x);
    const uint32_t ep_send = epochs[0] + 1u, ep_recv = epochs[1] + 1u;
    if ((phase_mask & CAM_PHASE_SEND) && tid < R && dbg_drop_flags == 0) {
        __threadfence_system();
        st_release_sys_u32(reinterpret_cast<uint32_t*>(peer_base[tid] + off_barrier_flag) + rank, ep_send);
    }
    if ((phase_mask & CAM_PHASE_RECV) && tid < R) {
        const uint32_t* f = reinterpret_cast<const uint32_t*>(peer_base[rank] + off_barrier_flag) + tid;
        if (!wait_flag_eq_sys(f, ep_recv, timeout_ns) && atomicCAS(&status->code, 0, CAM_ERR_TIMEOUT_BARRIER) == 0) {
            status->who = tid;
            status->detail = static_cast<int>(ld_acquire_sys_u32(f));
            status->block = 0;
        }
    }
    __syncthreads();
    if (tid == 0) {
        if (phase_mask & CAM_PHASE_SEND) epochs[0] = ep_send;
        if (phase_mask & CAM_PHASE_RECV) epochs[1] = ep_recv;
    }
}

// Copies `bytes` (a multiple of 512) from src to dst with the whole grid, 16 bytes per lane per step.
__global__ void p2p_copy_kernel(uint8_t* dst, const uint8_t* src, size_t bytes) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x * 16;
    for (size_t o = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 16; o < bytes; o += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (o + u * stride < bytes) v[u] = ld_nc_v4(src + o + u * stride);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (o + u * stride < bytes) st_na_v4(dst + o + u * stride, v[u]);
    }
}

// Flag ping-pong between two ranks: `iters` round trips; the initiator writes i, the responder
// answers i.  One thread; every wait is bounded.
__global__ void p2p_pingpong_kernel(uint32_t* my_flag, uint32_t* peer_flag, uint32_t base, int iters, int initiator,
                                    uint64_t timeout_ns, CamStatus* status) {
    for (int i = 1; i <= iters; ++i) {
        const uint32_t v = base + static_cast<uint32_t>(i);
        if (initiator) st_release_sys_u32(peer_flag, v);
        if (!wait_flag_eq_sys(my_flag, v, timeout_ns)) {
            if (atomicCAS(&status->code, 0, CAM_ERR_TIMEOUT_BARRIER) == 0) {
                status->who = -1;
                status->detail = i;
                status->block = 0;
            }
            return;
        }
        if (!initiator) st_release_sys_u32(peer_flag, v);
    }
}

}  // namespace cam

extern "C" int cam_launch_barrier(uint8_t* const* peer_base, uint64_t off_barrier_flag, uint32_t* epochs, int R, int rank,
                                  int phase_mask, int dbg_drop_flags, uint64_t timeout_ns, CamStatus* status,
                                  cudaStream_t stream) {
    cam::barrier_kernel<<<1, CAM_MAX_RANKS < 96 ? 96 : CAM_MAX_RANKS, 0, stream>>>(peer_base, off_barrier_flag, epochs, R, rank,
                                                                                phase_mask, dbg_drop_flags, timeout_ns, status);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int cam_launch_p2p_copy(void* dst, const void* src, size_t bytes, int grid, cudaStream_t stream) {
    cam::p2p_copy_kernel<<<grid, 512, 0, stream>>>(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), bytes);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int cam_launch_p2p_pingpong(uint32_t* my_flag, uint32_t* peer_flag, uint32_t base, int iters, int initiator,
                                       uint64_t timeout_ns, CamStatus* status, cudaStream_t stream) {
    cam::p2p_pingpong_kernel<<<1, 1, 0, stream>>>(my_flag, peer_flag, base, iters, initiator, timeout_ns, status);
    return static_cast<int>(cudaGetLastError());
}
