// Combine for sm_100a: every expert-output row is pushed with P2P stores into the (token, k)
// slot of its origin rank, a per-source completion flag follows, and the origin fuses the
// top-k weighted sum in fp32 (k order) with a round-to-nearest bf16 store.
//
// Same data flow as the reference's moe_combine_normal
// (ascend_kernels/moe_combine_normal/op_kernel/moe_combine_normal.h:211-374) and, with the row
// table that low-latency dispatch keeps, as moe_combine_shmem (moe_combine_shmem.h:919-930);
// the per-(token,k) float flags summed by a vector reduce become one integer epoch flag per
// source rank, raised once by the last CTA of the sender.  Pairs whose expert id is negative
// are skipped instead of waited for.
//
// comm_quant = 2 sends a row as int8 with one fp32 scale per 128 elements (h + h/32 bytes instead
// of 2 h) and dequantises inside the reduce: the counterpart of the reference's commQuantMode 2
// (moe_combine_shmem.h:567-591 quantises per 8 elements; 128 keeps the scales at 3 % of the row).
#include "../common/cam_types.h"
#include "../common/ptx.cuh"
#include "../common/quant.cuh"
#include "launch.h"

namespace cam {

constexpr int kCombThreads = 512;
constexpr int kCombWarps = kCombThreads / 32;

__device__ __forceinline__ void comb_record_status(CamStatus* st, int code, int who, int detail) {
    if (atomicCAS(&st->code, 0, code) == 0) {
        st->who = who;
        st->detail = detail;
        st->block = static_cast<int>(blockIdx.x);
    }
}

__device__ __forceinline__ void fma_bf16x8(float (&acc)[8], const uint4& v, float w) {
    acc[0] = fmaf(w, bf16_lo(v.x), acc[0]);
    acc[1] = fmaf(w, bf16_hi(v.x), acc[1]);
    acc[2] = fmaf(w, bf16_lo(v.y), acc[2]);
    acc[3] = fmaf(w, bf16_hi(v.y), acc[3]);
    acc[4] = fmaf(w, bf16_lo(v.z), acc[4]);
    acc[5] = fmaf(w, bf16_hi(v.z), acc[5]);
    acc[6] = fmaf(w, bf16_lo(v.w), acc[6]);
    acc[7] = fmaf(w, bf16_hi(v.w), acc[7]);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
}

__global__ void __launch_bounds__(kCombThreads, 1) combine_kernel(const CombineParams p) {
    __shared__ uint32_t s_abort;
    __shared__ float s_w[kCombWarps][CAM_MAX_TOPK];
    const int tid = static_cast<int>(threadIdx.x);
    const int warp = tid >> 5;
    const uint32_t lane = lane_id();
    const int nb = static_cast<int>(gridDim.x);
    const int gwarp = static_cast<int>(blockIdx.x) * kCombWarps + warp;
    const int nwarps = nb * kCombWarps;
    const int row_bytes = p.h * 2;
    const uint32_t ep_send = p.epochs[0] + 1u, ep_recv = p.epochs[1] + 1u;
    if (tid == 0) s_abort = 0u;
    __syncthreads();

    trace_point(p.trace, 0);  // kernel start
    // ------------------------------------------------------------------ SEND
    if (p.phase_mask & CAM_PHASE_SEND) {
        const int n = p.total_rows[0];
        // Rows are ordered by expert and, inside an expert, by origin rank.  Every rank starts its walk somewhere else
        // (its share of the rows plus one grid-wide step per rank further on), so that at any one time the ranks of the
        // group push to different origins instead of all filling the same GPU's ingress.
        const int shift = (p.R > 1 && n > 0) ? static_cast<int>((static_cast<long long>(p.rank) * (n / p.R + nwarps)) % n) : 0;
        for (int i0 = gwarp; i0 < n; i0 += nwarps) {
            const int i = (i0 + shift < n) ? i0 + shift : i0 + shift - n;
            const int src = p.row_src[static_cast<size_t>(i) * 3 + 0];
            const int t = p.row_src[static_cast<size_t>(i) * 3 + 1];
            const int k = p.row_src[static_cast<size_t>(i) * 3 + 2];
            if (src < 0 || src >= p.R || t < 0 || t >= p.max_tokens || k < 0 || k >= p.K) {
                // never store out of range: the row is dropped and the status word says which one it was
                if (lane == 0) comb_record_status(p.status, CAM_ERR_BAD_INDEX, 1, i);
                continue;
            }
            const uint8_t* s = reinterpret_cast<const uint8_t*>(p.y) + static_cast<size_t>(i) * row_bytes;
            uint8_t* d = p.peer_base[src] + p.off_combine_buf +
                         (static_cast<size_t>(t) * p.K + k) * static_cast<size_t>(row_bytes);
            if (p.comm_quant == 2) {
                // int8 on the wire: lane owns 8 elements per step of 256, 16 lanes share a 128-element block
                float* dscale = reinterpret_cast<float*>(d + p.h);
                for (int base = 0; base < p.h; base += 1024) {
                    uint4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int c = base + u * 256 + static_cast<int>(lane) * 8;
                        v[u] = (c < p.h) ? ld_nc_v4(s + static_cast<size_t>(c) * 2) : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int c = base + u * 256 + static_cast<int>(lane) * 8;
                        float f[8] = {bf16_lo(v[u].x), bf16_hi(v[u].x), bf16_lo(v[u].y), bf16_hi(v[u].y),
                                      bf16_lo(v[u].z), bf16_hi(v[u].z), bf16_lo(v[u].w), bf16_hi(v[u].w)};
                        float amax = 0.f;
#pragma unroll
                        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
#pragma unroll
                        for (int sft = 8; sft >= 1; sft >>= 1)
                            amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, sft));
                        const float a = fmaxf(amax, 1e-12f);
                        const float inv = 127.f / a;
                        uint32_t w0 = 0u, w1 = 0u;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            w0 |= (static_cast<uint32_t>(__float2int_rn(f[j] * inv)) & 0xFFu) << (8 * j);
                            w1 |= (static_cast<uint32_t>(__float2int_rn(f[4 + j] * inv)) & 0xFFu) << (8 * j);
                        }
                        if (c < p.h) {
                            st_na_v2(d + c, make_uint2(w0, w1));
                            if ((lane & 15u) == 0u) dscale[c >> 7] = a / 127.f;
                        }
                    }
                }
                continue;
            }
            int o = static_cast<int>(lane) * 16;
            for (; o + 3 * 512 < row_bytes; o += 4 * 512) {
                const uint4 a = ld_nc_v4(s + o), b4 = ld_nc_v4(s + o + 512), c = ld_nc_v4(s + o + 1024),
                            e = ld_nc_v4(s + o + 1536);
                st_na_v4(d + o, a);
                st_na_v4(d + o + 512, b4);
                st_na_v4(d + o + 1024, c);
                st_na_v4(d + o + 1536, e);
            }
            for (; o < row_bytes; o += 512) st_na_v4(d + o, ld_nc_v4(s + o));
        }
        __syncthreads();
        trace_point(p.trace, 1);  // this CTA's rows are issued
        if (tid == 0) {
            __threadfence_system();
            if (p.trace != nullptr && blockIdx.x == 0) p.trace[2] = globaltimer_ns();  // system fence done
            const unsigned int old = atomicAdd(p.done_ctr, 1u);
            if (old == static_cast<unsigned int>(nb - 1)) {
                p.done_ctr[0] = 0u;
                __threadfence_system();
                if (p.dbg_drop_flags == 0) {
                    for (int d = 0; d < p.R; ++d)
                        st_release_sys_u32(
                            reinterpret_cast<uint32_t*>(p.peer_base[d] + p.off_combine_flag) + p.rank, ep_send);
                }
            }
        }
    }

    // ------------------------------------------------------------------ RECV
    if (p.phase_mask & CAM_PHASE_RECV) {
        uint8_t* const my_base = p.peer_base[p.rank];
        if (tid < p.R) {
            const uint32_t* f = reinterpret_cast<const uint32_t*>(my_base + p.off_combine_flag) + tid;
            const bool keep = blockIdx.x == 0 && p.stats != nullptr;
            const uint64_t t_wait = keep ? globaltimer_ns() : 0ull;
            if (!wait_flag_eq_sys(f, ep_recv, p.timeout_ns)) {
                comb_record_status(p.status, CAM_ERR_TIMEOUT_COMBINE_FLAG, tid,
                                   static_cast<int>(ld_acquire_sys_u32(f)));
                s_abort = 1u;
            }
            if (keep) {
                atomicMax(&p.stats->max_wait_ns[2][tid], globaltimer_ns() - t_wait);
                if (tid == 0) atomicAdd(&p.stats->calls[1], 1ull);
            }
        }
        __syncthreads();
        trace_point(p.trace, 3);  // all sources' flags have arrived
        if (s_abort) goto done;

        const uint8_t* buf = my_base + p.off_combine_buf;
        if (p.comm_quant == 2) {
            // rows arrived as int8 + one scale per 128 elements; a lane reduces 16 elements per step
            const int chunks_q = (p.h + 511) / 512;
            const int nsplit_q = min(chunks_q, max(1, nwarps / max(p.T, 1)));
            const int per_q = (chunks_q + nsplit_q - 1) / nsplit_q;
            for (int it = gwarp; it < p.T * nsplit_q; it += nwarps) {
                const int t = it / nsplit_q;
                const int e_begin = (it - t * nsplit_q) * per_q * 512;
                const int e_end = min(p.h, e_begin + per_q * 512);
                bool pair_ok = false;
                if (lane < static_cast<uint32_t>(p.K)) {
                    const int id = load_expert_id(p.topk_idx, p.idx_is_i64, static_cast<size_t>(t) * p.K + lane);
                    s_w[warp][lane] = p.topk_weights[static_cast<size_t>(t) * p.K + lane];
                    pair_ok = (id >= 0 && id < p.E);
                }
                const uint32_t valid = __ballot_sync(0xFFFFFFFFu, pair_ok);
                __syncwarp();
                const uint8_t* trow = buf + static_cast<size_t>(t) * p.K * row_bytes;
                uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) + static_cast<size_t>(t) * row_bytes;
                for (int c = e_begin + static_cast<int>(lane) * 16; c < e_end; c += 512) {
                    float acc[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[j] = 0.f;
                    for (int k = 0; k < p.K; ++k) {
                        if (!((valid >> k) & 1u)) continue;
                        const uint8_t* krow = trow + static_cast<size_t>(k) * row_bytes;
                        const uint4 q = ld_cg_v4(krow + c);
                        const float sc = __ldcg(reinterpret_cast<const float*>(krow + p.h) + (c >> 7)) * s_w[warp][k];
                        const uint32_t wq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int b8 = static_cast<int>(static_cast<int8_t>((wq[j >> 2] >> (8 * (j & 3))) & 0xFFu));
                            acc[j] = fmaf(sc, static_cast<float>(b8), acc[j]);
                        }
                    }
                    uint4 r0, r1;
                    r0.x = pack_bf16x2(acc[0], acc[1]);   r0.y = pack_bf16x2(acc[2], acc[3]);
                    r0.z = pack_bf16x2(acc[4], acc[5]);   r0.w = pack_bf16x2(acc[6], acc[7]);
                    r1.x = pack_bf16x2(acc[8], acc[9]);   r1.y = pack_bf16x2(acc[10], acc[11]);
                    r1.z = pack_bf16x2(acc[12], acc[13]); r1.w = pack_bf16x2(acc[14], acc[15]);
                    st_na_v4(orow + static_cast<size_t>(c) * 2, r0);
                    st_na_v4(orow + static_cast<size_t>(c) * 2 + 16, r1);
                }
                __syncwarp();
            }
            goto done;
        }
        // Work item = (token, slice of the row).  With few tokens (decode) a row is cut into as many
        // 512-byte-aligned slices as there are warps to spare, so the whole grid takes part.
        const int chunks = (row_bytes + 511) / 512;
        const int nsplit = min(chunks, max(1, nwarps / max(p.T, 1)));
        const int per = (chunks + nsplit - 1) / nsplit;
        for (int it = gwarp; it < p.T * nsplit; it += nwarps) {
            const int t = it / nsplit;
            const int o_begin = (it - t * nsplit) * per * 512;
            const int o_end = min(row_bytes, o_begin + per * 512);
            bool pair_ok = false;
            if (lane < static_cast<uint32_t>(p.K)) {
                const int id = load_expert_id(p.topk_idx, p.idx_is_i64, static_cast<size_t>(t) * p.K + lane);
                s_w[warp][lane] = p.topk_weights[static_cast<size_t>(t) * p.K + lane];
                pair_ok = (id >= 0 && id < p.E);
            }
            const uint32_t valid = __ballot_sync(0xFFFFFFFFu, pair_ok);  // bit k: pair (t, k) has a row
            __syncwarp();
            const uint8_t* trow = buf + static_cast<size_t>(t) * p.K * row_bytes;
            uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) + static_cast<size_t>(t) * row_bytes;
            for (int o = o_begin + static_cast<int>(lane) * 16; o < o_end; o += 512) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int k0 = 0; k0 < p.K; k0 += 8) {
                    uint4 v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int k = k0 + j;
                        const bool ok = (k < p.K) && ((valid >> k) & 1u);
                        v[j] = ok ? ld_cg_v4(trow + static_cast<size_t>(k) * row_bytes + o) : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int k = k0 + j;
                        if (k < p.K && ((valid >> k) & 1u)) fma_bf16x8(acc, v[j], s_w[warp][k]);
                    }
                }
                uint4 r;
                r.x = pack_bf16x2(acc[0], acc[1]);
                r.y = pack_bf16x2(acc[2], acc[3]);
                r.z = pack_bf16x2(acc[4], acc[5]);
                r.w = pack_bf16x2(acc[6], acc[7]);
                st_na_v4(orow + o, r);
            }
            __syncwarp();
        }
    }

done:
    __syncthreads();
    trace_point(p.trace, 4);  // CTA 0 reduced its tokens
    if (tid == 0 && last_cta_out(p.exit_ctr, static_cast<unsigned int>(nb))) {
        if (p.trace != nullptr) p.trace[5] = globaltimer_ns();  // the last CTA leaves
        if (p.phase_mask & CAM_PHASE_SEND) p.epochs[0] = ep_send;
        if (p.phase_mask & CAM_PHASE_RECV) p.epochs[1] = ep_recv;
    }
}

}  // namespace cam

extern "C" int cam_combine_max_grid(int device) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
    return sms;
}

extern "C" int cam_launch_combine(const cam::CombineParams* p, int grid, cudaStream_t stream) {
    void* args[] = {const_cast<cam::CombineParams*>(p)};
    return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(cam::combine_kernel), dim3(grid),
                                                        dim3(cam::kCombThreads), args, 0, stream));
}
