// Grouped (per-expert, ragged-M) int8 x int8 -> int32 GEMM for sm_100a on tcgen05.mma kind::i8: the
// exact W8A8 arithmetic of the reference's fused operator (int8 activations with one dynamic scale
// per token, int8 weights with one scale per output channel, int32 accumulation:
// fused_deep_moe/gemm/kernel/grouped_matmul_slice_m_per_token_dequant_swiglu_quant_multistage_
// workspace.h:558-632 on the cube cores, dequantisation in
// epilogue/block/block_epilogue_per_token_dequant_swiglu.h:236-272 and
// block_epilogue_per_token_dequant.hpp:664-684 on the vector cores).
//
// Same pipeline as grouped_gemm_mx.cu without scale factors in tensor memory: the whole K is
// accumulated as int32 in one TMEM tile and the epilogue multiplies by token scale x channel scale.
//   mode 0  bf16 tile to a local [rows, N] tensor
//   mode 1  GEMM1: SiLU(gate) * up in fp32 written to a workspace, plus the running maximum of |.|
//           of every row (atomicMax), from which rowquant_int8_kernel derives the per-token scale of
//           the second GEMM's activations (the reference's BlockQuant pass, ...workspace.h:161-277)
//   mode 2  GEMM2: bf16 rows pushed into the combine slots of their origin ranks
// a_scales is [rows] (one per token), b_scales is [E, N] (one per output channel).
#include "gemm_common.cuh"

namespace cam {

constexpr int kI8Threads = 768;
constexpr int kI8EpiThreads = 512;
constexpr int kI8SfWarp0 = 4, kI8EpiWarp0 = 8;
// Shared memory: 4 pipeline stages | bf16 staging of half an output tile (128 rows x 256 bytes,
// rows 272 bytes apart so that 16-byte stores of neighbouring rows fall into different banks; the
// SwiGLU epilogue uses the same bytes for 64 rows of fp32 activations at a time) | barriers.  232448 bytes, the
// whole 227 KiB a CTA can have, so the dynamic segment must start on a 1024-byte boundary.
constexpr int kI8StgPitch = 272;
constexpr int kI8StgBytes = BM * kI8StgPitch;  // 34816
constexpr int kI8ActPitchF = 132;  // SwiGLU epilogue: floats between the staging rows of two tokens (64 rows x 528 bytes)
static_assert(64 * kI8ActPitchF * 4 <= kI8StgBytes, "fp32 staging of 64 rows must fit the staging area");
constexpr int kI8SmemCtrl = 1024;
constexpr int kI8Smem = kStages * kStageBytes + kI8StgBytes + kI8SmemCtrl;
static_assert(kI8Smem <= 232448, "exceeds the shared memory of one CTA");
constexpr uint32_t kI8TmemCols = 512;
// Register re-partitioning (setmaxnreg): the CTA is launched with kI8LaunchRegs per thread (what
// ptxas reports for this kernel); the control and scale-factor warp-groups give registers back
// and the four epilogue warp-groups take them.  setmaxnreg.inc waits for the CTA's pool without
// any time limit, so the sum below must not exceed what the CTA owns.
constexpr uint32_t kI8LaunchRegs = 80, kI8CtrlRegs = 32, kI8SfRegs = 56, kI8EpiRegs = 96;
static_assert(128 * kI8CtrlRegs + 128 * kI8SfRegs + kI8EpiThreads * kI8EpiRegs <= kI8LaunchRegs * kI8Threads,
              "setmaxnreg budget exceeds the registers the CTA owns: the kernel would hang");

__global__ void __launch_bounds__(kI8Threads, 1)
grouped_gemm_w8a8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const GroupedGemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {  // swizzled TMA tiles need it; nothing has been set up yet, so just leave
        if (threadIdx.x == 0) gemm_record_status(p.status, CAM_ERR_BAD_INDEX, 4, static_cast<int>(smem_u32(smem) & 1023u));
        return;
    }
    uint8_t* stg = smem + kStages * kStageBytes;
    uint8_t* ctrl = stg + kI8StgBytes;
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(ctrl);   // TMA bytes of a stage have landed
    uint64_t* bar_sf = bar_full + kStages;                    // scale factors of a stage are in TMEM
    uint64_t* bar_empty = bar_sf + kStages;                   // the MMAs that read a stage have retired
    uint64_t* bar_tfull = bar_empty + kStages;                // accumulator of a tile is complete
    uint64_t* bar_tempty = bar_tfull + 1;                     // accumulator has been drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const uint32_t lane = lane_id();
    const int kblocks = p.k_dim / BK;
    // combine-send form: this rank starts every expert's row blocks at its own offset (see TileWalkerT::locate)
    const int rot_num = (p.mode == 2 && p.num_ranks > 1) ? p.rank : 0, rot_den = (p.mode == 2 && p.num_ranks > 1) ? p.num_ranks : 0;
    const int n_tiles = (p.mode == 1) ? (p.n_dim / 2) / 128 : (p.n_dim + BN - 1) / BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_sf[s], 4);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(bar_tfull, 1);
        mbar_init(bar_tempty, kI8EpiThreads / 32);
        *abort_flag = 0u;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kI8TmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < kI8SfWarp0) {
        reg_dealloc<kI8CtrlRegs>();
        if (warp == 0 && lane == 0) {
            // ------------------------------------------------------------ TMA producer
            prefetch_tensormap(&tmap_a);
            prefetch_tensormap(&tmap_b);
            TileWalker w(p.expert_offsets, p.num_experts, n_tiles);
            uint32_t it = 0;
            int e, mt, nt, row0, rows;
            bool ok = true;
            for (int tile = static_cast<int>(blockIdx.x); ok && w.locate(tile, e, mt, nt, row0, rows, rot_num, rot_den);
                 tile += static_cast<int>(gridDim.x)) {
                const int brow_lo = e * p.n_dim + ((p.mode == 1) ? nt * 128 : nt * BN);
                const int brow_hi = (p.mode == 1) ? (e * p.n_dim + p.n_dim / 2 + nt * 128) : (brow_lo + 128);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    if (!mbar_wait_bounded(&bar_empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    uint8_t* sa = smem + s * kStageBytes;
                    mbar_arrive_expect_tx(&bar_full[s], kStageBytes);
                    tma_load_2d(sa, &tmap_a, &bar_full[s], kb * BK, row0);
                    tma_load_2d(sa + kATile, &tmap_b, &bar_full[s], kb * BK, brow_lo);
                    tma_load_2d(sa + kATile + kBTile / 2, &tmap_b, &bar_full[s], kb * BK, brow_hi);
                }
            }
            if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 0, static_cast<int>(it));
        } else if (warp == 1 && lane == 0) {
            // ------------------------------------------------------------ MMA issuer
            constexpr uint32_t idesc = umma_idesc(BM, BN, /*c = s32*/ 2u, /*signed 8-bit*/ 1u);
            TileWalker w(p.expert_offsets, p.num_experts, n_tiles);
            uint32_t it = 0, tcount = 0;
            int e, mt, nt, row0, rows;
            bool ok = true;
            for (int tile = static_cast<int>(blockIdx.x); ok && w.locate(tile, e, mt, nt, row0, rows, rot_num, rot_den);
                 tile += static_cast<int>(gridDim.x), ++tcount) {
                // the epilogue must have drained the previous tile before its columns are overwritten
                if (!mbar_wait_bounded(bar_tempty, (tcount & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    if (!mbar_wait_bounded(&bar_full[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * kStageBytes);
                    const uint64_t adesc = umma_desc_k_sw128(sa);
                    const uint64_t bdesc = umma_desc_k_sw128(sa + kATile);
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)  // 32 bytes (= 2 x 16) further along K inside the swizzle atom
                        tc_mma_i8(tmem_base, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) ? 1u : 0u);
                    tc_commit(&bar_empty[s]);  // stage (smem and scale columns) reusable once these MMAs retire
                }
                if (!ok) break;
                tc_commit(bar_tfull);  // accumulator complete once every MMA of the tile has retired
            }
            if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 1, static_cast<int>(it));
        }
    } else if (warp < kI8EpiWarp0) {
        reg_dealloc<kI8SfRegs>();
        // this warp-group has no work in the int8 kernel (no scale factors in tensor memory)
    } else {
        reg_alloc<kI8EpiRegs>();
        // ---------------------------------------------------------------- epilogue warps
        const int ew = warp - kI8EpiWarp0;
        const int q = warp & 3;   // TMEM lane quarter this warp may read
        const int cq = ew >> 2;   // which 32-column quarter of each 128-column half
        const int r = q * 32 + static_cast<int>(lane);
        TileWalker w(p.expert_offsets, p.num_experts, n_tiles);
        uint32_t tcount = 0;
        int e, mt, nt, row0, rows;
        bool ok = true;
        for (int tile = static_cast<int>(blockIdx.x); ok && w.locate(tile, e, mt, nt, row0, rows, rot_num, rot_den);
             tile += static_cast<int>(gridDim.x), ++tcount) {
            const bool valid = r < rows && row0 + r < p.a_rows;  // never a row at or past the end of A
            const int grow = row0 + (valid ? r : 0);
            if (!mbar_wait_bounded(bar_tfull, tcount & 1u, abort_flag, 2000000000ull, 256u)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + cq * 32;
            uint32_t v0[32], v1[32];  // columns cq*32.. of the first 128-column half, same of the second
            tmem_ld_32x32b_x32(t0, v0);
            tmem_ld_32x32b_x32(t0 + 128, v1);
            tc_wait_ld_regs(v0);
            tc_wait_ld_regs(v1);
            // the tile now lives in registers: hand the accumulator back to the MMA issuer
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty);

            // dequantise: int32 accumulator x token scale x output-channel scale
            const float sa = __ldg(p.a_scales + grow);
            const int col_lo = (p.mode == 1) ? nt * 128 + cq * 32 : nt * BN + cq * 32;              // first half
            const int col_hi = (p.mode == 1) ? p.n_dim / 2 + nt * 128 + cq * 32 : col_lo + 128;     // second half
            const float* sb_lo = p.b_scales + static_cast<size_t>(e) * p.n_dim + col_lo;
            const float* sb_hi = p.b_scales + static_cast<size_t>(e) * p.n_dim + min(col_hi, p.n_dim - 32);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                v0[j] = __float_as_uint(static_cast<float>(static_cast<int>(v0[j])) * sa * __ldg(sb_lo + j));
                v1[j] = __float_as_uint(static_cast<float>(static_cast<int>(v1[j])) * sa * __ldg(sb_hi + j));
            }
            if (p.mode == 1) {
                // SiLU(gate) * up in fp32 to the workspace, and the row's running max of |.| for the
                // per-token scale of the second GEMM's activations
                const int ia = p.n_dim / 2;
                float act[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float g = __uint_as_float(v0[j]);
                    act[j] = (g / (1.f + expf(-g))) * __uint_as_float(v1[j]);
                }
                // 64 rows at a time go through shared memory as fp32 [row][128 features], so that 8 threads write one
                // row's 512 contiguous bytes (a warp instruction stores four whole rows instead of 16-byte pieces of
                // 32 rows) and the row maximum costs one atomic per row and tile instead of four
                float* stgf = reinterpret_cast<float*>(stg);
                const int te = ew * 32 + static_cast<int>(lane);  // 0..511
                const int rr = te >> 3, pc = te & 7;
                for (int pass = 0; pass * 64 < rows; ++pass) {  // the same trip count in every thread of the CTA
                    if ((q >> 1) == pass) {
                        float* drow = stgf + (r & 63) * kI8ActPitchF + cq * 32;
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4*>(drow + j) = make_float4(act[j], act[j + 1], act[j + 2], act[j + 3]);
                    }
                    named_bar_sync(1, kI8EpiThreads);
                    const float4* src = reinterpret_cast<const float4*>(stgf + rr * kI8ActPitchF + pc * 16);
                    const float4 x0 = src[0], x1 = src[1], x2 = src[2], x3 = src[3];
                    float m = fmaxf(fmaxf(fmaxf(fabsf(x0.x), fabsf(x0.y)), fmaxf(fabsf(x0.z), fabsf(x0.w))),
                                    fmaxf(fmaxf(fabsf(x1.x), fabsf(x1.y)), fmaxf(fabsf(x1.z), fabsf(x1.w))));
                    m = fmaxf(m, fmaxf(fmaxf(fmaxf(fabsf(x2.x), fabsf(x2.y)), fmaxf(fabsf(x2.z), fabsf(x2.w))),
                                       fmaxf(fmaxf(fabsf(x3.x), fabsf(x3.y)), fmaxf(fabsf(x3.z), fabsf(x3.w)))));
                    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
                    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
                    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 4));
                    const int trow = pass * 64 + rr;
                    if (trow < rows) {
                        float4* dst = reinterpret_cast<float4*>(p.act_f32 + static_cast<size_t>(row0 + trow) * ia + nt * 128 +
                                                                pc * 16);
                        dst[0] = x0; dst[1] = x1; dst[2] = x2; dst[3] = x3;
                        if (pc == 0) atomicMax(reinterpret_cast<int*>(p.row_amax + row0 + trow), __float_as_int(m));  // m >= 0
                    }
                    named_bar_sync(1, kI8EpiThreads);  // the staging area may be overwritten
                }
            } else {
                // bf16 tile, either to the local output or straight to the origin rank's combine slot
                __nv_bfloat16* orow = nullptr;
                if (valid) {
                    if (p.mode == 0) {
                        orow = p.out + static_cast<size_t>(grow) * p.n_dim;
                    } else {
                        const int src = p.row_src[static_cast<size_t>(grow) * 3 + 0];
                        const int tok = p.row_src[static_cast<size_t>(grow) * 3 + 1];
                        const int kk = p.row_src[static_cast<size_t>(grow) * 3 + 2];
                        if (src >= 0 && src < p.num_ranks && tok >= 0 && tok < p.max_tokens && kk >= 0 && kk < p.topk)
                            orow = reinterpret_cast<__nv_bfloat16*>(p.peer_base[src] + p.off_combine_buf) +
                                   (static_cast<size_t>(tok) * p.topk + kk) * static_cast<size_t>(p.n_dim);
                    }
                }
                // 256-byte row segments through shared memory, as in grouped_gemm_mx.cu
                uint8_t* srow = stg + r * kI8StgPitch;
                auto push_half = [&](const uint32_t (&v)[32], int c0) {
                    named_bar_sync(1, kI8EpiThreads);  // the previous half has left the staging area
#pragma unroll
                    for (int j = 0; j < 32; j += 8)
                        *reinterpret_cast<uint4*>(srow + cq * 64 + j * 2) =
                            pack_bf16x8(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                        __uint_as_float(v[j + 3]), __uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]),
                                        __uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                    if (cq == 0)
                        *reinterpret_cast<uint64_t*>(srow + 256) =
                            (orow != nullptr) ? reinterpret_cast<uint64_t>(orow + c0) : 0ull;
                    named_bar_sync(1, kI8EpiThreads);
                    const int seg = static_cast<int>(lane & 15u) * 16;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint8_t* src = stg + (ew * 8 + 2 * i + static_cast<int>(lane >> 4)) * kI8StgPitch;
                        const uint64_t dst = *reinterpret_cast<const uint64_t*>(src + 256);
                        if (dst != 0ull)
                            st_na_v4(reinterpret_cast<uint8_t*>(dst) + seg, *reinterpret_cast<const uint4*>(src + seg));
                    }
                };
                const int c_lo = nt * BN;
                push_half(v0, c_lo);
                if (c_lo + 128 < p.n_dim) push_half(v1, c_lo + 128);  // same answer in every thread of the CTA
            }
        }
        if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 2, static_cast<int>(tcount));
    }

    // ------------------------------------------------------------------ teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kI8TmemCols);
    }
    if (p.mode == 2 && threadIdx.x == 0) {
        __threadfence_system();
        const unsigned int old = atomicAdd(p.done_ctr, 1u);
        if (old == gridDim.x - 1) {
            p.done_ctr[0] = 0u;
            __threadfence_system();
            const uint32_t epoch = *p.epoch_send + 1u;  // this launch is the send phase of a combine
            if (p.dbg_drop_flags == 0) {
                for (int d = 0; d < p.num_ranks; ++d)
                    st_release_sys_u32(reinterpret_cast<uint32_t*>(p.peer_base[d] + p.off_combine_flag) + p.rank,
                                       epoch);
            }
            *p.epoch_send = epoch;
        }
    }
}


// Per-token int8 quantisation of the SwiGLU output (one warp per row): scale = max|row| / 127 from the
// maxima GEMM1 accumulated, q = rint(x / scale).  Clears the row maximum for the next call.
__global__ void rowquant_int8_kernel(const float* __restrict__ act, float* row_amax, const int* __restrict__ expert_offsets,
                                     int num_experts, int inter, int8_t* __restrict__ out_q, float* __restrict__ out_s) {
    const int rows = expert_offsets[num_experts];
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t lane = lane_id();
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const float amax = fmaxf(row_amax[r], 1e-12f);
        __syncwarp();
        if (lane == 0) row_amax[r] = 0.f;
        const float inv = 127.f / amax;
        const float* src = act + static_cast<size_t>(r) * inter;
        int8_t* dst = out_q + static_cast<size_t>(r) * inter;
        for (int c = static_cast<int>(lane) * 4; c < inter; c += 128) {
            const float4 v = *reinterpret_cast<const float4*>(src + c);
            const int a0 = max(-127, min(127, __float2int_rn(v.x * inv))), a1 = max(-127, min(127, __float2int_rn(v.y * inv)));
            const int a2 = max(-127, min(127, __float2int_rn(v.z * inv))), a3 = max(-127, min(127, __float2int_rn(v.w * inv)));
            *reinterpret_cast<uint32_t*>(dst + c) = (static_cast<uint32_t>(a0) & 0xFFu) | ((static_cast<uint32_t>(a1) & 0xFFu) << 8) |
                                                    ((static_cast<uint32_t>(a2) & 0xFFu) << 16) | ((static_cast<uint32_t>(a3) & 0xFFu) << 24);
        }
        if (lane == 0) out_s[r] = amax / 127.f;
    }
}

}  // namespace cam

extern "C" int cam_launch_rowquant_int8(const float* act, float* row_amax, const int* expert_offsets, int num_experts,
                                        int inter, void* out_q, float* out_s, cudaStream_t stream) {
    cam::rowquant_int8_kernel<<<4 * cam::sm_count_of_current_device(), 256, 0, stream>>>(act, row_amax, expert_offsets, num_experts, inter,
                                                           static_cast<int8_t*>(out_q), out_s);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int cam_grouped_gemm_w8a8_smem_bytes(void) { return cam::kI8Smem; }

extern "C" int cam_launch_grouped_gemm_w8a8(const cam::GroupedGemmParams* p, const CUtensorMap* tmap_a,
                                             const CUtensorMap* tmap_b, int grid, cudaStream_t stream) {
    static cam::SmemLimitCache limit;
    cudaError_t e = limit.ensure(cam::grouped_gemm_w8a8_kernel, cam::kI8Smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    cam::grouped_gemm_w8a8_kernel<<<grid, cam::kI8Threads, cam::kI8Smem, stream>>>(*tmap_a, *tmap_b, *p);
    return static_cast<int>(cudaGetLastError());
}
