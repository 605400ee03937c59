// Grouped (per-expert, ragged-M) block-scaled fp8 GEMM for sm_100a, written directly on
// tcgen05 / TMEM / TMA, with three epilogues:
//   mode 0  dequantised bf16 tile to a local [rows, N] tensor (stand-alone grouped GEMM)
//   mode 1  GEMM1 of the MoE MLP: SiLU(gate) * up on the fp32 accumulators, then 1x128 fp8
//           re-quantisation -> feeds GEMM2 without an extra pass over memory
//   mode 2  GEMM2: bf16 tile pushed with P2P stores straight into the (token, k) combine slot
//           of the token's origin rank; the last CTA raises this rank's combine flag in every
//           peer, so the combine transfer overlaps the tensor-core tiles
//
// It stands where the reference has its two CATLASS-based kernels
// GroupedMatmulSliceMPerTokenDequantSwigluQuant (fused_deep_moe/gemm/kernel/
// grouped_matmul_slice_m_per_token_dequant_swiglu_quant_multistage_workspace.h:355-1718) and
// GroupedMatmulSliceMPerTokenDequant (..._dequant_multistage_workspace.h:24-378), the SwiGLU
// epilogue (epilogue/block/block_epilogue_per_token_dequant_swiglu.h:236-272: first half of N is
// the gate) and the combine-send epilogue (block_epilogue_per_token_dequant.hpp:531-570).
//
// Tile: 128 rows x 256 columns x 128 K per pipeline stage.  The 256 columns are two 128-row
// B boxes, which for mode 1 are the gate rows [n, n+128) and the up rows [I+n, I+n+128) of the
// same expert, so one thread owns matching gate/up columns.
// Scaling: activations carry one fp32 scale per (row, 128 K), weights one per (128 N, 128 K).
// Each 128-K block is multiplied into a fresh TMEM accumulator (two TMEM stages of 256 columns)
// and promoted into fp32 registers by the epilogue warps while the tensor core works on the
// next block.
//
// Warp roles (640 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 4..19 = epilogue (warp w reads TMEM lanes 32*(w%4).., 32-column quarter (w-4)/4 of each
// 128-column block; four epilogue warps per scheduler hide the TMEM load latency).
// Every mbarrier wait is bounded; a role that gives up sets a shared abort word that releases
// the others, a status word is recorded and the CTA frees its TMEM and returns.
#include "gemm_common.cuh"

namespace cam {

constexpr int kGemmThreads = 640;   // 4 control warps + 16 epilogue warps
constexpr int kEpiThreads = 512;
// Shared memory: 4 pipeline stages | bf16 staging of half an output tile (128 rows x 256 bytes, rows 272 bytes
// apart so that 16-byte stores of neighbouring rows fall into different banks; the per-row amax exchange of the
// SwiGLU epilogue uses the same bytes) | barriers.  232448 bytes, the whole 227 KiB a CTA can have, so the
// dynamic segment must start on a 1024-byte boundary.
constexpr int kStgPitch = 272;
constexpr int kStgBytes = BM * kStgPitch;  // 34816
constexpr int kSmemCtrl = 1024;
constexpr int kGemmSmem = kStages * kStageBytes + kStgBytes + kSmemCtrl;
static_assert(kGemmSmem <= 232448, "exceeds the shared memory of one CTA");
constexpr uint32_t kTmemCols = 512;
// Register re-partitioning (setmaxnreg).  The CTA is launched with kLaunchRegs per thread (what
// ptxas reports for __launch_bounds__(640, 1)); the control warp-group gives registers back and
// the four epilogue warp-groups take them.  setmaxnreg.inc blocks until the CTA's pool has the
// registers, without any time limit, so the budget below must hold exactly.
constexpr uint32_t kLaunchRegs = 96, kCtrlRegs = 32, kEpiRegs = 112;
static_assert(128 * kCtrlRegs + kEpiThreads * kEpiRegs <= kLaunchRegs * kGemmThreads,
              "setmaxnreg budget exceeds the registers the CTA owns: the kernel would hang");

__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const GroupedGemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {  // swizzled TMA tiles need it; nothing has been set up yet, so just leave
        if (threadIdx.x == 0) gemm_record_status(p.status, CAM_ERR_BAD_INDEX, 4, static_cast<int>(smem_u32(smem) & 1023u));
        return;
    }
    uint8_t* stg = smem + kStages * kStageBytes;
    uint8_t* ctrl = stg + kStgBytes;
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(ctrl);
    uint64_t* bar_empty = bar_full + kStages;
    uint64_t* bar_tfull = bar_empty + kStages;
    uint64_t* bar_tempty = bar_tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* s_amax = reinterpret_cast<float*>(stg);  // mode 1 only: [2 parities][4 column quarters][128 rows]

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const uint32_t lane = lane_id();
    const int kblocks = p.k_dim / BK;
    // combine-send form: this rank starts every expert's row blocks at its own offset (see TileWalkerT::locate)
    const int rot_num = (p.mode == 2 && p.num_ranks > 1) ? p.rank : 0, rot_den = (p.mode == 2 && p.num_ranks > 1) ? p.num_ranks : 0;
    const int n_tiles = (p.mode == 1) ? (p.n_dim / 2) / 128 : (p.n_dim + BN - 1) / BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&bar_tfull[a], 1);
            mbar_init(&bar_tempty[a], kEpiThreads / 32);
        }
        *abort_flag = 0u;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        reg_dealloc<kCtrlRegs>();
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
            constexpr uint32_t idesc = umma_idesc(BM, BN, /*c=f32*/ 1u, /*e4m3*/ 0u);
            TileWalker w(p.expert_offsets, p.num_experts, n_tiles);
            uint32_t it = 0;
            int e, mt, nt, row0, rows;
            bool ok = true;
            for (int tile = static_cast<int>(blockIdx.x); ok && w.locate(tile, e, mt, nt, row0, rows, rot_num, rot_den);
                 tile += static_cast<int>(gridDim.x)) {
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    const uint32_t a = it & 1u, aph = (it >> 1) & 1u;
                    if (!mbar_wait_bounded(&bar_tempty[a], aph ^ 1u, abort_flag)) { ok = false; break; }
                    if (!mbar_wait_bounded(&bar_full[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * kStageBytes);
                    const uint64_t adesc = umma_desc_k_sw128(sa);
                    const uint64_t bdesc = umma_desc_k_sw128(sa + kATile);
                    const uint32_t d = tmem_base + a * BN;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)  // advance 32 bytes (= 2 x 16) along K inside the swizzle atom
                        tc_mma_f8(d, adesc + 2u * k, bdesc + 2u * k, idesc, k > 0 ? 1u : 0u);
                    tc_commit(&bar_empty[s]);  // smem stage reusable once these MMAs retire
                    tc_commit(&bar_tfull[a]);  // accumulator stage ready for the epilogue
                }
            }
            if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 1, static_cast<int>(it));
        }
    } else {
        reg_alloc<kEpiRegs>();
        // ---------------------------------------------------------------- epilogue warps
        const int ew = warp - 4;
        const int q = warp & 3;   // TMEM lane quarter this warp may read
        const int cq = ew >> 2;   // which 32-column quarter of each 128-column block
        const int r = q * 32 + static_cast<int>(lane);
        const int kbs = kblocks;  // scales per row of A
        const int nblk = p.n_dim / 128;
        TileWalker w(p.expert_offsets, p.num_experts, n_tiles);
        uint32_t it = 0;
        uint32_t tile_parity = 0;
        int e, mt, nt, row0, rows;
        bool ok = true;
        for (int tile = static_cast<int>(blockIdx.x); ok && w.locate(tile, e, mt, nt, row0, rows, rot_num, rot_den);
             tile += static_cast<int>(gridDim.x), tile_parity ^= 1u) {
            const bool valid = r < rows && row0 + r < p.a_rows;  // never a row at or past the end of A
            const int grow = row0 + (valid ? r : 0);
            const float* as = p.a_scales + static_cast<size_t>(grow) * kbs;
            int nb_lo, nb_hi;
            if (p.mode == 1) { nb_lo = nt; nb_hi = nblk / 2 + nt; }
            else { nb_lo = 2 * nt; nb_hi = min(2 * nt + 1, nblk - 1); }
            const float* bs_lo = p.b_scales + (static_cast<size_t>(e) * nblk + nb_lo) * kbs;
            const float* bs_hi = p.b_scales + (static_cast<size_t>(e) * nblk + nb_hi) * kbs;

            float acc[64];  // [0,32): columns cq*32.. of the first 128-column block, [32,64): same of the second
#pragma unroll
            for (int j = 0; j < 64; ++j) acc[j] = 0.f;

            // scales are fetched two K-blocks ahead of their use
            float sa0 = __ldg(as), wl0 = __ldg(bs_lo), wh0 = __ldg(bs_hi);
            float sa1 = sa0, wl1 = wl0, wh1 = wh0;
            if (kblocks > 1) { sa1 = __ldg(as + 1); wl1 = __ldg(bs_lo + 1); wh1 = __ldg(bs_hi + 1); }
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                const float s_lo = sa0 * wl0, s_hi = sa0 * wh0;
                sa0 = sa1; wl0 = wl1; wh0 = wh1;
                if (kb + 2 < kblocks) {
                    sa1 = __ldg(as + kb + 2);
                    wl1 = __ldg(bs_lo + kb + 2);
                    wh1 = __ldg(bs_hi + kb + 2);
                }
                const uint32_t a = it & 1u, aph = (it >> 1) & 1u;
                if (!mbar_wait_bounded(&bar_tfull[a], aph, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * BN + cq * 32;
                uint32_t v[32];
                tmem_ld_32x32b_x32(t0, v);
                tc_wait_ld_regs(v);
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[j] = fmaf(s_lo, __uint_as_float(v[j]), acc[j]);
                tmem_ld_32x32b_x32(t0 + 128, v);
                tc_wait_ld_regs(v);
                // all TMEM reads of this stage are done: hand it back to the MMA issuer
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_tempty[a]);
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[32 + j] = fmaf(s_hi, __uint_as_float(v[j]), acc[32 + j]);
            }
            if (!ok) break;

            if (p.mode == 1) {
                // SwiGLU on matching gate/up columns, then 1x128 fp8 requantisation of the row block.
                const int ia = p.n_dim / 2;
                float amax = 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float g = acc[j];
                    const float act = (g / (1.f + expf(-g))) * acc[32 + j];
                    acc[j] = act;
                    amax = fmaxf(amax, fabsf(act));
                }
                float* xch = s_amax + tile_parity * 512;
                xch[cq * 128 + r] = amax;
                named_bar_sync(1, kEpiThreads);
                amax = fmaxf(fmaxf(xch[r], xch[128 + r]), fmaxf(xch[256 + r], xch[384 + r]));
                const float a_cl = fmaxf(amax, 1e-4f);
                const float inv = 448.f / a_cl;
                if (valid) {
                    uint8_t* dst = p.act_q + static_cast<size_t>(grow) * ia + nt * 128 + cq * 32;
#pragma unroll
                    for (int j = 0; j < 32; j += 16) {
                        uint4 o;
                        o.x = pack_e4m3x4(acc[j + 0] * inv, acc[j + 1] * inv, acc[j + 2] * inv, acc[j + 3] * inv);
                        o.y = pack_e4m3x4(acc[j + 4] * inv, acc[j + 5] * inv, acc[j + 6] * inv, acc[j + 7] * inv);
                        o.z = pack_e4m3x4(acc[j + 8] * inv, acc[j + 9] * inv, acc[j + 10] * inv, acc[j + 11] * inv);
                        o.w = pack_e4m3x4(acc[j + 12] * inv, acc[j + 13] * inv, acc[j + 14] * inv, acc[j + 15] * inv);
                        *reinterpret_cast<uint4*>(dst + j) = o;
                    }
                    if (cq == 0) p.act_s[static_cast<size_t>(grow) * (ia / 128) + nt] = a_cl / 448.f;
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
                // Half a tile (128 columns) at a time goes through shared memory as bf16 and leaves as 256-byte row
                // segments: one bulk copy per row (local or over NVLink), or, with bulk_push off, 16 lanes storing one
                // row, instead of 16-byte pieces of 32 different rows per warp instruction.  The row's destination
                // address travels in the 16 spare bytes at the end of its staging row.
                uint8_t* srow = stg + r * kStgPitch;
                auto push_half = [&](const float* v, int c0) {
                    if (p.bulk_push && cq == 0) bulk_wait_group_read<0>();  // the previous copies have read the staging area
                    named_bar_sync(1, kEpiThreads);  // the previous half has left the staging area
#pragma unroll
                    for (int j = 0; j < 32; j += 8)
                        *reinterpret_cast<uint4*>(srow + cq * 64 + j * 2) =
                            pack_bf16x8(v[j], v[j + 1], v[j + 2], v[j + 3], v[j + 4], v[j + 5], v[j + 6], v[j + 7]);
                    if (cq == 0)
                        *reinterpret_cast<uint64_t*>(srow + 256) =
                            (orow != nullptr) ? reinterpret_cast<uint64_t>(orow + c0) : 0ull;
                    if (p.bulk_push) {
                        fence_proxy_async_smem();
                        named_bar_sync(1, kEpiThreads);
                        if (cq == 0) {
                            if (orow != nullptr) bulk_store_s2g(orow + c0, srow, 256);
                            bulk_commit_group();
                        }
                        return;
                    }
                    named_bar_sync(1, kEpiThreads);
                    const int seg = static_cast<int>(lane & 15u) * 16;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint8_t* src = stg + (ew * 8 + 2 * i + static_cast<int>(lane >> 4)) * kStgPitch;
                        const uint64_t dst = *reinterpret_cast<const uint64_t*>(src + 256);
                        if (dst != 0ull)
                            st_na_v4(reinterpret_cast<uint8_t*>(dst) + seg, *reinterpret_cast<const uint4*>(src + seg));
                    }
                };
                const int c_lo = nt * BN;
                push_half(acc, c_lo);
                if (c_lo + 128 < p.n_dim) push_half(acc + 32, c_lo + 128);  // same answer in every thread of the CTA
            }
        }
        if (p.mode != 1 && p.bulk_push && cq == 0) bulk_wait_group<0>();  // every row this thread sent has been written
        if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 2, static_cast<int>(it));
    }

    // ------------------------------------------------------------------ teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
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

}  // namespace cam

extern "C" int cam_grouped_gemm_smem_bytes(void) { return cam::kGemmSmem; }

extern "C" int cam_launch_grouped_gemm_fp8(const cam::GroupedGemmParams* p, const CUtensorMap* tmap_a,
                                           const CUtensorMap* tmap_b, int grid, cudaStream_t stream) {
    static cam::SmemLimitCache limit;
    cudaError_t e = limit.ensure(cam::grouped_gemm_fp8_kernel, cam::kGemmSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    cam::grouped_gemm_fp8_kernel<<<grid, cam::kGemmThreads, cam::kGemmSmem, stream>>>(*tmap_a, *tmap_b, *p);
    return static_cast<int>(cudaGetLastError());
}
