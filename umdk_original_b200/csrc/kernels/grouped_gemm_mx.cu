// Grouped (per-expert, ragged-M) fp8 GEMM for sm_100a whose block scaling is done by the tensor
// core: tcgen05.mma kind::mxf8f6f4.block_scale multiplies every 32-element K-slice of an A row
// and of a B row by a UE8M0 (power-of-two) scale factor held in tensor memory, so the whole
// reduction accumulates in ONE TMEM tile and the epilogue runs once per output tile instead of
// once per 128-K block.  It is the fast path of the expert MLP; the kernel in grouped_gemm.cu
// keeps arbitrary fp32 scales by promoting every K-block in registers and is about 2x slower.
//
// Contract: a_scales [rows, K/128] and b_scales [E, N/128, K/128] are fp32 numbers that are exact
// powers of two (what quantisation with `ue8m0` scale rounding produces); only their exponent
// byte is used.  Same three epilogues as grouped_gemm.cu (mode 0 bf16 tile, mode 1 SwiGLU + 1x128
// fp8 requantisation with power-of-two scales, mode 2 bf16 rows pushed into the combine slots of
// the origin ranks), same role in the layer as the reference's two CATLASS kernels
// (fused_deep_moe/gemm/kernel/grouped_matmul_slice_m_per_token_dequant_swiglu_quant_multistage_
// workspace.h:355-1718 and ..._dequant_multistage_workspace.h:24-378): there the per-token and
// per-channel scales are applied by vector cores after an int32 cube GEMM
// (epilogue/block/block_epilogue_per_token_dequant_swiglu.h:236-272).
//
// Tile 128 x 256 x 128 per pipeline stage, four stages of shared memory fed by TMA.
// Tensor memory (512 columns): accumulator in columns [0, 256); scale factors of pipeline stage
// s in columns [256 + 16 s, 256 + 16 s + 12): 4 columns for the 128 A rows (row m sits in lane
// m % 32, column m / 32, replicated in the four 32-lane quarters), 8 columns for the 256 B rows.
// Each 32-bit scale column holds the scale bytes of 4 consecutive 32-element K-slices; with 1x128
// scaling the four bytes are equal, so every MMA of a stage uses byte 0.
//
// Warp roles (768 threads): warp 0 lane 0 = TMA producer, warp 1 lane 0 = MMA issuer (warp 1 owns
// the TMEM allocation), warps 4..7 = scale-factor writers (one per TMEM lane quarter: they load
// the fp32 scales two K-blocks ahead, take the exponent bytes and tcgen05.st them), warps 8..23 =
// epilogue (warp w drains lanes 32 (w % 4).., 32-column quarter (w - 8) / 4 of each 128-column
// half into registers, hands the accumulator back, then does the math and the stores while the
// tensor core already works on the next tile).
// Every mbarrier wait is bounded; a role that gives up sets a shared abort word that releases
// the others, a status word is recorded and the CTA frees its TMEM and returns.
//
// SWAP = true is the form for small experts (about a tile of rows or less each).  tcgen05.mma fixes
// M at 128 but lets N go in steps of 16, so a tile that holds 2 rows of an expert costs as much as a
// full one when the rows are the M operand.  With the operands exchanged the two 128-row halves of the
// weight tile are the M operands of two MMAs, the token rows are the N operand with N = rows rounded up
// to 16, and the accumulators hold the tile transposed: lane = output feature, column = token, first
// half of the features in columns [0, 128), second half in [128, 256).  Shared-memory tiles, TMA loads
// and scale-factor columns are the same (the scale-factor layouts of A and B coincide); only the MMA
// issue and the epilogue, which transposes through shared memory, differ.
#include "gemm_common.cuh"

namespace cam {

constexpr int kMxThreads = 768;
constexpr int kMxEpiThreads = 512;
constexpr int kMxSfWarp0 = 4, kMxEpiWarp0 = 8;
// Shared memory: 4 pipeline stages | bf16 staging of half an output tile (128 rows x 256 bytes,
// rows 272 bytes apart so that 16-byte stores of neighbouring rows fall into different banks; the
// per-row amax exchange of the SwiGLU epilogue uses the same bytes) | barriers.  232448 bytes, the
// whole 227 KiB a CTA can have, so the dynamic segment must start on a 1024-byte boundary.
constexpr int kMxStgPitch = 272;
constexpr int kMxStgBytes = BM * kMxStgPitch;  // 34816
constexpr int kMxSmemCtrl = 1024;
// The combine-send form (mode 2) trades one pipeline stage for a second staging buffer, so that the epilogue can
// convert the next half tile while the copies of the previous one are still reading theirs.
constexpr int kMxStagesSend = 3;
template <int NS, int NSTG>
constexpr int mx_smem() { return NS * kStageBytes + NSTG * kMxStgBytes + kMxSmemCtrl; }
constexpr int kMxSmem = mx_smem<kStages, 1>();
static_assert(kMxSmem <= 232448 && mx_smem<kMxStagesSend, 2>() <= 232448, "exceeds the shared memory of one CTA");
constexpr int kMxTPitchF = 132;  // SWAP, SwiGLU epilogue: floats between the staging rows of two tokens (64 x 132 x 4 bytes)
static_assert(64 * kMxTPitchF * 4 <= kMxStgBytes, "transposed fp32 staging of 64 tokens must fit the staging area");
constexpr uint32_t kMxTmemCols = 512;
constexpr uint32_t kMxSfCol0 = 256, kMxSfStride = 16;
// Register re-partitioning (setmaxnreg): the CTA is launched with kMxLaunchRegs per thread (what
// ptxas reports for this kernel); the control and scale-factor warp-groups give registers back
// and the four epilogue warp-groups take them.  setmaxnreg.inc waits for the CTA's pool without
// any time limit, so the sum below must not exceed what the CTA owns.
constexpr uint32_t kMxLaunchRegs = 80, kMxCtrlRegs = 32, kMxSfRegs = 56, kMxEpiRegs = 96;
static_assert(128 * kMxCtrlRegs + 128 * kMxSfRegs + kMxEpiThreads * kMxEpiRegs <= kMxLaunchRegs * kMxThreads,
              "setmaxnreg budget exceeds the registers the CTA owns: the kernel would hang");

template <bool SWAP, int NS, int NSTG>
__global__ void __launch_bounds__(kMxThreads, 1)
grouped_gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const GroupedGemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {  // swizzled TMA tiles need it; nothing has been set up yet, so just leave
        if (threadIdx.x == 0) gemm_record_status(p.status, CAM_ERR_BAD_INDEX, 4, static_cast<int>(smem_u32(smem) & 1023u));
        return;
    }
    uint8_t* stg = smem + NS * kStageBytes;
    uint8_t* ctrl = stg + NSTG * kMxStgBytes;
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(ctrl);   // TMA bytes of a stage have landed
    uint64_t* bar_sf = bar_full + NS;                    // scale factors of a stage are in TMEM
    uint64_t* bar_empty = bar_sf + NS;                   // the MMAs that read a stage have retired
    uint64_t* bar_tfull = bar_empty + NS;                // accumulator of a tile is complete
    uint64_t* bar_tempty = bar_tfull + 1;                     // accumulator has been drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* s_amax = reinterpret_cast<float*>(stg);  // mode 1 only: [2 parities][4 column quarters][128 rows]

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const uint32_t lane = lane_id();
    const int kblocks = p.k_dim / BK;
    // combine-send form: this rank starts every expert's row blocks at its own offset (see TileWalkerT::locate)
    const int rot_num = (p.mode == 2 && p.num_ranks > 1) ? p.rank : 0, rot_den = (p.mode == 2 && p.num_ranks > 1) ? p.num_ranks : 0;
    const int n_tiles = (p.mode == 1) ? (p.n_dim / 2) / 128 : (p.n_dim + BN - 1) / BN;
    const int nblk = p.n_dim / 128;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_sf[s], 4);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(bar_tfull, 1);
        mbar_init(bar_tempty, kMxEpiThreads / 32);
        *abort_flag = 0u;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kMxTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < kMxSfWarp0) {
        reg_dealloc<kMxCtrlRegs>();
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
                    const uint32_t s = it % NS, ph = (it / NS) & 1u;
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
            constexpr uint32_t idesc = umma_idesc_mxf8(BM, BN);
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
                    const uint32_t s = it % NS, ph = (it / NS) & 1u;
                    if (!mbar_wait_bounded(&bar_sf[s], ph, abort_flag)) { ok = false; break; }
                    if (!mbar_wait_bounded(&bar_full[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * kStageBytes);
                    const uint64_t adesc = umma_desc_k_sw128(sa);
                    const uint64_t bdesc = umma_desc_k_sw128(sa + kATile);
                    const uint32_t sfa = tmem_base + kMxSfCol0 + s * kMxSfStride;
                    const uint32_t sfb = sfa + 4u;
                    if constexpr (SWAP) {
                        // weights are the M operand (two halves, two accumulators), the tile's rows the N operand
                        const uint32_t idesc_t = umma_idesc_mxf8(128u, static_cast<uint32_t>((rows + 15) & ~15));
                        const uint64_t bdesc_hi = umma_desc_k_sw128(sa + kATile + kBTile / 2);
#pragma unroll
                        for (int k = 0; k < BK / 32; ++k) {
                            tc_mma_mxf8(tmem_base, bdesc + 2u * k, adesc + 2u * k, idesc_t, (kb | k) ? 1u : 0u, sfb, sfa);
                            tc_mma_mxf8(tmem_base + 128u, bdesc_hi + 2u * k, adesc + 2u * k, idesc_t, (kb | k) ? 1u : 0u,
                                        sfb + 4u, sfa);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < BK / 32; ++k)  // 32 bytes (= 2 x 16) further along K inside the swizzle atom
                            tc_mma_mxf8(tmem_base, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) ? 1u : 0u, sfa, sfb);
                    }
                    tc_commit(&bar_empty[s]);  // stage (smem and scale columns) reusable once these MMAs retire
                }
                if (!ok) break;
                tc_commit(bar_tfull);  // accumulator complete once every MMA of the tile has retired
            }
            if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 1, static_cast<int>(it));
        }
    } else if (warp < kMxEpiWarp0) {
        reg_dealloc<kMxSfRegs>();
        // ---------------------------------------------------------------- scale-factor writers
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        TileWalker w(p.expert_offsets, p.num_experts, n_tiles);
        uint32_t it = 0;
        int e, mt, nt, row0, rows;
        bool ok = true;
        // rows of scales can be read 16 bytes at a time when K is a multiple of 512 and the arrays are aligned
        const bool vec_scales = (kblocks & 3) == 0 &&
                                ((reinterpret_cast<uintptr_t>(p.a_scales) | reinterpret_cast<uintptr_t>(p.b_scales)) & 15u) == 0u;
        for (int tile = static_cast<int>(blockIdx.x); ok && w.locate(tile, e, mt, nt, row0, rows, rot_num, rot_den);
             tile += static_cast<int>(gridDim.x)) {
            const float* as[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = min(row0 + 32 * j + static_cast<int>(lane), p.a_rows - 1);
                as[j] = p.a_scales + static_cast<size_t>(r) * kblocks;
            }
            int nb_lo, nb_hi;
            if (p.mode == 1) { nb_lo = nt; nb_hi = nblk / 2 + nt; }
            else { nb_lo = 2 * nt; nb_hi = min(2 * nt + 1, nblk - 1); }
            const float* bs_lo = p.b_scales + (static_cast<size_t>(e) * nblk + nb_lo) * kblocks;
            const float* bs_hi = p.b_scales + (static_cast<size_t>(e) * nblk + nb_hi) * kblocks;
            // One K-block: write the six scale words of stage s into TMEM and tell the MMA issuer.
            auto put = [&](uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t w4, uint32_t w5) -> bool {
                const uint32_t s = it % NS, ph = (it / NS) & 1u;
                const bool got = mbar_wait_bounded(&bar_empty[s], ph ^ 1u, abort_flag);
                if (!__all_sync(0xFFFFFFFFu, got)) return false;
                tc_fence_after_sync();
                const uint32_t col = tmem_base + lane_base + kMxSfCol0 + s * kMxSfStride;
                tmem_st_32x32b_x4(col, w0, w1, w2, w3);
                tmem_st_32x32b_x4(col + 4u, w4, w4, w4, w4);
                tmem_st_32x32b_x4(col + 8u, w5, w5, w5, w5);
                tc_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_sf[s]);
                ++it;
                return true;
            };
            if (vec_scales) {
                // Scales move in groups of four K-blocks: one 16-byte load per row and group, issued a whole group
                // before its first use, so that a load that misses L1 still arrives in time (a load that is only one
                // K-block ahead makes these warps, and with them the MMA issuer, run at one K-block per L2 latency
                // whenever it misses).  A group is packed to one exponent byte per K-block as soon as it is there.
                const int ngroups = kblocks >> 2;
                float4 na[4], nbl, nbh;
                auto load_group = [&](int g) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) na[j] = __ldg(reinterpret_cast<const float4*>(as[j]) + g);
                    nbl = __ldg(reinterpret_cast<const float4*>(bs_lo) + g);
                    nbh = __ldg(reinterpret_cast<const float4*>(bs_hi) + g);
                };
                load_group(0);
                for (int g = 0; ok && g < ngroups; ++g) {
                    uint32_t pk[6];
#pragma unroll
                    for (int j = 0; j < 4; ++j) pk[j] = ue8m0_pack4(na[j]);
                    pk[4] = ue8m0_pack4(nbl);
                    pk[5] = ue8m0_pack4(nbh);
                    ok = put(__byte_perm(pk[0], 0, 0x0000), __byte_perm(pk[1], 0, 0x0000), __byte_perm(pk[2], 0, 0x0000),
                             __byte_perm(pk[3], 0, 0x0000), __byte_perm(pk[4], 0, 0x0000), __byte_perm(pk[5], 0, 0x0000));
                    // the next group's loads go out only after the arrive above, which has release semantics and
                    // would otherwise wait for them
                    if (g + 1 < ngroups) load_group(g + 1);
                    if (ok)
                        ok = put(__byte_perm(pk[0], 0, 0x1111), __byte_perm(pk[1], 0, 0x1111), __byte_perm(pk[2], 0, 0x1111),
                                 __byte_perm(pk[3], 0, 0x1111), __byte_perm(pk[4], 0, 0x1111), __byte_perm(pk[5], 0, 0x1111));
                    if (ok)
                        ok = put(__byte_perm(pk[0], 0, 0x2222), __byte_perm(pk[1], 0, 0x2222), __byte_perm(pk[2], 0, 0x2222),
                                 __byte_perm(pk[3], 0, 0x2222), __byte_perm(pk[4], 0, 0x2222), __byte_perm(pk[5], 0, 0x2222));
                    if (ok)
                        ok = put(__byte_perm(pk[0], 0, 0x3333), __byte_perm(pk[1], 0, 0x3333), __byte_perm(pk[2], 0, 0x3333),
                                 __byte_perm(pk[3], 0, 0x3333), __byte_perm(pk[4], 0, 0x3333), __byte_perm(pk[5], 0, 0x3333));
                }
                continue;
            }
            // any other K: scalar loads, fetched two K-blocks ahead of their use
            float c[6], n1[6];
#pragma unroll
            for (int j = 0; j < 4; ++j) c[j] = __ldg(as[j]);
            c[4] = __ldg(bs_lo); c[5] = __ldg(bs_hi);
#pragma unroll
            for (int j = 0; j < 6; ++j) n1[j] = c[j];
            if (kblocks > 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) n1[j] = __ldg(as[j] + 1);
                n1[4] = __ldg(bs_lo + 1); n1[5] = __ldg(bs_hi + 1);
            }
            for (int kb = 0; ok && kb < kblocks; ++kb) {
                ok = put(ue8m0_word(c[0]), ue8m0_word(c[1]), ue8m0_word(c[2]), ue8m0_word(c[3]), ue8m0_word(c[4]),
                         ue8m0_word(c[5]));
#pragma unroll
                for (int j = 0; j < 6; ++j) c[j] = n1[j];
                if (kb + 2 < kblocks) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) n1[j] = __ldg(as[j] + kb + 2);
                    n1[4] = __ldg(bs_lo + kb + 2); n1[5] = __ldg(bs_hi + kb + 2);
                }
            }
        }
        if (!ok && lane == 0) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 3, static_cast<int>(it));
    } else {
        reg_alloc<kMxEpiRegs>();
        // ---------------------------------------------------------------- epilogue warps
        const int ew = warp - kMxEpiWarp0;
        const int q = warp & 3;   // TMEM lane quarter this warp may read
        const int cq = ew >> 2;   // which 32-column quarter of each 128-column half
        const int r = q * 32 + static_cast<int>(lane);
        TileWalker w(p.expert_offsets, p.num_experts, n_tiles);
        uint32_t tcount = 0, halves = 0;
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
            // SWAP: lane r is an output feature and these are tokens cq*32.. of the tile; column quarters past the
            // tile's rows were not written by its MMAs and are not read
            const bool has_cols = !SWAP || cq * 32 < rows;
            if (has_cols) {
                tmem_ld_32x32b_x32(t0, v0);
                tmem_ld_32x32b_x32(t0 + 128, v1);
                tc_wait_ld_regs(v0);
                tc_wait_ld_regs(v1);
            }
            // the tile now lives in registers: hand the accumulator back to the MMA issuer
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty);

            if (SWAP && p.mode == 1) {
                // SwiGLU: lane r holds gate feature nt*128 + r (first accumulator) and the matching up feature (second)
                // for 32 tokens.  The 128 lanes are one 1x128 quantisation block of every token, so the tile is
                // transposed through shared memory, 64 tokens at a time as fp32 [token][feature], and then 8 threads
                // per token take the maximum, quantise and store 16 bytes each: one 128-byte segment per token.
                const int ia = p.n_dim / 2;
                if (has_cols) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {  // the product replaces the gate value
                        const float g = __uint_as_float(v0[j]);
                        v0[j] = __float_as_uint((g / (1.f + expf(-g))) * __uint_as_float(v1[j]));
                    }
                }
                float* stgf = reinterpret_cast<float*>(stg);
                const int te = ew * 32 + static_cast<int>(lane);  // 0..511
                const int tl = te >> 3, pc = te & 7;
                for (int half = 0; half * 64 < rows; ++half) {  // the same trip count in every thread of the CTA
                    if (has_cols && (cq >> 1) == half) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) stgf[((cq & 1) * 32 + j) * kMxTPitchF + r] = __uint_as_float(v0[j]);
                    }
                    named_bar_sync(1, kMxEpiThreads);
                    const int tok = half * 64 + tl;
                    const float4* src = reinterpret_cast<const float4*>(stgf + tl * kMxTPitchF + pc * 16);
                    const float4 x0 = src[0], x1 = src[1], x2 = src[2], x3 = src[3];
                    float amax = fmaxf(fmaxf(fmaxf(fabsf(x0.x), fabsf(x0.y)), fmaxf(fabsf(x0.z), fabsf(x0.w))),
                                       fmaxf(fmaxf(fabsf(x1.x), fabsf(x1.y)), fmaxf(fabsf(x1.z), fabsf(x1.w))));
                    amax = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(x2.x), fabsf(x2.y)), fmaxf(fabsf(x2.z), fabsf(x2.w))),
                                             fmaxf(fmaxf(fabsf(x3.x), fabsf(x3.y)), fmaxf(fabsf(x3.z), fabsf(x3.w)))));
                    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
                    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
                    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 4));
                    float scale, inv;
                    ue8m0_scale(amax, scale, inv);
                    if (tok < rows && row0 + tok < p.a_rows) {
                        uint4 o;
                        o.x = pack_e4m3x4(x0.x * inv, x0.y * inv, x0.z * inv, x0.w * inv);
                        o.y = pack_e4m3x4(x1.x * inv, x1.y * inv, x1.z * inv, x1.w * inv);
                        o.z = pack_e4m3x4(x2.x * inv, x2.y * inv, x2.z * inv, x2.w * inv);
                        o.w = pack_e4m3x4(x3.x * inv, x3.y * inv, x3.z * inv, x3.w * inv);
                        const size_t orow = static_cast<size_t>(row0 + tok);
                        *reinterpret_cast<uint4*>(p.act_q + orow * ia + nt * 128 + pc * 16) = o;
                        if (pc == 0) p.act_s[orow * (ia / 128) + nt] = scale;
                    }
                    named_bar_sync(1, kMxEpiThreads);  // the staging area may be overwritten
                }
            } else if (p.mode == 1) {
                // SwiGLU on matching gate/up columns, then 1x128 fp8 requantisation (power-of-two scale).
                const int ia = p.n_dim / 2;
                float act[32];
                float amax = 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float g = __uint_as_float(v0[j]);
                    act[j] = (g / (1.f + expf(-g))) * __uint_as_float(v1[j]);
                    amax = fmaxf(amax, fabsf(act[j]));
                }
                float* xch = s_amax + (tcount & 1u) * 512;
                xch[cq * 128 + r] = amax;
                named_bar_sync(1, kMxEpiThreads);
                amax = fmaxf(fmaxf(xch[r], xch[128 + r]), fmaxf(xch[256 + r], xch[384 + r]));
                float scale, inv;
                ue8m0_scale(amax, scale, inv);
                if (valid) {
                    uint8_t* dst = p.act_q + static_cast<size_t>(grow) * ia + nt * 128 + cq * 32;
#pragma unroll
                    for (int j = 0; j < 32; j += 16) {
                        uint4 o;
                        o.x = pack_e4m3x4(act[j + 0] * inv, act[j + 1] * inv, act[j + 2] * inv, act[j + 3] * inv);
                        o.y = pack_e4m3x4(act[j + 4] * inv, act[j + 5] * inv, act[j + 6] * inv, act[j + 7] * inv);
                        o.z = pack_e4m3x4(act[j + 8] * inv, act[j + 9] * inv, act[j + 10] * inv, act[j + 11] * inv);
                        o.w = pack_e4m3x4(act[j + 12] * inv, act[j + 13] * inv, act[j + 14] * inv, act[j + 15] * inv);
                        *reinterpret_cast<uint4*>(dst + j) = o;
                    }
                    if (cq == 0) p.act_s[static_cast<size_t>(grow) * (ia / 128) + nt] = scale;
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
                // Half a tile (128 columns) at a time goes through shared memory as bf16 and leaves as
                // 256-byte row segments: 16 lanes store one row, so a warp instruction writes two whole
                // segments (local or over NVLink) instead of 16-byte pieces of 32 different rows.  The row's
                // destination address travels in the 16 spare bytes at the end of its staging row.
                auto push_half = [&](const uint32_t (&v)[32], int c0) {
                    // with two staging buffers the copies of the previous half may still be reading theirs
                    uint8_t* sbuf = stg + (NSTG == 2 ? (halves & 1u) * kMxStgBytes : 0u);
                    uint8_t* srow = sbuf + r * kMxStgPitch;
                    ++halves;
                    if (p.bulk_push && cq == 0) bulk_wait_group_read<NSTG - 1>();  // the copies that read this buffer are done with it
                    named_bar_sync(1, kMxEpiThreads);  // the half that used this buffer has left it
                    if constexpr (SWAP) {
                        // transposed tile: this lane's feature r of tokens cq*32.., one bf16 per staging row
                        if (has_cols) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                *reinterpret_cast<__nv_bfloat16*>(sbuf + (cq * 32 + j) * kMxStgPitch + r * 2) =
                                    __float2bfloat16_rn(__uint_as_float(v[j]));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += 8)
                            *reinterpret_cast<uint4*>(srow + cq * 64 + j * 2) =
                                pack_bf16x8(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                            __uint_as_float(v[j + 3]), __uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]),
                                            __uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                    }
                    if (cq == 0)
                        *reinterpret_cast<uint64_t*>(srow + 256) =
                            (orow != nullptr) ? reinterpret_cast<uint64_t>(orow + c0) : 0ull;
                    if (p.bulk_push) {  // alternative: one 256-byte bulk copy per row, issued by the row's first thread
                        fence_proxy_async_smem();
                        named_bar_sync(1, kMxEpiThreads);
                        if (cq == 0) {
                            if (orow != nullptr) bulk_store_s2g(orow + c0, srow, 256);
                            bulk_commit_group();
                        }
                        return;
                    }
                    named_bar_sync(1, kMxEpiThreads);
                    const int seg = static_cast<int>(lane & 15u) * 16;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint8_t* src = sbuf + (ew * 8 + 2 * i + static_cast<int>(lane >> 4)) * kMxStgPitch;
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
        if (p.bulk_push && cq == 0) bulk_wait_group<0>();  // every row this thread sent has been written
        if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 2, static_cast<int>(tcount));
    }

    // ------------------------------------------------------------------ teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kMxTmemCols);
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

extern "C" int cam_grouped_gemm_mx_smem_bytes(void) { return cam::kMxSmem; }

namespace {
template <bool SWAP, int NS, int NSTG>
int launch_mx(const cam::GroupedGemmParams* p, const CUtensorMap* tmap_a, const CUtensorMap* tmap_b, int grid,
              cudaStream_t stream) {
    static cam::SmemLimitCache limit;
    constexpr int smem = cam::mx_smem<NS, NSTG>();
    cudaError_t e = limit.ensure(cam::grouped_gemm_mxfp8_kernel<SWAP, NS, NSTG>, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    cam::grouped_gemm_mxfp8_kernel<SWAP, NS, NSTG><<<grid, cam::kMxThreads, smem, stream>>>(*tmap_a, *tmap_b, *p);
    return static_cast<int>(cudaGetLastError());
}
}  // namespace

// `swap`: operands exchanged (weights as the M operand), the form for experts of about one tile of rows or less.
// `two_staging` (mode 2 only): two staging buffers in the combine-send epilogue, three pipeline stages.
extern "C" int cam_launch_grouped_gemm_mxfp8(const cam::GroupedGemmParams* p, const CUtensorMap* tmap_a,
                                             const CUtensorMap* tmap_b, int grid, int swap, int two_staging,
                                             cudaStream_t stream) {
    const bool send = two_staging && p->mode == 2;
    if (swap) return send ? launch_mx<true, cam::kMxStagesSend, 2>(p, tmap_a, tmap_b, grid, stream)
                          : launch_mx<true, cam::kStages, 1>(p, tmap_a, tmap_b, grid, stream);
    return send ? launch_mx<false, cam::kMxStagesSend, 2>(p, tmap_a, tmap_b, grid, stream)
                : launch_mx<false, cam::kStages, 1>(p, tmap_a, tmap_b, grid, stream);
}
