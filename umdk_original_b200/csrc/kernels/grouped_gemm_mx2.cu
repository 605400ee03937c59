// CTA-pair version of the block-scaled grouped GEMM (grouped_gemm_mx.cu): a cluster of two CTAs
// works on a 256-row x 256-column tile with ONE tcgen05.mma.cta_group::2 stream issued by the
// pair's first CTA.  Every CTA keeps its own 128 rows of A and HALF of the B tile (128 of the 256
// weight rows: the gate half in the first CTA, the up half in the second for the SwiGLU GEMM) in
// shared memory, so a weight tile crosses L2 -> SM once per pair and a pipeline stage is 32 KiB
// instead of 48 KiB, which buys six stages.  This is how the kernel shares weight tiles inside a
// thread-block cluster; no load carries a multicast qualifier (each CTA issues plain TMA loads of
// its own pieces, counted on the first CTA's mbarrier through the cta_group::2 form of the load).
//
// Used when experts have enough rows to fill 256-row tiles (the runtime picks it from the mean
// rows per local expert); the one-CTA kernel stays for small experts.
//
// Barriers.  In the first CTA: full[s] (the bytes of both CTAs' loads), sf[s] (scale factors of
// both CTAs are in their TMEM: 4 + 4 warp arrivals), tempty (both CTAs drained their accumulator:
// 16 + 16 warp arrivals).  In each CTA: empty[s] and tfull, raised by tcgen05.commit from the
// first CTA once the MMAs that read a stage / complete a tile have retired in both CTAs.
// Both CTAs always reach the cluster barrier at the end, also after a timed-out wait.
#include "gemm_common.cuh"

namespace cam {

constexpr int kP2Threads = 768;
constexpr int kP2EpiThreads = 512;
constexpr int kP2SfWarp0 = 4, kP2EpiWarp0 = 8;
constexpr int kP2Stages = 6;        // modes 0 / 1
constexpr int kP2StagesSend = 4;    // mode 2 with two staging buffers
constexpr int kP2ATile = BM * BK;          // this CTA's 128 rows of A, 16 KiB
constexpr int kP2BTile = 128 * BK;         // this CTA's half of the 256-row B tile, 16 KiB
constexpr int kP2StageBytes = kP2ATile + kP2BTile;
// Shared memory: 6 pipeline stages | bf16 staging of half an output tile (128 rows x 256 bytes,
// rows 272 bytes apart so that 16-byte stores of neighbouring rows fall into different banks; the
// per-row amax exchange of the SwiGLU epilogue uses the same bytes) | barriers.  232448 bytes, the
// whole 227 KiB a CTA can have, so the dynamic segment must start on a 1024-byte boundary.
constexpr int kP2StgPitch = 272;
constexpr int kP2StgBytes = BM * kP2StgPitch;  // 34816
constexpr int kP2SmemCtrl = 1024;
// The combine-send epilogue (mode 2) is bound by how fast its rows leave over NVLink.  With one staging buffer the
// epilogue cannot convert the next half tile while the copies of the previous one are still reading shared memory,
// and the link idles in between; the send form of the kernel therefore has TWO staging buffers and pays for them
// with two pipeline stages (its reduction is short, K = intermediate size, and the mainloop has slack there).
template <int NS, int NSTG>
constexpr int p2_smem() { return NS * kP2StageBytes + NSTG * kP2StgBytes + kP2SmemCtrl; }
constexpr int kP2Smem = p2_smem<kP2Stages, 1>();
static_assert(kP2Smem <= 232448 && p2_smem<kP2StagesSend, 2>() <= 232448, "exceeds the shared memory of one CTA");
constexpr uint32_t kP2TmemCols = 512;
constexpr uint32_t kP2SfCol0 = 256, kP2SfStride = 16;
// Register re-partitioning (setmaxnreg): the CTA is launched with kP2LaunchRegs per thread (what
// ptxas reports for this kernel); the control and scale-factor warp-groups give registers back
// and the four epilogue warp-groups take them.  setmaxnreg.inc waits for the CTA's pool without
// any time limit, so the sum below must not exceed what the CTA owns.
constexpr uint32_t kP2LaunchRegs = 80, kP2CtrlRegs = 32, kP2SfRegs = 56, kP2EpiRegs = 96;
static_assert(128 * kP2CtrlRegs + 128 * kP2SfRegs + kP2EpiThreads * kP2EpiRegs <= kP2LaunchRegs * kP2Threads,
              "setmaxnreg budget exceeds the registers the CTA owns: the kernel would hang");

template <int NS, int NSTG>
__global__ void __launch_bounds__(kP2Threads, 1)
grouped_gemm_mxfp8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const GroupedGemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {  // swizzled TMA tiles need it; nothing has been set up yet, so just leave
        if (threadIdx.x == 0) gemm_record_status(p.status, CAM_ERR_BAD_INDEX, 4, static_cast<int>(smem_u32(smem) & 1023u));
        return;
    }
    uint8_t* stg = smem + NS * kP2StageBytes;
    uint8_t* ctrl = stg + NSTG * kP2StgBytes;
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(ctrl);   // first CTA: TMA bytes of both CTAs' stage have landed
    uint64_t* bar_sf = bar_full + NS;                  // first CTA: scale factors of both CTAs are in TMEM
    uint64_t* bar_empty = bar_sf + NS;                 // each CTA: the MMAs that read a stage have retired
    uint64_t* bar_tfull = bar_empty + NS;              // each CTA: accumulator of a tile is complete
    uint64_t* bar_tempty = bar_tfull + 1;                     // first CTA: both accumulators have been drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* s_amax = reinterpret_cast<float*>(stg);  // mode 1 only: [2 parities][4 column quarters][128 rows]

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const uint32_t lane = lane_id();
    const uint32_t cta = cluster_cta_rank();                  // 0 = first CTA of the pair (issues the MMAs)
    const int pair_id = static_cast<int>(blockIdx.x) >> 1;
    const int num_pairs = static_cast<int>(gridDim.x) >> 1;
    const int kblocks = p.k_dim / BK;
    // combine-send form: this rank starts every expert's row blocks at its own offset (see TileWalkerT::locate)
    const int rot_num = (p.mode == 2 && p.num_ranks > 1) ? p.rank : 0, rot_den = (p.mode == 2 && p.num_ranks > 1) ? p.num_ranks : 0;
    const int n_tiles = (p.mode == 1) ? (p.n_dim / 2) / 128 : (p.n_dim + BN - 1) / BN;
    const int nblk = p.n_dim / 128;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_sf[s], 8);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(bar_tfull, 1);
        mbar_init(bar_tempty, 2 * (kP2EpiThreads / 32));
        *abort_flag = 0u;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, kP2TmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers are initialised before anything signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < kP2SfWarp0) {
        reg_dealloc<kP2CtrlRegs>();
        if (warp == 0 && lane == 0) {
            // ------------------------------------------------------------ TMA producer (both CTAs)
            prefetch_tensormap(&tmap_a);
            prefetch_tensormap(&tmap_b);
            TileWalkerT<2 * BM> w(p.expert_offsets, p.num_experts, n_tiles);
            uint32_t it = 0;
            int e, mt, nt, row0, rows;
            bool ok = true;
            for (int tile = pair_id; ok && w.locate(tile, e, mt, nt, row0, rows, rot_num, rot_den); tile += num_pairs) {
                const int brow_lo = e * p.n_dim + ((p.mode == 1) ? nt * 128 : nt * BN);
                const int brow_hi = (p.mode == 1) ? (e * p.n_dim + p.n_dim / 2 + nt * 128) : (brow_lo + 128);
                const int my_arow = row0 + static_cast<int>(cta) * BM;
                const int my_brow = cta ? brow_hi : brow_lo;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const uint32_t s = it % NS, ph = (it / NS) & 1u;
                    if (!mbar_wait_bounded(&bar_empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    uint8_t* sa = smem + s * kP2StageBytes;
                    if (cta == 0) mbar_arrive_expect_tx(&bar_full[s], 2 * kP2StageBytes);
                    const uint32_t full0 = map_to_cta(&bar_full[s], 0);
                    tma_load_2d_pair(sa, &tmap_a, full0, kb * BK, my_arow);
                    tma_load_2d_pair(sa + kP2ATile, &tmap_b, full0, kb * BK, my_brow);
                }
            }
            if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 0, static_cast<int>(it));
        } else if (warp == 1 && lane == 0 && cta == 0) {
            // ------------------------------------------------------------ MMA issuer (first CTA only)
            constexpr uint32_t idesc = umma_idesc_mxf8(2 * BM, BN);
            TileWalkerT<2 * BM> w(p.expert_offsets, p.num_experts, n_tiles);
            uint32_t it = 0, tcount = 0;
            int e, mt, nt, row0, rows;
            bool ok = true;
            const uint32_t tfull0 = map_to_cta(bar_tfull, 0), tfull1 = map_to_cta(bar_tfull, 1);
            for (int tile = pair_id; ok && w.locate(tile, e, mt, nt, row0, rows, rot_num, rot_den); tile += num_pairs, ++tcount) {
                // both epilogues must have drained the previous tile before its columns are overwritten
                if (!mbar_wait_bounded(bar_tempty, (tcount & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const uint32_t s = it % NS, ph = (it / NS) & 1u;
                    if (!mbar_wait_bounded(&bar_sf[s], ph, abort_flag)) { ok = false; break; }
                    if (!mbar_wait_bounded(&bar_full[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * kP2StageBytes);
                    const uint64_t adesc = umma_desc_k_sw128(sa);
                    const uint64_t bdesc = umma_desc_k_sw128(sa + kP2ATile);
                    const uint32_t sfa = tmem_base + kP2SfCol0 + s * kP2SfStride;
                    const uint32_t sfb = sfa + 4u;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)  // 32 bytes (= 2 x 16) further along K inside the swizzle atom
                        tc_mma_mxf8_pair(tmem_base, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) ? 1u : 0u, sfa, sfb);
                    // the stage (smem and scale columns, in both CTAs) is reusable once these MMAs retire
                    tc_commit_pair(map_to_cta(&bar_empty[s], 0));
                    tc_commit_pair(map_to_cta(&bar_empty[s], 1));
                }
                if (!ok) break;
                tc_commit_pair(tfull0);  // accumulators complete once every MMA of the tile has retired
                tc_commit_pair(tfull1);
            }
            if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 1, static_cast<int>(it));
        }
    } else if (warp < kP2EpiWarp0) {
        reg_dealloc<kP2SfRegs>();
        // ---------------------------------------------------------------- scale-factor writers
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        TileWalkerT<2 * BM> w(p.expert_offsets, p.num_experts, n_tiles);
        uint32_t it = 0;
        int e, mt, nt, row0, rows;
        bool ok = true;
        // rows of scales can be read 16 bytes at a time when K is a multiple of 512 and the arrays are aligned
        const bool vec_scales = (kblocks & 3) == 0 &&
                                ((reinterpret_cast<uintptr_t>(p.a_scales) | reinterpret_cast<uintptr_t>(p.b_scales)) & 15u) == 0u;
        for (int tile = pair_id; ok && w.locate(tile, e, mt, nt, row0, rows, rot_num, rot_den); tile += num_pairs) {
            const float* as[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // this CTA's 128 rows of the 256-row tile
                const int r = min(row0 + static_cast<int>(cta) * BM + 32 * j + static_cast<int>(lane), p.a_rows - 1);
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
                const uint32_t col = tmem_base + lane_base + kP2SfCol0 + s * kP2SfStride;
                tmem_st_32x32b_x4(col, w0, w1, w2, w3);
                tmem_st_32x32b_x4(col + 4u, w4, w4, w4, w4);
                tmem_st_32x32b_x4(col + 8u, w5, w5, w5, w5);
                tc_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {  // the first CTA's barrier counts the warps of both CTAs
                    if (cta == 0) mbar_arrive(&bar_sf[s]);
                    else mbar_arrive_cluster(map_to_cta(&bar_sf[s], 0));
                }
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
        reg_alloc<kP2EpiRegs>();
        // ---------------------------------------------------------------- epilogue warps
        const int ew = warp - kP2EpiWarp0;
        const int q = warp & 3;   // TMEM lane quarter this warp may read
        const int cq = ew >> 2;   // which 32-column quarter of each 128-column half
        const int r = q * 32 + static_cast<int>(lane);
        TileWalkerT<2 * BM> w(p.expert_offsets, p.num_experts, n_tiles);
        uint32_t tcount = 0, halves = 0;
        int e, mt, nt, row0, rows;
        bool ok = true;
        for (int tile = pair_id; ok && w.locate(tile, e, mt, nt, row0, rows, rot_num, rot_den); tile += num_pairs, ++tcount) {
            row0 += static_cast<int>(cta) * BM;            // this CTA's half of the 256-row tile
            rows = max(0, min(BM, rows - static_cast<int>(cta) * BM));
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
            if (lane == 0) {
                if (cta == 0) mbar_arrive(bar_tempty);
                else mbar_arrive_cluster(map_to_cta(bar_tempty, 0));
            }

            if (p.mode == 1) {
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
                named_bar_sync(1, kP2EpiThreads);
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
                    uint8_t* sbuf = stg + (NSTG == 2 ? (halves & 1u) * kP2StgBytes : 0u);
                    uint8_t* srow = sbuf + r * kP2StgPitch;
                    ++halves;
                    if (p.bulk_push && cq == 0) bulk_wait_group_read<NSTG - 1>();  // the copies that read this buffer are done with it
                    named_bar_sync(1, kP2EpiThreads);  // the half that used this buffer has left it
#pragma unroll
                    for (int j = 0; j < 32; j += 8)
                        *reinterpret_cast<uint4*>(srow + cq * 64 + j * 2) =
                            pack_bf16x8(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                        __uint_as_float(v[j + 3]), __uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]),
                                        __uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                    if (cq == 0)
                        *reinterpret_cast<uint64_t*>(srow + 256) =
                            (orow != nullptr) ? reinterpret_cast<uint64_t>(orow + c0) : 0ull;
                    if (p.bulk_push) {  // alternative: one 256-byte bulk copy per row, issued by the row's first thread
                        fence_proxy_async_smem();
                        named_bar_sync(1, kP2EpiThreads);
                        if (cq == 0) {
                            if (orow != nullptr) bulk_store_s2g(orow + c0, srow, 256);
                            bulk_commit_group();
                        }
                        return;
                    }
                    named_bar_sync(1, kP2EpiThreads);
                    const int seg = static_cast<int>(lane & 15u) * 16;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint8_t* src = sbuf + (ew * 8 + 2 * i + static_cast<int>(lane >> 4)) * kP2StgPitch;
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
    cluster_sync_all();  // the other CTA may still read this CTA's shared memory or signal its barriers
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kP2TmemCols);
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

extern "C" int cam_grouped_gemm_mx_pair_smem_bytes(void) { return cam::kP2Smem; }

namespace {

template <int NS, int NSTG>
void pair_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int grid, cudaStream_t stream) {
    cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid & ~1));  // whole pairs only
    cfg.blockDim = dim3(cam::kP2Threads);
    cfg.dynamicSmemBytes = cam::p2_smem<NS, NSTG>();
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
}

// Number of CTA pairs of one form of the kernel that can be resident on the current device at once (cached per device).
template <int NS, int NSTG>
int pair_max_clusters() {
    static cam::SmemLimitCache limit;
    if (limit.ensure(cam::grouped_gemm_mxfp8_pair_kernel<NS, NSTG>, cam::p2_smem<NS, NSTG>()) != cudaSuccess) return -1;
    static int max_pairs[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    if (max_pairs[dev] == 0) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        pair_config<NS, NSTG>(cfg, attr, 2, nullptr);
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, cam::grouped_gemm_mxfp8_pair_kernel<NS, NSTG>, &cfg) == cudaSuccess && n > 0)
            max_pairs[dev] = n;
        else
            max_pairs[dev] = -1;
    }
    return max_pairs[dev];
}

template <int NS, int NSTG>
int launch_pair(const cam::GroupedGemmParams* p, const CUtensorMap* tmap_a, const CUtensorMap* tmap_b, int grid,
                cudaStream_t stream) {
    // Not every SM can always be paired inside its GPC: run exactly as many pairs as fit at once.
    const int fit = pair_max_clusters<NS, NSTG>();
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    pair_config<NS, NSTG>(cfg, attr, grid, stream);
    if (fit > 0 && 2 * fit < static_cast<int>(cfg.gridDim.x)) cfg.gridDim = dim3(static_cast<unsigned>(2 * fit));
    return static_cast<int>(cudaLaunchKernelEx(&cfg, cam::grouped_gemm_mxfp8_pair_kernel<NS, NSTG>, *tmap_a, *tmap_b, *p));
}

}  // namespace

extern "C" int cam_grouped_gemm_mx_pair_max_clusters(void) { return pair_max_clusters<cam::kP2Stages, 1>(); }

// `two_staging` selects the send form (mode 2 only): two staging buffers, four pipeline stages.
extern "C" int cam_launch_grouped_gemm_mxfp8_pair(const cam::GroupedGemmParams* p, const CUtensorMap* tmap_a,
                                                  const CUtensorMap* tmap_b, int grid, int two_staging,
                                                  cudaStream_t stream) {
    if (two_staging && p->mode == 2) return launch_pair<cam::kP2StagesSend, 2>(p, tmap_a, tmap_b, grid, stream);
    return launch_pair<cam::kP2Stages, 1>(p, tmap_a, tmap_b, grid, stream);
}
