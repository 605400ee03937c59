// Deep-fused MoE layer for sm_100a: ONE persistent kernel of CTA pairs that
//   * sends this rank's quantised tokens to their expert ranks, in the order of the destination's
//     local experts, and counts every landed row on a per-expert arrival counter in the
//     destination's memory (bulk copies through a small ring in shared memory, driven by one thread
//     per CTA, beside the tensor-core pipeline);
//   * runs the first grouped GEMM (+ SwiGLU + 1x128 fp8 requantisation) of a local expert as soon
//     as that expert's counter says all of its rows are in, while later experts still arrive;
//   * runs the second grouped GEMM of a row block as soon as the first one has finished that
//     block, and pushes its bf16 rows from the epilogue straight into the combine slots of the
//     tokens' origin ranks (bulk copies shared memory -> peer memory).
// Tiles of the two GEMMs are interleaved expert by expert (the second GEMM of expert e follows the
// first GEMM of expert e + lag), so the combine traffic is spread over the whole compute time
// instead of being squeezed into the second GEMM.
//
// This is the B200 form of the reference's deep-fused kernel: there the cube core spins on a
// per-expert token counter before it starts that expert
// (fused_deep_moe/gemm/kernel/grouped_matmul_slice_m_per_token_dequant_swiglu_quant_multistage_workspace.h:558-574),
// senders emit tokens in local-expert order (:948-961), receivers add per-expert counts (:1259-1274)
// and the second GEMM's epilogue is the combine send
// (fused_deep_moe/epilogue/block/block_epilogue_per_token_dequant.hpp:531-570).
//
// Tensor-core pipeline, barriers and epilogues are those of the CTA-pair grouped GEMM
// (grouped_gemm_mx2.cu): tcgen05.mma.cta_group::2 with UE8M0 block scaling, operands by plain TMA
// loads (no multicast qualifier anywhere), accumulators in TMEM.  Warps: 0 TMA producer, 1 MMA
// issuer (first CTA of the pair), 2 dispatch sender, 4-7 scale-factor writers, 8-23 epilogue.  The sender is one
// thread that moves the dispatch rows with the bulk-copy engine (this rank's quantised token -> a ring in shared
// memory -> the destination rank's receive buffer), so that the rows cost the other warps neither issue slots nor
// load/store bandwidth.
//
// Every wait is bounded.  A wait that runs out records a status word, raises the CTA's abort flag
// (and the partner CTA's), and every role leaves its loop; both CTAs always reach the cluster
// barrier at the end and free their tensor memory.
#include "gemm_common.cuh"

namespace cam {

constexpr int kFmThreads = 768;
constexpr int kFmEpiThreads = 512;
constexpr int kFmSfWarp0 = 4, kFmEpiWarp0 = 8;
constexpr int kFmStagesSend = 5, kFmStagesGemm = 6;
constexpr int kFmATile = BM * BK;    // this CTA's 128 rows of A, 16 KiB
constexpr int kFmBTile = 128 * BK;   // this CTA's half of the 256-row B tile, 16 KiB
constexpr int kFmStageBytes = kFmATile + kFmBTile;
constexpr int kFmStgPitch = 272;
constexpr int kFmStgBytes = BM * kFmStgPitch;  // 34816: bf16 staging of half an output tile (combine-send epilogue)
// arrivals on a g1_done counter per 128-column tile of the first GEMM: every epilogue warp of both CTAs
constexpr int kFmG1Signals = 2 * (kFmEpiThreads / 32);
// The sender's ring: kFmSendSlots rows in flight (a row of at most 7168 e4m3 values followed by its scales).
constexpr int kFmSendSlots = 4;
constexpr int kFmSendRowMax = 7168;
constexpr int kFmSendSlotBytes = kFmSendRowMax + 256;
constexpr int kFmSendAhead = 1;                // rows whose load is issued before the previous row's stores
constexpr int kFmCommBatch = 16;               // rows of one run of the send list, counted with one release
constexpr int kFmSmemCtrl = 1024;
// five pipeline stages | one staging buffer | the sender's ring | barriers
template <int NS>
constexpr int fm_smem() {
    return NS * kFmStageBytes + kFmStgBytes + (NS == kFmStagesSend ? kFmSendSlots * kFmSendSlotBytes : 0) + kFmSmemCtrl;
}
constexpr int kFmSmem = fm_smem<kFmStagesGemm>();  // the larger of the two
static_assert(fm_smem<kFmStagesSend>() <= kFmSmem && kFmSmem <= 232448, "exceeds the shared memory of one CTA");
constexpr uint32_t kFmTmemCols = 512;
constexpr uint32_t kFmSfCol0 = 256, kFmSfStride = 16;
// Register re-partitioning, see grouped_gemm_mx2.cu: the launch count is what ptxas reports.
constexpr uint32_t kFmLaunchRegs = 80, kFmCtrlRegs = 40, kFmSfRegs = 80, kFmEpiRegs = 88;
static_assert(128 * kFmCtrlRegs + 128 * kFmSfRegs + kFmEpiThreads * kFmEpiRegs <= kFmLaunchRegs * kFmThreads,
              "setmaxnreg budget exceeds the registers the CTA owns: the kernel would hang");

// Activation scales are read through L1 although other SMs or GPUs write them during this kernel.  Every warp that
// reads a row has itself acquired the counter that says the row is complete (a system- or GPU-scope acquire load, after
// which its ordinary loads must observe the released stores, whichever cache operator they carry), and rows outside
// the tile's valid range are not read at all.  The asm is volatile so that the compiler cannot move the load above
// the acquire.
__device__ __forceinline__ float4 ld_ca_v4f32(const float4* p) {
    float4 v;
    asm volatile("ld.global.ca.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// Order of the tiles of one launch.  Step j of the walk holds the first GEMM of expert j (while j < E_local) and
// then the second GEMM of expert j - lag (once j >= lag).  `tile` must not decrease from call to call.
struct FusedWalker {
    int j = 0, sub = 0, base = 0;  // everything else comes from the kernel parameters (constant bank, no registers)
    // kind 0 = first GEMM, 1 = second GEMM; cnt = rows of the expert.
    __device__ __forceinline__ bool locate(const FusedMoeParams& p, int tile, int& kind, int& e_out, int& mt, int& nt,
                                           int& row0, int& rows, int& cnt_out) {
        const int num_experts = p.num_experts, lag = p.lag;
        while (j < num_experts + lag) {
            const int e = sub ? j - lag : j;
            const bool has = sub ? (j >= lag) : (j < num_experts);
            int first = 0, cnt = 0, tiles = 0;
            const int per = sub ? (p.h + BN - 1) / BN : p.inter / 128;
            if (has) {
                first = __ldg(p.expert_offsets + e);
                cnt = __ldg(p.expert_offsets + e + 1) - first;
                tiles = ((cnt + 2 * BM - 1) / (2 * BM)) * per;
            }
            if (tile < base + tiles) {
                const int local = tile - base;
                mt = local / per;
                nt = local - mt * per;
                if (sub && p.num_ranks > 1) {
                    // second GEMM: this rank starts the expert's row blocks (ordered by origin rank) at its own offset, so
                    // that the ranks of the group push their combine rows to different origins at any one time
                    const int blocks = (cnt + 2 * BM - 1) / (2 * BM);
                    mt += p.rank * blocks / p.num_ranks;
                    if (mt >= blocks) mt -= blocks;
                }
                row0 = first + mt * 2 * BM;
                rows = min(2 * BM, cnt - mt * 2 * BM);
                e_out = e;
                kind = sub;
                cnt_out = cnt;
                return true;
            }
            base += tiles;
            if (sub) { sub = 0; ++j; } else { sub = 1; }
        }
        return false;
    }
};

// What a wait needs when it does not succeed at once.  One copy per CTA in shared memory, so that the roles (above all
// the single threads that issue TMA loads and MMAs) hold one pointer instead of a dozen registers.
struct FmWait {
    volatile uint32_t abort_flag;   // raised by any role of this CTA (or of the partner CTA) that gave up
    uint32_t partner_abort;         // cluster address of the partner's abort flag
    const volatile int* status_code;
    // absolute times (globaltimer) at which the waits of this launch give up
    uint64_t deadline_arrival;  // for another GPU's rows: launch + the budget the caller set
    uint64_t deadline_gemm1;    // for the first GEMM of a row block, which itself may wait for arrivals: a second later
    uint64_t deadline_pipe;     // inside the pipeline, behind both: another second later
};

__device__ __forceinline__ void fm_raise_abort(FmWait* w) {
    w->abort_flag = 1u;
    st_shared_cluster_u32(w->partner_abort, 1u);
}

// mbarrier wait that also gives up when any CTA of the launch has recorded an error.
// A wait first tries once.  The loop behind it is kept to a handful of instructions (the loop bodies of the producer,
// the MMA issuer and the scale-factor writers share a scheduler's instruction cache): every 4096 unsuccessful tries it
// looks at the abort flag, at the status word of the launch and at the deadline.
__device__ __forceinline__ bool fm_give_up(FmWait* w, uint64_t deadline) {
    if (w->abort_flag) return true;
    if (*w->status_code != 0 || globaltimer_ns() > deadline) {
        fm_raise_abort(w);
        return true;
    }
    return false;
}
__device__ __forceinline__ bool fm_mbar_wait(uint64_t* bar, uint32_t parity, FmWait* w) {
    if (mbar_try_wait(bar, parity)) return true;
    uint32_t polls = 0;
    while (!mbar_try_wait(bar, parity))
        if ((++polls & 4095u) == 0u && fm_give_up(w, w->deadline_pipe)) return false;
    return true;
}
// for the epilogue warps, which wait a whole tile: sleeps between tries
__device__ __forceinline__ bool fm_mbar_wait_sleep(uint64_t* bar, uint32_t parity, FmWait* w) {
    if (mbar_try_wait(bar, parity)) return true;
    uint32_t polls = 0;
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(256);
        if ((++polls & 255u) == 0u && fm_give_up(w, w->deadline_pipe)) return false;
    }
    return true;
}

// Spin until *ctr >= want.  SYS: the counter is written by other GPUs.  Called by single threads or whole warps.
template <bool SYS>
__device__ __forceinline__ bool fm_wait_counter(const uint32_t* ctr, uint32_t want, FmWait* w, uint32_t& seen) {
    seen = SYS ? ld_acquire_sys_u32(ctr) : ld_acquire_gpu_u32(ctr);
    if (seen >= want) return true;
    const uint64_t deadline = SYS ? w->deadline_arrival : w->deadline_gemm1;
    uint32_t polls = 0;
    while (true) {
        seen = SYS ? ld_acquire_sys_u32(ctr) : ld_acquire_gpu_u32(ctr);
        if (seen >= want) return true;
        __nanosleep(100);
        if ((++polls & 31u) == 0u) {
            if (w->abort_flag) return false;
            if (*w->status_code != 0 || globaltimer_ns() > deadline) return false;
        }
    }
}

// Dispatch send.  One thread per CTA walks its share of the expert-ordered send list and moves every row with three bulk copies: token and scales from this rank's quantised copy into a ring slot in
// shared memory (counted on the slot's mbarrier), then both out of the slot into the destination rank's receive buffer.
// The (rank, token, k) triple of the row goes by plain stores.  Up to kFmSendSlots rows are in flight.  A row is counted
// on the arrival counter of its expert at the destination once its stores are complete (cp.async.bulk.wait_group
// leaves only the newest groups pending), with a system-scope release; rows of one (rank, expert) are counted together,
// kFmCommBatch at most.
struct FmSender {
    const FusedMoeParams& p;
    FmWait* wt;
    uint8_t* ring;       // kFmSendSlots x kFmSendSlotBytes
    uint64_t* bar;       // [kFmSendSlots]
    int4* meta;          // [kFmSendSlots] list entries of the rows in the slots
    uint64_t off_arrival;  // of this call's parity
    int pend_d = -1, pend_le = 0, pend_n = 0;

    __device__ void flush() {
        if (pend_n > 0 && p.dbg_drop_flags == 0) {  // drop: host-side fault injection, the rows are never counted
            uint32_t* ctr = reinterpret_cast<uint32_t*>(p.peer_base[pend_d] + off_arrival) + pend_le;
            // Rows that stay on this GPU are released at GPU scope: a system-scope release also waits for the path to
            // the host, which is slow while copies between host and device are running.
            if (pend_d == p.rank) red_release_gpu_add_u32(ctr, static_cast<uint32_t>(pend_n));
            else red_release_sys_add_u32(ctr, static_cast<uint32_t>(pend_n));
        }
        pend_n = 0;
    }
    __device__ void count(const int4& ent) {
        const int d = ent.y, le = ent.w & 0xFFFF;
        if (pend_n > 0 && (d != pend_d || le != pend_le || pend_n >= kFmCommBatch)) flush();
        pend_d = d;
        pend_le = le;
        ++pend_n;
    }
    __device__ void run() {
        constexpr int kPend = kFmSendSlots - 1 - kFmSendAhead;  // store groups that may stay pending when a slot is reused
        const int nlist = min(p.send_list_len[0], p.send_list_cap);
        // The list is dealt out in runs of kFmCommBatch consecutive entries (run q of this CTA is run q * gridDim.x +
        // blockIdx.x of the list): consecutive entries nearly always go to the same (rank, expert), so that one
        // system-scope release counts a whole run.
        const int first = static_cast<int>(blockIdx.x), stride = static_cast<int>(gridDim.x);
        const int runs = (nlist + kFmCommBatch - 1) / kFmCommBatch;
        const int my_runs = first < runs ? (runs - first + stride - 1) / stride : 0;
        int n = my_runs * kFmCommBatch;  // rows of this CTA
        if (my_runs > 0 && (my_runs - 1) * stride + first == runs - 1) n -= runs * kFmCommBatch - nlist;  // the list's last run may be short
        auto entry = [&](int i) { return ((i / kFmCommBatch) * stride + first) * kFmCommBatch + (i % kFmCommBatch); };
        const uint32_t row_bytes = static_cast<uint32_t>(p.h);
        const uint32_t sc_bytes = static_cast<uint32_t>(p.h >> 7) * 4u;  // a multiple of 16: h is a multiple of 512
        bool ok = true;
        int stored = 0, counted = 0;  // rows whose stores were committed / that were counted at their destination
        for (int i = 0; ok && i < n + kFmSendAhead; ++i) {
            if (i < n) {
                // Row i takes the slot of row i - kFmSendSlots.  Rows [0, stored) have their stores committed, and
                // stored = i - kFmSendAhead here, so with kPend groups pending rows up to i - kFmSendSlots are complete:
                // count them (their list entries still sit in `meta`) before the slot is overwritten.
                bulk_wait_group<kPend>();
                for (; counted < stored - kPend; ++counted) count(meta[counted % kFmSendSlots]);
                const int4 ent = p.send_list[entry(i)];
                const int t = ent.x, d = ent.y, row = ent.z;
                if (t < 0 || t >= p.max_tokens || d < 0 || d >= p.num_ranks || row < 0 || row >= p.a_rows) {
                    gemm_record_status(p.status, CAM_ERR_BAD_INDEX, 5, entry(i));
                    ok = false;
                    break;
                }
                const int slot = i % kFmSendSlots;
                meta[slot] = ent;
                uint8_t* sl = ring + slot * kFmSendSlotBytes;
                mbar_arrive_expect_tx(&bar[slot], row_bytes + sc_bytes);
                bulk_load_g2s(sl, p.xq + static_cast<size_t>(t) * p.h, row_bytes, &bar[slot]);
                bulk_load_g2s(sl + kFmSendRowMax, reinterpret_cast<const uint8_t*>(p.xs) + static_cast<size_t>(t) * sc_bytes,
                              sc_bytes, &bar[slot]);
            }
            const int j = i - kFmSendAhead;
            if (j >= 0) {
                const int slot = j % kFmSendSlots;
                if (!fm_mbar_wait_sleep(&bar[slot], static_cast<uint32_t>(j / kFmSendSlots) & 1u, wt)) {
                    gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 4, j);
                    ok = false;
                    break;
                }
                const int4 ent = meta[slot];
                const int t = ent.x, d = ent.y, row = ent.z, kk = ent.w >> 16;
                uint8_t* pb = p.peer_base[d];
                const uint8_t* sl = ring + slot * kFmSendSlotBytes;
                bulk_store_s2g(pb + p.off_recv_x + static_cast<size_t>(row) * p.h, sl, row_bytes);
                bulk_store_s2g(pb + p.off_recv_scales + static_cast<size_t>(row) * p.a1_scale_pitch * 4, sl + kFmSendRowMax,
                               sc_bytes);
                bulk_commit_group();
                int* tri = reinterpret_cast<int*>(pb + p.off_recv_src) + static_cast<size_t>(row) * 3;
                tri[0] = p.rank;
                tri[1] = t;
                tri[2] = kk;
                ++stored;
            }
        }
        // whatever happened, nothing may still read the ring or be in flight when the CTA leaves
        bulk_wait_group<0>();
        for (; counted < stored; ++counted) count(meta[counted % kFmSendSlots]);
        flush();
    }
};

// Unique counter index of the 256-row block that starts at `row0` of local expert `e` (experts own contiguous rows).
__device__ __forceinline__ int fm_block_index(int row0, int e) { return (row0 >> 8) + e; }

// NS pipeline stages.  The form that sends the dispatch rows itself has five and the sender's ring; a launch that only
// runs the GEMMs (the rows were sent before it) has six and no ring.
template <int NS>
__global__ void __launch_bounds__(kFmThreads, 1)
fused_moe_pair_kernel(const __grid_constant__ CUtensorMap tmap_a1, const __grid_constant__ CUtensorMap tmap_b1,
                      const __grid_constant__ CUtensorMap tmap_a2, const __grid_constant__ CUtensorMap tmap_b2,
                      const FusedMoeParams p) {
    constexpr int kSlots = NS == kFmStagesSend ? kFmSendSlots : 0;
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {  // swizzled TMA tiles need it; nothing has been set up yet, so just leave
        if (threadIdx.x == 0) gemm_record_status(p.status, CAM_ERR_BAD_INDEX, 4, static_cast<int>(smem_u32(smem) & 1023u));
        return;
    }
    uint8_t* stg = smem + NS * kFmStageBytes;
    uint8_t* send_ring = stg + kFmStgBytes;
    uint8_t* ctrl = send_ring + kSlots * kFmSendSlotBytes;
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(ctrl);
    uint64_t* bar_sf = bar_full + NS;
    uint64_t* bar_empty = bar_sf + NS;
    uint64_t* bar_tfull = bar_empty + NS;
    uint64_t* bar_tempty = bar_tfull + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 1);
    FmWait* wt = reinterpret_cast<FmWait*>(ctrl + 384);
    uint64_t* bar_send = reinterpret_cast<uint64_t*>(ctrl + 512);   // [kSlots]
    int4* send_meta = reinterpret_cast<int4*>(ctrl + 576);          // [kSlots]
    static_assert(576 + kSlots * 16 <= kFmSmemCtrl && 512 + kSlots * 8 <= 576 && 384 + sizeof(FmWait) <= 512 &&
                      (3 * NS + 2) * 8 + 8 <= 384, "control area layout");
    float* s_amax = reinterpret_cast<float*>(stg);  // first-GEMM epilogue: [2 parities][4 column quarters][128 rows]

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const uint32_t lane = lane_id();
    const uint32_t cta = cluster_cta_rank();
    const int pair_id = static_cast<int>(blockIdx.x) >> 1;
    const int num_pairs = static_cast<int>(gridDim.x) >> 1;
    const bool do_send = (p.phase_mask & CAM_PHASE_SEND) != 0;
    const bool do_gemm = (p.phase_mask & CAM_PHASE_RECV) != 0;
    const int kb1 = p.h / BK, kb2 = p.inter / BK;
    const int nt1 = p.inter / 128;
    const int nblk1 = 2 * p.inter / 128, nblk2 = p.h / 128;
    const uint32_t parity = *p.epoch_dispatch & 1u;  // the first launch of the layer has already advanced it
    const uint32_t* my_arrival = reinterpret_cast<const uint32_t*>(p.peer_base[p.rank] + p.off_arrival) +
                                 static_cast<size_t>(parity) * p.arrival_stride;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_sf[s], 8);
            mbar_init(&bar_empty[s], 1);
        }
        for (int s = 0; s < kSlots; ++s) mbar_init(&bar_send[s], 1);
        mbar_init(bar_tfull, 1);
        mbar_init(bar_tempty, 2 * (kFmEpiThreads / 32));
        wt->abort_flag = 0u;
        wt->partner_abort = map_to_cta(const_cast<uint32_t*>(&wt->abort_flag), cta ^ 1u);
        wt->status_code = &p.status->code;
        wt->deadline_arrival = globaltimer_ns() + p.timeout_ns;
        wt->deadline_gemm1 = wt->deadline_arrival + 1000000000ull;
        wt->deadline_pipe = wt->deadline_arrival + 2000000000ull;
        mbar_fence_init();
        if (blockIdx.x == 0 && p.trace != nullptr) p.trace[p.num_experts] = globaltimer_ns();
    }
    if (do_gemm && warp == 1) {
        tmem_alloc_pair(tmem_slot, kFmTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers are initialised before anything signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = do_gemm ? *tmem_slot : 0u;

    if (warp < kFmSfWarp0) {
        reg_dealloc<kFmCtrlRegs>();
        if (warp == 0 && lane == 0 && do_gemm) {
            // ------------------------------------------------------------ TMA producer (both CTAs)
            prefetch_tensormap(&tmap_a1);
            prefetch_tensormap(&tmap_b1);
            prefetch_tensormap(&tmap_a2);
            prefetch_tensormap(&tmap_b2);
            FusedWalker w;
            uint32_t it = 0;
            int kind, e, mt, nt, row0, rows, cnt;
            int ready_e = -1, ready_blk = -1;
            bool ok = true;
            for (int tile = pair_id; ok && w.locate(p, tile, kind, e, mt, nt, row0, rows, cnt); tile += num_pairs) {
                const int kblocks = kind ? kb2 : kb1;
                int brow_lo, brow_hi;
                if (kind == 0) {
                    brow_lo = e * 2 * p.inter + nt * 128;
                    brow_hi = brow_lo + p.inter;
                    if (!p.skip_arrival && e != ready_e) {  // the expert's rows (from every rank) must have landed
                        uint32_t seen;
                        if (!fm_wait_counter<true>(my_arrival + e, static_cast<uint32_t>(cnt), wt, seen)) {
                            gemm_record_status(p.status, CAM_ERR_TIMEOUT_ARRIVAL, e, static_cast<int>(seen));
                            fm_raise_abort(wt);
                            ok = false;
                            break;
                        }
                        ready_e = e;
                        if (p.trace != nullptr)
                            atomicCAS(p.trace + e, 0ull, static_cast<unsigned long long>(globaltimer_ns()));
                    }
                } else {
                    brow_lo = e * p.h + nt * BN;
                    brow_hi = brow_lo + 128;
                    const int blk = fm_block_index(row0, e);
                    if (blk != ready_blk) {  // every column tile of the first GEMM has written this row block
                        uint32_t seen;
                        if (!fm_wait_counter<false>(p.g1_done + blk, static_cast<uint32_t>(kFmG1Signals * nt1), wt, seen)) {
                            gemm_record_status(p.status, CAM_ERR_TIMEOUT_GEMM1, e, static_cast<int>(seen));
                            fm_raise_abort(wt);
                            ok = false;
                            break;
                        }
                        ready_blk = blk;
                    }
                }
                fence_proxy_async_all();  // rows written by other SMs / GPUs are read by TMA below
                const int my_arow = row0 + static_cast<int>(cta) * BM;
                const int my_brow = cta ? brow_hi : brow_lo;
                // the two GEMMs get their own copy of the loop, so that each TMA instruction names its descriptor by
                // its fixed place among the kernel parameters instead of through a pointer chosen at run time
                auto load_tile = [&](const CUtensorMap& ma, const CUtensorMap& mb) {
                    for (int kb = 0; kb < kblocks; ++kb, ++it) {
                        const uint32_t s = it % NS, ph = (it / NS) & 1u;
                        if (!fm_mbar_wait(&bar_empty[s], ph ^ 1u, wt)) { ok = false; break; }
                        uint8_t* sa = smem + s * kFmStageBytes;
                        if (cta == 0) mbar_arrive_expect_tx(&bar_full[s], 2 * kFmStageBytes);
                        const uint32_t full0 = map_to_cta(&bar_full[s], 0);
                        tma_load_2d_pair(sa, &ma, full0, kb * BK, my_arow);
                        tma_load_2d_pair(sa + kFmATile, &mb, full0, kb * BK, my_brow);
                    }
                };
                if (kind == 0) load_tile(tmap_a1, tmap_b1);
                else load_tile(tmap_a2, tmap_b2);
            }
            if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 0, static_cast<int>(it));
        } else if (warp == 1 && lane == 0 && cta == 0 && do_gemm) {
            // ------------------------------------------------------------ MMA issuer (first CTA only)
            constexpr uint32_t idesc = umma_idesc_mxf8(2 * BM, BN);
            FusedWalker w;
            uint32_t it = 0, tcount = 0;
            int kind, e, mt, nt, row0, rows, cnt;
            bool ok = true;
            const uint32_t tfull0 = map_to_cta(bar_tfull, 0), tfull1 = map_to_cta(bar_tfull, 1);
            // with tracing on, the first pair adds up what its MMA issuer waited for (clock cycles)
            const bool prof = p.trace != nullptr && blockIdx.x == 0;
            long long w_acc = 0, w_sf = 0, w_full = 0, w_issue = 0, t_begin = clock64();
            for (int tile = pair_id; ok && w.locate(p, tile, kind, e, mt, nt, row0, rows, cnt); tile += num_pairs, ++tcount) {
                const int kblocks = kind ? kb2 : kb1;
                long long c0 = prof ? clock64() : 0;
                if (!fm_mbar_wait(bar_tempty, (tcount & 1u) ^ 1u, wt)) { ok = false; break; }
                if (prof) w_acc += clock64() - c0;
                tc_fence_after_sync();
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const uint32_t s = it % NS, ph = (it / NS) & 1u;
                    if (prof) c0 = clock64();
                    if (!fm_mbar_wait(&bar_sf[s], ph, wt)) { ok = false; break; }
                    if (prof) { const long long c1 = clock64(); w_sf += c1 - c0; c0 = c1; }
                    if (!fm_mbar_wait(&bar_full[s], ph, wt)) { ok = false; break; }
                    if (prof) { const long long c1 = clock64(); w_full += c1 - c0; c0 = c1; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * kFmStageBytes);
                    const uint64_t adesc = umma_desc_k_sw128(sa);
                    const uint64_t bdesc = umma_desc_k_sw128(sa + kFmATile);
                    const uint32_t sfa = tmem_base + kFmSfCol0 + s * kFmSfStride;
                    const uint32_t sfb = sfa + 4u;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)
                        tc_mma_mxf8_pair(tmem_base, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) ? 1u : 0u, sfa, sfb);
                    tc_commit_pair(map_to_cta(&bar_empty[s], 0));
                    tc_commit_pair(map_to_cta(&bar_empty[s], 1));
                    if (prof) w_issue += clock64() - c0;
                }
                if (!ok) break;
                tc_commit_pair(tfull0);
                tc_commit_pair(tfull1);
            }
            if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 1, static_cast<int>(it));
            if (prof) p.trace[p.num_experts + 7] = static_cast<unsigned long long>(w_issue);
            if (prof) {
                unsigned long long* t = p.trace + p.num_experts + 1;
                t[0] = static_cast<unsigned long long>(clock64() - t_begin);  // the issuer's whole loop
                t[1] = static_cast<unsigned long long>(w_acc);                // ... waiting for the accumulator to be drained
                t[2] = static_cast<unsigned long long>(w_sf);                 // ... for scale factors
                t[3] = static_cast<unsigned long long>(w_full);               // ... for operand tiles
                t[4] = it;                                                    // K-blocks issued
                t[5] = tcount;                                                // tiles
            }
        } else if (kSlots > 0 && warp == 2 && lane == 0 && do_send) {
            // ------------------------------------------------------------ dispatch sender
            FmSender sender{p, wt, send_ring, bar_send, send_meta,
                            p.off_arrival + static_cast<uint64_t>(parity) * p.arrival_stride * sizeof(uint32_t)};
            sender.run();
        }
    } else if (warp < kFmEpiWarp0) {
        reg_dealloc<kFmSfRegs>();
        // ---------------------------------------------------------------- scale-factor writers
        if (do_gemm) {
            const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
            FusedWalker w;
            uint32_t it = 0;
            int kind, e, mt, nt, row0, rows, cnt;
            int ready_e = -1, ready_blk = -1;
            bool ok = true;
            for (int tile = pair_id; ok && w.locate(p, tile, kind, e, mt, nt, row0, rows, cnt); tile += num_pairs) {
                const int kblocks = kind ? kb2 : kb1;
                const float* a_scales = kind ? p.act_s : p.a1_scales;
                // activation scales arrive during this kernel (from peers or from the first GEMM): wait like the
                // producer does, and read them with L2-coherent loads only
                if (kind == 0) {
                    if (!p.skip_arrival && e != ready_e) {
                        uint32_t seen;
                        const bool got = fm_wait_counter<true>(my_arrival + e, static_cast<uint32_t>(cnt), wt, seen);
                        if (!__all_sync(0xFFFFFFFFu, got)) {
                            if (lane == 0) gemm_record_status(p.status, CAM_ERR_TIMEOUT_ARRIVAL, e, static_cast<int>(seen));
                            ok = false;
                            break;
                        }
                        ready_e = e;
                    }
                } else {
                    const int blk = fm_block_index(row0, e);
                    if (blk != ready_blk) {
                        uint32_t seen;
                        const bool got = fm_wait_counter<false>(p.g1_done + blk, static_cast<uint32_t>(kFmG1Signals * nt1), wt, seen);
                        if (!__all_sync(0xFFFFFFFFu, got)) {
                            if (lane == 0) gemm_record_status(p.status, CAM_ERR_TIMEOUT_GEMM1, e, static_cast<int>(seen));
                            ok = false;
                            break;
                        }
                        ready_blk = blk;
                    }
                }
                // row 32 j + lane of this CTA's half of the tile, clamped to the tile's last valid row: rows behind it
                // may belong to an expert or row block that is not complete yet
                const int rbase = row0 + static_cast<int>(cta) * BM + static_cast<int>(lane);
                const int rlast = min(row0 + rows, p.a_rows) - 1;
                const int pitch = kind ? p.act_scale_pitch : p.a1_scale_pitch;  // a multiple of four floats
                const float4* ap0 = reinterpret_cast<const float4*>(a_scales + static_cast<size_t>(min(rbase, rlast)) * pitch);
                const float4* ap1 = reinterpret_cast<const float4*>(a_scales + static_cast<size_t>(min(rbase + 32, rlast)) * pitch);
                const float4* ap2 = reinterpret_cast<const float4*>(a_scales + static_cast<size_t>(min(rbase + 64, rlast)) * pitch);
                const float4* ap3 = reinterpret_cast<const float4*>(a_scales + static_cast<size_t>(min(rbase + 96, rlast)) * pitch);
                int nb_lo, nb_hi, nblk;
                const float* b_scales;
                if (kind == 0) { nb_lo = nt; nb_hi = nblk1 / 2 + nt; nblk = nblk1; b_scales = p.b1_scales; }
                else { nb_lo = 2 * nt; nb_hi = min(2 * nt + 1, nblk2 - 1); nblk = nblk2; b_scales = p.b2_scales; }
                const float* bs_lo = b_scales + (static_cast<size_t>(e) * nblk + nb_lo) * kblocks;
                const float* bs_hi = b_scales + (static_cast<size_t>(e) * nblk + nb_hi) * kblocks;
                // One K-block: write the six scale words of stage s into TMEM and tell the MMA issuer.
                auto put = [&](uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) -> bool {
                    const uint32_t s = it % NS, ph = (it / NS) & 1u;
                    const bool got = fm_mbar_wait(&bar_empty[s], ph ^ 1u, wt);
                    if (!__all_sync(0xFFFFFFFFu, got)) return false;
                    tc_fence_after_sync();
                    const uint32_t col = tmem_base + lane_base + kFmSfCol0 + s * kFmSfStride;
                    tmem_st_32x32b_x4(col, a0, a1, a2, a3);
                    tmem_st_32x32b_x4(col + 4u, b0, b0, b0, b0);
                    tmem_st_32x32b_x4(col + 8u, b1, b1, b1, b1);
                    tc_wait_st();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if (cta == 0) mbar_arrive(&bar_sf[s]);
                        else mbar_arrive_cluster(map_to_cta(&bar_sf[s], 0));
                    }
                    ++it;
                    return true;
                };
                // Scales move in groups of four K-blocks: one 16-byte load per row and group, issued a whole group
                // (three to four K-blocks of work) before its first use, so that a load that misses L1 still arrives
                // in time.  A load that is only one K-block ahead makes these warps, and with them the MMA issuer,
                // run at one K-block per L2 latency.  Each group is packed to one exponent byte per K-block at once.
                const int ngroups = (kblocks + 3) >> 2;
                float4 na0, na1, na2, na3;
                float nbl[4], nbh[4];
                auto load_group = [&](int g) {
                    na0 = ld_ca_v4f32(ap0 + g); na1 = ld_ca_v4f32(ap1 + g); na2 = ld_ca_v4f32(ap2 + g); na3 = ld_ca_v4f32(ap3 + g);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int kb = min(4 * g + i, kblocks - 1);
                        nbl[i] = __ldg(bs_lo + kb);
                        nbh[i] = __ldg(bs_hi + kb);
                    }
                };
                load_group(0);
                for (int g = 0; ok && g < ngroups; ++g) {
                    const uint32_t pa0 = ue8m0_pack4(na0.x, na0.y, na0.z, na0.w), pa1 = ue8m0_pack4(na1.x, na1.y, na1.z, na1.w);
                    const uint32_t pa2 = ue8m0_pack4(na2.x, na2.y, na2.z, na2.w), pa3 = ue8m0_pack4(na3.x, na3.y, na3.z, na3.w);
                    const uint32_t pbl = ue8m0_pack4(nbl[0], nbl[1], nbl[2], nbl[3]), pbh = ue8m0_pack4(nbh[0], nbh[1], nbh[2], nbh[3]);
                    const int left = kblocks - 4 * g;
                    ok = put(__byte_perm(pa0, 0, 0x0000), __byte_perm(pa1, 0, 0x0000), __byte_perm(pa2, 0, 0x0000),
                             __byte_perm(pa3, 0, 0x0000), __byte_perm(pbl, 0, 0x0000), __byte_perm(pbh, 0, 0x0000));
                    // the next group's loads go out only after the arrive above, which has release semantics and would
                    // otherwise wait for them
                    if (g + 1 < ngroups) load_group(g + 1);
                    if (ok && left > 1)
                        ok = put(__byte_perm(pa0, 0, 0x1111), __byte_perm(pa1, 0, 0x1111), __byte_perm(pa2, 0, 0x1111),
                                 __byte_perm(pa3, 0, 0x1111), __byte_perm(pbl, 0, 0x1111), __byte_perm(pbh, 0, 0x1111));
                    if (ok && left > 2)
                        ok = put(__byte_perm(pa0, 0, 0x2222), __byte_perm(pa1, 0, 0x2222), __byte_perm(pa2, 0, 0x2222),
                                 __byte_perm(pa3, 0, 0x2222), __byte_perm(pbl, 0, 0x2222), __byte_perm(pbh, 0, 0x2222));
                    if (ok && left > 3)
                        ok = put(__byte_perm(pa0, 0, 0x3333), __byte_perm(pa1, 0, 0x3333), __byte_perm(pa2, 0, 0x3333),
                                 __byte_perm(pa3, 0, 0x3333), __byte_perm(pbl, 0, 0x3333), __byte_perm(pbh, 0, 0x3333));
                }
            }
            if (!ok && lane == 0) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 3, static_cast<int>(it));
        }
    } else {
        reg_alloc<kFmEpiRegs>();
        // ---------------------------------------------------------------- epilogue warps
        if (do_gemm) {
            const int ew = warp - kFmEpiWarp0;
            const int q = warp & 3;   // TMEM lane quarter this warp may read
            const int cq = ew >> 2;   // which 32-column quarter of each 128-column half
            const int r = q * 32 + static_cast<int>(lane);
            FusedWalker w;
            uint32_t tcount = 0;
            int kind, e, mt, nt, row0, rows, cnt;
            bool ok = true;
            for (int tile = pair_id; ok && w.locate(p, tile, kind, e, mt, nt, row0, rows, cnt); tile += num_pairs, ++tcount) {
                const int blk = fm_block_index(row0, e);
                row0 += static_cast<int>(cta) * BM;            // this CTA's half of the 256-row tile
                rows = max(0, min(BM, rows - static_cast<int>(cta) * BM));
                const bool valid = r < rows && row0 + r < p.a_rows;
                const int grow = row0 + (valid ? r : 0);
                // one decision for all epilogue threads: a thread that gave up must not leave the others at a
                // named barrier further down
                if (!named_bar_and(1, kFmEpiThreads, fm_mbar_wait_sleep(bar_tfull, tcount & 1u, wt))) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + cq * 32;
                uint32_t v0[32], v1[32];
                tmem_ld_32x32b_x32(t0, v0);
                tmem_ld_32x32b_x32(t0 + 128, v1);
                tc_wait_ld_regs(v0);
                tc_wait_ld_regs(v1);
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (cta == 0) mbar_arrive(bar_tempty);
                    else mbar_arrive_cluster(map_to_cta(bar_tempty, 0));
                }

                if (kind == 0) {
                    // SwiGLU on matching gate/up columns, then 1x128 fp8 requantisation (power-of-two scale).
                    float act[32];
                    float amax = 0.f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float g = __uint_as_float(v0[j]);
                        act[j] = (g / (1.f + expf(-g))) * __uint_as_float(v1[j]);
                        amax = fmaxf(amax, fabsf(act[j]));
                    }
                    // the exchange area lies inside the first staging buffer: copies of an earlier combine send
                    // that still read it must be through before it is overwritten
                    if (cq == 0) bulk_wait_group_read<0>();
                    named_bar_sync(1, kFmEpiThreads);
                    float* xch = s_amax + (tcount & 1u) * 512;
                    xch[cq * 128 + r] = amax;
                    named_bar_sync(1, kFmEpiThreads);
                    amax = fmaxf(fmaxf(xch[r], xch[128 + r]), fmaxf(xch[256 + r], xch[384 + r]));
                    float scale, inv;
                    ue8m0_scale(amax, scale, inv);
                    if (valid) {
                        uint8_t* dst = p.act_q + static_cast<size_t>(grow) * p.inter + nt * 128 + cq * 32;
#pragma unroll
                        for (int j = 0; j < 32; j += 16) {
                            uint4 o;
                            o.x = pack_e4m3x4(act[j + 0] * inv, act[j + 1] * inv, act[j + 2] * inv, act[j + 3] * inv);
                            o.y = pack_e4m3x4(act[j + 4] * inv, act[j + 5] * inv, act[j + 6] * inv, act[j + 7] * inv);
                            o.z = pack_e4m3x4(act[j + 8] * inv, act[j + 9] * inv, act[j + 10] * inv, act[j + 11] * inv);
                            o.w = pack_e4m3x4(act[j + 12] * inv, act[j + 13] * inv, act[j + 14] * inv, act[j + 15] * inv);
                            *reinterpret_cast<uint4*>(dst + j) = o;
                        }
                        if (cq == 0) p.act_s[static_cast<size_t>(grow) * p.act_scale_pitch + nt] = scale;
                    }
                    // This warp's 32 rows x 32 columns are in memory: tell the second GEMM of this row block.  Every warp
                    // releases its own stores; one thread releasing for the whole CTA after a barrier (a fence that
                    // is cumulative over all 512 threads' stores) cost a sixth of the kernel's time.
                    __syncwarp();
                    if (lane == 0) red_release_gpu_add_u32(p.g1_done + blk, 1u);
                } else {
                    // bf16 rows straight to the origin rank's combine slots (256-byte bulk copies out of the staging buffer)
                    __nv_bfloat16* orow = nullptr;
                    if (valid) {
                        const int src = p.row_src[static_cast<size_t>(grow) * 3 + 0];
                        const int tok = p.row_src[static_cast<size_t>(grow) * 3 + 1];
                        const int kk = p.row_src[static_cast<size_t>(grow) * 3 + 2];
                        if (src >= 0 && src < p.num_ranks && tok >= 0 && tok < p.max_tokens && kk >= 0 && kk < p.topk)
                            orow = reinterpret_cast<__nv_bfloat16*>(p.peer_base[src] + p.off_combine_buf) +
                                   (static_cast<size_t>(tok) * p.topk + kk) * static_cast<size_t>(p.h);
                    }
                    auto push_half = [&](const uint32_t (&v)[32], int c0) {
                        uint8_t* srow = stg + r * kFmStgPitch;
                        if (cq == 0) bulk_wait_group_read<0>();  // the copies that read the staging buffer are done with it
                        named_bar_sync(1, kFmEpiThreads);
#pragma unroll
                        for (int j = 0; j < 32; j += 8)
                            *reinterpret_cast<uint4*>(srow + cq * 64 + j * 2) =
                                pack_bf16x8(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                            __uint_as_float(v[j + 3]), __uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]),
                                            __uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                        fence_proxy_async_smem();
                        named_bar_sync(1, kFmEpiThreads);
                        if (cq == 0) {
                            if (orow != nullptr) bulk_store_s2g(orow + c0, srow, 256);
                            bulk_commit_group();
                        }
                    };
                    const int c_lo = nt * BN;
                    push_half(v0, c_lo);
                    if (c_lo + 128 < p.h) push_half(v1, c_lo + 128);
                }
            }
            if (cq == 0) bulk_wait_group<0>();  // every row this thread sent has been written
            if (!ok) gemm_record_status(p.status, CAM_ERR_TIMEOUT_PIPELINE, 2, static_cast<int>(tcount));
        }
    }

    // ------------------------------------------------------------------ teardown
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // the other CTA may still read this CTA's shared memory or signal its barriers
    if (do_gemm && warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kFmTmemCols);
    }
    if (do_gemm && threadIdx.x == 0) {
        __threadfence_system();
        const unsigned int old = atomicAdd(p.done_ctr, 1u);
        if (old == gridDim.x - 1) {
            p.done_ctr[0] = 0u;
            __threadfence_system();
            const uint32_t epoch = *p.epoch_send + 1u;  // this launch is the send phase of a combine
            if (p.dbg_drop_flags == 0) {
                for (int d = 0; d < p.num_ranks; ++d)
                    st_release_sys_u32(reinterpret_cast<uint32_t*>(p.peer_base[d] + p.off_combine_flag) + p.rank, epoch);
            }
            *p.epoch_send = epoch;
        }
    }
}

}  // namespace cam

extern "C" int cam_fused_moe_smem_bytes(void) { return cam::kFmSmem; }

namespace {

void fm_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int grid, int smem, cudaStream_t stream) {
    cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid & ~1));
    cfg.blockDim = dim3(cam::kFmThreads);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem);
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
}

}  // namespace

// CTA pairs of the fused kernel that can be resident at once on the current device (cached per device; -1 on error).
extern "C" int cam_fused_moe_max_pairs(void) {
    static cam::SmemLimitCache limit_send, limit_gemm;
    if (limit_send.ensure(cam::fused_moe_pair_kernel<cam::kFmStagesSend>, cam::fm_smem<cam::kFmStagesSend>()) != cudaSuccess) return -1;
    if (limit_gemm.ensure(cam::fused_moe_pair_kernel<cam::kFmStagesGemm>, cam::fm_smem<cam::kFmStagesGemm>()) != cudaSuccess) return -1;
    static int max_pairs[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    if (max_pairs[dev] == 0) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        // both forms take (nearly) all the shared memory of an SM and the same threads and registers: one answer
        fm_config(cfg, attr, 2, cam::kFmSmem, nullptr);
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, cam::fused_moe_pair_kernel<cam::kFmStagesGemm>, &cfg) == cudaSuccess && n > 0)
            max_pairs[dev] = n;
        else max_pairs[dev] = -1;
    }
    return max_pairs[dev];
}

// The tiles of the launch are walked with a fixed stride by CTA pairs that wait for one another's
// results (second GEMM after first), so the grid never exceeds what is resident at once.
extern "C" int cam_launch_fused_moe(const cam::FusedMoeParams* p, const CUtensorMap* tmap_a1, const CUtensorMap* tmap_b1,
                                    const CUtensorMap* tmap_a2, const CUtensorMap* tmap_b2, int grid, cudaStream_t stream) {
    const int fit = cam_fused_moe_max_pairs();
    if (fit <= 0) return static_cast<int>(cudaErrorLaunchOutOfResources);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    const bool sends = (p->phase_mask & CAM_PHASE_SEND) != 0;
    fm_config(cfg, attr, grid, sends ? cam::fm_smem<cam::kFmStagesSend>() : cam::fm_smem<cam::kFmStagesGemm>(), stream);
    if (2 * fit < static_cast<int>(cfg.gridDim.x)) cfg.gridDim = dim3(static_cast<unsigned>(2 * fit));
    if (sends)
        return static_cast<int>(cudaLaunchKernelEx(&cfg, cam::fused_moe_pair_kernel<cam::kFmStagesSend>, *tmap_a1, *tmap_b1,
                                                   *tmap_a2, *tmap_b2, *p));
    return static_cast<int>(cudaLaunchKernelEx(&cfg, cam::fused_moe_pair_kernel<cam::kFmStagesGemm>, *tmap_a1, *tmap_b1, *tmap_a2,
                                               *tmap_b2, *p));
}
