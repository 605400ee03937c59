// Parameter blocks and C-ABI launchers of every kernel in the library.  The launchers take raw
// device pointers only, so they can be driven from the torch bindings, from the C runtime or
// straight from ctypes.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "../common/cam_types.h"

namespace cam {

// Per-buffer statistics kept on the device (Buffer.stats()): which peer this rank waited for longest, and how many rows
// it routed to every peer.  Written by CTA 0 of the comm kernels; never reset by the kernels.
struct CamStatsDev {
    unsigned long long max_wait_ns[3][CAM_MAX_RANKS];  // [0] dispatch counts, [1] dispatch rows, [2] combine rows; per peer
    unsigned long long rows_routed[CAM_MAX_RANKS];     // (token, k) pairs routed to every rank since the last reset
    unsigned long long calls[3];                       // dispatches, combines (reduce side), spare
};

struct DispatchNormalParams {
    const __nv_bfloat16* x;  // [T, h]
    const void* topk_idx;    // [T, K] int64 or int32, ids outside [0, E) are skipped
    int idx_is_i64;
    int T, K, h, E, R, rank;
    int quant_mode;  // CamQuantMode
    int capacity;    // rows of every rank's receive buffer
    uint32_t* epochs;        // device counters [count, send, recv]; a phase uses counter + 1 as its epoch (flags carry
                             // it, double-buffered regions ping-pong on its parity) and stores it back when the kernel ends
    unsigned int* exit_ctr;  // [1], self-resetting: finds the CTA that leaves last
    uint64_t timeout_ns;
    int phase_mask;      // CamPhase bits
    int dbg_drop_flags;  // host-side fault injection: this rank withholds its flags
    uint8_t* const* peer_base;  // [R] base of every rank's symmetric allocation (device array)
    uint64_t off_count_flag, off_data_flag, off_count_matrix, off_recv_x, off_recv_scales, off_recv_src;
    uint64_t off_dup_cnt, off_dup_list;  // replicate lists: rows the receiver copies locally instead of receiving twice
    int dup_cap;                         // entries per (parity, source) list
    unsigned int* dup_ctr;               // [R] local cursors into the lists this rank writes
    // local workspace / outputs
    int* cta_hist;                  // [grid, E]
    int* slot_in_expert;            // [T*K]
    int* send_row;                  // [T*K] row at the destination, -1 when skipped
    int* recv_count;                // [E_local*R] inclusive cumsum (expert major, source minor)
    int* expert_offsets;            // [E_local+1]
    int64_t* num_recv_per_expert;   // [E_local]
    int* total_recv;                // [1]
    int* num_tokens_per_expert_out; // [E] optional (may be null)
    unsigned int* done_ctr;         // [1], self-resetting
    CamStatus* status;
    // Deferred push (the fused layer's first launch): the SEND phase pushes nothing.  It quantises every token once
    // into local memory and writes the list of rows to send, ordered by (local expert at the destination, destination
    // rank, scan order), so that the fused kernel's copy warps complete expert 0 of every rank first, then expert 1, ...
    CamStatsDev* stats;             // optional
    int defer_push;
    uint8_t* xq;                    // [T, h] e4m3
    float* xs;                      // [T, h/128]
    int4* send_list;                // [T*K] {token, destination rank, row at the destination, local expert | k << 16}
    int* send_list_len;             // [1]
    uint32_t* g1_done;              // [g1_done_len] per-row-block counters of the fused kernel, zeroed here
    int g1_done_len;
    uint64_t off_arrival;           // u32[2][E] in the symmetric region: rows landed per local expert
};

struct CombineParams {
    const __nv_bfloat16* y;   // [N, h] expert outputs in receive order (SEND phase)
    const int* row_src;       // [N, 3] (src rank, src token, src k)
    const int* total_rows;    // [1] device-side N
    const void* topk_idx;     // [T, K] of this rank's own tokens (RECV phase)
    int idx_is_i64;
    const float* topk_weights;  // [T, K]
    __nv_bfloat16* out;         // [T, h]
    int T, K, h, E, R, rank;
    int max_tokens;  // tokens per rank the combine slots hold (SEND drops rows that name a later token)
    int comm_quant;  // 0: bf16 rows on the wire, 2: int8 rows + one fp32 scale per 128 elements
    uint32_t* epochs;        // device counters [send, recv]
    unsigned int* exit_ctr;
    unsigned long long* trace;  // optional [8] timeline of CTA 0
    uint64_t timeout_ns;
    int phase_mask;
    int dbg_drop_flags;
    uint8_t* const* peer_base;
    uint64_t off_combine_buf, off_combine_flag;
    unsigned int* done_ctr;
    CamStatus* status;
    CamStatsDev* stats;  // optional
};

struct DispatchLLParams {
    const __nv_bfloat16* x;  // [T, h]
    const void* expert_ids;  // [T, K]
    int idx_is_i64;
    const float* smooth;     // optional [E, h] smooth scales (may be null)
    int T, K, h, E, R, rank;
    int active_tokens;       // tokens [0, active_tokens) take part (x_active_mask prefix count)
    int quant_mode;
    int max_tokens;          // slab depth per (src, local expert) cell
    int count_type;          // 1 = per-expert counts, 0 = cumulative
    uint32_t* epochs;        // device counters [send, recv]
    unsigned int* exit_ctr;
    unsigned long long* trace;  // optional [8] timeline of CTA 0 (see trace_point), null when tracing is off
    int slot_table_bytes;       // > 0: shared memory holds a chunk x expert table for the parallel slot computation
    uint64_t timeout_ns;
    int phase_mask;
    int dbg_drop_flags;
    uint8_t* const* peer_base;
    uint64_t off_ll_cells, off_ll_x, off_ll_scales, off_ll_meta;
    // outputs (local)
    uint8_t* expand_x;        // [A, row_bytes]
    float* expand_scales;     // [A, nscale]
    int* expand_idx;          // [T*K] slot of every pair inside its (src, expert) cell
    int* expand_src;          // [A, 3] (src rank, src token, src k) of every packed row
    int64_t* expert_token_nums;  // [E_local]
    int* ep_send_counts;      // [E_local*R] inclusive cumsum
    int* total_rows;          // [1]
    CamStatus* status;
};

// Grouped GEMM  D[rows of expert e] = A[rows of expert e] * B[e]^T  with block-scaled fp8.
struct GroupedGemmParams {
    const int* expert_offsets;  // [E_local+1] first row of every expert in A (device memory)
    int num_experts;            // E_local
    int n_dim;                  // output columns per expert (2I for gemm1, h for gemm2)
    int k_dim;                  // reduction length
    int a_rows;                 // rows covered by the A tensor map
    const float* a_scales;      // [a_rows, k_dim/128] row major
    const float* b_scales;      // [E_local, n_dim/128, k_dim/128]
    int mode;                   // 0: plain bf16 out, 1: SwiGLU + fp8 requant, 2: bf16 out pushed to combine slots
    // mode 0
    __nv_bfloat16* out;         // [a_rows, n_dim]
    // mode 1
    uint8_t* act_q;             // [a_rows, n_dim/2] e4m3
    float* act_s;               // [a_rows, n_dim/2/128]
    // mode 1 of the int8 kernel: fp32 SwiGLU output and per-row max |.| (quantised per token afterwards)
    float* act_f32;             // [a_rows, n_dim/2]
    float* row_amax;            // [a_rows], zero on entry
    // mode 2
    const int* row_src;         // [a_rows, 3]
    uint8_t* const* peer_base;
    uint64_t off_combine_buf, off_combine_flag;
    int topk, num_ranks, rank;
    int max_tokens;             // mode 2: tokens per rank the combine slots hold (rows naming a later token are dropped)
    uint32_t* epoch_send;       // device counter of the combine send phase (mode 2 plays that phase)
    int bulk_push;              // modes 0/2 of the block-scaled kernels: rows leave as bulk copies instead of vector stores
    int dbg_drop_flags;
    unsigned int* done_ctr;
    CamStatus* status;
};

// Deep-fused layer (kernels/fused_moe_mx.cu): dispatch send, both grouped GEMMs and the combine send in one launch.
// GEMM1: A = this rank's receive buffer [a_rows, h], B = w1 [E_local * 2I, h]; GEMM2: A = act_q [a_rows, I],
// B = w2 [E_local * h, I] (four TMA descriptors passed beside this block).
struct FusedMoeParams {
    const int* expert_offsets;  // [E_local+1] first row of every local expert (written by the layer's first launch)
    int num_experts;            // E_local
    int h, inter;               // hidden size, intermediate size
    int a_rows;                 // rows of the receive buffer (capacity)
    int max_tokens;             // tokens per rank the combine slots are sized for
    const float* a1_scales;     // [a_rows, a1_scale_pitch] scales of the received rows (arrive during the kernel)
    int a1_scale_pitch;         // floats per scale row: h/128 rounded up to 4 (rows are read 16 bytes at a time)
    int act_scale_pitch;        // the same for act_s (I/128 rounded up to 4)
    const float* b1_scales;     // [E_local, 2I/128, h/128]
    const float* b2_scales;     // [E_local, h/128, I/128]
    uint8_t* act_q;             // [a_rows, I] e4m3, between the two GEMMs
    float* act_s;               // [a_rows, act_scale_pitch]
    const int* row_src;         // [a_rows, 3] (src rank, src token, src k) of every received row
    uint8_t* const* peer_base;
    uint64_t off_combine_buf, off_combine_flag, off_recv_x, off_recv_scales, off_recv_src, off_arrival;
    int arrival_stride;         // entries per parity of the arrival counters (= number of experts of the call)
    int topk, num_ranks, rank;
    uint32_t* epoch_send;            // device counter of the combine send phase (this launch plays that phase)
    const uint32_t* epoch_dispatch;  // device counter of the dispatch send phase, already advanced by the first launch
    int dbg_drop_flags;
    unsigned int* done_ctr;
    CamStatus* status;
    uint32_t* g1_done;          // per 256-row block: column tiles of GEMM1 written (zeroed by the first launch)
    int skip_arrival;           // the rows were brought by a dispatch that finished before this launch: no arrival counters
    int lag;                    // GEMM2 of expert e is scheduled after GEMM1 of expert e + lag
    // dispatch send
    const uint8_t* xq;          // [T, h] this rank's quantised tokens
    const float* xs;            // [T, h/128]
    const int4* send_list;      // {token, destination rank, row at the destination, local expert | k << 16}
    const int* send_list_len;   // [1]
    int send_list_cap;
    int phase_mask;             // CAM_PHASE_SEND: copy warps run, CAM_PHASE_RECV: the GEMM roles run
    uint64_t timeout_ns;
    unsigned long long* trace;  // optional [E_local+1]: time GEMM1 of every expert was released, kernel start
};

// Exchange between the two tensor-parallel ranks of one expert-parallel position (kernels/tp_exchange.cu).
struct TpExchangeParams {
    int reduce;              // 0: all-gather after dispatch, 1: reduce-scatter before combine
    const uint8_t* rows;     // all-gather: my received rows; reduce-scatter: partial outputs for [mine | partner's]
    const float* scales;     // all-gather only, optional [rows, nscale]
    int row_bytes, nscale;
    const int* n_own;        // [1] device: rows of my own tokens
    const int* n_peer;       // [1] device: rows of the partner's tokens (reduce-scatter)
    int max_rows;            // rows the exchange region holds
    uint8_t* out;            // all-gather: the same tensor as rows (partner rows appended); reduce-scatter: [n_own, row_bytes]
    float* scales_out;
    int out_rows;            // rows `out` can hold
    int* tp_counts;          // [2] all-gather output: rows per TP rank
    int tp_rank;
    uint8_t* my_base;
    uint8_t* peer_base;      // the partner's symmetric allocation
    uint64_t off_tp_flag, off_tp_cnt, off_tp_x, off_tp_scales;
    uint32_t* epochs;        // [send, recv]
    unsigned int* exit_ctr;
    unsigned int* done_ctr;
    uint64_t timeout_ns;
    int phase_mask;
    int dbg_drop_flags;
    CamStatus* status;
};

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) costs microseconds per call; the launchers go
// through this helper, which remembers per device what it has already set for one kernel.
struct SmemLimitCache {
    int set[64] = {0};
    template <class Kernel>
    cudaError_t ensure(Kernel k, int bytes) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64 && set[dev] >= bytes && bytes > 0) return cudaSuccess;
        if (bytes <= 0) return cudaSuccess;
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e == cudaSuccess && dev >= 0 && dev < 64) set[dev] = bytes;
        return e;
    }
};

// SMs of the current device (cached per device; 148 on a B200, which is also the answer if the query fails).
inline int sm_count_of_current_device() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        cached[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
    }
    return cached[dev];
}

}  // namespace cam

extern "C" {
int cam_dispatch_normal_smem_bytes(int h, int quant_mode);
int cam_dispatch_normal_max_grid(int device, int h, int quant_mode);
int cam_launch_dispatch_normal(const cam::DispatchNormalParams* p, int grid, cudaStream_t stream);
int cam_launch_layout(const void* topk_idx, int idx_is_i64, int T, int K, int E, int R,
                      int* num_tokens_per_rank, int* num_tokens_per_expert, uint8_t* is_token_in_rank,
                      cudaStream_t stream);
int cam_combine_max_grid(int device);
int cam_launch_combine(const cam::CombineParams* p, int grid, cudaStream_t stream);
int cam_dispatch_ll_slot_table_bytes(int T, int K, int E);
int cam_dispatch_ll_smem_bytes(int h, int quant_mode, int T, int K, int E);
int cam_dispatch_ll_max_grid(int device, int h, int quant_mode, int T, int K, int E);
int cam_launch_dispatch_ll(const cam::DispatchLLParams* p, int grid, cudaStream_t stream);
int cam_launch_grouped_gemm_fp8(const cam::GroupedGemmParams* p, const CUtensorMap* tmap_a,
                                const CUtensorMap* tmap_b, int grid, cudaStream_t stream);
int cam_grouped_gemm_smem_bytes(void);
int cam_launch_grouped_gemm_mxfp8(const cam::GroupedGemmParams* p, const CUtensorMap* tmap_a,
                                  const CUtensorMap* tmap_b, int grid, int swap, int two_staging, cudaStream_t stream);
int cam_grouped_gemm_mx_smem_bytes(void);
int cam_launch_grouped_gemm_mxfp8_pair(const cam::GroupedGemmParams* p, const CUtensorMap* tmap_a,
                                       const CUtensorMap* tmap_b, int grid, int two_staging, cudaStream_t stream);
int cam_grouped_gemm_mx_pair_smem_bytes(void);
int cam_launch_grouped_gemm_w8a8(const cam::GroupedGemmParams* p, const CUtensorMap* tmap_a,
                                 const CUtensorMap* tmap_b, int grid, cudaStream_t stream);
int cam_fused_moe_smem_bytes(void);
int cam_fused_moe_max_pairs(void);
int cam_launch_fused_moe(const cam::FusedMoeParams* p, const CUtensorMap* tmap_a1, const CUtensorMap* tmap_b1,
                         const CUtensorMap* tmap_a2, const CUtensorMap* tmap_b2, int grid, cudaStream_t stream);
int cam_launch_barrier(uint8_t* const* peer_base, uint64_t off_barrier_flag, uint32_t* epochs, int R, int rank,
                       int phase_mask, int dbg_drop_flags, uint64_t timeout_ns, CamStatus* status, cudaStream_t stream);
int cam_launch_p2p_copy(void* dst, const void* src, size_t bytes, int grid, cudaStream_t stream);
int cam_launch_p2p_pingpong(uint32_t* my_flag, uint32_t* peer_flag, uint32_t base, int iters, int initiator,
                            uint64_t timeout_ns, CamStatus* status, cudaStream_t stream);
int cam_launch_tp_exchange(const cam::TpExchangeParams* p, int grid, cudaStream_t stream);
int cam_launch_rowquant_int8(const float* act, float* row_amax, const int* expert_offsets, int num_experts,
                             int inter, void* out_q, float* out_s, cudaStream_t stream);
}
