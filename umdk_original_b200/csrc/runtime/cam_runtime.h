// C ABI of the host runtime: symmetric buffers, peer tables, epochs, status words and the
// host-side halves of every op (argument validation, workspace carving, launches).
//
// The reference has no explicit buffer object: its kernels find peer "windows" through HCCL's
// HcclOpResParam (ascend_kernels/utils/op_kernel/moe_distribute_base.h:123-173) and keep the
// ping-pong state inside the window itself (moe_dispatch_normal.h:217-229).  Here that state is
// an explicit CamBuffer: one symmetric allocation per rank, a device table of every peer's base
// address, per-op epoch counters and a status word that bounded device waits report into.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include "../common/cam_types.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CamBuffer CamBuffer;

#define CAM_IPC_HANDLE_BYTES 64

const char* cam_last_error(void);
const char* cam_status_string(int code);

int cam_layout_compute(CamLayout* out, int num_ranks, int num_experts, int max_tokens, int hidden, int topk,
                       int capacity, int ll_max_tokens);

// Same with a tensor-parallel exchange region of tp_rows rows (tpWorldSize = 2 in the low-latency ops).
int cam_layout_compute_tp(CamLayout* out, int num_ranks, int num_experts, int max_tokens, int hidden, int topk,
                          int capacity, int ll_max_tokens, int tp_rows);

// Creates the symmetric allocation (cudaMalloc, so that it can be exported with CUDA IPC), the
// local workspace and the status word on `device`.  Returns NULL on failure.
CamBuffer* cam_buffer_create(int device, int rank, int num_ranks, const CamLayout* layout);
int cam_buffer_destroy(CamBuffer* b);
int cam_buffer_ipc_handle(CamBuffer* b, void* out_handle /* CAM_IPC_HANDLE_BYTES */);
// Multi-process: open every peer's IPC handle (handles = num_ranks * 64 bytes, own slot ignored).
int cam_buffer_open_ipc_peers(CamBuffer* b, const void* handles);
// Single-process virtual ranks: every rank is a CamBuffer of this process on the same device.
int cam_buffer_set_local_peers(CamBuffer* b, CamBuffer* const* peers);
// Tensor-parallel partner of this rank (the same expert-parallel position in the other TP group).
int cam_buffer_open_ipc_tp_peer(CamBuffer* b, const void* handle, int tp_rank);
int cam_buffer_set_local_tp_peer(CamBuffer* b, CamBuffer* peer, int tp_rank);
int cam_tp_allgather(CamBuffer* b, void* rows, float* scales, int row_bytes, int nscale, const int* n_own, int out_rows,
                     int* tp_counts, int phase_mask, cudaStream_t stream);
int cam_tp_reduce_scatter(CamBuffer* b, const void* y, int row_bytes, const int* n_own, const int* n_peer, void* out,
                          int phase_mask, cudaStream_t stream);
int cam_buffer_reset(CamBuffer* b, cudaStream_t stream);
void* cam_buffer_base(CamBuffer* b);
const CamLayout* cam_buffer_layout(CamBuffer* b);
int cam_buffer_rank(CamBuffer* b);
int cam_buffer_num_ranks(CamBuffer* b);
int cam_buffer_device(CamBuffer* b);
int cam_buffer_tp_rank(CamBuffer* b);
void cam_buffer_set_timeout_ms(CamBuffer* b, double ms);
void cam_buffer_set_debug_drop_flags(CamBuffer* b, int on);
// Per-stage device timing of the fused layer.  While on, every full fused call records CUDA events
// around its four launches; read_profile waits for the last one and fills
// {dispatch, GEMM1, GEMM2 + combine send, combine reduce} in milliseconds.  Off by default.
// In-kernel timelines (globaltimer stamps of CTA 0) of the low-latency dispatch [0..7] and of combine [8..15].
int cam_buffer_set_trace(CamBuffer* b, int on);
int cam_buffer_read_trace(CamBuffer* b, unsigned long long* out16);
int cam_buffer_check_guards(CamBuffer* b, cudaStream_t stream, int* damaged);  // bit i: guard behind region i was overwritten
unsigned long long cam_buffer_launch_count(CamBuffer* b);
// Route the block-scaled fused layer (power-of-two scales) takes for these shapes on this Buffer: 0 = four launches,
// 1 = deep-fused kernel, 2 = normal dispatch + fused GEMMs.  T = tokens of this rank, K = top-k, E = all experts.
int cam_buffer_fused_route(CamBuffer* b, int T, int K, int h, int inter, int E);
int cam_buffer_read_stats(CamBuffer* b, unsigned long long* out_wait_ns, unsigned long long* out_rows,
                          unsigned long long* out_calls, int reset);  // kernels launched by this buffer's ops so far
int cam_buffer_set_fused_trace(CamBuffer* b, int on);
int cam_buffer_read_fused_trace(CamBuffer* b, long long* out, int num_local_experts);
int cam_buffer_read_fused_waits(CamBuffer* b, long long* out6, int num_local_experts);
int cam_buffer_set_profile(CamBuffer* b, int on);
int cam_buffer_read_profile(CamBuffer* b, float* ms4);
// Copies the device status word (after synchronising `stream`) into *out and clears it on the device.
int cam_buffer_poll_status(CamBuffer* b, cudaStream_t stream, CamStatus* out);
// Device pointers of the results that normal dispatch leaves in the buffer's workspace.
int* cam_buffer_recv_count(CamBuffer* b);
int* cam_buffer_expert_offsets(CamBuffer* b);
int64_t* cam_buffer_num_recv_per_expert(CamBuffer* b);
int* cam_buffer_total_recv(CamBuffer* b);
int* cam_buffer_send_row(CamBuffer* b);
int* cam_buffer_num_tokens_per_expert(CamBuffer* b);
uint8_t* cam_buffer_act_q(CamBuffer* b);
float* cam_buffer_act_s(CamBuffer* b);

// Device barrier over all ranks (kernels/sync_p2p.cu); phase_mask CAM_PHASE_SEND | CAM_PHASE_RECV for a real group.
int cam_buffer_barrier(CamBuffer* b, int phase_mask, cudaStream_t stream);
// P2P microbenchmark kernels (one-sided write bandwidth, flag round-trip latency).
int cam_buffer_p2p_write(CamBuffer* b, int peer, size_t bytes, int grid, cudaStream_t stream);
int cam_buffer_p2p_pingpong(CamBuffer* b, int peer, unsigned int base, int iters, int initiator, cudaStream_t stream);

// get_dispatch_layout: outputs must be zero-initialised by the caller.
int cam_get_dispatch_layout(const void* topk_idx, int idx_is_i64, int T, int K, int E, int R,
                            int* num_tokens_per_rank, int* num_tokens_per_expert, uint8_t* is_token_in_rank,
                            cudaStream_t stream);

// Normal-mode dispatch.  Rows land in the symmetric buffer's recv_x / recv_scales / recv_src
// regions of their destination; counts land in this buffer's workspace.
int cam_dispatch_normal(CamBuffer* b, const void* x_bf16, const void* topk_idx, int idx_is_i64, int T, int K,
                        int h, int E, int quant_mode, int phase_mask, cudaStream_t stream);

// Combine (push + flag + weighted reduce).  `y` rows follow `row_src` ([N,3] device ints), N is
// read on the device from `total_rows`.  low_latency selects the low-latency slot/flag regions.
// comm_quant 2 sends rows as int8 with one fp32 scale per 128 elements (both phases of a call must agree).
int cam_combine(CamBuffer* b, const void* y_bf16, const int* row_src, const int* total_rows, const void* topk_idx,
                int idx_is_i64, const float* topk_weights, void* out_bf16, int T, int K, int h, int E,
                int low_latency, int comm_quant, int phase_mask, cudaStream_t stream);

int cam_dispatch_ll(CamBuffer* b, const void* x_bf16, const void* expert_ids, int idx_is_i64, const float* smooth,
                    int T, int K, int h, int E, int active_tokens, int quant_mode, int count_type,
                    void* expand_x, float* expand_scales, int* expand_idx, int* expand_src,
                    int64_t* expert_token_nums, int* ep_send_counts, int* total_rows, int phase_mask,
                    cudaStream_t stream);

// Grouped block-scaled fp8 GEMM (see kernels/grouped_gemm.cu for the modes).  For mode 2 `b`
// must be non-NULL: rows are pushed into the combine slots of their origin ranks and this rank's
// combine flag is raised (that call plays the SEND phase of combine).
int cam_grouped_gemm_fp8(CamBuffer* b, const void* a_q, const float* a_scales, int a_rows, const void* w_q,
                         const float* w_scales, const int* expert_offsets, int num_experts, int n_dim, int k_dim,
                         int mode, void* out_bf16, void* act_q, float* act_s, const int* row_src, int topk,
                         int low_latency, cudaStream_t stream);

// Same, with the tensor core's own block scaling (kernels/grouped_gemm_mx.cu): every scale must be an
// exact power of two; mode 1 emits power-of-two activation scales.
int cam_grouped_gemm_mxfp8(CamBuffer* b, const void* a_q, const float* a_scales, int a_rows, const void* w_q,
                           const float* w_scales, const int* expert_offsets, int num_experts, int n_dim, int k_dim,
                           int mode, void* out_bf16, void* act_q, float* act_s, const int* row_src, int topk,
                           int low_latency, cudaStream_t stream);

// Whole fp8 MoE layer on the normal-mode path:
// dispatch (fp8 1x128) -> GEMM1 + SwiGLU + requant -> GEMM2 with combine-send epilogue -> reduce.
// gemm_experts: local experts that have weights (0 = E / R; 1 on a shared-expert rank).
int cam_fused_moe_fp8(CamBuffer* b, const void* x_bf16, const void* expert_ids, int idx_is_i64,
                      const float* topk_weights, const void* w1_q, const float* w1_s, const void* w2_q,
                      const float* w2_s, void* out_bf16, int64_t* expert_token_nums, int T, int K, int h,
                      int inter, int E, int gemm_experts, int phase_mask, cudaStream_t stream);

// Same layer with power-of-two scales end to end: dispatch quantises with UE8M0 scale rounding, the
// weights' 128x128 scales must be powers of two, both GEMMs run on the block-scaled tensor-core path.
int cam_fused_moe_mxfp8(CamBuffer* b, const void* x_bf16, const void* expert_ids, int idx_is_i64,
                        const float* topk_weights, const void* w1_q, const float* w1_s, const void* w2_q,
                        const float* w2_s, void* out_bf16, int64_t* expert_token_nums, int T, int K, int h,
                        int inter, int E, int gemm_experts, int phase_mask, cudaStream_t stream);

// Exact W8A8 (kernels/grouped_gemm_i8.cu): int8 activations [rows, K] with one fp32 scale per row, int8
// weights [E, N, K] (K contiguous) with one fp32 scale per output channel [E, N], int32 accumulation.
int cam_grouped_gemm_w8a8(const void* a_q, const float* a_scales, int a_rows, const void* w_q, const float* w_scales,
                          const int* expert_offsets, int num_experts, int n_dim, int k_dim, void* out_bf16,
                          cudaStream_t stream);
// The fused layer in that arithmetic: dispatch with per-token int8 quantisation, GEMM1 -> fp32 SwiGLU +
// row maxima -> per-token int8 requantisation -> GEMM2 with combine-send epilogue -> reduce.
// w1_q [E_local, 2I, h], w1_s [E_local, 2I], w2_q [E_local, h, I], w2_s [E_local, h].
int cam_fused_moe_w8a8(CamBuffer* b, const void* x_bf16, const void* expert_ids, int idx_is_i64,
                       const float* topk_weights, const void* w1_q, const float* w1_s, const void* w2_q,
                       const float* w2_s, void* out_bf16, int64_t* expert_token_nums, int T, int K, int h, int inter,
                       int E, int gemm_experts, int phase_mask, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
