// Plain-C types shared by the host runtime, the kernel launchers and the device code.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Error codes a kernel can record in its status word.  A kernel never traps: every wait has a
// budget, and when it runs out the kernel writes {code, who, detail}, abandons the remaining
// work and returns, so the CUDA context stays usable and the host can raise an exception.
enum CamStatusCode {
    CAM_OK = 0,
    CAM_ERR_TIMEOUT_COUNT_FLAG = 1,    // peer never delivered its per-expert counts
    CAM_ERR_TIMEOUT_DATA_FLAG = 2,     // peer never signalled "all rows for you are written"
    CAM_ERR_TIMEOUT_COMBINE_FLAG = 3,  // peer never signalled its combine rows
    CAM_ERR_RECV_OVERFLOW = 4,         // rows routed to one rank exceed the buffer capacity
    CAM_ERR_TIMEOUT_PIPELINE = 5,      // mbarrier wait inside the GEMM pipeline ran out
    CAM_ERR_TIMEOUT_LL_CELL = 6,       // low-latency count cell never arrived
    CAM_ERR_TIMEOUT_BARRIER = 7,       // device barrier across ranks ran out
    CAM_ERR_BAD_INDEX = 8,             // debug bounds check recorded an out-of-range index
    CAM_ERR_TIMEOUT_ARRIVAL = 9,       // fused layer: the rows of one local expert never all arrived
    CAM_ERR_TIMEOUT_GEMM1 = 10,        // fused layer: the first GEMM of a row block never completed
};

typedef struct CamStatus {
    int32_t code;    // CamStatusCode, first error wins
    int32_t who;     // peer rank / expert the waiter was waiting for
    int32_t detail;  // extra value (observed flag, row count, ...)
    int32_t block;   // blockIdx.x that recorded the error
} CamStatus;

// Quantisation carried by dispatch.
enum CamQuantMode {
    CAM_QUANT_NONE = 0,        // rows travel as bf16
    CAM_QUANT_INT8_TOKEN = 2,  // per-token dynamic int8 + one fp32 scale per row
    CAM_QUANT_FP8_1x128 = 3,   // e4m3 + one fp32 scale per 128 contiguous hidden elements
    CAM_QUANT_FP8_1x128_UE8M0 = 4,  // same layout, scales rounded up to powers of two (tensor-core block scaling)
};

// Phases of the comm kernels.  A real multi-GPU call runs all phases in one launch.  The
// single-GPU "virtual rank" test mode launches phase by phase for all ranks in turn, so no
// launch ever waits for a launch that has not run yet.
#define CAM_QUANT_IS_FP8(q) ((q) == CAM_QUANT_FP8_1x128 || (q) == CAM_QUANT_FP8_1x128_UE8M0)

enum CamPhase {
    CAM_PHASE_COUNT = 1,  // dispatch: histogram, slots, count all-gather
    CAM_PHASE_SEND = 2,   // dispatch: wait counts, push rows, raise data flags / combine: push rows
    CAM_PHASE_RECV = 4,   // dispatch: wait data flags / combine: wait flags + weighted reduce
    CAM_PHASE_ALL = 7,
};

#define CAM_GUARD_BYTES 64
#define CAM_MAX_RANKS 72
#define CAM_MAX_EXPERTS 1024
#define CAM_MAX_TOPK 16

// Byte offsets of the regions inside every rank's symmetric allocation (identical on all ranks).
typedef struct CamLayout {
    int32_t num_ranks;
    int32_t num_experts;      // routed experts the buffer is sized for (upper bound)
    int32_t max_tokens;       // tokens per rank, normal mode
    int32_t hidden;           // hidden size upper bound
    int32_t topk;             // top-k upper bound
    int32_t capacity;         // rows of the normal-mode receive buffer
    int32_t ll_max_tokens;    // tokens per rank, low-latency mode (0 = no low-latency regions)
    int32_t tp_rows;          // rows of the tensor-parallel exchange region (0 = none)
    uint64_t off_count_flag;    // u32[CAM_MAX_RANKS]
    uint64_t off_data_flag;     // u32[CAM_MAX_RANKS]
    uint64_t off_combine_flag;  // u32[CAM_MAX_RANKS]
    uint64_t off_barrier_flag;  // u32[CAM_MAX_RANKS]
    uint64_t off_ll_combine_flag;  // u32[CAM_MAX_RANKS]
    uint64_t off_count_matrix;  // i32[2][R][E]
    uint64_t off_ll_cells;      // u64[2][R * E_local]   (cell index = src * E_local + local expert)
    uint64_t off_recv_x;        // u8[capacity][hidden*2]
    uint64_t off_recv_scales;   // f32[capacity][hidden/128]
    uint64_t off_recv_src;      // i32[capacity][3]
    uint64_t off_combine_buf;   // bf16[max_tokens][topk][hidden]
    uint64_t off_ll_x;          // u8[2][E cells][ll_max_tokens][hidden*2]
    uint64_t off_ll_scales;     // f32[2][E cells][ll_max_tokens][hidden/128]
    uint64_t off_ll_meta;       // i32[2][E cells][ll_max_tokens][2]
    uint64_t off_ll_combine_buf;  // bf16[ll_max_tokens][topk][hidden]
    uint64_t off_tp_flag;       // u32[2]: all-gather, reduce-scatter
    uint64_t off_tp_cnt;        // u32[2]
    uint64_t off_tp_x;          // u8[tp_rows][hidden*2]
    uint64_t off_tp_scales;     // f32[tp_rows][hidden/128]
    uint64_t off_dup_cnt;       // u32[2][CAM_MAX_RANKS]: replicate-list lengths per source (normal dispatch)
    uint64_t off_dup_list;      // i32[2][R][max_tokens*topk][2]: (row that arrived, row to copy it to)
    uint64_t off_arrival;       // u32[2][E]: rows that have landed per local expert (fused layer, parity of the epoch)
    // Guard words (CAM_GUARD_BYTES of 0xA5 each) directly behind the four regions that peers write rows into: recv_x,
    // recv_scales, recv_src, combine_buf.  Nothing ever writes them; cam_buffer_check_guards tells if something did.
    uint64_t off_guard0, off_guard1, off_guard2, off_guard3;
    uint64_t total_bytes;
} CamLayout;

#ifdef __cplusplus
}
#endif
