// Allocation-free single-rank dispatch.  This entry point has no counterpart in the reference.
//
// Who it is for: code that must not, or cannot, allocate device memory when it wants tokens
// grouped by expert -- a plug-in running inside a host application whose memory pool owns the
// whole GPU, a caller on a real-time path where cudaMalloc's implicit device synchronisation
// is unacceptable, or a C program that links this library without PyTorch and without the
// Buffer object (which allocates its workspace up front with cudaMalloc).
//
// What it does: the single-rank form of normal-mode dispatch.  Every valid (token, k) pair of
// `topk_idx` becomes one output row; rows are ordered by expert, and inside an expert by the
// (token-major) scan order of the pairs -- the same order, bit for bit the same rows, scales and
// (0, token, k) source triples as dispatch on a one-rank Buffer produces.
//
// How it avoids allocating: the kernel's scratch (per-CTA expert histograms, the slot of every
// pair inside its expert, per-expert bases, a status word) lives in one file-scope
// `static __device__` array of CAM_NOALLOC_SCRATCH_BYTES inside the library.  Every GPU whose
// context loads the library holds that array until the process exits.  The entry point calls
// no cudaMalloc, cudaFree or any allocating library routine.
//
// Limits (a call outside them is rejected with a message, nothing is launched):
//   tokens * topk <= CAM_NOALLOC_MAX_PAIRS, experts <= CAM_NOALLOC_MAX_EXPERTS,
//   topk <= 16, hidden a multiple of 128 and <= 8192, quant_mode in {0, 2, 3, 4} (4: e4m3 with power-of-two scales),
//   x, recv_x and recv_scales 16-byte aligned (rows move as 16-byte vectors), the integer arrays aligned to
//   their element size,
//   `capacity` (rows the caller's outputs can hold) >= the number of valid pairs, else the call
//   returns CAM_NOALLOC_OVERFLOW after the kernel ran without writing any row.
// Expert ids outside [0, experts) are skipped; a 64-bit id is compared as 64 bits (2^32 + 3 is not expert 3).
//
// Sharing: all calls on a device use the same scratch array.  The kernel rewrites every word it
// later reads, so nothing has to be cleared between calls, but two calls that overlap on the GPU
// (different streams, or different host threads) race on it -- serialise them.
//
// First call on a device: it looks up the array's device address (cudaGetSymbolAddress with
// that device current) and sizes the launch; make that first call outside any stream capture.
// The call is asynchronous on `stream`; `cam_dispatch_local_noalloc_status` synchronises the
// stream it is given and returns the status the last call on the current device recorded.  Pass
// it the stream of that call: on any other stream the read is not ordered after the kernel.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CAM_NOALLOC_MAX_PAIRS (8192 * 16)
#define CAM_NOALLOC_MAX_EXPERTS 1024
#define CAM_NOALLOC_MAX_GRID 160
#define CAM_NOALLOC_SCRATCH_BYTES                                                          \
    (4u * CAM_NOALLOC_MAX_GRID * CAM_NOALLOC_MAX_EXPERTS /* per-CTA histograms */ +          \
     4u * CAM_NOALLOC_MAX_PAIRS /* slot of every pair */ + 4u * CAM_NOALLOC_MAX_EXPERTS + 256u)

#define CAM_NOALLOC_OK 0
#define CAM_NOALLOC_BAD_ARGUMENT (-1)
#define CAM_NOALLOC_CUDA_ERROR (-2)
#define CAM_NOALLOC_OVERFLOW (-3)

// x          [tokens, hidden] bf16 (device)          topk_idx [tokens, topk] int64 or int32 (device)
// recv_x     [capacity, hidden] bf16 (quant 0) or 1-byte elements (quant 2: int8, 3 and 4: e4m3)
// recv_scales[capacity, hidden/128] (quant 3, 4) or [capacity] (quant 2); may be NULL for quant 0
// recv_src   [capacity, 3] int32: (0, token, k) of every row
// expert_offsets [experts + 1] int32: first row of every expert, last entry = number of rows
// Returns CAM_NOALLOC_OK or a negative code; cam_dispatch_local_noalloc_error() has the text.
int cam_dispatch_local_noalloc(const void* x, const void* topk_idx, int idx_is_i64, int tokens, int topk,
                               int hidden, int experts, int quant_mode, int capacity, void* recv_x,
                               float* recv_scales, int32_t* recv_src, int32_t* expert_offsets,
                               cudaStream_t stream);
int cam_dispatch_local_noalloc_status(cudaStream_t stream);
const char* cam_dispatch_local_noalloc_error(void);

#ifdef __cplusplus
}
#endif
