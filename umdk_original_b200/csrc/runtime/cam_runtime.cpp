// Host runtime: symmetric buffers over CUDA IPC, peer tables, epochs, status, TMA descriptors and
// the host halves of the ops.  Argument checks mirror the reference's tiling-time validation
// (moe_dispatch_normal_tiling.cc:88-108, moe_dispatch_shmem_tiling.cpp:83-92,
// fused_deep_moe_tiling.cpp:49-58) with limits that fit one NVSwitch domain.
#include "cam_runtime.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "../kernels/launch.h"

namespace {

thread_local std::string g_last_error;

int fail(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return -1;
}

#define CAM_CUDA(call)                                                                      \
    do {                                                                                    \
        cudaError_t e__ = (call);                                                           \
        if (e__ != cudaSuccess) return fail("%s failed: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

#define CAM_CHECK(cond, ...)                   \
    do {                                       \
        if (!(cond)) return fail(__VA_ARGS__); \
    } while (0)

uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }
// Floats between two rows of activation scales on the deep-fused route: the fused kernel reads a row four K-blocks
// (16 bytes) at a time.
uint64_t scale_row_pitch(uint64_t blocks) { return align_up(blocks, 4); }

}  // namespace

struct CamBuffer {
    int device = 0, rank = 0, num_ranks = 1;
    CamLayout layout{};
    uint8_t* base = nullptr;             // own symmetric allocation
    std::vector<uint8_t*> peer_ptr;      // host copy of the peer table
    std::vector<bool> peer_is_ipc;
    uint8_t** d_peer_table = nullptr;    // device copy
    int tp_rank = 0;                     // position in the tensor-parallel pair
    uint8_t* tp_peer = nullptr;          // the TP partner's symmetric allocation (null without TP)
    bool tp_peer_is_ipc = false;
    // workspace (local)
    int grid_dispatch = 0, grid_combine = 0, num_sms = 0;
    int* cta_hist = nullptr;
    int* slot_in_expert = nullptr;
    int* send_row = nullptr;
    int* recv_count = nullptr;
    int* expert_offsets = nullptr;
    int64_t* num_recv_per_expert = nullptr;
    int* total_recv = nullptr;
    int* num_tokens_per_expert = nullptr;
    unsigned int* done_ctr = nullptr;  // [4]: dispatch, combine, gemm, spare
    unsigned int* dup_ctr = nullptr;   // [CAM_MAX_RANKS] replicate-list cursors of normal dispatch (self-resetting)
    CamStatus* d_status = nullptr;
    CamStatus* h_status = nullptr;  // pinned
    uint8_t* act_q = nullptr;       // [capacity, hidden] scratch between the two GEMMs (sized for I <= hidden)
    float* act_s = nullptr;
    float* act_f32 = nullptr;       // [capacity, hidden] fp32 SwiGLU output of the int8 path (allocated on first use)
    float* row_amax = nullptr;      // [capacity]
    // Epochs live on the device (a kernel reads counter + 1 and its last CTA stores it back), so the
    // host passes no per-call value and captured CUDA graphs can be replayed.
    // [0..2] normal dispatch count/send/recv, [3..4] combine send/recv, [5..6] low-latency dispatch
    // send/recv, [7..8] low-latency combine send/recv.
    uint32_t* d_epochs = nullptr;     // [16]
    unsigned int* exit_ctr = nullptr;  // [4]: dispatch, combine, low-latency dispatch, spare
    uint64_t timeout_ns = 10ull * 1000ull * 1000ull * 1000ull;
    int dbg_drop_flags = 0;
    // per-stage device timing of the fused layer (off by default): events around the four launches
    unsigned long long* d_trace = nullptr;  // [2][8] in-kernel timelines: low-latency dispatch, combine (null = off)
    bool profile = false;
    bool profile_valid = false;
    cudaEvent_t prof_ev[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    // deep-fused layer (allocated on first use): quantised tokens, send list, per-row-block counters, optional trace
    uint8_t* xq = nullptr;
    float* xs = nullptr;
    int4* send_list = nullptr;
    int* send_list_len = nullptr;
    uint32_t* g1_done = nullptr;
    int g1_done_len = 0;
    unsigned long long* fused_trace = nullptr;  // [E + 1], null = off
    unsigned long long launches = 0;            // kernels this buffer's ops have launched (host-side count)
    cam::CamStatsDev* d_stats = nullptr;        // per-peer waits and routed rows (normal-mode ops)
    // switches read from the environment once, when the buffer is created (UMDK_CAM_GEMM_*, UMDK_CAM_DEEP_FUSE):
    // -1 = not set (the runtime decides), 0 / 1 = forced
    int env_bulk_push = -1, env_pair = -1, env_swap = -1, env_staging2 = -1, env_deep_fuse = -1, env_fuse_lag = -1;
    std::map<std::tuple<const void*, uint64_t, uint64_t>, std::pair<CUtensorMap, uint64_t>> tmap_cache;  // map, last use
    uint64_t tmap_clock = 0;
    std::map<std::tuple<int, int, int, int>, int> ll_grid_cache;  // (h, quant, T, K) -> co-resident grid
};

extern "C" const char* cam_last_error(void) { return g_last_error.c_str(); }

extern "C" const char* cam_status_string(int code) {
    switch (code) {
        case CAM_OK: return "ok";
        case CAM_ERR_TIMEOUT_COUNT_FLAG: return "timeout waiting for a peer's per-expert counts";
        case CAM_ERR_TIMEOUT_DATA_FLAG: return "timeout waiting for a peer's dispatch completion flag";
        case CAM_ERR_TIMEOUT_COMBINE_FLAG: return "timeout waiting for a peer's combine completion flag";
        case CAM_ERR_RECV_OVERFLOW: return "rows routed to one rank or cell exceed the buffer capacity";
        case CAM_ERR_TIMEOUT_PIPELINE: return "timeout inside the GEMM pipeline (mbarrier wait)";
        case CAM_ERR_TIMEOUT_LL_CELL: return "timeout waiting for a low-latency count cell";
        case CAM_ERR_TIMEOUT_BARRIER: return "timeout in the cross-rank barrier";
        case CAM_ERR_BAD_INDEX: return "index out of range recorded by a device-side check";
        case CAM_ERR_TIMEOUT_ARRIVAL: return "timeout waiting for the rows of one local expert to arrive (fused layer)";
        case CAM_ERR_TIMEOUT_GEMM1: return "timeout waiting for the first GEMM of a row block (fused layer)";
        default: return "unknown status";
    }
}

extern "C" int cam_layout_compute_tp(CamLayout* L, int R, int E, int max_tokens, int hidden, int topk, int capacity,
                                     int ll_max_tokens, int tp_rows);

extern "C" int cam_layout_compute(CamLayout* L, int R, int E, int max_tokens, int hidden, int topk, int capacity,
                                  int ll_max_tokens) {
    return cam_layout_compute_tp(L, R, E, max_tokens, hidden, topk, capacity, ll_max_tokens, 0);
}

extern "C" int cam_layout_compute_tp(CamLayout* L, int R, int E, int max_tokens, int hidden, int topk, int capacity,
                                     int ll_max_tokens, int tp_rows) {
    CAM_CHECK(L != nullptr, "layout: null output");
    CAM_CHECK(R >= 1 && R <= CAM_MAX_RANKS, "layout: num_ranks %d outside [1, %d]", R, CAM_MAX_RANKS);
    CAM_CHECK(E >= R && E <= CAM_MAX_EXPERTS && E % R == 0, "layout: num_experts %d must be a multiple of num_ranks %d and <= %d",
              E, R, CAM_MAX_EXPERTS);
    CAM_CHECK(topk >= 1 && topk <= CAM_MAX_TOPK, "layout: topk %d outside [1, %d]", topk, CAM_MAX_TOPK);
    CAM_CHECK(hidden >= 128 && hidden % 128 == 0 && hidden <= 16384, "layout: hidden %d must be a multiple of 128 in [128, 16384]", hidden);
    CAM_CHECK(max_tokens >= 1 && capacity >= 1 && ll_max_tokens >= 0 && tp_rows >= 0, "layout: bad token counts");
    memset(L, 0, sizeof(*L));
    L->num_ranks = R;
    L->num_experts = E;
    L->max_tokens = max_tokens;
    L->hidden = hidden;
    L->topk = topk;
    L->capacity = capacity;
    L->ll_max_tokens = ll_max_tokens;
    L->tp_rows = tp_rows;
    uint64_t off = 0;
    auto take = [&](uint64_t bytes) {
        uint64_t o = off;
        off = align_up(off + bytes, 1024);
        return o;
    };
    L->off_count_flag = take(sizeof(uint32_t) * CAM_MAX_RANKS);
    L->off_data_flag = take(sizeof(uint32_t) * CAM_MAX_RANKS);
    L->off_combine_flag = take(sizeof(uint32_t) * CAM_MAX_RANKS);
    L->off_barrier_flag = take(sizeof(uint32_t) * CAM_MAX_RANKS);
    L->off_ll_combine_flag = take(sizeof(uint32_t) * CAM_MAX_RANKS);
    L->off_tp_flag = take(sizeof(uint32_t) * 2);
    L->off_tp_cnt = take(sizeof(uint32_t) * 2);
    L->off_dup_cnt = take(sizeof(uint32_t) * 2ull * CAM_MAX_RANKS);
    L->off_count_matrix = take(sizeof(int32_t) * 2ull * R * E);
    L->off_ll_cells = take(sizeof(uint64_t) * 2ull * E);
    L->off_arrival = take(sizeof(uint32_t) * 2ull * E);
    const uint64_t ctrl_end = off;
    (void)ctrl_end;
    // every region peers push rows into is followed, byte for byte, by a guard block
    auto take_guarded = [&](uint64_t bytes, uint64_t* guard) {
        uint64_t o = off;
        *guard = align_up(off + bytes, 16);
        off = align_up(*guard + CAM_GUARD_BYTES, 1024);
        return o;
    };
    L->off_recv_x = take_guarded(static_cast<uint64_t>(capacity) * hidden * 2, &L->off_guard0);
    // sized for scale rows padded to whole 128-byte lines (the fused layer's layout); the stand-alone ops pack them
    L->off_recv_scales = take_guarded(static_cast<uint64_t>(capacity) * scale_row_pitch(hidden / 128) * 4, &L->off_guard1);
    L->off_recv_src = take_guarded(static_cast<uint64_t>(capacity) * 3 * 4, &L->off_guard2);
    L->off_combine_buf = take_guarded(static_cast<uint64_t>(max_tokens) * topk * hidden * 2, &L->off_guard3);
    L->off_dup_list = take(2ull * R * static_cast<uint64_t>(max_tokens) * topk * 8);
    if (tp_rows > 0) {
        L->off_tp_x = take(static_cast<uint64_t>(tp_rows) * hidden * 2);
        L->off_tp_scales = take(static_cast<uint64_t>(tp_rows) * (hidden / 128) * 4);
    }
    if (ll_max_tokens > 0) {
        const uint64_t cells = 2ull * E;
        L->off_ll_x = take(cells * ll_max_tokens * hidden * 2);
        L->off_ll_scales = take(cells * ll_max_tokens * (hidden / 128) * 4);
        L->off_ll_meta = take(cells * ll_max_tokens * 2 * 4);
        L->off_ll_combine_buf = take(static_cast<uint64_t>(ll_max_tokens) * topk * hidden * 2);
    }
    L->total_bytes = off;
    return 0;
}

extern "C" CamBuffer* cam_buffer_create(int device, int rank, int num_ranks, const CamLayout* layout) {
    auto bad = [](const char* what, cudaError_t e) -> CamBuffer* {
        fail("%s failed: %s", what, cudaGetErrorString(e));
        return nullptr;
    };
    if (layout == nullptr || layout->num_ranks != num_ranks || rank < 0 || rank >= num_ranks) {
        fail("buffer_create: bad rank/layout");
        return nullptr;
    }
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return bad("cudaSetDevice", e);
    CamBuffer* b = new CamBuffer();
    b->device = device;
    b->rank = rank;
    b->num_ranks = num_ranks;
    b->layout = *layout;
    auto env_switch = [](const char* name) {
        const char* v = getenv(name);
        return (v == nullptr || v[0] == '\0') ? -1 : atoi(v);
    };
    b->env_bulk_push = env_switch("UMDK_CAM_GEMM_BULK_PUSH");
    b->env_pair = env_switch("UMDK_CAM_GEMM_PAIR");
    b->env_swap = env_switch("UMDK_CAM_GEMM_SWAP");
    b->env_staging2 = env_switch("UMDK_CAM_GEMM_STAGING2");
    b->env_deep_fuse = env_switch("UMDK_CAM_DEEP_FUSE");
    b->env_fuse_lag = env_switch("UMDK_CAM_FUSE_LAG");
    const int E = layout->num_experts, R = num_ranks;
    if ((e = cudaDeviceGetAttribute(&b->num_sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) {
        delete b;
        return bad("cudaDeviceGetAttribute", e);
    }
    if ((e = cudaMalloc(&b->base, layout->total_bytes)) != cudaSuccess) {
        delete b;
        return bad("cudaMalloc(symmetric region)", e);
    }
    // control words (everything before recv_x) start at zero
    cudaMemset(b->base, 0, layout->off_recv_x);
    for (uint64_t g : {layout->off_guard0, layout->off_guard1, layout->off_guard2, layout->off_guard3})
        cudaMemset(b->base + g, 0xA5, CAM_GUARD_BYTES);
    b->peer_ptr.assign(R, nullptr);
    b->peer_is_ipc.assign(R, false);
    b->peer_ptr[rank] = b->base;
    const size_t pairs = static_cast<size_t>(layout->max_tokens > layout->ll_max_tokens ? layout->max_tokens
                                                                                        : layout->ll_max_tokens) *
                         layout->topk;
    bool ok = true;
    ok &= cudaMalloc(&b->d_peer_table, sizeof(uint8_t*) * R) == cudaSuccess;
    ok &= cudaMalloc(&b->cta_hist, sizeof(int) * static_cast<size_t>(b->num_sms) * E) == cudaSuccess;
    ok &= cudaMalloc(&b->slot_in_expert, sizeof(int) * pairs) == cudaSuccess;
    ok &= cudaMalloc(&b->send_row, sizeof(int) * pairs) == cudaSuccess;
    ok &= cudaMalloc(&b->recv_count, sizeof(int) * E) == cudaSuccess;
    ok &= cudaMalloc(&b->expert_offsets, sizeof(int) * (E + 1)) == cudaSuccess;
    ok &= cudaMalloc(&b->num_recv_per_expert, sizeof(int64_t) * E) == cudaSuccess;
    ok &= cudaMalloc(&b->total_recv, sizeof(int) * 4) == cudaSuccess;
    ok &= cudaMalloc(&b->num_tokens_per_expert, sizeof(int) * E) == cudaSuccess;
    ok &= cudaMalloc(&b->done_ctr, sizeof(unsigned int) * 4) == cudaSuccess;
    ok &= cudaMalloc(&b->dup_ctr, sizeof(unsigned int) * CAM_MAX_RANKS) == cudaSuccess;
    ok &= cudaMalloc(&b->d_epochs, sizeof(uint32_t) * 16) == cudaSuccess;
    ok &= cudaMalloc(&b->exit_ctr, sizeof(unsigned int) * 4) == cudaSuccess;
    ok &= cudaMalloc(&b->d_status, sizeof(CamStatus)) == cudaSuccess;
    ok &= cudaMallocHost(&b->h_status, sizeof(CamStatus)) == cudaSuccess;
    ok &= cudaMalloc(&b->d_stats, sizeof(cam::CamStatsDev)) == cudaSuccess;
    ok &= cudaMalloc(&b->act_q, static_cast<size_t>(layout->capacity) * layout->hidden) == cudaSuccess;
    ok &= cudaMalloc(&b->act_s, static_cast<size_t>(layout->capacity) * scale_row_pitch(layout->hidden / 128) * 4) == cudaSuccess;
    if (!ok) {
        fail("buffer_create: workspace allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
        cam_buffer_destroy(b);
        return nullptr;
    }
    cudaMemset(b->d_stats, 0, sizeof(cam::CamStatsDev));
    cudaMemset(b->done_ctr, 0, sizeof(unsigned int) * 4);
    cudaMemset(b->dup_ctr, 0, sizeof(unsigned int) * CAM_MAX_RANKS);
    cudaMemset(b->d_epochs, 0, sizeof(uint32_t) * 16);
    cudaMemset(b->exit_ctr, 0, sizeof(unsigned int) * 4);
    cudaMemset(b->d_status, 0, sizeof(CamStatus));
    cudaMemset(b->total_recv, 0, sizeof(int) * 4);
    cudaMemset(b->expert_offsets, 0, sizeof(int) * (E + 1));
    memset(b->h_status, 0, sizeof(CamStatus));
    cudaMemcpy(b->d_peer_table, b->peer_ptr.data(), sizeof(uint8_t*) * R, cudaMemcpyHostToDevice);
    cudaDeviceSynchronize();
    return b;
}

extern "C" int cam_buffer_destroy(CamBuffer* b) {
    if (b == nullptr) return 0;
    cudaSetDevice(b->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < b->num_ranks; ++r)
        if (r != b->rank && b->peer_is_ipc[r] && b->peer_ptr[r] != nullptr) cudaIpcCloseMemHandle(b->peer_ptr[r]);
    if (b->tp_peer != nullptr && b->tp_peer_is_ipc) cudaIpcCloseMemHandle(b->tp_peer);
    void* frees[] = {b->base, b->d_peer_table, b->cta_hist, b->slot_in_expert, b->send_row, b->recv_count,
                     b->expert_offsets, b->num_recv_per_expert, b->total_recv, b->num_tokens_per_expert,
                     b->done_ctr, b->dup_ctr, b->d_epochs, b->exit_ctr, b->d_status, b->act_q, b->act_s};
    for (void* p : frees)
        if (p != nullptr) cudaFree(p);
    if (b->h_status != nullptr) cudaFreeHost(b->h_status);
    if (b->d_stats != nullptr) cudaFree(b->d_stats);
    if (b->d_trace != nullptr) cudaFree(b->d_trace);
    if (b->act_f32 != nullptr) cudaFree(b->act_f32);
    if (b->row_amax != nullptr) cudaFree(b->row_amax);
    for (void* p : {static_cast<void*>(b->xq), static_cast<void*>(b->xs), static_cast<void*>(b->send_list),
                    static_cast<void*>(b->send_list_len), static_cast<void*>(b->g1_done),
                    static_cast<void*>(b->fused_trace)})
        if (p != nullptr) cudaFree(p);
    for (auto e : b->prof_ev)
        if (e != nullptr) cudaEventDestroy(e);
    delete b;
    return 0;
}

extern "C" int cam_buffer_ipc_handle(CamBuffer* b, void* out_handle) {
    CAM_CHECK(b != nullptr && out_handle != nullptr, "ipc_handle: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == CAM_IPC_HANDLE_BYTES, "IPC handle size");
    cudaIpcMemHandle_t h;
    CAM_CUDA(cudaSetDevice(b->device));
    CAM_CUDA(cudaIpcGetMemHandle(&h, b->base));
    memcpy(out_handle, &h, sizeof(h));
    return 0;
}

static int upload_peer_table(CamBuffer* b) {
    for (int r = 0; r < b->num_ranks; ++r) CAM_CHECK(b->peer_ptr[r] != nullptr, "peer %d has no mapping", r);
    CAM_CUDA(cudaMemcpy(b->d_peer_table, b->peer_ptr.data(), sizeof(uint8_t*) * b->num_ranks, cudaMemcpyHostToDevice));
    return 0;
}

extern "C" int cam_buffer_open_ipc_peers(CamBuffer* b, const void* handles) {
    CAM_CHECK(b != nullptr && handles != nullptr, "open_ipc_peers: null argument");
    CAM_CUDA(cudaSetDevice(b->device));
    const uint8_t* hp = static_cast<const uint8_t*>(handles);
    for (int r = 0; r < b->num_ranks; ++r) {
        if (r == b->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, hp + static_cast<size_t>(r) * CAM_IPC_HANDLE_BYTES, sizeof(h));
        void* p = nullptr;
        CAM_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        b->peer_ptr[r] = static_cast<uint8_t*>(p);
        b->peer_is_ipc[r] = true;
    }
    return upload_peer_table(b);
}

extern "C" int cam_buffer_set_local_peers(CamBuffer* b, CamBuffer* const* peers) {
    CAM_CHECK(b != nullptr && peers != nullptr, "set_local_peers: null argument");
    CAM_CUDA(cudaSetDevice(b->device));
    for (int r = 0; r < b->num_ranks; ++r) {
        CAM_CHECK(peers[r] != nullptr && peers[r]->device == b->device && peers[r]->rank == r &&
                      peers[r]->layout.total_bytes == b->layout.total_bytes,
                  "set_local_peers: peer %d is not a matching buffer on the same device", r);
        b->peer_ptr[r] = peers[r]->base;
        b->peer_is_ipc[r] = false;
    }
    return upload_peer_table(b);
}

extern "C" int cam_buffer_reset(CamBuffer* b, cudaStream_t stream) {
    CAM_CHECK(b != nullptr, "reset: null buffer");
    CAM_CUDA(cudaSetDevice(b->device));
    CAM_CUDA(cudaMemsetAsync(b->base, 0, b->layout.off_recv_x, stream));
    CAM_CUDA(cudaMemsetAsync(b->done_ctr, 0, sizeof(unsigned int) * 4, stream));
    CAM_CUDA(cudaMemsetAsync(b->dup_ctr, 0, sizeof(unsigned int) * CAM_MAX_RANKS, stream));
    CAM_CUDA(cudaMemsetAsync(b->d_epochs, 0, sizeof(uint32_t) * 16, stream));
    CAM_CUDA(cudaMemsetAsync(b->exit_ctr, 0, sizeof(unsigned int) * 4, stream));
    CAM_CUDA(cudaMemsetAsync(b->d_status, 0, sizeof(CamStatus), stream));
    CAM_CUDA(cudaStreamSynchronize(stream));
    return 0;
}

extern "C" void* cam_buffer_base(CamBuffer* b) { return b ? b->base : nullptr; }
extern "C" const CamLayout* cam_buffer_layout(CamBuffer* b) { return b ? &b->layout : nullptr; }
extern "C" int cam_buffer_rank(CamBuffer* b) { return b ? b->rank : -1; }
extern "C" int cam_buffer_num_ranks(CamBuffer* b) { return b ? b->num_ranks : -1; }
extern "C" int cam_buffer_device(CamBuffer* b) { return b ? b->device : -1; }
extern "C" int cam_buffer_tp_rank(CamBuffer* b) { return b ? b->tp_rank : -1; }
extern "C" void cam_buffer_set_timeout_ms(CamBuffer* b, double ms) {
    if (b != nullptr && ms > 0) b->timeout_ns = static_cast<uint64_t>(ms * 1e6);
}
// In-kernel timeline of the low-latency dispatch and of combine (globaltimer stamps of CTA 0, see
// trace_point in ptx.cuh).  read_trace synchronises the device and copies 2 x 8 stamps (ns).
extern "C" int cam_buffer_set_trace(CamBuffer* b, int on) {
    CAM_CHECK(b != nullptr, "set_trace: null buffer");
    CAM_CUDA(cudaSetDevice(b->device));
    if (on && b->d_trace == nullptr) {
        CAM_CUDA(cudaMalloc(&b->d_trace, sizeof(unsigned long long) * 16));
        CAM_CUDA(cudaMemset(b->d_trace, 0, sizeof(unsigned long long) * 16));
    } else if (!on && b->d_trace != nullptr) {
        CAM_CUDA(cudaDeviceSynchronize());
        CAM_CUDA(cudaFree(b->d_trace));
        b->d_trace = nullptr;
    }
    return 0;
}
extern "C" int cam_buffer_read_trace(CamBuffer* b, unsigned long long* out16) {
    CAM_CHECK(b != nullptr && out16 != nullptr && b->d_trace != nullptr, "read_trace: tracing is off");
    CAM_CUDA(cudaSetDevice(b->device));
    CAM_CUDA(cudaDeviceSynchronize());
    CAM_CUDA(cudaMemcpy(out16, b->d_trace, sizeof(unsigned long long) * 16, cudaMemcpyDeviceToHost));
    return 0;
}
// Timeline of the deep-fused layer: for every local expert the time (ns after the fused kernel started) at which
// its first GEMM was released because all of its rows had arrived; 0 = never released.  Off by default.
extern "C" int cam_buffer_set_fused_trace(CamBuffer* b, int on) {
    CAM_CHECK(b != nullptr, "set_fused_trace: null buffer");
    CAM_CUDA(cudaSetDevice(b->device));
    const size_t bytes = sizeof(unsigned long long) * (b->layout.num_experts + 8);
    if (on && b->fused_trace == nullptr) {
        CAM_CUDA(cudaMalloc(&b->fused_trace, bytes));
        CAM_CUDA(cudaMemset(b->fused_trace, 0, bytes));
    } else if (!on && b->fused_trace != nullptr) {
        CAM_CUDA(cudaDeviceSynchronize());
        CAM_CUDA(cudaFree(b->fused_trace));
        b->fused_trace = nullptr;
    }
    return 0;
}
extern "C" int cam_buffer_read_fused_trace(CamBuffer* b, long long* out, int num_local_experts) {
    CAM_CHECK(b != nullptr && out != nullptr && b->fused_trace != nullptr, "read_fused_trace: tracing is off");
    CAM_CHECK(num_local_experts >= 1 && num_local_experts <= b->layout.num_experts, "read_fused_trace: bad expert count");
    CAM_CUDA(cudaSetDevice(b->device));
    CAM_CUDA(cudaDeviceSynchronize());
    std::vector<unsigned long long> t(num_local_experts + 1);
    CAM_CUDA(cudaMemcpy(t.data(), b->fused_trace, sizeof(unsigned long long) * (num_local_experts + 1), cudaMemcpyDeviceToHost));
    const unsigned long long t0 = t[num_local_experts];
    for (int e = 0; e < num_local_experts; ++e)
        out[e] = t[e] == 0ull ? -1ll : static_cast<long long>(t[e] - t0);
    return 0;
}
// What the MMA issuer of the first CTA pair waited for during the last traced fused kernel, in clock cycles:
// {whole loop, accumulator drained, scale factors, operand tiles, K-blocks issued, tiles}.
extern "C" int cam_buffer_read_fused_waits(CamBuffer* b, long long* out6, int num_local_experts) {
    CAM_CHECK(b != nullptr && out6 != nullptr && b->fused_trace != nullptr, "read_fused_waits: tracing is off");
    CAM_CUDA(cudaSetDevice(b->device));
    CAM_CUDA(cudaDeviceSynchronize());
    CAM_CUDA(cudaMemcpy(out6, b->fused_trace + num_local_experts + 1, sizeof(long long) * 7, cudaMemcpyDeviceToHost));
    return 0;
}
extern "C" int cam_buffer_set_profile(CamBuffer* b, int on) {
    CAM_CHECK(b != nullptr, "set_profile: null buffer");
    CAM_CUDA(cudaSetDevice(b->device));
    if (on && b->prof_ev[0] == nullptr)
        for (auto& e : b->prof_ev) CAM_CUDA(cudaEventCreate(&e));
    b->profile = on != 0;
    b->profile_valid = false;
    return 0;
}
extern "C" int cam_buffer_read_profile(CamBuffer* b, float* ms4) {
    CAM_CHECK(b != nullptr && ms4 != nullptr, "read_profile: null argument");
    CAM_CHECK(b->profile_valid, "read_profile: no fused layer has run with profiling on");
    CAM_CUDA(cudaSetDevice(b->device));
    CAM_CUDA(cudaEventSynchronize(b->prof_ev[4]));
    for (int i = 0; i < 4; ++i) CAM_CUDA(cudaEventElapsedTime(&ms4[i], b->prof_ev[i], b->prof_ev[i + 1]));
    return 0;
}
extern "C" void cam_buffer_set_debug_drop_flags(CamBuffer* b, int on) {
    if (b != nullptr) b->dbg_drop_flags = on ? 1 : 0;
}
// Guard blocks behind the receive regions: *damaged gets one bit per guard (0: recv_x, 1: recv_scales, 2: recv_src,
// 3: combine_buf) whose bytes are no longer 0xA5, i.e. something wrote past the end of that region.  Synchronises
// `stream`.  Damaged guards are restored, so one overrun is reported once.
extern "C" int cam_buffer_check_guards(CamBuffer* b, cudaStream_t stream, int* damaged) {
    CAM_CHECK(b != nullptr && damaged != nullptr, "check_guards: null argument");
    CAM_CUDA(cudaSetDevice(b->device));
    const uint64_t offs[4] = {b->layout.off_guard0, b->layout.off_guard1, b->layout.off_guard2, b->layout.off_guard3};
    unsigned char host[4][CAM_GUARD_BYTES];
    for (int i = 0; i < 4; ++i)
        CAM_CUDA(cudaMemcpyAsync(host[i], b->base + offs[i], CAM_GUARD_BYTES, cudaMemcpyDeviceToHost, stream));
    CAM_CUDA(cudaStreamSynchronize(stream));
    *damaged = 0;
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < CAM_GUARD_BYTES; ++j)
            if (host[i][j] != 0xA5) {
                *damaged |= 1 << i;
                break;
            }
    for (int i = 0; i < 4; ++i)
        if (*damaged & (1 << i)) CAM_CUDA(cudaMemsetAsync(b->base + offs[i], 0xA5, CAM_GUARD_BYTES, stream));
    return 0;
}

// Statistics of the normal-mode ops since the buffer was created or since the last call with reset = 1 (synchronises the
// device).  out_wait_ns: [3][num_ranks] longest wait for every peer's dispatch counts / dispatch rows / combine rows (ns);
// out_rows: [num_ranks] (token, k) pairs routed to every rank; out_calls: [2] dispatches, combines.
extern "C" int cam_buffer_read_stats(CamBuffer* b, unsigned long long* out_wait_ns, unsigned long long* out_rows,
                                     unsigned long long* out_calls, int reset) {
    CAM_CHECK(b != nullptr && out_wait_ns && out_rows && out_calls, "read_stats: null argument");
    CAM_CUDA(cudaSetDevice(b->device));
    CAM_CUDA(cudaDeviceSynchronize());
    cam::CamStatsDev h;
    CAM_CUDA(cudaMemcpy(&h, b->d_stats, sizeof(h), cudaMemcpyDeviceToHost));
    for (int k = 0; k < 3; ++k)
        for (int r = 0; r < b->num_ranks; ++r) out_wait_ns[k * b->num_ranks + r] = h.max_wait_ns[k][r];
    for (int r = 0; r < b->num_ranks; ++r) out_rows[r] = h.rows_routed[r];
    out_calls[0] = h.calls[0];
    out_calls[1] = h.calls[1];
    if (reset) CAM_CUDA(cudaMemset(b->d_stats, 0, sizeof(h)));
    return 0;
}

extern "C" unsigned long long cam_buffer_launch_count(CamBuffer* b) { return b ? b->launches : 0ull; }
extern "C" int* cam_buffer_recv_count(CamBuffer* b) { return b->recv_count; }
extern "C" int* cam_buffer_expert_offsets(CamBuffer* b) { return b->expert_offsets; }
extern "C" int64_t* cam_buffer_num_recv_per_expert(CamBuffer* b) { return b->num_recv_per_expert; }
extern "C" int* cam_buffer_total_recv(CamBuffer* b) { return b->total_recv; }
extern "C" int* cam_buffer_send_row(CamBuffer* b) { return b->send_row; }
extern "C" int* cam_buffer_num_tokens_per_expert(CamBuffer* b) { return b->num_tokens_per_expert; }
extern "C" uint8_t* cam_buffer_act_q(CamBuffer* b) { return b->act_q; }
extern "C" float* cam_buffer_act_s(CamBuffer* b) { return b->act_s; }

extern "C" int cam_buffer_poll_status(CamBuffer* b, cudaStream_t stream, CamStatus* out) {
    CAM_CHECK(b != nullptr && out != nullptr, "poll_status: null argument");
    CAM_CUDA(cudaSetDevice(b->device));
    CAM_CUDA(cudaMemcpyAsync(b->h_status, b->d_status, sizeof(CamStatus), cudaMemcpyDeviceToHost, stream));
    CAM_CUDA(cudaStreamSynchronize(stream));
    *out = *b->h_status;
    if (out->code != CAM_OK) {
        CAM_CUDA(cudaMemsetAsync(b->d_status, 0, sizeof(CamStatus), stream));
        CAM_CUDA(cudaMemsetAsync(b->done_ctr, 0, sizeof(unsigned int) * 4, stream));
        CAM_CUDA(cudaMemsetAsync(b->dup_ctr, 0, sizeof(unsigned int) * CAM_MAX_RANKS, stream));
        CAM_CUDA(cudaMemsetAsync(b->exit_ctr, 0, sizeof(unsigned int) * 4, stream));
        CAM_CUDA(cudaStreamSynchronize(stream));
    }
    return 0;
}

// Tensor-parallel partner (tpWorldSize = 2): the rank at the same expert-parallel position of the other TP group.
extern "C" int cam_buffer_open_ipc_tp_peer(CamBuffer* b, const void* handle, int tp_rank) {
    CAM_CHECK(b != nullptr && handle != nullptr && (tp_rank == 0 || tp_rank == 1), "open_ipc_tp_peer: bad argument");
    CAM_CHECK(b->layout.tp_rows > 0, "open_ipc_tp_peer: the buffer was created without a tensor-parallel region");
    CAM_CUDA(cudaSetDevice(b->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    CAM_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    b->tp_peer = static_cast<uint8_t*>(p);
    b->tp_peer_is_ipc = true;
    b->tp_rank = tp_rank;
    return 0;
}

extern "C" int cam_buffer_set_local_tp_peer(CamBuffer* b, CamBuffer* peer, int tp_rank) {
    CAM_CHECK(b != nullptr && peer != nullptr && (tp_rank == 0 || tp_rank == 1), "set_local_tp_peer: bad argument");
    CAM_CHECK(b->layout.tp_rows > 0 && peer->layout.total_bytes == b->layout.total_bytes && peer->device == b->device,
              "set_local_tp_peer: the partner must be a buffer of the same layout on the same device");
    b->tp_peer = peer->base;
    b->tp_peer_is_ipc = false;
    b->tp_rank = tp_rank;
    return 0;
}

static int tp_exchange(CamBuffer* b, int reduce, const void* rows, const float* scales, int row_bytes, int nscale,
                       const int* n_own, const int* n_peer, void* out, float* scales_out, int out_rows, int* tp_counts,
                       int phase_mask, cudaStream_t stream) {
    CAM_CHECK(b != nullptr && b->tp_peer != nullptr, "tp exchange: the buffer has no tensor-parallel partner");
    CAM_CHECK(row_bytes > 0 && row_bytes % 16 == 0 && row_bytes <= b->layout.hidden * 2, "tp exchange: bad row size %d", row_bytes);
    CAM_CUDA(cudaSetDevice(b->device));
    cam::TpExchangeParams p{};
    p.reduce = reduce;
    p.rows = static_cast<const uint8_t*>(rows);
    p.scales = scales;
    p.row_bytes = row_bytes;
    p.nscale = nscale;
    p.n_own = n_own;
    p.n_peer = n_peer;
    p.max_rows = b->layout.tp_rows;
    p.out = static_cast<uint8_t*>(out);
    p.scales_out = scales_out;
    p.out_rows = out_rows;
    p.tp_counts = tp_counts;
    p.tp_rank = b->tp_rank;
    p.my_base = b->base;
    p.peer_base = b->tp_peer;
    p.off_tp_flag = b->layout.off_tp_flag;
    p.off_tp_cnt = b->layout.off_tp_cnt;
    p.off_tp_x = b->layout.off_tp_x;
    p.off_tp_scales = b->layout.off_tp_scales;
    p.epochs = b->d_epochs + (reduce ? 13 : 11);
    p.exit_ctr = b->exit_ctr + 3;
    p.done_ctr = b->done_ctr + 3;
    p.timeout_ns = b->timeout_ns;
    p.phase_mask = phase_mask;
    p.dbg_drop_flags = b->dbg_drop_flags;
    p.status = b->d_status;
    const int rc = cam_launch_tp_exchange(&p, b->num_sms, stream);
    CAM_CHECK(rc == 0, "tp exchange launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    if (b != nullptr) ++b->launches;
    return 0;
}

// After low-latency dispatch: appends the TP partner's received rows (and scales) behind this rank's own
// n_own rows in `rows` / `scales` (which must hold out_rows rows) and writes the two counts.
extern "C" int cam_tp_allgather(CamBuffer* b, void* rows, float* scales, int row_bytes, int nscale, const int* n_own,
                                int out_rows, int* tp_counts, int phase_mask, cudaStream_t stream) {
    return tp_exchange(b, 0, rows, scales, row_bytes, nscale, n_own, n_own, rows, scales, out_rows, tp_counts, phase_mask,
                       stream);
}

// Before combine: y holds partial outputs for [my n_own rows | the partner's n_peer rows]; sends the
// partner its rows, adds what the partner sends for mine, result in out [n_own rows].
extern "C" int cam_tp_reduce_scatter(CamBuffer* b, const void* y, int row_bytes, const int* n_own, const int* n_peer,
                                     void* out, int phase_mask, cudaStream_t stream) {
    return tp_exchange(b, 1, y, nullptr, row_bytes, 0, n_own, n_peer, out, nullptr, 0, nullptr, phase_mask, stream);
}

// Device barrier over all ranks of the buffer (epochs [9..10]).  Enqueued on `stream`; returns at once.
extern "C" int cam_buffer_barrier(CamBuffer* b, int phase_mask, cudaStream_t stream) {
    CAM_CHECK(b != nullptr, "barrier: null buffer");
    CAM_CUDA(cudaSetDevice(b->device));
    const int rc = cam_launch_barrier(b->d_peer_table, b->layout.off_barrier_flag, b->d_epochs + 9, b->num_ranks, b->rank,
                                      phase_mask, b->dbg_drop_flags, b->timeout_ns, b->d_status, stream);
    CAM_CHECK(rc == 0, "barrier launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    if (b != nullptr) ++b->launches;
    return 0;
}

// P2P microbenchmark pieces.  write: copies `bytes` from this rank's receive region into the same
// region of `peer` with `grid` CTAs (0 = one per SM).  pingpong: `iters` flag round trips with `peer`
// on the pair's barrier-flag words; `base` must grow by at least `iters` from call to call.
extern "C" int cam_buffer_p2p_write(CamBuffer* b, int peer, size_t bytes, int grid, cudaStream_t stream) {
    CAM_CHECK(b != nullptr && peer >= 0 && peer < b->num_ranks, "p2p_write: bad peer");
    const size_t region = static_cast<size_t>(b->layout.capacity) * b->layout.hidden * 2;
    CAM_CHECK(bytes > 0 && bytes <= region && bytes % 512 == 0, "p2p_write: bytes must be a multiple of 512 within the receive region (%zu)", region);
    CAM_CUDA(cudaSetDevice(b->device));
    const int rc = cam_launch_p2p_copy(b->peer_ptr[peer] + b->layout.off_recv_x, b->base + b->layout.off_recv_x, bytes,
                                       grid > 0 ? grid : b->num_sms, stream);
    CAM_CHECK(rc == 0, "p2p_write launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    return 0;
}

extern "C" int cam_buffer_p2p_pingpong(CamBuffer* b, int peer, unsigned int base, int iters, int initiator,
                                       cudaStream_t stream) {
    CAM_CHECK(b != nullptr && peer >= 0 && peer < b->num_ranks && peer != b->rank, "p2p_pingpong: bad peer");
    CAM_CUDA(cudaSetDevice(b->device));
    // word CAM_MAX_RANKS - 1 - x of the count-flag array is never used by the ops for groups below that size
    CAM_CHECK(b->num_ranks < CAM_MAX_RANKS - 1, "p2p_pingpong: group too large");
    uint32_t* mine = reinterpret_cast<uint32_t*>(b->base + b->layout.off_count_flag) + (CAM_MAX_RANKS - 1);
    uint32_t* theirs = reinterpret_cast<uint32_t*>(b->peer_ptr[peer] + b->layout.off_count_flag) + (CAM_MAX_RANKS - 1);
    const int rc = cam_launch_p2p_pingpong(mine, theirs, base, iters, initiator, b->timeout_ns, b->d_status, stream);
    CAM_CHECK(rc == 0, "p2p_pingpong launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    return 0;
}

extern "C" int cam_get_dispatch_layout(const void* topk_idx, int idx_is_i64, int T, int K, int E, int R,
                                       int* num_tokens_per_rank, int* num_tokens_per_expert,
                                       uint8_t* is_token_in_rank, cudaStream_t stream) {
    CAM_CHECK(R >= 1 && R <= CAM_MAX_RANKS, "get_dispatch_layout: num_ranks %d outside [1, %d]", R, CAM_MAX_RANKS);
    CAM_CHECK(E >= R && E <= CAM_MAX_EXPERTS && E % R == 0, "get_dispatch_layout: num_experts %d vs num_ranks %d", E, R);
    CAM_CHECK(K >= 1 && K <= CAM_MAX_TOPK, "get_dispatch_layout: topk %d outside [1, %d]", K, CAM_MAX_TOPK);
    CAM_CHECK(T >= 0, "get_dispatch_layout: negative token count");
    const int rc = cam_launch_layout(topk_idx, idx_is_i64, T, K, E, R, num_tokens_per_rank, num_tokens_per_expert,
                                     is_token_in_rank, stream);
    CAM_CHECK(rc == 0, "layout kernel launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    return 0;
}

static int check_common(const CamBuffer* b, int T, int K, int h, int E, const char* op) {
    CAM_CHECK(b != nullptr, "%s: null buffer", op);
    const CamLayout& L = b->layout;
    CAM_CHECK(E >= b->num_ranks && E <= L.num_experts && E % b->num_ranks == 0,
              "%s: num_experts %d must be a multiple of num_ranks %d and <= %d (buffer)", op, E, b->num_ranks, L.num_experts);
    CAM_CHECK(K >= 1 && K <= L.topk, "%s: topk %d outside [1, %d (buffer)]", op, K, L.topk);
    CAM_CHECK(h >= 128 && h <= L.hidden && h % 128 == 0, "%s: hidden %d must be a multiple of 128 and <= %d (buffer)", op, h, L.hidden);
    CAM_CHECK(T >= 0, "%s: negative token count", op);
    return 0;
}

// Workspace of the deep-fused layer, allocated on the first call that takes that route.
static int ensure_deep_workspace(CamBuffer* b) {
    if (b->xq != nullptr) return 0;
    const CamLayout& L = b->layout;
    CAM_CUDA(cudaSetDevice(b->device));
    const size_t pairs = static_cast<size_t>(L.max_tokens) * L.topk;
    b->g1_done_len = L.capacity / 256 + L.num_experts + 2;
    CAM_CUDA(cudaMalloc(&b->xq, static_cast<size_t>(L.max_tokens) * L.hidden));
    CAM_CUDA(cudaMalloc(&b->xs, static_cast<size_t>(L.max_tokens) * (L.hidden / 128) * sizeof(float)));
    CAM_CUDA(cudaMalloc(&b->send_list, pairs * sizeof(int4)));
    CAM_CUDA(cudaMalloc(&b->send_list_len, sizeof(int)));
    CAM_CUDA(cudaMalloc(&b->g1_done, sizeof(uint32_t) * b->g1_done_len));
    CAM_CUDA(cudaMemset(b->send_list_len, 0, sizeof(int)));
    CAM_CUDA(cudaMemset(b->g1_done, 0, sizeof(uint32_t) * b->g1_done_len));
    return 0;
}

static int dispatch_normal_impl(CamBuffer* b, const void* x, const void* topk_idx, int idx_is_i64, int T, int K, int h,
                                int E, int quant_mode, int phase_mask, bool defer_push, cudaStream_t stream) {
    if (check_common(b, T, K, h, E, "dispatch_normal") != 0) return -1;
    CAM_CHECK(T <= b->layout.max_tokens, "dispatch_normal: %d tokens exceed the buffer's max_tokens %d", T, b->layout.max_tokens);
    CAM_CHECK(quant_mode == CAM_QUANT_NONE || quant_mode == CAM_QUANT_INT8_TOKEN || CAM_QUANT_IS_FP8(quant_mode),
              "dispatch_normal: quant_mode %d is not one of 0 (bf16), 2 (int8 per token), 3 (fp8 1x128), "
              "4 (fp8 1x128, power-of-two scales)", quant_mode);
    CAM_CUDA(cudaSetDevice(b->device));
    cam::DispatchNormalParams p{};
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.topk_idx = topk_idx;
    p.idx_is_i64 = idx_is_i64;
    p.T = T; p.K = K; p.h = h; p.E = E; p.R = b->num_ranks; p.rank = b->rank;
    p.quant_mode = quant_mode;
    p.capacity = b->layout.capacity;
    p.epochs = b->d_epochs + 0;
    p.exit_ctr = b->exit_ctr + 0;
    p.timeout_ns = b->timeout_ns;
    p.phase_mask = phase_mask;
    p.dbg_drop_flags = b->dbg_drop_flags;
    p.peer_base = b->d_peer_table;
    p.off_count_flag = b->layout.off_count_flag;
    p.off_data_flag = b->layout.off_data_flag;
    p.off_count_matrix = b->layout.off_count_matrix;
    p.off_recv_x = b->layout.off_recv_x;
    p.off_recv_scales = b->layout.off_recv_scales;
    p.off_recv_src = b->layout.off_recv_src;
    p.off_dup_cnt = b->layout.off_dup_cnt;
    p.off_dup_list = b->layout.off_dup_list;
    p.dup_cap = b->layout.max_tokens * b->layout.topk;
    p.dup_ctr = b->dup_ctr;
    p.cta_hist = b->cta_hist;
    p.slot_in_expert = b->slot_in_expert;
    p.send_row = b->send_row;
    p.recv_count = b->recv_count;
    p.expert_offsets = b->expert_offsets;
    p.num_recv_per_expert = b->num_recv_per_expert;
    p.total_recv = b->total_recv;
    p.num_tokens_per_expert_out = b->num_tokens_per_expert;
    p.done_ctr = b->done_ctr + 0;
    p.status = b->d_status;
    p.off_arrival = b->layout.off_arrival;
    p.stats = b->d_stats;
    if (defer_push) {
        CAM_CHECK(CAM_QUANT_IS_FP8(quant_mode), "dispatch_normal: the deferred push carries fp8 rows only");
        if (ensure_deep_workspace(b) != 0) return -1;
        p.defer_push = 1;
        p.xq = b->xq;
        p.xs = b->xs;
        p.send_list = b->send_list;
        p.send_list_len = b->send_list_len;
        p.g1_done = b->g1_done;
        p.g1_done_len = b->g1_done_len;
    } else if (b->g1_done != nullptr) {
        // the fused kernel may follow this dispatch as a GEMM-only launch: its row-block counters start at zero
        p.g1_done = b->g1_done;
        p.g1_done_len = b->g1_done_len;
    }
    // The count matrix is laid out for layout.num_experts; a call with fewer experts still uses
    // stride E because every rank of the call passes the same E.
    int grid = b->num_sms;  // fixed per device so that the COUNT and SEND phases agree on token chunks
    const int rc = cam_launch_dispatch_normal(&p, grid, stream);
    CAM_CHECK(rc == 0, "dispatch_normal launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    if (b != nullptr) ++b->launches;
    return 0;
}

extern "C" int cam_dispatch_normal(CamBuffer* b, const void* x, const void* topk_idx, int idx_is_i64, int T, int K,
                                   int h, int E, int quant_mode, int phase_mask, cudaStream_t stream) {
    return dispatch_normal_impl(b, x, topk_idx, idx_is_i64, T, K, h, E, quant_mode, phase_mask, false, stream);
}

extern "C" int cam_combine(CamBuffer* b, const void* y, const int* row_src, const int* total_rows,
                           const void* topk_idx, int idx_is_i64, const float* topk_weights, void* out, int T, int K,
                           int h, int E, int low_latency, int comm_quant, int phase_mask, cudaStream_t stream) {
    if (check_common(b, T, K, h, E, "combine") != 0) return -1;
    const int maxT = low_latency ? b->layout.ll_max_tokens : b->layout.max_tokens;
    CAM_CHECK(T <= maxT, "combine: %d tokens exceed the buffer's limit %d", T, maxT);
    CAM_CHECK(comm_quant == 0 || comm_quant == 2, "combine: comm_quant %d must be 0 (bf16) or 2 (int8 per 128)", comm_quant);
    CAM_CUDA(cudaSetDevice(b->device));
    cam::CombineParams p{};
    p.y = static_cast<const __nv_bfloat16*>(y);
    p.row_src = row_src;
    p.total_rows = total_rows;
    p.topk_idx = topk_idx;
    p.idx_is_i64 = idx_is_i64;
    p.topk_weights = topk_weights;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.T = T; p.K = K; p.h = h; p.E = E; p.R = b->num_ranks; p.rank = b->rank;
    p.comm_quant = comm_quant;
    p.max_tokens = maxT;
    p.epochs = b->d_epochs + (low_latency ? 7 : 3);
    p.exit_ctr = b->exit_ctr + 1;
    p.trace = b->d_trace ? b->d_trace + 8 : nullptr;
    p.timeout_ns = b->timeout_ns;
    p.phase_mask = phase_mask;
    p.dbg_drop_flags = b->dbg_drop_flags;
    p.peer_base = b->d_peer_table;
    p.off_combine_buf = low_latency ? b->layout.off_ll_combine_buf : b->layout.off_combine_buf;
    p.off_combine_flag = low_latency ? b->layout.off_ll_combine_flag : b->layout.off_combine_flag;
    p.done_ctr = b->done_ctr + 1;
    p.status = b->d_status;
    p.stats = low_latency ? nullptr : b->d_stats;
    const int rc = cam_launch_combine(&p, b->num_sms, stream);
    CAM_CHECK(rc == 0, "combine launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    if (b != nullptr) ++b->launches;
    return 0;
}

extern "C" int cam_dispatch_ll(CamBuffer* b, const void* x, const void* expert_ids, int idx_is_i64,
                               const float* smooth, int T, int K, int h, int E, int active_tokens, int quant_mode,
                               int count_type, void* expand_x, float* expand_scales, int* expand_idx,
                               int* expand_src, int64_t* expert_token_nums, int* ep_send_counts, int* total_rows,
                               int phase_mask, cudaStream_t stream) {
    if (check_common(b, T, K, h, E, "dispatch_ll") != 0) return -1;
    CAM_CHECK(b->layout.ll_max_tokens > 0, "dispatch_ll: the buffer was created without low-latency regions");
    CAM_CHECK(T <= b->layout.ll_max_tokens, "dispatch_ll: %d tokens exceed ll_max_tokens %d", T, b->layout.ll_max_tokens);
    CAM_CHECK(E == b->layout.num_experts, "dispatch_ll: num_experts %d must equal the buffer's %d", E, b->layout.num_experts);
    CAM_CHECK(quant_mode == CAM_QUANT_NONE || quant_mode == CAM_QUANT_INT8_TOKEN || CAM_QUANT_IS_FP8(quant_mode),
              "dispatch_ll: quant_mode %d is not one of 0, 2, 3, 4 (static quantisation, mode 1, is not supported)", quant_mode);
    CAM_CHECK(count_type == 0 || count_type == 1, "dispatch_ll: expertTokenNumsType must be 0 (cumulative) or 1 (counts)");
    CAM_CUDA(cudaSetDevice(b->device));
    cam::DispatchLLParams p{};
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.expert_ids = expert_ids;
    p.idx_is_i64 = idx_is_i64;
    p.smooth = smooth;
    p.T = T; p.K = K; p.h = h; p.E = E; p.R = b->num_ranks; p.rank = b->rank;
    p.active_tokens = active_tokens < 0 ? T : active_tokens;
    p.quant_mode = quant_mode;
    p.max_tokens = b->layout.ll_max_tokens;
    p.count_type = count_type;
    p.epochs = b->d_epochs + 5;
    p.exit_ctr = b->exit_ctr + 2;
    p.trace = b->d_trace;
    p.slot_table_bytes = cam_dispatch_ll_slot_table_bytes(T, K, E);
    p.timeout_ns = b->timeout_ns;
    p.phase_mask = phase_mask;
    p.dbg_drop_flags = b->dbg_drop_flags;
    p.peer_base = b->d_peer_table;
    p.off_ll_cells = b->layout.off_ll_cells;
    p.off_ll_x = b->layout.off_ll_x;
    p.off_ll_scales = b->layout.off_ll_scales;
    p.off_ll_meta = b->layout.off_ll_meta;
    p.expand_x = static_cast<uint8_t*>(expand_x);
    p.expand_scales = expand_scales;
    p.expand_idx = expand_idx;
    p.expand_src = expand_src;
    p.expert_token_nums = expert_token_nums;
    p.ep_send_counts = ep_send_counts;
    p.total_rows = total_rows;
    p.status = b->d_status;
    int grid;
    const auto gkey = std::make_tuple(h, quant_mode, T, K);
    auto git = b->ll_grid_cache.find(gkey);
    if (git != b->ll_grid_cache.end()) {
        grid = git->second;
    } else {
        grid = cam_dispatch_ll_max_grid(b->device, h, quant_mode, T, K, E);
        b->ll_grid_cache[gkey] = grid;
    }
    CAM_CHECK(grid > 0, "dispatch_ll: kernel does not fit (shared memory for T=%d K=%d h=%d)", T, K, h);
    // one token per CTA when sending, one row per warp when packing: no more CTAs than that needs
    // (a smaller grid makes the grid-wide barrier cheaper)
    int want = (T * K + 15) / 16;
    if (want < T) want = T;
    if (want < 8) want = 8;
    if (grid > want) grid = want;
    const int rc = cam_launch_dispatch_ll(&p, grid, stream);
    CAM_CHECK(rc == 0, "dispatch_ll launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    if (b != nullptr) ++b->launches;
    return 0;
}

// ---------------------------------------------------------------------------------------------
// TMA descriptors
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

constexpr size_t kTmapCacheEntries = 64;

// 2-D byte tensor [rows, inner] with row pitch == inner, boxes of 128 bytes x 128 rows, 128-byte swizzle.
static int make_tmap(CamBuffer* cache_owner, CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows) {
    if (cache_owner != nullptr) {
        auto it = cache_owner->tmap_cache.find(std::make_tuple(base, inner, rows));
        if (it != cache_owner->tmap_cache.end()) {
            *out = it->second.first;
            it->second.second = ++cache_owner->tmap_clock;
            return 0;
        }
    }
    EncodeTiledFn fn = get_encode_fn();
    CAM_CHECK(fn != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
    CAM_CHECK((reinterpret_cast<uintptr_t>(base) & 15u) == 0, "tensor map base %p is not 16-byte aligned", base);
    CAM_CHECK(inner % 16 == 0 && inner >= 128, "tensor map inner extent %llu must be a multiple of 16 and >= 128",
              static_cast<unsigned long long>(inner));
    CAM_CHECK(rows >= 1, "tensor map needs at least one row");
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {inner};
    cuuint32_t box[2] = {128, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CAM_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    if (cache_owner != nullptr) {
        // bounded: when full, the entry used longest ago makes room (a layer uses four to six maps per call)
        if (cache_owner->tmap_cache.size() >= kTmapCacheEntries) {
            auto oldest = cache_owner->tmap_cache.begin();
            for (auto c = cache_owner->tmap_cache.begin(); c != cache_owner->tmap_cache.end(); ++c)
                if (c->second.second < oldest->second.second) oldest = c;
            cache_owner->tmap_cache.erase(oldest);
        }
        cache_owner->tmap_cache[std::make_tuple(base, inner, rows)] = std::make_pair(*out, ++cache_owner->tmap_clock);
    }
    return 0;
}

// Mean rows per expert below which the block-scaled GEMM runs with its operands exchanged (0 = never by default).
constexpr int kSwapRowsPerExpert = 0;

static int grouped_gemm_impl(CamBuffer* b, const void* a_q, const float* a_scales, int a_rows, const void* w_q,
                             const float* w_scales, const int* expert_offsets, int num_experts, int n_dim, int k_dim,
                             int mode, void* out_bf16, void* act_q, float* act_s, const int* row_src, int topk,
                             int low_latency, bool ue8m0, int rows_per_expert_hint, cudaStream_t stream) {
    CAM_CHECK(a_q && a_scales && w_q && w_scales && expert_offsets, "grouped_gemm: null operand");
    CAM_CHECK(num_experts >= 1 && a_rows >= 1, "grouped_gemm: empty problem");
    CAM_CHECK(k_dim >= 128 && k_dim % 128 == 0, "grouped_gemm: K %d must be a multiple of 128", k_dim);
    CAM_CHECK(mode >= 0 && mode <= 2, "grouped_gemm: mode %d", mode);
    if (mode == 1) {
        CAM_CHECK(n_dim % 256 == 0, "grouped_gemm: gate+up width %d must be a multiple of 256", n_dim);
        CAM_CHECK(act_q && act_s, "grouped_gemm: mode 1 needs act_q / act_s");
    } else {
        CAM_CHECK(n_dim % 128 == 0, "grouped_gemm: N %d must be a multiple of 128", n_dim);
    }
    if (mode == 0) CAM_CHECK(out_bf16 != nullptr, "grouped_gemm: mode 0 needs an output");
    if (mode == 2) CAM_CHECK(b != nullptr && row_src != nullptr && topk >= 1, "grouped_gemm: mode 2 needs a buffer, row_src and topk");
    CAM_CHECK(static_cast<uint64_t>(num_experts) * n_dim < (1ull << 31), "grouped_gemm: weight rows overflow");
    int device = 0;
    if (b != nullptr) {
        CAM_CUDA(cudaSetDevice(b->device));
        device = b->device;
    } else {
        CAM_CUDA(cudaGetDevice(&device));
    }
    CUtensorMap ta, tb;
    if (make_tmap(b, &ta, a_q, static_cast<uint64_t>(k_dim), static_cast<uint64_t>(a_rows)) != 0) return -1;
    if (make_tmap(b, &tb, w_q, static_cast<uint64_t>(k_dim), static_cast<uint64_t>(num_experts) * n_dim) != 0) return -1;
    cam::GroupedGemmParams p{};
    p.expert_offsets = expert_offsets;
    p.num_experts = num_experts;
    p.n_dim = n_dim;
    p.k_dim = k_dim;
    p.a_rows = a_rows;
    p.a_scales = a_scales;
    p.b_scales = w_scales;
    p.mode = mode;
    p.out = static_cast<__nv_bfloat16*>(out_bf16);
    p.act_q = static_cast<uint8_t*>(act_q);
    p.act_s = act_s;
    p.row_src = row_src;
    // stand-alone calls (no Buffer): one status word and counter per device, allocated on that device's first call
    static CamStatus* s_fallback_status_dev[64] = {nullptr};
    static unsigned int* s_fallback_ctr_dev[64] = {nullptr};
    if (b == nullptr) CAM_CHECK(device >= 0 && device < 64, "grouped_gemm: device index %d not supported", device);
    CamStatus*& s_fallback_status = s_fallback_status_dev[b ? 0 : device];
    unsigned int*& s_fallback_ctr = s_fallback_ctr_dev[b ? 0 : device];
    if (b != nullptr) {
        p.peer_base = b->d_peer_table;
        p.off_combine_buf = low_latency ? b->layout.off_ll_combine_buf : b->layout.off_combine_buf;
        p.off_combine_flag = low_latency ? b->layout.off_ll_combine_flag : b->layout.off_combine_flag;
        p.num_ranks = b->num_ranks;
        p.rank = b->rank;
        p.dbg_drop_flags = b->dbg_drop_flags;
        p.done_ctr = b->done_ctr + 2;
        p.status = b->d_status;
        p.epoch_send = b->d_epochs + (low_latency ? 7 : 3);
        p.max_tokens = low_latency ? b->layout.ll_max_tokens : b->layout.max_tokens;
    } else {
        if (s_fallback_status == nullptr) {
            CAM_CUDA(cudaMalloc(&s_fallback_status, sizeof(CamStatus)));
            CAM_CUDA(cudaMemset(s_fallback_status, 0, sizeof(CamStatus)));
            CAM_CUDA(cudaMalloc(&s_fallback_ctr, sizeof(unsigned int)));
            CAM_CUDA(cudaMemset(s_fallback_ctr, 0, sizeof(unsigned int)));
        }
        p.status = s_fallback_status;
        p.done_ctr = s_fallback_ctr;
    }
    p.topk = topk;
    int sms = 0;
    CAM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    // Switches: a Buffer reads UMDK_CAM_GEMM_* once when it is created; the stand-alone ops (no Buffer) read the
    // environment per call.  -1 = not set.
    auto env_now = [](const char* name) {
        const char* v = getenv(name);
        return (v == nullptr || v[0] == '\0') ? -1 : atoi(v);
    };
    const int sw_bulk = b ? b->env_bulk_push : env_now("UMDK_CAM_GEMM_BULK_PUSH");
    const int sw_pair = b ? b->env_pair : env_now("UMDK_CAM_GEMM_PAIR");
    const int sw_swap = b ? b->env_swap : env_now("UMDK_CAM_GEMM_SWAP");
    const int sw_stg2 = b ? b->env_staging2 : env_now("UMDK_CAM_GEMM_STAGING2");
    // rows leave the GEMM2 epilogue as 256-byte bulk copies (measured a few percent ahead of vector stores at 2 and 4
    // GPUs); UMDK_CAM_GEMM_BULK_PUSH=0 selects the vector-store form
    p.bulk_push = sw_bulk < 0 ? 1 : (sw_bulk == 1);
    // CTA pairs (256-row tiles, B tile shared inside the cluster) pay off once experts fill such tiles;
    // UMDK_CAM_GEMM_PAIR=0/1 forces the choice.
    bool pair = ue8m0 && rows_per_expert_hint >= 384;
    if (sw_pair >= 0) pair = ue8m0 && sw_pair == 1;
    // Small experts (a tile of rows or less each) take the kernel with the operands exchanged, whose tensor-core
    // time follows the rows actually present instead of whole 128-row tiles; UMDK_CAM_GEMM_SWAP=0/1 forces the choice.
    bool swap = ue8m0 && !pair && rows_per_expert_hint < kSwapRowsPerExpert;
    if (sw_swap >= 0) swap = ue8m0 && !pair && sw_swap == 1;
    // The combine-send epilogue of the block-scaled kernels overlaps converting a half tile with the copies of the previous
    // one (two staging buffers, paid for with pipeline stages); UMDK_CAM_GEMM_STAGING2=0 keeps the one-buffer form.
    // On by default in the CTA-pair kernel only: the one-CTA kernel, used for small experts, lives on streaming weights
    // and loses more from its fourth pipeline stage than the epilogue gains (measured on one GPU, 256 experts).
    bool two_staging = mode == 2 && p.bulk_push != 0 && pair;
    if (sw_stg2 >= 0) two_staging = mode == 2 && p.bulk_push != 0 && sw_stg2 == 1;
    const int rc = !ue8m0 ? cam_launch_grouped_gemm_fp8(&p, &ta, &tb, sms, stream)
                   : pair ? cam_launch_grouped_gemm_mxfp8_pair(&p, &ta, &tb, sms, two_staging ? 1 : 0, stream)
                          : cam_launch_grouped_gemm_mxfp8(&p, &ta, &tb, sms, swap ? 1 : 0, two_staging ? 1 : 0, stream);
    CAM_CHECK(rc == 0, "grouped_gemm launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    if (b != nullptr) ++b->launches;
    return 0;
}

extern "C" int cam_grouped_gemm_fp8(CamBuffer* b, const void* a_q, const float* a_scales, int a_rows,
                                    const void* w_q, const float* w_scales, const int* expert_offsets,
                                    int num_experts, int n_dim, int k_dim, int mode, void* out_bf16, void* act_q,
                                    float* act_s, const int* row_src, int topk, int low_latency,
                                    cudaStream_t stream) {
    return grouped_gemm_impl(b, a_q, a_scales, a_rows, w_q, w_scales, expert_offsets, num_experts, n_dim, k_dim, mode,
                             out_bf16, act_q, act_s, row_src, topk, low_latency, false, 0, stream);
}

extern "C" int cam_grouped_gemm_mxfp8(CamBuffer* b, const void* a_q, const float* a_scales, int a_rows,
                                      const void* w_q, const float* w_scales, const int* expert_offsets,
                                      int num_experts, int n_dim, int k_dim, int mode, void* out_bf16, void* act_q,
                                      float* act_s, const int* row_src, int topk, int low_latency,
                                      cudaStream_t stream) {
    return grouped_gemm_impl(b, a_q, a_scales, a_rows, w_q, w_scales, expert_offsets, num_experts, n_dim, k_dim, mode,
                             out_bf16, act_q, act_s, row_src, topk, low_latency, true, num_experts > 0 ? a_rows / num_experts : 0, stream);
}

// ---------------------------------------------------------------------------------------------
// int8 W8A8 path (exact int32 accumulation)
// ---------------------------------------------------------------------------------------------
static int grouped_gemm_w8a8_impl(CamBuffer* b, const void* a_q, const float* a_scales, int a_rows, const void* w_q,
                                  const float* w_scales, const int* expert_offsets, int num_experts, int n_dim,
                                  int k_dim, int mode, void* out_bf16, float* act_f32, float* row_amax,
                                  const int* row_src, int topk, cudaStream_t stream) {
    CAM_CHECK(a_q && a_scales && w_q && w_scales && expert_offsets, "grouped_gemm_w8a8: null operand");
    CAM_CHECK(num_experts >= 1 && a_rows >= 1, "grouped_gemm_w8a8: empty problem");
    CAM_CHECK(k_dim >= 128 && k_dim % 128 == 0, "grouped_gemm_w8a8: K %d must be a multiple of 128", k_dim);
    CAM_CHECK(mode >= 0 && mode <= 2, "grouped_gemm_w8a8: mode %d", mode);
    if (mode == 1) {
        CAM_CHECK(n_dim % 256 == 0 && act_f32 && row_amax, "grouped_gemm_w8a8: mode 1 needs 2I %% 256 == 0 and a workspace");
    } else {
        CAM_CHECK(n_dim % 128 == 0, "grouped_gemm_w8a8: N %d must be a multiple of 128", n_dim);
    }
    if (mode == 0) CAM_CHECK(out_bf16 != nullptr, "grouped_gemm_w8a8: mode 0 needs an output");
    if (mode == 2) CAM_CHECK(b != nullptr && row_src != nullptr && topk >= 1, "grouped_gemm_w8a8: mode 2 needs a buffer");
    int device = 0;
    if (b != nullptr) {
        CAM_CUDA(cudaSetDevice(b->device));
        device = b->device;
    } else {
        CAM_CUDA(cudaGetDevice(&device));
    }
    CUtensorMap ta, tb;
    if (make_tmap(b, &ta, a_q, static_cast<uint64_t>(k_dim), static_cast<uint64_t>(a_rows)) != 0) return -1;
    if (make_tmap(b, &tb, w_q, static_cast<uint64_t>(k_dim), static_cast<uint64_t>(num_experts) * n_dim) != 0) return -1;
    cam::GroupedGemmParams p{};
    p.expert_offsets = expert_offsets;
    p.num_experts = num_experts;
    p.n_dim = n_dim;
    p.k_dim = k_dim;
    p.a_rows = a_rows;
    p.a_scales = a_scales;
    p.b_scales = w_scales;
    p.mode = mode;
    p.out = static_cast<__nv_bfloat16*>(out_bf16);
    p.act_f32 = act_f32;
    p.row_amax = row_amax;
    p.row_src = row_src;
    p.topk = topk;
    static CamStatus* s_status_dev[64] = {nullptr};
    static unsigned int* s_ctr_dev[64] = {nullptr};
    if (b == nullptr) CAM_CHECK(device >= 0 && device < 64, "grouped_gemm_w8a8: device index %d not supported", device);
    CamStatus*& s_status = s_status_dev[b ? 0 : device];
    unsigned int*& s_ctr = s_ctr_dev[b ? 0 : device];
    if (b != nullptr) {
        p.peer_base = b->d_peer_table;
        p.off_combine_buf = b->layout.off_combine_buf;
        p.off_combine_flag = b->layout.off_combine_flag;
        p.num_ranks = b->num_ranks;
        p.rank = b->rank;
        p.dbg_drop_flags = b->dbg_drop_flags;
        p.done_ctr = b->done_ctr + 2;
        p.status = b->d_status;
        p.epoch_send = b->d_epochs + 3;
        p.max_tokens = b->layout.max_tokens;
    } else {
        if (s_status == nullptr) {
            CAM_CUDA(cudaMalloc(&s_status, sizeof(CamStatus)));
            CAM_CUDA(cudaMemset(s_status, 0, sizeof(CamStatus)));
            CAM_CUDA(cudaMalloc(&s_ctr, sizeof(unsigned int)));
            CAM_CUDA(cudaMemset(s_ctr, 0, sizeof(unsigned int)));
        }
        p.status = s_status;
        p.done_ctr = s_ctr;
    }
    int sms = 0;
    CAM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const int rc = cam_launch_grouped_gemm_w8a8(&p, &ta, &tb, sms, stream);
    CAM_CHECK(rc == 0, "grouped_gemm_w8a8 launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    if (b != nullptr) ++b->launches;
    return 0;
}

extern "C" int cam_grouped_gemm_w8a8(const void* a_q, const float* a_scales, int a_rows, const void* w_q,
                                     const float* w_scales, const int* expert_offsets, int num_experts, int n_dim,
                                     int k_dim, void* out_bf16, cudaStream_t stream) {
    return grouped_gemm_w8a8_impl(nullptr, a_q, a_scales, a_rows, w_q, w_scales, expert_offsets, num_experts, n_dim,
                                  k_dim, 0, out_bf16, nullptr, nullptr, nullptr, 1, stream);
}

extern "C" int cam_fused_moe_w8a8(CamBuffer* b, const void* x, const void* expert_ids, int idx_is_i64,
                                  const float* topk_weights, const void* w1_q, const float* w1_s, const void* w2_q,
                                  const float* w2_s, void* out, int64_t* expert_token_nums, int T, int K, int h,
                                  int inter, int E, int gemm_experts, int phase_mask, cudaStream_t stream) {
    if (check_common(b, T, K, h, E, "fused_moe_w8a8") != 0) return -1;
    CAM_CHECK(inter >= 128 && inter % 128 == 0 && inter <= b->layout.hidden,
              "fused_moe_w8a8: intermediate size %d must be a multiple of 128 and <= the buffer's hidden %d", inter, b->layout.hidden);
    CAM_CHECK(w1_q && w1_s && w2_q && w2_s && topk_weights && out, "fused_moe_w8a8: null operand");
    const int El = (gemm_experts > 0 && gemm_experts <= E / b->num_ranks) ? gemm_experts : E / b->num_ranks;
    const CamLayout& L = b->layout;
    CAM_CUDA(cudaSetDevice(b->device));
    if (b->act_f32 == nullptr) {  // first use of the int8 path on this buffer
        CAM_CUDA(cudaMalloc(&b->act_f32, static_cast<size_t>(L.capacity) * L.hidden * sizeof(float)));
        CAM_CUDA(cudaMalloc(&b->row_amax, static_cast<size_t>(L.capacity) * sizeof(float)));
        CAM_CUDA(cudaMemset(b->row_amax, 0, static_cast<size_t>(L.capacity) * sizeof(float)));
    }
    const bool prof = b->profile && phase_mask == 15;
    auto stamp = [&](int i) { if (prof) cudaEventRecord(b->prof_ev[i], stream); };
    stamp(0);
    if (phase_mask & CAM_PHASE_ALL) {
        if (cam_dispatch_normal(b, x, expert_ids, idx_is_i64, T, K, h, E, CAM_QUANT_INT8_TOKEN, phase_mask & CAM_PHASE_ALL,
                                stream) != 0)
            return -1;
    }
    stamp(1);
    if (phase_mask & CAM_PHASE_RECV) {
        const uint8_t* recv_x = b->base + L.off_recv_x;
        const float* recv_s = reinterpret_cast<const float*>(b->base + L.off_recv_scales);
        const int* recv_src = reinterpret_cast<const int*>(b->base + L.off_recv_src);
        if (grouped_gemm_w8a8_impl(b, recv_x, recv_s, L.capacity, w1_q, w1_s, b->expert_offsets, El, 2 * inter, h, 1,
                                   nullptr, b->act_f32, b->row_amax, nullptr, K, stream) != 0)
            return -1;
        const int rc = cam_launch_rowquant_int8(b->act_f32, b->row_amax, b->expert_offsets, El, inter, b->act_q, b->act_s,
                                                stream);
        CAM_CHECK(rc == 0, "rowquant launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    if (b != nullptr) ++b->launches;
        stamp(2);
        if (grouped_gemm_w8a8_impl(b, b->act_q, b->act_s, L.capacity, w2_q, w2_s, b->expert_offsets, El, h, inter, 2,
                                   nullptr, nullptr, nullptr, recv_src, K, stream) != 0)
            return -1;
        if (expert_token_nums != nullptr)
            CAM_CUDA(cudaMemcpyAsync(expert_token_nums, b->num_recv_per_expert, sizeof(int64_t) * El,
                                     cudaMemcpyDeviceToDevice, stream));
    }
    stamp(3);
    if (phase_mask & 8) {
        if (cam_combine(b, nullptr, nullptr, nullptr, expert_ids, idx_is_i64, topk_weights, out, T, K, h, E, 0, 0,
                        CAM_PHASE_RECV, stream) != 0)
            return -1;
    }
    stamp(4);
    if (prof) b->profile_valid = true;
    return 0;
}

// Deep-fused route of the layer: launch 1 exchanges the counts, quantises the tokens locally and writes the
// expert-ordered send list; launch 2 sends the rows, runs both grouped GEMMs as their inputs become complete and
// pushes the outputs into the origins' combine slots; launch 3 is the weighted reduce.
static int fused_moe_deep(CamBuffer* b, const void* x, const void* expert_ids, int idx_is_i64,
                          const float* topk_weights, const void* w1_q, const float* w1_s, const void* w2_q,
                          const float* w2_s, void* out, int64_t* expert_token_nums, int T, int K, int h, int inter,
                          int E, int El, int rows_hint, int phase_mask, bool own_dispatch, cudaStream_t stream) {
    const CamLayout& L = b->layout;
    const bool prof = b->profile && phase_mask == 15;
    auto stamp = [&](int i) { if (prof) cudaEventRecord(b->prof_ev[i], stream); };
    stamp(0);
    // own_dispatch: the fused kernel sends the rows itself, launch 1 only prepares them.  Otherwise launch 1 is the
    // whole normal dispatch and the fused kernel is just the two GEMMs with their tiles interleaved.
    const int prep_mask = own_dispatch ? phase_mask & (CAM_PHASE_COUNT | CAM_PHASE_SEND) : phase_mask & CAM_PHASE_ALL;
    if (prep_mask) {
        if (ensure_deep_workspace(b) != 0) return -1;
        if (dispatch_normal_impl(b, x, expert_ids, idx_is_i64, T, K, h, E, CAM_QUANT_FP8_1x128_UE8M0, prep_mask,
                                 own_dispatch, stream) != 0)
            return -1;
    }
    stamp(1);
    const int fmask = own_dispatch ? phase_mask & (CAM_PHASE_SEND | CAM_PHASE_RECV) : phase_mask & CAM_PHASE_RECV;
    if (fmask) {
        if (ensure_deep_workspace(b) != 0) return -1;
        uint8_t* recv_x = b->base + L.off_recv_x;
        CUtensorMap ta1, tb1, ta2, tb2;
        if (make_tmap(b, &ta1, recv_x, static_cast<uint64_t>(h), static_cast<uint64_t>(L.capacity)) != 0) return -1;
        if (make_tmap(b, &tb1, w1_q, static_cast<uint64_t>(h), static_cast<uint64_t>(El) * 2 * inter) != 0) return -1;
        if (make_tmap(b, &ta2, b->act_q, static_cast<uint64_t>(inter), static_cast<uint64_t>(L.capacity)) != 0) return -1;
        if (make_tmap(b, &tb2, w2_q, static_cast<uint64_t>(inter), static_cast<uint64_t>(El) * h) != 0) return -1;
        const int fit = cam_fused_moe_max_pairs();
        CAM_CHECK(fit > 0, "fused_moe: the fused kernel does not fit on this device");
        cam::FusedMoeParams p{};
        p.expert_offsets = b->expert_offsets;
        p.num_experts = El;
        p.h = h;
        p.inter = inter;
        p.a_rows = L.capacity;
        p.max_tokens = L.max_tokens;
        p.a1_scales = reinterpret_cast<const float*>(b->base + L.off_recv_scales);
        p.a1_scale_pitch = static_cast<int>(scale_row_pitch(h / 128));
        p.act_scale_pitch = static_cast<int>(scale_row_pitch(inter / 128));
        p.b1_scales = w1_s;
        p.b2_scales = w2_s;
        p.act_q = b->act_q;
        p.act_s = b->act_s;
        p.row_src = reinterpret_cast<const int*>(b->base + L.off_recv_src);
        p.peer_base = b->d_peer_table;
        p.off_combine_buf = L.off_combine_buf;
        p.off_combine_flag = L.off_combine_flag;
        p.off_recv_x = L.off_recv_x;
        p.off_recv_scales = L.off_recv_scales;
        p.off_recv_src = L.off_recv_src;
        p.off_arrival = L.off_arrival;
        p.arrival_stride = E;
        p.topk = K;
        p.num_ranks = b->num_ranks;
        p.rank = b->rank;
        p.epoch_send = b->d_epochs + 3;
        p.epoch_dispatch = b->d_epochs + 1;
        p.dbg_drop_flags = b->dbg_drop_flags;
        p.done_ctr = b->done_ctr + 2;
        p.status = b->d_status;
        p.g1_done = b->g1_done;
        p.skip_arrival = own_dispatch ? 0 : 1;
        // The second GEMM of an expert is scheduled `lag` experts behind the first, far enough that the tiles it
        // waits for were started a whole wave of CTA pairs earlier.
        const int tiles1 = ((rows_hint + 255) / 256) * (inter / 128);
        int lag = tiles1 > 0 ? (fit + tiles1 - 1) / tiles1 : 1;
        if (b->env_fuse_lag >= 0) lag = b->env_fuse_lag;
        if (lag < 1) lag = 1;
        if (lag > El) lag = El;
        p.lag = lag;
        p.xq = b->xq;
        p.xs = b->xs;
        p.send_list = b->send_list;
        p.send_list_len = b->send_list_len;
        p.send_list_cap = L.max_tokens * L.topk;
        p.phase_mask = fmask;
        p.timeout_ns = b->timeout_ns;
        p.trace = b->fused_trace;
        if (b->fused_trace != nullptr && (fmask & CAM_PHASE_RECV))
            CAM_CUDA(cudaMemsetAsync(b->fused_trace, 0, sizeof(unsigned long long) * (L.num_experts + 8), stream));
        const int rc = cam_launch_fused_moe(&p, &ta1, &tb1, &ta2, &tb2, b->num_sms, stream);
        CAM_CHECK(rc == 0, "fused_moe launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    if (b != nullptr) ++b->launches;
        if ((fmask & CAM_PHASE_RECV) && expert_token_nums != nullptr)
            CAM_CUDA(cudaMemcpyAsync(expert_token_nums, b->num_recv_per_expert, sizeof(int64_t) * El,
                                     cudaMemcpyDeviceToDevice, stream));
    }
    stamp(2);
    stamp(3);
    if (phase_mask & 8) {
        if (cam_combine(b, nullptr, nullptr, nullptr, expert_ids, idx_is_i64, topk_weights, out, T, K, h, E, 0, 0,
                        CAM_PHASE_RECV, stream) != 0)
            return -1;
    }
    stamp(4);
    if (prof) b->profile_valid = true;
    return 0;
}

// Which route serves the block-scaled fused layer: 0 = four launches, 1 = deep-fused (the fused kernel sends the
// dispatch rows itself), 2 = normal dispatch, then the fused kernel for the two GEMMs.  UMDK_CAM_DEEP_FUSE=0/1/2 (read
// when the Buffer is created) forces one.  Unset, the deep-fused route is taken where it measured faster: on 8 GPUs with
// experts of about a thousand rows (DeepSeek-V3 shapes, 4096 tokens per rank: 1.85 ms against 2.07 ms per layer),
// because seven eighths of the combine rows then cross NVLink and the second GEMM alone cannot hide them, while the
// fused kernel spreads them over both GEMMs.  On 1, 2 and 4 GPUs the four launches measured faster (the two GEMMs inside
// the fused kernel run 7 - 18 % slower than the stand-alone kernels, most on small experts).
// The fused kernel needs power-of-two scales and hidden sizes whose scale rows are whole 16-byte pieces.
static int use_deep_fuse(const CamBuffer* b, bool ue8m0, int h, int inter, int rows_hint) {
    if (!ue8m0 || b->env_deep_fuse == 0) return 0;
    if (!(h % 512 == 0 && h <= 7168 && inter % 128 == 0)) return 0;
    if (b->env_deep_fuse == 1 || b->env_deep_fuse == 2) return b->env_deep_fuse;
    return (b->num_ranks >= 8 && rows_hint >= 768) ? 1 : 0;
}

extern "C" int cam_buffer_fused_route(CamBuffer* b, int T, int K, int h, int inter, int E) {
    if (b == nullptr || E <= 0) return 0;
    const int rows_hint = static_cast<int>(static_cast<int64_t>(T) * K * b->num_ranks / E);
    return use_deep_fuse(b, true, h, inter, rows_hint);
}

static int fused_moe_impl(CamBuffer* b, const void* x, const void* expert_ids, int idx_is_i64,
                          const float* topk_weights, const void* w1_q, const float* w1_s, const void* w2_q,
                          const float* w2_s, void* out, int64_t* expert_token_nums, int T, int K, int h, int inter,
                          int E, int gemm_experts, int phase_mask, bool ue8m0, cudaStream_t stream) {
    if (check_common(b, T, K, h, E, "fused_moe_fp8") != 0) return -1;
    CAM_CHECK(inter >= 128 && inter % 128 == 0 && inter <= b->layout.hidden,
              "fused_moe_fp8: intermediate size %d must be a multiple of 128 and <= the buffer's hidden %d", inter, b->layout.hidden);
    CAM_CHECK(w1_q && w1_s && w2_q && w2_s && topk_weights && out, "fused_moe_fp8: null operand");
    // local experts that have weights: E / R, or fewer on a shared-expert rank (1: only its first
    // local expert ever receives rows)
    const int El = (gemm_experts > 0 && gemm_experts <= E / b->num_ranks) ? gemm_experts : E / b->num_ranks;
    const CamLayout& L = b->layout;
    // mean rows per local expert when routing is balanced: every rank sends T * K rows in total
    const int rows_hint = static_cast<int>(static_cast<int64_t>(T) * K * b->num_ranks / E);
    CAM_CUDA(cudaSetDevice(b->device));
    if (const int deep = use_deep_fuse(b, ue8m0, h, inter, rows_hint))
        return fused_moe_deep(b, x, expert_ids, idx_is_i64, topk_weights, w1_q, w1_s, w2_q, w2_s, out, expert_token_nums, T,
                              K, h, inter, E, El, rows_hint, phase_mask, deep == 1, stream);
    const int disp_mask = phase_mask & CAM_PHASE_ALL;
    const bool prof = b->profile && phase_mask == 15;
    auto stamp = [&](int i) { if (prof) cudaEventRecord(b->prof_ev[i], stream); };
    stamp(0);
    if (disp_mask) {
        if (cam_dispatch_normal(b, x, expert_ids, idx_is_i64, T, K, h, E,
                                ue8m0 ? CAM_QUANT_FP8_1x128_UE8M0 : CAM_QUANT_FP8_1x128, disp_mask, stream) != 0)
            return -1;
    }
    stamp(1);
    if (phase_mask & CAM_PHASE_RECV) {
        const uint8_t* recv_x = b->base + L.off_recv_x;
        const float* recv_s = reinterpret_cast<const float*>(b->base + L.off_recv_scales);
        const int* recv_src = reinterpret_cast<const int*>(b->base + L.off_recv_src);
        if (grouped_gemm_impl(b, recv_x, recv_s, L.capacity, w1_q, w1_s, b->expert_offsets, El, 2 * inter, h, 1,
                              nullptr, b->act_q, b->act_s, nullptr, K, 0, ue8m0, rows_hint, stream) != 0)
            return -1;
        stamp(2);
        if (grouped_gemm_impl(b, b->act_q, b->act_s, L.capacity, w2_q, w2_s, b->expert_offsets, El, h, inter, 2,
                              nullptr, nullptr, nullptr, recv_src, K, 0, ue8m0, rows_hint, stream) != 0)
            return -1;
        if (expert_token_nums != nullptr)
            CAM_CUDA(cudaMemcpyAsync(expert_token_nums, b->num_recv_per_expert, sizeof(int64_t) * El,
                                     cudaMemcpyDeviceToDevice, stream));
    }
    stamp(3);
    if (phase_mask & 8) {
        if (cam_combine(b, nullptr, nullptr, nullptr, expert_ids, idx_is_i64, topk_weights, out, T, K, h, E, 0, 0,
                        CAM_PHASE_RECV, stream) != 0)
            return -1;
    }
    stamp(4);
    if (prof) b->profile_valid = true;
    return 0;
}

extern "C" int cam_fused_moe_fp8(CamBuffer* b, const void* x, const void* expert_ids, int idx_is_i64,
                                 const float* topk_weights, const void* w1_q, const float* w1_s, const void* w2_q,
                                 const float* w2_s, void* out, int64_t* expert_token_nums, int T, int K, int h,
                                 int inter, int E, int gemm_experts, int phase_mask, cudaStream_t stream) {
    return fused_moe_impl(b, x, expert_ids, idx_is_i64, topk_weights, w1_q, w1_s, w2_q, w2_s, out, expert_token_nums,
                          T, K, h, inter, E, gemm_experts, phase_mask, false, stream);
}

extern "C" int cam_fused_moe_mxfp8(CamBuffer* b, const void* x, const void* expert_ids, int idx_is_i64,
                                   const float* topk_weights, const void* w1_q, const float* w1_s, const void* w2_q,
                                   const float* w2_s, void* out, int64_t* expert_token_nums, int T, int K, int h,
                                   int inter, int E, int gemm_experts, int phase_mask, cudaStream_t stream) {
    return fused_moe_impl(b, x, expert_ids, idx_is_i64, topk_weights, w1_q, w1_s, w2_q, w2_s, out, expert_token_nums,
                          T, K, h, inter, E, gemm_experts, phase_mask, true, stream);
}
