// Single-rank dispatch that allocates nothing: see dispatch_noalloc.h for the contract, the
// limits and which callers it exists for.  The kernel is the one-rank variant of
// dispatch_normal_kernel (same chunking, same slot arithmetic, same warp-per-token quantise and
// push), with the scratch that kernel takes from a Buffer's workspace placed in a file-scope
// device array instead.
#include <cooperative_groups.h>
#include <cstdarg>
#include <cstdio>

#include "../common/cam_types.h"
#include "../common/ptx.cuh"
#include "../common/quant.cuh"
#include "dispatch_noalloc.h"

namespace cg = cooperative_groups;

namespace {

// Scratch shared by every call on this device.  In host code this name is only a stand-in for
// the symbol: its device address is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CAM_NOALLOC_SCRATCH_BYTES];

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;

struct LocalParams {
    const __nv_bfloat16* x;
    const void* topk_idx;
    int idx_is_i64;
    int T, K, h, E, quant_mode, capacity;
    uint8_t* recv_x;
    float* recv_scales;
    int* recv_src;
    int* expert_offsets;
    // carved out of the scratch array
    int* cta_hist;  // [grid, E]
    int* slot;      // [T*K] chunk-local slot of every pair inside its expert
    int* status;    // [0] = 0 ok / CAM_NOALLOC_OVERFLOW, [1] = rows needed
};


__global__ void __launch_bounds__(kThreads, 1) dispatch_local_kernel(const LocalParams p) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    __shared__ int s_hist[CAM_NOALLOC_MAX_EXPERTS];
    __shared__ int s_pre[CAM_NOALLOC_MAX_EXPERTS];   // rows of this expert held by earlier CTAs
    __shared__ int s_tot[CAM_NOALLOC_MAX_EXPERTS];
    __shared__ int s_base[CAM_NOALLOC_MAX_EXPERTS];  // first output row of every expert
    __shared__ int s_ids[kThreads];
    __shared__ int s_total;

    const int tid = static_cast<int>(threadIdx.x);
    const int nb = static_cast<int>(gridDim.x), b = static_cast<int>(blockIdx.x);
    const int E = p.E, K = p.K;
    const int tpc = (p.T + nb - 1) / nb;
    const int t0 = min(p.T, b * tpc), t1 = min(p.T, t0 + tpc);
    const int npairs = (t1 - t0) * K;

    for (int e = tid; e < E; e += kThreads) s_hist[e] = 0;
    __syncthreads();
    for (int sub = 0; sub < npairs; sub += kThreads) {
        const int i = sub + tid;
        int id = -1;
        if (i < npairs) {
            id = cam::load_expert_id(p.topk_idx, p.idx_is_i64, static_cast<size_t>(t0) * K + i);
            if (id < 0 || id >= E) id = -1;
        }
        s_ids[tid] = id;
        __syncthreads();
        if (i < npairs) {
            int r = -1;
            if (id >= 0) {
                r = s_hist[id];
                for (int j = 0; j < tid; ++j) r += (s_ids[j] == id) ? 1 : 0;
            }
            p.slot[static_cast<size_t>(t0) * K + i] = r;  // every word that is read later is written here
        }
        __syncthreads();
        if (id >= 0) atomicAdd(&s_hist[id], 1);
        __syncthreads();
    }
    for (int e = tid; e < E; e += kThreads) p.cta_hist[static_cast<size_t>(b) * E + e] = s_hist[e];
    __threadfence();
    cg::this_grid().sync();

    for (int e = tid; e < E; e += kThreads) {
        int pre = 0, tot = 0;
        for (int bb = 0; bb < nb; ++bb) {
            const int c = __ldcg(&p.cta_hist[static_cast<size_t>(bb) * E + e]);
            pre += (bb < b) ? c : 0;
            tot += c;
        }
        s_pre[e] = pre;
        s_tot[e] = tot;
    }
    __syncthreads();
    for (int e = tid; e < E; e += kThreads) {
        int base = 0;
        for (int l = 0; l < e; ++l) base += s_tot[l];
        s_base[e] = base;
        if (e == E - 1) s_total = base + s_tot[e];
    }
    __syncthreads();
    const int total = s_total;
    if (b == 0) {
        for (int e = tid; e < E; e += kThreads) p.expert_offsets[e] = s_base[e];
        if (tid == 0) {
            p.expert_offsets[E] = total;
            p.status[0] = (total > p.capacity) ? CAM_NOALLOC_OVERFLOW : CAM_NOALLOC_OK;
            p.status[1] = total;
        }
    }
    if (total > p.capacity) return;  // every CTA sees the same total: nobody writes a row

    const int warp = tid >> 5;
    const uint32_t lane = cam::lane_id();
    const int nscale = CAM_QUANT_IS_FP8(p.quant_mode) ? (p.h >> 7) : (p.quant_mode == CAM_QUANT_INT8_TOKEN) ? 1 : 0;
    const int row_bytes = (p.quant_mode == CAM_QUANT_NONE) ? p.h * 2 : p.h;
    const int stage_bytes = (p.quant_mode == CAM_QUANT_NONE) ? 0 : ((p.h + nscale * 4 + 15) & ~15);
    uint8_t* stage_q = dyn_smem + static_cast<size_t>(warp) * stage_bytes;
    float* stage_s = reinterpret_cast<float*>(stage_q + p.h);
    for (int t = t0 + warp; t < t1; t += kWarps) {
        const __nv_bfloat16* xrow = p.x + static_cast<size_t>(t) * p.h;
        if (p.quant_mode == CAM_QUANT_FP8_1x128) cam::warp_quant_fp8_1x128<false>(xrow, p.h, stage_q, stage_s);
        else if (p.quant_mode == CAM_QUANT_FP8_1x128_UE8M0) cam::warp_quant_fp8_1x128<true>(xrow, p.h, stage_q, stage_s);
        else if (p.quant_mode == CAM_QUANT_INT8_TOKEN) cam::warp_quant_int8_token(xrow, p.h, stage_q, stage_s);
        __syncwarp();
        for (int k = 0; k < K; ++k) {
            const size_t g = static_cast<size_t>(t) * K + k;
            const int id = cam::load_expert_id(p.topk_idx, p.idx_is_i64, g);
            if (id < 0 || id >= E) continue;
            const int row = s_base[id] + s_pre[id] + p.slot[g];
            uint8_t* dst = p.recv_x + static_cast<size_t>(row) * row_bytes;
            if (p.quant_mode == CAM_QUANT_NONE) {
                const uint8_t* src = reinterpret_cast<const uint8_t*>(xrow);
                for (int o = static_cast<int>(lane) * 16; o < row_bytes; o += 512) cam::st_na_v4(dst + o, cam::ld_nc_v4(src + o));
            } else {
                for (int o = static_cast<int>(lane) * 16; o < row_bytes; o += 512)
                    cam::st_na_v4(dst + o, *reinterpret_cast<const uint4*>(stage_q + o));
                float* sdst = p.recv_scales + static_cast<size_t>(row) * nscale;
                for (int o = static_cast<int>(lane); o < nscale; o += 32) sdst[o] = stage_s[o];
            }
            if (lane < 3) p.recv_src[static_cast<size_t>(row) * 3 + lane] = (lane == 0) ? 0 : (lane == 1) ? t : k;
        }
        __syncwarp();
    }
}

// Per-device set-up state (host side).
constexpr int kMaxDevices = 64;
struct DeviceState {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_noalloc_scratch on this device
    int grid = 0;
};
DeviceState g_dev[kMaxDevices];
char g_error[512] = "";
int g_host_status[2] = {0, 0};

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int smem_bytes(int h, int quant_mode) {
    if (quant_mode == CAM_QUANT_NONE) return 0;
    const int nscale = CAM_QUANT_IS_FP8(quant_mode) ? h / 128 : 1;
    return kWarps * ((h + nscale * 4 + 15) & ~15);
}

}  // namespace

extern "C" const char* cam_dispatch_local_noalloc_error(void) { return g_error; }

extern "C" int cam_dispatch_local_noalloc(const void* x, const void* topk_idx, int idx_is_i64, int tokens, int topk,
                                          int hidden, int experts, int quant_mode, int capacity, void* recv_x,
                                          float* recv_scales, int32_t* recv_src, int32_t* expert_offsets,
                                          cudaStream_t stream) {
    if (x == nullptr || topk_idx == nullptr || recv_x == nullptr || recv_src == nullptr || expert_offsets == nullptr)
        return set_error(CAM_NOALLOC_BAD_ARGUMENT, "null input or output pointer");
    if (tokens < 0 || topk < 1 || topk > CAM_MAX_TOPK)
        return set_error(CAM_NOALLOC_BAD_ARGUMENT, "tokens %d / topk %d outside the supported range (topk 1..%d)", tokens, topk, CAM_MAX_TOPK);
    if (static_cast<long long>(tokens) * topk > CAM_NOALLOC_MAX_PAIRS)
        return set_error(CAM_NOALLOC_BAD_ARGUMENT, "tokens*topk = %lld exceeds the built-in scratch limit of %d pairs",
                         static_cast<long long>(tokens) * topk, CAM_NOALLOC_MAX_PAIRS);
    if (experts < 1 || experts > CAM_NOALLOC_MAX_EXPERTS)
        return set_error(CAM_NOALLOC_BAD_ARGUMENT, "experts %d outside [1, %d]", experts, CAM_NOALLOC_MAX_EXPERTS);
    if (hidden < 128 || hidden % 128 != 0 || hidden > 8192)
        return set_error(CAM_NOALLOC_BAD_ARGUMENT, "hidden %d must be a multiple of 128 in [128, 8192]", hidden);
    if (quant_mode != CAM_QUANT_NONE && quant_mode != CAM_QUANT_INT8_TOKEN && !CAM_QUANT_IS_FP8(quant_mode))
        return set_error(CAM_NOALLOC_BAD_ARGUMENT, "quant_mode %d is not one of 0, 2, 3, 4", quant_mode);
    if (quant_mode != CAM_QUANT_NONE && recv_scales == nullptr)
        return set_error(CAM_NOALLOC_BAD_ARGUMENT, "recv_scales is required for quant_mode %d", quant_mode);
    if (capacity < 1) return set_error(CAM_NOALLOC_BAD_ARGUMENT, "capacity must be positive");
    // rows and scales move as 16-byte vectors
    if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(recv_x) & 15u) ||
        (recv_scales != nullptr && (reinterpret_cast<uintptr_t>(recv_scales) & 15u)))
        return set_error(CAM_NOALLOC_BAD_ARGUMENT, "x, recv_x and recv_scales must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(topk_idx) & (idx_is_i64 ? 7u : 3u)) || (reinterpret_cast<uintptr_t>(recv_src) & 3u) ||
        (reinterpret_cast<uintptr_t>(expert_offsets) & 3u))
        return set_error(CAM_NOALLOC_BAD_ARGUMENT, "topk_idx, recv_src and expert_offsets must be aligned to their element size");

    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error(CAM_NOALLOC_CUDA_ERROR, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return set_error(CAM_NOALLOC_BAD_ARGUMENT, "device index %d not supported", dev);
    DeviceState& st = g_dev[dev];
    if (!st.ready) {
        // One-time set-up for this device (current right now): the array's name is a host-side
        // stand-in, the kernel needs the address the symbol has on this device.
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return set_error(CAM_NOALLOC_CUDA_ERROR, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return set_error(CAM_NOALLOC_CUDA_ERROR, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
        e = cudaFuncSetAttribute(dispatch_local_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(8192, CAM_QUANT_FP8_1x128));
        if (e != cudaSuccess) return set_error(CAM_NOALLOC_CUDA_ERROR, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        st.scratch = static_cast<unsigned char*>(ptr);
        st.grid = sms < CAM_NOALLOC_MAX_GRID ? sms : CAM_NOALLOC_MAX_GRID;
        st.ready = true;
    }

    LocalParams p{};
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.topk_idx = topk_idx;
    p.idx_is_i64 = idx_is_i64;
    p.T = tokens; p.K = topk; p.h = hidden; p.E = experts; p.quant_mode = quant_mode; p.capacity = capacity;
    p.recv_x = static_cast<uint8_t*>(recv_x);
    p.recv_scales = recv_scales;
    p.recv_src = recv_src;
    p.expert_offsets = expert_offsets;
    unsigned char* s = st.scratch;
    p.cta_hist = reinterpret_cast<int*>(s);
    s += 4u * CAM_NOALLOC_MAX_GRID * CAM_NOALLOC_MAX_EXPERTS;
    p.slot = reinterpret_cast<int*>(s);
    s += 4u * CAM_NOALLOC_MAX_PAIRS;
    p.status = reinterpret_cast<int*>(s);
    void* args[] = {&p};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(dispatch_local_kernel), dim3(st.grid), dim3(kThreads), args,
                                    smem_bytes(hidden, quant_mode), stream);
    if (e != cudaSuccess) return set_error(CAM_NOALLOC_CUDA_ERROR, "kernel launch: %s", cudaGetErrorString(e));
    g_error[0] = '\0';
    return CAM_NOALLOC_OK;
}

extern "C" int cam_dispatch_local_noalloc_status(cudaStream_t stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices || !g_dev[dev].ready)
        return set_error(CAM_NOALLOC_BAD_ARGUMENT, "no call has been made on the current device");
    const unsigned char* status = g_dev[dev].scratch + 4u * CAM_NOALLOC_MAX_GRID * CAM_NOALLOC_MAX_EXPERTS + 4u * CAM_NOALLOC_MAX_PAIRS;
    e = cudaMemcpyAsync(g_host_status, status, sizeof(g_host_status), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return set_error(CAM_NOALLOC_CUDA_ERROR, "status read: %s", cudaGetErrorString(e));
    if (g_host_status[0] == CAM_NOALLOC_OVERFLOW)
        return set_error(CAM_NOALLOC_OVERFLOW, "%d rows are needed but the outputs hold fewer; no row was written", g_host_status[1]);
    return CAM_NOALLOC_OK;
}
