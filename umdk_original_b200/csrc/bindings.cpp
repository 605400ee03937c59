// PyTorch binding layer: the six ops of the reference's `umdk_cam_op_lib`
// (pybind/pybind.cpp:13-42, same names, same positional order) registered three ways like the
// reference does -- schema (TORCH_LIBRARY), device implementation (CUDA key where the reference
// uses PrivateUse1), Meta implementation for shape inference where shapes are not data dependent
// (pybind/fused_deep_moe.cpp:87-122) and an Autograd-key wrapper that runs the op without
// recording a graph (pybind/fused_deep_moe.cpp:152-217 returns empty grads) -- plus the explicit
// symmetric `Buffer` object that replaces the HCCL group name / SHMEM heap pointer.
//
// `group_ep` / `groupEp` names a registered Buffer, `extInfo` is a registered Buffer's integer id.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <map>
#include <memory>
#include <mutex>
#include <string>

#include "runtime/cam_runtime.h"

namespace {

#define CAM_ASSERT(cond, ...) TORCH_CHECK(cond, "umdk_cam_op_lib: ", __VA_ARGS__)
#define CAM_RT(call) TORCH_CHECK((call) == 0, "umdk_cam_op_lib: ", cam_last_error())

class Buffer;
std::mutex g_reg_mutex;
std::map<std::string, Buffer*> g_by_name;
std::map<int64_t, Buffer*> g_by_id;
int64_t g_next_id = 1;
// all phases; the single-GPU virtual-rank harness narrows it.  Bits: 1 count, 2 send, 4 receive,
// 8 final reduce of the fused layer, 16 / 32 send / receive of the tensor-parallel pair exchange.
int g_phase_mask = 63;

class Buffer {
public:
    Buffer(int64_t device, int64_t rank, int64_t num_ranks, int64_t num_experts, int64_t max_tokens, int64_t hidden,
           int64_t topk, int64_t capacity, int64_t ll_max_tokens, int64_t tp_rows) {
        CAM_RT(cam_layout_compute_tp(&layout_, static_cast<int>(num_ranks), static_cast<int>(num_experts),
                                     static_cast<int>(max_tokens), static_cast<int>(hidden), static_cast<int>(topk),
                                     static_cast<int>(capacity), static_cast<int>(ll_max_tokens), static_cast<int>(tp_rows)));
        buf_ = cam_buffer_create(static_cast<int>(device), static_cast<int>(rank), static_cast<int>(num_ranks), &layout_);
        TORCH_CHECK(buf_ != nullptr, "umdk_cam_op_lib: ", cam_last_error());
        // Tensors that view the buffer's memory (the outputs of the dispatch ops) share ownership of it, so the
        // memory is released when the Buffer has been destroyed AND the last such tensor is gone.
        hold_ = std::shared_ptr<CamBuffer>(buf_, [](CamBuffer* b) { cam_buffer_destroy(b); });
        std::lock_guard<std::mutex> g(g_reg_mutex);
        id_ = g_next_id++;
        g_by_id[id_] = this;
    }
    ~Buffer() { destroy(); }
    void destroy() {
        if (buf_ == nullptr) return;
        {
            std::lock_guard<std::mutex> g(g_reg_mutex);
            g_by_id.erase(id_);
            if (!name_.empty()) g_by_name.erase(name_);
        }
        ll_src_ = at::Tensor();
        ll_total_ = at::Tensor();
        tp_counts_ = tp_reduced_ = tp_rows_ = tp_scales_ = at::Tensor();
        buf_ = nullptr;
        hold_.reset();  // frees now unless views of the memory are still alive
    }
    // Outputs of the prefill dispatch: views of the symmetric memory (default; valid until the next dispatch on
    // this Buffer, reset() or destroy()) or private copies that the caller may keep for as long as it likes.
    void set_copy_outputs(bool on) { copy_outputs_ = on; }
    bool copy_outputs() const { return copy_outputs_; }
    void register_name(const std::string& name) {
        std::lock_guard<std::mutex> g(g_reg_mutex);
        if (!name_.empty()) g_by_name.erase(name_);
        name_ = name;
        g_by_name[name] = this;
    }
    int64_t id() const { return id_; }
    std::string name() const { return name_; }
    py::bytes ipc_handle() {
        char h[CAM_IPC_HANDLE_BYTES];
        CAM_RT(cam_buffer_ipc_handle(buf_, h));
        return py::bytes(h, CAM_IPC_HANDLE_BYTES);
    }
    void open_ipc_peers(const std::vector<std::string>& handles) {
        CAM_ASSERT(static_cast<int>(handles.size()) == cam_buffer_num_ranks(buf_), "need one IPC handle per rank");
        std::string all;
        for (auto& h : handles) {
            CAM_ASSERT(h.size() == CAM_IPC_HANDLE_BYTES, "bad IPC handle size");
            all += h;
        }
        CAM_RT(cam_buffer_open_ipc_peers(buf_, all.data()));
    }
    void set_local_peers(const std::vector<Buffer*>& peers) {
        std::vector<CamBuffer*> raw;
        for (auto* p : peers) raw.push_back(p->buf_);
        CAM_ASSERT(static_cast<int>(raw.size()) == cam_buffer_num_ranks(buf_), "need one peer per rank");
        CAM_RT(cam_buffer_set_local_peers(buf_, raw.data()));
    }
    void open_ipc_tp_peer(const std::string& handle, int64_t tp_rank) {
        CAM_ASSERT(handle.size() == CAM_IPC_HANDLE_BYTES, "bad IPC handle size");
        CAM_RT(cam_buffer_open_ipc_tp_peer(buf_, handle.data(), static_cast<int>(tp_rank)));
        has_tp_ = true;
    }
    void set_local_tp_peer(Buffer* peer, int64_t tp_rank) {
        CAM_RT(cam_buffer_set_local_tp_peer(buf_, peer->buf_, static_cast<int>(tp_rank)));
        has_tp_ = true;
    }
    bool has_tp() const { return has_tp_; }
    void reset() { CAM_RT(cam_buffer_reset(buf_, stream())); }
    void set_timeout_ms(double ms) { cam_buffer_set_timeout_ms(buf_, ms); }
    void set_debug_drop_flags(bool on) { cam_buffer_set_debug_drop_flags(buf_, on ? 1 : 0); }
    void barrier() { CAM_RT(cam_buffer_barrier(buf_, (g_phase_mask & 7) & (CAM_PHASE_SEND | CAM_PHASE_RECV), stream())); }
    void p2p_write(int64_t peer, int64_t bytes, int64_t grid) {
        CAM_RT(cam_buffer_p2p_write(buf_, static_cast<int>(peer), static_cast<size_t>(bytes), static_cast<int>(grid), stream()));
    }
    void p2p_pingpong(int64_t peer, int64_t base, int64_t iters, bool initiator) {
        CAM_RT(cam_buffer_p2p_pingpong(buf_, static_cast<int>(peer), static_cast<unsigned int>(base), static_cast<int>(iters),
                                       initiator ? 1 : 0, stream()));
    }
    void set_trace(bool on) { CAM_RT(cam_buffer_set_trace(buf_, on ? 1 : 0)); }
    std::tuple<std::vector<int64_t>, std::vector<int64_t>, std::vector<int64_t>> read_stats(bool reset) {
        const int R = cam_buffer_num_ranks(buf_);
        std::vector<unsigned long long> w(3 * R), rows(R), calls(2);
        CAM_RT(cam_buffer_read_stats(buf_, w.data(), rows.data(), calls.data(), reset ? 1 : 0));
        return {std::vector<int64_t>(w.begin(), w.end()), std::vector<int64_t>(rows.begin(), rows.end()),
                std::vector<int64_t>(calls.begin(), calls.end())};
    }
    int64_t check_guards() {
        int damaged = 0;
        CAM_RT(cam_buffer_check_guards(buf_, stream(), &damaged));
        return damaged;
    }
    at::Tensor guard(int64_t i) const {
        const uint64_t offs[4] = {layout_.off_guard0, layout_.off_guard1, layout_.off_guard2, layout_.off_guard3};
        CAM_ASSERT(i >= 0 && i < 4, "guard index must be 0..3");
        return view(static_cast<uint8_t*>(cam_buffer_base(buf_)) + offs[i], {CAM_GUARD_BYTES}, at::kByte);
    }
    int64_t launch_count() const { return static_cast<int64_t>(cam_buffer_launch_count(buf_)); }
    int64_t fused_route(int64_t tokens, int64_t topk, int64_t hidden, int64_t inter, int64_t experts) const {
        return cam_buffer_fused_route(buf_, static_cast<int>(tokens), static_cast<int>(topk), static_cast<int>(hidden),
                                      static_cast<int>(inter), static_cast<int>(experts));
    }
    void set_fused_trace(bool on) { CAM_RT(cam_buffer_set_fused_trace(buf_, on ? 1 : 0)); }
    std::vector<int64_t> read_fused_trace(int64_t num_local_experts) {
        std::vector<long long> t(static_cast<size_t>(num_local_experts));
        CAM_RT(cam_buffer_read_fused_trace(buf_, t.data(), static_cast<int>(num_local_experts)));
        return std::vector<int64_t>(t.begin(), t.end());
    }
    std::vector<int64_t> read_fused_waits(int64_t num_local_experts) {
        long long t[7];
        CAM_RT(cam_buffer_read_fused_waits(buf_, t, static_cast<int>(num_local_experts)));
        return std::vector<int64_t>(t, t + 7);
    }
    std::vector<int64_t> read_trace() {
        unsigned long long t[16];
        CAM_RT(cam_buffer_read_trace(buf_, t));
        return std::vector<int64_t>(t, t + 16);
    }
    void set_profile(bool on) { CAM_RT(cam_buffer_set_profile(buf_, on ? 1 : 0)); }
    std::vector<double> read_profile() {
        float ms[4];
        CAM_RT(cam_buffer_read_profile(buf_, ms));
        return {ms[0], ms[1], ms[2], ms[3]};
    }
    std::tuple<int64_t, int64_t, int64_t, int64_t, std::string> poll_status() {
        CamStatus st;
        CAM_RT(cam_buffer_poll_status(buf_, stream(), &st));
        return {st.code, st.who, st.detail, st.block, cam_status_string(st.code)};
    }
    int64_t total_bytes() const { return static_cast<int64_t>(layout_.total_bytes); }
    int64_t capacity() const { return layout_.capacity; }

    cudaStream_t stream() const { return at::cuda::getCurrentCUDAStream(cam_buffer_device(buf_)).stream(); }
    c10::Device device() const { return c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(cam_buffer_device(buf_))); }
    at::Tensor view(void* ptr, at::IntArrayRef sizes, at::ScalarType dt) const {
        std::shared_ptr<CamBuffer> keep = hold_;
        return at::from_blob(ptr, sizes, [keep](void*) mutable { keep.reset(); },
                             at::TensorOptions().dtype(dt).device(device()));
    }
    at::Tensor recv_x(int64_t rows, int64_t h, int64_t quant_mode) const {
        auto* base = static_cast<uint8_t*>(cam_buffer_base(buf_));
        const at::ScalarType dt = quant_mode == 0 ? at::kBFloat16 : quant_mode == 2 ? at::kChar : at::kFloat8_e4m3fn;
        return view(base + layout_.off_recv_x, {rows, h}, dt);
    }
    at::Tensor recv_scales(int64_t rows, int64_t n) const {
        auto* base = static_cast<uint8_t*>(cam_buffer_base(buf_));
        return view(base + layout_.off_recv_scales, {rows, n}, at::kFloat);
    }
    at::Tensor recv_src(int64_t rows) const {
        auto* base = static_cast<uint8_t*>(cam_buffer_base(buf_));
        return view(base + layout_.off_recv_src, {rows * 3}, at::kInt);
    }
    at::Tensor recv_count(int64_t n) const { return view(cam_buffer_recv_count(buf_), {n}, at::kInt); }
    at::Tensor expert_offsets(int64_t n) const { return view(cam_buffer_expert_offsets(buf_), {n}, at::kInt); }
    at::Tensor num_recv_per_expert(int64_t n) const { return view(cam_buffer_num_recv_per_expert(buf_), {n}, at::kLong); }
    at::Tensor total_recv() const { return view(cam_buffer_total_recv(buf_), {1}, at::kInt); }
    at::Tensor send_row(int64_t n) const { return view(cam_buffer_send_row(buf_), {n}, at::kInt); }
    at::Tensor num_tokens_per_expert(int64_t n) const { return view(cam_buffer_num_tokens_per_expert(buf_), {n}, at::kInt); }
    at::Tensor act_q(int64_t rows, int64_t cols) const { return view(cam_buffer_act_q(buf_), {rows, cols}, at::kFloat8_e4m3fn); }
    at::Tensor act_s(int64_t rows, int64_t cols) const { return view(cam_buffer_act_s(buf_), {rows, cols}, at::kFloat); }

    CamBuffer* raw() const { return buf_; }
    const CamLayout& layout() const { return layout_; }
    int rank() const { return cam_buffer_rank(buf_); }
    int num_ranks() const { return cam_buffer_num_ranks(buf_); }
    // state that low-latency dispatch leaves for the matching combine
    at::Tensor ll_src_, ll_total_;
    at::Tensor tp_counts_;  // [2] rows per tensor-parallel rank after the all-gather (own rows first)
    at::Tensor tp_reduced_;  // [rows, h] output of the reduce-scatter that precedes combine
    at::Tensor tp_rows_, tp_scales_;  // outputs of the last dispatch (the phase-by-phase test harness re-enters with them)
    bool has_tp_ = false;

    // A weight argument given as a list of per-expert tensors (the reference's "tensor list" form for
    // dynamic expert placement, fused_deep_moe_tiling.cpp:83-127) is stacked into one [E_local, ...]
    // tensor, which the kernels' single TMA descriptor needs.  The stacked copy is kept until one
    // of the list's tensors changes (address or version), so steady-state calls do not copy.
    at::Tensor stacked(int slot, at::TensorList list) {
        if (list.size() == 1 && list[0].dim() == 3) return list[0];
        StackCache& c = stack_cache_[slot];
        bool same = c.value.defined() && c.ptrs.size() == list.size();
        for (size_t i = 0; same && i < list.size(); ++i)
            same = c.ptrs[i] == list[i].data_ptr() && c.versions[i] == list[i]._version();
        if (!same) {
            c.value = at::stack(list).contiguous();
            c.ptrs.clear();
            c.versions.clear();
            for (const at::Tensor& t : list) {
                c.ptrs.push_back(t.data_ptr());
                c.versions.push_back(t._version());
            }
        }
        return c.value;
    }

    // Reference-format int8 weights are [E_local, K, N] (N contiguous); the tensor cores want K
    // contiguous.  The transposed copy is made once and kept until the tensor changes.
    at::Tensor k_major(int slot, const at::Tensor& w) {
        StackCache& c = kmajor_cache_[slot];
        const bool same = c.value.defined() && c.ptrs.size() == 1 && c.ptrs[0] == w.data_ptr() &&
                          c.versions[0] == static_cast<int64_t>(w._version());
        if (!same) {
            c.value = w.transpose(1, 2).contiguous();
            c.ptrs = {w.data_ptr()};
            c.versions = {static_cast<int64_t>(w._version())};
        }
        return c.value;
    }

private:
    struct StackCache {
        at::Tensor value;
        std::vector<void*> ptrs;
        std::vector<int64_t> versions;
    };
    StackCache stack_cache_[4];
    StackCache kmajor_cache_[2];
    CamBuffer* buf_ = nullptr;
    std::shared_ptr<CamBuffer> hold_;
    bool copy_outputs_ = false;
    CamLayout layout_{};
    int64_t id_ = 0;
    std::string name_;
};

Buffer* buffer_by_name(c10::string_view name) {
    std::lock_guard<std::mutex> g(g_reg_mutex);
    auto it = g_by_name.find(std::string(name));
    CAM_ASSERT(it != g_by_name.end(), "no Buffer is registered under the group name '", std::string(name),
               "' (create a Buffer and call register_name first)");
    return it->second;
}
Buffer* buffer_by_id(int64_t id) {
    std::lock_guard<std::mutex> g(g_reg_mutex);
    auto it = g_by_id.find(id);
    CAM_ASSERT(it != g_by_id.end(), "extInfo ", id, " is not the id of a live Buffer");
    return it->second;
}

int idx_kind(const at::Tensor& t, const char* what) {
    CAM_ASSERT(t.scalar_type() == at::kLong || t.scalar_type() == at::kInt, what, " must be int64 or int32");
    return t.scalar_type() == at::kLong ? 1 : 0;
}
// Activations may be bfloat16 or float16, as in the reference (fused_deep_moe/op_host/fused_deep_moe.cpp:17-19,
// moe_dispatch_normal/op_host/moe_dispatch_normal.cpp:19).  The kernels read bfloat16.  A dispatch that moves rows
// unchanged (quant mode 0) takes float16 rows as they are (two bytes per element either way); everything that computes
// on the values (quantisation, weighted sums) converts float16 once on entry, and results go back to the input's dtype.
bool is_half(const at::Tensor& t, const char* what) {
    CAM_ASSERT(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kHalf, what, " must be bfloat16 or float16");
    return t.scalar_type() == at::kHalf;
}
at::Tensor rows_for_kernel(const at::Tensor& x, bool half, bool moved_unchanged) {
    if (!half) return x;
    return moved_unchanged ? x.view(at::kBFloat16) : x.to(at::kBFloat16);
}

void check_cuda_contig(const at::Tensor& t, const char* what) {
    CAM_ASSERT(t.is_cuda(), what, " must be a CUDA tensor");
    CAM_ASSERT(t.is_contiguous(), what, " must be contiguous");
}

// --------------------------------------------------------------------------------------------
// Shared-expert ranks.  The first S ranks of the group hold a replica of the shared expert instead of
// routed experts (moe_dispatch_shmem.h:408-489); every token also goes to one of them, chosen so that
// each replica gets an equal slice of every rank's batch, and combine adds that row unweighted
// (moe_combine_shmem.h:876-908).  The kernels see this as ordinary routing over R * E_l "virtual"
// experts with one more column: routed expert e becomes e + S * E_l (it lives on rank S + e / E_l),
// the replica on rank s is virtual expert s * E_l, and the extra pair carries weight 1.
// The Buffer must have been created for R * E_l experts and top-k + 1.
// --------------------------------------------------------------------------------------------
struct SharedRemap {
    at::Tensor ids;      // [T, K + 1] same dtype as the input ids
    at::Tensor weights;  // [T, K + 1] float32 (undefined when no weights were given)
    int64_t num_virtual_experts = 0;
    int64_t experts_per_rank = 0;
};

SharedRemap remap_for_shared_ranks(const at::Tensor& ids, const c10::optional<at::Tensor>& weights, int64_t num_ranks,
                                   int64_t moe_expert_num, int64_t shared_rank_num) {
    CAM_ASSERT(shared_rank_num > 0 && shared_rank_num < num_ranks, "sharedExpertRankNum must be in [0, epWorldSize)");
    CAM_ASSERT(moe_expert_num % (num_ranks - shared_rank_num) == 0,
               "moeExpertNum must be a multiple of the number of routed-expert ranks");
    SharedRemap r;
    r.experts_per_rank = moe_expert_num / (num_ranks - shared_rank_num);
    r.num_virtual_experts = r.experts_per_rank * num_ranks;
    const int64_t T = ids.size(0);
    const int64_t shift = shared_rank_num * r.experts_per_rank;
    at::Tensor routed = at::where(ids >= 0, ids + shift, at::full_like(ids, -1));
    // token t of every rank goes to replica min(S - 1, t * S / T)
    at::Tensor t = at::arange(T, ids.options());
    at::Tensor replica = at::clamp_max(at::floor_divide(t * shared_rank_num, std::max<int64_t>(T, 1)), shared_rank_num - 1);
    r.ids = at::cat({routed, (replica * r.experts_per_rank).unsqueeze(1)}, 1).contiguous();
    if (weights.has_value() && weights->defined())
        r.weights = at::cat({weights->to(at::kFloat), at::ones({T, 1}, weights->options().dtype(at::kFloat))}, 1).contiguous();
    return r;
}

// --------------------------------------------------------------------------------------------
// get_dispatch_layout  (pybind/get_dispatch_layout.cpp:25-55)
// --------------------------------------------------------------------------------------------
std::tuple<at::Tensor, at::Tensor, at::Tensor> get_dispatch_layout_cuda(const at::Tensor& topk_idx,
                                                                        int64_t num_experts, int64_t num_ranks) {
    CAM_ASSERT(topk_idx.dim() == 2, "topk_idx must be 2-D [tokens, topk]");
    check_cuda_contig(topk_idx, "topk_idx");
    const int is64 = idx_kind(topk_idx, "topk_idx");
    c10::cuda::CUDAGuard guard(topk_idx.device());
    const int64_t T = topk_idx.size(0), K = topk_idx.size(1);
    auto opts = topk_idx.options().dtype(at::kInt);
    at::Tensor per_rank = at::zeros({num_ranks}, opts);
    at::Tensor per_expert = at::zeros({num_experts}, opts);
    at::Tensor in_rank = at::zeros({T, num_ranks}, topk_idx.options().dtype(at::kBool));
    CAM_RT(cam_get_dispatch_layout(topk_idx.data_ptr(), is64, static_cast<int>(T), static_cast<int>(K),
                                   static_cast<int>(num_experts), static_cast<int>(num_ranks),
                                   per_rank.data_ptr<int>(), per_expert.data_ptr<int>(),
                                   reinterpret_cast<uint8_t*>(in_rank.data_ptr<bool>()),
                                   at::cuda::getCurrentCUDAStream().stream()));
    return {per_rank, per_expert, in_rank};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> get_dispatch_layout_meta(const at::Tensor& topk_idx,
                                                                        int64_t num_experts, int64_t num_ranks) {
    auto opts = topk_idx.options().dtype(at::kInt);
    return {at::empty({num_ranks}, opts), at::empty({num_experts}, opts),
            at::empty({topk_idx.size(0), num_ranks}, topk_idx.options().dtype(at::kBool))};
}

// --------------------------------------------------------------------------------------------
// moe_dispatch_prefill  (pybind/moe_dispatch_prefill.cpp:26-192)
// --------------------------------------------------------------------------------------------
std::vector<at::Tensor> dispatch_prefill_impl(const at::Tensor& x, const at::Tensor& topk_idx,
                                              const at::Tensor& topk_weights, int64_t num_worst_tokens,
                                              c10::string_view group_ep, int64_t rank, int64_t num_ranks,
                                              int64_t quant_mode, int64_t num_experts) {
    Buffer* b = buffer_by_name(group_ep);
    CAM_ASSERT(x.dim() == 2 && topk_idx.dim() == 2, "x must be [tokens, hidden] and topk_idx [tokens, topk]");
    const bool half = is_half(x, "x");
    check_cuda_contig(x, "x");
    check_cuda_contig(topk_idx, "topk_idx");
    CAM_ASSERT(topk_weights.sizes() == topk_idx.sizes(), "topk_weights must match topk_idx");
    CAM_ASSERT(rank == b->rank() && num_ranks == b->num_ranks(), "rank/num_ranks do not match the Buffer of group '",
               std::string(group_ep), "'");
    CAM_ASSERT(x.size(0) == topk_idx.size(0), "x and topk_idx disagree on the token count");
    const int is64 = idx_kind(topk_idx, "topk_idx");
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t T = x.size(0), h = x.size(1), K = topk_idx.size(1);
    const int64_t E = num_experts > 0 ? num_experts : b->layout().num_experts, El = E / num_ranks;
    const at::Tensor xk = rows_for_kernel(x, half, quant_mode == 0);
    CAM_RT(cam_dispatch_normal(b->raw(), xk.data_ptr(), topk_idx.data_ptr(), is64, static_cast<int>(T),
                               static_cast<int>(K), static_cast<int>(h), static_cast<int>(E),
                               static_cast<int>(quant_mode), g_phase_mask & 7, b->stream()));
    int64_t rows = num_worst_tokens;
    at::Tensor per_expert = b->num_recv_per_expert(El);
    if (num_worst_tokens <= 0) {
        // exact-size outputs need the row count on the host: one 4-byte copy (the reference syncs twice)
        rows = b->total_recv().cpu().item<int>();
        per_expert = per_expert.cpu();
    }
    CAM_ASSERT(rows <= b->capacity(), "num_worst_tokens exceeds the Buffer capacity");
    const int64_t nscale = (quant_mode == 3 || quant_mode == 4) ? h / 128 : (quant_mode == 2 ? 1 : 0);
    at::Tensor scales = nscale > 0 ? b->recv_scales(rows, nscale) : at::empty({0}, x.options().dtype(at::kFloat));
    // The four device outputs are views of the Buffer's memory: the next dispatch on the same Buffer (from this rank
    // or from a peer that has moved on), reset() and destroy() change or void them.  The reference returns fresh
    // tensors (pybind/moe_dispatch_prefill.cpp:166-191); Buffer.set_copy_outputs(True) gives the same here at the
    // cost of one device copy of the received rows.
    std::vector<at::Tensor> outs = {b->recv_x(rows, h, quant_mode), b->recv_src(rows), b->recv_count(E), per_expert, scales};
    if (half && quant_mode == 0) outs[0] = outs[0].view(at::kHalf);
    if (b->copy_outputs())
        for (at::Tensor& t : outs)
            if (t.is_cuda()) t = t.clone();
    return outs;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> moe_dispatch_prefill_cuda(
    const at::Tensor& x, const at::Tensor& topk_idx, const at::Tensor& topk_weights,
    const at::Tensor& num_tokens_per_rank, const at::Tensor& is_token_in_rank,
    const at::Tensor& num_tokens_per_expert, int64_t num_worst_tokens, c10::string_view group_ep, int64_t rank,
    int64_t num_ranks) {
    (void)num_tokens_per_rank; (void)is_token_in_rank;  // the layout is recomputed on the device
    auto r = dispatch_prefill_impl(x, topk_idx, topk_weights, num_worst_tokens, group_ep, rank, num_ranks, 0,
                                   num_tokens_per_expert.numel());
    return {r[0], r[1], r[2], r[3]};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> moe_dispatch_prefill_quant_cuda(
    const at::Tensor& x, const at::Tensor& topk_idx, const at::Tensor& topk_weights, int64_t num_worst_tokens,
    c10::string_view group_ep, int64_t rank, int64_t num_ranks, int64_t quant_mode) {
    auto r = dispatch_prefill_impl(x, topk_idx, topk_weights, num_worst_tokens, group_ep, rank, num_ranks, quant_mode, 0);
    return {r[0], r[1], r[2], r[3], r[4]};
}

// --------------------------------------------------------------------------------------------
// moe_combine_prefill  (pybind/moe_combine_prefill.cpp:26-74)
// --------------------------------------------------------------------------------------------
at::Tensor moe_combine_prefill_cuda(const at::Tensor& x, const at::Tensor& topk_idx, const at::Tensor& topk_weights,
                                    const at::Tensor& src_idx, const at::Tensor& send_head,
                                    c10::string_view group_ep, int64_t rank, int64_t num_ranks) {
    Buffer* b = buffer_by_name(group_ep);
    CAM_ASSERT(x.dim() == 2, "x must be a 2-D tensor of expert outputs");
    const bool half = is_half(x, "x");
    check_cuda_contig(x, "x");
    check_cuda_contig(topk_idx, "topk_idx");
    check_cuda_contig(src_idx, "src_idx");
    CAM_ASSERT(src_idx.scalar_type() == at::kInt && src_idx.numel() >= x.size(0) * 3, "src_idx must hold 3 int32 per row of x");
    CAM_ASSERT(topk_weights.scalar_type() == at::kFloat && topk_weights.sizes() == topk_idx.sizes(),
               "topk_weights must be float32 with the shape of topk_idx");
    CAM_ASSERT(rank == b->rank() && num_ranks == b->num_ranks(), "rank/num_ranks do not match the Buffer");
    const int is64 = idx_kind(topk_idx, "topk_idx");
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t T = topk_idx.size(0), K = topk_idx.size(1), h = x.size(1);
    const int64_t E = send_head.numel();
    at::Tensor w = topk_weights.contiguous();
    const at::Tensor xk = rows_for_kernel(x, half, false);
    at::Tensor out = at::empty({T, h}, xk.options());
    // rows actually present: the smaller of x's rows and the device-side count of the last dispatch
    at::Tensor total = at::minimum(b->total_recv(), at::full({1}, x.size(0), b->total_recv().options()));
    CAM_RT(cam_combine(b->raw(), xk.data_ptr(), src_idx.data_ptr<int>(), total.data_ptr<int>(), topk_idx.data_ptr(),
                       is64, w.data_ptr<float>(), out.data_ptr(), static_cast<int>(T), static_cast<int>(K),
                       static_cast<int>(h), static_cast<int>(E), 0, 0,
                       (g_phase_mask & 7) & (CAM_PHASE_SEND | CAM_PHASE_RECV), b->stream()));
    return half ? out.to(at::kHalf) : out;
}

// --------------------------------------------------------------------------------------------
// moe_dispatch_shmem / moe_combine_shmem  (pybind/moe_dispatch_shmem.cpp:27-153, moe_combine_shmem.cpp:27-85)
// --------------------------------------------------------------------------------------------
std::vector<at::Tensor> moe_dispatch_shmem_bf16(const at::Tensor& x, const at::Tensor& expertIds,
                                                const c10::optional<at::Tensor>& scales,
                                                const c10::optional<at::Tensor>& xActiveMask, int64_t epWorldSize,
                                                int64_t epRankId, int64_t moeExpertNum, int64_t tpWorldSize,
                                                int64_t tpRankId, int64_t expertShardType, int64_t sharedExpertNum,
                                                int64_t sharedExpertRankNum, int64_t quantMode, int64_t globalBS,
                                                int64_t expertTokenNumsType, int64_t extInfo) {
    (void)expertShardType; (void)globalBS; (void)sharedExpertNum;
    Buffer* b = buffer_by_id(extInfo);
    CAM_ASSERT(x.dim() == 2 && expertIds.dim() == 2, "x must be [bs, h] and expertIds [bs, k]");
    CAM_ASSERT(x.scalar_type() == at::kBFloat16, "x must be bfloat16");
    check_cuda_contig(x, "x");
    check_cuda_contig(expertIds, "expertIds");
    CAM_ASSERT(epWorldSize == b->num_ranks() && epRankId == b->rank(), "epWorldSize/epRankId do not match the Buffer");
    CAM_ASSERT(tpWorldSize <= 2 && tpRankId >= 0 && tpRankId < std::max<int64_t>(tpWorldSize, 1),
               "tpWorldSize must be 1 or 2 (as in the reference) with tpRankId inside it");
    CAM_ASSERT(tpWorldSize < 2 || b->has_tp(), "tpWorldSize 2 needs a Buffer created with a tensor-parallel partner");
    CAM_ASSERT(quantMode != 1, "static quantisation (quantMode 1) is rejected, as in the reference");
    idx_kind(expertIds, "expertIds");
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t T = x.size(0), h = x.size(1), Kuser = expertIds.size(1);
    const int64_t S = sharedExpertRankNum;
    const bool shared_rank = epRankId < S;
    at::Tensor ids = expertIds;
    int64_t E = moeExpertNum, El = moeExpertNum / epWorldSize;
    if (S > 0) {
        SharedRemap rm = remap_for_shared_ranks(expertIds, c10::nullopt, epWorldSize, moeExpertNum, S);
        ids = rm.ids;
        E = rm.num_virtual_experts;
        El = rm.experts_per_rank;
    }
    const int is64 = idx_kind(ids, "expertIds");
    const int64_t K = ids.size(1);
    // rows this rank can receive (pybind/moe_dispatch_shmem.cpp:50-62)
    const int64_t A1 = std::max<int64_t>(1, shared_rank ? (T * epWorldSize + S - 1) / S
                                                        : T * epWorldSize * std::min<int64_t>(El, Kuser));
    const int64_t A = A1 * std::max<int64_t>(tpWorldSize, 1);  // with TP the partner's rows follow this rank's own
    // x_active_mask: tokens whose entry is false do not take part.  Applied on the device (no host
    // read of the mask), so the call can be captured in a CUDA graph; for the prefix masks the
    // reference defines (only the popcount is used there, GMM1.h:647-678) the result is the same.
    const int64_t active = T;
    if (xActiveMask.has_value() && xActiveMask->defined())
        ids = at::where(xActiveMask->to(at::kBool).unsqueeze(1), ids, at::full_like(ids, -1)).contiguous();
    const float* smooth = nullptr;
    at::Tensor smooth_t;
    if (scales.has_value() && scales->defined() && quantMode == 2) {
        smooth_t = scales->to(at::kFloat).contiguous();
        CAM_ASSERT(smooth_t.dim() == 2 && smooth_t.size(0) >= moeExpertNum && smooth_t.size(1) == h,
                   "scales must be [>= moeExpertNum, h]");
        CAM_ASSERT(S == 0, "smooth scales together with shared-expert ranks are not supported");
        smooth = smooth_t.data_ptr<float>();
    }
    const at::ScalarType xdt = quantMode == 0 ? at::kBFloat16 : quantMode == 2 ? at::kChar : at::kFloat8_e4m3fn;
    const bool fp8 = quantMode == 3 || quantMode == 4;
    const int64_t nscale = fp8 ? h / 128 : 1;
    at::Tensor expandX = at::empty({A, h}, x.options().dtype(xdt));
    at::Tensor dynScales = fp8 ? at::empty({A, nscale}, x.options().dtype(at::kFloat))
                               : at::empty({A}, x.options().dtype(at::kFloat));
    at::Tensor expandIdx = at::empty({T * K}, x.options().dtype(at::kInt));
    at::Tensor expandSrc = at::empty({A, 3}, x.options().dtype(at::kInt));
    at::Tensor tokenNums = at::empty({El}, x.options().dtype(at::kLong));
    at::Tensor epSend = at::empty({epWorldSize * El}, x.options().dtype(at::kInt));
    at::Tensor tpSend = at::zeros({std::max<int64_t>(tpWorldSize, 1)}, x.options().dtype(at::kInt));
    at::Tensor total = at::zeros({1}, x.options().dtype(at::kInt));
    if (g_phase_mask & 6)
    CAM_RT(cam_dispatch_ll(b->raw(), x.data_ptr(), ids.data_ptr(), is64, smooth, static_cast<int>(T),
                           static_cast<int>(K), static_cast<int>(h), static_cast<int>(E),
                           static_cast<int>(active), static_cast<int>(quantMode), static_cast<int>(expertTokenNumsType),
                           expandX.data_ptr(), dynScales.data_ptr<float>(), expandIdx.data_ptr<int>(),
                           expandSrc.data_ptr<int>(), tokenNums.data_ptr<int64_t>(), epSend.data_ptr<int>(),
                           total.data_ptr<int>(), (g_phase_mask & 7) & (CAM_PHASE_SEND | CAM_PHASE_RECV), b->stream()));
    if (g_phase_mask & 6) {
        b->ll_src_ = expandSrc;
        b->ll_total_ = total;
    }
    if (tpWorldSize == 2) {
        // all-gather inside the TP pair (moe_dispatch_shmem.h:936-1018): the partner's rows are appended
        const int tp_mask = ((g_phase_mask & 16) ? CAM_PHASE_SEND : 0) | ((g_phase_mask & 32) ? CAM_PHASE_RECV : 0);
        if (tp_mask) {
            at::Tensor rows = (g_phase_mask & 6) ? expandX : b->tp_rows_;
            at::Tensor sc = (g_phase_mask & 6) ? dynScales : b->tp_scales_;
            at::Tensor cnt = (g_phase_mask & 6) ? tpSend : b->tp_counts_;
            CAM_RT(cam_tp_allgather(b->raw(), rows.data_ptr(), quantMode == 0 ? nullptr : sc.data_ptr<float>(),
                                    static_cast<int>(rows.size(1) * rows.element_size()), static_cast<int>(nscale),
                                    b->ll_total_.data_ptr<int>(), static_cast<int>(A), cnt.data_ptr<int>(), tp_mask,
                                    b->stream()));
            expandX = rows;
            dynScales = sc;
            tpSend = cnt;
        }
        b->tp_rows_ = expandX;
        b->tp_scales_ = dynScales;
        b->tp_counts_ = tpSend;
    }
    if (S > 0) {
        // reference shapes: expandIdx covers the routed pairs only; a shared rank reports one expert
        expandIdx = expandIdx.view({T, K}).slice(1, 0, Kuser).contiguous().view({T * Kuser});
        if (shared_rank) {
            tokenNums = tokenNums.slice(0, 0, 1);
            epSend = epSend.slice(0, 0, epWorldSize);
        }
    }
    return {expandX, dynScales, expandIdx, tokenNums, epSend, tpSend};
}

std::vector<at::Tensor> moe_dispatch_shmem_cuda(const at::Tensor& x, const at::Tensor& expertIds,
                                                const c10::optional<at::Tensor>& scales,
                                                const c10::optional<at::Tensor>& xActiveMask, int64_t epWorldSize,
                                                int64_t epRankId, int64_t moeExpertNum, int64_t tpWorldSize,
                                                int64_t tpRankId, int64_t expertShardType, int64_t sharedExpertNum,
                                                int64_t sharedExpertRankNum, int64_t quantMode, int64_t globalBS,
                                                int64_t expertTokenNumsType, int64_t extInfo) {
    const bool half = is_half(x, "x");
    auto outs = moe_dispatch_shmem_bf16(rows_for_kernel(x, half, quantMode == 0), expertIds, scales, xActiveMask, epWorldSize,
                                        epRankId, moeExpertNum, tpWorldSize, tpRankId, expertShardType, sharedExpertNum,
                                        sharedExpertRankNum, quantMode, globalBS, expertTokenNumsType, extInfo);
    if (half && quantMode == 0) outs[0] = outs[0].view(at::kHalf);  // rows travelled unchanged
    return outs;
}

std::vector<at::Tensor> moe_dispatch_shmem_meta(const at::Tensor& x, const at::Tensor& expertIds,
                                                const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&,
                                                int64_t epWorldSize, int64_t epRankId, int64_t moeExpertNum,
                                                int64_t tpWorldSize, int64_t, int64_t, int64_t,
                                                int64_t sharedExpertRankNum, int64_t quantMode, int64_t, int64_t,
                                                int64_t) {
    const int64_t T = x.size(0), h = x.size(1), K = expertIds.size(1);
    const int64_t S = sharedExpertRankNum, El = moeExpertNum / (epWorldSize - S);
    const bool shared_rank = epRankId < S;
    const int64_t A = std::max<int64_t>(1, shared_rank ? (T * epWorldSize + S - 1) / S
                                                       : T * epWorldSize * std::min<int64_t>(El, K));
    const at::ScalarType xdt = quantMode == 0 ? at::kBFloat16 : quantMode == 2 ? at::kChar : at::kFloat8_e4m3fn;
    if (S > 0)
        return {at::empty({A, h}, x.options().dtype(xdt)),
                (quantMode == 3 || quantMode == 4) ? at::empty({A, h / 128}, x.options().dtype(at::kFloat))
                                                   : at::empty({A}, x.options().dtype(at::kFloat)),
                at::empty({T * K}, x.options().dtype(at::kInt)),
                at::empty({shared_rank ? 1 : El}, x.options().dtype(at::kLong)),
                at::empty({shared_rank ? epWorldSize : epWorldSize * El}, x.options().dtype(at::kInt)),
                at::empty({std::max<int64_t>(tpWorldSize, 1)}, x.options().dtype(at::kInt))};
    return {at::empty({A, h}, x.options().dtype(xdt)),
            (quantMode == 3 || quantMode == 4) ? at::empty({A, h / 128}, x.options().dtype(at::kFloat))
                                               : at::empty({A}, x.options().dtype(at::kFloat)),
            at::empty({T * K}, x.options().dtype(at::kInt)), at::empty({El}, x.options().dtype(at::kLong)),
            at::empty({epWorldSize * El}, x.options().dtype(at::kInt)),
            at::empty({std::max<int64_t>(tpWorldSize, 1)}, x.options().dtype(at::kInt))};
}

at::Tensor moe_combine_shmem_bf16(const at::Tensor& expandX, const at::Tensor& expertIds, const at::Tensor& expandIdx,
                                  const at::Tensor& epSendCounts, const at::Tensor& expertScales,
                                  const c10::optional<at::Tensor>& tpSendCounts,
                                  const c10::optional<at::Tensor>& xActiveMask,
                                  const c10::optional<at::Tensor>& activationScale,
                                  const c10::optional<at::Tensor>& weightScale,
                                  const c10::optional<at::Tensor>& groupList,
                                  const c10::optional<at::Tensor>& expandScales, int64_t epWorldSize, int64_t epRankId,
                                  int64_t moeExpertNum, int64_t tpWorldSize, int64_t tpRankId, int64_t expertShardType,
                                  int64_t sharedExpertNum, int64_t sharedExpertRankNum, int64_t globalBS,
                                  int64_t commQuantMode, int64_t extInfo, int64_t outDtype, int64_t groupListType) {
    (void)expandIdx; (void)epSendCounts; (void)tpSendCounts; (void)activationScale;
    (void)weightScale; (void)groupList; (void)expandScales; (void)tpRankId; (void)expertShardType;
    (void)sharedExpertNum; (void)globalBS; (void)outDtype; (void)groupListType;
    Buffer* b = buffer_by_id(extInfo);
    CAM_ASSERT(expandX.dim() == 2 && expandX.scalar_type() == at::kBFloat16, "expandX must be 2-D bfloat16");
    check_cuda_contig(expandX, "expandX");
    check_cuda_contig(expertIds, "expertIds");
    CAM_ASSERT(epWorldSize == b->num_ranks() && epRankId == b->rank(), "epWorldSize/epRankId do not match the Buffer");
    CAM_ASSERT(tpWorldSize <= 2, "tpWorldSize must be 1 or 2 (as in the reference)");
    CAM_ASSERT(tpWorldSize < 2 || (b->has_tp() && b->tp_counts_.defined()),
               "tpWorldSize 2 needs a Buffer with a tensor-parallel partner and a preceding moe_dispatch_shmem");
    CAM_ASSERT(commQuantMode == 0 || commQuantMode == 2, "commQuantMode must be 0 (bf16 rows) or 2 (int8 rows)");
    CAM_ASSERT(b->ll_src_.defined(), "moe_combine_shmem needs a preceding moe_dispatch_shmem on the same Buffer");
    CAM_ASSERT(expertScales.scalar_type() == at::kFloat, "expertScales must be float32");
    c10::cuda::CUDAGuard guard(expandX.device());
    at::Tensor ids = expertIds;
    at::Tensor w = expertScales.contiguous();
    int64_t E = moeExpertNum;
    if (sharedExpertRankNum > 0) {
        SharedRemap rm = remap_for_shared_ranks(expertIds, expertScales, epWorldSize, moeExpertNum, sharedExpertRankNum);
        ids = rm.ids;
        w = rm.weights;
        E = rm.num_virtual_experts;
    }
    if (xActiveMask.has_value() && xActiveMask->defined())  // masked tokens sent nothing: their pairs are skipped
        ids = at::where(xActiveMask->to(at::kBool).unsqueeze(1), ids, at::full_like(ids, -1)).contiguous();
    const int is64 = idx_kind(ids, "expertIds");
    const int64_t T = ids.size(0), K = ids.size(1), h = expandX.size(1);
    at::Tensor y = expandX;
    if (tpWorldSize == 2) {
        // reduce-scatter inside the TP pair (moe_combine_shmem.h:438-470): the partner gets the partial outputs of its
        // rows, this rank adds the partner's partial outputs for its own
        const int tp_mask = ((g_phase_mask & 16) ? CAM_PHASE_SEND : 0) | ((g_phase_mask & 32) ? CAM_PHASE_RECV : 0);
        if (!b->tp_reduced_.defined() || b->tp_reduced_.size(0) != expandX.size(0) || b->tp_reduced_.size(1) != h)
            b->tp_reduced_ = at::empty_like(expandX);
        if (tp_mask) {
            at::Tensor cnts = b->tp_counts_;
            const int me = cam_buffer_tp_rank(b->raw());
            CAM_RT(cam_tp_reduce_scatter(b->raw(), expandX.data_ptr(), static_cast<int>(h * 2), cnts.data_ptr<int>() + me,
                                         cnts.data_ptr<int>() + (1 - me), b->tp_reduced_.data_ptr(), tp_mask, b->stream()));
        }
        y = b->tp_reduced_;
    }
    at::Tensor out = at::empty({T, h}, expandX.options());
    if (g_phase_mask & 6)
    CAM_RT(cam_combine(b->raw(), y.data_ptr(), b->ll_src_.data_ptr<int>(), b->ll_total_.data_ptr<int>(),
                       ids.data_ptr(), is64, w.data_ptr<float>(), out.data_ptr(), static_cast<int>(T),
                       static_cast<int>(K), static_cast<int>(h), static_cast<int>(E), 1,
                       static_cast<int>(commQuantMode),
                       (g_phase_mask & 7) & (CAM_PHASE_SEND | CAM_PHASE_RECV), b->stream()));
    return out;
}

at::Tensor moe_combine_shmem_cuda(const at::Tensor& expandX, const at::Tensor& expertIds, const at::Tensor& expandIdx,
                                  const at::Tensor& epSendCounts, const at::Tensor& expertScales,
                                  const c10::optional<at::Tensor>& tpSendCounts,
                                  const c10::optional<at::Tensor>& xActiveMask,
                                  const c10::optional<at::Tensor>& activationScale,
                                  const c10::optional<at::Tensor>& weightScale,
                                  const c10::optional<at::Tensor>& groupList,
                                  const c10::optional<at::Tensor>& expandScales, int64_t epWorldSize, int64_t epRankId,
                                  int64_t moeExpertNum, int64_t tpWorldSize, int64_t tpRankId, int64_t expertShardType,
                                  int64_t sharedExpertNum, int64_t sharedExpertRankNum, int64_t globalBS,
                                  int64_t commQuantMode, int64_t extInfo, int64_t outDtype, int64_t groupListType) {
    const bool half = is_half(expandX, "expandX");
    at::Tensor out = moe_combine_shmem_bf16(rows_for_kernel(expandX, half, false), expertIds, expandIdx, epSendCounts, expertScales, tpSendCounts, xActiveMask, activationScale, weightScale, groupList, expandScales, epWorldSize, epRankId, moeExpertNum, tpWorldSize, tpRankId, expertShardType, sharedExpertNum, sharedExpertRankNum, globalBS, commQuantMode, extInfo, outDtype, groupListType);
    return half ? out.to(at::kHalf) : out;
}

at::Tensor moe_combine_shmem_meta(const at::Tensor& expandX, const at::Tensor& expertIds, const at::Tensor&,
                                  const at::Tensor&, const at::Tensor&, const c10::optional<at::Tensor>&,
                                  const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&,
                                  const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&,
                                  const c10::optional<at::Tensor>&, int64_t, int64_t, int64_t, int64_t, int64_t,
                                  int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t) {
    return at::empty({expertIds.size(0), expandX.size(1)}, expandX.options());
}

// --------------------------------------------------------------------------------------------
// fused_deep_moe  (pybind/fused_deep_moe.cpp:26-79).  quantMode 3 = block-scaled fp8 weights with
// arbitrary fp32 scales, quantMode 4 = the same layout with power-of-two scales (tensor-core block scaling):
// gmm1PermutedWeight [E_l, 2I, h] e4m3 (gate rows first) with scales [E_l, 2I/128, h/128],
// gmm2Weight [E_l, h, I] e4m3 with scales [E_l, h/128, I/128]; a list of E_l per-expert tensors
// is stacked once and cached by the Python layer before it reaches this function.
// --------------------------------------------------------------------------------------------
std::vector<at::Tensor> fused_deep_moe_bf16(const at::Tensor& x, const at::Tensor& expertIds,
                                            at::TensorList gmm1PermutedWeight, at::TensorList gmm1PermutedWeightScale,
                                            at::TensorList gmm2Weight, at::TensorList gmm2WeightScale,
                                            const at::Tensor& expertScales,
                                            const c10::optional<at::Tensor>& expertSmoothScales,
                                            const c10::optional<at::Tensor>& xActiveMask, c10::string_view groupEp,
                                            int64_t epRankSize, int64_t epRankId, int64_t moeExpertNum,
                                            int64_t sharedExpertNum, int64_t sharedExpertRankNum, int64_t quantMode,
                                            int64_t globalBs) {
    (void)sharedExpertNum; (void)globalBs;
    // The reference multiplies every row by its expert's smooth vector before the per-token quantisation
    // (fused_deep_moe.h:398, cam_moe_distribute_dispatch.h:704-714); the dispatch of the fused layer here quantises a
    // token once for all of its experts, so the argument is refused rather than silently dropped.
    CAM_ASSERT(!(expertSmoothScales.has_value() && expertSmoothScales->defined()),
               "expertSmoothScales is not supported by fused_deep_moe (pass None; moe_dispatch_shmem applies smooth scales)");
    Buffer* b = buffer_by_name(groupEp);
    CAM_ASSERT(x.dim() == 2 && expertIds.dim() == 2, "x must be [bs, h] and expertIds [bs, k]");
    CAM_ASSERT(x.scalar_type() == at::kBFloat16, "x must be bfloat16");
    check_cuda_contig(x, "x");
    check_cuda_contig(expertIds, "expertIds");
    CAM_ASSERT(epRankSize == b->num_ranks() && epRankId == b->rank(), "epRankSize/epRankId do not match the Buffer");
    CAM_ASSERT(sharedExpertRankNum >= 0 && sharedExpertRankNum < epRankSize, "sharedExpertRankNum must be in [0, epRankSize)");
    CAM_ASSERT(quantMode == 0 || quantMode == 2 || quantMode == 3 || quantMode == 4,
               "quantMode must be 0 / 2 (int8 W8A8 weights in the reference's layout), 3 (fp8, fp32 block scales) or "
               "4 (fp8, power-of-two block scales)");
    CAM_ASSERT(gmm1PermutedWeight.size() >= 1 && gmm2Weight.size() == gmm1PermutedWeight.size() &&
                   gmm1PermutedWeightScale.size() == gmm1PermutedWeight.size() &&
                   gmm2WeightScale.size() == gmm1PermutedWeight.size(),
               "the four weight arguments must be lists of the same length (1 stacked tensor or E_local tensors)");
    c10::cuda::CUDAGuard wguard(x.device());
    const at::Tensor w1 = b->stacked(0, gmm1PermutedWeight);
    const at::Tensor s1 = b->stacked(1, gmm1PermutedWeightScale);
    const at::Tensor w2 = b->stacked(2, gmm2Weight);
    const at::Tensor s2 = b->stacked(3, gmm2WeightScale);
    // local experts: E / (R - S) on a routed rank, 1 (the shared expert) on a shared-expert rank
    const bool shared_rank = epRankId < sharedExpertRankNum;
    const int64_t T = x.size(0), h = x.size(1);
    const int64_t El = shared_rank ? 1 : moeExpertNum / (epRankSize - sharedExpertRankNum);
    const bool w8a8 = quantMode == 0 || quantMode == 2;
    for (const at::Tensor* t : {&w1, &s1, &w2, &s2}) check_cuda_contig(*t, "weight/scale");
    int64_t I = 0;
    at::Tensor w1k, w2k;  // K-major int8 weights of the W8A8 route
    if (w8a8) {
        // reference layout (pybind/fused_deep_moe.cpp:26-79): w1 [E_local, h, 2I] int8 + s1 [E_local, 2I],
        // w2 [E_local, I, h] int8 + s2 [E_local, h]
        CAM_ASSERT(w1.scalar_type() == at::kChar && w2.scalar_type() == at::kChar, "W8A8 weights must be int8");
        CAM_ASSERT(w1.dim() == 3 && w1.size(0) == El && w1.size(1) == h && w1.size(2) % 256 == 0,
                   "gmm1PermutedWeight must be [E_local, h, 2I] int8 with 2I a multiple of 256");
        I = w1.size(2) / 2;
        CAM_ASSERT(w2.dim() == 3 && w2.size(0) == El && w2.size(1) == I && w2.size(2) == h, "gmm2Weight must be [E_local, I, h]");
        CAM_ASSERT(s1.scalar_type() == at::kFloat && s1.numel() == El * 2 * I, "gmm1 scale must be [E_local, 2I] float32");
        CAM_ASSERT(s2.scalar_type() == at::kFloat && s2.numel() == El * h, "gmm2 scale must be [E_local, h] float32");
        w1k = b->k_major(0, w1);
        w2k = b->k_major(1, w2);
    } else {
        CAM_ASSERT(w1.dim() == 3 && w1.size(0) == El && w1.size(2) == h && w1.size(1) % 256 == 0,
                   "gmm1PermutedWeight must be [E_local, 2I, h] with 2I a multiple of 256");
        I = w1.size(1) / 2;
        CAM_ASSERT(w2.dim() == 3 && w2.size(0) == El && w2.size(1) == h && w2.size(2) == I, "gmm2Weight must be [E_local, h, I]");
        CAM_ASSERT(w1.scalar_type() == at::kFloat8_e4m3fn && w2.scalar_type() == at::kFloat8_e4m3fn, "weights must be float8_e4m3fn");
        CAM_ASSERT(s1.scalar_type() == at::kFloat && s1.numel() == El * (2 * I / 128) * (h / 128), "gmm1 scale must be [E_local, 2I/128, h/128] float32");
        CAM_ASSERT(s2.scalar_type() == at::kFloat && s2.numel() == El * (h / 128) * (I / 128), "gmm2 scale must be [E_local, h/128, I/128] float32");
    }
    CAM_ASSERT(expertScales.scalar_type() == at::kFloat, "expertScales must be float32");
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor ids = expertIds;
    at::Tensor w = expertScales.contiguous();
    int64_t E = moeExpertNum;
    if (sharedExpertRankNum > 0) {
        SharedRemap rm = remap_for_shared_ranks(expertIds, expertScales, epRankSize, moeExpertNum, sharedExpertRankNum);
        ids = rm.ids;
        w = rm.weights;
        E = rm.num_virtual_experts;
    }
    if (xActiveMask.has_value() && xActiveMask->defined())  // applied on the device: no host read, graph-capturable
        ids = at::where(xActiveMask->to(at::kBool).unsqueeze(1), ids, at::full_like(ids, -1)).contiguous();
    const int is64 = idx_kind(ids, "expertIds");
    const int64_t K = ids.size(1);
    at::Tensor out = at::empty({T, h}, x.options());
    at::Tensor nums = at::zeros({El}, x.options().dtype(at::kLong));
    auto fused = w8a8 ? &cam_fused_moe_w8a8 : quantMode == 4 ? &cam_fused_moe_mxfp8 : &cam_fused_moe_fp8;
    const void* w1p = w8a8 ? w1k.data_ptr() : w1.data_ptr();
    const void* w2p = w8a8 ? w2k.data_ptr() : w2.data_ptr();
    CAM_RT(fused(b->raw(), x.data_ptr(), ids.data_ptr(), is64, w.data_ptr<float>(), w1p, s1.data_ptr<float>(),
                 w2p, s2.data_ptr<float>(), out.data_ptr(), nums.data_ptr<int64_t>(), static_cast<int>(T),
                 static_cast<int>(K), static_cast<int>(h), static_cast<int>(I), static_cast<int>(E),
                 static_cast<int>(El), g_phase_mask & 15, b->stream()));
    return {out, nums};
}

std::vector<at::Tensor> fused_deep_moe_cuda(const at::Tensor& x, const at::Tensor& expertIds,
                                            at::TensorList gmm1PermutedWeight, at::TensorList gmm1PermutedWeightScale,
                                            at::TensorList gmm2Weight, at::TensorList gmm2WeightScale,
                                            const at::Tensor& expertScales,
                                            const c10::optional<at::Tensor>& expertSmoothScales,
                                            const c10::optional<at::Tensor>& xActiveMask, c10::string_view groupEp,
                                            int64_t epRankSize, int64_t epRankId, int64_t moeExpertNum,
                                            int64_t sharedExpertNum, int64_t sharedExpertRankNum, int64_t quantMode,
                                            int64_t globalBs) {
    const bool half = is_half(x, "x");
    auto outs = fused_deep_moe_bf16(rows_for_kernel(x, half, false), expertIds, gmm1PermutedWeight, gmm1PermutedWeightScale, gmm2Weight, gmm2WeightScale, expertScales, expertSmoothScales, xActiveMask, groupEp, epRankSize, epRankId, moeExpertNum, sharedExpertNum, sharedExpertRankNum, quantMode, globalBs);
    if (half) outs[0] = outs[0].to(at::kHalf);
    return outs;
}

std::vector<at::Tensor> fused_deep_moe_meta(const at::Tensor& x, const at::Tensor&, at::TensorList, at::TensorList,
                                            at::TensorList, at::TensorList, const at::Tensor&,
                                            const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&,
                                            c10::string_view, int64_t epRankSize, int64_t epRankId, int64_t moeExpertNum,
                                            int64_t, int64_t sharedExpertRankNum, int64_t, int64_t) {
    const int64_t local = (epRankId < sharedExpertRankNum) ? 1 : moeExpertNum / (epRankSize - sharedExpertRankNum);
    return {at::empty_like(x), at::empty({local}, x.options().dtype(at::kLong))};
}

// Stand-alone grouped GEMM (mode 0) for tests and for engines that only want the expert MLP.
at::Tensor grouped_gemm_fp8_cuda(const at::Tensor& a_q, const at::Tensor& a_s, const at::Tensor& w_q,
                                 const at::Tensor& w_s, const at::Tensor& expert_offsets, bool ue8m0) {
    check_cuda_contig(a_q, "a_q");
    check_cuda_contig(a_s, "a_s");
    check_cuda_contig(w_q, "w_q");
    check_cuda_contig(w_s, "w_s");
    check_cuda_contig(expert_offsets, "expert_offsets");
    CAM_ASSERT(a_q.dim() == 2 && w_q.dim() == 3 && a_q.size(1) == w_q.size(2), "a_q [M, K], w_q [E, N, K]");
    CAM_ASSERT(a_q.scalar_type() == at::kFloat8_e4m3fn && w_q.scalar_type() == at::kFloat8_e4m3fn, "operands must be float8_e4m3fn");
    CAM_ASSERT(expert_offsets.scalar_type() == at::kInt && expert_offsets.numel() == w_q.size(0) + 1, "expert_offsets must be int32 [E+1]");
    const int64_t M = a_q.size(0), Kd = a_q.size(1), E = w_q.size(0), N = w_q.size(1);
    CAM_ASSERT(a_s.scalar_type() == at::kFloat && a_s.numel() == M * (Kd / 128), "a_s must be float32 [M, K/128]");
    CAM_ASSERT(w_s.scalar_type() == at::kFloat && w_s.numel() == E * (N / 128) * (Kd / 128), "w_s must be float32 [E, N/128, K/128]");
    c10::cuda::CUDAGuard guard(a_q.device());
    at::Tensor out = at::empty({M, N}, a_q.options().dtype(at::kBFloat16));
    auto gemm = ue8m0 ? &cam_grouped_gemm_mxfp8 : &cam_grouped_gemm_fp8;
    CAM_RT(gemm(nullptr, a_q.data_ptr(), a_s.data_ptr<float>(), static_cast<int>(M), w_q.data_ptr(),
                w_s.data_ptr<float>(), expert_offsets.data_ptr<int>(), static_cast<int>(E), static_cast<int>(N),
                static_cast<int>(Kd), 0, out.data_ptr(), nullptr, nullptr, nullptr, 1, 0,
                at::cuda::getCurrentCUDAStream().stream()));
    return out;
}

// GEMM1 flavour stand-alone: returns (act_q [M, I] e4m3, act_s [M, I/128]).
std::tuple<at::Tensor, at::Tensor> grouped_gemm_fp8_swiglu_cuda(const at::Tensor& a_q, const at::Tensor& a_s,
                                                                const at::Tensor& w_q, const at::Tensor& w_s,
                                                                const at::Tensor& expert_offsets, bool ue8m0) {
    check_cuda_contig(a_q, "a_q");
    check_cuda_contig(a_s, "a_s");
    check_cuda_contig(w_q, "w_q");
    check_cuda_contig(w_s, "w_s");
    const int64_t M = a_q.size(0), Kd = a_q.size(1), E = w_q.size(0), N = w_q.size(1);
    CAM_ASSERT(N % 256 == 0 && a_q.size(1) == w_q.size(2), "w_q must be [E, 2I, K] with 2I a multiple of 256");
    c10::cuda::CUDAGuard guard(a_q.device());
    at::Tensor q = at::zeros({M, N / 2}, a_q.options());
    at::Tensor s = at::zeros({M, N / 2 / 128}, a_s.options());
    auto gemm = ue8m0 ? &cam_grouped_gemm_mxfp8 : &cam_grouped_gemm_fp8;
    CAM_RT(gemm(nullptr, a_q.data_ptr(), a_s.data_ptr<float>(), static_cast<int>(M), w_q.data_ptr(),
                w_s.data_ptr<float>(), expert_offsets.data_ptr<int>(), static_cast<int>(E), static_cast<int>(N),
                static_cast<int>(Kd), 1, nullptr, q.data_ptr(), s.data_ptr<float>(), nullptr, 1, 0,
                at::cuda::getCurrentCUDAStream().stream()));
    return {q, s};
}

// Stand-alone exact W8A8 grouped GEMM: a_q [M, K] int8 + a_s [M], w_q [E, N, K] int8 (K contiguous) + w_s [E, N].
at::Tensor grouped_gemm_w8a8_cuda(const at::Tensor& a_q, const at::Tensor& a_s, const at::Tensor& w_q,
                                  const at::Tensor& w_s, const at::Tensor& expert_offsets) {
    check_cuda_contig(a_q, "a_q");
    check_cuda_contig(a_s, "a_s");
    check_cuda_contig(w_q, "w_q");
    check_cuda_contig(w_s, "w_s");
    check_cuda_contig(expert_offsets, "expert_offsets");
    CAM_ASSERT(a_q.dim() == 2 && w_q.dim() == 3 && a_q.size(1) == w_q.size(2), "a_q [M, K], w_q [E, N, K]");
    CAM_ASSERT(a_q.scalar_type() == at::kChar && w_q.scalar_type() == at::kChar, "operands must be int8");
    const int64_t M = a_q.size(0), Kd = a_q.size(1), E = w_q.size(0), N = w_q.size(1);
    CAM_ASSERT(a_s.scalar_type() == at::kFloat && a_s.numel() == M, "a_s must be float32 [M]");
    CAM_ASSERT(w_s.scalar_type() == at::kFloat && w_s.numel() == E * N, "w_s must be float32 [E, N]");
    CAM_ASSERT(expert_offsets.scalar_type() == at::kInt && expert_offsets.numel() == E + 1, "expert_offsets must be int32 [E+1]");
    c10::cuda::CUDAGuard guard(a_q.device());
    at::Tensor out = at::empty({M, N}, a_q.options().dtype(at::kBFloat16));
    CAM_RT(cam_grouped_gemm_w8a8(a_q.data_ptr(), a_s.data_ptr<float>(), static_cast<int>(M), w_q.data_ptr(),
                                 w_s.data_ptr<float>(), expert_offsets.data_ptr<int>(), static_cast<int>(E),
                                 static_cast<int>(N), static_cast<int>(Kd), out.data_ptr(),
                                 at::cuda::getCurrentCUDAStream().stream()));
    return out;
}

// Autograd-key wrapper: runs below autograd, outputs carry no graph (inference-only op).
std::vector<at::Tensor> fused_deep_moe_autograd(const at::Tensor& x, const at::Tensor& ids, at::TensorList a,
                                                at::TensorList b2, at::TensorList c, at::TensorList d,
                                                const at::Tensor& es, const c10::optional<at::Tensor>& sm,
                                                const c10::optional<at::Tensor>& mask, c10::string_view g, int64_t i0,
                                                int64_t i1, int64_t i2, int64_t i3, int64_t i4, int64_t i5, int64_t i6) {
    at::AutoDispatchBelowADInplaceOrView guard;
    static auto op = c10::Dispatcher::singleton().findSchemaOrThrow("umdk_cam_op_lib::fused_deep_moe", "")
                         .typed<std::vector<at::Tensor>(const at::Tensor&, const at::Tensor&, at::TensorList, at::TensorList,
                                                        at::TensorList, at::TensorList, const at::Tensor&,
                                                        const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&,
                                                        c10::string_view, int64_t, int64_t, int64_t, int64_t, int64_t,
                                                        int64_t, int64_t)>();
    return op.call(x, ids, a, b2, c, d, es, sm, mask, g, i0, i1, i2, i3, i4, i5, i6);
}

}  // namespace

TORCH_LIBRARY(umdk_cam_op_lib, m) {
    m.def("fused_deep_moe(Tensor x, Tensor expertIds, Tensor[] gmm1PermutedWeight, Tensor[] gmm1PermutedWeightScale, "
          "Tensor[] gmm2Weight, Tensor[] gmm2WeightScale, Tensor expertScales, Tensor? expertSmoothScales, "
          "Tensor? xActiveMask, str groupEp, int epRankSize, int epRankId, int moeExpertNum, int sharedExpertNum, "
          "int sharedExpertRankNum, int quantMode, int globalBs) -> Tensor[]");
    m.def("get_dispatch_layout(Tensor topk_idx, int num_experts, int num_ranks) -> (Tensor, Tensor, Tensor)");
    m.def("moe_dispatch_prefill(Tensor x, Tensor topk_idx, Tensor topk_weights, Tensor num_tokens_per_rank, "
          "Tensor is_token_in_rank, Tensor num_tokens_per_expert, int num_worst_tokens, str group_ep, int rank, "
          "int num_ranks) -> (Tensor, Tensor, Tensor, Tensor)");
    m.def("moe_combine_prefill(Tensor x, Tensor topk_idx, Tensor topk_weights, Tensor src_idx, Tensor send_head, "
          "str group_ep, int rank, int num_ranks) -> Tensor");
    m.def("moe_dispatch_shmem(Tensor x, Tensor expertIds, Tensor? scales, Tensor? xActiveMask, int epWorldSize, "
          "int epRankId, int moeExpertNum, int tpWorldSize, int tpRankId, int expertShardType, int sharedExpertNum, "
          "int sharedExpertRankNum, int quantMode, int globalBS, int expertTokenNumsType, int extInfo) -> Tensor[]");
    m.def("moe_combine_shmem(Tensor expandX, Tensor expertIds, Tensor expandIdx, Tensor epSendCounts, "
          "Tensor expertScales, Tensor? tpSendCounts, Tensor? xActiveMask, Tensor? activationScale, "
          "Tensor? weightScale, Tensor? groupList, Tensor? expandScales, int epWorldSize, int epRankId, "
          "int moeExpertNum, int tpWorldSize, int tpRankId, int expertShardType, int sharedExpertNum, "
          "int sharedExpertRankNum, int globalBS, int commQuantMode, int extInfo, int outDtype, int groupListType) "
          "-> Tensor");
    // additions of this library (no counterpart schema in the reference)
    m.def("moe_dispatch_prefill_quant(Tensor x, Tensor topk_idx, Tensor topk_weights, int num_worst_tokens, "
          "str group_ep, int rank, int num_ranks, int quant_mode) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");
    m.def("grouped_gemm_fp8(Tensor a_q, Tensor a_s, Tensor w_q, Tensor w_s, Tensor expert_offsets, "
          "bool ue8m0=False) -> Tensor");
    m.def("grouped_gemm_fp8_swiglu(Tensor a_q, Tensor a_s, Tensor w_q, Tensor w_s, Tensor expert_offsets, "
          "bool ue8m0=False) -> (Tensor, Tensor)");
    m.def("grouped_gemm_w8a8(Tensor a_q, Tensor a_s, Tensor w_q, Tensor w_s, Tensor expert_offsets) -> Tensor");
}

TORCH_LIBRARY_IMPL(umdk_cam_op_lib, CUDA, m) {
    m.impl("fused_deep_moe", &fused_deep_moe_cuda);
    m.impl("get_dispatch_layout", &get_dispatch_layout_cuda);
    m.impl("moe_dispatch_prefill", &moe_dispatch_prefill_cuda);
    m.impl("moe_combine_prefill", &moe_combine_prefill_cuda);
    m.impl("moe_dispatch_shmem", &moe_dispatch_shmem_cuda);
    m.impl("moe_combine_shmem", &moe_combine_shmem_cuda);
    m.impl("moe_dispatch_prefill_quant", &moe_dispatch_prefill_quant_cuda);
    m.impl("grouped_gemm_fp8", &grouped_gemm_fp8_cuda);
    m.impl("grouped_gemm_fp8_swiglu", &grouped_gemm_fp8_swiglu_cuda);
    m.impl("grouped_gemm_w8a8", &grouped_gemm_w8a8_cuda);
}

TORCH_LIBRARY_IMPL(umdk_cam_op_lib, Meta, m) {
    m.impl("fused_deep_moe", &fused_deep_moe_meta);
    m.impl("get_dispatch_layout", &get_dispatch_layout_meta);
    m.impl("moe_dispatch_shmem", &moe_dispatch_shmem_meta);
    m.impl("moe_combine_shmem", &moe_combine_shmem_meta);
}

TORCH_LIBRARY_IMPL(umdk_cam_op_lib, Autograd, m) {
    m.impl("fused_deep_moe", &fused_deep_moe_autograd);
    m.impl("get_dispatch_layout", torch::autograd::autogradNotImplementedFallback());
    m.impl("moe_dispatch_prefill", torch::autograd::autogradNotImplementedFallback());
    m.impl("moe_combine_prefill", torch::autograd::autogradNotImplementedFallback());
    m.impl("moe_dispatch_shmem", torch::autograd::autogradNotImplementedFallback());
    m.impl("moe_combine_shmem", torch::autograd::autogradNotImplementedFallback());
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "umdk_cam_op_lib for B200: symmetric Buffer + op registrations";
    py::class_<Buffer>(m, "Buffer")
        .def(py::init<int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t>(),
             py::arg("device"), py::arg("rank"), py::arg("num_ranks"), py::arg("num_experts"), py::arg("max_tokens"),
             py::arg("hidden"), py::arg("topk"), py::arg("capacity"), py::arg("ll_max_tokens") = 0,
             py::arg("tp_rows") = 0)
        .def("open_ipc_tp_peer", &Buffer::open_ipc_tp_peer)
        .def("set_local_tp_peer", &Buffer::set_local_tp_peer)
        .def("destroy", &Buffer::destroy)
        .def("register_name", &Buffer::register_name)
        .def_property_readonly("id", &Buffer::id)
        .def_property_readonly("name", &Buffer::name)
        .def_property_readonly("total_bytes", &Buffer::total_bytes)
        .def_property_readonly("capacity", &Buffer::capacity)
        .def("ipc_handle", &Buffer::ipc_handle)
        .def("open_ipc_peers", &Buffer::open_ipc_peers)
        .def("set_local_peers", &Buffer::set_local_peers)
        .def("reset", &Buffer::reset)
        .def("set_timeout_ms", &Buffer::set_timeout_ms)
        .def("set_debug_drop_flags", &Buffer::set_debug_drop_flags)
        .def("set_copy_outputs", &Buffer::set_copy_outputs)
        .def("barrier", &Buffer::barrier)
        .def("p2p_write", &Buffer::p2p_write)
        .def("p2p_pingpong", &Buffer::p2p_pingpong)
        .def("set_trace", &Buffer::set_trace)
        .def("read_trace", &Buffer::read_trace)
        .def("launch_count", &Buffer::launch_count)
        .def("fused_route", &Buffer::fused_route)
        .def("read_stats", &Buffer::read_stats)
        .def("check_guards", &Buffer::check_guards)
        .def("guard", &Buffer::guard)
        .def("set_fused_trace", &Buffer::set_fused_trace)
        .def("read_fused_trace", &Buffer::read_fused_trace)
        .def("read_fused_waits", &Buffer::read_fused_waits)
        .def("set_profile", &Buffer::set_profile)
        .def("read_profile", &Buffer::read_profile)
        .def("poll_status", &Buffer::poll_status)
        .def("recv_x", &Buffer::recv_x)
        .def("recv_scales", &Buffer::recv_scales)
        .def("recv_src", &Buffer::recv_src)
        .def("recv_count", &Buffer::recv_count)
        .def("expert_offsets", &Buffer::expert_offsets)
        .def("num_recv_per_expert", &Buffer::num_recv_per_expert)
        .def("total_recv", &Buffer::total_recv)
        .def("send_row", &Buffer::send_row)
        .def("num_tokens_per_expert", &Buffer::num_tokens_per_expert)
        .def("act_q", &Buffer::act_q)
        .def("act_s", &Buffer::act_s);
    m.def("set_phase_mask", [](int mask) { g_phase_mask = mask; });
    m.def("get_phase_mask", []() { return g_phase_mask; });
    m.def("status_string", [](int code) { return std::string(cam_status_string(code)); });
}
