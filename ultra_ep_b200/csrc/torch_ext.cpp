// PyTorch extension shim: the `_C` module of the reference (csrc/python_api.cpp,
// csrc/ultra_ep.hpp:328-613, csrc/runtime.cpp:69-73, csrc/utils/event.hpp:46-50 of the
// reference) re-created on top of the C ABI in include/uep_b200.h.
//
// The shim holds no logic of the balancing path. It converts tensors to pointers, looks up
// the current stream, wraps library-owned memory as tensors without a deleter (valid until
// destroy(), as in the reference) and turns status codes into Python exceptions.

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <cstring>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

#include "uep_b200.h"

namespace py = pybind11;

namespace {

[[noreturn]] void raise_last(const char* what) {
    throw std::runtime_error(std::string(what) + ": " + uep_last_error());
}
void check(int rc, const char* what) {
    if (rc != UEP_OK) raise_last(what);
}
#define UEP_ASSERT(cond)                                                                                  \
    do {                                                                                                  \
        if (!(cond)) throw std::runtime_error(std::string("Assertion exception (" __FILE__ "): ") + #cond); \
    } while (0)

// ---- process-wide runtime facts (csrc/runtime.cpp:10-14 of the reference) ----------------
struct Runtime {
    bool initialized = false;
    int rank = -1, num_ranks = 0, num_nvl_ranks = 0;
    // callable(bytes) -> list[bytes], all-gather over the EP group. Held through a pointer that is
    // never deleted: a static py::object would drop its reference after the interpreter is gone.
    py::object* exchange = nullptr;
} g_rt;

void* current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

struct EventHandle {
    std::shared_ptr<uep_event> ev;
    EventHandle() {
        uep_event* e = nullptr;
        check(uep_event_record(current_stream(), &e), "EventHandle");
        ev = std::shared_ptr<uep_event>(e, uep_event_destroy);
    }
    explicit EventHandle(uep_event* e) : ev(e, uep_event_destroy) {}
    void current_stream_wait() const { check(uep_event_stream_wait(ev.get(), current_stream()), "current_stream_wait"); }
};

torch::Tensor wrap(uep_manager* m, int buffer_id, torch::ScalarType dtype, int device) {
    void* ptr = nullptr;
    int ndim = 0;
    int64_t shape[3], stride[3];
    check(uep_manager_buffer(m, 0, buffer_id, &ptr, &ndim, shape, stride), "manager_buffer");
    std::vector<int64_t> sh(shape, shape + ndim), st(stride, stride + ndim);
    auto opts = torch::TensorOptions().dtype(dtype).device(torch::Device(torch::kCUDA, device));
    bool empty = false;
    for (auto s : sh) empty = empty || s == 0;
    if (empty || ptr == nullptr) return torch::empty(sh, opts);
    return torch::from_blob(ptr, sh, st, opts);
}

const int64_t* ptr_table(const torch::Tensor& t, int expect, const char* name) {
    if (!(t.is_cuda() && t.dtype() == torch::kInt64 && t.numel() == expect))
        throw std::runtime_error(std::string(name) + " must be a cuda int64 tensor with one entry per local master expert");
    return t.data_ptr<int64_t>();
}

class Manager {
    uep_manager* m_ = nullptr;
    bool available_ = false;
    bool explicitly_destroy_ = false;
    bool is_train_ = true;
    int M_ = 0, R_ = 0, L_ = 0, P_ = 0, device_ = 0;
    bool has_scales_ = false;
    bool legacy_ = false;

public:
    Manager(int num_layers, int num_local_master_experts, int num_local_redundant_experts, int64_t expert_fc1_numel,
            int64_t expert_fc2_numel, int weight_data_element_bytes, int weight_scale_element_bytes,
            int64_t expert_fc1_weight_scale_numel, int64_t expert_fc2_weight_scale_numel, int grad_element_bytes,
            bool is_train, bool explicitly_destroy, bool legacy_placement, float balance_threshold,
            bool quota_locality_aware, int32_t quota_min_tokens_per_replica, bool quota_allow_zero_master_quota,
            float quota_oracle_eps, int quota_kernel_stage, bool quota_reroute_interleave, int grad_reduce_num_sms,
            bool grad_reduce_deterministic, int weight_sync_plan_mode, int weight_sync_relay_min_replicas,
            int weight_sync_relay_max_relays, int weight_sync_relay_min_fanout_gain)
        : explicitly_destroy_(explicitly_destroy), is_train_(is_train), legacy_(legacy_placement) {
        if (!g_rt.initialized) throw std::runtime_error("Runtime must be initialized before creating Manager");
        uep_config cfg;
        std::memset(&cfg, 0, sizeof(cfg));
        cfg.num_ranks = g_rt.num_ranks;
        cfg.nvl_ranks = g_rt.num_nvl_ranks;
        cfg.rank = g_rt.rank;
        cfg.sim_ranks = 0;
        cfg.num_layers = num_layers;
        cfg.num_local_master_experts = num_local_master_experts;
        cfg.num_local_redundant_experts = num_local_redundant_experts;
        cfg.expert_fc1_numel = expert_fc1_numel;
        cfg.expert_fc2_numel = expert_fc2_numel;
        cfg.weight_data_element_bytes = weight_data_element_bytes;
        cfg.weight_scale_element_bytes = weight_scale_element_bytes;
        cfg.expert_fc1_weight_scale_numel = expert_fc1_weight_scale_numel;
        cfg.expert_fc2_weight_scale_numel = expert_fc2_weight_scale_numel;
        cfg.grad_element_bytes = grad_element_bytes;
        cfg.is_train = is_train;
        cfg.legacy_placement = legacy_placement;
        cfg.solver.balance_threshold = balance_threshold;
        cfg.solver.locality_aware = quota_locality_aware;
        cfg.solver.min_tokens_per_replica = quota_min_tokens_per_replica;
        cfg.solver.allow_zero_master_quota = quota_allow_zero_master_quota;
        cfg.solver.oracle_eps = quota_oracle_eps;
        cfg.solver.reroute_interleave = quota_reroute_interleave;
        cfg.quota_kernel_stage = quota_kernel_stage;
        cfg.grad_reduce_num_sms = grad_reduce_num_sms;
        cfg.grad_reduce_deterministic = grad_reduce_deterministic;
        cfg.weight_sync_plan_mode = weight_sync_plan_mode;
        cfg.weight_sync_relay_min_replicas = weight_sync_relay_min_replicas;
        cfg.weight_sync_relay_max_relays = weight_sync_relay_max_relays;
        cfg.weight_sync_relay_min_fanout_gain = weight_sync_relay_min_fanout_gain;
        const char* sms = std::getenv("ULTRA_EP_WEIGHT_SYNC_NUM_SMS");
        cfg.weight_sync_num_sms = sms ? std::atoi(sms) : 0;
        const char* to = std::getenv("ULTRA_EP_WAIT_TIMEOUT_MS");
        cfg.wait_timeout_ms = to ? std::atoi(to) : 0;
        const char* mt = std::getenv("ULTRA_EP_REROUTE_MAX_TOKENS");  // > 0: the reroute scratch never grows after construction
        cfg.reroute_max_tokens = mt ? std::atoi(mt) : 0;
        const char* mk = std::getenv("ULTRA_EP_REROUTE_MAX_TOPK");
        cfg.reroute_max_topk = mk ? std::atoi(mk) : 0;
        check(uep_manager_create(&cfg, &m_), "Manager");
        M_ = num_local_master_experts;
        R_ = num_local_redundant_experts;
        L_ = M_ * g_rt.num_ranks;
        P_ = (M_ + R_) * g_rt.num_ranks;
        has_scales_ = (expert_fc1_weight_scale_numel + expert_fc2_weight_scale_numel) > 0;
        device_ = at::cuda::current_device();
        // collective part: all-gather the 64-byte arena handles over the EP group
        try {
            char handle[UEP_IPC_HANDLE_BYTES];
            check(uep_manager_export_handle(m_, handle), "export_handle");
            std::string all;
            if (g_rt.num_ranks > 1) {
                if (g_rt.exchange == nullptr || g_rt.exchange->is_none())
                    throw std::runtime_error("no handle exchange registered (call init_runtime first)");
                py::list parts = (*g_rt.exchange)(py::bytes(handle, sizeof(handle)));
                if (static_cast<int>(py::len(parts)) != g_rt.num_ranks) throw std::runtime_error("handle exchange returned a wrong count");
                for (auto item : parts) {
                    std::string s = py::cast<py::bytes>(item);
                    if (s.size() != UEP_IPC_HANDLE_BYTES) throw std::runtime_error("handle exchange returned a wrong size");
                    all += s;
                }
            } else {
                all.assign(handle, sizeof(handle));
            }
            check(uep_manager_connect(m_, all.data()), "connect");
        } catch (...) {
            uep_manager_destroy(m_);
            m_ = nullptr;
            throw;
        }
        available_ = true;
    }

    ~Manager() {
        if (!available_) return;
        // The arena is mapped by the peers, and their kernels store into it. It may only be freed behind a barrier
        // over the group, which this destructor cannot make (the reference's destructor can: its barrier is
        // NVSHMEM's, csrc/ultra_ep.cpp:534-549). The Python Manager makes it and then calls destroy(); if nobody
        // did, a group of several ranks keeps the memory until the process exits instead of freeing it under a peer.
        if (!explicitly_destroy_ && g_rt.num_ranks <= 1) {
            uep_manager_destroy(m_);  // no exception from a destructor
        } else {
            std::printf("WARNING: destroy() was not called before UltraEP manager destruction; its peer-visible memory "
                        "stays allocated until the process exits.\n");
            std::fflush(stdout);
        }
        m_ = nullptr;
        available_ = false;
    }

    // Gives up the native resources without freeing them (no barrier over the group could be made).
    void abandon() {
        m_ = nullptr;
        available_ = false;
    }

    void destroy() {
        UEP_ASSERT(available_);
        check(uep_manager_destroy(m_), "destroy");
        m_ = nullptr;
        available_ = false;
    }
    bool is_available() const { return available_; }

    void update_placement(int layer_id, torch::Tensor& routing_map) {
        UEP_ASSERT(available_);
        UEP_ASSERT(routing_map.is_cuda() && routing_map.dim() == 2 && routing_map.size(1) == L_ &&
                   routing_map.dtype() == torch::kBool);
        auto rm = routing_map.contiguous();
        const void* in = rm.data_ptr();
        const int T = static_cast<int>(rm.size(0));
        check(uep_update_placement(m_, layer_id, 0, &in, &T, L_, current_stream()), "update_placement");
    }

    void update_placement_sparse(int layer_id, torch::Tensor& topk_ids) {
        UEP_ASSERT(available_);
        UEP_ASSERT(topk_ids.is_cuda() && topk_ids.dim() == 2);
        UEP_ASSERT(topk_ids.dtype() == torch::kInt64 || topk_ids.dtype() == torch::kInt32);
        auto ids = topk_ids.contiguous();
        // as the reference: on the communication stream, after the current stream (csrc/ultra_ep.cpp:757-759)
        void* comm = uep_manager_comm_stream(m_);
        uep_event* ev = nullptr;
        check(uep_event_record(current_stream(), &ev), "update_placement_sparse");
        const int rc = uep_event_stream_wait(ev, comm);
        uep_event_destroy(ev);
        check(rc, "update_placement_sparse");
        const void* in = ids.data_ptr();
        const int T = static_cast<int>(ids.size(0));
        const int kind = ids.dtype() == torch::kInt64 ? 2 : 1;
        check(uep_update_placement(m_, layer_id, kind, &in, &T, static_cast<int>(ids.size(1)), comm),
              "update_placement_sparse");
    }

    void reroute_sparse(int layer_id, torch::Tensor& topk_ids) {
        UEP_ASSERT(available_);
        UEP_ASSERT(topk_ids.is_cuda() && topk_ids.dim() == 2 && topk_ids.is_contiguous());
        UEP_ASSERT(topk_ids.dtype() == torch::kInt64 || topk_ids.dtype() == torch::kInt32);
        const void* in = topk_ids.data_ptr();
        void* out = topk_ids.data_ptr();
        const int T = static_cast<int>(topk_ids.size(0));
        const int kind = topk_ids.dtype() == torch::kInt64 ? 2 : 1;
        check(uep_reroute_sparse(m_, layer_id, kind, &in, &out, &T, static_cast<int>(topk_ids.size(1)), current_stream()),
              "reroute_sparse");
    }

    std::tuple<torch::Tensor, torch::Tensor> dense_reroute_forward(int layer_id, torch::Tensor& probs,
                                                                   torch::Tensor& routing_map) {
        UEP_ASSERT(available_);
        UEP_ASSERT(routing_map.is_cuda() && probs.is_cuda());
        UEP_ASSERT(routing_map.dtype() == torch::kBool);
        UEP_ASSERT(probs.scalar_type() == torch::kFloat32);
        UEP_ASSERT(routing_map.dim() == 2 && routing_map.size(1) == L_ && probs.sizes() == routing_map.sizes());
        probs = probs.contiguous();
        routing_map = routing_map.contiguous();
        const int T = static_cast<int>(routing_map.size(0));
        auto dev = routing_map.device();
        // every element is written by the kernel: no zero-fill pass
        auto expanded_probs = torch::empty({T, P_}, torch::TensorOptions().dtype(torch::kFloat32).device(dev));
        auto expanded_rmap = torch::empty({T, P_}, torch::TensorOptions().dtype(torch::kBool).device(dev));
        const uint8_t* maps = reinterpret_cast<const uint8_t*>(routing_map.data_ptr());
        const float* pr = probs.data_ptr<float>();
        uint8_t* om = reinterpret_cast<uint8_t*>(expanded_rmap.data_ptr());
        float* op = expanded_probs.data_ptr<float>();
        check(uep_reroute_dense_forward(m_, layer_id, &maps, &pr, &om, &op, &T, current_stream()), "dense_reroute_forward");
        return std::make_tuple(expanded_probs, expanded_rmap);
    }

    torch::Tensor dense_reroute_backward(int layer_id, torch::Tensor& grad_expanded_probs, torch::Tensor& routing_map,
                                         torch::Tensor& expanded_routing_map) {
        UEP_ASSERT(available_);
        UEP_ASSERT(grad_expanded_probs.is_cuda() && routing_map.is_cuda() && expanded_routing_map.is_cuda());
        UEP_ASSERT(grad_expanded_probs.scalar_type() == torch::kFloat32);
        grad_expanded_probs = grad_expanded_probs.contiguous();
        routing_map = routing_map.contiguous();
        auto em = expanded_routing_map.contiguous();
        const int T = static_cast<int>(routing_map.size(0));
        const int P = static_cast<int>(grad_expanded_probs.size(1));
        auto grad_probs = torch::empty({T, L_}, torch::TensorOptions().dtype(torch::kFloat32).device(routing_map.device()));
        const float* g = grad_expanded_probs.data_ptr<float>();
        const uint8_t* maps = reinterpret_cast<const uint8_t*>(routing_map.data_ptr());
        const uint8_t* emaps = reinterpret_cast<const uint8_t*>(em.data_ptr());
        float* out = grad_probs.data_ptr<float>();
        check(uep_reroute_dense_backward(m_, layer_id, &g, &maps, &emaps, &out, &T, P, current_stream()),
              "dense_reroute_backward");
        return grad_probs;
    }

    std::optional<EventHandle> grad_reduce(int layer_id, torch::Tensor& fc1_grad_ptrs, torch::Tensor& fc2_grad_ptrs,
                                           std::optional<EventHandle>& previous_event, bool async_finish) {
        UEP_ASSERT(available_);
        const int64_t* a = ptr_table(fc1_grad_ptrs, M_, "local_master_fc1_grad_ptr_tensor");
        const int64_t* b = ptr_table(fc2_grad_ptrs, M_, "local_master_fc2_grad_ptr_tensor");
        uep_event* done = nullptr;
        check(uep_grad_reduce(m_, layer_id, &a, &b, previous_event ? previous_event->ev.get() : nullptr, async_finish,
                              current_stream(), &done), "grad_reduce");
        if (async_finish) return EventHandle(done);
        return std::nullopt;
    }

    std::optional<EventHandle> weight_sync(int layer_id, torch::Tensor& fc1_ptrs, torch::Tensor& fc2_ptrs,
                                           torch::Tensor& fc1_scale_ptrs, torch::Tensor& fc2_scale_ptrs,
                                           std::optional<EventHandle>& previous_event, bool async_finish) {
        UEP_ASSERT(available_);
        const int64_t* a = ptr_table(fc1_ptrs, M_, "local_master_fc1_weight_ptr_tensor");
        const int64_t* b = ptr_table(fc2_ptrs, M_, "local_master_fc2_weight_ptr_tensor");
        const int64_t* c = nullptr;
        const int64_t* d = nullptr;
        if (has_scales_) {
            c = ptr_table(fc1_scale_ptrs, M_, "local_master_fc1_weight_scale_ptr_tensor");
            d = ptr_table(fc2_scale_ptrs, M_, "local_master_fc2_weight_scale_ptr_tensor");
        }
        uep_event* done = nullptr;
        check(uep_weight_sync(m_, layer_id, &a, &b, has_scales_ ? &c : nullptr, has_scales_ ? &d : nullptr,
                              previous_event ? previous_event->ev.get() : nullptr, async_finish, current_stream(), &done),
              "weight_sync");
        if (async_finish) return EventHandle(done);
        return std::nullopt;
    }

    torch::Stream get_comm_stream() const {
        return at::cuda::getStreamFromExternal(static_cast<cudaStream_t>(uep_manager_comm_stream(m_)), device_).unwrap();
    }
    void set_weight_sync_plan_mode(int plan_mode) { check(uep_set_weight_sync_plan_mode(m_, plan_mode), "set_weight_sync_plan_mode"); }
    void set_grad_reduce_deterministic(bool deterministic, int num_sms) {
        check(uep_set_grad_reduce_deterministic(m_, deterministic, num_sms), "set_grad_reduce_deterministic");
    }
    std::tuple<int, int> poll_status() const {
        int code = 0, detail = 0;
        uep_poll_status(m_, 0, &code, &detail);
        return std::make_tuple(code, detail);
    }
    void clear_status() { check(uep_clear_status(m_), "clear_status"); }

    torch::Tensor buf(int id, torch::ScalarType dt) const {
        UEP_ASSERT(available_);
        return wrap(m_, id, dt, device_);
    }
    torch::Tensor grad_buf(int id) const {
        if (!is_train_) throw std::runtime_error("Assertion exception: is_train && \"Grad buffer not available in inference mode\"");
        return buf(id, torch::kFloat32);
    }
};

// Single-GPU test hooks with the reference's signatures (csrc/ultra_ep.hpp:427-612).
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor>
solve_placement_for_test(torch::Tensor expert_loads, torch::Tensor expert_loads_per_rank, int num_ranks,
                         int num_local_master_experts, int num_local_redundant_experts, int num_nvl_ranks,
                         bool legacy_placement, float balance_threshold, int32_t min_tokens_per_replica,
                         bool allow_zero_master_quota, bool locality_aware, float oracle_eps, int kernel_stage,
                         int rank_quota_source_rank) {
    UEP_ASSERT(expert_loads.is_cuda() && expert_loads.dtype() == torch::kInt32 && expert_loads.dim() == 1);
    UEP_ASSERT(num_ranks > 0 && num_nvl_ranks > 0 && num_ranks % num_nvl_ranks == 0);
    UEP_ASSERT(num_local_master_experts > 0 && num_local_redundant_experts >= 0);
    UEP_ASSERT(kernel_stage == 0 || kernel_stage == 1);
    const int L = static_cast<int>(expert_loads.size(0));
    UEP_ASSERT(L == num_ranks * num_local_master_experts);
    UEP_ASSERT(expert_loads_per_rank.defined() && expert_loads_per_rank.is_cuda() &&
               expert_loads_per_rank.dtype() == torch::kInt32 && expert_loads_per_rank.dim() == 2 &&
               expert_loads_per_rank.size(0) == num_ranks && expert_loads_per_rank.size(1) == L);
    const int P = num_ranks * (num_local_master_experts + num_local_redundant_experts);
    auto opts = torch::TensorOptions().dtype(torch::kInt32).device(expert_loads.device());
    auto p2l = torch::empty({P}, opts);
    auto l2p = torch::empty({L, num_ranks}, opts);
    auto lcnts = torch::empty({L}, opts);
    auto quota = torch::empty({L, num_ranks}, opts);
    auto quota_prefix = torch::empty({L, num_ranks}, opts);
    auto rqp = torch::empty({L, num_ranks}, opts);
    auto loads_sum = torch::empty({L}, opts);  // the sum over ranks is recomputed on the device
    auto lpr = expert_loads_per_rank.contiguous();
    uep_solver_params prm{balance_threshold, locality_aware, min_tokens_per_replica, allow_zero_master_quota, oracle_eps, 1};
    const int src = rank_quota_source_rank >= 0 ? rank_quota_source_rank : (g_rt.initialized ? g_rt.rank : 0);
    if (legacy_placement) {  // counts-only greedy plan from the total loads; quotas zero (csrc/ultra_ep.hpp:480-505 of the reference)
        auto loads = expert_loads.contiguous();
        check(uep_legacy_solve_placement(loads.data_ptr<int32_t>(), p2l.data_ptr<int32_t>(), l2p.data_ptr<int32_t>(),
                                         lcnts.data_ptr<int32_t>(), quota.data_ptr<int32_t>(),
                                         quota_prefix.data_ptr<int32_t>(), rqp.data_ptr<int32_t>(), num_ranks,
                                         num_nvl_ranks, num_local_master_experts, num_local_redundant_experts, num_ranks,
                                         balance_threshold, nullptr, current_stream()), "solve_placement_for_test");
        return std::make_tuple(p2l, l2p, lcnts, quota, quota_prefix, rqp);
    }
    check(uep_solve_placement(lpr.data_ptr<int32_t>(), loads_sum.data_ptr<int32_t>(), p2l.data_ptr<int32_t>(),
                              l2p.data_ptr<int32_t>(), lcnts.data_ptr<int32_t>(), quota.data_ptr<int32_t>(),
                              quota_prefix.data_ptr<int32_t>(), rqp.data_ptr<int32_t>(), num_ranks, num_nvl_ranks,
                              num_local_master_experts, num_local_redundant_experts, num_ranks, &prm, src, nullptr,
                              current_stream()), "solve_placement_for_test");
    return std::make_tuple(p2l, l2p, lcnts, quota, quota_prefix, rqp);
}

std::tuple<torch::Tensor, torch::Tensor> dense_reroute_for_test(torch::Tensor routing_map, torch::Tensor probs,
                                                                torch::Tensor l2p, torch::Tensor lcnts,
                                                                torch::Tensor rank_quota_prefix,
                                                                int num_global_physical_experts, bool quota_reroute,
                                                                bool interleave_by_rank_quota) {
    UEP_ASSERT(routing_map.is_cuda() && routing_map.dtype() == torch::kBool);
    UEP_ASSERT(probs.is_cuda() && probs.dtype() == torch::kFloat32);
    UEP_ASSERT(l2p.is_cuda() && l2p.dtype() == torch::kInt32 && l2p.dim() == 2);
    UEP_ASSERT(lcnts.is_cuda() && lcnts.dtype() == torch::kInt32 && lcnts.dim() == 1);
    UEP_ASSERT(rank_quota_prefix.is_cuda() && rank_quota_prefix.dtype() == torch::kInt32 && rank_quota_prefix.dim() == 2);
    UEP_ASSERT(routing_map.dim() == 2 && probs.dim() == 2 && routing_map.sizes() == probs.sizes());
    const int T = static_cast<int>(routing_map.size(0)), L = static_cast<int>(routing_map.size(1));
    const int D = static_cast<int>(l2p.size(1));
    UEP_ASSERT(l2p.size(0) == L && lcnts.size(0) == L && rank_quota_prefix.size(0) == L && rank_quota_prefix.size(1) == D);
    auto rm = routing_map.contiguous();
    auto pr = probs.contiguous();
    auto l2pc = l2p.contiguous();
    auto lc = lcnts.contiguous();
    auto rq = rank_quota_prefix.contiguous();
    const int P = num_global_physical_experts;
    auto out_probs = torch::empty({T, P}, torch::TensorOptions().dtype(torch::kFloat32).device(probs.device()));
    auto out_map = torch::empty({T, P}, torch::TensorOptions().dtype(torch::kBool).device(probs.device()));
    auto scratch = torch::empty({uep_reroute_scratch_elems(T, 0, L)},
                                torch::TensorOptions().dtype(torch::kInt32).device(probs.device()));
    check(uep_dense_reroute_forward(reinterpret_cast<const uint8_t*>(rm.data_ptr()), pr.data_ptr<float>(),
                                    l2pc.data_ptr<int32_t>(), lc.data_ptr<int32_t>(), rq.data_ptr<int32_t>(),
                                    reinterpret_cast<uint8_t*>(out_map.data_ptr()), out_probs.data_ptr<float>(),
                                    scratch.data_ptr<int32_t>(), T, L, P, D, quota_reroute, interleave_by_rank_quota,
                                    current_stream()), "dense_reroute_for_test");
    return std::make_tuple(out_probs, out_map);
}

// NVLink-domain size: ranks of the group that sit on this host and whose devices this
// device can reach peer-to-peer (the reference probes with a test allocation,
// csrc/utils/ipc_manager.cu:174-209; the answer is the same on a single NVSwitch box).
struct IpcManager {
    bool is_fabric_supported() const { return false; }
    int detect_accessible_ranks(py::object group) const {
        py::module_ dist = py::module_::import("torch.distributed");
        py::module_ socket = py::module_::import("socket");
        const int world = py::cast<int>(dist.attr("get_world_size")(group));
        int device = 0;
        cudaGetDevice(&device);
        py::list gathered;
        for (int i = 0; i < world; ++i) gathered.append(py::none());
        dist.attr("all_gather_object")(gathered, py::make_tuple(socket.attr("gethostname")(), device), group);
        const std::string my_host = py::cast<std::string>(socket.attr("gethostname")());
        int count = 0;
        for (auto item : gathered) {
            py::tuple t = py::cast<py::tuple>(item);
            const std::string host = py::cast<std::string>(t[0]);
            const int dev = py::cast<int>(t[1]);
            if (host != my_host) continue;
            int can = dev == device ? 1 : 0;
            if (!can) cudaDeviceCanAccessPeer(&can, device, dev);
            count += can ? 1 : 0;
        }
        return count;
    }
};

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "B200-native drop-in for the reference's ultra_ep._C module";
    m.def("get_local_nvshmem_unique_id", [](int rank) {
        // kept for call compatibility: there is no NVSHMEM here, the token is not used
        if (rank != 0) throw std::runtime_error("Only rank 0 can get the unique id");
        return py::bytes(std::string(128, '\0'));
    });
    m.def("is_runtime_initialized", []() { return g_rt.initialized; });
    m.def("init_runtime", [](int rank, int num_ranks, int max_nvl_peers, py::object root_unique_id) {
        (void)root_unique_id;
        if (num_ranks <= 0 || rank < 0 || rank >= num_ranks) throw std::runtime_error("init_runtime: bad rank / size");
        if (max_nvl_peers <= 0 || max_nvl_peers > 72 || num_ranks % max_nvl_peers != 0)
            throw std::runtime_error("init_runtime: num_ranks must be a multiple of the NVLink-domain size (<= 72)");
        g_rt.rank = rank;
        g_rt.num_ranks = num_ranks;
        g_rt.num_nvl_ranks = max_nvl_peers;
        g_rt.initialized = true;
    });
    m.def("set_handle_exchange", [](py::object fn) {
              if (g_rt.exchange == nullptr) g_rt.exchange = new py::object();
              *g_rt.exchange = fn;
          },
          "callable(bytes) -> list[bytes]: all-gather over the EP group, used once per Manager construction");
    m.def("shutdown_runtime", []() {
        if (g_rt.exchange != nullptr) *g_rt.exchange = py::none();
        g_rt.initialized = false;
    });
    m.def("launch_count", []() { return uep_launch_count(); });
    m.def("reset_launch_count", []() { uep_reset_launch_count(); });

    py::class_<IpcManager>(m, "IpcManager")
        .def(py::init<>())
        .def("is_fabric_supported", &IpcManager::is_fabric_supported)
        .def("detect_accessible_ranks", &IpcManager::detect_accessible_ranks);

    py::class_<EventHandle>(m, "EventHandle").def(py::init<>()).def("current_stream_wait", &EventHandle::current_stream_wait);

    py::class_<Manager>(m, "Manager")
        .def(py::init<int, int, int, int64_t, int64_t, int, int, int64_t, int64_t, int, bool, bool, bool, float, bool,
                      int32_t, bool, float, int, bool, int, bool, int, int, int, int>(),
             py::arg("num_layers"), py::arg("num_local_master_experts"), py::arg("num_local_redundant_experts"),
             py::arg("expert_fc1_numel"), py::arg("expert_fc2_numel"), py::arg("weight_data_element_bytes"),
             py::arg("weight_scale_element_bytes"), py::arg("expert_fc1_weight_scale_numel"),
             py::arg("expert_fc2_weight_scale_numel"), py::arg("grad_element_bytes"), py::arg("is_train"),
             py::arg("explicitly_destroy"), py::arg("legacy_placement") = false, py::arg("balance_threshold") = 1.0f,
             py::arg("quota_locality_aware") = true, py::arg("quota_min_tokens_per_replica") = 1,
             py::arg("quota_allow_zero_master_quota") = true, py::arg("quota_oracle_eps") = 0.01f,
             py::arg("quota_kernel_stage") = 1, py::arg("quota_reroute_interleave") = true,
             py::arg("grad_reduce_num_sms") = 24, py::arg("grad_reduce_deterministic") = true,
             py::arg("weight_sync_plan_mode") = 1, py::arg("weight_sync_relay_min_replicas") = 4,
             py::arg("weight_sync_relay_max_relays") = 8, py::arg("weight_sync_relay_min_fanout_gain") = 2)
        .def("destroy", &Manager::destroy)
        .def("abandon", &Manager::abandon)
        .def("is_available", &Manager::is_available)
        .def("update_placement", &Manager::update_placement)
        .def("update_placement_sparse", &Manager::update_placement_sparse)
        .def("reroute_sparse", &Manager::reroute_sparse)
        .def("dense_reroute_forward", &Manager::dense_reroute_forward)
        .def("dense_reroute_backward", &Manager::dense_reroute_backward)
        .def("grad_reduce", &Manager::grad_reduce, py::arg("layer_id"), py::arg("local_master_fc1_grad_ptr_tensor"),
             py::arg("local_master_fc2_grad_ptr_tensor"), py::arg("previous_event"), py::arg("async_finish"))
        .def("weight_sync", &Manager::weight_sync, py::arg("layer_id"), py::arg("local_master_fc1_weight_ptr_tensor"),
             py::arg("local_master_fc2_weight_ptr_tensor"), py::arg("local_master_fc1_weight_scale_ptr_tensor"),
             py::arg("local_master_fc2_weight_scale_ptr_tensor"), py::arg("previous_event"), py::arg("async_finish"))
        .def("set_weight_sync_plan_mode", &Manager::set_weight_sync_plan_mode)
        .def("set_grad_reduce_deterministic", &Manager::set_grad_reduce_deterministic)
        .def("get_comm_stream", &Manager::get_comm_stream)
        .def("poll_status", &Manager::poll_status)
        .def("clear_status", &Manager::clear_status)
        .def("get_local_replica_weight_buffer_tensor", [](const Manager& s) { return s.buf(UEP_BUF_REPLICA_WEIGHT, torch::kUInt8); })
        .def("get_local_replica_fc1_weight_buffer_tensor", [](const Manager& s) { return s.buf(UEP_BUF_REPLICA_FC1_WEIGHT, torch::kUInt8); })
        .def("get_local_replica_fc2_weight_buffer_tensor", [](const Manager& s) { return s.buf(UEP_BUF_REPLICA_FC2_WEIGHT, torch::kUInt8); })
        .def("get_local_replica_weight_scale_buffer_tensor", [](const Manager& s) { return s.buf(UEP_BUF_REPLICA_SCALE, torch::kUInt8); })
        .def("get_local_replica_fc1_weight_scale_buffer_tensor", [](const Manager& s) { return s.buf(UEP_BUF_REPLICA_FC1_SCALE, torch::kUInt8); })
        .def("get_local_replica_fc2_weight_scale_buffer_tensor", [](const Manager& s) { return s.buf(UEP_BUF_REPLICA_FC2_SCALE, torch::kUInt8); })
        .def("get_local_replica_grad_buffer_tensor", [](const Manager& s) { return s.grad_buf(UEP_BUF_REPLICA_GRAD); })
        .def("get_local_replica_fc1_grad_buffer_tensor", [](const Manager& s) { return s.grad_buf(UEP_BUF_REPLICA_FC1_GRAD); })
        .def("get_local_replica_fc2_grad_buffer_tensor", [](const Manager& s) { return s.grad_buf(UEP_BUF_REPLICA_FC2_GRAD); })
        .def("get_physical_to_logical_map_tensor", [](const Manager& s) { return s.buf(UEP_BUF_P2L, torch::kInt32); })
        .def("get_logical_to_physical_map_tensor", [](const Manager& s) { return s.buf(UEP_BUF_L2P, torch::kInt32); })
        .def("get_logical_replica_counts_tensor", [](const Manager& s) { return s.buf(UEP_BUF_LCNTS, torch::kInt32); })
        .def("get_logical_instance_quota_tensor", [](const Manager& s) { return s.buf(UEP_BUF_QUOTA, torch::kInt32); })
        .def("get_logical_instance_quota_prefix_tensor", [](const Manager& s) { return s.buf(UEP_BUF_QUOTA_PREFIX, torch::kInt32); })
        .def("get_rank_quota_prefix_tensor", [](const Manager& s) { return s.buf(UEP_BUF_RANK_QUOTA_PREFIX, torch::kInt32); })
        .def("get_global_logical_expert_loads_tensor", [](const Manager& s) { return s.buf(UEP_BUF_GLOBAL_LOADS, torch::kInt32); })
        .def("get_expert_loads_per_rank_tensor", [](const Manager& s) { return s.buf(UEP_BUF_LOADS_PER_RANK, torch::kInt32); })
        .def("get_physical_expert_loads_tensor", [](const Manager& s) { return s.buf(UEP_BUF_PHYSICAL_LOADS, torch::kInt32); });

    m.def("solve_placement_for_test", &solve_placement_for_test, py::arg("expert_loads"), py::arg("expert_loads_per_rank"),
          py::arg("num_ranks"), py::arg("num_local_master_experts"), py::arg("num_local_redundant_experts"),
          py::arg("num_nvl_ranks"), py::arg("legacy_placement") = false, py::arg("balance_threshold") = 1.0f,
          py::arg("min_tokens_per_replica") = 1, py::arg("allow_zero_master_quota") = true,
          py::arg("locality_aware") = true, py::arg("oracle_eps") = 0.01f, py::arg("kernel_stage") = 1,
          py::arg("rank_quota_source_rank") = -1);
    m.def("dense_reroute_for_test", &dense_reroute_for_test, py::arg("routing_map"), py::arg("probs"),
          py::arg("logical_to_physical_map"), py::arg("logical_replica_counts"), py::arg("rank_quota_prefix"),
          py::arg("num_global_physical_experts"), py::arg("quota_reroute") = true,
          py::arg("interleave_by_rank_quota") = true);
}
