// Host runtime behind the C ABI: the manager of one expert-parallel group.
//
// Takes the place of the reference's Manager / GlobalExpertPlacement / runtime globals
// (csrc/ultra_ep.cpp, csrc/ultra_ep.hpp, csrc/runtime.cpp of the reference) with two
// structural differences:
//   * peer-visible memory is ONE cudaMalloc arena per rank, exported as one cudaIpc handle
//     (the reference allocates several NVSHMEM symmetric buffers); the caller carries the
//     64-byte handles between processes, so this library has no transport of its own;
//   * a manager can host all ranks of a group on one device ("simulated EP"): the same
//     kernels then serve every rank in one launch, and the peers are plain device buffers.
// Per layer it issues one launch for the plan, one for weight_sync, two for reroute and
// one for the Wgrad reduce; the reference issues about twenty stream operations.

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "internal.h"

using namespace uep;

struct uep_event {
    cudaEvent_t ev = nullptr;
};

namespace {

struct ArenaLayout {
    size_t gather, sync_flags, reduce_flags, relay_flags, replica_weight, replica_scale, replica_grad, total;
};

struct RankHost {
    int rank = -1;
    uint8_t* arena = nullptr;                   // peer-visible
    void* peer_arena[kMaxPeers] = {nullptr};    // all ranks' arenas as seen from this rank
    bool peer_opened[kMaxPeers] = {false};      // mapped through cudaIpcOpenMemHandle
    int32_t* plan_blob = nullptr;               // [layers][stride]
    int32_t* rank_quota_prefix = nullptr;       // [layers][L][D]
    int32_t* physical_loads = nullptr;          // [layers][P]
    uint64_t* hist_parts = nullptr;             // [kPlanMaxCtas][Lpad]
    int* tickets = nullptr;                     // [4 + kReduceSegments]: spare, sync ticket, sync unit counter, spare, reduce segment counters
    uint64_t* epochs = nullptr;                 // [4]: plan epoch, sync epoch, reduce epoch (device-counted), spare
    int32_t* global_loads = nullptr;            // [L]
    int32_t* loads_per_rank = nullptr;          // [N][L]
    DeviceStatus* status_host = nullptr;        // mapped pinned
    DeviceStatus* status_dev = nullptr;
    RankDev* dev = nullptr;
    // reroute scratch (per-tile expert counts), one buffer per form so that a dense and a sparse
    // reroute of different layers never share one: [0] dense, [1] sparse
    int32_t* scratch[2] = {nullptr, nullptr};
    int64_t scratch_elems[2] = {0, 0};
};

}  // namespace

struct uep_manager {
    uep_config cfg{};
    int nlocal = 1;
    int device = 0;
    int num_sms = 0;
    int N = 0, G = 0, M = 0, R = 0, Lp = 0, L = 0, P = 0, D = 0, Lpad = 0;
    int64_t fc1_bytes = 0, fc2_bytes = 0, fc1_scale_bytes = 0, fc2_scale_bytes = 0;
    int64_t scale_fc2_offset = 0, scale_stride = 0, weight_stride = 0, total_numel = 0;
    int64_t layer_stride = 0;  // int32 elements per layer in plan_blob
    ArenaLayout arena{};
    std::vector<RankHost> ranks;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t order_event = nullptr;  // reusable event for stream-to-stream ordering
    std::vector<cudaEvent_t> plan_ready;
    std::vector<cudaStream_t> plan_stream;
    std::vector<char> plan_recorded;
    uint64_t timeout_ns = 0;
    bool connected = false;
    int grad_reduce_ctas = 42;
    int weight_sync_ctas = 0;
    int withhold_rank = -1;
    int relay_cap = 0;  // ready-flag words per replica slot
    unsigned long long* sync_trace = nullptr;  // UEP_SYNC_TRACE=1: per-CTA phase stamps of the last weight_sync
};

namespace {

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

PlanPtrs plan_ptrs(const uep_manager* m, const RankHost& r, int layer) {
    int32_t* base = r.plan_blob + static_cast<int64_t>(layer) * m->layer_stride;
    PlanPtrs p;
    p.p2l = base;
    p.l2p = base + m->P;
    p.lcnts = p.l2p + static_cast<int64_t>(m->L) * m->D;
    p.quota = p.lcnts + m->L;
    p.quota_prefix = p.quota + static_cast<int64_t>(m->L) * m->D;
    p.rank_quota_prefix = r.rank_quota_prefix + static_cast<int64_t>(layer) * m->L * m->D;
    p.physical_loads = r.physical_loads + static_cast<int64_t>(layer) * m->P;
    return p;
}

int plan_slot(const uep_manager* m, int layer) { return m->cfg.is_train ? layer : 0; }

int check_layer(const uep_manager* m, int layer, const char* what) {
    if (m == nullptr) return fail(UEP_ERR_INVALID, std::string(what) + ": null manager");
    if (!m->connected) return fail(UEP_ERR_STATE, std::string(what) + ": manager is not connected");
    if (layer < 0 || layer >= m->cfg.num_layers) return fail(UEP_ERR_INVALID, std::string(what) + ": layer_id out of range");
    return UEP_OK;
}

int wait_for_plan(uep_manager* m, int layer, cudaStream_t stream) {
    const int slot = plan_slot(m, layer);
    if (!m->plan_recorded[slot] || m->plan_stream[slot] == stream) return UEP_OK;
    UEP_CUDA_TRY(cudaStreamWaitEvent(stream, m->plan_ready[slot], 0));
    return UEP_OK;
}

int order_after(uep_manager* m, cudaStream_t later, cudaStream_t earlier) {
    if (later == earlier) return UEP_OK;
    UEP_CUDA_TRY(cudaEventRecord(m->order_event, earlier));
    UEP_CUDA_TRY(cudaStreamWaitEvent(later, m->order_event, 0));
    return UEP_OK;
}

// `which`: 0 dense, 1 sparse. With reroute_max_tokens set at creation the buffers already have their
// final size and this never allocates; otherwise a first call at a larger token count grows the buffer
// (cudaFree waits for the device, so no kernel can still be using the old one; not allowed while a
// stream is being captured: make a warm-up call at the largest size first).
int ensure_scratch(RankHost& r, int which, int64_t elems) {
    if (elems <= r.scratch_elems[which]) return UEP_OK;
    if (r.scratch[which] != nullptr) UEP_CUDA_TRY(cudaFree(r.scratch[which]));
    r.scratch[which] = nullptr;
    r.scratch_elems[which] = 0;
    const int64_t want = elems + elems / 4;
    UEP_CUDA_TRY(cudaMalloc(&r.scratch[which], sizeof(int32_t) * want));
    r.scratch_elems[which] = want;
    return UEP_OK;
}

int upload_rank_dev(uep_manager* m, RankHost& r) {
    RankDev d;
    std::memset(&d, 0, sizeof(d));
    d.my_rank = r.rank;
    d.num_ranks = m->N;
    d.hist_parts = r.hist_parts;
    d.sync_ticket = r.tickets + 1;
    d.reduce_counters = r.tickets + 4;
    d.epochs = r.epochs;
    d.global_loads = r.global_loads;
    d.loads_per_rank = r.loads_per_rank;
    d.status = r.status_dev;
    for (int p = 0; p < m->N; ++p) {
        uint8_t* base = static_cast<uint8_t*>(r.peer_arena[p]);
        if (base == nullptr) return fail(UEP_ERR_STATE, "connect: a peer arena is not mapped");
        d.peer_gather[p] = reinterpret_cast<uint64_t*>(base + m->arena.gather);
        d.peer_sync_flags[p] = reinterpret_cast<uint64_t*>(base + m->arena.sync_flags);
        d.peer_reduce_flags[p] = reinterpret_cast<uint64_t*>(base + m->arena.reduce_flags);
        d.peer_relay_flags[p] = reinterpret_cast<uint64_t*>(base + m->arena.relay_flags);
        d.peer_replica_weight[p] = base + m->arena.replica_weight;
        d.peer_replica_scale[p] = base + m->arena.replica_scale;
        d.peer_replica_grad[p] = reinterpret_cast<float*>(base + m->arena.replica_grad);
    }
    UEP_CUDA_TRY(cudaMemcpy(r.dev, &d, sizeof(d), cudaMemcpyHostToDevice));
    return UEP_OK;
}

void free_rank(RankHost& r, int my_rank_count) {
    (void)my_rank_count;
    for (int p = 0; p < kMaxPeers; ++p) {
        if (r.peer_opened[p] && r.peer_arena[p] != nullptr) cudaIpcCloseMemHandle(r.peer_arena[p]);
        r.peer_arena[p] = nullptr;
        r.peer_opened[p] = false;
    }
    cudaFree(r.arena);
    cudaFree(r.plan_blob);
    cudaFree(r.rank_quota_prefix);
    cudaFree(r.physical_loads);
    cudaFree(r.hist_parts);
    cudaFree(r.tickets);
    cudaFree(r.epochs);
    cudaFree(r.global_loads);
    cudaFree(r.loads_per_rank);
    cudaFree(r.dev);
    cudaFree(r.scratch[0]);
    cudaFree(r.scratch[1]);
    if (r.status_host != nullptr) cudaFreeHost(r.status_host);
    r = RankHost{};
}

int finish_sync_op(uep_manager* m, int async_finish, cudaStream_t current, uep_event** done_event) {
    if (async_finish) {
        if (done_event == nullptr) return fail(UEP_ERR_INVALID, "async_finish requires done_event");
        uep_event* ev = new uep_event();
        cudaError_t e = cudaEventCreateWithFlags(&ev->ev, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventRecord(ev->ev, m->comm_stream);
        if (e != cudaSuccess) {
            if (ev->ev) cudaEventDestroy(ev->ev);
            delete ev;
            return fail_cuda(e, "event for async_finish");
        }
        *done_event = ev;
    } else {
        if (done_event != nullptr) *done_event = nullptr;
        return order_after(m, current, m->comm_stream);
    }
    return UEP_OK;
}

int begin_comm_op(uep_manager* m, uep_event* wait_event, cudaStream_t current) {
    if (wait_event != nullptr) {
        UEP_CUDA_TRY(cudaStreamWaitEvent(m->comm_stream, wait_event->ev, 0));
        return UEP_OK;
    }
    return order_after(m, m->comm_stream, current);
}

}  // namespace

extern "C" {

int uep_manager_create(const uep_config* cfg, uep_manager** out) {
    if (cfg == nullptr || out == nullptr) return fail(UEP_ERR_INVALID, "manager_create: null argument");
    *out = nullptr;
    const int N = cfg->num_ranks, G = cfg->nvl_ranks, M = cfg->num_local_master_experts,
              R = cfg->num_local_redundant_experts;
    // the checks of the reference constructor (csrc/ultra_ep.cpp:259-287) and solver launcher
    if (N <= 0 || G <= 0 || N % G != 0) return fail(UEP_ERR_INVALID, "manager_create: num_ranks must be a positive multiple of nvl_ranks");
    if (M <= 0 || R < 0) return fail(UEP_ERR_INVALID, "manager_create: bad expert counts");
    if (G * M > kMaxExpertsPerDomain || G > kMaxRanksPerDomain || G * R > kMaxExportsPerDomain)
        return fail(UEP_ERR_INVALID, "manager_create: NVLink domain exceeds the static limits (512 experts, 72 ranks, 512 replicas)");
    if (N > kMaxPeers) return fail(UEP_ERR_UNSUPPORTED, "manager_create: more than 72 ranks in one group");
    if (N != G) return fail(UEP_ERR_UNSUPPORTED, "manager_create: groups spanning several NVLink domains are not supported (load all-gather uses peer memory)");
    if (cfg->num_layers <= 0) return fail(UEP_ERR_INVALID, "manager_create: num_layers must be positive");
    if (cfg->weight_data_element_bytes <= 0 || cfg->weight_scale_element_bytes <= 0) return fail(UEP_ERR_INVALID, "manager_create: element bytes must be positive");
    if (cfg->grad_element_bytes != 4) return fail(UEP_ERR_INVALID, "manager_create: only fp32 gradients are supported");
    if (cfg->expert_fc1_numel < 0 || cfg->expert_fc2_numel < 0 || cfg->expert_fc1_weight_scale_numel < 0 || cfg->expert_fc2_weight_scale_numel < 0)
        return fail(UEP_ERR_INVALID, "manager_create: negative numel");
    if (cfg->quota_kernel_stage != 0 && cfg->quota_kernel_stage != 1) return fail(UEP_ERR_INVALID, "manager_create: quota_kernel_stage supports only {0,1}");
    if (cfg->weight_sync_plan_mode < 0 || cfg->weight_sync_plan_mode > 2) return fail(UEP_ERR_INVALID, "manager_create: weight_sync_plan_mode must be 0, 1 or 2");
    if (cfg->weight_sync_relay_min_replicas < 0 || cfg->weight_sync_relay_max_relays < 1 || cfg->weight_sync_relay_min_fanout_gain < 0)
        return fail(UEP_ERR_INVALID, "manager_create: bad relay parameters");
    if (cfg->grad_reduce_num_sms <= 0 || cfg->grad_reduce_num_sms % 2 != 0) return fail(UEP_ERR_INVALID, "manager_create: grad_reduce_num_sms must be positive and even");
    if (cfg->reroute_max_tokens < 0 || cfg->reroute_max_topk < 0) return fail(UEP_ERR_INVALID, "manager_create: negative reroute bounds");
    const int64_t fc1B = cfg->expert_fc1_numel * cfg->weight_data_element_bytes;
    const int64_t fc2B = cfg->expert_fc2_numel * cfg->weight_data_element_bytes;
    if (fc1B % 16 != 0 || fc2B % 16 != 0) return fail(UEP_ERR_INVALID, "manager_create: weight shard bytes must be multiples of 16");
    int nlocal = 1;
    if (cfg->sim_ranks > 0) {
        if (cfg->sim_ranks != N) return fail(UEP_ERR_INVALID, "manager_create: sim_ranks must equal num_ranks");
        if (N > kMaxLocalRanks) return fail(UEP_ERR_UNSUPPORTED, "manager_create: at most 8 ranks can be hosted on one device");
        nlocal = N;
    } else if (cfg->rank < 0 || cfg->rank >= N) {
        return fail(UEP_ERR_INVALID, "manager_create: rank out of range");
    }

    uep_manager* m = new uep_manager();
    m->cfg = *cfg;
    m->nlocal = nlocal;
    m->N = N; m->G = G; m->M = M; m->R = R; m->Lp = M + R; m->L = N * M; m->P = N * (M + R); m->D = N;
    m->Lpad = (m->L + 3) / 4 * 4;
    m->fc1_bytes = fc1B;
    m->fc2_bytes = fc2B;
    m->weight_stride = fc1B + fc2B;
    m->fc1_scale_bytes = cfg->expert_fc1_weight_scale_numel * cfg->weight_scale_element_bytes;
    m->fc2_scale_bytes = cfg->expert_fc2_weight_scale_numel * cfg->weight_scale_element_bytes;
    m->scale_fc2_offset = align_up_i64(m->fc1_scale_bytes, 16);                      // csrc/ultra_ep.cpp:275-277
    m->scale_stride = align_up_i64(m->scale_fc2_offset + m->fc2_scale_bytes, 16);
    m->total_numel = cfg->expert_fc1_numel + cfg->expert_fc2_numel;
    const int64_t per_layer = static_cast<int64_t>(m->P) + 3LL * m->L * m->D + m->L;  // p2l | l2p | lcnts | quota | quota_prefix
    m->layer_stride = (per_layer * 4 + 255) / 256 * 256 / 4;                           // 256-byte aligned, csrc/ultra_ep.cpp:135
    m->timeout_ns = static_cast<uint64_t>(cfg->wait_timeout_ms > 0 ? cfg->wait_timeout_ms : 5000) * 1000000ull;

    auto bail = [&](int rc) {
        for (auto& r : m->ranks) free_rank(r, nlocal);
        if (m->comm_stream) cudaStreamDestroy(m->comm_stream);
        if (m->order_event) cudaEventDestroy(m->order_event);
        for (auto e : m->plan_ready) cudaEventDestroy(e);
        delete m;
        return rc;
    };
#define UEP_TRY_BAIL(expr)                                   \
    do {                                                     \
        cudaError_t _e = (expr);                             \
        if (_e != cudaSuccess) return bail(fail_cuda(_e, #expr)); \
    } while (0)

    UEP_TRY_BAIL(cudaGetDevice(&m->device));
    cudaDeviceProp prop{};
    UEP_TRY_BAIL(cudaGetDeviceProperties(&prop, m->device));
    m->num_sms = prop.multiProcessorCount;
    m->grad_reduce_ctas = std::min(cfg->grad_reduce_num_sms, m->num_sms);
    const int sync_cap = weight_sync_max_ctas_per_rank(nlocal, m->num_sms);
    m->weight_sync_ctas = cfg->weight_sync_num_sms > 0 ? std::min(cfg->weight_sync_num_sms, sync_cap)
                                                       : std::min(nlocal > 1 ? sync_cap : 64, sync_cap);

    // arena layout (identical on every rank, so offsets need not be exchanged)
    size_t off = 0;
    m->arena.gather = off;        off = align256(off + sizeof(uint64_t) * 2 * N * m->Lpad);
    m->arena.sync_flags = off;    off = align256(off + sizeof(uint64_t) * N);
    m->arena.reduce_flags = off;  off = align256(off + sizeof(uint64_t) * N);
    // ready flags of relayed tiles: one word per (replica slot, tile), sized for the smallest tile geometry
    m->relay_cap = 4;
    for (int64_t b : {m->fc1_bytes, m->fc2_bytes, m->fc1_scale_bytes, m->fc2_scale_bytes}) m->relay_cap += static_cast<int>((b + 8191) / 8192);
    m->arena.relay_flags = off;   off = align256(off + sizeof(uint64_t) * static_cast<size_t>(R) * m->relay_cap);
    m->arena.replica_weight = off; off = align256(off + static_cast<size_t>(R) * m->weight_stride);
    m->arena.replica_scale = off;  off = align256(off + static_cast<size_t>(R) * m->scale_stride);
    m->arena.replica_grad = off;
    if (cfg->is_train) off = align256(off + static_cast<size_t>(R) * m->total_numel * sizeof(float));
    m->arena.total = std::max<size_t>(off, 256);

    int prio_lo = 0, prio_hi = 0;
    UEP_TRY_BAIL(cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi));
    UEP_TRY_BAIL(cudaStreamCreateWithPriority(&m->comm_stream, cudaStreamNonBlocking, prio_hi));
    UEP_TRY_BAIL(cudaEventCreateWithFlags(&m->order_event, cudaEventDisableTiming));
    const int slots = cfg->is_train ? cfg->num_layers : 1;
    m->plan_ready.assign(slots, nullptr);
    m->plan_stream.assign(slots, nullptr);
    m->plan_recorded.assign(slots, 0);
    for (int i = 0; i < slots; ++i) UEP_TRY_BAIL(cudaEventCreateWithFlags(&m->plan_ready[i], cudaEventDisableTiming));

    m->ranks.resize(nlocal);
    for (int i = 0; i < nlocal; ++i) {
        RankHost& r = m->ranks[i];
        r.rank = nlocal > 1 ? i : cfg->rank;
        UEP_TRY_BAIL(cudaMalloc(&r.arena, m->arena.total));
        UEP_TRY_BAIL(cudaMemset(r.arena, 0, m->arena.total));  // flags at epoch 0, replica grads zero (csrc/ultra_ep.cpp:394)
        UEP_TRY_BAIL(cudaMalloc(&r.plan_blob, sizeof(int32_t) * m->layer_stride * cfg->num_layers));
        UEP_TRY_BAIL(cudaMemset(r.plan_blob, 0, sizeof(int32_t) * m->layer_stride * cfg->num_layers));
        UEP_TRY_BAIL(cudaMalloc(&r.rank_quota_prefix, sizeof(int32_t) * static_cast<size_t>(m->L) * m->D * cfg->num_layers));
        UEP_TRY_BAIL(cudaMalloc(&r.physical_loads, sizeof(int32_t) * static_cast<size_t>(m->P) * cfg->num_layers));
        UEP_TRY_BAIL(cudaMemset(r.physical_loads, 0, sizeof(int32_t) * static_cast<size_t>(m->P) * cfg->num_layers));
        UEP_TRY_BAIL(cudaMalloc(&r.hist_parts, sizeof(uint64_t) * kPlanMaxCtas * m->Lpad));
        UEP_TRY_BAIL(cudaMemset(r.hist_parts, 0, sizeof(uint64_t) * kPlanMaxCtas * m->Lpad));
        UEP_TRY_BAIL(cudaMalloc(&r.tickets, sizeof(int) * (4 + kReduceSegments)));
        UEP_TRY_BAIL(cudaMemset(r.tickets, 0, sizeof(int) * (4 + kReduceSegments)));
        UEP_TRY_BAIL(cudaMalloc(&r.epochs, sizeof(uint64_t) * 4));
        UEP_TRY_BAIL(cudaMemset(r.epochs, 0, sizeof(uint64_t) * 4));
        UEP_TRY_BAIL(cudaMalloc(&r.global_loads, sizeof(int32_t) * m->L));
        UEP_TRY_BAIL(cudaMemset(r.global_loads, 0, sizeof(int32_t) * m->L));
        UEP_TRY_BAIL(cudaMalloc(&r.loads_per_rank, sizeof(int32_t) * static_cast<size_t>(N) * m->L));
        UEP_TRY_BAIL(cudaMemset(r.loads_per_rank, 0, sizeof(int32_t) * static_cast<size_t>(N) * m->L));
        UEP_TRY_BAIL(cudaMalloc(&r.dev, sizeof(RankDev)));
        UEP_TRY_BAIL(cudaHostAlloc(&r.status_host, sizeof(DeviceStatus), cudaHostAllocMapped));
        r.status_host->code = 0;
        r.status_host->detail = 0;
        UEP_TRY_BAIL(cudaHostGetDevicePointer(reinterpret_cast<void**>(&r.status_dev), r.status_host, 0));
        if (cfg->reroute_max_tokens > 0) {  // final size now: no reroute call allocates or frees afterwards
            const int64_t topk_bound = cfg->reroute_max_topk > 0 ? cfg->reroute_max_topk : 8;
            if (ensure_scratch(r, 0, dense_scratch_elems(cfg->reroute_max_tokens, m->L)) != UEP_OK ||
                ensure_scratch(r, 1, sparse_scratch_elems(static_cast<int64_t>(cfg->reroute_max_tokens) * topk_bound, m->L)) != UEP_OK)
                return bail(UEP_ERR_CUDA);
        }
        // masters-only plan in every virtual layer (csrc/ultra_ep.cpp:511-527)
        for (int layer = 0; layer < cfg->num_layers; ++layer) {
            const PlanPtrs p = plan_ptrs(m, r, layer);
            const int rc = uep_init_master_placement(p.p2l, p.l2p, p.lcnts, p.quota, p.quota_prefix,
                                                     p.rank_quota_prefix, N, M, R, m->D, nullptr);
            if (rc != UEP_OK) return bail(rc);
        }
    }
    if (const char* tr = std::getenv("UEP_SYNC_TRACE")) {
        if (tr[0] == '1') {
            UEP_TRY_BAIL(cudaMalloc(&m->sync_trace, sizeof(unsigned long long) * 8 * 1024));
            UEP_TRY_BAIL(cudaMemset(m->sync_trace, 0, sizeof(unsigned long long) * 8 * 1024));
        }
    }
    UEP_TRY_BAIL(cudaDeviceSynchronize());
#undef UEP_TRY_BAIL
    *out = m;
    return UEP_OK;
}

int uep_manager_export_handle(uep_manager* m, void* handle_out) {
    if (m == nullptr || handle_out == nullptr) return fail(UEP_ERR_INVALID, "export_handle: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == UEP_IPC_HANDLE_BYTES, "cudaIpcMemHandle_t is 64 bytes");
    if (m->nlocal != 1) return fail(UEP_ERR_STATE, "export_handle: a simulated group has no peers to export to");
    cudaIpcMemHandle_t h;
    UEP_CUDA_TRY(cudaIpcGetMemHandle(&h, m->ranks[0].arena));
    std::memcpy(handle_out, &h, sizeof(h));
    return UEP_OK;
}

int uep_manager_connect(uep_manager* m, const void* all_handles) {
    if (m == nullptr) return fail(UEP_ERR_INVALID, "connect: null manager");
    if (m->connected) return fail(UEP_ERR_STATE, "connect: already connected");
    if (m->nlocal > 1) {
        for (auto& r : m->ranks) {
            for (int p = 0; p < m->N; ++p) r.peer_arena[p] = m->ranks[p].arena;
            const int rc = upload_rank_dev(m, r);
            if (rc != UEP_OK) return rc;
        }
    } else {
        RankHost& r = m->ranks[0];
        if (all_handles == nullptr && m->N > 1) return fail(UEP_ERR_INVALID, "connect: handles required");
        for (int p = 0; p < m->N; ++p) {
            if (p == r.rank) {
                r.peer_arena[p] = r.arena;
                continue;
            }
            cudaIpcMemHandle_t h;
            std::memcpy(&h, static_cast<const uint8_t*>(all_handles) + static_cast<size_t>(p) * UEP_IPC_HANDLE_BYTES, sizeof(h));
            void* ptr = nullptr;
            cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) return fail_cuda(e, "cudaIpcOpenMemHandle (is the peer in the same NVLink domain?)");
            r.peer_arena[p] = ptr;
            r.peer_opened[p] = true;
        }
        const int rc = upload_rank_dev(m, r);
        if (rc != UEP_OK) return rc;
    }
    UEP_CUDA_TRY(cudaDeviceSynchronize());
    m->connected = true;
    return UEP_OK;
}

int uep_manager_destroy(uep_manager* m) {
    if (m == nullptr) return UEP_OK;
    cudaDeviceSynchronize();
    for (auto& r : m->ranks) free_rank(r, m->nlocal);
    if (m->comm_stream) cudaStreamDestroy(m->comm_stream);
    if (m->order_event) cudaEventDestroy(m->order_event);
    for (auto e : m->plan_ready) cudaEventDestroy(e);
    cudaFree(m->sync_trace);
    delete m;
    return UEP_OK;
}

int uep_manager_num_local(const uep_manager* m) { return m ? m->nlocal : 0; }
int uep_manager_num_sms(const uep_manager* m) { return m ? m->num_sms : 0; }
void* uep_manager_comm_stream(uep_manager* m) { return m ? m->comm_stream : nullptr; }

int uep_manager_buffer(uep_manager* m, int local_rank, int buffer_id, void** ptr, int* ndim, int64_t shape[3],
                       int64_t stride[3]) {
    if (m == nullptr || ptr == nullptr || ndim == nullptr || shape == nullptr || stride == nullptr)
        return fail(UEP_ERR_INVALID, "manager_buffer: null argument");
    if (local_rank < 0 || local_rank >= m->nlocal) return fail(UEP_ERR_INVALID, "manager_buffer: local_rank out of range");
    RankHost& r = m->ranks[local_rank];
    const int64_t layers = m->cfg.num_layers, L = m->L, P = m->P, D = m->D, R = m->R;
    int32_t* blob = r.plan_blob;
    auto set = [&](void* p, int nd, int64_t s0, int64_t s1, int64_t s2, int64_t t0, int64_t t1, int64_t t2) {
        *ptr = p; *ndim = nd;
        shape[0] = s0; shape[1] = s1; shape[2] = s2;
        stride[0] = t0; stride[1] = t1; stride[2] = t2;
    };
    uint8_t* w = r.arena + m->arena.replica_weight;
    uint8_t* sc = r.arena + m->arena.replica_scale;
    float* g = reinterpret_cast<float*>(r.arena + m->arena.replica_grad);
    const bool has_scale = (m->fc1_scale_bytes + m->fc2_scale_bytes) > 0;
    switch (buffer_id) {
        case UEP_BUF_P2L: set(blob, 2, layers, P, 1, m->layer_stride, 1, 1); break;
        case UEP_BUF_L2P: set(blob + P, 3, layers, L, D, m->layer_stride, D, 1); break;
        case UEP_BUF_LCNTS: set(blob + P + L * D, 2, layers, L, 1, m->layer_stride, 1, 1); break;
        case UEP_BUF_QUOTA: set(blob + P + L * D + L, 3, layers, L, D, m->layer_stride, D, 1); break;
        case UEP_BUF_QUOTA_PREFIX: set(blob + P + 2 * L * D + L, 3, layers, L, D, m->layer_stride, D, 1); break;
        case UEP_BUF_RANK_QUOTA_PREFIX: set(r.rank_quota_prefix, 3, layers, L, D, L * D, D, 1); break;
        case UEP_BUF_PHYSICAL_LOADS: set(r.physical_loads, 2, layers, P, 1, P, 1, 1); break;
        case UEP_BUF_GLOBAL_LOADS: set(r.global_loads, 1, L, 1, 1, 1, 1, 1); break;
        case UEP_BUF_LOADS_PER_RANK: set(r.loads_per_rank, 2, m->N, L, 1, L, 1, 1); break;
        case UEP_BUF_REPLICA_WEIGHT: set(w, 2, R, m->weight_stride, 1, m->weight_stride, 1, 1); break;
        case UEP_BUF_REPLICA_FC1_WEIGHT: set(w, 2, R, m->fc1_bytes, 1, m->weight_stride, 1, 1); break;
        case UEP_BUF_REPLICA_FC2_WEIGHT: set(w + m->fc1_bytes, 2, R, m->fc2_bytes, 1, m->weight_stride, 1, 1); break;
        case UEP_BUF_REPLICA_SCALE: set(sc, 2, R, has_scale ? m->scale_stride : 0, 1, m->scale_stride, 1, 1); break;
        case UEP_BUF_REPLICA_FC1_SCALE: set(sc, 2, R, m->fc1_scale_bytes, 1, m->scale_stride, 1, 1); break;
        case UEP_BUF_REPLICA_FC2_SCALE: set(sc + m->scale_fc2_offset, 2, R, m->fc2_scale_bytes, 1, m->scale_stride, 1, 1); break;
        case UEP_BUF_REPLICA_GRAD:
        case UEP_BUF_REPLICA_FC1_GRAD:
        case UEP_BUF_REPLICA_FC2_GRAD:
            if (!m->cfg.is_train) return fail(UEP_ERR_STATE, "Grad buffer not available in inference mode");
            if (buffer_id == UEP_BUF_REPLICA_GRAD) set(g, 2, R, m->total_numel, 1, m->total_numel, 1, 1);
            else if (buffer_id == UEP_BUF_REPLICA_FC1_GRAD) set(g, 2, R, m->cfg.expert_fc1_numel, 1, m->total_numel, 1, 1);
            else set(g + m->cfg.expert_fc1_numel, 2, R, m->cfg.expert_fc2_numel, 1, m->total_numel, 1, 1);
            break;
        default: return fail(UEP_ERR_INVALID, "manager_buffer: unknown buffer id");
    }
    return UEP_OK;
}

int uep_manager_peer_buffer(uep_manager* m, int local_rank, int peer_rank, int buffer_id, void** ptr) {
    if (m == nullptr || ptr == nullptr) return fail(UEP_ERR_INVALID, "manager_peer_buffer: null argument");
    if (!m->connected) return fail(UEP_ERR_STATE, "manager_peer_buffer: manager is not connected");
    if (local_rank < 0 || local_rank >= m->nlocal || peer_rank < 0 || peer_rank >= m->N)
        return fail(UEP_ERR_INVALID, "manager_peer_buffer: rank out of range");
    uint8_t* base = static_cast<uint8_t*>(m->ranks[local_rank].peer_arena[peer_rank]);
    switch (buffer_id) {
        case UEP_BUF_REPLICA_WEIGHT: *ptr = base + m->arena.replica_weight; break;
        case UEP_BUF_REPLICA_SCALE: *ptr = base + m->arena.replica_scale; break;
        case UEP_BUF_REPLICA_GRAD:
            if (!m->cfg.is_train) return fail(UEP_ERR_STATE, "Grad buffer not available in inference mode");
            *ptr = base + m->arena.replica_grad;
            break;
        default: return fail(UEP_ERR_INVALID, "manager_peer_buffer: only the replica weight, scale and grad buffers are peer-visible");
    }
    return UEP_OK;
}

namespace {
// One-directional copy for the link probe: plain 16-byte loads and streaming stores, enough CTAs to fill the link.
__global__ void __launch_bounds__(256) probe_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int64_t nvec) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
        const uint4 a = ld_global_nc_v4(src + i), b = ld_global_nc_v4(src + i + stride);
        const uint4 c = ld_global_nc_v4(src + i + 2 * stride), d = ld_global_nc_v4(src + i + 3 * stride);
        st_global_cs_v4(dst + i, a);
        st_global_cs_v4(dst + i + stride, b);
        st_global_cs_v4(dst + i + 2 * stride, c);
        st_global_cs_v4(dst + i + 3 * stride, d);
    }
    for (; i < nvec; i += stride) st_global_cs_v4(dst + i, ld_global_nc_v4(src + i));
}
}  // namespace

int uep_debug_link_probe(uep_manager* m, int peer_rank, int64_t bytes, int iters, int use_kernel, float* ms_out) {
    if (m == nullptr || ms_out == nullptr) return fail(UEP_ERR_INVALID, "link_probe: null argument");
    if (!m->connected || m->nlocal != 1) return fail(UEP_ERR_STATE, "link_probe: needs a connected one-rank-per-process manager");
    if (peer_rank < 0 || peer_rank >= m->N || peer_rank == m->ranks[0].rank) return fail(UEP_ERR_INVALID, "link_probe: peer must be another rank");
    const int64_t region = static_cast<int64_t>(m->R) * m->weight_stride;
    if (bytes <= 0 || bytes > region || bytes % 16 != 0 || iters <= 0) return fail(UEP_ERR_INVALID, "link_probe: bytes must be a positive multiple of 16 within the replica weight buffer");
    RankHost& r = m->ranks[0];
    // use_kernel bit 1: the other direction (this rank READS the peer's buffer into its own)
    const bool pull = (use_kernel & 2) != 0;
    use_kernel &= 1;
    uint8_t* local = r.arena + m->arena.replica_weight;
    uint8_t* remote = static_cast<uint8_t*>(r.peer_arena[peer_rank]) + m->arena.replica_weight;
    const uint8_t* src = pull ? remote : local;
    uint8_t* dst = pull ? local : remote;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    UEP_CUDA_TRY(cudaEventCreate(&e0));
    UEP_CUDA_TRY(cudaEventCreate(&e1));
    cudaStream_t st = m->comm_stream;
    auto once = [&]() -> cudaError_t {
        if (!use_kernel) return cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice, st);
        probe_copy_kernel<<<m->num_sms * 8, 256, 0, st>>>(reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), bytes / 16);
        return cudaGetLastError();
    };
    cudaError_t e = once();  // warm-up
    if (e == cudaSuccess) e = cudaEventRecord(e0, st);
    for (int i = 0; i < iters && e == cudaSuccess; ++i) e = once();
    if (e == cudaSuccess) e = cudaEventRecord(e1, st);
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess) return fail_cuda(e, "link_probe");
    *ms_out = ms / static_cast<float>(iters);
    return UEP_OK;
}

int uep_update_placement(uep_manager* m, int layer_id, int input_kind, const void* const* inputs, const int* T,
                         int K_or_L, void* stream_) {
    int rc = check_layer(m, layer_id, "update_placement");
    if (rc != UEP_OK) return rc;
    if (input_kind < 0 || input_kind > 2 || inputs == nullptr || T == nullptr) return fail(UEP_ERR_INVALID, "update_placement: bad input description");
    if (input_kind == 0 && K_or_L != m->L) return fail(UEP_ERR_INVALID, "update_placement: routing_map must have one column per logical expert");
    if (input_kind != 0 && K_or_L < 0) return fail(UEP_ERR_INVALID, "update_placement: negative top-k");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PlanCall call;
    std::memset(&call, 0, sizeof(call));
    int max_T = 0;
    for (int i = 0; i < m->nlocal; ++i) {
        if (T[i] < 0) return fail(UEP_ERR_INVALID, "update_placement: negative token count");
        if (T[i] > 0 && K_or_L > 0 && inputs[i] == nullptr) return fail(UEP_ERR_INVALID, "update_placement: null input");
        call.rank[i] = m->ranks[i].dev;
        call.input[i] = inputs[i];
        call.T[i] = T[i];
        call.plan[i] = plan_ptrs(m, m->ranks[i], layer_id);
        max_T = std::max(max_T, T[i]);
    }
    call.nlocal = m->nlocal;
    call.input_kind = input_kind;
    call.K_or_L = K_or_L;
    call.N = m->N; call.G = m->G; call.M = m->M; call.R = m->R; call.D = m->D;
    call.params = m->cfg.solver;
    call.timeout_ns = m->timeout_ns;
    call.ctas_per_rank = plan_ctas_per_rank(input_kind, max_T, K_or_L, m->nlocal, m->num_sms);
    call.withhold_rank = m->withhold_rank;
    call.legacy = m->cfg.legacy_placement ? 1 : 0;
    call.trace = m->sync_trace ? m->sync_trace + 8 * 1000 : nullptr;  // the last rows of the trace buffer
    UEP_CUDA_TRY(launch_plan(call, stream));
    const int slot = plan_slot(m, layer_id);
    UEP_CUDA_TRY(cudaEventRecord(m->plan_ready[slot], stream));
    m->plan_stream[slot] = stream;
    m->plan_recorded[slot] = 1;
    return UEP_OK;
}

int uep_weight_sync(uep_manager* m, int layer_id, const int64_t* const* fc1_ptrs, const int64_t* const* fc2_ptrs,
                    const int64_t* const* fc1_scale_ptrs, const int64_t* const* fc2_scale_ptrs,
                    uep_event* wait_event, int async_finish, void* current_stream, uep_event** done_event) {
    int rc = check_layer(m, layer_id, "weight_sync");
    if (rc != UEP_OK) return rc;
    if (fc1_ptrs == nullptr || fc2_ptrs == nullptr) return fail(UEP_ERR_INVALID, "weight_sync: null pointer tables");
    const bool has_scale = (m->fc1_scale_bytes + m->fc2_scale_bytes) > 0;
    if (has_scale && (fc1_scale_ptrs == nullptr || fc2_scale_ptrs == nullptr))
        return fail(UEP_ERR_INVALID, "weight_sync: scale pointer tables are required when scale numel is non-zero");
    cudaStream_t current = static_cast<cudaStream_t>(current_stream);
    rc = begin_comm_op(m, wait_event, current);
    if (rc != UEP_OK) return rc;
    // the plan was produced on `current` in the common case: the wait above already covers it
    if (!(wait_event == nullptr && m->plan_stream[plan_slot(m, layer_id)] == current)) {
        rc = wait_for_plan(m, layer_id, m->comm_stream);
        if (rc != UEP_OK) return rc;
    }

    SyncCall call;
    std::memset(&call, 0, sizeof(call));
    for (int i = 0; i < m->nlocal; ++i) {
        if (fc1_ptrs[i] == nullptr || fc2_ptrs[i] == nullptr) return fail(UEP_ERR_INVALID, "weight_sync: null pointer table");
        call.rank[i] = m->ranks[i].dev;
        call.my_rank[i] = m->ranks[i].rank;
        call.plan[i] = plan_ptrs(m, m->ranks[i], layer_id);
        call.src_ptrs[i][0] = fc1_ptrs[i];
        call.src_ptrs[i][1] = fc2_ptrs[i];
        call.src_ptrs[i][2] = has_scale ? fc1_scale_ptrs[i] : nullptr;
        call.src_ptrs[i][3] = has_scale ? fc2_scale_ptrs[i] : nullptr;
        if (has_scale && (call.src_ptrs[i][2] == nullptr || call.src_ptrs[i][3] == nullptr))
            return fail(UEP_ERR_INVALID, "weight_sync: null scale pointer table");
    }
    call.nlocal = m->nlocal;
    call.N = m->N; call.M = m->M; call.R = m->R; call.D = m->D;
    ShardLayout& sh = call.shards;
    sh.num_shards = has_scale ? 4 : 2;
    sh.bytes[0] = m->fc1_bytes; sh.bytes[1] = m->fc2_bytes; sh.bytes[2] = m->fc1_scale_bytes; sh.bytes[3] = m->fc2_scale_bytes;
    sh.slot_offset[0] = 0; sh.slot_offset[1] = m->fc1_bytes; sh.slot_offset[2] = 0; sh.slot_offset[3] = m->scale_fc2_offset;
    sh.weight_slot_stride = m->weight_stride;
    sh.scale_slot_stride = m->scale_stride;
    call.timeout_ns = m->timeout_ns;
    call.ctas_per_rank = m->weight_sync_ctas;
    call.withhold_rank = m->withhold_rank;
    // plan mode 0: every master writes all its replicas; 1 (adaptive): experts with at least relay_min_replicas
    // replicas, and the experts of a rank whose outbound volume exceeds every rank's inbound volume, are scattered
    // over their replicas and forwarded replica to replica; 2: every expert with two or more replicas is
    const int mode = m->cfg.weight_sync_plan_mode;
    call.relay_min_replicas = mode == 0 ? 0 : (mode == 2 ? 2 : std::max(2, m->cfg.weight_sync_relay_min_replicas));
    call.relay_adaptive = mode == 1 ? 1 : 0;
    call.relay_cap = m->relay_cap;
    call.sync_epoch = m->ranks[0].epochs + 1;
    call.trace = m->sync_trace;
    if (m->R > 0) UEP_CUDA_TRY(launch_weight_sync(call, m->comm_stream));
    return finish_sync_op(m, async_finish, current, done_event);
}

int uep_grad_reduce(uep_manager* m, int layer_id, const int64_t* const* fc1_grad_ptrs,
                    const int64_t* const* fc2_grad_ptrs, uep_event* wait_event, int async_finish,
                    void* current_stream, uep_event** done_event) {
    int rc = check_layer(m, layer_id, "grad_reduce");
    if (rc != UEP_OK) return rc;
    if (!m->cfg.is_train) return fail(UEP_ERR_STATE, "grad_reduce: manager was created for inference");
    if (fc1_grad_ptrs == nullptr || fc2_grad_ptrs == nullptr) return fail(UEP_ERR_INVALID, "grad_reduce: null pointer tables");
    cudaStream_t current = static_cast<cudaStream_t>(current_stream);
    rc = begin_comm_op(m, wait_event, current);
    if (rc != UEP_OK) return rc;
    if (!(wait_event == nullptr && m->plan_stream[plan_slot(m, layer_id)] == current)) {
        rc = wait_for_plan(m, layer_id, m->comm_stream);
        if (rc != UEP_OK) return rc;
    }
    ReduceCall call;
    std::memset(&call, 0, sizeof(call));
    for (int i = 0; i < m->nlocal; ++i) {
        if (fc1_grad_ptrs[i] == nullptr || fc2_grad_ptrs[i] == nullptr) return fail(UEP_ERR_INVALID, "grad_reduce: null pointer table");
        call.rank[i] = m->ranks[i].dev;
        call.my_rank[i] = m->ranks[i].rank;
        call.plan[i] = plan_ptrs(m, m->ranks[i], layer_id);
        call.fc1_grad_ptrs[i] = fc1_grad_ptrs[i];
        call.fc2_grad_ptrs[i] = fc2_grad_ptrs[i];
    }
    call.nlocal = m->nlocal;
    call.N = m->N; call.M = m->M; call.R = m->R; call.D = m->D;
    call.fc1_numel = m->cfg.expert_fc1_numel;
    call.fc2_numel = m->cfg.expert_fc2_numel;
    call.timeout_ns = m->timeout_ns;
    // one CTA per SM at most (128 KiB of shared memory each): hosted ranks share the device's SMs
    call.ctas_per_rank = std::max(1, std::min(m->grad_reduce_ctas, m->num_sms / m->nlocal));
    call.trace = m->sync_trace;
    call.reduce_epoch = m->ranks[0].epochs + 2;
    if (m->R > 0 && m->total_numel > 0) UEP_CUDA_TRY(launch_grad_reduce(call, m->comm_stream));
    return finish_sync_op(m, async_finish, current, done_event);
}

int uep_reroute_dense_forward(uep_manager* m, int layer_id, const uint8_t* const* routing_maps,
                              const float* const* probs, uint8_t* const* expanded_maps, float* const* expanded_probs,
                              const int* T, void* stream_) {
    int rc = check_layer(m, layer_id, "dense_reroute_forward");
    if (rc != UEP_OK) return rc;
    if (!routing_maps || !probs || !expanded_maps || !expanded_probs || !T) return fail(UEP_ERR_INVALID, "dense_reroute_forward: null argument");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    rc = wait_for_plan(m, layer_id, stream);
    if (rc != UEP_OK) return rc;
    Batch<DenseFwdArgs> b{};
    b.n = m->nlocal;
    for (int i = 0; i < m->nlocal; ++i) {
        if (T[i] < 0) return fail(UEP_ERR_INVALID, "dense_reroute_forward: negative token count");
        if (T[i] > 0 && (!routing_maps[i] || !probs[i] || !expanded_maps[i] || !expanded_probs[i]))
            return fail(UEP_ERR_INVALID, "dense_reroute_forward: null tensor");
        rc = ensure_scratch(m->ranks[i], 0, dense_scratch_elems(T[i], m->L));
        if (rc != UEP_OK) return rc;
        const PlanPtrs p = plan_ptrs(m, m->ranks[i], layer_id);
        b.a[i] = DenseFwdArgs{routing_maps[i], probs[i], p.l2p, p.lcnts, p.rank_quota_prefix, m->ranks[i].scratch[0],
                              expanded_maps[i], expanded_probs[i], T[i]};
    }
    // legacy placement has no quotas: its reroute is round-robin over an expert's instances
    UEP_CUDA_TRY(launch_dense_forward(b, m->L, m->P, m->D, m->cfg.legacy_placement ? 0 : 1, m->cfg.solver.reroute_interleave, stream));
    return UEP_OK;
}

int uep_reroute_dense_backward(uep_manager* m, int layer_id, const float* const* grad_expanded,
                               const uint8_t* const* routing_maps, const uint8_t* const* expanded_maps,
                               float* const* grad_probs, const int* T, int P, void* stream_) {
    int rc = check_layer(m, layer_id, "dense_reroute_backward");
    if (rc != UEP_OK) return rc;
    if (!grad_expanded || !routing_maps || !expanded_maps || !grad_probs || !T) return fail(UEP_ERR_INVALID, "dense_reroute_backward: null argument");
    if (P != m->P) return fail(UEP_ERR_INVALID, "dense_reroute_backward: grad_expanded must have one column per physical expert");
    Batch<DenseBwdArgs> b{};
    b.n = m->nlocal;
    for (int i = 0; i < m->nlocal; ++i) {
        if (T[i] < 0) return fail(UEP_ERR_INVALID, "dense_reroute_backward: negative token count");
        if (T[i] > 0 && (!grad_expanded[i] || !routing_maps[i] || !expanded_maps[i] || !grad_probs[i]))
            return fail(UEP_ERR_INVALID, "dense_reroute_backward: null tensor");
        const PlanPtrs p = plan_ptrs(m, m->ranks[i], layer_id);
        b.a[i] = DenseBwdArgs{grad_expanded[i], routing_maps[i], expanded_maps[i], p.l2p, p.lcnts, grad_probs[i], T[i]};
    }
    UEP_CUDA_TRY(launch_dense_backward(b, m->L, m->P, m->D, static_cast<cudaStream_t>(stream_)));
    return UEP_OK;
}

int uep_reroute_sparse(uep_manager* m, int layer_id, int ids_kind, const void* const* ids, void* const* out,
                       const int* T, int K, void* stream_) {
    int rc = check_layer(m, layer_id, "reroute_sparse");
    if (rc != UEP_OK) return rc;
    if ((ids_kind != 1 && ids_kind != 2) || !ids || !out || !T || K < 0) return fail(UEP_ERR_INVALID, "reroute_sparse: bad argument");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    rc = wait_for_plan(m, layer_id, stream);
    if (rc != UEP_OK) return rc;
    Batch<SparseArgs> b{};
    b.n = m->nlocal;
    for (int i = 0; i < m->nlocal; ++i) {
        if (T[i] < 0) return fail(UEP_ERR_INVALID, "reroute_sparse: negative token count");
        if (static_cast<int64_t>(T[i]) * K > 0 && (!ids[i] || !out[i])) return fail(UEP_ERR_INVALID, "reroute_sparse: null tensor");
        rc = ensure_scratch(m->ranks[i], 1, sparse_scratch_elems(static_cast<int64_t>(T[i]) * K, m->L));
        if (rc != UEP_OK) return rc;
        const PlanPtrs p = plan_ptrs(m, m->ranks[i], layer_id);
        b.a[i] = SparseArgs{ids[i], out[i], p.l2p, p.lcnts, p.rank_quota_prefix, m->ranks[i].scratch[1], T[i]};
    }
    UEP_CUDA_TRY(launch_sparse_reroute(b, ids_kind, K, m->L, m->D, m->cfg.legacy_placement ? 2 : m->cfg.solver.reroute_interleave, stream));
    return UEP_OK;
}

int uep_set_weight_sync_plan_mode(uep_manager* m, int plan_mode) {
    if (m == nullptr) return fail(UEP_ERR_INVALID, "set_weight_sync_plan_mode: null manager");
    if (plan_mode < 0 || plan_mode > 2) return fail(UEP_ERR_INVALID, "set_weight_sync_plan_mode: plan_mode must be 0, 1 or 2");
    UEP_CUDA_TRY(cudaDeviceSynchronize());  // as the reference does (csrc/ultra_ep.cpp:989)
    m->cfg.weight_sync_plan_mode = plan_mode;
    return UEP_OK;
}

int uep_set_grad_reduce_deterministic(uep_manager* m, int deterministic, int num_sms) {
    if (m == nullptr) return fail(UEP_ERR_INVALID, "set_grad_reduce_deterministic: null manager");
    if (num_sms <= 0 || num_sms % 2 != 0) return fail(UEP_ERR_INVALID, "grad_reduce_num_sms must be positive and even");
    m->cfg.grad_reduce_deterministic = deterministic;
    m->cfg.grad_reduce_num_sms = num_sms;
    m->grad_reduce_ctas = std::min(num_sms, m->num_sms);
    return UEP_OK;
}

int uep_event_record(void* stream, uep_event** out) {
    if (out == nullptr) return fail(UEP_ERR_INVALID, "event_record: null output");
    uep_event* ev = new uep_event();
    cudaError_t e = cudaEventCreateWithFlags(&ev->ev, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(ev->ev, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        if (ev->ev) cudaEventDestroy(ev->ev);
        delete ev;
        return fail_cuda(e, "event_record");
    }
    *out = ev;
    return UEP_OK;
}

int uep_event_stream_wait(uep_event* ev, void* stream) {
    if (ev == nullptr) return fail(UEP_ERR_INVALID, "event_stream_wait: null event");
    UEP_CUDA_TRY(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), ev->ev, 0));
    return UEP_OK;
}

int uep_event_synchronize(uep_event* ev) {
    if (ev == nullptr) return fail(UEP_ERR_INVALID, "event_synchronize: null event");
    UEP_CUDA_TRY(cudaEventSynchronize(ev->ev));
    return UEP_OK;
}

void uep_event_destroy(uep_event* ev) {
    if (ev == nullptr) return;
    if (ev->ev) cudaEventDestroy(ev->ev);
    delete ev;
}

int uep_poll_status(uep_manager* m, int local_rank, int* code, int* detail) {
    if (m == nullptr || local_rank < 0 || local_rank >= m->nlocal) return fail(UEP_ERR_INVALID, "poll_status: bad argument");
    const volatile DeviceStatus* st = m->ranks[local_rank].status_host;
    const int c = st->code, d = st->detail;
    if (code) *code = c;
    if (detail) *detail = d;
    if (c != 0) return fail(UEP_ERR_DEVICE, "device reported status " + std::to_string(c) + " (detail " + std::to_string(d) + ")");
    return UEP_OK;
}

int uep_debug_sync_trace(uep_manager* m, unsigned long long* host_out, int max_ctas) {
    if (m == nullptr || host_out == nullptr || max_ctas <= 0) return fail(UEP_ERR_INVALID, "debug_sync_trace: bad argument");
    if (m->sync_trace == nullptr) return fail(UEP_ERR_STATE, "debug_sync_trace: tracing is off (set UEP_SYNC_TRACE=1 before creating the manager)");
    const int n = max_ctas < 1024 ? max_ctas : 1024;
    UEP_CUDA_TRY(cudaMemcpy(host_out, m->sync_trace, sizeof(unsigned long long) * 8 * n, cudaMemcpyDeviceToHost));
    return UEP_OK;
}

int uep_debug_withhold_rank(uep_manager* m, int rank) {
    if (m == nullptr) return fail(UEP_ERR_INVALID, "debug_withhold_rank: null manager");
    m->withhold_rank = rank;
    return UEP_OK;
}

int uep_clear_status(uep_manager* m) {
    if (m == nullptr) return fail(UEP_ERR_INVALID, "clear_status: null manager");
    UEP_CUDA_TRY(cudaDeviceSynchronize());
    for (auto& r : m->ranks) {
        r.status_host->code = 0;
        r.status_host->detail = 0;
        // a timed-out plan may have left the exchange scratch half used: reset it
        UEP_CUDA_TRY(cudaMemset(r.hist_parts, 0, sizeof(uint64_t) * kPlanMaxCtas * m->Lpad));
        UEP_CUDA_TRY(cudaMemset(r.tickets, 0, sizeof(int) * (4 + kReduceSegments)));
    }
    return UEP_OK;
}

}  // extern "C"
