// C entry points around the reference's own kernel launchers.
//
// THIS FILE IS TEST INFRASTRUCTURE. It is compiled together with the reference's
// unmodified kernel sources (csrc/kernels/{placement,reroute,load_compute,grad_reduce,
// weight_sync}.cu, read in place from the reference checkout, never copied) into
// oracle/_ref/libuep_ref.so. It adds nothing to the arithmetic: every function below
// forwards to a launcher declared in the reference's csrc/kernels/api.cuh. Used to
// (1) pin the CPU oracle and the new kernels against the real reference on a GPU and
// (2) time the reference's sm_100 build next to the new kernels.
//
// The reference's placement.cu expects two runtime globals (csrc/kernels/placement.cu:12-16);
// they are defined here so that the NVSHMEM-dependent runtime.cpp is not needed.

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

#include "kernels/api.cuh"
#include "utils/exception.cuh"

namespace ultra_ep::runtime {
bool is_runtime_initialized = false;
int rank_idx = 0;
}  // namespace ultra_ep::runtime

namespace {
thread_local std::string g_last_error;

template <typename Fn>
int guarded(Fn&& fn) {
    try {
        fn();
        return 0;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return -1;
    }
}

// Device-side scratch the reference Manager allocates per rank (csrc/ultra_ep.cpp:424-491).
struct RefWorkspace {
    ultra_ep::kernels::TaskBuildConfig config{};
    ultra_ep::kernels::TaskBuildConfig* d_config = nullptr;
    void** d_remote_weight_ptrs = nullptr;
    void** d_remote_scale_ptrs = nullptr;
    void** d_remote_grad_ptrs = nullptr;
    uint64_t** d_remote_flag_ptrs = nullptr;
    uint64_t* d_local_flags = nullptr;
    ultra_ep::kernels::GradReduceTask* d_grad_tasks = nullptr;
    ultra_ep::kernels::WeightSyncTask* d_ws_tasks = nullptr;
    ultra_ep::kernels::WeightSyncTask* d_relay_tasks = nullptr;
    int* d_ws_remaining = nullptr;
    int* d_tile_offsets = nullptr;
    int* d_relay_tile_offsets = nullptr;
    int* d_task_metadata = nullptr;
    int* d_relay_metadata = nullptr;
    int* d_counter = nullptr;
    int* d_relay_counter = nullptr;
    int ws_task_capacity = 0;
    int max_ws_total_tiles = 0;
    int num_sms = 0;
    uint64_t epoch = 0;
};

int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }
}  // namespace

extern "C" {

const char* uep_ref_last_error() { return g_last_error.c_str(); }

// csrc/kernels/api.cuh:17-38
int uep_ref_solve_placement(const int32_t* loads, const int32_t* loads_per_rank, int32_t* p2l, int32_t* l2p,
                            int32_t* lcnts, int32_t* quota, int32_t* quota_prefix, int32_t* rank_quota_prefix,
                            void* stream, int L, int num_ranks, int M, int R, int nvl_ranks, int D,
                            float balance_threshold, int32_t min_tokens, int allow_zero, int locality, float eps,
                            int kernel_stage, int source_rank) {
    return guarded([&] {
        ultra_ep::kernels::solve_placement(loads, loads_per_rank, p2l, l2p, lcnts, quota, quota_prefix,
                                           rank_quota_prefix, static_cast<cudaStream_t>(stream), L, num_ranks, M, R,
                                           nvl_ranks, D, balance_threshold, min_tokens, allow_zero != 0,
                                           locality != 0, eps, kernel_stage, source_rank);
    });
}

int uep_ref_rmap_local_sum(int T, int L, const bool* routing_map, int32_t* loads, void* stream) {
    return guarded([&] { ultra_ep::kernels::rmap_local_sum(T, L, routing_map, loads, static_cast<cudaStream_t>(stream)); });
}

int uep_ref_topk_local_sum(const int64_t* ids, int T, int K, int L, int32_t* loads, void* stream) {
    return guarded([&] { ultra_ep::kernels::topk_local_sum(ids, T, K, L, loads, static_cast<cudaStream_t>(stream)); });
}

int uep_ref_reduce_per_rank_loads(const int32_t* per_rank, int32_t* global_loads, int G, int L, void* stream) {
    return guarded([&] {
        ultra_ep::kernels::reduce_per_rank_loads(per_rank, global_loads, G, L, static_cast<cudaStream_t>(stream));
    });
}

// Outputs must be zero-filled by the caller, as csrc/ultra_ep.cpp:891-892 does.
int uep_ref_dense_reroute_forward_quota(const bool* routing_map, const float* probs, const int32_t* l2p,
                                        const int32_t* lcnts, const int32_t* rank_quota_prefix, bool* expanded_map,
                                        float* expanded_probs, int32_t* tile_counts, int T, int L, int P,
                                        int max_replicas, int interleave, void* stream) {
    return guarded([&] {
        ultra_ep::kernels::run_dense_reroute_forward_quota(routing_map, probs, l2p, lcnts, rank_quota_prefix,
                                                           expanded_map, expanded_probs, tile_counts, T, L, P,
                                                           max_replicas, interleave != 0,
                                                           static_cast<cudaStream_t>(stream));
    });
}

int uep_ref_dense_reroute_backward(const float* grad_expanded, const bool* routing_map, const bool* expanded_map,
                                   const int32_t* l2p, const int32_t* lcnts, float* grad_probs, int T, int L, int P,
                                   int max_replicas, void* stream) {
    return guarded([&] {
        ultra_ep::kernels::run_dense_reroute_backward(grad_expanded, routing_map, expanded_map, l2p, lcnts,
                                                      grad_probs, T, L, P, max_replicas,
                                                      static_cast<cudaStream_t>(stream));
    });
}

int uep_ref_sparse_reroute_quota(int64_t* ids, const int32_t* l2p, const int32_t* lcnts,
                                 const int32_t* rank_quota_prefix, int* counters, int T, int K, int L,
                                 int max_replicas, void* stream) {
    return guarded([&] {
        ultra_ep::kernels::run_sparse_reroute_quota(ids, l2p, lcnts, rank_quota_prefix, counters, T, K, L,
                                                    max_replicas, static_cast<cudaStream_t>(stream));
    });
}

// One rank's worth of the scratch that csrc/ultra_ep.cpp:424-498 allocates. The peer
// pointer tables are given as host arrays of device addresses (one per NVLink-domain
// rank; on one GPU every "peer" is a buffer on the same device).
void* uep_ref_workspace_create(int rank, int nvl_ranks, int M, int R, int64_t fc1_numel, int64_t fc2_numel,
                               int weight_elem_bytes, int scale_elem_bytes, int64_t fc1_scale_numel,
                               int64_t fc2_scale_numel, int max_replicas_dim, int plan_mode,
                               void* const* remote_weight_ptrs, void* const* remote_scale_ptrs,
                               void* const* remote_grad_ptrs) {
    using namespace ultra_ep::kernels;
    RefWorkspace* ws = new RefWorkspace();
    const int rc = guarded([&] {
        TaskBuildConfig& c = ws->config;
        c.rank_idx = rank;
        c.nvl_rank_idx = rank % nvl_ranks;
        c.num_nvl_ranks = nvl_ranks;
        c.num_local_master_experts = M;
        c.num_local_physical_experts = M + R;
        c.num_local_redundant_experts = R;
        c.expert_fc1_numel = fc1_numel;
        c.expert_fc2_numel = fc2_numel;
        c.expert_total_numel = fc1_numel + fc2_numel;
        c.expert_fc1_weight_scale_numel = fc1_scale_numel;
        c.expert_fc2_weight_scale_numel = fc2_scale_numel;
        c.expert_weight_scale_total_numel = fc1_scale_numel + fc2_scale_numel;
        c.expert_fc1_weight_scale_bytes = fc1_scale_numel * scale_elem_bytes;
        c.expert_fc2_weight_scale_bytes = fc2_scale_numel * scale_elem_bytes;
        c.expert_weight_scale_fc2_offset_bytes = align_up(c.expert_fc1_weight_scale_bytes, 16);
        c.expert_weight_scale_stride_bytes =
            align_up(c.expert_weight_scale_fc2_offset_bytes + c.expert_fc2_weight_scale_bytes, 16);
        c.weight_data_element_bytes = weight_elem_bytes;
        c.weight_scale_element_bytes = scale_elem_bytes;
        c.max_replicas_dim = max_replicas_dim;
        c.weight_sync_plan_mode = plan_mode;
        c.weight_sync_relay_min_replicas = 4;
        c.weight_sync_relay_max_relays = 8;
        c.weight_sync_relay_min_fanout_gain = 2;

        const size_t shard_bytes[4] = {static_cast<size_t>(fc1_numel) * weight_elem_bytes,
                                       static_cast<size_t>(fc2_numel) * weight_elem_bytes,
                                       static_cast<size_t>(c.expert_fc1_weight_scale_bytes),
                                       static_cast<size_t>(c.expert_fc2_weight_scale_bytes)};
        int chunks = 0, tiles = 0, max_chunks = 0;
        for (size_t b : shard_bytes) {
            chunks += weight_sync_num_chunks(b);
            tiles += weight_sync_num_tiles(b);
            max_chunks = max_chunks > weight_sync_num_chunks(b) ? max_chunks : weight_sync_num_chunks(b);
        }
        ws->ws_task_capacity = (M + R) * chunks;
        ws->max_ws_total_tiles = (M + R) * tiles;
        const int shards = c.expert_weight_scale_total_numel > 0 ? 4 : 2;
        const int64_t flag_count = static_cast<int64_t>(R) * shards * max_chunks;

        cudaDeviceProp prop{};
        int dev = 0;
        CUDA_RUNTIME_CHECK(cudaGetDevice(&dev));
        CUDA_RUNTIME_CHECK(cudaGetDeviceProperties(&prop, dev));
        ws->num_sms = prop.multiProcessorCount;

        auto upload_table = [&](void*** dst, void* const* src) {
            CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(dst), kMaxNvlDomainSize * sizeof(void*)));
            void* host[kMaxNvlDomainSize] = {nullptr};
            if (src != nullptr) {
                for (int i = 0; i < nvl_ranks; ++i) host[i] = src[i];
            }
            CUDA_RUNTIME_CHECK(cudaMemcpy(*dst, host, sizeof(host), cudaMemcpyHostToDevice));
        };
        upload_table(&ws->d_remote_weight_ptrs, remote_weight_ptrs);
        upload_table(&ws->d_remote_scale_ptrs, remote_scale_ptrs);
        upload_table(&ws->d_remote_grad_ptrs, remote_grad_ptrs);

        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_local_flags),
                                      (flag_count > 0 ? flag_count : 1) * sizeof(uint64_t)));
        CUDA_RUNTIME_CHECK(cudaMemset(ws->d_local_flags, 0, (flag_count > 0 ? flag_count : 1) * sizeof(uint64_t)));
        {
            void* flag_table[kMaxNvlDomainSize] = {nullptr};
            for (int i = 0; i < nvl_ranks; ++i) flag_table[i] = ws->d_local_flags;  // direct mode never signals
            upload_table(reinterpret_cast<void***>(&ws->d_remote_flag_ptrs), flag_table);
        }
        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_config), sizeof(TaskBuildConfig)));
        CUDA_RUNTIME_CHECK(cudaMemcpy(ws->d_config, &ws->config, sizeof(TaskBuildConfig), cudaMemcpyHostToDevice));
        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_grad_tasks),
                                      kMaxGradReduceTaskCount * sizeof(GradReduceTask)));
        const int shared_cap = ws->ws_task_capacity > kMaxGradReduceTaskCount ? ws->ws_task_capacity
                                                                               : kMaxGradReduceTaskCount;
        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_tile_offsets), (shared_cap + 1) * sizeof(int)));
        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_ws_tasks),
                                      ws->ws_task_capacity * sizeof(WeightSyncTask)));
        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_relay_tasks),
                                      ws->ws_task_capacity * sizeof(WeightSyncTask)));
        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_ws_remaining),
                                      ws->ws_task_capacity * sizeof(int)));
        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_relay_tile_offsets),
                                      (ws->ws_task_capacity + 1) * sizeof(int)));
        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_task_metadata), 2 * sizeof(int)));
        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_relay_metadata), 2 * sizeof(int)));
        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_counter), sizeof(int)));
        CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&ws->d_relay_counter), sizeof(int)));
    });
    if (rc != 0) {
        delete ws;
        return nullptr;
    }
    return ws;
}

void uep_ref_workspace_destroy(void* handle) {
    RefWorkspace* ws = static_cast<RefWorkspace*>(handle);
    if (ws == nullptr) return;
    cudaFree(ws->d_config);
    cudaFree(ws->d_remote_weight_ptrs);
    cudaFree(ws->d_remote_scale_ptrs);
    cudaFree(ws->d_remote_grad_ptrs);
    cudaFree(ws->d_remote_flag_ptrs);
    cudaFree(ws->d_local_flags);
    cudaFree(ws->d_grad_tasks);
    cudaFree(ws->d_ws_tasks);
    cudaFree(ws->d_relay_tasks);
    cudaFree(ws->d_ws_remaining);
    cudaFree(ws->d_tile_offsets);
    cudaFree(ws->d_relay_tile_offsets);
    cudaFree(ws->d_task_metadata);
    cudaFree(ws->d_relay_metadata);
    cudaFree(ws->d_counter);
    cudaFree(ws->d_relay_counter);
    delete ws;
}

// The two launches of csrc/ultra_ep.cpp:1143-1179 (task build, then the stage-1 copy
// kernel; with an NVLink domain of at most 8 ranks that is weight_sync_thread_copy_kernel).
int uep_ref_weight_sync(void* handle, const int32_t* p2l, const int32_t* l2p, const int32_t* lcnts,
                        const int64_t* fc1_ptrs, const int64_t* fc2_ptrs, const int64_t* fc1_scale_ptrs,
                        const int64_t* fc2_scale_ptrs, uint8_t* local_replica_weight, uint8_t* local_replica_scale,
                        void* stream_) {
    RefWorkspace* ws = static_cast<RefWorkspace*>(handle);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    return guarded([&] {
        using namespace ultra_ep::kernels;
        build_weight_sync_task_lists(ws->d_config, p2l, l2p, lcnts, ws->d_remote_weight_ptrs,
                                     ws->d_remote_scale_ptrs, fc1_ptrs, fc2_ptrs, fc1_scale_ptrs, fc2_scale_ptrs,
                                     local_replica_weight, local_replica_scale, ws->d_ws_tasks, ws->d_tile_offsets,
                                     ws->d_task_metadata, ws->d_ws_remaining, ws->d_counter, ws->d_relay_tasks,
                                     ws->d_relay_tile_offsets, ws->d_relay_metadata, ws->d_relay_counter, stream);
        run_weight_sync(ws->d_ws_tasks, ws->d_tile_offsets, ws->d_task_metadata, ws->d_counter, ws->d_ws_remaining,
                        ws->d_local_flags, ws->d_remote_flag_ptrs, ++ws->epoch, stream, ws->num_sms,
                        ws->config.num_nvl_ranks, ws->max_ws_total_tiles, 2);
    });
}

// The two launches of csrc/ultra_ep.cpp:1064-1083.
int uep_ref_grad_reduce(void* handle, const int32_t* p2l, const int32_t* l2p, const int32_t* lcnts,
                        const int64_t* fc1_grad_ptrs, const int64_t* fc2_grad_ptrs, int num_sms, int deterministic,
                        void* stream_) {
    RefWorkspace* ws = static_cast<RefWorkspace*>(handle);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    return guarded([&] {
        using namespace ultra_ep::kernels;
        build_grad_reduce_tasks(ws->d_config, p2l, l2p, lcnts, ws->d_remote_grad_ptrs, fc1_grad_ptrs, fc2_grad_ptrs,
                                ws->d_grad_tasks, ws->d_tile_offsets, ws->d_task_metadata, ws->d_counter, stream);
        run_grad_reduce(ws->d_grad_tasks, ws->d_tile_offsets, ws->d_task_metadata, ws->d_counter, stream,
                        num_sms < ws->num_sms ? num_sms : ws->num_sms, deterministic != 0);
    });
}

}  // extern "C"
