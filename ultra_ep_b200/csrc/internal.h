// Host-side declarations shared by the kernel translation units and the manager.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "../../include/uep_b200.h"
#include "common.cuh"

namespace uep {

constexpr int kMaxLocalRanks = 8;  // ranks one manager can host on one device (simulated EP)
constexpr int kMaxPeers = kMaxRanksPerDomain;
constexpr int kReduceSegments = 16;  // a replica's gradient is released for zeroing in this many pieces
constexpr unsigned long long kReduceFlagRadix = 64;  // progress word = epoch * radix + segments done

// Device-resident, per hosted rank, immutable after connect. Peer tables are indexed
// by global rank; entry [my_rank] is this rank's own buffer.
constexpr int kPlanMaxCtas = 32;  // CTAs of one rank in the plan kernel

struct RankDev {
    int my_rank;
    int num_ranks;
    // plan exchange
    uint64_t* hist_parts;    // [kPlanMaxCtas][Lpad] words, (epoch tag << 32) | partial count of one CTA of the plan kernel
    uint64_t* peer_gather[kMaxPeers];  // each: [2][N][Lpad] words, (epoch tag << 32) | token count
    int32_t* global_loads;   // [L]
    int32_t* loads_per_rank; // [N][L] latest gathered matrix (contiguous copy)
    // weight sync / grad reduce
    int* sync_ticket;        // zero between calls
    uint8_t* peer_replica_weight[kMaxPeers];
    uint8_t* peer_replica_scale[kMaxPeers];
    float* peer_replica_grad[kMaxPeers];
    uint64_t* peer_sync_flags[kMaxPeers];  // each: [N], entry [src] = last epoch src finished sending to that rank
    uint64_t* peer_relay_flags[kMaxPeers]; // each: [R][relay_cap], entry [slot][tile] = epoch in which the master delivered that tile
    uint64_t* peer_reduce_flags[kMaxPeers]; // each: [N], entry [src] = epoch * 64 + segments of its pulls master rank src has finished
    int* reduce_counters;    // [kReduceSegments]: CTAs of the running Wgrad reduce that have passed each segment; zero between calls
    DeviceStatus* status;    // mapped pinned host memory
    // [0] plan epoch, [1] sync epoch, [2] Wgrad-reduce epoch: counted on the device (by one CTA of every launch), not
    // passed by value, so that a captured CUDA graph can be replayed: every replay is a new epoch
    uint64_t* epochs;
};

struct PlanPtrs {
    int32_t *p2l, *l2p, *lcnts, *quota, *quota_prefix, *rank_quota_prefix;
    int32_t* physical_loads;  // [P] tokens per physical slot under this plan (may be null)
};

struct ShardLayout {  // bytes of the four weight shards and their place inside a replica slot
    int64_t bytes[4];        // fc1, fc2, fc1 scale, fc2 scale
    int64_t slot_offset[4];  // offset inside the weight slot (0,1) / scale slot (2,3)
    int64_t weight_slot_stride, scale_slot_stride;
    int num_shards;          // 2 or 4
};

// ---- launchers (defined in the .cu files; every launch bumps the launch counter) ----
void count_launch(int n = 1);

struct PlanCall {
    const RankDev* rank[kMaxLocalRanks];
    const void* input[kMaxLocalRanks];
    int T[kMaxLocalRanks];
    PlanPtrs plan[kMaxLocalRanks];
    int nlocal;
    int input_kind;  // 0 bool map, 1 ids32, 2 ids64
    int K_or_L;
    int N, G, M, R, D;
    uep_solver_params params;
    uint64_t timeout_ns;
    int ctas_per_rank;
    int withhold_rank;  // test hook: this rank does not publish its flags (-1: none)
    int legacy;         // 1: legacy placement solver (counts only; the reroute is then round-robin)
    unsigned long long* trace;  // optional: 8 globaltimer stamps per hosted rank (tuning aid), or null
};
cudaError_t launch_plan(const PlanCall& call, cudaStream_t stream);
int plan_ctas_per_rank(int input_kind, int max_T, int K_or_L, int nlocal, int num_sms);

struct SyncCall {
    const RankDev* rank[kMaxLocalRanks];
    int my_rank[kMaxLocalRanks];  // rank ids by value: one pointer hop less in every CTA's set-up
    PlanPtrs plan[kMaxLocalRanks];
    const int64_t* src_ptrs[kMaxLocalRanks][4];  // device int64[M] tables; scale tables may be null
    int nlocal;
    int N, M, R, D;
    ShardLayout shards;
    uint64_t timeout_ns;
    int ctas_per_rank;
    int withhold_rank;  // test hook, as in PlanCall
    int relay_min_replicas;  // 0: every master writes all its replicas itself; else experts with at least this many
                             // replicas are scattered over them and forwarded replica to replica
    int relay_adaptive;      // 1: also relay the experts of ranks that send more than any rank receives (see weight_sync.cu)
    int relay_cap;           // chunks per slot the ready-flag table has room for
    uint64_t* sync_epoch;    // the sync epoch counter of the first hosted rank (by value: one load, not two)
    unsigned long long* trace;  // optional: 8 globaltimer stamps per CTA (tuning aid), or null
};
cudaError_t launch_weight_sync(const SyncCall& call, cudaStream_t stream);
int weight_sync_max_ctas_per_rank(int nlocal, int num_sms);

struct ReduceCall {
    const RankDev* rank[kMaxLocalRanks];
    int my_rank[kMaxLocalRanks];
    PlanPtrs plan[kMaxLocalRanks];
    const int64_t* fc1_grad_ptrs[kMaxLocalRanks];
    const int64_t* fc2_grad_ptrs[kMaxLocalRanks];
    int nlocal;
    int N, M, R, D;
    int64_t fc1_numel, fc2_numel;
    uint64_t timeout_ns;
    int ctas_per_rank;
    uint64_t* reduce_epoch;     // the reduce epoch counter of the first hosted rank
    unsigned long long* trace;  // optional: 8 globaltimer stamps per CTA (tuning aid), or null
};
cudaError_t launch_grad_reduce(const ReduceCall& call, cudaStream_t stream);

// Reroute launchers. One launch serves every hosted rank (blockIdx.y selects the rank).
struct DenseFwdArgs {
    const uint8_t* map;
    const float* probs;
    const int32_t *l2p, *lcnts, *rqp;
    int32_t* scratch;  // [dense tiles][L]
    uint8_t* out_map;
    float* out_probs;
    int T;
};
struct DenseBwdArgs {
    const float* grad_expanded;
    const uint8_t *map, *expanded_map;
    const int32_t *l2p, *lcnts;
    float* grad_probs;
    int T;
};
struct SparseArgs {
    const void* ids;
    void* out;
    const int32_t *l2p, *lcnts, *rqp;
    int32_t* scratch;  // [sparse tiles][L]
    int T;
};
template <typename A>
struct Batch {
    A a[kMaxLocalRanks];
    int n;
};
int64_t dense_scratch_elems(int T, int L);
int64_t sparse_scratch_elems(int64_t entries, int L);
cudaError_t launch_dense_forward(const Batch<DenseFwdArgs>& b, int L, int P, int D, int quota_mode, int interleave,
                                 cudaStream_t stream);
cudaError_t launch_dense_backward(const Batch<DenseBwdArgs>& b, int L, int P, int D, cudaStream_t stream);
cudaError_t launch_sparse_reroute(const Batch<SparseArgs>& b, int ids_kind, int K, int L, int D, int interleave,
                                  cudaStream_t stream);

int device_sm_count();  // of the current device; launch sizes are multiples of it
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
int fail_cuda(cudaError_t e, const char* what);

}  // namespace uep

#define UEP_CUDA_TRY(expr)                                         \
    do {                                                           \
        cudaError_t _e = (expr);                                   \
        if (_e != cudaSuccess) return ::uep::fail_cuda(_e, #expr); \
    } while (0)
