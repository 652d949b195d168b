/*
 * uep_b200 — C ABI of the B200-native expert-balancing hot path.
 *
 * Plain C: pointers, sizes and integer status codes only; no torch or C++ types.
 * Every entry point returns UEP_OK (0) or a negative uep_status; uep_last_error()
 * gives the message of the last failure on the calling thread. Streams and events
 * are passed as void* holding a cudaStream_t / an opaque uep_event.
 *
 * Two groups:
 *   (A) stateless kernel entry points: raw device pointers in, results out. These are
 *       what the reference's single-GPU test hooks bind to.
 *   (B) the manager: owns the plan storage, the peer-visible replica slots, streams
 *       and events; one per expert-parallel group. It hosts either ONE rank of a
 *       multi-process group (peer memory mapped through cudaIpc handles that the
 *       caller exchanges) or ALL ranks of a simulated group on one device.
 *
 * Each declaration names the reference interface it replaces (file:line, paths
 * relative to the reference project root).
 */
#ifndef UEP_B200_H
#define UEP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum uep_status {
    UEP_OK = 0,
    UEP_ERR_INVALID = -1,       /* bad argument / size outside the static limits   */
    UEP_ERR_CUDA = -2,          /* a CUDA runtime call failed                       */
    UEP_ERR_STATE = -3,         /* call not legal in the manager's current state    */
    UEP_ERR_UNSUPPORTED = -4,   /* feature outside the hot path (e.g. legacy mode)  */
    UEP_ERR_DEVICE = -5         /* a kernel reported an error (see uep_poll_status) */
} uep_status;

/* Device-side status word values (uep_poll_status). 0 means healthy. */
enum {
    UEP_DEV_OK = 0,
    UEP_DEV_TIMEOUT_GATHER = 1,     /* a peer's load row did not arrive in time       */
    UEP_DEV_TIMEOUT_SYNC = 2,       /* a peer's weight_sync completion flag timed out */
    UEP_DEV_TIMEOUT_COPY = 3,       /* an async bulk copy did not complete in time    */
    UEP_DEV_SOLVER_INFEASIBLE = 4,  /* final plan rebuild infeasible (cannot happen on valid loads) */
    UEP_DEV_BAD_PLAN = 5            /* plan entry outside its table                   */
};

const char* uep_last_error(void);
const char* uep_version(void);

/* Solver tunables. Defaults of the reference's environment layer
 * (ultra_ep/config.py:54-71): 1.0, 1, 1024, 0, 0.01, 1. */
typedef struct uep_solver_params {
    float balance_threshold;
    int32_t locality_aware;
    int32_t min_tokens_per_replica;
    int32_t allow_zero_master_quota;
    float oracle_eps;
    int32_t reroute_interleave;
} uep_solver_params;

/* ------------------------------------------------------------------------------------
 * (A) Stateless kernel entry points. All pointers are device pointers unless noted.
 * ------------------------------------------------------------------------------------ */

/* Per-expert token counts of one rank.
 * Replaces kernels::topk_local_sum (csrc/kernels/load_compute.cu:111-129; ids outside
 * [0,L) ignored) for int64 ids, adds the int32 form, and kernels::rmap_local_sum
 * (csrc/kernels/load_compute.cu:51-73) for the dense bool map. loads[L] is overwritten. */
int uep_histogram_ids32(const int32_t* ids, int64_t num_entries, int L, int32_t* loads, void* stream);
int uep_histogram_ids64(const int64_t* ids, int64_t num_entries, int L, int32_t* loads, void* stream);
int uep_histogram_map(const uint8_t* routing_map, int T, int L, int32_t* loads, void* stream);

/* Replication plan from per-rank loads.
 * Replaces kernels::reduce_per_rank_loads + kernels::solve_placement
 * (csrc/kernels/load_compute.cu:144-151, csrc/kernels/placement.cu:1561-1663) and the
 * test hook _C.solve_placement_for_test (csrc/ultra_ep.hpp:427-533).
 *   loads_per_rank [num_ranks, L] int32;  global_loads_out [L] int32 (required; receives the sum over ranks)
 *   p2l [P], l2p [L,D], lcnts [L], quota [L,D], quota_prefix [L,D], rank_quota_prefix [L,D]
 *   L = num_ranks*M, P = num_ranks*(M+R); D = max_replicas_dim (the reference uses num_ranks)
 *   my_rank selects whose rank_quota_prefix is produced.
 *   status: device int32[2] {code, detail}, zero-initialised by the caller, or NULL. */
int uep_solve_placement(const int32_t* loads_per_rank, int32_t* global_loads_out, int32_t* p2l, int32_t* l2p,
                        int32_t* lcnts, int32_t* quota, int32_t* quota_prefix, int32_t* rank_quota_prefix,
                        int num_ranks, int nvl_ranks, int M, int R, int D, const uep_solver_params* params,
                        int my_rank, int32_t* status, void* stream);

/* Plan of legacy_placement=True from the group's total loads [L]: p2l, l2p, lcnts; the quota tensors are zeroed
 * (the reroute of this mode is round-robin). Replaces kernels::legacy::solve_placement
 * (csrc/kernels/legacy/placement_cpu.cpp:17-241), which copies the loads to the host, synchronises the stream
 * and solves there; this one is a kernel with the same arithmetic (doubles) and tie-breaks. */
int uep_legacy_solve_placement(const int32_t* global_loads, int32_t* p2l, int32_t* l2p, int32_t* lcnts, int32_t* quota,
                               int32_t* quota_prefix, int32_t* rank_quota_prefix, int num_ranks, int nvl_ranks, int M,
                               int R, int D, float balance_threshold, int32_t* status, void* stream);

/* Masters-only plan. Replaces kernels::init_master_placement (csrc/kernels/placement.cu:1504-1559). */
int uep_init_master_placement(int32_t* p2l, int32_t* l2p, int32_t* lcnts, int32_t* quota, int32_t* quota_prefix,
                              int32_t* rank_quota_prefix, int num_ranks, int M, int R, int D, void* stream);

/* Scratch the reroute entry points need: int32 elements. */
int64_t uep_reroute_scratch_elems(int64_t T, int K_or_0, int L);

/* Dense logical->physical expansion. Replaces kernels::run_dense_reroute_forward_quota
 * (csrc/kernels/reroute.cu:346-389) and _C.dense_reroute_for_test (csrc/ultra_ep.hpp:535-612).
 * expanded_map [T,P] and expanded_probs [T,P] are written completely (no pre-zeroing needed).
 * quota_mode 0 selects the round-robin rule of run_dense_reroute_forward_round_robin (:303-344). */
int uep_dense_reroute_forward(const uint8_t* routing_map, const float* probs, const int32_t* l2p,
                              const int32_t* lcnts, const int32_t* rank_quota_prefix, uint8_t* expanded_map,
                              float* expanded_probs, int32_t* scratch, int T, int L, int P, int D, int quota_mode,
                              int interleave, void* stream);

/* grad_probs [T,L] written completely. Replaces kernels::run_dense_reroute_backward
 * (csrc/kernels/reroute.cu:391-423). */
int uep_dense_reroute_backward(const float* grad_expanded, const uint8_t* routing_map, const uint8_t* expanded_map,
                               const int32_t* l2p, const int32_t* lcnts, float* grad_probs, int T, int L, int P, int D,
                               void* stream);

/* Sparse ids [T,K] logical -> physical, deterministic: the ordinal of an entry is its
 * row-major position among the entries naming the same expert (the dense rule applied per
 * (t,k)). out may alias ids (in place, as kernels::run_sparse_reroute_quota,
 * csrc/kernels/reroute.cu:547-577, which this replaces for int64 ids). */
int uep_sparse_reroute_i32(const int32_t* ids, int32_t* out, int T, int K, int L, const int32_t* l2p,
                           const int32_t* lcnts, const int32_t* rank_quota_prefix, int D, int interleave,
                           int32_t* scratch, void* stream);
int uep_sparse_reroute_i64(const int64_t* ids, int64_t* out, int T, int K, int L, const int32_t* l2p,
                           const int32_t* lcnts, const int32_t* rank_quota_prefix, int D, int interleave,
                           int32_t* scratch, void* stream);

/* Same result as uep_sparse_reroute_i32 for callers that cannot allocate device memory where
 * routing happens (a server whose memory pool owns the whole device, a frozen-allocator region,
 * a plugin boundary that only forwards its tensors): the scratch lives in a fixed 1 MiB array
 * inside the library image, so only inputs and outputs are passed and no allocation call of any
 * kind is made. Refused with UEP_ERR_INVALID when ceil(T*K/2048)*L + 4 exceeds 262144 int32.
 * All calls on a device share the array: calls that may overlap on the GPU must be ordered by
 * the caller. The first call on a device looks up the array's device address; make it before
 * any stream capture. This entry point has no counterpart in the reference. */
int uep_sparse_reroute_i32_static(const int32_t* ids, int32_t* out, int T, int K, int L, const int32_t* l2p,
                                  const int32_t* lcnts, const int32_t* rank_quota_prefix, int D, int interleave,
                                  void* stream);

/* Row order of the (token,k) entries once grouped by physical expert (stable), and the
 * per-expert row offsets [P+1]. No counterpart in the reference (its dispatcher is external). */
int uep_dispatch_positions(const int32_t* phys_ids, int64_t num_entries, int P, int32_t* pos,
                           int32_t* expert_offsets, int32_t* scratch, void* stream);
int64_t uep_dispatch_scratch_elems(int64_t num_entries, int P);

/* out[i,:] = in[pos[i],:] for rows of row_bytes bytes: the backward gather of token
 * gradients from physical-expert order back to (token,k) order. `in` has num_src_rows rows;
 * an index outside it is clamped to row 0 and recorded in status (device int32[2] or NULL).
 * No counterpart in the reference. */
int uep_gather_rows(const void* in, const int32_t* pos, void* out, int64_t num_rows, int64_t num_src_rows,
                    int64_t row_bytes, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------
 * (B) Manager
 * ------------------------------------------------------------------------------------ */
typedef struct uep_manager uep_manager;
typedef struct uep_event uep_event;

/* Mirrors the constructor of the reference's _C.Manager (csrc/ultra_ep.hpp:212-237) plus
 * the runtime facts the reference keeps in process globals (csrc/runtime.cpp:10-14). */
typedef struct uep_config {
    int32_t num_ranks;       /* EP size N                                                    */
    int32_t nvl_ranks;       /* NVLink-domain size G (N % G == 0)                            */
    int32_t rank;            /* this process's rank; ignored when sim_ranks > 0              */
    int32_t sim_ranks;       /* 0: one rank per process. N: host all N ranks on this device  */
    int32_t num_layers;      /* virtual layers ((real+3)*max_microbatches in the reference)  */
    int32_t num_local_master_experts;
    int32_t num_local_redundant_experts;
    int64_t expert_fc1_numel, expert_fc2_numel;
    int32_t weight_data_element_bytes, weight_scale_element_bytes;
    int64_t expert_fc1_weight_scale_numel, expert_fc2_weight_scale_numel;
    int32_t grad_element_bytes; /* must be 4 */
    int32_t is_train;
    int32_t legacy_placement;   /* 1: counts-only greedy plan (uep_legacy_solve_placement's rule) + round-robin reroute */
    uep_solver_params solver;
    int32_t quota_kernel_stage;         /* 0 or 1; both give identical plans, accepted for compatibility */
    int32_t grad_reduce_num_sms;        /* even, > 0, clamped to the SM count                */
    int32_t grad_reduce_deterministic;  /* 0 accepted; the fixed-order kernel always runs    */
    int32_t weight_sync_plan_mode;      /* 0 direct; 1 adaptive: experts with >= relay_min_replicas replicas, and the experts of
                                         * a rank that sends more than any rank receives, are relayed (scatter over the
                                         * replicas + replica-to-replica forward); 2 force relay (>= 2 replicas) */
    int32_t weight_sync_relay_min_replicas, weight_sync_relay_max_relays, weight_sync_relay_min_fanout_gain;
    int32_t weight_sync_num_sms;        /* CTAs of the copy kernel per rank; 0 = default     */
    int32_t wait_timeout_ms;            /* bound of every device-side wait; 0 = default 5000 */
    int32_t reroute_max_tokens;         /* > 0: the reroute scratch is sized for this many tokens per rank at creation, so
                                         * that no reroute call allocates or frees (the reference allocates per call,
                                         * csrc/ultra_ep.cpp:891-907); 0: grown on demand by the first call that needs more */
    int32_t reroute_max_topk;           /* top-k bound that goes with reroute_max_tokens (sparse form); 0 = 8 */
} uep_config;

#define UEP_IPC_HANDLE_BYTES 64

/* Collective construction, in three steps so that the caller owns the transport:
 *   create -> (export handle, all-gather the 64-byte blobs by any means) -> connect.
 * With sim_ranks > 0 connect takes NULL. Replaces Manager::Manager (csrc/ultra_ep.cpp:194-532),
 * runtime::init_runtime (csrc/runtime.cpp:29-55) and the nvshmem::alloc / nvshmem::ptr calls. */
int uep_manager_create(const uep_config* cfg, uep_manager** out);
int uep_manager_export_handle(uep_manager* m, void* handle_out /* UEP_IPC_HANDLE_BYTES, host */);
int uep_manager_connect(uep_manager* m, const void* all_handles /* [num_ranks][UEP_IPC_HANDLE_BYTES], host */);
/* Replaces Manager::destroy (csrc/ultra_ep.cpp:545-647). Device-synchronises. */
int uep_manager_destroy(uep_manager* m);
int uep_manager_num_local(const uep_manager* m); /* 1, or sim_ranks */
int uep_manager_num_sms(const uep_manager* m);

/* Buffers handed to the caller (device memory owned by the manager, valid until destroy).
 * Replaces the get_*_tensor accessors (csrc/ultra_ep.hpp:290-325). shape/stride in elements
 * of the buffer's own dtype (int32 for plan maps, uint8 for weights/scales, float for grads). */
typedef enum uep_buffer_id {
    UEP_BUF_P2L = 0,            /* int32 [layers, P]       */
    UEP_BUF_L2P,                /* int32 [layers, L, D]    */
    UEP_BUF_LCNTS,              /* int32 [layers, L]       */
    UEP_BUF_QUOTA,              /* int32 [layers, L, D]    */
    UEP_BUF_QUOTA_PREFIX,       /* int32 [layers, L, D]    */
    UEP_BUF_RANK_QUOTA_PREFIX,  /* int32 [layers, L, D]    */
    UEP_BUF_GLOBAL_LOADS,       /* int32 [L]               */
    UEP_BUF_LOADS_PER_RANK,     /* int32 [N, L] (latest gather) */
    UEP_BUF_REPLICA_WEIGHT,     /* uint8 [R, fc1B+fc2B]    */
    UEP_BUF_REPLICA_FC1_WEIGHT, /* uint8 [R, fc1B] strided */
    UEP_BUF_REPLICA_FC2_WEIGHT, /* uint8 [R, fc2B] strided */
    UEP_BUF_REPLICA_SCALE,      /* uint8 [R, scale_stride] */
    UEP_BUF_REPLICA_FC1_SCALE,  /* uint8 [R, fc1_scaleB] strided */
    UEP_BUF_REPLICA_FC2_SCALE,  /* uint8 [R, fc2_scaleB] strided */
    UEP_BUF_REPLICA_GRAD,       /* float [R, fc1+fc2]      */
    UEP_BUF_REPLICA_FC1_GRAD,   /* float [R, fc1] strided  */
    UEP_BUF_REPLICA_FC2_GRAD,   /* float [R, fc2] strided  */
    /* Tokens each physical slot receives under the stored plan (its quota; 0 for an empty slot),
     * written by the plan kernel as it emits the plan. Replaces the reference's separate
     * profiling kernel profile_physical_loads_from_quota_triton (ultra_ep/util.py:72-176) and
     * its scatter_add fallback (ultra_ep/manager.py:332-357). */
    UEP_BUF_PHYSICAL_LOADS      /* int32 [layers, P]       */
} uep_buffer_id;
int uep_manager_buffer(uep_manager* m, int local_rank, int buffer_id, void** ptr, int* ndim, int64_t shape[3],
                       int64_t stride[3]);

/* Address, in this process, of a PEER rank's replica buffer (UEP_BUF_REPLICA_WEIGHT, _SCALE or _GRAD): the
 * cudaIpc mapping the manager opened at connect (the rank's own buffer for peer_rank == its rank). What
 * nvshmem::ptr returns in the reference (csrc/ultra_ep.cpp:400-421); lets other kernels, e.g. the reference's
 * own copy kernel in a side-by-side measurement, address the same peer memory. */
int uep_manager_peer_buffer(uep_manager* m, int local_rank, int peer_rank, int buffer_id, void** ptr);

/* Per-call arguments are arrays of length uep_manager_num_local(m): element i belongs to
 * local rank i (a single element in the one-rank-per-process case).
 *
 * update_placement: histogram -> load all-gather over peer memory -> reduce -> solve, one
 * launch on `stream`. input_kind: 0 dense bool map [T,L]; 1 int32 ids [T,K]; 2 int64 ids [T,K].
 * Collective: every rank of the group must call it the same number of times.
 * Replaces Manager::update_placement / update_placement_sparse (csrc/ultra_ep.cpp:668-832). */
int uep_update_placement(uep_manager* m, int layer_id, int input_kind, const void* const* inputs, const int* T,
                         int K_or_L, void* stream);

/* weight_sync: push every replicated local master (weights + scales) into its peers' slots.
 * ptr tables are device arrays int64[M] of raw device addresses, re-supplied per call.
 * Runs on the manager's comm stream after `wait_event` (or after `current_stream` if NULL).
 * async_finish != 0: *done_event receives an event to wait on; else current_stream waits.
 * Replaces Manager::weight_sync (csrc/ultra_ep.cpp:1095-1211). */
int uep_weight_sync(uep_manager* m, int layer_id, const int64_t* const* fc1_ptrs, const int64_t* const* fc2_ptrs,
                    const int64_t* const* fc1_scale_ptrs, const int64_t* const* fc2_scale_ptrs,
                    uep_event* wait_event, int async_finish, void* current_stream, uep_event** done_event);

/* grad_reduce: master += replicas (fp32, replicas in plan order), replicas zeroed.
 * Replaces Manager::grad_reduce (csrc/ultra_ep.cpp:1036-1093). */
int uep_grad_reduce(uep_manager* m, int layer_id, const int64_t* const* fc1_grad_ptrs,
                    const int64_t* const* fc2_grad_ptrs, uep_event* wait_event, int async_finish,
                    void* current_stream, uep_event** done_event);

/* Reroute with the stored plan of `layer_id`; waits for that layer's plan if it was
 * produced on another stream. Outputs are caller-allocated device buffers.
 * Replace Manager::dense_reroute_forward/_backward and reroute_sparse
 * (csrc/ultra_ep.cpp:874-984, 834-872). ids_kind: 1 int32, 2 int64. */
int uep_reroute_dense_forward(uep_manager* m, int layer_id, const uint8_t* const* routing_maps,
                              const float* const* probs, uint8_t* const* expanded_maps, float* const* expanded_probs,
                              const int* T, void* stream);
int uep_reroute_dense_backward(uep_manager* m, int layer_id, const float* const* grad_expanded,
                               const uint8_t* const* routing_maps, const uint8_t* const* expanded_maps,
                               float* const* grad_probs, const int* T, int P, void* stream);
int uep_reroute_sparse(uep_manager* m, int layer_id, int ids_kind, const void* const* ids, void* const* out,
                       const int* T, int K, void* stream);

/* Mutators. Replace set_weight_sync_plan_mode / set_grad_reduce_deterministic
 * (csrc/ultra_ep.cpp:986-1034). */
int uep_set_weight_sync_plan_mode(uep_manager* m, int plan_mode);
int uep_set_grad_reduce_deterministic(uep_manager* m, int deterministic, int num_sms);

void* uep_manager_comm_stream(uep_manager* m); /* cudaStream_t; csrc/ultra_ep.hpp:286 */

/* Events. Replace EventHandle (csrc/utils/event.hpp:12-28). */
int uep_event_record(void* stream, uep_event** out);
int uep_event_stream_wait(uep_event* ev, void* stream);
int uep_event_synchronize(uep_event* ev);
void uep_event_destroy(uep_event* ev);

/* Latest device-side status of local rank `local_rank` (UEP_DEV_*), read without
 * synchronising; detail receives a kernel-specific value (e.g. the peer that timed out).
 * Replaces the reference's device asserts (csrc/utils/exception.cuh:41-47), which trap. */
int uep_poll_status(uep_manager* m, int local_rank, int* code, int* detail);
int uep_clear_status(uep_manager* m);

/* Failure-detection test hook, host side only: from the next call on, the hosted rank `rank`
 * completes its work but does not publish its load row / completion flags, so the ranks
 * that wait for it run into their time limit and report UEP_DEV_TIMEOUT_*; -1 switches the
 * hook off. No device fault is involved. No counterpart in the reference (its waits are
 * unbounded, csrc/kernels/weight_sync.cu:666-677, csrc/kernels/ptx.cuh:73-86). */
int uep_debug_withhold_rank(uep_manager* m, int rank);

/* Tuning aid: with UEP_SYNC_TRACE=1 in the environment when the manager is created, the
 * weight_sync kernel records eight %globaltimer stamps per CTA (start, set-up done, copies
 * issued, copies complete, fenced, ticket taken, completion flags received, completion flags
 * sent; the last two only in the CTA that finishes last); this copies the stamps of the first
 * max_ctas CTAs of the latest launch to host memory [max_ctas][8]. Rows 1000.. and 1008.. of the
 * same buffer hold, per hosted rank, the plan kernel's phases (histogram done, row published, rows
 * gathered and reduced, -, solved, CTA start) and the solver's (enter, loads staged, sorted,
 * searched, emitted, split). The withhold hook also makes a withheld rank skip publishing its
 * load row. No counterpart in the reference. */
int uep_debug_sync_trace(uep_manager* m, unsigned long long* host_out, int max_ctas);

/* Measurement aid: time of one one-directional copy of `bytes` bytes (a multiple of 16, at most the replica
 * weight buffer) from this rank's replica weight buffer into peer_rank's, averaged over `iters` copies on the
 * communication stream; use_kernel 0: cudaMemcpyAsync (copy engine), 1: a plain load/store kernel; add 2 to copy
 * the other way (this rank reads the peer's buffer: the direction of the Wgrad reduce's loads). Overwrites
 * the peer's replica slots; the peer must be idle. Gives the link bandwidth the copy and reduce kernels are
 * measured against. No counterpart in the reference. */
int uep_debug_link_probe(uep_manager* m, int peer_rank, int64_t bytes, int iters, int use_kernel, float* ms_out);

/* Counters for benchmarks: kernels launched by this library since the last reset. */
int64_t uep_launch_count(void);
void uep_reset_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* UEP_B200_H */
