// Kernel 3 — weight_sync: every replicated local master expert (weights and scales) is
// pushed into the replica slots of its peers, straight from the stored plan.
//
// The reference first builds a task list with a single-thread kernel and then runs a
// thread-copy kernel (16-byte loads, streaming stores) when the NVLink domain has at most
// 8 ranks, or a two-stage bulk-copy kernel above that (csrc/kernels/weight_sync.cu:205-522,
// 714-775, 782-986 of the reference). Here there is no task list and one kernel:
//   * every CTA derives the send list from the plan rows of this rank's masters
//     (l2p / lcnts) with a block-wide scan; all global reads of the set-up are issued together;
//   * one elected thread per CTA drives a 4-stage ring of 32 KiB bulk copies: the tile is
//     read from local HBM once (cp.async.bulk global->shared, mbarrier) and stored to each
//     destination slot (cp.async.bulk shared->global, peer memory over NVLink); loads run
//     up to three tiles ahead of the stores;
//   * work is handed out by an atomic counter, interleaved over masters so that concurrent
//     CTAs feed different peers; when several ranks are hosted on one device their work forms
//     one pool shared by all CTAs;
//   * the CTA that finishes last issues one system-scope fence and then tells the ranks it
//     sent to "rank r has delivered epoch e" (relaxed stores), and waits, bounded, for the same
//     word from the ranks that send to it. When the kernel ends, this rank's replica slots are
//     complete.
// Pointers or sizes that are not multiples of 16 bytes take a plain vector/byte copy path.
//
// Relay (optional; the reference's relay plan, csrc/kernels/weight_sync.cu:129-191, 295-502,
// exists only for NVLink domains above 8 ranks and raises one ready flag per chunk of tiles,
// :638-677). A relayed expert with r replicas is broadcast as scatter + forward in chunks of
// four tiles (128 KiB; one-tile chunks with a flag each measured slower): its master sends chunk
// c only to replica c mod r and raises that chunk's ready flag there once the chunk's stores are
// complete (a system-scope fence in a thread of its own, one fence for all flags that are due);
// every replica forwards the chunks it received from the master to the other r-1 replicas. The
// master's rank then sends the expert once instead of r times, and the forwarding load is
// spread over the replicas' ranks. Which experts are relayed is a pure function of the plan and
// the configuration, so all ranks agree without talking:
//   * force mode: every expert with at least two replicas;
//   * adaptive mode: experts with at least relay_min_replicas replicas, and, on a rank whose
//     outbound volume exceeds the largest inbound volume of any rank in this plan (which no
//     relaying can reduce), that rank's experts with the most replicas until it no longer does.
// Relayed chunks are handed out first (a second hop depends on them), then the direct tiles,
// then the forward chunks: a CTA that waits (bounded) for a ready flag waits for a chunk that a
// running CTA, on this or another device, is already sending.

#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "internal.h"

namespace uep {

namespace {

constexpr int kSyncThreads = 128;
constexpr int kMaxSends = kMaxExportsPerDomain;  // replicas of one rank's masters never exceed G*R <= 512
constexpr int kMaxFwd = 64;                       // replica slots of the hosted ranks that may forward
constexpr int kMaxRelayReplicas = 16;
constexpr int kMaxFwdDst = kMaxFwd * (kMaxRelayReplicas - 1);
constexpr int kChunkTiles = 4;                    // tiles per relayed chunk (one ready flag per chunk)
// A relayed chunk's flag is raised once the store group kFlagDepth groups behind the newest one is complete.
// A CTA moves about 32 KiB per NVLink round trip when 64 of them share the link, so every group of depth
// delays the second hop by about 3 us; the issuing thread waits at a chunk's end only.
constexpr int kFlagDepth = 1;

// One unit of work as the counter hands it out.
struct Unit {
    int kind;            // 0: one tile of a direct expert; 1: a chunk a master scatters; 2: a chunk a replica forwards
    int who;             // kind 0/1: index of the active master; kind 2: forward entry
    int tile, tile_end;  // tile range over the expert's shards
    int chunk;           // kind 1/2: chunk index (selects the ready flag)
};

struct TileRef {
    int kind, who;
    int tile_in_expert;  // tile index over the expert's shards
    int shard;           // 0..3
    int64_t offset;      // byte offset inside the shard
    int bytes;           // bytes of this tile
    int chunk;
};

struct SyncShared {
    int n_active;          // masters (of all hosted ranks) that have replicas
    int total_reps;        // sum of their replica counts
    int all_aligned;       // every source pointer 16-byte aligned
    int is_last;
    int n_relay;           // relayed ones among the active masters
    int n_fwd;             // forward entries
    int fwd_units;         // forward units: rounds x entries (a unit whose chunk lies behind the expert's end is empty)
    int floor_in;          // adaptive relay: the largest inbound expert count of any rank
    unsigned send_mask[kMaxLocalRanks][3];  // per hosted rank: ranks it writes to (as master or as forwarder)
    unsigned recv_mask[kMaxLocalRanks][3];  // per hosted rank: ranks that write to it
    int timeout_peer;
    int s_unit;
    unsigned long long epoch;
    int shard_tiles[4];
    int w_a[kSyncThreads / 32], w_r[kSyncThreads / 32];
    int rank_out[kMaxPeers], rank_in[kMaxPeers];  // adaptive relay: experts each rank sends / receives under this plan
    short rep_start[kMaxExpertsPerDomain + 1];  // [n_active+1] offsets into dst_*
    short order[kMaxExpertsPerDomain];          // hand-out order of the active masters: relayed ones first
    unsigned char relay_r[kMaxExpertsPerDomain];  // [n_active] 0: direct, else the replica count of a relayed expert
    unsigned char relay_of[kMaxExpertsPerDomain]; // [logical expert of the domain] the same for every expert of the plan
    unsigned char reps_of[kMaxExpertsPerDomain];  // [logical expert of the domain] its replica count (capped at 255)
    // Addresses are resolved once per CTA: the issuing thread must not chase pointers
    // through global memory for every 32 KiB tile.
    const uint8_t* src[kMaxExpertsPerDomain][4];  // [n_active][shard] master shard base
    uint8_t* dst_weight[kMaxSends];               // replica slot base in the peer's weight buffer (null: skip)
    uint8_t* dst_scale[kMaxSends];                // replica slot base in the peer's scale buffer
    uint64_t* dst_flags[kMaxSends];               // that slot's row of ready flags on the peer (relay)
    // replica buffer bases of every (hosted rank, peer): nlocal * N entries (at most 72: several
    // hosted ranks mean a simulated group of at most 8)
    uint8_t* peer_weight[kMaxPeers];
    uint8_t* peer_scale[kMaxPeers];
    uint64_t* peer_flags[kMaxPeers];
    // forward entries: one per local replica slot that holds a relayed expert
    uint8_t* fwd_src_w[kMaxFwd];        // the slot itself
    uint8_t* fwd_src_s[kMaxFwd];
    const uint64_t* fwd_flags[kMaxFwd]; // its row of ready flags
    unsigned char fwd_r[kMaxFwd], fwd_k[kMaxFwd], fwd_lr[kMaxFwd];
    short fwd_dst_start[kMaxFwd + 1];
    uint8_t* fwd_dst_w[kMaxFwdDst];
    uint8_t* fwd_dst_s[kMaxFwdDst];
    __align__(8) uint64_t bars[8];
    // State of the issuing thread's ring, kept here rather than in its local memory: the kernels that run
    // next to this one evict the L1 lines a stack frame lives in, and every miss would sit on the critical
    // path of a tile.
    // Ready flags handed to the posting thread: the system-scope fence in front of a flag would make the issuing
    // thread wait for its own stores in flight; a thread without stores of its own pays almost nothing for it.
    uint64_t* post[8];
    volatile int post_head, post_tail, post_done;
    TileRef ring[8];         // the tile held by each stage
    uint64_t* ring_flag[8];  // ready flag to raise once that stage's tile is stored (last tile of a chunk)
    uint64_t* owed[8];       // ready flag owed for the k-th stored tile, slot k % stages
    int ring_valid[8];
};

template <int kSyncTile>
__device__ __forceinline__ void locate_tile(TileRef& t, const ShardLayout& sh, const int* shard_tiles) {
    int tile = t.tile_in_expert;
    t.shard = 0;
    while (t.shard < sh.num_shards - 1 && tile >= shard_tiles[t.shard]) {
        tile -= shard_tiles[t.shard];
        ++t.shard;
    }
    t.offset = static_cast<int64_t>(tile) * kSyncTile;
    const int64_t left = sh.bytes[t.shard] - t.offset;
    t.bytes = static_cast<int>(left < kSyncTile ? left : kSyncTile);
}

__device__ __forceinline__ uint8_t* shard_base(uint8_t* weight_slot, uint8_t* scale_slot, const ShardLayout& sh, int shard) {
    return (shard < 2 ? weight_slot : scale_slot) + sh.slot_offset[shard];
}

// `streaming`: the source is read-only for the whole launch (a master). A forwarded tile was written
// by a peer during this launch and must be read through L2.
__device__ void copy_plain(const uint8_t* src, uint8_t* dst, int bytes, bool streaming) {
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    int done = 0;
    if (vec) {
        const int nvec = bytes / 16;
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
            const void* p = src + static_cast<int64_t>(i) * 16;
            st_global_cs_v4(dst + static_cast<int64_t>(i) * 16, streaming ? ld_global_nc_v4(p) : ld_global_cg_v4(p));
        }
        done = nvec * 16;
    }
    for (int i = done + threadIdx.x; i < bytes; i += blockDim.x) dst[i] = streaming ? src[i] : __ldcg(src + i);
}

// kRelay = false compiles the relay machinery out: the direct fan-out pays neither for its code nor for
// its per-tile bookkeeping (the kernel runs once per layer from a cold instruction cache, and the one
// issuing thread per CTA is on the critical path of every tile).
template <int kSyncTile, int kSyncStages, bool kRelay>
__global__ void __launch_bounds__(kSyncThreads) weight_sync_kernel(SyncCall call) {
    extern __shared__ __align__(128) char smem_raw[];  // kSyncStages * kSyncTile, then SyncShared
    SyncShared& sm = *reinterpret_cast<SyncShared*>(smem_raw + static_cast<size_t>(kSyncStages) * kSyncTile);
    uint64_t* bars = sm.bars;
    int* shard_tiles = sm.shard_tiles;

    const ShardLayout& sh = call.shards;
    const int M = call.M, R = call.R, D = call.D, Lp = M + R, N = call.N, nlocal = call.nlocal;
    const int tid = threadIdx.x;
    // Relaying needs a forward entry per local replica slot and a ready flag per chunk; the limits depend on
    // the configuration only, so every rank comes to the same answer.
    int tiles_per_expert = 0;
    for (int s = 0; s < sh.num_shards; ++s) tiles_per_expert += static_cast<int>((sh.bytes[s] + kSyncTile - 1) / kSyncTile);
    const int chunks_per_expert = (tiles_per_expert + kChunkTiles - 1) / kChunkTiles;
    const bool relay_on = kRelay && call.relay_min_replicas > 0 && nlocal * R <= kMaxFwd && chunks_per_expert <= call.relay_cap &&
                          N * M <= kMaxExpertsPerDomain && N <= kMaxPeers;
    auto stamp = [&](int slot) {
        if (call.trace != nullptr && tid == 0) call.trace[blockIdx.x * 8 + slot] = global_timer_ns();
    };
    stamp(0);

    // ---- setup: send list of the hosted ranks from their plans ---------------------------
    if (tid == 0) {
        sm.n_active = 0;
        sm.total_reps = 0;
        sm.all_aligned = 1;
        sm.is_last = 0;
        sm.n_relay = 0;
        sm.n_fwd = 0;
        sm.fwd_units = 0;
        sm.floor_in = 1;
        sm.timeout_peer = -1;
        sm.post_head = 0;
        sm.post_tail = 0;
        sm.post_done = 0;
        for (int s = 0; s < 4; ++s) shard_tiles[s] = s < sh.num_shards ? static_cast<int>((sh.bytes[s] + kSyncTile - 1) / kSyncTile) : 0;
        for (int s = 0; s < kSyncStages; ++s) mbar_init(&bars[s], 1);
        fence_mbar_init();
    }
    for (int i = tid; i < kMaxLocalRanks * 3; i += blockDim.x) {
        sm.send_mask[i / 3][i % 3] = 0;
        sm.recv_mask[i / 3][i % 3] = 0;
    }
    if (kRelay) {
        for (int i = tid; i < N && i < kMaxPeers; i += blockDim.x) {
            sm.rank_out[i] = 0;
            sm.rank_in[i] = 0;
        }
    }
    __syncthreads();
    // Every global read of the set-up is issued here, before anything depends on one of them, so
    // that they share one memory round trip instead of forming a chain (counts -> l2p rows ->
    // peer tables): the plan rows of the first 128 masters (speculatively the whole l2p row when
    // it has at most 8 entries), their source addresses, the peers' buffer bases and the
    // owners of this rank's redundant slots.
    const int total_masters = nlocal * M;
    const bool row_cached = D <= 8;
    int pre_reps = 0, pre_row[7];
    uintptr_t pre_src[4];
    {
        const bool valid = tid < total_masters;
        const int lr = valid ? tid / M : 0, m = valid ? tid % M : 0;
        const int l = call.my_rank[lr] * M + m;
        const PlanPtrs& plan = call.plan[lr];
        pre_reps = valid ? plan.lcnts[l] - 1 : 0;
#pragma unroll
        for (int j = 0; j < 7; ++j) pre_row[j] = (valid && row_cached && j < D - 1) ? plan.l2p[static_cast<int64_t>(l) * D + 1 + j] : -1;
#pragma unroll
        for (int sh_i = 0; sh_i < 4; ++sh_i) {
            const bool present = valid && sh_i < sh.num_shards && sh.bytes[sh_i] != 0;
            pre_src[sh_i] = present ? static_cast<uintptr_t>(call.src_ptrs[lr][sh_i][m]) : 0;
        }
    }
    uint8_t *pre_pw = nullptr, *pre_ps = nullptr;
    uint64_t* pre_pf = nullptr;
    if (tid < nlocal * N) {
        const RankDev& rk = *call.rank[tid / N];
        pre_pw = rk.peer_replica_weight[tid % N];
        pre_ps = rk.peer_replica_scale[tid % N];
        if (kRelay) pre_pf = rk.peer_relay_flags[tid % N];
    }
    // Ranks hosted together share the first one's epoch counter: they always run in the same launches.
    // The CTA that finishes last stores the new value; nobody reads the counter after that.
    unsigned long long pre_epoch = 0;
    if (tid == 0) pre_epoch = *call.sync_epoch;
    int pre_owner = -1;
    if (tid < nlocal * R) pre_owner = call.plan[tid / R].p2l[call.my_rank[tid / R] * Lp + M + tid % R];
    // relay decision: the replica count of logical expert `tid` and the owner of redundant slot `tid` of the group
    int pre_lc = 1, pre_slot_owner = -1;
    if (kRelay && relay_on) {
        if (tid < N * M) pre_lc = call.plan[0].lcnts[tid];
        if (call.relay_adaptive && tid < N * R) pre_slot_owner = call.plan[0].p2l[(tid / R) * Lp + M + tid % R];
    }
    if (tid < nlocal * N) {
        sm.peer_weight[tid] = pre_pw;
        sm.peer_scale[tid] = pre_ps;
        sm.peer_flags[tid] = pre_pf;
    }
    if (tid == 0) sm.epoch = pre_epoch + 1;

    // Which experts are relayed: one answer per logical expert, the same on every rank (the plan is).
    if (kRelay) {
        const PlanPtrs& plan0 = call.plan[0];
        const int L = min(N * M, kMaxExpertsPerDomain);
        for (int l = tid; l < L; l += blockDim.x) {
            int reps = relay_on ? (l == tid ? pre_lc : plan0.lcnts[l]) - 1 : 0;
            reps = reps < 0 ? 0 : (reps > D - 1 ? D - 1 : reps);
            const bool by_count = reps >= call.relay_min_replicas && reps >= 2 && reps <= kMaxRelayReplicas;
            sm.relay_of[l] = by_count ? static_cast<unsigned char>(reps) : 0;
            sm.reps_of[l] = static_cast<unsigned char>(reps > 255 ? 255 : reps);
            if (relay_on && call.relay_adaptive && reps > 0) atomicAdd(&sm.rank_out[l / M], reps);
        }
        if (relay_on && call.relay_adaptive) {
            for (int i = tid; i < N * R; i += blockDim.x) {
                const int r = i / R;
                if ((i == tid ? pre_slot_owner : plan0.p2l[r * Lp + M + i % R]) >= 0) atomicAdd(&sm.rank_in[r], 1);
            }
        }
        __syncthreads();
        if (relay_on && call.relay_adaptive) {
            if (tid < 32) {  // the inbound volume no relaying can reduce
                int mx = 1;
                for (int r = tid; r < N; r += 32) mx = max(mx, sm.rank_in[r]);
                mx = warp_max(mx);
                if (tid == 0) sm.floor_in = mx;
            }
            __syncthreads();
            // one thread per rank: while the rank sends more experts than that, relay its expert with the most
            // replicas (ties: lower index); a relayed expert leaves its master's rank once instead of reps times
            for (int r = tid; r < N; r += blockDim.x) {
                int out = sm.rank_out[r];
                while (out > sm.floor_in) {
                    int best = -1, best_reps = 1;
                    for (int m = 0; m < M; ++m) {
                        const int l = r * M + m;
                        if (sm.relay_of[l]) continue;
                        const int reps = sm.reps_of[l];
                        if (reps > best_reps && reps <= kMaxRelayReplicas) {
                            best = l;
                            best_reps = reps;
                        }
                    }
                    if (best < 0) break;
                    sm.relay_of[best] = static_cast<unsigned char>(best_reps);
                    out -= best_reps - 1;
                }
            }
        }
        __syncthreads();
    }
    // (the scan below synchronises the CTA before the tables are read)

    // blocked scan over (hosted rank, master): active index and replica offsets
    for (int g0 = 0; g0 < total_masters; g0 += blockDim.x) {
        const int gm = g0 + tid;
        const int lr = gm < total_masters ? gm / M : 0;
        const int m = gm < total_masters ? gm % M : 0;
        const RankDev& rk = *call.rank[lr];
        const PlanPtrs& plan = call.plan[lr];
        const int me = call.my_rank[lr];
        int reps = 0;
        if (gm < total_masters) {
            reps = g0 == 0 ? pre_reps : plan.lcnts[me * M + m] - 1;
            reps = reps < 0 ? 0 : (reps > D - 1 ? D - 1 : reps);
        }
        const int act = reps > 0 ? 1 : 0;
        // warp-level inclusive scans, then across warps through shared memory
        int a_incl = act, r_incl = reps;
        const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int oa = __shfl_up_sync(kFullMask, a_incl, d), orr = __shfl_up_sync(kFullMask, r_incl, d);
            if (lane >= d) {
                a_incl += oa;
                r_incl += orr;
            }
        }
        if (lane == 31) {
            sm.w_a[warp] = a_incl;
            sm.w_r[warp] = r_incl;
        }
        __syncthreads();
        int a_off = sm.n_active, r_off = sm.total_reps;
        for (int w = 0; w < warp; ++w) {
            a_off += sm.w_a[w];
            r_off += sm.w_r[w];
        }
        if (act) {
            const int ai = a_off + a_incl - 1;
            const int rs = r_off + r_incl - reps;
            sm.rep_start[ai] = static_cast<short>(rs);
            const int l = me * M + m;
            if (kRelay) sm.relay_r[ai] = sm.relay_of[l];
            auto place = [&](int j, int phys) {
                const int drank = phys / Lp, dslot = phys % Lp - M;
                if (phys < 0 || drank >= N || dslot < 0 || dslot >= R) {  // never store outside a slot table
                    report_error(rk.status, UEP_DEV_BAD_PLAN, l);
                    sm.dst_weight[rs + j] = nullptr;
                    sm.dst_scale[rs + j] = nullptr;
                    if (kRelay) sm.dst_flags[rs + j] = nullptr;
                } else {
                    atomicOr(&sm.send_mask[lr][drank >> 5], 1u << (drank & 31));
                    sm.dst_weight[rs + j] = sm.peer_weight[lr * N + drank] + static_cast<int64_t>(dslot) * sh.weight_slot_stride;
                    sm.dst_scale[rs + j] = sm.peer_scale[lr * N + drank] + static_cast<int64_t>(dslot) * sh.scale_slot_stride;
                    if (kRelay) sm.dst_flags[rs + j] = sm.peer_flags[lr * N + drank] + static_cast<int64_t>(dslot) * call.relay_cap;
                }
            };
            if (g0 == 0 && row_cached) {
#pragma unroll
                for (int j = 0; j < 7; ++j) {
                    if (j < reps && rs + j < kMaxSends) place(j, pre_row[j]);
                }
            } else {
                for (int j = 0; j < reps && rs + j < kMaxSends; ++j) place(j, plan.l2p[static_cast<int64_t>(l) * D + 1 + j]);
            }
            // source addresses and their alignment
            for (int s = 0; s < 4; ++s) {
                const bool present = s < sh.num_shards && sh.bytes[s] != 0;
                uintptr_t p = 0;
                if (g0 == 0) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) p = (u == s) ? pre_src[u] : p;
                } else if (present) {
                    p = static_cast<uintptr_t>(call.src_ptrs[lr][s][m]);
                }
                sm.src[ai][s] = reinterpret_cast<const uint8_t*>(p);
                if (p & 15u) atomicAnd(&sm.all_aligned, 0);
            }
        }
        __syncthreads();
        if (tid == blockDim.x - 1) {
            sm.n_active = a_off + a_incl;
            sm.total_reps = r_off + r_incl;
        }
        __syncthreads();
    }
    if (tid == 0) {
        sm.rep_start[sm.n_active] = static_cast<short>(sm.total_reps < kMaxSends ? sm.total_reps : kMaxSends);
        if (kRelay) {  // hand-out order: relayed masters first (their chunks have a second hop behind them)
            int k = 0;
            for (int a = 0; a < sm.n_active; ++a) {
                if (sm.relay_r[a]) sm.order[k++] = static_cast<short>(a);
            }
            sm.n_relay = k;
            for (int a = 0; a < sm.n_active; ++a) {
                if (!sm.relay_r[a]) sm.order[k++] = static_cast<short>(a);
            }
        }
    }
    // Owners of the local replica slots: who sends to this rank; and, for relayed experts, what this
    // rank forwards. One thread per (hosted rank, slot).
    int my_fwd_r = 0, my_fwd_k = -1, my_l = -1;
    for (int i = tid; i < nlocal * R; i += blockDim.x) {
        const int lr = i / R, slot = i % R;
        const int me = call.my_rank[lr];
        const int l = i == tid ? pre_owner : call.plan[lr].p2l[me * Lp + M + slot];
        if (l >= 0) {
            const int src = l / M;
            if (src >= 0 && src < N && src != me) atomicOr(&sm.recv_mask[lr][src >> 5], 1u << (src & 31));
            if (kRelay && relay_on && i == tid && l < N * M) {  // nlocal * R <= kMaxFwd <= blockDim.x: one pass
                const int reps = sm.relay_of[l];
                if (reps > 0) {
                    const int mine = me * Lp + M + slot;
                    for (int j = 0; j < reps; ++j) {
                        if (call.plan[lr].l2p[static_cast<int64_t>(l) * D + 1 + j] == mine) my_fwd_k = j;
                    }
                    if (my_fwd_k >= 0) {
                        my_fwd_r = reps;
                        my_l = l;
                    }
                }
            }
        }
    }
    if (kRelay && relay_on) {
        // compact the forward entries (thread order = slot order) and lay out their destination lists
        const unsigned has = __ballot_sync(kFullMask, my_fwd_r > 0);
        const int lane = tid & 31, warp = tid >> 5;
        if (lane == 0) sm.w_a[warp] = __popc(has);
        __syncthreads();
        int f = __popc(has & ((1u << lane) - 1u));
        for (int w = 0; w < warp; ++w) f += sm.w_a[w];
        if (my_fwd_r > 0) {
            const int lr = tid / R, slot = tid % R;
            const int me = call.my_rank[lr];
            sm.fwd_src_w[f] = sm.peer_weight[lr * N + me] + static_cast<int64_t>(slot) * sh.weight_slot_stride;
            sm.fwd_src_s[f] = sm.peer_scale[lr * N + me] + static_cast<int64_t>(slot) * sh.scale_slot_stride;
            sm.fwd_flags[f] = sm.peer_flags[lr * N + me] + static_cast<int64_t>(slot) * call.relay_cap;
            sm.fwd_r[f] = static_cast<unsigned char>(my_fwd_r);
            sm.fwd_k[f] = static_cast<unsigned char>(my_fwd_k);
            sm.fwd_lr[f] = static_cast<unsigned char>(lr);
            sm.fwd_dst_start[f + 1] = static_cast<short>(my_fwd_r - 1);
        }
        __syncthreads();
        if (tid == 0) {
            int nf = 0;
            for (int w = 0; w < kSyncThreads / 32; ++w) nf += sm.w_a[w];
            sm.fwd_dst_start[0] = 0;
            for (int e = 0; e < nf; ++e) sm.fwd_dst_start[e + 1] = static_cast<short>(sm.fwd_dst_start[e + 1] + sm.fwd_dst_start[e]);
            sm.n_fwd = nf;
            // entry f forwards the chunks k_f, k_f + r_f, ...: round j of every entry comes before round j + 1 of any,
            // which is the order the chunks arrive in; r >= 2, so ceil(chunks / 2) rounds cover every entry
            sm.fwd_units = nf * ((chunks_per_expert + 1) / 2);
        }
        __syncthreads();
        if (my_fwd_r > 0) {
            const int lr = tid / R;
            const int me = call.my_rank[lr];
            int o = sm.fwd_dst_start[f];
            for (int j = 0; j < my_fwd_r; ++j) {
                const int phys = call.plan[lr].l2p[static_cast<int64_t>(my_l) * D + 1 + j];
                const int drank = phys / Lp, dslot = phys % Lp - M;
                const bool bad = phys < 0 || drank >= N || dslot < 0 || dslot >= R;
                if (!bad && drank != me) atomicOr(&sm.recv_mask[lr][drank >> 5], 1u << (drank & 31));  // it forwards to me
                if (j == my_fwd_k) continue;
                if (bad) {
                    sm.fwd_dst_w[o] = nullptr;
                    sm.fwd_dst_s[o] = nullptr;
                } else {
                    atomicOr(&sm.send_mask[lr][drank >> 5], 1u << (drank & 31));
                    sm.fwd_dst_w[o] = sm.peer_weight[lr * N + drank] + static_cast<int64_t>(dslot) * sh.weight_slot_stride;
                    sm.fwd_dst_s[o] = sm.peer_scale[lr * N + drank] + static_cast<int64_t>(dslot) * sh.scale_slot_stride;
                }
                ++o;
            }
        }
    }
    __syncthreads();

    stamp(1);
    // ---- copy -------------------------------------------------------------------------
    // The copy loop exists twice inside the relay-capable kernel: with and without the relay machinery. A rank
    // that neither scatters nor forwards anything in this launch takes the compact one: the kernel runs once per
    // layer from a cold instruction cache, and every extra line of code on the path of the first tiles is a miss.
    const uint64_t epoch = sm.epoch;
    DeviceStatus* status0 = call.rank[0]->status;
    int* unit_counter = call.rank[0]->sync_ticket + 1;
    auto run_copy = [&](auto relay_tag) {
        constexpr bool kR = decltype(relay_tag)::value;
        const int n_relay = kR ? sm.n_relay : 0;
        const int n_direct = sm.n_active - n_relay;
        const int relay_units = n_relay * chunks_per_expert;
        const int send_units = relay_units + n_direct * tiles_per_expert;
        const int total_units = send_units + (kR ? sm.fwd_units : 0);
        // Work is handed out by an atomic counter: CTAs that run on busy SMs (the reroute and the
        // model's own kernels run next to this one) simply take less, and replica counts that differ
        // between masters cannot leave some CTAs with several times the work of others.

        auto decode_unit = [&](int u) -> Unit {
            Unit un;
            if (kR && u < relay_units) {
                const int nr = kR ? n_relay : 1;  // (never zero where this branch can run)
                un.kind = 1;
                un.who = sm.order[u % nr];
                un.chunk = u / nr;
                un.tile = un.chunk * kChunkTiles;
                un.tile_end = min(un.tile + kChunkTiles, tiles_per_expert);
            } else if (!kR || u < send_units) {
                const int v = u - relay_units;
                un.kind = 0;
                un.who = kR ? sm.order[n_relay + v % n_direct] : v % n_direct;
                un.chunk = 0;
                un.tile = v / n_direct;
                un.tile_end = un.tile + 1;
            } else {
                const int v = u - send_units;
                const int f = v % sm.n_fwd;
                un.kind = 2;
                un.who = f;
                un.chunk = sm.fwd_k[f] + (v / sm.n_fwd) * sm.fwd_r[f];
                un.tile = min(un.chunk * kChunkTiles, tiles_per_expert);  // behind the end: an empty unit
                un.tile_end = min(un.tile + kChunkTiles, tiles_per_expert);
            }
            return un;
        };
        // Source of a tile (a forwarded tile is read from the local slot it landed in).
        auto tile_source = [&](const TileRef& t) -> const uint8_t* {
            if (!kR || t.kind != 2) return sm.src[t.who][t.shard] + t.offset;
            return shard_base(sm.fwd_src_w[t.who], sm.fwd_src_s[t.who], sh, t.shard) + t.offset;
        };
        // A forwarded chunk may be read once the master has delivered it here: bounded wait on its ready flag
        // (relaxed polls, closed by one acquire load: an acquire does not wait for this thread's own stores in flight).
        auto chunk_arrived = [&](const Unit& un) -> bool {
            return un.tile >= un.tile_end || ld_relaxed_sys_u64(sm.fwd_flags[un.who] + un.chunk) >= epoch;
        };
        auto wait_chunk = [&](const Unit& un) -> bool {
            if (un.tile >= un.tile_end) return true;  // empty unit
            bool ok = true;
            if (!wait_flag_ge_relaxed(sm.fwd_flags[un.who] + un.chunk, epoch, call.timeout_ns)) {
                ok = false;
                report_error(call.rank[sm.fwd_lr[un.who]]->status, UEP_DEV_TIMEOUT_SYNC, un.chunk);
            }
            (void)ld_acquire_sys_u64(sm.fwd_flags[un.who] + un.chunk);  // acquire side of the flag
            fence_proxy_async_global();                                 // ... also for the bulk copies that read the chunk next
            return ok;
        };
        // Destinations of a tile: d = first .. first+count-1 -> address (null: skip). A scattered chunk has one
        // destination, replica (chunk mod r).
        auto dest_range = [&](const TileRef& t, int& first, int& count) {
            if (!kR || t.kind != 2) {
                const int r0 = sm.rep_start[t.who], r1 = sm.rep_start[t.who + 1];
                if (!kR || t.kind == 0) {
                    first = r0;
                    count = r1 - r0;
                } else {
                    first = r0 + t.chunk % sm.relay_r[t.who];
                    count = first < r1 ? 1 : 0;
                }
            } else {
                first = sm.fwd_dst_start[t.who];
                count = sm.fwd_dst_start[t.who + 1] - first;
            }
        };
        auto dest_addr = [&](const TileRef& t, int d) -> uint8_t* {
            uint8_t* w = (!kR || t.kind != 2) ? sm.dst_weight[d] : sm.fwd_dst_w[d];
            if (w == nullptr) return nullptr;
            uint8_t* s = (!kR || t.kind != 2) ? sm.dst_scale[d] : sm.fwd_dst_s[d];
            return shard_base(w, s, sh, t.shard) + t.offset;
        };
        // Ready flag of a scattered chunk on the replica that receives it (null: nothing to raise).
        auto chunk_flag = [&](const Unit& un) -> uint64_t* {
            const int r0 = sm.rep_start[un.who], r1 = sm.rep_start[un.who + 1];
            const int d = r0 + un.chunk % sm.relay_r[un.who];
            if (d >= r1 || sm.dst_flags[d] == nullptr) return nullptr;
            return sm.dst_flags[d] + un.chunk;
        };

        if (sm.all_aligned) {
            if (tid == 0) {
                TileRef* ring = sm.ring;
                int* ring_valid = sm.ring_valid;
                uint64_t** ring_flag = sm.ring_flag;
                uint64_t** owed = sm.owed;
                uint32_t phase_bits = 0;           // bit s: parity the next wait on stage s expects
                bool ok = true;
                int posted = 0;
                // hands a ready flag whose chunk is complete to the posting thread (which fences and stores it)
                auto post_flag = [&](uint64_t* flag) {
                    // the posting thread never blocks; bounded all the same (a flag that is dropped here shows up
                    // as a time-out of the rank that waits for it)
                    const uint64_t t_begin = global_timer_ns();
                    while (posted - sm.post_tail >= 8) {
                        if (global_timer_ns() - t_begin > call.timeout_ns) {
                            report_error(status0, UEP_DEV_TIMEOUT_COPY, -1);
                            return;
                        }
                        __nanosleep(50);
                    }
                    sm.post[posted & 7] = flag;
                    __threadfence_block();
                    sm.post_head = ++posted;
                };
                // The index of the next unit is requested one load ahead, so the round trip of the
                // atomic overlaps with the copies instead of sitting in front of every load.
                int pending = atomicAdd(unit_counter, 1);
                Unit cur{};
                int cur_tile = 0;
                bool have_cur = false;
                bool deferred = false;  // `cur` is a forward chunk that had not arrived when it was taken
    #pragma unroll
                for (int s = 0; s < kSyncStages; ++s) owed[s] = nullptr;
                // Two passes over the same ring: first the send units, then the forward units. A CTA must
                // not wait for a ready flag while it still holds send tiles it has loaded but not stored:
                // another CTA (here or on a peer) may be waiting for exactly those. So the first pass stops
                // at the first forward unit and drains, and only the second pass waits; even there the wait
                // blocks only once the ring is empty (a chunk that has not arrived is not allowed to hold
                // up the stores of the chunk in front of it).
                for (int pass = 0; pass < (kR ? 2 : 1); ++pass) {
                    const int limit = pass == 0 ? send_units : total_units;
                    if (pending >= limit && !have_cur) continue;
                    // Everything about the next tile except the load itself: what it is, where it comes from. Done before
                    // the wait for the stage to become free, so that this arithmetic hides behind the stores in flight.
                    const uint8_t* next_src = nullptr;
                    uint32_t next_bytes16 = 0;
                    auto prepare_load = [&](int s) {
                        ring_valid[s] = 0;
                        if (kR && deferred) return;
                        while (!have_cur || cur_tile >= cur.tile_end) {
                            have_cur = false;
                            if (pending >= limit) return;  // keeps `pending`: a claimed forward unit waits for the second pass
                            cur = decode_unit(pending);
                            cur_tile = cur.tile;
                            have_cur = true;
                            pending = atomicAdd(unit_counter, 1);
                            if (kR && cur.kind == 2 && cur_tile < cur.tile_end) {
                                if (!chunk_arrived(cur)) {
                                    deferred = true;
                                    return;
                                }
                                (void)wait_chunk(cur);  // arrived: only the acquire side remains
                            }
                        }
                        TileRef t;
                        t.kind = cur.kind;
                        t.who = cur.who;
                        t.chunk = cur.chunk;
                        t.tile_in_expert = cur_tile;
                        locate_tile<kSyncTile>(t, sh, shard_tiles);
                        ++cur_tile;
                        ring[s] = t;
                        ring_valid[s] = 1;
                        ring_flag[s] = (kR && cur.kind == 1 && cur_tile == cur.tile_end) ? chunk_flag(cur) : nullptr;
                        next_src = tile_source(t);
                        next_bytes16 = static_cast<uint32_t>(t.bytes) & ~15u;
                    };
                    // the load itself, once the stage's previous contents have left
                    auto fire_load = [&](int s) {
                        if (ring_valid[s] && next_bytes16) {
                            mbar_expect_tx(&bars[s], next_bytes16);
                            bulk_load(smem_raw + s * kSyncTile, next_src, next_bytes16, &bars[s]);
                        }
                    };
    #pragma unroll
                    for (int s = 0; s < kSyncStages; ++s) ring_valid[s] = 0;
    #pragma unroll
                    for (int s = 0; s < kSyncStages - 1; ++s) {
                        prepare_load(s);
                        fire_load(s);
                    }
                    int k = 0;
                    while (true) {
                        const int s = k % kSyncStages;
                        if (!ring_valid[s]) {
                            if (!(kR && deferred)) break;  // units are handed out in order: nothing is left for this pass
                            // the ring is empty: now the wait for the chunk may block
                            bulk_wait_read<0>();
                            if (!wait_chunk(cur)) ok = false;
                            deferred = false;
                            for (int j = 0; j < kSyncStages - 1; ++j) {
                                prepare_load((k + j) % kSyncStages);
                                fire_load((k + j) % kSyncStages);
                            }
                            if (!ring_valid[s]) break;
                        }
                        const TileRef t = ring[s];
                        const uint32_t bytes16 = static_cast<uint32_t>(t.bytes) & ~15u;
                        if (bytes16) {
                            if (!mbar_wait(&bars[s], (phase_bits >> s) & 1u, call.timeout_ns)) {
                                ok = false;
                                report_error(status0, UEP_DEV_TIMEOUT_COPY, k);
                                break;  // the stage stays marked valid: its load is waited for below
                            }
                            phase_bits ^= 1u << s;
                        }
                        ring_valid[s] = 0;
                        int first, count;
                        dest_range(t, first, count);
                        for (int d = first; d < first + count; ++d) {
                            uint8_t* dst = dest_addr(t, d);
                            if (dst == nullptr) continue;
                            if (bytes16) bulk_store(dst, smem_raw + s * kSyncTile, bytes16);
                            if (static_cast<uint32_t>(t.bytes) != bytes16) {  // up to 15 trailing bytes of a shard
                                const uint8_t* src = tile_source(t);
                                for (int b = bytes16; b < t.bytes; ++b) dst[b] = __ldcg(src + b);
                            }
                        }
                        bulk_commit();
                        // A chunk's ready flag may go out once its stores are complete, not merely read: the flag
                        // owed for the tile stored kFlagDepth iterations ago is due now (groups complete in order,
                        // so the earlier tiles of that chunk are complete as well).
                        if (kR) {
                            const int ds = (k + kSyncStages - kFlagDepth) % kSyncStages;
                            uint64_t* due = owed[ds];
                            owed[ds] = nullptr;
                            owed[s] = ring_flag[s];
                            if (due != nullptr) {
                                bulk_wait_all<kFlagDepth>();
                                post_flag(due);
                            }
                        }
                        // refill the stage that the previous tile's stores have finished reading
                        const int refill = (k + kSyncStages - 1) % kSyncStages;
                        prepare_load(refill);
                        if (k >= 1) bulk_wait_read<1>();
                        fire_load(refill);
                        ++k;
                    }
                    if (pass == 0) stamp(2);
                    bulk_wait_all<0>();
                    if (kR) {
    #pragma unroll
                        for (int s = 0; s < kSyncStages; ++s) {
                            if (owed[s] != nullptr) post_flag(owed[s]);
                            owed[s] = nullptr;
                        }
                    }
                    if (!ok) {
                        // loads still in flight must land before the shared memory is released or reused
                        for (int s = 0; s < kSyncStages; ++s) {
                            if (ring_valid[s] && (static_cast<uint32_t>(ring[s].bytes) & ~15u)) {
                                mbar_wait(&bars[s], (phase_bits >> s) & 1u, call.timeout_ns);
                            }
                        }
                        break;
                    }
                }
                if (kR) {
                    __threadfence_block();
                    sm.post_done = 1;
                }
                stamp(3);
            } else if (kR && tid == 32) {
                // ---- posting thread: raises the ready flags the issuing thread hands over ------------------
                int tail = 0;
                uint64_t t_idle = global_timer_ns();  // since the last flag: the issuing thread's own waits are bounded,
                                                      // so is this one
                while (true) {
                    const int head = sm.post_head;
                    if (tail < head) {
                        t_idle = global_timer_ns();
                        // one fence for every flag handed over so far: a system-scope fence takes about a link
                        // round trip while the CTA's stores are in flight, the flags queue up behind it
                        __threadfence_block();
                        __threadfence_system();  // the chunks' stores, seen complete by the issuing thread, before the flags
                        for (; tail < head; ++tail) st_relaxed_sys_u64(sm.post[tail & 7], epoch);
                        sm.post_tail = tail;
                    } else if (sm.post_done && tail >= sm.post_head) {
                        break;
                    } else {
                        if (global_timer_ns() - t_idle > 8 * call.timeout_ns) break;
                        __nanosleep(100);
                    }
                }
            }
        } else {
            while (true) {
                __syncthreads();
                if (tid == 0) sm.s_unit = atomicAdd(unit_counter, 1);
                __syncthreads();
                const int u = sm.s_unit;
                if (u >= total_units) break;
                const Unit un = decode_unit(u);
                if (kR && un.kind == 2) {  // forward chunk: one thread waits for the master's delivery
                    if (tid == 0) (void)wait_chunk(un);
                    __syncthreads();
                }
                for (int tile = un.tile; tile < un.tile_end; ++tile) {
                    TileRef t;
                    t.kind = un.kind;
                    t.who = un.who;
                    t.chunk = un.chunk;
                    t.tile_in_expert = tile;
                    locate_tile<kSyncTile>(t, sh, shard_tiles);
                    const uint8_t* src = tile_source(t);
                    int first, count;
                    dest_range(t, first, count);
                    for (int d = first; d < first + count; ++d) {
                        uint8_t* dst = dest_addr(t, d);
                        if (dst != nullptr) copy_plain(src, dst, t.bytes, !kR || t.kind != 2);
                    }
                }
                if (kR && un.kind == 1) {  // every thread's stores, then the chunk's flag
                    uint64_t* flag = chunk_flag(un);
                    __threadfence_system();
                    __syncthreads();
                    if (tid == 0 && flag != nullptr) st_relaxed_sys_u64(flag, epoch);
                }
            }
        }
    };
    if (kRelay && (sm.n_relay != 0 || sm.n_fwd != 0)) {
        run_copy(std::true_type{});
    } else {
        run_copy(std::false_type{});
    }
    // Order this CTA's copies before its ticket. On the bulk-copy path only thread 0 issued
    // copies and it has already waited for their completion.
    // Device scope is enough here: the ticket below hands these writes to the last CTA, whose
    // system-scope fence in front of the flags then covers them (causality is transitive across scopes).
    if (!sm.all_aligned || tid == 0) __threadfence();
    __syncthreads();
    stamp(4);

    // ---- completion: the last CTA of the launch signals the receivers of every hosted rank
    // and waits for their senders
    int* ticket_ptr = call.rank[0]->sync_ticket;
    if (tid == 0) {
        const int ticket = atomicAdd(ticket_ptr, 1);
        if (ticket == static_cast<int>(gridDim.x) - 1) {
            __threadfence();  // the other CTAs' copies, fenced before their tickets, are ordered before the flags
            *ticket_ptr = 0;
            *unit_counter = 0;  // every CTA has stopped taking work
            sm.is_last = 1;
            *call.sync_epoch = epoch;  // this launch's epoch is closed
        }
    }
    __syncthreads();
    stamp(5);
    if (!sm.is_last) return;
    // Every CTA's copies are complete and ordered before this point (fence + ticket above).
    // Ranks hosted by this very launch need no flag at all: the ticket is their proof. Towards
    // ranks on other devices one thread issues a single system-scope fence and then the flags
    // (a fence followed by relaxed stores is a release of everything observed so far); the
    // waits are relaxed polls closed by one acquire fence. The test hook that withholds a rank
    // forces the flags between hosted ranks too, so that the time-out path can be exercised on
    // one device.
    const bool flags_needed = nlocal == 1 || call.withhold_rank >= 0;
    if (flags_needed) {
        if (tid == 0) {
            __threadfence_system();
            for (int lr = 0; lr < nlocal; ++lr) {
                const int me = call.my_rank[lr];
                if (me == call.withhold_rank) continue;
                const RankDev& rk = *call.rank[lr];
                for (int p = 0; p < N; ++p) {
                    if (sm.send_mask[lr][p >> 5] & (1u << (p & 31))) st_relaxed_sys_u64(rk.peer_sync_flags[p] + me, epoch);
                }
            }
        }
        stamp(7);
        unsigned any_recv = 0;
        for (int lr = 0; lr < nlocal; ++lr) any_recv |= sm.recv_mask[lr][0] | sm.recv_mask[lr][1] | sm.recv_mask[lr][2];
        if (any_recv == 0) {  // a rank that only sends has nothing to wait for
            stamp(6);
            return;
        }
        for (int i = tid; i < nlocal * N; i += blockDim.x) {
            const int lr = i / N, p = i % N;
            if (sm.recv_mask[lr][p >> 5] & (1u << (p & 31))) {
                const RankDev& rk = *call.rank[lr];
                if (!wait_flag_ge_relaxed(rk.peer_sync_flags[call.my_rank[lr]] + p, epoch, call.timeout_ns)) {
                    atomicMax(&sm.timeout_peer, p);
                    report_error(rk.status, UEP_DEV_TIMEOUT_SYNC, p);
                }
            }
        }
        __syncthreads();
        if (tid == 0) __threadfence_system();  // acquire side of the flags seen by the polls above
    }
    stamp(6);
}

// Tile / ring geometry. The default keeps 128 KiB of loads and stores in flight per CTA; the
// environment variable UEP_SYNC_GEOMETRY=<tile KiB>x<stages> selects another compiled variant
// (tuning aid).
struct SyncGeometry {
    int tile_kib, stages;
    const void* fn;        // direct fan-out only
    const void* fn_relay;  // with the relay machinery
};
#define UEP_SYNC_VARIANT(T, S)                                                        \
    {T, S, reinterpret_cast<const void*>(weight_sync_kernel<T * 1024, S, false>), \
     reinterpret_cast<const void*>(weight_sync_kernel<T * 1024, S, true>)}
const SyncGeometry kGeometries[] = {UEP_SYNC_VARIANT(32, 4), UEP_SYNC_VARIANT(16, 4), UEP_SYNC_VARIANT(16, 8),
                                    UEP_SYNC_VARIANT(8, 8)};
#undef UEP_SYNC_VARIANT

const SyncGeometry& sync_geometry() {
    static const SyncGeometry* chosen = nullptr;
    if (chosen == nullptr) {
        chosen = &kGeometries[0];
        if (const char* env = std::getenv("UEP_SYNC_GEOMETRY")) {
            int t = 0, st = 0;
            if (std::sscanf(env, "%dx%d", &t, &st) == 2) {
                for (const auto& g : kGeometries) {
                    if (g.tile_kib == t && g.stages == st) chosen = &g;
                }
            }
        }
    }
    return *chosen;
}

size_t sync_smem_bytes(const SyncGeometry& g) {
    return static_cast<size_t>(g.stages) * g.tile_kib * 1024 + sizeof(SyncShared);
}

}  // namespace

int weight_sync_max_ctas_per_rank(int nlocal, int num_sms) {
    // CTAs that fit one wave: shared memory bounds the CTAs per SM; hosted ranks share the device
    const size_t smem = sync_smem_bytes(sync_geometry()) + 1024;
    int per_sm = static_cast<int>((227 * 1024) / smem);
    per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
    const int per = num_sms * per_sm / (nlocal > 0 ? nlocal : 1);
    return per < 1 ? 1 : per;
}

int weight_sync_tile_bytes() { return sync_geometry().tile_kib * 1024; }

cudaError_t launch_weight_sync(const SyncCall& call, cudaStream_t stream) {
    const SyncGeometry& g = sync_geometry();
    const size_t smem = sync_smem_bytes(g);
    // two ranks: an expert has at most one replica away from its master, nothing can be relayed; the
    // compact kernel is the same on every rank because N is
    const bool relay = call.relay_min_replicas > 0 && call.N > 2;
    const void* fn = relay ? g.fn_relay : g.fn;
    static const void* attr_set_for[2] = {nullptr, nullptr};
    if (attr_set_for[relay] != fn) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        attr_set_for[relay] = fn;
    }
    // Hosted ranks pool their work over all CTAs. Without relaying, the only waits are those of the
    // last CTA, on flags that peers on other devices write. With relaying, CTAs that forward wait for
    // CTAs that send; when both are in this launch (ranks hosted together) they must be co-resident,
    // which a cooperative launch guarantees.
    const dim3 grid(call.nlocal * call.ctas_per_rank), block(kSyncThreads);
    count_launch();
    SyncCall copy = call;
    void* args[] = {&copy};
    cudaError_t e = (call.nlocal > 1 && relay) ? cudaLaunchCooperativeKernel(fn, grid, block, args, smem, stream)
                                               : cudaLaunchKernel(fn, grid, block, args, smem, stream);
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace uep
