// Kernel 3 — weight_sync: every replicated local master expert (weights and scales) is
// pushed into the replica slots of its peers, straight from the stored plan.
//
// The reference first builds a task list with a single-thread kernel and then runs a
// thread-copy kernel (16-byte loads, streaming stores) when the NVLink domain has at most
// 8 ranks, or a two-stage bulk-copy kernel above that (csrc/kernels/weight_sync.cu:205-522,
// 714-775, 782-986 of the reference). Here there is no task list and one kernel:
//   * every CTA derives the send list from the plan rows of this rank's masters
//     (l2p / lcnts) with a block-wide scan, a few hundred nanoseconds of work;
//   * one elected thread per CTA drives a 4-stage ring of 32 KiB bulk copies: the tile is
//     read from local HBM once (cp.async.bulk global->shared, mbarrier) and stored to each
//     destination slot (cp.async.bulk shared->global, peer memory over NVLink); loads run
//     up to three tiles ahead of the stores;
//   * tiles are interleaved over masters so that concurrent CTAs feed different peers; when
//     several ranks are hosted on one device their tiles form one pool shared by all CTAs;
//   * the CTA that finishes last publishes "rank r has delivered epoch e" to the ranks it
//     sent to (system-scope release) and waits, bounded, for the same word from the ranks
//     that send to it. When the kernel ends, this rank's replica slots are complete.
//     No CTA waits for another CTA of the same launch.
// Pointers or sizes that are not multiples of 16 bytes take a plain vector/byte copy path.

#include <cstdio>
#include <cstdlib>

#include "internal.h"

namespace uep {

namespace {

constexpr int kSyncThreads = 128;
constexpr int kSyncTileDefault = 32 * 1024;
constexpr int kSyncStagesDefault = 4;
constexpr int kMaxSends = kMaxExportsPerDomain;  // replicas of one rank's masters never exceed G*R <= 512

struct SyncShared {
    int n_active;          // masters (of all hosted ranks) that have replicas
    int total_reps;        // sum of their replica counts
    int all_aligned;       // every source pointer 16-byte aligned
    int is_last;
    unsigned send_mask[kMaxLocalRanks][3];  // per hosted rank: ranks it sends to
    unsigned recv_mask[kMaxLocalRanks][3];  // per hosted rank: ranks that send to it
    int timeout_peer;
    unsigned long long epoch;  // opened by the last CTA of the launch
    short rep_start[kMaxExpertsPerDomain + 1];  // [n_active+1] offsets into dst_*
    // Addresses are resolved once per CTA: the issuing thread must not chase pointers
    // through global memory for every 32 KiB tile.
    const uint8_t* src[kMaxExpertsPerDomain][4];  // [n_active][shard] master shard base
    uint8_t* dst_weight[kMaxSends];               // replica slot base in the peer's weight buffer (null: skip)
    uint8_t* dst_scale[kMaxSends];                // replica slot base in the peer's scale buffer
    // replica buffer bases of every (hosted rank, peer): nlocal * N entries (at most 72: several
    // hosted ranks mean a simulated group of at most 8)
    uint8_t* peer_weight[kMaxPeers];
    uint8_t* peer_scale[kMaxPeers];
};

struct TileRef {
    int active;      // index into active_master
    int shard;       // 0..3
    int64_t offset;  // byte offset inside the shard
    int bytes;       // bytes of this tile
};

template <int kSyncTile>
__device__ __forceinline__ TileRef decode_tile(int64_t idx, int n_active, const ShardLayout& sh, const int* shard_tiles) {
    TileRef t;
    const int idx32 = static_cast<int>(idx);  // tile counts fit 32 bits (checked on the host side by construction)
    t.active = idx32 % n_active;
    int tile = idx32 / n_active;
    t.shard = 0;
    while (t.shard < sh.num_shards - 1 && tile >= shard_tiles[t.shard]) {
        tile -= shard_tiles[t.shard];
        ++t.shard;
    }
    t.offset = static_cast<int64_t>(tile) * kSyncTile;
    const int64_t left = sh.bytes[t.shard] - t.offset;
    t.bytes = static_cast<int>(left < kSyncTile ? left : kSyncTile);
    return t;
}

__device__ __forceinline__ uint8_t* dest_addr(const SyncShared& sm, const ShardLayout& sh, int shard, int rep) {
    return (shard < 2 ? sm.dst_weight[rep] : sm.dst_scale[rep]) + sh.slot_offset[shard];
}

__device__ void copy_plain(const uint8_t* src, uint8_t* dst, int bytes) {
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    int done = 0;
    if (vec) {
        const int nvec = bytes / 16;
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
            st_global_cs_v4(dst + static_cast<int64_t>(i) * 16, ld_global_nc_v4(src + static_cast<int64_t>(i) * 16));
        }
        done = nvec * 16;
    }
    for (int i = done + threadIdx.x; i < bytes; i += blockDim.x) dst[i] = src[i];
}

template <int kSyncTile, int kSyncStages>
__global__ void __launch_bounds__(kSyncThreads) weight_sync_kernel(SyncCall call) {
    extern __shared__ __align__(128) char smem_raw[];  // kSyncStages * kSyncTile
    __shared__ SyncShared sm;
    __shared__ __align__(8) uint64_t bars[kSyncStages];
    __shared__ int shard_tiles[4];

    const ShardLayout& sh = call.shards;
    const int M = call.M, R = call.R, D = call.D, Lp = M + R, N = call.N, nlocal = call.nlocal;
    const int tid = threadIdx.x;
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
        sm.timeout_peer = -1;
        for (int s = 0; s < 4; ++s) shard_tiles[s] = s < sh.num_shards ? static_cast<int>((sh.bytes[s] + kSyncTile - 1) / kSyncTile) : 0;
        for (int s = 0; s < kSyncStages; ++s) mbar_init(&bars[s], 1);
        fence_mbar_init();
    }
    for (int i = tid; i < kMaxLocalRanks * 3; i += blockDim.x) {
        sm.send_mask[i / 3][i % 3] = 0;
        sm.recv_mask[i / 3][i % 3] = 0;
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
    if (tid < nlocal * N) {
        const RankDev& rk = *call.rank[tid / N];
        pre_pw = rk.peer_replica_weight[tid % N];
        pre_ps = rk.peer_replica_scale[tid % N];
    }
    int pre_owner = -1;
    if (tid < nlocal * R) pre_owner = call.plan[tid / R].p2l[call.my_rank[tid / R] * Lp + M + tid % R];
    if (tid < nlocal * N) {
        sm.peer_weight[tid] = pre_pw;
        sm.peer_scale[tid] = pre_ps;
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
        __shared__ int w_a[kSyncThreads / 32], w_r[kSyncThreads / 32];
        if (lane == 31) {
            w_a[warp] = a_incl;
            w_r[warp] = r_incl;
        }
        __syncthreads();
        int a_off = sm.n_active, r_off = sm.total_reps;
        for (int w = 0; w < warp; ++w) {
            a_off += w_a[w];
            r_off += w_r[w];
        }
        if (act) {
            const int ai = a_off + a_incl - 1;
            const int rs = r_off + r_incl - reps;
            sm.rep_start[ai] = static_cast<short>(rs);
            const int l = me * M + m;
            auto place = [&](int j, int phys) {
                const int drank = phys / Lp, dslot = phys % Lp - M;
                if (phys < 0 || drank >= N || dslot < 0 || dslot >= R) {  // never store outside a slot table
                    report_error(rk.status, UEP_DEV_BAD_PLAN, l);
                    sm.dst_weight[rs + j] = nullptr;
                    sm.dst_scale[rs + j] = nullptr;
                } else {
                    atomicOr(&sm.send_mask[lr][drank >> 5], 1u << (drank & 31));
                    sm.dst_weight[rs + j] = sm.peer_weight[lr * N + drank] + static_cast<int64_t>(dslot) * sh.weight_slot_stride;
                    sm.dst_scale[rs + j] = sm.peer_scale[lr * N + drank] + static_cast<int64_t>(dslot) * sh.scale_slot_stride;
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
    if (tid == 0) sm.rep_start[sm.n_active] = static_cast<short>(sm.total_reps < kMaxSends ? sm.total_reps : kMaxSends);
    for (int i = tid; i < nlocal * R; i += blockDim.x) {
        const int lr = i / R, slot = i % R;
        const int me = call.my_rank[lr];
        const int l = i == tid ? pre_owner : call.plan[lr].p2l[me * Lp + M + slot];
        if (l >= 0) {
            const int src = l / M;
            if (src >= 0 && src < N && src != me) atomicOr(&sm.recv_mask[lr][src >> 5], 1u << (src & 31));
        }
    }
    __syncthreads();

    stamp(1);
    // ---- copy -------------------------------------------------------------------------
    int tiles_per_expert = 0;
    for (int s = 0; s < sh.num_shards; ++s) tiles_per_expert += shard_tiles[s];
    const int total_tiles = sm.n_active * tiles_per_expert;
    DeviceStatus* status0 = call.rank[0]->status;
    // Tiles are handed out by an atomic counter: CTAs that run on busy SMs (the reroute and the
    // model's own kernels run next to this one) simply take fewer, and replica counts that differ
    // between masters cannot leave some CTAs with several times the work of others.
    int* tile_counter = call.rank[0]->sync_ticket + 1;

    if (sm.all_aligned) {
        if (tid == 0) {
            int ring_tile[kSyncStages];  // tile index held by each stage (>= total_tiles: none)
            // The index of the next tile is requested one load ahead, so the round trip of the
            // atomic overlaps with the copies instead of sitting in front of every load.
            int pending = atomicAdd(tile_counter, 1);
            auto issue_load = [&](int s) {
                const int idx = pending;
                pending = idx < total_tiles ? atomicAdd(tile_counter, 1) : idx;
                ring_tile[s] = idx;
                if (idx >= total_tiles) return;
                const TileRef t = decode_tile<kSyncTile>(idx, sm.n_active, sh, shard_tiles);
                const uint8_t* src = sm.src[t.active][t.shard] + t.offset;
                const uint32_t bytes16 = static_cast<uint32_t>(t.bytes) & ~15u;
                if (bytes16) {
                    mbar_expect_tx(&bars[s], bytes16);
                    bulk_load(smem_raw + s * kSyncTile, src, bytes16, &bars[s]);
                }
            };
#pragma unroll
            for (int s = 0; s < kSyncStages; ++s) ring_tile[s] = total_tiles;
#pragma unroll
            for (int s = 0; s < kSyncStages - 1; ++s) issue_load(s);
            uint32_t phase_bits = 0;  // bit s: parity the next wait on stage s expects
            bool ok = true;
            int k = 0;
            while (true) {
                const int s = k % kSyncStages;
                const int idx = ring_tile[s];
                if (idx >= total_tiles) break;  // indices are handed out in order: nothing is left
                const TileRef t = decode_tile<kSyncTile>(idx, sm.n_active, sh, shard_tiles);
                const uint32_t bytes16 = static_cast<uint32_t>(t.bytes) & ~15u;
                if (bytes16) {
                    if (!mbar_wait(&bars[s], (phase_bits >> s) & 1u, call.timeout_ns)) {
                        ok = false;
                        break;
                    }
                    phase_bits ^= 1u << s;
                }
                const int r0 = sm.rep_start[t.active], r1 = sm.rep_start[t.active + 1];
                for (int r = r0; r < r1; ++r) {
                    if (sm.dst_weight[r] == nullptr) continue;
                    uint8_t* dst = dest_addr(sm, sh, t.shard, r) + t.offset;
                    if (bytes16) bulk_store(dst, smem_raw + s * kSyncTile, bytes16);
                    if (static_cast<uint32_t>(t.bytes) != bytes16) {  // up to 15 trailing bytes of a shard
                        const uint8_t* src = sm.src[t.active][t.shard] + t.offset;
                        for (int b = bytes16; b < t.bytes; ++b) dst[b] = src[b];
                    }
                }
                bulk_commit();
                // refill the stage that the previous tile's stores have finished reading
                const int refill = (k + kSyncStages - 1) % kSyncStages;
                if (k >= 1) bulk_wait_read<1>();
                issue_load(refill);
                ++k;
            }
            stamp(2);
            bulk_wait_all<0>();
            stamp(3);
            if (!ok) {
                report_error(status0, UEP_DEV_TIMEOUT_COPY, k);
                // loads still in flight must land before the shared memory is released
                for (int j = 0; j < kSyncStages; ++j) {
                    const int s = (k + j) % kSyncStages;
                    if (ring_tile[s] < total_tiles) mbar_wait(&bars[s], (phase_bits >> s) & 1u, call.timeout_ns);
                }
            }
        }
    } else {
        __shared__ int s_tile;
        while (true) {
            __syncthreads();
            if (tid == 0) s_tile = atomicAdd(tile_counter, 1);
            __syncthreads();
            const int idx = s_tile;
            if (idx >= total_tiles) break;
            const TileRef t = decode_tile<kSyncTile>(idx, sm.n_active, sh, shard_tiles);
            const uint8_t* src = sm.src[t.active][t.shard] + t.offset;
            const int r0 = sm.rep_start[t.active], r1 = sm.rep_start[t.active + 1];
            for (int r = r0; r < r1; ++r) {
                if (sm.dst_weight[r] == nullptr) continue;
                copy_plain(src, dest_addr(sm, sh, t.shard, r) + t.offset, t.bytes);
            }
        }
    }
    // Order this CTA's copies before its ticket. On the bulk-copy path only thread 0 issued
    // copies and it has already waited for their completion.
    // Device scope is enough here: the ticket below hands these writes to the last CTA, whose
    // system-scope release of the flags then covers them (causality is transitive across scopes).
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
            *tile_counter = 0;  // every CTA has stopped taking tiles
            sm.is_last = 1;
            // ranks hosted together share the first one's counter: they always run in the same launches
            sm.epoch = call.rank[0]->epochs[1] + 1;
            call.rank[0]->epochs[1] = sm.epoch;
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
                    if (sm.send_mask[lr][p >> 5] & (1u << (p & 31))) st_relaxed_sys_u64(rk.peer_sync_flags[p] + me, sm.epoch);
                }
            }
        }
        stamp(7);
        for (int i = tid; i < nlocal * N; i += blockDim.x) {
            const int lr = i / N, p = i % N;
            if (sm.recv_mask[lr][p >> 5] & (1u << (p & 31))) {
                const RankDev& rk = *call.rank[lr];
                if (!wait_flag_ge_relaxed(rk.peer_sync_flags[call.my_rank[lr]] + p, sm.epoch, call.timeout_ns)) {
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
    const void* fn;
};
const SyncGeometry kGeometries[] = {
    {32, 4, reinterpret_cast<const void*>(weight_sync_kernel<32 * 1024, 4>)},
    {16, 4, reinterpret_cast<const void*>(weight_sync_kernel<16 * 1024, 4>)},
    {16, 8, reinterpret_cast<const void*>(weight_sync_kernel<16 * 1024, 8>)},
    {8, 8, reinterpret_cast<const void*>(weight_sync_kernel<8 * 1024, 8>)},
    {32, 6, reinterpret_cast<const void*>(weight_sync_kernel<32 * 1024, 6>)},
    {64, 3, reinterpret_cast<const void*>(weight_sync_kernel<64 * 1024, 3>)},
};

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

}  // namespace

int weight_sync_max_ctas_per_rank(int nlocal, int num_sms) {
    // CTAs that fit one wave: shared memory bounds the CTAs per SM; hosted ranks share the device
    const SyncGeometry& g = sync_geometry();
    const int smem = g.tile_kib * 1024 * g.stages + 30 * 1024;
    int per_sm = (227 * 1024) / smem;
    per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
    const int per = num_sms * per_sm / (nlocal > 0 ? nlocal : 1);
    return per < 1 ? 1 : per;
}

cudaError_t launch_weight_sync(const SyncCall& call, cudaStream_t stream) {
    const SyncGeometry& g = sync_geometry();
    const size_t smem = static_cast<size_t>(g.stages) * g.tile_kib * 1024;
    static const void* attr_set_for = nullptr;
    if (attr_set_for != g.fn) {
        cudaError_t e = cudaFuncSetAttribute(g.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        attr_set_for = g.fn;
    }
    // Hosted ranks pool their tiles over all CTAs. The only waits are those of the last CTA,
    // on flags that peers on other devices (or, for hosted ranks, this very CTA) write.
    const dim3 grid(call.nlocal * call.ctas_per_rank), block(kSyncThreads);
    count_launch();
    SyncCall copy = call;
    void* args[] = {&copy};
    cudaError_t e = cudaLaunchKernel(g.fn, grid, block, args, smem, stream);
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace uep
