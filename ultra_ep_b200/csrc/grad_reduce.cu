// Kernel 4 — replica Wgrad reduce: for every local master that has replicas,
//     master = ((master + g_1) + g_2) + ...      (fp32, replicas in plan slot order)
// where g_j is read from the peer that hosts replica j, and every consumed replica region
// is overwritten with zeros. The order is fixed, so the result is bit-exact and equal to
// the reference's deterministic kernel (csrc/kernels/grad_reduce.cu:289-394 of the
// reference; task order :41-69).
//
// The reference builds a task list with a single-thread kernel, then per tile loads one
// replica sub-tile at a time through a single shared-memory buffer (load, wait, add, zero
// with per-thread stores, repeat). Here:
//   * no task list: every CTA derives the pull list from the plan rows with a block scan;
//   * a consumed replica region is not zeroed over the link. Pulling 75 MB and pushing 75 MB of
//     zeros back at the same time measured 450 GB/s against 660 GB/s for the pull alone (the link
//     is full duplex, but one kernel reading from a peer and writing to it through the same SMs
//     did not get both directions at full rate). Instead the rank that HOSTS a replica
//     zeroes it in its own memory: the master's launch reports its progress in 16 segments
//     (a counter per segment that every CTA bumps when it has consumed its items of the segment;
//     the CTA that completes a segment stores "epoch, segments done" into a flag word on every
//     rank it pulls from), and the host rank's launch, once its own pulls are done, clears each
//     segment of its used slots as soon as the flag allows, from a warp of its own that runs beside
//     the pulls (bulk stores from a zero tile into local memory);
//   * roles are split. Two producer warps (one lane each) only issue bulk loads: one feeds the
//     ring of replica tiles, the other the ring of master tiles. Eight
//     consumer warps wait on a stage's "full" mbarrier, add it into accumulators in registers
//     (16 floats per thread per tile) and arrive on its "empty" mbarrier: there is no CTA-wide
//     barrier per stage;
//   * two rings of 16 KiB stages: nine for the REMOTE replica tiles (144 KiB in flight per CTA,
//     6 MB over the default 42 CTAs: the bandwidth-delay product of NVLink reads under load is
//     several MB) and three for the local master tiles. In one common ring a master tile would
//     hold a stage as long as a remote tile does, and with one replica per master half of the
//     ring would be taken away from the remote loads;
//   * tiles are interleaved over masters so that concurrent CTAs pull from different peers.
// The CTA budget (SMs used while the backward pass runs next to it) is the caller's knob
// (grad_reduce_num_sms); each CTA holds about 215 KiB of shared memory.

#include "internal.h"

namespace uep {

namespace {

constexpr int kReduceConsumers = 256;
constexpr int kReduceThreads = kReduceConsumers + 128;  // eight consumer warps, two producer warps (replica ring, master ring),
                                                        // one clearing warp, one reporting warp
constexpr int kReduceZeroBytes = 8192;                 // zero tile the clearing warp stores from
constexpr int kReduceTileElems = 4096;                 // 16 KiB
constexpr int kReduceTileBytes = kReduceTileElems * 4;
constexpr int kReduceStages = 9;                       // ring of remote replica tiles
constexpr int kMasterStages = 3;                       // ring of local master tiles
constexpr int kReduceVecPerThread = kReduceTileElems / 4 / kReduceConsumers;  // float4 per thread per tile
constexpr int kMaxPulls = kMaxExportsPerDomain;
constexpr int kMaxOwned = 64;  // used replica slots of the hosted ranks

struct ReduceShared {
    int n_active, total_reps, vector_ok;
    volatile int error;
    int n_owned, s_go;
    volatile long long done_items;                 // items of this CTA whose replica tiles have all been consumed
    volatile int pull_finished;                    // the pull phase of this CTA is over (all items, or given up)
    unsigned long long epoch;
    int w_a[kReduceThreads / 32], w_r[kReduceThreads / 32];
    unsigned pull_mask[kMaxLocalRanks][3];         // per hosted rank: ranks it pulls replica gradients from
    float* own_base[kMaxOwned];                    // used local replica slots: base of the slot ...
    const uint64_t* own_flag[kMaxOwned];           // ... and the progress word its master's rank writes
    short rep_start[kMaxExpertsPerDomain + 1];
    float* rep_base[kMaxPulls];                    // replica slot base in the peer's grad buffer (null: skip)
    float* master[kMaxExpertsPerDomain][2];        // [n_active][fc1, fc2] master gradient base
    __align__(8) uint64_t full[kReduceStages];     // a remote tile has landed in the stage
    __align__(8) uint64_t empty[kReduceStages];    // all eight consumer warps are done with the stage
    __align__(8) uint64_t m_full[kMasterStages];   // the same for the ring of master tiles
    __align__(8) uint64_t m_empty[kMasterStages];
};

struct ReduceItem {
    int active;       // index into active_master
    int shard;        // 0 fc1, 1 fc2
    int64_t offset;   // element offset inside the shard
    int elems;
};

__device__ __forceinline__ ReduceItem decode_item(int64_t idx, int n_active, int64_t fc1_numel, int64_t fc2_numel,
                                                  int tiles_fc1) {
    ReduceItem it;
    const int idx32 = static_cast<int>(idx);
    it.active = idx32 % n_active;
    const int tile = idx32 / n_active;
    it.shard = tile < tiles_fc1 ? 0 : 1;
    const int t = it.shard == 0 ? tile : tile - tiles_fc1;
    it.offset = static_cast<int64_t>(t) * kReduceTileElems;
    const int64_t left = (it.shard == 0 ? fc1_numel : fc2_numel) - it.offset;
    it.elems = static_cast<int>(left < kReduceTileElems ? left : kReduceTileElems);
    return it;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__global__ void __launch_bounds__(kReduceThreads, 1) grad_reduce_kernel(ReduceCall call) {
    extern __shared__ __align__(128) char smem_raw[];  // kReduceStages replica tiles, kMasterStages master tiles, the zero tile
    __shared__ ReduceShared sm;

    const int M = call.M, R = call.R, D = call.D, Lp = M + R, N = call.N, nlocal = call.nlocal;
    const int tid = threadIdx.x;
    const int64_t fc1 = call.fc1_numel, fc2 = call.fc2_numel, total_numel = fc1 + fc2;
    char* master_ring = smem_raw + kReduceStages * kReduceTileBytes;
    char* zero_tile = master_ring + kMasterStages * kReduceTileBytes;
    DeviceStatus* status0 = call.rank[0]->status;
    auto stamp = [&](int slot) {
        if (call.trace != nullptr && tid == 0) call.trace[blockIdx.x * 8 + slot] = global_timer_ns();
    };
    stamp(0);

    if (tid == 0) {
        sm.n_active = 0;
        sm.total_reps = 0;
        sm.vector_ok = ((fc1 & 3) == 0 && (fc2 & 3) == 0) ? 1 : 0;
        sm.error = 0;
        sm.n_owned = 0;
        sm.done_items = 0;
        sm.pull_finished = 0;
        sm.epoch = *call.reduce_epoch + 1;  // ranks hosted together share the first one's counter
        for (int s = 0; s < kReduceStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], kReduceConsumers / 32);
        }
        for (int s = 0; s < kMasterStages; ++s) {
            mbar_init(&sm.m_full[s], 1);
            mbar_init(&sm.m_empty[s], kReduceConsumers / 32);
        }
        fence_mbar_init();
    }
    for (int i = tid; i < kMaxLocalRanks * 3; i += blockDim.x) sm.pull_mask[i / 3][i % 3] = 0;
    for (int i = tid; i < kReduceZeroBytes / 4; i += blockDim.x) reinterpret_cast<float*>(zero_tile)[i] = 0.f;
    fence_proxy_async_smem();
    __syncthreads();

    // pull list: masters of the hosted ranks with replicas, and where each replica lives.
    // Hosted ranks pool their tiles over all CTAs of the launch.
    const int total_masters = nlocal * M;
    for (int g0 = 0; g0 < total_masters; g0 += blockDim.x) {
        const int gm = g0 + tid;
        const int lr = gm < total_masters ? gm / M : 0;
        const int m = gm < total_masters ? gm % M : 0;
        const RankDev& rk = *call.rank[lr];
        const PlanPtrs& plan = call.plan[lr];
        const int me = call.my_rank[lr];
        int reps = 0;
        if (gm < total_masters) {
            reps = plan.lcnts[me * M + m] - 1;
            reps = reps < 0 ? 0 : (reps > D - 1 ? D - 1 : reps);
        }
        const int act = reps > 0 ? 1 : 0;
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
            for (int j = 0; j < reps && rs + j < kMaxPulls; ++j) {
                const int phys = plan.l2p[static_cast<int64_t>(l) * D + 1 + j];
                const int prank = phys / Lp, pslot = phys % Lp - M;
                if (phys < 0 || prank >= N || pslot < 0 || pslot >= R) {
                    report_error(rk.status, UEP_DEV_BAD_PLAN, l);
                    sm.rep_base[rs + j] = nullptr;
                } else {
                    sm.rep_base[rs + j] = rk.peer_replica_grad[prank] + static_cast<int64_t>(pslot) * total_numel;
                    atomicOr(&sm.pull_mask[lr][prank >> 5], 1u << (prank & 31));
                }
            }
            const uintptr_t p1 = static_cast<uintptr_t>(call.fc1_grad_ptrs[lr][m]);
            const uintptr_t p2 = static_cast<uintptr_t>(call.fc2_grad_ptrs[lr][m]);
            sm.master[ai][0] = reinterpret_cast<float*>(p1);
            sm.master[ai][1] = reinterpret_cast<float*>(p2);
            if ((p1 & 15u) || (p2 & 15u)) atomicAnd(&sm.vector_ok, 0);
        }
        __syncthreads();
        if (tid == blockDim.x - 1) {
            sm.n_active = a_off + a_incl;
            sm.total_reps = r_off + r_incl;
        }
        __syncthreads();
    }
    if (tid == 0) sm.rep_start[sm.n_active] = static_cast<short>(sm.total_reps < kMaxPulls ? sm.total_reps : kMaxPulls);
    // The used replica slots of the hosted ranks: this launch clears them once their master's rank has pulled them.
    {
        const int i = tid;
        const bool in = i < nlocal * R && nlocal * R <= kMaxOwned;
        int l = -1;
        if (in) l = call.plan[i / R].p2l[call.my_rank[i / R] * Lp + M + i % R];
        const bool used = in && l >= 0 && l / M < N;
        const unsigned has = __ballot_sync(kFullMask, used);
        const int lane = tid & 31, warp = tid >> 5;
        if (lane == 0) sm.w_a[warp] = __popc(has);
        __syncthreads();
        int f = __popc(has & ((1u << lane) - 1u));
        for (int w = 0; w < warp; ++w) f += sm.w_a[w];
        if (used) {
            const int lr = i / R, me = call.my_rank[lr];
            const RankDev& rk = *call.rank[lr];
            sm.own_base[f] = rk.peer_replica_grad[me] + static_cast<int64_t>(i % R) * total_numel;
            sm.own_flag[f] = rk.peer_reduce_flags[me] + l / M;
        }
        if (tid == 0) {
            int n = 0;
            for (int w = 0; w < kReduceThreads / 32; ++w) n += sm.w_a[w];
            sm.n_owned = n;
        }
    }
    __syncthreads();
    stamp(1);

    const int n_active = sm.n_active;
    const uint64_t epoch = sm.epoch;
    const int tiles_fc1 = static_cast<int>((fc1 + kReduceTileElems - 1) / kReduceTileElems);
    const int tiles_fc2 = static_cast<int>((fc2 + kReduceTileElems - 1) / kReduceTileElems);
    const int tiles_total = tiles_fc1 + tiles_fc2;
    const int64_t total_items = static_cast<int64_t>(n_active) * tiles_total;
    const int64_t first = blockIdx.x, step = gridDim.x;
    const int64_t count = first < total_items ? (total_items - first + step - 1) / step : 0;
    // segment s covers the tiles [seg_end(s-1), seg_end(s)) of an expert; items come tile after tile
    auto seg_end = [&](int s) -> int { return static_cast<int>(static_cast<int64_t>(s + 1) * tiles_total / kReduceSegments); };

    // One thread per CTA reports progress: `done` of this CTA's items are consumed. When the CTA has passed a
    // segment it bumps that segment's counter; the CTA that completes the count tells every rank the launch pulls
    // from, and the one that completes the last segment closes the epoch.
    int seg_next = 0;
    auto report_progress = [&](int64_t done) {
        while (seg_next < kReduceSegments) {
            const int64_t boundary = static_cast<int64_t>(seg_end(seg_next)) * n_active;  // first item index behind the segment
            if (done < count && first + done * step < boundary) break;
            __threadfence();
            int* counters = call.rank[0]->reduce_counters;
            if (atomicAdd(&counters[seg_next], 1) == static_cast<int>(gridDim.x) - 1) {
                counters[seg_next] = 0;
                const uint64_t word = epoch * kReduceFlagRadix + static_cast<uint64_t>(seg_next + 1);
                for (int lr = 0; lr < nlocal; ++lr) {
                    const RankDev& rk = *call.rank[lr];
                    for (int p = 0; p < N; ++p) {
                        if (sm.pull_mask[lr][p >> 5] & (1u << (p & 31))) st_relaxed_sys_u64(rk.peer_reduce_flags[p] + call.my_rank[lr], word);
                    }
                }
                if (seg_next == kReduceSegments - 1) *call.reduce_epoch = epoch;
            }
            ++seg_next;
        }
    };

    auto replica_ptr = [&](const ReduceItem& it, int r) -> float* {
        return sm.rep_base[r] + (it.shard == 0 ? 0 : fc1) + it.offset;
    };
    auto master_ptr = [&](const ReduceItem& it) -> float* { return sm.master[it.active][it.shard] + it.offset; };

    // ---- clearing warp: the used replica slots hosted here, segment by segment as their master's rank releases
    //      them; runs beside the pulls of this CTA (every CTA of the launch takes every gridDim-th tile) ----------
    if (tid >= kReduceConsumers + 96) {
        // ---- reporting warp: keeps the atomics and the flag stores of the progress report off the threads that
        //      feed the rings (each costs a round trip to memory) -----------------------------------------------
        if (tid == kReduceConsumers + 96) {
            // waits for threads of its own CTA only, whose waits are all bounded; bounded itself all the same
            const uint64_t t_begin = global_timer_ns();
            while (true) {
                const int fin = sm.pull_finished;
                const long long done = fin ? static_cast<long long>(count) : sm.done_items;
                report_progress(done);
                if (fin || seg_next >= kReduceSegments) break;
                if (global_timer_ns() - t_begin > 4 * call.timeout_ns) {
                    report_error(status0, UEP_DEV_TIMEOUT_COPY, blockIdx.x);
                    break;
                }
                __nanosleep(200);
            }
            report_progress(count);  // whatever happened, the counter of every segment sees this CTA exactly once
        }
    } else if (tid >= kReduceConsumers + 64) {
        const int lane = tid & 31;
        const int n_owned = sm.n_owned;
        const bool vec_zero = ((fc1 & 3) == 0) && ((fc2 & 3) == 0);
        bool ok = true;
        for (int u = 0; u < n_owned && ok; ++u) {
            float* base = sm.own_base[u];
            for (int sg = 0; sg < kReduceSegments && ok; ++sg) {
                int go = 1;
                if (lane == 0 && !wait_flag_ge_relaxed(sm.own_flag[u], epoch * kReduceFlagRadix + static_cast<uint64_t>(sg + 1), call.timeout_ns)) {
                    report_error(status0, UEP_DEV_TIMEOUT_SYNC, u);  // the slot keeps what it holds; no further wait runs
                    go = 0;
                }
                go = __shfl_sync(kFullMask, go, 0);
                if (!go) {
                    ok = false;
                    break;
                }
                const int t0 = sg == 0 ? 0 : seg_end(sg - 1), t1 = seg_end(sg);
                for (int t = t0 + static_cast<int>(blockIdx.x); t < t1; t += static_cast<int>(gridDim.x)) {
                    const bool in1 = t < tiles_fc1;
                    const int64_t off = in1 ? static_cast<int64_t>(t) * kReduceTileElems
                                            : fc1 + static_cast<int64_t>(t - tiles_fc1) * kReduceTileElems;
                    const int64_t left = (in1 ? fc1 : total_numel) - off;
                    const int elems = static_cast<int>(left < kReduceTileElems ? left : kReduceTileElems);
                    float* dst = base + off;
                    if (vec_zero) {
                        if (lane == 0) {
                            const uint32_t bytes = static_cast<uint32_t>(elems) * 4u;
                            for (uint32_t o = 0; o < bytes; o += kReduceZeroBytes) {
                                bulk_store(reinterpret_cast<char*>(dst) + o, zero_tile, bytes - o < kReduceZeroBytes ? bytes - o : kReduceZeroBytes);
                            }
                            bulk_commit();
                        }
                    } else {
                        for (int i = lane; i < elems; i += 32) dst[i] = 0.f;
                    }
                }
            }
        }
        if (lane == 0) bulk_wait_all<0>();
    } else if (!sm.vector_ok) {
        // element-wise path for sizes / pointers that are not multiples of 16 bytes
        for (int64_t k = 0; k < count; ++k) {
            const ReduceItem it = decode_item(first + k * step, n_active, fc1, fc2, tiles_fc1);
            float* mp = master_ptr(it);
            const int r0 = sm.rep_start[it.active], r1 = sm.rep_start[it.active + 1];
            for (int i = tid; i < it.elems; i += kReduceConsumers + 64) {  // every thread but the clearing and reporting warps
                float acc = mp[i];
                for (int r = r0; r < r1; ++r) {
                    if (sm.rep_base[r] == nullptr) continue;
                    acc = __fadd_rn(acc, __ldcg(replica_ptr(it, r) + i));
                }
                mp[i] = acc;
            }
        }
        // every thread's loads of the replicas have returned (the clearing and reporting warps are not part of this path: named barrier)
        asm volatile("bar.sync 1, %0;" ::"r"(kReduceConsumers + 64) : "memory");
        if (tid == 0) sm.pull_finished = 1;
    } else if (tid >= kReduceConsumers + 32) {
        // ---- producer of the master ring: one load per item, in item order -----------------------
        if (tid == kReduceConsumers + 32) {
            int64_t m_issued = 0;
            for (; m_issued < count; ++m_issued) {
                const int s = static_cast<int>(m_issued % kMasterStages);
                if (m_issued >= kMasterStages) {  // the stage's previous tile has been read by every consumer warp
                    const int64_t prev = m_issued - kMasterStages;
                    if (!mbar_wait(&sm.m_empty[s], static_cast<uint32_t>((prev / kMasterStages) & 1), sm.error ? 0 : call.timeout_ns)) {
                        sm.error = 1;
                        break;
                    }
                }
                const ReduceItem it = decode_item(first + m_issued * step, n_active, fc1, fc2, tiles_fc1);
                const uint32_t bytes = static_cast<uint32_t>(it.elems) * 4u;
                mbar_expect_tx(&sm.m_full[s], bytes);
                bulk_load(master_ring + s * kReduceTileBytes, master_ptr(it), bytes, &sm.m_full[s]);
            }
            if (sm.error) {  // loads that never completed must not find the shared memory released under them
                for (int64_t j = m_issued > kMasterStages ? m_issued - kMasterStages : 0; j < m_issued; ++j) {
                    mbar_wait(&sm.m_full[j % kMasterStages], static_cast<uint32_t>((j / kMasterStages) & 1), call.timeout_ns);
                }
            }
        }
    } else if (tid >= kReduceConsumers) {
        // ---- producer of the replica ring: every remote load; reports this CTA's progress ------------
        if (tid == kReduceConsumers) {
            // (item, replica) pairs in the order the consumers take them
            int64_t k_rep = 0;
            int r_issue = -1, r_issue_end = -1;
            ReduceItem it_rep{};
            bool last_of_item = false;
            auto next_replica = [&](float*& src, int& elems) -> bool {
                while (true) {
                    if (r_issue < 0) {
                        if (k_rep >= count) return false;
                        it_rep = decode_item(first + k_rep * step, n_active, fc1, fc2, tiles_fc1);
                        r_issue = sm.rep_start[it_rep.active];
                        r_issue_end = sm.rep_start[it_rep.active + 1];
                    }
                    while (r_issue < r_issue_end && sm.rep_base[r_issue] == nullptr) ++r_issue;
                    if (r_issue >= r_issue_end) {
                        ++k_rep;
                        r_issue = -1;
                        continue;
                    }
                    src = replica_ptr(it_rep, r_issue);
                    elems = it_rep.elems;
                    ++r_issue;
                    int nxt = r_issue;  // is another replica of this item still to come?
                    while (nxt < r_issue_end && sm.rep_base[nxt] == nullptr) ++nxt;
                    last_of_item = nxt >= r_issue_end;
                    return true;
                }
            };
            bool ring_last[kReduceStages];
            int64_t issued = 0, retired = 0, done_items = 0;
            bool more = true;
            while (true) {
                while (more && issued - retired < kReduceStages) {
                    float* src = nullptr;
                    int elems = 0;
                    more = next_replica(src, elems);
                    if (!more) break;
                    const int s = static_cast<int>(issued % kReduceStages);
                    ring_last[s] = last_of_item;
                    const uint32_t bytes = static_cast<uint32_t>(elems) * 4u;
                    mbar_expect_tx(&sm.full[s], bytes);
                    bulk_load(smem_raw + s * kReduceTileBytes, src, bytes, &sm.full[s]);
                    ++issued;
                }
                if (retired == issued) break;  // every replica tile has been consumed
                // the oldest stage: every consumer warp has read it
                const int s = static_cast<int>(retired % kReduceStages);
                if (!mbar_wait(&sm.empty[s], static_cast<uint32_t>((retired / kReduceStages) & 1), sm.error ? 0 : call.timeout_ns)) {
                    sm.error = 1;
                    break;
                }
                ++retired;
                if (ring_last[s]) sm.done_items = ++done_items;  // the reporting warp turns this into segment counts
            }
            if (sm.error) {
                report_error(status0, UEP_DEV_TIMEOUT_COPY, static_cast<int>(retired));
                for (int64_t j = issued > kReduceStages ? issued - kReduceStages : 0; j < issued; ++j) {
                    mbar_wait(&sm.full[j % kReduceStages], static_cast<uint32_t>((j / kReduceStages) & 1), call.timeout_ns);
                }
            }
            sm.pull_finished = 1;
        }
    } else {
        // ---- consumer warps ---------------------------------------------------------------------
        const int lane = tid & 31;
        int64_t consumed = 0;
        stamp(2);
        for (int64_t k = 0; k < count; ++k) {
            const ReduceItem it = decode_item(first + k * step, n_active, fc1, fc2, tiles_fc1);
            const int nvec = it.elems >> 2;
            float4 acc[kReduceVecPerThread];
            {
                const int s = static_cast<int>(k % kMasterStages);
                if (!mbar_wait(&sm.m_full[s], static_cast<uint32_t>((k / kMasterStages) & 1), sm.error ? 0 : call.timeout_ns)) {
                    sm.error = 1;  // keep the control flow uniform; the result of this tile is void
                }
                const float4* stage = reinterpret_cast<const float4*>(master_ring + s * kReduceTileBytes);
#pragma unroll
                for (int u = 0; u < kReduceVecPerThread; ++u) {
                    const int i = tid + u * kReduceConsumers;
                    acc[u] = i < nvec ? stage[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.m_empty[s]);
            }
            const int r0 = sm.rep_start[it.active], r1 = sm.rep_start[it.active + 1];
            for (int r = r0; r < r1; ++r) {
                if (sm.rep_base[r] == nullptr) continue;
                const int s = static_cast<int>(consumed % kReduceStages);
                if (!mbar_wait(&sm.full[s], static_cast<uint32_t>((consumed / kReduceStages) & 1), sm.error ? 0 : call.timeout_ns)) {
                    sm.error = 1;
                }
                const float4* stage = reinterpret_cast<const float4*>(smem_raw + s * kReduceTileBytes);
#pragma unroll
                for (int u = 0; u < kReduceVecPerThread; ++u) {
                    const int i = tid + u * kReduceConsumers;
                    if (i < nvec) {
                        const float4 v = stage[i];
                        acc[u].x = __fadd_rn(acc[u].x, v.x); acc[u].y = __fadd_rn(acc[u].y, v.y);
                        acc[u].z = __fadd_rn(acc[u].z, v.z); acc[u].w = __fadd_rn(acc[u].w, v.w);
                    }
                }
                ++consumed;
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.empty[s]);  // this warp no longer reads the stage
            }
            float4* mp = reinterpret_cast<float4*>(master_ptr(it));
#pragma unroll
            for (int u = 0; u < kReduceVecPerThread; ++u) {
                const int i = tid + u * kReduceConsumers;
                if (i < nvec) mp[i] = acc[u];
            }
        }
        stamp(3);
    }

    stamp(5);
}

}  // namespace

cudaError_t launch_grad_reduce(const ReduceCall& call, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(kReduceStages + kMasterStages) * kReduceTileBytes + kReduceZeroBytes;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(grad_reduce_kernel),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    if (call.nlocal * call.R > kMaxOwned) return cudaErrorInvalidValue;  // more replica slots per launch than the kernel's table holds
    count_launch();
    const dim3 grid(call.nlocal * call.ctas_per_rank), block(kReduceThreads);
    if (call.nlocal > 1) {
        // hosted ranks clear their slots behind other hosted ranks' pulls inside this one launch: the CTAs that
        // wait and the CTAs they wait for must be resident together
        ReduceCall copy = call;
        void* args[] = {&copy};
        return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(grad_reduce_kernel), grid, block, args, smem, stream);
    }
    grad_reduce_kernel<<<grid, block, smem, stream>>>(call);
    return cudaGetLastError();
}

}  // namespace uep
