// Placement solver: per-expert token counts -> hot-expert replication plan, for one
// NVLink domain, executed by one CTA (>= 4 warps).
//
// Results are bit-identical to the reference solver
// (csrc/kernels/placement.cu:788-1482 of the reference): same fp32 threshold
// arithmetic, same tie-breaks, same probe schedule of the threshold search, same
// largest-remainder splits. The execution is different:
//   * one lane per rank with slack / slot counters in registers for any domain size
//     (1-3 ranks per lane), warp-wide redux instructions instead of shuffle trees,
//     occupancy of an expert as a ballot word;
//   * each rank's masters are ranked by counting instead of a serial insertion sort;
//   * the per-rank load matrix is read through L2 where it is needed instead of being
//     staged in shared memory, so shared memory stays under 48 KB at the static limits;
//   * output arrays are cleared by the same CTA instead of six memsets.
#pragma once

#include <climits>

#include "common.cuh"

namespace uep {

struct ExportEntry {
    int expert_local;
    int target_rank_local;
    int quota;
};

struct SolveArgs {
    const int32_t* global_loads;    // [L]
    const int32_t* loads_per_rank;  // [N, L]
    int32_t* p2l;                   // [P]
    int32_t* l2p;                   // [L, D]
    int32_t* lcnts;                 // [L]
    int32_t* quota;                 // [L, D]
    int32_t* quota_prefix;          // [L, D]
    int32_t* rank_quota_prefix;     // [L, D]
    int32_t* physical_loads;        // [P] quota of every physical slot, 0 when empty (optional: may be null)
    int N, G, M, R, D;
    float balance_threshold;
    int min_tokens;
    int allow_zero_master;
    int locality;
    float eps;
    int my_rank;
    int legacy;  // 1: legacy placement (counts-only greedy, round-robin reroute) instead of the quota solver
    unsigned long long* trace;  // optional: 8 globaltimer stamps of the solver phases (tuning aid), or null
};

constexpr int kSolverProbeWarps = 4;

// Control words in shared memory.
enum SolverCtrl {
    kCtlLo = 0, kCtlHi, kCtlPrecheckDone, kCtlFastDone, kCtlNumExports, kCtlSmallRange,
    kCtlProbe0, kCtlValid0 = kCtlProbe0 + kSolverProbeWarps, kCtlFeasible0 = kCtlValid0 + kSolverProbeWarps,
    kCtlMultiCount = kCtlFeasible0 + kSolverProbeWarps, kCtlCount
};

struct SolverSmem {
    int32_t* loads;           // [E]
    int32_t* my_loads;        // [E]
    int32_t* sorted_experts;  // [E]
    int32_t* expert_slot;     // [E]
    int32_t* rank_load;       // [Gp]
    int32_t* source_order;    // [Gp]
    int32_t* next_slot;       // [Gp]
    int32_t* export_sum;      // [4][E]
    uint32_t* occ;            // [4][E*NS]
    ExportEntry* plan;        // [kMaxExportsPerDomain]
    int* ctrl;                // [kCtlCount]
};

__host__ __device__ inline int solver_ns(int G) { return (G + 31) / 32; }
__host__ __device__ inline int solver_gpad(int G) { return (G + 3) / 4 * 4; }
__host__ __device__ inline size_t solver_smem_bytes(int E, int G) {
    const int ns = solver_ns(G), gp = solver_gpad(G);
    return sizeof(int32_t) * (4 * static_cast<size_t>(E) + 3 * gp + kSolverProbeWarps * static_cast<size_t>(E) +
                              kSolverProbeWarps * static_cast<size_t>(E) * ns) +
           sizeof(ExportEntry) * kMaxExportsPerDomain + sizeof(int) * 32;
}

__device__ inline SolverSmem carve_solver_smem(char* raw, int E, int G) {
    const int ns = solver_ns(G), gp = solver_gpad(G);
    SolverSmem s;
    int32_t* p = reinterpret_cast<int32_t*>(raw);
    s.loads = p; p += E;
    s.my_loads = p; p += E;
    s.sorted_experts = p; p += E;
    s.expert_slot = p; p += E;
    s.rank_load = p; p += gp;
    s.source_order = p; p += gp;
    s.next_slot = p; p += gp;
    s.export_sum = p; p += kSolverProbeWarps * E;
    s.occ = reinterpret_cast<uint32_t*>(p); p += kSolverProbeWarps * E * ns;
    s.plan = reinterpret_cast<ExportEntry*>(p); p += 3 * kMaxExportsPerDomain;
    s.ctrl = reinterpret_cast<int*>(p);
    return s;
}

// Greedy export plan for one threshold, by one warp. Returns feasibility (uniform over
// the warp). Semantics of csrc/kernels/placement.cu:337-667 of the reference.
template <int NS, bool STORE>
__device__ bool warp_build_plan(const SolverSmem& sm, int32_t* export_sum, uint32_t* occ, ExportEntry* plan,
                                int& num_exports, int thr, int E, int G, int M, int R, int min_tokens,
                                bool allow_zero_master, bool dynamic_floor, int lane) {
    num_exports = 0;
    // state init (:86-109)
    for (int e = lane; e < E; e += kWarp) {
        export_sum[e] = 0;
        const int home = e / M;
#pragma unroll
        for (int s = 0; s < NS; ++s) occ[e * NS + s] = ((home >> 5) == s) ? (1u << (home & 31)) : 0u;
    }
    int slack[NS], slots[NS];
    int local_excess = 0, local_slack = 0;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
        const int r = lane + kWarp * s;
        const int rl = (r < G) ? sm.rank_load[r] : thr;
        slack[s] = max(thr - rl, 0);
        slots[s] = 0;
        local_excess += max(rl - thr, 0);
        local_slack += slack[s];
    }
    __syncwarp();
    const int total_excess = warp_sum(local_excess);
    const int total_slack = warp_sum(local_slack);
    if (total_excess == 0) return true;
    if (total_excess > total_slack) return false;

    int running_excess = total_excess;
    int running_slack = total_slack;
    for (int ord = 0; ord < G; ++ord) {
        const int src = sm.source_order[ord];
        int need = max(sm.rank_load[src] - thr, 0);
        if (need <= 0) continue;
        if (need > running_slack) return false;

        for (int pos = 0; pos < M; ++pos) {
            const int e = sm.sorted_experts[src * M + pos];
            const int load_e = sm.loads[e];
            const int keep = (!allow_zero_master && load_e > 0) ? 1 : 0;
            int es = export_sum[e];
            int avail = max(load_e - keep - es, 0);
            if (avail <= 0) continue;

            bool my_occ[NS];
#pragma unroll
            for (int s = 0; s < NS; ++s) my_occ[s] = ((occ[e * NS + s] >> lane) & 1u) != 0u;
            bool changed = false;

            while (need > 0 && avail > 0) {
                bool ok[NS];
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    ok[s] = (lane + kWarp * s < G) && slack[s] > 0 && slots[s] < R && !my_occ[s];
                }
                int floor_tokens = min_tokens;
                if (dynamic_floor) {
                    int feasible = 0;
#pragma unroll
                    for (int s = 0; s < NS; ++s) {
                        feasible += __popc(__ballot_sync(kFullMask, ok[s] && min(min(need, slack[s]), avail) > 0));
                    }
                    if (feasible <= 0) break;
                    floor_tokens = max(1, (need + feasible - 1) / feasible);
                }
                int cands[NS];
                int cand = -1;
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    cands[s] = (ok[s] && min(min(need, slack[s]), avail) >= floor_tokens) ? slack[s] : -1;
                    cand = max(cand, cands[s]);
                }
                const int best_cap = warp_max(cand);
                if (best_cap < 0) break;
                int best = -1;  // largest slack, ties to the lower rank
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    const unsigned b = __ballot_sync(kFullMask, cands[s] == best_cap);
                    if (best < 0 && b != 0u) best = (__ffs(b) - 1) + kWarp * s;
                }
                if (STORE && num_exports >= kMaxExportsPerDomain) return false;
                const int q = min(min(need, best_cap), avail);
                if (STORE) {
                    if (lane == 0) plan[num_exports] = ExportEntry{e, best, q};
                    num_exports += 1;
                }
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    if (lane + kWarp * s == best) {
                        slack[s] -= q;
                        slots[s] += 1;
                        my_occ[s] = true;
                    }
                }
                es += q;
                running_excess -= q;
                running_slack -= q;
                need -= q;
                avail -= q;
                changed = true;
            }
            if (changed) {
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    const unsigned w = __ballot_sync(kFullMask, my_occ[s]);
                    if (lane == 0) occ[e * NS + s] = w;
                }
                if (lane == 0) export_sum[e] = es;
                __syncwarp();
            }
            if (need == 0) break;
        }
        if (need > 0) return false;
        if (running_excess > running_slack) return false;
    }
    return true;
}

// Split of this rank's tokens of one expert over the expert's replicas, as an inclusive
// prefix. Semantics of csrc/kernels/placement.cu:1342-1481 / :669-786 of the reference.
template <int MAXC>
__device__ void build_rank_quota_prefix(const SolveArgs& a, int l_global, int C, int my_load, const int* phys,
                                        const int* q, int Lp, int L) {
    // phys[j] / q[j]: physical id and quota of replica j (j = 0 is the master), handed over from
    // shared memory by the caller so that no plan row has to be read back from global memory.
    const int64_t row = static_cast<int64_t>(l_global) * a.D;
    int host_rank[MAXC], my_alloc[MAXC];
    long long remainders[MAXC];
    for (int j = 0; j < C; ++j) {
        host_rank[j] = phys[j] / Lp;
        my_alloc[j] = 0;
        remainders[j] = -1;
    }
    if (!a.locality) {
        const int rem_my = my_load;
        int assigned = 0, total_quota = 0;
        for (int j = 0; j < C; ++j) total_quota += q[j];
        if (rem_my > 0 && total_quota > 0) {
            for (int j = 0; j < C; ++j) {
                const long long scaled = static_cast<long long>(rem_my) * q[j];
                const int share = static_cast<int>(scaled / total_quota);
                my_alloc[j] = share;
                remainders[j] = scaled % total_quota;
                assigned += share;
            }
            int remaining = rem_my - assigned;
            while (remaining > 0) {
                int best_j = -1;
                for (int j = 0; j < C; ++j) {
                    if (best_j < 0 || remainders[j] > remainders[best_j]) best_j = j;  // ties keep the lower j
                }
                my_alloc[best_j] += 1;
                remainders[best_j] = -1;
                --remaining;
            }
        }
    } else {
        int remote_cap[MAXC];
        int host_left[MAXC];  // remaining own load of host_rank[j]'s rank, shared between equal hosts via `first`
        int first[MAXC];
        int rem_my = my_load;
        int total_remote_cap = 0;
        for (int j = 0; j < C; ++j) {
            int f = j;
            for (int u = 0; u < j; ++u) {
                if (host_rank[u] == host_rank[j]) {
                    f = first[u];
                    break;
                }
            }
            first[j] = f;
            if (f == j) {
                host_left[j] = __ldcg(a.loads_per_rank + static_cast<int64_t>(host_rank[j]) * L + l_global);
            }
            const int qj = q[j];
            const int local_fill = min(host_left[f], qj);
            host_left[f] -= local_fill;
            remote_cap[j] = qj - local_fill;
            total_remote_cap += remote_cap[j];
            if (host_rank[j] == a.my_rank) {
                my_alloc[j] += local_fill;
                rem_my -= local_fill;
            }
        }
        rem_my = max(rem_my, 0);
        if (rem_my > 0 && total_remote_cap > 0) {
            int assigned = 0;
            for (int j = 0; j < C; ++j) {
                if (host_rank[j] == a.my_rank || remote_cap[j] <= 0) continue;
                const long long scaled = static_cast<long long>(rem_my) * remote_cap[j];
                const int share = static_cast<int>(scaled / total_remote_cap);
                my_alloc[j] += share;
                remainders[j] = scaled % total_remote_cap;
                assigned += share;
            }
            int remaining = rem_my - assigned;
            while (remaining > 0) {
                int best_j = -1;
                for (int j = 0; j < C; ++j) {
                    if (host_rank[j] == a.my_rank || remote_cap[j] <= 0) continue;
                    if (best_j < 0 || remainders[j] > remainders[best_j] ||
                        (remainders[j] == remainders[best_j] &&
                         (host_rank[j] < host_rank[best_j] || (host_rank[j] == host_rank[best_j] && j < best_j)))) {
                        best_j = j;
                    }
                }
                if (best_j < 0) break;
                my_alloc[best_j] += 1;
                remainders[best_j] = -1;
                --remaining;
            }
        }
    }
    int prefix = 0;
    for (int j = 0; j < C; ++j) {
        prefix += my_alloc[j];
        a.rank_quota_prefix[row + j] = prefix;
    }
}

__device__ __forceinline__ int warp_inclusive_scan(int v, int lane) {
#pragma unroll
    for (int off = 1; off < kWarp; off <<= 1) {
        const int t = __shfl_up_sync(kFullMask, v, off);
        if (lane >= off) v += t;
    }
    return v;
}

// The split of build_rank_quota_prefix for an expert with 2..32 replicas, by one warp: lane j
// holds replica j, the sums and arg-max searches are warp reductions, and the hosts' own loads
// are fetched by all lanes at once. Returns false (nothing written) when two replicas share a
// host rank, which the sequential bookkeeping of the general version is needed for.
__device__ __forceinline__ bool warp_rank_quota_prefix(const SolveArgs& a, int l_global, int C, int my_load, int phys,
                                                       int q, int Lp, int L, int lane) {
    const bool active = lane < C;
    const int host = active ? phys / Lp : -1 - lane;
    int my_alloc = 0;
    if (!a.locality) {
        const int total_quota = __reduce_add_sync(kFullMask, active ? q : 0);
        if (my_load > 0 && total_quota > 0) {
            const long long scaled = static_cast<long long>(my_load) * (active ? q : 0);
            const int share = static_cast<int>(scaled / total_quota);
            int rem = active ? static_cast<int>(scaled % total_quota) : INT_MIN;
            my_alloc = share;
            int remaining = my_load - __reduce_add_sync(kFullMask, share);  // < C: a sum of C fractional parts
            for (int it = 0; it < C && remaining > 0; ++it) {
                const int best = __reduce_max_sync(kFullMask, rem);
                const int pick = __ffs(__ballot_sync(kFullMask, active && rem == best)) - 1;  // ties: the lower j
                if (lane == pick) {
                    my_alloc += 1;
                    rem = -1;
                }
                --remaining;
            }
        }
    } else {
        const unsigned same_host = __match_any_sync(kFullMask, host);  // all 32 lanes take part: not under `active &&`
        if (__any_sync(kFullMask, active && __popc(same_host) > 1)) return false;
        const int own = active ? __ldcg(a.loads_per_rank + static_cast<int64_t>(host) * L + l_global) : 0;
        const int local_fill = active ? min(own, q) : 0;
        const int remote_cap = active ? q - local_fill : 0;
        const int total_remote_cap = __reduce_add_sync(kFullMask, remote_cap);
        const bool mine = active && host == a.my_rank;
        if (mine) my_alloc = local_fill;
        const int rem_my = max(my_load - __reduce_add_sync(kFullMask, mine ? local_fill : 0), 0);
        if (rem_my > 0 && total_remote_cap > 0) {
            const bool eligible = active && !mine && remote_cap > 0;
            const long long scaled = static_cast<long long>(rem_my) * (eligible ? remote_cap : 0);
            const int share = static_cast<int>(scaled / total_remote_cap);
            int rem = eligible ? static_cast<int>(scaled % total_remote_cap) : INT_MIN;
            my_alloc += share;
            int remaining = rem_my - __reduce_add_sync(kFullMask, share);  // < number of eligible replicas
            for (int it = 0; it < C && remaining > 0; ++it) {
                const int best = __reduce_max_sync(kFullMask, rem);
                if (best == INT_MIN) break;  // nobody can take a unit
                // ties: the lower host rank, then the lower j
                const bool cand = eligible && rem == best;
                const int best_host = __reduce_min_sync(kFullMask, cand ? host : INT_MAX);
                const int pick = __ffs(__ballot_sync(kFullMask, cand && host == best_host)) - 1;
                if (lane == pick) {
                    my_alloc += 1;
                    rem = -1;
                }
                --remaining;
            }
        }
    }
    const int prefix = warp_inclusive_scan(my_alloc, lane);
    if (active) a.rank_quota_prefix[static_cast<int64_t>(l_global) * a.D + lane] = prefix;
    return true;
}

// Solve one NVLink domain. All threads of the CTA must call it (blockDim.x >= 128,
// multiple of 32). smem_raw must hold solver_smem_bytes(E, G) bytes, 16-byte aligned.
template <int NS>
__device__ void solve_domain(const SolveArgs& a, int domain, char* smem_raw, DeviceStatus* status) {
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int G = a.G, M = a.M, R = a.R, D = a.D;
    const int E = G * M, Lp = M + R, L = a.N * M;
    const int domain_start_rank = domain * G;
    const int domain_start_log = domain_start_rank * M;
    SolverSmem sm = carve_solver_smem(smem_raw, E, G);
    auto stamp = [&](int slot) {
        if (a.trace != nullptr && tid == 0) a.trace[slot] = global_timer_ns();
    };
    stamp(0);

    // Clear this domain's slice of every output, then place the masters.
    for (int i = tid; i < G * Lp; i += nthreads) {
        a.p2l[domain_start_rank * Lp + i] = -1;
        if (a.physical_loads != nullptr) a.physical_loads[domain_start_rank * Lp + i] = 0;
    }
    for (int i = tid; i < E * D; i += nthreads) {
        const int64_t idx = static_cast<int64_t>(domain_start_log) * D + i;
        a.l2p[idx] = -1;
        a.quota[idx] = 0;
        a.quota_prefix[idx] = 0;
        a.rank_quota_prefix[idx] = 0;
    }
    __syncthreads();
    for (int i = tid; i < E; i += nthreads) {
        const int l_global = domain_start_log + i;
        sm.loads[i] = __ldcg(a.global_loads + l_global);
        sm.my_loads[i] = __ldcg(a.loads_per_rank + static_cast<int64_t>(a.my_rank) * L + l_global);
        sm.expert_slot[i] = 1;
        const int phys = (domain_start_rank + i / M) * Lp + i % M;
        a.p2l[phys] = l_global;
        a.l2p[static_cast<int64_t>(l_global) * D] = phys;
    }
    __syncthreads();
    stamp(1);
    for (int r = tid; r < G; r += nthreads) {
        int sum = 0;
        for (int m = 0; m < M; ++m) sum += sm.loads[r * M + m];
        sm.rank_load[r] = sum;
        sm.next_slot[r] = 0;
    }
    __syncthreads();
    // ranks by load descending, ties to the lower index; each rank's masters likewise
    for (int i = tid; i < G; i += nthreads) {
        const int mine = sm.rank_load[i];
        int pos = 0;
        for (int j = 0; j < G; ++j) {
            const int other = sm.rank_load[j];
            pos += (other > mine || (other == mine && j < i)) ? 1 : 0;
        }
        sm.source_order[pos] = i;
    }
    for (int i = tid; i < E; i += nthreads) {
        const int base = (i / M) * M;
        const int mine = sm.loads[i];
        int pos = 0;
        for (int j = base; j < base + M; ++j) {
            const int other = sm.loads[j];
            pos += (other > mine || (other == mine && j < i)) ? 1 : 0;
        }
        sm.sorted_experts[base + pos] = i;
    }
    const bool do_search = (R > 0 && G > 1);
    if (tid == 0) {
        sm.ctrl[kCtlNumExports] = 0;
        sm.ctrl[kCtlFastDone] = 0;
        sm.ctrl[kCtlPrecheckDone] = 0;
        if (do_search) {
            int total = 0, mx = 0;
            for (int r = 0; r < G; ++r) {
                total += sm.rank_load[r];
                mx = max(mx, sm.rank_load[r]);
            }
            // fp32, in the reference's order: ceilf((float(total) / G) * bt)
            const float bt = fmaxf(a.balance_threshold, 1.0f);
            const float mean = __fdiv_rn(static_cast<float>(total), static_cast<float>(G));
            const int lo = static_cast<int>(ceilf(__fmul_rn(mean, bt)));
            sm.ctrl[kCtlLo] = lo;
            sm.ctrl[kCtlHi] = max(mx, lo);
        }
    }
    __syncthreads();

    stamp(2);
    const bool allow0 = a.allow_zero_master != 0;
    if (do_search) {
        if (warp == 0) {  // fast path: up to three builds with the dynamic floor
            const int lo = sm.ctrl[kCtlLo], hi = sm.ctrl[kCtlHi];
            const float eps = fmaxf(a.eps, 0.0f);
            int thr = static_cast<int>(ceilf(__fmul_rn(static_cast<float>(lo), __fadd_rn(1.0f, eps))));
            thr = max(thr, lo);
            const int step = max(1, (hi + 99) / 100);
            bool done = false;
            for (int retry = 0; retry <= 2 && !done; ++retry) {
                int n = 0;
                done = warp_build_plan<NS, true>(sm, sm.export_sum, sm.occ, sm.plan, n, thr, E, G, M, R, a.min_tokens,
                                                 allow0, true, lane);
                if (done) {
                    if (lane == 0) {
                        sm.ctrl[kCtlNumExports] = n;
                        sm.ctrl[kCtlFastDone] = 1;
                        sm.ctrl[kCtlLo] = thr;
                    }
                } else {
                    thr = min(hi, thr + step);
                }
                __syncwarp();
            }
        }
        __syncthreads();
        if (!sm.ctrl[kCtlFastDone]) {
            if (warp == 0) {
                int lo = sm.ctrl[kCtlLo], hi = sm.ctrl[kCtlHi];
                while (lo < hi) {  // capacity bisection
                    const int probe = lo + ((hi - lo) >> 1);
                    int ex = 0, sl = 0;
                    for (int r = lane; r < G; r += kWarp) {
                        ex += max(sm.rank_load[r] - probe, 0);
                        sl += max(probe - sm.rank_load[r], 0);
                    }
                    if (warp_sum(ex) <= warp_sum(sl)) hi = probe;
                    else lo = probe + 1;
                }
                int n = 0;
                const bool ok = warp_build_plan<NS, true>(sm, sm.export_sum, sm.occ, sm.plan, n, lo, E, G, M, R,
                                                          a.min_tokens, allow0, false, lane);
                if (lane == 0) {
                    sm.ctrl[kCtlPrecheckDone] = ok ? 1 : 0;
                    if (ok) {
                        sm.ctrl[kCtlNumExports] = n;
                        sm.ctrl[kCtlLo] = lo;
                    } else {
                        sm.ctrl[kCtlLo] = min(lo + 1, sm.ctrl[kCtlHi]);
                    }
                }
            }
            __syncthreads();
            while (true) {
                if (sm.ctrl[kCtlPrecheckDone] || sm.ctrl[kCtlLo] >= sm.ctrl[kCtlHi]) break;
                __syncthreads();  // everyone has read lo/hi before thread 0 rewrites the probe table
                if (tid == 0) {
                    const int lo = sm.ctrl[kCtlLo], hi = sm.ctrl[kCtlHi];
                    const int range = hi - lo;
                    const int small_range = (range <= kSolverProbeWarps) ? 1 : 0;
                    sm.ctrl[kCtlSmallRange] = small_range;
                    for (int w = 0; w < kSolverProbeWarps; ++w) {
                        if (small_range) {
                            sm.ctrl[kCtlProbe0 + w] = lo + w;
                            sm.ctrl[kCtlValid0 + w] = (lo + w < hi) ? 1 : 0;
                        } else {
                            sm.ctrl[kCtlProbe0 + w] =
                                lo + static_cast<int>((static_cast<long long>(range) * (w + 1)) / (kSolverProbeWarps + 1));
                            sm.ctrl[kCtlValid0 + w] = 1;
                        }
                        sm.ctrl[kCtlFeasible0 + w] = 0;
                    }
                }
                __syncthreads();
                if (warp < kSolverProbeWarps && sm.ctrl[kCtlValid0 + warp]) {
                    int n = 0;
                    const bool ok = warp_build_plan<NS, false>(sm, sm.export_sum + warp * E, sm.occ + warp * E * NS,
                                                               nullptr, n, sm.ctrl[kCtlProbe0 + warp], E, G, M, R,
                                                               a.min_tokens, allow0, false, lane);
                    if (lane == 0) sm.ctrl[kCtlFeasible0 + warp] = ok ? 1 : 0;
                }
                __syncthreads();
                if (tid == 0) {
                    if (sm.ctrl[kCtlSmallRange]) {
                        int best = -1;
                        for (int w = 0; w < kSolverProbeWarps; ++w) {
                            if (sm.ctrl[kCtlValid0 + w] && sm.ctrl[kCtlFeasible0 + w]) {
                                best = sm.ctrl[kCtlProbe0 + w];
                                break;
                            }
                        }
                        if (best >= 0) {
                            sm.ctrl[kCtlLo] = best;
                            sm.ctrl[kCtlHi] = best;
                        } else {
                            sm.ctrl[kCtlLo] = sm.ctrl[kCtlHi];
                        }
                    } else {
                        int first = -1;
                        for (int w = 0; w < kSolverProbeWarps; ++w) {
                            if (sm.ctrl[kCtlFeasible0 + w]) {
                                first = w;
                                break;
                            }
                        }
                        if (first >= 0) {
                            sm.ctrl[kCtlHi] = sm.ctrl[kCtlProbe0 + first];
                            if (first > 0) sm.ctrl[kCtlLo] = sm.ctrl[kCtlProbe0 + first - 1] + 1;
                        } else {
                            sm.ctrl[kCtlLo] = sm.ctrl[kCtlProbe0 + kSolverProbeWarps - 1] + 1;
                        }
                    }
                }
                __syncthreads();
            }
            if (!sm.ctrl[kCtlPrecheckDone]) {
                if (warp == 0) {
                    int n = 0;
                    const bool ok = warp_build_plan<NS, true>(sm, sm.export_sum, sm.occ, sm.plan, n, sm.ctrl[kCtlLo], E,
                                                              G, M, R, a.min_tokens, allow0, false, lane);
                    if (lane == 0) {
                        sm.ctrl[kCtlNumExports] = ok ? n : 0;
                        if (!ok) report_error(status, UEP_DEV_SOLVER_INFEASIBLE, sm.ctrl[kCtlLo]);
                    }
                }
                __syncthreads();
            }
        }
    }

    stamp(3);
    // Emit: master quotas, then replicas in plan order. Two tables of the search are free by now
    // and are reused: sorted_experts becomes "first plan entry of this expert" (an expert's
    // exports are consecutive in the plan: they are all made while its one source rank is being
    // drained), and the probe warps' scratch becomes the list of experts that have replicas.
    int* first_entry = sm.sorted_experts;
    int* multi_list = sm.export_sum + E;
    for (int e = tid; e < E; e += nthreads) {
        const int64_t row = static_cast<int64_t>(domain_start_log + e) * D;
        const int master_quota = do_search ? (sm.loads[e] - sm.export_sum[e]) : sm.loads[e];
        a.quota[row] = master_quota;
        if (a.physical_loads != nullptr) a.physical_loads[(domain_start_rank + e / M) * Lp + e % M] = master_quota;
    }
    if (tid == 0) sm.ctrl[kCtlMultiCount] = 0;
    __syncthreads();
    if (warp == 0) {
        // 32 plan entries at a time: an entry's replica slot (and its target's redundant slot) is
        // the counter left by the earlier chunks plus the number of lower lanes that name the same
        // expert (the same target), which is exactly the creation order of a serial walk.
        const int n = sm.ctrl[kCtlNumExports];
        for (int base = 0; base < n; base += kWarp) {
            const int k = base + lane;
            const bool active = k < n;
            const unsigned amask = __ballot_sync(kFullMask, active);
            if (active) {
                const ExportEntry entry = sm.plan[k];
                const unsigned same_e = __match_any_sync(amask, entry.expert_local);
                const unsigned same_t = __match_any_sync(amask, entry.target_rank_local);
                const unsigned below = (1u << lane) - 1u;
                const int slot = sm.expert_slot[entry.expert_local] + __popc(same_e & below);
                const int tslot = sm.next_slot[entry.target_rank_local] + __popc(same_t & below);
                __syncwarp(amask);  // every lane has read the counters
                if ((same_e >> lane) == 1u) sm.expert_slot[entry.expert_local] = slot + 1;  // highest lane of its group
                if ((same_t >> lane) == 1u) sm.next_slot[entry.target_rank_local] = tslot + 1;
                if (slot == 1) first_entry[entry.expert_local] = k;
                const int l_global = domain_start_log + entry.expert_local;
                const int64_t row = static_cast<int64_t>(l_global) * D;
                const int phys = (domain_start_rank + entry.target_rank_local) * Lp + M + tslot;
                if (slot >= D || phys >= (domain_start_rank + entry.target_rank_local + 1) * Lp) {
                    report_error(status, UEP_DEV_BAD_PLAN, k);
                } else {
                    a.p2l[phys] = l_global;
                    a.l2p[row + slot] = phys;
                    a.quota[row + slot] = entry.quota;
                    if (a.physical_loads != nullptr) a.physical_loads[phys] = entry.quota;
                    sm.plan[k].target_rank_local = phys;  // from here on the entry carries the physical id
                }
            }
            __syncwarp();
        }
    }
    __syncthreads();
    stamp(4);
    // Counts and prefixes. An expert without replicas keeps all of this rank's tokens (every
    // branch of the split reduces to that), so one thread writes its row; the others go to the
    // warps, one expert per warp at a time.
    for (int e = tid; e < E; e += nthreads) {
        const int l_global = domain_start_log + e;
        const int64_t row = static_cast<int64_t>(l_global) * D;
        const int C = min(sm.expert_slot[e], D);
        a.lcnts[l_global] = C;
        if (C == 1) {
            a.quota_prefix[row] = do_search ? (sm.loads[e] - sm.export_sum[e]) : sm.loads[e];
            a.rank_quota_prefix[row] = sm.my_loads[e];
        } else {
            multi_list[atomicAdd(&sm.ctrl[kCtlMultiCount], 1)] = e;
        }
    }
    __syncthreads();
    const int n_multi = sm.ctrl[kCtlMultiCount];
    for (int idx = warp; idx < n_multi; idx += nthreads / kWarp) {
        const int e = multi_list[idx];
        const int l_global = domain_start_log + e;
        const int64_t row = static_cast<int64_t>(l_global) * D;
        const int C = min(sm.expert_slot[e], D);
        const int master_quota = sm.loads[e] - sm.export_sum[e];
        const int master_phys = (domain_start_rank + e / M) * Lp + e % M;
        const int first = first_entry[e];
        bool done = false;
        if (C <= kWarp) {
            int phys = 0, q = 0;
            if (lane == 0) {
                phys = master_phys;
                q = master_quota;
            } else if (lane < C) {
                const ExportEntry entry = sm.plan[first + lane - 1];
                phys = entry.target_rank_local;
                q = entry.quota;
            }
            const int qp = warp_inclusive_scan(q, lane);
            if (lane < C) a.quota_prefix[row + lane] = qp;
            done = warp_rank_quota_prefix(a, l_global, C, sm.my_loads[e], phys, q, Lp, L, lane);
        }
        if (!done && lane == 0) {  // more than 32 replicas, or two replicas on one rank: the serial version
            int phys[kMaxRanksPerDomain], q[kMaxRanksPerDomain];
            phys[0] = master_phys;
            q[0] = master_quota;
            int prefix = 0;
            for (int j = 0; j < C; ++j) {
                if (j > 0) {
                    phys[j] = sm.plan[first + j - 1].target_rank_local;
                    q[j] = sm.plan[first + j - 1].quota;
                }
                prefix += q[j];
                a.quota_prefix[row + j] = prefix;
            }
            build_rank_quota_prefix<kMaxRanksPerDomain>(a, l_global, C, sm.my_loads[e], phys, q, Lp, L);
        }
        __syncwarp();
    }
    __syncthreads();
    stamp(5);
}

// ---------------------------------------------------------------------------------------------
// Legacy placement (legacy_placement=True). The reference solves this mode on the host after copying the
// loads back and synchronising the stream (csrc/kernels/legacy/placement_cpu.cpp:17-241); here it is one
// warp of the plan kernel, so the mode costs no host round trip. Same greedy, same doubles (IEEE
// division and addition, never contracted), same tie-breaks:
//   1. redundant slots are granted one at a time to the expert with the largest load per instance
//      (ties: lower id; at most G-1 extra instances per expert; with balance_threshold > 1 the granting
//      stops once the best load per instance is within threshold x the mean load per master slot);
//   2. the extra instances, ordered by load per instance descending then expert id, go to the rank
//      with the smallest accumulated load (ties: lower rank) that has a free slot and does not hold
//      the expert; an instance that finds no rank is dropped.
// Quotas are not used in this mode: the reroute is round-robin over an expert's instances.
// Shared memory: legacy_smem_bytes(E, G). All threads of the CTA must call it.
// ---------------------------------------------------------------------------------------------
__host__ __device__ inline size_t legacy_smem_bytes(int E, int G) {
    return sizeof(double) * (static_cast<size_t>(E) + 2 * kMaxExportsPerDomain + solver_gpad(G)) +
           sizeof(int32_t) * (3 * static_cast<size_t>(E) + 2 * kMaxExportsPerDomain + solver_gpad(G) + 8) +
           sizeof(uint32_t) * static_cast<size_t>(E) * solver_ns(G);
}

__device__ __noinline__ void legacy_solve_domain(const SolveArgs& a, int domain, char* smem_raw, DeviceStatus* status) {
    const int tid = threadIdx.x, nthreads = blockDim.x, lane = tid & 31, warp = tid >> 5;
    const int G = a.G, M = a.M, R = a.R, D = a.D, E = G * M, Lp = M + R, ns = solver_ns(G);
    const int rank0 = domain * G, log0 = rank0 * M;
    double* score = reinterpret_cast<double*>(smem_raw);        // [E] load per instance
    double* xkey = score + E;                                    // [512] extras: load per instance
    double* xkey_sorted = xkey + kMaxExportsPerDomain;           // [512]
    double* rank_load = xkey_sorted + kMaxExportsPerDomain;      // [Gpad]
    int32_t* loads = reinterpret_cast<int32_t*>(rank_load + solver_gpad(G));  // [E]
    int32_t* cnt = loads + E;                                    // [E] instances
    int32_t* placed = cnt + E;                                   // [E] instances placed so far (incl. master)
    int32_t* xid = placed + E;                                   // [512] extras: expert
    int32_t* xid_sorted = xid + kMaxExportsPerDomain;            // [512]
    int32_t* used = xid_sorted + kMaxExportsPerDomain;           // [Gpad] redundant slots used per rank
    int32_t* ctl = used + solver_gpad(G);                        // [8]
    uint32_t* holds = reinterpret_cast<uint32_t*>(ctl + 8);      // [E][ns] ranks that hold the expert

    for (int i = tid; i < G * Lp; i += nthreads) {
        a.p2l[rank0 * Lp + i] = -1;
        if (a.physical_loads != nullptr) a.physical_loads[rank0 * Lp + i] = 0;
    }
    for (int i = tid; i < E * D; i += nthreads) {
        const int64_t idx = static_cast<int64_t>(log0) * D + i;
        a.l2p[idx] = -1;
        a.quota[idx] = 0;
        a.quota_prefix[idx] = 0;
        a.rank_quota_prefix[idx] = 0;
    }
    __syncthreads();
    for (int e = tid; e < E; e += nthreads) {
        const int l = log0 + e;
        loads[e] = __ldcg(a.global_loads + l);
        cnt[e] = 1;
        placed[e] = 1;
        score[e] = static_cast<double>(loads[e]);
        const int phys = (rank0 + e / M) * Lp + e % M;
        a.p2l[phys] = l;
        a.l2p[static_cast<int64_t>(l) * D] = phys;
        for (int w = 0; w < ns; ++w) holds[e * ns + w] = 0;
        holds[e * ns + ((e / M) >> 5)] = 1u << ((e / M) & 31);
    }
    __syncthreads();
    const bool search = R > 0 && G > 1;
    if (warp == 0 && search) {
        // 1. grant the slots
        double total = 0.0;
        for (int e = lane; e < E; e += kWarp) total = __dadd_rn(total, static_cast<double>(loads[e]));  // integers: exact in any order
        for (int off = 16; off > 0; off >>= 1) total = __dadd_rn(total, __shfl_xor_sync(kFullMask, total, off));
        const double mean_per_slot = total > 0.0 ? __ddiv_rn(total, static_cast<double>(G * M)) : 0.0;
        const double stop_at = __dmul_rn(mean_per_slot, static_cast<double>(a.balance_threshold));
        for (int slot = 0; slot < G * R; ++slot) {
            double best = -1.0;
            int best_e = -1;
            for (int e = lane; e < E; e += kWarp) {
                if (cnt[e] - 1 >= G - 1) continue;
                if (score[e] > best) {  // ascending scan: equal scores keep the lower id
                    best = score[e];
                    best_e = e;
                }
            }
            for (int off = 16; off > 0; off >>= 1) {
                const double ob = __shfl_xor_sync(kFullMask, best, off);
                const int oe = __shfl_xor_sync(kFullMask, best_e, off);
                if (oe >= 0 && (best_e < 0 || ob > best || (ob == best && oe < best_e))) {
                    best = ob;
                    best_e = oe;
                }
            }
            if (a.balance_threshold > 1.0f && mean_per_slot > 0.0 && best <= stop_at) break;
            if (best_e < 0) break;
            if (lane == 0) {
                cnt[best_e] += 1;
                score[best_e] = __ddiv_rn(static_cast<double>(loads[best_e]), static_cast<double>(cnt[best_e]));
            }
            __syncwarp();
        }
        // the extra instances, expert after expert
        int n = 0;
        for (int e0 = 0; e0 < E; e0 += kWarp) {
            const int e = e0 + lane;
            const int extra = e < E ? cnt[e] - 1 : 0;
            int incl = extra;
            for (int off = 1; off < kWarp; off <<= 1) {
                const int t = __shfl_up_sync(kFullMask, incl, off);
                if (lane >= off) incl += t;
            }
            for (int j = 0; j < extra; ++j) {
                const int o = n + incl - extra + j;
                if (o < kMaxExportsPerDomain) {
                    xid[o] = e;
                    xkey[o] = score[e];
                }
            }
            n += __shfl_sync(kFullMask, incl, kWarp - 1);
        }
        if (lane == 0) ctl[0] = n < kMaxExportsPerDomain ? n : kMaxExportsPerDomain;
    }
    __syncthreads();
    if (search) {
        // order the extras: larger load per instance first, then the lower expert; instances of one expert are
        // identical, their mutual order is their list order. Rank by counting, all threads.
        const int n = ctl[0];
        for (int i = tid; i < n; i += nthreads) {
            const double k = xkey[i];
            const int e = xid[i];
            int pos = 0;
            for (int j = 0; j < n; ++j) {
                const double kj = xkey[j];
                const int ej = xid[j];
                pos += (kj > k || (kj == k && (ej < e || (ej == e && j < i)))) ? 1 : 0;
            }
            xkey_sorted[pos] = k;
            xid_sorted[pos] = e;
        }
        for (int r = tid; r < G; r += nthreads) {
            double sum = 0.0;
            for (int m = 0; m < M; ++m) sum = __dadd_rn(sum, score[r * M + m]);  // load / instances, masters in order
            rank_load[r] = sum;
            used[r] = 0;
        }
    }
    __syncthreads();
    if (warp == 0 && search) {
        // 2. place them
        const int n = ctl[0];
        for (int i = 0; i < n; ++i) {
            const int e = xid_sorted[i];
            double best = 0.0;
            int target = -1;
            for (int r = lane; r < G; r += kWarp) {
                if (used[r] >= R || ((holds[e * ns + (r >> 5)] >> (r & 31)) & 1u)) continue;
                if (target < 0 || rank_load[r] < best) {  // ascending scan: equal loads keep the lower rank
                    best = rank_load[r];
                    target = r;
                }
            }
            for (int off = 16; off > 0; off >>= 1) {
                const double ob = __shfl_xor_sync(kFullMask, best, off);
                const int ot = __shfl_xor_sync(kFullMask, target, off);
                if (ot >= 0 && (target < 0 || ob < best || (ob == best && ot < target))) {
                    best = ob;
                    target = ot;
                }
            }
            if (lane == 0) {
                if (target < 0) {
                    cnt[e] -= 1;
                } else {
                    const int l = log0 + e;
                    const int phys = (rank0 + target) * Lp + M + used[target];
                    const int slot = placed[e];
                    if (slot < D) {
                        a.p2l[phys] = l;
                        a.l2p[static_cast<int64_t>(l) * D + slot] = phys;
                    } else {
                        report_error(status, UEP_DEV_BAD_PLAN, l);
                    }
                    placed[e] = slot + 1;
                    rank_load[target] = __dadd_rn(rank_load[target], xkey_sorted[i]);
                    used[target] += 1;
                    holds[e * ns + (target >> 5)] |= 1u << (target & 31);
                }
            }
            __syncwarp();
        }
    }
    __syncthreads();
    for (int e = tid; e < E; e += nthreads) a.lcnts[log0 + e] = cnt[e];
    __syncthreads();
}

__device__ inline void solve_domain_dispatch(const SolveArgs& a, int domain, char* smem_raw, DeviceStatus* status) {
    if (a.legacy) {
        legacy_solve_domain(a, domain, smem_raw, status);
        return;
    }
    const int ns = solver_ns(a.G);
    if (ns == 1) solve_domain<1>(a, domain, smem_raw, status);
    else if (ns == 2) solve_domain<2>(a, domain, smem_raw, status);
    else solve_domain<3>(a, domain, smem_raw, status);
}

}  // namespace uep
