// CPU oracle for the per-layer expert-balancing path.
//
// THIS FILE IS TEST INFRASTRUCTURE. It is a sequential, single-file restatement of
// what the reference's CUDA kernels compute, written so that every decision
// (threshold arithmetic in fp32, tie-breaks, probe schedule of the threshold search,
// largest-remainder splits) follows the reference step by step. Only tests, the
// smoke check and the CPU-baseline leg of the benchmark may call it; the product
// path never does.
//
// Each function cites the reference file:line it follows (paths are relative to
// the reference project root).
//
// Parity status: the reference has no golden vectors for this path. This oracle is
// pinned against outputs of the reference's own kernels (built unmodified from the
// reference sources into oracle/_ref and run on a B200); the recorded outputs live
// in tests/golden/ together with the script that generated them.
//
// Build: see oracle/Makefile (g++ -O2 -ffp-contract=off; no fast-math, the grad
// reduction order and the two fp32 threshold computations must not be reassociated).

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr int kMaxReplicasPerNvl = 512;  // csrc/kernels/placement.cu:24
constexpr int kSolverWarps = 4;          // csrc/kernels/placement.cu:25-26

struct ExportEntry {
    int expert_local;
    int target_rank_local;
    int quota;
};

struct DomainState {
    int E, G, M, R;
    std::vector<int32_t> loads;          // [E] global load of each domain-local expert
    std::vector<int32_t> rank_load;      // [G]
    std::vector<int> source_order;       // [G]
    std::vector<int> sorted_experts;     // [G*M]
    // oracle state (one copy; the reference keeps one per warp, results do not depend on which)
    std::vector<int32_t> export_sum;     // [E]
    std::vector<int32_t> excess, slack, slots_used;  // [G]
    std::vector<std::vector<uint8_t>> occ;           // [E][G]
};

// csrc/kernels/placement.cu:86-109
void init_oracle_state(DomainState& s, int threshold) {
    for (int e = 0; e < s.E; ++e) {
        s.export_sum[e] = 0;
        std::fill(s.occ[e].begin(), s.occ[e].end(), 0);
        s.occ[e][e / s.M] = 1;
    }
    for (int r = 0; r < s.G; ++r) {
        s.excess[r] = std::max(s.rank_load[r] - threshold, 0);
        s.slack[r] = std::max(threshold - s.rank_load[r], 0);
        s.slots_used[r] = 0;
    }
}

// csrc/kernels/placement.cu:337-667 (batch_k == 1; register-state and shared-state
// branches compute the same thing).
bool build_export_plan(DomainState& s,
                       int threshold,
                       int min_tokens_per_replica,
                       bool allow_zero_master_quota,
                       bool use_dynamic_q_floor,
                       bool store_plan,
                       std::vector<ExportEntry>& plan) {
    (void)threshold;
    plan.clear();
    int64_t total_excess = 0, total_slack = 0;
    for (int r = 0; r < s.G; ++r) {
        total_excess += s.excess[r];
        total_slack += s.slack[r];
    }
    // The reference sums in int32; loads are far below 2^31 in every supported size.
    if (static_cast<int>(total_excess) == 0) return true;
    if (static_cast<int>(total_excess) > static_cast<int>(total_slack)) return false;

    int running_excess = static_cast<int>(total_excess);
    int running_slack = static_cast<int>(total_slack);
    for (int ord = 0; ord < s.G; ++ord) {
        const int src = s.source_order[ord];
        int need = s.excess[src];
        if (need <= 0) continue;
        if (need > running_slack) return false;  // :403-410

        for (int pos = 0; pos < s.M; ++pos) {
            const int e = s.sorted_experts[src * s.M + pos];
            const int keep = (!allow_zero_master_quota && s.loads[e] > 0) ? 1 : 0;  // :414
            int available = std::max(s.loads[e] - keep - s.export_sum[e], 0);       // :419

            while (need > 0 && available > 0) {
                int floor_tokens = min_tokens_per_replica;
                if (use_dynamic_q_floor) {  // :424-441
                    int feasible = 0;
                    for (int r = 0; r < s.G; ++r) {
                        if (s.slack[r] > 0 && s.slots_used[r] < s.R && !s.occ[e][r] &&
                            std::min(std::min(need, s.slack[r]), available) > 0) {
                            ++feasible;
                        }
                    }
                    if (feasible <= 0) break;
                    floor_tokens = std::max(1, (need + feasible - 1) / feasible);
                }
                // :159-208 — max slack, ties to the lower rank
                int best = -1, best_cap = -1;
                for (int r = 0; r < s.G; ++r) {
                    if (s.slack[r] <= 0 || s.slots_used[r] >= s.R || s.occ[e][r]) continue;
                    const int q = std::min(std::min(need, s.slack[r]), available);
                    if (q < floor_tokens) continue;
                    if (s.slack[r] > best_cap) {
                        best = r;
                        best_cap = s.slack[r];
                    }
                }
                if (best < 0) break;
                if (store_plan && static_cast<int>(plan.size()) >= kMaxReplicasPerNvl) return false;  // :519-528
                const int q = std::min(std::min(need, s.slack[best]), available);
                if (q < floor_tokens) break;  // :544
                if (store_plan) plan.push_back({e, best, q});
                s.slack[best] -= q;
                s.slots_used[best] += 1;
                s.occ[e][best] = 1;
                s.export_sum[e] += q;
                running_excess -= q;
                running_slack -= q;
                need -= q;
                available -= q;
            }
            if (need == 0) break;  // :648
        }
        if (need > 0) return false;                        // :653
        if (running_excess > running_slack) return false;  // :656-663
    }
    return true;
}

// csrc/kernels/placement.cu:76-84
bool capacity_feasible(const DomainState& s, int threshold) {
    int excess = 0, slack = 0;
    for (int r = 0; r < s.G; ++r) {
        excess += std::max(s.rank_load[r] - threshold, 0);
        slack += std::max(threshold - s.rank_load[r], 0);
    }
    return excess <= slack;
}

// csrc/kernels/placement.cu:669-786 and :1342-1481 (same arithmetic for every C)
void build_rank_quota_prefix(int row_offset,
                             int C,
                             int my_load,
                             const int32_t* per_rank_loads_of_expert,  // [G] indexed by domain-local rank
                             int domain_start_rank,
                             int num_local_physical,
                             int my_rank,
                             bool locality_aware,
                             const int32_t* quota,
                             const int32_t* l2p,
                             int32_t* rank_quota_prefix,
                             int G) {
    std::vector<int> host_rank(C), my_alloc(C, 0);
    std::vector<int64_t> remainders(C, -1);
    for (int j = 0; j < C; ++j) host_rank[j] = l2p[row_offset + j] / num_local_physical;

    if (!locality_aware) {
        const int rem_my = my_load;
        int assigned = 0, total_quota = 0;
        for (int j = 0; j < C; ++j) total_quota += quota[row_offset + j];
        if (rem_my > 0 && total_quota > 0) {
            for (int j = 0; j < C; ++j) {
                const int64_t scaled = static_cast<int64_t>(rem_my) * quota[row_offset + j];
                const int share = static_cast<int>(scaled / total_quota);
                my_alloc[j] = share;
                remainders[j] = scaled % total_quota;
                assigned += share;
            }
            int remaining = rem_my - assigned;
            while (remaining > 0) {
                int best_j = -1;
                for (int j = 0; j < C; ++j) {
                    if (best_j < 0 || remainders[j] > remainders[best_j] ||
                        (remainders[j] == remainders[best_j] && j < best_j)) {
                        best_j = j;
                    }
                }
                my_alloc[best_j] += 1;
                remainders[best_j] = -1;
                --remaining;
            }
        }
    } else {
        std::vector<int> host_remaining(G), remote_cap(C);
        for (int r = 0; r < G; ++r) host_remaining[r] = per_rank_loads_of_expert[r];
        int rem_my = my_load;
        int total_remote_cap = 0;
        for (int j = 0; j < C; ++j) {
            const int q = quota[row_offset + j];
            const int host_local = host_rank[j] - domain_start_rank;
            const int local_fill = std::min(host_remaining[host_local], q);
            host_remaining[host_local] -= local_fill;
            remote_cap[j] = q - local_fill;
            total_remote_cap += remote_cap[j];
            if (host_rank[j] == my_rank) {
                my_alloc[j] += local_fill;
                rem_my -= local_fill;
            }
        }
        rem_my = std::max(rem_my, 0);
        if (rem_my > 0 && total_remote_cap > 0) {
            int assigned = 0;
            for (int j = 0; j < C; ++j) {
                if (host_rank[j] == my_rank || remote_cap[j] <= 0) continue;
                const int64_t scaled = static_cast<int64_t>(rem_my) * remote_cap[j];
                const int share = static_cast<int>(scaled / total_remote_cap);
                my_alloc[j] += share;
                remainders[j] = scaled % total_remote_cap;
                assigned += share;
            }
            int remaining = rem_my - assigned;
            while (remaining > 0) {
                int best_j = -1;
                for (int j = 0; j < C; ++j) {
                    if (host_rank[j] == my_rank || remote_cap[j] <= 0) continue;
                    if (best_j < 0 || remainders[j] > remainders[best_j] ||
                        (remainders[j] == remainders[best_j] &&
                         (host_rank[j] < host_rank[best_j] || (host_rank[j] == host_rank[best_j] && j < best_j)))) {
                        best_j = j;
                    }
                }
                if (best_j < 0) break;  // the reference asserts; unreachable when total_remote_cap > 0
                my_alloc[best_j] += 1;
                remainders[best_j] = -1;
                --remaining;
            }
        }
    }
    int prefix = 0;
    for (int j = 0; j < C; ++j) {
        prefix += my_alloc[j];
        rank_quota_prefix[row_offset + j] = prefix;
    }
}

int gcd_int(int a, int b) {  // csrc/kernels/reroute.cu:9-16
    while (b != 0) {
        const int t = a % b;
        a = b;
        b = t;
    }
    return a;
}

// csrc/kernels/reroute.cu:182-209, 239-257: ordinal -> replica index of one logical expert
struct ExpertRouter {
    int C = 0, total = 0, stride = 1, offset = 0;
    bool interleave = false;
    const int32_t* prefix = nullptr;
    const int32_t* l2p = nullptr;

    void init(int expert_id, const int32_t* l2p_map, const int32_t* lcnts, const int32_t* rank_quota_prefix,
              int max_replicas, bool interleave_by_rank_quota) {
        C = lcnts[expert_id];
        prefix = rank_quota_prefix + static_cast<int64_t>(expert_id) * max_replicas;
        l2p = l2p_map + static_cast<int64_t>(expert_id) * max_replicas;
        total = C > 0 ? prefix[C - 1] : 0;
        interleave = interleave_by_rank_quota && total > 1;
        stride = 1;
        offset = 0;
        if (interleave) {
            int s = total / 2 + 1;
            if (s >= total) s = total - 1;
            if (s < 1) s = 1;
            while (gcd_int(s, total) != 1) {
                ++s;
                if (s >= total) s = 1;
            }
            stride = s;
            offset = expert_id % total;
        }
    }
    int physical(int ordinal) const {
        int quota_rank = ordinal;
        if (interleave) {
            quota_rank = static_cast<int>((static_cast<int64_t>(ordinal) * stride + offset) % total);
        }
        int idx = 0;
        for (int j = 0; j < C; ++j) idx += (quota_rank >= prefix[j]) ? 1 : 0;
        idx = std::min(idx, std::max(C - 1, 0));
        return l2p[idx];
    }
};

}  // namespace

extern "C" {

// csrc/kernels/load_compute.cu:85-129 (sparse ids; ids outside [0,L) are ignored) with
// either int32 or int64 ids, and :7-73 (dense bool map).
void uep_oracle_histogram_ids32(const int32_t* ids, int64_t n, int L, int32_t* loads) {
    std::fill(loads, loads + L, 0);
    for (int64_t i = 0; i < n; ++i) {
        const int32_t e = ids[i];
        if (e >= 0 && e < L) loads[e] += 1;
    }
}
void uep_oracle_histogram_ids64(const int64_t* ids, int64_t n, int L, int32_t* loads) {
    std::fill(loads, loads + L, 0);
    for (int64_t i = 0; i < n; ++i) {
        const int64_t e = ids[i];
        if (e >= 0 && e < L) loads[e] += 1;
    }
}
void uep_oracle_histogram_map(const uint8_t* routing_map, int T, int L, int32_t* loads) {
    std::fill(loads, loads + L, 0);
    for (int t = 0; t < T; ++t)
        for (int l = 0; l < L; ++l) loads[l] += routing_map[static_cast<int64_t>(t) * L + l] ? 1 : 0;
}

// csrc/kernels/load_compute.cu:131-151
void uep_oracle_reduce_loads(const int32_t* per_rank, int N, int L, int32_t* global_loads) {
    for (int l = 0; l < L; ++l) {
        int32_t total = 0;
        for (int r = 0; r < N; ++r) total += per_rank[static_cast<int64_t>(r) * L + l];
        global_loads[l] = total;
    }
}

// csrc/kernels/placement.cu:1486-1559 — masters-only plan written at construction time.
void uep_oracle_init_master_placement(int32_t* p2l, int32_t* l2p, int32_t* lcnts, int32_t* quota,
                                      int32_t* quota_prefix, int32_t* rank_quota_prefix, int num_ranks, int M,
                                      int R, int D) {
    const int Lp = M + R, L = num_ranks * M, P = num_ranks * Lp;
    std::fill(p2l, p2l + P, -1);
    std::fill(l2p, l2p + static_cast<int64_t>(L) * D, -1);
    std::fill(lcnts, lcnts + L, 0);
    std::fill(quota, quota + static_cast<int64_t>(L) * D, 0);
    std::fill(quota_prefix, quota_prefix + static_cast<int64_t>(L) * D, 0);
    std::fill(rank_quota_prefix, rank_quota_prefix + static_cast<int64_t>(L) * D, 0);
    for (int l = 0; l < L; ++l) {
        const int phys = (l / M) * Lp + l % M;
        p2l[phys] = l;
        l2p[static_cast<int64_t>(l) * D] = phys;
        lcnts[l] = 1;
    }
}

// csrc/kernels/legacy/placement_cpu.cpp:17-172 — the host-side solver of legacy_placement=True, per
// NVLink domain: (1) redundant slots are granted one at a time to the expert with the largest load per
// instance (ties: lower id; an expert gets at most G-1 extra instances; with balance_threshold > 1 the
// granting stops once the best load per instance is within threshold x the mean load per master slot);
// (2) the extra instances, ordered by load per instance descending then expert id, go to the rank with the
// smallest accumulated load (ties: lower rank) that has a free slot and does not hold the expert yet; an
// instance that finds no rank is dropped. Loads per instance are doubles, as in the reference. Quotas are
// not used in this mode (the reroute is round-robin), the caller zeroes them (:235-240).
void uep_oracle_legacy_solve_placement(const int32_t* expert_loads, int32_t* p2l, int32_t* l2p, int32_t* lcnts,
                                       int num_ranks, int M, int R, int nvl_ranks, int D, float balance_threshold) {
    const int Lp = M + R, L = num_ranks * M, P = num_ranks * Lp, E = nvl_ranks * M;
    std::fill(p2l, p2l + P, -1);
    std::fill(l2p, l2p + static_cast<int64_t>(L) * D, -1);
    for (int l = 0; l < L; ++l) {
        const int phys = (l / M) * Lp + l % M;
        p2l[phys] = l;
        l2p[static_cast<int64_t>(l) * D] = phys;
        lcnts[l] = 1;
    }
    if (R == 0 || nvl_ranks <= 1) return;
    for (int dom = 0; dom < num_ranks / nvl_ranks; ++dom) {
        const int rank0 = dom * nvl_ranks, log0 = rank0 * M;
        double total = 0.0;
        for (int e = 0; e < E; ++e) total += expert_loads[log0 + e];
        const double mean_per_slot = total > 0.0 ? total / (nvl_ranks * M) : 0.0;
        // (1) how many instances each expert gets
        for (int slot = 0; slot < nvl_ranks * R; ++slot) {
            int best = -1;
            double best_score = -1.0;
            for (int e = 0; e < E; ++e) {
                const int l = log0 + e;
                if (lcnts[l] - 1 >= nvl_ranks - 1) continue;
                const double score = static_cast<double>(expert_loads[l]) / lcnts[l];
                if (score > best_score) {  // equal scores keep the lower id (ascending scan)
                    best_score = score;
                    best = l;
                }
            }
            if (balance_threshold > 1.0f && mean_per_slot > 0.0 && best_score <= mean_per_slot * balance_threshold) break;
            if (best < 0) break;
            lcnts[best] += 1;
        }
        // (2) where the extra instances live
        struct Extra {
            int l;
            double per_instance;
        };
        std::vector<Extra> extras;
        for (int e = 0; e < E; ++e) {
            const int l = log0 + e;
            for (int j = 1; j < lcnts[l]; ++j) extras.push_back({l, static_cast<double>(expert_loads[l]) / lcnts[l]});
        }
        std::stable_sort(extras.begin(), extras.end(), [](const Extra& a, const Extra& b) {
            return a.per_instance != b.per_instance ? a.per_instance > b.per_instance : a.l < b.l;
        });
        std::vector<double> rank_load(nvl_ranks, 0.0);
        std::vector<int> used(nvl_ranks, 0);
        std::vector<char> holds(static_cast<size_t>(nvl_ranks) * E, 0);
        for (int r = 0; r < nvl_ranks; ++r) {
            for (int m = 0; m < M; ++m) {
                const int l = (rank0 + r) * M + m;
                rank_load[r] += static_cast<double>(expert_loads[l]) / lcnts[l];
                holds[static_cast<size_t>(r) * E + r * M + m] = 1;
            }
        }
        for (const Extra& x : extras) {
            const int e = x.l - log0;
            int target = -1;
            for (int r = 0; r < nvl_ranks; ++r) {
                if (used[r] >= R || holds[static_cast<size_t>(r) * E + e]) continue;
                if (target < 0 || rank_load[r] < rank_load[target]) target = r;
            }
            if (target < 0) {
                lcnts[x.l] -= 1;
                continue;
            }
            const int phys = (rank0 + target) * Lp + M + used[target];
            p2l[phys] = x.l;
            int32_t* row = l2p + static_cast<int64_t>(x.l) * D;
            for (int j = 1; j < D; ++j) {
                if (row[j] == -1) {
                    row[j] = phys;
                    break;
                }
            }
            rank_load[target] += x.per_instance;
            used[target] += 1;
            holds[static_cast<size_t>(target) * E + e] = 1;
        }
    }
}

// csrc/kernels/placement.cu:788-1482 (kernel) and :1561-1663 (pre-clears + launch).
// Returns 0 on success; -1 on a parameter outside the reference's static limits
// (:1589-1597); -2 if the final rebuild is infeasible (the reference traps, :1277).
int uep_oracle_solve_placement(const int32_t* expert_loads,           // [L]
                               const int32_t* expert_loads_per_rank,  // [N, L]
                               int32_t* p2l,                          // [P]
                               int32_t* l2p,                          // [L, D]
                               int32_t* lcnts,                        // [L]
                               int32_t* quota,                        // [L, D]
                               int32_t* quota_prefix,                 // [L, D]
                               int32_t* rank_quota_prefix,            // [L, D]
                               int num_ranks, int num_nvl_ranks, int M, int R, int D, float balance_threshold,
                               int32_t min_tokens_per_replica, int allow_zero_master_quota, int locality_aware,
                               float oracle_eps, int my_rank, int32_t* out_threshold /* [num_domains] or null */,
                               int32_t* out_path /* [num_domains] or null: low 4 bits 0 none,1 fast,2 precheck,3 search */) {
    const int N = num_ranks, G = num_nvl_ranks;
    if (G <= 0 || N % G != 0 || M <= 0 || R < 0 || D < 1) return -1;
    const int Lp = M + R, L = N * M, P = N * Lp, E = G * M;
    if (E > 512 || G > 72 || G * R > 512) return -1;
    const int num_domains = N / G;

    // :1602-1625
    std::fill(p2l, p2l + P, -1);
    std::fill(l2p, l2p + static_cast<int64_t>(L) * D, -1);
    std::fill(lcnts, lcnts + L, 0);
    std::fill(quota, quota + static_cast<int64_t>(L) * D, 0);
    std::fill(quota_prefix, quota_prefix + static_cast<int64_t>(L) * D, 0);
    std::fill(rank_quota_prefix, rank_quota_prefix + static_cast<int64_t>(L) * D, 0);

    for (int domain = 0; domain < num_domains; ++domain) {
        const int domain_start_rank = domain * G;
        const int domain_start_log = domain_start_rank * M;
        DomainState s;
        s.E = E; s.G = G; s.M = M; s.R = R;
        s.loads.resize(E); s.rank_load.resize(G); s.source_order.resize(G); s.sorted_experts.resize(E);
        s.export_sum.assign(E, 0); s.excess.resize(G); s.slack.resize(G); s.slots_used.resize(G);
        s.occ.assign(E, std::vector<uint8_t>(G, 0));

        // :869-889
        for (int i = 0; i < E; ++i) {
            const int l_global = domain_start_log + i;
            s.loads[i] = expert_loads[l_global];
            const int phys = (domain_start_rank + i / M) * Lp + i % M;
            p2l[phys] = l_global;
            l2p[static_cast<int64_t>(l_global) * D] = phys;
        }
        for (int r = 0; r < G; ++r) {
            int sum = 0;
            for (int m = 0; m < M; ++m) sum += s.loads[r * M + m];
            s.rank_load[r] = sum;
        }
        // :64-74 — ranks by load descending, ties to the lower index
        for (int i = 0; i < G; ++i) {
            int pos = 0;
            for (int j = 0; j < G; ++j) {
                pos += (s.rank_load[j] > s.rank_load[i] || (s.rank_load[j] == s.rank_load[i] && j < i)) ? 1 : 0;
            }
            s.source_order[pos] = i;
        }
        // :897-917 — each rank's masters by load descending, ties to the lower index
        for (int r = 0; r < G; ++r) {
            int* row = s.sorted_experts.data() + r * M;
            for (int m = 0; m < M; ++m) row[m] = r * M + m;
            std::stable_sort(row, row + M, [&](int a, int b) {
                return s.loads[a] > s.loads[b] || (s.loads[a] == s.loads[b] && a < b);
            });
        }

        const bool do_search = (R > 0 && G > 1);  // :955
        std::vector<ExportEntry> plan;
        int path = 0, final_threshold = 0, small_rounds = 0, wide_rounds = 0;
        if (do_search) {
            // :961-970 — fp32 arithmetic
            int total_rank_load = 0, max_rank_load = 0;
            for (int r = 0; r < G; ++r) {
                total_rank_load += s.rank_load[r];
                max_rank_load = std::max(max_rank_load, static_cast<int>(s.rank_load[r]));
            }
            const float bt = fmaxf(balance_threshold, 1.0f);
            volatile float mean = static_cast<float>(total_rank_load) / static_cast<float>(G);
            volatile float scaled = mean * bt;
            int bs_lo = static_cast<int>(ceilf(scaled));
            int bs_hi = std::max(max_rank_load, bs_lo);

            // :1000-1062 — fast path: up to 3 builds with the dynamic floor
            bool fast_done = false;
            {
                const float eps = fmaxf(oracle_eps, 0.0f);
                volatile float one_plus = 1.0f + eps;
                volatile float prod = static_cast<float>(bs_lo) * one_plus;
                int fast_threshold = static_cast<int>(ceilf(prod));
                fast_threshold = std::max(fast_threshold, bs_lo);
                const int fast_step = std::max(1, (bs_hi + 99) / 100);
                for (int retry = 0; retry <= 2 && !fast_done; ++retry) {
                    init_oracle_state(s, fast_threshold);
                    const bool ok = build_export_plan(s, fast_threshold, min_tokens_per_replica,
                                                      allow_zero_master_quota != 0, true, true, plan);
                    if (ok) {
                        fast_done = true;
                        bs_lo = fast_threshold;
                        path = 1;
                    } else {
                        fast_threshold = std::min(bs_hi, fast_threshold + fast_step);
                    }
                }
            }
            if (!fast_done) {
                // :1066-1080 coarse bisection on capacity feasibility
                int coarse_lo = bs_lo, coarse_hi = bs_hi;
                while (coarse_lo < coarse_hi) {
                    const int probe = coarse_lo + ((coarse_hi - coarse_lo) >> 1);
                    if (capacity_feasible(s, probe)) coarse_hi = probe;
                    else coarse_lo = probe + 1;
                }
                bs_lo = coarse_lo;
                // :1086-1129 precheck with the static floor
                init_oracle_state(s, bs_lo);
                bool precheck = build_export_plan(s, bs_lo, min_tokens_per_replica, allow_zero_master_quota != 0,
                                                  false, true, plan);
                if (precheck) path = 2;
                else bs_lo = std::min(bs_lo + 1, bs_hi);

                // :1133-1236 four probes per round
                std::vector<ExportEntry> scratch;
                while (!(precheck || bs_lo >= bs_hi)) {
                    const int range = bs_hi - bs_lo;
                    const bool small = range <= kSolverWarps;
                    if (small) ++small_rounds; else ++wide_rounds;
                    int probes[kSolverWarps], valid[kSolverWarps], feasible[kSolverWarps];
                    for (int w = 0; w < kSolverWarps; ++w) {
                        if (small) {
                            probes[w] = bs_lo + w;
                            valid[w] = probes[w] < bs_hi ? 1 : 0;
                        } else {
                            probes[w] = bs_lo + static_cast<int>((static_cast<int64_t>(range) * (w + 1)) /
                                                                 (kSolverWarps + 1));
                            valid[w] = 1;
                        }
                        feasible[w] = 0;
                        if (valid[w]) {
                            init_oracle_state(s, probes[w]);
                            feasible[w] = build_export_plan(s, probes[w], min_tokens_per_replica,
                                                            allow_zero_master_quota != 0, false, false, scratch)
                                              ? 1 : 0;
                        }
                    }
                    if (small) {
                        int best_probe = -1;
                        for (int w = 0; w < kSolverWarps; ++w) {
                            if (valid[w] && feasible[w]) { best_probe = probes[w]; break; }
                        }
                        if (best_probe >= 0) { bs_lo = best_probe; bs_hi = best_probe; }
                        else bs_lo = bs_hi;
                    } else {
                        int first = -1;
                        for (int w = 0; w < kSolverWarps; ++w) {
                            if (feasible[w]) { first = w; break; }
                        }
                        if (first >= 0) {
                            bs_hi = probes[first];
                            if (first > 0) bs_lo = probes[first - 1] + 1;
                        } else {
                            bs_lo = probes[kSolverWarps - 1] + 1;
                        }
                    }
                }
                if (!precheck) {  // :1238-1282
                    init_oracle_state(s, bs_lo);
                    const bool ok = build_export_plan(s, bs_lo, min_tokens_per_replica,
                                                      allow_zero_master_quota != 0, false, true, plan);
                    if (!ok) return -2;
                    path = 3;
                }
            }
            final_threshold = bs_lo;
        }
        if (out_threshold) out_threshold[domain] = final_threshold;
        // low nibble: branch taken; then the number of small-range and wide-range probe rounds
        if (out_path) out_path[domain] = path | (std::min(small_rounds, 255) << 4) | (std::min(wide_rounds, 255) << 12);

        // :1286-1331 emit
        std::vector<int> next_slot(G, 0), expert_slot(E, 1);
        for (int e = 0; e < E; ++e) {
            const int64_t row = static_cast<int64_t>(domain_start_log + e) * D;
            quota[row] = do_search ? (s.loads[e] - s.export_sum[e]) : s.loads[e];
        }
        for (const ExportEntry& entry : plan) {
            const int l_global = domain_start_log + entry.expert_local;
            const int64_t row = static_cast<int64_t>(l_global) * D;
            const int slot = expert_slot[entry.expert_local]++;
            const int phys = (domain_start_rank + entry.target_rank_local) * Lp + M + next_slot[entry.target_rank_local]++;
            p2l[phys] = l_global;
            l2p[row + slot] = phys;
            quota[row + slot] = entry.quota;
        }
        for (int e = 0; e < E; ++e) {
            const int l_global = domain_start_log + e;
            const int64_t row = static_cast<int64_t>(l_global) * D;
            const int C = expert_slot[e];
            lcnts[l_global] = C;
            int prefix = 0;
            for (int j = 0; j < C; ++j) {
                prefix += quota[row + j];
                quota_prefix[row + j] = prefix;
            }
        }
        // :1342-1481 rank-specific split
        std::vector<int32_t> per_rank_of_expert(G);
        for (int e = 0; e < E; ++e) {
            const int l_global = domain_start_log + e;
            for (int r = 0; r < G; ++r) {
                per_rank_of_expert[r] = expert_loads_per_rank[static_cast<int64_t>(domain_start_rank + r) * L + l_global];
            }
            const int my_load = expert_loads_per_rank[static_cast<int64_t>(my_rank) * L + l_global];
            build_rank_quota_prefix(static_cast<int>(static_cast<int64_t>(l_global) * D), lcnts[l_global], my_load,
                                    per_rank_of_expert.data(), domain_start_rank, Lp, my_rank, locality_aware != 0,
                                    quota, l2p, rank_quota_prefix, G);
        }
    }
    return 0;
}

// csrc/kernels/reroute.cu:21-51, 138-264 (dense quota reroute; outputs fully written,
// zero where not routed, as the reference's zero-fill + scatter leaves them).
void uep_oracle_dense_reroute_forward(const uint8_t* routing_map, const float* probs, const int32_t* l2p,
                                      const int32_t* lcnts, const int32_t* rank_quota_prefix, uint8_t* expanded_map,
                                      float* expanded_probs, int T, int L, int P, int max_replicas,
                                      int interleave) {
    std::memset(expanded_map, 0, static_cast<size_t>(T) * P);
    std::memset(expanded_probs, 0, static_cast<size_t>(T) * P * sizeof(float));
    for (int e = 0; e < L; ++e) {
        ExpertRouter router;
        router.init(e, l2p, lcnts, rank_quota_prefix, max_replicas, interleave != 0);
        int ordinal = 0;
        for (int t = 0; t < T; ++t) {
            if (!routing_map[static_cast<int64_t>(t) * L + e]) continue;
            const int phys = router.physical(ordinal++);
            expanded_map[static_cast<int64_t>(t) * P + phys] = 1;
            expanded_probs[static_cast<int64_t>(t) * P + phys] = probs[static_cast<int64_t>(t) * L + e];
        }
    }
}

// Round-robin variant, csrc/kernels/reroute.cu:56-136 (legacy placement mode).
void uep_oracle_dense_reroute_forward_rr(const uint8_t* routing_map, const float* probs, const int32_t* l2p,
                                         const int32_t* lcnts, uint8_t* expanded_map, float* expanded_probs, int T,
                                         int L, int P, int max_replicas) {
    std::memset(expanded_map, 0, static_cast<size_t>(T) * P);
    std::memset(expanded_probs, 0, static_cast<size_t>(T) * P * sizeof(float));
    for (int e = 0; e < L; ++e) {
        const int C = lcnts[e];
        int ordinal = 0;
        for (int t = 0; t < T; ++t) {
            if (!routing_map[static_cast<int64_t>(t) * L + e]) continue;
            const int phys = l2p[static_cast<int64_t>(e) * max_replicas + (ordinal++ % C)];
            expanded_map[static_cast<int64_t>(t) * P + phys] = 1;
            expanded_probs[static_cast<int64_t>(t) * P + phys] = probs[static_cast<int64_t>(t) * L + e];
        }
    }
}

// Sparse form of the same rule: the ordinal of entry (t,k) is the number of entries
// before it in row-major order that name the same logical expert. With at most one
// entry per (token, expert) this is exactly the dense rule above applied per (t,k).
// The reference's own sparse kernel (csrc/kernels/reroute.cu:492-515) takes ordinals
// from an atomic counter, so only its per-(expert, replica) counts are defined; it
// also never interleaves. Ids outside [0,L) and experts with C <= 0 are left unchanged.
void uep_oracle_sparse_reroute32(const int32_t* ids, int32_t* out, int64_t n, int L, const int32_t* l2p,
                                 const int32_t* lcnts, const int32_t* rank_quota_prefix, int max_replicas,
                                 int interleave) {
    std::vector<ExpertRouter> routers(L);
    std::vector<int> counters(L, 0);
    for (int e = 0; e < L; ++e) routers[e].init(e, l2p, lcnts, rank_quota_prefix, max_replicas, interleave != 0);
    for (int64_t i = 0; i < n; ++i) {
        const int32_t e = ids[i];
        if (e < 0 || e >= L || routers[e].C <= 0) {
            out[i] = e;
            continue;
        }
        out[i] = routers[e].physical(counters[e]++);
    }
}
void uep_oracle_sparse_reroute64(const int64_t* ids, int64_t* out, int64_t n, int L, const int32_t* l2p,
                                 const int32_t* lcnts, const int32_t* rank_quota_prefix, int max_replicas,
                                 int interleave) {
    std::vector<ExpertRouter> routers(L);
    std::vector<int> counters(L, 0);
    for (int e = 0; e < L; ++e) routers[e].init(e, l2p, lcnts, rank_quota_prefix, max_replicas, interleave != 0);
    for (int64_t i = 0; i < n; ++i) {
        const int64_t e = ids[i];
        if (e < 0 || e >= L || routers[e].C <= 0) {
            out[i] = e;
            continue;
        }
        out[i] = routers[e].physical(counters[e]++);
    }
}

// csrc/kernels/reroute.cu:269-297 (output zero-filled by the caller, csrc/ultra_ep.cpp:961)
void uep_oracle_dense_reroute_backward(const float* grad_expanded, const uint8_t* routing_map,
                                       const uint8_t* expanded_map, const int32_t* l2p, const int32_t* lcnts,
                                       float* grad_probs, int T, int L, int P, int max_replicas) {
    std::memset(grad_probs, 0, static_cast<size_t>(T) * L * sizeof(float));
    for (int t = 0; t < T; ++t) {
        for (int l = 0; l < L; ++l) {
            const int64_t idx = static_cast<int64_t>(t) * L + l;
            if (!routing_map[idx]) continue;
            const int C = lcnts[l];
            for (int r = 0; r < C; ++r) {
                const int phys = l2p[static_cast<int64_t>(l) * max_replicas + r];
                if (expanded_map[static_cast<int64_t>(t) * P + phys]) {
                    grad_probs[idx] = grad_expanded[static_cast<int64_t>(t) * P + phys];
                    break;
                }
            }
        }
    }
}

// Dispatch order of the (token, k) entries: a stable counting sort by physical expert id.
// pos[i] is the row that entry i occupies once entries are grouped by physical expert
// (entries with ids outside [0,P) go last, in order). No counterpart in the reference:
// its dispatcher is external; this defines the row order used by the token-gradient gather.
void uep_oracle_dispatch_positions(const int32_t* phys_ids, int64_t n, int P, int32_t* pos,
                                   int32_t* expert_offsets /* [P+1] or null */) {
    std::vector<int64_t> count(P + 1, 0);
    for (int64_t i = 0; i < n; ++i) {
        const int32_t p = phys_ids[i];
        count[(p >= 0 && p < P) ? p : P] += 1;
    }
    std::vector<int64_t> base(P + 2, 0);
    for (int p = 0; p <= P; ++p) base[p + 1] = base[p] + count[p];
    if (expert_offsets)
        for (int p = 0; p <= P; ++p) expert_offsets[p] = static_cast<int32_t>(base[p]);
    std::vector<int64_t> cursor(base.begin(), base.end() - 1);
    for (int64_t i = 0; i < n; ++i) {
        const int32_t p = phys_ids[i];
        pos[i] = static_cast<int32_t>(cursor[(p >= 0 && p < P) ? p : P]++);
    }
}

// Token-gradient gather back to logical (token, k) order: out[i, :] = in[pos[i], :].
// Rows are opaque 2-byte elements (bf16); the copy is bit-exact by construction.
void uep_oracle_gather_rows16(const uint16_t* in, const int32_t* pos, uint16_t* out, int64_t n, int hidden) {
    for (int64_t i = 0; i < n; ++i)
        std::memcpy(out + i * hidden, in + static_cast<int64_t>(pos[i]) * hidden, static_cast<size_t>(hidden) * 2);
}

// weight_sync on rank `rank`: what this rank's redundant slots hold afterwards.
// Follows csrc/kernels/weight_sync.cu:242-292 (direct fan-out; slot = phys % Lp - M,
// shards at the offsets of :37-64) seen from the receiving side. masters[r*M+m] points
// at the contiguous bytes of one master shard on rank r. Unused slots are untouched.
void uep_oracle_weight_sync_recv(int rank, int M, int R, const int32_t* p2l, const int32_t* l2p, int D,
                                 const uint8_t* const* master_shard /* [N*M] */, int64_t shard_bytes,
                                 uint8_t* replica_buf, int64_t slot_stride_bytes, int64_t shard_offset_bytes) {
    const int Lp = M + R;
    for (int s = 0; s < R; ++s) {
        const int logical = p2l[rank * Lp + M + s];
        if (logical < 0) continue;
        const int master_phys = l2p[static_cast<int64_t>(logical) * D];
        const int master_rank = master_phys / Lp, master_local = master_phys % Lp;
        std::memcpy(replica_buf + s * slot_stride_bytes + shard_offset_bytes,
                    master_shard[master_rank * M + master_local], static_cast<size_t>(shard_bytes));
    }
}

// Replica Wgrad reduce for one shard of one local master:
// master = ((master + g_1) + g_2) + ... in fp32, replicas in l2p slot order, then each
// consumed replica region is zeroed. csrc/kernels/grad_reduce.cu:41-69 (task order),
// :344-383 (accumulation order), :377 (zeroing).
void uep_oracle_grad_reduce_shard(float* master, float* const* replicas, int num_replicas, int64_t numel) {
    for (int64_t i = 0; i < numel; ++i) {
        float acc = master[i];
        for (int j = 0; j < num_replicas; ++j) acc = acc + replicas[j][i];
        master[i] = acc;
    }
    for (int j = 0; j < num_replicas; ++j) std::memset(replicas[j], 0, static_cast<size_t>(numel) * sizeof(float));
}

// ---------------------------------------------------------------------------------
// Timed CPU baseline: one layer of the forward path for all N ranks of one NVLink
// domain on host threads. Histogram -> all-gather (shared memory) -> reduce -> solve
// (every rank solves redundantly, as on the GPU) -> sparse reroute -> weight_sync
// (memcpy of each used redundant slot). Returns seconds of wall time for `iters`
// repetitions; threads = min(num_threads, N). Outputs land in caller buffers so the
// benchmark can cross-check them.
// ---------------------------------------------------------------------------------
double uep_oracle_time_forward_layer(const int32_t* ids /* [N, T*K] */, int T, int K, int N, int M, int R,
                                     float balance_threshold, int32_t min_tokens, int allow_zero, int locality,
                                     float eps, int interleave, const uint8_t* const* master_bytes /* [N*M] or null */,
                                     int64_t expert_bytes, uint8_t* const* replica_bufs /* [N] or null */,
                                     int32_t* out_plan_p2l /* [P] from rank 0 */, int32_t* out_phys_ids /* [N,T*K] */,
                                     int iters, int num_threads, double* out_plan_s, double* out_reroute_s,
                                     double* out_sync_s) {
    const int L = N * M, Lp = M + R, P = N * Lp, D = N;
    const int64_t n = static_cast<int64_t>(T) * K;
    std::vector<int32_t> per_rank(static_cast<size_t>(N) * L), global_loads(L);
    struct RankPlan {
        std::vector<int32_t> p2l, l2p, lcnts, quota, qp, rqp;
    };
    std::vector<RankPlan> plans(N);
    for (auto& p : plans) {
        p.p2l.resize(P); p.l2p.resize(static_cast<size_t>(L) * D); p.lcnts.resize(L);
        p.quota.resize(static_cast<size_t>(L) * D); p.qp.resize(static_cast<size_t>(L) * D);
        p.rqp.resize(static_cast<size_t>(L) * D);
    }
    const int nt = std::max(1, std::min(num_threads, N));
    auto parallel_ranks = [&](auto&& fn) {
        std::vector<std::thread> pool;
        std::atomic<int> next{0};
        for (int t = 0; t < nt; ++t) {
            pool.emplace_back([&] {
                for (int r = next.fetch_add(1); r < N; r = next.fetch_add(1)) fn(r);
            });
        }
        for (auto& th : pool) th.join();
    };
    double plan_s = 0, reroute_s = 0, sync_s = 0;
    const auto t_begin = std::chrono::steady_clock::now();
    for (int it = 0; it < iters; ++it) {
        auto t0 = std::chrono::steady_clock::now();
        parallel_ranks([&](int r) { uep_oracle_histogram_ids32(ids + r * n, n, L, per_rank.data() + static_cast<size_t>(r) * L); });
        uep_oracle_reduce_loads(per_rank.data(), N, L, global_loads.data());
        parallel_ranks([&](int r) {
            RankPlan& p = plans[r];
            uep_oracle_solve_placement(global_loads.data(), per_rank.data(), p.p2l.data(), p.l2p.data(),
                                       p.lcnts.data(), p.quota.data(), p.qp.data(), p.rqp.data(), N, N, M, R, D,
                                       balance_threshold, min_tokens, allow_zero, locality, eps, r, nullptr, nullptr);
        });
        auto t1 = std::chrono::steady_clock::now();
        parallel_ranks([&](int r) {
            RankPlan& p = plans[r];
            uep_oracle_sparse_reroute32(ids + r * n, out_phys_ids + r * n, n, L, p.l2p.data(), p.lcnts.data(),
                                        p.rqp.data(), D, interleave);
        });
        auto t2 = std::chrono::steady_clock::now();
        if (master_bytes && replica_bufs) {
            parallel_ranks([&](int r) {
                RankPlan& p = plans[r];
                uep_oracle_weight_sync_recv(r, M, R, p.p2l.data(), p.l2p.data(), D, master_bytes, expert_bytes,
                                            replica_bufs[r], expert_bytes, 0);
            });
        }
        auto t3 = std::chrono::steady_clock::now();
        plan_s += std::chrono::duration<double>(t1 - t0).count();
        reroute_s += std::chrono::duration<double>(t2 - t1).count();
        sync_s += std::chrono::duration<double>(t3 - t2).count();
    }
    const auto t_end = std::chrono::steady_clock::now();
    if (out_plan_p2l) std::memcpy(out_plan_p2l, plans[0].p2l.data(), sizeof(int32_t) * P);
    if (out_plan_s) *out_plan_s = plan_s;
    if (out_reroute_s) *out_reroute_s = reroute_s;
    if (out_sync_s) *out_sync_s = sync_s;
    return std::chrono::duration<double>(t_end - t_begin).count();
}

int uep_oracle_hardware_threads() { return static_cast<int>(std::thread::hardware_concurrency()); }

}  // extern "C"
