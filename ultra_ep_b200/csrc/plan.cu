// Kernel 1 — the plan: per-expert token counts, load all-gather over peer memory,
// reduction and placement solve in ONE launch per layer.
//
// What the reference does with about a dozen stream operations (memset + histogram,
// device copy, NVSHMEM fcollect, reduce kernel, six memsets, solver kernel;
// csrc/ultra_ep.cpp:676-745 and csrc/kernels/placement.cu:1602-1663 of the reference)
// is one kernel here:
//   * every CTA of a rank counts a slice of the routing input into shared memory; all but the
//     rank's first CTA store their partial counts as self-validating 64-bit words (epoch
//     tag << 32 | count; an aligned 8-byte store is single-copy atomic, so a word needs neither
//     a fence nor a flag) into a row of their own and are done;
//   * the rank's first CTA owns the rest: it adds up the partials (bounded wait on words of
//     its own launch's CTAs, none of which waits for it), stores the row into every peer's
//     gather buffer as the same kind of words, polls its own buffer (bounded) until every
//     rank's words carry this epoch's tag, reduces the matrix and runs the solver (solver.cuh).
// The gather buffers are double-buffered by epoch parity: a peer can be at most one
// call ahead, because it cannot pass call e+1 without this rank's row for e+1.
//
// With several ranks hosted on one device (simulated EP) the same kernel runs all of
// them in one cooperative launch, so the ranks that wait for each other are co-resident.

#include <cooperative_groups.h>

#include <atomic>

#include <algorithm>
#include <cstring>

#include "internal.h"
#include "solver.cuh"

namespace uep {

namespace {

constexpr int kPlanThreads = 256;

__device__ __forceinline__ void hist_add_swar(uint32_t word, int32_t* hist, int col) {
    // four byte-wide counters packed in `word`
    const int c0 = word & 0xFF, c1 = (word >> 8) & 0xFF, c2 = (word >> 16) & 0xFF, c3 = word >> 24;
    if (c0) atomicAdd(hist + col, c0);
    if (c1) atomicAdd(hist + col + 1, c1);
    if (c2) atomicAdd(hist + col + 2, c2);
    if (c3) atomicAdd(hist + col + 3, c3);
}

// Count this CTA's slice of the input into hist[L] (shared memory, zeroed by the caller).
// part / nparts split the rows (dense) or the entries (sparse) evenly.
// (not inlined: its vector-load registers must not add to the solver's register pressure in plan_kernel)
__device__ __noinline__ void histogram_slice(int input_kind, const void* input, int T, int K_or_L, int L, int part, int nparts,
                                int32_t* hist) {
    const int tid = threadIdx.x, nthreads = blockDim.x;
    if (input_kind == 0) {
        const uint8_t* map = static_cast<const uint8_t*>(input);
        const int rows_per = ceil_div_i(T, nparts);
        const int r0 = min(part * rows_per, T), r1 = min(r0 + rows_per, T);
        const bool vec_ok = (L % 16 == 0) && ((reinterpret_cast<uintptr_t>(map) & 15u) == 0) && (nthreads % (L / 16) == 0);
        if (vec_ok) {
            // one thread owns a 16-column group and walks rows; 0/1 bytes are summed four at a
            // time inside 32-bit words and spilled to the histogram before a byte can overflow
            const int groups = L / 16;
            const int g = tid % groups;
            const int row_lane = tid / groups, row_lanes = nthreads / groups;
            uint4 acc = make_uint4(0, 0, 0, 0);
            int pending = 0;
            for (int r = r0 + row_lane; r < r1; r += row_lanes) {
                const uint4 v = ld_global_nc_v4(map + static_cast<int64_t>(r) * L + g * 16);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                if (++pending == 255) {
                    hist_add_swar(acc.x, hist, g * 16); hist_add_swar(acc.y, hist, g * 16 + 4);
                    hist_add_swar(acc.z, hist, g * 16 + 8); hist_add_swar(acc.w, hist, g * 16 + 12);
                    acc = make_uint4(0, 0, 0, 0);
                    pending = 0;
                }
            }
            hist_add_swar(acc.x, hist, g * 16); hist_add_swar(acc.y, hist, g * 16 + 4);
            hist_add_swar(acc.z, hist, g * 16 + 8); hist_add_swar(acc.w, hist, g * 16 + 12);
        } else {
            const int64_t begin = static_cast<int64_t>(r0) * L, end = static_cast<int64_t>(r1) * L;
            for (int64_t i = begin + tid; i < end; i += nthreads) {
                if (map[i]) atomicAdd(hist + static_cast<int>(i % L), 1);
            }
        }
    } else {
        const int64_t n = static_cast<int64_t>(T) * K_or_L;
        // slices start at multiples of four entries so that aligned inputs can be read 16 bytes at a time;
        // a thread issues all of its vector loads before it touches the first result
        const int64_t per = ((n + nparts - 1) / nparts + 3) & ~static_cast<int64_t>(3);
        const int64_t begin = min(static_cast<int64_t>(part) * per, n), end = min(begin + per, n);
        if (input_kind == 1) {
            const int32_t* ids = static_cast<const int32_t*>(input);
            int64_t i0 = begin;
            if ((reinterpret_cast<uintptr_t>(ids) & 15u) == 0) {
                const int64_t nvec = (end - begin) / 4;
                const int4* v = reinterpret_cast<const int4*>(ids + begin);
                for (int64_t j0 = 0; j0 < nvec; j0 += 4 * nthreads) {
                    int4 x[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int64_t j = j0 + tid + static_cast<int64_t>(u) * nthreads;
                        x[u] = j < nvec ? __ldg(v + j) : make_int4(-1, -1, -1, -1);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int e[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            if (e[c] >= 0 && e[c] < L) atomicAdd(hist + e[c], 1);
                        }
                    }
                }
                i0 = begin + nvec * 4;
            }
            for (int64_t i = i0 + tid; i < end; i += nthreads) {
                const int32_t e = ids[i];
                if (e >= 0 && e < L) atomicAdd(hist + e, 1);
            }
        } else {
            const int64_t* ids = static_cast<const int64_t*>(input);
            int64_t i0 = begin;
            if ((reinterpret_cast<uintptr_t>(ids) & 15u) == 0) {
                const int64_t nvec = (end - begin) / 2;
                const longlong2* v = reinterpret_cast<const longlong2*>(ids + begin);
                for (int64_t j0 = 0; j0 < nvec; j0 += 4 * nthreads) {
                    longlong2 x[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int64_t j = j0 + tid + static_cast<int64_t>(u) * nthreads;
                        x[u] = j < nvec ? __ldg(v + j) : make_longlong2(-1, -1);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (x[u].x >= 0 && x[u].x < L) atomicAdd(hist + static_cast<int>(x[u].x), 1);
                        if (x[u].y >= 0 && x[u].y < L) atomicAdd(hist + static_cast<int>(x[u].y), 1);
                    }
                }
                i0 = begin + nvec * 2;
            }
            for (int64_t i = i0 + tid; i < end; i += nthreads) {
                const int64_t e = ids[i];
                if (e >= 0 && e < L) atomicAdd(hist + static_cast<int>(e), 1);
            }
        }
    }
}

__global__ void __launch_bounds__(kPlanThreads) histogram_kernel(int input_kind, const void* input, int T, int K_or_L,
                                                                 int L, int32_t* loads) {
    extern __shared__ __align__(128) char smem_raw[];
    int32_t* hist = reinterpret_cast<int32_t*>(smem_raw);
    for (int i = threadIdx.x; i < L; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    histogram_slice(input_kind, input, T, K_or_L, L, blockIdx.x, gridDim.x, hist);
    __syncthreads();
    for (int i = threadIdx.x; i < L; i += blockDim.x) {
        if (hist[i]) atomicAdd(loads + i, hist[i]);
    }
}

// Stateless solve: one CTA per NVLink domain.
__global__ void __launch_bounds__(kPlanThreads) solve_kernel(SolveArgs a, int32_t* global_loads_out, int reduce_loads,
                                                             DeviceStatus* status) {
    extern __shared__ __align__(128) char smem_raw[];
    const int domain = blockIdx.x;
    const int E = a.G * a.M, L = a.N * a.M;
    if (reduce_loads) {
        // total load of this domain's experts over all ranks
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            const int l = domain * E + i;
            int32_t total = 0;
            for (int r = 0; r < a.N; ++r) total += __ldcg(a.loads_per_rank + static_cast<int64_t>(r) * L + l);
            global_loads_out[l] = total;
        }
        __syncthreads();
    }
    solve_domain_dispatch(a, domain, smem_raw, status);
}

__global__ void __launch_bounds__(256) init_master_kernel(int32_t* p2l, int32_t* l2p, int32_t* lcnts, int32_t* quota,
                                                          int32_t* quota_prefix, int32_t* rqp, int N, int M, int R,
                                                          int D) {
    const int Lp = M + R, L = N * M, P = N * Lp;
    const int gtid = blockIdx.x * blockDim.x + threadIdx.x, gsize = gridDim.x * blockDim.x;
    for (int i = gtid; i < P; i += gsize) {
        const int local = i % Lp;
        p2l[i] = local < M ? (i / Lp) * M + local : -1;
    }
    for (int i = gtid; i < L * D; i += gsize) {
        const int l = i / D, j = i % D;
        l2p[i] = j == 0 ? (l / M) * Lp + l % M : -1;
        quota[i] = 0;
        quota_prefix[i] = 0;
        rqp[i] = 0;
    }
    for (int i = gtid; i < L; i += gsize) lcnts[i] = 1;
}

// The fused per-layer plan kernel. gridDim.x = nlocal * ctas_per_rank.
__global__ void __launch_bounds__(kPlanThreads) plan_kernel(PlanCall call) {
    extern __shared__ __align__(128) char smem_raw[];
    __shared__ int s_timeout_peer;
    __shared__ uint64_t s_epoch;

    const int local = blockIdx.x / call.ctas_per_rank;
    const int part = blockIdx.x % call.ctas_per_rank;
    const RankDev& rk = *call.rank[local];
    const int N = call.N, M = call.M;
    const int L = N * M;
    const int Lpad = (L + 3) / 4 * 4;
    const int tid = threadIdx.x;
    const unsigned long long t_start = call.trace != nullptr ? global_timer_ns() : 0ull;

    // 1. histogram slice -> shared. The rank's first CTA owns the rest of the kernel; the others hand it their
    //    partial counts as self-validating words (epoch tag << 32 | count) in a row of their own and are done:
    //    no atomics on a common row, no fence, no ticket, and the owner sees a partial one memory round trip
    //    after it was stored. The owner waits (bounded) for CTAs of its own launch; none of them waits for it,
    //    so they need not be resident at the same time.
    int32_t* hist = reinterpret_cast<int32_t*>(smem_raw);
    for (int i = tid; i < L; i += blockDim.x) hist[i] = 0;
    if (tid == 0) {
        s_timeout_peer = -1;
        // the epoch this launch opens: the owner stores it once it holds every partial, so every CTA of the
        // launch reads the same value here
        s_epoch = *reinterpret_cast<volatile uint64_t*>(rk.epochs) + 1;
    }
    __syncthreads();
    histogram_slice(call.input_kind, call.input[local], call.T[local], call.K_or_L, L, part, call.ctas_per_rank, hist);
    __syncthreads();
    const uint64_t epoch = s_epoch;
    // never zero (the buffers start zeroed), period 2^32 - 1: an odd period, so the word that carried the same
    // tag one period ago sat in the other parity slot and cannot be mistaken for this epoch's
    const uint32_t tag = static_cast<uint32_t>(epoch % 0xFFFFFFFFull) + 1u;
    if (part != 0) {
        uint64_t* row = rk.hist_parts + static_cast<int64_t>(part) * Lpad;
        for (int i = tid; i < L; i += blockDim.x) st_relaxed_sys_u64(row + i, tag_word(tag, static_cast<uint32_t>(hist[i])));
        return;
    }
    auto stamp = [&](int slot) {
        if (call.trace != nullptr && tid == 0) call.trace[local * 8 + slot] = global_timer_ns();
    };
    if (call.trace != nullptr && tid == 0) call.trace[local * 8 + 5] = t_start;  // when this CTA started
    for (int i = tid; i < L; i += blockDim.x) {
        int32_t total = hist[i];
        for (int c0 = 1; c0 < call.ctas_per_rank; c0 += 8) {
            uint64_t w[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (c0 + u < call.ctas_per_rank) w[u] = ld_relaxed_sys_u64(rk.hist_parts + static_cast<int64_t>(c0 + u) * Lpad + i);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (c0 + u < call.ctas_per_rank) {
                    if (static_cast<uint32_t>(w[u] >> 32) != tag &&
                        !wait_tagged_word(rk.hist_parts + static_cast<int64_t>(c0 + u) * Lpad + i, tag,
                                          *reinterpret_cast<volatile int*>(&s_timeout_peer) >= 0 ? 0 : call.timeout_ns, w[u])) {
                        atomicMax(&s_timeout_peer, rk.my_rank);
                        w[u] = 0;
                    }
                    total += static_cast<int32_t>(static_cast<uint32_t>(w[u]));
                }
            }
        }
        hist[i] = total;
    }
    __syncthreads();
    if (tid == 0) *rk.epochs = epoch;  // every CTA of the launch has read the old value: its partial carried the tag
    if (s_timeout_peer >= 0) {  // a CTA of this very launch never delivered
        if (tid == 0) report_error(rk.status, UEP_DEV_TIMEOUT_GATHER, s_timeout_peer);
        return;
    }
    stamp(0);

    // 2. publish the row to every rank (itself included). Every 64-bit word carries the epoch beside its
    //    count, so a row needs neither a fence nor a flag: one NVLink crossing, and the reader knows a word
    //    is this layer's when it sees it.
    const int slot = static_cast<int>(epoch & 1ull);
    const int me = rk.my_rank;
    if (me != call.withhold_rank) {
        for (int idx = tid; idx < N * L; idx += blockDim.x) {
            const int p = idx / L, i = idx % L;
            st_relaxed_sys_u64(rk.peer_gather[p] + (static_cast<int64_t>(slot) * N + me) * Lpad + i,
                               tag_word(tag, static_cast<uint32_t>(hist[i])));
        }
    }

    stamp(1);
    // 3. collect every rank's row (bounded), expose the matrix, reduce. A thread owns one expert:
    //    it first issues the loads of eight ranks' words together and only then looks at them,
    //    so the common case (all rows already here) costs one memory round trip.
    const uint64_t* gathered = rk.peer_gather[me] + static_cast<int64_t>(slot) * N * Lpad;
    for (int i = tid; i < L; i += blockDim.x) {
        int32_t total = 0;
        for (int r0 = 0; r0 < N; r0 += 8) {
            uint64_t w[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (r0 + u < N) w[u] = ld_relaxed_sys_u64(gathered + static_cast<int64_t>(r0 + u) * Lpad + i);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (r0 + u < N) {
                    // one time limit for the whole gather: once a wait has run out, no other word is waited for
                    if (static_cast<uint32_t>(w[u] >> 32) != tag &&
                        !wait_tagged_word(gathered + static_cast<int64_t>(r0 + u) * Lpad + i, tag,
                                          *reinterpret_cast<volatile int*>(&s_timeout_peer) >= 0 ? 0 : call.timeout_ns, w[u])) {
                        atomicMax(&s_timeout_peer, r0 + u);
                        w[u] = 0;
                    }
                    const int32_t v = static_cast<int32_t>(static_cast<uint32_t>(w[u]));
                    rk.loads_per_rank[static_cast<int64_t>(r0 + u) * L + i] = v;
                    total += v;
                }
            }
        }
        rk.global_loads[i] = total;
    }
    __threadfence_block();
    __syncthreads();
    if (s_timeout_peer >= 0) {
        if (tid == 0) report_error(rk.status, UEP_DEV_TIMEOUT_GATHER, s_timeout_peer);
        return;  // plan of this layer is left as it was; the host raises on the status word
    }

    stamp(2);
    stamp(3);
    SolveArgs a;
    a.global_loads = rk.global_loads;
    a.loads_per_rank = rk.loads_per_rank;
    const PlanPtrs& pp = call.plan[local];
    a.p2l = pp.p2l; a.l2p = pp.l2p; a.lcnts = pp.lcnts; a.quota = pp.quota; a.quota_prefix = pp.quota_prefix;
    a.rank_quota_prefix = pp.rank_quota_prefix;
    a.physical_loads = pp.physical_loads;
    a.N = N; a.G = call.G; a.M = M; a.R = call.R; a.D = call.D;
    a.balance_threshold = call.params.balance_threshold;
    a.min_tokens = call.params.min_tokens_per_replica;
    a.allow_zero_master = call.params.allow_zero_master_quota;
    a.locality = call.params.locality_aware;
    a.eps = call.params.oracle_eps;
    a.my_rank = me;
    a.legacy = call.legacy;
    a.trace = call.trace != nullptr ? call.trace + (kMaxLocalRanks + local) * 8 : nullptr;
    const int num_domains = N / call.G;
    for (int d = 0; d < num_domains; ++d) solve_domain_dispatch(a, d, smem_raw, rk.status);
    stamp(4);
}

size_t plan_smem_bytes(int N, int G, int M) {
    const size_t solver = std::max(solver_smem_bytes(G * M, G), legacy_smem_bytes(G * M, G));
    const size_t hist = sizeof(int32_t) * static_cast<size_t>(N) * M;
    return (solver > hist ? solver : hist) + 16;
}

cudaError_t ensure_smem(const void* fn, size_t bytes) {
    if (bytes <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
}

std::atomic<int64_t> g_launches{0};

}  // namespace

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int plan_ctas_per_rank(int input_kind, int max_T, int K_or_L, int nlocal, int num_sms) {
    const int64_t bytes = static_cast<int64_t>(max_T) * K_or_L * (input_kind == 0 ? 1 : (input_kind == 1 ? 4 : 8));
    int ctas = static_cast<int>((bytes + 16 * 1024 - 1) / (16 * 1024));
    const int cap = nlocal > 1 ? (num_sms / nlocal) : kPlanMaxCtas;
    ctas = ctas < 1 ? 1 : ctas;
    ctas = ctas > cap ? cap : ctas;
    return ctas > kPlanMaxCtas ? kPlanMaxCtas : (ctas < 1 ? 1 : ctas);
}

cudaError_t launch_plan(const PlanCall& call, cudaStream_t stream) {
    const size_t smem = plan_smem_bytes(call.N, call.G, call.M);
    cudaError_t e = ensure_smem(reinterpret_cast<const void*>(plan_kernel), smem);
    if (e != cudaSuccess) return e;
    const dim3 grid(call.nlocal * call.ctas_per_rank), block(kPlanThreads);
    count_launch();
    if (call.nlocal > 1) {
        // ranks wait for each other inside the kernel: co-residency is required
        PlanCall copy = call;
        void* args[] = {&copy};
        return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(plan_kernel), grid, block, args, smem, stream);
    }
    plan_kernel<<<grid, block, smem, stream>>>(call);
    return cudaGetLastError();
}

}  // namespace uep

// ------------------------------------------------------------------------------------
// C ABI: stateless entry points
// ------------------------------------------------------------------------------------
using namespace uep;

extern "C" {

int64_t uep_launch_count(void) { return g_launches.load(); }
void uep_reset_launch_count(void) { g_launches.store(0); }

static int histogram_common(int kind, const void* input, int T, int K_or_L, int L, int32_t* loads, void* stream_) {
    if (L <= 0 || L > 65536 || T < 0 || K_or_L < 0 || loads == nullptr) return fail(UEP_ERR_INVALID, "histogram: bad sizes");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    UEP_CUDA_TRY(cudaMemsetAsync(loads, 0, sizeof(int32_t) * L, stream));
    const int64_t n = static_cast<int64_t>(T) * K_or_L;
    if (n == 0) return UEP_OK;
    if (input == nullptr) return fail(UEP_ERR_INVALID, "histogram: null input");
    const int ctas = plan_ctas_per_rank(kind, T, K_or_L, 1, std::max(device_sm_count(), 1));
    const size_t smem = sizeof(int32_t) * L;
    UEP_CUDA_TRY(ensure_smem(reinterpret_cast<const void*>(histogram_kernel), smem));
    count_launch();
    histogram_kernel<<<ctas, kPlanThreads, smem, stream>>>(kind, input, T, K_or_L, L, loads);
    UEP_CUDA_TRY(cudaGetLastError());
    return UEP_OK;
}

int uep_histogram_ids32(const int32_t* ids, int64_t num_entries, int L, int32_t* loads, void* stream) {
    if (num_entries < 0 || num_entries > INT32_MAX) return fail(UEP_ERR_INVALID, "histogram: too many entries");
    return histogram_common(1, ids, static_cast<int>(num_entries), 1, L, loads, stream);
}
int uep_histogram_ids64(const int64_t* ids, int64_t num_entries, int L, int32_t* loads, void* stream) {
    if (num_entries < 0 || num_entries > INT32_MAX) return fail(UEP_ERR_INVALID, "histogram: too many entries");
    return histogram_common(2, ids, static_cast<int>(num_entries), 1, L, loads, stream);
}
int uep_histogram_map(const uint8_t* routing_map, int T, int L, int32_t* loads, void* stream) {
    return histogram_common(0, routing_map, T, L, L, loads, stream);
}

int uep_solve_placement(const int32_t* loads_per_rank, int32_t* global_loads_out, int32_t* p2l, int32_t* l2p,
                        int32_t* lcnts, int32_t* quota, int32_t* quota_prefix, int32_t* rank_quota_prefix,
                        int num_ranks, int nvl_ranks, int M, int R, int D, const uep_solver_params* params,
                        int my_rank, int32_t* status, void* stream_) {
    if (params == nullptr || loads_per_rank == nullptr || global_loads_out == nullptr)
        return fail(UEP_ERR_INVALID, "solve_placement: null argument (global_loads_out is required as workspace)");
    if (nvl_ranks <= 0 || num_ranks <= 0 || num_ranks % nvl_ranks != 0 || M <= 0 || R < 0 || D < 1)
        return fail(UEP_ERR_INVALID, "solve_placement: bad group shape");
    if (nvl_ranks * M > kMaxExpertsPerDomain || nvl_ranks > kMaxRanksPerDomain || nvl_ranks * R > kMaxExportsPerDomain)
        return fail(UEP_ERR_INVALID, "solve_placement: domain exceeds the static limits (512 experts, 72 ranks, 512 replicas)");
    if (D < (nvl_ranks < num_ranks ? nvl_ranks : num_ranks))
        return fail(UEP_ERR_INVALID, "solve_placement: max_replicas_dim smaller than the NVLink domain");
    if (my_rank < 0 || my_rank >= num_ranks) return fail(UEP_ERR_INVALID, "solve_placement: my_rank out of range");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    SolveArgs a;
    a.global_loads = global_loads_out;
    a.loads_per_rank = loads_per_rank;
    a.p2l = p2l; a.l2p = l2p; a.lcnts = lcnts; a.quota = quota; a.quota_prefix = quota_prefix;
    a.rank_quota_prefix = rank_quota_prefix;
    a.physical_loads = nullptr;
    a.N = num_ranks; a.G = nvl_ranks; a.M = M; a.R = R; a.D = D;
    a.balance_threshold = params->balance_threshold;
    a.min_tokens = params->min_tokens_per_replica;
    a.allow_zero_master = params->allow_zero_master_quota;
    a.locality = params->locality_aware;
    a.eps = params->oracle_eps;
    a.my_rank = my_rank;
    a.legacy = 0;
    a.trace = nullptr;
    const size_t smem = solver_smem_bytes(nvl_ranks * M, nvl_ranks) + 16;
    UEP_CUDA_TRY(ensure_smem(reinterpret_cast<const void*>(solve_kernel), smem));
    count_launch();
    solve_kernel<<<num_ranks / nvl_ranks, kPlanThreads, smem, stream>>>(a, global_loads_out, 1,
                                                                        reinterpret_cast<DeviceStatus*>(status));
    UEP_CUDA_TRY(cudaGetLastError());
    return UEP_OK;
}

int uep_legacy_solve_placement(const int32_t* global_loads, int32_t* p2l, int32_t* l2p, int32_t* lcnts, int32_t* quota,
                               int32_t* quota_prefix, int32_t* rank_quota_prefix, int num_ranks, int nvl_ranks, int M,
                               int R, int D, float balance_threshold, int32_t* status, void* stream_) {
    if (global_loads == nullptr) return fail(UEP_ERR_INVALID, "legacy_solve_placement: null loads");
    if (nvl_ranks <= 0 || num_ranks <= 0 || num_ranks % nvl_ranks != 0 || M <= 0 || R < 0 || D < 1)
        return fail(UEP_ERR_INVALID, "legacy_solve_placement: bad group shape");
    if (nvl_ranks * M > kMaxExpertsPerDomain || nvl_ranks > kMaxRanksPerDomain || nvl_ranks * R > kMaxExportsPerDomain)
        return fail(UEP_ERR_INVALID, "legacy_solve_placement: domain exceeds the static limits (512 experts, 72 ranks, 512 replicas)");
    if (D < (nvl_ranks < num_ranks ? nvl_ranks : num_ranks))
        return fail(UEP_ERR_INVALID, "legacy_solve_placement: max_replicas_dim smaller than the NVLink domain");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    SolveArgs a;
    std::memset(&a, 0, sizeof(a));
    a.global_loads = global_loads;
    a.p2l = p2l; a.l2p = l2p; a.lcnts = lcnts; a.quota = quota; a.quota_prefix = quota_prefix;
    a.rank_quota_prefix = rank_quota_prefix;
    a.N = num_ranks; a.G = nvl_ranks; a.M = M; a.R = R; a.D = D;
    a.balance_threshold = balance_threshold;
    a.legacy = 1;
    const size_t smem = legacy_smem_bytes(nvl_ranks * M, nvl_ranks) + 16;
    UEP_CUDA_TRY(ensure_smem(reinterpret_cast<const void*>(solve_kernel), smem));
    count_launch();
    solve_kernel<<<num_ranks / nvl_ranks, kPlanThreads, smem, stream>>>(a, nullptr, 0, reinterpret_cast<DeviceStatus*>(status));
    UEP_CUDA_TRY(cudaGetLastError());
    return UEP_OK;
}

int uep_init_master_placement(int32_t* p2l, int32_t* l2p, int32_t* lcnts, int32_t* quota, int32_t* quota_prefix,
                              int32_t* rank_quota_prefix, int num_ranks, int M, int R, int D, void* stream) {
    if (num_ranks <= 0 || M <= 0 || R < 0 || D < 1) return fail(UEP_ERR_INVALID, "init_master_placement: bad shape");
    const int work = num_ranks * M * D;
    const int grid = work / 256 + 1 > 64 ? 64 : work / 256 + 1;
    count_launch();
    init_master_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p2l, l2p, lcnts, quota, quota_prefix,
                                                                           rank_quota_prefix, num_ranks, M, R, D);
    UEP_CUDA_TRY(cudaGetLastError());
    return UEP_OK;
}

}  // extern "C"
