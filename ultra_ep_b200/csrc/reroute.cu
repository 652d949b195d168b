// Kernel 2 — reroute: logical expert ids -> physical replica ids under the rank's
// quota split, in dense ([T,L] -> [T,P]) and sparse ([T,K]) form, the dense backward
// gather, and the token-gradient row gather.
//
// The reference resolves the ordinal of a token inside its expert with one warp per
// (expert, 128-token tile) reading the bool map column-wise, and writes the [T,P]
// outputs twice (zero-fill, then scatter): csrc/kernels/reroute.cu:21-51, 138-264 and
// csrc/ultra_ep.cpp:891-892 of the reference. Here:
//   * pass 1 counts keys per (tile, expert) from coalesced row reads;
//   * pass 2 turns the counts of the preceding tiles into a base per expert, resolves
//     ordinals inside the tile in row-major order (sparse: per-warp sub-counts, then match.any
//     inside the warp; dense: the map tile is staged in shared memory, one thread per expert
//     walks its column only to count, and the replica arithmetic runs over the marked cells
//     spread over the CTA), and writes every output element exactly once with coalesced
//     vector stores (zeros included), so no pre-zeroing pass exists.
// Results equal the reference's dense rule bit for bit; the sparse form applies the same
// rule per (token, k) entry and therefore is deterministic, which the reference's
// atomic-counter sparse kernel (reroute.cu:492-515) is not.

#include <mutex>
#include <string>

#include "internal.h"

namespace uep {

namespace {

constexpr int kRerouteThreads = 256;
constexpr int kDenseTileRows = 64;
constexpr int kSparseTileEntries = 2048;  // 8 warps x 256 entries

__device__ __forceinline__ int gcd_int(int a, int b) {
    while (b != 0) {
        const int t = a % b;
        a = b;
        b = t;
    }
    return a;
}

// Per-expert routing parameters (csrc/kernels/reroute.cu:182-209 of the reference).
struct Router {
    int C, total, stride, offset;
};

__device__ __forceinline__ Router make_router(int e, const int32_t* lcnts, const int32_t* rqp, int D, bool quota_mode,
                                              bool interleave) {
    Router r;
    r.C = lcnts[e];
    r.total = 0;
    r.stride = 1;
    r.offset = 0;
    if (quota_mode && r.C > 0) r.total = rqp[static_cast<int64_t>(e) * D + r.C - 1];
    if (quota_mode && interleave && r.total > 1) {
        int s = r.total / 2 + 1;
        if (s >= r.total) s = r.total - 1;
        if (s < 1) s = 1;
        while (gcd_int(s, r.total) != 1) {
            ++s;
            if (s >= r.total) s = 1;
        }
        r.stride = s;
        r.offset = e % r.total;
    } else {
        r.stride = 0;  // marks "no interleave"
    }
    return r;
}

// ordinal -> replica index (reroute.cu:239-254 of the reference; round-robin: :126)
__device__ __forceinline__ int replica_index(const Router& r, int e, int ordinal, const int32_t* rqp, int D,
                                             bool quota_mode) {
    if (r.C <= 1) return 0;  // one instance: every branch below ends at index 0
    if (!quota_mode) return ordinal % r.C;
    int qr = ordinal;
    if (r.stride != 0) qr = static_cast<int>((static_cast<long long>(ordinal) * r.stride + r.offset) % r.total);
    const int32_t* prefix = rqp + static_cast<int64_t>(e) * D;
    int idx = 0;
    for (int j = 0; j < r.C; ++j) idx += (qr >= prefix[j]) ? 1 : 0;
    return min(idx, max(r.C - 1, 0));
}

// ----------------------------------------------------------------------------- dense
// Copies rows [r0, r1) of the bool map into shared memory, 16 bytes per thread when the tile starts on a
// 16-byte boundary. The per-expert walks below then run over shared memory: walking a column of the map in
// global memory costs one dependent memory round trip per row.
__device__ __forceinline__ void stage_map_tile(const uint8_t* __restrict__ map, int r0, int r1, int L, uint8_t* smap) {
    const int64_t first = static_cast<int64_t>(r0) * L;
    const int bytes = (r1 - r0) * L;
    const uint8_t* src = map + first;
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
        const int nvec = bytes / 16;
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
            reinterpret_cast<uint4*>(smap)[i] = ld_global_nc_v4(src + static_cast<int64_t>(i) * 16);
        }
        done = nvec * 16;
    }
    for (int i = done + threadIdx.x; i < bytes; i += blockDim.x) smap[i] = src[i];
}

__global__ void __launch_bounds__(kRerouteThreads) dense_count_kernel(Batch<DenseFwdArgs> batch, int L) {
    extern __shared__ __align__(128) char smem_raw[];  // [kDenseTileRows][L] bytes
    const DenseFwdArgs& a = batch.a[blockIdx.y];
    const int T = a.T;
    const int tile = blockIdx.x;
    const int r0 = tile * kDenseTileRows, r1 = min(r0 + kDenseTileRows, T);
    if (r0 >= T) return;
    uint8_t* smap = reinterpret_cast<uint8_t*>(smem_raw);
    stage_map_tile(a.map, r0, r1, L, smap);
    __syncthreads();
    for (int e = threadIdx.x; e < L; e += blockDim.x) {
        int c = 0;
        for (int t = 0; t < r1 - r0; ++t) c += smap[t * L + e] ? 1 : 0;
        a.scratch[static_cast<int64_t>(tile) * L + e] = c;
    }
}

__global__ void __launch_bounds__(kRerouteThreads)
dense_scatter_kernel(Batch<DenseFwdArgs> batch, int L, int P, int D, int quota_mode, int interleave) {
    const DenseFwdArgs& a = batch.a[blockIdx.y];
    const uint8_t* __restrict__ map = a.map;
    const float* __restrict__ probs = a.probs;
    const int32_t* __restrict__ l2p = a.l2p;
    const int32_t* __restrict__ lcnts = a.lcnts;
    const int32_t* __restrict__ rqp = a.rqp;
    const int32_t* __restrict__ tile_counts = a.scratch;
    uint8_t* __restrict__ out_map = a.out_map;
    float* __restrict__ out_probs = a.out_probs;
    const int T = a.T;
    if (static_cast<int>(blockIdx.x) * kDenseTileRows >= T) return;
    const int vec_ok = ((P & 3) == 0) && ((reinterpret_cast<uintptr_t>(out_probs) & 15u) == 0) &&
                       ((reinterpret_cast<uintptr_t>(out_map) & 3u) == 0);
    extern __shared__ __align__(128) char smem_raw[];
    // layout: inv[P] int32 | routers[L] | base[L] int32 | choice[rows][L] uint8 (16-byte aligned)
    int32_t* inv = reinterpret_cast<int32_t*>(smem_raw);
    Router* routers = reinterpret_cast<Router*>(inv + (P + 3) / 4 * 4);
    int32_t* base_of = reinterpret_cast<int32_t*>(routers + L);
    uint8_t* choice = reinterpret_cast<uint8_t*>(base_of + (L + 3) / 4 * 4);

    const int tile = blockIdx.x;
    const int r0 = tile * kDenseTileRows, r1 = min(r0 + kDenseTileRows, T);
    const int rows = r1 - r0;

    for (int p = threadIdx.x; p < P; p += blockDim.x) inv[p] = -1;
    stage_map_tile(map, r0, r1, L, choice);  // the passes below turn each map byte into its replica choice in place
    __syncthreads();
    // Pass 1, one thread per expert: which slots it owns, its ordinal base in this tile, its routing parameters, and
    // a walk down its column that only counts: a routed cell of an expert with several instances is marked
    // 0x80 | (its rank among the tile's routed rows, < 64); with one instance the choice is 0 at once.
    for (int e = threadIdx.x; e < L; e += blockDim.x) {
        const int C = lcnts[e];
        for (int j = 0; j < C; ++j) {
            const int p = l2p[static_cast<int64_t>(e) * D + j];
            if (p >= 0 && p < P) inv[p] = e;
        }
        int base = 0;
        for (int tl = 0; tl < tile; ++tl) base += tile_counts[static_cast<int64_t>(tl) * L + e];
        base_of[e] = base;
        routers[e] = make_router(e, lcnts, rqp, D, quota_mode != 0, interleave != 0);
        int seen = 0;
        for (int t = 0; t < rows; ++t) {
            uint8_t c = 0xFF;
            if (choice[t * L + e]) {
                c = C <= 1 ? 0 : static_cast<uint8_t>(0x80 | seen);
                ++seen;
            }
            choice[t * L + e] = c;
        }
    }
    __syncthreads();
    // Pass 2, all threads over the tile's cells: the replica arithmetic (a 64-bit multiply and modulo, a prefix
    // search) only for the marked cells, spread over the CTA instead of sitting in the hot experts' threads.
    for (int cell = threadIdx.x; cell < rows * L; cell += blockDim.x) {
        const uint8_t c = choice[cell];
        if (c >= 0x80 && c != 0xFF) {
            const int e = cell % L;
            choice[cell] = static_cast<uint8_t>(replica_index(routers[e], e, base_of[e] + (c & 0x3F), rqp, D, quota_mode != 0));
        }
    }
    __syncthreads();
    // every output element of the tile, once
    if (vec_ok) {
        const int quads = P / 4;
        for (int idx = threadIdx.x; idx < rows * quads; idx += blockDim.x) {
            const int t = idx / quads, p0 = (idx % quads) * 4;
            float4 pv = make_float4(0.f, 0.f, 0.f, 0.f);
            uint32_t mv = 0;
            float* pvf = reinterpret_cast<float*>(&pv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int e = inv[p0 + k];
                if (e >= 0) {
                    const uint8_t c = choice[t * L + e];
                    if (c != 0xFF && l2p[static_cast<int64_t>(e) * D + c] == p0 + k) {
                        pvf[k] = probs[static_cast<int64_t>(r0 + t) * L + e];
                        mv |= 1u << (8 * k);
                    }
                }
            }
            const int64_t o = static_cast<int64_t>(r0 + t) * P + p0;
            *reinterpret_cast<float4*>(out_probs + o) = pv;
            *reinterpret_cast<uint32_t*>(out_map + o) = mv;
        }
    } else {
        for (int idx = threadIdx.x; idx < rows * P; idx += blockDim.x) {
            const int t = idx / P, p = idx % P;
            float v = 0.f;
            uint8_t m = 0;
            const int e = inv[p];
            if (e >= 0) {
                const uint8_t c = choice[t * L + e];
                if (c != 0xFF && l2p[static_cast<int64_t>(e) * D + c] == p) {
                    v = probs[static_cast<int64_t>(r0 + t) * L + e];
                    m = 1;
                }
            }
            out_probs[static_cast<int64_t>(r0 + t) * P + p] = v;
            out_map[static_cast<int64_t>(r0 + t) * P + p] = m;
        }
    }
}

__device__ __forceinline__ float routed_grad(const float* __restrict__ grad_expanded, const uint8_t* __restrict__ expanded_map,
                                             const int32_t* __restrict__ l2p, const int32_t* __restrict__ lcnts, int64_t t,
                                             int l, int P, int D) {
    const int C = lcnts[l];
    for (int r = 0; r < C; ++r) {
        const int phys = l2p[static_cast<int64_t>(l) * D + r];
        if (expanded_map[t * P + phys]) return grad_expanded[t * P + phys];
    }
    return 0.f;
}

// One thread per four logical experts of a token when the rows allow it (L a multiple of 4, map rows 4-byte and
// gradient rows 16-byte aligned): the routing map is read a word at a time and the gradients leave as float4.
// Most entries are not routed, so the kernel is a zero fill plus a few gathers.
__global__ void __launch_bounds__(kRerouteThreads) dense_backward_kernel(Batch<DenseBwdArgs> batch, int L, int P, int D) {
    const DenseBwdArgs& a = batch.a[blockIdx.y];
    const float* __restrict__ grad_expanded = a.grad_expanded;
    const uint8_t* __restrict__ map = a.map;
    const uint8_t* __restrict__ expanded_map = a.expanded_map;
    const int32_t* __restrict__ l2p = a.l2p;
    const int32_t* __restrict__ lcnts = a.lcnts;
    float* __restrict__ grad_probs = a.grad_probs;
    const int64_t total = static_cast<int64_t>(a.T) * L;
    const int64_t gtid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t gsize = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const bool vec = (L % 4 == 0) && ((reinterpret_cast<uintptr_t>(map) & 3u) == 0) &&
                     ((reinterpret_cast<uintptr_t>(grad_probs) & 15u) == 0);
    if (vec) {
        const int groups = L / 4;
        for (int64_t q = gtid; q < total / 4; q += gsize) {
            const uint32_t m = __ldg(reinterpret_cast<const uint32_t*>(map) + q);
            float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
            if (m != 0) {
                const int64_t t = q / groups;
                const int l0 = static_cast<int>(q % groups) * 4;
                if (m & 0x000000FFu) g.x = routed_grad(grad_expanded, expanded_map, l2p, lcnts, t, l0, P, D);
                if (m & 0x0000FF00u) g.y = routed_grad(grad_expanded, expanded_map, l2p, lcnts, t, l0 + 1, P, D);
                if (m & 0x00FF0000u) g.z = routed_grad(grad_expanded, expanded_map, l2p, lcnts, t, l0 + 2, P, D);
                if (m & 0xFF000000u) g.w = routed_grad(grad_expanded, expanded_map, l2p, lcnts, t, l0 + 3, P, D);
            }
            reinterpret_cast<float4*>(grad_probs)[q] = g;
        }
        return;
    }
    for (int64_t idx = gtid; idx < total; idx += gsize) {
        float g = 0.f;
        if (map[idx]) g = routed_grad(grad_expanded, expanded_map, l2p, lcnts, idx / L, static_cast<int>(idx % L), P, D);
        grad_probs[idx] = g;
    }
}

// ---------------------------------------------------------------------------- sparse
// bucket of a key: itself when in [0,nb_valid), else the last bucket (if there is one) or none
template <typename IdT>
__device__ __forceinline__ int key_bucket(IdT key, int nb_valid, bool tail_bucket) {
    if (key >= 0 && key < nb_valid) return static_cast<int>(key);
    return tail_bucket ? nb_valid : -1;
}

template <typename IdT>
__global__ void __launch_bounds__(kRerouteThreads) key_count_kernel(const IdT* __restrict__ keys, int64_t n,
                                                                    int nb_valid, int tail_bucket,
                                                                    int32_t* __restrict__ tile_counts) {
    extern __shared__ __align__(128) char smem_raw[];
    int32_t* hist = reinterpret_cast<int32_t*>(smem_raw);
    const int nb = nb_valid + (tail_bucket ? 1 : 0);
    for (int i = threadIdx.x; i < nb; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const int64_t begin = static_cast<int64_t>(blockIdx.x) * kSparseTileEntries;
    const int64_t end = min(begin + kSparseTileEntries, n);
    for (int64_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const int b = key_bucket<IdT>(keys[i], nb_valid, tail_bucket != 0);
        if (b >= 0) atomicAdd(hist + b, 1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nb; i += blockDim.x) tile_counts[static_cast<int64_t>(blockIdx.x) * nb + i] = hist[i];
}

// Row-major ordinal of every entry of this CTA's tile inside its bucket. On return
// `warp_base[w][b]` has been consumed; ordinals are handed to `emit(i, bucket, ordinal)`.
// warp_base must hold (blockDim/32) * nb ints and already contain, for warp 0, nothing:
// the function fills it. base[b] = number of entries of bucket b before this tile.
template <typename IdT, typename Emit>
__device__ void tile_ordinals(const IdT* keys, int64_t n, int nb_valid, bool tail_bucket,
                              const int32_t* base, int32_t* warp_base, Emit emit) {
    const int nb = nb_valid + (tail_bucket ? 1 : 0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int per_warp = kSparseTileEntries / nwarps;
    const int64_t tile_begin = static_cast<int64_t>(blockIdx.x) * kSparseTileEntries;
    const int64_t wbegin = min(tile_begin + static_cast<int64_t>(warp) * per_warp, n);
    const int64_t wend = min(wbegin + per_warp, n);

    for (int i = threadIdx.x; i < nwarps * nb; i += blockDim.x) warp_base[i] = 0;
    __syncthreads();
    // A: per-warp counts
    for (int64_t i = wbegin + lane; i < wend; i += kWarp) {
        const int b = key_bucket<IdT>(keys[i], nb_valid, tail_bucket);
        if (b >= 0) atomicAdd(warp_base + warp * nb + b, 1);
    }
    __syncthreads();
    // B: exclusive scan over warps, seeded with the tile base
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        int run = base[b];
        for (int w = 0; w < nwarps; ++w) {
            const int c = warp_base[w * nb + b];
            warp_base[w * nb + b] = run;
            run += c;
        }
    }
    __syncthreads();
    // C: in-order resolution inside the warp
    int32_t* mine = warp_base + warp * nb;
    for (int64_t i0 = wbegin; i0 < wend; i0 += kWarp) {
        const int64_t i = i0 + lane;
        const bool in = i < wend;
        const int b = in ? key_bucket<IdT>(keys[i], nb_valid, tail_bucket) : -1;
        const unsigned active = __ballot_sync(kFullMask, b >= 0);
        int ordinal = -1;
        if (b >= 0) {
            const unsigned peers = __match_any_sync(active, b);
            const int before = __popc(peers & ((1u << lane) - 1u));
            ordinal = mine[b] + before;
            __syncwarp(active);
            if (before == 0) mine[b] += __popc(peers);
        }
        __syncwarp();
        if (in) emit(i, b, ordinal);
    }
}

template <typename IdT>
__global__ void __launch_bounds__(kRerouteThreads) sparse_count_kernel(Batch<SparseArgs> batch, int K, int L) {
    extern __shared__ __align__(128) char smem_raw[];
    const SparseArgs& a = batch.a[blockIdx.y];
    const IdT* keys = static_cast<const IdT*>(a.ids);
    const int64_t n = static_cast<int64_t>(a.T) * K;
    const int64_t begin = static_cast<int64_t>(blockIdx.x) * kSparseTileEntries;
    if (begin >= n) return;
    int32_t* hist = reinterpret_cast<int32_t*>(smem_raw);
    for (int i = threadIdx.x; i < L; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const int64_t end = min(begin + kSparseTileEntries, n);
    for (int64_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const int b = key_bucket<IdT>(keys[i], L, false);
        if (b >= 0) atomicAdd(hist + b, 1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < L; i += blockDim.x) a.scratch[static_cast<int64_t>(blockIdx.x) * L + i] = hist[i];
}

template <typename IdT>
__global__ void __launch_bounds__(kRerouteThreads)
sparse_reroute_kernel(Batch<SparseArgs> batch, int K, int L, int D, int interleave) {
    extern __shared__ __align__(128) char smem_raw[];
    const SparseArgs& a = batch.a[blockIdx.y];
    const IdT* ids = static_cast<const IdT*>(a.ids);
    IdT* out = static_cast<IdT*>(a.out);
    const int32_t* __restrict__ l2p = a.l2p;
    const int32_t* __restrict__ lcnts = a.lcnts;
    const int32_t* __restrict__ rqp = a.rqp;
    const int32_t* __restrict__ tile_counts = a.scratch;
    const int64_t n = static_cast<int64_t>(a.T) * K;
    if (static_cast<int64_t>(blockIdx.x) * kSparseTileEntries >= n) return;
    // layout: base[L] | routers[L] | warp_base[nwarps][L]
    int32_t* base = reinterpret_cast<int32_t*>(smem_raw);
    Router* routers = reinterpret_cast<Router*>(base + L);
    int32_t* warp_base = reinterpret_cast<int32_t*>(routers + L);
    const int tile = blockIdx.x;
    for (int e = threadIdx.x; e < L; e += blockDim.x) {
        int b = 0;
        for (int tl = 0; tl < tile; ++tl) b += tile_counts[static_cast<int64_t>(tl) * L + e];
        base[e] = b;
        routers[e] = make_router(e, lcnts, rqp, D, interleave != 2, interleave == 1);  // 2: round-robin (legacy placement)
    }
    __syncthreads();
    // ids may alias out: every entry is read and written by the same lane, the write comes
    // last, and tiles do not overlap.
    tile_ordinals<IdT>(ids, n, L, false, base, warp_base, [&](int64_t i, int b, int ordinal) {
        if (b < 0) {
            out[i] = ids[i];
            return;
        }
        const Router r = routers[b];
        if (r.C <= 0) {
            out[i] = ids[i];
            return;
        }
        const int j = replica_index(r, b, ordinal, rqp, D, interleave != 2);
        out[i] = static_cast<IdT>(l2p[static_cast<int64_t>(b) * D + j]);
    });
}

// Experts with C <= 0 keep their id but still consume ordinals in the count pass; the
// reference skips them before taking an ordinal (reroute.cu:505-509), which is equivalent
// because such an expert never maps anything.

__global__ void __launch_bounds__(kRerouteThreads)
dispatch_positions_kernel(const int32_t* __restrict__ phys, int64_t n, int P, const int32_t* __restrict__ tile_counts,
                          int num_tiles, int32_t* __restrict__ pos, int32_t* __restrict__ expert_offsets) {
    extern __shared__ __align__(128) char smem_raw[];
    const int nb = P + 1;
    // layout: base[nb] | totals[nb] | warp_base[nwarps][nb]
    int32_t* base = reinterpret_cast<int32_t*>(smem_raw);
    int32_t* totals = base + nb;
    int32_t* warp_base = totals + nb;
    __shared__ int s_carry;
    const int tile = blockIdx.x;
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        int before = 0, total = 0;
        for (int tl = 0; tl < num_tiles; ++tl) {
            const int c = tile_counts[static_cast<int64_t>(tl) * nb + b];
            if (tl < tile) before += c;
            total += c;
        }
        base[b] = before;
        totals[b] = total;
    }
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    // exclusive scan of totals over buckets (blocked: 256 buckets per round, warp shuffles)
    for (int b0 = 0; b0 < nb; b0 += blockDim.x) {
        const int b = b0 + threadIdx.x;
        const int v = b < nb ? totals[b] : 0;
        int incl = v;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(kFullMask, incl, d);
            if (lane >= d) incl += o;
        }
        __shared__ int warp_tot[kRerouteThreads / 32];
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        int woff = 0;
        for (int w = 0; w < warp; ++w) woff += warp_tot[w];
        const int carry = s_carry;
        const int excl = carry + woff + incl - v;
        if (b < nb) {
            base[b] += excl;
            if (tile == 0 && expert_offsets != nullptr) expert_offsets[b] = excl;
        }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) s_carry = carry + woff + incl;
        __syncthreads();
    }
    tile_ordinals<int32_t>(phys, n, P, true, base, warp_base,
                           [&](int64_t i, int, int ordinal) { pos[i] = ordinal; });
}

// ------------------------------------------------------------------- row gather (HBM)
// out[i,:] = in[pos[i],:]. One elected thread per CTA drives a ring of bulk copies:
// global -> shared (mbarrier) -> global. Rows are cut into chunks of at most kGatherChunk.
constexpr int kGatherChunk = 16 * 1024;
constexpr int kGatherStages = 6;

__global__ void __launch_bounds__(32) gather_rows_kernel(const uint8_t* __restrict__ in, const int32_t* __restrict__ pos,
                                                         uint8_t* __restrict__ out, int64_t num_rows,
                                                         int64_t row_bytes, int chunks_per_row, int64_t num_src_rows,
                                                         uint64_t timeout_ns, DeviceStatus* status) {
    extern __shared__ __align__(128) char smem_raw[];
    __shared__ __align__(8) uint64_t bars[kGatherStages];
    if (threadIdx.x != 0) return;
    for (int s = 0; s < kGatherStages; ++s) mbar_init(&bars[s], 1);
    fence_mbar_init();

    const int64_t total = num_rows * chunks_per_row;
    const int64_t first = blockIdx.x, step = gridDim.x;
    const int64_t count = first < total ? (total - first + step - 1) / step : 0;

    auto chunk_bytes = [&](int64_t off) -> uint32_t {
        const int64_t left = row_bytes - off;
        return static_cast<uint32_t>(left < kGatherChunk ? left : kGatherChunk);
    };
    auto issue_load = [&](int64_t k) {
        const int64_t item = first + k * step;
        const int64_t row = item / chunks_per_row;
        const int64_t off = (item % chunks_per_row) * static_cast<int64_t>(kGatherChunk);
        int64_t src_row = pos[row];
        if (src_row < 0 || src_row >= num_src_rows) {  // never read out of bounds: record and clamp
            report_error(status, UEP_DEV_BAD_PLAN, static_cast<int>(row));
            src_row = 0;
        }
        const int s = static_cast<int>(k % kGatherStages);
        mbar_expect_tx(&bars[s], chunk_bytes(off));
        bulk_load(smem_raw + s * kGatherChunk, in + src_row * row_bytes + off, chunk_bytes(off), &bars[s]);
    };

    int64_t issued = count < kGatherStages - 1 ? count : kGatherStages - 1;
    for (int64_t k = 0; k < issued; ++k) issue_load(k);
    int64_t k = 0;
    for (; k < count; ++k) {
        const int s = static_cast<int>(k % kGatherStages);
        if (!mbar_wait(&bars[s], static_cast<uint32_t>((k / kGatherStages) & 1), timeout_ns)) break;
        const int64_t item = first + k * step;
        const int64_t row = item / chunks_per_row;
        const int64_t off = (item % chunks_per_row) * static_cast<int64_t>(kGatherChunk);
        bulk_store(out + row * row_bytes + off, smem_raw + s * kGatherChunk, chunk_bytes(off));
        bulk_commit();
        if (issued < count) {
            if (k >= 1) bulk_wait_read<1>();
            issue_load(issued);
            ++issued;
        }
    }
    bulk_wait_all<0>();
    if (k < count) {
        // a load did not land in time: report, then give every load still in flight one more
        // bounded wait so that shared memory is not released under it
        report_error(status, UEP_DEV_TIMEOUT_COPY, static_cast<int>(k));
        for (int64_t j = k; j < issued; ++j) {
            mbar_wait(&bars[j % kGatherStages], static_cast<uint32_t>((j / kGatherStages) & 1), timeout_ns);
        }
    }
}

// Plain vector-load variant for rows that are not 16-byte sized/aligned multiples.
__global__ void __launch_bounds__(256) gather_rows_plain_kernel(const uint8_t* __restrict__ in,
                                                                const int32_t* __restrict__ pos,
                                                                uint8_t* __restrict__ out, int64_t num_rows,
                                                                int64_t row_bytes, int64_t num_src_rows,
                                                                DeviceStatus* status) {
    for (int64_t row = blockIdx.x; row < num_rows; row += gridDim.x) {
        int64_t src = pos[row];
        if (src < 0 || src >= num_src_rows) {
            if (threadIdx.x == 0) report_error(status, UEP_DEV_BAD_PLAN, static_cast<int>(row));
            src = 0;
        }
        for (int64_t b = threadIdx.x; b < row_bytes; b += blockDim.x) out[row * row_bytes + b] = in[src * row_bytes + b];
    }
}

cudaError_t ensure_smem_attr(const void* fn, size_t bytes) {
    if (bytes <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
}

int dense_tiles(int T) { return (T + kDenseTileRows - 1) / kDenseTileRows; }
int64_t sparse_tiles(int64_t n) { return (n + kSparseTileEntries - 1) / kSparseTileEntries; }

}  // namespace

int64_t dense_scratch_elems(int T, int L) { return static_cast<int64_t>(dense_tiles(T)) * L + 4; }
int64_t sparse_scratch_elems(int64_t entries, int L) { return sparse_tiles(entries) * L + 4; }

cudaError_t launch_dense_forward(const Batch<DenseFwdArgs>& b, int L, int P, int D, int quota_mode, int interleave,
                                 cudaStream_t stream) {
    int max_T = 0;
    for (int i = 0; i < b.n; ++i) max_T = b.a[i].T > max_T ? b.a[i].T : max_T;
    if (max_T == 0) return cudaSuccess;
    const dim3 grid(dense_tiles(max_T), b.n);
    const size_t smem_count = static_cast<size_t>(kDenseTileRows) * L + 16;
    static_assert(kDenseTileRows <= 64, "a routed cell's rank inside its tile is kept in six bits");
    const size_t smem = sizeof(int32_t) * ((P + 3) / 4 * 4) + sizeof(Router) * L + sizeof(int32_t) * ((L + 3) / 4 * 4) + smem_count;
    cudaError_t e = ensure_smem_attr(reinterpret_cast<const void*>(dense_scatter_kernel), smem);
    if (e != cudaSuccess) return e;
    e = ensure_smem_attr(reinterpret_cast<const void*>(dense_count_kernel), smem_count);
    if (e != cudaSuccess) return e;
    count_launch(2);
    dense_count_kernel<<<grid, kRerouteThreads, smem_count, stream>>>(b, L);
    dense_scatter_kernel<<<grid, kRerouteThreads, smem, stream>>>(b, L, P, D, quota_mode, interleave);
    return cudaGetLastError();
}

cudaError_t launch_dense_backward(const Batch<DenseBwdArgs>& b, int L, int P, int D, cudaStream_t stream) {
    int max_T = 0;
    for (int i = 0; i < b.n; ++i) max_T = b.a[i].T > max_T ? b.a[i].T : max_T;
    if (max_T == 0) return cudaSuccess;
    int64_t blocks = (static_cast<int64_t>(max_T) * L / 4 + kRerouteThreads - 1) / kRerouteThreads + 1;
    const int64_t cap = (148 * 16) / b.n > 1 ? (148 * 16) / b.n : 1;
    if (blocks > cap) blocks = cap;
    count_launch();
    dense_backward_kernel<<<dim3(static_cast<unsigned>(blocks), b.n), kRerouteThreads, 0, stream>>>(b, L, P, D);
    return cudaGetLastError();
}

template <typename IdT>
static cudaError_t launch_sparse_typed(const Batch<SparseArgs>& b, int K, int L, int D, int interleave,
                                       cudaStream_t stream) {
    int64_t max_n = 0;
    for (int i = 0; i < b.n; ++i) {
        const int64_t n = static_cast<int64_t>(b.a[i].T) * K;
        max_n = n > max_n ? n : max_n;
    }
    if (max_n == 0) return cudaSuccess;
    const dim3 grid(static_cast<unsigned>(sparse_tiles(max_n)), b.n);
    const size_t smem1 = sizeof(int32_t) * L;
    const size_t smem2 = sizeof(int32_t) * L + sizeof(Router) * L + sizeof(int32_t) * (kRerouteThreads / 32) * L;
    cudaError_t e = ensure_smem_attr(reinterpret_cast<const void*>(sparse_count_kernel<IdT>), smem1);
    if (e != cudaSuccess) return e;
    e = ensure_smem_attr(reinterpret_cast<const void*>(sparse_reroute_kernel<IdT>), smem2);
    if (e != cudaSuccess) return e;
    count_launch(2);
    sparse_count_kernel<IdT><<<grid, kRerouteThreads, smem1, stream>>>(b, K, L);
    sparse_reroute_kernel<IdT><<<grid, kRerouteThreads, smem2, stream>>>(b, K, L, D, interleave);
    return cudaGetLastError();
}

cudaError_t launch_sparse_reroute(const Batch<SparseArgs>& b, int ids_kind, int K, int L, int D, int interleave,
                                  cudaStream_t stream) {
    if (ids_kind == 2) return launch_sparse_typed<long long>(b, K, L, D, interleave, stream);
    return launch_sparse_typed<int32_t>(b, K, L, D, interleave, stream);
}

}  // namespace uep

using namespace uep;

extern "C" {

int64_t uep_reroute_scratch_elems(int64_t T, int K_or_0, int L) {
    if (K_or_0 <= 0) return dense_scratch_elems(static_cast<int>(T), L);
    return sparse_scratch_elems(T * K_or_0, L);
}

int uep_dense_reroute_forward(const uint8_t* routing_map, const float* probs, const int32_t* l2p,
                              const int32_t* lcnts, const int32_t* rank_quota_prefix, uint8_t* expanded_map,
                              float* expanded_probs, int32_t* scratch, int T, int L, int P, int D, int quota_mode,
                              int interleave, void* stream_) {
    if (T < 0 || L <= 0 || P <= 0 || D < 1) return fail(UEP_ERR_INVALID, "dense_reroute_forward: bad sizes");
    if (T == 0) return UEP_OK;
    if (!routing_map || !probs || !l2p || !lcnts || !expanded_map || !expanded_probs || !scratch ||
        (quota_mode && !rank_quota_prefix))
        return fail(UEP_ERR_INVALID, "dense_reroute_forward: null pointer");
    if (D > 255) return fail(UEP_ERR_INVALID, "dense_reroute_forward: more than 255 replicas per expert");
    Batch<DenseFwdArgs> b{};
    b.n = 1;
    b.a[0] = DenseFwdArgs{routing_map, probs, l2p, lcnts, rank_quota_prefix, scratch, expanded_map, expanded_probs, T};
    UEP_CUDA_TRY(launch_dense_forward(b, L, P, D, quota_mode, interleave, static_cast<cudaStream_t>(stream_)));
    return UEP_OK;
}

int uep_dense_reroute_backward(const float* grad_expanded, const uint8_t* routing_map, const uint8_t* expanded_map,
                               const int32_t* l2p, const int32_t* lcnts, float* grad_probs, int T, int L, int P, int D,
                               void* stream_) {
    if (T < 0 || L <= 0 || P <= 0 || D < 1) return fail(UEP_ERR_INVALID, "dense_reroute_backward: bad sizes");
    if (T == 0) return UEP_OK;
    if (!grad_expanded || !routing_map || !expanded_map || !l2p || !lcnts || !grad_probs)
        return fail(UEP_ERR_INVALID, "dense_reroute_backward: null pointer");
    Batch<DenseBwdArgs> b{};
    b.n = 1;
    b.a[0] = DenseBwdArgs{grad_expanded, routing_map, expanded_map, l2p, lcnts, grad_probs, T};
    UEP_CUDA_TRY(launch_dense_backward(b, L, P, D, static_cast<cudaStream_t>(stream_)));
    return UEP_OK;
}

static int sparse_common(int kind, const void* ids, void* out, int T, int K, int L, const int32_t* l2p,
                         const int32_t* lcnts, const int32_t* rqp, int D, int interleave, int32_t* scratch,
                         void* stream_) {
    if (T < 0 || K < 0 || L <= 0 || D < 1) return fail(UEP_ERR_INVALID, "sparse_reroute: bad sizes");
    if (static_cast<int64_t>(T) * K == 0) return UEP_OK;
    if (!ids || !out || !scratch || !l2p || !lcnts || !rqp) return fail(UEP_ERR_INVALID, "sparse_reroute: null pointer");
    Batch<SparseArgs> b{};
    b.n = 1;
    b.a[0] = SparseArgs{ids, out, l2p, lcnts, rqp, scratch, T};
    UEP_CUDA_TRY(launch_sparse_reroute(b, kind, K, L, D, interleave, static_cast<cudaStream_t>(stream_)));
    return UEP_OK;
}

int uep_sparse_reroute_i32(const int32_t* ids, int32_t* out, int T, int K, int L, const int32_t* l2p,
                           const int32_t* lcnts, const int32_t* rank_quota_prefix, int D, int interleave,
                           int32_t* scratch, void* stream) {
    return sparse_common(1, ids, out, T, K, L, l2p, lcnts, rank_quota_prefix, D, interleave, scratch, stream);
}
int uep_sparse_reroute_i64(const int64_t* ids, int64_t* out, int T, int K, int L, const int32_t* l2p,
                           const int32_t* lcnts, const int32_t* rank_quota_prefix, int D, int interleave,
                           int32_t* scratch, void* stream) {
    return sparse_common(2, ids, out, T, K, L, l2p, lcnts, rank_quota_prefix, D, interleave, scratch, stream);
}

// ---------------------------------------------------------------------------------------
// Sparse reroute for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc on the path where routing happens: an
// inference server that has handed the whole device to its own memory pool, a caller inside
// a region where the allocator is frozen, or a plugin boundary that only passes the tensors
// it was given. The regular entry point needs a caller-provided scratch buffer (per-tile
// expert counts); this variant keeps that scratch in a fixed array that is part of the
// loaded library image on every device, so the caller passes inputs and outputs only.
//
// Limits and rules:
//   * the per-tile counts must fit the array: ceil(T*K / 2048) * L + 4 <= 262144 int32 (1 MiB);
//     e.g. 131072 entries (16384 tokens x top-8) with up to 4096 experts, or 1M entries with 512.
//     Larger problems are refused with UEP_ERR_INVALID and a message, nothing is launched;
//   * the array is shared by every call on a device and keeps the previous call's counts. The
//     count pass overwrites every element the second pass reads, so nothing has to start at
//     zero; but two calls that can overlap on the GPU (different streams without an ordering
//     between them) would race on it: order them;
//   * the first call on a device resolves the array's device address (once per device, with
//     that device current). It launches nothing else extra, but it should be made before any
//     stream capture begins.
static constexpr int64_t kStaticRerouteScratchElems = 256 * 1024;
static __device__ __align__(256) int32_t g_static_reroute_scratch[kStaticRerouteScratchElems];

int uep_sparse_reroute_i32_static(const int32_t* ids, int32_t* out, int T, int K, int L, const int32_t* l2p,
                                  const int32_t* lcnts, const int32_t* rank_quota_prefix, int D, int interleave,
                                  void* stream) {
    if (T < 0 || K < 0 || L <= 0 || D < 1) return fail(UEP_ERR_INVALID, "sparse_reroute_static: bad sizes");
    const int64_t need = sparse_scratch_elems(static_cast<int64_t>(T) * K, L);
    if (need > kStaticRerouteScratchElems) {
        return fail(UEP_ERR_INVALID, "sparse_reroute_static: needs " + std::to_string(need) +
                                         " int32 of scratch, the built-in array holds " +
                                         std::to_string(kStaticRerouteScratchElems) +
                                         " (use uep_sparse_reroute_i32 with your own scratch)");
    }
    // In host code the array's name is only a handle for the runtime: the address a kernel can
    // use has to be asked for, per device, while that device is current.
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static int32_t* device_ptr[kMaxDevices] = {nullptr};
    int dev = -1;
    UEP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(UEP_ERR_UNSUPPORTED, "sparse_reroute_static: device index above 63");
    int32_t* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (device_ptr[dev] == nullptr) {
            void* p = nullptr;
            UEP_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_reroute_scratch));
            device_ptr[dev] = static_cast<int32_t*>(p);
        }
        scratch = device_ptr[dev];
    }
    return sparse_common(1, ids, out, T, K, L, l2p, lcnts, rank_quota_prefix, D, interleave, scratch, stream);
}

int64_t uep_dispatch_scratch_elems(int64_t num_entries, int P) { return sparse_tiles(num_entries) * (P + 1) + 4; }

int uep_dispatch_positions(const int32_t* phys_ids, int64_t num_entries, int P, int32_t* pos,
                           int32_t* expert_offsets, int32_t* scratch, void* stream_) {
    if (num_entries < 0 || P <= 0) return fail(UEP_ERR_INVALID, "dispatch_positions: bad sizes");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (num_entries == 0) {
        if (expert_offsets) UEP_CUDA_TRY(cudaMemsetAsync(expert_offsets, 0, sizeof(int32_t) * (P + 1), stream));
        return UEP_OK;
    }
    if (!phys_ids || !pos || !scratch) return fail(UEP_ERR_INVALID, "dispatch_positions: null pointer");
    const int tiles = static_cast<int>(sparse_tiles(num_entries));
    const int nb = P + 1;
    const size_t smem1 = sizeof(int32_t) * nb;
    const size_t smem2 = sizeof(int32_t) * nb * (2 + kRerouteThreads / 32);
    UEP_CUDA_TRY(ensure_smem_attr(reinterpret_cast<const void*>(key_count_kernel<int32_t>), smem1));
    UEP_CUDA_TRY(ensure_smem_attr(reinterpret_cast<const void*>(dispatch_positions_kernel), smem2));
    count_launch(2);
    key_count_kernel<int32_t><<<tiles, kRerouteThreads, smem1, stream>>>(phys_ids, num_entries, P, 1, scratch);
    dispatch_positions_kernel<<<tiles, kRerouteThreads, smem2, stream>>>(phys_ids, num_entries, P, scratch, tiles, pos,
                                                                         expert_offsets);
    UEP_CUDA_TRY(cudaGetLastError());
    return UEP_OK;
}

int uep_gather_rows(const void* in, const int32_t* pos, void* out, int64_t num_rows, int64_t num_src_rows,
                    int64_t row_bytes, int32_t* status, void* stream_) {
    if (num_rows < 0 || row_bytes <= 0 || num_src_rows < 0) return fail(UEP_ERR_INVALID, "gather_rows: bad sizes");
    if (num_rows == 0) return UEP_OK;
    if (!in || !pos || !out) return fail(UEP_ERR_INVALID, "gather_rows: null pointer");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    DeviceStatus* st = reinterpret_cast<DeviceStatus*>(status);
    const bool aligned = (row_bytes % 16 == 0) && ((reinterpret_cast<uintptr_t>(in) & 15u) == 0) &&
                         ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
    count_launch();
    if (aligned) {
        const int chunks = static_cast<int>((row_bytes + kGatherChunk - 1) / kGatherChunk);
        const size_t smem = static_cast<size_t>(kGatherStages) * kGatherChunk;
        UEP_CUDA_TRY(ensure_smem_attr(reinterpret_cast<const void*>(gather_rows_kernel), smem));
        int64_t ctas = num_rows * chunks;
        if (ctas > 2 * 148) ctas = 2 * 148;
        gather_rows_kernel<<<static_cast<int>(ctas), 32, smem, stream>>>(
            static_cast<const uint8_t*>(in), pos, static_cast<uint8_t*>(out), num_rows, row_bytes, chunks,
            num_src_rows, 2000000000ull, st);
    } else {
        int64_t ctas = num_rows > 148 * 8 ? 148 * 8 : num_rows;
        gather_rows_plain_kernel<<<static_cast<int>(ctas), 256, 0, stream>>>(
            static_cast<const uint8_t*>(in), pos, static_cast<uint8_t*>(out), num_rows, row_bytes, num_src_rows, st);
    }
    UEP_CUDA_TRY(cudaGetLastError());
    return UEP_OK;
}

}  // extern "C"
