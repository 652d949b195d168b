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

#include <cstdlib>
#include <mutex>
#include <string>
#include <utility>

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

// (ordinal * stride + offset) mod total; all operands are non-negative. The product fits 32 bits for every
// realistic token count, where the remainder is one hardware-assisted division instead of the 64-bit routine.
__device__ __forceinline__ int mod_product(int ordinal, int stride, int offset, int total) {
    const unsigned long long prod = static_cast<unsigned long long>(static_cast<unsigned>(ordinal)) * static_cast<unsigned>(stride) +
                                    static_cast<unsigned>(offset);
    if ((prod >> 32) == 0) return static_cast<int>(static_cast<unsigned>(prod) % static_cast<unsigned>(total));
    return static_cast<int>(prod % static_cast<unsigned long long>(total));
}

// ordinal -> replica index (reroute.cu:239-254 of the reference; round-robin: :126). `prefix` is the expert's
// row of inclusive rank-quota prefixes (at least C entries).
__device__ __forceinline__ int replica_index(const Router& r, int ordinal, const int32_t* prefix, bool quota_mode) {
    if (r.C <= 1) return 0;  // one instance: every branch below ends at index 0
    if (!quota_mode) return ordinal % r.C;
    int qr = ordinal;
    if (r.stride != 0) qr = mod_product(ordinal, r.stride, r.offset, r.total);
    int idx = 0;
    for (int j = 0; j < r.C; ++j) idx += (qr >= prefix[j]) ? 1 : 0;
    return min(idx, max(r.C - 1, 0));
}

// The first kStagedReps entries of every expert's plan rows (rank-quota prefixes and physical ids) are copied
// into shared memory once per CTA: resolving an entry then costs no global load. Experts with more instances
// than that read their rows from global memory.
constexpr int kStagedReps = 8;

// Thread-per-expert set-up: routing parameters and the staged rows; every global load of an expert is issued
// before the first one is used (two dependent round trips in all: the count, then the rows).
__device__ __forceinline__ void stage_expert(int e, const int32_t* __restrict__ lcnts, const int32_t* __restrict__ rqp,
                                             const int32_t* __restrict__ l2p, int D, bool quota_mode, bool interleave,
                                             Router* routers, int32_t* prefix_s, int32_t* l2p_s) {
    Router r;
    r.C = lcnts[e];
    const int n = min(min(r.C, D), kStagedReps);
    int32_t pre[kStagedReps], phys[kStagedReps];
    int last = 0;
#pragma unroll
    for (int j = 0; j < kStagedReps; ++j) {
        pre[j] = (j < n && quota_mode) ? rqp[static_cast<int64_t>(e) * D + j] : 0;
        phys[j] = j < n ? l2p[static_cast<int64_t>(e) * D + j] : -1;
    }
    if (quota_mode && r.C > kStagedReps) last = rqp[static_cast<int64_t>(e) * D + r.C - 1];
#pragma unroll
    for (int j = 0; j < kStagedReps; ++j) {
        prefix_s[e * kStagedReps + j] = pre[j];
        l2p_s[e * kStagedReps + j] = phys[j];
        if (j == r.C - 1) last = pre[j];
    }
    r.total = (quota_mode && r.C > 0) ? last : 0;
    r.stride = 0;  // marks "no interleave"
    r.offset = 0;
    if (quota_mode && interleave && r.total > 1) {
        int st = r.total / 2 + 1;
        if (st >= r.total) st = r.total - 1;
        if (st < 1) st = 1;
        while (gcd_int(st, r.total) != 1) {
            ++st;
            if (st >= r.total) st = 1;
        }
        r.stride = st;
        r.offset = e % r.total;
    }
    routers[e] = r;
}

// Programmatic dependent launch: the second kernel of a pair is launched with the stream-serialisation
// attribute, so its prologue (everything that does not read the first kernel's output) overlaps the first
// kernel. `pdl_wait` returns once the first kernel has completed and its writes are visible; without the
// launch attribute both instructions do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

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

// The count of a (tile, expert) pair is at most kDenseTileRows = 64: it is kept in ONE BYTE, row-major
// [tile][L] in the scratch buffer, so that the second kernel can add up the tiles in front of it sixteen
// experts per load. `fast`: L is a multiple of 16 with L/16 in {1,2,4,...,32}, the map and the scratch are
// 16-byte aligned: a thread then always meets the same sixteen columns and can add map bytes as packed words.
__device__ __forceinline__ bool dense_fast_path(const uint8_t* map, const void* scratch, int L) {
    const int G = L / 16;
    return (L % 16 == 0) && G <= 32 && (G & (G - 1)) == 0 &&
           ((reinterpret_cast<uintptr_t>(map) | reinterpret_cast<uintptr_t>(scratch)) & 15u) == 0;
}

__global__ void __launch_bounds__(kRerouteThreads) dense_count_kernel(Batch<DenseFwdArgs> batch, int L) {
    pdl_launch_dependents();  // the scatter kernel may start its prologue now
    extern __shared__ __align__(128) char smem_raw[];  // fast: [L/4] packed words; else [kDenseTileRows][L] bytes
    const DenseFwdArgs& a = batch.a[blockIdx.y];
    const int T = a.T;
    const int tile = blockIdx.x;
    const int r0 = tile * kDenseTileRows, r1 = min(r0 + kDenseTileRows, T);
    if (r0 >= T) return;
    uint8_t* counts = reinterpret_cast<uint8_t*>(a.scratch) + static_cast<int64_t>(tile) * L;
    if (dense_fast_path(a.map, a.scratch, L)) {
        const int G = L / 16;
        uint32_t* cnt = reinterpret_cast<uint32_t*>(smem_raw);
        for (int i = threadIdx.x; i < L / 4; i += blockDim.x) cnt[i] = 0;
        __syncthreads();
        // vector i of the tile covers row i / G, columns 16 * (i % G) ..; blockDim is a multiple of G, so a
        // thread always meets the same column group and adds the 0/1 bytes of its rows as packed words
        const uint8_t* src = a.map + static_cast<int64_t>(r0) * L;
        const int nvec = (r1 - r0) * G;
        uint4 acc = make_uint4(0, 0, 0, 0);
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
            const uint4 v = ld_global_nc_v4(src + static_cast<int64_t>(i) * 16);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        // lanes with the same column group inside the warp
        for (int d = G; d < 32; d <<= 1) {
            acc.x += __shfl_xor_sync(kFullMask, acc.x, d); acc.y += __shfl_xor_sync(kFullMask, acc.y, d);
            acc.z += __shfl_xor_sync(kFullMask, acc.z, d); acc.w += __shfl_xor_sync(kFullMask, acc.w, d);
        }
        const int lane = threadIdx.x & 31;
        if (lane < G) {  // a byte never exceeds 64, so packed adds cannot carry into the next byte
            atomicAdd(cnt + lane * 4 + 0, acc.x); atomicAdd(cnt + lane * 4 + 1, acc.y);
            atomicAdd(cnt + lane * 4 + 2, acc.z); atomicAdd(cnt + lane * 4 + 3, acc.w);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < L / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(counts)[i] = cnt[i];
        return;
    }
    uint8_t* smap = reinterpret_cast<uint8_t*>(smem_raw);
    stage_map_tile(a.map, r0, r1, L, smap);
    __syncthreads();
    for (int e = threadIdx.x; e < L; e += blockDim.x) {
        int c = 0;
        for (int t = 0; t < r1 - r0; ++t) c += smap[t * L + e] ? 1 : 0;
        counts[e] = static_cast<uint8_t>(c);
    }
}

// Second kernel: one CTA per tile of 64 tokens builds the tile of both outputs in shared memory (zeros,
// then the tile's routed cells: 64 x top-k of them, against 64 x P output elements) and writes it out with
// bulk stores. Only the probabilities of routed cells are read. Outputs wider than kDenseMaxChunkCols
// columns are produced in column chunks.
constexpr int kDenseMaxChunkCols = 512;

// Row stride of the staged map tile: 16 bytes of padding keep the row starts 16-byte aligned and spread the
// rows over the shared-memory banks when a thread per row walks across the columns.
__host__ __device__ __forceinline__ int dense_row_stride(int L) { return (L + 15) / 16 * 16 + 16; }

__global__ void __launch_bounds__(kRerouteThreads)
dense_scatter_kernel(Batch<DenseFwdArgs> batch, int L, int P, int D, int quota_mode, int interleave, int chunk_cols,
                     int overlapped) {
    const DenseFwdArgs& a = batch.a[blockIdx.y];
    const uint8_t* __restrict__ map = a.map;
    const float* __restrict__ probs = a.probs;
    const int32_t* __restrict__ l2p = a.l2p;
    const int32_t* __restrict__ lcnts = a.lcnts;
    const int32_t* __restrict__ rqp = a.rqp;
    uint8_t* __restrict__ out_map = a.out_map;
    float* __restrict__ out_probs = a.out_probs;
    const int T = a.T;
    if (static_cast<int>(blockIdx.x) * kDenseTileRows >= T) return;
    extern __shared__ __align__(128) char smem_raw[];
    // layout: probs tile [64][chunk] f32 | map tile [64][chunk] u8 | choice [64][Ls] u8 | routers[L] | base[L] i32 |
    //         prefix rows [L][8] i32 | l2p rows [L][8] i32
    const int Ls = dense_row_stride(L);
    float* tile_probs = reinterpret_cast<float*>(smem_raw);
    uint8_t* tile_map = reinterpret_cast<uint8_t*>(tile_probs + static_cast<size_t>(kDenseTileRows) * chunk_cols);
    uint8_t* choice = tile_map + (static_cast<size_t>(kDenseTileRows) * chunk_cols + 15) / 16 * 16;
    Router* routers = reinterpret_cast<Router*>(choice + static_cast<size_t>(kDenseTileRows) * Ls);
    int32_t* base_of = reinterpret_cast<int32_t*>(routers + L);
    int32_t* prefix_s = base_of + (L + 3) / 4 * 4;
    int32_t* l2p_s = prefix_s + static_cast<size_t>(L) * kStagedReps;

    const int tile = blockIdx.x;
    const int r0 = tile * kDenseTileRows, r1 = min(r0 + kDenseTileRows, T);
    const int rows = r1 - r0;
    const int tid = threadIdx.x;

    auto zero_tile = [&](int cols) {  // both output tiles of the chunk (16-byte stores; the regions are padded)
        uint4* z = reinterpret_cast<uint4*>(tile_probs);
        const int n1 = (rows * cols * 4 + 15) / 16;
        for (int i = tid; i < n1; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
        uint4* zm = reinterpret_cast<uint4*>(tile_map);
        const int n2 = (rows * cols + 15) / 16;
        for (int i = tid; i < n2; i += blockDim.x) zm[i] = make_uint4(0, 0, 0, 0);
    };

    // ---- prologue: nothing here depends on the count kernel ---------------------------------
    // the map tile, row by row into the padded rows (the passes below turn each map byte into its replica choice in place)
    {
        const uint8_t* src = map + static_cast<int64_t>(r0) * L;
        if ((L % 16) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
            const int G = L / 16;
            for (int i = tid; i < rows * G; i += blockDim.x) {
                const int t = i / G, g = i - t * G;
                *reinterpret_cast<uint4*>(choice + t * Ls + g * 16) = ld_global_nc_v4(src + static_cast<int64_t>(i) * 16);
            }
        } else {
            for (int i = tid; i < rows * L; i += blockDim.x) {
                const int t = i / L, e = i - t * L;
                choice[t * Ls + e] = src[i];
            }
        }
    }
    for (int e = tid; e < L; e += blockDim.x) {
        stage_expert(e, lcnts, rqp, l2p, D, quota_mode != 0, interleave != 0, routers, prefix_s, l2p_s);
        base_of[e] = 0;
    }
    {   // the tile's probabilities are needed only after the wait below: ask for their lines now
        const char* pbase = reinterpret_cast<const char*>(probs + static_cast<int64_t>(r0) * L);
        const int64_t pbytes = static_cast<int64_t>(rows) * L * 4;
        for (int64_t off = static_cast<int64_t>(tid) * 128; off < pbytes; off += static_cast<int64_t>(blockDim.x) * 128) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(pbase + off));
        }
    }
    zero_tile(min(chunk_cols, P));
    __syncthreads();
    // ---- ordinal base of every expert: tokens routed to it in the tiles in front of this one ---
    const uint8_t* counts = reinterpret_cast<const uint8_t*>(a.scratch);
    auto sum_earlier_tiles = [&]() {
    if (dense_fast_path(map, a.scratch, L)) {
        const int G = L / 16;
        const int g = tid % G, sub = tid / G, nsub = blockDim.x / G;
        // bytes are widened to 16-bit lanes; a lane overflows after 1024 tiles of 64 rows, so it is spilled before
        uint32_t lo[4] = {0, 0, 0, 0}, hi[4] = {0, 0, 0, 0};
        const int lane = tid & 31;
        auto spill = [&]() {
            // lanes of the warp that hold the same sixteen columns first (their sum stays below 2^16), then one
            // shared-memory add per column from the first of them
            for (int d = G; d < 32; d <<= 1) {
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    lo[w] += __shfl_xor_sync(kFullMask, lo[w], d);
                    hi[w] += __shfl_xor_sync(kFullMask, hi[w], d);
                }
            }
            if (lane < G) {
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int e = g * 16 + w * 4;
                    if (lo[w] & 0xFFFFu) atomicAdd(base_of + e, static_cast<int>(lo[w] & 0xFFFFu));
                    if (hi[w] & 0xFFFFu) atomicAdd(base_of + e + 1, static_cast<int>(hi[w] & 0xFFFFu));
                    if (lo[w] >> 16) atomicAdd(base_of + e + 2, static_cast<int>(lo[w] >> 16));
                    if (hi[w] >> 16) atomicAdd(base_of + e + 3, static_cast<int>(hi[w] >> 16));
                }
            }
#pragma unroll
            for (int w = 0; w < 4; ++w) lo[w] = hi[w] = 0;
        };
        // every thread runs the same number of rounds (the shuffles above need the whole warp)
        const int rounds = (tile + 4 * nsub - 1) / (4 * nsub);
        int since = 0;
        for (int rd = 0; rd < rounds; ++rd) {
            const int tl0 = sub + rd * 4 * nsub;
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {  // four independent loads in flight
                const int tl = tl0 + u * nsub;
                v[u] = tl < tile ? __ldcg(reinterpret_cast<const uint4*>(counts + static_cast<int64_t>(tl) * L) + g)
                                 : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t w4[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    lo[w] += w4[w] & 0x00FF00FFu;
                    hi[w] += (w4[w] >> 8) & 0x00FF00FFu;
                }
            }
            since += 4;
            if (since >= 4 * G) {  // at most (4G + 4) counts of at most 64 per lane, times 32 / G lanes in the shuffle: < 2^15
                spill();
                since = 0;
            }
        }
        spill();
    } else {
        for (int e = tid; e < L; e += blockDim.x) {
            int b = 0;
#pragma unroll 8
            for (int tl = 0; tl < tile; ++tl) b += __ldcg(counts + static_cast<int64_t>(tl) * L + e);
            base_of[e] = b;
        }
    }
    };
    // Launched behind the count kernel in the ordinary way, its counts are complete already and their loads go out
    // before the column walk; launched as a dependent kernel, everything up to the wait reads the map and the plan only.
    if (!overlapped) sum_earlier_tiles();
    // one thread per expert walks its column only to count: a routed cell of an expert with several instances
    // is marked 0x80 | (its rank among the tile's routed rows, < 64); with one instance the choice is 0 at once
    for (int e = tid; e < L; e += blockDim.x) {
        const int C = routers[e].C;
        int seen = 0;
        for (int t = 0; t < rows; ++t) {
            uint8_t c = 0xFF;
            if (choice[t * Ls + e]) {
                c = C <= 1 ? 0 : static_cast<uint8_t>(0x80 | seen);
                ++seen;
            }
            choice[t * Ls + e] = c;
        }
    }

    if (overlapped) {
        pdl_wait();
        sum_earlier_tiles();
    }
    __syncthreads();

    // ---- resolve the marked cells and scatter the routed cells into the output tile. A thread owns one row
    //      and every (blockDim / rows)-th word of it: a row has top-k routed cells, so the work is even however
    //      skewed the experts are (a hot expert's column is spread over all rows' threads). --------------------
    const int words_per_row = (L + 3) / 4;
    const int row_threads = blockDim.x / kDenseTileRows;  // 4
    const int my_row = tid % kDenseTileRows, my_first = tid / kDenseTileRows;
    for (int p_lo = 0; p_lo < P; p_lo += chunk_cols) {
        const int cols = min(chunk_cols, P - p_lo);
        if (p_lo > 0) {
            __syncthreads();  // the previous chunk has left the tile
            zero_tile(cols);
            __syncthreads();
        }
        if (my_row < rows) {
            const float* prow = probs + static_cast<int64_t>(r0 + my_row) * L;
            for (int wd = my_first; wd < words_per_row; wd += row_threads) {
                const uint32_t word = *reinterpret_cast<const uint32_t*>(choice + my_row * Ls + wd * 4);
                if (word == 0xFFFFFFFFu) continue;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    uint8_t c = static_cast<uint8_t>(word >> (8 * k));
                    const int e = wd * 4 + k;
                    if (c == 0xFF || e >= L) continue;
                    const float pv = prow[e];  // issued before the arithmetic below
                    const Router r = routers[e];
                    if (p_lo == 0 && c >= 0x80) {
                        const int32_t* prefix = r.C <= kStagedReps ? prefix_s + e * kStagedReps : rqp + static_cast<int64_t>(e) * D;
                        c = static_cast<uint8_t>(replica_index(r, base_of[e] + (c & 0x3F), prefix, quota_mode != 0));
                        choice[my_row * Ls + e] = c;
                    }
                    const int phys = c < kStagedReps ? l2p_s[e * kStagedReps + c] : l2p[static_cast<int64_t>(e) * D + c];
                    const int p = phys - p_lo;
                    if (p >= 0 && p < cols) {
                        tile_probs[my_row * cols + p] = pv;
                        tile_map[my_row * cols + p] = 1;
                    }
                }
            }
        }
        fence_proxy_async_smem();  // the tile was written with ordinary stores and may leave through bulk stores
        __syncthreads();
        // ---- the tile leaves: one bulk store per output when it is a contiguous, 16-byte aligned block ----
        const int64_t o = static_cast<int64_t>(r0) * P;
        const bool whole = cols == P;
        const bool bulk_p = whole && ((rows * P) % 4 == 0) && ((reinterpret_cast<uintptr_t>(out_probs + o) & 15u) == 0);
        const bool bulk_m = whole && ((rows * P) % 16 == 0) && ((reinterpret_cast<uintptr_t>(out_map + o) & 15u) == 0);
        if ((bulk_p || bulk_m) && tid == 0) {
            if (bulk_p) bulk_store(out_probs + o, tile_probs, static_cast<uint32_t>(rows * P * 4));
            if (bulk_m) bulk_store(out_map + o, tile_map, static_cast<uint32_t>(rows * P));
            bulk_commit();
        }
        if (!bulk_p) {
            for (int i = tid; i < rows * cols; i += blockDim.x) {
                const int t = i / cols, p = i - t * cols;
                out_probs[o + static_cast<int64_t>(t) * P + p_lo + p] = tile_probs[i];
            }
        }
        if (!bulk_m) {
            for (int i = tid; i < rows * cols; i += blockDim.x) {
                const int t = i / cols, p = i - t * cols;
                out_map[o + static_cast<int64_t>(t) * P + p_lo + p] = tile_map[i];
            }
        }
        if ((bulk_p || bulk_m) && tid == 0) bulk_wait_read<0>();  // shared memory must outlive the stores' reads
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
    pdl_launch_dependents();
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

// Row-major ordinal of every entry of this CTA's tile inside its bucket, in two steps so that the first
// one (which reads only the keys) can run before the count kernel has finished:
//   tile_warp_counts: warp_base[w][b] = entries of bucket b in warp w's part of the tile;
//   tile_resolve:     with base[b] = entries of bucket b in front of this tile, turns the counts into
//                     running offsets and hands every entry to emit(i, bucket, ordinal).
// warp_base holds (blockDim/32) * nb ints.
template <typename IdT>
__device__ void tile_warp_counts(const IdT* keys, int64_t n, int nb_valid, bool tail_bucket, int32_t* warp_base) {
    const int nb = nb_valid + (tail_bucket ? 1 : 0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int per_warp = kSparseTileEntries / nwarps;
    const int64_t tile_begin = static_cast<int64_t>(blockIdx.x) * kSparseTileEntries;
    const int64_t wbegin = min(tile_begin + static_cast<int64_t>(warp) * per_warp, n);
    const int64_t wend = min(wbegin + per_warp, n);
    for (int i = threadIdx.x; i < nwarps * nb; i += blockDim.x) warp_base[i] = 0;
    __syncthreads();
    for (int64_t i = wbegin + lane; i < wend; i += kWarp) {
        const int b = key_bucket<IdT>(keys[i], nb_valid, tail_bucket);
        if (b >= 0) atomicAdd(warp_base + warp * nb + b, 1);
    }
    __syncthreads();
}

template <typename IdT, typename Emit>
__device__ void tile_resolve(const IdT* keys, int64_t n, int nb_valid, bool tail_bucket, const int32_t* base,
                             int32_t* warp_base, Emit emit) {
    const int nb = nb_valid + (tail_bucket ? 1 : 0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int per_warp = kSparseTileEntries / nwarps;
    const int64_t tile_begin = static_cast<int64_t>(blockIdx.x) * kSparseTileEntries;
    const int64_t wbegin = min(tile_begin + static_cast<int64_t>(warp) * per_warp, n);
    const int64_t wend = min(wbegin + per_warp, n);
    // exclusive scan over warps, seeded with the tile base
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        int run = base[b];
        for (int w = 0; w < nwarps; ++w) {
            const int c = warp_base[w * nb + b];
            warp_base[w * nb + b] = run;
            run += c;
        }
    }
    __syncthreads();
    // in-order resolution inside the warp
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
    pdl_launch_dependents();  // the reroute kernel may start its prologue now
    extern __shared__ __align__(128) char smem_raw[];
    const SparseArgs& a = batch.a[blockIdx.y];
    const IdT* keys = static_cast<const IdT*>(a.ids);
    const int64_t n = static_cast<int64_t>(a.T) * K;
    const int64_t begin = static_cast<int64_t>(blockIdx.x) * kSparseTileEntries;
    // (a tile behind this rank's entries: the second pass launches the same grid and returns at the same test, so
    // every count it reads has been written by this pass, whatever the scratch buffer held before)
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
sparse_reroute_kernel(Batch<SparseArgs> batch, int K, int L, int D, int interleave, int overlapped) {
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
    // layout: base[L] | routers[L] | prefix rows [L][8] | l2p rows [L][8] | warp_base[nwarps][L]
    int32_t* base = reinterpret_cast<int32_t*>(smem_raw);
    Router* routers = reinterpret_cast<Router*>(base + L);
    int32_t* prefix_s = reinterpret_cast<int32_t*>(routers + L);
    int32_t* l2p_s = prefix_s + static_cast<size_t>(L) * kStagedReps;
    int32_t* warp_base = l2p_s + static_cast<size_t>(L) * kStagedReps;
    const int tile = blockIdx.x;
    auto sum_earlier_tiles = [&]() {
        for (int e = threadIdx.x; e < L; e += blockDim.x) {
            int b = 0;
#pragma unroll 8
            for (int tl = 0; tl < tile; ++tl) b += __ldcg(tile_counts + static_cast<int64_t>(tl) * L + e);
            base[e] = b;
        }
    };
    // Launched behind the count kernel in the ordinary way, its counts are complete already: their loads go out
    // together with those of the plan rows. Launched as a dependent kernel, everything up to the wait reads the
    // plan and the ids only.
    if (!overlapped) sum_earlier_tiles();
    for (int e = threadIdx.x; e < L; e += blockDim.x) {
        stage_expert(e, lcnts, rqp, l2p, D, interleave != 2, interleave == 1, routers, prefix_s, l2p_s);  // 2: round-robin (legacy placement)
    }
    tile_warp_counts<IdT>(ids, n, L, false, warp_base);
    if (overlapped) {
        pdl_wait();  // the tile counts of the first kernel are complete from here on
        sum_earlier_tiles();
        __syncthreads();
    }
    // ids may alias out: every entry is read and written by the same lane, the write comes
    // last, and tiles do not overlap.
    tile_resolve<IdT>(ids, n, L, false, base, warp_base, [&](int64_t i, int b, int ordinal) {
        if (b < 0) {
            out[i] = ids[i];
            return;
        }
        const Router r = routers[b];
        if (r.C <= 0) {
            out[i] = ids[i];
            return;
        }
        const int32_t* prefix = r.C <= kStagedReps ? prefix_s + b * kStagedReps : rqp + static_cast<int64_t>(b) * D;
        const int j = replica_index(r, ordinal, prefix, interleave != 2);
        out[i] = static_cast<IdT>(j < kStagedReps ? l2p_s[b * kStagedReps + j] : l2p[static_cast<int64_t>(b) * D + j]);
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
    tile_warp_counts<int32_t>(phys, n, P, true, warp_base);
    pdl_wait();
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        int before = 0, total = 0;
#pragma unroll 8
        for (int tl = 0; tl < num_tiles; ++tl) {
            const int c = __ldcg(tile_counts + static_cast<int64_t>(tl) * nb + b);
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
    tile_resolve<int32_t>(phys, n, P, true, base, warp_base,
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
    // Remembered per kernel. On first use the kernel also asks for the largest shared-memory carve-out: these
    // kernels run next to weight_sync, whose CTAs need most of an SM's shared memory, and an SM that was set up
    // with a small carve-out for a reroute CTA cannot take a weight_sync CTA until it has drained.
    static std::mutex mu;
    static const void* fns[16];
    static size_t granted[16];
    static int n = 0;
    std::lock_guard<std::mutex> lock(mu);
    int i = 0;
    while (i < n && fns[i] != fn) ++i;
    if (i == n) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        if (n < 16) {
            fns[n] = fn;
            granted[n] = 48 * 1024;
            ++n;
        }
    }
    if (bytes <= 48 * 1024 || (i < 16 && granted[i] >= bytes)) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (e != cudaSuccess) return e;
    if (i < 16) granted[i] = bytes;
    return cudaSuccess;
}

int dense_tiles(int T) { return (T + kDenseTileRows - 1) / kDenseTileRows; }
int64_t sparse_tiles(int64_t n) { return (n + kSparseTileEntries - 1) / kSparseTileEntries; }

}  // namespace

int64_t dense_scratch_elems(int T, int L) { return static_cast<int64_t>(dense_tiles(T)) * L + 4; }
int64_t sparse_scratch_elems(int64_t entries, int L) { return sparse_tiles(entries) * L + 4; }

// Launch of a kernel that may start before the kernel in front of it in the stream has finished
// (programmatic dependent launch); the kernel calls pdl_wait() before it reads that kernel's output.
// UEP_DISABLE_PDL=1 turns the attribute off (the pair then runs strictly one after the other).
bool pdl_enabled() {
    static const bool disabled = [] {
        const char* e = std::getenv("UEP_DISABLE_PDL");
        return e != nullptr && e[0] == '1';
    }();
    return !disabled;
}

template <typename... Params, typename... Args>
cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             bool overlap, Args&&... args) {
    const bool disabled = !pdl_enabled();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (disabled || !overlap) ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

cudaError_t launch_dense_forward(const Batch<DenseFwdArgs>& b, int L, int P, int D, int quota_mode, int interleave,
                                 cudaStream_t stream) {
    int max_T = 0;
    for (int i = 0; i < b.n; ++i) max_T = b.a[i].T > max_T ? b.a[i].T : max_T;
    if (max_T == 0) return cudaSuccess;
    const dim3 grid(dense_tiles(max_T), b.n);
    static_assert(kDenseTileRows <= 64, "a routed cell's rank inside its tile is kept in six bits");
    const size_t smem_count = static_cast<size_t>(kDenseTileRows) * L + 16;
    // shared memory of the scatter kernel: the map tile, the per-expert tables, and as many output columns
    // (five bytes per row and column) as fit beside them
    const size_t fixed = static_cast<size_t>(kDenseTileRows) * dense_row_stride(L) + sizeof(Router) * L +
                         sizeof(int32_t) * ((L + 3) / 4 * 4) + 2 * sizeof(int32_t) * kStagedReps * L + 64;
    const size_t budget = 200 * 1024;
    if (fixed + static_cast<size_t>(kDenseTileRows) * 5 * 16 > budget) return cudaErrorInvalidValue;  // L in the thousands
    int chunk = static_cast<int>((budget - fixed) / (static_cast<size_t>(kDenseTileRows) * 5));
    chunk = chunk > kDenseMaxChunkCols ? kDenseMaxChunkCols : chunk;
    chunk = chunk >= P ? P : chunk / 16 * 16;
    const size_t smem = static_cast<size_t>(kDenseTileRows) * chunk * 4 + (static_cast<size_t>(kDenseTileRows) * chunk + 15) / 16 * 16 + fixed;
    cudaError_t e = ensure_smem_attr(reinterpret_cast<const void*>(dense_scatter_kernel), smem);
    if (e != cudaSuccess) return e;
    e = ensure_smem_attr(reinterpret_cast<const void*>(dense_count_kernel), smem_count);
    if (e != cudaSuccess) return e;
    count_launch(2);
    dense_count_kernel<<<grid, kRerouteThreads, smem_count, stream>>>(b, L);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    // With one rank per launch the pair is latency-bound and the overlap pays; a launch that hosts several ranks
    // fills the device with the first kernel alone, and early CTAs of the second only get in its way.
    const bool overlap = b.n == 1 && pdl_enabled();
    return launch_dependent(dense_scatter_kernel, grid, dim3(kRerouteThreads), smem, stream, overlap, b, L, P, D, quota_mode,
                            interleave, chunk, overlap ? 1 : 0);
}

cudaError_t launch_dense_backward(const Batch<DenseBwdArgs>& b, int L, int P, int D, cudaStream_t stream) {
    int max_T = 0;
    for (int i = 0; i < b.n; ++i) max_T = b.a[i].T > max_T ? b.a[i].T : max_T;
    if (max_T == 0) return cudaSuccess;
    int64_t blocks = (static_cast<int64_t>(max_T) * L / 4 + kRerouteThreads - 1) / kRerouteThreads + 1;
    const int64_t sms = device_sm_count() > 0 ? device_sm_count() : 1;
    const int64_t cap = (sms * 16) / b.n > 1 ? (sms * 16) / b.n : 1;
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
    const size_t smem2 = sizeof(int32_t) * L + sizeof(Router) * L + 2 * sizeof(int32_t) * kStagedReps * L +
                         sizeof(int32_t) * (kRerouteThreads / 32) * L;
    cudaError_t e = ensure_smem_attr(reinterpret_cast<const void*>(sparse_count_kernel<IdT>), smem1);
    if (e != cudaSuccess) return e;
    e = ensure_smem_attr(reinterpret_cast<const void*>(sparse_reroute_kernel<IdT>), smem2);
    if (e != cudaSuccess) return e;
    count_launch(2);
    sparse_count_kernel<IdT><<<grid, kRerouteThreads, smem1, stream>>>(b, K, L);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const bool overlap = b.n == 1 && pdl_enabled();
    return launch_dependent(sparse_reroute_kernel<IdT>, grid, dim3(kRerouteThreads), smem2, stream, overlap, b, K, L, D, interleave,
                            overlap ? 1 : 0);
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
    if (!ids || !out || !scratch || !l2p || !lcnts || (interleave != 2 && !rqp)) return fail(UEP_ERR_INVALID, "sparse_reroute: null pointer");
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
//     e.g. 131072 entries (16384 tokens x top-8) with up to 4095 experts, or 511 tiles (1,046,528
//     entries) with 512 experts: the four spare words count against the limit.
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
    UEP_CUDA_TRY(cudaGetLastError());
    UEP_CUDA_TRY(launch_dependent(dispatch_positions_kernel, dim3(tiles), dim3(kRerouteThreads), smem2, stream, true, phys_ids,
                                  num_entries, P, static_cast<const int32_t*>(scratch), tiles, pos, expert_offsets));
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
        const int64_t sms = device_sm_count() > 0 ? device_sm_count() : 1;
        if (ctas > 2 * sms) ctas = 2 * sms;  // two single-thread CTAs per SM
        gather_rows_kernel<<<static_cast<int>(ctas), 32, smem, stream>>>(
            static_cast<const uint8_t*>(in), pos, static_cast<uint8_t*>(out), num_rows, row_bytes, chunks,
            num_src_rows, 2000000000ull, st);
    } else {
        const int64_t sms = device_sm_count() > 0 ? device_sm_count() : 1;
        int64_t ctas = num_rows > sms * 8 ? sms * 8 : num_rows;
        gather_rows_plain_kernel<<<static_cast<int>(ctas), 256, 0, stream>>>(
            static_cast<const uint8_t*>(in), pos, static_cast<uint8_t*>(out), num_rows, row_bytes, num_src_rows, st);
    }
    UEP_CUDA_TRY(cudaGetLastError());
    return UEP_OK;
}

}  // extern "C"
