// Device-side building blocks shared by the four kernels: system-scope flag
// loads/stores, bounded waits, mbarrier + 1-D bulk-copy (TMA) wrappers, and the
// status word that replaces device asserts.
//
// Rule of this code base: no wait is unbounded and nothing traps. A wait that
// runs past its time limit records a code in the status word and the kernel
// finishes normally, so the context stays usable and the host can raise.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/uep_b200.h"

namespace uep {

constexpr int kMaxExpertsPerDomain = 512;  // same static limits as the reference solver
constexpr int kMaxRanksPerDomain = 72;
constexpr int kMaxExportsPerDomain = 512;
constexpr int kWarp = 32;
constexpr unsigned kFullMask = 0xFFFFFFFFu;

// Status word: {code, detail}. Lives in mapped pinned host memory in the manager, or in
// device memory for the stateless entry points. First error wins.
struct DeviceStatus {
    int code;
    int detail;
};

__device__ __forceinline__ void report_error(DeviceStatus* st, int code, int detail) {
    if (st == nullptr) return;
    if (atomicCAS(&st->code, 0, code) == 0) {
        st->detail = detail;
        __threadfence_system();
    }
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u64(uint64_t* p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu_s32(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Spin until *flag >= target or the time limit passes. Returns true on success.
__device__ __forceinline__ bool wait_flag_ge(const uint64_t* flag, uint64_t target, uint64_t timeout_ns) {
    if (ld_acquire_sys_u64(flag) >= target) return true;
    const uint64_t start = global_timer_ns();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (ld_acquire_sys_u64(flag) >= target) return true;
            __nanosleep(40);
        }
        if (global_timer_ns() - start > timeout_ns) return false;
    }
}

// A 64-bit word that carries its own validity: high half = epoch tag, low half = payload.
// An aligned 8-byte store is single-copy atomic, so a reader that sees the tag sees the
// payload: no fence and no separate flag are needed between the two.
__device__ __forceinline__ uint64_t ld_relaxed_sys_u64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys_u64(uint64_t* p, uint64_t v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t tag_word(uint32_t tag, uint32_t payload) {
    return (static_cast<uint64_t>(tag) << 32) | payload;
}
// Spin until the word at p carries `tag` or the time limit passes. Returns true on success and
// leaves the word in `w`.
__device__ __forceinline__ bool wait_tagged_word(const uint64_t* p, uint32_t tag, uint64_t timeout_ns, uint64_t& w) {
    w = ld_relaxed_sys_u64(p);
    if (static_cast<uint32_t>(w >> 32) == tag) return true;
    const uint64_t start = global_timer_ns();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            w = ld_relaxed_sys_u64(p);
            if (static_cast<uint32_t>(w >> 32) == tag) return true;
            __nanosleep(20);
        }
        if (global_timer_ns() - start > timeout_ns) return false;
    }
}

// As wait_flag_ge, with relaxed polls: the caller closes the wait with one acquire fence.
__device__ __forceinline__ bool wait_flag_ge_relaxed(const uint64_t* flag, uint64_t target, uint64_t timeout_ns) {
    if (ld_relaxed_sys_u64(flag) >= target) return true;
    const uint64_t start = global_timer_ns();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (ld_relaxed_sys_u64(flag) >= target) return true;
            __nanosleep(20);
        }
        if (global_timer_ns() - start > timeout_ns) return false;
    }
}

// ---------------------------------------------------------------------------------
// mbarrier + bulk async copies (non-multicast, 1-D). Addresses and sizes must be
// multiples of 16 bytes; callers check and take a plain-load path otherwise.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test of an mbarrier phase (try_wait may suspend the thread for a while before it answers).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait on an mbarrier phase. Returns false on timeout.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t timeout_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_timer_ns();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (global_timer_ns() - start > timeout_ns) return false;
    }
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// orders this thread's earlier generic-proxy accesses (e.g. the acquire of a ready flag) before its
// later bulk copies (async proxy) on global memory
__device__ __forceinline__ void fence_proxy_async_global() {
    asm volatile("fence.proxy.async.global;" ::: "memory");
}
// global -> shared, completion counted on an mbarrier
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_addr(smem_dst)),
        "l"(gsrc), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}
// shared -> global (local or peer memory), tracked by the bulk async-group
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_addr(smem_src)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() {  // smem of all but the N newest groups is reusable
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {  // writes of all but the N newest groups are complete
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint4 ld_global_cg_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_global_nc_v4(const void* p) {  // read-only local data, streaming
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_global_cs_v4(void* p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ int warp_sum(int v) { return __reduce_add_sync(kFullMask, v); }
__device__ __forceinline__ int warp_max(int v) { return __reduce_max_sync(kFullMask, v); }

__host__ __device__ __forceinline__ int64_t align_up_i64(int64_t v, int64_t a) { return (v + a - 1) / a * a; }
__host__ __device__ __forceinline__ int ceil_div_i(int a, int b) { return (a + b - 1) / b; }

}  // namespace uep
