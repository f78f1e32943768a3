// Shared device helpers for libshainet_attn (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef __CUDA_ARCH__
#define SHAINET_HOST_SIDE 1
#endif

namespace shainet {

// Device-side status word values (written to AttnStatus::code by kernels that
// give up on a bounded wait; the host reads the word after synchronising).
enum DeviceStatus : int {
    DEV_OK = 0,
    DEV_WAIT_TIMEOUT = 1,   // an mbarrier wait ran past its time limit
};

struct AttnStatus {
    int code;
    int where;   // kernel-specific location id of the first failure
};

// ~1 s at the nominal 1 GHz global timer; long enough that only a programming
// error (never a slow copy) can trip it, short enough that a GPU is not held.
constexpr unsigned long long WAIT_LIMIT_NS = 1000ull * 1000ull * 1000ull;

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: returns false (and records where) once WAIT_LIMIT_NS has
// passed without the phase completing.  Callers must then stop using the
// pipeline and leave the kernel.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, AttnStatus* status, int where) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = globaltimer_ns();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
            if (status != nullptr && atomicCAS(&status->code, DEV_OK, DEV_WAIT_TIMEOUT) == DEV_OK) status->where = where;
            return false;
        }
    }
}

// 1-D bulk asynchronous copy global -> shared (TMA engine, no tensor map, no
// multicast).  dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
        "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ float4 lds128(const float* p) { return *reinterpret_cast<const float4*>(p); }

#endif  // __CUDACC__

}  // namespace shainet
