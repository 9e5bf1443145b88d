// Bulk asynchronous copies (TMA, untiled cp.async.bulk) with mbarrier completion, programmatic
// dependent launch, and the launch helper shared by the streaming kernels.
//
// Every wait is bounded (Waiter): when a wait runs out the waiter records an error code in the
// device state and carries on (results are then garbage, but the kernel terminates and the host
// reports the failure).  Every copy targets the issuing CTA only.
#pragma once
#include "brrr_dev.cuh"

namespace brrr {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// make freshly initialised barriers visible to the async proxy
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// global -> this CTA's shared memory; src, dst 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}

// the same with a suspend-time hint: the warp sleeps in hardware until the phase completes or about `ns`
// nanoseconds have passed, so a thread that waits long issues few instructions while it waits
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t *bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
                 : "memory");
    return ok != 0;
}

// non-blocking probe: cheap when the phase has already completed
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}

constexpr long long WAIT_CYCLES = 2000000000ll;      // about one second of SM clock

// Bounded waiting on copy barriers.  A wait that exceeds WAIT_CYCLES records the error once in
// the device state and marks the thread dead: every later wait returns at once, so a lost copy
// costs about a second, not a hang.  A kernel that starts with the error word already set skips
// its waits altogether (poison_if_failed).
struct Waiter {
    uint32_t *err;
    bool dead;
    __device__ __forceinline__ explicit Waiter(uint32_t *e) : err(e), dead(false) {}
    __device__ __forceinline__ void poison_if_failed() {
        if (err && *reinterpret_cast<volatile uint32_t *>(err) != 0u) dead = true;
    }
    __device__ __forceinline__ bool wait(uint64_t *bar, uint32_t parity) {
        if (dead) return false;
        if (mbar_test_wait(bar, parity)) return true;
        if (mbar_try_wait(bar, parity)) return true;
        const long long t0 = clock64();
        do {
            for (int i = 0; i < 128; i++)
                if (mbar_try_wait(bar, parity)) return true;
        } while (clock64() - t0 < WAIT_CYCLES);
        dead = true;
        if (err) atomicCAS(err, (uint32_t)DEV_ERR_NONE, (uint32_t)DEV_ERR_COPY_TIMEOUT);
        return false;
    }
    // The same bounded wait with hardware suspension between probes (see mbar_try_wait_hint): for roles that
    // spend most of their time waiting beside busy warps (producers, issuing threads) and must still wake at once.
    __device__ __forceinline__ bool wait_suspended(uint64_t *bar, uint32_t parity) {
        if (dead) return false;
        if (mbar_test_wait(bar, parity)) return true;
        const long long t0 = clock64();
        do {
            for (int i = 0; i < 16; i++)
                if (mbar_try_wait_hint(bar, parity, 4000u)) return true;
        } while (clock64() - t0 < WAIT_CYCLES);
        dead = true;
        if (err) atomicCAS(err, (uint32_t)DEV_ERR_NONE, (uint32_t)DEV_ERR_COPY_TIMEOUT);
        return false;
    }
    // The same bounded wait for a thread that is not on the critical path (a producer or an issuing
    // thread that runs ahead of its consumers): it sleeps between polls, because a thread that
    // polls a barrier back to back keeps the shared-memory pipeline busy and slows every other
    // shared-memory access of the SM.
    __device__ __forceinline__ bool wait_relaxed(uint64_t *bar, uint32_t parity) {
        if (dead) return false;
        if (mbar_test_wait(bar, parity)) return true;
        const long long t0 = clock64();
        do {
            for (int i = 0; i < 64; i++) {
                __nanosleep(32);
                if (mbar_test_wait(bar, parity)) return true;
            }
        } while (clock64() - t0 < WAIT_CYCLES);
        dead = true;
        if (err) atomicCAS(err, (uint32_t)DEV_ERR_NONE, (uint32_t)DEV_ERR_COPY_TIMEOUT);
        return false;
    }
};

// ---- words that another GPU writes or reads over NVLink peer memory (expert parallelism)
constexpr long long EP_WAIT_CYCLES = 20000000000ll;     // about ten seconds of SM clock
__device__ __forceinline__ uint32_t ld_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_sys(uint32_t *p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ float ld_f32_sys(const float *p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
// Wait until *p >= want (wrap-safe), at most EP_WAIT_CYCLES; on expiry record the error and give up.
__device__ __forceinline__ bool ep_wait(const uint32_t *p, uint32_t want, uint32_t *err) {
    if (err && *reinterpret_cast<volatile uint32_t *>(err) != 0u) return false;
    const long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if ((int32_t)(ld_sys(p) - want) >= 0) return true;
        if (clock64() - t0 > EP_WAIT_CYCLES) break;
    }
    if (err) atomicCAS(err, (uint32_t)DEV_ERR_NONE, (uint32_t)DEV_ERR_PEER_TIMEOUT);
    return false;
}

// Programmatic dependent launch.  pdl_wait(): block until the preceding kernel in the stream has
// completed and its writes are visible.  pdl_trigger(): allow the next kernel's CTAs to be
// scheduled.  Kernels here issue their weight copies first, then wait, then trigger, so the
// next kernel starts only after the kernel before this one has finished.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Opt a kernel in to `bytes` of dynamic shared memory, once per kernel and device: the attribute
// belongs to the device's copy of the kernel, and one process may open models on several GPUs.
// done_mask: a static word of the caller, one bit per device.
template <typename K>
inline cudaError_t smem_optin(K kern, int bytes, unsigned long long &done_mask) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && ((done_mask >> dev) & 1ull)) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && dev >= 0 && dev < 64) done_mask |= 1ull << dev;
    return e;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

}  // namespace brrr
