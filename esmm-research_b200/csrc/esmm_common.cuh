// Shared host/device helpers of libesmm_b200 (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/esmm.h"

namespace esmm {

constexpr int BK = 8;    // K offsets per pattern byte (the reference's BK)
constexpr int PAT_N = 32;  // columns of B per pattern byte (the reference's WN)

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Records a CUDA error for esmm_last_cuda_error() and maps it to ESMM_ERR_CUDA.
int record_cuda_error(cudaError_t e, const char *what);
int record_cuda_error_text(const char *text);

#define ESMM_CUDA_TRY(expr)                                              \
    do {                                                                 \
        cudaError_t _e = (expr);                                         \
        if (_e != cudaSuccess) return esmm::record_cuda_error(_e, #expr); \
    } while (0)

// Tuning and test hooks (esmm_tuning_set): the value set for `name`, else `dflt`.  Nothing is read
// from the process environment.
int tuning_get(const char *name, int dflt);

// Device status word shared by all kernels of the library (0 = ok).
int *device_status_ptr();  // device address, valid after the first call on the current device

#ifdef __CUDACC__
// Launch of a kernel that calls grid_dependency_wait() before its first read of global memory: it may be placed on the
// GPU while the kernel before it in the stream is still finishing, so that its launch latency and set-up are hidden
// (esmm_tuning_set("NO_DEPENDENT_LAUNCH", 1): the ordinary launch).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning_get("NO_DEPENDENT_LAUNCH", 0) ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}
#endif

#ifdef __CUDACC__
// ---------------------------------------------------------------------------
// Checked build (-DESMM_CHECKED; libesmm_b200_checked.so): indices into shared or global memory that
// depend on the problem's shape or data (not the copy engine's boxes, which the tensor maps bound in
// hardware, nor offsets that are constants of the thread) are tested before the access.  A failed test records ESMM_ERR_BOUNDS and
// the number of the site in the device status word - the first failure wins - and the access is
// skipped: no trap, no fault, the context stays usable and esmm_device_status() reports it.  In the
// product build bounds_ok() is the constant true and the tests compile away.
// ---------------------------------------------------------------------------
#ifdef ESMM_CHECKED
constexpr bool kCheckedBuild = true;
#else
constexpr bool kCheckedBuild = false;
#endif

__device__ __forceinline__ bool bounds_ok(bool in_bounds, int *status, int site)
{
    if (kCheckedBuild && !in_bounds && status) atomicCAS(status, 0, (int)ESMM_ERR_BOUNDS | (site << 8));
    return !kCheckedBuild || in_bounds;
}

// ---------------------------------------------------------------------------
// PTX wrappers: mbarrier, TMA (cp.async.bulk.tensor), timers.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// non-blocking: has the phase with this parity completed?
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Every wait in the library is bounded.  The first tries are a plain spin; after that
// the loop watches a CTA-wide abort flag and a wall-clock budget.  On expiry the flag
// is raised (so that the CTA's other waiters leave too) and false is returned.
constexpr uint64_t WAIT_BUDGET_NS = 2000000000ull;  // 2 s: far above any legitimate wait

// Programmatic dependent launch.  A kernel launched with the stream-serialisation attribute may start while the kernel
// before it in the stream is still running; grid_dependency_wait() returns once that kernel has completed and its
// writes are visible (at once, in a kernel launched the ordinary way).  grid_launch_dependents() in the earlier kernel
// lets the next one's CTAs be placed as soon as there is room for them.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ bool mbar_wait_budget(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                                 uint64_t budget_ns)
{
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
#pragma unroll 1
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - t0 > budget_ns) {
            *abort_flag = 1;
            return false;
        }
    }
}

// The same wait for a warp with nothing to do until the barrier completes and no hurry afterwards: it sleeps
// between polls, so that it takes next to no issue slots from the warps that work.
__device__ __forceinline__ bool mbar_wait_idle(uint32_t bar, uint32_t parity, volatile int *abort_flag)
{
    const uint64_t t0 = global_timer_ns();
#pragma unroll 1
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - t0 > WAIT_BUDGET_NS) {
            *abort_flag = 1;
            return false;
        }
        __nanosleep(2000);
    }
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag)
{
    return mbar_wait_budget(bar, parity, abort_flag, WAIT_BUDGET_NS);
}

// 2-D tiled TMA load, completion counted in bytes on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y,
                                            uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z,
                                            uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
#endif  // __CUDACC__

}  // namespace esmm
