// Shared host/device helpers for libb200_kernels (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/b200_kernels.h"

namespace b200k {

// ---- host: status + thread-local message ---------------------------------
int fail(int code, const char *fmt, ...);
int launch_status(const char *what);
// Per-device default workspace (allocated on first use unless installed by the caller).
int default_workspace(void **ptr, size_t *bytes);
int sm_count();
// The device status word kernels report through (first word of the default workspace); nullptr when the
// workspace cannot be had, in which case kernels skip the report.
int *status_word();

#define B200K_REQUIRE(cond, code, ...)                 \
    do {                                               \
        if (!(cond)) return b200k::fail(code, __VA_ARGS__); \
    } while (0)

// Integer value of an environment variable, read once per process and variable (tuning overrides are not meant
// to change while the process runs); `dflt` when unset or empty.
int env_int(const char *name, int dflt);
// First character of an environment variable (0 when unset), read once.
int env_char(const char *name);

// Runs a set-up call (e.g. cudaFuncSetAttribute, which is per device) at most once per device, thread-safely.
// A failed call is not remembered: the next caller tries again.
struct OncePerDevice {
    std::mutex mu;
    bool done[16] = {};
    template <typename F> cudaError_t run(F f) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 16) return f();
        std::lock_guard<std::mutex> lk(mu);
        if (done[dev]) return cudaSuccess;
        cudaError_t e = f();
        if (e == cudaSuccess) done[dev] = true;
        return e;
    }
};

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline cudaStream_t to_stream(b200k_stream s) { return reinterpret_cast<cudaStream_t>(s); }
static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- programmatic dependent launch ------------------------------------------------------------
// Kernels of a decode step follow one another on one stream, each a few microseconds long.  Launched with the
// programmatic-serialization attribute, a kernel may start (be scheduled, run its set-up) while its predecessor
// is still draining; it must execute pdl_wait() before it touches anything the predecessor wrote or still reads,
// and pdl_wait() returns only when the predecessor has completed and its writes are visible.
// pdl_launch_dependents() tells the scheduler that the successor may be brought in as soon as there is room.
// Both are no-ops in a kernel launched without the attribute.  B200K_PDL=0 turns the attribute off.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- device: reductions ----------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over a block of up to 1024 threads; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float *smem32) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    v = warp_sum(v);
    if (lane == 0) smem32[wid] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float r = lane < nw ? smem32[lane] : 0.f;
    r = warp_sum(r);
    __syncthreads();
    return r;
}

// ---- device: 128-bit access -----------------------------------------------
struct __align__(16) half8 {
    __half2 v[4];
};
__device__ __forceinline__ uint4 ldg_nc_v4(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
__device__ __forceinline__ float2 h2_to_f2(uint32_t u) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&u));
}
__device__ __forceinline__ uint32_t f2_to_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

}  // namespace b200k
