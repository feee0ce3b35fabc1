// common.cuh -- status/error plumbing and dtype helpers shared by every kernel file.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "nncu.h"

typedef __nv_bfloat16 bf16;

// last error message of the calling thread (nncu_last_error)
extern thread_local char g_nncu_err[512];
int nncu_fail(int code, const char *fmt, ...);

#define CUDA_TRY(expr)                                                                     \
    do {                                                                                   \
        cudaError_t e_ = (expr);                                                           \
        if (e_ != cudaSuccess)                                                             \
            return nncu_fail(e_ == cudaErrorMemoryAllocation ? NNCU_ERR_NOMEM : NNCU_ERR_CUDA, \
                             "%s:%d: %s -> %s", __FILE__, __LINE__, #expr,                 \
                             cudaGetErrorString(e_));                                      \
    } while (0)

#define NNCU_TRY(expr)       \
    do {                     \
        int rc_ = (expr);    \
        if (rc_ != NNCU_OK)  \
            return rc_;      \
    } while (0)

// Programmatic dependent launch.  A kernel started through launch_k may begin while the kernel
// before it on the stream is still draining: its CTAs become resident, run whatever comes before
// pdl_wait() (barrier set-up, TMEM allocation, index arithmetic) and block there until the
// predecessor has completed and its writes are visible.  Rules for a kernel launched this way:
// every thread executes pdl_wait() before its first global-memory access and before any early
// return, so that the kernel cannot complete before its predecessor has.  Both calls are no-ops in
// a kernel launched the ordinary way.  Off unless NNCU_PDL=1: on the c2 train step (graph replay,
// kernels of 3-20 us) it measured within 1 % of ordinary launches.  pdl_trigger() (successor
// starts as soon as all CTAs of this kernel are resident) is compiled in only with
// -DNNCU_PDL_TRIGGER: it measured 4 % slower, the resident successors taking SM resources from
// the side stream's kernels.
__device__ __forceinline__ void pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// the same signal, given late in a kernel (its successor's launch then overlaps only the tail)
__device__ __forceinline__ void pdl_trigger_late()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_trigger()
{
#ifdef NNCU_PDL_TRIGGER
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
inline bool nncu_pdl_enabled()
{
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("NNCU_PDL");
        on = (e && e[0] == '1') ? 1 : 0;
    }
    return on != 0;
}
template <typename... KArgs, typename... Args>
static cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                            Args &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = nncu_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// every kernel launch in the library is followed by exactly one KERNEL_CHECK
extern unsigned long long g_nncu_launches;
#define KERNEL_CHECK()                 \
    do {                               \
        g_nncu_launches++;             \
        CUDA_TRY(cudaGetLastError());  \
    } while (0)

// optional per-launch timing of the tensor-core GEMM (nncu_profile_begin/end)
struct GemmProfiler {
    static const int MAX_EV = 8192;
    cudaEvent_t ev[2 * MAX_EV];
    double flops[MAX_EV];
    int n;
    bool ready;
};
extern GemmProfiler *g_nncu_prof;

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16_rn(x); }
// value after a round trip through the storage type
template <typename T> __device__ __forceinline__ float round_to(float x) { return to_f(from_f<T>(x)); }

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// fixed-order warp reductions (xor butterfly: every lane ends with the same value,
// and the association depends on nothing but the lane count)
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
