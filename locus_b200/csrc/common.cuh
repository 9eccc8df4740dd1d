// Shared helpers of the sm_100a kernels: element types, conversions, launch checks.
//
// Element type codes used across the C entry points:
//   0 = float32, 1 = bfloat16.
// Every entry point is `extern "C"`, takes raw device pointers plus sizes and the
// stream to launch on, allocates nothing, and returns a cudaError_t as int
// (0 = success).  Arguments that a kernel cannot handle are refused with
// LOCUS_ERR_UNSUPPORTED before anything is launched, never run with a wrong result.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LOCUS_DT_F32 0
#define LOCUS_DT_BF16 1

// Returned (as int) when sizes or type combinations are outside what the kernel takes.
#define LOCUS_ERR_UNSUPPORTED 10001

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

// Load element i of an array whose element type is only known at run time.
__device__ __forceinline__ float ld_dyn(const void* p, int dt, size_t i) {
    return dt == LOCUS_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                              : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}

__device__ __forceinline__ void st_dyn(void* p, int dt, size_t i, float v) {
    if (dt == LOCUS_DT_F32) {
        reinterpret_cast<float*>(p)[i] = v;
    } else {
        reinterpret_cast<bf16*>(p)[i] = __float2bfloat16_rn(v);
    }
}

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

static inline int locus_launch_status() { return static_cast<int>(cudaGetLastError()); }

// Programmatic dependent launch.  A kernel launched with the attribute may be scheduled before the
// kernel in front of it in the stream has drained; its blocks wait in pdl_entry() until that grid has
// finished and its writes are visible.  Kernels signal late (pdl_trigger() below): a signal at the
// start of a grid of many waves let waiting blocks take SM slots from the running kernel and measured
// slower.  What is saved is launch processing between the many short kernels of a decode step.  Launches go through locus_launch();
// the attribute is only set while the module's switch is on (locus_set_pdl), otherwise the wait is
// a no-op and the launch an ordinary one.
static int g_locus_pdl = 0;
extern "C" void locus_set_pdl(int on) { g_locus_pdl = on; }

__device__ __forceinline__ void pdl_entry() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Lets the next kernel of the stream be scheduled once every block of this grid has passed this point
// (or finished).  The next kernel still waits in its pdl_entry() until this grid is complete, so only
// its launch and block start-up move under this grid's tail.  Place it where the block has no more
// blocks of its own grid waiting for a slot behind it: at the start of a grid of one wave, after the
// main loop of a grid of many.
__device__ __forceinline__ void pdl_trigger() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static inline void locus_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_locus_pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
