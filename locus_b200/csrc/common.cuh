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

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
