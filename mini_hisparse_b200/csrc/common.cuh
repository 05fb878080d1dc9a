// Shared helpers of the sm_100a kernels: scalar types, conversions, reductions and the
// error channel of the C entry points.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and a stream, launches
// on that stream and returns 0 or a negative code; mhb_last_error() gives the text.  Nothing
// here allocates device memory: the caller owns inputs, outputs and scratch.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#define MHB_EXPORT extern "C" __attribute__((visibility("default")))

enum MhbDtype : int { MHB_F32 = 0, MHB_BF16 = 1 };

namespace mhb {

// ---- error text -----------------------------------------------------------
inline char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}
inline int fail(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
}  // namespace mhb
#include <stdarg.h>
namespace mhb {
inline int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return -1;
}
inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("%s: %s", what, cudaGetErrorString(e));
    return 0;
}

// ---- scalar conversions ------------------------------------------------------
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// ---- reductions -----------------------------------------------------------------
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
// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace mhb

// Dispatch on a runtime dtype code: CALL is a statement that uses the type name T.
#define MHB_DISPATCH_DTYPE(code, T, ...)                                         \
    do {                                                                         \
        if ((code) == MHB_F32) { using T = float; __VA_ARGS__; }                 \
        else if ((code) == MHB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }   \
        else return mhb::fail("unknown dtype code %d", (int)(code));             \
    } while (0)
