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
#include <stdlib.h>

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

// ---- programmatic dependent launch -----------------------------------------------------------
// Every kernel of the step is launched with the programmatic-stream-serialization attribute and
// begins with pdl_launch_dependents(); pdl_wait().  The first lets the NEXT kernel's CTAs start as
// soon as SM resources allow (its start-up, and in the matrix products the first weight tiles,
// overlap this kernel's tail); the second holds this kernel until its predecessor has completed
// and its writes are visible.  Before pdl_wait() a kernel touches constant data only (weights,
// tensor maps).  Since every kernel waits for its predecessor, completion stays in stream order.
// MHB_PDL=0 in the environment switches the attribute off (then both calls are no-ops).
namespace mhb {
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("MHB_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
}  // namespace mhb

// Dispatch on a runtime dtype code: CALL is a statement that uses the type name T.
#define MHB_DISPATCH_DTYPE(code, T, ...)                                         \
    do {                                                                         \
        if ((code) == MHB_F32) { using T = float; __VA_ARGS__; }                 \
        else if ((code) == MHB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }   \
        else return mhb::fail("unknown dtype code %d", (int)(code));             \
    } while (0)
