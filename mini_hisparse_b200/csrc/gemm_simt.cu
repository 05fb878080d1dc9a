// C[M,N] = A[M,K] * W[N,K]^T (+ bias) on the CUDA cores with float32 accumulation.
//
// This is the matrix product of the true 32-bit path (plain FFMA: no TF32, no tensor core,
// no reduced-precision intermediate) and the any-shape product of the bfloat16 path for sizes
// the tensor-core kernel refuses.  A and W are row-major with K contiguous, the layout of
// nn.Linear (mini_hisparse/model.py:57-60: y = x W^T + b).
//
// With nsplit > 1 the K range is cut into nsplit parts; part z writes a float32 partial
// matrix at C + z*split_stride and the consumer sums the parts in order.
#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, THREADS = 256;

template <typename AT, typename WT, typename OT>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const AT* __restrict__ A, const WT* __restrict__ W, OT* __restrict__ C,
                 const float* __restrict__ bias, int M, int N, int K, long long lda, long long ldw,
                 long long ldc, int k_per_split, long long split_stride) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int k_begin = blockIdx.z * k_per_split;
    const int k_end = min(K, k_begin + k_per_split);
    const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, 4 x 4 outputs each
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    const int lrow = tid / 4;        // 0..63
    const int lk = (tid % 4) * 4;    // 0,4,8,12
    for (int k0 = k_begin; k0 < k_end; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + j][lrow] = (am < M && k < k_end) ? to_float(A[(size_t)am * lda + k]) : 0.f;
            Ws[lk + j][lrow] = (wn < N && k < k_end) ? to_float(W[(size_t)wn * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
    OT* Cz = C + (size_t)blockIdx.z * split_stride;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias && blockIdx.z == 0) v += bias[n];
            Cz[(size_t)m * ldc + n] = from_float<OT>(v);
        }
    }
}
}  // namespace

MHB_EXPORT int mhb_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C,
                             int c_dtype, const float* bias, int M, int N, int K, long long lda,
                             long long ldw, long long ldc, int nsplit, long long split_stride,
                             cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return fail("gemm: K must be positive");
    if (nsplit < 1) nsplit = 1;
    if (nsplit > 1 && c_dtype != MHB_F32) return fail("gemm: split-K partials must be float32");
    int k_per_split = (K + nsplit - 1) / nsplit;
    k_per_split = (k_per_split + BK - 1) / BK * BK;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, nsplit);
    if (grid.y > 65535) return fail("gemm: M %d too large for one launch", M);
    MHB_DISPATCH_DTYPE(a_dtype, AT, MHB_DISPATCH_DTYPE(w_dtype, WT, MHB_DISPATCH_DTYPE(c_dtype, OT,
        launch_kernel(gemm_simt_kernel<AT, WT, OT>, grid, dim3(THREADS), 0, stream,
            (const AT*)A, (const WT*)W, (OT*)C, bias, M, N, K, lda, ldw, ldc, k_per_split,
            (long long)split_stride))));
    return check_launch("gemm_simt");
}


// ---- the same product for callers that cannot allocate (see gemm_simt_noalloc.h) -----------------
#include <mutex>

#include "gemm_simt_noalloc.h"

namespace {
// Scratch of the no-allocation entry point: nsplit partial matrices of M x N floats.  Every GPU
// that loads this library holds these 8 MiB until the process exits.  In HOST code this name is
// only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_noalloc_scratch[MHB_NOALLOC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_noalloc_ptr[MAX_DEVICES] = {nullptr};
std::mutex g_noalloc_mutex;      // host threads may make their first calls at the same time

// C[m, n] = sum over the splits, in split order
__global__ void sum_partials_kernel(const float* __restrict__ parts, float* __restrict__ C, int M, int N,
                                    long long ldc, int nsplit) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)M * N) return;
    float v = parts[idx];
    for (int s = 1; s < nsplit; ++s) v += parts[(size_t)s * M * N + idx];
    C[(idx / N) * ldc + idx % N] = v;
}

// The device address of the scratch array on the current device; looked up once per device.
int noalloc_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail("gemm_simt_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return fail("gemm_simt_noalloc: device %d is beyond the %d this library tracks", dev, MAX_DEVICES);
    std::lock_guard<std::mutex> guard(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail("gemm_simt_noalloc: cudaGetSymbolAddress on device %d: %s", dev, cudaGetErrorString(e));
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return 0;
}
}  // namespace

MHB_EXPORT int mhb_gemm_simt_noalloc(const void* A, int a_dtype, const void* W, int w_dtype, float* C, int M,
                                     int N, int K, long long lda, long long ldw, long long ldc, int nsplit,
                                     cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return fail("gemm_simt_noalloc: K must be positive");
    if (nsplit < 1) nsplit = 1;
    if (nsplit > 65535) return fail("gemm_simt_noalloc: %d splits; at most 65535 (the grid's third extent)", nsplit);
    if (ldc < N) return fail("gemm_simt_noalloc: the output's row stride %lld is shorter than its %d columns", ldc, N);
    const long long need = (long long)nsplit * M * N;
    if (need > (long long)MHB_NOALLOC_SCRATCH_FLOATS)
        return fail("gemm_simt_noalloc: %d splits of a %d x %d product need %lld floats of scratch; the built-in "
                    "array holds %d (use fewer splits, or mhb_gemm_simt with a buffer of your own)",
                    nsplit, M, N, need, (int)MHB_NOALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    int rc = noalloc_scratch(&scratch);
    if (rc) return rc;
    // every partial element is written by the product below before the sum reads it
    rc = mhb_gemm_simt(A, a_dtype, W, w_dtype, scratch, MHB_F32, nullptr, M, N, K, lda, ldw, N, nsplit,
                       (long long)M * N, stream);
    if (rc) return rc;
    const size_t total = (size_t)M * N;
    const int threads = 256;
    launch_kernel(sum_partials_kernel, dim3((unsigned)((total + threads - 1) / threads)), dim3(threads), 0, stream,
                  (const float*)scratch, C, M, N, ldc, nsplit);
    return check_launch("gemm_simt_noalloc");
}
