// Next-token choice on the device: greedy argmax and temperature sampling, one CTA per row.
//
// The reference chooses greedily, int(logits.argmax()) (mini_hisparse/engine.py:72): the lowest
// index wins a tie.  Temperature sampling is this engine's addition: softmax(logits / T) in
// float32, then the inverse CDF at a uniform number that is a pure function of the request's
// (seed, counter), so a draw does not depend on what else is in the batch:
//   z = splitmix64(seed * 0x9E3779B97F4A7C15 + counter),  u = (z >> 40) / 2^24.
#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
constexpr int THREADS = 1024;

__device__ __forceinline__ float uniform_from_counter(unsigned long long seed,
                                                      unsigned long long counter) {
    unsigned long long z = seed * 0x9E3779B97F4A7C15ull + counter + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long long ld, int V,
              const float* __restrict__ temperature, const long long* __restrict__ seed,
              const long long* __restrict__ counter, int* __restrict__ out) {
    __shared__ float s_val[THREADS];
    __shared__ int s_idx[THREADS];
    __shared__ float s_scan[THREADS + 1];
    __shared__ int s_result;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * ld;
    // contiguous chunk per thread, so that prefix sums follow the index order
    const int chunk = (V + THREADS - 1) / THREADS;
    const int c0 = min(V, tid * chunk), c1 = min(V, c0 + chunk);

    // ---- argmax (lowest index on ties; NaN never wins) ----
    // Consecutive threads read consecutive values (a thread sees its own indices in rising order, so
    // it keeps the first of equal values; the reduction below prefers the lower index on ties).
    float best = -INFINITY;
    int best_i = tid < V ? tid : V - 1;
    for (int i = tid; i < V; i += THREADS) {
        const float v = row[i];
        if (v > best) { best = v; best_i = i; }
    }
    s_val[tid] = best;
    s_idx[tid] = best_i;
    __syncthreads();
    for (int stride = THREADS / 2; stride > 0; stride >>= 1) {
        if (tid < stride) {
            const float ov = s_val[tid + stride];
            const int oi = s_idx[tid + stride];
            if (ov > s_val[tid] || (ov == s_val[tid] && oi < s_idx[tid])) {
                s_val[tid] = ov;
                s_idx[tid] = oi;
            }
        }
        __syncthreads();
    }
    const float row_max = s_val[0];
    const int arg = s_idx[0];
    const float temp = temperature ? temperature[r] : 0.f;
    if (!(temp > 0.f)) {
        if (tid == 0) out[r] = arg;
        return;
    }
    // ---- temperature: inverse CDF over exp((x - max) / T) ----
    const float inv_t = 1.f / temp;
    float sum = 0.f;
    for (int i = c0; i < c1; ++i) sum += expf((row[i] - row_max) * inv_t);
    __syncthreads();
    s_scan[tid + 1] = sum;
    if (tid == 0) { s_scan[0] = 0.f; s_result = arg; }
    __syncthreads();
    if (tid == 0) {  // 1024 additions in index order: exact tiling of [0, total)
        float run = 0.f;
        for (int i = 1; i <= THREADS; ++i) { run += s_scan[i]; s_scan[i] = run; }
    }
    __syncthreads();
    const float total = s_scan[THREADS];
    const float target = uniform_from_counter((unsigned long long)seed[r],
                                              (unsigned long long)counter[r]) * total;
    const float lo = s_scan[tid], hi = s_scan[tid + 1];
    if (c0 < c1 && target >= lo && target < hi) {
        float run = lo;
        int pick = c1 - 1;
        for (int i = c0; i < c1; ++i) {
            run += expf((row[i] - row_max) * inv_t);
            if (run > target) { pick = i; break; }
        }
        s_result = pick;
    }
    __syncthreads();
    if (tid == 0) out[r] = s_result;
}
}  // namespace

// logits [R, V] float32 with row stride ld; temperature/seed/counter per row (temperature may be
// null or <= 0 for greedy); out [R] int32.
MHB_EXPORT int mhb_sample(const float* logits, long long ld, int R, int V, const float* temperature,
                          const long long* seed, const long long* counter, int* out,
                          cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return fail("sample: empty vocabulary");
    launch_kernel(sample_kernel, dim3(R), dim3(THREADS), 0, stream, logits, ld, V, temperature, seed, counter, out);
    return check_launch("sample");
}
