// Memory-bound kernels of the step: embedding gather, (residual add +) RMSNorm, rotary
// position encoding fused with the paged KV append, and the SwiGLU gate.
//
// The residual stream is float32 in every mode; normalisation, rotation angles and the
// residual sum are computed in float32 (the reference computes its norm in float32,
// mini_hisparse/model.py:49-51, and its angles in float32, model.py:141-147).
//
// Inputs that come from a split-K matrix product arrive as `nsplit` float32 partial
// matrices `split_stride` elements apart; they are summed here in a fixed order, so the
// result does not depend on timing.
#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

// ---- load helpers -----------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float load_split(const T* p, size_t idx, int nsplit, size_t split_stride) {
    float v = to_float(p[idx]);
    for (int s = 1; s < nsplit; ++s) v += to_float(p[idx + (size_t)s * split_stride]);
    return v;
}

// ---- embedding ---------------------------------------------------------------------------
// out[t, :] = table[tokens[t], :]   (mini_hisparse/model.py:166: plain lookup, no scaling)
template <typename WT>
__global__ void embed_kernel(const WT* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int H, int V, int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* o = out + (size_t)t * H;
    if (tok < 0 || tok >= V) {  // the host validates ids; never read outside the table
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        if (threadIdx.x == 0 && status) atomicOr(status, 1);
        return;
    }
    const WT* row = table + (size_t)tok * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]);
}

MHB_EXPORT int mhb_embed(const void* table, int table_dtype, const int* tokens, float* out, int T,
                         int H, int V, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    MHB_DISPATCH_DTYPE(table_dtype, WT,
        launch_kernel(embed_kernel<WT>, dim3(T), dim3(threads), 0, stream, (const WT*)table, tokens, out, H, V, status));
    return check_launch("embed");
}

// ---- (add +) RMSNorm -----------------------------------------------------------------------
// For output row r (source row s = rows ? rows[r] : r):
//   v = x[s] (+ delta[s]);  if delta and !rows: x[s] = v  (residual updated in place)
//   out[r] = (v * rsqrt(mean(v^2) + eps)) * weight        (mini_hisparse/model.py:49-51)
template <typename DT, typename OT>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const DT* __restrict__ delta, int nsplit,
                                   size_t split_stride, const float* __restrict__ weight,
                                   float eps, const int* __restrict__ rows, OT* __restrict__ out,
                                   int H) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* xr = x + (size_t)s * H;
    const bool write_back = (delta != nullptr) && (rows == nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (delta) {
            v += load_split(delta, (size_t)s * H + i, nsplit, split_stride);
            if (write_back) xr[i] = v;
        }
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float rstd = rsqrtf(total / (float)H + eps);
    OT* o = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (delta && !write_back) v += load_split(delta, (size_t)s * H + i, nsplit, split_stride);
        const float n = v * rstd;
        o[i] = from_float<OT>(n * weight[i]);
    }
}

// The same with 4 elements per thread and the row kept in registers between the two passes
// (rows of up to 4 * VEC_CACHE * blockDim elements; H % 4 == 0, 16-byte aligned rows).
constexpr int VEC_CACHE = 4;

template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *(const float4*)p; }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 u = *(const uint2*)p;
    const __nv_bfloat162 a = *(const __nv_bfloat162*)&u.x, b = *(const __nv_bfloat162*)&u.y;
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *(float4*)p = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *(const uint32_t*)&a;
    u.y = *(const uint32_t*)&b;
    *(uint2*)p = u;
}

// VC vectors per thread: 4 for many rows; 1 for few rows (a decode step), where the kernel's time is
// the chain of memory round trips of one thread and more threads make that chain shorter.
template <typename DT, typename OT, int VC>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ x, const DT* __restrict__ delta, int nsplit,
                                       size_t split_stride, const float* __restrict__ weight, float eps,
                                       const int* __restrict__ rows, OT* __restrict__ out, int H) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    const int nvec = H >> 2;
    // few rows: the weights (constant) are fetched while the kernel before this one still runs; with
    // many rows the registers are worth more
    float4 wv = make_float4(0.f, 0.f, 0.f, 0.f);
    if constexpr (VC == 1) {
        if ((int)threadIdx.x < nvec) wv = *(const float4*)(weight + 4 * threadIdx.x);
    }
    pdl_wait();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* xr = x + (size_t)s * H;
    const bool write_back = (delta != nullptr) && (rows == nullptr);
    float4 v[VC];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < VC; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            float4 a = *(const float4*)(xr + 4 * i);
            if (delta) {
                const DT* dp = delta + (size_t)s * H + 4 * i;
                int sp = 0;
                for (; sp + 8 <= nsplit; sp += 8) {      // eight loads in flight; summed in order
                    float4 d[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) d[q] = load4<DT>(dp + (size_t)(sp + q) * split_stride);
#pragma unroll
                    for (int q = 0; q < 8; ++q) { a.x += d[q].x; a.y += d[q].y; a.z += d[q].z; a.w += d[q].w; }
                }
                for (; sp + 4 <= nsplit; sp += 4) {      // four loads in flight; summed in order
                    const float4 d0 = load4<DT>(dp + (size_t)(sp + 0) * split_stride);
                    const float4 d1 = load4<DT>(dp + (size_t)(sp + 1) * split_stride);
                    const float4 d2 = load4<DT>(dp + (size_t)(sp + 2) * split_stride);
                    const float4 d3 = load4<DT>(dp + (size_t)(sp + 3) * split_stride);
                    a.x += d0.x; a.y += d0.y; a.z += d0.z; a.w += d0.w;
                    a.x += d1.x; a.y += d1.y; a.z += d1.z; a.w += d1.w;
                    a.x += d2.x; a.y += d2.y; a.z += d2.z; a.w += d2.w;
                    a.x += d3.x; a.y += d3.y; a.z += d3.z; a.w += d3.w;
                }
                for (; sp < nsplit; ++sp) {
                    const float4 d = load4<DT>(dp + (size_t)sp * split_stride);
                    a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
                }
                if (write_back) *(float4*)(xr + 4 * i) = a;
            }
            v[c] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    const float total = block_sum(ss, scratch);
    const float rstd = rsqrtf(total / (float)H + eps);
    OT* o = out + (size_t)r * H;
#pragma unroll
    for (int c = 0; c < VC; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            const float4 w = VC == 1 ? wv : *(const float4*)(weight + 4 * i);
            float4 a = v[c];
            a.x = (a.x * rstd) * w.x; a.y = (a.y * rstd) * w.y;
            a.z = (a.z * rstd) * w.z; a.w = (a.w * rstd) * w.w;
            store4<OT>(o + 4 * i, a);
        }
    }
}

// Residual add alone (the last feed-forward's output when no norm follows on all rows).
template <typename DT>
__global__ void residual_add_kernel(float* __restrict__ x, const DT* __restrict__ delta, int nsplit,
                                    size_t split_stride, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += load_split(delta, i, nsplit, split_stride);
}

MHB_EXPORT int mhb_add_rmsnorm(float* x, const void* delta, int delta_dtype, int nsplit,
                               long long split_stride, const float* weight, float eps,
                               const int* rows, void* out, int out_dtype, int R, int H,
                               cudaStream_t stream) {
    if (R <= 0) return 0;
    if (nsplit > 1 && delta_dtype != MHB_F32) return fail("add_rmsnorm: split partials must be float32");
    const bool aligned = H % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)weight & 15) == 0 &&
                         ((uintptr_t)out & 15) == 0 && ((uintptr_t)delta & 15) == 0 && split_stride % 4 == 0;
    int vthreads = ((H / 4 + VEC_CACHE - 1) / VEC_CACHE + 31) / 32 * 32;
    if (vthreads < 64) vthreads = 64;
    const int wide = (H / 4 + 31) / 32 * 32;          // threads when each takes one vector
    if (aligned && R <= 128 && wide <= 1024 && wide >= 64) {
        MHB_DISPATCH_DTYPE(delta_dtype, DT, MHB_DISPATCH_DTYPE(out_dtype, OT,
            launch_kernel((add_rmsnorm_vec_kernel<DT, OT, 1>), dim3(R), dim3(wide), 0, stream,
                x, (const DT*)delta, nsplit, (size_t)split_stride, weight, eps, rows, (OT*)out, H)));
        return check_launch("add_rmsnorm");
    }
    if (aligned && vthreads <= 1024) {
        MHB_DISPATCH_DTYPE(delta_dtype, DT, MHB_DISPATCH_DTYPE(out_dtype, OT,
            launch_kernel((add_rmsnorm_vec_kernel<DT, OT, VEC_CACHE>), dim3(R), dim3(vthreads), 0, stream,
                x, (const DT*)delta, nsplit, (size_t)split_stride, weight, eps, rows, (OT*)out, H)));
        return check_launch("add_rmsnorm");
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    MHB_DISPATCH_DTYPE(delta_dtype, DT, MHB_DISPATCH_DTYPE(out_dtype, OT,
        launch_kernel(add_rmsnorm_kernel<DT, OT>, dim3(R), dim3(threads), 0, stream, 
            x, (const DT*)delta, nsplit, (size_t)split_stride, weight, eps, rows, (OT*)out, H)));
    return check_launch("add_rmsnorm");
}

MHB_EXPORT int mhb_residual_add(float* x, const void* delta, int delta_dtype, int nsplit,
                                long long split_stride, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (nsplit > 1 && delta_dtype != MHB_F32) return fail("residual_add: split partials must be float32");
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    MHB_DISPATCH_DTYPE(delta_dtype, DT,
        launch_kernel(residual_add_kernel<DT>, dim3(blocks), dim3(threads), 0, stream, x, (const DT*)delta, nsplit,
                                                                 (size_t)split_stride, (size_t)n));
    return check_launch("residual_add");
}

// ---- rotary positions + paged KV append -----------------------------------------------------
// qkv[t] = [q heads | k heads | v heads], each head `d` wide, plus an optional float32 bias.
// q and k are rotated by the half-split rule of mini_hisparse/model.py:141-151:
//   angle = float(position) * inv_freq[i],  out[j] = t[j]*cos + (j < d/2 ? -t[j+d/2] : t[j-d/2])*sin
// Rotated q goes to q_out [T, nq*d]; rotated k and plain v go into the cache page of the
// token's position (the append happens before attention, model.py:169-170, 201):
//   cache[page][0 or 1][kv head][position % P][d],  page = block_table[seg][position / P].
// With write_kv == 0 nothing is appended (a layer that reads another layer's cache).
template <typename IT, typename QT, typename CT>
__global__ void rope_append_kernel(const IT* __restrict__ qkv, int nsplit, size_t split_stride,
                                   const float* __restrict__ bias, const int* __restrict__ positions,
                                   const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                                   int table_width, const float* __restrict__ inv_freq,
                                   QT* __restrict__ q_out, CT* __restrict__ cache, int nq, int nkv,
                                   int d, int P, int num_pages, int write_kv, int rotate_q_k,
                                   int heads_per_block, int* __restrict__ status) {
    extern __shared__ float cs_table[];      // cos[d/2], sin[d/2] of this token's position
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = d >> 1;
    const int width = (nq + 2 * nkv) * d;
    const size_t base = (size_t)t * width;
    // heads are numbered q heads, then k heads, then v heads; this block takes a run of them
    const int head_begin = blockIdx.y * heads_per_block;
    const int head_end = min(nq + 2 * nkv, head_begin + heads_per_block);
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn = 0.f, cs = 1.f;
        if (rotate_q_k) sincosf((float)pos * inv_freq[i], &sn, &cs);
        cs_table[i] = cs;
        cs_table[half + i] = sn;
    }
    int page = -1;
    if (write_kv && head_end > nq) {
        page = block_table[(size_t)tok_seg[t] * table_width + pos / P];
        if (page < 0 || page >= num_pages) {  // never write outside the pool
            if (threadIdx.x == 0 && status) atomicOr(status, 2);
            page = -1;
        }
    }
    const int within = pos % P;
    __syncthreads();
    // q and k heads: one thread per (head, i < d/2) pair
    const int rot_end = min(head_end, nq + nkv);
    for (int idx = head_begin * half + threadIdx.x; idx < rot_end * half; idx += blockDim.x) {
        const int head = idx / half, i = idx - head * half;
        const int col = head * d + i;
        float a = load_split(qkv, base + col, nsplit, split_stride);
        float b = load_split(qkv, base + col + half, nsplit, split_stride);
        if (bias) { a += bias[col]; b += bias[col + half]; }
        const float cs = cs_table[i], sn = cs_table[half + i];
        const float oa = a * cs - b * sn;
        const float ob = b * cs + a * sn;
        if (head < nq) {
            q_out[(size_t)t * nq * d + col] = from_float<QT>(oa);
            q_out[(size_t)t * nq * d + col + half] = from_float<QT>(ob);
        } else if (page >= 0) {
            const int kh = head - nq;
            CT* dst = cache + ((((size_t)page * 2 + 0) * nkv + kh) * P + within) * d;
            dst[i] = from_float<CT>(oa);
            dst[i + half] = from_float<CT>(ob);
        }
    }
    if (page >= 0) {
        const int v_begin = max(head_begin, nq + nkv);
        for (int idx = v_begin * d + threadIdx.x; idx < head_end * d; idx += blockDim.x) {
            const int kh = idx / d - (nq + nkv), e = idx % d;
            float v = load_split(qkv, base + idx, nsplit, split_stride);
            if (bias) v += bias[idx];
            cache[((((size_t)page * 2 + 1) * nkv + kh) * P + within) * d + e] = from_float<CT>(v);
        }
    }
}

// The same with four elements per thread (head sizes are multiples of 8 and every row, bias and
// cache row is 16-byte aligned then): 16-byte loads, 8- or 16-byte stores.
template <typename IT>
__device__ __forceinline__ float4 load4_split(const IT* p, size_t idx, int nsplit, size_t split_stride) {
    float4 v = load4<IT>(p + idx);
    int s = 1;
    for (; s + 4 <= nsplit; s += 4) {       // four loads in flight; summed in order
        float4 w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) w[q] = load4<IT>(p + idx + (size_t)(s + q) * split_stride);
#pragma unroll
        for (int q = 0; q < 4; ++q) { v.x += w[q].x; v.y += w[q].y; v.z += w[q].z; v.w += w[q].w; }
    }
    for (; s < nsplit; ++s) {
        const float4 w = load4<IT>(p + idx + (size_t)s * split_stride);
        v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
    }
    return v;
}

template <typename IT, typename QT, typename CT>
__global__ void rope_append_vec_kernel(const IT* __restrict__ qkv, int nsplit, size_t split_stride,
                                       const float* __restrict__ bias, const int* __restrict__ positions,
                                       const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                                       int table_width, const float* __restrict__ inv_freq,
                                       QT* __restrict__ q_out, CT* __restrict__ cache, int nq, int nkv,
                                       int d, int P, int num_pages, int write_kv, int rotate_q_k,
                                       int heads_per_block, int* __restrict__ status) {
    extern __shared__ __align__(16) float cs_table[];      // cos[d/2], sin[d/2] of this token's position
    // positions, segments and the block table were copied in before the step's first kernel: the
    // rotation table and the page are worked out while the kernel before this one still runs
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = d >> 1, quarter = d >> 3;             // quarter: groups of 4 in a half
    const int width = (nq + 2 * nkv) * d;
    const size_t base = (size_t)t * width;
    const int head_begin = blockIdx.y * heads_per_block;
    const int head_end = min(nq + 2 * nkv, head_begin + heads_per_block);
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn = 0.f, cs = 1.f;
        if (rotate_q_k) sincosf((float)pos * inv_freq[i], &sn, &cs);
        cs_table[i] = cs;
        cs_table[half + i] = sn;
    }
    int page = -1;
    if (write_kv && head_end > nq) {
        page = block_table[(size_t)tok_seg[t] * table_width + pos / P];
        if (page < 0 || page >= num_pages) {  // never write outside the pool
            if (threadIdx.x == 0 && status) atomicOr(status, 2);
            page = -1;
        }
    }
    const int within = pos % P;
    __syncthreads();
    pdl_wait();
    const int rot_end = min(head_end, nq + nkv);
    for (int idx = head_begin * quarter + threadIdx.x; idx < rot_end * quarter; idx += blockDim.x) {
        const int head = idx / quarter, i = (idx - head * quarter) * 4;
        const int col = head * d + i;
        float4 a = load4_split(qkv, base + col, nsplit, split_stride);
        float4 b = load4_split(qkv, base + col + half, nsplit, split_stride);
        if (bias) {
            const float4 ba = *(const float4*)(bias + col), bb = *(const float4*)(bias + col + half);
            a.x += ba.x; a.y += ba.y; a.z += ba.z; a.w += ba.w;
            b.x += bb.x; b.y += bb.y; b.z += bb.z; b.w += bb.w;
        }
        const float4 cs = *(const float4*)(cs_table + i), sn = *(const float4*)(cs_table + half + i);
        const float4 oa = make_float4(a.x * cs.x - b.x * sn.x, a.y * cs.y - b.y * sn.y, a.z * cs.z - b.z * sn.z,
                                      a.w * cs.w - b.w * sn.w);
        const float4 ob = make_float4(b.x * cs.x + a.x * sn.x, b.y * cs.y + a.y * sn.y, b.z * cs.z + a.z * sn.z,
                                      b.w * cs.w + a.w * sn.w);
        if (head < nq) {
            store4<QT>(q_out + (size_t)t * nq * d + col, oa);
            store4<QT>(q_out + (size_t)t * nq * d + col + half, ob);
        } else if (page >= 0) {
            CT* dst = cache + ((((size_t)page * 2 + 0) * nkv + (head - nq)) * P + within) * d;
            store4<CT>(dst + i, oa);
            store4<CT>(dst + i + half, ob);
        }
    }
    if (page >= 0) {
        const int v_begin = max(head_begin, nq + nkv);
        const int dq = d >> 2;
        for (int idx = v_begin * dq + threadIdx.x; idx < head_end * dq; idx += blockDim.x) {
            const int head = idx / dq, e = (idx - head * dq) * 4;
            float4 v = load4_split(qkv, base + (size_t)head * d + e, nsplit, split_stride);
            if (bias) {
                const float4 bv = *(const float4*)(bias + head * d + e);
                v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
            }
            store4<CT>(cache + ((((size_t)page * 2 + 1) * nkv + (head - nq - nkv)) * P + within) * d + e, v);
        }
    }
}

MHB_EXPORT int mhb_rope_append(const void* qkv, int in_dtype, int nsplit, long long split_stride,
                               const float* bias, const int* positions, const int* tok_seg,
                               const int* block_table, int table_width, const float* inv_freq,
                               void* q_out, void* cache, int act_dtype, int T, int nq, int nkv,
                               int d, int P, int num_pages, int write_kv, int rotate,
                               int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d % 2) return fail("rope_append: head_dim %d must be even", d);
    if (nsplit > 1 && in_dtype != MHB_F32) return fail("rope_append: split partials must be float32");
    const int threads = 128;
    // few tokens: spread the heads of a token over several blocks so that the GPU is not idle
    const int heads = nq + 2 * nkv;
    int blocks_y = T >= 512 ? 1 : (512 + T - 1) / T;
    if (blocks_y > heads) blocks_y = heads;
    const int hpb = (heads + blocks_y - 1) / blocks_y;
    blocks_y = (heads + hpb - 1) / hpb;
    dim3 grid(T, blocks_y);
    const size_t smem = sizeof(float) * d;
    const bool aligned = d % 8 == 0 && split_stride % 4 == 0 && (((uintptr_t)qkv | (uintptr_t)bias | (uintptr_t)q_out |
                                                                  (uintptr_t)cache) & 15) == 0;
    if (aligned) {
        MHB_DISPATCH_DTYPE(in_dtype, IT, MHB_DISPATCH_DTYPE(act_dtype, AT,
            launch_kernel(rope_append_vec_kernel<IT, AT, AT>, dim3(grid), dim3(threads), smem, stream,
                (const IT*)qkv, nsplit, (size_t)split_stride, bias, positions, tok_seg, block_table,
                table_width, inv_freq, (AT*)q_out, (AT*)cache, nq, nkv, d, P, num_pages, write_kv,
                rotate, hpb, status)));
        return check_launch("rope_append");
    }
    MHB_DISPATCH_DTYPE(in_dtype, IT, MHB_DISPATCH_DTYPE(act_dtype, AT,
        launch_kernel(rope_append_kernel<IT, AT, AT>, dim3(grid), dim3(threads), smem, stream, 
            (const IT*)qkv, nsplit, (size_t)split_stride, bias, positions, tok_seg, block_table,
            table_width, inv_freq, (AT*)q_out, (AT*)cache, nq, nkv, d, P, num_pages, write_kv,
            rotate, hpb, status)));
    return check_launch("rope_append");
}

// cos and sin of every token's rotation angles, [T, d]: cos[d/2] then sin[d/2]; once per step for
// all layers (the matrix product's q/k/v epilogue reads it).  Float32 angles as in rope_append.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ table, int T, int half, int rotate) {
    pdl_launch_dependents();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, i = idx - t * half;
    float sn = 0.f, cs = 1.f;
    if (rotate) sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
    table[(size_t)t * 2 * half + i] = cs;
    table[(size_t)t * 2 * half + half + i] = sn;
}

MHB_EXPORT int mhb_rope_table(const int* positions, const float* inv_freq, float* table, int T, int d, int rotate,
                              cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d % 2) return fail("rope_table: head_dim %d must be even", d);
    const int half = d / 2, threads = 256;
    launch_kernel(rope_table_kernel, dim3((T * half + threads - 1) / threads), dim3(threads), 0, stream, positions,
                  inv_freq, table, T, half, rotate);
    return check_launch("rope_table");
}

// ---- SwiGLU gate ------------------------------------------------------------------------------
// out[t, i] = silu(gate_i) * up_i   (mini_hisparse/model.py:70-71).  gu[t] holds 2 I values in
// blocks: `block` gate values, then the `block` up values of the same indices (block = I is the
// plain [gate | up] layout).
template <typename IT, typename OT>
__global__ void swiglu_kernel(const IT* __restrict__ gu, int nsplit, size_t split_stride,
                              OT* __restrict__ out, int I, int block, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const int gcol = (i / block) * 2 * block + i % block;
    const float g = load_split(gu, t * 2 * I + gcol, nsplit, split_stride);
    const float u = load_split(gu, t * 2 * I + gcol + block, nsplit, split_stride);
    const float s = g / (1.f + expf(-g));
    out[idx] = from_float<OT>(s * u);
}

MHB_EXPORT int mhb_swiglu(const void* gu, int in_dtype, int nsplit, long long split_stride,
                          void* out, int out_dtype, int T, int I, int block, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (block <= 0 || I % block) return fail("swiglu: block %d does not divide %d", block, I);
    if (nsplit > 1 && in_dtype != MHB_F32) return fail("swiglu: split partials must be float32");
    const size_t total = (size_t)T * I;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    MHB_DISPATCH_DTYPE(in_dtype, IT, MHB_DISPATCH_DTYPE(out_dtype, OT,
        launch_kernel(swiglu_kernel<IT, OT>, dim3(blocks), dim3(threads), 0, stream, (const IT*)gu, nsplit,
                                                            (size_t)split_stride, (OT*)out, I, block, total)));
    return check_launch("swiglu");
}
