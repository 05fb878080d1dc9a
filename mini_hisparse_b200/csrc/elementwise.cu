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

// Many rows (a prompt portion), every row in place, one matrix of deltas: a CTA walks rows
// blockIdx.x, blockIdx.x + gridDim.x, ... and asks for the next row before it reduces and stores
// the current one.  With a CTA per row the GPU's CTAs all load, then all reduce, then all store,
// wave after wave; walking keeps loads and stores of different rows in flight together (2,048 rows
// of 3,584 without a delta, caches cold: 18.3 -> 16.4 us; with a bfloat16 delta 20.5 us; the registers
// of two rows leave three CTAs per SM, which is what limits it now).
template <typename DT, typename OT>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(float* __restrict__ x, const DT* __restrict__ delta, const float* __restrict__ weight,
                        float eps, OT* __restrict__ out, int R, int H) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    const int nvec = H >> 2;
    pdl_wait();
    float4 cur[VEC_CACHE], dcur[VEC_CACHE], nxt[VEC_CACHE], dnxt[VEC_CACHE];
    auto fetch = [&](int r, float4 (&a)[VEC_CACHE], float4 (&d)[VEC_CACHE]) {
#pragma unroll
        for (int c = 0; c < VEC_CACHE; ++c) {
            const int i = threadIdx.x + c * blockDim.x;
            if (i < nvec) {
                a[c] = *(const float4*)(x + (size_t)r * H + 4 * i);
                d[c] = delta ? load4<DT>(delta + (size_t)r * H + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    };
    int r = blockIdx.x;
    if (r < R) fetch(r, cur, dcur);
    for (; r < R; r += gridDim.x) {
        const int rn = r + gridDim.x;
        if (rn < R) fetch(rn, nxt, dnxt);
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < VEC_CACHE; ++c) {
            const int i = threadIdx.x + c * blockDim.x;
            if (i < nvec) {
                float4 a = cur[c];
                a.x += dcur[c].x; a.y += dcur[c].y; a.z += dcur[c].z; a.w += dcur[c].w;
                if (delta) *(float4*)(x + (size_t)r * H + 4 * i) = a;
                cur[c] = a;
                ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            }
        }
        const float total = block_sum(ss, scratch);
        const float rstd = rsqrtf(total / (float)H + eps);
#pragma unroll
        for (int c = 0; c < VEC_CACHE; ++c) {
            const int i = threadIdx.x + c * blockDim.x;
            if (i < nvec) {
                const float4 w = *(const float4*)(weight + 4 * i);
                float4 a = cur[c];
                a.x = (a.x * rstd) * w.x; a.y = (a.y * rstd) * w.y;
                a.z = (a.z * rstd) * w.z; a.w = (a.w * rstd) * w.w;
                store4<OT>(out + (size_t)r * H + 4 * i, a);
            }
        }
#pragma unroll
        for (int c = 0; c < VEC_CACHE; ++c) { cur[c] = nxt[c]; dcur[c] = dnxt[c]; }
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
    if (aligned && vthreads <= 256 && R >= 512 && rows == nullptr && nsplit == 1) {
        // a prompt portion: a few CTAs per SM walk the rows
        static int sms = 0;
        if (!sms) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (sms <= 0) sms = 148;
        }
        MHB_DISPATCH_DTYPE(delta_dtype, DT, MHB_DISPATCH_DTYPE(out_dtype, OT, {
            int per_sm = 0;       // as many CTAs as are resident at once
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, add_rmsnorm_rows_kernel<DT, OT>, vthreads, 0) !=
                    cudaSuccess || per_sm < 1)
                per_sm = 2;
            const int grid = R < per_sm * sms ? R : per_sm * sms;
            launch_kernel((add_rmsnorm_rows_kernel<DT, OT>), dim3(grid), dim3(vthreads), 0, stream,
                x, (const DT*)delta, weight, eps, (OT*)out, R, H);
        }));
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
// The first `rdim` elements of every q and k head are rotated, the rest pass unchanged; v is never
// rotated.  angle_i = float(position) * inv_freq[i], i < rdim / 2, and the pair that angle i turns is
//   half-split (mini_hisparse/model.py:141-151, "rotate_half"):  (i, i + rdim/2)
//   interleaved:                                                  (2 i, 2 i + 1)
// with (a, b) -> (a cos - b sin, b cos + a sin).  The reference has the half-split rule over the
// whole head only (rdim = d); the other two are parameters of the position part.
// Rotated q goes to q_out [T, nq*d]; rotated k and plain v go into the cache page of the
// token's position (the append happens before attention, model.py:169-170, 201):
//   cache[page][0 or 1][kv head][position % P][d],  page = block_table[seg][position / P].
// With write_kv == 0 nothing is appended (a layer that reads another layer's cache).
struct RopeStyle {
    int rdim;          // rotated elements per head: even, <= d; 0 = no rotation
    int interleaved;   // 0: pairs (i, i + rdim/2); 1: pairs (2 i, 2 i + 1)
};

template <typename IT, typename QT, typename CT>
__global__ void rope_append_kernel(const IT* __restrict__ qkv, int nsplit, size_t split_stride,
                                   const float* __restrict__ bias, const int* __restrict__ positions,
                                   const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                                   int table_width, const float* __restrict__ inv_freq,
                                   QT* __restrict__ q_out, CT* __restrict__ cache, int nq, int nkv,
                                   int d, int P, int num_pages, int write_kv, RopeStyle style,
                                   int heads_per_block, int* __restrict__ status) {
    extern __shared__ float cs_table[];      // cos[rdim/2], sin[rdim/2] of this token's position
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int rhalf = style.rdim >> 1;
    const int width = (nq + 2 * nkv) * d;
    const size_t base = (size_t)t * width;
    // heads are numbered q heads, then k heads, then v heads; this block takes a run of them
    const int head_begin = blockIdx.y * heads_per_block;
    const int head_end = min(nq + 2 * nkv, head_begin + heads_per_block);
    for (int i = threadIdx.x; i < rhalf; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        cs_table[i] = cs;
        cs_table[rhalf + i] = sn;
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
    // q and k heads: one thread per unit; a head has rdim/2 rotated pairs and d - rdim plain elements
    const int rot_end = min(head_end, nq + nkv);
    const int units = rhalf + (d - style.rdim);
    for (int idx = head_begin * units + threadIdx.x; idx < rot_end * units; idx += blockDim.x) {
        const int head = idx / units, u = idx - head * units;
        QT* qdst = head < nq ? q_out + (size_t)t * nq * d + head * d : nullptr;
        CT* kdst = (head >= nq && page >= 0) ? cache + ((((size_t)page * 2 + 0) * nkv + (head - nq)) * P + within) * d : nullptr;
        if (u < rhalf) {
            const int ea = style.interleaved ? 2 * u : u, eb = style.interleaved ? 2 * u + 1 : u + rhalf;
            float a = load_split(qkv, base + head * d + ea, nsplit, split_stride);
            float b = load_split(qkv, base + head * d + eb, nsplit, split_stride);
            if (bias) { a += bias[head * d + ea]; b += bias[head * d + eb]; }
            const float cs = cs_table[u], sn = cs_table[rhalf + u];
            const float oa = a * cs - b * sn;
            const float ob = b * cs + a * sn;
            if (qdst) { qdst[ea] = from_float<QT>(oa); qdst[eb] = from_float<QT>(ob); }
            else if (kdst) { kdst[ea] = from_float<CT>(oa); kdst[eb] = from_float<CT>(ob); }
        } else {
            const int e = style.rdim + (u - rhalf);
            float a = load_split(qkv, base + head * d + e, nsplit, split_stride);
            if (bias) a += bias[head * d + e];
            if (qdst) qdst[e] = from_float<QT>(a);
            else if (kdst) kdst[e] = from_float<CT>(a);
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

// The same with four elements per thread (head size and rotated width are multiples of 8 and every
// row, bias and cache row is 16-byte aligned then): 16-byte loads, 8- or 16-byte stores.
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
__device__ __forceinline__ void add4(float4& a, const float4 b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }

template <typename IT, typename QT, typename CT>
__global__ void rope_append_vec_kernel(const IT* __restrict__ qkv, int nsplit, size_t split_stride,
                                       const float* __restrict__ bias, const int* __restrict__ positions,
                                       const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                                       int table_width, const float* __restrict__ inv_freq,
                                       QT* __restrict__ q_out, CT* __restrict__ cache, int nq, int nkv,
                                       int d, int P, int num_pages, int write_kv, RopeStyle style,
                                       int heads_per_block, int* __restrict__ status) {
    extern __shared__ __align__(16) float cs_table[];      // cos[rdim/2], sin[rdim/2] of this token's position
    // positions, segments and the block table were copied in before the step's first kernel: the
    // rotation table and the page are worked out while the kernel before this one still runs
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int rhalf = style.rdim >> 1;
    const int width = (nq + 2 * nkv) * d;
    const size_t base = (size_t)t * width;
    const int head_begin = blockIdx.y * heads_per_block;
    const int head_end = min(nq + 2 * nkv, head_begin + heads_per_block);
    for (int i = threadIdx.x; i < rhalf; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        cs_table[i] = cs;
        cs_table[rhalf + i] = sn;
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
    // q and k heads: a unit is four angles (eight rotated elements) or four plain elements
    const int rot_end = min(head_end, nq + nkv);
    const int runits = style.rdim >> 3, units = runits + ((d - style.rdim) >> 2);
    for (int idx = head_begin * units + threadIdx.x; idx < rot_end * units; idx += blockDim.x) {
        const int head = idx / units, u = idx - head * units;
        const int col0 = head * d;
        QT* qdst = head < nq ? q_out + (size_t)t * nq * d + col0 : nullptr;
        CT* kdst = (head >= nq && page >= 0) ? cache + ((((size_t)page * 2 + 0) * nkv + (head - nq)) * P + within) * d : nullptr;
        if (u < runits) {
            // the two vectors of inputs: half-split (4u .., rhalf + 4u ..), interleaved (8u .., 8u + 4 ..)
            const int ea = style.interleaved ? 8 * u : 4 * u, eb = style.interleaved ? 8 * u + 4 : rhalf + 4 * u;
            float4 a = load4_split(qkv, base + col0 + ea, nsplit, split_stride);
            float4 b = load4_split(qkv, base + col0 + eb, nsplit, split_stride);
            if (bias) {
                add4(a, *(const float4*)(bias + col0 + ea));
                add4(b, *(const float4*)(bias + col0 + eb));
            }
            const float4 cs = *(const float4*)(cs_table + 4 * u), sn = *(const float4*)(cs_table + rhalf + 4 * u);
            float4 oa, ob;
            if (style.interleaved) {     // pairs (a.x, a.y) (a.z, a.w) (b.x, b.y) (b.z, b.w)
                oa = make_float4(a.x * cs.x - a.y * sn.x, a.y * cs.x + a.x * sn.x, a.z * cs.y - a.w * sn.y, a.w * cs.y + a.z * sn.y);
                ob = make_float4(b.x * cs.z - b.y * sn.z, b.y * cs.z + b.x * sn.z, b.z * cs.w - b.w * sn.w, b.w * cs.w + b.z * sn.w);
            } else {                     // pairs (a.x, b.x) ...
                oa = make_float4(a.x * cs.x - b.x * sn.x, a.y * cs.y - b.y * sn.y, a.z * cs.z - b.z * sn.z, a.w * cs.w - b.w * sn.w);
                ob = make_float4(b.x * cs.x + a.x * sn.x, b.y * cs.y + a.y * sn.y, b.z * cs.z + a.z * sn.z, b.w * cs.w + a.w * sn.w);
            }
            if (qdst) { store4<QT>(qdst + ea, oa); store4<QT>(qdst + eb, ob); }
            else if (kdst) { store4<CT>(kdst + ea, oa); store4<CT>(kdst + eb, ob); }
        } else {
            const int e = style.rdim + 4 * (u - runits);
            float4 a = load4_split(qkv, base + col0 + e, nsplit, split_stride);
            if (bias) add4(a, *(const float4*)(bias + col0 + e));
            if (qdst) store4<QT>(qdst + e, a);
            else if (kdst) store4<CT>(kdst + e, a);
        }
    }
    if (page >= 0) {
        const int v_begin = max(head_begin, nq + nkv);
        const int dq = d >> 2;
        for (int idx = v_begin * dq + threadIdx.x; idx < head_end * dq; idx += blockDim.x) {
            const int head = idx / dq, e = (idx - head * dq) * 4;
            float4 v = load4_split(qkv, base + (size_t)head * d + e, nsplit, split_stride);
            if (bias) add4(v, *(const float4*)(bias + head * d + e));
            store4<CT>(cache + ((((size_t)page * 2 + 1) * nkv + (head - nq - nkv)) * P + within) * d + e, v);
        }
    }
}

// rotary_dim: rotated elements per head (0: none; else even and <= d); interleaved: the pairing.
MHB_EXPORT int mhb_rope_append(const void* qkv, int in_dtype, int nsplit, long long split_stride,
                               const float* bias, const int* positions, const int* tok_seg,
                               const int* block_table, int table_width, const float* inv_freq,
                               void* q_out, void* cache, int act_dtype, int T, int nq, int nkv,
                               int d, int P, int num_pages, int write_kv, int rotary_dim, int interleaved,
                               int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > d || rotary_dim % 2)
        return fail("rope_append: %d rotated elements in a head of %d (even, at most the head size)", rotary_dim, d);
    if (rotary_dim > 0 && inv_freq == nullptr) return fail("rope_append: a rotation needs its frequencies");
    if (nsplit > 1 && in_dtype != MHB_F32) return fail("rope_append: split partials must be float32");
    const int threads = 128;
    // few tokens: spread the heads of a token over several blocks so that the GPU is not idle
    const int heads = nq + 2 * nkv;
    int blocks_y = T >= 512 ? 1 : (512 + T - 1) / T;
    if (blocks_y > heads) blocks_y = heads;
    const int hpb = (heads + blocks_y - 1) / blocks_y;
    blocks_y = (heads + hpb - 1) / hpb;
    dim3 grid(T, blocks_y);
    const size_t smem = sizeof(float) * (rotary_dim > 0 ? rotary_dim : 2);
    RopeStyle style = {rotary_dim, interleaved ? 1 : 0};
    const bool aligned = d % 8 == 0 && rotary_dim % 8 == 0 && split_stride % 4 == 0 &&
                         (((uintptr_t)qkv | (uintptr_t)bias | (uintptr_t)q_out | (uintptr_t)cache) & 15) == 0;
    if (aligned) {
        MHB_DISPATCH_DTYPE(in_dtype, IT, MHB_DISPATCH_DTYPE(act_dtype, AT,
            launch_kernel(rope_append_vec_kernel<IT, AT, AT>, dim3(grid), dim3(threads), smem, stream,
                (const IT*)qkv, nsplit, (size_t)split_stride, bias, positions, tok_seg, block_table,
                table_width, inv_freq, (AT*)q_out, (AT*)cache, nq, nkv, d, P, num_pages, write_kv,
                style, hpb, status)));
        return check_launch("rope_append");
    }
    MHB_DISPATCH_DTYPE(in_dtype, IT, MHB_DISPATCH_DTYPE(act_dtype, AT,
        launch_kernel(rope_append_kernel<IT, AT, AT>, dim3(grid), dim3(threads), smem, stream, 
            (const IT*)qkv, nsplit, (size_t)split_stride, bias, positions, tok_seg, block_table,
            table_width, inv_freq, (AT*)q_out, (AT*)cache, nq, nkv, d, P, num_pages, write_kv,
            style, hpb, status)));
    return check_launch("rope_append");
}

// cos and sin of every token's rotation angles, [T, rdim]: cos[rdim/2] then sin[rdim/2]; once per step
// for all layers (the matrix product's q/k/v epilogue reads it).  Float32 angles as in rope_append.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ table, int T, int half) {
    pdl_launch_dependents();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, i = idx - t * half;
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
    table[(size_t)t * 2 * half + i] = cs;
    table[(size_t)t * 2 * half + half + i] = sn;
}

MHB_EXPORT int mhb_rope_table(const int* positions, const float* inv_freq, float* table, int T, int rotary_dim,
                              cudaStream_t stream) {
    if (T <= 0 || rotary_dim <= 0) return 0;
    if (rotary_dim % 2) return fail("rope_table: %d rotated elements (must be even)", rotary_dim);
    const int half = rotary_dim / 2, threads = 256;
    launch_kernel(rope_table_kernel, dim3((T * half + threads - 1) / threads), dim3(threads), 0, stream, positions,
                  inv_freq, table, T, half);
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
