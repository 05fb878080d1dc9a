// Causal grouped-query attention over the paged KV cache, for prefill portions and decode
// tokens alike, with float32 scores, softmax and accumulation on the CUDA cores.
//
// Math (mini_hisparse/model.py:173-179 for prompts, mini_hisparse/attention.py:26-35 for a
// decoded token): query head h reads KV head h / groups; s_t = (K[t] . q) * scale for every
// cached key t <= the query's position (the token's own key was appended before);
// w = softmax(s); o = sum_t w_t V[t].  An optional window keeps keys t > position - window.
//
// Work is described by items (8 ints each) that the host writes:
//   {segment, first token (index in the batch), tokens, first head in the group, heads,
//    kv_begin, kv_end, split}
// One CTA handles one item for one KV head: rows = tokens x heads (<= 16) against keys
// [kv_begin, kv_end).  split < 0: the normalised output is written to `out`.  split >= 0:
// the CTA writes an un-normalised partial (max, sum, accumulator) and combine merges the
// splits with the rule of reference/attention.py:11-20.
#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
constexpr int R_TILE = 16;   // query rows per CTA
constexpr int KT = 32;       // keys per tile: one per lane
constexpr int WARPS = 4;
constexpr int ROWS_PER_WARP = R_TILE / WARPS;
constexpr int ITEM_INTS = 8;

struct AttnArgs {
    const void* q;             // [T, nq, d]
    const void* cache;         // [pages, 2, nkv, P, d] of one layer
    void* out;                 // [T, nq, d]
    float* part_acc;           // [rows, nq, d]
    float* part_ml;            // [rows, nq, 2]
    const int* items;
    const int* positions;      // [T]
    const int* block_table;    // [S, width]
    const int* tok_part_row;   // [T] first partial row of a token
    int num_items, width, nq, nkv, d, P, num_pages, window;
    float scale;
};

template <typename CT, int DPL>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const AttnArgs a) {
    extern __shared__ float smem[];
    const int d = a.d;
    float* q_s = smem;                       // [R_TILE][d]
    float* k_s = q_s + R_TILE * d;           // [KT][d + 1]
    float* v_s = k_s + KT * (d + 1);         // [KT][d]
    __shared__ int row_pos[R_TILE];

    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.x >= a.num_items) return;
    const int* it = a.items + (size_t)blockIdx.x * ITEM_INTS;
    const int seg = it[0], tok0 = it[1], ntok = it[2], head0 = it[3], nheads = it[4];
    const int kv_begin = it[5], kv_end = it[6], split = it[7];
    const int kvh = blockIdx.y;
    const int groups = a.nq / a.nkv;
    const int nrows = ntok * nheads;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const CT* q = (const CT*)a.q;
    const CT* cache = (const CT*)a.cache;

    // stage the queries (float32) and the rows' positions
    for (int idx = threadIdx.x; idx < R_TILE * d; idx += blockDim.x) {
        const int r = idx / d, e = idx - r * d;
        float v = 0.f;
        if (r < nrows) {
            const int t = tok0 + r / nheads, h = kvh * groups + head0 + r % nheads;
            v = to_float(q[((size_t)t * a.nq + h) * d + e]);
        }
        q_s[idx] = v;
    }
    if (threadIdx.x < R_TILE) {
        const int r = threadIdx.x;
        row_pos[r] = r < nrows ? a.positions[tok0 + r / nheads] : -1;
    }
    __syncthreads();

    float m[ROWS_PER_WARP], l[ROWS_PER_WARP], acc[ROWS_PER_WARP][DPL];
#pragma unroll
    for (int rs = 0; rs < ROWS_PER_WARP; ++rs) {
        m[rs] = -INFINITY;
        l[rs] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[rs][i] = 0.f;
    }

    const int* table = a.block_table + (size_t)seg * a.width;
    for (int t0 = kv_begin; t0 < kv_end; t0 += KT) {
        // load KT keys and values: warp w takes keys w*8 .. w*8+7, lanes run along d
        for (int j = warp * (KT / WARPS); j < (warp + 1) * (KT / WARPS); ++j) {
            const int kp = t0 + j;
            int page = -1;
            if (kp < kv_end) {
                page = table[kp / a.P];
                if (page >= a.num_pages) page = -1;
            }
            if (page >= 0) {
                const size_t off = ((((size_t)page * 2) * a.nkv + kvh) * a.P + kp % a.P) * (size_t)d;
                const size_t voff = off + (size_t)a.nkv * a.P * d;
                for (int e = lane; e < d; e += 32) {
                    k_s[j * (d + 1) + e] = to_float(cache[off + e]);
                    v_s[j * d + e] = to_float(cache[voff + e]);
                }
            } else {
                for (int e = lane; e < d; e += 32) {
                    k_s[j * (d + 1) + e] = 0.f;
                    v_s[j * d + e] = 0.f;
                }
            }
        }
        __syncthreads();
        const int kp = t0 + lane;  // this lane's key
#pragma unroll
        for (int rs = 0; rs < ROWS_PER_WARP; ++rs) {
            const int r = rs * WARPS + warp;
            if (r >= nrows) continue;  // uniform within the warp
            const int qp = row_pos[r];
            const float* qr = q_s + r * d;
            const float* kr = k_s + lane * (d + 1);
            float s = 0.f;
            for (int e = 0; e < d; ++e) s = fmaf(qr[e], kr[e], s);
            s *= a.scale;
            const bool valid = kp < kv_end && kp <= qp && (a.window <= 0 || kp > qp - a.window);
            if (!valid) s = -INFINITY;
            const float m_new = fmaxf(m[rs], warp_max(s));
            float p = 0.f, alpha = 1.f;
            if (m_new > -INFINITY) {
                p = valid ? expf(s - m_new) : 0.f;
                alpha = m[rs] > -INFINITY ? expf(m[rs] - m_new) : 0.f;
            }
            l[rs] = l[rs] * alpha + warp_sum(p);
            m[rs] = m_new;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[rs][i] *= alpha;
            for (int j = 0; j < KT; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int e = lane + 32 * i;
                    if (e < d) acc[rs][i] = fmaf(pj, v_s[j * d + e], acc[rs][i]);
                }
            }
        }
        __syncthreads();
    }

#pragma unroll
    for (int rs = 0; rs < ROWS_PER_WARP; ++rs) {
        const int r = rs * WARPS + warp;
        if (r >= nrows) continue;
        const int t = tok0 + r / nheads, h = kvh * groups + head0 + r % nheads;
        if (split < 0) {
            const float inv = l[rs] > 0.f ? 1.f / l[rs] : 0.f;
            CT* o = (CT*)a.out + ((size_t)t * a.nq + h) * d;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int e = lane + 32 * i;
                if (e < d) o[e] = from_float<CT>(acc[rs][i] * inv);
            }
        } else {
            const size_t prow = (size_t)a.tok_part_row[t] + split;
            float* pa = a.part_acc + (prow * a.nq + h) * d;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int e = lane + 32 * i;
                if (e < d) pa[e] = acc[rs][i];
            }
            if (lane == 0) {
                a.part_ml[(prow * a.nq + h) * 2 + 0] = m[rs];
                a.part_ml[(prow * a.nq + h) * 2 + 1] = l[rs];
            }
        }
    }
}

// Merge the splits of a token (reference/attention.py:11-20):
//   M = max m_s;  w_s = exp(m_s - M) (0 where m_s = -inf);  o = sum w_s acc_s / sum w_s l_s
template <typename OT>
__global__ void attention_combine_kernel(const float* __restrict__ part_acc,
                                         const float* __restrict__ part_ml,
                                         const int* __restrict__ tok_part_row,
                                         const int* __restrict__ tok_nsplit, OT* __restrict__ out,
                                         int nq, int d, int every) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    // every > 0: each token has exactly that many parts, in the rows t * every ...
    const int ns = every > 0 ? every : tok_nsplit[t];
    if (ns <= 0) return;  // written directly by the attention kernel
    const size_t row0 = every > 0 ? (size_t)t * every : tok_part_row[t];
    float M = -INFINITY;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, part_ml[((row0 + s) * nq + h) * 2]);
    float L = 0.f;
    for (int s = 0; s < ns; ++s) {
        const float ms = part_ml[((row0 + s) * nq + h) * 2];
        const float w = ms > -INFINITY ? expf(ms - M) : 0.f;
        L += w * part_ml[((row0 + s) * nq + h) * 2 + 1];
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < ns; ++s) {
            const float ms = part_ml[((row0 + s) * nq + h) * 2];
            const float w = ms > -INFINITY ? expf(ms - M) : 0.f;
            o += w * part_acc[((row0 + s) * nq + h) * d + e];
        }
        out[((size_t)t * nq + h) * d + e] = from_float<OT>(o * inv);
    }
}

template <typename CT>
int launch_attention(const AttnArgs& a, int max_items, cudaStream_t stream) {
    const int dpl = (a.d + 31) / 32;
    const size_t smem = sizeof(float) * ((size_t)R_TILE * a.d + (size_t)KT * (a.d + 1) + (size_t)KT * a.d);
    dim3 grid(max_items, a.nkv);
#define MHB_ATTN_CASE(N)                                                                        \
    case N: {                                                                                   \
        auto kern = attention_simt_kernel<CT, N>;                                               \
        if (smem > 48 * 1024) {                                                                 \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 (int)smem);                                    \
            if (e != cudaSuccess) return fail("attention: shared memory %zu: %s", smem,        \
                                              cudaGetErrorString(e));                           \
        }                                                                                       \
        launch_kernel(kern, grid, dim3(WARPS * 32), smem, stream, a);                           \
        break;                                                                                  \
    }
    switch (dpl) {
        MHB_ATTN_CASE(1) MHB_ATTN_CASE(2) MHB_ATTN_CASE(3) MHB_ATTN_CASE(4)
        MHB_ATTN_CASE(5) MHB_ATTN_CASE(6) MHB_ATTN_CASE(7) MHB_ATTN_CASE(8)
        default: return fail("attention: head_dim %d is larger than 256", a.d);
    }
#undef MHB_ATTN_CASE
    return check_launch("attention_simt");
}
}  // namespace

MHB_EXPORT int mhb_attention_simt(const void* q, const void* cache, void* out, int dtype,
                                  float* part_acc, float* part_ml, const int* items, int num_items,
                                  int max_items, const int* positions, const int* block_table,
                                  int width, const int* tok_part_row, int nq, int nkv, int d, int P,
                                  int num_pages, int window, float scale, cudaStream_t stream) {
    if (max_items <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return fail("attention: %d query heads over %d KV heads", nq, nkv);
    if (nkv > 65535) return fail("attention: too many KV heads");
    AttnArgs a;
    a.q = q; a.cache = cache; a.out = out; a.part_acc = part_acc; a.part_ml = part_ml;
    a.items = items; a.positions = positions; a.block_table = block_table;
    a.tok_part_row = tok_part_row; a.num_items = num_items; a.width = width; a.nq = nq;
    a.nkv = nkv; a.d = d; a.P = P; a.num_pages = num_pages; a.window = window; a.scale = scale;
    MHB_DISPATCH_DTYPE(dtype, CT, return launch_attention<CT>(a, max_items, stream));
    return 0;
}

// every > 0: token t has `every` parts in the rows t * every ... of the partial buffers (tok_part_row and
// tok_nsplit are not read); else token t has tok_nsplit[t] parts from row tok_part_row[t].
MHB_EXPORT int mhb_attention_combine(const float* part_acc, const float* part_ml,
                                     const int* tok_part_row, const int* tok_nsplit, void* out,
                                     int dtype, int T, int nq, int d, int every, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (every <= 0 && (!tok_part_row || !tok_nsplit)) return fail("attention_combine: no list of parts");
    dim3 grid(T, nq);
    const int threads = d >= 128 ? 128 : 32 * ((d + 31) / 32);
    MHB_DISPATCH_DTYPE(dtype, OT,
        launch_kernel(attention_combine_kernel<OT>, grid, dim3(threads), 0, stream, part_acc, part_ml,
                      tok_part_row, tok_nsplit, (OT*)out, nq, d, every));
    return check_launch("attention_combine");
}
