// Causal grouped-query attention over the paged KV cache on the tensor cores (bfloat16 inputs,
// float32 scores, softmax and accumulation), for prefill portions and decode tokens alike.
//
// Math as in attention_simt.cu (mini_hisparse/model.py:173-179, mini_hisparse/attention.py:26-35):
// s_t = (K[t] . q) * scale over the cached keys t <= the query's position (and inside the window,
// if there is one), w = softmax(s), o = sum_t w_t V[t]; query head h reads KV head h / groups.
// The work items are the same 8 ints {segment, first token, tokens, first head of the group,
// heads, kv_begin, kv_end, split}; split >= 0 writes an un-normalised partial.  With a counter
// array the CTA that finishes a token's last split merges all its splits (in split order, so the
// result does not depend on which CTA comes last); without one, attention_combine does it.
//
// One CTA (4 warps) serves one item and one KV head.  The query heads of a KV group are stacked
// into the row dimension of the tile, so a page of keys is read once for the whole group.
//   ROWS = 64 (long portions): each warp owns 16 query rows and walks all keys.
//   ROWS = 16 (decode tokens, tiny portions): the four warps share the 16 rows and each takes
//     16 of the 64 keys of a tile; their partial results are merged at the end.
// Keys and values arrive in tiles of 64 by cp.async (16-byte chunks gathered through the block
// table, two or three stages deep); rows are padded by 16 bytes, which keeps ldmatrix conflict-free for
// every head size that is a multiple of 16.  Products are mma.sync m16n8k16: the score tile
// feeds the value product straight from registers.
#include "common.cuh"
#include "mma_helpers.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
constexpr int KT = 64;          // keys per tile
constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int ITEM_INTS = 8;
constexpr int MAX_MERGE_SPLITS = 64;   // most key splits of a token that the fused merge takes

struct AttnArgs {
    const __nv_bfloat16* q;     // [T, nq, d]
    const __nv_bfloat16* cache; // [pages, 2, nkv, P, d] of one layer
    __nv_bfloat16* out;         // [T, nq, d]
    float* part_acc;            // [rows, nq, d]
    float* part_ml;             // [rows, nq, 2]
    const int* items;
    const int* positions;
    const int* block_table;
    const int* tok_part_row;
    const int* tok_nsplit;      // splits of each token (used by the fused merge)
    int* counters;              // one per (first token, KV head, head chunk): zero between launches
    int num_items, width, nq, nkv, P, num_pages, window;
    int page_shift;             // log2(P) if P is a power of two, else -1
    float scale;
};

template <int D, int ROWS>
struct Layout {
    static constexpr int LD = D + 8;                        // padded row, in elements
    static constexpr int Q_BYTES = ROWS * LD * 2;
    static constexpr int KV_BYTES = KT * LD * 2;            // one of K or V, one stage
    static constexpr int MERGE_BYTES = ROWS == 16 ? WARPS * 16 * (D + 2) * 4 : 0;
    // decode tiles are bound by memory latency: three stages keep two tiles in flight per CTA
    static constexpr int STAGES = ROWS == 16 ? 3 : 2;
    static constexpr int LOOP_BYTES = Q_BYTES + STAGES * 2 * KV_BYTES;
    static constexpr int TOTAL = LOOP_BYTES > MERGE_BYTES ? LOOP_BYTES : MERGE_BYTES;
};

template <int D, int ROWS>
__global__ void __launch_bounds__(THREADS)
attention_mma_kernel(const AttnArgs a) {
    using L = Layout<D, ROWS>;
    constexpr int LD = L::LD;
    constexpr int KSTEPS = D / 16;        // k-steps of Q K^T
    constexpr int DTILES = D / 8;         // n-tiles of the output
    constexpr bool SPLIT_KEYS = ROWS == 16;
    constexpr int NT = SPLIT_KEYS ? 2 : 8;   // score n-tiles (8 keys each) per warp per tile
    constexpr bool Q_IN_REGS = D <= 128;
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ int row_pos[ROWS];

    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.x >= a.num_items) return;
    const int* it = a.items + (size_t)blockIdx.x * ITEM_INTS;
    const int seg = it[0], tok0 = it[1], ntok = it[2], head0 = it[3], nheads = it[4];
    const int kv_begin = it[5], kv_end = it[6], split = it[7];
    const int kvh = blockIdx.y;
    const int groups = a.nq / a.nkv;
    const int nrows = ntok * nheads;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t q_s = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t kv_s = q_s + L::Q_BYTES;       // [stage][K|V][KT][LD]
    const int* table = a.block_table + (size_t)seg * a.width;
    const size_t plane = (size_t)a.nkv * a.P * D;  // elements between the K and V planes of a page

    // ---- stage the queries --------------------------------------------------------------------
    for (int c = tid; c < ROWS * (D / 8); c += THREADS) {
        const int r = c / (D / 8), ch = c % (D / 8);
        const bool live = r < nrows;
        const int t = tok0 + (live ? r / nheads : 0), h = kvh * groups + head0 + (live ? r % nheads : 0);
        const __nv_bfloat16* src = a.q + ((size_t)t * a.nq + h) * D + ch * 8;
        cp_async16(q_s + (r * LD + ch * 8) * 2, src, live ? 16 : 0);
    }
    if (tid < ROWS) row_pos[tid] = tid < nrows ? a.positions[tok0 + tid / nheads] : -1;

    // Consecutive threads copy consecutive 16-byte chunks of a key row, so a warp's request covers
    // whole rows (full 32-byte sectors).  A thread meets KT * (D/8) / THREADS rows per tile.
    auto load_tile = [&](int stage, int t0) {
        constexpr int CPR = D / 8;                         // chunks per row
        constexpr int ITERS = KT * CPR / THREADS;
        const uint32_t kbase = kv_s + stage * 2 * L::KV_BYTES;
#pragma unroll
        for (int i = 0; i < ITERS; ++i) {
            const int c = i * THREADS + tid;
            const int j = c / CPR, ch = c % CPR;
            const int kp = t0 + j;
            int page = -1;
            if (kp < kv_end) {
                page = table[a.page_shift >= 0 ? (kp >> a.page_shift) : (kp / a.P)];
                if (page >= a.num_pages) page = -1;
            }
            const int within = a.page_shift >= 0 ? (kp & (a.P - 1)) : (kp % a.P);
            const __nv_bfloat16* src = a.cache;
            if (page >= 0) src += (((size_t)page * 2) * a.nkv + kvh) * a.P * D + (size_t)within * D + ch * 8;
            const int bytes = page >= 0 ? 16 : 0;
            const uint32_t kdst = kbase + (j * LD + ch * 8) * 2;
            cp_async16(kdst, src, bytes);
            cp_async16(kdst + L::KV_BYTES, src + (page >= 0 ? plane : 0), bytes);
        }
    };

    constexpr int STAGES = L::STAGES;
    const int ntiles = (kv_end - kv_begin + KT - 1) / KT;
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (st < ntiles) load_tile(st, kv_begin + st * KT);
        cp_async_commit();
    }

    // ---- per-thread state: rows r0 = lane/4 and r0 + 8 of this warp's 16 rows ------------------
    const int wrow = SPLIT_KEYS ? 0 : warp * 16;
    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
    const float scale_log2 = a.scale * 1.4426950408889634f;

    for (int itile = 0; itile < ntiles; ++itile) {
        const int stage = itile % STAGES;
        if (itile + STAGES - 1 < ntiles)
            load_tile((itile + STAGES - 1) % STAGES, kv_begin + (itile + STAGES - 1) * KT);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        if (itile == 0 && Q_IN_REGS) {
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k) {
                const int r = wrow + (lane & 7) + 8 * ((lane >> 3) & 1), c = k * 16 + 8 * (lane >> 4);
                ldmatrix_x4(q_s + (r * LD + c) * 2, qf[k][0], qf[k][1], qf[k][2], qf[k][3]);
            }
        }
        const uint32_t k_s = kv_s + stage * 2 * L::KV_BYTES;
        const uint32_t v_s = k_s + L::KV_BYTES;
        const int t0 = kv_begin + itile * KT;
        const int key0 = SPLIT_KEYS ? warp * 16 : 0;      // first key of this warp inside the tile

        // ---- S = Q K^T -------------------------------------------------------------------------
        float s[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KSTEPS; k += 2) {
            uint32_t qa[2][4];
            if (Q_IN_REGS) {
#pragma unroll
                for (int x = 0; x < 4; ++x) { qa[0][x] = qf[k][x]; qa[1][x] = qf[k + 1 < KSTEPS ? k + 1 : k][x]; }
            } else {
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    if (k + kk < KSTEPS) {
                        const int r = wrow + (lane & 7) + 8 * ((lane >> 3) & 1), c = (k + kk) * 16 + 8 * (lane >> 4);
                        ldmatrix_x4(q_s + (r * LD + c) * 2, qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                // K rows = keys key0 + 8j .. +7; columns = two k-steps (32 elements) when available
                uint32_t b0, b1, b2, b3;
                const int r = key0 + j * 8 + (lane & 7);
                int c = k * 16 + 8 * (lane >> 3);
                if (KSTEPS % 2 == 1 && k + 1 >= KSTEPS) c = k * 16 + 8 * ((lane >> 3) & 1);   // last odd step: stay inside the row
                ldmatrix_x4(k_s + (r * LD + c) * 2, b0, b1, b2, b3);
                mma_bf16(s[j], qa[0], b0, b1);
                if (k + 1 < KSTEPS) mma_bf16(s[j], qa[1], b2, b3);
            }
        }

        // ---- mask, online softmax -----------------------------------------------------------------
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < NT; ++j) {
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int row = wrow + (lane >> 2) + 8 * (x >> 1);
                const int kp = t0 + key0 + j * 8 + (lane & 3) * 2 + (x & 1);
                const int qp = row_pos[row];
                const bool valid = kp < kv_end && kp <= qp && (a.window <= 0 || kp > qp - a.window);
                s[j][x] = valid ? s[j][x] : -INFINITY;
                mx[x >> 1] = fmaxf(mx[x >> 1], s[j][x]);
            }
        }
        float alpha[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            m_use[h] = m_new == -INFINITY ? 0.f : m_new;
            alpha[h] = exp2f((m_run[h] - m_use[h]) * scale_log2);     // exp2(-inf) = 0 on the first tile
            m_run[h] = m_new;
            l_run[h] *= alpha[h];
        }
        uint32_t pf[NT / 2][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            float p[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                p[x] = exp2f((s[j][x] - m_use[x >> 1]) * scale_log2);
                l_run[x >> 1] += p[x];
            }
            pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
            pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
        }
#pragma unroll
        for (int i = 0; i < DTILES; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }

        // ---- O += P V ---------------------------------------------------------------------------------
#pragma unroll
        for (int kk = 0; kk < NT / 2; ++kk) {
#pragma unroll
            for (int i = 0; i < DTILES; i += 2) {
                uint32_t b0, b1, b2, b3;
                const int r = key0 + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = i * 8 + 8 * (lane >> 4);
                ldmatrix_x4_trans(v_s + (r * LD + c) * 2, b0, b1, b2, b3);
                mma_bf16(o[i], pf[kk], b0, b1);
                mma_bf16(o[i + 1], pf[kk], b2, b3);
            }
        }
        __syncthreads();      // everyone is done with this stage before it is loaded again
    }
    cp_async_wait<0>();

    // ---- finish: sums across the quad, merge of the warps (16-row mode), output -----------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    if (ntiles == 0) __syncthreads();
    if (SPLIT_KEYS) {
        // scratch (aliases the tiles, which nobody reads any more): [warp][row][D + 2] floats
        float* mg = (float*)smem;
        constexpr int MS = D + 2;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            float* dst = mg + (warp * 16 + row) * MS;
#pragma unroll
            for (int i = 0; i < DTILES; ++i) {
                dst[i * 8 + (lane & 3) * 2 + 0] = o[i][2 * h + 0];
                dst[i * 8 + (lane & 3) * 2 + 1] = o[i][2 * h + 1];
            }
            if ((lane & 3) == 0) { dst[D] = m_run[h]; dst[D + 1] = l_run[h]; }
        }
        __syncthreads();
        for (int idx = tid; idx < nrows * D; idx += THREADS) {
            const int row = idx / D, e = idx - row * D;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) M = fmaxf(M, mg[(w * 16 + row) * MS + D]);
            float acc = 0.f, lsum = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float mw = mg[(w * 16 + row) * MS + D];
                const float wgt = mw == -INFINITY ? 0.f : exp2f((mw - M) * scale_log2);
                acc += wgt * mg[(w * 16 + row) * MS + e];
                lsum += wgt * mg[(w * 16 + row) * MS + D + 1];
            }
            const int t = tok0 + row / nheads, hq = kvh * groups + head0 + row % nheads;
            if (split < 0) {
                a.out[((size_t)t * a.nq + hq) * D + e] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
            } else {
                const size_t prow = (size_t)a.tok_part_row[t] + split;
                a.part_acc[(prow * a.nq + hq) * D + e] = acc;
                if (e == 0) {
                    a.part_ml[(prow * a.nq + hq) * 2 + 0] = M == -INFINITY ? -INFINITY : M * a.scale;
                    a.part_ml[(prow * a.nq + hq) * 2 + 1] = lsum;
                }
            }
        }
        if (split >= 0 && a.counters != nullptr) {
            // the last CTA of this tile's splits merges them (reference/attention.py:11-20)
            __shared__ int is_last;
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const int chunks = (groups + 15) / 16;
                int* counter = a.counters + ((size_t)tok0 * a.nkv + kvh) * chunks + head0 / 16;
                const int ns = a.tok_nsplit[tok0];
                const int prev = atomicAdd(counter, 1);
                is_last = prev == ns - 1;
                if (is_last) *counter = 0;
            }
            __syncthreads();
            if (is_last) {
                __threadfence();
                // weights of every (row, split) once, then one load per split and output element
                __shared__ float wgt_s[16][MAX_MERGE_SPLITS];
                __shared__ float inv_s[16];
                const int ns = min(a.tok_nsplit[tok0], MAX_MERGE_SPLITS);
                if (tid < nrows) {
                    const int t = tok0 + tid / nheads, hq = kvh * groups + head0 + tid % nheads;
                    const size_t row0 = a.tok_part_row[t];
                    float M = -INFINITY;
                    for (int sp = 0; sp < ns; ++sp) M = fmaxf(M, __ldcg(a.part_ml + ((row0 + sp) * a.nq + hq) * 2));
                    float lsum = 0.f;
                    for (int sp = 0; sp < ns; ++sp) {
                        const float ms = __ldcg(a.part_ml + ((row0 + sp) * a.nq + hq) * 2);
                        const float w = ms > -INFINITY ? expf(ms - M) : 0.f;
                        wgt_s[tid][sp] = w;
                        lsum += w * __ldcg(a.part_ml + ((row0 + sp) * a.nq + hq) * 2 + 1);
                    }
                    inv_s[tid] = lsum > 0.f ? 1.f / lsum : 0.f;
                }
                __syncthreads();
                for (int idx = tid; idx < nrows * D; idx += THREADS) {
                    const int row = idx / D, e = idx - row * D;
                    const int t = tok0 + row / nheads, hq = kvh * groups + head0 + row % nheads;
                    const float* src = a.part_acc + ((size_t)a.tok_part_row[t] * a.nq + hq) * D + e;
                    const size_t step = (size_t)a.nq * D;
                    float acc = 0.f;
#pragma unroll 4
                    for (int sp = 0; sp < ns; ++sp) acc += wgt_s[row][sp] * __ldcg(src + sp * step);
                    a.out[((size_t)t * a.nq + hq) * D + e] = __float2bfloat16_rn(acc * inv_s[row]);
                }
            }
        }
    } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = wrow + (lane >> 2) + 8 * h;
            if (row >= nrows) continue;
            const int t = tok0 + row / nheads, hq = kvh * groups + head0 + row % nheads;
            if (split < 0) {
                const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
                __nv_bfloat16* dst = a.out + ((size_t)t * a.nq + hq) * D + (lane & 3) * 2;
#pragma unroll
                for (int i = 0; i < DTILES; ++i)
                    *(uint32_t*)(dst + i * 8) = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
            } else {
                const size_t prow = (size_t)a.tok_part_row[t] + split;
                float* dst = a.part_acc + (prow * a.nq + hq) * D + (lane & 3) * 2;
#pragma unroll
                for (int i = 0; i < DTILES; ++i) {
                    dst[i * 8] = o[i][2 * h];
                    dst[i * 8 + 1] = o[i][2 * h + 1];
                }
                if ((lane & 3) == 0) {
                    a.part_ml[(prow * a.nq + hq) * 2 + 0] = m_run[h] == -INFINITY ? -INFINITY : m_run[h] * a.scale;
                    a.part_ml[(prow * a.nq + hq) * 2 + 1] = l_run[h];
                }
            }
        }
    }
}

template <int D, int ROWS>
int launch(const AttnArgs& a, int launch_items, cudaStream_t stream) {
    auto kern = attention_mma_kernel<D, ROWS>;
    constexpr int smem = Layout<D, ROWS>::TOTAL;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("attention_mma: shared memory %d: %s", smem, cudaGetErrorString(e));
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        configured = true;
    }
    dim3 grid(launch_items, a.nkv);
    launch_kernel(kern, grid, dim3(THREADS), smem, stream, a);
    return check_launch("attention_mma");
}

template <int ROWS>
int dispatch_d(int d, const AttnArgs& a, int launch_items, cudaStream_t stream) {
    switch (d) {
        case 32: return launch<32, ROWS>(a, launch_items, stream);
        case 64: return launch<64, ROWS>(a, launch_items, stream);
        case 96: return launch<96, ROWS>(a, launch_items, stream);
        case 128: return launch<128, ROWS>(a, launch_items, stream);
    }
    return fail("attention_mma: head_dim %d has no tensor-core instance (32, 64, 96, 128)", d);
}
}  // namespace

// rows = 64 or 16: the tile height the items were planned for.
MHB_EXPORT int mhb_attention_mma(const void* q, const void* cache, void* out, float* part_acc,
                                 float* part_ml, const int* items, int num_items, int launch_items,
                                 int rows, const int* positions, const int* block_table, int width,
                                 const int* tok_part_row, const int* tok_nsplit, int* counters, int nq,
                                 int nkv, int d, int P, int num_pages, int window, float scale,
                                 cudaStream_t stream) {
    if (launch_items <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return fail("attention: %d query heads over %d KV heads", nq, nkv);
    AttnArgs a;
    a.q = (const __nv_bfloat16*)q; a.cache = (const __nv_bfloat16*)cache; a.out = (__nv_bfloat16*)out;
    a.part_acc = part_acc; a.part_ml = part_ml; a.items = items; a.positions = positions;
    a.block_table = block_table; a.tok_part_row = tok_part_row; a.tok_nsplit = tok_nsplit;
    a.counters = counters; a.num_items = num_items; a.width = width;
    a.nq = nq; a.nkv = nkv; a.P = P; a.num_pages = num_pages; a.window = window; a.scale = scale;
    a.page_shift = -1;
    if (P > 0 && (P & (P - 1)) == 0) { a.page_shift = 0; while ((1 << a.page_shift) < P) ++a.page_shift; }
    if (rows == 64) return dispatch_d<64>(d, a, launch_items, stream);
    if (rows == 16) return dispatch_d<16>(d, a, launch_items, stream);
    return fail("attention_mma: tile height %d", rows);
}

MHB_EXPORT int mhb_attention_mma_supports(int d) { return d == 32 || d == 64 || d == 96 || d == 128; }
