// Causal grouped-query attention for long prompt portions on the 5th-generation tensor cores.
//
// Math and work items as in attention_tma.cu (mini_hisparse/model.py:173-179): one CTA serves one
// item (a run of tokens of one request times the heads of one KV group: up to 128 query rows) and
// one KV head, against the cached keys [kv_begin, kv_end) read through the block table.
//
// Per tile of 64 keys:
//   S = Q K^T        tcgen05.mma, M = 128 rows, N = 64 keys, K = head_dim; Q and the key tile are
//                    K-major in shared memory (TMA, 128-byte swizzle); S lands in tensor memory.
//   softmax          four warps, ONE QUERY ROW PER THREAD: tcgen05.ld brings the row's 64 scores into
//                    registers, so maximum and sum need no shuffles; scores, exponentials and sums
//                    are float32; P goes back to tensor memory as bfloat16 (tcgen05.st), over the
//                    first half of the score buffer it came from.
//   O += P V         tcgen05.mma with P as the operand in tensor memory, M = 128, N = head_dim,
//                    K = 64, accumulated in tensor memory; the value tile [keys, head_dim] is the
//                    MN-major operand exactly as TMA wrote it.
// The running maximum that the exponentials refer to is only raised when a row's true maximum has
// grown by more than 2^8 (so p <= 256, exact enough in bfloat16 and float32); only then the row's
// accumulator in tensor memory is rescaled (tcgen05.ld, multiply, tcgen05.st).  That is rare after
// the first tiles, so a softmax thread normally touches 64 scores per tile and nothing else.
// Two S buffers let the MMA warp compute the next tile's scores while the softmax warps work, and
// since each tile's P has a buffer of its own the softmax warps never wait for a P V product
// (except to rescale).  Keys and values travel in rings of their own (three key tiles, two value
// tiles), each fed by a producer warp of its own: a key tile is free as soon as its scores are
// done, long before its values are used, so the key loads run two tiles ahead.  Two CTAs share an
// SM (tensor memory 2 x 256 columns).  What sets the pace is the thread that issues the MMAs: every
// barrier it looks at costs it some 290 cycles, so it looks at two per tile (P and V together, the
// key tile) and commits three times (scores, key ring, P V).
// Warps 0 and 6 issue the TMA loads (keys, values), warp 1 owns tensor memory and issues the MMAs,
// warps 2-5 are the softmax warps.  Every mbarrier wait is bounded (status bit 16 when one runs out).
//
// Needs head_dim 64 or 128 and a page size that divides 64.  An item may cover a part of its keys
// (the planner splits long tiles when there are too few of them for the GPU): it then leaves its
// unnormalised sums for attention_combine.
#include "mma_helpers.cuh"
#include "tc_helpers.cuh"
#include "tma_helpers.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
constexpr int ROWS = 128;
constexpr int KT = 64;
constexpr int THREADS = 224;
constexpr int ITEM_INTS = 8;

struct AttnArgs {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const int* items;
    const int* positions;
    const int* block_table;
    const int* tok_part_row;     // for items that cover a part of their keys (split >= 0)
    float* part_acc;             // [rows, nq, d] unnormalised sums
    float* part_ml;              // [rows, nq, 2] reference maximum (scaled) and sum of exponentials
    int* status;
    int num_items, width, nq, nkv, P, num_pages, window;
    float scale;
};

constexpr int K_STAGES = 3;
constexpr int V_STAGES = 2;      // value tile j shares its barriers with P(j): both are indexed by j & 1

template <int D>
struct Layout {
    static constexpr int HALVES = D / 64;
    static constexpr int Q_BYTES = HALVES * ROWS * 128;
    static constexpr int K_BYTES = HALVES * KT * 128;          // one key tile; a value tile has the same size
    static constexpr int K_OFFSET = Q_BYTES;
    static constexpr int V_OFFSET = K_OFFSET + K_STAGES * K_BYTES;
    static constexpr int BAR_OFFSET = V_OFFSET + V_STAGES * K_BYTES;
    static constexpr int NUM_BARS = 2 * K_STAGES + 1 + 2 + 2 + 3 + 1;   // k full/empty, q, s full, p+v full, o done, o final, drain
    static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16;
    static constexpr int TMEM_COLS = 256;                      // S/P: 2 x 64 columns, O tile: D columns from column 128
};

// 2^x by the special-function unit (about 2 ulp; the result is rounded to bfloat16 anyway); 2^-inf = 0
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t swz_addr(uint32_t base, int rows_per_half, int r, int e) {
    return base + (e >> 6) * rows_per_half * 128 + r * 128 + ((((e & 63) >> 3) ^ (r & 7)) << 4);
}

template <int D>
__global__ void __launch_bounds__(THREADS, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap kv_map, const AttnArgs a) {
    using L = Layout<D>;
    constexpr int HALVES = L::HALVES;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t base = smem_addr(smem);
    const uint32_t q_s = base, k_ring = base + L::K_OFFSET, v_ring = base + L::V_OFFSET;
    const uint32_t bars = base + L::BAR_OFFSET;
    auto k_full = [&](int s) { return bars + 8 * s; };
    auto k_empty = [&](int s) { return bars + 8 * (K_STAGES + s); };
    constexpr int B0 = 2 * K_STAGES;
    const uint32_t q_full = bars + 8 * B0;
    auto s_full = [&](int b) { return bars + 8 * (B0 + 1 + b); };
    // P(j) is in tensor memory AND V(j) has landed: one barrier (four softmax warps and the value
    // producer arrive on it), because every barrier the MMA thread looks at costs it some 290 cycles.
    // A softmax warp may be one tile ahead of another, so even and odd tiles have barriers of their own;
    // V(j + 2) is only asked for when P V(j) has completed, so nothing of a later tile arrives early.
    auto pv_full = [&](int b) { return bars + 8 * (B0 + 3 + b); };
    // P V(j) has completed: a barrier for even and one for odd tiles, since the waiting threads are
    // not in step with the value warp and a parity wait cannot tell phases two apart
    auto o_done = [&](int b) { return bars + 8 * (B0 + 5 + b); };
    const uint32_t o_final = bars + 8 * (B0 + 7);     // the last P V has completed
    const uint32_t drain = bars + 8 * (B0 + 8);       // only used when a wait has run out (see the MMA warp)
    uint32_t* tmem_slot = (uint32_t*)(smem + L::BAR_OFFSET + 8 * L::NUM_BARS);

    pdl_launch_dependents();
    pdl_wait();
    // CTAs start in the order of the linear block index: item-major, so that the longest items (the
    // planner sorts them first) of ALL KV heads start first
    const int linear = blockIdx.x;
    const int item = linear / a.nkv;
    if (item >= a.num_items) return;
    const int* it = a.items + (size_t)item * ITEM_INTS;
    const int seg = it[0], tok0 = it[1], ntok = it[2], head0 = it[3], nheads = it[4];
    const int kv_begin = it[5], kv_end = it[6], split = it[7];
    if (split >= 0 && (!a.part_acc || !a.part_ml || !a.tok_part_row)) {     // nowhere to put a part: refuse
        if (threadIdx.x == 0 && a.status) atomicOr(a.status, 16);
        return;
    }
    const int kvh = linear % a.nkv;
    const int groups = a.nq / a.nkv;
    const int nrows = ntok * nheads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* table = a.block_table + (size_t)seg * a.width;
    const int tile_begin = (kv_begin / KT) * KT;
    const int ntiles = kv_end > kv_begin ? (kv_end - tile_begin + KT - 1) / KT : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < K_STAGES; ++s) { mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1); }
        mbar_init(q_full, 4);
        for (int b = 0; b < 2; ++b) mbar_init(s_full(b), 1);
        for (int b = 0; b < 2; ++b) mbar_init(pv_full(b), 5);
        for (int b = 0; b < 2; ++b) mbar_init(o_done(b), 1);
        mbar_init(o_final, 1);
        mbar_init(drain, 1);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(smem_addr(tmem_slot), L::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool ok = true;

    if (warp == 0 || warp == 6) {
        // ---- TMA warps: warp 0 brings the key tiles, warp 6 the value tiles, one lane per page of a
        // tile; every page slot of a stage is filled.  Two warps because each waits for its own ring:
        // a key tile is free as soon as its scores are done, a value tile only after P V two tiles
        // later, and one warp doing both in turn held every key tile back behind a value tile (the MMA
        // thread then waited over a thousand cycles per tile for keys).
        const bool values = warp == 6;
        const int pages_per_tile = KT / a.P;
        const int stages = values ? V_STAGES : K_STAGES;
        int armed = 0;
        for (int j = 0; j < ntiles && ok; ++j) {
            const int stage = j % stages;
            const uint32_t full = values ? pv_full(stage) : k_full(stage);
            // a value stage is free when P V two tiles back has completed (o_done of the same parity)
            if (lane == 0) ok = mbar_wait(values ? o_done(stage) : k_empty(stage), ((j / stages) & 1) ^ 1);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            const int kp0 = tile_begin + j * KT + lane * a.P;
            int page = -1;
            if (lane < pages_per_tile) {
                if (kp0 < kv_end) page = table[kp0 / a.P];
                if (page < 0 || page >= a.num_pages) page = table[kv_begin / a.P];   // masked keys: any finite data
                if (page >= a.num_pages) page = -1;
            }
            const unsigned have = __ballot_sync(0xffffffffu, page >= 0);
            if (lane == 0) mbar_expect_tx(full, __popc(have) * a.P * D * 2);
            __syncwarp();
            if (page >= 0) {
                const int row0 = ((page * 2 + (values ? 1 : 0)) * a.nkv + kvh) * a.P;
                const uint32_t dst = (values ? v_ring : k_ring) + stage * L::K_BYTES + lane * a.P * 128;
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_2d(dst + h * KT * 128, &kv_map, h * 64, row0, full);
            }
            armed = j + 1;
        }
        if (!ok && lane == 0 && !values) {
            // a wait ran out: the key copies this warp armed must have landed before the CTA leaves (a
            // value tile's barrier also counts the softmax warps' arrivals, so its copies are waited
            // for by time alone: the same bounded wait on the last key stage covers them, since the
            // value warp armed them no later)
            for (int i = max(0, armed - K_STAGES); i < armed; ++i) mbar_wait(k_full(i % K_STAGES), (i / K_STAGES) & 1);
        }
    } else if (warp == 1) {
        // ---- MMA warp ----------------------------------------------------------------------------------
        // One thread issues all products, in the order S(0), S(1), then per tile P V(j), S(j + 2).
        // S(j + 2) overwrites the columns of S(j) and P(j): the softmax warps have read S(j) (they have
        // announced P(j)), and P V(j), which reads P(j), was issued before it by the same thread, and
        // the tensor pipe runs one thread's products in order.  A thread that has issued MMAs pays
        // some 250 cycles for the first barrier it looks at afterwards and little for the next ones,
        // so all of a tile's waits come first and its eight to twelve MMAs follow in one go.
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(KT, false);      // S: N = 64 keys, both operands K-major
            constexpr uint32_t idesc_o = umma_idesc(D, true);        // O tile: N = head_dim, V is MN-major
            // Descriptors are built once: a step inside a tile only moves the address field (units of 16
            // bytes; the tiles are 1024-byte aligned, so the field never carries).  This thread runs
            // alone in its warp, and every dependent instruction it saves is four or five cycles per MMA.
            const uint64_t q_desc = smem_desc_kmajor(q_s), k_desc0 = smem_desc_kmajor(k_ring);
            const uint64_t v_desc0 = smem_desc_mnmajor(v_ring, KT * 128, 1024);
            auto issue_s = [&](int j) {
                const uint64_t k_desc = k_desc0 + (uint64_t)((j % K_STAGES) * (L::K_BYTES / 16));
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint64_t da = q_desc + (uint64_t)(((k >> 2) * (ROWS * 128) + (k & 3) * 32) / 16);
                    const uint64_t db = k_desc + (uint64_t)(((k >> 2) * (KT * 128) + (k & 3) * 32) / 16);
                    umma_bf16(tmem + (j & 1) * KT, da, db, idesc_s, k > 0 ? 1u : 0u);
                }
                umma_commit(s_full(j & 1));
                umma_commit(k_empty(j % K_STAGES));     // the key tile is free once its scores are done
            };
            ok = mbar_wait(q_full, 0);
            for (int j = 0; j < 2 && j < ntiles && ok; ++j) {
                ok = mbar_wait(k_full(j), 0);
                if (ok) { tc_fence_after(); issue_s(j); }
            }
            for (int j = 0; j < ntiles && ok; ++j) {
                ok = mbar_wait(pv_full(j & 1), (j >> 1) & 1);        // P(j) is in tensor memory, O is rescaled if needed, V(j) has landed
                if (ok && j + 2 < ntiles) ok = mbar_wait(k_full((j + 2) % K_STAGES), ((j + 2) / K_STAGES) & 1);
                if (!ok) break;
                tc_fence_after();
                const uint64_t v_desc = v_desc0 + (uint64_t)((j % V_STAGES) * (L::K_BYTES / 16));
#pragma unroll
                for (int k = 0; k < KT / 16; ++k)
                    umma_bf16_tmem_a(tmem + 128, tmem + (j & 1) * KT + k * 8, v_desc + (uint64_t)(k * 16 * 128 / 16), idesc_o,
                                     (j > 0 || k > 0) ? 1u : 0u);
                umma_commit(o_done(j & 1));             // O holds tiles 0..j and V(j) is consumed when this completes
                if (j + 1 == ntiles) umma_commit(o_final);
                if (j + 2 < ntiles) issue_s(j + 2);
            }
            if (!ok) {
                // leaving early: tensor memory must not be freed under a product that still runs
                umma_commit(drain);
                mbar_wait(drain, 0);
            }
        }
    } else {
        // ---- softmax warps: thread = query row -----------------------------------------------------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const bool live = row < nrows;
        const int t = tok0 + (live ? row / nheads : 0), hq = kvh * groups + head0 + (live ? row % nheads : 0);
        {   // stage this thread's query row (swizzled, K-major)
            const __nv_bfloat16* src = a.q + ((size_t)t * a.nq + hq) * D;
#pragma unroll
            for (int ch = 0; ch < D / 8; ++ch) cp_async16(swz_addr(q_s, ROWS, row, ch * 8), src + ch * 8, live ? 16 : 0);
            cp_async_commit();
            cp_async_wait<0>();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);
        }
        // a row beyond the tile's rows sees every key (its queries are zeros and nothing of it is
        // stored): it must not drag its warp through the masked path on every tile
        const int qp = live ? a.positions[t] : 0x3fffffff;
        const float scale_log2 = a.scale * 1.4426950408889634f;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        float m_ref = -INFINITY;      // the maximum the exponentials refer to (at most 2^8 below the true one)
        float l_run = 0.f;

        for (int j = 0; j < ntiles; ++j) {
            ok = mbar_wait(s_full(j & 1), (j >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            uint32_t sr[KT];
            tmem_ld64(lane_addr + (j & 1) * KT, sr);
            tmem_ld_wait();
            const int t0 = tile_begin + j * KT;
            // most tiles lie wholly inside this row's range of keys: no mask then
            const int lo = max(kv_begin, a.window > 0 ? qp - a.window + 1 : 0), hi = min(kv_end - 1, qp);
            if (!(t0 >= lo && t0 + KT - 1 <= hi)) {
#pragma unroll
                for (int x = 0; x < KT; ++x) {
                    const int kp = t0 + x;
                    if (!(kp >= lo && kp <= hi)) sr[x] = __float_as_uint(-INFINITY);
                }
            }
            // the maximum as four independent chains (one chain of 64 dependent operations was a
            // quarter of this thread's time per tile)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int x = 0; x < KT; x += 4) {
#pragma unroll
                for (int q = 0; q < 4; ++q) mx4[q] = fmaxf(mx4[q], __uint_as_float(sr[x + q]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // raise the reference maximum only when the row's maximum outgrew it by more than 2^8
            const bool raise = mx > -INFINITY && (m_ref == -INFINITY || (mx - m_ref) * scale_log2 > 8.f);
            const float m_old = m_ref;
            if (raise) m_ref = mx;
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            // the exponentials (2^(s * c - m * c): one FMA and one ex2 each), packed to bfloat16, while
            // the previous tile's P V may still run
            const float m_scaled = m_use * scale_log2;
            float ps4[4] = {0.f, 0.f, 0.f, 0.f};       // four independent chains again
            uint32_t pw[KT / 2];
#pragma unroll
            for (int x = 0; x < KT; x += 2) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(sr[x]), scale_log2, -m_scaled));
                const float p1 = fast_exp2(fmaf(__uint_as_float(sr[x + 1]), scale_log2, -m_scaled));
                ps4[(x >> 1) & 3] += p0 + p1;
                pw[x >> 1] = pack_bf16(p0, p1);
            }
            const float psum = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
            const bool rescale = raise && m_old > -INFINITY;     // there is an accumulator to rescale
            if (__any_sync(0xffffffffu, rescale)) {
                // O is only ours once the previous tile's P V has completed
                ok = mbar_wait(o_done((j - 1) & 1), ((j - 1) >> 1) & 1);
                if (!ok) break;
                tc_fence_after();
                const float alpha = rescale ? exp2f((m_old - m_use) * scale_log2) : 1.f;
                l_run *= alpha;
#pragma unroll
                for (int c = 0; c < D; c += 16) {
                    uint32_t r[16];
                    tmem_ld16(lane_addr + 128 + c, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int x = 0; x < 16; ++x) r[x] = __float_as_uint(__uint_as_float(r[x]) * alpha);
                    tmem_st16(lane_addr + 128 + c, r);
                }
            }
            // P(j) over the first 32 columns of S(j)'s buffer: column i holds keys 2i and 2i + 1
            tmem_st32(lane_addr + (j & 1) * KT, pw);
            tmem_st_wait();
            l_run += psum;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(pv_full(j & 1));
        }
        if (ok && ntiles > 0) ok = mbar_wait(o_final, 0);
        tc_fence_after();
        if (ok && split >= 0) {
            // a part of the keys: the unnormalised sums, the reference maximum and the sum of the
            // exponentials go to the partial buffers; attention_combine merges the parts in order
            const size_t prow = live ? (size_t)a.tok_part_row[t] + split : 0;
            float* dst = a.part_acc + (prow * a.nq + hq) * D;
#pragma unroll
            for (int c = 0; c < D; c += 16) {
                uint32_t r[16];
                if (ntiles > 0) {
                    tmem_ld16(lane_addr + 128 + c, r);      // warp-wide: every lane takes part
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int x = 0; x < 16; ++x) r[x] = 0;
                }
                if (live) {
#pragma unroll
                    for (int x = 0; x < 16; x += 4) *(uint4*)(dst + c + x) = make_uint4(r[x], r[x + 1], r[x + 2], r[x + 3]);
                }
            }
            if (live) {
                float* ml = a.part_ml + (prow * a.nq + hq) * 2;
                ml[0] = (l_run > 0.f && m_ref > -INFINITY) ? m_ref * a.scale : -INFINITY;
                ml[1] = l_run;
            }
        } else if (ok) {
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            __nv_bfloat16* dst = a.out + ((size_t)t * a.nq + hq) * D;
#pragma unroll
            for (int c = 0; c < D; c += 16) {
                uint32_t r[16];
                if (ntiles > 0) {
                    tmem_ld16(lane_addr + 128 + c, r);      // warp-wide: every lane takes part
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int x = 0; x < 16; ++x) r[x] = 0;
                }
                if (live) {
                    uint4 v0, v1;
                    v0.x = pack_bf16(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv);
                    v0.y = pack_bf16(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv);
                    v0.z = pack_bf16(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv);
                    v0.w = pack_bf16(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv);
                    v1.x = pack_bf16(__uint_as_float(r[8]) * inv, __uint_as_float(r[9]) * inv);
                    v1.y = pack_bf16(__uint_as_float(r[10]) * inv, __uint_as_float(r[11]) * inv);
                    v1.z = pack_bf16(__uint_as_float(r[12]) * inv, __uint_as_float(r[13]) * inv);
                    v1.w = pack_bf16(__uint_as_float(r[14]) * inv, __uint_as_float(r[15]) * inv);
                    *(uint4*)(dst + c) = v0;
                    *(uint4*)(dst + c + 8) = v1;
                }
            }
        }
    }
    if (!ok && lane == 0 && a.status) atomicOr(a.status, 16);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, L::TMEM_COLS);
}

template <int D>
int launch(const CUtensorMap& map, const AttnArgs& a, int launch_items, cudaStream_t stream) {
    auto kern = attention_tc_kernel<D>;
    constexpr int smem = Layout<D>::TOTAL;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("attention_tc: shared memory %d: %s", smem, cudaGetErrorString(e));
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        configured = true;
    }
    launch_kernel(kern, dim3((unsigned)launch_items * a.nkv), dim3(THREADS), smem, stream, map, a);
    return check_launch("attention_tc");
}
}  // namespace

MHB_EXPORT int mhb_attention_tc_supports(int d, int P) {
    return (d == 64 || d == 128) && P >= 2 && P <= KT && KT % P == 0;
}

// Items must be planned for tiles of 128 rows.  An item with split >= 0 covers a part of its keys
// and writes to row tok_part_row[token] + split of the partial buffers (as the other attention
// kernels do; attention_combine merges); split = -1 writes the output.  cache: one layer's pool
// [num_pages, 2, nkv, P, d] bfloat16.
MHB_EXPORT int mhb_attention_tc(const void* q, const void* cache, void* out, const int* items, int num_items,
                                const int* positions, const int* block_table, int width,
                                const int* tok_part_row, float* part_acc, float* part_ml, int nq, int nkv, int d,
                                int P, int num_pages, int window, float scale, int* status, cudaStream_t stream) {
    if (num_items <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return fail("attention: %d query heads over %d KV heads", nq, nkv);
    if (!mhb_attention_tc_supports(d, P))
        return fail("attention_tc: head_dim %d with pages of %d keys is not built (head_dim 64 or 128, page size dividing 64)", d, P);
    const long long total_rows = (long long)num_pages * 2 * nkv * P;
    if (total_rows > 0x7fffffffLL) return fail("attention_tc: the pool has too many rows for one tensor map");
    CUtensorMap map;
    int rc = make_bf16_map(&map, cache, total_rows, d, d, P);
    if (rc) return rc;
    AttnArgs a;
    a.q = (const __nv_bfloat16*)q; a.out = (__nv_bfloat16*)out; a.items = items; a.positions = positions;
    a.block_table = block_table; a.tok_part_row = tok_part_row; a.part_acc = part_acc; a.part_ml = part_ml;
    a.status = status; a.num_items = num_items; a.width = width; a.nq = nq;
    a.nkv = nkv; a.P = P; a.num_pages = num_pages; a.window = window; a.scale = scale;
    return d == 128 ? launch<128>(map, a, num_items, stream) : launch<64>(map, a, num_items, stream);
}
