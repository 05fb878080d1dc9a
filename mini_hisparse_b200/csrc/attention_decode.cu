// Decode attention in one kernel: for a batch of single new tokens it sums the split-K partials
// of the q/k/v product, adds the bias, rotates q and k, appends k and v to the paged cache,
// attends over the cache and merges a token's key splits inside a thread-block cluster.
//
// The math is that of mini_hisparse/model.py:135-153 (project, rotate), 169-170 / 201 (append before
// attending) and mini_hisparse/attention.py:26-35 (softmax(K q * d^-0.5) V over every cached key,
// the new one included); query head h reads KV head h / groups.  What the separate kernels
// (rotary + append, then attention_tma.cu, then a merge through global memory by a token's last
// CTA) do in three dependent passes happens here in one:
//   * grid (tokens * nsplit, KV heads), cluster (nsplit, 1, 1): the CTAs of a cluster are the key
//     splits of one token and one KV head; split s walks the keys [b_s, e_s) in tiles of 64.
//   * a producer warp streams the tiles by TMA (one cp.async.bulk.tensor per page, plane and
//     64-column half, 128-byte swizzle) into a ring of mbarrier-guarded stages.  Every tile holds
//     keys of earlier steps only, so the ring fills while the kernel before this one still runs.
//   * the four compute warps meanwhile build q (the heads of this KV group: 7 of the 16 tile rows at
//     the 7B shape) from the product's partials, and the CTA that owns the token's own position
//     builds the new k and v, patches them into its last tile in shared memory and, when it has
//     walked its keys, stores them into the page for the steps to come.
//   * the splits' (max, sum, accumulator) meet in distributed shared memory: a CTA that has walked
//     its keys sends every row of its part to the CTA that owns that row (CTA r owns the rows r,
//     r + nsplit, ...; plain st.shared::cluster), one cluster barrier follows, and each owner merges
//     what it received in split order (so the result does not depend on timing) from its own shared
//     memory and writes the row; no partial goes through global memory.
//   * one request far into a long context has too few clusters of 16 to keep the memory busy (four
//     KV heads: 64 CTAs).  Its keys can then be cut into ngroups x nsplit shares: ngroups clusters per
//     token and KV head, each merging its own nsplit shares as above and leaving ONE unnormalised part
//     per query head (accumulator, scaled maximum, sum) in the partial buffers that attention_combine
//     merges; the cluster that owns the token's position appends its key and value.
// Head size 64 or 128, pages that divide 64, at most 16 heads per KV head, at most 16 splits a cluster, and
// at most 16 received rows per CTA (splits x rows owned).
// Every mbarrier wait is bounded (status bit 8); a CTA whose wait ran out still walks through the
// cluster barriers, waits for its armed copies, and writes nothing.
#include "mma_helpers.cuh"
#include "tma_helpers.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
constexpr int KT = 64;
constexpr int ROWS = 16;
constexpr int CWARPS = 4;
constexpr int THREADS = (CWARPS + 1) * 32;
constexpr int STAGES = 3;
constexpr int MAX_CLUSTER = 16;

struct DecodeArgs {
    const float* qkv;          // [qkv_nsplit][T][(nq + 2 nkv) D] float32 partial products
    const float* bias;         // [(nq + 2 nkv) D] or null
    const float* inv_freq;     // [rdim / 2] or null
    __nv_bfloat16* cache;      // this layer's pool [pages, 2, nkv, P, D]
    __nv_bfloat16* out;        // [T, nq D]
    float* part_acc;           // ngroups > 1: [T * ngroups, nq, D] unnormalised sums of each cluster
    float* part_ml;            // ngroups > 1: [T * ngroups, nq, 2] scaled maximum and sum of exponentials
    const int* positions;      // [T]
    const int* block_table;    // [T, width]: token i is segment i
    int* status;
    long long qkv_split_stride;
    int qkv_nsplit, rdim, interleaved;
    int T, width, nq, nkv, P, num_pages, window, nsplit, ngroups;
    float scale;
};

template <int D>
struct Layout {
    static constexpr int HALVES = D / 64;
    static constexpr int Q_BYTES = ROWS * D * 2;
    static constexpr int KV_BYTES = KT * D * 2;
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;
    static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
    static constexpr int MS = D + 4;                                    // a partial row: accumulator, max, sum (16-byte rows)
    static constexpr int MERGE_BYTES = CWARPS * ROWS * MS * 4;          // the four warps' parts, in the ring
    static constexpr int RECV_ROWS = 16;                                // rows this CTA receives: splits x rows it owns
    static constexpr int BAR_OFFSET = Q_BYTES + RING_BYTES;
    static constexpr int CS_OFFSET = BAR_OFFSET + 2 * STAGES * 8 + 16;  // cos, sin of this token
    static constexpr int NEW_OFFSET = CS_OFFSET + D * 4;                // the token's own k and v (bfloat16)
    // what the peers send: not in the ring, since a peer may be done while this CTA still streams tiles
    static constexpr int RECV_OFFSET = NEW_OFFSET + 2 * D * 2;
    static constexpr int TOTAL = RECV_OFFSET + RECV_ROWS * MS * 4 + 1024;
    static_assert(MERGE_BYTES <= RING_BYTES, "the four warps' parts must fit in the ring");
};

__device__ __forceinline__ uint32_t swz(uint32_t base, int rows_per_half, int r, int e) {
    return base + (e >> 6) * rows_per_half * 128 + r * 128 + ((((e & 63) >> 3) ^ (r & 7)) << 4) + (e & 7) * 2;
}
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CWARPS * 32) : "memory"); }
__device__ __forceinline__ void prologue_sync() { asm volatile("bar.sync 2, %0;" ::"n"(THREADS) : "memory"); }
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_addr(uint32_t local, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local), "r"(rank));
    return a;
}
__device__ __forceinline__ void st_peer4(uint32_t addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void st_peer2(uint32_t addr, float2 v) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(v.x), "f"(v.y) : "memory");
}
__device__ __forceinline__ void st_smem_8(uint32_t addr, uint32_t lo, uint32_t hi) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(lo), "r"(hi) : "memory");
}

__device__ __forceinline__ void add4(float4& a, const float4 b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }

// The sums over the product's K splits of two groups of four elements (pa, pb; pb may be null), in
// split order, with the loads of eight splits of both groups in flight at once: a CTA has a few
// hundred of these to do before it can start, and each would otherwise be a chain of round trips.
__device__ __forceinline__ void sum_pair(const float* pa, const float* pb, int nsplit, long long stride, float4& a,
                                         float4& b) {
    a = b = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < nsplit; s0 += 8) {
        float4 va[8], vb[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const size_t off = (size_t)min(s0 + q, nsplit - 1) * stride;
            va[q] = *(const float4*)(pa + off);
            if (pb) vb[q] = *(const float4*)(pb + off);
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            if (s0 + q < nsplit) {
                add4(a, va[q]);
                if (pb) add4(b, vb[q]);
            }
        }
    }
}

// One head of the product (bias added, the first rdim elements rotated) as bfloat16: unit u of the
// head gives two groups of four elements (a rotated unit) or one (a plain unit); emit(e, v) takes them.
template <typename Emit>
__device__ __forceinline__ void head_unit(const DecodeArgs& a, const float* row, int col0, int u, const float* cs,
                                          Emit emit) {
    const int rhalf = a.rdim >> 1, runits = a.rdim >> 3;
    if (u < runits) {
        const int ea = a.interleaved ? 8 * u : 4 * u, eb = a.interleaved ? 8 * u + 4 : rhalf + 4 * u;
        float4 x, y;
        sum_pair(row + col0 + ea, row + col0 + eb, a.qkv_nsplit, a.qkv_split_stride, x, y);
        if (a.bias) {
            add4(x, *(const float4*)(a.bias + col0 + ea));
            add4(y, *(const float4*)(a.bias + col0 + eb));
        }
        const float4 c = *(const float4*)(cs + 4 * u), s = *(const float4*)(cs + rhalf + 4 * u);
        float4 oa, ob;
        if (a.interleaved) {
            oa = make_float4(x.x * c.x - x.y * s.x, x.y * c.x + x.x * s.x, x.z * c.y - x.w * s.y, x.w * c.y + x.z * s.y);
            ob = make_float4(y.x * c.z - y.y * s.z, y.y * c.z + y.x * s.z, y.z * c.w - y.w * s.w, y.w * c.w + y.z * s.w);
        } else {
            oa = make_float4(x.x * c.x - y.x * s.x, x.y * c.y - y.y * s.y, x.z * c.z - y.z * s.z, x.w * c.w - y.w * s.w);
            ob = make_float4(y.x * c.x + x.x * s.x, y.y * c.y + x.y * s.y, y.z * c.z + x.z * s.z, y.w * c.w + x.w * s.w);
        }
        emit(ea, oa);
        emit(eb, ob);
    } else {
        const int e = a.rdim + 4 * (u - runits);
        float4 x, unused;
        sum_pair(row + col0 + e, nullptr, a.qkv_nsplit, a.qkv_split_stride, x, unused);
        if (a.bias) add4(x, *(const float4*)(a.bias + col0 + e));
        emit(e, x);
    }
}

template <int D>
__global__ void __launch_bounds__(THREADS, 2)
attention_decode_kernel(const __grid_constant__ CUtensorMap kv_map, const DecodeArgs a) {
    using L = Layout<D>;
    constexpr int KSTEPS = D / 16;
    constexpr int DTILES = D / 8;
    constexpr int NT = 2;                       // each warp takes 16 of a tile's 64 keys
    constexpr int MS = L::MS;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int cta_failed;          // a bounded wait ran out somewhere in this CTA: it stores nothing
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // blockIdx.x = (token, group of shares, share in the group); the share in the group is the rank in the cluster
    const int per_token = a.ngroups * a.nsplit;
    const int t = blockIdx.x / per_token, share = blockIdx.x - t * per_token;
    const int group = share / a.nsplit, split = share - group * a.nsplit;
    const int kvh = blockIdx.y;
    const int groups = a.nq / a.nkv, nrows = groups;
    const int pos = a.positions[t];
    const int kv_end = pos + 1;
    const int kv_first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    // the split's keys: equal shares rounded up to whole tiles, as the host's plan for such a batch
    const int span = kv_end - kv_first;
    const int chunk = (((span + per_token - 1) / per_token + KT - 1) / KT) * KT;
    const int kv_begin = min(kv_end, kv_first + share * chunk);
    const int kv_stop = min(kv_end, kv_begin + chunk);
    const bool owner = kv_stop == kv_end && kv_stop > kv_begin;             // this CTA sees the token's own key
    const int tile_begin = (kv_begin / KT) * KT;
    const int ntiles = kv_stop > kv_begin ? (kv_stop - tile_begin + KT - 1) / KT : 0;

    const uint32_t q_s = smem_addr(smem);
    const uint32_t kv_s = q_s + L::Q_BYTES;
    const uint32_t bar0 = q_s + L::BAR_OFFSET;
    auto full_bar = [&](int s) { return bar0 + 8 * s; };
    auto empty_bar = [&](int s) { return bar0 + 8 * (STAGES + s); };
    float* cs = (float*)(smem + L::CS_OFFSET);
    __nv_bfloat16* kv_new = (__nv_bfloat16*)(smem + L::NEW_OFFSET);
    float* recv = (float*)(smem + L::RECV_OFFSET);        // [split][row this CTA owns][MS]
    const int owned = (nrows + a.nsplit - 1) / a.nsplit;   // rows a CTA owns at most
    const int* table = a.block_table + (size_t)t * a.width;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), CWARPS); }
        mbar_fence_init();
        cta_failed = 0;
    }
    __syncthreads();

    bool ok = true;
    if (warp == CWARPS) {
        // ---- TMA warp: one lane per page of the tile; nothing it loads is written during this step
        const int pages_per_tile = KT / a.P;
        int armed = 0;
        bool met = false;
        // After the tiles that fill the ring (or all, if they are fewer) this warp has nothing to do
        // until the compute warps free a stage: if the CTA owns the token's own position, its lanes
        // build the new value row meanwhile (the compute warps build q and the new key); then all
        // warps meet once, so that the rows are in shared memory before anybody reads them.
        auto meet = [&]() {
            if (owner) {
                pdl_wait();     // the product's partials come from the kernel before this one
                const float* row = a.qkv + (size_t)t * (a.nq + 2 * a.nkv) * D;
                for (int e = 4 * lane; e < D; e += 128) {
                    const int col = (a.nq + a.nkv + kvh) * D + e;
                    float4 v, unused;
                    sum_pair(row + col, nullptr, a.qkv_nsplit, a.qkv_split_stride, v, unused);
                    if (a.bias) add4(v, *(const float4*)(a.bias + col));
                    *(uint2*)(kv_new + D + e) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
                }
            }
            prologue_sync();
            met = true;
        };
        // Every page slot of a stage is filled: a slot past the last key (or before the first, inside
        // a page that a window has given back) gets the page of key kv_begin again, so that the
        // masked positions hold finite numbers.  The page ids of a tile are fetched one tile ahead:
        // a look-up in the block table is a round trip to L2 that would otherwise sit between the
        // release of a stage and its next copy.
        const int spare = ntiles > 0 ? table[kv_begin / a.P] : -1;
        auto page_of = [&](int itile) {
            const int kp0 = tile_begin + itile * KT + lane * a.P;
            return (lane < pages_per_tile && itile < ntiles && kp0 < kv_stop) ? table[kp0 / a.P] : -1;
        };
        int page_ahead = page_of(0);
        for (int itile = 0; itile < ntiles; ++itile) {
            const int stage = itile % STAGES;
            if (itile == STAGES) meet();
            int page = page_ahead;
            page_ahead = page_of(itile + 1);
            if (lane == 0) ok = mbar_wait(empty_bar(stage), ((itile / STAGES) & 1) ^ 1);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < pages_per_tile) {
                if (page < 0 || page >= a.num_pages) page = spare;
                if (page >= a.num_pages) page = -1;
            } else {
                page = -1;
            }
            const unsigned have = __ballot_sync(0xffffffffu, page >= 0);
            if (lane == 0) mbar_expect_tx(full_bar(stage), __popc(have) * 2 * a.P * D * 2);
            __syncwarp();
            if (page >= 0) {
                const int row0 = ((page * 2) * a.nkv + kvh) * a.P;
                const uint32_t dst = kv_s + stage * L::STAGE_BYTES + lane * a.P * 128;
#pragma unroll
                for (int h = 0; h < L::HALVES; ++h) {
                    tma_load_2d(dst + h * KT * 128, &kv_map, h * 64, row0, full_bar(stage));
                    tma_load_2d(dst + L::KV_BYTES + h * KT * 128, &kv_map, h * 64, row0 + a.nkv * a.P, full_bar(stage));
                }
            }
            armed = itile + 1;
        }
        if (!met) meet();
        if (!ok) {
            // nothing of ours may still be in flight when the ring is reused or the CTA leaves
            if (lane == 0)
                for (int i = max(0, armed - STAGES); i < armed; ++i) mbar_wait(full_bar(i % STAGES), (i / STAGES) & 1);
            if (lane == 0) cta_failed = 1;
            if (lane == 0 && a.status) atomicOr(a.status, 8);
        }
    } else {
        // ---- compute warps: q, the new k and v, then the tiles ---------------------------------------
        const int rhalf = a.rdim >> 1;
        for (int i = tid; i < rhalf; i += CWARPS * 32) {      // the angles need positions and constants only
            float sn, c;
            sincosf((float)pos * a.inv_freq[i], &sn, &c);
            cs[i] = c;
            cs[rhalf + i] = sn;
        }
        for (int c = tid; c < (ROWS - nrows) * (D / 8); c += CWARPS * 32) {     // rows without a head hold zeros
            const int r = nrows + c / (D / 8), e = (c % (D / 8)) * 8;
            st_smem_8(swz(q_s, ROWS, r, e), 0u, 0u);
            st_smem_8(swz(q_s, ROWS, r, e + 4), 0u, 0u);
        }
        compute_sync();
        pdl_wait();         // the product's partials come from the kernel before this one
        const float* row = a.qkv + (size_t)t * (a.nq + 2 * a.nkv) * D;
        const int units = (a.rdim >> 3) + ((D - a.rdim) >> 2);
        // one list of units: the group's query heads, then (in the CTA that owns the token's position)
        // the new key; at the 7B shape that is one unit for each of the 128 threads
        for (int idx = tid; idx < (nrows + (owner ? 1 : 0)) * units; idx += CWARPS * 32) {
            const int r = idx / units, u = idx - r * units;
            if (r < nrows) {
                head_unit(a, row, (kvh * groups + r) * D, u, cs, [&](int e, float4 v) {
                    st_smem_8(swz(q_s, ROWS, r, e), pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
                });
            } else {
                head_unit(a, row, (a.nq + kvh) * D, u, cs, [&](int e, float4 v) {
                    *(uint2*)(kv_new + e) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
                });
            }
        }
        prologue_sync();      // q, the new key and (from the TMA warp) the new value are in shared memory

        float o[DTILES][4];
#pragma unroll
        for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
        uint32_t qf[KSTEPS][4];
#pragma unroll
        for (int k = 0; k < KSTEPS; ++k) {
            const int r = (lane & 7) + 8 * ((lane >> 3) & 1), c = k * 16 + 8 * (lane >> 4);
            ldmatrix_x4(swz(q_s, ROWS, r, c), qf[k][0], qf[k][1], qf[k][2], qf[k][3]);
        }
        const float scale_log2 = a.scale * 1.4426950408889634f;
        const int key0 = warp * 16;

        for (int itile = 0; itile < ntiles; ++itile) {
            const int stage = itile % STAGES;
            ok = mbar_wait(full_bar(stage), (itile / STAGES) & 1);
            if (!ok) break;
            const uint32_t k_s = kv_s + stage * L::STAGE_BYTES;
            const uint32_t v_s = k_s + L::KV_BYTES;
            const int t0 = tile_begin + itile * KT;
            if (owner && pos >= t0 + key0 && pos < t0 + key0 + 16) {
                // the token's own key and value are not in the page yet: this warp's 16 keys include it
                const int r = pos - t0, ch = lane & 15;
                if (ch < D / 8) {
                    const uint4 v = *(const uint4*)(kv_new + (lane >> 4) * D + ch * 8);
                    const uint32_t dst = swz(lane < 16 ? k_s : v_s, KT, r, ch * 8);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                }
                __syncwarp();
            }

            // scores: two accumulators per key group (even and odd steps along the head), so that the
            // chain of dependent products is half as long; their sum is the score
            float s[NT][4], s2[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
                s2[j][0] = s2[j][1] = s2[j][2] = s2[j][3] = 0.f;
            }
#pragma unroll
            for (int k = 0; k < KSTEPS; k += 2) {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    uint32_t b0, b1, b2, b3;
                    const int r = key0 + j * 8 + (lane & 7), c = k * 16 + 8 * (lane >> 3);
                    ldmatrix_x4(swz(k_s, KT, r, c), b0, b1, b2, b3);
                    mma_bf16(s[j], qf[k], b0, b1);
                    mma_bf16(s2[j], qf[k + 1], b2, b3);
                }
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
#pragma unroll
                for (int x = 0; x < 4; ++x) s[j][x] += s2[j][x];
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const int kp = t0 + key0 + j * 8 + (lane & 3) * 2 + (x & 1);
                    const bool valid = kp >= kv_begin && kp < kv_stop;      // causal and window limits are the split's
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
                alpha[h] = exp2f((m_run[h] - m_use[h]) * scale_log2);
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
#pragma unroll
            for (int i = 0; i < DTILES; i += 2) {
                uint32_t b0, b1, b2, b3;
                const int r = key0 + (lane & 7) + 8 * ((lane >> 3) & 1), c = i * 8 + 8 * (lane >> 4);
                ldmatrix_x4_trans(swz(v_s, KT, r, c), b0, b1, b2, b3);
                mma_bf16(o[i], pf[0], b0, b1);
                mma_bf16(o[i + 1], pf[0], b2, b3);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(stage));     // this warp is done with the stage
        }
        if (!ok && lane == 0) {
            cta_failed = 1;
            if (a.status) atomicOr(a.status, 8);
        }

#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
        }
        // the four warps' parts meet in the ring (every tile has been consumed; if a wait ran out the
        // TMA warp waits for its armed copies itself and nothing below is stored to global memory)
        compute_sync();
        ok = cta_failed == 0;
        float* mg = (float*)(smem + L::Q_BYTES);
        if (ok) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = (lane >> 2) + 8 * h;
                float* dst = mg + (warp * ROWS + r) * MS;
#pragma unroll
                for (int i = 0; i < DTILES; ++i)
                    *(float2*)(dst + i * 8 + (lane & 3) * 2) = make_float2(o[i][2 * h + 0], o[i][2 * h + 1]);
                if ((lane & 3) == 0) *(float2*)(dst + D) = make_float2(m_run[h], l_run[h]);
            }
        }
        compute_sync();
        // four columns of a row per thread and turn: the row's weights are worked out once per turn
        for (int idx = tid; idx < nrows * (D / 4); idx += CWARPS * 32) {
            const int r = idx / (D / 4), e = (idx - r * (D / 4)) * 4;
            float2 ml[CWARPS];
#pragma unroll
            for (int w = 0; w < CWARPS; ++w) ml[w] = *(const float2*)(mg + (w * ROWS + r) * MS + D);
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < CWARPS; ++w) M = fmaxf(M, ml[w].x);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float lsum = 0.f;
#pragma unroll
            for (int w = 0; w < CWARPS; ++w) {
                const float wgt = ml[w].x == -INFINITY ? 0.f : exp2f((ml[w].x - M) * scale_log2);
                const float4 v = *(const float4*)(mg + (w * ROWS + r) * MS + e);
                acc.x += wgt * v.x; acc.y += wgt * v.y; acc.z += wgt * v.z; acc.w += wgt * v.w;
                lsum += wgt * ml[w].y;
            }
            if (!ok) { M = -INFINITY; acc = make_float4(0.f, 0.f, 0.f, 0.f); lsum = 0.f; }
            // to the CTA that owns row r, into the place of this split
            const uint32_t dst = peer_addr(smem_addr(recv + (split * owned + r / a.nsplit) * MS), r % a.nsplit);
            st_peer4(dst + e * 4, acc);
            if (e == 0) st_peer2(dst + D * 4, make_float2(M, lsum));
        }
    }

    // ---- the splits of the token meet: every part has been sent when the barrier completes; CTA r
    // merges the rows r, r + nsplit, ... from its own shared memory ----------------------------------------
    cluster_sync();
    if (warp < CWARPS) {
        const float scale_log2 = a.scale * 1.4426950408889634f;
        for (int r = split, k = 0; r < nrows; r += a.nsplit, ++k) {
            for (int e = tid; e < D; e += CWARPS * 32) {
                float M = -INFINITY;
                for (int p = 0; p < a.nsplit; ++p) M = fmaxf(M, recv[(p * owned + k) * MS + D]);
                float acc = 0.f, lsum = 0.f;
                for (int p = 0; p < a.nsplit; ++p) {           // in split order
                    const float* src = recv + (p * owned + k) * MS;
                    const float w = src[D] == -INFINITY ? 0.f : exp2f((src[D] - M) * scale_log2);
                    acc += w * src[e];
                    lsum += w * src[D + 1];
                }
                const size_t head = (size_t)kvh * groups + r;
                if (a.ngroups == 1) {
                    a.out[((size_t)t * a.nq + head) * D + e] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
                } else if (cta_failed == 0) {
                    // this cluster's part of the token: attention_combine merges the groups in order
                    const size_t prow = (size_t)t * a.ngroups + group;
                    a.part_acc[(prow * a.nq + head) * D + e] = acc;
                    if (e == 0) {
                        float* ml = a.part_ml + (prow * a.nq + head) * 2;
                        ml[0] = (lsum > 0.f && M > -INFINITY) ? M * a.scale : -INFINITY;
                        ml[1] = lsum;
                    }
                }
            }
        }
        if (owner && cta_failed == 0) {
            // the token's own key and value go into their page for the steps to come (last, so that
            // the peers do not wait for it at the barrier above)
            const int page = table[pos / a.P];
            if (page < 0 || page >= a.num_pages) {
                if (tid == 0 && a.status) atomicOr(a.status, 2);      // never write outside the pool
            } else {
                for (int c = tid; c < 2 * (D / 8); c += CWARPS * 32) {
                    const int plane = c / (D / 8), ch = c % (D / 8);
                    __nv_bfloat16* dst = a.cache + ((((size_t)page * 2 + plane) * a.nkv + kvh) * a.P + pos % a.P) * D;
                    *(uint4*)(dst + ch * 8) = *(const uint4*)(kv_new + plane * D + ch * 8);
                }
            }
        }
    }
    // no second barrier: after the one above nobody touches another CTA's shared memory
}

template <int D>
int configure() {
    auto kern = attention_decode_kernel<D>;
    constexpr int smem = Layout<D>::TOTAL;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("attention_decode: shared memory %d: %s", smem, cudaGetErrorString(e));
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);     // clusters of up to 16
        if (e != cudaSuccess) return fail("attention_decode: clusters of more than 8: %s", cudaGetErrorString(e));
        configured = true;
    }
    return 0;
}

// How many clusters of `nsplit` CTAs of this kernel the device can hold at once (the CTAs of a
// cluster share a GPC, so this is not the number of CTA slots divided by nsplit).
template <int D>
int max_clusters(int nsplit) {
    int rc = configure<D>();
    if (rc) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nsplit, 1);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = Layout<D>::TOTAL;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = nsplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, attention_decode_kernel<D>, &cfg);
    if (e != cudaSuccess) return fail("attention_decode: clusters of %d: %s", nsplit, cudaGetErrorString(e));
    return n;
}

template <int D>
int launch(const CUtensorMap& map, const DecodeArgs& a, cudaStream_t stream) {
    auto kern = attention_decode_kernel<D>;
    constexpr int smem = Layout<D>::TOTAL;
    int rc = configure<D>();
    if (rc) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.T * a.ngroups * a.nsplit, a.nkv);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = a.nsplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map, a);
    if (e != cudaSuccess) return fail("attention_decode: launch of clusters of %d: %s", a.nsplit, cudaGetErrorString(e));
    return check_launch("attention_decode");
}
}  // namespace

MHB_EXPORT int mhb_attention_decode_supports(int d, int P, int groups, int nsplit, int rotary_dim) {
    return (d == 64 || d == 128) && P >= 2 && P <= KT && KT % P == 0 && groups >= 1 && groups <= ROWS && nsplit >= 1 &&
           nsplit <= MAX_CLUSTER && nsplit * ((groups + nsplit - 1) / nsplit) <= 16 && rotary_dim >= 0 &&
           rotary_dim <= d && rotary_dim % 8 == 0;
}

// Clusters of nsplit CTAs that run at once on the current device (0: such clusters cannot be placed); < 0: error.
MHB_EXPORT int mhb_attention_decode_max_clusters(int d, int nsplit) {
    if ((d != 64 && d != 128) || nsplit < 1 || nsplit > MAX_CLUSTER) return fail("attention_decode: head_dim %d, %d splits", d, nsplit);
    return d == 128 ? max_clusters<128>(nsplit) : max_clusters<64>(nsplit);
}

// qkv: the stacked q/k/v product of T single tokens as qkv_nsplit float32 partial matrices
// [T, (nq + 2 nkv) d], qkv_split_stride elements apart; cache: one layer's pool [num_pages, 2, nkv, P, d]
// bfloat16, block_table [T, width] (row i: the pages of token i's request), positions [T].
// Every token's keys are cut into ngroups * nsplit equal shares (whole tiles of 64), nsplit of them to a
// cluster; out [T, nq d] bfloat16.  With ngroups > 1 nothing is written to out: each cluster leaves its part
// in part_acc [T * ngroups, nq, d] and part_ml [T * ngroups, nq, 2] (row t * ngroups + g) for attention_combine.
MHB_EXPORT int mhb_attention_decode(const float* qkv, int qkv_nsplit, long long qkv_split_stride, const float* bias,
                                    const float* inv_freq, int rotary_dim, int interleaved, void* cache, void* out,
                                    const int* positions, const int* block_table, int width, int T, int nq, int nkv,
                                    int d, int P, int num_pages, int window, int nsplit, int ngroups, float* part_acc,
                                    float* part_ml, float scale, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (ngroups < 1 || ngroups > 64) return fail("attention_decode: %d groups of key shares", ngroups);
    if (ngroups > 1 && (!part_acc || !part_ml)) return fail("attention_decode: groups of key shares need the partial buffers");
    if (nkv <= 0 || nq % nkv) return fail("attention: %d query heads over %d KV heads", nq, nkv);
    if (!mhb_attention_decode_supports(d, P, nq / nkv, nsplit, rotary_dim))
        return fail("attention_decode: head_dim %d, pages of %d keys, %d heads per KV head, %d key splits, %d rotated "
                    "elements is not built (head_dim 64 or 128, page size dividing 64, at most 16 heads per KV head, "
                    "at most 16 splits and 16 received rows per CTA, rotated elements a multiple of 8)", d, P, nq / nkv, nsplit, rotary_dim);
    if (rotary_dim > 0 && inv_freq == nullptr) return fail("attention_decode: a rotation needs its frequencies");
    if (qkv_nsplit < 1 || (qkv_nsplit > 1 && qkv_split_stride % 4) || ((uintptr_t)qkv & 15) || ((uintptr_t)bias & 15) ||
        ((uintptr_t)cache & 15))
        return fail("attention_decode: the product's parts, the bias and the pool must be 16-byte aligned");
    const long long total_rows = (long long)num_pages * 2 * nkv * P;
    if (total_rows > 0x7fffffffLL) return fail("attention_decode: the pool has too many rows for one tensor map");
    CUtensorMap map;
    int rc = make_bf16_map(&map, cache, total_rows, d, d, P);
    if (rc) return rc;
    DecodeArgs a;
    a.qkv = qkv; a.bias = bias; a.inv_freq = inv_freq; a.cache = (__nv_bfloat16*)cache; a.out = (__nv_bfloat16*)out;
    a.positions = positions; a.block_table = block_table; a.status = status; a.qkv_split_stride = qkv_split_stride;
    a.qkv_nsplit = qkv_nsplit; a.rdim = rotary_dim; a.interleaved = interleaved ? 1 : 0; a.T = T; a.width = width;
    a.nq = nq; a.nkv = nkv; a.P = P; a.num_pages = num_pages; a.window = window; a.nsplit = nsplit; a.scale = scale;
    a.ngroups = ngroups; a.part_acc = part_acc; a.part_ml = part_ml;
    return d == 128 ? launch<128>(map, a, stream) : launch<64>(map, a, stream);
}
