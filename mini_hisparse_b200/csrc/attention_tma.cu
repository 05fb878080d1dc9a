// Causal grouped-query attention over the paged KV cache with TMA-fed key/value tiles, for decode
// tokens and short portions (long portions go to attention_tc.cu).
//
// The math, the work items and the tile shape are those of attention_mma.cu
// (mini_hisparse/model.py:173-179, mini_hisparse/attention.py:26-35): 16 query rows per CTA, the
// keys of a tile split over the four compute warps, key splits across CTAs merged by the last CTA
// of a token.  (The 64-row shape of the template is kept for reference but not instantiated: the
// tcgen05 kernel serves every size this one takes.)  What differs is how keys and
// values reach shared memory: a fifth warp walks the block table and issues one
// cp.async.bulk.tensor (TMA) per page, plane and 64-column half, with the 128-byte swizzle, into a
// ring of stages guarded by full/empty mbarriers.  The compute warps never issue a load, so the
// ring stays full while they work, which is what a decode step needs: it is bound by how many
// bytes are in flight.  ldmatrix reads the swizzled tiles without bank conflicts.
//
// Needs head_dim 64 or 128 and a page size that divides 64; other shapes use attention_mma.cu or
// attention_simt.cu.  Every mbarrier wait is bounded (status bit 8 when one runs out).
#include "mma_helpers.cuh"
#include "tma_helpers.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
constexpr int KT = 64;
constexpr int CWARPS = 4;                    // compute warps
constexpr int THREADS = (CWARPS + 1) * 32;   // + the TMA warp
constexpr int ITEM_INTS = 8;
constexpr int MAX_MERGE_SPLITS = 64;

struct AttnArgs {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    float* part_acc;
    float* part_ml;
    const int* items;
    const int* positions;
    const int* block_table;
    const int* tok_part_row;
    const int* tok_nsplit;
    int* counters;
    int* status;
    int num_items, width, nq, nkv, P, num_pages, window;
    int fresh;      // keys at positions > positions[tok0] - fresh may have been written by the kernel
                    // before this one (the append of this step); 0: any key may
    float scale;
};

template <int D, int ROWS>
struct Layout {
    static constexpr int HALVES = D / 64;
    static constexpr int STAGES = ROWS == 16 ? 3 : 2;
    static constexpr int Q_BYTES = ROWS * D * 2;            // [HALVES][ROWS][128 B], swizzled
    static constexpr int KV_BYTES = KT * D * 2;             // K or V of one stage: [HALVES][64][128 B]
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;
    static constexpr int BAR_OFFSET = Q_BYTES + STAGES * STAGE_BYTES;
    static constexpr int LOOP_BYTES = BAR_OFFSET + 2 * STAGES * 8;
    static constexpr int MERGE_BYTES = ROWS == 16 ? CWARPS * 16 * (D + 2) * 4 : 0;
    static constexpr int TOTAL = (LOOP_BYTES > MERGE_BYTES ? LOOP_BYTES : MERGE_BYTES) + 1024;
};

// Address of element (row r, column e) of a tile stored as halves of 64 columns, rows of 128 bytes,
// 16-byte chunks XOR-ed with the row's low three bits (what TMA's 128-byte swizzle writes).
__device__ __forceinline__ uint32_t swz(uint32_t base, int rows_per_half, int r, int e) {
    return base + (e >> 6) * rows_per_half * 128 + r * 128 + ((((e & 63) >> 3) ^ (r & 7)) << 4);
}
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CWARPS * 32) : "memory"); }

template <int D, int ROWS>
__global__ void __launch_bounds__(THREADS, 2)
attention_tma_kernel(const __grid_constant__ CUtensorMap kv_map, const AttnArgs a) {
    using L = Layout<D, ROWS>;
    constexpr int STAGES = L::STAGES;
    constexpr int KSTEPS = D / 16;
    constexpr int DTILES = D / 8;
    constexpr bool SPLIT_KEYS = ROWS == 16;
    constexpr int NT = SPLIT_KEYS ? 2 : 8;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int row_pos[ROWS];
    __shared__ int cta_failed;      // a bounded wait ran out somewhere in this CTA: it merges and stores nothing
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

    // Programmatic dependent launch: this kernel may start while the append of this step's keys
    // still runs.  Work items, positions and the block table were copied in before the step's first
    // kernel, and all keys but the step's own are older still, so everything up to the first tile
    // that may hold a fresh key (and the queries) is done before waiting for the append.
    pdl_launch_dependents();
    if ((int)blockIdx.x >= a.num_items) return;
    const int* it = a.items + (size_t)blockIdx.x * ITEM_INTS;
    const int seg = it[0], tok0 = it[1], ntok = it[2], head0 = it[3], nheads = it[4];
    const int kv_begin = it[5], kv_end = it[6], split = it[7];
    const int kvh = blockIdx.y;
    const int groups = a.nq / a.nkv;
    const int nrows = ntok * nheads;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t q_s = smem_addr(smem);
    const uint32_t kv_s = q_s + L::Q_BYTES;
    const uint32_t bar0 = q_s + L::BAR_OFFSET;
    auto full_bar = [&](int s) { return bar0 + 8 * s; };
    auto empty_bar = [&](int s) { return bar0 + 8 * (STAGES + s); };
    const int* table = a.block_table + (size_t)seg * a.width;
    // tiles start on a multiple of 64 keys (so on a page edge); keys before kv_begin are masked
    const int tile_begin = (kv_begin / KT) * KT;
    const int ntiles = kv_end > kv_begin ? (kv_end - tile_begin + KT - 1) / KT : 0;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), CWARPS); }
        mbar_fence_init();
        cta_failed = 0;
    }
    __syncthreads();

    if (warp == CWARPS) {
        // ---- TMA warp: one lane per page of the tile ----------------------------------------------
        const int pages_per_tile = KT / a.P;
        bool ok = true, waited = false;
        int armed = 0;
        const int first_fresh = a.fresh > 0 ? a.positions[tok0] - (a.fresh - 1) : -0x7fffffff;
        for (int itile = 0; itile < ntiles && ok; ++itile) {
            const int stage = itile % STAGES;
            const uint32_t phase = (itile / STAGES) & 1;
            if (!waited && tile_begin + (itile + 1) * KT > first_fresh) {
                pdl_wait();
                waited = true;
            }
            if (lane == 0) ok = mbar_wait(empty_bar(stage), phase ^ 1);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            // Every page slot of the stage is filled: a slot past the last key (or before the first,
            // inside a page that a window has given back) gets the page of key kv_begin again, so
            // that the masked positions hold finite numbers (0 * NaN would poison the output).
            const int kp0 = tile_begin + itile * KT + lane * a.P;
            int page = -1;
            if (lane < pages_per_tile) {
                if (kp0 < kv_end) page = table[kp0 / a.P];
                if (page < 0 || page >= a.num_pages) page = table[kv_begin / a.P];
                if (page >= a.num_pages) page = -1;
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
        if (!ok && lane == 0) {
            // Nothing of ours may still be in flight when the CTA leaves (the copies would land in shared
            // memory that belongs to the next CTA on this SM): wait, bounded again, for the armed stages.
            cta_failed = 1;
            for (int i = max(0, armed - STAGES); i < armed; ++i) mbar_wait(full_bar(i % STAGES), (i / STAGES) & 1);
            if (a.status) atomicOr(a.status, 8);
        }
        return;
    }

    // ---- compute warps ---------------------------------------------------------------------------------
    if (tid < ROWS) row_pos[tid] = tid < nrows ? a.positions[tok0 + tid / nheads] : -1;
    pdl_wait();         // the queries come from the kernel before this one
    for (int c = tid; c < ROWS * (D / 8); c += CWARPS * 32) {
        const int r = c / (D / 8), ch = c % (D / 8);
        const bool live = r < nrows;
        const int t = tok0 + (live ? r / nheads : 0), h = kvh * groups + head0 + (live ? r % nheads : 0);
        const __nv_bfloat16* src = a.q + ((size_t)t * a.nq + h) * D + ch * 8;
        cp_async16(swz(q_s, ROWS, r, ch * 8), src, live ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    compute_sync();

    const int wrow = SPLIT_KEYS ? 0 : warp * 16;
    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    uint32_t qf[KSTEPS][4];
#pragma unroll
    for (int k = 0; k < KSTEPS; ++k) {
        const int r = wrow + (lane & 7) + 8 * ((lane >> 3) & 1), c = k * 16 + 8 * (lane >> 4);
        ldmatrix_x4(swz(q_s, ROWS, r, c), qf[k][0], qf[k][1], qf[k][2], qf[k][3]);
    }
    const float scale_log2 = a.scale * 1.4426950408889634f;
    bool ok = true;

    for (int itile = 0; itile < ntiles; ++itile) {
        const int stage = itile % STAGES;
        ok = mbar_wait(full_bar(stage), (itile / STAGES) & 1);
        if (!ok) break;
        const uint32_t k_s = kv_s + stage * L::STAGE_BYTES;
        const uint32_t v_s = k_s + L::KV_BYTES;
        const int t0 = tile_begin + itile * KT;
        const int key0 = SPLIT_KEYS ? warp * 16 : 0;

        float s[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KSTEPS; k += 2) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                uint32_t b0, b1, b2, b3;
                const int r = key0 + j * 8 + (lane & 7), c = k * 16 + 8 * (lane >> 3);
                ldmatrix_x4(swz(k_s, KT, r, c), b0, b1, b2, b3);
                mma_bf16(s[j], qf[k], b0, b1);
                mma_bf16(s[j], qf[k + 1], b2, b3);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < NT; ++j) {
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int row = wrow + (lane >> 2) + 8 * (x >> 1);
                const int kp = t0 + key0 + j * 8 + (lane & 3) * 2 + (x & 1);
                const int qp = row_pos[row];
                const bool valid = kp >= kv_begin && kp < kv_end && kp <= qp && (a.window <= 0 || kp > qp - a.window);
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
        for (int kk = 0; kk < NT / 2; ++kk) {
#pragma unroll
            for (int i = 0; i < DTILES; i += 2) {
                uint32_t b0, b1, b2, b3;
                const int r = key0 + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = i * 8 + 8 * (lane >> 4);
                ldmatrix_x4_trans(swz(v_s, KT, r, c), b0, b1, b2, b3);
                mma_bf16(o[i], pf[kk], b0, b1);
                mma_bf16(o[i + 1], pf[kk], b2, b3);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(stage));     // this warp is done with the stage
    }
    // A wait that ran out is reported; the warp still walks through the barriers below so that
    // the others are not left waiting for it, but the CTA then merges and stores nothing: the ring
    // may still receive copies (the TMA warp waits for them before it leaves).
    if (!ok && lane == 0) {
        cta_failed = 1;
        if (a.status) atomicOr(a.status, 8);
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    if (SPLIT_KEYS) {
        compute_sync();     // all warps are past their last tile: the ring can become merge scratch
        if (cta_failed) return;
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
        compute_sync();
        for (int idx = tid; idx < nrows * D; idx += CWARPS * 32) {
            const int row = idx / D, e = idx - row * D;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < CWARPS; ++w) M = fmaxf(M, mg[(w * 16 + row) * MS + D]);
            float acc = 0.f, lsum = 0.f;
#pragma unroll
            for (int w = 0; w < CWARPS; ++w) {
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
            compute_sync();
            if (tid == 0) {
                const int chunks = (groups + 15) / 16;
                int* counter = a.counters + ((size_t)tok0 * a.nkv + kvh) * chunks + head0 / 16;
                const int ns = a.tok_nsplit[tok0];
                // more parts than the merge below has scratch for: say so rather than merge a part of them
                if (ns > MAX_MERGE_SPLITS && a.status) atomicOr(a.status, 32);
                const int prev = atomicAdd(counter, 1);
                is_last = prev == ns - 1;
                if (is_last) *counter = 0;
            }
            compute_sync();
            if (is_last) {
                // The merge is a chain of round trips to L2 on the kernel's critical path: every load
                // that does not depend on another is issued at once.
                __threadfence();
                // scratch in the ring, which nobody reads any more (12 KB + 64 bytes)
                float (*wgt_s)[MAX_MERGE_SPLITS] = (float (*)[MAX_MERGE_SPLITS])smem;
                float2 (*ml_s)[MAX_MERGE_SPLITS] = (float2 (*)[MAX_MERGE_SPLITS])(smem + 16 * MAX_MERGE_SPLITS * 4);
                float* inv_s = (float*)(smem + 16 * MAX_MERGE_SPLITS * 12);
                const int ns = min(a.tok_nsplit[tok0], MAX_MERGE_SPLITS);
                for (int idx = tid; idx < nrows * ns; idx += CWARPS * 32) {     // all (maximum, sum) pairs at once
                    const int row = idx / ns, sp = idx - row * ns;
                    const int t = tok0 + row / nheads, hq = kvh * groups + head0 + row % nheads;
                    ml_s[row][sp] = __ldcg((const float2*)(a.part_ml + (((size_t)a.tok_part_row[t] + sp) * a.nq + hq) * 2));
                }
                compute_sync();
                if (tid < nrows) {
                    float M = -INFINITY;
                    for (int sp = 0; sp < ns; ++sp) M = fmaxf(M, ml_s[tid][sp].x);
                    float lsum = 0.f;
                    for (int sp = 0; sp < ns; ++sp) {
                        const float ms = ml_s[tid][sp].x;
                        const float w = ms > -INFINITY ? expf(ms - M) : 0.f;
                        wgt_s[tid][sp] = w;
                        lsum += w * ml_s[tid][sp].y;
                    }
                    inv_s[tid] = lsum > 0.f ? 1.f / lsum : 0.f;
                }
                compute_sync();
                // four elements per thread and step, eight splits in flight; summed in the splits' order
                for (int idx = tid; idx < nrows * (D / 4); idx += CWARPS * 32) {
                    const int row = idx / (D / 4), e = (idx - row * (D / 4)) * 4;
                    const int t = tok0 + row / nheads, hq = kvh * groups + head0 + row % nheads;
                    const float* src = a.part_acc + ((size_t)a.tok_part_row[t] * a.nq + hq) * D + e;
                    const size_t step = (size_t)a.nq * D;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int s0 = 0; s0 < ns; s0 += 8) {
                        float4 v[8];
#pragma unroll
                        for (int q = 0; q < 8; ++q) v[q] = __ldcg((const float4*)(src + (size_t)min(s0 + q, ns - 1) * step));
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            if (s0 + q < ns) {
                                const float w = wgt_s[row][s0 + q];
                                acc.x += w * v[q].x; acc.y += w * v[q].y; acc.z += w * v[q].z; acc.w += w * v[q].w;
                            }
                        }
                    }
                    const float inv = inv_s[row];
                    uint2 packed;
                    packed.x = pack_bf16(acc.x * inv, acc.y * inv);
                    packed.y = pack_bf16(acc.z * inv, acc.w * inv);
                    *(uint2*)(a.out + ((size_t)t * a.nq + hq) * D + e) = packed;
                }
            }
        }
    } else {
        if (!ok) return;
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
int launch(const CUtensorMap& map, const AttnArgs& a, int launch_items, cudaStream_t stream) {
    auto kern = attention_tma_kernel<D, ROWS>;
    constexpr int smem = Layout<D, ROWS>::TOTAL;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("attention_tma: shared memory %d: %s", smem, cudaGetErrorString(e));
        // two CTAs per SM need the large shared-memory carve-out even when one CTA would fit a small one
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        configured = true;
    }
    launch_kernel(kern, dim3(launch_items, a.nkv), dim3(THREADS), smem, stream, map, a);
    return check_launch("attention_tma");
}
}  // namespace

MHB_EXPORT int mhb_attention_tma_supports(int d, int P) {
    return (d == 64 || d == 128) && P >= 2 && P <= KT && KT % P == 0;
}

// cache: one layer's pool [num_pages, 2, nkv, P, d] bfloat16; rows = 16 (items of short segments).
// fresh: the kernel launched before this one may have written the keys of the last `fresh` positions
// up to an item's first token (and later ones); older keys are loaded without waiting for it.
// 0: it may have written any key.
MHB_EXPORT int mhb_attention_tma(const void* q, const void* cache, void* out, float* part_acc, float* part_ml,
                                 const int* items, int num_items, int launch_items, int rows,
                                 const int* positions, const int* block_table, int width,
                                 const int* tok_part_row, const int* tok_nsplit, int* counters, int nq, int nkv,
                                 int d, int P, int num_pages, int window, int fresh, float scale, int* status,
                                 cudaStream_t stream) {
    if (launch_items <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return fail("attention: %d query heads over %d KV heads", nq, nkv);
    if (!mhb_attention_tma_supports(d, P))
        return fail("attention_tma: head_dim %d with pages of %d keys is not built (head_dim 64 or 128, page size dividing 64)", d, P);
    const long long total_rows = (long long)num_pages * 2 * nkv * P;
    if (total_rows > 0x7fffffffLL) return fail("attention_tma: the pool has too many rows for one tensor map");
    CUtensorMap map;
    int rc = make_bf16_map(&map, cache, total_rows, d, d, P);
    if (rc) return rc;
    AttnArgs a;
    a.q = (const __nv_bfloat16*)q; a.out = (__nv_bfloat16*)out; a.part_acc = part_acc; a.part_ml = part_ml;
    a.items = items; a.positions = positions; a.block_table = block_table; a.tok_part_row = tok_part_row;
    a.tok_nsplit = tok_nsplit; a.counters = counters; a.status = status; a.num_items = num_items;
    a.width = width; a.nq = nq; a.nkv = nkv; a.P = P; a.num_pages = num_pages; a.window = window;
    a.scale = scale;
    a.fresh = fresh;
    if (rows == 16) return d == 128 ? launch<128, 16>(map, a, launch_items, stream) : launch<64, 16>(map, a, launch_items, stream);
    return fail("attention_tma: tile height %d", rows);
}
