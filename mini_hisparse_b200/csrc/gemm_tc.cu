// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a:
//   D[128 x BN] += A_tile[128 x 64] * B_tile[BN x 64]^T   per pipeline stage,
// operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), products
// issued by one thread with tcgen05.mma, the float32 accumulator held in tensor memory and read
// back with tcgen05.ld for the epilogue.
//
// Both operands are row-major with K contiguous (nn.Linear layout, mini_hisparse/model.py:57-60:
// y = x W^T).  Three shapes of use:
//   * few tokens (decode):   A = weights [N, K] (the 128-row operand streams the weights),
//     B = activations [M <= 256, K]; the tile is written transposed, C[m, n] row-major again.
//     One tile per CTA, two CTAs per SM for tiles of up to 64 tokens.
//   * tokens in between:     the same one-tile kernel with A = activations, B = weights.
//     With nsplit > 1 the K range is cut; split z writes a float32 partial matrix at
//     C + z * split_stride and the consumer sums the parts in order.
//   * many tokens (prefill): a persistent kernel, one CTA per SM (further down), with the plain,
//     the SwiGLU and the rotate-and-append epilogue.
//
// Warp roles (192 threads): warp 0 issues TMA loads, warp 1 owns tensor memory and issues the
// MMAs, warps 2-5 read the accumulator (warp w may touch lanes 32*(w%4) .. +31) and store.
// The thread that issues MMAs pays some 250-290 cycles for every mbarrier it looks at afterwards
// (measured: a loop of MMAs alone runs at 128 cycles per 128 x 256 x 16 MMA and 64 for N = 128,
// but a K block of four MMAs costs 480 cycles as soon as the loop waits on a barrier, whatever
// N): tiles narrower than 256 are not faster per K block, only their last round may fit better.
// Every wait on an mbarrier is bounded; a wait that runs out sets bit 4 of *status and the CTA
// leaves through the common exit, which frees its tensor memory.  What holds on that path: the
// thread that issued MMAs commits them to a barrier of its own and waits (bounded) for it before
// the CTA's final barrier, so tensor memory is not freed under a product that still runs; the
// TMA warp waits (bounded) for the stages it armed, so no copy lands in shared memory that the
// SM's next CTA owns; and the epilogue stores nothing once its wait has run out.
#include <cuda.h>
#include <climits>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

using namespace mhb;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {

constexpr int BM = 128;          // rows of the A operand per tile = TMEM lanes
constexpr int BK = 64;           // bf16 elements per stage along K = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr uint32_t WAIT_LIMIT = 1u << 20;

// ---- PTX wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: false if the phase did not complete within the limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = WAIT_LIMIT) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// One look at the barrier, no waiting.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ void mbar_arrive_plain(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B): groups of 8 rows are
// 1024 bytes apart (SBO); the leading offset is unused for this layout; version 1 = sm_100.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);          // start address, bits 0-13
    d |= (uint64_t)1 << 16;                           // leading byte offset (ignored), bits 16-29
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset, bits 32-45
    d |= (uint64_t)1 << 46;                           // descriptor version
    d |= (uint64_t)2 << 61;                           // layout: 128-byte swizzle
    return d;
}
// A step of 16 elements along K inside a 128-byte swizzled row moves the start address by 32 bytes,
// i.e. the descriptor's address field (units of 16 bytes) by 2.  The tiles are 1024-byte aligned and
// the steps stay inside a row, so the field never carries: a descriptor is built once per tile and
// stepped with one addition (the thread that issues the MMAs runs alone in its warp; every dependent
// instruction it saves is four or five cycles per MMA).
__device__ __forceinline__ uint64_t desc_step(uint64_t desc, int k) { return desc + (uint64_t)(k * (UMMA_K * 2 / 16)); }

// Instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = BN.
__host__ __device__ constexpr uint32_t make_idesc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

template <int BN, int STAGES>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BARRIER_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = BARRIER_OFFSET + (2 * STAGES + 2) * 8 + 16 + 1024;   // + alignment slack
};

template <typename OT> __device__ __forceinline__ void store_out(OT* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.f + expf(-g)) * u; }

// C element of (a-row ra, b-row rb): TRANSPOSED ? C[rb, ra] : C[ra, rb].
// EPI = 1 (SwiGLU): the weight operand holds gate and up rows interleaved in blocks of 16
// (rows 32j .. 32j+15 = gate rows 16j .., rows 32j+16 .. 32j+31 = up rows 16j ..); the epilogue
// writes silu(gate) * up, so C has half as many columns as the weight has rows
// (mini_hisparse/model.py:70-71).  Not combined with split K.
template <int BN, int STAGES, bool TRANSPOSED, typename OT, int EPI>
__global__ void __launch_bounds__(THREADS, (Smem<BN, STAGES>::TOTAL <= 112 * 1024) ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               OT* __restrict__ C, int Ra, int Rb, int K, long long ldc, int kb_per_split,
               long long split_stride, int constant_operand, int* __restrict__ status) {
    using S = Smem<BN, STAGES>;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + S::BARRIER_OFFSET;
    auto full_bar = [&](int s) { return bar_base + 8 * s; };
    auto empty_bar = [&](int s) { return bar_base + 8 * (STAGES + s); };
    const uint32_t tmem_full_bar = bar_base + 8 * (2 * STAGES);
    const uint32_t drain_bar = bar_base + 8 * (2 * STAGES + 1);      // only used when a wait has run out
    uint32_t* tmem_slot = (uint32_t*)(smem + S::BARRIER_OFFSET + 8 * (2 * STAGES + 2));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ra0 = blockIdx.x * BM, rb0 = blockIdx.y * BN;
    const int total_kb = (K + BK - 1) / BK;
    const int kb_begin = blockIdx.z * kb_per_split;
    const int kb_end = min(total_kb, kb_begin + kb_per_split);
    const int num_kb = max(0, kb_end - kb_begin);

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(tmem_full_bar, 1);
        mbar_init(drain_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
            int issued = 0;
            // The operand that holds weights does not depend on the kernel before this one: its
            // tiles of the first STAGES K blocks are requested before waiting for that kernel.
            const int early = constant_operand ? min(num_kb, STAGES) : 0;
            for (int i = 0; i < early; ++i) {
                mbar_expect_tx(full_bar(i), S::STAGE_BYTES);
                const uint32_t a_dst = smem_base + i * S::STAGE_BYTES;
                if (constant_operand == 1) tma_load_2d(a_dst, &map_a, (kb_begin + i) * BK, ra0, full_bar(i));
                else tma_load_2d(a_dst + S::A_BYTES, &map_b, (kb_begin + i) * BK, rb0, full_bar(i));
                issued = i + 1;
            }
            pdl_wait();
            for (int i = 0; i < early; ++i) {
                const uint32_t a_dst = smem_base + i * S::STAGE_BYTES;
                if (constant_operand == 1) tma_load_2d(a_dst + S::A_BYTES, &map_b, (kb_begin + i) * BK, rb0, full_bar(i));
                else tma_load_2d(a_dst, &map_a, (kb_begin + i) * BK, ra0, full_bar(i));
            }
            for (int i = early; i < num_kb && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (i / STAGES) & 1;
                ok = mbar_wait(empty_bar(s), phase ^ 1);
                if (!ok) break;
                mbar_expect_tx(full_bar(s), S::STAGE_BYTES);
                const uint32_t a_dst = smem_base + s * S::STAGE_BYTES;
                tma_load_2d(a_dst, &map_a, (kb_begin + i) * BK, ra0, full_bar(s));
                tma_load_2d(a_dst + S::A_BYTES, &map_b, (kb_begin + i) * BK, rb0, full_bar(s));
                issued = i + 1;
            }
            if (!ok) {
                // do not leave while our own copies are in flight: wait (bounded) for the armed stages
                for (int i = max(0, issued - STAGES); i < issued; ++i)
                    mbar_wait(full_bar(i % STAGES), (i / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BN);
            for (int i = 0; i < num_kb && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (i / STAGES) & 1;
                ok = mbar_wait(full_bar(s), phase);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_base + s * S::STAGE_BYTES;
                const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + S::A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    umma_bf16(tmem_base, desc_step(da, k), desc_step(db, k), idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty_bar(s));       // frees the stage when these MMAs have read it
            }
            if (ok) {
                umma_commit(tmem_full_bar);      // the accumulator is complete
            } else {
                umma_commit(drain_bar);          // leaving early: not before what was issued has run
                mbar_wait(drain_bar, 0);
            }
        }
    } else {
        // epilogue: warp w reads TMEM lanes 32*(w%4) .. +31 = rows of the A operand
        const int quarter = warp & 3;
        const int ra = ra0 + quarter * 32 + lane;
        if (num_kb > 0) ok = mbar_wait(tmem_full_bar, 0);
        else pdl_wait();       // nothing was loaded: still do not write before the previous kernel is done
        tc_fence_after();
        OT* Cz = C + (size_t)blockIdx.z * split_stride;
        if (ok && EPI == 1) {
            if constexpr (EPI == 1 && TRANSPOSED) {
                // lanes 0-15 of a warp hold gate rows, lanes 16-31 the up rows of the same block
                const int out_col = (ra0 + quarter * 32) / 2 + (lane & 15);
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float mine = __uint_as_float(r[j]);
                        const float up = __shfl_down_sync(0xffffffffu, mine, 16);
                        const int rb = rb0 + c0 + j;
                        if (lane < 16 && rb < Rb && 2 * out_col < Ra)
                            store_out<OT>(C + (size_t)rb * ldc + out_col, silu_mul(mine, up));
                    }
                }
            } else if constexpr (EPI == 1) {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t g[16], u[16];     // the loads are warp-wide: every lane takes part
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + c0, g);
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + c0 + 16, u);
                    tmem_ld_wait();
                    if (ra >= Ra) continue;
                    const int oc = (rb0 + c0) / 2;
                    OT* row = C + (size_t)ra * ldc + oc;
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = silu_mul(__uint_as_float(g[j]), __uint_as_float(u[j]));
                    if (rb0 + c0 + 32 <= Rb && ((uintptr_t)row & 15) == 0 && sizeof(OT) == 2) {
                        uint32_t p[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            __nv_bfloat162 t2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                            p[j] = *(uint32_t*)&t2;
                        }
                        *(uint4*)(row) = make_uint4(p[0], p[1], p[2], p[3]);
                        *(uint4*)((uint8_t*)row + 16) = make_uint4(p[4], p[5], p[6], p[7]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (rb0 + c0 + 16 + j < Rb) store_out<OT>(row + j, v[j]);
                    }
                }
            }
        } else if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t r[16];
                if (num_kb > 0) {
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + c0, r);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0;   // an empty split contributes zeros
                }
                if (TRANSPOSED) {
                    // lanes run along ra = the contiguous dimension of C: coalesced per column
                    if (ra < Ra) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int rb = rb0 + c0 + j;
                            if (rb < Rb) store_out<OT>(Cz + (size_t)rb * ldc + ra, __uint_as_float(r[j]));
                        }
                    }
                } else if (ra < Ra) {
                    OT* row = Cz + (size_t)ra * ldc + rb0 + c0;
                    if (rb0 + c0 + 16 <= Rb && ((uintptr_t)row & 15) == 0) {
                        if constexpr (sizeof(OT) == 4) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4)
                                *(uint4*)(row + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                        } else {
                            uint32_t p[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                                p[j] = *(uint32_t*)&v;
                            }
                            *(uint4*)(row) = make_uint4(p[0], p[1], p[2], p[3]);
                            *(uint4*)(row + 8) = make_uint4(p[4], p[5], p[6], p[7]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (rb0 + c0 + j < Rb) store_out<OT>(row + j, __uint_as_float(r[j]));
                    }
                }
            }
        }
    }
    if (!ok && status) atomicOr(status, 4);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}


// ---- persistent variant for more than 64 tokens -------------------------------------------------------
// One CTA per SM; tiles of 128 tokens x bn features (bn = 256 unless the matrix is narrower: a
// 128 x N x 16 MMA with N < 256 is issued no faster than it runs, so narrower tiles only lose).
// Whole rounds of tiles are dealt round-robin, so that the CTAs of a round read neighbouring
// tiles at the same K and share them in L2.  The tiles of the last, incomplete round are not given
// to some CTAs while the others idle: each is cut along K into `ways` equal parts, and the parts
// are dealt round-robin too, part-major, so that the CTAs on one part still walk the same K
// blocks together.  (Contiguous "stream-K" ranges balance better on paper but put every CTA at
// another K: the 7B-shape down projection then read 1.05 GB from memory instead of 0.30 GB.)
// Every holder of a shared tile writes its float32 partial tile to a workspace; when a CTA has
// gone through all its work it comes back to its shared tiles (two at most), waits (bounded) for
// the other holders' parts, and reduces ITS share of the tile's columns: the parts are added in
// the order of their K ranges, so the sum is deterministic.  All CTAs reach that point at about
// the same time, so the waits are short, and all are resident (one per SM), so nobody waits for
// a CTA that cannot run.
// Tensor memory holds TWO accumulators of 256 columns: while the epilogue warps read one, the MMA
// warp fills the other.  A = activations [M, K], B = weights [N, K].
constexpr int P_STAGES = 4;
constexpr int P_BN_MAX = 256;
constexpr int P_FLAG_CAP = 1 << 16;              // tiles the flag array covers
constexpr int P_MAX_CTAS = 160;                  // the workspace has two tiles for each
constexpr uint32_t P_PARTIAL_FLOATS = BM * P_BN_MAX;
struct PSmem {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = P_BN_MAX * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BARRIER_OFFSET = P_STAGES * STAGE_BYTES;
    static constexpr int TOTAL = BARRIER_OFFSET + (2 * P_STAGES + 5) * 8 + 16 + 1024;
};

// Epilogue 2: the tile is a run of tokens x two (head size 128) or four (head size 64) heads of the
// stacked q/k/v product.  Instead of storing it, the epilogue adds the bias, rotates the first
// `rdim` elements of q and k heads by the token's row of a cos/sin table (half-split pairs
// i, i + rdim/2 as in mini_hisparse/model.py:141-151, or interleaved pairs 2i, 2i + 1), and writes
// q as bfloat16 and k, v into the token's page of the KV cache (model.py:169-170): no float32
// q/k/v matrix goes to memory and no separate pass reads it back.
struct QkvRopeArgs {
    const float* bias;          // [(nq + 2 nkv) d] or null
    const float* cos_sin;       // [T, rdim]: cos of the rdim/2 angles, then sin (unused if rdim == 0)
    int rdim, interleaved;      // rotated elements per head (multiple of 32, or of 16 if interleaved)
    const int* positions;       // [T]
    const int* tok_seg;         // [T]
    const int* block_table;     // [segments, table_width]
    __nv_bfloat16* q_out;       // [T, nq d]
    __nv_bfloat16* cache;       // [pages, 2, nkv, P, d]
    int table_width, nq, nkv, d, P, num_pages, write_kv;
};

// Store one unit of a row of a tile: 16 sums (or, for the SwiGLU epilogue, 16 gate and 16 up sums) at
// columns c0.. of the tile whose first column is rb0.
template <typename OT, int EPI>
__device__ __forceinline__ void emit_unit(OT* __restrict__ C, long long ldc, int Ra, int Rb, int ra, int rb0, int c0,
                                          const uint32_t (&r)[16], const uint32_t (&r2)[16]) {
    if (ra >= Ra) return;
    if constexpr (EPI == 1) {
        OT* row = C + (size_t)ra * ldc + (rb0 + c0) / 2;
        float v[16];
#pragma unroll
        for (int x = 0; x < 16; ++x) v[x] = silu_mul(__uint_as_float(r[x]), __uint_as_float(r2[x]));
        if (rb0 + c0 + 32 <= Rb && ((uintptr_t)row & 15) == 0 && sizeof(OT) == 2) {
            uint32_t p[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                __nv_bfloat162 t2 = __floats2bfloat162_rn(v[2 * x], v[2 * x + 1]);
                p[x] = *(uint32_t*)&t2;
            }
            *(uint4*)(row) = make_uint4(p[0], p[1], p[2], p[3]);
            *(uint4*)((uint8_t*)row + 16) = make_uint4(p[4], p[5], p[6], p[7]);
        } else {
#pragma unroll
            for (int x = 0; x < 16; ++x)
                if (rb0 + c0 + 16 + x < Rb) store_out<OT>(row + x, v[x]);
        }
    } else {
        OT* row = C + (size_t)ra * ldc + rb0 + c0;
        if (rb0 + c0 + 16 <= Rb && ((uintptr_t)row & 15) == 0) {
            if constexpr (sizeof(OT) == 4) {
#pragma unroll
                for (int x = 0; x < 16; x += 4)
                    *(uint4*)(row + x) = make_uint4(r[x], r[x + 1], r[x + 2], r[x + 3]);
            } else {
                uint32_t p[8];
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    __nv_bfloat162 v2 = __floats2bfloat162_rn(__uint_as_float(r[2 * x]), __uint_as_float(r[2 * x + 1]));
                    p[x] = *(uint32_t*)&v2;
                }
                *(uint4*)(row) = make_uint4(p[0], p[1], p[2], p[3]);
                *(uint4*)(row + 8) = make_uint4(p[4], p[5], p[6], p[7]);
            }
        } else {
#pragma unroll
            for (int x = 0; x < 16; ++x)
                if (rb0 + c0 + x < Rb) store_out<OT>(row + x, __uint_as_float(r[x]));
        }
    }
}

// The epilogue of one whole tile: this thread's row (row_in_tile of the 128 rows at ra0) of the accumulator at
// `acc` (tensor memory, this warp's lanes) goes to C, through the SwiGLU gate (EPI 1), or, rotated, to q and
// the cache pages (EPI 2).
template <typename OT, int EPI>
__device__ __forceinline__ void store_tile(uint32_t acc, int ra0, int rb0, int bn, int row_in_tile, OT* __restrict__ C,
                                           long long ldc, int Ra, int Rb, const QkvRopeArgs& qr,
                                           int* __restrict__ status) {
    constexpr int UNIT = EPI == 1 ? 32 : 16;        // columns that are stored together
    if constexpr (EPI == 2) {
        const int ra = ra0 + row_in_tile;
        const bool live = ra < Ra;
        const int d = qr.d, rdim = qr.rdim, half = rdim >> 1;
        const int pos = live ? qr.positions[ra] : 0;
        const float* cs = qr.cos_sin + (size_t)(live ? ra : 0) * rdim;
        const int head0 = rb0 / d;
        int page = -1;
        if (live && qr.write_kv && head0 + bn / d > qr.nq) {        // the tile holds k or v heads
            page = qr.block_table[(size_t)qr.tok_seg[ra] * qr.table_width + pos / qr.P];
            if (page < 0 || page >= qr.num_pages) {                 // never write outside the pool
                if (status) atomicOr(status, 2);
                page = -1;
            }
        }
        const int within = pos % qr.P;
        const int total_heads = qr.nq + 2 * qr.nkv;
        auto head_dst = [&](int head) -> __nv_bfloat16* {
            return head < qr.nq ? qr.q_out + (size_t)ra * qr.nq * d + head * d
                                : qr.cache + ((((size_t)page * 2 + 0) * qr.nkv + (head - qr.nq)) * qr.P + within) * d;
        };
        auto load_bias16 = [&](float (&b)[16], int col) {
            if (qr.bias) {
#pragma unroll
                for (int x = 0; x < 4; ++x) *(float4*)(b + 4 * x) = *(const float4*)(qr.bias + col + 4 * x);
            } else {
#pragma unroll
                for (int x = 0; x < 16; ++x) b[x] = 0.f;
            }
        };
        auto store16 = [&](__nv_bfloat16* dst, const float (&v)[16]) {
            uint32_t pk[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                __nv_bfloat162 t2 = __floats2bfloat162_rn(v[2 * x], v[2 * x + 1]);
                pk[x] = *(uint32_t*)&t2;
            }
            *(uint4*)(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            *(uint4*)(dst + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        };
        // rotated heads: the chunk of angles is the outer loop, so that a row's cos and
        // sin are fetched once (16-byte loads) for all heads of the tile
        if (!qr.interleaved) {
#pragma unroll 1
            for (int c = 0; c < half; c += 16) {
                float4 cs4[4], sn4[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    cs4[x] = *(const float4*)(cs + c + 4 * x);
                    sn4[x] = *(const float4*)(cs + half + c + 4 * x);
                }
                const float* cf = (const float*)cs4;
                const float* sf = (const float*)sn4;
#pragma unroll 1
                for (int hh = 0; hh < bn / d; ++hh) {
                    const int head = head0 + hh;
                    if (head >= qr.nq + qr.nkv) break;               // value heads and the edge: below
                    const bool is_q = head < qr.nq;
                    uint32_t ra16[16], rb16[16];
                    tmem_ld16(acc + hh * d + c, ra16);
                    tmem_ld16(acc + hh * d + half + c, rb16);
                    tmem_ld_wait();
                    if (!live || (!is_q && page < 0)) continue;
                    __nv_bfloat16* dst = head_dst(head);
                    float ba[16], bb[16], oa[16], ob[16];
                    load_bias16(ba, head * d + c);
                    load_bias16(bb, head * d + half + c);
#pragma unroll
                    for (int x = 0; x < 16; ++x) {
                        const float a0 = __uint_as_float(ra16[x]) + ba[x], b0 = __uint_as_float(rb16[x]) + bb[x];
                        oa[x] = a0 * cf[x] - b0 * sf[x];
                        ob[x] = b0 * cf[x] + a0 * sf[x];
                    }
                    store16(dst + c, oa);
                    store16(dst + half + c, ob);
                }
            }
        } else {
#pragma unroll 1
            for (int c = 0; c < rdim; c += 16) {        // 16 columns = 8 pairs = angles c/2 .. c/2 + 7
                float4 cs4[2], sn4[2];
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    cs4[x] = *(const float4*)(cs + (c >> 1) + 4 * x);
                    sn4[x] = *(const float4*)(cs + half + (c >> 1) + 4 * x);
                }
                const float* cf = (const float*)cs4;
                const float* sf = (const float*)sn4;
#pragma unroll 1
                for (int hh = 0; hh < bn / d; ++hh) {
                    const int head = head0 + hh;
                    if (head >= qr.nq + qr.nkv) break;
                    const bool is_q = head < qr.nq;
                    uint32_t r16[16];
                    tmem_ld16(acc + hh * d + c, r16);
                    tmem_ld_wait();
                    if (!live || (!is_q && page < 0)) continue;
                    float bv[16], o[16];
                    load_bias16(bv, head * d + c);
#pragma unroll
                    for (int x = 0; x < 8; ++x) {
                        const float a0 = __uint_as_float(r16[2 * x]) + bv[2 * x], b0 = __uint_as_float(r16[2 * x + 1]) + bv[2 * x + 1];
                        o[2 * x] = a0 * cf[x] - b0 * sf[x];
                        o[2 * x + 1] = b0 * cf[x] + a0 * sf[x];
                    }
                    store16(head_dst(head) + c, o);
                }
            }
        }
        // the elements of q and k heads behind the rotated ones: bias only
#pragma unroll 1
        for (int c = rdim; c < d; c += 16) {
#pragma unroll 1
            for (int hh = 0; hh < bn / d; ++hh) {
                const int head = head0 + hh;
                if (head >= qr.nq + qr.nkv) break;
                uint32_t r16[16];
                tmem_ld16(acc + hh * d + c, r16);
                tmem_ld_wait();
                if (!live || (head >= qr.nq && page < 0)) continue;
                float bv[16], o[16];
                load_bias16(bv, head * d + c);
#pragma unroll
                for (int x = 0; x < 16; ++x) o[x] = __uint_as_float(r16[x]) + bv[x];
                store16(head_dst(head) + c, o);
            }
        }
        // value heads: bias, no rotation
#pragma unroll 1
        for (int hh = 0; hh < bn / d; ++hh) {
            const int head = head0 + hh;
            if (head < qr.nq + qr.nkv) continue;
            if (head >= total_heads) break;
            const int col0 = head * d;
            __nv_bfloat16* dst = qr.cache + ((((size_t)(page < 0 ? 0 : page) * 2 + 1) * qr.nkv + (head - qr.nq - qr.nkv)) * qr.P + within) * d;
#pragma unroll 1
            for (int c = 0; c < d; c += 16) {
                uint32_t r[16];
                tmem_ld16(acc + hh * d + c, r);
                tmem_ld_wait();
                if (page < 0) continue;
                float bv[16];
                if (qr.bias) {
#pragma unroll
                    for (int x = 0; x < 4; ++x) *(float4*)(bv + 4 * x) = *(const float4*)(qr.bias + col0 + c + 4 * x);
                } else {
#pragma unroll
                    for (int x = 0; x < 16; ++x) bv[x] = 0.f;
                }
                uint32_t pk[8];
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(r[2 * x]) + bv[2 * x], __uint_as_float(r[2 * x + 1]) + bv[2 * x + 1]);
                    pk[x] = *(uint32_t*)&t2;
                }
                *(uint4*)(dst + c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *(uint4*)(dst + c + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
        }
    } else {
#pragma unroll 1
        for (int c0 = 0; c0 < bn; c0 += UNIT) {
            uint32_t r[16], r2[16];
            tmem_ld16(acc + c0, r);
            if constexpr (EPI == 1) tmem_ld16(acc + c0 + 16, r2);
            tmem_ld_wait();
            emit_unit<OT, EPI>(C, ldc, Ra, Rb, ra0 + row_in_tile, rb0, c0, r, r2);
        }
    }
}

template <typename OT, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          OT* __restrict__ C, int Ra, int Rb, int K, long long ldc, int bn, int tiles_m,
                          int whole_tiles, int tail_tiles, int ways, float* __restrict__ partials,
                          int* __restrict__ flags, int* __restrict__ status, const QkvRopeArgs qr,
                          const uint32_t wait_limit) {
    using S = PSmem;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + S::BARRIER_OFFSET;
    auto full_bar = [&](int s) { return bar_base + 8 * s; };
    auto empty_bar = [&](int s) { return bar_base + 8 * (P_STAGES + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8 * (2 * P_STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8 * (2 * P_STAGES + 2 + b); };
    const uint32_t drain_bar = bar_base + 8 * (2 * P_STAGES + 4);       // only used when a wait has run out
    uint32_t* tmem_slot = (uint32_t*)(smem + S::BARRIER_OFFSET + 8 * (2 * P_STAGES + 5));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_kb = (K + BK - 1) / BK;
    // First the ways * tail_tiles parts of the tiles [whole_tiles, + tail_tiles) (entry e is part
    // e / tail_tiles of tile e % tail_tiles), then the tiles [0, whole_tiles) as whole tiles, both
    // round-robin.  The parts come first so that their exchange and reduction (the epilogue warps'
    // business) happen while the MMA warp is busy with the whole tiles, not at the kernel's end.
    const int entries = tail_tiles * ways;
    const int my_parts = entries > (int)blockIdx.x ? (entries - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    // segment j of this CTA: a tile, a range of its K blocks and, for a part, its entry (else -1)
    auto segment = [&](int j, int& t, int& kb0, int& kb1, int& entry) -> bool {
        if (j < my_parts) {
            const int e = (int)blockIdx.x + j * (int)gridDim.x;
            const int part = e / tail_tiles;
            t = whole_tiles + e % tail_tiles;
            kb0 = (int)((long long)part * total_kb / ways);
            kb1 = (int)((long long)(part + 1) * total_kb / ways);
            entry = ways > 1 ? e : -1;
            return true;
        }
        const long long whole = (long long)blockIdx.x + (long long)(j - my_parts) * gridDim.x;
        if (whole >= whole_tiles) return false;
        t = (int)whole; kb0 = 0; kb1 = total_kb; entry = -1;
        return true;
    };
    const uint32_t stage_tx = S::A_BYTES + bn * BK * 2;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full_bar(b), 1); mbar_init(acc_empty_bar(b), 4); }
        mbar_init(drain_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
            // The weights are constant: the weight tiles of the first stages are asked for while the
            // kernel before this one still runs; the activations only after it has finished.
            int it = 0, t, kb0, kb1, entry, early = 0;
            if (segment(0, t, kb0, kb1, entry)) {
                const int rb0 = (t / tiles_m) * bn;
                for (int kb = kb0; kb < kb1 && early < P_STAGES; ++kb, ++early) {
                    mbar_expect_tx(full_bar(early), stage_tx);
                    tma_load_2d(smem_base + early * S::STAGE_BYTES + S::A_BYTES, &map_b, kb * BK, rb0, full_bar(early));
                }
            }
            pdl_wait();
            for (int j = 0; ok && segment(j, t, kb0, kb1, entry); ++j) {
                const int ra0 = (t % tiles_m) * BM, rb0 = (t / tiles_m) * bn;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % P_STAGES;
                    const uint32_t a_dst = smem_base + s * S::STAGE_BYTES;
                    if (it < early) {                   // the weight tile is on its way already
                        tma_load_2d(a_dst, &map_a, kb * BK, ra0, full_bar(s));
                        continue;
                    }
                    ok = mbar_wait(empty_bar(s), ((it / P_STAGES) & 1) ^ 1, wait_limit);
                    if (!ok) break;
                    mbar_expect_tx(full_bar(s), stage_tx);
                    tma_load_2d(a_dst, &map_a, kb * BK, ra0, full_bar(s));
                    tma_load_2d(a_dst + S::A_BYTES, &map_b, kb * BK, rb0, full_bar(s));
                }
            }
            // nothing of ours may still be in flight when the CTA leaves: wait for the last stages
            for (int back = 1; back <= P_STAGES && back <= it; ++back) {
                const int i = it - back;
                mbar_wait(full_bar(i % P_STAGES), (i / P_STAGES) & 1, wait_limit);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc(bn);
            // the operand descriptors of stage 0, built once; stage s is S::STAGE_BYTES / 16 address units on
            const uint64_t desc_a0 = make_smem_desc(smem_base), desc_b0 = make_smem_desc(smem_base + S::A_BYTES);
            int it = 0, t, kb0, kb1, entry;
            for (int j = 0; ok && segment(j, t, kb0, kb1, entry); ++j) {
                const int b = j & 1;
                ok = mbar_wait(acc_empty_bar(b), ((j >> 1) & 1) ^ 1, wait_limit);     // the epilogue has read this buffer
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + b * P_BN_MAX;
                // The first shared-memory access after an MMA or a commit stalls this thread for some
                // 250 cycles; a second look right behind it is cheap.  So when the next stage has
                // landed as well, both are issued in one round (never waiting for the second).
                for (int kb = kb0; kb < kb1 && ok;) {
                    const int s0 = it % P_STAGES, s1 = (it + 1) % P_STAGES;
                    ok = mbar_wait(full_bar(s0), (it / P_STAGES) & 1, wait_limit);
                    if (!ok) break;
                    const int n = (kb1 - kb >= 2 && mbar_test(full_bar(s1), ((it + 1) / P_STAGES) & 1)) ? 2 : 1;
                    tc_fence_after();
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (h < n) {
                            const uint64_t step = (uint64_t)((h ? s1 : s0) * (S::STAGE_BYTES / 16));
                            const uint64_t da = desc_a0 + step, db = desc_b0 + step;
#pragma unroll
                            for (int k = 0; k < BK / UMMA_K; ++k)
                                umma_bf16(acc, desc_step(da, k), desc_step(db, k), idesc, (kb + h > kb0 || k > 0) ? 1u : 0u);
                            umma_commit(empty_bar(h ? s1 : s0));
                        }
                    }
                    kb += n;
                    it += n;
                }
                if (ok) umma_commit(acc_full_bar(b));
            }
            if (!ok) {
                umma_commit(drain_bar);          // leaving early: not before what was issued has run
                mbar_wait(drain_bar, 0, wait_limit);
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        constexpr int UNIT = EPI == 1 ? 32 : 16;        // columns that are stored together
        // ---- second pass: the shared tiles.  The CTAs that hold parts of a tile divide its columns
        // among themselves; each adds the parts in the order of their K ranges and stores. ---------
        auto reduce_shared = [&](const int (&shared_entry)[2], int shared_count) {
        for (int i = 0; i < shared_count && ok; ++i) {
            const int tail_index = shared_entry[i] % tail_tiles, rank = shared_entry[i] / tail_tiles;
            const int ts = whole_tiles + tail_index, parts = ways;
            const volatile int* flag = flags + 4 * ts + quarter;
            uint32_t spins = 0;
            while (*flag < parts && ++spins < wait_limit) __nanosleep(32);
            if (spins >= wait_limit) { ok = false; break; }
            __threadfence();
            const int ra0 = (ts % tiles_m) * BM, rb0 = (ts / tiles_m) * bn;
#pragma unroll 1
            for (int c0 = rank * UNIT; c0 < bn; c0 += parts * UNIT) {
                float s[16], s2[16];
#pragma unroll
                for (int x = 0; x < 16; ++x) s[x] = s2[x] = 0.f;
                // the loads of several parts are in flight together; the sums stay in the parts' order
                constexpr int BATCH = EPI == 1 ? 2 : 4;
                for (int p0 = 0; p0 < parts; p0 += BATCH) {
                    uint4 v[BATCH][4], w[EPI == 1 ? BATCH : 1][4];
#pragma unroll
                    for (int q = 0; q < BATCH; ++q) {
                        const int p = p0 + q < parts ? p0 + q : parts - 1;
                        const int e = p * tail_tiles + tail_index;        // part p of this tile: its CTA and slot
                        const float* src = partials + (size_t)(2 * (e % (int)gridDim.x) + e / (int)gridDim.x) * P_PARTIAL_FLOATS;
                        const uint4* a = (const uint4*)(src + ((size_t)(c0 >> 4) * BM + row_in_tile) * 16);
#pragma unroll
                        for (int x = 0; x < 4; ++x) v[q][x] = __ldcg(a + x);
                        if constexpr (EPI == 1) {
#pragma unroll
                            for (int x = 0; x < 4; ++x) w[q][x] = __ldcg(a + BM * 4 + x);    // the next 16 columns: the up half
                        }
                    }
#pragma unroll
                    for (int q = 0; q < BATCH; ++q) {
                        if (p0 + q < parts) {
#pragma unroll
                            for (int x = 0; x < 4; ++x) {
                                s[4 * x] += __uint_as_float(v[q][x].x); s[4 * x + 1] += __uint_as_float(v[q][x].y);
                                s[4 * x + 2] += __uint_as_float(v[q][x].z); s[4 * x + 3] += __uint_as_float(v[q][x].w);
                            }
                            if constexpr (EPI == 1) {
#pragma unroll
                                for (int x = 0; x < 4; ++x) {
                                    s2[4 * x] += __uint_as_float(w[q][x].x); s2[4 * x + 1] += __uint_as_float(w[q][x].y);
                                    s2[4 * x + 2] += __uint_as_float(w[q][x].z); s2[4 * x + 3] += __uint_as_float(w[q][x].w);
                                }
                            }
                        }
                    }
                }
                uint32_t r[16], r2[16];
#pragma unroll
                for (int x = 0; x < 16; ++x) { r[x] = __float_as_uint(s[x]); r2[x] = __float_as_uint(s2[x]); }
                emit_unit<OT, EPI>(C, ldc, Ra, Rb, ra0 + row_in_tile, rb0, c0, r, r2);
            }
            __syncwarp();
            // the last quarter-warp to have read puts the counter back to zero for the next launch
            if (lane == 0 && atomicAdd(flags + 4 * ts + quarter, 1) == 2 * parts - 1) flags[4 * ts + quarter] = 0;
        }
        };
        // ---- first pass: every segment; a tile that is shared goes to the workspace ----------------
        int shared_entry[2], shared_count = 0;
        bool reduced = false;
        int t, kb0, kb1, entry;
        for (int j = 0; ok && (j < my_parts || !reduced || segment(j, t, kb0, kb1, entry)); ++j) {
            if (j >= my_parts && !reduced) {
                // all of this CTA's parts are in the workspace: reduce its share of the shared tiles
                // now, while the MMA warp works on the first whole tile
                reduce_shared(shared_entry, shared_count);
                reduced = true;
                --j;
                continue;
            }
            if (j < my_parts) segment(j, t, kb0, kb1, entry);
            const int b = j & 1;
            const int ra0 = (t % tiles_m) * BM, rb0 = (t / tiles_m) * bn;
            ok = mbar_wait(acc_full_bar(b), (j >> 1) & 1, wait_limit);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + b * P_BN_MAX;
            if (entry >= 0) {
                // a part of a shared tile: this CTA's first part goes to its slot 0, its second to slot 1
                float* mine = partials + (size_t)(2 * blockIdx.x + entry / (int)gridDim.x) * P_PARTIAL_FLOATS;
#pragma unroll 1
                for (int c0 = 0; c0 < bn; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(acc + c0, r);
                    tmem_ld_wait();
                    uint4* dst = (uint4*)(mine + ((size_t)(c0 >> 4) * BM + row_in_tile) * 16);
#pragma unroll
                    for (int x = 0; x < 4; ++x) dst[x] = make_uint4(r[4 * x], r[4 * x + 1], r[4 * x + 2], r[4 * x + 3]);
                }
                tc_fence_before();
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_plain(acc_empty_bar(b));
                    atomicAdd(flags + 4 * t + quarter, 1);      // this quarter of the rows has landed
                }
                if (shared_count < 2) shared_entry[shared_count++] = entry;
                continue;
            }
            store_tile<OT, EPI>(acc, ra0, rb0, bn, row_in_tile, C, ldc, Ra, Rb, qr, status);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(acc_empty_bar(b));    // this warp has read its quarter
        }
    }
    if (!ok && status) atomicOr(status, 4);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---- two SMs on one tile ---------------------------------------------------------------------------------
// The persistent kernel above is paced by shared memory, not by the tensor pipe: per K block of 64 a CTA's
// TMA writes 48 KB into shared memory and its MMAs read 48 KB back, some 190 bytes a cycle against the 512
// cycles the four 128 x 256 x 16 MMAs take (measured: 600 to 670 cycles per K block).  Here two CTAs on
// neighbouring SMs (a cluster of two) share a tile of 256 tokens x bn features: tcgen05.mma with
// cta_group::2 multiplies each CTA's 128 rows of activations by ALL bn weight rows, of which each CTA holds
// and loads only half; the tensor cores fetch the other half from the partner's shared memory.  A K block
// is 32 KB per CTA instead of 48.
//   * every CTA loads its halves with cp.async.bulk.tensor ... .cta_group::2 (no multicast) whose bytes are
//     counted by the full barrier of the pair's first CTA (the leader), which alone arms it;
//   * the leader's MMA thread issues for both, and commits with tcgen05.commit ... .multicast::cluster to the
//     barriers of both CTAs (stage free, accumulator complete);
//   * both CTAs' epilogue warps read their own 128 lanes of tensor memory and tell the LEADER's barrier when
//     an accumulator may be overwritten (mbarrier.arrive on the leader's shared memory);
//   * tensor memory is allocated and freed with cta_group::2 by the same warp of both CTAs, and a cluster
//     barrier before the end keeps either CTA's shared and tensor memory alive while the other may use it.
// Whole tiles only (no sharing of a tile's K range); every wait is bounded as above.
//
// A stage of the ring holds one or two K blocks of 64 (`kbs`).  The thread that issues the MMAs pays some
// 250 cycles for the barrier it looks at before a stage, whatever the stage holds: with tiles 256 wide
// the four MMAs of one K block (512 cycles) hide that, with narrower tiles they do not (a K block took
// some 600 cycles at any width).  Two K blocks per stage halve the looks, so a tile half as wide takes
// about half as long, and tile widths that fill one round of pairs (few tokens, short weight matrices)
// pay off.  The ring has as many stages as fit (at most PAIR_MAX_STAGES); a stage is
// [A block 0 | A block 1 | B block 0 | B block 1] with each CTA's half of the B rows.
constexpr int PAIR_MAX_STAGES = 8;
constexpr int PAIR_DATA_BYTES = 216 * 1024;     // operand stages of one CTA
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;     // clears the bit that tells the pair's second CTA from its first
struct PairSmem {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int BARRIER_OFFSET = PAIR_DATA_BYTES;
    static constexpr int TOTAL = BARRIER_OFFSET + (2 * PAIR_MAX_STAGES + 5) * 8 + 16 + 1024;
};
struct PairRing {
    int kbs;                 // K blocks of 64 per stage: 1 or 2
    int stages;              // stages in the ring
    uint32_t stage_bytes;    // kbs * (A_BYTES + half_bn * 128)
};

__device__ __forceinline__ uint32_t pair_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void pair_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// a tile for this CTA's shared memory whose bytes are counted by `bar`, which may be the partner's
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
}
// arrive on the barrier at this offset in BOTH CTAs when every MMA issued so far has completed
__device__ __forceinline__ void umma_commit_both(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & PEER_MASK) : "memory");
}
// D float32, A and B bfloat16, both K-major, M = 256 over the two CTAs, N = bn
__host__ __device__ constexpr uint32_t make_idesc_pair(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <typename OT, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    OT* __restrict__ C, int Ra, int Rb, int K, long long ldc, int bn, int tiles_m, int num_tiles,
                    const PairRing ring, int* __restrict__ status, const QkvRopeArgs qr,
                    const uint32_t wait_limit) {
    using S = PairSmem;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + S::BARRIER_OFFSET;
    auto full_bar = [&](int s) { return bar_base + 8 * s; };                                  // the leader's counts
    auto empty_bar = [&](int s) { return bar_base + 8 * (PAIR_MAX_STAGES + s); };                 // each CTA's own
    auto acc_full_bar = [&](int b) { return bar_base + 8 * (2 * PAIR_MAX_STAGES + b); };          // each CTA's own
    auto acc_empty_bar = [&](int b) { return bar_base + 8 * (2 * PAIR_MAX_STAGES + 2 + b); };     // the leader's counts
    const uint32_t drain_bar = bar_base + 8 * (2 * PAIR_MAX_STAGES + 4);
    uint32_t* tmem_slot = (uint32_t*)(smem + S::BARRIER_OFFSET + 8 * (2 * PAIR_MAX_STAGES + 5));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)pair_rank();
    const bool leader = rank == 0;
    const int pair = (int)blockIdx.x >> 1, npairs = (int)gridDim.x >> 1;
    const int total_kb = (K + BK - 1) / BK;
    const int half_bn = bn >> 1;
    const int kbs = ring.kbs, nstages = ring.stages;
    const int total_st = (total_kb + kbs - 1) / kbs;              // stages a tile takes (the last may hold a K block of zeros)
    const uint32_t b_bytes = half_bn * BK * 2;                    // this CTA's rows of one K block of the weights
    const uint32_t half_tx = kbs * (S::A_BYTES + b_bytes);        // what one CTA loads per stage
    const uint32_t b_offset = kbs * S::A_BYTES;                   // the weights' place in a stage

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_MAX_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full_bar(b), 1); mbar_init(acc_empty_bar(b), 8); }
        mbar_init(drain_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    pair_sync();            // the partner's barriers exist before anything is sent to them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
            const uint32_t count_bar0 = full_bar(0) & PEER_MASK;      // the leader's barrier of stage 0
            int it = 0, early = 0;
            // the weight halves of the first stages are asked for while the kernel before this one still runs
            // (a K block beyond the matrix is a box outside the tensor map: zeros, counted like any other)
            if (pair < num_tiles) {
                const int rbh0 = (pair / tiles_m) * bn + rank * half_bn;
                for (int st = 0; st < total_st && early < nstages; ++st, ++early) {
                    if (leader) mbar_expect_tx(full_bar(early), 2 * half_tx);
                    for (int kk = 0; kk < kbs; ++kk)
                        tma_load_2d_pair(smem_base + early * ring.stage_bytes + b_offset + kk * b_bytes, &map_b,
                                         (st * kbs + kk) * BK, rbh0, count_bar0 + 8 * early);
                }
            }
            pdl_wait();
            // (the stage and its turn of the ring are counted, not divided out: this thread's loop is what
            // feeds the tensor pipe, and a division by a run-time number costs it dozens of cycles)
            int s = 0;
            uint32_t turn = 0;
            for (int t = pair; ok && t < num_tiles; t += npairs) {
                const int ra0 = (t % tiles_m) * 2 * BM + rank * BM, rbh0 = (t / tiles_m) * bn + rank * half_bn;
                for (int st = 0; st < total_st; ++st, ++it, turn ^= (s + 1 == nstages), s = (s + 1 == nstages) ? 0 : s + 1) {
                    const uint32_t a_dst = smem_base + s * ring.stage_bytes;
                    if (it < early) {                   // the weight half is on its way already
                        for (int kk = 0; kk < kbs; ++kk)
                            tma_load_2d_pair(a_dst + kk * S::A_BYTES, &map_a, (st * kbs + kk) * BK, ra0, count_bar0 + 8 * s);
                        continue;
                    }
                    ok = mbar_wait(empty_bar(s), turn ^ 1, wait_limit);
                    if (!ok) break;
                    if (leader) mbar_expect_tx(full_bar(s), 2 * half_tx);
                    for (int kk = 0; kk < kbs; ++kk) {
                        tma_load_2d_pair(a_dst + kk * S::A_BYTES, &map_a, (st * kbs + kk) * BK, ra0, count_bar0 + 8 * s);
                        tma_load_2d_pair(a_dst + b_offset + kk * b_bytes, &map_b, (st * kbs + kk) * BK, rbh0, count_bar0 + 8 * s);
                    }
                }
            }
            // nothing may still be in flight when the CTAs leave: the leader's barriers count both CTAs' bytes
            if (leader)
                for (int back = 1; back <= nstages && back <= it; ++back) {
                    const int i = it - back;
                    mbar_wait(full_bar(i % nstages), (i / nstages) & 1, wait_limit);
                }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            const uint32_t idesc = make_idesc_pair(bn);
            const uint64_t desc_a0 = make_smem_desc(smem_base), desc_b0 = make_smem_desc(smem_base + b_offset);
            const uint64_t a_step = (uint64_t)(S::A_BYTES / 16), b_step = (uint64_t)(b_bytes / 16);
            const uint64_t stage_step = (uint64_t)(ring.stage_bytes / 16);
            int j = 0, s = 0;
            uint32_t turn = 0;
            uint64_t step = 0;
            for (int t = pair; ok && t < num_tiles; t += npairs, ++j) {
                const int b = j & 1;
                ok = mbar_wait(acc_empty_bar(b), ((j >> 1) & 1) ^ 1, wait_limit);     // both epilogues have read this buffer
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + b * P_BN_MAX;
                for (int st = 0; st < total_st; ++st) {
                    ok = mbar_wait(full_bar(s), turn, wait_limit);
                    if (!ok) break;
                    tc_fence_after();
                    uint64_t da = desc_a0 + step, db = desc_b0 + step;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(acc, desc_step(da, k), desc_step(db, k), idesc, (st > 0 || k > 0) ? 1u : 0u);
                    if (kbs > 1) {
                        da += a_step;
                        db += b_step;
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            umma_bf16_pair(acc, desc_step(da, k), desc_step(db, k), idesc, 1u);
                    }
                    umma_commit_both(empty_bar(s));         // frees the stage in both CTAs
                    if (++s == nstages) { s = 0; turn ^= 1; step = 0; } else { step += stage_step; }
                }
                if (!ok) break;
                umma_commit_both(acc_full_bar(b));          // the accumulator is complete in both CTAs
            }
            if (!ok) {
                umma_commit_pair(drain_bar);                // leaving early: not before what was issued has run
                mbar_wait(drain_bar, 0, wait_limit);
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        int j = 0;
        for (int t = pair; ok && t < num_tiles; t += npairs, ++j) {
            const int b = j & 1;
            const int ra0 = (t % tiles_m) * 2 * BM + rank * BM, rb0 = (t / tiles_m) * bn;
            ok = mbar_wait(acc_full_bar(b), (j >> 1) & 1, wait_limit);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + b * P_BN_MAX;
            store_tile<OT, EPI>(acc, ra0, rb0, bn, row_in_tile, C, ldc, Ra, Rb, qr, status);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(acc_empty_bar(b));    // this warp has read its quarter
        }
    }
    if (!ok && status) atomicOr(status, 4);
    tc_fence_before();
    __syncthreads();
    pair_sync();            // the partner may still read this CTA's shared memory or write its tensor memory
    if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

// ---- host: tensor maps ----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// A [rows, K] bfloat16 matrix with row stride ld (elements); box = box_rows x 64, 128-byte swizzle,
// zeros outside the matrix.
int make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    typedef std::tuple<const void*, long long, long long, long long, int> Key;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    Key key(ptr, rows, K, ld, box_rows);
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *map = it->second; return 0; }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail("gemm_tc: the driver has no cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("gemm_tc: cuTensorMapEncodeTiled failed with code %d (rows %lld, K %lld, ld %lld)",
                                       (int)r, rows, K, ld);
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *map;
    return 0;
}

template <int BN, int STAGES, bool TRANSPOSED, typename OT, int EPI>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* C, int Ra, int Rb, int K, long long ldc,
           int nsplit, int kb_per_split, long long split_stride, int constant_operand, int* status,
           cudaStream_t stream) {
    auto kern = gemm_tc_kernel<BN, STAGES, TRANSPOSED, OT, EPI>;
    constexpr int smem = Smem<BN, STAGES>::TOTAL;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail("gemm_tc: cannot set %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((Ra + BM - 1) / BM, (Rb + BN - 1) / BN, nsplit);
    launch_kernel(kern, grid, dim3(THREADS), smem, stream, ma, mb, (OT*)C, Ra, Rb, K, ldc, kb_per_split,
                  split_stride, constant_operand, status);
    return check_launch("gemm_tc");
}

template <bool TRANSPOSED, typename OT, int EPI>
int dispatch_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, void* C, int Ra, int Rb, int K,
                long long ldc, int nsplit, int kbps, long long ss, int co, int* status, cudaStream_t st) {
    switch (bn) {
        // the narrow tiles stream weights: two CTAs per SM (<= 112 KB each) overlap one CTA's
        // start-up and epilogue with the other's loads
        case 16:
            if (EPI == 1 && !TRANSPOSED) break;      // the SwiGLU epilogue pairs 16 + 16 columns
            return launch<16, 6, TRANSPOSED, OT, EPI>(ma, mb, C, Ra, Rb, K, ldc, nsplit, kbps, ss, co, status, st);
        case 32: return launch<32, 5, TRANSPOSED, OT, EPI>(ma, mb, C, Ra, Rb, K, ldc, nsplit, kbps, ss, co, status, st);
        case 64: return launch<64, 4, TRANSPOSED, OT, EPI>(ma, mb, C, Ra, Rb, K, ldc, nsplit, kbps, ss, co, status, st);
        case 128: return launch<128, 6, TRANSPOSED, OT, EPI>(ma, mb, C, Ra, Rb, K, ldc, nsplit, kbps, ss, co, status, st);
        case 256: return launch<256, 4, TRANSPOSED, OT, EPI>(ma, mb, C, Ra, Rb, K, ldc, nsplit, kbps, ss, co, status, st);
    }
    return fail("gemm_tc: no tile for BN %d", bn);
}

// Iterations a bounded wait of the persistent product may take; tests shorten it to see a wait run out.
uint32_t g_wait_limit = WAIT_LIMIT;

// MHB_GEMM_PAIR=0 in the environment keeps every tile on one SM (the kernel with cta_group::1 only).
inline bool pair_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("MHB_GEMM_PAIR");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

// MHB_GEMM_KBS=1|2 in the environment fixes the K blocks per stage of the two-SM kernel (default: by tile width).
inline int pair_kbs() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("MHB_GEMM_KBS");
        v = (e && (e[0] == '1' || e[0] == '2')) ? e[0] - '0' : 0;
    }
    return v;
}

// Tile width (multiple of 16, 128..256; for the SwiGLU epilogue a multiple of 32) that wastes the
// least of the last round of whole tiles on `sms` persistent CTAs.
int choose_persistent_bn(int tiles_m, int N, int sms, int step) {
    int best = 256;
    double best_cost = 1e30;
    for (int bn = 256; bn >= 128; bn -= step) {
        const int tiles = tiles_m * ((N + bn - 1) / bn);
        const int rounds = (tiles + sms - 1) / sms;
        const double cost = (double)rounds * (bn + 24);      // + a tile's fixed cost
        if (cost < best_cost - 1e-9) { best_cost = cost; best = bn; }
    }
    return best;
}

// `partials` (2 P_MAX_CTAS tiles of 128 x 256 floats) and `flags` (4 P_FLAG_CAP ints, zero; the kernel
// leaves them zero) let CTAs share a tile's K range; without them the ranges are cut at tile
// boundaries only.
template <typename OT, int EPI>
int launch_persistent(const void* X, const void* W, void* C, int M, int N, int K, long long lda, long long ldw,
                      long long ldc, float* partials, int* flags, int* status, cudaStream_t stream,
                      const QkvRopeArgs* qr = nullptr) {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        if (sms > P_MAX_CTAS) sms = P_MAX_CTAS;
    }
    const int step = EPI == 1 ? 32 : 16;
    int bn = N >= P_BN_MAX ? P_BN_MAX : (N + step - 1) / step * step;
    const int tiles_m = (M + BM - 1) / BM;
    long long num_tiles = (long long)tiles_m * ((N + bn - 1) / bn);
    const int total_kb = (K + BK - 1) / BK;
    if (num_tiles > INT_MAX / 2) return fail("gemm_tc: too many tiles (%lld)", num_tiles);
    long long whole_tiles = num_tiles, tail_tiles = 0;
    int ways = 1;
    const long long rest = num_tiles % sms;
    // Cut the tiles of the last round along K when that round would leave SMs idle: into the number
    // of parts (two per CTA at most, eight K blocks a part at least) that makes the parts' rounds
    // shortest.  Measured, the parts cost some 15-20 us more than their K blocks (short segments:
    // each has its own start-up, partial store and exchange), so the gain must be worth it
    // (a K block takes about 0.36 us): in practice K of 8192 and more.
    if (EPI != 2 && partials && flags && num_tiles <= P_FLAG_CAP && num_tiles > sms && rest > 0) {
        double best = 1.0;
        for (int w = 2; w <= 8 && rest * w <= 2LL * sms && total_kb / w >= 8; ++w) {
            const double rounds = (double)((rest * w + sms - 1) / sms) / w;
            if (rounds < best - 1e-9) { best = rounds; ways = w; }
        }
        if ((1.0 - best) * total_kb * 0.36 < 40.0) ways = 1;
        if (ways > 1) {
            tail_tiles = rest;
            whole_tiles = num_tiles - rest;
        }
    }
    const bool share = ways > 1;
    if (pair_enabled() && !share && M > BM) {
        // two SMs on one tile of 256 tokens: whole tiles only
        const int pairs = sms / 2;
        int pbn = N >= P_BN_MAX ? P_BN_MAX : (N + 31) / 32 * 32;
        const int tiles_m2 = (M + 2 * BM - 1) / (2 * BM);
        if (EPI != 2 && N >= P_BN_MAX) pbn = choose_persistent_bn(tiles_m2, N, pairs, EPI == 1 ? 32 : 16);
        if (EPI == 2 && qr && qr->d <= 128 && N >= P_BN_MAX) {
            // tiles begin and end on heads: 256 wide, or 128 where that fills the rounds of pairs better
            const long long wide = ((long long)tiles_m2 * ((N + 255) / 256) + pairs - 1) / pairs * (256 + 24);
            const long long narrow = ((long long)tiles_m2 * ((N + 127) / 128) + pairs - 1) / pairs * (128 + 24);
            if (narrow < wide) pbn = 128;
        }
        const long long pair_tiles = (long long)tiles_m2 * ((N + pbn - 1) / pbn);
        // two K blocks per stage (see PairRing): three stages of 64 KB with tiles 256 wide, four or more below 176
        PairRing ring;
        ring.kbs = pair_kbs() ? pair_kbs() : 2;
        ring.stage_bytes = (uint32_t)ring.kbs * (PairSmem::A_BYTES + (pbn / 2) * BK * 2);
        ring.stages = PAIR_DATA_BYTES / (int)ring.stage_bytes;
        if (ring.stages > PAIR_MAX_STAGES) ring.stages = PAIR_MAX_STAGES;
        if (ring.stages < 2) return fail("gemm_tc: a stage of %u bytes leaves no ring", ring.stage_bytes);
        CUtensorMap pa, pb;
        int prc;
        if ((prc = make_map(&pa, X, M, K, lda, BM))) return prc;
        if ((prc = make_map(&pb, W, N, K, ldw, pbn / 2))) return prc;
        auto pkern = gemm_tc_pair_kernel<OT, EPI>;
        static bool pair_configured = false;
        if (!pair_configured) {
            cudaError_t e = cudaFuncSetAttribute(pkern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL);
            if (e != cudaSuccess) return fail("gemm_tc: cannot set %d bytes of shared memory: %s", PairSmem::TOTAL, cudaGetErrorString(e));
            pair_configured = true;
        }
        QkvRopeArgs none = {};
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(2 * (pair_tiles < pairs ? pair_tiles : pairs)));
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = PairSmem::TOTAL;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, pkern, pa, pb, (OT*)C, M, N, K, ldc, pbn, tiles_m2, (int)pair_tiles, ring,
                                           status, qr ? *qr : none, g_wait_limit);
        if (e != cudaSuccess) return fail("gemm_tc: launch of the two-SM kernel: %s", cudaGetErrorString(e));
        return check_launch("gemm_tc_pair");
    }
    if (EPI != 2 && !share && N >= P_BN_MAX) {     // (epilogue 2 needs tiles that begin and end on heads)
        // whole tiles only: a narrower tile may fill the last round better
        bn = choose_persistent_bn(tiles_m, N, sms, step);
        num_tiles = whole_tiles = (long long)tiles_m * ((N + bn - 1) / bn);
    }
    const long long grid = num_tiles < sms ? num_tiles : sms;
    CUtensorMap ma, mb;
    int rc;
    if ((rc = make_map(&ma, X, M, K, lda, BM))) return rc;
    if ((rc = make_map(&mb, W, N, K, ldw, bn))) return rc;
    auto kern = gemm_tc_persistent_kernel<OT, EPI>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PSmem::TOTAL);
        if (e != cudaSuccess) return fail("gemm_tc: cannot set %d bytes of shared memory: %s", PSmem::TOTAL, cudaGetErrorString(e));
        configured = true;
    }
    QkvRopeArgs none = {};
    launch_kernel(kern, dim3((unsigned)grid), dim3(THREADS), PSmem::TOTAL, stream, ma, mb, (OT*)C, M, N, K, ldc, bn,
                  tiles_m, (int)whole_tiles, (int)tail_tiles, ways, partials, flags, status, qr ? *qr : none, g_wait_limit);
    return check_launch("gemm_tc_persistent");
}
}  // namespace

// The iteration limit of the persistent product's bounded waits (0: the default).  For tests that make a
// wait run out on purpose (a flag that nothing sets): with a short limit the kernel gives up within
// milliseconds, sets bit 4 of the status word and leaves in order.  Returns the limit that was in force.
MHB_EXPORT unsigned mhb_gemm_tc_wait_limit(unsigned limit) {
    const unsigned before = g_wait_limit;
    g_wait_limit = limit ? limit : WAIT_LIMIT;
    return before;
}

// C[M, N] = X[M, K] * W[N, K]^T, bfloat16 in, float32 accumulation, C float32 or bfloat16.
// swap != 0 streams W through the 128-row operand (few tokens); bn is the tile width along the
// other operand (16..256), or 0 for the persistent kernel (which then takes `partials` and `flags`,
// see launch_persistent; both may be null).  Requirements (else an error, never a wrong result): K % 8 == 0,
// lda % 8 == 0, ldw % 8 == 0, pointers 16-byte aligned.
MHB_EXPORT int mhb_gemm_tc(const void* X, const void* W, void* C, int c_dtype, int M, int N, int K,
                           long long lda, long long ldw, long long ldc, int swap, int bn, int nsplit,
                           long long split_stride, float* partials, int* flags, int* status,
                           cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || lda % 8 || ldw % 8) return fail("gemm_tc: K, lda and ldw must be multiples of 8 (K %d, lda %lld, ldw %lld)", K, lda, ldw);
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return fail("gemm_tc: operands must be 16-byte aligned");
    if (nsplit < 1) nsplit = 1;
    if (nsplit > 1 && c_dtype != MHB_F32) return fail("gemm_tc: split-K partials must be float32");
    const int total_kb = (K + BK - 1) / BK;
    if (nsplit > total_kb) return fail("gemm_tc: %d splits for %d K blocks", nsplit, total_kb);
    const int kbps = (total_kb + nsplit - 1) / nsplit;
    if ((long long)kbps * (nsplit - 1) >= total_kb) return fail("gemm_tc: split %d of K blocks %d leaves an empty split", nsplit, total_kb);
    CUtensorMap ma, mb;
    int rc;
    if (swap) {
        if ((rc = make_map(&ma, W, N, K, ldw, BM))) return rc;
        if ((rc = make_map(&mb, X, M, K, lda, bn))) return rc;
        if (c_dtype == MHB_F32) return dispatch_bn<true, float, 0>(bn, ma, mb, C, N, M, K, ldc, nsplit, kbps, split_stride, swap ? 1 : 2, status, stream);
        return dispatch_bn<true, __nv_bfloat16, 0>(bn, ma, mb, C, N, M, K, ldc, nsplit, kbps, split_stride, swap ? 1 : 2, status, stream);
    }
    if (bn == 0) {       // the persistent kernel picks its own tiles
        if (nsplit != 1) return fail("gemm_tc: the persistent kernel takes no split K");
        if (c_dtype == MHB_F32) return launch_persistent<float, 0>(X, W, C, M, N, K, lda, ldw, ldc, partials, flags, status, stream);
        return launch_persistent<__nv_bfloat16, 0>(X, W, C, M, N, K, lda, ldw, ldc, partials, flags, status, stream);
    }
    if ((rc = make_map(&ma, X, M, K, lda, BM))) return rc;
    if ((rc = make_map(&mb, W, N, K, ldw, bn))) return rc;
    if (c_dtype == MHB_F32) return dispatch_bn<false, float, 0>(bn, ma, mb, C, M, N, K, ldc, nsplit, kbps, split_stride, swap ? 1 : 2, status, stream);
    return dispatch_bn<false, __nv_bfloat16, 0>(bn, ma, mb, C, M, N, K, ldc, nsplit, kbps, split_stride, swap ? 1 : 2, status, stream);
}

// The stacked q/k/v product of more than 64 tokens with bias, rotation and the append to the paged
// KV cache done by its epilogue (see QkvRopeArgs): q_out [M, nq d] bfloat16, cache one layer's pool
// [pages, 2, nkv, P, d] bfloat16, cos_sin [M, rotary_dim] float32 (mhb_rope_table).  Head size 64 or
// 128; rotary_dim a multiple of 32 (half-split pairs) or of 16 (interleaved pairs), or 0.
MHB_EXPORT int mhb_gemm_tc_qkv_rope_supports(int d, int rotary_dim, int interleaved) {
    return (d == 64 || d == 128) && rotary_dim >= 0 && rotary_dim <= d && rotary_dim % (interleaved ? 16 : 32) == 0;
}

MHB_EXPORT int mhb_gemm_tc_qkv_rope(const void* X, const void* W, int M, int K, long long lda, long long ldw,
                                    const float* bias, const float* cos_sin, int rotary_dim, int interleaved,
                                    const int* positions,
                                    const int* tok_seg, const int* block_table, int table_width, void* q_out,
                                    void* cache, int nq, int nkv, int d, int P, int num_pages, int write_kv,
                                    int* status, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (!mhb_gemm_tc_qkv_rope_supports(d, rotary_dim, interleaved))
        return fail("gemm_tc_qkv_rope: head size %d with %d rotated elements (%s pairs) is not built: head size 64 or "
                    "128, rotated elements a multiple of %d", d, rotary_dim, interleaved ? "interleaved" : "half-split",
                    interleaved ? 16 : 32);
    if (rotary_dim > 0 && (cos_sin == nullptr || ((uintptr_t)cos_sin & 15)))
        return fail("gemm_tc_qkv_rope: the cos/sin table must be given and 16-byte aligned");
    if (K <= 0 || K % 8 || lda % 8 || ldw % 8) return fail("gemm_tc: K, lda and ldw must be multiples of 8 (K %d, lda %lld, ldw %lld)", K, lda, ldw);
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15) || ((uintptr_t)q_out & 15) || ((uintptr_t)cache & 15))
        return fail("gemm_tc_qkv_rope: operands must be 16-byte aligned");
    if (nq <= 0 || nkv <= 0 || P <= 0) return fail("gemm_tc_qkv_rope: bad head counts or page size");
    QkvRopeArgs qr;
    qr.bias = bias; qr.cos_sin = cos_sin; qr.rdim = rotary_dim; qr.interleaved = interleaved ? 1 : 0; qr.positions = positions; qr.tok_seg = tok_seg; qr.block_table = block_table;
    qr.q_out = (__nv_bfloat16*)q_out; qr.cache = (__nv_bfloat16*)cache; qr.table_width = table_width;
    qr.nq = nq; qr.nkv = nkv; qr.d = d; qr.P = P; qr.num_pages = num_pages; qr.write_kv = write_kv;
    const int N = (nq + 2 * nkv) * d;
    return launch_persistent<__nv_bfloat16, 2>(X, W, nullptr, M, N, K, lda, ldw, 0, nullptr, nullptr, status, stream, &qr);
}

// act[M, I] = silu(X Wg^T) * (X Wu^T) where W [2 I, K] holds gate and up rows interleaved in
// blocks of 16 (see the kernel).  I must be a multiple of 16; no split K.
MHB_EXPORT int mhb_gemm_tc_swiglu(const void* X, const void* W, void* C, int c_dtype, int M, int I, int K,
                                  long long lda, long long ldw, long long ldc, int swap, int bn, float* partials,
                                  int* flags, int* status, cudaStream_t stream) {
    if (M <= 0 || I <= 0) return 0;
    if (I % 16) return fail("gemm_tc_swiglu: the intermediate size %d must be a multiple of 16", I);
    if (K <= 0 || K % 8 || lda % 8 || ldw % 8) return fail("gemm_tc: K, lda and ldw must be multiples of 8 (K %d, lda %lld, ldw %lld)", K, lda, ldw);
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return fail("gemm_tc: operands must be 16-byte aligned");
    if (c_dtype != MHB_BF16) return fail("gemm_tc_swiglu: the output must be bfloat16");
    const int N = 2 * I;
    const int total_kb = (K + BK - 1) / BK;
    CUtensorMap ma, mb;
    int rc;
    if (swap) {
        if ((rc = make_map(&ma, W, N, K, ldw, BM))) return rc;
        if ((rc = make_map(&mb, X, M, K, lda, bn))) return rc;
        return dispatch_bn<true, __nv_bfloat16, 1>(bn, ma, mb, C, N, M, K, ldc, 1, total_kb, 0, 1, status, stream);
    }
    if (bn == 0)
        return launch_persistent<__nv_bfloat16, 1>(X, W, C, M, N, K, lda, ldw, ldc, partials, flags, status, stream);
    if ((rc = make_map(&ma, X, M, K, lda, BM))) return rc;
    if ((rc = make_map(&mb, W, N, K, ldw, bn))) return rc;
    return dispatch_bn<false, __nv_bfloat16, 1>(bn, ma, mb, C, M, N, K, ldc, 1, total_kb, 0, 2, status, stream);
}
