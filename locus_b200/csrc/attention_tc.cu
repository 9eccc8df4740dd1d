// Attention of long prompt portions on the Blackwell tensor cores (tcgen05.mma, scores and the
// weighted sums of V in tensor memory), bfloat16 queries / keys / values, softmax in float32.
//
// A block takes 128 consecutive new tokens of one request and one head.  Keys and values come in
// tiles of 128 positions through the request's block table: TMA boxes of 64 rows x 64 elements
// (pages are a multiple of 64 tokens, so a box never straddles pages; a box whose page does not
// exist is fetched from outside the tensor and arrives as zeros), two stages each for K and V.
//
//   MMA 1:  S[q, t] = sum_d Q[q, d] K[t, d]        (A = Q, B = K, both K-major; 128 x 128 in TMEM)
//   softmax warps: the threads of a query row read its row of S (tcgen05.ld), mask (causal, window,
//           end of the sequence), keep the running maximum and denominator (base 2), write
//           P = exp2(s - m) as bfloat16 into shared memory in the swizzled K-major operand layout
//   MMA 2:  O[q, d] += sum_t P[q, t] V[t, d]      (A = P, B = V read MN-major: V lies [t][d] in the
//           cache, which is the transposed operand; 128 x 128 in TMEM, ONE sum from the first tile to the last)
//   The row's threads rescale O in tensor memory (tcgen05.ld, multiply, tcgen05.st) only when the row's maximum
//   has run ahead of the reference its probabilities are formed against by more than 2^8, and read it once at
//   the end: O / denominator.  (Adding every tile's P V into registers cost 400 cycles a tile.)
//
// S is double-buffered in tensor memory (2 x 128 columns beside the 128 of O), so the tensor pipe computes the
// scores of the next tile while the softmax warps work on this one; P has two buffers in shared memory.
// Warp 0: TMA; warp 1: MMA issue (one thread);
// warps 2-9: softmax and output, two threads per query row (64 keys and 64 output dimensions each).  Head size 128 only (other sizes and pages that are not a multiple
// of 64 tokens go to the mma.sync kernel).
//
// Every wait on an mbarrier is bounded; when one runs out the kernel sets the module's error word,
// and every later wait of every role returns at once, so the kernel ends quickly instead of hanging.
#include <cuda.h>
#include <string.h>

#include "common.cuh"

#define AT_HD 128        // head size
#define AT_MQ 128        // queries per block
#define AT_MK 128        // keys per tile
#define AT_HALF_BYTES (128 * 128)     // 128 rows x 64 elements: one swizzled half of an operand tile
#define AT_TILE_BYTES (2 * AT_HALF_BYTES)
#define AT_WAIT_LIMIT 200000000LL

__device__ int g_at_error = 0;

struct TcAttnArgs {
    bf16* out;
    const int* seg_q0;
    const int* seg_qn;
    const int* seg_ctx;
    const int* block_table;
    int table_stride;
    const int* items;
    int nh, nkv, page_tokens, window;
    float scale;
    // Ranges of key tiles per block of queries (1: a block writes the result itself).  With more, a block takes
    // one range (blockIdx.z) and leaves, per query row of the step and head, its unnormalised sum, its running
    // maximum (base 2, scaled) and its denominator; attn_chunk_tc_merge_kernel adds the ranges up in ascending order.
    int n_splits;
    float* part_o;    // [row][head][split][128]
    float* part_ml;   // [row][head][split][2]
};

// Key tiles of a block of nq queries whose first sits at position p0: the first tile's first position and their
// number, and how they are cut into ranges (the same in both kernels).
__device__ __forceinline__ void at_tiles(int p0, int nq, int window, int n_splits, int& first_tile, int& n_tiles,
                                         int& per_split) {
    const int t_hi = p0 + nq - 1;
    const int t_lo = window > 0 ? max(0, p0 - window + 1) : 0;
    first_tile = (t_lo / AT_MK) * AT_MK;
    n_tiles = (t_hi - first_tile) / AT_MK + 1;
    per_split = (n_tiles + n_splits - 1) / n_splits;
}

__device__ __forceinline__ uint32_t at_smem(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void at_bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void at_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool at_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false when the limit ran out here or anywhere else in the grid before.
__device__ __forceinline__ bool at_wait(uint32_t bar, uint32_t parity, int code) {
    if (at_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!at_try_wait(bar, parity)) {
        if (*reinterpret_cast<volatile int*>(&g_at_error) != 0) return false;
        if (clock64() - t0 > AT_WAIT_LIMIT) {
            atomicCAS(&g_at_error, 0, code);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void at_tma_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
// Shared-memory operand descriptors, 128-byte swizzle.  K-major: rows of 128 bytes, 8-row groups
// 1024 bytes apart.  MN-major (the operand lies transposed): 64 elements of the M/N side are the
// contiguous 128 bytes, the next 64 are `lbo_bytes` further on, 8-row groups of the k side 1024 apart.
__device__ __forceinline__ uint64_t at_desc_k(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
__device__ __forceinline__ uint64_t at_desc_mn(uint32_t saddr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
__device__ __forceinline__ void at_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void at_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void at_ld32(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
        "%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
}
// 2^x for x <= 0 by the special-function unit alone (exp2f adds range handling that the softmax does
// not need: a result that underflows may be zero).
__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two probabilities (finite, in [0, 1]) as bfloat16, rounded to nearest (ties upward) with integer
// arithmetic: the conversion instruction runs on the same narrow pipe as ex2 and would add half as
// much again to what already takes as long as the tile's MMAs.
__device__ __forceinline__ uint32_t at_pack_prob(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}
__device__ __forceinline__ uint32_t at_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Packed float32 pairs (one instruction for two lanes of arithmetic) and a three-way maximum: the softmax
// warps are bound by instruction issue as much as by the special-function unit.
__device__ __forceinline__ unsigned long long at_pair(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void at_unpair(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long at_fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long at_add2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long at_mul2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float at_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void at_st32(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
          "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
          "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

// The weighted sum of V stays in tensor memory from a block's first key tile to its last: the MMAs of every tile add
// to it.  A row's probabilities are formed against a reference maximum that follows the row's true running maximum
// only when that has run ahead by more than 2^AT_LAG_LOG2; then, and only then, the row's sum is read, rescaled
// and written back.  Probabilities reach 2^8 at most, far inside bfloat16's and float32's range, and the quotient
// sum / denominator is the same number whatever reference it was formed with.
#define AT_LAG_LOG2 8.0f

__global__ void __launch_bounds__(320, 1)
attn_chunk_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, TcAttnArgs a) {
    extern __shared__ __align__(1024) uint8_t at_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the late tiles of a prompt see the most keys: the grid takes them first, for all heads (the heads are the
    // fast index of the grid, so that the blocks go out longest first and the last SMs to finish hold short ones)
    const int item = gridDim.y - 1 - blockIdx.y;
    const int seg = a.items[2 * item], qoff = a.items[2 * item + 1];
    if (qoff & 64) return;  // items are tiles of 64 queries; a block takes an even one and its upper neighbour
    const int h = blockIdx.x, kvh = h / (a.nh / a.nkv);
    const int nq = min(AT_MQ, a.seg_qn[seg] - qoff);
    const int row0 = a.seg_q0[seg] + qoff;
    const int p0 = a.seg_ctx[seg] + qoff;
    const int t_hi = p0 + nq - 1;
    const int t_lo = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
    const int P = a.page_tokens;
    // this block's range of the key tiles (all of them when the keys are not cut)
    int first_tile, n_tiles_all, per_split;
    at_tiles(p0, nq, a.window, a.n_splits, first_tile, n_tiles_all, per_split);
    const int split = blockIdx.z;
    first_tile += split * per_split * AT_MK;
    const int n_tiles = max(0, min(per_split, n_tiles_all - split * per_split));
    if (n_tiles == 0) return;  // the merge counts the live ranges the same way
    const int* table = a.block_table + static_cast<size_t>(seg) * a.table_stride;

    // shared memory: Q, K[2], V[2], P[2] (each a tile of two swizzled halves), then the barriers.  That is
    // all the shared memory a block can have, so the tiles start at the very base, which must be
    // 1024-byte aligned for the swizzle (checked: a block that finds it otherwise reports and leaves).
    const uint32_t base = at_smem(at_raw);
    if (base & 1023u) {
        if (threadIdx.x == 0) atomicCAS(&g_at_error, 0, 12);
        return;
    }
    const uint32_t sQ = base, sK = sQ + AT_TILE_BYTES, sV = sK + 2 * AT_TILE_BYTES, sP = sV + 2 * AT_TILE_BYTES;
    const uint32_t bars = sP + 2 * AT_TILE_BYTES;
    const uint32_t q_full = bars, k_full = bars + 8, v_full = bars + 24, k_free = bars + 40, v_free = bars + 56;
    const uint32_t s_full = bars + 72, s_free = bars + 88, pv_done = bars + 104, p_ready = bars + 136;
    const uint32_t slot = bars + 144;
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(at_raw + (slot - at_smem(at_raw)));

    if (threadIdx.x == 0) {
        at_bar_init(q_full, 1);
        for (int b = 0; b < 2; ++b) {
            at_bar_init(k_full + 8 * b, 1);
            at_bar_init(v_full + 8 * b, 1);
            at_bar_init(k_free + 8 * b, 1);
            at_bar_init(v_free + 8 * b, 1);
            at_bar_init(s_full + 8 * b, 1);
            at_bar_init(s_free + 8 * b, 8);    // one arrival per softmax warp
            at_bar_init(pv_done + 8 * b, 1);
        }
        at_bar_init(p_ready, 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *slot_ptr;
    const uint32_t tS = tmem, tO = tmem + 2 * AT_MK;  // S0, S1, O: 128 columns each

    if (warp == 0) {
        if (lane == 0) {
            // Q: two halves of 64 elements, rows row0 .. row0 + 127 (rows past the portion are never stored)
            at_expect_tx(q_full, AT_TILE_BYTES);
            at_tma_2d(sQ, &map_q, h * AT_HD, row0, q_full);
            at_tma_2d(sQ + AT_HALF_BYTES, &map_q, h * AT_HD + 64, row0, q_full);
            const long long rows_per_page = 2LL * a.nkv * P;
            for (int j = 0; j < n_tiles; ++j) {
                const int b = j & 1;
                const uint32_t par = ((j >> 1) & 1) ^ 1;
                const int tile0 = first_tile + j * AT_MK;
                // rows of the pool (viewed as [pages * 2 * nkv * P][hd]) of the two 64-key halves; a half with
                // no page, or wholly outside the keys this block may see, is fetched from outside the tensor
                int krow[2];
                for (int hh = 0; hh < 2; ++hh) {
                    const int t = tile0 + 64 * hh;
                    int page = -1;
                    if (t <= t_hi && t + 63 >= t_lo) page = table[t / P];
                    krow[hh] = page < 0 ? -64 : static_cast<int>(page * rows_per_page + static_cast<long long>(kvh) * P + t % P);
                }
                const int v_shift = a.nkv * P;  // V rows of a page lie nkv * P rows behind its K rows
                if (!at_wait(k_free + 8 * b, par, 1)) break;
                at_expect_tx(k_full + 8 * b, AT_TILE_BYTES);
                for (int hh = 0; hh < 2; ++hh)
                    for (int ch = 0; ch < 2; ++ch)
                        at_tma_2d(sK + b * AT_TILE_BYTES + ch * AT_HALF_BYTES + hh * (64 * 128), &map_kv, 64 * ch, krow[hh],
                                  k_full + 8 * b);
                if (!at_wait(v_free + 8 * b, par, 2)) break;
                at_expect_tx(v_full + 8 * b, AT_TILE_BYTES);
                for (int hh = 0; hh < 2; ++hh)
                    for (int ch = 0; ch < 2; ++ch)
                        at_tma_2d(sV + b * AT_TILE_BYTES + ch * AT_HALF_BYTES + hh * (64 * 128), &map_kv, 64 * ch,
                                  krow[hh] < 0 ? -64 : krow[hh] + v_shift, v_full + 8 * b);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // f32 accumulate, bf16 x bf16, M = 128, N = 128; MMA 2 reads its B operand MN-major
            const uint32_t idesc1 = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(AT_MK >> 3) << 17) |
                                    (static_cast<uint32_t>(AT_MQ >> 4) << 24);
            const uint32_t idesc2 = idesc1 | (1u << 16);
            auto scores = [&](int j) -> bool {  // S_j = Q K_j^T
                const int b = j & 1;
                if (!at_wait(k_full + 8 * b, (j >> 1) & 1, 3)) return false;
                if (!at_wait(s_free + 8 * b, ((j >> 1) & 1) ^ 1, 4)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int ks = 0; ks < AT_HD / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * AT_HALF_BYTES + (ks & 3) * 32;
                    at_mma(tS + b * AT_MK, at_desc_k(sQ + off), at_desc_k(sK + b * AT_TILE_BYTES + off), idesc1, ks > 0);
                }
                at_commit(s_full + 8 * b);
                at_commit(k_free + 8 * b);
                return true;
            };
            bool ok = at_wait(q_full, 0, 5) && scores(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int b = j & 1;
                if (j + 1 < n_tiles && !scores(j + 1)) break;
                // O += P_j V_j: the sum stays in tensor memory from the first tile to the last
                if (!at_wait(p_ready, j & 1, 6)) break;
                if (!at_wait(v_full + 8 * b, (j >> 1) & 1, 7)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int ks = 0; ks < AT_MK / 16; ++ks) {
                    const uint64_t dp = at_desc_k(sP + b * AT_TILE_BYTES + (ks >> 2) * AT_HALF_BYTES + (ks & 3) * 32);
                    const uint64_t dv = at_desc_mn(sV + b * AT_TILE_BYTES + ks * (16 * 128), AT_HALF_BYTES);
                    at_mma(tO, dp, dv, idesc2, (j > 0 || ks > 0) ? 1u : 0u);  // O += P_j V_j
                }
                at_commit(pv_done + 8 * b);  // tells the softmax warps (P's buffer is free, the sum may be touched) ...
                at_commit(v_free + 8 * b);   // ... and the loader (the stage's V is free)
            }
        }
    } else {
        // Softmax and output: two threads per query row (warps w and w + 4 reach the same quarter of the
        // lanes of tensor memory); each takes 64 of the tile's 128 keys and 64 of the 128 output dimensions.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;  // this thread's query row
        const int pq = p0 + r;              // its position
        const uint32_t lane_bits = static_cast<uint32_t>(quarter * 32) << 16;
        const float scale_log2 = a.scale * 1.4426950408889634f;
        const unsigned long long scale2 = at_pair(scale_log2, scale_log2);
        float m_run = -INFINITY, l_run = 0.f;  // the row's reference maximum (base 2, scaled); this thread's part of the denominator
        uint8_t* at_generic = at_raw + (base - at_smem(at_raw));
        uint8_t* gP0 = at_generic + (sP - base) + half * AT_HALF_BYTES + r * 128;
        float* xch = reinterpret_cast<float*>(at_generic + (slot + 16 - base));  // [2 tile parities][2 halves][128 rows]
        bool ok = true;
        const int lo = a.window > 0 ? max(0, pq - a.window + 1) : 0;  // first key this row sees
        const uint32_t tOmine = tO + lane_bits + 64 * half;           // this thread's 64 columns of the row's sum

        // the two threads of a row exchange a value through shared memory (a barrier of their two warps)
        auto with_partner = [&](int parity, float mine) -> float {
            float* slot_f = xch + parity * 256;
            slot_f[half * 128 + r] = mine;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
            return slot_f[(half ^ 1) * 128 + r];
        };

        // (When a wait gives up, this loop still runs to its end -- every later wait returns at once -- so that
        // the two warps of a row meet at every one of their barriers.)
        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1;
            const int tile0 = first_tile + j * AT_MK + 64 * half;  // first key of this thread's half of the tile
            if (!at_wait(s_full + 8 * b, (j >> 1) & 1, 10)) ok = false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t s0[32], s1[32];
            at_ld32(tS + b * AT_MK + lane_bits + 64 * half, s0);
            at_ld32(tS + b * AT_MK + lane_bits + 64 * half + 32, s1);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            // a key t counts for this row when lo <= t <= pq; only tiles at an edge need the test
            const int tile_first = first_tile + j * AT_MK;
            const bool need_mask = tile_first + AT_MK - 1 > p0 || tile_first < t_lo ||
                                   (a.window > 0 && tile_first <= p0 + AT_MQ - 1 - a.window);
            float mx = -INFINITY;
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int t = tile0 + i;
                    if (!(t <= pq && t >= lo)) s0[i] = 0xff800000u;            // -inf
                    if (!(t + 32 <= pq && t + 32 >= lo)) s1[i] = 0xff800000u;
                }
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = at_max3(mx, __uint_as_float(s0[i]), __uint_as_float(s1[i]));
            mx = fmaxf(mx, with_partner(b, mx)) * scale_log2;  // the scale is positive: the maximum can be scaled last
            const float m_new = fmaxf(mx, m_run);               // the same in both threads of the row
            // The buffer of P_{j-2} is free when its product is finished (the same barrier frees the stage's V).
            if (j > 1 && !at_wait(pv_done + 8 * b, ((j >> 1) & 1) ^ 1, 9)) ok = false;
            // Does the reference maximum follow?  Only when some row of the warp has run ahead of its reference by
            // more than 2^AT_LAG_LOG2 (always at a row's first key: -inf is infinitely far; -inf - -inf is not a
            // number and compares false, so a row without a key yet keeps -inf).  Both warps of a row hold the same
            // rows and the same maxima, so they decide alike.  Then every row of the warp moves its reference and
            // rescales its sum, which needs the product of the tile before this one finished.
            if (__any_sync(0xffffffffu, m_new - m_run > AT_LAG_LOG2)) {
                if (j > 0) {
                    if (!at_wait(pv_done + 8 * (b ^ 1), ((j - 1) >> 1) & 1, 12)) ok = false;
                    const float f = m_run == -INFINITY ? 1.f : at_exp2(m_run - m_new);
                    const unsigned long long f2 = at_pair(f, f);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t v[32];
                        at_ld32(tOmine + 32 * c, v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int d = 0; d < 32; d += 2) {
                            float x, y;
                            at_unpair(at_mul2(at_pair(__uint_as_float(v[d]), __uint_as_float(v[d + 1])), f2), x, y);
                            v[d] = __float_as_uint(x);
                            v[d + 1] = __float_as_uint(y);
                        }
                        at_st32(tOmine + 32 * c, v);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    l_run *= f;
                }
                m_run = m_new;
            }
            const float m_ref = m_run == -INFINITY ? 0.f : m_run;  // exp2(-inf - 0) = 0 for a row without keys so far
            const unsigned long long neg_m2 = at_pair(-m_ref, -m_ref);
            // P = exp2(s * scale - m_ref) as bfloat16 into shared memory (K-major operand, 128-byte swizzle)
            uint8_t* gP = gP0 + b * AT_TILE_BYTES;
            unsigned long long sum2 = at_pair(0.f, 0.f);
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {  // 16-byte pieces of 8 probabilities
                float pr[8];
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const uint32_t r0 = q8 < 4 ? s0[8 * q8 + i] : s1[8 * (q8 - 4) + i];
                    const uint32_t r1 = q8 < 4 ? s0[8 * q8 + i + 1] : s1[8 * (q8 - 4) + i + 1];
                    float x, y;
                    at_unpair(at_fma2(at_pair(__uint_as_float(r0), __uint_as_float(r1)), scale2, neg_m2), x, y);
                    pr[i] = at_exp2(x);
                    pr[i + 1] = at_exp2(y);
                    sum2 = at_add2(sum2, at_pair(pr[i], pr[i + 1]));
                }
                uint4 pk;
                pk.x = at_pack_prob(pr[0], pr[1]);
                pk.y = at_pack_prob(pr[2], pr[3]);
                pk.z = at_pack_prob(pr[4], pr[5]);
                pk.w = at_pack_prob(pr[6], pr[7]);
                *reinterpret_cast<uint4*>(gP + ((q8 ^ (r & 7)) << 4)) = pk;
            }
            {
                float x, y;
                at_unpair(sum2, x, y);
                l_run += x + y;
            }
            // the last tile may hold rows of V behind the sequence's end (never written, any bit pattern): zero them
            if (tile_first + AT_MK - 1 > t_hi) {
                if (!at_wait(v_full + 8 * b, (j >> 1) & 1, 11)) ok = false;
                if (tile_first + r > t_hi) {
                    uint8_t* gV = at_generic + (sV - base) + b * AT_TILE_BYTES + half * AT_HALF_BYTES + r * 128;
#pragma unroll
                    for (int q8 = 0; q8 < 8; ++q8) *reinterpret_cast<uint4*>(gV + q8 * 16) = make_uint4(0, 0, 0, 0);
                }
            }
            // S_j is read, P_j is written, the sum is where the MMAs may add to it: tell the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                at_arrive(s_free + 8 * b);
                at_arrive(p_ready);
            }
        }
        // the sum is complete when the last product is
        if (!at_wait(pv_done + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, 13)) ok = false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        {
            const float l = l_run + with_partner(n_tiles & 1, l_run);
            const float inv = 1.0f / l;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t v[32];
                at_ld32(tOmine + 32 * c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (a.n_splits > 1) {
                    if (ok && r < nq) {
                        const size_t unit = (static_cast<size_t>(row0 + r) * a.nh + h) * a.n_splits + split;
                        float* po = a.part_o + unit * AT_HD + 64 * half + 32 * c;
#pragma unroll
                        for (int d = 0; d < 32; d += 4)
                            *reinterpret_cast<uint4*>(po + d) = make_uint4(v[d], v[d + 1], v[d + 2], v[d + 3]);
                        if (half == 0 && c == 0) *reinterpret_cast<float2*>(a.part_ml + unit * 2) = make_float2(m_run, l);
                    }
                } else if (ok && r < nq) {
                    bf16* dst = a.out + (static_cast<size_t>(row0 + r) * a.nh + h) * AT_HD + 64 * half + 32 * c;
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint4 pk;
                        pk.x = at_pack(__uint_as_float(v[d]) * inv, __uint_as_float(v[d + 1]) * inv);
                        pk.y = at_pack(__uint_as_float(v[d + 2]) * inv, __uint_as_float(v[d + 3]) * inv);
                        pk.z = at_pack(__uint_as_float(v[d + 4]) * inv, __uint_as_float(v[d + 5]) * inv);
                        pk.w = at_pack(__uint_as_float(v[d + 6]) * inv, __uint_as_float(v[d + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + d) = pk;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

#define AT_MAX_SPLITS 16

// out[row][head] = sum over the live ranges s (ascending) of o_s 2^(m_s - M) / sum of l_s 2^(m_s - M), M = max m_s.
// One thread per (query row, four adjacent dimensions) of a block of queries and a head; the loads of all ranges
// are issued together (the loops are unrolled over the most ranges there can be).
__global__ void __launch_bounds__(128) attn_chunk_tc_merge_kernel(TcAttnArgs a) {
    const int item = blockIdx.y, h = blockIdx.z;
    const int seg = a.items[2 * item], qoff = a.items[2 * item + 1];
    if (qoff & 64) return;
    const int nq = min(AT_MQ, a.seg_qn[seg] - qoff);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nq * (AT_HD / 4)) return;
    const int r = i / (AT_HD / 4), d = (i - r * (AT_HD / 4)) * 4;
    const int row = a.seg_q0[seg] + qoff + r;
    int first_tile, n_tiles, per_split;
    at_tiles(a.seg_ctx[seg] + qoff, nq, a.window, a.n_splits, first_tile, n_tiles, per_split);
    const int live = (n_tiles + per_split - 1) / per_split;
    const size_t unit0 = (static_cast<size_t>(row) * a.nh + h) * a.n_splits;
    float2 ml[AT_MAX_SPLITS];
    float4 v[AT_MAX_SPLITS];
#pragma unroll
    for (int s = 0; s < AT_MAX_SPLITS; ++s) {
        ml[s] = make_float2(-INFINITY, 0.f);
        v[s] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (s < live) {
            ml[s] = *reinterpret_cast<const float2*>(a.part_ml + (unit0 + s) * 2);
            v[s] = *reinterpret_cast<const float4*>(a.part_o + (unit0 + s) * AT_HD + d);
        }
    }
    float M = -INFINITY;
#pragma unroll
    for (int s = 0; s < AT_MAX_SPLITS; ++s) M = fmaxf(M, ml[s].x);
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < AT_MAX_SPLITS; ++s) {
        const float w = ml[s].x == -INFINITY ? 0.f : exp2f(ml[s].x - M);
        L += ml[s].y * w;
        acc.x += v[s].x * w;
        acc.y += v[s].y * w;
        acc.z += v[s].z * w;
        acc.w += v[s].w * w;
    }
    const float inv = 1.0f / L;
    uint2 pk;
    pk.x = at_pack(acc.x * inv, acc.y * inv);
    pk.y = at_pack(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(a.out + (static_cast<size_t>(row) * a.nh + h) * AT_HD + d) = pk;
}

// ---------------------------------------------------------------------------
typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static AtEncodeFn at_encode_fn() {
    static AtEncodeFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<AtEncodeFn>(p);
        }
    }
    return fn;
}

// rows x cols bfloat16 matrix, row stride ld elements; box = box_rows x 64 elements, 128-byte swizzle; reads
// outside the matrix give zeros.
static bool at_make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
    AtEncodeFn fn = at_encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// q, out [T, nh * 128] bfloat16; pool: one layer's pages [n_pages][2][nkv][page_tokens][128] bfloat16;
// items: [n_items, 2] = (segment, first query of a 64-query tile), a segment's tiles in ascending order.
// Head size 128 and pages of a multiple of 64 tokens only (LOCUS_ERR_UNSUPPORTED otherwise).
// n_splits > 1: the key tiles of every block are cut into that many ranges (at most 16); part_o holds
// T * nh * n_splits * 128 floats, part_ml T * nh * n_splits * 2; a second launch merges.
extern "C" int locus_attn_chunk_tc(const void* q, long long T, const void* pool, long long n_pages, void* out,
                                   const int* seg_q0, const int* seg_qn, const int* seg_ctx, const int* block_table,
                                   int table_stride, const int* items, int n_items, int nh, int nkv, int hd,
                                   int page_tokens, int window, float scale, int n_splits, float* part_o,
                                   float* part_ml, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (n_splits < 1 || n_splits > AT_MAX_SPLITS) return LOCUS_ERR_UNSUPPORTED;
    if (n_splits > 1 && (part_o == nullptr || part_ml == nullptr ||
                         ((reinterpret_cast<uintptr_t>(part_o) | reinterpret_cast<uintptr_t>(part_ml)) & 15)))
        return LOCUS_ERR_UNSUPPORTED;
    if (hd != AT_HD || page_tokens <= 0 || page_tokens % 64 != 0 || window < 0) return LOCUS_ERR_UNSUPPORTED;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || nh > 65535) return LOCUS_ERR_UNSUPPORTED;
    const long long pool_rows = n_pages * 2 * nkv * page_tokens;
    if (T <= 0 || n_pages <= 0 || pool_rows >= (1LL << 31) || T >= (1LL << 31)) return LOCUS_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(pool) | reinterpret_cast<uintptr_t>(out)) & 15)
        return LOCUS_ERR_UNSUPPORTED;
    CUtensorMap map_q, map_kv;
    if (!at_make_map(&map_q, q, T, static_cast<long long>(nh) * hd, static_cast<long long>(nh) * hd, AT_MQ))
        return LOCUS_ERR_UNSUPPORTED;
    if (!at_make_map(&map_kv, pool, pool_rows, hd, hd, 64)) return LOCUS_ERR_UNSUPPORTED;
    TcAttnArgs a;
    a.out = static_cast<bf16*>(out); a.seg_q0 = seg_q0; a.seg_qn = seg_qn; a.seg_ctx = seg_ctx;
    a.block_table = block_table; a.table_stride = table_stride; a.items = items; a.nh = nh; a.nkv = nkv;
    a.page_tokens = page_tokens; a.window = window; a.scale = scale;
    a.n_splits = n_splits; a.part_o = part_o; a.part_ml = part_ml;
    const size_t smem = 7 * AT_TILE_BYTES + 160 + 2 * 2 * 128 * 4;
    static bool set = false;
    if (!set) {
        if (cudaFuncSetAttribute(attn_chunk_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return static_cast<int>(cudaGetLastError());
        set = true;
    }
    if (n_items > 65535) return LOCUS_ERR_UNSUPPORTED;
    dim3 grid(nh, n_items, n_splits);
    attn_chunk_tc_kernel<<<grid, 320, smem, stream>>>(map_q, map_kv, a);
    if (n_splits > 1)
        attn_chunk_tc_merge_kernel<<<dim3(AT_MQ * (AT_HD / 4) / 128, n_items, nh), 128, 0, stream>>>(a);
    return locus_launch_status();
}

// Reads and clears the module's error word (0 = no bounded wait ran out).  Synchronises.
extern "C" int locus_attn_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_at_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_at_error, &zero, sizeof(int));
    return v;
}
