// Decode attention for grouped-query models: one new token per request, G = heads / kv_heads query heads
// share a key/value head.  A warp takes a range of keys of ONE (request, key/value head) and serves all G
// query heads of the group from a single pass over those keys, so every key and value row is read once
// however many query heads share it (the kernel of attention.cu reads them once per query head, through
// the L2: measured 4.2 times slower at 28 heads on 4 and 64 requests of 8,192 tokens).
//
// With G query heads per loaded row the arithmetic no longer fits the CUDA cores at memory speed, so scores
// and weighted sums run on the tensor cores (mma.sync m16n8k16, bfloat16 in, float32 accumulate), everything
// in registers, in the transposed form that puts the 16 keys of a chunk into the M dimension of the tiles and
// eight heads into N (a group of up to eight heads needs one tile of heads, up to sixteen two):
//   S^T [16 keys x 8 heads] = K [16 keys x hd] . Q^T   K rows are the A fragments straight from memory: the
//                       k-index of the MMA is a permutation of the head dimension (the same for K and Q),
//                       chosen so that a lane's fragments of a key are whole 16-byte pieces;
//   softmax            per head (a column) online, base 2, float32; a column lives in eight lanes;
//   O^T [hd x 8 heads] += V^T [hd x 16 keys] . P^T   P^T, the B fragment, is the transpose of S^T's accumulator
//                       layout (movmatrix); V^T's A fragments hold one dimension of two consecutive keys per
//                       register: a lane interleaves its 16-byte pieces of two key rows with byte permutes
//                       (the rows of O^T are a permutation of the head dimension, undone at the store).
// Keeping the memory busy: the K rows and the V rows of a chunk of 16 keys are two runs of 16 x hd x 2 bytes, each
// contiguous in a page.  One lane of the warp asks for each run with ONE bulk copy (cp.async.bulk, global to shared
// memory, completion counted on an mbarrier of the warp's own), two chunks deep; the warp reads the fragments back
// when the chunk's turn comes.  (Copies of 16 bytes per lane were bound first by the number of requests to the L2,
// then, coalesced, by their 200 instructions of address arithmetic per chunk: 465 instructions per chunk at two
// warps per scheduler.)  Rows of V that belong to no live key (before a window's start, behind the range's end) are
// zeroed in shared memory before use: unwritten cache may hold any bits, and 0 x NaN is NaN.  One block of ten
// warps per SM, 16 KB of copies in flight per warp; a warp synchronises only with itself.  Every wait on a barrier
// is bounded: when the limit runs out the warp records it in the module's error word and leaves.
// The cut of the batch into ranges, the partial results, the counters and the ordered merge are those of the
// streaming kernel (attn_ranges.cuh; ranges x key/value heads are the units of work).
//
// Takes bfloat16, head sizes 64 and 128, groups of 2 to 16 query heads, pages of a multiple of 16 tokens.
#include "common.cuh"
#include "attn_ranges.cuh"

struct GqaArgs {
    const bf16* q;            // [T, nh * hd]
    const bf16* pool;         // this layer's pages [n_pages][2][nkv][P][hd]
    bf16* out;                // [T, nh * hd]
    const int* seg_q0;
    const int* seg_ctx;
    const int* block_table;
    int table_stride;
    const int* items;         // [n_items] segments with one new token
    int nh, nkv, page_tokens, window;
    float scale;
    float* part_o;            // [units * G][hd]
    float* part_ml;           // [units * G][2]
    int* counters;            // [n_items * nh], zero between launches (one per (request, kv head) is used)
};

// Warps of a block (one block per SM) and chunks of 16 keys whose copies are in flight per warp.  Shared memory
// (8 KB per chunk at head size 128) allows 8 x 3, 10 x 2, 12 x 2 or 6 x 4; measured at 28 heads on 4 and 8,192 keys,
// 64 / 8 requests: 202 / 52 us, 184 / 56, 190 / 58, 231 / 47.  More warps hide the latency of a chunk's chain of
// dependent instructions better than a deeper ring does.
#ifndef GQ_WARPS
#define GQ_WARPS 10
#endif
#ifndef GQ_STAGES
#define GQ_STAGES 2
#endif

#define GQ_WAIT_LIMIT 2000000000LL   // cycles a warp waits for a copy before it gives up (about a second)

// Error word of the module: 1 = a wait for a bulk copy ran out (the output of that call is invalid).
__device__ int g_gqa_error = 0;
extern "C" int locus_attn_gqa_error() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gqa_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_gqa_error, &zero, sizeof(int));
    }
    return v;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > GQ_WAIT_LIMIT) {
            atomicCAS(&g_gqa_error, 0, 1);
            return false;
        }
    }
    return true;
}
// `bytes` (a multiple of 16) from global to shared memory, both 16-byte aligned; completion on the mbarrier
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void sts16_zero(uint32_t addr) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(addr), "r"(0u) : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint4 ldg16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// transpose of an 8 x 8 matrix of 16-bit elements held as mma fragments (two elements of a row per lane)
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// HD: head size (64 or 128).  WIDE: groups of more than 8 heads (a second tile of heads).
// GQW warps of a block, GQS chunks of 16 keys in flight per warp (10 x 2 for many pairs, 6 x 4 for few: see above).
template <int HD, bool WIDE, int GQW, int GQS>
__global__ void __launch_bounds__(32 * GQW, 1) attn_decode_gqa_kernel(GqaArgs a, int n_items, long long max_units,
                                                                           int cost_range, int cost_merge) {
    pdl_trigger();  // every block of this grid is resident from the start
    constexpr int KS = HD / 16;      // k-steps of a score tile
    constexpr int NL = HD / 32;      // 16-byte pieces of a lane per key row (keys)
    constexpr int MT = HD / 16;      // row tiles of O^T
    constexpr int VL = HD / 64;      // 16-byte pieces of a lane per value row
    constexpr int HT = WIDE ? 2 : 1;  // tiles of eight heads
    constexpr uint32_t ROW_BYTES = HD * 2;
    constexpr uint32_t TILE_BYTES = 16 * ROW_BYTES;  // K (or V) of a chunk
    constexpr uint32_t STAGE_BYTES = 2 * TILE_BYTES;
    extern __shared__ __align__(16) unsigned char gq_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t4 = lane & 3;   // row of the fragments, and the lane's place in its row
    const int P = a.page_tokens, G = a.nh / a.nkv;

    __shared__ KeyRanges kr;
    __shared__ __align__(8) unsigned long long gq_bars[GQW * GQS];
    const uint32_t bars = smem_u32(gq_bars) + warp * (GQS * 8);  // this warp's barriers, one per stage
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < GQS; ++i) mbar_init(bars + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    uint32_t parity = 0;  // bit i: the phase of stage i's barrier that the next wait on it looks for
    const int n_warps = gridDim.x * GQW;
    // a unit (range, kv head) leaves G partial results: the scratch holds max_units of them
    const int len = plan_key_ranges(kr, a.items, a.seg_ctx, a.seg_q0, a.window, n_items, a.nkv, max_units / G, n_warps,
                                    cost_range, cost_merge);
    // (the cut read only the step's descriptors; q and the newest keys and values come from the kernel in front)
    pdl_entry();
    if (len == 0) return;
    const int n_ranges = kr.pref[n_items];
    const long long n_units = static_cast<long long>(n_ranges) * a.nkv;
    const float qscale = a.scale * 1.4426950408889634f;  // scores in base 2
    const size_t plane = static_cast<size_t>(a.nkv) * P * HD;  // elements of the K (or V) half of a page

    for (long long u = static_cast<long long>(blockIdx.x) * GQW + warp; u < n_units; u += n_warps) {
        const int kvh = static_cast<int>(u % a.nkv);
        const int r = static_cast<int>(u / a.nkv);
        int item = 0;
        while (kr.pref[item + 1] <= r) ++item;
        const int split = r - kr.pref[item];
        const int seg = kr.seg[item], p = kr.pos[item], row = kr.row[item];
        const int t_lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
        const int k_begin = kr.first[item] + split * len;   // a multiple of 32
        const int k_end = min(p + 1, k_begin + len);        // exclusive
        const int* table = a.block_table + static_cast<size_t>(seg) * a.table_stride;
        const bf16* pool_kv = a.pool + static_cast<size_t>(kvh) * P * HD;

        // Q as B fragments: head gq (and gq + 8 in the second tile), dims 32 i + 8 t4 .. + 7 per piece; k-step 2i takes
        // the first two registers of piece i, k-step 2i + 1 the other two (the permutation that K shares)
        uint32_t qb[HT][KS][2];
        {
            const bf16* q0 = a.q + (static_cast<size_t>(row) * a.nh + static_cast<size_t>(kvh) * G) * HD + 8 * t4;
#pragma unroll
            for (int ht = 0; ht < HT; ++ht) {
                const int g = gq + 8 * ht;
#pragma unroll
                for (int i = 0; i < NL; ++i) {
                    const uint4 v = g < G ? ldg16(q0 + static_cast<size_t>(g) * HD + 32 * i) : make_uint4(0, 0, 0, 0);
                    qb[ht][2 * i][0] = v.x; qb[ht][2 * i][1] = v.y; qb[ht][2 * i + 1][0] = v.z; qb[ht][2 * i + 1][1] = v.w;
                }
            }
        }
        // O^T: row tile j holds dims 8 gq + 2 j + {0, 1} (j < 4) and 64 + 8 gq + 2 (j - 4) + {0, 1} in its rows gq and
        // gq + 8; columns are heads 2 t4 + {0, 1} of the head tile.  m, l: of this lane's two heads per tile
        // (l: this lane's share of the keys).
        float o[HT][MT][4];
        float m[HT][2], l[HT][2];
#pragma unroll
        for (int ht = 0; ht < HT; ++ht) {
#pragma unroll
            for (int j = 0; j < MT; ++j) o[ht][j][0] = o[ht][j][1] = o[ht][j][2] = o[ht][j][3] = 0.f;
            m[ht][0] = m[ht][1] = -INFINITY;
            l[ht][0] = l[ht][1] = 0.f;
        }

        // A stage of the warp's ring: the K tile [16 keys][hd], then the V tile, rows as they lie in the page.
        const uint32_t ring = smem_u32(gq_smem) + warp * (GQS * STAGE_BYTES);
        auto issue = [&](int k0, int st) {
            if (k0 < k_end && lane == 0) {
                const int page = table[k0 / P];
                const bf16* kbase = pool_kv + static_cast<size_t>(page) * 2 * plane + static_cast<size_t>(k0 % P) * HD;
                const uint32_t dst = ring + st * STAGE_BYTES, bar = bars + 8 * st;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // after this warp's own stores to the slot
                mbar_expect_tx(bar, 2 * TILE_BYTES);
                bulk_copy(dst, kbase, TILE_BYTES, bar);
                bulk_copy(dst + TILE_BYTES, kbase + plane, TILE_BYTES, bar);
            }
        };
        // the first chunk that holds a live key (a window may start up to 31 keys into the range's first 32)
        const int k_start = max(k_begin, t_lo & ~15);
        bool ok = true;
#pragma unroll
        for (int c = 0; c < GQS - 1; ++c) issue(k_start + 16 * c, c);
        int st = 0;
        for (int k0 = k_start; k0 < k_end; k0 += 16) {
            __syncwarp();  // every lane has read the chunk before this one: its slot may be overwritten
            {
                int st_new = st + GQS - 1;
                if (st_new >= GQS) st_new -= GQS;
                issue(k0 + 16 * (GQS - 1), st_new);
            }
            if (!mbar_wait(bars + 8 * st, (parity >> st) & 1u)) {  // the copies of chunk k0 have landed
                ok = false;
                break;
            }
            parity ^= 1u << st;
            const uint32_t src = ring + st * STAGE_BYTES;
            if (++st == GQS) st = 0;
            if (k0 < t_lo || k0 + 16 > k_end) {
                // a chunk with dead keys: their V rows become zeros (two lanes per row, 8 x 16 bytes of its 2 hd each)
                const int r = lane >> 1, t = k0 + r;
                if (t < t_lo || t >= k_end) {
#pragma unroll
                    for (int x = 0; x < ROW_BYTES / 32; ++x) sts16_zero(src + TILE_BYTES + r * ROW_BYTES + (lane & 1) * (ROW_BYTES / 2) + 16 * x);
                }
                __syncwarp();
            }
            // K as A fragments: rows are keys k0 + gq and k0 + 8 + gq; piece 4 i + t4 of the row
            uint4 k_lo[NL], k_hi[NL];
#pragma unroll
            for (int i = 0; i < NL; ++i) {
                k_lo[i] = lds16(src + gq * ROW_BYTES + (4 * i + t4) * 16);
                k_hi[i] = lds16(src + (gq + 8) * ROW_BYTES + (4 * i + t4) * 16);
            }
            // V: rows of keys k0 + 2 t4 + {0, 1} and k0 + 8 + 2 t4 + {0, 1}, piece gq + 8 i
            uint4 vreg[4][VL];
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const int r = (kk >> 1) * 8 + 2 * t4 + (kk & 1);
#pragma unroll
                for (int i = 0; i < VL; ++i) vreg[kk][i] = lds16(src + TILE_BYTES + r * ROW_BYTES + (gq + 8 * i) * 16);
            }
            const bool live_lo = k0 + gq >= t_lo && k0 + gq < k_end, live_hi = k0 + 8 + gq >= t_lo && k0 + 8 + gq < k_end;
            uint32_t pb[HT][2];
#pragma unroll
            for (int ht = 0; ht < HT; ++ht) {
                // S^T: two chains of MMAs over the k-steps, added at the end
                float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < NL; ++i) {
                    const uint32_t a_even[4] = {k_lo[i].x, k_hi[i].x, k_lo[i].y, k_hi[i].y};
                    const uint32_t a_odd[4] = {k_lo[i].z, k_hi[i].z, k_lo[i].w, k_hi[i].w};
                    mma_bf16(s0, a_even, qb[ht][2 * i][0], qb[ht][2 * i][1]);
                    mma_bf16(s1, a_odd, qb[ht][2 * i + 1][0], qb[ht][2 * i + 1][1]);
                }
                // s[0], s[1]: key k0 + gq, heads 2 t4 + {0, 1};  s[2], s[3]: key k0 + 8 + gq, the same heads
                float sc[4];
                sc[0] = live_lo ? (s0[0] + s1[0]) * qscale : -INFINITY;
                sc[1] = live_lo ? (s0[1] + s1[1]) * qscale : -INFINITY;
                sc[2] = live_hi ? (s0[2] + s1[2]) * qscale : -INFINITY;
                sc[3] = live_hi ? (s0[3] + s1[3]) * qscale : -INFINITY;
                float mx[2] = {fmaxf(sc[0], sc[2]), fmaxf(sc[1], sc[3])};
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 4));
                    mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 8));
                    mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 16));
                }
                float e[4];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float n = fmaxf(m[ht][c], mx[c]);
                    // a chunk without a live key (before a window's start) leaves the head as it was
                    const float corr = n == -INFINITY ? 1.f : exp2f(m[ht][c] - n);
                    m[ht][c] = n;
                    e[c] = n == -INFINITY ? 0.f : exp2f(sc[c] - n);
                    e[2 + c] = n == -INFINITY ? 0.f : exp2f(sc[2 + c] - n);
                    l[ht][c] = l[ht][c] * corr + e[c] + e[2 + c];
#pragma unroll
                    for (int j = 0; j < MT; ++j) {
                        o[ht][j][c] *= corr;
                        o[ht][j][2 + c] *= corr;
                    }
                }
                // P^T as the B fragment: the transpose of the accumulator layout, 8 keys at a time
                pb[ht][0] = movmatrix_trans(pack_bf16(e[0], e[1]));
                pb[ht][1] = movmatrix_trans(pack_bf16(e[2], e[3]));
            }
            // O^T += V^T . P^T: row tile j takes word j of this lane's value pieces (two consecutive dims); an A fragment
            // register holds one dim of two consecutive keys
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                const int i = j >> 2, w = j & 3;
                const uint32_t va = reinterpret_cast<const uint32_t*>(&vreg[0][i])[w], vb = reinterpret_cast<const uint32_t*>(&vreg[1][i])[w];
                const uint32_t vc = reinterpret_cast<const uint32_t*>(&vreg[2][i])[w], vd = reinterpret_cast<const uint32_t*>(&vreg[3][i])[w];
                const uint32_t af[4] = {__byte_perm(va, vb, 0x5410u), __byte_perm(va, vb, 0x7632u),
                                        __byte_perm(vc, vd, 0x5410u), __byte_perm(vc, vd, 0x7632u)};
#pragma unroll
                for (int ht = 0; ht < HT; ++ht) mma_bf16(o[ht][j], af, pb[ht][0], pb[ht][1]);
            }
        }
        if (!ok) return;  // a copy never came: the error word is set, the warp leaves (its other copies are lost with it)
        // partial results of the group's heads: head g of unit u is slot u * G + g.  A head's denominator lives in
        // the eight lanes of its column.
#pragma unroll
        for (int ht = 0; ht < HT; ++ht) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float lc = l[ht][c];
                lc += __shfl_xor_sync(0xffffffffu, lc, 4);
                lc += __shfl_xor_sync(0xffffffffu, lc, 8);
                lc += __shfl_xor_sync(0xffffffffu, lc, 16);
                const int g = 8 * ht + 2 * t4 + c;
                if (g < G) {
                    float* po = a.part_o + (static_cast<size_t>(u) * G + g) * HD + 8 * gq;
#pragma unroll
                    for (int jj = 0; jj < MT; jj += 2) {
                        // tiles jj and jj + 1: dims 2 (jj % 4) .. + 3 of this lane's run of eight (the second run is 64 on)
                        *reinterpret_cast<float4*>(po + 64 * (jj >> 2) + 2 * (jj & 3)) =
                            make_float4(o[ht][jj][c], o[ht][jj][2 + c], o[ht][jj + 1][c], o[ht][jj + 1][2 + c]);
                    }
                    if (gq == 0) {
                        a.part_ml[2 * (static_cast<size_t>(u) * G + g)] = m[ht][c];
                        a.part_ml[2 * (static_cast<size_t>(u) * G + g) + 1] = lc;
                    }
                }
            }
        }
        // the warp that finishes the last range of this (request, kv head) merges its heads' ranges
        __syncwarp();
        int last = 0;
        const int n_splits = kr.pref[item + 1] - kr.pref[item];
        if (lane == 0) {
            __threadfence();
            int* counter = a.counters + static_cast<size_t>(item) * a.nh + kvh;
            last = atomicAdd(counter, 1) == n_splits - 1;
            if (last) *counter = 0;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) continue;
        __threadfence();
        // two heads at a time, so that twice as many loads are in flight (the merge is a chain of loads)
        const size_t ustep = static_cast<size_t>(a.nkv) * G;
        for (int g = 0; g < G; g += 2) {
            const bool two = g + 1 < G;
            // range s of head g: slot ((pref + s) * nkv + kvh) * G + g
            const size_t u0 = (static_cast<size_t>(kr.pref[item]) * a.nkv + kvh) * G + g, u1 = u0 + (two ? 1 : 0);
            float M0 = -INFINITY, M1 = -INFINITY;
            for (int sidx = lane; sidx < n_splits; sidx += 32) {
                M0 = fmaxf(M0, __ldcg(a.part_ml + 2 * (u0 + sidx * ustep)));
                M1 = fmaxf(M1, __ldcg(a.part_ml + 2 * (u1 + sidx * ustep)));
            }
            M0 = warp_max(M0);
            M1 = warp_max(M1);
            for (int d = lane * 4; d < HD; d += 128) {
                float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
                float L0 = 0.f, L1 = 0.f;
#pragma unroll 8
                for (int sidx = 0; sidx < n_splits; ++sidx) {
                    const size_t us0 = u0 + sidx * ustep, us1 = u1 + sidx * ustep;
                    const float2 ml0 = __ldcg(reinterpret_cast<const float2*>(a.part_ml + 2 * us0));
                    const float2 ml1 = __ldcg(reinterpret_cast<const float2*>(a.part_ml + 2 * us1));
                    const float4 v0 = __ldcg(reinterpret_cast<const float4*>(a.part_o + us0 * HD + d));
                    const float4 v1 = __ldcg(reinterpret_cast<const float4*>(a.part_o + us1 * HD + d));
                    const float w0 = ml0.x == -INFINITY ? 0.f : exp2f(ml0.x - M0);
                    const float w1 = ml1.x == -INFINITY ? 0.f : exp2f(ml1.x - M1);
                    L0 = fmaf(ml0.y, w0, L0);
                    L1 = fmaf(ml1.y, w1, L1);
                    acc0.x = fmaf(v0.x, w0, acc0.x); acc0.y = fmaf(v0.y, w0, acc0.y);
                    acc0.z = fmaf(v0.z, w0, acc0.z); acc0.w = fmaf(v0.w, w0, acc0.w);
                    acc1.x = fmaf(v1.x, w1, acc1.x); acc1.y = fmaf(v1.y, w1, acc1.y);
                    acc1.z = fmaf(v1.z, w1, acc1.z); acc1.w = fmaf(v1.w, w1, acc1.w);
                }
                const float inv0 = 1.0f / L0, inv1 = 1.0f / L1;
                bf16* dst = a.out + (static_cast<size_t>(row) * a.nh + static_cast<size_t>(kvh) * G + g) * HD + d;
                dst[0] = from_f<bf16>(acc0.x * inv0);
                dst[1] = from_f<bf16>(acc0.y * inv0);
                dst[2] = from_f<bf16>(acc0.z * inv0);
                dst[3] = from_f<bf16>(acc0.w * inv0);
                if (two) {
                    dst[HD] = from_f<bf16>(acc1.x * inv1);
                    dst[HD + 1] = from_f<bf16>(acc1.y * inv1);
                    dst[HD + 2] = from_f<bf16>(acc1.z * inv1);
                    dst[HD + 3] = from_f<bf16>(acc1.w * inv1);
                }
            }
        }
    }
}

// Whether the kernel takes a case (the caller falls back to locus_attn_decode otherwise).
extern "C" int locus_attn_decode_gqa_takes(int dt, int nh, int nkv, int hd, int page_tokens, int n_items) {
    if (dt != LOCUS_DT_BF16 || nkv <= 0 || nh % nkv != 0) return 0;
    const int G = nh / nkv;
    return (G >= 2 && G <= 16 && (hd == 64 || hd == 128) && page_tokens % 16 == 0 && n_items <= DS_MAX_ITEMS) ? 1 : 0;
}

// Up to this many (request, key/value head) pairs the 6 x 4 shape runs; g_gqa_deep forces it on (1) or off (0) for
// tests and measurements (-1: by the number of pairs).
#define GQ_DEEP_PAIRS 48
static int g_gqa_deep = -1;
extern "C" void locus_attn_decode_gqa_set_deep(int deep) { g_gqa_deep = deep; }

// Scratch as for locus_attn_decode: part_o holds max_units partial results of hd floats (at least
// n_items * nh), part_ml two floats each, counters n_items * nh ints that are zero before and after the call.
extern "C" int locus_attn_decode_gqa(const void* q, const void* pool, void* out, const int* seg_q0, const int* seg_ctx,
                                     const int* block_table, int table_stride, const int* items, int n_items, int nh,
                                     int nkv, int hd, int page_tokens, int window, float scale, float* part_o,
                                     float* part_ml, int* counters, long long max_units, int cost_range,
                                     int cost_merge, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (!locus_attn_decode_gqa_takes(LOCUS_DT_BF16, nh, nkv, hd, page_tokens, n_items) || window < 0 || counters == nullptr)
        return LOCUS_ERR_UNSUPPORTED;
    if (max_units < static_cast<long long>(n_items) * nh) return LOCUS_ERR_UNSUPPORTED;
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) {
            n_sm = 0;
            return static_cast<int>(cudaGetLastError());
        }
    }
    GqaArgs a;
    a.q = static_cast<const bf16*>(q);
    a.pool = static_cast<const bf16*>(pool);
    a.out = static_cast<bf16*>(out);
    a.seg_q0 = seg_q0; a.seg_ctx = seg_ctx; a.block_table = block_table; a.table_stride = table_stride; a.items = items;
    a.nh = nh; a.nkv = nkv; a.page_tokens = page_tokens; a.window = window; a.scale = scale;
    a.part_o = part_o; a.part_ml = part_ml; a.counters = counters;
    const dim3 grid(n_sm);
    const bool wide = nh / nkv > 8;
    // few (request, key/value head) pairs: fewer warps with a deeper ring (a warp's chain of chunks sets the time);
    // many: more warps.  28 heads on 4 at 8,192 tokens, 6 x 4 against 10 x 2: 8 requests (32 pairs) 45.8 against
    // 54.5 us, 16 requests (64 pairs) 66.7 against 65.8, 64 requests 230 against 184; 16 heads on 2 at 4,000 tokens:
    // 16 requests (32 pairs) 35.7 against 42.6 us, 32 requests (64 pairs) 44.6 against 45.0
    const bool few = g_gqa_deep >= 0 ? g_gqa_deep != 0 : static_cast<long long>(n_items) * nkv <= GQ_DEEP_PAIRS;
#define GQA_LAUNCH_WS(HD_, WIDE_, W_, S_)                                                                              \
    do {                                                                                                               \
        const size_t smem = static_cast<size_t>(W_) * S_ * 2 * 16 * hd * 2;                                            \
        static bool attr_set = false;                                                                                  \
        if (!attr_set) {                                                                                               \
            if (cudaFuncSetAttribute(attn_decode_gqa_kernel<HD_, WIDE_, W_, S_>,                                       \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) \
                return static_cast<int>(cudaGetLastError());                                                           \
            attr_set = true;                                                                                           \
        }                                                                                                              \
        locus_launch(attn_decode_gqa_kernel<HD_, WIDE_, W_, S_>, grid, 32 * W_, smem, stream, a, n_items, max_units,   \
                     cost_range, cost_merge);                                                                          \
    } while (0)
#define GQA_LAUNCH(HD_, WIDE_)                                                                                         \
    do {                                                                                                               \
        if (few) GQA_LAUNCH_WS(HD_, WIDE_, 6, 4);                                                                      \
        else GQA_LAUNCH_WS(HD_, WIDE_, GQ_WARPS, GQ_STAGES);                                                           \
    } while (0)
    if (hd == 128) {
        if (wide) GQA_LAUNCH(128, true);
        else GQA_LAUNCH(128, false);
    } else {
        if (wide) GQA_LAUNCH(64, true);
        else GQA_LAUNCH(64, false);
    }
#undef GQA_LAUNCH_WS
#undef GQA_LAUNCH
    return locus_launch_status();
}
