// bfloat16 matrix products on the Blackwell tensor cores (tcgen05.mma, accumulators in
// tensor memory), operands staged in shared memory by TMA through a multi-stage mbarrier
// pipeline:  out = x . W^T  with the same fused epilogues as the CUDA-core kernel.
//
// Roles are swapped so that the WEIGHT rows are the 128-row M side of the MMA and the
// tokens are its N side (16..256 columns): a decode step with a handful of tokens streams
// each weight tile once at full tile height, and a prefill step uses 128- or 256-token tiles.
//
//   D[n, t] (tensor memory, lane n, column t) = sum_k W[n0 + n, k] * x[t0 + t, k]
//
// One CTA computes one 128 x TN output tile over the whole K (no split of K: the order of
// the sum for an element depends on K only).  Warp 0 issues TMA loads (one elected thread),
// warp 1 allocates tensor memory and issues the MMAs (one elected thread), warps 2-5 read
// the accumulators back (tcgen05.ld, each warp its own 32 lanes) and run the epilogue:
// bias, SwiGLU of two accumulators, per-row scale, store as bfloat16 / float32 or add into
// a float32 tensor.  Grouped products (experts) take the tile list that moe_sort built.
//
// Pairs (an option, off unless switched on: locus_gemm_tc_set_pair).  Two CTAs on neighbouring SMs (a
// cluster of two) work as one: tcgen05.mma.cta_group::2 multiplies 256 weight rows (128 from each CTA's shared
// memory) by the token tile, of which each CTA has loaded only half the rows, so a k-block costs a
// CTA a third less traffic from L2 for the same MMA work.  Each CTA keeps the accumulators of its own
// 128 weight rows in its own tensor memory and runs its own epilogue.  The CTA of rank 0 issues the
// MMAs; the loads of both CTAs count their bytes at rank 0's barrier of the stage, and rank 0's commits
// release the stage in both.  Measured on the products of a 2,048-token prefill step it is as fast as
// two independent CTAs per SM, not faster: the thread that issues the MMAs, not the traffic from L2,
// sets the pace there (an MMA instruction is accepted only when the tensor pipe has room: 4 MMAs of a
// k-block take about 560 cycles to issue, the whole loop about 700).
//
// Every wait on an mbarrier is bounded (about a second of clock cycles); when a wait runs
// out the kernel records a code in the module's error word, stops waiting and finishes, so
// a fault in the pipeline shows as an error on the host, never as a hang.  No load uses
// cluster multicast.
#include <cuda.h>

#include "common.cuh"

#define TILE_W 128      // weight rows per tile (MMA M)
#define TILE_K 64       // k elements per stage: 128 bytes of bfloat16, one swizzle row
#define A_BYTES (TILE_W * TILE_K * 2)
#define WAIT_LIMIT 2000000000LL

__device__ int g_tc_error = 0;

struct TcArgs {
    int M, N, K, TN, dual, stages, tmem_cols, pair, kps;
    int accumulate;
    void* out;
    int out_dt;
    long long ldo;
    const void* bias;
    int bias_dt;
    const float* row_scale;
    const int* scale_rows;
    const int* tile_expert;
    const int* tile_row0;
    const int* tile_rows;
    const int* n_tiles;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
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

__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Bounded wait: false (and the error word set to `code`) when the limit runs out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > WAIT_LIMIT) {
            atomicCAS(&g_tc_error, 0, code);
            return false;
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

// The load of the second CTA of a pair: the data goes to its own shared memory, the bytes are counted
// at the barrier at the same place in the FIRST CTA's shared memory (cta_group::2 allows a barrier of
// the other CTA of the pair; no multicast).
__device__ __forceinline__ void tma_load_2d_to_leader(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "{\n\t.reg .b32 rb;\n\t"
        "mapa.shared::cluster.u32 rb, %4, 0;\n\t"
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [rb];\n\t}"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    // K-major, 128-byte swizzle: 8 rows of 128 bytes per swizzle atom, atoms 1024 bytes apart
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);   // start address
    d |= static_cast<uint64_t>(1) << 16;                   // leading byte offset (unused with swizzle)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;           // stride byte offset between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;                   // descriptor version of sm_100
    d |= static_cast<uint64_t>(2) << 61;                   // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// The pair's forms: one MMA over both CTAs' operands, and a commit that arrives at the barrier at
// this place in both CTAs.
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}

__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(static_cast<uint16_t>(3))
        : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}

// PAIR: the form for clusters of two CTAs.  (A kernel that contains cta_group::2 instructions can only
// be launched in such clusters, hence two instantiations.)
template <bool PAIR>
__global__ void __launch_bounds__(192, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
               const __grid_constant__ CUtensorMap map_x, TcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = PAIR ? (blockIdx.x & 1) : 0;  // place in the pair (the cluster is 2 x 1 x 1)

    int x_row0, rows_valid;
    long long w_row0 = static_cast<long long>(blockIdx.x) * TILE_W;
    if (a.tile_expert != nullptr) {
        const int tile = blockIdx.y;
        if (tile >= *a.n_tiles) return;  // uniform for the whole block
        x_row0 = a.tile_row0[tile];
        rows_valid = a.tile_rows[tile];
        w_row0 += static_cast<long long>(a.tile_expert[tile]) * a.N;
    } else {
        x_row0 = blockIdx.y * a.TN;
        rows_valid = min(a.TN, a.M - x_row0);
    }

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    const uint32_t x_bytes = static_cast<uint32_t>(PAIR ? a.TN / 2 : a.TN) * TILE_K * 2;  // a pair: half the rows each
    // a stage holds a.kps k-blocks ("sub-stages": weights, second weights, tokens, each of one k-block)
    const uint32_t sub_bytes = A_BYTES * (1 + a.dual) + x_bytes;
    const uint32_t stage_bytes = a.kps * sub_bytes;
    const uint32_t bars = base + a.stages * stage_bytes;
    // barriers: full[s] at bars + 8 s, empty[s] at bars + 8 (stages + s), accumulator-ready, then the TMEM slot
    const uint32_t bar_full = bars, bar_empty = bars + 8 * a.stages, bar_acc = bars + 16 * a.stages;
    const uint32_t slot = bar_acc + 8;
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (slot - smem_u32(smem_raw)));

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {  // warp 1 of both CTAs, the same slot in both
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(a.tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(a.tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (PAIR) cluster_sync();  // the other CTA's barriers are initialised before anything arrives at them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *slot_ptr;
    const int nkb = (a.K + TILE_K - 1) / TILE_K;

    // MMA N covers only the valid token rows of this tile, rounded up to 16: a ragged last tile (or an
    // expert with few rows) costs MMA time for its rows, not for the whole tile.  In a pair the MMA takes
    // the first n_mma / 2 token rows from each CTA, so rank 1 loads the rows from x_row0 + n_mma / 2 on.
    const int n_mma = min(a.TN, (rows_valid + 15) & ~15);
    if (warp == 0) {
        if (lane == 0) {
            const int x_first = x_row0 + rank * (n_mma / 2);
            int s = 0;
            uint32_t round = 0;  // how often the ring has wrapped (its low bit is the barriers' phase)
            for (int kb = 0; kb < nkb; kb += a.kps, ++s) {
                if (s == a.stages) {
                    s = 0;
                    ++round;
                }
                mbar_wait(bar_empty + 8 * s, (round & 1) ^ 1, 1);
                const int nsub = min(a.kps, nkb - kb);
                if (!(PAIR && rank == 1))  // rank 0's barrier counts the bytes of both CTAs of a pair
                    mbar_expect_tx(bar_full + 8 * s, (PAIR ? 2 : 1) * nsub * sub_bytes);
                for (int j = 0; j < nsub; ++j) {
                    const uint32_t st = base + s * stage_bytes + j * sub_bytes;
                    const int k0 = (kb + j) * TILE_K;
                    if (PAIR && rank == 1) {
                        tma_load_2d_to_leader(st, &map_w, k0, static_cast<int>(w_row0), bar_full + 8 * s);
                        if (a.dual) tma_load_2d_to_leader(st + A_BYTES, &map_w2, k0, static_cast<int>(w_row0), bar_full + 8 * s);
                        tma_load_2d_to_leader(st + A_BYTES * (1 + a.dual), &map_x, k0, x_first, bar_full + 8 * s);
                    } else {
                        tma_load_2d(st, &map_w, k0, static_cast<int>(w_row0), bar_full + 8 * s);
                        if (a.dual) tma_load_2d(st + A_BYTES, &map_w2, k0, static_cast<int>(w_row0), bar_full + 8 * s);
                        tma_load_2d(st + A_BYTES * (1 + a.dual), &map_x, k0, x_first, bar_full + 8 * s);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {  // rank 0 issues the MMAs of a pair
            // instruction descriptor: f32 accumulate, bf16 x bf16, both operands K-major, N = n_mma,
            // M = 128 (256 over a pair)
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n_mma >> 3) << 17) |
                                   (static_cast<uint32_t>((PAIR ? 2 * TILE_W : TILE_W) >> 4) << 24);
            // The thread that issues the MMAs is the pace-maker of the tile: an MMA is accepted only when
            // the tensor pipe has room, so whatever this thread does between the last MMA of one k-block
            // and the first of the next is time the pipe may stand idle.  Hence: no divisions, descriptors
            // advanced by addition, and the barrier of the next stage is looked at right after this stage's
            // MMAs went out (while they run), so that the wait at the top of the loop is usually over.
            const uint64_t desc0 = make_desc(base);
            const uint64_t stage_units = stage_bytes >> 4;  // descriptors count in 16-byte units
            const uint64_t sub_units = sub_bytes >> 4;
            const uint64_t w2_units = A_BYTES >> 4, x_units = (A_BYTES * (1 + a.dual)) >> 4;
            int s = 0;
            uint32_t round = 0;
            bool ready = mbar_try_wait(bar_full, 0);
            for (int kb = 0; kb < nkb; kb += a.kps) {
                if (!ready) mbar_wait(bar_full + 8 * s, round & 1, 2);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int nsub = min(a.kps, nkb - kb);
                for (int j = 0; j < nsub; ++j) {
                    const uint64_t dw = desc0 + s * stage_units + j * sub_units, dw2 = dw + w2_units, dx = dw + x_units;
                    if (PAIR) {
#pragma unroll
                        for (int k4 = 0; k4 < TILE_K / 16; ++k4) {
                            const uint32_t acc = (kb + j > 0 || k4 > 0) ? 1u : 0u;
                            umma_bf16_pair(tmem, dw + 2 * k4, dx + 2 * k4, idesc, acc);  // 16 elements = 32 bytes = 2 units
                            if (a.dual) umma_bf16_pair(tmem + a.TN, dw2 + 2 * k4, dx + 2 * k4, idesc, acc);
                        }
                    } else {
#pragma unroll
                        for (int k4 = 0; k4 < TILE_K / 16; ++k4) {
                            const uint32_t acc = (kb + j > 0 || k4 > 0) ? 1u : 0u;
                            umma_bf16(tmem, dw + 2 * k4, dx + 2 * k4, idesc, acc);
                            if (a.dual) umma_bf16(tmem + a.TN, dw2 + 2 * k4, dx + 2 * k4, idesc, acc);
                        }
                    }
                }
                // the stage is free when these MMAs have read it (in both CTAs of a pair)
                if (PAIR) umma_commit_pair(bar_empty + 8 * s); else umma_commit(bar_empty + 8 * s);
                if (++s == a.stages) {
                    s = 0;
                    ++round;
                }
                ready = kb + a.kps < nkb && mbar_try_wait(bar_full + 8 * s, round & 1);
            }
            if (PAIR) umma_commit_pair(bar_acc); else umma_commit(bar_acc);
        }
    } else {
        const int quarter = warp & 3;  // tensor-memory lanes this warp may read
        const int row = quarter * 32 + lane;
        const long long n = static_cast<long long>(blockIdx.x) * TILE_W + row;  // output column
        const bool n_ok = n < a.N;
        // while the MMAs run: the scale of every token row of the tile -> shared memory
        float* scales = reinterpret_cast<float*>(smem_raw + (slot + 16 - smem_u32(smem_raw)));
        if (a.row_scale) {
            for (int c = threadIdx.x - 64; c < a.TN; c += 128) {
                const int r = x_row0 + c;
                scales[c] = c < rows_valid ? a.row_scale[a.scale_rows ? a.scale_rows[r] : r] : 0.f;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
        }
        const float bias = (a.bias && n_ok) ? ld_dyn(a.bias, a.bias_dt, n) : 0.f;
        // Wide stores: the warp's 32 output columns x 16 token rows go through a small transpose in
        // shared memory so that a lane writes 8 consecutive columns of one token (16 or 32 bytes).
        // Needs rows of out that start on 16-byte boundaries and a full 32-column stripe.
        float* stage = reinterpret_cast<float*>(smem_raw + ((slot + 16 + 4 * a.TN + 15) & ~15u) - smem_u32(smem_raw)) +
                       (warp - 2) * (16 * 36);
        const long long n_warp = static_cast<long long>(blockIdx.x) * TILE_W + quarter * 32;
        const int esize = a.out_dt == LOCUS_DT_F32 ? 4 : 2;
        const bool wide = n_warp + 32 <= a.N && (a.ldo * esize) % 16 == 0 &&
                          (reinterpret_cast<uintptr_t>(a.out) & 15) == 0;
        mbar_wait(bar_acc, 0, 3);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
        float* outf = static_cast<float*>(a.out);
        for (int c0 = 0; c0 < a.TN; c0 += 16) {
            if (c0 >= rows_valid) break;  // uniform
            uint32_t v[16], u[16];
            tmem_ld16(lane_addr + c0, v);
            if (a.dual) tmem_ld16(lane_addr + a.TN + c0, u);
            // narrow add-into epilogue: fetch the 16 old values while the accumulators arrive
            float old[16];
            if (a.accumulate && !wide) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const bool ok = n_ok && c0 + j < rows_valid;
                    old[j] = ok ? outf[static_cast<size_t>(x_row0 + c0 + j) * a.ldo + n] : 0.f;
                }
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            float val[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                float x = __uint_as_float(v[j]);
                if (a.dual) {
                    const float g = x;
                    x = g / (1.0f + expf(-g)) * __uint_as_float(u[j]);
                }
                x += bias;
                if (a.row_scale) x *= scales[c0 + j];
                val[j] = x;
            }
            if (wide) {
#pragma unroll
                for (int j = 0; j < 16; ++j) stage[j * 36 + lane] = val[j];
                __syncwarp();
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int j = (lane >> 2) + 8 * half;
                    if (c0 + j < rows_valid) {
                        const int c = (lane & 3) * 8;
                        const float4 lo = *reinterpret_cast<const float4*>(stage + j * 36 + c);
                        const float4 hi = *reinterpret_cast<const float4*>(stage + j * 36 + c + 4);
                        const size_t o = static_cast<size_t>(x_row0 + c0 + j) * a.ldo + n_warp + c;
                        if (a.out_dt == LOCUS_DT_F32) {
                            float4* dst = reinterpret_cast<float4*>(outf + o);
                            if (a.accumulate) {
                                const float4 p0 = dst[0], p1 = dst[1];
                                dst[0] = make_float4(p0.x + lo.x, p0.y + lo.y, p0.z + lo.z, p0.w + lo.w);
                                dst[1] = make_float4(p1.x + hi.x, p1.y + hi.y, p1.z + hi.z, p1.w + hi.w);
                            } else {
                                dst[0] = lo;
                                dst[1] = hi;
                            }
                        } else {
                            __nv_bfloat162 b0 = __floats2bfloat162_rn(lo.x, lo.y), b1 = __floats2bfloat162_rn(lo.z, lo.w);
                            __nv_bfloat162 b2 = __floats2bfloat162_rn(hi.x, hi.y), b3 = __floats2bfloat162_rn(hi.z, hi.w);
                            uint4 pk;
                            pk.x = *reinterpret_cast<uint32_t*>(&b0);
                            pk.y = *reinterpret_cast<uint32_t*>(&b1);
                            pk.z = *reinterpret_cast<uint32_t*>(&b2);
                            pk.w = *reinterpret_cast<uint32_t*>(&b3);
                            *reinterpret_cast<uint4*>(static_cast<bf16*>(a.out) + o) = pk;
                        }
                    }
                }
                __syncwarp();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (c0 + j >= rows_valid || !n_ok) continue;
                    const size_t o = static_cast<size_t>(x_row0 + c0 + j) * a.ldo + n;
                    if (a.accumulate) {
                        outf[o] = old[j] + val[j];
                    } else {
                        st_dyn(a.out, a.out_dt, o, val[j]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (PAIR) cluster_sync();  // neither CTA leaves while the other may still reach into it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (PAIR) {
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(a.tmem_cols) : "memory");
        } else {
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(a.tmem_cols) : "memory");
        }
    }
}

// ---------------------------------------------------------------------------
// host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    }
    return fn;
}

// rows x K bfloat16 matrix, row stride ld elements; box = box_rows x 64 elements, 128-byte swizzle.
// Rows and k beyond the matrix read as zero.
static bool make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {TILE_K, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Shared-memory budget of the pipeline in KiB; 0 = chosen from the grid size (see below).
static int g_budget_kb = 0;
// Pairs of CTAs on (1) or off (0).
static int g_pair = 0;
// k-blocks per pipeline stage (1 or 2): with 2 a barrier round covers 8 MMAs instead of 4.
static int g_kps = 1;
extern "C" void locus_gemm_tc_set_kps(int k) { g_kps = k == 2 ? 2 : 1; }
extern "C" void locus_gemm_tc_set_pair(int on) { g_pair = on; }
extern "C" void locus_gemm_tc_set_budget_kb(int kb) { g_budget_kb = kb; }

static int pow2_at_least(int v) {
    int p = 32;
    while (p < v) p <<= 1;
    return p;
}

// x [x_rows_total, K] bfloat16 (row stride ldx), w (and w2) [w_rows_total, K] bfloat16 contiguous.
// Plain product: M rows of x, N = w_rows_total.  Grouped: w holds E experts of N rows each,
// x rows are the expert-sorted pairs, the tile list has tiles of TN rows.
// TN: token tile, a multiple of 16 in 16..256 (dual: at most 128... 256 columns of tensor memory each).
extern "C" int locus_gemm_tc(const void* x, long long x_rows_total, long long ldx, const void* w, const void* w2,
                             long long w_rows_total, const void* bias, int bias_dt, void* out, int out_dt,
                             int accumulate, const float* row_scale, const int* scale_rows, int M, int N, int K,
                             long long ldo, int TN, const int* tile_expert, const int* tile_row0,
                             const int* tile_rows, const int* n_tiles, int max_tiles, cudaStream_t stream) {
    const int dual = w2 != nullptr ? 1 : 0;
    if (N <= 0 || K <= 0 || K % 8 != 0 || ldx % 8 != 0) return LOCUS_ERR_UNSUPPORTED;
    if (TN < 16 || TN > 256 || TN % 16 != 0 || (dual && TN > 256)) return LOCUS_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(w2)) & 15)
        return LOCUS_ERR_UNSUPPORTED;
    if (accumulate && out_dt != LOCUS_DT_F32) return LOCUS_ERR_UNSUPPORTED;
    if (w_rows_total >= (1LL << 31) || x_rows_total >= (1LL << 31)) return LOCUS_ERR_UNSUPPORTED;
    CUtensorMap map_w, map_w2, map_x;
    if (!make_map(&map_w, w, w_rows_total, K, K, TILE_W)) return LOCUS_ERR_UNSUPPORTED;
    if (!make_map(&map_w2, dual ? w2 : w, w_rows_total, K, K, TILE_W)) return LOCUS_ERR_UNSUPPORTED;
    // pairs of CTAs (see the head of the file) wherever there are two weight tiles to pair
    const int pair = (g_pair && N > TILE_W) ? 1 : 0;
    if (!make_map(&map_x, x, x_rows_total, K, ldx, pair ? TN / 2 : TN)) return LOCUS_ERR_UNSUPPORTED;
    TcArgs a;
    a.M = M; a.N = N; a.K = K; a.TN = TN; a.dual = dual; a.pair = pair;
    const int kps = g_kps;
    a.kps = kps;
    const int stage_bytes = kps * (A_BYTES * (1 + dual) + (pair ? TN / 2 : TN) * TILE_K * 2);
    const int tiles_y = tile_expert ? max_tiles : ceil_div(M, TN);
    const long long n_blocks = static_cast<long long>(ceil_div(N, TILE_W)) * tiles_y;
    // A grid of more than one block per SM runs two blocks per SM (the epilogue of one overlaps
    // the MMAs of the other): half the shared memory each.  A small grid gets deep pipelines.
    const int budget = g_budget_kb > 0 ? g_budget_kb * 1024 : (n_blocks > 160 ? 100 * 1024 : 200 * 1024);
    int stages = budget / stage_bytes;
    if (stages > 12) stages = 12;
    if (stages < 2) stages = 2;
    const int nkb = (K + TILE_K - 1) / TILE_K;
    if (stages > (nkb + kps - 1) / kps) stages = (nkb + kps - 1) / kps;
    if (stages < 1) return LOCUS_ERR_UNSUPPORTED;
    a.stages = stages;
    a.tmem_cols = pow2_at_least(TN * (1 + dual));
    if (a.tmem_cols > 512) return LOCUS_ERR_UNSUPPORTED;
    a.accumulate = accumulate; a.out = out; a.out_dt = out_dt; a.ldo = ldo; a.bias = bias; a.bias_dt = bias_dt;
    a.row_scale = row_scale; a.scale_rows = scale_rows; a.tile_expert = tile_expert; a.tile_row0 = tile_row0;
    a.tile_rows = tile_rows; a.n_tiles = n_tiles;
    const size_t smem = static_cast<size_t>(stages) * stage_bytes + 16 * stages + 64 + 4 * TN + 4 * 16 * 36 * 4 + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
            return static_cast<int>(cudaGetLastError());
        attr_set = true;
    }
    if (tiles_y <= 0) return 0;
    if (tiles_y > 65535) return LOCUS_ERR_UNSUPPORTED;
    dim3 grid(ceil_div(N, TILE_W), tiles_y);
    if (pair) grid.x = (grid.x + 1) & ~1u;  // whole pairs: a last CTA without weight rows computes zeros and stores nothing
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pair ? 1 : 0;
    if (pair) {
        cudaLaunchKernelEx(&cfg, gemm_tc_kernel<true>, map_w, map_w2, map_x, a);
    } else {
        cudaLaunchKernelEx(&cfg, gemm_tc_kernel<false>, map_w, map_w2, map_x, a);
    }
    return locus_launch_status();
}

// Reads and clears the module's error word (0 = no bounded wait ran out).  Synchronises.
extern "C" int locus_gemm_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    return v;
}
