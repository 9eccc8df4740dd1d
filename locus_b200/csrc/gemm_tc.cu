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
// A 128 x TN output tile is computed over the whole K by one CTA (no split of K: the order of
// the sum for an element depends on K only).  The kernel is persistent: one CTA per SM walks
// over the tiles in a fixed stride.  Warp 0 issues TMA loads (one elected thread) and runs
// ahead across tile boundaries, so the pipeline never drains between tiles; warp 1 allocates
// tensor memory and issues the MMAs (one elected thread) into one of TWO accumulator buffers;
// warps 2-5 read the other buffer back (tcgen05.ld, each warp its own 32 lanes) and run the
// epilogue while the next tile's MMAs run: bias, SwiGLU of two accumulators, per-row scale,
// store as bfloat16 / float32 or add into a float32 tensor, through a small transpose in shared
// memory so that stores are 16 or 32 bytes wide.  Grouped products (experts) take the tile list
// that moe_sort built.
//
// What sets the pace (measured with clock stamps in the kernel, taken out again): the thread
// that issues the MMAs -- an MMA is accepted only when the tensor pipe has room, 4 MMAs of a
// k-block take about 560 cycles to issue and the whole loop about 700 -- and the epilogue, which
// must stay well below the main loop of a tile to hide behind it.  Hence the lean issue loop,
// and the SwiGLU switch as a template parameter: as a run-time flag the compiler evaluated the
// SwiGLU arithmetic for every product and selected afterwards, which made the epilogue as long
// as the main loop.
//
// Every wait on an mbarrier is bounded (about a second of clock cycles); when a wait runs
// out the kernel records a code in the module's error word, stops waiting and finishes, so
// a fault in the pipeline shows as an error on the host, never as a hang.  Every TMA load goes
// to the shared memory of the block that issued it; nothing is sent to other blocks.
#include <cuda.h>

#include "common.cuh"
#include <string.h>

#define TILE_W 128      // weight rows per tile (MMA M)
#define TILE_K 64       // k elements per stage: 128 bytes of bfloat16, one swizzle row
#define A_BYTES (TILE_W * TILE_K * 2)
#define WAIT_LIMIT 2000000000LL

__device__ int g_tc_error = 0;

// Tensor maps of the activations with boxes of 16, 32, 64, 96, ... 256 rows: a tile fetches the
// smallest box that covers its live rows (the tile of an expert with a handful of rows would
// otherwise pull a whole token tile through L2 for every k-block).
#define X_BOXES 9
struct XMaps {
    CUtensorMap m[X_BOXES];
};
__host__ __device__ __forceinline__ int x_box_index(int rows) { return rows <= 16 ? 0 : (rows + 31) / 32; }
__host__ __device__ __forceinline__ int x_box_rows(int index) { return index == 0 ? 16 : 32 * index; }

struct TileGeom {
    int x_row0, rows_valid, tx, w_row0;  // first token row, live token rows, weight tile, first weight row
    int kb0, kb1;   // k-blocks of this unit of work (all of them unless the product is split along K)
    int out_row0;   // first row of the tile in out (x_row0, or the split's rows in the scratch)
};

struct TcArgs {
    int M, N, K, TN, dual, stages, tmem_cols, tiles_x, tiles_y, acc_bufs;
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
    // A product with few tiles is split along K so that every SM has work: split s of a tile sums k-blocks
    // [s * kb_per_split, ...) and stores its float32 sums to rows [s * M, (s + 1) * M) of the scratch that
    // out then points to; splitk_reduce_kernel adds the splits up in order and does the epilogue.
    int splits, kb_per_split;
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

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}

// Persistent kernel: a block walks over output tiles (tile index t = blockIdx.x, + gridDim.x, ...;
// the token tile varies fastest so that blocks running at the same time share weight tiles in L2).
// The loader runs ahead across tile boundaries, so the pipeline never drains between tiles, and
// two accumulator buffers in tensor memory let the MMAs of the next tile run while the epilogue
// warps drain this one.
template <bool DUAL>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
               const __grid_constant__ XMaps maps_x, TcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int tiles_y = a.tiles_y;
    const int n_y = a.tile_expert != nullptr ? min(tiles_y, *a.n_tiles) : tiles_y;  // live token tiles
    // only live tiles are numbered, so that every block gets the same number of them (within one)
    const long long n_total = static_cast<long long>(a.tiles_x) * n_y * a.splits;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    const uint32_t x_bytes = static_cast<uint32_t>(a.TN) * TILE_K * 2;
    const uint32_t stage_bytes = A_BYTES * (1 + DUAL) + x_bytes;
    const uint32_t bars = base + a.stages * stage_bytes;
    // barriers: full[s], empty[s], accumulator full[2], accumulator empty[2], then the TMEM slot
    const uint32_t bar_full = bars, bar_empty = bars + 8 * a.stages;
    const uint32_t bar_acc_full = bars + 16 * a.stages, bar_acc_empty = bar_acc_full + 16;
    const uint32_t slot = bar_acc_empty + 16;
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (slot - smem_u32(smem_raw)));
    const int acc_cols = a.TN * (1 + DUAL);  // columns of one accumulator buffer

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 4);  // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *slot_ptr;
    const int nkb = (a.K + TILE_K - 1) / TILE_K;

    // Per-tile geometry, the same for every role.  For grouped products it comes from the tile list in
    // global memory; every role fetches it a tile or more ahead so that the latency of those loads
    // falls into the work on the tile before.
    auto tile_geom = [&](long long t) -> TileGeom {
        TileGeom g;
        g.x_row0 = 0;
        g.rows_valid = 0;
        g.tx = 0;
        g.w_row0 = 0;
        g.kb0 = g.kb1 = 0;
        g.out_row0 = 0;
        if (t >= n_total) return g;  // past the end: an empty tile, never worked on
        int ti = static_cast<int>(t);  // the host refuses products of 2^31 tiles or more
        int split = 0;
        if (a.splits > 1) {  // the splits of a tile run side by side
            split = ti % a.splits;
            ti /= a.splits;
        }
        g.kb0 = split * a.kb_per_split;
        g.kb1 = min(nkb, g.kb0 + a.kb_per_split);
        const int ty = ti / a.tiles_x;  // blocks that run together share a token tile
        g.tx = ti - ty * a.tiles_x;
        g.w_row0 = g.tx * TILE_W;
        if (a.tile_expert != nullptr) {
            g.x_row0 = a.tile_row0[ty];
            g.rows_valid = a.tile_rows[ty];
            g.w_row0 += a.tile_expert[ty] * a.N;  // the host refuses weights of 2^31 rows or more
        } else {
            g.x_row0 = ty * a.TN;
            g.rows_valid = min(a.TN, a.M - g.x_row0);
        }
        g.out_row0 = g.x_row0 + split * a.M;
        return g;
    };
    const long long t_step = gridDim.x;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;          // stage of the ring, running over all tiles
            uint32_t round = 0;  // how often the ring has wrapped (its low bit is the barriers' phase)
            bool ok = true;      // false once a bounded wait ran out: the role stops
            TileGeom g = tile_geom(blockIdx.x);
            for (long long t = blockIdx.x; t < n_total && ok; t += t_step) {
                const TileGeom g_next = tile_geom(t + t_step);
                const int x_row0 = g.x_row0, w_row0 = g.w_row0;
                const int box = x_box_index(g.rows_valid);
                const CUtensorMap* map_x = &maps_x.m[box];
                const uint32_t bytes = A_BYTES * (1 + DUAL) + static_cast<uint32_t>(min(x_box_rows(box), a.TN)) * (TILE_K * 2);
                const int kb_end = g.kb1;
                for (int kb = g.kb0; kb < kb_end; ++kb) {
                    if (!mbar_wait(bar_empty + 8 * s, (round & 1) ^ 1, 1)) {
                        ok = false;
                        break;
                    }
                    const uint32_t st = base + s * stage_bytes;
                    mbar_expect_tx(bar_full + 8 * s, bytes);
                    tma_load_2d(st, &map_w, kb * TILE_K, w_row0, bar_full + 8 * s);
                    if (DUAL) tma_load_2d(st + A_BYTES, &map_w2, kb * TILE_K, w_row0, bar_full + 8 * s);
                    tma_load_2d(st + A_BYTES * (1 + DUAL), map_x, kb * TILE_K, x_row0, bar_full + 8 * s);
                    if (++s == a.stages) {
                        s = 0;
                        ++round;
                    }
                }
                g = g_next;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // This thread sets the pace of the block: an MMA is accepted only when the tensor pipe has room,
            // so what the thread does between the last MMA of one k-block and the first of the next is time
            // the pipe may stand idle.  Hence no divisions, descriptors advanced by addition, and a look at
            // the next stage's barrier right after this stage's MMAs went out.
            unsigned n_done = 0;
            int s = 0, buf = 0;
            uint32_t round = 0, acc_round = 0;
            bool ok = true;
            const uint64_t desc0 = make_desc(base);
            const uint64_t stage_units = stage_bytes >> 4;  // descriptors count in 16-byte units
            const uint64_t w2_units = A_BYTES >> 4, x_units = (A_BYTES * (1 + DUAL)) >> 4;
            bool ready = false;
            TileGeom g = tile_geom(blockIdx.x);
            for (long long t = blockIdx.x; t < n_total && ok; t += t_step) {
                const TileGeom g_next = tile_geom(t + t_step);
                const int rows_valid = g.rows_valid, kb_first = g.kb0, kb_end = g.kb1;
                g = g_next;
                // the epilogue must have drained this buffer (acc_bufs tiles ago)
                if (!mbar_wait(bar_acc_empty + 8 * buf, (acc_round & 1) ^ 1, 4)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // instruction descriptor: f32 accumulate, bf16 x bf16, both operands K-major, M = 128; N covers
                // only the valid token rows of this tile, rounded up to 16: a ragged tile (or an expert with
                // few rows) costs MMA time for its rows, not for the whole tile
                const int n_mma = min(a.TN, (rows_valid + 15) & ~15);
                const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n_mma >> 3) << 17) |
                                       (static_cast<uint32_t>(TILE_W >> 4) << 24);
                const uint32_t d0 = tmem + buf * acc_cols;
                for (int kb = kb_first; kb < kb_end; ++kb) {
                    if (!ready && !mbar_wait(bar_full + 8 * s, round & 1, 2)) {
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t dw = desc0 + s * stage_units, dw2 = dw + w2_units, dx = dw + x_units;
#pragma unroll
                    for (int k4 = 0; k4 < TILE_K / 16; ++k4) {
                        const uint32_t acc = (kb > kb_first || k4 > 0) ? 1u : 0u;
                        umma_bf16(d0, dw + 2 * k4, dx + 2 * k4, idesc, acc);  // 16 elements = 32 bytes = 2 units
                        if (DUAL) umma_bf16(d0 + a.TN, dw2 + 2 * k4, dx + 2 * k4, idesc, acc);
                    }
                    umma_commit(bar_empty + 8 * s);  // the stage is free when these MMAs have read it
                    if (++s == a.stages) {
                        s = 0;
                        ++round;
                    }
                    ready = mbar_try_wait(bar_full + 8 * s, round & 1);  // (past the last stage: simply not ready)
                }
                if (!ok) break;
                umma_commit(bar_acc_full + 8 * buf);
                ++n_done;
                if (++buf == a.acc_bufs) {
                    buf = 0;
                    ++acc_round;
                }
            }
        }
    } else {
        const int quarter = warp & 3;  // tensor-memory lanes this warp may read
        const int row = quarter * 32 + lane;
        // each epilogue warp keeps its own copy of the tile's row scales: no barrier between the warps
        float* scales = reinterpret_cast<float*>(smem_raw + (slot + 16 - smem_u32(smem_raw))) + (warp - 2) * a.TN;
        float* stage = reinterpret_cast<float*>(smem_raw + ((slot + 16 + 16 * a.TN + 15) & ~15u) - smem_u32(smem_raw)) +
                       (warp - 2) * (16 * 36);
        const int esize = a.out_dt == LOCUS_DT_F32 ? 4 : 2;
        const bool rows_aligned = (a.ldo * esize) % 16 == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0;
        float* outf = static_cast<float*>(a.out);
        unsigned n_done = 0;
        int buf = 0;
        uint32_t acc_round = 0;
        // Row scales come through two dependent loads (row index, then scale) behind the tile list: the
        // lane holds the scales of this tile, the row indices of the next and the geometry of the two
        // after it, each fetched one tile before it is needed.
        constexpr int NS = 256 / 32;  // token rows of a tile per lane
        TileGeom g = tile_geom(blockIdx.x), g1 = tile_geom(blockIdx.x + t_step), g2 = tile_geom(blockIdx.x + 2 * t_step);
        auto scale_index = [&](const TileGeom& q, int k) -> int {
            const int c = lane + 32 * k;
            if (c >= q.rows_valid) return -1;
            return a.scale_rows ? a.scale_rows[q.x_row0 + c] : q.x_row0 + c;
        };
        float sc[NS];
        int idx1[NS];
        if (a.row_scale) {
#pragma unroll
            for (int k = 0; k < NS; ++k) {
                const int i0 = scale_index(g, k);
                sc[k] = i0 >= 0 ? a.row_scale[i0] : 0.f;
                idx1[k] = scale_index(g1, k);
            }
        }
        for (long long t = blockIdx.x; t < n_total; t += t_step) {
            const TileGeom g3 = tile_geom(t + 3 * t_step);
            const int rows_valid = g.rows_valid, tx = g.tx;
            const int x_row0 = g.out_row0;  // rows of out; the row scales go by the token rows (scale_index)
            const long long n = static_cast<long long>(tx) * TILE_W + row;  // output column of this lane
            const bool n_ok = n < a.N;
            if (a.row_scale) {
#pragma unroll
                for (int k = 0; k < NS; ++k) {
                    if (lane + 32 * k < a.TN) scales[lane + 32 * k] = sc[k];
                }
                __syncwarp();
#pragma unroll
                for (int k = 0; k < NS; ++k) {
                    sc[k] = idx1[k] >= 0 ? a.row_scale[idx1[k]] : 0.f;  // the next tile's
                    idx1[k] = scale_index(g2, k);                        // the one after
                }
            }
            g = g1;
            g1 = g2;
            g2 = g3;
            const float bias = (a.bias && n_ok) ? ld_dyn(a.bias, a.bias_dt, n) : 0.f;
            // Wide stores: the warp's 32 output columns x 16 token rows go through a small transpose in
            // shared memory so that a lane writes 8 consecutive columns of one token (16 or 32 bytes).
            const long long n_warp = static_cast<long long>(tx) * TILE_W + quarter * 32;
            const bool wide = rows_aligned && n_warp + 32 <= a.N;
            // Add-into with wide stores reads the old values of out: those loads do not depend on the
            // accumulators, so they are issued one 16-row step ahead (the first before the accumulators
            // are waited for) and their latency falls into the step before.
            const bool rmw = wide && a.accumulate;
            const int c_end = min(a.TN, rows_valid);
            const int wj = lane >> 2, wc = (lane & 3) * 8;  // token row (of 8) and first column of a wide store
            auto load_old = [&](int c0, float4 (&o)[4]) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int j = wj + 8 * half;
                    if (c0 + j < rows_valid) {
                        const float4* src = reinterpret_cast<const float4*>(
                            outf + static_cast<size_t>(x_row0 + c0 + j) * a.ldo + n_warp + wc);
                        o[2 * half] = src[0];
                        o[2 * half + 1] = src[1];
                    }
                }
            };
            float4 old_a[4], old_b[4];
            if (rmw) load_old(0, old_a);
            if (!mbar_wait(bar_acc_full + 8 * buf, acc_round & 1, 3)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t lane_addr = tmem + buf * acc_cols + (static_cast<uint32_t>(quarter * 32) << 16);
            auto do_cols = [&](int c0, const float4 (&oldw)[4]) {
                uint32_t v[16], u[16];
                tmem_ld16(lane_addr + c0, v);
                if (DUAL) tmem_ld16(lane_addr + a.TN + c0, u);
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
                    if (DUAL) {
                        const float g = x;
                        x = __fdividef(g, 1.0f + __expf(-g)) * __uint_as_float(u[j]);
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
                        const int j = wj + 8 * half;
                        if (c0 + j < rows_valid) {
                            float4 lo = *reinterpret_cast<const float4*>(stage + j * 36 + wc);
                            float4 hi = *reinterpret_cast<const float4*>(stage + j * 36 + wc + 4);
                            const size_t o = static_cast<size_t>(x_row0 + c0 + j) * a.ldo + n_warp + wc;
                            if (a.out_dt == LOCUS_DT_F32) {
                                float4* dst = reinterpret_cast<float4*>(outf + o);
                                if (a.accumulate) {
                                    const float4 p0 = oldw[2 * half], p1 = oldw[2 * half + 1];
                                    lo = make_float4(p0.x + lo.x, p0.y + lo.y, p0.z + lo.z, p0.w + lo.w);
                                    hi = make_float4(p1.x + hi.x, p1.y + hi.y, p1.z + hi.z, p1.w + hi.w);
                                }
                                dst[0] = lo;
                                dst[1] = hi;
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
            };
            for (int c0 = 0; c0 < c_end; c0 += 32) {  // uniform bounds
                if (rmw && c0 + 16 < c_end) load_old(c0 + 16, old_b);
                do_cols(c0, old_a);
                if (c0 + 16 < c_end) {
                    if (rmw && c0 + 32 < c_end) load_old(c0 + 32, old_a);
                    do_cols(c0 + 16, old_b);
                }
            }
            // this warp has read everything it needs from the buffer: hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_acc_empty + 8 * buf) : "memory");
            ++n_done;
            if (++buf == a.acc_bufs) {
                buf = 0;
                ++acc_round;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(a.tmem_cols) : "memory");
    }
}

// Sums the splits of a product that was split along K, in the order of the splits, and does the
// epilogue of the unsplit kernel: + bias, x row scale, then store or add into out.  part: [splits, M, N]
// float32; one thread per 4 columns (N is a multiple of 4).
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, int splits, int M, int N,
                                                            const void* __restrict__ bias, int bias_dt,
                                                            const float* __restrict__ row_scale,
                                                            const int* __restrict__ scale_rows, void* out, int out_dt,
                                                            long long ldo, int accumulate) {
    pdl_entry();
    pdl_trigger();
    const int n4 = N >> 2;
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<long long>(M) * n4) return;
    const int row = static_cast<int>(i / n4), c = static_cast<int>(i - static_cast<long long>(row) * n4) << 2;
    const size_t plane = static_cast<size_t>(M) * N;
    const float* p = part + static_cast<size_t>(row) * N + c;
    float4 acc = *reinterpret_cast<const float4*>(p);
    for (int s = 1; s < splits; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(p + s * plane);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float v[4] = {acc.x, acc.y, acc.z, acc.w};
    const float scale = row_scale ? row_scale[scale_rows ? scale_rows[row] : row] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (bias) v[j] += ld_dyn(bias, bias_dt, c + j);
        if (row_scale) v[j] *= scale;
        const size_t o = static_cast<size_t>(row) * ldo + c + j;
        if (accumulate) static_cast<float*>(out)[o] += v[j];
        else st_dyn(out, out_dt, o, v[j]);
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
// splits > 1 (plain products of one weight matrix, N a multiple of 4): the K range is cut into that many
// parts that run as tiles of their own and leave float32 sums in split_scratch [splits, M, N]; a second
// kernel adds them in order and does the epilogue.  The splits are renumbered so that none is empty.
extern "C" int locus_gemm_tc(const void* x, long long x_rows_total, long long ldx, const void* w, const void* w2,
                             long long w_rows_total, const void* bias, int bias_dt, void* out, int out_dt,
                             int accumulate, const float* row_scale, const int* scale_rows, int M, int N, int K,
                             long long ldo, int TN, const int* tile_expert, const int* tile_row0,
                             const int* tile_rows, const int* n_tiles, int max_tiles, float* split_scratch,
                             int splits, cudaStream_t stream) {
    const int dual = w2 != nullptr ? 1 : 0;
    if (N <= 0 || K <= 0 || K % 8 != 0 || ldx % 8 != 0) return LOCUS_ERR_UNSUPPORTED;
    if (TN < 16 || TN > 256 || TN % 16 != 0 || (dual && TN > 256)) return LOCUS_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(w2)) & 15)
        return LOCUS_ERR_UNSUPPORTED;
    if (accumulate && out_dt != LOCUS_DT_F32) return LOCUS_ERR_UNSUPPORTED;
    if (w_rows_total >= (1LL << 31) || x_rows_total >= (1LL << 31)) return LOCUS_ERR_UNSUPPORTED;
    CUtensorMap map_w, map_w2;
    XMaps maps_x;
    memset(&maps_x, 0, sizeof(maps_x));
    if (!make_map(&map_w, w, w_rows_total, K, K, TILE_W)) return LOCUS_ERR_UNSUPPORTED;
    if (!make_map(&map_w2, dual ? w2 : w, w_rows_total, K, K, TILE_W)) return LOCUS_ERR_UNSUPPORTED;
    {
        // boxes that tiles of this call can ask for: every size up to TN for a grouped product (the rows of
        // a tile are known on the device only), the full tile and the last, ragged one for a plain product
        const int full = x_box_index(TN), last = x_box_index(M % TN == 0 ? TN : M % TN);
        for (int i = 0; i <= full; ++i) {
            if (tile_expert == nullptr && i != full && i != last) continue;
            const int rows = x_box_rows(i) < TN ? x_box_rows(i) : TN;
            if (!make_map(&maps_x.m[i], x, x_rows_total, K, ldx, rows)) return LOCUS_ERR_UNSUPPORTED;
        }
    }
    TcArgs a;
    a.M = M; a.N = N; a.K = K; a.TN = TN; a.dual = dual;
    const int stage_bytes = A_BYTES * (1 + dual) + TN * TILE_K * 2;
    const int tiles_y = tile_expert ? max_tiles : ceil_div(M, TN);
    const int tiles_x = ceil_div(N, TILE_W);
    const long long n_tiles_all = static_cast<long long>(tiles_x) * tiles_y;
    // one block per SM with the whole shared memory as its pipeline
    const int budget = (g_budget_kb > 0 ? g_budget_kb : 200) * 1024;
    int stages = budget / stage_bytes;
    if (stages > 12) stages = 12;
    if (stages < 2) stages = 2;
    const int nkb = (K + TILE_K - 1) / TILE_K;
    if (stages > nkb) stages = nkb;
    if (stages < 1) return LOCUS_ERR_UNSUPPORTED;
    a.stages = stages;
    // two accumulator buffers where the 512 columns of tensor memory hold them
    a.acc_bufs = 2 * TN * (1 + dual) <= 512 ? 2 : 1;
    a.tmem_cols = pow2_at_least(a.acc_bufs * TN * (1 + dual));
    if (a.tmem_cols > 512) return LOCUS_ERR_UNSUPPORTED;
    a.tiles_x = tiles_x; a.tiles_y = tiles_y;
    a.splits = 1;
    a.kb_per_split = nkb;
    if (splits > 1) {
        if (dual || tile_expert != nullptr || split_scratch == nullptr || N % 4 != 0 ||
            (reinterpret_cast<uintptr_t>(split_scratch) & 15))
            return LOCUS_ERR_UNSUPPORTED;
        a.kb_per_split = ceil_div(nkb, splits < nkb ? splits : nkb);
        a.splits = ceil_div(nkb, a.kb_per_split);
        if (n_tiles_all * a.splits >= (1LL << 31)) return LOCUS_ERR_UNSUPPORTED;
    }
    const bool split = a.splits > 1;
    a.accumulate = split ? 0 : accumulate;
    a.out = split ? split_scratch : out;
    a.out_dt = split ? LOCUS_DT_F32 : out_dt;
    a.ldo = split ? N : ldo;
    a.bias = split ? nullptr : bias;
    a.bias_dt = bias_dt;
    a.row_scale = split ? nullptr : row_scale;
    a.scale_rows = split ? nullptr : scale_rows; a.tile_expert = tile_expert; a.tile_row0 = tile_row0;
    a.tile_rows = tile_rows; a.n_tiles = n_tiles;
    const size_t smem = static_cast<size_t>(stages) * stage_bytes + 16 * stages + 96 + 16 * TN + 4 * 16 * 36 * 4 + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
            return static_cast<int>(cudaGetLastError());
        attr_set = true;
    }
    if (tiles_y <= 0) return 0;
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0)
            return static_cast<int>(cudaGetLastError());
    }
    const long long n_units = n_tiles_all * a.splits;
    const unsigned grid = static_cast<unsigned>(n_units < n_sm ? n_units : n_sm);
    if (dual) gemm_tc_kernel<true><<<grid, 192, smem, stream>>>(map_w, map_w2, maps_x, a);
    else gemm_tc_kernel<false><<<grid, 192, smem, stream>>>(map_w, map_w2, maps_x, a);
    if (split) {
        const long long n_threads = static_cast<long long>(M) * (N / 4);
        locus_launch(splitk_reduce_kernel, static_cast<unsigned>((n_threads + 255) / 256), 256, 0, stream,
                     static_cast<const float*>(split_scratch), a.splits, M, N, bias, bias_dt, row_scale, scale_rows,
                     out, out_dt, ldo, accumulate);
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
