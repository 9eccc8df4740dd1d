// Expert routing: router logits, softmax, top-k selection and weights, the sigmoid gate of
// the shared expert, and the bookkeeping that lays (token, slot) pairs out by expert.
// Router logits, softmax, selection and weights are float32 and are computed by the same
// kernel, in the same order, for every batch shape, so that a token's experts do not
// depend on what else is in the batch.
#include "common.cuh"
#include "route_select.cuh"

#define RT_TOK 8    // tokens per block
#define RT_WARPS 8  // experts per block, one per warp

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* o);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* o) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<bf16>(const bf16* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        o[2 * i] = f.x;
        o[2 * i + 1] = f.y;
    }
}

// Grid (token tiles of RT_TOK, expert groups of RT_WARPS).  A block stages its tokens'
// activations in shared memory; each warp computes the router logit of one expert (the shared
// gate counts as expert E) for all tokens of the tile, every weight read once per tile, and
// writes it to `logits` [T, E (+1)].  The block that finishes a tile last (a counter per tile,
// reset for the next launch) runs softmax, selection and weights for the tile, one warp per token.
//   h        [T, H]   normed activations (float32 or bfloat16)
//   wr       [E, H]   router weight; wg [H] weight of the shared-expert gate (or null)
//   ids      [T, k]   picked experts in pick order; wts [T, k] their weights
//   gamma    [T]      sigmoid(wg . h) (written only when wg != null)
// Selection and weights: select_token above.
// The order in which a logit is summed depends on H only (8-element chunks per lane when H
// is a multiple of 8, single elements else), not on the tile or its other tokens.
template <typename TX, typename TW>
__global__ void __launch_bounds__(256) router_topk_kernel(
    const TX* __restrict__ h, const TW* __restrict__ wr, const void* __restrict__ wg, int wg_dt,
    float* __restrict__ logits, int* __restrict__ counters, int* __restrict__ ids,
    float* __restrict__ wts, float* __restrict__ gamma, int T, int H, int E, const RouteOpts o) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    TX* hs = reinterpret_cast<TX*>(smem_raw);                                        // [RT_TOK][H]
    float* probs = reinterpret_cast<float*>(smem_raw + sizeof(TX) * RT_TOK * H);     // [RT_TOK][2 E]
    __shared__ int is_last;
    const int E1 = E + (wg != nullptr ? 1 : 0);
    const int tile = blockIdx.x, grp = blockIdx.y;
    const int t0 = tile * RT_TOK, nt = min(RT_TOK, T - t0);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const TX* hsrc = h + static_cast<size_t>(t0) * H;
    for (int i = threadIdx.x; i < nt * H; i += blockDim.x) hs[i] = hsrc[i];
    __syncthreads();
    const int e = grp * RT_WARPS + wid;
    if (e < E1) {
        float acc[RT_TOK];
#pragma unroll
        for (int t = 0; t < RT_TOK; ++t) acc[t] = 0.f;
        const bool gate = e >= E;
        const bool vec = (H % 8 == 0) && (!gate || wg_dt == (sizeof(TW) == 4 ? LOCUS_DT_F32 : LOCUS_DT_BF16));
        if (vec) {
            const TW* w = gate ? static_cast<const TW*>(wg) : wr + static_cast<size_t>(e) * H;
            for (int j = lane * 8; j < H; j += 256) {
                float wv[8];
                load8<TW>(w + j, wv);
#pragma unroll
                for (int t = 0; t < RT_TOK; ++t) {
                    if (t < nt) {
                        float hv[8];
                        load8<TX>(hs + t * H + j, hv);
#pragma unroll
                        for (int u = 0; u < 8; ++u) acc[t] = fmaf(hv[u], wv[u], acc[t]);
                    }
                }
            }
        } else {
            for (int j = lane; j < H; j += 32) {
                const float wv = gate ? ld_dyn(wg, wg_dt, j) : to_f(wr[static_cast<size_t>(e) * H + j]);
#pragma unroll
                for (int t = 0; t < RT_TOK; ++t)
                    if (t < nt) acc[t] = fmaf(to_f(hs[t * H + j]), wv, acc[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < RT_TOK; ++t) {
            if (t < nt) {
                const float s = warp_sum(acc[t]);
                if (lane == 0) logits[static_cast<size_t>(t0 + t) * E1 + e] = s;
            }
        }
    }
    // the last block of the tile to get here selects
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(&counters[tile], 1) == static_cast<int>(gridDim.y) - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x == 0) counters[tile] = 0;
    if (wid >= nt) return;
    const int t = t0 + wid;
    select_token(logits + static_cast<size_t>(t) * E1, probs + wid * 2 * E, t, lane, ids, wts, gamma, nullptr, E,
                 wg != nullptr ? 1 : 0, o);
}

// logits: scratch [T, E (+1 with a gate)] floats; counters: ceil(T / 8) ints, zero before the
// first launch (every launch leaves them zero again).
extern "C" int locus_router_topk(const void* h, int x_dt, const void* wr, int w_dt, const void* wg,
                                 int wg_dt, float* logits, int* counters, int* ids, float* wts,
                                 float* gamma, int T, int H, int E, int k, int renorm, float scale,
                                 int score_fn, const float* sel_bias, int n_group, int n_group_used,
                                 cudaStream_t stream) {
    if (T <= 0) return 0;
    const RouteOpts o{k, renorm, score_fn, n_group, n_group_used, scale, sel_bias};
    if (!route_opts_ok(o, E)) return LOCUS_ERR_UNSUPPORTED;
    const int E1 = E + (wg != nullptr ? 1 : 0);
    const size_t xsize = x_dt == LOCUS_DT_F32 ? 4 : 2;
    const size_t smem = xsize * RT_TOK * H + sizeof(float) * RT_TOK * 2 * E;
    if (smem > 200 * 1024) return LOCUS_ERR_UNSUPPORTED;
    dim3 grid(ceil_div(T, RT_TOK), ceil_div(E1, RT_WARPS));
    if (grid.y > 65535) return LOCUS_ERR_UNSUPPORTED;
#define ROUTER_LAUNCH(TX, TW)                                                                    \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(router_topk_kernel<TX, TW>,                                     \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        router_topk_kernel<TX, TW><<<grid, 256, smem, stream>>>(                                 \
            static_cast<const TX*>(h), static_cast<const TW*>(wr), wg, wg_dt, logits, counters,  \
            ids, wts, gamma, T, H, E, o);                                                        \
    } while (0)
    if (x_dt == LOCUS_DT_F32 && w_dt == LOCUS_DT_F32) ROUTER_LAUNCH(float, float);
    else if (x_dt == LOCUS_DT_BF16 && w_dt == LOCUS_DT_BF16) ROUTER_LAUNCH(bf16, bf16);
    else if (x_dt == LOCUS_DT_BF16 && w_dt == LOCUS_DT_F32) ROUTER_LAUNCH(bf16, float);
    else if (x_dt == LOCUS_DT_F32 && w_dt == LOCUS_DT_BF16) ROUTER_LAUNCH(float, bf16);
    else return LOCUS_ERR_UNSUPPORTED;
#undef ROUTER_LAUNCH
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Selection alone, from router logits that another kernel produced (the bfloat16 path computes
// them on the tensor cores): one warp per token.  logits [T, E (+1)] float32; column E, when
// has_gate, is the logit of the shared-expert gate.  Same scores, selection and weights as above.
__global__ void __launch_bounds__(256) router_select_kernel(const float* __restrict__ logits, int ld,
                                                            int* __restrict__ ids, float* __restrict__ wts,
                                                            float* __restrict__ gamma, int T, int E,
                                                            int has_gate, const RouteOpts o) {
    pdl_entry();
    extern __shared__ float probs_all[];  // [warps][2 E]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + wid;
    if (t >= T) return;
    select_token(logits + static_cast<size_t>(t) * ld, probs_all + wid * 2 * E, t, lane, ids, wts, gamma, nullptr, E,
                 has_gate, o);
}

extern "C" int locus_router_select(const float* logits, int ld, int* ids, float* wts, float* gamma, int T, int E,
                                   int k, int has_gate, int renorm, float scale, int score_fn,
                                   const float* sel_bias, int n_group, int n_group_used, cudaStream_t stream) {
    if (T <= 0) return 0;
    const RouteOpts o{k, renorm, score_fn, n_group, n_group_used, scale, sel_bias};
    if (!route_opts_ok(o, E) || ld < E + (has_gate ? 1 : 0)) return LOCUS_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * 8 * 2 * E;
    if (smem > 200 * 1024) return LOCUS_ERR_UNSUPPORTED;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(router_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    locus_launch(router_select_kernel, ceil_div(T, 8), 256, smem, stream, logits, ld, ids, wts, gamma, T, E, has_gate, o);
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Bookkeeping.  A "pair" is p = token * k + slot.  Pairs are laid out by expert, pairs of
// one expert in ascending p (a stable order that does not depend on thread timing):
//   counts[e], offsets[e] (offsets[E] = n_pairs), sorted_pair[i] = p, pair_pos[p] = i,
// and a list of row tiles of tile_m rows: tile_expert[], tile_row0[], tile_rows[], *n_tiles.
__global__ void __launch_bounds__(256) moe_count_kernel(const int* __restrict__ ids, int n_pairs,
                                                         int* __restrict__ counts) {
    pdl_entry();
    __shared__ int warp_part[8];
    const int e = blockIdx.x;
    int c = 0;
    const int n4 = n_pairs >> 2;
    const int4* ids4 = reinterpret_cast<const int4*>(ids);
    for (int p = threadIdx.x; p < n4; p += blockDim.x) {
        const int4 v = ids4[p];
        c += (v.x == e) + (v.y == e) + (v.z == e) + (v.w == e);
    }
    for (int p = (n4 << 2) + threadIdx.x; p < n_pairs; p += blockDim.x) c += (ids[p] == e);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int tot = 0;
        for (int w = 0; w < 8; ++w) tot += warp_part[w];
        counts[e] = tot;
    }
}

// One block per expert.  Each of the 8 warps takes a contiguous eighth of the pairs.  With COUNT the block first
// counts every expert's pairs itself, per warp, in shared memory (E blocks each read the ids once from L2: cheaper
// than a launch of its own for the counts, which every block needs for its offset) and writes its own expert's
// count; without, the counts come from moe_count_kernel.  The block adds the warps' counts in order, then every
// warp ranks its own matches with ballots -- no block-wide barrier inside the loops.  Positions are ascending
// in p (stable).
template <bool COUNT>
__global__ void __launch_bounds__(256) moe_fill_kernel(const int* __restrict__ ids, int n_pairs, int E,
                                                        int* __restrict__ counts, int tile_m,
                                                        int* __restrict__ offsets, int* __restrict__ sorted_pair,
                                                        int* __restrict__ pair_pos, int* __restrict__ tile_expert,
                                                        int* __restrict__ tile_row0, int* __restrict__ tile_rows,
                                                        int* __restrict__ n_tiles, int tile2_m,
                                                        int* __restrict__ tile2_expert, int* __restrict__ tile2_row0,
                                                        int* __restrict__ tile2_rows, int* __restrict__ n_tiles2) {
    pdl_entry();
    extern __shared__ int hist[];  // COUNT: [8 warps][E] pairs of a warp's eighth per expert, then [E] totals
    __shared__ int s_off;
    __shared__ int warp_cnt[8];
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int per = ((n_pairs + 7) / 8 + 31) & ~31;  // pairs per warp, a multiple of 32
    const int p_begin = wid * per, p_end = min(n_pairs, p_begin + per);
    const int* cnt = counts;
    if (COUNT) {
        for (int i = threadIdx.x; i < 8 * E; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        for (int p = p_begin + lane; p < p_end; p += 32) {
            const int id = ids[p];
            if (id >= 0 && id < E) atomicAdd(&hist[wid * E + id], 1);
        }
        __syncthreads();
        int* tot = hist + 8 * E;
        for (int j = threadIdx.x; j < E; j += blockDim.x) {
            int c = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) c += hist[w * E + j];
            tot[j] = c;
        }
        __syncthreads();
        cnt = tot;
        if (threadIdx.x == 0) counts[e] = tot[e];
    }
    if (wid == 0) {
        // rows and tiles of the experts before this one
        int off = 0, tile = 0, tile2 = 0;
        for (int j = lane; j < e; j += 32) {
            const int c = cnt[j];
            off += c;
            tile += (c + tile_m - 1) / tile_m;
            if (tile2_m > 0) tile2 += (c + tile2_m - 1) / tile2_m;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            off += __shfl_xor_sync(0xffffffffu, off, o);
            tile += __shfl_xor_sync(0xffffffffu, tile, o);
            tile2 += __shfl_xor_sync(0xffffffffu, tile2, o);
        }
        if (lane == 0) {
            s_off = off;
            offsets[e] = off;
            const int mine = cnt[e];
            const int nt = (mine + tile_m - 1) / tile_m;
            for (int i = 0; i < nt; ++i) {
                tile_expert[tile + i] = e;
                tile_row0[tile + i] = off + i * tile_m;
                tile_rows[tile + i] = min(tile_m, mine - i * tile_m);
            }
            if (tile2_m > 0) {  // the same rows in tiles of another size (for a product with another token tile)
                const int nt2 = (mine + tile2_m - 1) / tile2_m;
                for (int i = 0; i < nt2; ++i) {
                    tile2_expert[tile2 + i] = e;
                    tile2_row0[tile2 + i] = off + i * tile2_m;
                    tile2_rows[tile2 + i] = min(tile2_m, mine - i * tile2_m);
                }
                if (e == E - 1) *n_tiles2 = tile2 + nt2;
            }
            if (e == E - 1) {
                offsets[E] = off + mine;
                *n_tiles = tile + nt;
            }
        }
    }
    if (COUNT) {
        if (lane == 0) warp_cnt[wid] = hist[wid * E + e];
    } else {
        int c = 0;
        for (int p = p_begin + lane; p < p_end; p += 32) c += (ids[p] == e);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        if (lane == 0) warp_cnt[wid] = c;
    }
    __syncthreads();
    int pos = s_off;
    for (int w = 0; w < wid; ++w) pos += warp_cnt[w];
    for (int p0 = p_begin; p0 < p_end; p0 += 32) {
        const int p = p0 + lane;
        const bool hit = p < p_end && ids[p] == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (hit) {
            const int at = pos + __popc(ballot & ((1u << lane) - 1u));
            sorted_pair[at] = p;
            pair_pos[p] = at;
        }
        pos += __popc(ballot);
    }
}

// tile2_m > 0: a second tile list over the same layout, with tiles of tile2_m rows (tile2_* and n_tiles2).
extern "C" int locus_moe_sort(const int* ids, int n_pairs, int E, int tile_m, int* counts,
                              int* offsets, int* sorted_pair, int* pair_pos, int* tile_expert,
                              int* tile_row0, int* tile_rows, int* n_tiles, int tile2_m, int* tile2_expert,
                              int* tile2_row0, int* tile2_rows, int* n_tiles2, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (E <= 0 || tile_m <= 0 || tile2_m < 0) return LOCUS_ERR_UNSUPPORTED;
    if (tile2_m > 0 && (tile2_expert == nullptr || tile2_row0 == nullptr || tile2_rows == nullptr || n_tiles2 == nullptr))
        return LOCUS_ERR_UNSUPPORTED;
    const size_t hist = sizeof(int) * 9 * static_cast<size_t>(E);
    if (hist <= 40 * 1024) {  // one launch: every block counts for itself
        locus_launch(moe_fill_kernel<true>, E, 256, hist, stream, ids, n_pairs, E, counts, tile_m, offsets, sorted_pair,
                     pair_pos, tile_expert, tile_row0, tile_rows, n_tiles, tile2_m, tile2_expert, tile2_row0, tile2_rows,
                     n_tiles2);
    } else {
        locus_launch(moe_count_kernel, E, 256, 0, stream, ids, n_pairs, counts);
        locus_launch(moe_fill_kernel<false>, E, 256, 0, stream, ids, n_pairs, E, counts, tile_m, offsets, sorted_pair,
                     pair_pos, tile_expert, tile_row0, tile_rows, n_tiles, tile2_m, tile2_expert, tile2_row0, tile2_rows,
                     n_tiles2);
    }
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Selection and bookkeeping of a decode-sized batch in one launch: one block selects the experts of
// every token (a warp per token, the arithmetic of router_select_kernel) and then lays the pairs out
// by expert (the result of moe_count_kernel and moe_fill_kernel), all through shared memory.
// Limits: n_pairs = T * k <= RS_MAX_PAIRS, E <= RS_MAX_E.
#define RS_WARPS 16   // a warp per token for up to 16 tokens
__global__ void __launch_bounds__(32 * RS_WARPS) route_small_kernel(const float* __restrict__ logits, int ld,
                                                          int* __restrict__ ids, float* __restrict__ wts,
                                                          float* __restrict__ gamma, int T, int E, int has_gate,
                                                          const RouteOpts o, const RouteLayoutOut lo) {
    pdl_entry();
    pdl_trigger();
    extern __shared__ float rs_smem[];
    route_small_block(rs_smem, logits, ld, ids, wts, gamma, T, E, has_gate, o, lo);
}

extern "C" int locus_route_small(const float* logits, int ld, int* ids, float* wts, float* gamma, int T, int E,
                                 int k, int has_gate, int renorm, float scale, int score_fn, const float* sel_bias,
                                 int n_group, int n_group_used, int tile_m, int* counts,
                                 int* offsets, int* sorted_pair, int* pair_pos, int* tile_expert, int* tile_row0,
                                 int* tile_rows, int* n_tiles, cudaStream_t stream) {
    if (T <= 0) return 0;
    const RouteOpts o{k, renorm, score_fn, n_group, n_group_used, scale, sel_bias};
    if (!route_opts_ok(o, E) || ld < E + (has_gate ? 1 : 0) || tile_m <= 0) return LOCUS_ERR_UNSUPPORTED;
    if (E > RS_MAX_E || static_cast<long long>(T) * k > RS_MAX_PAIRS) return LOCUS_ERR_UNSUPPORTED;
    const size_t smem = route_small_smem(RS_WARPS, T, E, k);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(route_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const RouteLayoutOut lo{tile_m, counts, offsets, sorted_pair, pair_pos, tile_expert, tile_row0, tile_rows, n_tiles};
    locus_launch(route_small_kernel, 1, 32 * RS_WARPS, smem, stream, logits, ld, ids, wts, gamma, T, E, has_gate, o, lo);
    return locus_launch_status();
}
