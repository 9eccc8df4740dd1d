// Expert selection and the expert layout of a decode-sized batch as device functions, shared by the routing
// kernels (moe_route.cu) and by the weight-streaming product that ends in them (gemm_skinny.cu: router logits,
// selection and layout in one launch).
#pragma once

// How a token's experts are chosen from its router logits, as the reference's moe_select does it
// (src/locus/model/llama.cpp:900-980): scores = softmax over all experts, or a sigmoid of each logit;
// selection scores = scores (+ sel_bias, which never enters the weights); with n_group > 1 only the
// n_group_used groups with the largest sum of their two best selection scores stay eligible (the others are
// masked to -1e30); k rounds of arg-max with strict '>' (ties to the lowest index); weight = score / wsum *
// scale, wsum = sum of the picked scores when renorm, else 1.
#define SCORE_SOFTMAX 0
#define SCORE_SIGMOID 1
struct RouteOpts {
    int k, renorm, score_fn, n_group, n_group_used;
    float scale;
    const float* sel_bias;  // [E] float32 or null
};

__host__ inline bool route_opts_ok(const RouteOpts& o, int E) {
    if (E <= 0 || o.k <= 0 || o.k > E) return false;
    if (o.score_fn != SCORE_SOFTMAX && o.score_fn != SCORE_SIGMOID) return false;
    if (o.n_group < 1 || o.n_group > 32 || E % o.n_group != 0) return false;
    if (o.n_group > 1 && (o.n_group_used < 1 || o.n_group_used > o.n_group)) return false;
    return true;
}

// Scores, selection and weights of one token by one warp.  lg: the token's logits (column E, when
// has_gate, is the logit of the shared-expert gate); p: 2 * E floats of shared memory of this warp;
// s_ids (or null): where the picks are also kept for the block.  The selection is total: a score that is
// not a number counts as the lowest, so every pick is an expert index below E whatever the logits hold.
__device__ __forceinline__ void select_token(const float* __restrict__ lg, float* p, int t, int lane,
                                             int* __restrict__ ids, float* __restrict__ wts,
                                             float* __restrict__ gamma, int* s_ids, int E, int has_gate,
                                             const RouteOpts o) {
    float* sel = p + E;
    const int k = o.k;
    if (o.score_fn == SCORE_SOFTMAX) {
        float mx = -INFINITY;
        for (int x = lane; x < E; x += 32) {
            const float v = __ldcg(lg + x);
            p[x] = v;
            mx = fmaxf(mx, v);
        }
        mx = warp_max(mx);
        float sum = 0.f;
        for (int x = lane; x < E; x += 32) {
            const float v = expf(p[x] - mx);
            p[x] = v;
            sum += v;
        }
        sum = warp_sum(sum);
        for (int x = lane; x < E; x += 32) p[x] = p[x] / sum;
    } else {
        for (int x = lane; x < E; x += 32) p[x] = 1.0f / (1.0f + expf(-__ldcg(lg + x)));
    }
    if (has_gate && lane == 0) gamma[t] = 1.0f / (1.0f + expf(-__ldcg(lg + E)));
    for (int x = lane; x < E; x += 32) {
        const float v = p[x] + (o.sel_bias != nullptr ? o.sel_bias[x] : 0.f);
        sel[x] = (v == v) ? v : -3.0e38f;
    }
    __syncwarp();
    if (o.n_group > 1) {
        const int per = E / o.n_group;
        const bool has_group = lane < o.n_group;
        float gs = -INFINITY;
        if (has_group) {
            float top1 = -1e30f, top2 = -1e30f;
            for (int e = lane * per; e < (lane + 1) * per; ++e) {
                const float v = sel[e];
                if (v > top1) {
                    top2 = top1;
                    top1 = v;
                } else if (v > top2) {
                    top2 = v;
                }
            }
            gs = top1 + (per > 1 ? top2 : 0.0f);
        }
        unsigned keep = 0;
        for (int r = 0; r < o.n_group_used; ++r) {
            const bool open = has_group && !((keep >> lane) & 1u);
            float best = open ? gs : -INFINITY;
            int bi = open ? lane : 0x7fffffff;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, d);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
                if (ov > best || (ov == best && oi < bi)) {
                    best = ov;
                    bi = oi;
                }
            }
            if (bi < 32) keep |= 1u << bi;
        }
        __syncwarp();
        for (int x = lane; x < E; x += 32)
            if (!((keep >> (x / per)) & 1u)) sel[x] = -1e30f;
        __syncwarp();
    }
    float wsum = 0.f;
    // After the butterfly every lane knows the pick; lane r keeps the score of pick r, so that the
    // weights go out with one store per lane at the end (up to 32 picks; beyond that they take the way
    // through global memory).
    const bool in_lanes = k <= 32;
    float my_w = 0.f;
    for (int r = 0; r < k; ++r) {
        float best = -INFINITY;  // taken experts hold -inf, everything else is above it
        int best_e = 0x7fffffff;
        for (int x = lane; x < E; x += 32) {
            const float v = sel[x];
            if (v > best) {  // ascending x keeps the lowest index on ties
                best = v;
                best_e = x;
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, d);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, d);
            if (ov > best || (ov == best && oe < best_e)) {
                best = ov;
                best_e = oe;
            }
        }
        if (best_e >= E) best_e = 0;  // cannot happen while k <= E; keeps every index in range regardless
        const float w = p[best_e];
        if (lane == r) my_w = w;
        if (lane == 0) {
            ids[t * k + r] = best_e;
            if (s_ids != nullptr) s_ids[t * k + r] = best_e;
            if (!in_lanes) wts[t * k + r] = w;
            sel[best_e] = -INFINITY;
        }
        wsum += w;
        __syncwarp();
    }
    const float div = o.renorm ? wsum : 1.0f;
    if (in_lanes) {
        if (lane < k) wts[t * k + lane] = my_w / div * o.scale;
    } else if (lane == 0) {
        for (int r = 0; r < k; ++r) wts[t * k + r] = wts[t * k + r] / div * o.scale;
    }
}

// Selection and bookkeeping of a decode-sized batch by ONE block: every token's experts are selected (a warp per
// token in turn) and the pairs are laid out by expert (the result of moe_count_kernel and moe_fill_kernel), all
// through shared memory.  smem: route_small_smem(...) bytes.  Limits: n_pairs = T * k <= RS_MAX_PAIRS, E <= RS_MAX_E.
#define RS_MAX_PAIRS 1024
#define RS_MAX_E 512

struct RouteLayoutOut {
    int tile_m;
    int* counts;
    int* offsets;
    int* sorted_pair;
    int* pair_pos;
    int* tile_expert;
    int* tile_row0;
    int* tile_rows;
    int* n_tiles;
};

__host__ __device__ inline size_t route_small_smem(int n_warps, int T, int E, int k) {
    return sizeof(float) * n_warps * 2 * E + sizeof(int) * (static_cast<size_t>(T) * k + 3 * E + 2);
}

__device__ __forceinline__ void route_small_block(float* rs_smem, const float* __restrict__ logits, int ld,
                                                  int* __restrict__ ids, float* __restrict__ wts,
                                                  float* __restrict__ gamma, int T, int E, int has_gate,
                                                  const RouteOpts o, const RouteLayoutOut lo) {
    const int n_warps = blockDim.x >> 5;
    const int k = o.k, tile_m = lo.tile_m;
    int* s_ids = reinterpret_cast<int*>(rs_smem + n_warps * 2 * E);  // [T * k]
    int* s_cnt = s_ids + T * k;                             // [E]
    int* s_off = s_cnt + E;                                 // [E + 1]
    int* s_tile = s_off + E + 1;                            // [E + 1]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int n_pairs = T * k;
    for (int t = wid; t < T; t += n_warps)
        select_token(logits + static_cast<size_t>(t) * ld, rs_smem + wid * 2 * E, t, lane, ids, wts, gamma, s_ids, E,
                     has_gate, o);
    __syncthreads();
    if (n_pairs <= 32 && E <= 64) {
        // A handful of pairs (a decode step of up to 8 requests): one warp lays them out with votes instead of loops
        // and block barriers.  Lane p holds pair p; the lanes of an expert find each other, the first of them counts.
        if (wid != 0) return;
        const int id = lane < n_pairs ? s_ids[lane] : -1 - lane;  // lanes without a pair match nobody
        const unsigned peers = __match_any_sync(0xffffffffu, id);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        for (int e = lane; e < E; e += 32) s_cnt[e] = 0;
        __syncwarp();
        if (lane < n_pairs && rank == 0) s_cnt[id] = __popc(peers);
        __syncwarp();
        // exclusive prefix sums of rows and tiles over the experts, two experts a lane
        const int e0 = 2 * lane, e1 = 2 * lane + 1;
        const int c0 = e0 < E ? s_cnt[e0] : 0, c1 = e1 < E ? s_cnt[e1] : 0;
        const int t0 = (c0 + tile_m - 1) / tile_m, t1 = (c1 + tile_m - 1) / tile_m;
        int rows_incl = c0 + c1, tiles_incl = t0 + t1;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int rr = __shfl_up_sync(0xffffffffu, rows_incl, d);
            const int tt = __shfl_up_sync(0xffffffffu, tiles_incl, d);
            if (lane >= d) {
                rows_incl += rr;
                tiles_incl += tt;
            }
        }
        const int rows_before = rows_incl - c0 - c1, tiles_before = tiles_incl - t0 - t1;
        if (e0 < E) {
            s_off[e0] = rows_before;
            lo.counts[e0] = c0;
            lo.offsets[e0] = rows_before;
            for (int i = 0; i < t0; ++i) {
                lo.tile_expert[tiles_before + i] = e0;
                lo.tile_row0[tiles_before + i] = rows_before + i * tile_m;
                lo.tile_rows[tiles_before + i] = min(tile_m, c0 - i * tile_m);
            }
        }
        if (e1 < E) {
            s_off[e1] = rows_before + c0;
            lo.counts[e1] = c1;
            lo.offsets[e1] = rows_before + c0;
            for (int i = 0; i < t1; ++i) {
                lo.tile_expert[tiles_before + t0 + i] = e1;
                lo.tile_row0[tiles_before + t0 + i] = rows_before + c0 + i * tile_m;
                lo.tile_rows[tiles_before + t0 + i] = min(tile_m, c1 - i * tile_m);
            }
        }
        if (lane == 31) {
            lo.offsets[E] = rows_incl;
            *lo.n_tiles = tiles_incl;
        }
        __syncwarp();
        if (lane < n_pairs) {
            const int at = s_off[id] + rank;   // pairs of an expert in ascending pair order
            lo.sorted_pair[at] = lane;
            lo.pair_pos[lane] = at;
        }
        return;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int c = 0;
        for (int p = 0; p < n_pairs; ++p) c += (s_ids[p] == e);
        s_cnt[e] = c;
        lo.counts[e] = c;
    }
    __syncthreads();
    if (wid == 0) {
        // exclusive prefix sums of rows and of tiles over the experts: a contiguous run of experts per lane
        const int per = (E + 31) / 32;
        const int e0 = min(E, lane * per), e1 = min(E, e0 + per);
        int rows = 0, tiles = 0;
        for (int e = e0; e < e1; ++e) {
            rows += s_cnt[e];
            tiles += (s_cnt[e] + tile_m - 1) / tile_m;
        }
        int rows_before = rows, tiles_before = tiles;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int r = __shfl_up_sync(0xffffffffu, rows_before, d);
            const int tl = __shfl_up_sync(0xffffffffu, tiles_before, d);
            if (lane >= d) {
                rows_before += r;
                tiles_before += tl;
            }
        }
        rows_before -= rows;
        tiles_before -= tiles;
        for (int e = e0; e < e1; ++e) {
            s_off[e] = rows_before;
            s_tile[e] = tiles_before;
            rows_before += s_cnt[e];
            tiles_before += (s_cnt[e] + tile_m - 1) / tile_m;
        }
        if (e1 == E && e0 < E) {
            s_off[E] = rows_before;
            s_tile[E] = tiles_before;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int off = s_off[e], mine = s_cnt[e], tile = s_tile[e];
        lo.offsets[e] = off;
        if (e == E - 1) {
            lo.offsets[E] = s_off[E];
            *lo.n_tiles = s_tile[E];
        }
        const int nt = (mine + tile_m - 1) / tile_m;
        for (int i = 0; i < nt; ++i) {
            lo.tile_expert[tile + i] = e;
            lo.tile_row0[tile + i] = off + i * tile_m;
            lo.tile_rows[tile + i] = min(tile_m, mine - i * tile_m);
        }
        int at = off;
        for (int p = 0; p < n_pairs && at < off + mine; ++p) {
            if (s_ids[p] == e) {
                lo.sorted_pair[at] = p;
                lo.pair_pos[p] = at;
                ++at;
            }
        }
    }
}
