// Expert routing: router logits, softmax, top-k selection and weights, the sigmoid gate of
// the shared expert, and the bookkeeping that lays (token, slot) pairs out by expert.
// Router logits, softmax, selection and weights are float32 and are computed by the same
// kernel, in the same order, for every batch shape, so that a token's experts do not
// depend on what else is in the batch.
#include "common.cuh"

// One block per token.
//   h        [T, H]   normed activations (float32 or bfloat16)
//   wr       [E, H]   router weight; wg [H] weight of the shared-expert gate (or null)
//   ids      [T, k]   picked experts in pick order; wts [T, k] their weights
//   gamma    [T]      sigmoid(wg . h) (written only when wg != null)
// Selection: k rounds of arg-max over softmax probabilities with strict '>' (ties go to
// the lowest index).  weight = p / wsum * scale with wsum = sum of picked p when renorm,
// else 1.
template <typename TX, typename TW>
__global__ void __launch_bounds__(256) router_topk_kernel(
    const TX* __restrict__ h, const TW* __restrict__ wr, const void* __restrict__ wg, int wg_dt,
    int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ gamma, int H, int E, int k,
    int renorm, float scale) {
    extern __shared__ float smem[];
    float* hs = smem;           // [H]
    float* logit = smem + H;    // [E]
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const TX* hrow = h + static_cast<size_t>(t) * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) hs[j] = to_f(hrow[j]);
    __syncthreads();
    for (int e = wid; e < E + (wg != nullptr ? 1 : 0); e += nw) {
        float acc = 0.f;
        if (e < E) {
            const TW* w = wr + static_cast<size_t>(e) * H;
            for (int j = lane; j < H; j += 32) acc = fmaf(hs[j], to_f(w[j]), acc);
        } else {
            for (int j = lane; j < H; j += 32) acc = fmaf(hs[j], ld_dyn(wg, wg_dt, j), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            if (e < E) {
                logit[e] = acc;
            } else {
                gamma[t] = 1.0f / (1.0f + expf(-acc));
            }
        }
    }
    __syncthreads();
    if (wid != 0) return;
    // softmax over all E experts
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, logit[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float v = expf(logit[e] - mx);
        logit[e] = v;
        sum += v;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < E; e += 32) logit[e] = logit[e] / sum;
    __syncwarp();
    float wsum = 0.f;
    for (int r = 0; r < k; ++r) {
        float best = -1.f;
        int best_e = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = logit[e];
            if (v > best) {  // taken experts hold -2; ascending e keeps the lowest index on ties
                best = v;
                best_e = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ov > best || (ov == best && oe < best_e)) {
                best = ov;
                best_e = oe;
            }
        }
        if (lane == 0) {
            ids[t * k + r] = best_e;
            wts[t * k + r] = best;
            logit[best_e] = -2.f;
        }
        wsum += best;
        __syncwarp();
    }
    if (lane == 0) {
        const float div = renorm ? wsum : 1.0f;
        for (int r = 0; r < k; ++r) wts[t * k + r] = wts[t * k + r] / div * scale;
    }
}

extern "C" int locus_router_topk(const void* h, int x_dt, const void* wr, int w_dt, const void* wg,
                                 int wg_dt, int* ids, float* wts, float* gamma, int T, int H,
                                 int E, int k, int renorm, float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || k <= 0 || k > E) return LOCUS_ERR_UNSUPPORTED;
    const size_t smem = static_cast<size_t>(H + E) * sizeof(float);
    if (smem > 200 * 1024) return LOCUS_ERR_UNSUPPORTED;
#define ROUTER_LAUNCH(TX, TW)                                                                    \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(router_topk_kernel<TX, TW>,                                     \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        router_topk_kernel<TX, TW><<<T, 256, smem, stream>>>(                                    \
            static_cast<const TX*>(h), static_cast<const TW*>(wr), wg, wg_dt, ids, wts, gamma,   \
            H, E, k, renorm, scale);                                                             \
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
// Bookkeeping.  A "pair" is p = token * k + slot.  Pairs are laid out by expert, pairs of
// one expert in ascending p (a stable order that does not depend on thread timing):
//   counts[e], offsets[e] (offsets[E] = n_pairs), sorted_pair[i] = p, pair_pos[p] = i,
// and a list of row tiles of tile_m rows: tile_expert[], tile_row0[], tile_rows[], *n_tiles.
__global__ void moe_count_kernel(const int* __restrict__ ids, int n_pairs, int* __restrict__ counts) {
    __shared__ int warp_part[32];
    const int e = blockIdx.x;
    int c = 0;
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) c += (ids[p] == e);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int tot = 0;
        for (int w = 0; w < (blockDim.x >> 5); ++w) tot += warp_part[w];
        counts[e] = tot;
    }
}

__global__ void moe_fill_kernel(const int* __restrict__ ids, int n_pairs, int E,
                                const int* __restrict__ counts, int tile_m,
                                int* __restrict__ offsets, int* __restrict__ sorted_pair,
                                int* __restrict__ pair_pos, int* __restrict__ tile_expert,
                                int* __restrict__ tile_row0, int* __restrict__ tile_rows,
                                int* __restrict__ n_tiles) {
    __shared__ int s_off, s_tile, s_base;
    __shared__ int warp_cnt[32];
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (threadIdx.x == 0) {
        int off = 0, tile = 0;
        for (int j = 0; j < e; ++j) {
            off += counts[j];
            tile += (counts[j] + tile_m - 1) / tile_m;
        }
        s_off = off;
        s_tile = tile;
        offsets[e] = off;
        const int mine = counts[e];
        const int nt = (mine + tile_m - 1) / tile_m;
        for (int i = 0; i < nt; ++i) {
            tile_expert[tile + i] = e;
            tile_row0[tile + i] = off + i * tile_m;
            tile_rows[tile + i] = min(tile_m, mine - i * tile_m);
        }
        if (e == E - 1) {
            offsets[E] = off + mine;
            *n_tiles = tile + nt;
        }
        s_base = 0;
    }
    __syncthreads();
    const int off = s_off;
    for (int p0 = 0; p0 < n_pairs; p0 += blockDim.x) {
        const int p = p0 + threadIdx.x;
        const bool hit = p < n_pairs && ids[p] == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) warp_cnt[wid] = __popc(ballot);
        __syncthreads();
        int before = s_base;
        for (int w = 0; w < wid; ++w) before += warp_cnt[w];
        if (hit) {
            const int pos = off + before + __popc(ballot & ((1u << lane) - 1u));
            sorted_pair[pos] = p;
            pair_pos[p] = pos;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int w = 0; w < nw; ++w) tot += warp_cnt[w];
            s_base += tot;
        }
        __syncthreads();
    }
}

extern "C" int locus_moe_sort(const int* ids, int n_pairs, int E, int tile_m, int* counts,
                              int* offsets, int* sorted_pair, int* pair_pos, int* tile_expert,
                              int* tile_row0, int* tile_rows, int* n_tiles, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (E <= 0 || tile_m <= 0) return LOCUS_ERR_UNSUPPORTED;
    moe_count_kernel<<<E, 256, 0, stream>>>(ids, n_pairs, counts);
    moe_fill_kernel<<<E, 256, 0, stream>>>(ids, n_pairs, E, counts, tile_m, offsets, sorted_pair,
                                           pair_pos, tile_expert, tile_row0, tile_rows, n_tiles);
    return locus_launch_status();
}
