// Sampling from float32 logits, one block per row: penalties, greedy arg-max, and
// temperature sampling with top-k, top-p and min-p filters.  The order of the filters is
// penalties -> top-k -> temperature softmax -> top-p -> min-p -> draw.
//
// All sums that decide which tokens are kept, and the draw itself, are made on 64-bit
// fixed-point integers (weight = exp((logit - max) / T) in (0, 1], scaled by 2^40), so a
// row's result does not depend on thread timing or on the other rows of the batch.  The
// random number is a counter-based hash of (seed, draw index); the token is found by
// walking the kept weights in ascending token order until the running sum passes u * total.
#include "common.cuh"

#define SAMPLE_THREADS 1024
typedef unsigned long long u64;

__device__ __forceinline__ unsigned order_key(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // ascending float -> ascending uint
}

__device__ __forceinline__ u64 mix64(u64 z) {
    z += 0x9e3779b97f4a7c15ULL;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    return z ^ (z >> 31);
}

__device__ __forceinline__ u64 fixed_weight(float logit, float mx, float inv_t) {
    // exp in float32, at most 1.0; 2^40 fixed point (a weight below 2^-40 counts as 0)
    const float w = expf((logit - mx) * inv_t);
    return static_cast<u64>(static_cast<double>(w) * 1099511627776.0);
}

// Penalties on the tokens of the history window (src/locus/model/sampling.cpp:16-43 of the
// reference): a repeated token's logit is divided (if positive) or multiplied (if negative)
// by repeat_penalty, then frequency * count + presence is subtracted.  history [R, n_hist],
// entries < 0 are padding.  Each distinct token is handled by the thread of its first
// occurrence.
__global__ void penalties_kernel(float* __restrict__ logits, long long row_stride, int V,
                                 const int* __restrict__ history, int n_hist,
                                 const float* __restrict__ repeat, const float* __restrict__ freq,
                                 const float* __restrict__ presence) {
    const int r = blockIdx.x;
    const float rp = repeat[r], fp = freq[r], pp = presence[r];
    if (rp == 1.0f && fp == 0.0f && pp == 0.0f) return;
    const int* hist = history + static_cast<size_t>(r) * n_hist;
    float* row = logits + r * row_stride;
    for (int i = threadIdx.x; i < n_hist; i += blockDim.x) {
        const int tok = hist[i];
        if (tok < 0 || tok >= V) continue;
        bool first = true;
        int c = 0;
        for (int j = 0; j < n_hist; ++j) {
            if (hist[j] == tok) {
                if (j < i) first = false;
                ++c;
            }
        }
        if (!first) continue;
        float l = row[tok];
        if (rp != 1.0f) l = l > 0.0f ? l / rp : l * rp;
        l -= fp * static_cast<float>(c) + pp;
        row[tok] = l;
    }
}

extern "C" int locus_apply_penalties(float* logits, long long row_stride, int R, int V,
                                     const int* history, int n_hist, const float* repeat,
                                     const float* freq, const float* presence,
                                     cudaStream_t stream) {
    if (R <= 0 || n_hist <= 0) return 0;
    penalties_kernel<<<R, 256, 0, stream>>>(logits, row_stride, V, history, n_hist, repeat, freq,
                                            presence);
    return locus_launch_status();
}

// Block-wide helpers (SAMPLE_THREADS threads) --------------------------------
__device__ u64 block_sum_u64(u64 v, u64* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    u64 tot = 0;
    for (int w = 0; w < SAMPLE_THREADS / 32; ++w) tot += scratch[w];
    return tot;
}

struct SampleRow {
    float temperature;
    int top_k;
    float top_p;
    float min_p;
};

// out_token [R]; kept_count [R] (optional, for tests): number of tokens that passed the filters.
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(
    const float* __restrict__ logits, long long row_stride, int V,
    const float* __restrict__ temperature, const int* __restrict__ top_k,
    const float* __restrict__ top_p, const float* __restrict__ min_p,
    const u64* __restrict__ seeds, const u64* __restrict__ counters, int* __restrict__ out_token,
    int* __restrict__ kept_count) {
    pdl_entry();
    __shared__ u64 scratch[SAMPLE_THREADS / 32];
    __shared__ u64 hist[256];
    __shared__ float wmax[32];
    __shared__ int widx[32];
    __shared__ unsigned sel_prefix;
    __shared__ u64 sel_above;
    __shared__ int found;
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const float* row = logits + r * row_stride;

    // ---- maximum and its first index (the greedy answer)
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float v = row[i];
        if (v > best) {
            best = v;
            best_i = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) {
            best = ov;
            best_i = oi;
        }
    }
    if (lane == 0) {
        wmax[wid] = best;
        widx[wid] = best_i;
    }
    __syncthreads();
    if (tid == 0) {
        float b = wmax[0];
        int bi = widx[0];
        for (int w = 1; w < SAMPLE_THREADS / 32; ++w) {
            if (wmax[w] > b || (wmax[w] == b && widx[w] < bi)) {
                b = wmax[w];
                bi = widx[w];
            }
        }
        wmax[0] = b;
        widx[0] = bi;
    }
    __syncthreads();
    const float mx = wmax[0];
    const int arg = widx[0];
    const float temp = temperature[r];
    if (!(temp > 0.0f)) {
        if (tid == 0) {
            out_token[r] = arg;
            if (kept_count) kept_count[r] = 1;
        }
        return;
    }
    const float inv_t = 1.0f / temp;

    // ---- top-k: the k-th largest logit by radix select on order-preserving keys
    unsigned key_thr = 0;  // keep tokens with order_key(logit) >= key_thr
    const int kk = top_k[r];
    if (kk > 0 && kk < V) {
        unsigned prefix = 0;
        u64 above = 0;  // tokens known to be above the current prefix bucket
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) hist[tid] = 0;
            __syncthreads();
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const unsigned k = order_key(row[i]);
                const bool match = pass == 0 || (k >> (shift + 8)) == (prefix >> (shift + 8));
                if (match) atomicAdd(&hist[(k >> shift) & 255u], 1ULL);
            }
            __syncthreads();
            if (tid == 0) {
                u64 cum = above;
                int b = 255;
                for (; b > 0; --b) {
                    if (cum + hist[b] >= static_cast<u64>(kk)) break;
                    cum += hist[b];
                }
                sel_prefix = prefix | (static_cast<unsigned>(b) << shift);
                sel_above = cum;
            }
            __syncthreads();
            prefix = sel_prefix;
            above = sel_above;
        }
        key_thr = prefix;
    }

    // ---- total weight of the top-k survivors
    u64 part = 0;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float v = row[i];
        if (order_key(v) >= key_thr) part += fixed_weight(v, mx, inv_t);
    }
    const u64 total = block_sum_u64(part, scratch);

    // ---- top-p: smallest weight w_thr such that the tokens with weight >= w_thr hold at
    // least top_p of the total; radix select on the fixed-point weights by mass
    u64 w_thr = 0;
    const float tp = top_p[r];
    if (tp < 1.0f) {
        const u64 target = static_cast<u64>(static_cast<double>(tp) * static_cast<double>(total));
        u64 prefix = 0, above = 0;
        for (int pass = 0; pass < 6; ++pass) {  // 48-bit weights (<= 2^40), 8 bits a pass
            const int shift = 40 - 8 * pass;
            if (tid < 256) hist[tid] = 0;
            __syncthreads();
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const float v = row[i];
                if (order_key(v) < key_thr) continue;
                const u64 w = fixed_weight(v, mx, inv_t);
                const bool match = pass == 0 || (w >> (shift + 8)) == (prefix >> (shift + 8));
                if (match) atomicAdd(&hist[(w >> shift) & 255ULL], w);
            }
            __syncthreads();
            if (tid == 0) {
                u64 cum = above;
                int b = 255;
                for (; b > 0; --b) {
                    if (cum + hist[b] >= target) break;
                    cum += hist[b];
                }
                sel_above = cum;
                hist[0] = prefix | (static_cast<u64>(b) << shift);
            }
            __syncthreads();
            prefix = hist[0];
            above = sel_above;
            __syncthreads();
        }
        w_thr = prefix;
    }
    // ---- min-p: weight >= min_p * (largest weight = 1.0)
    const float mp = min_p[r];
    if (mp > 0.0f) {
        const u64 m_thr = static_cast<u64>(static_cast<double>(mp) * 1099511627776.0);
        if (m_thr > w_thr) w_thr = m_thr;
    }

    // ---- kept total and count
    u64 kpart = 0, cpart = 0;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float v = row[i];
        if (order_key(v) < key_thr) continue;
        const u64 w = fixed_weight(v, mx, inv_t);
        if (w >= w_thr || i == arg) {
            kpart += w;
            cpart += 1;
        }
    }
    const u64 kept_total = block_sum_u64(kpart, scratch);
    const u64 kept_n = block_sum_u64(cpart, scratch);
    if (tid == 0 && kept_count) kept_count[r] = static_cast<int>(kept_n);

    // ---- draw: u in [0, 1) from (seed, counter); first index whose running sum exceeds it
    const u64 bits = mix64(mix64(seeds[r]) ^ (counters[r] * 0xd1342543de82ef95ULL + 1ULL));
    const double u = static_cast<double>(bits >> 11) * (1.0 / 9007199254740992.0);
    u64 goal = static_cast<u64>(u * static_cast<double>(kept_total));
    if (goal >= kept_total) goal = kept_total - 1;
    if (tid == 0) found = arg;  // fallback (kept_total of 0 cannot happen: arg weighs 2^40)
    u64 running = 0;
    __syncthreads();
    for (int base = 0; base < V; base += SAMPLE_THREADS) {
        const int i = base + tid;
        u64 w = 0;
        if (i < V) {
            const float v = row[i];
            if (order_key(v) >= key_thr) {
                const u64 ww = fixed_weight(v, mx, inv_t);
                if (ww >= w_thr || i == arg) w = ww;
            }
        }
        // inclusive scan over the block
        u64 inc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u64 up = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += up;
        }
        __syncthreads();
        if (lane == 31) scratch[wid] = inc;
        __syncthreads();
        u64 before = running;
        for (int w2 = 0; w2 < wid; ++w2) before += scratch[w2];
        u64 chunk_total = 0;
        for (int w2 = 0; w2 < SAMPLE_THREADS / 32; ++w2) chunk_total += scratch[w2];
        const u64 hi = before + inc, lo = hi - w;
        if (w > 0 && lo <= goal && goal < hi) found = i;  // exactly one thread overall
        running += chunk_total;
        if (running > goal) break;  // uniform across the block
    }
    __syncthreads();
    if (tid == 0) out_token[r] = found;
}

extern "C" int locus_sample(const float* logits, long long row_stride, int R, int V,
                            const float* temperature, const int* top_k, const float* top_p,
                            const float* min_p, const u64* seeds, const u64* counters,
                            int* out_token, int* kept_count, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return LOCUS_ERR_UNSUPPORTED;
    locus_launch(sample_kernel, R, SAMPLE_THREADS, 0, stream, logits, row_stride, V, temperature, top_k, top_p, min_p,
                 seeds, counters, out_token, kept_count);
    return locus_launch_status();
}
