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
    return __float2ull_rz(w * 1099511627776.0f);  // w * 2^40 is exact in float32: the value the double product gives
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

// Histogram updates without a fight over the popular bins.  Logits cluster: the tokens of a row fall into a few of
// a pass's 256 bins (all into one, in the passes over the weights), and 150,000 atomic additions to a few
// shared-memory words take milliseconds.  So every warp has a histogram of its own (32 x 256 words, added up
// after the pass), a thread gathers a run of equal bins in registers and adds it when the bin changes, and what
// it holds at the end goes out as one addition per warp when the whole warp holds the same bin.  The sums are
// integers: the result is the same whatever the order.
// hist[bin] += v in shared memory with two native 32-bit additions (a 64-bit addition to shared memory is a
// compare-and-swap loop): the low word's return value tells whether it wrapped, and the carry goes into the high
// word's addition.  Exact whatever the interleaving; the sums are read after a barrier.
__device__ __forceinline__ void hist_add(u64* hist, int bin, u64 v) {
    unsigned* h = reinterpret_cast<unsigned*>(hist + bin);
    const unsigned lo = static_cast<unsigned>(v);
    const unsigned old = atomicAdd(h, lo);
    const unsigned hi = static_cast<unsigned>(v >> 32) + ((old + lo) < old ? 1u : 0u);
    if (hi != 0) atomicAdd(h + 1, hi);
}

struct RunAcc {
    int bin;
    u64 sum;
};
__device__ __forceinline__ void run_add(RunAcc& acc, u64* hist, int bin, u64 val) {
    if (bin != acc.bin) {
        if (acc.sum != 0) hist_add(hist, acc.bin, acc.sum);
        acc.bin = bin;
        acc.sum = 0;
    }
    acc.sum += val;
}
__device__ __forceinline__ void run_flush(RunAcc& acc, u64* hist) {  // all threads of the warp call it
    int same = 0;
    __match_all_sync(0xffffffffu, acc.bin, &same);
    if (same) {
        u64 v = acc.sum;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) == 0 && v != 0) hist_add(hist, acc.bin, v);
    } else if (acc.sum != 0) {
        hist_add(hist, acc.bin, acc.sum);
    }
    acc.bin = 0;
    acc.sum = 0;
}

// f(i, row[i]) for the elements [begin, end) of a row, spread over `nt` threads of which this is `t`.  With `vec`
// (the row starts on a 16-byte boundary and begin is a multiple of 4) four elements come with one load: one block
// reads a whole row of the vocabulary, and what bounds it is the number of loads it has in flight.
template <typename F>
__device__ __forceinline__ void row_each(const float* __restrict__ row, int begin, int end, int t, int nt, bool vec, F f) {
    if (vec) {
        const float4* r4 = reinterpret_cast<const float4*>(row + begin);
        const int n4 = (end - begin) >> 2;
#pragma unroll 2
        for (int j = t; j < n4; j += nt) {
            const float4 v = r4[j];
            const int i = begin + 4 * j;
            f(i, v.x);
            f(i + 1, v.y);
            f(i + 2, v.z);
            f(i + 3, v.w);
        }
        for (int i = begin + 4 * n4 + t; i < end; i += nt) f(i, row[i]);
    } else {
        for (int i = begin + t; i < end; i += nt) f(i, row[i]);
    }
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
    extern __shared__ u64 warp_hist[];  // [SAMPLE_THREADS / 32][256]
    __shared__ u64 scratch[SAMPLE_THREADS / 32];
    __shared__ u64 hist[256];
    __shared__ float wmax[32];
    __shared__ int widx[32];
    __shared__ unsigned sel_prefix;
    __shared__ u64 sel_above;
    __shared__ u64 seg_total[SAMPLE_THREADS / 32];
    __shared__ u64 seg_count[SAMPLE_THREADS / 32];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const float* row = logits + r * row_stride;
    u64* const mine = warp_hist + wid * 256;

    // ---- maximum and its first index (the greedy answer)
    const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    row_each(row, 0, V, tid, SAMPLE_THREADS, vec, [&](int i, float v) {
        if (v > best || (v == best && i < best_i)) {
            best = v;
            best_i = i;
        }
    });
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
            for (int i = tid; i < SAMPLE_THREADS / 32 * 256; i += SAMPLE_THREADS) warp_hist[i] = 0;
            __syncthreads();
            RunAcc acc{0, 0};
            row_each(row, 0, V, tid, SAMPLE_THREADS, vec, [&](int, float v) {
                const unsigned k = order_key(v);
                const bool match = pass == 0 || (k >> (shift + 8)) == (prefix >> (shift + 8));
                if (match) run_add(acc, mine, static_cast<int>((k >> shift) & 255u), 1ULL);
            });
            run_flush(acc, mine);
            __syncthreads();
            if (tid < 256) {
                u64 c = 0;
                for (int w = 0; w < SAMPLE_THREADS / 32; ++w) c += warp_hist[w * 256 + tid];
                hist[tid] = c;
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

    // ---- top-p: smallest weight w_thr such that the tokens with weight >= w_thr hold at
    // least top_p of the total; radix select on the fixed-point weights by mass
    u64 w_thr = 0;
    const float tp = top_p[r];
    if (tp < 1.0f) {
        // total weight of the top-k survivors
        u64 part = 0;
        row_each(row, 0, V, tid, SAMPLE_THREADS, vec, [&](int, float v) {
            if (order_key(v) >= key_thr) part += fixed_weight(v, mx, inv_t);
        });
        const u64 total = block_sum_u64(part, scratch);
        const u64 target = static_cast<u64>(static_cast<double>(tp) * static_cast<double>(total));
        u64 prefix = 0, above = 0;
        for (int pass = 0; pass < 6; ++pass) {  // 48-bit weights (<= 2^40), 8 bits a pass
            const int shift = 40 - 8 * pass;
            for (int i = tid; i < SAMPLE_THREADS / 32 * 256; i += SAMPLE_THREADS) warp_hist[i] = 0;
            __syncthreads();
            RunAcc acc{0, 0};
            row_each(row, 0, V, tid, SAMPLE_THREADS, vec, [&](int, float v) {
                if (order_key(v) < key_thr) return;
                const u64 w = fixed_weight(v, mx, inv_t);
                const bool match = pass == 0 || (w >> (shift + 8)) == (prefix >> (shift + 8));
                if (match) run_add(acc, mine, static_cast<int>((w >> shift) & 255ULL), w);
            });
            run_flush(acc, mine);
            __syncthreads();
            if (tid < 256) {
                u64 c = 0;
                for (int w = 0; w < SAMPLE_THREADS / 32; ++w) c += warp_hist[w * 256 + tid];
                hist[tid] = c;
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

    // ---- kept weight and count of every warp's own stretch of the row (warp w holds the tokens
    // [w * seg, (w + 1) * seg), seg a multiple of 128: a lane takes four neighbours at a time)
    const int seg = ((V + SAMPLE_THREADS / 32 - 1) / (SAMPLE_THREADS / 32) + 127) & ~127;
    const int seg0 = min(V, wid * seg), seg1 = min(V, seg0 + seg);
    auto kept_weight = [&](int i, float v, bool& kept) -> u64 {  // a kept token may weigh 0 (below 2^-40 of the largest)
        kept = false;
        if (order_key(v) < key_thr) return 0;
        const u64 w = fixed_weight(v, mx, inv_t);
        kept = w >= w_thr || i == arg;
        return kept ? w : 0;
    };
    {
        u64 kpart = 0, cpart = 0;
        row_each(row, seg0, seg1, lane, 32, vec, [&](int i, float v) {
            bool kept;
            kpart += kept_weight(i, v, kept);
            cpart += kept;
        });
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            kpart += __shfl_xor_sync(0xffffffffu, kpart, o);
            cpart += __shfl_xor_sync(0xffffffffu, cpart, o);
        }
        if (lane == 0) {
            seg_total[wid] = kpart;
            seg_count[wid] = cpart;
        }
    }
    __syncthreads();
    u64 kept_total = 0, kept_n = 0, before = 0;
    for (int w = 0; w < SAMPLE_THREADS / 32; ++w) {
        if (w < wid) before += seg_total[w];
        kept_total += seg_total[w];
        kept_n += seg_count[w];
    }
    if (tid == 0 && kept_count) kept_count[r] = static_cast<int>(kept_n);

    // ---- draw: u in [0, 1) from (seed, counter); first index whose running sum exceeds it.  The warp whose
    // stretch holds the goal walks it 128 tokens at a time (a lane four neighbours, the next four already asked
    // for); nobody else has anything left to do.
    const u64 bits = mix64(mix64(seeds[r]) ^ (counters[r] * 0xd1342543de82ef95ULL + 1ULL));
    const double u = static_cast<double>(bits >> 11) * (1.0 / 9007199254740992.0);
    u64 goal = static_cast<u64>(u * static_cast<double>(kept_total));
    if (goal >= kept_total) goal = kept_total - 1;  // (a kept total of 0 cannot happen: arg weighs 2^40)
    if (!(before <= goal && goal < before + seg_total[wid])) return;
    u64 running = before;
    int found = arg;
    auto load4 = [&](int i0, float* v) {  // the tokens i0 .. i0 + 3 (zeros of no weight behind the stretch's end)
        if (vec && i0 + 3 < seg1) {
            const float4 t = *reinterpret_cast<const float4*>(row + i0);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = i0 + e < seg1 ? row[i0 + e] : -INFINITY;
        }
    };
    float cur[4], nxt[4];
    load4(seg0 + 4 * lane, cur);
    for (int base = seg0; base < seg1; base += 128) {
        const int i0 = base + 4 * lane;
        load4(i0 + 128, nxt);
        u64 w[4], mine_sum = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            bool kept = false;
            w[e] = i0 + e < seg1 ? kept_weight(i0 + e, cur[e], kept) : 0;
            mine_sum += w[e];
        }
        u64 inc = mine_sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u64 up = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += up;
        }
        const u64 hi = running + inc, lo = hi - mine_sum;
        const bool here = mine_sum > 0 && lo <= goal && goal < hi;  // at most one lane
        const unsigned hit = __ballot_sync(0xffffffffu, here);
        if (hit != 0) {
            if (here) {
                u64 at = lo;
                int e = 0;
                for (; e < 3; ++e) {
                    if (goal < at + w[e]) break;
                    at += w[e];
                }
                out_token[r] = i0 + e;
            }
            return;
        }
        running += __shfl_sync(0xffffffffu, inc, 31);
#pragma unroll
        for (int e = 0; e < 4; ++e) cur[e] = nxt[e];
    }
    if (lane == 0) out_token[r] = found;
}

// ---------------------------------------------------------------------------
// The same sampling for rows of up to SC_CTAS * SAMPLE_THREADS * SC_E tokens by a CLUSTER of eight blocks per row.
// One block has to make a dozen passes over the row, each bound by what one SM can issue (an exponential per
// token and pass); here a thread owns SC_E consecutive tokens, reads them once and keeps their logits, then their
// fixed-point weights, in registers, so that a pass is a few instructions per token, and eight SMs share the
// row.  What the passes need from the whole row (maximum, histograms, totals) is published in each block's
// shared memory, alternately in two slots, and read by all eight blocks across the cluster after one cluster
// barrier (a hardware barrier: every block of a row passes the same barriers in the same order).  Every block
// comes to the same decisions from the same sums; the block and thread whose tokens hold the draw's goal write
// the token.  Same filters, same fixed-point arithmetic, same draw and so the same token as sample_kernel.
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SC_CTAS 8
#define SC_E 20   // tokens of a thread (a multiple of 4): rows of up to 163,840 tokens

struct ClusterPub {            // what a block publishes for the others, two slots used alternately
    u64 hist[2][256];
    u64 sum[2][2];
    float max_v[2];
    int max_i[2];
};

__global__ void __launch_bounds__(SAMPLE_THREADS, 1) sample_cluster_kernel(
    const float* __restrict__ logits, long long row_stride, int V,
    const float* __restrict__ temperature, const int* __restrict__ top_k,
    const float* __restrict__ top_p, const float* __restrict__ min_p,
    const u64* __restrict__ seeds, const u64* __restrict__ counters, int* __restrict__ out_token,
    int* __restrict__ kept_count) {
    pdl_entry();
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = static_cast<int>(cluster.block_rank());
    __shared__ ClusterPub pub;
    __shared__ u64 scratch[SAMPLE_THREADS / 32];
    __shared__ u64 hist_all[256];
    __shared__ float wmax[32];
    __shared__ int widx[32];
    __shared__ u64 sel[2];
    const int r = blockIdx.x / SC_CTAS, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const float* row = logits + r * row_stride;
    const int t0 = (rank * SAMPLE_THREADS + tid) * SC_E;  // this thread's first token
    int slot = 0;                                          // the slot of `pub` that the next exchange uses

    // ---- the thread's tokens (tokens behind the row's end: -inf, never kept)
    float lg[SC_E];
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0 && t0 + SC_E <= V) {
#pragma unroll
        for (int j = 0; j < SC_E; j += 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + t0 + j);
            lg[j] = v.x; lg[j + 1] = v.y; lg[j + 2] = v.z; lg[j + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < SC_E; ++j) lg[j] = t0 + j < V ? row[t0 + j] : -INFINITY;
    }
    const int n_mine = max(0, min(SC_E, V - t0));  // tokens of this thread that exist

    // ---- maximum and its first index (the greedy answer)
    float best = -INFINITY;
    int best_i = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < SC_E; ++j)
        if (j < n_mine && lg[j] > best) {
            best = lg[j];
            best_i = t0 + j;
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
        for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
            if (wmax[w] > b || (wmax[w] == b && widx[w] < bi)) {
                b = wmax[w];
                bi = widx[w];
            }
        pub.max_v[slot] = b;
        pub.max_i[slot] = bi;
    }
    cluster.sync();
    float mx = -INFINITY;
    int arg = 0x7fffffff;
    for (int c = 0; c < SC_CTAS; ++c) {
        const ClusterPub* o = cluster.map_shared_rank(&pub, c);
        const float v = o->max_v[slot];
        const int i = o->max_i[slot];
        if (v > mx || (v == mx && i < arg)) {
            mx = v;
            arg = i;
        }
    }
    slot ^= 1;
    const float temp = temperature[r];
    if (!(temp > 0.0f)) {
        if (rank == 0 && tid == 0) {
            out_token[r] = arg;
            if (kept_count) kept_count[r] = 1;
        }
        cluster.sync();  // nobody leaves while another block may still read its shared memory
        return;
    }
    const float inv_t = 1.0f / temp;

    // One exchange of a 256-bin histogram: every block adds the eight published ones up into hist_all.
    auto all_hist = [&]() {
        cluster.sync();
        if (tid < 256) {
            u64 c = 0;
            for (int b = 0; b < SC_CTAS; ++b) c += cluster.map_shared_rank(&pub, b)->hist[slot][tid];
            hist_all[tid] = c;
        }
        slot ^= 1;
        __syncthreads();
    };
    // One exchange of two sums.
    auto all_sums = [&](u64 a, u64 b, u64& ta, u64& tb) {
        a = block_sum_u64(a, scratch);
        b = block_sum_u64(b, scratch);
        if (tid == 0) {
            pub.sum[slot][0] = a;
            pub.sum[slot][1] = b;
        }
        cluster.sync();
        ta = tb = 0;
        for (int c = 0; c < SC_CTAS; ++c) {
            const ClusterPub* o = cluster.map_shared_rank(&pub, c);
            ta += o->sum[slot][0];
            tb += o->sum[slot][1];
        }
        slot ^= 1;
    };

    // ---- top-k: the k-th largest logit by radix select on order-preserving keys
    unsigned key_thr = 0;  // keep tokens with order_key(logit) >= key_thr
    const int kk = top_k[r];
    if (kk > 0 && kk < V) {
        unsigned prefix = 0;
        u64 above = 0;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) pub.hist[slot][tid] = 0;
            __syncthreads();
            RunAcc acc{0, 0};
#pragma unroll
            for (int j = 0; j < SC_E; ++j) {
                const unsigned k = order_key(lg[j]);
                const bool match = j < n_mine && (pass == 0 || (k >> (shift + 8)) == (prefix >> (shift + 8)));
                if (match) run_add(acc, pub.hist[slot], static_cast<int>((k >> shift) & 255u), 1ULL);
            }
            run_flush(acc, pub.hist[slot]);
            all_hist();
            if (tid == 0) {
                u64 cum = above;
                int b = 255;
                for (; b > 0; --b) {
                    if (cum + hist_all[b] >= static_cast<u64>(kk)) break;
                    cum += hist_all[b];
                }
                sel[0] = prefix | (static_cast<unsigned>(b) << shift);
                sel[1] = cum;
            }
            __syncthreads();
            prefix = static_cast<unsigned>(sel[0]);
            above = sel[1];
            __syncthreads();
        }
        key_thr = prefix;
    }

    // ---- fixed-point weights of the top-k survivors; `alive` marks them (a survivor may weigh 0)
    u64 w[SC_E];
    unsigned alive = 0;
#pragma unroll
    for (int j = 0; j < SC_E; ++j) {
        const bool in = j < n_mine && order_key(lg[j]) >= key_thr;
        w[j] = in ? fixed_weight(lg[j], mx, inv_t) : 0;
        alive |= in ? 1u << j : 0u;
    }

    // ---- top-p: smallest weight w_thr such that the tokens with weight >= w_thr hold at least top_p of the total
    u64 w_thr = 0;
    const float tp = top_p[r];
    if (tp < 1.0f) {
        u64 part = 0;
#pragma unroll
        for (int j = 0; j < SC_E; ++j) part += w[j];
        u64 total, unused;
        all_sums(part, 0, total, unused);
        const u64 target = static_cast<u64>(static_cast<double>(tp) * static_cast<double>(total));
        u64 prefix = 0, above = 0;
        for (int pass = 0; pass < 6; ++pass) {  // 48-bit weights (<= 2^40), 8 bits a pass
            const int shift = 40 - 8 * pass;
            if (tid < 256) pub.hist[slot][tid] = 0;
            __syncthreads();
            RunAcc acc{0, 0};
#pragma unroll
            for (int j = 0; j < SC_E; ++j) {
                const bool match = ((alive >> j) & 1u) && (pass == 0 || (w[j] >> (shift + 8)) == (prefix >> (shift + 8)));
                if (match) run_add(acc, pub.hist[slot], static_cast<int>((w[j] >> shift) & 255ULL), w[j]);
            }
            run_flush(acc, pub.hist[slot]);
            all_hist();
            if (tid == 0) {
                u64 cum = above;
                int b = 255;
                for (; b > 0; --b) {
                    if (cum + hist_all[b] >= target) break;
                    cum += hist_all[b];
                }
                sel[0] = prefix | (static_cast<u64>(b) << shift);
                sel[1] = cum;
            }
            __syncthreads();
            prefix = sel[0];
            above = sel[1];
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

    // ---- what is kept: weight and count of this thread, of the threads before it in the block, of the blocks
    u64 mine_w = 0, mine_n = 0;
#pragma unroll
    for (int j = 0; j < SC_E; ++j) {
        const bool kept = ((alive >> j) & 1u) && (w[j] >= w_thr || t0 + j == arg);
        if (!kept) w[j] = 0;
        mine_w += w[j];
        mine_n += kept;
    }
    u64 inc = mine_w;  // inclusive scan over the block, in thread order
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 up = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += up;
    }
    __syncthreads();
    if (lane == 31) scratch[wid] = inc;
    __syncthreads();
    u64 before = 0, block_w = 0;
    for (int ww = 0; ww < SAMPLE_THREADS / 32; ++ww) {
        if (ww < wid) before += scratch[ww];
        block_w += scratch[ww];
    }
    const u64 block_n = block_sum_u64(mine_n, scratch);
    if (tid == 0) {
        pub.sum[slot][0] = block_w;
        pub.sum[slot][1] = block_n;
    }
    cluster.sync();
    u64 kept_total = 0, kept_n = 0, blocks_before = 0;
    for (int c = 0; c < SC_CTAS; ++c) {
        const ClusterPub* o = cluster.map_shared_rank(&pub, c);
        const u64 bw = o->sum[slot][0];
        if (c < rank) blocks_before += bw;
        kept_total += bw;
        kept_n += o->sum[slot][1];
    }
    if (rank == 0 && tid == 0 && kept_count) kept_count[r] = static_cast<int>(kept_n);

    // ---- draw: u in [0, 1) from (seed, counter); first token whose running sum exceeds it
    const u64 bits = mix64(mix64(seeds[r]) ^ (counters[r] * 0xd1342543de82ef95ULL + 1ULL));
    const double u = static_cast<double>(bits >> 11) * (1.0 / 9007199254740992.0);
    u64 goal = static_cast<u64>(u * static_cast<double>(kept_total));
    if (goal >= kept_total) goal = kept_total - 1;  // (a kept total of 0 cannot happen: arg weighs 2^40)
    const u64 hi = blocks_before + before + inc, lo = hi - mine_w;
    if (mine_w > 0 && lo <= goal && goal < hi) {  // exactly one thread of the cluster
        u64 at = lo;
        int j = 0;
#pragma unroll
        for (int e = 0; e < SC_E - 1; ++e) {
            if (j == e && !(goal < at + w[e])) {
                at += w[e];
                j = e + 1;
            }
        }
        out_token[r] = t0 + j;
    }
    cluster.sync();  // nobody leaves while another block may still read its shared memory
}

// A switch for tests and measurements: 0 keeps every row on the one-block kernel.
static int g_sample_cluster = 1;
static int g_sample_cluster_rows = 16;   // more rows than this fill the GPU with one block each
extern "C" void locus_sample_use_cluster(int on) { g_sample_cluster = on; g_sample_cluster_rows = on > 1 ? on : 16; }

extern "C" int locus_sample(const float* logits, long long row_stride, int R, int V,
                            const float* temperature, const int* top_k, const float* top_p,
                            const float* min_p, const u64* seeds, const u64* counters,
                            int* out_token, int* kept_count, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return LOCUS_ERR_UNSUPPORTED;
    // rows that a cluster's threads hold in registers (and that are worth eight blocks): the cluster kernel
    if (g_sample_cluster && R <= g_sample_cluster_rows && V >= 8192 && V <= SC_CTAS * SAMPLE_THREADS * SC_E) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(R) * SC_CTAS);
        cfg.blockDim = dim3(SAMPLE_THREADS);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = SC_CTAS;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_locus_pdl ? 2 : 1;
        cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, row_stride, V, temperature, top_k, top_p, min_p, seeds,
                           counters, out_token, kept_count);
        return locus_launch_status();
    }
    const size_t smem = sizeof(u64) * (SAMPLE_THREADS / 32) * 256;  // a histogram per warp
    static bool set = false;
    if (!set) {
        if (cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
            return static_cast<int>(cudaGetLastError());
        set = true;
    }
    locus_launch(sample_kernel, R, SAMPLE_THREADS, smem, stream, logits, row_stride, V, temperature, top_k, top_p, min_p,
                 seeds, counters, out_token, kept_count);
    return locus_launch_status();
}
