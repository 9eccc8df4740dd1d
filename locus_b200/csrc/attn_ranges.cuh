// How a decode step's keys are cut into ranges that fill the warps of a fixed grid: shared by the decode
// attention kernels (attention.cu, attention_gqa.cu).  Every block computes the same cut from the batch's
// context lengths.
#pragma once

#define DS_CAND 256       // candidate range lengths looked at
#define DS_MAX_ITEMS 1024

// The per-block tables of a cut (shared memory of the calling kernel).
struct KeyRanges {
    int first[DS_MAX_ITEMS];     // first key of item i, rounded down to 32
    int nkeys[DS_MAX_ITEMS];     // keys from there to the query's own position
    int pref[DS_MAX_ITEMS + 1];  // ranges of the items before i
    int seg[DS_MAX_ITEMS], pos[DS_MAX_ITEMS], row[DS_MAX_ITEMS];  // segment, position, row of q / out
    unsigned long long best[32];
    int len;
};

// Fills `kr` (all threads of the block take part; ends with a barrier) and returns the range length in keys,
// 0 when not even one range per (request, unit) fits max_units.  `per_range`: units of work per range of keys
// (query heads, or key/value heads when a warp serves a whole group); cost of a cut = rounds over the grid's
// n_warps warps x (range length + cost_range) + cost_merge x ranges of the longest request.
__device__ __forceinline__ int plan_key_ranges(KeyRanges& kr, const int* __restrict__ items,
                                               const int* __restrict__ seg_ctx, const int* __restrict__ seg_q0,
                                               int window, int n_items, int per_range, long long max_units,
                                               int n_warps, int cost_range, int cost_merge) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_block_warps = blockDim.x >> 5;
    int longest = 0;
    for (int i = tid; i < n_items; i += blockDim.x) {
        const int seg = items[i];
        const int p = seg_ctx[seg];
        const int t_lo = window > 0 ? max(0, p - window + 1) : 0;
        const int first = t_lo & ~31;
        kr.first[i] = first;
        kr.nkeys[i] = p - first + 1;
        kr.seg[i] = seg;
        kr.pos[i] = p;
        kr.row[i] = seg_q0[seg];
    }
    __syncthreads();
    for (int i = 0; i < n_items; ++i) longest = max(longest, kr.nkeys[i]);
    // candidates: multiples of `step` keys; a thread looks at a few of them
    const int step = 32 * ((longest + 32 * DS_CAND - 1) / (32 * DS_CAND));
    unsigned long long best = ~0ull;
    for (int c = tid; c < DS_CAND; c += blockDim.x) {
        const int len = step * (c + 1);
        if (len - step >= longest && c > 0) break;  // longer than any context: same cut as the one before
        long long units = 0;
        for (int i = 0; i < n_items; ++i) units += (kr.nkeys[i] + len - 1) / len;
        units *= per_range;
        if (units > max_units) continue;  // the scratch does not hold that many partial results
        const long long rounds = (units + n_warps - 1) / n_warps;
        // the merge of a (request, head) runs in one warp and grows with its number of ranges
        const unsigned long long cost = static_cast<unsigned long long>(rounds) * (len + cost_range) +
                                        cost_merge * static_cast<unsigned long long>((longest + len - 1) / len);
        best = min(best, (cost << 24) | static_cast<unsigned>(c));  // ties: the shorter range
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (lane == 0) kr.best[warp] = best;
    __syncthreads();
    if (tid == 0) {
        unsigned long long b = kr.best[0];
        for (int w = 1; w < n_block_warps; ++w) b = min(b, kr.best[w]);
        // nothing fits (a scratch smaller than one range per (request, unit)): refused on the host
        kr.len = b == ~0ull ? 0 : step * (static_cast<int>(b & 0xffffff) + 1);
        int acc = 0;
        const int len = max(32, kr.len);
        for (int i = 0; i < n_items; ++i) {
            kr.pref[i] = acc;
            acc += (kr.nkeys[i] + len - 1) / len;
        }
        kr.pref[n_items] = acc;
    }
    __syncthreads();
    return kr.len;
}
