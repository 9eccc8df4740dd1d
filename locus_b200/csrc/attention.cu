// Attention over the paged cache on CUDA cores, float32 arithmetic throughout: scores,
// scale, mask, softmax statistics and the weighted sum of V.  Two kernels:
//
//   * chunk:  a tile of up to 16 consecutive new tokens of one request against every key
//             it may see (earlier pages plus the causal triangle inside the portion);
//   * decode: one new token of a request, its keys split into fixed ranges of 128
//             absolute positions, partial results merged in ascending order.
//
// Both read K and V through the request's block table, honour an optional window (a query
// at position p sees keys t with p - window < t <= p; window 0 = all keys) and take any head
// size that is a multiple of 16 up to 256, any number of heads and any group ratio.
// Cache layout of one layer: [n_pages][2 (K, V)][nkv][page_tokens][hd].
#include "common.cuh"
#include "attn_ranges.cuh"

struct AttnArgs {
    const void* q;            // [T, nh * hd]
    const void* pool;         // this layer's pages
    void* out;                // [T, nh * hd]
    const int* seg_q0;        // [n_seg] first row of the segment in q / out
    const int* seg_qn;        // [n_seg] new tokens of the segment
    const int* seg_ctx;       // [n_seg] tokens already cached = position of its first new token
    const int* block_table;   // [n_seg, table_stride] page ids; entries behind a window may be -1
    int table_stride;
    const int* items;         // chunk: [n_items, 2] (segment, first query of the tile within it)
                              // decode: [n_items] segment ids
    int nh, nkv, hd, page_tokens, window;
    float scale;
    // decode only
    float* part_o;            // [n_items, nh, max_splits, hd]
    float* part_ml;           // [n_items, nh, max_splits, 2]
    int* counters;            // [n_items, nh], zero between launches
    int max_splits;
};

#define CHUNK_BQ 16
#define CHUNK_TK 32
#define DEC_SPLIT 128

// Error word of this module: set by a kernel that was launched with arguments that do not fit the batch it
// finds on the device (1: max_splits does not cover the longest context of a decode step); the kernel still
// ends in order and leaves its counters zero, but the output of the affected requests is incomplete.
__device__ int g_attn_error = 0;

extern "C" int locus_attn_error() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
    }
    return v;
}

template <typename T>
__device__ __forceinline__ const T* kv_row(const AttnArgs& a, const int* table, int t, int kvh,
                                            int which) {
    const int page = table[t / a.page_tokens];
    const int off = t % a.page_tokens;
    const size_t base = (static_cast<size_t>(page) * 2 + which) * a.nkv * a.page_tokens * a.hd;
    return static_cast<const T*>(a.pool) + base +
           (static_cast<size_t>(kvh) * a.page_tokens + off) * a.hd;
}

// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) attn_chunk_kernel(AttnArgs a) {
    extern __shared__ float smem[];
    const int hd = a.hd;
    float* qs = smem;                              // [BQ][hd]
    float* ks = qs + CHUNK_BQ * hd;                // [TK][hd + 1]
    float* vs = ks + CHUNK_TK * (hd + 1);          // [TK][hd]
    float* sc = vs + CHUNK_TK * hd;                // [BQ][TK + 1]
    float* m_s = sc + CHUNK_BQ * (CHUNK_TK + 1);   // [BQ]
    float* l_s = m_s + CHUNK_BQ;                   // [BQ]
    float* al_s = l_s + CHUNK_BQ;                  // [BQ]

    // the late tiles of a prompt see the most keys: the grid takes them first, for all heads (its fast index)
    const int item = gridDim.y - 1 - blockIdx.y;
    const int seg = a.items[2 * item], qoff = a.items[2 * item + 1];
    const int h = blockIdx.x;
    const int kvh = h / (a.nh / a.nkv);
    const int nq = min(CHUNK_BQ, a.seg_qn[seg] - qoff);
    const int row0 = a.seg_q0[seg] + qoff;
    const int p0 = a.seg_ctx[seg] + qoff;  // position of the tile's first query
    const int* table = a.block_table + static_cast<size_t>(seg) * a.table_stride;
    const int tid = threadIdx.x;

    for (int i = tid; i < CHUNK_BQ * hd; i += 128) {
        const int qi = i / hd, d = i % hd;
        qs[i] = qi < nq ? to_f(static_cast<const T*>(a.q)[(static_cast<size_t>(row0 + qi) * a.nh + h) * hd + d])
                        : 0.f;
    }
    if (tid < CHUNK_BQ) {
        m_s[tid] = -INFINITY;
        l_s[tid] = 0.f;
    }
    const int t_hi = p0 + nq - 1;
    const int t_lo = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
    const int nd = hd / 8;
    const int my_q = tid >> 3, dl = tid & 7;
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
    __syncthreads();

    for (int tile0 = (t_lo / CHUNK_TK) * CHUNK_TK; tile0 <= t_hi; tile0 += CHUNK_TK) {
        for (int i = tid; i < CHUNK_TK * hd; i += 128) {
            const int kj = i / hd, d = i % hd;
            const int t = tile0 + kj;
            float kv = 0.f, vv = 0.f;
            if (t >= t_lo && t <= t_hi) {
                kv = to_f(kv_row<T>(a, table, t, kvh, 0)[d]);
                vv = to_f(kv_row<T>(a, table, t, kvh, 1)[d]);
            }
            ks[kj * (hd + 1) + d] = kv;
            vs[kj * hd + d] = vv;
        }
        __syncthreads();
        for (int i = tid; i < CHUNK_BQ * CHUNK_TK; i += 128) {
            const int qi = i / CHUNK_TK, kj = i % CHUNK_TK;
            const int t = tile0 + kj, p = p0 + qi;
            float s = -INFINITY;
            if (qi < nq && t <= p && t >= t_lo && (a.window == 0 || t > p - a.window)) {
                float dot = 0.f;
                const float* qr = qs + qi * hd;
                const float* kr = ks + kj * (hd + 1);
                for (int d = 0; d < hd; ++d) dot = fmaf(qr[d], kr[d], dot);
                s = dot * a.scale;
            }
            sc[qi * (CHUNK_TK + 1) + kj] = s;
        }
        __syncthreads();
        if (tid < CHUNK_BQ) {
            float* row = sc + tid * (CHUNK_TK + 1);
            float mx = m_s[tid];
            for (int kj = 0; kj < CHUNK_TK; ++kj) mx = fmaxf(mx, row[kj]);
            float alpha = 1.f, sum = 0.f;
            if (mx == -INFINITY) {
                for (int kj = 0; kj < CHUNK_TK; ++kj) row[kj] = 0.f;
            } else {
                alpha = expf(m_s[tid] - mx);  // exp(-inf) = 0 on the first live tile
                for (int kj = 0; kj < CHUNK_TK; ++kj) {
                    const float pexp = expf(row[kj] - mx);
                    row[kj] = pexp;
                    sum += pexp;
                }
            }
            m_s[tid] = mx;
            l_s[tid] = l_s[tid] * alpha + sum;
            al_s[tid] = alpha;
        }
        __syncthreads();
        {
            const float alpha = al_s[my_q];
            const float* prow = sc + my_q * (CHUNK_TK + 1);
#pragma unroll
            for (int dd = 0; dd < 32; ++dd) {
                if (dd < nd) {
                    const int d = dl + 8 * dd;
                    float v = acc[dd] * alpha;
                    for (int kj = 0; kj < CHUNK_TK; ++kj) v = fmaf(prow[kj], vs[kj * hd + d], v);
                    acc[dd] = v;
                }
            }
        }
        __syncthreads();
    }
    if (my_q < nq) {
        const float inv = 1.0f / l_s[my_q];
        T* o = static_cast<T*>(a.out) + (static_cast<size_t>(row0 + my_q) * a.nh + h) * hd;
#pragma unroll
        for (int dd = 0; dd < 32; ++dd) {
            if (dd < nd) o[dl + 8 * dd] = from_f<T>(acc[dd] * inv);
        }
    }
}

// ---------------------------------------------------------------------------
template <typename T>
struct Vec;
template <>
struct Vec<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float* o) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
    __device__ static void unpack(const uint4& v, float* o) {
        o[0] = __uint_as_float(v.x); o[1] = __uint_as_float(v.y);
        o[2] = __uint_as_float(v.z); o[3] = __uint_as_float(v.w);
    }
};
template <>
struct Vec<bf16> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4& v, float* o) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            o[2 * i] = f.x;
            o[2 * i + 1] = f.y;
        }
    }
    __device__ static void load(const bf16* p, float* o) { unpack(*reinterpret_cast<const uint4*>(p), o); }
};

// grid (n_items, nh, max_splits); split s covers absolute key positions
// [s * DEC_SPLIT, (s + 1) * DEC_SPLIT).  Writes unnormalised partial sums with their
// running maximum m and denominator l, then the last block of a (request, head) merges its splits.
template <typename T>
__global__ void __launch_bounds__(128) attn_decode_split_kernel(AttnArgs a) {
    pdl_entry();
    extern __shared__ float smem[];
    constexpr int VEC = Vec<T>::N;
    const int hd = a.hd;
    float* qs = smem;                    // [hd]
    float* sc = qs + hd;                 // [DEC_SPLIT]
    float* red = sc + DEC_SPLIT;         // [kpp][hd]
    __shared__ float wred[4];
    __shared__ float m_sh, l_sh;

    const int item = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    const int seg = a.items[item];
    const int kvh = h / (a.nh / a.nkv);
    const int p = a.seg_ctx[seg];  // position of the single query
    const int row = a.seg_q0[seg];
    const int t_lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
    const int k0 = max(t_lo, split * DEC_SPLIT);
    const int k1 = min(p, (split + 1) * DEC_SPLIT - 1);  // inclusive
    const int tid = threadIdx.x;
    const size_t part = (static_cast<size_t>(item) * a.nh + h) * a.max_splits + split;
    // The grid has max_splits blocks per (request, head).  If the caller's max_splits does not reach the split of
    // position p, the keys beyond it are not read: say so, and count and merge only the splits that exist, so that
    // the counter still returns to zero.
    const bool short_grid = p / DEC_SPLIT >= a.max_splits;
    if (short_grid && split == 0 && h == 0 && tid == 0) atomicExch(&g_attn_error, 1);
    if (k0 > k1) return;  // a split without keys: neither written nor read
    const int* table = a.block_table + static_cast<size_t>(seg) * a.table_stride;
    for (int d = tid; d < hd; d += 128)
        qs[d] = to_f(static_cast<const T*>(a.q)[(static_cast<size_t>(row) * a.nh + h) * hd + d]);
    const int nk = k1 - k0 + 1;
    // where each key row of the split starts (elements from the pool base), looked up once
    // (in units of 16 elements: rows start at multiples of hd, a multiple of 16, and the pool may hold
    // more than 2^32 elements)
    __shared__ unsigned int krow[DEC_SPLIT];
    for (int j = tid; j < nk; j += 128)
        krow[j] = static_cast<unsigned int>((kv_row<T>(a, table, k0 + j, kvh, 0) - static_cast<const T*>(a.pool)) >> 4);
    const size_t v_off = static_cast<size_t>(a.nkv) * a.page_tokens * hd;  // V row = K row + v_off
    __syncthreads();
    float mx = -INFINITY;
    for (int j = tid; j < nk; j += 128) {
        const T* kr = static_cast<const T*>(a.pool) + (static_cast<size_t>(krow[j]) << 4);
        float dot = 0.f;
        int d = 0;
        for (; d + 4 * VEC <= hd; d += 4 * VEC) {  // four loads in flight
            float kv[4][VEC];
#pragma unroll
            for (int u4 = 0; u4 < 4; ++u4) Vec<T>::load(kr + d + u4 * VEC, kv[u4]);
#pragma unroll
            for (int u4 = 0; u4 < 4; ++u4)
#pragma unroll
                for (int u = 0; u < VEC; ++u) dot = fmaf(qs[d + u4 * VEC + u], kv[u4][u], dot);
        }
        for (; d < hd; d += VEC) {
            float kv[VEC];
            Vec<T>::load(kr + d, kv);
#pragma unroll
            for (int u = 0; u < VEC; ++u) dot = fmaf(qs[d + u], kv[u], dot);
        }
        const float s = dot * a.scale;
        sc[j] = s;
        mx = fmaxf(mx, s);
    }
    mx = warp_max(mx);
    if ((tid & 31) == 0) wred[tid >> 5] = mx;
    __syncthreads();
    if (tid == 0) m_sh = fmaxf(fmaxf(wred[0], wred[1]), fmaxf(wred[2], wred[3]));
    __syncthreads();
    mx = m_sh;
    float sum = 0.f;
    for (int j = tid; j < nk; j += 128) {
        const float e = expf(sc[j] - mx);
        sc[j] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    __syncthreads();
    if ((tid & 31) == 0) wred[tid >> 5] = sum;
    __syncthreads();
    if (tid == 0) l_sh = (wred[0] + wred[1]) + (wred[2] + wred[3]);
    // weighted sum of V: tpk threads share one key, VEC dims each; kpp keys per pass
    const int tpk = hd / VEC;
    const int kpp = 128 / tpk;
    const int g = tid / tpk, dv = (tid % tpk) * VEC;
    float acc[VEC];
#pragma unroll
    for (int u = 0; u < VEC; ++u) acc[u] = 0.f;
    if (g < kpp) {
        const T* vbase = static_cast<const T*>(a.pool) + v_off + dv;
        int j = g;
        for (; j + 3 * kpp < nk; j += 4 * kpp) {  // four rows in flight
            float vv[4][VEC];
#pragma unroll
            for (int u4 = 0; u4 < 4; ++u4) Vec<T>::load(vbase + (static_cast<size_t>(krow[j + u4 * kpp]) << 4), vv[u4]);
#pragma unroll
            for (int u4 = 0; u4 < 4; ++u4) {
                const float pj = sc[j + u4 * kpp];
#pragma unroll
                for (int u = 0; u < VEC; ++u) acc[u] = fmaf(pj, vv[u4][u], acc[u]);
            }
        }
        for (; j < nk; j += kpp) {
            float vv[VEC];
            Vec<T>::load(vbase + (static_cast<size_t>(krow[j]) << 4), vv);
            const float pj = sc[j];
#pragma unroll
            for (int u = 0; u < VEC; ++u) acc[u] = fmaf(pj, vv[u], acc[u]);
        }
#pragma unroll
        for (int u = 0; u < VEC; ++u) red[g * hd + dv + u] = acc[u];
    }
    __syncthreads();
    for (int d = tid; d < hd; d += 128) {
        float o = 0.f;
        for (int gg = 0; gg < kpp; ++gg) o += red[gg * hd + d];
        a.part_o[part * hd + d] = o;
    }
    if (tid == 0) {
        a.part_ml[2 * part] = m_sh;
        a.part_ml[2 * part + 1] = l_sh;
    }
    // The block that finishes last among the splits of this (request, head) merges them: a counter per
    // (request, head), zero before the launch and zero again after it.  The merge adds the splits in
    // ascending order whichever block runs it.
    const int s0 = t_lo / DEC_SPLIT, s1 = min(p / DEC_SPLIT, a.max_splits - 1);  // the splits that hold keys: all of them count
    __shared__ int last_sh;
    __syncthreads();  // every thread's partial results are written ...
    if (tid == 0) {
        __threadfence();  // ... and visible to the other blocks before this block counts itself done
        int* counter = a.counters + static_cast<size_t>(item) * a.nh + h;
        const int done = atomicAdd(counter, 1);
        last_sh = done == s1 - s0;
        if (last_sh) *counter = 0;
    }
    __syncthreads();
    if (!last_sh) return;
    __threadfence();
    const size_t base = (static_cast<size_t>(item) * a.nh + h) * a.max_splits;
    // weight of every split, exp(m_s - M), computed once (threads in parallel) into shared memory
    float* wsplit = red + kpp * hd;  // [s1 - s0 + 1]
    __shared__ float M_sh, inv_sh;
    const int ns = s1 - s0 + 1;
    float mloc = -INFINITY;
    for (int i = tid; i < ns; i += 128) mloc = fmaxf(mloc, __ldcg(a.part_ml + 2 * (base + s0 + i)));
    mloc = warp_max(mloc);
    if ((tid & 31) == 0) wred[tid >> 5] = mloc;
    __syncthreads();
    if (tid == 0) M_sh = fmaxf(fmaxf(wred[0], wred[1]), fmaxf(wred[2], wred[3]));
    __syncthreads();
    const float M = M_sh;
    for (int i = tid; i < ns; i += 128) wsplit[i] = expf(__ldcg(a.part_ml + 2 * (base + s0 + i)) - M);
    __syncthreads();
    if (tid == 0) {
        float L = 0.f;
        for (int i = 0; i < ns; ++i) L += __ldcg(a.part_ml + 2 * (base + s0 + i) + 1) * wsplit[i];
        inv_sh = 1.0f / L;
    }
    __syncthreads();
    const float inv = inv_sh;
    for (int d = tid; d < hd; d += 128) {
        float o = 0.f;
        for (int i = 0; i < ns; ++i) o += __ldcg(a.part_o + (base + s0 + i) * hd + d) * wsplit[i];
        static_cast<T*>(a.out)[(static_cast<size_t>(row) * a.nh + h) * hd + d] = from_f<T>(o * inv);
    }
}

// ---------------------------------------------------------------------------
// Streaming decode attention: the form for head sizes whose rows are 128, 256 or 512 bytes and pages
// that are a multiple of a chunk (8, 16 or 32 keys for those rows).
//
// Reading the cache is all there is to this work, so the kernel is built to keep loads in flight
// without pause.  The unit of work is a range of keys of one (request, head), done by ONE warp with
// no shared memory and no block barrier: LPK lanes share a key row (16 bytes each), 32 / LPK rows per
// load instruction, eight load instructions per chunk.  While the scores of a chunk are computed its
// V rows are already on their way, and the K rows of the next chunk are requested before the chunk's
// softmax update and weighted sum run.  Every lane group keeps its own running maximum, denominator
// and sum (online softmax, base 2); the groups are merged by shuffles at the end of the range.
//
// The grid is fixed (a few blocks per SM): every block first decides, from the batch's context
// lengths, how long a range is, so that the ranges fill the warps of the grid in as few rounds as
// possible (cost = rounds x (range length + a constant for the overhead of a range) + a term for the
// merge of the longest request); warps then take
// ranges in a fixed stride.  The warp that finishes last among the ranges of a (request, head) merges
// them in ascending order.  The range length depends on the batch, so a request's result can differ
// from batch to batch, in rounding only.
#define DS_WARPS 4        // warps of a block
#define DS_LOADS 8        // load instructions per chunk
#define DS_OVERHEAD 64    // fixed cost of a range, in keys
#define DS_MERGE 2        // cost of merging one more range, in keys

// a 16-byte load of cache data that is read once: no line of L1 is spent on it
__device__ __forceinline__ uint4 ld_once(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

struct true_tag { static constexpr bool value = true; };
struct false_tag { static constexpr bool value = false; };

template <typename T, int LPK, bool DEEP, bool PADDED>
__global__ void __launch_bounds__(32 * DS_WARPS, DEEP ? 2 : 4) attn_decode_stream_kernel(AttnArgs a, int n_items, int max_units,
                                                                              int cost_range, int cost_merge) {
    pdl_trigger();  // every block of this grid is resident from the start
    constexpr int VEC = 16 / sizeof(T);   // elements of a lane
    constexpr int KPL = 32 / LPK;         // key rows of a load instruction
    constexpr int CHUNK = DS_LOADS * KPL; // keys of a chunk
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hd = a.hd, P = a.page_tokens;

    // ---- how the batch is cut into ranges (the same result in every block) ----
    __shared__ KeyRanges kr;
    const int n_warps = gridDim.x * DS_WARPS;
    // The cut reads only the step's descriptors, which were on the device before the step's first kernel: under
    // programmatic dependent launch it is made while the kernel in front of this one (which writes q and the newest
    // keys and values) still runs; the wait for that kernel comes after it.
    plan_key_ranges(kr, a.items, a.seg_ctx, a.seg_q0, a.window, n_items, a.nh, max_units, n_warps, cost_range, cost_merge);
    bool waited = false;  // whether this warp has waited for the kernel in front (every path does before it leaves)
    int* const s_first = kr.first;
    int* const s_pref = kr.pref;
    int* const s_seg = kr.seg;
    int* const s_pos = kr.pos;
    int* const s_row = kr.row;
    const int s_len = kr.len;
    const int len = s_len;
    if (len == 0) {
        pdl_entry();
        return;
    }
    const int n_ranges = s_pref[n_items];
    const long long n_units = static_cast<long long>(n_ranges) * a.nh;

    const int grp = lane / LPK, sub = lane % LPK;  // which row of a load, which 16 bytes of the row
    const int d0 = sub * VEC;
    // A row of hd elements takes hd / VEC lanes.  PADDED: LPK is that number rounded up to a power of two (head
    // sizes like 96 or 48), and the lanes behind the row's end neither load nor store: they carry zeros through
    // the sums.  (A template parameter: at large batches the kernel is bound by instruction issue, and the
    // predicate on every load costs a tenth of its time.)
    const bool active = PADDED ? d0 < hd : true;
    const float qscale = a.scale * 1.4426950408889634f;  // scores in base 2
    const int pshift = (P & (P - 1)) == 0 ? __ffs(P) - 1 : -1;  // pages of 2^k tokens: shifts instead of divisions
    const size_t v_off = static_cast<size_t>(a.nkv) * P * hd;  // V row = K row + v_off
    const size_t v_units = v_off / VEC;
    const unsigned page_units = static_cast<unsigned>(2 * v_off / VEC), row_units = hd / VEC;

    for (long long u = static_cast<long long>(blockIdx.x) * DS_WARPS + warp; u < n_units; u += n_warps) {
        const int h = static_cast<int>(u % a.nh);
        const int r = static_cast<int>(u / a.nh);  // range index over the batch
        int item = 0;
        while (s_pref[item + 1] <= r) ++item;  // few items: a linear search
        const int split = r - s_pref[item];
        const int seg = s_seg[item], p = s_pos[item], row = s_row[item];
        const int t_lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
        const int k_begin = s_first[item] + split * len;           // a multiple of 32: chunks do not straddle pages
        const int k_end = min(p + 1, k_begin + len);               // exclusive
        const int kvh = h / (a.nh / a.nkv);
        const int* table = a.block_table + static_cast<size_t>(seg) * a.table_stride;
        const T* pool = static_cast<const T*>(a.pool) + static_cast<size_t>(kvh) * P * hd + d0;

        float m = -INFINITY, l = 0.f, acc[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = 0.f;

        // A chunk lies inside one page (chunks start at multiples of their size, which divides the page
        // size), so one block-table entry serves it; entries are fetched two chunks ahead.  Row starts are
        // kept in 16-byte units from the pool's base (the host refuses pools of 64 GiB or more).
        const uint4* pool4 = reinterpret_cast<const uint4*>(pool);
        auto page_of = [&](int k0) -> int {
            if (k0 >= k_end) return 0;
            return table[pshift >= 0 ? k0 >> pshift : k0 / P];
        };
        auto chunk_base = [&](int k0, int page) -> unsigned {
            const int po = pshift >= 0 ? k0 & (P - 1) : k0 % P;
            return static_cast<unsigned>(page) * page_units + static_cast<unsigned>(po + grp) * row_units;
        };
        auto live = [&](int k0, int g) -> bool {
            const int t = k0 + g * KPL + grp;
            return active && t >= t_lo && t < k_end;
        };
        auto t_live = [&](int k0, int g) -> bool {  // the key itself, whatever this lane's part of its row
            const int t = k0 + g * KPL + grp;
            return t >= t_lo && t < k_end;
        };
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
        float q[VEC];
        auto load_q = [&]() {
            float raw[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) raw[i] = 0.f;
            if (active) Vec<T>::load(static_cast<const T*>(a.q) + (static_cast<size_t>(row) * a.nh + h) * hd + d0, raw);
#pragma unroll
            for (int i = 0; i < VEC; ++i) q[i] = raw[i] * qscale;
        };
        if constexpr (DEEP) {
            // Few requests: a warp's time is the latency of its chain of chunks, not bandwidth.  K and V of TWO
            // chunks are kept in flight (twice the registers, half the blocks per SM): while one chunk is worked on
            // the next is already under way and the one after that is asked for as soon as registers are free.
            uint4 kb[2][DS_LOADS], vb[2][DS_LOADS];
            auto issue = [&](int slot, int k0) {
                const unsigned cb = chunk_base(k0, page_of(k0));
#pragma unroll
                for (int g = 0; g < DS_LOADS; ++g) {
                    const bool lv = live(k0, g);
                    kb[slot][g] = lv ? ld_once(pool4 + cb + g * KPL * row_units) : zero4;
                    vb[slot][g] = lv ? ld_once(pool4 + v_units + cb + g * KPL * row_units) : zero4;
                }
            };
            auto consume = [&](int slot, int k0) {
                float sc[DS_LOADS];
#pragma unroll
                for (int g = 0; g < DS_LOADS; ++g) {
                    float kf[VEC];
                    Vec<T>::unpack(kb[slot][g], kf);
                    float dot = 0.f;
#pragma unroll
                    for (int i = 0; i < VEC; ++i) dot = fmaf(q[i], kf[i], dot);
#pragma unroll
                    for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                    sc[g] = t_live(k0, g) ? dot : -INFINITY;
                }
                float mx = m;
#pragma unroll
                for (int g = 0; g < DS_LOADS; ++g) mx = fmaxf(mx, sc[g]);
                if (mx != -INFINITY) {
                    const float corr = exp2f(m - mx);  // 0 on the first live chunk
                    l *= corr;
#pragma unroll
                    for (int i = 0; i < VEC; ++i) acc[i] *= corr;
#pragma unroll
                    for (int g = 0; g < DS_LOADS; ++g) {
                        const float pr = exp2f(sc[g] - mx);  // 0 for a key that is not there
                        l += pr;
                        float vf[VEC];
                        Vec<T>::unpack(vb[slot][g], vf);
#pragma unroll
                        for (int i = 0; i < VEC; ++i) acc[i] = fmaf(pr, vf[i], acc[i]);
                    }
                    m = mx;
                }
            };
            // chunks that end before the request's own position hold old keys and values only: asked for before the
            // wait for the kernel in front, which writes q and the newest key and value
            const bool early0 = !waited && k_begin + CHUNK <= p, early1 = !waited && k_begin + 2 * CHUNK <= p;
            if (early0) issue(0, k_begin);
            if (early1) issue(1, k_begin + CHUNK);
            if (!waited) {
                pdl_entry();
                waited = true;
            }
            if (!early0) issue(0, k_begin);
            if (!early1) issue(1, k_begin + CHUNK);
            load_q();
            for (int k0 = k_begin; k0 < k_end; k0 += 2 * CHUNK) {
                consume(0, k0);
                issue(0, k0 + 2 * CHUNK);
                consume(1, k0 + CHUNK);
                issue(1, k0 + 3 * CHUNK);
            }
        } else {
            uint4 kreg[DS_LOADS], vreg[DS_LOADS];
            int page_next = page_of(k_begin + CHUNK), page_next2 = page_of(k_begin + 2 * CHUNK);
            unsigned base = chunk_base(k_begin, page_of(k_begin));
            // Keys before the request's own position were written by earlier steps: a first chunk that ends before that
            // position is asked for before the wait for the kernel in front, which writes q and the newest key and value.
            const bool early = !waited && k_begin + CHUNK <= p;
            if (early) {
#pragma unroll
                for (int g = 0; g < DS_LOADS; ++g)
                    kreg[g] = live(k_begin, g) ? ld_once(pool4 + base + g * KPL * row_units) : zero4;
            }
            if (!waited) {
                pdl_entry();
                waited = true;
            }
            if (!early) {
#pragma unroll
                for (int g = 0; g < DS_LOADS; ++g)
                    kreg[g] = live(k_begin, g) ? ld_once(pool4 + base + g * KPL * row_units) : zero4;
            }
            load_q();
            // One chunk: FAST when this chunk and the next lie wholly inside the range (the steady state), so
            // that no load and no score needs a check of its own.
            auto chunk = [&](int k0, auto fast_tag) {
                constexpr bool FAST = decltype(fast_tag)::value;
                // V of this chunk
#pragma unroll
                for (int g = 0; g < DS_LOADS; ++g)
                    vreg[g] = ((FAST && active) || live(k0, g)) ? ld_once(pool4 + v_units + base + g * KPL * row_units) : zero4;
                // scores of this chunk
                float sc[DS_LOADS];
#pragma unroll
                for (int g = 0; g < DS_LOADS; ++g) {
                    float kf[VEC];
                    Vec<T>::unpack(kreg[g], kf);
                    float dot = 0.f;
#pragma unroll
                    for (int i = 0; i < VEC; ++i) dot = fmaf(q[i], kf[i], dot);
#pragma unroll
                    for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                    sc[g] = (FAST || t_live(k0, g)) ? dot : -INFINITY;
                }
                // K of the next chunk, and the block-table entry of the chunk after the next two
                base = chunk_base(k0 + CHUNK, page_next);
                page_next = page_next2;
                page_next2 = page_of(k0 + 3 * CHUNK);
#pragma unroll
                for (int g = 0; g < DS_LOADS; ++g)
                    kreg[g] = ((FAST && active) || live(k0 + CHUNK, g)) ? ld_once(pool4 + base + g * KPL * row_units) : zero4;
                // running softmax of this lane group, then the weighted sum
                float mx = m;
#pragma unroll
                for (int g = 0; g < DS_LOADS; ++g) mx = fmaxf(mx, sc[g]);
                if (FAST || mx != -INFINITY) {
                    const float corr = exp2f(m - mx);  // 0 on the first live chunk
                    l *= corr;
#pragma unroll
                    for (int i = 0; i < VEC; ++i) acc[i] *= corr;
#pragma unroll
                    for (int g = 0; g < DS_LOADS; ++g) {
                        const float pr = exp2f(sc[g] - mx);  // 0 for a key that is not there
                        l += pr;
                        float vf[VEC];
                        Vec<T>::unpack(vreg[g], vf);
#pragma unroll
                        for (int i = 0; i < VEC; ++i) acc[i] = fmaf(pr, vf[i], acc[i]);
                    }
                    m = mx;
                }
            };
            for (int k0 = k_begin; k0 < k_end; k0 += CHUNK) {
                if (k0 >= t_lo && k0 + 2 * CHUNK <= k_end) {
                    chunk(k0, true_tag());
                } else {
                    chunk(k0, false_tag());
                }
            }
        }
        // merge the lane groups (ascending group order is kept by always putting the lower group first)
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) {
            const float m_o = __shfl_xor_sync(0xffffffffu, m, o);
            const float l_o = __shfl_xor_sync(0xffffffffu, l, o);
            float acc_o[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc_o[i] = __shfl_xor_sync(0xffffffffu, acc[i], o);
            const float mx = fmaxf(m, m_o);
            const float wa = mx == -INFINITY ? 0.f : exp2f(m - mx), wb = mx == -INFINITY ? 0.f : exp2f(m_o - mx);
            const bool low = (lane & o) == 0;
            // the same expression in both lanes of a pair: (lower group) + (upper group)
            l = low ? l * wa + l_o * wb : l_o * wb + l * wa;
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = low ? acc[i] * wa + acc_o[i] * wb : acc_o[i] * wb + acc[i] * wa;
            m = mx;
        }
        if (grp == 0 && active) {
            float* po = a.part_o + static_cast<size_t>(u) * hd + d0;
#pragma unroll
            for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4*>(po + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
            if (sub == 0) {
                a.part_ml[2 * u] = m;
                a.part_ml[2 * u + 1] = l;
            }
        }
        // the warp that finishes the last range of this (request, head) merges them
        __syncwarp();
        int last = 0;
        const int n_splits = s_pref[item + 1] - s_pref[item];
        if (lane == 0) {
            __threadfence();
            int* counter = a.counters + static_cast<size_t>(item) * a.nh + h;
            last = atomicAdd(counter, 1) == n_splits - 1;
            if (last) *counter = 0;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) continue;
        __threadfence();
        const long long u0 = static_cast<long long>(s_pref[item]) * a.nh + h;  // range s of this head: u0 + s * nh
        float M = -INFINITY;
        for (int sidx = lane; sidx < n_splits; sidx += 32) M = fmaxf(M, __ldcg(a.part_ml + 2 * (u0 + static_cast<long long>(sidx) * a.nh)));
        M = warp_max(M);
        // one more pass over the ranges, in ascending order: the denominator (every lane forms the same one)
        // and this lane's four dimensions of the sum
        for (int d = lane * 4; d < hd; d += 128) {
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            float L = 0.f;
#pragma unroll 16
            for (int sidx = 0; sidx < n_splits; ++sidx) {
                const long long us = u0 + static_cast<long long>(sidx) * a.nh;
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(a.part_ml + 2 * us));
                const float w = exp2f(ml.x - M);
                const float4 v = __ldcg(reinterpret_cast<const float4*>(a.part_o + us * hd + d));
                L = fmaf(ml.y, w, L);
                o.x = fmaf(v.x, w, o.x);
                o.y = fmaf(v.y, w, o.y);
                o.z = fmaf(v.z, w, o.z);
                o.w = fmaf(v.w, w, o.w);
            }
            const float inv = 1.0f / L;
            T* dst = static_cast<T*>(a.out) + (static_cast<size_t>(row) * a.nh + h) * hd + d;
            dst[0] = from_f<T>(o.x * inv);
            dst[1] = from_f<T>(o.y * inv);
            dst[2] = from_f<T>(o.z * inv);
            dst[3] = from_f<T>(o.w * inv);
        }
    }
    if (!waited) pdl_entry();  // a warp without work: the grid must not finish before the kernel in front has
}

// The two constants of the streaming kernel's cost model (in keys); a switch for measurements.
static int g_ds_cost_range = DS_OVERHEAD, g_ds_cost_merge = DS_MERGE;
// Up to this many (request, head) pairs, or pairs x splits of 128 keys of the longest context, the variant with two
// chunks in flight runs (16 heads, 4,000 cached tokens: 20.4 -> 17.4 us at one request, 32.0 -> 30.0 at four, equal at
// eight, 90.7 -> 95.9 at sixteen; 500 cached tokens at eight requests: 21.5 -> 17.2 us); g_ds_deep forces it on (1)
// or off (0) for measurements (-1: by these bounds).
#define DS_DEEP_PAIRS 64
#define DS_DEEP_SPLITS 2048
static int g_ds_deep = -1;
extern "C" void locus_attn_decode_set_deep(int deep) { g_ds_deep = deep; }
extern "C" void locus_attn_decode_set_cost(int range_overhead, int merge_per_range) {
    g_ds_cost_range = range_overhead;
    g_ds_cost_merge = merge_per_range;
}

static int check_common(int nh, int nkv, int hd, int page_tokens, int window) {
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0) return LOCUS_ERR_UNSUPPORTED;
    if (hd <= 0 || hd % 16 != 0 || hd > 256) return LOCUS_ERR_UNSUPPORTED;
    if (page_tokens <= 0 || window < 0) return LOCUS_ERR_UNSUPPORTED;
    return 0;
}

static AttnArgs make_args(const void* q, const void* pool, void* out, const int* seg_q0,
                          const int* seg_qn, const int* seg_ctx, const int* block_table,
                          int table_stride, const int* items, int nh, int nkv, int hd,
                          int page_tokens, int window, float scale) {
    AttnArgs a;
    a.q = q; a.pool = pool; a.out = out; a.seg_q0 = seg_q0; a.seg_qn = seg_qn; a.seg_ctx = seg_ctx;
    a.block_table = block_table; a.table_stride = table_stride; a.items = items; a.nh = nh;
    a.nkv = nkv; a.hd = hd; a.page_tokens = page_tokens; a.window = window; a.scale = scale;
    a.part_o = nullptr; a.part_ml = nullptr; a.counters = nullptr; a.max_splits = 0;
    return a;
}

extern "C" int locus_attn_chunk(const void* q, int dt, const void* pool, void* out,
                                const int* seg_q0, const int* seg_qn, const int* seg_ctx,
                                const int* block_table, int table_stride, const int* items,
                                int n_items, int nh, int nkv, int hd, int page_tokens, int window,
                                float scale, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (int e = check_common(nh, nkv, hd, page_tokens, window)) return e;
    if (n_items > 65535) return LOCUS_ERR_UNSUPPORTED;
    AttnArgs a = make_args(q, pool, out, seg_q0, seg_qn, seg_ctx, block_table, table_stride, items,
                           nh, nkv, hd, page_tokens, window, scale);
    const size_t smem = sizeof(float) * (CHUNK_BQ * hd + CHUNK_TK * (hd + 1) + CHUNK_TK * hd +
                                         CHUNK_BQ * (CHUNK_TK + 1) + 3 * CHUNK_BQ);
    dim3 grid(nh, n_items);
    if (dt == LOCUS_DT_F32) {
        cudaFuncSetAttribute(attn_chunk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attn_chunk_kernel<float><<<grid, 128, smem, stream>>>(a);
    } else if (dt == LOCUS_DT_BF16) {
        cudaFuncSetAttribute(attn_chunk_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attn_chunk_kernel<bf16><<<grid, 128, smem, stream>>>(a);
    } else {
        return LOCUS_ERR_UNSUPPORTED;
    }
    return locus_launch_status();
}

// Scratch: part_o holds max_units partial results of hd floats, part_ml two floats for each, counters
// n_items * nh ints that are zero before the call (the call leaves them zero).  The streaming kernel
// cuts the batch into at most max_units ranges (at least n_items * nh; a few thousand more let short
// batches fill the GPU); the kernel for other head sizes needs n_items * nh * max_splits units, where
// max_splits must cover the longest context: max_splits >= (longest position) / DEC_SPLIT + 1.
extern "C" int locus_attn_decode(const void* q, int dt, const void* pool, void* out,
                                 const int* seg_q0, const int* seg_qn, const int* seg_ctx,
                                 const int* block_table, int table_stride, const int* items,
                                 int n_items, int nh, int nkv, int hd, int page_tokens, int window,
                                 float scale, float* part_o, float* part_ml, int* counters, int max_splits,
                                 long long max_units, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (int e = check_common(nh, nkv, hd, page_tokens, window)) return e;
    if (nh > 65535 || max_splits <= 0 || max_splits > 65535) return LOCUS_ERR_UNSUPPORTED;
    AttnArgs a = make_args(q, pool, out, seg_q0, seg_qn, seg_ctx, block_table, table_stride, items,
                           nh, nkv, hd, page_tokens, window, scale);
    a.part_o = part_o; a.part_ml = part_ml; a.counters = counters; a.max_splits = max_splits;
    if (counters == nullptr) return LOCUS_ERR_UNSUPPORTED;
    if (max_units < static_cast<long long>(n_items) * nh) return LOCUS_ERR_UNSUPPORTED;
    // rows of 64 to 512 bytes: the streaming kernel on a fixed grid, 8, 16 or 32 lanes to a row (the row's 16-byte
    // pieces rounded up to a power of two: a head of 96 bfloat16 elements takes 12 of 16 lanes)
    const int pieces = hd * (dt == LOCUS_DT_F32 ? 4 : 2) / 16;
    const int lpk = pieces < 4 ? 0 : pieces <= 8 ? 8 : pieces <= 16 ? 16 : pieces <= 32 ? 32 : 0;
    const int chunk_keys = lpk > 0 ? DS_LOADS * 32 / lpk : 1;
    if ((dt == LOCUS_DT_F32 || dt == LOCUS_DT_BF16) && lpk > 0 && n_items <= DS_MAX_ITEMS &&
        page_tokens % chunk_keys == 0) {
        static int n_sm = 0;
        if (n_sm == 0) {
            int dev = 0;
            if (cudaGetDevice(&dev) != cudaSuccess ||
                cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) {
                n_sm = 0;
                return static_cast<int>(cudaGetLastError());
            }
        }
        // few (request, head) pairs: the variant with two chunks in flight per warp on half the blocks (see the kernel)
        const long long pairs = static_cast<long long>(n_items) * nh;
        const bool deep = g_ds_deep >= 0 ? g_ds_deep != 0 : (pairs <= DS_DEEP_PAIRS || pairs * max_splits <= DS_DEEP_SPLITS);
        const dim3 sgrid(n_sm * (deep ? 2 : 4));
        const int units = static_cast<int>(max_units < (1 << 30) ? max_units : (1 << 30));
#define DS_LAUNCH(TT, L)                                                                                               \
        do {                                                                                                           \
            if (deep) locus_launch(attn_decode_stream_kernel<TT, L, true, true>, sgrid, 32 * DS_WARPS, 0, stream, a, n_items, units, g_ds_cost_range, g_ds_cost_merge); \
            else if (pieces != L) locus_launch(attn_decode_stream_kernel<TT, L, false, true>, sgrid, 32 * DS_WARPS, 0, stream, a, n_items, units, g_ds_cost_range, g_ds_cost_merge); \
            else locus_launch(attn_decode_stream_kernel<TT, L, false, false>, sgrid, 32 * DS_WARPS, 0, stream, a, n_items, units, g_ds_cost_range, g_ds_cost_merge); \
        } while (0)
        if (dt == LOCUS_DT_F32) {
            if (lpk == 8) DS_LAUNCH(float, 8);
            else if (lpk == 16) DS_LAUNCH(float, 16);
            else DS_LAUNCH(float, 32);
        } else {
            if (lpk == 8) DS_LAUNCH(bf16, 8);
            else if (lpk == 16) DS_LAUNCH(bf16, 16);
            else DS_LAUNCH(bf16, 32);
        }
#undef DS_LAUNCH
        return locus_launch_status();
    }
    if (max_units < static_cast<long long>(n_items) * nh * max_splits) return LOCUS_ERR_UNSUPPORTED;
    dim3 grid(n_items, nh, max_splits);
    if (dt == LOCUS_DT_F32) {
        const int kpp = 128 / (hd / 4);
        const size_t smem = sizeof(float) * (hd + DEC_SPLIT + kpp * hd + max_splits);
        if (smem > 48 * 1024) return LOCUS_ERR_UNSUPPORTED;
        locus_launch(attn_decode_split_kernel<float>, grid, 128, smem, stream, a);
    } else if (dt == LOCUS_DT_BF16) {
        const int kpp = 128 / (hd / 8);
        const size_t smem = sizeof(float) * (hd + DEC_SPLIT + kpp * hd + max_splits);
        if (smem > 48 * 1024) return LOCUS_ERR_UNSUPPORTED;
        locus_launch(attn_decode_split_kernel<bf16>, grid, 128, smem, stream, a);
    } else {
        return LOCUS_ERR_UNSUPPORTED;
    }
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Decode attention with the scratch inside the library (see attention_static.h for who this
// is for, what it costs and the rules of use).  The kernels are the ones above; only the
// home of the partial results differs.
#include "attention_static.h"

// The scratch itself.  On the host this name is only a handle for cudaGetSymbolAddress; the
// device address it stands for is looked up once per device below.
static __device__ __align__(256) float g_attn_static_scratch[LOCUS_ATTN_STATIC_SCRATCH_FLOATS];
// One counter per (request, head): zero when the library is loaded, and every call leaves them zero.
static __device__ int g_attn_static_counters[LOCUS_ATTN_STATIC_COUNTERS];

#define LOCUS_MAX_DEVICES 64
static float* g_attn_static_ptr[LOCUS_MAX_DEVICES];  // device address of the array, per device
static int* g_attn_static_cnt_ptr[LOCUS_MAX_DEVICES];

extern "C" int locus_attn_decode_static(const void* q, int dt, const void* pool, void* out,
                                        const int* seg_q0, const int* seg_qn, const int* seg_ctx,
                                        const int* block_table, int table_stride, const int* items,
                                        int n_items, int nh, int nkv, int hd, int page_tokens,
                                        int window, float scale, int max_splits, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (int e = check_common(nh, nkv, hd, page_tokens, window)) return e;
    if (max_splits <= 0) return LOCUS_ERR_UNSUPPORTED;
    // part_o: n_items * nh * max_splits * hd floats, then part_ml: 2 floats per (item, head, split)
    const long long units = static_cast<long long>(n_items) * nh * max_splits;
    const long long need = units * (hd + 2);
    if (need > LOCUS_ATTN_STATIC_SCRATCH_FLOATS) return LOCUS_ERR_SCRATCH_TOO_SMALL;
    const long long cap = LOCUS_ATTN_STATIC_SCRATCH_FLOATS / (hd + 2);  // partial results that the array holds
    if (static_cast<long long>(n_items) * nh > LOCUS_ATTN_STATIC_COUNTERS) return LOCUS_ERR_SCRATCH_TOO_SMALL;
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return static_cast<int>(err);
    if (dev < 0 || dev >= LOCUS_MAX_DEVICES) return LOCUS_ERR_UNSUPPORTED;
    if (g_attn_static_ptr[dev] == nullptr) {
        // first call on this device (it is the current one): resolve the array's device address
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_attn_static_scratch);
        if (err != cudaSuccess) return static_cast<int>(err);
        if (p == nullptr) return LOCUS_ERR_UNSUPPORTED;
        void* c = nullptr;
        err = cudaGetSymbolAddress(&c, g_attn_static_counters);
        if (err != cudaSuccess) return static_cast<int>(err);
        if (c == nullptr) return LOCUS_ERR_UNSUPPORTED;
        g_attn_static_cnt_ptr[dev] = static_cast<int*>(c);
        g_attn_static_ptr[dev] = static_cast<float*>(p);
    }
    float* part_o = g_attn_static_ptr[dev];
    float* part_ml = part_o + cap * hd;  // hd is a multiple of 16 floats: stays aligned
    // Nothing to clear: the kernel writes the sums, m and l of every split that it later reads,
    // and the counters are zero between calls.
    return locus_attn_decode(q, dt, pool, out, seg_q0, seg_qn, seg_ctx, block_table, table_stride,
                             items, n_items, nh, nkv, hd, page_tokens, window, scale, part_o, part_ml,
                             g_attn_static_cnt_ptr[dev], max_splits, cap, stream);
}
