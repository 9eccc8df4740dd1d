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
    int max_splits;
};

#define CHUNK_BQ 16
#define CHUNK_TK 32
#define DEC_SPLIT 128

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

    const int seg = a.items[2 * blockIdx.x], qoff = a.items[2 * blockIdx.x + 1];
    const int h = blockIdx.y;
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
};
template <>
struct Vec<bf16> {
    static constexpr int N = 8;
    __device__ static void load(const bf16* p, float* o) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            o[2 * i] = f.x;
            o[2 * i + 1] = f.y;
        }
    }
};

// grid (n_items, nh, max_splits); split s covers absolute key positions
// [s * DEC_SPLIT, (s + 1) * DEC_SPLIT).  Writes unnormalised partial sums with their
// running maximum m and denominator l; a split outside the key range writes l = 0.
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
    if (k0 > k1) {
        if (tid == 0) {
            a.part_ml[2 * part] = -INFINITY;
            a.part_ml[2 * part + 1] = 0.f;
        }
        return;
    }
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
}

// grid (n_items, nh); merges the splits of one (request, head) in ascending order.
template <typename T>
__global__ void attn_decode_merge_kernel(AttnArgs a) {
    pdl_entry();
    const int item = blockIdx.x, h = blockIdx.y;
    const int seg = a.items[item];
    const int p = a.seg_ctx[seg];
    const int row = a.seg_q0[seg];
    const int t_lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
    const int s0 = t_lo / DEC_SPLIT, s1 = p / DEC_SPLIT;
    const size_t base = (static_cast<size_t>(item) * a.nh + h) * a.max_splits;
    // weight of every split, exp(m_s - M), computed once (threads in parallel) into shared memory;
    // the sums over splits stay in ascending order
    extern __shared__ float wsplit[];  // [s1 - s0 + 1]
    __shared__ float M_sh, inv_sh;
    const int ns = s1 - s0 + 1;
    float mloc = -INFINITY;
    for (int i = threadIdx.x; i < ns; i += blockDim.x) mloc = fmaxf(mloc, a.part_ml[2 * (base + s0 + i)]);
    mloc = warp_max(mloc);
    __shared__ float wm[8];
    if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = mloc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float M = wm[0];
        for (int w = 1; w < static_cast<int>((blockDim.x + 31) >> 5); ++w) M = fmaxf(M, wm[w]);
        M_sh = M;
    }
    __syncthreads();
    const float M = M_sh;
    for (int i = threadIdx.x; i < ns; i += blockDim.x) wsplit[i] = expf(a.part_ml[2 * (base + s0 + i)] - M);
    __syncthreads();
    if (threadIdx.x == 0) {
        float L = 0.f;
        for (int i = 0; i < ns; ++i) L += a.part_ml[2 * (base + s0 + i) + 1] * wsplit[i];
        inv_sh = 1.0f / L;
    }
    __syncthreads();
    const float inv = inv_sh;
    for (int d = threadIdx.x; d < a.hd; d += blockDim.x) {
        float o = 0.f;
        for (int i = 0; i < ns; ++i) o += a.part_o[(base + s0 + i) * a.hd + d] * wsplit[i];
        static_cast<T*>(a.out)[(static_cast<size_t>(row) * a.nh + h) * a.hd + d] = from_f<T>(o * inv);
    }
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
    a.part_o = nullptr; a.part_ml = nullptr; a.max_splits = 0;
    return a;
}

extern "C" int locus_attn_chunk(const void* q, int dt, const void* pool, void* out,
                                const int* seg_q0, const int* seg_qn, const int* seg_ctx,
                                const int* block_table, int table_stride, const int* items,
                                int n_items, int nh, int nkv, int hd, int page_tokens, int window,
                                float scale, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (int e = check_common(nh, nkv, hd, page_tokens, window)) return e;
    if (nh > 65535) return LOCUS_ERR_UNSUPPORTED;
    AttnArgs a = make_args(q, pool, out, seg_q0, seg_qn, seg_ctx, block_table, table_stride, items,
                           nh, nkv, hd, page_tokens, window, scale);
    const size_t smem = sizeof(float) * (CHUNK_BQ * hd + CHUNK_TK * (hd + 1) + CHUNK_TK * hd +
                                         CHUNK_BQ * (CHUNK_TK + 1) + 3 * CHUNK_BQ);
    dim3 grid(n_items, nh);
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

// Scratch: part_o needs n_items * nh * max_splits * hd floats, part_ml twice
// n_items * nh * max_splits.  max_splits must cover the longest context:
// max_splits >= (longest position) / DEC_SPLIT + 1.
extern "C" int locus_attn_decode(const void* q, int dt, const void* pool, void* out,
                                 const int* seg_q0, const int* seg_qn, const int* seg_ctx,
                                 const int* block_table, int table_stride, const int* items,
                                 int n_items, int nh, int nkv, int hd, int page_tokens, int window,
                                 float scale, float* part_o, float* part_ml, int max_splits,
                                 cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (int e = check_common(nh, nkv, hd, page_tokens, window)) return e;
    if (nh > 65535 || max_splits <= 0 || max_splits > 65535) return LOCUS_ERR_UNSUPPORTED;
    AttnArgs a = make_args(q, pool, out, seg_q0, seg_qn, seg_ctx, block_table, table_stride, items,
                           nh, nkv, hd, page_tokens, window, scale);
    a.part_o = part_o; a.part_ml = part_ml; a.max_splits = max_splits;
    dim3 grid(n_items, nh, max_splits);
    dim3 mgrid(n_items, nh);
    const int mthreads = hd <= 32 ? 32 : (hd <= 64 ? 64 : 128);
    if (dt == LOCUS_DT_F32) {
        const int kpp = 128 / (hd / 4);
        const size_t smem = sizeof(float) * (hd + DEC_SPLIT + kpp * hd);
        locus_launch(attn_decode_split_kernel<float>, grid, 128, smem, stream, a);
        locus_launch(attn_decode_merge_kernel<float>, mgrid, mthreads, sizeof(float) * max_splits, stream, a);
    } else if (dt == LOCUS_DT_BF16) {
        const int kpp = 128 / (hd / 8);
        const size_t smem = sizeof(float) * (hd + DEC_SPLIT + kpp * hd);
        locus_launch(attn_decode_split_kernel<bf16>, grid, 128, smem, stream, a);
        locus_launch(attn_decode_merge_kernel<bf16>, mgrid, mthreads, sizeof(float) * max_splits, stream, a);
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

#define LOCUS_MAX_DEVICES 64
static float* g_attn_static_ptr[LOCUS_MAX_DEVICES];  // device address of the array, per device

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
        g_attn_static_ptr[dev] = static_cast<float*>(p);
    }
    float* part_o = g_attn_static_ptr[dev];
    float* part_ml = part_o + units * hd;  // units * hd is a multiple of 16 floats: stays aligned
    // Nothing to clear: the split kernel writes m and l for every (item, head, split) of the
    // grid and the sums of every split the merge kernel reads.
    return locus_attn_decode(q, dt, pool, out, seg_q0, seg_qn, seg_ctx, block_table, table_stride,
                             items, n_items, nh, nkv, hd, page_tokens, window, scale, part_o, part_ml,
                             max_splits, stream);
}
