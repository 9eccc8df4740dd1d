// Matrix products for a handful of rows (decode steps): out[m, n] = sum_k x[m, k] W[n, k],
// at most 8 rows of x per tile.  The work is bound by reading W once from HBM, so the layout
// is that of a matrix-vector product: one warp per output column n streams the weight row
// W[n, :] with 16-byte loads (four in flight per lane), multiplies it with up to 8 rows of x
// (read through L1; they are shared by every warp) in float32, reduces across the warp and
// runs the epilogue.  Same epilogues and the same gathered / grouped forms as the other
// products: bias, SwiGLU of two weight rows, per-row scale, store or add into float32.
//
// The order of the sum for an element depends on K only (8-element chunks per lane, lanes
// combined by a fixed shuffle tree), not on the number of rows or on the other rows.
#include "common.cuh"

#define GV_ROWS 8    // rows of x per tile
#define GV_WARPS 8   // output columns per block

struct GemvArgs {
    const void* x;
    const void* w;
    const void* w2;
    const void* bias;
    int bias_dt;
    void* out;
    int out_dt;
    int accumulate;
    const float* row_scale;
    const int* scale_rows;
    const int* x_rows;
    int x_row_div;
    int M, N, K;
    long long ldx, ldo;
    const int* tile_expert;
    const int* tile_row0;
    const int* tile_rows;
    const int* n_tiles;
    long long w_expert_stride;
};

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

// streaming load of weights: read once, do not keep in L1
template <typename T>
__device__ __forceinline__ void load8_stream(const T* p, float* o);
template <>
__device__ __forceinline__ void load8_stream<float>(const float* p, float* o) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p + 4));
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <>
__device__ __forceinline__ void load8_stream<bf16>(const bf16* p, float* o) {
    const uint4 v = __ldcs(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        o[2 * i] = f.x;
        o[2 * i + 1] = f.y;
    }
}

template <typename TX, typename TW, bool DUAL, int ROWS>
__device__ __forceinline__ void gemv_body(const GemvArgs& a, const TW* __restrict__ w, const TW* __restrict__ w2,
                                          const TX* const* xr, int rows, int lane, float* acc, float* acc2) {
    const int K = a.K;
    // 8-element chunks, four weight loads in flight per lane
    int j = lane * 8;
    for (; j + 3 * 256 < K; j += 4 * 256) {
        float wv[4][8], uv[DUAL ? 4 : 1][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            load8_stream<TW>(w + j + u * 256, wv[u]);
            if (DUAL) load8_stream<TW>(w2 + j + u * 256, uv[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
            for (int t = 0; t < ROWS; ++t) {
                if (t < rows) {
                    float hv[8];
                    load8<TX>(xr[t] + j + u * 256, hv);
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        acc[t] = fmaf(hv[v], wv[u][v], acc[t]);
                        if (DUAL) acc2[t] = fmaf(hv[v], uv[u][v], acc2[t]);
                    }
                }
            }
        }
    }
    for (; j < K; j += 256) {
        float wv[8], uv[8];
        load8_stream<TW>(w + j, wv);
        if (DUAL) load8_stream<TW>(w2 + j, uv);
#pragma unroll
        for (int t = 0; t < ROWS; ++t) {
            if (t < rows) {
                float hv[8];
                load8<TX>(xr[t] + j, hv);
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    acc[t] = fmaf(hv[v], wv[v], acc[t]);
                    if (DUAL) acc2[t] = fmaf(hv[v], uv[v], acc2[t]);
                }
            }
        }
    }
}

template <typename TX, typename TW, bool DUAL>
__global__ void __launch_bounds__(32 * GV_WARPS) rowstream_kernel(GemvArgs a) {
    int row0, rows;
    const TW* W = static_cast<const TW*>(a.w);
    const TW* W2 = static_cast<const TW*>(a.w2);
    if (a.tile_expert != nullptr) {
        const int tile = blockIdx.y;
        if (tile >= *a.n_tiles) return;
        const long long e = a.tile_expert[tile];
        row0 = a.tile_row0[tile];
        rows = a.tile_rows[tile];
        W += e * a.w_expert_stride;
        if (DUAL) W2 += e * a.w_expert_stride;
    } else {
        row0 = blockIdx.y * GV_ROWS;
        rows = min(GV_ROWS, a.M - row0);
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int n = blockIdx.x * GV_WARPS + wid;
    if (n >= a.N) return;
    const TX* xr[GV_ROWS];
#pragma unroll
    for (int t = 0; t < GV_ROWS; ++t) {
        const int r = row0 + (t < rows ? t : 0);
        const long long xrow = a.x_rows ? a.x_rows[r] / a.x_row_div : r;
        xr[t] = static_cast<const TX*>(a.x) + xrow * a.ldx;
    }
    float acc[GV_ROWS], acc2[GV_ROWS];
#pragma unroll
    for (int t = 0; t < GV_ROWS; ++t) acc[t] = acc2[t] = 0.f;
    const TW* w = W + static_cast<long long>(n) * a.K;
    const TW* w2 = DUAL ? W2 + static_cast<long long>(n) * a.K : nullptr;
    // fewer unrolled rows when the tile is small keeps registers and instructions down
    if (rows == 1) gemv_body<TX, TW, DUAL, 1>(a, w, w2, xr, rows, lane, acc, acc2);
    else if (rows <= 2) gemv_body<TX, TW, DUAL, 2>(a, w, w2, xr, rows, lane, acc, acc2);
    else if (rows <= 4) gemv_body<TX, TW, DUAL, 4>(a, w, w2, xr, rows, lane, acc, acc2);
    else gemv_body<TX, TW, DUAL, GV_ROWS>(a, w, w2, xr, rows, lane, acc, acc2);
#pragma unroll
    for (int t = 0; t < GV_ROWS; ++t) {
        if (t >= rows) break;
        float v = warp_sum(acc[t]);
        float u = DUAL ? warp_sum(acc2[t]) : 0.f;
        if (lane != 0) continue;
        if (DUAL) v = v / (1.0f + expf(-v)) * u;
        if (a.bias) v += ld_dyn(a.bias, a.bias_dt, n);
        const int r = row0 + t;
        if (a.row_scale) v *= a.row_scale[a.scale_rows ? a.scale_rows[r] : r];
        const size_t o = static_cast<size_t>(r) * a.ldo + n;
        if (a.accumulate) {
            static_cast<float*>(a.out)[o] += v;
        } else {
            st_dyn(a.out, a.out_dt, o, v);
        }
    }
}

template <typename TX, typename TW>
static int launch(const GemvArgs& a, int tiles, bool dual, cudaStream_t stream) {
    dim3 grid(ceil_div(a.N, GV_WARPS), tiles);
    if (grid.x == 0 || grid.y == 0) return 0;
    if (grid.y > 65535) return LOCUS_ERR_UNSUPPORTED;
    if (dual) {
        rowstream_kernel<TX, TW, true><<<grid, 32 * GV_WARPS, 0, stream>>>(a);
    } else {
        rowstream_kernel<TX, TW, false><<<grid, 32 * GV_WARPS, 0, stream>>>(a);
    }
    return locus_launch_status();
}

// Same arguments as locus_gemm_simt.  Needs K a multiple of 8, rows of x and W that start on
// 16-byte (bfloat16) / 32-byte (float32) boundaries, and, for a grouped product, tiles of at
// most 8 rows.
extern "C" int locus_gemv(const void* x, int x_dt, const void* w, const void* w2, int w_dt, const void* bias,
                          int bias_dt, void* out, int out_dt, int accumulate, const float* row_scale,
                          const int* scale_rows, const int* x_rows, int x_row_div, int M, int N, int K,
                          long long ldx, long long ldo, const int* tile_expert, const int* tile_row0,
                          const int* tile_rows, const int* n_tiles, int max_tiles, long long w_expert_stride,
                          cudaStream_t stream) {
    if (N <= 0 || K <= 0 || K % 8 != 0 || ldx % 8 != 0) return LOCUS_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(w2)) & 31)
        return LOCUS_ERR_UNSUPPORTED;
    if (accumulate && out_dt != LOCUS_DT_F32) return LOCUS_ERR_UNSUPPORTED;
    if (x_rows != nullptr && x_row_div <= 0) return LOCUS_ERR_UNSUPPORTED;
    GemvArgs a;
    a.x = x; a.w = w; a.w2 = w2; a.bias = bias; a.bias_dt = bias_dt; a.out = out; a.out_dt = out_dt;
    a.accumulate = accumulate; a.row_scale = row_scale; a.scale_rows = scale_rows; a.x_rows = x_rows;
    a.x_row_div = x_row_div; a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldo = ldo;
    a.tile_expert = tile_expert; a.tile_row0 = tile_row0; a.tile_rows = tile_rows; a.n_tiles = n_tiles;
    a.w_expert_stride = w_expert_stride;
    const int tiles = tile_expert ? max_tiles : ceil_div(M, GV_ROWS);
    const bool dual = w2 != nullptr;
    if (x_dt == LOCUS_DT_F32 && w_dt == LOCUS_DT_F32) return launch<float, float>(a, tiles, dual, stream);
    if (x_dt == LOCUS_DT_BF16 && w_dt == LOCUS_DT_BF16) return launch<bf16, bf16>(a, tiles, dual, stream);
    if (x_dt == LOCUS_DT_BF16 && w_dt == LOCUS_DT_F32) return launch<bf16, float>(a, tiles, dual, stream);
    if (x_dt == LOCUS_DT_F32 && w_dt == LOCUS_DT_BF16) return launch<float, bf16>(a, tiles, dual, stream);
    return LOCUS_ERR_UNSUPPORTED;
}
