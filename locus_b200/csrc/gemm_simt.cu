// Matrix products on CUDA cores with float32 FMA: out = x . W^T with fused epilogues.
//
// This is the true-32-bit path of every linear layer (no tensor cores, no TF32) and the
// general fallback of the bfloat16 path for shapes the tensor-core kernels refuse.  Each
// output element is accumulated by one thread over k = 0..K-1 in ascending order, so its
// value does not depend on M, on the other rows of the batch or on the tile it falls in.
//
// One kernel covers:
//   * plain      out[m, n]  = sum_k x[m, k] W[n, k]          (+ bias[n]) (* row_scale[m])
//   * SwiGLU     out[m, n]  = silu(x . Wg[n]) * (x . Wu[n])   (two accumulators)
//   * gathered   x row of logical row m is x_rows[m] / x_row_div
//   * grouped    logical rows are sorted by expert; a device-built tile list names, for
//                each 64-row tile, its expert, first row and row count; W of expert e
//                starts at W + e * w_expert_stride
//   * epilogue   store as float32 or bfloat16, or add into a float32 tensor (residual)
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

struct GemmArgs {
    const void* x;
    const void* w;
    const void* w2;          // up-projection for SwiGLU, else null
    const void* bias;        // [N] or null
    int bias_dt;
    void* out;
    int out_dt;
    int accumulate;          // out (float32) += result
    const float* row_scale;  // or null: row m is scaled by row_scale[scale_rows ? scale_rows[m] : m]
    const int* scale_rows;
    const int* x_rows;       // [M] or null
    int x_row_div;
    int M, N, K;
    long long ldx, ldo;
    // grouped
    const int* tile_expert;  // null when not grouped
    const int* tile_row0;
    const int* tile_rows;
    const int* n_tiles;
    long long w_expert_stride;
};

template <typename TX, typename TW, bool SWIGLU>
__global__ void __launch_bounds__(256) gemm_simt_kernel(GemmArgs a) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    __shared__ float ws2[SWIGLU ? BK : 1][BN + 4];

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
        if (SWIGLU) W2 += e * a.w_expert_stride;
    } else {
        row0 = blockIdx.y * BM;
        rows = min(BM, a.M - row0);
    }
    const int col0 = blockIdx.x * BN;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    const TX* X = static_cast<const TX*>(a.x);

    // loader mapping: thread loads elements (lr, lk..lk+3) of the x tile and of the W tile
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    long long xrow = -1;
    if (lr < rows) {
        const int r = row0 + lr;
        xrow = a.x_rows ? a.x_rows[r] / a.x_row_div : r;
    }
    const int wrow = col0 + lr;

    float acc[4][4], acc2[SWIGLU ? 4 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.f;
            if (SWIGLU) acc2[i][j] = 0.f;
        }

    for (int k0 = 0; k0 < a.K; k0 += BK) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int k = k0 + lk + u;
            float xv = 0.f, wv = 0.f, wv2 = 0.f;
            if (k < a.K) {
                if (xrow >= 0) xv = to_f(X[xrow * a.ldx + k]);
                if (wrow < a.N) {
                    wv = to_f(W[static_cast<long long>(wrow) * a.K + k]);
                    if (SWIGLU) wv2 = to_f(W2[static_cast<long long>(wrow) * a.K + k]);
                }
            }
            xs[lk + u][lr] = xv;
            ws[lk + u][lr] = wv;
            if (SWIGLU) ws2[lk + u][lr] = wv2;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[4], bv[4], bv2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                bv[j] = ws[kk][tx * 4 + j];
                if (SWIGLU) bv2[j] = ws2[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
                    if (SWIGLU) acc2[i][j] = fmaf(av[i], bv2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int lrow = ty * 4 + i;
        if (lrow >= rows) continue;
        const int r = row0 + lrow;
        const float rs = a.row_scale ? a.row_scale[a.scale_rows ? a.scale_rows[r] : r] : 1.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = col0 + tx * 4 + j;
            if (n >= a.N) continue;
            float v = acc[i][j];
            if (SWIGLU) {
                const float g = v;
                v = g / (1.0f + expf(-g)) * acc2[i][j];
            }
            if (a.bias) v += ld_dyn(a.bias, a.bias_dt, n);
            if (a.row_scale) v *= rs;
            const size_t o = static_cast<size_t>(r) * a.ldo + n;
            if (a.accumulate) {
                static_cast<float*>(a.out)[o] += v;
            } else {
                st_dyn(a.out, a.out_dt, o, v);
            }
        }
    }
}

template <typename TX, typename TW>
static int launch(const GemmArgs& a, int max_tiles, bool swiglu, cudaStream_t stream) {
    dim3 grid(ceil_div(a.N, BN), max_tiles);
    if (grid.y == 0 || grid.x == 0) return 0;
    if (grid.y > 65535) return LOCUS_ERR_UNSUPPORTED;
    if (swiglu) {
        gemm_simt_kernel<TX, TW, true><<<grid, 256, 0, stream>>>(a);
    } else {
        gemm_simt_kernel<TX, TW, false><<<grid, 256, 0, stream>>>(a);
    }
    return locus_launch_status();
}

// x_dt / w_dt: element types of x and of W (and W2).  max_tiles: number of 64-row tiles
// to launch; for a grouped product an upper bound (tiles past *n_tiles return at once).
extern "C" int locus_gemm_simt(const void* x, int x_dt, const void* w, const void* w2, int w_dt,
                               const void* bias, int bias_dt, void* out, int out_dt,
                               int accumulate, const float* row_scale, const int* scale_rows,
                               const int* x_rows,
                               int x_row_div, int M, int N, int K, long long ldx, long long ldo,
                               const int* tile_expert, const int* tile_row0,
                               const int* tile_rows, const int* n_tiles, int max_tiles,
                               long long w_expert_stride, cudaStream_t stream) {
    if (N <= 0 || K <= 0) return LOCUS_ERR_UNSUPPORTED;
    if (accumulate && out_dt != LOCUS_DT_F32) return LOCUS_ERR_UNSUPPORTED;
    if (x_rows != nullptr && x_row_div <= 0) return LOCUS_ERR_UNSUPPORTED;
    GemmArgs a;
    a.x = x; a.w = w; a.w2 = w2; a.bias = bias; a.bias_dt = bias_dt; a.out = out;
    a.out_dt = out_dt; a.accumulate = accumulate; a.row_scale = row_scale; a.scale_rows = scale_rows; a.x_rows = x_rows;
    a.x_row_div = x_row_div; a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldo = ldo;
    a.tile_expert = tile_expert; a.tile_row0 = tile_row0; a.tile_rows = tile_rows;
    a.n_tiles = n_tiles; a.w_expert_stride = w_expert_stride;
    const int tiles = tile_expert ? max_tiles : ceil_div(M, BM);
    const bool swiglu = w2 != nullptr;
    if (x_dt == LOCUS_DT_F32 && w_dt == LOCUS_DT_F32) return launch<float, float>(a, tiles, swiglu, stream);
    if (x_dt == LOCUS_DT_BF16 && w_dt == LOCUS_DT_BF16) return launch<bf16, bf16>(a, tiles, swiglu, stream);
    if (x_dt == LOCUS_DT_BF16 && w_dt == LOCUS_DT_F32) return launch<bf16, float>(a, tiles, swiglu, stream);
    if (x_dt == LOCUS_DT_F32 && w_dt == LOCUS_DT_BF16) return launch<float, bf16>(a, tiles, swiglu, stream);
    return LOCUS_ERR_UNSUPPORTED;
}
