// bfloat16 products for a few dozen rows (decode steps, the router): out = x . W^T with at
// most 32 rows of x per tile.  Reading W once from HBM is what bounds this work, so a block
// takes only 16 rows of W and streams them with 16-byte loads straight from global memory
// into tensor-core fragments (mma.sync m16n8k16, bfloat16 in, float32 accumulate): the 16
// weight rows are the M side, up to 32 tokens (four 8-wide tiles) the N side.  The eight
// warps of a block split K between them in interleaved 32-element steps, so a block of 16
// weight rows keeps 8 x 4 x 16 bytes per lane in flight, and N / 16 blocks cover the GPU even
// for a 2048-row matrix.  Partial sums of the warps are added in warp order through shared
// memory, then the usual epilogue runs (bias, SwiGLU of two weight matrices, per-row scale,
// store or add into float32); gathered and grouped (expert tile list) forms as elsewhere.
//
// Within a k-step the 32 k-values are handed to the two MMAs in a permuted order (lane
// quad q takes the 8 consecutive elements 8q..8q+7 of every row), the same for W and x, so
// every load is a full 16-byte vector of one row.  The order of the sum of an element
// depends on K only.
#include "common.cuh"
#include "route_select.cuh"

#define SK_WARPS 8
#define SK_ROWS 16

struct SkinnyArgs {
    const bf16* x;
    const bf16* w;
    const bf16* w2;
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
    // The tile list was written by a kernel that finished before the kernel in front of this one started (the
    // second product of the experts: the list comes from the router, the kernel in front is the first product):
    // the block may read it, and ask for its first weights, before it waits for the kernel in front.
    int lists_ready;
    // Optional tail (the router of a decode-sized batch): when route_counter is set, `out` holds float32 router
    // logits [T, ldo] of all T = M tokens (one row tile), and the block that finishes last selects every token's
    // experts from them and lays the pairs out by expert (route_select.cuh), all in this launch.  The counter is
    // zero before the launch and zero after it.
    int* route_counter;
    int* route_ids;
    float* route_wts;
    float* route_gamma;
    int route_experts, route_has_gate;
    RouteOpts route_opts;
    RouteLayoutOut route_layout;
};

__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const bf16* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }

template <int NT, bool DUAL, bool ROUTE = false>
__global__ void __launch_bounds__(32 * SK_WARPS, ROUTE ? 1 : (NT == 1 ? 4 : ((NT == 4 && DUAL) ? 2 : 3))) skinny_kernel(SkinnyArgs a) {
    extern __shared__ float red[];  // [SK_WARPS][(DUAL ? 2 : 1)][NT][16 * 8]
    // Under programmatic dependent launch this block may be resident while the kernel in front of it still runs.
    // The weights do not depend on that kernel, so a plain product asks for its first weights before it waits;
    // a grouped product learns its expert from the tile list, which the kernel in front may have written.
    const bool grouped = a.tile_expert != nullptr;
    const bool wait_first = grouped && !a.lists_ready;
    if (wait_first) pdl_entry();
    int tok0, ntok;
    const bf16* W = a.w;
    const bf16* W2 = a.w2;
    if (grouped) {
        const int tile = blockIdx.y;
        if (tile >= *a.n_tiles) {
            if (!wait_first) pdl_entry();  // the grid must not finish before the kernel in front has
            return;
        }
        const long long e = a.tile_expert[tile];
        tok0 = a.tile_row0[tile];
        ntok = a.tile_rows[tile];
        W += e * a.w_expert_stride;
        if (DUAL) W2 += e * a.w_expert_stride;
    } else {
        tok0 = blockIdx.y * (NT * 8);
        ntok = min(NT * 8, a.M - tok0);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int n0 = blockIdx.x * SK_ROWS;
    const int K = a.K;
    // weight rows of this lane (clamped: rows past N are computed and dropped)
    const long long r_lo = min(n0 + g, a.N - 1), r_hi = min(n0 + g + 8, a.N - 1);
    const bf16* wl = W + r_lo * K;
    const bf16* wh = W + r_hi * K;
    const bf16* ul = DUAL ? W2 + r_lo * K : nullptr;
    const bf16* uh = DUAL ? W2 + r_hi * K : nullptr;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // this warp's k-steps: 32 elements each, interleaved with the other warps'; four steps at a time
    // (the router's launch is a handful of blocks whose whole share of the weights fits eight steps per warp: they
    // are all asked for at once, before the wait for the kernel in front)
    constexpr int STEP = 32, STRIDE = STEP * SK_WARPS, UNROLL = ROUTE ? 8 : (DUAL ? 2 : 4);
    uint4 al[UNROLL], ah[UNROLL], bl[DUAL ? UNROLL : 1], bh[DUAL ? UNROLL : 1];
    auto load_weights = [&](int kb) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = kb + u * STRIDE + q * 8;
            const bool in = k < K;  // K is a multiple of 8: a chunk is inside or outside as a whole
            al[u] = in ? ld_stream(wl + k) : zero;
            ah[u] = in ? ld_stream(wh + k) : zero;
            if (DUAL) {
                bl[u] = in ? ld_stream(ul + k) : zero;
                bh[u] = in ? ld_stream(uh + k) : zero;
            }
        }
    };
    const int kb_first = warp * STEP;
    if (kb_first < K) load_weights(kb_first);
    if (!wait_first) pdl_entry();
    // token rows of this lane, one per 8-wide tile
    const bf16* xr[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int t = j * 8 + g;
        if (t < ntok) {
            const int r = tok0 + t;
            const long long xrow = a.x_rows ? a.x_rows[r] / a.x_row_div : r;
            xr[j] = a.x + xrow * a.ldx;
        } else {
            xr[j] = nullptr;
        }
    }
    float c[NT][4], c2[DUAL ? NT : 1][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            c[j][i] = 0.f;
            if (DUAL) c2[j][i] = 0.f;
        }
    for (int kb = kb_first; kb < K; kb += STRIDE * UNROLL) {
        if (kb != kb_first) load_weights(kb);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = kb + u * STRIDE + q * 8;
            if (kb + u * STRIDE >= K) break;  // uniform in the warp
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 xv = (xr[j] != nullptr && k < K) ? *reinterpret_cast<const uint4*>(xr[j] + k) : zero;
                mma_bf16(c[j], al[u].x, ah[u].x, al[u].y, ah[u].y, xv.x, xv.y);
                mma_bf16(c[j], al[u].z, ah[u].z, al[u].w, ah[u].w, xv.z, xv.w);
                if (DUAL) {
                    mma_bf16(c2[j], bl[u].x, bh[u].x, bl[u].y, bh[u].y, xv.x, xv.y);
                    mma_bf16(c2[j], bl[u].z, bh[u].z, bl[u].w, bh[u].w, xv.z, xv.w);
                }
            }
        }
    }
    pdl_trigger();  // the weights are read: the next kernel may start up under this block's reduction
    // partial sums of the warps -> shared memory; element (row r, token col) of tile j at [j][col * 16 + r]
    constexpr int SETS = DUAL ? 2 : 1;
    float* mine = red + static_cast<size_t>(warp) * SETS * NT * 128;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        float* d = mine + j * 128;
        d[(2 * q) * 16 + g] = c[j][0];
        d[(2 * q + 1) * 16 + g] = c[j][1];
        d[(2 * q) * 16 + g + 8] = c[j][2];
        d[(2 * q + 1) * 16 + g + 8] = c[j][3];
        if (DUAL) {
            float* d2 = mine + (NT + j) * 128;
            d2[(2 * q) * 16 + g] = c2[j][0];
            d2[(2 * q + 1) * 16 + g] = c2[j][1];
            d2[(2 * q) * 16 + g + 8] = c2[j][2];
            d2[(2 * q + 1) * 16 + g + 8] = c2[j][3];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < NT * 128; idx += blockDim.x) {
        const int j = idx / 128, col = (idx % 128) / 16, r = idx % 16;
        const int t = j * 8 + col, n = n0 + r;
        if (t >= ntok || n >= a.N) continue;
        float v = 0.f, u = 0.f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) {
            v += red[static_cast<size_t>(w) * SETS * NT * 128 + idx];
            if (DUAL) u += red[static_cast<size_t>(w) * SETS * NT * 128 + NT * 128 + idx];
        }
        if (DUAL) v = v / (1.0f + expf(-v)) * u;
        if (a.bias) v += ld_dyn(a.bias, a.bias_dt, n);
        const int row = tok0 + t;
        if (a.row_scale) v *= a.row_scale[a.scale_rows ? a.scale_rows[row] : row];
        const size_t o = static_cast<size_t>(row) * a.ldo + n;
        if (a.accumulate) {
            static_cast<float*>(a.out)[o] += v;
        } else {
            st_dyn(a.out, a.out_dt, o, v);
        }
    }
    if (ROUTE) {
        // the block that writes its logits last routes: selection and expert layout from the complete logits
        __shared__ int is_last;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            is_last = atomicAdd(a.route_counter, 1) == static_cast<int>(gridDim.x) - 1;
            if (is_last) *a.route_counter = 0;
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        route_small_block(red, static_cast<const float*>(a.out), static_cast<int>(a.ldo), a.route_ids, a.route_wts,
                          a.route_gamma, a.M, a.route_experts, a.route_has_gate, a.route_opts, a.route_layout);
    }
}

template <int NT>
static int launch(const SkinnyArgs& a, int tiles, bool dual, cudaStream_t stream, size_t smem_tail = 0) {
    dim3 grid(ceil_div(a.N, SK_ROWS), tiles);
    if (grid.x == 0 || grid.y == 0) return 0;
    if (grid.y > 65535) return LOCUS_ERR_UNSUPPORTED;
    size_t smem = sizeof(float) * SK_WARPS * (dual ? 2 : 1) * NT * 128;
    if (smem_tail > smem) smem = smem_tail;
    if (smem > 200 * 1024) return LOCUS_ERR_UNSUPPORTED;
    if (a.route_counter != nullptr) {
        if (dual || NT > 2) return LOCUS_ERR_UNSUPPORTED;
        constexpr int NTR = NT > 2 ? 2 : NT;
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(skinny_kernel<NTR, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        locus_launch(skinny_kernel<NTR, false, true>, grid, 32 * SK_WARPS, smem, stream, a);
    } else if (dual) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(skinny_kernel<NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        locus_launch(skinny_kernel<NT, true>, grid, 32 * SK_WARPS, smem, stream, a);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(skinny_kernel<NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        locus_launch(skinny_kernel<NT, false>, grid, 32 * SK_WARPS, smem, stream, a);
    }
    return locus_launch_status();
}

// tile_tokens: 8, 16 or 32 rows of x per tile (for a grouped product: the tile size of the
// tile list).  x and W bfloat16; K a multiple of 8; 16-byte aligned rows.
extern "C" int locus_gemm_skinny(const void* x, const void* w, const void* w2, const void* bias, int bias_dt,
                                 void* out, int out_dt, int accumulate, const float* row_scale,
                                 const int* scale_rows, const int* x_rows, int x_row_div, int M, int N, int K,
                                 long long ldx, long long ldo, int tile_tokens, const int* tile_expert,
                                 const int* tile_row0, const int* tile_rows, const int* n_tiles, int max_tiles,
                                 long long w_expert_stride, int lists_ready, cudaStream_t stream) {
    if (N <= 0 || K <= 0 || K % 8 != 0 || ldx % 8 != 0) return LOCUS_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(w2)) & 15)
        return LOCUS_ERR_UNSUPPORTED;
    if (accumulate && out_dt != LOCUS_DT_F32) return LOCUS_ERR_UNSUPPORTED;
    if (x_rows != nullptr && x_row_div <= 0) return LOCUS_ERR_UNSUPPORTED;
    if (tile_tokens != 8 && tile_tokens != 16 && tile_tokens != 32) return LOCUS_ERR_UNSUPPORTED;
    SkinnyArgs a;
    a.x = static_cast<const bf16*>(x); a.w = static_cast<const bf16*>(w); a.w2 = static_cast<const bf16*>(w2);
    a.bias = bias; a.bias_dt = bias_dt; a.out = out; a.out_dt = out_dt; a.accumulate = accumulate;
    a.row_scale = row_scale; a.scale_rows = scale_rows; a.x_rows = x_rows; a.x_row_div = x_row_div;
    a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldo = ldo; a.tile_expert = tile_expert; a.tile_row0 = tile_row0;
    a.tile_rows = tile_rows; a.n_tiles = n_tiles; a.w_expert_stride = w_expert_stride;
    a.lists_ready = lists_ready;
    a.route_counter = nullptr;
    const int tiles = tile_expert ? max_tiles : ceil_div(M, tile_tokens);
    const bool dual = w2 != nullptr;
    if (tile_tokens == 8) return launch<1>(a, tiles, dual, stream);
    if (tile_tokens == 16) return launch<2>(a, tiles, dual, stream);
    return launch<4>(a, tiles, dual, stream);
}

// The router of a decode-sized batch in one launch: logits[t, e] = w_all[e] . h[t] for the E (+1 with a gate) rows of
// w_all by the kernel above -- the same kernel, and the same order of every sum, as locus_gemm_skinny gives for any
// number of tokens -- and in its last block the selection (locus_router_select) and the expert layout
// (locus_moe_sort) of route_select.cuh.  T <= 16 tokens (one row tile), T * k <= RS_MAX_PAIRS, E <= RS_MAX_E.
// counter: one int, zero before the call and zero after it.
extern "C" int locus_router_fused_small(const void* h, const void* w_all, float* logits, int ld, int* counter, int* ids,
                                        float* wts, float* gamma, int T, int H, long long ldh, int E, int k, int has_gate,
                                        int renorm, float scale, int score_fn, const float* sel_bias, int n_group,
                                        int n_group_used, int tile_m, int* counts, int* offsets, int* sorted_pair,
                                        int* pair_pos, int* tile_expert, int* tile_row0, int* tile_rows, int* n_tiles,
                                        cudaStream_t stream) {
    if (T <= 0) return 0;
    const RouteOpts o{k, renorm, score_fn, n_group, n_group_used, scale, sel_bias};
    const int n_rows = E + (has_gate ? 1 : 0);
    if (!route_opts_ok(o, E) || ld < n_rows || tile_m <= 0 || counter == nullptr) return LOCUS_ERR_UNSUPPORTED;
    if (T > 16 || E > RS_MAX_E || static_cast<long long>(T) * k > RS_MAX_PAIRS) return LOCUS_ERR_UNSUPPORTED;
    if (H <= 0 || H % 8 != 0 || ldh % 8 != 0) return LOCUS_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(w_all)) & 15) return LOCUS_ERR_UNSUPPORTED;
    SkinnyArgs a;
    a.x = static_cast<const bf16*>(h); a.w = static_cast<const bf16*>(w_all); a.w2 = nullptr;
    a.bias = nullptr; a.bias_dt = 0; a.out = logits; a.out_dt = LOCUS_DT_F32; a.accumulate = 0;
    a.row_scale = nullptr; a.scale_rows = nullptr; a.x_rows = nullptr; a.x_row_div = 1;
    a.M = T; a.N = n_rows; a.K = H; a.ldx = ldh; a.ldo = ld; a.tile_expert = nullptr; a.tile_row0 = nullptr;
    a.tile_rows = nullptr; a.n_tiles = nullptr; a.w_expert_stride = 0; a.lists_ready = 0;
    a.route_counter = counter; a.route_ids = ids; a.route_wts = wts; a.route_gamma = gamma;
    a.route_experts = E; a.route_has_gate = has_gate; a.route_opts = o;
    a.route_layout = RouteLayoutOut{tile_m, counts, offsets, sorted_pair, pair_pos, tile_expert, tile_row0, tile_rows, n_tiles};
    const size_t tail = route_small_smem(SK_WARPS, T, E, k);
    // the same row tile that locus_gemm_skinny's callers use for this many tokens
    if (T <= 8) return launch<1>(a, 1, false, stream, tail);
    return launch<2>(a, 1, false, stream, tail);
}
