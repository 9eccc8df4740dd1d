// Attention of prompt portions over the paged cache on the tensor cores (bfloat16 keys, values
// and queries; mma.sync m16n8k16 with float32 accumulation), online softmax in float32.
//
// A block of four warps takes 64 consecutive new tokens of one request and one head; each
// warp owns 16 queries.  Keys and values are streamed in tiles of 64 positions through the
// request's block table into shared memory with cp.async (two buffers, the next tile loads
// while this one is used), scores S = Q K^T are accumulated in registers, masked (causal,
// optional window, end of the sequence), scaled, reduced with a running maximum and sum per
// query, and the probabilities, rounded to bfloat16, go straight back into the tensor cores
// as the left operand of P V.  Same cache layout and descriptors as the CUDA-core kernel
// (attention.cu): [n_pages][2][nkv][page_tokens][hd]; items are (segment, first query of
// a 64-query tile).
//
// A step with few such blocks (a short portion behind a long context) leaves most SMs idle and each
// block streaming thousands of keys alone; the key tiles of an item are then cut into n_splits ranges
// that run as blocks of their own (blockIdx.z) and leave unnormalised sums, running maxima and
// denominators in a scratch; attn_chunk_merge_kernel adds the ranges up in ascending order.
//
// Head sizes: every multiple of 16 up to 256 (a template instance each); other sizes are refused and the
// caller uses the CUDA-core kernel.  Rows in shared memory are
// padded by 16 bytes so that ldmatrix reads no bank twice.
#include "common.cuh"

#define MQ 64    // queries per block
#define MK 64    // keys per tile

struct MmaAttnArgs {
    const bf16* q;
    const bf16* pool;
    bf16* out;
    const int* seg_q0;
    const int* seg_qn;
    const int* seg_ctx;
    const int* block_table;
    int table_stride;
    const int* items;
    int nh, nkv, page_tokens, window;
    float scale;
    int n_splits;     // ranges of key tiles per item (1: the block writes out itself)
    float* part_o;    // [item][head][split][MQ][hd] unnormalised sums
    float* part_ml;   // [item][head][split][MQ][2] running maximum (base 2, scaled) and denominator
};

// Key tiles of an item: the first tile's first position and their number (the same in both kernels).
__device__ __forceinline__ void item_tiles(int p0, int nq, int window, int& first_tile, int& n_tiles) {
    const int t_hi = p0 + nq - 1;
    const int t_lo = window > 0 ? max(0, p0 - window + 1) : 0;
    first_tile = (t_lo / MK) * MK;
    n_tiles = (t_hi - first_tile) / MK + 1;
}

__device__ __forceinline__ uint32_t sm_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(128) attn_chunk_mma_kernel(MmaAttnArgs a) {
    constexpr int LDS = HD + 8;          // padded row, elements
    constexpr int CH = HD / 8;           // 16-byte chunks per row
    constexpr int KS = HD / 16;          // k-steps of Q K^T
    constexpr int DT = HD / 8;           // 8-wide output tiles of O
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);      // [MQ][LDS]
    bf16* sK = sQ + MQ * LDS;                          // [2][MK][LDS]
    bf16* sV = sK + 2 * MK * LDS;                      // [2][MK][LDS]

    // Items are listed in ascending position; the late tiles of a prompt see the most keys, so the grid
    // takes them first, for all heads (the heads are the grid's fast index), and the short ones fill the tail.
    const int item = gridDim.y - 1 - blockIdx.y;
    const int seg = a.items[2 * item], qoff = a.items[2 * item + 1];
    const int h = blockIdx.x, kvh = h / (a.nh / a.nkv);
    const int nq = min(MQ, a.seg_qn[seg] - qoff);
    const int row0 = a.seg_q0[seg] + qoff;
    const int p0 = a.seg_ctx[seg] + qoff;
    const int* table = a.block_table + static_cast<size_t>(seg) * a.table_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, qd = lane & 3;
    const int t_hi = p0 + nq - 1;
    const int t_lo = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
    const int P = a.page_tokens;
    const int pshift = (P & (P - 1)) == 0 ? __ffs(P) - 1 : -1;  // pages of 2^k tokens: shifts instead of divisions
    const float scale_log2 = a.scale * 1.4426950408889634f;

    // this block's range of the item's key tiles
    int first_tile, n_tiles_all;
    item_tiles(p0, nq, a.window, first_tile, n_tiles_all);
    const int split = blockIdx.z;
    const int per_split = (n_tiles_all + a.n_splits - 1) / a.n_splits;
    first_tile += split * per_split * MK;
    const int n_tiles = max(0, min(per_split, n_tiles_all - split * per_split));
    if (n_tiles == 0) return;  // the merge counts the live ranges the same way

    // ---- Q tile -> shared (rows past nq are zero)
    for (int i = tid; i < MQ * CH; i += 128) {
        const int r = i / CH, c = i % CH;
        const bf16* src = a.q + (static_cast<size_t>(row0 + min(r, nq - 1)) * a.nh + h) * HD + c * 8;
        cp_async16(sm_addr(sQ + r * LDS + c * 8), src, r < nq ? 16 : 0);
    }
    cp_commit();

    auto load_kv = [&](int tile0, int buf) {
        bf16* dk = sK + buf * MK * LDS;
        bf16* dv = sV + buf * MK * LDS;
        for (int i = tid; i < MK * CH; i += 128) {
            const int r = i / CH, c = i % CH;
            const int t = tile0 + r;
            const bool ok = t >= t_lo && t <= t_hi;
            const int tt = ok ? t : t_hi;  // any valid position: the copy size is 0 when !ok
            const int page = table[pshift >= 0 ? tt >> pshift : tt / P];
            const int off = pshift >= 0 ? tt & (P - 1) : tt % P;
            const bf16* kb = a.pool + ((static_cast<size_t>(page) * 2) * a.nkv + kvh) * P * HD +
                             static_cast<size_t>(off) * HD + c * 8;
            const bf16* vb = kb + static_cast<size_t>(a.nkv) * P * HD;
            cp_async16(sm_addr(dk + r * LDS + c * 8), kb, ok ? 16 : 0);
            cp_async16(sm_addr(dv + r * LDS + c * 8), vb, ok ? 16 : 0);
        }
        cp_commit();
    };

    load_kv(first_tile, 0);

    // ---- Q fragments of this warp's 16 rows, kept in registers
    cp_wait<1>();   // the Q group is done (the first K/V group may still fly)
    __syncthreads();
    uint32_t qf[KS][4];
    {
        const int r = warp * 16 + (lane & 15);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int col = ks * 16 + (lane >> 4) * 8;
            ldsm_x4(sm_addr(sQ + r * LDS + col), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
        }
    }

    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[d][i] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int pq[2] = {p0 + warp * 16 + g, p0 + warp * 16 + g + 8};  // positions of this lane's two query rows

    for (int it = 0; it < n_tiles; ++it) {
        const int tile0 = first_tile + it * MK;
        const int buf = it & 1;
        if (it + 1 < n_tiles) {
            load_kv(tile0 + MK, buf ^ 1);
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        const bf16* tK = sK + buf * MK * LDS;
        const bf16* tV = sV + buf * MK * LDS;

        // ---- S = Q K^T : 8 tiles of 8 keys
        float s[MK / 8][4];
#pragma unroll
        for (int j = 0; j < MK / 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int jp = 0; jp < MK / 16; ++jp) {
                // B fragments of keys jp*16 .. +15 for k-step ks: matrices (keys 0-7, d 0-7), (keys 0-7, d 8-15),
                // (keys 8-15, d 0-7), (keys 8-15, d 8-15)
                const int r = jp * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int col = ks * 16 + ((lane >> 3) & 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4(sm_addr(tK + r * LDS + col), b0, b1, b2, b3);
                mma16816(s[2 * jp], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                mma16816(s[2 * jp + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
            }
        }
        // ---- scale, mask, online softmax (rows g and g + 8 of the warp's 16), in the base-2 domain:
        // exp(x * scale - m) = exp2(x * scale * log2(e) - m').  The mask test runs only on tiles that
        // can hold a masked key for one of this warp's rows (the diagonal, the window's edge, the start).
        float mx[2] = {m_run[0], m_run[1]};
        const int p_first = p0 + warp * 16;
        const bool need_mask = tile0 + MK - 1 > p_first || tile0 < t_lo ||
                               (a.window > 0 && tile0 <= p_first + 15 - a.window);
        if (need_mask) {
#pragma unroll
            for (int j = 0; j < MK / 8; ++j) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = i >> 1;
                    const int t = tile0 + j * 8 + qd * 2 + (i & 1);
                    const int p = pq[rr];
                    const bool ok = t <= p && t >= t_lo && (a.window == 0 || t > p - a.window);
                    const float v = ok ? s[j][i] * scale_log2 : -INFINITY;
                    s[j][i] = v;
                    mx[rr] = fmaxf(mx[rr], v);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < MK / 8; ++j) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float v = s[j][i] * scale_log2;
                    s[j][i] = v;
                    mx[i >> 1] = fmaxf(mx[i >> 1], v);
                }
            }
        }
        float alpha[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            alpha[rr] = (mx[rr] == -INFINITY) ? 1.f : exp2f(m_run[rr] - mx[rr]);
            m_run[rr] = mx[rr];
        }
        float sum[2] = {0.f, 0.f};
        const float m0 = mx[0] == -INFINITY ? 0.f : mx[0], m1 = mx[1] == -INFINITY ? 0.f : mx[1];  // exp2(-inf - 0) = 0
#pragma unroll
        for (int j = 0; j < MK / 8; ++j) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float e = exp2f(s[j][i] - ((i >> 1) ? m1 : m0));
                s[j][i] = e;
                sum[i >> 1] += e;
            }
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) l_run[rr] = l_run[rr] * alpha[rr] + sum[rr];  // quad-partial sums
#pragma unroll
        for (int d = 0; d < DT; ++d) {
            o[d][0] *= alpha[0];
            o[d][1] *= alpha[0];
            o[d][2] *= alpha[1];
            o[d][3] *= alpha[1];
        }
        // ---- O += P V : k-steps of 16 keys
#pragma unroll
        for (int kk = 0; kk < MK / 16; ++kk) {
            const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            const uint32_t a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            const uint32_t a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                // V is [key][d]: transposed loads give B fragments (k = key, n = d):
                // matrices (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15)
                const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int col = dp * 16 + (lane >> 4) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(sm_addr(tV + r * LDS + col), b0, b1, b2, b3);
                mma16816(o[2 * dp], a0, a1, a2, a3, b0, b1);
                mma16816(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();  // everyone is done with this buffer before the tile after next overwrites it
    }
    // ---- normalise and store
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
    }
    if (a.n_splits > 1) {
        const size_t unit = (static_cast<size_t>(item) * a.nh + h) * a.n_splits + split;
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int r = warp * 16 + g + rr * 8;
            if (r >= nq) continue;
            float* po = a.part_o + (unit * MQ + r) * HD;
#pragma unroll
            for (int d = 0; d < DT; ++d)
                *reinterpret_cast<float2*>(po + d * 8 + qd * 2) = make_float2(o[d][rr * 2], o[d][rr * 2 + 1]);
            if (qd == 0) *reinterpret_cast<float2*>(a.part_ml + (unit * MQ + r) * 2) = make_float2(m_run[rr], l_run[rr]);
        }
        return;
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int r = warp * 16 + g + rr * 8;
        if (r >= nq) continue;
        const float inv = 1.0f / l_run[rr];
        bf16* dst = a.out + (static_cast<size_t>(row0 + r) * a.nh + h) * HD;
#pragma unroll
        for (int d = 0; d < DT; ++d) {
            *reinterpret_cast<uint32_t*>(dst + d * 8 + qd * 2) = pack_bf16(o[d][rr * 2] * inv, o[d][rr * 2 + 1] * inv);
        }
    }
}

#define MERGE_MAX_SPLITS 16

// out[row][head] = sum over the live ranges s (ascending) of o_s 2^(m_s - M) / sum of l_s 2^(m_s - M), M = max m_s.
// One thread per (query row, two adjacent dimensions) of an (item, head); the loads of all ranges are
// issued together (the loops are unrolled over the most ranges there can be).
__global__ void __launch_bounds__(128) attn_chunk_merge_kernel(MmaAttnArgs a, int hd) {
    const int item = blockIdx.y, h = blockIdx.z;
    const int seg = a.items[2 * item], qoff = a.items[2 * item + 1];
    const int nq = min(MQ, a.seg_qn[seg] - qoff);
    const int half = hd >> 1;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nq * half) return;
    const int r = i / half, d = (i - r * half) * 2;
    const int row0 = a.seg_q0[seg] + qoff;
    int first_tile, n_tiles;
    item_tiles(a.seg_ctx[seg] + qoff, nq, a.window, first_tile, n_tiles);
    const int per_split = (n_tiles + a.n_splits - 1) / a.n_splits;
    const int live = (n_tiles + per_split - 1) / per_split;
    const size_t unit0 = (static_cast<size_t>(item) * a.nh + h) * a.n_splits;
    float2 ml[MERGE_MAX_SPLITS], v[MERGE_MAX_SPLITS];
#pragma unroll
    for (int s = 0; s < MERGE_MAX_SPLITS; ++s) {
        ml[s] = make_float2(-INFINITY, 0.f);
        v[s] = make_float2(0.f, 0.f);
        if (s < live) {
            ml[s] = *reinterpret_cast<const float2*>(a.part_ml + ((unit0 + s) * MQ + r) * 2);
            v[s] = *reinterpret_cast<const float2*>(a.part_o + ((unit0 + s) * MQ + r) * hd + d);
        }
    }
    float M = -INFINITY;
#pragma unroll
    for (int s = 0; s < MERGE_MAX_SPLITS; ++s) M = fmaxf(M, ml[s].x);
    float L = 0.f, x = 0.f, y = 0.f;
#pragma unroll
    for (int s = 0; s < MERGE_MAX_SPLITS; ++s) {
        const float w = ml[s].x == -INFINITY ? 0.f : exp2f(ml[s].x - M);
        L += ml[s].y * w;
        x += v[s].x * w;
        y += v[s].y * w;
    }
    const float inv = 1.0f / L;
    *reinterpret_cast<uint32_t*>(a.out + (static_cast<size_t>(row0 + r) * a.nh + h) * hd + d) = pack_bf16(x * inv, y * inv);
}

template <int HD>
static int launch(const MmaAttnArgs& a, int n_items, cudaStream_t stream) {
    constexpr size_t smem = sizeof(bf16) * (HD + 8) * (MQ + 4 * MK);
    static bool set = false;
    if (!set) {
        if (cudaFuncSetAttribute(attn_chunk_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return static_cast<int>(cudaGetLastError());
        set = true;
    }
    if (n_items > 65535) return LOCUS_ERR_UNSUPPORTED;
    dim3 grid(a.nh, n_items, a.n_splits);
    attn_chunk_mma_kernel<HD><<<grid, 128, smem, stream>>>(a);
    if (a.n_splits > 1)
        attn_chunk_merge_kernel<<<dim3((MQ * (HD / 2) + 127) / 128, n_items, a.nh), 128, 0, stream>>>(a, HD);
    return locus_launch_status();
}

// items: [n_items, 2] = (segment, first query of a 64-query tile).  bfloat16 only.
// n_splits > 1: part_o holds n_items * nh * n_splits * 64 * hd floats, part_ml n_items * nh * n_splits * 128.
extern "C" int locus_attn_chunk_mma(const void* q, const void* pool, void* out, const int* seg_q0, const int* seg_qn,
                                    const int* seg_ctx, const int* block_table, int table_stride, const int* items,
                                    int n_items, int nh, int nkv, int hd, int page_tokens, int window, float scale,
                                    int n_splits, float* part_o, float* part_ml, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || nh > 65535 || page_tokens <= 0 || window < 0) return LOCUS_ERR_UNSUPPORTED;
    if (n_splits < 1 || n_splits > MERGE_MAX_SPLITS || (n_splits > 1 && n_items > 65535) || (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)) ||
        ((reinterpret_cast<uintptr_t>(part_o) | reinterpret_cast<uintptr_t>(part_ml)) & 7))
        return LOCUS_ERR_UNSUPPORTED;
    MmaAttnArgs a;
    a.q = static_cast<const bf16*>(q); a.pool = static_cast<const bf16*>(pool); a.out = static_cast<bf16*>(out);
    a.seg_q0 = seg_q0; a.seg_qn = seg_qn; a.seg_ctx = seg_ctx; a.block_table = block_table;
    a.table_stride = table_stride; a.items = items; a.nh = nh; a.nkv = nkv; a.page_tokens = page_tokens;
    a.window = window; a.scale = scale;
    a.n_splits = n_splits; a.part_o = part_o; a.part_ml = part_ml;
    switch (hd) {
        case 16: return launch<16>(a, n_items, stream);
        case 32: return launch<32>(a, n_items, stream);
        case 48: return launch<48>(a, n_items, stream);
        case 64: return launch<64>(a, n_items, stream);
        case 80: return launch<80>(a, n_items, stream);
        case 96: return launch<96>(a, n_items, stream);
        case 112: return launch<112>(a, n_items, stream);
        case 128: return launch<128>(a, n_items, stream);
        case 144: return launch<144>(a, n_items, stream);
        case 160: return launch<160>(a, n_items, stream);
        case 176: return launch<176>(a, n_items, stream);
        case 192: return launch<192>(a, n_items, stream);
        case 208: return launch<208>(a, n_items, stream);
        case 224: return launch<224>(a, n_items, stream);
        case 240: return launch<240>(a, n_items, stream);
        case 256: return launch<256>(a, n_items, stream);
        default: return LOCUS_ERR_UNSUPPORTED;
    }
}
