// Memory-bound row kernels: embedding gather, RMSNorm, rotary position encoding fused
// with the write of K and V into cache pages, and the slot-ordered sum of routed-expert
// outputs into the residual stream.  All statistics, angles and sums are float32.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = table[tokens[t], :] as float32 (the residual stream is float32).
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const void* __restrict__ table,
                                  int table_dt, float* __restrict__ out, int H) {
    pdl_entry();
    pdl_trigger();
    const int t = blockIdx.x;
    const size_t row = static_cast<size_t>(tokens[t]) * H;
    float* o = out + static_cast<size_t>(t) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = ld_dyn(table, table_dt, row + i);
}

extern "C" int locus_embed_rows(const int* tokens, const void* table, int table_dt, float* out,
                                int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    locus_launch(embed_rows_kernel, T, 256, 0, stream, tokens, table, table_dt, out, H);
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// RMSNorm of rows: out[i, :] = x[r, :] * rsqrt(mean(x[r]^2) + eps) * w, r = rows ? rows[i] : i.
// The multiplication order (x * scale) * w follows the reference.  One block per row; the
// sum of squares is reduced in an order that depends on H only.
__global__ void rmsnorm_kernel(const void* __restrict__ x, int x_dt, const void* __restrict__ w,
                               int w_dt, float eps, void* __restrict__ out, int out_dt,
                               const int* __restrict__ rows, int H) {
    __shared__ float warp_part[32];
    __shared__ float scale_s;
    const int i = blockIdx.x;
    const size_t src = static_cast<size_t>(rows ? rows[i] : i) * H;
    const size_t dst = static_cast<size_t>(i) * H;
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float v = ld_dyn(x, x_dt, src + j);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) warp_part[wid] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        const int nw = blockDim.x >> 5;
        for (int k = 0; k < nw; ++k) tot += warp_part[k];
        scale_s = 1.0f / sqrtf(tot / static_cast<float>(H) + eps);
    }
    __syncthreads();
    const float scale = scale_s;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float v = ld_dyn(x, x_dt, src + j);
        st_dyn(out, out_dt, dst + j, v * scale * ld_dyn(w, w_dt, j));
    }
}

// The common case (float32 in, width a multiple of 4): 16-byte loads, the row kept in registers.
//
// With add_src: first x[i] += sum over slots s < add_k (in slot order) of add_src[add_pos[i * add_k + s]]
// (the outputs of a row's experts, the sum that moe_combine_kernel forms, in the same order), written
// back to x, then the norm of the new row.  With rows the sum goes into the norm only and x stays as
// it was (a row may be named twice, and nobody reads the other rows' sums).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void put4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void put4(bf16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = pk;
}
// dst[c .. c + 3] = t * scale * w[c .. c + 3], every element rounded once as from_f does
template <typename TW, typename TO>
__device__ __forceinline__ void store4(TO* dst, const TW* w, int c, float4 t, float scale, bool wide) {
    if (wide) {
        const float4 g = load4(w + c);
        put4(dst + c, t.x * scale * g.x, t.y * scale * g.y, t.z * scale * g.z, t.w * scale * g.w);
    } else {
        dst[c] = from_f<TO>(t.x * scale * to_f(w[c]));
        dst[c + 1] = from_f<TO>(t.y * scale * to_f(w[c + 1]));
        dst[c + 2] = from_f<TO>(t.z * scale * to_f(w[c + 2]));
        dst[c + 3] = from_f<TO>(t.w * scale * to_f(w[c + 3]));
    }
}

template <typename TW, typename TO>
__global__ void __launch_bounds__(256) rmsnorm_f32_kernel(float* __restrict__ x, const TW* __restrict__ w,
                                                          float eps, TO* __restrict__ out,
                                                          const int* __restrict__ rows, int H,
                                                          const void* __restrict__ add_src, int add_bf16,
                                                          const int* __restrict__ add_pos, int add_k, int vec_io) {
    __shared__ float warp_part[8];
    __shared__ float scale_s;
    const int i = blockIdx.x;
    const int n4 = H >> 2;
    const bool wide = vec_io;
    // The norm's weights do not depend on the kernel in front: under programmatic dependent launch they are asked
    // for before the wait for it (the row itself is what that kernel writes).
    float4 g[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int j = threadIdx.x + u * 256;
        g[u] = (wide && j < n4) ? load4(w + (j << 2)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_entry();
    pdl_trigger();
    const int r = rows ? rows[i] : i;
    float4* src = reinterpret_cast<float4*>(x + static_cast<size_t>(r) * H);
    const bool write_back = rows == nullptr;
    auto fetch = [&](int j) -> float4 {
        float4 t = src[j];
        if (add_src != nullptr) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < add_k; ++s) {
                const size_t at = static_cast<size_t>(add_pos[r * add_k + s]) * H;
                float4 p;
                if (add_bf16) {
                    const uint2 raw = reinterpret_cast<const uint2*>(static_cast<const bf16*>(add_src) + at)[j];
                    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                    p = make_float4(lo.x, lo.y, hi.x, hi.y);
                } else {
                    p = reinterpret_cast<const float4*>(static_cast<const float*>(add_src) + at)[j];
                }
                acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
            }
            t.x += acc.x; t.y += acc.y; t.z += acc.z; t.w += acc.w;
            if (write_back) src[j] = t;
        }
        return t;
    };
    // second reading of a row too wide for the registers: x holds the sum already unless it was left alone
    auto fetch_again = [&](int j) -> float4 { return write_back ? src[j] : fetch(j); };
    float4 v[4];  // up to 4096 elements per row in registers; wider rows re-read
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int j = threadIdx.x + u * 256;
        if (j < n4) {
            v[u] = fetch(j);
            ss = fmaf(v[u].x, v[u].x, ss); ss = fmaf(v[u].y, v[u].y, ss);
            ss = fmaf(v[u].z, v[u].z, ss); ss = fmaf(v[u].w, v[u].w, ss);
        }
    }
    for (int j = threadIdx.x + 1024; j < n4; j += 256) {
        const float4 t = fetch(j);
        ss = fmaf(t.x, t.x, ss); ss = fmaf(t.y, t.y, ss); ss = fmaf(t.z, t.z, ss); ss = fmaf(t.w, t.w, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int k = 0; k < 8; ++k) tot += warp_part[k];
        scale_s = 1.0f / sqrtf(tot / static_cast<float>(H) + eps);
    }
    __syncthreads();
    const float scale = scale_s;
    TO* dst = out + static_cast<size_t>(i) * H;
    // four weights in, four results out, each as one access where the rows are aligned for it (checked by the host)
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int j = threadIdx.x + u * 256;
        if (j >= n4) continue;
        if (wide) {
            const int c = j << 2;
            put4(dst + c, v[u].x * scale * g[u].x, v[u].y * scale * g[u].y, v[u].z * scale * g[u].z, v[u].w * scale * g[u].w);
        } else {
            store4(dst, w, j << 2, v[u], scale, false);
        }
    }
    for (int j = threadIdx.x + 1024; j < n4; j += 256) store4(dst, w, j << 2, fetch_again(j), scale, wide);
}

// add_src (float32 or bfloat16 rows, add_dt) / add_pos / add_k: see rmsnorm_f32_kernel; only with float32 x, H a
// multiple of 4, 16-byte aligned x and add_src.
extern "C" int locus_rmsnorm(void* x, int x_dt, const void* w, int w_dt, float eps, void* out,
                             int out_dt, const int* rows, int n_rows, int H, const void* add_src, int add_dt,
                             const int* add_pos, int add_k, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const bool fast = x_dt == LOCUS_DT_F32 && H % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    if (add_src != nullptr &&
        (!fast || add_pos == nullptr || add_k <= 0 || (reinterpret_cast<uintptr_t>(add_src) & 15) ||
         (add_dt != LOCUS_DT_F32 && add_dt != LOCUS_DT_BF16)))
        return LOCUS_ERR_UNSUPPORTED;
    const int add_bf16 = add_dt == LOCUS_DT_BF16 ? 1 : 0;
    // weights and output rows start on 16-byte boundaries (H % 4 == 0 keeps every row of out aligned for 4 elements)
    const int vec_io = ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 ? 1 : 0;
    if (fast) {
        float* xf = static_cast<float*>(x);
#define NORM_LAUNCH(TW, TO)                                                                             \
        locus_launch(rmsnorm_f32_kernel<TW, TO>, n_rows, 256, 0, stream, xf, static_cast<const TW*>(w), eps,      \
                     static_cast<TO*>(out), rows, H, add_src, add_bf16, add_pos, add_k, vec_io)
        if (w_dt == LOCUS_DT_BF16 && out_dt == LOCUS_DT_BF16) NORM_LAUNCH(bf16, bf16);
        else if (w_dt == LOCUS_DT_F32 && out_dt == LOCUS_DT_F32) NORM_LAUNCH(float, float);
        else if (w_dt == LOCUS_DT_F32 && out_dt == LOCUS_DT_BF16) NORM_LAUNCH(float, bf16);
        else NORM_LAUNCH(bf16, float);
#undef NORM_LAUNCH
        return locus_launch_status();
    }
    rmsnorm_kernel<<<n_rows, 256, 0, stream>>>(x, x_dt, w, w_dt, eps, out, out_dt, rows, H);
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Rotary encoding of q and k (angles = position * inv_freq[i], float32; sinf/cosf, no
// fast-math) and write of the rotated K and the unrotated V into the page pool.
//   qkv      [T, (nh + 2*nkv) * hd]   projections with bias already added
//   q_out    [T, nh * hd]             rotated queries
//   pool     one layer's pages: [n_pages][2 (K,V)][nkv][page_tokens][hd]
//   slots    [T] page * page_tokens + offset of each token (from the block table)
//   pairing  0: half-split pairs (i, i + rot/2); 1: interleaved pairs (2i, 2i+1)
// Dimensions >= rot_dim of a head pass through unrotated.  inv_freq == nullptr applies
// no rotation at all (a mixer without rotary encoding still uses the K/V write).
// write_kv == 0 leaves the pages alone (a layer that reads another layer's cache).
template <typename TA>
__global__ void rope_kv_write_kernel(const TA* __restrict__ qkv, const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq, TA* __restrict__ q_out,
                                     TA* __restrict__ pool, const int* __restrict__ slots, int nh,
                                     int nkv, int hd, int rot_dim, int pairing, int page_tokens,
                                     int write_kv) {
    const int t = blockIdx.x;
    const int half = rot_dim / 2;
    const float pos = static_cast<float>(positions[t]);
    const TA* src = qkv + static_cast<size_t>(t) * (nh + 2 * nkv) * hd;
    const int slot = slots[t];
    const int page = slot / page_tokens, off = slot % page_tokens;
    const size_t page_base = static_cast<size_t>(page) * 2 * nkv * page_tokens * hd;
    // rotated part of q and k heads: one work item per (head, pair)
    const int n_rot_heads = nh + nkv;
    // sine and cosine once per pair index, shared by all heads of the token
    __shared__ float cs_c[256], cs_s[256];
    if (inv_freq != nullptr) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float theta = pos * inv_freq[i];
            cs_c[i] = cosf(theta);
            cs_s[i] = sinf(theta);
        }
    }
    __syncthreads();
    if (inv_freq != nullptr) {
        for (int it = threadIdx.x; it < n_rot_heads * half; it += blockDim.x) {
            const int h = it / half, i = it % half;
            const int d0 = pairing == 0 ? i : 2 * i;
            const int d1 = pairing == 0 ? i + half : 2 * i + 1;
            const float c = cs_c[i], s = cs_s[i];
            const float x0 = to_f(src[h * hd + d0]);
            const float x1 = to_f(src[h * hd + d1]);
            const float y0 = x0 * c - x1 * s;
            const float y1 = x0 * s + x1 * c;
            if (h < nh) {
                TA* q = q_out + (static_cast<size_t>(t) * nh + h) * hd;
                q[d0] = from_f<TA>(y0);
                q[d1] = from_f<TA>(y1);
            } else if (write_kv) {
                TA* k = pool + page_base + (static_cast<size_t>(h - nh) * page_tokens + off) * hd;
                k[d0] = from_f<TA>(y0);
                k[d1] = from_f<TA>(y1);
            }
        }
    }
    // pass-through part of q and k heads, and all of v
    const int rot = inv_freq != nullptr ? rot_dim : 0;
    const int pass = hd - rot;
    for (int it = threadIdx.x; it < n_rot_heads * pass; it += blockDim.x) {
        const int h = it / pass, d = rot + it % pass;
        const TA v = src[h * hd + d];
        if (h < nh) {
            q_out[(static_cast<size_t>(t) * nh + h) * hd + d] = v;
        } else if (write_kv) {
            pool[page_base + (static_cast<size_t>(h - nh) * page_tokens + off) * hd + d] = v;
        }
    }
    if (!write_kv) return;
    const TA* vsrc = src + static_cast<size_t>(nh + nkv) * hd;
    TA* vdst = pool + page_base + static_cast<size_t>(nkv) * page_tokens * hd;
    for (int it = threadIdx.x; it < nkv * hd; it += blockDim.x) {
        const int h = it / hd, d = it % hd;
        vdst[(static_cast<size_t>(h) * page_tokens + off) * hd + d] = vsrc[it];
    }
}

// bfloat16, half-split pairs over the whole head: 16-byte loads and stores, eight pairs per thread.
__global__ void __launch_bounds__(256) rope_kv_write_bf16_kernel(
    const bf16* __restrict__ qkv, const int* __restrict__ positions, const float* __restrict__ inv_freq,
    bf16* __restrict__ q_out, bf16* __restrict__ pool, const int* __restrict__ slots, int nh, int nkv, int hd,
    int page_tokens, int write_kv) {
    // Positions, slots and frequencies were on the device before the step's first kernel: under programmatic
    // dependent launch the angles' sines and cosines are ready before the wait for the kernel that writes q, k, v.
    __shared__ float cs_c[128], cs_s[128];
    const int t = blockIdx.x;
    const int half = hd / 2;
    const float pos = static_cast<float>(positions[t]);
    const int slot = slots[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float theta = pos * inv_freq[i];
        cs_c[i] = cosf(theta);
        cs_s[i] = sinf(theta);
    }
    __syncthreads();
    pdl_entry();
    pdl_trigger();
    const bf16* src = qkv + static_cast<size_t>(t) * (nh + 2 * nkv) * hd;
    const int page = slot / page_tokens, off = slot % page_tokens;
    bf16* kbase = pool + static_cast<size_t>(page) * 2 * nkv * page_tokens * hd + static_cast<size_t>(off) * hd;
    const int cpb = half / 8;  // 16-byte chunks per half head
    for (int it = threadIdx.x; it < (nh + nkv) * cpb; it += blockDim.x) {
        const int h = it / cpb, i0 = (it % cpb) * 8;
        if (h >= nh && !write_kv) continue;
        const uint4 lo = *reinterpret_cast<const uint4*>(src + h * hd + i0);
        const uint4 hi = *reinterpret_cast<const uint4*>(src + h * hd + half + i0);
        const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&lo);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&hi);
        uint4 olo, ohi;
        __nv_bfloat162* ol = reinterpret_cast<__nv_bfloat162*>(&olo);
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&ohi);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float2 x0 = __bfloat1622float2(l2[u]), x1 = __bfloat1622float2(h2[u]);
            const float c0 = cs_c[i0 + 2 * u], s0 = cs_s[i0 + 2 * u], c1 = cs_c[i0 + 2 * u + 1], s1 = cs_s[i0 + 2 * u + 1];
            ol[u] = __floats2bfloat162_rn(x0.x * c0 - x1.x * s0, x0.y * c1 - x1.y * s1);
            oh[u] = __floats2bfloat162_rn(x0.x * s0 + x1.x * c0, x0.y * s1 + x1.y * c1);
        }
        bf16* dst = h < nh ? q_out + (static_cast<size_t>(t) * nh + h) * hd
                           : kbase + static_cast<size_t>(h - nh) * page_tokens * hd;
        *reinterpret_cast<uint4*>(dst + i0) = olo;
        *reinterpret_cast<uint4*>(dst + half + i0) = ohi;
    }
    if (!write_kv) return;
    const bf16* vsrc = src + static_cast<size_t>(nh + nkv) * hd;
    bf16* vbase = kbase + static_cast<size_t>(nkv) * page_tokens * hd;
    for (int it = threadIdx.x; it < nkv * (hd / 8); it += blockDim.x) {
        const int h = it / (hd / 8), d = (it % (hd / 8)) * 8;
        *reinterpret_cast<uint4*>(vbase + static_cast<size_t>(h) * page_tokens * hd + d) =
            *reinterpret_cast<const uint4*>(vsrc + h * hd + d);
    }
}

extern "C" int locus_rope_kv_write(const void* qkv, int dt, const int* positions,
                                   const float* inv_freq, void* q_out, void* pool,
                                   const int* slots, int T, int nh, int nkv, int hd, int rot_dim,
                                   int pairing, int page_tokens, int write_kv,
                                   cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || (pairing != 0 && pairing != 1) || rot_dim > 512)
        return LOCUS_ERR_UNSUPPORTED;
    if (dt == LOCUS_DT_BF16 && inv_freq != nullptr && pairing == 0 && rot_dim == hd && hd % 16 == 0 && hd <= 256 &&
        ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(pool)) & 15) == 0) {
        locus_launch(rope_kv_write_bf16_kernel, T, 256, 0, stream, static_cast<const bf16*>(qkv), positions, inv_freq,
                     static_cast<bf16*>(q_out), static_cast<bf16*>(pool), slots, nh, nkv, hd, page_tokens, write_kv);
        return locus_launch_status();
    }
    if (dt == LOCUS_DT_F32) {
        rope_kv_write_kernel<float><<<T, 256, 0, stream>>>(
            static_cast<const float*>(qkv), positions, inv_freq, static_cast<float*>(q_out),
            static_cast<float*>(pool), slots, nh, nkv, hd, rot_dim, pairing, page_tokens, write_kv);
    } else if (dt == LOCUS_DT_BF16) {
        rope_kv_write_kernel<bf16><<<T, 256, 0, stream>>>(
            static_cast<const bf16*>(qkv), positions, inv_freq, static_cast<bf16*>(q_out),
            static_cast<bf16*>(pool), slots, nh, nkv, hd, rot_dim, pairing, page_tokens, write_kv);
    } else {
        return LOCUS_ERR_UNSUPPORTED;
    }
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Routed-expert combine: x[t, :] += sum over slot = 0..k-1 (in that order) of
// pair_out[pair_pos[t * k + slot], :].  The routing weight is already applied to
// pair_out.  No atomics: the sum order is the selection order, for every batch.
template <typename TP>
__global__ void moe_combine_kernel(float* __restrict__ x, const TP* __restrict__ pair_out,
                                   const int* __restrict__ pair_pos, int k, int H) {
    pdl_entry();
    pdl_trigger();
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < k; ++s) {
            acc += to_f(pair_out[static_cast<size_t>(pair_pos[t * k + s]) * H + j]);
        }
        x[static_cast<size_t>(t) * H + j] += acc;
    }
}

// pair_out: float32 or bfloat16 rows (pair_dt); the sum is float32 either way.
extern "C" int locus_moe_combine(float* x, const void* pair_out, int pair_dt, const int* pair_pos, int T,
                                 int k, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (pair_dt == LOCUS_DT_F32)
        locus_launch(moe_combine_kernel<float>, T, 256, 0, stream, x, static_cast<const float*>(pair_out), pair_pos, k, H);
    else if (pair_dt == LOCUS_DT_BF16)
        locus_launch(moe_combine_kernel<bf16>, T, 256, 0, stream, x, static_cast<const bf16*>(pair_out), pair_pos, k, H);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Row gather: out[i, :] = src[idx[i] / div, :]  (used to lay tokens out in expert order).
template <typename TA>
__global__ void gather_rows_kernel(const TA* __restrict__ src, const int* __restrict__ idx, int div,
                                   TA* __restrict__ out, int W) {
    const int i = blockIdx.x;
    const TA* s = src + static_cast<size_t>(idx[i] / div) * W;
    TA* o = out + static_cast<size_t>(i) * W;
    for (int j = threadIdx.x; j < W; j += blockDim.x) o[j] = s[j];
}

// The same in 16-byte pieces (rows that start on 16-byte boundaries and are a multiple of 16 bytes long).
__global__ void gather_rows16_kernel(const uint4* __restrict__ src, const int* __restrict__ idx, int div,
                                     uint4* __restrict__ out, int W16) {
    const int i = blockIdx.x;
    const uint4* s = src + static_cast<size_t>(idx[i] / div) * W16;
    uint4* o = out + static_cast<size_t>(i) * W16;
    for (int j = threadIdx.x; j < W16; j += blockDim.x) o[j] = s[j];
}

extern "C" int locus_gather_rows(const void* src, int dt, const int* idx, int div, void* out,
                                 int n, int W, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (div <= 0) return LOCUS_ERR_UNSUPPORTED;
    const size_t row_bytes = static_cast<size_t>(W) * (dt == LOCUS_DT_F32 ? 4 : 2);
    if ((dt == LOCUS_DT_F32 || dt == LOCUS_DT_BF16) && row_bytes % 16 == 0 &&
        ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        const int W16 = static_cast<int>(row_bytes / 16);
        gather_rows16_kernel<<<n, W16 < 256 ? 128 : 256, 0, stream>>>(static_cast<const uint4*>(src), idx, div,
                                                                  static_cast<uint4*>(out), W16);
        return locus_launch_status();
    }
    if (dt == LOCUS_DT_F32) {
        gather_rows_kernel<float><<<n, 256, 0, stream>>>(static_cast<const float*>(src), idx, div,
                                                         static_cast<float*>(out), W);
    } else if (dt == LOCUS_DT_BF16) {
        gather_rows_kernel<bf16><<<n, 256, 0, stream>>>(static_cast<const bf16*>(src), idx, div,
                                                        static_cast<bf16*>(out), W);
    } else {
        return LOCUS_ERR_UNSUPPORTED;
    }
    return locus_launch_status();
}
