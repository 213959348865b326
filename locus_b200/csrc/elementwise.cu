// Memory-bound row kernels: embedding gather, RMSNorm, rotary position encoding fused
// with the write of K and V into cache pages, and the slot-ordered sum of routed-expert
// outputs into the residual stream.  All statistics, angles and sums are float32.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = table[tokens[t], :] as float32 (the residual stream is float32).
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const void* __restrict__ table,
                                  int table_dt, float* __restrict__ out, int H, int copies, float scale) {
    pdl_entry();
    pdl_trigger();
    const int t = blockIdx.x;
    const size_t row = static_cast<size_t>(tokens[t]) * H;
    float* o = out + static_cast<size_t>(t) * H * copies;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = ld_dyn(table, table_dt, row + i) * scale;
        for (int c = 0; c < copies; ++c) o[c * H + i] = v;
    }
}

// scale: a factor on the row (1: none).  copies > 1: a row of out holds the table's row that many times, one behind the other (a model that keeps
// several copies of the residual stream starts them all from the embedding).
extern "C" int locus_embed_rows(const int* tokens, const void* table, int table_dt, float* out,
                                int T, int H, int copies, float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (copies < 1) return LOCUS_ERR_UNSUPPORTED;
    locus_launch(embed_rows_kernel, T, 256, 0, stream, tokens, table, table_dt, out, H, copies, scale);
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

// ---------------------------------------------------------------------------
// Rows of the float32 residual stream in another element type: out[i, :] = x[i, :] (a sublayer that
// reads the stream itself, without a norm in front of it, takes its rounding to the model's type).
template <typename TO>
__global__ void __launch_bounds__(256) cast_rows_kernel(const float* __restrict__ x, TO* __restrict__ out,
                                                        long long n4, long long n) {
    pdl_entry();
    pdl_trigger();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n4) {
        const float4 v = reinterpret_cast<const float4*>(x)[i];
        put4(out + 4 * i, v.x, v.y, v.z, v.w);
    }
    if (i == 0)
        for (long long j = 4 * n4; j < n; ++j) out[j] = from_f<TO>(x[j]);
}

extern "C" int locus_cast_rows(const float* x, void* out, int out_dt, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) return LOCUS_ERR_UNSUPPORTED;
    const long long n4 = n / 4;
    const long long blocks = (n4 > 0 ? n4 : 1) / 256 + 1;
    if (blocks > 0x7fffffffLL) return LOCUS_ERR_UNSUPPORTED;
    if (out_dt == LOCUS_DT_BF16)
        locus_launch(cast_rows_kernel<bf16>, static_cast<int>(blocks), 256, 0, stream, x, static_cast<bf16*>(out), n4, n);
    else if (out_dt == LOCUS_DT_F32)
        locus_launch(cast_rows_kernel<float>, static_cast<int>(blocks), 256, 0, stream, x, static_cast<float*>(out), n4, n);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// The norm of a sublayer's OUTPUT, added to the residual stream: x[i, :] += y[i, :] * rsqrt(mean(y[i]^2) + eps) * w
// (y and x float32, statistics float32, the sum of squares in an order that depends on H only).  One block per
// row; a row of up to 4096 elements stays in registers between the two passes.
template <typename TW>
__global__ void __launch_bounds__(256) rmsnorm_add_kernel(const float* __restrict__ y, const TW* __restrict__ w,
                                                          float eps, float* __restrict__ x, int H) {
    __shared__ float warp_part[8];
    __shared__ float scale_s;
    pdl_entry();
    pdl_trigger();
    const size_t base = static_cast<size_t>(blockIdx.x) * H;
    float v[16];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 16; ++u) {
        const int j = threadIdx.x + u * 256;
        v[u] = j < H ? y[base + j] : 0.f;
        ss = fmaf(v[u], v[u], ss);
    }
    for (int j = threadIdx.x + 4096; j < H; j += 256) {
        const float t = y[base + j];
        ss = fmaf(t, t, ss);
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
#pragma unroll
    for (int u = 0; u < 16; ++u) {
        const int j = threadIdx.x + u * 256;
        if (j < H) x[base + j] += v[u] * scale * to_f(w[j]);
    }
    for (int j = threadIdx.x + 4096; j < H; j += 256) x[base + j] += y[base + j] * scale * to_f(w[j]);
}

extern "C" int locus_rmsnorm_add(const float* y, const void* w, int w_dt, float eps, float* x, int n_rows, int H,
                                 cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0) return LOCUS_ERR_UNSUPPORTED;
    if (w_dt == LOCUS_DT_BF16)
        locus_launch(rmsnorm_add_kernel<bf16>, n_rows, 256, 0, stream, y, static_cast<const bf16*>(w), eps, x, H);
    else if (w_dt == LOCUS_DT_F32)
        locus_launch(rmsnorm_add_kernel<float>, n_rows, 256, 0, stream, y, static_cast<const float*>(w), eps, x, H);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Layer norm with weight and bias over a weighted sum of S copies of the residual stream:
//     u = sum_s coef[s] x[r, s, :]   (coef null: the plain sum; S = 1 and coef null: the row itself)
//     out[i, :] = (u - mean(u)) / sqrt(mean((u - mean)^2) + eps) * w + b,      r = rows ? rows[i] : i.
// x [n, S, H] float32.  One block per row; the mean first, then the squared deviations from it; every sum in an order
// that depends on H alone.
#define LN_MAX_STREAMS 8

__device__ __forceinline__ float block_sum_256(float v, float* part) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    __syncthreads();  // part may still be read from the call before
    if (lane == 0) part[wid] = v;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < 8; ++k) tot += part[k];
    return tot;
}

template <typename TO>
__global__ void __launch_bounds__(256) layernorm_kernel(const float* __restrict__ x, int S,
                                                        const float* __restrict__ coef, const void* __restrict__ w,
                                                        const void* __restrict__ b, int w_dt, float eps,
                                                        TO* __restrict__ out, const int* __restrict__ rows, int H) {
    __shared__ float part[8];
    pdl_entry();
    pdl_trigger();
    const int i = blockIdx.x;
    const float* src = x + static_cast<size_t>(rows ? rows[i] : i) * S * H;
    float cf[LN_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < LN_MAX_STREAMS; ++s) cf[s] = s < S ? (coef ? coef[s] : 1.0f) : 0.f;
    auto u_at = [&](int j) {
        float u = cf[0] * src[j];
#pragma unroll
        for (int s = 1; s < LN_MAX_STREAMS; ++s)
            if (s < S) u = fmaf(cf[s], src[static_cast<size_t>(s) * H + j], u);
        return u;
    };
    float sum = 0.f;
    for (int j = threadIdx.x; j < H; j += 256) sum += u_at(j);
    const float mean = block_sum_256(sum, part) / static_cast<float>(H);
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += 256) {
        const float dlt = u_at(j) - mean;
        ss = fmaf(dlt, dlt, ss);
    }
    const float scale = 1.0f / sqrtf(block_sum_256(ss, part) / static_cast<float>(H) + eps);
    TO* dst = out + static_cast<size_t>(i) * H;
    for (int j = threadIdx.x; j < H; j += 256)
        dst[j] = from_f<TO>(fmaf((u_at(j) - mean) * scale, ld_dyn(w, w_dt, j), ld_dyn(b, w_dt, j)));
}

extern "C" int locus_layernorm(const float* x, int n_streams, const float* coef, const void* w, const void* b, int w_dt,
                               float eps, void* out, int out_dt, const int* rows, int n, int H, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (n_streams < 1 || n_streams > LN_MAX_STREAMS || H <= 0) return LOCUS_ERR_UNSUPPORTED;
    if (out_dt == LOCUS_DT_BF16)
        locus_launch(layernorm_kernel<bf16>, n, 256, 0, stream, x, n_streams, coef, w, b, w_dt, eps,
                     static_cast<bf16*>(out), rows, H);
    else if (out_dt == LOCUS_DT_F32)
        locus_launch(layernorm_kernel<float>, n, 256, 0, stream, x, n_streams, coef, w, b, w_dt, eps,
                     static_cast<float*>(out), rows, H);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// The write-back of a sublayer's output y into S copies of the residual stream, which are mixed among themselves
// in the same pass:  x[r, t, :] <- sum_s mix[s, t] x[r, s, :] + out_coef[t] * y[r, :]   (all t at once from the old
// copies; mix is indexed [from, to]).  S = 1, mix = [1]: x += out_coef[0] * y.
__global__ void __launch_bounds__(256) stream_update_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                            const float* __restrict__ mix,
                                                            const float* __restrict__ out_coef, int S, int H) {
    __shared__ float m_s[LN_MAX_STREAMS * LN_MAX_STREAMS], c_s[LN_MAX_STREAMS];
    pdl_entry();
    pdl_trigger();
    if (threadIdx.x < S * S) m_s[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < S) c_s[threadIdx.x] = out_coef[threadIdx.x];
    __syncthreads();
    float* xr = x + static_cast<size_t>(blockIdx.x) * S * H;
    const float* yr = y + static_cast<size_t>(blockIdx.x) * H;
    for (int j = threadIdx.x; j < H; j += 256) {
        float old[LN_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < LN_MAX_STREAMS; ++s) old[s] = s < S ? xr[static_cast<size_t>(s) * H + j] : 0.f;
        const float yv = yr[j];
#pragma unroll
        for (int t = 0; t < LN_MAX_STREAMS; ++t) {
            if (t < S) {
                float v = c_s[t] * yv;
#pragma unroll
                for (int s = 0; s < LN_MAX_STREAMS; ++s)
                    if (s < S) v = fmaf(m_s[s * S + t], old[s], v);
                xr[static_cast<size_t>(t) * H + j] = v;
            }
        }
    }
}

extern "C" int locus_stream_update(float* x, const float* y, const float* mix, const float* out_coef, int n_streams,
                                   int n, int H, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (n_streams < 1 || n_streams > LN_MAX_STREAMS || H <= 0) return LOCUS_ERR_UNSUPPORTED;
    locus_launch(stream_update_kernel, n, 256, 0, stream, x, y, mix, out_coef, n_streams, H);
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Embedding with a second table addressed by a hash of the previous and the current token:
//     out[t, :] = table[tok_t, :] + pair[r_t, :],   r_t = (prev_t * mul_prev + tok_t * mul_cur) mod buckets,
// where prev_t is the token before tok_t in its request and r_t = buckets (the table's last row) for a request's first
// token.  A segment's first token finds its predecessor in the request's state slot (`last` [n_slots, ld] int32, the
// token that the step before ended on) unless it stands at position 0.  The hash is formed in 64-bit integers.  A second
// small launch (pair_state_kernel) writes every segment's last token into its slot: it must not run beside the reads.
#define EP_TOKENS 4   // tokens of a segment per block

__global__ void __launch_bounds__(256) embed_pair_kernel(
    const int* __restrict__ tokens, const int* __restrict__ positions, const void* __restrict__ table,
    const void* __restrict__ pair, int table_dt, float* __restrict__ out, const int* __restrict__ seg_q0,
    const int* __restrict__ seg_qn, const int* __restrict__ state_slots, const int* __restrict__ last, long long last_ld,
    int H, long long buckets, long long mul_prev, long long mul_cur) {
    pdl_entry();
    pdl_trigger();
    const int seg = blockIdx.y, qn = seg_qn[seg], q0 = seg_q0[seg];
    for (int i = blockIdx.x * EP_TOKENS; i < min(qn, (blockIdx.x + 1) * EP_TOKENS); ++i) {
        const int t = q0 + i;
        const long long tok = tokens[t];
        long long r = buckets;
        if (positions[t] > 0) {
            const long long prev = i > 0 ? tokens[t - 1] : last[static_cast<size_t>(state_slots[seg]) * last_ld];
            r = (prev * mul_prev + tok * mul_cur) % buckets;
        }
        const size_t row = static_cast<size_t>(tok) * H, prow = static_cast<size_t>(r) * H;
        float* o = out + static_cast<size_t>(t) * H;
        for (int j = threadIdx.x; j < H; j += 256) o[j] = ld_dyn(table, table_dt, row + j) + ld_dyn(pair, table_dt, prow + j);
    }
}

__global__ void pair_state_kernel(const int* __restrict__ tokens, const int* __restrict__ seg_q0,
                                  const int* __restrict__ seg_qn, const int* __restrict__ state_slots,
                                  int* __restrict__ last, long long last_ld, int n_seg) {
    pdl_entry();
    pdl_trigger();
    const int seg = blockIdx.x * blockDim.x + threadIdx.x;
    if (seg < n_seg && seg_qn[seg] > 0)
        last[static_cast<size_t>(state_slots[seg]) * last_ld] = tokens[seg_q0[seg] + seg_qn[seg] - 1];
}

extern "C" int locus_embed_pair(const int* tokens, const int* positions, const void* table, const void* pair, int table_dt,
                                float* out, const int* seg_q0, const int* seg_qn, const int* state_slots, int* last,
                                long long last_ld, int n_seg, int longest_new, int H, long long buckets, long long mul_prev,
                                long long mul_cur, cudaStream_t stream) {
    if (n_seg <= 0 || longest_new <= 0) return 0;
    if (buckets <= 0 || mul_prev < 0 || mul_cur < 0 || n_seg > 65535 || H <= 0) return LOCUS_ERR_UNSUPPORTED;
    locus_launch(embed_pair_kernel, dim3((longest_new + EP_TOKENS - 1) / EP_TOKENS, n_seg), dim3(256), 0, stream, tokens,
                 positions, table, pair, table_dt, out, seg_q0, seg_qn, state_slots, static_cast<const int*>(last), last_ld,
                 H, buckets, mul_prev, mul_cur);
    locus_launch(pair_state_kernel, dim3((n_seg + 63) / 64), dim3(64), 0, stream, tokens, seg_q0, seg_qn, state_slots, last,
                 last_ld, n_seg);
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// The norm of a post-norm layer, in place on the float32 residual stream:
//     u = alpha * x[i, :] + y[i, :];    x[i, :] = (u - mean(u)) / sqrt(mean((u - mean)^2) + eps) * w + b,
// and, when `cast` is given, the new row once more in that buffer's element type (what the next sublayer reads).
// One block per row; the mean first, then the squared deviations; every sum in an order that depends on H alone.
template <typename TC>
__global__ void __launch_bounds__(256) layernorm_post_kernel(float* __restrict__ x, const float* __restrict__ y, float alpha,
                                                             const void* __restrict__ w, const void* __restrict__ b,
                                                             int w_dt, float eps, TC* __restrict__ cast, int H) {
    __shared__ float part[8];
    pdl_entry();
    pdl_trigger();
    float* xr = x + static_cast<size_t>(blockIdx.x) * H;
    const float* yr = y + static_cast<size_t>(blockIdx.x) * H;
    auto u_at = [&](int j) { return fmaf(alpha, xr[j], yr[j]); };
    float sum = 0.f;
    for (int j = threadIdx.x; j < H; j += 256) sum += u_at(j);
    const float mean = block_sum_256(sum, part) / static_cast<float>(H);
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += 256) {
        const float dlt = u_at(j) - mean;
        ss = fmaf(dlt, dlt, ss);
    }
    const float scale = 1.0f / sqrtf(block_sum_256(ss, part) / static_cast<float>(H) + eps);
    for (int j = threadIdx.x; j < H; j += 256) {
        const float v = fmaf((u_at(j) - mean) * scale, ld_dyn(w, w_dt, j), ld_dyn(b, w_dt, j));
        xr[j] = v;
        if (cast) cast[static_cast<size_t>(blockIdx.x) * H + j] = from_f<TC>(v);
    }
}

extern "C" int locus_layernorm_post(float* x, const float* y, float alpha, const void* w, const void* b, int w_dt, float eps,
                                    void* cast, int cast_dt, int n, int H, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (H <= 0) return LOCUS_ERR_UNSUPPORTED;
    if (cast != nullptr && cast_dt == LOCUS_DT_BF16)
        locus_launch(layernorm_post_kernel<bf16>, n, 256, 0, stream, x, y, alpha, w, b, w_dt, eps, static_cast<bf16*>(cast), H);
    else if (cast == nullptr || cast_dt == LOCUS_DT_F32)
        locus_launch(layernorm_post_kernel<float>, n, 256, 0, stream, x, y, alpha, w, b, w_dt, eps, static_cast<float*>(cast), H);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// RMS norm in place over up to two spans of columns of float32 rows, each span with a weight of its own:
//     x[t, off : off + n] <- x[t, off : off + n] / sqrt(mean(x[t, off : off + n]^2) + eps) * w.
// (A norm over a whole projection, all heads at once, of a row that holds several projections.)  Block (t, span).
__global__ void __launch_bounds__(256) span_rmsnorm_kernel(float* __restrict__ x, int ld, int off0, int n0,
                                                           const void* __restrict__ w0, int off1, int n1,
                                                           const void* __restrict__ w1, int w_dt, float eps) {
    __shared__ float part[8];
    pdl_entry();
    pdl_trigger();
    const int off = blockIdx.y ? off1 : off0, n = blockIdx.y ? n1 : n0;
    const void* w = blockIdx.y ? w1 : w0;
    float* xr = x + static_cast<size_t>(blockIdx.x) * ld + off;
    float ss = 0.f;
    for (int j = threadIdx.x; j < n; j += 256) ss = fmaf(xr[j], xr[j], ss);
    const float scale = 1.0f / sqrtf(block_sum_256(ss, part) / static_cast<float>(n) + eps);
    for (int j = threadIdx.x; j < n; j += 256) xr[j] = xr[j] * scale * ld_dyn(w, w_dt, j);
}

extern "C" int locus_span_rmsnorm(float* x, int ld, int T, int off0, int n0, const void* w0, int off1, int n1, const void* w1,
                                  int w_dt, float eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n0 <= 0 || off0 < 0 || off0 + n0 > ld || (w1 != nullptr && (n1 <= 0 || off1 < 0 || off1 + n1 > ld)))
        return LOCUS_ERR_UNSUPPORTED;
    locus_launch(span_rmsnorm_kernel, dim3(T, w1 != nullptr ? 2 : 1), dim3(256), 0, stream, x, ld, off0, n0, w0, off1, n1, w1,
                 w_dt, eps);
    return locus_launch_status();
}
