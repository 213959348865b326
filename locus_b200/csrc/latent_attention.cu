// Latent attention: queries and keys/values that go through low-rank latents, one latent row per token in
// the paged cache, shared by all heads.
//
// Per token the mixer keeps a row of R = kv_rank + rot_dim elements: the normed latent c (kv_rank) and one
// rotated key part (rot_dim) that all heads share.  A head's unrotated key is W_uk[h] c and its value
// W_uv[h] c, so the score of query (t, h) against key j is
//
//     s = ((W_uk[h]^T q_nope) . c_j + q_rot . k_rot_j) * scale
//
// and the head's output W_uv[h] (sum_j p_j c_j): with the query carried into the latent space first
// ("absorbed"), attention runs over the cached rows as they are, as one key/value head of width R (keys) and
// kv_rank (values = the first kv_rank elements of the same row) for all query heads, and nothing per head is
// ever expanded per key.  The two per-head products are grouped products of the framework (the heads take
// the place of experts); for them the queries and the attention output are laid out head-major,
// [head][token][...].
//
// Kernels of this file:
//   latent_prep     norms of the two latents, rotation of the shared key part, cache write (one pass over
//                   the down-projection's output)
//   latent_q_split  the up-projected query: unrotated parts to head-major rows, rotated parts turned
//   latent_attn     attention over the latent rows, float32 arithmetic: a sliding window (a query at position p
//                   sees p - window < j <= p; 0 = all), and a sink per head: exp(sink[h]) joins the softmax's
//                   denominator, without a key or a value
//   heads_to_rows   [head][token][d] -> [token][head * d]
//
// Angles: position * frequency and its sine and cosine are formed in float64 from float64 frequencies (the
// host computes them, ramp of a long-context scaling included) and rounded once; `magnitude` multiplies both.
// Pairs are interleaved, (2i, 2i + 1), or with `half_split` the halves of the turned stretch, (i, i + rot_pairs);
// i < rot_pairs; elements behind 2 * rot_pairs pass unchanged.  q_rank = 0: no query latent (the queries are projected
// elsewhere), the row holds the key/value side alone.
#include "common.cuh"

__device__ __forceinline__ float block_sum_256(float v, float* part) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += part[k];
    __syncthreads();
    return tot;
}

// ---------------------------------------------------------------------------
// dqkv [T, ld] float32, of which the first q_rank + kv_rank + rot_dim columns are the stacked down-projections of a
// token (write = 0: the first q_rank alone).
//   cq[t]            = rmsnorm(dqkv[t, :q_rank]) * wq                       -> cq_out [T, q_rank]
//   row[:kv_rank]    = rmsnorm(dqkv[t, q_rank : q_rank + kv_rank]) * wkv    -> the token's cache row
//   row[kv_rank:]    = rotate(dqkv[t, q_rank + kv_rank :], position)
template <typename TO, typename TW>
__global__ void __launch_bounds__(256) latent_prep_kernel(
    const float* __restrict__ dqkv, const int* __restrict__ positions, const double* __restrict__ freq,
    float magnitude, const TW* __restrict__ wq, const TW* __restrict__ wkv, float eps, TO* __restrict__ cq_out,
    TO* __restrict__ pool, const int* __restrict__ slots, int q_rank, int kv_rank, int rot_dim, int rot_pairs,
    int write, int half_split, int ld) {
    __shared__ float part[8];
    pdl_entry();
    pdl_trigger();
    const int t = blockIdx.x;
    const float* src = dqkv + static_cast<size_t>(t) * ld;
    float sq = 0.f, sk = 0.f;
    for (int j = threadIdx.x; j < q_rank; j += 256) sq = fmaf(src[j], src[j], sq);
    if (write)
        for (int j = threadIdx.x; j < kv_rank; j += 256) sk = fmaf(src[q_rank + j], src[q_rank + j], sk);
    sq = block_sum_256(sq, part);
    sk = block_sum_256(sk, part);
    const float scale_q = q_rank > 0 ? 1.0f / sqrtf(sq / static_cast<float>(q_rank) + eps) : 0.f;
    const float scale_k = 1.0f / sqrtf(sk / static_cast<float>(kv_rank) + eps);
    TO* cq = cq_out + static_cast<size_t>(t) * q_rank;
    for (int j = threadIdx.x; j < q_rank; j += 256) cq[j] = from_f<TO>(src[j] * scale_q * to_f(wq[j]));
    if (!write) return;
    TO* row = pool + static_cast<size_t>(slots[t]) * (kv_rank + rot_dim);
    for (int j = threadIdx.x; j < kv_rank; j += 256) row[j] = from_f<TO>(src[q_rank + j] * scale_k * to_f(wkv[j]));
    const float* kr = src + q_rank + kv_rank;
    const double pos = static_cast<double>(positions[t]);
    for (int i = threadIdx.x; i < rot_pairs; i += 256) {
        double s, c;
        sincos(pos * freq[i], &s, &c);
        const float cs = static_cast<float>(c) * magnitude, sn = static_cast<float>(s) * magnitude;
        const int i0 = half_split ? i : 2 * i, i1 = half_split ? i + rot_pairs : 2 * i + 1;
        const float u = kr[i0], v = kr[i1];
        row[kv_rank + i0] = from_f<TO>(u * cs - v * sn);
        row[kv_rank + i1] = from_f<TO>(v * cs + u * sn);
    }
    for (int j = 2 * rot_pairs + threadIdx.x; j < rot_dim; j += 256) row[kv_rank + j] = from_f<TO>(kr[j]);
}

extern "C" int locus_latent_prep(const float* dqkv, const int* positions, const double* freq, float magnitude,
                                 const void* wq, const void* wkv, int w_dt, float eps, void* cq_out, void* pool,
                                 int dt, const int* slots, int T, int q_rank, int kv_rank, int rot_dim,
                                 int rot_pairs, int write, int half_split, int ld, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (ld < q_rank + (write ? kv_rank + rot_dim : 0)) return LOCUS_ERR_UNSUPPORTED;
    if (q_rank < 0 || kv_rank <= 0 || rot_dim < 0 || rot_pairs < 0 || 2 * rot_pairs > rot_dim) return LOCUS_ERR_UNSUPPORTED;
    if (rot_pairs > 0 && freq == nullptr) return LOCUS_ERR_UNSUPPORTED;
#define PREP(TO, TW)                                                                                              \
    locus_launch(latent_prep_kernel<TO, TW>, T, 256, 0, stream, dqkv, positions, freq, magnitude,                  \
                 static_cast<const TW*>(wq), static_cast<const TW*>(wkv), eps, static_cast<TO*>(cq_out),           \
                 static_cast<TO*>(pool), slots, q_rank, kv_rank, rot_dim, rot_pairs, write, half_split, ld)
    if (dt == LOCUS_DT_BF16 && w_dt == LOCUS_DT_BF16) PREP(bf16, bf16);
    else if (dt == LOCUS_DT_F32 && w_dt == LOCUS_DT_F32) PREP(float, float);
    else if (dt == LOCUS_DT_F32 && w_dt == LOCUS_DT_BF16) PREP(float, bf16);
    else if (dt == LOCUS_DT_BF16 && w_dt == LOCUS_DT_F32) PREP(bf16, float);
    else return LOCUS_ERR_UNSUPPORTED;
#undef PREP
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// q [T, H * (dn + dr)], head by head [dn unrotated | dr rotated]:
//   q_nope_hm [H, T, dn]   the unrotated parts, head-major (the rows of the grouped product with W_uk^T)
//   q_rot     [T, H, dr]   the rotated parts, turned by the token's position
template <typename TA>
__global__ void __launch_bounds__(256) latent_q_split_kernel(
    const TA* __restrict__ q, const int* __restrict__ positions, const double* __restrict__ freq, float magnitude,
    TA* __restrict__ q_nope_hm, TA* __restrict__ q_rot, int T, int H, int dn, int dr, int rot_pairs, int half_split) {
    extern __shared__ float cs_tab[];  // [rot_pairs][2]
    pdl_entry();
    pdl_trigger();
    const int t = blockIdx.x;
    const double pos = static_cast<double>(positions[t]);
    for (int i = threadIdx.x; i < rot_pairs; i += 256) {
        double s, c;
        sincos(pos * freq[i], &s, &c);
        cs_tab[2 * i] = static_cast<float>(c) * magnitude;
        cs_tab[2 * i + 1] = static_cast<float>(s) * magnitude;
    }
    __syncthreads();
    const int hw = dn + dr;
    const TA* src = q + static_cast<size_t>(t) * H * hw;
    for (int i = threadIdx.x; i < H * dn; i += 256) {
        const int h = i / dn, d = i % dn;
        q_nope_hm[(static_cast<size_t>(h) * T + t) * dn + d] = src[h * hw + d];
    }
    TA* dst = q_rot + static_cast<size_t>(t) * H * dr;
    if (half_split) {
        // element e < rot_pairs is the first of its pair, rot_pairs <= e < 2 rot_pairs the second; the rest pass
        for (int i = threadIdx.x; i < H * dr; i += 256) {
            const int h = i / dr, e = i % dr;
            const TA* hs = src + h * hw + dn;
            float val = to_f(hs[e]);
            if (e < 2 * rot_pairs) {
                const int p = e < rot_pairs ? e : e - rot_pairs;
                const float u = to_f(hs[p]), v = to_f(hs[p + rot_pairs]);
                const float cs = cs_tab[2 * p], sn = cs_tab[2 * p + 1];
                val = e < rot_pairs ? u * cs - v * sn : v * cs + u * sn;
            }
            dst[i] = from_f<TA>(val);
        }
        return;
    }
    const int half = dr / 2;  // pairs of a head, turned or not
    for (int i = threadIdx.x; i < H * half; i += 256) {
        const int h = i / half, p = i % half;
        const float u = to_f(src[h * hw + dn + 2 * p]), v = to_f(src[h * hw + dn + 2 * p + 1]);
        float a = u, b = v;
        if (p < rot_pairs) {
            const float cs = cs_tab[2 * p], sn = cs_tab[2 * p + 1];
            a = u * cs - v * sn;
            b = v * cs + u * sn;
        }
        dst[h * dr + 2 * p] = from_f<TA>(a);
        dst[h * dr + 2 * p + 1] = from_f<TA>(b);
    }
    if (dr & 1)
        for (int h = threadIdx.x; h < H; h += 256) dst[h * dr + dr - 1] = src[h * hw + dn + dr - 1];
}

extern "C" int locus_latent_q_split(const void* q, int dt, const int* positions, const double* freq,
                                    float magnitude, void* q_nope_hm, void* q_rot, int T, int H, int dn, int dr,
                                    int rot_pairs, int half_split, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dn <= 0 || dr < 0 || rot_pairs < 0 || 2 * rot_pairs > dr) return LOCUS_ERR_UNSUPPORTED;
    if (rot_pairs > 0 && freq == nullptr) return LOCUS_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * 2 * (rot_pairs > 0 ? rot_pairs : 1);
    if (smem > 48 * 1024) return LOCUS_ERR_UNSUPPORTED;
    if (dt == LOCUS_DT_BF16)
        locus_launch(latent_q_split_kernel<bf16>, T, 256, smem, stream, static_cast<const bf16*>(q), positions, freq,
                     magnitude, static_cast<bf16*>(q_nope_hm), static_cast<bf16*>(q_rot), T, H, dn, dr, rot_pairs, half_split);
    else if (dt == LOCUS_DT_F32)
        locus_launch(latent_q_split_kernel<float>, T, 256, smem, stream, static_cast<const float*>(q), positions, freq,
                     magnitude, static_cast<float*>(q_nope_hm), static_cast<float*>(q_rot), T, H, dn, dr, rot_pairs, half_split);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// src [H, T, d] -> out [T, H * d]
template <typename TA>
__global__ void __launch_bounds__(256) heads_to_rows_kernel(const TA* __restrict__ src, TA* __restrict__ out, int T,
                                                            int H, int d) {
    pdl_entry();
    pdl_trigger();
    const int t = blockIdx.x;
    TA* dst = out + static_cast<size_t>(t) * H * d;
    for (int i = threadIdx.x; i < H * d; i += 256) {
        const int h = i / d, e = i % d;
        dst[i] = src[(static_cast<size_t>(h) * T + t) * d + e];
    }
}

extern "C" int locus_heads_to_rows(const void* src, int dt, void* out, int T, int H, int d, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || d <= 0) return LOCUS_ERR_UNSUPPORTED;
    if (dt == LOCUS_DT_BF16)
        locus_launch(heads_to_rows_kernel<bf16>, T, 256, 0, stream, static_cast<const bf16*>(src), static_cast<bf16*>(out), T, H, d);
    else if (dt == LOCUS_DT_F32)
        locus_launch(heads_to_rows_kernel<float>, T, 256, 0, stream, static_cast<const float*>(src), static_cast<float*>(out), T, H, d);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Attention over the latent rows on the CUDA cores, float32 arithmetic throughout.
struct LatentArgs {
    const void* q_abs;       // [H, T, kv_rank] head-major: the unrotated queries carried into the latent space
    const void* q_rot;       // [T, H, rot_dim]
    const void* pool;        // this layer's pages: [n_pages][page_tokens][kv_rank + rot_dim]
    const float* sink;       // [H] or null
    void* out;               // [H, T, kv_rank] head-major: sum_j p_j c_j
    const int* seg_q0;
    const int* seg_qn;
    const int* seg_ctx;
    const int* block_table;  // [n_seg, table_stride]; entries behind a window may be -1
    int table_stride;
    const int* items;        // [n_items, 2] (segment, first query of a tile of LAT_BQ queries within it)
    int T, H, kv_rank, rot_dim, page_tokens, window;
    float scale;
};

#define LAT_BQ 16
#define LAT_TK 32

template <typename T, int NACC>
__global__ void __launch_bounds__(128) latent_attn_kernel(LatentArgs a) {
    extern __shared__ float smem[];
    const int kvr = a.kv_rank, R = a.kv_rank + a.rot_dim;
    float* qs = smem;                            // [BQ][R]
    float* ks = qs + LAT_BQ * R;                 // [TK][R + 1]
    float* sc = ks + LAT_TK * (R + 1);           // [BQ][TK + 1]
    float* m_s = sc + LAT_BQ * (LAT_TK + 1);     // [BQ]
    float* l_s = m_s + LAT_BQ;                   // [BQ]
    float* al_s = l_s + LAT_BQ;                  // [BQ]
    pdl_entry();
    pdl_trigger();
    // the late tiles of a prompt see the most keys: the grid takes them first, for all heads (its fast index)
    const int item = gridDim.y - 1 - blockIdx.y;
    const int seg = a.items[2 * item], qoff = a.items[2 * item + 1];
    const int h = blockIdx.x;
    const int nq = min(LAT_BQ, a.seg_qn[seg] - qoff);
    const int row0 = a.seg_q0[seg] + qoff;
    const int p0 = a.seg_ctx[seg] + qoff;  // position of the tile's first query
    const int* table = a.block_table + static_cast<size_t>(seg) * a.table_stride;
    const int tid = threadIdx.x;
    const T* qa = static_cast<const T*>(a.q_abs) + (static_cast<size_t>(h) * a.T + row0) * kvr;
    const T* qr = static_cast<const T*>(a.q_rot);
    for (int i = tid; i < LAT_BQ * R; i += 128) {
        const int qi = i / R, d = i % R;
        float v = 0.f;
        if (qi < nq)
            v = d < kvr ? to_f(qa[static_cast<size_t>(qi) * kvr + d])
                        : to_f(qr[(static_cast<size_t>(row0 + qi) * a.H + h) * a.rot_dim + (d - kvr)]);
        qs[i] = v;
    }
    if (tid < LAT_BQ) {
        // the sink is a score of its own in the denominator: the running maximum starts at it, with weight 1
        const bool has = a.sink != nullptr;
        m_s[tid] = has ? a.sink[h] : -INFINITY;
        l_s[tid] = has ? 1.f : 0.f;
    }
    const int t_hi = p0 + nq - 1;
    const int t_lo = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
    const int my_q = tid >> 3, dl = tid & 7;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    __syncthreads();

    for (int tile0 = (t_lo / LAT_TK) * LAT_TK; tile0 <= t_hi; tile0 += LAT_TK) {
        for (int i = tid; i < LAT_TK * R; i += 128) {
            const int kj = i / R, d = i % R;
            const int t = tile0 + kj;
            float kv = 0.f;
            if (t >= t_lo && t <= t_hi) {
                const size_t slot = static_cast<size_t>(table[t / a.page_tokens]) * a.page_tokens + t % a.page_tokens;
                kv = to_f(static_cast<const T*>(a.pool)[slot * R + d]);
            }
            ks[kj * (R + 1) + d] = kv;
        }
        __syncthreads();
        for (int i = tid; i < LAT_BQ * LAT_TK; i += 128) {
            const int qi = i / LAT_TK, kj = i % LAT_TK;
            const int t = tile0 + kj, p = p0 + qi;
            float s = -INFINITY;
            if (qi < nq && t <= p && t >= t_lo && (a.window == 0 || t > p - a.window)) {
                float dot = 0.f;
                const float* qrow = qs + qi * R;
                const float* krow = ks + kj * (R + 1);
                for (int d = 0; d < R; ++d) dot = fmaf(qrow[d], krow[d], dot);
                s = dot * a.scale;
            }
            sc[qi * (LAT_TK + 1) + kj] = s;
        }
        __syncthreads();
        if (tid < LAT_BQ) {
            float* row = sc + tid * (LAT_TK + 1);
            float mx = m_s[tid];
            for (int kj = 0; kj < LAT_TK; ++kj) mx = fmaxf(mx, row[kj]);
            float alpha = 1.f, sum = 0.f;
            if (mx == -INFINITY) {
                for (int kj = 0; kj < LAT_TK; ++kj) row[kj] = 0.f;
            } else {
                alpha = expf(m_s[tid] - mx);  // exp(-inf) = 0 on the first live tile
                for (int kj = 0; kj < LAT_TK; ++kj) {
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
            const float* prow = sc + my_q * (LAT_TK + 1);
#pragma unroll
            for (int dd = 0; dd < NACC; ++dd) {
                const int d = dl + 8 * dd;
                if (d < kvr) {
                    float v = acc[dd] * alpha;
                    for (int kj = 0; kj < LAT_TK; ++kj) v = fmaf(prow[kj], ks[kj * (R + 1) + d], v);
                    acc[dd] = v;
                }
            }
        }
        __syncthreads();
    }
    if (my_q < nq) {
        const float inv = 1.0f / l_s[my_q];
        T* o = static_cast<T*>(a.out) + (static_cast<size_t>(h) * a.T + row0 + my_q) * kvr;
#pragma unroll
        for (int dd = 0; dd < NACC; ++dd) {
            const int d = dl + 8 * dd;
            if (d < kvr) o[d] = from_f<T>(acc[dd] * inv);
        }
    }
}

template <typename T, int NACC>
static int launch_latent(const LatentArgs& a, int n_items, size_t smem, cudaStream_t stream) {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(latent_attn_kernel<T, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
        return LOCUS_ERR_UNSUPPORTED;
    locus_launch(latent_attn_kernel<T, NACC>, dim3(a.H, n_items), dim3(128), smem, stream, a);
    return locus_launch_status();
}

// window: 0 = every earlier key.  sink: float32 [H] or null.  kv_rank up to 512, rows of up to 640 elements.
extern "C" int locus_latent_attn(const void* q_abs, const void* q_rot, int dt, const void* pool, const float* sink,
                                 void* out, const int* seg_q0, const int* seg_qn, const int* seg_ctx,
                                 const int* block_table, int table_stride, const int* items, int n_items, int T,
                                 int H, int kv_rank, int rot_dim, int page_tokens, int window, float scale,
                                 cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (H <= 0 || kv_rank <= 0 || kv_rank > 512 || rot_dim < 0 || page_tokens <= 0 || window < 0 || n_items > 65535)
        return LOCUS_ERR_UNSUPPORTED;
    const int R = kv_rank + rot_dim;
    const size_t smem = sizeof(float) * (static_cast<size_t>(LAT_BQ) * R + LAT_TK * (R + 1) + LAT_BQ * (LAT_TK + 1) + 3 * LAT_BQ);
    if (smem > 200 * 1024) return LOCUS_ERR_UNSUPPORTED;
    LatentArgs a;
    a.q_abs = q_abs; a.q_rot = q_rot; a.pool = pool; a.sink = sink; a.out = out; a.seg_q0 = seg_q0; a.seg_qn = seg_qn;
    a.seg_ctx = seg_ctx; a.block_table = block_table; a.table_stride = table_stride; a.items = items; a.T = T; a.H = H;
    a.kv_rank = kv_rank; a.rot_dim = rot_dim; a.page_tokens = page_tokens; a.window = window; a.scale = scale;
    const int nacc = (kv_rank + 7) / 8;
#define LATENT(TT)                                                                \
    do {                                                                          \
        if (nacc <= 8) return launch_latent<TT, 8>(a, n_items, smem, stream);     \
        if (nacc <= 16) return launch_latent<TT, 16>(a, n_items, smem, stream);   \
        if (nacc <= 32) return launch_latent<TT, 32>(a, n_items, smem, stream);   \
        return launch_latent<TT, 64>(a, n_items, smem, stream);                   \
    } while (0)
    if (dt == LOCUS_DT_BF16) LATENT(bf16);
    if (dt == LOCUS_DT_F32) LATENT(float);
#undef LATENT
    return LOCUS_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------
// The same attention on the tensor cores (bfloat16; mma.sync m16n8k16, float32 accumulation, softmax in float32).
//
// All heads read the same cache rows, so a block's 64 rows are QB queries x HB heads (HB a power of two, rows
// r -> query r / HB, head h0 + r % HB): a tile of keys is fetched into shared memory once for all of them.  Eight
// warps: warp (rg, dh) owns the rows 16 rg .. 16 rg + 15 and the half dh of a key tile for S = Q K^T, and the half
// dh of the latent's dimensions for O += P C.  Scores go through shared memory once per tile so that both warps
// of a row group see the whole tile's 32 keys: each forms the rows' running maximum and denominator itself (the
// same numbers) and multiplies its P, rounded to bfloat16, with its half of the rows' latents.  Key tiles of 32
// rows arrive by cp.async, two buffers.  kv_rank is a template parameter (32 to 512); rot_dim a multiple of 16.
#define LM_ROWS 64
#define LM_KEYS 32

struct LatentMmaArgs {
    const bf16* q_abs;
    const bf16* q_rot;
    const bf16* pool;
    const float* sink;
    bf16* out;
    const int* seg_q0;
    const int* seg_qn;
    const int* seg_ctx;
    const int* block_table;
    int table_stride;
    const int* items;        // [n_items, 2] (segment, first query of a tile of 64 >> hb_shift queries)
    int T, H, rot_dim, page_tokens, window, hb_shift;
    float scale;
    // A step with few blocks (single tokens, or a short portion, behind long contexts) cuts every block's key tiles
    // into n_splits ranges that run as blocks of their own (blockIdx.z) and leave unnormalised sums, running
    // maxima and denominators in a scratch; latent_attn_merge_kernel adds the ranges up in ascending order.
    int n_splits;
    float* part_o;    // [item][head block][split][64][kv_rank]
    float* part_ml;   // [item][head block][split][64][2]  maximum (base 2) and denominator
};

// Key tiles of an item (the same in both kernels): the first tile's first position and their number.
__device__ __forceinline__ void lm_item_tiles(int p0, int nq, int window, int& first_tile, int& n_tiles) {
    const int t_hi = p0 + nq - 1;
    const int t_lo = window > 0 ? max(0, p0 - window + 1) : 0;
    first_tile = (t_lo / LM_KEYS) * LM_KEYS;
    n_tiles = (t_hi - first_tile) / LM_KEYS + 1;
}

__device__ __forceinline__ uint32_t lm_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void lm_cp16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void lm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void lm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void lm_ldsm(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lm_ldsm_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lm_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int KVR>
__global__ void __launch_bounds__(256) latent_attn_mma_kernel(LatentMmaArgs a) {
    constexpr int DH = KVR / 2;          // latent dimensions of one warp
    constexpr int DT = DH / 8;           // its 8-wide output tiles
    const int R = KVR + a.rot_dim;
    const int LDS = R + 8;               // padded row, elements (16 bytes: ldmatrix reads no bank twice)
    const int CH = R / 8;                // 16-byte pieces of a row
    const int KS = R / 16;               // k-steps of Q K^T
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);                       // [64][LDS]
    bf16* sK = sQ + LM_ROWS * LDS;                                      // [2][32][LDS]
    float* sS = reinterpret_cast<float*>(sK + 2 * LM_KEYS * LDS);       // [64][33]
    pdl_entry();
    pdl_trigger();
    const int item = gridDim.y - 1 - blockIdx.y;   // the tiles with the most keys first
    const int seg = a.items[2 * item], qoff = a.items[2 * item + 1];
    const int HB = 1 << a.hb_shift, QB = LM_ROWS >> a.hb_shift;
    const int h0 = blockIdx.x * HB;
    const int nq = min(QB, a.seg_qn[seg] - qoff);
    const int row0 = a.seg_q0[seg] + qoff;
    const int p0 = a.seg_ctx[seg] + qoff;
    const int* table = a.block_table + static_cast<size_t>(seg) * a.table_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rg = warp & 3, dh = warp >> 2;
    const int g = lane >> 2, qd = lane & 3;
    const int t_hi = p0 + nq - 1;
    const int t_lo = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
    const int P = a.page_tokens;
    const float scale_log2 = a.scale * 1.4426950408889634f;
    int first_tile, n_tiles_all;
    lm_item_tiles(p0, nq, a.window, first_tile, n_tiles_all);
    const int split = blockIdx.z;
    const int per_split = (n_tiles_all + a.n_splits - 1) / a.n_splits;
    first_tile += split * per_split * LM_KEYS;
    const int n_tiles = max(0, min(per_split, n_tiles_all - split * per_split));
    if (n_tiles == 0) return;  // the merge counts the live ranges the same way

    // ---- the 64 query rows -> shared: [carried into the latent space | rotated part]; rows without a query are zero
    const int chq = KVR / 8;
    for (int i = tid; i < LM_ROWS * CH; i += 256) {
        const int r = i / CH, c = i % CH;
        const int qi = r >> a.hb_shift, h = h0 + (r & (HB - 1));
        const bool ok = qi < nq && h < a.H;
        const int qq = ok ? qi : 0, hh = ok ? h : h0;
        const bf16* src = c < chq ? a.q_abs + (static_cast<size_t>(hh) * a.T + row0 + qq) * KVR + c * 8
                                  : a.q_rot + (static_cast<size_t>(row0 + qq) * a.H + hh) * a.rot_dim + (c - chq) * 8;
        lm_cp16(lm_addr(sQ + r * LDS + c * 8), src, ok ? 16 : 0);
    }
    lm_commit();
    auto load_keys = [&](int tile0, int buf) {
        bf16* dk = sK + buf * LM_KEYS * LDS;
        for (int i = tid; i < LM_KEYS * CH; i += 256) {
            const int r = i / CH, c = i % CH;
            const int t = tile0 + r;
            const bool ok = t >= t_lo && t <= t_hi;
            const int tt = ok ? t : t_hi;  // any live position: nothing is copied when !ok
            const size_t slot = static_cast<size_t>(table[tt / P]) * P + tt % P;
            lm_cp16(lm_addr(dk + r * LDS + c * 8), a.pool + slot * R + c * 8, ok ? 16 : 0);
        }
        lm_commit();
    };
    load_keys(first_tile, 0);

    // this lane's two rows (g and g + 8 of the warp's 16): their positions, and whether they hold a query at all
    int pq[2];
    bool live[2];
    float m_run[2], l_run[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int r = rg * 16 + g + 8 * rr;
        const int qi = r >> a.hb_shift, h = h0 + (r & (HB - 1));
        live[rr] = qi < nq && h < a.H;
        pq[rr] = p0 + qi;
        // the sink is a score of its own in the denominator (counted once per row: by the quad's first lane of
        // the first range of keys)
        const bool has = a.sink != nullptr && live[rr] && split == 0;
        m_run[rr] = has ? a.sink[h] * 1.4426950408889634f : -INFINITY;
        l_run[rr] = (has && qd == 0) ? 1.f : 0.f;
    }
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[d][i] = 0.f;

    for (int it = 0; it < n_tiles; ++it) {
        const int tile0 = first_tile + it * LM_KEYS;
        const int buf = it & 1;
        if (it + 1 < n_tiles) {
            load_keys(tile0 + LM_KEYS, buf ^ 1);
            lm_wait<1>();
        } else {
            lm_wait<0>();
        }
        __syncthreads();
        const bf16* tK = sK + buf * LM_KEYS * LDS;
        // ---- S = Q K^T for this warp's 16 rows and its 16 keys of the tile
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
        {
            const uint32_t qa = lm_addr(sQ + (rg * 16 + (lane & 15)) * LDS + (lane >> 4) * 8);
            const uint32_t ka = lm_addr(tK + (dh * 16 + (lane & 7) + ((lane >> 4) << 3)) * LDS + ((lane >> 3) & 1) * 8);
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                lm_ldsm(qa + ks * 32, a0, a1, a2, a3);
                lm_ldsm(ka + ks * 32, b0, b1, b2, b3);
                lm_mma(s[0], a0, a1, a2, a3, b0, b1);
                lm_mma(s[1], a0, a1, a2, a3, b2, b3);
            }
        }
        // scaled (base 2) and masked scores -> shared, for both warps of the row group
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int rr = i >> 1;
                const int kcol = dh * 16 + j * 8 + qd * 2 + (i & 1);
                const int t = tile0 + kcol, p = pq[rr];
                const bool ok = live[rr] && t <= p && t >= t_lo && (a.window == 0 || t > p - a.window);
                sS[(rg * 16 + g + 8 * rr) * (LM_KEYS + 1) + kcol] = ok ? s[j][i] * scale_log2 : -INFINITY;
            }
        }
        __syncthreads();
        // ---- the rows' 32 scores in the layout of the left operand of P C
        float pz[4][4];
        float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float v = sS[(rg * 16 + g + 8 * (i >> 1)) * (LM_KEYS + 1) + j * 8 + qd * 2 + (i & 1)];
                pz[j][i] = v;
                mx[i >> 1] = fmaxf(mx[i >> 1], v);
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
        const float m0 = mx[0] == -INFINITY ? 0.f : mx[0], m1 = mx[1] == -INFINITY ? 0.f : mx[1];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float e = exp2f(pz[j][i] - ((i >> 1) ? m1 : m0));
                pz[j][i] = e;
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
        // ---- O += P C over this warp's half of the latent's dimensions
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            const uint32_t a0 = lm_pack(pz[2 * kk][0], pz[2 * kk][1]);
            const uint32_t a1 = lm_pack(pz[2 * kk][2], pz[2 * kk][3]);
            const uint32_t a2 = lm_pack(pz[2 * kk + 1][0], pz[2 * kk + 1][1]);
            const uint32_t a3 = lm_pack(pz[2 * kk + 1][2], pz[2 * kk + 1][3]);
            const uint32_t va = lm_addr(tK + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + dh * DH + (lane >> 4) * 8);
#pragma unroll
            for (int dp = 0; dp < DH / 16; ++dp) {
                uint32_t b0, b1, b2, b3;
                lm_ldsm_t(va + dp * 32, b0, b1, b2, b3);
                lm_mma(o[2 * dp], a0, a1, a2, a3, b0, b1);
                lm_mma(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();  // everyone is done with this buffer and with the scores before they are overwritten
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
        if (!live[rr]) continue;
        const int r = rg * 16 + g + 8 * rr;
        if (a.n_splits > 1) {
            const size_t unit = (static_cast<size_t>(item) * gridDim.x + blockIdx.x) * a.n_splits + split;
            float* po = a.part_o + (unit * LM_ROWS + r) * KVR + dh * DH + qd * 2;
#pragma unroll
            for (int d = 0; d < DT; ++d)
                *reinterpret_cast<float2*>(po + d * 8) = make_float2(o[d][2 * rr], o[d][2 * rr + 1]);
            if (dh == 0 && qd == 0) {
                a.part_ml[(unit * LM_ROWS + r) * 2] = m_run[rr];
                a.part_ml[(unit * LM_ROWS + r) * 2 + 1] = l_run[rr];
            }
            continue;
        }
        const int qi = r >> a.hb_shift, h = h0 + (r & (HB - 1));
        const float inv = 1.0f / l_run[rr];
        bf16* dst = a.out + (static_cast<size_t>(h) * a.T + row0 + qi) * KVR + dh * DH + qd * 2;
#pragma unroll
        for (int d = 0; d < DT; ++d)
            *reinterpret_cast<uint32_t*>(dst + d * 8) = lm_pack(o[d][2 * rr] * inv, o[d][2 * rr + 1] * inv);
    }
}

// One block per (item, head block): the ranges' partial results, in ascending order of the ranges.
__global__ void __launch_bounds__(256) latent_attn_merge_kernel(LatentMmaArgs a, int kvr) {
    __shared__ float s_w[16][LM_ROWS];   // weight of every range for every row
    __shared__ float s_inv[LM_ROWS];
    pdl_entry();
    pdl_trigger();
    const int item = blockIdx.y;
    const int seg = a.items[2 * item], qoff = a.items[2 * item + 1];
    const int HB = 1 << a.hb_shift, QB = LM_ROWS >> a.hb_shift;
    const int h0 = blockIdx.x * HB;
    const int nq = min(QB, a.seg_qn[seg] - qoff);
    const int row0 = a.seg_q0[seg] + qoff;
    int first_tile, n_tiles_all;
    lm_item_tiles(a.seg_ctx[seg] + qoff, nq, a.window, first_tile, n_tiles_all);
    const int per_split = (n_tiles_all + a.n_splits - 1) / a.n_splits;
    const int n_live = (n_tiles_all + per_split - 1) / per_split;
    const size_t unit0 = (static_cast<size_t>(item) * gridDim.x + blockIdx.x) * a.n_splits;
    if (threadIdx.x < LM_ROWS) {
        const int r = threadIdx.x;
        float m = -INFINITY;
        for (int sp = 0; sp < n_live; ++sp) m = fmaxf(m, a.part_ml[((unit0 + sp) * LM_ROWS + r) * 2]);
        float l = 0.f;
        for (int sp = 0; sp < n_live; ++sp) {
            const float ms = a.part_ml[((unit0 + sp) * LM_ROWS + r) * 2];
            const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
            s_w[sp][r] = w;
            l += a.part_ml[((unit0 + sp) * LM_ROWS + r) * 2 + 1] * w;
        }
        s_inv[r] = 1.0f / l;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < LM_ROWS * kvr; i += 256) {
        const int r = i / kvr, d = i % kvr;
        const int qi = r >> a.hb_shift, h = h0 + (r & (HB - 1));
        if (qi >= nq || h >= a.H) continue;
        float acc = 0.f;
        for (int sp = 0; sp < n_live; ++sp) acc += a.part_o[((unit0 + sp) * LM_ROWS + r) * kvr + d] * s_w[sp][r];
        a.out[(static_cast<size_t>(h) * a.T + row0 + qi) * kvr + d] = __float2bfloat16_rn(acc * s_inv[r]);
    }
}

template <int KVR>
static int launch_latent_mma(const LatentMmaArgs& a, int n_items, size_t smem, cudaStream_t stream) {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(latent_attn_mma_kernel<KVR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
        return LOCUS_ERR_UNSUPPORTED;
    const int HB = 1 << a.hb_shift;
    locus_launch(latent_attn_mma_kernel<KVR>, dim3((a.H + HB - 1) / HB, n_items, a.n_splits), dim3(256), smem, stream, a);
    if (a.n_splits > 1)
        locus_launch(latent_attn_merge_kernel, dim3((a.H + HB - 1) / HB, n_items), dim3(256), 0, stream, a, KVR);
    return locus_launch_status();
}

// bfloat16; kv_rank 32, 64, 128, 256 or 512; rot_dim a multiple of 16 (0 allowed); a block's 64 rows are
// (64 >> hb_shift) queries x (1 << hb_shift) heads, and items lists tiles of 64 >> hb_shift queries.  n_splits > 1
// (up to 16): the key tiles of every block are cut into that many ranges; part_o holds n_items * head blocks *
// n_splits * 64 * kv_rank floats and part_ml n_items * head blocks * n_splits * 128.
extern "C" int locus_latent_attn_mma(const void* q_abs, const void* q_rot, const void* pool, const float* sink,
                                     void* out, const int* seg_q0, const int* seg_qn, const int* seg_ctx,
                                     const int* block_table, int table_stride, const int* items, int n_items, int T,
                                     int H, int kv_rank, int rot_dim, int page_tokens, int window, float scale,
                                     int hb_shift, int n_splits, float* part_o, float* part_ml, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (n_splits < 1 || n_splits > 16 || (n_splits > 1 && (part_o == nullptr || part_ml == nullptr))) return LOCUS_ERR_UNSUPPORTED;
    if (H <= 0 || rot_dim < 0 || rot_dim % 16 != 0 || page_tokens <= 0 || window < 0 || n_items > 65535 ||
        hb_shift < 0 || hb_shift > 6)
        return LOCUS_ERR_UNSUPPORTED;
    const int R = kv_rank + rot_dim;
    const size_t smem = sizeof(bf16) * static_cast<size_t>(LM_ROWS + 2 * LM_KEYS) * (R + 8) + sizeof(float) * LM_ROWS * (LM_KEYS + 1);
    if (smem > 220 * 1024) return LOCUS_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q_abs) | reinterpret_cast<uintptr_t>(q_rot) | reinterpret_cast<uintptr_t>(pool) |
         reinterpret_cast<uintptr_t>(out)) & 15)
        return LOCUS_ERR_UNSUPPORTED;
    LatentMmaArgs a;
    a.q_abs = static_cast<const bf16*>(q_abs); a.q_rot = static_cast<const bf16*>(q_rot);
    a.pool = static_cast<const bf16*>(pool); a.sink = sink; a.out = static_cast<bf16*>(out); a.seg_q0 = seg_q0;
    a.seg_qn = seg_qn; a.seg_ctx = seg_ctx; a.block_table = block_table; a.table_stride = table_stride; a.items = items;
    a.T = T; a.H = H; a.rot_dim = rot_dim; a.page_tokens = page_tokens; a.window = window; a.hb_shift = hb_shift;
    a.scale = scale; a.n_splits = n_splits; a.part_o = part_o; a.part_ml = part_ml;
    switch (kv_rank) {
        case 32: return launch_latent_mma<32>(a, n_items, smem, stream);
        case 64: return launch_latent_mma<64>(a, n_items, smem, stream);
        case 128: return launch_latent_mma<128>(a, n_items, smem, stream);
        case 256: return launch_latent_mma<256>(a, n_items, smem, stream);
        case 512: return launch_latent_mma<512>(a, n_items, smem, stream);
    }
    return LOCUS_ERR_UNSUPPORTED;
}
