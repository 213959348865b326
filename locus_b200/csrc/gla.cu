// Gated linear attention: per request and head a matrix state S [d, dv] (float32, in the request's state slot, zero when
// the request opens) whose rows -- one per key channel -- decay each by a factor of their own at every token:
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t * q_scale,
//
// with a_t [d] in (0, 1) per token and head.  Everything is float32; q, k, v and the decays are columns of float32 row
// matrices given by pointer, row stride and offset.  The decays travel as c = 1 - a and a row is decayed as S - c S: a
// channel that forgets slowly has a within a few float32 spacings of 1, so that a itself would carry its rate 1 - a
// with a relative error of 1e-4 and more, which a few hundred tokens turn into as much in the state; c keeps the rate
// to float32's own precision.
//
//   gla_decay   c = 1 - sigmoid(z)^(1 / tau) = -expm1(-softplus(-z) / tau) in place over rows of logits z (softplus in its
//               stable form max(x, 0) + log1p(exp(-|x|)); no fast-math)
//   gla_scan    a warp owns GL_CW = 4 columns of one head's state for one request and walks the request's new tokens in
//               order.  Its lanes are 8 groups of rows x 4 columns: lane (lr, lc) keeps, of column lc, the rows
//               32 j + 4 lr + {0, 1, 2, 3} (j = 0, 1, ...; d <= 256) in registers, so a token's read-out crosses 8
//               lanes in three exchanges; four rows of q, k and a are one 16-byte load each where the operands allow
//               it.  The next token's operands are fetched while this one is worked on.  The order of every sum is
//               fixed by d alone, so a cut of a prompt changes nothing at all, and the same kernel serves prompt
//               portions and single tokens.  (A chunked form -- per chunk of 16 tokens the products with e^(L_i - L_j),
//               L the running sum of log a, every exponent <= 0, the chunks' own term for all chunks at once and a walk
//               over the chunks with 16 columns of the state per block -- was built and gave the same numbers, but took
//               1,931 us where this walk takes 745 us on 2,048 tokens of 16 heads of 128 x 128, and 6,105 against 4,569 us
//               on eight such requests: the walk over 128 chunks with one block of four warps per SM is the longer chain.)
#include "common.cuh"

struct GlaArgs {
    const float* q;
    const float* k;
    const float* v;
    const float* a;       // 1 - decay
    float* state;
    const int* state_slots;
    const int* seg_q0;
    const int* seg_qn;
    float* out;           // [T, ldo]: head h's columns start at h * dv
    long long slot_stride;
    int ldq, off_q, ldk, off_k, ldv, off_v, lda, off_a, ldo;
    int H, d, dv;
    float q_scale;
};

#define GL_CW 4   // columns of a warp

// R: rows of a column that a lane keeps (d <= 8 R).  VEC: the rows of q, k and a of a head start on 16-byte boundaries
// and d is a multiple of 4, so four rows are one load.
template <int R, bool VEC>
__global__ void __launch_bounds__(128) gla_scan_kernel(const GlaArgs a, int col_groups) {
    pdl_entry();
    pdl_trigger();
    constexpr int CW = GL_CW, NG = 32 / CW;
    const int lane = threadIdx.x & 31, lr = lane / CW, lc = lane % CW;
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);  // (head, column group)
    const int seg = blockIdx.y;
    if (unit >= a.H * col_groups) return;
    const int qn = a.seg_qn[seg];
    const int h = unit / col_groups, col = (unit % col_groups) * CW + lc;
    const int d = a.d, dv = a.dv, q0 = a.seg_q0[seg];
    const bool col_ok = col < dv;
    float* S = a.state + static_cast<size_t>(a.state_slots[seg]) * a.slot_stride + static_cast<size_t>(h) * d * dv;
    auto row_of = [&](int i) { return 4 * NG * (i >> 2) + 4 * lr + (i & 3); };
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = row_of(i);
        s[i] = (r < d && col_ok) ? S[static_cast<size_t>(r) * dv + col] : 0.f;
    }
    const int off_q = a.off_q + h * d, off_k = a.off_k + h * d, off_a = a.off_a + h * d, off_v = a.off_v + h * dv;
    float qn_[R], kn_[R], an_[R], vn_ = 0.f;
    auto fetch = [&](int t) {  // token t's operands into the look-ahead registers
        if (t >= qn) return;
        const size_t row = static_cast<size_t>(q0 + t);
        const float* qp = a.q + row * a.ldq + off_q;
        const float* kp = a.k + row * a.ldk + off_k;
        const float* ap = a.a + row * a.lda + off_a;
        if (VEC) {
#pragma unroll
            for (int b = 0; b < R / 4; ++b) {
                const int r = 4 * NG * b + 4 * lr;
                float4 qv = make_float4(0.f, 0.f, 0.f, 0.f), kv = qv, av = qv;
                if (r < d) {
                    qv = *reinterpret_cast<const float4*>(qp + r);
                    kv = *reinterpret_cast<const float4*>(kp + r);
                    av = *reinterpret_cast<const float4*>(ap + r);
                }
                qn_[4 * b] = qv.x; qn_[4 * b + 1] = qv.y; qn_[4 * b + 2] = qv.z; qn_[4 * b + 3] = qv.w;
                kn_[4 * b] = kv.x; kn_[4 * b + 1] = kv.y; kn_[4 * b + 2] = kv.z; kn_[4 * b + 3] = kv.w;
                an_[4 * b] = av.x; an_[4 * b + 1] = av.y; an_[4 * b + 2] = av.z; an_[4 * b + 3] = av.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const int r = row_of(i);
                qn_[i] = r < d ? qp[r] : 0.f;
                kn_[i] = r < d ? kp[r] : 0.f;
                an_[i] = r < d ? ap[r] : 0.f;
            }
        }
        vn_ = col_ok ? a.v[row * a.ldv + off_v + col] : 0.f;
    };
    fetch(0);
    for (int t = 0; t < qn; ++t) {
        float qq[R], kk[R], aa[R];
        const float vv = vn_;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            qq[i] = qn_[i];
            kk[i] = kn_[i];
            aa[i] = an_[i];
        }
        fetch(t + 1);  // the next token's operands are on their way while this one is worked on
        float o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int i = 0; i < R; i += 2) {
            s[i] = fmaf(kk[i], vv, fmaf(-aa[i], s[i], s[i]));
            s[i + 1] = fmaf(kk[i + 1], vv, fmaf(-aa[i + 1], s[i + 1], s[i + 1]));
            o0 = fmaf(s[i], qq[i], o0);
            o1 = fmaf(s[i + 1], qq[i + 1], o1);
        }
        float o = o0 + o1;
#pragma unroll
        for (int m = CW; m < 32; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);  // across the row groups of this column
        if (lr == 0 && col_ok) a.out[static_cast<size_t>(q0 + t) * a.ldo + h * dv + col] = o * a.q_scale;
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = row_of(i);
        if (r < d && col_ok) S[static_cast<size_t>(r) * dv + col] = s[i];
    }
}

// z [T, ld] float32, columns [off, off + n): z <- 1 - exp(-softplus(-z) / tau).
__global__ void __launch_bounds__(256) gla_decay_kernel(float* __restrict__ z, int ld, int off, int n, float inv_tau,
                                                        long long total) {
    pdl_entry();
    pdl_trigger();
    const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= total) return;
    float* p = z + (i / n) * ld + off + (i % n);
    const float x = -*p;                                          // softplus(x) = max(x, 0) + log1p(exp(-|x|))
    const float sp = fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
    *p = -expm1f(-sp * inv_tau);
}

extern "C" int locus_gla_decay(float* z, int ld, int off, int n, int T, float tau, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n <= 0 || off < 0 || ld < off + n || !(tau > 0.f)) return LOCUS_ERR_UNSUPPORTED;
    const long long total = static_cast<long long>(T) * n;
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return LOCUS_ERR_UNSUPPORTED;
    locus_launch(gla_decay_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, z, ld, off, n, 1.0f / tau, total);
    return locus_launch_status();
}

extern "C" int locus_gla_scan(const float* q, int ldq, int off_q, const float* k, int ldk, int off_k, const float* v, int ldv,
                              int off_v, const float* dec, int lda, int off_a, float* state, long long slot_stride,
                              const int* state_slots, const int* seg_q0, const int* seg_qn, int n_seg, float* out, int ldo,
                              int H, int d, int dv, float q_scale, cudaStream_t stream) {
    if (n_seg <= 0) return 0;
    if (H <= 0 || d <= 0 || d > 256 || dv <= 0 || n_seg > 65535 || H > 65535) return LOCUS_ERR_UNSUPPORTED;
    GlaArgs a;
    a.q = q; a.k = k; a.v = v; a.a = dec; a.state = state; a.state_slots = state_slots; a.seg_q0 = seg_q0; a.seg_qn = seg_qn;
    a.out = out; a.slot_stride = slot_stride; a.ldq = ldq; a.off_q = off_q; a.ldk = ldk; a.off_k = off_k; a.ldv = ldv;
    a.off_v = off_v; a.lda = lda; a.off_a = off_a; a.ldo = ldo; a.H = H; a.d = d; a.dv = dv; a.q_scale = q_scale;
    {   // (the scope of the launch macro)
        const bool vec = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(dec)) & 15) == 0 &&
                         ((ldq | off_q | ldk | off_k | lda | off_a | d) & 3) == 0;
        const int col_groups = (dv + GL_CW - 1) / GL_CW;
        const dim3 grid((H * col_groups + 3) / 4, n_seg);
#define GL_SCAN(R)                                                                              \
    do {                                                                                        \
        if (vec) locus_launch(gla_scan_kernel<R, true>, grid, dim3(128), 0, stream, a, col_groups);  \
        else locus_launch(gla_scan_kernel<R, false>, grid, dim3(128), 0, stream, a, col_groups);     \
    } while (0)
        if (d <= 32) GL_SCAN(4);
        else if (d <= 64) GL_SCAN(8);
        else if (d <= 128) GL_SCAN(16);
        else GL_SCAN(32);
#undef GL_SCAN
    }
    return locus_launch_status();
}
