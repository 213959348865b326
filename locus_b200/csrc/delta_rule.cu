// The gated delta rule: per request and head a matrix state S [d, dv] (float32, in the request's state slot, zero
// when the request opens) that every token first decays, then corrects towards its value along its key, then reads:
//
//     S <- g_t S;     u_t = beta_t (v_t - S^T k_t);     S <- S + k_t u_t^T;     o_t = S^T q_t,
//
// with g_t (a decay in (0, 1]) and beta_t (a step in (0, 1)) one float32 number per token and head, made by the
// caller.  q and k of head h are those of its group h / heads_per_group; v is the head's own.  Everything is float32;
// q, k and v are columns of float32 row matrices given by pointer, row stride and offset.
//
// The columns of S do not meet: with a = S_old^T k, b = S_old^T q (both of the state BEFORE the token) and the number
// k . q, u = beta (v - g a) and o = g b + u (k . q).  So a token costs one round of warp sums, not two in a row.
//
//   delta_scan   a warp owns DR_CW columns of one head's state for one request and walks the request's new tokens in
//                order; lane l keeps the rows l, l + 32, ... of its columns in registers (d <= 256).  The order of
//                every sum is fixed by d alone, so a cut of a prompt changes nothing at all.
//   delta_out    a head's read-out divided by its root mean square, times a weight, times silu(gate).
#include "common.cuh"

#define DR_CW 4

struct DeltaArgs {
    const float* q;
    const float* k;
    const float* v;
    const float* beta;    // [T, H]
    const float* decay;   // [T, H]
    float* state;
    const int* state_slots;
    const int* seg_q0;
    const int* seg_qn;
    float* out;           // [T, ldo]: head h's columns start at h * dv
    long long slot_stride;
    int ldq, off_q, ldk, off_k, ldv, off_v, ldo;
    int H, heads_per_group, d, dv;
};

template <int RPL>
__global__ void __launch_bounds__(128) delta_scan_kernel(const DeltaArgs a, int col_groups) {
    pdl_entry();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);  // (head, column group)
    const int seg = blockIdx.y;
    if (unit >= a.H * col_groups) return;
    const int qn = a.seg_qn[seg];
    const int h = unit / col_groups, c0 = (unit % col_groups) * DR_CW;
    const int d = a.d, dv = a.dv, q0 = a.seg_q0[seg];
    float* S = a.state + static_cast<size_t>(a.state_slots[seg]) * a.slot_stride + static_cast<size_t>(h) * d * dv;
    float s[RPL][DR_CW];
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = lane + 32 * r;
#pragma unroll
        for (int c = 0; c < DR_CW; ++c) s[r][c] = (i < d && c0 + c < dv) ? S[static_cast<size_t>(i) * dv + c0 + c] : 0.f;
    }
    const int g = h / a.heads_per_group;
    const int off_q = a.off_q + g * d, off_k = a.off_k + g * d, off_v = a.off_v + h * dv;
    float qn_[RPL], kn_[RPL], vn_[DR_CW], beta_n = 0.f, decay_n = 0.f;
    auto fetch = [&](int t) {
        const size_t row = static_cast<size_t>(q0 + t);
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            const int i = lane + 32 * r;
            qn_[r] = i < d ? a.q[row * a.ldq + off_q + i] : 0.f;
            kn_[r] = i < d ? a.k[row * a.ldk + off_k + i] : 0.f;
        }
#pragma unroll
        for (int c = 0; c < DR_CW; ++c) vn_[c] = c0 + c < dv ? a.v[row * a.ldv + off_v + c0 + c] : 0.f;
        beta_n = a.beta[row * a.H + h];
        decay_n = a.decay[row * a.H + h];
    };
    if (qn > 0) fetch(0);
    for (int t = 0; t < qn; ++t) {
        float qq[RPL], kk[RPL], vv[DR_CW];
        const float beta = beta_n, gd = decay_n;
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            qq[r] = qn_[r];
            kk[r] = kn_[r];
        }
#pragma unroll
        for (int c = 0; c < DR_CW; ++c) vv[c] = vn_[c];
        if (t + 1 < qn) fetch(t + 1);  // the next token's operands are on their way while this one is worked on
        float sk[DR_CW], sq[DR_CW], kq = 0.f;
#pragma unroll
        for (int c = 0; c < DR_CW; ++c) sk[c] = sq[c] = 0.f;
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            kq = fmaf(kk[r], qq[r], kq);
#pragma unroll
            for (int c = 0; c < DR_CW; ++c) {
                sk[c] = fmaf(s[r][c], kk[r], sk[c]);
                sq[c] = fmaf(s[r][c], qq[r], sq[c]);
            }
        }
        kq = warp_sum(kq);
        float u[DR_CW], o[DR_CW];
#pragma unroll
        for (int c = 0; c < DR_CW; ++c) {
            sk[c] = warp_sum(sk[c]);
            sq[c] = warp_sum(sq[c]);
            u[c] = beta * (vv[c] - gd * sk[c]);
            o[c] = fmaf(u[c], kq, gd * sq[c]);
        }
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
#pragma unroll
            for (int c = 0; c < DR_CW; ++c) s[r][c] = fmaf(gd, s[r][c], kk[r] * u[c]);
        }
        if (lane < DR_CW && c0 + lane < dv) {
            float ov = o[0];
#pragma unroll
            for (int c = 1; c < DR_CW; ++c)
                if (lane == c) ov = o[c];
            a.out[static_cast<size_t>(q0 + t) * a.ldo + h * dv + c0 + lane] = ov;
        }
    }
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = lane + 32 * r;
#pragma unroll
        for (int c = 0; c < DR_CW; ++c)
            if (i < d && c0 + c < dv) S[static_cast<size_t>(i) * dv + c0 + c] = s[r][c];
    }
}

extern "C" int locus_delta_scan(const float* q, int ldq, int off_q, const float* k, int ldk, int off_k, const float* v, int ldv,
                                int off_v, const float* beta, const float* decay, float* state, long long slot_stride,
                                const int* state_slots, const int* seg_q0, const int* seg_qn, int n_seg, float* out, int ldo,
                                int H, int heads_per_group, int d, int dv, cudaStream_t stream) {
    if (n_seg <= 0) return 0;
    if (H <= 0 || heads_per_group <= 0 || H % heads_per_group || d <= 0 || d > 256 || dv <= 0 || n_seg > 65535)
        return LOCUS_ERR_UNSUPPORTED;
    DeltaArgs a;
    a.q = q; a.k = k; a.v = v; a.beta = beta; a.decay = decay; a.state = state; a.state_slots = state_slots;
    a.seg_q0 = seg_q0; a.seg_qn = seg_qn; a.out = out; a.slot_stride = slot_stride; a.ldq = ldq; a.off_q = off_q;
    a.ldk = ldk; a.off_k = off_k; a.ldv = ldv; a.off_v = off_v; a.ldo = ldo; a.H = H; a.heads_per_group = heads_per_group;
    a.d = d; a.dv = dv;
    const int col_groups = (dv + DR_CW - 1) / DR_CW;
    const dim3 grid((H * col_groups + 3) / 4, n_seg);
    const int rpl = (d + 31) / 32;
#define DR_SCAN(R) locus_launch(delta_scan_kernel<R>, grid, dim3(128), 0, stream, a, col_groups)
    if (rpl <= 1) DR_SCAN(1);
    else if (rpl <= 2) DR_SCAN(2);
    else if (rpl <= 4) DR_SCAN(4);
    else DR_SCAN(8);
#undef DR_SCAN
    return locus_launch_status();
}

__device__ __forceinline__ float dr_silu(float x) { return x / (1.0f + expf(-x)); }

// One warp per (token, head).
template <typename TO>
__global__ void __launch_bounds__(256) delta_out_kernel(const float* __restrict__ o, const float* __restrict__ proj, int ld,
                                                        int off_g, const void* __restrict__ w, int w_dt, int w_len, float eps,
                                                        TO* __restrict__ out, int n_units, int H, int dv) {
    pdl_entry();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (unit >= n_units) return;
    const int t = unit / H, h = unit % H;
    const float* orow = o + (static_cast<size_t>(t) * H + h) * dv;
    const float* grow = proj + static_cast<size_t>(t) * ld + off_g + h * dv;
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) ss = fmaf(orow[j], orow[j], ss);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / static_cast<float>(dv) + eps);
    TO* dst = out + (static_cast<size_t>(t) * H + h) * dv;
    for (int j = lane; j < dv; j += 32)
        dst[j] = from_f<TO>(orow[j] * scale * ld_dyn(w, w_dt, (h * dv + j) % w_len) * dr_silu(grow[j]));
}

// o [T, H * dv] float32; the gate's columns [off_g, off_g + H * dv) of proj [T, ld] float32; w [w_len] with w_len = dv
// (one weight for all heads) or H * dv; out [T, H * dv].
extern "C" int locus_delta_out(const float* o, const float* proj, int ld, int off_g, const void* w, int w_dt, int w_len,
                               float eps, void* out, int out_dt, int T, int H, int dv, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dv <= 0 || (w_len != dv && w_len != H * dv)) return LOCUS_ERR_UNSUPPORTED;
    const long long units = static_cast<long long>(T) * H;
    if (units > 0x7fffffffLL) return LOCUS_ERR_UNSUPPORTED;
    const int n = static_cast<int>(units), blocks = (n + 7) / 8;
    if (out_dt == LOCUS_DT_BF16)
        locus_launch(delta_out_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, o, proj, ld, off_g, w, w_dt, w_len, eps,
                     static_cast<bf16*>(out), n, H, dv);
    else if (out_dt == LOCUS_DT_F32)
        locus_launch(delta_out_kernel<float>, dim3(blocks), dim3(256), 0, stream, o, proj, ld, off_g, w, w_dt, w_len, eps,
                     static_cast<float*>(out), n, H, dv);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}
