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
// k . q, u = beta (v - g a) and o = g b + u (k . q).  So a token costs one round of sums across lanes, not two in a row.
//
//   delta_scan   a warp owns DR_CW = 4 columns of one head's state for one request and walks the request's new tokens
//                in order.  Its lanes are 8 groups of rows x 4 columns: lane (lr, lc) keeps, of column lc, the rows
//                32 j + 4 lr + {0, 1, 2, 3} (j = 0, 1, ...; d <= 256) in registers, so that the three sums of a token
//                (a, b and k . q) cross 8 lanes in three exchanges each -- nine shuffles a token and warp, where a
//                lane that kept rows l, l + 32, ... of all four columns needed forty-five: with many requests the
//                shuffle unit, one warp instruction a cycle and SM, was the limit.  The four rows are one 16-byte load
//                of k and of q where the operands allow it, and the 8 row groups read one 128-byte line.  The next
//                token's operands are fetched while this one is worked on: one token ahead, into registers.  (Measured
//                at one request of 2,048 tokens, 16 heads of 128 x 128, where each scheduler has one warp: two or three
//                tokens ahead, a ring of operands in shared memory filled by asynchronous copies or through registers,
//                and one column to a warp with four times the warps were all slower, by a tenth to a factor of two:
//                each adds instructions or loads in flight to a walk that issues one dependent instruction every six
//                cycles.)  The order of every sum is fixed by d alone, so a cut of a prompt changes nothing at all.
//   delta_out    a head's read-out divided by its root mean square, times a weight, times silu(gate).
#include "common.cuh"


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

#define DR_CW 4   // columns of a warp
#define DR_PF 1   // tokens whose operands are fetched ahead into registers

// R: rows of a column that a lane keeps (d <= 8 R).  VEC: q's and k's rows of a head start on 16-byte boundaries and d
// is a multiple of 4, so four rows are one load.
template <int R, bool VEC>
__global__ void __launch_bounds__(128) delta_scan_kernel(const DeltaArgs a, int col_groups) {
    pdl_entry();
    pdl_trigger();
    constexpr int CW = DR_CW, PF = DR_PF, NG = 32 / CW;  // (NG groups of rows)
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
    const int g = h / a.heads_per_group;
    const int off_q = a.off_q + g * d, off_k = a.off_k + g * d, off_v = a.off_v + h * dv;
    float qn_[PF][R], kn_[PF][R], vn_[PF], beta_n[PF], decay_n[PF];
    auto fetch = [&](int t, int j) {  // token t's operands into register set j
        if (t >= qn) return;
        const size_t row = static_cast<size_t>(q0 + t);
        const float* qp = a.q + row * a.ldq + off_q;
        const float* kp = a.k + row * a.ldk + off_k;
        if (VEC) {
#pragma unroll
            for (int b = 0; b < R / 4; ++b) {
                const int r = 4 * NG * b + 4 * lr;
                float4 qv = make_float4(0.f, 0.f, 0.f, 0.f), kv = qv;
                if (r < d) {
                    qv = *reinterpret_cast<const float4*>(qp + r);
                    kv = *reinterpret_cast<const float4*>(kp + r);
                }
                qn_[j][4 * b] = qv.x; qn_[j][4 * b + 1] = qv.y; qn_[j][4 * b + 2] = qv.z; qn_[j][4 * b + 3] = qv.w;
                kn_[j][4 * b] = kv.x; kn_[j][4 * b + 1] = kv.y; kn_[j][4 * b + 2] = kv.z; kn_[j][4 * b + 3] = kv.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const int r = row_of(i);
                qn_[j][i] = r < d ? qp[r] : 0.f;
                kn_[j][i] = r < d ? kp[r] : 0.f;
            }
        }
        vn_[j] = col_ok ? a.v[row * a.ldv + off_v + col] : 0.f;
        beta_n[j] = a.beta[row * a.H + h];
        decay_n[j] = a.decay[row * a.H + h];
    };
#pragma unroll
    for (int j = 0; j < PF; ++j) fetch(j, j);
    for (int t0 = 0; t0 < qn; t0 += PF) {
#pragma unroll
        for (int j = 0; j < PF; ++j) {
            const int t = t0 + j;
            if (t >= qn) break;
            float qq[R], kk[R];
            const float beta = beta_n[j], gd = decay_n[j], vv = vn_[j];
#pragma unroll
            for (int i = 0; i < R; ++i) {
                qq[i] = qn_[j][i];
                kk[i] = kn_[j][i];
            }
            fetch(t + PF, j);  // a later token's operands are on their way while this one is worked on
            // two partial sums each: a chain of R dependent additions is as long as the exchanges behind it
            float sk0 = 0.f, sk1 = 0.f, sq0 = 0.f, sq1 = 0.f, kq0 = 0.f, kq1 = 0.f;
#pragma unroll
            for (int i = 0; i < R; i += 2) {
                sk0 = fmaf(s[i], kk[i], sk0);
                sq0 = fmaf(s[i], qq[i], sq0);
                kq0 = fmaf(kk[i], qq[i], kq0);
                sk1 = fmaf(s[i + 1], kk[i + 1], sk1);
                sq1 = fmaf(s[i + 1], qq[i + 1], sq1);
                kq1 = fmaf(kk[i + 1], qq[i + 1], kq1);
            }
            float sk = sk0 + sk1, sq = sq0 + sq1, kq = kq0 + kq1;
#pragma unroll
            for (int m = CW; m < 32; m <<= 1) {  // across the row groups of this column
                sk += __shfl_xor_sync(0xffffffffu, sk, m);
                sq += __shfl_xor_sync(0xffffffffu, sq, m);
                kq += __shfl_xor_sync(0xffffffffu, kq, m);
            }
            const float u = beta * (vv - gd * sk);
            const float o = fmaf(u, kq, gd * sq);
#pragma unroll
            for (int i = 0; i < R; ++i) s[i] = fmaf(gd, s[i], kk[i] * u);
            if (lr == 0 && col_ok) a.out[static_cast<size_t>(q0 + t) * a.ldo + h * dv + col] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = row_of(i);
        if (r < d && col_ok) S[static_cast<size_t>(r) * dv + col] = s[i];
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
    const bool vec = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k)) & 15) == 0 &&
                     ((ldq | off_q | ldk | off_k | d) & 3) == 0;
    const int col_groups = (dv + DR_CW - 1) / DR_CW;
    const dim3 grid((H * col_groups + 3) / 4, n_seg);
#define DR_SCAN(R)                                                                              \
    do {                                                                                        \
        if (vec) locus_launch(delta_scan_kernel<R, true>, grid, dim3(128), 0, stream, a, col_groups);  \
        else locus_launch(delta_scan_kernel<R, false>, grid, dim3(128), 0, stream, a, col_groups);     \
    } while (0)
    if (d <= 32) DR_SCAN(4);
    else if (d <= 64) DR_SCAN(8);
    else if (d <= 128) DR_SCAN(16);
    else DR_SCAN(32);
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
