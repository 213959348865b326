// What stands between a mixer's stacked projection and its attention or recurrence kernel, in one launch, float32
// arithmetic throughout: a short causal convolution over time per channel, an activation, a rotation by position, a
// unit norm per head, and the write of q into rows and of k and v into rows or into the layer's cache pages.
//
//   head_prep        one warp per (token, q | k | v, head).  The head's channels pass, in this order and each only
//                    if asked for: the convolution y_t = sum_j w[c, j] u_(t - taps + 1 + j) (a portion's first
//                    tokens read the inputs of the tokens before it from the request's state slot; zeros at a
//                    request's start, since a slot is zeroed when a request opens), silu, the rotation of the pairs
//                    (i, i + rot/2) of the first `rot` channels of a q or k head by position * inv_freq[i], and
//                    for q and k the division by sqrt(mean(x^2) + eps) (norm 1) or sqrt(sum(x^2) + eps) (norm 2)
//                    and q's factor.  The result goes, in the output's element type, to q's rows and to k's and
//                    v's rows or cache pages, laid out at `laid` elements per head (zeros behind the head's own).
//                    With gates (a gated delta rule's), one more warp per token forms beta = sigmoid(b) and
//                    decay = exp(-exp(A_log) * softplus(a + dt_bias)) for every head.
//   conv_state_move  afterwards: the slot's last taps - 1 inputs move on by the portion's tokens.
#include "common.cuh"

#define PREP_MAX_TAPS 16
#define PREP_MAX_DIM 256

__device__ __forceinline__ float sc_softplus(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float sc_silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sc_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

struct PrepArgs {
    const float* proj;        // [T, ld]
    int ld;
    int off[3], heads[3], dim[3], laid[3];   // q, k, v: first column, heads, per-head size, laid-out size
    const void* conv;         // [channels, taps] in q, k, v order, or null
    int conv_dt, taps, act;
    const float* conv_state;  // slot 0's [channels, taps - 1]
    long long slot_stride;
    const int* state_slots;
    const int* seg_q0;
    const int* seg_qn;
    const int* positions;     // [T]
    const float* inv_freq;    // [rot / 2] or null
    int rot, norm;
    float eps, q_scale;
    void* q_out;              // [T, heads[0] * laid[0]]
    void* k_out;              // rows [T, heads[1] * laid[1]] and v_out alike, or, with pool set, unused
    void* v_out;
    void* pool;               // [n_pages][2][heads[1]][page_tokens][laid[1]] (laid[1] == laid[2]), or null
    const int* slots;         // [T] page * page_tokens + offset
    int page_tokens, write_kv;
    // gates of a gated delta rule (null: none)
    float* beta;              // [T, gate_heads]
    float* decay;
    int off_b, off_a, gate_heads;
    const void* a_log;
    const void* dt_bias;
    int gate_dt;
};

template <typename T>
__global__ void __launch_bounds__(128) head_prep_kernel(const PrepArgs a) {
    __shared__ float bufs[4][PREP_MAX_DIM];
    pdl_entry();
    pdl_trigger();
    const int seg = blockIdx.z, t = blockIdx.y;
    const int qn = a.seg_qn[seg];
    if (t >= qn) return;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nq = a.heads[0], nk = a.heads[1], nv = a.heads[2];
    const int n_units = nq + nk + nv + (a.beta != nullptr ? 1 : 0);
    const int unit = blockIdx.x * 4 + wid;
    if (unit >= n_units) return;
    const size_t row = static_cast<size_t>(a.seg_q0[seg] + t);
    const float* pr = a.proj + row * a.ld;
    if (unit == nq + nk + nv) {
        for (int h = lane; h < a.gate_heads; h += 32) {
            a.beta[row * a.gate_heads + h] = sc_sigmoid(pr[a.off_b + h]);
            const float dt = sc_softplus(pr[a.off_a + h] + ld_dyn(a.dt_bias, a.gate_dt, h));
            a.decay[row * a.gate_heads + h] = expf(-expf(ld_dyn(a.a_log, a.gate_dt, h)) * dt);
        }
        return;
    }
    const int which = unit < nq ? 0 : (unit < nq + nk ? 1 : 2);
    const int head = unit - (which == 0 ? 0 : (which == 1 ? nq : nq + nk));
    if (which > 0 && !a.write_kv) return;
    const int d = a.dim[which], laid = a.laid[which];
    int ch0 = head * d;   // the head's first channel among all channels of q, k, v
    if (which >= 1) ch0 += nq * a.dim[0];
    if (which == 2) ch0 += nk * a.dim[1];
    float* buf = bufs[wid];
    const int taps = a.taps;
    const float* old = a.conv ? a.conv_state + static_cast<size_t>(a.state_slots[seg]) * a.slot_stride : nullptr;
    for (int i = lane; i < d; i += 32) {
        const int c = a.off[which] + head * d + i;
        float acc;
        if (a.conv) {
            const size_t cc = static_cast<size_t>(ch0 + i);
            acc = 0.f;
            for (int j = 0; j < taps; ++j) {
                const int p = t - (taps - 1) + j;   // the input's place within the portion; negative: before it
                const float x = p >= 0 ? a.proj[(row - (t - p)) * a.ld + c] : old[cc * (taps - 1) + (taps - 1 + p)];
                acc = fmaf(ld_dyn(a.conv, a.conv_dt, cc * taps + j), x, acc);
            }
        } else {
            acc = pr[c];
        }
        buf[i] = a.act ? sc_silu(acc) : acc;
    }
    __syncwarp();
    if (which < 2 && a.rot > 0 && a.inv_freq != nullptr) {
        const int half = a.rot / 2;
        const float pos = static_cast<float>(a.positions[row]);
        for (int i = lane; i < half; i += 32) {
            float sn, cs;
            sincosf(pos * a.inv_freq[i], &sn, &cs);
            const float u = buf[i], v = buf[i + half];
            buf[i] = u * cs - v * sn;
            buf[i + half] = v * cs + u * sn;
        }
        __syncwarp();
    }
    float r = 1.0f;
    if (which < 2 && a.norm != 0) {
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) ss = fmaf(buf[i], buf[i], ss);
        ss = warp_sum(ss);
        r = a.norm == 1 ? 1.0f / sqrtf(ss / static_cast<float>(d) + a.eps) : 1.0f / sqrtf(ss + a.eps);
    }
    if (which == 0) r *= a.q_scale;
    T* dst;
    if (which == 0) {
        dst = static_cast<T*>(a.q_out) + (row * nq + head) * laid;
    } else if (a.pool != nullptr) {
        const int slot = a.slots[row];
        const int page = slot / a.page_tokens, o = slot % a.page_tokens;
        dst = static_cast<T*>(a.pool) + ((static_cast<size_t>(page) * 2 + (which - 1)) * nk + head) * a.page_tokens * laid +
              static_cast<size_t>(o) * laid;
    } else {
        dst = static_cast<T*>(which == 1 ? a.k_out : a.v_out) + (row * a.heads[which] + head) * laid;
    }
    for (int i = lane; i < laid; i += 32) dst[i] = from_f<T>(i < d ? buf[i] * r : 0.f);
}

__global__ void __launch_bounds__(256) conv_state_move_kernel(const float* __restrict__ proj, int ld, int off0, int n0,
                                                              int off1, int n1, int off2, float* __restrict__ conv_state,
                                                              long long slot_stride, const int* __restrict__ state_slots,
                                                              const int* __restrict__ seg_q0, const int* __restrict__ seg_qn,
                                                              int channels, int taps) {
    pdl_entry();
    pdl_trigger();
    const int seg = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    // channel c of the stacked q, k, v lives in column col of proj
    const int col = c < n0 ? off0 + c : (c < n0 + n1 ? off1 + (c - n0) : off2 + (c - n0 - n1));
    const int qn = seg_qn[seg], q0 = seg_q0[seg], keep_n = taps - 1;
    float* st = conv_state + static_cast<size_t>(state_slots[seg]) * slot_stride + static_cast<size_t>(c) * keep_n;
    float nv[PREP_MAX_TAPS];
    for (int j = 0; j < keep_n; ++j) {
        const int p = qn - keep_n + j;
        nv[j] = p >= 0 ? proj[static_cast<size_t>(q0 + p) * ld + col] : st[j + qn];
    }
    for (int j = 0; j < keep_n; ++j) st[j] = nv[j];
}

// sizes [12]: off, heads, dim, laid of q, k, v.  conv [channels, taps] (element type conv_dt) or null; conv_state: the
// address of the convolution's part of slot 0, moved on by the call when move_state is set.  out_dt: the element type
// of q_out, k_out, v_out and the pool.  pool: the layer's pages (k and v go there, at slots[t]) or null (k_out, v_out).
// gates: beta, decay [T, gate_heads] float32 from columns off_b, off_a of proj, or beta null.
extern "C" int locus_head_prep(const float* proj, int ld, const int* sizes, const void* conv, int conv_dt, int taps, int act,
                               float* conv_state, long long slot_stride, int move_state, const int* state_slots,
                               const int* seg_q0, const int* seg_qn, int n_seg, int longest_new, const int* positions,
                               const float* inv_freq, int rot, int norm, float eps, float q_scale, void* q_out, void* k_out,
                               void* v_out, void* pool, const int* slots, int page_tokens, int write_kv, int out_dt,
                               float* beta, float* decay, int off_b, int off_a, int gate_heads, const void* a_log,
                               const void* dt_bias, int gate_dt, cudaStream_t stream) {
    if (n_seg <= 0 || longest_new <= 0) return 0;
    PrepArgs a;
    int channels = 0;
    for (int w = 0; w < 3; ++w) {
        a.off[w] = sizes[w]; a.heads[w] = sizes[3 + w]; a.dim[w] = sizes[6 + w]; a.laid[w] = sizes[9 + w];
        if (a.heads[w] < 0 || a.dim[w] <= 0 || a.dim[w] > PREP_MAX_DIM || a.laid[w] < a.dim[w]) return LOCUS_ERR_UNSUPPORTED;
        channels += a.heads[w] * a.dim[w];
    }
    if (taps < 1 || taps > PREP_MAX_TAPS || n_seg > 65535 || longest_new > 65535) return LOCUS_ERR_UNSUPPORTED;
    if (rot < 0 || rot % 2 || rot > a.dim[0] || rot > a.dim[1] || (rot > 0 && inv_freq == nullptr)) return LOCUS_ERR_UNSUPPORTED;
    if (conv != nullptr && taps > 1 && conv_state == nullptr) return LOCUS_ERR_UNSUPPORTED;
    if (pool != nullptr && (a.laid[1] != a.laid[2] || page_tokens <= 0 || slots == nullptr)) return LOCUS_ERR_UNSUPPORTED;
    if (beta != nullptr && (decay == nullptr || gate_heads <= 0 || a_log == nullptr || dt_bias == nullptr)) return LOCUS_ERR_UNSUPPORTED;
    a.proj = proj; a.ld = ld; a.conv = conv; a.conv_dt = conv_dt; a.taps = conv ? taps : 1; a.act = act;
    a.conv_state = conv_state; a.slot_stride = slot_stride; a.state_slots = state_slots; a.seg_q0 = seg_q0; a.seg_qn = seg_qn;
    a.positions = positions; a.inv_freq = inv_freq; a.rot = rot; a.norm = norm; a.eps = eps; a.q_scale = q_scale;
    a.q_out = q_out; a.k_out = k_out; a.v_out = v_out; a.pool = pool; a.slots = slots; a.page_tokens = page_tokens;
    a.write_kv = write_kv; a.beta = beta; a.decay = decay; a.off_b = off_b; a.off_a = off_a; a.gate_heads = gate_heads;
    a.a_log = a_log; a.dt_bias = dt_bias; a.gate_dt = gate_dt;
    const int units = a.heads[0] + a.heads[1] + a.heads[2] + (beta != nullptr ? 1 : 0);
    const dim3 grid((units + 3) / 4, longest_new, n_seg);
    if (out_dt == LOCUS_DT_F32) locus_launch(head_prep_kernel<float>, grid, dim3(128), 0, stream, a);
    else if (out_dt == LOCUS_DT_BF16) locus_launch(head_prep_kernel<bf16>, grid, dim3(128), 0, stream, a);
    else return LOCUS_ERR_UNSUPPORTED;
    if (conv != nullptr && taps > 1 && move_state)
        locus_launch(conv_state_move_kernel, dim3((channels + 255) / 256, n_seg), dim3(256), 0, stream, proj, ld, a.off[0],
                     a.heads[0] * a.dim[0], a.off[1], a.heads[1] * a.dim[1], a.off[2], conv_state, slot_stride, state_slots,
                     seg_q0, seg_qn, channels, taps);
    return locus_launch_status();
}

// out[t, e] = o[t, e] * sigmoid(proj[t, off + e]) in place (o in its own element type; the gate's columns float32).
template <typename T>
__global__ void __launch_bounds__(256) gate_rows_kernel(T* __restrict__ o, const float* __restrict__ proj, int ld, int off,
                                                        int width, int o_ld, int col_map_dim, int col_map_laid, long long n) {
    pdl_entry();
    pdl_trigger();
    const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= n) return;
    const long long t = i / width;
    const int e = static_cast<int>(i % width);
    // element e of the gate (heads of col_map_dim) multiplies the laid-out element of o (heads of col_map_laid)
    const int oe = (e / col_map_dim) * col_map_laid + e % col_map_dim;
    T* p = o + t * o_ld + oe;
    *p = from_f<T>(to_f(*p) * sc_sigmoid(proj[t * ld + off + e]));
}

// o [T, o_ld] (heads laid out at `laid` elements of which the first `dim` are the head's own), gate columns
// [off, off + width) of proj [T, ld] float32, width = heads * dim.
extern "C" int locus_gate_rows(void* o, int o_dt, int o_ld, const float* proj, int ld, int off, int width, int dim, int laid,
                               int T, cudaStream_t stream) {
    if (T <= 0 || width <= 0) return 0;
    if (dim <= 0 || laid < dim || width % dim) return LOCUS_ERR_UNSUPPORTED;
    const long long n = static_cast<long long>(T) * width;
    const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
    if (o_dt == LOCUS_DT_F32)
        locus_launch(gate_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, static_cast<float*>(o), proj, ld, off, width, o_ld, dim, laid, n);
    else if (o_dt == LOCUS_DT_BF16)
        locus_launch(gate_rows_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, static_cast<bf16*>(o), proj, ld, off, width, o_ld, dim, laid, n);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}
