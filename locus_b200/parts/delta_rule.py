"""A gated delta rule mixer: a matrix memory that every token first decays, then corrects towards its value along
its key, then reads.

With h the mixer's input, H heads of values (size v_dim) and G heads of queries and keys (size dim; value head a uses
q/k head a // (H / G)): q = W_q h, k = W_k h, v = W_v h each pass a short causal convolution per channel over the last
``taps`` tokens (zeros before a request's start) and silu; q and k are then made unit vectors per head, x / sqrt(sum(x^2)
+ 1e-6), and q is multiplied by dim^(-1/2).  beta = sigmoid(W_b h) and the decay g = exp(-exp(A_log) * softplus(W_a h +
dt_bias)) are one number per token and head.  Per head a state S [dim, v_dim] is carried from token to token:

    S <- g S;    u = beta (v - S^T k);    S <- S + k u^T;    o = S^T q      (the read-out sees the token's own write).

Each head's o is divided by its root mean square, multiplied by a weight [v_dim] that the heads share and by silu(W_g
h), and projected by W_o.  One product gives [q | k | v | b | a | g] as float32 rows; the convolution, the gates, the
unit norms, the recurrence and the output norm are float32.  State per request: S [H, dim, v_dim] and the
convolution's last taps - 1 inputs [channels, taps - 1], in one slot.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from .base import Mixer, StateSpec, TensorSource, register_mixer

UNIT_EPS = 1e-6   # inside the root of the unit norms of q and k


class GatedDeltaRule(Mixer):
    can_overwrite = True

    def __init__(self, prefix: str, *, hidden: int, n_heads: int, n_qk_heads: int, dim: int, v_dim: int, taps: int,
                 eps: float, out_scale: float = 1.0, names: Optional[dict] = None) -> None:
        """``eps``: inside the root of the output norm.  ``out_scale``: a factor on the mixer's output (a mixer that runs
        beside another one)."""
        super().__init__(prefix)
        if n_heads % n_qk_heads:
            raise ValueError(f"gated_delta: {n_heads} heads are not a multiple of {n_qk_heads} query/key heads")
        if dim > K.DELTA_MAX_DIM:
            raise ValueError(f"gated_delta: dim {dim} exceeds {K.DELTA_MAX_DIM}")
        if not (1 <= taps <= K.PREP_MAX_TAPS):
            raise ValueError(f"gated_delta: a convolution over {taps} tokens (at most {K.PREP_MAX_TAPS})")
        self.hidden, self.H, self.G, self.d, self.dv = int(hidden), int(n_heads), int(n_qk_heads), int(dim), int(v_dim)
        self.taps, self.eps, self.out_scale = int(taps), float(eps), float(out_scale)
        self.inner = self.H * self.dv
        qk = self.G * self.d
        self.rows = [("q", 0, qk), ("k", qk, qk), ("v", 2 * qk, self.inner), ("b", 2 * qk + self.inner, self.H),
                     ("a", 2 * qk + self.inner + self.H, self.H), ("g", 2 * qk + self.inner + 2 * self.H, self.inner)]
        self.off = {r: o for r, o, _ in self.rows}
        self.used = self.rows[-1][1] + self.rows[-1][2]
        self.width = -(-self.used // 8) * 8
        self.channels = 2 * qk + self.inner
        self.state_floats = self.H * self.d * self.dv
        self.names = {"q": "q", "k": "k", "v": "v", "b": "b", "a": "a", "g": "g", "q_conv": "q.conv", "k_conv": "k.conv",
                      "v_conv": "v.conv", "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm", "o": "o", **(names or {})}

    def param_shapes(self):
        return {"w_in": (self.width, self.hidden), "conv": (self.channels, self.taps), "a_log": (self.H,),
                "dt_bias": (self.H,), "norm": (self.dv,), "w_o": (self.hidden, self.inner)}

    def sources(self):
        p, n = self.prefix, self.names
        out = [TensorSource(f"{p}.{n[r]}", (size, self.hidden), "w_in", row0) for r, row0, size in self.rows]
        out += [TensorSource(f"{p}.{n[r + '_conv']}", (size, self.taps), "conv", row0, "bias") for r, row0, size in self.rows[:3]]
        out += [TensorSource(f"{p}.{n['A_log']}", (self.H,), "a_log", 0, "bias"),
                TensorSource(f"{p}.{n['dt_bias']}", (self.H,), "dt_bias", 0, "bias"),
                TensorSource(f"{p}.{n['norm']}", (self.dv,), "norm", 0, "norm"),
                TensorSource(f"{p}.{n['o']}", (self.hidden, self.inner), "w_o")]
        return out

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv", "short_conv", "delta_rule"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def cache_needs(self):
        return None, StateSpec((self.state_floats + self.channels * (self.taps - 1),), torch.float32)

    def bind(self, rt) -> None:
        self.params["w_in"][self.used:].zero_()
        self._scale = None
        if self.out_scale != 1.0:
            self._scale = rt.shared_object(("row_scale", self.out_scale), lambda: torch.full(
                (rt.max_tokens,), self.out_scale, dtype=torch.float32, device=rt.device))

    def forward(self, h, batch, cache, residual, rt, accumulate=True) -> None:
        self.finish(self.prepare(h, batch, cache, rt), residual, rt, accumulate)

    # The mixer in two steps, for a caller that runs it beside another mixer: everything up to the input of the output
    # projection touches only this mixer's own buffers and state; the projection writes (or adds into) ``residual``.
    def prepare(self, h, batch, cache, rt):
        T, H, G, d, dv = batch.T, self.H, self.G, self.d, self.dv
        proj = rt.rows(f"delta.proj{self.width}", self.width, torch.float32, T)
        K.linear(h, self.params["w_in"], proj)
        if cache.writes:
            state = cache.state
        else:
            state = rt.buf("delta.state_copy", tuple(cache.state.shape), torch.float32)
            state.copy_(cache.state)
        q = rt.rows("delta.q", G * d, torch.float32, T)
        k = rt.rows("delta.k", G * d, torch.float32, T)
        v = rt.rows("delta.v", self.inner, torch.float32, T)
        beta = rt.rows("delta.beta", H, torch.float32, T)
        decay = rt.rows("delta.decay", H, torch.float32, T)
        K.head_prep(proj, offsets=(self.off["q"], self.off["k"], self.off["v"]), heads=(G, G, H), dims=(d, d, dv),
                    laid=(d, d, dv), state_slots=batch.state_slots, seg_q0=batch.seg_q0, seg_qn=batch.seg_qn,
                    n_seg=batch.n_seg, longest_new=max(batch.host_seg_qn) if batch.host_seg_qn else T,
                    positions=batch.positions, q_out=q, k_out=k, v_out=v, conv=self.params["conv"], state=state,
                    conv_offset=self.state_floats, act=True, norm="unit", eps=UNIT_EPS, q_scale=d ** -0.5,
                    gates=(beta, decay, self.off["b"], self.off["a"], self.params["a_log"], self.params["dt_bias"]))
        y = rt.rows("delta.y", self.inner, torch.float32, T)
        K.delta_rule(q, 0, k, 0, v, 0, beta, decay, state, 0, batch.state_slots, batch.seg_q0, batch.seg_qn, batch.n_seg, y,
                     n_heads=H, heads_per_group=H // G, dim=d, v_dim=dv)
        o = rt.rows("delta.o", self.inner, rt.dtype, T)
        K.delta_out(y, proj, self.off["g"], self.params["norm"], self.eps, o, n_heads=H, v_dim=dv)
        return o

    def finish(self, o, residual, rt, accumulate=True) -> None:
        K.linear(o, self.params["w_o"], residual, accumulate=accumulate, row_scale=self._scale)


register_mixer("gated_delta", GatedDeltaRule)
