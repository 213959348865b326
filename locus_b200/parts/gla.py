"""Gated linear attention: a linear recurrence whose decay is a vector over the key channels, made from the token.

Per token, with h the mixer's input: q = (W_q h) * dim^(-1/2), k = W_k h (heads x dim), v = W_v h (heads x v_dim), a decay
per key channel a = sigmoid(z)^(1 / tau) with z = W_a2 (W_a1 h) + b_a2 (heads x dim; W_a1 maps to a few channels), and per
head a state S [dim, v_dim] that is carried from token to token:

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t.

Every head's o_t is RMS-normed over v_dim with one weight [v_dim] for all heads, the heads are concatenated, multiplied
by silu(W_g h) and projected by W_o.  The state starts at zero, is float32, and lives in the request's state slot.  The
projections are one product whose result stays float32, so that everything that enters the recurrence -- q, k, v, the
decay's logits, sigmoid, root and the state -- is float32; the decay travels as 1 - a = -expm1(-softplus(-z) / tau), which
keeps the rate of a slow channel (a within a few float32 spacings of 1) to float32's own precision.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from .base import Mixer, StateSpec, TensorSource, register_mixer


class GatedLinearAttention(Mixer):
    can_overwrite = True

    def __init__(self, prefix: str, *, hidden: int, n_heads: int, dim: int, v_dim: int, decay_rank: int, tau: float,
                 eps: float, names: Optional[dict] = None) -> None:
        """``decay_rank``: the width of the decay's first projection (rows of W_a1).  ``tau``: the root taken of the
        sigmoid.  ``names``: tensor names below the prefix where they differ from the defaults."""
        super().__init__(prefix)
        if dim > K.GLA_MAX_DIM:
            raise ValueError(f"gla: dim {dim} exceeds {K.GLA_MAX_DIM} (a lane keeps its rows of the state in registers)")
        if not tau > 0:
            raise ValueError(f"gla: tau {tau} must be positive")
        self.hidden, self.H, self.d, self.dv = int(hidden), int(n_heads), int(dim), int(v_dim)
        self.rank, self.tau, self.eps = int(decay_rank), float(tau), float(eps)
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "a1": "a1", "a2": "a2", "a2_bias": "a2.b",
                      "norm": "norm", **(names or {})}
        qk, vv = self.H * self.d, self.H * self.dv
        # the stacked projection [q | k | v | gate | decay's first projection], every part on a 16-byte boundary
        self.rows, at = [], 0
        for role, size in (("q", qk), ("k", qk), ("v", vv), ("g", vv), ("a1", self.rank)):
            self.rows.append((role, at, size))
            at = -(-(at + size) // 4) * 4
        self.off = {role: row0 for role, row0, _ in self.rows}
        self.width = -(-at // 8) * 8

    def param_shapes(self):
        return {"w_in": (self.width, self.hidden), "w_a2": (self.H * self.d, self.rank), "b_a2": (self.H * self.d,),
                "norm": (self.dv,), "w_o": (self.hidden, self.H * self.dv)}

    def sources(self):
        p, n = self.prefix, self.names
        out = [TensorSource(f"{p}.{n[r]}", (size, self.hidden), "w_in", row0) for r, row0, size in self.rows]
        out += [TensorSource(f"{p}.{n['a2']}", (self.H * self.d, self.rank), "w_a2"),
                TensorSource(f"{p}.{n['a2_bias']}", (self.H * self.d,), "b_a2", 0, "bias"),
                TensorSource(f"{p}.{n['norm']}", (self.dv,), "norm", 0, "norm"),
                TensorSource(f"{p}.{n['o']}", (self.hidden, self.H * self.dv), "w_o")]
        return out

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv", "gla", "delta_rule"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def cache_needs(self):
        return None, StateSpec((self.H * self.d * self.dv,), torch.float32)

    def bind(self, rt) -> None:
        # rows of the stacked weight that no tensor fills (the parts' padding) give zeros
        w = self.params["w_in"]
        used = torch.zeros(self.width, dtype=torch.bool, device=w.device)
        for _, row0, size in self.rows:
            used[row0:row0 + size] = True
        w[~used] = 0

    def forward(self, h, batch, cache, residual, rt, accumulate=True) -> None:
        T, H, d, dv = batch.T, self.H, self.d, self.dv
        proj = rt.rows(f"gla.proj{self.width}", self.width, torch.float32, T)
        K.linear(h, self.params["w_in"], proj)
        # the decay's logits: the second projection reads the first one's float32 result
        decay = rt.rows("gla.decay", H * d, torch.float32, T)
        K.linear(proj[:, self.off["a1"]:self.off["a1"] + self.rank], self.params["w_a2"], decay, bias=self.params["b_a2"])
        K.gla_decay(decay, 0, H * d, self.tau)
        if cache.writes:
            state = cache.state
        else:
            # a call that reads another call's state must leave it as it found it
            state = rt.buf("gla.state_copy", tuple(cache.state.shape), torch.float32)
            state.copy_(cache.state)
        y = rt.rows("gla.y", H * dv, torch.float32, T)
        K.gla_scan(proj, self.off["q"], proj, self.off["k"], proj, self.off["v"], decay, 0, state, 0, batch.state_slots,
                   batch.seg_q0, batch.seg_qn, batch.n_seg, y, n_heads=H, dim=d, v_dim=dv, q_scale=d ** -0.5)
        o = rt.rows("gla.o", H * dv, rt.dtype, T)
        K.delta_out(y, proj, self.off["g"], self.params["norm"], self.eps, o, n_heads=H, v_dim=dv)
        K.linear(o, self.params["w_o"], residual, accumulate=accumulate)


register_mixer("gla", GatedLinearAttention)
