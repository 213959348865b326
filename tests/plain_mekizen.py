"""A plain, slow, whole-sequence implementation of the Mekizen design: one function per mechanism, float64 on the
CPU, written from the design's equations and sharing no code with the engine.

The design: a pre-norm decoder, x <- x + mixer(norm1(x)); x <- x + ff(norm2(x)), whose RMS norms store their weight
around zero (the factor is 1 + w), with a scaled embedding.  Mixers: ``attention`` (grouped-query attention with
biases, a partial rotation, a sliding window that also keeps a sequence's first tokens, a softmax whose denominator
has one added, a sigmoid gate on the heads' outputs; a layer may use an earlier layer's keys and values) and
``parallel`` (causal softmax attention whose q, k, v pass a short convolution, a partial rotation and, for q and k, a
unit root mean square per head -- beside a gated delta rule; each side's output is RMS-normed over the width and
the two are averaged).  Feed-forward: W_down relu(W_up h)^2.

``weights`` is a dict name -> tensor (any float type; converted to float64 here), ``cfg`` the dictionary of the
model's config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def _w(weights, name) -> torch.Tensor:
    return weights[name].to(F64)


# ---------------------------------------------------------------------------
# small functions


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * (1.0 + w)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rotate(x: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, heads, dim], positions 0 .. T - 1: the first ``dims`` of every head rotated, pairs (i, i + dims/2)."""
    T = x.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = torch.arange(T, dtype=F64)[:, None] * f[None, :]          # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    """Whether position i sees j; ``size`` 0: no window."""
    if j > i:
        return False
    return size <= 0 or i - j < size or j < keep_first


def softmax_attention(q, k, v, scale: float, size: int = 0, keep_first: int = 0, sink: bool = False) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; ``sink``: one added to the softmax's denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if size > 0:
        seen = seen & ((i - j < size) | (j < keep_first))
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = ((q[:, h] @ k[:, g].T) * scale).masked_fill(~seen, -math.inf)     # [T, T]
        m = s.max(-1, keepdim=True).values
        if sink:
            m = torch.clamp(m, min=0.0)
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + (torch.exp(-m) if sink else 0.0)
        out[:, h] = (e / den) @ v[:, g]
    return out


def delta_rule(q, k, v, beta, g) -> torch.Tensor:
    """Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  q, k [T, H, d] (already per value
    head), v [T, H, dv], beta, g [T, H] -> [T, H, dv]."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, d, dv, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hde,hd->he", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out


# ---------------------------------------------------------------------------
# mixers (h: [T, width], one sequence from its first token)


def conv_attention(weights, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """The left side of a parallel mixer, up to and including its output projection."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = short_conv(h @ _w(weights, p + ".q").T, _w(weights, p + ".q.conv")).view(T, H, d)
    k = short_conv(h @ _w(weights, p + ".k").T, _w(weights, p + ".k.conv")).view(T, G, d)
    v = short_conv(h @ _w(weights, p + ".v").T, _w(weights, p + ".v.conv")).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q, k = rotate(q, float(rot["base"]), int(rot["dims"])), rotate(k, float(rot["base"]), int(rot["dims"]))
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    o = softmax_attention(q, k, v, float(m["scale"]))
    return o.reshape(T, H * dv) @ _w(weights, p + ".o").T


def gated_delta(weights, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """The right side of a parallel mixer, up to and including its output projection."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(short_conv(h @ _w(weights, p + ".q").T, _w(weights, p + ".q.conv"))).view(T, G, d)
    k = silu(short_conv(h @ _w(weights, p + ".k").T, _w(weights, p + ".k.conv"))).view(T, G, d)
    v = silu(short_conv(h @ _w(weights, p + ".v").T, _w(weights, p + ".v.conv"))).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = sigmoid(h @ _w(weights, p + ".b").T)
    g = torch.exp(-torch.exp(_w(weights, p + ".A_log")) * softplus(h @ _w(weights, p + ".a").T + _w(weights, p + ".dt_bias")))
    o = delta_rule(q, k, v, beta, g)
    o = rms_unit(o, eps) * _w(weights, p + ".norm")
    o = o.reshape(T, H * dv) * silu(h @ _w(weights, p + ".g").T)
    return o @ _w(weights, p + ".o").T


def parallel(weights, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    left = conv_attention(weights, p + ".left", m["left"], h, eps)
    right = gated_delta(weights, p + ".right", m["right"], h, eps)
    return 0.5 * (rms_unit(left, eps) * _w(weights, p + ".left.out") + rms_unit(right, eps) * _w(weights, p + ".right.out"))


def attention_kv(weights, p: str, m: dict, h: torch.Tensor):
    """Keys (rotated) and values of an attention layer that has projections of its own."""
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k = (h @ _w(weights, p + ".k").T + _w(weights, p + ".k.b")).view(T, G, d)
    v = (h @ _w(weights, p + ".v").T + _w(weights, p + ".v.b")).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        k = rotate(k, float(rot["base"]), int(rot["dims"]))
    return k, v


def gated_attention(weights, p: str, m: dict, h: torch.Tensor, kv, sink: bool = True) -> torch.Tensor:
    """``kv``: (keys, values) of this layer or of the layer it takes them from."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ _w(weights, p + ".q").T + _w(weights, p + ".q.b")).view(T, H, d)
    rot = m.get("rot")
    if rot:
        q = rotate(q, float(rot["base"]), int(rot["dims"]))
    mask = m.get("mask") or {}
    o = softmax_attention(q, kv[0], kv[1], float(m["scale"]), int(mask.get("size", 0)), int(mask.get("keep_first", 0)),
                          sink=sink)
    o = o.reshape(T, H * dv) * sigmoid(h @ _w(weights, p + ".g").T)
    return o @ _w(weights, p + ".o").T + _w(weights, p + ".o.b")


def dense_ff(weights, p: str, h: torch.Tensor) -> torch.Tensor:
    z = torch.clamp(h @ _w(weights, p + ".up").T, min=0.0)
    return (z * z) @ _w(weights, p + ".down").T


# ---------------------------------------------------------------------------
# the model


def forward(weights: Dict[str, torch.Tensor], cfg: dict, tokens: List[int], layers_out: Optional[list] = None,
            sink: bool = True, own_kv: Optional[dict] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``layers_out`` collects the residual stream after every layer.  For tests that
    show that a fault would be seen: ``sink`` off leaves the one out of the softmax's denominator; ``own_kv`` {layer:
    other layer} lets a layer project keys and values from its own input with the other layer's weights instead of
    using that layer's."""
    eps = float(cfg["norm"]["eps"])
    x = _w(weights, "embed")[torch.tensor(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    kvs = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = norm_one_plus(x, _w(weights, p + ".norm1"), eps)
        if layer["type"] == "parallel":
            x = x + parallel(weights, p + ".mix", m, h, eps)
        elif layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kvs[i] = attention_kv(weights, p + ".mix", m, h)
                src = i
            kv = kvs[src]
            if own_kv and i in own_kv:
                kv = attention_kv(weights, f"l{own_kv[i]}.mix", m, h)
            x = x + gated_attention(weights, p + ".mix", m, h, kv, sink)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + dense_ff(weights, p + ".mlp", norm_one_plus(x, _w(weights, p + ".norm2"), eps))
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_one_plus(x, _w(weights, "final.norm"), eps) @ _w(weights, "head").T
