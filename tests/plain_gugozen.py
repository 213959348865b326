"""The Gugozen design, plainly: float64, whole sequences, one function per mechanism, written from the equations.

Nothing here is shared with ``locus_b200``: the configuration is the raw nested dictionary of config.json and the weights
a dictionary of tensors by their stored names.  ``forward`` runs one sequence from its first token.

Notation: x [T, width] the residual stream, h a sublayer's input (x itself), p a position counted from 0.

* embedding: x_p = embed[tok_p] + bigram[r_p], r_p = (tok_(p-1) * mul_prev + tok_p * mul_cur) mod buckets, r_0 = buckets;
* layer: x <- LN1(a x + mixer(x)); x <- LN2(a x + ff(x)) with a = postln_alpha and LN a layer norm with weight and bias;
* mixers ``attention`` (grouped queries, one RMS norm over the whole q and the whole k projection, rotation of part of
  each head, a learned sink in the softmax's denominator), ``latent_attention`` (keys and values from one normed latent
  and one shared rotated key part, a sigmoid gate on the heads' outputs, optionally on an earlier layer's latent) and
  ``gla`` (a linear recurrence whose decay is a vector over the key channels);
* feed-forward: sigmoid-scored top-k experts whose weight multiplies their INPUT, plus a shared expert; an expert is
  W_down (g sigmoid(1.702 g) (u + 1)) with g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def _w(weights, name):
    return weights[name].to(F64)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotate(v, positions, base, dims):
    """v [T, ..., d]: the first ``dims`` elements of the last axis turned, pair (i, i + dims/2) by p * base^(-2i/dims)."""
    if not dims:
        return v
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None] * f[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], -1)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    rows = [buckets]
    for p in range(1, len(tokens)):
        rows.append((int(tokens[p - 1]) * mul_prev + int(tokens[p]) * mul_cur) % buckets)
    return rows


def embed(cfg, weights, tokens):
    x = _w(weights, "embed")[torch.tensor(tokens, dtype=torch.long)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        rows = bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])
        x = x + _w(weights, "bigram")[torch.tensor(rows, dtype=torch.long)]
    return x


def attention(m, weights, pre, h, eps):
    """Grouped-query softmax attention with a sink: p_j = e^(s_j) / (e^(sink) + sum_l e^(s_l)) over the keys j <= i."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rms_norm(h @ _w(weights, pre + "q").T, _w(weights, pre + "q.norm"), eps).view(T, H, d)
    k = rms_norm(h @ _w(weights, pre + "k").T, _w(weights, pre + "k.norm"), eps).view(T, G, d)
    v = (h @ _w(weights, pre + "v").T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q, k = rotate(q, pos, rot["base"], rot["dims"]), rotate(k, pos, rot["base"], rot["dims"])
    sink = _w(weights, pre + "sink")
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, hd]) * m["scale"]
            mx = max(float(s.max()), float(sink[hd]))
            e = torch.exp(s - mx)
            den = e.sum() + math.exp(float(sink[hd]) - mx)
            out[i, hd] = (e / den) @ v[: i + 1, g]
    return out.reshape(T, H * dv) @ _w(weights, pre + "o").T


def latent_kv(m, weights, pre, h, eps):
    """What a latent layer caches: the normed latent c [T, kv_rank] and the rotated shared key part [T, rot_dim]."""
    T = h.shape[0]
    r, dr = m["kv_rank"], m["rot_dim"]
    d = h @ _w(weights, pre + "dkv").T
    c = rms_norm(d[:, :r], _w(weights, pre + "dkv.norm"), eps)
    rot = m.get("rot")
    kr = d[:, r:r + dr]
    if rot:
        kr = rotate(kr, torch.arange(T), rot["base"], rot["dims"])
    return c, kr


def latent_attention(m, weights, pre, h, eps, kv):
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = kv
    q = (h @ _w(weights, pre + "q").T).view(T, H, dn + dr)
    qn, qr = q[..., :dn], q[..., dn:]
    rot = m.get("rot")
    if rot:
        qr = rotate(qr, torch.arange(T), rot["base"], rot["dims"])
    kn = (c @ _w(weights, pre + "uk").T).view(T, H, dn)
    v = (c @ _w(weights, pre + "uv").T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        for i in range(T):
            s = (kn[: i + 1, hd] @ qn[i, hd] + kr[: i + 1] @ qr[i, hd]) * m["scale"]
            out[i, hd] = torch.softmax(s, 0) @ v[: i + 1, hd]
    gate = torch.sigmoid(h @ _w(weights, pre + "g").T)
    return (out.reshape(T, H * dv) * gate) @ _w(weights, pre + "o").T


def gla(m, weights, pre, h, eps, state=None):
    """S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head, a_t = sigmoid(z_t)^(1/tau) per key channel."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ _w(weights, pre + "q").T).view(T, H, d) * d ** -0.5
    k = (h @ _w(weights, pre + "k").T).view(T, H, d)
    v = (h @ _w(weights, pre + "v").T).view(T, H, dv)
    z = (h @ _w(weights, pre + "a1").T) @ _w(weights, pre + "a2").T + _w(weights, pre + "a2.b")
    a = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F64) if state is None else state
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, _w(weights, pre + "norm"), eps)
    g = h @ _w(weights, pre + "g").T
    return (o.reshape(T, H * dv) * (g * torch.sigmoid(g))) @ _w(weights, pre + "o").T


def clamped_expert(weights, pre, h, limit):
    g = torch.clamp(h @ _w(weights, pre + "gate").T, max=limit)
    u = torch.clamp(h @ _w(weights, pre + "up").T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ _w(weights, pre + "down").T


def route(weights, pre, h, top):
    """Picked experts and their weights per token: the ``top`` largest sigmoid scores, as they are."""
    s = torch.sigmoid(h @ _w(weights, pre + "router").T)
    picks = []
    for t in range(h.shape[0]):
        order = sorted(range(s.shape[1]), key=lambda e: (-float(s[t, e]), e))[:top]
        picks.append([(e, s[t, e]) for e in order])
    return picks


def moe_ff(f, weights, pre, h, picks=None):
    """``picks``: the experts to use per token (a list of lists of expert numbers, or a function of the router's logits
    [T, experts] that returns one) instead of the router's own choice; the weights are always the router's scores."""
    T = h.shape[0]
    out = torch.zeros_like(h)
    chosen = route(weights, pre, h, f["router"]["top"])
    if picks is not None:
        if callable(picks):
            picks = picks(h @ _w(weights, pre + "router").T)
        s = torch.sigmoid(h @ _w(weights, pre + "router").T)
        chosen = [[(e, s[t, e]) for e in picks[t]] for t in range(T)]
    for t in range(T):
        for e, w in chosen[t]:
            out[t] += clamped_expert(weights, f"{pre}e{e}.", (w * h[t])[None, :], f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + clamped_expert(weights, pre + "shared.", h, f["shared"]["limit"])
    return out, [[e for e, _ in c] for c in chosen], h @ _w(weights, pre + "router").T


def forward(cfg, weights, tokens, picks=None, layers_out=None, aux=None):
    """Logits [T, vocab] of one sequence.  ``picks[layer][token]``: experts to follow (a layer without an entry follows
    its own router); ``layers_out``: a list that receives the residual stream after every layer; ``aux``: a dictionary
    that receives the router's logits [T, experts] by feed-forward prefix ("l<i>.mlp").  Returns (logits, the experts
    picked per layer)."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = embed(cfg, weights, tokens)
    kept = {}
    picked = []
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            y = attention(m, weights, pre, x, eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_kv(m, weights, pre, x, eps)
                src = i
            y = latent_attention(m, weights, pre, x, eps, kept[src])
        elif layer["type"] == "gla":
            y = gla(m, weights, pre, x, eps)
        else:
            raise ValueError(layer["type"])
        x = layer_norm(alpha * x + y, _w(weights, f"l{i}.norm1"), _w(weights, f"l{i}.norm1.b"), eps)
        if layer.get("mlp") is not None:
            y, ch, z = moe_ff(layer["mlp"], weights, f"l{i}.mlp.", x, None if picks is None else picks.get(i))
            picked.append(ch)
            if aux is not None:
                aux[f"l{i}.mlp"] = z
            x = layer_norm(alpha * x + y, _w(weights, f"l{i}.norm2"), _w(weights, f"l{i}.norm2.b"), eps)
        else:
            picked.append(None)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, _w(weights, "final.norm"), _w(weights, "final.norm.b"), eps)
    return x @ _w(weights, "embed").T, picked
