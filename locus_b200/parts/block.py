"""Block arrangements and the parts at the two ends of the model.

``PreNorm``: x += mixer(norm1(x)); x += feed_forward(norm2(x)) -- the residual placement
of the reference's forward (src/locus/model/llama.cpp:485-509).  The residual stream x is
float32 in every mode; the normed activations have the model's element type.

``OutputNorm``: x += norm1(mixer(x)); x += norm2(feed_forward(x)): the sublayers read x itself and the
norms sit on what they give.

``StreamedPreNorm``: pre-norm sublayers over several copies of the residual stream that are read as a weighted sum
and mixed among themselves at every write-back (below).

``PostNorm``: x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + feed_forward(x)): the sublayers read x itself and the
norm sits on the sum.

``Embedding``: x = table[token] (llama.cpp:450); optionally plus a row of a second table addressed by a hash of the
previous and the current token.  ``LmHead``: logits = W . h in float32,
W being the embedding table when the head is tied (llama.cpp:292-297, 512-513): the head then
names the embedding's tensor as the source of its weight.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from .base import (Arrangement, Part, PartSpec, StateSpec, TensorSource, make_part, register_arrangement,
                   register_embedding, register_head)


class PreNorm(Arrangement):
    def __init__(self, prefix: str, *, hidden: int, norm: PartSpec, mixer: PartSpec,
                 feed_forward: PartSpec, mixer_prefix: str = "self_attn", ff_prefix: str = "mlp",
                 norm1_name: str = "input_layernorm", norm2_name: str = "post_attention_layernorm",
                 plain_norm_names: bool = False) -> None:
        """``plain_norm_names``: the norms' tensors carry the plain name of the norm (no ".weight" behind it).
        ``feed_forward`` may be absent (kind "none"): the layer is then its mixer alone and has no second norm."""
        super().__init__(prefix)
        self.hidden = hidden

        def norm_part(name):
            spec = PartSpec(norm.kind, {**norm.args, "tensor": f"{prefix}.{name}"}) if plain_norm_names else norm
            return make_part("norm", spec, f"{prefix}.{name}")

        self.norm1 = norm_part(norm1_name)
        self.mixer = make_part("mixer", mixer, f"{prefix}.{mixer_prefix}")
        self.ff = None if feed_forward.kind == "none" else make_part("feed_forward", feed_forward, f"{prefix}.{ff_prefix}")
        self.norm2 = norm_part(norm2_name) if self.ff is not None else None

    takes_pending_add = True

    def sub_parts(self):
        return [self.norm1, self.mixer] + ([self.norm2, self.ff] if self.ff is not None else [])

    def forward(self, x, batch, cache, rt) -> None:
        T = batch.T
        h = rt.rows("block.h", self.hidden, rt.dtype, T)
        self.norm1.forward(x, h, add=rt.take_pending())
        self.mixer.forward(h, batch, cache, x, rt)
        if self.ff is None:
            return
        self.norm2.forward(x, h)
        self.ff.forward(h, batch, x, rt)


class OutputNorm(Arrangement):
    """Norm on a sublayer's OUTPUT only: x += norm1(mixer(x)); x += norm2(feed_forward(x)).  The sublayers read
    the residual stream itself (in a bfloat16 model: its rounding to bfloat16); what they give is collected in
    float32 rows, normed with float32 statistics and added.  ``feed_forward`` may be absent (kind "none"): the
    layer is then its mixer alone and has no second norm."""

    def __init__(self, prefix: str, *, hidden: int, norm: PartSpec, mixer: PartSpec, feed_forward: PartSpec,
                 mixer_prefix: str = "mix", ff_prefix: str = "mlp", norm1_name: str = "norm1",
                 norm2_name: str = "norm2") -> None:
        super().__init__(prefix)
        self.hidden = hidden

        def norm_part(name):
            # the norms' tensors carry the plain name of the norm (no ".weight" behind it)
            spec = PartSpec(norm.kind, {**norm.args, "tensor": f"{prefix}.{name}"})
            return make_part("norm", spec, f"{prefix}.{name}")

        self.norm1 = norm_part(norm1_name)
        self.mixer = make_part("mixer", mixer, f"{prefix}.{mixer_prefix}")
        self.ff = None if feed_forward.kind == "none" else make_part("feed_forward", feed_forward, f"{prefix}.{ff_prefix}")
        self.norm2 = norm_part(norm2_name) if self.ff is not None else None

    def sub_parts(self):
        return [self.norm1, self.mixer] + ([self.norm2, self.ff] if self.ff is not None else [])

    def _read(self, x, rt, T):
        if rt.dtype == torch.float32:
            return x
        h = rt.rows("block.h", self.hidden, rt.dtype, T)
        K.cast_rows(x, h)
        return h

    def forward(self, x, batch, cache, rt) -> None:
        T = batch.T
        rt.defer_add = False   # what a sublayer gives is normed here, at once: nothing may be left pending
        y = rt.rows("block.y", self.hidden, torch.float32, T)
        h = self._read(x, rt, T)
        if self.mixer.can_overwrite:
            self.mixer.forward(h, batch, cache, y, rt, accumulate=False)
        else:
            y.zero_()
            self.mixer.forward(h, batch, cache, y, rt)
        self.norm1.forward_add(y, x)
        if self.ff is None:
            return
        h = self._read(x, rt, T)
        if self.ff.can_overwrite:
            self.ff.forward(h, batch, y, rt, accumulate=False)
        else:
            y.zero_()
            self.ff.forward(h, batch, y, rt)
        self.norm2.forward_add(y, x)


class PostNorm(Arrangement):
    """The norm behind the sum: x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + feed_forward(x)), with a layer norm
    (weight and bias) whose statistics, like the sum and the residual stream, are float32.  The sublayers read x itself
    (in a bfloat16 model its rounding, which the norm's own pass writes beside the float32 row) and write float32 rows.
    ``feed_forward`` may be absent (kind "none"): the layer is then its mixer and the first norm alone."""

    def __init__(self, prefix: str, *, hidden: int, norm: PartSpec, mixer: PartSpec, feed_forward: PartSpec,
                 alpha: float = 1.0, mixer_prefix: str = "mix", ff_prefix: str = "mlp", norm1_name: str = "norm1",
                 norm2_name: str = "norm2", bias_suffix: str = ".b") -> None:
        super().__init__(prefix)
        self.hidden, self.alpha = int(hidden), float(alpha)
        if norm.kind != "layernorm":
            raise ValueError(f"post_norm: the norm behind the sum is a layer norm, got {norm.kind!r}")

        def norm_part(name):
            spec = PartSpec(norm.kind, {**norm.args, "tensor": f"{prefix}.{name}", "bias_tensor": f"{prefix}.{name}{bias_suffix}"})
            return make_part("norm", spec, f"{prefix}.{name}")

        self.norm1 = norm_part(norm1_name)
        self.mixer = make_part("mixer", mixer, f"{prefix}.{mixer_prefix}")
        self.ff = None if feed_forward.kind == "none" else make_part("feed_forward", feed_forward, f"{prefix}.{ff_prefix}")
        self.norm2 = norm_part(norm2_name) if self.ff is not None else None

    def sub_parts(self):
        return [self.norm1, self.mixer] + ([self.norm2, self.ff] if self.ff is not None else [])

    def kernel_modules(self, dtype):
        return ["elementwise"]

    def forward(self, x, batch, cache, rt) -> None:
        T = batch.T
        rt.defer_add = False   # what a sublayer gives is summed and normed here, at once: nothing may be left pending
        y = rt.rows("block.y", self.hidden, torch.float32, T)
        # what the sublayers read: x itself; in a bfloat16 model the copy that the norm in front wrote (the first
        # layer's first sublayer makes its own)
        low = rt.dtype != torch.float32
        h = rt.rows("block.h", self.hidden, rt.dtype, T) if low else x
        if low and getattr(rt, "_post_norm_rows", None) is not x:
            K.cast_rows(x, h)
        rt._post_norm_rows = None
        if self.mixer.can_overwrite:
            self.mixer.forward(h, batch, cache, y, rt, accumulate=False)
        else:
            y.zero_()
            self.mixer.forward(h, batch, cache, y, rt)
        self.norm1.forward_post(x, y, self.alpha, cast=h if low else None)
        if self.ff is not None:
            if self.ff.can_overwrite:
                self.ff.forward(h, batch, y, rt, accumulate=False)
            else:
                y.zero_()
                self.ff.forward(h, batch, y, rt)
            self.norm2.forward_post(x, y, self.alpha, cast=h if low else None)
        if low:
            rt._post_norm_rows = x   # block.h holds x's rounding for the block behind this one


class StreamedPreNorm(Arrangement):
    """Pre-norm sublayers over ``streams`` copies x_1 .. x_S of the residual stream (a row of x holds them one behind
    the other).  For sublayer q (1: the mixer, 2: the feed-forward) with its own read weights a [S], write weights b
    [S] and mixing matrix M [S, S] (indexed [from, to]):

        u = sum_s a[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s M[s, t] x_s + mult * b[t] * y   (all t at once).

    ``streams`` = 0: one stream and no such tensors, x <- x + mult * sublayer(norm_q(x)).  ``feed_forward`` may be
    absent (kind "none").  The sublayers write float32 rows; read, norm statistics and write-back are float32."""

    def __init__(self, prefix: str, *, hidden: int, norm: PartSpec, mixer: PartSpec, feed_forward: PartSpec,
                 streams: int = 0, mult: float = 1.0, mixer_prefix: str = "mix", ff_prefix: str = "mlp",
                 norm1_name: str = "norm1", norm2_name: str = "norm2", bias_suffix: str = ".b",
                 hc_names: tuple = ("hc1", "hc2")) -> None:
        super().__init__(prefix)
        self.hidden, self.mult = int(hidden), float(mult)
        self.hyper = int(streams) > 0
        self.S = max(int(streams), 1)
        if self.S > K.MAX_STREAMS:
            raise ValueError(f"streamed_pre_norm: {streams} streams exceed {K.MAX_STREAMS}")

        def norm_part(name):
            spec = PartSpec(norm.kind, {**norm.args, "streams": self.S, "tensor": f"{prefix}.{name}",
                                        "bias_tensor": f"{prefix}.{name}{bias_suffix}"})
            return make_part("norm", spec, f"{prefix}.{name}")

        self.norm1 = norm_part(norm1_name)
        self.mixer = make_part("mixer", mixer, f"{prefix}.{mixer_prefix}")
        self.ff = None if feed_forward.kind == "none" else make_part("feed_forward", feed_forward, f"{prefix}.{ff_prefix}")
        self.norm2 = norm_part(norm2_name) if self.ff is not None else None
        self.hc_names = tuple(hc_names)[: 2 if self.ff is not None else 1]
        self._coef = {}

    def sub_parts(self):
        return [self.norm1, self.mixer] + ([self.norm2, self.ff] if self.ff is not None else [])

    def param_shapes(self):
        if not self.hyper:
            return {}
        out = {}
        for n in self.hc_names:
            out.update({f"{n}.in": (self.S,), f"{n}.out": (self.S,), f"{n}.mix": (self.S, self.S)})
        return out

    def sources(self):
        return [TensorSource(f"{self.prefix}.{name}", shape, name, 0, "norm" if name.endswith((".in", ".out")) else "bias")
                for name, shape in self.param_shapes().items()]

    def kernel_modules(self, dtype):
        return ["elementwise"]

    def bind(self, rt) -> None:
        # the small tables as float32; the write weights carry the sublayers' common factor
        self._coef = {}
        for n in self.hc_names:
            if self.hyper:
                a = self.params[f"{n}.in"].float().contiguous()
                b = (self.params[f"{n}.out"].float() * self.mult).contiguous()
                m = self.params[f"{n}.mix"].float().contiguous()
            else:
                a = None
                b = torch.full((1,), self.mult, dtype=torch.float32, device=rt.device)
                m = torch.ones((1, 1), dtype=torch.float32, device=rt.device)
            self._coef[n] = (a, b, m)

    def _sublayer(self, which, norm, run, x, rt, T) -> None:
        a, b, m = self._coef[which]
        h = rt.rows("block.h", self.hidden, rt.dtype, T)
        y = rt.rows("block.y", self.hidden, torch.float32, T)
        norm.forward(x, h, coef=a)
        run(h, y)
        K.stream_update(x, y, m, b, self.S)

    def forward(self, x, batch, cache, rt) -> None:
        T = batch.T
        rt.defer_add = False   # what a sublayer gives is written back here, at once: nothing may be left pending

        def mixer(h, y):
            if self.mixer.can_overwrite:
                self.mixer.forward(h, batch, cache, y, rt, accumulate=False)
            else:
                y.zero_()
                self.mixer.forward(h, batch, cache, y, rt)

        def ff(h, y):
            if self.ff.can_overwrite:
                self.ff.forward(h, batch, y, rt, accumulate=False)
            else:
                y.zero_()
                self.ff.forward(h, batch, y, rt)

        self._sublayer(self.hc_names[0], self.norm1, mixer, x, rt, T)
        if self.ff is not None:
            self._sublayer(self.hc_names[1], self.norm2, ff, x, rt, T)


class Embedding(Part):
    def __init__(self, prefix: str, *, vocab: int, hidden: int, tensor: str = "", copies: int = 1,
                 scale: float = 1.0, pair: Optional[dict] = None) -> None:
        """``tensor``: the checkpoint tensor's name where it is not ``<prefix>.weight``.  ``copies`` > 1: a row of the
        output holds the embedding that many times (a model with several copies of the residual stream).  ``scale``:
        a factor on the embedding, applied in float32.  ``pair`` = {tensor, buckets, mul_prev, mul_cur}: a second table
        of buckets + 1 rows whose row (previous token * mul_prev + token * mul_cur) mod buckets is added (its last row for
        a request's first token).  The token that a request's last step ended on is kept in the request's state slot
        (``state_needs``), so that a prompt may be cut anywhere."""
        super().__init__(prefix)
        self.vocab, self.hidden, self.copies, self.scale = int(vocab), int(hidden), int(copies), float(scale)
        self.tensor = str(tensor or prefix + ".weight")
        self.pair = dict(pair) if pair else None
        if self.pair is not None:
            if self.copies != 1 or self.scale != 1.0:
                raise ValueError("embedding: the pair table goes with one copy and no factor")
            if int(self.pair["buckets"]) <= 0 or int(self.pair["mul_prev"]) < 0 or int(self.pair["mul_cur"]) < 0:
                raise ValueError("embedding: the pair table needs positive buckets and multipliers that are not negative")

    def param_shapes(self):
        s = {"table": (self.vocab, self.hidden)}
        if self.pair is not None:
            s["pair"] = (int(self.pair["buckets"]) + 1, self.hidden)
        return s

    def sources(self):
        out = [TensorSource(self.tensor, (self.vocab, self.hidden), "table")]
        if self.pair is not None:
            out.append(TensorSource(str(self.pair["tensor"]), (int(self.pair["buckets"]) + 1, self.hidden), "pair"))
        return out

    def kernel_modules(self, dtype):
        return ["elementwise"]

    def state_needs(self) -> Optional[StateSpec]:
        """What the embedding keeps per request: the last token it saw, when it has a pair table."""
        return StateSpec((1,), torch.int32) if self.pair is not None else None

    def forward(self, tokens: torch.Tensor, out: torch.Tensor, batch=None, cache=None) -> None:
        if self.pair is not None:
            if batch is None or cache is None or cache.state is None:
                raise ValueError("embedding: a pair table needs the step's segments and the requests' state slots")
            K.embed_pair(tokens, batch.positions, self.params["table"], self.params["pair"], out, seg_q0=batch.seg_q0,
                         seg_qn=batch.seg_qn, state_slots=batch.state_slots, last=cache.state, n_seg=batch.n_seg,
                         longest_new=max(batch.host_seg_qn) if batch.host_seg_qn else batch.T,
                         mul_prev=int(self.pair["mul_prev"]), mul_cur=int(self.pair["mul_cur"]))
            return
        if self.copies > 1 or self.scale != 1.0:
            K.embed_rows(tokens, self.params["table"], out, copies=self.copies, scale=self.scale)
        else:
            K.embed_rows(tokens, self.params["table"], out)


class LmHead(Part):
    """``tied_to``: the checkpoint tensor that is the head's weight when the head has none of its own
    (the embedding table of a tied model); two parts that name the same tensor share one device copy."""

    def __init__(self, prefix: str, *, vocab: int, hidden: int, tied_to: str = "", tensor: str = "") -> None:
        super().__init__(prefix)
        self.vocab, self.hidden, self.tied_to = int(vocab), int(hidden), str(tied_to or "")
        self.tensor = str(tensor or prefix + ".weight")   # the head's own tensor, when it is not tied

    def param_shapes(self):
        return {"weight": (self.vocab, self.hidden)}

    def sources(self):
        return [TensorSource(self.tied_to or self.tensor, (self.vocab, self.hidden), "weight")]

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def forward(self, h: torch.Tensor, logits: torch.Tensor) -> None:
        K.linear(h, self.params["weight"], logits)


register_arrangement("pre_norm", PreNorm)
register_arrangement("output_norm", OutputNorm)
register_arrangement("streamed_pre_norm", StreamedPreNorm)
register_arrangement("post_norm", PostNorm)
register_embedding("embedding", Embedding)
register_head("linear", LmHead)
