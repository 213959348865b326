"""Attention mixer over the paged cache: grouped-query attention with optional q/k/v bias,
a position encoding, an optional window, and an output projection.

Per token, as the reference computes it (``qwen2moe_attention``,
src/locus/model/arch.cpp:596-696): q = Wq.h + bq, k = Wk.h + bk, v = Wv.h + bv
(arch.cpp:618-620, 650-655); q and k rotated (arch.cpp:621-622, 656-657), v not; k and v
written to the cache at the token's position; for head h with kv head h // (heads/kv_heads):
scores = q.k * 1/sqrt(head_dim) over the keys 0..pos (arch.cpp:668-681), softmax
(arch.cpp:682), weighted sum of v (arch.cpp:683-694); output = Wo.concat(heads), added to
the residual stream (src/locus/model/llama.cpp:487-490).

The three projections are one product against the stacked weight [(heads + 2 kv_heads) *
head_dim, hidden]; that is layout only.  Scores, softmax and the weighted sum are float32.

Values may have another size than queries and keys (``v_dim``), and either size need not be one the attention
kernels take: the heads are then laid out at the next multiple of 16 that holds both, with zero rows in the stacked
weight and bias and zero columns in the output projection, so that the padding is exact zeros in q, k, v and the cache
and contributes nothing to a score or an output.  The score's factor is then the caller's (``softmax_scale``).

Further forms, each an option of its own: a window that keeps a request's first ``keep_first`` tokens in sight (query i
sees key j <= i if i - j < window or j < keep_first; kept tokens stay at their positions); a softmax with a ``sink`` (one
more term in the denominator that has no value: of score 0, or with ``sink`` "learned" of a score per query head that is
a tensor of the layer and is not multiplied by the scores' factor); a short causal convolution over time on every channel of q, k
and v directly behind the projection (``conv_taps``; the last taps - 1 projected rows of a request are its state); q
and k divided by their root mean square per head behind the rotation (``qk_norm`` "rms"), or an RMS norm with weights over
the whole q and the whole k projection, all heads at once, in front of the rotation (``qk_norm`` "whole"); the heads' outputs multiplied by
sigmoid(W_g h) in front of the output projection (``out_gate``); a layer without keys and values of its own
(``has_kv`` off: it reads the cache of the layer call that the run order names).  With any of these (or ``shaped``)
the projections are one product into float32 rows [q | k | v | gate] at the stored sizes, and one kernel
(``kernels.head_prep``) convolves, rotates, norms and writes q and the cache pages at the kernels' head size in
float32 arithmetic, so that padded heads take a rotation there too.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels as K
from .base import Mixer, PagedKvSpec, PartSpec, StateSpec, StepPlan, TensorSource, make_part, register_mixer
from .position import NoPosition as _NoRotation

CHUNK_TILE = 16  # queries per work item of the CUDA-core chunk kernel


class AttentionTiles(StepPlan):
    """The work lists of this file's attention kernels: tiles of 16 queries (CUDA-core kernel) and of 64 queries
    (tensor-core kernels) over the segments with more than one new token, and the segments with exactly one
    (the decode kernel).  One plan serves every attention layer of a model.  The lists are made by two small
    native helpers (csrc/host_core.cpp: ``locus_plan_query_tiles``, ``locus_plan_segments_with``).  The tiles are
    listed by the position of their first query, ascending, across requests: the kernels walk a list from its end,
    so the tiles with the most keys start first (``locus_sort_tiles_by_position``)."""

    key = ("attention.tiles", CHUNK_TILE, K.MMA_QUERY_TILE)

    def __init__(self) -> None:
        from ..cache import native

        self._lib = native.lib()

    def capacity(self, max_tokens: int, max_segments: int) -> int:
        tiles = max_tokens // CHUNK_TILE + max_tokens // K.MMA_QUERY_TILE + 2 * max_segments
        return 2 * tiles + max_segments

    def build(self, seg_q0, seg_qn, seg_ctx, out):
        n_seg, qn, cap = len(seg_qn), seg_qn.ctypes.data, len(out)
        base = out.ctypes.data
        n16 = self._lib.locus_plan_query_tiles(n_seg, qn, CHUNK_TILE, 2, base, cap)
        o64 = 2 * max(n16, 0)
        n64 = self._lib.locus_plan_query_tiles(n_seg, qn, K.MMA_QUERY_TILE, 2, base + 4 * o64, cap - o64)
        o1 = o64 + 2 * max(n64, 0)
        n1 = self._lib.locus_plan_segments_with(n_seg, qn, 1, base + 4 * o1, cap - o1)
        if n16 < 0 or n64 < 0 or n1 < 0:
            raise ValueError("attention: the step has more tiles than the plan's capacity holds")
        ctx = seg_ctx.ctypes.data
        self._lib.locus_sort_tiles_by_position(n16, base, ctx)
        self._lib.locus_sort_tiles_by_position(n64, base + 4 * o64, ctx)
        return {"chunk_items": (0, 2 * n16, (-1, 2)), "n_chunk_items": n16,
                "chunk_items64": (o64, 2 * n64, (-1, 2)), "n_chunk_items64": n64,
                "decode_items": (o1, n1, None), "n_decode_items": n1}


# tensor names below an attention's prefix, by role; an architecture with other names passes its own
NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
         "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "o_bias": "o_proj.bias",
         "q_conv": "q_proj.conv", "k_conv": "k_proj.conv", "v_conv": "v_proj.conv", "gate": "g_proj.weight",
         "sink": "sink", "q_norm": "q_norm.weight", "k_norm": "k_norm.weight"}


class Attention(Mixer):
    can_overwrite = True

    def __init__(self, prefix: str, *, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 qkv_bias: bool, o_bias: bool = False, window: int = 0,
                 position: PartSpec = PartSpec("none"), softmax_scale: Optional[float] = None,
                 v_dim: Optional[int] = None, out_scale: float = 1.0, names: Optional[dict] = None,
                 keep_first: int = 0, sink: bool = False, conv_taps: int = 0, qk_norm: Optional[str] = None,
                 qk_norm_eps: float = 0.0, out_gate: bool = False, has_kv: bool = True, shaped: bool = False,
                 cache_window: Optional[int] = None, cache_keep: Optional[int] = None) -> None:
        """``v_dim``: the values' size per head where it is not ``head_dim``.  ``out_scale``: a factor on the mixer's
        output (a mixer that runs beside another one).  ``names``: tensor names below the prefix where they differ
        from ``NAMES``.  ``keep_first``, ``sink``, ``conv_taps``, ``qk_norm`` ("rms"), ``out_gate``, ``has_kv``,
        ``shaped``: see the head of the file.  ``cache_window`` / ``cache_keep``: what the layer's pages must hold
        where that is more than its own window and kept tokens (another layer call reads them with a wider mask)."""
        super().__init__(prefix)
        self.keep_first, self.sink = (int(keep_first) if window else 0), bool(sink)
        if sink not in (False, True, "learned"):
            raise ValueError(f"attention: sink {sink!r} (known: False, True, 'learned')")
        self.sink_learned = sink == "learned"
        self.conv_taps, self.qk_norm, self.qk_norm_eps = int(conv_taps), qk_norm, float(qk_norm_eps)
        self.out_gate, self.has_kv = bool(out_gate), bool(has_kv)
        self.shaped = bool(shaped or self.conv_taps > 0 or qk_norm or out_gate or not has_kv)
        if qk_norm == "whole" and self.conv_taps > 0:
            raise ValueError("attention: a norm over the whole projections does not go with a convolution behind them")
        if self.conv_taps > K.PREP_MAX_TAPS:
            raise ValueError(f"attention: a convolution over {conv_taps} tokens (at most {K.PREP_MAX_TAPS})")
        if qk_norm not in (None, "rms", "unit", "whole"):
            raise ValueError(f"attention: qk_norm {qk_norm!r} (known: rms, unit, whole)")
        self.cache_window = int(window if cache_window is None else cache_window)
        self.cache_keep = int(self.keep_first if cache_keep is None else cache_keep) if self.cache_window else 0
        if n_heads % n_kv_heads:
            raise ValueError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        self.qk_dim, self.v_dim = int(head_dim), int(v_dim if v_dim is not None else head_dim)
        # the size the kernels see: a multiple of 16 that holds queries, keys and values
        laid = -(-max(self.qk_dim, self.v_dim) // 16) * 16
        self.padded = laid != self.qk_dim or laid != self.v_dim
        if not (16 <= laid <= 256):
            raise ValueError(f"attention: heads of {self.qk_dim} (values {self.v_dim}) exceed 256 "
                             "(the attention kernels take no larger head)")
        if self.padded and not self.shaped and not isinstance(make_part("position", position, prefix + ".position"), _NoRotation):
            raise ValueError("attention: heads that are padded to the kernels' sizes take no rotation")
        head_dim = laid
        self.hidden, self.n_heads, self.n_kv_heads, self.head_dim = hidden, n_heads, n_kv_heads, head_dim
        self.qkv_bias, self.o_bias, self.window = bool(qkv_bias), bool(o_bias), int(window)
        self.scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(self.qk_dim)
        self.out_scale = float(out_scale)
        self.names = {**NAMES, **(names or {})}
        self.position = make_part("position", position, prefix + ".position")
        self.q_dim = n_heads * head_dim
        self.kv_dim = n_kv_heads * head_dim
        # the shaped form's stacked projection: [q | k | v | gate] at the stored sizes, its width a multiple of 8
        kv = self.n_kv_heads if self.has_kv else 0
        self.in_rows = [("q", 0, n_heads * self.qk_dim)]
        self.in_rows.append(("k", self.in_rows[-1][1] + self.in_rows[-1][2], kv * self.qk_dim))
        self.in_rows.append(("v", self.in_rows[-1][1] + self.in_rows[-1][2], kv * self.v_dim))
        self.in_rows.append(("gate", self.in_rows[-1][1] + self.in_rows[-1][2], n_heads * self.v_dim if self.out_gate else 0))
        self.in_used = self.in_rows[-1][1] + self.in_rows[-1][2]
        self.in_width = -(-self.in_used // 8) * 8
        self.channels = self.in_rows[3][1]   # what the convolution covers: q, k, v

    def sub_parts(self):
        return [self.position]

    # -- weights ------------------------------------------------------------
    def _stored(self):
        """(role, rows as stored) of the three projections."""
        return [("q", self.n_heads * self.qk_dim), ("k", self.n_kv_heads * self.qk_dim), ("v", self.n_kv_heads * self.v_dim)]

    def param_shapes(self):
        if self.shaped:
            if getattr(self, "_laid_out", False):   # bind has widened the output projection to the kernels' head size
                return {n: tuple(t.shape) for n, t in self.params.items()}
            shapes = {"w_in": (self.in_width, self.hidden)}
            if self.qkv_bias:
                shapes["b_in"] = (self.in_width,)
            if self.conv_taps > 0:
                shapes["conv"] = (self.channels, self.conv_taps)
            shapes["wo_stored" if self.head_dim != self.v_dim else "wo"] = (self.hidden, self.n_heads * self.v_dim)
            if self.o_bias:
                shapes["bo"] = (self.hidden,)
            shapes.update(self._extra_shapes())
            return shapes
        if self.padded and "wqkv" not in self.params:
            # loaded as stored, laid out for the kernels in bind
            shapes = {f"w{r}_stored": (n, self.hidden) for r, n in self._stored()}
            shapes["wo_stored"] = (self.hidden, self.n_heads * self.v_dim)
            if self.qkv_bias:
                shapes.update({f"b{r}_stored": (n,) for r, n in self._stored()})
        elif self.padded:
            return {n: tuple(t.shape) for n, t in self.params.items()}
        else:
            shapes = {"wqkv": (self.q_dim + 2 * self.kv_dim, self.hidden), "wo": (self.hidden, self.q_dim)}
            if self.qkv_bias:
                shapes["bqkv"] = (self.q_dim + 2 * self.kv_dim,)
        if self.o_bias:
            shapes["bo"] = (self.hidden,)
        shapes.update(self._extra_shapes())
        return shapes

    def _extra_shapes(self):
        """A learned sink per query head; the weights of a norm over the whole q and k projections."""
        s = {}
        if self.sink_learned:
            s["sink"] = (self.n_heads,)
        if self.qk_norm == "whole":
            s["q_norm"] = (self.n_heads * self.qk_dim,)
            if self.has_kv:
                s["k_norm"] = (self.n_kv_heads * self.qk_dim,)
        return s

    def _extra_sources(self):
        p, nm = self.prefix, self.names
        kinds = {"sink": "bias", "q_norm": "norm", "k_norm": "norm"}
        return [TensorSource(f"{p}.{nm[name]}", shape, name, 0, kinds[name]) for name, shape in self._extra_shapes().items()]

    def sources(self):
        p, nm = self.prefix, self.names
        if self.shaped:
            out = [TensorSource(f"{p}.{nm[r]}", (n, self.hidden), "w_in", row0) for r, row0, n in self.in_rows if n]
            if self.qkv_bias:
                out += [TensorSource(f"{p}.{nm[r + '_bias']}", (n,), "b_in", row0, "bias")
                        for r, row0, n in self.in_rows[:3] if n]
            if self.conv_taps > 0:
                out += [TensorSource(f"{p}.{nm[r + '_conv']}", (n, self.conv_taps), "conv", row0, "bias")
                        for r, row0, n in self.in_rows[:3] if n]
            out.append(TensorSource(f"{p}.{nm['o']}", (self.hidden, self.n_heads * self.v_dim),
                                    "wo_stored" if self.head_dim != self.v_dim else "wo"))
            if self.o_bias:
                out.append(TensorSource(f"{p}.{nm['o_bias']}", (self.hidden,), "bo", 0, "bias"))
            return out + self._extra_sources()
        if self.padded:
            out = [TensorSource(f"{p}.{nm[r]}", (n, self.hidden), f"w{r}_stored") for r, n in self._stored()]
            if self.qkv_bias:
                out += [TensorSource(f"{p}.{nm[r + '_bias']}", (n,), f"b{r}_stored", 0, "bias") for r, n in self._stored()]
            out.append(TensorSource(f"{p}.{nm['o']}", (self.hidden, self.n_heads * self.v_dim), "wo_stored"))
        else:
            rows = [("q", 0, self.q_dim), ("k", self.q_dim, self.kv_dim), ("v", self.q_dim + self.kv_dim, self.kv_dim)]
            out = [TensorSource(f"{p}.{nm[r]}", (size, self.hidden), "wqkv", row0) for r, row0, size in rows]
            if self.qkv_bias:
                out += [TensorSource(f"{p}.{nm[r + '_bias']}", (size,), "bqkv", row0, "bias") for r, row0, size in rows]
            out.append(TensorSource(f"{p}.{nm['o']}", (self.hidden, self.q_dim), "wo"))
        if self.o_bias:
            out.append(TensorSource(f"{p}.{nm['o_bias']}", (self.hidden,), "bo", 0, "bias"))
        return out + self._extra_sources()

    def bind(self, rt) -> None:
        self._scale = None
        # what the kernels get as the sink: a flag, or the learned scores as float32
        self._sink_arg = self.params["sink"].float().contiguous() if self.sink_learned else self.sink
        if self.out_scale != 1.0:
            self._scale = rt.shared_object(("row_scale", self.out_scale), lambda: torch.full(
                (rt.max_tokens,), self.out_scale, dtype=torch.float32, device=rt.device))
        if self.shaped:
            P = self.params
            if "wo_stored" in P:
                # zero columns behind every head of the output projection (the kernels' head size is wider than a value)
                wo = torch.zeros((self.hidden, self.q_dim), dtype=P["wo_stored"].dtype, device=P["wo_stored"].device)
                wo.view(self.hidden, self.n_heads, self.head_dim)[:, :, : self.v_dim] = P["wo_stored"].view(self.hidden, self.n_heads, self.v_dim)
                del P["wo_stored"]
                P["wo"] = wo
                self._laid_out = True
            P["w_in"][self.in_used:].zero_()
            if "b_in" in P:
                P["b_in"][self.in_rows[3][1]:].zero_()   # the gate and the padding have no bias
            return
        if not self.padded or "wqkv" in self.params:
            return
        # the stored heads at the kernels' head size: zero rows behind every head of q, k and v, zero columns behind
        # every head of the output projection
        D, P = self.head_dim, self.params
        some = P["wq_stored"]
        wqkv = torch.zeros((self.q_dim + 2 * self.kv_dim, self.hidden), dtype=some.dtype, device=some.device)
        bqkv = torch.zeros((self.q_dim + 2 * self.kv_dim,), dtype=P["bq_stored"].dtype, device=some.device) if self.qkv_bias else None
        row0 = 0
        for r, heads, size in (("q", self.n_heads, self.qk_dim), ("k", self.n_kv_heads, self.qk_dim),
                               ("v", self.n_kv_heads, self.v_dim)):
            wqkv[row0:row0 + heads * D].view(heads, D, self.hidden)[:, :size] = P[f"w{r}_stored"].view(heads, size, self.hidden)
            if bqkv is not None:
                bqkv[row0:row0 + heads * D].view(heads, D)[:, :size] = P[f"b{r}_stored"].view(heads, size)
            row0 += heads * D
        wo = torch.zeros((self.hidden, self.q_dim), dtype=some.dtype, device=some.device)
        wo.view(self.hidden, self.n_heads, D)[:, :, : self.v_dim] = P["wo_stored"].view(self.hidden, self.n_heads, self.v_dim)
        for name in [n for n in P if n.endswith("_stored")]:
            del P[name]
        P["wqkv"], P["wo"] = wqkv, wo
        if bqkv is not None:
            P["bqkv"] = bqkv

    def kernel_modules(self, dtype):
        special = bool(self.keep_first or self.sink)   # such an attention runs on the kernels that know of both
        return (["elementwise", "gemm_simt", "gemv", "attention"] + (["short_conv"] if self.shaped else [])
                + (["gemm_skinny", "gemm_tc", "attention_mma", "attention_tc", "attention_gqa"] if dtype == torch.bfloat16 else []))

    def cache_needs(self):
        state = None
        if self.conv_taps > 1:
            state = StateSpec((self.channels * (self.conv_taps - 1),), torch.float32)
        return PagedKvSpec(self.n_kv_heads, self.head_dim, self.cache_window, keep_first=self.cache_keep), state

    def step_plans(self):
        return [AttentionTiles()]

    # -- forward ------------------------------------------------------------
    def _forward_shaped(self, h, batch, cache, residual, rt, accumulate) -> None:
        T = batch.T
        gb = batch.groups[cache.group]
        proj = rt.rows(f"attention.proj{self.in_width}", self.in_width, torch.float32, T)
        K.linear(h, self.params["w_in"], proj, bias=self.params.get("b_in"))
        table = self.position.rotary_table()
        if table is not None and (table.magnitude != 1.0 or table.interleaved):
            raise ValueError("attention: the shaped form rotates half-split pairs without a factor on cosine and sine")
        if self.conv_taps > 1 and not cache.writes:
            raise ValueError("attention: a layer call that reads another call's cache has no convolution state of its own")
        q = rt.rows("attention.q", self.q_dim, rt.dtype, T)
        kv = self.n_kv_heads if self.has_kv else 0
        D = self.head_dim
        if self.qk_norm == "whole":
            spans = [(self.in_rows[0][1], self.in_rows[0][2], self.params["q_norm"])]
            if kv:
                spans.append((self.in_rows[1][1], self.in_rows[1][2], self.params["k_norm"]))
            K.span_rmsnorm(proj, spans, self.qk_norm_eps)
        K.head_prep(proj, offsets=[r[1] for r in self.in_rows[:3]], heads=(self.n_heads, kv, kv),
                    dims=(self.qk_dim, self.qk_dim, self.v_dim), laid=(D, D, D), state_slots=batch.state_slots,
                    seg_q0=batch.seg_q0, seg_qn=batch.seg_qn, n_seg=batch.n_seg,
                    longest_new=max(batch.host_seg_qn) if batch.host_seg_qn else T, positions=batch.positions, q_out=q,
                    pool=cache.pool if kv else None, slots=gb.slots if kv else None, page_tokens=gb.page_tokens,
                    write_kv=cache.writes, conv=self.params.get("conv"), state=cache.state if self.conv_taps > 1 else None,
                    inv_freq=table.inv_freq if table else None, rot=table.rot_dim if table else 0,
                    norm=None if self.qk_norm == "whole" else self.qk_norm,
                    eps=self.qk_norm_eps)
        o = rt.rows("attention.o", self.q_dim, rt.dtype, T)
        self._attend(q, o, batch, cache, gb, rt)
        if self.out_gate:
            K.gate_rows(o, proj, self.in_rows[3][1], n_heads=self.n_heads, dim=self.v_dim, laid=D)
        K.linear(o, self.params["wo"], residual, bias=self.params.get("bo"), accumulate=accumulate, row_scale=self._scale)

    def forward(self, h, batch, cache, residual, rt, accumulate=True) -> None:
        if self.shaped:
            return self._forward_shaped(h, batch, cache, residual, rt, accumulate)
        T = batch.T
        gb = batch.groups[cache.group]
        qkv = rt.rows("attention.qkv", self.q_dim + 2 * self.kv_dim, rt.dtype, T)
        K.linear(h, self.params["wqkv"], qkv, bias=self.params.get("bqkv"))
        table = self.position.rotary_table()
        if table is not None and table.magnitude != 1.0:
            raise ValueError("attention: the fused rotation takes no factor on cosine and sine")
        if table is None:
            # an encoding without a rotary table transforms q and k in place itself
            self.position.apply(qkv[:, : self.q_dim], qkv[:, self.q_dim : self.q_dim + self.kv_dim],
                                batch.positions)
        q = rt.rows("attention.q", self.q_dim, rt.dtype, T)
        K.rope_kv_write(
            qkv, batch.positions, table.inv_freq if table else None, q, cache.pool, gb.slots,
            n_heads=self.n_heads, n_kv_heads=self.n_kv_heads, head_dim=self.head_dim,
            rot_dim=table.rot_dim if table else 0, interleaved=table.interleaved if table else False,
            page_tokens=gb.page_tokens, write_kv=cache.writes,
        )
        o = rt.rows("attention.o", self.q_dim, rt.dtype, T)
        self._attend(q, o, batch, cache, gb, rt)
        K.linear(o, self.params["wo"], residual, bias=self.params.get("bo"), accumulate=accumulate, row_scale=self._scale)

    def _attend(self, q, o, batch, cache, gb, rt) -> None:
        """o = attention of the step's queries ``q`` over the layer's pages, by the kernels that fit the step."""
        T = batch.T
        special = bool(self.keep_first or self.sink)
        extra = dict(keep_first=self.keep_first, sink=self._sink_arg) if special else {}
        common = dict(seg_q0=batch.seg_q0, seg_qn=batch.seg_qn, seg_ctx=batch.seg_ctx,
                      block_table=gb.block_table, n_heads=self.n_heads, n_kv_heads=self.n_kv_heads,
                      head_dim=self.head_dim, page_tokens=gb.page_tokens, window=self.window,
                      scale=self.scale)
        tiles = batch.plans[AttentionTiles.key]
        # splits of 128 keys that cover the longest context (all that the block table can describe when the
        # step's launches must not depend on its lengths)
        cap_splits = (gb.block_table.shape[1] * gb.page_tokens - 1) // K.DECODE_SPLIT + 1
        max_splits = cap_splits if batch.static_shapes else min(cap_splits, (max(batch.longest, 1) - 1) // K.DECODE_SPLIT + 1)
        if tiles["n_chunk_items"]:
            # few query tiles behind a long context: the keys of every tile are cut into ranges
            keys = max_splits * K.DECODE_SPLIT
            if self.window > 0:
                keys = min(keys, self.window + self.keep_first + K.TC_ATTN_QUERY_BLOCK)
            if K.attn_chunk_tc_takes(q, self.head_dim, gb.page_tokens, T, keys):
                n_splits = K.attn_chunk_tc_splits(tiles["n_chunk_items64"], self.n_heads, keys)
                part_o = part_ml = None
                if n_splits > 1:
                    n_o, n_ml = K.attn_chunk_tc_scratch()
                    part_o = rt.buf("attention.chunk_tc_part_o", (n_o,), torch.float32)
                    part_ml = rt.buf("attention.chunk_tc_part_ml", (n_ml,), torch.float32)
                K.attn_chunk_tc(q, cache.pool, o, items=tiles["chunk_items64"], n_items=tiles["n_chunk_items64"],
                                n_splits=n_splits, part_o=part_o, part_ml=part_ml, **extra, **common)
            elif K.attn_chunk_mma_takes(q, self.head_dim):
                n_splits = K.attn_chunk_mma_splits(tiles["n_chunk_items64"], self.n_heads, keys)
                part_o = part_ml = None
                if n_splits > 1:
                    n_o, n_ml = K.attn_chunk_mma_scratch(self.head_dim)
                    part_o = rt.buf("attention.chunk_part_o", (n_o,), torch.float32)
                    part_ml = rt.buf("attention.chunk_part_ml", (n_ml,), torch.float32)
                K.attn_chunk_mma(q, cache.pool, o, items=tiles["chunk_items64"], n_items=tiles["n_chunk_items64"],
                                 n_splits=n_splits, part_o=part_o, part_ml=part_ml, **extra, **common)
            else:
                K.attn_chunk(q, cache.pool, o, items=tiles["chunk_items"], n_items=tiles["n_chunk_items"], **extra, **common)
        if tiles["n_decode_items"]:
            n = tiles["n_decode_items"]
            # scratch sized once, for the longest context that the block table can describe
            units = K.decode_units(rt.max_segments, self.n_heads, self.head_dim, q.dtype, cap_splits, rt.device,
                                   gb.page_tokens, self.n_kv_heads, fixed_ranges=self.keep_first > 0)
            part_o = rt.buf("attention.part_o", (units * self.head_dim,), torch.float32)
            part_ml = rt.buf("attention.part_ml", (2 * units,), torch.float32)
            counters = rt.shared_object(
                ("attention.counters", rt.max_segments * self.n_heads),
                lambda: torch.zeros(rt.max_segments * self.n_heads, dtype=torch.int32, device=rt.device),
            )
            K.attn_decode(q, cache.pool, o, items=tiles["decode_items"], n_items=n, part_o=part_o,
                          part_ml=part_ml, counters=counters, max_splits=max_splits, **extra, **common)


register_mixer("attention", Attention)
