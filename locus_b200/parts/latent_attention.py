"""Latent attention: queries and keys/values projected through low-rank latents, one latent row per token
in the paged cache for all heads, a sliding window and a sink in the softmax.

Per token, with h the mixer's input (H heads; per head ``nope_dim`` unrotated and ``rot_dim`` rotated
query/key dimensions, values of ``v_dim``):

    c_q = rmsnorm(W_dq h) * g_q                    the query latent (q_rank)
    q   = W_uq c_q                                 head by head [nope_dim | rot_dim]
    c   = rmsnorm((W_dkv h)[:kv_rank]) * g_kv      the key/value latent (kv_rank)
    k_r = (W_dkv h)[kv_rank:]                      one rotated key part for all heads (rot_dim, not normed)
    score(t, j, head) = (q_nope . (W_uk c_j) + rot(q_rot) . rot(k_r_j)) * scale,   value_j = W_uv c_j

Only c and rot(k_r) are cached: a row of kv_rank + rot_dim elements per token.  The heads' keys and values
are never expanded per key: W_uk is applied to the query instead (q_abs = W_uk^T q_nope), attention runs over
the cached rows as they are, and W_uv is applied to the attention's output (sum_j p_j c_j).  The two per-head
products are grouped products (the heads in the place of experts) over head-major rows [head][token].

Options: ``q_rank`` 0: no query latent, q = W_q h directly.  ``out_gate``: the concatenated heads' outputs are
multiplied by sigmoid(W_g h) in front of the output projection.  ``has_kv`` off: the layer has no W_dkv; it reads the
cache rows of the layer call that the run order names (that layer's latent and rotated key part as cached) with its own
W_uk, W_uv and queries.  The rotated parts' pairs are interleaved, (2i, 2i + 1), or the halves (i, i + dims/2), as the
position encoding says.

The softmax's denominator may hold a learned sink per head, exp(sink_h), without a key or a value.  A query at
position p sees the keys j with p - window < j <= p (window 0: all).  Scores, softmax, the norms' statistics,
positions and angles are float32 (angles are formed in float64 and rounded once).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .. import kernels as K
from .base import Mixer, PagedKvSpec, PartSpec, StepPlan, TensorSource, make_part, register_mixer


class LatentTiles(StepPlan):
    """Work items of the latent attention kernels: tiles of ``tile`` queries over every segment, one token or
    many, ordered by the position of their first query (the kernels walk the list from its end, so the tiles
    with the most keys start first)."""

    def __init__(self, tile: int = K.LATENT_QUERY_TILE) -> None:
        from ..cache import native

        self._lib = native.lib()
        self.tile = int(tile)
        self.key = ("latent_attention.tiles", self.tile)

    def capacity(self, max_tokens: int, max_segments: int) -> int:
        return 2 * (max_tokens // self.tile + max_segments)

    def build(self, seg_q0, seg_qn, seg_ctx, out):
        n = self._lib.locus_plan_query_tiles(len(seg_qn), seg_qn.ctypes.data, self.tile, 1,
                                             out.ctypes.data, len(out))
        if n < 0:
            raise ValueError("latent attention: the step has more query tiles than the plan's capacity holds")
        self._lib.locus_sort_tiles_by_position(n, out.ctypes.data, seg_ctx.ctypes.data)
        return {"items": (0, 2 * n, (-1, 2)), "n_items": n}


class HeadTiles(StepPlan):
    """Tile lists of the per-head grouped products over head-major rows [H * T, ...] (head h owns the rows
    h * T .. (h + 1) * T): (head, first row, rows) of every tile, their number, and the heads' row offsets.  The
    tile's size follows the kernel that the product runs on (``K.head_tile``)."""

    def __init__(self, n_heads: int, dtype: torch.dtype, widths_ok: bool) -> None:
        self.n_heads, self.dtype, self.widths_ok = int(n_heads), dtype, bool(widths_ok)
        self.key = ("latent_attention.head_tiles", self.n_heads, str(dtype), self.widths_ok)

    def capacity(self, max_tokens: int, max_segments: int) -> int:
        tiles = self.n_heads * (max_tokens // 8 + 1)
        return 3 * tiles + 1 + self.n_heads + 1

    def build(self, seg_q0, seg_qn, seg_ctx, out):
        H, T = self.n_heads, int(seg_qn.sum())
        tile = K.head_tile(T, self.dtype, self.widths_ok)
        per = -(-T // tile)
        n = H * per
        if 3 * n + H + 2 > len(out):
            raise ValueError("latent attention: the step has more head tiles than the plan's capacity holds")
        first = np.arange(per, dtype=np.int32) * tile
        out[0:n] = np.repeat(np.arange(H, dtype=np.int32), per)
        out[n:2 * n] = (np.arange(H, dtype=np.int32)[:, None] * T + first[None, :]).reshape(-1)
        out[2 * n:3 * n] = np.tile(np.minimum(tile, T - first), H)
        out[3 * n] = n
        out[3 * n + 1:3 * n + 2 + H] = np.arange(H + 1, dtype=np.int32) * T
        return {"tile_head": (0, n, None), "tile_row0": (n, n, None), "tile_rows": (2 * n, n, None),
                "n_tiles": (3 * n, 1, None), "offsets": (3 * n + 1, H + 1, None), "tile": tile, "count": n}


class LatentAttention(Mixer):
    can_overwrite = True

    def __init__(self, prefix: str, *, hidden: int, n_heads: int, nope_dim: int, rot_dim: int, v_dim: int,
                 q_rank: int, kv_rank: int, scale: float, eps: float, window: int = 0, sink: bool = False,
                 position: PartSpec = PartSpec("none"), names: Optional[dict] = None, out_gate: bool = False,
                 has_kv: bool = True) -> None:
        """``position``: the encoding of the rotated parts (a "rotary" spec over ``rot_dim`` with interleaved
        pairs, or "none").  ``names``: tensor names below the prefix where they differ from the defaults."""
        super().__init__(prefix)
        if kv_rank > K.LATENT_MAX_RANK:
            raise ValueError(f"latent_attention: kv_rank {kv_rank} exceeds {K.LATENT_MAX_RANK} "
                             "(the attention kernel keeps a query's latent sum in registers)")
        self.hidden, self.H, self.dn, self.dr, self.dv = int(hidden), int(n_heads), int(nope_dim), int(rot_dim), int(v_dim)
        self.q_rank, self.kv_rank, self.scale, self.eps = int(q_rank), int(kv_rank), float(scale), float(eps)
        self.window, self.has_sink = int(window), bool(sink)
        self.out_gate, self.has_kv = bool(out_gate), bool(has_kv)
        if self.q_rank < 0:
            raise ValueError(f"latent_attention: q_rank {q_rank}")
        self.position = make_part("position", position, prefix + ".position")
        self.names = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
                      "uv": "uv", "sink": "sink", "o": "o", "q": "q", "gate": "g", **(names or {})}
        self.row = self.kv_rank + self.dr
        # the product whose result stays float32: [query latent | key/value latent and shared key part | gate]
        self.n_down = self.q_rank + (self.row if self.has_kv else 0)
        self.n_gate = self.H * self.dv if self.out_gate else 0
        self.down_width = -(-(self.n_down + self.n_gate) // 8) * 8
        # whether the per-head products may run on the kernels that want rows of whole 16-byte pieces
        self.widths_ok = self.dn % 8 == 0 and self.kv_rank % 8 == 0

    def sub_parts(self):
        return [self.position]

    # -- weights ------------------------------------------------------------
    def param_shapes(self):
        s = {"w_uq": (self.H * (self.dn + self.dr), self.q_rank or self.hidden), "w_uk": (self.H * self.dn, self.kv_rank),
             "w_uv": (self.H * self.dv, self.kv_rank), "w_o": (self.hidden, self.H * self.dv)}
        if self.n_down + self.n_gate:
            s["w_down"] = (self.down_width, self.hidden)
        if self.q_rank:
            s["g_q"] = (self.q_rank,)
        if self.has_kv:
            s["g_kv"] = (self.kv_rank,)
        if self.has_sink:
            s["sink"] = (self.H,)
        return s

    def sources(self):
        p, n = self.prefix, self.names
        out = []
        if self.q_rank:
            out += [TensorSource(f"{p}.{n['dq']}", (self.q_rank, self.hidden), "w_down", 0),
                    TensorSource(f"{p}.{n['dq_norm']}", (self.q_rank,), "g_q", 0, "norm"),
                    TensorSource(f"{p}.{n['uq']}", (self.H * (self.dn + self.dr), self.q_rank), "w_uq")]
        else:
            out.append(TensorSource(f"{p}.{n['q']}", (self.H * (self.dn + self.dr), self.hidden), "w_uq"))
        if self.has_kv:
            out += [TensorSource(f"{p}.{n['dkv']}", (self.row, self.hidden), "w_down", self.q_rank),
                    TensorSource(f"{p}.{n['dkv_norm']}", (self.kv_rank,), "g_kv", 0, "norm")]
        if self.out_gate:
            out.append(TensorSource(f"{p}.{n['gate']}", (self.n_gate, self.hidden), "w_down", self.n_down))
        out += [TensorSource(f"{p}.{n['uk']}", (self.H * self.dn, self.kv_rank), "w_uk"),
               TensorSource(f"{p}.{n['uv']}", (self.H * self.dv, self.kv_rank), "w_uv"),
               TensorSource(f"{p}.{n['o']}", (self.hidden, self.H * self.dv), "w_o")]
        if self.has_sink:
            out.append(TensorSource(f"{p}.{n['sink']}", (self.H,), "sink", 0, "bias"))
        return out

    def kernel_modules(self, dtype):
        return ["elementwise", "gemm_simt", "gemv", "latent_attention"] + (["short_conv"] if self.out_gate else []) + (
            ["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def cache_needs(self):
        return PagedKvSpec(1, self.row, self.window, has_v=False), None

    def step_plans(self):
        return [self._query_tiles, self._head_tiles]

    @property
    def _query_tiles(self) -> LatentTiles:
        """Tiles of 16 queries for the CUDA-core kernel, or of 64 / (heads that share a block) for the tensor-core
        kernel where it takes this mixer's sizes."""
        dtype = getattr(self, "_dtype", torch.float32)
        self._mma = K.latent_attn_mma_takes(dtype, self.kv_rank, self.dr)
        self._head_shift = K.latent_mma_head_shift(self.H)
        return LatentTiles(64 >> self._head_shift if self._mma else K.LATENT_QUERY_TILE)

    @property
    def _head_tiles(self) -> HeadTiles:
        ht = getattr(self, "_ht", None)
        if ht is None or ht.dtype != getattr(self, "_dtype", torch.float32):
            ht = self._ht = HeadTiles(self.H, getattr(self, "_dtype", torch.float32), self.widths_ok)
        return ht

    def bind(self, rt) -> None:
        self._dtype = rt.dtype
        # W_uk per head, transposed: the weight [kv_rank, nope_dim] of the product that carries a head's query into
        # the latent space (a layout of the same numbers)
        self._w_uk_t = self.params["w_uk"].view(self.H, self.dn, self.kv_rank).transpose(1, 2).contiguous()
        self._w_uv = self.params["w_uv"].view(self.H, self.dv, self.kv_rank)
        self._sink = self.params["sink"].float().contiguous() if self.has_sink else None
        self._gq, self._gkv = self.params.get("g_q"), self.params.get("g_kv")
        if "w_down" in self.params:
            self.params["w_down"][self.n_down + self.n_gate:].zero_()
        self._tiles_key = self._query_tiles.key   # also settles which attention kernel this mixer runs

    # -- forward ------------------------------------------------------------
    def forward(self, h, batch, cache, residual, rt, accumulate=True) -> None:
        T, H = batch.T, self.H
        gb = batch.groups[cache.group]
        table = self.position.rotary_table()
        freq = table.freq64 if table is not None else None
        pairs = table.rot_dim // 2 if table is not None else 0
        mag = table.magnitude if table is not None else 1.0
        half = table is not None and not table.interleaved
        if not self.has_kv and cache.writes:
            raise ValueError("latent_attention: a layer without a latent of its own must read another call's cache")
        # the down-projections (and the gate's) as one product, kept in float32 for the norms and the sigmoid
        down = None
        if self.n_down + self.n_gate:
            down = rt.rows(f"latent.down{self.down_width}", self.down_width, torch.float32, T)
            K.linear(h, self.params["w_down"], down)
        cq = rt.rows("latent.cq", self.q_rank, rt.dtype, T) if self.q_rank else None
        if self.n_down:
            K.latent_prep(down[:, :self.n_down], batch.positions, freq, mag,
                          self._gq, self._gkv, self.eps, cq, cache.pool, gb.slots, q_rank=self.q_rank, kv_rank=self.kv_rank,
                          rot_dim=self.dr, rot_pairs=pairs, write=cache.writes and self.has_kv, half_split=half)
        q = rt.rows("latent.q", H * (self.dn + self.dr), rt.dtype, T)
        K.linear(cq if self.q_rank else h, self.params["w_uq"], q)
        q_nope = rt.rows(f"latent.q_nope{self.dn}", self.dn, rt.dtype, H * T, per_token=H)
        q_rot = rt.rows("latent.q_rot", H * self.dr, rt.dtype, T)
        K.latent_q_split(q, batch.positions, freq, mag, q_nope, q_rot, n_heads=H, nope_dim=self.dn, rot_dim=self.dr,
                         rot_pairs=pairs, half_split=half)
        ht = batch.plans[self._head_tiles.key]
        lay = K.HeadLayout(H, ht["tile"], ht["offsets"], ht["tile_head"], ht["tile_row0"], ht["tile_rows"],
                           ht["n_tiles"], ht["count"])
        q_abs = rt.rows(f"latent.q_abs{self.kv_rank}", self.kv_rank, rt.dtype, H * T, per_token=H)
        K.linear(q_nope, self._w_uk_t, q_abs, layout=lay, n_rows=H * T, lists_ready=True)
        o_lat = rt.rows(f"latent.o_lat{self.kv_rank}", self.kv_rank, rt.dtype, H * T, per_token=H)
        tiles = batch.plans[self._tiles_key]
        common = dict(seg_q0=batch.seg_q0, seg_qn=batch.seg_qn, seg_ctx=batch.seg_ctx, block_table=gb.block_table,
                      items=tiles["items"], n_items=tiles["n_items"], n_tokens=T, n_heads=H, kv_rank=self.kv_rank,
                      rot_dim=self.dr, page_tokens=gb.page_tokens, window=self.window, scale=self.scale)
        if self._mma:
            # the most keys a query of this step sees (all that the block table can describe when the step's
            # launches must not depend on its lengths)
            keys = gb.block_table.shape[1] * gb.page_tokens if batch.static_shapes else max(batch.longest, 1)
            if self.window > 0:
                keys = min(keys, self.window + (64 >> self._head_shift))
            n_splits = K.latent_attn_mma_splits(tiles["n_items"], H, self._head_shift, keys)
            part_o = part_ml = None
            if n_splits > 1:
                n_o, n_ml = K.latent_attn_mma_scratch(self.kv_rank)
                part_o = rt.buf("latent.part_o", (n_o,), torch.float32)
                part_ml = rt.buf("latent.part_ml", (n_ml,), torch.float32)
            K.latent_attn_mma(q_abs, q_rot, cache.pool, self._sink, o_lat, head_shift=self._head_shift,
                              n_splits=n_splits, part_o=part_o, part_ml=part_ml, **common)
        else:
            K.latent_attn(q_abs, q_rot, cache.pool, self._sink, o_lat, **common)
        o_hm = rt.rows(f"latent.o_hm{self.dv}", self.dv, rt.dtype, H * T, per_token=H)
        K.linear(o_lat, self._w_uv, o_hm, layout=lay, n_rows=H * T, lists_ready=True)
        o = rt.rows("latent.o", H * self.dv, rt.dtype, T)
        K.heads_to_rows(o_hm, o, n_tokens=T, n_heads=H)
        if self.out_gate:
            K.gate_rows(o, down, self.n_down, n_heads=H, dim=self.dv, laid=self.dv)
        K.linear(o, self.params["w_o"], residual, accumulate=accumulate)


register_mixer("latent_attention", LatentAttention)
