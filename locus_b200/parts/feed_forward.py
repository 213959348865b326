"""Feed-forward parts: the dense SwiGLU MLP and the sparse mixture of experts.

Dense (src/locus/model/llama.cpp:493-503 of the reference):
    out = Wdown . (silu(Wgate . h) * (Wup . h)),  silu(g) = g / (1 + exp(-g))
    (``silu_mul``, src/locus/backend/cpu_ops.cpp:1736-1743).

Sparse (``moe_ffn`` llama.cpp:992-1077, ``moe_select`` llama.cpp:900-980):
    r = Wr . h; p = softmax(r) over all experts; pick top-k by k rounds of arg-max with
    strict '>' (ties to the lowest index); weight w_e = p_e / wsum * scale with
    wsum = sum of picked p_e when ``norm_topk`` else 1; out = sum over picked e, in pick
    order, of w_e * SwiGLU_e(h); then the shared expert, scaled by
    sigmoid(w_shared_gate . h) when it is gated (llama.cpp:1062-1076), is added.

Further forms: ``activation`` "relu2" (down(max(up h, 0)^2), no gate matrix) and "glu_clamp", a clamped gated unit

    g = min(W_gate h, limit),  u = clamp(W_up h, -limit, limit),  out = W_down (g sigmoid(1.702 g) (u + 1)),

which is an epilogue of the product kernels like SwiGLU (two accumulators); and ``weight_on_input``: a picked expert's
weight multiplies its input, out = sum expert_e(w_e h), not its output (the two first products carry the weight as a
factor, so the epilogue applies it to both sums in front of the clamps, in float32).

The batched form lays the (token, slot) pairs out by expert, runs each expert over its
tokens, and sums each token's pairs in slot order without atomics (the reference's
``moe_ffn_batch``, llama.cpp:1079-1235, does the same to stay byte-identical).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from .base import FeedForward, PendingAdd, TensorSource, register_feed_forward


ACTIVATIONS = ("swiglu", "relu2", "glu_clamp")
# tensor names below a feed-forward's prefix, by role; an architecture with other names passes its own
DENSE_NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}


class DenseMlp(FeedForward):
    """``activation`` "swiglu": down(silu(gate h) * (up h)); "relu2": down(max(up h, 0)^2), no gate matrix; "glu_clamp":
    the clamped gated unit of the head of the file with its ``limit``."""

    can_overwrite = True

    def __init__(self, prefix: str, *, hidden: int, intermediate: int, activation: str = "swiglu",
                 names: Optional[dict] = None, limit: float = 0.0) -> None:
        super().__init__(prefix)
        if activation not in ACTIVATIONS:
            raise ValueError(f"dense_mlp: activation {activation!r} (known: {', '.join(ACTIVATIONS)})")
        self.hidden, self.inter, self.activation, self.limit = int(hidden), int(intermediate), activation, float(limit)
        if activation == "glu_clamp" and not self.limit > 0:
            raise ValueError(f"dense_mlp: a clamped gated unit needs a positive limit, got {limit}")
        self.names = {**DENSE_NAMES, **(names or {})}

    def param_shapes(self):
        s = {"w_up": (self.inter, self.hidden), "w_down": (self.hidden, self.inter)}
        if self.activation in ("swiglu", "glu_clamp"):
            s["w_gate"] = (self.inter, self.hidden)
        return s

    def sources(self):
        p, n = self.prefix, self.names
        out = [TensorSource(f"{p}.{n['up']}", (self.inter, self.hidden), "w_up"),
               TensorSource(f"{p}.{n['down']}", (self.hidden, self.inter), "w_down")]
        if self.activation in ("swiglu", "glu_clamp"):
            out.insert(0, TensorSource(f"{p}.{n['gate']}", (self.inter, self.hidden), "w_gate"))
        return out

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def forward(self, h, batch, residual, rt, row_scale=None, accumulate=True) -> None:
        self.forward_down(self.forward_up(h, rt), residual, rt, row_scale, accumulate)

    # The two products on their own, for a caller that has something to do between them (the shared expert of a
    # routed feed-forward starts before the router has made the scale of its second product).
    def forward_up(self, h, rt) -> torch.Tensor:
        act = rt.rows(f"dense_mlp.act{self.inter}", self.inter, rt.dtype, h.shape[0])
        if self.activation == "swiglu":
            K.linear(h, self.params["w_gate"], act, w2=self.params["w_up"])
        elif self.activation == "glu_clamp":
            K.linear(h, self.params["w_gate"], act, w2=self.params["w_up"], act="glu_clamp", act_limit=self.limit)
        else:
            K.linear(h, self.params["w_up"], act, act="relu2")
        return act

    def forward_down(self, act, residual, rt, row_scale=None, accumulate=True) -> None:
        K.linear(act, self.params["w_down"], residual, accumulate=accumulate, row_scale=row_scale)


# Up to this many tokens in a step the shared expert's first product starts beside the router instead of behind it
# (decode steps of the 2.7B sizes at 4,096 tokens of context: 1.995 -> 1.81 ms at one request, 4.14 -> 3.97 at 8,
# 6.83 -> 6.40 at 16, 9.00 -> 8.88 at 32; at 64 the router and the product get in each other's way: 13.27 -> 13.37).
SHARED_EARLY_TOKENS = 32
SHARED_OVERLAP_FROM = 1024   # steps of at least this many tokens ...
SHARED_OVERLAP_ROWS = 192    # ... and at most this many rows per routed expert run the shared expert on the side stream


# tensor names below a routed feed-forward's prefix ({e}: the expert's number)
MOE_NAMES = {"router": "gate.weight", "router_bias": "gate.bias", "selection_bias": "gate.selection_bias",
             "expert_gate": "experts.{e}.gate_proj.weight", "expert_up": "experts.{e}.up_proj.weight",
             "expert_down": "experts.{e}.down_proj.weight", "shared": "shared_expert",
             "shared_gate": "shared_expert_gate.weight"}


class SparseMoe(FeedForward):
    """Softmax top-k routed experts plus an optional (gated) shared expert; the experts are SwiGLU layers or, with
    ``activation`` "relu2", down(max(up h, 0)^2)."""

    can_overwrite = True

    def __init__(self, prefix: str, *, hidden: int, n_experts: int, top_k: int, norm_topk: bool,
                 expert_intermediate: int, shared_intermediate: int = 0, shared_gate: bool = True,
                 weight_scale: float = 1.0, score_fn: str = "softmax", selection_bias: bool = False,
                 n_group: int = 1, n_group_used: int = 1, activation: str = "swiglu", router_bias: bool = False,
                 names: Optional[dict] = None, shared_names: Optional[dict] = None, n_identity: int = 0,
                 group_score: str = "top2", limit: float = 0.0, shared_limit: Optional[float] = None,
                 weight_on_input: bool = False) -> None:
        """``router_bias``: the router has a bias [n_experts] that is part of its logits (selection and weights
        alike; with softmax scores and ``norm_topk`` the weights are then the softmax over the picked logits).
        ``names`` / ``shared_names``: tensor names where they differ from ``MOE_NAMES`` / ``DENSE_NAMES``.
        ``score_fn``: "softmax" over all experts or "sigmoid" of each router logit; ``selection_bias``:
        a float32 tensor ``<prefix>.gate.selection_bias`` [n_experts] is added to the scores for the
        selection only; ``n_group`` > 1: group-limited routing with ``n_group_used`` groups (the
        parameters of the reference's ``moe_select``, src/locus/model/llama.cpp:900-980); ``group_score``: what a group
        is judged by, "top2" (the sum of its two best selection scores) or "best" (its best one).
        ``n_identity``: the router has that many outputs more than there are experts with weights; they stand for
        experts whose output is their input (times the weight).  Scores, selection bias, groups and top-k run over
        all ``n_experts + n_identity`` router outputs.  ``limit`` / ``shared_limit``: the clamps of "glu_clamp" experts
        and of the shared one (default: the experts').  ``weight_on_input``: see the head of the file ("glu_clamp" only)."""
        super().__init__(prefix)
        self.limit, self.weight_on_input = float(limit), bool(weight_on_input)
        if activation == "glu_clamp" and not self.limit > 0:
            raise ValueError(f"sparse_moe: clamped gated experts need a positive limit, got {limit}")
        if self.weight_on_input and (activation != "glu_clamp" or n_identity):
            raise ValueError("sparse_moe: the weight on an expert's input goes with glu_clamp experts and no identity experts")
        self.n_identity = int(n_identity)
        if self.n_identity < 0:
            raise ValueError(f"sparse_moe: {n_identity} identity experts")
        self.R = int(n_experts) + self.n_identity        # the router's outputs
        if not (1 <= top_k <= self.R):
            raise ValueError(f"sparse_moe: top_k {top_k} must be within 1..{self.R}")
        if group_score not in K.GROUP_SCORES:
            raise ValueError(f"sparse_moe: group score {group_score!r} (known: {', '.join(K.GROUP_SCORES)})")
        self.group_score = group_score
        if score_fn not in K.SCORE_FUNCTIONS:
            raise ValueError(f"sparse_moe: score function {score_fn!r} (known: {', '.join(K.SCORE_FUNCTIONS)})")
        if not (1 <= n_group <= 32) or self.R % n_group or not (1 <= n_group_used <= n_group):
            raise ValueError(f"sparse_moe: {n_group} groups ({n_group_used} used) do not fit {self.R} router outputs")
        self.score_fn, self.has_sel_bias = score_fn, bool(selection_bias)
        self.n_group, self.n_group_used = int(n_group), int(n_group_used)
        self.hidden, self.E, self.k = int(hidden), int(n_experts), int(top_k)
        self.norm_topk, self.I, self.Is = bool(norm_topk), int(expert_intermediate), int(shared_intermediate)
        self.shared_gate = bool(shared_gate) and self.Is > 0
        self.weight_scale = float(weight_scale)
        if activation not in ACTIVATIONS:
            raise ValueError(f"sparse_moe: activation {activation!r} (known: {', '.join(ACTIVATIONS)})")
        self.activation, self.has_router_bias = activation, bool(router_bias)
        self.names = {**MOE_NAMES, **(names or {})}
        self.shared = (DenseMlp(f"{prefix}.{self.names['shared']}", hidden=hidden, intermediate=self.Is,
                                activation=activation, names=shared_names,
                                limit=self.limit if shared_limit is None else float(shared_limit))
                       if self.Is > 0 else None)
        self._layout = None
        self._scratch = None
        self._router_all = None
        # telemetry hook: called with (prefix, ids [T, k], weights [T, k]) after routing; the
        # reference counts expert hits per layer the same way (src/locus/model/moe_stats.cpp:23-78)
        self.observer = None

    def sub_parts(self):
        return [self.shared] if self.shared is not None else []

    def param_shapes(self):
        s = {
            "router": (self.R, self.hidden),
            "up_exps": (self.E, self.I, self.hidden),
            "down_exps": (self.E, self.hidden, self.I),
        }
        if self.activation in ("swiglu", "glu_clamp"):
            s["gate_exps"] = (self.E, self.I, self.hidden)
        if self.has_router_bias:
            s["router_bias"] = (self.R,)
        if self.shared_gate:
            s["shared_gate"] = (1, self.hidden)
        if self.has_sel_bias:
            s["sel_bias"] = (self.R,)
        return s

    def sources(self):
        p, n = self.prefix, self.names
        out = [TensorSource(f"{p}.{n['router']}", (self.R, self.hidden), "router")]
        for e in range(self.E):
            if self.activation in ("swiglu", "glu_clamp"):
                out.append(TensorSource(f"{p}.{n['expert_gate'].format(e=e)}", (self.I, self.hidden), "gate_exps", e * self.I))
            out.append(TensorSource(f"{p}.{n['expert_up'].format(e=e)}", (self.I, self.hidden), "up_exps", e * self.I))
            out.append(TensorSource(f"{p}.{n['expert_down'].format(e=e)}", (self.hidden, self.I), "down_exps",
                                    e * self.hidden))
        if self.has_router_bias:
            out.append(TensorSource(f"{p}.{n['router_bias']}", (self.R,), "router_bias", 0, "bias"))
        if self.shared_gate:
            out.append(TensorSource(f"{p}.{n['shared_gate']}", (1, self.hidden), "shared_gate"))
        if self.has_sel_bias:
            out.append(TensorSource(f"{p}.{n['selection_bias']}", (self.R,), "sel_bias", 0, "bias"))
        return out

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv", "moe_route", "elementwise"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def bind(self, rt) -> None:
        self._layout = rt.shared_object(
            ("expert_layout", self.R, self.k),
            lambda: K.ExpertLayout(rt.max_tokens * self.k, self.R, 64, rt.device),
        )
        self._scratch = rt.shared_object(
            ("router_scratch", self.R + 1),
            lambda: K.RouterScratch(rt.max_tokens, self.R + 1, rt.device),
        )
        self._router_all = None
        bias = self.params.get("sel_bias")
        self._rule = dict(top_k=self.k, renorm=self.norm_topk, scale=self.weight_scale, score_fn=self.score_fn,
                          sel_bias=bias.float().contiguous() if bias is not None else None, n_group=self.n_group,
                          n_group_used=self.n_group_used)
        if self.group_score != "top2":
            self._rule["group_score"] = self.group_score
        # the router's own bias as float32 over the logit rows (the gate's row, when there is one, gets none)
        self._logit_bias = None
        if self.has_router_bias:
            lb = torch.zeros(self.R + 1, dtype=torch.float32, device=rt.device)
            lb[: self.R] = self.params["router_bias"].float()
            self._logit_bias = lb
        r, g = self.params["router"], self.params.get("shared_gate")
        if (rt.dtype == torch.bfloat16 and r.dtype == torch.bfloat16 and self.hidden % 8 == 0
                and (g is None or g.dtype == torch.bfloat16)):
            # router rows and the gate row as one matrix (a copy of a few hundred KB)
            self._router_all = torch.cat([r, g.view(1, -1)], 0).contiguous() if g is not None else r

    def _first_product(self, x, act, scale=None, **kw) -> None:
        """``scale`` = (weights, the pairs' order): the picks' weights as a factor on the experts' input."""
        if self.activation == "swiglu":
            K.linear(x, self.params["gate_exps"], act, w2=self.params["up_exps"], **kw)
        elif self.activation == "glu_clamp":
            K.linear(x, self.params["gate_exps"], act, w2=self.params["up_exps"], act="glu_clamp", act_limit=self.limit,
                     row_scale=scale[0] if scale else None, scale_rows=scale[1] if scale else None, **kw)
        else:
            K.linear(x, self.params["up_exps"], act, act="relu2", **kw)

    def forward(self, h, batch, residual, rt, accumulate=True) -> None:
        T = h.shape[0]
        n_pairs = T * self.k
        if not accumulate and self.shared is None:
            residual.zero_()   # nothing else writes the rows before the experts' sum is added
        ids = rt.buf("moe.ids", (rt.max_tokens * self.k,), torch.int32)
        wts = rt.buf("moe.wts", (rt.max_tokens * self.k,), torch.float32)
        gamma = rt.buf("moe.gamma", (rt.max_tokens,), torch.float32) if self.shared_gate else None
        lay = self._layout
        # which kernels the expert products run on decides the row tile of the expert layout
        tile = K.FEW_ROWS if T <= K.FEW_ROWS else K.expert_tile(n_pairs, self.E)
        widths_ok = self.I % 8 == 0 and self.hidden % 8 == 0
        on_input = (wts, lay.sorted_pair) if self.weight_on_input else None
        all_bf16 = (K.tensor_cores_take(h, self.params["up_exps"]) and widths_ok
                    and self.params["down_exps"].dtype == torch.bfloat16)
        if not all_bf16 and widths_ok and n_pairs <= K.FEW_ROWS * self.E:
            # No tensor-core form (float32) and a handful of rows per expert: tiles of 8 rows on the row-streaming
            # kernel read an expert's weights once per tile, where the CUDA-core product would compute a 64-row
            # tile for every expert that has a row.
            tile = K.FEW_ROWS
        streamed = (all_bf16 and tile <= K.SKINNY_TILE_ROWS) or (widths_ok and tile <= K.FEW_ROWS)
        if not streamed and not all_bf16:
            tile = 64
        sorted_already = False
        # The shared expert needs only h for its first product: for a few tokens, where no kernel fills the GPU, it
        # starts on the side stream beside the router; its second product waits for the router's gate (below).
        # Long portions, too, while the routed experts wait for their weights rather than for the tensor cores
        # (fewer than about 190 rows per expert: flops / peak < bytes / bandwidth): the shared expert's products,
        # which are bound by the tensor cores, then run beside the router, the selection, the layout and the gather
        # and fill what the routed products leave idle.  (2,048 tokens of the 2.7B sizes in one step 12.6 -> 11.7 ms,
        # in two steps of 1,024 17.5 -> 15.2 ms; steps of 512 tokens lose, 27.6 -> 28.7 ms, and so do the 57B sizes'
        # steps of 4,096 and 8,192 tokens, whose experts are bound by the tensor cores: 1,254 -> 1,289 ms.)
        long_overlap = T >= SHARED_OVERLAP_FROM and n_pairs <= SHARED_OVERLAP_ROWS * self.E
        overlap = self.shared is not None and (T <= 64 or long_overlap)
        shared_act = None
        if overlap and (T <= SHARED_EARLY_TOKENS or long_overlap):
            with rt.side():
                shared_act = self.shared.forward_up(h, rt)
        if self._router_all is not None and K.USE_TENSOR_CORES:
            # bfloat16: router (and gate) logits on the tensor cores, one kernel for every batch shape
            logits = self._scratch.logits.view(rt.max_tokens, self.R + 1)
            if K.route_small_takes(T, self.k, self.R):
                # a decode-sized batch: logits, selection and the expert layout in one launch
                K.route_fused_small(h, self._router_all, logits, self.R, self.shared_gate, ids, wts, gamma, lay,
                                    self._scratch.fused_counter, n_tokens=T, tile_m=tile,
                                    logit_bias=self._logit_bias, **self._rule)
                sorted_already = True
            else:
                K.router_logits(h, self._router_all, logits, bias=self._logit_bias)
                K.router_select(logits, self.R, self.shared_gate, ids, wts, gamma, n_tokens=T, **self._rule)
        else:
            K.router_topk(h, self.params["router"], self.params.get("shared_gate"), ids, wts, gamma,
                          scratch=self._scratch, logit_bias=self._logit_bias, **self._rule)
        if self.observer is not None:
            self.observer(self.prefix, ids[:n_pairs].view(T, self.k), wts[:n_pairs].view(T, self.k))
        # The rest of the shared expert runs beside the routed experts on the side stream and is joined before the
        # combine (both add into the residual, so they must not overlap there).
        if overlap:
            with rt.side():
                if shared_act is not None:
                    self.shared.forward_down(shared_act, residual, rt, row_scale=gamma, accumulate=accumulate)
                else:
                    self.shared.forward(h, batch, residual, rt, row_scale=gamma, accumulate=accumulate)
        act = rt.rows(f"moe.act{self.I}", self.I, rt.dtype, n_pairs, per_token=self.k)
        if not sorted_already:
            # the second product of the tensor-core path may walk the layout in larger tiles
            tile2 = K.expert_second_tile(n_pairs, self.E) if (all_bf16 and not streamed) else 0
            K.moe_sort(ids, n_pairs, lay, tile, tile2)
        # the experts' weighted outputs, one row per (token, slot): in the model's element type (in bfloat16 a row is
        # rounded once more, like every activation between kernels; their sum, the residual stream, stays float32)
        pair_dt = torch.bfloat16 if (all_bf16 and rt.dtype == torch.bfloat16) else torch.float32
        pair_out = rt.rows("moe.pair_out", self.hidden, pair_dt, n_pairs, per_token=self.k)
        if self.n_identity:
            # the picks without weights: their rows are the input itself, and the products below never see them
            K.moe_identity(h, wts, lay, pair_out, n_pairs=n_pairs, top_k=self.k, n_real=self.E)
        if streamed or not all_bf16:
            # few rows per expert (or no tensor-core form): the kernels gather the token rows themselves
            self._first_product(h, act, scale=on_input, x_rows=lay.sorted_pair, x_row_div=self.k, layout=lay,
                                n_rows=n_pairs)
        else:
            # tcgen05 kernel: TMA reads whole row ranges, so lay the tokens out in expert order first
            xs = rt.rows("moe.x_sorted", self.hidden, rt.dtype, n_pairs, per_token=self.k)
            K.gather_rows(h, lay.sorted_pair, self.k, xs, n_pairs)
            self._first_product(xs, act, scale=on_input, layout=lay, n_rows=n_pairs)
        K.linear(act, self.params["down_exps"], pair_out, layout=lay, n_rows=n_pairs,
                 row_scale=None if self.weight_on_input else wts,
                 scale_rows=None if self.weight_on_input else lay.sorted_pair, lists_ready=True, second_tiles=True)
        if overlap:
            rt.join()
        if self.shared is not None and not overlap:
            self.shared.forward(h, batch, residual, rt, row_scale=gamma, accumulate=accumulate)
        if rt.defer_add and K.rmsnorm_adds(residual):
            # the sum of the experts' outputs is folded into the next block's first norm
            rt.leave_pending(PendingAdd(pair_out, lay.pair_pos, self.k))
        else:
            K.moe_combine(residual, pair_out, lay.pair_pos, self.k)


register_feed_forward("dense_mlp", DenseMlp)
register_feed_forward("sparse_moe", SparseMoe)
