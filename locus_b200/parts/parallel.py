"""Mixers side by side: every branch reads the same input, and their outputs are added with fixed factors.

``branches``: (name, mixer spec, factor) each; a branch's tensors live under ``<prefix>.<name>`` and the branch gets
its factor as its ``out_scale``.  The branches share the layer's cache: at most one of them may keep pages; the
per-request states of several branches lie one behind the other in the layer's one state slot, and each branch sees
its own stretch of it.

``branch_norm`` = {"width", "eps", "name"}: every branch's output is first divided by its root mean square over the
model width and multiplied by a weight of its own (``<prefix>.<branch>.<name>``, used as stored), and the factor
applies behind that: out = sum_b factor_b * w_b * y_b / sqrt(mean(y_b^2) + eps).  The branches then write float32 rows
of their own, and the norm adds them into the output.

A branch behind the first that can run in two steps (``prepare``: all but its last product, on buffers and state of its
own; ``finish``: the product that adds into the output) is prepared on the runtime's side stream while the first branch
runs, and finished when both are done.
"""
from __future__ import annotations

from typing import Sequence, Tuple

import dataclasses
from typing import Optional

import torch

from .. import kernels as K
from .base import Mixer, PartSpec, StateSpec, TensorSource, make_part, register_mixer


class ParallelMixers(Mixer):
    can_overwrite = True

    def __init__(self, prefix: str, *, branches: Sequence[Tuple[str, PartSpec, float]],
                 branch_norm: Optional[dict] = None) -> None:
        super().__init__(prefix)
        if not branches:
            raise ValueError("parallel: no branches")
        self.branch_norm = dict(branch_norm) if branch_norm else None
        self.branch_names = [name for name, _, _ in branches]
        self.factors = [float(scale) for _, _, scale in branches]
        self.branches = [make_part("mixer", PartSpec(spec.kind, {**spec.args, "out_scale": 1.0 if self.branch_norm else float(scale)}),
                                   f"{prefix}.{name}")
                         for name, spec, scale in branches]
        if self.branch_norm and not all(b.can_overwrite for b in self.branches):
            raise ValueError("parallel: branches whose outputs are normed must be able to write rows of their own")
        paged = [b for b in self.branches if b.cache_needs()[0] is not None]
        if len(paged) > 1:
            raise ValueError("parallel: at most one branch may keep pages")
        # where each branch's state lies in the layer's slot (several states: float32, one behind the other)
        self._state_at = {}
        states = [(i, b.cache_needs()[1]) for i, b in enumerate(self.branches) if b.cache_needs()[1] is not None]
        self._state_spec = None
        if len(states) == 1:
            self._state_spec = states[0][1]
        elif states:
            at = 0
            for i, sp in states:
                if sp.dtype != torch.float32:
                    raise ValueError("parallel: several branches with a state need float32 states")
                n = 1
                for e in sp.shape:
                    n *= int(e)
                self._state_at[i] = (at, n)
                at += n
            self._state_spec = StateSpec((at,), torch.float32)
        self._views = {}

    def sub_parts(self):
        return list(self.branches)

    def param_shapes(self):
        if not self.branch_norm:
            return {}
        return {f"norm_{n}": (int(self.branch_norm["width"]),) for n in self.branch_names}

    def sources(self):
        if not self.branch_norm:
            return []
        w = int(self.branch_norm["width"])
        return [TensorSource(f"{self.prefix}.{n}.{self.branch_norm['name']}", (w,), f"norm_{n}", 0, "norm") for n in self.branch_names]

    def kernel_modules(self, dtype):
        return ["elementwise"] if self.branch_norm else []

    def bind(self, rt) -> None:
        if self.branch_norm and not getattr(self, "_bound", False):
            # the factor rides on the norm's weight, in float32
            for n, f in zip(self.branch_names, self.factors):
                self.params[f"norm_{n}"] = (self.params[f"norm_{n}"].float() * f).contiguous()
            self._bound = True

    def cache_needs(self):
        paged = None
        for b in self.branches:
            paged = paged or b.cache_needs()[0]
        return paged, self._state_spec

    def _cache_of(self, i, cache):
        """The layer's cache as branch ``i`` sees it: with its own stretch of the state slot."""
        if i not in self._state_at or cache.state is None:
            return cache
        key = (i, cache.state.data_ptr(), cache.writes)
        view = self._views.get(key)
        if view is None:
            at, n = self._state_at[i]
            view = self._views[key] = dataclasses.replace(cache, state=cache.state[:, at:at + n])
        return view

    def step_plans(self):
        return [pl for b in self.branches for pl in b.step_plans()]

    def _forward_normed(self, h, batch, cache, residual, rt, accumulate) -> None:
        width, eps = int(self.branch_norm["width"]), float(self.branch_norm["eps"])
        T = batch.T
        ys = [rt.rows(f"parallel.y{i}", width, torch.float32, T) for i in range(len(self.branches))]
        early = {}
        for i, b in enumerate(self.branches[1:], 1):
            if hasattr(b, "prepare") and hasattr(b, "finish"):
                with rt.side():
                    early[i] = b.prepare(h, batch, self._cache_of(i, cache), rt)
                    b.finish(early[i], ys[i], rt, accumulate=False)
        if not accumulate:
            residual.zero_()
        for i, b in enumerate(self.branches):
            if i in early:
                if i == min(early):   # the side stream's work is done in order: one wait covers every branch on it
                    rt.join()
            else:
                b.forward(h, batch, self._cache_of(i, cache), ys[i], rt, accumulate=False)
            K.rmsnorm_add(ys[i], self.params[f"norm_{self.branch_names[i]}"], eps, residual)

    def forward(self, h, batch, cache, residual, rt, accumulate=True) -> None:
        if self.branch_norm:
            return self._forward_normed(h, batch, cache, residual, rt, accumulate)
        if self._state_at:
            caches = [self._cache_of(i, cache) for i in range(len(self.branches))]
        else:
            caches = [cache] * len(self.branches)
        early = {}
        for i, b in enumerate(self.branches[1:], 1):
            if hasattr(b, "prepare") and hasattr(b, "finish"):
                with rt.side():
                    early[i] = b.prepare(h, batch, caches[i], rt)
        for i, b in enumerate(self.branches):
            cache = caches[i]
            if i in early:
                if i == min(early):   # the side stream's work is done in order: one wait covers every branch on it
                    rt.join()
                b.finish(early[i], residual, rt, accumulate=True)
            elif i == 0 and not accumulate and not b.can_overwrite:
                residual.zero_()
                b.forward(h, batch, cache, residual, rt)
            elif b.can_overwrite:
                b.forward(h, batch, cache, residual, rt, accumulate=accumulate or i > 0)
            else:
                b.forward(h, batch, cache, residual, rt)


register_mixer("parallel", ParallelMixers)
