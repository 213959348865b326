"""Norms.  RMSNorm(eps): out = x * rsqrt(mean(x^2) + eps) * w, statistics in float32; with ``offset`` the stored
weight is taken as w + offset (a weight stored around zero: offset 1).
LayerNorm(eps): out = (x - mean) / sqrt(var + eps) * w + b (below).

Formula and multiplication order of the reference's ``rmsnorm``
(src/locus/backend/cpu_ops.cpp:1687-1699): no mean subtraction, no bias, the weight used
as stored (not 1 + w).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from .base import Norm, TensorSource, register_norm


class RMSNorm(Norm):
    def __init__(self, prefix: str, *, width: int, eps: float, tensor: str = "", offset: float = 0.0) -> None:
        """``tensor``: the checkpoint tensor's name where it is not ``<prefix>.weight``.  ``offset``: added to the
        stored weight, in float32 (at bind, so that 1 + w is not rounded to the weight's 16 bits)."""
        super().__init__(prefix)
        self.width = int(width)
        self.eps = float(eps)
        self.offset = float(offset)
        self.tensor = str(tensor or prefix + ".weight")

    def bind(self, rt) -> None:
        if self.offset != 0.0 and not getattr(self, "_offset_done", False):
            self.params["weight"] = (self.params["weight"].float() + self.offset).contiguous()
            self._offset_done = True

    def param_shapes(self):
        return {"weight": (self.width,)}

    def sources(self):
        return [TensorSource(self.tensor, (self.width,), "weight", 0, "norm")]

    def kernel_modules(self, dtype):
        return ["elementwise"]

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None, add=None) -> None:
        if add is not None and not K.rmsnorm_adds(x):
            add.apply(x)
            add = None
        K.rmsnorm(x, self.params["weight"], self.eps, out, rows,
                  add=None if add is None else (add.pair_out, add.pair_pos, add.top_k))


    def forward_add(self, y: torch.Tensor, x: torch.Tensor) -> None:
        """x += norm(y): the norm of a sublayer's output (float32 rows) added to the residual stream."""
        K.rmsnorm_add(y, self.params["weight"], self.eps, x)


class LayerNorm(Norm):
    """Layer norm with weight and bias, mean and variance (the mean of the squared deviations) in float32.  With
    ``streams`` > 1 a row of x holds that many copies of the residual stream, one behind the other, and the norm
    reads their weighted sum (``coef`` [streams] float32 on the device; None: the plain sum)."""

    def __init__(self, prefix: str, *, width: int, eps: float, streams: int = 1, tensor: str = "",
                 bias_tensor: str = "") -> None:
        """``tensor`` / ``bias_tensor``: the checkpoint tensors' names where they are not ``<prefix>.weight`` and
        ``<prefix>.bias``."""
        super().__init__(prefix)
        self.width, self.eps, self.streams = int(width), float(eps), int(streams)
        self.tensor = str(tensor or prefix + ".weight")
        self.bias_tensor = str(bias_tensor or prefix + ".bias")

    def param_shapes(self):
        return {"weight": (self.width,), "bias": (self.width,)}

    def sources(self):
        return [TensorSource(self.tensor, (self.width,), "weight", 0, "norm"),
                TensorSource(self.bias_tensor, (self.width,), "bias", 0, "bias")]

    def kernel_modules(self, dtype):
        return ["elementwise"]

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None, add=None,
                coef: Optional[torch.Tensor] = None) -> None:
        if add is not None:
            add.apply(x)   # nothing is folded into this norm's pass
        K.layernorm(x, self.params["weight"], self.params["bias"], self.eps, out, rows, n_streams=self.streams, coef=coef)

    def forward_post(self, x: torch.Tensor, y: torch.Tensor, alpha: float, cast: Optional[torch.Tensor] = None) -> None:
        """x <- norm(alpha x + y) in place on the float32 residual stream (the norm behind a sublayer's sum); ``cast``:
        the new rows once more in that buffer's element type."""
        if self.streams != 1:
            raise ValueError("layernorm: the norm behind a sum works on one residual stream")
        K.layernorm_post(x, y, alpha, self.params["weight"], self.params["bias"], self.eps, cast)


register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
