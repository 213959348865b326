"""Typed configuration of the Mekizen design.

config.json of this design is nested: the model's ``width``, ``vocab``, ``norm.eps``, ``embedding.scale`` (a factor on
the embedding; absent: 1) and a list ``layers`` whose entries each give the ``type`` of their mixer, the mixer's sizes
and constants (``mixer``) and their feed-forward (``mlp``, or null for none).  Layers may differ from each other in
everything.  Every size and constant is read here; nothing about a particular model is fixed in code.

Mixer ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot`` = {``base``, ``dims``} (absent: no
rotation), ``mask`` = {``size``, ``keep_first``} (absent: every earlier token; ``keep_first`` absent: 0), ``kv_from``
(the layer whose keys and values this one uses; absent: its own).
Mixer ``parallel``: ``left`` = {``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``conv`` (taps), ``rot``}, ``right`` =
{``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``}.
Feed-forward ``dense``: ``ff``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, take
from .lalepel import _num, _pos, _sub


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int


@dataclass(frozen=True)
class GatedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotation]
    window: int                      # 0: every earlier token
    keep_first: int
    kv_from: Optional[int]

    kind = "attention"


@dataclass(frozen=True)
class ConvAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int
    rot: Optional[Rotation]


@dataclass(frozen=True)
class DeltaRuleConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class ParallelConfig:
    left: ConvAttentionConfig
    right: DeltaRuleConfig

    kind = "parallel"


@dataclass(frozen=True)
class DenseFfConfig:
    ff: int

    kind = "dense"


@dataclass(frozen=True)
class MekizenLayer:
    mixer: Any                       # GatedAttentionConfig | ParallelConfig
    mlp: Optional[DenseFfConfig]


def _rot(m: Dict[str, Any], where: str, dim: int) -> Optional[Rotation]:
    r = _sub(m, "rot", where, optional=True)
    if r is None:
        return None
    rot = Rotation(base=_num(r, "base", where + "rot."), dims=_pos(r, "dims", where + "rot."))
    if rot.dims % 2 or rot.dims > dim:
        raise ConfigError(f"config.json: {where}rot.dims {rot.dims} must be even and at most dim {dim}")
    if not rot.base > 0:
        raise ConfigError(f"config.json: {where}rot.base must be positive, got {rot.base}")
    return rot


def _heads(m: Dict[str, Any], where: str):
    heads, kv = _pos(m, "heads", where), _pos(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}heads {heads} must be a multiple of kv_heads {kv}")
    return heads, kv, _pos(m, "dim", where), _pos(m, "vdim", where)


def _attention(m: Dict[str, Any], where: str, index: int) -> GatedAttentionConfig:
    heads, kv, dim, vdim = _heads(m, where)
    mask = _sub(m, "mask", where, optional=True)
    window = _pos(mask, "size", where + "mask.") if mask is not None else 0
    keep = take(mask, "keep_first", int, 0) if mask is not None else 0
    if keep < 0:
        raise ConfigError(f"config.json: {where}mask.keep_first must not be negative")
    src = take(m, "kv_from", int, None)
    if src is not None and not (0 <= src < index):
        raise ConfigError(f"config.json: {where}kv_from {src} must name an earlier layer")
    return GatedAttentionConfig(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=_num(m, "scale", where),
                                rot=_rot(m, where, dim), window=window, keep_first=keep, kv_from=src)


def _parallel(m: Dict[str, Any], where: str) -> ParallelConfig:
    lw, rw = where + "left.", where + "right."
    l, r = _sub(m, "left", where), _sub(m, "right", where)
    heads, kv, dim, vdim = _heads(l, lw)
    left = ConvAttentionConfig(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=_num(l, "scale", lw),
                               conv=_pos(l, "conv", lw), rot=_rot(l, lw, dim))
    heads, kv, dim, vdim = _heads(r, rw)
    right = DeltaRuleConfig(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=_pos(r, "conv", rw))
    return ParallelConfig(left=left, right=right)


def _mlp(raw: Optional[Dict[str, Any]], where: str) -> Optional[DenseFfConfig]:
    if raw is None:
        return None
    if raw.get("kind") != "dense":
        raise ConfigError(f"config.json: {where}kind must be 'dense', got {raw.get('kind')!r}")
    return DenseFfConfig(ff=_pos(raw, "ff", where))


@dataclass(frozen=True)
class MekizenConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[MekizenLayer, ...]

    architecture = "Mekizen"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "MekizenConfig":
        norm = _sub(raw, "norm", "")
        emb = _sub(raw, "embedding", "", optional=True)
        layers_raw = take(raw, "layers", list)
        if not layers_raw:
            raise ConfigError("config.json: layers must not be empty")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]."
            if not isinstance(lr, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = lr.get("type")
            mixer = _sub(lr, "mixer", where)
            if kind == "attention":
                mx = _attention(mixer, where + "mixer.", i)
                if mx.kv_from is not None:
                    src = layers[mx.kv_from].mixer
                    if not isinstance(src, GatedAttentionConfig) or src.kv_from is not None:
                        raise ConfigError(f"config.json: {where}mixer.kv_from {mx.kv_from} must name an attention layer "
                                          "with keys and values of its own")
                    if (src.kv_heads, src.dim, src.vdim, src.rot) != (mx.kv_heads, mx.dim, mx.vdim, mx.rot):
                        raise ConfigError(f"config.json: {where}mixer: kv_heads, dim, vdim and rot must equal those of "
                                          f"layer {mx.kv_from}, whose keys and values it uses")
            elif kind == "parallel":
                mx = _parallel(mixer, where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type must be 'attention' or 'parallel', got {kind!r}")
            mlp = lr.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            layers.append(MekizenLayer(mixer=mx, mlp=_mlp(mlp, where + "mlp.")))
        return cls(vocab=_pos(raw, "vocab", ""), width=_pos(raw, "width", ""), eps=_num(norm, "eps", "norm."),
                   embedding_scale=take(emb, "scale", float, 1.0) if emb is not None else 1.0, layers=tuple(layers))
