"""Typed configuration of the Gugozen design.

config.json of this design is nested: the model's ``width``, ``vocab``, ``norm.eps``, ``postln_alpha`` (the factor on the
residual stream in front of every norm), ``embedding.bigram`` = {``buckets``, ``mul_prev``, ``mul_cur``} (a second
embedding table addressed by a hash of the previous and the current token; absent: none) and a list ``layers`` whose
entries each give the ``type`` of their mixer, the mixer's sizes and constants (``mixer``) and their feed-forward
(``mlp``, or null for none).  Layers may differ from each other in everything.  Every size and constant is read here;
nothing about a particular model is fixed in code.

Mixer ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot`` = {``base``, ``dims``} (absent: no
rotation).
Mixer ``latent_attention``: ``heads``, ``dim`` (unrotated), ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``rot``,
``kv_from`` (the layer whose cached latent and rotated key part this one reads; absent: its own).
Mixer ``gla``: ``heads``, ``dim``, ``vdim``, ``tau``.
Feed-forward ``moe``: ``router`` = {``experts``, ``top``}, ``expert`` = {``ff``, ``limit``}, ``shared`` = {``ff``,
``limit``} (absent: no shared expert).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, take
from .lalepel import _num, _pos, _sub
from .mekizen import Rotation, _rot


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotation]

    kind = "attention"


@dataclass(frozen=True)
class GatedLatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: Optional[Rotation]
    kv_from: Optional[int]

    kind = "latent_attention"


@dataclass(frozen=True)
class GlaConfig:
    heads: int
    dim: int
    vdim: int
    tau: float

    kind = "gla"


@dataclass(frozen=True)
class ClampedExpertConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoeConfig:
    experts: int
    top: int
    expert: ClampedExpertConfig
    shared: Optional[ClampedExpertConfig]

    kind = "moe"


@dataclass(frozen=True)
class BigramConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class GugozenLayer:
    mixer: Any                       # SinkAttentionConfig | GatedLatentConfig | GlaConfig
    mlp: Optional[MoeConfig]


def _attention(m: Dict[str, Any], where: str) -> SinkAttentionConfig:
    heads, kv = _pos(m, "heads", where), _pos(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}heads {heads} must be a multiple of kv_heads {kv}")
    dim = _pos(m, "dim", where)
    return SinkAttentionConfig(heads=heads, kv_heads=kv, dim=dim, vdim=_pos(m, "vdim", where), scale=_num(m, "scale", where),
                               rot=_rot(m, where, dim))


def _latent(m: Dict[str, Any], where: str, index: int) -> GatedLatentConfig:
    rot_dim = _pos(m, "rot_dim", where)
    rot = _rot(m, where, rot_dim)
    src = take(m, "kv_from", int, None)
    if src is not None and not (0 <= src < index):
        raise ConfigError(f"config.json: {where}kv_from {src} must name an earlier layer")
    return GatedLatentConfig(heads=_pos(m, "heads", where), dim=_pos(m, "dim", where), rot_dim=rot_dim,
                             vdim=_pos(m, "vdim", where), kv_rank=_pos(m, "kv_rank", where), scale=_num(m, "scale", where),
                             rot=rot, kv_from=src)


def _gla(m: Dict[str, Any], where: str) -> GlaConfig:
    tau = _num(m, "tau", where)
    if not tau > 0:
        raise ConfigError(f"config.json: {where}tau must be positive, got {tau}")
    return GlaConfig(heads=_pos(m, "heads", where), dim=_pos(m, "dim", where), vdim=_pos(m, "vdim", where), tau=tau)


def _expert(raw: Dict[str, Any], where: str) -> ClampedExpertConfig:
    limit = _num(raw, "limit", where)
    if not limit > 0:
        raise ConfigError(f"config.json: {where}limit must be positive, got {limit}")
    return ClampedExpertConfig(ff=_pos(raw, "ff", where), limit=limit)


def _mlp(raw: Optional[Dict[str, Any]], where: str) -> Optional[MoeConfig]:
    if raw is None:
        return None
    if raw.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}kind must be 'moe', got {raw.get('kind')!r}")
    router = _sub(raw, "router", where)
    experts, top = _pos(router, "experts", where + "router."), _pos(router, "top", where + "router.")
    if top > experts:
        raise ConfigError(f"config.json: {where}router.top {top} exceeds router.experts {experts}")
    shared = _sub(raw, "shared", where, optional=True)
    return MoeConfig(experts=experts, top=top, expert=_expert(_sub(raw, "expert", where), where + "expert."),
                     shared=_expert(shared, where + "shared.") if shared is not None else None)


@dataclass(frozen=True)
class GugozenConfig:
    vocab: int
    width: int
    eps: float
    alpha: float
    bigram: Optional[BigramConfig]
    layers: Tuple[GugozenLayer, ...]

    architecture = "Gugozen"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "GugozenConfig":
        norm = _sub(raw, "norm", "")
        emb = _sub(raw, "embedding", "", optional=True)
        bg = _sub(emb, "bigram", "embedding.", optional=True) if emb is not None else None
        bigram = None
        if bg is not None:
            w = "embedding.bigram."
            bigram = BigramConfig(buckets=_pos(bg, "buckets", w), mul_prev=take(bg, "mul_prev", int),
                                  mul_cur=take(bg, "mul_cur", int))
            if bigram.mul_prev < 0 or bigram.mul_cur < 0:
                raise ConfigError("config.json: embedding.bigram.mul_prev and mul_cur must not be negative")
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
                mx = _attention(mixer, where + "mixer.")
            elif kind == "latent_attention":
                mx = _latent(mixer, where + "mixer.", i)
                if mx.kv_from is not None:
                    src = layers[mx.kv_from].mixer
                    if not isinstance(src, GatedLatentConfig) or src.kv_from is not None:
                        raise ConfigError(f"config.json: {where}mixer.kv_from {mx.kv_from} must name a latent_attention "
                                          "layer with a latent of its own")
                    if (src.kv_rank, src.rot_dim, src.rot) != (mx.kv_rank, mx.rot_dim, mx.rot):
                        raise ConfigError(f"config.json: {where}mixer: kv_rank, rot_dim and rot must equal those of layer "
                                          f"{mx.kv_from}, whose latent it reads")
            elif kind == "gla":
                mx = _gla(mixer, where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type must be 'attention', 'latent_attention' or 'gla', got {kind!r}")
            mlp = lr.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            layers.append(GugozenLayer(mixer=mx, mlp=_mlp(mlp, where + "mlp.")))
        return cls(vocab=_pos(raw, "vocab", ""), width=_pos(raw, "width", ""), eps=_num(norm, "eps", "norm."),
                   alpha=_num(raw, "postln_alpha", ""), bigram=bigram, layers=tuple(layers))
