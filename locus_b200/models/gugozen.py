"""The Gugozen design as a plan of parts.

A post-norm decoder: x <- LN1(alpha x + mixer(x)); x <- LN2(alpha x + ff(x)), the sublayers reading x itself and the layer
norms (weight and bias) sitting behind the sums.  The embedding adds a row of a second table addressed by a hash of the
previous and the current token.  Each layer names its mixer: ``attention`` (grouped-query attention with an RMS norm over
the whole q and the whole k projection, a rotation of part of each head and a learned sink per head in the softmax),
``latent_attention`` (keys and values from one cached latent and one shared rotated key part, a sigmoid gate on the heads'
outputs; it may read an earlier layer's cached rows instead of projecting its own) or ``gla`` (gated linear attention with
a decay per key channel).  The feed-forward is a mixture of clamped gated experts with sigmoid scores whose weights
multiply the experts' inputs, plus a shared expert.  The head is the embedding table.  Tensor names: ``embed``,
``bigram``, ``l<i>.norm1|norm2`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.router|e<j>.gate|up|down|shared.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.base import ArchEntry, register_arch
from ..config.gugozen import GatedLatentConfig, GlaConfig, GugozenConfig, SinkAttentionConfig
from ..parts.base import LayerCall, LayerSpec, ModelPlan, PartSpec

# positions enter the rotation's angle as float32: exact up to 2^24
MAX_POSITIONS = 1 << 24

_ATTN_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}
_MOE_NAMES = {"router": "router", "expert_gate": "e{e}.gate", "expert_up": "e{e}.up", "expert_down": "e{e}.down",
              "shared": "shared"}
_DENSE_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def _position(rot, dim: int) -> PartSpec:
    if rot is None:
        return PartSpec("none")
    return PartSpec("rotary", {"head_dim": dim, "theta": rot.base, "rot_dim": rot.dims})


def _mixer(cfg: GugozenConfig, index: int, decay_rank) -> PartSpec:
    m = cfg.layers[index].mixer
    if isinstance(m, SinkAttentionConfig):
        return PartSpec("attention", {
            "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
            "qkv_bias": False, "sink": "learned", "qk_norm": "whole", "qk_norm_eps": cfg.eps, "softmax_scale": m.scale,
            "position": _position(m.rot, m.dim), "shaped": True, "names": _ATTN_NAMES})
    if isinstance(m, GatedLatentConfig):
        return PartSpec("latent_attention", {
            "hidden": cfg.width, "n_heads": m.heads, "nope_dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim, "q_rank": 0,
            "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.eps, "position": _position(m.rot, m.rot_dim),
            "out_gate": True, "has_kv": m.kv_from is None})
    if isinstance(m, GlaConfig):
        return PartSpec("gla", {"hidden": cfg.width, "n_heads": m.heads, "dim": m.dim, "v_dim": m.vdim,
                                "decay_rank": decay_rank(index), "tau": m.tau, "eps": cfg.eps})
    raise TypeError(m)


def _feed_forward(cfg: GugozenConfig, f) -> PartSpec:
    if f is None:
        return PartSpec("none")
    return PartSpec("sparse_moe", {
        "hidden": cfg.width, "n_experts": f.experts, "top_k": f.top, "norm_topk": False, "expert_intermediate": f.expert.ff,
        "shared_intermediate": f.shared.ff if f.shared is not None else 0, "shared_gate": False, "score_fn": "sigmoid",
        "activation": "glu_clamp", "limit": f.expert.limit, "shared_limit": f.shared.limit if f.shared is not None else None,
        "weight_on_input": True, "names": _MOE_NAMES, "shared_names": _DENSE_NAMES})


def build_plan(cfg: GugozenConfig, tensor_shapes=None) -> ModelPlan:
    """``tensor_shapes``: name -> shape of the model's stored tensors, where a size is given by a tensor's shape alone
    (the width of a gla layer's first decay projection, ``l<i>.mix.a1``); without it that width is ``DECAY_RANK``."""

    def decay_rank(i: int) -> int:
        shape = (tensor_shapes or {}).get(f"l{i}.mix.a1")
        return int(shape[0]) if shape else DECAY_RANK

    norm = PartSpec("layernorm", {"width": cfg.width, "eps": cfg.eps})
    arrangement = PartSpec("post_norm", {"hidden": cfg.width, "alpha": cfg.alpha})
    layers = [LayerSpec(prefix=f"l{i}", arrangement=arrangement, norm=norm, mixer=_mixer(cfg, i, decay_rank),
                        feed_forward=_feed_forward(cfg, layer.mlp))
              for i, layer in enumerate(cfg.layers)]
    # every layer runs once, in order, so a layer's index is also its place in the run order
    order = [LayerCall(i, cache_of=getattr(layer.mixer, "kv_from", None)) for i, layer in enumerate(cfg.layers)]
    pair = None
    if cfg.bigram is not None:
        pair = {"tensor": "bigram", "buckets": cfg.bigram.buckets, "mul_prev": cfg.bigram.mul_prev,
                "mul_cur": cfg.bigram.mul_cur}
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        eos_token_id=-1,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "embed", "tensor": "embed",
                                         "pair": pair}),
        layers=layers, order=order,
        final_norm=PartSpec("layernorm", {"width": cfg.width, "eps": cfg.eps, "prefix": "final.norm", "tensor": "final.norm",
                                          "bias_tensor": "final.norm.b"}),
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "head", "tied_to": "embed"}),
        config=cfg,
    )


# the width of a gla layer's first decay projection where no stored tensor says it (random-weights mode)
DECAY_RANK = 32

register_arch(ArchEntry(
    name="Gugozen",
    description="Gugozen: post-norm decoder with layer norms and a hashed bigram embedding; grouped-query attention with "
                "whole-projection q/k norms and a learned softmax sink; gated latent attention that may share another "
                "layer's cached latent; gated linear attention with a decay per key channel; clamped gated experts with "
                "sigmoid scores on their inputs and a shared expert; tied head",
    parse_config=GugozenConfig.from_dict,
    build_plan=build_plan,
    sizes_from_tensors=True,
))
