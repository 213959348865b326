"""The Mekizen design as a plan of parts.

A pre-norm decoder whose RMS norms store their weight around zero (the factor is 1 + w), with a scaled embedding and
squared-ReLU feed-forwards.  Each layer names its mixer: ``attention`` (grouped-query attention with biases, a rotation
of part of each head, a sliding window that keeps a request's first tokens in sight, a softmax with a sink, a sigmoid
gate on the heads' outputs; it may read the keys and values of an earlier layer instead of projecting its own) or
``parallel`` (causal attention whose q, k, v pass a short convolution and whose q and k are normed per head behind the
rotation, beside a gated delta rule; each side's output is RMS-normed over the width, and the mixer gives half their
sum).  Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*`` (``.left.*`` / ``.right.*`` in a parallel mixer),
``l<i>.mlp.up|down``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import ArchEntry, register_arch
from ..config.mekizen import GatedAttentionConfig, MekizenConfig, ParallelConfig
from ..parts.base import LayerCall, LayerSpec, ModelPlan, PartSpec

# positions enter the rotation's angle as float32: exact up to 2^24
MAX_POSITIONS = 1 << 24

_ATTN_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
               "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "gate": "g"}


def _position(rot, dim: int) -> PartSpec:
    if rot is None:
        return PartSpec("none")
    return PartSpec("rotary", {"head_dim": dim, "theta": rot.base, "rot_dim": rot.dims})


def _mixer(cfg: MekizenConfig, index: int) -> PartSpec:
    m = cfg.layers[index].mixer
    if isinstance(m, GatedAttentionConfig):
        # the pages of a layer whose keys and values later layers use hold what the widest of their masks sees
        readers = [m] + [l.mixer for l in cfg.layers if isinstance(l.mixer, GatedAttentionConfig) and l.mixer.kv_from == index]
        window = 0 if any(r.window == 0 for r in readers) else max(r.window for r in readers)
        keep = max(r.keep_first for r in readers) if window else 0
        return PartSpec("attention", {
            "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
            "qkv_bias": True, "o_bias": True, "window": m.window, "keep_first": m.keep_first, "sink": True,
            "out_gate": True, "has_kv": m.kv_from is None, "softmax_scale": m.scale, "position": _position(m.rot, m.dim),
            "shaped": True, "cache_window": window, "cache_keep": keep, "names": _ATTN_NAMES})
    if isinstance(m, ParallelConfig):
        l, r = m.left, m.right
        left = PartSpec("attention", {
            "hidden": cfg.width, "n_heads": l.heads, "n_kv_heads": l.kv_heads, "head_dim": l.dim, "v_dim": l.vdim,
            "qkv_bias": False, "conv_taps": l.conv, "qk_norm": "rms", "qk_norm_eps": cfg.eps, "softmax_scale": l.scale,
            "position": _position(l.rot, l.dim), "shaped": True, "names": _ATTN_NAMES})
        right = PartSpec("gated_delta", {"hidden": cfg.width, "n_heads": r.heads, "n_qk_heads": r.kv_heads, "dim": r.dim,
                                         "v_dim": r.vdim, "taps": r.conv, "eps": cfg.eps})
        return PartSpec("parallel", {"branches": (("left", left, 0.5), ("right", right, 0.5)),
                                     "branch_norm": {"width": cfg.width, "eps": cfg.eps, "name": "out"}})
    raise TypeError(m)


def _feed_forward(cfg: MekizenConfig, f) -> PartSpec:
    if f is None:
        return PartSpec("none")
    return PartSpec("dense_mlp", {"hidden": cfg.width, "intermediate": f.ff, "activation": "relu2",
                                  "names": {"up": "up", "down": "down"}})


def build_plan(cfg: MekizenConfig) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.eps, "offset": 1.0})
    arrangement = PartSpec("pre_norm", {"hidden": cfg.width, "mixer_prefix": "mix", "ff_prefix": "mlp",
                                        "norm1_name": "norm1", "norm2_name": "norm2", "plain_norm_names": True})
    layers = [LayerSpec(prefix=f"l{i}", arrangement=arrangement, norm=norm, mixer=_mixer(cfg, i),
                        feed_forward=_feed_forward(cfg, layer.mlp))
              for i, layer in enumerate(cfg.layers)]
    # every layer runs once, in order, so a layer's index is also its place in the run order
    order = [LayerCall(i, cache_of=getattr(layer.mixer, "kv_from", None)) for i, layer in enumerate(cfg.layers)]
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        eos_token_id=-1,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "embed", "tensor": "embed",
                                         "scale": cfg.embedding_scale}),
        layers=layers, order=order,
        final_norm=PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.eps, "offset": 1.0, "prefix": "final.norm",
                                        "tensor": "final.norm"}),
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "head", "tensor": "head"}),
        config=cfg,
    )


register_arch(ArchEntry(
    name="Mekizen",
    description="Mekizen: pre-norm decoder with one-plus RMS norms; gated grouped-query attention with a sliding window "
                "that keeps the first tokens, a softmax sink and shared keys and values between layers; convolved, "
                "normed attention beside a gated delta rule, each RMS-normed and averaged; squared-ReLU feed-forwards",
    parse_config=MekizenConfig.from_dict,
    build_plan=build_plan,
))
