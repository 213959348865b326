"""Tiny Gugozen configurations, random model folders with weights shaped so that faults show, and the helpers that the
host tests (plain twins of the kernels, CPU) and the gpu tests share to run schedules against the plain implementation
of ``plain_gugozen``.

Random weights of standard deviation 0.02 hide faults: attention is nearly uniform, a sink outweighs or never matters,
every decay is the same and the experts' clamps are never reached.  ``sharpen`` spreads the scores, gives the sinks
values that compete with the keys, decays from slow to fast, router scores from near 0 to near 1 and expert inputs that
reach the clamps."""
import copy
import json
import os

import torch

import plain_gugozen as plain
from lalepel_cases import cuts, make_runner, run_steps, schedules, tokens  # noqa: F401  (shared schedule helpers)


def attention(heads, kv_heads, dim, vdim, rot=None, scale=None, base=10000.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    return {"type": "attention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, kv_rank, kv_from=None, scale=None, base=10000.0, rot=True):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if rot:
        m["rot"] = {"base": base, "dims": rot_dim}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def gla(heads, dim, vdim, tau=16.0):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def with_mlp(layer, experts=0, top=1, ff=16, limit=1.5, shared=None):
    """``shared`` = (ff, limit) or None; ``experts`` 0: no feed-forward."""
    layer = copy.deepcopy(layer)
    layer["mlp"] = None
    if experts:
        layer["mlp"] = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
        if shared:
            layer["mlp"]["shared"] = {"ff": shared[0], "limit": shared[1]}
    return layer


def model(width, vocab, layers, eps=1e-5, alpha=2.0, bigram=(53, 31, 5)):
    cfg = {"architecture": "Gugozen", "width": width, "vocab": vocab, "norm": {"eps": eps}, "postln_alpha": alpha,
           "layers": layers}
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return cfg


CONFIGS = {
    # every mechanism: the three mixers, a latent layer on an earlier one's cached rows, experts with and without a
    # shared one, top 2 of 6, a layer without a feed-forward
    "mix": model(64, 97, [
        with_mlp(attention(4, 2, 32, 16, rot=16, base=500.0, scale=0.21), 6, 2, 24, 1.25, shared=(40, 2.0)),
        with_mlp(gla(2, 24, 16, tau=8.0), 4, 1, 16, 1.5),
        with_mlp(latent(4, 16, 8, 16, 32, scale=0.17), 5, 3, 8, 0.75, shared=(16, 1.0)),
        with_mlp(gla(3, 8, 24, tau=1.0), 0),
        with_mlp(latent(2, 16, 8, 32, 32, kv_from=2, scale=0.3), 6, 2, 24, 1.25),
    ], alpha=2.5),
    # nothing a multiple of 16, 8 or 4; one head; equal head counts; top = experts; one expert; no rotation in one
    # layer; a rotation of the whole head in another; no bigram table; alpha 1
    "odd": model(50, 61, [
        with_mlp(attention(3, 3, 10, 6, rot=6), 1, 1, 9, 0.5),
        with_mlp(gla(1, 7, 5, tau=3.0), 3, 3, 5, 2.0, shared=(7, 0.5)),
        with_mlp(latent(1, 6, 4, 10, 9, rot=False), 0),
        with_mlp(attention(2, 1, 6, 14, rot=0), 4, 2, 6, 1.0),
        with_mlp(latent(3, 5, 6, 3, 7, base=77.0), 2, 1, 11, 3.0),
        with_mlp(attention(2, 2, 12, 4, rot=12, base=77.0), 0),
    ], eps=1e-6, alpha=1.0, bigram=None),
    # one mechanism each
    "attention_only": model(48, 50, [with_mlp(attention(4, 2, 16, 16, rot=8), 0)], bigram=None),
    "gla_only": model(48, 50, [with_mlp(gla(4, 16, 12, tau=4.0), 0)], bigram=None),
    "latent_only": model(48, 50, [with_mlp(latent(2, 16, 8, 16, 24), 0), with_mlp(latent(4, 8, 8, 8, 24, kv_from=0), 0)],
                         bigram=None),
    "moe_only": model(48, 50, [with_mlp(gla(1, 8, 8, tau=2.0), 8, 2, 16, 1.0, shared=(24, 1.5))], bigram=(17, 3, 7)),
    # larger heads: heads of 128 with values of 96 (the kernels' head size above the values'), rows of the recurrence
    # beyond a lane's first registers, a latent of 64 + 16 on the tensor-core kernel's sizes
    "wide": model(128, 211, [
        with_mlp(attention(4, 2, 128, 96, rot=48, base=5e5, scale=0.09), 8, 2, 32, 1.75, shared=(64, 2.5)),
        with_mlp(gla(2, 72, 40, tau=12.0), 8, 1, 32, 1.75),
        with_mlp(latent(4, 32, 16, 32, 64, scale=0.14), 4, 1, 48, 1.25, shared=(32, 2.5)),
        with_mlp(latent(2, 32, 16, 48, 64, kv_from=2, scale=0.14), 0),
    ], alpha=3.0, bigram=(257, 113, 9)),
}
SEEDS = {n: 171 + i for i, n in enumerate(CONFIGS)}
# other widths of a gla layer's first decay projection than the random-weights mode draws (configuration -> layer -> rows)
DECAY_RANKS = {"mix": {1: 5, 3: 12}, "odd": {1: 3}, "gla_only": {0: 8}}


def sharpen(name, w, strength=1.0):
    """Weights (name -> float32 tensor) changed in place so that far keys, sinks, states, clamps and the router matter.
    ``strength`` < 1 moves the factors on the projections towards 1 (deep bfloat16 models, whose rounding sharp scores
    amplify)."""
    g = torch.Generator().manual_seed(9)
    f = lambda m: 1.0 + (m - 1.0) * strength
    for layer, rank in DECAY_RANKS.get(name, {}).items():
        a1, a2 = w[f"l{layer}.mix.a1"], w[f"l{layer}.mix.a2"]
        w[f"l{layer}.mix.a1"] = torch.randn(rank, a1.shape[1], generator=g) * 0.02
        w[f"l{layer}.mix.a2"] = torch.randn(a2.shape[0], rank, generator=g) * 0.02
    for n in list(w):
        t = w[n]
        if n.endswith((".norm1", ".norm2", ".dkv.norm", ".q.norm", ".k.norm", ".mix.norm")) or n == "final.norm":
            w[n] = 0.6 + 0.8 * torch.rand(t.shape, generator=g)
        elif n.endswith((".norm1.b", ".norm2.b")) or n == "final.norm.b":
            w[n] = (torch.rand(t.shape, generator=g) - 0.5) * 0.4
        elif n.endswith((".mix.q", ".mix.k", ".mix.dkv", ".mix.uk")):
            # scores spread over several units, whatever the width (scores of tens turn every rounding of a layer's
            # input into ten times as much behind its softmax)
            w[n] = t * f(12.0 * min(1.0, (64.0 / t.shape[1]) ** 0.5))
        elif n.endswith((".mix.v", ".mix.uv", ".mix.o")):
            w[n] = t * f(5.0)
        elif n.endswith(".mix.g"):
            w[n] = t * f(8.0)
        elif n.endswith(".mix.sink"):
            w[n] = torch.linspace(-1.0, 2.0, t.numel())                      # sinks that compete with the keys
        elif n.endswith(".mix.a1"):
            w[n] = t * 20.0
        elif n.endswith(".mix.a2"):
            w[n] = t * 20.0
        elif n.endswith(".mix.a2.b"):
            w[n] = torch.linspace(-3.0, 6.0, t.numel())                      # channels from fast to slow
        elif n.endswith(".router"):
            w[n] = t * f(25.0)                                               # scores from near 0 to near 1
        elif n.endswith((".gate", ".up")):
            w[n] = t * f(15.0)                                               # the clamps are reached
        elif n.endswith(".down"):
            w[n] = t * 4.0
        elif n in ("embed", "bigram"):
            w[n] = t * 30.0


def make_dir(tmp_path, name, store_dtype=torch.bfloat16, raw=None, tweak=sharpen, seed=None):
    """A model folder of configuration ``name`` (or ``raw``): seeded random weights, then ``tweak``, stored in
    ``store_dtype``.  Returns (folder, config dict, weights as stored, float32)."""
    from locus_b200.weights.loader import write_random_model
    from locus_b200.weights.safetensors_io import ModelFiles, write_safetensors
    import locus_b200.models  # noqa: F401

    cfg = copy.deepcopy(raw if raw is not None else CONFIGS[name])
    d = os.path.join(str(tmp_path), f"gugozen_{name}_{str(store_dtype).split('.')[-1]}")
    write_random_model(cfg, SEEDS.get(name, 5) if seed is None else seed, d, torch.float32)
    mf = ModelFiles(d)
    w = {n: mf.tensor(n).clone().float() for n in mf.names()}
    mf.close()
    if tweak is not None:
        tweak(name, w)
    w = {n: t.to(store_dtype) for n, t in w.items()}
    write_safetensors(os.path.join(d, "model.safetensors"), [(n, tuple(t.shape), store_dtype) for n, t in w.items()],
                      lambda n: w[n], metadata={"format": "pt"})
    with open(os.path.join(d, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    return d, cfg, {n: t.float() for n, t in w.items()}


class Case:
    def __init__(self, name, tmp_path, store_dtype=torch.bfloat16, raw=None, requests=(), tweak=sharpen, seed=None):
        self.name = name
        self.dir, self.cfg, self.weights = make_dir(tmp_path, name, store_dtype, raw=raw, tweak=tweak, seed=seed)
        self.tokens = {f"r{i}": tokens(n, self.cfg["vocab"], 1000 * (i + 1) + n) for i, n in enumerate(requests)}
        self._ref = {}

    def ref(self, rid, picks=None):
        """(plain logits [T, vocab] float64, router logits by feed-forward prefix)."""
        if picks is None and rid in self._ref:
            return self._ref[rid]
        aux = {}
        lg, _ = plain.forward(self.cfg, self.weights, self.tokens[rid], picks=picks, aux=aux)
        if picks is None:
            self._ref[rid] = (lg, aux)
        return lg, aux

    def ref_following(self, rid, routed, near_tie):
        """The plain logits when the plain implementation takes the engine's picks (``routed``: prefix -> {position:
        picks}) where they differ from its own, layer by layer, so that every layer's scores are those of the activations
        that the picks before it gave.  A difference is allowed only at a near-tie: every expert the engine picked must
        have a score within ``near_tie`` times the spread of the token's scores (at least 0.25: two experts that lie close
        have none) of the plain implementation's weakest own pick."""
        if not routed:
            return self.ref(rid)[0]
        name = self.name

        def follow(prefix, per_pos):
            def choose(logits):
                z = torch.sigmoid(logits)
                top = len(next(iter(per_pos.values())))
                own = torch.topk(logits, top, dim=-1).indices
                rows = []
                for pos in range(z.shape[0]):
                    mine = own[pos].tolist()
                    eng = per_pos.get(pos, mine)
                    if sorted(eng) != sorted(mine) and near_tie is not None:
                        weakest = min(float(z[pos, e]) for e in mine)
                        spread = max(float(z[pos].max() - z[pos].min()), 0.25)
                        for e in eng:
                            assert float(z[pos, e]) >= weakest - near_tie * spread, (
                                f"{name}/{rid} {prefix} position {pos}: the engine picked expert {e} with score "
                                f"{float(z[pos, e]):.5f}; the plain implementation's weakest pick has {weakest:.5f}")
                    rows.append(eng)
                return rows
            return choose

        forced = {int(prefix.split(".")[0][1:]): follow(prefix, per_pos) for prefix, per_pos in routed.items() if per_pos}
        return plain.forward(self.cfg, self.weights, self.tokens[rid], picks=forced)[0]


def errors(out, ref):
    """Per row: the largest difference of the logits (mean taken off) over the largest logit of the request."""
    d = out - ref
    d = d - d.mean(-1, keepdim=True)
    top = float((ref - ref.mean(-1, keepdim=True)).abs().max())
    return d.abs().max(-1).values / top, float(d.abs().mean()) / top


def compare(case, got, routed, tol_max, tol_mean, near_tie):
    for rid, out in got.items():
        ref = case.ref_following(rid, routed.get(rid), near_tie)
        assert out.shape == ref.shape, rid
        assert bool(torch.isfinite(out).all()), f"{case.name}/{rid}: logits that are not numbers (a page or slot read stale?)"
        err, mean = errors(out, ref)
        worst = int(err.argmax())
        assert float(err.max()) <= tol_max, f"{case.name}/{rid}: position {worst} is off by {float(err.max()):.2e} of the largest logit"
        assert mean <= tol_mean, f"{case.name}/{rid}: mean error {mean:.2e}"


def compare_together(case, got, routed, tol_max, tol_mean, one_in=10, cap=5.0):
    """As ``compare``, for bfloat16 models in which single positions amplify the rounding of the activations (sharp
    softmaxes over scores of tens, five or six post-norm layers on top of each other): the engine's picks are followed
    without judging them, all but one row in ``one_in`` lie within ``tol_max``, none beyond ``cap`` times that, and the
    mean error is held.  The kernels' plain twins with bfloat16 buffers are off in such rows by as much."""
    for rid, out in got.items():
        ref = case.ref_following(rid, routed.get(rid), None)
        assert out.shape == ref.shape and bool(torch.isfinite(out).all()), rid
        err, mean = errors(out, ref)
        assert mean <= tol_mean, f"{case.name}/{rid}: mean error {mean:.2e}"
        assert float(err.max()) <= cap * tol_max, f"{case.name}/{rid}: position {int(err.argmax())} is off by {float(err.max()):.2e}"
        assert int((err > tol_max).sum()) <= max(1, len(err) // one_in), f"{case.name}/{rid}: {int((err > tol_max).sum())} rows beyond {tol_max}"


def random_config(seed):
    """A configuration drawn from the ranges a small model of this design may have: layer order, head counts and sizes,
    rotated parts, latents, shared latents, decays, experts and constants all vary."""
    import random

    r = random.Random(seed)
    width = r.choice([64, 96, 128, 192, 256])
    n = r.randint(3, 7)
    layers, owners = [], []
    for i in range(n):
        experts = r.choice([0, 4, 8, 16])
        top = r.choice([1, 1, 2, 4]) if experts else 1
        shared = r.choice([None, (r.choice([32, 64, 128]), r.choice([1.0, 2.0]))])
        kind = r.random()
        if kind < 0.35:
            heads = r.choice([1, 2, 4, 6, 8])
            kv = r.choice([k for k in (1, 2, 3, 4, 8) if heads % k == 0])
            dim = r.choice([16, 32, 48, 64, 80, 128])
            lay = attention(heads, kv, dim, r.choice([dim, 32, 64, 80]), rot=r.choice([0, dim // 4 * 2, dim]),
                            base=r.choice([1e4, 1e6]), scale=round(r.uniform(0.05, 0.3), 3))
        elif kind < 0.6:
            lay = gla(r.choice([1, 2, 4]), r.choice([16, 32, 48, 64]), r.choice([16, 32, 64]), tau=r.choice([1.0, 4.0, 16.0]))
        elif owners and r.random() < 0.5:
            j = r.choice(owners)
            m = layers[j]["mixer"]
            lay = latent(r.choice([1, 2, 4]), r.choice([16, 32, 64]), m["rot_dim"], r.choice([16, 32, 64]), m["kv_rank"],
                         kv_from=j, scale=round(r.uniform(0.05, 0.3), 3), base=m["rot"]["base"])
        else:
            lay = latent(r.choice([1, 2, 4, 8]), r.choice([16, 32, 64]), r.choice([8, 16, 32]), r.choice([16, 32, 64]),
                         r.choice([32, 64, 96, 128]), scale=round(r.uniform(0.05, 0.3), 3), base=r.choice([1e4, 1e6]))
            owners.append(i)
        layers.append(with_mlp(lay, experts, min(top, experts or 1), r.choice([16, 32, 64]), r.choice([1.0, 1.5, 3.0]), shared))
    bigram = r.choice([None, (r.choice([101, 509, 2039]), r.choice([3, 131, 1000003]), r.choice([1, 11, 65537]))])
    return model(width, r.randint(100, 700), layers, eps=r.choice([1e-5, 1e-6]), alpha=r.choice([1.0, 2.0, 2.5, 4.0]), bigram=bigram)
