"""Tiny Mekizen configurations, random model folders with weights shaped so that faults show, and the helpers that
the host tests (plain twins of the kernels, CPU) and the gpu tests share to run schedules against the plain
implementation of ``plain_mekizen``.

Random weights of standard deviation 0.02 hide faults: attention is nearly uniform, a sink outweighs every key, every
state decays in a few tokens and a convolution's taps hardly matter.  ``sharpen`` spreads the scores, gives the delta
rule slow and fast heads and strong steps, convolution taps of the size of one, and norm weights that are not all
alike."""
import copy
import json
import os

import torch

import plain_mekizen as plain
from lalepel_cases import cuts, make_runner, schedules, tokens  # noqa: F401  (shared schedule helpers)


def attention(heads, kv_heads, dim, vdim, window=0, keep_first=0, rot=None, kv_from=None, scale=None, base=10000.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def parallel(heads, kv_heads, dim, vdim, conv, rot, r_heads, r_kv, r_dim, r_vdim, r_conv, scale=None, base=10000.0):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
            "scale": scale if scale is not None else dim ** -0.5}
    if rot:
        left["rot"] = {"base": base, "dims": rot}
    right = {"heads": r_heads, "kv_heads": r_kv, "dim": r_dim, "vdim": r_vdim, "conv": r_conv}
    return {"type": "parallel", "mixer": {"left": left, "right": right}}


def with_mlp(layer, ff):
    layer = copy.deepcopy(layer)
    layer["mlp"] = {"kind": "dense", "ff": ff} if ff else None
    return layer


def model(width, vocab, layers, eps=1e-5, embed_scale=None):
    cfg = {"architecture": "Mekizen", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}
    if embed_scale is not None:
        cfg["embedding"] = {"scale": embed_scale}
    return cfg


CONFIGS = {
    # every mechanism: both mixers, a window with kept first tokens, a later layer on an earlier layer's keys and values
    # with a wider mask of its own, a layer without a feed-forward
    "mix": model(64, 97, [
        with_mlp(parallel(4, 2, 32, 16, 3, 16, 4, 2, 16, 8, 4), 48),
        with_mlp(attention(4, 2, 16, 32, window=11, keep_first=3, rot=8, base=500.0), 32),
        with_mlp(parallel(2, 1, 16, 16, 2, 16, 2, 2, 24, 16, 2), None),
        with_mlp(attention(4, 2, 16, 32, window=20, keep_first=5, rot=8, base=500.0, kv_from=1), 40),
    ], embed_scale=2.5),
    # nothing a multiple of 16, 8 or 4; one head; equal head counts; a window of one token; a convolution of one tap and
    # of five; no rotation in one layer; no mask in another; kept tokens without end (more than the window); no scale
    "odd": model(50, 61, [
        with_mlp(parallel(1, 1, 10, 6, 1, 4, 3, 3, 7, 5, 5), 30),
        with_mlp(attention(3, 3, 10, 6, window=1, keep_first=2, rot=6), 9),
        with_mlp(parallel(3, 1, 6, 10, 5, 0, 1, 1, 11, 3, 1), None),
        with_mlp(attention(2, 1, 6, 14, rot=0), 21),
        with_mlp(attention(2, 2, 12, 4, window=4, keep_first=9, rot=12, base=77.0), None),
    ], eps=1e-6),
    # one mechanism each
    "conv_attention_only": model(48, 50, [with_mlp(parallel(4, 1, 16, 16, 3, 8, 1, 1, 8, 8, 2), None)]),
    "delta_only": model(48, 50, [with_mlp(parallel(1, 1, 16, 16, 2, 0, 4, 2, 16, 12, 4), None)]),
    "attention_only": model(48, 50, [with_mlp(attention(4, 2, 16, 16, window=9, keep_first=2, rot=16), None)], embed_scale=1.0),
    "shared_kv": model(48, 50, [with_mlp(attention(2, 1, 16, 16, window=6, keep_first=1, rot=8), 24),
                                with_mlp(attention(2, 1, 16, 16, rot=8, kv_from=0), 24),
                                with_mlp(attention(2, 1, 16, 16, window=3, keep_first=4, rot=8, kv_from=0), None)]),
    # larger heads: rows of the delta rule beyond one lane's first registers, heads of 80 and 72, a window beyond a page
    "wide": model(128, 211, [
        with_mlp(parallel(2, 1, 80, 64, 4, 40, 4, 2, 72, 40, 3), 96),
        with_mlp(attention(4, 1, 96, 80, window=70, keep_first=6, rot=48, base=50000.0), 64),
        with_mlp(parallel(2, 2, 128, 128, 3, 128, 2, 1, 136, 20, 4), 64),
    ], embed_scale=3.0),
}
SEEDS = {n: 71 + i for i, n in enumerate(CONFIGS)}


def sharpen(name, w):
    """Weights (name -> float32 tensor) changed in place so that windows, far keys, kept tokens, the sink, states and
    convolution taps matter."""
    g = torch.Generator().manual_seed(9)
    for n in list(w):
        t = w[n]
        if n.endswith((".norm1", ".norm2")) or n == "final.norm":
            w[n] = (torch.rand(t.shape, generator=g) - 0.5) * 0.6          # stored around zero
        elif n.endswith((".left.out", ".right.out", ".right.norm")):
            w[n] = 0.5 + torch.rand(t.shape, generator=g)
        elif n.endswith(".conv"):
            w[n] = (torch.rand(t.shape, generator=g) - 0.3) * 1.5
        elif n.endswith((".left.q", ".left.k")):
            w[n] = t * 3.0                                                   # (their heads are normed: the scale decides)
        elif n.endswith((".mix.q", ".mix.k")):
            w[n] = t * 6.0                                                   # scores around zero: the sink has its say
        elif n.endswith((".mix.v", ".mix.o")):
            w[n] = t * 4.0
        elif n.endswith((".q.b", ".k.b", ".v.b", ".o.b")):
            w[n] = t * 10.0
        elif n.endswith((".right.q", ".right.k", ".right.v")):
            w[n] = t * 6.0
        elif n.endswith(".right.b"):
            w[n] = t * 20.0                                                  # steps from near 0 to near 1
        elif n.endswith(".right.a"):
            w[n] = t * 10.0
        elif n.endswith(".right.A_log"):
            w[n] = torch.linspace(-5.0, 0.5, t.numel())                      # decays per unit step from 0.993 to 0.19
        elif n.endswith(".right.dt_bias"):
            w[n] = torch.linspace(-2.0, 1.0, t.numel())
        elif n.endswith((".mix.g", ".right.g")):
            w[n] = t * 8.0
        elif n == "embed":
            w[n] = t * 30.0


def make_dir(tmp_path, name, store_dtype=torch.bfloat16, raw=None, tweak=sharpen, seed=None):
    """A model folder of configuration ``name`` (or ``raw``): seeded random weights, then ``tweak``, stored in
    ``store_dtype``.  Returns (folder, config dict, weights as stored, float32)."""
    from locus_b200.weights.loader import write_random_model
    from locus_b200.weights.safetensors_io import ModelFiles, write_safetensors
    import locus_b200.models  # noqa: F401

    cfg = copy.deepcopy(raw if raw is not None else CONFIGS[name])
    d = os.path.join(str(tmp_path), f"mekizen_{name}_{str(store_dtype).split('.')[-1]}")
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

    def ref(self, rid):
        if rid not in self._ref:
            self._ref[rid] = plain.forward(self.weights, self.cfg, self.tokens[rid])
        return self._ref[rid]


def run_steps(runner, cache, case, steps, want=None):
    """steps: lists of (request id, n tokens); every fed position's logits are wanted.  A request is released after
    its last token (its pages and its state slot are used again by whoever comes next).  Returns {rid: [T, V] logits on
    the CPU}."""
    from locus_b200.engine.step import StepEntry

    fed, got = {}, {}
    for step in steps:
        entries = []
        for rid, n in step:
            a = fed.get(rid, 0)
            seq = cache.get(rid) or cache.open(rid)
            assert cache.ensure_capacity(seq, n), (rid, n)
            entries.append(StepEntry(seq, case.tokens[rid][a:a + n], list(range(n))))
        lg = runner.step(entries).detach().cpu().double()
        row = 0
        for rid, n in step:
            a = fed.get(rid, 0)
            got.setdefault(rid, []).append(lg[row:row + n].clone())
            row += n
            fed[rid] = a + n
        for rid, n in step:
            if fed[rid] == len(case.tokens[rid]):
                cache.release(cache.get(rid))
        cache.check_invariants()
    if hasattr(runner, "check_device_errors"):
        runner.check_device_errors()
    return {r: torch.cat(v) for r, v in got.items()}


def errors(out, ref):
    """Per row: the largest difference of the logits (mean taken off) over the largest logit of the request."""
    d = out - ref
    d = d - d.mean(-1, keepdim=True)
    top = float((ref - ref.mean(-1, keepdim=True)).abs().max())
    return d.abs().max(-1).values / top, float(d.abs().mean()) / top


def compare(case, got, tol_max, tol_mean):
    for rid, out in got.items():
        ref = case.ref(rid)
        assert out.shape == ref.shape, rid
        assert bool(torch.isfinite(out).all()), f"{case.name}/{rid}: logits that are not numbers (a page or slot read stale?)"
        err, mean = errors(out, ref)
        worst = int(err.argmax())
        assert float(err.max()) <= tol_max, f"{case.name}/{rid}: position {worst} is off by {float(err.max()):.2e} of the largest logit"
        assert mean <= tol_mean, f"{case.name}/{rid}: mean error {mean:.2e}"


def compare_together(case, got, tol_max, tol_mean, one_in=10, cap=5.0):
    """As ``compare``, for bfloat16 models in which single positions amplify the rounding of the activations (a head of
    a few elements whose root mean square passes near zero, scores of a window of one token): the mean error as
    everywhere, all but one row in ``one_in`` within ``tol_max``, and no row beyond ``cap`` times that.  The kernels'
    plain twins in bfloat16 are off in the same rows by as much, for every cut of the prompt."""
    for rid, out in got.items():
        ref = case.ref(rid)
        assert out.shape == ref.shape and bool(torch.isfinite(out).all()), rid
        err, mean = errors(out, ref)
        assert mean <= tol_mean, f"{case.name}/{rid}: mean error {mean:.2e}"
        assert float(err.max()) <= cap * tol_max, f"{case.name}/{rid}: position {int(err.argmax())} is off by {float(err.max()):.2e}"
        assert int((err > tol_max).sum()) <= max(1, len(err) // one_in), f"{case.name}/{rid}: {int((err > tol_max).sum())} rows beyond {tol_max}"


def random_config(seed):
    """A configuration drawn from the ranges a small model of this design may have: layer order, head counts and sizes,
    rotated parts, windows, kept tokens, taps, shared keys and values and constants all vary."""
    import random

    r = random.Random(seed)
    width = r.choice([64, 96, 128, 192, 256])
    n = r.randint(3, 7)
    layers, owners = [], []
    for i in range(n):
        ff = r.choice([0, 32, 64, 96, 128])
        if r.random() < 0.55:
            heads = r.choice([1, 2, 4, 8])
            kv = r.choice([k for k in (1, 2, 4, 8) if heads % k == 0])
            dim = r.choice([16, 24, 32, 48, 64, 96, 128])
            rh = r.choice([1, 2, 4])
            layers.append(with_mlp(parallel(heads, kv, dim, r.choice([dim, dim, 32, 64]), r.choice([1, 2, 3, 4]),
                                            r.choice([0, dim // 2 // 2 * 2, dim // 2 * 2]), rh, r.choice([k for k in (1, 2, 4) if rh % k == 0]),
                                            r.choice([16, 32, 48, 64]), r.choice([16, 32, 64]), r.choice([2, 3, 4]),
                                            scale=round(r.uniform(0.05, 0.3), 3), base=r.choice([1e4, 1e6])), ff))
        elif owners and r.random() < 0.4:
            j = r.choice(owners)
            m = layers[j]["mixer"]
            heads = m["kv_heads"] * r.choice([1, 2, 4])
            layers.append(with_mlp(attention(heads, m["kv_heads"], m["dim"], m["vdim"], window=r.choice([0, 5, 40, 64, 100]),
                                             keep_first=r.choice([0, 1, 4, 7]), rot=m.get("rot", {}).get("dims", 0),
                                             base=m.get("rot", {}).get("base", 1e4), kv_from=j, scale=round(r.uniform(0.05, 0.3), 3)), ff))
        else:
            heads = r.choice([1, 2, 4, 8])
            kv = r.choice([k for k in (1, 2, 4, 8) if heads % k == 0])
            dim = r.choice([16, 32, 48, 64, 80, 128])
            layers.append(with_mlp(attention(heads, kv, dim, r.choice([dim, 32, 64]), window=r.choice([0, 8, 33, 64, 96, 144]),
                                             keep_first=r.choice([0, 2, 6, 20]), rot=r.choice([0, dim // 2, dim]),
                                             base=r.choice([1e4, 5e4]), scale=round(r.uniform(0.05, 0.3), 3)), ff))
            owners.append(i)
    return model(width, r.randint(100, 700), layers, eps=r.choice([1e-5, 1e-6]), embed_scale=r.choice([None, 1.0, 2.0, 3.5]))
