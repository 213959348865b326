"""The Gugozen design through the engine's host logic on the CPU (the kernels replaced by their plain torch twins):
configuration and plan, weights by name, sizes that only a tensor's shape gives, a latent layer on an earlier layer's
cached rows, the embedding's last token in a request's slot, state slots that are freed and used again, whole prompts,
decoding token by token, portions down to two tokens, mixed batches, and greedy generation through the scheduler -- all
against the plain implementation, which shares no code with any of it.  The kernels themselves are covered by the gpu
tests."""
import copy
import math

import pytest
import torch

import emulated_kernels as EK
import plain_gugozen as plain
from gugozen_cases import CONFIGS, Case, compare, make_runner, random_config, run_steps, schedules
import locus_b200.models  # noqa: F401  (registers the architectures)
from locus_b200.config import ConfigError, find_arch
from locus_b200.config.gugozen import GugozenConfig

TOL = (2e-5, 4e-6)   # max and mean |error| of the logits relative to the largest |logit|; float32 twins
TIE = 2e-5
F64 = torch.float64
SHOWS = 40 * TOL[0]   # what a fault must move the logits by to count as shown: far beyond the tolerance


@pytest.fixture(autouse=True)
def _emulate(monkeypatch):
    EK.install(monkeypatch)


def test_config_reads_every_size_and_refuses_what_is_wrong():
    cfg = GugozenConfig.from_dict(copy.deepcopy(CONFIGS["mix"]))
    assert find_arch("Gugozen").parse_config is not None
    a, g, l, s = (cfg.layers[i].mixer for i in (0, 1, 2, 4))
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.rot.dims, a.rot.base) == (4, 2, 32, 16, 0.21, 16, 500.0)
    assert (g.heads, g.dim, g.vdim, g.tau) == (2, 24, 16, 8.0)
    assert (l.heads, l.dim, l.rot_dim, l.vdim, l.kv_rank, l.scale, l.kv_from) == (4, 16, 8, 16, 32, 0.17, None)
    assert (s.heads, s.vdim, s.kv_from) == (2, 32, 2)
    f = cfg.layers[0].mlp
    assert (f.experts, f.top, f.expert.ff, f.expert.limit, f.shared.ff, f.shared.limit) == (6, 2, 24, 1.25, 40, 2.0)
    assert cfg.layers[1].mlp.shared is None and cfg.layers[3].mlp is None
    assert (cfg.alpha, cfg.eps, cfg.width, cfg.vocab) == (2.5, 1e-5, 64, 97)
    assert (cfg.bigram.buckets, cfg.bigram.mul_prev, cfg.bigram.mul_cur) == (53, 31, 5)
    odd = GugozenConfig.from_dict(copy.deepcopy(CONFIGS["odd"]))
    assert odd.bigram is None and odd.layers[2].mixer.rot is None and odd.layers[3].mixer.rot is None and odd.alpha == 1.0
    for path, value, word in ((("layers", 0, "type"), "conv", "type"), (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 0, "mixer", "rot", "dims"), 34, "rot.dims"),
                              (("layers", 4, "mixer", "kv_from"), 4, "kv_from"), (("layers", 4, "mixer", "kv_from"), 1, "kv_from"),
                              (("layers", 4, "mixer", "kv_rank"), 16, "kv_rank"), (("layers", 0, "mlp", "kind"), "dense", "kind"),
                              (("norm",), None, "norm"), (("layers", 1, "mixer", "tau"), 0.0, "tau"),
                              (("layers", 0, "mlp", "router", "top"), 7, "top"), (("layers", 0, "mlp", "expert", "limit"), 0, "limit"),
                              (("postln_alpha",), None, "postln_alpha"), (("embedding", "bigram", "buckets"), 0, "buckets")):
        raw = copy.deepcopy(CONFIGS["mix"])
        node = raw
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            GugozenConfig.from_dict(raw)


def test_plan_shares_rows_between_layers_and_gives_the_embedding_a_slot(tmp_path):
    from locus_b200.models.model import Model, load_model

    e = find_arch("Gugozen")
    m = Model(e.build_plan(e.parse_config(copy.deepcopy(CONFIGS["mix"]))), torch.float32, "cpu")
    needs = m.cache_needs()
    # five layer calls and, behind them, the embedding's entry: one int32 per request
    assert [c for _, _, c in needs] == [None, None, None, None, 2, None] and len(needs) == 6
    assert needs[5][0] is None and needs[5][1].shape == (1,) and needs[5][1].dtype == torch.int32
    assert (needs[0][0].n_kv_heads, needs[0][0].head_dim, needs[0][0].window) == (2, 32, 0) and needs[0][1] is None
    assert needs[1][0] is None and needs[1][1].shape == (2 * 24 * 16,)
    assert (needs[2][0].head_dim, needs[2][0].has_v, needs[2][0].n_kv_heads) == (32 + 8, False, 1)
    names = {s.name for _, s in m.tensor_sources()}
    assert {"embed", "bigram", "final.norm", "final.norm.b", "l0.norm1", "l0.norm1.b", "l0.norm2.b", "l0.mix.q.norm", "l0.mix.k.norm",
            "l0.mix.sink", "l1.mix.a1", "l1.mix.a2", "l1.mix.a2.b", "l1.mix.norm", "l2.mix.dkv", "l2.mix.dkv.norm", "l2.mix.g",
            "l4.mix.uk", "l4.mix.q", "l0.mlp.router", "l0.mlp.e5.gate", "l0.mlp.shared.down", "l2.mlp.shared.up"} <= names
    assert not {"l4.mix.dkv", "l4.mix.dkv.norm", "l3.norm2", "l3.norm2.b", "head", "l1.mlp.shared.up", "l0.mix.g"} & names
    # without a pair table the embedding keeps nothing
    odd = Model(e.build_plan(e.parse_config(copy.deepcopy(CONFIGS["odd"]))), torch.float32, "cpu")
    assert len(odd.cache_needs()) == 6 and "bigram" not in {s.name for _, s in odd.tensor_sources()}
    # the width of a gla layer's first decay projection comes from the stored tensor's shape
    case = Case("mix", tmp_path, torch.float32)
    loaded = load_model(case.dir, torch.float32, "cpu")
    assert loaded.blocks[1].mixer.rank == 5 and loaded.blocks[3].mixer.rank == 12
    assert tuple(case.weights["l1.mix.a1"].shape) == (5, 64)


def test_plain_mechanisms_against_their_closed_forms():
    g = torch.Generator().manual_seed(5)
    # the hashed rows: the last row for the first token, then (prev * a + cur * b) mod buckets in whole numbers
    assert plain.bigram_rows([5, 9, 9, 0], 7, 3, 10 ** 12 + 1) == [7, (15 + 9 * (10 ** 12 + 1)) % 7, (27 + 9 * (10 ** 12 + 1)) % 7, 27 % 7]
    # the recurrence against its closed form o_t = sum_j (prod_(j<l<=t) a_l * k_j . q_t) v_j, one head
    T, d, dv = 9, 3, 2
    w = {"p.q": torch.randn(d, 4, generator=g, dtype=F64), "p.k": torch.randn(d, 4, generator=g, dtype=F64),
         "p.v": torch.randn(dv, 4, generator=g, dtype=F64), "p.g": torch.randn(dv, 4, generator=g, dtype=F64),
         "p.a1": torch.randn(2, 4, generator=g, dtype=F64), "p.a2": torch.randn(d, 2, generator=g, dtype=F64),
         "p.a2.b": torch.randn(d, generator=g, dtype=F64), "p.norm": torch.ones(dv, dtype=F64), "p.o": torch.eye(dv, dtype=F64)}
    h = torch.randn(T, 4, generator=g, dtype=F64)
    m = {"heads": 1, "dim": d, "vdim": dv, "tau": 3.0}
    got = plain.gla(m, w, "p.", h, 1e-6)
    q, k, v = h @ w["p.q"].T * d ** -0.5, h @ w["p.k"].T, h @ w["p.v"].T
    a = torch.sigmoid(h @ w["p.a1"].T @ w["p.a2"].T + w["p.a2.b"]) ** (1.0 / 3.0)
    gate = h @ w["p.g"].T
    for t in (0, 4, 8):
        o = torch.zeros(dv, dtype=F64)
        for j in range(t + 1):
            dec = torch.ones(d, dtype=F64)
            for l in range(j + 1, t + 1):
                dec = dec * a[l]
            o = o + float((dec * k[j] * q[t]).sum()) * v[j]
        o = o / torch.sqrt((o * o).mean() + 1e-6) * (gate[t] * torch.sigmoid(gate[t]))
        assert torch.allclose(got[t], o, atol=1e-12)
    # the sink: p_j = exp(s_j) / (exp(sink) + sum exp(s)), the sink itself taken as it is (no factor)
    w = {"a.q": torch.eye(2, dtype=F64), "a.k": torch.eye(2, dtype=F64), "a.v": torch.eye(2, dtype=F64), "a.o": torch.eye(2, dtype=F64),
         "a.q.norm": torch.ones(2, dtype=F64), "a.k.norm": torch.ones(2, dtype=F64), "a.sink": torch.tensor([0.7], dtype=F64)}
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 0.5}
    h = torch.tensor([[1.0, 0.0], [0.0, 2.0]], dtype=F64)
    o = plain.attention(m, w, "a.", h, 0.0)
    qn = h / torch.sqrt((h * h).mean(-1, keepdim=True))
    s = torch.tensor([float(qn[1] @ qn[0]), float(qn[1] @ qn[1])], dtype=F64) * 0.5
    p = torch.exp(s) / (math.exp(0.7) + torch.exp(s).sum())
    assert torch.allclose(o[1], p[0] * h[0] + p[1] * h[1], atol=1e-12)
    # the expert: the clamps, and a weight on the input that is not a weight on the output
    w = {"e.gate": torch.tensor([[1.0]], dtype=F64), "e.up": torch.tensor([[1.0]], dtype=F64), "e.down": torch.tensor([[1.0]], dtype=F64)}
    y = plain.clamped_expert(w, "e.", torch.tensor([[5.0], [-5.0], [0.5]], dtype=F64), 1.5)
    assert math.isclose(float(y[0]), 1.5 / (1 + math.exp(-1.702 * 1.5)) * 2.5)
    assert math.isclose(float(y[1]), -5.0 / (1 + math.exp(1.702 * 5.0)) * (-1.5 + 1.0))
    assert math.isclose(float(y[2]), 0.5 / (1 + math.exp(-1.702 * 0.5)) * 1.5)
    # the rotation: pairs (i, i + dims/2) of the first dims, the rest untouched, position 0 unchanged
    x = torch.randn(4, 1, 6, generator=g, dtype=F64)
    r = plain.rotate(x, torch.arange(4), 100.0, 4)
    assert torch.equal(r[0], x[0]) and torch.equal(r[..., 4:], x[..., 4:])
    ang = 3.0 * 100.0 ** (-2.0 / 4)
    assert math.isclose(float(r[3, 0, 1]), float(x[3, 0, 1]) * math.cos(ang) - float(x[3, 0, 3]) * math.sin(ang))
    assert math.isclose(float(r[3, 0, 3]), float(x[3, 0, 3]) * math.cos(ang) + float(x[3, 0, 1]) * math.sin(ang))


@pytest.mark.parametrize("name", ["mix", "odd", "latent_only", "wide", "moe_only"])
def test_every_schedule_against_the_plain_implementation(tmp_path, name):
    lens = (41, 1, 23, 37, 2, 30) if name != "wide" else (90, 33, 5)
    case = Case(name, tmp_path, torch.float32, requests=lens)
    for sched, steps in schedules(case).items():
        runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=40, max_tokens=160, slots=4)
        got, routed = run_steps(runner, cache, case, steps)
        compare(case, got, routed, *TOL, TIE)
        assert cache.free_pages() == cache.total_pages() and cache.state_slots.free == cache.state_slots.total, sched


def test_a_drawn_configuration_in_mixed_batches(tmp_path):
    for seed in (3, 8):
        case = Case(f"drawn{seed}", tmp_path, torch.float32, raw=random_config(seed), requests=(70, 9, 44, 21), seed=seed)
        runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=16, n_pages=24, max_tokens=160, slots=4)
        got, routed = run_steps(runner, cache, case, schedules(case)["mixed"])
        compare(case, got, routed, 1e-4, 2e-5, TIE)


def test_the_sharpened_weights_show_each_fault(tmp_path, monkeypatch):
    """What the comparisons rest on: with these weights a lost sink, a sink that took the scores' factor, a weight on an
    expert's output instead of its input, a lost clamp, another root of the decay, another factor in front of the norms,
    a lost pair table, another rotated part, a latent layer that projects rows of its own, lost states and a far token
    each move the logits by far more than the tolerance."""
    case = Case("mix", tmp_path, torch.float32, requests=(60,))
    ref = case.ref("r0")[0]
    scale = float((ref - ref.mean(-1, keepdim=True)).abs().max())

    def moved(cfg=None, weights=None, toks=None, last=20):
        lg = plain.forward(cfg or case.cfg, weights or case.weights, toks or case.tokens["r0"])[0]
        return float((lg[-last:] - ref[-last:]).abs().max()) / scale

    w = dict(case.weights)
    w["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -30.0)               # no sink
    assert moved(weights=w) > SHOWS
    w["l0.mix.sink"] = case.weights["l0.mix.sink"] * case.cfg["layers"][0]["mixer"]["scale"]   # the sink times the factor
    assert moved(weights=w) > SHOWS
    for key, value in ((("layers", 0, "mixer", "rot", "dims"), 8), (("layers", 0, "mixer", "scale"), 0.3),
                       (("layers", 2, "mixer", "scale"), 0.3), (("layers", 2, "mixer", "rot", "base"), 400.0),
                       (("layers", 1, "mixer", "tau"), 4.0), (("postln_alpha",), 2.0), (("layers", 0, "mlp", "expert", "limit"), 9.0),
                       (("layers", 2, "mlp", "shared", "limit"), 9.0), (("embedding", "bigram", "mul_prev"), 30),
                       (("layers", 0, "mlp", "router", "top"), 1), (("norm", "eps"), 1e-2)):
        cfg = copy.deepcopy(case.cfg)
        node = cfg
        for k in key[:-1]:
            node = node[k]
        node[key[-1]] = value
        assert moved(cfg) > SHOWS, key
    for name in ("l0.mix.q.norm", "l0.mix.k.norm", "l2.mix.dkv.norm", "l1.mix.norm", "l1.mix.a2.b", "l0.norm1.b", "bigram", "l2.mix.g"):
        w = dict(case.weights)
        w[name] = torch.ones_like(w[name]) if name.endswith("norm") else torch.zeros_like(w[name])
        assert moved(weights=w) > SHOWS, name
    # the weight on the expert's output instead of its input
    real = plain.clamped_expert
    monkeypatch.setattr(plain, "moe_ff", lambda f, weights, pre, h, picks=None: _weight_on_output(real, f, weights, pre, h))
    assert moved() > SHOWS
    monkeypatch.undo()
    EK.install(monkeypatch)
    # layer 4 with rows of its own kind (layer 2's projection once more, applied to its own input)
    cfg = copy.deepcopy(case.cfg)
    del cfg["layers"][4]["mixer"]["kv_from"]
    w = dict(case.weights)
    w["l4.mix.dkv"], w["l4.mix.dkv.norm"] = w["l2.mix.dkv"], w["l2.mix.dkv.norm"]
    assert moved(cfg, w) > SHOWS
    # lost states, rows and the last token: a sequence that starts 25 tokens later has forgotten what came before
    lg = plain.forward(case.cfg, case.weights, case.tokens["r0"][25:])[0]
    assert float((lg[-20:] - ref[-20:]).abs().max()) / scale > SHOWS
    toks = list(case.tokens["r0"])
    toks[1] = (toks[1] + 1) % case.cfg["vocab"]     # a token 40 and more back
    assert moved(toks=toks) > SHOWS


def _weight_on_output(expert, f, weights, pre, h):
    out = torch.zeros_like(h)
    chosen = plain.route(weights, pre, h, f["router"]["top"])
    for t in range(h.shape[0]):
        for e, wt in chosen[t]:
            out[t] += wt * expert(weights, f"{pre}e{e}.", h[t][None, :], f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + expert(weights, pre + "shared.", h, f["shared"]["limit"])
    return out, [[e for e, _ in c] for c in chosen], h @ weights[pre + "router"].to(F64).T


def test_far_tokens_reach_through_each_mechanism_alone(tmp_path):
    """One-layer models: a token 45 positions back moves the last logits through the recurrence's state alone, through
    softmax attention alone and through latent attention alone (with a second layer on the first one's rows)."""
    for name in ("gla_only", "attention_only", "latent_only"):
        case = Case(name, tmp_path, torch.float32, requests=(50,))
        ref = case.ref("r0")[0]
        scale = float((ref - ref.mean(-1, keepdim=True)).abs().max())
        toks = list(case.tokens["r0"])
        toks[2] = (toks[2] + 1) % case.cfg["vocab"]
        lg = plain.forward(case.cfg, case.weights, toks)[0]
        assert float((lg[-3:] - ref[-3:]).abs().max()) / scale > SHOWS, name


def test_the_last_token_lives_in_the_slot_and_a_slot_used_again_starts_anew(tmp_path):
    """Requests through one state slot one after the other, cut so that portions start behind every kind of step: the
    pair table's row of a portion's first token comes from the token the step before ended on, a request's first token
    takes the table's last row whatever the slot held, and the recurrence's state starts at zero."""
    case = Case("mix", tmp_path, torch.float32, requests=(30, 30, 12))
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=16, max_tokens=64, slots=1)
    got, routed = run_steps(runner, cache, case, [[("r0", 30)], [("r1", 7)], [("r1", 1)], [("r1", 22)], [("r2", 2)], [("r2", 10)]])
    compare(case, got, routed, *TOL, TIE)
    # the embedding's slot holds the last token fed
    emb_state = cache.layer_caches()[-1].state
    assert emb_state.dtype == torch.int32 and int(emb_state[0, 0]) == case.tokens["r2"][-1]
    # a pair table matters at a portion's first token: the same cut with the slot's token lost differs there
    w = dict(case.weights)
    w["bigram"] = torch.zeros_like(w["bigram"])
    lg = plain.forward(case.cfg, w, case.tokens["r1"])[0]
    ref = case.ref("r1")[0]
    assert float((lg[7] - ref[7]).abs().max()) / float(ref.abs().max()) > SHOWS


def test_pages_and_slots_are_used_again_under_a_small_pool(tmp_path):
    case = Case("wide", tmp_path, torch.float32, requests=(90, 90, 40, 40, 40))
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=24, max_tokens=72, slots=2)
    steps = [[("r0", 30)], [("r0", 30)], [("r0", 30)], [("r1", 24), ("r2", 8)], [("r1", 33), ("r2", 32)],
             [("r1", 33), ("r3", 2)], [("r3", 38), ("r4", 1)], [("r4", 39)]]
    got, routed = run_steps(runner, cache, case, steps)
    compare(case, got, routed, *TOL, TIE)
    assert cache.free_pages() == cache.total_pages()


def test_long_decoding_token_by_token(tmp_path):
    case = Case("mix", tmp_path, torch.float32, requests=(120,))
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=20, max_tokens=32, slots=2)
    got, routed = run_steps(runner, cache, case, [[("r0", 3)]] + [[("r0", 1)]] * 117)
    compare(case, got, routed, *TOL, TIE)


def test_greedy_generation_through_the_scheduler(tmp_path):
    from locus_b200.engine.engine import Engine
    from locus_b200.models import load_model

    case = Case("mix", tmp_path, torch.float32, requests=(9, 21, 3))
    m = load_model(case.dir, torch.float32, "cpu")
    eng = Engine.from_model(m, ctx=256, page_tokens=8, max_batch_tokens=16, chunk=8, max_running=2, use_graphs=False)
    prompts = [case.tokens[r] for r in ("r0", "r1", "r2")]
    outs = eng.generate(prompts, max_new_tokens=6)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg = plain.forward(case.cfg, case.weights, seq)[0]
            top2 = torch.topk(lg[-1], 2).values
            if float(top2[0] - top2[1]) > 1e-4 * float(lg[-1].abs().max()):
                assert int(torch.argmax(lg[-1])) == tok
            seq.append(tok)
    assert eng.cache.free_pages() == eng.cache.total_pages()
